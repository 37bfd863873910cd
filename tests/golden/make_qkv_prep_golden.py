"""Generates tests/golden/qkv_prep_ref.npz: inputs and OUTPUTS OF THE REFERENCE'S OWN KERNELS for the QKV
prologue + append (k_qkv_prep_fast, k_qkv_prep_fast_ms, k_rope_tables_rows; engine/src/bruce.cu:1732-1918,
1641-1654), in the reference's native geometry (16 q heads / 4 kv heads / head_dim 256 / window 1024).

Needs a GPU and oracle/_ref/libbruce_ref.so (built by oracle/ref_build.py where the reference tree is
present).  Run from the repository root:  python tests/golden/make_qkv_prep_golden.py [out.npz]
The committed fixture was produced by exactly this script on a B200."""
import ctypes as C
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
N_HEAD, N_KV, HD, W, SLOT_CTX, REC = 16, 4, 256, 1024, 2048, 272


def _p(t):
    return C.c_void_p(t.data_ptr())


def main(out_path):
    lib = C.CDLL(os.path.join(ROOT, "oracle", "_ref", "libbruce_ref.so"))
    rng = np.random.default_rng(20240607)
    dev = "cuda"
    res = {}

    # ---- case A: 6 rows of one sequence at position 1000, full layer, table 1; and window layer, table 2
    rows, p0 = 6, 1000
    q = rng.standard_normal((rows, N_HEAD, HD), dtype=np.float32)
    k = rng.standard_normal((rows, N_KV, HD), dtype=np.float32)
    v = rng.standard_normal((rows, N_KV, HD), dtype=np.float32)
    sqk = (1.0 + 0.1 * rng.standard_normal((N_HEAD, HD))).astype(np.float32)
    posd = torch.tensor([p0], dtype=torch.int32, device=dev)
    csd = torch.zeros((rows, 256), device=dev)
    snd = torch.zeros((rows, 256), device=dev)
    assert lib.ref_rope_tables(_p(csd), _p(snd), _p(posd), rows, 0) == 0
    kd, vd, sqkd = torch.from_numpy(k).to(dev), torch.from_numpy(v).to(dev), torch.from_numpy(sqk).to(dev)
    res.update(a_q=q, a_k=k, a_v=v, sqk=sqk, a_pos=np.int32(p0), a_cs=csd.cpu().numpy(), a_sn=snd.cpu().numpy())
    for tag, is_swa, theta in (("full", 0, 1), ("swa", 1, 2)):
        pstride = 2 * W if is_swa else SLOT_CTX
        kvk = torch.zeros(N_KV * pstride * REC, dtype=torch.uint8, device=dev)
        kvv = torch.zeros_like(kvk)
        qd = torch.from_numpy(q.copy()).to(dev)
        torch.cuda.synchronize()
        rc = lib.ref_kv_append_theta(_p(qd), _p(kd), _p(vd), _p(sqkd), _p(kvk), _p(kvv), _p(posd), rows, is_swa, theta,
                                     SLOT_CTX, _p(csd), _p(snd))
        assert rc == 0
        slots = [(p0 + r) & (pstride - 1) if is_swa else p0 + r for r in range(rows)]
        kk = kvk.cpu().numpy().reshape(N_KV, pstride, REC)[:, slots]
        vv = kvv.cpu().numpy().reshape(N_KV, pstride, REC)[:, slots]
        res[f"a_{tag}_q_out"] = qd.cpu().numpy()
        res[f"a_{tag}_krec"] = kk
        res[f"a_{tag}_vrec"] = vv

    # ---- case B: multi-slot decode, 5 slots (one idle), per-row positions, full layer, table 1
    n = 5
    pos = np.array([17, 1900, 0, 512, 2047], dtype=np.int32)
    slot = np.array([3, 0, 4, 1, 2], dtype=np.int32)
    act = np.array([1, 1, 0, 1, 1], dtype=np.int32)
    q = rng.standard_normal((n, N_HEAD, HD), dtype=np.float32)
    k = rng.standard_normal((n, N_KV, HD), dtype=np.float32)
    v = rng.standard_normal((n, N_KV, HD), dtype=np.float32)
    posd, slotd, actd = (torch.from_numpy(a).to(dev) for a in (pos, slot, act))
    csd = torch.zeros((n, 256), device=dev)
    snd = torch.zeros((n, 256), device=dev)
    assert lib.ref_rope_tables(_p(csd), _p(snd), _p(posd), n, 1) == 0
    n_slots = 5
    kvk = torch.zeros(n_slots * N_KV * SLOT_CTX * REC, dtype=torch.uint8, device=dev)
    kvv = torch.zeros_like(kvk)
    qd, kd, vd = torch.from_numpy(q.copy()).to(dev), torch.from_numpy(k).to(dev), torch.from_numpy(v).to(dev)
    torch.cuda.synchronize()
    rc = lib.ref_kv_append_ms(_p(qd), _p(kd), _p(vd), _p(sqkd), _p(kvk), _p(kvv), _p(posd), _p(slotd), _p(actd), n, 0, 1,
                              SLOT_CTX, _p(csd), _p(snd))
    assert rc == 0
    kall = kvk.cpu().numpy().reshape(n_slots, N_KV, SLOT_CTX, REC)
    vall = kvv.cpu().numpy().reshape(n_slots, N_KV, SLOT_CTX, REC)
    res.update(b_q=q, b_k=k, b_v=v, b_pos=pos, b_slot=slot, b_act=act, b_cs=csd.cpu().numpy(), b_sn=snd.cpu().numpy(),
               b_q_out=qd.cpu().numpy(),
               b_krec=np.stack([kall[slot[i], :, pos[i]] for i in range(n)]),
               b_vrec=np.stack([vall[slot[i], :, pos[i]] for i in range(n)]),
               b_k_nonzero_bytes=np.int64(np.count_nonzero(kall)), b_v_nonzero_bytes=np.int64(np.count_nonzero(vall)))
    np.savez_compressed(out_path, **res)
    print("wrote", out_path, {k_: getattr(v_, "shape", ()) for k_, v_ in res.items()})


if __name__ == "__main__":
    main(sys.argv[1] if len(sys.argv) > 1 else os.path.join(ROOT, "tests", "golden", "qkv_prep_ref.npz"))
