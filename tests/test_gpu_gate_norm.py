"""The step after attention on the GPU: battn_gate_norm must reproduce the reference's own kernel bit for bit (the
committed outputs of k_gate_norm_vec4, tests/golden/gate_norm_ref.npz, and -- when the reference library is
present -- the kernel itself on fresh inputs); battn_prefill_gate_norm (attention + merge + gate-norm in one call)
must agree with the two-step path and with the oracle."""
import ctypes as C
import os

import numpy as np
import pytest
import torch

from oracle import oracle as O
from tests.gpu_util import dev_i32, dev_q, gpu_fill, to_np
from tests.util import oracle_fill, oracle_geom

pytestmark = pytest.mark.gpu

HERE = os.path.dirname(os.path.abspath(__file__))
GOLD = os.path.join(HERE, "golden", "gate_norm_ref.npz")
REF_LIB = os.path.join(os.path.dirname(HERE), "oracle", "_ref", "libbruce_ref.so")


def _run(eng, aout, gate, sgate, want_dst=True):
    rows, n = gate.shape
    dev = eng.device
    a = torch.from_numpy(aout).to(dev).to(eng.out_torch).contiguous()
    g, s = torch.from_numpy(gate).to(dev), torch.from_numpy(sgate).to(dev)
    dst = torch.zeros((rows, n), device=dev) if want_dst else None
    xq = torch.zeros((rows, n), dtype=torch.int8, device=dev)
    xd = torch.zeros((rows, n // 32), device=dev)
    xs = torch.zeros((rows, n // 32), dtype=torch.int32, device=dev)
    eng.gate_norm(dst, a, g, s, xq, xd, xs, rows)
    torch.cuda.synchronize()
    return (None if dst is None else dst.cpu().numpy()), xq.cpu().numpy(), xd.cpu().numpy(), xs.cpu().numpy()


@pytest.mark.parametrize("name", ["R", "B32"])
def test_gate_norm_is_bit_identical_to_the_reference_kernel_outputs(name):
    from bruce_engine_b200.engine import AttnEngine
    from bruce_engine_b200.layout import F32, G_B, G_R
    g = G_R if name == "R" else G_B.with_(out_dtype=F32)       # both have n_head * head_dim = 4096
    eng = AttnEngine(g.with_(slot_ctx=64, window=64))
    z = np.load(GOLD)
    dst, xq, xd, xs = _run(eng, z["aout"], z["gate"], z["sgate"])
    assert (dst.view(np.uint32) == z["dst"].view(np.uint32)).all()
    assert (xq == z["xq"]).all() and (xd.view(np.uint32) == z["xd"].view(np.uint32)).all() and (xs == z["xsum"]).all()
    _, xq2, xd2, xs2 = _run(eng, z["aout"], z["gate"], z["sgate"], want_dst=False)       # dst is optional
    assert (xq2 == xq).all() and (xd2 == xd).all() and (xs2 == xs).all()
    assert eng.device_status() == 0


def test_gate_norm_against_the_reference_kernel_on_fresh_inputs():
    if not os.path.exists(REF_LIB):
        pytest.skip("oracle/_ref/libbruce_ref.so not built (reference tree unavailable)")
    from bruce_engine_b200.engine import AttnEngine
    from bruce_engine_b200.layout import G_R
    lib = C.CDLL(REF_LIB)
    if not hasattr(lib, "ref_gate_norm"):
        pytest.skip("reference harness predates ref_gate_norm")
    eng = AttnEngine(G_R.with_(slot_ctx=64, window=64))
    rng = np.random.default_rng(77)
    rows, n = 37, 4096
    aout = rng.standard_normal((rows, n), dtype=np.float32) * rng.uniform(0.01, 10, size=(rows, 1)).astype(np.float32)
    gate = (4 * rng.standard_normal((rows, n))).astype(np.float32)
    sgate = rng.uniform(0.5, 1.5, n).astype(np.float32)
    dst, xq, xd, xs = _run(eng, aout, gate, sgate)
    P = lambda t: C.c_void_p(t.data_ptr())   # noqa: E731
    a, g, s = (torch.from_numpy(x).cuda() for x in (aout, gate, sgate))
    rd = torch.zeros((rows, n), device="cuda")
    rq = torch.zeros((rows, n), dtype=torch.int8, device="cuda")
    rxd = torch.zeros((rows, n // 32), device="cuda")
    rxs = torch.zeros((rows, n // 32), dtype=torch.int32, device="cuda")
    assert lib.ref_gate_norm(P(rd), P(a), P(g), P(s), P(rq), P(rxd), P(rxs), rows) == 0
    assert (dst.view(np.uint32) == rd.cpu().numpy().view(np.uint32)).all()
    assert (xq == rq.cpu().numpy()).all() and (xd == rxd.cpu().numpy()).all() and (xs == rxs.cpu().numpy()).all()


@pytest.mark.parametrize("name,rows,depth,is_swa", [("B32", 200, 700, False), ("B32", 512, 3584, False), ("B32", 512, 3584, True),
                                                    ("R", 384, 1500, False), ("B", 96, 2000, False)])
def test_prefill_fused_with_gate_norm(name, rows, depth, is_swa):
    """Attention of a prompt chunk + merge + gate + norm + q8 in one call (split records never become an attention
    output in memory) against (a) battn_prefill followed by battn_gate_norm and (b) the oracle."""
    from bruce_engine_b200.engine import AttnEngine
    from bruce_engine_b200.layout import F32, G_B, G_R
    base = {"B": G_B, "B32": G_B.with_(out_dtype=F32), "R": G_R}[name]
    g = base.with_(slot_ctx=depth + rows, window=1024)
    eng, og = AttnEngine(g), oracle_geom(g)
    rng = np.random.default_rng(rows + depth)
    n_pos = depth + rows
    q = rng.standard_normal((1, rows, g.n_head, g.head_dim), dtype=np.float32)
    if g.q_dtype == 1:
        q = q.astype(np.float16).astype(np.float32)
    k = rng.standard_normal((n_pos, g.n_kv, g.head_dim), dtype=np.float32)
    v = rng.standard_normal((n_pos, g.n_kv, g.head_dim), dtype=np.float32)
    kvk, kvv = eng.alloc_kv_layer(is_swa, fill=0)
    gpu_fill(eng, k, v, kvk, kvv, is_swa)
    okvk, okvv = oracle_fill(og, k, v, is_swa)
    n = g.n_head * g.head_dim
    gate = (2 * rng.standard_normal((rows, n))).astype(np.float32)
    sgate = rng.uniform(0.5, 1.5, n).astype(np.float32)
    gd, sd = torch.from_numpy(gate).cuda(), torch.from_numpy(sgate).cuda()
    pos = dev_i32([depth], "cuda")
    part = eng.alloc_part(1, rows)
    qd = dev_q(eng, q)
    # fused
    dst = torch.zeros((rows, n), device="cuda")
    xq = torch.zeros((rows, n), dtype=torch.int8, device="cuda")
    xd = torch.zeros((rows, n // 32), device="cuda")
    xs = torch.zeros((rows, n // 32), dtype=torch.int32, device="cuda")
    eng.prefill_gate_norm(dst, qd, kvk, kvv, pos, part, gd, sd, xq, xd, xs, rows, is_swa)
    # two steps
    out = torch.zeros((1, rows, g.n_head, g.head_dim), dtype=eng.out_torch, device="cuda")
    eng.launch_attn_m(out, qd, kvk, kvv, pos, part, rows, is_swa)
    dst2 = torch.zeros_like(dst); xq2 = torch.zeros_like(xq); xd2 = torch.zeros_like(xd); xs2 = torch.zeros_like(xs)
    eng.gate_norm(dst2, out.view(rows, n), gd, sd, xq2, xd2, xs2, rows)
    torch.cuda.synchronize()
    assert eng.device_status() == 0
    # oracle: exact attention (double), then the restated gate-norm step
    want_a = O.attend(og, q, okvk, okvv, [depth], rows=rows, is_swa=is_swa)[0].reshape(rows, n)
    wdst, wxq, wxd, wxs = O.gate_norm(want_a, gate, sgate)
    for what, (d_, q_, xd_, xs_) in (("fused", (dst, xq, xd, xs)), ("two steps", (dst2, xq2, xd2, xs2))):
        d_, q_, xd_, xs_ = d_.cpu().numpy(), q_.cpu().numpy(), xd_.cpu().numpy(), xs_.cpu().numpy()
        # the normalised vector has unit length: compare per token row relative to its largest element
        err = np.abs(d_ - wdst).max(axis=1) / np.abs(wdst).max(axis=1)
        assert err.max() < (2e-3 if name == "B" else 1.2e-3), f"{what}: {err.max():.2e}"
        # the q8 copy is self-consistent and dequantises to the fp32 result within half a step
        assert (xs_ == q_.astype(np.int32).reshape(rows, -1, 32).sum(-1)).all()
        deq = q_.astype(np.float32).reshape(rows, -1, 32) * xd_[..., None]
        assert (np.abs(deq.reshape(rows, n) - d_) <= 0.5001 * np.repeat(xd_, 32, axis=1) + 1e-12).all()
        assert np.allclose(xd_, np.abs(d_).reshape(rows, -1, 32).max(-1) * np.float32(1 / 127), rtol=1e-6)
    # fused and two-step forms differ only by the rounding of the intermediate attention output
    assert np.abs(dst.cpu().numpy() - dst2.cpu().numpy()).max() < (5e-4 if name == "B" else 5e-6) * np.abs(wdst).max()
