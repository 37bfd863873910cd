"""The shapes the host-side control produces, on the real kernels:
  * a batched multi-slot decode step gives every slot what the same slot gets when it runs alone (the reference's
    own --ms-test check, bruce.cu:8109-8221);
  * one captured launch sequence per verify row count (2..8), replayed at advancing device-resident positions, gives
    what eager calls give (capture_verify_graphs, bruce.cu:7877-7900);
  * prefix sharing between slots: a copied prefix is byte-identical and attends like the original."""
import numpy as np
import pytest
import torch

from oracle import oracle as O
from tests.gpu_util import dev_i32, dev_q, gpu_fill, new_out, to_np
from tests.util import assert_close, draw_qkv, oracle_fill, oracle_geom

pytestmark = pytest.mark.gpu


def _engine(**kw):
    from bruce_engine_b200.engine import AttnEngine
    from bruce_engine_b200.layout import G_B
    g = G_B.with_(**kw)
    return g, AttnEngine(g)


@pytest.mark.parametrize("is_swa", [False, True])
def test_batched_rows_equal_per_slot_rows(is_swa):
    g, eng = _engine(slot_ctx=4096, window=512, n_slots=12)
    lens = [4096, 37, 1500, 2049, 640, 4000, 1, 777, 3333, 129, 2500, 64]
    kvk, kvv = eng.alloc_kv_layer(is_swa, fill=0)
    for s, n in enumerate(lens):
        _, k, v = draw_qkv(g, n, 1, seed=500 + s)
        gpu_fill(eng, k, v, kvk, kvv, is_swa, slot=s)
    rng = np.random.default_rng(3)
    q = torch.from_numpy(rng.standard_normal((12, 1, g.n_head, g.head_dim), dtype=np.float32)).cuda().half()
    pos = dev_i32([n - 1 for n in lens], "cuda")
    kslot = dev_i32(list(range(12)), "cuda")
    part = eng.alloc_part(12, 1)
    batched = new_out(eng, 12, 1, g.n_head, g.head_dim)
    eng.launch_attn_ms(batched, q, kvk, kvv, pos, kslot, None, part, 12, is_swa)
    alone = new_out(eng, 12, 1, g.n_head, g.head_dim)
    for s in range(12):
        eng.launch_attn_ms(alone[s:s + 1], q[s:s + 1], kvk, kvv, pos[s:s + 1], kslot[s:s + 1], None, part, 1, is_swa)
    torch.cuda.synchronize()
    assert_close(to_np(batched), to_np(alone), f"batched step vs one slot at a time, swa={is_swa}")
    assert eng.device_status() == 0


def test_one_graph_per_verify_row_count_replayed_at_new_positions():
    g, eng = _engine(slot_ctx=2048, window=256)
    og = oracle_geom(g)
    n = 1800
    q_all, k, v = draw_qkv(g, n, 8, seed=8)
    kvk, kvv = eng.alloc_kv_layer(False, fill=0)
    gpu_fill(eng, k, v, kvk, kvv, False)
    okvk, okvv = oracle_fill(og, k, v, False)
    part = eng.alloc_part(1, 8)
    pos = dev_i32([0], "cuda")                                 # device-resident: the graphs read it at replay time
    graphs, bufs = {}, {}
    for rows in range(2, 9):
        qd = dev_q(eng, q_all[:, :rows])
        out = new_out(eng, 1, rows, g.n_head, g.head_dim)
        eng.launch_attn_m(out, qd, kvk, kvv, pos, part, rows)            # warm-up outside capture
        torch.cuda.synchronize()
        gr = torch.cuda.CUDAGraph()
        with torch.cuda.graph(gr):
            eng.launch_attn_m(out, qd, kvk, kvv, pos, part, rows)
        graphs[rows], bufs[rows] = gr, (qd, out)
    p = 1000
    for rows in (3, 8, 2, 5, 8, 7, 4, 6):                     # rounds of varying width, each advancing the position
        pos.fill_(p)
        graphs[rows].replay()
        torch.cuda.synchronize()
        want = O.attend(og, q_all[:, :rows], okvk, okvv, [p], rows=rows)
        assert_close(to_np(bufs[rows][1]), want, f"verify graph rows={rows} at p0={p}")
        p += rows
    assert eng.device_status() == 0


@pytest.mark.parametrize("is_swa", [False, True])
def test_prefix_copied_between_slots_is_identical_and_attends_alike(is_swa):
    g, eng = _engine(slot_ctx=2048, window=256, n_slots=3)
    og = oracle_geom(g)
    n_shared, n_total = 1331, 1700
    _, k, v = draw_qkv(g, n_total, 1, seed=21)
    kvk, kvv = eng.alloc_kv_layer(is_swa, fill=0)
    gpu_fill(eng, k[:n_shared], v[:n_shared], kvk, kvv, is_swa, slot=0)
    eng.kv_copy_prefix(kvk, kvv, 0, 2, n_shared, is_swa)
    torch.cuda.synchronize()
    per_slot = g.layer_bytes(is_swa) // g.n_slots
    a, b = kvk.cpu().numpy(), kvv.cpu().numpy()
    for buf in (a, b):
        src, dst = buf[:per_slot].reshape(g.n_kv, -1, g.rec), buf[2 * per_slot:].reshape(g.n_kv, -1, g.rec)
        if is_swa:
            live = sorted({p & (2 * g.window - 1) for p in range(max(0, n_shared - 2 * g.window), n_shared)})
        else:
            live = list(range(n_shared))
        assert (dst[:, live] == src[:, live]).all()
        assert (buf[per_slot:2 * per_slot] == 0).all()                    # the slot in between is untouched
    # the rest of the prompt goes to the copy only; it must attend like a cache filled from scratch
    gpu_fill(eng, k[n_shared:], v[n_shared:], kvk, kvv, is_swa, slot=2, start=n_shared)
    okvk, okvv = oracle_fill(og, k, v, is_swa, slot=2)
    rng = np.random.default_rng(2)
    q = rng.standard_normal((1, 1, g.n_head, g.head_dim), dtype=np.float32).astype(np.float16).astype(np.float32)
    out = new_out(eng, 1, 1, g.n_head, g.head_dim)
    eng.launch_attn_ms(out, dev_q(eng, q), kvk, kvv, dev_i32([n_total - 1], "cuda"), dev_i32([2], "cuda"), None,
                       eng.alloc_part(1, 1), 1, is_swa)
    torch.cuda.synchronize()
    want = O.attend(og, q, okvk, okvv, [n_total - 1], kslot=[2], rows=1, is_swa=is_swa)
    assert_close(to_np(out), want, f"decode on a copied prefix, swa={is_swa}")
    assert eng.device_status() == 0


def test_early_kv_streaming_waits_when_the_previous_launch_wrote_other_rows():
    """With early KV streaming on, a decode that directly follows a prefix copy into its slot, or the append of a
    300-row chunk, must still see those rows: the library streams early only behind the append of the call's own rows."""
    g, eng = _engine(slot_ctx=2048, window=256, n_slots=2)
    eng.set_early_kv_stream(True)
    og = oracle_geom(g)
    n0, n1 = 1500, 1800
    _, k, v = draw_qkv(g, n1, 1, seed=33)
    kvk, kvv = eng.alloc_kv_layer(False, fill=0)
    gpu_fill(eng, k[:n0], v[:n0], kvk, kvv, False, slot=0)
    okvk, okvv = oracle_fill(og, k[:n0], v[:n0], False, slot=0)
    rng = np.random.default_rng(3)
    q = rng.standard_normal((1, 1, g.n_head, g.head_dim), dtype=np.float32).astype(np.float16).astype(np.float32)
    qd, part = dev_q(eng, q), eng.alloc_part(1, 1)
    want = O.attend(og, q, okvk, okvv, [n0 - 1], kslot=[0], rows=1)
    per_slot = g.layer_bytes(False) // g.n_slots
    pos, one = dev_i32([n0 - 1], "cuda"), dev_i32([1], "cuda")
    for trial in range(4):
        kvk[per_slot:].zero_()
        kvv[per_slot:].zero_()
        out = new_out(eng, 1, 1, g.n_head, g.head_dim)
        eng.kv_copy_prefix(kvk, kvv, 0, 1, n0)                       # no synchronisation before the decode
        eng.launch_attn_ms(out, qd, kvk, kvv, pos, one, None, part, 1)
        torch.cuda.synchronize()
        assert_close(to_np(out), want, f"decode right behind a prefix copy, trial {trial}")
    # a 300-row chunk appended at n0, then a decode at the chunk's last row through another position buffer
    kd, vd = torch.from_numpy(k[n0:]).cuda(), torch.from_numpy(v[n0:]).cuda()
    out = new_out(eng, 1, 1, g.n_head, g.head_dim)
    eng.qkv_prep_store(kd, vd, kvk, kvv, dev_i32([n0], "cuda"), kslot=dev_i32([0], "cuda"), rows=n1 - n0)
    eng.launch_attn_ms(out, qd, kvk, kvv, dev_i32([n1 - 1], "cuda"), dev_i32([0], "cuda"), None, part, 1)
    torch.cuda.synchronize()
    okvk, okvv = oracle_fill(og, k, v, False, slot=0)
    assert_close(to_np(out), O.attend(og, q, okvk, okvv, [n1 - 1], kslot=[0], rows=1), "decode right behind a chunk append")
    assert eng.device_status() == 0
