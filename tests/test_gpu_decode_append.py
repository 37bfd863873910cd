"""battn_decode_append: the decode call that appends its own row, through the C ABI.

Two copies of the same cache are stepped side by side with the same seeded rows: one by battn_kv_append followed by
battn_decode (both pinned to the CPU oracle by the other tests), one by battn_decode_append.  After every step the
outputs must be equal bit for bit, and at the end so must every byte of the two caches.  Covered: both geometries,
full-causal and sliding-window layers (the ring wraps inside the run), ragged multi-slot batches with idle rows, an
empty sequence (position 0), positions on both sides of a tile boundary, the paged cache, early KV streaming.  The
last test pins the call to the CPU oracle directly, inside a CUDA graph replayed at advancing positions."""
import numpy as np
import pytest
import torch

from tests.gpu_util import dev_i32, dev_q, gpu_fill, new_out
from tests.util import draw_qkv

pytestmark = pytest.mark.gpu


def _geom(name, **kw):
    from bruce_engine_b200.layout import F32, G_B, G_R
    base = {"B": G_B, "B32": G_B.with_(out_dtype=F32), "R": G_R}[name]
    return base.with_(**kw)


def _engine(g, early):
    from bruce_engine_b200.engine import AttnEngine
    eng = AttnEngine(g)
    eng.set_early_kv_stream(early)
    return eng


def _bits(t):
    return t.view(torch.int16 if t.element_size() == 2 else torch.int32)


@pytest.mark.parametrize("early", [False, True])
@pytest.mark.parametrize("name,is_swa", [("B32", False), ("B32", True), ("B", False), ("R", False), ("R", True)])
def test_decode_append_equals_append_then_decode(name, is_swa, early):
    window = 256
    lens = [0, 1, 15, 16, 17, 255, 500, 2 * window - 3, 1500, 4097]
    n_seq, steps = len(lens), 12
    g = _geom(name, slot_ctx=4352, n_slots=n_seq + 2, window=window)
    eng = _engine(g, early)
    dev = eng.device
    ka, va = eng.alloc_kv_layer(is_swa, fill=0x7F)
    slots = [1, 0, 3, 2, 5, 4, 7, 6, 9, 11]                      # slot 8 and 10 stay untouched
    for i, n in enumerate(lens):
        if n:
            _, k, v = draw_qkv(g, n, 1, 700 + i)
            gpu_fill(eng, k, v, ka, va, is_swa, slot=slots[i])
    torch.cuda.synchronize()
    kb, vb = ka.clone(), va.clone()
    part = eng.alloc_part(n_seq, 1)
    kslot = dev_i32(slots, dev)
    rng = np.random.default_rng(5)
    for s in range(steps):
        act_np = (rng.random(n_seq) < 0.8).astype(np.int32)
        act_np[s % n_seq] = 0
        pos_np = np.array(lens, dtype=np.int32)
        q, k, v = draw_qkv(g, n_seq, 1, 900 + s, n_seq=n_seq, q_f16=(g.q_dtype == 1))
        qd = dev_q(eng, q[:, 0])
        kd = torch.from_numpy(k).to(dev)
        vd = torch.from_numpy(v).to(dev)
        pos, act = dev_i32(pos_np, dev), dev_i32(act_np, dev)
        oa = new_out(eng, n_seq, g.n_head, g.head_dim)
        ob = new_out(eng, n_seq, g.n_head, g.head_dim)
        eng.qkv_prep_store(kd, vd, ka, va, pos, kslot=kslot, act=act, is_swa=is_swa)
        eng.launch_attn_ms(oa, qd, ka, va, pos, kslot, act, part, n_seq, is_swa=is_swa)
        eng.decode_append(ob, qd, kd, vd, kb, vb, pos, part, kslot=kslot, act=act, is_swa=is_swa)
        torch.cuda.synchronize()
        assert eng.device_status() == 0
        assert torch.equal(_bits(oa), _bits(ob)), f"step {s}: outputs differ"
        live = torch.from_numpy(act_np.astype(bool)).to(dev)
        assert not torch.isnan(ob[live].float()).any() and torch.isnan(ob[~live].float()).all()
        lens = [n + int(a) for n, a in zip(lens, act_np)]
    assert torch.equal(ka, kb) and torch.equal(va, vb)


def test_decode_append_single_sequence_without_slot_tables():
    g = _geom("B32", slot_ctx=2048, n_slots=1)
    eng = _engine(g, True)
    dev = eng.device
    ka, va = eng.alloc_kv_layer(False, fill=0x7F)
    _, k, v = draw_qkv(g, 1000, 1, 3)
    gpu_fill(eng, k, v, ka, va, False)
    kb, vb = ka.clone(), va.clone()
    part = eng.alloc_part(1, 1)
    for s in range(20):
        q, k, v = draw_qkv(g, 1, 1, 40 + s)
        qd, kd, vd = dev_q(eng, q[:, 0]), torch.from_numpy(k).to(dev), torch.from_numpy(v).to(dev)
        pos = dev_i32([1000 + s], dev)
        oa, ob = new_out(eng, 1, g.n_head, g.head_dim), new_out(eng, 1, g.n_head, g.head_dim)
        eng.qkv_prep_store(kd, vd, ka, va, pos)
        eng.launch_attn_m(oa, qd, ka, va, pos, part, 1)
        eng.decode_append(ob, qd, kd, vd, kb, vb, pos, part)
        assert torch.equal(_bits(oa), _bits(ob))
    assert torch.equal(ka, kb) and torch.equal(va, vb)


@pytest.mark.parametrize("name", ["B32", "R"])
def test_decode_append_paged(name):
    page_len, lens = 128, [0, 127, 128, 300, 1000]
    n_seq, steps = len(lens), 10
    max_pages = 10
    g = _geom(name, slot_ctx=page_len * max_pages, n_slots=n_seq)
    eng = _engine(g, True)
    dev = eng.device
    rng = np.random.default_rng(11)
    n_pages = n_seq * max_pages + 2
    table_np = rng.permutation(n_pages)[:n_seq * max_pages].reshape(n_seq, max_pages).astype(np.int32)
    table = torch.from_numpy(table_np).to(dev)
    pa, pak, pav = eng.alloc_pages(n_pages, page_len, table, fill=0x7F)
    for i, n in enumerate(lens):
        if n:
            _, k, v = draw_qkv(g, n, 1, 70 + i)
            kd, vd = torch.from_numpy(k).to(dev), torch.from_numpy(v).to(dev)
            for a in range(0, n, 512):
                b = min(n, a + 512)
                eng.kv_append_paged(pa, kd[a:b], vd[a:b], dev_i32([a], dev), ktab=dev_i32([i], dev), rows=b - a)
    torch.cuda.synchronize()
    pb, pbk, pbv = eng.alloc_pages(n_pages, page_len, table)
    pbk.copy_(pak)
    pbv.copy_(pav)
    part = eng.alloc_part(n_seq, 1)
    ktab = dev_i32(range(n_seq), dev)
    for s in range(steps):
        act_np = np.ones(n_seq, dtype=np.int32)
        act_np[s % n_seq] = 0
        q, k, v = draw_qkv(g, n_seq, 1, 300 + s, n_seq=n_seq, q_f16=(g.q_dtype == 1))
        qd, kd, vd = dev_q(eng, q[:, 0]), torch.from_numpy(k).to(dev), torch.from_numpy(v).to(dev)
        pos, act = dev_i32(lens, dev), dev_i32(act_np, dev)
        oa, ob = new_out(eng, n_seq, g.n_head, g.head_dim), new_out(eng, n_seq, g.n_head, g.head_dim)
        eng.kv_append_paged(pa, kd, vd, pos, ktab=ktab, act=act)
        eng.attn_paged(oa, qd, pa, pos, part, rows=1, ktab=ktab, act=act)
        eng.decode_append_paged(ob, qd, kd, vd, pb, pos, part, ktab=ktab, act=act)
        torch.cuda.synchronize()
        assert eng.device_status() == 0
        assert torch.equal(_bits(oa), _bits(ob)), f"step {s}: outputs differ"
        lens = [n + int(a) for n, a in zip(lens, act_np)]
    assert torch.equal(pak, pbk) and torch.equal(pav, pbv)


def test_decode_append_in_a_replayed_graph_against_the_oracle():
    """The appending decode captured once and replayed at device-resident positions that advance on the device;
    cache bytes and outputs of every replay against the CPU oracle (append, then attend)."""
    from oracle import oracle as O
    from tests.util import assert_close, oracle_geom
    n_seq, steps = 4, 6
    g = _geom("B", slot_ctx=512, window=64, n_slots=n_seq)
    eng, og = _engine(g, True), oracle_geom(g)
    dev = eng.device
    rng = np.random.default_rng(23)
    start = np.array([130, 0, 255, 61], dtype=np.int32)           # ragged; the last one crosses the window edge
    kslot = np.array([2, 0, 3, 1], dtype=np.int32)
    act = np.array([1, 1, 0, 1], dtype=np.int32)
    layers = []
    for is_swa in (False, True):
        okvk, okvv = O.new_cache(og, is_swa), O.new_cache(og, is_swa)
        for i in range(n_seq):
            n0 = int(start[i])
            if n0 and act[i]:
                kh = rng.standard_normal((1, n0, g.n_kv, g.head_dim), dtype=np.float32)
                vh = rng.standard_normal((1, n0, g.n_kv, g.head_dim), dtype=np.float32)
                O.kv_append(og, kh, vh, okvk, okvv, [0], kslot=[kslot[i]], rows=n0, is_swa=is_swa)
        layers.append(dict(is_swa=is_swa, okvk=okvk, okvv=okvv, kvk=torch.from_numpy(okvk).to(dev),
                           kvv=torch.from_numpy(okvv).to(dev), out=new_out(eng, n_seq, g.n_head, g.head_dim),
                           part=eng.alloc_part(n_seq, 1)))
    q_in = torch.zeros((n_seq, g.n_head, g.head_dim), dtype=torch.float16, device=dev)
    k_in = torch.zeros((n_seq, g.n_kv, g.head_dim), device=dev)
    v_in = torch.zeros((n_seq, g.n_kv, g.head_dim), device=dev)
    pos_d, slot_d, act_d = dev_i32(start, dev), dev_i32(kslot, dev), dev_i32(act, dev)

    def step():
        for L in layers:
            eng.decode_append(L["out"], q_in, k_in, v_in, L["kvk"], L["kvv"], pos_d, L["part"], kslot=slot_d, act=act_d,
                              is_swa=L["is_swa"])
        pos_d.add_(act_d)

    snap = [(L["kvk"].clone(), L["kvv"].clone()) for L in layers]
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        step()
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        step()
    for L, (a, b) in zip(layers, snap):
        L["kvk"].copy_(a)
        L["kvv"].copy_(b)
    pos_d.copy_(dev_i32(start, dev))
    pos = start.copy()
    for t in range(steps):
        q = rng.standard_normal((n_seq, 1, g.n_head, g.head_dim), dtype=np.float32).astype(np.float16).astype(np.float32)
        k = rng.standard_normal((n_seq, 1, g.n_kv, g.head_dim), dtype=np.float32)
        v = rng.standard_normal((n_seq, 1, g.n_kv, g.head_dim), dtype=np.float32)
        q_in.copy_(torch.from_numpy(q[:, 0]).to(dev))
        k_in.copy_(torch.from_numpy(k[:, 0]).to(dev))
        v_in.copy_(torch.from_numpy(v[:, 0]).to(dev))
        graph.replay()
        torch.cuda.synchronize()
        for L in layers:
            O.kv_append(og, k, v, L["okvk"], L["okvv"], pos, kslot=kslot, act=act, rows=1, is_swa=L["is_swa"])
            assert (L["kvk"].cpu().numpy() == L["okvk"]).all() and (L["kvv"].cpu().numpy() == L["okvv"]).all(), \
                f"cache bytes differ at step {t}"
            want = O.attend(og, q, L["okvk"], L["okvv"], pos, kslot=kslot, act=act, rows=1, is_swa=L["is_swa"])
            got = L["out"].float().cpu().numpy()
            live = act.astype(bool)
            assert_close(got[live], want[live][:, 0] if want.ndim == 4 else want[live],
                         f"appending decode in a graph, step {t} swa={L['is_swa']}")
        pos = pos + act
        assert (pos_d.cpu().numpy() == pos).all()
    assert eng.device_status() == 0


@pytest.mark.parametrize("name", ["B32", "R"])
def test_consecutive_appending_decodes_on_one_cache_without_a_sync(name):
    """Forty appending decode calls on the SAME cache queued back to back with early KV streaming on, across several
    tile boundaries: the merge of call n releases call n + 1 before the decode kernel of call n (which writes the
    row call n + 1 reads) has finished, so the library must not let call n + 1 stream that cache early."""
    g = _geom(name, slot_ctx=1024, n_slots=1)
    eng = _engine(g, True)
    dev = eng.device
    n0, steps = 100, 40
    ka, va = eng.alloc_kv_layer(False, fill=0x7F)
    _, k, v = draw_qkv(g, n0, 1, 9)
    gpu_fill(eng, k, v, ka, va, False)
    kb, vb = ka.clone(), va.clone()
    part = eng.alloc_part(1, 1)
    q, k, v = draw_qkv(g, steps, 1, 77, n_seq=steps, q_f16=(g.q_dtype == 1))
    qd, kd, vd = dev_q(eng, q[:, 0]), torch.from_numpy(k).to(dev), torch.from_numpy(v).to(dev)
    pos = [dev_i32([n0 + s], dev) for s in range(steps)]
    oa = new_out(eng, steps, g.n_head, g.head_dim)
    ob = new_out(eng, steps, g.n_head, g.head_dim)
    torch.cuda.synchronize()
    for s in range(steps):
        eng.decode_append(ob[s:s + 1], qd[s:s + 1], kd[s:s + 1], vd[s:s + 1], kb, vb, pos[s], part)
    for s in range(steps):
        eng.qkv_prep_store(kd[s:s + 1], vd[s:s + 1], ka, va, pos[s])
        eng.launch_attn_m(oa[s:s + 1], qd[s:s + 1], ka, va, pos[s], part, 1)
    torch.cuda.synchronize()
    assert eng.device_status() == 0
    assert torch.equal(_bits(oa), _bits(ob))
    assert torch.equal(ka, kb) and torch.equal(va, vb)


@pytest.mark.parametrize("name,is_swa", [("B32", False), ("B32", True), ("R", False), ("R", True)])
def test_qkv_decode_equals_prologue_then_decode(name, is_swa):
    """battn_qkv_decode (the decode kernel runs the QKV prologue of its row) against battn_qkv_prep followed by
    battn_decode -- both pinned to the reference's own kernels and to the oracle by other tests -- on two copies of a
    cache stepped side by side: equal output bits every step, equal cache bytes at the end."""
    window = 256
    lens = [0, 1, 63, 64, 65, 300, 2 * window - 2, 1500]
    n_seq, steps = len(lens), 8
    g = _geom(name, slot_ctx=2048, n_slots=n_seq + 1, window=window)
    eng = _engine(g, True)
    dev = eng.device
    HD = g.head_dim
    ka, va = eng.alloc_kv_layer(is_swa, fill=0x7F)
    slots = [1, 0, 3, 2, 5, 4, 8, 6]
    for i, n in enumerate(lens):
        if n:
            _, k, v = draw_qkv(g, n, 1, 1700 + i)
            gpu_fill(eng, k, v, ka, va, is_swa, slot=slots[i])
    torch.cuda.synchronize()
    kb, vb = ka.clone(), va.clone()
    part = eng.alloc_part(n_seq, 1)
    kslot = dev_i32(slots, dev)
    rng = np.random.default_rng(31)
    sqk = torch.from_numpy((8.0 + rng.standard_normal((g.n_head, HD))).astype(np.float32)).to(dev)
    cs = torch.zeros((n_seq, HD), device=dev)
    sn = torch.zeros((n_seq, HD), device=dev)
    theta = 2 if is_swa else 1
    for s in range(steps):
        act_np = (rng.random(n_seq) < 0.8).astype(np.int32)
        act_np[s % n_seq] = 0
        q = torch.from_numpy(rng.standard_normal((n_seq, 1, g.n_head, HD), dtype=np.float32)).to(dev)
        k = torch.from_numpy(rng.standard_normal((n_seq, 1, g.n_kv, HD), dtype=np.float32)).to(dev)
        v = torch.from_numpy(rng.standard_normal((n_seq, 1, g.n_kv, HD), dtype=np.float32)).to(dev)
        pos, act = dev_i32(lens, dev), dev_i32(act_np, dev)
        eng.rope_tables(cs, sn, pos, rows=1)
        qp = torch.zeros((n_seq, 1, g.n_head, HD), dtype=eng.q_torch, device=dev)
        oa = new_out(eng, n_seq, g.n_head, HD)
        ob = new_out(eng, n_seq, g.n_head, HD)
        eng.qkv_prep(qp, q, k, v, sqk, cs, sn, ka, va, pos, kslot=kslot, act=act, rows=1, is_swa=is_swa, theta_sel=theta)
        eng.launch_attn_ms(oa, qp, ka, va, pos, kslot, act, part, n_seq, is_swa=is_swa)
        eng.qkv_decode(ob, q, k, v, sqk, cs, sn, kb, vb, pos, part, kslot=kslot, act=act, is_swa=is_swa, theta_sel=theta)
        torch.cuda.synchronize()
        assert eng.device_status() == 0
        assert torch.equal(_bits(oa), _bits(ob)), f"step {s}: outputs differ"
        live = torch.from_numpy(act_np.astype(bool)).to(dev)
        assert not torch.isnan(ob[live].float()).any() and torch.isnan(ob[~live].float()).all()
        lens = [n + int(a) for n, a in zip(lens, act_np)]
    assert torch.equal(ka, kb) and torch.equal(va, vb)


def test_qkv_decode_paged():
    """The fused decode step over a paged cache against battn_qkv_prep_paged + battn_decode_paged."""
    page_len, lens = 128, [0, 127, 128, 300, 900]
    n_seq, steps, max_pages = len(lens), 6, 8
    g = _geom("B32", slot_ctx=page_len * max_pages, n_slots=n_seq)
    eng = _engine(g, True)
    dev, HD = eng.device, g.head_dim
    rng = np.random.default_rng(41)
    n_pages = n_seq * max_pages + 2
    table = torch.from_numpy(rng.permutation(n_pages)[:n_seq * max_pages].reshape(n_seq, max_pages).astype(np.int32)).to(dev)
    pa, pak, pav = eng.alloc_pages(n_pages, page_len, table, fill=0x7F)
    for i, n in enumerate(lens):
        if n:
            _, k, v = draw_qkv(g, n, 1, 170 + i)
            kd, vd = torch.from_numpy(k).to(dev), torch.from_numpy(v).to(dev)
            for a in range(0, n, 512):
                b = min(n, a + 512)
                eng.kv_append_paged(pa, kd[a:b], vd[a:b], dev_i32([a], dev), ktab=dev_i32([i], dev), rows=b - a)
    torch.cuda.synchronize()
    pb, pbk, pbv = eng.alloc_pages(n_pages, page_len, table)
    pbk.copy_(pak)
    pbv.copy_(pav)
    part = eng.alloc_part(n_seq, 1)
    ktab = dev_i32(range(n_seq), dev)
    sqk = torch.from_numpy((8.0 + rng.standard_normal((g.n_head, HD))).astype(np.float32)).to(dev)
    cs, sn = torch.zeros((n_seq, HD), device=dev), torch.zeros((n_seq, HD), device=dev)
    for s in range(steps):
        act_np = np.ones(n_seq, dtype=np.int32)
        act_np[s % n_seq] = 0
        q = torch.from_numpy(rng.standard_normal((n_seq, 1, g.n_head, HD), dtype=np.float32)).to(dev)
        k = torch.from_numpy(rng.standard_normal((n_seq, 1, g.n_kv, HD), dtype=np.float32)).to(dev)
        v = torch.from_numpy(rng.standard_normal((n_seq, 1, g.n_kv, HD), dtype=np.float32)).to(dev)
        pos, act = dev_i32(lens, dev), dev_i32(act_np, dev)
        eng.rope_tables(cs, sn, pos, rows=1)
        qp = torch.zeros((n_seq, 1, g.n_head, HD), dtype=eng.q_torch, device=dev)
        oa, ob = new_out(eng, n_seq, g.n_head, HD), new_out(eng, n_seq, g.n_head, HD)
        eng.qkv_prep_paged(qp, q, k, v, sqk, cs, sn, pa, pos, ktab=ktab, act=act, rows=1)
        eng.attn_paged(oa, qp, pa, pos, part, rows=1, ktab=ktab, act=act)
        eng.qkv_decode_paged(ob, q, k, v, sqk, cs, sn, pb, pos, part, ktab=ktab, act=act)
        torch.cuda.synchronize()
        assert eng.device_status() == 0
        assert torch.equal(_bits(oa), _bits(ob)), f"step {s}: outputs differ"
        lens = [n + int(a) for n, a in zip(lens, act_np)]
    assert torch.equal(pak, pbk) and torch.equal(pav, pbv)
