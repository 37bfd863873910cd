"""A whole serving step captured ONCE into a CUDA graph and replayed at new positions, as the reference
does (bruce.cu:7877-7900, 8223-8241): RoPE tables -> fused QKV prologue + append -> multi-slot decode
attention on a full-causal and a sliding-window layer (as three launches per layer, or as the one call whose decode
kernel runs prologue and append itself), then the device-side position increment.  Positions,
slot map and activity flags live in device memory, so the same graph serves every token; no call allocates,
synchronises or reads on the host.  Every replayed step is checked against the oracle stepping alongside."""
import numpy as np
import pytest
import torch

from oracle import oracle as O
from tests.gpu_util import dev_i32
from tests.util import assert_close, oracle_geom

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("fused", [False, True])
def test_decode_step_graph_replays_at_new_positions(fused):
    from bruce_engine_b200.engine import AttnEngine
    from bruce_engine_b200.layout import G_B
    n_seq, steps = 4, 7
    g = G_B.with_(slot_ctx=512, window=64, n_slots=n_seq)
    eng, og = AttnEngine(g), oracle_geom(g)
    eng.set_early_kv_stream(True)          # append -> attention inside the graph: the order the option asks for
    HD = g.head_dim
    rng = np.random.default_rng(17)
    start = np.array([130, 0, 255, 61], dtype=np.int32)           # ragged; slot 3 crosses the window edge
    kslot = np.array([2, 0, 3, 1], dtype=np.int32)
    act = np.array([1, 1, 0, 1], dtype=np.int32)                  # sequence 2 is idle: no KV writes
    sqk = (8.0 + rng.standard_normal((g.n_head, HD))).astype(np.float32)

    layers = []
    for is_swa, theta in ((False, 1), (True, 2)):
        kvk, kvv = eng.alloc_kv_layer(is_swa, fill=0)
        okvk, okvv = O.new_cache(og, is_swa), O.new_cache(og, is_swa)
        # history before the captured steps: every active sequence already holds start[i] positions
        for i in range(n_seq):
            n0 = int(start[i])
            if n0 == 0 or not act[i]:
                continue
            kh = rng.standard_normal((1, n0, g.n_kv, HD), dtype=np.float32)
            vh = rng.standard_normal((1, n0, g.n_kv, HD), dtype=np.float32)
            O.kv_append(og, kh, vh, okvk, okvv, [0], kslot=[kslot[i]], rows=n0, is_swa=is_swa)
        kvk.copy_(torch.from_numpy(okvk).cuda())
        kvv.copy_(torch.from_numpy(okvv).cuda())
        layers.append(dict(is_swa=is_swa, theta=theta, kvk=kvk, kvv=kvv, okvk=okvk, okvv=okvv,
                           q16=torch.zeros((n_seq, 1, g.n_head, HD), dtype=torch.float16, device="cuda"),
                           out=torch.zeros((n_seq, 1, g.n_head, HD), dtype=torch.float16, device="cuda"),
                           part=eng.alloc_part(n_seq, 1)))

    # static device buffers the graph reads; the host refreshes their CONTENT between replays
    q_in = torch.zeros((n_seq, 1, g.n_head, HD), device="cuda")
    k_in = torch.zeros((n_seq, 1, g.n_kv, HD), device="cuda")
    v_in = torch.zeros((n_seq, 1, g.n_kv, HD), device="cuda")
    sqk_d = torch.from_numpy(sqk).cuda()
    cs = torch.zeros((n_seq, HD), device="cuda")
    sn = torch.zeros((n_seq, HD), device="cuda")
    pos_d, slot_d, act_d = dev_i32(start, "cuda"), dev_i32(kslot, "cuda"), dev_i32(act, "cuda")

    def step():
        eng.rope_tables(cs, sn, pos_d, rows=1)
        for L in layers:
            if fused:       # prologue, append and attention by the decode kernel itself (battn_qkv_decode)
                eng.qkv_decode(L["out"], q_in, k_in, v_in, sqk_d, cs, sn, L["kvk"], L["kvv"], pos_d, L["part"], kslot=slot_d,
                               act=act_d, is_swa=L["is_swa"], theta_sel=L["theta"])
                continue
            eng.qkv_prep(L["q16"], q_in, k_in, v_in, sqk_d, cs, sn, L["kvk"], L["kvv"], pos_d, kslot=slot_d, act=act_d,
                         rows=1, is_swa=L["is_swa"], theta_sel=L["theta"])
            eng.launch_attn_ms(L["out"], L["q16"], L["kvk"], L["kvv"], pos_d, slot_d, act_d, L["part"], n_seq, L["is_swa"])
        pos_d.add_(act_d)                                          # the next token's positions, on the device

    # warm-up on a side stream (sets lazy kernel attributes), then undo its effects and capture
    snap = [(L["kvk"].clone(), L["kvv"].clone()) for L in layers]
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        step()
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    for L, (a, b) in zip(layers, snap):
        L["kvk"].copy_(a)
        L["kvv"].copy_(b)
    pos_d.copy_(dev_i32(start, "cuda"))
    launches_before = eng.launch_count()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        step()
    per_step = eng.launch_count() - launches_before
    for L, (a, b) in zip(layers, snap):                            # capture does not execute; be explicit anyway
        L["kvk"].copy_(a)
        L["kvv"].copy_(b)
    pos_d.copy_(dev_i32(start, "cuda"))

    pos = start.copy()
    for t in range(steps):
        q = rng.standard_normal((n_seq, 1, g.n_head, HD), dtype=np.float32)
        k = rng.standard_normal((n_seq, 1, g.n_kv, HD), dtype=np.float32)
        v = rng.standard_normal((n_seq, 1, g.n_kv, HD), dtype=np.float32)
        q_in.copy_(torch.from_numpy(q).cuda())
        k_in.copy_(torch.from_numpy(k).cuda())
        v_in.copy_(torch.from_numpy(v).cuda())
        graph.replay()
        torch.cuda.synchronize()
        tables_c, tables_s = cs.cpu().numpy(), sn.cpu().numpy()     # the oracle takes the tables the device made
        wc, ws = O.rope_tables(HD, pos)
        assert np.abs(tables_c - wc).max() < 1e-4 and np.abs(tables_s - ws).max() < 1e-4
        for L in layers:
            q_want = O.qkv_prep(og, q, k, v, sqk, tables_c, tables_s, L["okvk"], L["okvv"], pos, kslot=kslot, act=act,
                                rows=1, is_swa=L["is_swa"], theta_sel=L["theta"])
            if not fused:
                assert (L["q16"].cpu().numpy().view(np.uint16) == q_want.astype(np.float16).view(np.uint16)).all()
            assert (L["kvk"].cpu().numpy() == L["okvk"]).all() and (L["kvv"].cpu().numpy() == L["okvv"]).all(), \
                f"cache bytes differ at step {t}"
            want = O.attend(og, q_want.astype(np.float16).astype(np.float32), L["okvk"], L["okvv"], pos, kslot=kslot,
                            act=act, rows=1, is_swa=L["is_swa"])
            got = L["out"].float().cpu().numpy()
            live = act.astype(bool)
            assert_close(got[live], want[live], f"graph step {t} swa={L['is_swa']}")
        pos = pos + act
        assert (pos_d.cpu().numpy() == pos).all()
    assert eng.device_status() == 0
    assert per_step == 1 + 2 * (2 if fused else 3), "one table kernel, then (prologue +) flash-decode + merge per layer"
