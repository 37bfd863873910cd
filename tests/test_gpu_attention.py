"""Parity of the CUDA attention paths with the CPU oracle, through the C ABI.

Tolerance (fp32-accumulated outputs): max-abs <= 2e-3; per (row, head) and per token row
||diff||_2 / ||ref||_2 <= 1e-3; per (row, head) max|diff| / max|ref| <= 1e-3 on fp32 outputs (the "R" and "B32"
geometries; tests/util.py explains why not on fp16 outputs).  KV bytes are produced by the append kernel under test and compared with
the oracle's bytes before any attention is checked."""
import numpy as np
import pytest
import torch

from oracle import oracle as O
from tests.gpu_util import dev_i32, dev_q, gpu_fill, new_out, to_np
from tests.util import assert_close, draw_qkv, oracle_fill, oracle_geom

pytestmark = pytest.mark.gpu


def _geom(name, **kw):
    """"B": the graded geometry (fp16 q and out); "B32": the same with fp32 outputs, where the max-norm ratio is
    gated as well (tests/util.py); "R": the reference's own geometry (fp32 q and out)."""
    from bruce_engine_b200.layout import F32, G_B, G_R
    base = {"B": G_B, "B32": G_B.with_(out_dtype=F32), "R": G_R}[name]
    return base.with_(**kw)


def _engine(g):
    """Early KV streaming on: positions reach the device by copies and the kernel before an attention call is this
    library's append or merge, the order the option asks for; every case below therefore also checks that path."""
    from bruce_engine_b200.engine import AttnEngine
    eng = AttnEngine(g)
    eng.set_early_kv_stream(True)
    return eng


class Case:
    """One sequence's cache on both sides, filled from the same seeded K/V."""

    def __init__(self, g, n, is_swa, seed=0, rows_q=8):
        self.g, self.n, self.is_swa = g, n, is_swa
        self.eng = _engine(g)
        self.og = oracle_geom(g)
        self.q, k, v = draw_qkv(g, n, rows_q, seed, q_f16=(g.q_dtype == 1))
        self.kvk, self.kvv = self.eng.alloc_kv_layer(is_swa, fill=0x7F)
        gpu_fill(self.eng, k, v, self.kvk, self.kvv, is_swa)
        self.okvk, self.okvv = O.new_cache(self.og, is_swa, fill=0x7F), O.new_cache(self.og, is_swa, fill=0x7F)
        oracle_fill(self.og, k, v, is_swa, kvk=self.okvk, kvv=self.okvv)
        assert (self.kvk.cpu().numpy() == self.okvk).all() and (self.kvv.cpu().numpy() == self.okvv).all()
        self.part = self.eng.alloc_part(1, 8)

    def run(self, p0, rows):
        g, eng = self.g, self.eng
        q = self.q[:, :rows]
        out = new_out(eng, 1, rows, g.n_head, g.head_dim)
        eng.launch_attn_m(out, dev_q(eng, q), self.kvk, self.kvv, dev_i32([p0], eng.device), self.part, rows,
                          self.is_swa)
        torch.cuda.synchronize()
        want = O.attend(self.og, q, self.okvk, self.okvv, [p0], rows=rows, is_swa=self.is_swa)
        return to_np(out), want


@pytest.mark.parametrize("name", ["B", "B32", "R"])
def test_decode_config0_8k_full_causal(name):
    """BASELINE config 0: batch 1, context 8192, one query row at position 8191, seed 0."""
    c = Case(_geom(name, slot_ctx=8192), 8192, False, seed=0)
    got, want = c.run(8191, 1)
    assert_close(got, want, f"decode 8K {name}")
    assert c.eng.device_status() == 0


@pytest.mark.parametrize("name", ["B", "B32", "R"])
@pytest.mark.parametrize("is_swa", [False, True])
def test_decode_position_edges(name, is_swa):
    """Positions around tile (64), window and ring boundaries; non-multiples of the tile."""
    g = _geom(name, slot_ctx=1024, window=128)
    W = g.window
    n = 2 * W + 200 if is_swa else 1000
    c = Case(g, n, is_swa, seed=1)
    pts = [0, 1, 62, 63, 64, 65, 127, 128, 129, W - 1, W, W + 1, 2 * W - 1, 2 * W, 2 * W + 1, n - 1]
    for p in sorted(set(pts)):
        if p >= n:
            continue
        if is_swa and p + 1 < n - W:            # the ring no longer holds this row's window
            continue
        got, want = c.run(p, 1)
        assert_close(got, want, f"{name} swa={is_swa} pos={p}")
    assert c.eng.device_status() == 0


@pytest.mark.parametrize("name", ["B", "B32", "R"])
@pytest.mark.parametrize("is_swa", [False, True])
def test_verify_rows_share_one_kv_sweep(name, is_swa):
    """rows 1..8 at p0..p0+rows-1, causal among themselves (bruce.cu:2056, 3686-3689)."""
    g = _geom(name, slot_ctx=1024, window=128)
    n = 2 * g.window + 150 if is_swa else 900
    c = Case(g, n, is_swa, seed=2)
    for rows in range(1, 9):
        for p0 in (n - rows, n - rows - 61, 0 if not is_swa else n - g.window - rows + 3):
            if p0 < 0:
                continue
            got, want = c.run(p0, rows)
            assert_close(got, want, f"{name} swa={is_swa} rows={rows} p0={p0}")
    assert c.eng.device_status() == 0


@pytest.mark.parametrize("name", ["B", "B32", "R"])
def test_multi_slot_decode_and_idle_rows(name):
    """launch_attn_ms: independent sequences with their own partition and position; idle rows
    produce no output (bruce.cu:3398-3406)."""
    g = _geom(name, slot_ctx=2048, window=256, n_slots=6)
    eng, og = _engine(g), oracle_geom(_geom(name, slot_ctx=2048, window=256, n_slots=6))
    lens = [1, 70, 2048, 700, 1333, 64]
    for is_swa in (False, True):
        kvk, kvv = eng.alloc_kv_layer(is_swa, fill=0x7F)
        okvk, okvv = O.new_cache(og, is_swa, fill=0x7F), O.new_cache(og, is_swa, fill=0x7F)
        for s, n in enumerate(lens):
            _, k, v = draw_qkv(g, n, 1, seed=100 + s)
            gpu_fill(eng, k, v, kvk, kvv, is_swa, slot=s)
            oracle_fill(og, k, v, is_swa, slot=s, kvk=okvk, kvv=okvv)
        assert (kvk.cpu().numpy() == okvk).all() and (kvv.cpu().numpy() == okvv).all()
        # rows in a permuted slot order, one idle
        kslot = [4, 0, 2, 5, 1, 3]
        act = [1, 1, 1, 0, 1, 1]
        pos = [lens[s] - 1 for s in kslot]
        rng = np.random.default_rng(5)
        q = rng.standard_normal((6, 1, g.n_head, g.head_dim), dtype=np.float32)
        if g.q_dtype == 1:
            q = q.astype(np.float16).astype(np.float32)
        out = new_out(eng, 6, 1, g.n_head, g.head_dim)
        part = eng.alloc_part(6, 1)
        eng.launch_attn_ms(out, dev_q(eng, q), kvk, kvv, dev_i32(pos, eng.device), dev_i32(kslot, eng.device),
                           dev_i32(act, eng.device), part, 6, is_swa)
        torch.cuda.synchronize()
        got = to_np(out)
        want = O.attend(og, q, okvk, okvv, pos, kslot=kslot, act=act, rows=1, is_swa=is_swa)
        live = np.array(act, dtype=bool)
        assert np.isnan(got[~live]).all(), "idle row was written"
        assert_close(got[live], want[live], f"multi-slot {name} swa={is_swa}")
    assert eng.device_status() == 0


def test_batched_verify_multi_slot():
    """Config 3 shape at small size: several sequences x 8 rows in one call."""
    g = _geom("B", slot_ctx=1024, window=128, n_slots=3)
    eng, og = _engine(g), oracle_geom(g)
    lens = [900, 333, 64]
    kvk, kvv = eng.alloc_kv_layer(False, fill=0)
    okvk, okvv = O.new_cache(og, False), O.new_cache(og, False)
    for s, n in enumerate(lens):
        _, k, v = draw_qkv(g, n, 1, seed=200 + s)
        gpu_fill(eng, k, v, kvk, kvv, False, slot=s)
        oracle_fill(og, k, v, False, slot=s, kvk=okvk, kvv=okvv)
    rows = 8
    pos = [n - rows for n in lens]
    rng = np.random.default_rng(6)
    q = rng.standard_normal((3, rows, g.n_head, g.head_dim), dtype=np.float32).astype(np.float16).astype(np.float32)
    out = new_out(eng, 3, rows, g.n_head, g.head_dim)
    part = eng.alloc_part(3, rows)
    eng.launch_attn_ms(out, dev_q(eng, q), kvk, kvv, dev_i32(pos, eng.device), dev_i32([0, 1, 2], eng.device), None,
                       part, 3, False, rows_per_seq=rows)
    torch.cuda.synchronize()
    want = O.attend(og, q, okvk, okvv, pos, kslot=[0, 1, 2], rows=rows)
    assert_close(to_np(out), want, "batched verify")
    assert eng.device_status() == 0


@pytest.mark.parametrize("name", ["B", "B32", "R"])
@pytest.mark.parametrize("is_swa", [False, True])
def test_exact_path_and_prompt_chunk(name, is_swa):
    """The exact fp32 path (k_attn / k_attn_rows arithmetic) at several split counts, and a prompt
    chunk (rows > 8) attending the cache after its own rows were appended (bruce.cu:7665-7737)."""
    g = _geom(name, slot_ctx=1024, window=128)
    n = 2 * g.window + 100 if is_swa else 700
    c = Case(g, n, is_swa, seed=3, rows_q=96)
    eng = c.eng
    for rows, nsplit in ((1, 1), (1, 7), (5, 3), (96, 2)):
        p0 = n - rows
        q = c.q[:, :rows]
        out = new_out(eng, 1, rows, g.n_head, g.head_dim)
        ws = torch.empty(eng.exact_workspace_bytes(1, rows, nsplit), dtype=torch.uint8, device=eng.device)
        eng.attn_exact(out, dev_q(eng, q), c.kvk, c.kvv, dev_i32([p0], eng.device), ws, 1, rows, nsplit, is_swa)
        torch.cuda.synchronize()
        want = O.attend(c.og, q, c.okvk, c.okvv, [p0], rows=rows, is_swa=is_swa)
        mabs, rel = assert_close(to_np(out), want, f"exact {name} rows={rows} ns={nsplit}")
        if g.out_dtype == 0:
            assert mabs < 5e-5, "the fp32 path should sit at fp32 rounding level"
    # prompt chunk through the public dispatch
    rows = 96
    out = new_out(eng, 1, rows, g.n_head, g.head_dim)
    part = eng.alloc_part(1, rows)
    eng.launch_attn_m(out, dev_q(eng, c.q[:, :rows]), c.kvk, c.kvv, dev_i32([n - rows], eng.device), part, rows, is_swa)
    torch.cuda.synchronize()
    want = O.attend(c.og, c.q[:, :rows], c.okvk, c.okvv, [n - rows], rows=rows, is_swa=is_swa)
    assert_close(to_np(out), want, f"prefill chunk {name}")
    assert eng.device_status() == 0


def test_partials_and_merge_restate_a_sequence_split():
    """A sequence cut into position shards: per-shard (o, m, l) records merged by battn_merge equal
    the unsplit result (the exchange unit of a multi-device sequence split)."""
    g = _geom("B", slot_ctx=1024, window=128, n_slots=4)
    eng, og = _engine(g), oracle_geom(g)
    n, shards = 1000, 4
    q, k, v = draw_qkv(g, n, 2, seed=9)
    per = n // shards
    kvk, kvv = eng.alloc_kv_layer(False, fill=0)
    for s in range(shards):                       # shard s lives in slot s with local positions
        gpu_fill(eng, k[s * per:(s + 1) * per], v[s * per:(s + 1) * per], kvk, kvv, False, slot=s)
    okvk, okvv = oracle_fill(oracle_geom(g.with_(n_slots=1)), k, v, False)
    rows = 2
    # query rows at global positions n-2, n-1: shards 0..2 see all their keys (local pos = per-1 for
    # every row, i.e. a 1-row-shaped range), the last shard holds the rows' own keys
    recs = torch.zeros((shards, rows, g.n_head, g.head_dim + 2), dtype=torch.float32, device=eng.device)
    part = eng.alloc_part(1, rows)
    qd = dev_q(eng, q)
    for s in range(shards):
        off = g.slot_offset(s, False)
        if s < shards - 1:
            for r in range(rows):                 # every local key is visible to both rows
                eng.attn_partials(recs[s, r], qd[:, r].contiguous(), kvk[off:], kvv[off:],
                                  dev_i32([per - 1], eng.device), part, rows=1)
        else:
            eng.attn_partials(recs[s], qd, kvk[off:], kvv[off:], dev_i32([per - rows], eng.device), part, rows=rows)
    out = new_out(eng, rows, g.n_head, g.head_dim)
    eng.attn_combine(out, recs, shards, rows)
    torch.cuda.synchronize()
    want = O.attend(oracle_geom(g.with_(n_slots=1)), q, okvk, okvv, [n - rows], rows=rows)
    assert_close(to_np(out)[None], want, "sequence split")
    # the records themselves agree with the oracle's restricted-range records
    orec = O.attend(oracle_geom(g.with_(n_slots=1)), q, okvk, okvv, [n - rows], rows=rows, key_lo=0, key_hi=per,
                    records=True)
    got = recs[0].cpu().numpy()
    # compare in normalised form (o / l) and the log-sum-exp (m + log l)
    assert np.abs(got[..., :-2] / got[..., -1:] - orec[0][..., :-2] / orec[0][..., -1:]).max() < 2e-3
    assert np.abs((got[..., -2] + np.log(got[..., -1])) - (orec[0][..., -2] + np.log(orec[0][..., -1]))).max() < 1e-3
    assert eng.device_status() == 0


def test_bad_arguments_and_positions():
    from bruce_engine_b200 import capi
    g = _geom("B", slot_ctx=256, window=64)
    eng = _engine(g)
    kvk, kvv = eng.alloc_kv_layer(False, fill=0)
    part = eng.alloc_part(1, 8)
    q = torch.zeros((1, 9, g.n_head, g.head_dim), dtype=torch.float16, device="cuda")
    out = new_out(eng, 1, 9, g.n_head, g.head_dim)
    import ctypes as C
    rc = eng.lib.battn_verify(eng.h, C.c_void_p(out.data_ptr()), C.c_void_p(q.data_ptr()), C.c_void_p(kvk.data_ptr()),
                              C.c_void_p(kvv.data_ptr()), C.c_void_p(dev_i32([0], "cuda").data_ptr()), None, None,
                              C.c_void_p(part.data_ptr()), 9, 1, 0, None)
    assert rc == capi.ERR_CAPACITY                                  # more than 8 verify rows
    rc = eng.lib.battn_decode(eng.h, None, None, None, None, None, None, None, None, 1, 0, None)
    assert rc == capi.ERR_ARG
    # a position beyond the cache: row skipped, status bit set, output untouched
    eng.launch_attn_m(out[:, :1], q[:, :1].contiguous(), kvk, kvv, dev_i32([256], "cuda"), part, 1, False)
    torch.cuda.synchronize()
    assert eng.device_status() & capi.DEV_BAD_POSITION
    assert torch.isnan(out[:, :1]).all()


@pytest.mark.parametrize("name", ["B", "B32"])
@pytest.mark.parametrize("ctx", [65536])
def test_decode_and_verify_64k(ctx, name):
    """Config 1 / config 3 at 64K: decode and an 8-row verify against the CPU oracle."""
    g = _geom(name, slot_ctx=ctx + 64)
    c = Case(g, ctx + 8, False, seed=0)
    got, want = c.run(ctx - 1, 1)
    assert_close(got, want, "decode 64K")
    got, want = c.run(ctx, 8)                                       # rows at 65536..65543
    assert_close(got, want, "verify 64K x 8")
    cs = Case(_geom(name, slot_ctx=64), ctx, True, seed=0)
    got, want = cs.run(ctx - 1, 1)
    assert_close(got, want, "decode 64K swa")
    assert c.eng.device_status() == 0


def test_decode_256k_against_exact_device_path():
    """At 256K the CPU oracle is too slow for the suite; the fast kernel is checked against the
    exact fp32 device path (itself oracle-checked above) and through a split-invariance property:
    the result must not depend on how the key range is cut."""
    ctx = 262144
    g = _geom("B", slot_ctx=ctx)
    eng = _engine(g)
    rng = np.random.default_rng(0)
    q = rng.standard_normal((1, 1, g.n_head, g.head_dim), dtype=np.float32).astype(np.float16).astype(np.float32)
    kvk, kvv = eng.alloc_kv_layer(False)
    blk = 65536
    for a in range(0, ctx, blk):                                    # K, V drawn in 65,536-position blocks
        k = rng.standard_normal((blk, g.n_kv, g.head_dim), dtype=np.float32)
        v = rng.standard_normal((blk, g.n_kv, g.head_dim), dtype=np.float32)
        gpu_fill(eng, k, v, kvk, kvv, False, start=a)
    pos = dev_i32([ctx - 1], eng.device)
    qd = dev_q(eng, q)
    out = new_out(eng, 1, 1, g.n_head, g.head_dim)
    eng.launch_attn_m(out, qd, kvk, kvv, pos, eng.alloc_part(1, 1), 1, False)
    ref = torch.empty((1, 1, g.n_head, g.head_dim), dtype=torch.float16, device="cuda")
    for ns in (64, 128):
        ws = torch.empty(eng.exact_workspace_bytes(1, 1, ns), dtype=torch.uint8, device="cuda")
        eng.attn_exact(ref, qd, kvk, kvv, pos, ws, 1, 1, ns, False)
        torch.cuda.synchronize()
        assert_close(to_np(out), to_np(ref), f"decode 256K vs exact ns={ns}")
    assert eng.device_status() == 0


def test_many_ragged_slots_in_one_call():
    """257 sequences with ragged lengths (1 .. 700 keys, several at position 0) in one multi-slot decode:
    exercises the prefix sum over sequences, CTAs that span many items and items split over CTAs."""
    n_seq = 257
    g = _geom("B", slot_ctx=704, window=64, n_slots=n_seq)
    eng, og = _engine(g), oracle_geom(g)
    rng = np.random.default_rng(77)
    lens = rng.integers(1, 701, size=n_seq)
    lens[[0, 5, 200]] = 1
    lens[[1, 256]] = 700
    kvk, kvv = eng.alloc_kv_layer(False, fill=0x7F)
    okvk, okvv = O.new_cache(og, False, fill=0x7F), O.new_cache(og, False, fill=0x7F)
    _, kall, vall = draw_qkv(g, 700, 1, seed=78)
    for s in range(n_seq):                                   # every slot gets a different slice order
        n = int(lens[s])
        k = np.roll(kall, s, axis=0)[:n]
        v = np.roll(vall, 3 * s, axis=0)[:n]
        gpu_fill(eng, k, v, kvk, kvv, False, slot=s)
        oracle_fill(og, k, v, False, slot=s, kvk=okvk, kvv=okvv)
    act = np.ones(n_seq, dtype=np.int32)
    act[[7, 100]] = 0
    q = rng.standard_normal((n_seq, 1, g.n_head, g.head_dim), dtype=np.float32).astype(np.float16).astype(np.float32)
    out = new_out(eng, n_seq, 1, g.n_head, g.head_dim)
    part = eng.alloc_part(n_seq, 1)
    kslot = np.arange(n_seq)
    eng.launch_attn_ms(out, dev_q(eng, q), kvk, kvv, dev_i32(lens - 1, eng.device), dev_i32(kslot, eng.device),
                       dev_i32(act, eng.device), part, n_seq, False)
    torch.cuda.synchronize()
    got = to_np(out)
    want = O.attend(og, q, okvk, okvv, lens - 1, kslot=kslot, act=act, rows=1)
    live = act.astype(bool)
    assert np.isnan(got[~live]).all()
    assert_close(got[live], want[live], "257 ragged slots")
    assert eng.device_status() == 0


def test_all_idle_batch_and_zero_sized_calls():
    from bruce_engine_b200 import capi
    import ctypes as C
    g = _geom("B", slot_ctx=256, window=64, n_slots=4)
    eng = _engine(g)
    kvk, kvv = eng.alloc_kv_layer(False, fill=0)
    q = torch.zeros((4, 1, g.n_head, g.head_dim), dtype=torch.float16, device="cuda")
    out = new_out(eng, 4, 1, g.n_head, g.head_dim)
    part = eng.alloc_part(4, 1)
    # every row idle: nothing is read, nothing is written, no error
    eng.launch_attn_ms(out, q, kvk, kvv, dev_i32([3, 9, 0, 255], "cuda"), dev_i32([0, 1, 2, 3], "cuda"),
                       dev_i32([0, 0, 0, 0], "cuda"), part, 4, False)
    torch.cuda.synchronize()
    assert torch.isnan(out).all() and eng.device_status() == 0
    # zero sequences / zero rows are argument errors, not launches
    p = lambda t: C.c_void_p(t.data_ptr())
    pos = dev_i32([0], "cuda")
    assert eng.lib.battn_decode(eng.h, p(out), p(q), p(kvk), p(kvv), p(pos), p(pos), None, p(part), 0, 0, None) == capi.ERR_ARG
    assert eng.lib.battn_verify(eng.h, p(out), p(q), p(kvk), p(kvv), p(pos), None, None, p(part), 0, 1, 0, None) == capi.ERR_ARG
    assert eng.lib.battn_kv_append(eng.h, p(q), p(q), p(kvk), p(kvv), p(pos), None, None, 1, 0, 0, None) == capi.ERR_ARG
    assert eng.lib.battn_prefill(eng.h, p(out), p(q), p(kvk), p(kvv), p(pos), p(part), 513, 0, None) == capi.ERR_CAPACITY
    assert eng.launch_count() == 2                            # only the idle decode (flash + merge) was launched
