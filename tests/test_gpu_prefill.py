"""Parity of the tcgen05 prompt-chunk kernels with the CPU oracle (tolerances: tests/util.py).  A prompt is processed the way the reference does it (bruce.cu:7665-7737): for
each chunk, append the chunk's K/V rows, then attend the chunk's query rows against the cache."""
import numpy as np
import pytest
import torch

from oracle import oracle as O
from tests.gpu_util import dev_i32, dev_q, gpu_fill, new_out, to_np
from tests.util import PROMPT_HEAD_REL_TOL, assert_close, draw_qkv, oracle_fill, oracle_geom

pytestmark = pytest.mark.gpu


def _geom(name, **kw):
    """"B": the graded geometry (fp16 q and out); "B32": the same with fp32 outputs, where the max-norm ratio is
    gated as well (tests/util.py); "R": the reference's own geometry (fp32 q and out)."""
    from bruce_engine_b200.layout import F32, G_B, G_R
    base = {"B": G_B, "B32": G_B.with_(out_dtype=F32), "R": G_R}[name]
    return base.with_(**kw)


def _run_prompt(name, n_prompt, chunk, is_swa, window, seed, check_chunks=None):
    from bruce_engine_b200.engine import AttnEngine
    g = _geom(name, slot_ctx=max(n_prompt, 64), window=window)
    eng, og = AttnEngine(g), oracle_geom(g)
    rng = np.random.default_rng(seed)
    q = rng.standard_normal((n_prompt, g.n_head, g.head_dim), dtype=np.float32)
    if g.q_dtype == 1:
        q = q.astype(np.float16).astype(np.float32)
    k = rng.standard_normal((n_prompt, g.n_kv, g.head_dim), dtype=np.float32)
    v = rng.standard_normal((n_prompt, g.n_kv, g.head_dim), dtype=np.float32)
    kvk, kvv = eng.alloc_kv_layer(is_swa, fill=0xFF)       # 0xFF..: NaN scales in never-written slots
    okvk, okvv = O.new_cache(og, is_swa, fill=0xFF), O.new_cache(og, is_swa, fill=0xFF)
    part = eng.alloc_part(1, chunk)
    worst = (0.0, 0.0)
    for ci, a in enumerate(range(0, n_prompt, chunk)):
        rows = min(chunk, n_prompt - a)
        gpu_fill(eng, k[a:a + rows], v[a:a + rows], kvk, kvv, is_swa, start=a)
        oracle_fill(og, k[a:a + rows], v[a:a + rows], is_swa, kvk=okvk, kvv=okvv, start=a)
        out = new_out(eng, 1, rows, g.n_head, g.head_dim)
        eng.launch_attn_m(out, dev_q(eng, q[None, a:a + rows]), kvk, kvv, dev_i32([a], eng.device), part, rows, is_swa)
        torch.cuda.synchronize()
        if check_chunks is not None and ci not in check_chunks:
            continue
        want = O.attend(og, q[None, a:a + rows], okvk, okvv, [a], rows=rows, is_swa=is_swa)
        mabs, rel = assert_close(to_np(out), want, f"{name} swa={is_swa} chunk {ci} rows {rows}",
                                 head_tol=PROMPT_HEAD_REL_TOL)
        worst = (max(worst[0], mabs), max(worst[1], rel))
    assert (kvk.cpu().numpy() == okvk).all() and (kvv.cpu().numpy() == okvv).all()
    assert eng.device_status() == 0
    return worst


@pytest.mark.parametrize("name", ["B", "B32", "R"])
@pytest.mark.parametrize("is_swa", [False, True])
def test_chunked_prompt_small(name, is_swa):
    """Ragged sizes: prompt not a multiple of the chunk, chunk not a multiple of the M tile."""
    _run_prompt(name, n_prompt=700, chunk=200, is_swa=is_swa, window=256, seed=21)


@pytest.mark.parametrize("name", ["B", "B32", "R"])
def test_single_small_chunks(name):
    """Chunks of 9..40 rows (one partial M tile) at position 0 and deeper."""
    for rows, n0 in ((9, 0), (33, 0), (40, 300), (31, 129)):
        _run_prompt(name, n_prompt=n0 + rows, chunk=max(n0, rows) if n0 else rows, is_swa=False, window=64, seed=22)


@pytest.mark.parametrize("is_swa", [False, True])
def test_prompt_4k_in_512_row_chunks(is_swa):
    """BASELINE config 2 at reduced length: 512-row chunks against a growing cache, window 1024 so
    that later chunks exercise the sliding window; all rows of chunks 0, 3 and 7 are checked."""
    _run_prompt("B", n_prompt=4096, chunk=512, is_swa=is_swa, window=1024, seed=0, check_chunks={0, 3, 7})


@pytest.mark.parametrize("name", ["B", "B32"])
@pytest.mark.parametrize("is_swa", [False, True])
def test_prompt_16k_config2_full_size(name, is_swa):
    """BASELINE config 2 at full size: a 16,384-token prompt in 512-row chunks against the growing cache, window
    4096 on the sliding-window layer; ALL rows of chunks 0, 15 and 31 are compared with the CPU oracle (OpenMP),
    the other chunks only feed the cache; the cache bytes of the whole prompt must equal the oracle's."""
    _run_prompt(name, n_prompt=16384, chunk=512, is_swa=is_swa, window=4096, seed=0, check_chunks={0, 15, 31})


def test_prefill_matches_exact_device_path_at_depth():
    """A 512-row chunk at depth 32K (window 4096 and full): compared with the exact fp32 device path
    (itself oracle-checked) because the CPU oracle would need minutes."""
    from bruce_engine_b200.engine import AttnEngine
    g = _geom("B", slot_ctx=33280, window=4096)
    eng = AttnEngine(g)
    gen = torch.Generator(device="cuda"); gen.manual_seed(5)
    n, rows = 33280, 512
    for is_swa in (False, True):
        kvk, kvv = eng.alloc_kv_layer(is_swa)
        start = n - 8192 if is_swa else 0
        pos = torch.zeros(1, dtype=torch.int32, device="cuda")
        for a in range(start, n, 512):
            kk = torch.randn((1, 512, g.n_kv, g.head_dim), generator=gen, device="cuda")
            vv = torch.randn((1, 512, g.n_kv, g.head_dim), generator=gen, device="cuda")
            pos.fill_(a)
            eng.qkv_prep_store(kk, vv, kvk, kvv, pos, rows=512, is_swa=is_swa)
        q = torch.randn((1, rows, g.n_head, g.head_dim), generator=gen, device="cuda").half()
        pos.fill_(n - rows)
        out = new_out(eng, 1, rows, g.n_head, g.head_dim)
        eng.launch_attn_m(out, q, kvk, kvv, pos, eng.alloc_part(1, rows), rows, is_swa)
        ref = torch.empty_like(out)
        ws = torch.empty(eng.exact_workspace_bytes(1, rows, 4), dtype=torch.uint8, device="cuda")
        eng.attn_exact(ref, q, kvk, kvv, pos, ws, 1, rows, 4, is_swa)
        torch.cuda.synchronize()
        assert_close(to_np(out), to_np(ref), f"prefill at depth swa={is_swa}", head_tol=PROMPT_HEAD_REL_TOL)
    assert eng.device_status() == 0


@pytest.mark.parametrize("name", ["R", "B"])
def test_scratch_sized_for_512_rows_serves_every_shorter_chunk(name):
    """`part` is allocated once for the longest chunk (MBUF rows, bruce.cu:1058-1066, 5564) and reused for a prompt's
    shorter last chunk.  Shorter chunks take MORE key splits, so their split records can outgrow those of the
    512-row chunk: the size battn_workspace_bytes reports must cover them all.  A guard region behind the buffer
    must stay untouched, and the results must still match the exact path."""
    import ctypes as C

    from bruce_engine_b200 import capi
    from bruce_engine_b200.engine import AttnEngine
    depth = 4096
    g = _geom(name, slot_ctx=depth + 512, window=1024)
    eng = AttnEngine(g)
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    size = eng.workspace_bytes(1, 512)
    cg = capi.CGeom(g.n_head, g.n_kv, g.head_dim, g.window, g.slot_ctx, g.n_slots, g.q_dtype, g.out_dtype, 0.0)
    for r in range(1, 513):
        n = C.c_size_t()
        assert eng.lib.battn_call_workspace_bytes(C.byref(cg), sms, 1, r, C.byref(n)) == capi.OK
        assert n.value <= size, f"a {r}-row call needs {n.value} B, the 512-row buffer has {size} B"
    guard = 1 << 20
    buf = torch.full((size + guard,), 0xA5, dtype=torch.uint8, device="cuda")
    part = buf[:size]
    gen = torch.Generator(device="cuda"); gen.manual_seed(17)
    kvk, kvv = eng.alloc_kv_layer(False)
    pos = torch.zeros(1, dtype=torch.int32, device="cuda")
    for a in range(0, depth + 512, 512):
        kk = torch.randn((1, 512, g.n_kv, g.head_dim), generator=gen, device="cuda")
        vv = torch.randn((1, 512, g.n_kv, g.head_dim), generator=gen, device="cuda")
        pos.fill_(a)
        eng.qkv_prep_store(kk, vv, kvk, kvv, pos, rows=512)
    pos.fill_(depth)
    for rows in (96, 160, 192, 384, 512):
        q = torch.randn((1, rows, g.n_head, g.head_dim), generator=gen, device="cuda").to(eng.q_torch)
        out = new_out(eng, 1, rows, g.n_head, g.head_dim)
        eng.launch_attn_m(out, q, kvk, kvv, pos, part, rows, False)
        ref = torch.empty_like(out)
        ws = torch.empty(eng.exact_workspace_bytes(1, rows, 4), dtype=torch.uint8, device="cuda")
        eng.attn_exact(ref, q, kvk, kvv, pos, ws, 1, rows, 4, False)
        torch.cuda.synchronize()
        assert bool((buf[size:] == 0xA5).all()), f"a {rows}-row chunk wrote past the end of the scratch buffer"
        # (a sanity check of the result next to the guard check, against the fp32 device path rather than the
        # oracle: max-abs and the 2-norm ratios; the max-norm gate belongs to the oracle comparisons above)
        assert_close(to_np(out), to_np(ref), f"{name} {rows}-row chunk on the 512-row scratch", maxnorm=False)
    assert eng.device_status() == 0


@pytest.mark.parametrize("name", ["B32", "B"])
@pytest.mark.parametrize("is_swa", [False, True])
def test_pair_kernel_tile_count_edges(name, is_swa):
    """Chunks of two to five M tiles (CTA pairs; an odd count leaves the last pair's second CTA without rows) at
    depths where a pair walks one, two, three, ... key tiles -- a last tile without a partner in the two-tile S
    product -- with and without key splits, full-causal and with a window of four pair spans."""
    from bruce_engine_b200.engine import AttnEngine
    window = 256                                   # a window layer takes at most `window` rows per chunk
    for rows, depth, seed in ((64, 0, 1), (64, 64, 2), (96, 100, 3), (128, 130, 4), (160, 190, 5), (64, 1000, 6),
                              (100, 2000, 7), (33, 3000, 8)):
        n = depth + rows
        g = _geom(name, slot_ctx=n + (n & 1), window=window)
        eng, og = AttnEngine(g), oracle_geom(g)
        q, k, v = draw_qkv(g, n, rows, seed, q_f16=(g.q_dtype == 1))
        kvk, kvv = eng.alloc_kv_layer(is_swa, fill=0xFF)
        gpu_fill(eng, k, v, kvk, kvv, is_swa)
        okvk, okvv = O.new_cache(og, is_swa, fill=0xFF), O.new_cache(og, is_swa, fill=0xFF)
        oracle_fill(og, k, v, is_swa, kvk=okvk, kvv=okvv)
        out = new_out(eng, 1, rows, g.n_head, g.head_dim)
        eng.launch_attn_m(out, dev_q(eng, q), kvk, kvv, dev_i32([depth], eng.device), eng.alloc_part(1, rows), rows, is_swa)
        torch.cuda.synchronize()
        want = O.attend(og, q, okvk, okvv, [depth], rows=rows, is_swa=is_swa)
        assert_close(to_np(out), want, f"pair edges {name} swa={is_swa} rows {rows} depth {depth}")
        assert eng.device_status() == 0


@pytest.mark.parametrize("name", ["B32", "R"])
@pytest.mark.parametrize("is_swa", [False, True])
def test_prompt_chunks_with_early_kv_streaming(name, is_swa):
    """The prompt flow with early KV streaming on: every chunk's append and its attention call share one position
    buffer (the pattern the library recognises), nothing synchronises in between, and the attention kernel starts
    streaming the older tiles while the append of the chunk's own rows is still running.  All chunks are checked."""
    from bruce_engine_b200.engine import AttnEngine
    n_prompt, chunk, window = 1800, 384, 512
    g = _geom(name, slot_ctx=n_prompt, window=window)
    eng, og = AttnEngine(g), oracle_geom(g)
    eng.set_early_kv_stream(True)
    q, k, v = draw_qkv(g, n_prompt, n_prompt, 31, q_f16=True)     # fp16-representable queries in both geometries
    kvk, kvv = eng.alloc_kv_layer(is_swa, fill=0xFF)
    okvk, okvv = O.new_cache(og, is_swa, fill=0xFF), O.new_cache(og, is_swa, fill=0xFF)
    kd, vd, qd = torch.from_numpy(k).cuda(), torch.from_numpy(v).cuda(), dev_q(eng, q)
    part = eng.alloc_part(1, chunk)
    outs = []
    for a in range(0, n_prompt, chunk):
        rows = min(chunk, n_prompt - a)
        pos_d = dev_i32([a], eng.device)                    # a copy: complete before the append starts
        eng.qkv_prep_store(kd[a:a + rows], vd[a:a + rows], kvk, kvv, pos_d, rows=rows, is_swa=is_swa)
        out = new_out(eng, 1, rows, g.n_head, g.head_dim)
        eng.launch_attn_m(out, qd[:, a:a + rows], kvk, kvv, pos_d, part, rows, is_swa)
        outs.append((a, rows, out))
    torch.cuda.synchronize()
    for a, rows, out in outs:
        oracle_fill(og, k[a:a + rows], v[a:a + rows], is_swa, kvk=okvk, kvv=okvv, start=a)
        want = O.attend(og, q[:, a:a + rows], okvk, okvv, [a], rows=rows, is_swa=is_swa)
        assert_close(to_np(out), want, f"early prompt chunk {name} at {a} swa={is_swa}")
    assert eng.device_status() == 0
