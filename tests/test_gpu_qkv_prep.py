"""The fused QKV prologue + append kernel (battn_qkv_prep) and the table kernel (battn_rope_tables):
bit-exact against the oracle (whose arithmetic is pinned by outputs of the reference's own kernel,
tests/golden/qkv_prep_ref.npz) in both geometries, single sequence and multi-slot, fp32 and fp16 q; and,
where the reference harness is present, bit-exact against the reference kernels themselves."""
import ctypes as C
import os

import numpy as np
import pytest
import torch

from oracle import oracle as O
from tests.gpu_util import dev_i32
from tests.util import oracle_geom

pytestmark = pytest.mark.gpu

REF_LIB = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "oracle", "_ref", "libbruce_ref.so")


def _geom(name, **kw):
    from bruce_engine_b200.layout import G_B, G_R
    return (G_B if name == "B" else G_R).with_(**kw)


def _u32(a):
    return np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)


def _run(name, n_seq, rows, is_swa, theta_sel, seed, q_f16, multi):
    from bruce_engine_b200.engine import AttnEngine
    g = _geom(name, slot_ctx=1024, window=256, n_slots=max(n_seq, 1), q_dtype=1 if q_f16 else 0)
    eng, og = AttnEngine(g), oracle_geom(g)
    rng = np.random.default_rng(seed)
    HD = g.head_dim
    q = rng.standard_normal((n_seq, rows, g.n_head, HD), dtype=np.float32)
    k = rng.standard_normal((n_seq, rows, g.n_kv, HD), dtype=np.float32) * 3.0
    v = rng.standard_normal((n_seq, rows, g.n_kv, HD), dtype=np.float32)
    sqk = (1.0 + 0.2 * rng.standard_normal((g.n_head, HD))).astype(np.float32)
    pos = rng.integers(0, 1024 - rows, size=n_seq).astype(np.int32)
    if is_swa:
        pos = pos + 3000                                            # deep into the ring
    kslot = rng.permutation(n_seq).astype(np.int32) if multi else None
    act = (rng.random(n_seq) > 0.3).astype(np.int32) if multi else None
    positions = (pos[:, None] + np.arange(rows)[None]).reshape(-1)
    cs, sn = O.rope_tables(HD, positions)
    # oracle
    okvk, okvv = O.new_cache(og, is_swa), O.new_cache(og, is_swa)
    q_want = O.qkv_prep(og, q, k, v, sqk, cs, sn, okvk, okvv, pos, kslot=kslot, act=act, rows=rows, is_swa=is_swa,
                        theta_sel=theta_sel)
    # device
    kvk, kvv = eng.alloc_kv_layer(is_swa, fill=0)
    qd = torch.from_numpy(q).cuda()
    q_out = torch.empty_like(qd, dtype=torch.float16) if q_f16 else qd
    eng.qkv_prep(q_out, qd, torch.from_numpy(k).cuda(), torch.from_numpy(v).cuda(), torch.from_numpy(sqk).cuda(),
                 torch.from_numpy(cs).cuda(), torch.from_numpy(sn).cuda(), kvk, kvv, dev_i32(pos, "cuda"),
                 kslot=None if kslot is None else dev_i32(kslot, "cuda"), act=None if act is None else dev_i32(act, "cuda"),
                 rows=rows, is_swa=is_swa, theta_sel=theta_sel)
    torch.cuda.synchronize()
    assert eng.device_status() == 0
    if q_f16:
        assert (q_out.cpu().numpy().view(np.uint16) == q_want.astype(np.float16).view(np.uint16)).all(), "fp16 q differs"
    else:
        assert (_u32(q_out.cpu().numpy()) == _u32(q_want)).all(), "fp32 q differs from the oracle"
    assert (kvk.cpu().numpy() == okvk).all(), "K cache bytes differ from the oracle"
    assert (kvv.cpu().numpy() == okvv).all(), "V cache bytes differ from the oracle"
    assert okvk.any()


@pytest.mark.parametrize("name", ["B", "R"])
@pytest.mark.parametrize("is_swa", [False, True])
def test_rows_of_one_sequence_bit_exact(name, is_swa):
    _run(name, 1, 37, is_swa, theta_sel=2 if is_swa else 1, seed=5, q_f16=False, multi=False)


@pytest.mark.parametrize("name", ["B", "R"])
def test_multi_slot_with_idle_rows_bit_exact(name):
    _run(name, 9, 1, False, theta_sel=1, seed=6, q_f16=False, multi=True)
    _run(name, 4, 3, True, theta_sel=2, seed=7, q_f16=True, multi=True)


def test_prompt_chunk_fp16_q_feeds_attention():
    """512-row chunk: prepared fp16 q and the appended cache go straight into the prompt kernel; the result
    equals the oracle's attention over the oracle's prepared q and cache."""
    from bruce_engine_b200.engine import AttnEngine
    from tests.util import PROMPT_HEAD_REL_TOL, assert_close
    g = _geom("B", slot_ctx=512, window=256, q_dtype=1)
    eng, og = AttnEngine(g), oracle_geom(g)
    rng = np.random.default_rng(8)
    rows, HD = 512, g.head_dim
    q = rng.standard_normal((1, rows, g.n_head, HD), dtype=np.float32) * 20.0
    k = rng.standard_normal((1, rows, g.n_kv, HD), dtype=np.float32)
    v = rng.standard_normal((1, rows, g.n_kv, HD), dtype=np.float32)
    sqk = np.full((g.n_head, HD), 11.0, dtype=np.float32)             # unit-norm q and k: scale the scores up
    cs, sn = O.rope_tables(HD, np.arange(rows))
    okvk, okvv = O.new_cache(og, False), O.new_cache(og, False)
    q_want = O.qkv_prep(og, q, k, v, sqk, cs, sn, okvk, okvv, [0], rows=rows)
    want = O.attend(og, q_want.astype(np.float16).astype(np.float32), okvk, okvv, [0], rows=rows)
    kvk, kvv = eng.alloc_kv_layer(False, fill=0)
    q16 = torch.empty((1, rows, g.n_head, HD), dtype=torch.float16, device="cuda")
    pos = dev_i32([0], "cuda")
    eng.qkv_prep(q16, torch.from_numpy(q).cuda(), torch.from_numpy(k).cuda(), torch.from_numpy(v).cuda(),
                 torch.from_numpy(sqk).cuda(), torch.from_numpy(cs).cuda(), torch.from_numpy(sn).cuda(), kvk, kvv, pos, rows=rows)
    out = torch.zeros((1, rows, g.n_head, HD), dtype=torch.float16 if g.out_dtype == 1 else torch.float32, device="cuda")
    eng.launch_attn_m(out, q16, kvk, kvv, pos, eng.alloc_part(1, rows), rows, False)
    torch.cuda.synchronize()
    assert_close(out.float().cpu().numpy(), want, "prepared q -> prompt kernel", head_tol=PROMPT_HEAD_REL_TOL)
    assert eng.device_status() == 0


def test_rope_tables_close_to_double_precision():
    """The table kernel evaluates the reference's fp32 expressions; against a double-precision evaluation the
    angle carries the fp32 error of p * powf(...), i.e. up to ~|theta| * 2^-22."""
    from bruce_engine_b200.engine import AttnEngine
    for name in ("B", "R"):
        g = _geom(name, slot_ctx=4096)
        eng = AttnEngine(g)
        HD = g.head_dim
        pos = np.array([0, 7, 300, 4000], dtype=np.int32)
        rows = 3
        cs = torch.zeros((pos.size * rows, HD), device="cuda")
        sn = torch.zeros_like(cs)
        eng.rope_tables(cs, sn, dev_i32(pos, "cuda"), rows=rows)
        torch.cuda.synchronize()
        positions = (pos[:, None] + np.arange(rows)[None]).reshape(-1)
        wc, ws = O.rope_tables(HD, positions)
        tol = 4e-6 + positions.max() * 2.0 ** -21
        assert np.abs(cs.cpu().numpy() - wc).max() < tol and np.abs(sn.cpu().numpy() - ws).max() < tol
        assert (cs.cpu().numpy()[0] == 1.0).all() and (sn.cpu().numpy()[0] == 0.0).all()     # position 0


@pytest.fixture(scope="module")
def ref():
    if not os.path.exists(REF_LIB):
        pytest.skip("oracle/_ref/libbruce_ref.so not built (reference tree unavailable)")
    return C.CDLL(REF_LIB)


def _p(t):
    return C.c_void_p(t.data_ptr())


def test_bit_exact_against_the_reference_kernels(ref):
    """k_rope_tables_rows + k_qkv_prep_fast (rows of one sequence, wrapped ring, table 2) and
    k_rope_tables_rows_ms + k_qkv_prep_fast_ms (slots, one idle) versus battn_rope_tables + battn_qkv_prep."""
    from bruce_engine_b200.engine import AttnEngine
    g = _geom("R", slot_ctx=2048, window=1024, n_slots=4, q_dtype=0)
    eng = AttnEngine(g)
    rng = np.random.default_rng(9)
    HD = g.head_dim
    sqk = torch.from_numpy((1.0 + 0.1 * rng.standard_normal((g.n_head, HD))).astype(np.float32)).cuda()
    for multi in (False, True):
        rows = 4 if multi else 300
        q = torch.from_numpy(rng.standard_normal((rows, g.n_head, HD), dtype=np.float32)).cuda()
        k = torch.from_numpy(rng.standard_normal((rows, g.n_kv, HD), dtype=np.float32)).cuda()
        v = torch.from_numpy(rng.standard_normal((rows, g.n_kv, HD), dtype=np.float32)).cuda()
        is_swa = not multi
        pos = dev_i32([5, 2040, 77, 1024] if multi else [1900], "cuda")
        slot = dev_i32([2, 0, 3, 1], "cuda")
        act = dev_i32([1, 0, 1, 1], "cuda")
        # reference
        cs_r, sn_r = torch.zeros((rows, 256), device="cuda"), torch.zeros((rows, 256), device="cuda")
        assert ref.ref_rope_tables(_p(cs_r), _p(sn_r), _p(pos), rows, int(multi)) == 0
        kvk_r, kvv_r = eng.alloc_kv_layer(is_swa, fill=0)
        q_r = q.clone()
        torch.cuda.synchronize()
        if multi:
            rc = ref.ref_kv_append_ms(_p(q_r), _p(k), _p(v), _p(sqk), _p(kvk_r), _p(kvv_r), _p(pos), _p(slot), _p(act),
                                      rows, int(is_swa), 1, g.slot_ctx, _p(cs_r), _p(sn_r))
        else:
            rc = ref.ref_kv_append_theta(_p(q_r), _p(k), _p(v), _p(sqk), _p(kvk_r), _p(kvv_r), _p(pos), rows, int(is_swa), 2,
                                         g.slot_ctx, _p(cs_r), _p(sn_r))
        assert rc == 0
        # this repository
        cs, sn = torch.zeros((rows, HD), device="cuda"), torch.zeros((rows, HD), device="cuda")
        eng.rope_tables(cs, sn, pos, rows=1 if multi else rows)
        kvk, kvv = eng.alloc_kv_layer(is_swa, fill=0)
        q_o = q.clone()
        eng.qkv_prep(q_o, q_o, k, v, sqk, cs, sn, kvk, kvv, pos, kslot=slot if multi else None, act=act if multi else None,
                     rows=1 if multi else rows, is_swa=is_swa, theta_sel=1 if multi else 2)
        torch.cuda.synchronize()
        assert torch.equal(cs.view(torch.int32), cs_r.view(torch.int32)) and torch.equal(sn.view(torch.int32), sn_r.view(torch.int32)), \
            "RoPE tables differ from the reference kernel's"
        assert torch.equal(q_o.view(torch.int32), q_r.view(torch.int32)), "q differs from the reference kernel's"
        assert torch.equal(kvk, kvk_r) and torch.equal(kvv, kvv_r), "cache bytes differ from the reference kernel's"
        assert kvk.any()
    assert eng.device_status() == 0


def test_bad_requests_are_refused_or_reported_not_executed():
    from bruce_engine_b200 import capi
    from bruce_engine_b200.engine import AttnEngine
    g = _geom("B", slot_ctx=64, window=32, q_dtype=0)
    eng = AttnEngine(g)
    HD = g.head_dim
    rows = 2
    q = torch.randn((1, rows, g.n_head, HD), device="cuda")
    k = torch.randn((1, rows, g.n_kv, HD), device="cuda")
    sqk = torch.ones((g.n_head, HD), device="cuda")
    cs, sn = torch.ones((rows, HD), device="cuda"), torch.zeros((rows, HD), device="cuda")
    kvk, kvv = eng.alloc_kv_layer(False, fill=0x11)
    pos = dev_i32([0], "cuda")
    with pytest.raises(capi.BattnError) as ei:                       # only tables 1 and 2 exist
        eng.qkv_prep(q, q, k, k, sqk, cs, sn, kvk, kvv, pos, rows=rows, theta_sel=3)
    assert ei.value.code == capi.ERR_ARG
    with pytest.raises(capi.BattnError) as ei:                       # 16-byte alignment of the fp32 operands
        eng.qkv_prep(q, q, k, k, sqk, cs.view(-1)[1:], sn, kvk, kvv, pos, rows=rows)
    assert ei.value.code == capi.ERR_ARG
    kvk_w, kvv_w = eng.alloc_kv_layer(True, fill=0)
    big = 2 * g.window + 1
    qb = torch.zeros((1, big, g.n_head, HD), device="cuda")
    kb = torch.zeros((1, big, g.n_kv, HD), device="cuda")
    tb = torch.zeros((big, HD), device="cuda")
    with pytest.raises(capi.BattnError) as ei:                       # one call must not wrap the ring onto itself
        eng.qkv_prep(qb, qb, kb, kb, sqk, tb, tb, kvk_w, kvv_w, pos, rows=big, is_swa=True)
    assert ei.value.code == capi.ERR_CAPACITY
    # a position past the end of the slot: q is still prepared, nothing is written, the status word says why
    before = q.clone()
    eng.qkv_prep(q, q, k, k, sqk, cs, sn, kvk, kvv, dev_i32([63], "cuda"), rows=rows)
    torch.cuda.synchronize()
    assert eng.device_status() & capi.DEV_BAD_POSITION
    assert not torch.equal(q, before)
    rec = kvk.view(g.n_kv, g.slot_ctx, HD + HD // 16)
    assert (rec[:, :63] == 0x11).all() and not (rec[:, 63] == 0x11).all()       # row 0 (position 63) stored, row 1 refused
    assert eng.device_status() == 0
