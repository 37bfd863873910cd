"""The oracle's QKV prologue + append against OUTPUTS OF THE REFERENCE'S OWN KERNELS
(tests/golden/qkv_prep_ref.npz, produced on a B200 by tests/golden/make_qkv_prep_golden.py from
k_rope_tables_rows, k_qkv_prep_fast and k_qkv_prep_fast_ms), and against an independent numpy restatement."""
import os

import numpy as np
import pytest

from oracle import oracle as O

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "qkv_prep_ref.npz")
G = O.Geom(16, 4, 256, 1024, 2048, 5, 1.0 / 16.0)          # the reference's native geometry, 5 slots


def _u32(a):
    return np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)


@pytest.fixture(scope="module")
def gold():
    return np.load(GOLD)


@pytest.mark.parametrize("tag,is_swa,theta", [("full", False, 1), ("swa", True, 2)])
def test_rows_of_one_sequence_reproduce_the_reference_kernel(gold, tag, is_swa, theta):
    rows, p0 = gold["a_q"].shape[0], int(gold["a_pos"])
    kvk, kvv = O.new_cache(G, is_swa), O.new_cache(G, is_swa)
    q = O.qkv_prep(G, gold["a_q"][None], gold["a_k"][None], gold["a_v"][None], gold["sqk"], gold["a_cs"], gold["a_sn"],
                   kvk, kvv, [p0], rows=rows, is_swa=is_swa, theta_sel=theta)
    assert (_u32(q[0]) == _u32(gold[f"a_{tag}_q_out"])).all(), "q differs from the reference kernel's output"
    pstride = 2 * G.window if is_swa else G.slot_ctx
    slots = [(p0 + r) & (pstride - 1) if is_swa else p0 + r for r in range(rows)]
    per_slot = G.n_kv * pstride * 272
    kk = kvk[:per_slot].reshape(G.n_kv, pstride, 272)[:, slots]
    vv = kvv[:per_slot].reshape(G.n_kv, pstride, 272)[:, slots]
    assert (kk == gold[f"a_{tag}_krec"]).all(), "K records differ from the reference kernel's"
    assert (vv == gold[f"a_{tag}_vrec"]).all(), "V records differ from the reference kernel's"


def test_multi_slot_rows_reproduce_the_reference_kernel(gold):
    pos, slot, act = gold["b_pos"], gold["b_slot"], gold["b_act"]
    n = pos.size
    kvk, kvv = O.new_cache(G, False), O.new_cache(G, False)
    q = O.qkv_prep(G, gold["b_q"][:, None], gold["b_k"][:, None], gold["b_v"][:, None], gold["sqk"], gold["b_cs"], gold["b_sn"],
                   kvk, kvv, pos, kslot=slot, act=act, rows=1)
    assert (_u32(q[:, 0]) == _u32(gold["b_q_out"])).all()
    kall = kvk.reshape(5, G.n_kv, G.slot_ctx, 272)
    vall = kvv.reshape(5, G.n_kv, G.slot_ctx, 272)
    for i in range(n):
        assert (kall[slot[i], :, pos[i]] == gold["b_krec"][i]).all()
        assert (vall[slot[i], :, pos[i]] == gold["b_vrec"][i]).all()
    # the idle row wrote nothing, and nothing else was touched
    assert act[2] == 0 and not kall[slot[2], :, pos[2]].any()
    assert np.count_nonzero(kall) == int(gold["b_k_nonzero_bytes"])
    assert np.count_nonzero(vall) == int(gold["b_v_nonzero_bytes"])


def test_numpy_restatement_agrees(gold):
    c = gold["a_cs"][:, None, :128]
    s = gold["a_sn"][:, None, :128]
    q = O.np_qkv_prologue(gold["a_q"], c, s, gold["sqk"][None])
    assert (_u32(q) == _u32(gold["a_full_q_out"])).all()
    kr = O.np_qkv_prologue(gold["a_k"], c, s)
    rec = O.np_quant_records(kr.reshape(-1, 256)).reshape(-1, 4, 272).transpose(1, 0, 2)
    assert (rec == gold["a_full_krec"]).all()


def test_head_dim_128_oracle_matches_numpy_restatement():
    """No reference kernel exists at head_dim 128; there the C oracle and the numpy restatement pin each other."""
    g = O.Geom(32, 8, 128, 4096, 256, 1, 128 ** -0.5)
    rng = np.random.default_rng(3)
    rows = 5
    q = rng.standard_normal((1, rows, 32, 128), dtype=np.float32)
    k = rng.standard_normal((1, rows, 8, 128), dtype=np.float32)
    v = rng.standard_normal((1, rows, 8, 128), dtype=np.float32)
    sqk = (1.0 + 0.3 * rng.standard_normal((32, 128))).astype(np.float32)
    cs, sn = O.rope_tables(128, 100 + np.arange(rows))
    kvk, kvv = O.new_cache(g, False), O.new_cache(g, False)
    qo = O.qkv_prep(g, q, k, v, sqk, cs, sn, kvk, kvv, [100], rows=rows, theta_sel=2)
    c, s = cs[:, None, 64:], sn[:, None, 64:]
    assert (_u32(qo[0]) == _u32(O.np_qkv_prologue(q[0], c, s, sqk[None]))).all()
    kr = O.np_qkv_prologue(k[0], c, s)
    rec = O.np_quant_records(kr.reshape(-1, 128)).reshape(rows, 8, 136)
    got = kvk.reshape(8, 256, 136)[:, 100:100 + rows].transpose(1, 0, 2)
    assert (got == rec).all()
    # unit length before sqk: |k row| == 1 / sqrt(HD) * sqrt(HD) ... the prologue leaves k with norm 1
    assert np.allclose(np.sqrt((kr.astype(np.float64) ** 2).sum(-1)), 1.0, atol=1e-5)
