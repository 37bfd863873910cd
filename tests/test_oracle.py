"""CPU tests of the oracle: known answers derived by hand from the reference formula
(engine/src/bruce.cu:698-710), agreement with the independent numpy restatement, layout, masks,
ring wrap, split + merge.  No GPU."""
import os

import numpy as np
import pytest

from oracle import oracle as O

GOLD = os.path.join(os.path.dirname(__file__), "golden", "attn_golden.npz")
SMALL = O.Geom(n_head=8, n_kv=2, head_dim=128, window=64, slot_ctx=512, n_slots=2)
SMALL_R = O.Geom(n_head=4, n_kv=1, head_dim=256, window=32, slot_ctx=256, n_slots=1)


def test_f16_conversion_matches_ieee():
    rng = np.random.default_rng(1)
    xs = np.concatenate([rng.standard_normal(3000).astype(np.float32) * np.float32(s)
                         for s in (1e-8, 6e-8, 1e-5, 6.1e-5, 1e-3, 1.0, 100.0, 6.5e4, 7e4)])
    xs = np.concatenate([xs, np.array([0.0, -0.0, 65504.0, 65519.9, 65520.0, 2.0 ** -24, 2.0 ** -25,
                                       2.0 ** -25 * 1.0001, 2.0 ** -14, 1.0009765625, 1.00048828125],
                                      dtype=np.float32)])
    with np.errstate(over="ignore"):
        want = xs.astype(np.float16).view(np.uint16)
    got = np.array([O.f32_to_f16_bits(float(x)) for x in xs], dtype=np.uint16)
    assert (got == want).all()


def test_quantiser_known_answers():
    g = O.Geom(n_head=4, n_kv=1, head_dim=128, window=32, slot_ctx=4)
    x = np.zeros((1, 1, 1, 128), dtype=np.float32)
    # block 0: amax = 127 -> d = 1, q = x exactly (ties to even: 0.5 -> 0, 1.5 -> 2, 2.5 -> 2)
    x[0, 0, 0, :8] = [127.0, -127.0, 0.5, 1.5, 2.5, -0.5, -1.5, 63.49]
    # block 1: all zero -> scale 0, all q 0
    # block 2: amax = 2 -> d = 2/127; x = 1 -> 63.5 in exact arithmetic; fp32 1 * (1/(2/127)) decides
    x[0, 0, 0, 64:67] = [2.0, 1.0, -2.0]
    # block 3: a tiny block still quantises to +-127
    x[0, 0, 0, 96:98] = [1e-20, -1e-20]
    kvk, kvv = O.new_cache(g, False), O.new_cache(g, False)
    O.kv_append(g, x, x, kvk, kvv, [0], rows=1)
    rec = kvk[:g.rec]
    scales = rec[:8].view(np.float16)
    q = rec[8:].view(np.int8)
    assert scales[0] == np.float16(1.0) and scales[1] == 0 and scales[2] == np.float16(np.float32(2.0) / np.float32(127.0))
    assert list(q[:8]) == [127, -127, 0, 2, 2, 0, -2, 63]
    assert (q[32:64] == 0).all()
    inv = np.float32(1.0) / (np.float32(2.0) / np.float32(127.0))
    assert q[64] == 127 and q[66] == -127 and q[65] == int(np.rint(np.float32(1.0) * inv))
    assert q[96] == 127 and q[97] == -127
    assert (kvk == kvv).all()


@pytest.mark.parametrize("g", [SMALL, SMALL_R])
def test_quantiser_matches_numpy_restatement(g):
    rng = np.random.default_rng(2)
    n = 200
    for scale in (1.0, 1e-3, 300.0):
        k = (rng.standard_normal((1, n, g.n_kv, g.head_dim)) * scale).astype(np.float32)
        v = (rng.standard_normal((1, n, g.n_kv, g.head_dim)) * scale).astype(np.float32)
        kvk, kvv = O.new_cache(g, False), O.new_cache(g, False)
        O.kv_append(g, k, v, kvk, kvv, [3], kslot=[g.n_slots - 1], rows=n)
        view = O.np_cache_view(g, kvk, False)
        assert (view[g.n_slots - 1, :, 3:3 + n] == O.np_quant_records(k[0]).transpose(1, 0, 2)).all()
        view = O.np_cache_view(g, kvv, False)
        assert (view[g.n_slots - 1, :, 3:3 + n] == O.np_quant_records(v[0]).transpose(1, 0, 2)).all()
        if g.n_slots > 1:
            assert (O.np_cache_view(g, kvk, False)[0] == 0).all()     # other slots untouched


def test_ring_wrap_and_idle_rows():
    g = SMALL
    rng = np.random.default_rng(3)
    n = 2 * g.window + 17                       # wraps the 2W ring
    k = rng.standard_normal((1, n, g.n_kv, g.head_dim)).astype(np.float32)
    kvk, kvv = O.new_cache(g, True), O.new_cache(g, True)
    O.kv_append(g, k, k, kvk, kvv, [0], rows=n, is_swa=True)
    view = O.np_cache_view(g, kvk, True)
    want = O.np_quant_records(k[0]).transpose(1, 0, 2)
    for p in (n - 1, n - 17, 2 * g.window, 2 * g.window - 1, 17):     # newest survivor per ring slot
        assert (view[0, :, p & (2 * g.window - 1)] == want[:, p]).all()
    # idle sequences write nothing (bruce.cu:1869)
    kvk2, kvv2 = O.new_cache(g, False, fill=0xAB), O.new_cache(g, False, fill=0xAB)
    kk = rng.standard_normal((2, 1, g.n_kv, g.head_dim)).astype(np.float32)
    O.kv_append(g, kk, kk, kvk2, kvv2, [5, 6], kslot=[0, 1], act=[0, 1], rows=1)
    v2 = O.np_cache_view(g, kvk2, False)
    assert (v2[0] == 0xAB).all() and (v2[1, :, 6] != 0xAB).any() and (v2[1, :, 5] == 0xAB).all()


def _filled(g, n, is_swa, seed=4, slot=0):
    rng = np.random.default_rng(seed)
    k = rng.standard_normal((1, n, g.n_kv, g.head_dim)).astype(np.float32)
    v = rng.standard_normal((1, n, g.n_kv, g.head_dim)).astype(np.float32)
    kvk, kvv = O.new_cache(g, is_swa), O.new_cache(g, is_swa)
    O.kv_append(g, k, v, kvk, kvv, [0], kslot=[slot], rows=n, is_swa=is_swa)
    return rng, kvk, kvv


@pytest.mark.parametrize("g", [SMALL, SMALL_R])
@pytest.mark.parametrize("is_swa", [False, True])
@pytest.mark.parametrize("rows", [1, 3, 8])
def test_attention_matches_numpy_restatement(g, is_swa, rows):
    n = 3 * g.window + 5 if is_swa else 200
    if not is_swa:
        n = min(n, g.slot_ctx)
    rng, kvk, kvv = _filled(g, n, is_swa)
    q = rng.standard_normal((1, rows, g.n_head, g.head_dim)).astype(np.float32)
    for p0 in {n - rows, max(0, n // 2 - rows), 0}:
        got = O.attend(g, q, kvk, kvv, [p0], rows=rows, is_swa=is_swa)
        if is_swa and p0 + rows < n - g.window:
            continue                                # older keys were overwritten in the ring
        want = O.np_attend(g, q, kvk, kvv, [p0], rows=rows, is_swa=is_swa)
        assert np.abs(got - want).max() < 2e-6
        f32 = O.attend_f32(g, q, kvk, kvv, [p0], rows=rows, is_swa=is_swa, nsplit=5)
        assert np.abs(got - f32).max() < 2e-5


def test_causal_mask_among_verify_rows():
    """Row r must not see keys beyond pos + r (bruce.cu:2056): changing a later key leaves earlier
    rows untouched."""
    g = SMALL
    rng, kvk, kvv = _filled(g, 100, False)
    q = rng.standard_normal((1, 4, g.n_head, g.head_dim)).astype(np.float32)
    base = O.attend(g, q, kvk, kvv, [96], rows=4)
    kvv2 = kvv.copy()
    O.np_cache_view(g, kvv2, False)[0, :, 98, 8:] ^= 0x55       # perturb V payload at position 98
    pert = O.attend(g, q, kvk, kvv2, [96], rows=4)
    assert (base[0, :2] == pert[0, :2]).all()                  # rows at 96, 97 unaffected
    assert np.abs(base[0, 2:] - pert[0, 2:]).max() > 1e-4      # rows at 98, 99 see it


def test_window_excludes_old_keys():
    g = SMALL
    rng, kvk, kvv = _filled(g, 150, True)
    q = rng.standard_normal((1, 1, g.n_head, g.head_dim)).astype(np.float32)
    base = O.attend(g, q, kvk, kvv, [149], is_swa=True)
    kvv2 = kvv.copy()
    view = O.np_cache_view(g, kvv2, True)
    view[0, :, (149 - g.window) & (2 * g.window - 1), 8:] ^= 0x55    # just outside the window
    assert (O.attend(g, q, kvk, kvv2, [149], is_swa=True) == base).all()
    view[0, :, (150 - g.window) & (2 * g.window - 1), 8:] ^= 0x55    # oldest key inside it
    assert np.abs(O.attend(g, q, kvk, kvv2, [149], is_swa=True) - base).max() > 1e-5


def test_split_records_merge_back():
    g = SMALL
    rng, kvk, kvv = _filled(g, 300, False)
    q = rng.standard_normal((1, 2, g.n_head, g.head_dim)).astype(np.float32)
    whole = O.attend(g, q, kvk, kvv, [298], rows=2)
    cuts = [0, 1, 64, 65, 299, 300, 10 ** 9]
    parts = [O.attend(g, q, kvk, kvv, [298], rows=2, key_lo=a, key_hi=b, records=True)
             for a, b in zip(cuts[:-1], cuts[1:])]
    assert parts[-1][..., -1].max() == 0 and parts[-1][..., -2].max() <= -1e29     # empty split record
    assert np.abs(O.merge(np.stack(parts)) - whole).max() < 1e-6
    # merge is order independent
    assert np.abs(O.merge(np.stack(parts[::-1])) - whole).max() < 1e-6


def test_multi_slot_rows_are_independent():
    g = SMALL
    rng = np.random.default_rng(7)
    kvk, kvv = O.new_cache(g, False), O.new_cache(g, False)
    lens = [37, 200]
    for s, n in enumerate(lens):
        k = rng.standard_normal((1, n, g.n_kv, g.head_dim)).astype(np.float32)
        v = rng.standard_normal((1, n, g.n_kv, g.head_dim)).astype(np.float32)
        O.kv_append(g, k, v, kvk, kvv, [0], kslot=[s], rows=n)
    q = rng.standard_normal((2, 1, g.n_head, g.head_dim)).astype(np.float32)
    both = O.attend(g, q, kvk, kvv, [36, 199], kslot=[0, 1])
    # swapped row order and slots gives swapped outputs
    swapped = O.attend(g, q[::-1], kvk, kvv, [199, 36], kslot=[1, 0])
    assert (both[0] == swapped[1]).all() and (both[1] == swapped[0]).all()
    idle = O.attend(g, q, kvk, kvv, [36, 199], kslot=[0, 1], act=[1, 0])
    assert (idle[0] == both[0]).all() and (idle[1] == 0).all()


def test_golden_fixture():
    """The committed fixture (tests/golden/make_golden.py) pins the oracle against drift."""
    z = np.load(GOLD)
    for name in ("B", "R"):
        g = O.Geom(*[int(x) for x in z[f"{name}_geom"]])
        k, v, q = z[f"{name}_k"], z[f"{name}_v"], z[f"{name}_q"]
        n = k.shape[0]
        for is_swa in (False, True):
            kvk, kvv = O.new_cache(g, is_swa), O.new_cache(g, is_swa)
            O.kv_append(g, k[None], v[None], kvk, kvv, [0], rows=n, is_swa=is_swa)
            tag = f"{name}_{'swa' if is_swa else 'full'}"
            assert (kvk == z[f"{tag}_kvk"]).all() and (kvv == z[f"{tag}_kvv"]).all()
            for rows in (1, 8):
                out = O.attend(g, q[:, :rows], kvk, kvv, [n - rows], rows=rows, is_swa=is_swa)
                assert np.abs(out - z[f"{tag}_out{rows}"]).max() < 1e-6
