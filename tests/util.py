"""Shared helpers of the test-suite: seeded inputs, the oracle-side cache, error metrics."""
from __future__ import annotations

import numpy as np

from oracle import oracle as O

# tolerances of the attention outputs against the fp32/double-accumulated oracle
MAX_ABS_TOL = 2e-3     # max |gpu - oracle|
REL_TOL = 1e-3         # max |gpu - oracle| / max |oracle|, per (row, head)


def oracle_geom(g) -> O.Geom:
    """bruce_engine_b200.Geom -> oracle Geom (the oracle has no dtype fields)."""
    return O.Geom(g.n_head, g.n_kv, g.head_dim, g.window, g.slot_ctx, g.n_slots, g.softmax_scale)


def draw_qkv(g, n_pos: int, rows: int, seed: int, n_seq: int = 1, q_f16: bool = True):
    """Seeded N(0,1) inputs drawn in the order Q, K, V.  Q is rounded through fp16 when the
    geometry takes fp16 queries.  K, V: [n_pos][n_kv][head_dim] float32."""
    rng = np.random.default_rng(seed)
    q = rng.standard_normal((n_seq, rows, g.n_head, g.head_dim), dtype=np.float32)
    if q_f16:
        q = q.astype(np.float16).astype(np.float32)
    k = rng.standard_normal((n_pos, g.n_kv, g.head_dim), dtype=np.float32)
    v = rng.standard_normal((n_pos, g.n_kv, g.head_dim), dtype=np.float32)
    return q, k, v


def oracle_fill(og: O.Geom, k, v, is_swa: bool, slot: int = 0, kvk=None, kvv=None, start: int = 0):
    """Append k, v ([n][n_kv][HD]) at positions start.. of `slot` through the oracle quantiser."""
    if kvk is None:
        kvk, kvv = O.new_cache(og, is_swa), O.new_cache(og, is_swa)
    n = k.shape[0]
    O.kv_append(og, k[None], v[None], kvk, kvv, [start], kslot=[slot], rows=n, is_swa=is_swa)
    return kvk, kvv


def errors(got: np.ndarray, ref: np.ndarray):
    """(max-abs error, worst per-(row, head) normwise relative error)."""
    got = np.asarray(got, dtype=np.float64)
    ref = np.asarray(ref, dtype=np.float64)
    diff = np.abs(got - ref)
    denom = np.maximum(np.abs(ref).max(axis=-1), 1e-30)
    rel = (diff.max(axis=-1) / denom).max()
    return float(diff.max()), float(rel)


def assert_close(got, ref, what=""):
    mabs, rel = errors(got, ref)
    assert np.isfinite(np.asarray(got, dtype=np.float64)).all(), f"{what}: non-finite output"
    assert mabs <= MAX_ABS_TOL, f"{what}: max-abs {mabs:.3e} > {MAX_ABS_TOL}"
    assert rel <= REL_TOL, f"{what}: relative {rel:.3e} > {REL_TOL}"
    return mabs, rel
