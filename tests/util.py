"""Shared helpers of the test-suite: seeded inputs, the oracle-side cache, error metrics."""
from __future__ import annotations

import numpy as np

from oracle import oracle as O

# Tolerances of the attention outputs against the double-accumulated oracle:
#   max-abs  : max |gpu - oracle| over every element                                   <= 2e-3
#   relative : per (row, head), ||gpu - oracle||_2 / ||oracle||_2                      <= 1e-3
# The per-(row, head) max-norm ratio max|diff| / max|oracle| is also computed and printed; it is not
# the gate because rounding the OUTPUT to fp16 alone contributes up to 4.9e-4 to it on rows that see
# one or two keys (nothing averages out there), on top of the fp16 P and V operand roundings.
MAX_ABS_TOL = 2e-3
REL_TOL = 1e-3


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
    """(max-abs error, worst per-(row, head) 2-norm relative error, worst max-norm relative error)."""
    got = np.asarray(got, dtype=np.float64)
    ref = np.asarray(ref, dtype=np.float64)
    diff = got - ref
    l2 = np.sqrt((diff ** 2).sum(axis=-1)) / np.maximum(np.sqrt((ref ** 2).sum(axis=-1)), 1e-30)
    mx = np.abs(diff).max(axis=-1) / np.maximum(np.abs(ref).max(axis=-1), 1e-30)
    return float(np.abs(diff).max()), float(l2.max()), float(mx.max())


def assert_close(got, ref, what=""):
    mabs, rel, relmax = errors(got, ref)
    assert np.isfinite(np.asarray(got, dtype=np.float64)).all(), f"{what}: non-finite output"
    assert mabs <= MAX_ABS_TOL, f"{what}: max-abs {mabs:.3e} > {MAX_ABS_TOL}"
    assert rel <= REL_TOL, f"{what}: relative (2-norm) {rel:.3e} > {REL_TOL} (max-norm {relmax:.3e})"
    print(f"[parity] {what}: max-abs {mabs:.2e} rel-l2 {rel:.2e} rel-max {relmax:.2e}")
    return mabs, rel
