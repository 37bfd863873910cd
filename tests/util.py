"""Shared helpers of the test-suite: seeded inputs, the oracle-side cache, error metrics."""
from __future__ import annotations

import numpy as np

from oracle import oracle as O

# Tolerances of the attention outputs against the double-accumulated oracle (every path, every geometry):
#   max-abs   : max |gpu - oracle| over every element                                        <= 2e-3
#   relative  : per (row, head), max|gpu - oracle| / max|oracle|                             <= 1e-3   (*)
#               per (row, head) and per token row (all heads: the vector the engine consumes),
#               ||gpu - oracle||_2 / ||oracle||_2                                            <= 1e-3
# (*) The max-norm ratio is gated on fp32 outputs.  When the library writes fp16 outputs, rounding the OUTPUT alone
#     contributes up to 4.9e-4 to it on rows that see one or two keys (half an fp16 ulp of the largest element,
#     nothing averages out there), which says nothing about the attention arithmetic; the same cases therefore run
#     a second time with out_dtype = fp32 (geometry "B32" in the GPU tests) and are gated there.  The 2-norm
#     ratios and max-abs are gated for both output types.
# Error sources by design: Q, dequantised V and P are fp16 MMA operands (one rounding each); K enters the decode
# and verify kernels as exact integers with the block scale applied in fp32, and the prompt kernels as an exact
# two-part fp16 operand (hi + lo); every accumulation is fp32.
MAX_ABS_TOL = 2e-3
REL_TOL = 1e-3
PROMPT_HEAD_REL_TOL = REL_TOL        # the prompt path has no bound of its own any more


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
    """(max-abs error, worst per-(row, head) 2-norm relative error, worst max-norm relative error,
    worst per-token-row 2-norm relative error).  Arrays are [..., n_head, head_dim]."""
    got = np.asarray(got, dtype=np.float64)
    ref = np.asarray(ref, dtype=np.float64)
    diff = got - ref
    l2 = np.sqrt((diff ** 2).sum(axis=-1)) / np.maximum(np.sqrt((ref ** 2).sum(axis=-1)), 1e-30)
    mx = np.abs(diff).max(axis=-1) / np.maximum(np.abs(ref).max(axis=-1), 1e-30)
    row = np.sqrt((diff ** 2).sum(axis=(-1, -2))) / np.maximum(np.sqrt((ref ** 2).sum(axis=(-1, -2))), 1e-30)
    return float(np.abs(diff).max()), float(l2.max()), float(mx.max()), float(row.max())


def is_fp16_valued(x: np.ndarray) -> bool:
    """True when every element is exactly representable in fp16 (the library wrote an fp16 output)."""
    x = np.asarray(x, dtype=np.float32)
    with np.errstate(over="ignore"):
        return bool(np.array_equal(x, x.astype(np.float16).astype(np.float32), equal_nan=True))


def assert_close(got, ref, what="", head_tol: float = REL_TOL, maxnorm=None):
    """Gates max-abs, the per-token-row and per-(row, head) 2-norm ratios, and -- for fp32 outputs, or when
    maxnorm=True -- the per-(row, head) max-norm ratio max|diff| / max|ref|."""
    mabs, rel, relmax, relrow = errors(got, ref)
    assert np.isfinite(np.asarray(got, dtype=np.float64)).all(), f"{what}: non-finite output"
    assert mabs <= MAX_ABS_TOL, f"{what}: max-abs {mabs:.3e} > {MAX_ABS_TOL}"
    assert relrow <= REL_TOL, f"{what}: relative per token row {relrow:.3e} > {REL_TOL}"
    assert rel <= head_tol, f"{what}: relative per (row, head) {rel:.3e} > {head_tol} (max-norm {relmax:.3e})"
    if maxnorm is None:
        maxnorm = not is_fp16_valued(got)
    if maxnorm:
        assert relmax <= REL_TOL, f"{what}: max-norm ratio per (row, head) {relmax:.3e} > {REL_TOL}"
    print(f"[parity] {what}: max-abs {mabs:.2e} rel-row {relrow:.2e} rel-head {rel:.2e} rel-max {relmax:.2e}"
          f"{' (gated)' if maxnorm else ''}")
    return mabs, rel
