"""CPU model of the prompt path's operand roundings, the basis of its per-(row, head) tolerance.

The tensor-core prompt kernel feeds fp16 operands with the q8_0 block scale folded in: K = fp16(q * d),
V = fp16(q * d), P = fp16(2^(s - ref)); everything else is fp32 or exact.  This test applies exactly
those three roundings, one at a time and together, to a double-precision causal attention over
quantised N(0,1) inputs and records how far a single (row, head) softmax can move.  No kernel runs
here: the figures bound what ANY schedule of that arithmetic can achieve, and the GPU parity tests use
PROMPT_HEAD_REL_TOL from tests/util.py accordingly."""
import numpy as np

from oracle import oracle as O
from tests.util import PROMPT_HEAD_REL_TOL, REL_TOL

HD, N, H, HKV = 128, 384, 8, 2


def _quantised(x):
    """Dequantised values of x through the reference quantiser: (exact double, fp16-folded)."""
    rec = O.np_quant_records(x.reshape(-1, HD))
    exact = O.np_dequant_records(rec, HD).astype(np.float64).reshape(x.shape)
    return exact, exact.astype(np.float16).astype(np.float64)


def _attend(q, K, V, round_p):
    out = np.zeros((N, H, HD))
    causal = np.tril(np.ones((N, N), bool))
    for h in range(H):
        kv = h // (H // HKV)
        s = np.where(causal, (q[:, h] @ K[:, kv].T) / np.sqrt(HD), -np.inf)
        p = np.exp(s - s.max(1, keepdims=True))
        if round_p:
            p = p.astype(np.float16).astype(np.float64)
        out[:, h] = (p @ V[:, kv]) / p.sum(1, keepdims=True)
    return out


def test_operand_rounding_bounds_the_prompt_path_error():
    rng = np.random.default_rng(0)
    q = rng.standard_normal((N, H, HD), dtype=np.float32).astype(np.float16).astype(np.float64)
    k = rng.standard_normal((N, HKV, HD), dtype=np.float32)
    v = rng.standard_normal((N, HKV, HD), dtype=np.float32)
    Kx, K16 = _quantised(k)
    Vx, V16 = _quantised(v)
    ref = _attend(q, Kx, Vx, False)

    def worst(o):
        d = o - ref
        head = np.sqrt((d ** 2).sum(-1)) / np.sqrt((ref ** 2).sum(-1))
        row = np.sqrt((d ** 2).sum((-1, -2))) / np.sqrt((ref ** 2).sum((-1, -2)))
        return head.max(), row.max()

    k_only, _ = worst(_attend(q, K16, Vx, False))
    v_only, _ = worst(_attend(q, Kx, V16, False))
    p_only, _ = worst(_attend(q, Kx, Vx, True))
    all_head, all_row = worst(_attend(q, K16, V16, True))
    print(f"[rounding model] per-(row, head): K {k_only:.2e} V {v_only:.2e} P {p_only:.2e} all {all_head:.2e};"
          f" per row: {all_row:.2e}")
    # the folded K operand is the largest single source and already takes half of a 1e-3 budget
    assert k_only > 4e-4 and k_only > v_only and k_only > p_only
    assert 2e-4 < v_only < 4e-4 and 2e-4 < p_only < 4e-4
    # all three together: close to 1e-3 per (row, head) on a few thousand softmaxes, well inside the bounds used
    assert 5e-4 < all_head < PROMPT_HEAD_REL_TOL
    assert all_row < 0.6 * REL_TOL
