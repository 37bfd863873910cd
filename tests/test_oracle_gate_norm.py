"""The oracle's gate-norm step against outputs of the reference's own kernel (tests/golden/gate_norm_ref.npz,
produced on a B200 by tests/golden/make_gate_norm_golden.py from k_gate_norm_vec4, bruce.cu:1526).

The CPU cannot reproduce the kernel's exponential bit for bit (the kernel uses the GPU's approximate ex2 unit), so
the comparison is: normalised values and group scales to a few ulp, quantised bytes equal except for a handful that
sit on a rounding boundary (and then off by one step), group sums consistent with the bytes."""
import os

import numpy as np

from oracle import oracle as O

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "gate_norm_ref.npz")


def test_oracle_gate_norm_matches_the_reference_kernel():
    z = np.load(GOLD)
    dst, xq, xd, xsum = O.gate_norm(z["aout"], z["gate"], z["sgate"])
    ref = z["dst"]
    scale = np.abs(ref).max(axis=1, keepdims=True) + 1e-30
    assert (np.abs(dst - ref) / scale).max() < 2e-6
    assert np.allclose(xd, z["xd"], rtol=4e-6, atol=0)
    dq = xq.astype(np.int32) - z["xq"].astype(np.int32)
    assert np.abs(dq).max() <= 1
    assert (dq != 0).mean() < 2e-3
    assert (xsum == xq.astype(np.int32).reshape(xq.shape[0], -1, 32).sum(-1)).all()
    assert (z["xsum"] == z["xq"].astype(np.int32).reshape(xq.shape[0], -1, 32).sum(-1)).all()
    # the edge cases of the fixture: an all-zero group has scale 0 and zero bytes; an all-zero row stays zero
    assert xd[5, 2] == 0 and (xq[5, 64:96] == 0).all() and z["xd"][5, 2] == 0
    assert (dst[7] == 0).all() and (z["dst"][7] == 0).all()


def test_gate_norm_semantics_in_numpy():
    """Independent restatement in float64 numpy: the C oracle must agree with the formula it claims to follow."""
    rng = np.random.default_rng(5)
    a = rng.standard_normal((3, 4096)).astype(np.float32)
    g = rng.standard_normal((3, 4096)).astype(np.float32)
    s = (1 + 0.1 * rng.standard_normal(4096)).astype(np.float32)
    dst, xq, xd, xsum = O.gate_norm(a, g, s)
    t = a.astype(np.float64) / (1 + np.exp(-(g.astype(np.float64) * s)))
    n = 4096
    k = 1 / np.sqrt((t ** 2).sum(1, keepdims=True) / n + 1e-6 / n) / np.sqrt(n)
    v = t * k
    assert np.abs(dst - v).max() < 1e-6
    d = np.abs(v).reshape(3, -1, 32).max(-1) / 127
    assert np.allclose(xd, d, rtol=1e-5)
    q = np.clip(np.rint(v.reshape(3, -1, 32) / d[..., None]), -127, 127).reshape(3, -1)
    assert (np.abs(q - xq) <= 1).all() and (q != xq).mean() < 2e-3
