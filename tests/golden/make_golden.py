"""Generates tests/golden/attn_golden.npz from the CPU oracle.

The reference repository commits no fixtures for its attention path and its kernels cannot run
without a GPU and the model file, so these vectors come from the oracle restatement (itself checked
against hand-derived answers and an independent numpy restatement in tests/test_oracle.py).
Run from the repository root:  python tests/golden/make_golden.py
"""
import os
import sys

import numpy as np

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
from oracle import oracle as O  # noqa: E402

OUT = os.path.join(os.path.dirname(os.path.abspath(__file__)), "attn_golden.npz")


def main():
    data = {}
    geoms = {"B": O.Geom(n_head=8, n_kv=2, head_dim=128, window=32, slot_ctx=128, n_slots=1),
             "R": O.Geom(n_head=4, n_kv=1, head_dim=256, window=32, slot_ctx=128, n_slots=1)}
    for name, g in geoms.items():
        rng = np.random.default_rng(20241 if name == "B" else 20242)
        n = 100
        q = rng.standard_normal((1, 8, g.n_head, g.head_dim), dtype=np.float32).astype(np.float16).astype(np.float32)
        k = rng.standard_normal((n, g.n_kv, g.head_dim), dtype=np.float32)
        v = rng.standard_normal((n, g.n_kv, g.head_dim), dtype=np.float32)
        k[5, 0, :32] = 0.0                      # an all-zero block: scale 0
        k[6, 0, 32:64] *= 1e4                   # a large-magnitude block
        data[f"{name}_geom"] = np.array([g.n_head, g.n_kv, g.head_dim, g.window, g.slot_ctx, g.n_slots])
        data[f"{name}_q"], data[f"{name}_k"], data[f"{name}_v"] = q, k, v
        for is_swa in (False, True):
            kvk, kvv = O.new_cache(g, is_swa), O.new_cache(g, is_swa)
            O.kv_append(g, k[None], v[None], kvk, kvv, [0], rows=n, is_swa=is_swa)
            tag = f"{name}_{'swa' if is_swa else 'full'}"
            data[f"{tag}_kvk"], data[f"{tag}_kvv"] = kvk, kvv
            for rows in (1, 8):
                data[f"{tag}_out{rows}"] = O.attend(g, q[:, :rows], kvk, kvv, [n - rows], rows=rows, is_swa=is_swa)
    np.savez_compressed(OUT, **data)
    print(OUT, os.path.getsize(OUT), "bytes")


if __name__ == "__main__":
    main()
