"""Generates tests/golden/gate_norm_ref.npz: inputs and OUTPUTS OF THE REFERENCE'S OWN KERNEL for the step after
attention, k_gate_norm_vec4 (engine/src/bruce.cu:1526-1568): sigmoid gate, L2 norm over the token's 4096 values,
q8 activation copy.  The kernel depends on n = n_head * head_dim only (4096 in the reference's geometry and in the
32 / 8 / 128 one alike), so one fixture pins both.

Needs a GPU and oracle/_ref/libbruce_ref.so (built by oracle/ref_build.py where the reference tree is present).
Run from the repository root:  python tests/golden/make_gate_norm_golden.py [out.npz]
The committed fixture was produced by exactly this script on a B200."""
import ctypes as C
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
N = 4096


def _p(t):
    return C.c_void_p(t.data_ptr())


def main(out_path):
    lib = C.CDLL(os.path.join(ROOT, "oracle", "_ref", "libbruce_ref.so"))
    rng = np.random.default_rng(20240611)
    rows = 12
    aout = rng.standard_normal((rows, N), dtype=np.float32)
    aout[3] *= 1e-3                                  # a quiet row
    aout[5, 64:96] = 0.0                             # an all-zero q8 group (d = 0, id = 0)
    aout[7] = 0.0                                    # an all-zero row (the epsilon of the norm)
    gate = (3.0 * rng.standard_normal((rows, N))).astype(np.float32)
    sgate = (1.0 + 0.2 * rng.standard_normal(N)).astype(np.float32)
    dev = "cuda"
    a, g, s = (torch.from_numpy(x).to(dev) for x in (aout, gate, sgate))
    dst = torch.zeros((rows, N), device=dev)
    xq = torch.zeros((rows, N), dtype=torch.int8, device=dev)
    xd = torch.zeros((rows, N // 32), device=dev)
    xs = torch.zeros((rows, N // 32), dtype=torch.int32, device=dev)
    assert lib.ref_gate_norm(_p(dst), _p(a), _p(g), _p(s), _p(xq), _p(xd), _p(xs), rows) == 0
    np.savez_compressed(out_path, aout=aout, gate=gate, sgate=sgate, dst=dst.cpu().numpy(), xq=xq.cpu().numpy(),
                        xd=xd.cpu().numpy(), xsum=xs.cpu().numpy())
    print("wrote", out_path)


if __name__ == "__main__":
    main(sys.argv[1] if len(sys.argv) > 1 else os.path.join(ROOT, "tests", "golden", "gate_norm_ref.npz"))
