"""B200-native attention hot path of the Bruce inference engine (q8_0 scale-first KV cache).

The product is the CUDA library `libbattn.so` (C ABI in include/battn.h).  This package holds its
build script, a ctypes binding and a host-side mirror of the reference engine's attention call
surface (`k_qkv_prep*`, `launch_attn_m`, `launch_attn_ms`, `k_attn_combine*`;
engine/src/bruce.cu:7665-7761).  There is no CPU path: importing `capi` without a built library, or
creating an engine without a CUDA device, raises.
"""
from .layout import Geom, G_B, G_R  # noqa: F401

__all__ = ["Geom", "G_B", "G_R"]
