"""GPU-side helpers of the parity tests: every call goes through the C ABI (libbattn.so)."""
from __future__ import annotations

import numpy as np
import torch

from bruce_engine_b200.engine import AttnEngine
from bruce_engine_b200.layout import F16


def dev_i32(x, dev):
    return torch.tensor(np.asarray(x, dtype=np.int32).reshape(-1), dtype=torch.int32, device=dev)


def dev_q(eng: AttnEngine, q: np.ndarray):
    return torch.from_numpy(np.ascontiguousarray(q)).to(eng.device).to(eng.q_torch).contiguous()


def gpu_fill(eng: AttnEngine, k: np.ndarray, v: np.ndarray, kvk, kvv, is_swa: bool, slot: int | None = None,
             start: int = 0, chunk: int = 512):
    """Append k, v ([n][n_kv][HD] float32) at positions start.. through battn_kv_append, `chunk`
    rows per call.  slot=None uses the single-sequence form with the slot-base pointer."""
    g = eng.geom
    n = k.shape[0]
    if is_swa:
        chunk = min(chunk, 2 * g.window)        # one call must not wrap the ring onto itself
    kd = torch.from_numpy(np.ascontiguousarray(k)).to(eng.device)
    vd = torch.from_numpy(np.ascontiguousarray(v)).to(eng.device)
    for a in range(0, n, chunk):
        b = min(n, a + chunk)
        pos = dev_i32([start + a], eng.device)
        if slot is None:
            eng.qkv_prep_store(kd[a:b], vd[a:b], kvk, kvv, pos, rows=b - a, is_swa=is_swa)
        else:
            eng.qkv_prep_store(kd[a:b], vd[a:b], kvk, kvv, pos, kslot=dev_i32([slot], eng.device),
                               rows=b - a, is_swa=is_swa)
    return kvk, kvv


def to_np(t: torch.Tensor) -> np.ndarray:
    return t.detach().float().cpu().numpy() if t.dtype in (torch.float16, torch.float32) else t.cpu().numpy()


def new_out(eng: AttnEngine, *shape):
    # NaN-poisoned so that rows the library must not write are detectable
    return torch.full(shape, float("nan"), dtype=eng.out_torch, device=eng.device)
