"""Device-side fault reporting: a bounded in-kernel wait that runs out must set BATTN_DEV_WAIT_TIMEOUT in the
device status word, return normally and leave the context usable.  The wait is made to run out the harmless
way: a test-only kernel waits on an mbarrier that nothing arrives on, with a short poll limit (no trap, no bad
address, no endless loop)."""
import ctypes as C

import numpy as np
import pytest
import torch

from tests.gpu_util import dev_i32, gpu_fill, new_out, to_np
from tests.util import draw_qkv

pytestmark = pytest.mark.gpu


def test_bounded_wait_that_runs_out_sets_the_status_bit_and_the_context_survives():
    from bruce_engine_b200 import capi
    from bruce_engine_b200.engine import AttnEngine
    from bruce_engine_b200.layout import G_B
    g = G_B.with_(slot_ctx=1024, window=128)
    eng = AttnEngine(g)
    assert eng.device_status() == 0
    st = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    assert eng.lib.battn_selftest_wait_timeout(eng.h, 0, st) == capi.ERR_ARG
    assert eng.lib.battn_selftest_wait_timeout(eng.h, 2000, st) == capi.OK
    torch.cuda.synchronize()
    assert eng.device_status(clear=False) == capi.DEV_WAIT_TIMEOUT      # reported ...
    assert eng.device_status(clear=True) == capi.DEV_WAIT_TIMEOUT       # ... sticky until cleared ...
    assert eng.device_status() == 0                                     # ... and cleared
    # the context is intact: an ordinary decode still runs and is correct
    _, k, v = draw_qkv(g, 600, 1, seed=3)
    kvk, kvv = eng.alloc_kv_layer(False, fill=0)
    gpu_fill(eng, k, v, kvk, kvv, False)
    q = torch.randn((1, 1, g.n_head, g.head_dim), device="cuda").half()
    out = new_out(eng, 1, 1, g.n_head, g.head_dim)
    ref = torch.empty_like(out)
    pos = dev_i32([599], "cuda")
    eng.launch_attn_m(out, q, kvk, kvv, pos, eng.alloc_part(1, 1), 1)
    ws = torch.empty(eng.exact_workspace_bytes(1, 1, 4), dtype=torch.uint8, device="cuda")
    eng.attn_exact(ref, q, kvk, kvv, pos, ws, 1, 1, 4)
    torch.cuda.synchronize()
    assert np.abs(to_np(out) - to_np(ref)).max() < 2e-3
    assert eng.device_status() == 0


def test_misaligned_pointers_are_rejected_on_the_host():
    from bruce_engine_b200 import capi
    from bruce_engine_b200.engine import AttnEngine
    from bruce_engine_b200.layout import G_B
    g = G_B.with_(slot_ctx=1024, window=128)
    eng = AttnEngine(g)
    kvk, kvv = eng.alloc_kv_layer(False, fill=0)
    raw = torch.zeros(g.n_head * g.head_dim * 2 + 64, dtype=torch.uint8, device="cuda")
    q_bad = raw[2:2 + g.n_head * g.head_dim * 2].view(torch.float16).view(1, 1, g.n_head, g.head_dim)
    q_ok = raw[:g.n_head * g.head_dim * 2].view(torch.float16).view(1, 1, g.n_head, g.head_dim)
    out = new_out(eng, 1, 1, g.n_head, g.head_dim)
    pos = dev_i32([10], "cuda")
    part = eng.alloc_part(1, 1)
    with pytest.raises(capi.BattnError) as ei:
        eng.launch_attn_m(out, q_bad, kvk, kvv, pos, part, 1)
    assert ei.value.code == capi.ERR_ARG
    with pytest.raises(capi.BattnError) as ei:
        eng.launch_attn_m(out, q_ok, kvk, kvv, pos, part[8:], 1)
    assert ei.value.code == capi.ERR_ARG
    assert torch.isnan(out).all()                  # nothing was launched
