"""battn_decode_noalloc: decode attention whose split-K scratch lives inside the library instead of
in a caller-provided buffer (for hosts that cannot allocate device memory while they serve, e.g.
because their KV pool already owns all of it).  Called through the C ABI and compared with the
ordinary battn_decode on the same inputs, twice in a row with different shapes, because every call
reuses the one built-in array and finds the previous call's contents in it.

Collected last on purpose: a failure here must not hide the rest of the suite from `pytest -x`."""
import ctypes as C

import numpy as np
import pytest
import torch

from tests.gpu_util import dev_i32, gpu_fill, new_out, to_np
from oracle import oracle as O
from tests.util import assert_close, draw_qkv, oracle_fill, oracle_geom

pytestmark = pytest.mark.gpu


def _p(t):
    return None if t is None else C.c_void_p(t.data_ptr())


def test_noalloc_decode_matches_decode_on_two_consecutive_calls():
    from bruce_engine_b200 import capi
    from bruce_engine_b200.engine import AttnEngine
    from bruce_engine_b200.layout import G_B
    g = G_B.with_(slot_ctx=4096, window=512, n_slots=3)
    eng = AttnEngine(g)
    lens = [4096, 777, 65]
    og = oracle_geom(g)
    okvk, okvv = {}, {}
    for is_swa in (False, True):
        kvk, kvv = eng.alloc_kv_layer(is_swa, fill=0)
        okvk[is_swa], okvv[is_swa] = O.new_cache(og, is_swa), O.new_cache(og, is_swa)
        for s, n in enumerate(lens):
            _, k, v = draw_qkv(g, n, 1, seed=300 + s)
            gpu_fill(eng, k, v, kvk, kvv, is_swa, slot=s)
            oracle_fill(og, k, v, is_swa, slot=s, kvk=okvk[is_swa], kvv=okvv[is_swa])
        rng = np.random.default_rng(8)
        q = torch.from_numpy(rng.standard_normal((3, 1, g.n_head, g.head_dim), dtype=np.float32)).cuda().half()
        part = eng.alloc_part(3, 1)
        st = C.c_void_p(torch.cuda.current_stream().cuda_stream)
        # call 1: three sequences; call 2: one sequence at another position (a smaller scratch footprint,
        # so stale records of call 1 stay behind it in the array)
        calls = [
            (dev_i32([n - 1 for n in lens], "cuda"), dev_i32([0, 1, 2], "cuda"), dev_i32([1, 1, 1], "cuda"), q),
            (dev_i32([500], "cuda"), dev_i32([1], "cuda"), None, q[1:2].contiguous()),
        ]
        for pos, kslot, act, qq in calls:
            n_seq = pos.numel()
            want = new_out(eng, n_seq, 1, g.n_head, g.head_dim)
            got = new_out(eng, n_seq, 1, g.n_head, g.head_dim)
            rc = eng.lib.battn_decode(eng.h, _p(want), _p(qq), _p(kvk), _p(kvv), _p(pos), _p(kslot), _p(act),
                                      _p(part), n_seq, int(is_swa), st)
            assert rc == capi.OK
            rc = eng.lib.battn_decode_noalloc(eng.h, _p(got), _p(qq), _p(kvk), _p(kvv), _p(pos), _p(kslot), _p(act),
                                              n_seq, int(is_swa), st)
            assert rc == capi.OK
            torch.cuda.synchronize()
            assert_close(to_np(got), to_np(want), f"noalloc vs decode swa={is_swa} n_seq={n_seq}")
            # ... and against the CPU oracle, so that this is not only a comparison of the library with itself
            sl = [int(x) for x in kslot.cpu()]
            ref = O.attend(og, to_np(qq), okvk[is_swa], okvv[is_swa], [int(x) for x in pos.cpu()], kslot=sl, rows=1,
                           is_swa=is_swa)
            assert_close(to_np(got), ref, f"noalloc vs oracle swa={is_swa} n_seq={n_seq}")
    assert eng.device_status() == 0


def test_noalloc_rejects_requests_beyond_the_built_in_scratch():
    from bruce_engine_b200 import capi
    from bruce_engine_b200.engine import AttnEngine
    from bruce_engine_b200.layout import G_B
    g = G_B.with_(slot_ctx=64, window=32, n_slots=1024)
    eng = AttnEngine(g)
    kvk, kvv = eng.alloc_kv_layer(False, fill=0)
    n_seq = 1024                                   # needs ~18 MB of records, the array holds 4 MiB
    q = torch.zeros((n_seq, 1, g.n_head, g.head_dim), dtype=torch.float16, device="cuda")
    out = new_out(eng, n_seq, 1, g.n_head, g.head_dim)
    pos = dev_i32([0] * n_seq, "cuda")
    kslot = dev_i32(list(range(n_seq)), "cuda")
    with pytest.raises(capi.BattnError) as ei:
        eng.decode_noalloc(out, q, kvk, kvv, pos, kslot=kslot)
    assert ei.value.code == capi.ERR_CAPACITY
    assert torch.isnan(out).all()                  # nothing was launched
