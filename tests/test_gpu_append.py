"""KV append on the GPU must produce the oracle's bytes exactly (engine/src/bruce.cu:698-710)."""
import numpy as np
import pytest
import torch

from oracle import oracle as O
from tests.gpu_util import dev_i32, gpu_fill
from tests.util import draw_qkv, oracle_fill, oracle_geom

pytestmark = pytest.mark.gpu


def _engine(g):
    from bruce_engine_b200.engine import AttnEngine
    return AttnEngine(g)


@pytest.mark.parametrize("name", ["B", "R"])
@pytest.mark.parametrize("is_swa", [False, True])
def test_append_bytes_exact(name, is_swa):
    from bruce_engine_b200.layout import G_B, G_R
    g = (G_B if name == "B" else G_R).with_(slot_ctx=1536, window=256, n_slots=2)
    eng = _engine(g)
    og = oracle_geom(g)
    n = 1400 if not is_swa else 2 * g.window + 300          # the ring wraps
    for scale in (1.0, 1e-4, 1e3):
        _, k, v = draw_qkv(g, n, 1, seed=11)
        k *= np.float32(scale)
        v *= np.float32(scale)
        k[3, 0, :32] = 0.0                                   # zero block -> scale 0
        kvk, kvv = eng.alloc_kv_layer(is_swa, fill=0xCD)
        ok, ov = O.new_cache(og, is_swa, fill=0xCD), O.new_cache(og, is_swa, fill=0xCD)
        # slot 1 through the multi-slot form, rows in ragged chunks
        gpu_fill(eng, k, v, kvk, kvv, is_swa, slot=1, chunk=333)
        oracle_fill(og, k, v, is_swa, slot=1, kvk=ok, kvv=ov)
        assert (kvk.cpu().numpy() == ok).all(), f"K bytes differ (scale {scale})"
        assert (kvv.cpu().numpy() == ov).all(), f"V bytes differ (scale {scale})"
    assert eng.device_status() == 0


def test_append_single_sequence_form_and_slot_base_pointer():
    from bruce_engine_b200.layout import G_B
    g = G_B.with_(slot_ctx=512, window=64, n_slots=3)
    eng = _engine(g)
    og = oracle_geom(g)
    _, k, v = draw_qkv(g, 300, 1, seed=12)
    kvk, kvv = eng.alloc_kv_layer(False, fill=0)
    off = g.slot_offset(2, False)
    gpu_fill(eng, k, v, kvk[off:], kvv[off:], False, slot=None, start=7, chunk=100)   # M.kvk_ptr[b] form
    ok, ov = oracle_fill(og, k, v, False, slot=2, start=7)
    assert (kvk.cpu().numpy() == ok).all() and (kvv.cpu().numpy() == ov).all()


def test_append_multi_slot_rows_and_idle_rows():
    from bruce_engine_b200.layout import G_B
    g = G_B.with_(slot_ctx=256, window=64, n_slots=4)
    eng = _engine(g)
    og = oracle_geom(g)
    rng = np.random.default_rng(13)
    k = rng.standard_normal((4, 1, g.n_kv, g.head_dim), dtype=np.float32)
    v = rng.standard_normal((4, 1, g.n_kv, g.head_dim), dtype=np.float32)
    pos, kslot, act = [5, 200, 0, 255], [2, 0, 3, 1], [1, 0, 1, 1]
    for is_swa in (False, True):
        kvk, kvv = eng.alloc_kv_layer(is_swa, fill=0xEE)
        ok, ov = O.new_cache(og, is_swa, fill=0xEE), O.new_cache(og, is_swa, fill=0xEE)
        eng.qkv_prep_store(torch.from_numpy(k).cuda(), torch.from_numpy(v).cuda(), kvk, kvv,
                           dev_i32(pos, eng.device), kslot=dev_i32(kslot, eng.device),
                           act=dev_i32(act, eng.device), rows=1, is_swa=is_swa)
        O.kv_append(og, k, v, ok, ov, pos, kslot=kslot, act=act, rows=1, is_swa=is_swa)
        assert (kvk.cpu().numpy() == ok).all() and (kvv.cpu().numpy() == ov).all()
    assert eng.device_status() == 0


def test_append_out_of_range_position_is_reported_not_written():
    from bruce_engine_b200 import capi
    from bruce_engine_b200.layout import G_B
    g = G_B.with_(slot_ctx=64, window=32)
    eng = _engine(g)
    k = torch.zeros((1, 1, g.n_kv, g.head_dim), device="cuda") + 1.0
    kvk, kvv = eng.alloc_kv_layer(False, fill=0x11)
    eng.qkv_prep_store(k, k, kvk, kvv, dev_i32([64], eng.device), rows=1)        # one past the end
    assert eng.device_status() & capi.DEV_BAD_POSITION
    assert (kvk == 0x11).all() and (kvv == 0x11).all()
    assert eng.device_status() == 0                                              # cleared by the read


def test_append_rejects_a_call_that_wraps_the_ring():
    from bruce_engine_b200 import capi
    from bruce_engine_b200.layout import G_B
    g = G_B.with_(slot_ctx=1024, window=64)
    eng = _engine(g)
    kvk, kvv = eng.alloc_kv_layer(True, fill=0)
    k = torch.zeros((1, 129, g.n_kv, g.head_dim), device="cuda")
    with pytest.raises(capi.BattnError) as ei:
        eng.qkv_prep_store(k, k, kvk, kvv, dev_i32([0], eng.device), rows=129, is_swa=True)
    assert ei.value.code == capi.ERR_CAPACITY
    eng.qkv_prep_store(k[:, :128], k[:, :128], kvk, kvv, dev_i32([0], eng.device), rows=128, is_swa=True)
