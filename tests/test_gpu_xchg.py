"""The cross-device exchange of split records (battn_partials_push / battn_merge_wait) exercised on ONE GPU: two
"devices" of a sequence split are two exchange objects on the same GPU whose receive areas are connected by raw
pointers.  All launches go to one stream in an order in which no kernel waits for a later one (both shards push
first, then both merge), so nothing here depends on two kernels running at the same time.

Also here: the bounded wait of the merge.  A shard whose peer never pushes must give up after its poll limit, set
BATTN_DEV_WAIT_TIMEOUT, leave the output untouched and leave the context and the exchange usable."""
import numpy as np
import pytest
import torch

from oracle import oracle as O
from tests.gpu_util import dev_i32, dev_q, gpu_fill, new_out, to_np
from tests.util import assert_close, draw_qkv, oracle_fill, oracle_geom

pytestmark = pytest.mark.gpu


def _pair(n_total, rows_q=8, seed=5):
    """One sequence of n_total positions split in two halves, each half in the cache of its own engine."""
    from bruce_engine_b200.engine import AttnEngine
    from bruce_engine_b200.layout import G_B
    half = n_total // 2
    g = G_B.with_(slot_ctx=half, window=128)
    q, k, v = draw_qkv(g, n_total, rows_q, seed)
    engs, caches, xs = [], [], []
    for r in range(2):
        eng = AttnEngine(g)
        kvk, kvv = eng.alloc_kv_layer(False, fill=0)
        gpu_fill(eng, k[r * half:(r + 1) * half], v[r * half:(r + 1) * half], kvk, kvv, False)
        x, _ = eng.xchg_create(r, 2, 8)
        engs.append(eng); caches.append((kvk, kvv)); xs.append(x)
    areas = [engs[r].xchg_area(xs[r])[0] for r in range(2)]
    for r in range(2):
        engs[r].xchg_connect_ptrs(xs[r], areas)
    og = oracle_geom(g.with_(slot_ctx=n_total))
    okvk, okvv = oracle_fill(og, k, v, False)
    return g, q, engs, caches, xs, (og, okvk, okvv)


def test_two_shards_on_one_gpu_push_then_merge():
    n_total = 3000
    g, q, engs, caches, xs, (og, okvk, okvv) = _pair(n_total)
    half = n_total // 2
    epochs = [torch.zeros(1, dtype=torch.int32, device="cuda") for _ in range(2)]
    parts = [e.alloc_part(8, 1) for e in engs]
    parts1 = [e.alloc_part(1, 8) for e in engs]
    kslot = dev_i32([0] * 8, "cuda")
    for step, rows in enumerate((1, 4, 8, 1)):
        p0 = n_total - rows
        qd = dev_q(engs[0], q[:, :rows])[0].contiguous()
        outs = [new_out(engs[r], rows, g.n_head, g.head_dim) for r in range(2)]
        # shard 0 lies wholly before the block: `rows` one-row sequences at its last position;
        # shard 1 holds the block: one sequence of `rows` rows
        engs[0].attn_partials_push(xs[0], None, qd, *caches[0], dev_i32([half - 1] * rows, "cuda"), parts[0], epochs[0],
                                   rows=1, batch=rows, kslot=kslot[:rows])
        engs[1].attn_partials_push(xs[1], None, qd, *caches[1], dev_i32([p0 - half], "cuda"), parts1[1], epochs[1],
                                   rows=rows, batch=1)
        for r in range(2):
            engs[r].attn_merge_wait(xs[r], outs[r], rows, epochs[r])
        torch.cuda.synchronize()
        assert int(epochs[0].item()) == int(epochs[1].item()) == step + 1
        want = O.attend(og, q[:, :rows], okvk, okvv, [p0], rows=rows)[0]
        for r in range(2):
            assert_close(to_np(outs[r]), want, f"two shards, rows={rows}, merged on shard {r}")
        assert torch.equal(outs[0], outs[1])
    for r in range(2):
        assert engs[r].device_status() == 0
        engs[r].xchg_destroy(xs[r])


def test_single_device_exchange_equals_plain_decode():
    """world = 1: the fused push + wait + merge of one launch must give exactly battn_decode's result."""
    from bruce_engine_b200.engine import AttnEngine
    from bruce_engine_b200.layout import G_B
    g = G_B.with_(slot_ctx=2048, window=128)
    eng = AttnEngine(g)
    q, k, v = draw_qkv(g, 2000, 1, seed=9)
    kvk, kvv = eng.alloc_kv_layer(False, fill=0)
    gpu_fill(eng, k, v, kvk, kvv, False)
    x, _ = eng.xchg_create(0, 1, 8)
    eng.xchg_connect(x, b"")
    epoch = torch.zeros(1, dtype=torch.int32, device="cuda")
    part = eng.alloc_part(1, 1)
    qd = dev_q(eng, q)
    pos = dev_i32([1999], "cuda")
    want = new_out(eng, 1, 1, g.n_head, g.head_dim)
    eng.launch_attn_m(want, qd, kvk, kvv, pos, part, 1)
    for step in range(3):
        got = new_out(eng, 1, g.n_head, g.head_dim)
        eng.attn_partials_push(x, got, qd[0], kvk, kvv, pos, part, epoch)
        torch.cuda.synchronize()
        assert torch.equal(got, want[0]), f"step {step}"
    assert eng.device_status() == 0
    eng.xchg_destroy(x)


def test_merge_gives_up_when_a_peer_never_pushes_and_recovers():
    from bruce_engine_b200 import capi
    n_total = 1024
    g, q, engs, caches, xs, (og, okvk, okvv) = _pair(n_total, seed=6)
    half = n_total // 2
    for r in range(2):
        engs[r].xchg_set_wait_polls(xs[r], 2000)                 # a fraction of a millisecond
    epochs = [torch.zeros(1, dtype=torch.int32, device="cuda") for _ in range(2)]
    parts = [e.alloc_part(1, 1) for e in engs]
    qd = dev_q(engs[0], q[:, :1])[0].contiguous()
    p0 = n_total - 1
    pos0, pos1 = dev_i32([half - 1], "cuda"), dev_i32([p0 - half], "cuda")
    # step 1: shard 1 sits the step out.  Shard 0 pushes, waits for a record that never comes, gives up.
    out0 = new_out(engs[0], 1, g.n_head, g.head_dim)
    engs[0].attn_partials_push(xs[0], out0, qd, *caches[0], pos0, parts[0], epochs[0])
    torch.cuda.synchronize()
    assert engs[0].device_status() == capi.DEV_WAIT_TIMEOUT
    assert torch.isnan(out0).all(), "a timed-out merge must not write an output"
    # step 2: shard 1 is back, one step behind: it advances its counter by two.  Shard 1 pushes first (push only),
    # then shard 0 pushes and merges, then shard 1 merges.
    outs = [new_out(engs[r], 1, g.n_head, g.head_dim) for r in range(2)]
    engs[1].attn_partials_push(xs[1], None, qd, *caches[1], pos1, parts[1], epochs[1], epoch_advance=2)
    engs[0].attn_partials_push(xs[0], outs[0], qd, *caches[0], pos0, parts[0], epochs[0])
    engs[1].attn_merge_wait(xs[1], outs[1], 1, epochs[1])
    torch.cuda.synchronize()
    want = O.attend(og, q[:, :1], okvk, okvv, [p0], rows=1)[0]
    for r in range(2):
        assert engs[r].device_status() == 0
        assert_close(to_np(outs[r]), want, f"step after the time-out, shard {r}")
        engs[r].xchg_destroy(xs[r])
