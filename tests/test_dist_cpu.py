"""Host-side logic of the multi-GPU schemes, run as world_size-2 (and 4) gloo ranks on CPU.
The per-shard attention is provided by the CPU oracle here (this is the test of the partitioning and
exchange logic, not of the kernels); the CUDA counterpart is tests/test_gpu_dist.py."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from bruce_engine_b200 import dist as bd
from oracle import oracle as O


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def test_balance_slots_is_a_balanced_partition():
    rng = np.random.default_rng(0)
    ctx = rng.integers(1024, 131073, size=64)            # BASELINE config 4a draw
    for world in (1, 2, 4, 8):
        parts = bd.balance_slots(ctx, world)
        assert sorted(i for p in parts for i in p) == list(range(64))
        loads = [int(ctx[p].sum()) for p in parts]
        assert max(loads) - min(loads) <= int(ctx.max())
        assert max(loads) <= 1.05 * sum(loads) / world + 1
    assert bd.kv_heads_of(1, 4, 8) == [1, 5] and bd.kv_heads_of(0, 8, 8) == [0]
    with pytest.raises(ValueError):
        bd.kv_heads_of(0, 3, 8)


def test_shard_ranges_cover_the_sequence():
    for n, world in ((1_048_576, 8), (1000, 4), (7, 4), (10, 1)):
        shards = [bd.shard_of(n, r, world) for r in range(world)]
        assert shards[0].start == 0 and shards[-1].end == n
        for a, b in zip(shards[:-1], shards[1:]):
            assert a.end == b.start and a.start % 2 == 0
        for p in (0, n // 2, n - 1):
            o = bd.owner_of(p, n, world)
            assert shards[o].start <= p < shards[o].end
    sh = bd.shard_of(1000, 1, 4)                          # [250, 500)
    assert bd.local_query(sh, 999, 1) == (True, 249, 0)   # every key of the shard is visible
    assert bd.local_query(sh, 300, 2) == (True, 50, 2)
    assert bd.local_query(sh, 100, 1) == (False, 0, 0)
    with pytest.raises(ValueError):
        bd.local_query(sh, 499, 2)


def _seq_split_worker(rank, world, port, n_total, p0, rows, q, k, v, ret):
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        g = O.Geom(n_head=8, n_kv=2, head_dim=128, window=64, slot_ctx=max(2, bd.shard_of(n_total, 0, world).capacity))
        sh = bd.shard_of(n_total, rank, world)
        kvk, kvv = O.new_cache(g, False), O.new_cache(g, False)
        if sh.capacity:
            O.kv_append(g, k[None, sh.start:sh.end], v[None, sh.start:sh.end], kvk, kvv, [0], rows=sh.capacity)
        active, lp0, lrows = bd.local_query(sh, p0, rows)
        rec = bd.empty_records(rows, g.n_head, g.head_dim, "cpu")
        if active and lrows == 0:
            r = O.attend(g, q.reshape(rows, 1, g.n_head, g.head_dim), kvk, kvv, [lp0] * rows, kslot=[0] * rows,
                         rows=1, records=True)
            rec = torch.from_numpy(r.reshape(rows, g.n_head, g.head_dim + 2))
        elif active:
            r = O.attend(g, q[None], kvk, kvv, [lp0], rows=rows, records=True)
            rec = torch.from_numpy(r[0])
        recs = bd.gather_records(rec)                                   # [world][rows][heads][HD+2]
        assert recs.shape == (world, rows, g.n_head, g.head_dim + 2)
        out = O.merge(recs.numpy())
        if rank == 0:
            ret.put(out)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4])
def test_sequence_split_decode_over_gloo_ranks(world):
    n_total, rows = 1000, 2
    rng = np.random.default_rng(world)
    g = O.Geom(n_head=8, n_kv=2, head_dim=128, window=64, slot_ctx=n_total)
    q = rng.standard_normal((rows, g.n_head, g.head_dim), dtype=np.float32)
    k = rng.standard_normal((n_total, g.n_kv, g.head_dim), dtype=np.float32)
    v = rng.standard_normal((n_total, g.n_kv, g.head_dim), dtype=np.float32)
    kvk, kvv = O.new_cache(g, False), O.new_cache(g, False)
    O.kv_append(g, k[None], v[None], kvk, kvv, [0], rows=n_total)
    for p0 in (n_total - rows, 600):                                    # tail block; a block inside shard 2 of 4 / 1 of 2
        want = O.attend(g, q[None], kvk, kvv, [p0], rows=rows)[0]
        ctx = mp.get_context("spawn")
        ret = ctx.Queue()
        port = _free_port()
        procs = [ctx.Process(target=_seq_split_worker, args=(r, world, port, n_total, p0, rows, q, k, v, ret))
                 for r in range(world)]
        for p in procs:
            p.start()
        got = ret.get(timeout=120)
        for p in procs:
            p.join(timeout=60)
            assert p.exitcode == 0
        assert np.abs(got - want).max() < 1e-5


# ---- the exchange protocol of the sequence split (step numbers, parity buffers, bounded wait) among CPU ranks --------
def _xchg_worker(rank, world, port, ret):
    """Four steps of a 3-rank group.  Step 2: the last rank sits out (its peers time out, it catches up with
    advance = 2).  Step 3: rank 0's push to rank 1 is dropped (only rank 1 times out).  Steps 1 and 4: everybody
    merges the same records."""
    store = dist.TCPStore("127.0.0.1", port, world, is_master=(rank == 0), timeout=__import__("datetime").timedelta(seconds=30))
    x = bd.HostExchange(store, rank, world, wait_s=0.4)
    store.set(f"ready/{rank}", "1")
    store.wait([f"ready/{r}" for r in range(world)])
    H, HD = 4, 8
    log = []

    def record(step):
        rng = np.random.default_rng(1000 * step + rank)
        rec = rng.standard_normal((1, H, HD + 2)).astype(np.float32)
        rec[..., HD + 1] = np.abs(rec[..., HD + 1]) + 0.5          # l > 0
        return rec

    def fix_l(a):
        a = a.copy(); a[..., HD + 1] = np.abs(a[..., HD + 1]) + 0.5; return a

    def want(step):
        return O.merge(np.stack([fix_l(np.random.default_rng(1000 * step + r).standard_normal((1, H, HD + 2)).astype(np.float32))
                                 for r in range(world)]))

    def barrier(tag):
        store.set(f"bar/{tag}/{rank}", "1")
        store.wait([f"bar/{tag}/{r}" for r in range(world)])

    # step 1: ordinary
    x.push(record(1)); out = x.wait_merge((1, H, HD + 2)); log.append(out is not bd.HostExchange.TIMEOUT and np.allclose(out, want(1), atol=1e-6))
    barrier(1)
    # step 2: the last rank sits out; the others find a STALE record (step 0 or 1) from it and must not accept it
    if rank != world - 1:
        x.push(record(2)); out = x.wait_merge((1, H, HD + 2)); log.append(out is bd.HostExchange.TIMEOUT)
    else:
        log.append(True)
    barrier(2)
    # step 3: everybody takes part again (the absentee advances by two); rank 0's copy for rank 1 is dropped
    adv = 2 if rank == world - 1 else 1
    x.push(record(3), advance=adv, drop_to=(1,) if rank == 0 else ())
    out = x.wait_merge((1, H, HD + 2))
    if rank == 1:
        log.append(out is bd.HostExchange.TIMEOUT)              # sees rank 0's record of step 1 only
    else:
        log.append(out is not bd.HostExchange.TIMEOUT and np.allclose(out, want(3), atol=1e-6))
    barrier(3)
    # step 4: ordinary again, and in the parity buffer that step 2 used: nothing stale may leak in
    x.push(record(4)); out = x.wait_merge((1, H, HD + 2)); log.append(out is not bd.HostExchange.TIMEOUT and np.allclose(out, want(4), atol=1e-6))
    barrier(4)
    assert x.epoch == 4
    ret.put((rank, log))


def test_exchange_protocol_stale_flag_dropped_push_and_absent_rank():
    world = 3
    ctx = mp.get_context("spawn")
    ret = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_xchg_worker, args=(r, world, port, ret)) for r in range(world)]
    for p in procs:
        p.start()
    got = dict(ret.get(timeout=120) for _ in range(world))
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for r in range(world):
        assert got[r] == [True, True, True, True], f"rank {r}: {got[r]}"
