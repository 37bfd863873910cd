"""Sequence split across GPUs (BASELINE config 4b at small size): every rank decodes on its position shard; the
per-shard (o, m, l) records are exchanged either by the push epilogue (plain stores into the peers' receive areas
over NVLink, battn_partials_push) or by an NCCL all-gather (battn_partials + battn_merge); the result must equal
the single-cache oracle on every rank.  Also: a rank that sits out a step between two steps (a host-side decision;
no kernel is in flight on it) makes its peers' merge give up at its wait bound and report the status bit, and the
step after that is correct again.  Needs >= 2 GPUs (skipped otherwise)."""
import os
import socket

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, n_total, cases, q_all, k, v, exchange, skip_case, ret):
    import torch.distributed as dist

    from bruce_engine_b200 import capi
    from bruce_engine_b200 import dist as bd
    from bruce_engine_b200.engine import AttnEngine
    from bruce_engine_b200.layout import G_B
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        sh = bd.shard_of(n_total, rank, world)
        g = G_B.with_(slot_ctx=max(2, sh.capacity), window=128)
        eng = AttnEngine(g, rank)
        kvk, kvv = eng.alloc_kv_layer(False, fill=0)
        dec = bd.SeqSplitDecoder(eng, n_total, exchange=exchange)
        if dec.x is not None:
            eng.xchg_set_wait_polls(dec.x, 20000)           # a few milliseconds: the skipped step must not take long
        kd, vd = torch.from_numpy(k).cuda(), torch.from_numpy(v).cuda()
        for a in range(0, n_total, 128):                    # every rank sees every append; owners store
            b = min(n_total, a + 128)
            for s in range(world):                         # blocks are cut at shard boundaries
                so = bd.shard_of(n_total, s, world)
                lo, hi = max(a, so.start), min(b, so.end)
                if lo < hi:
                    dec.append(kd[None, lo:hi], vd[None, lo:hi], kvk, kvv, lo, hi - lo)
        outs, status = [], []
        for ci, (p0, rows) in enumerate(cases):
            q = torch.from_numpy(q_all[ci][:rows]).cuda().half().contiguous()
            out = torch.full((rows, g.n_head, g.head_dim), float("nan"), dtype=torch.float16, device="cuda")
            if ci == skip_case and rank == world - 1:
                dec.skip_step()                             # this rank sits the step out (decided between steps)
            else:
                dec.decode(out, q, kvk, kvv, p0, rows)
            torch.cuda.synchronize()
            dist.barrier()                                  # a step ends before the next one starts
            outs.append(out.float().cpu().numpy())
            status.append(eng.device_status())
        # every rank that took part must hold the same merged output
        for ci in range(len(cases)):
            if ci == skip_case:
                continue
            chk = torch.from_numpy(outs[ci].reshape(-1)).cuda()
            ref = chk.clone()
            dist.broadcast(ref, 0)
            assert torch.equal(chk, ref)
        if skip_case is not None:
            want = 0 if rank == world - 1 else capi.DEV_WAIT_TIMEOUT
            assert status[skip_case] == want, f"rank {rank}: status {status[skip_case]} on the skipped step"
            assert np.isnan(outs[skip_case]).all()
            assert all(s == 0 for i, s in enumerate(status) if i != skip_case)
        else:
            assert all(s == 0 for s in status)
        dec.close()
        if rank == 0:
            ret.put(outs)
    finally:
        dist.destroy_process_group()


def _window_worker(rank, world, port, n_total, W, q, k, v, ret):
    import torch.distributed as dist

    from bruce_engine_b200 import dist as bd
    from bruce_engine_b200.engine import AttnEngine
    from bruce_engine_b200.layout import G_B
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        sh = bd.shard_of(n_total, rank, world)
        g = G_B.with_(slot_ctx=max(2, sh.capacity), window=W)
        eng = AttnEngine(g, rank)
        dec = bd.SeqSplitDecoder(eng, n_total, exchange="nccl")
        kvk, kvv = eng.alloc_kv_layer(True, fill=0)                 # the ring of the window layer (2W slots)
        p0 = n_total - 1
        owner = bd.owner_of(p0, n_total, world)
        if rank == owner:                                           # only the tail's owner holds the layer
            kd, vd = torch.from_numpy(k).cuda(), torch.from_numpy(v).cuda()
            first = max(0, n_total - 2 * W)
            for a in range(first, n_total, 64):
                b = min(n_total, a + 64)
                eng.qkv_prep_store(kd[None, a:b], vd[None, a:b], kvk, kvv, torch.tensor([a], dtype=torch.int32, device="cuda"),
                                   rows=b - a, is_swa=True)
        qd = torch.from_numpy(q).cuda().half().contiguous()
        out = torch.full((1, g.n_head, g.head_dim), float("nan"), dtype=torch.float16, device="cuda")
        dec.decode_window(out, qd, kvk, kvv, p0, 1)
        torch.cuda.synchronize()
        assert eng.device_status() == 0
        ret.put((rank, out.float().cpu().numpy()))
        dist.barrier()
    finally:
        dist.destroy_process_group()


def test_window_layer_of_a_split_sequence_is_served_by_the_owner_of_the_tail():
    import torch.multiprocessing as mp

    from oracle import oracle as O
    from tests.util import assert_close
    world = min(torch.cuda.device_count(), 4)
    if world < 2:
        pytest.skip("needs at least 2 GPUs")
    n_total, W = 3000, 256
    g = O.Geom(n_head=32, n_kv=8, head_dim=128, window=W, slot_ctx=n_total)
    rng = np.random.default_rng(53)
    k = rng.standard_normal((n_total, g.n_kv, g.head_dim), dtype=np.float32)
    v = rng.standard_normal((n_total, g.n_kv, g.head_dim), dtype=np.float32)
    q = rng.standard_normal((1, g.n_head, g.head_dim), dtype=np.float32).astype(np.float16).astype(np.float32)
    kvk, kvv = O.new_cache(g, True), O.new_cache(g, True)
    first = max(0, n_total - 2 * W)
    O.kv_append(g, k[None, first:], v[None, first:], kvk, kvv, [first], rows=n_total - first, is_swa=True)
    want = O.attend(g, q[None], kvk, kvv, [n_total - 1], rows=1, is_swa=True)[0]
    ctx = mp.get_context("spawn")
    ret = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_window_worker, args=(r, world, port, n_total, W, q, k, v, ret)) for r in range(world)]
    for p in procs:
        p.start()
    outs = dict(ret.get(timeout=300) for _ in range(world))
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    for r in range(world):
        assert_close(outs[r], want, f"window layer of the split sequence on rank {r}")


def _run(n_total, cases, exchange, skip_case=None, seed=31):
    import torch.multiprocessing as mp

    from oracle import oracle as O
    from tests.util import assert_close
    world = min(torch.cuda.device_count(), 4)
    if world < 2:
        pytest.skip("needs at least 2 GPUs")
    g = O.Geom(n_head=32, n_kv=8, head_dim=128, window=128, slot_ctx=n_total)
    rng = np.random.default_rng(seed)
    k = rng.standard_normal((n_total, g.n_kv, g.head_dim), dtype=np.float32)
    v = rng.standard_normal((n_total, g.n_kv, g.head_dim), dtype=np.float32)
    q_all = [rng.standard_normal((8, g.n_head, g.head_dim), dtype=np.float32).astype(np.float16).astype(np.float32)
             for _ in cases]
    kvk, kvv = O.new_cache(g, False), O.new_cache(g, False)
    O.kv_append(g, k[None], v[None], kvk, kvv, [0], rows=n_total)
    ctx = mp.get_context("spawn")
    ret = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, n_total, cases, q_all, k, v, exchange, skip_case, ret))
             for r in range(world)]
    for p in procs:
        p.start()
    outs = ret.get(timeout=300)
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    for ci, ((p0, rows), q, got) in enumerate(zip(cases, q_all, outs)):
        if ci == skip_case:
            continue
        want = O.attend(g, q[None, :rows], kvk, kvv, [p0], rows=rows)[0]
        assert_close(got, want, f"sequence split ({exchange}) world={world} p0={p0} rows={rows}")


@pytest.mark.parametrize("exchange", ["push", "nccl"])
def test_sequence_split_decode(exchange):
    world = min(torch.cuda.device_count(), 4)
    n_total = 4000
    # the same shape twice in a row: the second and third use run from the captured graph
    cases = [(n_total - 1, 1), (n_total - 1, 1), (n_total - 1, 1), (n_total - 4, 4), (n_total // max(world, 1) - 2, 2),
             (0, 1), (n_total - 4, 4), (n_total - 4, 4)]
    _run(n_total, cases, exchange)


def test_eight_rows_on_deep_shards():
    """rows = 8 (the wide verify kernel, 32 (row, head) pairs per KV head) on shards of more than 4K positions:
    the scratch must be sized for this shape on the rank that holds the block and for 8 one-row sequences elsewhere."""
    n_total = 20000
    _run(n_total, [(n_total - 8, 8), (n_total - 8, 8), (n_total - 8, 8)], "push", seed=37)


def test_a_rank_that_sits_out_a_step_times_out_its_peers_and_the_next_step_recovers():
    n_total = 3000
    _run(n_total, [(n_total - 1, 1), (n_total - 1, 1), (n_total - 2, 2), (n_total - 1, 1)], "push", skip_case=1, seed=41)
