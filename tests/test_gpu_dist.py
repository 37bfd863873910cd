"""Sequence split across GPUs (BASELINE config 4b at small size): every rank runs battn_partials on
its position shard, the (o, m, l) records are all-gathered over NCCL and merged by battn_merge; the
result must equal the single-cache oracle.  Needs >= 2 GPUs (skipped otherwise)."""
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


def _worker(rank, world, port, n_total, cases, q_all, k, v, ret):
    import torch.distributed as dist

    from bruce_engine_b200 import dist as bd
    from bruce_engine_b200.engine import AttnEngine
    from bruce_engine_b200.layout import G_B
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        sh = bd.shard_of(n_total, rank, world)
        g = G_B.with_(slot_ctx=max(2, sh.capacity), window=128)
        eng = AttnEngine(g, rank)
        kvk, kvv = eng.alloc_kv_layer(False, fill=0)
        dec = bd.SeqSplitDecoder(eng, n_total)
        kd, vd = torch.from_numpy(k).cuda(), torch.from_numpy(v).cuda()
        for a in range(0, n_total, 128):                    # every rank sees every append; owners store
            b = min(n_total, a + 128)
            for s in range(world):                         # blocks are cut at shard boundaries
                so = bd.shard_of(n_total, s, world)
                lo, hi = max(a, so.start), min(b, so.end)
                if lo < hi:
                    dec.append(kd[None, lo:hi], vd[None, lo:hi], kvk, kvv, lo, hi - lo)
        outs = []
        for ci, (p0, rows) in enumerate(cases):
            q = torch.from_numpy(q_all[ci][:rows]).cuda().half().contiguous()
            out = torch.full((rows, g.n_head, g.head_dim), float("nan"), dtype=torch.float16, device="cuda")
            dec.decode(out, q, kvk, kvv, p0, rows)
            torch.cuda.synchronize()
            outs.append(out.float().cpu().numpy())
        assert eng.device_status() == 0
        # every rank must hold the same merged output
        chk = torch.from_numpy(np.concatenate([o.reshape(-1) for o in outs])).cuda()
        ref = chk.clone()
        dist.broadcast(ref, 0)
        assert torch.equal(chk, ref)
        if rank == 0:
            ret.put(outs)
    finally:
        dist.destroy_process_group()


def test_sequence_split_decode_over_nccl():
    import torch.multiprocessing as mp

    from oracle import oracle as O
    from tests.util import assert_close
    world = min(torch.cuda.device_count(), 4)
    if world < 2:
        pytest.skip("needs at least 2 GPUs")
    n_total = 4000
    g = O.Geom(n_head=32, n_kv=8, head_dim=128, window=128, slot_ctx=n_total)
    rng = np.random.default_rng(31)
    k = rng.standard_normal((n_total, g.n_kv, g.head_dim), dtype=np.float32)
    v = rng.standard_normal((n_total, g.n_kv, g.head_dim), dtype=np.float32)
    cases = [(n_total - 1, 1), (n_total - 4, 4), (n_total // world - 2, 2), (0, 1)]
    q_all = [rng.standard_normal((4, g.n_head, g.head_dim), dtype=np.float32).astype(np.float16).astype(np.float32)
             for _ in cases]
    kvk, kvv = O.new_cache(g, False), O.new_cache(g, False)
    O.kv_append(g, k[None], v[None], kvk, kvv, [0], rows=n_total)
    ctx = mp.get_context("spawn")
    ret = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, n_total, cases, q_all, k, v, ret)) for r in range(world)]
    for p in procs:
        p.start()
    outs = ret.get(timeout=300)
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    for (p0, rows), q, got in zip(cases, q_all, outs):
        want = O.attend(g, q[None, :rows], kvk, kvv, [p0], rows=rows)[0]
        assert_close(got, want, f"sequence split world={world} p0={p0} rows={rows}")
