"""Multi-GPU partitioning of the attention path (one process per GPU, torch.distributed).

The reference engine is single-GPU; both schemes below are new functionality built on its split
record (o[HD], m, l) and merge (engine/src/bruce.cu:781-783, 992-1007):

* Batched serving: sequences (slots) and KV heads are independent, so they are simply dealt out to the
  ranks -- no collective on the data path.  `balance_slots` does longest-processing-time balancing on
  the context lengths; `kv_heads_of` is the h mod world rule.
* One very long sequence: the position range is cut evenly, rank r holds [r*N/g, (r+1)*N/g) in its own
  cache with LOCAL positions.  A decode step runs the ordinary kernel on every shard
  (`battn_partials`), all-gathers one record per (row, head) -- n_head*(HD+2)*4 bytes per row -- and
  merges them (`battn_merge`).  The host logic here (shard ranges, local positions, record gathering)
  is backend-neutral and is tested with gloo on CPU; `SeqSplitDecoder` binds it to the CUDA engine.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.distributed as dist


# ---- batched serving: independent work, no exchange ------------------------------------------------------
def balance_slots(ctx_lens, world: int):
    """Longest-processing-time assignment of slots to ranks by context length.
    Returns a list (per rank) of slot indices; every slot appears exactly once."""
    order = sorted(range(len(ctx_lens)), key=lambda i: (-int(ctx_lens[i]), i))
    load = [0] * world
    out = [[] for _ in range(world)]
    for i in order:
        r = min(range(world), key=lambda j: (load[j], j))
        out[r].append(i)
        load[r] += int(ctx_lens[i])
    return [sorted(x) for x in out]


def kv_heads_of(rank: int, world: int, n_kv: int):
    """KV heads served by `rank` when the cache is sharded by head (h mod world)."""
    if n_kv % world:
        raise ValueError("n_kv must be a multiple of the world size for head sharding")
    return [h for h in range(n_kv) if h % world == rank]


# ---- one long sequence split by position range -----------------------------------------------------------
@dataclass(frozen=True)
class Shard:
    rank: int
    world: int
    start: int      # first global position held by this rank
    end: int        # one past the last

    @property
    def capacity(self) -> int:
        return self.end - self.start


def shard_of(n_total: int, rank: int, world: int, align: int = 2) -> Shard:
    """Even split of [0, n_total) into `world` ranges whose boundaries are multiples of `align`
    (cache capacities must be even)."""
    per = -(-n_total // world)
    per = -(-per // align) * align
    start = min(n_total, rank * per)
    end = min(n_total, start + per)
    return Shard(rank, world, start, end)


def owner_of(pos: int, n_total: int, world: int, align: int = 2) -> int:
    per = -(-n_total // world)
    per = -(-per // align) * align
    return min(world - 1, pos // per)


def local_query(shard: Shard, p0: int, rows: int = 1):
    """How a query block at global positions p0 .. p0+rows-1 (full-causal layer) looks to `shard`.

    Returns (active, local_p0, local_rows):
      * keys of the shard all precede p0          -> every row sees the whole shard: the call is made
                                                     with `rows` rows that all sit at the shard's last
                                                     local position (the caller passes rows as 1-row
                                                     sequences), signalled by local_rows == 0
      * the block starts inside the shard         -> ordinary call at local position p0 - start
      * the shard starts after the block's end    -> inactive (contributes the empty record)
    Blocks that straddle a shard boundary are not supported (append keeps a block inside one shard)."""
    if shard.capacity == 0 or shard.start > p0 + rows - 1:
        return False, 0, 0
    if shard.end <= p0:
        return True, shard.capacity - 1, 0
    if p0 < shard.start or p0 + rows > shard.end:
        raise ValueError("a query block must not straddle a shard boundary")
    return True, p0 - shard.start, rows


def gather_records(rec_local: torch.Tensor, group=None) -> torch.Tensor:
    """All-gather one split-record block per rank: [rows][n_head][HD+2] -> [world][rows][n_head][HD+2]."""
    world = dist.get_world_size(group)
    rec_local = rec_local.contiguous()
    flat = torch.empty((world * rec_local.shape[0],) + tuple(rec_local.shape[1:]), dtype=rec_local.dtype,
                       device=rec_local.device)
    dist.all_gather_into_tensor(flat, rec_local, group=group)          # concatenated along dim 0, rank-major
    return flat.view((world,) + tuple(rec_local.shape))


EMPTY_M = -1e30


def empty_records(rows: int, n_head: int, head_dim: int, device) -> torch.Tensor:
    """The record of an empty key range: (0, -1e30, 0) (bruce.cu:2319-2322)."""
    rec = torch.zeros((rows, n_head, head_dim + 2), dtype=torch.float32, device=device)
    rec[..., head_dim] = EMPTY_M
    return rec


class HostExchange:
    """Host-side model of the device exchange of split records (battn_partials_push / battn_merge_wait): the same
    receive slots, the same two record buffers selected by the step's parity, the same rule that a record is the
    step's record when the step number stored WITH it has reached the step ("number >= step"; on the device every
    8-byte word of a record carries the number, here the record as a whole does), the same bounded wait.  The ranks'
    memory is a key-value store they share (any torch.distributed Store); records are numpy arrays
    [rows][n_head][head_dim + 2] with m in natural-log units.
    It exists to test the protocol -- stale records, a dropped push, a rank that sits a step out -- among CPU ranks;
    the data path on GPUs is the kernel."""

    TIMEOUT = object()

    def __init__(self, store, rank: int, world: int, wait_s: float = 0.5, poll_s: float = 0.002):
        self.store, self.rank, self.world = store, rank, world
        self.wait_s, self.poll_s = wait_s, poll_s
        self.epoch = 0
        for src in range(world):                       # this rank's receive area starts with numbers below every step
            for parity in (0, 1):
                store.set(f"rec/{rank}/{parity}/{src}", (0).to_bytes(4, "little", signed=True))

    def push(self, rec, advance: int = 1, drop_to=()):
        """Advance the step counter and store this rank's record of the step, tagged with the step number, in every
        rank's receive slot.  `drop_to`: destinations whose copy is lost (a test's way of dropping a message)."""
        import numpy as np
        self.epoch += advance
        blob = self.epoch.to_bytes(4, "little", signed=True) + np.ascontiguousarray(rec, dtype=np.float32).tobytes()
        for dst in range(self.world):
            if dst in drop_to:
                continue
            self.store.set(f"rec/{dst}/{self.epoch & 1}/{self.rank}", blob)

    def wait_merge(self, shape):
        """Wait (bounded) until every rank's record of the current step has landed here, then merge.  Returns the
        merged output [rows][n_head][head_dim], or HostExchange.TIMEOUT (nothing merged: the step is void)."""
        import time

        import numpy as np

        from oracle import oracle as O
        deadline = time.monotonic() + self.wait_s
        parts = []
        for src in range(self.world):
            while True:
                blob = self.store.get(f"rec/{self.rank}/{self.epoch & 1}/{src}")
                if int.from_bytes(blob[:4], "little", signed=True) - self.epoch >= 0:
                    break
                if time.monotonic() > deadline:
                    return HostExchange.TIMEOUT
                time.sleep(self.poll_s)
            parts.append(np.frombuffer(blob[4:], dtype=np.float32).reshape(shape))
        return O.merge(np.stack(parts))


class SeqSplitDecoder:
    """Decode attention over one sequence whose KV cache is split by position range across the ranks of a process
    group (full-causal layers: `decode`).  Sliding-window layers read only the last `window` keys: they are not
    split -- the rank that owns the tail serves them alone (`decode_window`).

    Two exchanges of the per-shard (o, m, l) records:
      * "push" (default on CUDA): the decode kernel's merge epilogue stores the records straight into every peer's
        receive area over NVLink and merges what the peers stored (battn_partials_push) -- no collective call;
      * "nccl": battn_partials, all_gather_into_tensor, battn_merge -- the baseline the push form is measured against.
    Everything a step needs is allocated here; a step allocates nothing, and each (mode, rows) shape is captured
    into a CUDA graph on its second use and replayed from then on (the shard's local position, its activity flag
    and the step counter are device-resident)."""

    MAX_ROWS = 8     # rows per decode call (the verify limit, bruce.cu:94)

    def __init__(self, engine, n_total: int, group=None, exchange: str = "push", use_graphs: bool = True):
        self.eng, self.group = engine, group
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        self.shard = shard_of(n_total, self.rank, self.world)
        self.n_total = n_total
        g = engine.geom
        if g.slot_ctx < self.shard.capacity:
            raise ValueError("engine slot_ctx is smaller than this rank's shard")
        if exchange not in ("push", "nccl"):
            raise ValueError("exchange must be 'push' or 'nccl'")
        dev = engine.device
        R = self.MAX_ROWS
        # decode() runs either `rows` one-row sequences (shards that lie wholly before the block) or one
        # sequence of `rows` rows (the shard that holds the block): the scratch must serve both shapes
        self.part = torch.empty(max(engine.workspace_bytes(R, 1), engine.workspace_bytes(1, R)),
                                dtype=torch.uint8, device=dev)
        # device-resident step parameters (the kernels read them, so captured graphs replay at new values): local
        # position and activity flag of this shard, and the step counter, which the decode kernel advances itself
        self._pos = torch.zeros(R, dtype=torch.int32, device=dev)
        self._act = torch.ones(R, dtype=torch.int32, device=dev)
        self._epoch = torch.zeros(1, dtype=torch.int32, device=dev)
        self._wpos = torch.zeros(1, dtype=torch.int32, device=dev)      # position of a window-layer call (global)
        self._wpos_host = 0
        self._cur = (0, 1)                                   # (position, activity) currently held on the device
        self._behind = 0                                     # steps of the group this rank sat out
        self._kslot = torch.zeros(R, dtype=torch.int32, device=dev)
        self._rec = torch.zeros((R, g.n_head, g.head_dim + 2), dtype=torch.float32, device=dev)
        self._recs = torch.zeros((self.world, R, g.n_head, g.head_dim + 2), dtype=torch.float32, device=dev)
        self.exchange, self.use_graphs = exchange, use_graphs
        self.step = 0
        self._graphs, self._seen = {}, set()
        self.x = None
        if exchange == "push":
            self.x, mine = engine.xchg_create(self.rank, self.world, R)
            handles = [None] * self.world
            dist.all_gather_object(handles, mine, group=group)
            engine.xchg_connect(self.x, b"".join(handles))
            dist.barrier(group=group)                        # every area is mapped before anyone pushes

    def close(self):
        if self.x is not None:
            torch.cuda.synchronize()
            dist.barrier(group=self.group)                   # nobody still pushes into an area that goes away
            self.eng.xchg_destroy(self.x)
            self.x = None

    def append(self, k, v, kvk, kvv, p0: int, rows: int = 1):
        """Store rows at global positions p0.. on their owner (other ranks do nothing)."""
        if not (self.shard.start <= p0 and p0 + rows <= self.shard.end):
            return False
        pos = torch.tensor([p0 - self.shard.start], dtype=torch.int32, device=self.eng.device)
        self.eng.qkv_prep_store(k, v, kvk, kvv, pos, rows=rows)
        return True

    # ---- one step -----------------------------------------------------------------------------------------
    def _enqueue(self, mode: str, rows: int, out, q, kvk, kvv, advance: int = 1):
        """The device work of one step (no allocation, no host synchronisation: capturable)."""
        eng, g = self.eng, self.eng.geom
        if mode == "seqs":          # every row sees the whole shard: `rows` one-row sequences of slot 0
            n_seq, r = rows, 1
        else:                       # "block": the shard holds the block; "idle": it starts behind it (act = 0)
            n_seq, r = 1, rows
        pos, act, kslot = self._pos[:n_seq], self._act[:n_seq], self._kslot[:n_seq]
        if self.exchange == "push":
            eng.attn_partials_push(self.x, out, q, kvk, kvv, pos, self.part, self._epoch, rows=r, batch=n_seq,
                                   kslot=kslot, act=act, epoch_advance=advance)
        else:
            rec = self._rec[:rows]
            eng.attn_partials(rec, q, kvk, kvv, pos, self.part, rows=r, batch=n_seq, kslot=kslot, act=act)
            flat = self._recs.view(-1)[:self.world * rec.numel()]
            dist.all_gather_into_tensor(flat, rec.reshape(-1), group=self.group)
            eng.attn_combine(out, flat.view(self.world, rows, g.n_head, g.head_dim + 2), self.world, rows)

    def decode_window(self, out, q, kvk_swa, kvv_swa, p0: int, rows: int = 1):
        """A sliding-window layer of the split sequence: it reads only the last `window` keys, so it is not split --
        the rank that owns position p0 keeps the layer's ring (under GLOBAL positions, p & (2W - 1)) and serves the
        rows alone; the others receive the result (one small broadcast).  Appends to this layer go to that rank only
        (`owner_of`)."""
        owner = owner_of(p0, self.n_total, self.world)
        if self.rank == owner:
            if self._wpos_host != p0:
                self._wpos.fill_(p0)
                self._wpos_host = p0
            self.eng.launch_attn_m(out.view((1,) + tuple(out.shape)), q.view((1,) + tuple(q.shape)), kvk_swa, kvv_swa,
                                   self._wpos, self.part, rows, True)
        if self.world > 1:
            dist.broadcast(out, src=owner if self.group is None else dist.get_global_rank(self.group, owner), group=self.group)
        return out

    def skip_step(self):
        """This rank sits out one step of the group (it neither pushes nor merges).  Its peers' merge of that step
        runs into the bounded wait and reports BATTN_DEV_WAIT_TIMEOUT; the step after it is in step again."""
        self._behind += 1

    def decode(self, out, q, kvk, kvv, p0: int, rows: int = 1):
        """q, out: [rows][n_head][head_dim] (replicated on every rank).  Returns out."""
        g = self.eng.geom
        if not 1 <= rows <= self.MAX_ROWS or rows * g.group > 32:
            raise ValueError(f"rows must be 1..{self.MAX_ROWS} with rows * heads-per-kv-head <= 32")
        active, lp0, lrows = local_query(self.shard, p0, rows)
        mode = "idle" if not active else ("seqs" if lrows == 0 else "block")
        if self._cur != (lp0, int(active)):                  # stream-ordered updates, only when something changed
            if self._cur[0] != lp0:
                self._pos.fill_(lp0)
            if self._cur[1] != int(active):
                self._act.fill_(int(active))
            self._cur = (lp0, int(active))
        if self.exchange == "nccl" and not active:
            # the plain-partials path writes no record for an inactive sequence: keep the empty one in place
            self._rec[:rows].zero_()
            self._rec[:rows, :, g.head_dim] = EMPTY_M
        advance, self._behind = 1 + self._behind, 0
        key = (mode, rows, out.data_ptr(), q.data_ptr(), kvk.data_ptr(), kvv.data_ptr())
        gr = self._graphs.get(key) if advance == 1 else None
        if gr is not None:
            gr.replay()
        elif self.use_graphs and advance == 1 and key in self._seen and self.exchange == "push":
            # second use of this shape: capture it (the captured launches do not run), then replay
            gr = torch.cuda.CUDAGraph()
            torch.cuda.synchronize()
            with torch.cuda.graph(gr):
                self._enqueue(mode, rows, out, q, kvk, kvv)
            self._graphs[key] = gr
            gr.replay()
        else:
            self._seen.add(key)
            self._enqueue(mode, rows, out, q, kvk, kvv, advance)
        return out
