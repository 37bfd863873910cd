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


class SeqSplitDecoder:
    """Decode attention over one sequence whose KV cache is split by position range across the ranks
    of a process group (full-causal layers; window layers stay on the owner of the tail)."""

    MAX_ROWS = 8     # rows per decode call (the verify limit, bruce.cu:94)

    def __init__(self, engine, n_total: int, group=None):
        self.eng, self.group = engine, group
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        self.shard = shard_of(n_total, self.rank, self.world)
        g = engine.geom
        if g.slot_ctx < self.shard.capacity:
            raise ValueError("engine slot_ctx is smaller than this rank's shard")
        dev = engine.device
        # decode() runs either `rows` one-row sequences (shards that lie wholly before the block) or one
        # sequence of `rows` rows (the shard that holds the block): the scratch must serve both shapes
        self.part = torch.empty(max(engine.workspace_bytes(self.MAX_ROWS, 1), engine.workspace_bytes(1, self.MAX_ROWS)),
                                dtype=torch.uint8, device=dev)
        self._pos = torch.zeros(8, dtype=torch.int32, device=dev)
        self._kslot = torch.zeros(8, dtype=torch.int32, device=dev)

    def append(self, k, v, kvk, kvv, p0: int, rows: int = 1):
        """Store rows at global positions p0.. on their owner (other ranks do nothing)."""
        if not (self.shard.start <= p0 and p0 + rows <= self.shard.end):
            return False
        pos = torch.tensor([p0 - self.shard.start], dtype=torch.int32, device=self.eng.device)
        self.eng.qkv_prep_store(k, v, kvk, kvv, pos, rows=rows)
        return True

    def decode(self, out, q, kvk, kvv, p0: int, rows: int = 1):
        """q, out: [rows][n_head][head_dim] (replicated on every rank).  Returns out."""
        g, eng = self.eng.geom, self.eng
        if not 1 <= rows <= self.MAX_ROWS or rows * g.group > 32:
            raise ValueError(f"rows must be 1..{self.MAX_ROWS} with rows * heads-per-kv-head <= 32")
        active, lp0, lrows = local_query(self.shard, p0, rows)
        rec = empty_records(rows, g.n_head, g.head_dim, eng.device)
        if active and lrows == 0:
            # every row sees the whole shard: rows become independent 1-row sequences of slot 0
            self._pos[:rows].fill_(lp0)
            eng.attn_partials(rec, q, kvk, kvv, self._pos[:rows], self.part, rows=1, batch=rows,
                              kslot=self._kslot[:rows])
        elif active:
            self._pos[:1].fill_(lp0)
            eng.attn_partials(rec, q, kvk, kvv, self._pos[:1], self.part, rows=rows, batch=1)
        recs = gather_records(rec, self.group)
        eng.attn_combine(out, recs, self.world, rows)
        return out
