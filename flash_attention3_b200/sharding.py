"""Partition of one backward problem over the GPUs of a node.

The backward has no reduction across (batch, KV head): dQ of a query head needs
only its own Q, dO, O, LSE and the K, V of its KV head; dK/dV of a KV head need
only the query heads of its group.  In BHSD layout a contiguous range of the
flattened (batch, KV head) index is a contiguous byte range of every tensor as
long as it is either whole batches or a head range inside one batch, so a shard
is described by offset pointers plus smaller batch / head counts and is run
through the same C entry point.  No collective is involved.
"""
from __future__ import annotations

import dataclasses


@dataclasses.dataclass(frozen=True)
class Shard:
    batch_begin: int      # first batch entry
    batch_count: int      # whole batches (>= 1) ...
    kv_head_begin: int    # ... or, when batch_count == 1, a KV-head range inside that batch
    kv_head_count: int

    def q_heads(self, group: int) -> tuple[int, int]:
        return self.kv_head_begin * group, self.kv_head_count * group


def plan(batch: int, heads_kv: int, world: int) -> list[list[Shard]]:
    """Contiguous split of the batch*heads_kv units over `world` ranks, as evenly as possible.

    Returns, per rank, a list of shards (usually one; two or three when a rank's range starts
    or ends inside a batch entry)."""
    units = batch * heads_kv
    out = []
    for r in range(world):
        lo = units * r // world
        hi = units * (r + 1) // world
        shards = []
        while lo < hi:
            b, h = divmod(lo, heads_kv)
            if h == 0 and hi - lo >= heads_kv:
                nb = (hi - lo) // heads_kv
                shards.append(Shard(b, nb, 0, heads_kv))
                lo += nb * heads_kv
            else:
                nh = min(heads_kv - h, hi - lo)
                shards.append(Shard(b, 1, h, nh))
                lo += nh
        out.append(shards)
    return out


def slice_tensors(shard: Shard, group: int, q_like: list, kv_like: list, row_like: list):
    """Views of BHSD tensors for one shard: q_like [B,Hq,S,D], kv_like [B,Hkv,S,D], row_like [B,Hq,S]."""
    bs = slice(shard.batch_begin, shard.batch_begin + shard.batch_count)
    qh0, qhn = shard.q_heads(group)
    qs = slice(qh0, qh0 + qhn)
    ks = slice(shard.kv_head_begin, shard.kv_head_begin + shard.kv_head_count)
    return ([t[bs, qs] for t in q_like], [t[bs, ks] for t in kv_like], [t[bs, qs] for t in row_like])


def max_over_ranks(value: float, dist=None, device=None) -> float:
    """Largest value over all ranks (the time of the slowest rank decides the job)."""
    if dist is None or not dist.is_initialized() or dist.get_world_size() == 1:
        return value
    import torch
    t = torch.tensor([value], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())
