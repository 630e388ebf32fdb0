"""Replica sharding of the attention path over the GPUs of one node.

Every (batch row, kv head) slab of the operators is independent, so the path
shards over batch (then heads) with no exchange step: each rank runs the same
operator on its own shard.  The only cross-rank traffic is the reduction of
timings for reporting (maximum step time, summed work).
"""

from __future__ import annotations

import torch
import torch.distributed as dist


def shard_range(total: int, rank: int, world: int) -> tuple[int, int]:
    """[begin, end) of `total` units owned by `rank`; earlier ranks take the remainder."""
    if not 0 <= rank < world:
        raise ValueError("rank must be in [0, world)")
    base, extra = divmod(total, world)
    begin = rank * base + min(rank, extra)
    return begin, begin + base + (1 if rank < extra else 0)


def shard_batch_heads(batch: int, heads: int, rank: int, world: int, kv_heads: int | None = None):
    """Batch slice and head slice of a rank: batch first, heads only when there are more ranks than rows.

    With grouped query heads (``kv_heads`` given and smaller than ``heads``) the heads are cut between KV heads, so
    that a rank holds whole groups, and three slices come back: batch, query heads, KV heads.
    """
    kv = heads if kv_heads is None else kv_heads
    if kv < 1 or heads % kv:
        raise ValueError("heads must be a multiple of kv_heads")
    group = heads // kv
    if world <= batch:
        b0, b1 = shard_range(batch, rank, world)
        rows, q_part, kv_part = slice(b0, b1), slice(0, heads), slice(0, kv)
    else:
        per_row = -(-world // batch)  # ranks sharing one batch row
        if kv % per_row or batch * per_row != world:
            raise ValueError("world size must be batch * (a divisor of the KV heads) when it exceeds the batch")
        row, part = divmod(rank, per_row)
        h0, h1 = shard_range(kv, part, per_row)
        rows, q_part, kv_part = slice(row, row + 1), slice(h0 * group, h1 * group), slice(h0, h1)
    if kv_heads is None:
        return rows, q_part
    return rows, q_part, kv_part


def aggregate_throughput(local_ms: float, local_units: float, device: torch.device | None = None) -> tuple[float, float]:
    """(max step time over ranks in ms, summed units over ranks); a no-op without a process group."""
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size() == 1:
        return local_ms, local_units
    t = torch.tensor([local_ms], dtype=torch.float64, device=device)
    u = torch.tensor([local_units], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    dist.all_reduce(u, op=dist.ReduceOp.SUM)
    return t.item(), u.item()
