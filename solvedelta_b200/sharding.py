"""Multi-GPU layout of the operator: independent (batch, head) streams.

Every (batch, head) stream of the recurrence is independent in forward and in
backward (causallsso/reference.py:156-227 has no cross-stream term; every
upstream kernel indexes batch*heads on its last grid axis), so the path
shards over ranks without any data-path collective: each rank runs the
operator on its own slice of the batch, then of the heads when there are
fewer batch rows than ranks.  The only cross-rank traffic of the benchmark is
the reduction of the step time (max over ranks).
"""
from __future__ import annotations

from typing import List, Tuple


def stream_shard(batch: int, heads: int, rank: int, world: int) -> Tuple[slice, slice]:
    """Slices of the batch and head axes owned by `rank` (strong scaling).

    Batch rows are dealt out first; when world > batch the ranks that share a
    batch row split its heads.  Shards are disjoint and cover every stream.
    """
    if not (0 <= rank < world):
        raise ValueError("rank out of range")
    if world <= batch:
        lo = (batch * rank) // world
        hi = (batch * (rank + 1)) // world
        return slice(lo, hi), slice(0, heads)
    if world % batch:
        raise ValueError("world size must be a multiple of the batch when it exceeds it")
    per_row = world // batch
    if per_row > heads:
        raise ValueError("more ranks than (batch, head) streams")
    row, part = divmod(rank, per_row)
    lo = (heads * part) // per_row
    hi = (heads * (part + 1)) // per_row
    return slice(row, row + 1), slice(lo, hi)


def shard_streams(batch: int, heads: int, world: int) -> List[Tuple[slice, slice]]:
    return [stream_shard(batch, heads, r, world) for r in range(world)]


def rank_seed(base_seed: int, rank: int) -> int:
    """Weak scaling: every rank draws its own batch."""
    return base_seed + rank


def max_over_ranks(value: float, device=None) -> float:
    """Step time of the job = slowest rank (no-op without a process group)."""
    import torch
    import torch.distributed as dist

    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size() == 1:
        return float(value)
    t = torch.tensor([value], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def job_throughput(units_per_rank: int, seconds: float, world: int) -> float:
    """Whole-job units per second when every rank processes `units_per_rank`."""
    return world * units_per_rank / seconds
