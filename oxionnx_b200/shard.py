"""Batch sharding across replicas.

The hot path shards only along the batch: every node's output row / image depends on the same
row / image of its inputs, so each GPU holds a full weight replica, runs a contiguous slice of
the batch and no data-path collective exists.  (The one per-tensor statistic on the path,
DynamicQuantizeLinear's min/max, is why the dynamic-INT8 encoder is replicated whole rather
than sharded.)  The only cross-rank traffic is the host-side gather of the results and the
timing reduction of the benchmark.
"""
from typing import List, Tuple


def shard_bounds(total: int, world: int, rank: int) -> Tuple[int, int]:
    """Contiguous [begin, end) slice of `total` items for `rank` of `world`; the first
    `total % world` ranks take one extra item."""
    if world < 1 or not (0 <= rank < world):
        raise ValueError("bad world/rank")
    base, extra = divmod(total, world)
    begin = rank * base + min(rank, extra)
    return begin, begin + base + (1 if rank < extra else 0)


def all_bounds(total: int, world: int) -> List[Tuple[int, int]]:
    return [shard_bounds(total, world, r) for r in range(world)]


def gather_rows(local, world: int, rank: int, group=None):
    """Concatenate per-rank result rows on every rank (host side, torch.distributed)."""
    import numpy as np
    import torch
    import torch.distributed as dist

    if world == 1:
        return local
    parts = [None] * world
    dist.all_gather_object(parts, np.asarray(local), group=group)
    return np.concatenate(parts, axis=0)


def max_over_ranks(value: float, world: int, device=None) -> float:
    """The benchmark's clock: the slowest rank's device time."""
    import torch
    import torch.distributed as dist

    if world == 1:
        return value
    t = torch.tensor([value], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())
