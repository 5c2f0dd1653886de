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


class ShardedSession:
    """One process, several GPUs: a full replica of the graph on every device, each run on its own host thread
    with a contiguous slice of the batch, the results concatenated on the host.  This is the in-process
    counterpart of the one-rank-per-GPU launch: the library keeps its launch state per device, so contexts on
    different devices may plan and run concurrently.

    `build(device) -> Session` makes the replica for one device (the caller chooses graph, weights and tuning);
    every input is split along axis 0, every output concatenated along axis 0.
    """

    def __init__(self, build, devices):
        import threading
        self.devices = list(devices)
        if not self.devices:
            raise ValueError("no devices")
        self.sessions = [None] * len(self.devices)
        errors = [None] * len(self.devices)

        def make(i):
            try:
                self.sessions[i] = build(self.devices[i])
            except BaseException as e:  # re-raised on the calling thread
                errors[i] = e

        threads = [threading.Thread(target=make, args=(i,)) for i in range(len(self.devices))]
        for t in threads:
            t.start()
        for t in threads:
            t.join()
        for e in errors:
            if e is not None:
                self.close()
                raise e

    def run(self, feeds):
        """Splits every feed along its first axis over the replicas (shard_bounds), runs them concurrently and
        concatenates each output.  A replica whose slice is empty is skipped."""
        import threading
        import numpy as np
        world = len(self.sessions)
        totals = {int(np.asarray(v).shape[0]) for v in feeds.values()}
        if len(totals) != 1:
            raise ValueError(f"the feeds disagree on the batch: {sorted(totals)}")
        total = totals.pop()
        bounds = all_bounds(total, world)
        results, errors = [None] * world, [None] * world

        def work(i):
            b0, b1 = bounds[i]
            if b0 == b1:
                return
            try:
                results[i] = self.sessions[i].run({k: np.ascontiguousarray(np.asarray(v)[b0:b1]) for k, v in feeds.items()})
            except BaseException as e:
                errors[i] = e

        threads = [threading.Thread(target=work, args=(i,)) for i in range(world)]
        for t in threads:
            t.start()
        for t in threads:
            t.join()
        for e in errors:
            if e is not None:
                raise e
        parts = [r for r in results if r is not None]
        return {name: np.concatenate([p[name] for p in parts], axis=0) for name in parts[0]}

    def close(self):
        for s in self.sessions:
            if s is not None:
                s.close()
        self.sessions = []
