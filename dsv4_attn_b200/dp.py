"""Data-parallel plumbing for decode batches: one process per GPU, requests
partitioned across ranks, no collective on the attention path.  The only
communication is the timing barrier and the reduction of the per-rank
measurements (max of times, sum of bytes), over whichever torch.distributed
backend the process group uses (NCCL on GPUs, gloo in the CPU tests)."""
from __future__ import annotations

from typing import List, Optional, Sequence


def shard_requests(n_requests: int, world: int, rank: int, cost: Optional[Sequence[float]] = None,
                   balance: str = "contiguous") -> List[int]:
    """Indices of the requests rank `rank` of `world` owns.

    contiguous          : equal contiguous slices (the default for uniform batches).
    sorted_round_robin  : requests sorted by decreasing `cost` (e.g. context
                          length) and dealt out in a serpentine order, so that
                          every rank gets a similar total cost on ragged batches.
    Every request is owned by exactly one rank."""
    if not (0 <= rank < world):
        raise ValueError(f"rank {rank} outside world {world}")
    if balance == "contiguous" or cost is None:
        base, rem = divmod(n_requests, world)
        start = rank * base + min(rank, rem)
        return list(range(start, start + base + (1 if rank < rem else 0)))
    if balance != "sorted_round_robin":
        raise ValueError(f"unknown balance mode {balance!r}")
    if len(cost) != n_requests:
        raise ValueError("cost must have one value per request")
    order = sorted(range(n_requests), key=lambda i: (-float(cost[i]), i))
    mine = []
    for pos, idx in enumerate(order):
        rnd, slot = divmod(pos, world)
        owner = slot if rnd % 2 == 0 else world - 1 - slot
        if owner == rank:
            mine.append(idx)
    return mine


def reduce_scalar(value: float, op: str, device=None) -> float:
    """All-reduce one float over the default process group (identity when no
    group is initialised).  op: "max" or "sum"."""
    import torch
    import torch.distributed as dist
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size() == 1:
        return float(value)
    t = torch.tensor([value], dtype=torch.float64, device=device if device is not None else "cpu")
    dist.all_reduce(t, op=dist.ReduceOp.MAX if op == "max" else dist.ReduceOp.SUM)
    return float(t.item())


def aggregate_throughput(local_units: float, local_seconds: float, device=None) -> float:
    """Whole-job throughput: units processed by all ranks / slowest rank's time."""
    total = reduce_scalar(local_units, "sum", device)
    slowest = reduce_scalar(local_seconds, "max", device)
    return total / slowest if slowest > 0 else 0.0
