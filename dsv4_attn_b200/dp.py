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


# ── optional head-sharded variant ──────────────────────────────────────
# Every rank holds the whole batch's KV cache and computes a slice of the heads for all
# requests; one all-gather over the head dimension puts the outputs together.  It multiplies the
# KV bytes read by the number of ranks (each rank streams every entry) and is measured only for
# comparison with the request-sharded default, which needs no collective at all.

def head_shard(n_heads: int, world: int, rank: int):
    """[h0, h1): the heads rank `rank` of `world` computes; n_heads must divide evenly."""
    if not (0 <= rank < world):
        raise ValueError(f"rank {rank} outside world {world}")
    if n_heads % world != 0:
        raise ValueError(f"{n_heads} heads do not divide over {world} ranks")
    per = n_heads // world
    return rank * per, (rank + 1) * per


def head_sharded_decode(decode_fn, q, attn_sink=None, group=None):
    """q [B, s_q, H, D] on every rank (same values).  Calls decode_fn(q_slice, sink_slice) ->
    (out [B, s_q, H/world, Dv], lse [B, s_q, H/world]) for this rank's heads and all-gathers both
    along the head dimension (one collective each, NCCL over NVLink on GPUs).  Returns the full
    (out [B, s_q, H, Dv], lse [B, s_q, H]) on every rank."""
    import torch
    import torch.distributed as dist
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    rank = dist.get_rank(group) if dist.is_initialized() else 0
    H = q.shape[2]
    h0, h1 = head_shard(H, world, rank)
    out_l, lse_l = decode_fn(q[:, :, h0:h1].contiguous(), None if attn_sink is None else attn_sink[h0:h1].contiguous())
    if world == 1:
        return out_l, lse_l
    B, s_q, Hl, Dv = out_l.shape
    # gathered as a concatenation along the first dimension (the form every backend takes), then viewed per rank
    out_g = torch.empty((world * B, s_q, Hl, Dv), dtype=out_l.dtype, device=out_l.device)
    lse_g = torch.empty((world * B, s_q, Hl), dtype=lse_l.dtype, device=lse_l.device)
    dist.all_gather_into_tensor(out_g, out_l.contiguous(), group=group)
    dist.all_gather_into_tensor(lse_g, lse_l.contiguous(), group=group)
    out = out_g.view(world, B, s_q, Hl, Dv).permute(1, 2, 0, 3, 4).reshape(B, s_q, H, Dv)
    lse = lse_g.view(world, B, s_q, Hl).permute(1, 2, 0, 3).reshape(B, s_q, H)
    return out, lse
