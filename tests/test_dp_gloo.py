"""Data-parallel host logic on CPU: request sharding and the cross-rank
reduction of measurements, with world_size 2 over gloo."""
import os
import socket

import pytest

torch = pytest.importorskip("torch")
import torch.distributed as dist
import torch.multiprocessing as mp

from dsv4_attn_b200 import dp


def test_shards_partition_the_batch():
    for n, world in ((1024, 8), (10, 3), (5, 8)):
        seen = []
        for r in range(world):
            seen += dp.shard_requests(n, world, r)
        assert sorted(seen) == list(range(n))
    cost = [((i * 7919) % 1000) + 1 for i in range(1024)]
    totals, seen = [], []
    for r in range(8):
        mine = dp.shard_requests(1024, 8, r, cost=cost, balance="sorted_round_robin")
        seen += mine
        totals.append(sum(cost[i] for i in mine))
    assert sorted(seen) == list(range(1024))
    assert max(totals) / min(totals) < 1.02           # serpentine dealing balances the cost
    with pytest.raises(ValueError):
        dp.shard_requests(4, 2, 2)


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        mine = dp.shard_requests(101, world, rank)
        units = float(len(mine) * 656)
        seconds = 1.0 + rank                       # rank 1 is the slow one
        agg = dp.aggregate_throughput(units, seconds)
        n_total = dp.reduce_scalar(len(mine), "sum")
        dist.barrier()
        out.put((rank, agg, n_total))
    finally:
        dist.destroy_process_group()


def test_aggregate_over_two_gloo_ranks():
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = sorted(q.get(timeout=120) for _ in range(world))
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for _, agg, n_total in res:
        assert n_total == 101
        assert agg == pytest.approx(101 * 656 / 2.0)   # all units over the slowest rank's time



def _head_worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        g = torch.Generator().manual_seed(5)
        q = torch.randn(3, 2, 8, 16, generator=g)                 # the same on every rank
        sink = torch.arange(8, dtype=torch.float32)

        def fake_decode(q_slice, sink_slice):                      # per-head work only, like attention
            o = q_slice[..., :4] * 2.0 + sink_slice.view(1, 1, -1, 1)
            return o, q_slice.sum(-1)

        o, l = dp.head_sharded_decode(fake_decode, q, sink)
        want_o = q[..., :4] * 2.0 + sink.view(1, 1, -1, 1)
        out.put((rank, bool(torch.equal(o, want_o)), bool(torch.equal(l, q.sum(-1))), tuple(o.shape)))
    finally:
        dist.destroy_process_group()


def test_head_sharded_variant_over_two_gloo_ranks():
    assert dp.head_shard(128, 8, 3) == (48, 64)
    with pytest.raises(ValueError):
        dp.head_shard(10, 4, 0)
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_head_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = [q.get(timeout=120) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, ok_o, ok_l, shape in res:
        assert ok_o and ok_l and shape == (3, 2, 8, 4)
