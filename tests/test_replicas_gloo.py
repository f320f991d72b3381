"""The N > 1 host logic on CPU: two gloo ranks shard requests, run their share independently and agree on
the max-over-ranks time (the data path itself needs no collective)."""
from __future__ import annotations

import os

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from spikeinfer_b200.engine.replicas import aggregate_throughput, max_over_ranks, shard_requests


def test_shard_requests_partitions_exactly():
    for n, world in ((64, 1), (64, 2), (64, 8), (10, 4), (3, 8), (0, 2)):
        parts = [shard_requests(n, world, r) for r in range(world)]
        assert sorted(i for p in parts for i in p) == list(range(n))
        assert max(len(p) for p in parts) - min(len(p) for p in parts) <= 1


def _worker(rank: int, world: int, port: int, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    mine = shard_requests(128, world, rank)
    seconds = 1.0 + rank  # rank 1 is the slow one
    slow = max_over_ranks([seconds, float(len(mine))])
    tput = aggregate_throughput(len(mine), seconds)
    out.put((rank, list(mine)[:2], slow, tput))
    dist.barrier()
    dist.destroy_process_group()


def test_two_gloo_ranks_agree_on_the_slowest_time():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29500 + os.getpid() % 1000
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    results = sorted(q.get(timeout=120) for _ in procs)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert results[0][1] == [0, 1] and results[1][1] == [64, 65]
    for _, _, slow, tput in results:
        assert slow == [2.0, 64.0]
        assert tput == 64 * 2 / 2.0


def test_single_process_is_the_identity():
    assert max_over_ranks([3.0, 1.0]) == [3.0, 1.0]
    assert aggregate_throughput(64, 2.0) == 32.0
