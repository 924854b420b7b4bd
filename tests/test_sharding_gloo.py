"""The N>1 host path on CPU: two ``gloo`` ranks run the sharding helpers bench.py uses."""

from __future__ import annotations

import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from flashloop_b200 import sharding


def test_sequence_shard_partitions():
    for total in (0, 1, 7, 8, 64, 65):
        for world in (1, 2, 3, 8):
            spans = [sharding.sequence_shard(total, world, r) for r in range(world)]
            assert sum(c for _, c in spans) == total
            cursor = 0
            for first, count in spans:
                assert first == cursor
                cursor += count
            counts = [c for _, c in spans]
            assert max(counts) - min(counts) <= 1
    with pytest.raises(ValueError):
        sharding.sequence_shard(4, 2, 2)
    seeds = {sharding.sequence_seed(r, l, b) for r in range(8) for l in range(24) for b in range(8)}
    assert len(seeds) == 8 * 24 * 8


def test_single_process_is_identity():
    cpu = torch.device("cpu")
    sharding.barrier(cpu)
    assert sharding.max_over_ranks(3.5, cpu) == 3.5
    assert sharding.job_throughput(10.0, 500.0, cpu) == (20.0, 500.0)


def _worker(rank: int, world: int, port: int, results) -> None:
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        cpu = torch.device("cpu")
        first, count = sharding.sequence_shard(9, world, rank)
        sharding.barrier(cpu)
        local_ms = 10.0 * (rank + 1)           # rank 1 is the slow one
        rate, ms = sharding.job_throughput(float(count), local_ms, cpu)
        owned = torch.zeros(9, dtype=torch.int64)
        owned[first:first + count] = 1
        dist.all_reduce(owned)
        results[rank] = (first, count, rate, ms, owned.tolist())
    finally:
        dist.destroy_process_group()


def test_two_gloo_ranks():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    results = ctx.Manager().dict()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, results)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    assert results[0][:2] == (0, 5) and results[1][:2] == (5, 4)
    for r in range(2):
        _, _, rate, ms, owned = results[r]
        assert ms == 20.0                       # max over ranks
        assert rate == pytest.approx(9 / 0.020)  # all ranks' units over the slowest rank's time
        assert owned == [1] * 9                 # every sequence owned exactly once
