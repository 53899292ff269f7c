"""The multi-replica bookkeeping on CPU: world_size 2 over gloo (what runs over NCCL with one process per GPU)."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from tennis_b200 import sharding


def test_shard_ranges_partition_the_batch():
    for batch in (0, 1, 7, 64, 2048, 2049):
        for world in (1, 2, 3, 4, 8):
            seen = []
            for rank in range(world):
                start, count = sharding.shard_range(batch, world, rank)
                seen.extend(range(start, start + count))
            assert seen == list(range(batch))
            sizes = [sharding.shard_range(batch, world, r)[1] for r in range(world)]
            assert max(sizes) - min(sizes) <= 1
    assert sharding.shard_range(2048, 8, 3) == (768, 256)
    with pytest.raises(ValueError):
        sharding.shard_range(8, 2, 2)
    assert [sharding.shard_seed(r) for r in range(8)] == list(range(1000, 1008))
    # global batch 2048 in micro-batches of 64: 32 / 16 / 8 / 4 per replica at 1 / 2 / 4 / 8 replicas
    for world, per in ((1, 32), (2, 16), (4, 8), (8, 4)):
        assert sharding.micro_batches(sharding.shard_range(2048, world, world - 1)[1], 64) == [64] * per
    assert sharding.micro_batches(130, 64) == [64, 64, 2] and sharding.micro_batches(0, 64) == []


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        start, count = sharding.shard_range(65, world, rank)
        # rank 1 is the slow one; every rank processed `count` images
        elapsed_ms = 10.0 if rank == 0 else 25.0
        t, u = sharding.aggregate(elapsed_ms, count)
        tp = sharding.throughput(elapsed_ms, count)
        rates = sharding.gather_values([50.0 + rank, 40.0 - rank])      # per-rank copy rates, as bench.py reports them
        dist.barrier()
        out.put((rank, start, count, t, u, tp, rates))
    finally:
        dist.destroy_process_group()


def test_two_replicas_aggregate_over_gloo():
    world = 2
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, out)) for r in range(world)]
    for p in procs:
        p.start()
    results = sorted(out.get(timeout=120) for _ in range(world))
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert [(r[1], r[2]) for r in results] == [(0, 33), (33, 32)]
    for r in results:
        assert r[3] == 25.0 and r[4] == 65.0            # max of the times, sum of the work, on every rank
        assert abs(r[5] - 65.0 / 0.025) < 1e-9
        assert r[6] == [[50.0, 40.0], [51.0, 39.0]]      # every rank sees every rank's values, in rank order


def test_single_process_needs_no_group():
    assert sharding.aggregate(5.0, 3) == (5.0, 3.0)
    assert sharding.throughput(500.0, 100) == 200.0
