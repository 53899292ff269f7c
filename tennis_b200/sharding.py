"""Batch sharding across independent replicas (one process per GPU, no data-path collective).

Images are independent on this path, so N GPUs simply take N slices of the global batch.  The only
communication is bookkeeping: a barrier around the timed region and two reductions of scalars (the maximum of
the per-rank device time, the sum of the per-rank work) so that rank 0 can print the whole-job throughput.
"""
import torch
import torch.distributed as dist


def shard_range(global_batch, world, rank):
    """Contiguous slice [start, start + count) of the global batch owned by `rank`; sizes differ by at most one."""
    if world < 1 or not (0 <= rank < world) or global_batch < 0:
        raise ValueError("bad sharding request: batch %d world %d rank %d" % (global_batch, world, rank))
    base, extra = divmod(global_batch, world)
    count = base + (1 if rank < extra else 0)
    start = rank * base + min(rank, extra)
    return start, count


def shard_seed(rank, base_seed=1000):
    """Per-shard seed of the synthetic inputs: 1000 + rank (shard 0 draws from seed 1000, shard 1 from 1001, ...)."""
    if rank < 0:
        raise ValueError("negative rank")
    return base_seed + rank


def micro_batches(count, size):
    """Sizes of the micro-batches a shard of `count` images is processed in: full ones of `size`, then the remainder."""
    if count < 0 or size < 1:
        raise ValueError("bad micro-batch request")
    full, rest = divmod(count, size)
    return [size] * full + ([rest] if rest else [])


def aggregate(elapsed_ms, units, device=None):
    """(max over ranks of elapsed_ms, sum over ranks of units).  Works without a process group (single process)."""
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size() == 1:
        return float(elapsed_ms), float(units)
    t = torch.tensor([float(elapsed_ms)], dtype=torch.float64, device=device)
    u = torch.tensor([float(units)], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    dist.all_reduce(u, op=dist.ReduceOp.SUM)
    return float(t[0]), float(u[0])


def throughput(elapsed_ms, units, device=None):
    """Whole-job units per second: all ranks' units over the slowest rank's time."""
    t, u = aggregate(elapsed_ms, units, device)
    return u / (t / 1e3) if t > 0 else 0.0
