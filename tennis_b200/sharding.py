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


def gather_values(values, device=None):
    """Every rank's list of floats, as a list of lists on every rank (rank order).  Single process: [values]."""
    values = [float(v) for v in values]
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size() == 1:
        return [values]
    mine = torch.tensor(values, dtype=torch.float64, device=device)
    out = [torch.empty_like(mine) for _ in range(dist.get_world_size())]
    dist.all_gather(out, mine)
    return [[float(v) for v in t.tolist()] for t in out]


def parse_cpu_list(text):
    """"0-3,8,10-11" -> [0, 1, 2, 3, 8, 10, 11] (the format of sysfs cpulist files)."""
    cpus = []
    for part in text.strip().split(","):
        part = part.strip()
        if not part:
            continue
        lo, _, hi = part.partition("-")
        cpus.extend(range(int(lo), int(hi or lo) + 1))
    return cpus


def gpu_locality(pci_bus_id, sysfs="/sys/bus/pci/devices"):
    """NUMA node and local CPUs of the PCI device "dddd:bb:dd.f", read from sysfs (no setting is changed).  numa_node is
    -1 and cpus empty where the platform does not say (virtual machines usually)."""
    import os
    base = os.path.join(sysfs, pci_bus_id.lower())
    node, cpus = -1, []
    try:
        node = int(open(os.path.join(base, "numa_node")).read().strip())
    except (OSError, ValueError):
        pass
    try:
        cpus = parse_cpu_list(open(os.path.join(base, "local_cpulist")).read())
    except (OSError, ValueError):
        pass
    return node, cpus


def bind_to_gpu(pci_bus_id, sysfs="/sys/bus/pci/devices", setaffinity=None, getaffinity=None):
    """Pin this process to the CPUs next to its GPU, so that the pinned host buffers it allocates afterwards (first
    touch) and the threads that feed the GPU sit on the GPU's NUMA node.  Only the process's own affinity mask changes.
    Returns a record of what was found and done; binds nothing when the platform gives no locality or none of the local
    CPUs is available to the process."""
    import os
    setaffinity = setaffinity or os.sched_setaffinity
    getaffinity = getaffinity or os.sched_getaffinity
    node, local = gpu_locality(pci_bus_id, sysfs)
    allowed = sorted(getaffinity(0))
    usable = [c for c in local if c in set(allowed)]
    record = {"pci_bus_id": pci_bus_id, "numa_node": node, "local_cpus": len(local), "allowed_cpus": len(allowed), "bound_cpus": 0}
    if usable and len(usable) < len(allowed):
        try:
            setaffinity(0, usable)
            record["bound_cpus"] = len(usable)
        except OSError as e:
            record["error"] = repr(e)[:100]
    return record
