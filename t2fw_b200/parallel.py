"""Host-side helpers for running the recurrences on several GPUs of one node.

Every batch row (batch x head) is an independent recurrence, so the rows are split into
contiguous shards, one process per GPU, and nothing is exchanged on the data path.  The only
communication is for measurement: a barrier and a max-reduction of the per-rank device time.
"""
import torch
import torch.distributed as dist


def row_shard(n_rows, world_size, rank):
    """Contiguous [start, stop) slice of `n_rows` for `rank`; sizes differ by at most one."""
    if not (0 <= rank < world_size):
        raise ValueError("rank %d outside world of %d" % (rank, world_size))
    base, extra = divmod(n_rows, world_size)
    start = rank * base + min(rank, extra)
    return start, start + base + (1 if rank < extra else 0)


def max_over_ranks(value, device=None):
    """Maximum of a Python float over all ranks (identity without a process group)."""
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size() == 1:
        return float(value)
    t = torch.tensor([float(value)], dtype=torch.float64, device=device or "cpu")
    if t.is_cuda:
        t = t.float()
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def job_throughput(units_per_rank, world_size, elapsed_ms_max):
    """Whole-job units per second when every rank processed `units_per_rank` in the slowest
    rank's `elapsed_ms_max` milliseconds."""
    return units_per_rank * world_size / (elapsed_ms_max * 1e-3)


def _parse_cpulist(text):
    """'0-3,8,10-11' -> {0, 1, 2, 3, 8, 10, 11}"""
    cpus = set()
    for part in text.strip().split(","):
        if not part:
            continue
        lo, _, hi = part.partition("-")
        cpus.update(range(int(lo), int(hi or lo) + 1))
    return cpus


def bind_host_to_gpu_node(device_index, sysfs_root="/sys", allowed=None, apply=True):
    """Restrict this process to the CPUs of the NUMA node its GPU hangs off, so that pinned host
    buffers allocated afterwards (first touch) and the copy threads are local to the GPU's PCIe
    root.  With several ranks on one box each rank then uses its own socket's memory instead of
    all of them pinning from one node.  Does nothing (and says why) when the topology cannot be
    read or the node's CPUs are outside the process's allowed set.  Returns a small dict for logs.

    `allowed` (a set of CPU numbers) and `apply=False` exist for tests; `sysfs_root` likewise."""
    import os

    info = {"bound": False}
    try:
        props = torch.cuda.get_device_properties(device_index)
        bus_id = "%04x:%02x:%02x.0" % (props.pci_domain_id, props.pci_bus_id, props.pci_device_id)
    except Exception as e:      # no CUDA device / fields missing
        info["reason"] = "no PCI id for device %s (%s)" % (device_index, type(e).__name__)
        return info
    return _bind_to_pci_node(bus_id, sysfs_root, allowed, apply, info)


def _bind_to_pci_node(bus_id, sysfs_root, allowed, apply, info):
    import os

    info["pci"] = bus_id
    try:
        with open(os.path.join(sysfs_root, "bus/pci/devices", bus_id, "numa_node")) as fh:
            node = int(fh.read().strip())
        if node < 0:
            info["reason"] = "the platform reports no NUMA node for the device"
            return info
        with open(os.path.join(sysfs_root, "devices/system/node/node%d/cpulist" % node)) as fh:
            node_cpus = _parse_cpulist(fh.read())
    except (OSError, ValueError) as e:
        info["reason"] = "topology not readable (%s)" % type(e).__name__
        return info
    info["numa_node"] = node
    if allowed is None:
        allowed = os.sched_getaffinity(0) if hasattr(os, "sched_getaffinity") else set()
    cpus = node_cpus & set(allowed)
    if not cpus:
        info["reason"] = "none of node %d's CPUs is available to this process" % node
        return info
    if apply:
        try:
            os.sched_setaffinity(0, cpus)
        except OSError as e:
            info["reason"] = "sched_setaffinity refused (%s)" % e
            return info
    info["bound"] = True
    info["cpus"] = len(cpus)
    return info
