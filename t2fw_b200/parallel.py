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
