"""World-size-2 check of the multi-GPU host logic on CPU (gloo): the batch rows shard with no
data-path collective, and the timing reduction takes the slowest rank."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from helpers import lfw_inputs
from t2fw_b200.parallel import job_throughput, max_over_ranks, row_shard


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, result_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from oracle import fw_oracle

        B = 5
        x, f, q, k, fk, s, go, gs = lfw_inputs(B, 20, 6, 4, "sigmoid", 0.5, 77)
        lo, hi = row_shard(B, world, rank)
        out, fin = fw_oracle.lfw_forward(x[lo:hi], f[lo:hi], q[lo:hi], k[lo:hi], fk[lo:hi], s[lo:hi])
        np.save(os.path.join(result_dir, "out_%d.npy" % rank), out)
        slowest = max_over_ranks(10.0 + rank)         # rank 1 is "slower"
        assert slowest == 10.0 + world - 1
        assert job_throughput(100, world, slowest) == pytest.approx(100 * world / (slowest * 1e-3))
        dist.barrier()
    finally:
        dist.destroy_process_group()


def test_row_shard_partitions():
    for n in (1, 2, 5, 16, 96, 97):
        for w in (1, 2, 3, 4, 8):
            spans = [row_shard(n, w, r) for r in range(w)]
            assert spans[0][0] == 0 and spans[-1][1] == n
            for a, b in zip(spans, spans[1:]):
                assert a[1] == b[0]
            sizes = [b - a for a, b in spans]
            assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        row_shard(4, 2, 2)


def test_two_ranks_shard_rows_without_exchange(tmp_path):
    from oracle import fw_oracle

    world = 2
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    x, f, q, k, fk, s, _, _ = lfw_inputs(5, 20, 6, 4, "sigmoid", 0.5, 77)
    full, _ = fw_oracle.lfw_forward(x, f, q, k, fk, s)
    parts = [np.load(os.path.join(str(tmp_path), "out_%d.npy" % r)) for r in range(world)]
    assert np.array_equal(np.concatenate(parts, 0), full)
