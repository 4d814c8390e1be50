"""The time-axis split of the decay rule (t2fw_b200/seq_parallel.py) on CPU ranks: the exchange of
segment summaries and the folds are exercised with gloo, the segment work is done by the
step-by-step oracle (float64), and outputs, final state and every gradient are compared with the
oracle on the unsplit sequence."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from helpers import lfw_inputs


class OracleSegmentOps:
    """The three segment operations of seq_parallel on the CPU oracle (float64 tensors)."""

    def summary(self, val_d, gate_d, val_k, gate_k, backward):
        from oracle import fw_oracle

        B, T, D = val_d.shape
        K = val_k.shape[2]
        zs = np.zeros((B, D, K))
        if backward:    # state gradient at the start for a zero gradient at the end: needs only dO, f, q, f_key
            g = fw_oracle.lfw_backward(val_d, zs, np.zeros((B, T, D)), gate_d, val_k, np.zeros((B, T, K)), gate_k, zs)
            end = g[5]
        else:           # the state a zero state becomes: needs only x, f, k, f_key
            _, end = fw_oracle.lfw_forward(val_d, gate_d, np.zeros((B, T, K)), val_k, gate_k, zs)
        return (torch.from_numpy(np.asarray(end)), gate_d.prod(dim=1).double(), gate_k.prod(dim=1).double())

    def forward(self, x, f, q, k, fk, state):
        from oracle import fw_oracle

        out, fin = fw_oracle.lfw_forward(x, f, q, k, fk, state)
        return torch.from_numpy(out), torch.from_numpy(fin)[:, None]

    def backward(self, go, gs, x, f, q, k, fk, out, state, ckpt):
        from oracle import fw_oracle

        return [torch.from_numpy(np.asarray(g)) for g in fw_oracle.lfw_backward(go, gs, x, f, q, k, fk, state)]


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _bounds(T, world):
    # uneven on purpose: segments of different lengths
    cuts = [0] + [int(round(T * (r + 1) / world)) - (1 if r % 2 == 0 and r + 1 < world else 0) for r in range(world)]
    return list(zip(cuts[:-1], cuts[1:]))


def _worker(rank, world, port, result_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from t2fw_b200.seq_parallel import LFWSeqParallelFunction

        B, T, D, K = 3, 37, 6, 4
        x, f, q, k, fk, s, go, gs = [t.double() for t in lfw_inputs(B, T, D, K, "sigmoid", 0.5, 91)]
        lo, hi = _bounds(T, world)[rank]
        leaves = [t[:, lo:hi].clone().requires_grad_(True) for t in (x, f, q, k, fk)] + [s.clone().requires_grad_(True)]
        out, fin = LFWSeqParallelFunction.apply(*leaves, None, OracleSegmentOps())
        # every rank uses the final state in its "loss" with a third of the weight
        grads = torch.autograd.grad([out, fin], leaves, [go[:, lo:hi], gs / world])
        np.savez(os.path.join(result_dir, "r%d.npz" % rank), out=out.detach().numpy(), fin=fin.detach().numpy(),
                 **{"g%d" % i: g.numpy() for i, g in enumerate(grads)})
        dist.barrier()
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 3])
def test_time_split_matches_the_unsplit_sequence(tmp_path, world):
    from oracle import fw_oracle

    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    B, T, D, K = 3, 37, 6, 4
    x, f, q, k, fk, s, go, gs = [t.double() for t in lfw_inputs(B, T, D, K, "sigmoid", 0.5, 91)]
    r_out, r_fin = fw_oracle.lfw_forward(x, f, q, k, fk, s)
    r_grads = fw_oracle.lfw_backward(go, gs, x, f, q, k, fk, s)
    parts = [np.load(os.path.join(str(tmp_path), "r%d.npz" % r)) for r in range(world)]
    assert np.allclose(np.concatenate([p["out"] for p in parts], 1), r_out, rtol=1e-10, atol=1e-12)
    for p in parts:
        assert np.allclose(p["fin"], r_fin, rtol=1e-10, atol=1e-12)      # the same on every rank
    for i in range(5):      # sequence gradients: each rank holds its segment
        assert np.allclose(np.concatenate([p["g%d" % i] for p in parts], 1), r_grads[i], rtol=1e-9, atol=1e-11), i
    # the gradient of the replicated initial state is the sum over ranks (rank 0 holds it)
    assert np.allclose(sum(p["g5"] for p in parts), r_grads[5], rtol=1e-9, atol=1e-11)
    assert all(not p["g5"].any() for p in parts[1:])
