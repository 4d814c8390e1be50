"""The time-axis split on the GPU: the segment summary kernels against the oracle, the whole
split pipeline with the ranks emulated one after the other on one device, and (where two devices
are visible) two NCCL ranks."""
import os
import socket
import subprocess
import sys

import numpy as np
import pytest
import torch

from helpers import GRAD_TOL, OUT_TOL, lfw_inputs, max_rel_err, to_dev
from oracle import fw_oracle

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))


@pytest.mark.parametrize("T", [64, 200, 1000])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_segment_summary_matches_oracle(cuda, T, dtype):
    from t2fw_b200.seq_parallel import CudaSegmentOps

    ops = CudaSegmentOps()
    x, f, q, k, fk, s, go, gs = to_dev(lfw_inputs(3, T, 64, 64, "sigmoid", 0.5, 500 + T), dtype, cuda)
    zs = torch.zeros_like(s)
    L, A, G = ops.summary(x, f, k, fk, False)
    Gb, A2, G2 = ops.summary(go, f, q, fk, True)
    torch.cuda.synchronize()
    _, r_L = fw_oracle.lfw_forward(x, f, torch.zeros_like(q), k, fk, zs)
    r_Gb = fw_oracle.lfw_backward(go, zs, torch.zeros_like(x), f, q, torch.zeros_like(k), fk, zs)[5]
    assert max_rel_err(L, r_L) <= OUT_TOL[dtype]
    assert max_rel_err(Gb, r_Gb) <= GRAD_TOL[dtype]
    r_A, r_G = f.double().prod(dim=1), fk.double().prod(dim=1)
    for got, ref in ((A, r_A), (A2, r_A), (G, r_G), (G2, r_G)):
        assert got.dtype == torch.float32
        assert max_rel_err(got, ref) <= 1e-5


def test_flagged_row_poisons_its_summary(cuda):
    """A row whose gate products leave the supported range gets NaN decays (nothing downstream can
    silently use its summary); the other rows are untouched."""
    from t2fw_b200.seq_parallel import CudaSegmentOps

    x, f, q, k, fk, s, go, gs = lfw_inputs(3, 128, 64, 64, "sigmoid", 0.5, 7)
    fk[1, 10:60] = 1e3      # products beyond 2^100 inside one chunk
    x, f, q, k, fk = to_dev((x, f, q, k, fk), torch.float16, cuda)
    _, A, G = CudaSegmentOps().summary(x, f, k, fk, False)
    torch.cuda.synchronize()
    assert torch.isnan(A[1]).all() and torch.isnan(G[1]).all()
    assert torch.isfinite(A[0]).all() and torch.isfinite(G[2]).all()


@pytest.mark.parametrize("cuts", [(0, 256, 512), (0, 100, 300, 512), (0, 64, 128, 192, 512)])
def test_split_pipeline_with_emulated_ranks(cuda, cuts):
    """Summaries, folds and the ordinary kernels per segment, ranks run one after the other on one
    device (the collectives replaced by Python lists): equal to the oracle on the whole sequence."""
    from t2fw_b200.seq_parallel import CudaSegmentOps, fold_backward, fold_forward, pack_summary, unpack_summary

    ops = CudaSegmentOps()
    dt = torch.float16
    dev = to_dev(lfw_inputs(4, cuts[-1], 64, 64, "sigmoid", 0.5, 321), dt, cuda)
    x, f, q, k, fk, s, go, gs = dev
    spans = list(zip(cuts[:-1], cuts[1:]))
    seg = [[t[:, a:b].contiguous() for t in (x, f, q, k, fk, go)] for a, b in spans]
    summ = [pack_summary(*ops.summary(xs, fs, ks, fks, False)) for xs, fs, qs, ks, fks, gos in seg]
    outs, ckpts, s_ins = [], [], []
    for r, (xs, fs, qs, ks, fks, gos) in enumerate(seg):
        s_in = fold_forward(s, summ, r, 64, 64).to(dt).contiguous()
        o, c = ops.forward(xs, fs, qs, ks, fks, s_in)
        outs.append(o); ckpts.append(c); s_ins.append(s_in)
    final = fold_forward(s, summ, len(seg), 64, 64).to(dt)
    # the one-launch fold of the product path against the tensor-operation fold, every rank
    gathered = torch.stack(summ)
    for r in range(len(seg)):
        at_r, total = ops.fold(gathered, s.float().contiguous(), r, False)
        assert max_rel_err(at_r, fold_forward(s, summ, r, 64, 64)) <= 1e-6
        assert max_rel_err(total, fold_forward(s, summ, len(seg), 64, 64)) <= 1e-6
    bsum = []
    for r, (xs, fs, qs, ks, fks, gos) in enumerate(seg):
        Gb, _, _ = ops.summary(gos, fs, qs, fks, True)
        _, A, G = unpack_summary(summ[r], 64, 64)
        bsum.append(pack_summary(Gb, A, G))
    grads = []
    bgathered = torch.stack(bsum)
    for r, (xs, fs, qs, ks, fks, gos) in enumerate(seg):
        (r_end_k,) = ops.fold(bgathered, gs.float().contiguous(), r, True)
        assert max_rel_err(r_end_k, fold_backward(gs, bsum, r, 64, 64)) <= 1e-6
        r_end = fold_backward(gs, bsum, r, 64, 64).to(dt).contiguous()
        grads.append(ops.backward(gos, r_end, xs, fs, qs, ks, fks, outs[r], s_ins[r], ckpts[r]))
    torch.cuda.synchronize()
    r_out, r_fin = fw_oracle.lfw_forward(x, f, q, k, fk, s)
    r_grads = fw_oracle.lfw_backward(go, gs, x, f, q, k, fk, s)
    assert max_rel_err(torch.cat(outs, 1), r_out) <= OUT_TOL[dt]
    assert max_rel_err(final, r_fin) <= OUT_TOL[dt]
    for i in range(5):
        assert max_rel_err(torch.cat([g[i] for g in grads], 1), r_grads[i]) <= GRAD_TOL[dt], i
    assert max_rel_err(grads[0][5], r_grads[5]) <= GRAD_TOL[dt]


@pytest.mark.gpu
def test_single_rank_group_is_the_ordinary_call(cuda, tmp_path):
    """A group of one rank exchanges nothing: same results as LFWFunction, bit for bit."""
    import torch.distributed as dist

    from t2fw_b200.functional_lfw import LFWFunction
    from t2fw_b200.seq_parallel import LFWSeqParallelFunction

    dt = torch.float16
    x, f, q, k, fk, s, go, gs = to_dev(lfw_inputs(3, 200, 64, 64, "sigmoid", 0.5, 77), dt, cuda)
    dist.init_process_group("gloo", init_method="file://" + str(tmp_path / "store"), rank=0, world_size=1)
    try:
        la = [t.clone().requires_grad_(True) for t in (x, f, q, k, fk, s)]
        out_a, fin_a = LFWSeqParallelFunction.apply(*la)
        ga = torch.autograd.grad([out_a, fin_a], la, [go, gs])
    finally:
        dist.destroy_process_group()
    lb = [t.clone().requires_grad_(True) for t in (x, f, q, k, fk, s)]
    out_b, fin_b = LFWFunction.apply(*lb)
    gb = torch.autograd.grad([out_b, fin_b], lb, [go, gs])
    assert torch.equal(out_a, out_b) and torch.equal(fin_a, fin_b)
    for a, b in zip(ga, gb):
        assert torch.equal(a, b)


CHILD = r"""
import os, sys, numpy as np, torch, torch.distributed as dist
sys.path.insert(0, {tests!r}); sys.path.insert(0, {root!r})
from helpers import lfw_inputs
rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
torch.cuda.set_device(rank)
dev = torch.device("cuda", rank)
dist.init_process_group("nccl", device_id=dev)
from t2fw_b200.seq_parallel import LFWSeqParallelFunction
B, T = 4, 1024
full = [t.half() for t in lfw_inputs(B, T, 64, 64, "sigmoid", 0.5, 654)]
x, f, q, k, fk, s, go, gs = full
lo, hi = rank * T // world, (rank + 1) * T // world
leaves = [t[:, lo:hi].contiguous().to(dev).requires_grad_(True) for t in (x, f, q, k, fk)] + [s.to(dev).requires_grad_(True)]
out, fin = LFWSeqParallelFunction.apply(*leaves)
grads = torch.autograd.grad([out, fin], leaves, [go[:, lo:hi].contiguous().to(dev), (gs / world).to(dev)])
torch.cuda.synchronize()
np.savez(os.path.join({out!r}, "r%d.npz" % rank), out=out.detach().float().cpu().numpy(), fin=fin.detach().float().cpu().numpy(),
         **{{"g%d" % i: g.float().cpu().numpy() for i, g in enumerate(grads)}})
dist.barrier()
dist.destroy_process_group()
"""


def test_two_nccl_ranks(tmp_path):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    with socket.socket() as sk:
        sk.bind(("127.0.0.1", 0))
        port = sk.getsockname()[1]
    code = CHILD.format(tests=HERE, root=os.path.dirname(HERE), out=str(tmp_path))
    procs = []
    for r in range(2):
        env = dict(os.environ, RANK=str(r), WORLD_SIZE="2", LOCAL_RANK=str(r), MASTER_ADDR="127.0.0.1",
                   MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
        procs.append(subprocess.Popen([sys.executable, "-c", code], env=env, stdout=subprocess.PIPE,
                                      stderr=subprocess.STDOUT, text=True))
    for p in procs:
        out, _ = p.communicate(timeout=600)
        assert p.returncode == 0, out[-4000:]
    full = [t.half() for t in lfw_inputs(4, 1024, 64, 64, "sigmoid", 0.5, 654)]
    x, f, q, k, fk, s, go, gs = full
    r_out, r_fin = fw_oracle.lfw_forward(x, f, q, k, fk, s)
    r_grads = fw_oracle.lfw_backward(go, gs, x, f, q, k, fk, s)
    parts = [np.load(os.path.join(str(tmp_path), "r%d.npz" % r)) for r in range(2)]
    dt = torch.float16
    assert max_rel_err(np.concatenate([p["out"] for p in parts], 1), r_out) <= OUT_TOL[dt]
    for p in parts:
        assert max_rel_err(p["fin"], r_fin) <= OUT_TOL[dt]
    for i in range(5):
        assert max_rel_err(np.concatenate([p["g%d" % i] for p in parts], 1), r_grads[i]) <= GRAD_TOL[dt], i
    assert max_rel_err(parts[0]["g5"], r_grads[5]) <= GRAD_TOL[dt]
    assert not parts[1]["g5"].any()
