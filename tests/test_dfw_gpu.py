"""Parity of the CUDA delta-rule path with the oracle, through the C ABI and the autograd
wrapper.  The reference tests the delta rule in float32 only (tests/test_dfw.py:32-33)."""
import math

import pytest
import torch

from helpers import (GRAD_TOL, OUT_TOL, dfw_inputs, golden_files, load_golden, max_rel_err, to_dev)
from oracle import fw_oracle

pytestmark = pytest.mark.gpu

GRAD_NAMES = ("d_q", "d_k", "d_v", "d_state")


def run_cabi(q, k, v, s, go, gs):
    from t2fw_b200 import cabi

    out, fin, delta = cabi.dfw_forward(q, k, v, s)
    grads = cabi.dfw_backward(go, gs, q, k, delta, fin)
    torch.cuda.synchronize()
    return out, fin, grads


def check_against_oracle(dev_inputs, got, dtype, rows=None):
    q, k, v, s, go, gs = [t if rows is None else t[rows] for t in dev_inputs]
    out, fin, grads = got
    if rows is not None:
        out, fin, grads = out[rows], fin[rows], [g[rows] for g in grads]
    r_out, r_fin, _ = fw_oracle.dfw_forward(q, k, v, s)
    r_grads = fw_oracle.dfw_backward(go, gs, q, k, v, s)
    assert max_rel_err(out, r_out) <= OUT_TOL[dtype], "outputs"
    assert max_rel_err(fin, r_fin) <= OUT_TOL[dtype], "final_state"
    for g, r, n in zip(grads, r_grads, GRAD_NAMES):
        assert max_rel_err(g, r) <= GRAD_TOL[dtype], n


@pytest.mark.parametrize("path", golden_files("dfw_"), ids=lambda p: p.split("/")[-1][:-4])
def test_golden_fp32_direct(cuda, path):
    g = load_golden(path)
    names = ("q", "k", "v", "state", "grad_out", "grad_state")
    dev = to_dev([g[n] for n in names], torch.float32, cuda)
    out, fin, grads = run_cabi(*dev)
    assert max_rel_err(out, g["out"]) <= OUT_TOL[torch.float32]
    assert max_rel_err(fin, g["final_state"]) <= OUT_TOL[torch.float32]
    for got, n in zip(grads, GRAD_NAMES):
        assert max_rel_err(got, g[n]) <= GRAD_TOL[torch.float32], n


@pytest.mark.parametrize("dtype", [torch.float16, torch.float64])
@pytest.mark.parametrize("path", golden_files("dfw_"), ids=lambda p: p.split("/")[-1][:-4])
def test_golden_inputs_other_dtypes(cuda, path, dtype):
    g = load_golden(path)
    names = ("q", "k", "v", "state", "grad_out", "grad_state")
    dev = to_dev([g[n] for n in names], dtype, cuda)
    check_against_oracle(dev, run_cabi(*dev), dtype)


def reference_grid():
    # tests/test_dfw.py:20-26
    for bsz in range(1, 16, 4):
        for dim in range(1, 64, 32):
            for seqlen in range(1, 512, 128):
                yield bsz, seqlen, dim
    yield 2, 1024, 32
    yield 2, 1024, 96


@pytest.mark.parametrize("bsz,seqlen,dim", list(reference_grid()))
def test_reference_shape_grid_fp32(cuda, bsz, seqlen, dim):
    mdim = math.ceil(dim / 2)
    cpu = dfw_inputs(bsz, seqlen, dim, mdim, "softmax", 1.0, 200 + bsz + seqlen + dim)
    dev = to_dev(cpu, torch.float32, cuda)
    check_against_oracle(dev, run_cabi(*dev), torch.float32)


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16])
def test_config2_shape_full_size(cuda, dtype):
    """B*H=96, T=1024, D=M=64; three rows checked against the oracle."""
    cpu = dfw_inputs(96, 1024, 64, 64, "scaled", 0.0, 12)
    dev = to_dev(cpu, dtype, cuda)
    got = run_cabi(*dev)
    assert all(torch.isfinite(t).all() for t in (got[0], got[1], *got[2]))
    check_against_oracle(dev, got, dtype, rows=[0, 50, 95])


def test_autograd_wrapper(cuda):
    from t2fw_b200.functional_dfw import DFWFunction

    cpu = dfw_inputs(3, 130, 48, 24, "softmax", 1.0, 13)
    q, k, v, s, go, gs = to_dev(cpu, torch.float32, cuda)
    leaves = [t.clone().requires_grad_(True) for t in (q, k, v, s)]
    out, fin = DFWFunction.apply(*leaves)
    go_nc = go.transpose(0, 1).contiguous().transpose(0, 1)
    grads = torch.autograd.grad([out, fin], leaves, [go_nc, gs])
    check_against_oracle((q, k, v, s, go, gs), (out, fin, grads), torch.float32)
    out2, fin2 = DFWFunction.apply(*leaves)
    grads2 = torch.autograd.grad([out2, fin2], leaves, [go_nc, gs])
    assert torch.equal(out, out2) and torch.equal(fin, fin2)
    for a, b in zip(grads, grads2):
        assert torch.equal(a, b)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("B,T,keys,state_std", [
    (3, 1, "scaled", 0.5), (2, 37, "scaled", 0.3), (2, 64, "softmax", 1.0), (3, 129, "scaled", 0.1),
    (2, 200, "softmax", 0.5), (1, 1000, "scaled", 0.0), (2, 1024, "softmax", 0.2)])
def test_chunked_path_lengths(cuda, dtype, B, T, keys, state_std):
    """D = M = 64 in 16-bit storage runs on the chunked tensor-core kernels: whole and partial
    chunks, sequences shorter than a chunk, non-zero initial state, both key distributions."""
    cpu = dfw_inputs(B, T, 64, 64, keys, state_std, 20 + T)
    dev = to_dev(cpu, dtype, cuda)
    got = run_cabi(*dev)
    assert all(torch.isfinite(t).all() for t in (got[0], got[1], *got[2]))
    check_against_oracle(dev, got, dtype)


def test_scan_forward_pairs_with_chunked_backward(cuda):
    """The scratch-free forward (scan kernels) and the forward with scratch (chunked kernels) save
    the same delta, so either can feed the backward."""
    from t2fw_b200 import cabi

    cpu = dfw_inputs(2, 300, 64, 64, "scaled", 0.2, 31)
    dev = to_dev(cpu, torch.float16, cuda)
    q, k, v, s, go, gs = dev
    out_a, fin_a, delta_a = cabi.dfw_forward(q, k, v, s, use_scratch=False)
    out_b, fin_b, delta_b = cabi.dfw_forward(q, k, v, s)
    assert max_rel_err(out_b, out_a) <= 2e-3 and max_rel_err(fin_b, fin_a) <= 2e-3
    assert max_rel_err(delta_b, delta_a) <= 2e-3
    grads = cabi.dfw_backward(go, gs, q, k, delta_a, fin_a)
    torch.cuda.synchronize()
    check_against_oracle(dev, (out_a, fin_a, grads), torch.float16)
