"""Parity of the CUDA decay-rule path with the oracle, through the C ABI and through the
autograd wrapper.  Tolerances (max relative error, see helpers.max_rel_err): fp16 outputs and
states 1e-2, fp16 gradients 2e-2; fp32 2e-4 / 5e-4; fp64 1e-9."""
import math
import os

import numpy as np
import pytest
import torch

from helpers import (GRAD_TOL, OUT_TOL, golden_files, lfw_inputs, load_golden, max_rel_err, to_dev)
from oracle import fw_oracle

pytestmark = pytest.mark.gpu

GRAD_NAMES = ("d_x", "d_f", "d_q", "d_k", "d_f_key", "d_state")


def run_cabi(x, f, q, k, fk, s, go, gs, ckpt_every=None):
    from t2fw_b200 import cabi

    out = torch.full_like(x, float("nan"))
    out, ckpt = cabi.lfw_forward(x, f, q, k, fk, s, ckpt_every=ckpt_every, out=out)
    grads = cabi.lfw_backward(go, gs, x, f, q, k, fk, s, ckpt, ckpt_every=ckpt_every)
    torch.cuda.synchronize()
    return out, ckpt[:, -1], grads


def check_against_oracle(dev_inputs, got, dtype, rows=None):
    """dev_inputs are the (already rounded) device tensors; the oracle sees the same values."""
    x, f, q, k, fk, s, go, gs = [t if rows is None else t[rows] for t in dev_inputs]
    out, fin, grads = got
    if rows is not None:
        out, fin, grads = out[rows], fin[rows], [g[rows] for g in grads]
    r_out, r_fin = fw_oracle.lfw_forward(x, f, q, k, fk, s)
    r_grads = fw_oracle.lfw_backward(go, gs, x, f, q, k, fk, s)
    assert max_rel_err(out, r_out) <= OUT_TOL[dtype], "outputs"
    assert max_rel_err(fin, r_fin) <= OUT_TOL[dtype], "next_state"
    for g, r, n in zip(grads, r_grads, GRAD_NAMES):
        assert max_rel_err(g, r) <= GRAD_TOL[dtype], n


@pytest.mark.parametrize("path", golden_files("lfw_"), ids=lambda p: p.split("/")[-1][:-4])
def test_golden_fp32_direct(cuda, path):
    """fp32 kernels against the reference's own fp32 results (no oracle in between)."""
    g = load_golden(path)
    names = ("x", "f", "q", "k", "f_key", "state", "grad_out", "grad_state")
    dev = to_dev([g[n] for n in names], torch.float32, cuda)
    out, fin, grads = run_cabi(*dev)
    assert max_rel_err(out, g["out"]) <= OUT_TOL[torch.float32]
    assert max_rel_err(fin, g["final_state"]) <= OUT_TOL[torch.float32]
    for got, n in zip(grads, GRAD_NAMES):
        assert max_rel_err(got, g[n]) <= GRAD_TOL[torch.float32], n


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16, torch.float64])
@pytest.mark.parametrize("path", golden_files("lfw_"), ids=lambda p: p.split("/")[-1][:-4])
def test_golden_inputs_other_dtypes(cuda, path, dtype):
    g = load_golden(path)
    names = ("x", "f", "q", "k", "f_key", "state", "grad_out", "grad_state")
    dev = to_dev([g[n] for n in names], dtype, cuda)
    check_against_oracle(dev, run_cabi(*dev), dtype)


def reference_grid():
    # the reference's shape grid (tests/test_lfw.py:19-24): kdim = ceil(dim / 2)
    for bsz in range(1, 16, 4):
        for dim in range(1, 64, 32):
            for seqlen in range(1, 512, 128):
                yield bsz, seqlen, dim
    yield 2, 1024, 32


@pytest.mark.parametrize("bsz,seqlen,dim", list(reference_grid()))
def test_reference_shape_grid_fp16(cuda, bsz, seqlen, dim):
    kdim = math.ceil(dim / 2)
    # gates as in tests/test_lfw.py:38,41; state ~ N(0,1) as in tests/test_lfw.py:42
    cpu = lfw_inputs(bsz, seqlen, dim, kdim, "bias", 1.0, 100 + bsz + seqlen + dim)
    dev = to_dev(cpu, torch.float16, cuda)
    check_against_oracle(dev, run_cabi(*dev), torch.float16)


@pytest.mark.parametrize("ckpt_every", [1, 7, 16, 64, 100, 4096])
def test_checkpoint_interval_does_not_change_results(cuda, ckpt_every):
    cpu = lfw_inputs(3, 150, 24, 40, "sigmoid", 0.5, 21)
    dev = to_dev(cpu, torch.float32, cuda)
    check_against_oracle(dev, run_cabi(*dev, ckpt_every=ckpt_every), torch.float32)


@pytest.mark.parametrize("gates", ["raw_f1", "raw", "sigmoid"])
def test_config2_full_size_fp16(cuda, gates):
    """B*H=96, T=1024, D=K=64 at full size: every batch row against the oracle."""
    cpu = lfw_inputs(96, 1024, 64, 64, gates, 0.0, 2)
    dev = to_dev(cpu, torch.float16, cuda)
    got = run_cabi(*dev)
    assert all(torch.isfinite(t).all() for t in (got[0], got[1], *got[2]))
    check_against_oracle(dev, got, torch.float16)


def test_config2_split_sequence_matches_single_call(cuda):
    """Feeding next_state back in (two calls of T/2) reproduces the single call."""
    from t2fw_b200 import cabi

    x, f, q, k, fk, s, _, _ = to_dev(lfw_inputs(96, 1024, 64, 64, "sigmoid", 0.1, 3), torch.float16, cuda)
    out, ckpt = cabi.lfw_forward(x, f, q, k, fk, s)
    h = 512
    o1, c1 = cabi.lfw_forward(*[t[:, :h].contiguous() for t in (x, f, q, k, fk)], s)
    o2, c2 = cabi.lfw_forward(*[t[:, h:].contiguous() for t in (x, f, q, k, fk)], c1[:, -1].contiguous())
    assert max_rel_err(torch.cat([o1, o2], 1), out) <= OUT_TOL[torch.float16]
    assert max_rel_err(c2[:, -1], ckpt[:, -1]) <= OUT_TOL[torch.float16]


def test_config3_decode_steps_fp16(cuda):
    """B*H=4096, T=1, D=K=64: five chained steps, every element checked."""
    from t2fw_b200 import cabi

    torch.manual_seed(5)
    B, D, K = 4096, 64, 64
    s = (torch.randn(B, D, K) * 0.1).half().to(cuda)
    s_ref = s.double().cpu().numpy()
    for step in range(5):
        x, q, k, fk = (torch.randn(B, 1, n).half().to(cuda) for n in (D, K, K, K))
        f = torch.sigmoid(torch.randn(B, 1, D)).half().to(cuda)
        out, ckpt = cabi.lfw_forward(x, f, q, k, fk, s)
        r_out, r_fin = fw_oracle.lfw_forward(x, f, q, k, fk, s_ref)
        assert max_rel_err(out, r_out) <= OUT_TOL[torch.float16]
        assert max_rel_err(ckpt[:, -1], r_fin) <= OUT_TOL[torch.float16]
        s = ckpt[:, -1].contiguous()
        s_ref = s.double().cpu().numpy()  # the API round-trips the state through fp16


def test_config4_long_sequence_fp16(cuda):
    """B*H=16, T=16384, D=K=128 (more than 2^31 state-steps); four heads against the oracle."""
    cpu = lfw_inputs(16, 16384, 128, 128, "sigmoid", 0.1, 4)
    dev = to_dev(cpu, torch.float16, cuda)
    got = run_cabi(*dev)
    assert all(torch.isfinite(t).all() for t in (got[0], got[1], *got[2]))
    check_against_oracle(dev, got, torch.float16, rows=[0, 5, 10, 15])


def test_autograd_wrapper_matches_oracle_and_is_deterministic(cuda):
    from t2fw_b200.functional_lfw import LFWFunction

    cpu = lfw_inputs(4, 200, 64, 64, "sigmoid", 0.3, 6)
    x, f, q, k, fk, s, go, gs = to_dev(cpu, torch.float16, cuda)
    leaves = [t.clone().requires_grad_(True) for t in (x, f, q, k, fk, s)]
    out, nxt = LFWFunction.apply(*leaves)
    assert out.shape == x.shape and nxt.shape == s.shape and nxt.dtype == s.dtype
    # non-contiguous upstream gradient, as autograd may hand over
    go_nc = go.transpose(0, 1).contiguous().transpose(0, 1)
    assert not go_nc.is_contiguous()
    grads = torch.autograd.grad([out, nxt], leaves, [go_nc, gs])
    check_against_oracle((x, f, q, k, fk, s, go, gs), (out, nxt, grads), torch.float16)
    # inputs untouched, second run bitwise identical
    for a, b in zip(leaves, (x, f, q, k, fk, s)):
        assert torch.equal(a.detach(), b)
    out2, nxt2 = LFWFunction.apply(*leaves)
    grads2 = torch.autograd.grad([out2, nxt2], leaves, [go_nc, gs])
    assert torch.equal(out, out2) and torch.equal(nxt, nxt2)
    for a, b in zip(grads, grads2):
        assert torch.equal(a, b)


def test_next_state_feeds_the_next_call(cuda):
    """The returned state has the input dtype and can be passed straight back in."""
    from t2fw_b200.functional_lfw import LFWFunction

    x, f, q, k, fk, s, _, _ = to_dev(lfw_inputs(2, 40, 16, 8, "sigmoid", 0.2, 8), torch.float16, cuda)
    _, s1 = LFWFunction.apply(x, f, q, k, fk, s)
    o2, _ = LFWFunction.apply(x, f, q, k, fk, s1)
    r1, f1 = fw_oracle.lfw_forward(x, f, q, k, fk, s)
    r2, _ = fw_oracle.lfw_forward(x, f, q, k, fk, s1)
    assert max_rel_err(s1, f1) <= OUT_TOL[torch.float16]
    assert max_rel_err(o2, r2) <= OUT_TOL[torch.float16]


def test_second_device_stream_is_respected(cuda):
    """The op runs on the caller's current stream."""
    from t2fw_b200.functional_lfw import LFWFunction

    x, f, q, k, fk, s, _, _ = to_dev(lfw_inputs(2, 64, 32, 32, "sigmoid", 0.2, 9), torch.float16, cuda)
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        o, _ = LFWFunction.apply(x, f, q, k, fk, s)
    side.synchronize()
    r, _ = fw_oracle.lfw_forward(x, f, q, k, fk, s)
    assert max_rel_err(o, r) <= OUT_TOL[torch.float16]


@pytest.mark.parametrize("kind", ["tiny_constant", "exact_zeros", "large"])
def test_extreme_gates_d64(cuda, kind):
    """D=K=64 inputs whose gate products leave the range of the factored tensor-core form: the
    affected batch rows must still come out right (they are redone by the scan kernels)."""
    x, f, q, k, fk, s, go, gs = lfw_inputs(3, 200, 64, 64, "sigmoid", 0.5, 40)
    if kind == "tiny_constant":
        fk[1] = 1e-3          # (1e-3)^32 leaves the range of the anchored products
        f[2] = 2e-3
    elif kind == "exact_zeros":
        fk[0, 17, 5] = 0.0
        fk[0, 18, 5] = 0.0
        fk[0, 19, 5] = 0.0
        fk[0, 20, 5] = 0.0
        f[1, 100, :] = 0.0    # a hard reset of the whole state
    else:
        fk[2, 64:80] = 100.0  # one-sided products overflow the safe range ...
        f[2, 64:80] = 0.01    # ... while the state itself stays bounded
    dev = to_dev((x, f, q, k, fk, s, go, gs), torch.float16, cuda)
    check_against_oracle(dev, run_cabi(*dev), torch.float16)


@pytest.mark.parametrize("T", [1, 2, 15, 16, 17, 31, 32, 33, 63, 64, 65, 127, 128, 130])
def test_d64_sequence_lengths(cuda, T):
    """Chunk (64), anchor (32) and quarter (16) boundaries of the tensor-core path, including
    ragged tails."""
    dev = to_dev(lfw_inputs(2, T, 64, 64, "sigmoid", 0.5, 50 + T), torch.float16, cuda)
    check_against_oracle(dev, run_cabi(*dev), torch.float16)


@pytest.mark.parametrize("B,D,K", [(1, 64, 64), (300, 64, 64), (7, 8, 8), (5, 128, 128), (9, 24, 256), (3, 20, 64)])
def test_decode_shapes(cuda, B, D, K):
    """T=1 through both decode kernels (the bulk-copy pipelined one needs D % 8 == 0)."""
    from t2fw_b200 import _lib, cabi

    x, f, q, k, fk, s, _, _ = to_dev(lfw_inputs(B, 1, D, K, "sigmoid", 0.5, 60 + B), torch.float16, cuda)
    out, ckpt = cabi.lfw_forward(x, f, q, k, fk, s)
    torch.cuda.synchronize()
    r_out, r_fin = fw_oracle.lfw_forward(x, f, q, k, fk, s)
    assert max_rel_err(out, r_out) <= OUT_TOL[torch.float16]
    assert max_rel_err(ckpt[:, -1], r_fin) <= OUT_TOL[torch.float16]
    assert _lib.load_core().t2fw_device_status() == 0


@pytest.mark.parametrize("D,K", [(128, 64), (64, 128), (128, 128), (192, 64), (64, 256)])
def test_blocked_state_shapes(cuda, D, K):
    """D x K states that are grids of 64 x 64 blocks run on the tensor-core path as a virtual
    batch; outputs and gradients are sums over the other axis' blocks."""
    dev = to_dev(lfw_inputs(2, 150, D, K, "sigmoid", 0.5, D + K), torch.float16, cuda)
    check_against_oracle(dev, run_cabi(*dev), torch.float16)


def test_blocked_extreme_gates(cuda):
    """Flagged blocks of a D=K=128 problem fall back to the scan kernels block by block."""
    x, f, q, k, fk, s, go, gs = lfw_inputs(2, 100, 128, 128, "sigmoid", 0.5, 71)
    fk[1, :, 64:] = 1e-3
    f[0, 30, :] = 0.0
    dev = to_dev((x, f, q, k, fk, s, go, gs), torch.float16, cuda)
    check_against_oracle(dev, run_cabi(*dev), torch.float16)


def test_many_tiny_gates_in_one_chunk(cuda):
    """More gates below 2^-13 in a chunk than the direct-sum list holds, rows with a few of them (the
    direct pair sums), and rows full of small gates that stay on the factored form: results stay
    right whichever path serves the row."""
    x, f, q, k, fk, s, go, gs = lfw_inputs(4, 192, 64, 64, "sigmoid", 0.5, 41)
    fk[0, 70:74, :] = 5e-5        # 256 tiny gates in one chunk of row 0 (list capacity 128)
    f[1, 10, ::2] = 3e-5          # 32 tiny d-side gates at one step of row 1
    fk[2, 130, 7] = 1e-5          # a single one in row 2
    fk[2, 20, 9] = -6e-5          # and a negative one
    fk[3, 100:104, ::3] = 4e-4    # 2^-11.3: small, but above the threshold
    f[3, 30, :] = 2e-4            # 2^-12.3
    dev = to_dev((x, f, q, k, fk, s, go, gs), torch.float16, cuda)
    check_against_oracle(dev, run_cabi(*dev), torch.float16)


@pytest.mark.parametrize("D,T,ckpt_every", [(64, 300, 128), (64, 256, 128), (64, 500, 192), (64, 70, 256), (128, 330, 128)])
def test_checkpoint_intervals_of_several_chunks(cuda, D, T, ckpt_every):
    """Checkpoint intervals that are multiples of 64 (BASELINE config 4 names 128) stay on the
    tensor-core path: the per-chunk states live in scratch, the caller's checkpoints hold every
    ckpt_every-th state and the final one, and the backward call rebuilds what it needs."""
    from t2fw_b200 import cabi

    x, f, q, k, fk, s, go, gs = lfw_inputs(3, T, D, D, "sigmoid", 0.5, 300 + T)
    if D == 64:
        fk[1] = 1e-3          # one batch row that the scan kernels have to redo
    dev = to_dev((x, f, q, k, fk, s, go, gs), torch.float16, cuda)
    from t2fw_b200 import _lib

    need = _lib.load_core().t2fw_lfw_forward_scratch_bytes(3, T, D, D, 0, ckpt_every)
    assert need > 0, "not on the tensor-core path"
    got = run_cabi(*dev, ckpt_every=ckpt_every)
    check_against_oracle(dev, got, torch.float16)
    # every slot of the checkpoints against the oracle's state after that many steps
    xd, fd, qd, kd, fkd, sd = dev[:6]
    _, ckpt = cabi.lfw_forward(xd, fd, qd, kd, fkd, sd, ckpt_every=ckpt_every)
    torch.cuda.synchronize()
    slots = math.ceil(T / ckpt_every)
    assert ckpt.shape[1] == slots
    for j in range(slots):
        t_end = min((j + 1) * ckpt_every, T)
        _, r_state = fw_oracle.lfw_forward(xd[:, :t_end], fd[:, :t_end], qd[:, :t_end], kd[:, :t_end], fkd[:, :t_end], sd)
        assert max_rel_err(ckpt[:, j], r_state) <= OUT_TOL[torch.float16], j
