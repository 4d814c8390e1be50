"""The fused decay-rule layer core (heads read in place from the projection output, query scale and
gate activation applied in the kernels) against the same layer built from the plain operator and
separate PyTorch passes, and against the oracle."""
import pytest
import torch

from helpers import GRAD_TOL, OUT_TOL, max_rel_err
from oracle import fw_oracle

pytestmark = pytest.mark.gpu


def _inputs(B, T, H, dtype, dev, seed):
    g = torch.Generator().manual_seed(seed)
    C = H * 64
    qkvg = torch.randn(B, T, 4 * C, generator=g)
    qkvg[:, :, 3 * C:] = qkvg[:, :, 3 * C:] * 2.0 + 1.0          # gate pre-activations, some far below the floor
    state = torch.randn(B * H, 64, 64, generator=g) * 0.3
    go = torch.randn(B, T, C, generator=g)
    gs = torch.randn(B * H, 64, 64, generator=g)
    return [t.to(dtype).to(dev) for t in (qkvg, state, go, gs)]


@pytest.mark.parametrize("B,T,H", [(2, 200, 3), (1, 64, 1), (3, 130, 12), (2, 1000, 2)])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_fused_equals_the_layer_built_from_the_plain_operator(cuda, B, T, H, dtype):
    from t2fw_b200.functional_fused import LFWFusedFunction, unfused_reference

    qkvg, state, go, gs = _inputs(B, T, H, dtype, cuda, 7 * B + T + H)
    a = [qkvg.clone().requires_grad_(True), state.clone().requires_grad_(True)]
    out, nxt = LFWFusedFunction.apply(a[0], a[1], H)
    ga = torch.autograd.grad([out, nxt], a, [go, gs])
    b = [qkvg.clone().requires_grad_(True), state.clone().requires_grad_(True)]
    out_r, nxt_r = unfused_reference(b[0], b[1], H)
    gb = torch.autograd.grad([out_r, nxt_r], b, [go, gs])
    torch.cuda.synchronize()
    # forward: the kernels see the same rounded operands, so the results are identical
    assert torch.equal(out, out_r) and torch.equal(nxt, nxt_r)
    assert torch.equal(ga[1], gb[1])                                  # d_state
    C = H * 64
    assert torch.equal(ga[0][:, :, C:3 * C], gb[0][:, :, C:3 * C])   # d_key, d_value: no activation in between
    # d_query, d_gate: the composed path rounds the intermediate gradient to 16 bits before the
    # chain rule, the fused path applies it in fp32
    assert max_rel_err(ga[0][:, :, :C], gb[0][:, :, :C]) <= 2e-3
    assert max_rel_err(ga[0][:, :, 3 * C:], gb[0][:, :, 3 * C:]) <= 4e-3 * (8 if dtype == torch.bfloat16 else 1)


def test_fused_against_the_oracle(cuda):
    from t2fw_b200.functional_fused import GATE_FLOOR, LFWFusedFunction

    B, T, H = 2, 300, 4
    C = H * 64
    qkvg, state, go, gs = _inputs(B, T, H, torch.float16, cuda, 99)
    leaves = [qkvg.clone().requires_grad_(True), state.clone().requires_grad_(True)]
    out, nxt = LFWFusedFunction.apply(*leaves, H)
    d_qkvg, d_state = torch.autograd.grad([out, nxt], leaves, [go, gs])
    torch.cuda.synchronize()

    def fold(t):
        return t.view(B, T, H, 64).permute(0, 2, 1, 3).reshape(B * H, T, 64).double().cpu()

    q, k, v, g = (fold(p) for p in qkvg.split(C, dim=-1))
    sig = torch.sigmoid(g)
    gate = sig.clamp_min(GATE_FLOOR)
    ones = torch.ones_like(v)
    r_out, r_fin = fw_oracle.lfw_forward(v, ones, q / 8, k, gate, state.double().cpu())
    r = fw_oracle.lfw_backward(fold(go), gs.double().cpu(), v, ones, q / 8, k, gate, state.double().cpu())
    assert max_rel_err(fold(out), r_out) <= OUT_TOL[torch.float16]
    assert max_rel_err(nxt, r_fin) <= OUT_TOL[torch.float16]
    d_q, d_k, d_v, d_g = (fold(p) for p in d_qkvg.split(C, dim=-1))
    assert max_rel_err(d_v, r[0]) <= GRAD_TOL[torch.float16]
    assert max_rel_err(d_q, r[2] / 8) <= GRAD_TOL[torch.float16]
    assert max_rel_err(d_k, r[3]) <= GRAD_TOL[torch.float16]
    want_g = torch.as_tensor(r[4]) * torch.where(sig > GATE_FLOOR, sig * (1 - sig), torch.zeros_like(sig))
    assert max_rel_err(d_g, want_g) <= GRAD_TOL[torch.float16]
    assert max_rel_err(d_state, r[5]) <= GRAD_TOL[torch.float16]


def test_fused_layer_under_graph_capture(cuda):
    """Forward + backward of the fused entry points captured in a CUDA graph (the tensor maps are
    built on the host inside the capture, on the caller's thread and on autograd's worker thread)
    and replayed twice: bitwise equal to the eager result."""
    from t2fw_b200.functional_fused import LFWFusedFunction

    qkvg, state, go, gs = _inputs(2, 256, 3, torch.float16, cuda, 77)

    def run():
        leaves = [qkvg.detach().requires_grad_(True), state.detach().requires_grad_(True)]
        out, nxt = LFWFusedFunction.apply(leaves[0], leaves[1], 3)
        return [out, nxt] + list(torch.autograd.grad([out, nxt], leaves, [go, gs]))

    eager = [t.clone() for t in run()]
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        run()
    torch.cuda.current_stream().wait_stream(side)
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        static = run()
    for _ in range(2):
        for t in static:
            t.detach().fill_(float("nan"))
        g.replay()
        torch.cuda.synchronize()
        for a, b in zip(static, eager):
            assert torch.equal(a, b)
