"""The decay rule as a fused attention-replacement layer core (d_head = 64).

`LFWFusedFunction.apply(qkvg, state, n_head) -> (outputs, next_state)` takes the projection output
qkvg [B, T, 4*H*64] (query | key | value | gate pre-activation, heads inside a row) and does in the
kernels what a caller of the plain operator does around it in separate passes: the head fold
[B,T,H*d] -> [B*H,T,d], the 1/sqrt(d) query scale, the gate activation and the head unfold of the
outputs.  The reference leaves these to the caller (its wrapper "assumes the input is already
gated", t2fw/functional_lfw.py:26-29); this entry point is additive and `LFWFunction` is unchanged.

Defined as: x = value, forget gate = 1, query * 1/8, f_key = max(sigmoid(gate), 1/8).  The result
is bit-identical to `LFWFunction.apply` on the folded tensors with those activations applied and
rounded to the storage type (see tests/test_fused_gpu.py).
"""
import torch

from . import _lib

_lib.load_ops()

GATE_FLOOR = 0.125


class LFWFusedFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, qkvg, state, n_head):
        assert qkvg.dim() == 3 and qkvg.shape[2] == 4 * n_head * 64, "qkvg must be [B, T, 4*H*64]"
        assert state.shape == (qkvg.shape[0] * n_head, 64, 64), "state must be [B*H, 64, 64]"
        assert qkvg.dtype == state.dtype
        qkvg = qkvg.contiguous()
        state = state.contiguous()
        outputs, ckpt = torch.ops.lfw.fused_forward(qkvg, state, n_head)
        ctx.save_for_backward(qkvg, state, ckpt)
        ctx.n_head = n_head
        return outputs, ckpt[:, -1]

    @staticmethod
    def backward(ctx, grad_output, grad_state):
        qkvg, state, ckpt = ctx.saved_tensors
        d_qkvg, d_state = torch.ops.lfw.fused_backward(grad_output.contiguous(), grad_state.contiguous(), qkvg,
                                                       state, ckpt, ctx.n_head)
        return d_qkvg, d_state, None


def unfused_reference(qkvg, state, n_head):
    """The same layer core built from the plain operator and separate PyTorch passes (what the fused
    entry point replaces); used by the tests and as the fallback for head sizes other than 64."""
    from .functional_lfw import LFWFunction

    B, T, C4 = qkvg.shape
    C = C4 // 4
    d = C // n_head

    def fold(t):
        return t.view(B, T, n_head, d).permute(0, 2, 1, 3).reshape(B * n_head, T, d).contiguous()

    q, k, v, g = (fold(p) for p in qkvg.split(C, dim=-1))
    gate = torch.sigmoid(g.float()).clamp_min(GATE_FLOOR).to(qkvg.dtype)
    q = (q.float() * (d ** -0.5)).to(qkvg.dtype)
    out, nxt = LFWFunction.apply(v, torch.ones_like(v), q, k, gate, state)
    return out.view(B, n_head, T, d).permute(0, 2, 1, 3).reshape(B, T, C), nxt
