"""LFWFunction: the decay update rule ("linear fast weights") as a torch.autograd.Function.

Mirror of the reference's t2fw/functional_lfw.py:24-78: same class name, argument order,
assertions and return convention,

    outputs, next_state = LFWFunction.apply(value, forget, query, key, f_key, state)

    S_t = (forget_t f_key_t^T) * S_{t-1} + value_t key_t^T ,   outputs_t = S_t query_t

with gradients for all six inputs.  The gates are taken as given (the caller applies any
sigmoid).  Unlike the reference, nothing is compiled at import time: the operators come from
the prebuilt library and the import fails if it is absent.
"""
import torch

from . import _lib

_lib.load_ops()


class LFWFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, value, forget, query, key, f_key, state):
        """Returns (outputs [B,T,D], next_state [B,D,K])."""
        # same contract as t2fw/functional_lfw.py:42-49
        assert value.shape == forget.shape
        assert query.shape == key.shape
        assert query.shape == f_key.shape
        for other in (forget, query, f_key, state):
            assert other.dtype == value.dtype

        outputs, ckpt_states = torch.ops.lfw.forward(value, forget, query, key, f_key, state)
        ctx.save_for_backward(value, forget, query, key, f_key, outputs, state, ckpt_states)
        # the last checkpoint slot is the state after the final step
        return outputs, ckpt_states[:, -1]

    @staticmethod
    def backward(ctx, grad_output, grad_state):
        value, forget, query, key, f_key, outputs, state, ckpt_states = ctx.saved_tensors
        assert grad_state.dtype == value.dtype
        assert grad_output.dtype == value.dtype
        grads = torch.ops.lfw.backward(grad_output.contiguous(), grad_state.contiguous(),
                                       value, forget, query, key, f_key, outputs, state,
                                       ckpt_states)
        return tuple(grads)
