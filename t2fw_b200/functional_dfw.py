"""DFWFunction: the delta update rule as a torch.autograd.Function.

Mirror of the reference's t2fw/functional_dfw.py:24-65:

    outputs, final_state = DFWFunction.apply(query, key, value, state)

    outputs_t = S_{t-1} query_t
    S_t       = S_{t-1} + (value_t - S_{t-1} key_t) key_t^T

(the write strength is assumed to be folded into the key).  Gradients are returned for all
four inputs.  The operators come from the prebuilt library; the import fails if it is absent.
"""
import torch

from . import _lib

_lib.load_ops()


class DFWFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, query, key, value, state):
        """Returns (outputs [B,T,D], final_state [B,D,M])."""
        # same contract as t2fw/functional_dfw.py:38-40
        assert query.shape == key.shape
        assert query.dtype == value.dtype
        assert state.dtype == value.dtype

        outputs, final_state, delta_value = torch.ops.dfw.forward(query, key, value, state)
        ctx.save_for_backward(query, key, delta_value, final_state)
        return outputs, final_state

    @staticmethod
    def backward(ctx, grad_output, grad_state):
        query, key, delta_value, final_state = ctx.saved_tensors
        assert grad_state.dtype == query.dtype
        assert grad_output.dtype == query.dtype
        grads = torch.ops.dfw.backward(grad_output.contiguous(), grad_state.contiguous(),
                                       query, key, delta_value, final_state)
        return tuple(grads)
