"""Step-by-step PyTorch restatement of the reference's CPU path.  Test infrastructure only.

This is the "port" that stands in for the reference's TorchScript functions on machines where
the reference itself is not present: one Python-level loop over time, each step a handful of
dense torch operations on the [B, D, K] state, with autograd supplying the backward pass.  It
is what the benchmark times as the CPU baseline.

  lfw_loop  follows t2fw/torch.py:21-28 (decay rule)
  dfw_loop  follows t2fw/torch.py:44-52 (delta rule)
"""
import torch


def lfw_loop(x, f, query, key, f_key, state):
    """S_t = (f_t f_key_t^T) * S_{t-1} + x_t key_t^T ; o_t = S_t query_t."""
    outs = []
    for t in range(x.shape[1]):
        gate = torch.einsum("bd,bk->bdk", f[:, t], f_key[:, t])
        write = torch.einsum("bd,bk->bdk", x[:, t], key[:, t])
        state = gate * state + write
        outs.append(torch.einsum("bdk,bk->bd", state, query[:, t]))
    return torch.stack(outs, dim=1), state


def dfw_loop(query, key, value, state):
    """o_t = S_{t-1} q_t ; S_t = S_{t-1} + (v_t - S_{t-1} k_t) k_t^T."""
    outs = []
    for t in range(value.shape[1]):
        kt = key[:, t]
        outs.append(torch.einsum("bdm,bm->bd", state, query[:, t]))
        delta = value[:, t] - torch.einsum("bdm,bm->bd", state, kt)
        state = state + torch.einsum("bd,bm->bdm", delta, kt)
    return torch.stack(outs, dim=1), state


def lfw_fwd_bwd(x, f, q, k, f_key, state, grad_out, grad_state):
    """Forward + backward through autograd; returns (out, final_state, six gradients)."""
    leaves = [t.detach().clone().requires_grad_(True) for t in (x, f, q, k, f_key, state)]
    out, fin = lfw_loop(*leaves)
    grads = torch.autograd.grad([out, fin], leaves, [grad_out, grad_state])
    return out.detach(), fin.detach(), grads


def dfw_fwd_bwd(q, k, v, state, grad_out, grad_state):
    leaves = [t.detach().clone().requires_grad_(True) for t in (q, k, v, state)]
    out, fin = dfw_loop(*leaves)
    grads = torch.autograd.grad([out, fin], leaves, [grad_out, grad_state])
    return out.detach(), fin.detach(), grads
