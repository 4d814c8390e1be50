"""Step-by-step PyTorch statements of the two recurrences, with the names and signatures of the
reference's `t2fw/torch.py` (t2fw_torch :10-16, t2dfw_torch :35-39, t2dfw_torch_bw :59-67,
t2dfw_torch_bw_simple :148-156).

They run on whatever device and dtype their arguments have and define what the CUDA operators
compute; `LFWFunction` / `DFWFunction` never call them (the operators have no eager fallback).
"""
from typing import Tuple

import torch


def t2fw_torch(x: torch.Tensor, f: torch.Tensor, query: torch.Tensor, key: torch.Tensor,
               f_key: torch.Tensor, state: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """Decay rule: S_t = (f_t f_key_t^T) * S_{t-1} + x_t key_t^T, o_t = S_t query_t.
    x, f [B,T,D]; query, key, f_key [B,T,K]; state [B,D,K] -> (outputs [B,T,D], state [B,D,K])."""
    outputs = []
    for t in range(x.shape[1]):
        state = state * (f[:, t, :, None] * f_key[:, t, None, :]) + x[:, t, :, None] * key[:, t, None, :]
        outputs.append(torch.einsum("bdk,bk->bd", state, query[:, t]))
    return torch.stack(outputs, dim=1), state


def t2dfw_torch(query: torch.Tensor, key: torch.Tensor, value: torch.Tensor,
                state: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """Delta rule: o_t = S_{t-1} q_t, S_t = S_{t-1} + (v_t - S_{t-1} k_t) k_t^T.
    query, key [B,T,M]; value [B,T,D]; state [B,D,M] -> (outputs [B,T,D], state [B,D,M])."""
    outputs = []
    for t in range(value.shape[1]):
        k_t = key[:, t]
        outputs.append(torch.einsum("bdm,bm->bd", state, query[:, t]))
        delta = value[:, t] - torch.einsum("bdm,bm->bd", state, k_t)
        state = state + delta[:, :, None] * k_t[:, None, :]
    return torch.stack(outputs, dim=1), state


def t2dfw_torch_bw(grad_output: torch.Tensor, grad_state: torch.Tensor, query: torch.Tensor,
                   key: torch.Tensor, value: torch.Tensor, state: torch.Tensor,
                   final_state: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]:
    """Hand-written backward of the delta rule -> (d_query, d_key, d_value, d_state).

    The forward pass is replayed once to collect delta_t = v_t - S_{t-1} k_t; the reverse sweep then
    walks the state back from `final_state` (S_{t-1} = S_t - delta_t k_t^T), so no state is stored."""
    T = value.shape[1]
    deltas = []
    s = state
    for t in range(T):
        d_t = value[:, t] - torch.einsum("bdm,bm->bd", s, key[:, t])
        s = s + d_t[:, :, None] * key[:, t, None, :]
        deltas.append(d_t)
    r = grad_state          # gradient with respect to S_t
    s = final_state         # S_t
    d_q, d_k, d_v = [None] * T, [None] * T, [None] * T
    for t in range(T - 1, -1, -1):
        k_t, q_t, go_t, d_t = key[:, t], query[:, t], grad_output[:, t], deltas[t]
        s = s - d_t[:, :, None] * k_t[:, None, :]                     # S_{t-1}
        g_delta = torch.einsum("bdm,bm->bd", r, k_t)                  # through S_t = S_{t-1} + delta k^T
        d_v[t] = g_delta
        d_k[t] = torch.einsum("bdm,bd->bm", r, d_t) - torch.einsum("bdm,bd->bm", s, g_delta)
        d_q[t] = torch.einsum("bdm,bd->bm", s, go_t)
        r = r + go_t[:, :, None] * q_t[:, None, :] - g_delta[:, :, None] * k_t[:, None, :]
    return torch.stack(d_q, dim=1), torch.stack(d_k, dim=1), torch.stack(d_v, dim=1), r


def t2dfw_torch_bw_simple(grad_output: torch.Tensor, grad_state: torch.Tensor, query: torch.Tensor,
                          key: torch.Tensor, value: torch.Tensor, state: torch.Tensor,
                          final_state: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]:
    """The same gradients by automatic differentiation of `t2dfw_torch` (`final_state` is not needed)."""
    del final_state
    with torch.enable_grad():
        leaves = [t.detach().clone().requires_grad_(True) for t in (query, key, value, state)]
        out, fin = t2dfw_torch(*leaves)
        d_q, d_k, d_v, d_s = torch.autograd.grad([out, fin], leaves, [grad_output, grad_state])
    return d_q, d_k, d_v, d_s
