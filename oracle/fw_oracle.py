"""ctypes front end of the float64 C oracle (oracle/fw_oracle.c).  Test infrastructure only.

Every function takes array-likes (numpy arrays or CPU torch tensors), converts them to
contiguous float64 and returns numpy float64 arrays.  Argument order follows the reference's
Python API: LFWFunction.apply(value, forget, query, key, f_key, state)
(t2fw/functional_lfw.py:31-38) and DFWFunction.apply(query, key, value, state)
(t2fw/functional_dfw.py:29-34).
"""
import ctypes
import os

import numpy as np

from . import build_oracle

_lib = None


def _load():
    global _lib
    if _lib is None:
        path = build_oracle.OUT
        if not os.path.exists(path) or os.path.getmtime(path) < os.path.getmtime(build_oracle.SRC):
            path = build_oracle.build()
        _lib = ctypes.CDLL(path)
    return _lib


def _f64(a):
    if hasattr(a, "detach"):
        a = a.detach().to("cpu").double().numpy()
    return np.ascontiguousarray(np.asarray(a, dtype=np.float64))


def _p(a):
    return a.ctypes.data_as(ctypes.c_void_p)


_i64 = ctypes.c_int64


def lfw_forward(x, f, q, k, f_key, state):
    """Decay rule forward (t2fw/torch.py:21-28): returns (outputs[B,T,D], final_state[B,D,K])."""
    x, f, q, k, f_key, state = map(_f64, (x, f, q, k, f_key, state))
    B, T, D = x.shape
    K = q.shape[2]
    out = np.empty((B, T, D))
    fin = np.empty((B, D, K))
    _load().t2fw_oracle_lfw_forward(_p(x), _p(f), _p(q), _p(k), _p(f_key), _p(state),
                                    _i64(B), _i64(T), _i64(D), _i64(K), _p(out), _p(fin))
    return out, fin


def lfw_backward(grad_out, grad_state, x, f, q, k, f_key, state):
    """Gradients (d_x, d_f, d_q, d_k, d_f_key, d_state) of the decay rule, the order in which
    the reference returns them (t2fw/csrc/lfw.cpp:95)."""
    grad_out, grad_state, x, f, q, k, f_key, state = map(
        _f64, (grad_out, grad_state, x, f, q, k, f_key, state))
    B, T, D = x.shape
    K = q.shape[2]
    dx, df = np.empty((B, T, D)), np.empty((B, T, D))
    dq, dk, dfk = np.empty((B, T, K)), np.empty((B, T, K)), np.empty((B, T, K))
    ds = np.empty((B, D, K))
    _load().t2fw_oracle_lfw_backward(_p(grad_out), _p(grad_state), _p(x), _p(f), _p(q), _p(k),
                                     _p(f_key), _p(state), _i64(B), _i64(T), _i64(D), _i64(K),
                                     _p(dx), _p(df), _p(dq), _p(dk), _p(dfk), _p(ds))
    return dx, df, dq, dk, dfk, ds


def dfw_forward(q, k, v, state):
    """Delta rule forward (t2fw/torch.py:44-52): returns (outputs, final_state, delta)."""
    q, k, v, state = map(_f64, (q, k, v, state))
    B, T, D = v.shape
    M = q.shape[2]
    out, dl = np.empty((B, T, D)), np.empty((B, T, D))
    fin = np.empty((B, D, M))
    _load().t2fw_oracle_dfw_forward(_p(q), _p(k), _p(v), _p(state), _i64(B), _i64(T), _i64(D),
                                    _i64(M), _p(out), _p(fin), _p(dl))
    return out, fin, dl


def dfw_backward(grad_out, grad_state, q, k, v, state):
    """Gradients (d_q, d_k, d_v, d_state) of the delta rule (t2fw/torch.py:84-143)."""
    grad_out, grad_state, q, k, v, state = map(_f64, (grad_out, grad_state, q, k, v, state))
    B, T, D = v.shape
    M = q.shape[2]
    dq, dk = np.empty((B, T, M)), np.empty((B, T, M))
    dv = np.empty((B, T, D))
    ds = np.empty((B, D, M))
    _load().t2fw_oracle_dfw_backward(_p(grad_out), _p(grad_state), _p(q), _p(k), _p(v), _p(state),
                                     _i64(B), _i64(T), _i64(D), _i64(M),
                                     _p(dq), _p(dk), _p(dv), _p(ds))
    return dq, dk, dv, ds
