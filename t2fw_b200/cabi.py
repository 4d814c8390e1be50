"""Direct calls into the C ABI (include/t2fw_b200.h) on torch CUDA tensors.

These helpers do what a foreign-language binding would do: allocate outputs, pass raw device
pointers, sizes and the current stream, and raise on a non-zero status.  They bypass autograd
and the operator dispatcher; the tests use them to exercise the ABI itself and the benchmark
uses them to time the kernels without Python framework overhead.
"""
import os

import torch

from . import _lib

F16, BF16, F32, F64 = 0, 1, 2, 3
_DTYPES = {torch.float16: F16, torch.bfloat16: BF16, torch.float32: F32, torch.float64: F64}


def dtype_code(t):
    return _DTYPES[t.dtype]


def _stream():
    return torch.cuda.current_stream().cuda_stream


def _check(rc, what):
    if rc != 0:
        lib = _lib.load_core()
        raise RuntimeError("%s failed (status %d): %s" % (what, rc, lib.t2fw_last_error().decode()))


def _dev(*ts):
    for t in ts:
        if not (t.is_cuda and t.is_contiguous()):
            raise RuntimeError("t2fw_b200.cabi: tensors must be contiguous CUDA tensors")


def ckpt_every_for(T, D, K, dtype):
    env = os.environ.get("T2FW_CKPT_EVERY")
    if env and int(env) > 0:
        return int(env)
    return int(_lib.load_core().t2fw_lfw_default_ckpt_every(T, D, K, _DTYPES[dtype]))


def _scratch(nbytes, like):
    if nbytes == 0:
        return None, 0
    buf = torch.empty(nbytes, dtype=torch.uint8, device=like.device)
    return buf, nbytes


def lfw_forward(x, f, q, k, f_key, state, ckpt_every=None, out=None, ckpt=None, scratch=None):
    """Returns (outputs [B,T,D], ckpt_states [B,slots,D,K]); ckpt_states[:, -1] is the next state."""
    lib = _lib.load_core()
    _dev(x, f, q, k, f_key, state)
    B, T, D = x.shape
    K = q.shape[2]
    C = ckpt_every or ckpt_every_for(T, D, K, x.dtype)
    slots = int(lib.t2fw_lfw_ckpt_slots(T, C))
    if out is None:
        out = torch.empty_like(x)
    if ckpt is None:
        ckpt = torch.empty(B, slots, D, K, dtype=x.dtype, device=x.device)
    nb = lib.t2fw_lfw_forward_scratch_bytes(B, T, D, K, dtype_code(x), C)
    if scratch is None:
        scratch, nb = _scratch(nb, x)
    sp = scratch.data_ptr() if scratch is not None else None
    rc = lib.t2fw_lfw_forward(x.data_ptr(), f.data_ptr(), q.data_ptr(), k.data_ptr(),
                              f_key.data_ptr(), state.data_ptr(), out.data_ptr(), ckpt.data_ptr(),
                              B, T, D, K, dtype_code(x), C, sp,
                              scratch.numel() if scratch is not None else 0, _stream())
    _check(rc, "t2fw_lfw_forward")
    return out, ckpt


def lfw_backward(grad_out, grad_state, x, f, q, k, f_key, state, ckpt, ckpt_every=None,
                 grads=None, scratch=None):
    """Returns (d_x, d_f, d_q, d_k, d_f_key, d_state)."""
    lib = _lib.load_core()
    _dev(grad_out, grad_state, x, f, q, k, f_key, state, ckpt)
    B, T, D = x.shape
    K = q.shape[2]
    C = ckpt_every or ckpt_every_for(T, D, K, x.dtype)
    if grads is None:
        grads = (torch.empty_like(x), torch.empty_like(f), torch.empty_like(q),
                 torch.empty_like(k), torch.empty_like(f_key), torch.empty_like(state))
    nb = lib.t2fw_lfw_backward_scratch_bytes(B, T, D, K, dtype_code(x), C)
    if scratch is None:
        scratch, nb = _scratch(nb, x)
    sp = scratch.data_ptr() if scratch is not None else None
    rc = lib.t2fw_lfw_backward(grad_out.data_ptr(), grad_state.data_ptr(), x.data_ptr(),
                               f.data_ptr(), q.data_ptr(), k.data_ptr(), f_key.data_ptr(),
                               state.data_ptr(), ckpt.data_ptr(),
                               *[g.data_ptr() for g in grads],
                               B, T, D, K, dtype_code(x), C, sp,
                               scratch.numel() if scratch is not None else 0, _stream())
    _check(rc, "t2fw_lfw_backward")
    return grads


def _acc_dtype(t):
    return torch.float64 if t.dtype == torch.float64 else torch.float32


def dfw_forward(q, k, v, state, scratch=None, use_scratch=True):
    """Returns (outputs [B,T,D], final_state [B,D,M], delta [B,T,D] in float/double).
    use_scratch=False calls the scratch-free entry point (step-by-step scan kernels)."""
    lib = _lib.load_core()
    _dev(q, k, v, state)
    B, T, D = v.shape
    M = q.shape[2]
    out = torch.empty_like(v)
    fin = torch.empty_like(state)
    delta = torch.empty(B, T, D, dtype=_acc_dtype(v), device=v.device)
    if not use_scratch:
        rc = lib.t2fw_dfw_forward(q.data_ptr(), k.data_ptr(), v.data_ptr(), state.data_ptr(),
                                  out.data_ptr(), fin.data_ptr(), delta.data_ptr(), B, T, D, M,
                                  dtype_code(v), _stream())
        _check(rc, "t2fw_dfw_forward")
        return out, fin, delta
    nb = lib.t2fw_dfw_forward_scratch_bytes(B, T, D, M, dtype_code(v))
    if scratch is None:
        scratch, nb = _scratch(nb, v)
    sp = scratch.data_ptr() if scratch is not None else None
    rc = lib.t2fw_dfw_forward_ws(q.data_ptr(), k.data_ptr(), v.data_ptr(), state.data_ptr(),
                                 out.data_ptr(), fin.data_ptr(), delta.data_ptr(), B, T, D, M,
                                 dtype_code(v), sp, scratch.numel() if scratch is not None else 0,
                                 _stream())
    _check(rc, "t2fw_dfw_forward_ws")
    return out, fin, delta


def dfw_backward(grad_out, grad_state, q, k, delta, final_state, scratch=None):
    """Returns (d_q, d_k, d_v, d_state)."""
    lib = _lib.load_core()
    _dev(grad_out, grad_state, q, k, delta, final_state)
    B, T, D = grad_out.shape
    M = q.shape[2]
    dq, dk = torch.empty_like(q), torch.empty_like(k)
    dv, ds = torch.empty_like(grad_out), torch.empty_like(final_state)
    nb = lib.t2fw_dfw_backward_scratch_bytes(B, T, D, M, dtype_code(q))
    if scratch is None:
        scratch, nb = _scratch(nb, q)
    sp = scratch.data_ptr() if scratch is not None else None
    rc = lib.t2fw_dfw_backward(grad_out.data_ptr(), grad_state.data_ptr(), q.data_ptr(),
                               k.data_ptr(), delta.data_ptr(), final_state.data_ptr(),
                               dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), ds.data_ptr(),
                               B, T, D, M, dtype_code(q), sp,
                               scratch.numel() if scratch is not None else 0, _stream())
    _check(rc, "t2fw_dfw_backward")
    return dq, dk, dv, ds
