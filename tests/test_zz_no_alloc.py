"""The allocation-free delta-rule backward (t2fw_dfw_backward_noalloc).

It exists for hosts that cannot allocate device memory when they call the operator and cannot
pass scratch through their bridge; its scratch is a fixed array inside the library.  The test
drives it through the C ABI exactly as such a host would (raw pointers, no scratch argument)
and compares every gradient with the regular entry point AND with the float64 oracle, twice in a
row on different data so that whatever the first call left in the shared array is shown not to
matter.  The second problem is D = M = 64, where the regular entry point runs the chunked
tensor-core kernels and this one the sequential scan kernels: two different computations of the
same gradients.  This file sorts
last on purpose: a run that stops at the first failure has then already run everything else.
"""
import pytest
import torch

from helpers import GRAD_TOL, dfw_inputs, max_rel_err, to_dev
from oracle import fw_oracle


def _call_noalloc(lib, go, gs, q, k, delta, fin):
    B, T, D = go.shape
    M = q.shape[2]
    from t2fw_b200 import cabi

    dq, dk = torch.empty_like(q), torch.empty_like(k)
    dv, ds = torch.empty_like(go), torch.empty_like(fin)
    rc = lib.t2fw_dfw_backward_noalloc(go.data_ptr(), gs.data_ptr(), q.data_ptr(), k.data_ptr(),
                                       delta.data_ptr(), fin.data_ptr(), dq.data_ptr(),
                                       dk.data_ptr(), dv.data_ptr(), ds.data_ptr(), B, T, D, M,
                                       cabi.dtype_code(q), torch.cuda.current_stream().cuda_stream)
    assert rc == 0, lib.t2fw_last_error().decode()
    return dq, dk, dv, ds


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_noalloc_matches_regular_entry_point_twice(cuda, dtype):
    from t2fw_b200 import _lib, cabi

    lib = _lib.load_core()
    for seed, (B, T, D, M) in ((31, (6, 200, 64, 32)), (32, (5, 300, 64, 64)), (34, (3, 333, 40, 24))):
        q, k, v, s, go, gs = to_dev(dfw_inputs(B, T, D, M, "scaled", 0.3, seed), dtype, cuda)
        _, fin, delta = cabi.dfw_forward(q, k, v, s)
        want = cabi.dfw_backward(go, gs, q, k, delta, fin)
        got = _call_noalloc(lib, go, gs, q, k, delta, fin)
        torch.cuda.synchronize()
        oracle = fw_oracle.dfw_backward(go, gs, q, k, v, s)
        for g, w, o, name in zip(got, want, oracle, ("d_q", "d_k", "d_v", "d_state")):
            assert torch.isfinite(g).all(), name
            assert max_rel_err(g, w) <= GRAD_TOL[dtype], name
            assert max_rel_err(g, o) <= GRAD_TOL[dtype], name + " (oracle)"


@pytest.mark.gpu
def test_noalloc_fp32_needs_no_scratch(cuda):
    from t2fw_b200 import _lib, cabi

    lib = _lib.load_core()
    q, k, v, s, go, gs = to_dev(dfw_inputs(2, 50, 16, 8, "softmax", 1.0, 33), torch.float32, cuda)
    _, fin, delta = cabi.dfw_forward(q, k, v, s)
    want = cabi.dfw_backward(go, gs, q, k, delta, fin)
    got = _call_noalloc(lib, go, gs, q, k, delta, fin)
    torch.cuda.synchronize()
    for g, w in zip(got, want):
        assert max_rel_err(g, w) <= GRAD_TOL[torch.float32]


def test_noalloc_rejects_oversized_problems():
    """Size check happens before any CUDA call, so this part runs without a GPU."""
    from t2fw_b200 import _lib

    lib = _lib.load_core()
    cap = lib.t2fw_dfw_backward_noalloc_max_elems()
    assert cap == 4 * 1024 * 1024
    one = 1  # any non-null pointer value; nothing is dereferenced on this path
    ptrs = [one] * 10
    B, T, D = 64, 1024, 65          # 4,259,840 elements > capacity
    rc = lib.t2fw_dfw_backward_noalloc(*ptrs, B, T, D, 8, 0, None)
    assert rc == 3
    msg = lib.t2fw_last_error().decode()
    assert "exceeds the built-in scratch" in msg and "t2fw_dfw_backward" in msg
    # sizes whose product wraps around 64 bits are refused as well
    rc = lib.t2fw_dfw_backward_noalloc(*ptrs, 1 << 32, 1 << 32, 1, 8, 0, None)
    assert rc == 3
