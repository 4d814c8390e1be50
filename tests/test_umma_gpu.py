"""The tcgen05 building blocks (tensor memory, descriptors for both operand orientations, MMA,
accumulator loads) against a host matrix product, through the C ABI."""
import ctypes

import pytest
import torch



def _tf32(t):
    """Round to TF32 (10 mantissa bits) so that the tensor core's products are exact."""
    i = t.contiguous().view(torch.int32)
    i = (i + 0x1000) & ~0x1FFF
    return i.view(torch.float32)


@pytest.mark.gpu
@pytest.mark.parametrize("a_mn,b_mn", [(0, 0)])
@pytest.mark.parametrize("N,Kc", [(8, 8), (16, 8), (16, 16), (16, 64), (64, 16), (64, 64), (24, 40)])
def test_umma_products(cuda, N, Kc, a_mn, b_mn):
    from t2fw_b200 import _lib

    lib = _lib.load_core()
    fn = lib.t2fw_selftest_umma
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p] * 6 + [ctypes.c_int] * 4 + [ctypes.c_void_p, ctypes.c_void_p]
    g = torch.Generator().manual_seed(N * 100 + Kc)
    A1, A2 = (_tf32(torch.randn(64, Kc, generator=g)).to(cuda) for _ in range(2))
    B1, B2 = (_tf32(torch.randn(N, Kc, generator=g)).to(cuda) for _ in range(2))
    D1 = torch.full((64, N), float("nan"), device=cuda)
    D2 = torch.full((64, N), float("nan"), device=cuda)
    status = torch.zeros(1, dtype=torch.int32, device=cuda)
    rc = fn(A1.data_ptr(), B1.data_ptr(), A2.data_ptr(), B2.data_ptr(), D1.data_ptr(), D2.data_ptr(),
            N, Kc, a_mn, b_mn, status.data_ptr(), torch.cuda.current_stream().cuda_stream)
    assert rc == 0, lib.t2fw_last_error().decode()
    torch.cuda.synchronize()
    assert int(status.item()) == 0, "a bounded wait expired"
    for D, A, B in ((D1, A1, B1), (D2, A2, B2)):
        ref = (A.double() @ B.double().T)
        assert torch.isfinite(D).all()
        assert (D.double() - ref).abs().max().item() <= 1e-4 * max(1.0, ref.abs().max().item())


def test_mn_major_tf32_is_rejected():
    """No GPU needed: the orientation the hardware does not offer is refused up front."""
    from t2fw_b200 import _lib

    lib = _lib.load_core()
    fn = lib.t2fw_selftest_umma
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p] * 6 + [ctypes.c_int] * 4 + [ctypes.c_void_p, ctypes.c_void_p]
    assert fn(1, 1, 1, 1, 1, 1, 16, 16, 1, 0, 1, None) == 1
    assert b"K-major" in lib.t2fw_last_error()


def _bf16(t):
    return t.to(torch.bfloat16).to(torch.float32)


@pytest.mark.gpu
@pytest.mark.parametrize("a_mn", [0, 1])
@pytest.mark.parametrize("b_mn", [0, 1])
@pytest.mark.parametrize("N,Kc", [(8, 16), (16, 16), (16, 64), (64, 16), (64, 64), (32, 48)])
def test_umma16_products(cuda, N, Kc, a_mn, b_mn):
    from t2fw_b200 import _lib

    lib = _lib.load_core()
    fn = lib.t2fw_selftest_umma16
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p] * 6 + [ctypes.c_int] * 4 + [ctypes.c_void_p, ctypes.c_void_p]
    g = torch.Generator().manual_seed(N * 100 + Kc + 7)
    A1, A2 = (_bf16(torch.randn(64, Kc, generator=g)).to(cuda) for _ in range(2))
    B1, B2 = (_bf16(torch.randn(N, Kc, generator=g)).to(cuda) for _ in range(2))
    D1 = torch.full((64, N), float("nan"), device=cuda)
    D2 = torch.full((64, N), float("nan"), device=cuda)
    status = torch.zeros(1, dtype=torch.int32, device=cuda)
    rc = fn(A1.data_ptr(), B1.data_ptr(), A2.data_ptr(), B2.data_ptr(), D1.data_ptr(), D2.data_ptr(),
            N, Kc, a_mn, b_mn, status.data_ptr(), torch.cuda.current_stream().cuda_stream)
    assert rc == 0, lib.t2fw_last_error().decode()
    torch.cuda.synchronize()
    assert int(status.item()) == 0, "a bounded wait expired"
    for D, A, B in ((D1, A1, B1), (D2, A2, B2)):
        ref = (A.double() @ B.double().T)
        assert torch.isfinite(D).all()
        assert (D.double() - ref).abs().max().item() <= 1e-4 * max(1.0, ref.abs().max().item())


@pytest.mark.gpu
def test_umma_a_operand_from_tensor_memory(cuda):
    """A [64 x 64] written into tensor memory (both lane sets), B a 128-byte-swizzle shared-memory
    tile: the operand forms of the 64-step chunk kernels."""
    from t2fw_b200 import _lib

    lib = _lib.load_core()
    fn = lib.t2fw_selftest_umma_ts
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p] * 3 + [ctypes.c_void_p, ctypes.c_void_p]
    g = torch.Generator().manual_seed(11)
    A = _tf32(torch.randn(64, 64, generator=g)).to(cuda)
    B = _tf32(torch.randn(64, 64, generator=g)).to(cuda)
    D = torch.full((64, 64), float("nan"), device=cuda)
    status = torch.zeros(1, dtype=torch.int32, device=cuda)
    rc = fn(A.data_ptr(), B.data_ptr(), D.data_ptr(), status.data_ptr(), torch.cuda.current_stream().cuda_stream)
    assert rc == 0, lib.t2fw_last_error().decode()
    torch.cuda.synchronize()
    assert int(status.item()) == 0, "a bounded wait expired"
    ref = A.double() @ B.double().T
    assert (D.double() - ref).abs().max().item() <= 1e-4 * max(1.0, ref.abs().max().item())


def _trunc(t):
    """Drop the 13 low mantissa bits: what the tensor core keeps of an fp32 operand."""
    i = t.contiguous().view(torch.int32)
    return (i & ~0x1FFF).view(torch.float32)


@pytest.mark.gpu
def test_tf32_operands_are_truncated_not_rounded(cuda):
    """The chunk kernels store operands with the rounding increment added but the low 13 bits left
    in place, relying on the tensor core to ignore those bits - for operands in shared memory and in
    tensor memory.  Unrounded inputs must therefore give the product of the truncated inputs."""
    from t2fw_b200 import _lib

    lib = _lib.load_core()
    g = torch.Generator().manual_seed(23)
    status = torch.zeros(1, dtype=torch.int32, device=cuda)
    stream = torch.cuda.current_stream().cuda_stream

    fn = lib.t2fw_selftest_umma
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p] * 6 + [ctypes.c_int] * 4 + [ctypes.c_void_p, ctypes.c_void_p]
    A1, A2, B1, B2 = (torch.randn(64, 64, generator=g).to(cuda) for _ in range(4))
    D1 = torch.full((64, 64), float("nan"), device=cuda)
    D2 = torch.full((64, 64), float("nan"), device=cuda)
    rc = fn(A1.data_ptr(), B1.data_ptr(), A2.data_ptr(), B2.data_ptr(), D1.data_ptr(), D2.data_ptr(),
            64, 64, 0, 0, status.data_ptr(), stream)
    assert rc == 0, lib.t2fw_last_error().decode()

    fn_ts = lib.t2fw_selftest_umma_ts
    fn_ts.restype = ctypes.c_int
    fn_ts.argtypes = [ctypes.c_void_p] * 3 + [ctypes.c_void_p, ctypes.c_void_p]
    A3, B3 = (torch.randn(64, 64, generator=g).to(cuda) for _ in range(2))
    D3 = torch.full((64, 64), float("nan"), device=cuda)
    rc = fn_ts(A3.data_ptr(), B3.data_ptr(), D3.data_ptr(), status.data_ptr(), stream)
    assert rc == 0, lib.t2fw_last_error().decode()
    torch.cuda.synchronize()
    assert int(status.item()) == 0, "a bounded wait expired"
    for D, A, B in ((D1, A1, B1), (D2, A2, B2), (D3, A3, B3)):
        kept = _trunc(A).double() @ _trunc(B).double().T
        full = A.double() @ B.double().T
        assert (D.double() - kept).abs().max().item() <= 1e-4       # fp32 accumulation only
        assert (D.double() - full).abs().max().item() >= 1e-3       # the dropped bits do matter
