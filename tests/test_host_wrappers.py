"""Host-side behaviour of the autograd wrappers that needs no GPU: the reference's assertion
contract (t2fw/functional_lfw.py:42-49, t2fw/functional_dfw.py:38-40) and its RuntimeError for
non-CUDA inputs (t2fw/csrc/lfw.cpp:24-26)."""
import pytest
import torch

from t2fw_b200.functional_lfw import LFWFunction
from t2fw_b200.functional_dfw import DFWFunction


def _lfw_args(B=2, T=3, D=4, K=5, dtype=torch.float32):
    x, f = torch.randn(B, T, D, dtype=dtype), torch.rand(B, T, D, dtype=dtype)
    q, k, fk = (torch.randn(B, T, K, dtype=dtype) for _ in range(3))
    s = torch.zeros(B, D, K, dtype=dtype)
    return [x, f, q, k, fk, s]


def test_alias_package_exports_the_same_classes():
    from t2fw.functional_lfw import LFWFunction as A
    from t2fw.functional_dfw import DFWFunction as B

    assert A is LFWFunction and B is DFWFunction


def test_lfw_shape_mismatch_asserts():
    a = _lfw_args()
    a[1] = a[1][:, :, :3]
    with pytest.raises(AssertionError):
        LFWFunction.apply(*a)
    a = _lfw_args()
    a[4] = a[4][:, :2]
    with pytest.raises(AssertionError):
        LFWFunction.apply(*a)


def test_lfw_dtype_mismatch_asserts():
    a = _lfw_args()
    a[5] = a[5].double()
    with pytest.raises(AssertionError):
        LFWFunction.apply(*a)


def test_lfw_cpu_tensor_is_a_runtime_error():
    with pytest.raises(RuntimeError, match="must be a CUDA tensor"):
        LFWFunction.apply(*_lfw_args())


def test_dfw_contract():
    q, k = torch.randn(2, 3, 5), torch.randn(2, 3, 5)
    v, s = torch.randn(2, 3, 4), torch.zeros(2, 4, 5)
    with pytest.raises(AssertionError):
        DFWFunction.apply(q, k[:, :, :4], v, s)
    with pytest.raises(AssertionError):
        DFWFunction.apply(q, k, v.double(), s)
    with pytest.raises(RuntimeError, match="must be a CUDA tensor"):
        DFWFunction.apply(q, k, v, s)
