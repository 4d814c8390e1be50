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


def test_numa_binding_reads_the_topology(tmp_path):
    """bind_host_to_gpu_node's sysfs logic on a fake tree: node lookup, CPU list parsing, the
    intersection with the allowed set, and the reasons it gives when it cannot bind."""
    from t2fw_b200.parallel import _bind_to_pci_node, _parse_cpulist

    assert _parse_cpulist("0-3,8,10-11\n") == {0, 1, 2, 3, 8, 10, 11}
    dev = tmp_path / "bus/pci/devices/0000:1b:00.0"
    dev.mkdir(parents=True)
    (dev / "numa_node").write_text("1\n")
    node = tmp_path / "devices/system/node/node1"
    node.mkdir(parents=True)
    (node / "cpulist").write_text("16-31\n")
    ok = _bind_to_pci_node("0000:1b:00.0", str(tmp_path), set(range(0, 24)), False, {"bound": False})
    assert ok["bound"] and ok["numa_node"] == 1 and ok["cpus"] == 8
    none = _bind_to_pci_node("0000:1b:00.0", str(tmp_path), set(range(0, 16)), False, {"bound": False})
    assert not none["bound"] and "available" in none["reason"]
    missing = _bind_to_pci_node("0000:ff:00.0", str(tmp_path), {0}, False, {"bound": False})
    assert not missing["bound"] and "not readable" in missing["reason"]
    (dev / "numa_node").write_text("-1\n")
    flat = _bind_to_pci_node("0000:1b:00.0", str(tmp_path), {0}, False, {"bound": False})
    assert not flat["bound"] and "no NUMA node" in flat["reason"]
