"""Tensors that are contiguous but start at an odd element offset (views into a larger buffer) are
not 16-byte aligned: the tensor-core paths cannot take them, and the C ABI must route them to the
element-wise scan kernels instead of faulting."""
import pytest
import torch

from helpers import GRAD_TOL, OUT_TOL, dfw_inputs, lfw_inputs, max_rel_err, to_dev
from oracle import fw_oracle

pytestmark = pytest.mark.gpu


def _offset_view(t, off):
    """A contiguous tensor with t's values whose storage starts `off` elements into a buffer."""
    buf = torch.empty(t.numel() + 8, dtype=t.dtype, device=t.device)
    v = buf[off:off + t.numel()].view(t.shape)
    v.copy_(t)
    assert v.is_contiguous() and v.data_ptr() % 16 != 0
    return v


@pytest.mark.parametrize("which", [0, 4, 5])
def test_lfw_unaligned_views_take_the_scan_path(cuda, which):
    from t2fw_b200 import _lib, cabi

    dev = to_dev(lfw_inputs(3, 200, 64, 64, "sigmoid", 0.3, 95), torch.float16, cuda)
    dev[which] = _offset_view(dev[which], 1)       # x, f_key or the state
    x, f, q, k, fk, s, go, gs = dev
    n0 = _lib.load_core().t2fw_launch_count()
    out, ckpt = cabi.lfw_forward(x, f, q, k, fk, s)
    grads = cabi.lfw_backward(go, gs, x, f, q, k, fk, s, ckpt)
    torch.cuda.synchronize()
    assert _lib.load_core().t2fw_launch_count() - n0 == 3      # one scan forward + two scan backward launches
    r_out, r_fin = fw_oracle.lfw_forward(x, f, q, k, fk, s)
    r_grads = fw_oracle.lfw_backward(go, gs, x, f, q, k, fk, s)
    assert max_rel_err(out, r_out) <= OUT_TOL[torch.float16]
    assert max_rel_err(ckpt[:, -1], r_fin) <= OUT_TOL[torch.float16]
    for g, r in zip(grads, r_grads):
        assert max_rel_err(g, r) <= GRAD_TOL[torch.float16]


def test_dfw_unaligned_views_take_the_scan_path(cuda):
    from t2fw_b200 import cabi

    q, k, v, s, go, gs = to_dev(dfw_inputs(3, 150, 64, 64, "scaled", 0.3, 96), torch.float16, cuda)
    q = _offset_view(q, 1)
    go = _offset_view(go, 3)
    out, fin, delta = cabi.dfw_forward(q, k, v, s)
    grads = cabi.dfw_backward(go, gs, q, k, delta, fin)
    torch.cuda.synchronize()
    r_out, r_fin, _ = fw_oracle.dfw_forward(q, k, v, s)
    r_grads = fw_oracle.dfw_backward(go, gs, q, k, v, s)
    assert max_rel_err(out, r_out) <= OUT_TOL[torch.float16]
    assert max_rel_err(fin, r_fin) <= OUT_TOL[torch.float16]
    for g, r in zip(grads, r_grads):
        assert max_rel_err(g, r) <= GRAD_TOL[torch.float16]
