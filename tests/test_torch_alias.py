"""`t2fw.torch` (the reference's eager/TorchScript module, t2fw/torch.py:10-16,35-39,59-67,148-156):
the four functions exist under the reference's import path with its argument order, and reproduce
the golden vectors that were generated from the reference itself.  CPU only."""
import numpy as np
import pytest
import torch

from helpers import golden_files, load_golden, max_rel_err


def _t(g, names):
    return [torch.as_tensor(g[n]) for n in names]


@pytest.mark.parametrize("path", golden_files("lfw_"), ids=lambda p: p.split("/")[-1][:-4])
def test_t2fw_torch_reproduces_reference_results(path):
    from t2fw.torch import t2fw_torch

    g = load_golden(path)
    leaves = [t.requires_grad_(True) for t in _t(g, ("x", "f", "q", "k", "f_key", "state"))]
    out, fin = t2fw_torch(*leaves)
    assert max_rel_err(out, g["out"]) <= 1e-5 and max_rel_err(fin, g["final_state"]) <= 1e-5
    grads = torch.autograd.grad([out, fin], leaves, _t(g, ("grad_out", "grad_state")))
    for got, n in zip(grads, ("d_x", "d_f", "d_q", "d_k", "d_f_key", "d_state")):
        assert max_rel_err(got, g[n]) <= 1e-4, n


@pytest.mark.parametrize("path", golden_files("dfw_"), ids=lambda p: p.split("/")[-1][:-4])
def test_t2dfw_functions_reproduce_reference_results(path):
    from t2fw.torch import t2dfw_torch, t2dfw_torch_bw, t2dfw_torch_bw_simple

    g = load_golden(path)
    q, k, v, s = _t(g, ("q", "k", "v", "state"))
    go, gs = _t(g, ("grad_out", "grad_state"))
    out, fin = t2dfw_torch(q, k, v, s)
    assert max_rel_err(out, g["out"]) <= 1e-5 and max_rel_err(fin, g["final_state"]) <= 1e-5
    for fn in (t2dfw_torch_bw, t2dfw_torch_bw_simple):
        grads = fn(go, gs, q, k, v, s, fin)
        for got, n in zip(grads, ("d_q", "d_k", "d_v", "d_state")):
            assert max_rel_err(got, g[n]) <= 2e-4, (fn.__name__, n)
