"""The CPU oracle (C restatement and the PyTorch port) against golden vectors produced by the
reference's own TorchScript functions (tests/golden/make_golden.py)."""
import numpy as np
import pytest
import torch

from oracle import fw_oracle, torch_port
from helpers import golden_files, load_golden, max_rel_err

TOL = 5e-6  # float32 reference vs float64 oracle


@pytest.mark.parametrize("path", golden_files("lfw_"), ids=lambda p: p.split("/")[-1][:-4])
def test_lfw_c_oracle_matches_reference(path):
    g = load_golden(path)
    out, fin = fw_oracle.lfw_forward(g["x"], g["f"], g["q"], g["k"], g["f_key"], g["state"])
    assert max_rel_err(out, g["out"]) < TOL
    assert max_rel_err(fin, g["final_state"]) < TOL
    grads = fw_oracle.lfw_backward(g["grad_out"], g["grad_state"], g["x"], g["f"], g["q"], g["k"],
                                   g["f_key"], g["state"])
    for got, name in zip(grads, ("d_x", "d_f", "d_q", "d_k", "d_f_key", "d_state")):
        assert max_rel_err(got, g[name]) < TOL, name


@pytest.mark.parametrize("path", golden_files("dfw_"), ids=lambda p: p.split("/")[-1][:-4])
def test_dfw_c_oracle_matches_reference(path):
    g = load_golden(path)
    out, fin, _ = fw_oracle.dfw_forward(g["q"], g["k"], g["v"], g["state"])
    assert max_rel_err(out, g["out"]) < TOL
    assert max_rel_err(fin, g["final_state"]) < TOL
    grads = fw_oracle.dfw_backward(g["grad_out"], g["grad_state"], g["q"], g["k"], g["v"], g["state"])
    for got, name in zip(grads, ("d_q", "d_k", "d_v", "d_state")):
        assert max_rel_err(got, g[name]) < TOL, name


@pytest.mark.parametrize("path", golden_files("lfw_config1") + golden_files("lfw_odd"),
                         ids=lambda p: p.split("/")[-1][:-4])
def test_lfw_torch_port_matches_reference(path):
    g = {k: torch.from_numpy(v) for k, v in load_golden(path).items()}
    out, fin, grads = torch_port.lfw_fwd_bwd(g["x"], g["f"], g["q"], g["k"], g["f_key"], g["state"],
                                             g["grad_out"], g["grad_state"])
    assert max_rel_err(out, g["out"]) < TOL
    assert max_rel_err(fin, g["final_state"]) < TOL
    for got, name in zip(grads, ("d_x", "d_f", "d_q", "d_k", "d_f_key", "d_state")):
        assert max_rel_err(got, g[name]) < TOL, name


@pytest.mark.parametrize("path", golden_files("dfw_config1") + golden_files("dfw_odd"),
                         ids=lambda p: p.split("/")[-1][:-4])
def test_dfw_torch_port_matches_reference(path):
    g = {k: torch.from_numpy(v) for k, v in load_golden(path).items()}
    out, fin, grads = torch_port.dfw_fwd_bwd(g["q"], g["k"], g["v"], g["state"], g["grad_out"],
                                             g["grad_state"])
    assert max_rel_err(out, g["out"]) < TOL
    assert max_rel_err(fin, g["final_state"]) < TOL
    for got, name in zip(grads, ("d_q", "d_k", "d_v", "d_state")):
        assert max_rel_err(got, g[name]) < TOL, name


def test_oracle_segmented_backward_crosses_segments():
    """T larger than the oracle's internal segment length gives the same gradients as autograd."""
    from helpers import lfw_inputs
    x, f, q, k, fk, s, go, gs = lfw_inputs(1, 300, 5, 3, "sigmoid", 0.5, 7)
    args = [t.double() for t in (x, f, q, k, fk, s)]
    _, _, grads = torch_port.lfw_fwd_bwd(*args, go.double(), gs.double())
    got = fw_oracle.lfw_backward(go, gs, x, f, q, k, fk, s)
    for a, b in zip(got, grads):
        assert max_rel_err(a, b) < 1e-10
