"""oracle/_ref (the reference's own CPU module, placed there by oracle/make_ref.py) agrees with the
golden vectors and with the port that stands in for it where it is absent.  Skipped when
oracle/_ref has not been built (the reference is not present on every machine)."""
import pytest
import torch

from helpers import golden_files, load_golden, max_rel_err
from oracle import make_ref, torch_port


@pytest.fixture(scope="module")
def ref():
    mod = make_ref.load()
    if mod is None:
        pytest.skip("oracle/_ref not built")
    return mod


def test_reference_module_reproduces_golden_vectors(ref):
    g = load_golden(golden_files("lfw_config1_raw")[0])
    ins = [torch.as_tensor(g[n]) for n in ("x", "f", "q", "k", "f_key", "state")]
    out, fin = ref.t2fw_torch(*ins)
    assert max_rel_err(out, g["out"]) <= 1e-6 and max_rel_err(fin, g["final_state"]) <= 1e-6
    p_out, p_fin = torch_port.lfw_loop(*ins)
    assert max_rel_err(p_out, out) <= 1e-5 and max_rel_err(p_fin, fin) <= 1e-5
    g = load_golden(golden_files("dfw_config1_scaled")[0])
    ins = [torch.as_tensor(g[n]) for n in ("q", "k", "v", "state")]
    out, fin = ref.t2dfw_torch(*ins)
    assert max_rel_err(out, g["out"]) <= 1e-6 and max_rel_err(fin, g["final_state"]) <= 1e-6
