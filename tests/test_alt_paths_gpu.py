"""The kernel families that environment switches select instead of the default ones stay
parity-green: each case runs in a child process (the switches are read once per process) and
checks one delta-rule and one decay-rule problem against the oracle."""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu

HERE = os.path.dirname(os.path.abspath(__file__))

CHILD = r"""
import sys, torch
sys.path.insert(0, {tests!r}); sys.path.insert(0, {root!r})
from helpers import GRAD_TOL, OUT_TOL, dfw_inputs, lfw_inputs, max_rel_err, to_dev
from oracle import fw_oracle
from t2fw_b200 import cabi
dev = torch.device("cuda:0")
dt = torch.float16
# delta rule, D = M = 64: whole and partial chunks, non-zero initial state
q, k, v, s, go, gs = to_dev(dfw_inputs(2, 200, 64, 64, "scaled", 0.3, 77), dt, dev)
out, fin, delta = cabi.dfw_forward(q, k, v, s)
grads = cabi.dfw_backward(go, gs, q, k, delta, fin)
torch.cuda.synchronize()
r_out, r_fin, _ = fw_oracle.dfw_forward(q, k, v, s)
r_grads = fw_oracle.dfw_backward(go, gs, q, k, v, s)
assert max_rel_err(out, r_out) <= OUT_TOL[dt] and max_rel_err(fin, r_fin) <= OUT_TOL[dt]
for g, r in zip(grads, r_grads):
    assert max_rel_err(g, r) <= GRAD_TOL[dt]
# decay rule, D = K = 64, forward and backward
ins = to_dev(lfw_inputs(2, 200, 64, 64, "sigmoid", 0.3, 78), dt, dev)
x, f, qq, kk, fk, st, go2, gs2 = ins
out2, ckpt = cabi.lfw_forward(x, f, qq, kk, fk, st)
grads2 = cabi.lfw_backward(go2, gs2, x, f, qq, kk, fk, st, ckpt)
torch.cuda.synchronize()
o_out, o_fin = fw_oracle.lfw_forward(x, f, qq, kk, fk, st)
o_grads = fw_oracle.lfw_backward(go2, gs2, x, f, qq, kk, fk, st)
assert max_rel_err(out2, o_out) <= OUT_TOL[dt] and max_rel_err(ckpt[:, -1], o_fin) <= OUT_TOL[dt]
for g, r in zip(grads2, o_grads):
    assert max_rel_err(g, r) <= GRAD_TOL[dt]
from t2fw_b200._lib import load_core
assert load_core().t2fw_device_status() == 0
print("ok")
"""


@pytest.mark.parametrize("switch", ["T2FW_DISABLE_DFW_UMMA", "T2FW_DISABLE_DFW_CHUNK", "T2FW_DISABLE_CHUNK", "T2FW_DISABLE_PDL"])
def test_switched_path_matches_oracle(cuda, switch):
    env = dict(os.environ)
    env[switch] = "1"
    code = CHILD.format(tests=HERE, root=os.path.dirname(HERE))
    r = subprocess.run([sys.executable, "-c", code], env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-4000:]
    assert "ok" in r.stdout
