"""The give-up path of the kernels' bounded waits.  A kernel that waits on a barrier nothing
arrives on (and has nothing else in flight) must return, report through the status word that
`t2fw_device_status` reads, and leave the context usable.  Runs in a child process because the
status word is sticky for the life of the process."""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu

HERE = os.path.dirname(os.path.abspath(__file__))

CHILD = r"""
import sys
sys.path.insert(0, {root!r}); sys.path.insert(0, {tests!r})
import ctypes, torch
from helpers import OUT_TOL, lfw_inputs, max_rel_err, to_dev
from oracle import fw_oracle
from t2fw_b200 import _lib, cabi
lib = _lib.load_core()
dev = torch.device("cuda:0")
fn = lib.t2fw_selftest_bounded_wait
fn.restype = ctypes.c_int
fn.argtypes = [ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p]
ins = to_dev(lfw_inputs(2, 200, 64, 64, "sigmoid", 0.3, 97), torch.float16, dev)
out, ckpt = cabi.lfw_forward(*ins[:6])            # first call: status word set up, still clean
torch.cuda.synchronize()
assert lib.t2fw_device_status() == 0
own = torch.zeros(1, dtype=torch.int32, device=dev)
assert fn(8, own.data_ptr(), None) == 0            # the wait runs out after 8 polls
torch.cuda.synchronize()
assert int(own.item()) == 1 and lib.t2fw_device_status() == 0
assert fn(8, None, None) == 0                      # same, reported through the library's status word
torch.cuda.synchronize()
assert lib.t2fw_device_status() != 0
out2, ckpt2 = cabi.lfw_forward(*ins[:6])          # the context is still usable and results are right
torch.cuda.synchronize()
r_out, r_fin = fw_oracle.lfw_forward(*ins[:6])
assert max_rel_err(out2, r_out) <= OUT_TOL[torch.float16] and torch.equal(out, out2)
print("ok")
"""


def test_expired_wait_reports_and_returns(cuda):
    code = CHILD.format(tests=HERE, root=os.path.dirname(HERE))
    r = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-4000:]
    assert "ok" in r.stdout
