"""Shared test helpers: seeded inputs, the error metric, golden-vector loading."""
import glob
import importlib.util
import math
import os

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
GOLDEN = os.path.join(HERE, "golden")

_spec = importlib.util.spec_from_file_location("make_golden", os.path.join(GOLDEN, "make_golden.py"))
make_golden = importlib.util.module_from_spec(_spec)
_spec.loader.exec_module(make_golden)
lfw_inputs = make_golden.lfw_inputs      # (B,T,D,K,gates,state_std,seed) -> x,f,q,k,fk,s,go,gs
dfw_inputs = make_golden.dfw_inputs      # (B,T,D,M,keys,state_std,seed)  -> q,k,v,s,go,gs

# "max relative error": largest absolute deviation over the largest reference magnitude
OUT_TOL = {torch.float16: 1e-2, torch.bfloat16: 4e-2, torch.float32: 2e-4, torch.float64: 1e-9}
GRAD_TOL = {torch.float16: 2e-2, torch.bfloat16: 6e-2, torch.float32: 5e-4, torch.float64: 1e-9}


def max_rel_err(got, ref):
    got = np.asarray(got.detach().double().cpu() if hasattr(got, "detach") else got, dtype=np.float64)
    ref = np.asarray(ref.detach().double().cpu() if hasattr(ref, "detach") else ref, dtype=np.float64)
    assert got.shape == ref.shape, (got.shape, ref.shape)
    if not np.isfinite(got).all():
        return float("inf")
    return float(np.abs(got - ref).max() / max(np.abs(ref).max(), 1e-30))


def golden_files(prefix):
    return sorted(glob.glob(os.path.join(GOLDEN, prefix + "*.npz")))


def load_golden(path):
    with np.load(path) as z:
        return {k: z[k] for k in z.files}


def to_dev(arrs, dtype, device):
    return [torch.as_tensor(np.asarray(a)).to(dtype).to(device).contiguous() for a in arrs]
