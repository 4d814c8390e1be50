"""Ahead-of-time build of the native libraries, in-tree.

  lib/libt2fw_b200.so     CUDA kernels + the C ABI (include/t2fw_b200.h); nvcc, sm_100a only
  lib/t2fw_torch_ops.so   the PyTorch operator library (torch.ops.lfw / torch.ops.dfw), a thin
                          C++ adapter that links against the former

Run `python -m t2fw_b200.build` (add --force to rebuild everything).  nvcc cross-compiles
without a GPU.  Nothing is JIT-compiled at import time: the .so files must exist.
"""
import glob
import os
import subprocess
import sys

PKG = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(PKG)
CSRC = os.path.join(PKG, "csrc")
LIB_DIR = os.path.join(PKG, "lib")
OBJ_DIR = os.path.join(PKG, "lib", "obj")
CORE_LIB = os.path.join(LIB_DIR, "libt2fw_b200.so")
OPS_LIB = os.path.join(LIB_DIR, "t2fw_torch_ops.so")

NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "--expt-relaxed-constexpr", "-Xcompiler", "-fPIC", "-Xptxas", "-v",
]


def _newer(target, deps):
    if not os.path.exists(target):
        return False
    t = os.path.getmtime(target)
    return all(os.path.getmtime(d) <= t for d in deps)


def _run(cmd, log=None):
    res = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if log is not None:
        with open(log, "w") as fh:
            fh.write(" ".join(cmd) + "\n" + res.stdout)
    if res.returncode != 0:
        sys.stderr.write(res.stdout)
        raise RuntimeError("build step failed: " + " ".join(cmd))
    return res.stdout


def build_core(force=False, verbose=False):
    os.makedirs(OBJ_DIR, exist_ok=True)
    headers = glob.glob(os.path.join(CSRC, "*.cuh")) + glob.glob(os.path.join(ROOT, "include", "*.h"))
    objs = []
    procs = []
    for src in sorted(glob.glob(os.path.join(CSRC, "*.cu"))):
        obj = os.path.join(OBJ_DIR, os.path.basename(src)[:-3] + ".o")
        objs.append(obj)
        if not force and _newer(obj, [src] + headers):
            continue
        cmd = [NVCC] + NVCC_FLAGS + ["-c", src, "-o", obj]
        if verbose:
            print(" ".join(cmd))
        procs.append((cmd, obj, subprocess.Popen(cmd, stdout=subprocess.PIPE,
                                                 stderr=subprocess.STDOUT, text=True)))
    for cmd, obj, p in procs:
        out, _ = p.communicate()
        with open(obj + ".log", "w") as fh:
            fh.write(" ".join(cmd) + "\n" + out)
        if p.returncode != 0:
            sys.stderr.write(out)
            raise RuntimeError("nvcc failed: " + " ".join(cmd))
    if force or procs or not _newer(CORE_LIB, objs):
        _run([NVCC, "-shared", "-o", CORE_LIB] + objs + ["-gencode", "arch=compute_100a,code=sm_100a"])
    return CORE_LIB


def build_ops(force=False, verbose=False):
    import torch
    from torch.utils import cpp_extension

    src = os.path.join(CSRC, "torch_ops.cpp")
    deps = [src, os.path.join(ROOT, "include", "t2fw_b200.h")]
    if not force and _newer(OPS_LIB, deps) and _newer(OPS_LIB, [CORE_LIB]):
        return OPS_LIB
    tlib = os.path.join(os.path.dirname(torch.__file__), "lib")
    inc = []
    for p in cpp_extension.include_paths(device_type="cuda"):
        inc += ["-isystem", p]
    abi = int(torch._C._GLIBCXX_USE_CXX11_ABI)
    cmd = (["g++", "-O2", "-std=c++17", "-fPIC", "-shared", "-D_GLIBCXX_USE_CXX11_ABI=%d" % abi,
            "-DTORCH_API_INCLUDE_EXTENSION_H", src, "-o", OPS_LIB, "-I", os.path.join(ROOT, "include")]
           + inc + ["-L", tlib, "-L", LIB_DIR, "-L", "/usr/local/cuda/lib64",
                    "-lt2fw_b200", "-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch_cuda", "-ltorch",
                    "-Wl,-rpath,$ORIGIN", "-Wl,-rpath," + tlib])
    if verbose:
        print(" ".join(cmd))
    _run(cmd, log=os.path.join(OBJ_DIR, "torch_ops.log"))
    return OPS_LIB


def build_all(force=False, verbose=False):
    build_core(force=force, verbose=verbose)
    build_ops(force=force, verbose=verbose)
    return CORE_LIB, OPS_LIB


if __name__ == "__main__":
    print(build_all(force="--force" in sys.argv, verbose=True))
