"""Recipe for oracle/_ref: the reference's own CPU implementation of the path, taken from where it
lies, for use as the timed CPU baseline and as a cross-check of the restatements in this folder.

The reference is pure Python on this path (`t2fw/torch.py`: TorchScript loops over time), so
"building" it is placing that one module under oracle/_ref/t2fw/ where it can be imported without
the rest of the reference (whose package imports JIT-compile CUDA sources).  oracle/_ref/ is
git-ignored: nothing of the reference is committed; the folder travels to the GPU machine like the
other build outputs.  Test infrastructure only.

    python -m oracle.make_ref [/path/to/reference]

Without an argument the reference is looked for in $T2FW_REFERENCE_ROOT, then in a folder named
`reference` beside this repository.
"""
import os
import shutil
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
REF_DIR = os.path.join(HERE, "_ref")


def default_reference_root() -> str:
    return os.environ.get("T2FW_REFERENCE_ROOT") or os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")


def build(reference_root: str = "") -> str:
    """Returns the path of oracle/_ref/t2fw/torch.py, or "" if the reference is not present."""
    src = os.path.join(reference_root or default_reference_root(), "t2fw", "torch.py")
    if not os.path.exists(src):
        return ""
    dst_dir = os.path.join(REF_DIR, "t2fw")
    os.makedirs(dst_dir, exist_ok=True)
    dst = os.path.join(dst_dir, "torch.py")
    shutil.copyfile(src, dst)
    open(os.path.join(dst_dir, "__init__.py"), "w").close()
    return dst


def load():
    """The reference module `t2fw.torch` from oracle/_ref, or None if it was not built."""
    path = os.path.join(REF_DIR, "t2fw", "torch.py")
    if not os.path.exists(path):
        return None
    import importlib.util

    spec = importlib.util.spec_from_file_location("t2fw_reference_torch", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


if __name__ == "__main__":
    print(build(*sys.argv[1:2]) or "reference not found")
