"""The C-ABI library loads without a GPU and exports every symbol the header declares."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_functions():
    names = []
    inc = os.path.join(ROOT, "include")
    for fn in sorted(os.listdir(inc)):
        if not fn.endswith(".h"):
            continue
        text = open(os.path.join(inc, fn)).read()
        text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
        names += re.findall(r"\b(t2fw_[a-z0-9_]+)\s*\(", text)
    return sorted(set(names))


def test_header_declares_the_hot_path():
    names = declared_functions()
    for need in ("t2fw_lfw_forward", "t2fw_lfw_backward", "t2fw_dfw_forward", "t2fw_dfw_backward"):
        assert need in names


def test_library_exports_every_declared_symbol():
    from t2fw_b200 import _lib

    lib = ctypes.CDLL(_lib.CORE_PATH)
    for name in declared_functions():
        assert hasattr(lib, name), name
    assert set(declared_functions()) >= set(_lib.EXPORTS)


def test_library_is_not_an_instrumented_build():
    """The clock-counter instrumentation of the kernels (compile-time macros) exports debug entry
    points; a library built that way is slower and must not be the one that ships."""
    from t2fw_b200 import _lib

    lib = ctypes.CDLL(_lib.CORE_PATH)
    for name in ("t2fw_debug_prof", "t2fw_debug_dfw_prof", "t2fw_debug_c64_prof", "t2fw_debug_loc_prof"):
        assert not hasattr(lib, name), name + ": rebuild without the profiling macro"


def test_cheap_entry_points_run_without_gpu():
    from t2fw_b200 import _lib

    lib = _lib.load_core()
    assert lib.t2fw_version() >= 100
    assert lib.t2fw_lfw_ckpt_slots(1024, 64) == 16
    assert lib.t2fw_lfw_ckpt_slots(385, 64) == 7
    assert lib.t2fw_lfw_ckpt_slots(1, 64) == 1
    assert lib.t2fw_lfw_default_ckpt_every(1024, 64, 64, 0) == 64
    assert lib.t2fw_lfw_default_ckpt_every(16384, 128, 128, 0) == 64
    assert lib.t2fw_dfw_backward_scratch_bytes(2, 8, 4, 4, 0) == 256
    assert lib.t2fw_dfw_backward_scratch_bytes(2, 8, 4, 4, 2) == 0


def test_bad_arguments_are_rejected_before_any_launch():
    from t2fw_b200 import _lib

    lib = _lib.load_core()
    rc = lib.t2fw_lfw_forward(None, None, None, None, None, None, None, None, 1, 1, 1, 1, 0, 64,
                              None, 0, None)
    assert rc == 1 and b"null" in lib.t2fw_last_error()
    rc = lib.t2fw_lfw_forward(None, None, None, None, None, None, None, None, 1, 0, 1, 1, 0, 64,
                              None, 0, None)
    assert rc == 1 and b"positive" in lib.t2fw_last_error()
    rc = lib.t2fw_dfw_forward(None, None, None, None, None, None, None, 1, 1, 1, 1, 9, None)
    assert rc == 1 and b"dtype" in lib.t2fw_last_error()
