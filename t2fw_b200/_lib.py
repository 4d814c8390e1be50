"""Loading of the two native libraries.

  load_core() -> ctypes.CDLL of libt2fw_b200.so, the C ABI declared in include/t2fw_b200.h
  load_ops()  -> registers torch.ops.lfw / torch.ops.dfw from t2fw_torch_ops.so

Both fail loudly (ImportError) when the library has not been built: nothing falls back to a
slower path.
"""
import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
CORE_PATH = os.path.join(_HERE, "lib", "libt2fw_b200.so")
OPS_PATH = os.path.join(_HERE, "lib", "t2fw_torch_ops.so")

# every entry point include/t2fw_b200.h declares
EXPORTS = (
    "t2fw_last_error", "t2fw_version", "t2fw_launch_count", "t2fw_device_status",
    "t2fw_lfw_default_ckpt_every", "t2fw_lfw_ckpt_slots",
    "t2fw_lfw_forward_scratch_bytes", "t2fw_lfw_backward_scratch_bytes",
    "t2fw_dfw_backward_scratch_bytes",
    "t2fw_lfw_forward", "t2fw_lfw_backward", "t2fw_dfw_forward", "t2fw_dfw_backward",
    "t2fw_dfw_forward_ws", "t2fw_dfw_forward_scratch_bytes",
    "t2fw_dfw_backward_noalloc_max_elems", "t2fw_dfw_backward_noalloc",
    "t2fw_lfw_fused_scratch_bytes", "t2fw_lfw_fused_forward", "t2fw_lfw_fused_backward",
    "t2fw_lfw_segment_summary_scratch_bytes", "t2fw_lfw_segment_summary", "t2fw_lfw_fold_summaries",
)

_core = None
_ops_loaded = False

_i64 = ctypes.c_int64
_vp = ctypes.c_void_p
_int = ctypes.c_int
_sz = ctypes.c_size_t


def load_core():
    global _core
    if _core is not None:
        return _core
    if not os.path.exists(CORE_PATH):
        raise ImportError(
            "t2fw_b200: %s is missing; build it with `python -m t2fw_b200.build`" % CORE_PATH)
    lib = ctypes.CDLL(CORE_PATH, mode=ctypes.RTLD_GLOBAL)
    lib.t2fw_last_error.restype = ctypes.c_char_p
    lib.t2fw_last_error.argtypes = []
    lib.t2fw_version.restype = _int
    lib.t2fw_launch_count.restype = _i64
    lib.t2fw_device_status.restype = _int
    lib.t2fw_device_status.argtypes = []
    lib.t2fw_lfw_default_ckpt_every.restype = _i64
    lib.t2fw_lfw_default_ckpt_every.argtypes = [_i64, _i64, _i64, _int]
    lib.t2fw_lfw_ckpt_slots.restype = _i64
    lib.t2fw_lfw_ckpt_slots.argtypes = [_i64, _i64]
    for name in ("t2fw_lfw_forward_scratch_bytes", "t2fw_lfw_backward_scratch_bytes"):
        fn = getattr(lib, name)
        fn.restype = _sz
        fn.argtypes = [_i64, _i64, _i64, _i64, _int, _i64]
    lib.t2fw_dfw_backward_scratch_bytes.restype = _sz
    lib.t2fw_dfw_backward_scratch_bytes.argtypes = [_i64, _i64, _i64, _i64, _int]
    lib.t2fw_dfw_forward_scratch_bytes.restype = _sz
    lib.t2fw_dfw_forward_scratch_bytes.argtypes = [_i64, _i64, _i64, _i64, _int]
    lib.t2fw_dfw_forward_ws.restype = _int
    lib.t2fw_dfw_forward_ws.argtypes = [_vp] * 7 + [_i64] * 4 + [_int, _vp, _sz, _vp]
    lib.t2fw_lfw_forward.restype = _int
    lib.t2fw_lfw_forward.argtypes = [_vp] * 8 + [_i64] * 4 + [_int, _i64, _vp, _sz, _vp]
    lib.t2fw_lfw_backward.restype = _int
    lib.t2fw_lfw_backward.argtypes = [_vp] * 15 + [_i64] * 4 + [_int, _i64, _vp, _sz, _vp]
    lib.t2fw_dfw_forward.restype = _int
    lib.t2fw_dfw_forward.argtypes = [_vp] * 7 + [_i64] * 4 + [_int, _vp]
    lib.t2fw_dfw_backward.restype = _int
    lib.t2fw_dfw_backward.argtypes = [_vp] * 10 + [_i64] * 4 + [_int, _vp, _sz, _vp]
    lib.t2fw_dfw_backward_noalloc_max_elems.restype = _sz
    lib.t2fw_dfw_backward_noalloc_max_elems.argtypes = []
    lib.t2fw_dfw_backward_noalloc.restype = _int
    lib.t2fw_dfw_backward_noalloc.argtypes = [_vp] * 10 + [_i64] * 4 + [_int, _vp]
    lib.t2fw_lfw_fused_scratch_bytes.restype = _sz
    lib.t2fw_lfw_fused_scratch_bytes.argtypes = [_i64, _i64, _i64, _int]
    lib.t2fw_lfw_fused_forward.restype = _int
    lib.t2fw_lfw_fused_forward.argtypes = [_vp] * 4 + [_i64] * 3 + [_int, _vp, _sz, _vp]
    lib.t2fw_lfw_fused_backward.restype = _int
    lib.t2fw_lfw_fused_backward.argtypes = [_vp] * 7 + [_i64] * 3 + [_int, _vp, _sz, _vp]
    _core = lib
    return lib


def load_ops():
    global _ops_loaded
    if _ops_loaded:
        return
    import torch

    if not os.path.exists(OPS_PATH):
        raise ImportError(
            "t2fw_b200: %s is missing; build it with `python -m t2fw_b200.build`" % OPS_PATH)
    load_core()
    torch.ops.load_library(OPS_PATH)
    _ops_loaded = True
