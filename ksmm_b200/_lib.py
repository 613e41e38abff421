"""ctypes binding of libksmm_cu.so (the C ABI declared in include/ksmm_cu.h).

The library is built in-tree by ``ksmm_b200.build.build_library()`` (nvcc,
sm_100a only).  There is no CPU fallback: if the shared object is missing the
import of any operator fails with an explicit error.
"""
from __future__ import annotations

import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libksmm_cu.so")

# enum values of include/ksmm_cu.h
KSMM_OK = 0
KSMM_ERR_BAD_ARGUMENT = 1
KSMM_ERR_UNSUPPORTED = 2
KSMM_ERR_CUDA = 3
KSMM_ERR_WORKSPACE = 4
KSMM_ERR_DEVICE_TIMEOUT = 5
KSMM_ERR_NO_DEVICE = 6

KSMM_F32, KSMM_F16, KSMM_BF16, KSMM_F8E4M3 = 0, 1, 2, 3
KSMM_ALGO_AUTO, KSMM_ALGO_SIMT, KSMM_ALGO_TC, KSMM_ALGO_CONVERT = 0, 1, 2, 3
KSMM_ACT_NONE, KSMM_ACT_GELU, KSMM_ACT_RELU = 0, 1, 2
ACTIVATIONS = {None: KSMM_ACT_NONE, "none": KSMM_ACT_NONE, "gelu": KSMM_ACT_GELU, "relu": KSMM_ACT_RELU}
STATIC_SCRATCH_BYTES = 40 * 1024 * 1024  # KSMM_CU_STATIC_SCRATCH_BYTES

EXPORTS = (
    "ksmm_cu_version", "ksmm_cu_last_error", "ksmm_cu_status_string", "ksmm_cu_forward",
    "ksmm_cu_forward_ex", "ksmm_cu_chain_workspace_bytes", "ksmm_cu_chain_forward", "ksmm_cu_chain_forward_act",
    "ksmm_cu_chain_forward_static", "ksmm_cu_chain_forward_host", "ksmm_cu_num_configs", "ksmm_cu_config_supported",
    "ksmm_cu_tune", "ksmm_cu_set_choice", "ksmm_cu_get_choice", "ksmm_cu_default_choice",
    "ksmm_cu_check_device",
    "ksmm_cu_launch_count", "ksmm_cu_measure_ffma_peak",
    "ksmm_cu_layout_scratch_bytes", "ksmm_cu_release_scratch", "ksmm_cu_chain_workspace_bytes_ex",
    "ksmm_cu_alloc_count", "ksmm_cu_debug_wait_probe",
    "ksmm_cu_chain_forward_host_async", "ksmm_cu_host_wait", "ksmm_cu_clear_choice",
    "ksmm_cu_grouped_forward", "ksmm_cu_grouped_chain_forward",
    "ksmm_cu_chain_workspace_bytes_layouts", "ksmm_cu_chain_forward_layouts", "ksmm_cu_chain_forward_desc",
    "ksmm_cu_backward_input_workspace_bytes", "ksmm_cu_backward_input",
    "ksmm_cu_backward_weights_workspace_bytes", "ksmm_cu_backward_weights",
)


class ForwardDesc(ctypes.Structure):
    """Mirror of ksmm_forward_desc_t."""
    _fields_ = [
        ("input", ctypes.c_void_p), ("values", ctypes.c_void_p), ("output", ctypes.c_void_p),
        ("bias", ctypes.c_void_p), ("batch", ctypes.c_int64),
        ("a", ctypes.c_int32), ("b", ctypes.c_int32), ("c", ctypes.c_int32), ("d", ctypes.c_int32),
        ("in_dtype", ctypes.c_int32), ("out_dtype", ctypes.c_int32), ("bs_last", ctypes.c_int32),
        ("algo", ctypes.c_int32), ("config", ctypes.c_int32), ("alpha", ctypes.c_float),
        ("activation", ctypes.c_int32),
        ("scratch", ctypes.c_void_p), ("scratch_bytes", ctypes.c_size_t),
        ("residual", ctypes.c_void_p),
    ]


class ChainDesc(ctypes.Structure):
    """Mirror of ksmm_chain_desc_t."""
    _fields_ = [
        ("input", ctypes.c_void_p), ("values", ctypes.POINTER(ctypes.c_void_p)), ("output", ctypes.c_void_p),
        ("bias", ctypes.c_void_p), ("residual", ctypes.c_void_p), ("workspace", ctypes.c_void_p),
        ("workspace_bytes", ctypes.c_size_t), ("batch", ctypes.c_int64), ("nfactors", ctypes.c_int32),
        ("patterns", ctypes.POINTER(ctypes.c_int32)), ("dtype", ctypes.c_int32), ("bs_last", ctypes.c_int32),
        ("out_layout", ctypes.c_int32), ("activation", ctypes.c_int32),
    ]


class KsmmError(RuntimeError):
    def __init__(self, status, message):
        super().__init__(f"libksmm_cu status {status}: {message}")
        self.status = status


_lib = None


def load():
    """Load libksmm_cu.so once and declare every prototype."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python -m ksmm_b200.build` "
            "(nvcc, sm_100a).  There is no CPU or PyTorch fallback for algo='kernel'.")
    lib = ctypes.CDLL(LIB_PATH)
    vp, i32, i64 = ctypes.c_void_p, ctypes.c_int, ctypes.c_int64
    lib.ksmm_cu_version.restype = i32
    lib.ksmm_cu_last_error.restype = ctypes.c_char_p
    lib.ksmm_cu_status_string.restype = ctypes.c_char_p
    lib.ksmm_cu_status_string.argtypes = [i32]
    lib.ksmm_cu_forward.restype = i32
    lib.ksmm_cu_forward.argtypes = [vp, vp, vp, i64, i32, i32, i32, i32, i32, i32, vp]
    lib.ksmm_cu_forward_ex.restype = i32
    lib.ksmm_cu_forward_ex.argtypes = [ctypes.POINTER(ForwardDesc), vp]
    lib.ksmm_cu_chain_workspace_bytes.restype = ctypes.c_size_t
    lib.ksmm_cu_chain_workspace_bytes.argtypes = [i32, ctypes.POINTER(ctypes.c_int32), i64, i32]
    lib.ksmm_cu_chain_forward.restype = i32
    lib.ksmm_cu_chain_forward.argtypes = [vp, ctypes.POINTER(vp), vp, vp, vp, ctypes.c_size_t, i64,
                                          i32, ctypes.POINTER(ctypes.c_int32), i32, i32, vp]
    lib.ksmm_cu_chain_forward_act.restype = i32
    lib.ksmm_cu_chain_forward_act.argtypes = [vp, ctypes.POINTER(vp), vp, vp, vp, ctypes.c_size_t, i64,
                                              i32, ctypes.POINTER(ctypes.c_int32), i32, i32, i32, vp]
    lib.ksmm_cu_chain_forward_static.restype = i32
    lib.ksmm_cu_chain_forward_static.argtypes = [vp, ctypes.POINTER(vp), vp, vp, i64, i32,
                                                 ctypes.POINTER(ctypes.c_int32), i32, i32, vp]
    lib.ksmm_cu_chain_forward_host.restype = i32
    lib.ksmm_cu_chain_forward_host.argtypes = [vp, ctypes.POINTER(vp), vp, vp, i64, i32,
                                               ctypes.POINTER(ctypes.c_int32), i32, i32, i32]
    lib.ksmm_cu_chain_forward_host_async.restype = i32
    lib.ksmm_cu_chain_forward_host_async.argtypes = [vp, ctypes.POINTER(vp), vp, vp, i64, i32,
                                                     ctypes.POINTER(ctypes.c_int32), i32, i32, i32,
                                                     ctypes.POINTER(ctypes.c_uint64)]
    lib.ksmm_cu_chain_workspace_bytes_layouts.restype = ctypes.c_size_t
    lib.ksmm_cu_chain_workspace_bytes_layouts.argtypes = [i32, ctypes.POINTER(ctypes.c_int32), i64, i32, i32, i32]
    lib.ksmm_cu_chain_forward_layouts.restype = i32
    lib.ksmm_cu_chain_forward_layouts.argtypes = [vp, ctypes.POINTER(vp), vp, vp, vp, ctypes.c_size_t, i64,
                                                  i32, ctypes.POINTER(ctypes.c_int32), i32, i32, i32, i32, vp]
    lib.ksmm_cu_chain_forward_desc.restype = i32
    lib.ksmm_cu_chain_forward_desc.argtypes = [ctypes.POINTER(ChainDesc), vp]
    lib.ksmm_cu_grouped_forward.restype = i32
    lib.ksmm_cu_grouped_forward.argtypes = [vp, vp, vp, vp, i64, i32, i32, i32, i32, i32, i32, i32, i32, vp]
    lib.ksmm_cu_grouped_chain_forward.restype = i32
    lib.ksmm_cu_grouped_chain_forward.argtypes = [vp, ctypes.POINTER(vp), vp, vp, vp, ctypes.c_size_t, i64,
                                                  i32, ctypes.POINTER(ctypes.c_int32), i32, i32, i32, vp]
    for name in ("ksmm_cu_backward_input_workspace_bytes", "ksmm_cu_backward_weights_workspace_bytes"):
        fn = getattr(lib, name)
        fn.restype = ctypes.c_size_t
        fn.argtypes = [i64, i32, i32, i32, i32, i32, i32]
    for name in ("ksmm_cu_backward_input", "ksmm_cu_backward_weights"):
        fn = getattr(lib, name)
        fn.restype = i32
        fn.argtypes = [vp, vp, vp, vp, ctypes.c_size_t, i64, i32, i32, i32, i32, i32, i32, vp]
    lib.ksmm_cu_host_wait.restype = i32
    lib.ksmm_cu_host_wait.argtypes = [ctypes.c_uint64]
    lib.ksmm_cu_num_configs.restype = i32
    lib.ksmm_cu_num_configs.argtypes = [i32]
    lib.ksmm_cu_config_supported.restype = i32
    lib.ksmm_cu_config_supported.argtypes = [i32, i32, i64, i32, i32, i32, i32, i32, i32, i32]
    lib.ksmm_cu_tune.restype = i32
    lib.ksmm_cu_tune.argtypes = [ctypes.POINTER(ForwardDesc), i32, vp, ctypes.POINTER(i32),
                                 ctypes.POINTER(i32), ctypes.POINTER(ctypes.c_float)]
    lib.ksmm_cu_set_choice.restype = i32
    lib.ksmm_cu_set_choice.argtypes = [i64, i32, i32, i32, i32, i32, i32, i32, i32, i32]
    lib.ksmm_cu_get_choice.restype = i32
    lib.ksmm_cu_get_choice.argtypes = [i64, i32, i32, i32, i32, i32, i32, i32,
                                       ctypes.POINTER(i32), ctypes.POINTER(i32)]
    lib.ksmm_cu_clear_choice.restype = i32
    lib.ksmm_cu_clear_choice.argtypes = [i64, i32, i32, i32, i32, i32, i32, i32]
    lib.ksmm_cu_default_choice.restype = i32
    lib.ksmm_cu_default_choice.argtypes = [ctypes.POINTER(ForwardDesc), ctypes.POINTER(i32),
                                           ctypes.POINTER(i32), ctypes.POINTER(i32)]
    lib.ksmm_cu_check_device.restype = i32
    lib.ksmm_cu_check_device.argtypes = [vp]
    lib.ksmm_cu_launch_count.restype = ctypes.c_uint64
    lib.ksmm_cu_measure_ffma_peak.restype = i32
    lib.ksmm_cu_measure_ffma_peak.argtypes = [ctypes.POINTER(ctypes.c_float), vp]
    lib.ksmm_cu_layout_scratch_bytes.restype = ctypes.c_size_t
    lib.ksmm_cu_layout_scratch_bytes.argtypes = [ctypes.POINTER(ForwardDesc)]
    lib.ksmm_cu_release_scratch.restype = i32
    lib.ksmm_cu_chain_workspace_bytes_ex.restype = ctypes.c_size_t
    lib.ksmm_cu_chain_workspace_bytes_ex.argtypes = [i32, ctypes.POINTER(ctypes.c_int32), i64, i32, i32]
    lib.ksmm_cu_alloc_count.restype = ctypes.c_uint64
    lib.ksmm_cu_debug_wait_probe.restype = i32
    lib.ksmm_cu_debug_wait_probe.argtypes = [i64, vp]
    _lib = lib
    return lib


def check(status):
    """Raise KsmmError for a non-zero status (mirrors the library's message)."""
    if status != KSMM_OK:
        msg = load().ksmm_cu_last_error().decode("utf-8", "replace")
        raise KsmmError(status, msg)


def int32_array(values):
    arr = (ctypes.c_int32 * len(values))(*values)
    return arr
