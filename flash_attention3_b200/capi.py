"""ctypes binding of the C ABI declared in include/shaobo_fa3_api.h and
include/shaobo_fa3_components.h.  The structure mirrors ShaoboFa3Params field
for field (296 bytes on LP64)."""
from __future__ import annotations

import ctypes
import os
import pathlib

PKG = pathlib.Path(__file__).resolve().parent
LIB_PATH = PKG / "libfa3bwd_b200.so"

STATUS_SUCCESS, STATUS_INVALID_VALUE, STATUS_UNSUPPORTED, STATUS_NOT_IMPLEMENTED, STATUS_CUDA_ERROR = range(5)
DTYPE_FP16, DTYPE_BF16, DTYPE_FP8 = 0, 1, 2
LAYOUT_BHSD, LAYOUT_BSHD = 0, 1
AUX_SMAX_SSUM, AUX_LSE = 0, 1
DKV_PATH_REFERENCE, DKV_PATH_CANONICAL = 1, 5
DQ_PATH_REFERENCE, DQ_PATH_CANONICAL = 1, 6
RESERVED_PTR_DELTA, RESERVED_PTR_SIDECAR, RESERVED_PTR_STREAM = 0, 3, 7
STATIC_SCRATCH_BYTES = 32 << 20  # SHAOBO_FA3_B200_STATIC_SCRATCH_BYTES

FEATURE_BITS = {
    "FIXED_LENGTH": 1 << 0, "VARLEN": 1 << 1, "FP16": 1 << 2, "BF16": 1 << 3, "CAUSAL": 1 << 4,
    "LOCAL_WINDOW": 1 << 5, "GQA": 1 << 6, "SOFTCAP": 1 << 7, "DETERMINISTIC": 1 << 8,
    "SOFTMAX_LSE": 1 << 9, "BSHD": 1 << 10, "BHSD": 1 << 11, "FULL_ATTENTION": 1 << 12,
}


class Params(ctypes.Structure):
    _fields_ = [
        ("struct_size", ctypes.c_uint32),
        ("batch", ctypes.c_int32), ("seqlen_q", ctypes.c_int32), ("seqlen_k", ctypes.c_int32),
        ("num_heads_q", ctypes.c_int32), ("num_heads_kv", ctypes.c_int32),
        ("head_dim_qk", ctypes.c_int32), ("head_dim_v", ctypes.c_int32),
        ("causal", ctypes.c_int32), ("window_left", ctypes.c_int32), ("window_right", ctypes.c_int32),
        ("softmax_scale", ctypes.c_float), ("dropout_p", ctypes.c_float),
        ("dtype", ctypes.c_int32), ("layout", ctypes.c_int32), ("softmax_aux_mode", ctypes.c_int32),
        ("dkv_path", ctypes.c_int32), ("dq_path", ctypes.c_int32), ("block_threads", ctypes.c_int32),
        ("sync_after_launch", ctypes.c_int32),
        ("cu_seqlens_q", ctypes.c_void_p), ("cu_seqlens_k", ctypes.c_void_p),
        ("max_seqlen_q", ctypes.c_int32), ("max_seqlen_k", ctypes.c_int32),
        ("workspace", ctypes.c_void_p), ("workspace_bytes", ctypes.c_size_t),
        ("reserved_i32", ctypes.c_int32 * 16), ("reserved_ptr", ctypes.c_void_p * 8),
        ("seqused_q", ctypes.c_void_p), ("seqused_k", ctypes.c_void_p),
        ("total_q", ctypes.c_int64), ("total_k", ctypes.c_int64),
        ("softcap", ctypes.c_float), ("deterministic", ctypes.c_int32), ("sm_margin", ctypes.c_int32),
        ("softmax_scale_is_set", ctypes.c_int32),
    ]


class Capabilities(ctypes.Structure):
    _fields_ = [
        ("struct_size", ctypes.c_uint32), ("api_version", ctypes.c_uint32),
        ("feature_mask", ctypes.c_uint64),
        ("min_head_dim", ctypes.c_int32), ("max_head_dim", ctypes.c_int32),
        ("head_dim_alignment", ctypes.c_int32), ("sequence_alignment", ctypes.c_int32),
    ]


# every symbol the headers under include/ declare
EXPORTS = [
    "shaobo_fa3_params_init", "shaobo_fa3_bwd_get_capabilities", "shaobo_fa3_bwd_v2_validate",
    "shaobo_fa3_bwd_v2_workspace_bytes", "shaobo_fa3_bwd_v2", "shaobo_fa3_status_string",
    "shaobo_fa3_bwd_workspace_bytes", "shaobo_fa3_bwd",
    "shaobo_fa3_bwd_dot_do_o", "shaobo_fa3_bwd_fused5_workspace_bytes", "shaobo_fa3_bwd_fused5",
    "shaobo_fa3_bwd_dkv_workspace_bytes", "shaobo_fa3_bwd_dkv",
    "shaobo_fa3_bwd_dq_workspace_bytes", "shaobo_fa3_bwd_dq",
    # include/shaobo_fa3_b200_ext.h
    "shaobo_fa3_b200_device_error", "shaobo_fa3_b200_stage_timing", "shaobo_fa3_b200_last_stage_ms",
    "shaobo_fa3_b200_bwd_v2_noalloc", "shaobo_fa3_b200_fwd",
    "shaobo_fa3_b200_bwd_v2_host_staging_bytes", "shaobo_fa3_b200_bwd_v2_host",
]

_lib = None


def load(build_if_missing: bool = True) -> ctypes.CDLL:
    """Load the in-tree library.  There is no fallback: a missing or unloadable
    library raises."""
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists():
        if not build_if_missing:
            raise FileNotFoundError(f"{LIB_PATH} is not built")
        from . import build as _build
        _build.build()
    lib = ctypes.CDLL(str(LIB_PATH))
    vp, pp = ctypes.c_void_p, ctypes.POINTER(Params)
    lib.shaobo_fa3_params_init.argtypes = [pp]
    lib.shaobo_fa3_params_init.restype = None
    lib.shaobo_fa3_bwd_get_capabilities.argtypes = [ctypes.POINTER(Capabilities)]
    lib.shaobo_fa3_bwd_get_capabilities.restype = ctypes.c_int
    lib.shaobo_fa3_bwd_v2_validate.argtypes = [pp]
    lib.shaobo_fa3_bwd_v2_validate.restype = ctypes.c_int
    for name in ("shaobo_fa3_bwd_v2_workspace_bytes", "shaobo_fa3_bwd_workspace_bytes",
                 "shaobo_fa3_bwd_fused5_workspace_bytes", "shaobo_fa3_bwd_dkv_workspace_bytes",
                 "shaobo_fa3_bwd_dq_workspace_bytes"):
        getattr(lib, name).argtypes = [pp]
        getattr(lib, name).restype = ctypes.c_size_t
    lib.shaobo_fa3_bwd_v2.argtypes = [vp] * 10 + [pp]
    lib.shaobo_fa3_bwd_v2.restype = ctypes.c_int
    lib.shaobo_fa3_b200_bwd_v2_noalloc.argtypes = [vp] * 10 + [pp]
    lib.shaobo_fa3_b200_bwd_v2_noalloc.restype = ctypes.c_int
    for name in ("shaobo_fa3_bwd", "shaobo_fa3_bwd_dkv", "shaobo_fa3_bwd_dq"):
        getattr(lib, name).argtypes = [vp] * 10 + [pp]
        getattr(lib, name).restype = ctypes.c_int
    lib.shaobo_fa3_bwd_dot_do_o.argtypes = [vp] * 6 + [pp]
    lib.shaobo_fa3_bwd_dot_do_o.restype = ctypes.c_int
    lib.shaobo_fa3_bwd_fused5.argtypes = [vp] * 8 + [pp]
    lib.shaobo_fa3_bwd_fused5.restype = ctypes.c_int
    lib.shaobo_fa3_status_string.argtypes = [ctypes.c_int]
    lib.shaobo_fa3_status_string.restype = ctypes.c_char_p
    lib.shaobo_fa3_b200_device_error.argtypes = [ctypes.c_int]
    lib.shaobo_fa3_b200_device_error.restype = ctypes.c_int
    lib.shaobo_fa3_b200_stage_timing.argtypes = [ctypes.c_int]
    lib.shaobo_fa3_b200_stage_timing.restype = ctypes.c_int
    lib.shaobo_fa3_b200_bwd_v2_host_staging_bytes.argtypes = [ctypes.POINTER(Params)]
    lib.shaobo_fa3_b200_bwd_v2_host_staging_bytes.restype = ctypes.c_size_t
    lib.shaobo_fa3_b200_bwd_v2_host.argtypes = [ctypes.c_void_p] * 10 + [ctypes.c_size_t, ctypes.POINTER(Params)]
    lib.shaobo_fa3_b200_bwd_v2_host.restype = ctypes.c_int
    lib.shaobo_fa3_b200_fwd.argtypes = [ctypes.c_void_p] * 5 + [ctypes.POINTER(Params)]
    lib.shaobo_fa3_b200_fwd.restype = ctypes.c_int
    lib.shaobo_fa3_b200_last_stage_ms.argtypes = [ctypes.POINTER(ctypes.c_float)]
    lib.shaobo_fa3_b200_last_stage_ms.restype = ctypes.c_int
    _lib = lib
    return lib


def new_params(**fields) -> Params:
    p = Params()
    load().shaobo_fa3_params_init(ctypes.byref(p))
    for k, v in fields.items():
        setattr(p, k, v)
    return p


def status_string(code: int) -> str:
    return load().shaobo_fa3_status_string(code).decode()
