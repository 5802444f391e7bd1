"""ctypes view of libfa8_b200.so (declared in include/fa8_b200.h).

There is no fallback: if the library is missing or a symbol cannot be bound,
loading raises, and so does every operator call.
"""
from __future__ import annotations

import ctypes
import os

from .build import LIB_PATH, is_stale

FA8_OK = 0
FA8_ERR_BAD_ARG = -1
FA8_ERR_UNSUPPORTED = -2
FA8_ERR_CUDA = -3
FA8_ERR_DEVICE_TIMEOUT = -4

FA8_V_TRANSPOSED = 0
FA8_V_NATURAL = 1
FA8_FP8_E4M3 = 0
FA8_FP8_E5M2 = 1
FA8_DTYPE_FP16 = 0
FA8_DTYPE_BF16 = 1

# Every symbol include/fa8_b200.h declares.
EXPORTED_SYMBOLS = ("fa8_fwd", "fa8_check_status", "fa8_supported", "fa8_error_string",
                    "fa8_last_error_detail", "fa8_version", "fa8_selftest_expired_wait",
                    "fa8_quantize_e4m3", "fa8_quantize_e4m3_segments", "fa8_quantize_e4m3_segments_noalloc",
                    "fa8_work_plan")
FA8_NOALLOC_MAX_SEGMENTS = 4096


class Fa8FwdParams(ctypes.Structure):
    """struct fa8_fwd_params of include/fa8_b200.h."""
    _fields_ = [
        ("q", ctypes.c_void_p), ("k", ctypes.c_void_p), ("v", ctypes.c_void_p), ("o", ctypes.c_void_p),
        ("batch", ctypes.c_int32), ("heads", ctypes.c_int32), ("seqlen", ctypes.c_int32),
        ("head_dim", ctypes.c_int32), ("softmax_scale", ctypes.c_float), ("is_causal", ctypes.c_int32),
        ("v_layout", ctypes.c_int32), ("o_scale", ctypes.c_float), ("status_word", ctypes.c_void_p),
        ("softmax_lse", ctypes.c_void_p), ("heads_kv", ctypes.c_int32),
        ("descale_q", ctypes.c_void_p), ("descale_k", ctypes.c_void_p), ("descale_v", ctypes.c_void_p),
        ("fp8_format", ctypes.c_int32), ("seqlen_k", ctypes.c_int32),
        ("descale_per_head", ctypes.c_int32),
    ]


_lib = None


def load() -> ctypes.CDLL:
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python -m cutlass_flash_atten_fp8_b200.build` "
            "(there is no CPU or eager fallback)")
    if is_stale():
        raise ImportError(
            f"{LIB_PATH} is older than its sources: rebuild it with "
            "`python -m cutlass_flash_atten_fp8_b200.build` (a stale binary is never loaded silently)")
    lib = ctypes.CDLL(LIB_PATH)
    lib.fa8_fwd.argtypes = [ctypes.POINTER(Fa8FwdParams), ctypes.c_void_p]
    lib.fa8_fwd.restype = ctypes.c_int
    lib.fa8_check_status.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.POINTER(ctypes.c_int32)]
    lib.fa8_check_status.restype = ctypes.c_int
    lib.fa8_selftest_expired_wait.argtypes = [ctypes.c_void_p, ctypes.c_uint32, ctypes.c_void_p]
    lib.fa8_selftest_expired_wait.restype = ctypes.c_int
    lib.fa8_quantize_e4m3.argtypes = [ctypes.c_void_p, ctypes.c_int32, ctypes.c_void_p, ctypes.c_int64,
                                      ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p]
    lib.fa8_quantize_e4m3.restype = ctypes.c_int
    lib.fa8_quantize_e4m3_segments.argtypes = [ctypes.c_void_p, ctypes.c_int32, ctypes.c_void_p, ctypes.c_int64,
                                               ctypes.c_int32, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p]
    lib.fa8_quantize_e4m3_segments.restype = ctypes.c_int
    lib.fa8_quantize_e4m3_segments_noalloc.argtypes = [ctypes.c_void_p, ctypes.c_int32, ctypes.c_void_p, ctypes.c_int64,
                                                       ctypes.c_int32, ctypes.c_void_p, ctypes.c_void_p]
    lib.fa8_quantize_e4m3_segments_noalloc.restype = ctypes.c_int
    lib.fa8_supported.argtypes = [ctypes.c_int32, ctypes.c_int32, ctypes.c_int32]
    lib.fa8_supported.restype = ctypes.c_int
    lib.fa8_work_plan.argtypes = [ctypes.c_int32] * 6 + [ctypes.POINTER(ctypes.c_int32 * 4)]
    lib.fa8_work_plan.restype = ctypes.c_int
    lib.fa8_error_string.argtypes = [ctypes.c_int]
    lib.fa8_error_string.restype = ctypes.c_char_p
    lib.fa8_last_error_detail.argtypes = []
    lib.fa8_last_error_detail.restype = ctypes.c_char_p
    lib.fa8_version.argtypes = []
    lib.fa8_version.restype = ctypes.c_int
    _lib = lib
    return lib


def work_plan(slices: int, seqlen: int, head_dim: int, causal: bool, sm_count: int, seqlen_k: int = 0) -> dict:
    """fa8_work_plan as a dict: how a launch of this shape is cut into work items on a GPU
    with `sm_count` SMs (host arithmetic only)."""
    lib = load()
    out = (ctypes.c_int32 * 4)()
    rc = lib.fa8_work_plan(slices, seqlen, seqlen_k, head_dim, int(causal), sm_count, ctypes.byref(out))
    if rc != FA8_OK:
        raise ValueError(error_message(rc))
    return {"rows_per_item": out[0], "paired": bool(out[1]), "items_per_slice": out[2], "units": out[3]}


def error_message(code: int) -> str:
    lib = load()
    msg = lib.fa8_error_string(code).decode()
    detail = lib.fa8_last_error_detail().decode()
    return f"fa8 error {code}: {msg}" + (f" [{detail}]" if detail else "")
