"""ctypes binding of libhawk_b200.so (the C ABI declared in include/hawk_b200.h).

There is no CPU or eager fallback: if the library has not been built, or a call
returns an error status, a RuntimeError is raised.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import c_char_p, c_float, c_int, c_int64, c_longlong, c_size_t, c_void_p

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libhawk_b200.so")

HAWK_F32 = 0
HAWK_BF16 = 1
ABI_VERSION = 4

_P = c_void_p
# name -> (restype, argtypes); mirrors include/hawk_b200.h one to one
SIGNATURES = {
    "hawk_version": (c_int, []),
    "hawk_strerror": (c_char_p, [c_int]),
    "hawk_scan_fwd": (c_int, [_P, _P, _P, _P, _P, _P, _P, c_int, c_int, c_int, c_int, _P]),
    "hawk_scan_bwd_workspace_bytes": (c_size_t, [c_int, c_int]),
    "hawk_scan_bwd": (c_int, [_P] * 15 + [c_size_t, c_int, c_int, c_int, c_int, _P]),
    "hawk_scan_gelu_fwd": (c_int, [_P] * 6 + [c_int64, c_int64, _P, _P, c_int, c_int, c_int, c_int, _P]),
    "hawk_scan_gelu_bwd": (c_int, [_P] * 7 + [c_int64, c_int64] + [_P] * 5 + [c_int64, c_int64, _P, _P, _P, c_size_t,
                                  c_int, c_int, c_int, c_int, _P]),
    "hawk_scan_bwd_noalloc": (c_int, [_P] * 12 + [c_int, c_int, c_int, c_int, _P]),
    "hawk_scan_split_chunks": (c_int, [c_int, c_int, c_int, c_int]),
    "hawk_scan_split_workspace_bytes": (c_size_t, [c_int, c_int, c_int]),
    "hawk_scan_fwd_split": (c_int, [_P] * 7 + [c_int64, c_int64, _P, _P, c_int, _P, c_size_t, c_int, c_int, c_int, c_int, _P]),
    "hawk_scan_bwd_split": (c_int, [_P] * 8 + [c_int64, c_int64] + [_P] * 5 + [c_int64, c_int64, _P, _P, _P, c_int, _P,
                                   c_size_t, c_int, c_int, c_int, c_int, _P]),
    "hawk_conv1d_fwd": (c_int, [_P, c_int64, c_int64, _P, _P, _P, c_int, c_int, c_int, c_int, c_int, c_int, _P]),
    "hawk_conv1d_bwd_workspace_bytes": (c_size_t, [c_int, c_int, c_int, c_int]),
    "hawk_conv1d_bwd": (c_int, [_P, _P, c_int64, c_int64, _P, _P, c_int64, c_int64, _P, _P, _P, c_size_t,
                                c_int, c_int, c_int, c_int, c_int, c_int, _P]),
    "hawk_decode_conv_step": (c_int, [_P, c_int64, _P, _P, _P, _P, c_int, c_int, c_int, c_int, c_int, _P]),
    "hawk_decode_rglru_step": (c_int, [_P, _P, _P, _P, _P, _P, c_int, c_int, c_int, c_int, _P]),
    "hawk_decode_block_step": (c_int, [_P, c_int64] + [_P] * 10 + [c_int] * 7 + [_P]),
    "hawk_adamw_step": (c_int, [_P, _P, _P, _P, _P, c_int64, c_float, c_float, c_float, c_float, c_float, c_int64, _P]),
    "hawk_cast_f32_bf16": (c_int, [_P, _P, c_int64, _P]),
    "hawk_gelu_mul_fwd": (c_int, [_P, c_int64, _P, c_int64, _P, c_int64, c_int64, c_int, c_int, _P]),
    "hawk_gelu_mul_bwd": (c_int, [_P, c_int64, _P, c_int64, _P, c_int64, _P, c_int64, _P, c_int64, c_int64, c_int,
                                  c_int, _P]),
    "hawk_rms_norm_fwd": (c_int, [_P, _P, _P, _P, c_int64, c_int, c_float, c_int, c_int, _P]),
    "hawk_rms_norm_bwd_workspace_bytes": (c_size_t, [c_int]),
    "hawk_rms_norm_bwd": (c_int, [_P, _P, _P, _P, _P, _P, _P, c_size_t, c_int64, c_int, c_int, c_int, _P]),
    "hawk_add_rms_norm_fwd": (c_int, [_P, _P, _P, _P, _P, _P, c_int64, c_int, c_float, c_int, c_int, _P]),
    "hawk_add_rms_norm_bwd": (c_int, [_P, _P, _P, _P, _P, _P, _P, _P, _P, c_size_t, c_int64, c_int, c_int, c_int, _P]),
    "hawk_gates_packed_bytes": (c_size_t, [c_int, c_int]),
    "hawk_gates_bwd_workspace_bytes": (c_size_t, [c_int64, c_int, c_int]),
    "hawk_gates_pack_weights": (c_int, [_P, _P, c_int, _P, c_int, c_int, _P]),
    "hawk_gates_fwd": (c_int, [_P, _P, _P, _P, c_int64, c_int, c_int, _P, _P]),
    "hawk_gates_bwd": (c_int, [_P] * 8 + [c_size_t, c_int64, c_int, c_int, _P, _P]),
    "hawk_debug_wait_timeout": (c_int, [_P, c_size_t, c_longlong, _P, _P]),
    "hawk_linear_ce_workspace_bytes": (c_size_t, [c_int64, c_int64, c_int64]),
    "hawk_linear_ce_fwd_bwd": (c_int, [_P, _P, _P, _P, _P, _P, _P, c_size_t, c_int64, c_int64, c_int64, c_int, _P, _P]),
}

_lib = None


def load() -> ctypes.CDLL:
    """The loaded library; raises if it is missing or of another ABI version."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise RuntimeError(
            f"hawk_b200: {LIB_PATH} not found. Build it with `python hawk-pytorch_b200/build.py` "
            "(nvcc, sm_100a). There is no fallback path."
        )
    lib = ctypes.CDLL(LIB_PATH)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError if the symbol is not exported
        fn.restype = res
        fn.argtypes = args
    if lib.hawk_version() != ABI_VERSION:
        raise RuntimeError(f"hawk_b200: library ABI {lib.hawk_version()} != binding ABI {ABI_VERSION}; rebuild")
    _lib = lib
    return lib


def check(status: int, what: str) -> None:
    if status != 0:
        msg = load().hawk_strerror(status).decode()
        raise RuntimeError(f"hawk_b200: {what} failed: {msg} (status {status})")
