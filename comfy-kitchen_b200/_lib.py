"""Loads ``libck_b200.so`` (the C ABI declared in ``include/ck_b200.h``) through ctypes.

There is no fallback: if the library is missing or a symbol is absent, importing fails with an error
that says how to build it.
"""
from __future__ import annotations

import ctypes
import os

from .build import LIB_PATH

# every symbol include/ck_b200.h declares
EXPORTED_SYMBOLS = (
    "ck_b200_quantize_nvfp4",
    "ck_b200_dequantize_nvfp4",
    "ck_b200_scaled_mm_nvfp4",
    "ck_b200_scaled_mm_nvfp4_static_scratch",
    "ck_b200_scaled_mm_nvfp4_all_gather",
    "ck_b200_peer_barrier",
    "ck_b200_peer_alloc",
    "ck_b200_peer_open",
    "ck_b200_peer_close",
    "ck_b200_peer_free",
    "ck_b200_dynamic_scale_nvfp4",
    "ck_b200_quantize_nvfp4_dynamic",
    "ck_b200_quantize_mxfp8",
    "ck_b200_dequantize_mxfp8",
    "ck_b200_scaled_mm_mxfp8",
    "ck_b200_linear_nvfp4",
    "ck_b200_linear_nvfp4_workspace_bytes",
    "ck_b200_last_error",
    "ck_b200_query",
    "ck_b200_read_device_status",
    "ck_b200_read_gemm_counters",
    "ck_b200_set_tuning",
)

QUERY_ABI_VERSION, QUERY_SM_COUNT, QUERY_WORKSPACE_BYTES, QUERY_COMPUTE_CAPABILITY, QUERY_LAUNCHES, QUERY_LAST_GEMM_SPLITS = range(6)
TUNE_QUANT_VARIANT, TUNE_GEMM_VARIANT = 0, 1
TUNE_GEMM_SKINNY, TUNE_WEIGHTS_RESIDENT = 11, 12

_lib = None


def load() -> ctypes.CDLL:
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python -c 'import __graft_entry__ as g; g.build()'` "
            "(needs nvcc); comfy_kitchen_b200 has no CPU or PyTorch fallback")
    L = ctypes.CDLL(LIB_PATH)
    for name in EXPORTED_SYMBOLS:
        if not hasattr(L, name):
            raise ImportError(f"{LIB_PATH} does not export {name}; rebuild it")
    vp, i64, i32, sz = ctypes.c_void_p, ctypes.c_int64, ctypes.c_int, ctypes.c_size_t
    L.ck_b200_quantize_nvfp4.argtypes = [vp, i32, vp, vp, vp, i64, i64, i32, i32, vp]
    L.ck_b200_quantize_nvfp4.restype = i32
    L.ck_b200_dequantize_nvfp4.argtypes = [vp, vp, vp, vp, i32, i64, i64, i32, vp]
    L.ck_b200_dequantize_nvfp4.restype = i32
    L.ck_b200_scaled_mm_nvfp4.argtypes = [vp, vp, vp, vp, vp, vp, vp, vp, i32, vp, i32, i64, i64, i64, vp, sz, vp]
    L.ck_b200_scaled_mm_nvfp4.restype = i32
    L.ck_b200_scaled_mm_nvfp4_static_scratch.argtypes = [vp, vp, vp, vp, vp, vp, vp, vp, i32, vp, i32, i64, i64, i64, vp]
    L.ck_b200_scaled_mm_nvfp4_static_scratch.restype = i32
    L.ck_b200_scaled_mm_nvfp4_all_gather.argtypes = [vp, vp, vp, vp, vp, vp, vp, vp, i32, ctypes.POINTER(vp), i32, i32, i32,
                                                     i64, i64, i64, vp]
    L.ck_b200_scaled_mm_nvfp4_all_gather.restype = i32
    L.ck_b200_peer_barrier.argtypes = [ctypes.POINTER(vp), i32, i32, vp, vp]
    L.ck_b200_peer_barrier.restype = i32
    L.ck_b200_peer_alloc.argtypes = [sz, ctypes.POINTER(vp), vp]
    L.ck_b200_peer_alloc.restype = i32
    L.ck_b200_peer_open.argtypes = [vp, ctypes.POINTER(vp)]
    L.ck_b200_peer_open.restype = i32
    L.ck_b200_peer_close.argtypes = [vp]
    L.ck_b200_peer_close.restype = i32
    L.ck_b200_peer_free.argtypes = [vp]
    L.ck_b200_peer_free.restype = i32
    L.ck_b200_linear_nvfp4.argtypes = [vp, i32, i64, i64, vp, vp, vp, vp, i64, vp, i32, vp, i32, vp, sz, vp]
    L.ck_b200_linear_nvfp4.restype = i32
    L.ck_b200_linear_nvfp4_workspace_bytes.argtypes = [i64, i64]
    L.ck_b200_linear_nvfp4_workspace_bytes.restype = i64
    L.ck_b200_quantize_mxfp8.argtypes = [vp, i32, vp, vp, i64, i64, i32, vp]
    L.ck_b200_quantize_mxfp8.restype = i32
    L.ck_b200_dequantize_mxfp8.argtypes = [vp, vp, vp, i32, i64, i64, vp]
    L.ck_b200_dequantize_mxfp8.restype = i32
    L.ck_b200_scaled_mm_mxfp8.argtypes = [vp, vp, vp, vp, vp, i32, vp, i32, i64, i64, i64, vp, sz, vp]
    L.ck_b200_scaled_mm_mxfp8.restype = i32
    L.ck_b200_dynamic_scale_nvfp4.argtypes = [vp, i32, i64, vp, vp]
    L.ck_b200_dynamic_scale_nvfp4.restype = i32
    L.ck_b200_quantize_nvfp4_dynamic.argtypes = [vp, i32, vp, vp, vp, i64, i64, i32, i32, vp, vp]
    L.ck_b200_quantize_nvfp4_dynamic.restype = i32
    L.ck_b200_last_error.argtypes = []
    L.ck_b200_last_error.restype = ctypes.c_char_p
    L.ck_b200_query.argtypes = [i32]
    L.ck_b200_query.restype = i64
    L.ck_b200_read_device_status.argtypes = [ctypes.POINTER(i32)]
    L.ck_b200_read_device_status.restype = i32
    L.ck_b200_read_gemm_counters.argtypes = [ctypes.POINTER(ctypes.c_longlong)]
    L.ck_b200_read_gemm_counters.restype = i32
    L.ck_b200_set_tuning.argtypes = [i32, i32]
    L.ck_b200_set_tuning.restype = i32
    _lib = L
    return L


def last_error() -> str:
    return load().ck_b200_last_error().decode("utf-8", "replace")


def check(rc: int, what: str) -> None:
    """Raise RuntimeError for a non-zero status (the reference launchers throw std::runtime_error, which
    its bindings surface as RuntimeError: comfy_kitchen/backends/cuda/ops/quantize_nvfp4.cu:380-383)."""
    if rc != 0:
        raise RuntimeError(f"{what} failed (status {rc}): {last_error()}")
