"""ctypes front end of the CPU oracle (``nvfp4_oracle.c``) working on numpy arrays.

TEST INFRASTRUCTURE ONLY.  Importers are the test-suite, the smoke check and the benchmark's CPU
baseline; the product package never imports this module.

The functions mirror the reference operators for the NVFP4 linear path
(``comfy_kitchen/backends/eager/quantization.py:118-249``) with numpy arrays in place of tensors:
bf16 and fp16 arrays are passed as ``uint16`` bit patterns, e4m3 scales as ``uint8`` bit patterns.
"""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "libnvfp4_oracle.so")

F32, F16, BF16 = 0, 1, 2  # dtype codes, comfy_kitchen/backends/eager/quantization.py:34-42

_lib = None


def build(force: bool = False) -> str:
    """Compile the oracle with gcc (idempotent)."""
    src = os.path.join(_HERE, "nvfp4_oracle.c")
    if force or not os.path.exists(_SO) or os.path.getmtime(_SO) < os.path.getmtime(src):
        subprocess.run(["make", "-C", _HERE, "-B", "libnvfp4_oracle.so"], check=True, capture_output=True)
    return _SO


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(_SO):
            build()
        L = ctypes.CDLL(_SO)
        vp, i64, f32, i32 = ctypes.c_void_p, ctypes.c_int64, ctypes.c_float, ctypes.c_int
        L.nvfp4_oracle_quantize.argtypes = [vp, i32, i64, i64, f32, i32, i32, vp, vp]
        L.nvfp4_oracle_quantize.restype = i32
        L.nvfp4_oracle_dequantize.argtypes = [vp, f32, vp, i64, i64, i32, i32, vp]
        L.nvfp4_oracle_dequantize.restype = i32
        L.nvfp4_oracle_dequant_f32.argtypes = [vp, f32, vp, i64, i64, i32, vp]
        L.nvfp4_oracle_dequant_f32.restype = i32
        L.nvfp4_oracle_matmul_nt.argtypes = [vp, vp, vp, i64, i64, i64, i32, vp]
        L.nvfp4_oracle_matmul_nt.restype = i32
        L.nvfp4_oracle_round_array.argtypes = [vp, i64, i32, vp]
        L.nvfp4_oracle_round_array.restype = None
        L.nvfp4_oracle_widen_array.argtypes = [vp, i64, i32, vp]
        L.nvfp4_oracle_widen_array.restype = None
        L.nvfp4_oracle_dynamic_scale.argtypes = [vp, i32, i64]
        L.nvfp4_oracle_dynamic_scale.restype = f32
        L.nvfp4_oracle_sf_offset.argtypes = [i64, i64, i64]
        L.nvfp4_oracle_sf_offset.restype = i64
        L.mxfp8_oracle_quantize.argtypes = [vp, i32, i64, i64, i32, vp, vp]
        L.mxfp8_oracle_quantize.restype = i32
        L.mxfp8_oracle_dequantize.argtypes = [vp, vp, i64, i64, i32, vp]
        L.mxfp8_oracle_dequantize.restype = i32
        L.nvfp4_oracle_num_threads.argtypes = []
        L.nvfp4_oracle_num_threads.restype = i32
        L.nvfp4_oracle_set_num_threads.argtypes = [i32]
        L.nvfp4_oracle_set_num_threads.restype = None
        _lib = L
    return _lib


def _ptr(a: np.ndarray) -> ctypes.c_void_p:
    return ctypes.c_void_p(a.ctypes.data)


def roundup(x: int, m: int) -> int:
    return (x + m - 1) // m * m


def num_threads() -> int:
    return int(lib().nvfp4_oracle_num_threads())


def use_all_cores() -> int:
    """Make the oracle's OpenMP loops, numpy's BLAS and torch use every core this process may run on, whatever
    OMP_NUM_THREADS the launcher exported (torchrun sets it to 1), and return that count."""
    n = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    lib().nvfp4_oracle_set_num_threads(n)
    try:
        from threadpoolctl import threadpool_limits
        threadpool_limits(limits=n)      # numpy's BLAS (the fp32 matmul of the GEMM restatement)
    except Exception:
        pass
    try:
        import torch
        torch.set_num_threads(n)
    except Exception:
        pass
    return n


def _check_input(x: np.ndarray, dtype: int) -> np.ndarray:
    want = np.float32 if dtype == F32 else np.uint16
    if x.dtype != want:
        raise TypeError(f"dtype code {dtype} wants a {want.__name__} array, got {x.dtype}")
    return np.ascontiguousarray(x)


def quantize_nvfp4(x: np.ndarray, dtype: int, per_tensor_scale: float, pad_16x: bool = False,
                   hi_first: bool = True) -> tuple[np.ndarray, np.ndarray]:
    """x [rows, cols] (float32, or uint16 bits for fp16/bf16) -> (packed uint8 [R, C/2], swizzled e4m3
    bits uint8 [roundup(R,128), roundup(C/16,4)]).  eager/quantization.py:118-163."""
    x = _check_input(x, dtype)
    rows, cols = x.shape
    prow, pcol = (roundup(rows, 16), roundup(cols, 16)) if pad_16x else (rows, cols)
    q = np.empty((prow, pcol // 2), np.uint8)
    sf = np.empty((roundup(prow, 128), roundup(pcol // 16, 4)), np.uint8)
    rc = lib().nvfp4_oracle_quantize(_ptr(x), dtype, rows, cols, float(np.float32(per_tensor_scale)),
                                     int(pad_16x), int(hi_first), _ptr(q), _ptr(sf))
    if rc != 0:
        raise ValueError("quantize_nvfp4 without pad_16x needs rows and cols divisible by 16")
    return q, sf


def dequantize_nvfp4(q: np.ndarray, per_tensor_scale: float, sf: np.ndarray, out_dtype: int = BF16,
                     hi_first: bool = True) -> np.ndarray:
    """packed uint8 [R, C/2] + swizzled scales -> [R, C] (float32, or uint16 bits for fp16/bf16).
    eager/quantization.py:174-222."""
    q = np.ascontiguousarray(q, np.uint8)
    sf = np.ascontiguousarray(sf, np.uint8)
    rows, pcols = q.shape
    out = np.empty((rows, pcols * 2), np.float32 if out_dtype == F32 else np.uint16)
    rc = lib().nvfp4_oracle_dequantize(_ptr(q), float(np.float32(per_tensor_scale)), _ptr(sf), rows, pcols,
                                       out_dtype, int(hi_first), _ptr(out))
    if rc != 0:
        raise ValueError("dequantize_nvfp4 needs a column count divisible by 16")
    return out


def widen(a: np.ndarray, dtype: int) -> np.ndarray:
    """uint16 bit patterns of fp16/bf16 -> float32."""
    if dtype == F32:
        return np.ascontiguousarray(a, np.float32)
    a = np.ascontiguousarray(a, np.uint16)
    out = np.empty(a.shape, np.float32)
    lib().nvfp4_oracle_widen_array(_ptr(a), a.size, dtype, _ptr(out))
    return out


def narrow(a: np.ndarray, dtype: int) -> np.ndarray:
    """float32 -> uint16 bit patterns of fp16/bf16, round to nearest even."""
    a = np.ascontiguousarray(a, np.float32)
    if dtype == F32:
        return a
    out = np.empty(a.shape, np.uint16)
    lib().nvfp4_oracle_round_array(_ptr(a), a.size, dtype, _ptr(out))
    return out


def dynamic_scale(x: np.ndarray, dtype: int) -> float:
    """amax(|x|)/(448*6) computed in the input dtype, comfy_kitchen/tensor/nvfp4.py:66-71."""
    x = _check_input(x, dtype)
    return float(lib().nvfp4_oracle_dynamic_scale(_ptr(x), dtype, x.size))


def scaled_mm_nvfp4(a: np.ndarray, b: np.ndarray, tensor_scale_a: float, tensor_scale_b: float,
                    block_scale_a: np.ndarray, block_scale_b: np.ndarray, bias: np.ndarray | None = None,
                    bias_dtype: int = BF16, out_dtype: int = BF16, alpha: float | None = None,
                    blas: bool = True) -> np.ndarray:
    """CPU restatement of scaled_mm_nvfp4: dequantize both operands to fp32, fp32 matmul, add bias, round
    to the output dtype (the check the reference applies in tests/test_qdq.py:490-509).  a [M, K/2] and
    b [N, K/2] packed uint8.  With ``alpha`` given, the per-tensor scales are replaced by it
    (comfy_kitchen/backends/cuda/__init__.py:1748-1757).  ``blas=False`` uses the scalar C loop."""
    a = np.ascontiguousarray(a, np.uint8)
    b = np.ascontiguousarray(b, np.uint8)
    M, pk = a.shape
    N = b.shape[0]
    K = pk * 2
    L = lib()
    tsa, tsb = (float(tensor_scale_a), float(tensor_scale_b)) if alpha is None else (float(alpha), 1.0)
    da = np.empty((M, K), np.float32)
    db = np.empty((N, K), np.float32)
    sa = np.ascontiguousarray(block_scale_a, np.uint8)
    sb = np.ascontiguousarray(block_scale_b, np.uint8)
    L.nvfp4_oracle_dequant_f32(_ptr(a), float(np.float32(tsa)), _ptr(sa), M, pk, 1, _ptr(da))
    L.nvfp4_oracle_dequant_f32(_ptr(b), float(np.float32(tsb)), _ptr(sb), N, pk, 1, _ptr(db))
    bias_f = None if bias is None else widen(bias, bias_dtype)
    if blas:
        y = da @ db.T
        if bias_f is not None:
            y = y + bias_f[None, :]
        return narrow(y.astype(np.float32, copy=False), out_dtype)
    out = np.empty((M, N), np.float32 if out_dtype == F32 else np.uint16)
    L.nvfp4_oracle_matmul_nt(_ptr(da), _ptr(db), None if bias_f is None else _ptr(bias_f), M, N, K, out_dtype,
                             _ptr(out))
    return out


def rel_rms(y: np.ndarray, y_ref: np.ndarray) -> float:
    """sqrt(mean((y - y_ref)^2)) / sqrt(mean(y_ref^2)) in float64."""
    y = y.astype(np.float64)
    y_ref = y_ref.astype(np.float64)
    den = np.sqrt(np.mean(y_ref * y_ref))
    return float(np.sqrt(np.mean((y - y_ref) ** 2)) / (den if den > 0 else 1.0))


# ---- MXFP8 (comfy_kitchen/backends/eager/quantization.py:260-405) --------------------------------------------

def quantize_mxfp8(x: np.ndarray, dtype: int, pad_32x: bool = False) -> tuple[np.ndarray, np.ndarray]:
    """x [rows, cols] -> (e4m3 bytes uint8 [R, C], e8m0 block scales uint8 [roundup(R,128), roundup(C/32,4)] tiled)."""
    x = _check_input(x, dtype)
    rows, cols = x.shape
    prow, pcol = (roundup(rows, 32), roundup(cols, 32)) if pad_32x else (rows, cols)
    if pcol % 32:
        raise ValueError("cols must be a multiple of 32 without pad_32x")
    q = np.empty((prow, pcol), np.uint8)
    sf = np.empty((roundup(prow, 128), roundup(pcol // 32, 4)), np.uint8)
    rc = lib().mxfp8_oracle_quantize(_ptr(x), dtype, rows, cols, int(pad_32x), _ptr(q), _ptr(sf))
    assert rc == 0
    return q, sf


def dequantize_mxfp8(q: np.ndarray, sf: np.ndarray, out_dtype: int = BF16) -> np.ndarray:
    q, sf = np.ascontiguousarray(q, np.uint8), np.ascontiguousarray(sf, np.uint8)
    rows, cols = q.shape
    out = np.empty((rows, cols), np.float32 if out_dtype == F32 else np.uint16)
    rc = lib().mxfp8_oracle_dequantize(_ptr(q), _ptr(sf), rows, cols, out_dtype, _ptr(out))
    assert rc == 0
    return out


def scaled_mm_mxfp8(a: np.ndarray, b: np.ndarray, block_scale_a: np.ndarray, block_scale_b: np.ndarray,
                    bias: np.ndarray | None = None, bias_dtype: int = BF16, out_dtype: int = BF16) -> np.ndarray:
    """out_dtype( dequant(a) @ dequant(b)^T + bias ) with fp32 accumulation: the check the reference applies to
    scaled_mm_mxfp8 (dequantize -> linear), like scaled_mm_nvfp4 above."""
    af = dequantize_mxfp8(a, block_scale_a, F32)
    bf = dequantize_mxfp8(b, block_scale_b, F32)
    y = af @ bf.T
    if bias is not None:
        y = y + (bias.astype(np.float32) if bias_dtype == F32 else widen(bias, bias_dtype))[None, :]
    return y if out_dtype == F32 else narrow(np.ascontiguousarray(y, np.float32), out_dtype)
