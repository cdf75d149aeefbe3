"""comfy_kitchen_b200: the NVFP4 linear path of comfy-kitchen (quantize_nvfp4, dequantize_nvfp4,
scaled_mm_nvfp4) as hand-written CUDA for NVIDIA B200 (sm_100a), behind the reference's operator interface.

    import comfy_kitchen_b200 as ckb
    q, sf = ckb.quantize_nvfp4(x, per_tensor_scale)             # same signature as comfy_kitchen's
    y = ckb.scaled_mm_nvfp4(q, qw, ts_x, ts_w, sf, sfw)
    ckb.install()                                               # plug into comfy_kitchen's registry

The kernels live in ``libck_b200.so`` (C ABI in ``include/ck_b200.h``); there is no CPU or PyTorch fallback.
"""
from . import _lib
from .backend import install, uninstall
from .build import build_library
from .ops import (dequantize_mxfp8, dequantize_nvfp4, dynamic_scale_nvfp4, launches, linear_nvfp4, quantize_mxfp8,
                  quantize_nvfp4, quantize_nvfp4_dynamic, read_device_status, read_gemm_counters, scaled_mm_mxfp8,
                  scaled_mm_nvfp4, set_tuning, promise_resident_weights)
from .linear import NVFP4Linear
from .sharded import PeerGroup, PeerMemory, ShardedNVFP4Linear, shard_rows

__all__ = [
    "quantize_nvfp4", "quantize_nvfp4_dynamic", "dequantize_nvfp4", "scaled_mm_nvfp4", "dynamic_scale_nvfp4", "linear_nvfp4", "quantize_mxfp8", "dequantize_mxfp8", "scaled_mm_mxfp8", "install", "uninstall",
    "build_library", "NVFP4Linear", "PeerGroup", "PeerMemory", "ShardedNVFP4Linear", "shard_rows", "set_tuning", "promise_resident_weights", "launches", "read_device_status", "read_gemm_counters",
]
