"""Registers this package as a backend of the comfy_kitchen registry.

The reference selects an implementation per call from a priority list of registered backend modules
after checking each module's declared constraints (``comfy_kitchen/registry.py:41-59,180-233``).
``install()`` registers this package under the name ``"sm100"`` with constraints modelled on the reference
CUDA backend's (``comfy_kitchen/backends/cuda/__init__.py:3101-3139,3617-3645``) and puts it first in the
priority list, so ``ck.quantize_nvfp4``, ``ck.scaled_mm_nvfp4``, ``QuantizedTensor.from_float(...,
"TensorCoreNVFP4Layout")`` and ``F.linear`` on NVFP4 tensors reach the kernels here without any change
to the reference.  Calls the constraints reject (CPU tensors, non-contiguous inputs, unsupported
dtypes) fall through to the next backend, which is the registry's own convention.
"""
from __future__ import annotations

import sys
import types

import torch

from . import ops

BACKEND_NAME = "sm100"


def _call_rule_quantize(ValidationResult):
    def rule(kwargs):
        x = kwargs.get("x")
        if isinstance(x, torch.Tensor):
            if not x.is_contiguous():
                return ValidationResult.fail("x", "must be contiguous")
            if not kwargs.get("pad_16x", False) and (x.dim() != 2 or x.shape[0] % 16 or x.shape[1] % 16):
                return ValidationResult.fail("x", "rows and cols must be divisible by 16 unless pad_16x")
        return ValidationResult.ok()
    return rule


def _call_rule_dequantize(ValidationResult):
    def rule(kwargs):
        qx, bs = kwargs.get("qx"), kwargs.get("block_scales")
        if isinstance(qx, torch.Tensor):
            if not qx.is_contiguous():
                return ValidationResult.fail("qx", "must be contiguous")
            if isinstance(bs, torch.Tensor):
                want = ops.roundup(qx.shape[0], 128) * ops.roundup(qx.shape[1] * 2 // 16, 4)
                if bs.numel() != want or not bs.is_contiguous() or bs.device != qx.device:
                    return ValidationResult.fail("block_scales", "wrong size, layout or device")
        return ValidationResult.ok()
    return rule


def _call_rule_scaled_mm(ValidationResult):
    def rule(kwargs):
        a, b = kwargs.get("a"), kwargs.get("b")
        sa, sb = kwargs.get("block_scale_a"), kwargs.get("block_scale_b")
        bias = kwargs.get("bias")
        if not (isinstance(a, torch.Tensor) and isinstance(b, torch.Tensor)):
            return ValidationResult.ok()
        if a.dim() != 2 or b.dim() != 2 or a.shape[1] != b.shape[1]:
            return ValidationResult.fail("b", "K of a and b differ")
        if not (a.is_contiguous() and b.is_contiguous()):
            return ValidationResult.fail("a", "operands must be contiguous")
        if b.shape[0] % 8:
            return ValidationResult.fail("b", "N must be divisible by 8")
        sk = ops.roundup(a.shape[1] * 2 // 16, 4)
        for name, s, rows in (("block_scale_a", sa, a.shape[0]), ("block_scale_b", sb, b.shape[0])):
            if isinstance(s, torch.Tensor) and (tuple(s.shape) != (ops.roundup(rows, 128), sk) or not s.is_contiguous()
                                               or s.device != a.device):
                return ValidationResult.fail(name, "wrong shape, layout or device")
        if isinstance(bias, torch.Tensor) and bias.numel() > 0:
            if bias.dtype not in (torch.float16, torch.bfloat16) or bias.numel() != b.shape[0] or bias.device != a.device:
                return ValidationResult.fail("bias", "must be an fp16/bf16 [N] tensor on the operands' device")
        return ValidationResult.ok()
    return rule


def _call_rule_quantize_mx(ValidationResult):
    def rule(kwargs):
        x = kwargs.get("x")
        if isinstance(x, torch.Tensor):
            if not x.is_contiguous():
                return ValidationResult.fail("x", "must be contiguous")
            if not kwargs.get("pad_32x", False) and (x.dim() != 2 or x.shape[0] % 32 or x.shape[1] % 32):
                return ValidationResult.fail("x", "rows and cols must be divisible by 32 unless pad_32x")
        return ValidationResult.ok()
    return rule


def _call_rule_mx_operands(ValidationResult):
    """dequantize_mxfp8 (qx, block_scales) and scaled_mm_mxfp8 (a, b, block_scale_a, block_scale_b)."""
    def rule(kwargs):
        pairs = [(kwargs.get("qx"), kwargs.get("block_scales"), "block_scales"),
                 (kwargs.get("a"), kwargs.get("block_scale_a"), "block_scale_a"),
                 (kwargs.get("b"), kwargs.get("block_scale_b"), "block_scale_b")]
        for q, sf, name in pairs:
            if not isinstance(q, torch.Tensor):
                continue
            if q.dim() != 2 or not q.is_contiguous() or q.shape[1] % 32:
                return ValidationResult.fail(name, "data must be contiguous 2D with K divisible by 32")
            if isinstance(sf, torch.Tensor) and (tuple(sf.shape) != (ops.roundup(q.shape[0], 128), ops.roundup(q.shape[1] // 32, 4))
                                                or not sf.is_contiguous() or sf.device != q.device):
                return ValidationResult.fail(name, "wrong shape, layout or device")
        a, b, bias = kwargs.get("a"), kwargs.get("b"), kwargs.get("bias")
        if isinstance(a, torch.Tensor) and isinstance(b, torch.Tensor):
            if a.shape[1] != b.shape[1]:
                return ValidationResult.fail("b", "K of a and b differ")
            if b.shape[0] % 8:
                return ValidationResult.fail("b", "N must be divisible by 8")
            if isinstance(bias, torch.Tensor) and bias.numel() > 0 and (
                    bias.dtype not in (torch.float16, torch.bfloat16) or bias.numel() != b.shape[0] or bias.device != a.device):
                return ValidationResult.fail("bias", "must be an fp16/bf16 [N] tensor on the operands' device")
        return ValidationResult.ok()
    return rule


def build_constraints():
    """{function name: FunctionConstraints} for the operators of this backend (NVFP4 and MXFP8)."""
    from comfy_kitchen.constraints import (DivisibleBy, ExactDims, FunctionConstraints, ParamConstraint,
                                           ValidationResult)
    cuda = frozenset({"cuda"})
    floats = frozenset({torch.float32, torch.float16, torch.bfloat16})
    u8 = frozenset({torch.uint8})
    f32 = frozenset({torch.float32})
    e4m3 = frozenset({torch.float8_e4m3fn})
    return {
        "quantize_nvfp4": FunctionConstraints(
            params={"x": ParamConstraint(dtypes=floats, shape_rules=(ExactDims(2),)),
                    "per_tensor_scale": ParamConstraint(dtypes=f32)},
            default_devices=cuda, min_compute_capability=(10, 0),
            call_rules=(_call_rule_quantize(ValidationResult),)),
        "dequantize_nvfp4": FunctionConstraints(
            params={"qx": ParamConstraint(dtypes=u8, shape_rules=(ExactDims(2), DivisibleBy(dim=1, factor=8))),
                    "per_tensor_scale": ParamConstraint(dtypes=f32),
                    "block_scales": ParamConstraint(dtypes=e4m3),
                    "output_type": ParamConstraint(dtypes=floats)},
            default_devices=cuda, min_compute_capability=(10, 0),
            call_rules=(_call_rule_dequantize(ValidationResult),)),
        "scaled_mm_nvfp4": FunctionConstraints(
            params={"a": ParamConstraint(dtypes=u8, shape_rules=(ExactDims(2), DivisibleBy(dim=1, factor=16))),
                    "b": ParamConstraint(dtypes=u8, shape_rules=(ExactDims(2), DivisibleBy(dim=1, factor=16))),
                    "tensor_scale_a": ParamConstraint(dtypes=f32),
                    "tensor_scale_b": ParamConstraint(dtypes=f32),
                    "block_scale_a": ParamConstraint(dtypes=e4m3),
                    "block_scale_b": ParamConstraint(dtypes=e4m3),
                    "out_dtype": ParamConstraint(dtypes=frozenset({torch.float16, torch.bfloat16}))},
            default_devices=cuda, min_compute_capability=(10, 0),
            call_rules=(_call_rule_scaled_mm(ValidationResult),)),
        # the MXFP8 sibling path (comfy_kitchen/backends/eager/__init__.py:528-567)
        "quantize_mxfp8": FunctionConstraints(
            params={"x": ParamConstraint(dtypes=floats, shape_rules=(ExactDims(2),))},
            default_devices=cuda, min_compute_capability=(10, 0),
            call_rules=(_call_rule_quantize_mx(ValidationResult),)),
        "dequantize_mxfp8": FunctionConstraints(
            params={"qx": ParamConstraint(dtypes=e4m3, shape_rules=(ExactDims(2),)),
                    "block_scales": ParamConstraint(dtypes=frozenset({torch.float8_e8m0fnu})),
                    "output_type": ParamConstraint(dtypes=floats)},
            default_devices=cuda, min_compute_capability=(10, 0),
            call_rules=(_call_rule_mx_operands(ValidationResult),)),
        "scaled_mm_mxfp8": FunctionConstraints(
            params={"a": ParamConstraint(dtypes=e4m3, shape_rules=(ExactDims(2),)),
                    "b": ParamConstraint(dtypes=e4m3, shape_rules=(ExactDims(2),)),
                    "block_scale_a": ParamConstraint(dtypes=frozenset({torch.float8_e8m0fnu})),
                    "block_scale_b": ParamConstraint(dtypes=frozenset({torch.float8_e8m0fnu})),
                    "out_dtype": ParamConstraint(dtypes=floats)},
            default_devices=cuda, min_compute_capability=(10, 0),
            call_rules=(_call_rule_mx_operands(ValidationResult),)),
    }


def backend_module() -> types.ModuleType:
    """A module object exposing exactly the operator functions, as the registry expects
    (it resolves ``getattr(module, func_name)``, ``comfy_kitchen/registry.py:266-270``)."""
    mod = types.ModuleType("comfy_kitchen.backends.sm100")
    mod.__doc__ = "B200 (sm_100a) NVFP4 backend provided by comfy_kitchen_b200"
    mod.quantize_nvfp4 = ops.quantize_nvfp4
    mod.dequantize_nvfp4 = ops.dequantize_nvfp4
    mod.scaled_mm_nvfp4 = ops.scaled_mm_nvfp4
    mod.quantize_mxfp8 = ops.quantize_mxfp8
    mod.dequantize_mxfp8 = ops.dequantize_mxfp8
    mod.scaled_mm_mxfp8 = ops.scaled_mm_mxfp8
    return mod


def install(name: str = BACKEND_NAME, first: bool = True):
    """Register with the comfy_kitchen registry (which must be importable) and return the backend module."""
    import comfy_kitchen  # noqa: F401  (defines the custom ops and registers the stock backends)
    from comfy_kitchen.registry import registry
    mod = backend_module()
    registry.register(name, mod, build_constraints())
    sys.modules.setdefault("comfy_kitchen.backends." + name, mod)
    if first:
        order = [name] + [n for n in registry._priority if n != name]
        registry.set_priority(order)
    return mod


def uninstall(name: str = BACKEND_NAME) -> None:
    from comfy_kitchen.registry import registry
    registry.disable(name)
    registry.set_priority([n for n in registry._priority if n != name])
