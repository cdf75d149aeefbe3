"""``NVFP4Linear``: a linear layer that keeps its weight in NVFP4 and runs the B200 kernels directly.

Same constructor, state-dict keys and forward semantics as the reference sample layer
(``samples/nvfp4_linear.py:10-80``: ``weight`` packed uint8 ``[N, K/2]``, ``weight_scale`` e4m3 block scales in the
128x4 tiled layout stored as uint8, ``weight_scale_2`` fp32 per-tensor scale, optional ``input_scale``; without
``input_scale`` the activation scale is recomputed per call like ``TensorCoreNVFP4Layout.quantize`` does,
``comfy_kitchen/tensor/nvfp4.py:53-84``), but without the QuantizedTensor / dispatch machinery in between: forward
is ``quantize_nvfp4`` followed by ``scaled_mm_nvfp4``.  Checkpoints written for the reference layer load unchanged.
"""
from __future__ import annotations

import torch
import torch.nn as nn

from . import ops


class NVFP4Linear(nn.Module):
    def __init__(self, in_features: int, out_features: int, bias: bool = True, device=None, dtype=None) -> None:
        super().__init__()
        self.device = "cuda" if device is None else device
        self.compute_dtype = torch.bfloat16 if dtype is None else dtype
        self.in_features = in_features
        self.out_features = out_features
        kp, np_ = ops.roundup(in_features, 16), ops.roundup(out_features, 16)
        self.register_buffer("weight", torch.zeros((np_, kp // 2), dtype=torch.uint8, device=self.device))
        self.register_buffer("weight_scale", torch.zeros((ops.roundup(np_, 128), ops.roundup(kp // 16, 4)),
                                                         dtype=torch.uint8, device=self.device))
        self.register_buffer("weight_scale_2", torch.ones((), dtype=torch.float32, device=self.device))
        self.input_scale = None
        if bias:
            self.bias = nn.Parameter(torch.zeros(out_features, dtype=self.compute_dtype, device=self.device),
                                     requires_grad=False)
        else:
            self.register_parameter("bias", None)

    @classmethod
    def from_float(cls, weight: torch.Tensor, bias: torch.Tensor | None = None,
                   input_scale: torch.Tensor | None = None) -> "NVFP4Linear":
        """Quantize a floating-point [N, K] weight on its (CUDA) device."""
        n, k = weight.shape
        lin = cls(k, n, bias=bias is not None, device=weight.device, dtype=weight.dtype)
        scale = ops.dynamic_scale_nvfp4(weight.contiguous())
        q, sf = ops.quantize_nvfp4(weight.contiguous(), scale, pad_16x=(n % 16 != 0 or k % 16 != 0))
        lin.weight.copy_(q)
        lin.weight_scale.copy_(sf.view(torch.uint8))
        lin.weight_scale_2.copy_(scale)
        if bias is not None:
            lin.bias.data.copy_(bias)
        if input_scale is not None:
            lin.input_scale = input_scale.to(device=weight.device, dtype=torch.float32).reshape(())
        return lin

    def _load_from_state_dict(self, state_dict, prefix, local_metadata, strict, missing_keys, unexpected_keys, error_msgs):
        # same tolerant shapes as the reference layer: scales may come flat and as uint8 or float8_e4m3fn
        ws = state_dict.get(prefix + "weight_scale")
        if ws is not None:
            if ws.dtype != torch.uint8:
                ws = ws.view(torch.uint8)
            state_dict[prefix + "weight_scale"] = ws.reshape(self.weight_scale.shape)
        ws2 = state_dict.get(prefix + "weight_scale_2")
        if ws2 is not None:
            state_dict[prefix + "weight_scale_2"] = ws2.to(torch.float32).reshape(())
        inp = state_dict.pop(prefix + "input_scale", None)
        self.input_scale = None if inp is None else inp.to(device=self.device, dtype=torch.float32).reshape(())
        super()._load_from_state_dict(state_dict, prefix, local_metadata, strict, missing_keys, unexpected_keys, error_msgs)

    def state_dict(self, *args, **kwargs):
        sd = super().state_dict(*args, **kwargs)
        prefix = kwargs.get("prefix", "")
        if self.input_scale is not None:
            sd[prefix + "input_scale"] = self.input_scale
        return sd

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        lead = x.shape[:-1]
        x2 = x.reshape(-1, self.in_features)
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        out_dtype = x.dtype if x.dtype in (torch.float16, torch.bfloat16) else self.compute_dtype
        bias = self.bias
        if bias is not None and bias.shape[0] != self.weight.shape[0]:   # out_features padded to 16 rows
            bias = torch.nn.functional.pad(bias, (0, self.weight.shape[0] - bias.shape[0]))
        # one library call: activation scale, quantization of x (rows padded to 16) and the GEMM.  The quantized
        # activation sits in a per-device workspace, so calls on one device must be ordered on one stream.
        y = ops.linear_nvfp4(x2, self.weight, self.weight_scale, self.weight_scale_2,
                             input_scale=self.input_scale, bias=bias, out_dtype=out_dtype)
        if y.shape[1] != self.out_features:
            y = y[:, : self.out_features]
        return y if len(lead) == 1 else y.reshape(*lead, self.out_features)

    def forward_unfused(self, x: torch.Tensor) -> torch.Tensor:
        """The same result through the three operators of the reference interface, one call each."""
        lead = x.shape[:-1]
        x2 = x.reshape(-1, self.in_features)
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        m = x2.shape[0]
        scale = self.input_scale if self.input_scale is not None else ops.dynamic_scale_nvfp4(x2)
        pad = m % 16 != 0 or self.in_features % 16 != 0
        qx, sfx = ops.quantize_nvfp4(x2, scale, pad_16x=pad)
        out_dtype = x.dtype if x.dtype in (torch.float16, torch.bfloat16) else self.compute_dtype
        bias = self.bias
        if bias is not None and bias.shape[0] != self.weight.shape[0]:
            bias = torch.nn.functional.pad(bias, (0, self.weight.shape[0] - bias.shape[0]))
        y = ops.scaled_mm_nvfp4(qx, self.weight, scale, self.weight_scale_2, sfx,
                                self.weight_scale.view(torch.float8_e4m3fn), bias=bias, out_dtype=out_dtype)
        return y[:m, : self.out_features].reshape(*lead, self.out_features)
