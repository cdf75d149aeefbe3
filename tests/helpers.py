"""Conversions between torch tensors and the numpy bit-pattern arrays the CPU oracle works on."""
from __future__ import annotations

import numpy as np
import torch

CODE = {torch.float32: 0, torch.float16: 1, torch.bfloat16: 2}
TORCH_DT = {0: torch.float32, 1: torch.float16, 2: torch.bfloat16}


def to_bits(t: torch.Tensor) -> np.ndarray:
    t = t.detach().cpu().contiguous()
    if t.dtype == torch.float32:
        return t.numpy().copy()
    if t.dtype in (torch.float16, torch.bfloat16):
        return t.view(torch.int16).numpy().view(np.uint16).copy()
    return t.view(torch.uint8).numpy().copy()


def from_bits(a: np.ndarray, code: int) -> torch.Tensor:
    if code == 0:
        return torch.from_numpy(np.ascontiguousarray(a, np.float32).copy())
    return torch.from_numpy(np.ascontiguousarray(a).view(np.int16).copy()).view(TORCH_DT[code])


def seeded_randn(shape, seed, std=1.0, dtype=torch.bfloat16, outlier_cols=0):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(shape, generator=g, dtype=torch.float32) * std
    if outlier_cols:
        idx = torch.randperm(shape[1], generator=g)[:outlier_cols]
        x[:, idx] *= 20
    return x.to(dtype)


def amax_scale(x: torch.Tensor) -> torch.Tensor:
    """fp32 amax / (448*6), the scale the reference tests use (tests/test_qdq.py:478-483)."""
    return (x.abs().amax().float() / (448.0 * 6.0)).reshape(())
