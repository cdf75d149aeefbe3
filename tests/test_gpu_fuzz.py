"""Seeded random shapes, dtypes, padding and scales through both quantizers and dequantizers against the CPU oracle
(bit-exact), and random small GEMMs against the oracle's dequantize -> matmul restatement."""
from __future__ import annotations

import numpy as np
import pytest
import torch

from helpers import CODE, from_bits, to_bits

pytestmark = pytest.mark.gpu
DTYPES = [torch.bfloat16, torch.float16, torch.float32]


def _cases(seed, n, max_rows, max_cols):
    rng = np.random.default_rng(seed)
    out = []
    for i in range(n):
        rows = int(rng.integers(1, max_rows))
        cols = int(rng.integers(1, max_cols))
        if rng.random() < 0.4:          # aligned shapes take the bounds-free walks
            rows, cols = (rows + 127) // 128 * 128, (cols + 127) // 128 * 128
        out.append((i, rows, cols, DTYPES[int(rng.integers(0, 3))], float(10.0 ** rng.uniform(-3, 2)), bool(rng.integers(0, 2))))
    return out


@pytest.mark.parametrize("case", _cases(1, 24, 700, 1500), ids=lambda c: f"{c[0]}-{c[1]}x{c[2]}")
def test_nvfp4_quantize_fuzz(case, oracle):
    import comfy_kitchen_b200 as ckb
    i, rows, cols, dtype, std, hi_first = case
    g = torch.Generator().manual_seed(100 + i)
    x = (torch.randn((rows, cols), generator=g) * std).to(dtype)
    x[torch.rand((rows, cols), generator=g) < 0.05] = 0.0
    ts = torch.tensor(float(x.abs().amax().float()) / 2688.0 if i % 2 else std * 0.0123, dtype=torch.float32)
    q, sf = ckb.quantize_nvfp4(x.cuda(), ts.cuda(), pad_16x=True, hi_first=hi_first)
    q_ref, sf_ref = oracle.quantize_nvfp4(to_bits(x), CODE[dtype], float(ts), pad_16x=True, hi_first=hi_first)
    assert np.array_equal(to_bits(sf), sf_ref) and np.array_equal(to_bits(q), q_ref)
    d = ckb.dequantize_nvfp4(q, ts.cuda(), sf, dtype, hi_first=hi_first)
    d_ref = oracle.dequantize_nvfp4(q_ref, float(ts), sf_ref, CODE[dtype], hi_first=hi_first)
    got = to_bits(d)
    assert np.array_equal(got.view(np.uint32) if dtype == torch.float32 else got,
                          d_ref.view(np.uint32) if dtype == torch.float32 else d_ref)


@pytest.mark.parametrize("case", _cases(2, 24, 700, 1500), ids=lambda c: f"{c[0]}-{c[1]}x{c[2]}")
def test_mxfp8_quantize_fuzz(case, oracle):
    import comfy_kitchen_b200 as ckb
    i, rows, cols, dtype, std, _ = case
    if dtype == torch.float32:
        dtype = torch.bfloat16 if i % 2 else torch.float16   # the exact-ceiling rule is pinned on 16-bit inputs
    g = torch.Generator().manual_seed(200 + i)
    x = (torch.randn((rows, cols), generator=g) * std).to(dtype)
    x[torch.rand((rows, cols), generator=g) < 0.05] = 0.0
    q, sf = ckb.quantize_mxfp8(x.cuda(), pad_32x=True)
    q_ref, sf_ref = oracle.quantize_mxfp8(to_bits(x), CODE[dtype], True)
    assert np.array_equal(to_bits(sf), sf_ref) and np.array_equal(to_bits(q), q_ref)
    d = ckb.dequantize_mxfp8(q, sf, dtype)
    assert np.array_equal(to_bits(d), oracle.dequantize_mxfp8(q_ref, sf_ref, CODE[dtype]))


@pytest.mark.parametrize("seed", range(10))
def test_gemm_fuzz(seed, oracle):
    import comfy_kitchen_b200 as ckb
    rng = np.random.default_rng(300 + seed)
    M, N, K = int(rng.integers(1, 600)), int(rng.integers(1, 80)) * 8, int(rng.integers(1, 40)) * 32
    g = torch.Generator().manual_seed(400 + seed)
    x = torch.randn((M, K), generator=g).to(torch.bfloat16)
    w = (torch.randn((N, K), generator=g) * 0.05).to(torch.bfloat16)
    bias = torch.randn(N, generator=g).to(torch.bfloat16) if seed % 2 else None
    tsx = torch.tensor(float(x.abs().amax()) / 2688.0)
    tsw = torch.tensor(float(w.abs().amax()) / 2688.0)
    qx, sfx = ckb.quantize_nvfp4(x.cuda(), tsx.cuda(), pad_16x=True)
    qw, sfw = ckb.quantize_nvfp4(w.cuda(), tsw.cuda(), pad_16x=True)
    Np = qw.shape[0]
    bias_p = None if bias is None else torch.nn.functional.pad(bias, (0, Np - N)).cuda()
    y = ckb.scaled_mm_nvfp4(qx, qw, tsx.cuda(), tsw.cuda(), sfx, sfw, bias=bias_p, out_dtype=torch.float32)
    ref = oracle.scaled_mm_nvfp4(to_bits(qx), to_bits(qw), float(tsx), float(tsw), to_bits(sfx), to_bits(sfw),
                                 bias=None if bias_p is None else to_bits(bias_p), out_dtype=0)
    got = y.cpu().numpy()
    rel = float(np.sqrt(((got - ref) ** 2).mean()) / max(np.sqrt((ref ** 2).mean()), 1e-30))
    assert ckb.read_device_status() == 0 and rel <= 1e-2, f"M={M} N={N} K={K}: relative RMS error {rel:.3e}"
