"""The GEMM entry point that brings its own scratch (ck_b200_scaled_mm_nvfp4_static_scratch).

Some hosts of this library may launch kernels but cannot get device memory when they call: a plugin inside another
framework's pre-planned or captured execution, a real-time loop with a frozen memory plan, an embedding that keeps the
CUDA allocator to itself.  They cannot pass the split-K workspace, so the library carries one.  This test calls the
entry point through the C ABI with raw pointers, several times in a row on different operands (the array is shared and
keeps the previous call's contents), and compares bit for bit with the regular entry point, which gets a
caller-provided workspace, and within the GEMM tolerance with the CPU oracle.
It is collected last so that a failure here leaves every other test already run."""
from __future__ import annotations

import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu
REL_RMS_TOL = 1e-2   # the tolerance of the other GEMM tests


def _operands(ckb, M, N, K, seed):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn((M, K), generator=g).to(torch.bfloat16).cuda()
    w = (torch.randn((N, K), generator=g) * 0.02).to(torch.bfloat16).cuda()
    tsx = (x.abs().amax().float() / 2688).reshape(1)
    tsw = (w.abs().amax().float() / 2688).reshape(1)
    qx, sfx = ckb.quantize_nvfp4(x, tsx)
    qw, sfw = ckb.quantize_nvfp4(w, tsw)
    bias = (torch.randn(N, generator=g) * 0.1).to(torch.bfloat16).cuda()
    return qx, sfx, tsx, qw, sfw, tsw, bias


# (M, N, K, output dtype code): all take split-K (one tile row, several K stages per SM); the third is exactly at the
# limit of M * N = 1 048 576 outputs (two fp32 partial sums each fill the 8 MiB array), the fourth writes fp32.
# For each of them the built-in 8 MiB array and the regular entry point's 32 MiB workspace lead to the same split
# count, so the two results must be bit-identical, not merely close.
SHAPES = [(16, 4096, 10240, 2), (64, 2048, 4096, 2), (128, 8192, 1024, 2), (32, 1024, 2048, 0)]
OUT_DTYPE = {0: torch.float32, 1: torch.float16, 2: torch.bfloat16}


def test_static_scratch_entry_point_matches_regular_one():
    import numpy as np

    import comfy_kitchen_b200 as ckb
    from comfy_kitchen_b200 import _lib
    from helpers import from_bits, to_bits
    from oracle import oracle as o
    o.build()
    L = _lib.load()
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    for call, (M, N, K, code) in enumerate(SHAPES):   # calls in a row on different operands: the array is shared
        dt = OUT_DTYPE[code]
        qx, sfx, tsx, qw, sfw, tsw, bias = _operands(ckb, M, N, K, seed=100 + call)
        n0 = ckb.launches()
        expected = ckb.scaled_mm_nvfp4(qx, qw, tsx, tsw, sfx, sfw, bias=bias, out_dtype=dt)
        regular_launches = ckb.launches() - n0
        regular_splits = L.ck_b200_query(_lib.QUERY_LAST_GEMM_SPLITS)
        out = torch.full((M, N), float("nan"), dtype=dt, device="cuda")
        n0 = ckb.launches()
        rc = L.ck_b200_scaled_mm_nvfp4_static_scratch(
            qx.data_ptr(), sfx.data_ptr(), qw.data_ptr(), sfw.data_ptr(), tsx.data_ptr(), tsw.data_ptr(), None,
            bias.data_ptr(), 2, out.data_ptr(), code, M, N, K, stream)
        assert rc == 0, _lib.last_error()
        # the split-K path ran (partial sums through the built-in scratch, then the reduction kernel), cut into as
        # many pieces as the regular call's
        assert ckb.launches() - n0 == regular_launches == 2
        assert L.ck_b200_query(_lib.QUERY_LAST_GEMM_SPLITS) == regular_splits > 1
        torch.cuda.synchronize()
        assert torch.isfinite(out.float()).all()
        assert torch.equal(out, expected), "static-scratch result differs from the regular entry point's"
        # and against the CPU oracle on the same quantized operands
        ref = o.scaled_mm_nvfp4(to_bits(qx), to_bits(qw), float(tsx), float(tsw), to_bits(sfx), to_bits(sfw),
                                bias=to_bits(bias), out_dtype=code)
        ref = torch.from_numpy(ref) if code == 0 else from_bits(ref, code).float()
        got = out.float().cpu()
        err = (got - ref).double().pow(2).mean().sqrt() / ref.double().pow(2).mean().sqrt()
        assert float(err) <= REL_RMS_TOL
    assert ckb.read_device_status() == 0


def test_static_scratch_entry_point_rejects_sizes_beyond_its_limits():
    from comfy_kitchen_b200 import _lib
    L = _lib.load()
    dummy = torch.zeros(1 << 20, dtype=torch.uint8, device="cuda")
    p = dummy.data_ptr()
    rc = L.ck_b200_scaled_mm_nvfp4_static_scratch(p, p, p, p, p, p, None, None, 2, p, 2, 256, 1024, 1024, None)
    assert rc == 1 and "128 rows" in _lib.last_error()
    rc = L.ck_b200_scaled_mm_nvfp4_static_scratch(p, p, p, p, p, p, None, None, 2, p, 2, 128, 16384, 1024, None)
    assert rc == 1 and "beyond the limit" in _lib.last_error()
