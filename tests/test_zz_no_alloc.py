"""The GEMM entry point that brings its own scratch (ck_b200_scaled_mm_nvfp4_static_scratch).

Some hosts of this library may launch kernels but cannot get device memory when they call: a plugin inside another
framework's pre-planned or captured execution, a real-time loop with a frozen memory plan, an embedding that keeps the
CUDA allocator to itself.  They cannot pass the split-K workspace, so the library carries one.  This test calls the
entry point through the C ABI with raw pointers, twice in a row on different operands (the array is shared and keeps
the previous call's contents), and compares with the regular entry point, which gets a caller-provided workspace.
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


def test_static_scratch_entry_point_matches_regular_one():
    import comfy_kitchen_b200 as ckb
    from comfy_kitchen_b200 import _lib
    L = _lib.load()
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    for call, (M, N, K) in enumerate([(16, 4096, 10240), (64, 2048, 4096)]):   # two calls in a row, both split-K shapes
        qx, sfx, tsx, qw, sfw, tsw, bias = _operands(ckb, M, N, K, seed=100 + call)
        expected = ckb.scaled_mm_nvfp4(qx, qw, tsx, tsw, sfx, sfw, bias=bias, out_dtype=torch.bfloat16)
        out = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device="cuda")
        rc = L.ck_b200_scaled_mm_nvfp4_static_scratch(
            qx.data_ptr(), sfx.data_ptr(), qw.data_ptr(), sfw.data_ptr(), tsx.data_ptr(), tsw.data_ptr(), None,
            bias.data_ptr(), 2, out.data_ptr(), 2, M, N, K, stream)
        assert rc == 0, _lib.last_error()
        torch.cuda.synchronize()
        assert torch.isfinite(out.float()).all()
        err = (out.float() - expected.float()).pow(2).mean().sqrt() / expected.float().pow(2).mean().sqrt()
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
