"""MXFP8 on the GPU through the C ABI: quantize / dequantize bit-exact against the reference vectors and the CPU
oracle, GEMM within the relative-RMS tolerance of the restated dequantize -> fp32 matmul."""
from __future__ import annotations

import os

import numpy as np
import pytest
import torch

from helpers import CODE, TORCH_DT, from_bits, seeded_randn, to_bits

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))
REL_RMS_TOL = 1e-2   # the tolerance of the NVFP4 GEMM contract, applied to its sibling


@pytest.fixture(scope="module")
def ckb():
    import comfy_kitchen_b200 as m
    assert torch.cuda.is_available()
    return m


@pytest.fixture(scope="module")
def mx_golden():
    return np.load(os.path.join(HERE, "golden", "mxfp8_golden.npz"))


def mx_case_names():
    return [str(n) for n in np.load(os.path.join(HERE, "golden", "mxfp8_golden.npz"))["quantize_cases"]]


@pytest.mark.parametrize("name", mx_case_names())
def test_quantize_golden(name, mx_golden, ckb):
    dtype, pad = (int(v) for v in mx_golden[f"{name}/meta"])
    x = from_bits(mx_golden[f"{name}/x"], dtype).cuda()
    q, sf = ckb.quantize_mxfp8(x, pad_32x=bool(pad))
    assert q.dtype == torch.float8_e4m3fn and sf.dtype == torch.float8_e8m0fnu
    assert np.array_equal(to_bits(sf), mx_golden[f"{name}/sf"]), "scale bytes differ from the reference"
    assert np.array_equal(to_bits(q), mx_golden[f"{name}/q"]), "data bytes differ from the reference"
    for code in (0, 1, 2):
        key = f"{name}/dq{code}"
        if key in mx_golden.files:
            d = ckb.dequantize_mxfp8(q, sf, TORCH_DT[code])
            got = to_bits(d)
            want = mx_golden[key]
            assert np.array_equal(got.view(np.uint32) if code == 0 else got, want.view(np.uint32) if code == 0 else want)


@pytest.mark.parametrize("shape", [(32, 32), (96, 4096), (1000, 333), (4608, 3072), (129, 160), (16384, 5120)],
                         ids=lambda s: "x".join(map(str, s)))
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32], ids=["bf16", "f16", "f32"])
def test_quantize_vs_oracle(shape, dtype, ckb, oracle):
    if dtype != torch.bfloat16 and shape[0] * shape[1] > (1 << 23):
        pytest.skip("large shapes are covered in bf16")
    x = seeded_randn(shape, seed=shape[0] + shape[1], std=3.0, dtype=dtype, outlier_cols=min(4, shape[1]))
    pad = shape[0] % 32 != 0 or shape[1] % 32 != 0
    q, sf = ckb.quantize_mxfp8(x.cuda(), pad_32x=pad)
    q_ref, sf_ref = oracle.quantize_mxfp8(to_bits(x), CODE[dtype], pad)
    assert tuple(q.shape) == q_ref.shape and tuple(sf.shape) == sf_ref.shape
    assert np.array_equal(to_bits(sf), sf_ref) and np.array_equal(to_bits(q), q_ref)
    d = ckb.dequantize_mxfp8(q, sf, dtype)
    assert np.array_equal(to_bits(d), oracle.dequantize_mxfp8(q_ref, sf_ref, CODE[dtype]))


def test_scale_padding_is_written(ckb):
    poison = torch.full((1 << 22,), 0xAB, dtype=torch.uint8, device="cuda")
    del poison
    x = seeded_randn((65, 96), seed=1).cuda()
    q, sf = ckb.quantize_mxfp8(x, pad_32x=True)
    sfb = sf.view(torch.uint8).cpu()
    assert tuple(sfb.shape) == (128, 4)
    assert int((sfb != 0).sum()) <= 96 * 3     # only real blocks of padded rows < 96 may be non-zero
    qq = q.view(torch.uint8).cpu()
    assert int(qq[65:].abs().sum()) == 0 and int(qq[:, 96:].sum()) == 0 if qq.shape[1] > 96 else True


def test_bad_arguments(ckb):
    x = torch.zeros((30, 64), device="cuda", dtype=torch.bfloat16)
    with pytest.raises(AssertionError):
        ckb.quantize_mxfp8(x)
    with pytest.raises(TypeError):
        ckb.quantize_mxfp8(torch.zeros((32, 64), dtype=torch.bfloat16))


@pytest.fixture(params=[0, 1, 2, 3], ids=["auto", "bn128", "bn256", "pair256"])
def gemm_variant(request, ckb):
    prev = ckb.set_tuning(1, request.param)
    yield request.param
    ckb.set_tuning(1, prev)


GEMM_SHAPES = [(32, 128, 64), (96, 160, 256), (128, 256, 128), (256, 512, 1024), (300, 384, 4096), (1, 1024, 4096),
               (64, 4096, 10240), (1024, 3072, 3072), (520, 1032, 96)]


@pytest.mark.parametrize("shape", GEMM_SHAPES, ids=lambda s: "x".join(map(str, s)))
@pytest.mark.parametrize("with_bias", [False, True])
def test_gemm_vs_oracle(shape, with_bias, ckb, oracle, gemm_variant):
    M, N, K = shape
    x = seeded_randn((M, K), seed=21).cuda()
    w = seeded_randn((N, K), seed=22, std=0.05).cuda()
    bias = seeded_randn((1, N), seed=23, std=0.5).reshape(N).cuda() if with_bias else None
    qx, sfx = ckb.quantize_mxfp8(x, pad_32x=True)
    qw, sfw = ckb.quantize_mxfp8(w, pad_32x=True)
    # operands padded to multiples of 32 rows by the quantizer: the product has the padded shape
    bias_p = None if bias is None else torch.nn.functional.pad(bias, (0, qw.shape[0] - N))
    y = ckb.scaled_mm_mxfp8(qx, qw, sfx, sfw, bias=bias_p)
    assert tuple(y.shape) == (qx.shape[0], qw.shape[0])
    ref = oracle.scaled_mm_mxfp8(to_bits(qx), to_bits(qw), to_bits(sfx), to_bits(sfw),
                                 bias=None if bias_p is None else to_bits(bias_p), out_dtype=0)
    got = y.float().cpu().numpy()
    rel = float(np.sqrt(((got - ref) ** 2).mean()) / np.sqrt((ref ** 2).mean()))
    assert ckb.read_device_status() == 0
    assert rel <= REL_RMS_TOL, f"relative RMS error {rel:.3e}"


def test_gemm_golden(mx_golden, ckb, gemm_variant):
    for name in ("gemm_32x128x64", "gemm_96x160x256_bias"):
        qa = torch.from_numpy(mx_golden[f"{name}/qa"]).cuda().view(torch.float8_e4m3fn)
        qb = torch.from_numpy(mx_golden[f"{name}/qb"]).cuda().view(torch.float8_e4m3fn)
        sa = torch.from_numpy(mx_golden[f"{name}/sa"]).cuda().view(torch.float8_e8m0fnu)
        sb = torch.from_numpy(mx_golden[f"{name}/sb"]).cuda().view(torch.float8_e8m0fnu)
        bias = from_bits(mx_golden[f"{name}/bias"], 2).cuda() if f"{name}/bias" in mx_golden.files else None
        y = ckb.scaled_mm_mxfp8(qa, qb, sa, sb, bias=bias, out_dtype=torch.float32).cpu().numpy()
        ref = mx_golden[f"{name}/y_f32"]
        rel = float(np.sqrt(((y - ref) ** 2).mean()) / np.sqrt((ref ** 2).mean()))
        assert rel <= 1e-5, f"{name}: relative RMS error {rel:.3e}"
