"""NVFP4Linear on the GPU: state-dict round trip in the reference checkpoint format and forward parity with the
CPU oracle (quantize with the layout's dynamic scale, dequantize -> fp32 matmul)."""
from __future__ import annotations

import numpy as np
import pytest
import torch

from helpers import from_bits, seeded_randn, to_bits

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("shape", [(64, 256, 512), (49, 200, 96), (3, 1024, 2048)], ids=lambda s: "x".join(map(str, s)))
@pytest.mark.parametrize("static_input_scale", [False, True])
def test_linear_forward_matches_oracle(shape, static_input_scale, oracle):
    import comfy_kitchen_b200 as ckb
    M, N, K = shape
    w = seeded_randn((N, K), seed=1, std=0.02).cuda()
    b = seeded_randn((1, N), seed=2, std=0.1).reshape(N).cuda()
    x = seeded_randn((2, M, K), seed=3).cuda()           # leading batch dimension
    inp = torch.tensor(0.0123, dtype=torch.float32) if static_input_scale else None
    lin = ckb.NVFP4Linear.from_float(w, b, input_scale=inp)
    y = lin(x)
    assert tuple(y.shape) == (2, M, N) and y.dtype == torch.bfloat16
    assert torch.equal(y, lin.forward_unfused(x)), "the one-call linear differs from the three operators"

    x2 = x.reshape(-1, K).cpu()
    ts_w = oracle.dynamic_scale(to_bits(w), 2)
    ts_x = float(np.float32(0.0123)) if static_input_scale else oracle.dynamic_scale(to_bits(x2), 2)
    assert np.float32(ts_w) == np.float32(lin.weight_scale_2.item())
    qw, sfw = oracle.quantize_nvfp4(to_bits(w), 2, ts_w, pad_16x=True)
    qx, sfx = oracle.quantize_nvfp4(to_bits(x2), 2, ts_x, pad_16x=True)
    assert np.array_equal(qw, lin.weight.cpu().numpy()) and np.array_equal(sfw, lin.weight_scale.cpu().numpy())
    bias_p = np.zeros(qw.shape[0], np.uint16)
    bias_p[:N] = to_bits(b)
    ref = from_bits(oracle.scaled_mm_nvfp4(qx, qw, ts_x, ts_w, sfx, sfw, bias=bias_p), 2).float()[: 2 * M, :N]
    got = y.reshape(-1, N).cpu().float()
    rel = float((got - ref).pow(2).mean().sqrt() / ref.pow(2).mean().sqrt())
    assert rel <= 1e-2


def test_linear_state_dict_round_trip():
    import comfy_kitchen_b200 as ckb
    w = seeded_randn((128, 256), seed=5, std=0.02).cuda()
    lin = ckb.NVFP4Linear.from_float(w, None, input_scale=torch.tensor(0.02))
    sd = lin.state_dict()
    assert set(sd) == {"weight", "weight_scale", "weight_scale_2", "input_scale"}
    assert sd["weight"].dtype == torch.uint8 and sd["weight_scale"].dtype == torch.uint8
    # the reference sample stores the block scales flat
    sd = {k: v.clone() for k, v in sd.items()}
    sd["weight_scale"] = sd["weight_scale"].reshape(-1)
    other = ckb.NVFP4Linear(256, 128, bias=False, device="cuda")
    other.load_state_dict(sd)
    x = seeded_randn((32, 256), seed=6).cuda()
    assert torch.equal(lin(x), other(x))


def test_linear_small_m_and_fp16(oracle):
    """M = 1 (split-K path with the workspace's tail as scratch) and fp16 activations through the one-call entry."""
    import comfy_kitchen_b200 as ckb
    w = seeded_randn((512, 1024), seed=7, std=0.02).cuda()
    lin = ckb.NVFP4Linear.from_float(w, None)
    for m, dtype in ((1, torch.bfloat16), (5, torch.float16), (130, torch.bfloat16)):
        x = seeded_randn((m, 1024), seed=8 + m, dtype=dtype).cuda()
        y = lin(x)
        assert y.dtype == dtype and tuple(y.shape) == (m, 512)
        assert torch.equal(y, lin.forward_unfused(x))
    assert ckb.read_device_status() == 0


FUSED_SHAPES = [(256, 256, 512), (300, 384, 1024), (1000, 768, 3072), (4608, 3072, 3072), (520, 1024, 416),
                (2049, 512, 12288)]


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16], ids=["bf16", "fp16"])
def test_linear_quantizer_inside_the_gemm(dtype):
    """M > 128 and N > 128: one kernel quantizes the activations beside the tensor-core main loop.  Results must be
    bit-identical to the separate operators, over a sequence of shapes that share the workspace (rows that are not
    multiples of 16 or 128, K that is not a multiple of 128), with a dynamic and with a static activation scale."""
    import comfy_kitchen_b200 as ckb
    old = ckb.set_tuning(4, 1)
    try:
        _fused_shapes(ckb, dtype)
    finally:
        ckb.set_tuning(4, old)
    assert ckb.read_device_status() == 0


def _fused_shapes(ckb, dtype):
    for i, (M, N, K) in enumerate(FUSED_SHAPES * 2):
        w = seeded_randn((N, K), seed=20 + i, std=0.02).cuda()
        b = seeded_randn((1, N), seed=40 + i, std=0.1, dtype=dtype).reshape(N).cuda()
        x = seeded_randn((M, K), seed=60 + i, dtype=dtype, outlier_cols=3).cuda()
        inp = torch.tensor(0.0171, dtype=torch.float32) if i % 2 else None
        lin = ckb.NVFP4Linear.from_float(w, b, input_scale=inp)
        want = lin.forward_unfused(x)
        for _ in range(3):
            got = lin(x)
            assert got.dtype == dtype and torch.equal(got, want), f"{M}x{N}x{K}: fused linear differs"


def test_linear_quantizer_inside_the_gemm_is_opt_in_and_replays():
    import comfy_kitchen_b200 as ckb
    M, N, K = 1024, 1024, 2048
    w = seeded_randn((N, K), seed=81, std=0.02).cuda()
    x = seeded_randn((M, K), seed=82).cuda()
    lin = ckb.NVFP4Linear.from_float(w, None, input_scale=torch.tensor(0.02))
    want = lin.forward_unfused(x)
    n0 = ckb.launches()
    assert torch.equal(lin(x), want)
    assert ckb.launches() - n0 == 2, "default: quantizer kernel, then GEMM kernel"
    old = ckb.set_tuning(4, 1)
    try:
        _fused_one_kernel_and_replays(ckb, lin, x, want, M, K)
    finally:
        ckb.set_tuning(4, old)
    assert ckb.read_device_status() == 0


def _fused_one_kernel_and_replays(ckb, lin, x, want, M, K):
    n0 = ckb.launches()
    y = lin(x)
    assert ckb.launches() - n0 == 1, "the fused linear is one kernel when the activation scale is static"
    assert torch.equal(y, want)
    # replays of a captured call: the progress counters are left at zero by each replay
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        lin(x)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g, stream=side):
        y = lin(x)
    for it in range(4):
        x.copy_(seeded_randn((M, K), seed=90 + it).cuda())
        g.replay()
        torch.cuda.synchronize()
        assert torch.equal(y, lin.forward_unfused(x))
    assert ckb.read_device_status() == 0
