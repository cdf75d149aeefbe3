"""GPU parity of scaled_mm_nvfp4 (through the C ABI) against the CPU oracle (dequantize -> fp32 matmul), the
reference golden vectors and, at the full benchmark sizes, torch's cuBLASLt NVFP4 matmul on the same operands.

Tolerance (floating point): relative RMS error <= 1e-2 against the reference path on identical quantized
operands; in practice the error is bf16 output rounding (~2e-3)."""
from __future__ import annotations

import numpy as np
import pytest
import torch

from helpers import amax_scale, from_bits, seeded_randn, to_bits

pytestmark = pytest.mark.gpu
REL_RMS_TOL = 1e-2


@pytest.fixture(scope="module")
def ckb():
    import comfy_kitchen_b200 as m
    assert torch.cuda.is_available()
    return m


@pytest.fixture(params=[1, 2, 3, 4, 5, 6],
                ids=["bn128", "bn256", "pair256", "pair256-k128", "short-rows-bn64", "short-rows-cluster-splitk"])
def variant(request, ckb):
    prev = ckb.set_tuning(1, request.param)
    yield request.param
    ckb.set_tuning(1, prev)
    assert ckb.read_device_status() == 0, "a bounded wait ran out inside the GEMM kernel"


def rel_rms(y, ref):
    y, ref = y.double(), ref.double()
    return float(((y - ref).pow(2).mean().sqrt()) / ref.pow(2).mean().sqrt().clamp_min(1e-30))


def quantized_operands(ckb, M, N, K, seed, outliers=False):
    x = seeded_randn((M, K), seed=seed, outlier_cols=max(1, K // 1000) if outliers else 0).cuda()
    w = seeded_randn((N, K), seed=seed + 1, std=0.02).cuda()
    tsx, tsw = amax_scale(x).cuda(), amax_scale(w).cuda()
    padx = M % 16 != 0
    qx, sfx = ckb.quantize_nvfp4(x, tsx, pad_16x=padx)
    qw, sfw = ckb.quantize_nvfp4(w, tsw, pad_16x=N % 16 != 0)
    qw = qw[:N].contiguous()      # the scale tensor is padded to 128 rows either way
    return x, w, qx, sfx, tsx, qw, sfw, tsw


def torch_scaled_mm(qx, sfx, tsx, qw, sfw, tsw, bias=None, out_dtype=torch.bfloat16):
    """cuBLASLt NVFP4 through torch on the same operands: what the reference eager backend calls
    (comfy_kitchen/backends/eager/quantization.py:225-249, comfy_kitchen/scaled_mm_v2.py:113-126)."""
    from torch.nn.functional import ScalingType, SwizzleType, scaled_mm
    return scaled_mm(
        qx.view(torch.float4_e2m1fn_x2), qw.view(torch.float4_e2m1fn_x2).t(),
        scale_a=[sfx.view(-1), tsx.reshape(())], scale_b=[sfw.view(-1), tsw.reshape(())],
        scale_recipe_a=[ScalingType.BlockWise1x16, ScalingType.TensorWise],
        scale_recipe_b=[ScalingType.BlockWise1x16, ScalingType.TensorWise],
        swizzle_a=[SwizzleType.SWIZZLE_32_4_4, SwizzleType.NO_SWIZZLE],
        swizzle_b=[SwizzleType.SWIZZLE_32_4_4, SwizzleType.NO_SWIZZLE],
        bias=bias, output_dtype=out_dtype)


@pytest.mark.parametrize("name", ["gemm_64x128x256", "gemm_48x72x96"])
def test_gemm_golden(name, golden, ckb, variant):
    qa = torch.from_numpy(golden[f"{name}/qa"].copy()).cuda()
    qb = torch.from_numpy(golden[f"{name}/qb"].copy()).cuda()
    sfa = torch.from_numpy(golden[f"{name}/sfa"].copy()).cuda().view(torch.float8_e4m3fn)
    sfb = torch.from_numpy(golden[f"{name}/sfb"].copy()).cuda().view(torch.float8_e4m3fn)
    tsa, tsb = (torch.tensor(float(v), dtype=torch.float32).cuda() for v in golden[f"{name}/ts"])
    bias = from_bits(golden[f"{name}/bias"], 2).cuda() if f"{name}/bias" in golden else None
    y = ckb.scaled_mm_nvfp4(qa, qb, tsa, tsb, sfa, sfb, bias=bias, out_dtype=torch.bfloat16)
    ref = from_bits(golden[f"{name}/y"], 2)
    assert y.shape == ref.shape and y.dtype == torch.bfloat16
    assert rel_rms(y.cpu().float(), ref.float()) <= REL_RMS_TOL


SMALL = [(256, 1024, 1024), (128, 128, 256), (16, 8, 32), (100, 200, 96), (129, 136, 320), (384, 264, 1024),
         (1, 4096, 4096), (16, 10240, 4096), (64, 4096, 10240), (128, 4096, 4096), (512, 1024, 2048), (300, 520, 2080)]


@pytest.mark.parametrize("mnk", SMALL, ids=lambda s: "x".join(map(str, s)))
@pytest.mark.parametrize("with_bias", [False, True], ids=["nobias", "bias"])
def test_gemm_vs_oracle(mnk, with_bias, ckb, oracle, variant):
    M, N, K = mnk
    if M * N * K > 3e9:
        pytest.skip("too large for the CPU oracle")
    Mp = (M + 15) // 16 * 16
    x, w, qx, sfx, tsx, qw, sfw, tsw = quantized_operands(ckb, M, N, K, seed=M + N + K)
    bias = seeded_randn((1, N), seed=99, std=0.5).reshape(N).cuda() if with_bias else None
    y = ckb.scaled_mm_nvfp4(qx, qw, tsx, tsw, sfx, sfw, bias=bias, out_dtype=torch.bfloat16)
    assert tuple(y.shape) == (Mp, N)
    ref = oracle.scaled_mm_nvfp4(to_bits(qx), to_bits(qw), float(tsx), float(tsw), to_bits(sfx), to_bits(sfw),
                                 bias=None if bias is None else to_bits(bias))
    ref = from_bits(ref, 2).float()
    got = y.cpu().float()
    assert torch.isfinite(got).all()
    assert rel_rms(got[:M], ref[:M]) <= REL_RMS_TOL
    # also elementwise: nothing may be off by more than a few bf16 roundings of the row/column scale
    assert float((got[:M] - ref[:M]).abs().max()) <= 0.05 * float(ref[:M].abs().max()) + 1e-6


def test_gemm_alpha_fp16_fp32_outputs(ckb, oracle, variant):
    M, N, K = 128, 256, 512
    x, w, qx, sfx, tsx, qw, sfw, tsw = quantized_operands(ckb, M, N, K, seed=5)
    a = float(np.float32(0.37) * np.float32(float(tsx)) * np.float32(float(tsw)))
    alpha = torch.tensor(a, dtype=torch.float32).cuda()
    ref = oracle.scaled_mm_nvfp4(to_bits(qx), to_bits(qw), 0.0, 0.0, to_bits(sfx), to_bits(sfw), alpha=a, out_dtype=0)
    ref = torch.from_numpy(ref)
    for dt in (torch.float16, torch.float32, torch.bfloat16):
        y = ckb.scaled_mm_nvfp4(qx, qw, tsx, tsw, sfx, sfw, out_dtype=dt, alpha=alpha)
        assert y.dtype == dt
        assert rel_rms(y.cpu().float(), ref) <= REL_RMS_TOL
    y0 = ckb.scaled_mm_nvfp4(qx, qw, tsx, tsw, sfx, sfw)       # default out dtype
    assert y0.dtype == torch.bfloat16


def test_gemm_first_config_golden(ckb, golden_large, oracle, variant):
    import hashlib
    rng = np.random.default_rng(0)
    x32 = rng.standard_normal((256, 1024), dtype=np.float32)
    w32 = (rng.standard_normal((1024, 1024), dtype=np.float32) * np.float32(0.02)).astype(np.float32)
    xb, wb = oracle.narrow(x32, 2), oracle.narrow(w32, 2)
    if hashlib.sha256(xb.tobytes()).hexdigest() != golden_large["x_bits_sha256"]:
        pytest.skip("numpy generator stream differs")
    tsx = torch.tensor(golden_large["ts_x"], dtype=torch.float32).cuda()
    tsw = torch.tensor(golden_large["ts_w"], dtype=torch.float32).cuda()
    qx, sfx = ckb.quantize_nvfp4(from_bits(xb, 2).cuda(), tsx)
    qw, sfw = ckb.quantize_nvfp4(from_bits(wb, 2).cuda(), tsw)
    assert hashlib.sha256(to_bits(qw).tobytes()).hexdigest() == golden_large["qw_sha256"]
    y = ckb.scaled_mm_nvfp4(qx, qw, tsx, tsw, sfx, sfw)
    ref = from_bits(np.array(golden_large["y_sample_bits"], np.uint16), 2).float()
    assert rel_rms(y.cpu().float()[::8, ::8], ref) <= REL_RMS_TOL
    assert abs(float(y.float().pow(2).mean().sqrt()) - golden_large["y_rms"]) < 1e-2 * golden_large["y_rms"]


FLUX = [(4608, 9216, 3072), (4608, 3072, 3072), (4608, 12288, 3072), (4608, 3072, 12288)]
WAN_T5 = [(32760, 15360, 5120), (32760, 5120, 5120), (32760, 13824, 5120), (32760, 5120, 13824), (512, 10240, 4096),
          (64, 4096, 10240), (16, 10240, 4096)]


@pytest.mark.parametrize("mnk", FLUX + WAN_T5, ids=lambda s: "x".join(map(str, s)))
def test_gemm_full_size_vs_cublaslt(mnk, ckb, variant):
    """Benchmark-sized linears: same quantized operands through torch's cuBLASLt NVFP4 matmul (the kernel behind the
    reference eager backend) and through ours; plus linearity in alpha, which needs no reference at all."""
    M, N, K = mnk
    x, w, qx, sfx, tsx, qw, sfw, tsw = quantized_operands(ckb, M, N, K, seed=K + N, outliers=True)
    y = ckb.scaled_mm_nvfp4(qx, qw, tsx, tsw, sfx, sfw)
    assert torch.isfinite(y.float()).all()
    try:
        ref = torch_scaled_mm(qx, sfx, tsx, qw, sfw, tsw)
    except Exception as e:   # pragma: no cover - depends on the torch / cuBLASLt build on the box
        pytest.skip(f"torch scaled_mm NVFP4 unavailable here: {type(e).__name__}: {e}")
    Mr = min(M, ref.shape[0])
    assert rel_rms(y[:Mr].float(), ref[:Mr].float()) <= REL_RMS_TOL
    # quantization error against the unquantized bf16 linear stays at the format's level (~0.13 RMS on these inputs)
    hp = (x[:1024].float() @ w.float().t())
    assert rel_rms(y[:1024].float(), hp) < 0.25
    # linearity: alpha = 2 * tsx * tsw doubles the output exactly (power-of-two scaling commutes with rounding)
    y2 = ckb.scaled_mm_nvfp4(qx, qw, tsx, tsw, sfx, sfw, alpha=(2.0 * tsx * tsw))
    assert torch.equal(y2.float(), 2.0 * y.float())


@pytest.mark.parametrize("mnk", [(1, 4096, 4096), (16, 4096, 10240), (64, 2048, 4096), (128, 2048, 8192)],
                         ids=lambda s: "x".join(map(str, s)))
def test_split_k_repeats_and_graph_replays(mnk, ckb):
    """Small M is cut along K over the SMs and a second kernel adds the partial sums up in split order: repeated calls
    and replays of a captured call, also on changed operands, give the same bits every time."""
    from comfy_kitchen_b200 import _lib
    M, N, K = mnk
    x, w, qx, sfx, tsx, qw, sfw, tsw = quantized_operands(ckb, M, N, K, seed=7 * M + N)
    first = ckb.scaled_mm_nvfp4(qx, qw, tsx, tsw, sfx, sfw)
    assert _lib.load().ck_b200_query(_lib.QUERY_LAST_GEMM_SPLITS) > 1, "this shape is expected to take split-K"
    for _ in range(4):
        assert torch.equal(ckb.scaled_mm_nvfp4(qx, qw, tsx, tsw, sfx, sfw), first)
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        ckb.scaled_mm_nvfp4(qx, qw, tsx, tsw, sfx, sfw)      # this stream's workspace exists before the capture
    stream.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(stream), torch.cuda.graph(graph):
        y = ckb.scaled_mm_nvfp4(qx, qw, tsx, tsw, sfx, sfw)
    for i in range(3):
        with torch.cuda.stream(stream):
            graph.replay()
        stream.synchronize()
        assert torch.equal(y, first)
    # other operands through the same captured call
    x2, w2, qx2, sfx2, tsx2, qw2, sfw2, tsw2 = quantized_operands(ckb, M, N, K, seed=11 * M + N)
    want = ckb.scaled_mm_nvfp4(qx2, qw2, tsx2, tsw2, sfx2, sfw2)
    for dst, src in ((qx, qx2), (sfx, sfx2), (tsx, tsx2), (qw, qw2), (sfw, sfw2), (tsw, tsw2)):
        dst.copy_(src)
    with torch.cuda.stream(stream):
        graph.replay()
    stream.synchronize()
    assert torch.equal(y, want)
    assert ckb.read_device_status() == 0


SHORT_ROWS = [(16, 10240, 4096), (64, 10240, 4096), (1, 12288, 1024), (33, 10248, 4096), (16, 4096, 10240),
              (64, 4096, 10240), (48, 72, 96), (8, 8, 32), (16, 2560, 4096), (8, 128, 1024), (40, 136, 2080)]


@pytest.mark.parametrize("mnk", SHORT_ROWS, ids=lambda s: "x".join(map(str, s)))
def test_short_row_tiles_match_128_column_tiles(mnk, ckb):
    """M <= 64 on 64-column tiles with two CTAs per SM (a tile reads its scales from half of a 128-row band's chunk
    in tensor memory), and with K split over a thread-block cluster that adds the partial sums up through shared
    memory: bit-identical to the 128-column tiles whenever both cut K into the same number of splits, within the
    GEMM tolerance otherwise; N tails and single-tile problems included."""
    from comfy_kitchen_b200 import _lib
    M, N, K = mnk
    x, w, qx, sfx, tsx, qw, sfw, tsw = quantized_operands(ckb, M, N, K, seed=3 * M + N + K)
    bias = seeded_randn((1, N), seed=5, std=0.5).reshape(N).cuda()
    prev = ckb.set_tuning(1, 1)
    try:
        ref = ckb.scaled_mm_nvfp4(qx, qw, tsx, tsw, sfx, sfw, bias=bias)
        splits_ref = _lib.load().ck_b200_query(_lib.QUERY_LAST_GEMM_SPLITS)
        for v in (5, 6):
            ckb.set_tuning(1, v)
            for _ in range(3):
                y = ckb.scaled_mm_nvfp4(qx, qw, tsx, tsw, sfx, sfw, bias=bias)
                splits = _lib.load().ck_b200_query(_lib.QUERY_LAST_GEMM_SPLITS)
                if splits == splits_ref:
                    assert torch.equal(y, ref), f"variant {v}"
                else:
                    assert rel_rms(y[:M].float(), ref[:M].float()) <= 1e-3, f"variant {v}"
    finally:
        ckb.set_tuning(1, prev)
    assert ckb.read_device_status() == 0


@pytest.mark.parametrize("mnk", [(16, 10240, 4096), (64, 4096, 10240), (128, 4096, 4096), (1, 4096, 4096)],
                         ids=lambda s: "x".join(map(str, s)))
@pytest.mark.parametrize("variant_under_promise", [0, 5, 6], ids=["auto", "bn64", "cluster"])
def test_weight_loads_ahead_of_the_preceding_kernel(mnk, variant_under_promise, ckb):
    """With the caller's promise that weights are resident, a small-M GEMM asks for its weight before it waits for the
    preceding kernel of the stream.  Activations, their scales and the tensor scale are produced by the kernels right
    before it on the same stream with no synchronisation in between, so the test fails if anything but the weight is
    read early: a stack of layers captured in one graph, replayed on changed activations, must give the bits of the
    same stack without the promise."""
    M, N, K = mnk
    layers = []
    for i in range(4):
        w = seeded_randn((N, K), seed=100 + i, std=0.02).cuda()
        tsw = amax_scale(w).cuda()
        qw, sfw = ckb.quantize_nvfp4(w, tsw)
        layers.append((qw, sfw, tsw, seeded_randn((1, N), seed=7 + i, std=0.5).reshape(N).cuda()))
    xs = [seeded_randn((M, K), seed=50 + j).cuda() for j in range(3)]
    x = xs[0].clone()

    def stack():
        outs = []
        for qw, sfw, tsw, bias in layers:
            qx, sfx, tsx = ckb.quantize_nvfp4_dynamic(x, pad_16x=M % 16 != 0)   # written by the kernel right before the GEMM
            outs.append(ckb.scaled_mm_nvfp4(qx, qw, tsx, tsw, sfx, sfw, bias=bias))
        return outs

    torch.cuda.synchronize()      # the promise: the weights above are complete and stay untouched
    prev_variant = ckb.set_tuning(1, variant_under_promise)
    want = []
    for xj in xs:
        x.copy_(xj)
        want.append([o.clone() for o in stack()])
    prev = ckb.promise_resident_weights(True)
    try:
        for j, xj in enumerate(xs):
            x.copy_(xj)
            for o, wnt in zip(stack(), want[j]):
                assert torch.equal(o, wnt)
        stream = torch.cuda.Stream()
        with torch.cuda.stream(stream):
            stack()
        stream.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.stream(stream), torch.cuda.graph(graph):
            outs = stack()
        for rep in range(6):
            j = rep % 3
            with torch.cuda.stream(stream):
                x.copy_(xs[j], non_blocking=True)     # the activations change right before the replay, on its stream
                graph.replay()
            stream.synchronize()
            for o, wnt in zip(outs, want[j]):
                assert torch.equal(o, wnt)
    finally:
        ckb.set_tuning(1, prev_variant)
        ckb.promise_resident_weights(prev)
    assert ckb.read_device_status() == 0


def test_short_row_configurations_on_random_problems(ckb):
    """Random small-M problems (M <= 64; N any multiple of 8, K any multiple of 32, so tiles, bands of scales, K stages and
    the ranks of a cluster all meet ragged edges), every output and bias dtype, alpha in place of the two tensor scales:
    the 64-column tiles and the cluster split, with and without weight loads ahead of the preceding kernel, against
    the 128-column tiles - bit for bit when K is cut into the same number of splits, within 1e-3 relative RMS
    otherwise (the order in which fp32 partial sums are added differs)."""
    import random

    from comfy_kitchen_b200 import _lib
    L = _lib.load()
    rng = random.Random(1234)
    dtypes = [torch.bfloat16, torch.float16, torch.float32]
    prev = ckb.set_tuning(1, 0)
    try:
        for case in range(36):
            M = rng.choice([1, 3, 16, 17, 31, 32, 33, 48, 64])
            N = 8 * rng.randint(1, 400)
            K = 32 * rng.randint(1, 160)
            x, w, qx, sfx, tsx, qw, sfw, tsw = quantized_operands(ckb, M, N, K, seed=1000 + case)
            out_dtype = dtypes[case % 3]
            bias = None
            if case % 4:
                bias = seeded_randn((1, N), seed=case, std=0.5).reshape(N).cuda().to(dtypes[(case // 3) % 2])
            alpha = (tsx * tsw * 0.5).reshape(()) if case % 5 == 0 else None
            kw = dict(bias=bias, out_dtype=out_dtype, alpha=alpha)
            ckb.set_tuning(1, 1)
            ref = ckb.scaled_mm_nvfp4(qx, qw, tsx, tsw, sfx, sfw, **kw)
            splits_ref = L.ck_b200_query(_lib.QUERY_LAST_GEMM_SPLITS)
            torch.cuda.synchronize()
            for variant in (5, 6):
                for promise in (False, True):
                    ckb.set_tuning(1, variant)
                    was = ckb.promise_resident_weights(promise)
                    try:
                        y = ckb.scaled_mm_nvfp4(qx, qw, tsx, tsw, sfx, sfw, **kw)
                        splits = L.ck_b200_query(_lib.QUERY_LAST_GEMM_SPLITS)
                    finally:
                        ckb.promise_resident_weights(was)
                    what = f"case {case}: M={M} N={N} K={K} variant {variant} promise {promise} splits {splits}/{splits_ref}"
                    assert y.shape == ref.shape and y.dtype == ref.dtype, what
                    if splits == splits_ref:
                        assert torch.equal(y, ref), what
                    else:
                        assert rel_rms(y[:M].float(), ref[:M].float()) <= 1e-3, what
    finally:
        ckb.set_tuning(1, prev)
    assert ckb.read_device_status() == 0


EXACT = [(4608, 9216, 3072), (4608, 4608, 3072), (4608, 6144, 3072), (4608, 3072, 12288), (4608, 1536, 3072),
         (32760, 5120, 5120)]


@pytest.mark.parametrize("mnk", EXACT, ids=lambda s: "x".join(map(str, s)))
def test_gemm_tile_variants_are_bit_identical(mnk, ckb):
    """Every tile variant adds the K dimension up in the same order with the same instruction, so at full size the
    CTA-pair kernel must reproduce the one-CTA kernel bit for bit, launch after launch - a relative-RMS tolerance
    would not notice a few hundred elements of a 40-million-element matrix going wrong (for instance a staging tile
    handed out again while the store that reads it is still in flight).  Widths of N-sharded weights included."""
    M, N, K = mnk
    x, w, qx, sfx, tsx, qw, sfw, tsw = quantized_operands(ckb, M, N, K, seed=K + N, outliers=True)
    prev = ckb.set_tuning(1, 1)                      # 128 x 128 tiles, one CTA each
    try:
        ref = ckb.scaled_mm_nvfp4(qx, qw, tsx, tsw, sfx, sfw)
        for v in (2, 3, 3, 3, 4):                    # the default (CTA pairs) several times: the hazard is one of timing
            ckb.set_tuning(1, v)
            y = ckb.scaled_mm_nvfp4(qx, qw, tsx, tsw, sfx, sfw)
            bad = int((y != ref).sum())
            assert bad == 0, f"variant {v}: {bad} elements differ from the 128x128 one-CTA kernel"
    finally:
        ckb.set_tuning(1, prev)
    assert ckb.read_device_status() == 0


def test_gemm_rejects_bad_arguments(ckb):
    qx = torch.zeros((128, 64), dtype=torch.uint8, device="cuda")
    qw = torch.zeros((64, 64), dtype=torch.uint8, device="cuda")
    ts = torch.tensor(1.0, device="cuda")
    sfa = torch.zeros((128, 8), dtype=torch.uint8, device="cuda").view(torch.float8_e4m3fn)
    sfb = torch.zeros((128, 8), dtype=torch.uint8, device="cuda").view(torch.float8_e4m3fn)
    with pytest.raises(AssertionError):
        ckb.scaled_mm_nvfp4(qx, qw[:, :32].contiguous(), ts, ts, sfa, sfb)     # K mismatch
    with pytest.raises(AssertionError):
        ckb.scaled_mm_nvfp4(qx, qw, ts, ts, sfa[:64], sfb)                      # wrong scale shape
    from comfy_kitchen_b200 import _lib
    L = _lib.load()
    rc = L.ck_b200_scaled_mm_nvfp4(qx.data_ptr(), sfa.data_ptr(), qw.data_ptr(), sfb.data_ptr(), ts.data_ptr(),
                                   ts.data_ptr(), None, None, 2, qx.data_ptr(), 2, 128, 60, 128, None, 0, None)
    assert rc == 1 and "multiple of 8" in _lib.last_error()


def test_zero_sized(ckb):
    ts = torch.tensor(1.0, device="cuda")
    q, sf = ckb.quantize_nvfp4(torch.empty((0, 64), dtype=torch.bfloat16, device="cuda"), ts)
    assert tuple(q.shape) == (0, 32) and tuple(sf.shape) == (0, 4)
