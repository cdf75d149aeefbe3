"""GPU parity of quantize_nvfp4 / dequantize_nvfp4 / dynamic scale (through the C ABI) against the CPU oracle
and the reference golden vectors.  Bit-exact: packed bytes, scale bytes and dequantized values."""
from __future__ import annotations

import numpy as np
import pytest
import torch

from conftest import golden_case_names
from helpers import CODE, amax_scale, from_bits, seeded_randn, to_bits

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ckb():
    import comfy_kitchen_b200 as m
    assert torch.cuda.is_available()
    return m


@pytest.fixture(params=[1, 2, 0], ids=["bracket", "residual", "ieee-div"])
def variant(request, ckb):
    prev = ckb.set_tuning(0, request.param)
    yield request.param
    ckb.set_tuning(0, prev)


def _dev(t):
    return t.cuda()


@pytest.mark.parametrize("name", golden_case_names())
def test_quantize_golden(name, golden, ckb, variant):
    dtype, pad, hi = (int(v) for v in golden[f"{name}/meta"])
    ts = torch.tensor(float(golden[f"{name}/ts"][0]), dtype=torch.float32)
    x = _dev(from_bits(golden[f"{name}/x"], dtype))
    q, sf = ckb.quantize_nvfp4(x, _dev(ts), pad_16x=bool(pad), hi_first=bool(hi))
    assert sf.dtype == torch.float8_e4m3fn and q.dtype == torch.uint8
    assert tuple(q.shape) == golden[f"{name}/q"].shape and tuple(sf.shape) == golden[f"{name}/sf"].shape
    if name == "bf16_ts_zero":   # 0/0 in the reference for all-zero blocks: only the data bytes are pinned
        assert np.array_equal(to_bits(q), golden[f"{name}/q"])
        return
    assert np.array_equal(to_bits(sf), golden[f"{name}/sf"]), "scale bytes differ from the reference"
    assert np.array_equal(to_bits(q), golden[f"{name}/q"]), "packed bytes differ from the reference"


@pytest.mark.parametrize("name", golden_case_names())
def test_dequantize_golden(name, golden, ckb):
    _, _, hi = (int(v) for v in golden[f"{name}/meta"])
    ts = _dev(torch.tensor(float(golden[f"{name}/ts"][0]), dtype=torch.float32))
    q = _dev(torch.from_numpy(golden[f"{name}/q"].copy()))
    sf = _dev(torch.from_numpy(golden[f"{name}/sf"].copy())).view(torch.float8_e4m3fn)
    found = False
    for dt, tdt in ((0, torch.float32), (1, torch.float16), (2, torch.bfloat16)):
        if f"{name}/dq{dt}" not in golden:
            continue
        found = True
        y = ckb.dequantize_nvfp4(q, ts, sf, tdt, hi_first=bool(hi))
        ref = golden[f"{name}/dq{dt}"]
        got = to_bits(y)
        if dt == 0:
            assert np.array_equal(got.view(np.uint32), ref.view(np.uint32))
        else:
            assert np.array_equal(got, ref)
    if not found:
        pytest.skip("no dequantize vector")


SHAPES = [(16, 16), (16, 64), (128, 64), (256, 1024), (1024, 1024), (144, 80), (4608, 3072), (1024, 5120), (2048, 12288)]


@pytest.mark.parametrize("shape", SHAPES, ids=lambda s: f"{s[0]}x{s[1]}")
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32], ids=["bf16", "f16", "f32"])
def test_quantize_vs_oracle(shape, dtype, ckb, oracle, variant):
    if dtype != torch.bfloat16 and shape[0] * shape[1] > 3_000_000:
        pytest.skip("large shapes are covered in bf16")
    x = seeded_randn(shape, seed=shape[0] * 7 + shape[1], dtype=dtype, outlier_cols=max(1, shape[1] // 1000))
    ts = amax_scale(x)
    q, sf = ckb.quantize_nvfp4(_dev(x), _dev(ts))
    q_ref, sf_ref = oracle.quantize_nvfp4(to_bits(x), CODE[dtype], float(ts))
    assert np.array_equal(to_bits(sf), sf_ref)
    assert np.array_equal(to_bits(q), q_ref)
    # round trip through both dequantizers
    for out_dt in (torch.bfloat16, torch.float32):
        y = ckb.dequantize_nvfp4(q, _dev(ts), sf, out_dt)
        y_ref = oracle.dequantize_nvfp4(q_ref, float(ts), sf_ref, CODE[out_dt])
        got = to_bits(y)
        assert np.array_equal(got.view(np.uint32) if out_dt == torch.float32 else got,
                              y_ref.view(np.uint32) if out_dt == torch.float32 else y_ref)


# the last four: whole 128-column pairs, so the bounds-free walk runs, with input rows that end inside the bottom
# band (zero rows still inside the padded output) and with both nibble orders
@pytest.mark.parametrize("shape", [(33, 65), (1, 16), (17, 1000), (129, 130), (5, 7), (200, 24), (200, 256), (1000, 512),
                                   (4600, 3072), (256, 1024)],
                         ids=lambda s: f"{s[0]}x{s[1]}")
@pytest.mark.parametrize("hi_first", [True, False])
def test_quantize_padded_vs_oracle(shape, hi_first, ckb, oracle, variant):
    x = seeded_randn(shape, seed=11 + shape[0], std=4.0)
    ts = amax_scale(x)
    q, sf = ckb.quantize_nvfp4(_dev(x), _dev(ts), pad_16x=True, hi_first=hi_first)
    q_ref, sf_ref = oracle.quantize_nvfp4(to_bits(x), 2, float(ts), pad_16x=True, hi_first=hi_first)
    assert tuple(q.shape) == q_ref.shape and tuple(sf.shape) == sf_ref.shape
    assert np.array_equal(to_bits(sf), sf_ref) and np.array_equal(to_bits(q), q_ref)


def test_tie_heavy_inputs(ckb, oracle, variant):
    """Quotients that sit exactly on e2m1 rounding boundaries: coarse grid inputs with power-of-two scales."""
    g = torch.Generator().manual_seed(5)
    grid = torch.randint(-24, 25, (512, 1024), generator=g).float() * 0.25
    for dtype in (torch.bfloat16, torch.float32):
        x = grid.to(dtype)
        for ts in (2.0 ** -4, 2.0 ** -7, float(amax_scale(x)), 0.0371234):
            tsd = torch.tensor(ts, dtype=torch.float32)
            q, sf = ckb.quantize_nvfp4(_dev(x), _dev(tsd))
            q_ref, sf_ref = oracle.quantize_nvfp4(to_bits(x), CODE[dtype], ts)
            assert np.array_equal(to_bits(sf), sf_ref) and np.array_equal(to_bits(q), q_ref)


def test_extreme_magnitudes(ckb, oracle, variant):
    """Huge and tiny blocks: the guarded fast division must hand over to the IEEE one and agree with the oracle."""
    g = torch.Generator().manual_seed(6)
    x = torch.randn(64, 256, generator=g)
    x[0:16] *= 1e30
    x[16:32] *= 1e-30
    x[32:48] *= 1e-42     # subnormal inputs
    x[48:64, ::3] = 0.0
    for ts in (1.0, 1e-30, 1e30, 3e-39):
        tsd = torch.tensor(ts, dtype=torch.float32)
        q, sf = ckb.quantize_nvfp4(_dev(x), _dev(tsd))
        q_ref, sf_ref = oracle.quantize_nvfp4(to_bits(x), 0, float(tsd))
        assert np.array_equal(to_bits(sf), sf_ref) and np.array_equal(to_bits(q), q_ref)


def test_infinite_elements(ckb, oracle, variant):
    """Blocks holding +-inf: the block scale clamps at 448 and the infinite elements saturate to +-6."""
    g = torch.Generator().manual_seed(8)
    base = torch.randn(32, 128, generator=g)
    base[3, 5] = float("inf")
    base[3, 40] = float("-inf")
    base[17, 127] = float("-inf")
    base[20, 64:80] = float("inf")
    for dtype in (torch.float32, torch.float16, torch.bfloat16):
        x = base.to(dtype)
        for ts in (2.0 ** -7, 0.0123):
            tsd = torch.tensor(ts, dtype=torch.float32)
            q, sf = ckb.quantize_nvfp4(_dev(x), _dev(tsd))
            q_ref, sf_ref = oracle.quantize_nvfp4(to_bits(x), CODE[dtype], float(tsd))
            assert np.array_equal(to_bits(sf), sf_ref) and np.array_equal(to_bits(q), q_ref)


def test_scale_tensor_padding_is_written(ckb):
    """The kernel itself zero-fills the padded part of the scale tensor: poison the allocator's memory first."""
    poison = torch.full((1 << 22,), 0xAB, dtype=torch.uint8, device="cuda")
    del poison
    x = seeded_randn((144, 80), seed=3).cuda()
    q, sf = ckb.quantize_nvfp4(x, amax_scale(x).cuda())
    sfb = to_bits(sf)
    assert sfb.shape == (256, 8)
    # rows >= 144 and scale columns >= 5 are padding
    from oracle import oracle as o
    L = o.lib()
    flat = sfb.reshape(-1)
    for r in range(256):
        for c in range(8):
            if r >= 144 or c >= 5:
                assert flat[L.nvfp4_oracle_sf_offset(r, c, 8)] == 0


def test_full_size_properties(ckb):
    """Largest bandwidth-sweep shape (65536 x 12288): properties that hold without a CPU pass over 0.8 G elements."""
    g = torch.Generator(device="cuda").manual_seed(9)
    x = torch.randn((65536, 12288), generator=g, device="cuda", dtype=torch.bfloat16)
    ts = amax_scale(x).cuda()
    q, sf = ckb.quantize_nvfp4(x, ts)
    # determinism and row-slice consistency: quantizing a 128-aligned row slice gives the same bytes
    q2, sf2 = ckb.quantize_nvfp4(x[4096:4096 + 1024].contiguous(), ts)
    assert torch.equal(q[4096:4096 + 1024], q2)
    assert torch.equal(sf.view(torch.uint8)[4096:4096 + 1024], sf2.view(torch.uint8))
    # idempotence: dequantize(quantize(dequantize(quantize(x)))) == dequantize(quantize(x))
    y = ckb.dequantize_nvfp4(q[:8192], ts, sf[:8192], torch.bfloat16)
    q3, sf3 = ckb.quantize_nvfp4(y, ts)
    y3 = ckb.dequantize_nvfp4(q3, ts, sf3, torch.bfloat16)
    assert torch.equal(y, y3)
    # error bound of the format: |x - dq| <= half the largest e2m1 gap times the block scale, generously 0.5*amax/3
    err = (x[:8192].float() - y.float()).abs().amax()
    assert float(err) <= float(x[:8192].abs().amax()) / 5.0
    # nibble-order property on the big tensor
    ql, sfl = ckb.quantize_nvfp4(x[:8192], ts, hi_first=False)
    assert torch.equal(ql, ((q[:8192] << 4) | (q[:8192] >> 4)))
    assert torch.equal(sfl.view(torch.uint8), sf.view(torch.uint8)[:8192])


SWEEP = [(m, k) for m in (1024, 4096, 16384, 65536) for k in (3072, 5120, 12288)]


@pytest.mark.parametrize("mk", SWEEP, ids=lambda s: "x".join(map(str, s)))
def test_sweep_shapes_row_slices_vs_oracle(mk, ckb, oracle):
    """Every shape of the bandwidth-sweep configuration: the first, middle and last 256 rows of the whole-tensor
    result against the CPU oracle on those rows, bytes, scales and the bf16 round trip (the block scales depend on the
    row only, and 256 rows are two whole 128-row scale bands, so the slice of the result is the result of the slice)."""
    M, K = mk
    g = torch.Generator(device="cuda").manual_seed(M * 31 + K)
    x = torch.randn((M, K), generator=g, device="cuda", dtype=torch.bfloat16)
    ts = ckb.dynamic_scale_nvfp4(x)
    tsf = float(ts.item())
    assert np.float32(tsf) == np.float32(float((x.abs().amax() / 2688.0).float()))    # bf16 arithmetic, like the layout
    q, sf = ckb.quantize_nvfp4(x, ts)
    if M * K * 2 <= 33_000_000:
        # this size can also be quantized from shared memory with the whole input in flight (off by default); that
        # kernel must give the bytes of the register-ring kernels
        prev = ckb.set_tuning(10, 1)
        try:
            q_chip, sf_chip = ckb.quantize_nvfp4(x, ts)
        finally:
            ckb.set_tuning(10, prev)
        assert torch.equal(q, q_chip) and torch.equal(sf.view(torch.uint8), sf_chip.view(torch.uint8))
    y = ckb.dequantize_nvfp4(q, ts, sf, torch.bfloat16)
    sfu = sf.view(torch.uint8)
    for r0 in sorted({0, (M // 2) // 128 * 128, M - 256}):
        xb = to_bits(x[r0:r0 + 256])
        q_ref, sf_ref = oracle.quantize_nvfp4(xb, oracle.BF16, tsf)
        assert np.array_equal(to_bits(q[r0:r0 + 256]), q_ref), f"packed bytes differ in rows {r0}..{r0 + 255}"
        assert np.array_equal(to_bits(sfu[r0:r0 + 256]), sf_ref), f"scale bytes differ in rows {r0}..{r0 + 255}"
        y_ref = oracle.dequantize_nvfp4(q_ref, tsf, sf_ref, oracle.BF16)
        assert np.array_equal(to_bits(y[r0:r0 + 256]), y_ref), f"round trip differs in rows {r0}..{r0 + 255}"
    del x, q, sf, y
    torch.cuda.empty_cache()


def test_first_config_digests(ckb, golden_large, oracle):
    import hashlib
    rng = np.random.default_rng(0)
    x32 = rng.standard_normal((256, 1024), dtype=np.float32)
    xb = oracle.narrow(x32, oracle.BF16)
    if hashlib.sha256(xb.tobytes()).hexdigest() != golden_large["x_bits_sha256"]:
        pytest.skip("numpy generator stream differs")
    x = from_bits(xb, 2).cuda()
    ts = torch.tensor(golden_large["ts_x"], dtype=torch.float32).cuda()
    q, sf = ckb.quantize_nvfp4(x, ts)
    assert hashlib.sha256(to_bits(q).tobytes()).hexdigest() == golden_large["qx_sha256"]
    assert hashlib.sha256(to_bits(sf).tobytes()).hexdigest() == golden_large["sfx_sha256"]
    y = ckb.dequantize_nvfp4(q, ts, sf, torch.bfloat16)
    assert hashlib.sha256(to_bits(y).tobytes()).hexdigest() == golden_large["dqx_bf16_sha256"]


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32], ids=["bf16", "f16", "f32"])
def test_dynamic_scale(dtype, ckb, oracle, golden):
    x = seeded_randn((777, 130), seed=21, std=3.0, dtype=dtype)
    got = ckb.dynamic_scale_nvfp4(x.cuda())
    assert got.dtype == torch.float32 and got.dim() == 0
    assert np.float32(got.item()) == np.float32(oracle.dynamic_scale(to_bits(x), CODE[dtype]))
    if dtype == torch.bfloat16:
        xl = from_bits(golden["layout/x"], 2).cuda()
        assert np.float32(ckb.dynamic_scale_nvfp4(xl).item()) == golden["layout/scale"][0]


def test_rejects_bad_arguments(ckb):
    x = torch.randn(17, 32, device="cuda", dtype=torch.bfloat16)
    ts = torch.tensor(0.01, device="cuda")
    with pytest.raises(AssertionError):
        ckb.quantize_nvfp4(x, ts)                       # not 16-aligned without pad_16x
    with pytest.raises(TypeError):
        ckb.quantize_nvfp4(x.cpu(), ts)                 # no CPU path
    with pytest.raises(AssertionError):
        ckb.quantize_nvfp4(torch.randn(32, 64, device="cuda").t(), ts)   # not contiguous


def test_graph_capture_quantize(ckb):
    """Launch-only, allocation-free entry point: capturable on a side stream (reference tests/test_dlpack.py:99-136)."""
    from comfy_kitchen_b200 import _lib
    import ctypes
    L = _lib.load()
    x = seeded_randn((256, 512), seed=4).cuda()
    ts = amax_scale(x).cuda().reshape(1)
    q = torch.empty((256, 256), dtype=torch.uint8, device="cuda")
    sf = torch.empty((256, 32), dtype=torch.uint8, device="cuda")
    s = torch.cuda.Stream()
    graph = torch.cuda.CUDAGraph()
    torch.cuda.synchronize()
    with torch.cuda.stream(s):
        with torch.cuda.graph(graph, stream=s):
            rc = L.ck_b200_quantize_nvfp4(x.data_ptr(), 2, ts.data_ptr(), q.data_ptr(), sf.data_ptr(), 256, 512, 0, 1,
                                          ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
            assert rc == 0
    q.zero_()
    graph.replay()
    torch.cuda.synchronize()
    q_ref, sf_ref = ckb.quantize_nvfp4(x, ts)
    assert torch.equal(q, q_ref) and torch.equal(sf, sf_ref.view(torch.uint8))
