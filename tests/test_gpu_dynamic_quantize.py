"""quantize_nvfp4 with the per-tensor scale derived from the tensor itself in the same launch
(ck_b200_quantize_nvfp4_dynamic) against the CPU oracle: the scale as the reference layout computes it
(comfy_kitchen/tensor/nvfp4.py:66-71, in the input's dtype) and the bytes and block scales of quantize_nvfp4 with that
scale.  Bit-exact.  Also: the bounded wait at the kernel's grid-wide meeting point is made to run out once and the
status word read."""
from __future__ import annotations

import numpy as np
import pytest
import torch

from helpers import CODE, seeded_randn, to_bits

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ckb():
    import comfy_kitchen_b200 as m
    assert torch.cuda.is_available()
    return m


@pytest.fixture(params=[1, 0], ids=["onchip", "l2"])
def park(request, ckb):
    """Both forms of the one-launch kernel: small inputs parked in shared memory between its phases, or re-read from L2."""
    prev = ckb.set_tuning(8, request.param)
    yield request.param
    ckb.set_tuning(8, prev)


# (rows, cols, pad_16x)
SHAPES = [(256, 1024, False), (4608, 3072, False), (4608, 12288, False), (16, 4096, False), (32760, 5120, True),
          (129, 200, True), (48, 64, False), (1000, 1152, True)]


def expected_launches(rows, cols, pad, dtype):
    """One launch where the input is about the size of the L2 or smaller (128e6 bytes by default) and the one-wave geometry applies (rows of a
    multiple of 8 columns whose scale tensor has an even number of 4-column groups); otherwise the reduction, the
    scale and the quantizer as three launches inside the same call."""
    pcol = (cols + 15) // 16 * 16 if pad else cols
    groups = ((pcol // 16 + 3) // 4)
    nbytes = rows * cols * (4 if dtype == torch.float32 else 2)
    return 1 if (cols % 8 == 0 and groups % 2 == 0 and nbytes <= 128e6) else 3


@pytest.mark.parametrize("shape", SHAPES, ids=lambda s: "x".join(map(str, s[:2])))
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32], ids=["bf16", "f16", "f32"])
def test_dynamic_quantize_vs_oracle(shape, dtype, ckb, oracle, park):
    rows, cols, pad = shape
    want_launches = expected_launches(rows, cols, pad, dtype)
    if dtype != torch.bfloat16 and rows > 5000:
        pytest.skip("largest case in bf16 only")
    x = seeded_randn((rows, cols), seed=rows + cols, std=2.0, dtype=dtype, outlier_cols=max(1, cols // 1000))
    xd = x.cuda()
    n0 = ckb.launches()
    q, sf, ts = ckb.quantize_nvfp4_dynamic(xd, pad_16x=pad)
    assert ckb.launches() - n0 == want_launches
    assert ts.dtype == torch.float32 and ts.dim() == 0
    ts_ref = oracle.dynamic_scale(to_bits(x), CODE[dtype])
    assert np.float32(ts.item()) == np.float32(ts_ref), "per-tensor scale differs from the layout's"
    q_ref, sf_ref = oracle.quantize_nvfp4(to_bits(x), CODE[dtype], ts_ref, pad_16x=pad)
    assert np.array_equal(to_bits(sf), sf_ref), "scale bytes differ"
    assert np.array_equal(to_bits(q), q_ref), "packed bytes differ"
    # and the same bits as the two separate operators
    ts2 = ckb.dynamic_scale_nvfp4(xd)
    q2, sf2 = ckb.quantize_nvfp4(xd, ts2, pad_16x=pad)
    assert torch.equal(ts, ts2) and torch.equal(q, q2) and torch.equal(sf.view(torch.uint8), sf2.view(torch.uint8))
    assert ckb.read_device_status() == 0


def test_dynamic_quantize_repeats_and_graph_replays(ckb, park):
    """The meeting-point counters return to zero after every launch, so back-to-back launches and replays of a
    captured launch on changing data keep giving the separate operators' result."""
    x = seeded_randn((2048, 3072), seed=5).cuda()
    sync = torch.zeros(64, dtype=torch.uint8, device="cuda")
    for _ in range(5):
        q, sf, ts = ckb.quantize_nvfp4_dynamic(x, _sync=sync)
    torch.cuda.synchronize()
    assert int(sync.sum()) == 0
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        ckb.quantize_nvfp4_dynamic(x, _sync=sync)
    stream.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(stream), torch.cuda.graph(graph):
        q, sf, ts = ckb.quantize_nvfp4_dynamic(x, _sync=sync)
    for i in range(4):
        x.copy_(seeded_randn((2048, 3072), seed=50 + i, std=1.0 + i).cuda())
        with torch.cuda.stream(stream):
            graph.replay()
        stream.synchronize()
        ts2 = ckb.dynamic_scale_nvfp4(x)
        q2, sf2 = ckb.quantize_nvfp4(x, ts2)
        assert torch.equal(ts, ts2) and torch.equal(q, q2) and torch.equal(sf.view(torch.uint8), sf2.view(torch.uint8))
    assert int(sync.sum()) == 0 and ckb.read_device_status() == 0


def test_all_zero_input_matches_separate_operators(ckb):
    x = torch.zeros((64, 256), dtype=torch.bfloat16, device="cuda")
    q, sf, ts = ckb.quantize_nvfp4_dynamic(x)
    ts2 = ckb.dynamic_scale_nvfp4(x)
    q2, sf2 = ckb.quantize_nvfp4(x, ts2)
    assert float(ts) == 0.0 and torch.equal(q, q2) and torch.equal(sf.view(torch.uint8), sf2.view(torch.uint8))


def test_meeting_point_wait_runs_out_and_reports(ckb):
    """Failure detection without a fault: the kernel is told to expect one block more than the grid has, so the
    counter never reaches its target; after its limit (about 0.1 s in this mode) every block records code 8 in the
    status word and returns, the context stays usable and the next call works."""
    x = seeded_randn((16, 256), seed=1).cuda()          # one block
    sync = torch.zeros(64, dtype=torch.uint8, device="cuda")
    prev = ckb.set_tuning(6, 1)
    try:
        q, sf, ts = ckb.quantize_nvfp4_dynamic(x, _sync=sync)
        status = ckb.read_device_status()                # synchronises
    finally:
        ckb.set_tuning(6, prev)
    assert status == 8, f"expected the quantizer's meeting-point code, got {status}"
    assert ckb.read_device_status() == 0                 # reading clears the word
    # the counters of the abandoned launch are not reused; a fresh set works at once
    q, sf, ts = ckb.quantize_nvfp4_dynamic(x, _sync=torch.zeros(64, dtype=torch.uint8, device="cuda"))
    ts2 = ckb.dynamic_scale_nvfp4(x)
    q2, sf2 = ckb.quantize_nvfp4(x, ts2)
    assert torch.equal(ts, ts2) and torch.equal(q, q2) and ckb.read_device_status() == 0


def test_default_counters_recover_after_an_expired_wait(ckb):
    """The same expiry on the counters the Python operator keeps per stream: reading the status word puts them back to
    zero, so the calls that follow on that stream work (without that, every later launch would wait out its limit)."""
    x = seeded_randn((16, 256), seed=2).cuda()
    ckb.quantize_nvfp4_dynamic(x)                        # creates this stream's counters
    prev = ckb.set_tuning(6, 1)
    try:
        ckb.quantize_nvfp4_dynamic(x)
        status = ckb.read_device_status()
    finally:
        ckb.set_tuning(6, prev)
    assert status == 8
    q, sf, ts = ckb.quantize_nvfp4_dynamic(x)
    ts2 = ckb.dynamic_scale_nvfp4(x)
    q2, sf2 = ckb.quantize_nvfp4(x, ts2)
    assert torch.equal(ts, ts2) and torch.equal(q, q2) and torch.equal(sf.view(torch.uint8), sf2.view(torch.uint8))
    assert ckb.read_device_status() == 0
