"""Pins the CPU oracle to vectors produced by the reference eager backend (tests/golden/make_golden.py).

These tests need neither a GPU nor the reference checkout.
"""
from __future__ import annotations

import hashlib

import numpy as np
import pytest

from conftest import golden_case_names


def _sha(a):
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


@pytest.mark.parametrize("name", golden_case_names())
def test_quantize_matches_reference_bits(name, golden, oracle):
    dtype, pad, hi = (int(v) for v in golden[f"{name}/meta"])
    ts = float(golden[f"{name}/ts"][0])
    q, sf = oracle.quantize_nvfp4(golden[f"{name}/x"], dtype, ts, bool(pad), bool(hi))
    assert q.shape == golden[f"{name}/q"].shape and sf.shape == golden[f"{name}/sf"].shape
    if name == "bf16_ts_zero":
        # ts == 0 with all-zero blocks is 0/0 in the reference; only the non-degenerate part is pinned
        assert np.array_equal(q, golden[f"{name}/q"])
        return
    assert np.array_equal(sf, golden[f"{name}/sf"]), "block scale bytes differ from the reference"
    assert np.array_equal(q, golden[f"{name}/q"]), "packed e2m1 bytes differ from the reference"


@pytest.mark.parametrize("name", golden_case_names())
def test_dequantize_matches_reference_bits(name, golden, oracle):
    _, _, hi = (int(v) for v in golden[f"{name}/meta"])
    ts = float(golden[f"{name}/ts"][0])
    found = False
    for dt in (0, 1, 2):
        key = f"{name}/dq{dt}"
        if key not in golden:
            continue
        found = True
        y = oracle.dequantize_nvfp4(golden[f"{name}/q"], ts, golden[f"{name}/sf"], dt, bool(hi))
        ref = golden[key]
        if dt == 0:
            assert np.array_equal(y.view(np.uint32), ref.view(np.uint32)), f"fp32 dequantize differs ({name})"
        else:
            assert np.array_equal(y, ref), f"dequantize to dtype code {dt} differs ({name})"
    if not found:
        pytest.skip("no dequantize vector for this case")


def test_swizzle_offsets_match_to_blocked(golden, oracle):
    blocked = golden["swizzle/iota_blocked"]          # to_blocked(iota(256x12)), flattened
    L = oracle.lib()
    for r in range(256):
        for c in range(12):
            assert blocked[L.nvfp4_oracle_sf_offset(r, c, 12)] == r * 12 + c


def test_dynamic_scale_matches_layout(golden, oracle):
    x = golden["layout/x"]
    ts = oracle.dynamic_scale(x, oracle.BF16)
    assert np.float32(ts) == golden["layout/scale"][0]
    q, sf = oracle.quantize_nvfp4(x, oracle.BF16, ts)
    assert np.array_equal(q, golden["layout/q"]) and np.array_equal(sf, golden["layout/sf"])


@pytest.mark.parametrize("name", ["gemm_64x128x256", "gemm_48x72x96"])
@pytest.mark.parametrize("blas", [True, False])
def test_gemm_restatement_small(name, blas, golden, oracle):
    tsa, tsb = (float(v) for v in golden[f"{name}/ts"])
    bias = golden[f"{name}/bias"] if f"{name}/bias" in golden else None
    y = oracle.scaled_mm_nvfp4(golden[f"{name}/qa"], golden[f"{name}/qb"], tsa, tsb, golden[f"{name}/sfa"],
                               golden[f"{name}/sfb"], bias=bias, blas=blas)
    ref = oracle.widen(golden[f"{name}/y"], oracle.BF16)
    got = oracle.widen(y, oracle.BF16)
    # fp32 summation order differs between BLAS libraries: bf16 outputs may differ by one rounding
    assert oracle.rel_rms(got, ref) < 2e-3
    assert np.mean(got != ref) < 0.02


def test_first_config_digests(golden_large, oracle):
    """256x1024 activations and 1024x1024 weights of the CPU-runnable configuration."""
    rng = np.random.default_rng(0)
    x32 = rng.standard_normal((256, 1024), dtype=np.float32)
    w32 = (rng.standard_normal((1024, 1024), dtype=np.float32) * np.float32(0.02)).astype(np.float32)
    x, w = oracle.narrow(x32, oracle.BF16), oracle.narrow(w32, oracle.BF16)
    if _sha(x) != golden_large["x_bits_sha256"] or _sha(w) != golden_large["w_bits_sha256"]:
        pytest.skip("numpy generator stream differs from the one the vectors were made with")
    tsx, tsw = golden_large["ts_x"], golden_large["ts_w"]
    assert np.float32(np.abs(oracle.widen(x, oracle.BF16)).max() / np.float32(2688.0)) == np.float32(tsx)
    qx, sfx = oracle.quantize_nvfp4(x, oracle.BF16, tsx)
    qw, sfw = oracle.quantize_nvfp4(w, oracle.BF16, tsw)
    assert (_sha(qx), _sha(sfx)) == (golden_large["qx_sha256"], golden_large["sfx_sha256"])
    assert (_sha(qw), _sha(sfw)) == (golden_large["qw_sha256"], golden_large["sfw_sha256"])
    assert int(qx.astype(np.int64).sum()) == golden_large["qx_sum"]
    assert _sha(oracle.dequantize_nvfp4(qx, tsx, sfx, oracle.BF16)) == golden_large["dqx_bf16_sha256"]
    y = oracle.widen(oracle.scaled_mm_nvfp4(qx, qw, tsx, tsw, sfx, sfw), oracle.BF16)
    ref = oracle.widen(np.array(golden_large["y_sample_bits"], np.uint16), oracle.BF16)
    assert oracle.rel_rms(y[::8, ::8], ref) < 2e-3
    assert abs(np.sqrt(np.mean(y.astype(np.float64) ** 2)) - golden_large["y_rms"]) < 1e-3 * golden_large["y_rms"]


def test_nibble_order_property(golden, oracle):
    """hi_first=False equals the nibble swap of hi_first=True (reference tests/test_qdq.py:277-310)."""
    x = golden["bf16_64x256/x"]
    ts = float(golden["bf16_64x256/ts"][0])
    q_hi, sf_hi = oracle.quantize_nvfp4(x, oracle.BF16, ts, hi_first=True)
    q_lo, sf_lo = oracle.quantize_nvfp4(x, oracle.BF16, ts, hi_first=False)
    assert np.array_equal(sf_hi, sf_lo)
    assert np.array_equal(q_lo, ((q_hi << 4) | (q_hi >> 4)).astype(np.uint8))
    assert np.array_equal(oracle.dequantize_nvfp4(q_hi, ts, sf_hi, oracle.BF16, True),
                          oracle.dequantize_nvfp4(q_lo, ts, sf_lo, oracle.BF16, False))
