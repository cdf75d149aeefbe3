"""The CPU oracle's MXFP8 restatement against vectors produced by the reference eager backend
(tests/golden/make_golden_mxfp8.py): bit-exact data bytes, scale bytes and dequantized values."""
from __future__ import annotations

import os

import numpy as np
import pytest

HERE = os.path.dirname(os.path.abspath(__file__))


@pytest.fixture(scope="module")
def mx_golden():
    return np.load(os.path.join(HERE, "golden", "mxfp8_golden.npz"))


def mx_case_names():
    return [str(n) for n in np.load(os.path.join(HERE, "golden", "mxfp8_golden.npz"))["quantize_cases"]]


@pytest.mark.parametrize("name", mx_case_names())
def test_quantize_and_dequantize_match_reference(name, mx_golden, oracle):
    dtype, pad = (int(v) for v in mx_golden[f"{name}/meta"])
    q, sf = oracle.quantize_mxfp8(mx_golden[f"{name}/x"], dtype, bool(pad))
    assert np.array_equal(sf, mx_golden[f"{name}/sf"]), "scale bytes differ from the reference"
    assert np.array_equal(q, mx_golden[f"{name}/q"]), "data bytes differ from the reference"
    for code in (0, 1, 2):
        key = f"{name}/dq{code}"
        if key in mx_golden.files:
            d = oracle.dequantize_mxfp8(mx_golden[f"{name}/q"], mx_golden[f"{name}/sf"], code)
            want = mx_golden[key]
            assert np.array_equal(d.view(np.uint32) if code == 0 else d, want.view(np.uint32) if code == 0 else want)


@pytest.mark.parametrize("name", ["gemm_32x128x64", "gemm_96x160x256_bias"])
def test_gemm_restatement_matches_dequantize_linear(name, mx_golden, oracle):
    bias = mx_golden[f"{name}/bias"] if f"{name}/bias" in mx_golden.files else None
    y = oracle.scaled_mm_mxfp8(mx_golden[f"{name}/qa"], mx_golden[f"{name}/qb"], mx_golden[f"{name}/sa"],
                               mx_golden[f"{name}/sb"], bias=bias, out_dtype=0)
    ref = mx_golden[f"{name}/y_f32"]
    rel = float(np.sqrt(((y - ref) ** 2).mean()) / np.sqrt((ref ** 2).mean()))
    assert rel <= 1e-6
