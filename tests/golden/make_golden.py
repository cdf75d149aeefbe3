"""Generate the golden vectors in this directory by running the reference's eager backend on CPU.

Usage (needs the reference checkout; not needed to run the tests):

    PYTHONDONTWRITEBYTECODE=1 python tests/golden/make_golden.py --reference /path/to/comfy-kitchen

Outputs ``nvfp4_golden.npz`` (inputs and outputs of small cases, bit patterns as integers) and
``nvfp4_golden_large.json`` (SHA-256 digests, byte sums and samples of the full-size single-linear
config, whose inputs are regenerated from a seeded numpy generator by the tests).

Every expected value comes from calling the reference (``comfy_kitchen`` eager backend,
``comfy_kitchen.float_utils`` and ``TensorCoreNVFP4Layout``); nothing here restates its arithmetic.
"""
from __future__ import annotations

import argparse
import hashlib
import json
import os
import sys

import numpy as np


def bits16(t):
    import torch
    return t.contiguous().view(torch.int16).numpy().view(np.uint16).copy()


def u8(t):
    import torch
    return t.contiguous().view(torch.uint8).numpy().copy()


def sha(a: np.ndarray) -> str:
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.dirname(
        os.path.abspath(__file__))))), "reference"), help="checkout of comfy-kitchen (default: next to this repository)")
    args = ap.parse_args()
    sys.path.insert(0, args.reference)
    sys.dont_write_bytecode = True

    import torch
    import comfy_kitchen as ck
    from comfy_kitchen.float_utils import to_blocked
    from comfy_kitchen.tensor import QuantizedTensor

    torch.set_num_threads(8)
    here = os.path.dirname(os.path.abspath(__file__))
    out: dict[str, np.ndarray] = {}
    names: list[str] = []
    DT = {0: torch.float32, 1: torch.float16, 2: torch.bfloat16}

    def eager_q(x, ts, pad, hi):
        with ck.use_backend("eager"):
            return ck.quantize_nvfp4(x, torch.tensor(ts, dtype=torch.float32), pad_16x=pad, hi_first=hi)

    def eager_dq(q, ts, sf, dt, hi):
        with ck.use_backend("eager"):
            return ck.dequantize_nvfp4(q, torch.tensor(ts, dtype=torch.float32), sf, DT[dt], hi_first=hi)

    def add_quant_case(name, x, dtype_code, ts, pad, hi, dq_dtypes=(2,)):
        """x: torch tensor already in its dtype."""
        q, sf = eager_q(x, ts, pad, hi)
        names.append(name)
        out[f"{name}/x"] = x.numpy().copy() if dtype_code == 0 else bits16(x)
        out[f"{name}/meta"] = np.array([dtype_code, int(pad), int(hi)], np.int64)
        out[f"{name}/ts"] = np.array([ts], np.float32)
        out[f"{name}/q"] = u8(q)
        out[f"{name}/sf"] = u8(sf)
        for dt in dq_dtypes:
            y = eager_dq(q, ts, sf, dt, hi)
            out[f"{name}/dq{dt}"] = y.numpy().copy() if dt == 0 else bits16(y)

    g = torch.Generator().manual_seed(1234)

    def randn(r, c, scale=1.0):
        return torch.randn(r, c, generator=g, dtype=torch.float32) * scale

    def amax_scale(x):
        return float(torch.amax(x.abs()).float() / (448.0 * 6.0))

    # -- the shapes and distribution of the reference's own quantize tests (tests/test_qdq.py:136-190) --
    for (r, c) in [(33, 65), (129, 128), (64, 256)]:
        x = (randn(r, c) * 4).to(torch.bfloat16)
        pad = (r % 16 != 0) or (c % 16 != 0)
        add_quant_case(f"bf16_{r}x{c}", x, 2, amax_scale(x), pad, True, dq_dtypes=(2, 1, 0))
    x = (randn(128, 192) * 4).to(torch.bfloat16)
    add_quant_case("bf16_128x192_lofirst", x, 2, amax_scale(x), False, False, dq_dtypes=(2,))
    x = randn(48, 96).to(torch.float16)
    add_quant_case("f16_48x96", x, 1, amax_scale(x), False, True, dq_dtypes=(1, 2))
    x = randn(32, 160)
    add_quant_case("f32_32x160", x, 0, amax_scale(x), False, True, dq_dtypes=(0, 2))
    x = randn(17, 40)
    add_quant_case("f32_17x40_pad", x, 0, 0.0371234, True, True, dq_dtypes=(0,))

    # -- per-tensor scale variants: power of two, clamp at 448 (tiny ts), subnormal / zero block scales (huge ts) --
    x = randn(32, 128).to(torch.bfloat16)
    add_quant_case("bf16_ts_pow2", x, 2, 2.0 ** -5, False, True)
    add_quant_case("bf16_ts_tiny_clamps", x, 2, 1e-6, False, True)
    add_quant_case("bf16_ts_huge_subnormal", x, 2, 40.0, False, True)
    add_quant_case("bf16_ts_huger_zero", x, 2, 4000.0, False, True)
    add_quant_case("bf16_ts_zero", x, 2, 0.0, False, True, dq_dtypes=())

    # -- outlier channels as in the Flux-class configuration --
    x = randn(64, 512)
    x[:, 37] *= 20
    x = x.to(torch.bfloat16)
    add_quant_case("bf16_outliers", x, 2, amax_scale(x), False, True)

    # -- hand-made edge tile: every e2m1 rounding boundary (ties), signed zeros, saturation, zero blocks --
    ts = 2.0 ** -7
    s = 2.0  # block scale wanted: amax / 6 / ts = 2  -> amax = 12 * ts
    t = ts * s
    bounds = [0.0, 0.25, 0.5, 0.75, 1.0, 1.25, 1.5, 1.75, 2.0, 2.5, 3.0, 3.5, 4.0, 5.0, 6.0]
    rows = []
    for eps in (0.0, 2.0 ** -20, -(2.0 ** -20)):
        for sign in (1.0, -1.0):
            vals = [sign * (b * (1.0 + eps)) * t for b in bounds] + [sign * 6.0 * t]
            rows.append(vals[:16])
    edge = torch.tensor(rows, dtype=torch.float32)                     # [6,16]
    extra = torch.zeros(10, 16)
    extra[0, :] = 0.0                                                  # all-zero block
    extra[1, :] = -0.0
    extra[2, 0] = 6.0 * t
    extra[2, 1:] = torch.tensor([-1e-30, 1e-30, -0.0, 0.0, 1e-10, -1e-10, 0.2499999 * t, -0.2499999 * t,
                                 0.2500001 * t, -0.2500001 * t, 5.9999 * t, -5.9999 * t, 3.0 * t, -3.0 * t, 1e-38])
    extra[3, :] = 1e-12                                                # block scale rounds to zero -> +0 codes
    extra[3, 5] = -1e-12
    extra[4, :] = 3e4                                                  # clamps the block scale at 448
    extra[4, 3] = -7e4
    extra[5, :] = torch.linspace(-6.5, 6.5, 16) * t
    extra[6, :] = torch.linspace(-1.0, 1.0, 16) * t * 0.3
    extra[7, 0] = 2.0 ** -9 * 6 * ts                                   # smallest e4m3 subnormal scale
    extra[8, 0] = 2.0 ** -10 * 6 * ts                                  # tie between 0 and 2^-9 -> 0
    extra[9, 0] = 1.5 * 2.0 ** -9 * 6 * ts                             # tie between 2^-9 and 2^-8
    edge = torch.cat([edge, extra], 0)                                 # [16,16]
    edge = torch.cat([edge, edge.flip(0) * 0.5, edge * 1.0000001, edge.roll(3, 1)], 1).contiguous()  # [16,64]
    add_quant_case("f32_edge_tile", edge, 0, ts, False, True, dq_dtypes=(0, 2, 1))
    add_quant_case("bf16_edge_tile", edge.to(torch.bfloat16), 2, ts, False, True, dq_dtypes=(2,))
    add_quant_case("f16_edge_tile", edge.to(torch.float16), 1, ts, False, False, dq_dtypes=(1,))

    # -- exhaustive e4m3 scale rounding: one block per candidate block-scale value around every boundary --
    cand = []
    for code in range(0, 0x7F):
        v = torch.tensor([code], dtype=torch.uint8).view(torch.float8_e4m3fn).float().item()
        nxt = torch.tensor([code + 1], dtype=torch.uint8).view(torch.float8_e4m3fn).float().item() if code < 0x7E else 480.0
        mid = 0.5 * (v + nxt)
        for f in (v, mid, np.nextafter(np.float32(mid), np.float32(0)), np.nextafter(np.float32(mid), np.float32(1e9))):
            cand.append(float(f))
    cand = torch.tensor(cand, dtype=torch.float32)                     # wanted amax/6/ts values
    ts = 0.25
    xs = torch.zeros(cand.numel(), 16)
    xs[:, 0] = cand * 6.0 * ts
    xs[:, 1] = -0.37 * cand * 6.0 * ts
    n16 = (cand.numel() + 15) // 16 * 16
    xs = torch.cat([xs, torch.zeros(n16 - cand.numel(), 16)], 0)
    add_quant_case("f32_scale_boundaries", xs, 0, ts, False, True, dq_dtypes=())

    # -- swizzle: byte offsets of a (256 x 12) scale matrix under to_blocked --
    iota = torch.arange(256 * 12, dtype=torch.int32).reshape(256, 12)
    out["swizzle/iota_blocked"] = to_blocked(iota, flatten=True).numpy().astype(np.int32)

    # -- dynamic per-tensor scale of the layout (tensor/nvfp4.py:66-71) --
    x = (randn(48, 64) * 3).to(torch.bfloat16)
    qt = QuantizedTensor.from_float(x, "TensorCoreNVFP4Layout")
    out["layout/x"] = bits16(x)
    out["layout/scale"] = qt._params.scale.reshape(1).numpy().astype(np.float32)
    out["layout/q"] = u8(qt._qdata)
    out["layout/sf"] = u8(qt._params.block_scale)

    # -- GEMM restatement on small operands: dequantize(fp32) x2 -> fp32 matmul -> + bias -> bf16 --
    def gemm_ref(qa, tsa, sfa, qb, tsb, sfb, bias):
        da = eager_dq(qa, tsa, sfa, 0, True)
        db = eager_dq(qb, tsb, sfb, 0, True)
        y = da @ db.t()
        if bias is not None:
            y = y + bias.float()
        return y.to(torch.bfloat16)

    for (name, M, N, K, with_bias) in [("gemm_64x128x256", 64, 128, 256, True), ("gemm_48x72x96", 48, 72, 96, False)]:
        a = randn(M, K).to(torch.bfloat16)
        b = randn(N, K, 0.02).to(torch.bfloat16)
        tsa, tsb = amax_scale(a), amax_scale(b)
        qa, sfa = eager_q(a, tsa, False, True)
        qb, sfb = eager_q(b, tsb, False, True)
        bias = randn(1, N, 0.1).reshape(N).to(torch.bfloat16) if with_bias else None
        y = gemm_ref(qa, tsa, sfa, qb, tsb, sfb, bias)
        out[f"{name}/qa"], out[f"{name}/sfa"] = u8(qa), u8(sfa)
        out[f"{name}/qb"], out[f"{name}/sfb"] = u8(qb), u8(sfb)
        out[f"{name}/ts"] = np.array([tsa, tsb], np.float32)
        if bias is not None:
            out[f"{name}/bias"] = bits16(bias)
        out[f"{name}/y"] = bits16(y)

    out["names"] = np.array(names)
    np.savez_compressed(os.path.join(here, "nvfp4_golden.npz"), **out)

    # -- the single-linear configuration (256x1024 activations, 1024x1024 weights), inputs from numpy's generator --
    rng = np.random.default_rng(0)
    x32 = rng.standard_normal((256, 1024), dtype=np.float32)
    w32 = (rng.standard_normal((1024, 1024), dtype=np.float32) * np.float32(0.02)).astype(np.float32)
    x = torch.from_numpy(x32).to(torch.bfloat16)
    w = torch.from_numpy(w32).to(torch.bfloat16)
    tsx, tsw = amax_scale(x), amax_scale(w)
    qx, sfx = eager_q(x, tsx, False, True)
    qw, sfw = eager_q(w, tsw, False, True)
    y = gemm_ref(qx, tsx, sfx, qw, tsw, sfw, None)
    dqx = eager_dq(qx, tsx, sfx, 2, True)
    yb = bits16(y)
    large = {
        "generator": "numpy.random.default_rng(0): x = standard_normal((256,1024), float32); "
                     "w = standard_normal((1024,1024), float32) * float32(0.02); both cast to bf16 (RNE)",
        "x_bits_sha256": sha(bits16(x)), "w_bits_sha256": sha(bits16(w)),
        "ts_x": float(np.float32(tsx)), "ts_w": float(np.float32(tsw)),
        "qx_sha256": sha(u8(qx)), "sfx_sha256": sha(u8(sfx)), "qx_sum": int(u8(qx).astype(np.int64).sum()),
        "sfx_sum": int(u8(sfx).astype(np.int64).sum()),
        "qw_sha256": sha(u8(qw)), "sfw_sha256": sha(u8(sfw)), "qw_sum": int(u8(qw).astype(np.int64).sum()),
        "sfw_sum": int(u8(sfw).astype(np.int64).sum()),
        "dqx_bf16_sha256": sha(bits16(dqx)),
        "y_rms": float(y.float().pow(2).mean().sqrt()),
        "y_sample_stride": [8, 8],
        "y_sample_bits": yb[::8, ::8].astype(int).tolist(),
    }
    with open(os.path.join(here, "nvfp4_golden_large.json"), "w") as f:
        json.dump(large, f)
    print("cases:", len(names), "npz bytes:", os.path.getsize(os.path.join(here, "nvfp4_golden.npz")))


if __name__ == "__main__":
    main()
