"""Generate ``mxfp8_golden.npz`` by running the reference's eager MXFP8 operators on CPU.

Usage (needs the reference checkout; not needed to run the tests):

    PYTHONDONTWRITEBYTECODE=1 python tests/golden/make_golden_mxfp8.py --reference /path/to/comfy-kitchen

Every expected value comes from calling the reference (``comfy_kitchen`` eager backend: quantize_mxfp8,
dequantize_mxfp8); the GEMM expectation is the check the reference's tests apply to scaled_mm_mxfp8
(``tests/test_tensor.py:1181-1214``): linear on the dequantized operands.
"""
from __future__ import annotations

import argparse
import os
import sys

import numpy as np


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.dirname(
        os.path.abspath(__file__))))), "reference"), help="checkout of comfy-kitchen (default: next to this repository)")
    args = ap.parse_args()
    sys.path.insert(0, args.reference)
    sys.dont_write_bytecode = True
    import torch
    import comfy_kitchen as ck

    torch.set_num_threads(8)
    here = os.path.dirname(os.path.abspath(__file__))
    out: dict[str, np.ndarray] = {}
    names: list[str] = []
    CODE = {torch.float32: 0, torch.float16: 1, torch.bfloat16: 2}
    DT = {0: torch.float32, 1: torch.float16, 2: torch.bfloat16}

    def bits(t):
        t = t.contiguous()
        if t.dtype == torch.float32:
            return t.numpy().copy()
        if t.dtype in (torch.float16, torch.bfloat16):
            return t.view(torch.int16).numpy().view(np.uint16).copy()
        return t.view(torch.uint8).numpy().copy()

    def add(name, x, pad, dq=(2,)):
        with ck.use_backend("eager"):
            q, sf = ck.quantize_mxfp8(x, pad_32x=pad)
            out[f"{name}/x"] = bits(x)
            out[f"{name}/meta"] = np.array([CODE[x.dtype], int(pad)], np.int64)
            out[f"{name}/q"] = bits(q)
            out[f"{name}/sf"] = bits(sf)
            for code in dq:
                out[f"{name}/dq{code}"] = bits(ck.dequantize_mxfp8(q, sf, DT[code]))
        names.append(name)

    g = torch.Generator().manual_seed(0)
    # the shapes and distribution of the reference's own test (tests/test_qdq.py:406-418)
    add("bf16_128x256", (torch.randn((128, 256), generator=g) * 10).to(torch.bfloat16), False, dq=(2, 1, 0))
    add("bf16_65x96_pad", (torch.randn((65, 96), generator=g) * 10).to(torch.bfloat16), True)
    add("bf16_160x512", (torch.randn((160, 512), generator=g) * 10).to(torch.bfloat16), False)
    add("f16_128x256", torch.randn((128, 256), generator=g).to(torch.float16), False, dq=(1,))
    add("f32_128x512", torch.randn((128, 512), generator=g), False, dq=(0, 2))
    add("f32_150x200_pad", torch.randn((150, 200), generator=g) * 0.01, True, dq=(0,))
    # activations with outlier channels and a wide dynamic range
    x = torch.randn((128, 512), generator=g)
    x[:, ::97] *= 50
    x[40:80] *= 1e-3
    add("bf16_outliers", x.to(torch.bfloat16), False)
    # hand-made blocks: every e4m3 rounding boundary at scale 1 (amax = 448), zero blocks, signed zeros, block
    # amax on exact powers of two times 448 (quotient exactly a power of two), one step above and below
    e4 = torch.arange(0, 0x7f, dtype=torch.uint8).view(torch.float8_e4m3fn).float()          # all finite non-negative codes
    mids = (e4[:-1] + e4[1:]) / 2
    vals = torch.cat([e4, mids, torch.nextafter(mids, torch.tensor(0.0)), torch.nextafter(mids, torch.tensor(1e9))])
    vals = torch.cat([vals, -vals])
    n = (vals.numel() + 30) // 31
    rows = torch.zeros((n, 32))
    rows[:, 0] = 448.0                                                                         # pins the block scale to 1
    rows[:, 1:] = torch.nn.functional.pad(vals, (0, n * 31 - vals.numel())).reshape(n, 31)
    extra = torch.zeros((8, 32))
    extra[1] = -0.0
    extra[2, 0] = 448.0 * 4
    extra[2, 1:] = torch.linspace(-1800, 1800, 31)
    extra[3, 0] = 448.0 * 0.25
    extra[3, 1:] = torch.linspace(-112, 112, 31)
    extra[4, 0] = float(torch.nextafter(torch.tensor(448.0), torch.tensor(1e9)))              # just above a power of two
    extra[4, 1:] = torch.linspace(-448, 448, 31)
    extra[5, 0] = float(torch.nextafter(torch.tensor(448.0), torch.tensor(0.0)))
    extra[5, 1:] = torch.linspace(-448, 448, 31)
    extra[6] = 1e-30
    extra[7] = 3e30
    extra[7, 5] = -1e20
    tile = torch.cat([rows, extra], 0)
    pad_rows = (-tile.shape[0]) % 32
    tile = torch.nn.functional.pad(tile, (0, 0, 0, pad_rows))
    tile = torch.cat([tile, tile.flip(0) * 0.5, tile * 3.0, tile.roll(5, 1)], 1).contiguous()   # 128 columns
    add("f32_boundaries", tile, False, dq=(0, 2))
    add("bf16_boundaries", tile.to(torch.bfloat16), False)

    # small GEMMs, checked the way the reference's tests check scaled_mm_mxfp8: linear on the dequantized operands
    for name, (M, N, K, with_bias) in {"gemm_32x128x64": (32, 128, 64, False), "gemm_96x160x256_bias": (96, 160, 256, True)}.items():
        xa = torch.randn((M, K), generator=g).to(torch.bfloat16)
        wb = torch.randn((N, K), generator=g).to(torch.bfloat16)
        bias = torch.randn(N, generator=g).to(torch.bfloat16) if with_bias else None
        with ck.use_backend("eager"):
            qa, sa = ck.quantize_mxfp8(xa)
            qb, sb = ck.quantize_mxfp8(wb)
            da, db = ck.dequantize_mxfp8(qa, sa, torch.float32), ck.dequantize_mxfp8(qb, sb, torch.float32)
        y = torch.nn.functional.linear(da, db, None if bias is None else bias.float())
        out[f"{name}/qa"], out[f"{name}/sa"], out[f"{name}/qb"], out[f"{name}/sb"] = bits(qa), bits(sa), bits(qb), bits(sb)
        if bias is not None:
            out[f"{name}/bias"] = bits(bias)
        out[f"{name}/y_f32"] = y.numpy().copy()
    out["quantize_cases"] = np.array(names)
    np.savez_compressed(os.path.join(here, "mxfp8_golden.npz"), **out)
    print("wrote mxfp8_golden.npz with", len(names), "quantize cases,", sum(v.nbytes for v in out.values()) >> 10, "KiB raw")


if __name__ == "__main__":
    main()
