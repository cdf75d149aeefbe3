"""Loading a quantized linear in the reference's checkpoint format as per-rank shards (host logic, CPU only):
the shard cut from the full checkpoint is bit-identical to quantizing those weight rows directly."""
from __future__ import annotations

import os
import sys

import numpy as np
import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.join(ROOT, "tests"))

from test_sharded_gloo import _oracle_ops  # noqa: E402


def test_scale_tiling_round_trip_matches_reference_formula(oracle):
    from comfy_kitchen_b200.sharded import scale_offsets, tile_scales, untile_scales
    g = torch.Generator().manual_seed(0)
    for rows, kblocks in [(128, 4), (200, 6), (1, 1), (384, 192), (130, 7)]:
        logical = torch.randint(1, 255, (rows, kblocks), generator=g, dtype=torch.uint8)
        tiled = tile_scales(logical)
        assert tiled.shape == ((rows + 127) // 128 * 128, (kblocks + 3) // 4 * 4)
        assert torch.equal(untile_scales(tiled, rows, kblocks), logical)
        assert int(tiled.to(torch.int64).sum()) == int(logical.to(torch.int64).sum())   # padding is zero
        off = scale_offsets(rows, kblocks)
        assert len(set(off.reshape(-1).tolist())) == rows * kblocks                      # a permutation


@pytest.mark.parametrize("n_out,world", [(256, 2), (384, 2), (200, 4), (1728, 8)])
def test_shard_from_checkpoint_equals_quantizing_the_rows(n_out, world):
    import comfy_kitchen_b200 as ckb
    ops = _oracle_ops()
    g = torch.Generator().manual_seed(n_out)
    k = 192
    w = (torch.randn((n_out, k), generator=g) * 0.02).to(torch.bfloat16)
    bias = (torch.randn(n_out, generator=g) * 0.1).to(torch.bfloat16)
    ts = ops.dynamic_scale_nvfp4(w)
    q, sf = ops.quantize_nvfp4(w, ts, pad_16x=n_out % 16 != 0)
    sd = {"layer.weight": q[:n_out], "layer.weight_scale": sf.view(torch.uint8).reshape(-1),   # flat, like the sample
          "layer.weight_scale_2": ts, "layer.bias": bias, "layer.input_scale": torch.tensor(0.01)}
    for rank in range(world):
        direct = ckb.ShardedNVFP4Linear(w, bias, ops=ops, world=world, rank=rank, input_scale=torch.tensor(0.01))
        loaded = ckb.ShardedNVFP4Linear.from_state_dict(sd, "layer.", ops=ops, world=world, rank=rank)
        assert (loaded.n0, loaded.n1, loaded.local_rows) == (direct.n0, direct.n1, direct.local_rows)
        assert torch.equal(loaded.qweight, direct.qweight)
        assert torch.equal(loaded.weight_block_scale.view(torch.uint8), direct.weight_block_scale.view(torch.uint8))
        assert float(loaded.weight_scale) == float(direct.weight_scale) and float(loaded.input_scale) == float(torch.tensor(0.01))
        assert torch.equal(loaded.bias, direct.bias)
        x = (torch.randn((32, k), generator=g)).to(torch.bfloat16)
        assert torch.equal(loaded.local(x), direct.local(x))
