"""scaled_mm_nvfp4 fused with the all-gather of its column blocks.

On one GPU the ranks are emulated one after the other in one process: every "rank" gets the same list of output
matrices (all in local memory), so the kernel's store-to-the-other-ranks path runs exactly as it does over NVLink.
With two or more GPUs the real thing runs as one process per GPU (peer-mapped memory, the stream-ordered barrier)
and is compared with the NCCL all-gather of the same blocks.
"""
from __future__ import annotations

import os
import subprocess
import sys

import pytest
import torch

from helpers import amax_scale, seeded_randn

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.parametrize("shape", [(512, 1024, 1024, 2), (300, 768, 512, 2), (1024, 3072, 256, 4), (4608, 3072, 3072, 8)],
                         ids=lambda s: "x".join(map(str, s)))
@pytest.mark.parametrize("with_bias", [False, True])
def test_emulated_ranks_match_unsharded(shape, with_bias):
    import comfy_kitchen_b200 as ckb
    from comfy_kitchen_b200 import ops
    M, N, K, world = shape
    x = seeded_randn((M, K), seed=11).cuda()
    w = seeded_randn((N, K), seed=12, std=0.02).cuda()
    bias = seeded_randn((1, N), seed=13, std=0.5).reshape(N).cuda() if with_bias else None
    tsx, tsw = amax_scale(x).cuda(), amax_scale(w).cuda()
    pad = M % 16 != 0
    qx, sfx = ckb.quantize_nvfp4(x, tsx, pad_16x=pad)
    qw, sfw = ckb.quantize_nvfp4(w, tsw)
    want = ckb.scaled_mm_nvfp4(qx, qw, tsx, tsw, sfx, sfw, bias=bias)[:M]
    n_local = N // world
    outs = [torch.full((M, N), float("nan"), dtype=torch.bfloat16, device="cuda") for _ in range(world)]   # M rows: unpadded
    ptrs = [o.data_ptr() for o in outs]
    for rank in range(world):
        shard = w[rank * n_local:(rank + 1) * n_local].contiguous()
        qs, sfs = ckb.quantize_nvfp4(shard, tsw)
        b = None if bias is None else bias[rank * n_local:(rank + 1) * n_local].contiguous()
        ops.scaled_mm_nvfp4_all_gather(qx, qs, tsx, tsw, sfx, sfs, ptrs, rank, bias=b, rows=M)
    torch.cuda.synchronize()
    assert ckb.read_device_status() == 0
    for r, o in enumerate(outs):
        assert torch.equal(o, want), f"matrix of rank {r} differs from the unsharded product"


def test_gather_rejects_unsupported():
    import comfy_kitchen_b200 as ckb
    from comfy_kitchen_b200 import ops
    x = seeded_randn((64, 256), seed=1).cuda()
    w = seeded_randn((256, 256), seed=2, std=0.02).cuda()
    ts = amax_scale(x).cuda()
    qx, sfx = ckb.quantize_nvfp4(x, ts)
    qw, sfw = ckb.quantize_nvfp4(w, ts)
    out = torch.empty((64, 256), dtype=torch.bfloat16, device="cuda")
    with pytest.raises(RuntimeError, match="M > 128"):
        ops.scaled_mm_nvfp4_all_gather(qx, qw, ts, ts, sfx, sfw, [out.data_ptr()], 0)


def test_single_rank_barrier_and_peer_memory():
    """world = 1: the barrier has nobody to wait for, and peer memory is plain zeroed device memory."""
    import comfy_kitchen_b200 as ckb
    pg = ckb.PeerGroup(torch.device("cuda", 0))
    mem = pg.alloc(1 << 20)
    t = mem.tensor((512, 1024), torch.bfloat16)
    assert t.data_ptr() == mem.ptrs[0] and float(t.abs().sum()) == 0.0
    for _ in range(3):
        pg.barrier()
    torch.cuda.synchronize()
    assert int(pg.epoch.item()) == 3 and ckb.read_device_status() == 0
    pg.close()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_ranks_over_nvlink():
    """One process per GPU: fused GEMM + all-gather against the NCCL all-gather of the same column blocks."""
    n = min(torch.cuda.device_count(), 4)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}", "--master-addr",
           "127.0.0.1", "--master-port", "29533", os.path.join(ROOT, "tests", "multi_gpu_worker.py")]
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    res = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=240)
    assert res.returncode == 0, res.stdout[-3000:] + res.stderr[-3000:]
    assert "ALL_RANKS_OK" in res.stdout
