"""Host logic of the N-sharded NVFP4 linear on CPU: world_size-2 gloo ranks with the CPU oracle standing in
for the kernels.  Checks shard boundaries, the global weight scale, the all-gather and its re-layout, and that
a missing rank surfaces as an error on the host (no GPU involved)."""
from __future__ import annotations

import os
import socket
import sys
from types import SimpleNamespace

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _oracle_ops():
    """quantize / scaled_mm / dynamic scale with the operator signatures, computed by the CPU oracle."""
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    from helpers import CODE, from_bits, to_bits
    from oracle import oracle as o

    def quantize_nvfp4(x, per_tensor_scale, epsilon=0.0, pad_16x=False, hi_first=True):
        q, sf = o.quantize_nvfp4(to_bits(x), CODE[x.dtype], float(per_tensor_scale), pad_16x, hi_first)
        return torch.from_numpy(q), torch.from_numpy(sf).view(torch.float8_e4m3fn)

    def scaled_mm_nvfp4(a, b, tsa, tsb, sfa, sfb, bias=None, out_dtype=None, alpha=None):
        y = o.scaled_mm_nvfp4(a.numpy(), b.numpy(), float(tsa), float(tsb), sfa.view(torch.uint8).numpy(),
                              sfb.view(torch.uint8).numpy(), bias=None if bias is None else to_bits(bias))
        return from_bits(y, 2)

    def dynamic_scale_nvfp4(x):
        return torch.tensor(o.dynamic_scale(to_bits(x), CODE[x.dtype]), dtype=torch.float32)

    return SimpleNamespace(quantize_nvfp4=quantize_nvfp4, scaled_mm_nvfp4=scaled_mm_nvfp4,
                           dynamic_scale_nvfp4=dynamic_scale_nvfp4)


def _worker(rank, world, port, n_out, result_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        sys.path.insert(0, ROOT)
        import comfy_kitchen_b200 as ckb
        from comfy_kitchen_b200.sharded import replicated_from_seed
        ops = _oracle_ops()
        w = replicated_from_seed((n_out, 128), seed=1, std=0.02, dtype=torch.bfloat16, device="cpu")
        x = replicated_from_seed((48, 128), seed=2, std=1.0, dtype=torch.bfloat16, device="cpu")
        bias = replicated_from_seed((1, n_out), seed=3, std=0.1, dtype=torch.bfloat16, device="cpu").reshape(n_out)
        lin = ckb.ShardedNVFP4Linear(w, bias, ops=ops)
        assert (lin.n0, lin.n1) == ckb.shard_rows(n_out, world, rank)
        y = lin(x)
        assert tuple(y.shape) == (48, n_out)
        # unsharded result with the same global scale
        full = ckb.ShardedNVFP4Linear.__new__(ckb.ShardedNVFP4Linear)
        ts_w = ops.dynamic_scale_nvfp4(w)
        assert float(ts_w) == float(lin.weight_scale)
        qw, sfw = ops.quantize_nvfp4(w, ts_w, pad_16x=n_out % 16 != 0)
        ts_x = ops.dynamic_scale_nvfp4(x)
        qx, sfx = ops.quantize_nvfp4(x, ts_x)
        ref = ops.scaled_mm_nvfp4(qx, qw, ts_x, ts_w, sfx, sfw, bias=None)[:, :n_out].float() + bias.float()
        err = (y.float() - ref).abs().max().item()
        assert err <= 0.02 * ref.abs().max().item() + 1e-6, err
        if len({b - a for a, b in (ckb.shard_rows(n_out, world, r) for r in range(world))}) == 1:
            buf = lin.gather(lin.local(x), row_major=False)
            assert tuple(buf.shape) == (world, 48, n_out // world)
            assert torch.equal(buf.permute(1, 0, 2).reshape(48, n_out), y)
        # the two halves a caller may put on different streams give the block of local()
        qx2, sfx2, ts2 = lin.quantize_input(x)
        assert torch.equal(lin.local_from_quantized(qx2, sfx2, ts2, x.shape[0]), lin.local(x))
        # a dynamic quantizer, where the operator set has one, is what quantize_input uses when no scale is stored
        calls = []

        def quantize_nvfp4_dynamic(x, pad_16x=False, hi_first=True):
            calls.append(tuple(x.shape))
            t = ops.dynamic_scale_nvfp4(x)
            return ops.quantize_nvfp4(x, t, pad_16x=pad_16x, hi_first=hi_first) + (t,)

        ops2 = SimpleNamespace(**vars(ops), quantize_nvfp4_dynamic=quantize_nvfp4_dynamic)
        lin2 = ckb.ShardedNVFP4Linear(w, bias, ops=ops2)
        assert torch.equal(lin2(x), y) and calls == [(48, 128)]
        lin3 = ckb.ShardedNVFP4Linear(w, bias, ops=ops2, input_scale=ops.dynamic_scale_nvfp4(x))
        assert torch.equal(lin3(x), y) and len(calls) == 1     # a stored scale is used as it is
        # a group whose peer-mapping limit the layer's output matrices would pass: bind() declines with a warning and
        # fused() hands back the same matrix through the library collective
        if len({b - a for a, b in (ckb.shard_rows(n_out, world, r) for r in range(world))}) == 1:
            import warnings

            class FullGroup:      # the part of PeerGroup that bind() consults, with no room left
                world, mapped_bytes, map_limit_bytes = 2, 10 << 30, 10 << 30

                def fits(self, nbytes):
                    return False

                def alloc(self, nbytes):
                    raise AssertionError("bind() must not allocate beyond the limit")

            with warnings.catch_warnings(record=True) as caught:
                warnings.simplefilter("always")
                assert lin.bind(FullGroup(), 48) is None
            assert any("NCCL all-gather" in str(wn.message) for wn in caught)
            assert torch.equal(lin.fused(x), y)
        np.save(os.path.join(result_dir, f"ok{rank}.npy"), np.array([1]))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("n_out", [256, 264])
def test_sharded_linear_two_ranks(n_out, tmp_path):
    from oracle import oracle as o
    o.build()
    port = _free_port()
    mp.spawn(_worker, args=(2, port, n_out, str(tmp_path)), nprocs=2, join=True)
    assert os.path.exists(tmp_path / "ok0.npy") and os.path.exists(tmp_path / "ok1.npy")


def test_shard_rows_cover_and_align():
    sys.path.insert(0, ROOT)
    from comfy_kitchen_b200.sharded import shard_rows
    for n in (3072, 9216, 12288, 5120, 13824, 15360, 264, 8):
        for world in (1, 2, 4, 8):
            edges = [shard_rows(n, world, r) for r in range(world)]
            assert edges[0][0] == 0 and edges[-1][1] == n
            for (a0, a1), (b0, b1) in zip(edges, edges[1:]):
                assert a1 == b0
            assert all((b - a) % 8 == 0 for a, b in edges)
    with pytest.raises(ValueError):
        shard_rows(100, 2, 0)


def _absent_rank_worker(rank, world, port, result_dir):
    from datetime import timedelta
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=timedelta(seconds=5))
    if rank == 1:
        return            # leaves between steps, before the collective, with nothing in flight
    t = torch.zeros(4)
    try:
        dist.all_gather_into_tensor(torch.zeros(8), t)
        outcome = "completed"
    except Exception as e:   # the survivor learns of the failure on the host
        outcome = type(e).__name__
    with open(os.path.join(result_dir, "outcome.txt"), "w") as f:
        f.write(outcome)


def test_absent_rank_is_reported_on_the_host(tmp_path):
    port = _free_port()
    mp.spawn(_absent_rank_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    assert open(tmp_path / "outcome.txt").read() != "completed"
