"""Worker of test_gpu_gather.py::test_two_ranks_over_nvlink (one process per GPU under torch.distributed.run)."""
from __future__ import annotations

import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


def main() -> int:
    import comfy_kitchen_b200 as ckb
    from comfy_kitchen_b200.sharded import replicated_from_seed

    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    dev = torch.device("cuda", int(os.environ["LOCAL_RANK"]))
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", device_id=dev)
    ok = True
    peers = ckb.PeerGroup(dev)
    # small shapes, then the four linears of the Flux-class block at its full M (the shapes the benchmark times)
    for (M, K, N, seed) in [(1024, 1024, 2048, 1), (1024, 3072, 3072, 2), (4608, 3072, 9216, 3), (4608, 3072, 3072, 4),
                            (4608, 3072, 12288, 5), (4608, 12288, 3072, 6)]:
        if (N // world) % 8 or N // world <= 128:
            continue
        x = replicated_from_seed((M, K), seed, 1.0, torch.bfloat16, dev)
        w = replicated_from_seed((N, K), seed + 100, 0.02, torch.bfloat16, dev)
        lin = ckb.ShardedNVFP4Linear(w, None, input_scale=ckb.dynamic_scale_nvfp4(x))
        want = lin(x)                                  # NCCL all-gather of the column blocks
        lin.bind(peers, M)
        for it in range(3):                            # repeated steps reuse the matrices: barrier on both sides
            peers.barrier()
            got = lin.fused(x)
            peers.barrier()
            torch.cuda.synchronize()
            same = torch.equal(got, want)
            ok = ok and same
            if not same:
                nl = N // world
                blocks = [int((got[:, r * nl:(r + 1) * nl] != want[:, r * nl:(r + 1) * nl]).sum()) for r in range(world)]
                print(f"rank {rank}: M={M} K={K} N={N} iteration {it}: fused result differs; differing elements per "
                      f"rank's column block {blocks}", flush=True)
    status = ckb.read_device_status()
    ok = ok and status == 0
    flag = torch.tensor([1 if ok else 0], device=dev)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    peers.close()
    dist.barrier()
    if rank == 0 and int(flag.item()) == 1:
        print("ALL_RANKS_OK", flush=True)
    dist.destroy_process_group()
    return 0 if int(flag.item()) == 1 else 1


if __name__ == "__main__":
    sys.exit(main())
