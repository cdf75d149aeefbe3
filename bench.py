#!/usr/bin/env python
"""Benchmark of the NVFP4 linear hot path (quantize_nvfp4 -> scaled_mm_nvfp4) on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload flux|wan]

One "step" is one pass of the path over the four linears of a Flux-class DiT block (M = 4608 tokens,
hidden 3072: QKV 3072->9216, attn-out 3072->3072, MLP-up 3072->12288, MLP-down 12288->3072): for each linear
the bf16 activation is block-quantized to NVFP4 and multiplied with the resident NVFP4 weight, bf16 out.
Inputs are seeded synthetic tensors with the shapes and distributions of that model class (activations
N(0,1) with 0.1 % of the channels scaled x20, weights N(0,0.02)); no model weights or datasets are involved.

Prints ONE JSON line.  `value` is whole-job TFLOP/s (2*M*N*K summed over the linears / step time, device
resident inputs); `e2e` is the same metric with pinned host inputs and host outputs, copies inside the timed
region; `roofline` describes the dominant kernel (the GEMM); `cpu_baseline` is the CPU oracle timed on a
bounded sample of the same workload on this box's host cores.

With --gpus N > 1 (launched under torchrun, one rank per GPU) every weight is sharded along N, each rank
multiplies its shard and the bf16 column blocks are all-gathered over NCCL: total work is fixed ("strong").
`--impl reference` times the CPU restatement of the reference eager path (the oracle) as the reference arm.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

FLUX = {"name": "flux_dit_block_linears", "M": 4608,
        "linears": [("qkv", 3072, 9216), ("attn_out", 3072, 3072), ("mlp_up", 3072, 12288), ("mlp_down", 12288, 3072)]}
WAN = {"name": "wan14b_dit_block_linears", "M": 32760,
       "linears": [("qkv", 5120, 15360), ("attn_out", 5120, 5120), ("ffn_up", 5120, 13824), ("ffn_down", 13824, 5120)]}
WORKLOADS = {"flux": FLUX, "wan": WAN}
NOMINAL_NVFP4_TFLOPS = 9000.0   # vendor dense NVFP4 figure for B200; MEASURED_PEAKS.json holds no FP4 number
METRIC = "scaled_mm_nvfp4 TFLOPS over the NVFP4 linear path (quantize_nvfp4 + scaled_mm_nvfp4 per linear)"


def flops_per_step(wl) -> float:
    return sum(2.0 * wl["M"] * n * k for _, k, n in wl["linears"])


def make_inputs(wl, device, dtype):
    """Seeded activations and weights, generated on the CPU so that every rank and the CPU arm see the same bits."""
    import torch
    xs, ws = [], []
    for i, (_, k, n) in enumerate(wl["linears"]):
        g = torch.Generator().manual_seed(1000 + i)
        x = torch.randn((wl["M"], k), generator=g, dtype=torch.float32)
        cols = torch.randperm(k, generator=g)[: max(1, round(k / 1000))]
        x[:, cols] *= 20.0
        w = torch.randn((n, k), generator=g, dtype=torch.float32) * 0.02
        xs.append(x.to(dtype))
        ws.append(w.to(dtype))
    return xs, ws


class ClockSampler:
    """SM clock and throttle-reason samples taken through NVML (read-only) by a thread while the GPU is under load."""

    def __init__(self, gpu_index: int, period_s: float = 0.002):
        self.gpu_index = gpu_index
        self.period_s = period_s
        self.samples = []
        self.reasons = 0
        self.max_mhz = None
        self._stop = False
        self._thread = None
        self._nvml = None

    def start(self):
        try:
            import threading

            import pynvml
            pynvml.nvmlInit()
            # torch's device ordinal follows CUDA_VISIBLE_DEVICES; map it to the NVML handle through the PCI bus id
            import torch
            bus = torch.cuda.get_device_properties(self.gpu_index).pci_bus_id if hasattr(
                torch.cuda.get_device_properties(self.gpu_index), "pci_bus_id") else None
            handle = None
            if bus is not None:
                for i in range(pynvml.nvmlDeviceGetCount()):
                    h = pynvml.nvmlDeviceGetHandleByIndex(i)
                    if pynvml.nvmlDeviceGetPciInfo(h).bus == bus:
                        handle = h
                        break
            if handle is None:
                handle = pynvml.nvmlDeviceGetHandleByIndex(self.gpu_index)
            self._nvml = (pynvml, handle)
            self.max_mhz = float(pynvml.nvmlDeviceGetMaxClockInfo(handle, pynvml.NVML_CLOCK_SM))

            def loop():
                while not self._stop:
                    try:
                        self.samples.append(float(pynvml.nvmlDeviceGetClockInfo(handle, pynvml.NVML_CLOCK_SM)))
                        self.reasons |= int(pynvml.nvmlDeviceGetCurrentClocksEventReasons(handle))
                    except Exception:
                        pass
                    time.sleep(self.period_s)

            self._thread = threading.Thread(target=loop, daemon=True)
            self._thread.start()
        except Exception:
            self._thread = None

    def stop(self) -> dict:
        out = {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": [], "samples": 0}
        if self._thread is None:
            return out
        self._stop = True
        self._thread.join(timeout=2)
        pynvml, _ = self._nvml
        names = {"hw_slowdown": pynvml.nvmlClocksEventReasonHwSlowdown,
                 "hw_thermal_slowdown": pynvml.nvmlClocksEventReasonHwThermalSlowdown,
                 "sw_thermal_slowdown": pynvml.nvmlClocksEventReasonSwThermalSlowdown,
                 "sw_power_cap": pynvml.nvmlClocksEventReasonSwPowerCap,
                 "hw_power_brake": pynvml.nvmlClocksEventReasonHwPowerBrakeSlowdown}
        out["reasons"] = sorted(k for k, bit in names.items() if self.reasons & bit)
        if self.samples:
            sm = sorted(self.samples)
            out.update(sm_mhz=sm[len(sm) // 2], samples=len(sm), sm_min_mhz=sm[0], sm_p90_mhz=sm[int(len(sm) * 0.9)])
        return out


def measured_peaks() -> dict:
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return json.load(f)
    except Exception:
        return {}


# ------------------------------------------------------------------------------------------------ CPU arm


def cpu_reference_step(wl, xs_bits, w_q, rows: int):
    """One bounded sample of the workload through the CPU oracle: the first `rows` tokens of every linear.
    Quantize the activation slice, then dequantize both operands to fp32, fp32 matmul, bf16 out."""
    from oracle import oracle as o
    fl = 0.0
    for (x_bits, ts_x), (qw, sfw, ts_w), (_, k, n) in zip(xs_bits, w_q, wl["linears"]):
        qx, sfx = o.quantize_nvfp4(x_bits[:rows], o.BF16, ts_x)
        o.scaled_mm_nvfp4(qx, qw, ts_x, ts_w, sfx, sfw)
        fl += 2.0 * rows * n * k
    return fl


def prepare_cpu(wl, xs, ws):
    import numpy as np
    import torch
    from oracle import oracle as o
    o.build()
    xs_bits, w_q = [], []
    for x, w in zip(xs, ws):
        xb = x.view(torch.int16).numpy().view(np.uint16)
        wb = w.view(torch.int16).numpy().view(np.uint16)
        ts_x = float(x.abs().amax().float() / 2688.0)
        ts_w = float(w.abs().amax().float() / 2688.0)
        qw, sfw = o.quantize_nvfp4(wb, o.BF16, ts_w)
        xs_bits.append((xb, ts_x))
        w_q.append((qw, sfw, ts_w))
    return xs_bits, w_q, o.num_threads()


def run_reference_arm(args, wl):
    import torch
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    torch.manual_seed(0)
    xs, ws = make_inputs(wl, "cpu", torch.bfloat16)
    xs_bits, w_q, threads = prepare_cpu(wl, xs, ws)
    rows = min(1152, wl["M"])
    for _ in range(max(1, args.warmup)):
        cpu_reference_step(wl, xs_bits, w_q, rows)
    t0 = time.perf_counter()
    fl = 0.0
    for _ in range(args.steps):
        fl += cpu_reference_step(wl, xs_bits, w_q, rows)
    dt = time.perf_counter() - t0
    val = fl / dt / 1e12
    sample = f"first {rows} of {wl['M']} tokens of each of the {len(wl['linears'])} linears per step"
    line = {
        "impl": "reference", "metric": METRIC, "value": val, "unit": "TFLOP/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt / args.steps * 1e3, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "nvfp4 (e2m1 x e4m3 block scales), fp32 accumulate",
        "data": "synthetic", "config": {"workload": wl["name"], "M": wl["M"], "linears": wl["linears"], "sample": sample},
        "cpu_baseline": {"value": val, "unit": "TFLOP/s", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": val, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
        "note": "CPU restatement of the reference eager path (quantize_nvfp4 eager; scaled_mm_nvfp4 = dequantize to "
                "fp32 + fp32 BLAS matmul, the check the reference's own tests use since its eager GEMM has no CPU kernel)",
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------------ GPU arm


def run_ours(args, wl):
    import torch
    import torch.distributed as dist
    import comfy_kitchen_b200 as ckb

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: comfy_kitchen_b200 has no CPU path")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if args.no_dependent_launch:
        ckb.set_tuning(3, 0)
    elif args.dependent_launch_mask is not None:
        ckb.set_tuning(3, args.dependent_launch_mask)
    distributed = world > 1
    if distributed:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)
    # N > 1, default: the GEMM's epilogue stores its tiles into every rank's output matrix (peer memory over
    # NVLink) and the ranks meet at a stream-ordered barrier kernel before and after the step, so a step holds no
    # library collective and is captured in a CUDA graph like the single-GPU step.  --collective nccl keeps the
    # NCCL all-gather instead; it launches eagerly: a captured step with all-gathers in it ran 5 % faster on 2 GPUs
    # but the process then hung while tearing the process group down, so library collectives stay out of graphs
    fused = distributed and args.collective == "fused"
    use_graph = (not distributed or fused) and not args.no_graph
    # --fused-linear: each linear is one call of the library's whole-linear entry point with the quantizer inside
    # the GEMM kernel (same bits as quantize_nvfp4 followed by scaled_mm_nvfp4; measured slower, so not the default)
    one_call = args.fused_linear
    if one_call:
        ckb.set_tuning(4, 1)

    M = wl["M"]
    pad_m = M % 16 != 0
    xs_cpu, ws_cpu = make_inputs(wl, "cpu", torch.bfloat16)
    xs = [x.to(dev) for x in xs_cpu]
    # static per-tensor activation scales (the optional `input_scale` of an NVFP4 checkpoint), amax/(448*6)
    ts_x = [ckb.dynamic_scale_nvfp4(x) for x in xs]
    layers = [ckb.ShardedNVFP4Linear(w.to(dev), None, input_scale=t) for w, t in zip(ws_cpu, ts_x)]
    torch.cuda.synchronize()
    side = torch.cuda.Stream()
    graphs = []

    equal_shards = all(n % (8 * world) == 0 for _, _, n in wl["linears"])
    peers = None
    if fused and not (equal_shards and M > 128 and all(n // world > 128 for _, _, n in wl["linears"])):
        fused = False            # the fused kernel wants equal shards wider than 128 columns and more than 128 rows
        use_graph = False
    # The fused path maps every rank's output matrices into every process.  With 18 GB of peer mappings (the Wan
    # workload on 8 GPUs: 7 peers x 2.6 GB) its stores ran at 96 GB/s per rank, 23.4 ms per step, where the NCCL
    # all-gather, which stages through small buffers, took 4.1 ms; with 1.8 GB (Flux, 8 GPUs) and 2.6 GB (Wan, 2 GPUs)
    # the fused path ran at 420-480 GB/s.  Large footprints therefore take the NCCL path.
    peer_bytes = (world - 1) * sum(M * n * 2 for _, _, n in wl["linears"])
    fused_declined = None
    if fused and peer_bytes > (4 << 30):
        fused = False
        use_graph = False
        fused_declined = f"{peer_bytes / 2**30:.1f} GiB of peer-mapped output matrices per rank: NCCL all-gather instead"
    if fused:
        peers = ckb.PeerGroup(dev)
        for lin in layers:
            lin.bind(peers, M)

    def step(one_call=one_call):
        # the linears of a step are independent work items: the all-gather of one overlaps the quantizer and GEMM
        # of the next (the collective runs on the process group's stream); all of them are awaited before the
        # step ends
        if fused:
            peers.barrier()                       # every rank is done with the previous step's matrices
            outs = [lin.fused(x) for x, lin in zip(xs, layers)]
            peers.barrier()                       # every rank's column blocks have arrived
            return outs
        outs, pending = [], []
        for x, lin in zip(xs, layers):
            y = lin.local(x, one_call=one_call)
            if not distributed:
                outs.append(y)
            elif equal_shards:
                work, buf = lin.gather_async(y)
                pending.append(work)
                outs.append(buf)
            else:
                outs.append(lin.gather(y, row_major=False))
        for work in pending:
            work.wait()
        return outs

    def barrier():
        if distributed:
            dist.barrier()
        torch.cuda.synchronize()

    def graphed(fn):
        """Capture fn once (after warm-up on the capture stream) and return (replay, launches per replay)."""
        if not use_graph:
            n0 = ckb.launches()
            fn()
            return fn, ckb.launches() - n0
        with torch.cuda.stream(side):
            for _ in range(3):
                fn()
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        n0 = ckb.launches()
        with torch.cuda.graph(g, stream=side):
            keep = fn()
        n = ckb.launches() - n0
        g._keep = keep
        graphs.append(g)
        return g.replay, n

    def timed(replay, reps):
        """reps back-to-back replays between two CUDA events on the current stream; returns ms in total."""
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        a.record()
        for _ in range(reps):
            replay()
        b.record()
        barrier()
        ms = a.elapsed_time(b)
        if distributed:
            t = torch.tensor([ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()

    warm = max(3, args.warmup)
    for _ in range(warm):
        step()
    barrier()
    assert ckb.read_device_status() == 0, "a bounded wait ran out during warm-up"

    # ---- the timed region: exactly K steps ----
    replay_step, launches_per_step = graphed(step)
    for _ in range(warm):
        replay_step()
    ms = timed(replay_step, args.steps)
    launches = launches_per_step * args.steps
    fl = flops_per_step(wl)
    value = fl * args.steps / (ms * 1e-3) / 1e12
    fused_linear = None
    if not distributed and not one_call and not args.no_sweep:
        # the same step with the quantizer inside the GEMM kernel (one kernel per linear), for comparison
        ckb.set_tuning(4, 1)
        replay_f, _ = graphed(lambda: step(one_call=True))
        for _ in range(warm):
            replay_f()
        ms_f = timed(replay_f, args.steps)
        ckb.set_tuning(4, 0)
        fused_linear = {"ms_per_step": ms_f / args.steps, "value": fl * args.steps / (ms_f * 1e-3) / 1e12,
                        "what": "ck_b200_linear_nvfp4 with the activation quantizer inside the GEMM kernel "
                                "(CK_B200_TUNE_LINEAR_FUSED), one CUDA graph per step"}

    # ---- per-kernel timing: the same K steps with only the GEMMs, then only the quantizers, back to back ----
    qw = [(l.qweight, l.weight_block_scale, l.weight_scale) for l in layers]
    qx_all = [ckb.quantize_nvfp4(x, t, pad_16x=pad_m) for x, t in zip(xs, ts_x)]

    def one_gemm(i):
        (q, sf), t, (w_q, w_sf, w_ts) = qx_all[i], ts_x[i], qw[i]
        return lambda: ckb.scaled_mm_nvfp4(q, w_q, t, w_ts, sf, w_sf)

    def one_quant(i):
        return lambda: ckb.quantize_nvfp4(xs[i], ts_x[i], pad_16x=pad_m)

    per_linear = []
    gemm_ms = quant_ms = gemm_fl = quant_bytes = 0.0
    for i, ((name, k, n), lin) in enumerate(zip(wl["linears"], layers)):
        rg, _ = graphed(one_gemm(i))
        rq, _ = graphed(one_quant(i))
        tg = timed(rg, args.steps) / args.steps
        tq = timed(rq, args.steps) / args.steps
        n_local = lin.local_rows
        per_linear.append({"linear": name, "K": k, "N_local": n_local, "quantize_us": tq * 1e3, "gemm_us": tg * 1e3,
                           "gemm_tflops": 2.0 * M * n_local * k / (tg * 1e-3) / 1e12,
                           "quantize_gbs": M * k * 2.5625 / (tq * 1e-3) / 1e9})
        gemm_ms += tg
        quant_ms += tq
        gemm_fl += 2.0 * M * n_local * k
        quant_bytes += M * k * 2.5625
    # quantizer alone, row-sharded (the "GB/s at 1/2/4/8 GPU" reading of the metric): every rank quantizes its own
    # M/G rows of each activation, no exchange; aggregate = all ranks' bytes over the slowest rank's time
    row_sharded = None
    if distributed:
        r0, r1 = (rank * (M // 16) // world) * 16, ((rank + 1) * (M // 16) // world) * 16 if rank + 1 < world else M
        t_rows = 0.0
        for i in range(len(layers)):
            x_rows = xs[i][r0:r1]
            rs, _ = graphed(lambda x_rows=x_rows, i=i: ckb.quantize_nvfp4(x_rows, ts_x[i], pad_16x=True))
            t_rows += timed(rs, args.steps) / args.steps
        row_sharded = {"aggregate_gbs": quant_bytes / (t_rows * 1e-3) / 1e9, "rows_per_rank": r1 - r0,
                       "us_per_step": t_rows * 1e3, "note": "weak in bytes per rank / strong in total: M rows split over the ranks"}
    peaks = measured_peaks()
    gemm_tflops = gemm_fl / (gemm_ms * 1e-3) / 1e12
    quant_gbs = quant_bytes / (quant_ms * 1e-3) / 1e9
    hbm_peak = peaks.get("hbm_gbs", 6650.0)
    roofline = {
        "kernel": "gemm_nvfp4_kernel", "bound": "tensor", "achieved": gemm_tflops, "peak": NOMINAL_NVFP4_TFLOPS,
        "unit": "TFLOP/s", "frac": gemm_tflops / NOMINAL_NVFP4_TFLOPS,
        # dram__bytes_read.sum + dram__bytes_write.sum per launch (mean of the four Flux launches) from the ncu capture
        # summarised in profiles/gemm_nvfp4_pair_kernel_flux.md; other workloads / shard sizes were not captured
        "traffic": 56.45e6 if (args.workload == "flux" and world == 1) else None,
        "peak_source": "nominal dense NVFP4 (vendor figure); MEASURED_PEAKS.json has no FP4 entry",
        "frac_of_4x_measured_bf16": (gemm_tflops / (4.0 * peaks["bf16_tflops"])) if "bf16_tflops" in peaks else None,
        "algorithmic_flops_per_launch": gemm_fl / len(layers), "avg_launch_us": gemm_ms * 1e3 / len(layers),
        "timing": "each linear's kernel replayed back to back K times between CUDA events (same-input repeats: operands "
                  "stay in L2, as they do inside a step where the quantizer has just written them)",
        "quantize": {"kernel": "quantize_nvfp4_flat_kernel (inputs of 20 MB to 0.25 GB) / quantize_nvfp4_kernel", "bound": "hbm", "achieved": quant_gbs, "peak": hbm_peak,
                     "unit": "GB/s", "frac": quant_gbs / hbm_peak,
                     "peak_source": "measured copy (MEASURED_PEAKS.json)" if "hbm_gbs" in peaks else "fallback",
                     "frac_of_nominal_8000": quant_gbs / 8000.0, "algorithmic_bytes_per_element": 2.5625,
                     "note": "activations of 28-113 MB: repeats of one input are partly L2 resident"},
        "per_linear": per_linear,
    }

    # ---- bandwidth sweep of the quantizer / dequantizer (shapes of the M x K bandwidth-sweep configuration), single-GPU runs only:
    # timed() synchronises all ranks, so every rank would have to run it ----
    sweep = None
    if not distributed and not args.no_sweep:
        sweep = []
        for (sm, sk) in [(1024, 3072), (4096, 5120), (16384, 3072), (16384, 12288), (65536, 5120), (65536, 12288)]:
            gx = torch.Generator(device=dev).manual_seed(sm + sk)
            xx = torch.randn((sm, sk), generator=gx, device=dev, dtype=torch.bfloat16)
            tt = ckb.dynamic_scale_nvfp4(xx)
            qq, ss = ckb.quantize_nvfp4(xx, tt)
            reps = 10
            r_q, _ = graphed(lambda: ckb.quantize_nvfp4(xx, tt))
            r_d, _ = graphed(lambda: ckb.dequantize_nvfp4(qq, tt, ss, torch.bfloat16))
            t_q = timed(r_q, reps) / reps
            t_d = timed(r_d, reps) / reps
            nbytes = sm * sk * 2.5625
            sweep.append({"M": sm, "K": sk, "quantize_us": t_q * 1e3, "quantize_gbs": nbytes / (t_q * 1e-3) / 1e9,
                          "dequantize_us": t_d * 1e3, "dequantize_gbs": nbytes / (t_d * 1e-3) / 1e9})
            del xx, qq, ss, r_q, r_d
            graphs.clear()
        torch.cuda.empty_cache()

    # ---- small-M sweep (T5-XXL-style feed-forward shapes, d = 4096, ff = 10240), single-GPU runs:
    # latency of one linear (quantize + GEMM, split-K below 129 rows) per M ----
    small_m = None
    if not distributed and not args.no_sweep:
        small_m = []
        gsm = torch.Generator(device=dev).manual_seed(5)
        for (sk, sn) in [(4096, 10240), (10240, 4096)]:
            ww = torch.randn((sn, sk), generator=gsm, device=dev, dtype=torch.bfloat16) * 0.02
            wts = ckb.dynamic_scale_nvfp4(ww)
            wq, wsf = ckb.quantize_nvfp4(ww, wts)
            for sm in (1, 16, 64, 512):
                xx = torch.randn((sm, sk), generator=gsm, device=dev, dtype=torch.bfloat16)
                tt = ckb.dynamic_scale_nvfp4(xx)
                qq, ss = ckb.quantize_nvfp4(xx, tt, pad_16x=True)
                def lin_call(xx=xx, tt=tt, wq=wq, wts=wts, wsf=wsf):
                    q1, s1 = ckb.quantize_nvfp4(xx, tt, pad_16x=True)
                    return ckb.scaled_mm_nvfp4(q1, wq, tt, wts, s1, wsf)
                r_l, _ = graphed(lin_call)
                r_g, _ = graphed(lambda: ckb.scaled_mm_nvfp4(qq, wq, tt, wts, ss, wsf))
                reps = 50
                t_l = timed(r_l, reps) / reps
                t_g = timed(r_g, reps) / reps
                small_m.append({"M": sm, "K": sk, "N": sn, "linear_us": t_l * 1e3, "gemm_us": t_g * 1e3,
                                "gemm_tflops": 2.0 * sm * sn * sk / (t_g * 1e-3) / 1e12,
                                "weight_gbs": sn * sk * 0.5625 / (t_g * 1e-3) / 1e9})
                del r_l, r_g
                graphs.clear()
            del ww, wq, wsf
        torch.cuda.empty_cache()

    # ---- the MXFP8 sibling path on the same workload (single-GPU runs): quantizer GB/s (3.03125 algorithmic bytes per
    # element: 2 in, 1 out, 1/32 scale) and GEMM TFLOP/s per linear, with cuBLASLt's MXFP8 kernel beside it ----
    mxfp8 = None
    if not distributed and not args.no_sweep:
        mx_lin, mq_ms, mg_ms, mc_ms, m_fl, m_bytes = [], 0.0, 0.0, 0.0, 0.0, 0.0
        for i, (name, k, n) in enumerate(wl["linears"]):
            wq8, wsf8 = ckb.quantize_mxfp8(ws_cpu[i].to(dev), pad_32x=True)
            xq8, xsf8 = ckb.quantize_mxfp8(xs[i], pad_32x=True)
            rq8, _ = graphed(lambda i=i: ckb.quantize_mxfp8(xs[i], pad_32x=True))
            rg8, _ = graphed(lambda xq8=xq8, wq8=wq8, xsf8=xsf8, wsf8=wsf8: ckb.scaled_mm_mxfp8(xq8, wq8, xsf8, wsf8))
            tq8 = timed(rq8, args.steps) / args.steps
            tg8 = timed(rg8, args.steps) / args.steps
            entry = {"linear": name, "quantize_us": tq8 * 1e3, "quantize_gbs": M * k * 3.03125 / (tq8 * 1e-3) / 1e9,
                     "gemm_us": tg8 * 1e3, "gemm_tflops": 2.0 * M * n * k / (tg8 * 1e-3) / 1e12}
            try:
                from torch.nn.functional import ScalingType, SwizzleType, scaled_mm

                def lt(xq8=xq8, wq8=wq8, xsf8=xsf8, wsf8=wsf8):
                    return scaled_mm(xq8, wq8.t(), scale_a=xsf8.view(-1), scale_b=wsf8.view(-1),
                                     scale_recipe_a=ScalingType.BlockWise1x32, scale_recipe_b=ScalingType.BlockWise1x32,
                                     swizzle_a=SwizzleType.SWIZZLE_32_4_4, swizzle_b=SwizzleType.SWIZZLE_32_4_4,
                                     output_dtype=torch.bfloat16)
                rc8, _ = graphed(lt)
                tc8 = timed(rc8, args.steps) / args.steps
                entry["cublaslt_gemm_tflops"] = 2.0 * M * n * k / (tc8 * 1e-3) / 1e12
                mc_ms += tc8
            except Exception as ex:   # depends on the torch / cuBLASLt build
                entry["cublaslt_unavailable"] = f"{type(ex).__name__}: {ex}"[:160]
            mx_lin.append(entry)
            mq_ms += tq8
            mg_ms += tg8
            m_fl += 2.0 * M * n * k
            m_bytes += M * k * 3.03125
            del wq8, wsf8, xq8, xsf8
            graphs.clear()
        mxfp8 = {"gemm_tflops": m_fl / (mg_ms * 1e-3) / 1e12, "quantize_gbs": m_bytes / (mq_ms * 1e-3) / 1e9,
                 "cublaslt_gemm_tflops": (m_fl / (mc_ms * 1e-3) / 1e12) if mc_ms > 0 else None,
                 "nominal_dense_fp8_tflops": 4500.0, "per_linear": mx_lin,
                 "kernel": "gemm_nvfp4_kernel<BN, FMT = 1> (1-CTA tiles, tcgen05 kind::mxf8f6f4.block_scale)"}
        torch.cuda.empty_cache()

    # ---- cuBLASLt NVFP4 through torch on the same operands: the kernel behind the reference eager backend ----
    try:
        from torch.nn.functional import ScalingType, SwizzleType, scaled_mm
        tot = 0.0
        for i in range(len(layers)):
            (q, sf), t, (w_q, w_sf, w_ts) = qx_all[i], ts_x[i], qw[i]

            def call(q=q, sf=sf, t=t, w_q=w_q, w_sf=w_sf, w_ts=w_ts):
                return scaled_mm(q.view(torch.float4_e2m1fn_x2), w_q.view(torch.float4_e2m1fn_x2).t(),
                                 scale_a=[sf.view(-1), t.reshape(())], scale_b=[w_sf.view(-1), w_ts.reshape(())],
                                 scale_recipe_a=[ScalingType.BlockWise1x16, ScalingType.TensorWise],
                                 scale_recipe_b=[ScalingType.BlockWise1x16, ScalingType.TensorWise],
                                 swizzle_a=[SwizzleType.SWIZZLE_32_4_4, SwizzleType.NO_SWIZZLE],
                                 swizzle_b=[SwizzleType.SWIZZLE_32_4_4, SwizzleType.NO_SWIZZLE],
                                 output_dtype=torch.bfloat16)
            rc, _ = graphed(call)
            tot += timed(rc, args.steps) / args.steps
        cublaslt = {"gemm_tflops": gemm_fl / (tot * 1e-3) / 1e12,
                    "what": "torch.nn.functional.scaled_mm (cuBLASLt NVFP4), same operands, GEMM only, timed like ours"}
    except Exception as ex:   # depends on the torch / cuBLASLt build
        cublaslt = {"unavailable": f"{type(ex).__name__}: {ex}"[:200]}

    # ---- end to end: pinned host activations in, host outputs back, copies inside the timed region ----
    x_host = [x.pin_memory() for x in xs_cpu]
    y_host = [torch.empty((M, lin.local_rows), dtype=torch.bfloat16).pin_memory() for lin in layers]
    h2d = sum(x.numel() * 2 for x in x_host)
    d2h = sum(y.numel() * 2 for y in y_host)

    # Three streams: uploads, the operators (the current stream), downloads.  PCIe carries both directions at once and
    # the GPU has separate copy engines for them, so linear i's output goes back while linear i+1's activations come
    # in, also across step boundaries; events order upload -> operators -> download per linear.  Each linear has
    # its own device input buffer, reused every step once the operators of the previous step have read it.
    s_in, s_out = torch.cuda.Stream(), torch.cuda.Stream()
    x_dev = [torch.empty_like(x) for x in xs]
    ev_in = [torch.cuda.Event() for _ in layers]
    ev_cmp = [torch.cuda.Event() for _ in layers]
    ev_out = [torch.cuda.Event() for _ in layers]
    serial = args.e2e_serial

    def e2e_step():
        cur = torch.cuda.current_stream()
        for i, (xh, yh, lin) in enumerate(zip(x_host, y_host, layers)):
            s_in.wait_event(ev_cmp[i])                     # last step's operators are done with x_dev[i]
            if serial:
                s_in.wait_stream(s_out)
            with torch.cuda.stream(s_in):
                x_dev[i].copy_(xh, non_blocking=True)
                ev_in[i].record()
            cur.wait_event(ev_in[i])
            if fused:
                cur.wait_event(ev_out[i])                  # last step's download has read this rank's matrix
                peers.barrier()
                y = lin.fused(x_dev[i])
                peers.barrier()
                y = y[:, lin.n0:lin.n1]
            else:
                y = lin.local(x_dev[i])
                if distributed:
                    y = lin.gather(y, row_major=False)[rank]
            ev_cmp[i].record()
            s_out.wait_event(ev_cmp[i])
            with torch.cuda.stream(s_out):
                yh.copy_(y, non_blocking=True)
                ev_out[i].record()
            y.record_stream(s_out)
            if serial:
                cur.wait_stream(s_out)
        cur.wait_stream(s_out)                             # the closing event of the timed region covers the downloads

    for _ in range(2):
        e2e_step()
    ems = timed(e2e_step, args.steps)
    e2e = {"value": fl * args.steps / (ems * 1e-3) / 1e12, "unit": "TFLOP/s", "h2d_bytes_per_step": h2d,
           "d2h_bytes_per_step": d2h, "ms_per_step": ems / args.steps,
           "pcie_gbs": {"h2d": h2d / (ems / args.steps * 1e-3) / 1e9, "d2h": d2h / (ems / args.steps * 1e-3) / 1e9},
           "what": "pinned host bf16 activations -> device, quantize_nvfp4 + scaled_mm_nvfp4 through the operator "
                   "interface, bf16 outputs -> pinned host; per rank; "
                   + ("one transfer at a time" if serial else
                      "uploads, operators and downloads on three streams, so the two PCIe directions overlap")}
    if args.gemm_debug and rank == 0:
        # one launch per linear of the kernel build with cycle counters: CTA pair 0 prints (device printf, on stdout
        # before the JSON line) the cycles and nanoseconds its roles took and how long they waited
        ckb.set_tuning(2, 1)
        for i in range(len(layers)):
            one_gemm(i)()
            torch.cuda.synchronize()
        ckb.set_tuning(2, 0)
    status = ckb.read_device_status()
    clocks = sampler.stop() if rank == 0 else {}

    # ---- CPU baseline on a bounded sample (rank 0, single-GPU run only) ----
    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        xs_bits, w_q, threads = prepare_cpu(wl, xs_cpu, ws_cpu)
        rows = min(1152, M)
        cpu_reference_step(wl, xs_bits, w_q, rows)
        t0 = time.perf_counter()
        reps, cfl = 0, 0.0
        while reps < 2 or (time.perf_counter() - t0 < 12.0 and reps < 200):
            cfl += cpu_reference_step(wl, xs_bits, w_q, rows)
            reps += 1
        dt = time.perf_counter() - t0
        cpu = {"value": cfl / dt / 1e12, "unit": "TFLOP/s", "cores": threads, "kind": "port",
               "sample": f"first {rows} of {M} tokens of each linear, {reps} repetitions, {dt:.1f} s of CPU work"}

    if rank == 0:
        line = {
            "metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
            "warmup": warm, "ms_per_step": ms / args.steps, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "nvfp4 (e2m1 x e4m3 block scales), fp32 accumulate",
            "data": "synthetic",
            "config": {"workload": wl["name"], "M": M, "linears": wl["linears"],
                       "parallelism": f"weights N-sharded over {world} GPU(s)" + ((", all-gather of bf16 outputs fused into the GEMM epilogue (stores to peer memory over NVLink), "
                                         "barrier kernel before and after the step") if fused else
                                        ", NCCL all-gather of bf16 outputs (overlapping the next linear)"
                                        + (f" [{fused_declined}]" if fused_declined else "") if distributed else ""),
                       "launch": "one CUDA graph per step" if use_graph else "eager launches",
                       "linear": ("one kernel per linear: the GEMM kernel quantizes the activations beside its main loop "
                                  "(ck_b200_linear_nvfp4)") if one_call and not distributed else
                                 "quantize_nvfp4 kernel, then scaled_mm_nvfp4 kernel",
                       "l2": "no flush: one step touches ~0.6 GB (activations, packed operands, outputs), 5x the 126 MB L2"},
            "roofline": roofline, "cpu_baseline": cpu, "e2e": e2e, "gpu_launches": launches, "clocks": clocks,
            "cublaslt_comparator": cublaslt, "device_status": status,
            "quantize_gbs": quant_gbs, "quantize_row_sharded": row_sharded, "gemm_only_tflops": gemm_tflops,
            "quantize_sweep": sweep, "small_m_sweep": small_m, "mxfp8": mxfp8, "fused_linear": fused_linear,
        }
        if fused:
            # bytes this rank's GEMM epilogues push to the other ranks per step, against the measured peer-copy rate
            out_bytes = sum(M * lin.local_rows * 2 for lin in layers) * (world - 1)
            line["nvlink"] = {"bytes_out_per_rank_per_step": out_bytes,
                              "achieved_gbs": out_bytes / (ms / args.steps * 1e-3) / 1e9, "peak_gbs": 770.0,
                              "peak_source": "measured peer copy per direction on this pool",
                              "note": "whole step in the denominator, quantizer kernels (no traffic) included"}
        print(json.dumps(line), flush=True)
    if peers is not None:
        peers.close()
    if distributed:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="flux", choices=sorted(WORKLOADS))
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-sweep", action="store_true", help="skip the quantizer bandwidth sweep")
    ap.add_argument("--no-dependent-launch", action="store_true",
                    help="launch kernels fully serialised instead of with programmatic stream serialisation")
    ap.add_argument("--dependent-launch-mask", type=int, default=None,
                    help="which kernels get the programmatic-serialisation attribute: 1 GEMMs, 2 quantizers, 3 both")
    ap.add_argument("--collective", default="fused", choices=["fused", "nccl"],
                    help="N > 1: all-gather fused into the GEMM epilogue over peer memory, or a NCCL all-gather after it")
    ap.add_argument("--gemm-debug", action="store_true",
                    help="also launch each linear's GEMM once with in-kernel cycle counters (prints extra lines)")
    ap.add_argument("--fused-linear", action="store_true",
                    help="step = one kernel per linear (the GEMM kernel quantizes the activations) instead of "
                         "quantize_nvfp4 and scaled_mm_nvfp4 as two kernels")
    ap.add_argument("--e2e-serial", action="store_true",
                    help="end-to-end arm: one host<->device transfer at a time instead of overlapping the two directions")
    ap.add_argument("--no-graph", action="store_true", help="launch every kernel eagerly instead of one CUDA graph per step")
    args = ap.parse_args()
    wl = WORKLOADS[args.workload]
    if args.impl == "reference":
        run_reference_arm(args, wl)
    else:
        run_ours(args, wl)


if __name__ == "__main__":
    main()
