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
bounded sample of the same workload on this box's host cores.  Beside them: `parity` (the results of the timed
path checked inside this run), `sustained` (the step replayed for seconds, with the clocks seen), `fp4_ceiling`
(cuBLASLt's NVFP4 kernel on 8192^3 and 16384^3, the measured ceiling the GEMM fractions are also given against),
`wan` (a short record of the Wan-class workload, the one whose weights are sharded over the GPUs), the quantizer
sweep (L2-cold and L2-warm), comparators for the quantizer, and the small-M and MXFP8 records.

With --gpus N > 1 (launched under torchrun, one rank per GPU) every weight is sharded along N, each rank
multiplies its shard and the bf16 column blocks are all-gathered: total work is fixed ("strong").
`--impl reference` times the CPU restatement of the reference eager path (the oracle) as the reference arm.
"""
from __future__ import annotations

import argparse
import ctypes
import json
import os
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

FLUX = {"name": "flux_dit_block_linears", "M": 4608,
        "linears": [("qkv", 3072, 9216), ("attn_out", 3072, 3072), ("mlp_up", 3072, 12288), ("mlp_down", 12288, 3072)]}
WAN = {"name": "wan14b_dit_block_linears", "M": 32760,
       "linears": [("qkv", 5120, 15360), ("attn_out", 5120, 5120), ("ffn_up", 5120, 13824), ("ffn_down", 13824, 5120)]}
WORKLOADS = {"flux": FLUX, "wan": WAN}
NOMINAL_NVFP4_TFLOPS = 9000.0   # vendor dense NVFP4 figure for B200
METRIC = "scaled_mm_nvfp4 TFLOPS over the NVFP4 linear path (quantize_nvfp4 + scaled_mm_nvfp4 per linear)"
DTYPE = "nvfp4 (e2m1 x e4m3 block scales), fp32 accumulate"
SWEEP_SHAPES = [(m, k) for m in (1024, 4096, 16384, 65536) for k in (3072, 5120, 12288)]
L2_BYTES = 126 << 20
CPU_SAMPLE_ROWS = 1152


def flops_per_step(wl) -> float:
    return sum(2.0 * wl["M"] * n * k for _, k, n in wl["linears"])


def workload_config(wl) -> dict:
    """The `config` of the JSON line: what is computed, identical in both arms."""
    return {"workload": wl["name"], "M": wl["M"], "linears": [list(l) for l in wl["linears"]],
            "input_scale": "static per-tensor activation scales (amax/(448*6) of each activation, computed once "
                           "before the timed region, like the input_scale of an NVFP4 checkpoint)",
            "l2": "no flush: one step touches ~0.6 GB (activations, packed operands, outputs), 5x the 126 MB L2"}


def make_inputs(wl, dtype):
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


def make_inputs_on_device(wl, dev, dtype):
    """The same distributions from a seeded generator of the device (identical on every rank: same GPU model, same
    seed); used for the Wan-class record, whose 0.9 GB activations would take the host tens of seconds."""
    import torch
    xs, ws = [], []
    for i, (_, k, n) in enumerate(wl["linears"]):
        g = torch.Generator(device=dev).manual_seed(2000 + i)
        x = torch.randn((wl["M"], k), generator=g, device=dev, dtype=torch.float32)
        cols = torch.randperm(k, generator=g, device=dev)[: max(1, round(k / 1000))]
        x[:, cols] *= 20.0
        xs.append(x.to(dtype))
        del x
        w = torch.randn((n, k), generator=g, device=dev, dtype=torch.float32) * 0.02
        ws.append(w.to(dtype))
        del w
    return xs, ws


class ClockSampler:
    """SM clock and throttle-reason samples taken through NVML (read-only) by a thread while the GPU is under load."""

    def __init__(self, gpu_index: int, period_s: float = 0.002):
        self.gpu_index = gpu_index
        self.period_s = period_s
        self.samples = []
        self.power = []
        self.reasons = 0
        self.max_mhz = None
        self._stop = False
        self._thread = None
        self._nvml = None

    def start(self):
        try:
            import threading

            import pynvml
            import torch
            pynvml.nvmlInit()
            # torch's device ordinal follows CUDA_VISIBLE_DEVICES; map it to the NVML handle through the PCI bus id
            props = torch.cuda.get_device_properties(self.gpu_index)
            bus = props.pci_bus_id if hasattr(props, "pci_bus_id") else None
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
                        self.power.append(pynvml.nvmlDeviceGetPowerUsage(handle) / 1000.0)
                    except Exception:
                        pass
                    time.sleep(self.period_s)

            self._thread = threading.Thread(target=loop, daemon=True)
            self._thread.start()
        except Exception:
            self._thread = None
        return self

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
        if self.power:
            pw = sorted(self.power)
            out.update(power_w_median=pw[len(pw) // 2], power_w_max=pw[-1])
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
    threads = o.use_all_cores()    # explicit: a launcher's OMP_NUM_THREADS=1 must not shrink the baseline
    xs_bits, w_q = [], []
    for x, w in zip(xs, ws):
        xb = x.view(torch.int16).numpy().view(np.uint16)
        wb = w.view(torch.int16).numpy().view(np.uint16)
        ts_x = float(x.abs().amax().float() / 2688.0)
        ts_w = float(w.abs().amax().float() / 2688.0)
        qw, sfw = o.quantize_nvfp4(wb, o.BF16, ts_w)
        xs_bits.append((xb, ts_x))
        w_q.append((qw, sfw, ts_w))
    return xs_bits, w_q, threads


def cpu_sample_text(wl, rows):
    return f"first {rows} of {wl['M']} tokens of each of the {len(wl['linears'])} linears per step"


def run_reference_arm(args, wl):
    import torch
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    torch.manual_seed(0)
    xs, ws = make_inputs(wl, torch.bfloat16)
    xs_bits, w_q, threads = prepare_cpu(wl, xs, ws)
    rows = min(CPU_SAMPLE_ROWS, wl["M"])
    for _ in range(max(1, args.warmup)):
        cpu_reference_step(wl, xs_bits, w_q, rows)
    t0 = time.perf_counter()
    fl = 0.0
    for _ in range(args.steps):
        fl += cpu_reference_step(wl, xs_bits, w_q, rows)
    dt = time.perf_counter() - t0
    val = fl / dt / 1e12
    sample = cpu_sample_text(wl, rows)
    line = {
        "impl": "reference", "metric": METRIC, "value": val, "unit": "TFLOP/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt / args.steps * 1e3, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": DTYPE, "data": "synthetic", "config": workload_config(wl),
        "cpu_baseline": {"value": val, "unit": "TFLOP/s", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": val, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
        "run": {"sample": sample, "threads": threads, "omp_num_threads_env": os.environ.get("OMP_NUM_THREADS")},
        "note": "CPU restatement of the reference eager path (quantize_nvfp4 eager; scaled_mm_nvfp4 = dequantize to "
                "fp32 + fp32 BLAS matmul, the check the reference's own tests use since its eager GEMM has no CPU kernel)",
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------------ GPU arm


class Bench:
    """Device, ranks and the timing helpers shared by every record of the GPU arm."""

    def __init__(self, args):
        import torch
        import torch.distributed as dist
        self.torch, self.dist, self.args = torch, dist, args
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.rank = int(os.environ.get("RANK", "0"))
        self.local_rank = int(os.environ.get("LOCAL_RANK", "0"))
        if not torch.cuda.is_available():
            raise SystemExit("bench.py needs a CUDA device: comfy_kitchen_b200 has no CPU path")
        torch.cuda.set_device(self.local_rank)
        self.dev = torch.device("cuda", self.local_rank)
        self.distributed = self.world > 1
        if self.distributed:
            os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
            dist.init_process_group("nccl", device_id=self.dev)
        self.side = torch.cuda.Stream()       # capture stream
        self.side2 = torch.cuda.Stream()      # second branch of a captured step (the quantizers)
        self.side3 = torch.cuda.Stream()      # third branch (several GPUs: every other GEMM)
        self.graphs = []
        self.use_graph = not args.no_graph

    def barrier(self):
        if self.distributed:
            self.dist.barrier()
        self.torch.cuda.synchronize()

    def graphed(self, fn, use_graph=None):
        """Capture fn once (after warm-up on the capture stream) and return (replay, launches per replay)."""
        import comfy_kitchen_b200 as ckb
        torch = self.torch
        if not (self.use_graph if use_graph is None else use_graph):
            n0 = ckb.launches()
            fn()
            return fn, ckb.launches() - n0
        with torch.cuda.stream(self.side):
            for _ in range(3):
                fn()
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        n0 = ckb.launches()
        with torch.cuda.graph(g, stream=self.side):
            keep = fn()
        n = ckb.launches() - n0
        g._keep = keep
        self.graphs.append(g)
        return g.replay, n

    def timed(self, replay, reps, all_ranks=True):
        """reps back-to-back replays between two CUDA events on the current stream; returns ms in total (the maximum
        over the ranks when every rank takes part)."""
        torch = self.torch
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        if all_ranks:
            self.barrier()
        else:
            torch.cuda.synchronize()
        a.record()
        for _ in range(reps):
            replay()
        b.record()
        if all_ranks:
            self.barrier()
        else:
            torch.cuda.synchronize()
        ms = a.elapsed_time(b)
        if self.distributed and all_ranks:
            t = torch.tensor([ms], device=self.dev)
            self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms

    def for_seconds(self, replay, seconds, chunk):
        """Replays in chunks until `seconds` have passed; returns (ms in total, replays), single-rank helper."""
        torch = self.torch
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        a.record()
        n = 0
        while True:
            for _ in range(chunk):
                replay()
            n += chunk
            torch.cuda.synchronize()
            if time.perf_counter() - t0 >= seconds:
                break
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b), n


def cublaslt_nvfp4(torch, q, sf, t, w_q, w_sf, w_ts):
    """cuBLASLt NVFP4 through torch on the same operands: the kernel behind the reference eager backend
    (comfy_kitchen/backends/eager/quantization.py:225-249)."""
    from torch.nn.functional import ScalingType, SwizzleType, scaled_mm
    return scaled_mm(q.view(torch.float4_e2m1fn_x2), w_q.view(torch.float4_e2m1fn_x2).t(),
                     scale_a=[sf.view(-1), t.reshape(())], scale_b=[w_sf.view(-1), w_ts.reshape(())],
                     scale_recipe_a=[ScalingType.BlockWise1x16, ScalingType.TensorWise],
                     scale_recipe_b=[ScalingType.BlockWise1x16, ScalingType.TensorWise],
                     swizzle_a=[SwizzleType.SWIZZLE_32_4_4, SwizzleType.NO_SWIZZLE],
                     swizzle_b=[SwizzleType.SWIZZLE_32_4_4, SwizzleType.NO_SWIZZLE],
                     output_dtype=torch.bfloat16)


def rel_rms(y, ref) -> float:
    y, ref = y.double(), ref.double()
    return float((y - ref).pow(2).mean().sqrt() / ref.pow(2).mean().sqrt().clamp_min(1e-30))


class StepPlan:
    """The layers of one workload on this rank and the ways a step over them can be enqueued."""

    def __init__(self, B: Bench, wl, xs, ws, collective: str):
        import comfy_kitchen_b200 as ckb
        torch = B.torch
        self.B, self.wl, self.ckb = B, wl, ckb
        self.M = wl["M"]
        self.xs = xs
        # static per-tensor activation scales (the optional `input_scale` of an NVFP4 checkpoint), amax/(448*6)
        self.ts_x = [ckb.dynamic_scale_nvfp4(x) for x in xs]
        self.layers = [ckb.ShardedNVFP4Linear(w.to(B.dev), None, input_scale=t) for w, t in zip(ws, self.ts_x)]
        torch.cuda.synchronize()
        world, M = B.world, self.M
        self.equal_shards = all(n % (8 * world) == 0 for _, _, n in wl["linears"])
        self.fused = B.distributed and collective == "fused"
        self.declined = None
        if self.fused and not (self.equal_shards and M > 128 and all(n // world > 128 for _, _, n in wl["linears"])):
            self.fused = False
            self.declined = "the fused kernel wants equal shards wider than 128 columns and more than 128 rows"
        # The fused path maps every rank's output matrices into every process, and the library bounds those mappings
        # (PeerGroup.map_limit_bytes: with 16.8 GiB mapped - the Wan workload on 8 GPUs - the stores ran at 202 GB/s per
        # rank, with up to 7.7 GiB at 470-580).  A workload is taken fused as a whole or not at all, and the line says so.
        self.peers = None
        if self.fused:
            self.peers = ckb.PeerGroup(B.dev, map_limit_bytes=B.args.peer_map_limit_gib << 30)
            per_rank = sum(M * n * 2 for _, _, n in wl["linears"])
            if not self.peers.fits(per_rank):
                self.fused = False
                self.declined = (f"{(world - 1) * per_rank / 2**30:.1f} GiB of peer-mapped output matrices per rank is above "
                                 f"the library's limit of {B.args.peer_map_limit_gib} GiB: NCCL all-gather instead")
                self.peers.close()
                self.peers = None
        self.use_graph = B.use_graph and (not B.distributed or self.fused)
        self.half_pairs = max(1, int(ckb._lib.load().ck_b200_query(ckb._lib.QUERY_SM_COUNT)) // 4)   # half of the CTA pairs
        if self.fused:
            for lin in self.layers:
                lin.bind(self.peers, M)

    def close(self):
        if self.peers is not None:
            self.peers.close()
            self.peers = None

    def mode_text(self):
        B = self.B
        if not B.distributed:
            return "1 GPU"
        if self.fused:
            return (f"weights N-sharded over {B.world} GPUs, all-gather of bf16 outputs fused into the GEMM epilogue "
                    "(stores to peer memory over NVLink), barrier kernel before and after the step")
        return (f"weights N-sharded over {B.world} GPUs, NCCL all-gather of bf16 outputs (overlapping the next linear)"
                + (f" [{self.declined}]" if self.declined else ""))

    def step(self, one_call=False, dynamic=False):
        """The linears one after the other on the current stream."""
        B, layers, xs = self.B, self.layers, self.xs
        if dynamic:      # per-call activation scale (the layer's default when a checkpoint has no input_scale)
            saved = [l.input_scale for l in layers]
            for l in layers:
                l.input_scale = None
        try:
            if self.fused:
                self.peers.barrier()                       # every rank is done with the previous step's matrices
                outs = [lin.fused(x) for x, lin in zip(xs, layers)]
                self.peers.barrier()                       # every rank's column blocks have arrived
                return outs
            outs, pending = [], []
            for x, lin in zip(xs, layers):
                y = lin.local(x, one_call=one_call)
                if not B.distributed:
                    outs.append(y)
                elif self.equal_shards:
                    work, buf = lin.gather_async(y)
                    pending.append(work)
                    outs.append(buf)
                else:
                    outs.append(lin.gather(y, row_major=False))
            for work in pending:
                work.wait()
            return outs
        finally:
            if dynamic:
                for l, s in zip(layers, saved):
                    l.input_scale = s

    def step_overlapped(self):
        """The same work as several branches of one CUDA graph.  The quantizers run on a second stream, so the quantizer
        of linear i+1 overlaps the GEMM of linear i.  On several GPUs the GEMMs themselves alternate between two
        streams, each kernel on half of the CTA pairs (CK_B200_TUNE_GEMM_MAX_PAIRS): those kernels are bound by the
        link, not by the tensor cores, and side by side one kernel's stores fill the link while the other ramps up
        or drains.  Legitimate because the four linears of the step are independent work items; inside a real block,
        where each linear's input depends on the previous output, only the serial step applies."""
        torch, ckb = self.B.torch, self.ckb
        cur, qs, g1 = torch.cuda.current_stream(), self.B.side2, self.B.side3
        qs.wait_stream(cur)
        quant, events = [], []
        with torch.cuda.stream(qs):
            for x, lin in zip(self.xs, self.layers):
                quant.append(lin.quantize_input(x))
                e = torch.cuda.Event()
                e.record(qs)
                events.append(e)
        if self.fused:
            self.peers.barrier()
        two = self.fused and self.B.args.gemm_streams == 2
        if two:
            g1.wait_stream(cur)                 # after the opening barrier
            prev_cap = ckb.set_tuning(9, self.half_pairs)
        outs = []
        try:
            for i, ((qx, sfx, t), lin, e) in enumerate(zip(quant, self.layers, events)):
                stream = g1 if (two and i % 2 == 1) else cur
                stream.wait_event(e)
                with torch.cuda.stream(stream):
                    outs.append(lin.fused_from_quantized(qx, sfx, t, self.M) if self.fused
                                else lin.local_from_quantized(qx, sfx, t, self.M))
        finally:
            if two:
                ckb.set_tuning(9, prev_cap)
        if two:
            cur.wait_stream(g1)
        cur.wait_stream(qs)
        if self.fused:
            self.peers.barrier()
        return outs, quant

    def check_parity(self):
        """The results of the path that is timed, checked inside this run.  Several GPUs: every rank's fused matrix
        against the NCCL all-gather of the same column blocks, bit for bit, on every rank.  One GPU: each linear
        against cuBLASLt's NVFP4 kernel on the same quantized operands (relative RMS error, tolerance 1e-2)."""
        B, torch, ckb = self.B, self.B.torch, self.ckb
        out = {}
        if self.fused:
            self.peers.barrier()
            fused_out = [lin.fused(x) for x, lin in zip(self.xs, self.layers)]
            self.peers.barrier()
            torch.cuda.synchronize()
            ok = 1
            for (name, _, _), x, lin, got in zip(self.wl["linears"], self.xs, self.layers, fused_out):
                want = lin.gather(lin.local(x))          # NCCL all-gather, row-major [M, N]; own memory only
                if not torch.equal(got, want):
                    ok = 0
                    nl = lin.local_rows
                    per_block = [int((got[:, r * nl:(r + 1) * nl] != want[:, r * nl:(r + 1) * nl]).sum()) for r in range(B.world)]
                    bad_rows = (got != want).any(dim=1).nonzero().flatten()
                    print(f"[parity] rank {B.rank} linear {name}: differing elements per rank's column block {per_block}, "
                          f"{bad_rows.numel()} rows affected, first {bad_rows[:8].tolist()} last {bad_rows[-4:].tolist()}",
                          file=sys.stderr, flush=True)
            flag = torch.tensor([ok], device=B.dev)
            B.dist.all_reduce(flag, op=B.dist.ReduceOp.MIN)
            all_ok = int(flag.item()) == 1
            out = {"multi_gpu": "bit-equal to NCCL all-gather" if all_ok else "MISMATCH against NCCL all-gather",
                   "ranks": B.world, "linears_checked": len(self.layers), "ok": all_ok}
        elif not B.distributed:
            errs = {}
            try:
                for (name, _, _), x, lin, t in zip(self.wl["linears"], self.xs, self.layers, self.ts_x):
                    qx, sfx, _ = lin.quantize_input(x)
                    y = lin.local_from_quantized(qx, sfx, t, self.M)
                    ref = cublaslt_nvfp4(torch, qx, sfx, t, lin.qweight, lin.weight_block_scale, lin.weight_scale)
                    errs[name] = rel_rms(y.float(), ref[: self.M].float())
                    del y, ref
                out = {"gemm_rel_rms_vs_cublaslt": errs, "tolerance": 1e-2, "ok": max(errs.values()) <= 1e-2}
            except Exception as ex:   # depends on the torch / cuBLASLt build
                out = {"gemm_rel_rms_vs_cublaslt": None, "unavailable": f"{type(ex).__name__}: {ex}"[:160], "ok": True}
        else:
            out = {"multi_gpu": "NCCL all-gather path (library collective): nothing fused to check", "ranks": B.world,
                   "ok": True}
        return out


def reference_package():
    """The copy of the reference's Python package under baseline/_ref (comparators only), or None."""
    ref = os.path.join(ROOT, "baseline", "_ref")
    if not os.path.isdir(os.path.join(ref, "comfy_kitchen")):
        return None
    if ref not in sys.path:
        sys.path.insert(0, ref)
    sys.dont_write_bytecode = True
    try:
        import comfy_kitchen as ck
        return ck
    except Exception:
        return None


def quantize_comparators(B: Bench, xs, ts_x, names):
    """The reference's own GPU quantizers on the activations of the step, beside this library's: its Triton kernel
    (comfy_kitchen/backends/triton/quantization.py:333-415, run from the copy of the reference's Python package) and
    its CUDA kernel (comfy_kitchen/backends/cuda/ops/quantize_nvfp4.cu:323-384, compiled by itself), each with GB/s
    (2.5625 algorithmic bytes per element) and the number of output bytes that differ from the reference eager
    backend on the same tensor.  Eager is the contract; this library's count is zero."""
    import comfy_kitchen_b200 as ckb
    torch = B.torch
    ck = reference_package()
    if ck is None:
        return {"unavailable": "baseline/_ref/comfy_kitchen is absent (baseline/make_ref.py makes it)"}
    out = {"algorithmic_bytes_per_element": 2.5625, "shapes": []}
    lib_path = os.path.join(ROOT, "baseline", "_ref", "libref_quantize_nvfp4.so")
    ref_cuda = None
    if os.path.exists(lib_path):
        try:
            L = ctypes.CDLL(lib_path)
            vp, i64 = ctypes.c_void_p, ctypes.c_int64
            L.launch_quantize_nvfp4_kernel.argtypes = [vp, vp, vp, vp, i64, i64, i64, i64, ctypes.c_float, ctypes.c_int,
                                                       ctypes.c_bool, vp]
            L.launch_quantize_nvfp4_kernel.restype = None

            def ref_cuda(x, t):
                # what the reference's host wrapper does per call (comfy_kitchen/backends/cuda/__init__.py:582-667):
                # a zero-filled scale tensor (its kernel leaves the padding unwritten), then the launch
                m, k = x.shape
                q = torch.empty((m, k // 2), dtype=torch.uint8, device=x.device)
                sf = torch.zeros(((m + 127) // 128 * 128, (k // 16 + 3) // 4 * 4), dtype=torch.uint8, device=x.device)
                L.launch_quantize_nvfp4_kernel(x.data_ptr(), t.data_ptr(), q.data_ptr(), sf.data_ptr(), m, k, m, k, 0.0, 2,
                                               True, ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
                return q, sf
        except Exception as ex:
            out["reference_cuda_unavailable"] = f"{type(ex).__name__}: {ex}"[:160]
    triton_q = None
    try:
        from comfy_kitchen.backends.triton.quantization import quantize_nvfp4 as triton_q
    except Exception as ex:
        out["reference_triton_unavailable"] = f"{type(ex).__name__}: {ex}"[:160]
    seen = set()
    for name, x, t in zip(names, xs, ts_x):
        if tuple(x.shape) in seen or x.shape[0] % 16:
            continue
        seen.add(tuple(x.shape))
        nbytes = x.numel() * 2.5625
        with ck.use_backend("eager"):
            q_e, sf_e = ck.quantize_nvfp4(x, t.reshape(()))
        sf_e = sf_e.view(torch.uint8)
        entry = {"activation": name, "M": x.shape[0], "K": x.shape[1]}
        impls = {"ours": lambda x=x, t=t: ckb.quantize_nvfp4(x, t)}
        if ref_cuda is not None:
            impls["reference_cuda"] = lambda x=x, t=t: ref_cuda(x, t.reshape(1))
        if triton_q is not None:
            impls["reference_triton"] = lambda x=x, t=t: triton_q(x, t.reshape(()))
        for key, fn in impls.items():
            try:
                q, sf = fn()
                torch.cuda.synchronize()
                diff_q = int((q != q_e).sum())
                diff_sf = int((sf.view(torch.uint8) != sf_e).sum())
                replay, _ = B.graphed(fn)
                ms = B.timed(replay, 20, all_ranks=False) / 20
                entry[key] = {"us": ms * 1e3, "gbs": nbytes / (ms * 1e-3) / 1e9, "packed_bytes_differing_from_eager": diff_q,
                              "scale_bytes_differing_from_eager": diff_sf, "of_packed_bytes": q.numel()}
            except Exception as ex:
                entry[key] = {"unavailable": f"{type(ex).__name__}: {ex}"[:200]}
            B.graphs.clear()
        out["shapes"].append(entry)
    return out


def fp4_ceiling(B: Bench):
    """cuBLASLt's NVFP4 kernel (through torch) on 8192^3 and 16384^3, the measured ceiling for a block-scaled FP4 GEMM on
    this GPU: best of 10 single launches (burst) and back to back for about two seconds (sustained), with this
    library's kernel on the same operands beside it."""
    import comfy_kitchen_b200 as ckb
    torch = B.torch
    out = {"how": "torch.nn.functional.scaled_mm (cuBLASLt NVFP4) and ck_b200_scaled_mm_nvfp4 on the same quantized "
                  "N(0,1) operands; burst = best of 10 launches, sustained = back to back for ~2 s", "shapes": []}
    best = 0.0
    for n in (8192, 16384):
        g = torch.Generator(device=B.dev).manual_seed(n)
        a = torch.randn((n, n), generator=g, device=B.dev, dtype=torch.bfloat16)
        b = torch.randn((n, n), generator=g, device=B.dev, dtype=torch.bfloat16)
        ta, tb = ckb.dynamic_scale_nvfp4(a), ckb.dynamic_scale_nvfp4(b)
        qa, sfa = ckb.quantize_nvfp4(a, ta)
        qb, sfb = ckb.quantize_nvfp4(b, tb)
        del a, b
        fl = 2.0 * n * n * n
        entry = {"M": n, "N": n, "K": n}
        impls = {"ours": lambda: ckb.scaled_mm_nvfp4(qa, qb, ta, tb, sfa, sfb)}
        try:
            cublaslt_nvfp4(torch, qa, sfa, ta, qb, sfb, tb)
            impls["cublaslt"] = lambda: cublaslt_nvfp4(torch, qa, sfa, ta, qb, sfb, tb)
        except Exception as ex:   # depends on the torch / cuBLASLt build
            entry["cublaslt_unavailable"] = f"{type(ex).__name__}: {ex}"[:160]
        for key, fn in impls.items():
            replay, _ = B.graphed(fn)
            for _ in range(3):
                replay()
            burst = min(B.timed(replay, 1, all_ranks=False) for _ in range(10))
            sampler = ClockSampler(B.local_rank).start()
            ms, reps = B.for_seconds(replay, 2.0, 20)
            clocks = sampler.stop()
            entry[key] = {"burst_tflops": fl / (burst * 1e-3) / 1e12, "sustained_tflops": fl * reps / (ms * 1e-3) / 1e12,
                          "sustained_sm_mhz_median": clocks.get("sm_mhz"), "sustained_power_w_median": clocks.get("power_w_median"),
                          "sustained_reasons": clocks.get("reasons")}
            if key == "cublaslt":
                best = max(best, entry[key]["burst_tflops"])
            B.graphs.clear()
        out["shapes"].append(entry)
        del qa, qb, sfa, sfb
        torch.cuda.empty_cache()
    out["best_cublaslt_burst_tflops"] = best if best > 0 else None
    return out


def quantize_sweep(B: Bench):
    """quantize_nvfp4 / dequantize_nvfp4 on the twelve shapes of the bandwidth-sweep configuration, 2.5625 algorithmic
    bytes per element.  L2-warm: one input replayed (inputs up to ~100 MB then stay in the 126 MB L2).  L2-cold: a
    captured sequence over enough different inputs and outputs to exceed 4x the L2, so every launch reads HBM; for
    inputs above 0.5 GB one buffer is cold by itself."""
    import comfy_kitchen_b200 as ckb
    torch = B.torch
    sweep = []
    for (sm, sk) in SWEEP_SHAPES:
        in_bytes = sm * sk * 2
        nbuf = 1 if in_bytes > (512 << 20) else max(2, -(-(4 * L2_BYTES) // in_bytes))
        nbuf = min(nbuf, 96)
        gx = torch.Generator(device=B.dev).manual_seed(sm + sk)
        bufs = [torch.randn((sm, sk), generator=gx, device=B.dev, dtype=torch.bfloat16) for _ in range(nbuf)]
        tt = ckb.dynamic_scale_nvfp4(bufs[0])
        quant = [ckb.quantize_nvfp4(x, tt) for x in bufs]
        nbytes = sm * sk * 2.5625
        entry = {"M": sm, "K": sk, "input_mb": in_bytes / 1e6, "cold_buffers": nbuf}

        def q_all():
            return [ckb.quantize_nvfp4(x, tt) for x in bufs]

        def d_all():
            return [ckb.dequantize_nvfp4(q, tt, s, torch.bfloat16) for q, s in quant]

        for key, fn_all, fn_one in (("quantize", q_all, lambda: ckb.quantize_nvfp4(bufs[0], tt)),
                                    ("dequantize", d_all, lambda: ckb.dequantize_nvfp4(quant[0][0], tt, quant[0][1], torch.bfloat16))):
            reps = 5 if nbuf > 1 else 10
            r_cold, _ = B.graphed(fn_all)
            t_cold = B.timed(r_cold, reps, all_ranks=False) / (reps * nbuf)
            entry[f"{key}_cold_us"] = t_cold * 1e3
            entry[f"{key}_cold_gbs"] = nbytes / (t_cold * 1e-3) / 1e9
            B.graphs.clear()
            if nbuf > 1:
                r_warm, _ = B.graphed(fn_one)
                t_warm = B.timed(r_warm, 20, all_ranks=False) / 20
                entry[f"{key}_warm_us"] = t_warm * 1e3
                entry[f"{key}_warm_gbs"] = nbytes / (t_warm * 1e-3) / 1e9
                B.graphs.clear()
        sweep.append(entry)
        del bufs, quant
        torch.cuda.empty_cache()
    return sweep


def small_m_sweep(B: Bench):
    """T5-XXL-style feed-forward shapes (d = 4096, ff = 10240): one linear (quantize + GEMM, split-K below 129 rows)
    per M.  Two figures per shape.  `*_chain_us`: eight layers with eight different weights (189 MB, more than the L2,
    so every weight streams from HBM) launched one after the other inside one CUDA graph, time per layer - the way a
    stack of such layers runs.  `*_single_us`: a graph holding ONE launch, replayed back to back: this adds the gap
    between two graph launches (about 3 us for an empty kernel) and is the latency of an isolated call."""
    import comfy_kitchen_b200 as ckb
    torch = B.torch
    small_m = []
    gsm = torch.Generator(device=B.dev).manual_seed(5)
    LAYERS = 8
    for (sk, sn) in [(4096, 10240), (10240, 4096)]:
        weights = []
        for _ in range(LAYERS):
            ww = torch.randn((sn, sk), generator=gsm, device=B.dev, dtype=torch.bfloat16) * 0.02
            wts = ckb.dynamic_scale_nvfp4(ww)
            wq, wsf = ckb.quantize_nvfp4(ww, wts)
            weights.append((wq, wsf, wts))
            del ww
        for sm in (1, 16, 64, 512):
            xx = torch.randn((sm, sk), generator=gsm, device=B.dev, dtype=torch.bfloat16)
            tt = ckb.dynamic_scale_nvfp4(xx)
            qq, ss = ckb.quantize_nvfp4(xx, tt, pad_16x=True)

            def linear(w, xx=xx, tt=tt):
                q1, s1 = ckb.quantize_nvfp4(xx, tt, pad_16x=True)
                return ckb.scaled_mm_nvfp4(q1, w[0], tt, w[2], s1, w[1])

            def gemm(w, qq=qq, ss=ss, tt=tt):
                return ckb.scaled_mm_nvfp4(qq, w[0], tt, w[2], ss, w[1])

            r_lc, _ = B.graphed(lambda: [linear(w) for w in weights])
            r_gc, n_gc = B.graphed(lambda: [gemm(w) for w in weights])
            r_l1, _ = B.graphed(lambda: linear(weights[0]))
            r_g1, _ = B.graphed(lambda: gemm(weights[0]))
            # the same chains under the caller's promise that weights are resident (the GEMM asks for its weight before
            # it waits for the preceding kernel): what a model with weights quantized at load time may switch on
            torch.cuda.synchronize()
            prev = ckb.promise_resident_weights(True)
            r_lcr, _ = B.graphed(lambda: [linear(w) for w in weights])
            r_gcr, _ = B.graphed(lambda: [gemm(w) for w in weights])
            ckb.promise_resident_weights(prev)
            reps = 20
            t_lc = B.timed(r_lc, reps, all_ranks=False) / (reps * LAYERS)
            t_gc = B.timed(r_gc, reps, all_ranks=False) / (reps * LAYERS)
            t_lcr = B.timed(r_lcr, reps, all_ranks=False) / (reps * LAYERS)
            t_gcr = B.timed(r_gcr, reps, all_ranks=False) / (reps * LAYERS)
            t_l1 = B.timed(r_l1, 50, all_ranks=False) / 50
            t_g1 = B.timed(r_g1, 50, all_ranks=False) / 50
            small_m.append({"M": sm, "K": sk, "N": sn, "linear_chain_us": t_lc * 1e3, "gemm_chain_us": t_gc * 1e3,
                            "linear_chain_resident_weights_us": t_lcr * 1e3, "gemm_chain_resident_weights_us": t_gcr * 1e3,
                            "linear_single_us": t_l1 * 1e3, "gemm_single_us": t_g1 * 1e3,
                            "gemm_kernels": n_gc // LAYERS, "gemm_tflops": 2.0 * sm * sn * sk / (t_gc * 1e-3) / 1e12,
                            "weight_gbs": sn * sk * 0.5625 / (t_gc * 1e-3) / 1e9,
                            "weight_gbs_resident_weights": sn * sk * 0.5625 / (t_gcr * 1e-3) / 1e9})
            B.graphs.clear()
        del weights
    torch.cuda.empty_cache()
    return small_m


def eager_latency(B: Bench):
    """Wall-clock time per forward of a 4096 -> 4096 NVFP4 layer called eagerly (no CUDA graph), dynamic activation
    scale, as the reference layer is used (samples/nvfp4_linear.py:77-80): host work (Python, ctypes, tensor-map
    encoding, launches) plus device work, averaged over 200 back-to-back calls followed by one synchronise (best of three such runs)."""
    import comfy_kitchen_b200 as ckb
    torch = B.torch
    g = torch.Generator(device=B.dev).manual_seed(11)
    w = (torch.randn((4096, 4096), generator=g, device=B.dev) * 0.02).to(torch.bfloat16)
    lin = ckb.NVFP4Linear.from_float(w, None)
    out = []
    xs = {m: torch.randn((m, 4096), generator=g, device=B.dev, dtype=torch.bfloat16) for m in (1, 64, 512)}
    for x in xs.values():      # every shape and both forms once through before anything is timed
        for f in (lin.forward, lin.forward_unfused):
            for _ in range(50):
                f(x)
    torch.cuda.synchronize()
    for m, x in xs.items():
        rec = {"M": m}
        for name, f in (("one_call_us", lin.forward), ("three_operators_us", lin.forward_unfused)):
            best = None
            for _ in range(3):      # best of three runs of 200 forwards: host jitter is one-sided
                for _ in range(20):
                    f(x)
                torch.cuda.synchronize()
                t0 = time.perf_counter()
                for _ in range(200):
                    f(x)
                torch.cuda.synchronize()
                t = (time.perf_counter() - t0) / 200 * 1e6
                best = t if best is None else min(best, t)
            rec[name] = best
        out.append(rec)
    return {"layer": "NVFP4Linear 4096 -> 4096, bf16, input_scale=None", "per_forward": out,
            "one_call": "ck_b200_linear_nvfp4 (dynamic quantizer, GEMM: 2-3 launches from one library call)",
            "three_operators": "dynamic_scale_nvfp4, quantize_nvfp4, scaled_mm_nvfp4 (5-6 launches from three calls)"}


def mxfp8_record(B: Bench, wl, xs, ws_cpu, steps):
    """The MXFP8 sibling path on the same workload: quantizer GB/s (3.03125 algorithmic bytes per element: 2 in, 1 out,
    1/32 scale) and GEMM TFLOP/s per linear, with cuBLASLt's MXFP8 kernel beside it."""
    import comfy_kitchen_b200 as ckb
    torch = B.torch
    M = wl["M"]
    mx_lin, mq_ms, mg_ms, mc_ms, m_fl, m_bytes = [], 0.0, 0.0, 0.0, 0.0, 0.0
    for i, (name, k, n) in enumerate(wl["linears"]):
        wq8, wsf8 = ckb.quantize_mxfp8(ws_cpu[i].to(B.dev), pad_32x=True)
        xq8, xsf8 = ckb.quantize_mxfp8(xs[i], pad_32x=True)
        rq8, _ = B.graphed(lambda i=i: ckb.quantize_mxfp8(xs[i], pad_32x=True))
        rg8, _ = B.graphed(lambda xq8=xq8, wq8=wq8, xsf8=xsf8, wsf8=wsf8: ckb.scaled_mm_mxfp8(xq8, wq8, xsf8, wsf8))
        tq8 = B.timed(rq8, steps, all_ranks=False) / steps
        tg8 = B.timed(rg8, steps, all_ranks=False) / steps
        entry = {"linear": name, "quantize_us": tq8 * 1e3, "quantize_gbs": M * k * 3.03125 / (tq8 * 1e-3) / 1e9,
                 "gemm_us": tg8 * 1e3, "gemm_tflops": 2.0 * M * n * k / (tg8 * 1e-3) / 1e12}
        try:
            from torch.nn.functional import ScalingType, SwizzleType, scaled_mm

            def lt(xq8=xq8, wq8=wq8, xsf8=xsf8, wsf8=wsf8):
                return scaled_mm(xq8, wq8.t(), scale_a=xsf8.view(-1), scale_b=wsf8.view(-1),
                                 scale_recipe_a=ScalingType.BlockWise1x32, scale_recipe_b=ScalingType.BlockWise1x32,
                                 swizzle_a=SwizzleType.SWIZZLE_32_4_4, swizzle_b=SwizzleType.SWIZZLE_32_4_4,
                                 output_dtype=torch.bfloat16)
            rc8, _ = B.graphed(lt)
            tc8 = B.timed(rc8, steps, all_ranks=False) / steps
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
        B.graphs.clear()
    torch.cuda.empty_cache()
    return {"gemm_tflops": m_fl / (mg_ms * 1e-3) / 1e12, "quantize_gbs": m_bytes / (mq_ms * 1e-3) / 1e9,
            "cublaslt_gemm_tflops": (m_fl / (mc_ms * 1e-3) / 1e12) if mc_ms > 0 else None,
            "nominal_dense_fp8_tflops": 4500.0, "per_linear": mx_lin,
            "kernel": "gemm_nvfp4_pair_kernel<KB, DBG, FMT = 1> (CTA pairs, tcgen05 kind::mxf8f6f4.block_scale)"}


def wan_record(B: Bench, args):
    """A short record (5 steps) of the Wan-class workload (M = 32760, hidden 5120, FFN 13824), the configuration whose
    weights are N-sharded over the GPUs: step time and TFLOP/s at this GPU count, the collective used, and the check
    of the fused result against the NCCL all-gather."""
    torch = B.torch
    wl = WAN
    xs, ws = make_inputs_on_device(wl, B.dev, torch.bfloat16)
    plan = StepPlan(B, wl, xs, ws, args.collective)
    del ws
    torch.cuda.empty_cache()
    steps = 5
    try:
        for _ in range(3):
            plan.step()
        B.barrier()
        parity = plan.check_parity() if B.distributed else None
        overlap = plan.use_graph and not args.serial
        replay, launches = B.graphed(plan.step_overlapped if overlap else plan.step, use_graph=plan.use_graph)
        for _ in range(2):
            replay()
        ms = B.timed(replay, steps) / steps
        fl = flops_per_step(wl)
        rec = {"workload": wl["name"], "M": wl["M"], "linears": [list(l) for l in wl["linears"]], "steps": steps,
               "ms_per_step": ms, "value": fl / (ms * 1e-3) / 1e12, "unit": "TFLOP/s", "n_gpus": B.world,
               "mode": plan.mode_text(), "launch": ("one CUDA graph per step" + (", quantizers on a second branch" if overlap else ""))
               if plan.use_graph else "eager launches",
               "gpu_launches_per_step": launches, "parity": parity,
               "data": "synthetic, generated on the device from a seeded generator"}
        if plan.fused:
            out_bytes = sum(wl["M"] * lin.local_rows * 2 for lin in plan.layers) * (B.world - 1)
            rec["nvlink_achieved_gbs"] = out_bytes / (ms * 1e-3) / 1e9
        if B.distributed:
            ingress = (B.world - 1) / B.world * sum(wl["M"] * n * 2 for _, _, n in wl["linears"])
            rec["ingress_bound_ms_at_770_gbs"] = ingress / 770e9 * 1e3
        return rec
    finally:
        B.graphs.clear()
        plan.close()
        del plan, xs
        torch.cuda.empty_cache()


def run_kernels_only(args, wl):
    """A short, fixed sequence of the path's kernels for a profiler to pick launches from (ncu -k ... -s ... -c ...):
    two rounds over the workload's linears, each round launching per linear the quantizer with the given scale, the
    one-launch dynamic quantizer and the GEMM.  The first round warms up; nothing is timed."""
    import torch

    import comfy_kitchen_b200 as ckb
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    xs_cpu, ws_cpu = make_inputs(wl, torch.bfloat16)
    xs = [x.to(dev) for x in xs_cpu]
    weights = []
    for w in ws_cpu:
        wd = w.to(dev)
        tw = ckb.dynamic_scale_nvfp4(wd)
        weights.append(ckb.quantize_nvfp4(wd, tw) + (tw,))
        del wd
    ts = [ckb.dynamic_scale_nvfp4(x) for x in xs]
    torch.cuda.synchronize()
    n0 = ckb.launches()
    for _ in range(2):
        for x, t, (wq, wsf, tw) in zip(xs, ts, weights):
            q, sf = ckb.quantize_nvfp4(x, t)
            ckb.quantize_nvfp4_dynamic(x)
            ckb.scaled_mm_nvfp4(q, wq, t, tw, sf, wsf)
        torch.cuda.synchronize()
    # after the rounds: the small-M GEMM (M = 16) on the two feed-forward shapes of small_m_sweep, each tile configuration
    # (GEMM variants 1, 5, 6) three times on three different weights, so that every launch streams its weight from HBM
    gsm = torch.Generator(device=dev).manual_seed(5)
    for (sk, sn) in [(4096, 10240), (10240, 4096)]:
        small_w = []
        for _ in range(3):
            ww = torch.randn((sn, sk), generator=gsm, device=dev, dtype=torch.bfloat16) * 0.02
            wts = ckb.dynamic_scale_nvfp4(ww)
            small_w.append(ckb.quantize_nvfp4(ww, wts) + (wts,))
            del ww
        xx = torch.randn((16, sk), generator=gsm, device=dev, dtype=torch.bfloat16)
        tt = ckb.dynamic_scale_nvfp4(xx)
        qq, ss = ckb.quantize_nvfp4(xx, tt)
        torch.cuda.synchronize()
        for variant in (1, 5, 6):
            prev = ckb.set_tuning(1, variant)
            for wq, wsf, wts in small_w:
                ckb.scaled_mm_nvfp4(qq, wq, tt, wts, ss, wsf)
            ckb.set_tuning(1, prev)
            torch.cuda.synchronize()
    print(json.dumps({"kernels_only": wl["name"], "launches": ckb.launches() - n0, "device_status": ckb.read_device_status(),
                      "order_per_round": "per linear: quantize_nvfp4, quantize_nvfp4_dynamic, scaled_mm_nvfp4",
                      "then": "M = 16 GEMMs on 4096 -> 10240 and 10240 -> 4096: variants 1, 5, 6, three launches each"}), flush=True)


def run_ours(args, wl):
    import torch

    import comfy_kitchen_b200 as ckb

    B = Bench(args)
    dist, dev, rank, world, distributed = B.dist, B.dev, B.rank, B.world, B.distributed
    if args.no_dependent_launch:
        ckb.set_tuning(3, 0)
    elif args.dependent_launch_mask is not None:
        ckb.set_tuning(3, args.dependent_launch_mask)
    one_call = args.fused_linear
    if one_call:
        ckb.set_tuning(4, 1)
    for kv in args.tune:      # A/B runs of one library switch: --tune KEY=VALUE (ck_b200_set_tuning)
        key, value = kv.split("=")
        ckb.set_tuning(int(key), int(value))

    M = wl["M"]
    pad_m = M % 16 != 0
    xs_cpu, ws_cpu = make_inputs(wl, torch.bfloat16)
    xs = [x.to(dev) for x in xs_cpu]
    plan = StepPlan(B, wl, xs, ws_cpu, args.collective)
    layers, ts_x, fused = plan.layers, plan.ts_x, plan.fused

    sampler = ClockSampler(B.local_rank)
    if rank == 0:
        sampler.start()

    warm = max(3, args.warmup)
    for _ in range(warm):
        plan.step(one_call=one_call)
    B.barrier()
    assert ckb.read_device_status() == 0, "a bounded wait ran out during warm-up"

    # ---- parity of the path about to be timed, inside this run ----
    parity = plan.check_parity()
    if rank == 0 and not parity.get("ok", True):
        print(json.dumps({"error": "parity check failed", "parity": parity}), flush=True)
    if not parity.get("ok", True):
        plan.close()
        if distributed:
            dist.destroy_process_group()
        sys.exit(3)

    # ---- the timed region: exactly K steps ----
    # The step's four linears are independent work items (each has its own activation), so the step is one CUDA graph
    # with two branches: the quantizers on one, the GEMMs on the other, and the quantizer of linear i+1 runs beside the
    # GEMM of linear i (on several GPUs: beside its stores to the peers, so the link does not idle).  The same at every
    # GPU count.  `serial_chain` below is the same work with the eight kernels one after the other.
    overlap = plan.use_graph and not one_call and not args.serial
    step_fn = plan.step_overlapped if overlap else (lambda: plan.step(one_call=one_call))
    replay_step, launches_per_step = B.graphed(step_fn, use_graph=plan.use_graph)
    for _ in range(warm):
        replay_step()
    ms = B.timed(replay_step, args.steps)
    clocks = sampler.stop() if rank == 0 else {}      # the samples cover warm-up and the timed region only
    launches = launches_per_step * args.steps
    fl = flops_per_step(wl)
    value = fl * args.steps / (ms * 1e-3) / 1e12

    # the outputs the timed graph itself left behind, against the same linears computed outside it
    if plan.use_graph and overlap:
        kept = B.graphs[-1]._keep[0]
        ok = 1
        for x, lin, got in zip(xs, layers, kept):
            want = lin.gather(lin.local(x)) if fused else lin.local(x)
            if not torch.equal(got, want):
                ok = 0
        if distributed:
            flag = torch.tensor([ok], device=dev)
            dist.all_reduce(flag, op=dist.ReduceOp.MIN)
            ok = int(flag.item())
        parity["timed_graph"] = ("outputs of the last timed replay bit-equal to " +
                                 ("the NCCL all-gather of separately computed blocks" if fused else
                                  "the same linears launched one after the other")) if ok else "MISMATCH"
        parity["ok"] = bool(parity.get("ok", True) and ok)
        if not ok:
            if rank == 0:
                print(json.dumps({"error": "parity check of the timed graph failed", "parity": parity}), flush=True)
            plan.close()
            if distributed:
                dist.destroy_process_group()
            sys.exit(3)

    serial_chain = None
    if overlap:
        replay_s, n_s = B.graphed(lambda: plan.step(one_call=one_call), use_graph=plan.use_graph)
        for _ in range(warm):
            replay_s()
        ms_s = B.timed(replay_s, args.steps)
        serial_chain = {"ms_per_step": ms_s / args.steps, "value": fl * args.steps / (ms_s * 1e-3) / 1e12,
                        "gpu_launches_per_step": n_s,
                        "what": "the same eight kernels in one chain (quantize, GEMM, quantize, GEMM, ...): what a block "
                                "whose linears depend on one another can do"}
        if fused:
            out_bytes = sum(M * lin.local_rows * 2 for lin in layers) * (world - 1)
            serial_chain["nvlink_achieved_gbs"] = out_bytes / (ms_s / args.steps * 1e-3) / 1e9

    # ---- the step with per-call (dynamic) activation scales: what the layer does when a checkpoint has no input_scale
    dynamic = None
    if not one_call:
        replay_d, n_d = B.graphed(lambda: plan.step(dynamic=True), use_graph=plan.use_graph)
        for _ in range(warm):
            replay_d()
        ms_d = B.timed(replay_d, args.steps)
        dynamic = {"ms_per_step": ms_d / args.steps, "value": fl * args.steps / (ms_d * 1e-3) / 1e12,
                   "gpu_launches_per_step": n_d,
                   "slowdown_vs_static_serial_chain": (ms_d / args.steps) / (serial_chain["ms_per_step"] if serial_chain else ms / args.steps) - 1.0,
                   "what": "input_scale = None: amax(|x|)/(448*6) in the activation's dtype derived on the device in "
                           "front of every quantizer (comfy_kitchen/tensor/nvfp4.py:66-71), no host round trip"}

    # ---- sustained: the step graph replayed for seconds, with the clocks NVML shows meanwhile (single-GPU runs) ----
    sustained = None
    if not distributed and not args.no_sweep:
        s2 = ClockSampler(B.local_rank).start()
        ms_s, reps_s = B.for_seconds(replay_step, args.sustained_seconds, 200)
        c2 = s2.stop()
        v = fl * reps_s / (ms_s * 1e-3) / 1e12
        # right after the loop, while the GPU is at its sustained operating point: one launch per linear of the GEMM build
        # with cycle counters (CTA pair 0 reports cycles and nanoseconds of its epilogue role: the SM clock inside the
        # kernel, and the share of its time the MMA role spent waiting)
        in_kernel = {}
        qx_s = [lin.quantize_input(x) for x, lin in zip(xs, layers)]
        try:
            for (name, _, _), (q, sf, t), lin in zip(wl["linears"], qx_s, layers):
                ckb.set_tuning(2, 0)
                for _ in range(20):
                    lin.local_from_quantized(q, sf, t, M)          # keep the load on
                ckb.set_tuning(2, 2)                               # counting build, counters only (1 would also print)
                lin.local_from_quantized(q, sf, t, M)
                in_kernel[name] = ckb.read_gemm_counters()
        finally:
            ckb.set_tuning(2, 0)
        del qx_s
        sustained = {"seconds": ms_s / 1e3, "steps": reps_s, "ms_per_step": ms_s / reps_s, "value": v, "unit": "TFLOP/s",
                     "in_kernel": in_kernel,
                     "sm_mhz_median": c2.get("sm_mhz"), "sm_mhz_min": c2.get("sm_min_mhz"), "sm_max_mhz": c2.get("sm_max_mhz"),
                     "power_w_median": c2.get("power_w_median"), "power_w_max": c2.get("power_w_max"),
                     "reasons": c2.get("reasons"),
                     "value_scaled_to_max_clock": (v * c2["sm_max_mhz"] / c2["sm_mhz"]) if c2.get("sm_mhz") else None,
                     "burst_over_sustained": value / v,
                     "what": "the same CUDA graph as `value`, replayed back to back for this long; `value` itself is a "
                             "burst figure (K steps, a few ms)"}

    fused_linear = None
    if not distributed and not one_call and not args.no_sweep:
        # the same step with the quantizer inside the GEMM kernel (one kernel per linear), for comparison
        ckb.set_tuning(4, 1)
        replay_f, _ = B.graphed(lambda: plan.step(one_call=True))
        for _ in range(warm):
            replay_f()
        ms_f = B.timed(replay_f, args.steps)
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

    # R launches of one kernel per captured graph: inside a graph consecutive kernels follow one another like the
    # kernels of a step do (programmatic dependent launch, no host in between), so total / (K * R) is the kernel's own
    # duration; single-kernel graphs would add the gap between two graph launches (2-5 us) to every launch
    R = 10

    def repeated(fn):
        return lambda: [fn() for _ in range(R)]

    per_linear = []
    gemm_ms = quant_ms = gemm_fl = quant_bytes = 0.0
    for i, ((name, k, n), lin) in enumerate(zip(wl["linears"], layers)):
        rg, _ = B.graphed(repeated(one_gemm(i)))
        rq, _ = B.graphed(repeated(one_quant(i)))
        tg = B.timed(rg, args.steps) / (args.steps * R)
        tq = B.timed(rq, args.steps) / (args.steps * R)
        # the same quantizer launch through the kernel that parks inputs of up to ~32 MB in shared memory with the whole
        # input in flight (off by default: same time alone, and it cannot run beside a GEMM's CTAs)
        prev_onchip = ckb.set_tuning(10, 1)
        rq2, _ = B.graphed(repeated(one_quant(i)))
        tq_chip = B.timed(rq2, args.steps) / (args.steps * R)
        ckb.set_tuning(10, prev_onchip)
        B.graphs.clear()
        n_local = lin.local_rows
        per_linear.append({"linear": name, "K": k, "N_local": n_local, "quantize_us": tq * 1e3, "gemm_us": tg * 1e3,
                           "gemm_tflops": 2.0 * M * n_local * k / (tg * 1e-3) / 1e12,
                           "quantize_gbs": M * k * 2.5625 / (tq * 1e-3) / 1e9, "quantize_onchip_kernel_us": tq_chip * 1e3})
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
            rs, _ = B.graphed(lambda x_rows=x_rows, i=i: ckb.quantize_nvfp4(x_rows, ts_x[i], pad_16x=True))
            t_rows += B.timed(rs, args.steps) / args.steps
        row_sharded = {"aggregate_gbs": quant_bytes / (t_rows * 1e-3) / 1e9, "rows_per_rank": r1 - r0,
                       "us_per_step": t_rows * 1e3, "note": "weak in bytes per rank / strong in total: M rows split over the ranks"}
    B.graphs.clear()
    peaks = measured_peaks()
    gemm_tflops = gemm_fl / (gemm_ms * 1e-3) / 1e12
    quant_gbs = quant_bytes / (quant_ms * 1e-3) / 1e9
    hbm_peak = peaks.get("hbm_gbs", 6650.0)

    # ---- cuBLASLt NVFP4 through torch on the same operands: the kernel behind the reference eager backend ----
    try:
        tot, per = 0.0, {}
        for i in range(len(layers)):
            (q, sf), t, (w_q, w_sf, w_ts) = qx_all[i], ts_x[i], qw[i]
            rc, _ = B.graphed(repeated(lambda q=q, sf=sf, t=t, w_q=w_q, w_sf=w_sf, w_ts=w_ts: cublaslt_nvfp4(torch, q, sf, t, w_q, w_sf, w_ts)))
            tc = B.timed(rc, args.steps) / (args.steps * R)
            B.graphs.clear()
            tot += tc
            per[wl["linears"][i][0]] = 2.0 * M * layers[i].local_rows * wl["linears"][i][1] / (tc * 1e-3) / 1e12
        cublaslt = {"gemm_tflops": gemm_fl / (tot * 1e-3) / 1e12, "per_linear_tflops": per,
                    "ours_over_cublaslt": {pl["linear"]: pl["gemm_tflops"] / per[pl["linear"]] for pl in per_linear},
                    "what": "torch.nn.functional.scaled_mm (cuBLASLt NVFP4), same operands, GEMM only, timed like ours"}
    except Exception as ex:   # depends on the torch / cuBLASLt build
        cublaslt = {"unavailable": f"{type(ex).__name__}: {ex}"[:200]}
    B.graphs.clear()

    # ---- the measured ceiling for a block-scaled FP4 GEMM on this GPU (single-GPU runs) ----
    ceiling = None
    if not distributed and not args.no_sweep:
        ceiling = fp4_ceiling(B)
    ceiling_peak = (ceiling or {}).get("best_cublaslt_burst_tflops")

    roofline = {
        "kernel": "gemm_nvfp4_pair_kernel<128, false, 0, -1> (CTA pairs, 256x256 tiles, tcgen05 cta_group::2)",
        "bound": "tensor", "achieved": gemm_tflops, "peak": NOMINAL_NVFP4_TFLOPS,
        "unit": "TFLOP/s", "frac": gemm_tflops / NOMINAL_NVFP4_TFLOPS,
        # dram__bytes_read.sum + dram__bytes_write.sum per launch, mean of the four Flux launches
        "traffic": 56.45e6 if (args.workload == "flux" and world == 1) else None,
        "traffic_source": "one ncu capture of these four launches (summary under profiles/), not measured in this run",
        "peak_source": "nominal dense NVFP4 (vendor figure); MEASURED_PEAKS.json has no FP4 entry",
        "peak_measured_cublaslt": ceiling_peak,
        "frac_of_measured_cublaslt": (gemm_tflops / ceiling_peak) if ceiling_peak else None,
        "frac_of_4x_measured_bf16": (gemm_tflops / (4.0 * peaks["bf16_tflops"])) if "bf16_tflops" in peaks else None,
        "algorithmic_flops_per_launch": gemm_fl / len(layers), "avg_launch_us": gemm_ms * 1e3 / len(layers),
        "timing": "each linear's kernel launched 10 times per captured graph and the graph replayed K times between CUDA "
                  "events: total / (10 K) per launch (same operands every launch, so they stay in L2, as the activation "
                  "does inside a step where the quantizer has just written it; outputs rotate over 10 buffers)",
        "quantize": {"kernel": "quantize_nvfp4_flat_kernel<bf16, vec, 2> (inputs of 20 MB to 0.25 GB; "
                               "quantize_nvfp4_kernel outside that range)",
                     "bound": "hbm", "achieved": quant_gbs, "peak": hbm_peak,
                     "unit": "GB/s", "frac": quant_gbs / hbm_peak,
                     "peak_source": "measured copy (MEASURED_PEAKS.json)" if "hbm_gbs" in peaks else "fallback",
                     "frac_of_nominal_8000": quant_gbs / 8000.0, "algorithmic_bytes_per_element": 2.5625,
                     "note": "activations of 28-113 MB: repeats of one input are partly L2 resident; the sweep gives "
                             "L2-cold and L2-warm figures per shape"},
        "per_linear": per_linear,
    }

    sweep = small_m = mxfp8 = comparators = eager = None
    if not distributed and not args.no_sweep:
        sweep = quantize_sweep(B)
        small_m = small_m_sweep(B)
        eager = eager_latency(B)
        mxfp8 = mxfp8_record(B, wl, xs, ws_cpu, args.steps)
        comparators = quantize_comparators(B, xs, ts_x, [l[0] for l in wl["linears"]])

    # ---- end to end: pinned host activations in, host outputs back, copies inside the timed region ----
    # One GPU: the whole activation comes up, the whole output goes back.  Several GPUs: the job's input still crosses
    # PCIe once in total - rank r uploads rows [r M/G, (r+1) M/G) of every activation and the ranks all-gather the
    # slices over NVLink (every rank needs the whole activation for its column block) - and every rank downloads its
    # own column block of the output.
    x_host = [x.pin_memory() for x in xs_cpu]
    y_host = [torch.empty((M, lin.local_rows), dtype=torch.bfloat16).pin_memory() for lin in layers]
    shard_upload = distributed and M % world == 0
    r0, r1 = (rank * (M // world), (rank + 1) * (M // world)) if shard_upload else (0, M)
    h2d = sum((r1 - r0) * x.shape[1] * 2 for x in x_host)
    d2h = sum(y.numel() * 2 for y in y_host)

    # Three streams: uploads, the operators (the current stream), downloads.  PCIe carries both directions at once and
    # the GPU has separate copy engines for them, so linear i's output goes back while linear i+1's activations come
    # in, also across step boundaries; events order upload -> operators -> download per linear.  Each linear has
    # its own device input buffer, reused every step once the operators of the previous step have read it.
    s_in, s_out = torch.cuda.Stream(), torch.cuda.Stream()
    x_dev = [torch.empty_like(x) for x in xs]
    x_part = [torch.empty((r1 - r0, x.shape[1]), dtype=x.dtype, device=dev) for x in xs] if shard_upload else None
    ev_in = [torch.cuda.Event() for _ in layers]
    ev_cmp = [torch.cuda.Event() for _ in layers]
    ev_out = [torch.cuda.Event() for _ in layers]
    serial = args.e2e_serial
    peers = plan.peers

    def e2e_step():
        cur = torch.cuda.current_stream()
        for i, (xh, yh, lin) in enumerate(zip(x_host, y_host, layers)):
            s_in.wait_event(ev_cmp[i])                     # last step's operators are done with x_dev[i] / x_part[i]
            if serial:
                s_in.wait_stream(s_out)
            with torch.cuda.stream(s_in):
                if shard_upload:
                    x_part[i].copy_(xh[r0:r1], non_blocking=True)
                else:
                    x_dev[i].copy_(xh, non_blocking=True)
                ev_in[i].record()
            cur.wait_event(ev_in[i])
            if shard_upload:
                dist.all_gather_into_tensor(x_dev[i], x_part[i])      # rows of all ranks, in rank order, over NVLink
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
    ems = B.timed(e2e_step, args.steps)
    e2e = {"value": fl * args.steps / (ems * 1e-3) / 1e12, "unit": "TFLOP/s", "h2d_bytes_per_step": h2d,
           "d2h_bytes_per_step": d2h, "ms_per_step": ems / args.steps,
           "pcie_gbs": {"h2d": h2d / (ems / args.steps * 1e-3) / 1e9, "d2h": d2h / (ems / args.steps * 1e-3) / 1e9},
           "h2d_bytes_per_step_all_ranks": h2d * world, "d2h_bytes_per_step_all_ranks": d2h * world,
           "what": "pinned host bf16 activations -> device, quantize_nvfp4 + scaled_mm_nvfp4 through the operator "
                   "interface, bf16 outputs -> pinned host; bytes per rank; "
                   + ("each rank uploads its M/G rows of every activation and the ranks all-gather them over NVLink, "
                      "each downloads its own column block; " if shard_upload else "")
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

    nvlink = None
    if fused:
        # bytes this rank's GEMM epilogues push to the other ranks per step, against the measured peer-copy rate
        out_bytes = sum(M * lin.local_rows * 2 for lin in layers) * (world - 1)
        ingress = (world - 1) / world * sum(M * n * 2 for _, _, n in wl["linears"])
        nvlink = {"bytes_out_per_rank_per_step": out_bytes,
                  "achieved_gbs": out_bytes / (ms / args.steps * 1e-3) / 1e9, "peak_gbs": 770.0,
                  "peak_source": "measured peer copy per direction on this pool",
                  "ingress_bound_ms": ingress / 770e9 * 1e3,
                  "note": "whole step in the denominator, quantizer kernels (no traffic) included"}

    # release the Flux plan's peer memory before the Wan record maps its own
    del qx_all, qw, x_dev, x_host, y_host, replay_step
    B.graphs.clear()
    plan.close()
    torch.cuda.empty_cache()

    # ---- the Wan-class workload, briefly, at this GPU count ----
    wan = None
    if not args.no_wan and args.workload == "flux":
        try:
            wan = wan_record(B, args)
        except Exception as ex:
            wan = {"failed": f"{type(ex).__name__}: {ex}"[:300]}
        status = status or ckb.read_device_status()

    # ---- CPU baseline on a bounded sample (rank 0, single-GPU run only) ----
    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        xs_bits, w_q, threads = prepare_cpu(wl, xs_cpu, ws_cpu)
        rows = min(CPU_SAMPLE_ROWS, M)
        cpu_reference_step(wl, xs_bits, w_q, rows)
        t0 = time.perf_counter()
        reps, cfl = 0, 0.0
        while reps < 2 or (time.perf_counter() - t0 < 12.0 and reps < 200):
            cfl += cpu_reference_step(wl, xs_bits, w_q, rows)
            reps += 1
        dt = time.perf_counter() - t0
        cpu = {"value": cfl / dt / 1e12, "unit": "TFLOP/s", "cores": threads, "kind": "port",
               "sample": f"{cpu_sample_text(wl, rows)}, {reps} repetitions, {dt:.1f} s of CPU work"}

    if rank == 0:
        line = {
            "metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
            "warmup": warm, "ms_per_step": ms / args.steps, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": DTYPE, "data": "synthetic", "config": workload_config(wl),
            "run": {"parallelism": plan.mode_text(),
                    "gemm_streams": (args.gemm_streams if (fused and overlap) else 1),
                    "launch": "one CUDA graph per step" if plan.use_graph else "eager launches",
                    "linear": ("one kernel per linear: the GEMM kernel quantizes the activations beside its main loop "
                               "(ck_b200_linear_nvfp4)") if one_call and not distributed else
                              ("quantize_nvfp4 kernel and scaled_mm_nvfp4 kernel per linear; the four linears are independent "
                               "work items, so the quantizer of linear i+1 runs beside the GEMM of linear i (two branches of "
                               "one CUDA graph); serial_chain gives the same kernels one after the other") if overlap else
                              "quantize_nvfp4 kernel, then scaled_mm_nvfp4 kernel, the four linears one after the other"},
            "roofline": roofline, "cpu_baseline": cpu, "e2e": e2e, "gpu_launches": launches, "clocks": clocks,
            "parity": parity, "sustained": sustained, "serial_chain": serial_chain, "dynamic_scale_step": dynamic,
            "fp4_ceiling": ceiling, "cublaslt_comparator": cublaslt, "device_status": status,
            "quantize_gbs": quant_gbs, "quantize_row_sharded": row_sharded, "gemm_only_tflops": gemm_tflops,
            "quantize_sweep": sweep, "quantize_comparators": comparators, "small_m_sweep": small_m,
            "eager_latency": eager, "mxfp8": mxfp8,
            "fused_linear": fused_linear, "wan": wan,
        }
        if nvlink is not None:
            line["nvlink"] = nvlink
        print(json.dumps(line), flush=True)
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
    ap.add_argument("--no-sweep", action="store_true",
                    help="skip the single-GPU extras: sustained run, FP4 ceiling, quantizer sweep and comparators, "
                         "small-M sweep, MXFP8")
    ap.add_argument("--no-wan", action="store_true", help="skip the short record of the Wan-class workload")
    ap.add_argument("--gemm-streams", type=int, default=2, choices=[1, 2],
                    help="N > 1: run the link-bound GEMM + all-gather kernels on one stream, or alternate them between two "
                         "streams with half of the CTA pairs each")
    ap.add_argument("--serial", action="store_true",
                    help="time the eight kernels of a step as one chain instead of overlapping each quantizer with the "
                         "previous linear's GEMM")
    ap.add_argument("--sustained-seconds", type=float, default=3.0)
    ap.add_argument("--peer-map-limit-gib", type=int, default=12,
                    help="N > 1: above this many GiB of peer-mapped output matrices per rank the NCCL all-gather is used")
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
    ap.add_argument("--tune", action="append", default=[], metavar="KEY=VALUE",
                    help="set a library tuning switch (ck_b200_set_tuning) before anything runs; may be repeated")
    ap.add_argument("--kernels-only", action="store_true",
                    help="launch each kernel of the path twice on the workload's shapes and exit (a target for ncu captures)")
    args = ap.parse_args()
    wl = WORKLOADS[args.workload]
    if args.impl == "reference":
        run_reference_arm(args, wl)
    elif args.kernels_only:
        run_kernels_only(args, wl)
    else:
        run_ours(args, wl)


if __name__ == "__main__":
    main()
