#!/usr/bin/env python
"""Benchmark of the MX-FP6 GEMM path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl native|reference]

N = 1: one step = one GEMM of the headline configuration, M=N=K=8192, E2M3, per-32-block amplitudes drawn
       log-normal(0, 1.5) (synthetic, seeded).  `value` is TFLOP/s with the packed operands resident in HBM;
       `e2e` is the same metric with the packed operands starting in pinned host memory and C read back to
       the host inside the timed region.
N > 1: the column-parallel configuration M=16384, N=57344, K=8192: B split along N over the ranks, A
       replicated, each rank's [M, N/g] block of C all-gathered into the full C (one process per GPU,
       torch.distributed/NCCL).  `value` counts the whole job's FLOPs over the slowest rank's time.

`--impl reference` times the CPU dequantise-then-matmul path (the oracle) on the host cores instead.
Prints exactly one JSON line on rank 0.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "mxfp6_gemm_tflops"
UNIT = "TFLOP/s"
# The reference's own published figure for this metric: HipKittens FP6 GEMM at 8192^3 on an AMD MI355X
# (analysis/fp6_gemm/mi355x_fp6_gemm.json:2-6); the same file set records 3038.77 for NVIDIA's CUTLASS on a B200.
PUBLISHED_TFLOPS_8192 = 2861.52

HEADLINE = dict(M=8192, N=8192, K=8192, fmt="e2m3", dist="lognormal(0,1.5) block amplitudes")
SHARDED = dict(M=16384, N=57344, K=8192, fmt="e2m3", dist="N(0,1)")

# DRAM bytes (read + write) of one launch of the 8192^3 kernel from the ncu capture summarised in
# profiles/.
NCU_TRAFFIC_BYTES_8192 = 274.5e6   # profiles/mxfp6_gemm_pair_kernel_8192x8192x8192.md: 163.0 MB read + 111.5 MB written


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=1000)
    ap.add_argument("--warmup", type=int, default=100)
    ap.add_argument("--impl", default="native", choices=["native", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true", help="skip the CPU baseline leg (N=1)")
    ap.add_argument("--small", action="store_true", help="1024^3 instead of 8192^3 (profiling aid, not a bench value)")
    ap.add_argument("--shape", default=None, help="M,N,K of another single-GPU shape, e.g. 16,28672,8192 "
                                                   "(profiling aid: the line then reports that shape, HBM roofline for M<=128)")
    return ap.parse_args()


# ------------------------------------------------------------------------------------------ clocks
class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a timed region runs."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.idx = gpu_index
        self.lines: list[str] = []
        self.proc = None
        self.thread = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "20", "-i", str(self.idx)], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
        except Exception:
            self.proc = None
            return
        self.thread = threading.Thread(target=self._pump, daemon=True)
        self.thread.start()

    def _pump(self):
        for ln in self.proc.stdout:
            self.lines.append(ln.strip())

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons, power = [], [], set(), []
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])); mx.append(float(f[2])); power.append(float(f[3]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "power_w_max": max(power) if power else None, "samples": len(sm), "reasons": sorted(reasons)}


# ------------------------------------------------------------------------------------------ inputs
def make_operands(torch, hk, rows, K, dist_name, seed, device):
    """Seeded synthetic fp32 operand on the GPU, quantised to packed MX-FP6 by the library's quantiser."""
    g = torch.Generator(device=device).manual_seed(seed)
    x = torch.randn((rows, K), generator=g, device=device, dtype=torch.float32)
    if dist_name == "lognormal":
        amp = torch.exp(1.5 * torch.randn((rows, K // 32), generator=g, device=device, dtype=torch.float32))
        x = (x.view(rows, K // 32, 32) * amp.unsqueeze(-1)).view(rows, K)
    packed, scales = hk.quantize(x, hk.E2M3)
    del x
    return packed, scales


def algorithmic_bytes(M, N, K):
    return 0.75 * K * (M + N) + (M + N) * K / 32 + 2.0 * M * N


# ------------------------------------------------------------------------------------------ native arm
def run_native(args):
    import torch
    import torch.distributed as dist

    import hipkittensp_b200 as hk
    from hipkittensp_b200.sharded import ColumnParallelGemm, shard_bounds

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.gpus > 1 and world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} needs torchrun with {args.gpus} ranks (WORLD_SIZE={world})")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)

    peaks = {}
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            peaks = json.load(f)
    except Exception:
        pass

    K_steps, W = args.steps, max(args.warmup, 3)
    if world == 1:
        cfg = dict(HEADLINE)
        if args.small:
            cfg.update(M=1024, N=1024, K=1024)
        if args.shape:
            m_, n_, k_ = (int(x) for x in args.shape.split(","))
            cfg.update(M=m_, N=n_, K=k_)
        M, N, K = cfg["M"], cfg["N"], cfg["K"]
        n_sets = 2            # rotate operand sets: 2 x (A+B) + C > L2
        sets = []
        for i in range(n_sets):
            a, sa = make_operands(torch, hk, M, K, "lognormal", 10 + i, device)
            b, sb = make_operands(torch, hk, N, K, "lognormal", 20 + i, device)
            sets.append((a, sa, b, sb))
        C = torch.empty((M, N), dtype=torch.bfloat16, device=device)

        def step(i):
            a, sa, b, sb = sets[i % n_sets]
            hk.dispatch_micro(a, b, C, sa, sb, hk.E2M3)

        n_local, flops_step = N, 2.0 * M * N * K
        workload = f"mxfp6_e2m3_gemm_{M}x{N}x{K}"
        launches_per_step = 1
    else:
        cfg = dict(SHARDED)
        M, N, K = cfg["M"], cfg["N"], cfg["K"]
        lo, hi = shard_bounds(N, world, rank)
        a, sa = make_operands(torch, hk, M, K, "normal", 10, device)             # replicated: same seed on all ranks
        b, sb = make_operands(torch, hk, hi - lo, K, "normal", 100 + rank, device)  # this rank's rows of B
        try:
            op = ColumnParallelGemm(M, N, K, device=device)            # fused: tiles pushed to peers by the epilogue
        except Exception as e:                                          # symmetric memory unavailable on this box
            print(f"[bench] fused gather unavailable ({e!r}); using the NCCL all-gather", file=sys.stderr)
            op = ColumnParallelGemm(M, N, K, device=device, gather="nccl")

        def step(i):
            op(a, sa, b, sb)

        n_local, flops_step = hi - lo, 2.0 * M * N * K
        workload = f"mxfp6_e2m3_gemm_{M}x{N}x{K}_colparallel_gather"
        launches_per_step = 1

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- device-resident timing
    for i in range(W):
        step(i)
    assert hk.device_status() == 0
    sampler = ClockSampler(local_rank)
    barrier()
    sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record()
    for i in range(K_steps):
        step(i)
    e1.record()
    barrier()
    ms_total = e0.elapsed_time(e1)
    clocks = sampler.stop()
    assert hk.device_status() == 0

    # kernel-only time of the GEMM launch (events on the launch stream around each launch)
    kev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(K_steps)]
    barrier()
    if world == 1:
        for i, (s, e) in enumerate(kev):
            s.record(); step(i); e.record()
    else:
        for i, (s, e) in enumerate(kev):
            s.record(); op.local_gemm(a, sa, b, sb); e.record()
    barrier()
    kernel_ms = statistics.mean(s.elapsed_time(e) for s, e in kev)

    # ---- end to end: operands start in pinned host memory, result ends in pinned host memory
    if world == 1:
        a, sa, b, sb = sets[0]
    host_in = [t.cpu().pin_memory() for t in (a, sa, b, sb)]
    out_dev = C if world == 1 else op.c_shard
    host_out = torch.empty(out_dev.shape, dtype=out_dev.dtype).pin_memory()
    h2d = sum(t.numel() * t.element_size() for t in host_in)
    d2h = host_out.numel() * host_out.element_size()

    # The public host-memory entry: copy-in, kernel and copy-out of consecutive steps overlap on three streams.
    if world == 1:
        pipe = hk.HostGemm(M, N, K, device=device)
    else:
        def sharded_step(s):
            op(s["a"], s["sa"], s["b"], s["sb"])
            return op.c_shard
        pipe = hk.HostGemm(M, hi - lo, K, device=device, gemm=sharded_step)

    def e2e_step():
        pipe(host_in[0], host_in[1], host_in[2], host_in[3], host_out)

    for _ in range(3):
        e2e_step()
    pipe.synchronize()
    barrier()
    e0.record()
    for _ in range(K_steps):
        e2e_step()
    pipe.synchronize()
    e1.record()
    barrier()
    ms_e2e = e0.elapsed_time(e1)

    if world > 1:
        t = torch.tensor([ms_total, ms_e2e, kernel_ms], device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_total, ms_e2e, kernel_ms = (float(x) for x in t.cpu())

    if rank == 0:
        ms_step = ms_total / K_steps
        value = flops_step / (ms_step * 1e-3) / 1e12
        e2e_val = flops_step / (ms_e2e / K_steps * 1e-3) / 1e12
        # roofline of the GEMM kernel: tensor-bound; FP6 runs at the FP8 rate = 2x the measured dense bf16 rate
        bf16_peak = peaks.get("bf16_tflops_sustained")
        peak_src = "2 x MEASURED_PEAKS.json bf16_tflops_sustained (fp6 issues at the fp8 rate, twice bf16)"
        if bf16_peak is None:
            bf16_peak, peak_src = 1400.0, "2 x fallback sustained bf16 1.4 PFLOP/s"
        peak = 2.0 * bf16_peak
        flops_launch = 2.0 * M * n_local * K
        achieved = flops_launch / (kernel_ms * 1e-3) / 1e12
        traffic = NCU_TRAFFIC_BYTES_8192 if (world == 1 and not args.small and not args.shape) else None
        line = {
            "metric": METRIC, "value": round(value, 2), "unit": UNIT, "n_gpus": world, "steps": K_steps, "warmup": W,
            "ms_per_step": round(ms_step, 5), "higher_is_better": True,
            "scaling": "weak" if world == 1 else "strong",
            "vs_baseline": round(value / PUBLISHED_TFLOPS_8192, 4) if (world == 1 and not args.small and not args.shape) else None,
            "dtype": "fp6_e2m3xfp6_e2m3->f32->bf16",
            "data": "synthetic",
            "config": {"workload": workload, "M": M, "N": N, "K": K, "format": "e2m3", "scale": "e8m0 per 32 along K",
                       "l2": "operand sets rotate and A+B+C exceed L2" if world == 1 else "A+B shard+C exceed L2",
                       "parallelism": "single" if world == 1 else
                       (f"column-parallel x{world}, C tiles pushed to peers by the GEMM epilogue (symmetric memory)"
                        if op.mode == "fused" else f"column-parallel x{world}, nccl all-gather of C")},
            "e2e": {"value": round(e2e_val, 2), "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
            "gpu_launches": K_steps * launches_per_step,
            "clocks": clocks,
            "roofline": {"bound": "tensor", "achieved": round(achieved, 2), "peak": round(peak, 1), "unit": "TFLOP/s",
                         "frac": round(achieved / peak, 4), "traffic": traffic, "peak_source": peak_src,
                         "kernel_ms": round(kernel_ms, 5),
                         "frac_of_datasheet_4500": round(achieved / 4500.0, 4),
                         "algorithmic_bytes": algorithmic_bytes(M, n_local, K)},
        }
        if world == 1 and M <= 128:       # skinny shapes are HBM-bound: report against the measured copy bandwidth
            hbm = peaks.get("hbm_gbs", 6650.0)
            gbs = algorithmic_bytes(M, N, K) / (kernel_ms * 1e-3) / 1e9
            line["roofline"] = {"bound": "hbm", "achieved": round(gbs, 1), "peak": hbm, "unit": "GB/s",
                                "frac": round(gbs / hbm, 4), "traffic": None, "kernel_ms": round(kernel_ms, 5),
                                "peak_source": "MEASURED_PEAKS.json hbm_gbs" if "hbm_gbs" in peaks else "fallback 6.65 TB/s",
                                "frac_of_datasheet_8000": round(gbs / 8000.0, 4),
                                "algorithmic_bytes": algorithmic_bytes(M, N, K)}
        if world == 1 and not args.no_cpu_baseline:
            line["cpu_baseline"] = cpu_baseline([t.cpu() for t in sets[0]], M, N, K, budget_s=20.0)
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


# ------------------------------------------------------------------------------------------ CPU path
def cpu_baseline(operands, M, N, K, budget_s):
    """Times the oracle's dequantise-then-matmul path on the host cores for a bounded sample of the workload:
    the first `rows` rows of A against all of B (both dequantised inside the timed region)."""
    import torch

    from oracle import mxfp6_ref as R

    a, sa, b, sb = operands
    cores = torch.get_num_threads()
    R.gemm_cpu_path(a[:64], sa[:64], b[:512], sb[:512])          # warm the thread pool
    t0 = time.perf_counter()
    R.gemm_cpu_path(a[:256], sa[:256], b, sb)
    probe = time.perf_counter() - t0                              # 256 rows incl. the dequantisation of all of B
    rows = M
    while rows > 256 and probe * rows / 256 > budget_s:
        rows //= 2
    t0 = time.perf_counter()
    R.gemm_cpu_path(a[:rows], sa[:rows], b, sb)
    dt = time.perf_counter() - t0
    return {"value": round(2.0 * rows * N * K / dt / 1e12, 4), "unit": UNIT, "cores": cores, "kind": "port",
            "sample": f"rows 0..{rows} of A against all {N} rows of B, K={K}: torch dequantise + fp32 matmul + bf16 round, {dt:.2f} s"}


def run_reference(args):
    """The reference arm: the CPU dequantise-then-matmul path on this box's host cores (all threads torch uses)."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import numpy as np
    import torch

    from oracle import mxfp6_ref as R

    world = max(1, args.gpus)
    cfg = dict(HEADLINE) if world == 1 else dict(SHARDED)
    M, N, K = cfg["M"], cfg["N"], cfg["K"]
    K_steps, W = args.steps, args.warmup
    # bounded sample: a block of rows of A against a block of rows of B with the workload's K
    budget = 150.0 / max(1, K_steps + W)
    rows_b = min(N, 8192)
    rng = np.random.default_rng(0)
    xb = rng.standard_normal((rows_b, K), dtype=np.float32)
    pb, sb = R.c_quantize(xb, R.E2M3)
    del xb
    rows_a = min(M, 8192)
    xa = rng.standard_normal((rows_a, K), dtype=np.float32)
    pa, sa = R.c_quantize(xa, R.E2M3)
    del xa
    ta, tsa, tb, tsb = (torch.from_numpy(x) for x in (pa, sa, pb, sb))
    R.gemm_cpu_path(ta[:64], tsa[:64], tb[:512], tsb[:512])      # warm the thread pool
    t0 = time.perf_counter()
    R.gemm_cpu_path(ta[:256], tsa[:256], tb, tsb)
    probe = time.perf_counter() - t0                              # 256 rows of A against all sampled rows of B
    rows = rows_a
    while rows > 256 and probe * rows / 256 > budget:
        rows //= 2
    # many steps: shrink the B side of the sample too (its dequantisation is the floor of a step)
    while rows_b > 512 and probe * (rows / 256) * (rows_b / tb.shape[0]) > budget:
        rows_b //= 2
    tb, tsb = tb[:rows_b], tsb[:rows_b]
    for _ in range(W):
        R.gemm_cpu_path(ta[:rows], tsa[:rows], tb, tsb)
    t0 = time.perf_counter()
    for _ in range(K_steps):
        R.gemm_cpu_path(ta[:rows], tsa[:rows], tb, tsb)
    dt = (time.perf_counter() - t0) / max(1, K_steps)
    value = 2.0 * rows * rows_b * K / dt / 1e12
    cores = torch.get_num_threads()
    sample = f"per step: {rows} rows of A x {rows_b} rows of B, K={K} (dequantise both + fp32 matmul + bf16 round)"
    line = {
        "impl": "reference", "metric": METRIC, "value": round(value, 4), "unit": UNIT, "n_gpus": world,
        "steps": K_steps, "warmup": W, "ms_per_step": round(dt * 1e3, 3), "higher_is_better": True,
        "scaling": "weak" if world == 1 else "strong", "vs_baseline": None, "dtype": "fp6_e2m3xfp6_e2m3->f32->bf16",
        "data": "synthetic",
        "config": {"workload": f"mxfp6_e2m3_gemm_{M}x{N}x{K}" + ("" if world == 1 else "_colparallel_gather"),
                   "M": M, "N": N, "K": K, "format": "e2m3", "scale": "e8m0 per 32 along K"},
        "cpu_baseline": {"value": round(value, 4), "unit": UNIT, "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": round(value, 4), "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


if __name__ == "__main__":
    a = parse()
    if a.impl == "reference":
        run_reference(a)
    else:
        run_native(a)
