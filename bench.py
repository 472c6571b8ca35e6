#!/usr/bin/env python
"""Benchmark of the MX-FP6 GEMM path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl native|reference]

N = 1: one step = one GEMM of the headline configuration, M=N=K=8192, E2M3, per-32-block amplitudes drawn
       log-normal(0, 1.5) (synthetic, seeded).  `value` is TFLOP/s with the packed operands resident in HBM;
       `e2e` is the same metric with the packed operands starting in pinned host memory and C read back to
       the host inside the timed region.  The same line carries, measured in the same run: the other single-GPU
       configurations (`extra_configs`: the E3M2 FFN shape and 4096^3 against the tensor roofline, the decode
       shapes M = 1/16/64 against the HBM roofline), a figure for a seconds-long run (`sustained`), and a
       `check` of the timed operands' result against the fp64 CPU oracle on sampled rows.
N > 1: the column-parallel configuration M=16384, N=57344, K=8192: B split along N over the ranks, A
       replicated, each rank's [M, N/g] block of C gathered into the full C of every rank (one process per GPU,
       torch.distributed/NCCL).  `value` counts the whole job's FLOPs over the slowest rank's time.  After the
       timed regions every rank checks its gathered C (`check`): sampled full rows bit for bit against the
       single-GPU kernel, a checksum of the whole C equal on all ranks, the fused and the NCCL exchange
       against each other, and on rank 0 sampled rows against the fp64 CPU oracle.

`--impl reference` times the CPU dequantise-then-matmul path (the oracle) on the host cores instead.
Prints exactly one JSON line on rank 0; exits non-zero if a check fails.
"""
from __future__ import annotations

import argparse
import json
import os
import re
import statistics
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "mxfp6_gemm_tflops"
UNIT = "TFLOP/s"
# Figures the reference tree records for this metric at 8192^3 (analysis/fp6_gemm/mi355x_fp6_gemm.json:2-6 and
# analysis/fp6_gemm/plot.py:23-29): its own FP6 kernel on an AMD MI355X, and NVIDIA's CUTLASS on a B200.
PUBLISHED_TFLOPS_8192 = 2861.52
CUTLASS_B200_TFLOPS = {8192: 3038.77, 4096: 2757.18}
DATASHEET_TFLOPS = 4500.0        # dense FP6/FP8
DATASHEET_HBM_GBS = 8000.0

HEADLINE = dict(M=8192, N=8192, K=8192, fmt="e2m3", dist="lognormal(0,1.5) block amplitudes")
SHARDED = dict(M=16384, N=57344, K=8192, fmt="e2m3", dist="N(0,1)")
PAIR_PROFILE = os.path.join(ROOT, "profiles", "mxfp6_gemm_pair_kernel_8192x8192x8192.md")


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="native", choices=["native", "reference"])
    ap.add_argument("--gather", default="fused", choices=["fused", "copy"],
                    help="N > 1: the exchange that overlaps the GEMM and is timed (epilogue pushes, or copy engines behind block flags)")
    ap.add_argument("--no-cpu-baseline", action="store_true", help="skip the CPU baseline leg (N=1)")
    ap.add_argument("--no-extras", action="store_true", help="skip extra_configs, sustained and check (profiling aid)")
    ap.add_argument("--small", action="store_true", help="1024^3 instead of 8192^3 (profiling aid, not a bench value)")
    ap.add_argument("--shape", default=None, help="M,N,K of another single-GPU shape, e.g. 16,28672,8192 "
                                                   "(profiling aid: the line then reports that shape, HBM roofline for M<=128)")
    return ap.parse_args()


# ------------------------------------------------------------------------------------------ clocks
class ClockSampler:
    """Samples the SM clock, power and throttle reasons of one GPU through NVML from a thread of this process, as
    fast as NVML answers (about a millisecond per sample), each sample with its host time, so that the samples
    that fall inside a timed region of a few milliseconds can be told from the idle ones around it.  Reads only."""

    def __init__(self, gpu_index: int):
        self.idx = gpu_index
        self.samples: list[tuple[float, float, float, int]] = []     # (t, sm_mhz, power_w, reasons bitmask)
        self.max_mhz = None
        self._stop = threading.Event()
        self.thread = None
        self.err = None
        try:
            import pynvml

            self.nv = pynvml
            pynvml.nvmlInit()
            self.h = pynvml.nvmlDeviceGetHandleByIndex(self._physical_index(gpu_index))
            self.max_mhz = float(pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM))
            for _ in range(3):      # the first queries of a process are slow: make them here, not inside a timed region
                pynvml.nvmlDeviceGetClockInfo(self.h, pynvml.NVML_CLOCK_SM)
                pynvml.nvmlDeviceGetPowerUsage(self.h)
        except Exception as e:      # no NVML: the line says so
            self.nv, self.err = None, repr(e)

    @staticmethod
    def _physical_index(i: int) -> int:
        vis = os.environ.get("CUDA_VISIBLE_DEVICES")
        if vis:
            ids = [x for x in vis.split(",") if x.strip() != ""]
            if i < len(ids) and ids[i].strip().isdigit():
                return int(ids[i])
        return i

    def start(self):
        if self.nv is None:
            return
        self._stop.clear()
        self.thread = threading.Thread(target=self._run, daemon=True)
        self.thread.start()

    def _run(self):
        nv = self.nv
        while not self._stop.is_set():
            try:
                mhz = float(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                pw = nv.nvmlDeviceGetPowerUsage(self.h) / 1000.0
                rs = int(nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)) if hasattr(nv, "nvmlDeviceGetCurrentClocksEventReasons") \
                    else int(nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h))
                self.samples.append((time.perf_counter(), mhz, pw, rs))
            except Exception as e:
                self.err = repr(e)
                return
            time.sleep(0.0002)

    def stop(self):
        if self.thread is not None:
            self._stop.set()
            self.thread.join(timeout=2)
            self.thread = None

    def summary(self, t0: float | None = None, t1: float | None = None) -> dict:
        """Median SM clock and the throttle reasons seen between host times t0 and t1 (all samples if None)."""
        if self.nv is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvml unavailable: " + str(self.err)]}
        sel = [s for s in self.samples if (t0 is None or s[0] >= t0) and (t1 is None or s[0] <= t1)]
        note = "samples with a host time inside the region"
        if not sel and t0 is not None and self.samples:
            # a region of a few ms can fall between two answers of NVML: take the samples nearest to it
            mid = 0.5 * (t0 + t1)
            sel = sorted(self.samples, key=lambda s: abs(s[0] - mid))[:3]
            note = "no sample inside the region: the 3 nearest in time (%.1f ms away at most)" % (1e3 * max(abs(s[0] - mid) for s in sel))
        names = ((0x8, "hw_slowdown"), (0x40, "hw_thermal_slowdown"), (0x20, "sw_thermal_slowdown"), (0x4, "sw_power_cap"))
        reasons = sorted({n for s in sel for bit, n in names if s[3] & bit})
        return {"sm_mhz": statistics.median(s[1] for s in sel) if sel else None, "sm_max_mhz": self.max_mhz,
                "power_w_max": max((s[2] for s in sel), default=None), "samples": len(sel), "reasons": reasons,
                "how": "NVML polled from a thread of this process; " + note}


# ------------------------------------------------------------------------------------------ inputs
def make_operands(torch, hk, rows, K, dist_name, seed, device, fmt=None, scale=1.0, outlier_channels=0):
    """Seeded synthetic fp32 operand on the GPU, quantised to a packed MX operand by the library's quantiser."""
    g = torch.Generator(device=device).manual_seed(seed)
    x = torch.randn((rows, K), generator=g, device=device, dtype=torch.float32)
    if dist_name == "lognormal":
        amp = torch.exp(1.5 * torch.randn((rows, K // 32), generator=g, device=device, dtype=torch.float32))
        x = (x.view(rows, K // 32, 32) * amp.unsqueeze(-1)).view(rows, K)
    if scale != 1.0:
        x *= scale
    if outlier_channels:
        ch = torch.randperm(K, generator=torch.Generator(device="cpu").manual_seed(seed))[:outlier_channels].to(device)
        x[:, ch] *= 50.0
    packed, scales = hk.quantize(x, hk.E2M3 if fmt is None else fmt)
    del x
    return packed, scales


def algorithmic_bytes(M, N, K):
    return 0.75 * K * (M + N) + (M + N) * K / 32 + 2.0 * M * N


def tensor_peaks(peaks: dict, region_s: float) -> dict:
    """The tensor-rate ceilings a GEMM time is put against.  FP6 issues at the FP8 rate, twice the dense bf16 rate, so
    the measured ceiling is 2 x the cuBLAS bf16 figure: the burst one for a timed region shorter than a second, the
    sustained (power-capped) one for a longer region."""
    burst, sust = peaks.get("bf16_tflops"), peaks.get("bf16_tflops_sustained")
    src = "MEASURED_PEAKS.json"
    if burst is None or sust is None:
        burst, sust, src = 1590.0, 1400.0, "fallback (no MEASURED_PEAKS.json)"
    use_burst = region_s < 1.0
    return {"peak": 2.0 * (burst if use_burst else sust), "burst": 2.0 * burst, "sustained": 2.0 * sust,
            "source": f"2 x {src} {'bf16_tflops (burst: timed region shorter than 1 s)' if use_burst else 'bf16_tflops_sustained (timed region longer than 1 s)'}"}


def traffic_from_profile() -> float | None:
    """DRAM bytes (read + write) of one launch of the 8192^3 kernel, from the committed ncu summary."""
    try:
        m = re.search(r"traffic_bytes_per_launch:\s*([0-9.eE+]+)", open(PAIR_PROFILE).read())
        return float(m.group(1)) if m else None
    except Exception:
        return None


def oracle_rows_check(torch, C_rows, a_rows, sa_rows, b, sb, fmt):
    """Rows of a GPU result against the fp64-accumulated product of the exactly dequantised operands, computed on the
    host cores (the checker; outside every timed region).  Tolerances of the parity tests."""
    from oracle import mxfp6_ref as R

    Ad = R.dequantize_torch(a_rows.cpu(), sa_rows.cpu(), fmt).double()
    worst = {"row_rel": 0.0, "max_ulp": 0.0, "n_floor": 0}
    CH = 4096                      # rows of B per block: bounds the host memory of the dequantisation
    ref = torch.empty((Ad.shape[0], b.shape[0]), dtype=torch.float64)
    absdot = torch.empty_like(ref)
    for lo in range(0, b.shape[0], CH):
        Bd = R.dequantize_torch(b[lo:lo + CH].cpu(), sb[lo:lo + CH].cpu(), fmt).double()
        ref[:, lo:lo + CH] = Ad @ Bd.t()
        absdot[:, lo:lo + CH] = Ad.abs() @ Bd.abs().t()
    rep = R.error_report(C_rows.float().cpu().numpy(), ref.numpy(), absdot.numpy())
    for k in worst:
        worst[k] = rep[k]
    return worst


def graph_time_us(torch, launch, n_launch: int = 20, reps: int = 9, warm_ms: float = 10.0):
    """Time of one launch inside a CUDA graph of n_launch launches (no host time between them): the graph is replayed
    for at least warm_ms first (clocks up, caches in their steady state), then reps times between two events each.
    Returns (median, best) in microseconds."""
    launch(0)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        for i in range(n_launch):
            launch(i)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    g.replay()
    e1.record()
    torch.cuda.synchronize()
    first = max(e0.elapsed_time(e1), 1e-3)
    for _ in range(max(2, int(warm_ms / first))):
        g.replay()
    torch.cuda.synchronize()
    ts = []
    for _ in range(reps):
        e0.record()
        g.replay()
        e1.record()
        torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1) * 1e3 / n_launch)
    return statistics.median(ts), min(ts)


# ------------------------------------------------------------------------------------------ single GPU
def extra_configs(torch, hk, device, peaks):
    """The other single-GPU configurations, kernel-timed in CUDA graphs of 20 launches on rotating operand sets (median of
    9 replays after a few ms of warm-up replays).  Each is measured as a short burst after an idle pause, the memory-bound
    decode shapes first: a part that has just run a seconds-long dense GEMM stays power-capped for a while (SM clock about
    1.2 GHz of 1.965), which slows whatever is measured next, memory-bound kernels included.  The power-capped regime
    itself is the `sustained` figure of the headline configuration."""
    out = []
    hbm = peaks.get("hbm_gbs", 6650.0)
    hbm_src = "MEASURED_PEAKS.json hbm_gbs" if "hbm_gbs" in peaks else "fallback 6650"
    tp = tensor_peaks(peaks, 0.0)

    def pause():
        torch.cuda.synchronize()
        time.sleep(1.0)

    # decode: weights N(0, 0.02), activations N(0,1); two weight sets (176 MB each) rotate, so every launch streams
    # its weights from DRAM
    N, K = 28672, 8192
    wsets = [make_operands(torch, hk, N, K, "normal", 60 + i, device, hk.E2M3, scale=0.02) for i in range(2)]
    for M in (1, 16, 64):
        a, sa = make_operands(torch, hk, M, K, "normal", 70 + M, device, hk.E2M3)
        C = torch.empty((M, N), dtype=torch.bfloat16, device=device)

        def launch(i):
            b, sb = wsets[i % 2]
            hk.dispatch_micro(a, b, C, sa, sb, hk.E2M3)

        def launch_static(i):     # MXFP6_FLAG_B_STATIC: the caller declares the weights not written by the preceding kernel
            b, sb = wsets[i % 2]
            hk.dispatch_micro(a, b, C, sa, sb, hk.E2M3, b_static=True)

        pause()
        us, us_best = graph_time_us(torch, launch)
        us_static, _ = graph_time_us(torch, launch_static)
        gbs = algorithmic_bytes(M, N, K) / us / 1e3
        out.append({"workload": f"mxfp6_e2m3_gemm_{M}x{N}x{K}_decode", "M": M, "N": N, "K": K, "bound": "hbm",
                    "kernel_us": round(us, 2), "kernel_us_best": round(us_best, 2), "achieved": round(gbs, 1), "unit": "GB/s",
                    "frac": round(gbs / hbm, 4), "peak": hbm, "peak_source": hbm_src,
                    "frac_of_datasheet_8000": round(gbs / DATASHEET_HBM_GBS, 4), "algorithmic_bytes": algorithmic_bytes(M, N, K),
                    "kernel_us_weights_static": round(us_static, 2),
                    "frac_weights_static": round(algorithmic_bytes(M, N, K) / us_static / 1e3 / hbm, 4)})
    del wsets

    def tensor_case(name, M, N, K, fmt, a_kw, b_kw):
        sets = [(make_operands(torch, hk, M, K, "normal", 40 + i, device, fmt, **a_kw),
                 make_operands(torch, hk, N, K, "normal", 50 + i, device, fmt, **b_kw)) for i in range(2)]
        C = torch.empty((M, N), dtype=torch.bfloat16, device=device)

        def launch(i):
            (a, sa), (b, sb) = sets[i % 2]
            hk.dispatch_micro(a, b, C, sa, sb, fmt)

        pause()
        us, us_best = graph_time_us(torch, launch, warm_ms=3.0)
        tf = 2.0 * M * N * K / us / 1e6
        e = {"workload": name, "M": M, "N": N, "K": K, "bound": "tensor", "kernel_us": round(us, 2), "kernel_us_best": round(us_best, 2),
             "achieved": round(tf, 1), "unit": "TFLOP/s", "frac": round(tf / tp["burst"], 4), "peak": round(tp["burst"], 1),
             "frac_of_datasheet_4500": round(tf / DATASHEET_TFLOPS, 4)}
        if M == N == K and M in CUTLASS_B200_TFLOPS:
            e["vs_cutlass_b200"] = round(tf / CUTLASS_B200_TFLOPS[M], 4)
        out.append(e)
        del sets, C

    tensor_case("mxfp6_e2m3_gemm_4096x4096x4096", 4096, 4096, 4096, hk.E2M3, {}, {})
    tensor_case("mxfp6_e3m2_gemm_4096x14336x8192_ffn", 4096, 14336, 8192, hk.E3M2,
                dict(outlier_channels=8), dict(scale=0.02))
    assert hk.device_status() == 0
    return out


def run_single(args, torch, hk, device, peaks):
    K_steps, W = args.steps, max(args.warmup, 3)
    cfg = dict(HEADLINE)
    if args.small:
        cfg.update(M=1024, N=1024, K=1024)
    if args.shape:
        m_, n_, k_ = (int(x) for x in args.shape.split(","))
        cfg.update(M=m_, N=n_, K=k_)
    headline = not (args.small or args.shape)
    M, N, K = cfg["M"], cfg["N"], cfg["K"]
    sampler = ClockSampler(device.index)
    sampler.start()       # long before the timed region: the thread and NVML are in their stride when it starts
    n_sets = 4            # operand sets rotate (the reference's harness rotates 4, 8_wave.cu:255); with C they exceed L2
    sets = []
    for i in range(n_sets):
        a, sa = make_operands(torch, hk, M, K, "lognormal", 10 + i, device)
        b, sb = make_operands(torch, hk, N, K, "lognormal", 20 + i, device)
        sets.append((a, sa, b, sb))
    C = torch.empty((M, N), dtype=torch.bfloat16, device=device)

    def step(i):
        a, sa, b, sb = sets[i % n_sets]
        hk.dispatch_micro(a, b, C, sa, sb, hk.E2M3)

    flops_step = 2.0 * M * N * K
    # ---- device-resident timing: W warm-up steps, then exactly K steps between two events
    for i in range(W):
        step(i)
    assert hk.device_status() == 0
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    e0.record()
    for i in range(K_steps):
        step(i)
    e1.record()
    torch.cuda.synchronize()
    t1 = time.perf_counter()
    ms_total = e0.elapsed_time(e1)
    clocks = sampler.summary(t0, t1)
    assert hk.device_status() == 0

    # kernel-only time of the GEMM launch (events on the launch stream around each launch)
    kev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(K_steps)]
    torch.cuda.synchronize()
    for i, (s, e) in enumerate(kev):
        s.record(); step(i); e.record()
    torch.cuda.synchronize()
    kernel_ms = statistics.mean(s.elapsed_time(e) for s, e in kev)

    sampler.stop()

    # ---- the result of the timed operands against the CPU oracle, on sampled rows (outside every timed region)
    check = None
    if not args.no_extras:
        g = torch.Generator(device="cpu").manual_seed(123)
        n_rows = min(M, 32)
        rows = torch.sort(torch.randperm(M, generator=g)[:n_rows]).values
        if M >= 256:
            rows[:4] = torch.tensor([0, 127, 128, M - 1])
            rows = torch.sort(rows).values
        a, sa, b, sb = sets[(K_steps - 1) % n_sets]          # the operands of the last timed step: C holds their product
        step(K_steps - 1)
        torch.cuda.synchronize()
        rep = oracle_rows_check(torch, C[rows.to(device)], a[rows.to(device)], sa[rows.to(device)], b, sb, hk.E2M3)
        ok = rep["row_rel"] <= 1e-2 and rep["max_ulp"] <= 2.0
        check = {"ok": bool(ok), "rows": int(n_rows), "row_rel": float(f"{rep['row_rel']:.3e}"), "max_ulp": round(rep["max_ulp"], 3),
                 "n_floor": rep["n_floor"], "against": "fp64-accumulated product of the dequantised operands on the host cores",
                 "tolerance": "row_rel <= 1e-2, max_ulp <= 2 bf16 ulp"}

    # ---- the other single-GPU configurations, before anything long has heated the part (a short pause lets the
    # clocks settle as they would between unrelated kernels)
    extras = None
    if headline and not args.no_extras:
        extras = extra_configs(torch, hk, device, peaks)

    # ---- end to end: operands start in pinned host memory, result ends in pinned host memory
    a, sa, b, sb = sets[0]
    host_in = [t.cpu().pin_memory() for t in (a, sa, b, sb)]
    host_out = torch.empty(C.shape, dtype=C.dtype).pin_memory()
    h2d = sum(t.numel() * t.element_size() for t in host_in)
    d2h = host_out.numel() * host_out.element_size()
    # The public host-memory entry: copy-in, kernel and copy-out of consecutive steps overlap on three streams.
    pipe = hk.HostGemm(M, N, K, device=device)
    for _ in range(3):
        pipe(host_in[0], host_in[1], host_in[2], host_in[3], host_out)
    pipe.synchronize()
    torch.cuda.synchronize()
    n_e2e = min(K_steps, 50)          # PCIe-bound at about 2.7 ms per step
    e0.record()
    for _ in range(n_e2e):
        pipe(host_in[0], host_in[1], host_in[2], host_in[3], host_out)
    pipe.synchronize()
    e1.record()
    torch.cuda.synchronize()
    ms_e2e = e0.elapsed_time(e1) / n_e2e
    del pipe

    # ---- a seconds-long run of the same step: the power-capped regime, with its own clock record
    sustained = None
    if headline and not args.no_extras:
        sampler.samples.clear()
        sampler.start()
        n_long = max(K_steps, int(1.5 / (ms_total / K_steps * 1e-3)))
        torch.cuda.synchronize()
        ts0 = time.perf_counter()
        e0.record()
        for i in range(n_long):
            step(i)
        e1.record()
        torch.cuda.synchronize()
        ts1 = time.perf_counter()
        ms_long = e0.elapsed_time(e1)
        tf_long = flops_step * n_long / (ms_long * 1e-3) / 1e12
        tp_long = tensor_peaks(peaks, ms_long * 1e-3)
        sustained = {"steps": n_long, "seconds": round(ms_long * 1e-3, 3), "value": round(tf_long, 2), "unit": UNIT,
                     "frac_of_sustained_peak": round(tf_long / tp_long["sustained"], 4), "peak": round(tp_long["sustained"], 1),
                     "clocks": sampler.summary(ts0 + 0.3 * (ts1 - ts0), ts1)}
        sampler.stop()

    ms_step = ms_total / K_steps
    value = flops_step / (ms_step * 1e-3) / 1e12
    e2e_val = flops_step / (ms_e2e * 1e-3) / 1e12
    achieved = flops_step / (kernel_ms * 1e-3) / 1e12
    tp = tensor_peaks(peaks, ms_total * 1e-3)
    line = {
        "metric": METRIC, "value": round(value, 2), "unit": UNIT, "n_gpus": 1, "steps": K_steps, "warmup": W,
        "ms_per_step": round(ms_step, 5), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": round(value / PUBLISHED_TFLOPS_8192, 4) if headline else None,
        "vs_cutlass_b200": round(value / CUTLASS_B200_TFLOPS[8192], 4) if headline else None,
        "dtype": "fp6_e2m3xfp6_e2m3->f32->bf16", "data": "synthetic",
        "config": {"workload": f"mxfp6_e2m3_gemm_{M}x{N}x{K}", "M": M, "N": N, "K": K, "format": "e2m3",
                   "scale": "e8m0 per 32 along K"},
        "notes": {"l2": f"{n_sets} operand sets rotate; A+B+C of one step exceed L2", "parallelism": "single",
                  "vs_baseline": "value / 2861.52 (the reference's own kernel, MI355X); vs_cutlass_b200: value / 3038.77 "
                                 "(CUTLASS on a B200, as recorded in the reference tree)",
                  "e2e_steps": n_e2e},
        "e2e": {"value": round(e2e_val, 2), "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
        "gpu_launches": K_steps,
        "clocks": clocks,
        "roofline": {"bound": "tensor", "achieved": round(achieved, 2), "peak": round(tp["peak"], 1), "unit": "TFLOP/s",
                     "frac": round(achieved / tp["peak"], 4), "traffic": traffic_from_profile() if headline else None,
                     "peak_source": tp["source"], "kernel_ms": round(kernel_ms, 5),
                     "frac_of_burst_peak": round(achieved / tp["burst"], 4),
                     "frac_of_sustained_peak": round(achieved / tp["sustained"], 4),
                     "frac_of_datasheet_4500": round(achieved / DATASHEET_TFLOPS, 4),
                     "mhz_x_ms": round(clocks["sm_mhz"] * kernel_ms, 1) if clocks.get("sm_mhz") else None,
                     "algorithmic_bytes": algorithmic_bytes(M, N, K)},
    }
    if M <= 128:       # skinny shapes are HBM-bound: report against the measured copy bandwidth
        hbm = peaks.get("hbm_gbs", 6650.0)
        gbs = algorithmic_bytes(M, N, K) / (kernel_ms * 1e-3) / 1e9
        line["roofline"] = {"bound": "hbm", "achieved": round(gbs, 1), "peak": hbm, "unit": "GB/s",
                            "frac": round(gbs / hbm, 4), "traffic": None, "kernel_ms": round(kernel_ms, 5),
                            "peak_source": "MEASURED_PEAKS.json hbm_gbs" if "hbm_gbs" in peaks else "fallback 6.65 TB/s",
                            "frac_of_datasheet_8000": round(gbs / DATASHEET_HBM_GBS, 4),
                            "algorithmic_bytes": algorithmic_bytes(M, N, K)}
    if extras is not None:
        line["extra_configs"] = extras
    if sustained is not None:
        line["sustained"] = sustained
    if check is not None:
        line["check"] = check
    if not args.no_cpu_baseline:
        ops = [t.cpu() for t in (a, sa, b, sb)]
        line["cpu_baseline"] = cpu_baseline(ops, M, N, K, budget_s=20.0)
    print(json.dumps(line), flush=True)
    if check is not None and not check["ok"]:
        raise SystemExit(3)


# ------------------------------------------------------------------------------------------ several GPUs
def run_sharded(args, torch, hk, device, peaks, world, rank):
    import torch.distributed as dist

    from hipkittensp_b200.sharded import ColumnParallelGemm, shard_bounds

    K_steps, W = args.steps, max(args.warmup, 3)
    cfg = dict(SHARDED)
    M, N, K = cfg["M"], cfg["N"], cfg["K"]
    lo, hi = shard_bounds(N, world, rank)
    per = hi - lo
    sampler = ClockSampler(device.index)
    sampler.start()       # long before the timed region: the thread and NVML are in their stride when it starts
    a, sa = make_operands(torch, hk, M, K, "normal", 10, device)             # replicated: same seed on all ranks
    b, sb = make_operands(torch, hk, per, K, "normal", 100 + rank, device)   # this rank's rows of B
    def barrier():
        dist.barrier()
        torch.cuda.synchronize()

    # Two exchanges overlap the GEMM: tiles pushed to the peers by the epilogue ("fused", the default: the faster one on
    # every box measured so far) and blocks carried by the copy engines behind per-block flags the kernel raises ("copy").
    # The one named by --gather is timed; the other runs a few steps after the timed region, for the record and for the
    # check that both give the same matrix.  (Nothing runs before the timed region but its own warm-up: a second exchange
    # probed first would heat the part and cost the GEMM-bound configurations a few per cent.)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ops, probe_ms = {}, {}
    try:
        op = ColumnParallelGemm(M, N, K, device=device, gather=args.gather)
        if op.mode != args.gather:          # the operator fell back (shard too small for block flags)
            print(f"[bench] gather={args.gather} not available for this shard; timing gather={op.mode}", file=sys.stderr)
    except Exception as e:                                          # symmetric memory unavailable on this box
        print(f"[bench] gather={args.gather} unavailable ({e!r}); using the NCCL all-gather", file=sys.stderr)
        op = ColumnParallelGemm(M, N, K, device=device, gather="nccl")
    ops[op.mode] = op

    def step(i):
        return op(a, sa, b, sb)

    flops_step = 2.0 * M * N * K
    for i in range(W):
        step(i)
    assert hk.device_status() == 0
    barrier()
    t0 = time.perf_counter()
    e0.record()
    for i in range(K_steps):
        step(i)
    e1.record()
    barrier()
    t1 = time.perf_counter()
    ms_total = e0.elapsed_time(e1)
    clocks = sampler.summary(t0, t1)
    sampler.stop()
    assert hk.device_status() == 0

    # kernel-only time of this rank's shard GEMM (no exchange)
    kev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(min(K_steps, 20))]
    barrier()
    for s, e in kev:
        s.record(); op.local_gemm(a, sa, b, sb); e.record()
    barrier()
    kernel_ms = statistics.mean(s.elapsed_time(e) for s, e in kev)

    # ---- checks of the gathered result (outside the timed regions)
    if rank == 0:     # the launcher gives every rank one host thread; the oracle check on rank 0 may use the idle cores
        torch.set_num_threads(max(1, (os.cpu_count() or 8) - world))
    c_full = step(0)
    torch.cuda.synchronize()
    dist.barrier()
    check = {}
    # (i) sampled full rows against the single-GPU kernel, bit for bit: the rows of A are gathered into a small A and
    # multiplied by every rank's B shard (regenerated from its seed) with the same kernel (CTA-pair form forced, so each
    # element is accumulated over K in the same order)
    g = torch.Generator(device="cpu").manual_seed(321)
    n_rows = 64
    rows = torch.sort(torch.randperm(M, generator=g)[:n_rows]).values
    rows[:4] = torch.tensor([0, 127, 128, M - 1])
    rows = torch.sort(rows).values.to(device)
    a_s, sa_s = a[rows].contiguous(), sa[rows].contiguous()
    hk.debug_option("MXFP6_FORCE_CFG", "0,-1,-1,1")
    rows_equal = True
    oracle = {"row_rel": 0.0, "max_ulp": 0.0, "n_floor": 0}
    n_oracle = 16
    for r in range(world):
        b_r, sb_r = (b, sb) if r == rank else make_operands(torch, hk, per, K, "normal", 100 + r, device)
        want = hk.gemm(a_s, sa_s, b_r, sb_r)
        got = c_full[rows][:, r * per:(r + 1) * per]
        rows_equal = rows_equal and bool(torch.equal(want.view(torch.int16), got.contiguous().view(torch.int16)))
        if rank == 0:
            # (iii) rank 0: some of those rows against the fp64 CPU oracle
            rep = oracle_rows_check(torch, got[:n_oracle], a_s[:n_oracle], sa_s[:n_oracle], b_r, sb_r, hk.E2M3)
            oracle = {k: max(oracle[k], rep[k]) for k in oracle}
        del b_r, sb_r, want, got
    hk.debug_option("MXFP6_FORCE_CFG", None)
    # (ii) a 64-bit checksum of the whole gathered C, equal on all ranks
    def digest(c):
        acc = torch.zeros((), dtype=torch.int64, device=device)
        w = torch.arange(1, c.shape[1] + 1, device=device, dtype=torch.int64)
        for r0 in range(0, c.shape[0], 1024):
            blk = c[r0:r0 + 1024].view(torch.int16).to(torch.int64)
            acc += (blk * w).sum() * (1 + r0 // 1024)
        return acc
    d_fused = digest(c_full)
    all_d = [torch.zeros_like(d_fused) for _ in range(world)]
    dist.all_gather(all_d, d_fused)
    ranks_equal = all(int(x) == int(all_d[0]) for x in all_d)
    # (iv) the NCCL all-gather + re-layout exchange gives the same matrix
    nccl_equal = None
    others_equal = True
    # the overlapped exchange that was not timed: same matrix, and its time for the record (on up to 4 GPUs, where it has
    # been run before: this leg must not put the line of a larger run at risk)
    if op.mode in ("fused", "copy") and world <= 4:
        other_mode = "copy" if op.mode == "fused" else "fused"
        try:
            other = ColumnParallelGemm(M, N, K, device=device, gather=other_mode)
            built = 1
        except Exception as e:
            other, built = None, 0
            print(f"[bench] gather={other_mode} unavailable ({e!r})", file=sys.stderr)
        t_built = torch.tensor([built], device=device)
        dist.all_reduce(t_built, op=dist.ReduceOp.MIN)      # every rank or none
        if int(t_built) == 1 and other.mode == other_mode:
            c_o = other(a, sa, b, sb)
            torch.cuda.synchronize()
            others_equal = int(digest(c_o)) == int(d_fused)
            del c_o
            for _ in range(2):
                other(a, sa, b, sb)
            barrier()
            e0.record()
            for _ in range(3):
                other(a, sa, b, sb)
            e1.record()
            barrier()
            t = torch.tensor([e0.elapsed_time(e1) / 3], device=device)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            probe_ms[other_mode] = float(t)
        del other
        torch.cuda.empty_cache()
    if op.mode in ("fused", "copy"):
        op2 = ColumnParallelGemm(M, N, K, device=device, gather="nccl")
        c2 = op2(a, sa, b, sb)
        torch.cuda.synchronize()
        nccl_equal = int(digest(c2)) == int(d_fused)
        # exchange time of the baseline, for the record
        e0.record()
        for _ in range(3):
            op2(a, sa, b, sb)
        e1.record()
        barrier()
        nccl_ms = e0.elapsed_time(e1) / 3
        del op2, c2
        torch.cuda.empty_cache()
    flags = torch.tensor([int(rows_equal), int(ranks_equal), int(nccl_equal is not False and others_equal),
                          int(rank != 0 or (oracle["row_rel"] <= 1e-2 and oracle["max_ulp"] <= 2.0))], device=device)
    dist.all_reduce(flags, op=dist.ReduceOp.MIN)
    flags = [bool(x) for x in flags.cpu()]
    check = {"ok": all(flags), "rows_equal_single_gpu_kernel": flags[0], "ranks_equal": flags[1],
             "fused_equals_nccl_gather": flags[2] if nccl_equal is not None else None, "oracle_ok": flags[3],
             "rows": n_rows, "oracle_rows": n_oracle, "row_rel": float(f"{oracle['row_rel']:.3e}"), "max_ulp": round(oracle["max_ulp"], 3),
             "n_floor": oracle["n_floor"],
             "how": "every rank: 64 full rows of the gathered C bit for bit against the single-GPU kernel on regenerated shards; "
                    "64-bit checksum of the whole C all-gathered and compared; the epilogue-push, copy-engine and NCCL exchanges compared; rank 0: 16 rows "
                    "against the fp64 CPU oracle (row_rel <= 1e-2, <= 2 bf16 ulp)"}

    # ---- the whole problem on one GPU (rank 0's clock; the other ranks wait): the strong-scaling baseline
    single_ms = None
    if rank == 0:
        bs = [make_operands(torch, hk, per, K, "normal", 100 + r, device) for r in range(world)]
        b_all = torch.cat([x[0] for x in bs]); sb_all = torch.cat([x[1] for x in bs])
        del bs
        c_one = torch.empty((M, N), dtype=torch.bfloat16, device=device)
        for _ in range(3):
            hk.dispatch_micro(a, b_all, c_one, sa, sb_all, hk.E2M3)
        torch.cuda.synchronize()
        e0.record()
        for _ in range(10):
            hk.dispatch_micro(a, b_all, c_one, sa, sb_all, hk.E2M3)
        e1.record()
        torch.cuda.synchronize()
        single_ms = e0.elapsed_time(e1) / 10
        del b_all, sb_all, c_one
        torch.cuda.empty_cache()
    dist.barrier()

    # ---- end to end: operands start in pinned host memory, this rank's block of the result ends in pinned host memory
    host_in = [t.cpu().pin_memory() for t in (a, sa, b, sb)]
    host_out = torch.empty((M, per), dtype=torch.bfloat16).pin_memory()
    h2d = sum(t.numel() * t.element_size() for t in host_in)
    d2h = host_out.numel() * host_out.element_size()

    def sharded_step(s):
        op(s["a"], s["sa"], s["b"], s["sb"])
        return op.c_shard
    pipe = hk.HostGemm(M, per, K, device=device, gemm=sharded_step)
    for _ in range(3):
        pipe(host_in[0], host_in[1], host_in[2], host_in[3], host_out)
    pipe.synchronize()
    barrier()
    n_e2e = min(K_steps, 20)
    e0.record()
    for _ in range(n_e2e):
        pipe(host_in[0], host_in[1], host_in[2], host_in[3], host_out)
    pipe.synchronize()
    e1.record()
    barrier()
    ms_e2e = e0.elapsed_time(e1) / n_e2e

    t = torch.tensor([ms_total, ms_e2e, kernel_ms], device=device, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_total, ms_e2e, kernel_ms = (float(x) for x in t.cpu())
    assert hk.device_status() == 0

    if rank == 0:
        ms_step = ms_total / K_steps
        value = flops_step / (ms_step * 1e-3) / 1e12
        e2e_val = flops_step / (ms_e2e * 1e-3) / 1e12
        flops_launch = 2.0 * M * per * K
        achieved = flops_launch / (kernel_ms * 1e-3) / 1e12
        tp = tensor_peaks(peaks, ms_total * 1e-3)
        ingress = (world - 1) / world * 2.0 * M * N / (ms_step * 1e-3) / 1e9
        line = {
            "metric": METRIC, "value": round(value, 2), "unit": UNIT, "n_gpus": world, "steps": K_steps, "warmup": W,
            "ms_per_step": round(ms_step, 5), "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "fp6_e2m3xfp6_e2m3->f32->bf16", "data": "synthetic",
            "config": {"workload": f"mxfp6_e2m3_gemm_{M}x{N}x{K}_colparallel_gather", "M": M, "N": N, "K": K, "format": "e2m3",
                       "scale": "e8m0 per 32 along K"},
            "notes": {"l2": "A + B shard + C exceed L2",
                      "parallelism": f"column-parallel x{world}, " + {
                          "fused": "C tiles pushed to peers by the GEMM epilogue (symmetric memory, two alternating C buffers)",
                          "copy": "finished blocks of C carried to the peers by the copy engines behind per-block flags the GEMM "
                                  "raises (symmetric memory, two alternating C buffers)",
                          "nccl": "nccl all-gather of C"}[op.mode],
                      "workload_vs_n1": "the N=1 line of this benchmark times 8192^3; single_gpu_same_workload_ms below is this "
                                        "configuration's own one-GPU time"},
            "e2e": {"value": round(e2e_val, 2), "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
            "gpu_launches": K_steps,
            "clocks": clocks,
            "roofline": {"bound": "tensor", "achieved": round(achieved, 2), "peak": round(tp["peak"], 1), "unit": "TFLOP/s",
                         "frac": round(achieved / tp["peak"], 4), "traffic": None, "peak_source": tp["source"],
                         "kernel_ms": round(kernel_ms, 5), "frac_of_burst_peak": round(achieved / tp["burst"], 4),
                         "frac_of_sustained_peak": round(achieved / tp["sustained"], 4),
                         "frac_of_datasheet_4500": round(achieved / DATASHEET_TFLOPS, 4),
                         "algorithmic_bytes": algorithmic_bytes(M, per, K)},
            "check": check,
            "single_gpu_same_workload_ms": round(single_ms, 4),
            "strong_scaling_efficiency": round(single_ms / (world * ms_step), 4),
            "gemm_only_efficiency": round(single_ms / (world * kernel_ms), 4),
            "nvlink_ingress_gbs": round(ingress, 1),
            "nvlink_ingress_frac_of_770": round(ingress / 770.0, 4),
            "gather": {"timed": op.mode, "other_ms_per_step": {m: round(v, 4) for m, v in probe_ms.items()},
                       "how": "the exchange named by --gather is timed; the other overlapped exchange runs 3 steps after the timed "
                              "region (max over ranks), for the record"},
            "nccl_gather_ms_per_step": round(nccl_ms, 4) if op.mode in ("fused", "copy") else None,
        }
        print(json.dumps(line), flush=True)
    dist.barrier()
    dist.destroy_process_group()
    if not check["ok"]:
        raise SystemExit(3)


def run_native(args):
    import torch

    import hipkittensp_b200 as hk

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.gpus > 1 and world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} needs torchrun with {args.gpus} ranks (WORLD_SIZE={world})")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    peaks = {}
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            peaks = json.load(f)
    except Exception:
        pass
    if world == 1:
        run_single(args, torch, hk, device, peaks)
    else:
        import torch.distributed as dist

        dist.init_process_group("nccl", device_id=device)
        run_sharded(args, torch, hk, device, peaks, world, rank)


# ------------------------------------------------------------------------------------------ CPU path
def cpu_baseline(operands, M, N, K, budget_s):
    """Times the oracle's dequantise-then-matmul path on the host cores for a bounded sample of the workload:
    the first `rows` rows of A against all of B (both dequantised inside the timed region)."""
    import torch

    from oracle import mxfp6_ref as R

    a, sa, b, sb = operands
    torch.set_num_threads(os.cpu_count() or 1)
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
    """The reference arm: the CPU dequantise-then-matmul path on this box's host cores, all of them (a launcher that
    sets OMP_NUM_THREADS=1 for its ranks is overridden: this arm runs on rank 0 alone)."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    ncpu = os.cpu_count() or 1
    os.environ["OMP_NUM_THREADS"] = str(ncpu)
    os.environ["MKL_NUM_THREADS"] = str(ncpu)
    import numpy as np
    import torch

    from oracle import mxfp6_ref as R

    torch.set_num_threads(ncpu)
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
    whole = rows == M and rows_b == N
    sample = (("the whole workload per step" if whole else
               f"a sample of the workload per step: {rows} of its {M} rows of A x {rows_b} of its {N} rows of B, full K={K}")
              + " (dequantise both + fp32 matmul + bf16 round); TFLOP/s counts the sample's own flops")
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
