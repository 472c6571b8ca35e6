"""Benchmark and check harness for `dispatch_micro`, in the protocol of the reference's own harness.

The reference times its GEMM operator with `bench_gemm` (kernels/gemm/bf16fp32/utils.py:20-54, driven by
kernels/gemm/bf16fp32/bench.py:9-35): many untimed calls first, then per timed iteration fresh random operands, a
device synchronise, one call between two CUDA events, another synchronise; the mean of the per-call times gives
"m=..,n=..,k=..: T TFLOPS".  Its check script (kernels/gemm/bf16fp32/test.py:30-40) runs the operator once on random
operands and compares with a PyTorch product.  This module does both for the MX-FP6 operator: operands are drawn
on the GPU, block-quantised by the library's quantiser, and the check dequantises them with the library's
dequantiser and multiplies in fp32 with torch (a GPU-side check for quick use; the parity tests proper compare
with the CPU oracle).

    python -m hipkittensp_b200.harness                 # the reference's shape list, E2M3
    python -m hipkittensp_b200.harness --check         # asserting run on a few shapes
    python -m hipkittensp_b200.harness --quantize      # GB/s of the block quantiser
    python -m hipkittensp_b200.harness --edge          # shapes off the preferred multiples (odd K, unaligned N)
"""
from __future__ import annotations

import argparse
import os
import sys

import torch

from . import _lib as F
from .gemm import dequantize, device_status, quantize

try:        # the compiled binding, as the reference's harness uses (`import tk_kernel`); it sits beside this file
    sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
    from tk_kernel import dispatch_micro
except ImportError:
    from .gemm import dispatch_micro
finally:
    sys.path.pop(0)

# shapes of the reference's sweep (kernels/gemm/bf16fp32/bench.py:9-18), (m, n, k)
BENCH_SHAPES = [(8192, 8192, 8192), (4096, 8192, 2048), (8192, 4096, 2048), (8192, 2048, 4096),
                (4096, 4096, 4096), (2048, 4096, 4096), (2048, 2048, 4096), (2048, 2048, 2048)]


# Shapes off the fast path's preferred multiples, to show what they cost: K / 32 not a multiple of 16 (scale rows that
# cannot be TMA boxes), a Llama-2 FFN width (11008 = 21.5 x 512), an N whose rows are not 16-byte multiples
EDGE_SHAPES = [(8192, 8192, 8192 + 128), (8192, 8192, 8192 - 128), (4096, 11008, 4096), (4096, 4096, 11008),
               (8192, 8196, 8192), (4096, 4096, 4096)]


def print_title(title: str, width: int = 30) -> None:
    print("-" * width)
    print(title)
    print("-" * width)


def _fresh_operands(m: int, n: int, k: int, fmt: int, device):
    a = torch.randn((m, k), dtype=torch.bfloat16, device=device)
    b = torch.randn((n, k), dtype=torch.bfloat16, device=device)
    pa, sa = quantize(a, fmt)
    pb, sb = quantize(b, fmt)
    return pa, sa, pb, sb


def bench_gemm(gemm_params: dict, gemm_func=None, num_warmup: int = 500, num_iter: int = 500) -> float:
    """Mean TFLOP/s of gemm_func(A, B, C, scale_A, scale_B, fmt) over num_iter single calls, each on operands drawn
    and quantised just before it (so nothing of them is cached from the previous call)."""
    m, n, k = gemm_params["shape"]
    fmt = gemm_params.get("fmt", F.E2M3)
    device = gemm_params.get("device", "cuda:0")
    gemm_func = gemm_func or dispatch_micro
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    pa, sa, pb, sb = _fresh_operands(m, n, k, fmt, device)
    c = torch.empty((m, n), dtype=torch.bfloat16, device=device)
    for _ in range(num_warmup):
        gemm_func(pa, pb, c, sa, sb, fmt)
    total_ms = 0.0
    for _ in range(num_iter):
        pa, sa, pb, sb = _fresh_operands(m, n, k, fmt, device)
        c = torch.empty((m, n), dtype=torch.bfloat16, device=device)
        torch.cuda.synchronize()
        start.record()
        gemm_func(pa, pb, c, sa, sb, fmt)
        end.record()
        torch.cuda.synchronize()
        total_ms += start.elapsed_time(end)
    if device_status() != 0:
        raise RuntimeError("a kernel reported a device-side wait that ran out")
    tflops = 2.0 * m * n * k / (total_ms / num_iter * 1e9)
    print(f"m={m},n={n},k={k}: {tflops:.0f} TFLOPS")
    return tflops


def check_gemm(shape, fmt: int = F.E2M3, device="cuda:0", rel_tol: float = 1e-2) -> float:
    """One call on random operands against dequantise-then-matmul in fp32 on the GPU; asserts the reference's
    criterion (max |C - ref| over the row's L2 norm <= 1e-2) and returns the value."""
    m, n, k = shape
    pa, sa, pb, sb = _fresh_operands(m, n, k, fmt, device)
    c = torch.empty((m, n), dtype=torch.bfloat16, device=device)
    dispatch_micro(pa, pb, c, sa, sb, fmt)
    ref = dequantize(pa, sa, fmt) @ dequantize(pb, sb, fmt).T
    if device_status() != 0:
        raise RuntimeError("a kernel reported a device-side wait that ran out")
    err = ((c.float() - ref).abs().amax(dim=1) / ref.norm(dim=1).clamp_min(1e-30)).max().item()
    print(f"m={m},n={n},k={k}: max row-relative error {err:.3e}")
    assert err <= rel_tol, f"row-relative error {err} above {rel_tol}"
    return err


def bench_quantize(rows: int = 8192, K: int = 8192, fmt: int = F.E2M3, device="cuda:0", iters: int = 20) -> dict:
    """GB/s of the block quantiser (the step in front of the GEMM) for fp32 and bf16 sources: algorithmic bytes
    (source read once, codes and scale bytes written once) over the mean time of `iters` back-to-back launches."""
    out = {}
    for name, dtype in (("fp32", torch.float32), ("bf16", torch.bfloat16)):
        x = torch.randn((rows, K), dtype=torch.float32, device=device).to(dtype)
        for _ in range(3):
            p, s = quantize(x, fmt)
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        start.record()
        for _ in range(iters):
            p, s = quantize(x, fmt)
        end.record()
        torch.cuda.synchronize()
        us = start.elapsed_time(end) / iters * 1e3
        nbytes = x.numel() * x.element_size() + p.numel() + s.numel()
        out[name] = nbytes / us / 1e3
        print(f"quantize {name} [{rows},{K}] -> fmt {fmt}: {us:.1f} us, {out[name]:.0f} GB/s")
    if device_status() != 0:
        raise RuntimeError("a kernel reported a device-side wait that ran out")
    return out


def main(argv=None) -> None:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--check", action="store_true", help="asserting run instead of the timing sweep")
    ap.add_argument("--quantize", action="store_true", help="time the block quantiser instead of the GEMM")
    ap.add_argument("--edge", action="store_true", help="time shapes off the preferred multiples instead of the reference's list")
    ap.add_argument("--fmt", choices=["e2m3", "e3m2", "e4m3", "e5m2"], default="e2m3")
    ap.add_argument("--warmup", type=int, default=500)
    ap.add_argument("--iters", type=int, default=500)
    args = ap.parse_args(argv)
    fmt = {"e2m3": F.E2M3, "e3m2": F.E3M2, "e4m3": F.E4M3, "e5m2": F.E5M2}[args.fmt]
    torch.manual_seed(0)
    if args.quantize:
        print_title(f"MX {args.fmt} block quantiser (B200)")
        bench_quantize(fmt=fmt, iters=args.iters if args.iters != 500 else 20)
        return
    if args.check:
        print_title(f"MX {args.fmt} GEMM check")
        for shape in [(1024, 1024, 1024), (130, 200, 256), (16, 4096, 2048), (2048, 2048, 2048)]:
            check_gemm(shape, fmt)
        return
    print_title(f"MX {args.fmt} GEMM (B200)")
    for shape in (EDGE_SHAPES if args.edge else BENCH_SHAPES):
        bench_gemm({"shape": shape, "fmt": fmt}, None, args.warmup, args.iters)


if __name__ == "__main__":
    main()
