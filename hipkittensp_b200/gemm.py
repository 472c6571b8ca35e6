"""Host-side mirror of the reference's operator for the MX-FP6 GEMM path.

`dispatch_micro(A, B, C, scale_A, scale_B, fmt)` keeps the reference's calling convention
(kernels/gemm/bf16fp32/bench.py:34: positional tensors, output written in place, returns None;
scale tensors after C as in kernels/torch_scaled/scaled_matmul.cu:17-18) and its tensor-acceptance
errors (include/pyutils/pyutils.cuh:18-44), and forwards to the C ABI on torch's current stream.
torch is used for device memory and streams only.
"""
from __future__ import annotations

import torch

from . import _lib
from ._lib import E2M3, E3M2, E4M3, E5M2, check, lib


def _accept(t, name: str, dtype) -> None:
    if not isinstance(t, torch.Tensor):
        raise RuntimeError("Expected a torch.Tensor")
    if not t.is_contiguous():
        raise RuntimeError("Tensor must be contiguous")
    if t.device.type == "cpu":
        raise RuntimeError("Tensor must be on CUDA device")
    if t.dim() > 4:
        raise RuntimeError("Expected Tensor.ndim <= 4")
    if t.dtype != dtype:
        raise RuntimeError(f"{name} must be {dtype}, got {t.dtype}")
    if t.dim() != 2:
        raise RuntimeError(f"{name} must be 2-D")


def _k_of(t, fmt: int, name: str) -> int:
    """K of an operand [rows, bytes]: 4 elements per 3 bytes for fp6, 1 per byte for fp8."""
    if fmt in (E4M3, E5M2):
        return t.shape[1]
    if t.shape[1] % 3:
        raise RuntimeError(f"{name}.shape[1] must be 3K/4 bytes")
    return t.shape[1] // 3 * 4


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream_ptr() -> int:
    """Handle of torch's current stream on the current device."""
    if _raw_stream is not None:
        return _raw_stream(torch.cuda.current_device())
    return torch.cuda.current_stream().cuda_stream


class _NoGuard:
    def __enter__(self):
        return None

    def __exit__(self, *exc):
        return False


_NO_GUARD = _NoGuard()


def _on_device_of(t):
    """Context that makes t's device current; free when it already is (the common case)."""
    if t.device.index == torch.cuda.current_device():
        return _NO_GUARD
    return torch.cuda.device(t.device)


def dispatch_micro(A, B, C, scale_A, scale_B, fmt: int = E2M3, fmt_b: int | None = None, b_static: bool = False) -> None:
    """C[M,N] (bf16, in place) = A[M,K] @ B[N,K]^T.

    A [M,3K/4] u8 and B [N,3K/4] u8 are packed fp6, or [rows,K] u8 for the fp8 formats (format `fmt`; `fmt_b` if
    B differs),
    scale_A [M,K/32] u8 and scale_B [N,K/32] u8 are E8M0 bytes.  M is taken from A, N from C,
    K from A, as the reference does (256_256_64_32_with16x32.cpp:52-54).  b_static=True promises that B and
    scale_B are not written by the work queued just before this call (see MXFP6_FLAG_B_STATIC)."""
    _accept(A, "A", torch.uint8)
    _accept(B, "B", torch.uint8)
    _accept(C, "C", torch.bfloat16)
    _accept(scale_A, "scale_A", torch.uint8)
    _accept(scale_B, "scale_B", torch.uint8)
    M, N = A.shape[0], C.shape[1]
    fb = fmt if fmt_b is None else fmt_b
    K = _k_of(A, fmt, "A")
    if K % 128:
        raise RuntimeError("K must be a multiple of 128")
    if C.shape[0] != M:
        raise RuntimeError("C.shape[0] must equal A.shape[0]")
    if B.shape[0] != N or _k_of(B, fb, "B") != K:
        raise RuntimeError("B must be [N, 3K/4] (fp6) or [N, K] (fp8) with the K of A")
    if tuple(scale_A.shape) != (M, K // 32) or tuple(scale_B.shape) != (N, K // 32):
        raise RuntimeError("scales must be [rows, K/32]")
    if len({t.device for t in (A, B, C, scale_A, scale_B)}) != 1:
        raise RuntimeError("all tensors must be on the same device")
    with _on_device_of(A):
        check(lib.mxfp6_gemm_ex(A.data_ptr(), scale_A.data_ptr(), B.data_ptr(), scale_B.data_ptr(), C.data_ptr(),
                                M, N, K, fmt, fb, _lib.FLAG_B_STATIC if b_static else 0, _stream_ptr()))


def dispatch_multi(A, B, dests, col_offset: int, scale_A, scale_B, fmt: int = E2M3) -> None:
    """The [M,N] product written into the column window [col_offset, col_offset+N) of every matrix in `dests`.

    dests: bf16 tensors [M, ldc] that share one row stride; dests[0] is local, the others may be views of
    peer GPUs' memory (symmetric memory): the kernel's epilogue pushes each finished tile to all of them."""
    import ctypes

    _accept(A, "A", torch.uint8)
    _accept(B, "B", torch.uint8)
    _accept(scale_A, "scale_A", torch.uint8)
    _accept(scale_B, "scale_B", torch.uint8)
    M, N = A.shape[0], B.shape[0]
    K = _k_of(A, fmt, "A")
    if not 1 <= len(dests) <= 8:
        raise RuntimeError("1 to 8 destinations")
    ldc = dests[0].stride(0)
    for d in dests:
        if d.dtype != torch.bfloat16 or d.dim() != 2 or d.stride(1) != 1 or d.stride(0) != ldc or d.shape[0] != M:
            raise RuntimeError("destinations must be bf16 [M, ldc] matrices with one common row stride")
        if col_offset < 0 or col_offset + N > d.shape[1]:
            raise RuntimeError("column window outside the destination")
    ptrs = (ctypes.c_void_p * len(dests))(*[d.data_ptr() + 2 * col_offset for d in dests])
    with _on_device_of(A):
        check(lib.mxfp6_gemm_multi(A.data_ptr(), scale_A.data_ptr(), B.data_ptr(), scale_B.data_ptr(), ptrs, len(dests),
                                   ldc, M, N, K, fmt, fmt, _stream_ptr()))


def copy_gather_scratch_bytes(M: int, N: int, strip_tiles: int) -> int:
    """Bytes of device scratch `dispatch_copy_gather` needs for an [M, N] block."""
    return int(lib.mxfp6_copy_gather_scratch_bytes(M, N, strip_tiles))


def dispatch_copy_gather(A, B, dests, col_offset: int, scale_A, scale_B, scratch, copy_streams, strip_tiles: int = 8,
                         fmt: int = E2M3) -> None:
    """`dispatch_multi` with the peers served by the copy engines: the kernel writes dests[0] only and raises a flag per
    finished block of C; `copy_streams` (torch streams, a multiple of len(dests) - 1) wait for the flags and copy the
    blocks to the peers.  Work queued on the current stream after the call sees all copies done."""
    import ctypes

    _accept(A, "A", torch.uint8)
    _accept(B, "B", torch.uint8)
    _accept(scale_A, "scale_A", torch.uint8)
    _accept(scale_B, "scale_B", torch.uint8)
    M, N = A.shape[0], B.shape[0]
    K = _k_of(A, fmt, "A")
    if not 1 <= len(dests) <= 8:
        raise RuntimeError("1 to 8 destinations")
    ldc = dests[0].stride(0)
    for d in dests:
        if d.dtype != torch.bfloat16 or d.dim() != 2 or d.stride(1) != 1 or d.stride(0) != ldc or d.shape[0] != M:
            raise RuntimeError("destinations must be bf16 [M, ldc] matrices with one common row stride")
        if col_offset < 0 or col_offset + N > d.shape[1]:
            raise RuntimeError("column window outside the destination")
    if scratch.device != A.device or not scratch.is_contiguous():
        raise RuntimeError("scratch must be a contiguous tensor on the operands' device")
    ptrs = (ctypes.c_void_p * len(dests))(*[d.data_ptr() + 2 * col_offset for d in dests])
    streams = (ctypes.c_void_p * max(len(copy_streams), 1))(*[s.cuda_stream for s in copy_streams])
    with _on_device_of(A):
        check(lib.mxfp6_gemm_copy_gather(A.data_ptr(), scale_A.data_ptr(), B.data_ptr(), scale_B.data_ptr(), ptrs, len(dests),
                                         ldc, M, N, K, fmt, fmt, scratch.data_ptr(), scratch.numel() * scratch.element_size(),
                                         strip_tiles, streams, len(copy_streams), _stream_ptr()))


def gemm_requant(A, scale_A, B, scale_B, fmt: int = E2M3, fmt_b: int | None = None, out_fmt: int = E2M3):
    """C = A @ B^T delivered as an MX operand for the next layer: (operand bytes [M, 3N/4 | N], scales [M, N/32]),
    quantised in the GEMM epilogue from the fp32 accumulators (blocks of 32 along N)."""
    _accept(A, "A", torch.uint8)
    _accept(B, "B", torch.uint8)
    _accept(scale_A, "scale_A", torch.uint8)
    _accept(scale_B, "scale_B", torch.uint8)
    fb = fmt if fmt_b is None else fmt_b
    M, N, K = A.shape[0], B.shape[0], _k_of(A, fmt, "A")
    if _k_of(B, fb, "B") != K:
        raise RuntimeError("A and B disagree on K")
    if N % 64:
        raise RuntimeError("N must be a multiple of 64")
    out = torch.empty((M, N if out_fmt in (E4M3, E5M2) else N * 3 // 4), dtype=torch.uint8, device=A.device)
    scales = torch.empty((M, N // 32), dtype=torch.uint8, device=A.device)
    with _on_device_of(A):
        check(lib.mxfp6_gemm_requant(A.data_ptr(), scale_A.data_ptr(), B.data_ptr(), scale_B.data_ptr(), out.data_ptr(),
                                     scales.data_ptr(), M, N, K, fmt, fb, out_fmt, _stream_ptr()))
    return out, scales


def gemm_scaled(A, scale_A, B, scale_B, row_scale=None, col_scale=None, bias=None, fmt: int = E2M3,
                fmt_b: int | None = None, out=None):
    """C[m,n] = bf16((acc[m,n] * col_scale[n]) * row_scale[m] + bias[n]) with fp32 vectors row_scale [M], col_scale [N],
    bias [N] (any may be None), applied in the GEMM epilogue: the per-row / per-column scaling of the reference's
    scaled_matmul (kernels/torch_scaled/scaled_matmul.cu:253-265) on top of the MX block scales."""
    _accept(A, "A", torch.uint8)
    _accept(B, "B", torch.uint8)
    _accept(scale_A, "scale_A", torch.uint8)
    _accept(scale_B, "scale_B", torch.uint8)
    fb = fmt if fmt_b is None else fmt_b
    M, N, K = A.shape[0], B.shape[0], _k_of(A, fmt, "A")
    if _k_of(B, fb, "B") != K:
        raise RuntimeError("A and B disagree on K")
    for name, v, n in (("row_scale", row_scale, M), ("col_scale", col_scale, N), ("bias", bias, N)):
        if v is not None:
            if not isinstance(v, torch.Tensor) or v.dtype != torch.float32 or not v.is_contiguous():
                raise RuntimeError(f"{name} must be a contiguous fp32 tensor")
            if v.device != A.device:
                raise RuntimeError("Tensor must be on CUDA device")
            if v.numel() != n:
                raise RuntimeError(f"{name} must have {n} elements, has {v.numel()}")
    if out is None:
        out = torch.empty((M, N), dtype=torch.bfloat16, device=A.device)
    _accept(out, "C", torch.bfloat16)
    if tuple(out.shape) != (M, N):
        raise RuntimeError(f"C must be [{M}, {N}]")
    ptr = lambda v: 0 if v is None else v.data_ptr()
    with _on_device_of(A):
        check(lib.mxfp6_gemm_scaled(A.data_ptr(), scale_A.data_ptr(), B.data_ptr(), scale_B.data_ptr(), out.data_ptr(),
                                    ptr(row_scale), ptr(col_scale), ptr(bias), M, N, K, fmt, fb, _stream_ptr()))
    return out


def gemm(A, scale_A, B, scale_B, fmt: int = E2M3, fmt_b: int | None = None, out=None):
    """Allocating convenience wrapper around dispatch_micro; returns C."""
    M, N = A.shape[0], B.shape[0]
    if out is None:
        out = torch.empty((M, N), dtype=torch.bfloat16, device=A.device)
    dispatch_micro(A, B, out, scale_A, scale_B, fmt, fmt_b)
    return out


def quantize(x: torch.Tensor, fmt: int = E2M3):
    """fp32 or bf16 [rows,K] on the GPU -> (operand bytes u8 [rows,3K/4] for fp6 / [rows,K] for fp8, scales u8 [rows,K/32])."""
    if x.device.type == "cpu":
        raise RuntimeError("Tensor must be on CUDA device")
    if x.dtype not in (torch.float32, torch.bfloat16) or x.dim() != 2 or not x.is_contiguous():
        raise RuntimeError("quantize expects a contiguous 2-D fp32 or bf16 tensor")
    rows, K = x.shape
    if K % 32:
        raise RuntimeError("K must be a multiple of 32")
    packed = torch.empty((rows, K if fmt in (E4M3, E5M2) else K * 3 // 4), dtype=torch.uint8, device=x.device)
    scales = torch.empty((rows, K // 32), dtype=torch.uint8, device=x.device)
    with _on_device_of(x):
        check(lib.mxfp6_quantize(x.data_ptr(), 0 if x.dtype == torch.float32 else 1, rows, K, fmt,
                                 packed.data_ptr(), scales.data_ptr(), _stream_ptr()))
    return packed, scales


def dequantize(packed: torch.Tensor, scales: torch.Tensor, fmt: int = E2M3) -> torch.Tensor:
    """(packed, scales) on the GPU -> fp32 [rows,K]."""
    _accept(packed, "packed", torch.uint8)
    _accept(scales, "scales", torch.uint8)
    rows, K = packed.shape[0], _k_of(packed, fmt, "packed")
    out = torch.empty((rows, K), dtype=torch.float32, device=packed.device)
    with _on_device_of(packed):
        check(lib.mxfp6_dequantize(packed.data_ptr(), scales.data_ptr(), rows, K, fmt, out.data_ptr(), _stream_ptr()))
    return out


def device_status() -> int:
    """Synchronise and return the device status word (0 = ok); raises if a kernel wait ran out."""
    import ctypes

    st = ctypes.c_int(0)
    check(lib.mxfp6_device_status(ctypes.byref(st)))
    return st.value


def tma_dump(packed: torch.Tensor, row0: int = 0, k0: int = 0) -> torch.Tensor:
    """Diagnostic: the 16 KiB shared-memory image of one 128x128 operand box as the GEMM loads it."""
    rows, K = packed.shape[0], packed.shape[1] // 3 * 4
    out = torch.empty(16384, dtype=torch.uint8, device=packed.device)
    with _on_device_of(packed):
        check(lib.mxfp6_debug_tma_dump(packed.data_ptr(), rows, K, row0, k0, out.data_ptr(), _stream_ptr()))
    return out
