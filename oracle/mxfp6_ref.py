"""CPU oracle for the MX-FP6 GEMM path (numpy + torch on CPU).  TEST INFRASTRUCTURE ONLY.

Only tests, the smoke check and the CPU-baseline leg of the benchmark may import this module;
the shipped package never does.

PARITY UNPINNED against the reference: its tree holds no fp6 source, test or golden vector
(kernels/gemm/README.md:6-7).  The format follows the OCP MX v1.0 definitions and is pinned
against the CUDA toolkit host conversions (tests/golden/toolkit_fp6_kat.json) and
torch.float8_e8m0fnu.  The computation's shape follows the reference:
  * C = A @ B^T with K-contiguous operands   (kernels/gemm/bf16fp32/bench.py:34, utils.py:20-54)
  * fp32 accumulate, single RNE rounding to bf16 (kernels/gemm/fp8fp32/FP8_8wave/8_wave.cu:451-460)
  * the comparison style (count of |d| > 0.01*|ref|) follows
    analysis/bf16_gemm/mi350x/test_python.py:104-113.

This is the second, independent statement of the format (vectorised numpy); mxfp6_oracle.c is the
first (scalar C).  tests/test_oracle.py checks that the two agree bit for bit.
"""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

E2M3 = 0
E3M2 = 1
E4M3 = 2   # MX-FP8, OCP e4m3 ("fn": no infinities, 0x7f/0xff are NaN), one byte per element
E5M2 = 3   # MX-FP8, OCP e5m2 (IEEE-like: exponent 31 is inf/nan), one byte per element

# bits = container width; ncodes = finite non-negative codes (they ascend with the value, so the index of a
# magnitude in the table of finite magnitudes is its code)
_FMT = {
    E2M3: dict(bits=6, mbits=3, bias=1, emax=2, maxv=7.5, nfinite=32),
    E3M2: dict(bits=6, mbits=2, bias=3, emax=4, maxv=28.0, nfinite=32),
    E4M3: dict(bits=8, mbits=3, bias=7, emax=8, maxv=448.0, nfinite=127),
    E5M2: dict(bits=8, mbits=2, bias=15, emax=15, maxv=57344.0, nfinite=124),
}


def is_fp8(fmt: int) -> bool:
    return _FMT[fmt]["bits"] == 8


# --------------------------------------------------------------------------- tables
def decode_table(fmt: int) -> np.ndarray:
    """All 64 (fp6) or 256 (fp8) code -> fp32 values; fp8 NaN/inf codes decode to nan/inf."""
    p = _FMT[fmt]
    mb, bias, bits = p["mbits"], p["bias"], p["bits"]
    eb = bits - 1 - mb
    c = np.arange(1 << bits, dtype=np.int64)
    s = (c >> (bits - 1)) & 1
    e = (c >> mb) & ((1 << eb) - 1)
    m = c & ((1 << mb) - 1)
    mag = np.where(e == 0, m * 2.0 ** (1 - bias - mb), ((1 << mb) + m) * 2.0 ** (e - bias - mb))
    if fmt == E4M3:
        mag = np.where((e == 15) & (m == 7), np.nan, mag)
    if fmt == E5M2:
        mag = np.where(e == 31, np.where(m == 0, np.inf, np.nan), mag)
    return np.where(s == 1, -mag, mag).astype(np.float32)


def e8m0_decode(b: np.ndarray) -> np.ndarray:
    """byte -> 2^(byte-127) as fp32 (0xFF -> nan)."""
    b = np.asarray(b, dtype=np.uint8)
    with np.errstate(over="ignore"):
        out = np.ldexp(np.float32(1.0), b.astype(np.int32) - 127).astype(np.float32)
    return np.where(b == 255, np.float32(np.nan), out)


# --------------------------------------------------------------------------- element encode
def encode_elems(v: np.ndarray, fmt: int) -> np.ndarray:
    """fp32 (already divided by the block scale) -> codes, RNE + saturate to the largest finite value."""
    p = _FMT[fmt]
    maxv, nfin, bits = p["maxv"], p["nfinite"], p["bits"]
    v = np.asarray(v, dtype=np.float32)
    sign = ((v.view(np.uint32) >> 31).astype(np.uint8) << (bits - 1)).astype(np.uint8)
    a = np.abs(v).astype(np.float64)
    # finite non-negative magnitudes, ascending (index == code)
    grid = decode_table(fmt)[:nfin].astype(np.float64)
    # nearest grid point with ties to even code (even code == even mantissa lsb)
    idx_hi = np.searchsorted(grid, a, side="left").clip(0, nfin - 1)
    idx_lo = (idx_hi - 1).clip(0, nfin - 1)
    d_hi = np.abs(grid[idx_hi] - a)
    d_lo = np.abs(a - grid[idx_lo])
    pick_lo = (d_lo < d_hi) | ((d_lo == d_hi) & (idx_lo % 2 == 0))
    code = np.where(pick_lo, idx_lo, idx_hi).astype(np.uint8)
    code = np.where(a >= maxv, nfin - 1, code).astype(np.uint8)
    code = np.where(np.isnan(a), nfin - 1, code).astype(np.uint8)
    return (sign | code).astype(np.uint8)  # the sign of zero is kept (toolkit / hardware cvt behaviour)


def scale_bytes_from_amax(amax: np.ndarray, fmt: int) -> np.ndarray:
    """E8M0 byte = clamp(floor(log2(amax)) - emax_elem + 127, 0, 254); amax == 0 -> 0."""
    amax = np.asarray(amax, dtype=np.float32)
    _, ex = np.frexp(amax.astype(np.float64))  # amax = m * 2^ex, m in [0.5,1)  -> floor(log2) = ex-1
    e = ex.astype(np.int64) - 1 - _FMT[fmt]["emax"] + 127
    e = np.clip(e, 0, 254)
    e = np.where(amax > 0, e, 0)
    e = np.where(np.isinf(amax), 254, e)
    return e.astype(np.uint8)


# --------------------------------------------------------------------------- pack / unpack
def pack_codes(codes: np.ndarray) -> np.ndarray:
    """[..., K] uint8 codes -> [..., 3K/4] bytes, dense little-endian 6-bit stream."""
    codes = np.asarray(codes, dtype=np.uint8)
    assert codes.shape[-1] % 4 == 0
    c = codes.reshape(*codes.shape[:-1], -1, 4).astype(np.uint32) & 63
    w = c[..., 0] | (c[..., 1] << 6) | (c[..., 2] << 12) | (c[..., 3] << 18)
    out = np.stack([w & 255, (w >> 8) & 255, (w >> 16) & 255], axis=-1).astype(np.uint8)
    return out.reshape(*codes.shape[:-1], -1)


def unpack_codes(packed: np.ndarray) -> np.ndarray:
    """[..., 3K/4] bytes -> [..., K] uint8 codes."""
    packed = np.asarray(packed, dtype=np.uint8)
    assert packed.shape[-1] % 3 == 0
    b = packed.reshape(*packed.shape[:-1], -1, 3).astype(np.uint32)
    w = b[..., 0] | (b[..., 1] << 8) | (b[..., 2] << 16)
    out = np.stack([w & 63, (w >> 6) & 63, (w >> 12) & 63, (w >> 18) & 63], axis=-1).astype(np.uint8)
    return out.reshape(*packed.shape[:-1], -1)


# --------------------------------------------------------------------------- quantise / dequantise
def quantize(x: np.ndarray, fmt: int):
    """fp32 [rows,K] -> (packed uint8 [rows,3K/4] for fp6 or [rows,K] for fp8, scales uint8 [rows,K/32])."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    rows, K = x.shape
    assert K % 32 == 0
    xb = x.reshape(rows, K // 32, 32)
    amax = np.abs(xb).max(axis=-1)
    sb = scale_bytes_from_amax(amax, fmt)
    e = sb.astype(np.int32) - 127
    v = np.ldexp(xb.astype(np.float64), -e[..., None]).astype(np.float32)  # exact power-of-two scaling
    codes = encode_elems(v, fmt).reshape(rows, K)
    return (codes if is_fp8(fmt) else pack_codes(codes)), sb


def codes_of(packed: np.ndarray, fmt: int) -> np.ndarray:
    """Operand bytes -> one code per element."""
    return np.asarray(packed, dtype=np.uint8) if is_fp8(fmt) else unpack_codes(packed)


def dequantize(packed: np.ndarray, scales: np.ndarray, fmt: int) -> np.ndarray:
    """(operand bytes, scales [rows,K/32]) -> fp32 [rows,K]."""
    codes = codes_of(packed, fmt)
    rows, K = codes.shape
    vals = decode_table(fmt)[codes].reshape(rows, K // 32, 32)
    s = e8m0_decode(scales).reshape(rows, K // 32, 1)
    with np.errstate(over="ignore", invalid="ignore"):
        return (vals * s).reshape(rows, K).astype(np.float32)


def gemm_ref_torch(a_packed, sfa, b_packed, sfb, fmt_a=E2M3, fmt_b=None, threads=None, return_f32=False):
    """The dequantise-then-matmul path: fp32 dequantise, torch.matmul in fp32 on CPU, RNE to bf16.

    Returns a torch.bfloat16 tensor [M,N] (and the fp32 product if return_f32)."""
    import torch

    if fmt_b is None:
        fmt_b = fmt_a
    if threads:
        torch.set_num_threads(threads)
    A = torch.from_numpy(dequantize(np.asarray(a_packed), np.asarray(sfa), fmt_a))
    B = torch.from_numpy(dequantize(np.asarray(b_packed), np.asarray(sfb), fmt_b))
    C32 = A @ B.t()
    C = C32.to(torch.bfloat16)
    return (C, C32) if return_f32 else C


# --------------------------------------------------------------------------- synthetic inputs
def make_inputs(config: str, M: int, N: int, K: int, seed: int = 0):
    """Seeded fp32 operands with the value distributions of the benchmark configurations.

    config: 'normal'    A,B ~ N(0,1)
            'lognormal' per 32-block amplitude exp(N(0,1.5)) times N(0,1) values
            'ffn'       B ~ N(0,0.02); A ~ N(0,1) with 0.1 % of K channels scaled x50
            'decode'    B ~ N(0,0.02); A ~ N(0,1)
    """
    import torch

    g = torch.Generator(device="cpu").manual_seed(seed)

    def randn(*s):
        return torch.randn(*s, generator=g, dtype=torch.float32)

    if config == "normal":
        A, B = randn(M, K), randn(N, K)
    elif config == "lognormal":
        A = randn(M, K) * torch.exp(1.5 * randn(M, K // 32)).repeat_interleave(32, dim=1)
        B = randn(N, K) * torch.exp(1.5 * randn(N, K // 32)).repeat_interleave(32, dim=1)
    elif config == "ffn":
        A, B = randn(M, K), 0.02 * randn(N, K)
        n_out = max(1, K // 1000)
        ch = torch.randperm(K, generator=g)[:n_out]
        A[:, ch] *= 50.0
    elif config == "decode":
        A, B = randn(M, K), 0.02 * randn(N, K)
    else:
        raise ValueError(config)
    return A.numpy(), B.numpy()


# --------------------------------------------------------------------------- error metrics
def bf16_ulp(x: np.ndarray) -> np.ndarray:
    """Spacing of bf16 numbers at |x| (x fp32); the bf16 subnormal spacing below 2^-126."""
    _, ex = np.frexp(np.abs(x).astype(np.float64))
    ex = np.maximum(ex - 1, -126)
    return np.ldexp(1.0, ex - 7)


def error_report(c: np.ndarray, c_ref32: np.ndarray, absdot: np.ndarray | None = None) -> dict:
    """Error metrics of a bf16 result c (given as fp32 values) against an unrounded fp32 oracle.

    row_rel : max over rows of max_n |c-ref| / ||ref[r,:]||_2          (bound 1e-2)
    ulp     : max over elements of |c-ref| / ulp_bf16(ref), where elements whose error is inside
              the fp32 accumulation noise floor (2^-20 * sum_k|a_k b_k|) are excused; their number
              is reported as n_floor.
    n_1pct  : count of |c-ref| > 0.01*|ref| (the reference's printed statistic).
    """
    c = np.asarray(c, dtype=np.float64)
    r = np.asarray(c_ref32, dtype=np.float64)
    d = np.abs(c - r)
    norm = np.sqrt((r * r).sum(axis=1, keepdims=True))
    norm = np.where(norm == 0, 1.0, norm)
    row_rel = float((d / norm).max()) if d.size else 0.0
    ulp = d / bf16_ulp(r)
    if absdot is not None:
        floor = np.asarray(absdot, dtype=np.float64) * 2.0 ** -20
        excused = (ulp > 2.0) & (d <= floor + bf16_ulp(r))
        n_floor = int(excused.sum())
        ulp = np.where(excused, 0.0, ulp)
    else:
        n_floor = 0
    return dict(row_rel=row_rel, max_ulp=float(ulp.max()) if ulp.size else 0.0, n_floor=n_floor,
                n_1pct=int((d > 0.01 * np.abs(r)).sum()), max_abs=float(d.max()) if d.size else 0.0)


# --------------------------------------------------------------------------- C oracle (ctypes)
_HERE = os.path.dirname(os.path.abspath(__file__))
_CLIB = None


def build_c_oracle(force: bool = False) -> str:
    so = os.path.join(_HERE, "_build", "libmxfp6_oracle.so")
    src = os.path.join(_HERE, "mxfp6_oracle.c")
    if force or not os.path.exists(so) or os.path.getmtime(so) < os.path.getmtime(src):
        os.makedirs(os.path.dirname(so), exist_ok=True)
        subprocess.check_call(["gcc", "-O2", "-fopenmp", "-fno-fast-math", "-ffp-contract=off", "-shared", "-fPIC",
                               "-o", so, src, "-lm"])
    return so


def c_oracle():
    """ctypes handle on the scalar C oracle (built on demand with gcc)."""
    global _CLIB
    if _CLIB is None:
        L = ctypes.CDLL(build_c_oracle())
        u8p, f32p, u16p = ctypes.POINTER(ctypes.c_uint8), ctypes.POINTER(ctypes.c_float), ctypes.POINTER(ctypes.c_uint16)
        i64, ci = ctypes.c_int64, ctypes.c_int
        L.mxfp6_decode_elem.restype = ctypes.c_float
        L.mxfp6_decode_elem.argtypes = [ctypes.c_uint8, ci]
        L.mxfp6_encode_elem.restype = ctypes.c_uint8
        L.mxfp6_encode_elem.argtypes = [ctypes.c_float, ci]
        L.mxfp6_e8m0_decode.restype = ctypes.c_float
        L.mxfp6_e8m0_decode.argtypes = [ctypes.c_uint8]
        L.mxfp6_e8m0_from_amax.restype = ctypes.c_uint8
        L.mxfp6_e8m0_from_amax.argtypes = [ctypes.c_float, ci]
        L.mxfp6_pack.argtypes = [u8p, i64, u8p]
        L.mxfp6_unpack.argtypes = [u8p, i64, u8p]
        L.mxfp6_quantize.argtypes = [f32p, i64, i64, ci, u8p, u8p]
        L.mxfp6_dequantize.argtypes = [u8p, u8p, i64, i64, ci, f32p]
        L.mxfp6_f32_to_bf16.restype = ctypes.c_uint16
        L.mxfp6_f32_to_bf16.argtypes = [ctypes.c_float]
        L.mxfp6_gemm_ref.argtypes = [u8p, u8p, u8p, u8p, i64, i64, i64, ci, ci, ci, u16p, f32p, f32p]
        _CLIB = L
    return _CLIB


def _p(a, t):
    return a.ctypes.data_as(ctypes.POINTER(t))


def c_quantize(x: np.ndarray, fmt: int):
    x = np.ascontiguousarray(x, dtype=np.float32)
    rows, K = x.shape
    packed = np.empty((rows, K if is_fp8(fmt) else K * 3 // 4), np.uint8)
    scales = np.empty((rows, K // 32), np.uint8)
    c_oracle().mxfp6_quantize(_p(x, ctypes.c_float), rows, K, fmt, _p(packed, ctypes.c_uint8), _p(scales, ctypes.c_uint8))
    return packed, scales


def c_dequantize(packed: np.ndarray, scales: np.ndarray, fmt: int) -> np.ndarray:
    packed = np.ascontiguousarray(packed, dtype=np.uint8)
    scales = np.ascontiguousarray(scales, dtype=np.uint8)
    rows, K = packed.shape[0], (packed.shape[1] if is_fp8(fmt) else packed.shape[1] * 4 // 3)
    out = np.empty((rows, K), np.float32)
    c_oracle().mxfp6_dequantize(_p(packed, ctypes.c_uint8), _p(scales, ctypes.c_uint8), rows, K, fmt, _p(out, ctypes.c_float))
    return out


def c_gemm_ref(a_packed, sfa, b_packed, sfb, fmt_a=E2M3, fmt_b=None, acc_mode=0, want_absdot=False):
    """Scalar C GEMM oracle: returns (c_bf16_bits uint16 [M,N], c_f32 [M,N], absdot or None)."""
    if fmt_b is None:
        fmt_b = fmt_a
    a_packed = np.ascontiguousarray(a_packed, np.uint8)
    b_packed = np.ascontiguousarray(b_packed, np.uint8)
    sfa = np.ascontiguousarray(sfa, np.uint8)
    sfb = np.ascontiguousarray(sfb, np.uint8)
    M, N = a_packed.shape[0], b_packed.shape[0]
    K = a_packed.shape[1] if is_fp8(fmt_a) else a_packed.shape[1] * 4 // 3
    cb = np.empty((M, N), np.uint16)
    cf = np.empty((M, N), np.float32)
    ad = np.empty((M, N), np.float32) if want_absdot else None
    c_oracle().mxfp6_gemm_ref(_p(a_packed, ctypes.c_uint8), _p(sfa, ctypes.c_uint8), _p(b_packed, ctypes.c_uint8),
                              _p(sfb, ctypes.c_uint8), M, N, K, fmt_a, fmt_b, acc_mode,
                              _p(cb, ctypes.c_uint16), _p(cf, ctypes.c_float),
                              _p(ad, ctypes.c_float) if want_absdot else None)
    return cb, cf, ad


def bf16_bits_to_f32(bits: np.ndarray) -> np.ndarray:
    return (np.asarray(bits, np.uint16).astype(np.uint32) << 16).view(np.float32)


# --------------------------------------------------------------------------- the timed CPU path
def dequantize_torch(packed, scales, fmt: int):
    """torch-only dequantise (multi-threaded on the host cores): the first half of the CPU
    dequantise-then-matmul path that the benchmark times as the reference arm."""
    import torch

    rows = packed.shape[0]
    if is_fp8(fmt):
        K = packed.shape[1]
        codes = packed
    else:
        K = packed.shape[1] // 3 * 4
        b = packed.view(rows, -1, 3).to(torch.int32)
        w = b[..., 0] | (b[..., 1] << 8) | (b[..., 2] << 16)
        codes = torch.stack([w & 63, (w >> 6) & 63, (w >> 12) & 63, (w >> 18) & 63], dim=-1).view(rows, K)
    lut = torch.from_numpy(decode_table(fmt))
    vals = lut[codes.long()]
    s = torch.from_numpy(e8m0_decode(np.arange(256, dtype=np.uint8)))[scales.long()]
    return (vals.view(rows, K // 32, 32) * s.unsqueeze(-1)).view(rows, K)


def gemm_cpu_path(a_packed, sfa, b_packed, sfb, fmt_a=E2M3, fmt_b=None):
    """torch tensors in (uint8), bf16 tensor out: dequantise both operands, fp32 matmul, round to bf16."""
    import torch

    A = dequantize_torch(a_packed, sfa, fmt_a)
    B = dequantize_torch(b_packed, sfb, fmt_a if fmt_b is None else fmt_b)
    return (A @ B.t()).to(torch.bfloat16)
