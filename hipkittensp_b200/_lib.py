"""ctypes binding of libmxfp6.so (the C ABI in include/mxfp6.h).  There is no fallback: if the library
is missing or does not load, importing this module raises."""
from __future__ import annotations

import ctypes
import os

_PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.environ.get("MXFP6_LIBRARY") or os.path.join(_PKG, "libmxfp6.so")   # MXFP6_LIBRARY: load another build of the library

E2M3 = 0
E3M2 = 1
E4M3 = 2   # MX-FP8
E5M2 = 3   # MX-FP8

FLAG_B_STATIC = 1

OK, ERR_BAD_ARG, ERR_CUDA, ERR_DEVICE_WAIT, ERR_UNSUPPORTED = 0, 1, 2, 3, 4

# every symbol include/mxfp6.h declares
SYMBOLS = ("mxfp6_version", "mxfp6_last_error", "mxfp6_gemm", "mxfp6_gemm_workspace_bytes", "mxfp6_gemm_ws",
           "mxfp6_gemm_noalloc", "mxfp6_gemm_multi", "mxfp6_gemm_copy_gather", "mxfp6_copy_gather_scratch_bytes", "mxfp6_gemm_ex", "mxfp6_gemm_requant", "mxfp6_gemm_scaled",
           "mxfp6_quantize", "mxfp6_dequantize", "mxfp6_device_status", "mxfp6_debug_tma_dump", "mxfp6_debug_wait_timeout", "mxfp6_debug_option", "mxfp6_debug_plan")


class Mxfp6Error(RuntimeError):
    def __init__(self, code: int, msg: str):
        super().__init__(f"mxfp6 error {code}: {msg}")
        self.code = code


def _load() -> ctypes.CDLL:
    if not os.path.exists(LIB_PATH):
        raise ImportError(f"{LIB_PATH} is missing: build it with `python hipkittensp_b200/build.py` "
                          "(there is no CPU or PyTorch fallback for this path)")
    try:
        import torch  # noqa: F401  -- loads the CUDA runtime torch ships, so both share one runtime instance
    except Exception:
        pass
    lib = ctypes.CDLL(LIB_PATH)
    vp, i64, ci, sz = ctypes.c_void_p, ctypes.c_int64, ctypes.c_int, ctypes.c_size_t
    lib.mxfp6_version.restype = ci
    lib.mxfp6_version.argtypes = []
    lib.mxfp6_last_error.restype = ctypes.c_char_p
    lib.mxfp6_last_error.argtypes = []
    lib.mxfp6_gemm.restype = ci
    lib.mxfp6_gemm.argtypes = [vp, vp, vp, vp, vp, i64, i64, i64, ci, ci, vp]
    lib.mxfp6_gemm_noalloc.restype = ci
    lib.mxfp6_gemm_noalloc.argtypes = [vp, vp, vp, vp, vp, i64, i64, i64, ci, ci, vp]
    lib.mxfp6_gemm_ex.restype = ci
    lib.mxfp6_gemm_ex.argtypes = [vp, vp, vp, vp, vp, i64, i64, i64, ci, ci, ctypes.c_uint, vp]
    lib.mxfp6_gemm_requant.restype = ci
    lib.mxfp6_gemm_requant.argtypes = [vp, vp, vp, vp, vp, vp, i64, i64, i64, ci, ci, ci, vp]
    lib.mxfp6_gemm_scaled.restype = ci
    lib.mxfp6_gemm_scaled.argtypes = [vp, vp, vp, vp, vp, vp, vp, vp, i64, i64, i64, ci, ci, vp]
    lib.mxfp6_gemm_multi.restype = ci
    lib.mxfp6_gemm_multi.argtypes = [vp, vp, vp, vp, ctypes.POINTER(vp), ci, i64, i64, i64, i64, ci, ci, vp]
    lib.mxfp6_gemm_copy_gather.restype = ci
    lib.mxfp6_gemm_copy_gather.argtypes = [vp, vp, vp, vp, ctypes.POINTER(vp), ci, i64, i64, i64, i64, ci, ci, vp, sz, ci,
                                           ctypes.POINTER(vp), ci, vp]
    lib.mxfp6_copy_gather_scratch_bytes.restype = sz
    lib.mxfp6_copy_gather_scratch_bytes.argtypes = [i64, i64, ci]
    lib.mxfp6_gemm_workspace_bytes.restype = sz
    lib.mxfp6_gemm_workspace_bytes.argtypes = [i64, i64, i64]
    lib.mxfp6_gemm_ws.restype = ci
    lib.mxfp6_gemm_ws.argtypes = [vp, vp, vp, vp, vp, i64, i64, i64, ci, ci, vp, sz, vp]
    lib.mxfp6_quantize.restype = ci
    lib.mxfp6_quantize.argtypes = [vp, ci, i64, i64, ci, vp, vp, vp]
    lib.mxfp6_dequantize.restype = ci
    lib.mxfp6_dequantize.argtypes = [vp, vp, i64, i64, ci, vp, vp]
    lib.mxfp6_device_status.restype = ci
    lib.mxfp6_device_status.argtypes = [ctypes.POINTER(ci)]
    lib.mxfp6_debug_wait_timeout.restype = ci
    lib.mxfp6_debug_wait_timeout.argtypes = [ci, vp]
    lib.mxfp6_debug_option.restype = ci
    lib.mxfp6_debug_option.argtypes = [ctypes.c_char_p, ctypes.c_char_p]
    lib.mxfp6_debug_plan.restype = ci
    lib.mxfp6_debug_plan.argtypes = [i64, i64, i64, ci, ci, ci, ctypes.POINTER(ci)]
    lib.mxfp6_debug_tma_dump.restype = ci
    lib.mxfp6_debug_tma_dump.argtypes = [vp, i64, i64, i64, i64, vp, vp]
    return lib


lib = _load()


def check(rc: int) -> None:
    if rc != OK:
        raise Mxfp6Error(rc, lib.mxfp6_last_error().decode())


PLAN_FIELDS = ("bn", "swap", "streamk", "pair", "ctas", "p_tile", "q_tile", "tiles_p", "tiles_q", "grid", "tail_first", "tail_split")


def debug_plan(M: int, N: int, K: int, sm_count: int = 148, n_dst: int = 1, requant: bool = False) -> dict:
    """Test hook: the kernel choice and tiling for a problem on a device with sm_count SMs (touches no device)."""
    out = (ctypes.c_int * 12)()
    check(lib.mxfp6_debug_plan(M, N, K, sm_count, n_dst, int(requant), out))
    return dict(zip(PLAN_FIELDS, out))


def debug_option(name: str, value: str | None) -> None:
    """Test hook: set one of the library's switches (None restores the default); see mxfp6_debug_option."""
    check(lib.mxfp6_debug_option(name.encode(), None if value is None else str(value).encode()))
