"""B200-native MX-FP6 GEMM: C[M,N] (bf16) = A[M,K] @ B[N,K]^T with packed 6-bit operands and E8M0
block scales, behind the `tk_kernel.dispatch_micro` calling convention of benenzhu/HipKittensP.

The compute path is the CUDA library libmxfp6.so (C ABI: include/mxfp6.h); importing this package
fails if it has not been built (`python hipkittensp_b200/build.py`)."""
from ._lib import E2M3, E3M2, E4M3, E5M2, LIB_PATH, Mxfp6Error, debug_option, lib  # noqa: F401
from .host import HostGemm  # noqa: F401
from .gemm import copy_gather_scratch_bytes, dequantize, device_status, dispatch_copy_gather, dispatch_micro, dispatch_multi, gemm, gemm_requant, gemm_scaled, quantize, tma_dump  # noqa: F401

__all__ = ["E2M3", "E3M2", "E4M3", "E5M2", "dispatch_micro", "dispatch_multi", "dispatch_copy_gather", "copy_gather_scratch_bytes", "gemm", "gemm_requant", "gemm_scaled", "quantize", "dequantize", "device_status", "tma_dump",
           "HostGemm", "Mxfp6Error", "lib", "LIB_PATH", "debug_option"]
