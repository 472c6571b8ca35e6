"""CPU-only checks of the boundary: the shared library loads, exports every symbol the header declares,
and rejects bad arguments before touching the GPU."""
import ctypes
import os
import re

import pytest

import hipkittensp_b200 as hk
from hipkittensp_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _header_symbols():
    src = open(os.path.join(ROOT, "include", "mxfp6.h")).read()
    src = re.sub(r"/\*.*?\*/", "", src, flags=re.S)
    return sorted(set(re.findall(r"\b(mxfp6_[a-z0-9_]+)\s*\(", src)))


def test_library_exports_every_declared_symbol():
    declared = _header_symbols()
    assert declared, "no declarations found in include/mxfp6.h"
    raw = ctypes.CDLL(_lib.LIB_PATH)
    for name in declared:
        assert hasattr(raw, name), f"{name} is declared in mxfp6.h but not exported by libmxfp6.so"
    assert set(declared) == set(_lib.SYMBOLS)


def test_version_and_error_string():
    assert hk.lib.mxfp6_version() >= 100
    assert isinstance(hk.lib.mxfp6_last_error(), bytes)


def test_bad_arguments_rejected_without_gpu():
    L = hk.lib
    assert L.mxfp6_gemm(None, None, None, None, None, 16, 16, 100, 0, 0, None) == _lib.ERR_BAD_ARG
    assert b"multiple of 128" in L.mxfp6_last_error()
    assert L.mxfp6_gemm(None, None, None, None, None, -1, 16, 128, 0, 0, None) == _lib.ERR_BAD_ARG
    assert L.mxfp6_gemm(None, None, None, None, None, 16, 16, 128, 7, 0, None) == _lib.ERR_BAD_ARG
    assert L.mxfp6_gemm(None, None, None, None, None, 0, 16, 128, 0, 0, None) == _lib.OK      # empty problem
    assert L.mxfp6_gemm(None, None, None, None, None, 16, 16, 128, 0, 0, None) == _lib.ERR_BAD_ARG  # null C
    assert L.mxfp6_quantize(None, 0, 4, 33, 0, None, None, None) == _lib.ERR_BAD_ARG
    assert L.mxfp6_quantize(None, 5, 4, 32, 0, None, None, None) == _lib.ERR_BAD_ARG
    assert L.mxfp6_quantize(None, 0, 0, 32, 0, None, None, None) == _lib.OK
    assert L.mxfp6_dequantize(None, None, 4, 32, 3, None, None) == _lib.ERR_BAD_ARG
    assert L.mxfp6_gemm_workspace_bytes(16, 16, 100) == 0
    # the re-quantising GEMM stores two scale bytes at a time: an odd out_scales pointer is refused
    assert L.mxfp6_gemm_requant(None, None, None, None, 256, 257, 64, 64, 128, 0, 0, 0, None) == _lib.ERR_BAD_ARG
    assert b"2-byte aligned" in L.mxfp6_last_error()
    assert L.mxfp6_debug_option(b"MXFP6_NO_SUCH_SWITCH", b"1") == _lib.ERR_BAD_ARG
    assert L.mxfp6_debug_option(b"MXFP6_GROUP_P", b"8") == _lib.OK
    assert L.mxfp6_debug_option(b"MXFP6_GROUP_P", None) == _lib.OK


def test_copy_gather_arguments_and_block_count():
    """The copy-engine gather refuses bad arguments before it touches a device, and its scratch is two 32-bit words
    (flag, counter) per block of C: row groups of 16 tile rows by strips of `strip_tiles` 256-column tiles."""
    L = hk.lib
    vp = ctypes.c_void_p
    one = (vp * 1)(0x1000)
    two = (vp * 2)(0x1000, 0x2000)
    args = lambda dst, n, M, N, K, scratch, nbytes, strip, streams, ns: (None, None, None, None, dst, n, N, M, N, K, 0, 0, scratch, nbytes, strip, streams, ns, None)
    assert L.mxfp6_gemm_copy_gather(*args(None, 1, 512, 512, 128, None, 0, 1, None, 0)) == _lib.ERR_BAD_ARG
    assert b"destination" in L.mxfp6_last_error()
    assert L.mxfp6_gemm_copy_gather(*args(one, 9, 512, 512, 128, None, 0, 1, None, 0)) == _lib.ERR_BAD_ARG
    assert L.mxfp6_gemm_copy_gather(*args(one, 1, 0, 512, 128, None, 0, 1, None, 0)) == _lib.ERR_BAD_ARG
    assert L.mxfp6_gemm_copy_gather(*args(one, 1, 512, 512, 128, None, 0, 0, None, 0)) == _lib.ERR_BAD_ARG
    assert b"strip_tiles" in L.mxfp6_last_error()
    assert L.mxfp6_gemm_copy_gather(*args(two, 2, 512, 512, 128, None, 0, 1, None, 0)) == _lib.ERR_BAD_ARG
    assert b"copy streams" in L.mxfp6_last_error()
    assert L.mxfp6_gemm_copy_gather(*args(one, 1, 512, 512, 128, None, 0, 1, None, 0)) == _lib.ERR_BAD_ARG
    assert b"scratch too small" in L.mxfp6_last_error()
    assert L.mxfp6_copy_gather_scratch_bytes(16384, 14336, 8) == 4 * 7 * 8
    assert L.mxfp6_copy_gather_scratch_bytes(4352, 2304, 4) == 2 * 3 * 8
    assert L.mxfp6_copy_gather_scratch_bytes(4352, 2304, 1000) == 2 * 1 * 8
    assert L.mxfp6_copy_gather_scratch_bytes(0, 2304, 4) == 0


def test_python_wrapper_rejects_cpu_and_bad_tensors():
    import torch
    A = torch.zeros(16, 96, dtype=torch.uint8)
    C = torch.zeros(16, 16, dtype=torch.bfloat16)
    S = torch.zeros(16, 4, dtype=torch.uint8)
    with pytest.raises(RuntimeError, match="Tensor must be on CUDA device"):
        hk.dispatch_micro(A, A, C, S, S)
    with pytest.raises(RuntimeError, match="Tensor must be contiguous"):
        hk.dispatch_micro(A.t(), A, C, S, S)
    with pytest.raises(RuntimeError, match="Expected a torch.Tensor"):
        hk.dispatch_micro(1, A, C, S, S)


def test_tk_kernel_module_matches_reference_names():
    import sys
    sys.path.insert(0, os.path.join(ROOT, "hipkittensp_b200"))
    import tk_kernel
    import torch
    assert callable(tk_kernel.dispatch_micro)
    A = torch.zeros(16, 96, dtype=torch.uint8)
    C = torch.zeros(16, 16, dtype=torch.bfloat16)
    S = torch.zeros(16, 4, dtype=torch.uint8)
    with pytest.raises(RuntimeError, match="Tensor must be on CUDA device"):
        tk_kernel.dispatch_micro(A, A, C, S, S)
    with pytest.raises(RuntimeError, match="Tensor must be contiguous"):
        tk_kernel.dispatch_micro(A.t(), A, C, S, S)
    with pytest.raises(RuntimeError, match="Expected a torch.Tensor"):
        tk_kernel.dispatch_micro(3, A, C, S, S)


def test_cpp_host_harness_is_built_and_rejects_bad_arguments():
    import subprocess

    import hipkittensp_b200 as hk
    exe = os.path.join(os.path.dirname(hk.__file__), "matmul_host")
    assert os.path.exists(exe), "build it with `python hipkittensp_b200/build.py`"
    res = subprocess.run([exe, "128", "128", "100"], capture_output=True, text=True, timeout=60)   # K not a multiple of 128
    assert res.returncode == 2 and "usage" in res.stderr
