"""mxfp6_gemm_noalloc: the GEMM entry point for hosts that cannot allocate device memory at run time.

Some callers own all of the GPU's memory themselves (an inference server's pool), or run under a latency
bound that a cudaMalloc could break, or sit behind a plug-in interface that forbids allocation in the call
path.  For them the library keeps the scratch that split output tiles need in a buffer built into its own
image.  This test calls that entry point through the C ABI on shapes that do and do not need scratch and
checks, twice in a row, that it writes exactly what the allocating entry point mxfp6_gemm writes (same
kernel, same fixed summation order, hence bit-identical -- tighter than the 2-ulp tolerance of the parity
tests), and that an oversized request is refused with a clear message.

The file is named so that pytest collects it last."""
import os
import subprocess
import sys

import pytest
import torch

import hipkittensp_b200 as hk
from hipkittensp_b200 import _lib
from oracle import mxfp6_ref as R

pytestmark = pytest.mark.gpu


def _operands(M, N, K, seed):
    A, B = R.make_inputs("decode", M, N, K, seed)
    pa, sa = R.quantize(A, R.E2M3)
    pb, sb = R.quantize(B, R.E2M3)
    return [torch.from_numpy(x).cuda() for x in (pa, sa, pb, sb)]


def _call(fn, t, C, M, N, K):
    stream = torch.cuda.current_stream().cuda_stream
    return fn(t[0].data_ptr(), t[1].data_ptr(), t[2].data_ptr(), t[3].data_ptr(), C.data_ptr(), M, N, K, 0, 0, stream)


@pytest.mark.parametrize("shape", [(16, 4096, 4096),      # split tiles: uses the built-in scratch
                                   (64, 3584, 2048),      # split tiles, wider accumulator
                                   (256, 512, 1024)])     # whole tiles only: no scratch at all
def test_noalloc_matches_allocating_entry_point_twice(shape):
    M, N, K = shape
    t = _operands(M, N, K, seed=M)
    want = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device="cuda")
    _lib.check(_call(hk.lib.mxfp6_gemm, t, want, M, N, K))
    assert hk.device_status() == 0
    assert not torch.isnan(want).any()
    for attempt in range(2):                                 # the second call sees the first one's leftovers
        got = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device="cuda")
        _lib.check(_call(hk.lib.mxfp6_gemm_noalloc, t, got, M, N, K))
        assert hk.device_status() == 0
        assert torch.equal(got.view(torch.int16), want.view(torch.int16)), f"call {attempt + 1} differs"


def test_noalloc_refuses_more_scratch_than_it_has():
    # 300 split tiles with 64-wide fp32 partials need far more than the 8 MiB the library carries
    M, N, K = 64, 128 * 300, 1024
    need = hk.lib.mxfp6_gemm_workspace_bytes(M, N, K)
    assert need > 8 << 20
    dummy = torch.zeros(64, dtype=torch.uint8, device="cuda")
    p = dummy.data_ptr()
    rc = hk.lib.mxfp6_gemm_noalloc(p, p, p, p, p, M, N, K, 0, 0, None)
    assert rc == _lib.ERR_BAD_ARG
    msg = hk.lib.mxfp6_last_error().decode()
    assert "built-in buffer" in msg and str(need) in msg


# Run in a process of its own, so that the allocating entry point has not been called before and the library holds no
# scratch of its own yet: the no-allocation entry point must leave the device's free memory exactly as it found it,
# while the allocating one, called afterwards on the same shape, visibly takes its 8 MiB.
_FRESH = r"""
import sys, torch
sys.path.insert(0, sys.argv[1])
import hipkittensp_b200 as hk
from hipkittensp_b200 import _lib
torch.cuda.set_device(0)
def operands(M, N, K, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    pa, sa = hk.quantize(torch.randn(M, K, device="cuda", generator=g))
    pb, sb = hk.quantize(0.02 * torch.randn(N, K, device="cuda", generator=g))
    return pa, sa, pb, sb
def call(fn, t, C, M, N, K):
    return fn(t[0].data_ptr(), t[1].data_ptr(), t[2].data_ptr(), t[3].data_ptr(), C.data_ptr(), M, N, K, 0, 0,
              torch.cuda.current_stream().cuda_stream)
S1, S2 = (16, 4096, 4096), (16, 8192, 4096)           # both split tiles along K, with the same kernel variant
t1, t2 = operands(*S1, 1), operands(*S2, 2)
c1 = torch.empty(S1[:2], dtype=torch.bfloat16, device="cuda")
got = torch.full(S2[:2], float("nan"), dtype=torch.bfloat16, device="cuda")
want = torch.full(S2[:2], float("nan"), dtype=torch.bfloat16, device="cuda")
assert hk.lib.mxfp6_gemm_workspace_bytes(*S2) > 0
_lib.check(call(hk.lib.mxfp6_gemm_noalloc, t1, c1, *S1))      # first use: the kernel's code is loaded here
torch.cuda.synchronize()
free0 = torch.cuda.mem_get_info()[0]
_lib.check(call(hk.lib.mxfp6_gemm_noalloc, t2, got, *S2))
torch.cuda.synchronize()
free1 = torch.cuda.mem_get_info()[0]
_lib.check(call(hk.lib.mxfp6_gemm, t2, want, *S2))             # the allocating entry point, for contrast
torch.cuda.synchronize()
free2 = torch.cuda.mem_get_info()[0]
assert hk.device_status() == 0
assert free1 == free0, f"mxfp6_gemm_noalloc changed the free device memory by {free0 - free1} bytes"
assert free0 - free2 >= (8 << 20), f"the probe did not see mxfp6_gemm's own scratch allocation ({free0 - free2} bytes)"
assert torch.equal(got.view(torch.int16), want.view(torch.int16))
print("NOALLOC_FRESH_OK")
"""


def test_noalloc_leaves_free_memory_unchanged_in_a_fresh_process():
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    out = subprocess.run([sys.executable, "-c", _FRESH, root], capture_output=True, text=True, timeout=600)
    assert "NOALLOC_FRESH_OK" in out.stdout, out.stdout[-2000:] + out.stderr[-2000:]
