"""mxfp6_gemm_noalloc: the GEMM entry point for hosts that cannot allocate device memory at run time.

Some callers own all of the GPU's memory themselves (an inference server's pool), or run under a latency
bound that a cudaMalloc could break, or sit behind a plug-in interface that forbids allocation in the call
path.  For them the library keeps the scratch that split output tiles need in a buffer built into its own
image.  This test calls that entry point through the C ABI on shapes that do and do not need scratch and
checks, twice in a row, that it writes exactly what the allocating entry point mxfp6_gemm writes (same
kernel, same fixed summation order, hence bit-identical -- tighter than the 2-ulp tolerance of the parity
tests), and that an oversized request is refused with a clear message.

The file is named so that pytest collects it last."""
import ctypes

import numpy as np
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
    # 600 split tiles with 32-wide fp32 partials need far more than the 8 MiB the library carries
    M, N, K = 32, 128 * 600, 1024
    need = hk.lib.mxfp6_gemm_workspace_bytes(M, N, K)
    assert need > 8 << 20
    dummy = torch.zeros(64, dtype=torch.uint8, device="cuda")
    p = dummy.data_ptr()
    rc = hk.lib.mxfp6_gemm_noalloc(p, p, p, p, p, M, N, K, 0, 0, None)
    assert rc == _lib.ERR_BAD_ARG
    msg = hk.lib.mxfp6_last_error().decode()
    assert "built-in buffer" in msg and str(need) in msg
