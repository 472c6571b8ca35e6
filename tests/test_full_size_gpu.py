"""Parity at the full benchmark sizes against the fp64 oracle (the exactly dequantised operands multiplied in
float64 on the host cores): the whole 8192 x 8192 result of the headline configuration, and for the larger
configurations a seeded sample of 512 complete rows of C (every column of those rows, hence every tile column and
every K-block of the kernel's schedule); where two different kernels can compute the same problem, also agreement
between them over the whole matrix."""
import os

import numpy as np
import pytest
import torch

import hipkittensp_b200 as hk
from oracle import mxfp6_ref as R
from tests.gpu_util import FLOOR_SHARE, ROW_REL_TOL, ULP_TOL

pytestmark = pytest.mark.gpu


@pytest.fixture(autouse=True)
def _clean_env():
    yield
    hk.debug_option("MXFP6_FORCE_CFG", None)


def _quantized(config, M, N, K, fmt, seed):
    A, B = R.make_inputs(config, M, N, K, seed)
    pa, sa = R.c_quantize(A, fmt)
    pb, sb = R.c_quantize(B, fmt)
    return pa, sa, pb, sb


def _check_rows(C, pa, sa, pb, sb, fmt, rows, block=1024):
    """Rows `rows` of the GPU result against the fp64 oracle (tolerances of the parity tests), in blocks of rows."""
    Bd = torch.from_numpy(R.c_dequantize(pb, sb, fmt)).double()
    Bd_abs = None
    worst = dict(row_rel=0.0, max_ulp=0.0, n_floor=0)
    rows = np.asarray(rows)
    for i in range(0, len(rows), block):
        rb = rows[i:i + block]
        Ad = torch.from_numpy(R.c_dequantize(pa[rb], sa[rb], fmt)).double()
        ref = (Ad @ Bd.t()).numpy()
        got = C[torch.as_tensor(rb, device=C.device)].float().cpu().numpy()
        assert not np.isnan(got).any()
        rep = R.error_report(got, ref, None)
        if rep["max_ulp"] > ULP_TOL:
            # some element is more than ULP_TOL off: is it inside the accumulation noise floor of its own sum?
            if Bd_abs is None:
                Bd_abs = Bd.abs()
            rep = R.error_report(got, ref, (Ad.abs() @ Bd_abs.t()).numpy())
        assert rep["row_rel"] <= ROW_REL_TOL and rep["max_ulp"] <= ULP_TOL, rep
        worst = dict(row_rel=max(worst["row_rel"], rep["row_rel"]), max_ulp=max(worst["max_ulp"], rep["max_ulp"]),
                     n_floor=worst["n_floor"] + rep["n_floor"])
    assert worst["n_floor"] <= int(FLOOR_SHARE * len(rows) * C.shape[1]), worst
    return worst


def _gpu(pa, sa, pb, sb, fmt):
    t = [torch.from_numpy(x).cuda() for x in (pa, sa, pb, sb)]
    C = hk.gemm(t[0], t[1], t[2], t[3], fmt)
    assert hk.device_status() == 0
    return C


def test_config_8192_cubed_lognormal():
    M = N = K = 8192
    pa, sa, pb, sb = _quantized("lognormal", M, N, K, R.E2M3, seed=0)
    C = _gpu(pa, sa, pb, sb, R.E2M3)
    _check_rows(C, pa, sa, pb, sb, R.E2M3, np.arange(M))      # the whole matrix, as the reference's own check scans it (8_wave.cu:479-496)
    # the single-CTA kernel computes the same matrix
    hk.debug_option("MXFP6_FORCE_CFG", "256,0,0,0")
    C1 = _gpu(pa, sa, pb, sb, R.E2M3)
    diff = (C.float() - C1.float()).abs()
    assert float((diff / C1.float().abs().clamp_min(1e-30)).max()) <= 2 ** -7, "pair and single-CTA kernels disagree by more than 1 bf16 ulp"
    assert float((C != C1).float().mean()) < 1e-3


def test_config_ffn_e3m2_with_outlier_channels():
    M, N, K = 4096, 14336, 8192
    pa, sa, pb, sb = _quantized("ffn", M, N, K, R.E3M2, seed=0)
    C = _gpu(pa, sa, pb, sb, R.E3M2)
    rows = np.sort(np.random.default_rng(1).choice(M, 512, replace=False))
    rows[:4] = [0, 127, 128, M - 1]                        # tile edges
    _check_rows(C, pa, sa, pb, sb, R.E3M2, np.sort(rows), block=512)


@pytest.mark.parametrize("M", [1, 16, 64])
def test_config_decode_full(M):
    N, K = 28672, 8192
    pa, sa, pb, sb = _quantized("decode", M, N, K, R.E2M3, seed=M)
    C = _gpu(pa, sa, pb, sb, R.E2M3)
    rows = np.arange(M) if M <= 16 else np.sort(np.random.default_rng(2).choice(M, 16, replace=False))
    _check_rows(C, pa, sa, pb, sb, R.E2M3, rows)
    # whole-tile kernel (no K split) gives the same result up to the summation order of split tiles
    hk.debug_option("MXFP6_FORCE_CFG", "%d,1,0" % (16 if M <= 16 else 64))
    C1 = _gpu(pa, sa, pb, sb, R.E2M3)
    assert float(((C.float() - C1.float()).abs() / C1.float().abs().clamp_min(1e-30)).median()) == 0.0
    assert float((C != C1).float().mean()) < 2e-2


def test_config_sharded_one_shard():
    """One g=8 shard of the column-parallel configuration: A [16384, K] against 7168 rows of B."""
    M, N, K = 16384, 7168, 8192
    pa, sa, pb, sb = _quantized("normal", M, N, K, R.E2M3, seed=3)
    C = _gpu(pa, sa, pb, sb, R.E2M3)
    rows = np.sort(np.random.default_rng(3).choice(M, 512, replace=False))
    _check_rows(C, pa, sa, pb, sb, R.E2M3, rows, block=512)


# ------------------------------------------------------------------------------- size-independent properties
def _flip_signs_fp6(packed: torch.Tensor) -> torch.Tensor:
    """Negates every element of a packed fp6 operand: the sign is bit 5 of each 6-bit code, i.e. bits 5, 11, 17, 23
    of every 3-byte group."""
    mask = torch.tensor([0x20, 0x08, 0x82], dtype=torch.uint8, device=packed.device).repeat(packed.shape[1] // 3)
    return packed ^ mask


def test_full_size_exact_properties_8192_cubed():
    """Properties that hold bit for bit whatever the size, checked on the whole 8192 x 8192 result:
    a scale byte + 1 on every block of A doubles C exactly; negating A negates C; permuting the rows of A permutes
    the rows of C; a block of B's rows gives the matching block of C's columns."""
    M = N = K = 8192
    pa, sa, pb, sb = (torch.from_numpy(x).cuda() for x in _quantized("lognormal", M, N, K, R.E2M3, seed=1))
    C = hk.gemm(pa, sa, pb, sb, R.E2M3)
    assert hk.device_status() == 0
    assert int(sa.max()) < 254
    C2 = hk.gemm(pa, sa + 1, pb, sb, R.E2M3)
    assert torch.equal(C2.float(), 2.0 * C.float())
    Cn = hk.gemm(_flip_signs_fp6(pa), sa, pb, sb, R.E2M3)
    assert torch.equal(Cn.float(), -C.float())
    perm = torch.randperm(M, device="cuda", generator=torch.Generator(device="cuda").manual_seed(3))
    Cp = hk.gemm(pa[perm].contiguous(), sa[perm].contiguous(), pb, sb, R.E2M3)
    assert torch.equal(Cp, C[perm])
    lo, hi = 2048, 6144
    Cb = hk.gemm(pa, sa, pb[lo:hi].contiguous(), sb[lo:hi].contiguous(), R.E2M3)
    assert torch.equal(Cb, C[:, lo:hi])
    assert hk.device_status() == 0


def test_full_size_exact_properties_decode():
    """The same properties on the K-split kernel (M=16, N=28672, K=8192), whose split tiles are summed in a fixed order."""
    M, N, K = 16, 28672, 8192
    pa, sa, pb, sb = (torch.from_numpy(x).cuda() for x in _quantized("decode", M, N, K, R.E2M3, seed=2))
    C = hk.gemm(pa, sa, pb, sb, R.E2M3)
    assert int(sb.max()) < 254
    C2 = hk.gemm(pa, sa, pb, sb + 1, R.E2M3)
    assert torch.equal(C2.float(), 2.0 * C.float())
    Cn = hk.gemm(pa, sa, _flip_signs_fp6(pb), sb, R.E2M3)
    assert torch.equal(Cn.float(), -C.float())
    perm = torch.randperm(M, device="cuda", generator=torch.Generator(device="cuda").manual_seed(4))
    Cp = hk.gemm(pa[perm].contiguous(), sa[perm].contiguous(), pb, sb, R.E2M3)
    assert torch.equal(Cp, C[perm])
    assert hk.device_status() == 0
