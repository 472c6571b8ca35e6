"""Helpers shared by the GPU parity tests: seeded inputs, oracle results, tolerance checks."""
import numpy as np
import torch

import hipkittensp_b200 as hk
from oracle import mxfp6_ref as R

ROW_REL_TOL = 1e-2      # max_n |C - C_ref| / ||C_ref[r,:]||_2
ULP_TOL = 2.0           # bf16 ulps from the fp32/fp64-accumulated oracle (outside the accumulation noise floor)


def quantized_inputs(config, M, N, K, fmt=R.E2M3, seed=0, fmt_b=None):
    A, B = R.make_inputs(config, M, N, K, seed)
    pa, sa = R.quantize(A, fmt)
    pb, sb = R.quantize(B, fmt if fmt_b is None else fmt_b)
    return pa, sa, pb, sb


def oracle_f64(pa, sa, pb, sb, fmt, fmt_b=None):
    Ad = R.dequantize(pa, sa, fmt).astype(np.float64)
    Bd = R.dequantize(pb, sb, fmt if fmt_b is None else fmt_b).astype(np.float64)
    return Ad @ Bd.T, np.abs(Ad) @ np.abs(Bd).T


def run_gpu(pa, sa, pb, sb, fmt, fmt_b=None, guard=True):
    dev = torch.device("cuda:0")
    M, N = pa.shape[0], pb.shape[0]
    tA, tB = torch.from_numpy(pa).to(dev), torch.from_numpy(pb).to(dev)
    tsa, tsb = torch.from_numpy(sa).to(dev), torch.from_numpy(sb).to(dev)
    # C sits inside a larger NaN-filled buffer so that unwritten elements and out-of-bounds writes show
    pad = 64 if guard else 0
    buf = torch.full((M * N + 2 * pad,), float("nan"), dtype=torch.bfloat16, device=dev)
    C = buf[pad:pad + M * N].view(M, N)
    hk.dispatch_micro(tA, tB, C, tsa, tsb, fmt, fmt_b)
    assert hk.device_status() == 0
    if guard:
        assert torch.isnan(buf[:pad]).all() and torch.isnan(buf[pad + M * N:]).all(), "write outside C"
    return C.float().cpu().numpy()


# Elements whose error exceeds ULP_TOL but lies inside the fp32 accumulation noise floor of their own sum
# (2^-20 * sum_k |a_k b_k|: results that cancel to almost nothing) are excused by the oracle's report and counted as
# n_floor.  Their share is bounded: at most one element in 100 000, which means none at all in the small cases.
FLOOR_SHARE = 1e-5


def check(c, ref, absdot):
    assert not np.isnan(c).any(), f"{int(np.isnan(c).sum())} elements of C were not written"
    rep = R.error_report(c, ref, absdot)
    assert rep["row_rel"] <= ROW_REL_TOL, rep
    assert rep["max_ulp"] <= ULP_TOL, rep
    assert rep["n_floor"] <= int(FLOOR_SHARE * c.size), rep
    return rep
