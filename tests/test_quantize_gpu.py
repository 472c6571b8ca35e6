"""GPU quantiser / dequantiser against the oracle: bit-exact."""
import numpy as np
import pytest
import torch

import hipkittensp_b200 as hk
from oracle import mxfp6_ref as R

import os

pytestmark = pytest.mark.gpu


@pytest.fixture(autouse=True, params=["stream", "quad"])
def _quantiser_path(request):
    """Every test runs on both quantiser kernels: the TMA-fed streaming kernel (default) and the plain-load kernel."""
    if request.param == "quad":
        hk.debug_option("MXFP6_QUANT_PATH", "quad")
    yield
    hk.debug_option("MXFP6_QUANT_PATH", None)


@pytest.mark.parametrize("fmt", [R.E2M3, R.E4M3])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("rows,K", [(1, 32), (5, 96), (3, 32 * 43), (129, 32), (2048, 4096), (1000, 2464)])
def test_quantize_ragged_and_many_tiles(fmt, dtype, rows, K):
    """Block counts that are not multiples of the 128-block tile (the tail takes plain stores), a single block, and
    more tiles than resident CTAs (each CTA loops over its ring of stages several times)."""
    x = torch.randn(rows, K, generator=torch.Generator().manual_seed(rows + K)).to(dtype)
    pa, sa = R.c_quantize(np.ascontiguousarray(x.float().numpy()), fmt)
    gp, gs = hk.quantize(x.cuda(), fmt)
    assert hk.device_status() == 0
    np.testing.assert_array_equal(gs.cpu().numpy(), sa)
    np.testing.assert_array_equal(gp.cpu().numpy(), pa)


@pytest.mark.parametrize("fmt", [R.E2M3, R.E3M2])
@pytest.mark.parametrize("config", ["normal", "lognormal", "ffn", "decode"])
def test_quantize_bit_exact(fmt, config):
    A, B = R.make_inputs(config, 96, 200, 512, seed=7)
    for x in (A, B):
        pa, sa = R.quantize(x, fmt)
        gp, gs = hk.quantize(torch.from_numpy(x).cuda(), fmt)
        np.testing.assert_array_equal(gs.cpu().numpy(), sa)
        np.testing.assert_array_equal(gp.cpu().numpy(), pa)


@pytest.mark.parametrize("fmt", [R.E2M3, R.E3M2])
def test_quantize_edge_values(fmt):
    K = 256
    x = np.zeros((8, K), np.float32)
    x[0, :32] = 0.0
    x[1, :32] = 1.0
    x[2, 0] = 7.9 if fmt == R.E2M3 else 31.0
    x[3, :32] = 1e-30
    x[4, 5] = -0.0
    x[5, :64] = np.linspace(-100, 100, 64)
    x[6, :] = np.ldexp(1.0, -140)
    x[7, ::2] = 3.0e38
    pa, sa = R.quantize(x, fmt)
    gp, gs = hk.quantize(torch.from_numpy(x).cuda(), fmt)
    np.testing.assert_array_equal(gs.cpu().numpy(), sa)
    np.testing.assert_array_equal(gp.cpu().numpy(), pa)


def test_quantize_bf16_input():
    x = torch.randn(64, 1024, generator=torch.Generator().manual_seed(0)).to(torch.bfloat16)
    pa, sa = R.quantize(x.float().numpy(), R.E2M3)
    gp, gs = hk.quantize(x.cuda(), R.E2M3)
    np.testing.assert_array_equal(gs.cpu().numpy(), sa)
    np.testing.assert_array_equal(gp.cpu().numpy(), pa)


@pytest.mark.parametrize("fmt", [R.E2M3, R.E3M2])
def test_dequantize_bit_exact_all_codes_and_scales(fmt):
    rng = np.random.default_rng(1)
    codes = rng.integers(0, 64, size=(64, 512), dtype=np.uint8)
    codes[0, :64] = np.arange(64)
    packed = R.pack_codes(codes)
    scales = rng.integers(0, 255, size=(64, 16), dtype=np.uint8)
    scales[0, 0], scales[0, 1], scales[1, 0] = 0, 254, 127
    want = R.dequantize(packed, scales, fmt)
    got = hk.dequantize(torch.from_numpy(packed).cuda(), torch.from_numpy(scales).cuda(), fmt).cpu().numpy()
    np.testing.assert_array_equal(got.view(np.uint32), want.view(np.uint32))


def test_roundtrip_large_property():
    """quantise(dequantise(q)) == q at a size the oracle is not run on (64 Mi elements)."""
    x = torch.randn(8192, 8192, device="cuda", generator=torch.Generator(device="cuda").manual_seed(3))
    p, s = hk.quantize(x, R.E2M3)
    d = hk.dequantize(p, s, R.E2M3)
    p2, s2 = hk.quantize(d, R.E2M3)
    assert torch.equal(p, p2) and torch.equal(s, s2)
    assert hk.device_status() == 0


@pytest.mark.parametrize("fmt", [R.E4M3, R.E5M2])
@pytest.mark.parametrize("config", ["normal", "lognormal", "ffn"])
def test_fp8_quantize_bit_exact(fmt, config):
    A, B = R.make_inputs(config, 96, 200, 512, seed=7)
    for x in (A, B):
        pa, sa = R.quantize(x, fmt)
        gp, gs = hk.quantize(torch.from_numpy(x).cuda(), fmt)
        np.testing.assert_array_equal(gs.cpu().numpy(), sa)
        np.testing.assert_array_equal(gp.cpu().numpy(), pa)


@pytest.mark.parametrize("fmt", [R.E4M3, R.E5M2])
def test_fp8_dequantize_bit_exact(fmt):
    rng = np.random.default_rng(2)
    codes = rng.integers(0, 256, size=(32, 512), dtype=np.uint8)
    codes[0, :256] = np.arange(256)
    scales = rng.integers(1, 254, size=(32, 16), dtype=np.uint8)
    want = R.dequantize(codes, scales, fmt)
    got = hk.dequantize(torch.from_numpy(codes).cuda(), torch.from_numpy(scales).cuda(), fmt).cpu().numpy()
    fin = np.isfinite(want)
    np.testing.assert_array_equal(got[fin].view(np.uint32), want[fin].view(np.uint32))
    assert (np.isnan(got) == np.isnan(want)).all()
