"""CPU tests of the oracle itself: format tables, rounding, packing, the two implementations against
each other and against the CUDA-toolkit known answers."""
import json
import os

import numpy as np
import pytest

from oracle import mxfp6_ref as R

GOLD = os.path.join(os.path.dirname(__file__), "golden")


def _f32(bits):
    return np.array(bits, dtype=np.uint32).view(np.float32)


@pytest.fixture(scope="module")
def kat():
    with open(os.path.join(GOLD, "toolkit_fp6_kat.json")) as f:
        return json.load(f)


def test_decode_tables_match_toolkit(kat):
    np.testing.assert_array_equal(R.decode_table(R.E2M3), _f32(kat["decode_e2m3"]))
    np.testing.assert_array_equal(R.decode_table(R.E3M2), _f32(kat["decode_e3m2"]))
    L = R.c_oracle()
    for c in range(64):
        assert L.mxfp6_decode_elem(c, 0) == R.decode_table(R.E2M3)[c]
        assert L.mxfp6_decode_elem(c, 1) == R.decode_table(R.E3M2)[c]


def test_format_extremes():
    t2, t3 = R.decode_table(R.E2M3), R.decode_table(R.E3M2)
    assert t2[31] == 7.5 and t2[1] == 0.125 and t2[8] == 1.0 and t2[63] == -7.5
    assert t3[31] == 28.0 and t3[1] == 0.0625 and t3[4] == 0.25 and t3[63] == -28.0
    assert len(set(np.abs(t2).tolist())) == 32 and len(set(np.abs(t3).tolist())) == 32


def test_encode_matches_toolkit(kat):
    enc = np.array(kat["encode"], dtype=np.uint32)
    x = enc[:, 0].copy().view(np.float32)
    np.testing.assert_array_equal(R.encode_elems(x, R.E2M3), enc[:, 1].astype(np.uint8))
    np.testing.assert_array_equal(R.encode_elems(x, R.E3M2), enc[:, 2].astype(np.uint8))
    L = R.c_oracle()
    got2 = np.array([L.mxfp6_encode_elem(float(v), 0) for v in x], dtype=np.uint8)
    got3 = np.array([L.mxfp6_encode_elem(float(v), 1) for v in x], dtype=np.uint8)
    np.testing.assert_array_equal(got2, enc[:, 1].astype(np.uint8))
    np.testing.assert_array_equal(got3, enc[:, 2].astype(np.uint8))


def test_encode_ties_saturation_subnormals():
    e = lambda v, f: int(R.encode_elems(np.array([v], np.float32), f)[0])
    # ties to even: 0.0625 is halfway 0 / 0.125 -> 0 ; 0.1875 halfway 0.125/0.25 -> 0.25 (code 2)
    assert e(0.0625, R.E2M3) == 0 and e(0.1875, R.E2M3) == 2
    assert e(7.5, R.E2M3) == 31 and e(7.75, R.E2M3) == 31 and e(7.99, R.E2M3) == 31 and e(1e9, R.E2M3) == 31
    assert e(-7.9, R.E2M3) == 63
    assert e(28.0, R.E3M2) == 31 and e(30.0, R.E3M2) == 31 and e(31.99, R.E3M2) == 31 and e(-1e9, R.E3M2) == 63
    assert e(0.03125, R.E3M2) == 0 and e(0.09375, R.E3M2) == 2  # ties
    assert e(-0.0, R.E2M3) == 32 and e(-1e-9, R.E3M2) == 32      # sign of zero kept


def test_encode_decode_idempotent():
    for f in (R.E2M3, R.E3M2):
        t = R.decode_table(f)
        codes = R.encode_elems(t, f)
        np.testing.assert_array_equal(codes, np.arange(64, dtype=np.uint8))


def test_e8m0(kat):
    import torch
    b = np.arange(255, dtype=np.uint8)
    ref = torch.from_numpy(b.copy()).view(torch.float8_e8m0fnu).to(torch.float32).numpy()
    np.testing.assert_array_equal(R.e8m0_decode(b), ref)
    L = R.c_oracle()
    for x in (0, 1, 126, 127, 128, 254):
        assert L.mxfp6_e8m0_decode(x) == ref[x]
    assert np.isnan(R.e8m0_decode(np.array([255], np.uint8))[0])
    # floor(log2) pinned by the toolkit's round-toward-zero float->e8m0
    fl = np.array(kat["e8m0_floor"], dtype=np.uint32)
    x = fl[:, 0].copy().view(np.float32)
    for fmt, emax in ((R.E2M3, 2), (R.E3M2, 4)):
        want = np.clip(fl[:, 1].astype(np.int64) - emax, 0, 254).astype(np.uint8)
        np.testing.assert_array_equal(R.scale_bytes_from_amax(x, fmt), want)
        got = np.array([L.mxfp6_e8m0_from_amax(float(v), fmt) for v in x], np.uint8)
        np.testing.assert_array_equal(got, want)
    assert R.scale_bytes_from_amax(np.array([0.0], np.float32), R.E2M3)[0] == 0


def test_pack_byte_level_kat():
    # element i occupies bits [6i, 6i+6) of the little-endian byte string
    codes = np.array([[0x3f, 0, 0, 0], [0, 0x3f, 0, 0], [0, 0, 0x3f, 0], [0, 0, 0, 0x3f], [1, 2, 3, 4]], np.uint8)
    want = np.array([[0x3f, 0, 0], [0xc0, 0x0f, 0], [0, 0xf0, 0x03], [0, 0, 0xfc], [0x81, 0x30, 0x10]], np.uint8)
    np.testing.assert_array_equal(R.pack_codes(codes), want)
    np.testing.assert_array_equal(R.unpack_codes(want), codes)


def test_pack_roundtrip_and_c_agreement():
    rng = np.random.default_rng(0)
    codes = rng.integers(0, 64, size=(7, 256), dtype=np.uint8)
    p = R.pack_codes(codes)
    assert p.shape == (7, 192)
    np.testing.assert_array_equal(R.unpack_codes(p), codes)
    import ctypes
    L = R.c_oracle()
    out = np.empty(192, np.uint8)
    L.mxfp6_pack(codes[0].ctypes.data_as(ctypes.POINTER(ctypes.c_uint8)), 256, out.ctypes.data_as(ctypes.POINTER(ctypes.c_uint8)))
    np.testing.assert_array_equal(out, p[0])
    back = np.empty(256, np.uint8)
    L.mxfp6_unpack(out.ctypes.data_as(ctypes.POINTER(ctypes.c_uint8)), 256, back.ctypes.data_as(ctypes.POINTER(ctypes.c_uint8)))
    np.testing.assert_array_equal(back, codes[0])
    # random bytes round-trip through unpack -> pack
    raw = rng.integers(0, 256, size=(3, 96), dtype=np.uint8)
    np.testing.assert_array_equal(R.pack_codes(R.unpack_codes(raw)), raw)


@pytest.mark.parametrize("fmt", [R.E2M3, R.E3M2])
@pytest.mark.parametrize("config", ["normal", "lognormal", "ffn", "decode"])
def test_quantize_numpy_equals_c(fmt, config):
    A, B = R.make_inputs(config, 48, 40, 256, seed=3)
    for x in (A, B):
        p1, s1 = R.quantize(x, fmt)
        p2, s2 = R.c_quantize(x, fmt)
        np.testing.assert_array_equal(s1, s2)
        np.testing.assert_array_equal(p1, p2)
        np.testing.assert_array_equal(R.dequantize(p1, s1, fmt), R.c_dequantize(p1, s1, fmt))


@pytest.mark.parametrize("fmt", [R.E2M3, R.E3M2])
def test_quantize_block_rules(fmt):
    K = 128
    x = np.zeros((6, K), np.float32)
    x[0, :32] = 0.0                      # all-zero block
    x[1, :32] = 1.0                      # amax exactly a power of two
    x[2, :32] = np.linspace(-3.99, 3.99, 32)
    x[3, 0] = 7.9 if fmt == R.E2M3 else 31.0   # lands in the saturation gap after scaling
    x[4, :32] = 1e-30
    x[5, 5] = -0.0
    p, s = R.quantize(x, fmt)
    emax = 2 if fmt == R.E2M3 else 4
    assert s[0, 0] == 0 and (R.unpack_codes(p)[0, :32] == 0).all()
    assert s[1, 0] == 127 - emax
    assert s[2, 0] == 127 + 1 - emax
    d = R.dequantize(p, s, fmt)
    # saturated element decodes to max * scale, never wraps
    assert d[3, 0] == (7.5 if fmt == R.E2M3 else 28.0) * 2.0 ** (int(s[3, 0]) - 127)
    assert R.unpack_codes(p)[5, 5] == 32
    # quantise(dequantise(q)) == q
    p2, s2 = R.quantize(d, fmt)
    nz = np.abs(d.reshape(6, K // 32, 32)).max(-1) > 0
    np.testing.assert_array_equal(s2[nz], s[nz])
    np.testing.assert_array_equal(R.unpack_codes(p2).reshape(6, -1, 32)[nz], R.unpack_codes(p).reshape(6, -1, 32)[nz])
    # relative error of in-range values bounded by half an ulp of the format
    rel = np.abs(d[2, :32] - x[2, :32]).max() / 4.0
    assert rel <= 2.0 ** -(4 if fmt == R.E2M3 else 3)


def test_gemm_oracles_agree():
    A, B = R.make_inputs("lognormal", 33, 24, 256, seed=1)
    pa, sa = R.quantize(A, R.E2M3)
    pb, sb = R.quantize(B, R.E2M3)
    cb, cf, ad = R.c_gemm_ref(pa, sa, pb, sb, acc_mode=0, want_absdot=True)
    cb64, cf64, _ = R.c_gemm_ref(pa, sa, pb, sb, acc_mode=1)
    ct, ct32 = R.gemm_ref_torch(pa, sa, pb, sb, return_f32=True)
    rep = R.error_report(R.bf16_bits_to_f32(cb), cf64, ad)
    assert rep["row_rel"] < 1e-2 and rep["max_ulp"] <= 1.0
    rep_t = R.error_report(ct.float().numpy(), cf64, ad)
    assert rep_t["row_rel"] < 1e-2 and rep_t["max_ulp"] <= 1.0
    # bf16 rounding helper equals torch's
    import torch
    np.testing.assert_array_equal(cb, torch.from_numpy(cf).to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16))


def test_mixed_format_gemm():
    A, B = R.make_inputs("ffn", 8, 16, 128, seed=2)
    pa, sa = R.quantize(A, R.E3M2)
    pb, sb = R.quantize(B, R.E2M3)
    _, cf, _ = R.c_gemm_ref(pa, sa, pb, sb, fmt_a=R.E3M2, fmt_b=R.E2M3, acc_mode=1)
    want = R.dequantize(pa, sa, R.E3M2).astype(np.float64) @ R.dequantize(pb, sb, R.E2M3).astype(np.float64).T
    np.testing.assert_allclose(cf, want, rtol=1e-6)


# ------------------------------------------------------------------------------- MX-FP8 operands
@pytest.fixture(scope="module")
def kat8():
    with open(os.path.join(GOLD, "toolkit_fp8_kat.json")) as f:
        return json.load(f)


def test_fp8_decode_tables_match_toolkit_and_torch(kat8):
    import torch
    for fmt, key, tdt in ((R.E4M3, "decode_e4m3", torch.float8_e4m3fn), (R.E5M2, "decode_e5m2", torch.float8_e5m2)):
        mine = R.decode_table(fmt)
        tk = _f32(kat8[key])
        th = torch.arange(256, dtype=torch.uint8).view(tdt).float().numpy()
        fin = np.isfinite(mine)
        np.testing.assert_array_equal(mine[fin], tk[fin])
        np.testing.assert_array_equal(mine[fin], th[fin])
        assert (np.isnan(mine) == np.isnan(th)).all()
        L = R.c_oracle()
        for c in range(256):
            v = L.mxfp6_decode_elem(c, fmt)
            assert (np.isnan(v) and np.isnan(mine[c])) or v == mine[c]


def test_fp8_encode_matches_toolkit(kat8):
    enc = np.array(kat8["encode"], dtype=np.uint32)
    x = enc[:, 0].copy().view(np.float32)
    np.testing.assert_array_equal(R.encode_elems(x, R.E4M3), enc[:, 1].astype(np.uint8))
    np.testing.assert_array_equal(R.encode_elems(x, R.E5M2), enc[:, 2].astype(np.uint8))
    L = R.c_oracle()
    got4 = np.array([L.mxfp6_encode_elem(float(v), R.E4M3) for v in x], dtype=np.uint8)
    got5 = np.array([L.mxfp6_encode_elem(float(v), R.E5M2) for v in x], dtype=np.uint8)
    np.testing.assert_array_equal(got4, enc[:, 1].astype(np.uint8))
    np.testing.assert_array_equal(got5, enc[:, 2].astype(np.uint8))


@pytest.mark.parametrize("fmt", [R.E4M3, R.E5M2])
def test_fp8_quantize_numpy_equals_c_and_block_rule(fmt):
    A, _ = R.make_inputs("lognormal", 40, 8, 256, seed=4)
    p1, s1 = R.quantize(A, fmt)
    p2, s2 = R.c_quantize(A, fmt)
    assert p1.shape == (40, 256)
    np.testing.assert_array_equal(s1, s2)
    np.testing.assert_array_equal(p1, p2)
    np.testing.assert_array_equal(R.dequantize(p1, s1, fmt), R.c_dequantize(p1, s1, fmt))
    x = np.zeros((2, 64), np.float32)
    x[0, :32] = 1.0
    x[1, 0] = 500.0 if fmt == R.E4M3 else 60000.0     # scaled value lands between max and the next power of two
    p, s = R.quantize(x, fmt)
    emax = 8 if fmt == R.E4M3 else 15
    assert s[0, 0] == 127 - emax
    d = R.dequantize(p, s, fmt)
    assert d[1, 0] == (448.0 if fmt == R.E4M3 else 57344.0) * 2.0 ** (int(s[1, 0]) - 127)
    p2, s2 = R.quantize(d, fmt)
    np.testing.assert_array_equal(p2[0, :32], p[0, :32])


def test_mixed_fp8_fp6_gemm_oracles_agree():
    A, B = R.make_inputs("ffn", 8, 16, 128, seed=2)
    pa, sa = R.quantize(A, R.E4M3)
    pb, sb = R.quantize(B, R.E2M3)
    _, cf, _ = R.c_gemm_ref(pa, sa, pb, sb, fmt_a=R.E4M3, fmt_b=R.E2M3, acc_mode=1)
    want = R.dequantize(pa, sa, R.E4M3).astype(np.float64) @ R.dequantize(pb, sb, R.E2M3).astype(np.float64).T
    np.testing.assert_allclose(cf, want, rtol=1e-6)
