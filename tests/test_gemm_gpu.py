"""GPU parity tests of the MX-FP6 GEMM against the CPU oracle, through the C ABI.

Tolerances (the path's stated bar): per row, max_n |C-C_ref| / ||C_ref[r,:]||_2 <= 1e-2, and no element
further than 2 bf16 ulp from the oracle, where the oracle is the fp64-accumulated product of the exactly
dequantised operands and elements whose error lies inside the fp32 accumulation noise floor
(2^-20 * sum_k |a_k b_k|) are excused and counted."""
import os

import numpy as np
import pytest
import torch

import hipkittensp_b200 as hk
from oracle import mxfp6_ref as R
from tests.gpu_util import check, oracle_f64, quantized_inputs, run_gpu

pytestmark = pytest.mark.gpu


@pytest.fixture(autouse=True)
def _clean_env():
    yield
    hk.debug_option("MXFP6_FORCE_CFG", None)
    hk.debug_option("MXFP6_NO_SF_TMA", None)


def _case(config, M, N, K, fmt=R.E2M3, seed=0, force=None, fmt_b=None):
    if force:
        hk.debug_option("MXFP6_FORCE_CFG", force)
    pa, sa, pb, sb = quantized_inputs(config, M, N, K, fmt, seed, fmt_b)
    c = run_gpu(pa, sa, pb, sb, fmt, fmt_b)
    ref, absdot = oracle_f64(pa, sa, pb, sb, fmt, fmt_b)
    return check(c, ref, absdot)


def test_tma_image_of_packed_fp6():
    """The 6-bit tensor-map type expands each 12-byte group of 16 codes to a 16-byte slot; the packed
    stream is little-endian, 6 bits per element.  Pins the global packing against the hardware."""
    rows, K = 128, 256
    codes = (np.arange(K)[None, :] + np.arange(rows)[:, None]) % 64
    packed = torch.from_numpy(R.pack_codes(codes.astype(np.uint8))).cuda()
    for k0 in (0, 128):
        img = hk.tma_dump(packed, 0, k0).cpu().numpy()
        assert hk.device_status() == 0
        for r in range(rows):
            rowb = img[r * 128:(r + 1) * 128].reshape(8, 16)
            un = np.stack([rowb[c ^ (r % 8)] for c in range(8)])       # undo the 128-byte swizzle
            got = R.unpack_codes(un[:, :12].reshape(1, -1))[0]
            np.testing.assert_array_equal(got, codes[r, k0:k0 + 128])


def test_single_tile_unit_scales():
    hk.debug_option("MXFP6_FORCE_CFG", "128,0,0")
    pa, sa, pb, sb = quantized_inputs("normal", 128, 128, 128)
    sa[:] = 127
    sb[:] = 127
    c = run_gpu(pa, sa, pb, sb, R.E2M3)
    ref, absdot = oracle_f64(pa, sa, pb, sb, R.E2M3)
    check(c, ref, absdot)


def test_identity_operand_exposes_layout():
    """B = identity-like one-hot rows: C[m,n] must reproduce A[m,n] exactly (any operand- or scale-layout
    mistake permutes or rescales it)."""
    hk.debug_option("MXFP6_FORCE_CFG", "128,0,0")
    M = N = K = 256
    A, _ = R.make_inputs("lognormal", M, N, K, seed=5)
    pa, sa = R.quantize(A, R.E2M3)
    pb, sb = R.quantize(np.eye(N, K, dtype=np.float32), R.E2M3)
    c = run_gpu(pa, sa, pb, sb, R.E2M3)
    want = torch.from_numpy(R.dequantize(pa, sa, R.E2M3)).to(torch.bfloat16).float().numpy()
    np.testing.assert_array_equal(c, want)


def test_distinct_power_of_two_scales_per_block():
    hk.debug_option("MXFP6_FORCE_CFG", "128,0,0")
    M, N, K = 128, 128, 1024
    pa, sa, pb, sb = quantized_inputs("normal", M, N, K, seed=2)
    rng = np.random.default_rng(0)
    sa[:] = rng.integers(110, 140, size=sa.shape, dtype=np.uint8)
    sb[:] = rng.integers(110, 140, size=sb.shape, dtype=np.uint8)
    c = run_gpu(pa, sa, pb, sb, R.E2M3)
    ref, absdot = oracle_f64(pa, sa, pb, sb, R.E2M3)
    check(c, ref, absdot)


@pytest.mark.parametrize("K", [128, 256, 384, 512, 1024])
def test_k_sweep(K):
    _case("lognormal", 128, 128, K, force="128,0,0")


@pytest.mark.parametrize("force", ["128,0,0", "256,0,0", "128,0,1", "256,0,1"])
def test_tile_configs(force):
    _case("lognormal", 384, 768, 1024, force=force, seed=1)


@pytest.mark.parametrize("M", [1, 16, 17, 127, 129])
def test_ragged_m(M):
    _case("normal", M, 384, 512, seed=M)


@pytest.mark.parametrize("N", [16, 64, 128, 200, 520])
def test_ragged_n(N):
    _case("normal", 160, N, 512, seed=N)


def test_scale_plain_load_path():
    hk.debug_option("MXFP6_NO_SF_TMA", "1")
    _case("lognormal", 256, 256, 1024, seed=4)


@pytest.mark.parametrize("shape", [(512, 768, 640), (300, 520, 384), (1536, 1792, 1152)])
def test_pair_kernel_scale_plain_load_path(shape):
    """K / 32 not a multiple of 16: the scale rows cannot be TMA boxes, the CTA-pair kernel reads them with plain
    loads (forced on the small shapes, chosen by itself on the large one)."""
    M, N, K = shape
    _case("lognormal", M, N, K, seed=K, force=None if M * N >= 1536 * 1792 else "256,0,0,1")


def test_pair_kernel_scale_plain_load_path_unaligned_scales():
    hk.debug_option("MXFP6_NO_SF_TMA", "1")
    _case("lognormal", 512, 768, 1024, seed=6, force="256,0,0,1")


@pytest.mark.parametrize("M,N,K", [(16, 296 * 80, 512), (1, 296 * 80 + 40, 384), (32, 296 * 90 + 8, 640), (7, 50000, 256),
                                   (64, 148 * 160, 512), (128, 148 * 200 + 24, 384), (48, 46000, 256)])
def test_even_rows_forms(M, N, K):
    """Skinny M against many weight rows: the weight rows are dealt evenly to the CTAs (tiles of 48..128 rows of B in
    the swapped form for M <= 32, column tiles of a multiple of 8 between 128 and 256 in the unswapped form), including
    tile counts that do not divide N and more than one tile per CTA (N above 296 x 128)."""
    _case("decode", M, N, K, seed=M + N)


def test_even_rows_form_matches_k_split_form():
    """Both skinny forms on the same problem: equal up to the summation order of split tiles."""
    pa, sa, pb, sb = quantized_inputs("decode", 16, 296 * 88, 1024, seed=3)
    c1 = run_gpu(pa, sa, pb, sb, R.E2M3)
    hk.debug_option("MXFP6_DECODE_ROWS", "0")
    try:
        c0 = run_gpu(pa, sa, pb, sb, R.E2M3)
    finally:
        hk.debug_option("MXFP6_DECODE_ROWS", None)
    assert np.median(np.abs(c1 - c0)) == 0.0
    assert (c1 != c0).mean() < 2e-2


@pytest.mark.parametrize("M,N,K,fmt", [(4096, 4096, 512, R.E2M3),        # 256 tiles on 74 pairs: 34 left over, 2 slices each
                                       (2304, 2560, 256, R.E3M2),        # 90 tiles: 16 left over, 4 slices each
                                       (2204, 2500, 384, R.E2M3)])       # the same with ragged edges and plain-load scales
def test_pair_kernel_tail_slices(M, N, K, fmt):
    """The tiles left over after the last full wave of the CTA-pair kernel are cut into column slices.  Every element is
    still accumulated over K in one accumulator, so the result is bit for bit that of whole tiles."""
    pa, sa, pb, sb = quantized_inputs("lognormal", M, N, K, fmt, seed=M)
    c = run_gpu(pa, sa, pb, sb, fmt)
    ref, absdot = oracle_f64(pa, sa, pb, sb, fmt)
    check(c, ref, absdot)
    hk.debug_option("MXFP6_TAIL_SPLIT", "0")
    try:
        c_whole = run_gpu(pa, sa, pb, sb, fmt)
    finally:
        hk.debug_option("MXFP6_TAIL_SPLIT", None)
    np.testing.assert_array_equal(c, c_whole)


@pytest.mark.parametrize("shape,force", [((512, 772, 512), "256,0,0,1"), ((300, 514, 384), "256,0,0,1"), ((1536, 1797, 256), None)])
def test_pair_kernel_plain_store_path(shape, force):
    """N not a multiple of 8: rows of C are not 16-byte multiples, so C cannot be a TMA destination and the CTA-pair
    kernel writes its staged pieces with plain stores."""
    M, N, K = shape
    _case("lognormal", M, N, K, seed=N, force=force)


@pytest.mark.parametrize("shape", [(512, 768, 512), (300, 520, 384)])
def test_pair_kernel_plain_store_path_16_byte_rows(shape):
    """The plain-store epilogue where C's rows are 16-byte multiples (16 bytes per lane), forced by the test switch."""
    M, N, K = shape
    hk.debug_option("MXFP6_C_PLAIN", "1")
    try:
        _case("lognormal", M, N, K, seed=N + 1, force="256,0,0,1")
    finally:
        hk.debug_option("MXFP6_C_PLAIN", None)


@pytest.mark.parametrize("shape,force", [((64, 29600, 256), None),           # unswapped skinny form: 148 tiles of 200 columns, 3 whole pieces each
                                         ((128, 29600, 256), None),          # every row of the tile live
                                         ((96, 23680, 256), None),           # 160-column tiles: 2 whole pieces and a 32-column rest
                                         ((100, 1024, 384), "256,0,0"),      # rows past M clipped by the store
                                         ((300, 520, 384), "256,0,0"),       # ragged edges, tiles of the last row block clipped
                                         ((1536, 1792, 256), "128,0,0"),     # BN = 128, several tiles per CTA: only the last is staged
                                         ((2304, 2560, 256), "256,0,1")])    # K-split form: the last visited piece is a whole tile
def test_single_cta_last_tile_leaves_by_tma(shape, force):
    """The unswapped single-CTA kernel drains the last tile of every CTA through its idle ring and TMA stores; the
    values are those of the plain stores, bit for bit, and nothing outside C is written."""
    M, N, K = shape
    if force:
        hk.debug_option("MXFP6_FORCE_CFG", force)
    try:
        pa, sa, pb, sb = quantized_inputs("lognormal", M, N, K, seed=M + N)
        c = run_gpu(pa, sa, pb, sb, R.E2M3)
        ref, absdot = oracle_f64(pa, sa, pb, sb, R.E2M3)
        check(c, ref, absdot)
        hk.debug_option("MXFP6_C_TMA_LAST", "0")
        c_plain = run_gpu(pa, sa, pb, sb, R.E2M3)
    finally:
        hk.debug_option("MXFP6_C_TMA_LAST", None)
        hk.debug_option("MXFP6_FORCE_CFG", None)
    np.testing.assert_array_equal(c, c_plain)


@pytest.mark.parametrize("shape,strip,spp", [((4352, 2304, 512), 4, 2),      # 2 row groups, strips of 4, 4 and 1 tiles, sliced last wave
                                             ((2000, 2568, 256), 2, 1),      # ragged edges, one copy stream per peer
                                             ((2304, 2560, 256), 16, 2)])    # one block per row group
def test_copy_gather_on_one_gpu(shape, strip, spp):
    """`mxfp6_gemm_copy_gather` with the "peers" on the same GPU: the kernel writes destination 0 and raises a flag per
    finished block; copy streams wait for the flags and copy the blocks into the other destinations' column windows.
    Every destination ends with the plain GEMM's result bit for bit and nothing outside its window is touched.  Two
    calls in a row: the second starts from flags the first left set."""
    M, N, K = shape
    pa, sa, pb, sb = quantized_inputs("lognormal", M, N, K, seed=N)
    t = [torch.from_numpy(x).cuda() for x in (pa, sa, pb, sb)]
    want = torch.empty((M, N), dtype=torch.bfloat16, device="cuda")
    hk.dispatch_micro(t[0], t[2], want, t[1], t[3], R.E2M3)
    ldc, off, n_dst = N + 264, 136, 3
    streams = [torch.cuda.Stream() for _ in range(spp * (n_dst - 1))]
    scratch = torch.zeros(hk.copy_gather_scratch_bytes(M, N, strip) // 4, dtype=torch.int32, device="cuda")
    for _ in range(2):
        dests = [torch.full((M, ldc), float("nan"), dtype=torch.bfloat16, device="cuda") for _ in range(n_dst)]
        hk.dispatch_copy_gather(t[0], t[2], dests, off, t[1], t[3], scratch, streams, strip, R.E2M3)
        reader = [d[:, off:off + N].clone() for d in dests]      # queued on the launching stream, no host synchronisation
        torch.cuda.synchronize()
        assert hk.device_status() == 0
        for d, r in zip(dests, reader):
            assert torch.equal(r.view(torch.int16), want.view(torch.int16))
            assert torch.isnan(d[:, :off]).all() and torch.isnan(d[:, off + N:]).all(), "write outside the window"
    ref, absdot = oracle_f64(pa, sa, pb, sb, R.E2M3)
    check(want.float().cpu().numpy(), ref, absdot)


def test_copy_gather_refuses_what_it_cannot_signal():
    """Problems that do not run on the CTA-pair kernel have no per-block flags: the call says so and queues nothing."""
    M, N, K = 64, 1024, 256
    pa, sa, pb, sb = quantized_inputs("normal", M, N, K, seed=3)
    t = [torch.from_numpy(x).cuda() for x in (pa, sa, pb, sb)]
    dests = [torch.zeros((M, N), dtype=torch.bfloat16, device="cuda") for _ in range(2)]
    scratch = torch.zeros(64, dtype=torch.int32, device="cuda")
    with pytest.raises(RuntimeError, match="CTA-pair kernel"):
        hk.dispatch_copy_gather(t[0], t[2], dests, 0, t[1], t[3], scratch, [torch.cuda.Stream()], 8, R.E2M3)
    torch.cuda.synchronize()


def test_pair_kernel_plain_store_odd_window():
    """Several destinations whose column window starts at an odd element of rows with an odd stride."""
    hk.debug_option("MXFP6_FORCE_CFG", "256,0,0,1")
    M, N, K = 300, 520, 256
    pa, sa, pb, sb = quantized_inputs("lognormal", M, N, K, seed=12)
    t = [torch.from_numpy(x).cuda() for x in (pa, sa, pb, sb)]
    ldc, off = N + 263, 137
    dests = [torch.full((M, ldc), float("nan"), dtype=torch.bfloat16, device="cuda") for _ in range(2)]
    hk.dispatch_multi(t[0], t[2], dests, off, t[1], t[3], R.E2M3)
    assert hk.device_status() == 0
    ref, absdot = oracle_f64(pa, sa, pb, sb, R.E2M3)
    for d in dests:
        check(d[:, off:off + N].float().cpu().numpy(), ref, absdot)
        assert torch.isnan(d[:, :off]).all() and torch.isnan(d[:, off + N:]).all(), "write outside the window"


def test_zero_and_max_blocks():
    M, N, K = 128, 128, 256
    A, B = R.make_inputs("normal", M, N, K, seed=9)
    A[:, :32] = 0.0
    B[5, :] = 0.0
    A[7, 32:64] = 7.5 * 2.0 ** 20
    pa, sa = R.quantize(A, R.E2M3)
    pb, sb = R.quantize(B, R.E2M3)
    c = run_gpu(pa, sa, pb, sb, R.E2M3)
    ref, absdot = oracle_f64(pa, sa, pb, sb, R.E2M3)
    check(c, ref, absdot)
    assert (c[:, 5] == 0).all()


def test_config_cpu_runnable_1024_cubed():
    rep = _case("normal", 1024, 1024, 1024)
    assert rep["n_1pct"] < 0.02 * 1024 * 1024


def test_config_e3m2_ffn_shape_reduced():
    _case("ffn", 512, 1792, 2048, fmt=R.E3M2)


def test_mixed_formats():
    _case("ffn", 256, 256, 512, fmt=R.E3M2, fmt_b=R.E2M3)


@pytest.mark.parametrize("M", [1, 16, 64])
def test_config_decode_reduced(M):
    _case("decode", M, 3584, 2048, seed=M)


def test_skinny_full_k_many_tiles():
    _case("decode", 16, 28672, 1024)


def test_tk_kernel_module():
    import sys
    sys.path.insert(0, os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "hipkittensp_b200"))
    import tk_kernel
    pa, sa, pb, sb = quantized_inputs("normal", 256, 256, 512)
    t = [torch.from_numpy(x).cuda() for x in (pa, pb, sa, sb)]
    C = torch.empty(256, 256, dtype=torch.bfloat16, device="cuda")
    tk_kernel.dispatch_micro(t[0], t[1], C, t[2], t[3], 0)
    assert hk.device_status() == 0
    ref, absdot = oracle_f64(pa, sa, pb, sb, R.E2M3)
    check(C.float().cpu().numpy(), ref, absdot)


def test_repeat_calls_are_deterministic():
    pa, sa, pb, sb = quantized_inputs("decode", 16, 4096, 4096)
    c1 = run_gpu(pa, sa, pb, sb, R.E2M3)
    c2 = run_gpu(pa, sa, pb, sb, R.E2M3)
    np.testing.assert_array_equal(c1, c2)


@pytest.mark.parametrize("shape,force", [((512, 768, 1024), None), ((512, 768, 1024), "256,0,0,1"),
                                         ((300, 520, 512), "256,0,0,1"), ((64, 256, 512), None),
                                         ((1024, 512, 1024), "128,0,0,0")])
def test_multi_destination_column_window(shape, force):
    """mxfp6_gemm_multi: the block lands in the same column window of every destination and nowhere else."""
    M, N, K = shape
    if force:
        hk.debug_option("MXFP6_FORCE_CFG", force)
    pa, sa, pb, sb = quantized_inputs("lognormal", M, N, K, seed=11)
    t = [torch.from_numpy(x).cuda() for x in (pa, sa, pb, sb)]
    ldc, off = N + 264, 136
    dests = [torch.full((M, ldc), float("nan"), dtype=torch.bfloat16, device="cuda") for _ in range(3)]
    hk.dispatch_multi(t[0], t[2], dests, off, t[1], t[3], R.E2M3)
    assert hk.device_status() == 0
    ref, absdot = oracle_f64(pa, sa, pb, sb, R.E2M3)
    for d in dests:
        c = d[:, off:off + N].float().cpu().numpy()
        check(c, ref, absdot)
        assert torch.isnan(d[:, :off]).all() and torch.isnan(d[:, off + N:]).all(), "write outside the window"
    assert torch.equal(dests[0][:, off:off + N], dests[1][:, off:off + N])
    assert torch.equal(dests[0][:, off:off + N], dests[2][:, off:off + N])


@pytest.mark.parametrize("fmt", [R.E2M3, R.E4M3])
def test_host_gemm_pipeline_matches_direct_calls(fmt):
    """HostGemm: operands and results in pinned host memory, consecutive calls overlapped on three streams."""
    M, N, K = 256, 512, 1024
    sets = []
    for seed in range(3):
        pa, sa, pb, sb = quantized_inputs("lognormal", M, N, K, fmt, seed=seed)
        sets.append([torch.from_numpy(x).pin_memory() for x in (pa, sa, pb, sb)])
    pipe = hk.HostGemm(M, N, K, fmt=fmt)
    outs = [torch.empty((M, N), dtype=torch.bfloat16).pin_memory() for _ in range(6)]
    for i in range(6):
        h = sets[i % 3]
        pipe(h[0], h[1], h[2], h[3], outs[i])
    pipe.synchronize()
    assert hk.device_status() == 0
    for i in range(6):
        h = [t.cuda() for t in sets[i % 3]]
        want = hk.gemm(h[0], h[1], h[2], h[3], fmt).cpu()
        assert torch.equal(outs[i].view(torch.int16), want.view(torch.int16))


# ------------------------------------------------------------------------------- MX-FP8 operands
@pytest.mark.parametrize("fmt", [R.E4M3, R.E5M2])
@pytest.mark.parametrize("shape,force", [((256, 384, 512), None), ((512, 768, 1024), "256,0,0,1"),
                                         ((16, 2048, 1024), None), ((129, 200, 384), None)])
def test_fp8_operands(fmt, shape, force):
    M, N, K = shape
    _case("lognormal", M, N, K, fmt=fmt, seed=3, force=force)


@pytest.mark.parametrize("fa,fb", [(R.E4M3, R.E2M3), (R.E3M2, R.E5M2), (R.E2M3, R.E4M3)])
def test_mixed_fp8_fp6_operands(fa, fb):
    _case("ffn", 256, 512, 1024, fmt=fa, fmt_b=fb, seed=8)
    _case("decode", 16, 1024, 512, fmt=fa, fmt_b=fb, seed=9)


@pytest.mark.parametrize("M", [1, 16, 64])
def test_b_static_flag_back_to_back(M):
    """MXFP6_FLAG_B_STATIC: weights are requested before the preceding kernel has drained; results of
    back-to-back calls (each depending on nothing but its own inputs) stay bit-identical to the plain call."""
    N, K = 3584, 2048
    pa, sa, pb, sb = quantized_inputs("decode", M, N, K, seed=M)
    t = [torch.from_numpy(x).cuda() for x in (pa, sa, pb, sb)]
    want = hk.gemm(t[0], t[1], t[2], t[3])
    # with the L2 requests that every call makes while it waits (the promise then changes nothing), and without them
    # (the weights of the first stages are then loaded for real before the wait)
    for ahead in (None, "0"):
        hk.debug_option("MXFP6_L2_AHEAD", ahead)
        try:
            outs = [torch.full((M, N), float("nan"), dtype=torch.bfloat16, device="cuda") for _ in range(6)]
            for o in outs:                               # six launches queued without a host sync in between
                hk.dispatch_micro(t[0], t[2], o, t[1], t[3], R.E2M3, b_static=True)
            assert hk.device_status() == 0
        finally:
            hk.debug_option("MXFP6_L2_AHEAD", None)
        for o in outs:
            assert torch.equal(o.view(torch.int16), want.view(torch.int16))
    ref, absdot = oracle_f64(pa, sa, pb, sb, R.E2M3)
    check(want.float().cpu().numpy(), ref, absdot)


@pytest.mark.parametrize("M,N,K", [(16, 296 * 82, 1024), (32, 296 * 97, 512),
                                   (64, 148 * 200, 1024), (128, 148 * 160, 512),     # unswapped skinny forms: the weights are the Q operand
                                   (384, 1280, 1024)])                                # single-CTA tiles of a small unswapped problem
def test_b_static_flag_even_rows_form(M, N, K):
    """The same promise in the even-rows skinny forms (two CTAs per SM with rotated K loops; unswapped with the weights
    as the second operand) and in a small unswapped problem."""
    pa, sa, pb, sb = quantized_inputs("decode", M, N, K, seed=M)
    t = [torch.from_numpy(x).cuda() for x in (pa, sa, pb, sb)]
    want = hk.gemm(t[0], t[1], t[2], t[3])
    for ahead in (None, "0"):
        hk.debug_option("MXFP6_L2_AHEAD", ahead)
        try:
            outs = [torch.full((M, N), float("nan"), dtype=torch.bfloat16, device="cuda") for _ in range(6)]
            for o in outs:
                hk.dispatch_micro(t[0], t[2], o, t[1], t[3], R.E2M3, b_static=True)
            assert hk.device_status() == 0
        finally:
            hk.debug_option("MXFP6_L2_AHEAD", None)
        for o in outs:
            assert torch.equal(o.view(torch.int16), want.view(torch.int16))
    ref, absdot = oracle_f64(pa, sa, pb, sb, R.E2M3)
    check(want.float().cpu().numpy(), ref, absdot)


# ------------------------------------------------------------------------------- re-quantising epilogue
def _exact_inputs(M, N, K, seed):
    """Operands whose products and partial sums are small integers times a power of two: every accumulation order
    gives the same fp32 result, so the fused quantiser must agree with the oracle bit for bit."""
    rng = np.random.default_rng(seed)
    A = rng.integers(-3, 4, size=(M, K)).astype(np.float32)
    B = rng.integers(-3, 4, size=(N, K)).astype(np.float32)
    A *= 2.0 ** rng.integers(-2, 3, size=(M, 1))
    B *= 2.0 ** rng.integers(-2, 3, size=(N, 1))
    return A, B


@pytest.mark.parametrize("out_fmt", [R.E2M3, R.E3M2, R.E4M3, R.E5M2])
@pytest.mark.parametrize("shape,force", [((256, 512, 512), None), ((512, 768, 1024), "256,0,0,1"),
                                         ((130, 192, 256), None), ((16, 256, 512), None), ((16, 4096, 2048), None),
                                         ((64, 2048, 1024), None), ((100, 1024, 512), None), ((16, 512, 256), "16,1,0"),
                                         ((33, 1024, 1024), "64,1,1")])
def test_requant_epilogue_bit_exact_on_exact_sums(out_fmt, shape, force):
    M, N, K = shape
    if force:
        hk.debug_option("MXFP6_FORCE_CFG", force)
    A, B = _exact_inputs(M, N, K, seed=M + out_fmt)
    pa, sa = R.quantize(A, R.E2M3)
    pb, sb = R.quantize(B, R.E2M3)
    c32 = (R.dequantize(pa, sa, R.E2M3).astype(np.float64) @ R.dequantize(pb, sb, R.E2M3).astype(np.float64).T).astype(np.float32)
    want_p, want_s = R.quantize(c32, out_fmt)
    t = [torch.from_numpy(x).cuda() for x in (pa, sa, pb, sb)]
    got_p, got_s = hk.gemm_requant(t[0], t[1], t[2], t[3], R.E2M3, out_fmt=out_fmt)
    assert hk.device_status() == 0
    np.testing.assert_array_equal(got_s.cpu().numpy(), want_s)
    np.testing.assert_array_equal(got_p.cpu().numpy(), want_p)


def test_requant_epilogue_random_inputs_within_one_step():
    """On general inputs the fp32 sums differ in the last bits from the oracle's, so a value may land on the
    neighbouring code; after dequantisation the two results agree to within one quantisation step."""
    M, N, K = 512, 1024, 2048
    pa, sa, pb, sb = quantized_inputs("lognormal", M, N, K, seed=21)
    ref, _ = oracle_f64(pa, sa, pb, sb, R.E2M3)
    want_p, want_s = R.quantize(ref.astype(np.float32), R.E4M3)
    t = [torch.from_numpy(x).cuda() for x in (pa, sa, pb, sb)]
    got_p, got_s = hk.gemm_requant(t[0], t[1], t[2], t[3], R.E2M3, out_fmt=R.E4M3)
    assert hk.device_status() == 0
    got = R.dequantize(got_p.cpu().numpy(), got_s.cpu().numpy(), R.E4M3)
    want = R.dequantize(want_p, want_s, R.E4M3)
    step = 2.0 ** (want_s.astype(np.int32) - 127 + 8 - 3).repeat(32, axis=1)     # coarsest e4m3 spacing in the block
    assert (np.abs(got - want) <= step).all()
    assert (got_s.cpu().numpy() == want_s).mean() > 0.999
    # and it feeds the next GEMM directly: layer 2 = requantised activations [M, N] x W2 [256, N]
    W2, _ = R.make_inputs("normal", 256, 8, N, seed=5)
    pw, sw = R.quantize(W2, R.E4M3)
    C2 = hk.gemm(got_p, got_s, torch.from_numpy(pw).cuda(), torch.from_numpy(sw).cuda(), R.E4M3, fmt_b=R.E4M3)
    assert hk.device_status() == 0
    ref2 = got.astype(np.float64) @ R.dequantize(pw, sw, R.E4M3).astype(np.float64).T
    absdot2 = np.abs(got).astype(np.float64) @ np.abs(R.dequantize(pw, sw, R.E4M3)).astype(np.float64).T
    check(C2.float().cpu().numpy(), ref2, absdot2)


def test_bounded_wait_reports_and_context_survives():
    """Failure path without a fault: a wait that nothing satisfies runs out after its budget (1 ms here), the
    kernel returns, the status word names the waiter, and the GPU keeps working."""
    import time
    assert hk.device_status() == 0
    t0 = time.perf_counter()
    _lib_check = hk._lib.check
    _lib_check(hk.lib.mxfp6_debug_wait_timeout(1000, None))
    with pytest.raises(hk.Mxfp6Error) as ei:
        hk.device_status()
    assert time.perf_counter() - t0 < 2.0
    assert ei.value.code == hk._lib.ERR_DEVICE_WAIT and "role 9" in str(ei.value)
    assert hk.device_status() == 0                      # the status word was cleared
    _case("normal", 256, 256, 512)                      # and the context is still usable


# ------------------------------------------------------------------------------- scaled / biased epilogue
@pytest.mark.parametrize("shape,force", [((256, 384, 512), None), ((512, 768, 1024), "256,0,0,1"), ((130, 200, 256), None),
                                         ((16, 1024, 2048), None), ((64, 520, 1024), None), ((256, 512, 512), "256,0,0")])
@pytest.mark.parametrize("which", ["all", "row", "col", "bias"])
def test_scaled_epilogue_bit_exact_on_exact_sums(shape, force, which):
    """(acc * scale_b[n]) * scale_a[m] + bias[n], three fp32 roundings then bf16: with operands whose sums are exact
    in every order the result must equal the same arithmetic done on the CPU, bit for bit."""
    M, N, K = shape
    if force:
        hk.debug_option("MXFP6_FORCE_CFG", force)
    A, B = _exact_inputs(M, N, K, seed=7 * M + N)
    pa, sa = R.quantize(A, R.E2M3)
    pb, sb = R.quantize(B, R.E2M3)
    acc = (R.dequantize(pa, sa, R.E2M3).astype(np.float64) @ R.dequantize(pb, sb, R.E2M3).astype(np.float64).T).astype(np.float32)
    rng = np.random.default_rng(M + N)
    row = rng.lognormal(0, 1, M).astype(np.float32) if which in ("all", "row") else None
    col = rng.lognormal(0, 1, N).astype(np.float32) if which in ("all", "col") else None
    bias = rng.normal(0, 30, N).astype(np.float32) if which in ("all", "bias") else None
    want = acc
    if col is not None:
        want = want * col[None, :]
    if row is not None:
        want = want * row[:, None]
    if bias is not None:
        want = want + bias[None, :]
    assert want.dtype == np.float32
    want = torch.from_numpy(want).to(torch.bfloat16).float().numpy()
    t = [torch.from_numpy(x).cuda() for x in (pa, sa, pb, sb)]
    dev = lambda v: None if v is None else torch.from_numpy(v).cuda()
    C = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device="cuda")
    hk.gemm_scaled(t[0], t[1], t[2], t[3], dev(row), dev(col), dev(bias), R.E2M3, out=C)
    assert hk.device_status() == 0
    np.testing.assert_array_equal(C.float().cpu().numpy(), want)


def test_scaled_epilogue_k_zero_gives_bias():
    bias = torch.arange(64, dtype=torch.float32, device="cuda") - 7.25
    e = torch.empty((8, 0), dtype=torch.uint8, device="cuda")
    f = torch.empty((64, 0), dtype=torch.uint8, device="cuda")
    C = hk.gemm_scaled(e, e.clone(), f, f.clone(), None, None, bias, R.E2M3)
    torch.testing.assert_close(C.float(), bias.to(torch.bfloat16).float().expand(8, 64), rtol=0, atol=0)


def test_scaled_epilogue_argument_checks():
    pa, sa, pb, sb = [torch.from_numpy(x).cuda() for x in quantized_inputs("normal", 128, 128, 256)]
    with pytest.raises(RuntimeError, match="128 elements"):
        hk.gemm_scaled(pa, sa, pb, sb, torch.ones(64, device="cuda"))
    with pytest.raises(RuntimeError, match="fp32"):
        hk.gemm_scaled(pa, sa, pb, sb, None, torch.ones(128, device="cuda", dtype=torch.bfloat16))


# ------------------------------------------------------------------------------- reference-style harness
def test_reference_style_harness_runs_and_checks(capsys):
    from hipkittensp_b200 import harness
    harness.check_gemm((256, 384, 512))
    harness.check_gemm((16, 1024, 1024), fmt=R.E3M2)
    tf = harness.bench_gemm({"shape": (512, 512, 512)}, None, num_warmup=3, num_iter=3)
    assert tf > 0
    assert "m=512,n=512,k=512:" in capsys.readouterr().out


# ------------------------------------------------------------------------------- CUDA graph capture
@pytest.mark.parametrize("shape", [(256, 512, 512), (16, 2048, 2048), (512, 768, 1024)])
def test_calls_can_be_captured_in_a_cuda_graph(shape):
    """After one eager call (one-time set-up: attributes, scratch), the launch is plain stream work: capture it,
    replay it on new operand contents, and compare with an eager call."""
    M, N, K = shape
    pa, sa, pb, sb = [torch.from_numpy(x).cuda() for x in quantized_inputs("normal", M, N, K, seed=5)]
    C = torch.empty((M, N), dtype=torch.bfloat16, device="cuda")
    hk.dispatch_micro(pa, pb, C, sa, sb, R.E2M3)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        hk.dispatch_micro(pa, pb, C, sa, sb, R.E2M3)
    # new contents in the same buffers
    qa, ta, qb, tb = [torch.from_numpy(x).cuda() for x in quantized_inputs("normal", M, N, K, seed=6)]
    pa.copy_(qa); sa.copy_(ta); pb.copy_(qb); sb.copy_(tb)
    C.fill_(float("nan"))
    g.replay()
    g.replay()
    torch.cuda.synchronize()
    want = torch.empty_like(C)
    hk.dispatch_micro(pa, pb, want, sa, sb, R.E2M3)
    assert hk.device_status() == 0
    assert torch.equal(C, want)


_SCRATCH_GROWTH = r"""
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
small, big = (16, 4096, 4096), (64, 38400, 1024)      # both split tiles along K; the second needs more than the first 8 MiB
assert 0 < hk.lib.mxfp6_gemm_workspace_bytes(*small) <= (8 << 20) < hk.lib.mxfp6_gemm_workspace_bytes(*big)
pa, sa, pb, sb = operands(*small, 1)
qa, ta, qb, tb = operands(*big, 2)
C = torch.empty(small[:2], dtype=torch.bfloat16, device="cuda")
D = torch.empty(big[:2], dtype=torch.bfloat16, device="cuda")
hk.dispatch_micro(pa, pb, C, sa, sb)                   # eager: the library allocates its first scratch buffer
torch.cuda.synchronize()
want = C.clone()
g = torch.cuda.CUDAGraph()
with torch.cuda.graph(g):
    hk.dispatch_micro(pa, pb, C, sa, sb)               # the graph now holds that buffer's address
    # a shape that needs a larger buffer cannot get one during capture: refused with a message, the capture survives
    try:
        hk.dispatch_micro(qa, qb, D, ta, tb)
        raise SystemExit("growth during capture was not refused")
    except _lib.Mxfp6Error as e:
        assert e.code == _lib.ERR_BAD_ARG and "being captured" in str(e), str(e)
hk.dispatch_micro(qa, qb, D, ta, tb)                   # outside the capture the library adds a larger buffer ...
torch.cuda.synchronize()
C.fill_(float("nan"))
g.replay(); g.replay()                                 # ... and the graph still replays into the old one, which was not freed
torch.cuda.synchronize()
assert hk.device_status() == 0
assert torch.equal(C.view(torch.int16), want.view(torch.int16))
E = torch.empty_like(D)
hk.dispatch_micro(qa, qb, E, ta, tb)
torch.cuda.synchronize()
assert torch.equal(D.view(torch.int16), E.view(torch.int16))
print("SCRATCH_GROWTH_OK")
"""


def test_scratch_is_never_freed_under_a_captured_graph():
    """A CUDA graph captured earlier keeps the scratch address it was given; a later, larger shape gets an additional
    buffer (the old one stays), and asking for one while a stream is being captured is refused with a message."""
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    out = subprocess.run([sys.executable, "-c", _SCRATCH_GROWTH, root], capture_output=True, text=True, timeout=600)
    assert "SCRATCH_GROWTH_OK" in out.stdout, out.stdout[-2000:] + out.stderr[-2000:]


# ------------------------------------------------------------------------------- empty dimensions
def test_empty_dimensions():
    """M = 0 or N = 0: nothing to do, success.  K = 0: an empty sum, C is written as zeros."""
    dev = "cuda"
    u8 = lambda r, c: torch.empty((r, c), dtype=torch.uint8, device=dev)
    C = torch.full((8, 64), float("nan"), dtype=torch.bfloat16, device=dev)
    hk.dispatch_micro(u8(8, 0), u8(64, 0), C, u8(8, 0), u8(64, 0), R.E2M3)          # K = 0
    assert hk.device_status() == 0
    assert torch.equal(C.float(), torch.zeros(8, 64, device=dev))
    hk.dispatch_micro(u8(0, 96), u8(64, 96), torch.empty((0, 64), dtype=torch.bfloat16, device=dev), u8(0, 4), u8(64, 4), R.E2M3)   # M = 0
    hk.dispatch_micro(u8(8, 96), u8(0, 96), torch.empty((8, 0), dtype=torch.bfloat16, device=dev), u8(8, 4), u8(0, 4), R.E2M3)     # N = 0
    p, s = hk.quantize(torch.empty((0, 64), dtype=torch.float32, device=dev), R.E2M3)
    assert p.shape == (0, 48) and s.shape == (0, 2)
    assert hk.device_status() == 0


# ------------------------------------------------------------------------------- C++ host harness over the C ABI
@pytest.mark.parametrize("args", [["512", "768", "1024", "0", "5", "10", "8"], ["16", "2048", "1024", "1", "3", "5", "16"],
                                  ["256", "256", "512", "2", "3", "5", "4"]])
def test_cpp_host_harness(args):
    import subprocess
    exe = os.path.join(os.path.dirname(hk.__file__), "matmul_host")
    res = subprocess.run([exe] + args, capture_output=True, text=True, timeout=300)
    assert res.returncode == 0, res.stdout + res.stderr
    assert "TFLOP/s" in res.stdout and res.stdout.strip().endswith("OK")


# ------------------------------------------------------------------------------- seeded random shapes
def _random_shapes(n, seed):
    rng = np.random.default_rng(seed)
    shapes = []
    for _ in range(n):
        M = int(rng.choice([1, 7, 16, 33, 64, 100, 128, 129, 255, 256, 300, 512, 777, 1024, 1500, 2304]))
        N = int(rng.choice([8, 16, 72, 128, 200, 256, 264, 512, 1000, 1024, 2048, 2312, 4096]))
        K = int(rng.choice([128, 256, 384, 512, 640, 1024, 1536, 2048]))
        shapes.append((M, N, K))
    return shapes


@pytest.mark.parametrize("shape", _random_shapes(40, seed=2024), ids=lambda s: "x".join(map(str, s)))
def test_random_shapes_against_oracle(shape):
    """Shapes on both sides of every kernel-choice boundary (M <= 128 swap, pair-kernel threshold, TMA-able scale
    rows, vector-store alignment), mixed formats by seed, all against the fp64 oracle."""
    M, N, K = shape
    fmts = [(R.E2M3, R.E2M3), (R.E3M2, R.E3M2), (R.E2M3, R.E3M2), (R.E4M3, R.E2M3)]
    fa, fb = fmts[(M + N + K) % 4]
    pa, sa, pb, sb = quantized_inputs("lognormal" if (M * N) % 3 == 0 else "normal", M, N, K, fa, seed=M + 3 * N + K, fmt_b=fb)
    c = run_gpu(pa, sa, pb, sb, fa, fb)
    ref, absdot = oracle_f64(pa, sa, pb, sb, fa, fb)
    check(c, ref, absdot)
