"""Host-side planning logic, without a GPU: for every problem shape the tiling the library chooses must cover each
element of C exactly once.  The kernels' schedules (tile order of the single-CTA kernel, units of the CTA-pair kernel with
the column slices of its last partial wave) are restated here from the plan's numbers and replayed on the CPU."""
import itertools

import numpy as np
import pytest

from hipkittensp_b200 import _lib

SM = 148


def _cover_single(pl, M, N):
    """Rows/columns of C each tile of the single-CTA kernel stores (gemm_kernel.cuh: SegIter::coords and the store guards)."""
    cover = np.zeros((M, N), np.int32)
    prow, qrow = (N, M) if pl["swap"] else (M, N)
    for tp, tq in itertools.product(range(pl["tiles_p"]), range(pl["tiles_q"])):
        p0, q0 = tp * pl["p_tile"], tq * pl["q_tile"]
        p1, q1 = min(p0 + min(pl["p_tile"], 128), prow), min(q0 + min(pl["q_tile"], pl["bn"]), qrow)
        if pl["swap"]:
            cover[q0:q1, p0:p1] += 1
        else:
            cover[p0:p1, q0:q1] += 1
    return cover


def _cover_pair(pl, M, N):
    """Units of the CTA-pair kernel (gemm_kernel_2cta.cuh: pair_unit): whole 256 x 256 tiles, then column slices."""
    cover = np.zeros((M, N), np.int32)
    clusters = pl["grid"] // 2
    tiles = pl["tiles_p"] * pl["tiles_q"]
    group_p = 16

    def coords(t):
        per_group = group_p * pl["tiles_q"]
        group, inn = divmod(t, per_group)
        first_p = group * group_p
        gsz = min(pl["tiles_p"] - first_p, group_p)
        return (first_p + inn % gsz) * 256, (inn // gsz) * 256

    units_per_cluster = []
    for c in range(clusters):
        n = 0
        it = 0
        while True:
            t = c + it * clusters
            if t < pl["tail_first"]:
                p0, q0, ncols = *coords(t), 256
            else:
                idx = t - pl["tail_first"]
                if idx >= (tiles - pl["tail_first"]) * pl["tail_split"]:
                    break
                p0, q0 = coords(pl["tail_first"] + idx // pl["tail_split"])
                ncols = 256 // pl["tail_split"]
                q0 += (idx % pl["tail_split"]) * ncols
            cover[p0:min(p0 + 256, M), q0:min(q0 + ncols, N)] += 1
            n += ncols / 256
            it += 1
        units_per_cluster.append(n)
    return cover, units_per_cluster


SHAPES = [(8192, 8192, 8192), (4096, 4096, 4096), (4096, 14336, 8192), (16384, 7168, 8192), (2304, 2560, 256),
          (2204, 2500, 384), (1, 28672, 8192), (16, 28672, 8192), (32, 28672, 8192), (64, 28672, 8192), (128, 28672, 8192),
          (16, 57344, 1024), (7, 38000, 256), (16, 4096, 4096), (48, 37960, 256), (96, 23680, 512), (130, 200, 256),
          (300, 514, 384), (1536, 1797, 256), (257, 9999, 128), (33, 1024, 1024), (16, 296 * 80, 512), (16, 14336, 8192)]


@pytest.mark.parametrize("M,N,K", SHAPES)
def test_plan_covers_c_exactly_once(M, N, K):
    pl = _lib.debug_plan(M, N, K, SM)
    assert pl["grid"] >= 1 and pl["ctas"] in (1, 2)
    assert pl["grid"] <= SM * pl["ctas"]
    if pl["pair"]:
        assert pl["grid"] % 2 == 0 and pl["tail_split"] in (1, 2, 4)
        cover, per_cluster = _cover_pair(pl, M, N)
        # the slices exist to even out the last wave: no pair gets more than one tile's worth above the lightest
        assert max(per_cluster) - min(per_cluster) <= 1.0
    else:
        if pl["streamk"]:
            assert pl["p_tile"] == 128 and pl["q_tile"] == pl["bn"]        # split tiles keep the fixed tile shape
        if pl["ctas"] == 2:
            assert pl["swap"] and not pl["streamk"] and pl["bn"] <= 32 and 80 <= pl["p_tile"] <= 128
        if not pl["swap"] and pl["q_tile"] != pl["bn"]:
            assert pl["q_tile"] % 8 == 0 and 128 <= pl["q_tile"] <= 256
        cover = _cover_single(pl, M, N)
    assert (cover == 1).all(), f"{int((cover != 1).sum())} elements of C are covered {cover.min()}..{cover.max()} times"


def test_even_rows_forms_are_chosen_for_the_decode_configuration():
    for M in (1, 16):
        pl = _lib.debug_plan(M, 28672, 8192, SM)
        assert pl["swap"] and pl["ctas"] == 2 and not pl["streamk"] and pl["p_tile"] == 97 and pl["grid"] == 296
    pl = _lib.debug_plan(64, 28672, 8192, SM)
    assert not pl["swap"] and pl["bn"] == 256 and pl["q_tile"] == 200 and pl["grid"] == 144
    # a re-quantised result needs tiles on multiples of 32: the fixed tile shapes stay
    pl = _lib.debug_plan(16, 28672, 8192, SM, requant=True)
    assert pl["ctas"] == 1 and pl["p_tile"] == 128


def test_tail_slices_of_the_pair_kernel():
    pl = _lib.debug_plan(4096, 4096, 4096, SM)
    assert pl["pair"] and pl["tail_split"] == 2 and pl["tail_first"] == 222          # 256 tiles = 3 x 74 + 34
    pl = _lib.debug_plan(8192, 8192, 8192, SM)
    assert pl["pair"] and pl["tail_split"] == 1 and pl["tail_first"] == 1024         # 62 left over: more than half the pairs
    pl = _lib.debug_plan(2304, 2560, 256, SM)
    assert pl["pair"] and pl["tail_split"] == 4 and pl["tail_first"] == 74           # 90 tiles = 74 + 16


def test_several_destinations_use_whole_untransposed_tiles():
    pl = _lib.debug_plan(64, 28672, 8192, SM, n_dst=3)
    assert not pl["swap"] and not pl["streamk"] and pl["ctas"] == 1
