// CTA-pair variant of the MX-FP6 GEMM for large problems: two CTAs of a cluster (one per SM) share one
// 256x256 output tile through tcgen05 cta_group::2.
//
//   CTA rank r of the pair owns P rows p0+128r.. (its half of A, its 128x256 fp32 accumulator in its own
//   TMEM, its half of the epilogue) and loads Q rows q0+128r.. (its half of B); the 256-row MMA issued by
//   the even CTA reads A from both CTAs' shared memory and the two halves of B from the CTA that holds them.
//
// Per K-block of 128 each SM therefore loads 128+128 rows (24 KB of packed fp6) instead of 128+256, and a
// pipeline stage is 32 KB, so 5 stages plus two 16 KB output staging buffers fit where the single-CTA kernel
// has 4 stages.  The epilogue packs bf16 into the staging buffers (128-byte swizzle) and one thread issues a
// TMA store of each 128x64 piece to every destination of C: the local copy and, in the sharded
// configuration, the copies held by the peer GPUs, so the gather travels with the tiles.
//
// Synchronisation (all mbarriers live in shared memory of the CTA named):
//   full[s]      even CTA   1 arrival (+ bytes of both CTAs' TMA loads)        waited by the MMA thread
//   empty[s]     each CTA   1 arrival by multicast tcgen05.commit               waited by that CTA's producer
//   raw_full/raw_empty[r]  each CTA, local scale-slab ring
//   atom_full[g] even CTA   2 arrivals (the scale warp of each CTA), one per group of 4 K-blocks
//   atom_empty[g] each CTA  1 arrival by multicast commit
//   acc_full[b]  each CTA   1 arrival by multicast commit                       waited by that CTA's epilogue
//   ovl          even CTA   8 arrivals (epilogue warps of both CTAs)             waited by the MMA thread
#pragma once
#include "gemm_kernel.cuh"

namespace mxfp6 {

struct PairCfg {
    static constexpr int BM = 128;                        // P rows per CTA (256 per pair)
    static constexpr int BN = 256;                        // Q rows per pair (128 loaded by each CTA)
    static constexpr int BK = 128;
    static constexpr int P_BYTES = BM * BK;               // 16 KB
    static constexpr int Q_BYTES = (BN / 2) * BK;         // 16 KB: this CTA's half of B
    static constexpr int STAGE_BYTES = P_BYTES + Q_BYTES;
    // 5 stages of 32 KB; a sixth (paid for with a single 8 KB staging buffer and two scale-atom groups) measured
    // no faster: throughput rises from 3 to 4 to 5 stages and is flat beyond
    static constexpr int STAGES = 5;
    static constexpr int OUT_COLS = 64;                   // output staging: two buffers of 128 rows x 64 columns
    static constexpr int OUT_BUFS = 2;
    static constexpr int OUT_BYTES = BM * OUT_COLS * 2;
    static constexpr int RAW_SLOTS = 2;
    static constexpr int RAW_BYTES = (BM + BN) * 16;      // own P rows + all 256 Q rows, 16 scale bytes each
    static constexpr int ATOM_BYTES = 512 * 3;            // P atom + two Q atoms of one K-block
    static constexpr int GROUP_BYTES = 4 * ATOM_BYTES;    // the 4 K-blocks one raw slab covers
    static constexpr int ATOM_GROUPS = 3;
    static constexpr int ACC_COL1 = 224;
    static constexpr int SF_COL = 480;
    static constexpr int TMEM_COLS = 512;
    static constexpr int NUM_BARS = 2 * STAGES + 2 * RAW_SLOTS + 2 * ATOM_GROUPS + 3;
    static constexpr int AFF_BYTES = 2 * BN * 4;          // column scale and bias of the current tile (fp32 epilogue)
    static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + OUT_BUFS * OUT_BYTES + RAW_SLOTS * RAW_BYTES +
                                      ATOM_GROUPS * GROUP_BYTES + NUM_BARS * 8 + 64 + 16 + AFF_BYTES;
    static constexpr int SMEM_ALLOC = SMEM_BYTES + 1024;
    static constexpr int THREADS = 256;
    static_assert(SMEM_ALLOC <= 232448, "exceeds the shared memory of a CTA");
};

// bounded wait on a barrier that CTAs of the pair arrive on remotely
__device__ __forceinline__ bool wait_bar_cluster(uint32_t bar, uint32_t parity, volatile int* abort_flag,
                                                 const GemmParams& P, int code) {
    if (mbar_try_wait_cluster(bar, parity)) return true;
    long long t0 = clock64();
    uint32_t n = 0;
    while (!mbar_try_wait_cluster(bar, parity)) {
        if ((++n & 255u) == 0) {
            if (*abort_flag) return false;
            if ((unsigned long long)(clock64() - t0) > P.wait_cycles) {
                *abort_flag = 1;
                atomicCAS(P.status, 0, code | ((int)blockIdx.x << 8));
                return false;
            }
        }
    }
    return true;
}
__device__ __forceinline__ bool wait_bar_cluster_warp(uint32_t bar, uint32_t parity, volatile int* abort_flag,
                                                      const GemmParams& P, int code) {
    return __all_sync(0xffffffffu, wait_bar_cluster(bar, parity, abort_flag, P, code));
}

// Tensor maps of the destinations of C (this GEMM's [M,N] block inside each copy, bf16, box 64 x 128, 128-byte swizzle)
struct CMaps {
    CUtensorMap m[8];
};

// Pair tile t -> first P row / Q row of the pair.  tiles_p/tiles_q in P count 256x256 pair tiles.
__device__ __forceinline__ void pair_coords(const GemmParams& P, int t, int& p0, int& q0) {
    const int per_group = P.group_p * P.tiles_q;
    const int group = t / per_group, in = t % per_group;
    const int first_p = group * P.group_p;
    const int gsz = min(P.tiles_p - first_p, P.group_p);
    p0 = (first_p + in % gsz) * 256;
    q0 = (in / gsz) * 256;
}

// One unit of work of a pair: a whole 256x256 tile, or, in the last partial wave of a problem, a 256 x 128 or 256 x 64
// column slice of one, so that the tiles that are left over when the tile count is not a multiple of the number of
// pairs spread over more pairs.  A slice is an independent piece of C with the full K loop: nothing is summed across
// units, and every element is accumulated exactly as in a whole tile.
struct PairUnit {
    int p0, q0;      // first row of A / first row of B (column of C) of the unit
    int ncols;       // columns of C: 256, 128 or 64
};
// Unit number `it` of cluster `cluster_id`; false when the cluster has no more work.
__device__ __forceinline__ bool pair_unit(const GemmParams& P, int it, int cluster_id, int n_clusters, PairUnit& u) {
    const int t = cluster_id + it * n_clusters;
    if (t < P.tail_first) {
        pair_coords(P, t, u.p0, u.q0);
        u.ncols = 256;
        return true;
    }
    const int idx = t - P.tail_first;               // slices of the left-over tiles, tile-major
    if (idx >= (P.tiles_p * P.tiles_q - P.tail_first) * P.tail_split) return false;
    pair_coords(P, P.tail_first + idx / P.tail_split, u.p0, u.q0);
    u.ncols = 256 / P.tail_split;
    u.q0 += (idx % P.tail_split) * u.ncols;
    return true;
}

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(PairCfg::THREADS, 1)
mxfp6_gemm_pair_kernel(const __grid_constant__ CUtensorMap tm_p, const __grid_constant__ CUtensorMap tm_q,
                       const __grid_constant__ CUtensorMap tm_q_tail,
                       const __grid_constant__ CUtensorMap tm_sfp, const __grid_constant__ CUtensorMap tm_sfq,
                       const __grid_constant__ CMaps cmaps, const GemmParams P) {
    using Cfg = PairCfg;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));

    const uint32_t stage_base = smem_base;
    const uint32_t out_base = stage_base + Cfg::STAGES * Cfg::STAGE_BYTES;      // 1024-byte aligned
    const uint32_t raw_base = out_base + Cfg::OUT_BUFS * Cfg::OUT_BYTES;
    const uint32_t atom_base = raw_base + Cfg::RAW_SLOTS * Cfg::RAW_BYTES;
    const uint32_t bar_base = atom_base + Cfg::ATOM_GROUPS * Cfg::GROUP_BYTES;
    auto bar_full = [&](int s) { return bar_base + 8u * s; };
    auto bar_empty = [&](int s) { return bar_base + 8u * (Cfg::STAGES + s); };
    auto bar_raw_full = [&](int s) { return bar_base + 8u * (2 * Cfg::STAGES + s); };
    auto bar_raw_empty = [&](int s) { return bar_base + 8u * (2 * Cfg::STAGES + Cfg::RAW_SLOTS + s); };
    auto bar_atom_full = [&](int s) { return bar_base + 8u * (2 * Cfg::STAGES + 2 * Cfg::RAW_SLOTS + s); };
    auto bar_atom_empty = [&](int s) { return bar_base + 8u * (2 * Cfg::STAGES + 2 * Cfg::RAW_SLOTS + Cfg::ATOM_GROUPS + s); };
    const uint32_t bar_misc = bar_base + 8u * (2 * Cfg::STAGES + 2 * Cfg::RAW_SLOTS + 2 * Cfg::ATOM_GROUPS);
    auto bar_acc_full = [&](int b) { return bar_misc + 8u * b; };
    const uint32_t bar_ovl = bar_misc + 8u * 2;
    const uint32_t misc_off = (bar_base - smem_base) + Cfg::NUM_BARS * 8;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem_gen + misc_off);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem_gen + misc_off + 4);
    const uint32_t abort_addr = smem_base + misc_off + 4;
    float* aff_sn = reinterpret_cast<float*>(smem_gen + ((misc_off + 64 + 15) & ~15u));   // [256] column scales, then [256] biases (16-byte aligned)
    float* aff_bn = aff_sn + Cfg::BN;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    pdl_launch_dependents();     // the next kernel may set itself up on SMs this grid has left
    const uint32_t rank = cluster_ctarank();              // 0 = even CTA (issues the MMAs), 1 = its peer
    const bool leader = rank == 0;
    const int cluster_id = blockIdx.x >> 1, n_clusters = gridDim.x >> 1;

    if (threadIdx.x == 0) {
        for (int s = 0; s < Cfg::STAGES; ++s) { mbar_init(bar_full(s), 1); mbar_init(bar_empty(s), 1); }
        for (int s = 0; s < Cfg::RAW_SLOTS; ++s) { mbar_init(bar_raw_full(s), 1); mbar_init(bar_raw_empty(s), 32); }
        for (int s = 0; s < Cfg::ATOM_GROUPS; ++s) { mbar_init(bar_atom_full(s), 2); mbar_init(bar_atom_empty(s), 1); }
        for (int b = 0; b < 2; ++b) mbar_init(bar_acc_full(b), 1);
        mbar_init(bar_ovl, 8);
        *abort_flag = 0;
        fence_barrier_init();
    }
    if (warp == 0 && lane == 0) {
        tma_prefetch_desc(&tm_p); tma_prefetch_desc(&tm_q); tma_prefetch_desc(&tm_sfp); tma_prefetch_desc(&tm_sfq);
        if (P.tail_split > 1) tma_prefetch_desc(&tm_q_tail);
    }
    // Every thread arrives at the cluster's meeting point as soon as it can (thread 0 after it has initialised the
    // barriers): once the wait returns, the barriers of both CTAs are initialised, which is all the producer warp needs
    // before it signals the peer.  It does not wait for the TMEM allocation: it announces itself at the CTA's own meeting
    // point and goes on to request the first stages, everybody else meets there and picks up the TMEM address.
    __syncwarp();                // (warp 0 comes out of the one-thread blocks above)
    cluster_arrive();
    if (warp == 1) {
        tmem_alloc_pair(smem_u32(tmem_slot), Cfg::TMEM_COLS);
        tmem_relinquish_pair();
    }
    tc_fence_before();
    if (warp == 0) {
        __syncwarp();
        __threadfence_block();
        asm volatile("bar.arrive 2, 256;" ::: "memory");
    } else {
        asm volatile("bar.sync 2, 256;" ::: "memory");
    }
    cluster_wait();
    tc_fence_after();
    const uint32_t tmem_base = warp == 0 ? 0u : *tmem_slot;
    pdl_wait();                  // nothing above touches global memory; everything below may

    auto signal_abort_to_peer = [&]() { st_shared_cluster_u32(mapa_shared(abort_addr, rank ^ 1), 1u); };

    // =========================================================== warp 0: TMA producer (both CTAs)
    if (warp == 0) {
        uint32_t n_stage = 0, n_raw = 0;
        bool ok = true;
        const uint64_t pol_ld = l2_policy(P.l2_load);
        PairUnit u;
        for (int it = 0; ok && pair_unit(P, it, cluster_id, n_clusters, u); ++it) {
            const int p0 = u.p0, q0 = u.q0;
            const bool whole = u.ncols == 256;
            // each CTA brings its 128 rows of A and its half of the unit's rows of B
            const int my_p = p0 + 128 * (int)rank, my_q = q0 + (u.ncols >> 1) * (int)rank;
            const CUtensorMap* tq = whole ? &tm_q : &tm_q_tail;
            const uint32_t tx = whole ? (uint32_t)P.stage_tx_bytes : (uint32_t)P.stage_tx_bytes_tail;
            for (int kb = 0; kb < P.kblocks && ok; ++kb) {
                if (P.sf_tma && (kb & 3) == 0) {
                    const int r = n_raw % Cfg::RAW_SLOTS;
                    ok = wait_bar_warp(bar_raw_empty(r), ((n_raw / Cfg::RAW_SLOTS) & 1) ^ 1, abort_flag, P, kStatusTimeoutProducer);
                    if (!ok) break;
                    if (elect_one_sync()) {
                        const uint32_t dst = raw_base + r * Cfg::RAW_BYTES;
                        mbar_arrive_expect_tx(bar_raw_full(r), Cfg::RAW_BYTES);
                        tma_load_2d(dst, &tm_sfp, bar_raw_full(r), (kb >> 2) * 16, my_p);
                        tma_load_2d(dst + Cfg::BM * 16, &tm_sfq, bar_raw_full(r), (kb >> 2) * 16, q0);
                    }
                    ++n_raw;
                }
                const int s = n_stage % Cfg::STAGES;
                ok = wait_bar_warp(bar_empty(s), ((n_stage / Cfg::STAGES) & 1) ^ 1, abort_flag, P, kStatusTimeoutProducer);
                if (!ok) break;
                if (elect_one_sync()) {
                    const uint32_t dst = stage_base + s * Cfg::STAGE_BYTES;
                    const uint32_t full0 = mapa_shared(bar_full(s), 0);
                    // the even CTA announces the bytes of both CTAs' loads for this stage
                    {
                    if (leader) mbar_arrive_expect_tx(bar_full(s), 2u * tx);
                    tma_load_2d_pair_hint(dst, &tm_p, full0, kb * Cfg::BK, my_p, pol_ld);
                    tma_load_2d_pair_hint(dst + Cfg::P_BYTES, tq, full0, kb * Cfg::BK, my_q, pol_ld);
                    }
                }
                __syncwarp();
                ++n_stage;
            }
        }
        if (!ok && lane == 0) signal_abort_to_peer();
    }
    // =========================================================== warp 1: MMA issuer (even CTA only)
    else if (warp == 1) {
        if (leader) {
            uint32_t n_kb = 0, n_seg = 0, n_grp = 0;
            bool ok = true;
            PairUnit u;
            for (int it = 0; ok && pair_unit(P, it, cluster_id, n_clusters, u); ++it) {
                const int b = n_seg & 1;
                const uint32_t acc = tmem_base + (b ? Cfg::ACC_COL1 : 0);
                // the instruction's N is the unit's column count (bits 17..22 hold N / 8)
                const uint32_t idesc = (P.idesc & ~(0x3fu << 17)) | ((uint32_t)(u.ncols >> 3) << 17);
                if (n_seg > 0) ok = wait_bar_cluster_warp(bar_ovl, (n_seg - 1) & 1, abort_flag, P, kStatusTimeoutMma);
                if (!ok) break;
                tc_fence_after();
                for (int kb = 0; kb < P.kblocks; ++kb) {
                    const int s = n_kb % Cfg::STAGES;
                    const int g = n_grp % Cfg::ATOM_GROUPS;
                    if ((kb & 3) == 0)
                        ok = wait_bar_cluster_warp(bar_atom_full(g), (n_grp / Cfg::ATOM_GROUPS) & 1, abort_flag, P, kStatusTimeoutMma);
                    ok = ok && wait_bar_warp(bar_full(s), (n_kb / Cfg::STAGES) & 1, abort_flag, P, kStatusTimeoutMma);
                    if (!ok) break;
                    const bool group_done = (kb & 3) == 3 || kb == P.kblocks - 1;
                    if (elect_one_sync()) {
                        const uint32_t sfa = tmem_base + Cfg::SF_COL + (n_kb & 1) * 16;
                        const uint32_t sfb = sfa + 4;
                        const uint32_t atom = atom_base + g * Cfg::GROUP_BYTES + (kb & 3) * Cfg::ATOM_BYTES;
                        {
                        tc_cp_32x128b_warpx4_pair(sfa, smem_desc_sf(atom));
                        tc_cp_32x128b_warpx4_pair(sfb, smem_desc_sf(atom + 512));
                        tc_cp_32x128b_warpx4_pair(sfb + 4, smem_desc_sf(atom + 1024));
                        }
                        const uint32_t sp = stage_base + s * Cfg::STAGE_BYTES;
                        const uint64_t adesc = smem_desc_sw128(sp);
                        const uint64_t bdesc = smem_desc_sw128(sp + Cfg::P_BYTES);
#pragma unroll
                        for (uint32_t k = 0; k < 4; ++k) {
                            mma_mxf8f6f4_pair(acc, adesc + 2 * k, bdesc + 2 * k, idesc_with_sf(idesc, k),
                                              sfa | (k << 30), sfb | (k << 30), (kb > 0 || k > 0) ? 1u : 0u);
                        }
                        tc_commit_pair(bar_empty(s), 3);
                        if (group_done) tc_commit_pair(bar_atom_empty(g), 3);
                    }
                    __syncwarp();
                    ++n_kb;
                    if (group_done) ++n_grp;
                }
                if (!ok) break;
                if (elect_one_sync()) tc_commit_pair(bar_acc_full(b), 3);
                __syncwarp();
                ++n_seg;
            }
            if (!ok && lane == 0) signal_abort_to_peer();
        }
    }
    // =========================================================== warps 2-3: scale re-tilers (both CTAs)
    // groups of 4 K-blocks alternate between the two warps; each CTA builds the atoms of its own P rows and
    // of all 256 Q rows (the scale copy into TMEM runs in both CTAs from their own shared memory)
    else if (warp == 2 || warp == 3) {
        uint32_t n_grp = 0;
        bool ok = true;
        PairUnit u;
        for (int it = 0; ok && pair_unit(P, it, cluster_id, n_clusters, u); ++it) {
            for (int kb = 0; kb < P.kblocks && ok; kb += 4, ++n_grp) {
                if ((int)(n_grp & 1) != warp - 2) continue;
                uint32_t rp[4][4], rq[8][4];
                if (P.sf_tma) {
                    const int r = n_grp % Cfg::RAW_SLOTS;
                    ok = wait_bar_warp(bar_raw_full(r), (n_grp / Cfg::RAW_SLOTS) & 1, abort_flag, P, kStatusTimeoutScale);
                    if (!ok) break;
                    const uint8_t* raw = smem_gen + (raw_base - smem_base) + r * Cfg::RAW_BYTES;
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        const uint4 v = *reinterpret_cast<const uint4*>(raw + (lane + 32 * c) * 16);
                        rp[c][0] = v.x; rp[c][1] = v.y; rp[c][2] = v.z; rp[c][3] = v.w;
                    }
#pragma unroll
                    for (int c = 0; c < 8; ++c) {
                        const uint4 v = *reinterpret_cast<const uint4*>(raw + Cfg::BM * 16 + (lane + 32 * c) * 16);
                        rq[c][0] = v.x; rq[c][1] = v.y; rq[c][2] = v.z; rq[c][3] = v.w;
                    }
                    mbar_arrive(bar_raw_empty(r));
                } else {
                    // Scale rows that cannot be TMA boxes (K/32 not a multiple of 16, or unaligned arrays): the 4-byte
                    // words of the group's K-blocks are read from global memory directly.  Four adjacent lanes read the
                    // four words of one row (16 contiguous bytes), so an instruction touches 8 rows, not 32; each word goes
                    // straight to its place in the atom of its K-block: row (r % 32), 4-byte column (r / 32).
                    const int p0 = u.p0, q0 = u.q0;
                    const int w = lane & 3;
                    uint32_t v[48];
#pragma unroll
                    for (int i = 0; i < 48; ++i) {
                        const int ridx = 8 * i + (lane >> 2);           // 0..127: my rows of P, 128..383: the unit's rows of Q
                        const bool is_p = i < 16;
                        const int row = is_p ? p0 + 128 * (int)rank + ridx : q0 + ridx - 128;
                        const bool live = row < (is_p ? P.p_rows : P.q_rows) && kb + w < P.kblocks;
                        v[i] = live ? __ldg(reinterpret_cast<const uint32_t*>((is_p ? P.sfp : P.sfq) + (size_t)row * P.sf_ld + (kb + w) * 4)) : 0u;
                    }
                    const int g = n_grp % Cfg::ATOM_GROUPS;
                    ok = wait_bar_warp(bar_atom_empty(g), ((n_grp / Cfg::ATOM_GROUPS) & 1) ^ 1, abort_flag, P, kStatusTimeoutScale);
                    if (!ok) break;
                    uint8_t* atom = smem_gen + (atom_base - smem_base) + g * Cfg::GROUP_BYTES + w * Cfg::ATOM_BYTES;
#pragma unroll
                    for (int i = 0; i < 48; ++i) {
                        const int ridx = 8 * i + (lane >> 2);
                        const int part = ridx >> 7, r = ridx & 127;     // atom 0: P, atoms 1 and 2: Q rows 0..127 and 128..255
                        *reinterpret_cast<uint32_t*>(atom + 512 * part + (r & 31) * 16 + (r >> 5) * 4) = v[i];
                    }
                    fence_proxy_async_smem();
                    __syncwarp();
                    if (lane == 0) mbar_arrive_cluster(mapa_shared(bar_atom_full(g), 0));
                    continue;
                }
                const int g = n_grp % Cfg::ATOM_GROUPS;
                ok = wait_bar_warp(bar_atom_empty(g), ((n_grp / Cfg::ATOM_GROUPS) & 1) ^ 1, abort_flag, P, kStatusTimeoutScale);
                if (!ok) break;
                uint8_t* grp = smem_gen + (atom_base - smem_base) + g * Cfg::GROUP_BYTES;
#pragma unroll
                for (int jj = 0; jj < 4; ++jj) {
                    uint8_t* atom = grp + jj * Cfg::ATOM_BYTES;
                    *reinterpret_cast<uint4*>(atom + lane * 16) = make_uint4(rp[0][jj], rp[1][jj], rp[2][jj], rp[3][jj]);
                    *reinterpret_cast<uint4*>(atom + 512 + lane * 16) = make_uint4(rq[0][jj], rq[1][jj], rq[2][jj], rq[3][jj]);
                    *reinterpret_cast<uint4*>(atom + 1024 + lane * 16) = make_uint4(rq[4][jj], rq[5][jj], rq[6][jj], rq[7][jj]);
                }
                fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0) mbar_arrive_cluster(mapa_shared(bar_atom_full(g), 0));
            }
        }
        if (!ok && lane == 0) signal_abort_to_peer();
    }
    // =========================================================== warps 4-7: epilogue (both CTAs)
    else if (warp >= 4) {
        const int quad = warp & 3;
        const int prow = quad * 32 + lane;
        const int etid = threadIdx.x - 128;
        uint32_t n_seg = 0, n_out = 0;
        bool ok = true;
        const uint32_t ovl0 = mapa_shared(bar_ovl, 0);
        const uint64_t pol_st = l2_policy(P.l2_store);
        PairUnit u;
        for (int it = 0; ok && pair_unit(P, it, cluster_id, n_clusters, u); ++it) {
            const int p0 = u.p0, q0 = u.q0;
            const int b = n_seg & 1;
            const int my_p0 = p0 + 128 * (int)rank;
            const bool affine = has_affine(P);
            // fp32 epilogue: this thread's row factor and two of the tile's 256 column factors / biases are fetched
            // while the accumulator is still being computed
            float row_scale = 1.f;
            float2 col_scale = make_float2(1.f, 1.f), col_bias = make_float2(0.f, 0.f);
            if (affine) {
                const int c = q0 + 2 * etid;
                if (P.scale_m && my_p0 + prow < P.c_rows) row_scale = __ldg(P.scale_m + my_p0 + prow);
                if (P.scale_n) { if (c < P.c_cols) col_scale.x = __ldg(P.scale_n + c); if (c + 1 < P.c_cols) col_scale.y = __ldg(P.scale_n + c + 1); }
                if (P.bias_n) { if (c < P.c_cols) col_bias.x = __ldg(P.bias_n + c); if (c + 1 < P.c_cols) col_bias.y = __ldg(P.bias_n + c + 1); }
            }
            ok = epilogue_all(wait_bar_warp(bar_acc_full(b), (n_seg >> 1) & 1, abort_flag, P, kStatusTimeoutEpilogue));
            if (!ok) break;
            tc_fence_after();
            if (affine) {
                // (the agreement above was a barrier of these 128 threads: nobody still reads the previous tile's vectors)
                reinterpret_cast<float2*>(aff_sn)[etid] = col_scale;
                reinterpret_cast<float2*>(aff_bn)[etid] = col_bias;
                asm volatile("bar.sync 1, 128;" ::: "memory");
            }
            const uint32_t tacc = tmem_base + ((uint32_t)(quad * 32) << 16) + (b ? Cfg::ACC_COL1 : 0);
            constexpr int OC = Cfg::OUT_COLS;                 // columns per piece
            const int NP = u.ncols / OC;
#pragma unroll 1
            for (int ci = 0; ci < NP; ++ci) {
                // the piece that holds the 32 columns shared by the two accumulators goes first
                const int piece = b == 0 ? (ci + NP - 1) % NP : ci;
                const uint32_t buf = out_base + (n_out % Cfg::OUT_BUFS) * Cfg::OUT_BYTES;
                // accumulator columns first: the shared columns are released to the next tile's MMA as early as possible
                uint32_t v[OC];
#pragma unroll
                for (int h = 0; h < OC / 32; ++h) tmem_ld_x32(tacc + piece * OC + 32 * h, reinterpret_cast<uint32_t(&)[32]>(v[32 * h]));
                tmem_ld_wait();
                if (ci == 0) {
                    // one arrival per warp: every lane's loads are complete (wait::ld above) before the warp meets
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive_cluster(ovl0);
                }
                if (affine) {
                    // (acc * column scale) * row scale + bias, three roundings; the vectors are broadcast reads
#pragma unroll
                    for (int c = 0; c < OC; c += 4) {
                        const float4 sn = *reinterpret_cast<const float4*>(aff_sn + piece * OC + c);
                        const float4 bn = *reinterpret_cast<const float4*>(aff_bn + piece * OC + c);
                        v[c + 0] = __float_as_uint(__fadd_rn(__fmul_rn(__fmul_rn(__uint_as_float(v[c + 0]), sn.x), row_scale), bn.x));
                        v[c + 1] = __float_as_uint(__fadd_rn(__fmul_rn(__fmul_rn(__uint_as_float(v[c + 1]), sn.y), row_scale), bn.y));
                        v[c + 2] = __float_as_uint(__fadd_rn(__fmul_rn(__fmul_rn(__uint_as_float(v[c + 2]), sn.z), row_scale), bn.z));
                        v[c + 3] = __float_as_uint(__fadd_rn(__fmul_rn(__fmul_rn(__uint_as_float(v[c + 3]), sn.w), row_scale), bn.w));
                    }
                }
                // the stores that last used this staging buffer have finished reading it
                if (etid == 0) bulk_wait_group_read<Cfg::OUT_BUFS - 1>();
                asm volatile("bar.sync 1, 128;" ::: "memory");
                static_assert(OC == 64, "the staging layouts below assume pieces of 64 columns");
                if (P.q_fmt >= 0) {
                    // The result leaves as an MX operand of the next layer: this thread's 64 columns are two blocks of
                    // 32.  Their codes (2 x 24 or 2 x 32 bytes) are staged as one dense row of the piece and the piece
                    // is stored by TMA like a bf16 piece (cmaps.m[0] then describes the code bytes of the output).
                    const bool fp8 = P.q_fmt == kE4M3 || P.q_fmt == kE5M2;
                    const int row = my_p0 + prow;
                    uint32_t sbs = 0;
#pragma unroll
                    for (int hb = 0; hb < 2; ++hb) {
                        float f[32];
#pragma unroll
                        for (int i = 0; i < 32; ++i) f[i] = __uint_as_float(v[32 * hb + i]);
                        uint32_t w[8];
                        int sb;
                        if (P.q_fmt == kE2M3) sb = quant_block32<kE2M3>(f, w);
                        else if (P.q_fmt == kE3M2) sb = quant_block32<kE3M2>(f, w);
                        else if (P.q_fmt == kE4M3) sb = quant_block32<kE4M3>(f, w);
                        else sb = quant_block32<kE5M2>(f, w);
                        sbs |= (uint32_t)sb << (8 * hb);
                        if (fp8) {
                            // 64-byte rows, 64-byte swizzle: 16-byte chunk c sits at c ^ ((row / 2) % 4)
                            const uint32_t ra = buf + prow * 64, sw8 = (uint32_t)((prow >> 1) & 3);
                            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};"
                                         ::"r"(ra + (((2 * hb) ^ sw8) << 4)), "r"(w[0]), "r"(w[1]), "r"(w[2]), "r"(w[3]) : "memory");
                            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};"
                                         ::"r"(ra + (((2 * hb + 1) ^ sw8) << 4)), "r"(w[4]), "r"(w[5]), "r"(w[6]), "r"(w[7]) : "memory");
                        } else {
                            // 48-byte rows, no swizzle
                            const uint32_t ra = buf + prow * 48 + 24 * hb;
                            asm volatile("st.shared.v2.b32 [%0], {%1, %2};" ::"r"(ra), "r"(w[0]), "r"(w[1]) : "memory");
                            asm volatile("st.shared.v2.b32 [%0], {%1, %2};" ::"r"(ra + 8), "r"(w[2]), "r"(w[3]) : "memory");
                            asm volatile("st.shared.v2.b32 [%0], {%1, %2};" ::"r"(ra + 16), "r"(w[4]), "r"(w[5]) : "memory");
                        }
                    }
                    const int col = q0 + piece * OC;
                    if (row < P.c_rows && col < P.c_cols)
                        *reinterpret_cast<uint16_t*>(P.q_scales + (size_t)row * (P.c_cols / 32) + col / 32) = (uint16_t)sbs;
                    fence_proxy_async_smem();
                    asm volatile("bar.sync 1, 128;" ::: "memory");
                    if (etid == 0) {
                        tma_store_2d_hint(&cmaps.m[0], buf, (fp8 ? 64 : 48) * (col / 64), my_p0, pol_st);
                        bulk_commit_group();
                    }
                    ++n_out;
                    continue;
                }
                // row prow of the piece = 128 bytes in 16-byte chunks; chunk c is stored at c ^ (row % 8), the
                // 128-byte swizzle the TMA store expects
                const uint32_t rowaddr = buf + prow * (OC * 2);
                const uint32_t sw = (uint32_t)(prow & 7);
#pragma unroll
                for (int c = 0; c < OC / 8; ++c) {
                    const uint32_t x0 = pack_bf16x2(__uint_as_float(v[8 * c + 0]), __uint_as_float(v[8 * c + 1]));
                    const uint32_t x1 = pack_bf16x2(__uint_as_float(v[8 * c + 2]), __uint_as_float(v[8 * c + 3]));
                    const uint32_t x2 = pack_bf16x2(__uint_as_float(v[8 * c + 4]), __uint_as_float(v[8 * c + 5]));
                    const uint32_t x3 = pack_bf16x2(__uint_as_float(v[8 * c + 6]), __uint_as_float(v[8 * c + 7]));
                    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};"
                                 ::"r"(rowaddr + ((c ^ sw) << 4)), "r"(x0), "r"(x1), "r"(x2), "r"(x3) : "memory");
                }
                if (!P.c_tma) {
                    // The staged piece is written out with plain stores instead of TMA stores: always when C cannot be a TMA
                    // destination (rows that are not 16-byte multiples), where each warp writes its 32 rows 4 bytes per lane;
                    // with 16-byte rows (c_vec16) 16 bytes per lane, 4 rows per instruction.
                    asm volatile("bar.sync 1, 128;" ::: "memory");
                    const uint8_t* stage = smem_gen + (buf - smem_base);
                    if (P.c_vec16) {
                        const int chunk = lane & 7;                       // 16-byte chunk = 8 columns
                        const int col = q0 + piece * OC + 8 * chunk;
#pragma unroll
                        for (int i = 0; i < 8; ++i) {
                            const int r = quad * 32 + 4 * i + (lane >> 3);
                            const int row = my_p0 + r;
                            if (row < P.c_rows && col < P.c_cols) {       // N is a multiple of 8 here: a chunk is inside or outside
                                const uint4 x = *reinterpret_cast<const uint4*>(stage + r * (OC * 2) + ((chunk ^ (r & 7)) << 4));
                                for (int d = 0; d < P.ndst; ++d)
                                    *reinterpret_cast<uint4*>((d == 0 ? P.c : P.c_more[d - 1]) + (size_t)row * P.ldc + col) = x;
                            }
                        }
                    } else {
                    const int col = q0 + piece * OC + 2 * lane;
#pragma unroll 4
                    for (int r = quad * 32; r < quad * 32 + 32; ++r) {
                        const int row = my_p0 + r;
                        if (row >= P.c_rows) break;
                        const uint32_t x = *reinterpret_cast<const uint32_t*>(stage + r * (OC * 2) + ((((lane >> 2) ^ (r & 7)) << 4) | ((lane & 3) << 2)));
                        for (int d = 0; d < P.ndst; ++d) {
                            __nv_bfloat16* dst = (d == 0 ? P.c : P.c_more[d - 1]) + (size_t)row * P.ldc + col;
                            if (col + 1 < P.c_cols && (reinterpret_cast<uintptr_t>(dst) & 3) == 0) {
                                *reinterpret_cast<uint32_t*>(dst) = x;
                            } else {
                                if (col < P.c_cols) dst[0] = __ushort_as_bfloat16((unsigned short)(x & 0xffffu));
                                if (col + 1 < P.c_cols) dst[1] = __ushort_as_bfloat16((unsigned short)(x >> 16));
                            }
                        }
                    }
                    }
                    // (the next use of this buffer is two pieces away, behind the barrier that opens every piece)
                    ++n_out;
                    continue;
                }
                fence_proxy_async_smem();
                asm volatile("bar.sync 1, 128;" ::: "memory");
                if (etid == 0) {
                    // the local copy first, then the peers, starting with a different peer for every piece and CTA, so that
                    // the CTAs of one GPU do not all aim at the same peer at the same moment
                    tma_store_2d_hint(&cmaps.m[0], buf, q0 + piece * OC, my_p0, pol_st);
                    const int peers = P.ndst - 1;
                    const int first = (peers > 1 && P.push_rotate) ? (int)((n_out + blockIdx.x) % (uint32_t)peers) : 0;
                    for (int i = 0; i < peers; ++i) {
                        int d = first + i;
                        if (d >= peers) d -= peers;
                        tma_store_2d_hint(&cmaps.m[1 + d], buf, q0 + piece * OC, my_p0, pol_st);
                    }
                    bulk_commit_group();
                }
                ++n_out;
            }
            if (P.sig_flag && etid == 0) {
                // The unit's pieces are with the TMA unit; once they are written, they count towards the block of C the
                // unit lies in.  Release before the count, acquire after it: the CTA that completes the count has seen
                // every other CTA's pieces land, and only then raises the flag.
                bulk_wait_group<0>();
                const int grp = (p0 >> 8) / P.group_p;
                const int gsz = min(P.tiles_p - grp * P.group_p, P.group_p);
                const int strips = (P.tiles_q + P.sig_cols - 1) / P.sig_cols;
                const int strip = (q0 >> 8) / P.sig_cols;
                const int ncol = min(P.sig_cols, P.tiles_q - strip * P.sig_cols);
                const unsigned int total = (unsigned int)(gsz * ncol * 8);      // 2 CTAs x 4 pieces per tile
                const int blk = grp * strips + strip;
                __threadfence_system();
                const unsigned int old = atomicAdd(P.sig_counter + blk, (unsigned int)NP);
                if (old + (unsigned int)NP == total) {
                    __threadfence_system();
                    *reinterpret_cast<volatile unsigned int*>(P.sig_flag + blk) = 1u;
                }
            }
            ++n_seg;
        }
        // the staging buffers have been read before the CTA leaves; the writes themselves are complete when the grid is
        // (with completion flags every unit has already waited for its writes above)
        if (etid == 0) bulk_wait_group_read<0>();
        if (!ok && lane == 0) signal_abort_to_peer();
    }

    // ---- teardown
    if (*abort_flag) {
        const long long t0 = clock64();
        while (clock64() - t0 < 400000) { __nanosleep(1000); }
    }
    tc_fence_before();
    __syncthreads();
    cluster_arrive();            // neither CTA frees TMEM or exits while its peer may still touch it
    cluster_wait();
    tc_fence_after();
    if (warp == 1) tmem_dealloc_pair(tmem_base, Cfg::TMEM_COLS);
}

}  // namespace mxfp6
