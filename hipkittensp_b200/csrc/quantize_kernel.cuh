// Block quantiser fp32 / bf16 [rows, K] -> MX operand bytes + E8M0 scales, as a streaming kernel: HBM-bound
// byte work (reads 4 or 2 bytes per element, writes 0.78 or 1.03).
//
// The source is one long run of 32-element blocks (K % 32 == 0, rows contiguous), the outputs are one run of
// 24- or 32-byte code groups and one run of scale bytes, so the kernel is one-dimensional over blocks:
//
//   warp 0      one elected thread TMA-loads tiles of 128 blocks (16 KB of fp32 / 8 KB of bf16) into a ring of
//               shared-memory stages; the tensor map views the source as [blocks, 32] with the 128-byte (fp32) or
//               64-byte (bf16) swizzle, so that 128 threads can each read their own block without bank conflicts
//   warps 1-4   thread t quantises block t of the tile (amax, scale byte, hardware cvt, 6-bit packing), stores its
//               scale byte, writes its 24/32 code bytes to a staging buffer, and one lane per warp sends the warp's
//               768 / 1024 code bytes with one bulk copy; the warps never wait for each other
//
// Persistent: four (fp32) or seven (bf16: what registers and shared memory allow; 35.4 us against 37.1 us with six for
// an 8192 x 8192 source) CTAs per SM (a single group of four consumer warps cannot hide its own latencies), tiles dealt
// round-robin; 168-192 KB of loads in flight per SM.
// Every mbarrier wait is bounded: when one runs out the CTA records a status word and leaves.
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>

#include "ptx.cuh"
#include "quant.cuh"

namespace mxfp6 {

constexpr int kStatusTimeoutQuantLoad = 0x21;   // producer waited for a free stage
constexpr int kStatusTimeoutQuantData = 0x22;   // consumer waited for a loaded stage

template <typename T, int FMT>
struct QuantCfg {
    static constexpr int TILE_BLOCKS = 128;                          // blocks per tile = consumer threads
    static constexpr int IN_ROW = 32 * (int)sizeof(T);               // bytes of one block in the source
    static constexpr int IN_BYTES = TILE_BLOCKS * IN_ROW;            // 16 KB (fp32) or 8 KB (bf16)
    // several CTAs per SM: one group of four consumer warps cannot hide its own latencies
    static constexpr int CTAS_PER_SM = sizeof(T) == 4 ? 4 : 7;
    static constexpr int STAGES = 3;                                 // per SM 192 KB (fp32) / 168 KB (bf16) of loads in flight
    static constexpr bool FP8 = FMT == kE4M3 || FMT == kE5M2;
    static constexpr int OUT_ROW = FP8 ? 32 : 24;                    // code bytes of one block
    static constexpr int OUT_BYTES = TILE_BLOCKS * OUT_ROW;          // 4 KB or 3 KB, a multiple of 16
    static constexpr int OUT_BUFS = 2;
    static constexpr int THREADS = 32 + TILE_BLOCKS;
    static constexpr int SMEM_BYTES = STAGES * IN_BYTES + OUT_BUFS * OUT_BYTES + 2 * STAGES * 8 + 16;
    static constexpr int SMEM_ALLOC = SMEM_BYTES + 1024;
};

__device__ __forceinline__ void bulk_store_1d(void* dst_global, uint32_t src_smem, uint32_t bytes) {
    asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;"
                 ::"l"(dst_global), "r"(src_smem), "r"(bytes) : "memory");
}

__device__ __forceinline__ bool quant_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, int* status,
                                           unsigned long long wait_cycles, int code) {
    if (mbar_try_wait(bar, parity)) return true;
    const long long t0 = clock64();
    uint32_t n = 0;
    while (!mbar_try_wait(bar, parity)) {
        if ((++n & 255u) == 0) {
            if (*abort_flag) return false;
            if ((unsigned long long)(clock64() - t0) > wait_cycles) {
                *abort_flag = 1;
                atomicCAS(status, 0, code | ((int)blockIdx.x << 8));
                return false;
            }
        }
    }
    return true;
}

template <typename T, int FMT>
__global__ void __launch_bounds__(QuantCfg<T, FMT>::THREADS, QuantCfg<T, FMT>::CTAS_PER_SM)
quantize_tma_kernel(const __grid_constant__ CUtensorMap tm_src, long long n_blocks, uint8_t* __restrict__ packed,
                    uint8_t* __restrict__ scales, int* status, unsigned long long wait_cycles) {
    using Cfg = QuantCfg<T, FMT>;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
    const uint32_t out_off = Cfg::STAGES * Cfg::IN_BYTES;
    const uint32_t bar_off = out_off + Cfg::OUT_BUFS * Cfg::OUT_BYTES;
    auto bar_full = [&](int s) { return smem_base + bar_off + 8u * s; };
    auto bar_empty = [&](int s) { return smem_base + bar_off + 8u * (Cfg::STAGES + s); };
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem_gen + bar_off + 2 * Cfg::STAGES * 8);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        for (int s = 0; s < Cfg::STAGES; ++s) { mbar_init(bar_full(s), 1); mbar_init(bar_empty(s), 4); }
        *abort_flag = 0;
        fence_barrier_init();
        tma_prefetch_desc(&tm_src);
    }
    __syncthreads();
    // launched with programmatic stream serialisation: everything above overlapped the end of the preceding kernel,
    // nothing of global memory is touched before it has completed; the kernel after this one may likewise set
    // itself up as soon as SMs become free (it waits for this grid's completion before its own first access)
    pdl_launch_dependents();
    pdl_wait();

    const long long n_tiles = (n_blocks + Cfg::TILE_BLOCKS - 1) / Cfg::TILE_BLOCKS;
    if (warp == 0) {
        // ------------------------------------------------------------------ producer
        uint32_t n = 0;
        bool ok = true;
        for (long long tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x, ++n) {
            const int s = n % Cfg::STAGES;
            ok = __all_sync(0xffffffffu, quant_wait(bar_empty(s), ((n / Cfg::STAGES) & 1) ^ 1, abort_flag, status, wait_cycles,
                                                    kStatusTimeoutQuantLoad));
            if (!ok) break;
            if (elect_one_sync()) {
                // a tile that reaches past the last block is clipped by the TMA unit; the barrier is credited the whole box
                mbar_arrive_expect_tx(bar_full(s), Cfg::IN_BYTES);
                tma_load_2d(smem_base + s * Cfg::IN_BYTES, &tm_src, bar_full(s), 0, (int)(tile * Cfg::TILE_BLOCKS));
            }
            __syncwarp();
        }
    } else {
        // ------------------------------------------------------------------ consumers: thread t <-> block t of the tile
        // The four consumer warps never wait for each other: each takes its 32 blocks from the stage, and sends its own
        // 768 / 1024 code bytes with one bulk copy from its own slice of the staging buffers.
        const int t = threadIdx.x - 32;
        const int cw = t >> 5;                               // consumer warp 0..3
        uint32_t n = 0, s = 0, phase = 0;
        for (long long tile = blockIdx.x; tile < n_tiles; tile += gridDim.x, ++n, phase ^= (s + 1 == Cfg::STAGES), s = (s + 1 == Cfg::STAGES) ? 0 : s + 1) {
            if (!__all_sync(0xffffffffu, quant_wait(bar_full(s), phase, abort_flag, status, wait_cycles,
                                                    kStatusTimeoutQuantData)))
                break;
            float v[32];
            float amax;
            const uint8_t* row = smem_gen + s * Cfg::IN_BYTES + t * Cfg::IN_ROW;
            if constexpr (sizeof(T) == 4) {
                // 128-byte rows, 128-byte swizzle: 16-byte chunk c of row t sits at chunk c ^ (t % 8)
#pragma unroll
                for (int c = 0; c < 8; ++c) {
                    const float4 x = *reinterpret_cast<const float4*>(row + ((c ^ (t & 7)) << 4));
                    v[4 * c] = x.x; v[4 * c + 1] = x.y; v[4 * c + 2] = x.z; v[4 * c + 3] = x.w;
                }
                amax = amax32(v);
            } else {
                // 64-byte rows, 64-byte swizzle: chunk c of row t sits at chunk c ^ ((t / 2) % 4)
                __nv_bfloat162 m2;
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    const uint4 x = *reinterpret_cast<const uint4*>(row + ((c ^ ((t >> 1) & 3)) << 4));
                    const uint32_t w[4] = {x.x, x.y, x.z, x.w};
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        v[8 * c + 2 * e] = __uint_as_float(w[e] << 16);
                        v[8 * c + 2 * e + 1] = __uint_as_float(w[e] & 0xffff0000u);
                        // the largest magnitude is found on the packed pairs (half-precision pipe, not the ALU)
                        const __nv_bfloat162 a2 = __habs2(*reinterpret_cast<const __nv_bfloat162*>(&w[e]));
                        m2 = (c == 0 && e == 0) ? a2 : __hmax2(m2, a2);
                    }
                }
                amax = fmaxf(__low2float(m2), __high2float(m2));
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_empty(s));       // this warp's part of the stage is in registers

            uint32_t w[8];
            const int sb = quant_block32_amax<FMT>(v, amax, w);
            const long long blk = tile * Cfg::TILE_BLOCKS + t;
            const bool whole = (tile + 1) * Cfg::TILE_BLOCKS <= n_blocks;
            if (blk < n_blocks) scales[blk] = (uint8_t)sb;   // 32 consecutive bytes per warp
            if (whole) {
                const int ob = n & 1;
                // the bulk copy that last read this warp's slice of the staging buffer is done with it
                if (lane == 0) bulk_wait_group_read<Cfg::OUT_BUFS - 1>();
                __syncwarp();
                uint2* o = reinterpret_cast<uint2*>(smem_gen + out_off + ob * Cfg::OUT_BYTES + t * Cfg::OUT_ROW);
                o[0] = make_uint2(w[0], w[1]);
                o[1] = make_uint2(w[2], w[3]);
                o[2] = make_uint2(w[4], w[5]);
                if constexpr (Cfg::FP8) o[3] = make_uint2(w[6], w[7]);
                fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0) {
                    bulk_store_1d(packed + tile * Cfg::OUT_BYTES + cw * (32 * Cfg::OUT_ROW),
                                  smem_base + out_off + ob * Cfg::OUT_BYTES + cw * (32 * Cfg::OUT_ROW), 32 * Cfg::OUT_ROW);
                    bulk_commit_group();
                }
            } else if (blk < n_blocks) {
                // the last, partial tile: its size need not be a multiple of 16 bytes, so plain stores
                uint2* o = reinterpret_cast<uint2*>(packed + blk * Cfg::OUT_ROW);
                o[0] = make_uint2(w[0], w[1]);
                o[1] = make_uint2(w[2], w[3]);
                o[2] = make_uint2(w[4], w[5]);
                if constexpr (Cfg::FP8) o[3] = make_uint2(w[6], w[7]);
            }
        }
        if (lane == 0) bulk_wait_group<0>();
    }
    if (*abort_flag) {
        // give loads that are still in flight time to land before shared memory goes away
        const long long t0 = clock64();
        while (clock64() - t0 < 400000) { __nanosleep(1000); }
    }
}

}  // namespace mxfp6
