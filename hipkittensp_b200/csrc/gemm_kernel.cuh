// MX-FP6 block-scaled GEMM for sm_100a:  D[p,q] = sum_k P[p,k] * Q[q,k]   (both operands K-contiguous)
//
//   P : "row" operand of the tensor-core instruction, 128 rows per tile  (MMA operand A)
//   Q : "column" operand, BN rows per tile                               (MMA operand B)
//
// The host maps (A,B) of C = A*B^T onto (P,Q): normally P=A, Q=B and D is stored as C[p,q]; for
// skinny M the operands are swapped (P=B, Q=A, SWAP=true) and D is stored transposed, C[q,p], so the
// long dimension rides the 128-row side of the instruction.
//
// One persistent CTA per SM, 8 warps with fixed roles:
//   warp 0   TMA producer: packed 6-bit operand tiles (tensor-map type 16U6_ALIGN16B, 128-byte swizzle)
//            and raw E8M0 scale slabs into shared-memory rings
//   warp 1   MMA issuer: copies the scale atoms into TMEM (tcgen05.cp) and issues
//            tcgen05.mma.kind::mxf8f6f4.block_scale, accumulating in TMEM
//   warps 2-3 scale re-tilers: row-major [rows, K/32] scale bytes -> the 32x16-byte atoms the MMA wants,
//            one group of 4 K-blocks at a time, the two warps alternating
//   warps 4-7 epilogue: TMEM -> registers -> bf16 -> global (or fp32 partials for split tiles)
//
// Every wait on an mbarrier is bounded; on expiry the CTA records a status code and leaves cleanly.
#pragma once
#include "ptx.cuh"
#include "quant.cuh"

namespace mxfp6 {

// device status codes (0 = ok); the low byte is the code, the rest identifies the CTA
enum : int {
    kStatusOk = 0,
    kStatusTimeoutProducer = 1,
    kStatusTimeoutMma = 2,
    kStatusTimeoutScale = 3,
    kStatusTimeoutEpilogue = 4,
};

struct GemmParams {
    int p_rows, q_rows;        // valid rows of P and Q
    int kblocks;               // K / 128
    int tiles_p, tiles_q;      // ceil(p_rows/p_tile_rows), ceil(q_rows/q_tile_rows)
    int p_tile_rows;           // rows of P one tile covers (<= 128; 128 unless the rows of a streamed operand are dealt evenly to the CTAs)
    int q_tile_rows;           // rows of Q one tile covers (<= BN)
    int raw_tx_bytes;          // bytes the two scale-slab loads of a group report to their mbarrier
    // forms whose tiles hold fewer rows than a full box (skinny M): the operand ring is laid out at run time, because
    // such a tile needs less than the 16 KB + BN * 128 bytes of a full stage and the space saved buys more stages
    int n_stages;              // stages in the ring (<= STAGES_MAX)
    int stage_stride;          // bytes from one stage to the next (a multiple of 1024)
    int q_off;                 // offset of the Q box inside a stage (rows of P rounded up to 8, times 128)
    int load_batch;            // K-blocks the producer requests back to back
    int k_rot;                 // whole tiles start their K loop at a tile-dependent K-block and wrap around (kblocks % 4 == 0)
    int ldc;                   // row stride of C in elements (= N)
    int c_rows, c_cols;        // M, N
    uint32_t idesc;            // instruction descriptor without scale ids
    int sf_tma;                // 1: scale slabs come by TMA; 0: the scale warp reads them with plain loads
    int sf_ld;                 // K / 32, row stride of the scale arrays in bytes
    int stage_tx_bytes;        // bytes one operand stage reports to its mbarrier
    const uint8_t* sfp;        // scales of P / Q (row-major [rows, K/32])
    const uint8_t* sfq;
    __nv_bfloat16* c;          // first element of this GEMM's block inside destination 0 (row stride ldc)
    __nv_bfloat16* c_more[7];  // the same position in further destinations (peer GPUs' copies of C)
    int ndst;                  // number of destinations, 1..8
    int push_rotate;           // pair kernel: the order in which a piece goes to the peer destinations rotates from piece to piece
    int c_vec16;               // pair kernel, plain stores: destinations and row stride are 16-byte multiples and N % 8 == 0
    // pair kernel, optional: C is cut into blocks (group_p * 256 rows x sig_cols * 256 columns); every CTA adds the 64-column
    // pieces it has written to its block's counter, and the CTA that completes a block raises the block's flag, which
    // copy streams of the host wait for (stream memory operations)
    unsigned int* sig_counter;
    unsigned int* sig_flag;
    int sig_cols;
    int c_tma_last;            // single-CTA kernel, unswapped: the last tile of every CTA leaves through the idle ring and TMA stores (tm_c is a map of C)
    int c_tma;                 // pair kernel: C is stored by TMA (16-byte aligned destinations and row stride); else by plain stores
    uint8_t* q_out;            // re-quantised output instead of bf16 C: operand bytes [M, 3N/4 or N] ...
    uint8_t* q_scales;         // ... and E8M0 scales [M, N/32], blocks of 32 along N
    long long q_ld;            // row stride of q_out in bytes
    int q_fmt;                 // format code of the re-quantised output, -1 = store bf16 C
    float* ws_partial;         // split-tile partial sums: [tile][slot][BN][128] fp32
    unsigned int* ws_counter;  // per-tile arrival counters (zero between launches)
    int ws_slots;              // partial slots per tile
    int* status;               // device status word
    unsigned long long wait_cycles;  // budget of one wait in clock cycles
    int group_p;               // pair kernel: P-tiles per rasterisation group
    int tail_first;            // pair kernel: first tile of the last partial wave that is cut into column slices (= tile count if none)
    int tail_split;            // pair kernel: slices per such tile (1, 2 or 4)
    int stage_tx_bytes_tail;   // pair kernel: bytes one CTA's loads of a slice's stage report
    int l2_ahead;              // single-CTA kernel: while it waits for the preceding kernel the producer asks the weights of its first stages into L2
    int early_p;               // single-CTA kernel: the weights (B: P when swapped, Q otherwise) may be read before the preceding kernel has finished
    int l2_load, l2_store;     // L2 eviction policy of the operand loads / of the stores of C (0 normal, 1 evict_first, 2 evict_last)
    int l2_p, l2_q;            // single-CTA kernel: policy of the loads of P / of Q (an operand that is read once leaves L2 first, one that every CTA re-reads last)
    // optional fp32 epilogue, applied to the finished sum before it is rounded (null = absent):
    // C[m,n] = (acc * scale_n[n]) * scale_m[m] + bias_n[n]
    const float* scale_m;      // [M]
    const float* scale_n;      // [N]
    const float* bias_n;       // [N]
};

// The epilogue arithmetic for one element.  D[p,q] is C[p,q], or C[q,p] in the swapped form.  Three separate
// roundings (no fused multiply-add), in the order column scale, row scale, bias.
template <bool SWAP>
__device__ __forceinline__ float affine_one(const GemmParams& P, float x, int p, int q) {
    const int m = SWAP ? q : p, n = SWAP ? p : q;
    const float sn = (P.scale_n && n < P.c_cols) ? __ldg(P.scale_n + n) : 1.f;
    const float sm = (P.scale_m && m < P.c_rows) ? __ldg(P.scale_m + m) : 1.f;
    const float bn = (P.bias_n && n < P.c_cols) ? __ldg(P.bias_n + n) : 0.f;
    return __fadd_rn(__fmul_rn(__fmul_rn(x, sn), sm), bn);
}

__device__ __forceinline__ bool has_affine(const GemmParams& P) {
    return P.scale_m != nullptr || P.scale_n != nullptr || P.bias_n != nullptr;
}

// The same for the CW consecutive columns q0.. of row p that one epilogue thread holds.
template <bool SWAP, int CW>
__device__ __forceinline__ void affine_chunk(const GemmParams& P, uint32_t (&v)[CW], int p, int q0) {
    if (SWAP) {
        // p is the column of C: one scale and one bias for the whole chunk; the row scale varies along it
        const bool in = p < P.c_cols;
        const float sn = (P.scale_n && in) ? __ldg(P.scale_n + p) : 1.f;
        const float bn = (P.bias_n && in) ? __ldg(P.bias_n + p) : 0.f;
#pragma unroll
        for (int i = 0; i < CW; ++i) {
            const float sm = (P.scale_m && q0 + i < P.c_rows) ? __ldg(P.scale_m + q0 + i) : 1.f;
            v[i] = __float_as_uint(__fadd_rn(__fmul_rn(__fmul_rn(__uint_as_float(v[i]), sn), sm), bn));
        }
    } else {
        const float sm = (P.scale_m && p < P.c_rows) ? __ldg(P.scale_m + p) : 1.f;
        const bool whole = q0 + CW <= P.c_cols;     // q0 is a multiple of 16 and the vectors are 16-byte aligned
#pragma unroll
        for (int i = 0; i < CW; i += 4) {
            float4 sn = make_float4(1.f, 1.f, 1.f, 1.f), bn = make_float4(0.f, 0.f, 0.f, 0.f);
            if (whole) {
                if (P.scale_n) sn = __ldg(reinterpret_cast<const float4*>(P.scale_n + q0 + i));
                if (P.bias_n) bn = __ldg(reinterpret_cast<const float4*>(P.bias_n + q0 + i));
            } else {
                float* s4 = reinterpret_cast<float*>(&sn);
                float* b4 = reinterpret_cast<float*>(&bn);
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    if (q0 + i + e < P.c_cols) {
                        if (P.scale_n) s4[e] = __ldg(P.scale_n + q0 + i + e);
                        if (P.bias_n) b4[e] = __ldg(P.bias_n + q0 + i + e);
                    }
                }
            }
            v[i + 0] = __float_as_uint(__fadd_rn(__fmul_rn(__fmul_rn(__uint_as_float(v[i + 0]), sn.x), sm), bn.x));
            v[i + 1] = __float_as_uint(__fadd_rn(__fmul_rn(__fmul_rn(__uint_as_float(v[i + 1]), sn.y), sm), bn.y));
            v[i + 2] = __float_as_uint(__fadd_rn(__fmul_rn(__fmul_rn(__uint_as_float(v[i + 2]), sn.z), sm), bn.z));
            v[i + 3] = __float_as_uint(__fadd_rn(__fmul_rn(__fmul_rn(__uint_as_float(v[i + 3]), sn.w), sm), bn.w));
        }
    }
}

// CTAS_ = 2: a smaller pipeline so that two CTAs share an SM (BN <= 32: half the shared memory, a quarter of TMEM each).
// (For 32 < M <= 64 the same form with BN = 64 has room for 4 stages only and measured 45.3 us against 41.2 us for whole
// unswapped tiles at N = 28672, K = 8192.)
// (A third-size build, leaving room on every SM for a CTA of the next kernel of the stream, was measured and dropped:
// its shorter ring cost 8 % at M = 16, N = 28672, more than the overlap of consecutive kernels gave back.)
template <int BN_, bool SWAP_, bool STREAMK_, int CTAS_ = 1>
struct GemmCfg {
    static constexpr int BN = BN_;
    static constexpr bool SWAP = SWAP_;
    static constexpr bool STREAMK = STREAMK_;
    static constexpr int CTAS = CTAS_;
    static constexpr int BM = 128;
    static constexpr int BK = 128;                       // elements of K per pipeline stage (= bytes in smem)
    static constexpr int P_BYTES = BM * BK;
    static constexpr int Q_BYTES = BN * BK;
    static constexpr int STAGE_BYTES = P_BYTES + Q_BYTES;
    static constexpr int STAGES = CTAS_ == 2 ? (BN <= 16 ? 5 : 4)
                                             : BN >= 256 ? 4 : BN >= 128 ? 6 : BN >= 64 ? 8 : BN >= 32 ? 9 : 11;
    // bytes of the operand ring (two CTAs per SM: 6 stages of 104 x 128-byte rows + Q for BN = 16, 5 for BN = 32, the
    // stage of a 97-row tile; laid out at run time)
    static constexpr int RING_BYTES = CTAS_ == 2 ? (BN <= 16 ? 6 * (13312 + 2048) : 5 * (13312 + 4096)) : STAGES * STAGE_BYTES;
    static constexpr int LOAD_BATCH = SWAP_ ? (STAGES >= 8 ? 4 : 2) : 1;   // K-blocks the producer requests together
    // ring laid out at run time: the two-CTAs-per-SM form and the whole-tile 128 x 256 kernel (which serves skinny M)
    static constexpr bool RUNTIME_RING = CTAS_ == 2 || (BN_ == 256 && !SWAP_ && !STREAMK_);
    static constexpr int STAGES_MAX = RUNTIME_RING ? 8 : STAGES;           // barrier pairs provided (see GemmParams::n_stages)
    static constexpr int QATOMS = (BN + 127) / 128;      // 128-row scale atoms on the Q side
    static constexpr int RAW_SLOTS = (BN >= 256 || CTAS_ == 2) ? 2 : 4;  // each raw slab covers 4 K-blocks (16 scale bytes per row)
    static constexpr int RAW_Q_ROWS = BN < 32 ? 32 : BN;
    static constexpr int RAW_BYTES = (BM + RAW_Q_ROWS) * 16;
    static constexpr int ATOM_BYTES = 512 * (1 + QATOMS);  // scale atoms of one K-block: P atom + Q atoms
    static constexpr int GROUP_BYTES = 4 * ATOM_BYTES;     // a group = the 4 K-blocks one raw slab covers
    static constexpr int ATOM_GROUPS = (BN >= 256 || CTAS_ == 2) ? 3 : 4;
    static constexpr bool OVERLAP = BN == 256;           // two 256-column accumulators share 32 columns
    static constexpr int ACC_COL1 = OVERLAP ? 224 : BN;
    static constexpr int SF_COL = OVERLAP ? 480 : 2 * BN;
    // two CTAs of an SM share its 512 columns: each takes the power of two that holds its two accumulators and 32 scale columns
    static constexpr int TMEM_COLS = CTAS_ == 2 ? (2 * BN + 32 <= 64 ? 64 : 2 * BN + 32 <= 128 ? 128 : 256) : 512;
    static_assert(CTAS_ == 1 || (CTAS_ == 2 && BN <= 32 && !STREAMK_), "two CTAs per SM: small accumulators, whole tiles");
    static constexpr int NUM_BARS = 2 * STAGES_MAX + 2 * RAW_SLOTS + 2 * ATOM_GROUPS + 5;
    // unswapped form: column scale and bias of the current tile for the fp32 epilogue (2 x BN floats, 16-byte aligned)
    static constexpr int AFF_BYTES = SWAP ? 0 : 2 * BN * 4 + 16;
    static constexpr int SMEM_BYTES = RING_BYTES + RAW_SLOTS * RAW_BYTES + ATOM_GROUPS * GROUP_BYTES +
                                      NUM_BARS * 8 + 64 + AFF_BYTES;
    static constexpr int SMEM_ALLOC = SMEM_BYTES + 1024;  // slack for the 1024-byte alignment of the operand ring
    static constexpr int THREADS = 256;
    static constexpr int GROUP_P = 8;                     // tile rasterisation: groups of 8 P-tiles share Q-tiles
    static_assert(SMEM_ALLOC <= (CTAS_ == 1 ? 232448 : 233472 / CTAS_ - 1024), "exceeds the shared memory this CTA can have");
};

// One unit of work of a CTA: a K range of one output tile.
struct Segment {
    int tile, p0, q0, k0, k1;
    int nseg, segidx;           // how many CTAs contribute to this tile, and which of them this is
    int kofs;                   // K-block at which position k0 of the loop sits (the loop wraps at the last K-block)
};
// K-block that position i of a segment's loop addresses.  Skinny problems stream one operand once, every CTA from its own
// rows; started together at K-block 0 all CTAs would ask for the same columns of every row at the same time (addresses
// that differ by multiples of the row pitch, which fall on few DRAM channels).  Rotating each tile's loop spreads them.
__device__ __forceinline__ int k_at(const GemmParams& P, const Segment& sg, int i) {
    const int k = i + sg.kofs;
    return k < P.kblocks ? k : k - P.kblocks;
}

template <class Cfg>
struct SegIter {
    const GemmParams& P;
    int num_tiles;
    long long u_begin, u_end;    // STREAMK: this CTA's range of K-block units (tile-major)
    int first_tile, nsegs, i;    // STREAMK: tiles the range touches; next position in the visiting order
    int tile;                    // !STREAMK: current tile
    __device__ SegIter(const GemmParams& p) : P(p) {
        num_tiles = P.tiles_p * P.tiles_q;
        u_begin = u_end = 0; first_tile = nsegs = i = 0; tile = 0;
        if (Cfg::STREAMK) {
            const long long U = (long long)num_tiles * P.kblocks;
            u_begin = (U * blockIdx.x) / gridDim.x;
            u_end = (U * (blockIdx.x + 1)) / gridDim.x;
            if (u_end > u_begin) {
                first_tile = (int)(u_begin / P.kblocks);
                nsegs = (int)((u_end - 1) / P.kblocks) - first_tile + 1;
            }
        } else {
            tile = blockIdx.x;
        }
    }
    __device__ static int owner(long long unit, long long U, int G) { return (int)(((unit + 1) * G - 1) / U); }
    __device__ void coords(int t, int& p0, int& q0) const {
        int per_group = Cfg::GROUP_P * P.tiles_q;
        int group = t / per_group, in = t % per_group;
        int first_p = group * Cfg::GROUP_P;
        int gsz = min(P.tiles_p - first_p, Cfg::GROUP_P);
        p0 = (first_p + in % gsz) * P.p_tile_rows;
        q0 = (in / gsz) * P.q_tile_rows;
    }
    // after next() returned a segment: is it the last one of this CTA?
    __device__ bool last() const { return Cfg::STREAMK ? i >= nsegs : tile >= num_tiles; }
    __device__ bool next(Segment& s) {
        if (Cfg::STREAMK) {
            if (i >= nsegs) return false;
            // Visiting order: the first and the last piece of the range (the ones that may share their tile
            // with a neighbouring CTA) come first, whole tiles after them, so that split tiles are published
            // and summed while the mainloop still runs and the kernel ends on a plain tile epilogue.
            const int idx = i == 0 ? 0 : (i == 1 ? nsegs - 1 : i - 1);
            ++i;
            const long long U = (long long)num_tiles * P.kblocks;
            s.tile = first_tile + idx;
            const long long t0 = (long long)s.tile * P.kblocks;
            s.k0 = idx == 0 ? (int)(u_begin - t0) : 0;
            s.k1 = idx == nsegs - 1 ? (int)(u_end - t0) : P.kblocks;
            const int first = owner(t0, U, gridDim.x), last = owner(t0 + P.kblocks - 1, U, gridDim.x);
            s.nseg = last - first + 1;
            s.segidx = (int)blockIdx.x - first;
            s.kofs = 0;
            coords(s.tile, s.p0, s.q0);
            return true;
        } else {
            if (tile >= num_tiles) return false;
            s.tile = tile; s.k0 = 0; s.k1 = P.kblocks; s.nseg = 1; s.segidx = 0;
            s.kofs = P.k_rot ? (int)(((long long)tile * P.kblocks) / num_tiles) & ~3 : 0;
            coords(tile, s.p0, s.q0);
            tile += gridDim.x;
            return true;
        }
    }
};

// Bounded wait.  Returns false when the CTA is aborting (this wait ran out, or another one did).
__device__ __forceinline__ bool wait_bar(uint32_t bar, uint32_t parity, volatile int* abort_flag,
                                         const GemmParams& P, int code) {
    if (mbar_try_wait(bar, parity)) return true;
    long long t0 = clock64();
    uint32_t n = 0;
    while (!mbar_try_wait(bar, parity)) {
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

// Agreement among the 128 epilogue threads (named barrier 1): true only if every one of them passes true.
// The epilogue warps synchronise with each other inside a tile, so they must enter or skip it together.
__device__ __forceinline__ bool epilogue_all(bool ok) {
    uint32_t r;
    asm volatile(
        "{\n\t.reg .pred p, q;\n\t"
        "setp.ne.u32 q, %1, 0;\n\t"
        "bar.red.and.pred p, 1, 128, q;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(r) : "r"((uint32_t)ok) : "memory");
    return r != 0;
}

// Same, for a whole converged warp: every lane waits, and all lanes agree on the outcome.
__device__ __forceinline__ bool wait_bar_warp(uint32_t bar, uint32_t parity, volatile int* abort_flag,
                                              const GemmParams& P, int code) {
    return __all_sync(0xffffffffu, wait_bar(bar, parity, abort_flag, P, code));
}


template <class Cfg>
__global__ void __launch_bounds__(Cfg::THREADS, Cfg::CTAS)
mxfp6_gemm_kernel(const __grid_constant__ CUtensorMap tm_p, const __grid_constant__ CUtensorMap tm_q,
                  const __grid_constant__ CUtensorMap tm_sfp, const __grid_constant__ CUtensorMap tm_sfq,
                  const __grid_constant__ CUtensorMap tm_c, const GemmParams P) {
    constexpr int BN = Cfg::BN;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));

    // ---- shared-memory carve-up
    const uint32_t stage_base = smem_base;
    const uint32_t raw_base = stage_base + Cfg::RING_BYTES;
    const uint32_t atom_base = raw_base + Cfg::RAW_SLOTS * Cfg::RAW_BYTES;
    const uint32_t bar_base = atom_base + Cfg::ATOM_GROUPS * Cfg::GROUP_BYTES;
    auto bar_full = [&](int s) { return bar_base + 8u * s; };
    constexpr int SM_ = Cfg::STAGES_MAX;
    auto bar_empty = [&](int s) { return bar_base + 8u * (SM_ + s); };
    auto bar_raw_full = [&](int s) { return bar_base + 8u * (2 * SM_ + s); };
    auto bar_raw_empty = [&](int s) { return bar_base + 8u * (2 * SM_ + Cfg::RAW_SLOTS + s); };
    auto bar_atom_full = [&](int s) { return bar_base + 8u * (2 * SM_ + 2 * Cfg::RAW_SLOTS + s); };
    auto bar_atom_empty = [&](int s) { return bar_base + 8u * (2 * SM_ + 2 * Cfg::RAW_SLOTS + Cfg::ATOM_GROUPS + s); };
    const uint32_t bar_misc = bar_base + 8u * (2 * SM_ + 2 * Cfg::RAW_SLOTS + 2 * Cfg::ATOM_GROUPS);
    // ring geometry: fixed at compile time, except where tiles can be smaller than a full box
    const int n_stages = Cfg::RUNTIME_RING ? P.n_stages : Cfg::STAGES;
    const uint32_t stage_stride = Cfg::RUNTIME_RING ? (uint32_t)P.stage_stride : (uint32_t)Cfg::STAGE_BYTES;
    const uint32_t q_off = Cfg::RUNTIME_RING ? (uint32_t)P.q_off : (uint32_t)Cfg::P_BYTES;
    const int load_batch = Cfg::RUNTIME_RING ? P.load_batch : Cfg::LOAD_BATCH;
    auto bar_acc_full = [&](int b) { return bar_misc + 8u * b; };
    auto bar_acc_empty = [&](int b) { return bar_misc + 8u * (2 + b); };
    const uint32_t bar_ovl = bar_misc + 8u * 4;
    const uint32_t misc_off = (bar_base - smem_base) + Cfg::NUM_BARS * 8;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem_gen + misc_off);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem_gen + misc_off + 4);
    volatile int* ticket_slot = reinterpret_cast<volatile int*>(smem_gen + misc_off + 8);
    float* aff_sn = reinterpret_cast<float*>(smem_gen + ((misc_off + 64 + 15) & ~15u));    // [BN] column scales, then [BN] biases
    float* aff_bn = aff_sn + BN;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    pdl_launch_dependents();     // the next kernel may set itself up on SMs this grid has left

    if (threadIdx.x == 0) {
        for (int s = 0; s < n_stages; ++s) { mbar_init(bar_full(s), 1); mbar_init(bar_empty(s), 1); }
        for (int s = 0; s < Cfg::RAW_SLOTS; ++s) { mbar_init(bar_raw_full(s), 1); mbar_init(bar_raw_empty(s), 32); }
        for (int s = 0; s < Cfg::ATOM_GROUPS; ++s) { mbar_init(bar_atom_full(s), 32); mbar_init(bar_atom_empty(s), 1); }
        for (int b = 0; b < 2; ++b) { mbar_init(bar_acc_full(b), 1); mbar_init(bar_acc_empty(b), 128); }
        mbar_init(bar_ovl, 4);
        *abort_flag = 0;
        *ticket_slot = 0;
        fence_barrier_init();
    }
    if (warp == 0 && lane == 0) {
        tma_prefetch_desc(&tm_p); tma_prefetch_desc(&tm_q);
        if (P.sf_tma) { tma_prefetch_desc(&tm_sfp); tma_prefetch_desc(&tm_sfq); }
    }
    if (warp == 1) {
        tmem_alloc(smem_u32(tmem_slot), Cfg::TMEM_COLS);
        tmem_relinquish();
    }
    // The producer warp (which has just initialised the barriers) does not wait for the TMEM allocation: it announces
    // itself at the CTA's meeting point and goes on to request the first stages; everybody else meets there.
    tc_fence_before();
    if (warp == 0) {
        __syncwarp();
        __threadfence_block();
        asm volatile("bar.arrive 2, 256;" ::: "memory");
    } else {
        asm volatile("bar.sync 2, 256;" ::: "memory");
    }
    tc_fence_after();
    const uint32_t tmem_base = warp == 0 ? 0u : *tmem_slot;
    // Nothing above touches global memory; everything below may.  With early_p the producer warp alone goes
    // ahead and requests the first stages of the weights (which the preceding kernel does not write) before it waits.
    const bool early = P.early_p != 0;
    const bool ahead = early || P.l2_ahead != 0;      // the producer warp has something to do before the wait
    if (!(ahead && warp == 0)) pdl_wait();

    // =========================================================== warp 0: TMA producer
    if (warp == 0) {
        // the whole warp walks the schedule (so it stays converged for the final barrier); lane 0 issues
        SegIter<Cfg> it(P);
        Segment sg;
        uint32_t n_stage = 0, n_raw = 0;
        uint32_t st_idx = 0, st_phase = 0;        // ring position of stage number n_stage and the parity of its round (no division: the ring size may be a run-time value)
        uint32_t pre_stage = 0, pre_raw = 0;      // stages / scale slabs whose weights half is already on its way
        bool ok = true;
        const uint64_t pol_p = l2_policy(P.l2_p), pol_q = l2_policy(P.l2_q);
        // The weights are P in the swapped form and Q otherwise; "the other operand" is the activations.  Stage halves
        // and scale-slab parts of the two, as the early requests below and the loop after them issue them.
        constexpr bool WQ = !Cfg::SWAP;
        auto load_weights = [&](uint32_t stage_dst, uint32_t bar, int kblk, const Segment& s) {
            if (WQ) tma_load_2d_hint(stage_dst + q_off, &tm_q, bar, kblk * Cfg::BK, s.q0, pol_q);
            else tma_load_2d_hint(stage_dst, &tm_p, bar, kblk * Cfg::BK, s.p0, pol_p);
        };
        auto load_other = [&](uint32_t stage_dst, uint32_t bar, int kblk, const Segment& s) {
            if (WQ) tma_load_2d_hint(stage_dst, &tm_p, bar, kblk * Cfg::BK, s.p0, pol_p);
            else tma_load_2d_hint(stage_dst + q_off, &tm_q, bar, kblk * Cfg::BK, s.q0, pol_q);
        };
        auto slab_weights = [&](uint32_t slab_dst, uint32_t bar, int kblk, const Segment& s) {
            if (WQ) tma_load_2d_hint(slab_dst + Cfg::BM * 16, &tm_sfq, bar, (kblk >> 2) * 16, s.q0, pol_q);
            else tma_load_2d_hint(slab_dst, &tm_sfp, bar, (kblk >> 2) * 16, s.p0, pol_p);
        };
        auto slab_other = [&](uint32_t slab_dst, uint32_t bar, int kblk, const Segment& s) {
            if (WQ) tma_load_2d_hint(slab_dst, &tm_sfp, bar, (kblk >> 2) * 16, s.p0, pol_p);
            else tma_load_2d_hint(slab_dst + Cfg::BM * 16, &tm_sfq, bar, (kblk >> 2) * 16, s.q0, pol_q);
        };
        if (early) {
            SegIter<Cfg> it2(P);
            Segment s2;
            bool slabs = P.sf_tma != 0;
            // the ring's first fill is requested for real; the K-blocks behind it are asked into L2 (see below)
            uint32_t n_seen = 0;
            const uint32_t n_total = (uint32_t)(n_stages * (1 + P.l2_ahead));
            while (n_seen < n_total && it2.next(s2)) {
                for (int k = s2.k0; k < s2.k1 && n_seen < n_total; ++k, ++n_seen) {
                    if (n_seen >= (uint32_t)n_stages) {
                        if (elect_one_sync()) {
                            if (WQ) tma_prefetch_l2_2d(&tm_q, k_at(P, s2, k) * Cfg::BK, s2.q0);
                            else tma_prefetch_l2_2d(&tm_p, k_at(P, s2, k) * Cfg::BK, s2.p0);
                        }
                        continue;
                    }
                    if (P.sf_tma && (k == s2.k0 || (k & 3) == 0)) {
                        if (slabs && pre_raw < (uint32_t)Cfg::RAW_SLOTS) {
                            if (elect_one_sync()) {
                                mbar_arrive_expect_tx(bar_raw_full(pre_raw), (uint32_t)P.raw_tx_bytes);
                                slab_weights(raw_base + pre_raw * Cfg::RAW_BYTES, bar_raw_full(pre_raw), k_at(P, s2, k), s2);
                            }
                            ++pre_raw;
                        } else {
                            slabs = false;
                        }
                    }
                    if (elect_one_sync()) {
                        mbar_arrive_expect_tx(bar_full(pre_stage), (uint32_t)P.stage_tx_bytes);
                        load_weights(stage_base + pre_stage * stage_stride, bar_full(pre_stage), k_at(P, s2, k), s2);
                    }
                    __syncwarp();
                    ++pre_stage;
                }
            }
            __syncwarp();
            pdl_wait();          // the activations' halves and all stores come after the preceding kernel
        } else if (ahead) {
            // Without the caller's promise nothing may be read into shared memory yet, but the weights of the first
            // stages can be asked into L2: a cache fill consumes nothing, and whatever the preceding kernel (or a peer, or
            // the host) still writes to those lines goes through the same L2.  The loads after the wait then hit.
            SegIter<Cfg> it2(P);
            Segment s2;
            uint32_t n_pre = 0;
            const uint32_t want = (uint32_t)(n_stages * P.l2_ahead);      // l2_ahead ring fills
            while (n_pre < want && it2.next(s2)) {
                for (int k = s2.k0; k < s2.k1 && n_pre < want; ++k, ++n_pre) {
                    if (elect_one_sync()) {
                        // (the scale slab of the group first: the first MMA waits for the re-tiled scales as well)
                        if (P.sf_tma && (k == s2.k0 || (k & 3) == 0)) {
                            if (WQ) tma_prefetch_l2_2d(&tm_sfq, (k_at(P, s2, k) >> 2) * 16, s2.q0);
                            else tma_prefetch_l2_2d(&tm_sfp, (k_at(P, s2, k) >> 2) * 16, s2.p0);
                        }
                        if (WQ) tma_prefetch_l2_2d(&tm_q, k_at(P, s2, k) * Cfg::BK, s2.q0);
                        else tma_prefetch_l2_2d(&tm_p, k_at(P, s2, k) * Cfg::BK, s2.p0);
                    }
                }
            }
            __syncwarp();
            pdl_wait();
        }
        while (ok && it.next(sg)) {
            for (int kb = sg.k0; kb < sg.k1 && ok;) {
                // LOAD_BATCH K-blocks are requested back to back, so that each row's adjacent 96-byte pieces
                // reach DRAM together (one page activation serves the whole run)
                const int nb = min(load_batch, sg.k1 - kb);
                for (int j = 0; j < nb && ok; ++j) {
                    const int k = kb + j;
                    if (P.sf_tma && (k == sg.k0 || (k & 3) == 0)) {
                        const int r = n_raw % Cfg::RAW_SLOTS;
                        const uint32_t ph = (n_raw / Cfg::RAW_SLOTS) & 1;
                        ok = wait_bar_warp(bar_raw_empty(r), ph ^ 1, abort_flag, P, kStatusTimeoutProducer);
                        if (!ok) break;
                        if (elect_one_sync()) {
                            const uint32_t dst = raw_base + r * Cfg::RAW_BYTES;
                            if (n_raw >= pre_raw) {
                                mbar_arrive_expect_tx(bar_raw_full(r), (uint32_t)P.raw_tx_bytes);
                                slab_weights(dst, bar_raw_full(r), k_at(P, sg, k), sg);
                            }
                            slab_other(dst, bar_raw_full(r), k_at(P, sg, k), sg);
                        }
                        ++n_raw;
                    }
                }
                if (!ok) break;
                // stages are released in order: when the last one of the batch is free, all of them are
                uint32_t last = st_idx + nb - 1, last_phase = st_phase;
                if (last >= (uint32_t)n_stages) { last -= n_stages; last_phase ^= 1; }
                ok = wait_bar_warp(bar_empty(last), last_phase ^ 1, abort_flag, P, kStatusTimeoutProducer);
                if (!ok) break;
                if (elect_one_sync()) {
                    for (int j = 0; j < nb; ++j) {
                        int s = (int)st_idx + j;
                        if (s >= n_stages) s -= n_stages;
                        const uint32_t dst = stage_base + s * stage_stride;
                        if (n_stage + j >= pre_stage) {
                            mbar_arrive_expect_tx(bar_full(s), (uint32_t)P.stage_tx_bytes);
                            load_weights(dst, bar_full(s), k_at(P, sg, kb + j), sg);
                        }
                        load_other(dst, bar_full(s), k_at(P, sg, kb + j), sg);
                    }
                }
                __syncwarp();
                n_stage += nb;
                st_idx += nb;
                if (st_idx >= (uint32_t)n_stages) { st_idx -= n_stages; st_phase ^= 1; }
                kb += nb;
            }
        }
    }
    // =========================================================== warp 1: MMA issuer
    else if (warp == 1) {
        SegIter<Cfg> it(P);
        Segment sg;
        uint32_t n_kb = 0, n_seg = 0, n_grp = 0;
        uint32_t st_idx = 0, st_phase = 0;        // ring position and round parity of K-block number n_kb
        bool ok = true;
        while (ok && it.next(sg)) {
            const int b = n_seg & 1;
            const uint32_t acc = tmem_base + (b ? Cfg::ACC_COL1 : 0);
            if (Cfg::OVERLAP) {
                if (n_seg > 0) ok = wait_bar_warp(bar_ovl, (n_seg - 1) & 1, abort_flag, P, kStatusTimeoutMma);
            } else {
                ok = wait_bar_warp(bar_acc_empty(b), ((n_seg >> 1) & 1) ^ 1, abort_flag, P, kStatusTimeoutMma);
            }
            if (!ok) break;
            tc_fence_after();
            for (int kb = sg.k0; kb < sg.k1; ++kb) {
                const int s = (int)st_idx;
                const int g = n_grp % Cfg::ATOM_GROUPS;
                // the scale atoms arrive per group of 4 K-blocks (one raw slab)
                if (kb == sg.k0 || (kb & 3) == 0)
                    ok = wait_bar_warp(bar_atom_full(g), (n_grp / Cfg::ATOM_GROUPS) & 1, abort_flag, P, kStatusTimeoutMma);
                ok = ok && wait_bar_warp(bar_full(s), st_phase, abort_flag, P, kStatusTimeoutMma);
                if (!ok) break;
                const bool group_done = (kb & 3) == 3 || kb == sg.k1 - 1;
                if (elect_one_sync()) {
                    const uint32_t sfa = tmem_base + Cfg::SF_COL + (n_kb & 1) * 16;
                    const uint32_t sfb = sfa + 4;
                    const uint32_t atom = atom_base + g * Cfg::GROUP_BYTES + (kb & 3) * Cfg::ATOM_BYTES;
                    {
                    tc_cp_32x128b_warpx4(sfa, smem_desc_sf(atom));
#pragma unroll
                    for (int q = 0; q < Cfg::QATOMS; ++q) tc_cp_32x128b_warpx4(sfb + 4 * q, smem_desc_sf(atom + 512 * (1 + q)));
                    }
                    const uint32_t sp = stage_base + s * stage_stride;
                    const uint64_t adesc = smem_desc_sw128(sp);
                    const uint64_t bdesc = smem_desc_sw128(sp + q_off);
#pragma unroll
                    for (uint32_t k = 0; k < 4; ++k) {
                        mma_mxf8f6f4(acc, adesc + 2 * k, bdesc + 2 * k, idesc_with_sf(P.idesc, k),
                                     sfa | (k << 30), sfb | (k << 30), (kb > sg.k0 || k > 0) ? 1u : 0u);
                    }
                    tc_commit(bar_empty(s));
                    if (group_done) tc_commit(bar_atom_empty(g));
                }
                __syncwarp();
                ++n_kb;
                if (++st_idx == (uint32_t)n_stages) { st_idx = 0; st_phase ^= 1; }
                if (group_done) ++n_grp;
            }
            if (!ok) break;
            if (elect_one_sync()) tc_commit(bar_acc_full(b));
            __syncwarp();
            ++n_seg;
        }
    }
    // =========================================================== warps 2-3: scale re-tilers
    // Each group of 4 K-blocks (one raw slab of 16 scale bytes per row) is handled by one of the two warps,
    // alternately: raw words -> registers -> the 4 x (1+QATOMS) atoms of the group -> one proxy fence ->
    // one arrival.
    else if (warp == 2 || warp == 3) {
        SegIter<Cfg> it(P);
        Segment sg;
        uint32_t n_grp = 0;
        bool ok = true;
        constexpr int QG = (BN + 31) / 32;        // 32-row groups on the Q side
        while (ok && it.next(sg)) {
            for (int kb = sg.k0; kb < sg.k1 && ok;) {
                const int kb_next = min(sg.k1, (kb | 3) + 1);
                if ((int)(n_grp & 1) == warp - 2) {
                    uint32_t rp[4][4];                  // [32-row group][K-block of the slab]
                    uint32_t rq[Cfg::QATOMS * 4][4];
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
                        for (int c = 0; c < Cfg::QATOMS * 4; ++c) {
                            if (c < QG) {
                                const uint4 v = *reinterpret_cast<const uint4*>(raw + Cfg::BM * 16 + (lane + 32 * c) * 16);
                                rq[c][0] = v.x; rq[c][1] = v.y; rq[c][2] = v.z; rq[c][3] = v.w;
                            } else {
                                rq[c][0] = rq[c][1] = rq[c][2] = rq[c][3] = 0u;
                            }
                        }
                        mbar_arrive(bar_raw_empty(r));
                    } else {
                        // Scale rows that cannot be TMA boxes: the 4-byte words of the group's K-blocks are read from
                        // global memory directly.  Four adjacent lanes read the four words of one row (16 contiguous
                        // bytes), so an instruction touches 8 rows, not 32; each word goes straight to its place in the
                        // atom of its K-block: row (r % 32), 4-byte column (r / 32).
                        const int kb4 = k_at(P, sg, kb & ~3);
                        const int w = lane & 3;
                        constexpr int NI = 16 + 4 * QG;             // 8 rows per step: 128 rows of P, then the 32-row groups of Q
                        uint32_t v[NI];
#pragma unroll
                        for (int i = 0; i < NI; ++i) {
                            const int ridx = 8 * i + (lane >> 2);
                            const bool is_p = i < 16;
                            const int row = is_p ? sg.p0 + ridx : sg.q0 + ridx - 128;
                            const bool live = row < (is_p ? P.p_rows : P.q_rows) && kb4 + w < P.kblocks;
                            v[i] = live ? __ldg(reinterpret_cast<const uint32_t*>((is_p ? P.sfp : P.sfq) + (size_t)row * P.sf_ld + (kb4 + w) * 4)) : 0u;
                        }
                        const int g = n_grp % Cfg::ATOM_GROUPS;
                        ok = wait_bar_warp(bar_atom_empty(g), ((n_grp / Cfg::ATOM_GROUPS) & 1) ^ 1, abort_flag, P, kStatusTimeoutScale);
                        if (!ok) break;
                        uint8_t* atom = smem_gen + (atom_base - smem_base) + g * Cfg::GROUP_BYTES + w * Cfg::ATOM_BYTES;
#pragma unroll
                        for (int i = 0; i < NI; ++i) {
                            const int ridx = 8 * i + (lane >> 2);
                            const int part = ridx >> 7, r = ridx & 127;     // atom 0: P, then one atom per 128 rows of Q
                            *reinterpret_cast<uint32_t*>(atom + 512 * part + (r & 31) * 16 + (r >> 5) * 4) = v[i];
                        }
                        fence_proxy_async_smem();
                        mbar_arrive(bar_atom_full(g));
                        ++n_grp;
                        kb = kb_next;
                        continue;
                    }
                    const int g = n_grp % Cfg::ATOM_GROUPS;
                    ok = wait_bar_warp(bar_atom_empty(g), ((n_grp / Cfg::ATOM_GROUPS) & 1) ^ 1, abort_flag, P, kStatusTimeoutScale);
                    if (!ok) break;
                    uint8_t* grp = smem_gen + (atom_base - smem_base) + g * Cfg::GROUP_BYTES;
                    // atom layout: 32 rows of 16 bytes; row (r%32) holds, for the four 32-row groups c = r/32,
                    // the 4 scale bytes of one K-block: byte offset (r%32)*16 + c*4 + (k/32)%4
#pragma unroll
                    for (int jj = 0; jj < 4; ++jj) {
                        uint8_t* atom = grp + jj * Cfg::ATOM_BYTES;
                        *reinterpret_cast<uint4*>(atom + lane * 16) = make_uint4(rp[0][jj], rp[1][jj], rp[2][jj], rp[3][jj]);
#pragma unroll
                        for (int qa = 0; qa < Cfg::QATOMS; ++qa)
                            *reinterpret_cast<uint4*>(atom + 512 * (1 + qa) + lane * 16) =
                                make_uint4(rq[4 * qa][jj], rq[4 * qa + 1][jj], rq[4 * qa + 2][jj], rq[4 * qa + 3][jj]);
                    }
                    fence_proxy_async_smem();
                    mbar_arrive(bar_atom_full(g));
                }
                ++n_grp;
                kb = kb_next;
            }
        }
    }
    // =========================================================== warps 4-7: epilogue
    else if (warp >= 4) {
        const int quad = warp & 3;
        const int prow = quad * 32 + lane;                 // row of the tile this thread owns (TMEM lane)
        const int etid = threadIdx.x - 128;
        SegIter<Cfg> it(P);
        Segment sg;
        uint32_t n_seg = 0;
        bool ok = true;
        constexpr int CW = BN >= 32 ? 32 : 16;             // columns per TMEM load
        constexpr int NCH = BN / CW;
        while (ok && it.next(sg)) {
            const int b = n_seg & 1;
            const bool affine = has_affine(P);
            // unswapped fp32 epilogue: this thread's row factor and up to two of the tile's column factors / biases are
            // fetched while the accumulator is still being computed, then shared through shared memory
            float row_scale = 1.f, cs[2] = {1.f, 1.f}, cb[2] = {0.f, 0.f};
            if (!Cfg::SWAP && affine) {
                if (P.scale_m && sg.p0 + prow < P.c_rows) row_scale = __ldg(P.scale_m + sg.p0 + prow);
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    const int c = sg.q0 + etid + 128 * h;
                    if (etid + 128 * h < BN && c < P.c_cols) {
                        if (P.scale_n) cs[h] = __ldg(P.scale_n + c);
                        if (P.bias_n) cb[h] = __ldg(P.bias_n + c);
                    }
                }
            }
            ok = epilogue_all(wait_bar_warp(bar_acc_full(b), (n_seg >> 1) & 1, abort_flag, P, kStatusTimeoutEpilogue));
            if (!ok) break;
            tc_fence_after();
            if (!Cfg::SWAP && affine) {
                // (the agreement above was a barrier of these 128 threads: nobody still reads the previous tile's vectors)
#pragma unroll
                for (int h = 0; h < 2; ++h)
                    if (etid + 128 * h < BN) { aff_sn[etid + 128 * h] = cs[h]; aff_bn[etid + 128 * h] = cb[h]; }
                asm volatile("bar.sync 1, 128;" ::: "memory");
            }
            const uint32_t tacc = tmem_base + ((uint32_t)(quad * 32) << 16) + (b ? Cfg::ACC_COL1 : 0);
            const bool partial = Cfg::STREAMK && sg.nseg > 1;
            float* slot = nullptr;
            if (partial) slot = P.ws_partial + ((size_t)sg.tile * P.ws_slots + sg.segidx) * (size_t)(BN * 128);
            const int p = sg.p0 + prow;
            // with overlapping accumulators the 32 shared columns are drained first
            auto chunk_of = [&](int ci) { return Cfg::OVERLAP ? (b == 0 ? (ci + NCH - 1) % NCH : ci) : ci; };
            // The tile is read from TMEM in groups of up to four chunks per wait.  A load and its wait are a round trip of
            // about half a microsecond whatever the width: drained chunk by chunk, a 256-column tile took 4.3 us (a tenth
            // of a skinny launch), whether or not the next chunk's load was already under way and whether the stores went
            // to rows of C or to shared memory.  Chunks that lie wholly past the tile's own columns are not read.
            constexpr int G = NCH < 4 ? NCH : 4;
            // unswapped form: a warp whose 32 rows all lie below C (M <= 96) neither reads nor stores: the TMEM read-out
            // shares 64 bytes per clock among the warps
            const bool warp_live = Cfg::SWAP || sg.p0 + quad * 32 < (partial ? P.p_rows : P.c_rows);
            // The last tile of a CTA overlaps nothing, and in the unswapped form every lane stores to a row of its own: a
            // store instruction touches 32 lines and costs the load/store unit about 300 cycles, 2.2 to 2.8 us for a
            // 128 x 200 tile whatever the number of live rows.  By then the ring is idle (every load has landed and every MMA
            // has read it: that is what acc_full says), so the whole 64-column pieces of that tile are staged there as
            // swizzled 128-byte rows and leave by TMA stores; columns past the last whole piece keep the plain stores.
            const bool staged = !Cfg::SWAP && CW == 32 && P.c_tma_last && !partial && P.q_fmt < 0 && it.last();
            const int tile_cols = min(P.c_cols - sg.q0, P.q_tile_rows);
            const int n_pieces = staged ? tile_cols / 64 : 0;
            auto process = [&](int ch, uint32_t (&v)[CW]) {
                const int qc = sg.q0 + ch * CW;              // first D column of this chunk
                if (!Cfg::SWAP && ch * CW >= P.q_tile_rows) return;          // nothing of this chunk belongs to the tile
                if (!partial && affine) {
                    if constexpr (Cfg::SWAP) {
                        affine_chunk<true, CW>(P, v, p, qc);
                    } else {
                        // (acc * column scale) * row scale + bias, three roundings; the vectors are broadcast reads
#pragma unroll
                        for (int c = 0; c < CW; c += 4) {
                            const float4 sn = *reinterpret_cast<const float4*>(aff_sn + ch * CW + c);
                            const float4 bn = *reinterpret_cast<const float4*>(aff_bn + ch * CW + c);
                            v[c + 0] = __float_as_uint(__fadd_rn(__fmul_rn(__fmul_rn(__uint_as_float(v[c + 0]), sn.x), row_scale), bn.x));
                            v[c + 1] = __float_as_uint(__fadd_rn(__fmul_rn(__fmul_rn(__uint_as_float(v[c + 1]), sn.y), row_scale), bn.y));
                            v[c + 2] = __float_as_uint(__fadd_rn(__fmul_rn(__fmul_rn(__uint_as_float(v[c + 2]), sn.z), row_scale), bn.z));
                            v[c + 3] = __float_as_uint(__fadd_rn(__fmul_rn(__fmul_rn(__uint_as_float(v[c + 3]), sn.w), row_scale), bn.w));
                        }
                    }
                }
                if (partial) {
                    // rows past the end of P (a skinny unswapped A) are neither published nor summed
                    if (p < P.p_rows) {
#pragma unroll
                        for (int i = 0; i < CW; ++i) slot[(size_t)(ch * CW + i) * 128 + prow] = __uint_as_float(v[i]);
                    }
                } else if (Cfg::SWAP && P.q_fmt >= 0) {
                    // the result leaves as an MX operand: the warp's 32 rows p are one 32-column block of C row q
#pragma unroll
                    for (int i = 0; i < CW; ++i)
                        quant_store_lanes(__uint_as_float(v[i]), P.q_fmt, P.q_out, (size_t)P.q_ld, P.q_scales, P.c_cols,
                                          qc + i, sg.p0 + quad * 32, qc + i < P.c_rows && sg.p0 + quad * 32 < P.c_cols);
                } else if (Cfg::SWAP) {
                    // D[p,q] -> C[q,p]: consecutive lanes write consecutive bf16 of one C row
                    // (rows past the tile's own rows belong to the next tile)
                    if (p < P.c_cols && prow < P.p_tile_rows) {
#pragma unroll
                        for (int i = 0; i < CW; ++i)
                            if (qc + i < P.c_rows)
                                P.c[(size_t)(qc + i) * P.ldc + p] = __float2bfloat16_rn(__uint_as_float(v[i]));
                    }
                } else if (P.q_fmt >= 0) {
                    // the result leaves as an MX operand of the next layer: this thread's 32 columns are one block
                    if constexpr (CW == 32) {
                        if (p < P.c_rows && qc < P.c_cols)
                            quant_store32(v, P.q_fmt, P.q_out, (size_t)P.q_ld, P.q_scales, P.c_cols, p, qc);
                    }
                } else if (!Cfg::SWAP && CW == 32 && (ch >> 1) < n_pieces) {
                    // row prow of piece ch / 2 is 128 bytes in 16-byte units; unit u sits at u ^ (row % 8): the 128-byte
                    // swizzle the TMA store expects
                    const uint32_t rowaddr = stage_base + (uint32_t)(ch >> 1) * (128u * 128u) + (uint32_t)prow * 128u;
                    const uint32_t sw = (uint32_t)(prow & 7);
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        const uint32_t x0 = pack_bf16x2(__uint_as_float(v[8 * c + 0]), __uint_as_float(v[8 * c + 1]));
                        const uint32_t x1 = pack_bf16x2(__uint_as_float(v[8 * c + 2]), __uint_as_float(v[8 * c + 3]));
                        const uint32_t x2 = pack_bf16x2(__uint_as_float(v[8 * c + 4]), __uint_as_float(v[8 * c + 5]));
                        const uint32_t x3 = pack_bf16x2(__uint_as_float(v[8 * c + 6]), __uint_as_float(v[8 * c + 7]));
                        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};"
                                     ::"r"(rowaddr + ((((uint32_t)(ch & 1) * 4u + (uint32_t)c) ^ sw) << 4)), "r"(x0), "r"(x1), "r"(x2), "r"(x3) : "memory");
                    }
                } else {
                    // columns past the tile's own columns belong to the next tile
                    const int q_lim = min(P.c_cols, sg.q0 + P.q_tile_rows);
                    if (p < P.c_rows)
                    for (int d = 0; d < P.ndst; ++d) {          // every destination gets the tile (d > 0: peer memory)
                        __nv_bfloat16* cbase = d == 0 ? P.c : P.c_more[d - 1];
                        __nv_bfloat16* dst = cbase + (size_t)p * P.ldc + qc;
                        const bool vec = ((P.ldc & 7) == 0) && ((reinterpret_cast<uintptr_t>(cbase) & 15) == 0) && ((P.q_tile_rows & 7) == 0);
                        // whole 32-byte sectors where the chunk starts on one: a 16-byte store is a partial write of its sector
                        if (CW == 32 && vec && ((P.ldc & 15) == 0) && ((reinterpret_cast<uintptr_t>(dst) & 31) == 0) && qc + CW <= q_lim) {
#pragma unroll
                            for (int i = 0; i < CW; i += 16)
                                st_global_v8(dst + i, pack_bf16x2(__uint_as_float(v[i + 0]), __uint_as_float(v[i + 1])),
                                             pack_bf16x2(__uint_as_float(v[i + 2]), __uint_as_float(v[i + 3])),
                                             pack_bf16x2(__uint_as_float(v[i + 4]), __uint_as_float(v[i + 5])),
                                             pack_bf16x2(__uint_as_float(v[i + 6]), __uint_as_float(v[i + 7])),
                                             pack_bf16x2(__uint_as_float(v[i + 8]), __uint_as_float(v[i + 9])),
                                             pack_bf16x2(__uint_as_float(v[i + 10]), __uint_as_float(v[i + 11])),
                                             pack_bf16x2(__uint_as_float(v[i + 12]), __uint_as_float(v[i + 13])),
                                             pack_bf16x2(__uint_as_float(v[i + 14]), __uint_as_float(v[i + 15])));
                            continue;
                        }
#pragma unroll
                        for (int i = 0; i < CW; i += 8) {
                            if (vec && qc + i + 8 <= q_lim) {
                                uint4 o;
                                o.x = pack_bf16x2(__uint_as_float(v[i + 0]), __uint_as_float(v[i + 1]));
                                o.y = pack_bf16x2(__uint_as_float(v[i + 2]), __uint_as_float(v[i + 3]));
                                o.z = pack_bf16x2(__uint_as_float(v[i + 4]), __uint_as_float(v[i + 5]));
                                o.w = pack_bf16x2(__uint_as_float(v[i + 6]), __uint_as_float(v[i + 7]));
                                *reinterpret_cast<uint4*>(dst + i) = o;
                            } else {
#pragma unroll
                                for (int e = 0; e < 8; ++e)
                                    if (qc + i + e < q_lim) dst[i + e] = __float2bfloat16_rn(__uint_as_float(v[i + e]));
                            }
                        }
                    }
                }
            };
#pragma unroll 1
            for (int cg = 0; cg < NCH; cg += G) {
                uint32_t v[G][CW];
#pragma unroll
                for (int g = 0; g < G; ++g) {
                    const int ch = chunk_of(cg + g);
                    if (warp_live && (Cfg::SWAP || ch * CW < P.q_tile_rows)) {
                        if constexpr (CW == 32) tmem_ld_x32(tacc + ch * CW, reinterpret_cast<uint32_t(&)[32]>(v[g]));
                        else tmem_ld_x16(tacc + ch * CW, reinterpret_cast<uint32_t(&)[16]>(v[g]));
                    }
                }
                tmem_ld_wait();
                // (the first group holds the columns the two accumulators share; after the last group nothing of this
                // accumulator is left in TMEM)
                if (Cfg::OVERLAP && cg == 0) { tc_fence_before(); __syncwarp(); if (lane == 0) mbar_arrive(bar_ovl); }
                if (!Cfg::OVERLAP && cg + G >= NCH) { tc_fence_before(); mbar_arrive(bar_acc_empty(b)); }
                if (warp_live) {
#pragma unroll
                    for (int g = 0; g < G; ++g) process(chunk_of(cg + g), v[g]);
                }
            }
            if (n_pieces > 0) {
                fence_proxy_async_smem();
                asm volatile("bar.sync 1, 128;" ::: "memory");
                if (etid == 0) {
                    for (int pc = 0; pc < n_pieces; ++pc) tma_store_2d(&tm_c, stage_base + (uint32_t)pc * (128u * 128u), sg.q0 + 64 * pc, sg.p0);
                    bulk_commit_group();
                    bulk_wait_group_read<0>();       // the ring is read before the CTA leaves (this was its last tile)
                }
            }
            if (partial) {
                // publish this CTA's partial; the contributor that arrives last adds all partials of the
                // tile in slot order (a fixed order, so the result does not depend on timing)
                __threadfence();
                asm volatile("bar.sync 1, 128;" ::: "memory");
                if (etid == 0) *ticket_slot = (int)atomicAdd(P.ws_counter + sg.tile, 1u);
                asm volatile("bar.sync 1, 128;" ::: "memory");
                const bool last = (*ticket_slot == sg.nseg - 1);
                asm volatile("bar.sync 1, 128;" ::: "memory");
                if (last) {
                    __threadfence();
                    // Each thread sums 4 consecutive rows (one 16-byte load per slot) of every fourth column: JB columns
                    // at a time, their loads independent and in flight together; each element is still summed in slot
                    // order starting from zero, so the result does not depend on which CTA does the summing.
                    const int r4 = 4 * lane;                         // first of this thread's 4 rows
                    const float* base = P.ws_partial + (size_t)sg.tile * P.ws_slots * (size_t)(BN * 128) + r4;
                    constexpr int NJ = BN / 4;                       // columns per thread: quad + 4 * j
                    constexpr int JB = NJ >= 8 ? 8 : NJ;
                    const int pr = sg.p0 + r4;
                    // every lane owns 4 rows; lanes whose rows all lie past the end of P have
                    // nothing to sum (their partials were never written) but stay in the loop for the warp-wide steps
                    const bool rows_live = pr < P.p_rows;
#pragma unroll 1
                    for (int j0 = 0; j0 < NJ; j0 += JB) {
                        float4 acc[JB];
                        if (!rows_live) {
#pragma unroll
                            for (int j = 0; j < JB; ++j) acc[j] = make_float4(0.f, 0.f, 0.f, 0.f);
                        } else if (sg.nseg == 2) {                       // the common case: both slots fetched at once
                            float4 t0[JB], t1[JB];
#pragma unroll
                            for (int j = 0; j < JB; ++j) {
                                const float* src = base + (size_t)(quad + 4 * (j0 + j)) * 128;
                                t0[j] = __ldcg(reinterpret_cast<const float4*>(src));
                                t1[j] = __ldcg(reinterpret_cast<const float4*>(src + (size_t)(BN * 128)));
                            }
#pragma unroll
                            for (int j = 0; j < JB; ++j)
                                acc[j] = make_float4((0.f + t0[j].x) + t1[j].x, (0.f + t0[j].y) + t1[j].y,
                                                     (0.f + t0[j].z) + t1[j].z, (0.f + t0[j].w) + t1[j].w);
                        } else {
#pragma unroll
                            for (int j = 0; j < JB; ++j) acc[j] = make_float4(0.f, 0.f, 0.f, 0.f);
                            for (int sgi = 0; sgi < sg.nseg; ++sgi) {
                                float4 t[JB];
#pragma unroll
                                for (int j = 0; j < JB; ++j)
                                    t[j] = __ldcg(reinterpret_cast<const float4*>(base + (size_t)sgi * (BN * 128) + (size_t)(quad + 4 * (j0 + j)) * 128));
#pragma unroll
                                for (int j = 0; j < JB; ++j) { acc[j].x += t[j].x; acc[j].y += t[j].y; acc[j].z += t[j].z; acc[j].w += t[j].w; }
                            }
                        }
#pragma unroll
                        for (int j = 0; j < JB; ++j) {
                            const int q = sg.q0 + quad + 4 * (j0 + j);
                            float x[4] = {acc[j].x, acc[j].y, acc[j].z, acc[j].w};
                            if (affine) {
#pragma unroll
                                for (int e = 0; e < 4; ++e) x[e] = affine_one<Cfg::SWAP>(P, x[e], pr + e, q);
                            }
                            if (Cfg::SWAP && P.q_fmt >= 0) {
                                // 8 lanes x 4 rows are one 32-column block of C row q
                                // (every lane takes part in the shuffles; blocks past the edge only skip their stores)
                                quant_store_lanes4(x, P.q_fmt, P.q_out, (size_t)P.q_ld, P.q_scales, P.c_cols, q,
                                                   sg.p0 + (r4 & ~31), q < P.c_rows && sg.p0 + (r4 & ~31) < P.c_cols);
                            } else if (Cfg::SWAP) {
                                // D[p,q] -> C[q,p]: the 4 rows are 4 consecutive bf16 of C's row q
                                if (q < P.c_rows) {
                                    __nv_bfloat16* dst = P.c + (size_t)q * P.ldc + pr;
                                    if (pr + 3 < P.c_cols && (reinterpret_cast<uintptr_t>(dst) & 7) == 0) {
                                        uint2 o;
                                        o.x = pack_bf16x2(x[0], x[1]);
                                        o.y = pack_bf16x2(x[2], x[3]);
                                        *reinterpret_cast<uint2*>(dst) = o;
                                    } else {
#pragma unroll
                                        for (int e = 0; e < 4; ++e)
                                            if (pr + e < P.c_cols) dst[e] = __float2bfloat16_rn(x[e]);
                                    }
                                }
                            } else if (q < P.c_cols) {
#pragma unroll
                                for (int e = 0; e < 4; ++e)
                                    if (pr + e < P.c_rows) P.c[(size_t)(pr + e) * P.ldc + q] = __float2bfloat16_rn(x[e]);
                            }
                        }
                    }
                    if (etid == 0) P.ws_counter[sg.tile] = 0u;
                }
            }
            ++n_seg;
        }
    }

    // ---- teardown: every role loop above terminates (bounded waits), so all warps arrive here
    if (*abort_flag) {
        // give copies and MMAs that are still in flight time to land before shared memory and TMEM go away
        const long long t0 = clock64();
        while (clock64() - t0 < 400000) { __nanosleep(1000); }
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    if (warp == 1) tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
}

}  // namespace mxfp6
