// C ABI of the MX-FP6 GEMM path (see include/mxfp6.h): argument checks, tensor maps, kernel choice,
// launches.  Plain pointers and sizes only; no torch types.
#include "../../include/mxfp6.h"

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp6.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>

#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <atomic>
#include <cstring>
#include <map>
#include <memory>
#include <mutex>
#include <string>
#include <utility>
#include <vector>

#include "gemm_kernel_2cta.cuh"
#include "quantize_kernel.cuh"

namespace mxfp6 {

// ---------------------------------------------------------------------------------- errors
static thread_local std::string g_err;
static int fail(int code, const char* fmt, ...) {
    char buf[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof buf, fmt, ap);
    va_end(ap);
    g_err = buf;
    return code;
}
#define CUDA_TRY(expr)                                                                              \
    do {                                                                                            \
        cudaError_t e_ = (expr);                                                                    \
        if (e_ != cudaSuccess) return fail(MXFP6_ERR_CUDA, "%s: %s", #expr, cudaGetErrorString(e_)); \
    } while (0)

// ---------------------------------------------------------------------------------- options
// Test hooks.  Their first values come from the environment when the library is first used; afterwards only
// mxfp6_debug_option changes them, so no call path reads the environment.
struct Options {
    int force_bn = 0, force_swap = -1, force_sk = -1, force_pair = -1;   // MXFP6_FORCE_CFG = "bn,swap,streamk[,pair]"
    int no_sf_tma = 0;       // MXFP6_NO_SF_TMA: scale arrays read with plain loads
    int pdl = 1;             // MXFP6_PDL: programmatic dependent launch
    int group_p = 16;        // MXFP6_GROUP_P: pair tiles per rasterisation group
    int quant_quad = 0;      // MXFP6_QUANT_PATH=quad: the plain-load quantiser
    int wait_ms = 2000;      // MXFP6_WAIT_MS: budget of one bounded wait (read when a device is first used)
    // MXFP6_L2 = "load,store": L2 eviction policy of the pair kernel's TMA traffic (0 normal, 1 evict_first, 2 evict_last).
    // Operand tiles are asked for again by other pairs and C is written once: keeping the former and letting the latter
    // go first measured +2.6 % at 8192^3 and +2 % at 4096^3 against no hints.
    int l2_load = 2, l2_store = 1;
    int tail_split = 1;      // MXFP6_TAIL_SPLIT: the pair kernel splits the tiles of its last partial wave along K
    int decode_rows = 1;     // MXFP6_DECODE_ROWS: skinny problems take the row-balanced kernel when they qualify
    int decode_stages = 0, decode_batch = 0;   // MXFP6_DECODE_RING = "stages,batch": ring of that kernel (0 = chosen by the library)
    int push_rotate = 1;     // MXFP6_PUSH_ROTATE: pair kernel, rotate the order of the peer destinations from piece to piece
    int l2_ahead = 1;        // MXFP6_L2_AHEAD: the single-CTA kernel asks the weights of its first stages into L2 while it waits for the preceding kernel
    int c_tma_last = 1;      // MXFP6_C_TMA_LAST: the unswapped single-CTA kernel drains the last tile of every CTA through its idle ring and TMA stores
    int c_plain = 0;         // MXFP6_C_PLAIN: the pair kernel writes C with plain stores from its staging buffer even where TMA stores are possible
    int k_rot = 1;           // MXFP6_K_ROT: the even-rows skinny forms start each tile's K loop at its own K-block
};
static Options g_opt;
static std::once_flag g_opt_once;
static std::atomic<unsigned> g_opt_epoch{1};      // bumped by every change: cached launch recipes carry the epoch they were built in

static bool set_option(const char* name, const char* v) {
    const Options d{};
    if (!strcmp(name, "MXFP6_FORCE_CFG")) {
        g_opt.force_bn = d.force_bn; g_opt.force_swap = d.force_swap; g_opt.force_sk = d.force_sk; g_opt.force_pair = d.force_pair;
        if (v) sscanf(v, "%d,%d,%d,%d", &g_opt.force_bn, &g_opt.force_swap, &g_opt.force_sk, &g_opt.force_pair);
    } else if (!strcmp(name, "MXFP6_NO_SF_TMA")) g_opt.no_sf_tma = v ? atoi(v) : d.no_sf_tma;
    else if (!strcmp(name, "MXFP6_PDL")) g_opt.pdl = v ? atoi(v) : d.pdl;
    else if (!strcmp(name, "MXFP6_GROUP_P")) { g_opt.group_p = v ? atoi(v) : d.group_p; if (g_opt.group_p < 1) g_opt.group_p = 1; }
    else if (!strcmp(name, "MXFP6_QUANT_PATH")) g_opt.quant_quad = (v && !strcmp(v, "quad")) ? 1 : 0;
    else if (!strcmp(name, "MXFP6_WAIT_MS")) g_opt.wait_ms = v ? atoi(v) : d.wait_ms;
    else if (!strcmp(name, "MXFP6_L2")) {
        g_opt.l2_load = d.l2_load; g_opt.l2_store = d.l2_store;
        if (v) sscanf(v, "%d,%d", &g_opt.l2_load, &g_opt.l2_store);
    } else if (!strcmp(name, "MXFP6_TAIL_SPLIT")) g_opt.tail_split = v ? atoi(v) : d.tail_split;
    else if (!strcmp(name, "MXFP6_DECODE_ROWS")) g_opt.decode_rows = v ? atoi(v) : d.decode_rows;
    else if (!strcmp(name, "MXFP6_K_ROT")) g_opt.k_rot = v ? atoi(v) : d.k_rot;
    else if (!strcmp(name, "MXFP6_C_PLAIN")) g_opt.c_plain = v ? atoi(v) : d.c_plain;
    else if (!strcmp(name, "MXFP6_C_TMA_LAST")) g_opt.c_tma_last = v ? atoi(v) : d.c_tma_last;
    else if (!strcmp(name, "MXFP6_L2_AHEAD")) g_opt.l2_ahead = v ? atoi(v) : d.l2_ahead;
    else if (!strcmp(name, "MXFP6_PUSH_ROTATE")) g_opt.push_rotate = v ? atoi(v) : d.push_rotate;
    else if (!strcmp(name, "MXFP6_DECODE_RING")) {
        g_opt.decode_stages = d.decode_stages; g_opt.decode_batch = d.decode_batch;
        if (v) sscanf(v, "%d,%d", &g_opt.decode_stages, &g_opt.decode_batch);
    }
    else return false;
    return true;
}
static const char* const kOptionNames[] = {"MXFP6_FORCE_CFG", "MXFP6_NO_SF_TMA", "MXFP6_PDL", "MXFP6_GROUP_P", "MXFP6_QUANT_PATH",
                                           "MXFP6_WAIT_MS", "MXFP6_L2", "MXFP6_TAIL_SPLIT", "MXFP6_DECODE_ROWS", "MXFP6_DECODE_RING", "MXFP6_K_ROT", "MXFP6_PUSH_ROTATE", "MXFP6_C_PLAIN", "MXFP6_C_TMA_LAST", "MXFP6_L2_AHEAD"};
static const Options& options() {
    std::call_once(g_opt_once, [] {
        for (const char* n : kOptionNames)
            if (const char* v = getenv(n)) set_option(n, v);
    });
    return g_opt;
}

// ---------------------------------------------------------------------------------- device state
// Device-side status word written by kernels whose bounded waits run out.
static __device__ int g_status_word[4];

struct DeviceState {
    bool init = false;
    int sm_count = 0;
    int cc_major = 0;
    unsigned long long wait_cycles = 0;
    int* status = nullptr;       // device address of g_status_word on this device
    void* ws = nullptr;          // library-owned scratch for split tiles (the newest and largest buffer)
    size_t ws_bytes = 0;
    std::vector<std::pair<void*, size_t>> ws_all;   // every buffer ever handed out: none is freed, launches and graphs may hold them
    std::map<const void*, bool> smem_attr_set;
};
static std::mutex g_mu;
static DeviceState g_dev[64];

static int get_device_state(DeviceState** out, int* dev_out = nullptr) {
    int dev = 0;
    CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return fail(MXFP6_ERR_BAD_ARG, "device index %d out of range", dev);
    if (dev_out) *dev_out = dev;
    DeviceState& d = g_dev[dev];
    std::lock_guard<std::mutex> lk(g_mu);      // two threads may make their first call on a device together
    if (!d.init) {
        int khz = 0;
        CUDA_TRY(cudaDeviceGetAttribute(&d.sm_count, cudaDevAttrMultiProcessorCount, dev));
        CUDA_TRY(cudaDeviceGetAttribute(&d.cc_major, cudaDevAttrComputeCapabilityMajor, dev));
        CUDA_TRY(cudaDeviceGetAttribute(&khz, cudaDevAttrClockRate, dev));
        if (d.cc_major != 10) return fail(MXFP6_ERR_UNSUPPORTED, "device %d is sm_%d0; this library is sm_100a only", dev, d.cc_major);
        d.wait_cycles = (unsigned long long)khz * (unsigned long long)options().wait_ms;
        CUDA_TRY(cudaGetSymbolAddress((void**)&d.status, g_status_word));
        CUDA_TRY(cudaMemset(d.status, 0, sizeof(int) * 4));
        d.init = true;
    }
    *out = &d;
    return MXFP6_OK;
}

// smem attribute of a kernel, once per device (callers hold no lock)
static int ensure_smem_attr(DeviceState& d, const void* kern, int bytes) {
    std::lock_guard<std::mutex> lk(g_mu);
    if (!d.smem_attr_set[kern]) {
        CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes));
        d.smem_attr_set[kern] = true;
    }
    return MXFP6_OK;
}

// ---------------------------------------------------------------------------------- tensor maps
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static std::atomic<EncodeTiledFn> g_encode{nullptr};

static int get_encode_fn(EncodeTiledFn* out) {
    EncodeTiledFn f = g_encode.load(std::memory_order_acquire);
    if (!f) {
        void* fn = nullptr;
        cudaDriverEntryPointQueryResult qres;
        CUDA_TRY(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres));
        if (!fn || qres != cudaDriverEntryPointSuccess) return fail(MXFP6_ERR_CUDA, "cuTensorMapEncodeTiled not available from the driver");
        f = (EncodeTiledFn)fn;
        g_encode.store(f, std::memory_order_release);
    }
    *out = f;
    return MXFP6_OK;
}

// kind 0: packed 6-bit operand [rows, K] (inner = K elements), box 128 x box_rows, 128-byte swizzle
// kind 1: scale bytes [rows, K/32] (inner = K/32 bytes), box 16 x box_rows, no swizzle
// kind 3: fp8 operand [rows, K] (inner = K bytes), box 128 x box_rows, 128-byte swizzle
// kind 2: bf16 output block [rows, inner] with a row stride of stride_bytes, box 64 x box_rows, 128-byte swizzle
// kind 4: quantiser source, fp32 viewed as [blocks, 32] (128-byte rows), box 32 x box_rows, 128-byte swizzle
// kind 5: quantiser source, bf16 viewed as [blocks, 32] (64-byte rows), box 32 x box_rows, 64-byte swizzle
// kind 6: re-quantised fp6 output bytes [rows, 3N/4] (inner = bytes per row), box 48 x box_rows, no swizzle
// kind 7: re-quantised fp8 output bytes [rows, N], box 64 x box_rows, 64-byte swizzle
// Encoded maps are kept inside the launch recipe of the call that uses them; a small per-thread table of recent
// encodings serves callers that alternate between a few buffers with otherwise new argument combinations.
struct MapKey {
    const void* ptr; int64_t rows, inner, stride; int box_rows, kind;
    bool operator==(const MapKey& o) const {
        return ptr == o.ptr && rows == o.rows && inner == o.inner && stride == o.stride && box_rows == o.box_rows && kind == o.kind;
    }
};
constexpr int kMapSlots = 64;
struct MapCache {
    MapKey key[kMapSlots];
    CUtensorMap map[kMapSlots];
    bool used[kMapSlots] = {};
};
static thread_local std::unique_ptr<MapCache> t_maps;

static int make_map(const void* ptr, int64_t rows, int64_t inner, int box_rows, int kind, CUtensorMap* out,
                    int64_t stride_bytes = 0) {
    const MapKey mk{ptr, rows, inner, stride_bytes, box_rows, kind};
    if (!t_maps) t_maps.reset(new MapCache());
    const size_t h = ((reinterpret_cast<uintptr_t>(ptr) >> 8) * 0x9E3779B97F4A7C15ull + (uint64_t)rows * 31 + (uint64_t)box_rows * 7 + (uint64_t)kind) % kMapSlots;
    if (t_maps->used[h] && t_maps->key[h] == mk) { *out = t_maps->map[h]; return MXFP6_OK; }
    EncodeTiledFn encode = nullptr;
    int rc = get_encode_fn(&encode);
    if (rc) return rc;
    cuuint64_t dims[2] = {(cuuint64_t)inner, (cuuint64_t)rows};
    cuuint64_t strides[1];
    cuuint32_t box[2] = {128, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUtensorMapDataType dt = CU_TENSOR_MAP_DATA_TYPE_UINT8;
    CUtensorMapSwizzle sw = CU_TENSOR_MAP_SWIZZLE_128B;
    switch (kind) {
        case 0: strides[0] = (cuuint64_t)(inner * 3 / 4); dt = CU_TENSOR_MAP_DATA_TYPE_16U6_ALIGN16B; break;
        case 1: strides[0] = (cuuint64_t)inner; box[0] = 16; sw = CU_TENSOR_MAP_SWIZZLE_NONE; break;
        case 2: strides[0] = (cuuint64_t)stride_bytes; box[0] = 64; dt = CU_TENSOR_MAP_DATA_TYPE_BFLOAT16; break;
        case 3: strides[0] = (cuuint64_t)inner; break;
        case 4: strides[0] = 128; box[0] = 32; dt = CU_TENSOR_MAP_DATA_TYPE_FLOAT32; break;
        case 5: strides[0] = 64; box[0] = 32; dt = CU_TENSOR_MAP_DATA_TYPE_BFLOAT16; sw = CU_TENSOR_MAP_SWIZZLE_64B; break;
        case 6: strides[0] = (cuuint64_t)inner; box[0] = 48; sw = CU_TENSOR_MAP_SWIZZLE_NONE; break;
        case 7: strides[0] = (cuuint64_t)inner; box[0] = 64; sw = CU_TENSOR_MAP_SWIZZLE_64B; break;
        default: return fail(MXFP6_ERR_BAD_ARG, "make_map: unknown kind %d", kind);
    }
    CUresult r = encode(out, dt, 2, const_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, sw,
                        CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS)
        return fail(MXFP6_ERR_CUDA, "cuTensorMapEncodeTiled(kind=%d rows=%lld inner=%lld box_rows=%d) failed with %d",
                    kind, (long long)rows, (long long)inner, box_rows, (int)r);
    t_maps->key[h] = mk; t_maps->map[h] = *out; t_maps->used[h] = true;
    return MXFP6_OK;
}

// ---------------------------------------------------------------------------------- operand formats
static bool fmt_valid(int f) { return f == MXFP6_E2M3 || f == MXFP6_E3M2 || f == MXFP8_E4M3 || f == MXFP8_E5M2; }
static bool fmt_is_fp8(int f) { return f == MXFP8_E4M3 || f == MXFP8_E5M2; }
static int fmt_row_bytes_per_128(int f) { return fmt_is_fp8(f) ? 128 : 96; }   // bytes of 128 elements in HBM
static uint32_t fmt_mma_code(int f) {      // operand format field of kind::mxf8f6f4
    return f == MXFP6_E2M3 ? kFmtE2M3 : f == MXFP6_E3M2 ? kFmtE3M2 : f == MXFP8_E4M3 ? 0u : 1u;
}

// ---------------------------------------------------------------------------------- GEMM dispatch
struct Plan {
    int bn; bool swap; bool streamk;
    bool pair;                  // CTA-pair kernel (256x256 tile per cluster of 2)
    int ctas;                   // CTAs per SM the kernel variant is built for (1 or 2)
    int p_tile, q_tile;         // rows of P / Q one tile covers (128 / bn unless a streamed operand's rows are dealt evenly to the CTAs)
    int tail_first, tail_split; // pair kernel: first tile of the last partial wave and the number of column slices its tiles are cut into
    int grid;
    int tiles_p, tiles_q;
    int ws_slots;
    size_t ws_counter_bytes, ws_bytes;
};

static int ceil_div(int64_t a, int64_t b) { return (int)((a + b - 1) / b); }

// Most output tiles a problem may have and still split tiles along K (bounds the counter region).
constexpr int64_t kMaxSplitTiles = 65536;

static Plan make_plan(int64_t M, int64_t N, int64_t K, int sm_count, bool allow_pair = true, bool plain = false,
                      bool even_rows_ok = true) {
    Plan p{};
    p.ctas = 1;
    const Options& o = options();
    const int kb = (int)(K / 128);
    const int fbn = o.force_bn, fswap = o.force_swap, fsk = o.force_sk, fpair = o.force_pair;
    // Skinny M: the weights are what is streamed.  Up to M = 32 the swapped form (weights on the 128-row side, K-split
    // work units over all SMs) is fastest.  Above that, whole unswapped 128 x 256 tiles stream 256 weight rows per
    // K-block and store C untransposed, which is faster as long as the tiles cover most SMs (measured at
    // N = 28672, K = 8192: M = 64 / 96 / 128 in 41.8 / 42.3 / 43.3 us against 45.7 / 52.6 / 53.4 us swapped;
    // M = 16 in 52.4 against 38.5 us).
    const int64_t t256n = ceil_div(N, 256);
    const double cover = (double)t256n / (double)((int64_t)ceil_div(t256n, sm_count) * sm_count);
    const bool wide_rows = M > 32 && M <= 128 && cover >= 0.6;
    if (M <= 128 && N > M && !plain && !wide_rows) {      // plain: whole tiles, C stored untransposed (several destinations)
        p.swap = true;
        p.bn = M <= 16 ? 16 : M <= 32 ? 32 : M <= 64 ? 64 : 128;
        // K-split work units balance the SMs
        p.streamk = (int64_t)ceil_div(N, 128) <= kMaxSplitTiles;
    } else {
        p.swap = false; p.streamk = false;
        const int64_t t256 = (int64_t)ceil_div(M, 128) * ceil_div(N, 256);
        p.bn = (N >= 256 && (t256 >= sm_count || wide_rows)) ? 256 : 128;
    }
    // one 256x256 tile per CTA pair as soon as that occupies at least half of the pairs (measured: 2048^3 with
    // 64 pair tiles runs in 11.6 us against 17 us with 128x128 tiles)
    p.pair = !p.swap && !wide_rows && N >= 256 &&
             (int64_t)ceil_div(M, 256) * ceil_div(N, 256) >= sm_count / 4;
    if (fbn) { p.bn = fbn; p.pair = false; }
    if (fpair >= 0) p.pair = fpair != 0;
    if (!allow_pair) p.pair = false;
    if (p.pair) { p.bn = 256; p.swap = false; p.streamk = false; }
    if (fswap >= 0 && !p.pair) p.swap = fswap != 0;
    if (fsk >= 0 && !p.pair) p.streamk = fsk != 0;
    if (plain) { p.swap = false; p.streamk = false; }
    {
        const int64_t t = (int64_t)ceil_div(p.swap ? N : M, 128) * ceil_div(p.swap ? M : N, p.bn);
        if (t > kMaxSplitTiles) p.streamk = false;
    }
    const int64_t prow = p.swap ? N : M, qrow = p.swap ? M : N;
    p.p_tile = p.pair ? 256 : 128;
    p.q_tile = p.bn;
    // Skinny M with many weight rows: instead of 128-row tiles split along K, the weight rows are dealt evenly to the
    // CTAs, each CTA runs the whole K loop over its own rows and stores its block of C itself -- no partial sums, no
    // arrival counters, every CTA streams the same number of bytes.  M <= 32: swapped form, two CTAs per SM (97 rows
    // each at N = 28672).  32 < M <= 128: unswapped 128 x 256 tiles whose column count is N / SMs rounded up to 8.
    const bool forced = fbn || fswap >= 0 || fsk >= 0 || fpair >= 0;
    if (even_rows_ok && o.decode_rows && !forced && !p.pair && !plain) {
        if (p.swap && p.bn <= 32) {
            const int64_t slots = 2 * (int64_t)sm_count;
            const int64_t waves = ceil_div(N, slots * 128);
            const int64_t rows = ceil_div(N, slots * waves);
            // (measured at K = 8192: 97 rows per CTA, N = 28672, 34.9 against 38.5 us for the K-split form; 49 rows per
            // CTA, N = 14336, 27.7 against 24.5 us: with few rows per CTA the K-split form's parallelism along K wins)
            if (rows >= 80) { p.streamk = false; p.ctas = 2; p.p_tile = (int)rows; }
        } else if (!p.swap && wide_rows && p.bn == 256) {
            const int64_t waves = ceil_div(N, (int64_t)sm_count * 256);
            const int64_t rows = (ceil_div(N, (int64_t)sm_count * waves) + 7) / 8 * 8;
            if (rows >= 128 && rows <= 256) {
                p.q_tile = (int)rows;
                p.p_tile = (int)((M + 7) / 8 * 8);      // the rows of A that exist: the box, and with it the stage, shrinks
            }
        }
    }
    p.tiles_p = ceil_div(prow, p.p_tile);
    p.tiles_q = ceil_div(qrow, p.q_tile);
    const int64_t tiles = (int64_t)p.tiles_p * p.tiles_q;
    p.tail_first = (int)tiles; p.tail_split = 1;
    if (p.pair) {
        const int64_t clusters = tiles < sm_count / 2 ? tiles : sm_count / 2;
        p.grid = (int)(2 * clusters);
        p.ws_slots = 0; p.ws_counter_bytes = 0; p.ws_bytes = 0;
        // The tiles left over after the last full wave occupy only some of the pairs for a whole tile's time.  When
        // they are at most half (a quarter) as many as the pairs, each is cut into 2 (4) column slices of 128 (64)
        // columns, which run side by side (4096^3: 256 tiles on 74 pairs = 3 waves + 34 tiles -> 68 slices).
        const int64_t left = tiles % clusters;
        if (o.tail_split && tiles > clusters && left > 0 && 2 * left <= clusters) {
            p.tail_split = 4 * left <= clusters ? 4 : 2;
            p.tail_first = (int)(tiles - left);
        }
    } else if (p.streamk) {
        const int64_t U = tiles * kb;
        int64_t g = U / 4; if (g < 1) g = 1;
        p.grid = (int)(g < sm_count ? g : sm_count);
        const int64_t chunk = U / p.grid;           // smallest number of K-blocks a CTA gets (>= 1)
        int64_t maxseg = (kb + chunk - 1) / chunk + 1;
        if (maxseg > p.grid) maxseg = p.grid;
        p.ws_slots = (int)maxseg;
        // The arrival counters always occupy the same fixed region at the start of the scratch buffer, so a
        // buffer that is reused for another shape never sees partial sums where it expects zeroed counters.
        p.ws_counter_bytes = (size_t)kMaxSplitTiles * 4;
        p.ws_bytes = p.ws_counter_bytes + (size_t)tiles * maxseg * (size_t)p.bn * 128 * 4;
    } else {
        const int64_t resident = (int64_t)sm_count * p.ctas;
        p.grid = (int)(tiles < resident ? tiles : resident);
        p.ws_slots = 0; p.ws_counter_bytes = 0; p.ws_bytes = 0;
    }
    return p;
}

// Where the [M,N] result goes: n copies (the first is local, the others may be peer GPUs' memory), each the
// first element of the block inside a row-major matrix with a row stride of ldc elements.
struct Dest {
    void* c[8];
    int n;
    int64_t ldc;
};

// optional completion flags per block of C (pair kernel; null = absent)
struct Signal {
    unsigned int* counter = nullptr;   // [blocks], cleared before every launch
    unsigned int* flag = nullptr;      // [blocks], raised to 1 by the CTA that completes a block
    int cols = 0;                      // 256-column tiles per block; a block is as many rows as one row group of the tile order
};

// optional fp32 epilogue vectors (null = absent)
struct Affine {
    const float* scale_m = nullptr;   // [M]
    const float* scale_n = nullptr;   // [N]
    const float* bias_n = nullptr;    // [N]
};

// Where split-tile scratch comes from.
enum WsMode : int { kWsOwn = 0,       // the library's per-device buffer, allocated on first need
                    kWsCaller = 1,    // the caller's buffer
                    kWsBuiltin = 2 }; // the buffer built into the library image (mxfp6_gemm_noalloc)

// The operand-dependent facts the kernel choice needs, and the choice itself: one place for every entry point.
static bool scales_by_tma(const void* sfa, const void* sfb, int64_t K) {
    return ((K / 32) % 16 == 0) && !((uintptr_t)sfa & 15) && !((uintptr_t)sfb & 15) && !options().no_sf_tma;
}
static bool dest_by_tma(const Dest& dst) {
    bool ok = (dst.ldc % 8) == 0;      // the pair kernel stores C by TMA: 16-byte aligned destinations and row stride
    for (int i = 0; i < dst.n; ++i) ok = ok && !((uintptr_t)dst.c[i] & 15);
    return ok;
}
static Plan plan_for(const void* sfa, const void* sfb, const Dest& dst, int64_t M, int64_t N, int64_t K, int sm_count,
                     bool requant = false) {
    // several destinations are written untransposed from whole tiles; a re-quantised result needs tiles that start on
    // multiples of 32 rows and columns
    (void)sfa; (void)sfb; (void)dst;
    return make_plan(M, N, K, sm_count, true, dst.n > 1, !requant);
}

// Everything a call passes in.  Two calls with equal keys launch the same kernel with the same arguments, so the
// launch recipe of the first is reused by the second.  (Zero-filled before use: compared bytewise.)
struct CallKey {
    const void *a, *sfa, *b, *sfb;
    void* c[8];
    int64_t ldc, M, N, K;
    void* ws; size_t ws_bytes;
    void *q_out, *q_scales;
    const float *scale_m, *scale_n, *bias_n;
    int n_dst, fmt_a, fmt_b, ws_mode, q_fmt, dev;
    unsigned flags, epoch;
    unsigned int *sig_counter, *sig_flag;
    int64_t sig_cols;
};

struct Recipe {
    CallKey key;
    bool valid = false;
    const void* func = nullptr;
    int grid = 0, threads = 0, smem = 0;
    bool pair = false, pdl = true;
    size_t counter_bytes = 0;    // built-in scratch: counters to clear before every launch
    void* counter_ptr = nullptr;
    CUtensorMap tp, tq, tq_tail, tsp, tsq, tc;
    CMaps cm;
    GemmParams P;
};

// A small per-thread table: no lock on the hit path.
constexpr int kRecipeSlots = 32;
struct RecipeCache {
    Recipe slot[kRecipeSlots];
    unsigned next = 0;
};
static thread_local std::unique_ptr<RecipeCache> t_cache;

static int launch_recipe(const Recipe& r, cudaStream_t st) {
    if (r.counter_bytes) CUDA_TRY(cudaMemsetAsync(r.counter_ptr, 0, r.counter_bytes, st));
    cudaLaunchConfig_t lc{};
    lc.gridDim = dim3((unsigned)r.grid, 1, 1);
    lc.blockDim = dim3((unsigned)r.threads, 1, 1);
    lc.dynamicSmemBytes = (size_t)r.smem;
    lc.stream = st;
    // Programmatic stream serialisation lets the next kernel of the stream begin its set-up (barriers, TMEM,
    // descriptor prefetch) before this one has drained; the kernels call griddepcontrol.wait before their first
    // global access.
    cudaLaunchAttribute attr{};
    attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr.val.programmaticStreamSerializationAllowed = 1;
    lc.attrs = &attr;
    lc.numAttrs = r.pdl ? 1 : 0;
    if (r.pair) {
        void* args[] = {(void*)&r.tp, (void*)&r.tq, (void*)&r.tq_tail, (void*)&r.tsp, (void*)&r.tsq, (void*)&r.cm, (void*)&r.P};
        CUDA_TRY(cudaLaunchKernelExC(&lc, r.func, args));
    } else {
        void* args[] = {(void*)&r.tp, (void*)&r.tq, (void*)&r.tsp, (void*)&r.tsq, (void*)&r.tc, (void*)&r.P};
        CUDA_TRY(cudaLaunchKernelExC(&lc, r.func, args));
    }
    return MXFP6_OK;
}

template <class Cfg>
static int bind_cfg(DeviceState& d, Recipe& r) {
    auto kern = mxfp6_gemm_kernel<Cfg>;
    r.func = (const void*)kern;
    r.threads = Cfg::THREADS;
    r.smem = Cfg::SMEM_ALLOC;
    return ensure_smem_attr(d, r.func, Cfg::SMEM_ALLOC);
}

// Library-owned scratch of at least `bytes`.  Buffers are never freed or moved: an earlier launch, or a CUDA graph
// captured earlier, may still hold the address it was given.  A larger request gets a new, larger buffer.
static int own_scratch(DeviceState& d, size_t bytes, cudaStream_t st, void** out) {
    std::lock_guard<std::mutex> lk(g_mu);
    if (d.ws_bytes < bytes) {
        cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
        if (cudaStreamIsCapturing(st, &cap) == cudaSuccess && cap != cudaStreamCaptureStatusNone)
            return fail(MXFP6_ERR_BAD_ARG,
                        "this shape needs %zu bytes of scratch and the library holds %zu: it cannot allocate while the stream is "
                        "being captured; call once before the capture, or pass scratch through mxfp6_gemm_ws", bytes, d.ws_bytes);
        size_t want = d.ws_bytes * 2 > bytes ? d.ws_bytes * 2 : bytes;
        if (want < (size_t)(8u << 20)) want = (size_t)(8u << 20);
        void* p = nullptr;
        if (cudaMalloc(&p, want) != cudaSuccess) {
            (void)cudaGetLastError();
            want = bytes;
            CUDA_TRY(cudaMalloc(&p, want));
        }
        CUDA_TRY(cudaMemset(p, 0, want));
        d.ws_all.emplace_back(p, want);
        d.ws = p;
        d.ws_bytes = want;
    }
    *out = d.ws;
    return MXFP6_OK;
}

static int gemm_impl(const void* a, const void* sfa, const void* b, const void* sfb, const Dest& dst, int64_t M, int64_t N,
                     int64_t K, int fmt_a, int fmt_b, void* ws, size_t ws_bytes, int ws_mode, void* stream,
                     unsigned flags = 0, void* q_out = nullptr, void* q_scales = nullptr, int q_fmt = -1,
                     const Affine& aff = Affine{}, const Signal& sig = Signal{}) {
    cudaStream_t st = (cudaStream_t)stream;
    // ---- the recipe of an identical earlier call
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess) { (void)cudaGetLastError(); dev = -1; }   // no usable device: the checks below still answer
    CallKey key;
    memset(&key, 0, sizeof key);
    key.a = a; key.sfa = sfa; key.b = b; key.sfb = sfb;
    if (dst.n >= 1 && dst.n <= 8) for (int i = 0; i < dst.n; ++i) key.c[i] = dst.c[i];
    key.ldc = dst.ldc; key.M = M; key.N = N; key.K = K;
    key.ws = ws; key.ws_bytes = ws_bytes;
    key.q_out = q_out; key.q_scales = q_scales;
    key.scale_m = aff.scale_m; key.scale_n = aff.scale_n; key.bias_n = aff.bias_n;
    key.n_dst = dst.n; key.fmt_a = fmt_a; key.fmt_b = fmt_b; key.ws_mode = ws_mode; key.q_fmt = q_fmt; key.dev = dev;
    key.flags = flags; key.epoch = g_opt_epoch.load(std::memory_order_acquire);
    key.sig_counter = sig.counter; key.sig_flag = sig.flag; key.sig_cols = sig.cols;
    if (!t_cache) t_cache.reset(new RecipeCache());      // a few tens of KB per calling thread
    for (int i = 0; i < kRecipeSlots && dev >= 0; ++i) {
        const Recipe& r = t_cache->slot[i];
        if (r.valid && !memcmp(&r.key, &key, sizeof key)) return launch_recipe(r, st);
    }

    // ---- first call of this kind: check, plan, build
    void* c = dst.c[0];
    if (M < 0 || N < 0 || K < 0) return fail(MXFP6_ERR_BAD_ARG, "negative dimension (M=%lld N=%lld K=%lld)", (long long)M, (long long)N, (long long)K);
    if (K % 128 != 0) return fail(MXFP6_ERR_BAD_ARG, "K=%lld must be a multiple of 128", (long long)K);
    if (!fmt_valid(fmt_a) || !fmt_valid(fmt_b))
        return fail(MXFP6_ERR_BAD_ARG, "format must be MXFP6_E2M3 (0), MXFP6_E3M2 (1), MXFP8_E4M3 (2) or MXFP8_E5M2 (3)");
    if (M > 0x7fffff00LL || N > 0x7fffff00LL || K > 0x7fffff00LL) return fail(MXFP6_ERR_BAD_ARG, "dimension too large");
    if (M == 0 || N == 0) return MXFP6_OK;
    if (!c) return fail(MXFP6_ERR_BAD_ARG, "null C");
    if (dst.n < 1 || dst.n > 8) return fail(MXFP6_ERR_BAD_ARG, "1 to 8 destinations, got %d", dst.n);
    if (dst.ldc < N) return fail(MXFP6_ERR_BAD_ARG, "ldc=%lld is smaller than N=%lld", (long long)dst.ldc, (long long)N);
    for (int i = 0; i < dst.n; ++i) {
        if (!dst.c[i]) return fail(MXFP6_ERR_BAD_ARG, "null C (destination %d)", i);
        if ((uintptr_t)dst.c[i] & 1) return fail(MXFP6_ERR_BAD_ARG, "C must be 2-byte aligned");
    }
    if (K == 0) {
        for (int i = 0; i < dst.n; ++i)
            CUDA_TRY(cudaMemset2DAsync(dst.c[i], (size_t)dst.ldc * 2, 0, (size_t)N * 2, (size_t)M, st));
        return MXFP6_OK;
    }
    if (!a || !b || !sfa || !sfb) return fail(MXFP6_ERR_BAD_ARG, "null operand pointer");
    if (((uintptr_t)a & (fmt_is_fp8(fmt_a) ? 15 : 31)) || ((uintptr_t)b & (fmt_is_fp8(fmt_b) ? 15 : 31)))
        return fail(MXFP6_ERR_BAD_ARG, "operands must be 32-byte aligned (fp6) / 16-byte aligned (fp8)");
    if (((uintptr_t)sfa & 3) || ((uintptr_t)sfb & 3)) return fail(MXFP6_ERR_BAD_ARG, "scale arrays must be 4-byte aligned");

    DeviceState* dp = nullptr;
    int rc = get_device_state(&dp);
    if (rc) return rc;
    DeviceState& d = *dp;
    const Options& o = options();
    const bool sf_tma = scales_by_tma(sfa, sfb, K);
    const Plan pl = plan_for(sfa, sfb, dst, M, N, K, d.sm_count, q_fmt >= 0);

    Recipe r;
    r.key = key;
    if (sig.flag) {
        if (!pl.pair || pl.ws_bytes || q_fmt >= 0 || dst.n != 1 || !dest_by_tma(dst) || options().c_plain || sig.cols < 1 || !sig.counter)
            return fail(MXFP6_ERR_BAD_ARG, "completion flags need the CTA-pair kernel with TMA stores of C (M > 128, N >= 256, "
                                           "16-byte aligned C and row stride) and one destination");
        r.counter_ptr = sig.counter;
        r.counter_bytes = (size_t)ceil_div(pl.tiles_p, options().group_p) * ceil_div(pl.tiles_q, sig.cols) * sizeof(unsigned int);
    }
    if (pl.ws_bytes) {
        if (ws_mode == kWsOwn) {
            if ((rc = own_scratch(d, pl.ws_bytes, st, &ws))) return rc;
        } else {
            if (!ws || ws_bytes < pl.ws_bytes) return fail(MXFP6_ERR_BAD_ARG, "workspace too small: need %zu bytes, got %zu", pl.ws_bytes, ws_bytes);
            if ((uintptr_t)ws & 255) return fail(MXFP6_ERR_BAD_ARG, "workspace must be 256-byte aligned");
            if (ws_mode == kWsBuiltin) {
                // that buffer keeps whatever the previous call left: the arrival counters of this call's tiles must be zero
                r.counter_ptr = ws;
                r.counter_bytes = (size_t)pl.tiles_p * pl.tiles_q * sizeof(unsigned int);
            }
        }
    }

    const void* pp = pl.swap ? b : a; const void* qp = pl.swap ? a : b;
    const void* sp = pl.swap ? sfb : sfa; const void* sq = pl.swap ? sfa : sfb;
    const int64_t prow = pl.swap ? N : M, qrow = pl.swap ? M : N;
    const int fp = pl.swap ? fmt_b : fmt_a, fq = pl.swap ? fmt_a : fmt_b;

    const int p_box = pl.pair ? 128 : pl.p_tile, q_box = pl.pair ? 128 : pl.q_tile;      // rows one operand load brings
    if ((rc = make_map(pp, prow, K, p_box, fmt_is_fp8(fp) ? 3 : 0, &r.tp))) return rc;
    if ((rc = make_map(qp, qrow, K, q_box, fmt_is_fp8(fq) ? 3 : 0, &r.tq))) return rc;
    r.tq_tail = r.tq;
    if (pl.pair && pl.tail_split > 1 && (rc = make_map(qp, qrow, K, 128 / pl.tail_split, fmt_is_fp8(fq) ? 3 : 0, &r.tq_tail))) return rc;
    if (sf_tma) {
        if ((rc = make_map(sp, prow, K / 32, p_box, 1, &r.tsp))) return rc;
        if ((rc = make_map(sq, qrow, K / 32, pl.q_tile, 1, &r.tsq))) return rc;   // pair kernel: all 256 Q rows per CTA
    } else {
        r.tsp = r.tp; r.tsq = r.tq;   // unused by the kernel in this mode
    }

    GemmParams& P = r.P;
    memset(&P, 0, sizeof P);
    P.p_rows = (int)prow; P.q_rows = (int)qrow;
    P.kblocks = (int)(K / 128);
    P.tiles_p = pl.tiles_p; P.tiles_q = pl.tiles_q;
    P.p_tile_rows = pl.p_tile; P.q_tile_rows = pl.q_tile;
    P.raw_tx_bytes = (p_box + pl.q_tile) * 16;
    if (!pl.pair && (pl.ctas == 2 || (pl.bn == 256 && !pl.swap && !pl.streamk))) {
        // Ring laid out at run time: a stage holds the tile's rows of P and of Q, each rounded up to 8 rows (whole
        // 1024-byte swizzle groups); as many stages as the bytes the kernel variant reserves for its ring allow
        // (90 KB for BN = 16 and 85 KB for BN = 32 with two CTAs per SM, 4 x 48 KB for BN = 256).
        const int ring = pl.ctas == 2 ? (pl.bn <= 16 ? 6 * (13312 + 2048) : 5 * (13312 + 4096)) : 4 * (16384 + 256 * 128);
        P.q_off = (pl.p_tile + 7) / 8 * 1024;
        P.stage_stride = P.q_off + (pl.q_tile + 7) / 8 * 1024;
        int ns = ring / P.stage_stride;
        if (ns > 8) ns = 8;
        if (o.decode_stages >= 2 && o.decode_stages <= ns) ns = o.decode_stages;
        P.n_stages = ns;
        // K-blocks requested back to back (a row's adjacent 96-byte pieces then reach DRAM together).  Unswapped skinny
        // tiles: two with a ring of 5 stages (M = 64 / 96 at N = 28672: +3 / +5 %), one with 4 (M = 128: two cost 6 %)
        P.load_batch = !pl.swap ? (ns >= 5 ? 2 : 1) : ns >= 8 ? 4 : ns >= 6 ? 3 : 2;
        if (o.decode_batch >= 1 && o.decode_batch <= ns / 2) P.load_batch = o.decode_batch;
        // the even-rows forms of skinny problems (tiles narrower than a box) rotate their K loops
        const bool even_rows = pl.ctas == 2 || pl.q_tile != pl.bn;
        P.k_rot = (even_rows && o.k_rot && (K / 128) % 4 == 0) ? 1 : 0;
    }
    P.ldc = (int)dst.ldc; P.c_rows = (int)M; P.c_cols = (int)N;
    // The instruction's N: the accumulator's width, or, where an unswapped tile is narrower than its accumulator (the
    // skinny forms: 200 of 256 columns at N = 28672), the tile's columns rounded up to 16, so that the tensor cores do
    // not multiply the stale rows behind the tile (a fifth of the MMA work and of its power there).
    uint32_t mma_n = (uint32_t)pl.bn;
    if (!pl.pair && !pl.swap && pl.q_tile < pl.bn) mma_n = (uint32_t)((pl.q_tile + 15) / 16 * 16);
    P.idesc = make_idesc_m(fmt_mma_code(fp), fmt_mma_code(fq), pl.pair ? 256u : 128u, mma_n);
    P.sf_tma = sf_tma ? 1 : 0;
    P.sf_ld = (int)(K / 32);
    // bytes a stage's two loads credit to its mbarrier: the global bytes of the boxes (fp6: 96 per 128 elements)
    P.stage_tx_bytes = p_box * fmt_row_bytes_per_128(fp) + q_box * fmt_row_bytes_per_128(fq);
    P.tail_first = pl.tail_first; P.tail_split = pl.tail_split;
    P.stage_tx_bytes_tail = p_box * fmt_row_bytes_per_128(fp) + (128 / pl.tail_split) * fmt_row_bytes_per_128(fq);
    P.sfp = (const uint8_t*)sp; P.sfq = (const uint8_t*)sq;
    P.c = (__nv_bfloat16*)c;
    for (int i = 1; i < dst.n; ++i) P.c_more[i - 1] = (__nv_bfloat16*)dst.c[i];
    P.ndst = dst.n;
    P.push_rotate = o.push_rotate;
    P.c_tma = (q_fmt >= 0 || (dest_by_tma(dst) && !o.c_plain)) ? 1 : 0;
    P.c_vec16 = (dest_by_tma(dst) && N % 8 == 0) ? 1 : 0;
    // (a TMA store writes 128 rows: tiles of fewer rows only where there is a single row of tiles, so that what lies
    // below the tile lies below C and is clipped)
    P.c_tma_last = (!pl.pair && !pl.swap && o.c_tma_last && q_fmt < 0 && dst.n == 1 && dest_by_tma(dst) &&
                    (pl.p_tile == 128 || pl.tiles_p == 1)) ? 1 : 0;
    P.q_out = (uint8_t*)q_out; P.q_scales = (uint8_t*)q_scales; P.q_fmt = q_fmt;
    P.q_ld = q_fmt < 0 ? 0 : (fmt_is_fp8(q_fmt) ? N : N * 3 / 4);
    P.ws_counter = (unsigned int*)ws;
    P.ws_partial = ws ? (float*)((uint8_t*)ws + pl.ws_counter_bytes) : nullptr;
    P.ws_slots = pl.ws_slots;
    P.status = d.status;
    P.wait_cycles = d.wait_cycles;
    r.pdl = o.pdl != 0;
    // Asking the first weights into L2 before the wait needs no promise and measured 1 % faster than requesting them for
    // real under the promise (and 3 % faster than the promise alone), so the promise is only used when the former is off.
    P.l2_ahead = (!pl.pair && o.pdl && o.l2_ahead > 0) ? o.l2_ahead : 0;
    P.early_p = (!pl.pair && (flags & MXFP6_FLAG_B_STATIC) && o.pdl && !P.l2_ahead) ? 1 : 0;
    P.group_p = o.group_p;   // 16 pair-tiles (4096 rows of A) share each tile of B
    P.l2_load = o.l2_load; P.l2_store = o.l2_store;
    P.sig_counter = sig.counter; P.sig_flag = sig.flag; P.sig_cols = sig.cols;
    // single-CTA kernel: an operand whose tiles are loaded once (the weights of a skinny problem) is marked to leave L2
    // first, one that other CTAs ask for again (always the activations of a skinny problem) to leave last
    P.l2_p = !o.l2_load ? 0 : pl.tiles_q == 1 ? 1 : 2;
    P.l2_q = !o.l2_load ? 0 : pl.tiles_p == 1 ? 1 : 2;
    P.scale_m = aff.scale_m; P.scale_n = aff.scale_n; P.bias_n = aff.bias_n;

    r.grid = pl.grid;
    r.pair = pl.pair;
    if (pl.pair) {
        r.func = (const void*)mxfp6_gemm_pair_kernel;
        r.threads = PairCfg::THREADS;
        r.smem = PairCfg::SMEM_ALLOC;
        if ((rc = ensure_smem_attr(d, r.func, PairCfg::SMEM_ALLOC))) return rc;
        for (int i = 0; i < 8; ++i) {
            if (i >= dst.n) { r.cm.m[i] = r.cm.m[0]; continue; }     // unused slots hold a valid map all the same
            if (q_fmt >= 0) {       // the pieces of a re-quantised result are code bytes, not bf16
                if ((rc = make_map(q_out, M, fmt_is_fp8(q_fmt) ? N : N * 3 / 4, 128, fmt_is_fp8(q_fmt) ? 7 : 6, &r.cm.m[i]))) return rc;
            } else if (!P.c_tma) {
                r.cm.m[i] = r.tp;       // plain stores: the slot only has to hold a valid map
            } else if ((rc = make_map(dst.c[i], M, N, 128, 2, &r.cm.m[i], dst.ldc * 2))) return rc;
        }
    } else {
        r.tc = r.tp;            // (the slot only has to hold a valid map when the kernel does not use it)
        if (P.c_tma_last && (rc = make_map(dst.c[0], M, N, 128, 2, &r.tc, dst.ldc * 2))) return rc;
        rc = -1;
#define MXFP6_CASE(BN_, SWAP_, SK_)                                                              \
        if (pl.ctas == 1 && pl.bn == BN_ && pl.swap == SWAP_ && pl.streamk == SK_) rc = bind_cfg<GemmCfg<BN_, SWAP_, SK_>>(d, r);
        if (pl.ctas == 2 && pl.bn == 16 && pl.swap && !pl.streamk) rc = bind_cfg<GemmCfg<16, true, false, 2>>(d, r);
        if (pl.ctas == 2 && pl.bn == 32 && pl.swap && !pl.streamk) rc = bind_cfg<GemmCfg<32, true, false, 2>>(d, r);
        MXFP6_CASE(256, false, false)
        MXFP6_CASE(128, false, false)
        MXFP6_CASE(256, false, true)
        MXFP6_CASE(128, false, true)
        MXFP6_CASE(16, true, true)
        MXFP6_CASE(32, true, true)
        MXFP6_CASE(64, true, true)
        MXFP6_CASE(128, true, true)
        MXFP6_CASE(16, true, false)
        MXFP6_CASE(32, true, false)
        MXFP6_CASE(64, true, false)
        MXFP6_CASE(128, true, false)
#undef MXFP6_CASE
        if (rc == -1) return fail(MXFP6_ERR_BAD_ARG, "no kernel for bn=%d swap=%d streamk=%d", pl.bn, (int)pl.swap, (int)pl.streamk);
        if (rc) return rc;
    }
    if ((rc = launch_recipe(r, st))) return rc;
    r.valid = true;
    t_cache->slot[t_cache->next++ % kRecipeSlots] = r;
    return MXFP6_OK;
}

// ---------------------------------------------------------------------------------- quantise / dequantise
template <typename T> __device__ __forceinline__ void load4(const T* p, float (&x)[4]);
template <> __device__ __forceinline__ void load4<float>(const float* p, float (&x)[4]) {
    float4 v = *reinterpret_cast<const float4*>(p);
    x[0] = v.x; x[1] = v.y; x[2] = v.z; x[3] = v.w;
}
template <> __device__ __forceinline__ void load4<__nv_bfloat16>(const __nv_bfloat16* p, float (&x)[4]) {
    uint2 v = *reinterpret_cast<const uint2*>(p);
    x[0] = __uint_as_float(v.x << 16); x[1] = __uint_as_float(v.x & 0xffff0000u);
    x[2] = __uint_as_float(v.y << 16); x[3] = __uint_as_float(v.y & 0xffff0000u);
}

// One thread per 4 consecutive elements; 8 adjacent lanes share a 32-element block.
template <typename T, int FMT>
__global__ void __launch_bounds__(256) quantize_kernel(const T* __restrict__ src, int64_t n_quads, uint32_t* __restrict__ packed_words,
                                                       uint8_t* __restrict__ scales) {
    constexpr int EMAX = FMT == MXFP6_E2M3 ? 2 : FMT == MXFP6_E3M2 ? 4 : FMT == MXFP8_E4M3 ? 8 : 15;
    constexpr bool FP8 = FMT == MXFP8_E4M3 || FMT == MXFP8_E5M2;
    const int lane = threadIdx.x & 31;
    // n_quads is a multiple of 8, so whole warps share the loop trip count up to the tail handled by `live`;
    // four iterations are unrolled so that each thread has four independent 16-byte loads in flight
#pragma unroll 4
    for (int64_t q0 = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) & ~31LL; q0 < n_quads; q0 += (int64_t)gridDim.x * blockDim.x) {
        const int64_t q = q0 + lane;
        const bool live = q < n_quads;
        float x[4] = {0.f, 0.f, 0.f, 0.f};
        if (live) load4<T>(src + q * 4, x);
        float amax = fmaxf(fmaxf(fabsf(x[0]), fabsf(x[1])), fmaxf(fabsf(x[2]), fabsf(x[3])));
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 4));
        // floor(log2(amax)) from the exponent field (fp32 subnormals: from the leading mantissa bit)
        const uint32_t u = __float_as_uint(amax);
        int fl = (int)((u >> 23) & 0xff) - 127;
        if (((u >> 23) & 0xff) == 0) fl = 31 - __clz(u & 0x7fffff) - 149;
        int sb = fl - EMAX + 127;
        sb = sb < 0 ? 0 : sb > 254 ? 254 : sb;
        if (!(amax > 0.f)) sb = 0;
        if (isinf(amax)) sb = 254;
        const int e = sb - 127;
        const int h = (-e) / 2;
        const float f1 = __uint_as_float((uint32_t)(h + 127) << 23), f2 = __uint_as_float((uint32_t)(-e - h + 127) << 23);
        // hardware conversion, two values per instruction
        const uint32_t w = cvt_quad<FMT>(x[0] * f1 * f2, x[1] * f1 * f2, x[2] * f1 * f2, x[3] * f1 * f2);
        if constexpr (FP8) {
            // one byte per element: this thread's 4 codes are one 32-bit word of the operand
            if (live) packed_words[q] = w;
        } else {
            // 4 lanes hold 4 x 24 bits = three 32-bit words of the packed stream
            const uint32_t wn = __shfl_down_sync(0xffffffffu, w, 1);
            const int i4 = lane & 3;
            if (live && i4 < 3) packed_words[(q >> 2) * 3 + i4] = (w >> (8 * i4)) | (wn << (24 - 8 * i4));
        }
        if (live && (lane & 7) == 0) scales[q >> 3] = (uint8_t)sb;
    }
}

template <int FMT>
__global__ void __launch_bounds__(256) dequantize_kernel(const uint8_t* __restrict__ packed, const uint8_t* __restrict__ scales,
                                                         int64_t n_quads, float* __restrict__ out) {
    constexpr bool FP8 = FMT == MXFP8_E4M3 || FMT == MXFP8_E5M2;
    constexpr int BITS = FP8 ? 8 : 6;
    constexpr int MB = (FMT == MXFP6_E2M3 || FMT == MXFP8_E4M3) ? 3 : 2;
    constexpr int EB = BITS - 1 - MB;
    constexpr int BIAS = FMT == MXFP6_E2M3 ? 1 : FMT == MXFP6_E3M2 ? 3 : FMT == MXFP8_E4M3 ? 7 : 15;
    for (int64_t q = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; q < n_quads; q += (int64_t)gridDim.x * blockDim.x) {
        uint32_t w;
        if constexpr (FP8) {
            w = *reinterpret_cast<const uint32_t*>(packed + q * 4);
        } else {
            const uint8_t* p = packed + q * 3;
            w = (uint32_t)p[0] | ((uint32_t)p[1] << 8) | ((uint32_t)p[2] << 16);
        }
        const uint32_t sbyte = scales[q >> 3];
        // 2^(sbyte-127) as fp32 (sbyte 0 -> 2^-127, an fp32 subnormal)
        const float s = sbyte == 255 ? __uint_as_float(0x7fc00000u) : sbyte == 0 ? __uint_as_float(0x00400000u) : __uint_as_float(sbyte << 23);
        float4 o;
        float* of = reinterpret_cast<float*>(&o);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const uint32_t c = (w >> (BITS * i)) & ((1u << BITS) - 1);
            const uint32_t e = (c >> MB) & ((1u << EB) - 1), m = c & ((1u << MB) - 1);
            float mag = e ? __uint_as_float(((e - BIAS + 127) << 23) | (m << (23 - MB)))
                          : (float)m * __uint_as_float((uint32_t)(1 - BIAS - MB + 127) << 23);
            if (FMT == MXFP8_E4M3 && e == 15 && m == 7) mag = __uint_as_float(0x7fc00000u);
            if (FMT == MXFP8_E5M2 && e == 31) mag = m ? __uint_as_float(0x7fc00000u) : __uint_as_float(0x7f800000u);
            of[i] = ((c >> (BITS - 1)) ? -mag : mag) * s;
        }
        *reinterpret_cast<float4*>(out + q * 4) = o;
    }
}

// ---------------------------------------------------------------------------------- diagnostics
__global__ void tma_dump_kernel(const __grid_constant__ CUtensorMap tm, int x, int y, uint32_t tx_bytes,
                                unsigned long long wait_cycles, uint8_t* out, int* status) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* gen = smem_raw + (base - smem_u32(smem_raw));
    const uint32_t bar = base + 16384;
    for (int i = threadIdx.x; i < 16384 / 4; i += blockDim.x) reinterpret_cast<uint32_t*>(gen)[i] = 0xEEEEEEEEu;
    if (threadIdx.x == 0) { mbar_init(bar, 1); fence_barrier_init(); }
    fence_proxy_async_smem();
    __syncthreads();
    if (threadIdx.x == 0) {
        mbar_arrive_expect_tx(bar, tx_bytes);
        tma_load_2d(base, &tm, bar, x, y);
        const long long t0 = clock64();
        bool done = false;
        while (!(done = mbar_try_wait(bar, 0))) {
            if ((unsigned long long)(clock64() - t0) > wait_cycles) break;
        }
        if (!done) atomicCAS(status, 0, 0x7f);
    }
    __syncthreads();
    for (int i = threadIdx.x; i < 16384; i += blockDim.x) out[i] = gen[i];
}

// One warp waits on an mbarrier that nothing ever arrives on, with the same bounded wait the GEMM kernels use:
// the wait must run out, record its status word and return.
__global__ void wait_probe_kernel(GemmParams P) {
    __shared__ uint64_t bar;
    __shared__ int abort_flag;
    if (threadIdx.x == 0) { mbar_init(smem_u32(&bar), 1); abort_flag = 0; fence_barrier_init(); }
    __syncthreads();
    wait_bar_warp(smem_u32(&bar), 0, &abort_flag, P, 9);
}

}  // namespace mxfp6

// ====================================================================================== C ABI
using namespace mxfp6;

extern "C" int mxfp6_version(void) { return 100; }

extern "C" const char* mxfp6_last_error(void) { return g_err.c_str(); }

extern "C" int mxfp6_gemm(const void* a, const void* sfa, const void* b, const void* sfb, void* c, int64_t M, int64_t N,
                          int64_t K, int fmt_a, int fmt_b, void* stream) {
    return gemm_impl(a, sfa, b, sfb, Dest{{c}, 1, N}, M, N, K, fmt_a, fmt_b, nullptr, 0, kWsOwn, stream);
}

extern "C" size_t mxfp6_gemm_workspace_bytes(int64_t M, int64_t N, int64_t K) {
    if (M <= 0 || N <= 0 || K <= 0 || K % 128) return 0;
    DeviceState* d = nullptr;
    if (get_device_state(&d)) return 0;
    return make_plan(M, N, K, d->sm_count).ws_bytes;
}

extern "C" int mxfp6_gemm_ws(const void* a, const void* sfa, const void* b, const void* sfb, void* c, int64_t M, int64_t N,
                             int64_t K, int fmt_a, int fmt_b, void* workspace, size_t workspace_bytes, void* stream) {
    return gemm_impl(a, sfa, b, sfb, Dest{{c}, 1, N}, M, N, K, fmt_a, fmt_b, workspace, workspace_bytes, kWsCaller, stream);
}

extern "C" int mxfp6_gemm_ex(const void* a, const void* sfa, const void* b, const void* sfb, void* c, int64_t M, int64_t N,
                             int64_t K, int fmt_a, int fmt_b, unsigned flags, void* stream) {
    if (flags & ~(unsigned)MXFP6_FLAG_B_STATIC) return fail(MXFP6_ERR_BAD_ARG, "unknown flag bits 0x%x", flags);
    return gemm_impl(a, sfa, b, sfb, Dest{{c}, 1, N}, M, N, K, fmt_a, fmt_b, nullptr, 0, kWsOwn, stream, flags);
}

extern "C" int mxfp6_gemm_requant(const void* a, const void* sfa, const void* b, const void* sfb, void* out, void* out_scales,
                                  int64_t M, int64_t N, int64_t K, int fmt_a, int fmt_b, int out_fmt, void* stream) {
    if (!fmt_valid(out_fmt)) return fail(MXFP6_ERR_BAD_ARG, "requant: bad output format %d", out_fmt);
    if (N % 64 != 0) return fail(MXFP6_ERR_BAD_ARG, "requant: N=%lld must be a multiple of 64", (long long)N);
    if (M > 0 && N > 0 && (!out || !out_scales)) return fail(MXFP6_ERR_BAD_ARG, "requant: null output");
    if ((uintptr_t)out & 15) return fail(MXFP6_ERR_BAD_ARG, "requant: output must be 16-byte aligned");
    if ((uintptr_t)out_scales & 1) return fail(MXFP6_ERR_BAD_ARG, "requant: out_scales must be 2-byte aligned");
    if (K == 0 && M > 0 && N > 0) {   // all-zero result: codes 0, scale byte 0
        CUDA_TRY(cudaMemsetAsync(out, 0, (size_t)M * (fmt_is_fp8(out_fmt) ? N : N * 3 / 4), (cudaStream_t)stream));
        CUDA_TRY(cudaMemsetAsync(out_scales, 0, (size_t)M * (N / 32), (cudaStream_t)stream));
        return MXFP6_OK;
    }
    return gemm_impl(a, sfa, b, sfb, Dest{{out}, 1, N}, M, N, K, fmt_a, fmt_b, nullptr, 0, kWsOwn, stream, 0, out, out_scales, out_fmt);
}

// C = bias broadcast along rows: what the scaled GEMM yields for K = 0
__global__ void bias_fill_kernel(__nv_bfloat16* c, const float* bias, int64_t M, int64_t N) {
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < M * N; i += (int64_t)gridDim.x * blockDim.x)
        c[i] = __float2bfloat16_rn(__fadd_rn(0.f, bias[i % N]));
}

extern "C" int mxfp6_gemm_scaled(const void* a, const void* sfa, const void* b, const void* sfb, void* c,
                                 const float* scale_a, const float* scale_b, const float* bias,
                                 int64_t M, int64_t N, int64_t K, int fmt_a, int fmt_b, void* stream) {
    if (((uintptr_t)scale_a & 3) || ((uintptr_t)scale_b & 15) || ((uintptr_t)bias & 15))
        return fail(MXFP6_ERR_BAD_ARG, "scaled: scale_a must be 4-byte aligned, scale_b and bias 16-byte aligned");
    if (K == 0 && bias && M > 0 && N > 0) {
        if (!c) return fail(MXFP6_ERR_BAD_ARG, "null C");
        DeviceState* dp = nullptr;
        int rc = get_device_state(&dp);
        if (rc) return rc;
        bias_fill_kernel<<<dp->sm_count * 4, 256, 0, (cudaStream_t)stream>>>((__nv_bfloat16*)c, bias, M, N);
        CUDA_TRY(cudaGetLastError());
        return MXFP6_OK;
    }
    Affine aff;
    aff.scale_m = scale_a; aff.scale_n = scale_b; aff.bias_n = bias;
    return gemm_impl(a, sfa, b, sfb, Dest{{c}, 1, N}, M, N, K, fmt_a, fmt_b, nullptr, 0, kWsOwn, stream, 0, nullptr, nullptr, -1, aff);
}

extern "C" int mxfp6_gemm_multi(const void* a, const void* sfa, const void* b, const void* sfb, void* const* c_dst,
                                int n_dst, int64_t ldc, int64_t M, int64_t N, int64_t K, int fmt_a, int fmt_b,
                                void* stream) {
    if (!c_dst) return fail(MXFP6_ERR_BAD_ARG, "null destination list");
    if (n_dst < 1 || n_dst > 8) return fail(MXFP6_ERR_BAD_ARG, "1 to 8 destinations, got %d", n_dst);
    Dest d{};
    for (int i = 0; i < n_dst; ++i) d.c[i] = c_dst[i];
    d.n = n_dst;
    d.ldc = ldc;
    return gemm_impl(a, sfa, b, sfb, d, M, N, K, fmt_a, fmt_b, nullptr, 0, kWsOwn, stream);
}

// ---------------------------------------------------------------------------------- GEMM with a copy-engine gather
// The column-parallel step with the exchange carried by the copy engines instead of stores from the SMs.  The kernel
// writes its block into the local C and raises one flag per finished block of C; for every peer, side streams wait for
// each flag with a stream memory operation (no kernel spins) and copy the block to the peer with a 2-D copy.  Whatever
// happens to the kernel, the launching stream sets every flag after it, so every wait ends.
typedef CUresult (*StreamWaitValue32Fn)(CUstream, CUdeviceptr, cuuint32_t, unsigned int);
static std::atomic<StreamWaitValue32Fn> g_wait_value{nullptr};
static int get_wait_value_fn(StreamWaitValue32Fn* out) {
    StreamWaitValue32Fn f = g_wait_value.load(std::memory_order_acquire);
    if (!f) {
        void* fn = nullptr;
        cudaDriverEntryPointQueryResult qres;
        CUDA_TRY(cudaGetDriverEntryPoint("cuStreamWaitValue32", &fn, cudaEnableDefault, &qres));
        if (!fn || qres != cudaDriverEntryPointSuccess) return fail(MXFP6_ERR_CUDA, "cuStreamWaitValue32 not available from the driver");
        f = (StreamWaitValue32Fn)fn;
        g_wait_value.store(f, std::memory_order_release);
    }
    *out = f;
    return MXFP6_OK;
}

struct GatherBlocks {
    int rows_per_block, cols_per_block, n_row_blocks, n_col_blocks;
    int total() const { return n_row_blocks * n_col_blocks; }
};
static GatherBlocks gather_blocks(int64_t M, int64_t N, int strip_tiles) {
    GatherBlocks g;
    const int gp = options().group_p;
    g.rows_per_block = gp * 256;
    g.cols_per_block = strip_tiles * 256;
    g.n_row_blocks = ceil_div(ceil_div(M, 256), gp);
    g.n_col_blocks = ceil_div(ceil_div(N, 256), strip_tiles);
    return g;
}

// events of the calling thread, one set per device (created once, never destroyed)
static thread_local std::map<int, std::vector<cudaEvent_t>> t_events;
static int thread_events(int dev, int n, cudaEvent_t** out) {
    std::vector<cudaEvent_t>& v = t_events[dev];
    while ((int)v.size() < n) {
        cudaEvent_t e;
        CUDA_TRY(cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
        v.push_back(e);
    }
    *out = v.data();
    return MXFP6_OK;
}

extern "C" size_t mxfp6_copy_gather_scratch_bytes(int64_t M, int64_t N, int strip_tiles) {
    if (M <= 0 || N <= 0 || strip_tiles < 1) return 0;
    return (size_t)gather_blocks(M, N, strip_tiles).total() * 2 * sizeof(unsigned int);
}

extern "C" int mxfp6_gemm_copy_gather(const void* a, const void* sfa, const void* b, const void* sfb, void* const* c_dst,
                                      int n_dst, int64_t ldc, int64_t M, int64_t N, int64_t K, int fmt_a, int fmt_b,
                                      void* scratch, size_t scratch_bytes, int strip_tiles, void* const* copy_streams,
                                      int n_copy_streams, void* stream) {
    if (!c_dst) return fail(MXFP6_ERR_BAD_ARG, "null destination list");
    if (n_dst < 1 || n_dst > 8) return fail(MXFP6_ERR_BAD_ARG, "1 to 8 destinations, got %d", n_dst);
    if (M <= 0 || N <= 0 || K <= 0) return fail(MXFP6_ERR_BAD_ARG, "empty problem (M=%lld N=%lld K=%lld)", (long long)M, (long long)N, (long long)K);
    if (strip_tiles < 1) return fail(MXFP6_ERR_BAD_ARG, "strip_tiles must be at least 1");
    const int peers = n_dst - 1;
    if (peers > 0 && (!copy_streams || n_copy_streams < peers || n_copy_streams % peers))
        return fail(MXFP6_ERR_BAD_ARG, "need a multiple of %d copy streams (one or more per peer), got %d", peers, n_copy_streams);
    for (int i = 0; i < n_dst; ++i)
        if (!c_dst[i]) return fail(MXFP6_ERR_BAD_ARG, "null C (destination %d)", i);
    const GatherBlocks g = gather_blocks(M, N, strip_tiles);
    const int nb = g.total();
    if (!scratch || scratch_bytes < (size_t)nb * 2 * sizeof(unsigned int) || ((uintptr_t)scratch & 3))
        return fail(MXFP6_ERR_BAD_ARG, "scratch too small: need %zu bytes (mxfp6_copy_gather_scratch_bytes), got %zu",
                    (size_t)nb * 2 * sizeof(unsigned int), scratch_bytes);
    cudaStream_t st = (cudaStream_t)stream;
    unsigned int* flags = (unsigned int*)scratch;
    unsigned int* counters = flags + nb;
    StreamWaitValue32Fn wait_value = nullptr;
    int rc = get_wait_value_fn(&wait_value);
    if (rc) return rc;
    int dev = 0;
    CUDA_TRY(cudaGetDevice(&dev));
    cudaEvent_t* ev = nullptr;
    const int spp = peers ? n_copy_streams / peers : 0;      // streams per peer
    if ((rc = thread_events(dev, 1 + n_copy_streams, &ev))) return rc;

    CUDA_TRY(cudaMemsetAsync(flags, 0, (size_t)nb * sizeof(unsigned int), st));
    CUDA_TRY(cudaEventRecord(ev[0], st));
    Signal sig;
    sig.counter = counters; sig.flag = flags; sig.cols = strip_tiles;
    Dest d{};
    d.c[0] = c_dst[0]; d.n = 1; d.ldc = ldc;
    rc = gemm_impl(a, sfa, b, sfb, d, M, N, K, fmt_a, fmt_b, nullptr, 0, kWsOwn, stream, 0, nullptr, nullptr, -1, Affine{}, sig);
    if (rc) return rc;                                        // nothing waits yet
    // every flag is set behind the kernel: a kernel that gave up (bounded waits) leaves no stream waiting
    CUDA_TRY(cudaMemsetAsync(flags, 0x01, (size_t)nb * sizeof(unsigned int), st));
    if (!peers) return MXFP6_OK;
    for (int i = 0; i < n_copy_streams; ++i) CUDA_TRY(cudaStreamWaitEvent((cudaStream_t)copy_streams[i], ev[0], 0));
    // blocks in the order the kernel finishes them: row groups one after the other, column strips within a group
    for (int rb = 0; rb < g.n_row_blocks; ++rb) {
        for (int cb = 0; cb < g.n_col_blocks; ++cb) {
            const int blk = rb * g.n_col_blocks + cb;
            const int64_t row0 = (int64_t)rb * g.rows_per_block, col0 = (int64_t)cb * g.cols_per_block;
            const size_t rows = (size_t)(M - row0 < g.rows_per_block ? M - row0 : g.rows_per_block);
            const size_t width = (size_t)(N - col0 < g.cols_per_block ? N - col0 : g.cols_per_block) * 2;
            const size_t off = ((size_t)row0 * (size_t)ldc + (size_t)col0) * 2;
            for (int p = 0; p < peers; ++p) {
                // peers take turns being first, so that the first copies of a block do not all leave for the same GPU
                const int peer = (p + blk) % peers;
                cudaStream_t cs = (cudaStream_t)copy_streams[peer * spp + blk % spp];
                const CUresult cr = wait_value((CUstream)cs, (CUdeviceptr)(uintptr_t)(flags + blk), 1u, CU_STREAM_WAIT_VALUE_GEQ);
                if (cr != CUDA_SUCCESS) return fail(MXFP6_ERR_CUDA, "cuStreamWaitValue32 failed with %d", (int)cr);
                CUDA_TRY(cudaMemcpy2DAsync((uint8_t*)c_dst[1 + peer] + off, (size_t)ldc * 2, (const uint8_t*)c_dst[0] + off,
                                           (size_t)ldc * 2, width, rows, cudaMemcpyDeviceToDevice, cs));
            }
        }
    }
    for (int i = 0; i < n_copy_streams; ++i) {
        CUDA_TRY(cudaEventRecord(ev[1 + i], (cudaStream_t)copy_streams[i]));
        CUDA_TRY(cudaStreamWaitEvent(st, ev[1 + i], 0));
    }
    return MXFP6_OK;
}

// ---------------------------------------------------------------------------------- GEMM without allocation
// Scratch that is part of the library image: every GPU that loads libmxfp6.so holds these 8 MiB until the
// process exits.  In host code `g_builtin_scratch` is only a handle for the symbol, not a device address;
// the address each device gave it is looked up once with cudaGetSymbolAddress and kept here.
constexpr size_t kBuiltinScratchBytes = (size_t)8 << 20;
static __device__ __align__(256) unsigned char g_builtin_scratch[kBuiltinScratchBytes];
static void* g_builtin_scratch_addr[64];

extern "C" int mxfp6_gemm_noalloc(const void* a, const void* sfa, const void* b, const void* sfb, void* c, int64_t M,
                                  int64_t N, int64_t K, int fmt_a, int fmt_b, void* stream) {
    // malformed or empty problems take the common path, which rejects or finishes them without any scratch
    if (M <= 0 || N <= 0 || K <= 0 || K % 128 != 0)
        return gemm_impl(a, sfa, b, sfb, Dest{{c}, 1, N}, M, N, K, fmt_a, fmt_b, nullptr, 0, kWsCaller, stream);
    DeviceState* d = nullptr;
    int dev = 0;
    int rc = get_device_state(&d, &dev);
    if (rc) return rc;
    void* scratch = nullptr;
    {
        std::lock_guard<std::mutex> lk(g_mu);
        if (!g_builtin_scratch_addr[dev]) {
            // set-up, once per device, with that device current
            void* p = nullptr;
            CUDA_TRY(cudaGetSymbolAddress(&p, g_builtin_scratch));
            g_builtin_scratch_addr[dev] = p;
        }
        scratch = g_builtin_scratch_addr[dev];
    }
    const Dest dst{{c}, 1, N};
    const Plan pl = plan_for(sfa, sfb, dst, M, N, K, d->sm_count);      // the plan the common path will make
    if (pl.ws_bytes > kBuiltinScratchBytes)
        return fail(MXFP6_ERR_BAD_ARG,
                    "mxfp6_gemm_noalloc: M=%lld N=%lld K=%lld needs %zu bytes of scratch but the built-in buffer holds %zu; "
                    "use mxfp6_gemm or mxfp6_gemm_ws for this shape",
                    (long long)M, (long long)N, (long long)K, pl.ws_bytes, kBuiltinScratchBytes);
    // (the common path clears the arrival counters of this call's tiles on the stream before every launch)
    return gemm_impl(a, sfa, b, sfb, dst, M, N, K, fmt_a, fmt_b, scratch, kBuiltinScratchBytes, kWsBuiltin, stream);
}

extern "C" int mxfp6_quantize(const void* src, int src_dtype, int64_t rows, int64_t K, int fmt, void* packed, void* scales,
                              void* stream) {
    if (rows < 0 || K < 0 || K % 32) return fail(MXFP6_ERR_BAD_ARG, "quantize: rows=%lld K=%lld (K must be a multiple of 32)", (long long)rows, (long long)K);
    if (!fmt_valid(fmt)) return fail(MXFP6_ERR_BAD_ARG, "quantize: bad format %d", fmt);
    if (src_dtype != 0 && src_dtype != 1) return fail(MXFP6_ERR_BAD_ARG, "quantize: src_dtype must be 0 (fp32) or 1 (bf16)");
    if (rows == 0 || K == 0) return MXFP6_OK;
    if (!src || !packed || !scales) return fail(MXFP6_ERR_BAD_ARG, "quantize: null pointer");
    if (((uintptr_t)src & (src_dtype == 0 ? 15 : 7)) || ((uintptr_t)packed & 3)) return fail(MXFP6_ERR_BAD_ARG, "quantize: misaligned pointer");
    DeviceState* d = nullptr;
    int rc = get_device_state(&d);
    if (rc) return rc;
    const int64_t nq = rows * K / 4;
    int64_t blocks = (nq + 255) / 256;
    const int64_t cap = (int64_t)d->sm_count * 16;
    if (blocks > cap) blocks = cap;
    cudaStream_t st = (cudaStream_t)stream;
    // Two kernels: the streaming kernel of quantize_kernel.cuh when the pointers allow bulk copies (16-byte aligned
    // source, codes and scales), else the plain-load kernel with one thread per 4 elements.  MXFP6_QUANT_PATH=quad
    // forces the latter (for tests).  Measured on 8192 x 8192: fp32 source 55 us against 74 us, bf16 38 against 73 us.
    const int64_t nblk = rows * K / 32;
    const bool tma_ok = !((uintptr_t)src & 15) && !((uintptr_t)packed & 15) && !((uintptr_t)scales & 15) && nblk < 0x7fffff00LL;
    const int path = (tma_ok && !options().quant_quad) ? 2 : 0;
    if (path == 2) {
        CUtensorMap tm;
        if ((rc = make_map(src, nblk, 32, 128, src_dtype == 0 ? 4 : 5, &tm))) return rc;
        const int64_t n_tiles = (nblk + 127) / 128;
        const int64_t max_grid = (int64_t)d->sm_count * (src_dtype == 0 ? 4 : 7);      // QuantCfg::CTAS_PER_SM resident CTAs per SM
        const unsigned grid = (unsigned)(n_tiles < max_grid ? n_tiles : max_grid);
#define QT(T, F)                                                                                                     \
        do {                                                                                                         \
            auto kern = quantize_tma_kernel<T, F>;                                                                   \
            if ((rc = ensure_smem_attr(*d, (const void*)kern, QuantCfg<T, F>::SMEM_ALLOC))) return rc;                \
            cudaLaunchAttribute attr{};                                                                              \
            cudaLaunchConfig_t lc{};                                                                                 \
            lc.gridDim = dim3(grid, 1, 1);                                                                           \
            lc.blockDim = dim3(QuantCfg<T, F>::THREADS, 1, 1);                                                       \
            lc.dynamicSmemBytes = QuantCfg<T, F>::SMEM_ALLOC;                                                        \
            lc.stream = st;                                                                                          \
            attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;                                            \
            attr.val.programmaticStreamSerializationAllowed = 1;                                                     \
            lc.attrs = &attr;                                                                                        \
            lc.numAttrs = options().pdl ? 1 : 0;                                                                     \
            CUDA_TRY(cudaLaunchKernelEx(&lc, kern, tm, (long long)nblk, (uint8_t*)packed, (uint8_t*)scales, d->status, d->wait_cycles)); \
        } while (0)
        if (src_dtype == 0) {
            if (fmt == MXFP6_E2M3) QT(float, MXFP6_E2M3); else if (fmt == MXFP6_E3M2) QT(float, MXFP6_E3M2);
            else if (fmt == MXFP8_E4M3) QT(float, MXFP8_E4M3); else QT(float, MXFP8_E5M2);
        } else {
            if (fmt == MXFP6_E2M3) QT(__nv_bfloat16, MXFP6_E2M3); else if (fmt == MXFP6_E3M2) QT(__nv_bfloat16, MXFP6_E3M2);
            else if (fmt == MXFP8_E4M3) QT(__nv_bfloat16, MXFP8_E4M3); else QT(__nv_bfloat16, MXFP8_E5M2);
        }
#undef QT
        CUDA_TRY(cudaGetLastError());
        return MXFP6_OK;
    }
#define QK(T, F) quantize_kernel<T, F><<<(unsigned)blocks, 256, 0, st>>>((const T*)src, nq, (uint32_t*)packed, (uint8_t*)scales)
    if (src_dtype == 0) {
        if (fmt == MXFP6_E2M3) QK(float, MXFP6_E2M3); else if (fmt == MXFP6_E3M2) QK(float, MXFP6_E3M2);
        else if (fmt == MXFP8_E4M3) QK(float, MXFP8_E4M3); else QK(float, MXFP8_E5M2);
    } else {
        if (fmt == MXFP6_E2M3) QK(__nv_bfloat16, MXFP6_E2M3); else if (fmt == MXFP6_E3M2) QK(__nv_bfloat16, MXFP6_E3M2);
        else if (fmt == MXFP8_E4M3) QK(__nv_bfloat16, MXFP8_E4M3); else QK(__nv_bfloat16, MXFP8_E5M2);
    }
#undef QK
    CUDA_TRY(cudaGetLastError());
    return MXFP6_OK;
}

extern "C" int mxfp6_dequantize(const void* packed, const void* scales, int64_t rows, int64_t K, int fmt, void* out_f32,
                                void* stream) {
    if (rows < 0 || K < 0 || K % 32) return fail(MXFP6_ERR_BAD_ARG, "dequantize: rows=%lld K=%lld (K must be a multiple of 32)", (long long)rows, (long long)K);
    if (!fmt_valid(fmt)) return fail(MXFP6_ERR_BAD_ARG, "dequantize: bad format %d", fmt);
    if (rows == 0 || K == 0) return MXFP6_OK;
    if (!packed || !scales || !out_f32) return fail(MXFP6_ERR_BAD_ARG, "dequantize: null pointer");
    if ((uintptr_t)out_f32 & 15) return fail(MXFP6_ERR_BAD_ARG, "dequantize: output must be 16-byte aligned");
    DeviceState* d = nullptr;
    int rc = get_device_state(&d);
    if (rc) return rc;
    const int64_t nq = rows * K / 4;
    int64_t blocks = (nq + 255) / 256;
    const int64_t cap = (int64_t)d->sm_count * 16;
    if (blocks > cap) blocks = cap;
    cudaStream_t st = (cudaStream_t)stream;
#define DQ(F) dequantize_kernel<F><<<(unsigned)blocks, 256, 0, st>>>((const uint8_t*)packed, (const uint8_t*)scales, nq, (float*)out_f32)
    if (fmt == MXFP6_E2M3) DQ(MXFP6_E2M3); else if (fmt == MXFP6_E3M2) DQ(MXFP6_E3M2);
    else if (fmt == MXFP8_E4M3) DQ(MXFP8_E4M3); else DQ(MXFP8_E5M2);
#undef DQ
    CUDA_TRY(cudaGetLastError());
    return MXFP6_OK;
}

extern "C" int mxfp6_device_status(int* status_out) {
    DeviceState* d = nullptr;
    int rc = get_device_state(&d);
    if (rc) return rc;
    CUDA_TRY(cudaDeviceSynchronize());
    int h[4] = {0, 0, 0, 0};
    CUDA_TRY(cudaMemcpy(h, d->status, sizeof h, cudaMemcpyDeviceToHost));
    if (status_out) *status_out = h[0];
    if (h[0] != 0) {
        CUDA_TRY(cudaMemset(d->status, 0, sizeof h));
        // arrival counters of split tiles may be left non-zero by an aborted launch
        std::lock_guard<std::mutex> lk(g_mu);
        for (auto& w : d->ws_all) CUDA_TRY(cudaMemset(w.first, 0, w.second));
        return fail(MXFP6_ERR_DEVICE_WAIT, "a bounded wait ran out on the device: role %d, CTA %d", h[0] & 0xff, h[0] >> 8);
    }
    return MXFP6_OK;
}

extern "C" int mxfp6_debug_wait_timeout(int budget_us, void* stream) {
    if (budget_us < 1 || budget_us > 100000) return fail(MXFP6_ERR_BAD_ARG, "wait_timeout: budget must be 1..100000 us");
    DeviceState* d = nullptr;
    int rc = get_device_state(&d);
    if (rc) return rc;
    GemmParams P{};
    P.status = d->status;
    P.wait_cycles = d->wait_cycles / 2000000ull * (unsigned long long)budget_us;   // wait_cycles covers 2 s by default
    if (P.wait_cycles < 1000) P.wait_cycles = 1000;
    wait_probe_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(P);
    CUDA_TRY(cudaGetLastError());
    return MXFP6_OK;
}

extern "C" int mxfp6_debug_option(const char* name, const char* value) {
    if (!name) return fail(MXFP6_ERR_BAD_ARG, "debug_option: null name");
    (void)options();                      // the environment is read first, once
    std::lock_guard<std::mutex> lk(g_mu);
    if (!set_option(name, value)) return fail(MXFP6_ERR_BAD_ARG, "debug_option: unknown option %s", name);
    g_opt_epoch.fetch_add(1, std::memory_order_acq_rel);      // launch recipes built under the old values are not reused
    return MXFP6_OK;
}

extern "C" int mxfp6_debug_plan(int64_t M, int64_t N, int64_t K, int sm_count, int n_dst, int requant, int* out12) {
    if (!out12 || M <= 0 || N <= 0 || K <= 0 || K % 128 || sm_count < 2 || n_dst < 1 || n_dst > 8)
        return fail(MXFP6_ERR_BAD_ARG, "debug_plan: bad argument");
    const Plan p = make_plan(M, N, K, sm_count, true, n_dst > 1, !requant);
    const int v[12] = {p.bn, p.swap, p.streamk, p.pair, p.ctas, p.p_tile, p.q_tile, p.tiles_p, p.tiles_q, p.grid,
                       p.tail_first, p.tail_split};
    memcpy(out12, v, sizeof v);
    return MXFP6_OK;
}

extern "C" int mxfp6_debug_tma_dump(const void* packed, int64_t rows, int64_t K, int64_t row0, int64_t k0, void* out16k,
                                    void* stream) {
    if (!packed || !out16k || K <= 0 || K % 128 || k0 % 128 || rows <= 0) return fail(MXFP6_ERR_BAD_ARG, "tma_dump: bad argument");
    if ((uintptr_t)packed & 31) return fail(MXFP6_ERR_BAD_ARG, "tma_dump: operand must be 32-byte aligned");
    DeviceState* d = nullptr;
    int rc = get_device_state(&d);
    if (rc) return rc;
    CUtensorMap tm;
    if ((rc = make_map(packed, rows, K, 128, 0, &tm))) return rc;
    static bool attr = false;
    if (!attr) { CUDA_TRY(cudaFuncSetAttribute(tma_dump_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 16384 + 2048)); attr = true; }
    const uint32_t tx = 128u * 96u;     // the bytes the box occupies in global memory: 96 per 128-element row
    tma_dump_kernel<<<1, 128, 16384 + 2048, (cudaStream_t)stream>>>(tm, (int)k0, (int)row0, tx, d->wait_cycles / 20, (uint8_t*)out16k, d->status);
    CUDA_TRY(cudaGetLastError());
    return MXFP6_OK;
}
