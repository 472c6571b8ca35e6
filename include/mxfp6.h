/*
 * mxfp6.h -- C ABI of the B200 (sm_100a) MX-FP6 GEMM path.
 *
 *   C[M,N] (bf16) = A[M,K] * B[N,K]^T
 *
 * A and B are packed MX-FP6: 6-bit codes (E2M3 or E3M2), four values per three bytes, dense
 * little-endian along K (element i of a row occupies bits [6i, 6i+6) of the row's byte string,
 * row stride 3K/4 bytes), with one E8M0 scale byte (value 2^(x-127)) per 32 elements along K,
 * row-major [rows, K/32].  Accumulation is fp32, the output is rounded once to bf16 (RNE).
 *
 * Conventions shared by every entry point
 *   - all pointers are DEVICE pointers unless a comment says otherwise; the caller owns every
 *     buffer, the library keeps no pointer after a call returns;
 *   - `stream` is a cudaStream_t passed as void* (NULL = the legacy default stream); calls are
 *     asynchronous on that stream and do not synchronise;
 *   - the return value is 0 on success, a MXFP6_ERR_* code otherwise; mxfp6_last_error() gives
 *     the message of the calling thread's last failure;
 *   - the first call on a device (and the first call of a kernel variant) does one-time set-up (attribute
 *     calls, a memset, for split shapes a cudaMalloc): make it before any stream capture.  Later calls
 *     with the same pointers, sizes and formats reuse the launch recipe (tensor maps, kernel choice) of the first;
 *   - the test hooks (MXFP6_FORCE_CFG and the like) are read from the environment once, when the library is
 *     first used; afterwards only mxfp6_debug_option changes them;
 *   - preconditions: K % 128 == 0; packed operand pointers 32-byte aligned; C 2-byte aligned
 *     (16-byte aligned C with N % 8 == 0 takes the vector store path); M, N >= 0.
 *
 * Each declaration names the interface of the reference (benenzhu/HipKittensP) it stands in for.
 */
#ifndef MXFP6_H_
#define MXFP6_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define MXFP6_E2M3 0
#define MXFP6_E3M2 1
/* MX-FP8 operands run through the same instruction (kind::mxf8f6f4) and the same entry points: one byte per
 * element, row-major [rows, K], 16-byte aligned, same E8M0 scale per 32 elements.  A and B may differ in format.
 * (The reference's main-branch GEMMs are fp8: kernels/gemm/fp8fp32/FP8_8wave/8_wave.cu.) */
#define MXFP8_E4M3 2
#define MXFP8_E5M2 3

#define MXFP6_OK 0
#define MXFP6_ERR_BAD_ARG 1      /* shape / alignment / format / null pointer */
#define MXFP6_ERR_CUDA 2         /* a CUDA runtime or driver call failed */
#define MXFP6_ERR_DEVICE_WAIT 3  /* a bounded wait inside a kernel ran out (see mxfp6_device_status) */
#define MXFP6_ERR_UNSUPPORTED 4  /* not an sm_100 device */

/* Library version, major*10000 + minor*100 + patch.  (No counterpart in the reference.) */
int mxfp6_version(void);

/* Message of the calling thread's last failing call ("" if none).  Stands in for the reference's
 * CHECK_CUDA_ERROR printing (include/pyutils/util.cuh:7-19), as a queryable string. */
const char* mxfp6_last_error(void);

/*
 * The GEMM.  Replaces the launch made by dispatch_micro(micro_globals)
 * (kernels/gemm/bf16fp32/256_256_64_32_with16x32.cpp:383-387) with the operand set of
 * micro_globals (:47-58) extended by the two scale tensors in the argument order of the
 * reference's scale-taking kernel (kernels/torch_scaled/scaled_matmul.cu:17-18).
 *   a   [M, 3K/4] u8 (fp6) or [M, K] u8 (fp8)   sfa [M, K/32] u8    fmt_a one of the four format codes
 *   b   [N, 3K/4] u8 (fp6) or [N, K] u8 (fp8)   sfb [N, K/32] u8    fmt_b likewise
 *   c   [M, N] bf16, written in place
 * Shapes that split output tiles along K use a per-device scratch buffer that the library
 * allocates on first need (cudaMalloc) and keeps; concurrent calls on different streams of one
 * device must use mxfp6_gemm_ws with their own scratch instead.  A scratch buffer is never freed or
 * moved once a launch has been given it (a CUDA graph captured earlier keeps replaying into it): a shape
 * that needs more gets an additional, larger buffer.  That allocation cannot happen while the stream is
 * being captured; the call then fails with MXFP6_ERR_BAD_ARG and says so -- run the shape once before
 * the capture, or use mxfp6_gemm_ws.
 */
int mxfp6_gemm(const void* a, const void* sfa, const void* b, const void* sfb, void* c,
               int64_t M, int64_t N, int64_t K, int fmt_a, int fmt_b, void* stream);

/*
 * mxfp6_gemm with option flags.  MXFP6_FLAG_B_STATIC promises that B and its scales are not written by the work
 * queued on the stream directly before this call (weights of a layer): the single-CTA kernels may then request B
 * while the preceding kernel is still finishing (programmatic dependent launch), and only the reads of A and all
 * writes wait for it.  Without the flag nothing is read into the kernel before the preceding kernel has completed;
 * what every call does while it waits is to ask the first weight tiles into L2, which consumes nothing and sees
 * later writes through the same cache.  That measured faster than the early requests, so in the default
 * configuration the flag changes nothing; it takes effect when MXFP6_L2_AHEAD is switched off.  (No counterpart in
 * the reference.)
 */
#define MXFP6_FLAG_B_STATIC 1u
int mxfp6_gemm_ex(const void* a, const void* sfa, const void* b, const void* sfb, void* c,
                  int64_t M, int64_t N, int64_t K, int fmt_a, int fmt_b, unsigned flags, void* stream);

/*
 * The GEMM with its result handed to the next layer already quantised: instead of bf16 C the epilogue writes
 * C as an MX operand, blocks of 32 along N (the next layer's K): out [M, 3N/4] (fp6) or [M, N] (fp8) bytes and
 * out_scales [M, N/32] E8M0 bytes, quantised from the fp32 accumulators with the rule of mxfp6_quantize
 * (so a 2-byte round trip of C through HBM and a quantiser launch disappear).  N % 64 == 0, out 16-byte
 * aligned, out_scales 2-byte aligned (two scale bytes are stored at a time).  (No counterpart in the reference; the nearest is the epilogue scaling of
 * kernels/torch_scaled/scaled_matmul.cu:253-265.)
 */
int mxfp6_gemm_requant(const void* a, const void* sfa, const void* b, const void* sfb, void* out, void* out_scales,
                       int64_t M, int64_t N, int64_t K, int fmt_a, int fmt_b, int out_fmt, void* stream);

/*
 * The GEMM with the per-row / per-column fp32 scaling of the reference's scale-taking kernel and an optional bias,
 * applied to the finished fp32 sum before the single rounding to bf16:
 *     C[m,n] = bf16( (acc[m,n] * scale_b[n]) * scale_a[m] + bias[n] )
 * three separate fp32 roundings in this order (no fused multiply-add).  scale_a [M], scale_b [N] and bias [N] are
 * fp32 device vectors; any of them may be NULL (factor 1 / addend 0); scale_b and bias 16-byte aligned.  These
 * per-tensor-row factors come on top of the MX block scales, which act inside the MMA.  Stands in for the
 * epilogue of kernels/torch_scaled/scaled_matmul.cu:253-265 (mul_col by scale_b, then mul_row by scale_a; argument
 * order of :17-18); the bias has no counterpart there.
 */
int mxfp6_gemm_scaled(const void* a, const void* sfa, const void* b, const void* sfb, void* c,
                      const float* scale_a, const float* scale_b, const float* bias,
                      int64_t M, int64_t N, int64_t K, int fmt_a, int fmt_b, void* stream);

/* Scratch bytes mxfp6_gemm_ws needs for this shape on the current device (0 if none). */
size_t mxfp6_gemm_workspace_bytes(int64_t M, int64_t N, int64_t K);

/* Same as mxfp6_gemm with caller-provided scratch (256-byte aligned, zero-filled once before its
 * first use; the kernel leaves it zeroed where it must be).  (No counterpart in the reference,
 * which never splits tiles.) */
int mxfp6_gemm_ws(const void* a, const void* sfa, const void* b, const void* sfb, void* c,
                  int64_t M, int64_t N, int64_t K, int fmt_a, int fmt_b,
                  void* workspace, size_t workspace_bytes, void* stream);

/*
 * The GEMM with its [M,N] result written to n_dst (1..8) destinations at once: c_dst[i] points at the first
 * element of the block inside a row-major bf16 matrix whose row stride is ldc elements (ldc >= N), so a
 * column-parallel shard can place its block in the right column window of the full C.  Destination 0 is
 * local; the others may be peer GPUs' memory mapped into this process (CUDA IPC / symmetric memory): the
 * epilogue then pushes every finished tile over NVLink while later tiles are still being computed, which is
 * the gather of the sharded configuration fused into the GEMM.  With n_dst > 1 tiles are never split along K
 * and C is never stored transposed.  The caller orders the peers' later reads after this call (a cross-GPU
 * barrier on the stream).  Multi-GPU form of dispatch_micro in distributed-kernels/bf16_gemm/kernel.cpp:253-265,
 * which stores through iris_ctx.store(ptr, val, rank) (:58-59).
 */
int mxfp6_gemm_multi(const void* a, const void* sfa, const void* b, const void* sfb, void* const* c_dst,
                     int n_dst, int64_t ldc, int64_t M, int64_t N, int64_t K, int fmt_a, int fmt_b,
                     void* stream);

/*
 * The same multi-destination GEMM with the exchange carried by the GPU's copy engines instead of stores from the
 * SMs (on this fabric copy engines move an all-to-all of C windows at about 750 GB/s per GPU when each window is one
 * copy, stores issued by SMs at about 600; cut into blocks that can follow the GEMM the copies lose that advantage,
 * and they compete with the GEMM for HBM: a step of 16384 x 57344 x 8192 on 4 GPUs takes 3.3 ms this way against 2.3 ms
 * with mxfp6_gemm_multi, so this form is an alternative for callers that want the SMs free of the exchange, not a
 * faster one).  The kernel writes its [M,N] block to c_dst[0] only and raises one flag per finished block of C
 * (16 x 256 rows by strip_tiles x 256 columns; blocks finish in row-major order of this grid).  For every peer
 * destination c_dst[1..] the call queues, on the caller's copy streams, one stream memory operation per block that
 * waits for the block's flag, followed by a 2-D copy of the block from c_dst[0] to the peer; no kernel waits for
 * another.  `stream` itself sets every flag behind the kernel, so the copy streams drain even when the kernel gave up,
 * and finally waits for all copy streams: work queued on `stream` after the call sees all copies done.
 * copy_streams: a multiple of (n_dst - 1) streams of the same device, consecutive groups belonging to consecutive
 * peers.  Measured on 4 GPUs: the copy engines are at their best with few large copies (one copy of the whole window per
 * peer 737 GB/s, 4 row blocks 708, 16 row blocks 605, 4 x 7 blocks 579), and several copies in flight to the same peer
 * make it worse (16 blocks on two streams per peer 449), so: one stream per peer and strip_tiles large.  scratch: device memory of at least
 * mxfp6_copy_gather_scratch_bytes(M, N, strip_tiles) bytes, 4-byte aligned, owned by this call until `stream` has
 * passed it.  Needs the CTA-pair kernel with TMA stores of C (M > 128, N >= 256, 16-byte aligned destinations and
 * row stride); other problems are refused with MXFP6_ERR_BAD_ARG.  Not capturable into a CUDA graph.  Stands where
 * mxfp6_gemm_multi stands (distributed-kernels/bf16_gemm/kernel.cpp:253-265); the reference has no copy-engine path.
 */
size_t mxfp6_copy_gather_scratch_bytes(int64_t M, int64_t N, int strip_tiles);
int mxfp6_gemm_copy_gather(const void* a, const void* sfa, const void* b, const void* sfb, void* const* c_dst,
                           int n_dst, int64_t ldc, int64_t M, int64_t N, int64_t K, int fmt_a, int fmt_b,
                           void* scratch, size_t scratch_bytes, int strip_tiles, void* const* copy_streams,
                           int n_copy_streams, void* stream);

/*
 * The same GEMM for hosts that must not allocate device memory while they run: servers that hand all of the
 * GPU's memory to their own pool at start-up, control loops with a latency bound (cudaMalloc may synchronise
 * the device, and may fail when memory is tight), or plug-ins whose host forbids allocation in the call path.
 * Shapes that split output tiles along K take their scratch from an 8 MiB buffer built into the library image
 * (held by every GPU that loads the library until the process exits) instead of cudaMalloc.  A shape that
 * would need more is refused with MXFP6_ERR_BAD_ARG and a message that names both sizes; shapes that need no
 * scratch are never refused.  This function calls neither cudaMalloc nor cudaFree nor any allocating
 * library routine.  The first call on each device looks up the buffer's address and initialises the
 * per-device state; make that first call with the device current and before any stream capture begins.
 * All calls on a device share the one buffer: each call clears the counters it is about to use, on its
 * stream, so the contents left by the previous call do not matter, but two calls that overlap on the GPU
 * (different streams) would race on it -- serialise them or use mxfp6_gemm_ws with separate scratch.
 * (No counterpart in the reference, which neither splits tiles nor allocates.)
 */
int mxfp6_gemm_noalloc(const void* a, const void* sfa, const void* b, const void* sfb, void* c,
                       int64_t M, int64_t N, int64_t K, int fmt_a, int fmt_b, void* stream);

/*
 * Block quantiser: src [rows, K] (src_dtype 0 = fp32, 1 = bf16), K % 32 == 0  ->
 * packed [rows, 3K/4] (fp6) or [rows, K] (fp8) + scales [rows, K/32].  Scale exponent = floor(log2(amax)) - 2
 * (E2M3), - 4 (E3M2), - 8 (E4M3) or - 15 (E5M2); elements rounded to nearest even and saturated.  The step in front of the GEMM; the
 * reference's fp8 harness does it on the host (kernels/gemm/fp8fp32/FP8_8wave/8_wave.cu:258-268).
 */
int mxfp6_quantize(const void* src, int src_dtype, int64_t rows, int64_t K, int fmt,
                   void* packed, void* scales, void* stream);

/* Inverse, to fp32 [rows, K]: decode(code) * 2^(scale-127).  Test aid. */
int mxfp6_dequantize(const void* packed, const void* scales, int64_t rows, int64_t K, int fmt,
                     void* out_f32, void* stream);

/*
 * Synchronises the current device and reports the device-side status word of the kernels launched
 * so far (0 = ok; otherwise low byte = role whose wait ran out, upper bits = CTA index), then clears
 * it.  Returns MXFP6_ERR_DEVICE_WAIT if it was non-zero.  The reference ignores launch status
 * (256_256_64_32_with16x32.cpp:385 leaves `ret` unused); this is the checked alternative.
 */
int mxfp6_device_status(int* status_out);

/*
 * Diagnostic: launches one warp that waits, with the kernels' bounded wait and a budget of budget_us
 * microseconds, on an mbarrier that nothing arrives on.  The wait runs out, the kernel returns, and the next
 * mxfp6_device_status() reports MXFP6_ERR_DEVICE_WAIT with role 9: the failure path of the GEMM kernels,
 * exercised without a fault, trap or hang.  (No counterpart in the reference, whose kernels have no waits
 * that can be bounded.)
 */
int mxfp6_debug_wait_timeout(int budget_us, void* stream);

/*
 * Test hook: sets one of the library's switches (the names of the environment variables that give their first
 * values: "MXFP6_FORCE_CFG" = "bn,swap,streamk[,pair]" forces a kernel variant, "MXFP6_NO_SF_TMA", "MXFP6_PDL",
 * "MXFP6_GROUP_P", "MXFP6_QUANT_PATH", "MXFP6_L2", "MXFP6_TAIL_SPLIT", "MXFP6_DECODE_ROWS", "MXFP6_DECODE_RING", "MXFP6_K_ROT", "MXFP6_PUSH_ROTATE", "MXFP6_C_PLAIN", "MXFP6_C_TMA_LAST", "MXFP6_L2_AHEAD"); value NULL restores the
 * default.  Takes effect for calls made after it returns.  (No counterpart in the reference.)
 */
int mxfp6_debug_option(const char* name, const char* value);

/*
 * Test hook: the kernel choice and tiling the GEMM entry points would make for this problem on a device with
 * sm_count SMs (no device is touched), as 12 ints: tile width BN, operands swapped, tiles split along K, CTA-pair
 * kernel, CTAs per SM, rows of the first / second operand per tile, tile counts along both, grid size, first tile of
 * the pair kernel's last partial wave and the number of column slices its tiles are cut into.  (No counterpart in
 * the reference, whose tiling is fixed at compile time: kernels/gemm/bf16fp32/256_256_64_32_with16x32.cpp:23-32.)
 */
int mxfp6_debug_plan(int64_t M, int64_t N, int64_t K, int sm_count, int n_dst, int requant, int* out12);

/*
 * Diagnostic: TMA-loads one 128-row x 128-element box of a packed operand (rows row0.., elements
 * k0..k0+127, k0 % 128 == 0) exactly as the GEMM does and copies the 16 KiB of shared memory it
 * produced to out16k (device).  Used by the tests to pin the shared-memory image of the 6-bit type.
 */
int mxfp6_debug_tma_dump(const void* packed, int64_t rows, int64_t K, int64_t row0, int64_t k0,
                         void* out16k, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* MXFP6_H_ */
