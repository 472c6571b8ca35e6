// Block quantisation of 32 consecutive fp32 values to an MX format inside a kernel (used by the GEMM epilogues
// that hand their result to the next layer already quantised).  Same rule as the stand-alone quantiser:
// scale exponent = floor(log2(amax)) - emax_elem, clamp to [0,254], elements RNE + saturate by the hardware cvt.
#pragma once
#include <cuda_fp6.h>
#include <cuda_fp8.h>
#include <stdint.h>

namespace mxfp6 {

// format codes of the C ABI
constexpr int kE2M3 = 0, kE3M2 = 1, kE4M3 = 2, kE5M2 = 3;

__device__ __forceinline__ int quant_emax(int fmt) { return fmt == kE2M3 ? 2 : fmt == kE3M2 ? 4 : fmt == kE4M3 ? 8 : 15; }

// Hardware conversion of two fp32 values at once (round to nearest even, saturate to the largest finite value):
// returns code(x0) | code(x1) << 8, fp6 codes in the low 6 bits of their byte.
template <int FMT>
__device__ __forceinline__ uint32_t cvt_pair(float x0, float x1) {
    uint16_t r;
    if constexpr (FMT == kE2M3) asm("cvt.rn.satfinite.e2m3x2.f32 %0, %1, %2;" : "=h"(r) : "f"(x1), "f"(x0));
    else if constexpr (FMT == kE3M2) asm("cvt.rn.satfinite.e3m2x2.f32 %0, %1, %2;" : "=h"(r) : "f"(x1), "f"(x0));
    else if constexpr (FMT == kE4M3) asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(r) : "f"(x1), "f"(x0));
    else asm("cvt.rn.satfinite.e5m2x2.f32 %0, %1, %2;" : "=h"(r) : "f"(x1), "f"(x0));
    return r;
}
__device__ __forceinline__ uint32_t mad_u32(uint32_t a, uint32_t b, uint32_t c) {
    uint32_t d;
    asm("mad.lo.u32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}
// four values -> 4 codes: fp8 one per byte (32 bits), fp6 6 bits each (24 bits)
template <int FMT>
__device__ __forceinline__ uint32_t cvt_quad(float x0, float x1, float x2, float x3) {
    const uint32_t lo = cvt_pair<FMT>(x0, x1), hi = cvt_pair<FMT>(x2, x3);
    if constexpr (FMT == kE4M3 || FMT == kE5M2) return lo | (hi << 16);          // one code per byte
    // a pair is c0 + 256*c1; the 12-bit form c0 + 64*c1 is pair - 192*(pair >> 8), and two 12-bit forms join by
    // one more multiply-add: integer multiply-adds run on the FMA pipe, which this code leaves idle, not on the ALU
    const uint32_t lo12 = mad_u32(lo >> 8, 0xffffff40u, lo), hi12 = mad_u32(hi >> 8, 0xffffff40u, hi);
    return mad_u32(hi12, 4096u, lo12);
}

// E8M0 byte of a block whose largest magnitude is amax
__device__ __forceinline__ int quant_scale_byte(float amax, int fmt) {
    const uint32_t u = __float_as_uint(amax);
    int fl = (int)((u >> 23) & 0xff) - 127;
    if (((u >> 23) & 0xff) == 0) fl = 31 - __clz(u & 0x7fffff) - 149;     // fp32 subnormal
    int sb = fl - quant_emax(fmt) + 127;
    sb = sb < 0 ? 0 : sb > 254 ? 254 : sb;
    if (!(amax > 0.f)) sb = 0;
    if (isinf(amax)) sb = 254;
    return sb;
}

// max(|a|, |b|, |c|) in one instruction (three-input max of sm_100)
__device__ __forceinline__ float amax3(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(fabsf(a)), "f"(fabsf(b)), "f"(fabsf(c)));
    return d;
}

// largest magnitude of v[0..31]
__device__ __forceinline__ float amax32(const float* v) {
    float m[11];
#pragma unroll
    for (int i = 0; i < 10; ++i) m[i] = amax3(v[3 * i], v[3 * i + 1], v[3 * i + 2]);
    m[10] = fmaxf(fabsf(v[30]), fabsf(v[31]));
    const float a = amax3(m[0], m[1], m[2]), b = amax3(m[3], m[4], m[5]), c = amax3(m[6], m[7], m[8]);
    return amax3(amax3(a, b, c), m[9], m[10]);
}

// v[0..31] (fp32) with largest magnitude amax -> out[0..5] (fp6: 24 bytes) or out[0..7] (fp8: 32 bytes); returns
// the scale byte
template <int FMT>
__device__ __forceinline__ int quant_block32_amax(const float* v, float amax, uint32_t* out) {
    const int sb = quant_scale_byte(amax, FMT);
    const int e = sb - 127;
    // 2^-e, -127 <= -e <= 127, is an fp32 value (2^-127 a subnormal one) and the product with an element of the
    // block is exact: |x| * 2^-e < 2^(emax+1)
    const float f = e == 127 ? __uint_as_float(0x00400000u) : __uint_as_float((uint32_t)(127 - e) << 23);
    if constexpr (FMT == kE4M3 || FMT == kE5M2) {
#pragma unroll
        for (int g = 0; g < 8; ++g)
            out[g] = cvt_quad<FMT>(v[4 * g] * f, v[4 * g + 1] * f, v[4 * g + 2] * f, v[4 * g + 3] * f);
    } else {
        uint32_t w24[8];
#pragma unroll
        for (int g = 0; g < 8; ++g)
            w24[g] = cvt_quad<FMT>(v[4 * g] * f, v[4 * g + 1] * f, v[4 * g + 2] * f, v[4 * g + 3] * f);
#pragma unroll
        for (int h4 = 0; h4 < 2; ++h4) {      // 4 x 24 bits -> 3 words, twice
            const uint32_t* q = w24 + 4 * h4;
            out[3 * h4 + 0] = mad_u32(q[1], 1u << 24, q[0]);
            out[3 * h4 + 1] = mad_u32(q[2], 1u << 16, q[1] >> 8);
            out[3 * h4 + 2] = mad_u32(q[3], 1u << 8, q[2] >> 16);
        }
    }
    return sb;
}

template <int FMT>
__device__ __forceinline__ int quant_block32(const float* v, uint32_t* out) {
    return quant_block32_amax<FMT>(v, amax32(v), out);
}

// One code (low byte) from one value: the pair conversion with a zero partner.
__device__ __forceinline__ uint32_t cvt_one(float x, int fmt) {
    uint32_t r;
    if (fmt == kE2M3) r = cvt_pair<kE2M3>(x, 0.f);
    else if (fmt == kE3M2) r = cvt_pair<kE3M2>(x, 0.f);
    else if (fmt == kE4M3) r = cvt_pair<kE4M3>(x, 0.f);
    else r = cvt_pair<kE5M2>(x, 0.f);
    return r & 0xffu;
}
__device__ __forceinline__ uint32_t cvt_quad_rt(float x0, float x1, float x2, float x3, int fmt) {
    if (fmt == kE2M3) return cvt_quad<kE2M3>(x0, x1, x2, x3);
    if (fmt == kE3M2) return cvt_quad<kE3M2>(x0, x1, x2, x3);
    if (fmt == kE4M3) return cvt_quad<kE4M3>(x0, x1, x2, x3);
    return cvt_quad<kE5M2>(x0, x1, x2, x3);
}
__device__ __forceinline__ float quant_inv_scale(int sb) {          // 2^-(sb-127)
    const int e = sb - 127;
    return e == 127 ? __uint_as_float(0x00400000u) : __uint_as_float((uint32_t)(127 - e) << 23);
}

// A block of 32 consecutive columns of output row `row` whose elements sit one per lane of a warp (lane = column
// within the block): scale from the warp-wide largest magnitude, one conversion per lane, and the codes leave as
// 32 bytes (fp8) or, gathered by four lanes at a time, as six 32-bit words (fp6).  Whole warp, converged.
__device__ __forceinline__ void quant_store_lanes(float x, int fmt, uint8_t* q_out, size_t q_ld, uint8_t* q_scales,
                                                  int n_cols, int row, int col0, bool row_valid) {
    const int lane = threadIdx.x & 31;
    const float amax = __uint_as_float(__reduce_max_sync(0xffffffffu, __float_as_uint(fabsf(x))));
    const int sb = quant_scale_byte(amax, fmt);
    const uint32_t code = cvt_one(x * quant_inv_scale(sb), fmt);
    const bool fp8 = fmt == kE4M3 || fmt == kE5M2;
    if (fp8) {
        if (row_valid) q_out[(size_t)row * q_ld + col0 + lane] = (uint8_t)code;
    } else {
        // lanes 4j: 24 bits of the four codes 4j..4j+3; then lanes 4j, 4j+1, 4j+2 of every 16 write one word each
        uint32_t w = code | (__shfl_down_sync(0xffffffffu, code, 1) << 6) | (__shfl_down_sync(0xffffffffu, code, 2) << 12) |
                     (__shfl_down_sync(0xffffffffu, code, 3) << 18);
        const uint32_t w0 = __shfl_sync(0xffffffffu, w, (lane & ~15) + 0), w1 = __shfl_sync(0xffffffffu, w, (lane & ~15) + 4),
                       w2 = __shfl_sync(0xffffffffu, w, (lane & ~15) + 8), w3 = __shfl_sync(0xffffffffu, w, (lane & ~15) + 12);
        const int i = lane & 15;
        if (row_valid && i < 3) {
            const uint32_t word = i == 0 ? (w0 | (w1 << 24)) : i == 1 ? ((w1 >> 8) | (w2 << 16)) : ((w2 >> 16) | (w3 << 8));
            reinterpret_cast<uint32_t*>(q_out + (size_t)row * q_ld + col0 / 4 * 3)[(lane >> 4) * 3 + i] = word;
        }
    }
    if (row_valid && lane == 0) q_scales[(size_t)row * (n_cols / 32) + col0 / 32] = (uint8_t)sb;
}

// The same for a block whose 32 columns are held four per lane by 8 consecutive lanes (lane % 8 = column / 4).
__device__ __forceinline__ void quant_store_lanes4(const float (&x)[4], int fmt, uint8_t* q_out, size_t q_ld, uint8_t* q_scales,
                                                   int n_cols, int row, int col0, bool row_valid) {
    const int lane = threadIdx.x & 31;
    float amax = fmaxf(fmaxf(fabsf(x[0]), fabsf(x[1])), fmaxf(fabsf(x[2]), fabsf(x[3])));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 4));
    const int sb = quant_scale_byte(amax, fmt);
    const float f = quant_inv_scale(sb);
    const uint32_t w = cvt_quad_rt(x[0] * f, x[1] * f, x[2] * f, x[3] * f, fmt);
    const bool fp8 = fmt == kE4M3 || fmt == kE5M2;
    const int j = lane & 7;                                   // this lane's 4 columns: col0 + 4j ..
    if (fp8) {
        if (row_valid) reinterpret_cast<uint32_t*>(q_out + (size_t)row * q_ld + col0)[j] = w;
    } else {
        // lanes 4g..4g+3 hold 4 x 24 bits = three 32-bit words of the packed stream
        const uint32_t wn = __shfl_down_sync(0xffffffffu, w, 1);
        const int i4 = lane & 3;
        if (row_valid && i4 < 3)
            reinterpret_cast<uint32_t*>(q_out + (size_t)row * q_ld + col0 / 4 * 3)[(j >> 2) * 3 + i4] = (w >> (8 * i4)) | (wn << (24 - 8 * i4));
    }
    if (row_valid && j == 0) q_scales[(size_t)row * (n_cols / 32) + col0 / 32] = (uint8_t)sb;
}

// Quantise 32 consecutive columns [col, col+32) of row `row` and store codes + scale.
//   q_out: operand bytes, row stride q_ld bytes; q_scales: [rows, n_cols/32]
__device__ __forceinline__ void quant_store32(const uint32_t* vbits, int fmt, uint8_t* q_out, size_t q_ld, uint8_t* q_scales,
                                              int n_cols, int row, int col) {
    float v[32];
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(vbits[i]);
    uint32_t w[8];
    int sb;
    const bool fp8 = fmt == kE4M3 || fmt == kE5M2;
    if (fmt == kE2M3) sb = quant_block32<kE2M3>(v, w);
    else if (fmt == kE3M2) sb = quant_block32<kE3M2>(v, w);
    else if (fmt == kE4M3) sb = quant_block32<kE4M3>(v, w);
    else sb = quant_block32<kE5M2>(v, w);
    uint8_t* dst = q_out + (size_t)row * q_ld + (fp8 ? col : col / 4 * 3);
    // 24 (fp6) or 32 (fp8) bytes; 8-byte aligned in both cases when q_ld % 8 == 0 and col % 32 == 0
    uint2* d2 = reinterpret_cast<uint2*>(dst);
    d2[0] = make_uint2(w[0], w[1]);
    d2[1] = make_uint2(w[2], w[3]);
    d2[2] = make_uint2(w[4], w[5]);
    if (fp8) d2[3] = make_uint2(w[6], w[7]);
    q_scales[(size_t)row * (n_cols / 32) + col / 32] = (uint8_t)sb;
}

}  // namespace mxfp6
