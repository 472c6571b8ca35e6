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
// four values -> 4 codes: fp8 one per byte (32 bits), fp6 6 bits each (24 bits)
template <int FMT>
__device__ __forceinline__ uint32_t cvt_quad(float x0, float x1, float x2, float x3) {
    const uint32_t lo = cvt_pair<FMT>(x0, x1), hi = cvt_pair<FMT>(x2, x3);
    const uint32_t t = lo | (hi << 16);                   // one code per byte
    if constexpr (FMT == kE4M3 || FMT == kE5M2) return t;
    // four 6-bit fields at bit 0, 8, 16, 24 -> bit 0, 6, 12, 18: first within each half, then the halves
    const uint32_t u = (t & 0x003f003fu) | ((t >> 2) & 0x0fc00fc0u);
    return (u & 0xfffu) | ((u >> 4) & 0xfff000u);
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
            out[3 * h4 + 0] = q[0] | (q[1] << 24);
            out[3 * h4 + 1] = (q[1] >> 8) | (q[2] << 16);
            out[3 * h4 + 2] = (q[2] >> 16) | (q[3] << 8);
        }
    }
    return sb;
}

template <int FMT>
__device__ __forceinline__ int quant_block32(const float* v, uint32_t* out) {
    return quant_block32_amax<FMT>(v, amax32(v), out);
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
