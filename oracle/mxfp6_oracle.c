/*
 * mxfp6_oracle.c -- CPU restatement of the MX-FP6 GEMM path.  TEST INFRASTRUCTURE ONLY.
 *
 * This file is the checker for the CUDA path: tests, the smoke check and the CPU-baseline
 * leg of the benchmark call it; nothing in the shipped package may.
 *
 * PARITY UNPINNED: the reference tree holds no fp6 source, no fp6 test and no fp6 golden
 * vector (kernels/gemm/README.md:6-7 only says that the fp6 kernel lives on another branch).
 * The number format below therefore follows the OCP Microscaling (MX) v1.0 definitions of
 * FP6 E2M3 / E3M2 and E8M0, and is pinned instead against the CUDA toolkit's own host
 * conversions (tests/golden/toolkit_fp6_kat.json, made by tests/golden/gen_toolkit_fp6.cu)
 * and against torch.float8_e8m0fnu.
 *
 * What is followed from the reference is the *shape* of the computation:
 *   - C[M,N] = A[M,K] * B[N,K]^T, both operands K-contiguous
 *       (kernels/gemm/bf16fp32/256_256_64_32_with16x32.cpp:47-58, bench.py:34);
 *   - CPU check loop: one fp32 accumulator per output, k ascending, one rounding to bf16 at
 *       the end (kernels/gemm/fp8fp32/FP8_8wave/8_wave.cu:451-460);
 *   - bf16 conversion is round-to-nearest-even (include/common/base_types.cuh:281-283);
 *   - element-wise 1 % check with abs() on the threshold
 *       (kernels/torch_scaled/scaled_matmul.cu:542, fixing 8_wave.cu:488).
 *
 * Format summary
 *   E2M3: s ee mmm, bias 1, no inf/nan.  e==0: +-m/8 ; e>0: +-2^(e-1)*(1+m/8); max 7.5
 *   E3M2: s eee mm, bias 3, no inf/nan.  e==0: +-m/16; e>0: +-2^(e-3)*(1+m/4); max 28
 *   MX-FP8 operands (one byte per element) go through the same path: E4M3 (bias 7, max 448, 0x7f NaN) with
 *   emax_elem 8, E5M2 (bias 15, max 57344, exponent 31 inf/nan) with emax_elem 15; format codes 2 and 3.
 *   E8M0: byte x -> 2^(x-127); 0xFF is NaN and is never produced.
 *   Block of 32 along K: scale exponent = floor(log2(amax)) - emax_elem, emax_elem = 2 (E2M3)
 *   or 4 (E3M2); stored byte = clamp(exp+127, 0, 254); amax==0 -> byte 0, all codes +-0.
 *   Elements: v = x * 2^-exp (exact), round-to-nearest-even onto the fp6 grid, saturate.
 *   Packing: dense little-endian 6-bit stream along K: element i occupies bits [6i,6i+6)
 *   of the row's byte string (b0=v0|v1<<6, b1=v1>>2|v2<<4, b2=v2>>4|v3<<2).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define MXFP6_E2M3 0
#define MXFP6_E3M2 1

static inline uint32_t f32_bits(float f) { uint32_t u; memcpy(&u, &f, 4); return u; }
static inline float bits_f32(uint32_t u) { float f; memcpy(&f, &u, 4); return f; }

/* exact 2^e for e in [-149, 127] */
static inline float pow2i(int e) {
    if (e >= -126) return bits_f32((uint32_t)(e + 127) << 23);
    return bits_f32(1u << (uint32_t)(e + 149));
}

/* ---- format parameters ---------------------------------------------------- */
#define MXFP8_E4M3 2
#define MXFP8_E5M2 3
typedef struct { int bits, mbits, bias, emax; float maxv; int maxcode; } fmt_t;
static fmt_t fmt_of(int fmt) {
    switch (fmt) {
        case MXFP6_E2M3: { fmt_t f = {6, 3, 1, 2, 7.5f, 0x1f}; return f; }
        case MXFP6_E3M2: { fmt_t f = {6, 2, 3, 4, 28.0f, 0x1f}; return f; }
        case MXFP8_E4M3: { fmt_t f = {8, 3, 7, 8, 448.0f, 0x7e}; return f; }   /* 0x7f is NaN */
        default:         { fmt_t f = {8, 2, 15, 15, 57344.0f, 0x7b}; return f; } /* exponent 31 is inf/nan */
    }
}

/* ---- element decode ---------------------------------------------------- */
float mxfp6_decode_elem(uint8_t code, int fmt) {
    fmt_t f = fmt_of(fmt);
    int ebits = f.bits - 1 - f.mbits;
    int sign  = (code >> (f.bits - 1)) & 1;
    int e     = (code >> f.mbits) & ((1 << ebits) - 1);
    int m     = code & ((1 << f.mbits) - 1);
    float mag;
    if (fmt == MXFP8_E4M3 && e == 15 && m == 7) mag = NAN;
    else if (fmt == MXFP8_E5M2 && e == 31) mag = m ? NAN : INFINITY;
    else if (e == 0) mag = (float)m * pow2i(1 - f.bias - f.mbits);
    else             mag = (float)((1 << f.mbits) + m) * pow2i(e - f.bias - f.mbits);
    return sign ? -mag : mag;
}

/* ---- element encode: RNE, saturating, input already divided by the block scale ---- */
uint8_t mxfp6_encode_elem(float v, int fmt) {
    fmt_t f = fmt_of(fmt);
    int mbits = f.mbits, bias = f.bias;
    float maxv = f.maxv;
    uint8_t sign = (f32_bits(v) >> 31) ? (uint8_t)(1u << (f.bits - 1)) : 0;
    float a = fabsf(v);
    if (!(a == a)) return (uint8_t)(sign | f.maxcode);   /* NaN in -> max magnitude */
    if (a >= maxv) return (uint8_t)(sign | f.maxcode);   /* saturate (also +-inf) */
    /* quantum of the binade a lies in; the subnormal range shares the quantum of the first binade */
    int ex = (int)((f32_bits(a) >> 23) & 0xff) - 127;    /* floor(log2 a) for normal fp32 */
    if (a < pow2i(1 - bias)) ex = 1 - bias;              /* subnormal range of the target (and tiny/zero) */
    float q = pow2i(ex - mbits);                         /* spacing of representable values */
    /* a/q is exact (power-of-two divide); nearbyintf rounds to nearest even in default mode */
    float n = nearbyintf(a / q);
    float r = n * q;                                     /* rounded magnitude, may carry to next binade */
    if (r >= maxv) return (uint8_t)(sign | f.maxcode);
    if (r == 0.0f) return sign;                          /* the sign of zero is kept, as the toolkit and the hardware cvt do */
    int re = (int)((f32_bits(r) >> 23) & 0xff) - 127;
    uint8_t code;
    if (r < pow2i(1 - bias)) {
        code = (uint8_t)(r / pow2i(1 - bias - mbits));   /* subnormal: e=0, m = r/2^(1-bias-mbits) */
    } else {
        int e = re + bias;
        int m = (int)(r / pow2i(re - mbits)) - (1 << mbits);
        code = (uint8_t)((e << mbits) | m);
    }
    return (uint8_t)(sign | code);
}

/* ---- E8M0 ---------------------------------------------------------------- */
float mxfp6_e8m0_decode(uint8_t x) {
    if (x == 0xff) return NAN;
    return pow2i((int)x - 127);
}

/* scale byte for a block whose max |x| is amax */
uint8_t mxfp6_e8m0_from_amax(float amax, int fmt) {
    int emax_elem = fmt_of(fmt).emax;
    if (!(amax > 0.0f) || isinf(amax)) {
        if (isinf(amax)) return 254;
        return 0;
    }
    uint32_t u = f32_bits(amax);
    int ex = (int)((u >> 23) & 0xff);
    int fl;                                              /* floor(log2(amax)), exact */
    if (ex == 0) {                                       /* fp32 subnormal */
        uint32_t man = u & 0x7fffff; int p = 22;
        while (!((man >> p) & 1)) --p;
        fl = p - 149;
    } else fl = ex - 127;
    int e = fl - emax_elem + 127;
    if (e < 0) e = 0;
    if (e > 254) e = 254;
    return (uint8_t)e;
}

/* ---- pack / unpack ------------------------------------------------------- */
/* n must be a multiple of 4; out has 3n/4 bytes */
void mxfp6_pack(const uint8_t* codes, int64_t n, uint8_t* out) {
    for (int64_t i = 0, o = 0; i < n; i += 4, o += 3) {
        uint32_t w = (uint32_t)(codes[i] & 63) | ((uint32_t)(codes[i + 1] & 63) << 6) |
                     ((uint32_t)(codes[i + 2] & 63) << 12) | ((uint32_t)(codes[i + 3] & 63) << 18);
        out[o] = (uint8_t)w; out[o + 1] = (uint8_t)(w >> 8); out[o + 2] = (uint8_t)(w >> 16);
    }
}
void mxfp6_unpack(const uint8_t* packed, int64_t n, uint8_t* codes) {
    for (int64_t i = 0, o = 0; i < n; i += 4, o += 3) {
        uint32_t w = (uint32_t)packed[o] | ((uint32_t)packed[o + 1] << 8) | ((uint32_t)packed[o + 2] << 16);
        codes[i] = w & 63; codes[i + 1] = (w >> 6) & 63; codes[i + 2] = (w >> 12) & 63; codes[i + 3] = (w >> 18) & 63;
    }
}

/* ---- block quantiser ------------------------------------------------------ */
/* src [rows,K] fp32 row-major, K % 32 == 0 -> operand bytes (fp6: packed [rows,3K/4]; fp8: [rows,K]),
 * scales [rows,K/32] */
void mxfp6_quantize(const float* src, int64_t rows, int64_t K, int fmt, uint8_t* packed, uint8_t* scales) {
    const int fp8 = fmt_of(fmt).bits == 8;
    #pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < rows; ++r) {
        uint8_t codes[32];
        for (int64_t kb = 0; kb < K / 32; ++kb) {
            const float* x = src + r * K + kb * 32;
            float amax = 0.0f;
            for (int i = 0; i < 32; ++i) { float a = fabsf(x[i]); if (a > amax) amax = a; }
            uint8_t sb = mxfp6_e8m0_from_amax(amax, fmt);
            scales[r * (K / 32) + kb] = sb;
            int e = (int)sb - 127;
            /* multiply by 2^-e in two exact steps so that neither factor leaves fp32 range */
            int h = (-e) / 2;
            float f1 = pow2i(h), f2 = pow2i(-e - h);
            for (int i = 0; i < 32; ++i) codes[i] = mxfp6_encode_elem(x[i] * f1 * f2, fmt);
            if (fp8) memcpy(packed + r * K + kb * 32, codes, 32);
            else mxfp6_pack(codes, 32, packed + r * (K * 3 / 4) + kb * 24);
        }
    }
}

/* operand bytes + scales -> fp32 [rows,K]; decode(code)*2^(scale-127) */
void mxfp6_dequantize(const uint8_t* packed, const uint8_t* scales, int64_t rows, int64_t K, int fmt, float* out) {
    const int fp8 = fmt_of(fmt).bits == 8;
    float lut[256];
    for (int c = 0; c < (fp8 ? 256 : 64); ++c) lut[c] = mxfp6_decode_elem((uint8_t)c, fmt);
    #pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < rows; ++r) {
        uint8_t codes[32];
        for (int64_t kb = 0; kb < K / 32; ++kb) {
            if (fp8) memcpy(codes, packed + r * K + kb * 32, 32);
            else mxfp6_unpack(packed + r * (K * 3 / 4) + kb * 24, 32, codes);
            float s = mxfp6_e8m0_decode(scales[r * (K / 32) + kb]);
            for (int i = 0; i < 32; ++i) out[r * K + kb * 32 + i] = lut[codes[i]] * s;
        }
    }
}

/* ---- bf16 ------------------------------------------------------------------ */
uint16_t mxfp6_f32_to_bf16(float f) {
    uint32_t u = f32_bits(f);
    if ((u & 0x7fffffff) > 0x7f800000) return (uint16_t)((u >> 16) | 0x40);   /* quiet NaN */
    uint32_t lsb = (u >> 16) & 1;
    u += 0x7fff + lsb;                                                          /* RNE */
    return (uint16_t)(u >> 16);
}
float mxfp6_bf16_to_f32(uint16_t h) { return bits_f32((uint32_t)h << 16); }

/* ---- GEMM oracle ------------------------------------------------------------ */
/*
 * C[M,N] = dequant(A)[M,K] * dequant(B)[N,K]^T.
 * acc_mode 0: one fp32 accumulator, k ascending (the reference's CPU loop, 8_wave.cu:451-460)
 * acc_mode 1: one fp64 accumulator, k ascending (separates accumulation-order noise from errors)
 * c_bf16 (may be NULL) receives RNE bf16; c_f32 (may be NULL) receives the unrounded accumulator.
 * absdot (may be NULL) receives sum_k |a_k*b_k| in fp64 -> fp32 (the scale of accumulation noise).
 */
void mxfp6_gemm_ref(const uint8_t* a_packed, const uint8_t* sfa, const uint8_t* b_packed, const uint8_t* sfb,
                    int64_t M, int64_t N, int64_t K, int fmt_a, int fmt_b, int acc_mode,
                    uint16_t* c_bf16, float* c_f32, float* absdot) {
    float* A = (float*)malloc(sizeof(float) * (size_t)M * K);
    float* B = (float*)malloc(sizeof(float) * (size_t)N * K);
    mxfp6_dequantize(a_packed, sfa, M, K, fmt_a, A);
    mxfp6_dequantize(b_packed, sfb, N, K, fmt_b, B);
    #pragma omp parallel for schedule(static)
    for (int64_t m = 0; m < M; ++m) {
        for (int64_t n = 0; n < N; ++n) {
            const float* a = A + m * K; const float* b = B + n * K;
            float r; double ad = 0.0;
            if (acc_mode == 0) {
                float acc = 0.0f;
                for (int64_t k = 0; k < K; ++k) acc += a[k] * b[k];
                r = acc;
            } else {
                double acc = 0.0;
                for (int64_t k = 0; k < K; ++k) acc += (double)a[k] * (double)b[k];
                r = (float)acc;
            }
            if (absdot) { for (int64_t k = 0; k < K; ++k) ad += fabs((double)a[k] * (double)b[k]); absdot[m * N + n] = (float)ad; }
            if (c_f32) c_f32[m * N + n] = r;
            if (c_bf16) c_bf16[m * N + n] = mxfp6_f32_to_bf16(r);
        }
    }
    free(A); free(B);
}
