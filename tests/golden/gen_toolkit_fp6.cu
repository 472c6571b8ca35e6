// Generates tests/golden/toolkit_fp6_kat.json: known answers for FP6 (E2M3/E3M2) and E8M0 taken from the
// CUDA toolkit's own HOST conversion routines (cuda_fp6.h / cuda_fp8.h).  Runs on the CPU only.
//   nvcc -o /tmp/gen_toolkit_fp6 tests/golden/gen_toolkit_fp6.cu && /tmp/gen_toolkit_fp6 > tests/golden/toolkit_fp6_kat.json
// The oracle's encoder/decoder is checked against this file by tests/test_oracle.py.
#include <cuda_fp6.h>
#include <cuda_fp8.h>
#include <cuda_fp16.h>
#include <cstdio>
#include <cstring>
#include <cstdint>
#include <vector>

static uint32_t bits(float f) { uint32_t u; memcpy(&u, &f, 4); return u; }

int main() {
    std::vector<float> xs;
    // dense sweep around every rounding boundary of both formats: multiples of 1/64 up to 40, both signs
    for (int i = 0; i <= 40 * 64; ++i) { xs.push_back(i / 64.0f); xs.push_back(-(i / 64.0f)); }
    // just-above / just-below every midpoint (next representable fp32 on both sides)
    for (int i = 1; i <= 32 * 32; ++i) {
        float m = i / 32.0f;
        xs.push_back(nextafterf(m, 0.0f)); xs.push_back(nextafterf(m, 100.0f));
    }
    // tiny, huge
    const float extra[] = {1e-8f, 0.03f, 0.031f, 0.0312f, 0.03125f, 0.0313f, 0.0625f, 0.09374f, 0.09375f, 0.09376f,
                           29.9f, 30.0f, 31.9f, 32.0f, 100.0f, 1e30f, 7.74f, 7.75f, 7.76f, 7.99f};
    for (float e : extra) { xs.push_back(e); xs.push_back(-e); }

    printf("{\n\"encode\": [\n");
    for (size_t i = 0; i < xs.size(); ++i) {
        unsigned a = __nv_cvt_float_to_fp6(xs[i], __NV_E2M3, cudaRoundNearest);
        unsigned b = __nv_cvt_float_to_fp6(xs[i], __NV_E3M2, cudaRoundNearest);
        printf("[%u,%u,%u]%s\n", bits(xs[i]), a & 63u, b & 63u, i + 1 < xs.size() ? "," : "");
    }
    printf("],\n\"decode_e2m3\": [");
    for (int c = 0; c < 64; ++c) {
        __half_raw h = __nv_cvt_fp6_to_halfraw((__nv_fp6_storage_t)c, __NV_E2M3);
        __half hh(h);
        printf("%u%s", bits(__half2float(hh)), c < 63 ? "," : "");
    }
    printf("],\n\"decode_e3m2\": [");
    for (int c = 0; c < 64; ++c) {
        __half_raw h = __nv_cvt_fp6_to_halfraw((__nv_fp6_storage_t)c, __NV_E3M2);
        __half hh(h);
        printf("%u%s", bits(__half2float(hh)), c < 63 ? "," : "");
    }
    // E8M0: float -> e8m0 with round-toward-zero keeps floor(log2 x) for x>0, i.e. the exponent field
    printf("],\n\"e8m0_floor\": [\n");
    const float sv[] = {1.0f, 1.5f, 1.9999f, 2.0f, 3.0f, 0.5f, 0.75f, 1e-3f, 1e3f, 6.0f, 7.5f, 8.0f, 28.0f, 448.0f,
                        1.1754944e-38f, 3.0e38f, 0.015625f, 0.02f, 65504.0f};
    int ns = (int)(sizeof(sv) / sizeof(sv[0]));
    for (int i = 0; i < ns; ++i) {
        unsigned e = __nv_cvt_float_to_e8m0(sv[i], __NV_SATFINITE, cudaRoundZero);
        printf("[%u,%u]%s\n", bits(sv[i]), e & 255u, i + 1 < ns ? "," : "");
    }
    printf("]\n}\n");
    return 0;
}
