// Generates tests/golden/toolkit_fp8_kat.json: known answers for FP8 E4M3 / E5M2 from the CUDA toolkit's HOST
// conversion routines (cuda_fp8.h), saturating (SATFINITE) and round-to-nearest-even.  Runs on the CPU only.
//   nvcc -o /tmp/gen_toolkit_fp8 tests/golden/gen_toolkit_fp8.cu && /tmp/gen_toolkit_fp8 > tests/golden/toolkit_fp8_kat.json
#include <cuda_fp8.h>
#include <cuda_fp16.h>
#include <cmath>
#include <cstdio>
#include <cstring>
#include <cstdint>
#include <vector>

static uint32_t bits(float f) { uint32_t u; memcpy(&u, &f, 4); return u; }

int main() {
    std::vector<float> xs;
    // every e4m3 / e5m2 value, every midpoint between neighbours, and the fp32 neighbours of each midpoint
    for (int fmt = 0; fmt < 2; ++fmt) {
        float prev = 0.f;
        for (int c = 1; c < (fmt == 0 ? 0x7f : 0x7c); ++c) {
            __half_raw h = __nv_cvt_fp8_to_halfraw((__nv_fp8_storage_t)c, fmt == 0 ? __NV_E4M3 : __NV_E5M2);
            float v = __half2float(__half(h));
            float mid = 0.5f * (prev + v);
            const float cand[] = {v, mid, nextafterf(mid, 0.f), nextafterf(mid, 1e30f)};
            for (float x : cand) { xs.push_back(x); xs.push_back(-x); }
            prev = v;
        }
    }
    const float extra[] = {0.f, 1e-9f, 0.0009f, 0.001f, 449.f, 460.f, 464.f, 465.f, 480.f, 511.f, 512.f, 1e6f,
                           57344.f, 60000.f, 61440.f, 65535.f, 1e30f, 7.6e-6f, 1.5e-5f};
    for (float e : extra) { xs.push_back(e); xs.push_back(-e); }
    printf("{\n\"encode\": [\n");
    for (size_t i = 0; i < xs.size(); ++i) {
        unsigned a = __nv_cvt_float_to_fp8(xs[i], __NV_SATFINITE, __NV_E4M3);
        unsigned b = __nv_cvt_float_to_fp8(xs[i], __NV_SATFINITE, __NV_E5M2);
        printf("[%u,%u,%u]%s\n", bits(xs[i]), a & 255u, b & 255u, i + 1 < xs.size() ? "," : "");
    }
    printf("],\n\"decode_e4m3\": [");
    for (int c = 0; c < 256; ++c) {
        __half_raw h = __nv_cvt_fp8_to_halfraw((__nv_fp8_storage_t)c, __NV_E4M3);
        printf("%u%s", bits(__half2float(__half(h))), c < 255 ? "," : "");
    }
    printf("],\n\"decode_e5m2\": [");
    for (int c = 0; c < 256; ++c) {
        __half_raw h = __nv_cvt_fp8_to_halfraw((__nv_fp8_storage_t)c, __NV_E5M2);
        printf("%u%s", bits(__half2float(__half(h))), c < 255 ? "," : "");
    }
    printf("]\n}\n");
    return 0;
}
