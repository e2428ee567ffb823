// host_quant.cpp -- host-side weight preparation for the Q8 path: per-32 block symmetric
// quantization (d = amax / 127 stored as half, q = clamp(round(x / d), -127, 127)) into 34-byte
// Q8_0 blocks { half d; int8 qs[32] } and the repack into the planar Q8_0R layout
// ([nblocks*32] int8, then [nblocks] half).  Same results as the reference's host quantizers
// (include/ppml/QuantBlocks.h:62-79, :128-135), which its model applies when it switches the
// large linear layers to int8 (src/model/PPML.cpp:4504-4524).
#include <cuda_fp16.h>

#include <cmath>
#include <cstdint>
#include <cstring>

#include "../../include/ppml_b200.h"

extern "C" {

int ppml_b200_quantize_q8_0_host(const float* src, void* blocks34, int64_t n) {
    if (!src || !blocks34 || n <= 0 || (n % 32) != 0) return 1;
    uint8_t* out = static_cast<uint8_t*>(blocks34);
    const int64_t nb = n / 32;
    for (int64_t b = 0; b < nb; ++b) {
        const float* x = src + b * 32;
        float amax = 0.f;
        for (int i = 0; i < 32; ++i) amax = std::fmax(amax, std::fabs(x[i]));
        const float d = amax / 127.0f;
        const float inv = (amax == 0.0f) ? 0.0f : 1.0f / d;
        const __half hd = __float2half(d);
        std::memcpy(out + b * 34, &hd, 2);
        int8_t* qs = reinterpret_cast<int8_t*>(out + b * 34 + 2);
        for (int i = 0; i < 32; ++i) {
            float q = std::round(x[i] * inv);
            q = q > 127.0f ? 127.0f : (q < -127.0f ? -127.0f : q);
            qs[i] = static_cast<int8_t>(q);
        }
    }
    return 0;
}

int ppml_b200_repack_q8_0_host(const void* blocks34, int64_t nblocks, void* q8_0r) {
    if (!blocks34 || !q8_0r || nblocks <= 0) return 1;
    const uint8_t* in = static_cast<const uint8_t*>(blocks34);
    uint8_t* qs = static_cast<uint8_t*>(q8_0r);
    uint8_t* d = qs + nblocks * 32;
    for (int64_t b = 0; b < nblocks; ++b) {
        std::memcpy(qs + b * 32, in + b * 34 + 2, 32);
        std::memcpy(d + b * 2, in + b * 34, 2);
    }
    return 0;
}

}  // extern "C"
