// Device helpers of the MXFP8 format shared by the quantizer and by kernels that quantize in their epilogue.
#pragma once

#include "mok_common.cuh"

namespace mok {

// Quantizes one block of 32 bf16 values (16 packed pairs) to 32 e4m3 bytes (8 words) and one e8m0 scale byte.
// Same arithmetic as the reference's quantize_single_block (csrc/mxfp8.cuh:45-72).
__device__ __forceinline__ void mxfp8_quantize_block(const uint32_t (&in)[16], uint32_t (&out)[8], uint32_t& scale_byte) {
    float amax = 0.0f;
#pragma unroll
    for (int i = 0; i < 16; ++i) {
        const float2 f = unpack_bf16x2(in[i]);
        amax = fmaxf(amax, fmaxf(fabsf(f.x), fabsf(f.y)));
    }
    const float scale = fmaxf(amax * 0.002232142857f, 0.000000000001f);
    uint16_t e8m0x2;
    asm volatile("cvt.rp.satfinite.ue8m0x2.f32 %0, %1, %2;" : "=h"(e8m0x2) : "f"(scale), "f"(scale));
    scale_byte = e8m0x2 & 0xFFu;
    const float inv = __uint_as_float((254u - scale_byte) << 23);   // 2^(127 - e), exact
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const float2 a = unpack_bf16x2(in[2 * i]);
        const float2 b = unpack_bf16x2(in[2 * i + 1]);
        uint16_t lo, hi;
        asm volatile("cvt.rn.satfinite.e4m3x2.f32 %0, %2, %1;" : "=h"(lo) : "f"(a.x * inv), "f"(a.y * inv));
        asm volatile("cvt.rn.satfinite.e4m3x2.f32 %0, %2, %1;" : "=h"(hi) : "f"(b.x * inv), "f"(b.y * inv));
        out[i] = static_cast<uint32_t>(lo) | (static_cast<uint32_t>(hi) << 16);
    }
}

}  // namespace mok
