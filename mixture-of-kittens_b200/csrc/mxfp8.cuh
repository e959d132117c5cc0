// Device helpers of the MXFP8 format shared by the quantizer and by kernels that quantize in their epilogue.
#pragma once

#include <cuda_fp16.h>
#include <cuda_fp8.h>

#include "mok_common.cuh"

namespace mok {

// Quantizes schedule rows [row_begin, min(row_end, *num_tokens)) of a bf16 activation buffer whose row 0 (`x`) holds
// schedule row row_begin.  Normal output: q (same shape) + scale tiles at sc + row_tile * sc_row_tile_stride +
// col_tile * 512.  Transposed output: element (c, r) at qt[c * qt_ld + r] (qt points at the column of row_begin) +
// scale tiles at sct + col_tile * sct_row_tile_stride + row_tile * 512.  Either pair may be nullptr.
int launch_quantize_rows(const void* x, int cols, const int32_t* num_tokens, int row_begin, int row_end, void* q, void* sc,
                         long long sc_row_tile_stride, void* qt, long long qt_ld, void* sct, long long sct_row_tile_stride,
                         cudaStream_t stream);

// bf16 out[r, c] = value of the MXFP8 element (exact), same row window convention.
int launch_dequantize_rows(const void* q, const void* sc, long long sc_row_tile_stride, void* out, int cols,
                           const int32_t* num_tokens, int row_begin, int row_end, cudaStream_t stream);

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
