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

// The same quantization with the block of 32 spread over four adjacent lanes, eight consecutive bf16 values (`in`)
// each: the maximum is exchanged with two shuffles (every lane of the warp must call), the rest is per lane.
// Bit-identical to mxfp8_quantize_block.  All four lanes receive the scale byte.
__device__ __forceinline__ void mxfp8_quantize_quarter(const uint4& in, uint2& out, uint32_t& scale_byte) {
    const uint32_t w[4] = {in.x, in.y, in.z, in.w};
    float amax = 0.0f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 f = unpack_bf16x2(w[i]);
        amax = fmaxf(amax, fmaxf(fabsf(f.x), fabsf(f.y)));
    }
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
    const float scale = fmaxf(amax * 0.002232142857f, 0.000000000001f);
    uint16_t e8m0x2;
    asm volatile("cvt.rp.satfinite.ue8m0x2.f32 %0, %1, %2;" : "=h"(e8m0x2) : "f"(scale), "f"(scale));
    scale_byte = e8m0x2 & 0xFFu;
    const float inv = __uint_as_float((254u - scale_byte) << 23);
    uint32_t o[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const float2 a = unpack_bf16x2(w[2 * i]);
        const float2 b = unpack_bf16x2(w[2 * i + 1]);
        uint16_t lo, hi;
        asm volatile("cvt.rn.satfinite.e4m3x2.f32 %0, %2, %1;" : "=h"(lo) : "f"(a.x * inv), "f"(a.y * inv));
        asm volatile("cvt.rn.satfinite.e4m3x2.f32 %0, %2, %1;" : "=h"(hi) : "f"(b.x * inv), "f"(b.y * inv));
        o[i] = static_cast<uint32_t>(lo) | (static_cast<uint32_t>(hi) << 16);
    }
    out = make_uint2(o[0], o[1]);
}

// Eight e4m3 bytes with their e8m0 scale byte -> eight bf16 values (exact: three mantissa bits fit bf16).
__device__ __forceinline__ uint4 mxfp8_dequantize8(const uint2& q, uint32_t scale_byte) {
    const float scale = __uint_as_float(scale_byte << 23);
    const uint32_t words[2] = {q.x, q.y};
    uint32_t o[4];
#pragma unroll
    for (int w = 0; w < 2; ++w) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const __half2_raw hr = __nv_cvt_fp8x2_to_halfraw2(static_cast<__nv_fp8x2_storage_t>(words[w] >> (16 * h)), __NV_E4M3);
            const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&hr));
            o[w * 2 + h] = pack_bf16x2(f.x * scale, f.y * scale);
        }
    }
    return make_uint4(o[0], o[1], o[2], o[3]);
}

// Fused MXFP8 activation steps of the layer (mxfp8.cu).  Row window and pointer conventions as launch_quantize_rows:
// every pointer addresses the window's first row (transposed outputs: its column), scale pointers its first row tile.
// Forward: gate, up (bf16 [rows, cols]) -> e4m3 gate, up (normal layout), hidden = silu(gate) * up in both layouts.
int launch_swiglu_quantize_fwd(const void* gate, const void* up, int cols, const int32_t* num_tokens, int row_begin, int row_end,
                               void* gate_q, void* gate_sc, void* up_q, void* up_sc, void* hidden_q, void* hidden_sc,
                               long long sc_row_tile_stride, void* hidden_qt, long long qt_ld, void* hidden_sct,
                               long long sct_row_tile_stride, bool has_limit, float limit, cudaStream_t stream);

// Backward: saved e4m3 gate, up and bf16 d_hidden -> d_gate, d_up in both layouts, plus per (row, 128-column tile) the
// partial sums of d_hidden * hidden in row_partial[row * (cols / 128) + tile] for the router-weight gradient.
int launch_swiglu_quantize_bwd(const void* gate_q, const void* gate_sc, const void* up_q, const void* up_sc, const void* d_hidden,
                               int cols, const int32_t* num_tokens, int row_begin, int row_end, void* d_gate_q, void* d_gate_sc,
                               void* d_up_q, void* d_up_sc, long long sc_row_tile_stride, void* d_gate_qt, void* d_gate_sct,
                               void* d_up_qt, void* d_up_sct, long long qt_ld, long long sct_row_tile_stride, float* row_partial,
                               bool has_limit, float limit, cudaStream_t stream);

// row_grad[row] = (sum over tiles, ascending, of row_partial[row * tiles + tile]) / row_weight[row], 0 where the weight
// is not positive.
int launch_router_grad(const float* row_partial, int tiles, const float* row_weight, float* row_grad, const int32_t* num_tokens,
                       int row_begin, int row_end, cudaStream_t stream);

}  // namespace mok
