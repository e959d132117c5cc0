// SwiGLU arithmetic on packed bf16 pairs, shared by the stand-alone SwiGLU kernels (elementwise.cu) and the fused
// MXFP8 activation kernels (mxfp8.cu).  fp32 math on the stored bf16 values, results rounded to bf16.
#pragma once

#include "mok_common.cuh"

namespace mok {

__device__ __forceinline__ float sigmoid_fast(float x) { return 1.0f / (1.0f + __expf(-x)); }

// hidden = silu(gate) * up (reference csrc/megakernel/swiglu.cuh:135-165); with CLAMP gate is limited from above and
// up from both sides before the product.
template <bool CLAMP>
__device__ __forceinline__ uint32_t swiglu_pair(uint32_t g2, uint32_t u2, float limit) {
    float2 g = unpack_bf16x2(g2), u = unpack_bf16x2(u2);
    if (CLAMP) {
        g.x = fminf(g.x, limit); g.y = fminf(g.y, limit);
        u.x = fminf(fmaxf(u.x, -limit), limit); u.y = fminf(fmaxf(u.y, -limit), limit);
    }
    return pack_bf16x2(g.x * sigmoid_fast(g.x) * u.x, g.y * sigmoid_fast(g.y) * u.y);
}

// d_gate = dsilu(g) * u * dh, d_up = silu(g) * dh, zero where the forward clamp was active; returns
// dh * silu(g) * u for the router-weight gradient (reference csrc/megakernel/swiglu.cuh:1-36).
template <bool CLAMP>
__device__ __forceinline__ float swiglu_bwd_pair(uint32_t g2, uint32_t u2, uint32_t dh2, float limit, uint32_t& dg2,
                                                 uint32_t& du2) {
    float2 g = unpack_bf16x2(g2), u = unpack_bf16x2(u2);
    const float2 dh = unpack_bf16x2(dh2);
    bool gx = true, gy = true, ux = true, uy = true;
    if (CLAMP) {
        gx = g.x <= limit; gy = g.y <= limit;
        ux = u.x >= -limit && u.x <= limit; uy = u.y >= -limit && u.y <= limit;
        g.x = fminf(g.x, limit); g.y = fminf(g.y, limit);
        u.x = fminf(fmaxf(u.x, -limit), limit); u.y = fminf(fmaxf(u.y, -limit), limit);
    }
    const float sx = sigmoid_fast(g.x), sy = sigmoid_fast(g.y);
    const float silu_x = g.x * sx, silu_y = g.y * sy;
    const float dsx = (1.0f - silu_x) * sx + silu_x, dsy = (1.0f - silu_y) * sy + silu_y;
    dg2 = pack_bf16x2(gx ? dsx * u.x * dh.x : 0.0f, gy ? dsy * u.y * dh.y : 0.0f);
    du2 = pack_bf16x2(ux ? silu_x * dh.x : 0.0f, uy ? silu_y * dh.y : 0.0f);
    return dh.x * (silu_x * u.x) + dh.y * (silu_y * u.y);
}

}  // namespace mok
