// MXFP8 quantizer: bf16 -> e4m3 elements with one e8m0 scale per 32 elements along the row, for a matrix and /
// or its transpose.  HBM-bound: one 128 x 128 tile per CTA is staged in shared memory once and both layouts are
// produced from it (2 B read, up to 2 x 1.03 B written per element).
//
// Arithmetic (bit-exact with the reference device code, csrc/mxfp8.cuh:45-72): scale = max(amax * fp32(1/448),
// 1e-12) rounded UP to a power of two (cvt.rp.satfinite.ue8m0x2), elements multiplied by the exact reciprocal
// 2^(127-e) and converted with cvt.rn.satfinite.e4m3x2.  Scale bytes are stored in the tensor-core scale-factor
// layout: tile [rows/128][cols/128] of 512 bytes, byte (r % 32) * 16 + (r / 32) * 4 + kblock (csrc/mxfp8.cuh:181-184).
#include "mxfp8.cuh"

namespace mok {
namespace {

constexpr int kTile = 128;
constexpr int kRowPitch = kTile * 2 + 16;   // bytes; the 16-byte pad keeps row-wise 16 B reads conflict free

__global__ void __launch_bounds__(128) quantize_kernel(const bf16* __restrict__ x, int rows, int cols, uint8_t* __restrict__ q,
                                                        uint8_t* __restrict__ sc, uint8_t* __restrict__ qt,
                                                        uint8_t* __restrict__ sct) {
    __shared__ __align__(16) uint8_t tile[kTile * kRowPitch];
    const int tid = threadIdx.x;
    const int tc = blockIdx.x, tr = blockIdx.y, e = blockIdx.z;
    const bf16* src = x + (static_cast<size_t>(e) * rows + static_cast<size_t>(tr) * kTile) * cols + static_cast<size_t>(tc) * kTile;

    // 128 rows x 16 vectors of 16 bytes, coalesced along the row
#pragma unroll 4
    for (int i = tid; i < kTile * 16; i += 128) {
        const int r = i >> 4, v = i & 15;
        const uint4 val = *reinterpret_cast<const uint4*>(src + static_cast<size_t>(r) * cols + v * 8);
        *reinterpret_cast<uint4*>(tile + r * kRowPitch + v * 16) = val;
    }
    __syncthreads();

    if (q != nullptr) {   // thread = row of the tile, four blocks of 32 along the row
        uint32_t scale_word = 0;
        uint8_t* out = q + (static_cast<size_t>(e) * rows + static_cast<size_t>(tr) * kTile + tid) * cols + static_cast<size_t>(tc) * kTile;
#pragma unroll
        for (int kb = 0; kb < 4; ++kb) {
            uint32_t packed[16];
#pragma unroll
            for (int v = 0; v < 4; ++v) {
                const uint4 val = *reinterpret_cast<const uint4*>(tile + tid * kRowPitch + kb * 64 + v * 16);
                packed[v * 4 + 0] = val.x; packed[v * 4 + 1] = val.y; packed[v * 4 + 2] = val.z; packed[v * 4 + 3] = val.w;
            }
            uint32_t out8[8], sbyte;
            mxfp8_quantize_block(packed, out8, sbyte);
            scale_word |= sbyte << (kb * 8);
            *reinterpret_cast<uint4*>(out + kb * 32) = make_uint4(out8[0], out8[1], out8[2], out8[3]);
            *reinterpret_cast<uint4*>(out + kb * 32 + 16) = make_uint4(out8[4], out8[5], out8[6], out8[7]);
        }
        uint8_t* sdst = sc + ((static_cast<size_t>(e) * (rows / kTile) + tr) * (cols / kTile) + tc) * 512;
        *reinterpret_cast<uint32_t*>(sdst + (tid & 31) * 16 + (tid >> 5) * 4) = scale_word;
    }
    if (qt != nullptr) {  // thread = column of the tile = row of the transpose, four blocks of 32 down the column
        uint32_t scale_word = 0;
        uint8_t* out = qt + (static_cast<size_t>(e) * cols + static_cast<size_t>(tc) * kTile + tid) * rows + static_cast<size_t>(tr) * kTile;
#pragma unroll
        for (int kb = 0; kb < 4; ++kb) {
            uint32_t packed[16];
#pragma unroll
            for (int i = 0; i < 16; ++i) {
                const uint16_t lo = *reinterpret_cast<const uint16_t*>(tile + (kb * 32 + 2 * i) * kRowPitch + tid * 2);
                const uint16_t hi = *reinterpret_cast<const uint16_t*>(tile + (kb * 32 + 2 * i + 1) * kRowPitch + tid * 2);
                packed[i] = static_cast<uint32_t>(lo) | (static_cast<uint32_t>(hi) << 16);
            }
            uint32_t out8[8], sbyte;
            mxfp8_quantize_block(packed, out8, sbyte);
            scale_word |= sbyte << (kb * 8);
            *reinterpret_cast<uint4*>(out + kb * 32) = make_uint4(out8[0], out8[1], out8[2], out8[3]);
            *reinterpret_cast<uint4*>(out + kb * 32 + 16) = make_uint4(out8[4], out8[5], out8[6], out8[7]);
        }
        uint8_t* sdst = sct + ((static_cast<size_t>(e) * (cols / kTile) + tc) * (rows / kTile) + tr) * 512;
        *reinterpret_cast<uint32_t*>(sdst + (tid & 31) * 16 + (tid >> 5) * 4) = scale_word;
    }
}

}  // namespace
}  // namespace mok

extern "C" int mok_mxfp8_quantize(const void* x_bf16, int num_matrices, int rows, int cols, void* x_fp8, void* x_sc,
                                  void* x_fp8_t, void* x_sc_t, mok_stream_t stream) {
    using namespace mok;
    if (x_bf16 == nullptr || num_matrices <= 0 || rows <= 0 || cols <= 0 || rows % 128 != 0 || cols % 128 != 0)
        return MOK_ERR_INVALID_ARGUMENT;
    if ((x_fp8 == nullptr) != (x_sc == nullptr) || (x_fp8_t == nullptr) != (x_sc_t == nullptr)) return MOK_ERR_INVALID_ARGUMENT;
    if (x_fp8 == nullptr && x_fp8_t == nullptr) return MOK_ERR_INVALID_ARGUMENT;
    if (num_matrices > 65535 || rows / 128 > 65535) return MOK_ERR_TOO_LARGE;
    dim3 grid(cols / 128, rows / 128, num_matrices);
    quantize_kernel<<<grid, 128, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
        static_cast<const bf16*>(x_bf16), rows, cols, static_cast<uint8_t*>(x_fp8), static_cast<uint8_t*>(x_sc),
        static_cast<uint8_t*>(x_fp8_t), static_cast<uint8_t*>(x_sc_t));
    MOK_LAUNCH_CHECK("mxfp8_quantize_kernel");
    return MOK_OK;
}
