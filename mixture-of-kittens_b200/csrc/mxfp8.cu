// MXFP8 quantizer: bf16 -> e4m3 elements with one e8m0 scale per 32 elements along the row, for a matrix and /
// or its transpose.  HBM-bound: one 128 x 128 tile per CTA is staged in shared memory once and both layouts are
// produced from it (2 B read, up to 2 x 1.03 B written per element).
//
// Arithmetic (bit-exact with the reference device code, csrc/mxfp8.cuh:45-72): scale = max(amax * fp32(1/448),
// 1e-12) rounded UP to a power of two (cvt.rp.satfinite.ue8m0x2), elements multiplied by the exact reciprocal
// 2^(127-e) and converted with cvt.rn.satfinite.e4m3x2.  Scale bytes are stored in the tensor-core scale-factor
// layout: tile [rows/128][cols/128] of 512 bytes, byte (r % 32) * 16 + (r / 32) * 4 + kblock (csrc/mxfp8.cuh:181-184).
//
// The same kernel serves the stand-alone op (whole matrices) and the fused layer (a window of schedule rows of an
// activation buffer, limited on the device by the padded token count; the transposed output then is a column range
// of a wider [cols, buffer_rows] matrix).
#include "mxfp8.cuh"
#include "swiglu_math.cuh"

namespace mok {
namespace {

constexpr int kTile = 128;
constexpr int kRowPitch = kTile * 2 + 16;   // bytes; the 16-byte pad keeps row-wise 16 B reads conflict free
constexpr int kOutPitch = kTile + 16;       // bytes per staged e4m3 output row
constexpr int kQuantSmemBytes = kTile * (kRowPitch + kOutPitch);

int enable_quantize_smem();   // raises the kernel's dynamic shared-memory limit once per device

// 128 rows x 128 bytes from the staging tile to global memory, eight lanes per row: every store instruction of a
// warp writes four complete 128-byte lines (a thread writing its own row would touch 32 lines with 16 bytes each).
__device__ __forceinline__ void store_staged_rows(const uint8_t* otile, uint8_t* out, long long ld, int tid) {
#pragma unroll 4
    for (int i = tid; i < kTile * 8; i += 128) {
        const int r = i >> 3, seg = i & 7;
        *reinterpret_cast<uint4*>(out + static_cast<long long>(r) * ld + seg * 16) =
            *reinterpret_cast<const uint4*>(otile + r * kOutPitch + seg * 16);
    }
}

// Transposed layout of a staged bf16 tile: thread = column of the tile = row of the transpose, four blocks of 32 down
// the column.  `out` is the transposed tile's first byte (rows `ld` apart), `scale_tile` its 512-byte scale tile.
// Every thread of the block calls; the tile must be complete (a barrier before the call is the caller's).
// A thread takes two adjacent columns (one 32-bit shared-memory word per row, conflict free across the warp) and two of
// the four row blocks: threads 0..63 the blocks 0 and 1, threads 64..127 the blocks 2 and 3.
__device__ __forceinline__ void quantize_tile_transposed(const uint8_t* tile, uint8_t* otile, int tid, uint8_t* out, long long ld,
                                                         uint8_t* scale_tile) {
    const int pair = tid & 63, half = tid >> 6;
    const int col_a = 2 * pair, col_b = col_a + 1;
    uint32_t scales_a = 0, scales_b = 0;
#pragma unroll
    for (int k = 0; k < 2; ++k) {
        const int kb = 2 * half + k;
        uint32_t pa[16], pb[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            const uint32_t w0 = *reinterpret_cast<const uint32_t*>(tile + (kb * 32 + 2 * i) * kRowPitch + pair * 4);
            const uint32_t w1 = *reinterpret_cast<const uint32_t*>(tile + (kb * 32 + 2 * i + 1) * kRowPitch + pair * 4);
            pa[i] = __byte_perm(w0, w1, 0x5410);   // low halves: column a of rows 2i, 2i + 1
            pb[i] = __byte_perm(w0, w1, 0x7632);   // high halves: column b
        }
        uint32_t out8[8], sbyte;
        mxfp8_quantize_block(pa, out8, sbyte);
        scales_a |= sbyte << (k * 8);
        uint8_t* dst = otile + col_a * kOutPitch + kb * 32;
        *reinterpret_cast<uint4*>(dst) = make_uint4(out8[0], out8[1], out8[2], out8[3]);
        *reinterpret_cast<uint4*>(dst + 16) = make_uint4(out8[4], out8[5], out8[6], out8[7]);
        mxfp8_quantize_block(pb, out8, sbyte);
        scales_b |= sbyte << (k * 8);
        dst = otile + col_b * kOutPitch + kb * 32;
        *reinterpret_cast<uint4*>(dst) = make_uint4(out8[0], out8[1], out8[2], out8[3]);
        *reinterpret_cast<uint4*>(dst + 16) = make_uint4(out8[4], out8[5], out8[6], out8[7]);
    }
    __syncthreads();
    store_staged_rows(otile, out, ld, tid);
    // scale bytes of row blocks 2 * half and 2 * half + 1 of the transposed rows col_a and col_b
    *reinterpret_cast<uint16_t*>(scale_tile + (col_a & 31) * 16 + (col_a >> 5) * 4 + 2 * half) = static_cast<uint16_t>(scales_a);
    *reinterpret_cast<uint16_t*>(scale_tile + (col_b & 31) * 16 + (col_b >> 5) * 4 + 2 * half) = static_cast<uint16_t>(scales_b);
}

struct QuantArgs {
    const bf16* x;             // row 0 of the span / matrix 0
    long long x_ld;            // elements between rows
    long long x_mat_stride;    // elements between matrices (blockIdx.z)
    uint8_t* q;                // normal output, same shape as x
    long long q_mat_stride;
    uint8_t* sc;               // scale tile (row tile 0, col tile 0)
    long long sc_row_tile_stride, sc_mat_stride;   // bytes
    uint8_t* qt;               // transposed output: element (c, r) at qt[c * qt_ld + r]
    long long qt_ld, qt_mat_stride;
    uint8_t* sct;              // scale tile (col tile 0, row tile 0) of the transposed output
    long long sct_row_tile_stride, sct_mat_stride;
    const int* num_tokens;     // optional device row limit (schedule rows)
    int row_begin, row_end;    // schedule rows covered by the span (row_end also bounds a dense matrix)
};

__global__ void __launch_bounds__(128) quantize_kernel(const QuantArgs a) {
    extern __shared__ __align__(16) uint8_t quant_smem[];
    uint8_t* tile = quant_smem;                                  // bf16 input tile, padded rows
    uint8_t* otile = quant_smem + kTile * kRowPitch;             // e4m3 rows staged for full-line stores
    const int tid = threadIdx.x;
    const int tc = blockIdx.x, tr = blockIdx.y, e = blockIdx.z;
    const int limit = a.num_tokens != nullptr ? min(a.row_end, *a.num_tokens) : a.row_end;
    if (a.row_begin + tr * kTile >= limit) return;
    const bf16* src = a.x + e * a.x_mat_stride + static_cast<long long>(tr) * kTile * a.x_ld + static_cast<long long>(tc) * kTile;

#pragma unroll 4
    for (int i = tid; i < kTile * 16; i += 128) {   // 128 rows x 16 vectors of 16 bytes, coalesced along the row
        const int r = i >> 4, v = i & 15;
        const uint4 val = *reinterpret_cast<const uint4*>(src + static_cast<long long>(r) * a.x_ld + v * 8);
        *reinterpret_cast<uint4*>(tile + r * kRowPitch + v * 16) = val;
    }
    __syncthreads();

    if (a.q != nullptr) {   // thread = row of the tile, four blocks of 32 along the row
        uint32_t scale_word = 0;
        uint8_t* out = a.q + e * a.q_mat_stride + static_cast<long long>(tr) * kTile * a.x_ld + static_cast<long long>(tc) * kTile;
        uint8_t* mine = otile + tid * kOutPitch;
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
            *reinterpret_cast<uint4*>(mine + kb * 32) = make_uint4(out8[0], out8[1], out8[2], out8[3]);
            *reinterpret_cast<uint4*>(mine + kb * 32 + 16) = make_uint4(out8[4], out8[5], out8[6], out8[7]);
        }
        __syncthreads();
        store_staged_rows(otile, out, a.x_ld, tid);
        __syncthreads();
        uint8_t* sdst = a.sc + e * a.sc_mat_stride + tr * a.sc_row_tile_stride + static_cast<long long>(tc) * 512;
        *reinterpret_cast<uint32_t*>(sdst + (tid & 31) * 16 + (tid >> 5) * 4) = scale_word;
    }
    if (a.qt != nullptr)
        quantize_tile_transposed(tile, otile, tid,
                                 a.qt + e * a.qt_mat_stride + static_cast<long long>(tc) * kTile * a.qt_ld + static_cast<long long>(tr) * kTile,
                                 a.qt_ld, a.sct + e * a.sct_mat_stride + tc * a.sct_row_tile_stride + static_cast<long long>(tr) * 512);
}

// ---- fused activation steps ---------------------------------------------------------------------------------------
// Both kernels walk a 128 x 128 tile with 16 lanes per row and eight consecutive columns per lane, sixteen rows per
// thread: a block of 32 along the row is four adjacent lanes, so the normal layout is quantized straight from
// registers (mxfp8_quantize_quarter) and stored as full 128-byte lines; the values that also need the transposed
// layout go through the shared-memory tile.
struct FusedFwdArgs {
    const bf16 *gate, *up;
    uint8_t *gate_q, *gate_sc, *up_q, *up_sc, *hidden_q, *hidden_sc, *hidden_qt, *hidden_sct;
    long long sc_row_tile_stride, qt_ld, sct_row_tile_stride;
    const int* num_tokens;
    int row_begin, row_end, cols;
    float limit;
};

template <bool CLAMP>
__global__ void __launch_bounds__(128) swiglu_quantize_fwd_kernel(const FusedFwdArgs a) {
    extern __shared__ __align__(16) uint8_t quant_smem[];
    uint8_t* tile = quant_smem;
    uint8_t* otile = quant_smem + kTile * kRowPitch;
    const int tid = threadIdx.x, v = tid & 15, rq = tid >> 4;
    const int tc = blockIdx.x, tr = blockIdx.y;
    const int limit_row = min(a.row_end, *a.num_tokens);
    if (a.row_begin + tr * kTile >= limit_row) return;
    const long long sc_off = tr * a.sc_row_tile_stride + static_cast<long long>(tc) * 512;
#pragma unroll 4
    for (int j = 0; j < 16; ++j) {
        const int r = rq + 8 * j;
        const long long off = (static_cast<long long>(tr) * kTile + r) * a.cols + tc * kTile + v * 8;
        const uint4 g = *reinterpret_cast<const uint4*>(a.gate + off);
        const uint4 u = *reinterpret_cast<const uint4*>(a.up + off);
        uint4 h;
        h.x = swiglu_pair<CLAMP>(g.x, u.x, a.limit);
        h.y = swiglu_pair<CLAMP>(g.y, u.y, a.limit);
        h.z = swiglu_pair<CLAMP>(g.z, u.z, a.limit);
        h.w = swiglu_pair<CLAMP>(g.w, u.w, a.limit);
        const int sidx = (r & 31) * 16 + (r >> 5) * 4 + (v >> 2);
        uint2 q;
        uint32_t sb;
        mxfp8_quantize_quarter(g, q, sb);
        *reinterpret_cast<uint2*>(a.gate_q + off) = q;
        if ((v & 3) == 0) a.gate_sc[sc_off + sidx] = static_cast<uint8_t>(sb);
        mxfp8_quantize_quarter(u, q, sb);
        *reinterpret_cast<uint2*>(a.up_q + off) = q;
        if ((v & 3) == 0) a.up_sc[sc_off + sidx] = static_cast<uint8_t>(sb);
        mxfp8_quantize_quarter(h, q, sb);
        *reinterpret_cast<uint2*>(a.hidden_q + off) = q;
        if ((v & 3) == 0) a.hidden_sc[sc_off + sidx] = static_cast<uint8_t>(sb);
        *reinterpret_cast<uint4*>(tile + r * kRowPitch + v * 16) = h;
    }
    __syncthreads();
    quantize_tile_transposed(tile, otile, tid, a.hidden_qt + static_cast<long long>(tc) * kTile * a.qt_ld + static_cast<long long>(tr) * kTile,
                             a.qt_ld, a.hidden_sct + tc * a.sct_row_tile_stride + static_cast<long long>(tr) * 512);
}

struct FusedBwdArgs {
    const uint8_t *gate_q, *gate_sc, *up_q, *up_sc;
    const bf16* d_hidden;
    uint8_t *dg_q, *dg_sc, *du_q, *du_sc, *dg_qt, *dg_sct, *du_qt, *du_sct;
    long long sc_row_tile_stride, qt_ld, sct_row_tile_stride;
    float* row_partial;
    const int* num_tokens;
    int row_begin, row_end, cols;
    float limit;
};

template <bool CLAMP>
__global__ void __launch_bounds__(128) swiglu_quantize_bwd_kernel(const FusedBwdArgs a) {
    extern __shared__ __align__(16) uint8_t quant_smem[];
    uint8_t* tile = quant_smem;
    uint8_t* otile = quant_smem + kTile * kRowPitch;
    const int tid = threadIdx.x, v = tid & 15, rq = tid >> 4;
    const int tc = blockIdx.x, tr = blockIdx.y;
    const int limit_row = min(a.row_end, *a.num_tokens);
    if (a.row_begin + tr * kTile >= limit_row) return;
    const long long sc_off = tr * a.sc_row_tile_stride + static_cast<long long>(tc) * 512;
    const int tiles = a.cols / kTile;
    uint4 du_keep[16];   // d_up waits in registers while d_gate uses the shared-memory tile
#pragma unroll
    for (int j = 0; j < 16; ++j) {
        const int r = rq + 8 * j;
        const long long row = static_cast<long long>(tr) * kTile + r;
        const long long off = row * a.cols + tc * kTile + v * 8;
        const uint2 gq = *reinterpret_cast<const uint2*>(a.gate_q + off);
        const uint2 uq = *reinterpret_cast<const uint2*>(a.up_q + off);
        const uint4 dh = *reinterpret_cast<const uint4*>(a.d_hidden + off);
        const int sidx = (r & 31) * 16 + (r >> 5) * 4 + (v >> 2);
        const uint4 g = mxfp8_dequantize8(gq, a.gate_sc[sc_off + sidx]);
        const uint4 u = mxfp8_dequantize8(uq, a.up_sc[sc_off + sidx]);
        uint4 dg, du;
        float acc = swiglu_bwd_pair<CLAMP>(g.x, u.x, dh.x, a.limit, dg.x, du.x);
        acc += swiglu_bwd_pair<CLAMP>(g.y, u.y, dh.y, a.limit, dg.y, du.y);
        acc += swiglu_bwd_pair<CLAMP>(g.z, u.z, dh.z, a.limit, dg.z, du.z);
        acc += swiglu_bwd_pair<CLAMP>(g.w, u.w, dh.w, a.limit, dg.w, du.w);
#pragma unroll
        for (int off_l = 1; off_l < 16; off_l <<= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off_l);   // the row's 16 lanes
        if (v == 0) a.row_partial[row * tiles + tc] = acc;
        uint2 q;
        uint32_t sb;
        mxfp8_quantize_quarter(dg, q, sb);
        *reinterpret_cast<uint2*>(a.dg_q + off) = q;
        if ((v & 3) == 0) a.dg_sc[sc_off + sidx] = static_cast<uint8_t>(sb);
        mxfp8_quantize_quarter(du, q, sb);
        *reinterpret_cast<uint2*>(a.du_q + off) = q;
        if ((v & 3) == 0) a.du_sc[sc_off + sidx] = static_cast<uint8_t>(sb);
        *reinterpret_cast<uint4*>(tile + r * kRowPitch + v * 16) = dg;
        du_keep[j] = du;
    }
    __syncthreads();
    const long long t_off = static_cast<long long>(tc) * kTile * a.qt_ld + static_cast<long long>(tr) * kTile;
    const long long ts_off = tc * a.sct_row_tile_stride + static_cast<long long>(tr) * 512;
    quantize_tile_transposed(tile, otile, tid, a.dg_qt + t_off, a.qt_ld, a.dg_sct + ts_off);
    __syncthreads();
#pragma unroll
    for (int j = 0; j < 16; ++j) *reinterpret_cast<uint4*>(tile + (rq + 8 * j) * kRowPitch + v * 16) = du_keep[j];
    __syncthreads();
    quantize_tile_transposed(tile, otile, tid, a.du_qt + t_off, a.qt_ld, a.du_sct + ts_off);
}

__global__ void __launch_bounds__(256) router_grad_kernel(const float* __restrict__ row_partial, int tiles,
                                                           const float* __restrict__ row_weight, float* __restrict__ row_grad,
                                                           const int* __restrict__ num_tokens, int row_begin, int row_end) {
    const int rows = min(row_end, *num_tokens) - row_begin;
    for (int row = blockIdx.x * blockDim.x + threadIdx.x; row < rows; row += gridDim.x * blockDim.x) {
        float acc = 0.0f;
        for (int t = 0; t < tiles; ++t) acc += row_partial[static_cast<long long>(row) * tiles + t];
        const float w = row_weight[row];
        row_grad[row] = w > 0.0f ? acc / w : 0.0f;
    }
}

// bf16[r, c] = e4m3[r, c] * 2^(scale(r, c / 32) - 127); exact (3 mantissa bits fit bf16).  One thread per 16 elements.
__global__ void __launch_bounds__(256) dequantize_kernel(const uint8_t* __restrict__ q, const uint8_t* __restrict__ sc,
                                                          long long sc_row_tile_stride, bf16* __restrict__ out, int cols,
                                                          const int* __restrict__ num_tokens, int row_begin, int row_end) {
    const int limit = num_tokens != nullptr ? min(row_end, *num_tokens) : row_end;
    const long long rows = limit - row_begin;
    const int vec_per_row = cols / 16;
    const long long n = rows * vec_per_row;
    const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
    for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) {
        const long long r = i / vec_per_row;
        const int c = static_cast<int>(i - r * vec_per_row) * 16;
        const uint4 v = *reinterpret_cast<const uint4*>(q + r * cols + c);
        const int rr = static_cast<int>(r & 127);
        const uint8_t sbyte = sc[(r >> 7) * sc_row_tile_stride + static_cast<long long>(c >> 7) * 512 + (rr & 31) * 16 + (rr >> 5) * 4 +
                                 ((c & 127) >> 5)];
        const float scale = __uint_as_float(static_cast<uint32_t>(sbyte) << 23);
        const uint32_t words[4] = {v.x, v.y, v.z, v.w};
        uint32_t o[8];
#pragma unroll
        for (int w = 0; w < 4; ++w) {
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const __half2_raw hr = __nv_cvt_fp8x2_to_halfraw2(static_cast<__nv_fp8x2_storage_t>(words[w] >> (16 * h)), __NV_E4M3);
                const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&hr));
                o[w * 2 + h] = pack_bf16x2(f.x * scale, f.y * scale);
            }
        }
        uint4* dst = reinterpret_cast<uint4*>(out + r * cols + c);
        dst[0] = make_uint4(o[0], o[1], o[2], o[3]);
        dst[1] = make_uint4(o[4], o[5], o[6], o[7]);
    }
}

int enable_quantize_smem() {
    static bool done[16] = {false};
    int dev = 0;
    MOK_CUDA_CHECK(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 16) return MOK_ERR_UNSUPPORTED;
    if (!done[dev]) {
        MOK_CUDA_CHECK(cudaFuncSetAttribute(quantize_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kQuantSmemBytes));
        done[dev] = true;
    }
    return MOK_OK;
}

}  // namespace

int launch_quantize_rows(const void* x, int cols, const int32_t* num_tokens, int row_begin, int row_end, void* q, void* sc,
                         long long sc_row_tile_stride, void* qt, long long qt_ld, void* sct, long long sct_row_tile_stride,
                         cudaStream_t stream) {
    if (x == nullptr || cols <= 0 || cols % 128 != 0 || row_end <= row_begin || (row_end - row_begin) % 128 != 0)
        return MOK_ERR_INVALID_ARGUMENT;
    if ((q == nullptr) != (sc == nullptr) || (qt == nullptr) != (sct == nullptr) || (q == nullptr && qt == nullptr))
        return MOK_ERR_INVALID_ARGUMENT;
    QuantArgs a{};
    a.x = static_cast<const bf16*>(x);
    a.x_ld = cols;
    a.q = static_cast<uint8_t*>(q);
    a.sc = static_cast<uint8_t*>(sc);
    a.sc_row_tile_stride = sc_row_tile_stride;
    a.qt = static_cast<uint8_t*>(qt);
    a.qt_ld = qt_ld;
    a.sct = static_cast<uint8_t*>(sct);
    a.sct_row_tile_stride = sct_row_tile_stride;
    a.num_tokens = num_tokens;
    a.row_begin = row_begin;
    a.row_end = row_end;
    const int row_tiles = (row_end - row_begin) / 128;
    if (row_tiles > 65535) return MOK_ERR_TOO_LARGE;
    dim3 grid(cols / 128, row_tiles, 1);
    if (int rc = enable_quantize_smem()) return rc;
    quantize_kernel<<<grid, 128, kQuantSmemBytes, stream>>>(a);
    MOK_LAUNCH_CHECK("mxfp8_quantize_kernel");
    return MOK_OK;
}

int launch_dequantize_rows(const void* q, const void* sc, long long sc_row_tile_stride, void* out, int cols,
                           const int32_t* num_tokens, int row_begin, int row_end, cudaStream_t stream) {
    if (q == nullptr || sc == nullptr || out == nullptr || cols <= 0 || cols % 128 != 0 || row_end <= row_begin)
        return MOK_ERR_INVALID_ARGUMENT;
    const long long items = static_cast<long long>(row_end - row_begin) * (cols / 16);
    long long blocks = (items + 255) / 256;
    const long long cap = static_cast<long long>(sm_count()) * 16;
    if (blocks > cap) blocks = cap;
    dequantize_kernel<<<static_cast<int>(blocks), 256, 0, stream>>>(static_cast<const uint8_t*>(q), static_cast<const uint8_t*>(sc),
                                                                    sc_row_tile_stride, static_cast<bf16*>(out), cols, num_tokens,
                                                                    row_begin, row_end);
    MOK_LAUNCH_CHECK("mxfp8_dequantize_kernel");
    return MOK_OK;
}

namespace {

// Raises the dynamic shared-memory limit of one kernel instantiation once per device.
template <typename Kernel>
int enable_tile_smem(Kernel kernel, bool (&done)[16]) {
    int dev = 0;
    MOK_CUDA_CHECK(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 16) return MOK_ERR_UNSUPPORTED;
    if (!done[dev]) {
        MOK_CUDA_CHECK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kQuantSmemBytes));
        done[dev] = true;
    }
    return MOK_OK;
}

template <typename Kernel, typename Args>
int launch_tile_kernel(Kernel kernel, const char* name, bool (&done)[16], const Args& args, int cols, int rows, cudaStream_t stream) {
    if (rows / 128 > 65535) return MOK_ERR_TOO_LARGE;
    if (int rc = enable_tile_smem(kernel, done)) return rc;
    dim3 grid(cols / 128, rows / 128, 1);
    kernel<<<grid, 128, kQuantSmemBytes, stream>>>(args);
    MOK_LAUNCH_CHECK(name);
    return MOK_OK;
}

}  // namespace

int launch_swiglu_quantize_fwd(const void* gate, const void* up, int cols, const int32_t* num_tokens, int row_begin, int row_end,
                               void* gate_q, void* gate_sc, void* up_q, void* up_sc, void* hidden_q, void* hidden_sc,
                               long long sc_row_tile_stride, void* hidden_qt, long long qt_ld, void* hidden_sct,
                               long long sct_row_tile_stride, bool has_limit, float limit, cudaStream_t stream) {
    if (!gate || !up || !num_tokens || !gate_q || !gate_sc || !up_q || !up_sc || !hidden_q || !hidden_sc || !hidden_qt || !hidden_sct)
        return MOK_ERR_INVALID_ARGUMENT;
    if (cols <= 0 || cols % 128 != 0 || row_end <= row_begin || (row_end - row_begin) % 128 != 0) return MOK_ERR_INVALID_ARGUMENT;
    FusedFwdArgs a{};
    a.gate = static_cast<const bf16*>(gate);
    a.up = static_cast<const bf16*>(up);
    a.gate_q = static_cast<uint8_t*>(gate_q);
    a.gate_sc = static_cast<uint8_t*>(gate_sc);
    a.up_q = static_cast<uint8_t*>(up_q);
    a.up_sc = static_cast<uint8_t*>(up_sc);
    a.hidden_q = static_cast<uint8_t*>(hidden_q);
    a.hidden_sc = static_cast<uint8_t*>(hidden_sc);
    a.hidden_qt = static_cast<uint8_t*>(hidden_qt);
    a.hidden_sct = static_cast<uint8_t*>(hidden_sct);
    a.sc_row_tile_stride = sc_row_tile_stride;
    a.qt_ld = qt_ld;
    a.sct_row_tile_stride = sct_row_tile_stride;
    a.num_tokens = num_tokens;
    a.row_begin = row_begin;
    a.row_end = row_end;
    a.cols = cols;
    a.limit = limit;
    static bool done_clamp[16] = {false}, done_plain[16] = {false};
    if (has_limit)
        return launch_tile_kernel(swiglu_quantize_fwd_kernel<true>, "swiglu_quantize_fwd_kernel", done_clamp, a, cols,
                                  row_end - row_begin, stream);
    return launch_tile_kernel(swiglu_quantize_fwd_kernel<false>, "swiglu_quantize_fwd_kernel", done_plain, a, cols,
                              row_end - row_begin, stream);
}

int launch_swiglu_quantize_bwd(const void* gate_q, const void* gate_sc, const void* up_q, const void* up_sc, const void* d_hidden,
                               int cols, const int32_t* num_tokens, int row_begin, int row_end, void* d_gate_q, void* d_gate_sc,
                               void* d_up_q, void* d_up_sc, long long sc_row_tile_stride, void* d_gate_qt, void* d_gate_sct,
                               void* d_up_qt, void* d_up_sct, long long qt_ld, long long sct_row_tile_stride, float* row_partial,
                               bool has_limit, float limit, cudaStream_t stream) {
    if (!gate_q || !gate_sc || !up_q || !up_sc || !d_hidden || !num_tokens || !d_gate_q || !d_gate_sc || !d_up_q || !d_up_sc ||
        !d_gate_qt || !d_gate_sct || !d_up_qt || !d_up_sct || !row_partial)
        return MOK_ERR_INVALID_ARGUMENT;
    if (cols <= 0 || cols % 128 != 0 || row_end <= row_begin || (row_end - row_begin) % 128 != 0) return MOK_ERR_INVALID_ARGUMENT;
    FusedBwdArgs a{};
    a.gate_q = static_cast<const uint8_t*>(gate_q);
    a.gate_sc = static_cast<const uint8_t*>(gate_sc);
    a.up_q = static_cast<const uint8_t*>(up_q);
    a.up_sc = static_cast<const uint8_t*>(up_sc);
    a.d_hidden = static_cast<const bf16*>(d_hidden);
    a.dg_q = static_cast<uint8_t*>(d_gate_q);
    a.dg_sc = static_cast<uint8_t*>(d_gate_sc);
    a.du_q = static_cast<uint8_t*>(d_up_q);
    a.du_sc = static_cast<uint8_t*>(d_up_sc);
    a.dg_qt = static_cast<uint8_t*>(d_gate_qt);
    a.dg_sct = static_cast<uint8_t*>(d_gate_sct);
    a.du_qt = static_cast<uint8_t*>(d_up_qt);
    a.du_sct = static_cast<uint8_t*>(d_up_sct);
    a.sc_row_tile_stride = sc_row_tile_stride;
    a.qt_ld = qt_ld;
    a.sct_row_tile_stride = sct_row_tile_stride;
    a.row_partial = row_partial;
    a.num_tokens = num_tokens;
    a.row_begin = row_begin;
    a.row_end = row_end;
    a.cols = cols;
    a.limit = limit;
    static bool done_clamp[16] = {false}, done_plain[16] = {false};
    if (has_limit)
        return launch_tile_kernel(swiglu_quantize_bwd_kernel<true>, "swiglu_quantize_bwd_kernel", done_clamp, a, cols,
                                  row_end - row_begin, stream);
    return launch_tile_kernel(swiglu_quantize_bwd_kernel<false>, "swiglu_quantize_bwd_kernel", done_plain, a, cols,
                              row_end - row_begin, stream);
}

int launch_router_grad(const float* row_partial, int tiles, const float* row_weight, float* row_grad, const int32_t* num_tokens,
                       int row_begin, int row_end, cudaStream_t stream) {
    if (!row_partial || !row_weight || !row_grad || !num_tokens || tiles <= 0 || row_end <= row_begin) return MOK_ERR_INVALID_ARGUMENT;
    long long blocks = (static_cast<long long>(row_end - row_begin) + 255) / 256;
    const long long cap = static_cast<long long>(sm_count()) * 8;
    if (blocks > cap) blocks = cap;
    router_grad_kernel<<<static_cast<int>(blocks), 256, 0, stream>>>(row_partial, tiles, row_weight, row_grad, num_tokens, row_begin,
                                                                     row_end);
    MOK_LAUNCH_CHECK("router_grad_kernel");
    return MOK_OK;
}

}  // namespace mok

extern "C" int mok_mxfp8_quantize(const void* x_bf16, int num_matrices, int rows, int cols, void* x_fp8, void* x_sc,
                                  void* x_fp8_t, void* x_sc_t, mok_stream_t stream) {
    using namespace mok;
    if (x_bf16 == nullptr || num_matrices <= 0 || rows <= 0 || cols <= 0 || rows % 128 != 0 || cols % 128 != 0)
        return MOK_ERR_INVALID_ARGUMENT;
    if ((x_fp8 == nullptr) != (x_sc == nullptr) || (x_fp8_t == nullptr) != (x_sc_t == nullptr)) return MOK_ERR_INVALID_ARGUMENT;
    if (x_fp8 == nullptr && x_fp8_t == nullptr) return MOK_ERR_INVALID_ARGUMENT;
    if (num_matrices > 65535 || rows / 128 > 65535) return MOK_ERR_TOO_LARGE;
    const long long elems = static_cast<long long>(rows) * cols;
    QuantArgs a{};
    a.x = static_cast<const bf16*>(x_bf16);
    a.x_ld = cols;
    a.x_mat_stride = elems;
    a.q = static_cast<uint8_t*>(x_fp8);
    a.q_mat_stride = elems;
    a.sc = static_cast<uint8_t*>(x_sc);
    a.sc_row_tile_stride = static_cast<long long>(cols / 128) * 512;
    a.sc_mat_stride = static_cast<long long>(rows / 128) * a.sc_row_tile_stride;
    a.qt = static_cast<uint8_t*>(x_fp8_t);
    a.qt_ld = rows;
    a.qt_mat_stride = elems;
    a.sct = static_cast<uint8_t*>(x_sc_t);
    a.sct_row_tile_stride = static_cast<long long>(rows / 128) * 512;
    a.sct_mat_stride = static_cast<long long>(cols / 128) * a.sct_row_tile_stride;
    a.num_tokens = nullptr;
    a.row_begin = 0;
    a.row_end = rows;
    dim3 grid(cols / 128, rows / 128, num_matrices);
    if (int rc = enable_quantize_smem()) return rc;
    quantize_kernel<<<grid, 128, kQuantSmemBytes, reinterpret_cast<cudaStream_t>(stream)>>>(a);
    MOK_LAUNCH_CHECK("mxfp8_quantize_kernel");
    return MOK_OK;
}
