// Bandwidth-bound kernels of the MoE layer: SwiGLU forward / backward (with the router-weight gradient),
// the fixed-order forward / backward epilogues, and zeroing the weight gradients of experts without tokens.
#include "elementwise.cuh"
#include "swiglu_math.cuh"

namespace mok {
namespace {

template <bool CLAMP>
__global__ void __launch_bounds__(256) swiglu_fwd_kernel(const uint4* __restrict__ gate, const uint4* __restrict__ up,
                                                          uint4* __restrict__ hidden, const int* __restrict__ num_tokens,
                                                          int dense_rows, int row_begin, int row_end, int vec_per_row,
                                                          float limit) {
    const int total = num_tokens != nullptr ? *num_tokens : dense_rows;
    const int hi = min(row_end, total);
    if (hi <= row_begin) return;
    const long long n = static_cast<long long>(hi - row_begin) * vec_per_row;
    const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
    for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) {
        const uint4 g = gate[i], u = up[i];
        uint4 h;
        h.x = swiglu_pair<CLAMP>(g.x, u.x, limit);
        h.y = swiglu_pair<CLAMP>(g.y, u.y, limit);
        h.z = swiglu_pair<CLAMP>(g.z, u.z, limit);
        h.w = swiglu_pair<CLAMP>(g.w, u.w, limit);
        hidden[i] = h;
    }
}

// One warp per row.  With row_weight != nullptr the warp also reduces sum_i dh*hidden over the row (lanes own
// fixed column sets and the butterfly is fixed, so the result is reproducible) and stores it divided by the row's
// router weight (0 when the weight is not positive): d_router_weight of that route.
template <bool CLAMP>
__global__ void __launch_bounds__(256) swiglu_bwd_kernel(const uint4* __restrict__ gate, const uint4* __restrict__ up,
                                                          const uint4* __restrict__ d_hidden, uint4* __restrict__ d_gate,
                                                          uint4* __restrict__ d_up, const int* __restrict__ num_tokens,
                                                          int dense_rows, int row_begin, int row_end, int vec_per_row,
                                                          float limit, const float* __restrict__ row_weight,
                                                          float* __restrict__ row_grad) {
    const int total = num_tokens != nullptr ? *num_tokens : dense_rows;
    const int rows = min(row_end, total) - row_begin;
    const int warps = (gridDim.x * blockDim.x) >> 5;
    const int lane = threadIdx.x & 31;
    for (int row = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; row < rows; row += warps) {
        const size_t base = static_cast<size_t>(row) * vec_per_row;
        float acc = 0.0f;
        for (int v = lane; v < vec_per_row; v += 32) {
            const uint4 g = gate[base + v], u = up[base + v], dh = d_hidden[base + v];
            uint4 dg, du;
            acc += swiglu_bwd_pair<CLAMP>(g.x, u.x, dh.x, limit, dg.x, du.x);
            acc += swiglu_bwd_pair<CLAMP>(g.y, u.y, dh.y, limit, dg.y, du.y);
            acc += swiglu_bwd_pair<CLAMP>(g.z, u.z, dh.z, limit, dg.z, du.z);
            acc += swiglu_bwd_pair<CLAMP>(g.w, u.w, dh.w, limit, dg.w, du.w);
            d_gate[base + v] = dg;
            d_up[base + v] = du;
        }
        if (row_weight != nullptr) {
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
            if (lane == 0) {
                const float w = row_weight[row];
                row_grad[row] = w > 0.0f ? acc / w : 0.0f;
            }
        }
    }
}

__device__ __forceinline__ void fma_vec(float (&acc)[8], uint4 v, float w) {
    const float2 a = unpack_bf16x2(v.x), b = unpack_bf16x2(v.y), c = unpack_bf16x2(v.z), d = unpack_bf16x2(v.w);
    acc[0] = fmaf(w, a.x, acc[0]); acc[1] = fmaf(w, a.y, acc[1]);
    acc[2] = fmaf(w, b.x, acc[2]); acc[3] = fmaf(w, b.y, acc[3]);
    acc[4] = fmaf(w, c.x, acc[4]); acc[5] = fmaf(w, c.y, acc[5]);
    acc[6] = fmaf(w, d.x, acc[6]); acc[7] = fmaf(w, d.y, acc[7]);
}

// out[t] = bf16(shared[t] + sum_k w[t,k] * routed[t*K + k]), k ascending; WEIGHTED = false uses w = 1.
// With a status word that holds any error bit (schedule overflow dropped rows, a wait ran out, a bad schedule entry)
// the routed slots may hold stale or partial data: the whole output becomes NaN instead, so the failure cannot be
// trained through unnoticed; no host synchronisation is involved.
template <bool WEIGHTED>
__global__ void __launch_bounds__(256) epilogue_kernel(const uint4* __restrict__ shared, const uint4* __restrict__ routed,
                                                        const float* __restrict__ weights, uint4* __restrict__ out,
                                                        long long tokens, int vec_per_row, int topk,
                                                        const uint32_t* __restrict__ status) {
    const long long n = tokens * vec_per_row;
    const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
    if (status != nullptr && *status != 0u) {
        const uint4 nan4 = make_uint4(0x7FC07FC0u, 0x7FC07FC0u, 0x7FC07FC0u, 0x7FC07FC0u);   // bf16 quiet NaNs
        for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) out[i] = nan4;
        return;
    }
    for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) {
        const long long t = i / vec_per_row;
        const int v = static_cast<int>(i - t * vec_per_row);
        float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        if (shared != nullptr) fma_vec(acc, shared[i], 1.0f);
        const uint4* r = routed + (t * topk) * vec_per_row + v;
        const float* w = weights + t * topk;
        int k = 0;
        for (; k + 4 <= topk; k += 4) {   // four rows in flight, accumulated in ascending k
            const uint4 r0 = r[static_cast<long long>(k) * vec_per_row], r1 = r[static_cast<long long>(k + 1) * vec_per_row];
            const uint4 r2 = r[static_cast<long long>(k + 2) * vec_per_row], r3 = r[static_cast<long long>(k + 3) * vec_per_row];
            fma_vec(acc, r0, WEIGHTED ? w[k] : 1.0f);
            fma_vec(acc, r1, WEIGHTED ? w[k + 1] : 1.0f);
            fma_vec(acc, r2, WEIGHTED ? w[k + 2] : 1.0f);
            fma_vec(acc, r3, WEIGHTED ? w[k + 3] : 1.0f);
        }
        for (; k < topk; ++k) fma_vec(acc, r[static_cast<long long>(k) * vec_per_row], WEIGHTED ? w[k] : 1.0f);
        uint4 o;
        o.x = pack_bf16x2(acc[0], acc[1]);
        o.y = pack_bf16x2(acc[2], acc[3]);
        o.z = pack_bf16x2(acc[4], acc[5]);
        o.w = pack_bf16x2(acc[6], acc[7]);
        out[i] = o;
    }
}

__global__ void __launch_bounds__(256) zero_empty_kernel(const int* __restrict__ tokens_per_expert, uint4* a, uint4* b,
                                                          uint4* c, long long vec_per_expert) {
    const int e = blockIdx.y;
    if (tokens_per_expert[e] != 0) return;
    const uint4 z = make_uint4(0, 0, 0, 0);
    const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
    for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < vec_per_expert; i += stride) {
        a[e * vec_per_expert + i] = z;
        b[e * vec_per_expert + i] = z;
        c[e * vec_per_expert + i] = z;
    }
}

// One block per expert: occupied[e] = 1 + the last row (relative to the expert's first row) that carries a token, 0 if
// none.  Padding rows (peer_rank < 0) normally sit at the tail of an expert's range; scanning the whole range keeps the
// answer right for any placement.
__global__ void occupied_rows_kernel(const int32_t* __restrict__ peer_rank, const int32_t* __restrict__ tokens_per_expert,
                                     const int32_t* __restrict__ num_tokens, int schedule_capacity, int32_t* __restrict__ occupied) {
    __shared__ int partial[8];
    const int e = blockIdx.x;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    int before = 0;
    for (int i = threadIdx.x; i < e; i += blockDim.x) before += tokens_per_expert[i];
    before = __reduce_add_sync(0xffffffffu, before);
    if (lane == 0) partial[warp] = before;
    __syncthreads();
    int first = 0;
    for (int w = 0; w < 8; ++w) first += partial[w];
    __syncthreads();
    int limit = *num_tokens;
    if (limit > schedule_capacity) limit = schedule_capacity;
    int end = first + tokens_per_expert[e];
    if (end > limit) end = limit;
    int last = 0;
    for (int r = first + threadIdx.x; r < end; r += blockDim.x)
        if (peer_rank[r] >= 0) last = r - first + 1;
    last = __reduce_max_sync(0xffffffffu, last);
    if (lane == 0) partial[warp] = last;
    __syncthreads();
    if (threadIdx.x == 0) {
        int m = 0;
        for (int w = 0; w < 8; ++w) m = max(m, partial[w]);
        occupied[e] = m;
    }
}

int stream_grid(long long items, int threads) {
    long long blocks = (items + threads - 1) / threads;
    const long long cap = static_cast<long long>(sm_count()) * 16;
    if (blocks > cap) blocks = cap;
    return blocks < 1 ? 1 : static_cast<int>(blocks);
}

}  // namespace

int launch_swiglu_fwd(const void* gate, const void* up, void* hidden, const int32_t* num_tokens, int dense_rows,
                      int row_begin, int row_end, int intermediate, bool has_limit, float limit, cudaStream_t stream) {
    if (intermediate % 8 != 0 || row_end <= row_begin) return MOK_ERR_INVALID_ARGUMENT;
    const int vec = intermediate / 8;
    const int grid = stream_grid(static_cast<long long>(row_end - row_begin) * vec, 256);
    auto g = static_cast<const uint4*>(gate);
    auto u = static_cast<const uint4*>(up);
    auto h = static_cast<uint4*>(hidden);
    if (has_limit)
        swiglu_fwd_kernel<true><<<grid, 256, 0, stream>>>(g, u, h, num_tokens, dense_rows, row_begin, row_end, vec, limit);
    else
        swiglu_fwd_kernel<false><<<grid, 256, 0, stream>>>(g, u, h, num_tokens, dense_rows, row_begin, row_end, vec, limit);
    MOK_LAUNCH_CHECK("swiglu_fwd_kernel");
    return MOK_OK;
}

int launch_swiglu_bwd(const void* gate, const void* up, const void* d_hidden, void* d_gate, void* d_up,
                      const int32_t* num_tokens, int dense_rows, int row_begin, int row_end, int intermediate,
                      bool has_limit, float limit, const float* row_weight, float* row_grad, cudaStream_t stream) {
    if (intermediate % 8 != 0 || row_end <= row_begin) return MOK_ERR_INVALID_ARGUMENT;
    const int vec = intermediate / 8;
    const int grid = stream_grid(static_cast<long long>(row_end - row_begin) * 32, 256);
    auto g = static_cast<const uint4*>(gate);
    auto u = static_cast<const uint4*>(up);
    auto dh = static_cast<const uint4*>(d_hidden);
    auto dg = static_cast<uint4*>(d_gate);
    auto du = static_cast<uint4*>(d_up);
    if (has_limit)
        swiglu_bwd_kernel<true><<<grid, 256, 0, stream>>>(g, u, dh, dg, du, num_tokens, dense_rows, row_begin, row_end, vec,
                                                         limit, row_weight, row_grad);
    else
        swiglu_bwd_kernel<false><<<grid, 256, 0, stream>>>(g, u, dh, dg, du, num_tokens, dense_rows, row_begin, row_end, vec,
                                                          limit, row_weight, row_grad);
    MOK_LAUNCH_CHECK("swiglu_bwd_kernel");
    return MOK_OK;
}

int launch_occupied_rows(const int32_t* peer_rank, const int32_t* tokens_per_expert, const int32_t* num_tokens,
                         int schedule_capacity, int num_experts, int32_t* occupied, cudaStream_t stream) {
    if (!peer_rank || !tokens_per_expert || !num_tokens || !occupied || num_experts < 1) return MOK_ERR_INVALID_ARGUMENT;
    occupied_rows_kernel<<<num_experts, 256, 0, stream>>>(peer_rank, tokens_per_expert, num_tokens, schedule_capacity, occupied);
    MOK_LAUNCH_CHECK("occupied_rows_kernel");
    return MOK_OK;
}

int launch_zero_empty_wgrads(const int32_t* tokens_per_expert, int num_experts, void* a, void* b, void* c,
                             long long elems_per_expert, cudaStream_t stream) {
    if (elems_per_expert % 8 != 0) return MOK_ERR_INVALID_ARGUMENT;
    dim3 grid(64, num_experts);
    zero_empty_kernel<<<grid, 256, 0, stream>>>(tokens_per_expert, static_cast<uint4*>(a), static_cast<uint4*>(b),
                                                static_cast<uint4*>(c), elems_per_expert / 8);
    MOK_LAUNCH_CHECK("zero_empty_kernel");
    return MOK_OK;
}

}  // namespace mok

extern "C" int mok_fwd_epilogue(const void* y_shared, const void* combine_buffer, const float* topk_weights, void* out,
                                int64_t num_local_tokens, int hidden, int topk, const uint32_t* status, mok_stream_t stream) {
    using namespace mok;
    if (combine_buffer == nullptr || topk_weights == nullptr || out == nullptr || num_local_tokens <= 0 || hidden <= 0 ||
        hidden % 8 != 0 || topk <= 0)
        return MOK_ERR_INVALID_ARGUMENT;
    const int vec = hidden / 8;
    const int grid = stream_grid(num_local_tokens * vec, 256);
    epilogue_kernel<true><<<grid, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
        static_cast<const uint4*>(y_shared), static_cast<const uint4*>(combine_buffer), topk_weights, static_cast<uint4*>(out),
        num_local_tokens, vec, topk, status);
    MOK_LAUNCH_CHECK("fwd_epilogue_kernel");
    return MOK_OK;
}

extern "C" int mok_bwd_epilogue(const void* d_x_shared, const void* d_x_routed_buffer, void* out, int64_t num_local_tokens,
                                int hidden, int topk, const uint32_t* status, mok_stream_t stream) {
    using namespace mok;
    if (d_x_routed_buffer == nullptr || out == nullptr || num_local_tokens <= 0 || hidden <= 0 || hidden % 8 != 0 || topk <= 0)
        return MOK_ERR_INVALID_ARGUMENT;
    const int vec = hidden / 8;
    const int grid = stream_grid(num_local_tokens * vec, 256);
    epilogue_kernel<false><<<grid, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
        static_cast<const uint4*>(d_x_shared), static_cast<const uint4*>(d_x_routed_buffer), nullptr, static_cast<uint4*>(out),
        num_local_tokens, vec, topk, status);
    MOK_LAUNCH_CHECK("bwd_epilogue_kernel");
    return MOK_OK;
}
