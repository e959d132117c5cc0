// Router in front of the MoE layer: logits = x * W^T (+ bias) in fp32, top-k, softmax over the selected logits
// (= renormalised top-k weights), and its backward.  The reference has no router - routes and weights are inputs
// there (README.md:128-129) and its tests draw them with torch.topk / softmax (tests/utils.py:82-84); this file
// produces exactly those two tensors on the device so that nothing between the previous layer and the schedule
// leaves the GPU or goes through int64.
//
//   forward : logits [T, E_pad] fp32 by the tcgen05 grouped GEMM (dense form, fp32 output, weight as hi + lo bf16)
//             -> one warp per token picks the k largest of the first E logits (ties: lower index), writes int32 routes
//             and fp32 weights
//   backward: d_v = w * (d_w - sum_j w_j d_w_j) scattered into a dense bf16 d_logits [T, E_pad] (zero elsewhere)
//             -> d_W = d_logits^T x (weight-gradient form, fp32 output), d_x = d_logits W (dgrad form), d_bias = column sums
#include "elementwise.cuh"
#include "grouped_gemm.cuh"

namespace mok {
namespace {

constexpr int kMaxRouterExperts = 1024;   // 32 logits per lane
constexpr int kMaxRouterTopk = 32;

// (value, index) order of torch.topk with ties broken towards the lower index
__device__ __forceinline__ bool better(float v, int i, float bv, int bi) { return v > bv || (v == bv && i < bi); }

template <int PER_LANE>
__global__ void __launch_bounds__(256) topk_softmax_kernel(const float* __restrict__ logits, const float* __restrict__ bias,
                                                            int tokens, int experts, int ld, int topk,
                                                            int32_t* __restrict__ routes, float* __restrict__ weights) {
    const int lane = threadIdx.x & 31;
    const int warps = (gridDim.x * blockDim.x) >> 5;
    for (int t = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; t < tokens; t += warps) {
        float v[PER_LANE];
#pragma unroll
        for (int j = 0; j < PER_LANE; ++j) {      // lane owns experts lane, lane + 32, ... : coalesced reads
            const int e = lane + 32 * j;
            v[j] = e < experts ? logits[static_cast<long long>(t) * ld + e] + (bias != nullptr ? bias[e] : 0.0f) : -INFINITY;
        }
        float top_v = 0.0f, sum = 0.0f, mine_v = 0.0f;
        int mine_e = 0;
        for (int k = 0; k < topk; ++k) {
            float bv = -INFINITY;
            int bi = 0x7fffffff;
#pragma unroll
            for (int j = 0; j < PER_LANE; ++j)
                if (better(v[j], lane + 32 * j, bv, bi)) { bv = v[j]; bi = lane + 32 * j; }
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) {
                const float ov = __shfl_xor_sync(0xffffffffu, bv, off);
                const int oi = __shfl_xor_sync(0xffffffffu, bi, off);
                if (better(ov, oi, bv, bi)) { bv = ov; bi = oi; }
            }
            if (k == 0) top_v = bv;
            const float ex = expf(bv - top_v);
            sum += ex;
            if (lane == k) { mine_v = ex; mine_e = bi; }      // lane k keeps the k-th choice
#pragma unroll
            for (int j = 0; j < PER_LANE; ++j)
                if (lane + 32 * j == bi) v[j] = -INFINITY;     // the winner leaves the pool
        }
        if (lane < topk) {
            routes[static_cast<long long>(t) * topk + lane] = mine_e;
            weights[static_cast<long long>(t) * topk + lane] = mine_v / sum;
        }
    }
}

// One warp per token: softmax backward over the selected logits, written as a dense bf16 row (zeros elsewhere).
__global__ void __launch_bounds__(256) router_scatter_kernel(const int32_t* __restrict__ routes, const float* __restrict__ weights,
                                                             const float* __restrict__ d_weights, int tokens, int topk, int ld,
                                                             bf16* __restrict__ d_logits) {
    const int lane = threadIdx.x & 31;
    const int warps = (gridDim.x * blockDim.x) >> 5;
    for (int t = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; t < tokens; t += warps) {
        const long long base = static_cast<long long>(t) * topk;
        const float w = lane < topk ? weights[base + lane] : 0.0f;
        const float dw = lane < topk ? d_weights[base + lane] : 0.0f;
        float dot = w * dw;
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, off);
        bf16* row = d_logits + static_cast<long long>(t) * ld;
        for (int c = lane * 8; c < ld; c += 256) *reinterpret_cast<uint4*>(row + c) = make_uint4(0, 0, 0, 0);
        __syncwarp();
        if (lane < topk) {
            const int e = routes[base + lane];
            if (e >= 0 && e < ld) row[e] = __float2bfloat16(w * (dw - dot));   // a route outside the matrix is ignored
        }
    }
}

// d_bias[e] = sum over tokens of d_logits[t, e]: block = 32 columns x 8 row phases, rows and phases in fixed order.
__global__ void __launch_bounds__(256) column_sum_kernel(const bf16* __restrict__ d_logits, int tokens, int experts, int ld,
                                                         float* __restrict__ d_bias) {
    __shared__ float part[8][32];
    const int col = blockIdx.x * 32 + (threadIdx.x & 31);
    const int phase = threadIdx.x >> 5;
    float acc = 0.0f;
    if (col < experts)
        for (int t = phase; t < tokens; t += 8) acc += __bfloat162float(d_logits[static_cast<long long>(t) * ld + col]);
    part[phase][threadIdx.x & 31] = acc;
    __syncthreads();
    if (phase == 0 && col < experts) {
        float s = 0.0f;
        for (int p = 0; p < 8; ++p) s += part[p][threadIdx.x & 31];
        d_bias[col] = s;
    }
}

GemmProblem dense_problem(int tokens, uint32_t* status) {
    GemmProblem p;
    p.num_experts = 1;
    p.dense_rows = tokens;
    p.row_begin = 0;
    p.row_end = tokens;
    p.buffer_rows = tokens;
    p.status = status;
    return p;
}

int warp_grid(int tokens) {
    long long blocks = (static_cast<long long>(tokens) + 7) / 8;
    const long long cap = static_cast<long long>(sm_count()) * 8;
    return static_cast<int>(blocks < cap ? blocks : cap);
}

}  // namespace
}  // namespace mok

extern "C" int mok_router_forward(const void* x, const void* w_hi, const void* w_lo, const float* bias, int64_t num_tokens,
                                  int hidden, int num_experts, int padded_experts, int topk, float* logits, int32_t* top_experts,
                                  float* router_weights, uint32_t* status, mok_stream_t stream) {
    using namespace mok;
    if (!x || !w_hi || !logits || !top_experts || !router_weights) return MOK_ERR_INVALID_ARGUMENT;
    if (num_tokens <= 0 || num_tokens % 256 != 0 || num_tokens > 0x7fffff00 || hidden <= 0 || hidden % 64 != 0)
        return MOK_ERR_INVALID_ARGUMENT;
    if (num_experts <= 0 || padded_experts < num_experts || padded_experts % 256 != 0) return MOK_ERR_INVALID_ARGUMENT;
    if (topk <= 0 || topk > num_experts || topk > kMaxRouterTopk) return MOK_ERR_INVALID_ARGUMENT;
    if (num_experts > kMaxRouterExperts) return MOK_ERR_TOO_LARGE;
    cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
    const int T = static_cast<int>(num_tokens);
    MOK_TRY(launch_rows_gemm_f32(dense_problem(T, status), x, hidden, w_hi, w_lo, logits, padded_experts, s));
    const int grid = warp_grid(T);
    const int per_lane = (num_experts + 31) / 32;
#define MOK_TOPK_CASE(N)                                                                                                   \
    topk_softmax_kernel<N><<<grid, 256, 0, s>>>(logits, bias, T, num_experts, padded_experts, topk, top_experts, router_weights)
    if (per_lane <= 1) MOK_TOPK_CASE(1);
    else if (per_lane <= 2) MOK_TOPK_CASE(2);
    else if (per_lane <= 4) MOK_TOPK_CASE(4);
    else if (per_lane <= 8) MOK_TOPK_CASE(8);
    else if (per_lane <= 16) MOK_TOPK_CASE(16);
    else MOK_TOPK_CASE(32);
#undef MOK_TOPK_CASE
    MOK_LAUNCH_CHECK("topk_softmax_kernel");
    return MOK_OK;
}

extern "C" int mok_router_backward(const void* x, const void* w_hi, const int32_t* top_experts, const float* router_weights,
                                   const float* d_router_weights, int64_t num_tokens, int hidden, int num_experts,
                                   int padded_experts, int topk, void* d_logits, void* d_x, float* d_w, float* d_bias,
                                   uint32_t* status, mok_stream_t stream) {
    using namespace mok;
    if (!x || !w_hi || !top_experts || !router_weights || !d_router_weights || !d_logits || !d_x || !d_w)
        return MOK_ERR_INVALID_ARGUMENT;
    if (num_tokens <= 0 || num_tokens % 256 != 0 || num_tokens > 0x7fffff00 || hidden <= 0 || hidden % 256 != 0)
        return MOK_ERR_INVALID_ARGUMENT;
    if (num_experts <= 0 || padded_experts < num_experts || padded_experts % 256 != 0) return MOK_ERR_INVALID_ARGUMENT;
    if (topk <= 0 || topk > num_experts || topk > kMaxRouterTopk) return MOK_ERR_INVALID_ARGUMENT;
    cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
    const int T = static_cast<int>(num_tokens);
    router_scatter_kernel<<<warp_grid(T), 256, 0, s>>>(top_experts, router_weights, d_router_weights, T, topk, padded_experts,
                                                       static_cast<bf16*>(d_logits));
    MOK_LAUNCH_CHECK("router_scatter_kernel");
    const GemmProblem p = dense_problem(T, status);
    // d_W [E_pad, H] = d_logits^T x (fp32 out);  d_x [T, H] = d_logits W  (W is [E_pad, H]: K = E_pad, N = H)
    MOK_TRY(launch_wgrad_gemm(p, d_logits, padded_experts, x, hidden, d_w, s, true));
    MOK_TRY(launch_rows_gemm(p, d_logits, padded_experts, w_hi, nullptr, d_x, nullptr, hidden, true, s));
    if (d_bias != nullptr) {
        column_sum_kernel<<<(num_experts + 31) / 32, 256, 0, s>>>(static_cast<const bf16*>(d_logits), T, num_experts, padded_experts,
                                                                  d_bias);
        MOK_LAUNCH_CHECK("column_sum_kernel");
    }
    return MOK_OK;
}
