// Token de-duplication for dispatch.
//
// A token whose top-k names several experts of one rank occupies several rows of that rank's schedule, and a dispatch
// that pulls row by row (reference csrc/megakernel/dispatch_combine.cuh:74-77) moves the token over NVLink once per
// row.  The kernels here extend a finished schedule with what a dispatch needs to move every token once per
// destination rank: the distinct (source rank, token) pairs a rank serves, numbered in the order of their first row
// ("staged" tokens), and for every schedule row the number of its token.  Dispatch then pulls the staged tokens into
// a local staging buffer and fans them out to the rows with local copies; the rows end up with exactly the bytes a
// row-by-row pull gives.
//
// Numbering by first row makes the staged tokens needed by rows [0, r) a prefix [0, unique_before[r / 256]) of the
// staging buffer, so the pull can proceed chunk by chunk in schedule order, overlapped with the GEMMs, with nothing
// but two prefix values read on the device.
#include "mok_common.cuh"

namespace mok {
namespace {

constexpr int kRowsPerBlock = 256;   // granularity of unique_before: every chunk / window boundary is a multiple

// inverse[peer * routes + route] = schedule row of that route (entries of routes not served here stay -1)
__global__ void inverse_kernel(const int* __restrict__ peer_rank, const int* __restrict__ peer_token,
                               const int* __restrict__ num_tokens, int capacity, int ep, int routes, int* __restrict__ inverse) {
    const int limit = min(*num_tokens, capacity);
    const int stride = gridDim.x * blockDim.x;
    for (int row = blockIdx.x * blockDim.x + threadIdx.x; row < limit; row += stride) {
        const int p = peer_rank[row], route = peer_token[row];
        if (p >= 0 && p < ep && route >= 0 && route < routes) inverse[static_cast<size_t>(p) * routes + route] = row;
    }
}

// first_row[row] = lowest schedule row that carries the same (source rank, token), -1 on padding rows;
// block_count[b] = rows of block b that are the first row of their token.
__global__ void __launch_bounds__(kRowsPerBlock) first_use_kernel(const int* __restrict__ topk_all, const int* __restrict__ peer_rank,
                                                                  const int* __restrict__ peer_token,
                                                                  const int* __restrict__ num_tokens, int capacity, int ep,
                                                                  int routes, int topk, int first_expert, int e_loc,
                                                                  const int* __restrict__ inverse, int* __restrict__ first_row,
                                                                  int* __restrict__ block_count) {
    const int limit = min(*num_tokens, capacity);
    const int row = blockIdx.x * kRowsPerBlock + threadIdx.x;
    int first = -1;
    if (row < limit) {
        const int p = peer_rank[row], route = peer_token[row];
        if (p >= 0 && p < ep && route >= 0 && route < routes) {
            first = row;
            const size_t token_routes = static_cast<size_t>(p) * routes + static_cast<size_t>(route / topk) * topk;
            for (int k = 0; k < topk; ++k) {
                const int e = topk_all[token_routes + k] - first_expert;
                if (e < 0 || e >= e_loc) continue;
                const int other = inverse[token_routes + k];
                if (other >= 0 && other < first) first = other;
            }
        }
    }
    if (row < capacity) first_row[row] = first;
    const int firsts = __syncthreads_count(first >= 0 && first == row);
    if (threadIdx.x == 0) block_count[blockIdx.x] = firsts;
}

// One block: unique_before[b] = sum of block_count[0 .. b), unique_before[blocks] = num_unique = the total.
__global__ void __launch_bounds__(1024) block_prefix_kernel(const int* __restrict__ block_count, int blocks,
                                                            int* __restrict__ unique_before, int* __restrict__ num_unique) {
    __shared__ int warp_sums[32];
    __shared__ int carry_sh;
    if (threadIdx.x == 0) carry_sh = 0;
    __syncthreads();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (int base = 0; base < blocks; base += blockDim.x) {
        const int b = base + threadIdx.x;
        const int v = b < blocks ? block_count[b] : 0;
        int incl = v;
#pragma unroll
        for (int off = 1; off < 32; off <<= 1) {
            const int n = __shfl_up_sync(0xffffffffu, incl, off);
            if (lane >= off) incl += n;
        }
        if (lane == 31) warp_sums[warp] = incl;
        __syncthreads();
        if (warp == 0) {
            int w = warp_sums[lane];
#pragma unroll
            for (int off = 1; off < 32; off <<= 1) {
                const int n = __shfl_up_sync(0xffffffffu, w, off);
                if (lane >= off) w += n;
            }
            warp_sums[lane] = w;
        }
        __syncthreads();
        const int before = carry_sh + (warp ? warp_sums[warp - 1] : 0) + incl - v;
        if (b < blocks) unique_before[b] = before;
        __syncthreads();
        if (threadIdx.x == blockDim.x - 1) carry_sh = before + v;
        __syncthreads();
    }
    if (threadIdx.x == 0) {
        unique_before[blocks] = carry_sh;
        num_unique[0] = carry_sh;
    }
}

// First rows take the next number of their block (in row order) and record their token; other rows get -1 for now.
__global__ void __launch_bounds__(kRowsPerBlock) number_kernel(const int* __restrict__ peer_rank, const int* __restrict__ peer_token,
                                                               const int* __restrict__ first_row,
                                                               const int* __restrict__ unique_before, int capacity, int topk,
                                                               int max_unique, int* __restrict__ row_source,
                                                               int* __restrict__ unique_peer, int* __restrict__ unique_token) {
    __shared__ int warp_sums[kRowsPerBlock / 32];
    const int row = blockIdx.x * kRowsPerBlock + threadIdx.x;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const bool is_first = row < capacity && first_row[row] == row;
    const unsigned ballot = __ballot_sync(0xffffffffu, is_first);
    if (lane == 0) warp_sums[warp] = __popc(ballot);
    __syncthreads();
    int before = unique_before[blockIdx.x];
    for (int w = 0; w < warp; ++w) before += warp_sums[w];
    const int u = before + __popc(ballot & ((1u << lane) - 1u));
    if (row >= capacity) return;
    if (is_first && u < max_unique) {
        row_source[row] = u;
        unique_peer[u] = peer_rank[row];
        unique_token[u] = peer_token[row] / topk;
    } else {
        row_source[row] = -1;
    }
}

// Every other row takes the number of its token's first row.
__global__ void propagate_kernel(const int* __restrict__ first_row, int capacity, int* __restrict__ row_source) {
    const int stride = gridDim.x * blockDim.x;
    for (int row = blockIdx.x * blockDim.x + threadIdx.x; row < capacity; row += stride) {
        const int first = first_row[row];
        if (first >= 0 && first != row) row_source[row] = row_source[first];   // written by number_kernel, never here
    }
}

}  // namespace
}  // namespace mok

extern "C" int64_t mok_schedule_dedup_scratch_bytes(int ep_size, int num_local_tokens, int topk, int schedule_capacity) {
    const int64_t routes = static_cast<int64_t>(num_local_tokens) * topk;
    const int64_t blocks = (schedule_capacity + mok::kRowsPerBlock - 1) / mok::kRowsPerBlock;
    return 4 * (ep_size * routes + schedule_capacity + blocks);
}

extern "C" int mok_schedule_dedup(const int32_t* topk_all, int ep_size, int num_local_tokens, int topk, int num_local_experts,
                                  int schedule_capacity, int rank, const int32_t* peer_rank, const int32_t* peer_token_idx,
                                  const int32_t* num_tokens, int32_t* row_source, int32_t* unique_peer, int32_t* unique_token,
                                  int32_t* unique_before, int32_t* num_unique, int max_unique, int32_t* scratch,
                                  mok_stream_t stream_) {
    using namespace mok;
    if (!topk_all || !peer_rank || !peer_token_idx || !num_tokens || !row_source || !unique_peer || !unique_token ||
        !unique_before || !num_unique || !scratch)
        return MOK_ERR_INVALID_ARGUMENT;
    if (ep_size < 1 || ep_size > MOK_MAX_EP || num_local_tokens <= 0 || topk <= 0 || num_local_experts <= 0 || rank < 0 ||
        rank >= ep_size || schedule_capacity <= 0 || schedule_capacity % kRowsPerBlock != 0 || max_unique <= 0)
        return MOK_ERR_INVALID_ARGUMENT;
    const int64_t routes64 = static_cast<int64_t>(num_local_tokens) * topk;
    if (routes64 * ep_size > (1LL << 30)) return MOK_ERR_TOO_LARGE;
    const int routes = static_cast<int>(routes64);
    const int blocks = schedule_capacity / kRowsPerBlock;
    cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
    int* inverse = scratch;
    int* first_row = inverse + static_cast<size_t>(ep_size) * routes;
    int* block_count = first_row + schedule_capacity;
    MOK_CUDA_CHECK(cudaMemsetAsync(inverse, 0xFF, sizeof(int) * static_cast<size_t>(ep_size) * routes, stream));
    const int wide = sm_count() * 4;
    inverse_kernel<<<wide, 256, 0, stream>>>(peer_rank, peer_token_idx, num_tokens, schedule_capacity, ep_size, routes, inverse);
    MOK_LAUNCH_CHECK("inverse_kernel");
    first_use_kernel<<<blocks, kRowsPerBlock, 0, stream>>>(topk_all, peer_rank, peer_token_idx, num_tokens, schedule_capacity,
                                                           ep_size, routes, topk, rank * num_local_experts, num_local_experts,
                                                           inverse, first_row, block_count);
    MOK_LAUNCH_CHECK("first_use_kernel");
    block_prefix_kernel<<<1, 1024, 0, stream>>>(block_count, blocks, unique_before, num_unique);
    MOK_LAUNCH_CHECK("block_prefix_kernel");
    number_kernel<<<blocks, kRowsPerBlock, 0, stream>>>(peer_rank, peer_token_idx, first_row, unique_before, schedule_capacity, topk,
                                                        max_unique, row_source, unique_peer, unique_token);
    MOK_LAUNCH_CHECK("number_kernel");
    propagate_kernel<<<wide, 256, 0, stream>>>(first_row, schedule_capacity, row_source);
    MOK_LAUNCH_CHECK("propagate_kernel");
    return MOK_OK;
}
