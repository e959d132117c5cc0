// Host-side interface of the dispatch / combine kernels (comm.cu).
#pragma once

#include "mok_common.cuh"

namespace mok {

// A window of schedule rows [row_begin, min(row_end, *num_tokens)); local buffers are indexed by row - row_begin.
struct RowWindow {
    const int32_t* peer_rank;
    const int32_t* peer_token;
    const int32_t* num_tokens;
    int row_begin, row_end;
    uint32_t* status;
};

// dst[row - row_begin, :] = src_ptrs[peer_rank[row]][peer_token[row] / topk, :]; padding rows become zeros.
// With weight_ptrs != nullptr every row is multiplied by the fp32 weight weight_ptrs[peer][peer_token[row]]
// (rounded to bf16) and the weight is also written to row_weight[row - row_begin] (0 on padding rows).
// num_ctas <= 0 lets the launch fill the GPU.
int launch_dispatch(const uint64_t* src_ptrs, const uint64_t* weight_ptrs, int ep, const RowWindow& w, int topk,
                    int tokens_per_rank, int hidden, void* dst, float* row_weight, int num_ctas, cudaStream_t stream);

// dst_ptrs[peer_rank[row]][peer_token[row], :] = src[row - row_begin, :] for non-padding rows; with row_scalar
// != nullptr also scalar_ptrs[peer][peer_token[row]] = row_scalar[row - row_begin].
int launch_combine(const uint64_t* dst_ptrs, const uint64_t* scalar_ptrs, int ep, const RowWindow& w, int topk,
                   int tokens_per_rank, int hidden, const void* src, const float* row_scalar, int num_ctas,
                   cudaStream_t stream);

}  // namespace mok
