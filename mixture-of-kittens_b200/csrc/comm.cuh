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

// De-duplicated dispatch (see dedup.cu): the tokens a rank serves, numbered in the order of their first schedule row,
// are pulled once each into `staged` ([staged_rows, hidden] bf16, local) and the schedule rows read them from there.
// Tokens of this rank itself are never staged: their rows read the local input directly.
struct StagedTokens {
    const int32_t* row_source;      // [capacity] number of the row's token, -1 on padding rows
    const int32_t* unique_peer;     // [staged_rows] source rank of every staged token
    const int32_t* unique_token;    // [staged_rows] its token index on that rank
    const int32_t* unique_before;   // [capacity / 256 + 1] staged tokens first used by rows below 256 * i
    void* staged;
    int staged_rows;
    int self_rank;
};

// staged[u, :] = src_ptrs[unique_peer[u]][unique_token[u], :] for the tokens first used by schedule rows
// [from_row, min(to_row, *num_tokens)) (both multiples of 256), except tokens of this rank.
int launch_stage_tokens(const uint64_t* src_ptrs, int ep, const StagedTokens& t, const int32_t* num_tokens, int from_row, int to_row,
                        int tokens_per_rank, int hidden, int num_ctas, uint32_t* status, cudaStream_t stream);

// dst[row - row_begin, :] = src_ptrs[peer_rank[row]][peer_token[row] / topk, :]; padding rows become zeros.
// With weight_ptrs != nullptr every row is multiplied by the fp32 weight weight_ptrs[peer][peer_token[row]]
// (rounded to bf16) and the weight is also written to row_weight[row - row_begin] (0 on padding rows).
// num_ctas <= 0 lets the launch fill the GPU.  With `staged` the rows of other ranks' tokens are read from the staging
// buffer (the tokens must have been staged already) instead of the peers' memory; the result is the same.
int launch_dispatch(const uint64_t* src_ptrs, const uint64_t* weight_ptrs, int ep, const RowWindow& w, int topk,
                    int tokens_per_rank, int hidden, void* dst, float* row_weight, int num_ctas, cudaStream_t stream,
                    const StagedTokens* staged = nullptr);

// dst_ptrs[peer_rank[row]][peer_token[row], :] = src[row - row_begin, :] for non-padding rows; with row_scalar
// != nullptr also scalar_ptrs[peer][peer_token[row]] = row_scalar[row - row_begin].
int launch_combine(const uint64_t* dst_ptrs, const uint64_t* scalar_ptrs, int ep, const RowWindow& w, int topk,
                   int tokens_per_rank, int hidden, const void* src, const float* row_scalar, int num_ctas,
                   cudaStream_t stream);

}  // namespace mok
