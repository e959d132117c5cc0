// Host-side interface of the bandwidth-bound kernels (elementwise.cu).
#pragma once

#include "mok_common.cuh"

namespace mok {

// Rows are relative to the activation buffers: buffer row i holds schedule row row_begin + i, and only rows below
// min(row_end, *num_tokens) (or dense_rows when num_tokens == nullptr) are processed.
int launch_swiglu_fwd(const void* gate, const void* up, void* hidden, const int32_t* num_tokens, int dense_rows,
                      int row_begin, int row_end, int intermediate, bool has_limit, float limit, cudaStream_t stream);

// row_weight / row_grad (fp32 per buffer row) may be nullptr (shared expert: no router weight).
int launch_swiglu_bwd(const void* gate, const void* up, const void* d_hidden, void* d_gate, void* d_up,
                      const int32_t* num_tokens, int dense_rows, int row_begin, int row_end, int intermediate,
                      bool has_limit, float limit, const float* row_weight, float* row_grad, cudaStream_t stream);

// occupied[e] = rows of expert e up to and including its last row that carries a token (0 for an expert without
// tokens); the weight-gradient GEMMs stop their K loop there instead of running over the zero padding rows.
int launch_occupied_rows(const int32_t* peer_rank, const int32_t* tokens_per_expert, const int32_t* num_tokens,
                         int schedule_capacity, int num_experts, int32_t* occupied, cudaStream_t stream);

// Zeroes the three weight-gradient slices of every expert whose padded token count is 0.
int launch_zero_empty_wgrads(const int32_t* tokens_per_expert, int num_experts, void* a, void* b, void* c,
                             long long elems_per_expert, cudaStream_t stream);

}  // namespace mok
