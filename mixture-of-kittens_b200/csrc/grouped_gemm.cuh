// Host-side interface of the tcgen05 grouped GEMM (grouped_gemm.cu), used by the fused-layer entry points.
#pragma once

#include "mok_common.cuh"

namespace mok {

// A grouped-GEMM problem over schedule rows.  Rows are grouped by expert: expert e owns the contiguous,
// 256-aligned row range [cum[e], cum[e+1]) given by `tokens_per_expert`; only rows inside the window
// [row_begin, min(row_end, *num_tokens)) are touched, and activation buffers are indexed by (row - row_begin)
// (the macrobatch ring).  A dense problem (one expert, `dense_rows` rows) has tokens_per_expert == nullptr.
struct GemmProblem {
    const int32_t* tokens_per_expert = nullptr;
    const int32_t* num_tokens = nullptr;
    int num_experts = 1;
    int dense_rows = 0;
    int row_begin = 0, row_end = 0;
    int buffer_rows = 0;   // rows of the activation buffers (macrobatch size, or T for a dense problem)
    // optional, weight-gradient form only: rows of each expert that can be non-zero (the rest of its 256-aligned range
    // is zero padding); the K loop of expert e ends at this count rounded up to the K step
    const int32_t* occupied_rows = nullptr;
    uint32_t* status = nullptr;
};

// D_s[row, :] = A[row, :K] * B_s[e]^T for s < n_sets (two sets share A: gate and up projections).
// b_is_kn = false: B_s is [E, N, K];  true: B_s is [E, K, N].
int launch_rows_gemm(const GemmProblem& pb, const void* A, int K, const void* B0, const void* B1, void* D0, void* D1,
                     int N, bool b_is_kn, cudaStream_t stream);

// Forward gate and up projections with the SwiGLU in the epilogue: gate = A * Wg[e]^T, up = A * Wu[e]^T (both stored as
// bf16 [rows, N]) and hidden = silu(gate) * up computed from the stored (rounded) values, optionally clamped.
int launch_gate_up_fused(const GemmProblem& pb, const void* A, int K, const void* Wg, const void* Wu, void* gate, void* up,
                         void* hidden, int N, bool has_limit, float limit, cudaStream_t stream);

// D[row, :] = A0[row, :K] * B0[e] + A1[row, :K] * B1[e] with B_s stored [E, K, N] (gate+up input gradient).
int launch_rows_gemm_dual(const GemmProblem& pb, const void* A0, const void* A1, int K, const void* B0, const void* B1,
                          void* D, int N, cudaStream_t stream);

// D[e] [M, N] (+)= A[rows_e, M]^T * B[rows_e, N]; accumulates when expert e's rows began before row_begin.
// out_f32: D is fp32 and is overwritten (single-window problems only).
int launch_wgrad_gemm(const GemmProblem& pb, const void* A, int M, const void* B, int N, void* D, cudaStream_t stream,
                      bool out_f32 = false);

// fp32 D[row, :] = A[row, :K] * (B_hi[e] + B_lo[e])^T with B_* stored [E, N, K]; B_lo may be nullptr.  Two bf16 terms
// carry an fp32 weight matrix to about 16 mantissa bits, which the router logits need (fp32 accumulation throughout).
int launch_rows_gemm_f32(const GemmProblem& pb, const void* A, int K, const void* B_hi, const void* B_lo, float* D, int N,
                         cudaStream_t stream);

}  // namespace mok
