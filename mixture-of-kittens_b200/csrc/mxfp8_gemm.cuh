// Host-side interface of the block-scaled MXFP8 grouped GEMM (mxfp8_gemm.cu).
#pragma once

#include "grouped_gemm.cuh"

namespace mok {

// An MXFP8 operand: e4m3 bytes, K contiguous, plus e8m0 scales per 32 elements along K stored as 512-byte tiles
// [row tile of 128][K tile of 128] in the tensor-core scale layout (byte (r % 32) * 16 + (r / 32) * 4 + kblock).
struct Fp8Operand {
    const void* data = nullptr;      // first row of the operand (of expert 0 for weights)
    const void* scales = nullptr;    // scale tile of (row tile 0, K tile 0)
    long long ld = 0;                // bytes between rows of `data`
    long long rows = 0;              // addressable rows (all experts together for weights)
    long long k_extent = 0;          // addressable elements along K
    long long scale_row_tile_stride = 0;   // bytes between the scale tiles of consecutive row tiles
};

// D_s[row, :] = A[row, :K] * B_s[e]^T  (s < 2 when B1 is given); B_s is [E, N, K].  bf16 output.
int launch_fp8_rows_gemm(const GemmProblem& pb, const Fp8Operand& A, int K, const Fp8Operand& B0, const Fp8Operand* B1,
                         void* D0, void* D1, int N, cudaStream_t stream);

// D[row, :] = A0[row, :K] * B0[e]^T + A1[row, :K] * B1[e]^T.
int launch_fp8_rows_gemm_dual(const GemmProblem& pb, const Fp8Operand& A0, const Fp8Operand& A1, int K, const Fp8Operand& B0,
                              const Fp8Operand& B1, void* D, int N, cudaStream_t stream);

// Outputs of the fused gate / up projection: every pointer addresses the window's first row (the transposed matrix: its
// column), scale pointers its first 128-row tile.  Same conventions as launch_quantize_rows (mxfp8.cuh).
struct Fp8GateUpOut {
    void *gate_q = nullptr, *gate_sc = nullptr, *up_q = nullptr, *up_sc = nullptr;   // e4m3 [rows, N] + scale tiles
    void *hidden_q = nullptr, *hidden_sc = nullptr;                                   // silu(gate) * up, same layout
    void *hidden_qt = nullptr, *hidden_sct = nullptr;                                 // its transpose [N, buffer rows]
    long long sc_row_tile_stride = 0, qt_ld = 0, sct_row_tile_stride = 0;
    bool has_limit = false;
    float limit = 0.0f;
};

// gate = A * Wg[e]^T and up = A * Wu[e]^T in one accumulator (columns [0,128) / [128,256) of every tile), and in the
// epilogue what otherwise takes a bf16 round trip and a separate kernel: both are rounded to bf16 and quantized to
// MXFP8, hidden = silu(gate) * up is formed from the rounded values and quantized in both layouts.  Bitwise the same
// bytes as launch_fp8_rows_gemm followed by launch_swiglu_quantize_fwd.
int launch_fp8_gate_up_fused(const GemmProblem& pb, const Fp8Operand& A, int K, const Fp8Operand& Wg, const Fp8Operand& Wu, int N,
                             const Fp8GateUpOut& out, cudaStream_t stream);

// D[e] [M, N] (+)= At[:, rows_e] * Bt[:, rows_e]^T with At [M, rows] and Bt [N, rows] (transposed activations,
// K = schedule rows).  Column 0 of At / Bt is schedule row pb.row_begin.
int launch_fp8_wgrad_gemm(const GemmProblem& pb, const Fp8Operand& At, int M, const Fp8Operand& Bt, int N, void* D,
                          cudaStream_t stream);

}  // namespace mok
