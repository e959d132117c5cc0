/*
 * C ABI of the B200 (sm_100a) expert-parallel MoE layer library, libmok_b200.so.
 *
 * Every entry point takes raw device pointers, sizes and a CUDA stream, enqueues work on that
 * stream and returns immediately: 0 on success, a negative MOK_ERR_* code when an argument is
 * rejected or a launch fails.  Nothing here allocates device memory, synchronises with the host
 * or throws.  Device-side problems (schedule overflow, a wait that ran out) are reported through
 * the caller-provided `status` word (MOK_STATUS_* bits), which the host may read whenever it likes.
 *
 * Each function names the interface of the reference project it stands in for (paths are inside
 * that project).  Peer pointer arrays hold one device virtual address per expert-parallel rank,
 * as `torch.distributed._symmetric_memory` hands them out (mok/functional.py:211-225).
 */
#ifndef MOK_B200_H
#define MOK_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct CUstream_st* mok_stream_t;

enum {
    MOK_OK = 0,
    MOK_ERR_INVALID_ARGUMENT = -1,
    MOK_ERR_UNSUPPORTED = -2,
    MOK_ERR_CUDA = -3,
    MOK_ERR_TOO_LARGE = -4
};

/* bits of the device status word */
enum {
    MOK_STATUS_SCHEDULE_OVERFLOW = 1u,   /* padded routes exceed schedule_capacity; rows beyond it were dropped */
    MOK_STATUS_BARRIER_TIMEOUT = 2u,     /* a cross-GPU barrier wait ran out */
    MOK_STATUS_PIPELINE_TIMEOUT = 4u,    /* an mbarrier wait inside a GEMM kernel ran out */
    MOK_STATUS_BAD_SCHEDULE_ENTRY = 8u   /* a schedule row named a peer or token outside the buffers (skipped) */
};

#define MOK_MAX_EP 8
#define MOK_MAX_LOCAL_EXPERTS 1024

/* Library/ABI version (major*100+minor); also proves the library loaded. */
int mok_version(void);

/* Last CUDA error string seen by this library on the calling thread ("" if none). */
const char* mok_last_error(void);

/* Kernels this library has launched in this process so far (all threads). */
long long mok_launch_count(void);

/* Debugging aid: with MOK_TRACE=1 in the environment the layer entry points time their phases (pull / compute /
 * push per chunk, wgrad, shared expert) with CUDA events; this call synchronises the device, writes one line per
 * phase ("name chunk stream start_ms end_ms") to `path` and clears the record. */
int mok_trace_dump(const char* path);

/* Bytes of int32 scratch `mok_schedule` needs for these sizes. */
int64_t mok_schedule_scratch_bytes(int ep_size, int num_local_tokens, int topk, int num_local_experts);

/*
 * Builds this rank's padded per-expert receive schedule from the all-gathered routes.
 * Replaces: scheduler::schedule_entrypoint, csrc/scheduler.cuh:149-183 (count/pad/schedule kernels :35-147);
 * op `mok::schedule`, mok/ops.py:109-156.  Ordering contract: csrc/scheduler.cuh:134-139.
 *   topk_all            int32 [ep, T, K]
 *   peer_rank           int32 [cap]   (-1 on padding rows)
 *   peer_token_idx      int32 [cap]   (token*K + k on the source rank; -1 on padding rows)
 *   num_tokens          int32 [1]     padded total
 *   tokens_per_expert   int32 [E_loc] each padded to 256
 *   scratch             mok_schedule_scratch_bytes() bytes
 *   status              uint32 [1], OR-ed with MOK_STATUS_SCHEDULE_OVERFLOW instead of trapping (csrc/scheduler.cuh:86)
 */
int mok_schedule(const int32_t* topk_all, int ep_size, int num_local_tokens, int topk,
                 int num_local_experts, int schedule_capacity, int rank,
                 int32_t* peer_rank, int32_t* peer_token_idx, int32_t* num_tokens,
                 int32_t* tokens_per_expert, int32_t* scratch, uint32_t* status, mok_stream_t stream);

/*
 * Same result as mok_schedule, for callers that must not allocate device memory around the call: a serving
 * process whose memory pool is frozen after start-up, or a plugin running under another framework's allocator
 * lock.  It has no counterpart in the reference project.  The scratch is a fixed array inside the library (MOK_SCHEDULE_STATIC_SCRATCH_BYTES on every
 * GPU that loads the library, held until process exit), so:
 *   - sizes with mok_schedule_scratch_bytes() above that limit are rejected with MOK_ERR_TOO_LARGE;
 *   - the first call on each device looks up the array's device address; make that first call outside any
 *     stream capture;
 *   - all calls on one GPU share the array: two calls that may overlap on the GPU (different streams) race.
 * Neither this function nor anything it launches calls cudaMalloc / cudaFree.
 */
#define MOK_SCHEDULE_STATIC_SCRATCH_BYTES (4 * 1024 * 1024)
int mok_schedule_static(const int32_t* topk_all, int ep_size, int num_local_tokens, int topk,
                        int num_local_experts, int schedule_capacity, int rank,
                        int32_t* peer_rank, int32_t* peer_token_idx, int32_t* num_tokens,
                        int32_t* tokens_per_expert, uint32_t* status, mok_stream_t stream);

/*
 * Extends a finished schedule for de-duplicated dispatch: a token that several local experts use is pulled from its
 * source rank once and fanned out locally, instead of once per schedule row as the reference's dispatch does
 * (csrc/megakernel/dispatch_combine.cuh:74-77 pulls per row; the reference has no counterpart of this call).
 *   row_source     int32 [cap]            number of the row's token among the staged tokens, -1 on padding rows
 *   unique_peer    int32 [max_unique]     source rank of staged token u (numbered in the order of their first row)
 *   unique_token   int32 [max_unique]     its token index on that rank
 *   unique_before  int32 [cap / 256 + 1]  staged tokens whose first row lies below row 256 * i
 *   num_unique     int32 [1]
 *   scratch        mok_schedule_dedup_scratch_bytes() bytes
 * max_unique >= min(cap, ep_size * num_local_tokens) always suffices.
 */
int64_t mok_schedule_dedup_scratch_bytes(int ep_size, int num_local_tokens, int topk, int schedule_capacity);
int mok_schedule_dedup(const int32_t* topk_all, int ep_size, int num_local_tokens, int topk, int num_local_experts,
                       int schedule_capacity, int rank, const int32_t* peer_rank, const int32_t* peer_token_idx,
                       const int32_t* num_tokens, int32_t* row_source, int32_t* unique_peer, int32_t* unique_token,
                       int32_t* unique_before, int32_t* num_unique, int max_unique, int32_t* scratch, mok_stream_t stream);

/*
 * The two steps of a de-duplicated dispatch, exposed for tests and for hosts that drive the pieces themselves.
 * mok_stage_unique_rows: staged[u, :] = src_ptrs[unique_peer[u]][unique_token[u], :] for the staged tokens first used
 * by schedule rows [from_row, min(to_row, *num_tokens)) (multiples of 256), except this rank's own tokens.
 * mok_dispatch_rows_staged: mok_dispatch_rows, with the rows of other ranks' tokens read from `staged`.
 */
int mok_stage_unique_rows(const uint64_t* src_ptrs, int ep_size, int rank, const int32_t* unique_peer,
                          const int32_t* unique_token, const int32_t* unique_before, const int32_t* num_tokens,
                          int from_row, int to_row, int num_local_tokens, int hidden, void* staged, int staged_rows,
                          int num_ctas, uint32_t* status, mok_stream_t stream);
int mok_dispatch_rows_staged(const uint64_t* src_ptrs, const uint64_t* weight_ptrs, int ep_size, int rank,
                             const int32_t* peer_rank, const int32_t* peer_token_idx, const int32_t* num_tokens,
                             const int32_t* row_source, const void* staged, int staged_rows, int row_begin, int row_end,
                             int topk, int num_local_tokens, int hidden, void* dst, float* row_weight, int num_ctas,
                             uint32_t* status, mok_stream_t stream);

/*
 * Copies this rank's int32 routes [T*K] into slot `rank` of the [ep, T, K] buffer of every peer.
 * Replaces: all_gather_top_experts_kernel, csrc/utils.cuh:191-227 (op mok/ops.py:6-61).  Peers are
 * addressed one by one through `peer_buffers` (unicast stores); no multicast object is needed.
 */
int mok_all_gather_top_experts(const int32_t* top_experts, int64_t num_routes, const uint64_t* peer_buffers,
                               int ep_size, int rank, mok_stream_t stream);

/*
 * Device-side barrier across the EP ranks.  Replaces: barrier_all_kernel, csrc/utils.cuh:229-299
 * (op mok/ops.py:64-106).  `target` (int32 [1], local) is advanced by ep_size, every peer's counter
 * receives +1 with release/system semantics, then the local counter is polled until it reaches the
 * target.  The poll is bounded (`timeout_ms`, 0 = default 20 s): on expiry MOK_STATUS_BARRIER_TIMEOUT is
 * set and the kernel returns.
 */
int mok_barrier_all(int32_t* local_counter, const uint64_t* peer_counters, int ep_size, int32_t* target,
                    uint32_t* status, int timeout_ms, mok_stream_t stream);

/*
 * Token dispatch alone: dst[row - row_begin, :] = src_ptrs[peer_rank[row]][peer_token_idx[row] / topk, :] for schedule
 * rows [row_begin, min(row_end, *num_tokens)); padding rows become zeros.  With weight_ptrs != NULL each row is
 * multiplied by the fp32 router weight weight_ptrs[peer][peer_token_idx[row]] (rounded to bf16) and the weight is
 * stored in row_weight.  Replaces: dispatch_kernel, csrc/megakernel/dispatch_combine.cuh:1-150, and
 * preload_router_weights_kernel, csrc/megakernel/utils.cuh:15-48.  num_ctas <= 0 fills the GPU.
 */
int mok_dispatch_rows(const uint64_t* src_ptrs, const uint64_t* weight_ptrs, int ep_size, const int32_t* peer_rank,
                      const int32_t* peer_token_idx, const int32_t* num_tokens, int row_begin, int row_end, int topk,
                      int num_local_tokens, int hidden, void* dst, float* row_weight, int num_ctas, uint32_t* status,
                      mok_stream_t stream);

/*
 * Combine alone: dst_ptrs[peer_rank[row]][peer_token_idx[row], :] = src[row - row_begin, :] for non-padding rows, and
 * with row_scalar != NULL also scalar_ptrs[peer][peer_token_idx[row]] = row_scalar[row - row_begin].  Every route owns
 * its slot, so no atomics and no ordering dependence.  Replaces: combine_kernel, dispatch_combine.cuh:152-266.
 */
int mok_combine_rows(const uint64_t* dst_ptrs, const uint64_t* scalar_ptrs, int ep_size, const int32_t* peer_rank,
                     const int32_t* peer_token_idx, const int32_t* num_tokens, int row_begin, int row_end, int topk,
                     int num_local_tokens, int hidden, const void* src, const float* row_scalar, int num_ctas,
                     uint32_t* status, mok_stream_t stream);

/*
 * out[t] = bf16(y_shared[t] + sum_k w[t,k] * combine[t*K+k]) with k ascending in fp32.
 * Replaces: fwd_epilogue_kernel, csrc/utils.cuh:43-95 (op mok/ops.py:1279-1313).  y_shared may be NULL (treated as 0).
 * `status` (may be NULL) is the device status word of the layer calls: when it holds any MOK_STATUS_* bit the routed
 * slots cannot be trusted (the reference traps in that situation, csrc/scheduler.cuh:86) and `out` is filled with NaN.
 */
int mok_fwd_epilogue(const void* y_shared, const void* combine_buffer, const float* topk_weights, void* out,
                     int64_t num_local_tokens, int hidden, int topk, const uint32_t* status, mok_stream_t stream);

/*
 * d_x[t] = bf16(d_x_shared[t] + sum_k d_x_routed[t*K+k]).  Replaces: bwd_epilogue_kernel,
 * csrc/utils.cuh:140-176 (op mok/ops.py:1316-1349).  d_x_shared may be NULL.  `status` as for mok_fwd_epilogue.
 */
int mok_bwd_epilogue(const void* d_x_shared, const void* d_x_routed_buffer, void* out,
                     int64_t num_local_tokens, int hidden, int topk, const uint32_t* status, mok_stream_t stream);

/*
 * bf16 [E, M, N] -> e4m3 + e8m0 scale per 32 elements along the row, optionally also of the transpose.
 * Replaces: mxfp8::quantize_kernel, csrc/mxfp8.cuh:188-280 (op mok/ops.py:159-197).  Scale bytes go to the
 * [rows/128, cols/128, 32, 16] tensor-core layout (csrc/mxfp8.cuh:181-184).  Any of the four outputs may be
 * NULL in pairs (fp8, sc) / (fp8_t, sc_t).
 */
int mok_mxfp8_quantize(const void* x_bf16, int num_matrices, int rows, int cols,
                       void* x_fp8, void* x_sc, void* x_fp8_t, void* x_sc_t, mok_stream_t stream);

/* Arguments shared by the fused-layer entry points below.  All tensor pointers are device pointers;
 * bf16 unless stated.  Pointers not needed by a call may be NULL where noted. */
typedef struct mok_layer_args {
    /* sizes */
    int ep_size, rank;
    int num_local_tokens;      /* T */
    int hidden;                /* H */
    int intermediate;          /* I */
    int num_local_experts;     /* E_loc */
    int topk;                  /* K */
    int schedule_capacity;     /* rows of the schedule arrays */
    int macrobatch_size;       /* rows of the routed activation buffers */
    int minibatch_size;
    int num_comm_sms;
    int has_swiglu_limit;
    float swiglu_limit;
    int reserved0;
    /* schedule (mok_schedule outputs) */
    const int32_t* peer_rank;
    const int32_t* peer_token_idx;
    const int32_t* num_tokens;
    const int32_t* tokens_per_expert;
    /* this rank's own token-major inputs (what x_ptrs[rank] / d_y_ptrs[rank] point at) */
    const void* x_local;                  /* [T, H] */
    const void* d_y_local;                /* [T, H] (backward) */
    /* symmetric buffers: one address per rank */
    const uint64_t* x_ptrs;               /* [T, H] */
    const uint64_t* combine_ptrs;         /* [T*K, H] (forward) */
    const uint64_t* d_y_ptrs;             /* [T, H] (backward) */
    const uint64_t* d_x_routed_ptrs;      /* [T*K, H] (backward) */
    const uint64_t* router_weight_ptrs;   /* fp32 [T, K] (backward) */
    const uint64_t* d_router_weight_ptrs; /* fp32 [T, K] (backward) */
    /* weights; shared ones may be NULL = no shared expert */
    const void *w_shared_gate, *w_shared_up, *w_shared_down;   /* [I,H] [I,H] [H,I] */
    const void *w_routed_gate, *w_routed_up, *w_routed_down;   /* [E,I,H] [E,I,H] [E,H,I] */
    /* activations: forward writes, backward reads (and overwrites when it replays later macrobatches) */
    void *x_routed;        /* [MB, H] */
    void *gate_shared, *up_shared, *hidden_shared;   /* [T, I] */
    void *gate_routed, *up_routed, *hidden_routed;   /* [MB, I] */
    void *y_shared;        /* [T, H]  forward out */
    void *y_routed;        /* [MB, H] forward out */
    /* backward outputs / scratch */
    void *d_x_shared;      /* [T, H] */
    void *d_x_routed;      /* [MB, H] */
    void *d_gate_shared, *d_up_shared, *d_hidden_shared;   /* [T, I] */
    void *d_gate_routed, *d_up_routed, *d_hidden_routed;   /* [MB, I] */
    void *d_y_routed;      /* [MB, H] */
    void *d_w_shared_gate, *d_w_shared_up, *d_w_shared_down;
    void *d_w_routed_gate, *d_w_routed_up, *d_w_routed_down;
    float* row_scratch;    /* 4-byte words (backward): fp32 router weight [MB] and router-weight gradient [MB] of every
                              row, int32 occupied rows of every expert [num_local_experts], and for the MXFP8 backward
                              fp32 partial sums [MB * intermediate / 128] */
    uint32_t* status;      /* uint32 [1] */
    /* MXFP8 entry points only (NULL otherwise).  "fp8" = e4m3 bytes, "sc" = e8m0 scale tiles [rows/128, cols/128, 32, 16]
     * of the matrix as stored (scales along its last dimension).  In the MXFP8 calls the bf16 routed activation
     * fields above (x_routed ... d_x_routed) are scratch of the same shapes. */
    const void *w_gate_fp8, *w_gate_sc, *w_up_fp8, *w_up_sc, *w_down_fp8, *w_down_sc;   /* [E,I,H] [E,I,H] [E,H,I] */
    const void *w_gate_t_fp8, *w_gate_t_sc, *w_up_t_fp8, *w_up_t_sc;                     /* transposes [E,H,I] (backward) */
    const void *w_down_t_fp8, *w_down_t_sc;                                              /* transpose [E,I,H] (backward) */
    void *x_fp8, *x_sc;                             /* [MB,H] scratch */
    void *x_fp8_t, *x_sc_t;                         /* [H,MB] saved context */
    void *gate_fp8, *gate_sc, *up_fp8, *up_sc;      /* [MB,I] saved context */
    void *hidden_fp8, *hidden_sc;                   /* [MB,I] scratch */
    void *hidden_fp8_t, *hidden_sc_t;               /* [I,MB] saved context */
    void *d_y_fp8, *d_y_sc;                         /* [MB,H] backward out */
    void *d_y_fp8_t, *d_y_sc_t;                     /* [H,MB] scratch */
    void *d_gate_fp8, *d_gate_sc, *d_up_fp8, *d_up_sc;              /* [MB,I] backward out */
    void *d_gate_fp8_t, *d_gate_sc_t, *d_up_fp8_t, *d_up_sc_t;      /* [I,MB] scratch */
    /* De-duplicated dispatch (all NULL / 0 = every schedule row pulls its token itself).  The four index arrays are
     * mok_schedule_dedup outputs; the staging buffers are caller-provided scratch of staged_rows x H bf16: staged_x for
     * the forward / recompute calls and for the backward replay of later macrobatches, staged_d_y for the backward. */
    const int32_t *row_source, *unique_peer, *unique_token, *unique_before;
    void *staged_x, *staged_d_y;
    int staged_rows;
    int reserved1;
} mok_layer_args;

/*
 * BF16 forward: dispatch -> gate/up GEMM -> SwiGLU -> down GEMM -> combine, macrobatches last to first,
 * plus the shared expert.  Replaces: dispatch_mlp_swiglu_combine_fwd_bf16, csrc/megakernel/forward.cuh:293-428
 * (binding csrc/bindings.cu, op mok/ops.py:377-520).
 */
int mok_moe_forward_bf16(const mok_layer_args* args, mok_stream_t stream);

/*
 * BF16 forward without down projection / combine, macrobatch 0 only: rebuilds the saved context.
 * Replaces: recompute_forward_context_bf16, csrc/megakernel/recompute_forward_context.cuh (op mok/ops.py:668-782).
 */
int mok_moe_recompute_bf16(const mok_layer_args* args, mok_stream_t stream);

/*
 * BF16 backward: dgrad and wgrad of routed and shared experts, router-weight gradient, reverse dispatch/combine.
 * Replaces: dispatch_mlp_swiglu_combine_bwd_bf16, csrc/megakernel/backward.cuh:445-679 (op mok/ops.py:1079-1276),
 * including zero_empty_routed_wgrads (csrc/utils.cuh:301-322).
 */
int mok_moe_backward_bf16(const mok_layer_args* args, mok_stream_t stream);

/*
 * MXFP8 forward / context recomputation / backward: routed experts in e4m3 with e8m0 scales per 32 elements along K
 * (block-scaled tensor-core MMA), shared expert in bf16.  Activations are quantized where the reference quantizes
 * them: x after dispatch (normal for the gate/up GEMM, transposed for wgrad), gate and up after their GEMM (saved for
 * backward), hidden after SwiGLU (normal for the down GEMM, transposed for wgrad), d_y*w after dispatch, d_gate / d_up
 * after SwiGLU backward.  Replace: dispatch_mlp_swiglu_combine_fwd_mxfp8 (csrc/megakernel/forward.cuh:293-428,
 * op mok/ops.py:200-374), recompute_forward_context_mxfp8 (op mok/ops.py:523-665),
 * dispatch_mlp_swiglu_combine_bwd_mxfp8 (csrc/megakernel/backward.cuh:681-873, op mok/ops.py:785-1076).
 */
int mok_moe_forward_mxfp8(const mok_layer_args* args, mok_stream_t stream);
int mok_moe_recompute_mxfp8(const mok_layer_args* args, mok_stream_t stream);
int mok_moe_backward_mxfp8(const mok_layer_args* args, mok_stream_t stream);

/*
 * One grouped GEMM launch, exposed for tests and profiling.  D[rows, N] = A[rows, K] * B[e]^T with rows grouped
 * by `tokens_per_expert` (each a multiple of 256).  b_is_kn = 0: B is [E, N, K] (forward form, csrc/megakernel/
 * grouped_gemm.cuh mm2_ABt); 1: B is [E, K, N] (dgrad form, mm2_AB).  tokens_per_expert may be NULL for a dense
 * problem with `rows` rows and E = 1.
 */
int mok_grouped_gemm_bf16(const void* A, const void* B, void* D, const int32_t* tokens_per_expert,
                          const int32_t* num_tokens, int num_experts, int rows, int N, int K, int b_is_kn,
                          uint32_t* status, mok_stream_t stream);

/*
 * Weight-gradient form: D[e] [M, N] = A[rows_e, M]^T * B[rows_e, N] over the rows of expert e, in schedule order
 * (fixed reduction order).  Replaces the mm2_AtB use of csrc/megakernel/grouped_gemm.cuh:153-167,241-243.
 */
int mok_grouped_wgrad_bf16(const void* A, const void* B, void* D, const int32_t* tokens_per_expert,
                           const int32_t* num_tokens, int num_experts, int rows, int M, int N,
                           uint32_t* status, mok_stream_t stream);

/*
 * MXFP8 grouped GEMM, one launch: D[rows, N] (bf16) = A[rows, K] * B[e]^T with A, B in e4m3 and e8m0 scales per 32
 * elements along K in the [rows/128, K/128, 32, 16] layout that mok_mxfp8_quantize writes; B is [E, N, K] with
 * scales [E*N/128, K/128, 32, 16].  Replaces the MXFP8 form of expert_grouped_gemm_kernel
 * (csrc/megakernel/grouped_gemm.cuh:222-249, block-scaled mm2_ABt).  rows, N multiples of 256; K of 128.
 */
int mok_grouped_gemm_mxfp8(const void* A_fp8, const void* A_sc, const void* B_fp8, const void* B_sc, void* D,
                           const int32_t* tokens_per_expert, const int32_t* num_tokens, int num_experts, int rows,
                           int N, int K, uint32_t* status, mok_stream_t stream);

/*
 * MXFP8 weight-gradient form: D[e] [M, N] (bf16) = At[:, rows_e] * Bt[:, rows_e]^T where At [M, rows] and Bt [N, rows]
 * are transposed-quantized activations (scales along the row dimension of the schedule).  Replaces the MXFP8 wgrad
 * use of the reference grouped GEMM (csrc/megakernel/backward.cuh:369-403).
 */
int mok_grouped_wgrad_mxfp8(const void* At_fp8, const void* At_sc, const void* Bt_fp8, const void* Bt_sc, void* D,
                            const int32_t* tokens_per_expert, const int32_t* num_tokens, int num_experts, int rows,
                            int M, int N, uint32_t* status, mok_stream_t stream);

/*
 * Router in front of the layer.  No counterpart among the reference's operators: there the routes and router weights
 * are inputs that the caller computes (README.md:128-129; its tests use torch.topk and a softmax over the selected
 * logits, tests/utils.py:82-84).  These two entry points compute exactly those tensors, and their gradient, on the
 * device.
 *
 * forward:  logits [T, padded_experts] fp32 (scratch / output) = x [T, H] bf16 * (w_hi + w_lo)^T, with the weight
 *           given as one or two bf16 terms [padded_experts, H] (w_lo may be NULL; rows >= num_experts must be zero);
 *           top_experts int32 [T, topk] = indices of the topk largest of logits[:, :num_experts] + bias, descending,
 *           ties towards the lower index; router_weights fp32 [T, topk] = softmax over those topk values.
 *           T % 256 == 0, H % 64 == 0, padded_experts % 256 == 0, num_experts <= 1024, topk <= 32.
 * backward: d_logits bf16 [T, padded_experts] (scratch / output) = softmax backward of d_router_weights scattered to
 *           the selected columns; d_w fp32 [padded_experts, H] = d_logits^T x; d_x bf16 [T, H] = d_logits * w_hi;
 *           d_bias fp32 [num_experts] (may be NULL) = column sums of d_logits.  H % 256 == 0.
 */
int mok_router_forward(const void* x, const void* w_hi, const void* w_lo, const float* bias, int64_t num_tokens, int hidden,
                       int num_experts, int padded_experts, int topk, float* logits, int32_t* top_experts,
                       float* router_weights, uint32_t* status, mok_stream_t stream);
int mok_router_backward(const void* x, const void* w_hi, const int32_t* top_experts, const float* router_weights,
                        const float* d_router_weights, int64_t num_tokens, int hidden, int num_experts, int padded_experts,
                        int topk, void* d_logits, void* d_x, float* d_w, float* d_bias, uint32_t* status, mok_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* MOK_B200_H */
