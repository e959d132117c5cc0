// Fused-layer entry points: the launch sequences for the BF16 forward, context recomputation and backward of
// the expert-parallel MoE layer.  Everything is enqueued from the caller's stream; no host synchronisation.
//
// Routed activations live in buffers of `macrobatch_size` rows.  Schedule rows are processed in windows of that
// size ("macrobatches"); forward walks the windows last to first so that window 0's activations are what the
// buffers hold afterwards, and backward recomputes gate / up / hidden for windows >= 1 before using them
// (reference: csrc/megakernel/forward.cuh:117-129,202-209 and backward.cuh:147-176,296-329).
//
// Overlap of NVLink traffic with the GEMMs: a window is cut into chunks of eight minibatches.  Dispatch and
// combine kernels run on a second, internal stream with a bounded number of CTAs (`num_comm_sms` x 8; they need
// no shared memory, so they share SMs with the resident GEMM CTAs), the GEMM / SwiGLU kernels run on the
// caller's stream, and CUDA events at chunk granularity order them:
//     comm:  dispatch(c) ------> record d[c]            wait y[c] -> combine(c)
//     main:            wait d[c] -> GEMMs(c) -> record y[c]
// Dispatch runs two chunks ahead.  The internal stream is forked from and joined back into the caller's stream
// inside every call, so the caller sees ordinary stream semantics.  No kernel ever spins on another kernel.
#include <stdio.h>
#include <stdlib.h>

#include <vector>

#include "comm.cuh"
#include "elementwise.cuh"
#include "grouped_gemm.cuh"
#include "mxfp8.cuh"
#include "mxfp8_gemm.cuh"

namespace mok {
namespace {

constexpr int kMaxEvents = 512;
constexpr int kMinibatchesPerChunk = 8;

struct DeviceStreams {
    cudaStream_t comm = nullptr;
    cudaEvent_t events[kMaxEvents] = {};
    int next = 0;
    bool ready = false;
};

// One helper stream and an event pool per device, created on first use (single host thread per device).  The
// caller's stream must belong to the current device: the helper stream and the events are the current device's.
int streams_for_current_device(cudaStream_t caller, DeviceStreams** out) {
    static DeviceStreams table[16];
    int dev = 0, stream_dev = 0;
    MOK_CUDA_CHECK(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 16) return MOK_ERR_UNSUPPORTED;
    MOK_CUDA_CHECK(cudaStreamGetDevice(caller, &stream_dev));
    if (stream_dev != dev) return MOK_ERR_INVALID_ARGUMENT;
    DeviceStreams& d = table[dev];
    if (!d.ready) {
        int least = 0, greatest = 0;
        MOK_CUDA_CHECK(cudaDeviceGetStreamPriorityRange(&least, &greatest));
        MOK_CUDA_CHECK(cudaStreamCreateWithPriority(&d.comm, cudaStreamNonBlocking, greatest));
        for (int i = 0; i < kMaxEvents; ++i) MOK_CUDA_CHECK(cudaEventCreateWithFlags(&d.events[i], cudaEventDisableTiming));
        d.ready = true;
    }
    *out = &d;
    return MOK_OK;
}

cudaEvent_t next_event(DeviceStreams* d) {
    cudaEvent_t e = d->events[d->next];
    d->next = (d->next + 1) % kMaxEvents;
    return e;
}

// make `waiter` wait for everything enqueued on `signaller` so far
int order_after(DeviceStreams* d, cudaStream_t signaller, cudaStream_t waiter) {
    cudaEvent_t e = next_event(d);
    MOK_CUDA_CHECK(cudaEventRecord(e, signaller));
    MOK_CUDA_CHECK(cudaStreamWaitEvent(waiter, e, 0));
    return MOK_OK;
}

// Forks the internal stream off the caller's stream and guarantees the join: if an entry point returns early (a
// launch failed part-way), work already queued on the internal stream may still read and write the caller's buffers,
// so the caller's stream is made to wait for it before control goes back (after a regular join this is a no-op wait).
struct CommFork {
    DeviceStreams* d = nullptr;
    cudaStream_t caller = nullptr;
    int start(cudaStream_t s, DeviceStreams** out) {
        MOK_TRY(streams_for_current_device(s, out));
        MOK_TRY(order_after(*out, s, (*out)->comm));
        d = *out;
        caller = s;
        return MOK_OK;
    }
    ~CommFork() {
        if (d == nullptr) return;
        cudaEvent_t e = next_event(d);
        if (cudaEventRecord(e, d->comm) == cudaSuccess) (void)cudaStreamWaitEvent(caller, e, 0);
    }
};

// ---- optional phase timeline (MOK_TRACE=1): CUDA events around every pull / compute / push / wgrad phase ---------
struct TraceRecord {
    const char* name;
    int chunk;
    int on_comm_stream;
    cudaEvent_t begin, end;
};
std::vector<TraceRecord>& trace_records() {
    static std::vector<TraceRecord> records;
    return records;
}
bool trace_enabled() {
    static const bool on = [] {
        const char* v = getenv("MOK_TRACE");
        return v != nullptr && v[0] == '1';
    }();
    return on;
}
int trace_begin(const char* name, int chunk, bool on_comm, cudaStream_t st) {
    if (!trace_enabled()) return -1;
    TraceRecord r{name, chunk, on_comm ? 1 : 0, nullptr, nullptr};
    if (cudaEventCreate(&r.begin) != cudaSuccess || cudaEventCreate(&r.end) != cudaSuccess) return -1;
    cudaEventRecord(r.begin, st);
    trace_records().push_back(r);
    return static_cast<int>(trace_records().size()) - 1;
}
void trace_end(int index, cudaStream_t st) {
    if (index >= 0) cudaEventRecord(trace_records()[index].end, st);
}

bool overlap_enabled() {
    const char* v = getenv("MOK_NO_OVERLAP");
    return !(v != nullptr && v[0] == '1');
}

// Rows handed from dispatch to the GEMMs to combine in one piece: kMinibatchesPerChunk minibatches, so the caller's
// minibatch_size sets the hand-over granularity (the default 4096 gives 32768-row chunks, the size that measured best
// on the DeepSeek-V3-shaped layer).  MOK_CHUNK_ROWS overrides the row count (rounded up to whole minibatches).
int chunk_rows_for(const mok_layer_args* a) {
    long long rows = static_cast<long long>(kMinibatchesPerChunk) * a->minibatch_size;
    if (const char* v = getenv("MOK_CHUNK_ROWS")) {
        const int r = atoi(v);
        if (r > 0) rows = r;
    }
    rows = (rows + a->minibatch_size - 1) / a->minibatch_size * a->minibatch_size;
    // never more than ~100 chunks per window: events and launches stay bounded
    const long long min_rows = (a->macrobatch_size / 100 + a->minibatch_size) / a->minibatch_size * a->minibatch_size;
    if (rows < min_rows) rows = min_rows;
    if (rows > a->macrobatch_size) rows = a->macrobatch_size;
    return static_cast<int>(rows);
}

int check_common(const mok_layer_args* a, bool fp8 = false) {
    if (a == nullptr) return MOK_ERR_INVALID_ARGUMENT;
    if (a->ep_size < 1 || a->ep_size > MOK_MAX_EP || a->rank < 0 || a->rank >= a->ep_size) return MOK_ERR_INVALID_ARGUMENT;
    if (a->num_local_tokens <= 0 || a->num_local_tokens % 256 != 0) return MOK_ERR_INVALID_ARGUMENT;
    if (a->hidden <= 0 || a->hidden % 256 != 0 || a->intermediate <= 0 || a->intermediate % 256 != 0)
        return MOK_ERR_INVALID_ARGUMENT;
    if (a->num_local_experts < 1) return MOK_ERR_INVALID_ARGUMENT;
    if (a->num_local_experts > MOK_MAX_LOCAL_EXPERTS) return MOK_ERR_TOO_LARGE;
    if (a->topk < 1 || a->topk > 255) return MOK_ERR_INVALID_ARGUMENT;
    if (a->schedule_capacity <= 0 || a->schedule_capacity % 256 != 0) return MOK_ERR_INVALID_ARGUMENT;
    if (a->minibatch_size <= 0 || a->minibatch_size % 256 != 0) return MOK_ERR_INVALID_ARGUMENT;
    if (a->macrobatch_size <= 0 || a->macrobatch_size % a->minibatch_size != 0) return MOK_ERR_INVALID_ARGUMENT;
    if (a->num_comm_sms <= 0) return MOK_ERR_INVALID_ARGUMENT;
    if (!a->peer_rank || !a->peer_token_idx || !a->num_tokens || !a->tokens_per_expert) return MOK_ERR_INVALID_ARGUMENT;
    if (!a->x_ptrs || !a->x_local) return MOK_ERR_INVALID_ARGUMENT;
    if (!fp8 && (!a->w_routed_gate || !a->w_routed_up)) return MOK_ERR_INVALID_ARGUMENT;
    if (!a->x_routed || !a->gate_routed || !a->up_routed || !a->hidden_routed) return MOK_ERR_INVALID_ARGUMENT;
    const bool any_shared = a->w_shared_gate || a->w_shared_up;
    if (any_shared && !(a->w_shared_gate && a->w_shared_up && a->gate_shared && a->up_shared && a->hidden_shared))
        return MOK_ERR_INVALID_ARGUMENT;
    return MOK_OK;
}

int num_windows(const mok_layer_args* a) { return (a->schedule_capacity + a->macrobatch_size - 1) / a->macrobatch_size; }

// rows [begin, end) of the schedule; `base` is the schedule row held by row 0 of the activation buffers
struct Span {
    int begin, end, base;
};

Span window_span(const mok_layer_args* a, int w) {
    Span s;
    s.begin = s.base = w * a->macrobatch_size;
    s.end = s.begin + a->macrobatch_size;
    if (s.end > a->schedule_capacity) s.end = a->schedule_capacity;
    return s;
}

RowWindow rows_of(const mok_layer_args* a, const Span& s) {
    RowWindow r;
    r.peer_rank = a->peer_rank;
    r.peer_token = a->peer_token_idx;
    r.num_tokens = a->num_tokens;
    r.row_begin = s.begin;
    r.row_end = s.end;
    r.status = a->status;
    return r;
}

// activation buffer pointer of the span's first row
template <typename T>
T* at_row(T* buffer, const Span& s, int row_elems) {
    return buffer + static_cast<size_t>(s.begin - s.base) * row_elems;
}
bf16* rows_bf16(void* buffer, const Span& s, int row_elems) { return at_row(static_cast<bf16*>(buffer), s, row_elems); }
const bf16* rows_bf16(const void* buffer, const Span& s, int row_elems) {
    return at_row(static_cast<const bf16*>(buffer), s, row_elems);
}

GemmProblem routed_problem(const mok_layer_args* a, const Span& s) {
    GemmProblem p;
    p.tokens_per_expert = a->tokens_per_expert;
    p.num_tokens = a->num_tokens;
    p.num_experts = a->num_local_experts;
    p.row_begin = s.begin;
    p.row_end = s.end;
    p.buffer_rows = a->macrobatch_size - (s.begin - s.base);   // rows behind the (offset) buffer pointers
    p.status = a->status;
    return p;
}

// int32 [num_local_experts] behind the two per-row fp32 arrays of row_scratch
int32_t* occupied_rows_of(const mok_layer_args* a) {
    return reinterpret_cast<int32_t*>(a->row_scratch + 2 * static_cast<size_t>(a->macrobatch_size));
}

// MXFP8 backward: fp32 [MB, intermediate / 128] partial sums of the router-weight gradient, behind `occupied`
float* row_partials_of(const mok_layer_args* a) {
    return a->row_scratch + 2 * static_cast<size_t>(a->macrobatch_size) + a->num_local_experts;
}

// MOK_NO_FUSED_ACT=1 runs the MXFP8 activation steps as separate quantize / SwiGLU / dequantize kernels (same e4m3
// bytes; the router-weight gradient differs by summation order only)
bool fused_activations_enabled() {
    const char* v = getenv("MOK_NO_FUSED_ACT");
    return !(v != nullptr && v[0] == '1');
}

// MOK_NO_FUSED_EPILOGUE=1: the MXFP8 gate / up GEMM writes bf16 gate and up, and the fused SwiGLU + quantize kernel
// runs after it, instead of forming hidden and quantizing in the GEMM's own epilogue (same bytes either way)
bool fused_epilogue_enabled() {
    const char* v = getenv("MOK_NO_FUSED_EPILOGUE");
    return !(v != nullptr && v[0] == '1');
}

// MOK_NO_FUSED_SWIGLU=1: the bf16 gate / up GEMM writes gate and up only and a separate SwiGLU kernel reads them back to
// form hidden, instead of forming it in the GEMM's own epilogue (same bytes either way)
bool fused_swiglu_enabled() {
    const char* v = getenv("MOK_NO_FUSED_SWIGLU");
    return !(v != nullptr && v[0] == '1');
}

// MOK_NO_WGRAD_TRIM=1 lets the weight-gradient GEMMs run over the padding rows too (for measurements; same results)
bool wgrad_trim_enabled() {
    const char* v = getenv("MOK_NO_WGRAD_TRIM");
    return !(v != nullptr && v[0] == '1');
}

GemmProblem shared_problem(const mok_layer_args* a) {
    GemmProblem p;
    p.num_experts = 1;
    p.dense_rows = a->num_local_tokens;
    p.row_begin = 0;
    p.row_end = a->num_local_tokens;
    p.buffer_rows = a->num_local_tokens;
    p.status = a->status;
    return p;
}

// CTAs of a dispatch / combine launch that runs beside the GEMMs: num_comm_sms x 8 (MOK_COMM_CTAS overrides, for tuning)
int comm_ctas(const mok_layer_args* a, bool overlapped) {
    if (!overlapped) return 0;
    if (const char* v = getenv("MOK_COMM_CTAS")) {
        const int n = atoi(v);
        if (n > 0) return n;
    }
    return a->num_comm_sms * 8;
}

// ---- de-duplicated dispatch ------------------------------------------------------------------------------
// With the index arrays of mok_schedule_dedup in the arguments and more than one rank, a dispatch first stages the
// tokens its rows use (each pulled over NVLink once) and then fans them out with local copies.  Staged tokens are
// numbered by first row, so "everything rows below r need" is a prefix of the staging buffer: `Staging` remembers how
// far that prefix has been filled during the current call (per source buffer: x or d_y).
struct Staging {
    int staged_upto_row = 0;
};

bool dedup_enabled(const mok_layer_args* a) {
    return a->ep_size > 1 && a->row_source && a->unique_peer && a->unique_token && a->unique_before && a->staged_rows > 0;
}

StagedTokens staged_tokens(const mok_layer_args* a, void* buffer) {
    return StagedTokens{a->row_source, a->unique_peer, a->unique_token, a->unique_before, buffer, a->staged_rows, a->rank};
}

// Makes sure the tokens used by rows below s.end are in `buffer`, then copies the rows of the span.
int staged_dispatch(const mok_layer_args* a, const uint64_t* src_ptrs, const uint64_t* weight_ptrs, void* buffer, Staging* state,
                    const Span& s, void* dst, float* row_weight, int ctas, cudaStream_t st) {
    const StagedTokens t = staged_tokens(a, buffer);
    if (s.end > state->staged_upto_row) {
        MOK_TRY(launch_stage_tokens(src_ptrs, a->ep_size, t, a->num_tokens, state->staged_upto_row, s.end, a->num_local_tokens,
                                    a->hidden, ctas, a->status, st));
        state->staged_upto_row = s.end;
    }
    return launch_dispatch(src_ptrs, weight_ptrs, a->ep_size, rows_of(a, s), a->topk, a->num_local_tokens, a->hidden, dst,
                           row_weight, ctas, st, &t);
}

// ---- per-span building blocks ---------------------------------------------------------------------------
int dispatch_x(const mok_layer_args* a, const Span& s, int ctas, cudaStream_t st, Staging* staging) {
    if (dedup_enabled(a) && a->staged_x != nullptr)
        return staged_dispatch(a, a->x_ptrs, nullptr, a->staged_x, staging, s, rows_bf16(a->x_routed, s, a->hidden), nullptr, ctas, st);
    return launch_dispatch(a->x_ptrs, nullptr, a->ep_size, rows_of(a, s), a->topk, a->num_local_tokens, a->hidden,
                           rows_bf16(a->x_routed, s, a->hidden), nullptr, ctas, st);
}

int dispatch_d_y(const mok_layer_args* a, const Span& s, float* row_weight, int ctas, cudaStream_t st, Staging* staging) {
    void* dst = rows_bf16(a->d_y_routed, s, a->hidden);
    if (dedup_enabled(a) && a->staged_d_y != nullptr)
        return staged_dispatch(a, a->d_y_ptrs, a->router_weight_ptrs, a->staged_d_y, staging, s, dst, at_row(row_weight, s, 1), ctas, st);
    return launch_dispatch(a->d_y_ptrs, a->router_weight_ptrs, a->ep_size, rows_of(a, s), a->topk, a->num_local_tokens, a->hidden,
                           dst, at_row(row_weight, s, 1), ctas, st);
}

int gate_up_hidden(const mok_layer_args* a, const Span& s, cudaStream_t st) {
    const int H = a->hidden, I = a->intermediate;
    if (fused_swiglu_enabled())
        return launch_gate_up_fused(routed_problem(a, s), rows_bf16(a->x_routed, s, H), H, a->w_routed_gate, a->w_routed_up,
                                    rows_bf16(a->gate_routed, s, I), rows_bf16(a->up_routed, s, I),
                                    rows_bf16(a->hidden_routed, s, I), I, a->has_swiglu_limit != 0, a->swiglu_limit, st);
    MOK_TRY(launch_rows_gemm(routed_problem(a, s), rows_bf16(a->x_routed, s, H), H, a->w_routed_gate, a->w_routed_up,
                             rows_bf16(a->gate_routed, s, I), rows_bf16(a->up_routed, s, I), I, false, st));
    MOK_TRY(launch_swiglu_fwd(rows_bf16(a->gate_routed, s, I), rows_bf16(a->up_routed, s, I), rows_bf16(a->hidden_routed, s, I),
                              a->num_tokens, 0, s.begin, s.end, I, a->has_swiglu_limit != 0, a->swiglu_limit, st));
    return MOK_OK;
}

int shared_up_to_hidden(const mok_layer_args* a, cudaStream_t s) {
    const GemmProblem p = shared_problem(a);
    if (fused_swiglu_enabled())
        return launch_gate_up_fused(p, a->x_local, a->hidden, a->w_shared_gate, a->w_shared_up, a->gate_shared, a->up_shared,
                                    a->hidden_shared, a->intermediate, a->has_swiglu_limit != 0, a->swiglu_limit, s);
    MOK_TRY(launch_rows_gemm(p, a->x_local, a->hidden, a->w_shared_gate, a->w_shared_up, a->gate_shared, a->up_shared,
                             a->intermediate, false, s));
    MOK_TRY(launch_swiglu_fwd(a->gate_shared, a->up_shared, a->hidden_shared, nullptr, a->num_local_tokens, 0,
                              a->num_local_tokens, a->intermediate, a->has_swiglu_limit != 0, a->swiglu_limit, s));
    return MOK_OK;
}

// bf16 backward of the shared expert (dense over this rank's tokens)
int shared_backward(const mok_layer_args* a, cudaStream_t s) {
    const int H = a->hidden, I = a->intermediate, T = a->num_local_tokens;
    const GemmProblem p = shared_problem(a);
    const void* d_y = a->d_y_local;
    const void* x = a->x_local;
    // d_hidden = d_y * Wd   (Wd is [H, I]: K = H, N = I)
    MOK_TRY(launch_rows_gemm(p, d_y, H, a->w_shared_down, nullptr, a->d_hidden_shared, nullptr, I, true, s));
    MOK_TRY(launch_swiglu_bwd(a->gate_shared, a->up_shared, a->d_hidden_shared, a->d_gate_shared, a->d_up_shared, nullptr, T, 0,
                              T, I, a->has_swiglu_limit != 0, a->swiglu_limit, nullptr, nullptr, s));
    // d_x = d_gate * Wg + d_up * Wu   (W is [I, H]: K = I, N = H)
    MOK_TRY(launch_rows_gemm_dual(p, a->d_gate_shared, a->d_up_shared, I, a->w_shared_gate, a->w_shared_up, a->d_x_shared, H, s));
    MOK_TRY(launch_wgrad_gemm(p, d_y, H, a->hidden_shared, I, a->d_w_shared_down, s));
    MOK_TRY(launch_wgrad_gemm(p, a->d_gate_shared, I, x, H, a->d_w_shared_gate, s));
    MOK_TRY(launch_wgrad_gemm(p, a->d_up_shared, I, x, H, a->d_w_shared_up, s));
    return MOK_OK;
}

// ---- MXFP8 operands ----------------------------------------------------------------------------------------------
long long scale_tile_row_bytes(long long cols) { return (cols / 128) * 512; }

// rows [s.begin, ...) of a row-major [MB, cols] e4m3 activation buffer
Fp8Operand act_rows(const mok_layer_args* a, const void* data, const void* sc, int cols, const Span& s) {
    const long long off = s.begin - s.base;
    Fp8Operand op;
    op.data = static_cast<const uint8_t*>(data) + off * cols;
    op.scales = static_cast<const uint8_t*>(sc) + (off / 128) * scale_tile_row_bytes(cols);
    op.ld = cols;
    op.rows = a->macrobatch_size - off;
    op.k_extent = cols;
    op.scale_row_tile_stride = scale_tile_row_bytes(cols);
    return op;
}

// a transposed [cols, MB] e4m3 activation buffer (K = schedule rows of the window)
Fp8Operand act_transposed(const mok_layer_args* a, const void* data, const void* sc, int cols) {
    Fp8Operand op;
    op.data = data;
    op.scales = sc;
    op.ld = a->macrobatch_size;
    op.rows = cols;
    op.k_extent = a->macrobatch_size;
    op.scale_row_tile_stride = scale_tile_row_bytes(a->macrobatch_size);
    return op;
}

// expert weights [E, n, k]
Fp8Operand weight_operand(const mok_layer_args* a, const void* data, const void* sc, int n, int k) {
    Fp8Operand op;
    op.data = data;
    op.scales = sc;
    op.ld = k;
    op.rows = static_cast<long long>(a->num_local_experts) * n;
    op.k_extent = k;
    op.scale_row_tile_stride = scale_tile_row_bytes(k);
    return op;
}

// quantize span rows of a bf16 [MB, cols] buffer into the normal and / or transposed e4m3 buffers
int quantize_span(const mok_layer_args* a, const Span& s, const void* src, int cols, void* q, void* sc, void* qt, void* sct,
                  cudaStream_t st) {
    const long long off = s.begin - s.base;
    uint8_t* q_ = q ? static_cast<uint8_t*>(q) + off * cols : nullptr;
    uint8_t* sc_ = sc ? static_cast<uint8_t*>(sc) + (off / 128) * scale_tile_row_bytes(cols) : nullptr;
    uint8_t* qt_ = qt ? static_cast<uint8_t*>(qt) + off : nullptr;
    uint8_t* sct_ = sct ? static_cast<uint8_t*>(sct) + (off / 128) * 512 : nullptr;
    return launch_quantize_rows(rows_bf16(src, s, cols), cols, a->num_tokens, s.begin, s.end, q_, sc_, scale_tile_row_bytes(cols),
                                qt_, a->macrobatch_size, sct_, scale_tile_row_bytes(a->macrobatch_size), st);
}

// x (bf16, dispatched) -> x_fp8 (+ transpose) -> gate, up (bf16 scratch + saved e4m3) -> hidden (bf16 scratch, e4m3 + transpose)
int gate_up_hidden_mxfp8(const mok_layer_args* a, const Span& s, cudaStream_t st) {
    const int H = a->hidden, I = a->intermediate;
    MOK_TRY(quantize_span(a, s, a->x_routed, H, a->x_fp8, a->x_sc, a->x_fp8_t, a->x_sc_t, st));
    const Fp8Operand wg = weight_operand(a, a->w_gate_fp8, a->w_gate_sc, I, H);
    const Fp8Operand wu = weight_operand(a, a->w_up_fp8, a->w_up_sc, I, H);
    if (fused_activations_enabled() && fused_epilogue_enabled()) {   // SwiGLU and the quantizations in the GEMM epilogue
        const long long off = s.begin - s.base;
        const long long sc_I = scale_tile_row_bytes(I);
        Fp8GateUpOut o;
        o.gate_q = static_cast<uint8_t*>(a->gate_fp8) + off * I;
        o.gate_sc = static_cast<uint8_t*>(a->gate_sc) + (off / 128) * sc_I;
        o.up_q = static_cast<uint8_t*>(a->up_fp8) + off * I;
        o.up_sc = static_cast<uint8_t*>(a->up_sc) + (off / 128) * sc_I;
        o.hidden_q = static_cast<uint8_t*>(a->hidden_fp8) + off * I;
        o.hidden_sc = static_cast<uint8_t*>(a->hidden_sc) + (off / 128) * sc_I;
        o.hidden_qt = static_cast<uint8_t*>(a->hidden_fp8_t) + off;
        o.hidden_sct = static_cast<uint8_t*>(a->hidden_sc_t) + (off / 128) * 512;
        o.sc_row_tile_stride = sc_I;
        o.qt_ld = a->macrobatch_size;
        o.sct_row_tile_stride = scale_tile_row_bytes(a->macrobatch_size);
        o.has_limit = a->has_swiglu_limit != 0;
        o.limit = a->swiglu_limit;
        return launch_fp8_gate_up_fused(routed_problem(a, s), act_rows(a, a->x_fp8, a->x_sc, H, s), H, wg, wu, I, o, st);
    }
    MOK_TRY(launch_fp8_rows_gemm(routed_problem(a, s), act_rows(a, a->x_fp8, a->x_sc, H, s), H, wg, &wu,
                                 rows_bf16(a->gate_routed, s, I), rows_bf16(a->up_routed, s, I), I, st));
    if (fused_activations_enabled()) {   // one pass: e4m3 gate, up, and hidden in both layouts
        const long long off = s.begin - s.base;
        const long long sc_I = scale_tile_row_bytes(I);
        auto q_at = [&](void* q) { return static_cast<uint8_t*>(q) + off * I; };
        auto sc_at = [&](void* sc) { return static_cast<uint8_t*>(sc) + (off / 128) * sc_I; };
        return launch_swiglu_quantize_fwd(rows_bf16(a->gate_routed, s, I), rows_bf16(a->up_routed, s, I), I, a->num_tokens, s.begin,
                                          s.end, q_at(a->gate_fp8), sc_at(a->gate_sc), q_at(a->up_fp8), sc_at(a->up_sc),
                                          q_at(a->hidden_fp8), sc_at(a->hidden_sc), sc_I,
                                          static_cast<uint8_t*>(a->hidden_fp8_t) + off, a->macrobatch_size,
                                          static_cast<uint8_t*>(a->hidden_sc_t) + (off / 128) * 512,
                                          scale_tile_row_bytes(a->macrobatch_size), a->has_swiglu_limit != 0, a->swiglu_limit, st);
    }
    MOK_TRY(quantize_span(a, s, a->gate_routed, I, a->gate_fp8, a->gate_sc, nullptr, nullptr, st));
    MOK_TRY(quantize_span(a, s, a->up_routed, I, a->up_fp8, a->up_sc, nullptr, nullptr, st));
    MOK_TRY(launch_swiglu_fwd(rows_bf16(a->gate_routed, s, I), rows_bf16(a->up_routed, s, I), rows_bf16(a->hidden_routed, s, I),
                              a->num_tokens, 0, s.begin, s.end, I, a->has_swiglu_limit != 0, a->swiglu_limit, st));
    MOK_TRY(quantize_span(a, s, a->hidden_routed, I, a->hidden_fp8, a->hidden_sc, a->hidden_fp8_t, a->hidden_sc_t, st));
    return MOK_OK;
}

int check_mxfp8_forward_fields(const mok_layer_args* a) {
    if (!a->w_gate_fp8 || !a->w_gate_sc || !a->w_up_fp8 || !a->w_up_sc) return MOK_ERR_INVALID_ARGUMENT;
    if (!a->x_fp8 || !a->x_sc || !a->x_fp8_t || !a->x_sc_t || !a->gate_fp8 || !a->gate_sc || !a->up_fp8 || !a->up_sc ||
        !a->hidden_fp8 || !a->hidden_sc || !a->hidden_fp8_t || !a->hidden_sc_t)
        return MOK_ERR_INVALID_ARGUMENT;
    if (a->macrobatch_size % 256 != 0) return MOK_ERR_INVALID_ARGUMENT;
    return MOK_OK;
}

// ---- chunk pipeline -----------------------------------------------------------------------------------------
// Runs pull(c) -> compute(c) -> push(c) over the chunks of one window.  Overlapped: pull / push on the internal
// stream, compute on the caller's stream, ordered by events, pull two chunks ahead.  Not overlapped: one stream.
// On return every pull has been consumed; pushes may still be running on the internal stream (the caller joins).
template <class Pull, class Compute, class Push>
int run_chunks(const mok_layer_args* a, const Span& win, bool overlapped, DeviceStreams* d, cudaStream_t main_stream,
               Pull pull, Compute compute, Push push) {
    const int chunk = chunk_rows_for(a);
    const int n = (win.end - win.begin + chunk - 1) / chunk;
    auto span_of = [&](int c) {
        Span s;
        s.base = win.base;
        s.begin = win.begin + c * chunk;
        s.end = s.begin + chunk < win.end ? s.begin + chunk : win.end;
        return s;
    };
    if (!overlapped) {
        for (int c = 0; c < n; ++c) {
            const Span s = span_of(c);
            MOK_TRY(pull(s, 0, main_stream));
            MOK_TRY(compute(s, main_stream));
            MOK_TRY(push(s, 0, main_stream));
        }
        return MOK_OK;
    }
    const int ctas = comm_ctas(a, true);
    cudaEvent_t pulled[3], computed[3];   // rings: an event is re-recorded only after its waiter was enqueued
    for (int i = 0; i < 3; ++i) {
        pulled[i] = next_event(d);
        computed[i] = next_event(d);
    }
    for (int step = 0; step < n + 2; ++step) {
        const int c = step, m = step - 1, k = step - 2;
        if (c < n) {
            const int t = trace_begin("pull", c, true, d->comm);
            MOK_TRY(pull(span_of(c), ctas, d->comm));
            trace_end(t, d->comm);
            MOK_CUDA_CHECK(cudaEventRecord(pulled[c % 3], d->comm));
        }
        if (m >= 0 && m < n) {
            MOK_CUDA_CHECK(cudaStreamWaitEvent(main_stream, pulled[m % 3], 0));
            const int t = trace_begin("compute", m, false, main_stream);
            MOK_TRY(compute(span_of(m), main_stream));
            trace_end(t, main_stream);
            MOK_CUDA_CHECK(cudaEventRecord(computed[m % 3], main_stream));
        }
        if (k >= 0 && k < n) {
            MOK_CUDA_CHECK(cudaStreamWaitEvent(d->comm, computed[k % 3], 0));
            const int t = trace_begin("push", k, true, d->comm);
            MOK_TRY(push(span_of(k), ctas, d->comm));
            trace_end(t, d->comm);
        }
    }
    return MOK_OK;
}

}  // namespace
}  // namespace mok

extern "C" int mok_moe_forward_bf16(const mok_layer_args* a, mok_stream_t stream) {
    using namespace mok;
    MOK_TRY(check_common(a));
    if (!a->combine_ptrs || !a->w_routed_down || !a->y_routed) return MOK_ERR_INVALID_ARGUMENT;
    if (a->w_shared_gate && (!a->w_shared_down || !a->y_shared)) return MOK_ERR_INVALID_ARGUMENT;
    cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
    Staging x_staging, d_y_staging;   // how far the de-duplicated tokens of x / d_y have been staged in this call
    const bool overlapped = overlap_enabled();
    DeviceStreams* d = nullptr;
    CommFork fork;   // the internal stream starts after the caller's earlier work and is joined on every way out
    if (overlapped) MOK_TRY(fork.start(s, &d));
    const int H = a->hidden, I = a->intermediate;
    if (a->w_shared_gate) {   // runs on the caller's stream while the first chunks are being pulled
        MOK_TRY(shared_up_to_hidden(a, s));
        MOK_TRY(launch_rows_gemm(shared_problem(a), a->hidden_shared, I, a->w_shared_down, nullptr, a->y_shared, nullptr, H,
                                 false, s));
    }
    for (int wi = num_windows(a) - 1; wi >= 0; --wi) {
        const Span win = window_span(a, wi);
        MOK_TRY(run_chunks(
            a, win, overlapped, d, s,
            [&](const Span& c, int ctas, cudaStream_t st) { return dispatch_x(a, c, ctas, st, &x_staging); },
            [&](const Span& c, cudaStream_t st) {
                MOK_TRY(gate_up_hidden(a, c, st));
                return launch_rows_gemm(routed_problem(a, c), rows_bf16(a->hidden_routed, c, I), I, a->w_routed_down, nullptr,
                                        rows_bf16(a->y_routed, c, H), nullptr, H, false, st);
            },
            [&](const Span& c, int ctas, cudaStream_t st) {
                return launch_combine(a->combine_ptrs, nullptr, a->ep_size, rows_of(a, c), a->topk, a->num_local_tokens, H,
                                      rows_bf16(a->y_routed, c, H), nullptr, ctas, st);
            }));
        // the next window reuses the buffers: its pulls wait for this window's GEMMs, its GEMMs for these pushes
        if (overlapped) {
            MOK_TRY(order_after(d, d->comm, s));
            if (wi > 0) MOK_TRY(order_after(d, s, d->comm));
        }
    }
    return MOK_OK;
}

extern "C" int mok_moe_recompute_bf16(const mok_layer_args* a, mok_stream_t stream) {
    using namespace mok;
    MOK_TRY(check_common(a));
    cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
    Staging x_staging, d_y_staging;   // how far the de-duplicated tokens of x / d_y have been staged in this call
    if (a->w_shared_gate) MOK_TRY(shared_up_to_hidden(a, s));
    const Span win = window_span(a, 0);
    MOK_TRY(dispatch_x(a, win, 0, s, &x_staging));
    MOK_TRY(gate_up_hidden(a, win, s));
    return MOK_OK;
}

extern "C" int mok_moe_backward_bf16(const mok_layer_args* a, mok_stream_t stream) {
    using namespace mok;
    MOK_TRY(check_common(a));
    if (!a->d_y_ptrs || !a->d_x_routed_ptrs || !a->router_weight_ptrs || !a->d_router_weight_ptrs || !a->w_routed_down)
        return MOK_ERR_INVALID_ARGUMENT;
    if (!a->d_x_routed || !a->d_gate_routed || !a->d_up_routed || !a->d_hidden_routed || !a->d_y_routed ||
        !a->d_w_routed_gate || !a->d_w_routed_up || !a->d_w_routed_down || !a->row_scratch)
        return MOK_ERR_INVALID_ARGUMENT;
    const bool shared = a->w_shared_gate != nullptr;
    if (shared && !(a->d_y_local && a->w_shared_down && a->d_x_shared && a->d_gate_shared && a->d_up_shared && a->d_hidden_shared &&
                    a->d_w_shared_gate && a->d_w_shared_up && a->d_w_shared_down))
        return MOK_ERR_INVALID_ARGUMENT;
    cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
    Staging x_staging, d_y_staging;   // how far the de-duplicated tokens of x / d_y have been staged in this call
    const int H = a->hidden, I = a->intermediate, T = a->num_local_tokens;
    const bool clamp = a->has_swiglu_limit != 0;
    const bool overlapped = overlap_enabled();
    DeviceStreams* d = nullptr;
    CommFork fork;
    if (overlapped) MOK_TRY(fork.start(s, &d));

    if (shared) {
        const int ts = trace_begin("shared_bwd", 0, false, s);
        MOK_TRY(shared_backward(a, s));
        trace_end(ts, s);
    }

    float* row_weight = a->row_scratch;
    float* row_grad = a->row_scratch + a->macrobatch_size;
    int32_t* occupied = occupied_rows_of(a);
    MOK_TRY(launch_occupied_rows(a->peer_rank, a->tokens_per_expert, a->num_tokens, a->schedule_capacity, a->num_local_experts,
                                 occupied, s));
    for (int wi = 0; wi < num_windows(a); ++wi) {
        const Span win = window_span(a, wi);
        if (wi > 0) {   // the saved context only covers window 0: rebuild x_routed, gate, up, hidden of this window
            MOK_TRY(dispatch_x(a, win, 0, s, &x_staging));
            MOK_TRY(gate_up_hidden(a, win, s));
        }
        MOK_TRY(run_chunks(
            a, win, overlapped, d, s,
            [&](const Span& c, int ctas, cudaStream_t st) { return dispatch_d_y(a, c, row_weight, ctas, st, &d_y_staging); },
            [&](const Span& c, cudaStream_t st) {
                const GemmProblem p = routed_problem(a, c);
                MOK_TRY(launch_rows_gemm(p, rows_bf16(a->d_y_routed, c, H), H, a->w_routed_down, nullptr,
                                         rows_bf16(a->d_hidden_routed, c, I), nullptr, I, true, st));
                MOK_TRY(launch_swiglu_bwd(rows_bf16(a->gate_routed, c, I), rows_bf16(a->up_routed, c, I),
                                          rows_bf16(a->d_hidden_routed, c, I), rows_bf16(a->d_gate_routed, c, I),
                                          rows_bf16(a->d_up_routed, c, I), a->num_tokens, 0, c.begin, c.end, I, clamp,
                                          a->swiglu_limit, at_row(row_weight, c, 1), at_row(row_grad, c, 1), st));
                return launch_rows_gemm_dual(p, rows_bf16(a->d_gate_routed, c, I), rows_bf16(a->d_up_routed, c, I), I,
                                             a->w_routed_gate, a->w_routed_up, rows_bf16(a->d_x_routed, c, H), H, st);
            },
            [&](const Span& c, int ctas, cudaStream_t st) {
                return launch_combine(a->d_x_routed_ptrs, a->d_router_weight_ptrs, a->ep_size, rows_of(a, c), a->topk, T, H,
                                      rows_bf16(a->d_x_routed, c, H), at_row(row_grad, c, 1), ctas, st);
            }));
        // weight gradients over the whole window (fixed K order = schedule order), while the last pushes drain
        GemmProblem p = routed_problem(a, win);
        if (wgrad_trim_enabled()) p.occupied_rows = occupied;
        const int tw = trace_begin("wgrad", wi, false, s);
        MOK_TRY(launch_wgrad_gemm(p, a->d_y_routed, H, a->hidden_routed, I, a->d_w_routed_down, s));
        MOK_TRY(launch_wgrad_gemm(p, a->d_gate_routed, I, a->x_routed, H, a->d_w_routed_gate, s));
        MOK_TRY(launch_wgrad_gemm(p, a->d_up_routed, I, a->x_routed, H, a->d_w_routed_up, s));
        trace_end(tw, s);
        if (overlapped) {
            MOK_TRY(order_after(d, d->comm, s));
            if (wi + 1 < num_windows(a)) MOK_TRY(order_after(d, s, d->comm));
        }
    }
    MOK_TRY(launch_zero_empty_wgrads(a->tokens_per_expert, a->num_local_experts, a->d_w_routed_gate, a->d_w_routed_up,
                                     a->d_w_routed_down, static_cast<long long>(H) * I, s));
    return MOK_OK;
}

// ---------------------------------------------------------------------------------------------------------------------
// MXFP8 entry points: same launch structure, routed GEMMs block-scaled, activations quantized between the steps
// ---------------------------------------------------------------------------------------------------------------------
extern "C" int mok_moe_forward_mxfp8(const mok_layer_args* a, mok_stream_t stream) {
    using namespace mok;
    MOK_TRY(check_common(a, true));
    MOK_TRY(check_mxfp8_forward_fields(a));
    if (!a->combine_ptrs || !a->w_down_fp8 || !a->w_down_sc || !a->y_routed) return MOK_ERR_INVALID_ARGUMENT;
    if (a->w_shared_gate && (!a->w_shared_down || !a->y_shared)) return MOK_ERR_INVALID_ARGUMENT;
    cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
    Staging x_staging, d_y_staging;   // how far the de-duplicated tokens of x / d_y have been staged in this call
    const bool overlapped = overlap_enabled();
    DeviceStreams* d = nullptr;
    CommFork fork;
    if (overlapped) MOK_TRY(fork.start(s, &d));
    const int H = a->hidden, I = a->intermediate;
    if (a->w_shared_gate) {
        MOK_TRY(shared_up_to_hidden(a, s));
        MOK_TRY(launch_rows_gemm(shared_problem(a), a->hidden_shared, I, a->w_shared_down, nullptr, a->y_shared, nullptr, H,
                                 false, s));
    }
    const Fp8Operand wd = weight_operand(a, a->w_down_fp8, a->w_down_sc, H, I);
    for (int wi = num_windows(a) - 1; wi >= 0; --wi) {
        const Span win = window_span(a, wi);
        MOK_TRY(run_chunks(
            a, win, overlapped, d, s,
            [&](const Span& c, int ctas, cudaStream_t st) { return dispatch_x(a, c, ctas, st, &x_staging); },
            [&](const Span& c, cudaStream_t st) {
                MOK_TRY(gate_up_hidden_mxfp8(a, c, st));
                return launch_fp8_rows_gemm(routed_problem(a, c), act_rows(a, a->hidden_fp8, a->hidden_sc, I, c), I, wd, nullptr,
                                            rows_bf16(a->y_routed, c, H), nullptr, H, st);
            },
            [&](const Span& c, int ctas, cudaStream_t st) {
                return launch_combine(a->combine_ptrs, nullptr, a->ep_size, rows_of(a, c), a->topk, a->num_local_tokens, H,
                                      rows_bf16(a->y_routed, c, H), nullptr, ctas, st);
            }));
        if (overlapped) {
            MOK_TRY(order_after(d, d->comm, s));
            if (wi > 0) MOK_TRY(order_after(d, s, d->comm));
        }
    }
    return MOK_OK;
}

extern "C" int mok_moe_recompute_mxfp8(const mok_layer_args* a, mok_stream_t stream) {
    using namespace mok;
    MOK_TRY(check_common(a, true));
    MOK_TRY(check_mxfp8_forward_fields(a));
    cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
    Staging x_staging, d_y_staging;   // how far the de-duplicated tokens of x / d_y have been staged in this call
    if (a->w_shared_gate) MOK_TRY(shared_up_to_hidden(a, s));
    const Span win = window_span(a, 0);
    MOK_TRY(dispatch_x(a, win, 0, s, &x_staging));
    MOK_TRY(gate_up_hidden_mxfp8(a, win, s));
    return MOK_OK;
}

extern "C" int mok_moe_backward_mxfp8(const mok_layer_args* a, mok_stream_t stream) {
    using namespace mok;
    MOK_TRY(check_common(a, true));
    MOK_TRY(check_mxfp8_forward_fields(a));
    if (!a->d_y_ptrs || !a->d_x_routed_ptrs || !a->router_weight_ptrs || !a->d_router_weight_ptrs) return MOK_ERR_INVALID_ARGUMENT;
    if (!a->w_gate_t_fp8 || !a->w_gate_t_sc || !a->w_up_t_fp8 || !a->w_up_t_sc || !a->w_down_t_fp8 || !a->w_down_t_sc)
        return MOK_ERR_INVALID_ARGUMENT;
    if (!a->d_x_routed || !a->d_gate_routed || !a->d_up_routed || !a->d_hidden_routed || !a->d_y_routed || !a->d_w_routed_gate ||
        !a->d_w_routed_up || !a->d_w_routed_down || !a->row_scratch)
        return MOK_ERR_INVALID_ARGUMENT;
    if (!a->d_y_fp8 || !a->d_y_sc || !a->d_y_fp8_t || !a->d_y_sc_t || !a->d_gate_fp8 || !a->d_gate_sc || !a->d_up_fp8 ||
        !a->d_up_sc || !a->d_gate_fp8_t || !a->d_gate_sc_t || !a->d_up_fp8_t || !a->d_up_sc_t)
        return MOK_ERR_INVALID_ARGUMENT;
    const bool shared = a->w_shared_gate != nullptr;
    if (shared && !(a->d_y_local && a->w_shared_down && a->d_x_shared && a->d_gate_shared && a->d_up_shared && a->d_hidden_shared &&
                    a->d_w_shared_gate && a->d_w_shared_up && a->d_w_shared_down))
        return MOK_ERR_INVALID_ARGUMENT;
    cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
    Staging x_staging, d_y_staging;   // how far the de-duplicated tokens of x / d_y have been staged in this call
    const int H = a->hidden, I = a->intermediate, T = a->num_local_tokens;
    const bool clamp = a->has_swiglu_limit != 0;
    const bool overlapped = overlap_enabled();
    DeviceStreams* d = nullptr;
    CommFork fork;
    if (overlapped) MOK_TRY(fork.start(s, &d));
    if (shared) {
        const int ts = trace_begin("shared_bwd", 0, false, s);
        MOK_TRY(shared_backward(a, s));
        trace_end(ts, s);
    }

    const Fp8Operand wd_t = weight_operand(a, a->w_down_t_fp8, a->w_down_t_sc, I, H);   // [E, I, H]: N = I, K = H
    const Fp8Operand wg_t = weight_operand(a, a->w_gate_t_fp8, a->w_gate_t_sc, H, I);   // [E, H, I]: N = H, K = I
    const Fp8Operand wu_t = weight_operand(a, a->w_up_t_fp8, a->w_up_t_sc, H, I);
    float* row_weight = a->row_scratch;
    float* row_grad = a->row_scratch + a->macrobatch_size;
    const long long sc_I = scale_tile_row_bytes(I);
    int32_t* occupied = occupied_rows_of(a);
    MOK_TRY(launch_occupied_rows(a->peer_rank, a->tokens_per_expert, a->num_tokens, a->schedule_capacity, a->num_local_experts,
                                 occupied, s));
    for (int wi = 0; wi < num_windows(a); ++wi) {
        const Span win = window_span(a, wi);
        if (wi > 0) {
            MOK_TRY(dispatch_x(a, win, 0, s, &x_staging));
            MOK_TRY(gate_up_hidden_mxfp8(a, win, s));
        }
        MOK_TRY(run_chunks(
            a, win, overlapped, d, s,
            [&](const Span& c, int ctas, cudaStream_t st) { return dispatch_d_y(a, c, row_weight, ctas, st, &d_y_staging); },
            [&](const Span& c, cudaStream_t st) {
                const GemmProblem p = routed_problem(a, c);
                const long long off = c.begin - c.base;
                MOK_TRY(quantize_span(a, c, a->d_y_routed, H, a->d_y_fp8, a->d_y_sc, a->d_y_fp8_t, a->d_y_sc_t, st));
                MOK_TRY(launch_fp8_rows_gemm(p, act_rows(a, a->d_y_fp8, a->d_y_sc, H, c), H, wd_t, nullptr,
                                             rows_bf16(a->d_hidden_routed, c, I), nullptr, I, st));
                if (fused_activations_enabled()) {   // saved e4m3 gate / up + d_hidden -> e4m3 d_gate, d_up in one pass
                    auto q_at = [&](void* q) { return static_cast<uint8_t*>(q) + off * I; };
                    auto sc_at = [&](void* sc) { return static_cast<uint8_t*>(sc) + (off / 128) * sc_I; };
                    auto qt_at = [&](void* q) { return static_cast<uint8_t*>(q) + off; };
                    auto sct_at = [&](void* sc) { return static_cast<uint8_t*>(sc) + (off / 128) * 512; };
                    float* partial = row_partials_of(a) + off * (I / 128);
                    MOK_TRY(launch_swiglu_quantize_bwd(
                        q_at(a->gate_fp8), sc_at(a->gate_sc), q_at(a->up_fp8), sc_at(a->up_sc), rows_bf16(a->d_hidden_routed, c, I), I,
                        a->num_tokens, c.begin, c.end, q_at(a->d_gate_fp8), sc_at(a->d_gate_sc), q_at(a->d_up_fp8), sc_at(a->d_up_sc),
                        sc_I, qt_at(a->d_gate_fp8_t), sct_at(a->d_gate_sc_t), qt_at(a->d_up_fp8_t), sct_at(a->d_up_sc_t),
                        a->macrobatch_size, scale_tile_row_bytes(a->macrobatch_size), partial, clamp, a->swiglu_limit, st));
                    MOK_TRY(launch_router_grad(partial, I / 128, at_row(row_weight, c, 1), at_row(row_grad, c, 1), a->num_tokens,
                                               c.begin, c.end, st));
                    return launch_fp8_rows_gemm_dual(p, act_rows(a, a->d_gate_fp8, a->d_gate_sc, I, c),
                                                     act_rows(a, a->d_up_fp8, a->d_up_sc, I, c), I, wg_t, wu_t,
                                                     rows_bf16(a->d_x_routed, c, H), H, st);
                }
                // the saved gate / up are e4m3: expand them (exactly) into the bf16 scratch the SwiGLU backward reads
                MOK_TRY(launch_dequantize_rows(static_cast<const uint8_t*>(a->gate_fp8) + off * I,
                                               static_cast<const uint8_t*>(a->gate_sc) + (off / 128) * sc_I, sc_I,
                                               rows_bf16(a->gate_routed, c, I), I, a->num_tokens, c.begin, c.end, st));
                MOK_TRY(launch_dequantize_rows(static_cast<const uint8_t*>(a->up_fp8) + off * I,
                                               static_cast<const uint8_t*>(a->up_sc) + (off / 128) * sc_I, sc_I,
                                               rows_bf16(a->up_routed, c, I), I, a->num_tokens, c.begin, c.end, st));
                MOK_TRY(launch_swiglu_bwd(rows_bf16(a->gate_routed, c, I), rows_bf16(a->up_routed, c, I),
                                          rows_bf16(a->d_hidden_routed, c, I), rows_bf16(a->d_gate_routed, c, I),
                                          rows_bf16(a->d_up_routed, c, I), a->num_tokens, 0, c.begin, c.end, I, clamp,
                                          a->swiglu_limit, at_row(row_weight, c, 1), at_row(row_grad, c, 1), st));
                MOK_TRY(quantize_span(a, c, a->d_gate_routed, I, a->d_gate_fp8, a->d_gate_sc, a->d_gate_fp8_t, a->d_gate_sc_t, st));
                MOK_TRY(quantize_span(a, c, a->d_up_routed, I, a->d_up_fp8, a->d_up_sc, a->d_up_fp8_t, a->d_up_sc_t, st));
                return launch_fp8_rows_gemm_dual(p, act_rows(a, a->d_gate_fp8, a->d_gate_sc, I, c),
                                                 act_rows(a, a->d_up_fp8, a->d_up_sc, I, c), I, wg_t, wu_t,
                                                 rows_bf16(a->d_x_routed, c, H), H, st);
            },
            [&](const Span& c, int ctas, cudaStream_t st) {
                return launch_combine(a->d_x_routed_ptrs, a->d_router_weight_ptrs, a->ep_size, rows_of(a, c), a->topk, T, H,
                                      rows_bf16(a->d_x_routed, c, H), at_row(row_grad, c, 1), ctas, st);
            }));
        GemmProblem p = routed_problem(a, win);
        if (wgrad_trim_enabled()) p.occupied_rows = occupied;
        MOK_TRY(launch_fp8_wgrad_gemm(p, act_transposed(a, a->d_y_fp8_t, a->d_y_sc_t, H), H,
                                      act_transposed(a, a->hidden_fp8_t, a->hidden_sc_t, I), I, a->d_w_routed_down, s));
        MOK_TRY(launch_fp8_wgrad_gemm(p, act_transposed(a, a->d_gate_fp8_t, a->d_gate_sc_t, I), I,
                                      act_transposed(a, a->x_fp8_t, a->x_sc_t, H), H, a->d_w_routed_gate, s));
        MOK_TRY(launch_fp8_wgrad_gemm(p, act_transposed(a, a->d_up_fp8_t, a->d_up_sc_t, I), I,
                                      act_transposed(a, a->x_fp8_t, a->x_sc_t, H), H, a->d_w_routed_up, s));
        if (overlapped) {
            MOK_TRY(order_after(d, d->comm, s));
            if (wi + 1 < num_windows(a)) MOK_TRY(order_after(d, s, d->comm));
        }
    }
    MOK_TRY(launch_zero_empty_wgrads(a->tokens_per_expert, a->num_local_experts, a->d_w_routed_gate, a->d_w_routed_up,
                                     a->d_w_routed_down, static_cast<long long>(H) * I, s));
    return MOK_OK;
}

// Writes the phase timeline collected under MOK_TRACE=1 (one line per phase: name, chunk, stream, start and end in
// milliseconds since the first phase) and clears it.  Synchronises the device: a debugging aid, not for hot paths.
extern "C" int mok_trace_dump(const char* path) {
    using namespace mok;
    std::vector<TraceRecord>& recs = trace_records();
    if (path == nullptr) return MOK_ERR_INVALID_ARGUMENT;
    MOK_CUDA_CHECK(cudaDeviceSynchronize());
    FILE* f = fopen(path, "w");
    if (f == nullptr) return MOK_ERR_INVALID_ARGUMENT;
    for (size_t i = 0; i < recs.size(); ++i) {
        float t0 = 0.f, t1 = 0.f;
        const cudaError_t e0 = cudaEventElapsedTime(&t0, recs[0].begin, recs[i].begin);
        const cudaError_t e1 = cudaEventElapsedTime(&t1, recs[0].begin, recs[i].end);
        if (e0 != cudaSuccess || e1 != cudaSuccess)
            fprintf(f, "# %s %d: %s / %s\n", recs[i].name, recs[i].chunk, cudaGetErrorName(e0), cudaGetErrorName(e1));
        else
            fprintf(f, "%s %d %s %.4f %.4f\n", recs[i].name, recs[i].chunk, recs[i].on_comm_stream ? "comm" : "main", t0, t1);
    }
    for (size_t i = 0; i < recs.size(); ++i) {
        cudaEventDestroy(recs[i].begin);
        cudaEventDestroy(recs[i].end);
    }
    fclose(f);
    recs.clear();
    (void)cudaGetLastError();   // a failed query above must not surface in the next launch check
    return MOK_OK;
}
