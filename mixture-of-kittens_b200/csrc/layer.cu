// Fused-layer entry points: the launch sequences for the BF16 forward, context recomputation and backward of
// the expert-parallel MoE layer.  Everything is enqueued on the caller's stream; no host synchronisation.
//
// Routed activations live in buffers of `macrobatch_size` rows.  Schedule rows are processed in windows of that
// size ("macrobatches"); forward walks the windows last to first so that window 0's activations are what the
// buffers hold afterwards, and backward recomputes gate / up / hidden for windows >= 1 before using them
// (reference: csrc/megakernel/forward.cuh:117-129,202-209 and backward.cuh:147-176,296-329).
#include "comm.cuh"
#include "elementwise.cuh"
#include "grouped_gemm.cuh"

namespace mok {
namespace {

#define MOK_TRY(expr)                  \
    do {                               \
        int _rc = (expr);              \
        if (_rc != MOK_OK) return _rc; \
    } while (0)

int check_common(const mok_layer_args* a) {
    if (a == nullptr) return MOK_ERR_INVALID_ARGUMENT;
    if (a->ep_size < 1 || a->ep_size > MOK_MAX_EP || a->rank < 0 || a->rank >= a->ep_size) return MOK_ERR_INVALID_ARGUMENT;
    if (a->num_local_tokens <= 0 || a->num_local_tokens % 128 != 0) return MOK_ERR_INVALID_ARGUMENT;
    if (a->hidden <= 0 || a->hidden % 256 != 0 || a->intermediate <= 0 || a->intermediate % 256 != 0)
        return MOK_ERR_INVALID_ARGUMENT;
    if (a->num_local_experts < 1) return MOK_ERR_INVALID_ARGUMENT;
    if (a->num_local_experts > MOK_MAX_LOCAL_EXPERTS) return MOK_ERR_TOO_LARGE;
    if (a->topk < 1 || a->topk > 255) return MOK_ERR_INVALID_ARGUMENT;
    if (a->schedule_capacity <= 0 || a->schedule_capacity % 256 != 0) return MOK_ERR_INVALID_ARGUMENT;
    if (a->minibatch_size <= 0 || a->minibatch_size % 256 != 0) return MOK_ERR_INVALID_ARGUMENT;
    if (a->macrobatch_size <= 0 || a->macrobatch_size % a->minibatch_size != 0) return MOK_ERR_INVALID_ARGUMENT;
    if (!a->peer_rank || !a->peer_token_idx || !a->num_tokens || !a->tokens_per_expert) return MOK_ERR_INVALID_ARGUMENT;
    if (!a->x_ptrs || !a->x_local || !a->w_routed_gate || !a->w_routed_up) return MOK_ERR_INVALID_ARGUMENT;
    if (!a->x_routed || !a->gate_routed || !a->up_routed || !a->hidden_routed) return MOK_ERR_INVALID_ARGUMENT;
    const bool any_shared = a->w_shared_gate || a->w_shared_up;
    if (any_shared && !(a->w_shared_gate && a->w_shared_up && a->gate_shared && a->up_shared && a->hidden_shared))
        return MOK_ERR_INVALID_ARGUMENT;
    return MOK_OK;
}

int num_windows(const mok_layer_args* a) { return (a->schedule_capacity + a->macrobatch_size - 1) / a->macrobatch_size; }

RowWindow window(const mok_layer_args* a, int w) {
    RowWindow r;
    r.peer_rank = a->peer_rank;
    r.peer_token = a->peer_token_idx;
    r.num_tokens = a->num_tokens;
    r.row_begin = w * a->macrobatch_size;
    r.row_end = r.row_begin + a->macrobatch_size;
    if (r.row_end > a->schedule_capacity) r.row_end = a->schedule_capacity;
    r.status = a->status;
    return r;
}

GemmProblem routed_problem(const mok_layer_args* a, const RowWindow& w) {
    GemmProblem p;
    p.tokens_per_expert = a->tokens_per_expert;
    p.num_tokens = a->num_tokens;
    p.num_experts = a->num_local_experts;
    p.row_begin = w.row_begin;
    p.row_end = w.row_end;
    p.buffer_rows = a->macrobatch_size;
    p.status = a->status;
    return p;
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

// dispatch x -> gate / up GEMMs -> SwiGLU for one window (used by forward, recompute and backward replay)
int routed_up_to_hidden(const mok_layer_args* a, const RowWindow& w, cudaStream_t s) {
    MOK_TRY(launch_dispatch(a->x_ptrs, nullptr, a->ep_size, w, a->topk, a->num_local_tokens, a->hidden, a->x_routed, nullptr, 0, s));
    const GemmProblem p = routed_problem(a, w);
    MOK_TRY(launch_rows_gemm(p, a->x_routed, a->hidden, a->w_routed_gate, a->w_routed_up, a->gate_routed, a->up_routed,
                             a->intermediate, false, s));
    MOK_TRY(launch_swiglu_fwd(a->gate_routed, a->up_routed, a->hidden_routed, a->num_tokens, 0, w.row_begin, w.row_end,
                              a->intermediate, a->has_swiglu_limit != 0, a->swiglu_limit, s));
    return MOK_OK;
}

int shared_up_to_hidden(const mok_layer_args* a, cudaStream_t s) {
    const GemmProblem p = shared_problem(a);
    MOK_TRY(launch_rows_gemm(p, a->x_local, a->hidden, a->w_shared_gate, a->w_shared_up, a->gate_shared, a->up_shared,
                             a->intermediate, false, s));
    MOK_TRY(launch_swiglu_fwd(a->gate_shared, a->up_shared, a->hidden_shared, nullptr, a->num_local_tokens, 0,
                              a->num_local_tokens, a->intermediate, a->has_swiglu_limit != 0, a->swiglu_limit, s));
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

    if (a->w_shared_gate) {
        MOK_TRY(shared_up_to_hidden(a, s));
        MOK_TRY(launch_rows_gemm(shared_problem(a), a->hidden_shared, a->intermediate, a->w_shared_down, nullptr, a->y_shared,
                                 nullptr, a->hidden, false, s));
    }
    for (int wi = num_windows(a) - 1; wi >= 0; --wi) {
        const RowWindow w = window(a, wi);
        MOK_TRY(routed_up_to_hidden(a, w, s));
        MOK_TRY(launch_rows_gemm(routed_problem(a, w), a->hidden_routed, a->intermediate, a->w_routed_down, nullptr,
                                 a->y_routed, nullptr, a->hidden, false, s));
        MOK_TRY(launch_combine(a->combine_ptrs, nullptr, a->ep_size, w, a->topk, a->num_local_tokens, a->hidden, a->y_routed,
                               nullptr, 0, s));
    }
    return MOK_OK;
}

extern "C" int mok_moe_recompute_bf16(const mok_layer_args* a, mok_stream_t stream) {
    using namespace mok;
    MOK_TRY(check_common(a));
    cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
    if (a->w_shared_gate) MOK_TRY(shared_up_to_hidden(a, s));
    MOK_TRY(routed_up_to_hidden(a, window(a, 0), s));
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
    const int H = a->hidden, I = a->intermediate, T = a->num_local_tokens;
    const bool clamp = a->has_swiglu_limit != 0;

    if (shared) {
        const GemmProblem p = shared_problem(a);
        const void* d_y = a->d_y_local;
        const void* x = a->x_local;
        // d_hidden = d_y * Wd   (Wd is [H, I]: K = H, N = I)
        MOK_TRY(launch_rows_gemm(p, d_y, H, a->w_shared_down, nullptr, a->d_hidden_shared, nullptr, I, true, s));
        MOK_TRY(launch_swiglu_bwd(a->gate_shared, a->up_shared, a->d_hidden_shared, a->d_gate_shared, a->d_up_shared, nullptr,
                                  T, 0, T, I, clamp, a->swiglu_limit, nullptr, nullptr, s));
        // d_x = d_gate * Wg + d_up * Wu   (W is [I, H]: K = I, N = H)
        MOK_TRY(launch_rows_gemm_dual(p, a->d_gate_shared, a->d_up_shared, I, a->w_shared_gate, a->w_shared_up, a->d_x_shared, H, s));
        MOK_TRY(launch_wgrad_gemm(p, d_y, H, a->hidden_shared, I, a->d_w_shared_down, s));
        MOK_TRY(launch_wgrad_gemm(p, a->d_gate_shared, I, x, H, a->d_w_shared_gate, s));
        MOK_TRY(launch_wgrad_gemm(p, a->d_up_shared, I, x, H, a->d_w_shared_up, s));
    }

    float* row_weight = a->row_scratch;
    float* row_grad = a->row_scratch + a->macrobatch_size;
    for (int wi = 0; wi < num_windows(a); ++wi) {
        const RowWindow w = window(a, wi);
        const GemmProblem p = routed_problem(a, w);
        if (wi > 0) MOK_TRY(routed_up_to_hidden(a, w, s));   // the saved context only covers window 0
        MOK_TRY(launch_dispatch(a->d_y_ptrs, a->router_weight_ptrs, a->ep_size, w, a->topk, T, H, a->d_y_routed, row_weight, 0, s));
        MOK_TRY(launch_rows_gemm(p, a->d_y_routed, H, a->w_routed_down, nullptr, a->d_hidden_routed, nullptr, I, true, s));
        MOK_TRY(launch_swiglu_bwd(a->gate_routed, a->up_routed, a->d_hidden_routed, a->d_gate_routed, a->d_up_routed,
                                  a->num_tokens, 0, w.row_begin, w.row_end, I, clamp, a->swiglu_limit, row_weight, row_grad, s));
        MOK_TRY(launch_rows_gemm_dual(p, a->d_gate_routed, a->d_up_routed, I, a->w_routed_gate, a->w_routed_up, a->d_x_routed, H, s));
        MOK_TRY(launch_wgrad_gemm(p, a->d_y_routed, H, a->hidden_routed, I, a->d_w_routed_down, s));
        MOK_TRY(launch_wgrad_gemm(p, a->d_gate_routed, I, a->x_routed, H, a->d_w_routed_gate, s));
        MOK_TRY(launch_wgrad_gemm(p, a->d_up_routed, I, a->x_routed, H, a->d_w_routed_up, s));
        MOK_TRY(launch_combine(a->d_x_routed_ptrs, a->d_router_weight_ptrs, a->ep_size, w, a->topk, T, H, a->d_x_routed,
                               row_grad, 0, s));
    }
    MOK_TRY(launch_zero_empty_wgrads(a->tokens_per_expert, a->num_local_experts, a->d_w_routed_gate, a->d_w_routed_up,
                                     a->d_w_routed_down, static_cast<long long>(H) * I, s));
    return MOK_OK;
}
