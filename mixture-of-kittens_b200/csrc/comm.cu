// Cross-GPU pieces: route all-gather, device barrier, token dispatch (pull rows from the owning rank) and
// combine (push rows into the owning rank's slot buffer).  Peer memory is reached with plain loads and stores
// through the per-rank virtual addresses of the symmetric buffers; nothing here needs a multicast object.
#include "comm.cuh"

namespace mok {
namespace {

struct PeerTable {
    uint64_t ptr[MOK_MAX_EP];
};

int fill_table(PeerTable& t, const uint64_t* ptrs, int ep) {
    if (ptrs == nullptr || ep < 1 || ep > MOK_MAX_EP) return MOK_ERR_INVALID_ARGUMENT;
    for (int i = 0; i < MOK_MAX_EP; ++i) t.ptr[i] = i < ep ? ptrs[i] : 0;
    for (int i = 0; i < ep; ++i)
        if (t.ptr[i] == 0 || (t.ptr[i] & 15u) != 0) return MOK_ERR_INVALID_ARGUMENT;
    return MOK_OK;
}

// ---- all-gather of the int32 routes ----------------------------------------------------------------------
__global__ void all_gather_kernel(const int4* __restrict__ src, long long n_vec, PeerTable peers, int ep, int rank) {
    const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
    for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n_vec; i += stride) {
        const int4 v = src[i];
        for (int p = 0; p < ep; ++p) {
            const int peer = (rank + p) % ep;   // start at self, spread the first stores over different links
            reinterpret_cast<int4*>(peers.ptr[peer])[static_cast<long long>(rank) * n_vec + i] = v;
        }
    }
}

// ---- barrier -----------------------------------------------------------------------------------------------
__global__ void barrier_kernel(int* local_counter, PeerTable peers, int ep, int* target, uint32_t* status,
                               unsigned long long timeout_ns) {
    if (threadIdx.x != 0 || blockIdx.x != 0) return;
    const int goal = *target + ep;
    *target = goal;
    __threadfence_system();   // everything this GPU wrote before the barrier is visible before the arrival is
    for (int p = 0; p < ep; ++p) {
        int* remote = reinterpret_cast<int*>(peers.ptr[p]);
        asm volatile("red.release.sys.global.add.s32 [%0], 1;" ::"l"(remote) : "memory");
    }
    unsigned long long start;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(start));
    for (unsigned spin = 0;; ++spin) {
        int seen;
        asm volatile("ld.relaxed.sys.global.s32 %0, [%1];" : "=r"(seen) : "l"(local_counter) : "memory");
        if (seen - goal >= 0) break;
        if ((spin & 63u) == 63u) {
            unsigned long long now;
            asm volatile("mov.u64 %0, %globaltimer;" : "=l"(now));
            if (now - start > timeout_ns) {
                if (status != nullptr) atomicOr(status, (uint32_t)MOK_STATUS_BARRIER_TIMEOUT);
                break;
            }
            __nanosleep(64);
        }
    }
    asm volatile("fence.acquire.sys;" ::: "memory");
}

__device__ __forceinline__ uint32_t scale_pair(uint32_t v, float w) {
    const float2 f = unpack_bf16x2(v);
    return pack_bf16x2(f.x * w, f.y * w);
}
__device__ __forceinline__ uint4 scale_vec(uint4 a, float w) {
    return make_uint4(scale_pair(a.x, w), scale_pair(a.y, w), scale_pair(a.z, w), scale_pair(a.w, w));
}

// ---- staging of de-duplicated tokens -----------------------------------------------------------------------
// One warp per staged token of the range first used by rows [from_row, min(to_row, *num_tokens)).
__global__ void __launch_bounds__(256) stage_tokens_kernel(PeerTable src, const int* __restrict__ unique_peer,
                                                            const int* __restrict__ unique_token,
                                                            const int* __restrict__ unique_before,
                                                            const int* __restrict__ num_tokens, int from_row, int to_row, int ep,
                                                            int self_rank, int tokens_per_rank, int hidden, int staged_rows,
                                                            uint4* __restrict__ staged, uint32_t* status) {
    const int hi_row = min(to_row, *num_tokens);
    if (hi_row <= from_row) return;
    const int u_begin = unique_before[from_row / 256];
    const int u_end = min(unique_before[hi_row / 256], staged_rows);
    const int vec_per_row = hidden / 8;
    const int warps = (gridDim.x * blockDim.x) >> 5;
    const int lane = threadIdx.x & 31;
    for (int u = u_begin + ((blockIdx.x * blockDim.x + threadIdx.x) >> 5); u < u_end; u += warps) {
        const int peer = unique_peer[u];
        const int token = unique_token[u];
        if (peer == self_rank) continue;   // rows of local tokens read the local input directly
        if (peer < 0 || peer >= ep || token < 0 || token >= tokens_per_rank) {
            if (lane == 0 && status != nullptr) atomicOr(status, (uint32_t)MOK_STATUS_BAD_SCHEDULE_ENTRY);
            continue;
        }
        const uint4* in = reinterpret_cast<const uint4*>(src.ptr[peer]) + static_cast<size_t>(token) * vec_per_row;
        uint4* out = staged + static_cast<size_t>(u) * vec_per_row;
        int v = lane;
        for (; v + 96 < vec_per_row; v += 128) {   // four independent 16-byte loads in flight per lane
            const uint4 a = in[v], b = in[v + 32], c = in[v + 64], d = in[v + 96];
            out[v] = a; out[v + 32] = b; out[v + 64] = c; out[v + 96] = d;
        }
        for (; v < vec_per_row; v += 32) out[v] = in[v];
    }
}

// ---- dispatch ----------------------------------------------------------------------------------------------
// One warp per schedule row: dst[row - row_begin] = src_peer[token] (optionally * router weight, rounded to bf16).
// With row_source != nullptr the rows of other ranks' tokens are read from the local staging buffer instead.
template <bool SCALE>
__global__ void __launch_bounds__(256) dispatch_kernel(PeerTable src, PeerTable weights, const int* __restrict__ peer_rank,
                                                        const int* __restrict__ peer_token, const int* __restrict__ num_tokens,
                                                        int row_begin, int row_end, int ep, int topk, int tokens_per_rank,
                                                        int hidden, uint4* __restrict__ dst, float* __restrict__ row_weight,
                                                        uint32_t* status, const int* __restrict__ row_source,
                                                        const uint4* __restrict__ staged, int staged_rows, int self_rank) {
    const int hi = min(row_end, *num_tokens);
    const int vec_per_row = hidden / 8;
    const int warps = (gridDim.x * blockDim.x) >> 5;
    const int lane = threadIdx.x & 31;
    for (int row = row_begin + ((blockIdx.x * blockDim.x + threadIdx.x) >> 5); row < hi; row += warps) {
        const int peer = peer_rank[row];
        const int route = peer_token[row];
        uint4* out = dst + static_cast<size_t>(row - row_begin) * vec_per_row;
        bool valid = peer >= 0;
        if (valid && (peer >= ep || route < 0 || route >= tokens_per_rank * topk)) {
            if (lane == 0 && status != nullptr) atomicOr(status, (uint32_t)MOK_STATUS_BAD_SCHEDULE_ENTRY);
            valid = false;
        }
        if (!valid) {   // padding row: zeros keep the GEMMs and the weight gradients clean
            for (int v = lane; v < vec_per_row; v += 32) out[v] = make_uint4(0, 0, 0, 0);
            if (SCALE && lane == 0) row_weight[row - row_begin] = 0.0f;
            continue;
        }
        const uint4* in = reinterpret_cast<const uint4*>(src.ptr[peer]) + static_cast<size_t>(route / topk) * vec_per_row;
        if (row_source != nullptr && peer != self_rank) {
            const int u = row_source[row];
            if (u < 0 || u >= staged_rows) {
                if (lane == 0 && status != nullptr) atomicOr(status, (uint32_t)MOK_STATUS_BAD_SCHEDULE_ENTRY);
                for (int v = lane; v < vec_per_row; v += 32) out[v] = make_uint4(0, 0, 0, 0);
                if (SCALE && lane == 0) row_weight[row - row_begin] = 0.0f;
                continue;
            }
            in = staged + static_cast<size_t>(u) * vec_per_row;
        }
        float w = 1.0f;
        if (SCALE) {
            w = reinterpret_cast<const float*>(weights.ptr[peer])[route];
            if (lane == 0) row_weight[row - row_begin] = w;
        }
        int v = lane;
        for (; v + 96 < vec_per_row; v += 128) {   // four independent 16-byte loads in flight per lane
            uint4 a = in[v], b = in[v + 32], c = in[v + 64], d = in[v + 96];
            if (SCALE) { a = scale_vec(a, w); b = scale_vec(b, w); c = scale_vec(c, w); d = scale_vec(d, w); }
            out[v] = a; out[v + 32] = b; out[v + 64] = c; out[v + 96] = d;
        }
        for (; v < vec_per_row; v += 32) {
            uint4 a = in[v];
            if (SCALE) a = scale_vec(a, w);
            out[v] = a;
        }
    }
}

// ---- combine -----------------------------------------------------------------------------------------------
// One warp per schedule row: dst_peer[route] = src[row - row_begin]; optionally one fp32 per row as well.
__global__ void __launch_bounds__(256) combine_kernel(PeerTable dst, PeerTable dst_scalar, const int* __restrict__ peer_rank,
                                                       const int* __restrict__ peer_token, const int* __restrict__ num_tokens,
                                                       int row_begin, int row_end, int ep, int topk, int tokens_per_rank,
                                                       int hidden, const uint4* __restrict__ src,
                                                       const float* __restrict__ row_scalar, uint32_t* status) {
    const int hi = min(row_end, *num_tokens);
    const int vec_per_row = hidden / 8;
    const int warps = (gridDim.x * blockDim.x) >> 5;
    const int lane = threadIdx.x & 31;
    for (int row = row_begin + ((blockIdx.x * blockDim.x + threadIdx.x) >> 5); row < hi; row += warps) {
        const int peer = peer_rank[row];
        const int route = peer_token[row];
        if (peer < 0) continue;
        if (peer >= ep || route < 0 || route >= tokens_per_rank * topk) {
            if (lane == 0 && status != nullptr) atomicOr(status, (uint32_t)MOK_STATUS_BAD_SCHEDULE_ENTRY);
            continue;
        }
        const uint4* in = src + static_cast<size_t>(row - row_begin) * vec_per_row;
        uint4* out = reinterpret_cast<uint4*>(dst.ptr[peer]) + static_cast<size_t>(route) * vec_per_row;
        int v = lane;
        for (; v + 96 < vec_per_row; v += 128) {
            const uint4 a = in[v], b = in[v + 32], c = in[v + 64], d = in[v + 96];
            out[v] = a; out[v + 32] = b; out[v + 64] = c; out[v + 96] = d;
        }
        for (; v < vec_per_row; v += 32) out[v] = in[v];
        if (row_scalar != nullptr && lane == 0)
            reinterpret_cast<float*>(dst_scalar.ptr[peer])[route] = row_scalar[row - row_begin];
    }
}

int comm_grid(int rows, int num_ctas_hint) {
    int grid = num_ctas_hint > 0 ? num_ctas_hint : sm_count() * 8;
    const int needed = (rows + 7) / 8;   // 8 warps per CTA
    if (grid > needed) grid = needed;
    return grid < 1 ? 1 : grid;
}

}  // namespace

int launch_stage_tokens(const uint64_t* src_ptrs, int ep, const StagedTokens& t, const int32_t* num_tokens, int from_row, int to_row,
                        int tokens_per_rank, int hidden, int num_ctas, uint32_t* status, cudaStream_t stream) {
    PeerTable src;
    int rc = fill_table(src, src_ptrs, ep);
    if (rc != MOK_OK) return rc;
    if (hidden % 8 != 0 || from_row < 0 || to_row <= from_row || from_row % 256 != 0 || to_row % 256 != 0 || !t.unique_peer ||
        !t.unique_token || !t.unique_before || !t.staged || t.staged_rows <= 0 || num_tokens == nullptr)
        return MOK_ERR_INVALID_ARGUMENT;
    // at most one staged token per row of the range
    const int grid = comm_grid(to_row - from_row, num_ctas);
    stage_tokens_kernel<<<grid, 256, 0, stream>>>(src, t.unique_peer, t.unique_token, t.unique_before, num_tokens, from_row, to_row,
                                                  ep, t.self_rank, tokens_per_rank, hidden, t.staged_rows,
                                                  static_cast<uint4*>(t.staged), status);
    MOK_LAUNCH_CHECK("stage_tokens_kernel");
    return MOK_OK;
}

int launch_dispatch(const uint64_t* src_ptrs, const uint64_t* weight_ptrs, int ep, const RowWindow& w, int topk,
                    int tokens_per_rank, int hidden, void* dst, float* row_weight, int num_ctas, cudaStream_t stream,
                    const StagedTokens* staged) {
    PeerTable src, wt{};
    int rc = fill_table(src, src_ptrs, ep);
    if (rc != MOK_OK) return rc;
    if (hidden % 8 != 0 || w.row_end <= w.row_begin) return MOK_ERR_INVALID_ARGUMENT;
    if (staged != nullptr && (!staged->row_source || !staged->staged || staged->staged_rows <= 0)) return MOK_ERR_INVALID_ARGUMENT;
    const int* row_source = staged ? staged->row_source : nullptr;
    const uint4* staged_rows_ptr = staged ? static_cast<const uint4*>(staged->staged) : nullptr;
    const int n_staged = staged ? staged->staged_rows : 0, self = staged ? staged->self_rank : -1;
    const int grid = comm_grid(w.row_end - w.row_begin, num_ctas);
    if (weight_ptrs != nullptr) {
        if ((rc = fill_table(wt, weight_ptrs, ep)) != MOK_OK) return rc;
        dispatch_kernel<true><<<grid, 256, 0, stream>>>(src, wt, w.peer_rank, w.peer_token, w.num_tokens, w.row_begin,
                                                        w.row_end, ep, topk, tokens_per_rank, hidden,
                                                        static_cast<uint4*>(dst), row_weight, w.status, row_source,
                                                        staged_rows_ptr, n_staged, self);
    } else {
        dispatch_kernel<false><<<grid, 256, 0, stream>>>(src, wt, w.peer_rank, w.peer_token, w.num_tokens, w.row_begin,
                                                         w.row_end, ep, topk, tokens_per_rank, hidden,
                                                         static_cast<uint4*>(dst), nullptr, w.status, row_source,
                                                         staged_rows_ptr, n_staged, self);
    }
    MOK_LAUNCH_CHECK("dispatch_kernel");
    return MOK_OK;
}

int launch_combine(const uint64_t* dst_ptrs, const uint64_t* scalar_ptrs, int ep, const RowWindow& w, int topk,
                   int tokens_per_rank, int hidden, const void* src, const float* row_scalar, int num_ctas,
                   cudaStream_t stream) {
    PeerTable dst, sc{};
    int rc = fill_table(dst, dst_ptrs, ep);
    if (rc != MOK_OK) return rc;
    if (hidden % 8 != 0 || w.row_end <= w.row_begin) return MOK_ERR_INVALID_ARGUMENT;
    if (row_scalar != nullptr) {
        if (scalar_ptrs == nullptr) return MOK_ERR_INVALID_ARGUMENT;
        for (int i = 0; i < MOK_MAX_EP; ++i) sc.ptr[i] = i < ep ? scalar_ptrs[i] : 0;
    }
    const int grid = comm_grid(w.row_end - w.row_begin, num_ctas);
    combine_kernel<<<grid, 256, 0, stream>>>(dst, sc, w.peer_rank, w.peer_token, w.num_tokens, w.row_begin, w.row_end, ep,
                                             topk, tokens_per_rank, hidden, static_cast<const uint4*>(src), row_scalar,
                                             w.status);
    MOK_LAUNCH_CHECK("combine_kernel");
    return MOK_OK;
}

}  // namespace mok

extern "C" int mok_all_gather_top_experts(const int32_t* top_experts, int64_t num_routes, const uint64_t* peer_buffers,
                                          int ep_size, int rank, mok_stream_t stream) {
    using namespace mok;
    if (top_experts == nullptr || num_routes <= 0 || num_routes % 4 != 0 || rank < 0 || rank >= ep_size)
        return MOK_ERR_INVALID_ARGUMENT;
    PeerTable peers;
    int rc = fill_table(peers, peer_buffers, ep_size);
    if (rc != MOK_OK) return rc;
    const long long n_vec = num_routes / 4;
    int grid = static_cast<int>((n_vec + 255) / 256);
    if (grid > sm_count() * 4) grid = sm_count() * 4;
    all_gather_kernel<<<grid, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(reinterpret_cast<const int4*>(top_experts),
                                                                               n_vec, peers, ep_size, rank);
    MOK_LAUNCH_CHECK("all_gather_kernel");
    return MOK_OK;
}

extern "C" int mok_barrier_all(int32_t* local_counter, const uint64_t* peer_counters, int ep_size, int32_t* target,
                               uint32_t* status, int timeout_ms, mok_stream_t stream) {
    using namespace mok;
    if (local_counter == nullptr || target == nullptr) return MOK_ERR_INVALID_ARGUMENT;
    PeerTable peers;
    if (peer_counters == nullptr || ep_size < 1 || ep_size > MOK_MAX_EP) return MOK_ERR_INVALID_ARGUMENT;
    for (int i = 0; i < MOK_MAX_EP; ++i) peers.ptr[i] = i < ep_size ? peer_counters[i] : 0;
    for (int i = 0; i < ep_size; ++i)
        if (peers.ptr[i] == 0 || (peers.ptr[i] & 3u) != 0) return MOK_ERR_INVALID_ARGUMENT;
    const unsigned long long timeout_ns = (timeout_ms > 0 ? static_cast<unsigned long long>(timeout_ms) : 20000ull) * 1000000ull;
    barrier_kernel<<<1, 32, 0, reinterpret_cast<cudaStream_t>(stream)>>>(local_counter, peers, ep_size, target, status,
                                                                         timeout_ns);
    MOK_LAUNCH_CHECK("barrier_kernel");
    return MOK_OK;
}

extern "C" int mok_dispatch_rows(const uint64_t* src_ptrs, const uint64_t* weight_ptrs, int ep_size, const int32_t* peer_rank,
                                 const int32_t* peer_token_idx, const int32_t* num_tokens, int row_begin, int row_end, int topk,
                                 int num_local_tokens, int hidden, void* dst, float* row_weight, int num_ctas, uint32_t* status,
                                 mok_stream_t stream) {
    if (peer_rank == nullptr || peer_token_idx == nullptr || num_tokens == nullptr || dst == nullptr || topk <= 0 ||
        num_local_tokens <= 0 || (weight_ptrs != nullptr && row_weight == nullptr))
        return MOK_ERR_INVALID_ARGUMENT;
    const mok::RowWindow w{peer_rank, peer_token_idx, num_tokens, row_begin, row_end, status};
    return mok::launch_dispatch(src_ptrs, weight_ptrs, ep_size, w, topk, num_local_tokens, hidden, dst, row_weight, num_ctas,
                                reinterpret_cast<cudaStream_t>(stream));
}

extern "C" int mok_combine_rows(const uint64_t* dst_ptrs, const uint64_t* scalar_ptrs, int ep_size, const int32_t* peer_rank,
                                const int32_t* peer_token_idx, const int32_t* num_tokens, int row_begin, int row_end, int topk,
                                int num_local_tokens, int hidden, const void* src, const float* row_scalar, int num_ctas,
                                uint32_t* status, mok_stream_t stream) {
    if (peer_rank == nullptr || peer_token_idx == nullptr || num_tokens == nullptr || src == nullptr || topk <= 0 ||
        num_local_tokens <= 0)
        return MOK_ERR_INVALID_ARGUMENT;
    const mok::RowWindow w{peer_rank, peer_token_idx, num_tokens, row_begin, row_end, status};
    return mok::launch_combine(dst_ptrs, scalar_ptrs, ep_size, w, topk, num_local_tokens, hidden, src, row_scalar, num_ctas,
                               reinterpret_cast<cudaStream_t>(stream));
}

extern "C" int mok_stage_unique_rows(const uint64_t* src_ptrs, int ep_size, int rank, const int32_t* unique_peer,
                                     const int32_t* unique_token, const int32_t* unique_before, const int32_t* num_tokens,
                                     int from_row, int to_row, int num_local_tokens, int hidden, void* staged, int staged_rows,
                                     int num_ctas, uint32_t* status, mok_stream_t stream) {
    mok::StagedTokens t{nullptr, unique_peer, unique_token, unique_before, staged, staged_rows, rank};
    return mok::launch_stage_tokens(src_ptrs, ep_size, t, num_tokens, from_row, to_row, num_local_tokens, hidden, num_ctas, status,
                                    reinterpret_cast<cudaStream_t>(stream));
}

extern "C" int mok_dispatch_rows_staged(const uint64_t* src_ptrs, const uint64_t* weight_ptrs, int ep_size, int rank,
                                        const int32_t* peer_rank, const int32_t* peer_token_idx, const int32_t* num_tokens,
                                        const int32_t* row_source, const void* staged, int staged_rows, int row_begin, int row_end,
                                        int topk, int num_local_tokens, int hidden, void* dst, float* row_weight, int num_ctas,
                                        uint32_t* status, mok_stream_t stream) {
    if (peer_rank == nullptr || peer_token_idx == nullptr || num_tokens == nullptr || dst == nullptr || topk <= 0 ||
        num_local_tokens <= 0 || (weight_ptrs != nullptr && row_weight == nullptr) || rank < 0 || rank >= ep_size)
        return MOK_ERR_INVALID_ARGUMENT;
    const mok::RowWindow w{peer_rank, peer_token_idx, num_tokens, row_begin, row_end, status};
    const mok::StagedTokens t{row_source, nullptr, nullptr, nullptr, const_cast<void*>(staged), staged_rows, rank};
    return mok::launch_dispatch(src_ptrs, weight_ptrs, ep_size, w, topk, num_local_tokens, hidden, dst, row_weight, num_ctas,
                                reinterpret_cast<cudaStream_t>(stream), &t);
}
