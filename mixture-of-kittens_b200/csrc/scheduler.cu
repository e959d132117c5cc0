// Device-side schedule builder: per-(expert, peer) histogram, prefix sums, and a scatter that reproduces the
// row order of the reference scheduler bit for bit, without any host synchronisation.
//
// Order contract (reference csrc/scheduler.cuh:106-143): the routes of one peer are visited by a 1024-thread
// block with a thread stride, thread 0's routes first, then thread 1's, ...; the j-th visited route of peer p
// for local expert e lands on row  base_e + sum_r min(n_r, j) + #{r < p : n_r > j}.
//
// Here the visiting sequence of each peer is cut into chunks of 1024 positions.  Pass 1 counts routes per
// (peer, chunk, expert); pass 2 turns the counts into exclusive offsets and builds the padded expert bases with
// warp prefix sums; pass 3 re-reads each chunk, ranks its routes inside the chunk with warp match/ballot
// operations and writes the rows.  Each route is read twice in total, instead of 2 * E_loc times.
#include "mok_common.cuh"

namespace mok {
namespace {

constexpr int kChunk = 1024;          // positions of the visiting sequence per block (= threads per block)
constexpr int kVisitThreads = 1024;   // thread count of the reference scheduler block that defines the order
constexpr int kExpertPadding = 256;

// Route index visited at position q of the sequence "thread 0's routes, then thread 1's, ...".
__device__ __forceinline__ int route_at_position(int q, int routes) {
    const int full = routes / kVisitThreads;       // every thread owns at least `full` routes
    const int extra = routes - full * kVisitThreads;   // threads [0, extra) own one more
    const int head = extra * (full + 1);
    int thread, iter;
    if (q < head) {
        thread = q / (full + 1);
        iter = q - thread * (full + 1);
    } else {
        const int r = q - head;
        thread = extra + r / full;
        iter = r - (thread - extra) * full;
    }
    return iter * kVisitThreads + thread;
}

// scratch layout (int32):  counts[ep][chunks][E_loc] | totals[E_loc][ep] | expert_base[E_loc]
struct Scratch {
    int* counts;
    int* totals;
    int* expert_base;
};
__host__ __device__ inline Scratch carve(int* scratch, int ep, int chunks, int e_loc) {
    Scratch s;
    s.counts = scratch;
    s.totals = s.counts + static_cast<size_t>(ep) * chunks * e_loc;
    s.expert_base = s.totals + static_cast<size_t>(e_loc) * ep;
    return s;
}

__global__ void __launch_bounds__(kChunk) count_kernel(const int* __restrict__ topk_all, int routes, int chunks, int e_loc,
                                                       int first_expert, int* counts, int* peer_rank, int* peer_token,
                                                       int capacity) {
    extern __shared__ int hist[];
    const int peer = blockIdx.y;
    const int chunk = blockIdx.x;
    for (int i = threadIdx.x; i < e_loc; i += blockDim.x) hist[i] = 0;
    // the schedule arrays start as "padding everywhere"
    const int nblocks = gridDim.x * gridDim.y;
    const int block = blockIdx.y * gridDim.x + blockIdx.x;
    for (int i = block * kChunk + threadIdx.x; i < capacity; i += nblocks * kChunk) {
        peer_rank[i] = -1;
        peer_token[i] = -1;
    }
    __syncthreads();
    const int q = chunk * kChunk + threadIdx.x;
    if (q < routes) {
        const int e = topk_all[static_cast<size_t>(peer) * routes + route_at_position(q, routes)] - first_expert;
        if (e >= 0 && e < e_loc) atomicAdd(&hist[e], 1);
    }
    __syncthreads();
    int* out = counts + (static_cast<size_t>(peer) * chunks + chunk) * e_loc;
    for (int i = threadIdx.x; i < e_loc; i += blockDim.x) out[i] = hist[i];
}

// One block.  counts -> exclusive offsets over chunks (in place); totals[e][p]; padded per-expert sizes; bases.
__global__ void __launch_bounds__(1024) scan_kernel(int ep, int chunks, int e_loc, int capacity, Scratch s,
                                                    int* tokens_per_expert, int* num_tokens, uint32_t* status) {
    __shared__ int warp_sums[32];
    __shared__ int carry_sh;
    for (int pair = threadIdx.x; pair < e_loc * ep; pair += blockDim.x) {
        const int e = pair / ep, p = pair - e * ep;
        int running = 0;
        int* col = s.counts + static_cast<size_t>(p) * chunks * e_loc + e;
        for (int c = 0; c < chunks; ++c) {
            const int v = col[static_cast<size_t>(c) * e_loc];
            col[static_cast<size_t>(c) * e_loc] = running;
            running += v;
        }
        s.totals[pair] = running;
    }
    if (threadIdx.x == 0) carry_sh = 0;
    __syncthreads();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (int base = 0; base < e_loc; base += blockDim.x) {
        const int e = base + threadIdx.x;
        int padded = 0;
        if (e < e_loc) {
            int total = 0;
            for (int p = 0; p < ep; ++p) total += s.totals[e * ep + p];
            padded = (total + kExpertPadding - 1) / kExpertPadding * kExpertPadding;
            tokens_per_expert[e] = padded;
        }
        int incl = padded;   // block-wide inclusive scan: warp shuffles, then the warp totals
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
        const int before = carry_sh + (warp ? warp_sums[warp - 1] : 0) + incl - padded;
        if (e < e_loc) s.expert_base[e] = before;
        __syncthreads();
        if (threadIdx.x == blockDim.x - 1) carry_sh = before + padded;
        __syncthreads();
    }
    if (threadIdx.x == 0) {
        num_tokens[0] = carry_sh;
        if (carry_sh > capacity && status != nullptr) atomicOr(status, (uint32_t)MOK_STATUS_SCHEDULE_OVERFLOW);
    }
}

__global__ void __launch_bounds__(kChunk) scatter_kernel(const int* __restrict__ topk_all, int routes, int chunks, int ep,
                                                         int e_loc, int first_expert, Scratch s, int* peer_rank,
                                                         int* peer_token, int capacity) {
    extern __shared__ int warp_hist[];   // [32 warps][e_loc] -> exclusive offsets over warps
    const int peer = blockIdx.y;
    const int chunk = blockIdx.x;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (int i = threadIdx.x; i < 32 * e_loc; i += blockDim.x) warp_hist[i] = 0;
    __syncthreads();

    const int q = chunk * kChunk + threadIdx.x;
    int route = -1, e = -1;
    if (q < routes) {
        route = route_at_position(q, routes);
        e = topk_all[static_cast<size_t>(peer) * routes + route] - first_expert;
        if (e < 0 || e >= e_loc) e = -1;
    }
    // rank among the lanes of this warp that hold the same expert
    const unsigned same = __match_any_sync(0xffffffffu, e);
    const int rank_in_warp = __popc(same & ((1u << lane) - 1u));
    if (e >= 0 && rank_in_warp == 0) warp_hist[warp * e_loc + e] = __popc(same);
    __syncthreads();
    for (int x = threadIdx.x; x < e_loc; x += blockDim.x) {   // exclusive scan over the 32 warps, per expert
        int running = 0;
        for (int w = 0; w < 32; ++w) {
            const int v = warp_hist[w * e_loc + x];
            warp_hist[w * e_loc + x] = running;
            running += v;
        }
    }
    __syncthreads();
    if (e < 0) return;
    const int j = s.counts[(static_cast<size_t>(peer) * chunks + chunk) * e_loc + e] + warp_hist[warp * e_loc + e] + rank_in_warp;
    int dst = s.expert_base[e];
    const int* n = s.totals + e * ep;
    for (int r = 0; r < ep; ++r) {
        const int nr = n[r];
        dst += min(nr, j) + ((r < peer && nr > j) ? 1 : 0);
    }
    if (dst < capacity) {
        peer_rank[dst] = peer;
        peer_token[dst] = route;
    }
}

}  // namespace
}  // namespace mok

extern "C" int64_t mok_schedule_scratch_bytes(int ep_size, int num_local_tokens, int topk, int num_local_experts) {
    const int64_t routes = static_cast<int64_t>(num_local_tokens) * topk;
    const int64_t chunks = (routes + mok::kChunk - 1) / mok::kChunk;
    return 4 * (ep_size * chunks * num_local_experts + static_cast<int64_t>(num_local_experts) * ep_size + num_local_experts);
}

extern "C" int mok_schedule(const int32_t* topk_all, int ep_size, int num_local_tokens, int topk, int num_local_experts,
                            int schedule_capacity, int rank, int32_t* peer_rank, int32_t* peer_token_idx,
                            int32_t* num_tokens, int32_t* tokens_per_expert, int32_t* scratch, uint32_t* status,
                            mok_stream_t stream_) {
    using namespace mok;
    if (topk_all == nullptr || peer_rank == nullptr || peer_token_idx == nullptr || num_tokens == nullptr ||
        tokens_per_expert == nullptr || scratch == nullptr)
        return MOK_ERR_INVALID_ARGUMENT;
    if (ep_size < 1 || ep_size > MOK_MAX_EP || num_local_tokens <= 0 || topk <= 0 || num_local_experts <= 0 ||
        schedule_capacity <= 0 || rank < 0 || rank >= ep_size)
        return MOK_ERR_INVALID_ARGUMENT;
    if (num_local_experts > MOK_MAX_LOCAL_EXPERTS) return MOK_ERR_TOO_LARGE;
    const int64_t routes64 = static_cast<int64_t>(num_local_tokens) * topk;
    if (routes64 > (1LL << 30)) return MOK_ERR_TOO_LARGE;
    const int routes = static_cast<int>(routes64);
    const int chunks = (routes + kChunk - 1) / kChunk;
    cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
    Scratch s = carve(scratch, ep_size, chunks, num_local_experts);
    const int first = rank * num_local_experts;

    static bool configured[16] = {false};
    int dev = 0;
    MOK_CUDA_CHECK(cudaGetDevice(&dev));
    const size_t scatter_smem = 32 * static_cast<size_t>(num_local_experts) * 4;
    if (scatter_smem > 48 * 1024 && dev < 16 && !configured[dev]) {
        MOK_CUDA_CHECK(cudaFuncSetAttribute(scatter_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 32 * MOK_MAX_LOCAL_EXPERTS * 4));
        configured[dev] = true;
    }
    dim3 grid(chunks, ep_size);
    count_kernel<<<grid, kChunk, num_local_experts * 4, stream>>>(topk_all, routes, chunks, num_local_experts, first,
                                                                 s.counts, peer_rank, peer_token_idx, schedule_capacity);
    MOK_LAUNCH_CHECK("count_kernel");
    scan_kernel<<<1, 1024, 0, stream>>>(ep_size, chunks, num_local_experts, schedule_capacity, s, tokens_per_expert,
                                        num_tokens, status);
    MOK_LAUNCH_CHECK("scan_kernel");
    scatter_kernel<<<grid, kChunk, scatter_smem, stream>>>(topk_all, routes, chunks, ep_size, num_local_experts, first, s,
                                                          peer_rank, peer_token_idx, schedule_capacity);
    MOK_LAUNCH_CHECK("scatter_kernel");
    return MOK_OK;
}

// ---------------------------------------------------------------------------------------------------------
// Schedule builder for callers that cannot allocate device memory
// ---------------------------------------------------------------------------------------------------------
// Some hosts of this library may not call cudaMalloc at the point where they need a schedule: a serving loop
// whose memory pool is frozen after start-up (an allocation there would fragment or overrun a budget that was
// sized once), or a plugin that runs while another framework holds its allocator lock (a nested allocation would
// deadlock or bypass that framework's accounting).  For them the scheduler's scratch lives in this fixed array.
// Every GPU that loads the library holds its own copy until the process exits.
namespace mok {
namespace {
constexpr long long kStaticScratchInts = MOK_SCHEDULE_STATIC_SCRATCH_BYTES / 4;
static __device__ __align__(256) int32_t g_schedule_scratch[kStaticScratchInts];

// The array's name is only a host-side handle; kernels need its device address, which differs per device.
int32_t* static_scratch_address(int device, int* rc) {
    static int32_t* cached[16] = {nullptr};
    *rc = MOK_OK;
    if (device < 0 || device >= 16) {
        *rc = MOK_ERR_UNSUPPORTED;
        return nullptr;
    }
    if (cached[device] == nullptr) {
        void* p = nullptr;
        const cudaError_t err = cudaGetSymbolAddress(&p, g_schedule_scratch);   // resolves for the current device
        if (err != cudaSuccess || p == nullptr) {
            *rc = fail_cuda("cudaGetSymbolAddress(schedule scratch)", err);
            return nullptr;
        }
        cached[device] = static_cast<int32_t*>(p);
    }
    return cached[device];
}
}  // namespace
}  // namespace mok

extern "C" int mok_schedule_static(const int32_t* topk_all, int ep_size, int num_local_tokens, int topk,
                                   int num_local_experts, int schedule_capacity, int rank, int32_t* peer_rank,
                                   int32_t* peer_token_idx, int32_t* num_tokens, int32_t* tokens_per_expert,
                                   uint32_t* status, mok_stream_t stream) {
    if (ep_size < 1 || num_local_tokens <= 0 || topk <= 0 || num_local_experts <= 0) return MOK_ERR_INVALID_ARGUMENT;
    const int64_t need = mok_schedule_scratch_bytes(ep_size, num_local_tokens, topk, num_local_experts);
    if (need > MOK_SCHEDULE_STATIC_SCRATCH_BYTES) {
        mok::set_last_error("mok_schedule_static: sizes need more scratch than MOK_SCHEDULE_STATIC_SCRATCH_BYTES; "
                            "use mok_schedule with caller-provided scratch", cudaErrorInvalidValue);
        return MOK_ERR_TOO_LARGE;
    }
    int device = 0;
    MOK_CUDA_CHECK(cudaGetDevice(&device));
    int rc = MOK_OK;
    int32_t* scratch = mok::static_scratch_address(device, &rc);
    if (scratch == nullptr) return rc;
    // Every scratch word the kernels read is written earlier in the same call, so stale contents of the previous
    // call need no clearing.
    return mok_schedule(topk_all, ep_size, num_local_tokens, topk, num_local_experts, schedule_capacity, rank, peer_rank,
                        peer_token_idx, num_tokens, tokens_per_expert, scratch, status, stream);
}
