// Grouped bf16 GEMM for sm_100a: tcgen05.mma with fp32 accumulators in tensor memory, operands staged in
// shared memory by TMA (128-byte swizzle), persistent CTA pairs over a static tile list.
//
// Two CTAs (a cluster of 2, "cta_group::2") share one 256 x 256 output tile: each CTA stages its own 128 rows
// of A and its own 128-column half of B (plain TMA loads, 32 KB per K step and CTA instead of 48 KB for a
// 128 x 256 single-CTA tile), the leader CTA issues one 256-row MMA per 16-wide K slice that reads both CTAs'
// shared memory, and each CTA owns the 128 x 256 fp32 accumulator of its rows in its tensor memory.
// One CTA = 6 warps:
//   warp 0        TMA producer (one elected lane); credits the leader's "full" barrier
//   warp 1        MMA issuer (leader CTA only, one elected lane); owns the tensor-memory allocation
//   warps 2..5    epilogue: tensor memory -> registers -> bf16 -> global (each warp owns 32 accumulator lanes)
// K step 64, 6-stage operand ring, two 256-column accumulators so the epilogue of tile i overlaps the main
// loop of tile i+1.
//
// Three forms (the roles the reference gives its grouped GEMM, csrc/megakernel/grouped_gemm.cuh):
//   rows / B [E,N,K]   D[r,:] = A[r,:] B[e]^T          forward gate, up, down            (A, B K-major)
//   rows / B [E,K,N]   D[r,:] = sum_s A_s[r,:] B_s[e]  dgrad down; dgrad gate+up (2 sets) (B MN-major)
//   wgrad              D[e] (+)= A[rows_e,:]^T B[rows_e,:], K = rows of expert e          (A, B MN-major)
// Every output element has exactly one writer and a fixed K order, so results are run-to-run identical.
//
// Fused gate / up form (forward): one tile holds 128 gate columns and the same 128 up columns (CTA 0 stages the gate
// weights, CTA 1 the up weights, so accumulator columns [0, 128) are gate and [128, 256) up); the epilogue rounds both
// to bf16, stores them (backward needs them) and forms hidden = silu(gate) * up from the rounded values, which is
// exactly what a separate SwiGLU pass over the stored gate / up would compute, without reading them back.
#include "gemm_tiles.cuh"
#include "swiglu_math.cuh"

namespace mok {
namespace {

using namespace tiles;

constexpr int BK = 64;
constexpr int STAGES = 6;
constexpr int A_TILE_BYTES = BM_CTA * BK * 2;        // 16 KB
constexpr int B_TILE_BYTES = BN_CTA * BK * 2;        // 16 KB
constexpr int STAGE_BYTES = A_TILE_BYTES + B_TILE_BYTES;
constexpr int CHUNK_BYTES = 64 * BK * 2;             // one 64(MN) x 64(K) block of an MN-major operand: 8 KB


struct SharedLayout {
    // dynamic shared memory, 1024-byte aligned base (identical in both CTAs of a pair):
    //   [0, STAGES*STAGE_BYTES)  operand ring, then barriers, bookkeeping, and the expert row prefix
    static constexpr int kBarrierOffset = STAGES * STAGE_BYTES;
    static constexpr int kFull = kBarrierOffset;                  // STAGES x 8 B (leader's are used)
    static constexpr int kEmpty = kFull + 8 * STAGES;             // STAGES x 8 B
    static constexpr int kTmemFull = kEmpty + 8 * STAGES;         // 2 x 8 B
    static constexpr int kTmemEmpty = kTmemFull + 16;             // 2 x 8 B (leader's are used)
    static constexpr int kTmemPtr = kTmemEmpty + 16;              // 4 B
    static constexpr int kAbort = kTmemPtr + 4;                   // 4 B
    static constexpr int kEpilogue = kBarrierOffset + 256;        // 4 warps x 32 rows x 144 B staging patches
    static constexpr int kCum = kEpilogue + 4 * kEpiWarpBytes;    // (E + 1) x 4 B
};


template <int MODE, bool B_MN, bool FUSED>
__global__ void __launch_bounds__(NUM_THREADS, 1)
grouped_gemm_kernel(const __grid_constant__ CUtensorMap tmA0, const __grid_constant__ CUtensorMap tmB0,
                    const __grid_constant__ CUtensorMap tmA1, const __grid_constant__ CUtensorMap tmB1,
                    const KernelParams p) {
    constexpr bool A_MN = (MODE == MODE_WGRAD);
    static_assert(MODE == MODE_ROWS || B_MN, "the weight-gradient form reads both operands MN-major");
    static_assert(!FUSED || (MODE == MODE_ROWS && !B_MN), "the fused gate / up form is a forward rows form");

    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
    const uint32_t bar_full = smem_base + SharedLayout::kFull;
    const uint32_t bar_empty = smem_base + SharedLayout::kEmpty;
    const uint32_t bar_tmem_full = smem_base + SharedLayout::kTmemFull;
    const uint32_t bar_tmem_empty = smem_base + SharedLayout::kTmemEmpty;
    volatile uint32_t* tmem_ptr_slot = reinterpret_cast<volatile uint32_t*>(smem_gen + SharedLayout::kTmemPtr);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem_gen + SharedLayout::kAbort);
    int* cum = reinterpret_cast<int*>(smem_gen + SharedLayout::kCum);

    // A launch for a row window behind the schedule's last row (the host sizes launches for the capacity, the row
    // count stays on the device) leaves before anything is set up; both CTAs of every pair take the same branch.
    if (min(p.row_end, p.tokens_per_expert == nullptr ? p.dense_rows : *p.num_tokens) <= p.row_begin) return;

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int cta_rank = static_cast<int>(cluster_cta_rank());   // 0 = leader of the pair
    const int pair = blockIdx.x >> 1;
    const int num_pairs = gridDim.x >> 1;

    // ---- set-up ---------------------------------------------------------------------------------------
    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(bar_full + 8 * s, 1);      // leader: one arrive.expect_tx covering both CTAs' bytes
            mbar_init(bar_empty + 8 * s, 1);     // one commit per use, delivered to both CTAs
        }
        for (int s = 0; s < 2; ++s) {
            mbar_init(bar_tmem_full + 8 * s, 1);
            mbar_init(bar_tmem_empty + 8 * s, 8);   // leader: four epilogue warps of each CTA
        }
        *abort_flag = 0;
        mbar_fence_init();
        tma_prefetch_desc(&tmA0);
        tma_prefetch_desc(&tmB0);
        if (p.k_sets > 1) tma_prefetch_desc(&tmA1);
        if (p.k_sets > 1 || p.n_sets > 1) tma_prefetch_desc(&tmB1);
    }
    if (warp == 1) {
        tmem_alloc_pair(smem_u32(const_cast<uint32_t*>(tmem_ptr_slot)), TMEM_COLS);
        tmem_relinquish_pair();
    }
    if (warp == 2) expert_row_prefix(p, cum, lane);   // cum[0..E]: first schedule row of every expert
    tc_fence_before_sync();
    __syncthreads();
    cluster_sync_all();     // both CTAs' barriers exist before either one signals the other
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_ptr_slot;

    const int total_rows = p.tokens_per_expert == nullptr ? p.dense_rows : *p.num_tokens;
    const int lo = p.row_begin;
    const int hi = min(p.row_end, total_rows);
    const int num_tiles = total_tiles<MODE>(p, lo, hi);

    constexpr uint32_t kIdesc = umma_idesc_bf16(BM, BN, A_MN, B_MN);

    if (warp == 0) {
        // ---- TMA producer (both CTAs) -----------------------------------------------------------------
        int stage = 0;
        uint32_t phase = 0;
        bool ok = true;
        for (int t = pair; t < num_tiles && ok; t += num_pairs) {
            Tile tile;
            if (!decode_tile<MODE, BK>(p, cum, lo, hi, t, tile)) continue;
            for (int kb = 0; kb < tile.k_blocks; ++kb) {
                ok = mbar_wait(bar_empty + 8 * stage, phase ^ 1u, abort_flag, p.status);
                if (!ok) break;
                if (lane == 0) {
                    const uint32_t full_local = bar_full + 8 * stage;
                    const uint32_t full = full_local & kPairLeaderMask;   // the leader's barrier collects all bytes
                    const uint32_t a_dst = smem_base + stage * STAGE_BYTES;
                    const uint32_t b_dst = a_dst + A_TILE_BYTES;
                    if (cta_rank == 0) mbar_expect_tx(full_local, 2 * STAGE_BYTES);
                    if (MODE == MODE_ROWS) {
                        const int kset = kb >= p.k_blocks ? 1 : 0;
                        const int kk = (kb - kset * p.k_blocks) * BK;
                        tma_load_4d_pair(a_dst, kset ? &tmA1 : &tmA0, full, kk, tile.row0 - p.row_begin + cta_rank * BM_CTA, 0, 0);
                        // fused gate / up: CTA 0 stages the tile's 128 gate rows, CTA 1 the same 128 up rows
                        const CUtensorMap* bmap = FUSED ? (cta_rank ? &tmB1 : &tmB0) : ((kset || tile.set) ? &tmB1 : &tmB0);
                        const int n_cta = FUSED ? tile.n0 / 2 : tile.n0 + cta_rank * BN_CTA;
                        if (!B_MN) {
                            tma_load_4d_pair(b_dst, bmap, full, kk, n_cta, tile.expert, 0);
                        } else {
#pragma unroll
                            for (int c = 0; c < BN_CTA / 64; ++c)
                                tma_load_4d_pair(b_dst + c * CHUNK_BYTES, bmap, full, n_cta + c * 64, kk, tile.expert, 0);
                        }
                    } else {
                        const int krow = tile.row0 + kb * BK - p.row_begin;
#pragma unroll
                        for (int c = 0; c < BM_CTA / 64; ++c)
                            tma_load_4d_pair(a_dst + c * CHUNK_BYTES, &tmA0, full, tile.m0 + cta_rank * BM_CTA + c * 64, krow, 0, 0);
#pragma unroll
                        for (int c = 0; c < BN_CTA / 64; ++c)
                            tma_load_4d_pair(b_dst + c * CHUNK_BYTES, &tmB0, full, tile.n0 + cta_rank * BN_CTA + c * 64, krow, 0, 0);
                    }
                }
                __syncwarp();
                if (++stage == STAGES) { stage = 0; phase ^= 1u; }
            }
        }
    } else if (warp == 1) {
        // ---- MMA issuer (leader CTA only) ----------------------------------------------------------------
        if (cta_rank == 0) {
            int stage = 0;
            uint32_t phase = 0;
            int iter = 0;
            bool ok = true;
            // descriptor steps per 16-wide K slice (units of 16 bytes): 32 B inside a K-major swizzle row,
            // two 8-row groups (2 KB) of an MN-major tile
            constexpr uint32_t kAStep = A_MN ? 128u : 2u;
            constexpr uint32_t kBStep = B_MN ? 128u : 2u;
            for (int t = pair; t < num_tiles && ok; t += num_pairs) {
                Tile tile;
                if (!decode_tile<MODE, BK>(p, cum, lo, hi, t, tile)) continue;
                const int acc = iter & 1;
                const uint32_t acc_phase = (iter >> 1) & 1u;
                ok = mbar_wait(bar_tmem_empty + 8 * acc, acc_phase ^ 1u, abort_flag, p.status);
                if (!ok) break;
                tc_fence_after_sync();
                const uint32_t d_tmem = tmem_base + acc * BN;
                for (int kb = 0; kb < tile.k_blocks; ++kb) {
                    ok = mbar_wait(bar_full + 8 * stage, phase, abort_flag, p.status);
                    if (!ok) break;
                    tc_fence_after_sync();
                    if (lane == 0) {
                        const uint32_t a_addr = smem_base + stage * STAGE_BYTES;
                        const uint32_t b_addr = a_addr + A_TILE_BYTES;
                        const uint64_t a_desc = A_MN ? umma_smem_desc(a_addr, CHUNK_BYTES, 1024) : umma_smem_desc(a_addr, 16, 1024);
                        const uint64_t b_desc = B_MN ? umma_smem_desc(b_addr, CHUNK_BYTES, 1024) : umma_smem_desc(b_addr, 16, 1024);
#pragma unroll
                        for (int k = 0; k < BK / 16; ++k)
                            umma_bf16_pair(d_tmem, a_desc + k * kAStep, b_desc + k * kBStep, kIdesc, (kb | k) != 0 ? 1u : 0u);
                        umma_commit_pair(bar_empty + 8 * stage);                            // frees the stage in both CTAs
                        if (kb == tile.k_blocks - 1) umma_commit_pair(bar_tmem_full + 8 * acc);   // accumulators complete
                    }
                    __syncwarp();
                    if (++stage == STAGES) { stage = 0; phase ^= 1u; }
                }
                ++iter;
            }
        }
    } else {
        // ---- epilogue (both CTAs, each for its own 128 rows) ----------------------------------------------
        const int quarter = warp & 3;                 // tensor-memory lanes [32*quarter, 32*quarter + 32)
        const int row_in_tile = cta_rank * BM_CTA + quarter * 32 + lane;
        int iter = 0;
        bool ok = true;
        for (int t = pair; t < num_tiles && ok; t += num_pairs) {
            Tile tile;
            if (!decode_tile<MODE, BK>(p, cum, lo, hi, t, tile)) continue;
            const int acc = iter & 1;
            const uint32_t acc_phase = (iter >> 1) & 1u;
            ok = mbar_wait(bar_tmem_full + 8 * acc, acc_phase, abort_flag, p.status);
            if (!ok) break;
            tc_fence_after_sync();
            bf16* out;
            if (FUSED)
                out = p.D0;   // the fused form addresses its three outputs itself
            else if (MODE == MODE_ROWS)
                out = (tile.set ? p.D1 : p.D0) + static_cast<long long>(tile.row0 - p.row_begin + row_in_tile) * p.ldd + tile.n0;
            else
                out = p.D0 + static_cast<long long>(tile.expert) * p.d_expert_stride +
                      static_cast<long long>(tile.m0 + row_in_tile) * p.ldd + tile.n0;
            const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + acc * BN;
            uint8_t* patch = smem_gen + SharedLayout::kEpilogue + quarter * kEpiWarpBytes;
            bf16* warp_out = out - static_cast<long long>(lane) * p.ldd;   // row of lane 0
            if (FUSED) {
                // row of lane 0 at the tile's first gate / up / hidden column
                const long long first = static_cast<long long>(tile.row0 - p.row_begin + cta_rank * BM_CTA + quarter * 32) * p.ldd +
                                        tile.n0 / 2;
#pragma unroll 1
                for (int c = 0; c < 2; ++c) {   // 64 gate columns and the same 64 up columns per round
                    uint4 gate[8], up[8], hid[8];
                    {
                        uint32_t v0[32], v1[32];
                        tmem_ld_32x32(taddr + c * 64, v0);
                        tmem_ld_32x32(taddr + c * 64 + 32, v1);
                        tmem_ld_wait();
#pragma unroll
                        for (int i = 0; i < 4; ++i) { gate[i] = pack8_bf16(&v0[8 * i]); gate[4 + i] = pack8_bf16(&v1[8 * i]); }
                        tmem_ld_32x32(taddr + BN_CTA + c * 64, v0);
                        tmem_ld_32x32(taddr + BN_CTA + c * 64 + 32, v1);
                        tmem_ld_wait();
#pragma unroll
                        for (int i = 0; i < 4; ++i) { up[i] = pack8_bf16(&v0[8 * i]); up[4 + i] = pack8_bf16(&v1[8 * i]); }
                    }
                    if (p.clamp) {
#pragma unroll
                        for (int i = 0; i < 8; ++i)
                            hid[i] = make_uint4(swiglu_pair<true>(gate[i].x, up[i].x, p.limit), swiglu_pair<true>(gate[i].y, up[i].y, p.limit),
                                                swiglu_pair<true>(gate[i].z, up[i].z, p.limit), swiglu_pair<true>(gate[i].w, up[i].w, p.limit));
                    } else {
#pragma unroll
                        for (int i = 0; i < 8; ++i)
                            hid[i] = make_uint4(swiglu_pair<false>(gate[i].x, up[i].x, 0.f), swiglu_pair<false>(gate[i].y, up[i].y, 0.f),
                                                swiglu_pair<false>(gate[i].z, up[i].z, 0.f), swiglu_pair<false>(gate[i].w, up[i].w, 0.f));
                    }
                    epilogue_store_packed_64cols(patch, gate, p.D0 + first + c * 64, p.ldd, lane);
                    epilogue_store_packed_64cols(patch, up, p.D1 + first + c * 64, p.ldd, lane);
                    epilogue_store_packed_64cols(patch, hid, p.D2 + first + c * 64, p.ldd, lane);
                }
            } else
#pragma unroll 1
            for (int c = 0; c < BN / 64; ++c) {
                uint32_t v0[32], v1[32];
                tmem_ld_32x32(taddr + c * 64, v0);
                tmem_ld_32x32(taddr + c * 64 + 32, v1);
                tmem_ld_wait();
                if (p.out_f32) {         // router GEMMs: the accumulator goes out unrounded (`out` was computed for 2-byte elements)
                    float* out32 = reinterpret_cast<float*>(p.D0) + (out - p.D0) + c * 64;
                    store_row_chunk_f32(out32, v0);
                    store_row_chunk_f32(out32 + 32, v1);
                } else if (tile.accumulate) {   // rare (later windows of a multi-window backward): add in fp32 per row
                    store_row_chunk(out + c * 64, v0, true);
                    store_row_chunk(out + c * 64 + 32, v1, true);
                } else {
                    epilogue_store_64cols(patch, v0, v1, warp_out + c * 64, p.ldd, lane);
                }
            }
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive_leader(bar_tmem_empty + 8 * acc);
            ++iter;
        }
    }

    // ---- teardown -------------------------------------------------------------------------------------
    if (*abort_flag) {   // give copies that are still in flight time to land before shared memory is released
        for (int i = 0; i < 64; ++i) __nanosleep(2000);
    }
    tc_fence_before_sync();
    __syncthreads();
    cluster_sync_all();   // the peer's shared memory and barriers stay valid until both CTAs are done
    if (warp == 1) {
        tc_fence_after_sync();
        tmem_dealloc_pair(tmem_base, TMEM_COLS);
    }
}

// ---------------------------------------------------------------------------------------------------------
// Host side
// ---------------------------------------------------------------------------------------------------------

// Rank-4 bf16 map over a row-major [d2][d1][d0] array (d0 contiguous); box = {b0, b1, 1, 1}.
int make_map(CUtensorMap* map, const void* base, uint64_t d0, uint64_t d1, uint64_t d2, uint32_t b0, uint32_t b1) {
    const cuuint64_t dims[4] = {d0, d1, d2, 1};
    const cuuint64_t strides[3] = {d0 * 2, d0 * d1 * 2, d0 * d1 * d2 * 2};
    const cuuint32_t box[4] = {b0, b1, 1, 1};
    return encode_map(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, base, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
}

size_t smem_bytes(int num_experts) {
    return 1024 + SharedLayout::kCum + 4 * (static_cast<size_t>(num_experts) + 2);
}

template <int MODE, bool B_MN, bool FUSED = false>
int launch(const CUtensorMap& a0, const CUtensorMap& b0, const CUtensorMap& a1, const CUtensorMap& b1,
           const KernelParams& kp, int max_tiles, cudaStream_t stream) {
    static int resident_pairs[16] = {0};
    return launch_pairs(grouped_gemm_kernel<MODE, B_MN, FUSED>, "grouped_gemm_kernel", resident_pairs, smem_bytes(kp.num_experts),
                        max_tiles, stream, a0, b0, a1, b1, kp);
}


}  // namespace

int launch_rows_gemm(const GemmProblem& pb, const void* A, int K, const void* B0, const void* B1, void* D0, void* D1,
                     int N, bool b_is_kn, cudaStream_t stream) {
    int rc = check_problem(pb);
    if (rc != MOK_OK) return rc;
    if (K <= 0 || N <= 0 || K % BK != 0 || N % BN != 0) return MOK_ERR_INVALID_ARGUMENT;
    const int n_sets = (B1 != nullptr) ? 2 : 1;
    CUtensorMap a0, b0, b1;
    if ((rc = make_map(&a0, A, K, pb.buffer_rows, 1, BK, BM_CTA)) != MOK_OK) return rc;
    if (!b_is_kn) {
        if ((rc = make_map(&b0, B0, K, N, pb.num_experts, BK, BN_CTA)) != MOK_OK) return rc;
        if ((rc = make_map(&b1, n_sets == 2 ? B1 : B0, K, N, pb.num_experts, BK, BN_CTA)) != MOK_OK) return rc;
    } else {
        if ((rc = make_map(&b0, B0, N, K, pb.num_experts, 64, BK)) != MOK_OK) return rc;
        if ((rc = make_map(&b1, n_sets == 2 ? B1 : B0, N, K, pb.num_experts, 64, BK)) != MOK_OK) return rc;
    }
    KernelParams kp = base_params(pb);
    kp.n_blocks = N / BN;
    kp.k_blocks = K / BK;
    kp.n_sets = n_sets;
    kp.D0 = static_cast<bf16*>(D0);
    kp.D1 = static_cast<bf16*>(D1);
    kp.ldd = N;
    const int window = pb.row_end - pb.row_begin;
    const int max_tiles = (window / BM) * kp.n_blocks * n_sets;
    return b_is_kn ? launch<MODE_ROWS, true>(a0, b0, a0, b1, kp, max_tiles, stream)
                   : launch<MODE_ROWS, false>(a0, b0, a0, b1, kp, max_tiles, stream);
}

int launch_gate_up_fused(const GemmProblem& pb, const void* A, int K, const void* Wg, const void* Wu, void* gate, void* up,
                         void* hidden, int N, bool has_limit, float limit, cudaStream_t stream) {
    int rc = check_problem(pb);
    if (rc != MOK_OK) return rc;
    if (K <= 0 || N <= 0 || K % BK != 0 || N % BN_CTA != 0 || !Wg || !Wu || !gate || !up || !hidden) return MOK_ERR_INVALID_ARGUMENT;
    CUtensorMap a0, b0, b1;
    if ((rc = make_map(&a0, A, K, pb.buffer_rows, 1, BK, BM_CTA)) != MOK_OK) return rc;
    if ((rc = make_map(&b0, Wg, K, N, pb.num_experts, BK, BN_CTA)) != MOK_OK) return rc;
    if ((rc = make_map(&b1, Wu, K, N, pb.num_experts, BK, BN_CTA)) != MOK_OK) return rc;
    KernelParams kp = base_params(pb);
    kp.n_blocks = N / BN_CTA;   // one tile per 128 gate columns + the same 128 up columns
    kp.k_blocks = K / BK;
    kp.D0 = static_cast<bf16*>(gate);
    kp.D1 = static_cast<bf16*>(up);
    kp.D2 = static_cast<bf16*>(hidden);
    kp.clamp = has_limit ? 1 : 0;
    kp.limit = limit;
    kp.ldd = N;
    const int window = pb.row_end - pb.row_begin;
    return launch<MODE_ROWS, false, true>(a0, b0, a0, b1, kp, (window / BM) * kp.n_blocks, stream);
}

int launch_rows_gemm_dual(const GemmProblem& pb, const void* A0, const void* A1, int K, const void* B0, const void* B1,
                          void* D, int N, cudaStream_t stream) {
    int rc = check_problem(pb);
    if (rc != MOK_OK) return rc;
    if (K <= 0 || N <= 0 || K % BK != 0 || N % BN != 0) return MOK_ERR_INVALID_ARGUMENT;
    CUtensorMap a0, a1, b0, b1;
    if ((rc = make_map(&a0, A0, K, pb.buffer_rows, 1, BK, BM_CTA)) != MOK_OK) return rc;
    if ((rc = make_map(&a1, A1, K, pb.buffer_rows, 1, BK, BM_CTA)) != MOK_OK) return rc;
    if ((rc = make_map(&b0, B0, N, K, pb.num_experts, 64, BK)) != MOK_OK) return rc;
    if ((rc = make_map(&b1, B1, N, K, pb.num_experts, 64, BK)) != MOK_OK) return rc;
    KernelParams kp = base_params(pb);
    kp.n_blocks = N / BN;
    kp.k_blocks = K / BK;
    kp.k_sets = 2;
    kp.D0 = static_cast<bf16*>(D);
    kp.D1 = nullptr;
    kp.ldd = N;
    const int window = pb.row_end - pb.row_begin;
    return launch<MODE_ROWS, true>(a0, b0, a1, b1, kp, (window / BM) * kp.n_blocks, stream);
}

int launch_rows_gemm_f32(const GemmProblem& pb, const void* A, int K, const void* B_hi, const void* B_lo, float* D, int N,
                         cudaStream_t stream) {
    int rc = check_problem(pb);
    if (rc != MOK_OK) return rc;
    if (K <= 0 || N <= 0 || K % BK != 0 || N % BN != 0 || D == nullptr) return MOK_ERR_INVALID_ARGUMENT;
    CUtensorMap a0, b0, b1;
    if ((rc = make_map(&a0, A, K, pb.buffer_rows, 1, BK, BM_CTA)) != MOK_OK) return rc;
    if ((rc = make_map(&b0, B_hi, K, N, pb.num_experts, BK, BN_CTA)) != MOK_OK) return rc;
    if ((rc = make_map(&b1, B_lo ? B_lo : B_hi, K, N, pb.num_experts, BK, BN_CTA)) != MOK_OK) return rc;
    KernelParams kp = base_params(pb);
    kp.n_blocks = N / BN;
    kp.k_blocks = K / BK;
    kp.k_sets = B_lo ? 2 : 1;      // second K loop: the same A against the low-order term
    kp.D0 = reinterpret_cast<bf16*>(D);
    kp.D1 = nullptr;
    kp.out_f32 = 1;
    kp.ldd = N;
    const int window = pb.row_end - pb.row_begin;
    return launch<MODE_ROWS, false>(a0, b0, a0, b1, kp, (window / BM) * kp.n_blocks, stream);
}

int launch_wgrad_gemm(const GemmProblem& pb, const void* A, int M, const void* B, int N, void* D, cudaStream_t stream,
                      bool out_f32) {
    int rc = check_problem(pb);
    if (rc != MOK_OK) return rc;
    if (M <= 0 || N <= 0 || M % BM != 0 || N % BN != 0) return MOK_ERR_INVALID_ARGUMENT;
    CUtensorMap a0, b0;
    if ((rc = make_map(&a0, A, M, pb.buffer_rows, 1, 64, BK)) != MOK_OK) return rc;
    if ((rc = make_map(&b0, B, N, pb.buffer_rows, 1, 64, BK)) != MOK_OK) return rc;
    KernelParams kp = base_params(pb);
    kp.n_blocks = N / BN;
    kp.m_blocks_w = M / BM;
    kp.D0 = static_cast<bf16*>(D);
    kp.out_f32 = out_f32 ? 1 : 0;
    kp.ldd = N;
    kp.d_expert_stride = static_cast<long long>(M) * N;
    return launch<MODE_WGRAD, true>(a0, b0, a0, b0, kp, pb.num_experts * kp.m_blocks_w * kp.n_blocks, stream);
}

}  // namespace mok

// ---------------------------------------------------------------------------------------------------------
// C ABI: single launches, for tests and profiling
// ---------------------------------------------------------------------------------------------------------
static mok::GemmProblem single_launch_problem(const int32_t* tokens_per_expert, const int32_t* num_tokens, int num_experts,
                                              int rows, uint32_t* status) {
    mok::GemmProblem pb;
    pb.tokens_per_expert = tokens_per_expert;
    pb.num_tokens = num_tokens;
    pb.num_experts = tokens_per_expert ? num_experts : 1;
    pb.dense_rows = tokens_per_expert ? 0 : rows;
    pb.row_begin = 0;
    pb.row_end = rows;
    pb.buffer_rows = rows;
    pb.status = status;
    return pb;
}

extern "C" int mok_grouped_gemm_bf16(const void* A, const void* B, void* D, const int32_t* tokens_per_expert,
                                     const int32_t* num_tokens, int num_experts, int rows, int N, int K, int b_is_kn,
                                     uint32_t* status, mok_stream_t stream) {
    if (A == nullptr || B == nullptr || D == nullptr || rows <= 0 || rows % 256 != 0) return MOK_ERR_INVALID_ARGUMENT;
    const mok::GemmProblem pb = single_launch_problem(tokens_per_expert, num_tokens, num_experts, rows, status);
    return mok::launch_rows_gemm(pb, A, K, B, nullptr, D, nullptr, N, b_is_kn != 0, reinterpret_cast<cudaStream_t>(stream));
}

extern "C" int mok_grouped_wgrad_bf16(const void* A, const void* B, void* D, const int32_t* tokens_per_expert,
                                      const int32_t* num_tokens, int num_experts, int rows, int M, int N,
                                      uint32_t* status, mok_stream_t stream) {
    if (A == nullptr || B == nullptr || D == nullptr || rows <= 0 || rows % 256 != 0) return MOK_ERR_INVALID_ARGUMENT;
    const mok::GemmProblem pb = single_launch_problem(tokens_per_expert, num_tokens, num_experts, rows, status);
    return mok::launch_wgrad_gemm(pb, A, M, B, N, D, reinterpret_cast<cudaStream_t>(stream));
}
