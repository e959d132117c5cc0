// Block-scaled MXFP8 grouped GEMM for sm_100a: tcgen05.mma kind::mxf8f6f4.block_scale on CTA pairs.
//
// Same structure as the bf16 kernel (grouped_gemm.cu): a cluster of two CTAs owns a 256 x 256 output tile, each
// CTA stages its 128 rows of A and its 128-column half of B by TMA (K step 128 bytes = 128 e4m3 elements), the
// leader CTA issues the MMAs.  In addition every K step carries its e8m0 scales: one 512-byte tile for the CTA's
// 128 rows of A and two for the 256 columns of B (both CTAs need all B scales), loaded by TMA next to the data,
// copied to tensor memory with tcgen05.cp and consumed by four K = 32 MMAs whose descriptor selects the scale byte.
// Tensor memory: 256 accumulator columns + one 12-column scale slot per pipeline stage (16 columns apart), so the
// accumulator is single-buffered.
// Both operands are K-major; the dgrad and wgrad forms use transposed-quantized copies of weights / activations
// (the role MXFP8 plays in the reference grouped GEMM, csrc/megakernel/grouped_gemm.cuh:222-249).
#include "gemm_tiles.cuh"
#include "mxfp8.cuh"
#include "mxfp8_gemm.cuh"
#include "swiglu_math.cuh"

namespace mok {
namespace {

using namespace tiles;

constexpr int BK = 128;                               // e4m3 elements = bytes per K step
constexpr int STAGES = 6;
constexpr int A_TILE_BYTES = BM_CTA * BK;             // 16 KB
constexpr int B_TILE_BYTES = BN_CTA * BK;             // 16 KB
constexpr int DATA_STAGE_BYTES = A_TILE_BYTES + B_TILE_BYTES;
constexpr int SCALE_TILE_BYTES = 512;
constexpr int SCALE_STAGE_BYTES = 3 * SCALE_TILE_BYTES;   // A rows of this CTA, B columns [0,128), B columns [128,256)
constexpr int STAGE_TX_BYTES = DATA_STAGE_BYTES + SCALE_STAGE_BYTES;
constexpr int TMEM_SFA_COL = 256;                     // 4 columns
constexpr int TMEM_SFB_COL = 260;                     // 8 columns
constexpr int SCALE_SLOT_COLS = 16;                   // columns from one scale slot to the next (slots: up to STAGES)


struct SharedLayout {
    static constexpr int kScales = STAGES * DATA_STAGE_BYTES;
    static constexpr int kFull = kScales + STAGES * SCALE_STAGE_BYTES;
    static constexpr int kEmpty = kFull + 8 * STAGES;
    static constexpr int kTmemFull = kEmpty + 8 * STAGES;
    static constexpr int kTmemEmpty = kTmemFull + 8;
    static constexpr int kTmemPtr = kTmemEmpty + 8;
    static constexpr int kAbort = kTmemPtr + 4;
    static constexpr int kEpilogue = (kAbort + 4 + 127) / 128 * 128;   // 4 warps x 32 rows x 144 B staging patches
    static constexpr int kCum = kEpilogue + 4 * kEpiWarpBytes;
};


// One operand set: data and scale tensor maps of A and B.
struct MapSet {
    CUtensorMap a, sfa, b, sfb;
};

// ---- fused gate / up epilogue ---------------------------------------------------------------------------------------
// Device copy of Fp8GateUpOut.  With `enabled` a rows-form tile holds gate columns [c0, c0 + 128) in accumulator
// columns [0, 128) (CTA 0 stages the gate weights) and the same up columns in [128, 256) (CTA 1 stages the up weights).
struct FusedOut {
    uint8_t *gate_q, *gate_sc, *up_q, *up_sc, *hid_q, *hid_sc, *hid_qt, *hid_sct;
    long long sc_row_tile_stride, qt_ld, sct_row_tile_stride;
    int cols;      // N of gate / up = row length of the e4m3 outputs
    int enabled, clamp;
    float limit;
};

// One warp = 32 rows of the tile (buffer rows R0 .. R0 + 31, all in one 128-row tile), `packed` = this lane's row:
// vectors [0, 16) gate, [16, 32) up, already rounded to bf16.
template <bool CLAMP>
__device__ __forceinline__ void fused_gate_up_epilogue(const FusedOut& f, const uint4 (&packed)[32], uint8_t* patch, long long R0,
                                                       int col0, int quarter, int lane) {
    const long long row_tile = R0 >> 7;
    const int col_tile = col0 >> 7;
    const long long sc_off = row_tile * f.sc_row_tile_stride + static_cast<long long>(col_tile) * 512 + lane * 16 + quarter * 4;
    const long long q_off = R0 * f.cols + col0;
    // block by block (32 columns), so that the gate / up registers die as the bytes are produced
    uint4 h[16], gate_bytes[8], up_bytes[8], hid_bytes[8];
    uint32_t gate_scales = 0, up_scales = 0, hid_scales = 0;
#pragma unroll
    for (int b = 0; b < 4; ++b) {
        uint32_t g[16], u[16], hb[16], out8[8], sbyte;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const uint4 gv = packed[4 * b + i], uv = packed[16 + 4 * b + i];
            g[4 * i] = gv.x; g[4 * i + 1] = gv.y; g[4 * i + 2] = gv.z; g[4 * i + 3] = gv.w;
            u[4 * i] = uv.x; u[4 * i + 1] = uv.y; u[4 * i + 2] = uv.z; u[4 * i + 3] = uv.w;
        }
#pragma unroll
        for (int i = 0; i < 16; ++i) hb[i] = swiglu_pair<CLAMP>(g[i], u[i], f.limit);
#pragma unroll
        for (int i = 0; i < 4; ++i) h[4 * b + i] = make_uint4(hb[4 * i], hb[4 * i + 1], hb[4 * i + 2], hb[4 * i + 3]);
        mxfp8_quantize_block(g, out8, sbyte);
        gate_scales |= sbyte << (8 * b);
        gate_bytes[2 * b] = make_uint4(out8[0], out8[1], out8[2], out8[3]);
        gate_bytes[2 * b + 1] = make_uint4(out8[4], out8[5], out8[6], out8[7]);
        mxfp8_quantize_block(u, out8, sbyte);
        up_scales |= sbyte << (8 * b);
        up_bytes[2 * b] = make_uint4(out8[0], out8[1], out8[2], out8[3]);
        up_bytes[2 * b + 1] = make_uint4(out8[4], out8[5], out8[6], out8[7]);
        mxfp8_quantize_block(hb, out8, sbyte);
        hid_scales |= sbyte << (8 * b);
        hid_bytes[2 * b] = make_uint4(out8[0], out8[1], out8[2], out8[3]);
        hid_bytes[2 * b + 1] = make_uint4(out8[4], out8[5], out8[6], out8[7]);
    }
    *reinterpret_cast<uint32_t*>(f.gate_sc + sc_off) = gate_scales;
    *reinterpret_cast<uint32_t*>(f.up_sc + sc_off) = up_scales;
    *reinterpret_cast<uint32_t*>(f.hid_sc + sc_off) = hid_scales;
    // 128 bytes per row = 64 two-byte elements for the staging helper: full 128-byte lines
    const long long ld2 = f.cols / 2;
    epilogue_store_packed_64cols(patch, gate_bytes, reinterpret_cast<bf16*>(f.gate_q + q_off), ld2, lane);
    epilogue_store_packed_64cols(patch, up_bytes, reinterpret_cast<bf16*>(f.up_q + q_off), ld2, lane);
    epilogue_store_packed_64cols(patch, hid_bytes, reinterpret_cast<bf16*>(f.hid_q + q_off), ld2, lane);

    // transposed layout: for one column the warp's 32 rows are exactly one block of 32; two columns per word
    uint8_t* sct = f.hid_sct + col_tile * f.sct_row_tile_stride + row_tile * 512 + quarter;
#pragma unroll
    for (int i = 0; i < 16; ++i) {
        const uint32_t words[4] = {h[i].x, h[i].y, h[i].z, h[i].w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int c = 8 * i + 2 * j;   // columns c, c + 1 of the tile
            const float2 val = unpack_bf16x2(words[j]);
            float a0 = fabsf(val.x), a1 = fabsf(val.y);
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) {
                a0 = fmaxf(a0, __shfl_xor_sync(0xffffffffu, a0, off));
                a1 = fmaxf(a1, __shfl_xor_sync(0xffffffffu, a1, off));
            }
            const float s0 = fmaxf(a0 * 0.002232142857f, 0.000000000001f), s1 = fmaxf(a1 * 0.002232142857f, 0.000000000001f);
            uint16_t e8;
            asm volatile("cvt.rp.satfinite.ue8m0x2.f32 %0, %1, %2;" : "=h"(e8) : "f"(s1), "f"(s0));   // low byte: s0
            const uint32_t sb0 = e8 & 0xFFu, sb1 = (e8 >> 8) & 0xFFu;
            const float inv0 = __uint_as_float((254u - sb0) << 23), inv1 = __uint_as_float((254u - sb1) << 23);
            uint16_t q2;
            asm volatile("cvt.rn.satfinite.e4m3x2.f32 %0, %2, %1;" : "=h"(q2) : "f"(val.x * inv0), "f"(val.y * inv1));
            patch[c * 32 + lane] = static_cast<uint8_t>(q2 & 0xFFu);
            patch[(c + 1) * 32 + lane] = static_cast<uint8_t>(q2 >> 8);
            if (lane == (c & 31)) sct[(c & 31) * 16 + (c >> 5) * 4] = static_cast<uint8_t>(sb0);
            if (lane == ((c + 1) & 31)) sct[((c + 1) & 31) * 16 + ((c + 1) >> 5) * 4] = static_cast<uint8_t>(sb1);
        }
    }
    __syncwarp();
    uint8_t* qt = f.hid_qt + static_cast<long long>(col0) * f.qt_ld + R0;
#pragma unroll
    for (int it = 0; it < 8; ++it) {   // 16 columns per store instruction, 32 bytes (the warp's rows) each
        const int c = it * 16 + (lane >> 1), half = lane & 1;
        *reinterpret_cast<uint4*>(qt + static_cast<long long>(c) * f.qt_ld + half * 16) =
            *reinterpret_cast<const uint4*>(patch + c * 32 + half * 16);
    }
    __syncwarp();
}

template <int MODE, bool FUSED>
__global__ void __launch_bounds__(NUM_THREADS, 1)
mxfp8_gemm_kernel(const __grid_constant__ MapSet ms0, const __grid_constant__ MapSet ms1, const KernelParams p, const FusedOut f) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
    const uint32_t scale_base = smem_base + SharedLayout::kScales;
    const uint32_t bar_full = smem_base + SharedLayout::kFull;
    const uint32_t bar_empty = smem_base + SharedLayout::kEmpty;
    const uint32_t bar_tmem_full = smem_base + SharedLayout::kTmemFull;
    const uint32_t bar_tmem_empty = smem_base + SharedLayout::kTmemEmpty;
    volatile uint32_t* tmem_ptr_slot = reinterpret_cast<volatile uint32_t*>(smem_gen + SharedLayout::kTmemPtr);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem_gen + SharedLayout::kAbort);
    int* cum = reinterpret_cast<int*>(smem_gen + SharedLayout::kCum);

    // nothing to do for a row window behind the schedule's last row: leave before anything is set up (both CTAs alike)
    if (min(p.row_end, p.tokens_per_expert == nullptr ? p.dense_rows : *p.num_tokens) <= p.row_begin) return;

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int cta_rank = static_cast<int>(cluster_cta_rank());
    const int pair = blockIdx.x >> 1;
    const int num_pairs = gridDim.x >> 1;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(bar_full + 8 * s, 1);
            mbar_init(bar_empty + 8 * s, 1);
        }
        mbar_init(bar_tmem_full, 1);
        mbar_init(bar_tmem_empty, 8);
        *abort_flag = 0;
        mbar_fence_init();
        tma_prefetch_desc(&ms0.a); tma_prefetch_desc(&ms0.sfa); tma_prefetch_desc(&ms0.b); tma_prefetch_desc(&ms0.sfb);
        if (p.k_sets > 1 || p.n_sets > 1) { tma_prefetch_desc(&ms1.b); tma_prefetch_desc(&ms1.sfb); }
        if (p.k_sets > 1) { tma_prefetch_desc(&ms1.a); tma_prefetch_desc(&ms1.sfa); }
    }
    if (warp == 1) {
        tmem_alloc_pair(smem_u32(const_cast<uint32_t*>(tmem_ptr_slot)), TMEM_COLS);
        tmem_relinquish_pair();
    }
    if (warp == 2) expert_row_prefix(p, cum, lane);
    tc_fence_before_sync();
    __syncthreads();
    cluster_sync_all();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_ptr_slot;

    const int total_rows = p.tokens_per_expert == nullptr ? p.dense_rows : *p.num_tokens;
    const int lo = p.row_begin;
    const int hi = min(p.row_end, total_rows);
    const int num_tiles = total_tiles<MODE>(p, lo, hi);

    if (warp == 0) {
        // ---- TMA producer (both CTAs): data tiles and scale tiles of one K step land on the leader's barrier ----
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
                    const uint32_t full = full_local & kPairLeaderMask;
                    const uint32_t a_dst = smem_base + stage * DATA_STAGE_BYTES;
                    const uint32_t b_dst = a_dst + A_TILE_BYTES;
                    const uint32_t s_dst = scale_base + stage * SCALE_STAGE_BYTES;
                    if (cta_rank == 0) mbar_expect_tx(full_local, 2 * STAGE_TX_BYTES);
                    if (MODE == MODE_ROWS) {
                        const int kset = kb >= p.k_blocks ? 1 : 0;
                        const int kt = kb - kset * p.k_blocks;           // K tile of 128
                        const MapSet& am = kset ? ms1 : ms0;
                        const MapSet& bm = (kset || tile.set) ? ms1 : ms0;
                        const int row = tile.row0 - p.row_begin + cta_rank * BM_CTA;
                        tma_load_4d_pair(a_dst, &am.a, full, kt * BK, row, 0, 0);
                        tma_load_4d_pair(s_dst, &am.sfa, full, 0, kt, row / 128, 0);
                        if (FUSED) {   // CTA 0 stages 128 gate rows, CTA 1 the same 128 up rows; both need both scale tiles
                            const int col0 = tile.n0 / 2;
                            tma_load_4d_pair(b_dst, cta_rank ? &ms1.b : &ms0.b, full, kt * BK, col0, tile.expert, 0);
                            const int sfb_row = tile.expert * p.n_tiles_per_expert + col0 / 128;
                            tma_load_4d_pair(s_dst + SCALE_TILE_BYTES, &ms0.sfb, full, 0, kt, sfb_row, 0);
                            tma_load_4d_pair(s_dst + 2 * SCALE_TILE_BYTES, &ms1.sfb, full, 0, kt, sfb_row, 0);
                        } else {
                            tma_load_4d_pair(b_dst, &bm.b, full, kt * BK, tile.n0 + cta_rank * BN_CTA, tile.expert, 0);
                            const int sfb_row = tile.expert * p.n_tiles_per_expert + tile.n0 / 128;
                            tma_load_4d_pair(s_dst + SCALE_TILE_BYTES, &bm.sfb, full, 0, kt, sfb_row, 0);
                            tma_load_4d_pair(s_dst + 2 * SCALE_TILE_BYTES, &bm.sfb, full, 0, kt, sfb_row + 1, 0);
                        }
                    } else {
                        const int kcol = tile.row0 + kb * BK - p.row_begin;   // column of the transposed activations
                        tma_load_4d_pair(a_dst, &ms0.a, full, kcol, tile.m0 + cta_rank * BM_CTA, 0, 0);
                        tma_load_4d_pair(s_dst, &ms0.sfa, full, 0, kcol / 128, tile.m0 / 128 + cta_rank, 0);
                        tma_load_4d_pair(b_dst, &ms0.b, full, kcol, tile.n0 + cta_rank * BN_CTA, 0, 0);
                        tma_load_4d_pair(s_dst + SCALE_TILE_BYTES, &ms0.sfb, full, 0, kcol / 128, tile.n0 / 128, 0);
                        tma_load_4d_pair(s_dst + 2 * SCALE_TILE_BYTES, &ms0.sfb, full, 0, kcol / 128, tile.n0 / 128 + 1, 0);
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
            const uint32_t sfa_tmem = tmem_base + TMEM_SFA_COL;
            const uint32_t sfb_tmem = tmem_base + TMEM_SFB_COL;
            for (int t = pair; t < num_tiles && ok; t += num_pairs) {
                Tile tile;
                if (!decode_tile<MODE, BK>(p, cum, lo, hi, t, tile)) continue;
                ok = mbar_wait(bar_tmem_empty, (iter & 1u) ^ 1u, abort_flag, p.status);   // epilogue drained the accumulator
                if (!ok) break;
                tc_fence_after_sync();
                for (int kb = 0; kb < tile.k_blocks; ++kb) {
                    ok = mbar_wait(bar_full + 8 * stage, phase, abort_flag, p.status);
                    if (!ok) break;
                    tc_fence_after_sync();
                    if (lane == 0) {
                        const uint32_t a_addr = smem_base + stage * DATA_STAGE_BYTES;
                        const uint32_t b_addr = a_addr + A_TILE_BYTES;
                        // the scale columns rotate with the stage (one slot per stage when scale_slots == STAGES)
                        const uint32_t slot = static_cast<uint32_t>(stage % p.scale_slots) * SCALE_SLOT_COLS;
                        const uint32_t sfa = sfa_tmem + slot, sfb = sfb_tmem + slot;
                        const uint32_t s_addr = scale_base + stage * SCALE_STAGE_BYTES;
                        tmem_copy_scales_pair(sfa, umma_scale_desc(s_addr));
                        tmem_copy_scales_pair(sfb, umma_scale_desc(s_addr + SCALE_TILE_BYTES));
                        tmem_copy_scales_pair(sfb + 4, umma_scale_desc(s_addr + 2 * SCALE_TILE_BYTES));
                        const uint64_t a_desc = umma_smem_desc(a_addr, 16, 1024);
                        const uint64_t b_desc = umma_smem_desc(b_addr, 16, 1024);
#pragma unroll
                        for (int k = 0; k < BK / 32; ++k)   // 32 elements = 32 bytes = 2 descriptor units per slice
                            umma_mxfp8_pair(tmem_base, a_desc + k * 2u, b_desc + k * 2u, umma_idesc_mxfp8(BM, BN, k), sfa, sfb,
                                            (kb | k) != 0 ? 1u : 0u);
                        umma_commit_pair(bar_empty + 8 * stage);
                        if (kb == tile.k_blocks - 1) umma_commit_pair(bar_tmem_full);
                    }
                    __syncwarp();
                    if (++stage == STAGES) { stage = 0; phase ^= 1u; }
                }
                ++iter;
            }
        }
    } else {
        // ---- epilogue --------------------------------------------------------------------------------------
        const int quarter = warp & 3;
        const int row_in_tile = cta_rank * BM_CTA + quarter * 32 + lane;
        int iter = 0;
        bool ok = true;
        for (int t = pair; t < num_tiles && ok; t += num_pairs) {
            Tile tile;
            if (!decode_tile<MODE, BK>(p, cum, lo, hi, t, tile)) continue;
            ok = mbar_wait(bar_tmem_full, iter & 1u, abort_flag, p.status);
            if (!ok) break;
            tc_fence_after_sync();
            bf16* out;
            if (MODE == MODE_ROWS)
                out = (tile.set ? p.D1 : p.D0) + static_cast<long long>(tile.row0 - p.row_begin + row_in_tile) * p.ldd + tile.n0;
            else
                out = p.D0 + static_cast<long long>(tile.expert) * p.d_expert_stride +
                      static_cast<long long>(tile.m0 + row_in_tile) * p.ldd + tile.n0;
            const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);
            uint8_t* patch = smem_gen + SharedLayout::kEpilogue + quarter * kEpiWarpBytes;
            bf16* warp_out = out - static_cast<long long>(lane) * p.ldd;
            if (tile.accumulate) {   // rare (later windows of a multi-window backward): add in fp32 per row
#pragma unroll 1
                for (int c = 0; c < BN / 32; ++c) {
                    uint32_t v[32];
                    tmem_ld_32x32(taddr + c * 32, v);
                    tmem_ld_wait();
                    store_row_chunk(out + c * 32, v, true);
                }
                tc_fence_before_sync();
                __syncwarp();
                if (lane == 0) mbar_arrive_leader(bar_tmem_empty);
            } else {
                // The accumulator is single-buffered: read the whole row into registers as packed bf16 first and hand
                // tensor memory back to the MMA issuer before any of it is written out.
                uint4 packed[BN / 8];
#pragma unroll
                for (int c = 0; c < BN / 64; ++c) {   // two loads in flight per wait
                    uint32_t v0[32], v1[32];
                    tmem_ld_32x32(taddr + c * 64, v0);
                    tmem_ld_32x32(taddr + c * 64 + 32, v1);
                    tmem_ld_wait();
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        packed[c * 8 + i] = pack8_bf16(&v0[8 * i]);
                        packed[c * 8 + 4 + i] = pack8_bf16(&v1[8 * i]);
                    }
                }
                tc_fence_before_sync();
                __syncwarp();
                if (lane == 0) mbar_arrive_leader(bar_tmem_empty);
                if (MODE == MODE_ROWS && FUSED) {
                    const long long R0 = tile.row0 - p.row_begin + cta_rank * BM_CTA + quarter * 32;
                    if (f.clamp) fused_gate_up_epilogue<true>(f, packed, patch, R0, tile.n0 / 2, quarter, lane);
                    else fused_gate_up_epilogue<false>(f, packed, patch, R0, tile.n0 / 2, quarter, lane);
                } else {
#pragma unroll
                    for (int c = 0; c < BN / 64; ++c)
                        epilogue_store_packed_64cols(patch, &packed[c * 8], warp_out + c * 64, p.ldd, lane);
                }
            }
            ++iter;
        }
    }

    if (*abort_flag) {
        for (int i = 0; i < 64; ++i) __nanosleep(2000);
    }
    tc_fence_before_sync();
    __syncthreads();
    cluster_sync_all();
    if (warp == 1) {
        tc_fence_after_sync();
        tmem_dealloc_pair(tmem_base, TMEM_COLS);
    }
}

// ---------------------------------------------------------------------------------------------------------
// Host side
// ---------------------------------------------------------------------------------------------------------

// e4m3 bytes [groups][rows_per_group][k]: box 128 (K) x 128 (rows)
int data_map(CUtensorMap* map, const Fp8Operand& op, long long rows_per_group, long long groups) {
    const cuuint64_t dims[4] = {static_cast<cuuint64_t>(op.k_extent), static_cast<cuuint64_t>(rows_per_group),
                                static_cast<cuuint64_t>(groups), 1};
    const cuuint64_t strides[3] = {static_cast<cuuint64_t>(op.ld), static_cast<cuuint64_t>(op.ld * rows_per_group),
                                   static_cast<cuuint64_t>(op.ld * rows_per_group * groups)};
    const cuuint32_t box[4] = {BK, 128, 1, 1};
    return encode_map(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, op.data, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
}

// scale tiles [row tile][K tile][128 words]: one 512-byte tile per copy
int scale_map(CUtensorMap* map, const Fp8Operand& op) {
    const long long k_tiles = op.k_extent / 128;
    const long long row_tiles = op.rows / 128;
    const cuuint64_t dims[4] = {128, static_cast<cuuint64_t>(k_tiles), static_cast<cuuint64_t>(row_tiles), 1};
    const cuuint64_t strides[3] = {512, static_cast<cuuint64_t>(op.scale_row_tile_stride),
                                   static_cast<cuuint64_t>(op.scale_row_tile_stride * row_tiles)};
    const cuuint32_t box[4] = {128, 1, 1, 1};
    return encode_map(map, CU_TENSOR_MAP_DATA_TYPE_UINT32, op.scales, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_NONE);
}

bool operand_ok(const Fp8Operand& op) {
    return op.data != nullptr && op.scales != nullptr && op.ld > 0 && op.ld % 128 == 0 && op.rows > 0 && op.rows % 128 == 0 &&
           op.k_extent > 0 && op.k_extent % 128 == 0 && op.scale_row_tile_stride >= 512 && op.scale_row_tile_stride % 512 == 0 &&
           (reinterpret_cast<uintptr_t>(op.data) & 127) == 0 && (reinterpret_cast<uintptr_t>(op.scales) & 127) == 0;
}

int fill_set(MapSet* ms, const Fp8Operand& a, long long a_groups, const Fp8Operand& b, long long b_groups) {
    if (!operand_ok(a) || !operand_ok(b)) return MOK_ERR_INVALID_ARGUMENT;
    int rc;
    if ((rc = data_map(&ms->a, a, a.rows / a_groups, a_groups)) != MOK_OK) return rc;
    if ((rc = scale_map(&ms->sfa, a)) != MOK_OK) return rc;
    if ((rc = data_map(&ms->b, b, b.rows / b_groups, b_groups)) != MOK_OK) return rc;
    return scale_map(&ms->sfb, b);
}

size_t smem_bytes(int num_experts) { return 1024 + SharedLayout::kCum + 4 * (static_cast<size_t>(num_experts) + 2); }
// Scale slots in tensor memory: one per pipeline stage; MOK_SCALE_SLOTS (1..STAGES) overrides, for measurements.
int scale_slots() {
    static int slots = 0;
    if (slots == 0) {
        int n = STAGES;
        if (const char* v = getenv("MOK_SCALE_SLOTS")) {
            const int want = atoi(v);
            if (want >= 1 && want <= STAGES) n = want;
        }
        slots = n;
    }
    return slots;
}

template <int MODE, bool FUSED = false>
int launch(const MapSet& ms0, const MapSet& ms1, KernelParams kp, int max_tiles, cudaStream_t stream,
           const FusedOut& fused = FusedOut{}) {
    static int resident_pairs[16] = {0};
    kp.scale_slots = scale_slots();
    return launch_pairs(mxfp8_gemm_kernel<MODE, FUSED>, "mxfp8_gemm_kernel", resident_pairs, smem_bytes(kp.num_experts), max_tiles,
                        stream, ms0, ms1, kp, fused);
}


}  // namespace

int launch_fp8_rows_gemm(const GemmProblem& pb, const Fp8Operand& A, int K, const Fp8Operand& B0, const Fp8Operand* B1,
                         void* D0, void* D1, int N, cudaStream_t stream) {
    int rc = check_problem(pb);
    if (rc != MOK_OK) return rc;
    if (K <= 0 || N <= 0 || K % BK != 0 || N % BN != 0) return MOK_ERR_INVALID_ARGUMENT;
    MapSet ms0, ms1;
    if ((rc = fill_set(&ms0, A, 1, B0, pb.num_experts)) != MOK_OK) return rc;
    if ((rc = fill_set(&ms1, A, 1, B1 ? *B1 : B0, pb.num_experts)) != MOK_OK) return rc;
    KernelParams kp = base_params(pb);
    kp.n_blocks = N / BN;
    kp.k_blocks = K / BK;
    kp.n_sets = B1 ? 2 : 1;
    kp.n_tiles_per_expert = N / 128;
    kp.D0 = static_cast<bf16*>(D0);
    kp.D1 = static_cast<bf16*>(D1);
    kp.ldd = N;
    return launch<MODE_ROWS>(ms0, ms1, kp, ((pb.row_end - pb.row_begin) / BM) * kp.n_blocks * kp.n_sets, stream);
}

int launch_fp8_gate_up_fused(const GemmProblem& pb, const Fp8Operand& A, int K, const Fp8Operand& Wg, const Fp8Operand& Wu, int N,
                             const Fp8GateUpOut& out, cudaStream_t stream) {
    int rc = check_problem(pb);
    if (rc != MOK_OK) return rc;
    if (K <= 0 || N <= 0 || K % BK != 0 || N % 128 != 0) return MOK_ERR_INVALID_ARGUMENT;
    if (!out.gate_q || !out.gate_sc || !out.up_q || !out.up_sc || !out.hidden_q || !out.hidden_sc || !out.hidden_qt ||
        !out.hidden_sct || out.qt_ld <= 0 || out.qt_ld % 16 != 0)
        return MOK_ERR_INVALID_ARGUMENT;
    MapSet ms0, ms1;
    if ((rc = fill_set(&ms0, A, 1, Wg, pb.num_experts)) != MOK_OK) return rc;
    if ((rc = fill_set(&ms1, A, 1, Wu, pb.num_experts)) != MOK_OK) return rc;
    KernelParams kp = base_params(pb);
    kp.n_blocks = N / 128;              // one tile per 128 gate columns + the same 128 up columns
    kp.k_blocks = K / BK;
    kp.n_tiles_per_expert = N / 128;
    kp.D0 = nullptr;
    kp.D1 = nullptr;
    kp.ldd = N;
    FusedOut f{};
    f.gate_q = static_cast<uint8_t*>(out.gate_q);
    f.gate_sc = static_cast<uint8_t*>(out.gate_sc);
    f.up_q = static_cast<uint8_t*>(out.up_q);
    f.up_sc = static_cast<uint8_t*>(out.up_sc);
    f.hid_q = static_cast<uint8_t*>(out.hidden_q);
    f.hid_sc = static_cast<uint8_t*>(out.hidden_sc);
    f.hid_qt = static_cast<uint8_t*>(out.hidden_qt);
    f.hid_sct = static_cast<uint8_t*>(out.hidden_sct);
    f.sc_row_tile_stride = out.sc_row_tile_stride;
    f.qt_ld = out.qt_ld;
    f.sct_row_tile_stride = out.sct_row_tile_stride;
    f.cols = N;
    f.enabled = 1;
    f.clamp = out.has_limit ? 1 : 0;
    f.limit = out.limit;
    return launch<MODE_ROWS, true>(ms0, ms1, kp, ((pb.row_end - pb.row_begin) / BM) * kp.n_blocks, stream, f);
}

int launch_fp8_rows_gemm_dual(const GemmProblem& pb, const Fp8Operand& A0, const Fp8Operand& A1, int K, const Fp8Operand& B0,
                              const Fp8Operand& B1, void* D, int N, cudaStream_t stream) {
    int rc = check_problem(pb);
    if (rc != MOK_OK) return rc;
    if (K <= 0 || N <= 0 || K % BK != 0 || N % BN != 0) return MOK_ERR_INVALID_ARGUMENT;
    MapSet ms0, ms1;
    if ((rc = fill_set(&ms0, A0, 1, B0, pb.num_experts)) != MOK_OK) return rc;
    if ((rc = fill_set(&ms1, A1, 1, B1, pb.num_experts)) != MOK_OK) return rc;
    KernelParams kp = base_params(pb);
    kp.n_blocks = N / BN;
    kp.k_blocks = K / BK;
    kp.k_sets = 2;
    kp.n_tiles_per_expert = N / 128;
    kp.D0 = static_cast<bf16*>(D);
    kp.ldd = N;
    return launch<MODE_ROWS>(ms0, ms1, kp, ((pb.row_end - pb.row_begin) / BM) * kp.n_blocks, stream);
}

int launch_fp8_wgrad_gemm(const GemmProblem& pb, const Fp8Operand& At, int M, const Fp8Operand& Bt, int N, void* D,
                          cudaStream_t stream) {
    int rc = check_problem(pb);
    if (rc != MOK_OK) return rc;
    if (M <= 0 || N <= 0 || M % BM != 0 || N % BN != 0) return MOK_ERR_INVALID_ARGUMENT;
    MapSet ms0;
    if ((rc = fill_set(&ms0, At, 1, Bt, 1)) != MOK_OK) return rc;
    KernelParams kp = base_params(pb);
    kp.n_blocks = N / BN;
    kp.m_blocks_w = M / BM;
    kp.D0 = static_cast<bf16*>(D);
    kp.ldd = N;
    kp.d_expert_stride = static_cast<long long>(M) * N;
    return launch<MODE_WGRAD>(ms0, ms0, kp, pb.num_experts * kp.m_blocks_w * kp.n_blocks, stream);
}

}  // namespace mok

// ---------------------------------------------------------------------------------------------------------
// C ABI: single launches, for tests and profiling
// ---------------------------------------------------------------------------------------------------------
static mok::Fp8Operand plain_operand(const void* data, const void* scales, long long rows, long long k) {
    mok::Fp8Operand op;
    op.data = data;
    op.scales = scales;
    op.ld = k;
    op.rows = rows;
    op.k_extent = k;
    op.scale_row_tile_stride = (k / 128) * 512;
    return op;
}

static mok::GemmProblem single_problem(const int32_t* tokens_per_expert, const int32_t* num_tokens, int num_experts, int rows,
                                       uint32_t* status) {
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

extern "C" int mok_grouped_gemm_mxfp8(const void* A_fp8, const void* A_sc, const void* B_fp8, const void* B_sc, void* D,
                                      const int32_t* tokens_per_expert, const int32_t* num_tokens, int num_experts, int rows,
                                      int N, int K, uint32_t* status, mok_stream_t stream) {
    if (!A_fp8 || !A_sc || !B_fp8 || !B_sc || !D || rows <= 0 || rows % 256 != 0 || N <= 0 || K <= 0 || K % 128 != 0)
        return MOK_ERR_INVALID_ARGUMENT;
    const mok::GemmProblem pb = single_problem(tokens_per_expert, num_tokens, num_experts, rows, status);
    const mok::Fp8Operand a = plain_operand(A_fp8, A_sc, rows, K);
    const mok::Fp8Operand b = plain_operand(B_fp8, B_sc, static_cast<long long>(pb.num_experts) * N, K);
    return mok::launch_fp8_rows_gemm(pb, a, K, b, nullptr, D, nullptr, N, reinterpret_cast<cudaStream_t>(stream));
}

extern "C" int mok_grouped_wgrad_mxfp8(const void* At_fp8, const void* At_sc, const void* Bt_fp8, const void* Bt_sc, void* D,
                                       const int32_t* tokens_per_expert, const int32_t* num_tokens, int num_experts, int rows,
                                       int M, int N, uint32_t* status, mok_stream_t stream) {
    if (!At_fp8 || !At_sc || !Bt_fp8 || !Bt_sc || !D || rows <= 0 || rows % 256 != 0 || M <= 0 || N <= 0)
        return MOK_ERR_INVALID_ARGUMENT;
    const mok::GemmProblem pb = single_problem(tokens_per_expert, num_tokens, num_experts, rows, status);
    const mok::Fp8Operand a = plain_operand(At_fp8, At_sc, M, rows);
    const mok::Fp8Operand b = plain_operand(Bt_fp8, Bt_sc, N, rows);
    return mok::launch_fp8_wgrad_gemm(pb, a, M, b, N, D, reinterpret_cast<cudaStream_t>(stream));
}
