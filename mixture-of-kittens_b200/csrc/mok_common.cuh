// Shared device/host helpers for the sm_100a MoE kernels: error plumbing, bounded waits, and thin
// wrappers over the PTX this library needs (mbarrier, TMA bulk-tensor copies, tcgen05 / tensor memory).
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/mok_b200.h"

namespace mok {

// ---------------------------------------------------------------------------------------------
// Host-side error handling
// ---------------------------------------------------------------------------------------------
void set_last_error(const char* what, cudaError_t err);
int fail_cuda(const char* what, cudaError_t err);

#define MOK_CUDA_CHECK(expr)                                             \
    do {                                                                 \
        cudaError_t _e = (expr);                                         \
        if (_e != cudaSuccess) return ::mok::fail_cuda(#expr, _e);       \
    } while (0)

#define MOK_LAUNCH_CHECK(name)                                           \
    do {                                                                 \
        cudaError_t _e = cudaGetLastError();                             \
        if (_e != cudaSuccess) return ::mok::fail_cuda(name, _e);        \
        ::mok::note_launch();                                            \
    } while (0)

// Returns a library status code from the enclosing function unless it is MOK_OK.
#define MOK_TRY(expr)                  \
    do {                               \
        int _rc = (expr);              \
        if (_rc != MOK_OK) return _rc; \
    } while (0)

void note_launch();   // counts kernel launches of this library (mok_launch_count)

int sm_count();   // multiprocessors of the current device (cached per device)

typedef __nv_bfloat16 bf16;

// ---------------------------------------------------------------------------------------------
// Small device utilities
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ float2 unpack_bf16x2(uint32_t v) {
    return __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&v));
}

// ---------------------------------------------------------------------------------------------
// mbarrier
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_fence_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}

// Cycles a pipeline wait may take before the kernel gives up (about two seconds at 2 GHz).  A healthy wait
// is at most one tile main loop, i.e. tens of microseconds.
constexpr long long kPipelineWaitCycles = 4000000000LL;

// Waits for `parity` of `bar`.  Returns false when the wait ran out or another thread already aborted; in the
// first case the abort flag (shared memory) and the global status word are set.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, uint32_t* status) {
    if (mbar_try_wait(bar, parity)) return true;
    const long long start = clock64();
    for (uint32_t spin = 1;; ++spin) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((spin & 0xFF) == 0) {
            if (*abort_flag) return false;
            if (clock64() - start > kPipelineWaitCycles) {
                *abort_flag = 1;
                if (status != nullptr) atomicOr(status, (uint32_t)MOK_STATUS_PIPELINE_TIMEOUT);
                return false;
            }
        }
    }
}

// ---------------------------------------------------------------------------------------------
// TMA (bulk tensor copies, global -> shared; the loads themselves are with the CTA-pair helpers below)
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* map) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(map)) : "memory");
}

// ---------------------------------------------------------------------------------------------
// tcgen05 / tensor memory
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void tc_fence_before_sync() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after_sync() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// 32 lanes x 32 consecutive fp32 columns: thread i of the warp receives lane (base_lane + i).
__device__ __forceinline__ void tmem_ld_32x32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// ---------------------------------------------------------------------------------------------
// CTA pairs (cluster of two CTAs driving one 256-row MMA, "cta_group::2")
// ---------------------------------------------------------------------------------------------
// Clearing this bit of a shared-window address names the same offset in the even (leader) CTA of the pair.
constexpr uint32_t kPairLeaderMask = 0xFEFFFFFFu;

__device__ __forceinline__ uint32_t cluster_cta_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t dst_smem, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
// Load into this CTA's shared memory; the transaction bytes are credited to the mbarrier at `bar`, which may
// live in the leader CTA of the pair.
__device__ __forceinline__ void tma_load_4d_pair(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0, int c1, int c2,
                                                 int c3) {
    asm volatile(
        "cp.async.bulk.tensor.4d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
        : "memory");
}
// 256 x N MMA over both CTAs of the pair; issued by one thread of the leader CTA.
__device__ __forceinline__ void umma_bf16_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// Arrives on the mbarrier at the same shared-memory offset in both CTAs of the pair once the MMAs issued so far are done.
__device__ __forceinline__ void umma_commit_pair(uint32_t bar) {
    const uint16_t both = 3;
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 ::"r"(bar), "h"(both) : "memory");
}
// ---- block-scaled MXFP8 (e4m3 data, e8m0 scale per 32 elements along K) -------------------------------------
// Shared-memory descriptor of one 512-byte scale tile (32 rows x 16 bytes, no swizzle): 8-row groups 128 B apart.
__device__ __forceinline__ uint64_t umma_scale_desc(uint32_t saddr) {
    uint64_t d = 0;
    d |= static_cast<uint64_t>((saddr & 0x3FFFFu) >> 4);
    d |= static_cast<uint64_t>(128u >> 4) << 32;
    d |= 1ull << 46;
    return d;
}
// Copies a scale tile from each CTA's shared memory into the same tensor-memory columns of each CTA; the 32
// source rows are replicated to all four lane quarters.
__device__ __forceinline__ void tmem_copy_scales_pair(uint32_t taddr, uint64_t sdesc) {
    asm volatile("tcgen05.cp.cta_group::2.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(sdesc) : "memory");
}
// Instruction descriptor for kind::mxf8f6f4.block_scale, e4m3 x e4m3 -> fp32, both operands K-major, e8m0 scales.
// Bits: B scale id at 4, A/B formats (0 = e4m3) at 7 / 10, N >> 3 at 17, scale format (1 = e8m0) at 23, M >> 4 at
// 24, A scale id at 29.  The scale id picks which byte of the 32-bit scale column belongs to this K slice of 32.
__host__ __device__ constexpr uint32_t umma_idesc_mxfp8(int m, int n, uint32_t sf_id) {
    return (sf_id << 4) | (static_cast<uint32_t>(n >> 3) << 17) | (1u << 23) | (static_cast<uint32_t>(m >> 4) << 24) |
           (sf_id << 29);
}
__device__ __forceinline__ void umma_mxfp8_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                                uint32_t sfa_tmem, uint32_t sfb_tmem, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::mxf8f6f4.block_scale [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(sfa_tmem), "r"(sfb_tmem)
        : "memory");
}

// Arrive on an mbarrier of the leader CTA from either CTA of the pair.
__device__ __forceinline__ void mbar_arrive_leader(uint32_t bar) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(bar & kPairLeaderMask) : "memory");
}

// ---- GEMM epilogue staging -----------------------------------------------------------------------------------
// After tcgen05.ld a thread holds 64 consecutive fp32 columns of ONE accumulator row; written straight to global
// memory a warp would touch 32 rows with 16 bytes each per store instruction.  Each epilogue warp therefore owns a
// small shared-memory patch (32 rows x 128 B, rows padded to 144 B so both access patterns are conflict free):
// rows are written there as bf16, read back four rows per instruction, and stored as full 128-byte lines.
constexpr int kEpiRowPitch = 144;
constexpr int kEpiWarpBytes = 32 * kEpiRowPitch;

__device__ __forceinline__ uint4 pack8_bf16(const uint32_t* f) {
    return make_uint4(pack_bf16x2(__uint_as_float(f[0]), __uint_as_float(f[1])), pack_bf16x2(__uint_as_float(f[2]), __uint_as_float(f[3])),
                      pack_bf16x2(__uint_as_float(f[4]), __uint_as_float(f[5])), pack_bf16x2(__uint_as_float(f[6]), __uint_as_float(f[7])));
}

// v0 / v1: columns [0,32) / [32,64) of this lane's row.  row0_out: global address of the warp's first row at the
// first of the 64 columns; rows are ldd elements apart.
__device__ __forceinline__ void epilogue_store_64cols(uint8_t* warp_patch, const uint32_t (&v0)[32], const uint32_t (&v1)[32],
                                                      __nv_bfloat16* row0_out, long long ldd, int lane) {
    uint4* mine = reinterpret_cast<uint4*>(warp_patch + lane * kEpiRowPitch);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        mine[i] = pack8_bf16(&v0[8 * i]);
        mine[4 + i] = pack8_bf16(&v1[8 * i]);
    }
    __syncwarp();
    const int seg = lane & 7;
#pragma unroll
    for (int it = 0; it < 8; ++it) {
        const int r = it * 4 + (lane >> 3);
        const uint4 w = *reinterpret_cast<const uint4*>(warp_patch + r * kEpiRowPitch + seg * 16);
        *reinterpret_cast<uint4*>(row0_out + static_cast<long long>(r) * ldd + seg * 8) = w;
    }
    __syncwarp();
}

// Same, for 64 columns that are already packed to bf16 (8 x 16 bytes of this lane's row).
__device__ __forceinline__ void epilogue_store_packed_64cols(uint8_t* warp_patch, const uint4* row_vectors, __nv_bfloat16* row0_out,
                                                             long long ldd, int lane) {
    uint4* mine = reinterpret_cast<uint4*>(warp_patch + lane * kEpiRowPitch);
#pragma unroll
    for (int i = 0; i < 8; ++i) mine[i] = row_vectors[i];
    __syncwarp();
    const int seg = lane & 7;
#pragma unroll
    for (int it = 0; it < 8; ++it) {
        const int r = it * 4 + (lane >> 3);
        const uint4 w = *reinterpret_cast<const uint4*>(warp_patch + r * kEpiRowPitch + seg * 16);
        *reinterpret_cast<uint4*>(row0_out + static_cast<long long>(r) * ldd + seg * 8) = w;
    }
    __syncwarp();
}

// Shared-memory matrix descriptor for a 128-byte-swizzled operand tile whose base is 1024-byte aligned.
// Fields (Blackwell): start address >> 4 at bit 0, leading byte offset >> 4 at bit 16, stride byte offset >> 4
// at bit 32, descriptor version 1 at bit 46, layout type 2 (128B swizzle) at bit 61.
__device__ __forceinline__ uint64_t umma_smem_desc(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
    uint64_t d = 0;
    d |= static_cast<uint64_t>((saddr & 0x3FFFFu) >> 4);
    d |= static_cast<uint64_t>((lbo_bytes >> 4) & 0x3FFFu) << 16;
    d |= static_cast<uint64_t>((sbo_bytes >> 4) & 0x3FFFu) << 32;
    d |= 1ull << 46;
    d |= 2ull << 61;
    return d;
}

// Instruction descriptor for kind::f16 with bf16 A/B and fp32 D.  Bits: D format (1 = fp32) at 4, A format
// (1 = bf16) at 7, B format at 10, A major (1 = MN) at 15, B major at 16, N >> 3 at 17, M >> 4 at 24.
__host__ __device__ constexpr uint32_t umma_idesc_bf16(int m, int n, bool a_mn_major, bool b_mn_major) {
    return (1u << 4) | (1u << 7) | (1u << 10) | (static_cast<uint32_t>(a_mn_major) << 15) |
           (static_cast<uint32_t>(b_mn_major) << 16) | (static_cast<uint32_t>(n >> 3) << 17) |
           (static_cast<uint32_t>(m >> 4) << 24);
}

}  // namespace mok
