// Pieces shared by the bf16 and the MXFP8 grouped-GEMM kernels: tile geometry, the static tile list of the three
// forms, the per-row epilogue store used when accumulating, and the host-side launch plumbing (tensor-map encoder,
// CTA-pair launch, argument checks).
#pragma once

#include "grouped_gemm.cuh"

namespace mok {
namespace tiles {

constexpr int BM = 256;        // output tile rows of a CTA pair
constexpr int BM_CTA = 128;    // rows each CTA stages and accumulates
constexpr int BN = 256;
constexpr int BN_CTA = 128;    // B columns each CTA stages
constexpr int NUM_THREADS = 192;
constexpr int TMEM_COLS = 512;
constexpr int MODE_ROWS = 0;   // D[row, :] over schedule rows grouped by expert
constexpr int MODE_WGRAD = 1;  // D[e] = sum over the rows of expert e
constexpr int kWgradGroup = 8; // weight-gradient tile order: width of a group of the faster-running tile dimension

struct KernelParams {
    const int32_t* tokens_per_expert;
    const int32_t* num_tokens;
    const int32_t* occupied_rows;   // wgrad: see GemmProblem
    int scale_slots;                // MXFP8: tensor-memory slots the scale columns rotate through
    int num_experts;
    int dense_rows;
    int row_begin, row_end;
    int n_blocks;             // rows: N / 256 per output set; wgrad: N / 256
    int m_blocks_w;           // wgrad: M / 256
    int k_blocks;             // rows: K steps per operand set
    int n_sets;               // rows: output sets sharing A (1 or 2)
    int k_sets;               // rows: operand sets accumulated into one output (1 or 2)
    int n_tiles_per_expert;   // MXFP8 rows form: N / 128, scale row tiles of one expert's weight
    bf16* D0;
    bf16* D1;
    bf16* D2;                 // bf16 kernel, fused gate / up form: hidden = silu(gate) * up (D0 = gate, D1 = up)
    int clamp;                // fused gate / up form: SwiGLU clamp on
    float limit;
    int out_f32;              // bf16 kernel: D0 is an fp32 array (router logits and router weight gradient)
    long long ldd;
    long long d_expert_stride;
    uint32_t* status;
};

struct Tile {
    int expert;
    int row0;        // rows: first schedule row of the tile; wgrad: first K row
    int m0, n0;      // wgrad: output row / column offset; rows: n0 = column offset
    int set;         // rows: output set
    int k_blocks;    // K steps
    int accumulate;  // wgrad: add to what is already stored (the expert's rows began in an earlier window)
};

// Tile t of the static list.  rows: m tile major, then output set, then n tile, so that the tiles running at one
// time share an expert's weights in L2.  wgrad: expert major, then as described below.  Returns false for tiles
// without work.
// (host-callable too: tests/tile_math_host.cu walks the tile lists on the CPU)
template <int MODE, int BK>
__host__ __device__ __forceinline__ bool decode_tile(const KernelParams& p, const int* cum, int lo, int hi, int t, Tile& tile) {
    if (MODE == MODE_ROWS) {
        const int per_m = p.n_blocks * p.n_sets;
        const int mt = t / per_m;
        const int rem = t - mt * per_m;
        tile.set = rem / p.n_blocks;
        tile.n0 = (rem - tile.set * p.n_blocks) * BN;
        tile.row0 = lo + mt * BM;
        tile.m0 = 0;
        int e = 0;
        if (p.tokens_per_expert != nullptr) {   // largest e with cum[e] <= row0
            int a = 0, b = p.num_experts;
            while (b - a > 1) {
                const int mid = (a + b) >> 1;
                if (cum[mid] <= tile.row0) a = mid; else b = mid;
            }
            e = a;
        }
        tile.expert = e;
        tile.k_blocks = p.k_blocks * p.k_sets;
        tile.accumulate = 0;
        return true;
    } else {
        const int per_e = p.m_blocks_w * p.n_blocks;
        const int e = t / per_e;
        const int rem = t - e * per_e;
        // Order of an expert's output tiles: the tiles that run at one time (one per CTA pair) should share as few
        // operand panels as possible, so that the panels (K x 256 each, megabytes when an expert holds thousands of
        // rows) stay in L2: the dimension with fewer tiles runs fastest, in groups of at most kWgradGroup, the other
        // dimension next, the groups slowest.  74 pairs then touch about 8 + 9 panels instead of up to 28 + 3.
        const bool m_inner = p.m_blocks_w <= p.n_blocks;
        const int d_in = m_inner ? p.m_blocks_w : p.n_blocks;
        const int d_out = m_inner ? p.n_blocks : p.m_blocks_w;
        const int group = d_in <= kWgradGroup + kWgradGroup / 2 ? d_in : kWgradGroup;
        const int g = rem / (group * d_out);
        const int width = min(group, d_in - g * group);
        const int r2 = rem - g * group * d_out;
        const int outer = r2 / width;
        const int inner = g * group + (r2 - outer * width);
        tile.expert = e;
        tile.m0 = (m_inner ? inner : outer) * BM;
        tile.n0 = (m_inner ? outer : inner) * BN;
        tile.set = 0;
        const int ks = max(cum[e], lo);
        int ke = min(cum[e + 1], hi);
        // at least one K step, so that an expert whose range holds padding only still gets its (zero) gradient written
        if (p.occupied_rows != nullptr) ke = min(ke, cum[e] + (max(p.occupied_rows[e], 1) + BK - 1) / BK * BK);
        tile.row0 = ks;
        tile.k_blocks = ke > ks ? (ke - ks) / BK : 0;
        tile.accumulate = cum[e] < lo ? 1 : 0;
        return tile.k_blocks > 0;
    }
}

template <int MODE>
__host__ __device__ __forceinline__ int total_tiles(const KernelParams& p, int lo, int hi) {
    if (hi <= lo) return 0;
    return MODE == MODE_ROWS ? ((hi - lo) / BM) * p.n_blocks * p.n_sets : p.num_experts * p.m_blocks_w * p.n_blocks;
}

// One warp: exclusive prefix of the padded per-expert row counts, cum[0..E] (cum[E] = padded total).
__device__ __forceinline__ void expert_row_prefix(const KernelParams& p, int* cum, int lane) {
    if (p.tokens_per_expert == nullptr) {
        if (lane == 0) { cum[0] = 0; cum[1] = p.dense_rows; }
        return;
    }
    int carry = 0;
    if (lane == 0) cum[0] = 0;
    for (int base = 0; base < p.num_experts; base += 32) {
        const int idx = base + lane;
        int v = idx < p.num_experts ? p.tokens_per_expert[idx] : 0;
#pragma unroll
        for (int off = 1; off < 32; off <<= 1) {
            const int n = __shfl_up_sync(0xffffffffu, v, off);
            if (lane >= off) v += n;
        }
        if (idx < p.num_experts) cum[idx + 1] = carry + v;
        carry += __shfl_sync(0xffffffffu, v, 31);
    }
}

// 32 fp32 columns of this thread's row -> bf16, optionally added (in fp32) to what global memory holds.
__device__ __forceinline__ void store_row_chunk(bf16* dst, const uint32_t (&acc)[32], bool accumulate) {
    uint4* out = reinterpret_cast<uint4*>(dst);
#pragma unroll
    for (int v = 0; v < 4; ++v) {
        float f[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) f[i] = __uint_as_float(acc[v * 8 + i]);
        if (accumulate) {
            const uint4 old = out[v];
            const float2 o0 = unpack_bf16x2(old.x), o1 = unpack_bf16x2(old.y), o2 = unpack_bf16x2(old.z), o3 = unpack_bf16x2(old.w);
            f[0] += o0.x; f[1] += o0.y; f[2] += o1.x; f[3] += o1.y;
            f[4] += o2.x; f[5] += o2.y; f[6] += o3.x; f[7] += o3.y;
        }
        uint4 w;
        w.x = pack_bf16x2(f[0], f[1]);
        w.y = pack_bf16x2(f[2], f[3]);
        w.z = pack_bf16x2(f[4], f[5]);
        w.w = pack_bf16x2(f[6], f[7]);
        out[v] = w;
    }
}

// 32 fp32 columns of this thread's row, stored as they are (one 128-byte line per thread).
__device__ __forceinline__ void store_row_chunk_f32(float* dst, const uint32_t (&acc)[32]) {
    uint4* out = reinterpret_cast<uint4*>(dst);
#pragma unroll
    for (int v = 0; v < 8; ++v) out[v] = make_uint4(acc[v * 4], acc[v * 4 + 1], acc[v * 4 + 2], acc[v * 4 + 3]);
}

// ---------------------------------------------------------------------------------------------------------
// Host side
// ---------------------------------------------------------------------------------------------------------
constexpr int kMaxDynamicSmem = 232448 - 1024;

// Rank-4 tensor map; `what` names the operand in the error string.
inline int encode_map(CUtensorMap* map, CUtensorMapDataType type, const void* base, const cuuint64_t (&dims)[4],
                      const cuuint64_t (&strides)[3], const cuuint32_t (&box)[4], CUtensorMapSwizzle swizzle) {
    typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                      const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                      CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
    static EncodeTiledFn fn = nullptr;
    if (fn == nullptr) {
        void* sym = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(sym);
    }
    if (fn == nullptr) {
        set_last_error("cuTensorMapEncodeTiled unavailable", cudaErrorNotSupported);
        return MOK_ERR_CUDA;
    }
    cuuint32_t estr[4] = {1, 1, 1, 1};
    const CUresult r = fn(map, type, 4, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle,
                          CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        set_last_error("cuTensorMapEncodeTiled failed", cudaErrorInvalidValue);
        return MOK_ERR_CUDA;
    }
    return MOK_OK;
}

inline int check_problem(const GemmProblem& pb) {
    if (pb.num_experts < 1 || pb.num_experts > MOK_MAX_LOCAL_EXPERTS) return MOK_ERR_TOO_LARGE;
    if (pb.row_begin < 0 || pb.row_end < pb.row_begin || (pb.row_begin % BM) != 0 || (pb.row_end % BM) != 0)
        return MOK_ERR_INVALID_ARGUMENT;
    if (pb.tokens_per_expert == nullptr && (pb.num_experts != 1 || pb.dense_rows % BM != 0)) return MOK_ERR_INVALID_ARGUMENT;
    if (pb.tokens_per_expert != nullptr && pb.num_tokens == nullptr) return MOK_ERR_INVALID_ARGUMENT;
    return MOK_OK;
}

inline KernelParams base_params(const GemmProblem& pb) {
    KernelParams kp{};
    kp.tokens_per_expert = pb.tokens_per_expert;
    kp.num_tokens = pb.num_tokens;
    kp.occupied_rows = pb.occupied_rows;
    kp.scale_slots = 1;
    kp.num_experts = pb.num_experts;
    kp.dense_rows = pb.dense_rows;
    kp.row_begin = pb.row_begin;
    kp.row_end = pb.row_end;
    kp.n_sets = 1;
    kp.k_sets = 1;
    kp.status = pb.status;
    return kp;
}

// Launches `kernel` as clusters of two CTAs, as many pairs as can be resident at once (at most one per tile).
// `resident_pairs` caches the occupancy query per device and kernel instantiation.
template <typename Kernel, typename... Args>
int launch_pairs(Kernel kernel, const char* name, int (&resident_pairs)[16], size_t smem, int max_tiles, cudaStream_t stream,
                 const Args&... args) {
    int dev = 0;
    MOK_CUDA_CHECK(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 16) return MOK_ERR_UNSUPPORTED;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cudaLaunchConfig_t cfg = {};
    cfg.blockDim = dim3(NUM_THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    if (resident_pairs[dev] == 0) {
        MOK_CUDA_CHECK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kMaxDynamicSmem));
        cfg.gridDim = dim3(2 * sm_count());
        cfg.dynamicSmemBytes = kMaxDynamicSmem;
        int clusters = 0;
        MOK_CUDA_CHECK(cudaOccupancyMaxActiveClusters(&clusters, kernel, &cfg));
        cfg.dynamicSmemBytes = smem;
        resident_pairs[dev] = clusters > 0 ? clusters : sm_count() / 2;
    }
    const int pairs = resident_pairs[dev] < max_tiles ? resident_pairs[dev] : max_tiles;
    if (pairs <= 0) return MOK_OK;
    cfg.gridDim = dim3(2 * pairs);
    const cudaError_t err = cudaLaunchKernelEx(&cfg, kernel, args...);
    if (err != cudaSuccess) return fail_cuda(name, err);
    MOK_LAUNCH_CHECK(name);
    return MOK_OK;
}

}  // namespace tiles
}  // namespace mok
