// CPU walk over the grouped GEMM's static tile lists (the same decode_tile / total_tiles the kernels run): every
// output tile of the rows form appears exactly once and lies inside one expert's row range; the K ranges of the
// weight-gradient form, taken over all windows, cover each expert's occupied rows exactly once, in order, and the
// "accumulate" flag is set exactly for the windows that do not hold the expert's first row.
// Built and run by tests/test_tile_math_cpu.py (nvcc, host code only; no GPU needed).
#include <algorithm>
#include <cstdio>
#include <cstdlib>
#include <set>
#include <vector>

#include "../mixture-of-kittens_b200/csrc/gemm_tiles.cuh"

using namespace mok::tiles;

static unsigned g_seed = 12345;
static int rnd(int n) {
    g_seed = g_seed * 1664525u + 1013904223u;
    return static_cast<int>((g_seed >> 8) % static_cast<unsigned>(n));
}

#define CHECK(cond)                                                                    \
    do {                                                                               \
        if (!(cond)) {                                                                 \
            std::printf("FAILED %s (line %d, case %d)\n", #cond, __LINE__, case_index); \
            return 1;                                                                  \
        }                                                                              \
    } while (0)

template <int BK>
static int run_case(int case_index, int num_experts, int window_rows, bool trim, int m_blocks, int n_blocks) {
    std::vector<int> tokens(num_experts), occupied(num_experts), cum(num_experts + 1, 0);
    for (int e = 0; e < num_experts; ++e) {
        const int valid = rnd(4) == 0 ? 0 : 1 + rnd(900);
        tokens[e] = (valid + 255) / 256 * 256;
        occupied[e] = valid;
        cum[e + 1] = cum[e] + tokens[e];
    }
    const int total_rows = cum[num_experts];
    if (total_rows == 0) return 0;
    KernelParams p{};
    p.tokens_per_expert = tokens.data();
    p.num_experts = num_experts;
    p.occupied_rows = trim ? occupied.data() : nullptr;
    p.n_blocks = n_blocks;
    p.m_blocks_w = m_blocks;
    p.k_blocks = 5;
    p.n_sets = 2;
    p.k_sets = 1;

    std::set<long long> seen;                                   // rows form: (row0, set, n0) exactly once
    std::vector<std::vector<std::pair<int, int>>> k_ranges(num_experts);   // wgrad: per expert the [begin, end) pieces
    for (int lo = 0; lo < total_rows; lo += window_rows) {
        const int hi = lo + window_rows < total_rows ? lo + window_rows : total_rows;
        p.row_begin = lo;
        p.row_end = lo + window_rows;
        const int n_rows_tiles = total_tiles<MODE_ROWS>(p, lo, hi);
        CHECK(n_rows_tiles == (hi - lo) / BM * p.n_blocks * p.n_sets);
        for (int t = 0; t < n_rows_tiles; ++t) {
            Tile tile;
            CHECK((decode_tile<MODE_ROWS, BK>(p, cum.data(), lo, hi, t, tile)));
            CHECK(tile.row0 >= lo && tile.row0 + BM <= hi && tile.row0 % BM == 0);
            CHECK(tile.expert >= 0 && tile.expert < num_experts);
            CHECK(cum[tile.expert] <= tile.row0 && tile.row0 + BM <= cum[tile.expert + 1]);   // one expert per tile
            CHECK(tile.set >= 0 && tile.set < p.n_sets && tile.n0 % BN == 0 && tile.n0 / BN < p.n_blocks);
            CHECK(tile.k_blocks == p.k_blocks * p.k_sets && tile.accumulate == 0);
            const long long key = (static_cast<long long>(tile.row0) * 8 + tile.set) * 1024 + tile.n0 / BN;
            CHECK(seen.insert(key).second);
        }
        const int n_wgrad = total_tiles<MODE_WGRAD>(p, lo, hi);
        CHECK(n_wgrad == num_experts * p.m_blocks_w * p.n_blocks);
        std::set<long long> wgrad_seen;                         // (expert, m tile, n tile) exactly once per window
        for (int t = 0; t < n_wgrad; ++t) {
            Tile tile;
            const bool work = decode_tile<MODE_WGRAD, BK>(p, cum.data(), lo, hi, t, tile);
            const int e = tile.expert;
            CHECK(e == t / (p.m_blocks_w * p.n_blocks));
            CHECK(tile.m0 % BM == 0 && tile.m0 / BM < p.m_blocks_w && tile.n0 % BN == 0 && tile.n0 / BN < p.n_blocks);
            CHECK(wgrad_seen.insert((static_cast<long long>(e) * 1024 + tile.m0 / BM) * 1024 + tile.n0 / BN).second);
            if (!work) continue;
            CHECK(tile.k_blocks > 0 && tile.row0 >= lo && tile.row0 + tile.k_blocks * BK <= hi);
            CHECK(tile.row0 >= cum[e] && tile.row0 + tile.k_blocks * BK <= cum[e + 1]);
            CHECK(tile.accumulate == (cum[e] < lo ? 1 : 0));
            if (t % (p.m_blocks_w * p.n_blocks) == 0) k_ranges[e].push_back({tile.row0, tile.row0 + tile.k_blocks * BK});
        }
    }
    long long rows_tiles_expected = static_cast<long long>(total_rows / BM) * p.n_blocks * p.n_sets;
    CHECK(static_cast<long long>(seen.size()) == rows_tiles_expected);
    for (int e = 0; e < num_experts; ++e) {
        int covered_to = cum[e];
        for (auto& r : k_ranges[e]) {
            CHECK(r.first == covered_to);     // contiguous, in schedule order, no overlap between windows
            covered_to = r.second;
        }
        // all occupied rows are covered; with trimming nothing beyond them rounded up to the K step (an expert whose
        // range holds padding only still gets one K step so that its gradient is written)
        CHECK(covered_to >= cum[e] + occupied[e]);
        const int limit = trim ? cum[e] + ((occupied[e] > 0 ? occupied[e] : (tokens[e] > 0 ? 1 : 0)) + BK - 1) / BK * BK : cum[e + 1];
        CHECK(covered_to <= (limit < cum[e + 1] ? limit : cum[e + 1]) || tokens[e] == 0);
        if (!trim) CHECK(covered_to == cum[e + 1]);
    }
    return 0;
}

// The point of the weight-gradient tile order: the tiles that run at one time (one per CTA pair, 74 on a B200) should
// share few operand panels.  For every run of 74 consecutive tiles inside one expert, count the distinct row panels
// (m tiles, operand A) and column panels (n tiles, operand B) they touch.
static int worst_panels_in_flight(int m_blocks, int n_blocks, int in_flight) {
    std::vector<int> tokens(1, 1024), cum = {0, 1024};
    KernelParams p{};
    p.tokens_per_expert = tokens.data();
    p.num_experts = 1;
    p.m_blocks_w = m_blocks;
    p.n_blocks = n_blocks;
    p.row_begin = 0;
    p.row_end = 1024;
    const int total = m_blocks * n_blocks;
    std::vector<std::pair<int, int>> order(total);
    for (int t = 0; t < total; ++t) {
        Tile tile;
        decode_tile<MODE_WGRAD, 64>(p, cum.data(), 0, 1024, t, tile);
        order[t] = {tile.m0 / BM, tile.n0 / BN};
    }
    int worst = 0;
    for (int start = 0; start + in_flight <= total; ++start) {
        std::set<int> ms, ns;
        for (int t = start; t < start + in_flight; ++t) {
            ms.insert(order[t].first);
            ns.insert(order[t].second);
        }
        worst = std::max(worst, static_cast<int>(ms.size() + ns.size()));
    }
    return worst;
}

int main() {
    int case_index = 0;
    // the layer's two weight-gradient grids (2048 x 7168 and 7168 x 2048 outputs): at most 8 + 11 panels in flight,
    // where a plain row-major walk of the 8 x 28 grid touches 4 + 28
    if (worst_panels_in_flight(8, 28, 74) > 19 || worst_panels_in_flight(28, 8, 74) > 19) {
        std::printf("FAILED panels in flight: %d %d\n", worst_panels_in_flight(8, 28, 74), worst_panels_in_flight(28, 8, 74));
        return 1;
    }
    for (int experts : {1, 3, 17, 64}) {
        for (int window : {256, 1024, 4096, 1 << 20}) {
            for (int trim = 0; trim < 2; ++trim) {
                if (run_case<64>(case_index++, experts, window, trim != 0, 2, 3)) return 1;    // bf16 kernel's K step
                if (run_case<128>(case_index++, experts, window, trim != 0, 2, 3)) return 1;   // MXFP8 kernel's K step
            }
        }
        // output tile grids of the weight-gradient form: the benchmark's (8 x 28 and 28 x 8), square, one wide enough to
        // be cut into groups with a narrower last group, and single-tile edges
        for (auto mn : {std::pair<int, int>{8, 28}, {28, 8}, {13, 13}, {21, 30}, {1, 5}, {7, 1}})
            if (run_case<64>(case_index++, experts, 4096, true, mn.first, mn.second)) return 1;
    }
    std::printf("ok %d cases\n", case_index);
    return 0;
}
