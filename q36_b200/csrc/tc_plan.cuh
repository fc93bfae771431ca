// Work plan of the tensor-core grouped GEMM, shared by the kernels that build it and the one that reads it.
#pragma once
#include "kernels.cuh"

namespace q36 {

constexpr int TC_M = 128;          // weight rows per tile (UMMA M)
constexpr int TC_N_GATEUP = 112;   // token rows per gate/up tile (two accumulator sets of gate+up fit TMEM)
constexpr int TC_N_DOWN = 128;     // token rows per down tile

// Work plan of one grouped-FFN call, built on the device by k_tc_plan and read by both MMA launches.
// Groups are ranked by size (largest first); base[w][r] is the first tile of rank r for launch w
// (0 = gate/up, 1 = down), so a tile index maps to (group, token tile, row tile) by a binary search.
struct TcPlan {
    int n_groups, n_tiles[2];
    int tile_rows;                        // token rows per tile the plan was cut for, both launches (0: 112 / 128)
    int gu_done;                          // gate/up tiles whose epilogue has finished (fused decode kernel only)
    int order[DISPATCH_MAX_GROUPS + 1];   // rank -> group
    int row0[DISPATCH_MAX_GROUPS + 1];    // group -> first row of the sorted space
    int cnt[DISPATCH_MAX_GROUPS + 1];     // group -> rows
    int base[2][DISPATCH_MAX_GROUPS + 2];
    int done[DISPATCH_MAX_GROUPS + 1];    // group -> gate/up epilogue warps finished (fused decode kernel only)
};


// Block-wide: orders the groups (largest first when `rank`, else as they come -- enough when every group is
// at most one token tile) and lays the prefix sums of their tile counts.
// goffs[n_group+1] are the routed groups' row offsets; an extra group [s0, s1) follows when has_extra.
// scratch: 4 * (DISPATCH_MAX_GROUPS + 1) ints of shared memory.  Needs at least one full warp; ends with all
// plan fields written (no trailing barrier: the plan is read by later kernels only).
__device__ __forceinline__ void tc_plan_block(const int *goffs, int n_group, bool has_extra, int s0, int s1,
                                              TcPlan *plan, int mt_gu, int mt_dn, int *scratch, bool rank,
                                              int tile_rows = 0) {
    // tile_rows: token rows per tile of BOTH launches when not 0 (16: the one-launch decode kernel), else
    // TC_N_GATEUP / TC_N_DOWN
    int *cnt = scratch, *order = cnt + DISPATCH_MAX_GROUPS + 1, *tg = order + DISPATCH_MAX_GROUPS + 1,
        *td = tg + DISPATCH_MAX_GROUPS + 1;
    const int tid = threadIdx.x;
    const int G = n_group + (has_extra ? 1 : 0);
    for (int g = tid; g < G; g += blockDim.x) {
        const int r0 = (g < n_group) ? goffs[g] : s0;
        const int r1 = (g < n_group) ? goffs[g + 1] : s1;
        cnt[g] = max(0, r1 - r0);
        plan->row0[g] = r0;
        plan->cnt[g] = cnt[g];
        plan->done[g] = 0;
    }
    __syncthreads();
    for (int g = tid; g < G; g += blockDim.x) {
        int r = g;
        if (rank) {
            r = 0;
            for (int h = 0; h < G; h++) r += (cnt[h] > cnt[g]) || (cnt[h] == cnt[g] && h < g);
        }
        order[r] = g;
    }
    __syncthreads();
    for (int r = tid; r < G; r += blockDim.x) {
        const int n = cnt[order[r]];
        const int ngu = tile_rows ? tile_rows : TC_N_GATEUP, ndn = tile_rows ? tile_rows : TC_N_DOWN;
        tg[r] = ((n + ngu - 1) / ngu) * mt_gu;
        td[r] = ((n + ndn - 1) / ndn) * mt_dn;
        plan->order[r] = order[r];
    }
    __syncthreads();
    if (tid < 32) {   // exclusive scans of the two tile counts: each lane owns a contiguous run of ranks
        const int per = (G + 31) / 32;
        int sa = 0, sb = 0;
        for (int j = 0; j < per; j++) { const int r = tid * per + j; if (r < G) { sa += tg[r]; sb += td[r]; } }
        int ia = sa, ib = sb;
        for (int o = 1; o < 32; o <<= 1) {
            const int va = __shfl_up_sync(0xffffffffu, ia, o), vb = __shfl_up_sync(0xffffffffu, ib, o);
            if (tid >= o) { ia += va; ib += vb; }
        }
        int ra = ia - sa, rb = ib - sb;
        for (int j = 0; j < per; j++) {
            const int r = tid * per + j;
            if (r < G) { plan->base[0][r] = ra; plan->base[1][r] = rb; ra += tg[r]; rb += td[r]; }
        }
        if (tid == 31) {
            plan->gu_done = 0;
            plan->base[0][G] = ia; plan->base[1][G] = ib;
            plan->n_tiles[0] = ia; plan->n_tiles[1] = ib; plan->n_groups = G; plan->tile_rows = tile_rows;
        }
    }
}

}  // namespace q36
