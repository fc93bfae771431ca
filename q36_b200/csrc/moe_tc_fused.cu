// Decode-sized groups (every group has at most 16 rows): gate/up + SwiGLU + requantisation AND the down
// projection in ONE persistent tcgen05 launch.
//
// At decode the layer streams ~100 MB of expert weights and nothing else matters; two separate grouped-GEMM
// launches pay the launch, the prologue (TMEM allocation, barrier set-up, first descriptor and data fetch)
// and the drain twice.  Here every CTA walks one list: first all gate/up tiles, then all down tiles.  A down
// tile of group g reads the quantised intermediate Hq/Hs that the gate/up tiles of g wrote, possibly on other
// SMs: the gate/up epilogue warps publish with __threadfence + a counter per group, the consumers poll the
// counter (bounded), then order the generic-proxy writes before their async-proxy (TMA) reads with
// fence.proxy.async.  No deadlock: every CTA is resident (grid <= number of SMs, one CTA per SM) and a CTA
// only waits while it is in its down phase, for gate/up tiles that no CTA ever waits in.
//
// Same operand staging, scale images, descriptors and roles as k_grouped_mma (moe_tc.cu); N = 16 always.
#include "common.cuh"
#include "kernels.cuh"
#include "tc_plan.cuh"
#include "tc_ptx.cuh"

namespace q36 {

// What sets the layout (all measured on B200 with single-purpose timing loops around the instruction in question):
//  * a thread needs ~140 cycles to issue ANY asynchronous copy, so a stage is TWO K steps fetched by two copies
//    (one 4-bit weight box of 2 x [128 rows][128 elements], one box of 2 x [16 token rows][128 B]);
//  * a thread gets one block-scaled MMA through per ~90-110 cycles, the pipe takes one per ~40, so FOUR warps
//    issue, each into its own accumulator columns: warps 0,1 the two K steps of the even stages, warps 2,3 of
//    the odd ones.  A gate/up tile alternates gate and up stages, hence gate = acc0 + acc1, up = acc2 + acc3; a
//    down tile (2 stages) is the sum of all four;
//  * every role looks its tile up in a table built once per CTA (a binary search per tile per role cost ~900
//    cycles, more than a down tile's share of the HBM stream);
//  * three producer threads, because every asynchronous copy costs its issuing thread ~140 cycles: weights
//    (they depend on nothing, so this thread runs as far ahead as the ring allows), a tile's scale bytes (two
//    tiles ahead), and the token rows of each stage;
//  * gate/up tiles are dealt round-robin (tile b, b + grid, ...).  A gate/up tile is 2 D / FF (= 8) down tiles
//    of work and 260 of them do not divide by 148, so the CTAs that got one gate/up tile fewer first take a
//    few extra down tiles (the lowest ranks: their inputs are there first) -- only as many as they can finish
//    before the others join, since a group's rows arrive ~7000 cycles after its last gate/up MMA (epilogue,
//    release fence, the polls); the rest is dealt round-robin;
//  * a watcher thread walks the CTA's tile list ahead of everybody and, for a down tile, waits until the
//    gate/up tiles of its group -- possibly on other SMs -- have published Hq/Hs; the other roles poll a
//    count in shared memory, so that the L2 round trips of the check sit on nobody's issue path;
//  * publishing costs a device-scope release fence, measured at ~2500 cycles under the weight stream: a
//    publisher thread pays it, not the epilogue warps (they only signal through shared memory).
struct FusedCfg {
    static constexpr int STAGES = 4;
    static constexpr int KS = 2;                     // K steps per stage
    static constexpr int A_BYTES = TC_M * 128;       // one K step of one matrix, 4-bit codes in 8-bit containers
    static constexpr int A_TX_BYTES = TC_M * 64;     // the A box signals its packed bytes (see moe_tc.cu)
    static constexpr int B_BYTES = 16 * 128;
    static constexpr int SF_BYTES = 512;
    static constexpr int OFF_B = KS * A_BYTES, OFF_SF = OFF_B + KS * B_BYTES;
    static constexpr int STAGE_BYTES = OFF_SF + KS * 2 * SF_BYTES;          // 38 KB, 1024-aligned
    static constexpr int STAGE_TX_A = KS * A_TX_BYTES, STAGE_TX_B = KS * B_BYTES;
    // Scale bytes of a whole tile (all its K steps) are staged by bulk async copies, two tiles deep: the rows
    // of a tile are contiguous in the row-major scale planes (128 rows x K/32 bytes).  Loads issued by the
    // loader threads themselves were measured to expose a full HBM latency per 4 K steps (register prefetch
    // does not help: a warp's loads retire through a handful of shared scoreboards).
    static constexpr int K_MAX = 2048;               // largest D or FF this kernel takes (sizes the staged scale bytes)
    static constexpr int SFT_A = TC_M * (K_MAX / Q36_QK);   // 64 scale bytes per weight row
    static constexpr int SFT_B = 16 * (K_MAX / Q36_QK);
    static constexpr int SFT_BYTES = 2 * SFT_A + SFT_B;      // 17 KB: gate (or down), up, tokens
    static constexpr int SFT_SLOTS = 2;
    static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + SFT_SLOTS * SFT_BYTES + 1024 + 256;
    static constexpr int ISSUERS = 4;
    static constexpr int ACC_STRIDE = 64;            // per accumulator set: issuer w at [16 w, 16 w + 16)
    static constexpr int SF_COL0 = 128;              // per issuer: A (4), B (4)
    static constexpr int TMEM_COLS = 256;
    static constexpr int W_ISSUE0 = 3, W_EPI0 = W_ISSUE0 + ISSUERS, W_LOAD0 = W_EPI0 + 4, W_SCHED = W_LOAD0 + 4, W_PUB = W_SCHED + 1;
    // warps: weight producer, scale producer, token-row producer, issuers, epilogue, scale loaders, watcher, publisher
    static constexpr int THREADS = 32 * (W_PUB + 1);
    static constexpr int DONE_PER_GROUP_PER_MTILE = 4;   // epilogue warps
    static constexpr int MAX_GROUPS = DISPATCH_MAX_GROUPS + 1;   // the plan lists every group, empty ones included
    static constexpr int MAX_TILES = 192;                // per CTA
    static constexpr int TILE_ROWS = 16;                 // token rows per tile: the plan must be cut for this
    static constexpr int EXTRA_DOWN = 3;                 // extra down tiles of a CTA that is one gate/up tile short
};
static_assert(FusedCfg::STAGE_BYTES % 1024 == 0, "stage alignment");

struct FusedMaps { CUtensorMap g, u, d, sg, su, sd, x, h; };

struct FTile { int kind, g, mt, row0, nrows; };

__global__ void __launch_bounds__(FusedCfg::THREADS, 1)
k_ffn_fused_small(const __grid_constant__ FusedMaps maps, const uint8_t *__restrict__ sfG, const uint8_t *__restrict__ sfU,
                  const uint8_t *__restrict__ sfD, uint64_t sf_stride, const uint8_t *__restrict__ sfSG,
                  const uint8_t *__restrict__ sfSU, const uint8_t *__restrict__ sfSD, int n_routed,
                  const uint8_t *__restrict__ Xs, TcPlan *__restrict__ plan, uint8_t *__restrict__ Hq,
                  uint8_t *__restrict__ Hs, float *__restrict__ Y, int D, int FF, int *__restrict__ status,
                  const EpReturnArgs ep) {
    // ep.peers != nullptr (the expert-parallel step): the result row of sorted row r < ep.n_map is the answer to the
    // received slot ep.rowmap[r] and goes straight into the result area of that slot's source rank, over NVLink,
    // instead of row r of Y; the last CTA to finish publishes the call's epoch in every source's header
    using Cfg = FusedCfg;
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t *sft = smem + Cfg::STAGES * Cfg::STAGE_BYTES;
    uint64_t *bars = reinterpret_cast<uint64_t *>(sft + Cfg::SFT_SLOTS * Cfg::SFT_BYTES);
    __shared__ uint32_t tmem_base_s;
    __shared__ volatile int abort_flag;
    __shared__ int s_ready;                        // tile records [0, s_ready) are valid and their inputs are there
    __shared__ int s_pub;                          // gate/up epilogue warps finished (all tiles of this CTA)
    __shared__ int s_row0[Cfg::MAX_GROUPS + 1], s_base0[Cfg::MAX_GROUPS + 2], s_base1[Cfg::MAX_GROUPS + 2];
    __shared__ unsigned short s_order[Cfg::MAX_GROUPS + 1], s_cnt[Cfg::MAX_GROUPS + 1];
    __shared__ int4 s_tiles[Cfg::MAX_TILES];       // x = group | kind << 16, y = row tile, z = first row, w = rows

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t full0 = smem_u32(bars), empty0 = smem_u32(bars + Cfg::STAGES);
    const uint32_t acc_full0 = smem_u32(bars + 2 * Cfg::STAGES), acc_empty0 = smem_u32(bars + 2 * Cfg::STAGES + 2);
    const uint32_t sft_full0 = smem_u32(bars + 2 * Cfg::STAGES + 4), sft_empty0 = smem_u32(bars + 2 * Cfg::STAGES + 6);

    // ---- prologue that needs nothing from earlier kernels: runs while they drain
    if (threadIdx.x == 0) {
        abort_flag = 0;
        s_ready = 0;
        s_pub = 0;
        for (int s = 0; s < Cfg::STAGES; s++) {
            mbar_init(full0 + 8 * s, 2 + 4);              // the two producers' expect_tx arrives + one per scale warp
            mbar_init(empty0 + 8 * s, 2);                 // one tcgen05.commit per issuing warp of the stage
        }
        for (int b = 0; b < 2; b++) {
            mbar_init(sft_full0 + 8 * b, 1);              // producer's expect_tx arrive
            mbar_init(sft_empty0 + 8 * b, 4);             // one arrive per scale warp
            mbar_init(acc_full0 + 8 * b, Cfg::ISSUERS);   // one tcgen05.commit per issuing warp
            mbar_init(acc_empty0 + 8 * b, 4);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (threadIdx.x >= 32 && threadIdx.x < 40)     // the eight descriptors, fetched while the previous kernel drains
        asm volatile("prefetch.tensormap [%0];" ::"l"(&maps.g + (threadIdx.x - 32)) : "memory");
    if (warp == Cfg::W_ISSUE0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_s)), "r"(Cfg::TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    // Synchronise FIRST, then let the next kernel of the stream start: whatever follows this kernel may rely on
    // everything before it (the front end's routing results) being complete as soon as it runs at all.
    cudaGridDependencySynchronize();
    cudaTriggerProgrammaticLaunchCompletion();
    Q36_TR_BEGIN(status, 4)
    // from here on: global memory written by earlier kernels (the plan, Xq/Xs)

    const int G = plan->n_groups;
    const int n0 = plan->n_tiles[0], n_tiles = n0 + plan->n_tiles[1];
    const int mt_gu = FF / TC_M;
    const int n1 = n_tiles - n0, grid = gridDim.x, b = blockIdx.x;
    // this CTA's list: its gate/up tiles, its extra down tiles if it is one gate/up tile short, its share of the rest
    const int n_long = n0 % grid;                              // CTAs [0, n_long) have one gate/up tile more
    const int n_short = n_long ? grid - n_long : 0;
    // (a CTA without any gate/up tile has nothing to read before the first round is published: no extras then)
    const int extra_total = n0 >= grid ? min(n1, n_short * Cfg::EXTRA_DOWN) : 0;
    const int my_gu = b < n0 ? (n0 - b + grid - 1) / grid : 0;
    const int sb = b - n_long;                                 // index among the short CTAs
    const int my_extra = (n_short && sb >= 0 && sb < extra_total) ? (extra_total - sb + n_short - 1) / n_short : 0;
    const int n_rest = n1 - extra_total;
    const int my_rest = b < n_rest ? (n_rest - b + grid - 1) / grid : 0;
    int my_tiles = my_gu + my_extra + my_rest;
    const bool fits = G <= Cfg::MAX_GROUPS && my_tiles <= Cfg::MAX_TILES && plan->tile_rows == Cfg::TILE_ROWS;
    if (!fits) {                                               // (uniform over the CTA) nothing is computed, the status says so
        my_tiles = 0;
        if (threadIdx.x == 0) atomicCAS(status, 0, 0x900);
    }
    for (int i = threadIdx.x; i <= G && fits; i += blockDim.x) {
        s_base0[i] = plan->base[0][i];
        s_base1[i] = plan->base[1][i];
        if (i < G) { s_order[i] = (unsigned short)plan->order[i]; s_row0[i] = plan->row0[i]; s_cnt[i] = (unsigned short)plan->cnt[i]; }
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = tmem_base_s;
    if ((int)threadIdx.x < my_tiles) {
        const int i = threadIdx.x;
        const int kind = i >= my_gu;
        const int t = !kind ? b + i * grid
                            : (i < my_gu + my_extra ? sb + (i - my_gu) * n_short : extra_total + b + (i - my_gu - my_extra) * grid);
        const int *base = kind ? s_base1 : s_base0;
        int lo = 0, hi = G - 1;
        while (lo < hi) {
            const int mid = (lo + hi + 1) >> 1;
            if (base[mid] <= t) lo = mid; else hi = mid - 1;
        }
        // within a group: token tile slowest, row tile fastest (a group of more than 16 rows is several token tiles)
        const int g = s_order[lo], local = t - base[lo], m_tiles = kind ? D / TC_M : mt_gu;
        const int nt = local / m_tiles, mt = local - nt * m_tiles;
        s_tiles[i] = make_int4(g | (kind << 16), mt, s_row0[g] + nt * Cfg::TILE_ROWS, min(Cfg::TILE_ROWS, (int)s_cnt[g] - nt * Cfg::TILE_ROWS));
    }
    __syncthreads();
    auto get_tile = [&](int j) {
        const int4 v = s_tiles[j];
        return FTile{v.x >> 16, v.x & 0xffff, v.y, v.z, v.w};
    };
    // Every role walks j = 0, 1, ...: true once the watcher has seen tile j's inputs, false when the CTA has no
    // tile j.  Only the roles that READ a down tile's token rows have to wait; the others just walk the list.
    auto tile_wait = [&](int j, int where) -> bool {
        if (j >= my_tiles) return false;
        for (uint32_t i = 0; i < TC_SPIN_LIMIT; i++) {
            int v;
            asm volatile("ld.acquire.cta.shared.s32 %0, [%1];" : "=r"(v) : "r"(smem_u32(&s_ready)) : "memory");
            if (v > j) return true;
            if ((i & 255u) == 255u && abort_flag) return false;
        }
        abort_flag = 1;
        atomicCAS(status, 0, where);
        return false;
    };
    // gate/up of group g is complete when every epilogue warp of each of its tiles has published
    auto done_target_of = [&](int g) { return (((int)s_cnt[g] + Cfg::TILE_ROWS - 1) / Cfg::TILE_ROWS) * mt_gu * Cfg::DONE_PER_GROUP_PER_MTILE; };
    auto wait_group = [&](int g, int where) -> bool {
        const int done_target = done_target_of(g);
        const volatile int *p = plan->done + g;
        for (uint32_t i = 0; i < TC_SPIN_LIMIT; i++) {
            int v;
            asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
            if (v >= done_target) return true;
            if ((i & 255u) == 255u && abort_flag) return false;
            __nanosleep(64);
        }
        abort_flag = 1;
        atomicCAS(status, 0, where);
        return false;
    };
    if (warp == 0) {
        // ------------------------------------------- TMA producer: weights (they depend on nothing)
        if (lane == 0) {
            uint32_t it = 0;
            bool ok = true;
            const uint64_t w_policy = l2_policy_evict_first();
            for (int j = 0; j < my_tiles && ok; j++) {
                const FTile t = get_tile(j);
                const bool sh = t.g >= n_routed;
                const int ge = sh ? 0 : t.g;
                const bool once = (int)s_cnt[t.g] <= Cfg::TILE_ROWS;    // a group of one token tile: its weights are read once
                const CUtensorMap *ma0 = t.kind ? (sh ? &maps.sd : &maps.d) : (sh ? &maps.sg : &maps.g);
                const CUtensorMap *ma1 = sh ? &maps.su : &maps.u;
                const int nst = t.kind ? FF / (Cfg::KS * TC_KSTEP) : 2 * (D / (Cfg::KS * TC_KSTEP));   // gate, up, gate, ...
                for (int q = 0; q < nst; q++, it++) {
                    const int kpair = t.kind ? q : (q >> 1);
                    const int s = it % Cfg::STAGES;
                    const uint32_t ph = (it / Cfg::STAGES) & 1;
                    if (!(ok = mbar_wait(empty0 + 8 * s, ph ^ 1, &abort_flag, status, 0x100 + s))) break;
                    const uint32_t sb = smem_u32(smem + s * Cfg::STAGE_BYTES);
                    mbar_expect_tx(full0 + 8 * s, Cfg::STAGE_TX_A);
                    // weights that are read once per call: evict-first in L2, so that they do not displace the token rows,
                    // the intermediate and the scale bytes that other SMs re-read (measured: 25.95 against 26.5 us per launch)
                    if (once) tma_load_4d_hint(sb, (!t.kind && (q & 1)) ? ma1 : ma0, 0, t.mt * TC_M, kpair * Cfg::KS, ge, full0 + 8 * s, w_policy);
                    else tma_load_4d(sb, (!t.kind && (q & 1)) ? ma1 : ma0, 0, t.mt * TC_M, kpair * Cfg::KS, ge, full0 + 8 * s);
                }
            }
        }
    } else if (warp == 1) {
        // ----- scale producer: a tile's scale bytes, contiguous runs of the row-major planes, two tiles deep
        if (lane == 0) {
            bool ok = true;
            const uint64_t s_policy = l2_policy_evict_first();
            for (int j = 0; ok && tile_wait(j, 0x680); j++) {
                const FTile t = get_tile(j);
                // (the watcher's acquire ordered the other CTAs' generic-proxy stores of Hq/Hs; this orders them
                // before this thread's asynchronous reads.  The all-spaces form of the fence costs ~1000 cycles.)
                if (t.kind) asm volatile("fence.proxy.async.global;" ::: "memory");
                const bool sh = t.g >= n_routed;
                const int ge = sh ? 0 : t.g;
                const uint32_t slot = j & 1;
                if (!(ok = mbar_wait(sft_empty0 + 8 * slot, ((j >> 1) & 1) ^ 1, &abort_flag, status, 0x800 + slot))) break;
                const int nbk = (t.kind ? FF : D) / Q36_QK;
                const uint32_t a_bytes = TC_M * nbk, b_bytes = t.nrows * nbk;
                const size_t arow = (size_t)ge * sf_stride + (size_t)(t.mt * TC_M) * nbk;
                const uint8_t *p0 = t.kind ? (sh ? sfSD : sfD) : (sh ? sfSG : sfG);
                const uint32_t dst = smem_u32(sft + slot * Cfg::SFT_BYTES);
                mbar_expect_tx(sft_full0 + 8 * slot, a_bytes * (t.kind ? 1 : 2) + b_bytes);
                if ((int)s_cnt[t.g] <= Cfg::TILE_ROWS) {      // read once, like the tile's weights: evict-first
                    bulk_load_hint(dst, p0 + arow, a_bytes, sft_full0 + 8 * slot, s_policy);
                    if (!t.kind) bulk_load_hint(dst + Cfg::SFT_A, (sh ? sfSU : sfU) + arow, a_bytes, sft_full0 + 8 * slot, s_policy);
                } else {
                    bulk_load(dst, p0 + arow, a_bytes, sft_full0 + 8 * slot);
                    if (!t.kind) bulk_load(dst + Cfg::SFT_A, (sh ? sfSU : sfU) + arow, a_bytes, sft_full0 + 8 * slot);
                }
                bulk_load(dst + 2 * Cfg::SFT_A, (t.kind ? Hs : Xs) + (size_t)t.row0 * nbk, b_bytes, sft_full0 + 8 * slot);
            }
        }
    } else if (warp == 2) {
        // ----- token-row producer: per stage the 16 token rows of its two K steps
        if (lane == 0) {
            uint32_t it = 0;
            bool ok = true;
            for (int j = 0; ok && tile_wait(j, 0x690); j++) {
                const FTile t = get_tile(j);
                if (t.kind) asm volatile("fence.proxy.async.global;" ::: "memory");   // as in the scale producer
                const CUtensorMap *mb = t.kind ? &maps.h : &maps.x;
                const int nst = t.kind ? FF / (Cfg::KS * TC_KSTEP) : 2 * (D / (Cfg::KS * TC_KSTEP));
                for (int q = 0; q < nst; q++, it++) {
                    const int kpair = t.kind ? q : (q >> 1);
                    const int s = it % Cfg::STAGES;
                    const uint32_t ph = (it / Cfg::STAGES) & 1;
                    if (!(ok = mbar_wait(empty0 + 8 * s, ph ^ 1, &abort_flag, status, 0x180 + s))) break;
                    mbar_expect_tx(full0 + 8 * s, Cfg::STAGE_TX_B);
                    tma_load_3d(smem_u32(smem + s * Cfg::STAGE_BYTES) + Cfg::OFF_B, mb, 0, t.row0, kpair * Cfg::KS, full0 + 8 * s);
                }
            }
        }
    } else if (warp < Cfg::W_EPI0) {
        // ----------------------------------------------------- MMA issuers
        if (lane == 0) {
            const int w = warp - Cfg::W_ISSUE0;
            const int par = w >> 1, h = w & 1;             // stages with (stage & 1) == par, K step h of the stage
            const uint32_t t_sfa = tmem + Cfg::SF_COL0 + 8 * w, t_sfb = t_sfa + 4;
            uint32_t it0 = 0;
            bool ok = true;
            for (int j = 0; j < my_tiles && ok; j++) {
                const int kind = s_tiles[j].x >> 16;
                const int nst = kind ? FF / (Cfg::KS * TC_KSTEP) : 2 * (D / (Cfg::KS * TC_KSTEP));
                const uint32_t buf = j & 1;
                const uint32_t d_tmem = tmem + buf * Cfg::ACC_STRIDE + 16 * w;
                if (!(ok = mbar_wait(acc_empty0 + 8 * buf, ((j >> 1) & 1) ^ 1, &abort_flag, status, 0x200 + buf))) break;
                tc_fence_after();
                bool first = true;
                for (int q = par; q < nst; q += 2) {
                    const uint32_t it = it0 + q;
                    const int s = it % Cfg::STAGES;
                    const uint32_t ph = (it / Cfg::STAGES) & 1;
                    if (!(ok = mbar_wait(full0 + 8 * s, ph, &abort_flag, status, 0x300 + s))) break;
                    tc_fence_after();
                    const uint32_t sb = smem_u32(smem + s * Cfg::STAGE_BYTES);
                    const uint32_t sa = sb + h * Cfg::A_BYTES, sbb = sb + Cfg::OFF_B + h * Cfg::B_BYTES;
                    const uint32_t sf = sb + Cfg::OFF_SF + h * 2 * Cfg::SF_BYTES;
                    tc_cp_sf(t_sfa, desc_sf(sf));
                    tc_cp_sf(t_sfb, desc_sf(sf + Cfg::SF_BYTES));
#pragma unroll
                    for (int kb = 0; kb < 4; kb++) {
                        const uint32_t sfid = (uint32_t)kb << 30;
                        tc_mma(d_tmem, desc_sw128(sa + kb * 32), desc_sw128(sbb + kb * 32), idesc_mx(16, kb),
                               t_sfa | sfid, t_sfb | sfid, (first && kb == 0) ? 0u : 1u);
                    }
                    first = false;
                    tc_commit(empty0 + 8 * s);
                }
                it0 += nst;
                if (ok) tc_commit(acc_full0 + 8 * buf);
            }
        }
    } else if (warp < Cfg::W_LOAD0) {
        // -------------------------------------------------------- epilogue
        const int q = warp & 3;                            // the TMEM lane quadrant this warp may read
        bool ok = true;
        for (int j = 0; j < my_tiles && ok; j++) {
            const FTile t = get_tile(j);
            const uint32_t buf = j & 1;
            const uint32_t tq = tmem + buf * Cfg::ACC_STRIDE + ((uint32_t)(q * 32) << 16);
            if (!(ok = mbar_wait(acc_full0 + 8 * buf, (j >> 1) & 1, &abort_flag, status, 0x400 + buf))) break;
            tc_fence_after();
            const int mrow = t.mt * TC_M + q * 32 + lane;
            // four partial sums of 16 token columns each (see FusedCfg)
            float g[16], u[16];
            {
                uint32_t r0[32], r1[32];
                tc_ld32(tq, r0);
                tc_ld32(tq + 32, r1);
                tc_ld_wait();
#pragma unroll
                for (int c = 0; c < 16; c++) {
                    g[c] = __uint_as_float(r0[c]) + __uint_as_float(r0[16 + c]);
                    u[c] = __uint_as_float(r1[c]) + __uint_as_float(r1[16 + c]);
                    if (t.kind) g[c] += u[c];
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(acc_empty0 + 8 * buf);   // the registers hold the tile: TMEM is free again
            if (!t.kind) {
                const int blk = mrow / Q36_QK;
                if (t.nrows <= 2) {   // the usual routed group at decode: a short batch publishes sooner
                    const float g0[2] = {g[0], g[1]}, u0[2] = {u[0], u[1]};
                    swiglu_quant_store<2>(g0, u0, t.nrows, (size_t)t.row0, Hq, Hs, FF, blk, lane);
                } else {
                    float g0[8], u0[8], g1[8], u1[8];
#pragma unroll
                    for (int c = 0; c < 8; c++) { g0[c] = g[c]; u0[c] = u[c]; g1[c] = g[8 + c]; u1[c] = u[8 + c]; }
                    swiglu_quant_store<8>(g0, u0, t.nrows, (size_t)t.row0, Hq, Hs, FF, blk, lane);
                    if (t.nrows > 8) swiglu_quant_store<8>(g1, u1, t.nrows - 8, (size_t)t.row0 + 8, Hq, Hs, FF, blk, lane);
                }
                // hand the tile to the publisher: the lanes' stores are ordered before lane 0 by the warp barrier,
                // lane 0's CTA-scope release orders them before the publisher's device-scope one
                __syncwarp();
                if (lane == 0) asm volatile("red.release.cta.shared.add.s32 [%0], 1;" ::"r"(smem_u32(&s_pub)) : "memory");
            } else if (ep.peers && t.row0 < ep.n_map) {
                const bool odd = ((unsigned)ep.ctl[1] + 1u) & 1u;
                const uint64_t roff = odd ? ep.ret1 : ep.ret0;
#pragma unroll
                for (int c = 0; c < 16; c++) {
                    if (c >= t.nrows) continue;
                    const int row = t.row0 + c;
                    if (row < ep.n_map) {
                        const int sl = ep.rowmap[row];
                        if (sl >= 0) {
                            const int src = sl / ep.cap, j = sl - src * ep.cap;
                            float *dst = reinterpret_cast<float *>(ep.peers[src] + roff) + ((size_t)(ep.slot_major ? src : ep.me) * ep.cap + j) * D;
                            dst[mrow] = g[c];
                        }
                    } else {
                        Y[(size_t)row * D + mrow] = g[c];
                    }
                }
            } else {
#pragma unroll
                for (int c = 0; c < 16; c++)
                    if (c < t.nrows) Y[(size_t)(t.row0 + c) * D + mrow] = g[c];
            }
        }
    } else if (warp == Cfg::W_SCHED) {
        // --------------------------------------------------------- watcher
        if (lane == 0) {
            bool all_gu_done = false;
            for (int j = 0; j < my_tiles; j++) {
                const int4 v = s_tiles[j];
                if ((v.x >> 16) && !all_gu_done) {
                    // the group's own count first (one L2 round trip when it is there, as it mostly is); the
                    // global count only when a wait was needed, to stop polling once the whole phase is over
                    int a;
                    asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(a) : "l"(plan->done + (v.x & 0xffff)) : "memory");
                    if (a < done_target_of(v.x & 0xffff)) {
                        if (!wait_group(v.x & 0xffff, 0x600)) break;
                        asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(a) : "l"(&plan->gu_done) : "memory");
                        all_gu_done = a >= n0 * Cfg::DONE_PER_GROUP_PER_MTILE;
                    }
                }
                asm volatile("st.release.cta.shared.s32 [%0], %1;" ::"r"(smem_u32(&s_ready)), "r"(all_gu_done ? my_tiles : j + 1) : "memory");
                if (all_gu_done) break;
            }
        }
    } else if (warp == Cfg::W_PUB) {
        // ------------------------------------------------------- publisher
        // gate/up tiles come first in the CTA's list, in order: tile i is done when the four epilogue warps have
        // signalled 4 (i + 1) times in all
        if (lane == 0) {
            for (int gi = 0; gi < my_gu && gi < my_tiles; gi++) {
                bool ok = false;
                for (uint32_t i = 0; i < TC_SPIN_LIMIT; i++) {
                    int v;
                    asm volatile("ld.acquire.cta.shared.s32 %0, [%1];" : "=r"(v) : "r"(smem_u32(&s_pub)) : "memory");
                    if (v >= 4 * (gi + 1)) { ok = true; break; }
                    if ((i & 255u) == 255u && abort_flag) break;
                    __nanosleep(32);
                }
                if (!ok) { if (!abort_flag) { abort_flag = 1; atomicCAS(status, 0, 0x6a0); } break; }
                const int g = s_tiles[gi].x & 0xffff;
                asm volatile("fence.acq_rel.gpu;" ::: "memory");
                atomicAdd(plan->done + g, Cfg::DONE_PER_GROUP_PER_MTILE);
                atomicAdd(&plan->gu_done, Cfg::DONE_PER_GROUP_PER_MTILE);   // once every gate/up tile is in, nobody polls per group
            }
        }
    } else {
        // --------------------------------------------------- scale loaders
        // Thread i owns row i of the tile: per K step it moves the row's 4 scale bytes from the staged plane
        // rows into the 32 x 16 B image tcgen05.cp broadcasts (row m at (m % 32) * 16 + (m / 32) * 4).
        const int i = threadIdx.x - 32 * Cfg::W_LOAD0;
        const int w4 = i >> 5, m0 = i & 31;
        const uint32_t my_off = m0 * 16 + w4 * 4;
        uint32_t it = 0;
        bool ok = true;
        for (int j = 0; j < my_tiles && ok; j++) {
            const FTile t = get_tile(j);
            const uint32_t slot = j & 1;
            const int nbk = (t.kind ? FF : D) / Q36_QK;
            const int nst = t.kind ? FF / (Cfg::KS * TC_KSTEP) : 2 * (D / (Cfg::KS * TC_KSTEP));
            if (!(ok = mbar_wait(sft_full0 + 8 * slot, (j >> 1) & 1, &abort_flag, status, 0x700 + slot))) break;
            const uint8_t *st = sft + slot * Cfg::SFT_BYTES;
            const uint8_t *ra0 = st + i * nbk, *ra1 = st + Cfg::SFT_A + i * nbk, *rb = st + 2 * Cfg::SFT_A + i * nbk;
            const bool bvalid = i < t.nrows;
            for (int q0 = 0; q0 < nst && ok; q0 += 2) {   // two stages (four K steps) per cross-proxy fence
                const uint32_t it0 = it;
#pragma unroll
                for (int qq = 0; qq < 2; qq++) {
                    const int q = q0 + qq;
                    const int kpair = t.kind ? q : (q >> 1);
                    const uint8_t *ra = (!t.kind && (q & 1)) ? ra1 : ra0;
                    const uint2 va = *reinterpret_cast<const uint2 *>(ra + 8 * kpair);       // 2 K steps x 4 scale bytes
                    const uint2 vb = bvalid ? *reinterpret_cast<const uint2 *>(rb + 8 * kpair) : make_uint2(0x7f7f7f7fu, 0x7f7f7f7fu);
                    const int s = it % Cfg::STAGES;
                    const uint32_t ph = (it / Cfg::STAGES) & 1;
                    if (!(ok = mbar_wait(empty0 + 8 * s, ph ^ 1, &abort_flag, status, 0x500 + s))) break;
                    uint8_t *sf = smem + s * Cfg::STAGE_BYTES + Cfg::OFF_SF;
                    *reinterpret_cast<uint32_t *>(sf + my_off) = va.x;
                    *reinterpret_cast<uint32_t *>(sf + Cfg::SF_BYTES + my_off) = vb.x;
                    *reinterpret_cast<uint32_t *>(sf + 2 * Cfg::SF_BYTES + my_off) = va.y;
                    *reinterpret_cast<uint32_t *>(sf + 3 * Cfg::SF_BYTES + my_off) = vb.y;
                    it++;
                }
                if (!ok) break;
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                __syncwarp();
                if (lane == 0)
                    for (uint32_t x = it0; x < it; x++) mbar_arrive(full0 + 8 * (x % Cfg::STAGES));
            }
            __syncwarp();
            if (lane == 0 && ok) mbar_arrive(sft_empty0 + 8 * slot);   // this warp is done with the staged rows
        }
    }

    // ------------------------------------------------------------ teardown
    tc_fence_before();
    __syncthreads();
    if (abort_flag) {
        for (int i = 0; i < 200; i++) __nanosleep(1000);
        if (threadIdx.x == 0) atomicCAS(status, 0, 1);
    }
    if (warp == Cfg::W_ISSUE0) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base_s), "r"(Cfg::TMEM_COLS) : "memory");
    }
    if (ep.peers && threadIdx.x == 0) {
        // every CTA orders its remote stores (the barrier above gathered the epilogue warps') with one system-scope
        // fence, then counts itself in at every source rank: a home rank's combine waits for gridDim.x arrivals
        __threadfence_system();
        const unsigned epoch = (unsigned)ep.ctl[1] + 1u;
        const bool odd = epoch & 1u;
        for (int src = 0; src < ep.world; src++) {
            unsigned *h = reinterpret_cast<unsigned *>(ep.peers[src] + (odd ? ep.rhdr1 : ep.rhdr0) + 8 * (ep.slot_major ? src : ep.me));
            asm volatile("red.relaxed.sys.global.add.u32 [%0], 1;" ::"l"(h) : "memory");
        }
        if (atomicAdd(ep.ctl + 4, 1) == (int)gridDim.x - 1) { ep.ctl[4] = 0; ep.ctl[1] = (int)epoch; }   // the last CTA ends phase 1 of this call
    }
    Q36_TR_END(status, 4)
}

// every non-empty group has at least one row and one token tile, so the row count bounds the tiles of a CTA
// Does the per-CTA tile table hold a call of R_max rows in n_group (+ 1 shared) groups?  A group of c rows is
// ceil(c / 16) token tiles, so there are at most R_max / 16 + (non-empty groups) of them.
bool ffn_fused_small_fits(int R_max, int n_group, int D, int FF) {
    using Cfg = FusedCfg;
    // the staged scale bytes of a tile are sized for K <= K_MAX; larger layers take the two grouped-GEMM launches
    if (D > Cfg::K_MAX || FF > Cfg::K_MAX || D % (4 * TC_KSTEP) || FF % (4 * TC_KSTEP)) return false;
    const long tt = R_max / Cfg::TILE_ROWS + min(R_max, n_group + 1);
    const long grid = sm_count(), n0 = tt * (FF / TC_M), n1 = tt * (D / TC_M);
    return n_group + 1 <= Cfg::MAX_GROUPS && (n0 + grid - 1) / grid + (n1 + grid - 1) / grid + Cfg::EXTRA_DOWN + 1 <= Cfg::MAX_TILES;
}

// CTAs the launch below uses for a call of these sizes
int ffn_fused_small_grid(int R_max, int n_group, int D, int FF) {
    const long max_tiles = (long)(R_max + n_group + 1) * (FF / TC_M + D / TC_M);
    return (int)min((long)sm_count(), max_tiles);
}

int launch_ffn_fused_small(const void *Wg, const void *Wu, const void *Wd, const void *Sg, const void *Su,
                           const void *Sd, int n_group, int R_max, const uint8_t *Xq, const uint8_t *Xs, uint8_t *Hq,
                           uint8_t *Hs, float *Y, int D, int FF, void *plan, int *status, const EpReturnArgs *ep, cudaStream_t st) {
    using Cfg = FusedCfg;
    if (D % (4 * TC_KSTEP) || FF % (4 * TC_KSTEP) || !ffn_fused_small_fits(R_max, n_group, D, FF)) return Q36_MOE_EINVAL;
    const uint64_t estride = (uint64_t)FF * (D / 2) + (uint64_t)FF * (D / Q36_QK);   // same for [FF][D] and [D][FF]
    const uint64_t plane = (uint64_t)FF * (D / 2);
    if (!Sg) { Sg = Wg; Su = Wu; Sd = Wd; }
    FusedMaps maps;
    int rc;
    if ((rc = make_map_codes_ksteps(&maps.g, Wg, FF, D, n_group, estride, Cfg::KS))) return rc;
    if ((rc = make_map_codes_ksteps(&maps.u, Wu, FF, D, n_group, estride, Cfg::KS))) return rc;
    if ((rc = make_map_codes_ksteps(&maps.d, Wd, D, FF, n_group, estride, Cfg::KS))) return rc;
    if ((rc = make_map_codes_ksteps(&maps.sg, Sg, FF, D, 1, estride, Cfg::KS))) return rc;
    if ((rc = make_map_codes_ksteps(&maps.su, Su, FF, D, 1, estride, Cfg::KS))) return rc;
    if ((rc = make_map_codes_ksteps(&maps.sd, Sd, D, FF, 1, estride, Cfg::KS))) return rc;
    if ((rc = make_map_rows_ksteps(&maps.x, Xq, R_max, D, 16, Cfg::KS))) return rc;
    if ((rc = make_map_rows_ksteps(&maps.h, Hq, R_max, FF, 16, Cfg::KS))) return rc;
    static bool attr_done[MAX_DEVICES] = {false};
    if ((rc = ensure_smem_attr((const void *)k_ffn_fused_small, Cfg::SMEM_BYTES, attr_done))) return rc;
    const int grid = ffn_fused_small_grid(R_max, n_group, D, FF);
    launch_k_resident(k_ffn_fused_small, dim3(grid), dim3(Cfg::THREADS), Cfg::SMEM_BYTES, st, maps, (const uint8_t *)Wg + plane,
             (const uint8_t *)Wu + plane, (const uint8_t *)Wd + plane, estride, (const uint8_t *)Sg + plane,
             (const uint8_t *)Su + plane, (const uint8_t *)Sd + plane, n_group, Xs, (TcPlan *)plan, Hq, Hs, Y, D, FF, status,
             ep ? *ep : EpReturnArgs{nullptr, 0, 0, 0, 0, nullptr, nullptr, 0, 0, 0, 0, 0});
    return check_launch();
}

}  // namespace q36
