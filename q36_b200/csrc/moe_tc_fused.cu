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

// What sets the layout (all measured on B200, see ub_tma_rate.cu and ub_mma_issue.cu):
//  * a thread needs ~140 cycles to issue ANY asynchronous copy, so a stage is TWO K steps fetched by two copies
//    (one 4-bit weight box of 2 x [128 rows][128 elements], one box of 2 x [16 token rows][128 B]);
//  * a thread gets one block-scaled MMA through per ~90-110 cycles, the pipe takes one per ~40, so FOUR warps
//    issue, each into its own accumulator columns: warps 0,1 the two K steps of the even stages, warps 2,3 of
//    the odd ones.  A gate/up tile alternates gate and up stages, hence gate = acc0 + acc1, up = acc2 + acc3; a
//    down tile (2 stages) is the sum of all four;
//  * every role looks its tile up in a table built once per CTA (a binary search per tile per role cost ~900
//    cycles, more than a down tile's share of the HBM stream);
//  * the scale bytes have their own producer thread, so the two serial issue chains run side by side.
struct FusedCfg {
    static constexpr int STAGES = 4;
    static constexpr int KS = 2;                     // K steps per stage
    static constexpr int A_BYTES = TC_M * 128;       // one K step of one matrix, 4-bit codes in 8-bit containers
    static constexpr int A_TX_BYTES = TC_M * 64;     // the A box signals its packed bytes (see moe_tc.cu)
    static constexpr int B_BYTES = 16 * 128;
    static constexpr int SF_BYTES = 512;
    static constexpr int OFF_B = KS * A_BYTES, OFF_SF = OFF_B + KS * B_BYTES;
    static constexpr int STAGE_BYTES = OFF_SF + KS * 2 * SF_BYTES;          // 38 KB, 1024-aligned
    static constexpr int STAGE_TX = KS * (A_TX_BYTES + B_BYTES);
    // Scale bytes of a whole tile (all its K steps) are staged by bulk async copies, two tiles deep: the rows
    // of a tile are contiguous in the row-major scale planes (128 rows x K/32 bytes).  Loads issued by the
    // loader threads themselves were measured to expose a full HBM latency per 4 K steps (register prefetch
    // does not help: a warp's loads retire through a handful of shared scoreboards).
    static constexpr int SFT_A = TC_M * 64;          // up to K = 2048: 64 scale bytes per row
    static constexpr int SFT_B = 16 * 64;
    static constexpr int SFT_BYTES = 2 * SFT_A + SFT_B;      // 17 KB: gate (or down), up, tokens
    static constexpr int SFT_SLOTS = 2;
    static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + SFT_SLOTS * SFT_BYTES + 1024 + 256;
    static constexpr int ISSUERS = 4;
    static constexpr int ACC_STRIDE = 64;            // per accumulator set: issuer w at [16 w, 16 w + 16)
    static constexpr int SF_COL0 = 128;              // per issuer: A (4), B (4)
    static constexpr int TMEM_COLS = 256;
    static constexpr int W_ISSUE0 = 2, W_EPI0 = W_ISSUE0 + ISSUERS, W_LOAD0 = W_EPI0 + 4;
    static constexpr int THREADS = 32 * (W_LOAD0 + 4);   // weight producer, scale producer, issuers, epilogue, scale loaders
    static constexpr int DONE_PER_GROUP_PER_MTILE = 4;   // epilogue warps
    static constexpr int MAX_GROUPS = DISPATCH_MAX_GROUPS + 1;   // the plan lists every group, empty ones included
    static constexpr int MAX_TILES = 32;                 // per CTA
};
static_assert(FusedCfg::STAGE_BYTES % 1024 == 0, "stage alignment");

struct FusedMaps { CUtensorMap g, u, d, sg, su, sd, x, h; };

struct FTile { int kind, g, mt, row0, nrows; };

__global__ void __launch_bounds__(FusedCfg::THREADS, 1)
k_ffn_fused_small(const __grid_constant__ FusedMaps maps, const uint8_t *__restrict__ sfG, const uint8_t *__restrict__ sfU,
                  const uint8_t *__restrict__ sfD, uint64_t sf_stride, const uint8_t *__restrict__ sfSG,
                  const uint8_t *__restrict__ sfSU, const uint8_t *__restrict__ sfSD, int n_routed,
                  const uint8_t *__restrict__ Xs, TcPlan *__restrict__ plan, uint8_t *__restrict__ Hq,
                  uint8_t *__restrict__ Hs, float *__restrict__ Y, int D, int FF, int *__restrict__ status) {
    using Cfg = FusedCfg;
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t *sft = smem + Cfg::STAGES * Cfg::STAGE_BYTES;
    uint64_t *bars = reinterpret_cast<uint64_t *>(sft + Cfg::SFT_SLOTS * Cfg::SFT_BYTES);
    __shared__ uint32_t tmem_base_s;
    __shared__ volatile int abort_flag;
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
        for (int s = 0; s < Cfg::STAGES; s++) {
            mbar_init(full0 + 8 * s, 1 + 4);              // the producer's expect_tx arrive + one per scale warp
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
    if (warp == Cfg::W_ISSUE0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_s)), "r"(Cfg::TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    Q36_GDS();   // from here on: global memory written by earlier kernels (the plan, Xq/Xs)

    const int G = plan->n_groups;
    const int n0 = plan->n_tiles[0], n_tiles = n0 + plan->n_tiles[1];
    const int mt_gu = FF / TC_M;
    int my_tiles = blockIdx.x < n_tiles ? (n_tiles - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;
    const bool fits = G <= Cfg::MAX_GROUPS && my_tiles <= Cfg::MAX_TILES;
    if (!fits) {                                   // (uniform over the CTA) nothing is computed, the status says so
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
    if ((int)threadIdx.x < my_tiles) {             // this CTA's tiles: blockIdx.x, blockIdx.x + gridDim.x, ...
        const int ti = blockIdx.x + threadIdx.x * gridDim.x;
        const int kind = ti >= n0;
        const int *base = kind ? s_base1 : s_base0;
        const int t = kind ? ti - n0 : ti;
        int lo = 0, hi = G - 1;
        while (lo < hi) {
            const int mid = (lo + hi + 1) >> 1;
            if (base[mid] <= t) lo = mid; else hi = mid - 1;
        }
        const int g = s_order[lo];
        s_tiles[threadIdx.x] = make_int4(g | (kind << 16), t - base[lo], s_row0[g], s_cnt[g]);   // one token tile per group
    }
    __syncthreads();
    auto get_tile = [&](int j) {
        const int4 v = s_tiles[j];
        return FTile{v.x >> 16, v.x & 0xffff, v.y, v.z, v.w};
    };
    // gate/up of group g is complete when every epilogue warp of each of its row tiles has published
    const int done_target = mt_gu * Cfg::DONE_PER_GROUP_PER_MTILE;
    auto wait_group = [&](int g, int where) -> bool {
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
    // A down tile reads Hq/Hs written through the generic proxy, possibly by other SMs: wait for the group's
    // count, then order those writes before this thread's asynchronous reads.
    auto wait_inputs = [&](const FTile &t, bool &all_gu_done, int where) -> bool {
        if (!t.kind || all_gu_done) return true;
        if (!wait_group(t.g, where)) return false;
        int v;   // after the wait (acquire): if the whole gate/up phase is over, later tiles need no poll
        asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(&plan->gu_done) : "memory");
        all_gu_done = v >= n0 * Cfg::DONE_PER_GROUP_PER_MTILE;
        asm volatile("fence.proxy.async.global;" ::: "memory");   // (the all-spaces form costs ~1000 cycles here, this one ~20)
        return true;
    };

    if (warp == 0) {
        // ------------------------------------------- TMA producer: weights and token rows
        if (lane == 0) {
            uint32_t it = 0;
            bool ok = true, all_gu_done = false;
            for (int j = 0; j < my_tiles && ok; j++) {
                const FTile t = get_tile(j);
                const bool sh = t.g >= n_routed;
                const int ge = sh ? 0 : t.g;
                const CUtensorMap *ma0 = t.kind ? (sh ? &maps.sd : &maps.d) : (sh ? &maps.sg : &maps.g);
                const CUtensorMap *ma1 = sh ? &maps.su : &maps.u;
                const CUtensorMap *mb = t.kind ? &maps.h : &maps.x;
                if (!(ok = wait_inputs(t, all_gu_done, 0x600))) break;
                const int nst = t.kind ? FF / (Cfg::KS * TC_KSTEP) : 2 * (D / (Cfg::KS * TC_KSTEP));   // gate, up, gate, ...
                for (int q = 0; q < nst; q++, it++) {
                    const int kpair = t.kind ? q : (q >> 1);
                    const int s = it % Cfg::STAGES;
                    const uint32_t ph = (it / Cfg::STAGES) & 1;
                    if (!(ok = mbar_wait(empty0 + 8 * s, ph ^ 1, &abort_flag, status, 0x100 + s))) break;
                    const uint32_t sb = smem_u32(smem + s * Cfg::STAGE_BYTES);
                    mbar_expect_tx(full0 + 8 * s, Cfg::STAGE_TX);
                    tma_load_4d(sb, (!t.kind && (q & 1)) ? ma1 : ma0, 0, t.mt * TC_M, kpair * Cfg::KS, ge, full0 + 8 * s);
                    tma_load_3d(sb + Cfg::OFF_B, mb, 0, t.row0, kpair * Cfg::KS, full0 + 8 * s);
                }
            }
        }
    } else if (warp == 1) {
        // --------------------------- scale producer: a tile's scale bytes, contiguous runs of the row-major planes
        if (lane == 0) {
            bool ok = true, all_gu_done = false;
            for (int j = 0; j < my_tiles && ok; j++) {
                const FTile t = get_tile(j);
                const bool sh = t.g >= n_routed;
                const int ge = sh ? 0 : t.g;
                const uint32_t slot = j & 1;
                if (!(ok = wait_inputs(t, all_gu_done, 0x680))) break;
                if (!(ok = mbar_wait(sft_empty0 + 8 * slot, ((j >> 1) & 1) ^ 1, &abort_flag, status, 0x800 + slot))) break;
                const int nbk = (t.kind ? FF : D) / Q36_QK;
                const uint32_t a_bytes = TC_M * nbk, b_bytes = t.nrows * nbk;
                const size_t arow = (size_t)ge * sf_stride + (size_t)(t.mt * TC_M) * nbk;
                const uint8_t *p0 = t.kind ? (sh ? sfSD : sfD) : (sh ? sfSG : sfG);
                const uint32_t dst = smem_u32(sft + slot * Cfg::SFT_BYTES);
                mbar_expect_tx(sft_full0 + 8 * slot, a_bytes * (t.kind ? 1 : 2) + b_bytes);
                bulk_load(dst, p0 + arow, a_bytes, sft_full0 + 8 * slot);
                if (!t.kind) bulk_load(dst + Cfg::SFT_A, (sh ? sfSU : sfU) + arow, a_bytes, sft_full0 + 8 * slot);
                bulk_load(dst + 2 * Cfg::SFT_A, (t.kind ? Hs : Xs) + (size_t)t.row0 * nbk, b_bytes, sft_full0 + 8 * slot);
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
                {
                    float g0[8], u0[8], g1[8], u1[8];
#pragma unroll
                    for (int c = 0; c < 8; c++) { g0[c] = g[c]; u0[c] = u[c]; g1[c] = g[8 + c]; u1[c] = u[8 + c]; }
                    swiglu_quant_store<8>(g0, u0, t.nrows, (size_t)t.row0, Hq, Hs, FF, blk, lane);
                    if (t.nrows > 8) swiglu_quant_store<8>(g1, u1, t.nrows - 8, (size_t)t.row0 + 8, Hq, Hs, FF, blk, lane);
                }
                __threadfence();         // each lane's stores are visible device-wide before the count moves
                __syncwarp();
                if (lane == 0) {
                    atomicAdd(plan->done + t.g, 1);
                    atomicAdd(&plan->gu_done, 1);      // once every gate/up tile is in, consumers stop polling per group
                }
            } else {
#pragma unroll
                for (int c = 0; c < 16; c++)
                    if (c < t.nrows) Y[(size_t)(t.row0 + c) * D + mrow] = g[c];
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
}

// every non-empty group has at least one row and one token tile, so the row count bounds the tiles of a CTA
int ffn_fused_small_max_rows(int D, int FF) { return FusedCfg::MAX_TILES * sm_count() / (FF / TC_M + D / TC_M); }

int launch_ffn_fused_small(const void *Wg, const void *Wu, const void *Wd, const void *Sg, const void *Su,
                           const void *Sd, int n_group, int R_max, const uint8_t *Xq, const uint8_t *Xs, uint8_t *Hq,
                           uint8_t *Hs, float *Y, int D, int FF, void *plan, int *status, cudaStream_t st) {
    using Cfg = FusedCfg;
    if (D % (4 * TC_KSTEP) || FF % (4 * TC_KSTEP) || n_group + 1 > Cfg::MAX_GROUPS || R_max > ffn_fused_small_max_rows(D, FF)) return Q36_MOE_EINVAL;
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
    static bool attr_set = false;
    if (!attr_set) {
        if (cudaFuncSetAttribute(k_ffn_fused_small, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES) != cudaSuccess)
            return check_launch();
        attr_set = true;
    }
    const long max_tiles = (long)(R_max + n_group + 1) * (FF / TC_M + D / TC_M);
    const int grid = (int)min((long)sm_count(), max_tiles);
    launch_k(k_ffn_fused_small, dim3(grid), dim3(Cfg::THREADS), Cfg::SMEM_BYTES, st, maps, (const uint8_t *)Wg + plane,
             (const uint8_t *)Wu + plane, (const uint8_t *)Wd + plane, estride, (const uint8_t *)Sg + plane,
             (const uint8_t *)Su + plane, (const uint8_t *)Sd + plane, n_group, Xs, (TcPlan *)plan, Hq, Hs, Y, D, FF, status);
    return check_launch();
}

}  // namespace q36
