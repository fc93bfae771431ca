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

struct FusedCfg {
    static constexpr int STAGES = 6;
    static constexpr int A_BYTES = TC_M * 128;
    static constexpr int A_TX_BYTES = TC_M * 64;     // the A box signals its packed bytes (see moe_tc.cu)
    static constexpr int B_BYTES = 16 * 128;
    static constexpr int SF_BYTES = 512;
    static constexpr int STAGE_BYTES = 2 * A_BYTES + B_BYTES + 2048;   // 36 KB, 1024-aligned
    static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 + 256;
    static constexpr int ACC_STRIDE = 32;            // TMEM columns per accumulator set: gate [0,16), up [16,32)
    static constexpr int SF_COL0 = 64;               // A0 (4), A1 (4), B (4)
    static constexpr int TMEM_COLS = 128;
    static constexpr int DONE_PER_GROUP_PER_MTILE = 4;   // epilogue warps
};

struct FusedMaps { CUtensorMap g, u, d, sg, su, sd, x, h; };

struct FTile { int kind, g, mt, row0, nrows; };

__global__ void __launch_bounds__(TC_THREADS, 1)
k_ffn_fused_small(const __grid_constant__ FusedMaps maps, const uint8_t *__restrict__ sfG, const uint8_t *__restrict__ sfU,
                  const uint8_t *__restrict__ sfD, uint64_t sf_stride, const uint8_t *__restrict__ sfSG,
                  const uint8_t *__restrict__ sfSU, const uint8_t *__restrict__ sfSD, int n_routed,
                  const uint8_t *__restrict__ Xs, TcPlan *__restrict__ plan, uint8_t *__restrict__ Hq,
                  uint8_t *__restrict__ Hs, float *__restrict__ Y, int D, int FF, int *__restrict__ status) {
    using Cfg = FusedCfg;
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem + Cfg::STAGES * Cfg::STAGE_BYTES);
    __shared__ uint32_t tmem_base_s;
    __shared__ volatile int abort_flag;
    // (16-bit where the value allows it: static + dynamic shared memory sit 1.7 KB under the 227 KB limit)
    __shared__ int s_row0[DISPATCH_MAX_GROUPS + 1], s_base0[DISPATCH_MAX_GROUPS + 2], s_base1[DISPATCH_MAX_GROUPS + 2];
    __shared__ unsigned short s_order[DISPATCH_MAX_GROUPS + 1], s_cnt[DISPATCH_MAX_GROUPS + 1];

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t full0 = smem_u32(bars), empty0 = smem_u32(bars + Cfg::STAGES);
    const uint32_t acc_full0 = smem_u32(bars + 2 * Cfg::STAGES), acc_empty0 = smem_u32(bars + 2 * Cfg::STAGES + 2);

    // ---- prologue that needs nothing from earlier kernels: runs while they drain
    if (threadIdx.x == 0) {
        abort_flag = 0;
        for (int s = 0; s < Cfg::STAGES; s++) {
            mbar_init(full0 + 8 * s, 1 + 4);
            mbar_init(empty0 + 8 * s, 1);
        }
        for (int b = 0; b < 2; b++) {
            mbar_init(acc_full0 + 8 * b, 1);
            mbar_init(acc_empty0 + 8 * b, 4);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_s)), "r"(Cfg::TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    Q36_GDS();   // from here on: global memory written by earlier kernels (the plan, Xq/Xs)

    const int G = plan->n_groups;
    const int n0 = plan->n_tiles[0], n_tiles = n0 + plan->n_tiles[1];
    const int mt_gu = FF / TC_M;
    for (int i = threadIdx.x; i <= G; i += blockDim.x) {
        s_base0[i] = plan->base[0][i];
        s_base1[i] = plan->base[1][i];
        if (i < G) { s_order[i] = (unsigned short)plan->order[i]; s_row0[i] = plan->row0[i]; s_cnt[i] = (unsigned short)plan->cnt[i]; }
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = tmem_base_s;

    auto get_tile = [&](int ti) {
        const int kind = ti >= n0;
        const int *base = kind ? s_base1 : s_base0;
        const int t = kind ? ti - n0 : ti;
        int lo = 0, hi = G - 1;
        while (lo < hi) {
            const int mid = (lo + hi + 1) >> 1;
            if (base[mid] <= t) lo = mid; else hi = mid - 1;
        }
        const int g = s_order[lo];
        return FTile{kind, g, t - base[lo], s_row0[g], s_cnt[g]};   // one token tile per group: mt = local index
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

    if (warp == 0) {
        // ---------------------------------------------------- TMA producer
        if (lane == 0) {
            uint32_t it = 0;
            bool ok = true;
            for (int ti = blockIdx.x; ti < n_tiles && ok; ti += gridDim.x) {
                const FTile t = get_tile(ti);
                const bool sh = t.g >= n_routed;
                const int ge = sh ? 0 : t.g;
                const int na = t.kind ? 1 : 2;
                const int k_steps = (t.kind ? FF : D) / TC_KSTEP;
                const CUtensorMap *ma0 = t.kind ? (sh ? &maps.sd : &maps.d) : (sh ? &maps.sg : &maps.g);
                const CUtensorMap *ma1 = sh ? &maps.su : &maps.u;
                const CUtensorMap *mb = t.kind ? &maps.h : &maps.x;
                if (t.kind) {
                    if (!(ok = wait_group(t.g, 0x600))) break;
                    asm volatile("fence.proxy.async;" ::: "memory");   // generic-proxy Hq stores before the TMA reads
                }
                const uint32_t tx = na * Cfg::A_TX_BYTES + Cfg::B_BYTES;
                for (int ks = 0; ks < k_steps; ks++, it++) {
                    const int s = it % Cfg::STAGES;
                    const uint32_t ph = (it / Cfg::STAGES) & 1;
                    if (!(ok = mbar_wait(empty0 + 8 * s, ph ^ 1, &abort_flag, status, 0x100 + s))) break;
                    const uint32_t sb = smem_u32(smem + s * Cfg::STAGE_BYTES);
                    mbar_expect_tx(full0 + 8 * s, tx);
                    tma_load_3d(sb, ma0, ks * TC_KSTEP, t.mt * TC_M, ge, full0 + 8 * s);
                    if (!t.kind) tma_load_3d(sb + Cfg::A_BYTES, ma1, ks * TC_KSTEP, t.mt * TC_M, ge, full0 + 8 * s);
                    tma_load_2d(sb + 2 * Cfg::A_BYTES, mb, ks * TC_KSTEP, t.row0, full0 + 8 * s);
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------ MMA issuer
        if (lane == 0) {
            uint32_t it = 0, tcount = 0;
            bool ok = true;
            for (int ti = blockIdx.x; ti < n_tiles && ok; ti += gridDim.x, tcount++) {
                const FTile t = get_tile(ti);
                const int k_steps = (t.kind ? FF : D) / TC_KSTEP;
                const uint32_t buf = tcount & 1;
                const uint32_t d_tmem = tmem + buf * Cfg::ACC_STRIDE;
                if (!(ok = mbar_wait(acc_empty0 + 8 * buf, ((tcount >> 1) & 1) ^ 1, &abort_flag, status, 0x200 + buf))) break;
                tc_fence_after();
                for (int ks = 0; ks < k_steps; ks++, it++) {
                    const int s = it % Cfg::STAGES;
                    const uint32_t ph = (it / Cfg::STAGES) & 1;
                    if (!(ok = mbar_wait(full0 + 8 * s, ph, &abort_flag, status, 0x300 + s))) break;
                    tc_fence_after();
                    const uint32_t sb = smem_u32(smem + s * Cfg::STAGE_BYTES);
                    const uint32_t sf = sb + 2 * Cfg::A_BYTES + Cfg::B_BYTES;
                    const uint32_t t_sfa0 = tmem + Cfg::SF_COL0, t_sfb = tmem + Cfg::SF_COL0 + 8;
                    tc_cp_sf(t_sfa0, desc_sf(sf));
                    if (!t.kind) tc_cp_sf(t_sfa0 + 4, desc_sf(sf + Cfg::SF_BYTES));
                    tc_cp_sf(t_sfb, desc_sf(sf + 2 * Cfg::SF_BYTES));
#pragma unroll
                    for (int kb = 0; kb < 4; kb++) {
                        const uint32_t acc = (ks | kb) ? 1u : 0u;
                        const uint32_t id = idesc_mx(16, kb);
                        const uint64_t bd = desc_sw128(sb + 2 * Cfg::A_BYTES + kb * 32);
                        const uint32_t sfid = (uint32_t)kb << 30;
                        tc_mma(d_tmem, desc_sw128(sb + kb * 32), bd, id, t_sfa0 | sfid, t_sfb | sfid, acc);
                        if (!t.kind)
                            tc_mma(d_tmem + 16, desc_sw128(sb + Cfg::A_BYTES + kb * 32), bd, id, (t_sfa0 + 4) | sfid, t_sfb | sfid, acc);
                    }
                    tc_commit(empty0 + 8 * s);
                }
                if (ok) tc_commit(acc_full0 + 8 * buf);
            }
        }
    } else if (warp < 6) {
        // -------------------------------------------------------- epilogue
        const int q = warp & 3;
        uint32_t tcount = 0;
        bool ok = true;
        for (int ti = blockIdx.x; ti < n_tiles && ok; ti += gridDim.x, tcount++) {
            const FTile t = get_tile(ti);
            const uint32_t buf = tcount & 1;
            const uint32_t tq = tmem + buf * Cfg::ACC_STRIDE + ((uint32_t)(q * 32) << 16);
            if (!(ok = mbar_wait(acc_full0 + 8 * buf, (tcount >> 1) & 1, &abort_flag, status, 0x400 + buf))) break;
            tc_fence_after();
            const int mrow = t.mt * TC_M + q * 32 + lane;
            uint32_t acc[32];
            tc_ld32(tq, acc);            // gate columns [0,16), up columns [16,32) (or the down tile's 16 columns)
            tc_ld_wait();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(acc_empty0 + 8 * buf);   // the registers hold the tile: TMEM is free again
            if (!t.kind) {
                const int blk = mrow / Q36_QK, nbh = FF / Q36_QK;
#pragma unroll
                for (int j = 0; j < 16; j++) {
                    if (j < t.nrows) {
                        const float h = silu_f(__uint_as_float(acc[j])) * __uint_as_float(acc[16 + j]);
                        const uint32_t am = __reduce_max_sync(0xffffffffu, __float_as_uint(fabsf(h)));
                        const int e2 = e2_of_amax(__uint_as_float(am));
                        const size_t row = (size_t)(t.row0 + j);
                        Hq[row * FF + blk * Q36_QK + hw_pos(lane)] = f32_to_e4m3(h * inv_scale_of_e2(e2));
                        if (lane == 0) Hs[row * nbh + blk] = (uint8_t)(127 + e2);
                    }
                }
                __threadfence();         // each lane's stores are visible device-wide before the count moves
                __syncwarp();
                if (lane == 0) atomicAdd(plan->done + t.g, 1);
            } else {
#pragma unroll
                for (int j = 0; j < 16; j++)
                    if (j < t.nrows) Y[(size_t)(t.row0 + j) * D + mrow] = __uint_as_float(acc[j]);
            }
        }
    } else {
        // --------------------------------------------------- scale loaders
        const int i = threadIdx.x - 6 * 32;
        const int w4 = i >> 5, m0 = i & 31;
        const uint32_t my_off = m0 * 16 + w4 * 4;
        const uint4 ones = make_uint4(0x7f7f7f7fu, 0x7f7f7f7fu, 0x7f7f7f7fu, 0x7f7f7f7fu);
        struct Item { int ti, kg; };
        // A-scales (weights) can always be fetched ahead; B-scales of a down tile only once its group is done
        auto fetch_a = [&](const FTile &t, int kg, uint4 &a0, uint4 &a1) {
            const bool sh = t.g >= n_routed;
            const int nb = (t.kind ? FF : D) / Q36_QK;
            const size_t arow = (size_t)(sh ? 0 : t.g) * sf_stride + (size_t)(t.mt * TC_M + i) * nb + 16 * kg;
            const uint8_t *p0 = t.kind ? (sh ? sfSD : sfD) : (sh ? sfSG : sfG);
            a0 = __ldg(reinterpret_cast<const uint4 *>(p0 + arow));
            a1 = ones;
            if (!t.kind) a1 = __ldg(reinterpret_cast<const uint4 *>((sh ? sfSU : sfU) + arow));
        };
        auto fetch_b = [&](const FTile &t, int kg, uint4 &b) {
            b = ones;
            if (i < t.nrows) {
                const int nb = (t.kind ? FF : D) / Q36_QK;
                const uint8_t *src = (t.kind ? Hs : Xs) + (size_t)(t.row0 + i) * nb + 16 * kg;
                // Hs was written by other SMs in this same launch: read it at L2, not through the read-only path
                b = t.kind ? __ldcg(reinterpret_cast<const uint4 *>(src)) : __ldg(reinterpret_cast<const uint4 *>(src));
            }
        };
        uint32_t it = 0;
        bool ok = true;
        int ti = blockIdx.x, kg = 0;
        uint4 a0 = ones, a1 = ones, b = ones, na0 = ones, na1 = ones, nb4 = ones;
        bool b_ready = false, nb_ready = false;
        FTile t = {0, 0, 0, 0, 0}, nt = t;
        if (ti < n_tiles) {
            t = get_tile(ti);
            fetch_a(t, kg, a0, a1);
            if (!t.kind) { fetch_b(t, kg, b); b_ready = true; }
        }
        while (ti < n_tiles && ok) {
            int nti = ti, nkg = kg + 1;
            const int groups = ((t.kind ? FF : D) / TC_KSTEP) / 4;
            if (nkg == groups) { nkg = 0; nti = ti + gridDim.x; }
            nb_ready = false;
            if (nti < n_tiles) {
                nt = (nti == ti) ? t : get_tile(nti);
                fetch_a(nt, nkg, na0, na1);
                if (!nt.kind) { fetch_b(nt, nkg, nb4); nb_ready = true; }
            }
            if (!b_ready) {   // a down tile: its group's intermediate must be complete before Hs is read
                if (!(ok = wait_group(t.g, 0x700))) break;
                fetch_b(t, kg, b);
            }
            const uint32_t wa0[4] = {a0.x, a0.y, a0.z, a0.w}, wa1[4] = {a1.x, a1.y, a1.z, a1.w}, wb[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
            for (int j = 0; j < 4; j++, it++) {
                if (!ok) break;
                const int s = it % Cfg::STAGES;
                const uint32_t ph = (it / Cfg::STAGES) & 1;
                if (!(ok = mbar_wait(empty0 + 8 * s, ph ^ 1, &abort_flag, status, 0x500 + s))) break;
                uint8_t *sf = smem + s * Cfg::STAGE_BYTES + 2 * Cfg::A_BYTES + Cfg::B_BYTES;
                *reinterpret_cast<uint32_t *>(sf + my_off) = wa0[j];
                if (!t.kind) *reinterpret_cast<uint32_t *>(sf + Cfg::SF_BYTES + my_off) = wa1[j];
                *reinterpret_cast<uint32_t *>(sf + 2 * Cfg::SF_BYTES + my_off) = wb[j];
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                __syncwarp();
                if (lane == 0) mbar_arrive(full0 + 8 * s);
            }
            a0 = na0; a1 = na1; b = nb4; b_ready = nb_ready; t = nt; ti = nti; kg = nkg;
        }
    }

    // ------------------------------------------------------------ teardown
    tc_fence_before();
    __syncthreads();
    if (abort_flag) {
        for (int i = 0; i < 200; i++) __nanosleep(1000);
        if (threadIdx.x == 0) atomicCAS(status, 0, 1);
    }
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base_s), "r"(Cfg::TMEM_COLS) : "memory");
    }
}

int launch_ffn_fused_small(const void *Wg, const void *Wu, const void *Wd, const void *Sg, const void *Su,
                           const void *Sd, int n_group, int R_max, const uint8_t *Xq, const uint8_t *Xs, uint8_t *Hq,
                           uint8_t *Hs, float *Y, int D, int FF, void *plan, int *status, cudaStream_t st) {
    using Cfg = FusedCfg;
    if (D % (4 * TC_KSTEP) || FF % (4 * TC_KSTEP) || n_group + 1 > DISPATCH_MAX_GROUPS) return Q36_MOE_EINVAL;
    const uint64_t estride = (uint64_t)FF * (D / 2) + (uint64_t)FF * (D / Q36_QK);   // same for [FF][D] and [D][FF]
    const uint64_t plane = (uint64_t)FF * (D / 2);
    if (!Sg) { Sg = Wg; Su = Wu; Sd = Wd; }
    FusedMaps maps;
    int rc;
    if ((rc = make_map_codes(&maps.g, Wg, FF, D, n_group, estride))) return rc;
    if ((rc = make_map_codes(&maps.u, Wu, FF, D, n_group, estride))) return rc;
    if ((rc = make_map_codes(&maps.d, Wd, D, FF, n_group, estride))) return rc;
    if ((rc = make_map_codes(&maps.sg, Sg, FF, D, 1, estride))) return rc;
    if ((rc = make_map_codes(&maps.su, Su, FF, D, 1, estride))) return rc;
    if ((rc = make_map_codes(&maps.sd, Sd, D, FF, 1, estride))) return rc;
    if ((rc = make_map_rows(&maps.x, Xq, R_max, D, 16))) return rc;
    if ((rc = make_map_rows(&maps.h, Hq, R_max, FF, 16))) return rc;
    static bool attr_set = false;
    if (!attr_set) {
        if (cudaFuncSetAttribute(k_ffn_fused_small, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES) != cudaSuccess)
            return check_launch();
        attr_set = true;
    }
    const long max_tiles = (long)(R_max + n_group + 1) * (FF / TC_M + D / TC_M);
    const int grid = (int)min((long)sm_count(), max_tiles);
    launch_k(k_ffn_fused_small, dim3(grid), dim3(TC_THREADS), Cfg::SMEM_BYTES, st, maps, (const uint8_t *)Wg + plane,
             (const uint8_t *)Wu + plane, (const uint8_t *)Wd + plane, estride, (const uint8_t *)Sg + plane,
             (const uint8_t *)Su + plane, (const uint8_t *)Sd + plane, n_group, Xs, (TcPlan *)plan, Hq, Hs, Y, D, FF, status);
    return check_launch();
}

}  // namespace q36
