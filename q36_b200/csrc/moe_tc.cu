// Prefill-sized expert groups: grouped GEMMs on the 5th-generation tensor cores
// (tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale, accumulators in TMEM).
//
// Replaces k_gemm_expert_mma (q36_engine.cu:2435-2524; mma.sync m16n8k32
// block-scaled, an sm_120a-only instruction) for gate/up and k_gemm_expert_tc
// (:2723-2766) for an MXFP4 down projection.
//
// Kernels
//   k_gateup_wide     gate/up + SwiGLU + requantise: 128 token rows (E4M3) as the 128-row operand against the
//                     128 gate + 128 up rows of an ff tile as one N = 256 operand (E2M1)
//   k_grouped_mma<2>  the same with weights as the 128-row operand and up to 112 tokens as N (selectable)
//   k_down_resident   down for FF = 512: a token tile's rows stay in shared memory, weight-row tiles stream past
//   k_grouped_mma<1>  down for other shapes
// Operand staging
//   weights  TMA, CU_TENSOR_MAP_DATA_TYPE_16U4_ALIGN16B: the packed code plane (K/2 bytes per row, GGUF nibble
//            order) is expanded on the fly into the padded form the tensor core reads (16 codes in 8 B + 8 B
//            gap), 128 B of shared memory per row per 128 K-elements, 128B swizzle.
//   tokens   TMA, UINT8, boxes of token rows x 128 B, 128B swizzle.  Rows are in "hw order" inside each 32-block,
//            so that position p of a token row meets nibble p of a weight row.
//   scales   the E8M0 bytes arrive by TMA from the row-major scale planes (items of four K steps); four warps put
//            them into TMEM as the image the MMA reads: row m at lane m % 32, column m / 32, byte kb, once per
//            lane quarter -- by tcgen05.st, or through a 32 x 16 B shared-memory image and tcgen05.cp.32x128b.warpx4.
// One persistent CTA per SM walks a tile table built on the device (largest groups first); every role is a warp
// (or four) of its own.  Every mbarrier wait is bounded; a wait that gives up raises a status word that the host
// entry point reports as Q36_MOE_EDEVICE.  -DQ36_TCPROF adds clock64 sums per role, printed by a few CTAs.
#include <cuda.h>
#include <stdlib.h>

#include "common.cuh"
#include "kernels.cuh"
#include "tc_plan.cuh"
#include <cstdio>
#include "tc_ptx.cuh"

namespace q36 {

// ------------------------------------------------------------ configuration
// NA = 2: gate/up (two A operands, SwiGLU + E4M3 requantisation epilogue), token tile 112
// NA = 1: down (one A operand, f32 rows out), token tile 128
// The token tile of gate/up is 112 so that TWO accumulator sets (gate + up each) and the scale
// columns fit the 512 TMEM columns: the epilogue of one tile overlaps the MMAs of the next.
//
// Measured on B200 and built in:
//  * one thread gets a block-scaled MMA (M = 128, K = 32) through every ~90 cycles for any N <= 128 (N = 128
//    would need 64); two issuing warps reach the pipe rate.  Gate/up has two issuers, one per matrix.
//  * scale bytes fetched by the loader threads themselves (ld.global, even prefetched in registers) exposed a
//    full HBM latency every four K steps and set the pace of the whole kernel.  They now arrive by TMA: a
//    ring of items (four K steps: 16 scale bytes per row, boxes of 16 B x 128 rows), issued by the producer
//    with the operand tiles; the loader warps only reshuffle shared memory.
template <int NA>
struct TcCfg {
    static constexpr int N = (NA == 2) ? TC_N_GATEUP : TC_N_DOWN;   // token rows per tile (max UMMA N)
    static constexpr int ISSUERS = NA;
    static constexpr int STAGES = (NA == 2) ? 4 : 6;
    static constexpr int A_BYTES = TC_M * 128;               // 16 KB of shared memory per A operand per stage
    // What the A box signals on the mbarrier: the PACKED bytes read from global memory (64 B per row), not
    // the 128 B per row it occupies after expansion.  Measured on B200: expecting 16 KB leaves the barrier
    // pending for ever, expecting 8 KB completes it.
    static constexpr int A_TX_BYTES = TC_M * 64;
    static constexpr int B_BYTES = N * 128;                  // 14 KB or 16 KB
    static constexpr int SF_BYTES = 512;                     // one 32 x 16 B scale image
    // operand tiles are 128B-swizzled: every stage starts on a 1024-byte boundary
    static constexpr int STAGE_BYTES = NA * A_BYTES + B_BYTES + ((NA + 1) * SF_BYTES + 1023) / 1024 * 1024;
    static constexpr int SFR_SLOTS = 4;                      // ring of scale items
    static constexpr int SFR_PART = 128 * 16;                // 128 rows x 16 B
    static constexpr int SFR_BYTES = (NA + 1) * SFR_PART;
    static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + SFR_SLOTS * SFR_BYTES + 1024 /* alignment */ + 512 /* barriers */;
    static constexpr int ACC_STRIDE = (NA == 2) ? 256 : 128; // TMEM columns between the two accumulator sets
    // scale columns of stage s: one 4-column image per A operand, then the token rows' (gate/up: the columns the two
    // accumulator sets of 2 x 112 leave free in each half of the 512)
    static constexpr int SF_COLS = 4 * (NA + 1);
    __host__ __device__ static constexpr int sf_col(int s) { return (NA == 2) ? ((s < 2 ? 224 : 456) + SF_COLS * s) : 256 + SF_COLS * s; }
    static constexpr int TMEM_COLS = 512;
    static constexpr int B_FULL_MIN = 49;                    // token tiles of at least this many rows use one big box
    // Warps: 0 weight producer, 1 token-row + scale-item producer, 2..3 MMA issuers (3 idle for NA = 1), 4..7 scale
    // loaders, 8.. epilogue: every role group is a whole, aligned group of four warps so that the gate/up kernel can
    // move registers from the first eight warps to its epilogue warps (setmaxnreg works on such groups).
    static constexpr int EPI_WARP0 = 8;
    static constexpr int EPI_WARPS = (NA == 2) ? 16 : 8;     // EPI_WARPS / 4 per TMEM lane quarter, taking 16-column batches in turn
    static constexpr int THREADS = 32 * (EPI_WARP0 + EPI_WARPS);
    static constexpr bool REBALANCE = (NA == 2);             // 768 threads x 80 registers at launch -> 256 x 40 + 512 x 96
    static constexpr int REGS_LOW = 40, REGS_EPI = 96;
};

// ------------------------------------------------------------- tile plan
__global__ void __launch_bounds__(512)
k_tc_plan(const int *__restrict__ goffs, int n_group, const int *__restrict__ soffs, TcPlan *plan, int mt_gu,
          int mt_dn, int *status, int tile_rows) {
    Q36_GDS();
    __shared__ int scratch[4 * (DISPATCH_MAX_GROUPS + 1)];
    (void)status;   // (the status words are sticky: only q36_moe_ws_reset clears them)
    tc_plan_block(goffs, n_group, soffs != nullptr, soffs ? soffs[0] : 0, soffs ? soffs[1] : 0, plan, mt_gu, mt_dn, scratch, true, tile_rows);
}

// The give-up path of the bounded waits on its own: one warp waits on an mbarrier phase that nothing ever
// completes, with a limit of 1024 polls instead of 2^22, records `where` in the status word like every role of
// the grouped-GEMM kernels does, and returns.  Lets a test see Q36_MOE_EDEVICE reported with the context intact.
__global__ void k_wait_timeout(int *status) {
    Q36_GDS();
    __shared__ uint64_t bar;
    __shared__ volatile int abort_flag;
    if (threadIdx.x == 0) {
        abort_flag = 0;
        mbar_init(smem_u32(&bar), 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    if (threadIdx.x == 0) mbar_wait(smem_u32(&bar), 0, &abort_flag, status, 0xA00, 1024u);
    __syncthreads();
}
int launch_wait_timeout(int *status, cudaStream_t st) {
    launch_k(k_wait_timeout, dim3(1), dim3(32), 0, st, status);
    return check_launch();
}

// ------------------------------------------------------------ main kernel
struct TcMaps { CUtensorMap a0, a1, s0, s1, b16, bfull, fa0, fa1, fs0, fs1, fb; };

template <int NA>
__global__ void __launch_bounds__(TcCfg<NA>::THREADS, 1)
k_grouped_mma(const __grid_constant__ TcMaps maps, int n_routed, const TcPlan *__restrict__ plan,
              uint8_t *__restrict__ Hq, uint8_t *__restrict__ Hs, float *__restrict__ Y, int M_total, int K,
              int *__restrict__ status, int y_bf16) {
    using Cfg = TcCfg<NA>;
    constexpr int W = (NA == 2) ? 0 : 1;
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t *sfr = smem + Cfg::STAGES * Cfg::STAGE_BYTES;
    uint64_t *bars = reinterpret_cast<uint64_t *>(sfr + Cfg::SFR_SLOTS * Cfg::SFR_BYTES);
    // bars: full[STAGES], empty[STAGES], acc_full[2], acc_empty[2], sfr_full[SLOTS], sfr_empty[SLOTS]
    __shared__ uint32_t tmem_base_s;
    __shared__ volatile int abort_flag;
    __shared__ int s_row0[DISPATCH_MAX_GROUPS + 1], s_cnt[DISPATCH_MAX_GROUPS + 1], s_base[DISPATCH_MAX_GROUPS + 2];
    __shared__ unsigned short s_order[DISPATCH_MAX_GROUPS + 1];

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t full0 = smem_u32(bars), empty0 = smem_u32(bars + Cfg::STAGES);
    const uint32_t acc_full0 = smem_u32(bars + 2 * Cfg::STAGES), acc_empty0 = acc_full0 + 16;
    const uint32_t sfr_full0 = acc_empty0 + 16, sfr_empty0 = sfr_full0 + 8 * Cfg::SFR_SLOTS;

    // ---- prologue that needs nothing from earlier kernels
    if (threadIdx.x == 0) {
        abort_flag = 0;
        for (int s = 0; s < Cfg::STAGES; s++) {
            mbar_init(full0 + 8 * s, 2 + 4);               // each producer's expect_tx arrive + one arrive per scale warp
            mbar_init(empty0 + 8 * s, Cfg::ISSUERS);       // one tcgen05.commit per issuing warp
        }
        for (int b = 0; b < 2; b++) {
            mbar_init(acc_full0 + 8 * b, Cfg::ISSUERS);
            mbar_init(acc_empty0 + 8 * b, Cfg::EPI_WARPS); // one arrive per epilogue warp
        }
        for (int b = 0; b < Cfg::SFR_SLOTS; b++) {
            mbar_init(sfr_full0 + 8 * b, 1);
            mbar_init(sfr_empty0 + 8 * b, 4);              // one arrive per scale warp
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 2) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_s)), "r"(Cfg::TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    Q36_GDS();   // from here on: global memory written by earlier kernels

    const int n_tiles = plan->n_tiles[W];
    const int G = plan->n_groups;
    const int k_steps = K / TC_KSTEP;
    const int m_tiles = M_total / TC_M;
    for (int i = threadIdx.x; i <= G; i += blockDim.x) {
        s_base[i] = plan->base[W][i];
        if (i < G) { s_order[i] = (unsigned short)plan->order[i]; s_row0[i] = plan->row0[i]; s_cnt[i] = plan->cnt[i]; }
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = tmem_base_s;

    // tile index -> work item: rank by binary search over the tile prefix sums, row tile fastest
    auto get_tile = [&](int ti) {
        int lo = 0, hi = G - 1;
        while (lo < hi) {
            const int mid = (lo + hi + 1) >> 1;
            if (s_base[mid] <= ti) lo = mid; else hi = mid - 1;
        }
        const int g = s_order[lo], local = ti - s_base[lo];
        const int nt = local / m_tiles, mt = local - nt * m_tiles;
        return TcTile{g, mt, s_row0[g] + nt * Cfg::N, min(Cfg::N, s_cnt[g] - nt * Cfg::N)};
    };

    if (warp < Cfg::EPI_WARP0) {
        if (Cfg::REBALANCE) asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(Cfg::REGS_LOW));
        if (warp == 0) {
            // ------------------------------------------- TMA producer: weights
            // (One thread needs ~140 cycles to issue a copy whatever its size, ~300 with the wait and the expect_tx: all
            // of a K step's copies from one thread took longer than the step's MMAs.  Two threads share them.)
            if (lane == 0) {
                uint32_t it = 0;
                bool ok = true;
                for (int ti = blockIdx.x; ti < n_tiles && ok; ti += gridDim.x) {
                    const TcTile t = get_tile(ti);
                    const bool sh = t.g >= n_routed;
                    const CUtensorMap *ma0 = sh ? &maps.s0 : &maps.a0, *ma1 = sh ? &maps.s1 : &maps.a1;
                    const int ge = sh ? 0 : t.g;
                    for (int ks = 0; ks < k_steps; ks++, it++) {
                        const int s = it % Cfg::STAGES;
                        const uint32_t ph = (it / Cfg::STAGES) & 1;
                        if (!(ok = mbar_wait(empty0 + 8 * s, ph ^ 1, &abort_flag, status, 0x100 + s, TC_SPIN_LIMIT, TC_BACKOFF_NS))) break;
                        const uint32_t sb = smem_u32(smem + s * Cfg::STAGE_BYTES);
                        mbar_expect_tx(full0 + 8 * s, NA * Cfg::A_TX_BYTES);
                        tma_load_3d(sb, ma0, ks * TC_KSTEP, t.mt * TC_M, ge, full0 + 8 * s);
                        if (NA == 2) tma_load_3d(sb + Cfg::A_BYTES, ma1, ks * TC_KSTEP, t.mt * TC_M, ge, full0 + 8 * s);
                    }
                }
            }
        } else if (warp == 1) {
            // --------------------------- TMA producer: token rows and scale items
            if (lane == 0) {
                uint32_t it = 0, item = 0;
                bool ok = true;
                for (int ti = blockIdx.x; ti < n_tiles && ok; ti += gridDim.x) {
                    const TcTile t = get_tile(ti);
                    const bool sh = t.g >= n_routed;
                    const CUtensorMap *fa0 = sh ? &maps.fs0 : &maps.fa0, *fa1 = sh ? &maps.fs1 : &maps.fa1;
                    const int ge = sh ? 0 : t.g;
                    const bool full_box = t.nrows >= Cfg::B_FULL_MIN;
                    const int slabs = (t.nrows + 15) / 16;
                    const uint32_t tx = full_box ? Cfg::N * 128 : slabs * 2048;
                    for (int ks = 0; ks < k_steps; ks++, it++) {
                        if ((ks & 3) == 0) {   // the scale bytes of the next four K steps
                            const uint32_t sl = item % Cfg::SFR_SLOTS;
                            if (!(ok = mbar_wait(sfr_empty0 + 8 * sl, ((item / Cfg::SFR_SLOTS) & 1) ^ 1, &abort_flag, status, 0x800 + sl, TC_SPIN_LIMIT, TC_BACKOFF_NS))) break;
                            const uint32_t dst = smem_u32(sfr + sl * Cfg::SFR_BYTES);
                            mbar_expect_tx(sfr_full0 + 8 * sl, NA * Cfg::SFR_PART + Cfg::N * 16);
                            tma_load_3d(dst, fa0, 4 * ks, t.mt * TC_M, ge, sfr_full0 + 8 * sl);
                            if (NA == 2) tma_load_3d(dst + Cfg::SFR_PART, fa1, 4 * ks, t.mt * TC_M, ge, sfr_full0 + 8 * sl);
                            tma_load_2d(dst + NA * Cfg::SFR_PART, &maps.fb, 4 * ks, t.row0, sfr_full0 + 8 * sl);
                            item++;
                        }
                        const int s = it % Cfg::STAGES;
                        const uint32_t ph = (it / Cfg::STAGES) & 1;
                        if (!(ok = mbar_wait(empty0 + 8 * s, ph ^ 1, &abort_flag, status, 0x900 + s, TC_SPIN_LIMIT, TC_BACKOFF_NS))) break;
                        const uint32_t sb = smem_u32(smem + s * Cfg::STAGE_BYTES);
                        mbar_expect_tx(full0 + 8 * s, tx);
                        if (full_box) {
                            tma_load_2d(sb + NA * Cfg::A_BYTES, &maps.bfull, ks * TC_KSTEP, t.row0, full0 + 8 * s);
                        } else {
                            for (int i = 0; i < slabs; i++)
                                tma_load_2d(sb + NA * Cfg::A_BYTES + i * 2048, &maps.b16, ks * TC_KSTEP, t.row0 + 16 * i, full0 + 8 * s);
                        }
                    }
                }
            }
        } else if (warp < 4) {
            // ----------------------------------------------------- MMA issuers
            // NA = 2: issuer 0 drives the gate matrix, issuer 1 the up matrix of the SAME stage.  The scale images are in
            // TMEM already when the stage is full: the loader warps store them there (tcgen05.st), so that no
            // tcgen05.cp sits between the MMAs in the tensor pipe (four of them cost as much as the eight MMAs of a K step).
            if (lane == 0 && warp - 2 < Cfg::ISSUERS) {
                const int w = warp - 2;
                uint32_t it = 0, tcount = 0;
                bool ok = true;
#ifdef Q36_TCPROF
                long long pf_full = 0, pf_acc = 0, pf_t0 = clock64();
#endif
                for (int ti = blockIdx.x; ti < n_tiles && ok; ti += gridDim.x, tcount++) {
                    const TcTile t = get_tile(ti);
                    const int n_mma = (t.nrows >= Cfg::B_FULL_MIN) ? Cfg::N : max(16, (t.nrows + 15) & ~15);
                    const uint32_t buf = tcount & 1;
                    const uint32_t d_tmem = tmem + buf * Cfg::ACC_STRIDE + w * Cfg::N;
                    // this accumulator set must have been drained by the epilogue two tiles ago
#ifdef Q36_TCPROF
                    long long pf_a = clock64();
#endif
                    if (!(ok = mbar_wait(acc_empty0 + 8 * buf, ((tcount >> 1) & 1) ^ 1, &abort_flag, status, 0x200 + buf))) break;
#ifdef Q36_TCPROF
                    pf_acc += clock64() - pf_a;
#endif
                    tc_fence_after();
                    for (int ks = 0; ks < k_steps; ks++, it++) {
                        const int s = it % Cfg::STAGES;
                        const uint32_t ph = (it / Cfg::STAGES) & 1;
#ifdef Q36_TCPROF
                        long long pf_b = clock64();
#endif
                        if (!(ok = mbar_wait(full0 + 8 * s, ph, &abort_flag, status, 0x300 + s))) break;
#ifdef Q36_TCPROF
                        pf_full += clock64() - pf_b;
#endif
                        tc_fence_after();
                        const uint32_t sb = smem_u32(smem + s * Cfg::STAGE_BYTES);
                        const uint32_t t_sfa = tmem + Cfg::sf_col(s) + 4 * w, t_sfb = tmem + Cfg::sf_col(s) + 4 * NA;
    #pragma unroll
                        for (int kb = 0; kb < 4; kb++) {
                            const uint32_t sfid = (uint32_t)kb << 30;
                            tc_mma(d_tmem, desc_sw128(sb + w * Cfg::A_BYTES + kb * 32), desc_sw128(sb + NA * Cfg::A_BYTES + kb * 32),
                                   idesc_mx(n_mma, kb), t_sfa | sfid, t_sfb | sfid, (ks | kb) ? 1u : 0u);
                        }
                        tc_commit(empty0 + 8 * s);   // stage reusable once every issuer's MMAs have read it
                    }
                    if (ok) tc_commit(acc_full0 + 8 * buf);
                }
#ifdef Q36_TCPROF
                if (NA == 2 && w == 0 && (blockIdx.x == 0 || blockIdx.x == 77))
                    printf("issuer cta %d: tiles %u total %lld wait_full %lld wait_acc %lld\n", blockIdx.x, tcount, clock64() - pf_t0, pf_full, pf_acc);
#endif
            }
        } else {
            // --------------------------------------------------- scale loaders (warps 4..7)
            // The scale image of an operand for one K step is 32 lanes x 4 columns in each TMEM lane quarter: lane l,
            // column j, byte kb = scale of row l + 32 * j for K block kb -- one aligned word of the row's 16 staged
            // bytes.  Each of the four warps writes the image into its own lane quarter (the four copies the MMA
            // reads), lane = thread: four rows' words per operand per K step, straight from the staged item.
            const int q = warp & 3;
            uint32_t it = 0, item = 0;
            bool ok = true;
            for (int ti = blockIdx.x; ti < n_tiles && ok; ti += gridDim.x) {
                const TcTile t = get_tile(ti);
                for (int kg = 0; kg < k_steps / 4 && ok; kg++, item++) {
                    const uint32_t sl = item % Cfg::SFR_SLOTS;
                    if (!(ok = mbar_wait(sfr_full0 + 8 * sl, (item / Cfg::SFR_SLOTS) & 1, &abort_flag, status, 0x700 + sl, TC_SPIN_LIMIT, TC_BACKOFF_NS))) break;
                    const uint8_t *src = sfr + sl * Cfg::SFR_BYTES + lane * 16;
                    // rows beyond the tile's: scale 1.0 instead of stale bytes (a 0xff byte would be a NaN)
                    bool bval[4];
    #pragma unroll
                    for (int j = 0; j < 4; j++) bval[j] = lane + 32 * j < t.nrows;
    #pragma unroll
                    for (int x = 0; x < 4; x++) {                 // K step x of the item: word x of the rows l + 32 j
                        uint32_t wa0[4], wa1[4], wb[4];
    #pragma unroll
                        for (int j = 0; j < 4; j++) {
                            wa0[j] = *reinterpret_cast<const uint32_t *>(src + j * 512 + 4 * x);
                            wa1[j] = (NA == 2) ? *reinterpret_cast<const uint32_t *>(src + Cfg::SFR_PART + j * 512 + 4 * x) : 0u;
                            wb[j] = bval[j] ? *reinterpret_cast<const uint32_t *>(src + NA * Cfg::SFR_PART + j * 512 + 4 * x) : 0x7f7f7f7fu;
                        }
                        const int s = it % Cfg::STAGES;
                        const uint32_t ph = (it / Cfg::STAGES) & 1;
                        if (!(ok = mbar_wait(empty0 + 8 * s, ph ^ 1, &abort_flag, status, 0x500 + s, TC_SPIN_LIMIT, TC_BACKOFF_NS))) break;
                        tc_fence_after();
                        const uint32_t tq = tmem + Cfg::sf_col(s) + ((uint32_t)(q * 32) << 16);
                        tc_st4(tq, wa0[0], wa0[1], wa0[2], wa0[3]);
                        if (NA == 2) tc_st4(tq + 4, wa1[0], wa1[1], wa1[2], wa1[3]);
                        tc_st4(tq + 4 * NA, wb[0], wb[1], wb[2], wb[3]);
                        tc_st_wait();
                        tc_fence_before();
                        __syncwarp();
                        if (lane == 0) mbar_arrive(full0 + 8 * s);
                        it++;
                    }
                    if (!ok) break;
                    __syncwarp();
                    if (lane == 0) mbar_arrive(sfr_empty0 + 8 * sl);
                }
            }
        }
    } else {
        if (Cfg::REBALANCE) asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(Cfg::REGS_EPI));
        // -------------------------------------------------------- epilogue
        const int q = warp & 3;                  // TMEM lane quarter this warp may read
        constexpr int SUBS = Cfg::EPI_WARPS / 4; // warps per quarter
        const int sub = (warp - Cfg::EPI_WARP0) >> 2;
        uint32_t tcount = 0;
        bool ok = true;
#ifdef Q36_TCPROF
        long long pf_wait = 0, pf_busy = 0;
#endif
        for (int ti = blockIdx.x; ti < n_tiles && ok; ti += gridDim.x, tcount++) {
            const TcTile t = get_tile(ti);
            const uint32_t buf = tcount & 1;
            const uint32_t tq = tmem + buf * Cfg::ACC_STRIDE + ((uint32_t)(q * 32) << 16);
#ifdef Q36_TCPROF
            long long pf_a = clock64();
#endif
            if (!(ok = mbar_wait(acc_full0 + 8 * buf, (tcount >> 1) & 1, &abort_flag, status, 0x400 + buf, TC_SPIN_LIMIT, TC_BACKOFF_NS))) break;
#ifdef Q36_TCPROF
            long long pf_b = clock64();
            pf_wait += pf_b - pf_a;
#endif
            tc_fence_after();
            const int mrow = t.mt * TC_M + q * 32 + lane;   // weight row (output feature) of this thread
            if (NA == 2) {
                const int blk = mrow / Q36_QK;               // this warp's 32 rows are one scale block
                for (int c0 = 16 * sub; c0 < t.nrows; c0 += 16 * SUBS) {   // sixteen token columns per batch
                    uint32_t g[16], u[16];
                    tc_ld16(tq + c0, g);
                    tc_ld16(tq + Cfg::N + c0, u);
                    tc_ld_wait();
                    float gg[16], uu[16];
#pragma unroll
                    for (int c = 0; c < 16; c++) { gg[c] = __uint_as_float(g[c]); uu[c] = __uint_as_float(u[c]); }
                    swiglu_quant_store<16>(gg, uu, t.nrows - c0, (size_t)(t.row0 + c0), Hq, Hs, M_total, blk, lane);
                }
            } else {
                for (int c0 = 32 * sub; c0 < t.nrows; c0 += 32 * SUBS) {
                    uint32_t g[32];
                    tc_ld32(tq + c0, g);
                    tc_ld_wait();
#pragma unroll
                    for (int j = 0; j < 32; j++)
                        if (c0 + j < t.nrows) st_y(Y, (size_t)(t.row0 + c0 + j) * M_total + mrow, __uint_as_float(g[j]), y_bf16);
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(acc_empty0 + 8 * buf);
#ifdef Q36_TCPROF
            pf_busy += clock64() - pf_b;
#endif
        }
#ifdef Q36_TCPROF
        if (NA == 2 && lane == 0 && (warp == Cfg::EPI_WARP0 || warp == Cfg::EPI_WARP0 + 13) && (blockIdx.x == 0 || blockIdx.x == 77))
            printf("epilogue cta %d warp %d: tiles %u wait %lld busy %lld\n", blockIdx.x, warp, tcount, pf_wait, pf_busy);
#endif
    }

    // ------------------------------------------------------------ teardown
    tc_fence_before();
    __syncthreads();
    if (abort_flag) {
        // leave copies that may still be in flight time to land before the block retires
        for (int i = 0; i < 200; i++) __nanosleep(1000);
        if (threadIdx.x == 0) atomicCAS(status, 0, 1);
    }
    if (warp == 2) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(Cfg::TMEM_COLS) : "memory");
    }
}

// ------------------------------------------- gate/up, tokens as the 128-row operand
// k_grouped_mma<2> keeps weights as the 128-row operand and tokens as N <= 112: eight MMAs per K step from two
// threads, each of which gets one through per ~160 cycles among the epilogue warps of its scheduler (measured: the
// issuing threads, not the tensor pipe, set the pace).  Here a tile is 128 TOKEN rows (the M operand, E4M3) against
// the 128 gate rows + 128 up rows of one ff tile as ONE N = 256 operand (E2M1): four MMAs per K step from one
// thread, each 128 cycles of tensor pipe, so one thread issues at the pipe's rate.  An accumulator lane is a
// token and its columns are ff rows: the 32 values of a token's scale block sit in ONE thread of the epilogue (no
// cross-lane maximum, one exponent per thread, two 16-byte stores).  The 256 accumulator columns exist once; the
// epilogue warps release them as soon as they hold the values in registers, so their arithmetic overlaps the next
// tile's MMAs.
struct GuWide {
    static constexpr int N = 128;                       // token rows per tile (UMMA M)
    static constexpr int STAGES = 4;
    static constexpr int A_BYTES = N * 128;             // token rows of one K step
    static constexpr int B_HALF = TC_M * 128;           // gate (or up) rows of one K step, padded 4-bit form
    static constexpr int B_TX = TC_M * 64;              // ... and what its copy signals (packed bytes)
    static constexpr int STAGE_BYTES = A_BYTES + 2 * B_HALF;              // 48 KB
    static constexpr int SFR_SLOTS = 4, SFR_PART = 128 * 16, SFR_BYTES = 3 * SFR_PART;   // tokens | gate | up, four K steps each
    static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + SFR_SLOTS * SFR_BYTES + 1024 + 512;
    static constexpr int ACC_COLS = 256, SF_COLS = 12, TMEM_COLS = 512;   // scale columns of stage s: tokens 4 | gate 4 | up 4
    __host__ __device__ static constexpr int sf_col(int s) { return ACC_COLS + SF_COLS * s; }
    static constexpr int B_FULL_MIN = 49;               // token tiles of at least this many rows use one 128-row box
    static constexpr int EPI_WARP0 = 8, EPI_WARPS = 16, THREADS = 32 * (EPI_WARP0 + EPI_WARPS);
    static constexpr int REGS_LOW = 32, REGS_EPI = 104;
};

// instruction descriptor of that MMA: A = E4M3 (0), B = E2M1 (5), both K-major, UE8M0 scales, M = 128, N = 256
__device__ __forceinline__ uint32_t idesc_mx_wide(int kb) {
    return ((uint32_t)kb << 4) | (0u << 7) | (5u << 10) | ((uint32_t)(256 >> 3) << 17) | (1u << 23) |
           ((uint32_t)(128 >> 4) << 24) | ((uint32_t)kb << 29);
}

__global__ void __launch_bounds__(GuWide::THREADS, 1)
k_gateup_wide(const __grid_constant__ TcMaps maps, int n_routed, const TcPlan *__restrict__ plan, uint8_t *__restrict__ Hq,
              uint8_t *__restrict__ Hs, int FF, int K, int *__restrict__ status) {
    using C = GuWide;
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t *sfr = smem + C::STAGES * C::STAGE_BYTES;
    uint64_t *bars = reinterpret_cast<uint64_t *>(sfr + C::SFR_SLOTS * C::SFR_BYTES);
    // bars: full[STAGES], empty[STAGES], acc_full, acc_empty, sfr_full[SLOTS], sfr_empty[SLOTS]
    __shared__ uint32_t tmem_base_s;
    __shared__ volatile int abort_flag;
    __shared__ int s_row0[DISPATCH_MAX_GROUPS + 1], s_cnt[DISPATCH_MAX_GROUPS + 1], s_base[DISPATCH_MAX_GROUPS + 2];
    __shared__ unsigned short s_order[DISPATCH_MAX_GROUPS + 1];

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t full0 = smem_u32(bars), empty0 = smem_u32(bars + C::STAGES);
    const uint32_t acc_full = smem_u32(bars + 2 * C::STAGES), acc_empty = acc_full + 8;
    const uint32_t sfr_full0 = acc_empty + 8, sfr_empty0 = sfr_full0 + 8 * C::SFR_SLOTS;

    if (threadIdx.x == 0) {
        abort_flag = 0;
        for (int s = 0; s < C::STAGES; s++) {
            mbar_init(full0 + 8 * s, 2 + 4);      // each producer's expect_tx arrive + one arrive per scale warp
            mbar_init(empty0 + 8 * s, 1);         // the issuer's tcgen05.commit
        }
        mbar_init(acc_full, 1);
        mbar_init(acc_empty, C::EPI_WARPS);
        for (int b = 0; b < C::SFR_SLOTS; b++) {
            mbar_init(sfr_full0 + 8 * b, 1);
            mbar_init(sfr_empty0 + 8 * b, 4);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 2) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_s)), "r"(C::TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    Q36_GDS();   // from here on: global memory written by earlier kernels

    const int n_tiles = plan->n_tiles[0];
    const int G = plan->n_groups;
    const int k_steps = K / TC_KSTEP;
    const int m_tiles = FF / TC_M;
    const bool plan_ok = plan->tile_rows == C::N;      // the plan must have been cut in 128-row token tiles
    for (int i = threadIdx.x; i <= G; i += blockDim.x) {
        s_base[i] = plan->base[0][i];
        if (i < G) { s_order[i] = (unsigned short)plan->order[i]; s_row0[i] = plan->row0[i]; s_cnt[i] = plan->cnt[i]; }
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = tmem_base_s;
    if (!plan_ok && threadIdx.x == 0) atomicCAS(status, 0, 0xE00);
    const int my_first = plan_ok ? (int)blockIdx.x : n_tiles;

    auto get_tile = [&](int ti) {
        int lo = 0, hi = G - 1;
        while (lo < hi) {
            const int mid = (lo + hi + 1) >> 1;
            if (s_base[mid] <= ti) lo = mid; else hi = mid - 1;
        }
        const int g = s_order[lo], local = ti - s_base[lo];
        const int nt = local / m_tiles, mt = local - nt * m_tiles;
        return TcTile{g, mt, s_row0[g] + nt * C::N, min(C::N, s_cnt[g] - nt * C::N)};
    };

    if (warp < C::EPI_WARP0) {
        asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(C::REGS_LOW));
        if (warp == 0) {
            // ---------------------------------------- TMA producer: weights (gate rows, then up rows of the ff tile)
            // One thread needs ~360 cycles per copy (wait, expect_tx, issue) whatever its size: two copies per K step from
            // one thread are slower than the step's MMAs (512 cycles).  Lanes 0 and 1 issue the gate and the up copy in
            // the same instruction.
            if (lane < 2) {
                uint32_t it = 0;
                bool ok = true;
#ifdef Q36_TCPROF
                long long pf_w = 0, pf_x, pf_t0 = clock64();
#endif
                const uint64_t w_policy = l2_policy_evict_first();
                for (int ti = my_first; ti < n_tiles && ok; ti += gridDim.x) {
                    const TcTile t = get_tile(ti);
                    const bool sh = t.g >= n_routed;
                    const CUtensorMap *mm = sh ? (lane ? &maps.s1 : &maps.s0) : (lane ? &maps.a1 : &maps.a0);
                    const int ge = sh ? 0 : t.g;
                    const bool once = s_cnt[t.g] <= C::N;      // a group of one token tile: its weights are read once
                    for (int ks = 0; ks < k_steps; ks++, it++) {
                        const int s = it % C::STAGES;
#ifdef Q36_TCPROF
                        pf_x = clock64();
#endif
                        if (!(ok = mbar_wait(empty0 + 8 * s, ((it / C::STAGES) & 1) ^ 1, &abort_flag, status, 0x100 + s, TC_SPIN_LIMIT, TC_BACKOFF_NS))) break;
#ifdef Q36_TCPROF
                        pf_w += clock64() - pf_x;
#endif
                        const uint32_t sb = smem_u32(smem + s * C::STAGE_BYTES) + C::A_BYTES + lane * C::B_HALF;
                        if (lane == 0) mbar_expect_tx(full0 + 8 * s, 2 * C::B_TX);
                        __syncwarp(3u);                      // the expected bytes are registered before either copy can complete
                        if (once) tma_load_3d_hint(sb, mm, ks * TC_KSTEP, t.mt * TC_M, ge, full0 + 8 * s, w_policy);
                        else tma_load_3d(sb, mm, ks * TC_KSTEP, t.mt * TC_M, ge, full0 + 8 * s);
                    }
                }
#ifdef Q36_TCPROF
                if (lane == 0 && (blockIdx.x == 0 || blockIdx.x == 77)) printf("wide prodA cta %d: total %lld wait_empty %lld\n", blockIdx.x, clock64() - pf_t0, pf_w);
#endif
            }
        } else if (warp == 1) {
            // ---------------------------------------- TMA producer: token rows
            if (lane == 0) {
                uint32_t it = 0;
                bool ok = true;
                for (int ti = my_first; ti < n_tiles && ok; ti += gridDim.x) {
                    const TcTile t = get_tile(ti);
                    const bool full_box = t.nrows >= C::B_FULL_MIN;
                    const int slabs = (t.nrows + 15) / 16;
                    const uint32_t tx = full_box ? C::A_BYTES : slabs * 2048;
                    for (int ks = 0; ks < k_steps; ks++, it++) {
                        const int s = it % C::STAGES;
                        if (!(ok = mbar_wait(empty0 + 8 * s, ((it / C::STAGES) & 1) ^ 1, &abort_flag, status, 0x900 + s, TC_SPIN_LIMIT, TC_BACKOFF_NS))) break;
                        const uint32_t sb = smem_u32(smem + s * C::STAGE_BYTES);
                        mbar_expect_tx(full0 + 8 * s, tx);
                        if (full_box) {
                            tma_load_2d(sb, &maps.bfull, ks * TC_KSTEP, t.row0, full0 + 8 * s);
                        } else {
                            for (int i = 0; i < slabs; i++) tma_load_2d(sb + i * 2048, &maps.b16, ks * TC_KSTEP, t.row0 + 16 * i, full0 + 8 * s);
                        }
                    }
                }
            }
        } else if (warp == 3) {
            // ---------------------------------------- TMA producer: scale items (four K steps each), as far ahead as
            // their ring allows -- issued with the stage copies they arrived one latency late every fourth K step
            if (lane == 0) {
                uint32_t item = 0;
                bool ok = true;
                for (int ti = my_first; ti < n_tiles && ok; ti += gridDim.x) {
                    const TcTile t = get_tile(ti);
                    const bool sh = t.g >= n_routed;
                    const CUtensorMap *fg = sh ? &maps.fs0 : &maps.fa0, *fu = sh ? &maps.fs1 : &maps.fa1;
                    const int ge = sh ? 0 : t.g;
                    for (int ks = 0; ks < k_steps; ks += 4, item++) {
                        const uint32_t sl = item % C::SFR_SLOTS;
                        if (!(ok = mbar_wait(sfr_empty0 + 8 * sl, ((item / C::SFR_SLOTS) & 1) ^ 1, &abort_flag, status, 0x800 + sl, TC_SPIN_LIMIT, TC_BACKOFF_NS))) break;
                        const uint32_t dst = smem_u32(sfr + sl * C::SFR_BYTES);
                        mbar_expect_tx(sfr_full0 + 8 * sl, 3 * C::SFR_PART);
                        tma_load_2d(dst, &maps.fb, 4 * ks, t.row0, sfr_full0 + 8 * sl);
                        tma_load_3d(dst + C::SFR_PART, fg, 4 * ks, t.mt * TC_M, ge, sfr_full0 + 8 * sl);
                        tma_load_3d(dst + 2 * C::SFR_PART, fu, 4 * ks, t.mt * TC_M, ge, sfr_full0 + 8 * sl);
                    }
                }
            }
        } else if (warp == 2) {
            // ---------------------------------------- the MMA issuer
            if (lane == 0) {
                uint32_t it = 0, tcount = 0;
                bool ok = true;
#ifdef Q36_TCPROF
                long long pf_full = 0, pf_acc = 0, pf_t0 = clock64(), pf_x;
#endif
                for (int ti = my_first; ti < n_tiles && ok; ti += gridDim.x, tcount++) {
                    // the accumulator must have been read out by every epilogue warp
#ifdef Q36_TCPROF
                    pf_x = clock64();
#endif
                    if (!(ok = mbar_wait(acc_empty, (tcount & 1) ^ 1, &abort_flag, status, 0x200))) break;
#ifdef Q36_TCPROF
                    pf_acc += clock64() - pf_x;
#endif
                    tc_fence_after();
                    for (int ks = 0; ks < k_steps; ks++, it++) {
                        const int s = it % C::STAGES;
#ifdef Q36_TCPROF
                        pf_x = clock64();
#endif
                        if (!(ok = mbar_wait(full0 + 8 * s, (it / C::STAGES) & 1, &abort_flag, status, 0x300 + s))) break;
#ifdef Q36_TCPROF
                        pf_full += clock64() - pf_x;
#endif
                        tc_fence_after();
                        const uint32_t sb = smem_u32(smem + s * C::STAGE_BYTES);
                        const uint32_t t_sfa = tmem + C::sf_col(s), t_sfb = t_sfa + 4;
#pragma unroll
                        for (int kb = 0; kb < 4; kb++) {
                            const uint32_t sfid = (uint32_t)kb << 30;
                            tc_mma(tmem, desc_sw128(sb + kb * 32), desc_sw128(sb + C::A_BYTES + kb * 32), idesc_mx_wide(kb),
                                   t_sfa | sfid, t_sfb | sfid, (ks | kb) ? 1u : 0u);
                        }
                        tc_commit(empty0 + 8 * s);
                    }
                    if (ok) tc_commit(acc_full);
                }
#ifdef Q36_TCPROF
                if (blockIdx.x == 0 || blockIdx.x == 77 || blockIdx.x == 147)
                    printf("wide issuer cta %d: tiles %u total %lld wait_full %lld wait_acc %lld\n", blockIdx.x, tcount, clock64() - pf_t0, pf_full, pf_acc);
#endif
            }
        } else if (warp >= 4) {
            // ---------------------------------------- scale loaders: lane l writes the words of rows l + 32 j
            const int q = warp & 3;
            uint32_t it = 0, item = 0;
            bool ok = true;
#ifdef Q36_TCPROF
            long long pf_w = 0, pf_i = 0, pf_x, pf_t0 = clock64();
#endif
            for (int ti = my_first; ti < n_tiles && ok; ti += gridDim.x) {
                for (int kg = 0; kg < k_steps / 4 && ok; kg++, item++) {
                    const uint32_t sl = item % C::SFR_SLOTS;
#ifdef Q36_TCPROF
                    pf_x = clock64();
#endif
                    if (!(ok = mbar_wait(sfr_full0 + 8 * sl, (item / C::SFR_SLOTS) & 1, &abort_flag, status, 0x700 + sl, TC_SPIN_LIMIT, TC_BACKOFF_NS))) break;
#ifdef Q36_TCPROF
                    pf_i += clock64() - pf_x;
#endif
                    const uint8_t *src = sfr + sl * C::SFR_BYTES + lane * 16;
#pragma unroll
                    for (int x = 0; x < 4; x++) {
                        uint32_t wt[4], wg[4], wu[4];
#pragma unroll
                        for (int j = 0; j < 4; j++) {
                            wt[j] = *reinterpret_cast<const uint32_t *>(src + j * 512 + 4 * x);
                            wg[j] = *reinterpret_cast<const uint32_t *>(src + C::SFR_PART + j * 512 + 4 * x);
                            wu[j] = *reinterpret_cast<const uint32_t *>(src + 2 * C::SFR_PART + j * 512 + 4 * x);
                        }
                        const int s = it % C::STAGES;
#ifdef Q36_TCPROF
                        pf_x = clock64();
#endif
                        if (!(ok = mbar_wait(empty0 + 8 * s, ((it / C::STAGES) & 1) ^ 1, &abort_flag, status, 0x500 + s, TC_SPIN_LIMIT, TC_BACKOFF_NS))) break;
#ifdef Q36_TCPROF
                        pf_w += clock64() - pf_x;
#endif
                        tc_fence_after();
                        const uint32_t tq = tmem + C::sf_col(s) + ((uint32_t)(q * 32) << 16);
                        tc_st4(tq, wt[0], wt[1], wt[2], wt[3]);
                        tc_st4(tq + 4, wg[0], wg[1], wg[2], wg[3]);
                        tc_st4(tq + 8, wu[0], wu[1], wu[2], wu[3]);
                        tc_st_wait();
                        tc_fence_before();
                        __syncwarp();
                        if (lane == 0) mbar_arrive(full0 + 8 * s);
                        it++;
                    }
                    if (!ok) break;
                    __syncwarp();
                    if (lane == 0) mbar_arrive(sfr_empty0 + 8 * sl);
                }
            }
#ifdef Q36_TCPROF
            if (lane == 0 && warp == 4 && (blockIdx.x == 0 || blockIdx.x == 77))
                printf("wide loader cta %d: total %lld wait_empty %lld wait_item %lld\n", blockIdx.x, clock64() - pf_t0, pf_w, pf_i);
#endif
        }
    } else {
        asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(C::REGS_EPI));
        // -------------------------------------------- epilogue: warp (q, sub) = tokens 32 q .. + 31, scale block `sub` of the ff tile
        const int q = warp & 3, sub = (warp - C::EPI_WARP0) >> 2;
        const int nbh = FF / Q36_QK;
        uint32_t tcount = 0;
        bool ok = true;
        for (int ti = my_first; ti < n_tiles && ok; ti += gridDim.x, tcount++) {
            const TcTile t = get_tile(ti);
            if (!(ok = mbar_wait(acc_full, tcount & 1, &abort_flag, status, 0x400, TC_SPIN_LIMIT, TC_BACKOFF_NS))) break;
            tc_fence_after();
            const bool mine = q * 32 < t.nrows;          // warp-uniform: this lane quarter holds rows of the tile
            uint32_t g[32], u[32];
            if (mine) {
                const uint32_t tq = tmem + ((uint32_t)(q * 32) << 16);
                tc_ld32(tq + 32 * sub, g);
                tc_ld32(tq + 128 + 32 * sub, u);
                tc_ld_wait();
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(acc_empty);       // the next tile's MMAs may overwrite the columns now
            if (mine) {
                float h[32];
                float amax = 0.f;
#pragma unroll
                for (int c = 0; c < 32; c++) {
                    const float gv = __uint_as_float(g[c]);
                    h[c] = __fdividef(gv, 1.f + __expf(-gv)) * __uint_as_float(u[c]);
                    amax = fmaxf(amax, fabsf(h[c]));
                }
                const int e2 = e2_of_amax(amax);
                const float inv = inv_scale_of_e2(e2);
                uint32_t w[8];                            // hw order: byte 2 j <- element j, byte 2 j + 1 <- element j + 16
#pragma unroll
                for (int x = 0; x < 8; x++) {
                    const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(h[2 * x] * inv, h[2 * x + 16] * inv), __NV_SATFINITE, __NV_E4M3);
                    const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(h[2 * x + 1] * inv, h[2 * x + 17] * inv), __NV_SATFINITE, __NV_E4M3);
                    w[x] = lo | (hi << 16);
                }
                const int row = q * 32 + lane;
                if (row < t.nrows) {
                    const size_t r = (size_t)(t.row0 + row);
                    const int blk = t.mt * (TC_M / Q36_QK) + sub;
                    uint4 *dst = reinterpret_cast<uint4 *>(Hq + r * FF + (size_t)blk * Q36_QK);
                    dst[0] = make_uint4(w[0], w[1], w[2], w[3]);
                    dst[1] = make_uint4(w[4], w[5], w[6], w[7]);
                    Hs[r * nbh + blk] = (uint8_t)(127 + e2);
                }
            }
        }
    }

    // ------------------------------------------------------------ teardown
    tc_fence_before();
    __syncthreads();
    if (abort_flag) {
        for (int i = 0; i < 200; i++) __nanosleep(1000);   // copies that may still be in flight
        if (threadIdx.x == 0) atomicCAS(status, 0, 1);
    }
    if (warp == 2) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(C::TMEM_COLS) : "memory");
    }
}

// ----------------------------------------------- down projection, token tile resident
// The down projection of prefill-sized groups has K = FF = 512: a token tile's whole B operand (128 rows x 512 B
// = 64 KB) fits in shared memory.  k_grouped_mma<1> re-fetches it for every one of the D / 128 weight-row tiles
// (64 KB of tokens against 32 KB of weights per tile) from one producer thread and issues from one thread (N = 128
// needs an MMA per 64 cycles, one thread manages one per ~92).  Here a work item is (group, token tile, chunk of
// DR_MC consecutive weight-row tiles): the token rows and their scale images are loaded once per item and stay,
// weights stream through a ring of two-K-step stages (one 4-D copy each), two warps issue alternate row tiles into
// their own accumulators (which is also what lets the epilogue of one tile overlap the MMAs of the next), and the
// weight copies, the token copies and the scale images each have their own thread(s).
struct DownRes {
    static constexpr int N = TC_N_DOWN;                 // token rows per item
    static constexpr int KSTEPS = 4;                    // K = 512 in steps of 128
    static constexpr int KS = 2;                        // K steps per weight stage
    static constexpr int STAGES = 4;
    static constexpr int A_BYTES = TC_M * 128;          // one K step of weights in shared memory (padded 4-bit)
    static constexpr int A_TX = TC_M * 64;              // ... and what the copy signals (packed bytes)
    static constexpr int SF_BYTES = 512;
    static constexpr int STAGE_BYTES = KS * A_BYTES + KS * SF_BYTES + 1024 - KS * SF_BYTES;   // 33 KB: [A k0][A k1][SFA k0][SFA k1][pad]
    static constexpr int B_STEP = N * 128;              // one K step of the token tile
    static constexpr int B_BYTES = KSTEPS * B_STEP;     // 64 KB
    static constexpr int BIMG_BYTES = KSTEPS * SF_BYTES;   // token scale images, one per K step
    static constexpr int SFR_SLOTS = 2, SFR_BYTES = TC_M * 16;   // staged weight scale bytes of a row tile: 128 rows x 16 B
    static constexpr int BS_BYTES = N * 16;             // staged token scale bytes of an item
    static constexpr int OFF_B = STAGES * STAGE_BYTES, OFF_BIMG = OFF_B + B_BYTES, OFF_SFR = OFF_BIMG + BIMG_BYTES,
                         OFF_BS = OFF_SFR + SFR_SLOTS * SFR_BYTES, OFF_BARS = OFF_BS + BS_BYTES;
    static constexpr int SMEM_BYTES = OFF_BARS + 512 + 1024;
    static constexpr int W_PROD_A = 0, W_PROD_B = 1, W_ISSUE0 = 2, W_EPI0 = 4, EPI_WARPS = 16, W_LOAD0 = W_EPI0 + EPI_WARPS;
    static constexpr int THREADS = 32 * (W_LOAD0 + 4);
    static constexpr int ACC_BUFS = 3, ACC_STRIDE = 128, SF_COL0 = ACC_BUFS * ACC_STRIDE, TMEM_COLS = 512;
};
static_assert(DownRes::STAGE_BYTES % 1024 == 0 && DownRes::OFF_B % 1024 == 0, "swizzled tiles start on 1024-byte boundaries");
constexpr int DR_MC_MIN = 8;   // weight-row tiles per work item: 16 when the row tiles of a token tile divide by it (the token rows are
                            // then fetched once per token tile), else 8

struct DownMaps { CUtensorMap a, s, b, fa, fs, fb; };   // routed / shared code planes (2 K steps per box), token rows, scale planes

template <int YBF>      // result rows stored as bf16 (a compile-time choice: the store loop is what paces this kernel)
__global__ void __launch_bounds__(DownRes::THREADS, 1)
k_down_resident(const __grid_constant__ DownMaps maps, int n_routed, const TcPlan *__restrict__ plan, float *__restrict__ Y,
                int M_total, int *__restrict__ status, int DR_MC) {
    constexpr int y_bf16 = YBF;
    using C = DownRes;
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem + C::OFF_BARS);
    __shared__ uint32_t tmem_base_s;
    __shared__ volatile int abort_flag;
    __shared__ int s_row0[DISPATCH_MAX_GROUPS + 1], s_cnt[DISPATCH_MAX_GROUPS + 1], s_base[DISPATCH_MAX_GROUPS + 2];
    __shared__ unsigned short s_order[DISPATCH_MAX_GROUPS + 1];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // barriers: full[4] empty[4] | sfr_full[2] sfr_empty[2] | bq_full[4] | bimg_full b_empty bs_full bs_empty | acc_full[3] acc_empty[3]
    const uint32_t full0 = smem_u32(bars), empty0 = full0 + 8 * C::STAGES, sfr_full0 = empty0 + 8 * C::STAGES,
                   sfr_empty0 = sfr_full0 + 8 * C::SFR_SLOTS, bq_full0 = sfr_empty0 + 8 * C::SFR_SLOTS,
                   bimg_full = bq_full0 + 8 * C::KSTEPS, b_empty = bimg_full + 8, bs_full = b_empty + 8, bs_empty = bs_full + 8,
                   acc_full0 = bs_empty + 8, acc_empty0 = acc_full0 + 8 * C::ACC_BUFS;
    if (threadIdx.x == 0) {
        abort_flag = 0;
        for (int i = 0; i < C::STAGES; i++) { mbar_init(full0 + 8 * i, 1 + 4); mbar_init(empty0 + 8 * i, 1); }
        for (int i = 0; i < C::SFR_SLOTS; i++) { mbar_init(sfr_full0 + 8 * i, 1); mbar_init(sfr_empty0 + 8 * i, 4); }
        for (int i = 0; i < C::KSTEPS; i++) mbar_init(bq_full0 + 8 * i, 1);
        mbar_init(bimg_full, 4); mbar_init(b_empty, 2); mbar_init(bs_full, 1); mbar_init(bs_empty, 4);
        for (int i = 0; i < C::ACC_BUFS; i++) { mbar_init(acc_full0 + 8 * i, 1); mbar_init(acc_empty0 + 8 * i, C::EPI_WARPS); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == C::W_ISSUE0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_s)), "r"(C::TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    Q36_GDS();
    const int G = plan->n_groups, m_tiles = M_total / TC_M;
    const int n_items = plan->n_tiles[1] / DR_MC;          // every group's tile count is a multiple of m_tiles, and m_tiles of DR_MC
    for (int i = threadIdx.x; i <= G; i += blockDim.x) {
        s_base[i] = plan->base[1][i];
        if (i < G) { s_order[i] = (unsigned short)plan->order[i]; s_row0[i] = plan->row0[i]; s_cnt[i] = plan->cnt[i]; }
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = tmem_base_s;
    // item -> (group, first weight-row tile of its chunk, first token row, token rows)
    auto get_item = [&](int ii) {
        const int ti = ii * DR_MC;
        int lo = 0, hi = G - 1;
        while (lo < hi) {
            const int mid = (lo + hi + 1) >> 1;
            if (s_base[mid] <= ti) lo = mid; else hi = mid - 1;
        }
        const int g = s_order[lo], local = ti - s_base[lo];
        const int nt = local / m_tiles, mt = local - nt * m_tiles;
        return TcTile{g, mt, s_row0[g] + nt * C::N, min(C::N, s_cnt[g] - nt * C::N)};
    };

    if (warp == C::W_PROD_A) {
        // ------------------------------ weights: per row tile its scale bytes (one box) and two 2-K-step code boxes
        if (lane == 0) {
            uint32_t q = 0;
            bool ok = true;
            const uint64_t w_policy = l2_policy_evict_first();
            for (int ii = blockIdx.x; ii < n_items && ok; ii += gridDim.x) {
                const TcTile t = get_item(ii);
                const bool sh = t.g >= n_routed;
                const CUtensorMap *ma = sh ? &maps.s : &maps.a, *mf = sh ? &maps.fs : &maps.fa;
                const int ge = sh ? 0 : t.g;
                const bool once = s_cnt[t.g] <= C::N;      // a group of one token tile: its weights are read once (evict-first in L2)
                for (int j = 0; j < DR_MC && ok; j++, q++) {
                    const int mrow0 = (t.mt + j) * TC_M;
                    const uint32_t sl = q % C::SFR_SLOTS;
                    if (!(ok = mbar_wait(sfr_empty0 + 8 * sl, ((q / C::SFR_SLOTS) & 1) ^ 1, &abort_flag, status, 0x800 + sl, TC_SPIN_LIMIT, TC_BACKOFF_NS))) break;
                    mbar_expect_tx(sfr_full0 + 8 * sl, C::SFR_BYTES);
                    tma_load_3d(smem_u32(smem + C::OFF_SFR + sl * C::SFR_BYTES), mf, 0, mrow0, ge, sfr_full0 + 8 * sl);
                    for (int h = 0; h < C::KSTEPS / C::KS; h++) {
                        const uint32_t it = q * (C::KSTEPS / C::KS) + h, s = it % C::STAGES;
                        if (!(ok = mbar_wait(empty0 + 8 * s, ((it / C::STAGES) & 1) ^ 1, &abort_flag, status, 0x100 + s, TC_SPIN_LIMIT, TC_BACKOFF_NS))) break;
                        mbar_expect_tx(full0 + 8 * s, C::KS * C::A_TX);
                        if (once) tma_load_4d_hint(smem_u32(smem + s * C::STAGE_BYTES), ma, 0, mrow0, h * C::KS, ge, full0 + 8 * s, w_policy);
                        else tma_load_4d(smem_u32(smem + s * C::STAGE_BYTES), ma, 0, mrow0, h * C::KS, ge, full0 + 8 * s);
                    }
                }
            }
        }
    } else if (warp == C::W_PROD_B) {
        // ------------------------------ token rows of the item (one box per K step) and their scale bytes
        if (lane == 0) {
            uint32_t n = 0;
            bool ok = true;
            for (int ii = blockIdx.x; ii < n_items && ok; ii += gridDim.x, n++) {
                const TcTile t = get_item(ii);
                // the scale bytes first (their staging is free as soon as the loader warps have read the previous item's):
                // the images can then be written the moment the issuers let go of the previous item
                if (!(ok = mbar_wait(bs_empty, (n & 1) ^ 1, &abort_flag, status, 0x190, TC_SPIN_LIMIT, TC_BACKOFF_NS))) break;
                mbar_expect_tx(bs_full, C::BS_BYTES);
                tma_load_2d(smem_u32(smem + C::OFF_BS), &maps.fb, 0, t.row0, bs_full);
                if (!(ok = mbar_wait(b_empty, (n & 1) ^ 1, &abort_flag, status, 0x180, TC_SPIN_LIMIT, TC_BACKOFF_NS))) break;      // both issuers are done with the previous item's rows
                for (int ks = 0; ks < C::KSTEPS; ks++) {
                    mbar_expect_tx(bq_full0 + 8 * ks, C::B_STEP);
                    tma_load_2d(smem_u32(smem + C::OFF_B + ks * C::B_STEP), &maps.b, ks * TC_KSTEP, t.row0, bq_full0 + 8 * ks);
                }
            }
        }
    } else if (warp < C::W_EPI0) {
        // ------------------------------ MMA issuers: warp w takes the row tiles with sequence number q = w (mod 2)
        if (lane == 0) {
            const uint32_t w = warp - C::W_ISSUE0;
            const uint32_t t_sfa = tmem + C::SF_COL0 + 8 * w, t_sfb = t_sfa + 4;
            uint32_t n = 0;
            bool ok = true;
#ifdef Q36_TCPROF
            long long pf_full = 0, pf_acc = 0, pf_b = 0, pf_x, pf_t0 = clock64();
#endif
            for (int ii = blockIdx.x; ii < n_items && ok; ii += gridDim.x, n++) {
                const TcTile t = get_item(ii);
                const int n_mma = max(16, (t.nrows + 15) & ~15);
                bool first = true;
                for (int j = 0; j < DR_MC && ok; j++) {
                    const uint32_t q = n * DR_MC + j;
                    if ((q & 1u) != w) continue;
                    // accumulator q % 3: a third buffer lets the issuers run a row tile ahead of the epilogue, which is
                    // the slower side (64 KB of f32 rows to store per row tile)
                    const uint32_t buf = q % C::ACC_BUFS, use = q / C::ACC_BUFS;
                    const uint32_t d_tmem = tmem + buf * C::ACC_STRIDE;
#ifdef Q36_TCPROF
                    pf_x = clock64();
#endif
                    if (!(ok = mbar_wait(acc_empty0 + 8 * buf, (use & 1) ^ 1, &abort_flag, status, 0x200 + buf))) break;
#ifdef Q36_TCPROF
                    pf_acc += clock64() - pf_x; pf_x = clock64();
#endif
                    if (first) {                                   // the item's token scale images
                        if (!(ok = mbar_wait(bimg_full, n & 1, &abort_flag, status, 0x210))) break;
                    }
#ifdef Q36_TCPROF
                    pf_b += clock64() - pf_x;
#endif
                    tc_fence_after();
                    for (int h = 0; h < C::KSTEPS / C::KS && ok; h++) {
                        const uint32_t it = q * (C::KSTEPS / C::KS) + h, s = it % C::STAGES;
#ifdef Q36_TCPROF
                        pf_x = clock64();
#endif
                        if (!(ok = mbar_wait(full0 + 8 * s, (it / C::STAGES) & 1, &abort_flag, status, 0x300 + s))) break;
#ifdef Q36_TCPROF
                        pf_full += clock64() - pf_x;
#endif
                        const uint32_t sb = smem_u32(smem + s * C::STAGE_BYTES);
#pragma unroll
                        for (int x = 0; x < C::KS; x++) {
                            const int ks = h * C::KS + x;
#ifdef Q36_TCPROF
                            pf_x = clock64();
#endif
                            if (first && !(ok = mbar_wait(bq_full0 + 8 * ks, n & 1, &abort_flag, status, 0x220 + ks))) break;
#ifdef Q36_TCPROF
                            pf_b += clock64() - pf_x;
#endif
                            tc_fence_after();
                            tc_cp_sf(t_sfa, desc_sf(sb + C::KS * C::A_BYTES + x * C::SF_BYTES));
                            tc_cp_sf(t_sfb, desc_sf(smem_u32(smem + C::OFF_BIMG + ks * C::SF_BYTES)));
                            const uint32_t sa = sb + x * C::A_BYTES, sbb = smem_u32(smem + C::OFF_B + ks * C::B_STEP);
#pragma unroll
                            for (int kb = 0; kb < 4; kb++) {
                                const uint32_t sfid = (uint32_t)kb << 30;
                                tc_mma(d_tmem, desc_sw128(sa + kb * 32), desc_sw128(sbb + kb * 32), idesc_mx(n_mma, kb), t_sfa | sfid,
                                       t_sfb | sfid, (ks | kb) ? 1u : 0u);
                            }
                        }
                        if (!ok) break;
                        tc_commit(empty0 + 8 * s);
                    }
                    if (!ok) break;
                    first = false;
                    tc_commit(acc_full0 + 8 * buf);
                }
                if (ok) tc_commit(b_empty);     // (arrives when all of this warp's MMAs on the item have read the token rows)
            }
#ifdef Q36_TCPROF
            if (w == 0 && (blockIdx.x == 0 || blockIdx.x == 77 || blockIdx.x == 147))
                printf("down issuer cta %d: items %u total %lld wait_full %lld wait_acc %lld wait_tokens %lld\n", blockIdx.x, n, clock64() - pf_t0, pf_full, pf_acc, pf_b);
#endif
        }
    } else if (warp < C::W_LOAD0) {
        // ------------------------------ epilogue: accumulators -> f32 rows
        const int qd = warp & 3;                              // TMEM lane quarter this warp may read
        const int half = (warp - C::W_EPI0) >> 2;             // which of the quarter's warps: 32-column chunks in turn
        uint32_t n = 0;
        bool ok = true;
#ifdef Q36_TCPROF
        long long pf_w = 0, pf_busy = 0, pf_x, pf_y;
#endif
        for (int ii = blockIdx.x; ii < n_items && ok; ii += gridDim.x, n++) {
            const TcTile t = get_item(ii);
            for (int j = 0; j < DR_MC && ok; j++) {
                const uint32_t q = n * DR_MC + j, buf = q % C::ACC_BUFS;
#ifdef Q36_TCPROF
                pf_x = clock64();
#endif
                if (!(ok = mbar_wait(acc_full0 + 8 * buf, (q / C::ACC_BUFS) & 1, &abort_flag, status, 0x400 + buf, TC_SPIN_LIMIT, TC_BACKOFF_NS))) break;
#ifdef Q36_TCPROF
                pf_y = clock64(); pf_w += pf_y - pf_x;
#endif
                tc_fence_after();
                const uint32_t tq = tmem + buf * C::ACC_STRIDE + ((uint32_t)(qd * 32) << 16);
                const int mrow = (t.mt + j) * TC_M + qd * 32 + lane;
                for (int c0 = 32 * half; c0 < t.nrows; c0 += 8 * C::EPI_WARPS) {
                    uint32_t v[32];
                    tc_ld32(tq + c0, v);
                    tc_ld_wait();
#pragma unroll
                    for (int c = 0; c < 32; c++)
                        if (c0 + c < t.nrows) st_y(Y, (size_t)(t.row0 + c0 + c) * M_total + mrow, __uint_as_float(v[c]), y_bf16);
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(acc_empty0 + 8 * buf);
#ifdef Q36_TCPROF
                pf_busy += clock64() - pf_y;
#endif
            }
        }
#ifdef Q36_TCPROF
        if (lane == 0 && warp == C::W_EPI0 && (blockIdx.x == 0 || blockIdx.x == 77))
            printf("down epilogue cta %d: wait %lld busy %lld\n", blockIdx.x, pf_w, pf_busy);
#endif
    } else {
        // ------------------------------ scale images: thread i owns row i of the token tile and of every weight-row tile
        const int i = threadIdx.x - 32 * C::W_LOAD0;
        const uint32_t my_off = (i & 31) * 16 + (i >> 5) * 4;
        uint32_t n = 0;
        bool ok = true;
        for (int ii = blockIdx.x; ii < n_items && ok; ii += gridDim.x, n++) {
            const TcTile t = get_item(ii);
            // token scale images, once per item: wait for the staged bytes and for the previous item's images to be unused
            if (!(ok = mbar_wait(bs_full, n & 1, &abort_flag, status, 0x700, TC_SPIN_LIMIT, TC_BACKOFF_NS))) break;
            uint4 b = *reinterpret_cast<const uint4 *>(smem + C::OFF_BS + i * 16);
            if (i >= t.nrows) b = make_uint4(0x7f7f7f7fu, 0x7f7f7f7fu, 0x7f7f7f7fu, 0x7f7f7f7fu);
            if (!(ok = mbar_wait(b_empty, (n & 1) ^ 1, &abort_flag, status, 0x710, TC_SPIN_LIMIT, TC_BACKOFF_NS))) break;
            {
                uint8_t *img = smem + C::OFF_BIMG + my_off;
                *reinterpret_cast<uint32_t *>(img) = b.x;
                *reinterpret_cast<uint32_t *>(img + C::SF_BYTES) = b.y;
                *reinterpret_cast<uint32_t *>(img + 2 * C::SF_BYTES) = b.z;
                *reinterpret_cast<uint32_t *>(img + 3 * C::SF_BYTES) = b.w;
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            __syncwarp();
            if (lane == 0) { mbar_arrive(bimg_full); mbar_arrive(bs_empty); }
            // weight scale images, per row tile: 4 bytes per K step from the staged 16
            for (int j = 0; j < DR_MC && ok; j++) {
                const uint32_t q = n * DR_MC + j, sl = q % C::SFR_SLOTS;
                if (!(ok = mbar_wait(sfr_full0 + 8 * sl, (q / C::SFR_SLOTS) & 1, &abort_flag, status, 0x720 + sl, TC_SPIN_LIMIT, TC_BACKOFF_NS))) break;
                const uint4 a = *reinterpret_cast<const uint4 *>(smem + C::OFF_SFR + sl * C::SFR_BYTES + i * 16);
                const uint32_t wa[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
                for (int h = 0; h < C::KSTEPS / C::KS; h++) {
                    const uint32_t it = q * (C::KSTEPS / C::KS) + h, s = it % C::STAGES;
                    if (!(ok = mbar_wait(empty0 + 8 * s, ((it / C::STAGES) & 1) ^ 1, &abort_flag, status, 0x500 + s, TC_SPIN_LIMIT, TC_BACKOFF_NS))) break;
                    uint8_t *sf = smem + s * C::STAGE_BYTES + C::KS * C::A_BYTES + my_off;
                    *reinterpret_cast<uint32_t *>(sf) = wa[2 * h];
                    *reinterpret_cast<uint32_t *>(sf + C::SF_BYTES) = wa[2 * h + 1];
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                    __syncwarp();
                    if (lane == 0) mbar_arrive(full0 + 8 * s);
                }
                if (!ok) break;
                __syncwarp();
                if (lane == 0) mbar_arrive(sfr_empty0 + 8 * sl);
            }
        }
    }

    tc_fence_before();
    __syncthreads();
    if (abort_flag) {
        for (int i = 0; i < 200; i++) __nanosleep(1000);   // leave copies in flight time to land before the block retires
        if (threadIdx.x == 0) atomicCAS(status, 0, 1);
    }
    if (warp == C::W_ISSUE0) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(C::TMEM_COLS) : "memory");
    }
}

// ---------------------------------------------------------- host: tensor maps
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = (EncodeTiledFn)p;
    }
    return fn;
}
// Encoding a tensor map is host work (a driver call per map, 8 to 11 maps per launch); the engine builds everything
// that depends only on its buffers once at creation (q36_engine.cu:1467-1512).  The maps of a call depend only on
// pointers and shapes, which repeat from step to step, so every encode goes through a small per-thread cache.
struct MapKey {
    const void *base;
    uint64_t stride;
    int kind, a, b, c, d;
    bool operator==(const MapKey &o) const {
        return base == o.base && stride == o.stride && kind == o.kind && a == o.a && b == o.b && c == o.c && d == o.d;
    }
};
struct MapSlot { MapKey key; CUtensorMap map; bool used; };
constexpr int MAP_CACHE_SLOTS = 2048;   // direct-mapped; a collision just re-encodes
static MapSlot *map_cache() {
    static thread_local MapSlot *slots = nullptr;
    if (!slots) slots = new MapSlot[MAP_CACHE_SLOTS]();
    return slots;
}
static inline uint64_t mix64(uint64_t x) {
    x ^= x >> 33; x *= 0xff51afd7ed558ccdull; x ^= x >> 33; x *= 0xc4ceb9fe1a85ec53ull; x ^= x >> 33;
    return x;
}
static int encode_cached(CUtensorMap *m, const MapKey &k, CUtensorMapDataType dt, int rank, const cuuint64_t *dims,
                         const cuuint64_t *strides, const cuuint32_t *box, CUtensorMapSwizzle sw) {
    uint64_t h = mix64((uint64_t)(uintptr_t)k.base) ^ mix64(k.stride + 0x9e3779b97f4a7c15ull * (uint64_t)k.kind);
    h ^= mix64(((uint64_t)(uint32_t)k.a << 32) | (uint32_t)k.b) ^ mix64(((uint64_t)(uint32_t)k.c << 32) | (uint32_t)k.d);
    MapSlot &slot = map_cache()[h % MAP_CACHE_SLOTS];
    if (slot.used && slot.key == k) { *m = slot.map; return Q36_MOE_OK; }
    EncodeTiledFn fn = encode_fn();
    if (!fn) return Q36_MOE_ECUDA;
    const cuuint32_t el[5] = {1, 1, 1, 1, 1};
    // L2 promotion 256 B: every operand is consumed along K by the same SM, so what a copy pulls into L2 beyond its box is
    // the next stages' data (measured: decode kernel 26.5 against 26.9 us with 128 B, 27.7 with 64 B; Q36_L2PROMO overrides)
    static const int promo = getenv("Q36_L2PROMO") ? atoi(getenv("Q36_L2PROMO")) : 256;
    const CUtensorMapL2promotion l2p = promo == 256 ? CU_TENSOR_MAP_L2_PROMOTION_L2_256B
                                       : promo == 64 ? CU_TENSOR_MAP_L2_PROMOTION_L2_64B
                                       : promo == 0  ? CU_TENSOR_MAP_L2_PROMOTION_NONE
                                                     : CU_TENSOR_MAP_L2_PROMOTION_L2_128B;
    CUresult r = fn(m, dt, (cuuint32_t)rank, const_cast<void *>(k.base), dims, strides, box, el, CU_TENSOR_MAP_INTERLEAVE_NONE, sw,
                    l2p, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) { last_cuda_error() = 100000 + (int)r; return Q36_MOE_ECUDA; }
    slot.key = k; slot.map = *m; slot.used = true;
    return Q36_MOE_OK;
}

// code plane of n_group experts: [n_group][M][K] 4-bit elements
int make_map_codes(CUtensorMap *m, const void *base, int M, int K, int n_group, uint64_t expert_stride) {
    cuuint64_t dims[3] = {(cuuint64_t)K, (cuuint64_t)M, (cuuint64_t)n_group};
    cuuint64_t strides[2] = {(cuuint64_t)(K / 2), (cuuint64_t)expert_stride};
    cuuint32_t box[3] = {128, TC_M, 1};
    return encode_cached(m, MapKey{base, expert_stride, 1, M, K, n_group, 0}, CU_TENSOR_MAP_DATA_TYPE_16U4_ALIGN16B, 3, dims,
                         strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
}
// A thread needs ~140 cycles to issue any asynchronous copy, whatever its size, so the decode kernel fetches
// several K steps per copy: the K axis is split into (step, 128 elements) and the step index becomes a box
// dimension AFTER the rows, which lays the steps down as consecutive [rows][128 B] swizzled tiles.
int make_map_codes_ksteps(CUtensorMap *m, const void *base, int M, int K, int n_group, uint64_t expert_stride, int ksteps) {
    cuuint64_t dims[4] = {128, (cuuint64_t)M, (cuuint64_t)(K / 128), (cuuint64_t)n_group};
    cuuint64_t strides[3] = {(cuuint64_t)(K / 2), 64, (cuuint64_t)expert_stride};
    cuuint32_t box[4] = {128, TC_M, (cuuint32_t)ksteps, 1};
    return encode_cached(m, MapKey{base, expert_stride, 2, M, K, n_group, ksteps}, CU_TENSOR_MAP_DATA_TYPE_16U4_ALIGN16B, 4, dims,
                         strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
}
int make_map_rows_ksteps(CUtensorMap *m, const void *base, int R, int K, int box_rows, int ksteps) {
    cuuint64_t dims[3] = {128, (cuuint64_t)R, (cuuint64_t)(K / 128)};
    cuuint64_t strides[2] = {(cuuint64_t)K, 128};
    cuuint32_t box[3] = {128, (cuuint32_t)box_rows, (cuuint32_t)ksteps};
    return encode_cached(m, MapKey{base, 0, 3, R, K, box_rows, ksteps}, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, dims, strides, box,
                         CU_TENSOR_MAP_SWIZZLE_128B);
}
// activation rows: [R][K] bytes, boxes of box_rows rows x 128 B
int make_map_rows(CUtensorMap *m, const void *base, int R, int K, int box_rows) {
    cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)R};
    cuuint64_t strides[1] = {(cuuint64_t)K};
    cuuint32_t box[2] = {128, (cuuint32_t)box_rows};
    return encode_cached(m, MapKey{base, 0, 4, R, K, box_rows, 0}, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, dims, strides, box,
                         CU_TENSOR_MAP_SWIZZLE_128B);
}

// The multiprocessor count and the kernels' opt-in to more than 48 KB of dynamic shared memory are per DEVICE:
// a host thread that drives several devices in turn (q36_multi_create / q36_multi_prefill, q36_engine.cu:4234-4306)
// must find both set for whichever device is current.
int current_device() {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= MAX_DEVICES) return -1;
    return dev;
}
int sm_count() {
    static int n[MAX_DEVICES] = {0};
    const int dev = current_device();
    if (dev < 0) return 148;
    if (!n[dev]) {
        int v = 0;
        cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev);
        n[dev] = v > 0 ? v : 148;
    }
    return n[dev];
}
// Once per (kernel, device): allow `bytes` of dynamic shared memory.  done: MAX_DEVICES flags owned by the caller.
int ensure_smem_attr(const void *kernel, int bytes, bool *done) {
    const int dev = current_device();
    if (dev < 0) return Q36_MOE_EINVAL;
    if (done[dev]) return Q36_MOE_OK;
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes) != cudaSuccess) return check_launch();
    done[dev] = true;
    return Q36_MOE_OK;
}

uint64_t tc_ws_bytes() { return (sizeof(TcPlan) + 255) & ~(uint64_t)255; }

int launch_tc_plan(const int *goffs, int n_group, const int *soffs, int D, int FF, void *plan, int *status,
                   int tile_rows, cudaStream_t st) {
    if (n_group + 1 > DISPATCH_MAX_GROUPS) return Q36_MOE_EINVAL;
    launch_k(k_tc_plan, dim3(1), dim3(512), 0, st, goffs, n_group, soffs, (TcPlan *)plan, FF / TC_M, D / TC_M, status, tile_rows);
    return check_launch();
}

// scale plane of n_group experts: [n_group][rows][nb] bytes (n_group = 0: a plain [rows][nb] matrix),
// boxes of 16 B (four K steps) x box_rows rows
static int make_map_scales(CUtensorMap *m, const void *base, int rows, int nb, int n_group, uint64_t stride3, int box_rows) {
    cuuint64_t dims[3] = {(cuuint64_t)nb, (cuuint64_t)rows, (cuuint64_t)(n_group > 0 ? n_group : 1)};
    cuuint64_t strides[2] = {(cuuint64_t)nb, (cuuint64_t)stride3};
    cuuint32_t box[3] = {16, (cuuint32_t)box_rows, 1};
    return encode_cached(m, MapKey{base, stride3, 5, rows, nb, n_group, box_rows}, CU_TENSOR_MAP_DATA_TYPE_UINT8,
                         n_group > 0 ? 3 : 2, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_NONE);
}

// A0/A1: routed experts' planes (A1 unused for NA = 1); S0/S1: the shared expert's planes or NULL.
template <int NA>
static int run_grouped(const void *A0, const void *A1, const void *S0, const void *S1, int n_group, int R_max,
                       const uint8_t *Bq, const uint8_t *Bs, uint8_t *Hq, uint8_t *Hs, float *Y, int M, int K,
                       const void *plan, int *status, cudaStream_t st, int y_bf16 = 0) {
    using Cfg = TcCfg<NA>;
    if (M % TC_M || K % (4 * TC_KSTEP) || n_group + 1 > DISPATCH_MAX_GROUPS) return Q36_MOE_EINVAL;
    const uint64_t estride = (uint64_t)M * (K / 2) + (uint64_t)M * (K / Q36_QK);
    const uint64_t plane = (uint64_t)M * (K / 2);
    const int nb = K / Q36_QK;
    if (NA == 1) A1 = A0;
    if (!S0) { S0 = A0; S1 = A1; }
    if (NA == 1) S1 = S0;
    TcMaps maps;
    int rc;
    if ((rc = make_map_codes(&maps.a0, A0, M, K, n_group, estride))) return rc;
    if ((rc = make_map_codes(&maps.a1, A1, M, K, n_group, estride))) return rc;
    if ((rc = make_map_codes(&maps.s0, S0, M, K, 1, estride))) return rc;
    if ((rc = make_map_codes(&maps.s1, S1, M, K, 1, estride))) return rc;
    if ((rc = make_map_rows(&maps.b16, Bq, R_max, K, 16))) return rc;
    if ((rc = make_map_rows(&maps.bfull, Bq, R_max, K, Cfg::N))) return rc;
    if ((rc = make_map_scales(&maps.fa0, (const uint8_t *)A0 + plane, M, nb, n_group, estride, TC_M))) return rc;
    if ((rc = make_map_scales(&maps.fa1, (const uint8_t *)A1 + plane, M, nb, n_group, estride, TC_M))) return rc;
    if ((rc = make_map_scales(&maps.fs0, (const uint8_t *)S0 + plane, M, nb, 1, estride, TC_M))) return rc;
    if ((rc = make_map_scales(&maps.fs1, (const uint8_t *)S1 + plane, M, nb, 1, estride, TC_M))) return rc;
    if ((rc = make_map_scales(&maps.fb, Bs, R_max, nb, 0, 0, Cfg::N))) return rc;
    static bool attr_done[MAX_DEVICES] = {false};   // one array per instantiation
    if ((rc = ensure_smem_attr((const void *)k_grouped_mma<NA>, Cfg::SMEM_BYTES, attr_done))) return rc;
    if (Cfg::REBALANCE) {
        // the epilogue warps' setmaxnreg.inc waits for registers the first eight warps give back: never launch a build
        // whose register pool (registers per thread at launch x threads) cannot cover both groups' new sizes
        static int regs[MAX_DEVICES] = {0};
        const int dv = current_device();
        if (dv < 0) return Q36_MOE_ECUDA;
        int &nr = regs[dv];
        if (!nr) {
            cudaFuncAttributes fa;
            if (cudaFuncGetAttributes(&fa, (const void *)k_grouped_mma<NA>) != cudaSuccess) return Q36_MOE_ECUDA;
            nr = fa.numRegs;
        }
        if ((nr + 7) / 8 * 8 * Cfg::THREADS < 32 * (Cfg::EPI_WARP0 * Cfg::REGS_LOW + Cfg::EPI_WARPS * Cfg::REGS_EPI)) return Q36_MOE_EUNSUPPORTED;
    }
    const int m_tiles = M / TC_M;
    const long max_tiles = ((long)(R_max + Cfg::N - 1) / Cfg::N + n_group + 1) * m_tiles;
    const int grid = (int)min((long)sm_count(), max_tiles);
    launch_k(k_grouped_mma<NA>, dim3(grid), dim3(Cfg::THREADS), Cfg::SMEM_BYTES, st, maps, n_group, (const TcPlan *)plan, Hq, Hs,
             Y, M, K, status, y_bf16);
    return check_launch();
}

// Token rows per tile the work plan of a two-launch call must be cut in (0: the 112 / 128 defaults): 128 when the
// gate/up launch is k_gateup_wide.  Q36_GATEUP_NARROW in the environment keeps k_grouped_mma<2>.
int gateup_tile_rows() {
    static const bool narrow = getenv("Q36_GATEUP_NARROW") != nullptr;
    return narrow ? 0 : GuWide::N;
}

static int run_gateup_wide(const void *Wg, const void *Wu, const void *Sg, const void *Su, int n_group, int R_max, const uint8_t *Xq,
                           const uint8_t *Xs, uint8_t *Hq, uint8_t *Hs, int FF, int K, const void *plan, int *status, cudaStream_t st) {
    using C = GuWide;
    if (FF % TC_M || K % (4 * TC_KSTEP) || n_group + 1 > DISPATCH_MAX_GROUPS) return Q36_MOE_EINVAL;
    const uint64_t estride = (uint64_t)FF * (K / 2) + (uint64_t)FF * (K / Q36_QK), plane = (uint64_t)FF * (K / 2);
    const int nb = K / Q36_QK;
    if (!Sg) { Sg = Wg; Su = Wu; }
    TcMaps maps;
    int rc;
    if ((rc = make_map_codes(&maps.a0, Wg, FF, K, n_group, estride))) return rc;
    if ((rc = make_map_codes(&maps.a1, Wu, FF, K, n_group, estride))) return rc;
    if ((rc = make_map_codes(&maps.s0, Sg, FF, K, 1, estride))) return rc;
    if ((rc = make_map_codes(&maps.s1, Su, FF, K, 1, estride))) return rc;
    if ((rc = make_map_rows(&maps.b16, Xq, R_max, K, 16))) return rc;
    if ((rc = make_map_rows(&maps.bfull, Xq, R_max, K, C::N))) return rc;
    if ((rc = make_map_scales(&maps.fa0, (const uint8_t *)Wg + plane, FF, nb, n_group, estride, TC_M))) return rc;
    if ((rc = make_map_scales(&maps.fa1, (const uint8_t *)Wu + plane, FF, nb, n_group, estride, TC_M))) return rc;
    if ((rc = make_map_scales(&maps.fs0, (const uint8_t *)Sg + plane, FF, nb, 1, estride, TC_M))) return rc;
    if ((rc = make_map_scales(&maps.fs1, (const uint8_t *)Su + plane, FF, nb, 1, estride, TC_M))) return rc;
    if ((rc = make_map_scales(&maps.fb, Xs, R_max, nb, 0, 0, C::N))) return rc;
    static bool attr_done[MAX_DEVICES] = {false};
    if ((rc = ensure_smem_attr((const void *)k_gateup_wide, C::SMEM_BYTES, attr_done))) return rc;
    {   // as for k_grouped_mma<2>: the register pool must cover both warp groups' sizes after setmaxnreg
        static int regs[MAX_DEVICES] = {0};
        const int dv = current_device();
        if (dv < 0) return Q36_MOE_ECUDA;
        int &nr = regs[dv];
        if (!nr) {
            cudaFuncAttributes fa;
            if (cudaFuncGetAttributes(&fa, (const void *)k_gateup_wide) != cudaSuccess) return Q36_MOE_ECUDA;
            nr = fa.numRegs;
        }
        if ((nr + 7) / 8 * 8 * C::THREADS < 32 * (C::EPI_WARP0 * C::REGS_LOW + C::EPI_WARPS * C::REGS_EPI)) return Q36_MOE_EUNSUPPORTED;
    }
    const int m_tiles = FF / TC_M;
    const long max_tiles = ((long)(R_max + C::N - 1) / C::N + n_group + 1) * m_tiles;
    const int grid = (int)min((long)sm_count(), max_tiles);
    launch_k(k_gateup_wide, dim3(grid), dim3(C::THREADS), C::SMEM_BYTES, st, maps, n_group, (const TcPlan *)plan, Hq, Hs, FF, K, status);
    return check_launch();
}

int launch_gateup_tc(const void *Wg, const void *Wu, const void *Sg, const void *Su, int n_group, int R_max,
                     int max_group_rows, const uint8_t *Xq, const uint8_t *Xs, uint8_t *Hq, uint8_t *Hs, int D, int FF,
                     const void *plan, int *status, cudaStream_t st) {
    (void)max_group_rows;
    if (gateup_tile_rows() == GuWide::N)
        return run_gateup_wide(Wg, Wu, Sg, Su, n_group, R_max, Xq, Xs, Hq, Hs, FF, D, plan, status, st);
    return run_grouped<2>(Wg, Wu, Sg, Su, n_group, R_max, Xq, Xs, Hq, Hs, nullptr, FF, D, plan, status, st);
}
// K = 512 and D a multiple of DR_MC row tiles: the token-tile-resident kernel
static int run_down_resident(const void *Wd, const void *Sd, int n_group, int R_max, const uint8_t *Hq, const uint8_t *Hs, float *Y,
                             int M, int K, const void *plan, int *status, cudaStream_t st, int y_bf16) {
    using C = DownRes;
    const uint64_t estride = (uint64_t)M * (K / 2) + (uint64_t)M * (K / Q36_QK), plane = (uint64_t)M * (K / 2);
    const int nb = K / Q36_QK;
    if (!Sd) Sd = Wd;
    DownMaps maps;
    int rc;
    if ((rc = make_map_codes_ksteps(&maps.a, Wd, M, K, n_group, estride, C::KS))) return rc;
    if ((rc = make_map_codes_ksteps(&maps.s, Sd, M, K, 1, estride, C::KS))) return rc;
    if ((rc = make_map_rows(&maps.b, Hq, R_max, K, C::N))) return rc;
    if ((rc = make_map_scales(&maps.fa, (const uint8_t *)Wd + plane, M, nb, n_group, estride, TC_M))) return rc;
    if ((rc = make_map_scales(&maps.fs, (const uint8_t *)Sd + plane, M, nb, 1, estride, TC_M))) return rc;
    if ((rc = make_map_scales(&maps.fb, Hs, R_max, nb, 0, 0, C::N))) return rc;
    static bool attr_done[MAX_DEVICES] = {false}, attr_done_bf[MAX_DEVICES] = {false};
    if ((rc = ensure_smem_attr(y_bf16 ? (const void *)k_down_resident<1> : (const void *)k_down_resident<0>, C::SMEM_BYTES,
                               y_bf16 ? attr_done_bf : attr_done))) return rc;
    const int mc = (M / TC_M) % 16 == 0 ? 16 : DR_MC_MIN;
    const long max_items = ((long)(R_max + C::N - 1) / C::N + n_group + 1) * (M / TC_M / mc);
    const int grid = (int)min((long)sm_count(), max_items);
    if (y_bf16) launch_k(k_down_resident<1>, dim3(grid), dim3(C::THREADS), C::SMEM_BYTES, st, maps, n_group, (const TcPlan *)plan, Y, M, status, mc);
    else launch_k(k_down_resident<0>, dim3(grid), dim3(C::THREADS), C::SMEM_BYTES, st, maps, n_group, (const TcPlan *)plan, Y, M, status, mc);
    return check_launch();
}

int stage_y_bf16() {
    static const int on = getenv("Q36_Y_BF16") ? 1 : 0;
    return on;
}

int launch_down_tc(const void *Wd, const void *Sd, int n_group, int R_max, int max_group_rows, const uint8_t *Hq,
                   const uint8_t *Hs, float *Y, int D, int FF, const void *plan, int *status, cudaStream_t st, int y_bf16) {
    (void)max_group_rows;
    static const bool old_down = getenv("Q36_OLD_DOWN") != nullptr;
    if (!old_down && FF == DownRes::KSTEPS * TC_KSTEP && D % (TC_M * DR_MC_MIN) == 0 && n_group + 1 <= DISPATCH_MAX_GROUPS)
        return run_down_resident(Wd, Sd, n_group, R_max, Hq, Hs, Y, D, FF, plan, status, st, y_bf16);
    return run_grouped<1>(Wd, nullptr, Sd, nullptr, n_group, R_max, Hq, Hs, nullptr, nullptr, Y, D, FF, plan, status, st, y_bf16);
}

}  // namespace q36
