// Prefill-sized expert groups: grouped GEMM on the 5th-generation tensor cores.
//
//   D[128 weight rows x N tokens] += A[128 x K] (MXFP4 codes + E8M0 scales)
//                                  * B[N x K]^T (E4M3 codes + UE8M0 scales)
//   tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale, accumulators in TMEM.
//
// Replaces k_gemm_expert_mma (q36_engine.cu:2435-2524; mma.sync m16n8k32
// block-scaled, an sm_120a-only instruction) for gate/up and k_gemm_expert_tc
// (:2723-2766) for an MXFP4 down projection.
//
// Operand staging
//   A  TMA, CU_TENSOR_MAP_DATA_TYPE_16U4_ALIGN16B: the packed code plane
//      (K/2 bytes per row, GGUF nibble order) is expanded on the fly into the
//      padded form the tensor core reads (16 codes in 8 B + 8 B gap), 128 B of
//      shared memory per 128 K-elements, 128B swizzle.
//   B  TMA, UINT8, boxes of 16 token rows x 128 B, 128B swizzle.  Rows are in
//      "hw order" inside each 32-block, so that position p of B meets nibble p
//      of A.
//   SF four warps copy the E8M0 bytes of the tile's rows from the row-major
//      scale planes into shared memory in the 32 x 16 B image that
//      tcgen05.cp.32x128b.warpx4 broadcasts into TMEM: row m of the tile at
//      byte (m % 32) * 16 + (m / 32) * 4 + kb.
// Roles (320 threads): warp 0 TMA producer, warp 1 MMA issuer + TMEM owner,
// warps 2-5 epilogue (TMEM -> registers -> global), warps 6-9 scale loaders.
// One persistent CTA per SM walks a tile table built on the device (largest
// groups first).  Every mbarrier wait is bounded; a wait that gives up raises
// a status word that the host entry point reports as Q36_MOE_EDEVICE.
#include <cuda.h>

#include "common.cuh"
#include "kernels.cuh"

namespace q36 {

constexpr int TC_M = 128;        // weight rows per tile (UMMA M)
constexpr int TC_KSTEP = 128;    // K elements per pipeline stage (= 128 B per row in smem)
constexpr int TC_THREADS = 320;
constexpr uint32_t TC_SPIN_LIMIT = 1u << 22;

struct TcTile { int g, mt, row0, nrows; };

// Work plan of one grouped-FFN call, built on the device by k_tc_plan and read by both MMA launches.
// Groups are ranked by size (largest first); base[w][r] is the first tile of rank r for launch w
// (0 = gate/up, 1 = down), so a tile index maps to (group, token tile, row tile) by a binary search.
struct TcPlan {
    int n_groups, n_tiles[2], pad;
    int order[DISPATCH_MAX_GROUPS + 1];   // rank -> group
    int row0[DISPATCH_MAX_GROUPS + 1];    // group -> first row of the sorted space
    int cnt[DISPATCH_MAX_GROUPS + 1];     // group -> rows
    int base[2][DISPATCH_MAX_GROUPS + 2];
};

// ------------------------------------------------------------------ PTX
__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint32_t a, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(a), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t a, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(a), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t a) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(a) : "memory");
}
__device__ __forceinline__ bool mbar_try(uint32_t a, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(a), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait.  Returns false (and raises *abort_flag) when it gives up or
// when another role already gave up.
// `where` identifies the waiter (role * 256 + stage or tile parity) and is what the status word receives.
__device__ __forceinline__ bool mbar_wait(uint32_t a, uint32_t parity, volatile int *abort_flag, int *status, int where) {
    for (uint32_t i = 0; i < TC_SPIN_LIMIT; i++) {
        if (mbar_try(a, parity)) return true;
        if ((i & 1023u) == 1023u && *abort_flag) return false;
    }
    *abort_flag = 1;
    atomicCAS(status, 0, where);
    return false;
}
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap *m, int x, int y, int z, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
        ::"r"(dst), "l"(m), "r"(bar), "r"(x), "r"(y), "r"(z)
        : "memory");
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap *m, int x, int y, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst), "l"(m), "r"(bar), "r"(x), "r"(y)
        : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tc_cp_sf(uint32_t taddr, uint64_t sdesc) {
    asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(sdesc) : "memory");
}
__device__ __forceinline__ void tc_mma(uint32_t d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t sfa,
                                       uint32_t sfb, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
        ::"r"(d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(sfa), "r"(sfb)
        : "memory");
}
__device__ __forceinline__ void tc_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
        "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tc_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// K-major, 128B-swizzled operand tile (rows of 128 B, 8-row groups 1024 B
// apart): start address, LBO 1 (unused for swizzled K-major), SBO 1024 B,
// descriptor version 1, layout type 2 (SWIZZLE_128B).
__device__ __forceinline__ uint64_t desc_sw128(uint32_t saddr) {
    return (uint64_t)((saddr & 0x3FFFFu) >> 4) | ((uint64_t)1 << 16) | ((uint64_t)(1024 >> 4) << 32) |
           ((uint64_t)1 << 46) | ((uint64_t)2 << 61);
}
// Scale-factor image for tcgen05.cp: 32 rows x 16 B, no swizzle, 8-row core
// matrices 128 B apart.
__device__ __forceinline__ uint64_t desc_sf(uint32_t saddr) {
    return (uint64_t)((saddr & 0x3FFFFu) >> 4) | ((uint64_t)(128 >> 4) << 32) | ((uint64_t)1 << 46);
}
// Block-scaled instruction descriptor: A = E2M1 (5), B = E4M3 (0), both
// K-major, UE8M0 scales, M = 128, N = n; scale-factor byte ids select which
// of the four K-blocks of a 32-bit TMEM scale column this MMA uses.
__device__ __forceinline__ uint32_t idesc_mx(int n, int kb) {
    return ((uint32_t)kb << 4) | (5u << 7) | (0u << 10) | ((uint32_t)(n >> 3) << 17) | (1u << 23) |
           ((uint32_t)(TC_M >> 4) << 24) | ((uint32_t)kb << 29);
}

// ------------------------------------------------------------ configuration
// NA = 2: gate/up (two A operands, SwiGLU + E4M3 requantisation epilogue), token tile 112
// NA = 1: down (one A operand, f32 rows out), token tile 128
// The token tile of gate/up is 112 so that TWO accumulator sets (gate + up each) and the scale
// columns fit the 512 TMEM columns: the epilogue of one tile overlaps the MMAs of the next.
template <int NA>
struct TcCfg {
    static constexpr int N = (NA == 2) ? 112 : 128;          // token rows per tile (max UMMA N)
    static constexpr int STAGES = (NA == 2) ? 4 : 6;
    static constexpr int A_BYTES = TC_M * 128;               // 16 KB of shared memory per A operand per stage
    // What the A box signals on the mbarrier: the PACKED bytes read from global memory (64 B per row), not
    // the 128 B per row it occupies after expansion.  Measured on B200: expecting 16 KB leaves the barrier
    // pending for ever, expecting 8 KB completes it.
    static constexpr int A_TX_BYTES = TC_M * 64;
    static constexpr int B_BYTES = 128 * 128;                // 16 KB slot (N rows used)
    static constexpr int SF_BYTES = 512;
    static constexpr int STAGE_BYTES = NA * A_BYTES + B_BYTES + (NA + 1) * SF_BYTES;
    static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /* alignment slack */ + 256 /* barriers */;
    static constexpr int ACC_STRIDE = (NA == 2) ? 256 : 128; // TMEM columns between the two accumulator sets
    static constexpr int SF_COL0 = (NA == 2) ? 224 : 256;    // scale columns: A0 (4), [A1 (4)], B (4)
    static constexpr int TMEM_COLS = 512;
    static constexpr int B_FULL_MIN = 49;                    // token tiles of at least this many rows use one big box
};

// ------------------------------------------------------------- tile plan
// One block.  Ranks the groups by size and lays the prefix sums of their tile counts.
__global__ void __launch_bounds__(512)
k_tc_plan(const int *__restrict__ goffs, int n_group, const int *__restrict__ soffs, TcPlan *plan, int mt_gu,
          int mt_dn, int *status) {
    Q36_GDS();
    __shared__ int cnt[DISPATCH_MAX_GROUPS + 1], order[DISPATCH_MAX_GROUPS + 1], tg[DISPATCH_MAX_GROUPS + 1],
        td[DISPATCH_MAX_GROUPS + 1];
    const int tid = threadIdx.x;
    const int G = n_group + (soffs ? 1 : 0);
    for (int g = tid; g < G; g += blockDim.x) {
        const int r0 = (g < n_group) ? goffs[g] : soffs[0];
        const int r1 = (g < n_group) ? goffs[g + 1] : soffs[1];
        cnt[g] = max(0, r1 - r0);
        plan->row0[g] = r0;
        plan->cnt[g] = cnt[g];
    }
    if (tid < 4) status[tid] = 0;
    __syncthreads();
    for (int g = tid; g < G; g += blockDim.x) {
        int r = 0;
        for (int h = 0; h < G; h++) r += (cnt[h] > cnt[g]) || (cnt[h] == cnt[g] && h < g);
        order[r] = g;
    }
    __syncthreads();
    for (int r = tid; r < G; r += blockDim.x) {
        const int n = cnt[order[r]];
        tg[r] = ((n + TcCfg<2>::N - 1) / TcCfg<2>::N) * mt_gu;
        td[r] = ((n + TcCfg<1>::N - 1) / TcCfg<1>::N) * mt_dn;
        plan->order[r] = order[r];
    }
    __syncthreads();
    for (int r = tid; r <= G; r += blockDim.x) {
        int a = 0, b = 0;
        for (int h = 0; h < r; h++) { a += tg[h]; b += td[h]; }
        plan->base[0][r] = a;
        plan->base[1][r] = b;
        if (r == G) { plan->n_tiles[0] = a; plan->n_tiles[1] = b; plan->n_groups = G; }
    }
}

// ------------------------------------------------------------ main kernel
struct TcMaps { CUtensorMap a0, a1, s0, s1, b16, bfull; };

template <int NA>
__global__ void __launch_bounds__(TC_THREADS, 1)
k_grouped_mma(const __grid_constant__ TcMaps maps, const uint8_t *__restrict__ sfA0, const uint8_t *__restrict__ sfA1,
              uint64_t sfA_stride, const uint8_t *__restrict__ sfS0, const uint8_t *__restrict__ sfS1, int n_routed,
              const uint8_t *__restrict__ sfB, const TcPlan *__restrict__ plan, uint8_t *__restrict__ Hq,
              uint8_t *__restrict__ Hs, float *__restrict__ Y, int M_total, int K, int *__restrict__ status) {
    using Cfg = TcCfg<NA>;
    constexpr int W = (NA == 2) ? 0 : 1;
    Q36_GDS();
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem + Cfg::STAGES * Cfg::STAGE_BYTES);
    // bars: full[STAGES], empty[STAGES], acc_full[2], acc_empty[2]
    __shared__ uint32_t tmem_base_s;
    __shared__ volatile int abort_flag;
    __shared__ int s_order[DISPATCH_MAX_GROUPS + 1], s_row0[DISPATCH_MAX_GROUPS + 1], s_cnt[DISPATCH_MAX_GROUPS + 1],
        s_base[DISPATCH_MAX_GROUPS + 2];

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t full0 = smem_u32(bars), empty0 = smem_u32(bars + Cfg::STAGES);
    const uint32_t acc_full0 = smem_u32(bars + 2 * Cfg::STAGES), acc_empty0 = smem_u32(bars + 2 * Cfg::STAGES + 2);
    const int n_tiles = plan->n_tiles[W];
    const int G = plan->n_groups;
    const int k_steps = K / TC_KSTEP;
    const int nb = K / Q36_QK;
    const int m_tiles = M_total / TC_M;

    for (int i = threadIdx.x; i <= G; i += blockDim.x) {
        s_base[i] = plan->base[W][i];
        if (i < G) { s_order[i] = plan->order[i]; s_row0[i] = plan->row0[i]; s_cnt[i] = plan->cnt[i]; }
    }
    if (threadIdx.x == 0) {
        abort_flag = 0;
        for (int s = 0; s < Cfg::STAGES; s++) {
            mbar_init(full0 + 8 * s, 1 + 4);   // producer's expect_tx arrive + one arrive per scale warp
            mbar_init(empty0 + 8 * s, 1);      // tcgen05.commit
        }
        for (int b = 0; b < 2; b++) {
            mbar_init(acc_full0 + 8 * b, 1);   // tcgen05.commit
            mbar_init(acc_empty0 + 8 * b, 4);  // one arrive per epilogue warp
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_s)), "r"(Cfg::TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
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

    if (warp == 0) {
        // ---------------------------------------------------- TMA producer
        if (lane == 0) {
            uint32_t it = 0;
            bool ok = true;
            for (int ti = blockIdx.x; ti < n_tiles && ok; ti += gridDim.x) {
                const TcTile t = get_tile(ti);
                const bool sh = t.g >= n_routed;
                const CUtensorMap *ma0 = sh ? &maps.s0 : &maps.a0, *ma1 = sh ? &maps.s1 : &maps.a1;
                const int ge = sh ? 0 : t.g;
                const bool full_box = t.nrows >= Cfg::B_FULL_MIN;
                const int slabs = (t.nrows + 15) / 16;
                const uint32_t tx = NA * Cfg::A_TX_BYTES + (full_box ? Cfg::N * 128 : slabs * 2048);
                for (int ks = 0; ks < k_steps; ks++, it++) {
                    const int s = it % Cfg::STAGES;
                    const uint32_t ph = (it / Cfg::STAGES) & 1;
                    if (!(ok = mbar_wait(empty0 + 8 * s, ph ^ 1, &abort_flag, status, 0x100 + s))) break;
                    const uint32_t sb = smem_u32(smem + s * Cfg::STAGE_BYTES);
                    mbar_expect_tx(full0 + 8 * s, tx);
                    tma_load_3d(sb, ma0, ks * TC_KSTEP, t.mt * TC_M, ge, full0 + 8 * s);
                    if (NA == 2) tma_load_3d(sb + Cfg::A_BYTES, ma1, ks * TC_KSTEP, t.mt * TC_M, ge, full0 + 8 * s);
                    if (full_box) {
                        tma_load_2d(sb + NA * Cfg::A_BYTES, &maps.bfull, ks * TC_KSTEP, t.row0, full0 + 8 * s);
                    } else {
                        for (int i = 0; i < slabs; i++)
                            tma_load_2d(sb + NA * Cfg::A_BYTES + i * 2048, &maps.b16, ks * TC_KSTEP, t.row0 + 16 * i, full0 + 8 * s);
                    }
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------ MMA issuer
        if (lane == 0) {
            uint32_t it = 0, tcount = 0;
            bool ok = true;
            for (int ti = blockIdx.x; ti < n_tiles && ok; ti += gridDim.x, tcount++) {
                const TcTile t = get_tile(ti);
                const int n_mma = (t.nrows >= Cfg::B_FULL_MIN) ? Cfg::N : max(16, (t.nrows + 15) & ~15);
                const uint32_t buf = tcount & 1;
                const uint32_t d_tmem = tmem + buf * Cfg::ACC_STRIDE;
                // this accumulator set must have been drained by the epilogue two tiles ago
                if (!(ok = mbar_wait(acc_empty0 + 8 * buf, ((tcount >> 1) & 1) ^ 1, &abort_flag, status, 0x200 + buf))) break;
                tc_fence_after();
                for (int ks = 0; ks < k_steps; ks++, it++) {
                    const int s = it % Cfg::STAGES;
                    const uint32_t ph = (it / Cfg::STAGES) & 1;
                    if (!(ok = mbar_wait(full0 + 8 * s, ph, &abort_flag, status, 0x300 + s))) break;
                    tc_fence_after();
                    const uint32_t sb = smem_u32(smem + s * Cfg::STAGE_BYTES);
                    const uint32_t sf = sb + NA * Cfg::A_BYTES + Cfg::B_BYTES;
                    const uint32_t t_sfa0 = tmem + Cfg::SF_COL0, t_sfb = tmem + Cfg::SF_COL0 + 4 * NA;
                    tc_cp_sf(t_sfa0, desc_sf(sf));
                    if (NA == 2) tc_cp_sf(t_sfa0 + 4, desc_sf(sf + Cfg::SF_BYTES));
                    tc_cp_sf(t_sfb, desc_sf(sf + NA * Cfg::SF_BYTES));
#pragma unroll
                    for (int kb = 0; kb < 4; kb++) {
                        const uint32_t acc = (ks | kb) ? 1u : 0u;
                        const uint32_t id = idesc_mx(n_mma, kb);
                        const uint64_t bd = desc_sw128(sb + NA * Cfg::A_BYTES + kb * 32);
                        const uint32_t sfid = (uint32_t)kb << 30;
                        tc_mma(d_tmem, desc_sw128(sb + kb * 32), bd, id, t_sfa0 | sfid, t_sfb | sfid, acc);
                        if (NA == 2)
                            tc_mma(d_tmem + Cfg::N, desc_sw128(sb + Cfg::A_BYTES + kb * 32), bd, id, (t_sfa0 + 4) | sfid, t_sfb | sfid, acc);
                    }
                    tc_commit(empty0 + 8 * s);   // stage reusable once these MMAs have read it
                }
                if (ok) tc_commit(acc_full0 + 8 * buf);     // accumulators complete
            }
        }
    } else if (warp < 6) {
        // -------------------------------------------------------- epilogue
        const int q = warp & 3;                  // TMEM lane quarter this warp may read
        uint32_t tcount = 0;
        bool ok = true;
        for (int ti = blockIdx.x; ti < n_tiles && ok; ti += gridDim.x, tcount++) {
            const TcTile t = get_tile(ti);
            const uint32_t buf = tcount & 1;
            const uint32_t tq = tmem + buf * Cfg::ACC_STRIDE + ((uint32_t)(q * 32) << 16);
            if (!(ok = mbar_wait(acc_full0 + 8 * buf, (tcount >> 1) & 1, &abort_flag, status, 0x400 + buf))) break;
            tc_fence_after();
            const int mrow = t.mt * TC_M + q * 32 + lane;   // weight row (output feature) of this thread
            for (int c0 = 0; c0 < t.nrows; c0 += 32) {
                uint32_t g[32];
                tc_ld32(tq + c0, g);
                if (NA == 2) {
                    uint32_t u[32];
                    tc_ld32(tq + Cfg::N + c0, u);
                    tc_ld_wait();
                    const int blk = mrow / Q36_QK;           // this warp's 32 rows are one scale block
                    const int nbh = M_total / Q36_QK;
#pragma unroll
                    for (int j = 0; j < 32; j++) {
                        if (c0 + j < t.nrows) {              // warp-uniform
                            const float h = silu_f(__uint_as_float(g[j])) * __uint_as_float(u[j]);
                            const uint32_t am = __reduce_max_sync(0xffffffffu, __float_as_uint(fabsf(h)));
                            const int e2 = e2_of_amax(__uint_as_float(am));
                            const size_t row = (size_t)(t.row0 + c0 + j);
                            Hq[row * M_total + blk * Q36_QK + hw_pos(lane)] = f32_to_e4m3(h * inv_scale_of_e2(e2));
                            if (lane == 0) Hs[row * nbh + blk] = (uint8_t)(127 + e2);
                        }
                    }
                } else {
                    tc_ld_wait();
#pragma unroll
                    for (int j = 0; j < 32; j++)
                        if (c0 + j < t.nrows) Y[(size_t)(t.row0 + c0 + j) * M_total + mrow] = __uint_as_float(g[j]);
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(acc_empty0 + 8 * buf);
        }
    } else {
        // --------------------------------------------------- scale loaders
        // Work items are (tile, group of 4 K-steps): one 16-byte load per operand row covers four stages.
        // The loads of the NEXT item are issued before the current item waits for its stages.
        const int i = threadIdx.x - 6 * 32;      // 0..127: row of the tile
        const int w4 = i >> 5, m0 = i & 31;
        const uint32_t my_off = m0 * 16 + w4 * 4; // byte offset of this row's word in the 32x16 B image
        const int groups = k_steps / 4;
        const uint4 ones = make_uint4(0x7f7f7f7fu, 0x7f7f7f7fu, 0x7f7f7f7fu, 0x7f7f7f7fu);
        auto fetch = [&](int ti, int kg, uint4 &a0, uint4 &a1, uint4 &b) {
            const TcTile t = get_tile(ti);
            const bool sh = t.g >= n_routed;
            const size_t arow = (size_t)(sh ? 0 : t.g) * sfA_stride + (size_t)(t.mt * TC_M + i) * nb + 16 * kg;
            a0 = __ldg(reinterpret_cast<const uint4 *>((sh ? sfS0 : sfA0) + arow));
            a1 = ones;
            if (NA == 2) a1 = __ldg(reinterpret_cast<const uint4 *>((sh ? sfS1 : sfA1) + arow));
            b = ones;
            if (i < t.nrows) b = __ldg(reinterpret_cast<const uint4 *>(sfB + (size_t)(t.row0 + i) * nb + 16 * kg));
        };
        uint32_t it = 0;
        bool ok = true;
        int ti = blockIdx.x, kg = 0;
        uint4 a0, a1, b, na0 = ones, na1 = ones, nb4 = ones;
        if (ti < n_tiles) fetch(ti, kg, a0, a1, b);
        while (ti < n_tiles && ok) {
            int nti = ti, nkg = kg + 1;
            if (nkg == groups) { nkg = 0; nti = ti + gridDim.x; }
            if (nti < n_tiles) fetch(nti, nkg, na0, na1, nb4);
            const uint32_t wa0[4] = {a0.x, a0.y, a0.z, a0.w}, wa1[4] = {a1.x, a1.y, a1.z, a1.w}, wb[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
            for (int j = 0; j < 4; j++, it++) {
                if (!ok) break;
                const int s = it % Cfg::STAGES;
                const uint32_t ph = (it / Cfg::STAGES) & 1;
                if (!(ok = mbar_wait(empty0 + 8 * s, ph ^ 1, &abort_flag, status, 0x500 + s))) break;
                uint8_t *sf = smem + s * Cfg::STAGE_BYTES + NA * Cfg::A_BYTES + Cfg::B_BYTES;
                *reinterpret_cast<uint32_t *>(sf + my_off) = wa0[j];
                if (NA == 2) *reinterpret_cast<uint32_t *>(sf + Cfg::SF_BYTES + my_off) = wa1[j];
                *reinterpret_cast<uint32_t *>(sf + NA * Cfg::SF_BYTES + my_off) = wb[j];
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                __syncwarp();
                if (lane == 0) mbar_arrive(full0 + 8 * s);
            }
            a0 = na0; a1 = na1; b = nb4; ti = nti; kg = nkg;
        }
    }

    // ------------------------------------------------------------ teardown
    tc_fence_before();
    __syncthreads();
    if (abort_flag) {
        // leave copies that may still be in flight time to land before the block retires
        for (int i = 0; i < 200; i++) __nanosleep(1000);
        if (threadIdx.x == 0) atomicCAS(status, 0, 1);
    }
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(Cfg::TMEM_COLS) : "memory");
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
// code plane of n_group experts: [n_group][M][K] 4-bit elements
static int make_map_codes(CUtensorMap *m, const void *base, int M, int K, int n_group, uint64_t expert_stride) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return Q36_MOE_ECUDA;
    cuuint64_t dims[3] = {(cuuint64_t)K, (cuuint64_t)M, (cuuint64_t)n_group};
    cuuint64_t strides[2] = {(cuuint64_t)(K / 2), (cuuint64_t)expert_stride};
    cuuint32_t box[3] = {128, TC_M, 1}, el[3] = {1, 1, 1};
    CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_16U4_ALIGN16B, 3, const_cast<void *>(base), dims, strides, box, el,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) { last_cuda_error() = 100000 + (int)r; return Q36_MOE_ECUDA; }
    return Q36_MOE_OK;
}
// activation rows: [R][K] bytes, boxes of box_rows rows x 128 B
static int make_map_rows(CUtensorMap *m, const void *base, int R, int K, int box_rows) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return Q36_MOE_ECUDA;
    cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)R};
    cuuint64_t strides[1] = {(cuuint64_t)K};
    cuuint32_t box[2] = {128, (cuuint32_t)box_rows}, el[2] = {1, 1};
    CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void *>(base), dims, strides, box, el,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) { last_cuda_error() = 100000 + (int)r; return Q36_MOE_ECUDA; }
    return Q36_MOE_OK;
}

static int sm_count() {
    static int n = 0;
    if (!n) {
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
        if (n <= 0) n = 148;
    }
    return n;
}

uint64_t tc_ws_bytes() { return (sizeof(TcPlan) + 255) & ~(uint64_t)255; }

int launch_tc_plan(const int *goffs, int n_group, const int *soffs, int D, int FF, void *plan, int *status,
                   cudaStream_t st) {
    if (n_group + 1 > DISPATCH_MAX_GROUPS) return Q36_MOE_EINVAL;
    k_tc_plan<<<1, 512, 0, st>>>(goffs, n_group, soffs, (TcPlan *)plan, FF / TC_M, D / TC_M, status);
    return check_launch();
}

// A0/A1: routed experts' planes (A1 unused for NA = 1); S0/S1: the shared expert's planes or NULL.
template <int NA>
static int run_grouped(const void *A0, const void *A1, const void *S0, const void *S1, int n_group, int R_max,
                       const uint8_t *Bq, const uint8_t *Bs, uint8_t *Hq, uint8_t *Hs, float *Y, int M, int K,
                       const void *plan, int *status, cudaStream_t st) {
    using Cfg = TcCfg<NA>;
    if (M % TC_M || K % (4 * TC_KSTEP) || n_group + 1 > DISPATCH_MAX_GROUPS) return Q36_MOE_EINVAL;
    const uint64_t estride = (uint64_t)M * (K / 2) + (uint64_t)M * (K / Q36_QK);
    const uint64_t plane = (uint64_t)M * (K / 2);
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
    static bool attr_set[3] = {false, false, false};
    if (!attr_set[NA]) {
        if (cudaFuncSetAttribute(k_grouped_mma<NA>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES) != cudaSuccess)
            return check_launch();
        attr_set[NA] = true;
    }
    const int m_tiles = M / TC_M;
    const long max_tiles = ((long)(R_max + Cfg::N - 1) / Cfg::N + n_group + 1) * m_tiles;
    const int grid = (int)min((long)sm_count(), max_tiles);
    k_grouped_mma<NA><<<grid, TC_THREADS, Cfg::SMEM_BYTES, st>>>(
        maps, (const uint8_t *)A0 + plane, (const uint8_t *)A1 + plane, estride, (const uint8_t *)S0 + plane,
        (const uint8_t *)S1 + plane, n_group, Bs, (const TcPlan *)plan, Hq, Hs, Y, M, K, status);
    return check_launch();
}

int launch_gateup_tc(const void *Wg, const void *Wu, const void *Sg, const void *Su, int n_group, int R_max,
                     const uint8_t *Xq, const uint8_t *Xs, uint8_t *Hq, uint8_t *Hs, int D, int FF, const void *plan,
                     int *status, cudaStream_t st) {
    return run_grouped<2>(Wg, Wu, Sg, Su, n_group, R_max, Xq, Xs, Hq, Hs, nullptr, FF, D, plan, status, st);
}
int launch_down_tc(const void *Wd, const void *Sd, int n_group, int R_max, const uint8_t *Hq, const uint8_t *Hs,
                   float *Y, int D, int FF, const void *plan, int *status, cudaStream_t st) {
    return run_grouped<1>(Wd, nullptr, Sd, nullptr, n_group, R_max, Hq, Hs, nullptr, nullptr, Y, D, FF, plan, status, st);
}

}  // namespace q36
