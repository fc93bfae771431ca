// Routing, deterministic dispatch and the activation quantiser.
#include <cooperative_groups.h>
#include <stdio.h>

#include "common.cuh"
#include "kernels.cuh"
#include "tc_plan.cuh"

namespace q36 {

// ---------------------------------------------------------------- router
// One warp per token row; each lane holds n_expert/32 logits in registers.
// Same selection rule as k_router_topk (q36_ops.cuh:397-431): arg-max on the
// raw logits, ties to the lower expert id, k rounds with the winner masked.
template <int PER_LANE>
__device__ __forceinline__ void route_row(const float *__restrict__ l, int k, int *idx, float *wt,
                                          float scale, int renorm, int lane) {
    float v[PER_LANE];
#pragma unroll
    for (int j = 0; j < PER_LANE; j++) v[j] = l[lane + j * 32];
    float m = -1e30f;
#pragma unroll
    for (int j = 0; j < PER_LANE; j++) m = fmaxf(m, v[j]);
    m = warp_max(m);
    float s = 0.f;
#pragma unroll
    for (int j = 0; j < PER_LANE; j++) s += expf(v[j] - m);
    s = warp_sum(s);
    float w_keep = 0.f, wsum = 0.f;  // lane r keeps the weight of round r
    for (int r = 0; r < k; r++) {
        float bm = -1e30f;
        int bj = 0;
#pragma unroll
        for (int j = 0; j < PER_LANE; j++)
            if (v[j] > bm) { bm = v[j]; bj = j; }
        // warp arg-max in two reductions: the largest value as an order-preserving integer key, then the lowest
        // expert id among the lanes that hold it (the shuffle tree this replaces was 10 dependent shuffles)
        const uint32_t bits = __float_as_uint(bm + 0.f);                         // (-0 -> +0: equal floats, equal keys)
        const uint32_t key = (bits & 0x80000000u) ? ~bits : (bits | 0x80000000u);
        const uint32_t kmax = __reduce_max_sync(0xffffffffu, key);
        const int wi = (int)__reduce_min_sync(0xffffffffu, key == kmax ? (uint32_t)(lane + bj * 32) : 0xffffffffu);
        const uint32_t vb = (kmax & 0x80000000u) ? (kmax & 0x7fffffffu) : ~kmax;
        const float wv = __uint_as_float(vb);
        const float w = expf(wv - m) / s;
        if (lane == r) { w_keep = w; idx[r] = wi; }
        wsum += w;
        if (lane == (wi & 31)) {
#pragma unroll
            for (int j = 0; j < PER_LANE; j++)
                if (j == (wi >> 5)) v[j] = -1e30f;
        }
    }
    if (lane < k) wt[lane] = renorm ? (w_keep / wsum * scale) : (w_keep * scale);
}

__global__ void k_router_topk(const float *__restrict__ logits, int n_expert, int k, int *idx,
                              float *wt, float scale, int renorm, int T, int row_stride) {
    Q36_GDS();
    const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    if (warp >= T) return;
    const float *l = logits + (size_t)warp * row_stride;
    if (n_expert == 256) route_row<8>(l, k, idx + (size_t)warp * k, wt + (size_t)warp * k, scale, renorm, lane);
    else if (n_expert == 128) route_row<4>(l, k, idx + (size_t)warp * k, wt + (size_t)warp * k, scale, renorm, lane);
    else if (n_expert == 64) route_row<2>(l, k, idx + (size_t)warp * k, wt + (size_t)warp * k, scale, renorm, lane);
    else route_row<1>(l, k, idx + (size_t)warp * k, wt + (size_t)warp * k, scale, renorm, lane);
}

// -------------------------------------------------------------- dispatch
// Stable counting sort of entry ids by expert in three launches.  Entries are
// cut into chunks of DISPATCH_CHUNK; inside a chunk warp w owns entries
// [32w, 32w+32).
//   k_dispatch_count : per (chunk, expert) counts and each entry's rank among
//                      the chunk's earlier entries of the same expert
//   k_dispatch_scan  : per expert exclusive scan over chunks, then over experts
//   k_dispatch_place : elist / pos from eoffs + chunk base + rank
// The order inside a bucket is ascending entry id, one of the orders the
// engine's atomic k_moe_dispatch (q36_engine.cu:3387-3392) can produce.
constexpr int DISPATCH_CHUNK = 1024;
constexpr int DISPATCH_MAX_E = 512;

__global__ void __launch_bounds__(DISPATCH_CHUNK)
k_dispatch_count(const int *__restrict__ eid, int n, int n_expert, int se0, int se1,
                 int *__restrict__ chunk_cnt, int *__restrict__ lrank) {
    Q36_GDS();
    __shared__ unsigned short cnt[DISPATCH_CHUNK / 32][DISPATCH_MAX_E];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    for (int i = tid; i < (DISPATCH_CHUNK / 32) * DISPATCH_MAX_E; i += blockDim.x) (&cnt[0][0])[i] = 0;
    __syncthreads();
    const int i = blockIdx.x * DISPATCH_CHUNK + tid;
    int e = -1;
    if (i < n) {
        e = eid[i];
        if (e < 0 || e < se0 || e >= se1 || e >= n_expert) e = -1;
    }
    const unsigned peers = __match_any_sync(0xffffffffu, e);
    const int r_in_warp = __popc(peers & ((1u << lane) - 1u));
    if (e >= 0 && r_in_warp == 0) cnt[warp][e] = (unsigned short)__popc(peers);
    __syncthreads();
    for (int x = tid; x < n_expert; x += blockDim.x) {
        int run = 0;
        for (int w = 0; w < DISPATCH_CHUNK / 32; w++) {
            const int c = cnt[w][x];
            cnt[w][x] = (unsigned short)run;
            run += c;
        }
        chunk_cnt[(size_t)blockIdx.x * n_expert + x] = run;
    }
    __syncthreads();
    if (i < n) lrank[i] = (e >= 0) ? (cnt[warp][e] + r_in_warp) : -1;
}

// One block of 1024 threads.  Per-chunk counts -> exclusive prefix per expert over the chunks, in passes of as many
// chunks as fit in shared memory next to each other (the count table is read and written once, coalesced: a warp per
// expert going to global memory for every step of its scan took 19 us at 32 chunks x 256 experts); then warp 0 scans
// the expert totals, and -- when a plan is wanted -- the same block writes the tensor-core work plan of the grouped
// launches, which depends on nothing else.
constexpr int SCAN_SMEM_INTS = 8192;   // 32 KB: 32 chunks x 256 experts per pass
__global__ void __launch_bounds__(1024)
k_dispatch_scan(int *__restrict__ chunk_cnt, int n_chunk, int n_expert, int *__restrict__ ecount, int *__restrict__ eoffs,
                int *__restrict__ soffs, int s0, int s1, TcPlan *plan, int se0, int se1, int mt_gu, int mt_dn, int plan_tile_rows) {
    Q36_GDS();
    __shared__ int s_eoffs[DISPATCH_MAX_E + 1];
    __shared__ int scratch[4 * (DISPATCH_MAX_GROUPS + 1)];
    __shared__ int s_tab[SCAN_SMEM_INTS];
    const int tid = threadIdx.x;
    for (int x = tid; x < n_expert; x += blockDim.x) s_eoffs[x] = 0;     // running total per expert across the passes
    __syncthreads();
    const int cpp = max(1, SCAN_SMEM_INTS / n_expert);                   // chunks per pass
    for (int c0 = 0; c0 < n_chunk; c0 += cpp) {
        const int nc = min(cpp, n_chunk - c0), cells = nc * n_expert;
        for (int i = tid; i < cells; i += blockDim.x) s_tab[i] = chunk_cnt[(size_t)c0 * n_expert + i];
        __syncthreads();
        for (int x = tid; x < n_expert; x += blockDim.x) {                // a thread per expert walks the pass's chunks
            int run = s_eoffs[x];
            for (int c = 0; c < nc; c++) {
                const int v = s_tab[c * n_expert + x];
                s_tab[c * n_expert + x] = run;
                run += v;
            }
            s_eoffs[x] = run;
        }
        __syncthreads();
        for (int i = tid; i < cells; i += blockDim.x) chunk_cnt[(size_t)c0 * n_expert + i] = s_tab[i];
        __syncthreads();
    }
    for (int x = tid; x < n_expert; x += blockDim.x) ecount[x] = s_eoffs[x];
    __syncthreads();
    if (tid < 32) {   // exclusive scan of the expert totals: lane owns a contiguous run
        const int lane = tid;
        const int per = (n_expert + 31) / 32;
        int sum = 0;
        for (int j = 0; j < per; j++) { const int x = lane * per + j; if (x < n_expert) sum += s_eoffs[x]; }
        int incl = sum;
        for (int o = 1; o < 32; o <<= 1) { const int v = __shfl_up_sync(0xffffffffu, incl, o); if (lane >= o) incl += v; }
        int run = incl - sum;
        for (int j = 0; j < per; j++) {
            const int x = lane * per + j;
            if (x < n_expert) { const int c = s_eoffs[x]; s_eoffs[x] = run; run += c; }
        }
        if (lane == 31) s_eoffs[n_expert] = run;
    }
    __syncthreads();
    for (int x = tid; x <= n_expert; x += blockDim.x) eoffs[x] = s_eoffs[x];
    if (tid == 0 && soffs) { soffs[0] = s0; soffs[1] = s1; }
    if (plan) tc_plan_block(s_eoffs + se0, se1 - se0, s1 > s0, s0, s1, plan, mt_gu, mt_dn, scratch, true, plan_tile_rows);
}

__global__ void k_dispatch_place(const int *__restrict__ eid, int n, int n_expert,
                                 const int *__restrict__ chunk_base, const int *__restrict__ lrank,
                                 const int *__restrict__ eoffs, int *__restrict__ elist,
                                 int *__restrict__ pos) {
    Q36_GDS();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const int r = lrank[i];
    if (r < 0) { pos[i] = -1; return; }
    const int e = eid[i];
    const int p = eoffs[e] + chunk_base[(size_t)(i / DISPATCH_CHUNK) * n_expert + e] + r;
    elist[p] = i;
    pos[i] = p;
}

// ------------------------------------------------------------- quantiser
// One warp per (row, 32-block), one lane per element, as k_quant_e4m3 does
// (q36_engine.cu:2412-2428).  SCATTER = false: logical order into Xq[T][K].
// SCATTER = true: hw order into every row of the sorted space the token feeds.
// one (row, 32-block) task of a warp: lane = element
__device__ __forceinline__ float quant_load(const void *__restrict__ X, bool bf16, int t, int b, int K, int lane) {
    const size_t off = (size_t)t * K + (size_t)b * Q36_QK + lane;
    return bf16 ? __bfloat162float(((const __nv_bfloat16 *)X)[off]) : ((const float *)X)[off];
}
template <bool SCATTER>
__device__ __forceinline__ void quant_task(float v, uint8_t *__restrict__ Xq, uint8_t *__restrict__ Xs, int t, int b,
                                           int K, const int *pos, int k, int shared_row0, int lane) {
    const int nb = K / Q36_QK;
    const size_t off = (size_t)t * K + (size_t)b * Q36_QK + lane;
    const float a = warp_max(fabsf(v));
    const int e2 = e2_of_amax(a);
    const uint8_t q = f32_to_e4m3(v * inv_scale_of_e2(e2));
    if (!SCATTER) {
        Xq[off] = q;
        if (lane == 0) Xs[(size_t)t * nb + b] = (uint8_t)(127 + e2);
    } else {
        // gather the block's 32 codes in hw order: lane p receives the code of
        // the element that lives at position p
        const int src = (lane & 1) ? (16 + (lane >> 1)) : (lane >> 1);
        const uint32_t qp = __shfl_sync(0xffffffffu, (uint32_t)q, src);
        // pack 4 positions per lane (lanes 0..7 hold the 32 bytes)
        uint32_t w = qp;
        w |= __shfl_down_sync(0xffffffffu, qp, 1) << 8;
        w |= __shfl_down_sync(0xffffffffu, qp, 2) << 16;
        w |= __shfl_down_sync(0xffffffffu, qp, 3) << 24;
        const uint32_t word = __shfl_sync(0xffffffffu, w, (lane & 7) * 4);
        // lane l writes word (l & 7) of destination (l >> 3), 4 destinations a pass
        const int n_dst = k + (shared_row0 >= 0 ? 1 : 0);
        for (int d0 = 0; d0 < n_dst; d0 += 4) {
            const int d = d0 + (lane >> 3);
            if (d < n_dst) {
                const int row = (d < k) ? pos[(size_t)t * k + d] : (shared_row0 + t);
                if (row >= 0) {
                    ((uint32_t *)(Xq + (size_t)row * K + (size_t)b * Q36_QK))[lane & 7] = word;
                    if ((lane & 7) == 0) Xs[(size_t)row * nb + b] = (uint8_t)(127 + e2);
                }
            }
        }
    }
}


// ------------------------------------------- quantiser, one lane per 32-block
// The same arithmetic as quant_task, laid out for rows that are scattered to several destinations: a lane
// owns a whole 32-block (64 B of bf16 or 128 B of f32 in, its amax needs no shuffle), a warp 32 consecutive
// blocks of one token row, so every destination row receives 1 KB of codes and 32 scale bytes per warp in
// full sectors.  (One warp per block writes 32 B and one scale byte per destination: at 4096 tokens the
// single-byte stores alone are 2.4 M partial-sector writes.)
struct QBlock { uint4 lo, hi; int e2; };   // the block's 32 codes in hw order (element j at 2j, j+16 at 2j+1)

template <bool BF16>
__device__ __forceinline__ QBlock quant_block_lane(const void *__restrict__ X, size_t off) {
    float v[32];
    if (BF16) {
        const uint4 *p = reinterpret_cast<const uint4 *>((const __nv_bfloat16 *)X + off);
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const uint4 u = p[i];
            const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
            for (int j = 0; j < 4; j++) {
                v[8 * i + 2 * j] = __uint_as_float(w[j] << 16);
                v[8 * i + 2 * j + 1] = __uint_as_float(w[j] & 0xffff0000u);
            }
        }
    } else {
        const float4 *p = reinterpret_cast<const float4 *>((const float *)X + off);
#pragma unroll
        for (int i = 0; i < 8; i++) {
            const float4 u = p[i];
            v[4 * i] = u.x; v[4 * i + 1] = u.y; v[4 * i + 2] = u.z; v[4 * i + 3] = u.w;
        }
    }
    float a = 0.f;
#pragma unroll
    for (int i = 0; i < 32; i++) a = fmaxf(a, fabsf(v[i]));
    QBlock r;
    r.e2 = e2_of_amax(a);
    const float inv = inv_scale_of_e2(r.e2);
    uint32_t w[8];
#pragma unroll
    for (int i = 0; i < 8; i++) {   // bytes 4i..4i+3 = elements 2i, 2i+16, 2i+1, 2i+17
        w[i] = (uint32_t)f32_to_e4m3(v[2 * i] * inv) | ((uint32_t)f32_to_e4m3(v[2 * i + 16] * inv) << 8) |
               ((uint32_t)f32_to_e4m3(v[2 * i + 1] * inv) << 16) | ((uint32_t)f32_to_e4m3(v[2 * i + 17] * inv) << 24);
    }
    r.lo = make_uint4(w[0], w[1], w[2], w[3]);
    r.hi = make_uint4(w[4], w[5], w[6], w[7]);
    return r;
}
// Lane pairs swap halves so that each of the two store instructions of a warp covers 512 contiguous bytes (whole
// sectors); a lane storing its own two halves would leave every sector half-written twice.  All 32 lanes call.
struct QStore { uint4 first, second; };   // what this lane stores at byte 64 * (lane / 2) + 16 * (lane & 1) and + 32
__device__ __forceinline__ QStore quant_block_pair(const QBlock &q, int lane) {
    const bool odd = lane & 1;
    // even lane keeps lo, gives hi; odd lane keeps hi, gives lo
    const uint4 give = odd ? q.lo : q.hi;
    uint4 got;
    got.x = __shfl_xor_sync(0xffffffffu, give.x, 1); got.y = __shfl_xor_sync(0xffffffffu, give.y, 1);
    got.z = __shfl_xor_sync(0xffffffffu, give.z, 1); got.w = __shfl_xor_sync(0xffffffffu, give.w, 1);
    QStore r;
    r.first = odd ? got : q.lo;     // block 2i:   [lo_2i | hi_2i]     <- lanes 2i, 2i+1
    r.second = odd ? q.hi : got;    // block 2i+1: [lo_2i+1 | hi_2i+1] <- lanes 2i, 2i+1
    return r;
}
// blk0 = first block of the warp's run of 32
__device__ __forceinline__ void quant_block_put(const QStore &qs, int e2, uint8_t *__restrict__ Xq, uint8_t *__restrict__ Xs,
                                                int row, int blk0, int lane, int K) {
    uint8_t *base = Xq + (size_t)row * K + (size_t)blk0 * Q36_QK + 64 * (lane >> 1) + 16 * (lane & 1);
    *reinterpret_cast<uint4 *>(base) = qs.first;
    *reinterpret_cast<uint4 *>(base + 32) = qs.second;
    Xs[(size_t)row * (K / Q36_QK) + blk0 + lane] = (uint8_t)(127 + e2);
}

// warp = (token, run of 32 blocks); K must be a multiple of 1024
template <bool BF16>
__global__ void __launch_bounds__(256)
k_quant_rows(const void *__restrict__ X, uint8_t *__restrict__ Xq, uint8_t *__restrict__ Xs, int T, int K,
             const int *__restrict__ pos, int k, int shared_row0) {
    Q36_GDS();
    const int runs = K / (32 * Q36_QK);
    const long gwarp = ((long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (gwarp >= (long)T * runs) return;
    const int t = (int)(gwarp / runs), blk = (int)(gwarp % runs) * 32 + lane;
    int rows[9];
#pragma unroll
    for (int d = 0; d < 8; d++) rows[d] = (d < k) ? pos[(size_t)t * k + d] : -1;   // (issued before the row is read)
    rows[8] = shared_row0 >= 0 ? shared_row0 + t : -1;
    const QBlock q = quant_block_lane<BF16>(X, (size_t)t * K + (size_t)blk * Q36_QK);
    const QStore qs = quant_block_pair(q, lane);
#pragma unroll
    for (int d = 0; d < 9; d++)
        if (rows[d] >= 0) quant_block_put(qs, q.e2, Xq, Xs, rows[d], blk - lane, lane, K);
}

template <bool BF16, bool SCATTER>
__global__ void k_quant_e4m3(const void *__restrict__ X, uint8_t *__restrict__ Xq,
                             uint8_t *__restrict__ Xs, int T, int K, const int *__restrict__ pos,
                             int k, int shared_row0) {
    Q36_GDS();
    const int nb = K / Q36_QK;
    const long gwarp = ((long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (gwarp >= (long)T * nb) return;
    const int t = (int)(gwarp / nb), b = (int)(gwarp % nb);
    quant_task<SCATTER>(quant_load(X, BF16, t, b, K, lane), Xq, Xs, t, b, K, pos, k, shared_row0, lane);
}

// ------------------------------------------------- fused front end, small T
// Decode-sized steps spend more time launching the five small kernels above than running them, so for
// T * k <= FRONT_MAX_ENTRIES one block does router -> dispatch -> (tensor-core work plan) in a single launch.
// Same results as the separate kernels: the same route_row, the same stable order.
constexpr int FRONT_MAX_ENTRIES = 1024;

// Block-wide stable bucketing of up to FRONT_MAX_ENTRIES entries by expert (thread i owns entry i, e = its expert
// id or anything outside [se0, se1) for "not resident"), then the tensor-core work plan.  Shared arrays come from
// the caller.  All threads of the block call; ends with every output written (no trailing barrier).
struct SortSmem {
    unsigned short cnt[FRONT_MAX_ENTRIES / 32][DISPATCH_MAX_E];   // 32 KB: per (entry warp, expert) count, then base
    int s_eoffs[DISPATCH_MAX_E + 1];
    int scratch[4 * (DISPATCH_MAX_GROUPS + 1)];
};
__device__ __forceinline__ void sort_entries_block(SortSmem &sm, int e, int n, int n_expert, int se0, int se1,
                                                   int *__restrict__ ecount, int *__restrict__ eoffs, int *__restrict__ elist,
                                                   int *__restrict__ pos, int *__restrict__ soffs, int s0, int s1, TcPlan *plan,
                                                   int mt_gu, int mt_dn, int plan_tile_rows) {
    // precondition: sm.cnt rows [0, (n + 31) / 32) are zero and a barrier separates that from this call
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int used_warps = (n + 31) / 32;          // only the warps that own entries contribute counts
    if (tid >= n || e < 0 || e < se0 || e >= se1 || e >= n_expert) e = -1;
    const unsigned peers = __match_any_sync(0xffffffffu, e);
    const int r_in_warp = __popc(peers & ((1u << lane) - 1u));
    if (e >= 0 && r_in_warp == 0) sm.cnt[warp][e] = (unsigned short)__popc(peers);
    __syncthreads();
    for (int x = tid; x < n_expert; x += blockDim.x) {
        int run = 0;
        for (int w = 0; w < used_warps; w++) {
            const int c = sm.cnt[w][x];
            sm.cnt[w][x] = (unsigned short)run;
            run += c;
        }
        ecount[x] = run;
        sm.s_eoffs[x] = run;
    }
    __syncthreads();
    if (warp == 0) {   // exclusive scan of the expert totals: lane owns a contiguous run
        const int per = (n_expert + 31) / 32;
        int sum = 0;
        for (int j = 0; j < per; j++) { const int x = lane * per + j; if (x < n_expert) sum += sm.s_eoffs[x]; }
        int incl = sum;
        for (int o = 1; o < 32; o <<= 1) { const int v = __shfl_up_sync(0xffffffffu, incl, o); if (lane >= o) incl += v; }
        int run = incl - sum;
        for (int j = 0; j < per; j++) {
            const int x = lane * per + j;
            if (x < n_expert) { const int c = sm.s_eoffs[x]; sm.s_eoffs[x] = run; run += c; }
        }
        if (lane == 31) sm.s_eoffs[n_expert] = run;
    }
    __syncthreads();
    for (int x = tid; x <= n_expert; x += blockDim.x) eoffs[x] = sm.s_eoffs[x];
    if (tid == 0 && soffs) { soffs[0] = s0; soffs[1] = s1; }
    if (tid < n) {
        if (e >= 0) {
            const int p = sm.s_eoffs[e] + sm.cnt[warp][e] + r_in_warp;
            elist[p] = tid;
            pos[tid] = p;
        } else pos[tid] = -1;
    }
    // groups here hold at most a few token tiles: ranking by size would buy nothing
    if (plan) tc_plan_block(sm.s_eoffs + se0, se1 - se0, s1 > s0, s0, s1, plan, mt_gu, mt_dn, sm.scratch, false, plan_tile_rows);
}

__global__ void __launch_bounds__(1024)
k_front_small(const float *__restrict__ logits, int n_expert, int k, float scale, int T, int row_stride, int se0, int se1,
              int *__restrict__ idx, float *__restrict__ wt, int *__restrict__ ecount, int *__restrict__ eoffs,
              int *__restrict__ elist, int *__restrict__ pos, int *__restrict__ soffs, int s0, int s1,
              TcPlan *plan, int mt_gu, int mt_dn, const void *__restrict__ X, int x_is_bf16,
              uint8_t *__restrict__ Xq, uint8_t *__restrict__ Xs, int D, int shared_row0, int plan_tile_rows) {
    Q36_GDS();
    __shared__ SortSmem sm;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, nwarp = blockDim.x >> 5;
    const int n = T * k;
    const int used_warps = (n + 31) / 32;
    for (int i = tid; i < used_warps * DISPATCH_MAX_E; i += blockDim.x) (&sm.cnt[0][0])[i] = 0;
    for (int t = warp; t < T; t += nwarp) {
        const float *l = logits + (size_t)t * row_stride;
        int *ix = idx + (size_t)t * k;
        float *w = wt + (size_t)t * k;
        if (n_expert == 256) route_row<8>(l, k, ix, w, scale, 1, lane);
        else if (n_expert == 128) route_row<4>(l, k, ix, w, scale, 1, lane);
        else if (n_expert == 64) route_row<2>(l, k, ix, w, scale, 1, lane);
        else route_row<1>(l, k, ix, w, scale, 1, lane);
    }
    __syncthreads();   // idx written by this block is visible to it after the barrier
    sort_entries_block(sm, tid < n ? idx[tid] : -1, n, n_expert, se0, se1, ecount, eoffs, elist, pos, soffs, s0, s1, plan, mt_gu,
                       mt_dn, plan_tile_rows);
    if (X) {   // decode: quantise and scatter the T rows here as well (pos[] of this block is visible after the barrier)
        __syncthreads();
        const int nbk = D / Q36_QK;
        const int ntask = T * nbk;
        for (int base = warp; base < ntask; base += 8 * nwarp) {   // eight loads in flight per lane
            float v[8];
#pragma unroll
            for (int j = 0; j < 8; j++) {
                const int task = base + j * nwarp;
                v[j] = (task < ntask) ? quant_load(X, x_is_bf16 != 0, task / nbk, task % nbk, D, lane) : 0.f;
            }
#pragma unroll
            for (int j = 0; j < 8; j++) {
                const int task = base + j * nwarp;
                if (task < ntask) quant_task<true>(v[j], Xq, Xs, task / nbk, task % nbk, D, pos, k, shared_row0, lane);
            }
        }
    }
}

// ---------------------------------------- expert-parallel: received slots -> local plan
// The slots a rank received sit in its exchange window as [world sources][cap slots][row_bytes]; source s filled
// the first count_s of its slots and then published (count_s, epoch) in hdr[s].  One block waits (bounded) for
// every source's header of this call, then buckets the valid slots by local expert and writes the work plan:
// the dispatch step of the layer applied to what arrived.  world * cap <= FRONT_MAX_ENTRIES.
__device__ __forceinline__ unsigned long long ld_acquire_sys_u64(const unsigned long long *p) {
    unsigned long long v;
    asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}
// hdr word = count | epoch << 32.  Returns the count, or -1 after `limit` polls (status receives `where`).
__device__ __forceinline__ int ep_wait_hdr(const unsigned long long *hdr, unsigned epoch, unsigned limit, int *status, int where) {
    for (unsigned i = 0; i < limit; i++) {
        const unsigned long long v = ld_acquire_sys_u64(hdr);
        if ((unsigned)(v >> 32) == epoch) return (int)(unsigned)v;
        if (i > 64) __nanosleep(i < 4096 ? 32 : 256);
    }
    atomicCAS(status, 0, where);
    return -1;
}

__global__ void __launch_bounds__(1024)
k_ep_recv_plan(const uint8_t *__restrict__ win, uint64_t off_hdr0, uint64_t off_hdr1, uint64_t off_rows0, uint64_t off_rows1,
               const int *__restrict__ ctr, int world, int cap, int row_bytes, int eid_off, unsigned limit, int *status,
               int n_expert, int se0, int se1, int *__restrict__ ecount, int *__restrict__ eoffs, int *__restrict__ elist,
               int *__restrict__ pos, int *__restrict__ soffs, int s0, int s1, TcPlan *plan, int mt_gu, int mt_dn,
               int plan_tile_rows, int *__restrict__ counts_out) {
    Q36_GDS();
    Q36_TR_BEGIN(status, 2)
    __shared__ SortSmem sm;
    __shared__ int s_cnt[64];
    const int tid = threadIdx.x;
    const int n = world * cap;
    const unsigned epoch = (unsigned)ctr[1] + 1u;   // (this rank's phase-1 call counter)
    const bool odd = epoch & 1u;
    const int used_warps = (n + 31) / 32;
    for (int i = tid; i < used_warps * DISPATCH_MAX_E; i += blockDim.x) (&sm.cnt[0][0])[i] = 0;
    if (tid < world) {
        const unsigned long long *hdr = reinterpret_cast<const unsigned long long *>(win + (odd ? off_hdr1 : off_hdr0)) + tid;
        const int c = ep_wait_hdr(hdr, epoch, limit, status, 0xB00 + tid);
        s_cnt[tid] = max(0, min(c, cap));
        counts_out[tid] = s_cnt[tid];
    }
    __syncthreads();
    int e = -1;
    if (tid < n && (tid % cap) < s_cnt[tid / cap])
        e = *reinterpret_cast<const int *>(win + (odd ? off_rows1 : off_rows0) + (size_t)tid * row_bytes + eid_off);
    sort_entries_block(sm, e, n, n_expert, se0, se1, ecount, eoffs, elist, pos, soffs, s0, s1, plan, mt_gu, mt_dn, plan_tile_rows);
    Q36_TR_END(status, 2)
}

int launch_ep_recv_plan(const void *win, uint64_t off_hdr0, uint64_t off_hdr1, uint64_t off_rows0, uint64_t off_rows1, const int *ctr,
                        int world, int cap, int row_bytes, int eid_off, unsigned limit, int *status, int n_expert, int se0, int se1,
                        int *ecount, int *eoffs, int *elist, int *pos, int *soffs, int s0, int s1, void *plan, int D, int FF,
                        int plan_tile_rows, int *counts_out, cudaStream_t st) {
    if (world * cap > FRONT_MAX_ENTRIES || world > 64 || n_expert > DISPATCH_MAX_E) return Q36_MOE_EINVAL;
    launch_k(k_ep_recv_plan, dim3(1), dim3(1024), 0, st, (const uint8_t *)win, off_hdr0, off_hdr1, off_rows0, off_rows1, ctr, world, cap,
             row_bytes, eid_off, limit, status, n_expert, se0, se1, ecount, eoffs, elist, pos, soffs, s0, s1, (TcPlan *)plan,
             FF / TC_M, D / TC_M, plan_tile_rows, counts_out);
    return check_launch();
}

int launch_front_small(const float *logits, int n_expert, int k, float scale, int T, int row_stride, int se0, int se1,
                       int *idx, float *wt, int *ecount, int *eoffs, int *elist, int *pos, int *soffs, int s0, int s1,
                       void *plan, int D, int FF, int *status, const void *X, int x_is_bf16, uint8_t *Xq, uint8_t *Xs,
                       int shared_row0, int plan_tile_rows, cudaStream_t st) {
    if (T * k > FRONT_MAX_ENTRIES || n_expert > DISPATCH_MAX_E) return Q36_MOE_EINVAL;
    (void)status;   // (sticky status words: nothing to clear here)
    launch_k(k_front_small, dim3(1), dim3(1024), 0, st, logits, n_expert, k, scale, T, row_stride, se0, se1, idx, wt,
             ecount, eoffs, elist, pos, soffs, s0, s1, (TcPlan *)plan, FF / TC_M, D / TC_M, X, x_is_bf16, Xq, Xs, D,
             shared_row0, plan_tile_rows);
    return check_launch();
}


// ----------------------------------------------- decode front end: one cluster
// At most 16 tokens (T * k <= 128 entries), all experts resident.  One thread-block cluster, one launch:
//   CTA 0        router -> stable dispatch -> work plan of the fused tensor-core kernel
//   CTAs 1..7    quantise the token rows (needs no routing result), wait at the cluster barrier for CTA 0's
//                row positions, then write every block to the k + 1 rows it feeds.
// Same results as k_front_small + k_quant_e4m3<., true>: the same route_row, the same ascending-entry order
// inside an expert's bucket, the same quantiser.
constexpr int FD_CLUSTER = 8;
constexpr int FD_THREADS = 1024;
constexpr int FD_MAX_ENTRIES = 128;
constexpr int FD_QWARPS = (FD_CLUSTER - 1) * (FD_THREADS / 32);   // one (token, run of 32 blocks) per quantising warp

__global__ void __launch_bounds__(FD_THREADS)
k_front_decode(const float *__restrict__ logits, int n_expert, int k, float scale, int T, int row_stride,
               int *__restrict__ idx, float *__restrict__ wt, int *__restrict__ ecount, int *__restrict__ eoffs,
               int *__restrict__ elist, int *__restrict__ pos, int *__restrict__ soffs, int s0, int s1, TcPlan *plan,
               int mt_gu, int mt_dn, int *status, const void *__restrict__ X, int x_is_bf16, uint8_t *__restrict__ Xq,
               uint8_t *__restrict__ Xs, int D, int shared_row0, int put_k, const EpSendArgs ep) {
    // put_k: k for the sorted row space of a single-GPU layer; 0 when only the token-order rows (shared_row0 + t)
    // are wanted, as in the expert-parallel step
    Q36_GDS();
    Q36_TR_BEGIN(status, 0)
    namespace cg = cooperative_groups;
    cg::cluster_group cluster = cg::this_cluster();
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int n = T * k;
    __shared__ int s_pos[FD_MAX_ENTRIES];          // row of every entry; CTA 0 writes it into every CTA of the cluster
    // expert-parallel: where every entry's row goes, (destination rank << 20) | slot, or -1 (beyond the capacity)
    __shared__ int s_slot[FD_MAX_ENTRIES];
    const unsigned ep_epoch = ep.peers ? (unsigned)ep.ctl[0] + 1u : 0u;
    if (cluster.block_rank() != 0) {
        // ---- quantise now (warp = token x run of 32 blocks, lane = block), place after the barrier
        // (units are dealt across the CTAs first: one SM's store path would take microseconds for all rows)
        const int runs = D / (32 * Q36_QK);
        const int unit = ((int)cluster.block_rank() - 1) + (FD_CLUSTER - 1) * warp;
        const int t = unit / runs, blk0 = (unit % runs) * 32;
        const bool mine = unit < T * runs;
        QBlock q;
        QStore qs;
        if (mine) {
            q = x_is_bf16 ? quant_block_lane<true>(X, (size_t)t * D + (size_t)(blk0 + lane) * Q36_QK)
                          : quant_block_lane<false>(X, (size_t)t * D + (size_t)(blk0 + lane) * Q36_QK);
            qs = quant_block_pair(q, lane);
        }
        cluster.sync();
        if (mine) {
            for (int d = 0; d < put_k; d++) {
                const int row = s_pos[t * k + d];
                if (row >= 0) quant_block_put(qs, q.e2, Xq, Xs, row, blk0, lane, D);
            }
            if (shared_row0 >= 0) quant_block_put(qs, q.e2, Xq, Xs, shared_row0 + t, blk0, lane, D);
            if (ep.peers) {   // the same blocks straight into the windows of the ranks that own the token's experts
                const int row_bytes = D + D / Q36_QK + 16;
                for (int d = 0; d < k; d++) {
                    const int code = s_slot[t * k + d];
                    if (code < 0) continue;
                    const int r = code >> 20, j = code & 0xfffff;
                    uint8_t *rowbase = ep.peers[r] + ((ep_epoch & 1u) ? ep.rows1 : ep.rows0) +
                                       ((size_t)(ep.slot_major ? r : ep.me) * ep.cap + j) * row_bytes;
                    quant_block_put(qs, q.e2, rowbase, rowbase + D, 0, blk0, lane, D);
                }
            }
        }
        if (ep.peers) cluster.sync();   // every CTA's remote stores before CTA 0 publishes the headers
        return;
    }
    // ---- CTA 0: route, sort, plan
    __shared__ unsigned short cnt[FD_MAX_ENTRIES / 32][DISPATCH_MAX_E];   // per (entry warp, expert): count, then base
    __shared__ int s_idx[FD_MAX_ENTRIES];
    __shared__ float s_wt[FD_MAX_ENTRIES];
    __shared__ int s_eoffs[DISPATCH_MAX_E + 1];
    __shared__ int s_wsum[FD_THREADS / 32];
    const int used_warps = (n + 31) / 32;
    if (warp < T) {
        const float *l = logits + (size_t)warp * row_stride;
        if (n_expert == 256) route_row<8>(l, k, s_idx + warp * k, s_wt + warp * k, scale, 1, lane);
        else if (n_expert == 128) route_row<4>(l, k, s_idx + warp * k, s_wt + warp * k, scale, 1, lane);
        else if (n_expert == 64) route_row<2>(l, k, s_idx + warp * k, s_wt + warp * k, scale, 1, lane);
        else route_row<1>(l, k, s_idx + warp * k, s_wt + warp * k, scale, 1, lane);
    } else {
        for (int i = tid - 32 * T; i < used_warps * DISPATCH_MAX_E; i += FD_THREADS - 32 * T) (&cnt[0][0])[i] = 0;
    }
    __syncthreads();
    int e = -1;
    if (tid < n) {
        e = s_idx[tid];
        idx[tid] = e;
        wt[tid] = s_wt[tid];
        if (e < 0 || e >= n_expert) e = -1;
    }
    int r_in_warp = 0;
    if (warp < used_warps) {
        const unsigned peers = __match_any_sync(0xffffffffu, e);
        r_in_warp = __popc(peers & ((1u << lane) - 1u));
        if (e >= 0 && r_in_warp == 0) cnt[warp][e] = (unsigned short)__popc(peers);
    }
    __syncthreads();
    // per expert: rows, and (one scan for both) rows before it | non-empty experts before it << 16
    int tot = 0;
    if (tid < n_expert) {
        for (int w = 0; w < used_warps; w++) {
            const int c = cnt[w][tid];
            cnt[w][tid] = (unsigned short)tot;
            tot += c;
        }
    }
    const int val = tot | ((tot > 0) << 16);
    int incl = val;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) { const int u = __shfl_up_sync(0xffffffffu, incl, o); if (lane >= o) incl += u; }
    if (lane == 31) s_wsum[warp] = incl;
    __syncthreads();
    int before = 0;
    for (int w = 0; w < warp; w++) before += s_wsum[w];
    const int excl = before + incl - val;
    if (tid < n_expert) {
        const int row0 = excl & 0xffff, ne = excl >> 16;
        s_eoffs[tid] = row0;
        ecount[tid] = tot;
        eoffs[tid] = row0;
        if (plan) {
            plan->row0[tid] = row0; plan->cnt[tid] = tot; plan->done[tid] = 0; plan->order[tid] = tid;
            plan->base[0][tid] = ne * mt_gu; plan->base[1][tid] = ne * mt_dn;
        }
        if (tid == n_expert - 1) {
            const int total = (excl + val) & 0xffff, ne_all = (excl + val) >> 16;
            eoffs[n_expert] = total;
            s_eoffs[n_expert] = total;
            if (soffs) { soffs[0] = s0; soffs[1] = s1; }
            if (plan) {
                const bool extra = s1 > s0;
                int G = n_expert;
                int ta = ne_all * mt_gu, tb = ne_all * mt_dn;
                if (extra) {   // the shared expert's rows are one more group: T <= 16 rows, one token tile
                    plan->row0[G] = s0; plan->cnt[G] = s1 - s0; plan->done[G] = 0; plan->order[G] = G;
                    plan->base[0][G] = ta; plan->base[1][G] = tb;
                    ta += mt_gu; tb += mt_dn;
                    G++;
                }
                plan->base[0][G] = ta; plan->base[1][G] = tb;
                plan->n_tiles[0] = ta; plan->n_tiles[1] = tb; plan->n_groups = G; plan->gu_done = 0; plan->tile_rows = 16;
            }
        }
    }
    __syncthreads();
    if (tid < n) {
        int p = -1;
        if (e >= 0) {
            p = s_eoffs[e] + cnt[warp][e] + r_in_warp;
            elist[p] = tid;
        }
        pos[tid] = p;
        for (int r = 1; r < FD_CLUSTER; r++) *cluster.map_shared_rank(&s_pos[tid], r) = p;   // no L2 round trip for the scatter
        if (ep.peers) {
            int code = -1;
            if (e >= 0) {
                const int dr = e / ep.per, j = p - s_eoffs[dr * ep.per];
                if (j < ep.cap) {
                    code = (dr << 20) | j;
                    const int row_bytes = D + D / Q36_QK + 16;
                    uint8_t *rowbase = ep.peers[dr] + ((ep_epoch & 1u) ? ep.rows1 : ep.rows0) +
                                       ((size_t)(ep.slot_major ? dr : ep.me) * ep.cap + j) * row_bytes;
                    *reinterpret_cast<int4 *>(rowbase + D + D / Q36_QK) = make_int4(e, 0, 0, 0);     // the row's tail: its expert
                    ep.ypos[tid] = dr * ep.cap + j;
                } else {
                    ep.ypos[tid] = -1;                       // beyond the window's capacity: dropped, and reported
                    if (status) atomicCAS(status, 0, 0xD00);
                }
            } else ep.ypos[tid] = -1;
            for (int r = 1; r < FD_CLUSTER; r++) *cluster.map_shared_rank(&s_slot[tid], r) = code;
        }
    }
    cluster.sync();   // (release/acquire at cluster scope: the remote stores above are visible to their CTAs)
    if (ep.peers) {
        cluster.sync();   // the quantising CTAs have stored their blocks into the peers' windows
        if (tid < ep.world) {
            const int cnt = min(ep.cap, s_eoffs[(tid + 1) * ep.per] - s_eoffs[tid * ep.per]);
            unsigned long long *h = reinterpret_cast<unsigned long long *>(ep.peers[tid] + ((ep_epoch & 1u) ? ep.hdr1 : ep.hdr0)) +
                                    (ep.slot_major ? tid : ep.me);
            const unsigned long long v = (unsigned long long)(unsigned)cnt | ((unsigned long long)ep_epoch << 32);
            asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(h), "l"(v) : "memory");
        }
        __syncthreads();
        if (tid == 0) ep.ctl[0] = (int)ep_epoch;      // phase 0 of this call is over (every CTA read the counter before the barriers above)
    }
    Q36_TR_END(status, 0)
}

// 0 when this front end applies, else the caller takes the general kernels
int launch_front_decode(const float *logits, int n_expert, int k, float scale, int T, int row_stride, int *idx, float *wt,
                        int *ecount, int *eoffs, int *elist, int *pos, int *soffs, int s0, int s1, void *plan, int D, int FF,
                        int *status, const void *X, int x_is_bf16, uint8_t *Xq, uint8_t *Xs, int shared_row0, int put_k,
                        cudaStream_t st, const EpSendArgs *ep) {
    if (T > 16 || T * k > FD_MAX_ENTRIES || n_expert > DISPATCH_MAX_E || n_expert > FD_THREADS || D % (32 * Q36_QK) ||
        T * (D / (32 * Q36_QK)) > FD_QWARPS || s1 - s0 > 16)
        return Q36_MOE_EINVAL;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(FD_CLUSTER);
    cfg.blockDim = dim3(FD_THREADS);
    cfg.stream = st;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = FD_CLUSTER;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl_enabled() ? 2 : 1;
    cudaLaunchKernelEx(&cfg, k_front_decode, logits, n_expert, k, scale, T, row_stride, idx, wt, ecount, eoffs, elist, pos,
                       soffs, s0, s1, (TcPlan *)plan, FF / TC_M, D / TC_M, status, X, x_is_bf16, Xq, Xs, D, shared_row0, put_k,
                       ep ? *ep : EpSendArgs{nullptr, 0, 0, 0, 0, nullptr, nullptr, 0, 0, 1, 0, 0});
    return check_launch();
}

// -------------------------------------------------------------- launchers
int launch_router_topk(const float *logits, int n_expert, int k, int *idx, float *wt, float scale,
                       int renorm, int T, int row_stride, cudaStream_t st) {
    if (T <= 0) return Q36_MOE_OK;
    launch_k(k_router_topk, dim3((T + 7) / 8), dim3(256), 0, st, logits, n_expert, k, idx, wt, scale, renorm, T, row_stride);
    return check_launch();
}

uint64_t dispatch_ws_bytes(int n_entries, int n_expert) {
    const uint64_t n_chunk = ((uint64_t)n_entries + DISPATCH_CHUNK - 1) / DISPATCH_CHUNK;
    return (n_chunk * n_expert + (uint64_t)n_entries) * sizeof(int) + 256;
}

int launch_dispatch(const int *eid, int n, int n_expert, int se0, int se1, int *ecount, int *eoffs,
                    int *elist, int *pos, void *ws, int *soffs, int s0, int s1, cudaStream_t st, void *plan, int D, int FF,
                    int plan_tile_rows) {
    const int n_chunk = (n + DISPATCH_CHUNK - 1) / DISPATCH_CHUNK;
    int *chunk_cnt = (int *)ws;
    int *lrank = chunk_cnt + (size_t)n_chunk * n_expert;
    if (n > 0) launch_k(k_dispatch_count, dim3(n_chunk), dim3(DISPATCH_CHUNK), 0, st, eid, n, n_expert, se0, se1, chunk_cnt, lrank);
    launch_k(k_dispatch_scan, dim3(1), dim3(1024), 0, st, chunk_cnt, n_chunk, n_expert, ecount, eoffs, soffs, s0, s1, (TcPlan *)plan,
             se0, se1, plan ? FF / TC_M : 0, plan ? D / TC_M : 0, plan_tile_rows);
    if (n > 0) launch_k(k_dispatch_place, dim3((n + 255) / 256), dim3(256), 0, st, eid, n, n_expert, chunk_cnt, lrank, eoffs, elist, pos);
    return check_launch();
}

int launch_quant(const void *X, int bf16, uint8_t *Xq, uint8_t *Xs, int T, int K, const int *pos,
                 int k, int shared_row0, bool scatter, cudaStream_t st) {
    if (T <= 0) return Q36_MOE_OK;
    const long warps = (long)T * (K / Q36_QK);
    const unsigned grid = (unsigned)((warps + 7) / 8);
    if (scatter && K % (32 * Q36_QK) == 0 && k <= 8) {
        const long w2 = (long)T * (K / (32 * Q36_QK));
        const unsigned g2 = (unsigned)((w2 + 7) / 8);
        if (bf16) launch_k(k_quant_rows<true>, dim3(g2), dim3(256), 0, st, X, Xq, Xs, T, K, pos, k, shared_row0);
        else launch_k(k_quant_rows<false>, dim3(g2), dim3(256), 0, st, X, Xq, Xs, T, K, pos, k, shared_row0);
    } else if (scatter) {
        if (bf16) launch_k(k_quant_e4m3<true, true>, dim3(grid), dim3(256), 0, st, X, Xq, Xs, T, K, pos, k, shared_row0);
        else launch_k(k_quant_e4m3<false, true>, dim3(grid), dim3(256), 0, st, X, Xq, Xs, T, K, pos, k, shared_row0);
    } else {
        if (bf16) launch_k(k_quant_e4m3<true, false>, dim3(grid), dim3(256), 0, st, X, Xq, Xs, T, K, nullptr, 0, -1);
        else launch_k(k_quant_e4m3<false, false>, dim3(grid), dim3(256), 0, st, X, Xq, Xs, T, K, nullptr, 0, -1);
    }
    return check_launch();
}

}  // namespace q36

// ------------------------------------------------- dispatch without a workspace
// Scratch of q36_moe_dispatch_noalloc: the per-(chunk, expert) counters and the per-entry ranks of the three
// dispatch kernels for at most Q36_MOE_NOALLOC_MAX_ENTRIES entries and 512 experts.  It lives in the library
// image: every GPU that loads the library carries these 96 KiB until the process exits.
static constexpr int NOALLOC_MAX_ENTRIES = 16384;
static constexpr int NOALLOC_MAX_EXPERTS = q36::DISPATCH_MAX_E;
static constexpr size_t NOALLOC_SCRATCH_INTS =
    (size_t)(NOALLOC_MAX_ENTRIES / q36::DISPATCH_CHUNK) * NOALLOC_MAX_EXPERTS + NOALLOC_MAX_ENTRIES;
static __device__ __align__(256) int g_noalloc_scratch[NOALLOC_SCRATCH_INTS];

// Device address of the array above, looked up once per device.  In host code the symbol is only a
// stand-in: kernels must be given the address cudaGetSymbolAddress returns for the CURRENT device.
static int *g_noalloc_ptr[64] = {nullptr};

extern "C" int q36_moe_dispatch_noalloc(const int *expert_of_entry, int n_entries, int n_expert, int se0, int se1,
                                        int *ecount, int *eoffs, int *elist, int *pos, void *stream) {
    if (!ecount || !eoffs || n_entries < 0) return Q36_MOE_EINVAL;
    if (n_entries > 0 && (!expert_of_entry || !elist || !pos)) return Q36_MOE_EINVAL;   // no entries: nothing to read or place
    if (n_expert <= 0 || se0 < 0 || se0 > se1 || se1 > n_expert) return Q36_MOE_EINVAL;
    if (n_entries > NOALLOC_MAX_ENTRIES || n_expert > NOALLOC_MAX_EXPERTS) {
        fprintf(stderr,
                "q36_moe_dispatch_noalloc: %d entries / %d experts exceed the built-in scratch (max %d entries, %d "
                "experts); use q36_moe_dispatch with a caller workspace\n",
                n_entries, n_expert, NOALLOC_MAX_ENTRIES, NOALLOC_MAX_EXPERTS);
        return Q36_MOE_ENOSPACE;
    }
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) { q36::last_cuda_error() = (int)e; return Q36_MOE_ECUDA; }
    if (dev < 0 || dev >= 64) {
        fprintf(stderr, "q36_moe_dispatch_noalloc: device ordinal %d is beyond the 64 this entry keeps an address for\n", dev);
        return Q36_MOE_EINVAL;
    }
    if (!g_noalloc_ptr[dev]) {   // first call on this device: resolve the array's device address
        int *p = nullptr;
        e = cudaGetSymbolAddress((void **)&p, g_noalloc_scratch);
        if (e != cudaSuccess || !p) { q36::last_cuda_error() = (int)e; return Q36_MOE_ECUDA; }
        g_noalloc_ptr[dev] = p;
    }
    // Nothing in the scratch has to start at zero: k_dispatch_count writes every counter of every chunk it
    // covers and the rank of every entry before the later kernels read them.
    return q36::launch_dispatch(expert_of_entry, n_entries, n_expert, se0, se1, ecount, eoffs, elist, pos,
                                g_noalloc_ptr[dev], nullptr, 0, 0, (cudaStream_t)stream, nullptr, 0, 0, 0);
}
