// Decode-sized expert groups: streaming GEMV over the MXFP4 split planes.
//
// One lane owns one 32-element block of a weight row per step: a single
// 16-byte load brings the block's 32 codes, coalesced across the warp (512 B
// per row per warp-load).  Every lane keeps eight such loads in flight (eight
// rows), which is what hides DRAM latency when the whole grid is about one
// wave (the finding recorded at q36_ops.cuh:184-188).  Codes are expanded by
// the hardware E2M1 converter, activations (E4M3, hw order) sit in registers,
// accumulation is fp32, the block scales are applied once per block, and the
// row sum is a warp-shuffle reduction.
#include "common.cuh"
#include "kernels.cuh"

namespace q36 {

// 32 activations of one block for one token: 32 B of E4M3 -> 32 f32 registers.
__device__ __forceinline__ void load_x_block(const uint8_t *__restrict__ p, float (&x)[32]) {
    const uint4 a = *reinterpret_cast<const uint4 *>(p);
    const uint4 b = *reinterpret_cast<const uint4 *>(p + 16);
    const uint32_t w[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
#pragma unroll
    for (int i = 0; i < 8; i++) {
        const float2 lo = e4m3x2_to_f32x2((uint16_t)(w[i] & 0xffffu));
        const float2 hi = e4m3x2_to_f32x2((uint16_t)(w[i] >> 16));
        x[4 * i + 0] = lo.x; x[4 * i + 1] = lo.y; x[4 * i + 2] = hi.x; x[4 * i + 3] = hi.y;
    }
}

// dot of one weight block (16 code bytes) with NT activation blocks
template <int NT>
__device__ __forceinline__ void block_dot(const uint4 q, const float (&x)[NT][32], float (&part)[NT]) {
    const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
    for (int t = 0; t < NT; t++) part[t] = 0.f;
#pragma unroll
    for (int i = 0; i < 4; i++) {
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const float2 wv = e2m1x2_to_f32x2((w[i] >> (8 * j)) & 0xffu);
            const int p = 8 * i + 2 * j;  // hw positions of code byte 4i+j
#pragma unroll
            for (int t = 0; t < NT; t++) part[t] = fmaf(wv.y, x[t][p + 1], fmaf(wv.x, x[t][p], part[t]));
        }
    }
}

// ---------------------------------------------------------------- gate/up
// grid (FF/32, groups).  A block owns 32 consecutive ff indices of one group:
// warp w the ff rows 4w..4w+3 of BOTH gate and up (8 weight rows), so SwiGLU
// and the E4M3 requantisation of the 32-block finish inside the block.
// Replaces k_expert_gemv2 + k_silu_mul_slots (q36_engine.cu:752-783, 744-746).
template <int NT>
__device__ __forceinline__ void gateup_chunk(const uint8_t *__restrict__ wg, const uint8_t *__restrict__ wu,
                                             const uint8_t *__restrict__ Xq, const uint8_t *__restrict__ Xs,
                                             uint8_t *__restrict__ Hq, uint8_t *__restrict__ Hs, int D, int FF,
                                             int row0, int ff0, float (*hbuf)[32]) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int nb = D / Q36_QK;
    const size_t plane = (size_t)FF * (D / 2);
    float acc[8][NT];
#pragma unroll
    for (int r = 0; r < 8; r++)
#pragma unroll
        for (int t = 0; t < NT; t++) acc[r][t] = 0.f;
    for (int b = lane; b < nb; b += 32) {
        uint4 q[8];
        uint32_t s[8];
#pragma unroll
        for (int r = 0; r < 8; r++) {
            const uint8_t *base = (r < 4) ? wg : wu;
            const int row = ff0 + 4 * warp + (r & 3);
            q[r] = __ldg(reinterpret_cast<const uint4 *>(base + (size_t)row * (D / 2) + (size_t)b * 16));
            s[r] = __ldg(base + plane + (size_t)row * nb + b);
        }
        float x[NT][32];
        float xsc[NT];
#pragma unroll
        for (int t = 0; t < NT; t++) {
            load_x_block(Xq + (size_t)(row0 + t) * D + (size_t)b * Q36_QK, x[t]);
            xsc[t] = ue8m0_to_f32(Xs[(size_t)(row0 + t) * nb + b]);
        }
#pragma unroll
        for (int r = 0; r < 8; r++) {
            float part[NT];
            block_dot<NT>(q[r], x, part);
            const float ws = ue8m0_to_f32(s[r]);
#pragma unroll
            for (int t = 0; t < NT; t++) acc[r][t] = fmaf(part[t], ws * xsc[t], acc[r][t]);
        }
    }
#pragma unroll
    for (int r = 0; r < 8; r++)
#pragma unroll
        for (int t = 0; t < NT; t++) acc[r][t] = warp_sum(acc[r][t]);
    if (lane == 0) {
#pragma unroll
        for (int t = 0; t < NT; t++)
#pragma unroll
            for (int r = 0; r < 4; r++) hbuf[t][4 * warp + r] = silu_f(acc[r][t]) * acc[r + 4][t];
    }
    __syncthreads();
    if (warp < NT) {  // warp t requantises token t's 32-block (k_quant_e4m3 rule)
        const float v = hbuf[warp][lane];
        const int e2 = e2_of_amax(warp_max(fabsf(v)));
        const size_t row = (size_t)(row0 + warp);
        Hq[row * FF + ff0 + hw_pos(lane)] = f32_to_e4m3(v * inv_scale_of_e2(e2));
        if (lane == 0) Hs[row * (FF / Q36_QK) + ff0 / Q36_QK] = (uint8_t)(127 + e2);
    }
    __syncthreads();
}

__global__ void __launch_bounds__(256)
k_gateup_gemv(const uint8_t *__restrict__ Wg, const uint8_t *__restrict__ Wu, int n_group,
              const int *__restrict__ goffs, const uint8_t *__restrict__ Sg,
              const uint8_t *__restrict__ Su, const int *__restrict__ soffs,
              const uint8_t *__restrict__ Xq,
              const uint8_t *__restrict__ Xs, uint8_t *__restrict__ Hq, uint8_t *__restrict__ Hs,
              int D, int FF) {
    Q36_GDS();
    __shared__ float hbuf[2][32];
    const int g = blockIdx.y;
    const bool extra = g >= n_group;              // the shared expert's group
    const int r0 = extra ? soffs[0] : goffs[g];
    const int n = (extra ? soffs[1] : goffs[g + 1]) - r0;
    if (n <= 0) return;
    const size_t stride = (size_t)FF * (D / 2) + (size_t)FF * (D / Q36_QK);
    const uint8_t *wg = extra ? Sg : Wg + (size_t)g * stride, *wu = extra ? Su : Wu + (size_t)g * stride;
    const int ff0 = blockIdx.x * 32;
    int c = 0;
    for (; c + 2 <= n; c += 2) gateup_chunk<2>(wg, wu, Xq, Xs, Hq, Hs, D, FF, r0 + c, ff0, hbuf);
    if (c < n) gateup_chunk<1>(wg, wu, Xq, Xs, Hq, Hs, D, FF, r0 + c, ff0, hbuf);
}

// -------------------------------------------------------------------- down
// grid (D/128, groups).  K = FF has only FF/32 blocks per row, so a warp reads
// 32/(FF/32) rows per step (lane -> (row, block)); 8 steps cover 16 rows per
// warp at FF = 512, 128 rows per block.  Replaces k_expert_gemv
// (q36_engine.cu:711-742), with the E4M3 intermediate as input.
template <int NT>
__device__ __forceinline__ void down_chunk(const uint8_t *__restrict__ wd, const uint8_t *__restrict__ Hq,
                                           const uint8_t *__restrict__ Hs, float *__restrict__ Y, int D, int FF,
                                           int row0, int j0, float (*ybuf)[128]) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int nb = FF / Q36_QK;           // blocks per row (16)
    const int rows_per_step = 32 / nb;    // 2
    const int b = lane % nb, sub = lane / nb;
    const size_t plane = (size_t)D * (FF / 2);
    uint4 q[8];
    uint32_t s[8];
#pragma unroll
    for (int r = 0; r < 8; r++) {
        const int row = j0 + warp * 8 * rows_per_step + r * rows_per_step + sub;
        q[r] = __ldg(reinterpret_cast<const uint4 *>(wd + (size_t)row * (FF / 2) + (size_t)b * 16));
        s[r] = __ldg(wd + plane + (size_t)row * nb + b);
    }
    float x[NT][32];
    float xsc[NT];
#pragma unroll
    for (int t = 0; t < NT; t++) {
        load_x_block(Hq + (size_t)(row0 + t) * FF + (size_t)b * Q36_QK, x[t]);
        xsc[t] = ue8m0_to_f32(Hs[(size_t)(row0 + t) * nb + b]);
    }
#pragma unroll
    for (int r = 0; r < 8; r++) {
        float part[NT];
        block_dot<NT>(q[r], x, part);
        const float ws = ue8m0_to_f32(s[r]);
#pragma unroll
        for (int t = 0; t < NT; t++) {
            float v = part[t] * (ws * xsc[t]);
            for (int o = nb / 2; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
            if (b == 0) ybuf[t][warp * 8 * rows_per_step + r * rows_per_step + sub] = v;
        }
    }
    __syncthreads();
    for (int i = threadIdx.x; i < NT * 128; i += blockDim.x) {
        const int t = i >> 7, j = i & 127;
        Y[(size_t)(row0 + t) * D + j0 + j] = ybuf[t][j];
    }
    __syncthreads();
}

__global__ void __launch_bounds__(256)
k_down_gemv(const uint8_t *__restrict__ Wd, int n_group, const int *__restrict__ goffs,
            const uint8_t *__restrict__ Sd, const int *__restrict__ soffs,
            const uint8_t *__restrict__ Hq, const uint8_t *__restrict__ Hs, float *__restrict__ Y,
            int D, int FF) {
    Q36_GDS();
    __shared__ float ybuf[2][128];
    const int g = blockIdx.y;
    const bool extra = g >= n_group;
    const int r0 = extra ? soffs[0] : goffs[g];
    const int n = (extra ? soffs[1] : goffs[g + 1]) - r0;
    if (n <= 0) return;
    const size_t stride = (size_t)D * (FF / 2) + (size_t)D * (FF / Q36_QK);
    const uint8_t *wd = extra ? Sd : Wd + (size_t)g * stride;
    const int j0 = blockIdx.x * 128;
    int c = 0;
    for (; c + 2 <= n; c += 2) down_chunk<2>(wd, Hq, Hs, Y, D, FF, r0 + c, j0, ybuf);
    if (c < n) down_chunk<1>(wd, Hq, Hs, Y, D, FF, r0 + c, j0, ybuf);
}

// ----------------------------------------------------------------- combine
// k_moe_combine / k_moe_combine_pf (q36_engine.cu:785-791, 3393-3401): slot
// order, fp32.  grid (D/1024, T), 256 threads x float4.
// EARLY_META: the row positions, weights and gate logits are read BEFORE the grid dependency resolves.  Only
// for a launch whose predecessor in the stream (a) does not write them and (b) lets its successor start only
// after it has itself seen the kernel that wrote them complete -- the decode kernel, which synchronises on its
// own dependency before it signals its successor.  It takes one memory latency off a kernel that is nothing else.
template <bool EARLY_META>
__global__ void __launch_bounds__(256)
k_combine(float *__restrict__ out, const float *__restrict__ Y, const int *__restrict__ pos,
          const float *__restrict__ wt, const float *__restrict__ SH, const float *__restrict__ shgate,
          int shgate_stride, int D, int k, int y_bf16) {
    if (!EARLY_META) Q36_GDS();
    else cudaTriggerProgrammaticLaunchCompletion();
    const int t = blockIdx.y;
    const int i = (blockIdx.x * blockDim.x + threadIdx.x) * 4;
    if (i >= D) return;
    // All row positions, then all rows, are fetched before the first add: a loop that loads pos -> row -> adds
    // pays two dependent memory latencies per slot, which at decode sizes is the whole kernel.  The sum itself
    // keeps the slot order.
    constexpr int KMAX = 8;
    int p[KMAX];
    float w[KMAX];
    float4 y[KMAX];
#pragma unroll
    for (int s = 0; s < KMAX; s++) {
        p[s] = (s < k) ? pos[(size_t)t * k + s] : -1;
        w[s] = (s < k) ? wt[(size_t)t * k + s] : 0.f;
    }
    const float gs = (SH && shgate) ? sigm_f(shgate[(size_t)t * shgate_stride]) : 1.f;
    if (EARLY_META) cudaGridDependencySynchronize();
    float4 ysh = make_float4(0.f, 0.f, 0.f, 0.f);
    if (SH) ysh = ld_y4(SH, (size_t)t * D + i, y_bf16);
#pragma unroll
    for (int s = 0; s < KMAX; s++)
        y[s] = (p[s] >= 0) ? ld_y4(Y, (size_t)p[s] * D + i, y_bf16) : make_float4(0.f, 0.f, 0.f, 0.f);
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int s = 0; s < KMAX; s++) {
        if (p[s] < 0) continue;
        acc.x = fmaf(w[s], y[s].x, acc.x); acc.y = fmaf(w[s], y[s].y, acc.y);
        acc.z = fmaf(w[s], y[s].z, acc.z); acc.w = fmaf(w[s], y[s].w, acc.w);
    }
    if (SH) {
        acc.x = fmaf(gs, ysh.x, acc.x); acc.y = fmaf(gs, ysh.y, acc.y);
        acc.z = fmaf(gs, ysh.z, acc.z); acc.w = fmaf(gs, ysh.w, acc.w);
    }
    *reinterpret_cast<float4 *>(out + (size_t)t * D + i) = acc;
}

// dst row i = src row index[i] (16-byte units); negative index -> zeros
__global__ void k_gather_rows(const uint4 *__restrict__ src, const int *__restrict__ index,
                              uint4 *__restrict__ dst, int n_rows, int row_u4) {
    Q36_GDS();
    const long i = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (long)n_rows * row_u4) return;
    const int r = (int)(i / row_u4), c = (int)(i % row_u4);
    const int s = index[r];
    dst[i] = (s >= 0) ? src[(size_t)s * row_u4 + c] : make_uint4(0, 0, 0, 0);
}

// split planes -> f32 rows: thread per 32-block (q36_dequant.cuh:106-113 on device)
__global__ void k_dequant_mxfp4(const uint8_t *__restrict__ W, int M, int K, float *__restrict__ out) {
    Q36_GDS();
    const long i = (long)blockIdx.x * blockDim.x + threadIdx.x;
    const int nb = K / Q36_QK;
    if (i >= (long)M * nb) return;
    const uint4 q = *reinterpret_cast<const uint4 *>(W + (size_t)i * 16);
    const float d = ue8m0_to_f32(W[(size_t)M * (K / 2) + i]);
    const uint32_t w[4] = {q.x, q.y, q.z, q.w};
    float *o = out + (size_t)i * Q36_QK;
#pragma unroll
    for (int j = 0; j < 16; j++) {
        const float2 v = e2m1x2_to_f32x2((w[j >> 2] >> (8 * (j & 3))) & 0xffu);
        o[j] = v.x * d + 0.f;        // "+ 0" turns the -0 of code 8 into the +0 the integer table gives
        o[j + 16] = v.y * d + 0.f;
    }
}

// ---------------------------------------------------------------- launchers
int launch_gateup_gemv(const void *Wg, const void *Wu, int n_group, const int *goffs, const void *Sg,
                       const void *Su, const int *soffs, const uint8_t *Xq, const uint8_t *Xs,
                       uint8_t *Hq, uint8_t *Hs, int D, int FF, cudaStream_t st) {
    const int groups = n_group + (Sg ? 1 : 0);
    if (groups <= 0) return Q36_MOE_OK;
    if (FF % 32 || D % 32) return Q36_MOE_EINVAL;
    dim3 grid(FF / 32, groups);
    launch_k(k_gateup_gemv, dim3(grid), dim3(256), 0, st, (const uint8_t *)Wg, (const uint8_t *)Wu, n_group, goffs,
                                        (const uint8_t *)Sg, (const uint8_t *)Su, soffs, Xq, Xs, Hq, Hs, D, FF);
    return check_launch();
}
int launch_down_gemv(const void *Wd, int n_group, const int *goffs, const void *Sd, const int *soffs,
                     const uint8_t *Hq, const uint8_t *Hs, float *Y, int D, int FF, cudaStream_t st) {
    const int groups = n_group + (Sd ? 1 : 0);
    if (groups <= 0) return Q36_MOE_OK;
    if (FF != 512 || D % 128) return Q36_MOE_EINVAL;   // lane -> (row, block) map below assumes 16 blocks per row
    dim3 grid(D / 128, groups);
    launch_k(k_down_gemv, dim3(grid), dim3(256), 0, st, (const uint8_t *)Wd, n_group, goffs, (const uint8_t *)Sd, soffs, Hq, Hs, Y, D, FF);
    return check_launch();
}
int launch_combine(float *out, const float *Y, const int *pos, const float *wt, const float *SH,
                   const float *shgate, int shgate_stride, int D, int k, int T, bool early_meta, cudaStream_t st, int y_bf16) {
    if (T <= 0) return Q36_MOE_OK;
    if (k <= 0 || k > 8) return Q36_MOE_EINVAL;   // the kernel keeps one row per slot in registers
    dim3 grid((D / 4 + 255) / 256, T);
    if (early_meta) launch_k(k_combine<true>, dim3(grid), dim3(256), 0, st, out, Y, pos, wt, SH, shgate, shgate_stride, D, k, y_bf16);
    else launch_k(k_combine<false>, dim3(grid), dim3(256), 0, st, out, Y, pos, wt, SH, shgate, shgate_stride, D, k, y_bf16);
    return check_launch();
}
int launch_gather_rows(const void *src, const int *index, void *dst, int n_rows, int row_bytes,
                       cudaStream_t st) {
    if (n_rows <= 0) return Q36_MOE_OK;
    const int row_u4 = row_bytes / 16;
    const long n = (long)n_rows * row_u4;
    launch_k(k_gather_rows, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, st, (const uint4 *)src, index, (uint4 *)dst, n_rows, row_u4);
    return check_launch();
}
int launch_dequant_mxfp4(const void *W, int M, int K, float *out, cudaStream_t st) {
    const long n = (long)M * (K / Q36_QK);
    launch_k(k_dequant_mxfp4, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, st, (const uint8_t *)W, M, K, out);
    return check_launch();
}

}  // namespace q36
