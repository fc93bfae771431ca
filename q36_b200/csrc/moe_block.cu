// The steps either side of the expert computation, so that a block can be driven from the residual stream:
//
//   before  h += a; x = rmsnorm(h) * w; logits = router_w . x
//           k_add_rmsnorm (q36_engine.cu:696-706) + k_matvec_f32_row (q36_ops.cuh:331-342) at decode,
//           k_rmsnorm_b + pf_gemm(f32 router) + pf_gemm(shared gate) when batched (q36_engine.cu:3426-3427, 3469)
//   after   moe = combine(...); h += moe; x_next = rmsnorm(h) * w_next
//           k_moe_combine(_pf) (q36_engine.cu:785-791, 3393-3401) + k_add_rmsnorm (:696-706, :1966)
//
// The router logits are f32 dot products at every batch size (the engine's batched path rounds both operands
// to fp16 for its wmma GEMM; f32 keeps decode and prefill routing identical).
#include "common.cuh"
#include "kernels.cuh"

namespace q36 {

__device__ __forceinline__ float block_sum_256(float v, float *part) {
    v = warp_sum(v);
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    if (lane == 0) part[wid] = v;
    __syncthreads();
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < 8; i++) s += part[i];   // every thread adds the eight partials in the same order
    __syncthreads();
    return s;
}

// ------------------------------------------------------------------ before
// One block per token row.  Also computes the extra logit column `gate_row` (the shared-expert gate: one more
// router row) while the normalised row is in registers.  D <= 256 * 4 * ROW_F4 floats.
constexpr int ROW_F4 = 4;   // float4 per thread: rows up to 4096 floats
__global__ void __launch_bounds__(256)
k_add_rmsnorm_rows(float *__restrict__ h, const float *__restrict__ a, const float *__restrict__ w, float eps,
                   float *__restrict__ x, const float *__restrict__ gate_row, float *__restrict__ logits, int logit_stride,
                   int gate_col, int D) {
    Q36_GDS();
    __shared__ float part[8];
    const int t = blockIdx.x, n4 = D / 4;
    float4 *hr = reinterpret_cast<float4 *>(h + (size_t)t * D);
    const float4 *ar = a ? reinterpret_cast<const float4 *>(a + (size_t)t * D) : nullptr;
    float4 v[ROW_F4];
    float loc = 0.f;
#pragma unroll
    for (int j = 0; j < ROW_F4; j++) {
        const int i = threadIdx.x + j * 256;
        v[j] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (i < n4) {
            v[j] = hr[i];
            if (ar) {
                const float4 b = ar[i];
                v[j].x += b.x; v[j].y += b.y; v[j].z += b.z; v[j].w += b.w;
                hr[i] = v[j];
            }
            loc += v[j].x * v[j].x + v[j].y * v[j].y + v[j].z * v[j].z + v[j].w * v[j].w;
        }
    }
    const float ss = rsqrtf(block_sum_256(loc, part) / (float)D + eps);
    float gdot = 0.f;
#pragma unroll
    for (int j = 0; j < ROW_F4; j++) {
        const int i = threadIdx.x + j * 256;
        if (i < n4) {
            const float4 ww = reinterpret_cast<const float4 *>(w)[i];
            float4 o;
            o.x = v[j].x * ss * ww.x; o.y = v[j].y * ss * ww.y; o.z = v[j].z * ss * ww.z; o.w = v[j].w * ss * ww.w;
            reinterpret_cast<float4 *>(x + (size_t)t * D)[i] = o;
            if (gate_row) {
                const float4 g = reinterpret_cast<const float4 *>(gate_row)[i];
                gdot += o.x * g.x + o.y * g.y + o.z * g.z + o.w * g.w;
            }
        }
    }
    if (gate_row) {
        gdot = block_sum_256(gdot, part);
        if (threadIdx.x == 0) logits[(size_t)t * logit_stride + gate_col] = gdot;
    }
}

// Router logits for a handful of tokens: one warp per router row, the row read once and used for every token.
// T <= 16.  x rows come from L2 (T * D * 4 bytes, written by the kernel before).
constexpr int RL_T = 16;
__global__ void __launch_bounds__(128)
k_router_logits_small(const float *__restrict__ W, const float *__restrict__ x, float *__restrict__ logits, int logit_stride,
                      int n_rows, int T, int D) {
    Q36_GDS();
    const int row = blockIdx.x * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (row >= n_rows) return;
    const float4 *wr = reinterpret_cast<const float4 *>(W + (size_t)row * D);
    float acc[RL_T];
#pragma unroll
    for (int t = 0; t < RL_T; t++) acc[t] = 0.f;
    for (int i = lane; i < D / 4; i += 32) {
        const float4 ww = wr[i];
#pragma unroll
        for (int t = 0; t < RL_T; t++) {
            if (t < T) {
                const float4 xv = reinterpret_cast<const float4 *>(x + (size_t)t * D)[i];
                acc[t] += ww.x * xv.x + ww.y * xv.y + ww.z * xv.z + ww.w * xv.w;
            }
        }
    }
#pragma unroll
    for (int t = 0; t < RL_T; t++) {
        if (t < T) {
            const float s = warp_sum(acc[t]);
            if (lane == 0) logits[(size_t)t * logit_stride + row] = s;
        }
    }
}

// Router logits for a batch: logits[t][r] = x[t][:] . W[r][:], f32 FMA, 128 tokens x 64 rows per block, K in chunks
// of 16 through shared memory (register-prefetched), 8 x 4 outputs per thread.
constexpr int RG_BT = 128, RG_BR = 64, RG_BK = 16;
__global__ void __launch_bounds__(256)
k_router_logits_gemm(const float *__restrict__ W, const float *__restrict__ x, float *__restrict__ logits, int logit_stride,
                     int n_rows, int T, int D) {
    Q36_GDS();
    __shared__ float sx[RG_BK][RG_BT + 4];   // [k][token]
    __shared__ float sw[RG_BK][RG_BR + 4];   // [k][row]
    const int t0 = blockIdx.y * RG_BT, r0 = blockIdx.x * RG_BR, tid = threadIdx.x;
    const int tx = tid & 15, ty = tid >> 4;   // thread tile: tokens ty * 8 .. + 8, rows tx * 4 .. + 4
    // loaders: x tile 128 x 16 floats = 512 float4 (2 per thread), W tile 64 x 16 = 256 float4 (1 per thread)
    const int lx_t = tid >> 2, lx_k = (tid & 3) * 4;          // tokens lx_t and lx_t + 64
    const int lw_r = tid >> 2, lw_k = (tid & 3) * 4;
    float4 px0, px1, pw;
    auto fetch = [&](int k0) {
        const int ta = t0 + lx_t, tb = ta + 64, r = r0 + lw_r;
        px0 = (ta < T) ? *reinterpret_cast<const float4 *>(x + (size_t)ta * D + k0 + lx_k) : make_float4(0.f, 0.f, 0.f, 0.f);
        px1 = (tb < T) ? *reinterpret_cast<const float4 *>(x + (size_t)tb * D + k0 + lx_k) : make_float4(0.f, 0.f, 0.f, 0.f);
        pw = (r < n_rows) ? *reinterpret_cast<const float4 *>(W + (size_t)r * D + k0 + lw_k) : make_float4(0.f, 0.f, 0.f, 0.f);
    };
    auto stash = [&]() {
        sx[lx_k][lx_t] = px0.x; sx[lx_k + 1][lx_t] = px0.y; sx[lx_k + 2][lx_t] = px0.z; sx[lx_k + 3][lx_t] = px0.w;
        sx[lx_k][lx_t + 64] = px1.x; sx[lx_k + 1][lx_t + 64] = px1.y; sx[lx_k + 2][lx_t + 64] = px1.z; sx[lx_k + 3][lx_t + 64] = px1.w;
        sw[lw_k][lw_r] = pw.x; sw[lw_k + 1][lw_r] = pw.y; sw[lw_k + 2][lw_r] = pw.z; sw[lw_k + 3][lw_r] = pw.w;
    };
    float acc[8][4];
#pragma unroll
    for (int i = 0; i < 8; i++)
#pragma unroll
        for (int j = 0; j < 4; j++) acc[i][j] = 0.f;
    fetch(0);
    for (int k0 = 0; k0 < D; k0 += RG_BK) {
        stash();
        __syncthreads();
        if (k0 + RG_BK < D) fetch(k0 + RG_BK);
#pragma unroll
        for (int kk = 0; kk < RG_BK; kk++) {
            const float4 xa = *reinterpret_cast<const float4 *>(&sx[kk][ty * 8]);
            const float4 xb = *reinterpret_cast<const float4 *>(&sx[kk][ty * 8 + 4]);
            const float4 wv = *reinterpret_cast<const float4 *>(&sw[kk][tx * 4]);
            const float xs[8] = {xa.x, xa.y, xa.z, xa.w, xb.x, xb.y, xb.z, xb.w};
            const float ws[4] = {wv.x, wv.y, wv.z, wv.w};
#pragma unroll
            for (int i = 0; i < 8; i++)
#pragma unroll
                for (int j = 0; j < 4; j++) acc[i][j] = fmaf(xs[i], ws[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 8; i++) {
        const int t = t0 + ty * 8 + i;
        if (t >= T) continue;
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const int r = r0 + tx * 4 + j;
            if (r < n_rows) logits[(size_t)t * logit_stride + r] = acc[i][j];
        }
    }
}

// ------------------------------------------------------------------- after
// One block per token: the weighted combine in slot order (as k_combine), then the residual add and the next
// RMSNorm while the row is in registers.  EARLY_META: see k_combine (moe_gemv.cu).
template <bool EARLY_META>
__global__ void __launch_bounds__(256)
k_combine_add_rmsnorm(float *__restrict__ moe_out, const float *__restrict__ Y, const int *__restrict__ pos,
                      const float *__restrict__ wt, const float *__restrict__ SH, const float *__restrict__ shgate,
                      int shgate_stride, float *__restrict__ h, const float *__restrict__ w_next, float eps,
                      float *__restrict__ x_next, int D, int k, int y_bf16) {
    if (!EARLY_META) Q36_GDS();
    else cudaTriggerProgrammaticLaunchCompletion();
    __shared__ float part[8];
    const int t = blockIdx.x, n4 = D / 4;
    constexpr int KMAX = 8;
    int p[KMAX];
    float wgt[KMAX];
#pragma unroll
    for (int s = 0; s < KMAX; s++) {
        p[s] = (s < k) ? pos[(size_t)t * k + s] : -1;
        wgt[s] = (s < k) ? wt[(size_t)t * k + s] : 0.f;
    }
    const float gs = (SH && shgate) ? sigm_f(shgate[(size_t)t * shgate_stride]) : 1.f;
    if (EARLY_META) cudaGridDependencySynchronize();
    float4 acc[ROW_F4];
    float loc = 0.f;
#pragma unroll
    for (int j = 0; j < ROW_F4; j++) {
        const int i = threadIdx.x + j * 256;
        acc[j] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (i >= n4) continue;
        float4 y[KMAX];
        float4 ysh = make_float4(0.f, 0.f, 0.f, 0.f);
        if (SH) ysh = ld_y4(SH, (size_t)t * D + 4 * (size_t)i, y_bf16);
#pragma unroll
        for (int s = 0; s < KMAX; s++)
            y[s] = (p[s] >= 0) ? ld_y4(Y, (size_t)p[s] * D + 4 * (size_t)i, y_bf16) : make_float4(0.f, 0.f, 0.f, 0.f);
        const float4 hv = reinterpret_cast<const float4 *>(h + (size_t)t * D)[i];
        float4 m = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int s = 0; s < KMAX; s++) {
            if (p[s] < 0) continue;
            m.x = fmaf(wgt[s], y[s].x, m.x); m.y = fmaf(wgt[s], y[s].y, m.y);
            m.z = fmaf(wgt[s], y[s].z, m.z); m.w = fmaf(wgt[s], y[s].w, m.w);
        }
        if (SH) { m.x = fmaf(gs, ysh.x, m.x); m.y = fmaf(gs, ysh.y, m.y); m.z = fmaf(gs, ysh.z, m.z); m.w = fmaf(gs, ysh.w, m.w); }
        if (moe_out) reinterpret_cast<float4 *>(moe_out + (size_t)t * D)[i] = m;
        float4 r = make_float4(hv.x + m.x, hv.y + m.y, hv.z + m.z, hv.w + m.w);
        reinterpret_cast<float4 *>(h + (size_t)t * D)[i] = r;
        acc[j] = r;
        loc += r.x * r.x + r.y * r.y + r.z * r.z + r.w * r.w;
    }
    const float ss = rsqrtf(block_sum_256(loc, part) / (float)D + eps);
#pragma unroll
    for (int j = 0; j < ROW_F4; j++) {
        const int i = threadIdx.x + j * 256;
        if (i >= n4) continue;
        const float4 ww = reinterpret_cast<const float4 *>(w_next)[i];
        float4 o;
        o.x = acc[j].x * ss * ww.x; o.y = acc[j].y * ss * ww.y; o.z = acc[j].z * ss * ww.z; o.w = acc[j].w * ss * ww.w;
        reinterpret_cast<float4 *>(x_next + (size_t)t * D)[i] = o;
    }
}

// ---------------------------------------------------------------- launchers
int launch_pre_norm_router(float *h, const float *a, const float *norm_w, float eps, const float *router_w, int n_rows,
                           int gate_row, float *x, float *logits, int logit_stride, int T, int D, cudaStream_t st) {
    if (T <= 0) return Q36_MOE_OK;
    if (D % 4 || D > 256 * 4 * ROW_F4 || n_rows <= 0 || logit_stride < n_rows) return Q36_MOE_EINVAL;
    // the shared-gate row (one extra router row) is taken by the norm kernel itself when batched; the decode-sized
    // logits kernel reads every row once for all tokens and takes it along
    const bool small = T <= RL_T;
    const float *gate = (!small && gate_row >= 0) ? router_w + (size_t)gate_row * D : nullptr;
    launch_k(k_add_rmsnorm_rows, dim3(T), dim3(256), 0, st, h, a, norm_w, eps, x, gate, logits, logit_stride, gate_row, D);
    if (small) {
        launch_k(k_router_logits_small, dim3((n_rows + 3) / 4), dim3(128), 0, st, router_w, (const float *)x, logits, logit_stride,
                 n_rows, T, D);
    } else {
        if (D % RG_BK) return Q36_MOE_EINVAL;
        const int rows = (gate_row == n_rows - 1) ? n_rows - 1 : n_rows;   // the gate row is done already when it is the last one
        if (gate_row >= 0 && gate_row != n_rows - 1) return Q36_MOE_EINVAL;
        launch_k(k_router_logits_gemm, dim3((rows + RG_BR - 1) / RG_BR, (T + RG_BT - 1) / RG_BT), dim3(256), 0, st, router_w,
                 (const float *)x, logits, logit_stride, rows, T, D);
    }
    return check_launch();
}

int launch_combine_add_rmsnorm(float *moe_out, const float *Y, const int *pos, const float *wt, const float *SH,
                               const float *shgate, int shgate_stride, float *h, const float *w_next, float eps, float *x_next,
                               int D, int k, int T, bool early_meta, cudaStream_t st, int y_bf16) {
    if (T <= 0) return Q36_MOE_OK;
    if (k <= 0 || k > 8 || D % 4 || D > 256 * 4 * ROW_F4) return Q36_MOE_EINVAL;
    if (early_meta)
        launch_k(k_combine_add_rmsnorm<true>, dim3(T), dim3(256), 0, st, moe_out, Y, pos, wt, SH, shgate, shgate_stride, h, w_next,
                 eps, x_next, D, k, y_bf16);
    else
        launch_k(k_combine_add_rmsnorm<false>, dim3(T), dim3(256), 0, st, moe_out, Y, pos, wt, SH, shgate, shgate_stride, h, w_next,
                 eps, x_next, D, k, y_bf16);
    return check_launch();
}

}  // namespace q36
