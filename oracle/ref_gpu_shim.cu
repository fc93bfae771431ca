// Launchers over the reference's OWN device code for the routing, SwiGLU, RMSNorm, router-matvec and MXFP4
// dot-product kernels (q36_ops.cuh), compiled for sm_100a from where the header lies in the reference tree
// (never copied into this repository) by oracle/Makefile into oracle/_ref/libq36ref_gpu.so.
// TEST INFRASTRUCTURE ONLY: the GPU parity tests run these kernels beside the library's and compare.
// The kernels used here contain no instruction that is specific to the reference's own target.
#include <cuda_runtime.h>
#include <stdint.h>
#include "q36.h"
#include "q36_ops.cuh"

// one warp per (row, token): y[t][r] = dot_mxfp4_split(row r of the split planes, x[t])  (q36_ops.cuh:167-187)
__global__ void ref_k_dot_mxfp4_split(const uint8_t *qs, const uint8_t *es, const float *x, float *y, int M, int K, int T) {
    const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    if (warp >= M * T) return;
    const int t = warp / M, r = warp % M;
    const float acc = dot_mxfp4_split(qs + (size_t)r * (K / 2), es + (size_t)r * (K / 32), x + (size_t)t * K, K, lane);
    if (lane == 0) y[(size_t)t * M + r] = acc;   // (the function ends with the warp sum: lane 0 holds it)
}

extern "C" {
int ref_gpu_router_topk(const float *logits, int n_expert, int k, int *idx, float *wt, float scale, int renorm, int T, int row_stride) {
    // the engine's launch shape is one warp per row, <<<T,32>>>, over dense rows of n_expert logits; rows with a
    // larger stride (the decode layout keeps the shared-gate logit behind them) are launched one by one
    if (row_stride == n_expert) k_router_topk<<<T, 32>>>(logits, n_expert, k, idx, wt, scale, renorm);
    else
        for (int t = 0; t < T; t++)
            k_router_topk<<<1, 32>>>(logits + (size_t)t * row_stride, n_expert, k, idx + (size_t)t * k, wt + (size_t)t * k, scale, renorm);
    return (int)cudaDeviceSynchronize();
}
int ref_gpu_silu_mul(float *g, const float *u, int n) {
    k_silu_mul<<<(n + 255) / 256, 256>>>(g, u, n);
    return (int)cudaDeviceSynchronize();
}
int ref_gpu_rmsnorm(const float *x, const float *w, float *y, int n, float eps) {
    k_rmsnorm<<<1, 1024>>>(x, w, y, n, eps);
    return (int)cudaDeviceSynchronize();
}
int ref_gpu_matvec_f32_row(const float *W, const float *x, float *y, int M, int K) {
    k_matvec_f32_row<<<M, 256>>>(W, x, y, M, K);
    return (int)cudaDeviceSynchronize();
}
int ref_gpu_dot_mxfp4_split(const uint8_t *planes, const float *x, float *y, int M, int K, int T) {
    const long warps = (long)M * T;
    ref_k_dot_mxfp4_split<<<(unsigned)((warps + 7) / 8), 256>>>(planes, planes + (size_t)M * (K / 2), x, y, M, K, T);
    return (int)cudaDeviceSynchronize();
}
}
