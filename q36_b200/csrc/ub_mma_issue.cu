// Microbenchmark (not part of libq36moe): cycles per tcgen05.mma kind::mxf8f6f4.block_scale (M = 128, K = 32)
// against N and the number of issuing warps.  One CTA, operands are constant bytes in shared memory.
//   nvcc -O3 -std=c++17 -gencode arch=compute_100a,code=sm_100a -o ub_mma_issue q36_b200/csrc/ub_mma_issue.cu
#include <cstdio>
#include <cstdint>
#include <cuda_runtime.h>
#include "tc_ptx.cuh"
using namespace q36;
namespace q36 { int &last_cuda_error(){ static int e; return e;} int check_launch(){return 0;} bool pdl_enabled(){return false;} }

// mode: 0 = same accumulator, 1 = 4 rotating accumulators, 2 = mma + cp per 4 mma, 3 = two issuing warps (rotating acc)
__global__ void k_ub(int N, int iters, int mode, long long *out) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = (uint8_t *)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    __shared__ uint32_t tmem_s;
    __shared__ uint64_t bar[8];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int i = threadIdx.x; i < 48 * 1024 / 4; i += blockDim.x) ((uint32_t *)smem)[i] = 0x38383838u;  // e4m3 1.0 / fp4 codes
    if (threadIdx.x == 0) { for (int b = 0; b < 8; b++) mbar_init(smem_u32(&bar[b]), 1); asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_s)), "r"(512) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    tc_fence_before(); __syncthreads(); tc_fence_after();
    const uint32_t tmem = tmem_s;
    const uint32_t sa = smem_u32(smem), sb = smem_u32(smem + 16384), sf = smem_u32(smem + 32768);
    volatile int abortf = 0; int st = 0;
    if ((warp == 0 || (mode >= 3 && warp < mode - 1)) && lane == 0) {
        const uint32_t sfa = tmem + 448, sfb = tmem + 452;
        if (warp == 0) { tc_cp_sf(sfa, desc_sf(sf)); tc_cp_sf(sfb, desc_sf(sf + 512)); }
        long long t0 = clock64();
        for (int i = 0; i < iters; i++) {
            const int kb = i & 3;
            uint32_t d = tmem;
            if (mode == 1 || mode == 2) d = tmem + (i & 3) * (N <= 64 ? 64 : 0);
            if (mode >= 3) d = tmem + warp * 64;
            if (mode == 2 && kb == 0) { tc_cp_sf(sfa, desc_sf(sf)); tc_cp_sf(sfb, desc_sf(sf + 512)); }
            tc_mma(d, desc_sw128(sa + kb * 32), desc_sw128(sb + kb * 32), idesc_mx(N, kb), sfa | ((uint32_t)kb << 30), sfb | ((uint32_t)kb << 30), i >= 4);
        }
        long long t1 = clock64();
        tc_commit(smem_u32(&bar[warp]));
        mbar_wait(smem_u32(&bar[warp]), 0, (volatile int *)&abortf, &st, 1);
        long long t2 = clock64();
        if (warp < 2) { out[warp * 2 + 0] = t1 - t0; out[warp * 2 + 1] = t2 - t0; }
    }
    tc_fence_before(); __syncthreads();
    if (warp == 0) { tc_fence_after(); asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512) : "memory"); }
}
int main() {
    long long *d; cudaMalloc(&d, 64); long long h[4];
    cudaFuncSetAttribute(k_ub, cudaFuncAttributeMaxDynamicSharedMemorySize, 64 * 1024);
    const int iters = 2000;
    for (int mode : {3, 5, 7, 9})
        for (int N : {16, 32, 64}) {
            cudaMemset(d, 0, 64);
            k_ub<<<1, 256, 64 * 1024>>>(N, iters, mode, d);
            cudaError_t e = cudaDeviceSynchronize();
            cudaMemcpy(h, d, 32, cudaMemcpyDeviceToHost);
            printf("issuers %d (mode %d) N %3d: issue %.1f cyc/mma, complete %.1f cyc/mma (%s) w1: %.1f\n", mode - 1, mode, N, (double)h[0] / iters, (double)h[1] / iters, cudaGetErrorString(e), (double)h[3] / iters);
        }
    return 0;
}
