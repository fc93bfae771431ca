// Microbenchmark (not part of libq36moe): sustained rate of ONE SM's TMA unit for the box shapes the expert
// kernels could use to fetch a 128-row x 128-element tile of 4-bit weight codes (rows of 1024 B, as in the
// [512][2048] gate/up planes), against plain bulk copies.  One thread per CTA issues `iters` copies through a
// ring of shared-memory slots; cycles per copy by clock64, aggregate GB/s by CUDA events.
//   nvcc -O3 -std=c++17 -gencode arch=compute_100a,code=sm_100a -o ub_tma_rate q36_b200/csrc/ub_tma_rate.cu
//   ./ub_tma_rate
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <cstdint>
#include <cuda.h>
#include <cuda_runtime.h>
#include "tc_ptx.cuh"
using namespace q36;
namespace q36 { int &last_cuda_error(){ static int e; return e;} int check_launch(){return 0;} bool pdl_enabled(){return false;} }

struct Case {
    const char *name;
    int tensor;              // 1: tiled TMA through the map, 0: untiled bulk copy
    CUtensorMapDataType dt;
    int el_bytes_x2;         // element size in half-bytes (1 for 4-bit)
    int box_inner, box_rows; // elements, rows
    CUtensorMapSwizzle sw;
    uint32_t tx, slot;       // bytes signalled on the barrier, bytes of shared memory per copy
    uint32_t src_bytes;      // global bytes one copy reads
};

// rows of ROW_BYTES; a CTA owns `tiles` consecutive 128-row tiles and walks them K step by K step
constexpr int ROW_BYTES = 1024;

__global__ void k_rate(const __grid_constant__ CUtensorMap m, int tensor, const uint8_t *src, uint32_t tx, uint32_t slot,
                       int slots, int iters, int tiles, int warps, int box_rows, int inner_el, int inner_steps, uint32_t src_bytes,
                       long long *out) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = (uint8_t *)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    __shared__ uint64_t bar[32];
    if (threadIdx.x == 0) {
        for (int b = 0; b < slots * warps; b++) mbar_init(smem_u32(&bar[b]), 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    __shared__ volatile int abortf;
    __shared__ int st_s;
    int *st = &st_s;
    if (threadIdx.x == 0) {
        abortf = 0;
        st_s = 0;
    }
    __syncthreads();
    if ((threadIdx.x & 31) == 0 && (int)(threadIdx.x >> 5) < warps) {
        const int row_steps = 128 / box_rows > 0 ? 128 / box_rows : 1;
        const int per_tile = tensor ? inner_steps * row_steps : 128 * ROW_BYTES / (int)src_bytes;
        // all indices by counters: integer divisions in this loop would cost more than the copy
        int s = 0, ph = 0, ks = 0, rs = 0, within = 0, tile = 0;
        const int wslot0 = (threadIdx.x >> 5) * slots;       // this warp's own slots and tiles
        const int tile0 = (blockIdx.x * warps + (threadIdx.x >> 5)) * tiles;
        const long long t0 = clock64();
        for (int i = 0; i < iters; i++) {
            if (i >= slots && !mbar_wait(smem_u32(&bar[wslot0 + s]), ph ^ 1, &abortf, st, 1)) break;
            mbar_expect_tx(smem_u32(&bar[wslot0 + s]), tx);
            const int gt = tile + tile0;
            if (tensor)
                tma_load_2d(smem_u32(smem + (wslot0 + s) * slot), &m, ks * inner_el, gt * 128 + rs * box_rows, smem_u32(&bar[wslot0 + s]));
            else
                bulk_load(smem_u32(smem + (wslot0 + s) * slot), src + (size_t)gt * 128 * ROW_BYTES + (size_t)within * src_bytes,
                          src_bytes, smem_u32(&bar[wslot0 + s]));
            if (++s == slots) { s = 0; ph ^= 1; }
            if (++ks == inner_steps) { ks = 0; rs++; }
            if (++within == per_tile) { within = 0; rs = 0; if (++tile == tiles) tile = 0; }
        }
        for (int j = 0; j < slots && j < iters; j++) {   // drain: the last use of every slot
            mbar_wait(smem_u32(&bar[wslot0 + s]), ph ^ 1, &abortf, st, 2);
            if (++s == slots) { s = 0; ph ^= 1; }
        }
        out[blockIdx.x * warps + (threadIdx.x >> 5)] = clock64() - t0;
    }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                                  const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

int main() {
    void *p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess || !p) { printf("no encode fn\n"); return 1; }
    EncodeTiledFn enc = (EncodeTiledFn)p;
    const int SMS = 148;
    const size_t big = (size_t)SMS * 64 * 128 * ROW_BYTES;   // 64 tiles per CTA: 1.2 GB, far beyond L2
    uint8_t *src;
    long long *out;
    cudaMalloc(&src, big);
    cudaMemset(src, 0x22, big);
    cudaMalloc(&out, SMS * 8 * 8);
    cudaFuncSetAttribute(k_rate, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    const Case cases[] = {
        {"u4 align16  128el x 128 rows sw128 (in use)", 1, CU_TENSOR_MAP_DATA_TYPE_16U4_ALIGN16B, 1, 128, 128, CU_TENSOR_MAP_SWIZZLE_128B, 8192, 16384, 8192},
        {"u4 align16  128el x  64 rows sw128", 1, CU_TENSOR_MAP_DATA_TYPE_16U4_ALIGN16B, 1, 128, 64, CU_TENSOR_MAP_SWIZZLE_128B, 4096, 8192, 4096},
        {"u8          64 B  x 128 rows sw64", 1, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, 64, 128, CU_TENSOR_MAP_SWIZZLE_64B, 8192, 8192, 8192},
        {"u8          64 B  x 128 rows no swizzle", 1, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, 64, 128, CU_TENSOR_MAP_SWIZZLE_NONE, 8192, 8192, 8192},
        {"u8          128 B x 128 rows sw128", 1, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, 128, 128, CU_TENSOR_MAP_SWIZZLE_128B, 16384, 16384, 16384},
        {"u8          256 B x 128 rows no swizzle", 1, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, 256, 128, CU_TENSOR_MAP_SWIZZLE_NONE, 32768, 32768, 32768},
        {"u32         1024 B x 32 rows no swizzle", 1, CU_TENSOR_MAP_DATA_TYPE_UINT32, 8, 256, 32, CU_TENSOR_MAP_SWIZZLE_NONE, 32768, 32768, 32768},
        {"bulk copy   8 KB contiguous", 0, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, 0, 128, CU_TENSOR_MAP_SWIZZLE_NONE, 8192, 8192, 8192},
        {"bulk copy   32 KB contiguous", 0, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, 0, 128, CU_TENSOR_MAP_SWIZZLE_NONE, 32768, 32768, 32768},
    };
    printf("%-46s | 1 CTA, L2-resident: cyc/copy  B/clk | 148 CTAs L2-resident: cyc/copy  GB/s | 148 CTAs from HBM: cyc/copy  GB/s\n", "copy");
    for (const Case &c : cases) {
        CUtensorMap m;
        memset(&m, 0, sizeof m);
        int inner_steps = 1;
        if (c.tensor) {
            const cuuint64_t inner_total = (cuuint64_t)ROW_BYTES * 2 / c.el_bytes_x2;   // elements per row
            cuuint64_t dims[2] = {inner_total, (cuuint64_t)SMS * 64 * 128};
            cuuint64_t strides[1] = {ROW_BYTES};
            cuuint32_t box[2] = {(cuuint32_t)c.box_inner, (cuuint32_t)c.box_rows}, el[2] = {1, 1};
            CUresult r = enc(&m, c.dt, 2, src, dims, strides, box, el, CU_TENSOR_MAP_INTERLEAVE_NONE, c.sw,
                             CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
            if (r != CUDA_SUCCESS) { printf("%-46s | encode failed (%d)\n", c.name, (int)r); continue; }
            inner_steps = (int)(inner_total / c.box_inner);
        }
        const int slots = (int)(160 * 1024 / c.slot) > 12 ? 12 : (int)(160 * 1024 / c.slot);
        const int per_tile = 128 * ROW_BYTES / c.src_bytes;
        // returns cycles per copy of the slowest issuing warp; *ms = event time of the last pass
        auto run = [&](int grid, int tiles, int iters, int warps, int nslots, int passes, float *ms) -> double {
            cudaEvent_t e0, e1;
            cudaEventCreate(&e0); cudaEventCreate(&e1);
            for (int rep = 0; rep < passes; rep++) {   // a first pass warms L2 for the resident cases
                cudaEventRecord(e0);
                k_rate<<<grid, 32 * warps, 200 * 1024>>>(m, c.tensor, src, c.tx, c.slot, nslots, iters, tiles, warps, c.box_rows,
                                                         c.box_inner, inner_steps, c.src_bytes, out);
                cudaEventRecord(e1);
                if (cudaDeviceSynchronize() != cudaSuccess) { printf("%s: %s\n", c.name, cudaGetErrorString(cudaGetLastError())); exit(1); }
                cudaEventElapsedTime(ms, e0, e1);
            }
            static long long h[SMS * 8];
            cudaMemcpy(h, out, grid * warps * 8, cudaMemcpyDeviceToHost);
            long long mx = 0;
            for (int i = 0; i < grid * warps; i++) mx = h[i] > mx ? h[i] : mx;
            return (double)mx / iters;
        };
        float ms;
        const double c0 = run(1, 2, 64 * per_tile, 1, slots, 2, &ms);
        const double c1 = run(SMS, 2, 64 * per_tile, 1, slots, 2, &ms);
        const double g1 = (double)c.src_bytes * 64 * per_tile * SMS / (ms * 1e6);
        const double c2 = run(SMS, 64, 32 * per_tile, 1, slots, 1, &ms);
        const double g2 = (double)c.src_bytes * 32 * per_tile * SMS / (ms * 1e6);
        printf("%-46s | %8.1f %6.1f | %8.1f %7.0f | %8.1f %7.0f\n", c.name, c0, c.src_bytes / c0, c1, g1, c2, g2);
        if (c.src_bytes == 8192 && (c.tensor == 0 || c.dt == CU_TENSOR_MAP_DATA_TYPE_16U4_ALIGN16B)) {
            for (int warps : {2, 4}) {     // several issuing warps in one CTA, each with its own slots (L2-resident)
                const double cw = run(1, 2, 64 * per_tile, warps, 12 / warps, 2, &ms);
                printf("    %d issuing warps, 1 CTA: %.1f cycles per copy per warp, %.1f B/clk aggregate\n", warps, cw,
                       c.src_bytes * warps / cw);
            }
        }
    }
    return 0;
}
