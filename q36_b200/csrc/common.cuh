// Shared device/host helpers for the MXFP4 x E4M3 MoE expert path (sm_100a).
#pragma once
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/q36_moe.h"

#define Q36_QK 32  // elements per MXFP4 / activation scale block (q36.h:107)

// Every kernel opens with this so that it may be launched with the
// programmatic-dependent-launch attribute, as the reference's kernels are
// (q36_ops.cuh:21-30); without the attribute it is a no-op.
// The trigger lets the next kernel of the stream start launching while this one runs; the synchronise makes
// this kernel wait for the complete previous grid before it touches global memory.
#define Q36_GDS()                                \
    do {                                         \
        cudaTriggerProgrammaticLaunchCompletion(); \
        cudaGridDependencySynchronize();         \
    } while (0)

// Optional timing trace (compile with -DQ36_TRACE): thread 0 of block 0 of an instrumented kernel adds its own
// duration and the gap since the previous instrumented kernel ended to counters kept behind the status words of the
// workspace (u64 slots from byte 64: [0] last end, [1 + id] duration, [9 + id] gap before, [17 + id] launches).
#ifdef Q36_TRACE
__device__ __forceinline__ unsigned long long q36_globaltimer() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
#define Q36_TR_BEGIN(st, kid)                                                                  \
    unsigned long long tr_t0 = 0;                                                              \
    if ((st) && blockIdx.x == 0 && blockIdx.y == 0 && threadIdx.x == 0) {                      \
        tr_t0 = q36_globaltimer();                                                             \
        unsigned long long *tr = reinterpret_cast<unsigned long long *>((st) + 16);            \
        if (tr[0]) tr[9 + (kid)] += tr_t0 - tr[0];                                             \
    }
#define Q36_TR_END(st, kid)                                                                    \
    if ((st) && blockIdx.x == 0 && blockIdx.y == 0 && threadIdx.x == 0) {                      \
        const unsigned long long tr_t1 = q36_globaltimer();                                    \
        unsigned long long *tr = reinterpret_cast<unsigned long long *>((st) + 16);            \
        tr[1 + (kid)] += tr_t1 - tr_t0;                                                        \
        tr[0] = tr_t1;                                                                         \
        tr[17 + (kid)] += 1;                                                                   \
    }
#else
#define Q36_TR_BEGIN(st, kid)
#define Q36_TR_END(st, kid)
#endif

namespace q36 {

// Last CUDA error seen by an entry point of this thread (0 = none).
int &last_cuda_error();
int check_launch();  // cudaGetLastError() -> status code
bool pdl_enabled();  // false when the environment variable Q36_NOPDL is set (as in the engine, q36_engine.cu:2251-2286)

// Kernel launch with the programmatic-dependent-launch attribute: the launch may be processed while the
// previous kernel of the stream is still running; every kernel waits in Q36_GDS() before its first access.
template <typename... KArgs, typename... Args>
inline void launch_k(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl_enabled() ? 1 : 0;
    cudaLaunchKernelEx(&cfg, kern, static_cast<KArgs>(args)...);
}

// The same for a kernel whose blocks wait for one another: the cooperative attribute makes the runtime refuse the
// launch unless every block can be resident at once (instead of that being true by construction only).  Measured:
// no cost (1.450 against 1.445 ms per 40-layer step), and it combines with the programmatic-launch attribute inside a
// captured graph.  Q36_COOP=0 in the environment turns it off; 2 = cooperative without the programmatic attribute.
inline int coop_mode() {
    static int mode = -1;
    if (mode < 0) { const char *e = getenv("Q36_COOP"); mode = e ? atoi(e) : 1; }
    return mode;
}
template <typename... KArgs, typename... Args>
inline void launch_k_resident(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args... args) {
    const int mode = coop_mode();
    if (mode == 0) { launch_k(kern, grid, block, smem, st, args...); return; }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeCooperative;
    attr[0].val.cooperative = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = (mode == 1 && pdl_enabled()) ? 2 : 1;
    cudaLaunchKernelEx(&cfg, kern, static_cast<KArgs>(args)...);
}

// Smallest e2 with amax <= 448 * 2^e2, clamped to [-127,127]; 0 -> -127.
// Integer form of ceil(log2(amax/448)) (q36_engine.cu:2421); 448 = 1.75 * 2^8.
__device__ __forceinline__ int e2_of_amax(float amax) {
    const uint32_t u = __float_as_uint(amax);
    if (u == 0) return -127;
    int e2 = (int)(u >> 23) - 135 + ((u & 0x7FFFFFu) > 0x600000u ? 1 : 0);
    return max(-127, min(127, e2));
}
// 2^-e2 as the reference builds it (q36_engine.cu:2423-2425): exponent bits
// only, so e2 = 127 yields 0.0f.
__device__ __forceinline__ float inv_scale_of_e2(int e2) { return __uint_as_float((uint32_t)(127 - e2) << 23); }
// 2^(s-127) for a UE8M0 byte; s = 0 is the denormal 2^-127.
__device__ __forceinline__ float ue8m0_to_f32(uint32_t s) { return __uint_as_float(s ? (s << 23) : 0x00400000u); }

// f32 -> E4M3, round-to-nearest-even, saturate to +-448 (NaN -> 0x7F).
__device__ __forceinline__ uint8_t f32_to_e4m3(float v) {
    return (uint8_t)__nv_cvt_float_to_fp8(v, __NV_SATFINITE, __NV_E4M3);
}
// two E4M3 bytes (low byte first) -> two f32
__device__ __forceinline__ float2 e4m3x2_to_f32x2(uint16_t p) {
    __half2_raw h = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)p, __NV_E4M3);
    return __half22float2(*reinterpret_cast<__half2 *>(&h));
}
// one packed byte of two E2M1 codes (low nibble first) -> two f32 in the TRUE
// E2M1 convention {0,.5,1,1.5,2,3,4,6}; the block scale is then 2^(e-127),
// whose product equals the reference's doubled table times 2^(e-128)
// (q36_dequant.cuh:80-103).
__device__ __forceinline__ float2 e2m1x2_to_f32x2(uint32_t byte) {
    uint32_t h2;
    asm("{\n\t.reg .b8 b;\n\t.reg .b16 t;\n\tcvt.u16.u32 t, %1;\n\tcvt.u8.u16 b, t;\n\t"
        "cvt.rn.f16x2.e2m1x2 %0, b;\n\t}"
        : "=r"(h2)
        : "r"(byte));
    return __half22float2(*reinterpret_cast<__half2 *>(&h2));
}

// Position of logical element j (0..31) of a 32-block in the order the MXFP4
// code bytes imply: code byte i holds element i (low nibble) and element i+16
// (high nibble) (q36_dequant.cuh:109-112), so consecutive nibbles are elements
// 0,16,1,17,...  Activations are stored in that same order so that weights
// are consumed byte for byte as they sit in the GGUF block.
__host__ __device__ __forceinline__ int hw_pos(int j) { return (j < 16) ? (2 * j) : (2 * (j - 16) + 1); }

__device__ __forceinline__ float silu_f(float x) { return x / (1.f + __expf(-x)); }   // q36_ops.cuh:58
__device__ __forceinline__ float sigm_f(float x) { return 1.f / (1.f + __expf(-x)); } // q36_ops.cuh:59

// SwiGLU + E4M3 requantisation of NC token columns held by a warp whose 32 lanes are the 32 ff rows of one scale
// block: h = silu(g) * u, block amax by one redux per column, shared exponent, code stored at the lane's hw
// position of row (row0 + c).  Written without per-column branches so that the NC dependent chains (exp,
// divide, redux, convert, store: several hundred cycles each) overlap; only the stores are predicated.
template <int NC>
__device__ __forceinline__ void swiglu_quant_store(const float (&g)[NC], const float (&u)[NC], int n_valid, size_t row0,
                                                   uint8_t *__restrict__ Hq, uint8_t *__restrict__ Hs, int FF, int blk,
                                                   int lane) {
    float h[NC];
    uint32_t am[NC];
#pragma unroll
    for (int c = 0; c < NC; c++) h[c] = __fdividef(g[c], 1.f + __expf(-g[c])) * u[c];
#pragma unroll
    for (int c = 0; c < NC; c++) am[c] = __reduce_max_sync(0xffffffffu, __float_as_uint(fabsf(h[c])));
    const int p = hw_pos(lane);
    const int nbh = FF / Q36_QK;
#pragma unroll
    for (int c = 0; c < NC; c++) {
        const int e2 = e2_of_amax(__uint_as_float(am[c]));
        const uint8_t q = f32_to_e4m3(h[c] * inv_scale_of_e2(e2));
        if (c < n_valid) {
            Hq[(row0 + c) * FF + blk * Q36_QK + p] = q;
            if (lane == 0) Hs[(row0 + c) * nbh + blk] = (uint8_t)(127 + e2);
        }
    }
}

// Result rows between the down projection and the combine are staged as f32, or -- prefill-sized calls of the
// whole-layer entries, when asked for (stage_y_bf16) -- as bf16: half the bytes of the largest round trip through HBM
// of such a layer, for 1.6e-3 instead of 1.5e-7 against a float64 product (the path is held to 1e-2).  Four
// consecutive elements from element e.
__device__ __forceinline__ float4 ld_y4(const void *Y, size_t e, int y_bf16) {
    if (!y_bf16) return *reinterpret_cast<const float4 *>(reinterpret_cast<const float *>(Y) + e);
    const uint2 v = *reinterpret_cast<const uint2 *>(reinterpret_cast<const uint16_t *>(Y) + e);
    return make_float4(__uint_as_float(v.x << 16), __uint_as_float(v.x & 0xffff0000u), __uint_as_float(v.y << 16),
                       __uint_as_float(v.y & 0xffff0000u));
}
__device__ __forceinline__ void st_y(void *Y, size_t e, float v, int y_bf16) {
    if (y_bf16) reinterpret_cast<__nv_bfloat16 *>(Y)[e] = __float2bfloat16_rn(v);
    else reinterpret_cast<float *>(Y)[e] = v;
}
// row r of such a buffer
__host__ __device__ __forceinline__ const float *y_row(const void *Y, size_t r, int D, int y_bf16) {
    return reinterpret_cast<const float *>(reinterpret_cast<const uint8_t *>(Y) + r * (size_t)D * (y_bf16 ? 2 : 4));
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

}  // namespace q36
