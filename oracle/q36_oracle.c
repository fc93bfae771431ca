/* CPU oracle for the MXFP4-weight / 8-bit-activation MoE expert path.
 *
 * TEST INFRASTRUCTURE ONLY.  This file is a plain-C restatement of the
 * algorithm the q36 engine runs on the GPU for one MoE layer.  It is the
 * checker for the CUDA kernels and the timed CPU baseline; nothing in the
 * shipped library links, imports or calls it.
 *
 * Pinning: the dequantiser is checked bit-for-bit against the reference's own
 * header compiled as C (oracle/_ref, see oracle/Makefile) and against the
 * constants of the reference's test_dequant.c:46-62.  The E4M3 encoder is
 * checked against NVIDIA's host implementation in cuda_fp8.h (pin_e4m3.cpp).
 * The activation quantiser, router, dispatch, SwiGLU and combine have no
 * known-answer test in the reference: for those the kernel source cited at
 * each function is the only specification ("parity unpinned" for those
 * stages).
 *
 * Every function names the reference file:line it follows (paths relative to
 * the reference project root).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define QK 32            /* q36.h:107  QK_MXFP4                       */
#define BLK_BYTES 17     /* q36.h:114  sizeof(block_mxfp4)            */

/* ---------------------------------------------------------------- dequant */

/* q36_dequant.cuh:98-103: 0.5 * 2^(e-127), two denormal results for e < 2. */
float orc_e8m0_half(uint8_t e) {
    uint32_t bits = (e < 2) ? (0x00200000u << e) : ((uint32_t)(e - 1) << 23);
    float f;
    memcpy(&f, &bits, 4);
    return f;
}

/* q36_dequant.cuh:80-95: the doubled E2M1 table that pairs with the halved
 * scale above. */
static const int8_t k_e2m1x2[16] = {0, 1, 2, 3, 4, 6, 8, 12, 0, -1, -2, -3, -4, -6, -8, -12};

/* q36_dequant.cuh:106-113: byte j carries element j (low nibble) and element
 * j+16 (high nibble). */
void orc_deq_mxfp4_block(const uint8_t *blk, float *out) {
    const float d = orc_e8m0_half(blk[0]);
    for (int j = 0; j < QK / 2; ++j) {
        out[j] = (float)k_e2m1x2[blk[1 + j] & 0x0F] * d;
        out[j + QK / 2] = (float)k_e2m1x2[blk[1 + j] >> 4] * d;
    }
}

/* q36_dequant.cuh:172-173: a row of n values is n/32 consecutive blocks. */
void orc_deq_mxfp4_row(const uint8_t *blocks, int64_t n, float *out) {
    for (int64_t i = 0; i < n / QK; ++i) orc_deq_mxfp4_block(blocks + i * BLK_BYTES, out + i * QK);
}

/* q36_engine.cu:202-228 (upload(), MXFP4 branch): per resident expert the 16
 * code bytes of every block go to a row-major code plane, the scale bytes to
 * a row-major scale plane behind it. */
void orc_split_planes(const uint8_t *blocks, int K, int M, int e0, int e1, uint8_t *dst) {
    const int64_t nbr = K / QK;
    const int64_t qs_e = (int64_t)M * (K / 2), es_e = (int64_t)M * nbr;
    for (int ex = e0; ex < e1; ++ex) {
        uint8_t *qd = dst + (int64_t)(ex - e0) * (qs_e + es_e);
        uint8_t *ed = qd + qs_e;
        for (int64_t r = 0; r < M; ++r)
            for (int64_t b = 0; b < nbr; ++b) {
                const uint8_t *blk = blocks + (((int64_t)ex * M + r) * nbr + b) * BLK_BYTES;
                ed[r * nbr + b] = blk[0];
                memcpy(qd + (r * nbr + b) * 16, blk + 1, 16);
            }
    }
}

/* ------------------------------------------------------------------ E4M3 */

/* Round-to-nearest-even, saturate-to-finite conversion f32 -> E4M3 (4
 * exponent bits, bias 7, 3 mantissa bits, max 448, no infinity), the
 * conversion `__nv_fp8_e4m3(float)` performs at q36_engine.cu:2425. */
uint8_t orc_e4m3_encode(float x) {
    uint32_t u;
    memcpy(&u, &x, 4);
    const uint8_t sign = (uint8_t)((u >> 24) & 0x80);
    const uint32_t a = u & 0x7FFFFFFFu;
    if (a > 0x7F800000u) return 0x7F;                   /* NaN (sign dropped, as cuda_fp8.h does) */
    float ax;
    memcpy(&ax, &a, 4);
    if (ax >= 464.0f) return (uint8_t)(sign | 0x7E);    /* >= midpoint(448,512) -> 448 */
    if (ax < 0.0009765625f) return sign;                /* < 2^-10: below half the smallest step */
    /* step = 2^(max(e,-6)-3) with e = floor(log2 ax); round ax/step to even */
    int e;
    (void)frexpf(ax, &e);
    e -= 1;
    if (e < -6) e = -6;
    const float step = ldexpf(1.0f, e - 3);
    float q = ax / step;                       /* exact: power-of-two divide */
    float r = nearbyintf(q);                   /* default mode: ties to even */
    /* r in [0,16]: 16 means carry into the next binade */
    int ri = (int)r;
    int ebits, mbits;
    if (e == -6 && ri < 8) { ebits = 0; mbits = ri; }
    else {
        if (ri == 16) { ri = 8; e += 1; }
        ebits = e + 7; mbits = ri - 8;
    }
    if (ebits > 15 || (ebits == 15 && mbits > 6)) { ebits = 15; mbits = 6; }
    return (uint8_t)(sign | (ebits << 3) | mbits);
}

float orc_e4m3_decode(uint8_t b) {
    const int s = b >> 7, e = (b >> 3) & 15, m = b & 7;
    float v;
    if (e == 15 && m == 7) v = NAN;
    else if (e == 0) v = ldexpf((float)m, -9);
    else v = ldexpf((float)(8 + m), e - 10);
    return s ? -v : v;
}

/* Smallest integer e2 with amax <= 448 * 2^e2, clamped to [-127,127]; amax
 * == 0 gives -127.  q36_engine.cu:2421 writes this as ceilf(log2f(a/448.f));
 * the two agree wherever log2f is exact, and this integer form is the one
 * both the oracle and the CUDA kernel use so that "bit-exact" is well
 * defined (the reference is built with --use_fast_math, Makefile:38). */
static int orc_e2_of_amax(float amax) {
    uint32_t u;
    memcpy(&u, &amax, 4);
    if (u == 0) return -127;
    const int E = (int)(u >> 23);
    const uint32_t mant = u & 0x7FFFFFu;
    int e2 = E - 135 + (mant > 0x600000u ? 1 : 0);   /* 448 = 1.75 * 2^8 */
    if (e2 < -127) e2 = -127;
    if (e2 > 127) e2 = 127;
    return e2;
}

/* q36_engine.cu:2412-2428 (k_quant_e4m3): per (row, 32-block) amax -> shared
 * power-of-two scale -> E4M3 codes; scale byte 127+e2.  Values stay in
 * logical order. */
void orc_quant_e4m3(const float *X, uint8_t *Xq, uint8_t *Xs, int T, int K) {
    const int nb = K / QK;
    for (int64_t t = 0; t < T; ++t)
        for (int b = 0; b < nb; ++b) {
            const float *v = X + t * K + b * QK;
            float a = 0.f;
            for (int j = 0; j < QK; ++j) a = fmaxf(a, fabsf(v[j]));
            const int e2 = orc_e2_of_amax(a);
            uint32_t sb = (uint32_t)(127 - e2) << 23;   /* 2^-e2; e2=127 -> 0.0 as in :2423-2425 */
            float inv;
            memcpy(&inv, &sb, 4);
            for (int j = 0; j < QK; ++j) Xq[t * K + b * QK + j] = orc_e4m3_encode(v[j] * inv);
            Xs[t * nb + b] = (uint8_t)(127 + e2);
        }
}

/* value = e4m3(q) * 2^(s-127) */
void orc_dequant_e4m3(const uint8_t *Xq, const uint8_t *Xs, float *X, int T, int K) {
    const int nb = K / QK;
    for (int64_t t = 0; t < T; ++t)
        for (int b = 0; b < nb; ++b) {
            const float sc = ldexpf(1.0f, (int)Xs[t * nb + b] - 127);
            for (int j = 0; j < QK; ++j) X[t * K + b * QK + j] = orc_e4m3_decode(Xq[t * K + b * QK + j]) * sc;
        }
}

/* ---------------------------------------------------------------- router */

/* q36_ops.cuh:397-431 (k_router_topk): softmax statistics over all experts,
 * k rounds of arg-max on the RAW logits (ties go to the lower index, :423),
 * weight = exp(v-m)/s, then either renormalised to sum*scale (:428-429) or
 * just scaled. */
void orc_router_topk(const float *logits, int n_expert, int k, int *idx, float *wt,
                     float scale, int renorm, int T, int row_stride) {
    float *v = (float *)malloc(sizeof(float) * (size_t)n_expert);
    for (int64_t t = 0; t < T; ++t) {
        const float *l = logits + t * row_stride;
        float m = -1e30f;
        for (int i = 0; i < n_expert; ++i) { v[i] = l[i]; m = fmaxf(m, v[i]); }
        double s = 0;
        for (int i = 0; i < n_expert; ++i) s += exp((double)v[i] - (double)m);
        for (int r = 0; r < k; ++r) {
            int bi = 0; float bv = -1e30f;
            for (int i = 0; i < n_expert; ++i) if (v[i] > bv) { bv = v[i]; bi = i; }
            idx[t * k + r] = bi;
            wt[t * k + r] = (float)(exp((double)bv - (double)m) / s);
            v[bi] = -1e30f;
        }
        if (renorm) {
            double ws = 0;
            for (int r = 0; r < k; ++r) ws += wt[t * k + r];
            for (int r = 0; r < k; ++r) wt[t * k + r] = (float)(wt[t * k + r] / ws * scale);
        } else {
            for (int r = 0; r < k; ++r) wt[t * k + r] *= scale;
        }
    }
    free(v);
}

/* q36_engine.cu:3387-3392 (k_moe_dispatch): bucket entry ids i = t*k + s by
 * expert.  The reference's order inside a bucket is whatever the atomics
 * give; the oracle fixes the stable order (ascending entry id), which is one
 * of the orders the reference can produce.  eoffs[n_expert+1] is the
 * exclusive prefix sum of ecount; elist is packed by eoffs. */
void orc_dispatch(const int *topk, int *ecount, int *eoffs, int *elist, int T, int k, int n_expert) {
    memset(ecount, 0, sizeof(int) * (size_t)n_expert);
    for (int64_t i = 0; i < (int64_t)T * k; ++i) ecount[topk[i]]++;
    eoffs[0] = 0;
    for (int e = 0; e < n_expert; ++e) eoffs[e + 1] = eoffs[e] + ecount[e];
    int *cur = (int *)malloc(sizeof(int) * (size_t)n_expert);
    memcpy(cur, eoffs, sizeof(int) * (size_t)n_expert);
    for (int64_t i = 0; i < (int64_t)T * k; ++i) elist[cur[topk[i]]++] = (int)i;
    free(cur);
}

/* ------------------------------------------------------- expert FFN (f64) */

static double silu_d(double x) { return x / (1.0 + exp(-x)); }     /* q36_ops.cuh:58 */
static double sigm_d(double x) { return 1.0 / (1.0 + exp(-x)); }   /* q36_ops.cuh:59 */

/* y[M] = W[M][K] (GGUF MXFP4 blocks, row-major) * x[K], float64 accumulation
 * over the bit-exact dequantised weights. */
static void matvec_mxfp4_f64(const uint8_t *blocks, int M, int K, const float *x, double *y) {
    const int nb = K / QK;
    #pragma omp parallel for schedule(static)
    for (int r = 0; r < M; ++r) {
        float w[QK];
        double acc = 0;
        for (int b = 0; b < nb; ++b) {
            orc_deq_mxfp4_block(blocks + ((int64_t)r * nb + b) * BLK_BYTES, w);
            for (int j = 0; j < QK; ++j) acc += (double)w[j] * (double)x[b * QK + j];
        }
        y[r] = acc;
    }
}

/* One expert on one token.  xd is the dequantised quantised activation
 * (length D).  gate/up are [FF][D], down is [D][FF], all GGUF MXFP4 blocks.
 *   g = Wg xd, u = Wu xd                     (k_expert_gemv2, q36_engine.cu:752-783)
 *   h = silu(g) * u                           (k_silu_mul_slots, :744-746)
 *   (hq,hs) = quant_e4m3(float(h))            W4A8 down: same quantiser as :2412-2428
 *   y = Wd dequant(hq,hs)                     (k_expert_gemv, :711-742)
 * If hq_in is non-NULL the given quantised intermediate is used instead of
 * the oracle's own (stage-wise check).  Outputs: y[D] (f64); optional h_out[FF]
 * (f32), hq_out[FF], hs_out[FF/32]. */
void orc_expert_ffn(const uint8_t *gate, const uint8_t *up, const uint8_t *down, int D, int FF,
                    const float *xd, const uint8_t *hq_in, const uint8_t *hs_in,
                    double *y, float *h_out, uint8_t *hq_out, uint8_t *hs_out) {
    double *g = (double *)malloc(sizeof(double) * (size_t)FF * 2);
    double *u = g + FF;
    float *h = (float *)malloc(sizeof(float) * (size_t)FF * 2);
    float *hd = h + FF;
    uint8_t *hq = (uint8_t *)malloc((size_t)FF + (size_t)FF / QK);
    uint8_t *hs = hq + FF;
    matvec_mxfp4_f64(gate, FF, D, xd, g);
    matvec_mxfp4_f64(up, FF, D, xd, u);
    for (int i = 0; i < FF; ++i) h[i] = (float)(silu_d(g[i]) * u[i]);
    if (hq_in) { memcpy(hq, hq_in, (size_t)FF); memcpy(hs, hs_in, (size_t)FF / QK); }
    else orc_quant_e4m3(h, hq, hs, 1, FF);
    orc_dequant_e4m3(hq, hs, hd, 1, FF);
    matvec_mxfp4_f64(down, D, FF, hd, y);
    if (h_out) memcpy(h_out, h, sizeof(float) * (size_t)FF);
    if (hq_out) memcpy(hq_out, hq, (size_t)FF);
    if (hs_out) memcpy(hs_out, hs, (size_t)FF / QK);
    free(g); free(h); free(hq);
}

/* One MoE layer for a chosen subset of tokens.
 *   k_moe_combine / k_moe_combine_pf (q36_engine.cu:785-791, 3393-3401):
 *   out[t] = sum_s w[t][s] * y(expert idx[t][s], x_t) + inc_shared * sigmoid(shg[t]) * y(shared, x_t)
 * Experts outside [se0,se1) contribute zeros (:763-766, 2440).
 * W* hold all n_expert experts as GGUF blocks ([E][rows][K/32][17]); S* the
 * shared expert.  X is f32 [T][D]; tok[n_tok] lists the tokens to evaluate;
 * out is [n_tok][D] f64. */
void orc_moe_layer(const uint8_t *Wg, const uint8_t *Wu, const uint8_t *Wd,
                   const uint8_t *Sg, const uint8_t *Su, const uint8_t *Sd,
                   int D, int FF, int k, int se0, int se1, int inc_shared,
                   const float *X, const int *idx, const float *wt, const float *shg,
                   const int *tok, int n_tok, double *out) {
    const int64_t gu_bytes = (int64_t)FF * (D / QK) * BLK_BYTES;
    const int64_t dn_bytes = (int64_t)D * (FF / QK) * BLK_BYTES;
    uint8_t *xq = (uint8_t *)malloc((size_t)D + (size_t)D / QK);
    uint8_t *xs = xq + D;
    float *xd = (float *)malloc(sizeof(float) * (size_t)D);
    double *y = (double *)malloc(sizeof(double) * (size_t)D);
    for (int n = 0; n < n_tok; ++n) {
        const int t = tok[n];
        orc_quant_e4m3(X + (int64_t)t * D, xq, xs, 1, D);
        orc_dequant_e4m3(xq, xs, xd, 1, D);
        double *o = out + (int64_t)n * D;
        for (int j = 0; j < D; ++j) o[j] = 0;
        for (int s = 0; s < k; ++s) {
            const int e = idx[(int64_t)t * k + s];
            if (e < se0 || e >= se1) continue;
            orc_expert_ffn(Wg + e * gu_bytes, Wu + e * gu_bytes, Wd + e * dn_bytes, D, FF, xd,
                           NULL, NULL, y, NULL, NULL, NULL);
            const double w = wt[(int64_t)t * k + s];
            for (int j = 0; j < D; ++j) o[j] += w * y[j];
        }
        if (inc_shared && Sg) {
            orc_expert_ffn(Sg, Su, Sd, D, FF, xd, NULL, NULL, y, NULL, NULL, NULL);
            const double w = sigm_d((double)shg[t]);
            for (int j = 0; j < D; ++j) o[j] += w * y[j];
        }
    }
    free(xq); free(xd); free(y);
}

/* ------------------------------------------------ timed CPU baseline (f32) */

typedef void (*deq_row_fn)(const uint8_t *blocks, int64_t n, float *out);

/* The reference's CPU implementation of the path: its C dequantiser over the
 * three matrices of one expert (q36_dequant.cuh:168-181) followed by a
 * straightforward fp32 matmul (g = Wg x, u = Wu x, h = silu(g) u, y = Wd h).
 * `deq` is the dequantiser to time: the reference's own (oracle/_ref) or
 * orc_deq_mxfp4_row.  scratch holds 3*FF*D floats.  Rows are spread over the
 * OpenMP threads.  Returns nothing; y[D] receives the result. */
void orc_cpu_expert_f32(deq_row_fn deq, const uint8_t *gate, const uint8_t *up, const uint8_t *down,
                        int D, int FF, const float *xd, float *scratch, float *y) {
    float *wg = scratch, *wu = scratch + (int64_t)FF * D, *wd = wu + (int64_t)FF * D;
    const int64_t rb_gu = (int64_t)(D / QK) * BLK_BYTES, rb_dn = (int64_t)(FF / QK) * BLK_BYTES;
    #pragma omp parallel for schedule(static)
    for (int r = 0; r < FF; ++r) {
        deq(gate + r * rb_gu, D, wg + (int64_t)r * D);
        deq(up + r * rb_gu, D, wu + (int64_t)r * D);
    }
    #pragma omp parallel for schedule(static)
    for (int r = 0; r < D; ++r) deq(down + r * rb_dn, FF, wd + (int64_t)r * FF);
    float *h = (float *)malloc(sizeof(float) * (size_t)FF);
    #pragma omp parallel for schedule(static)
    for (int r = 0; r < FF; ++r) {
        float g = 0.f, u = 0.f;
        for (int c = 0; c < D; ++c) { g += wg[(int64_t)r * D + c] * xd[c]; u += wu[(int64_t)r * D + c] * xd[c]; }
        h[r] = g / (1.f + expf(-g)) * u;
    }
    #pragma omp parallel for schedule(static)
    for (int r = 0; r < D; ++r) {
        float a = 0.f;
        for (int c = 0; c < FF; ++c) a += wd[(int64_t)r * FF + c] * h[c];
        y[r] = a;
    }
    free(h);
}

int orc_num_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}
void orc_set_threads(int n) {
#ifdef _OPENMP
    omp_set_num_threads(n);
#else
    (void)n;
#endif
}
