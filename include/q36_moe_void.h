/* q36_moe_void.h -- source-compatibility shim over q36_moe.h for the engine.
 *
 * The engine's own extern "C" launchers return void (q36_cuda_matvec,
 * q36_cuda_rmsnorm, ... in q36_cuda.cu:226-292) and its runtime calls go
 * through CK(), which prints a message and exits (q36_engine.cu:45).  The
 * entry points of q36_moe.h return a status instead and never exit.  This
 * header gives every launch-style entry point a `void q36_cuda_moe_*` twin in
 * the engine's style: same arguments, and on a non-zero status a message on
 * stderr followed by exit(1), which is what CK() does.  Plain C99, header
 * only, no CUDA headers needed: streams travel as void*.
 */
#ifndef Q36_MOE_VOID_H
#define Q36_MOE_VOID_H

#include <stdio.h>
#include <stdlib.h>

#include "q36_moe.h"

#ifdef __cplusplus
extern "C" {
#endif

static inline void q36_cuda_moe_ck(int status, const char *what) {
    if (status != Q36_MOE_OK) {
        fprintf(stderr, "q36_moe %s: %s (detail %d)\n", what, q36_moe_strerror(status), q36_moe_last_cuda_error());
        exit(1);
    }
}

/* upload() MXFP4 branch (q36_engine.cu:202-228) */
static inline void q36_cuda_moe_repack_mxfp4(const void *host_blocks, int K, int M, int e0, int e1, void *host_dst) {
    q36_cuda_moe_ck(q36_moe_repack_mxfp4(host_blocks, K, M, e0, e1, host_dst), "repack_mxfp4");
}
static inline void q36_cuda_moe_upload_mxfp4(const void *host_blocks, int K, int M, int e0, int e1, void *dev_dst) {
    q36_cuda_moe_ck(q36_moe_upload_mxfp4(host_blocks, K, M, e0, e1, dev_dst), "upload_mxfp4");
}
/* k_router_topk<<<T,32>>> (q36_ops.cuh:397-431) */
static inline void q36_cuda_moe_router_topk(const float *logits, int n_expert, int k, int *idx, float *wt, float scale,
                                            int renorm, int T, int row_stride, void *stream) {
    q36_cuda_moe_ck(q36_moe_router_topk(logits, n_expert, k, idx, wt, scale, renorm, T, row_stride, stream), "router_topk");
}
/* k_quant_e4m3 (q36_engine.cu:2412-2428) */
static inline void q36_cuda_moe_quant_e4m3(const void *X, int x_is_bf16, uint8_t *Xq, uint8_t *Xs, int T, int K,
                                           void *stream) {
    q36_cuda_moe_ck(q36_moe_quant_e4m3(X, x_is_bf16, Xq, Xs, T, K, stream), "quant_e4m3");
}
/* k_moe_dispatch (q36_engine.cu:3387-3392) */
static inline void q36_cuda_moe_dispatch(const int *expert_of_entry, int n_entries, int n_expert, int se0, int se1,
                                         int *ecount, int *eoffs, int *elist, int *pos, void *ws, uint64_t ws_bytes,
                                         void *stream) {
    q36_cuda_moe_ck(q36_moe_dispatch(expert_of_entry, n_entries, n_expert, se0, se1, ecount, eoffs, elist, pos, ws, ws_bytes,
                                     stream), "dispatch");
}
/* k_moe_combine / k_moe_combine_pf (q36_engine.cu:785-791, 3393-3401) */
static inline void q36_cuda_moe_combine(float *out, const float *Y_rows, const int *pos, const float *wt,
                                        const float *SH_rows, const float *shgate, int shgate_stride, int D, int k, int T,
                                        void *stream) {
    q36_cuda_moe_ck(q36_moe_combine(out, Y_rows, pos, wt, SH_rows, shgate, shgate_stride, D, k, T, stream), "combine");
}
/* moe_ffn (q36_engine.cu:1592-1654) */
static inline void q36_cuda_moe_decode(const void *Wg, const void *Wu, const void *Wd, const void *Sg, const void *Su,
                                       const void *Sd, int n_expert, int se0, int se1, int k, int D, int FF, const void *X,
                                       int x_is_bf16, const float *logits, int logit_stride, int shgate_col,
                                       float route_scale, int inc_shared, float *out, int T, void *ws, uint64_t ws_bytes,
                                       void *stream) {
    q36_cuda_moe_ck(q36_moe_decode(Wg, Wu, Wd, Sg, Su, Sd, n_expert, se0, se1, k, D, FF, X, x_is_bf16, logits, logit_stride,
                                   shgate_col, route_scale, inc_shared, out, T, ws, ws_bytes, stream), "decode");
}
/* pf_moe_block (q36_engine.cu:3423-3472) */
static inline void q36_cuda_moe_prefill(const void *Wg, const void *Wu, const void *Wd, const void *Sg, const void *Su,
                                        const void *Sd, int n_expert, int se0, int se1, int k, int D, int FF, const void *X,
                                        int x_is_bf16, const float *logits, int logit_stride, int shgate_col,
                                        float route_scale, int inc_shared, float *out, int T, void *ws, uint64_t ws_bytes,
                                        void *stream) {
    q36_cuda_moe_ck(q36_moe_prefill(Wg, Wu, Wd, Sg, Su, Sd, n_expert, se0, se1, k, D, FF, X, x_is_bf16, logits, logit_stride,
                                    shgate_col, route_scale, inc_shared, out, T, ws, ws_bytes, stream), "prefill");
}
/* what CK(cudaDeviceSynchronize()) would have surfaced: a bounded wait that gave up */
static inline void q36_cuda_moe_check_ws(const void *ws, void *stream) {
    q36_cuda_moe_ck(q36_moe_ws_status(ws, stream), "device status");
}

#ifdef __cplusplus
}
#endif
#endif /* Q36_MOE_VOID_H */
