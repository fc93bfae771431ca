// extern "C" entry points of libq36moe (declared in include/q36_moe.h).
#include <cuda_bf16.h>
#include <stdlib.h>
#include <string.h>

#include "common.cuh"
#include "kernels.cuh"

namespace q36 {

int &last_cuda_error() {
    static thread_local int e = 0;
    return e;
}
int check_launch() {
    const cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) { last_cuda_error() = (int)e; return Q36_MOE_ECUDA; }
    return Q36_MOE_OK;
}
bool pdl_enabled() {
    static int on = -1;
    if (on < 0) on = getenv("Q36_NOPDL") ? 0 : 1;
    return on != 0;
}
static int ck(cudaError_t e) {
    if (e != cudaSuccess) { last_cuda_error() = (int)e; return Q36_MOE_ECUDA; }
    return Q36_MOE_OK;
}

bool router_supports(int n_expert) { return n_expert == 256 || n_expert == 128 || n_expert == 64 || n_expert == 32; }

static inline uint64_t al(uint64_t x) { return (x + 255) & ~(uint64_t)255; }

// Carves the caller's workspace of one layer call.  Every region is 256-byte
// aligned; the first 256 bytes hold the device-side status words of the
// tensor-core launches.
struct LayerWs {
    int *status;          // [4]
    int *idx; float *wt;  // [T*k]
    int *ecount, *eoffs, *soffs, *elist, *pos;
    void *disp;
    uint8_t *Xq, *Xs, *Hq, *Hs;
    float *Y;
    void *plan;
    uint64_t total;
};
static LayerWs carve(void *base, int T, int E, int k, int D, int FF) {
    LayerWs w;
    uint8_t *p = (uint8_t *)base;
    uint64_t o = 0;
    const uint64_t R = (uint64_t)T * (k + 1), n = (uint64_t)T * k;
    auto take = [&](uint64_t bytes) { uint8_t *r = p + o; o += al(bytes); return (void *)r; };
    w.status = (int *)take(256);
    w.idx = (int *)take(n * 4);
    w.wt = (float *)take(n * 4);
    w.ecount = (int *)take((uint64_t)E * 4);
    w.eoffs = (int *)take((uint64_t)(E + 1) * 4);
    w.soffs = (int *)take(8);
    w.elist = (int *)take(n * 4);
    w.pos = (int *)take(n * 4);
    w.disp = take(dispatch_ws_bytes((int)n, E));
    w.Xq = (uint8_t *)take(R * D);
    w.Xs = (uint8_t *)take(R * (D / Q36_QK));
    w.Hq = (uint8_t *)take(R * FF);
    w.Hs = (uint8_t *)take(R * (FF / Q36_QK));
    w.Y = (float *)take(R * D * 4);
    w.plan = take(tc_ws_bytes());
    w.total = o;
    return w;
}

// Rows up to which the one-launch decode kernel (token tiles of 16 rows) is used instead of the two grouped-GEMM
// launches (token tiles of 112 / 128 rows) when groups may exceed 16 rows.  Measured per layer on B200: 24 tokens 63 us
// against 100 us, 64 tokens 94 against 155, 256 tokens 118 against 165, 512 tokens 150 against 181, 1024 tokens 220
// against 198: the lines cross near 800 tokens (9 rows per token); the environment variable is there for experiments.
int fused_rows_limit() {
    static int v = -1;
    if (v < 0) { const char *e = getenv("Q36_FUSE_ROWS"); v = e ? atoi(e) : 4096; }
    return v;
}

static int pick_path(int path, int T) {
    if (path == Q36_MOE_PATH_GEMV || path == Q36_MOE_PATH_TC) return path;
    // The engine switches from its GEMV kernels to its tiled kernels at 14 rows (q36_engine.cu:2217-2221).
    // Measured on B200 the tensor-core path is at least as fast at every T (its weight stream needs no ALU
    // decode), so AUTO always takes it; the GEMV stays selectable.
    (void)T;
    return Q36_MOE_PATH_TC;
}

// What follows the combine when the caller drives the block from the residual stream: h += moe, then the next
// RMSNorm (q36_engine.cu:1966).  h == nullptr: the layer ends at the combine.
struct PostNorm { float *h; const float *w_next; float eps; float *x_next; };

static int layer_impl(const void *Wg, const void *Wu, const void *Wd, const void *Sg, const void *Su,
                      const void *Sd, int E, int se0, int se1, int k, int D, int FF, const void *X,
                      int x_is_bf16, const float *logits, int logit_stride, int shgate_col,
                      float route_scale, int inc_shared, float *out, int *idx_out, float *wt_out, int T,
                      int path, void *ws, uint64_t ws_bytes, cudaStream_t st, PostNorm post = PostNorm{nullptr, nullptr, 0.f, nullptr}) {
    if (!Wg || !Wu || !Wd || !X || !logits || (!out && !post.h) || !ws) return Q36_MOE_EINVAL;
    if (T <= 0 || k <= 0 || k > 8 || E <= 0 || E > DISPATCH_MAX_GROUPS || se0 < 0 || se1 > E || se0 >= se1)
        return Q36_MOE_EINVAL;
    if (D % 128 || FF % 128 || logit_stride < E) return Q36_MOE_EINVAL;
    if (!router_supports(E)) return Q36_MOE_EINVAL;   // the router keeps E / 32 logits per lane: 32, 64, 128 or 256 experts
    const LayerWs w = carve(ws, T, E, k, D, FF);
    if (w.total > ws_bytes) return Q36_MOE_ENOSPACE;
    const bool shared = Sg && Su && Sd && inc_shared;
    const int n = T * k, R = T * (k + 1);
    int rc;
    const bool use_tc = pick_path(path, T) == Q36_MOE_PATH_TC;
    const bool fused_front = n <= 1024;
    static const bool no_fuse = getenv("Q36_NOFUSE") != nullptr;
    // decode: gate/up and down in one persistent launch (its plan is cut in token tiles of 16 rows)
    const bool decode_kernel = use_tc && !no_fuse && R <= fused_rows_limit() && ffn_fused_small_fits(R, se1 - se0, D, FF);
    static const bool no_cluster = getenv("Q36_NOCLUSTER") != nullptr;
    // decode on the tensor-core path with every expert resident: one cluster launch does all of the front end
    const bool cluster_front = use_tc && T <= 16 && n <= 128 && se0 == 0 && se1 == E && D % 1024 == 0 && D * T <= 32 * 1024 && !no_cluster;
    const bool fused_quant = cluster_front || (fused_front && T <= 2);     // beyond a couple of rows the scatter serialises inside one block: measured slower than a launch
    if (cluster_front) {
        if ((rc = launch_front_decode(logits, E, k, route_scale, T, logit_stride, w.idx, w.wt, w.ecount, w.eoffs, w.elist,
                                      w.pos, w.soffs, n, shared ? n + T : n, w.plan, D, FF, w.status, X, x_is_bf16, w.Xq,
                                      w.Xs, shared ? n : -1, k, st)))
            return rc;
    } else if (fused_front) {
        if ((rc = launch_front_small(logits, E, k, route_scale, T, logit_stride, se0, se1, w.idx, w.wt, w.ecount, w.eoffs,
                                     w.elist, w.pos, w.soffs, n, shared ? n + T : n, use_tc ? w.plan : nullptr, D, FF,
                                     w.status, fused_quant ? X : nullptr, x_is_bf16, w.Xq, w.Xs, shared ? n : -1,
                                     decode_kernel ? 16 : gateup_tile_rows(), st)))
            return rc;
    } else {
        if ((rc = launch_router_topk(logits, E, k, w.idx, w.wt, route_scale, 1, T, logit_stride, st))) return rc;
        if ((rc = launch_dispatch(w.idx, n, E, se0, se1, w.ecount, w.eoffs, w.elist, w.pos, w.disp, w.soffs, n,
                                  shared ? n + T : n, st, use_tc ? w.plan : nullptr, D, FF, decode_kernel ? 16 : gateup_tile_rows())))   // (+ the work plan)
            return rc;
    }
    if (!fused_quant && (rc = launch_quant(X, x_is_bf16, w.Xq, w.Xs, T, D, w.pos, k, shared ? n : -1, true, st))) return rc;
    const int ng = se1 - se0;
    const int *goffs = w.eoffs + se0;
    // the two grouped-GEMM launches stage their result rows as bf16 for the combine (see ld_y4)
    const int ybf = (use_tc && !decode_kernel) ? stage_y_bf16() : 0;
    if (!use_tc) {
        if ((rc = launch_gateup_gemv(Wg, Wu, ng, goffs, shared ? Sg : nullptr, shared ? Su : nullptr, w.soffs, w.Xq,
                                     w.Xs, w.Hq, w.Hs, D, FF, st)))
            return rc;
        if ((rc = launch_down_gemv(Wd, ng, goffs, shared ? Sd : nullptr, w.soffs, w.Hq, w.Hs, w.Y, D, FF, st)))
            return rc;
    } else {
        if (decode_kernel) {
            if ((rc = launch_ffn_fused_small(Wg, Wu, Wd, shared ? Sg : nullptr, shared ? Su : nullptr, shared ? Sd : nullptr,
                                             ng, R, w.Xq, w.Xs, w.Hq, w.Hs, w.Y, D, FF, w.plan, w.status + 0, nullptr, st)))
                return rc;
        } else {
        if ((rc = launch_gateup_tc(Wg, Wu, shared ? Sg : nullptr, shared ? Su : nullptr, ng, R, T, w.Xq, w.Xs, w.Hq, w.Hs,
                                   D, FF, w.plan, w.status + 0, st)))
            return rc;
        if ((rc = launch_down_tc(Wd, shared ? Sd : nullptr, ng, R, T, w.Hq, w.Hs, w.Y, D, FF, w.plan, w.status + 1, st, ybf)))
            return rc;
        }
    }
    const float *shg = (shared && shgate_col >= 0) ? logits + shgate_col : nullptr;
    // (behind the decode kernel the combine may read the routing results before its grid dependency resolves:
    // that kernel lets its successor start only after it has seen the front end complete)
    if (post.h) {
        if ((rc = launch_combine_add_rmsnorm(out, w.Y, w.pos, w.wt, shared ? y_row(w.Y, n, D, ybf) : nullptr, shg, logit_stride,
                                             post.h, post.w_next, post.eps, post.x_next, D, k, T, decode_kernel, st, ybf)))
            return rc;
    } else if ((rc = launch_combine(out, w.Y, w.pos, w.wt, shared ? y_row(w.Y, n, D, ybf) : nullptr, shg, logit_stride, D, k,
                                    T, decode_kernel, st, ybf)))
        return rc;
    if (idx_out && (rc = ck(cudaMemcpyAsync(idx_out, w.idx, (size_t)n * 4, cudaMemcpyDeviceToDevice, st)))) return rc;
    if (wt_out && (rc = ck(cudaMemcpyAsync(wt_out, w.wt, (size_t)n * 4, cudaMemcpyDeviceToDevice, st)))) return rc;
    return Q36_MOE_OK;
}

}  // namespace q36

using namespace q36;

extern "C" {

const char *q36_moe_strerror(int s) {
    switch (s) {
        case Q36_MOE_OK: return "ok";
        case Q36_MOE_EINVAL: return "invalid argument";
        case Q36_MOE_ECUDA: return "CUDA error (see q36_moe_last_cuda_error)";
        case Q36_MOE_ENOSPACE: return "workspace too small";
        case Q36_MOE_EDEVICE: return "a bounded device-side wait gave up";
        case Q36_MOE_EUNSUPPORTED: return "input not supported by this path (see q36_gguf_last_error)";
        case Q36_MOE_EIO: return "file error (see q36_gguf_last_error)";
        default: return "unknown status";
    }
}
int q36_moe_last_cuda_error(void) { return last_cuda_error(); }
int q36_moe_abi_version(void) { return 2; }

uint64_t q36_moe_expert_stride(int M, int K) { return (uint64_t)M * (K / 2) + (uint64_t)M * (K / Q36_QK); }

int q36_moe_repack_mxfp4(const void *host_blocks, int K, int M, int e0, int e1, void *host_dst) {
    if (!host_blocks || !host_dst || K % Q36_QK || M <= 0 || e0 < 0 || e1 <= e0) return Q36_MOE_EINVAL;
    const uint64_t nbr = K / Q36_QK, qs_e = (uint64_t)M * (K / 2), es_e = (uint64_t)M * nbr;
    const uint8_t *src = (const uint8_t *)host_blocks;
    for (int ex = e0; ex < e1; ex++) {
        uint8_t *qd = (uint8_t *)host_dst + (uint64_t)(ex - e0) * (qs_e + es_e), *ed = qd + qs_e;
        const uint8_t *blk = src + (uint64_t)ex * M * nbr * 17;
        for (uint64_t i = 0; i < (uint64_t)M * nbr; i++, blk += 17) {
            ed[i] = blk[0];
            memcpy(qd + i * 16, blk + 1, 16);
        }
    }
    return Q36_MOE_OK;
}

int q36_moe_upload_mxfp4(const void *host_blocks, int K, int M, int e0, int e1, void *dev_dst) {
    if (!dev_dst) return Q36_MOE_EINVAL;
    const uint64_t bytes = (uint64_t)(e1 - e0) * q36_moe_expert_stride(M, K);
    void *tmp = malloc(bytes);
    if (!tmp) return Q36_MOE_ENOSPACE;
    int rc = q36_moe_repack_mxfp4(host_blocks, K, M, e0, e1, tmp);
    if (rc == Q36_MOE_OK) rc = ck(cudaMemcpy(dev_dst, tmp, bytes, cudaMemcpyHostToDevice));
    free(tmp);
    return rc;
}

int q36_moe_dequant_mxfp4(const void *W, int M, int K, float *out, void *stream) {
    if (!W || !out || K % Q36_QK) return Q36_MOE_EINVAL;
    return launch_dequant_mxfp4(W, M, K, out, (cudaStream_t)stream);
}

int q36_moe_router_topk(const float *logits, int n_expert, int k, int *idx, float *wt, float scale, int renorm,
                        int T, int row_stride, void *stream) {
    if (!logits || !idx || !wt || k <= 0 || k > 32 || k > n_expert) return Q36_MOE_EINVAL;
    if (!router_supports(n_expert)) return Q36_MOE_EINVAL;
    if (T < 0 || row_stride < n_expert) return Q36_MOE_EINVAL;
    return launch_router_topk(logits, n_expert, k, idx, wt, scale, renorm, T, row_stride, (cudaStream_t)stream);
}

int q36_moe_quant_e4m3(const void *X, int x_is_bf16, uint8_t *Xq, uint8_t *Xs, int T, int K, void *stream) {
    if (!X || !Xq || !Xs || K % Q36_QK || T < 0) return Q36_MOE_EINVAL;
    return launch_quant(X, x_is_bf16, Xq, Xs, T, K, nullptr, 0, -1, false, (cudaStream_t)stream);
}

uint64_t q36_moe_dispatch_ws_bytes(int n_entries, int n_expert) { return dispatch_ws_bytes(n_entries, n_expert); }

int q36_moe_dispatch(const int *expert_of_entry, int n_entries, int n_expert, int se0, int se1, int *ecount,
                     int *eoffs, int *elist, int *pos, void *ws, uint64_t ws_bytes, void *stream) {
    if (!ecount || !eoffs || !ws || n_entries < 0 || n_expert <= 0 || n_expert > DISPATCH_MAX_GROUPS) return Q36_MOE_EINVAL;
    if (n_entries > 0 && (!expert_of_entry || !elist || !pos)) return Q36_MOE_EINVAL;   // no entries: nothing to read or place
    if (se0 < 0 || se0 > se1 || se1 > n_expert) return Q36_MOE_EINVAL;
    if (ws_bytes < dispatch_ws_bytes(n_entries, n_expert)) return Q36_MOE_ENOSPACE;
    return launch_dispatch(expert_of_entry, n_entries, n_expert, se0, se1, ecount, eoffs, elist, pos, ws, nullptr, 0,
                           0, (cudaStream_t)stream);
}

int q36_moe_quant_scatter(const void *X, int x_is_bf16, const int *pos, int k, int shared_row0, uint8_t *Xq_rows,
                          uint8_t *Xs_rows, int T, int K, void *stream) {
    if (!X || !Xq_rows || !Xs_rows || (k > 0 && !pos) || K % Q36_QK || T < 0) return Q36_MOE_EINVAL;
    return launch_quant(X, x_is_bf16, Xq_rows, Xs_rows, T, K, pos, k, shared_row0, true, (cudaStream_t)stream);
}

uint64_t q36_moe_ffn_ws_bytes(int n_group, int R_max, int D, int FF) {
    (void)n_group; (void)R_max; (void)D; (void)FF;
    return 256 + tc_ws_bytes();
}

int q36_moe_one_launch_fits(int R_max, int n_group, int D, int FF) {
    if (R_max <= 0 || n_group <= 0 || D <= 0 || FF <= 0) return 0;
    return ffn_fused_small_fits(R_max, n_group, D, FF) ? 1 : 0;
}

int q36_moe_one_launch_rows(void) { return fused_rows_limit(); }

int q36_moe_expert_ffn_sorted(const void *Wg, const void *Wu, const void *Wd, int n_group, const int *goffs,
                              const void *Sg, const void *Su, const void *Sd, const int *soffs, int R_max,
                              const uint8_t *Xq_rows, const uint8_t *Xs_rows, uint8_t *Hq_rows, uint8_t *Hs_rows,
                              float *Y_rows, int D, int FF, int path, int stages, int max_group_rows, void *ws,
                              uint64_t ws_bytes, void *stream) {
    if (!Wg || !Wu || !Wd || !goffs || !Xq_rows || !Xs_rows || !Hq_rows || !Hs_rows || !Y_rows) return Q36_MOE_EINVAL;
    if (n_group <= 0 || n_group > DISPATCH_MAX_GROUPS || D % 128 || FF % 128 || R_max <= 0) return Q36_MOE_EINVAL;
    if (!(stages & 7) || (path != Q36_MOE_PATH_GEMV && path != Q36_MOE_PATH_TC)) return Q36_MOE_EINVAL;
    const bool shared = Sg && Su && Sd && soffs;
    cudaStream_t st = (cudaStream_t)stream;
    int rc;
    if (path == Q36_MOE_PATH_GEMV) {
        if ((stages & 1) && (rc = launch_gateup_gemv(Wg, Wu, n_group, goffs, shared ? Sg : nullptr, shared ? Su : nullptr,
                                                     soffs, Xq_rows, Xs_rows, Hq_rows, Hs_rows, D, FF, st)))
            return rc;
        if ((stages & 2) && (rc = launch_down_gemv(Wd, n_group, goffs, shared ? Sd : nullptr, soffs, Hq_rows, Hs_rows,
                                                   Y_rows, D, FF, st)))
            return rc;
        return Q36_MOE_OK;
    }
    if (!ws || ws_bytes < q36_moe_ffn_ws_bytes(n_group, R_max, D, FF)) return Q36_MOE_ENOSPACE;
    uint8_t *p = (uint8_t *)ws;
    int *status = (int *)p;
    void *plan = p + 256;
    const bool one_launch = stages == 3 && max_group_rows > 0 && ffn_fused_small_fits(R_max, n_group, D, FF) &&
                            (max_group_rows <= 16 || R_max <= fused_rows_limit());
    if ((rc = launch_tc_plan(goffs, n_group, shared ? soffs : nullptr, D, FF, plan, status, one_launch ? 16 : gateup_tile_rows(), st))) return rc;
    if (one_launch)
        return launch_ffn_fused_small(Wg, Wu, Wd, shared ? Sg : nullptr, shared ? Su : nullptr, shared ? Sd : nullptr, n_group,
                                      R_max, Xq_rows, Xs_rows, Hq_rows, Hs_rows, Y_rows, D, FF, plan, status, nullptr, st);
    const int mgr = max_group_rows > 0 ? max_group_rows : R_max;
    if ((stages & 1) && (rc = launch_gateup_tc(Wg, Wu, shared ? Sg : nullptr, shared ? Su : nullptr, n_group, R_max,
                                               mgr, Xq_rows, Xs_rows, Hq_rows, Hs_rows, D, FF, plan, status, st)))
        return rc;
    if ((stages & 2) && (rc = launch_down_tc(Wd, shared ? Sd : nullptr, n_group, R_max, mgr, Hq_rows, Hs_rows, Y_rows, D, FF,
                                             plan, status + 1, st)))
        return rc;
    return Q36_MOE_OK;
}

int q36_moe_combine(float *out, const float *Y_rows, const int *pos, const float *wt, const float *SH_rows,
                    const float *shgate, int shgate_stride, int D, int k, int T, void *stream) {
    if (!out || !Y_rows || !pos || !wt || D % 4 || k <= 0 || T < 0) return Q36_MOE_EINVAL;
    return launch_combine(out, Y_rows, pos, wt, SH_rows, shgate, shgate_stride, D, k, T, false, (cudaStream_t)stream);
}

uint64_t q36_moe_workspace_bytes(int T_max, int n_expert, int k, int D, int FF) {
    if (T_max <= 0 || n_expert <= 0 || k <= 0) return 0;
    return carve(nullptr, T_max, n_expert, k, D, FF).total;
}

int q36_moe_ws_reset(void *ws, void *stream) {
    if (!ws) return Q36_MOE_EINVAL;
    return ck(cudaMemsetAsync(ws, 0, 256, (cudaStream_t)stream));
}

int q36_moe_ws_status(const void *ws, void *stream) {
    if (!ws) return Q36_MOE_EINVAL;
    int h[4] = {0, 0, 0, 0};
    int rc = ck(cudaMemcpyAsync(h, ws, sizeof h, cudaMemcpyDeviceToHost, (cudaStream_t)stream));
    if (rc) return rc;
    if ((rc = ck(cudaStreamSynchronize((cudaStream_t)stream)))) return rc;
    if (h[0] | h[1] | h[2] | h[3]) {
        last_cuda_error() = 200000 + (h[0] ? h[0] : h[1] ? h[1] : h[2] ? h[2] : h[3]);   // which wait gave up
        return Q36_MOE_EDEVICE;
    }
    return Q36_MOE_OK;
}

int q36_moe_layer(const void *Wg, const void *Wu, const void *Wd, const void *Sg, const void *Su, const void *Sd,
                  int n_expert, int se0, int se1, int k, int D, int FF, const void *X, int x_is_bf16,
                  const float *logits, int logit_stride, int shgate_col, float route_scale, int inc_shared,
                  float *out, int *idx_out, float *wt_out, int T, int path, void *ws, uint64_t ws_bytes,
                  void *stream) {
    return layer_impl(Wg, Wu, Wd, Sg, Su, Sd, n_expert, se0, se1, k, D, FF, X, x_is_bf16, logits, logit_stride,
                      shgate_col, route_scale, inc_shared, out, idx_out, wt_out, T, path, ws, ws_bytes,
                      (cudaStream_t)stream);
}
int q36_moe_decode(const void *Wg, const void *Wu, const void *Wd, const void *Sg, const void *Su, const void *Sd,
                   int n_expert, int se0, int se1, int k, int D, int FF, const void *X, int x_is_bf16,
                   const float *logits, int logit_stride, int shgate_col, float route_scale, int inc_shared,
                   float *out, int T, void *ws, uint64_t ws_bytes, void *stream) {
    return layer_impl(Wg, Wu, Wd, Sg, Su, Sd, n_expert, se0, se1, k, D, FF, X, x_is_bf16, logits, logit_stride,
                      shgate_col, route_scale, inc_shared, out, nullptr, nullptr, T, Q36_MOE_PATH_AUTO, ws, ws_bytes,
                      (cudaStream_t)stream);
}
int q36_moe_prefill(const void *Wg, const void *Wu, const void *Wd, const void *Sg, const void *Su, const void *Sd,
                    int n_expert, int se0, int se1, int k, int D, int FF, const void *X, int x_is_bf16,
                    const float *logits, int logit_stride, int shgate_col, float route_scale, int inc_shared,
                    float *out, int T, void *ws, uint64_t ws_bytes, void *stream) {
    return layer_impl(Wg, Wu, Wd, Sg, Su, Sd, n_expert, se0, se1, k, D, FF, X, x_is_bf16, logits, logit_stride,
                      shgate_col, route_scale, inc_shared, out, nullptr, nullptr, T, Q36_MOE_PATH_AUTO, ws, ws_bytes,
                      (cudaStream_t)stream);
}

int q36_moe_pre_norm_router(float *h, const float *a, const float *norm_w, float eps, const float *router_w, int n_rows,
                            int gate_row, float *x, float *logits, int logit_stride, int T, int D, void *stream) {
    if (!h || !norm_w || !router_w || !x || !logits || T < 0) return Q36_MOE_EINVAL;
    return launch_pre_norm_router(h, a, norm_w, eps, router_w, n_rows, gate_row, x, logits, logit_stride, T, D, (cudaStream_t)stream);
}

int q36_moe_combine_add_rmsnorm(float *moe_out, const float *Y_rows, const int *pos, const float *wt, const float *SH_rows,
                                const float *shgate, int shgate_stride, float *h, const float *next_norm_w, float eps,
                                float *x_next, int D, int k, int T, void *stream) {
    if (!Y_rows || !pos || !wt || !h || !next_norm_w || !x_next || T < 0) return Q36_MOE_EINVAL;
    return launch_combine_add_rmsnorm(moe_out, Y_rows, pos, wt, SH_rows, shgate, shgate_stride, h, next_norm_w, eps, x_next, D, k, T,
                                      false, (cudaStream_t)stream);
}

// block workspace = [layer workspace][x: T*D f32][logits: T*(E+1) f32]
uint64_t q36_moe_block_workspace_bytes(int T_max, int n_expert, int k, int D, int FF) {
    const uint64_t base = q36_moe_workspace_bytes(T_max, n_expert, k, D, FF);
    if (!base) return 0;
    return base + al((uint64_t)T_max * D * 4) + al((uint64_t)T_max * (n_expert + 1) * 4);
}

int q36_moe_block(const void *Wg, const void *Wu, const void *Wd, const void *Sg, const void *Su, const void *Sd, int n_expert,
                  int se0, int se1, int k, int D, int FF, const float *post_norm_w, const float *router_w,
                  const float *next_norm_w, float eps, float route_scale, int inc_shared, float *h, const float *a,
                  float *x_next, float *moe_out, int T, void *ws, uint64_t ws_bytes, void *stream) {
    if (!post_norm_w || !router_w || !next_norm_w || !h || !x_next || !ws || T <= 0 || n_expert <= 0 || k <= 0) return Q36_MOE_EINVAL;
    const uint64_t base = q36_moe_workspace_bytes(T, n_expert, k, D, FF);
    if (!base) return Q36_MOE_EINVAL;
    if (q36_moe_block_workspace_bytes(T, n_expert, k, D, FF) > ws_bytes) return Q36_MOE_ENOSPACE;
    float *x = (float *)((uint8_t *)ws + base);
    float *logits = (float *)((uint8_t *)x + al((uint64_t)T * D * 4));
    const int stride = n_expert + 1;
    cudaStream_t st = (cudaStream_t)stream;
    int rc;
    if ((rc = launch_pre_norm_router(h, a, post_norm_w, eps, router_w, stride, n_expert, x, logits, stride, T, D, st))) return rc;
    return layer_impl(Wg, Wu, Wd, Sg, Su, Sd, n_expert, se0, se1, k, D, FF, x, 0, logits, stride, n_expert, route_scale, inc_shared,
                      moe_out, nullptr, nullptr, T, Q36_MOE_PATH_AUTO, ws, base, st, PostNorm{h, next_norm_w, eps, x_next});
}

uint64_t q36_moe_host_io_bytes(int T, int D, int logit_stride, int x_is_bf16) {
    return al((uint64_t)T * D * (x_is_bf16 ? 2 : 4)) + al((uint64_t)T * logit_stride * 4) + al((uint64_t)T * D * 4);
}

int q36_moe_layer_host(const void *Wg, const void *Wu, const void *Wd, const void *Sg, const void *Su,
                       const void *Sd, int n_expert, int se0, int se1, int k, int D, int FF, const void *host_X,
                       int x_is_bf16, const float *host_logits, int logit_stride, int shgate_col, float route_scale,
                       int inc_shared, float *host_out, int T, int path, void *dev_io, void *ws, uint64_t ws_bytes,
                       void *stream) {
    if (!host_X || !host_logits || !host_out || !dev_io || T <= 0) return Q36_MOE_EINVAL;
    cudaStream_t st = (cudaStream_t)stream;
    const uint64_t xb = (uint64_t)T * D * (x_is_bf16 ? 2 : 4), lb = (uint64_t)T * logit_stride * 4,
                   ob = (uint64_t)T * D * 4;
    uint8_t *dX = (uint8_t *)dev_io, *dL = dX + al(xb), *dO = dL + al(lb);
    int rc;
    if ((rc = ck(cudaMemcpyAsync(dX, host_X, xb, cudaMemcpyHostToDevice, st)))) return rc;
    if ((rc = ck(cudaMemcpyAsync(dL, host_logits, lb, cudaMemcpyHostToDevice, st)))) return rc;
    if ((rc = layer_impl(Wg, Wu, Wd, Sg, Su, Sd, n_expert, se0, se1, k, D, FF, dX, x_is_bf16, (const float *)dL,
                         logit_stride, shgate_col, route_scale, inc_shared, (float *)dO, nullptr, nullptr, T, path, ws,
                         ws_bytes, st)))
        return rc;
    if ((rc = ck(cudaMemcpyAsync(host_out, dO, ob, cudaMemcpyDeviceToHost, st)))) return rc;
    if ((rc = ck(cudaStreamSynchronize(st)))) return rc;
    if (pick_path(path, T) == Q36_MOE_PATH_TC) return q36_moe_ws_status(ws, stream);
    return Q36_MOE_OK;
}

// A stack of layers from host buffers: what a serving loop that keeps activations on the host would call per step.
int q36_moe_stack_host(int n_layers, const void *const *Wg, const void *const *Wu, const void *const *Wd, const void *const *Sg,
                       const void *const *Su, const void *const *Sd, int n_expert, int se0, int se1, int k, int D, int FF,
                       const void *host_X, int x_is_bf16, const float *host_logits, int logit_stride, int shgate_col,
                       float route_scale, int inc_shared, float *host_out, int T, int path, void *dev_io, void *ws,
                       uint64_t ws_bytes, void *stream) {
    if (n_layers <= 0 || !Wg || !Wu || !Wd || !host_X || !host_logits || !host_out || !dev_io || T <= 0) return Q36_MOE_EINVAL;
    cudaStream_t st = (cudaStream_t)stream;
    const uint64_t xb = (uint64_t)T * D * (x_is_bf16 ? 2 : 4), lb = (uint64_t)T * logit_stride * 4, ob = (uint64_t)T * D * 4;
    // device staging: all layers' X, then all logits, then all outputs: three copies per step
    uint8_t *dX = (uint8_t *)dev_io, *dL = dX + al(xb * n_layers), *dO = dL + al(lb * n_layers);
    int rc;
    if ((rc = ck(cudaMemcpyAsync(dX, host_X, xb * n_layers, cudaMemcpyHostToDevice, st)))) return rc;
    if ((rc = ck(cudaMemcpyAsync(dL, host_logits, lb * n_layers, cudaMemcpyHostToDevice, st)))) return rc;
    for (int l = 0; l < n_layers; l++)
        if ((rc = layer_impl(Wg[l], Wu[l], Wd[l], Sg ? Sg[l] : nullptr, Su ? Su[l] : nullptr, Sd ? Sd[l] : nullptr, n_expert, se0, se1,
                             k, D, FF, dX + xb * l, x_is_bf16, (const float *)(dL + lb * l), logit_stride, shgate_col, route_scale,
                             inc_shared, (float *)(dO + ob * l), nullptr, nullptr, T, path, ws, ws_bytes, st)))
            return rc;
    if ((rc = ck(cudaMemcpyAsync(host_out, dO, ob * n_layers, cudaMemcpyDeviceToHost, st)))) return rc;
    if ((rc = ck(cudaStreamSynchronize(st)))) return rc;
    if (pick_path(path, T) == Q36_MOE_PATH_TC) return q36_moe_ws_status(ws, stream);
    return Q36_MOE_OK;
}
uint64_t q36_moe_stack_host_io_bytes(int n_layers, int T, int D, int logit_stride, int x_is_bf16) {
    if (n_layers <= 0 || T <= 0) return 0;
    return al((uint64_t)n_layers * T * D * (x_is_bf16 ? 2 : 4)) + al((uint64_t)n_layers * T * logit_stride * 4) +
           al((uint64_t)n_layers * T * D * 4);
}

int q36_moe_gather_rows(const void *src, const int *index, void *dst, int n_rows, int row_bytes, void *stream) {
    if (!src || !index || !dst || row_bytes % 16 || n_rows < 0) return Q36_MOE_EINVAL;
    return launch_gather_rows(src, index, dst, n_rows, row_bytes, (cudaStream_t)stream);
}

int q36_moe_tc_selftest(const uint8_t *A_codes_scales, const uint8_t *B_q, const uint8_t *B_s, float *Dout, int N,
                        int K, void *ws, uint64_t ws_bytes, void *stream) {
    // A_codes_scales: one "expert" of 128 rows in the split layout
    // [128][K/2] codes then [128][K/32] scales; Dout: [N][128] (token-major).
    if (!A_codes_scales || !B_q || !B_s || !Dout || !ws || N <= 0 || N > 4096 || K % 512) return Q36_MOE_EINVAL;
    if (ws_bytes < 512 + tc_ws_bytes()) return Q36_MOE_ENOSPACE;
    cudaStream_t st = (cudaStream_t)stream;
    int h[2] = {0, N};
    int *goffs = (int *)((uint8_t *)ws + 256);
    int rc;
    if ((rc = ck(cudaMemsetAsync(ws, 0, 16, st)))) return rc;
    if ((rc = ck(cudaMemcpyAsync(goffs, h, sizeof h, cudaMemcpyHostToDevice, st)))) return rc;
    if ((rc = launch_tc_plan(goffs, 1, nullptr, 128, K, (uint8_t *)ws + 512, (int *)ws, 0, st))) return rc;
    if ((rc = launch_down_tc(A_codes_scales, nullptr, 1, N, N, B_q, B_s, Dout, 128, K, (uint8_t *)ws + 512, (int *)ws + 1, st)))
        return rc;
    return q36_moe_ws_status(ws, stream);
}

int q36_moe_selftest_wait_timeout(void *ws, void *stream) {
    if (!ws) return Q36_MOE_EINVAL;
    int rc = launch_wait_timeout((int *)ws, (cudaStream_t)stream);
    if (rc) return rc;
    return q36_moe_ws_status(ws, stream);
}

}  // extern "C"
