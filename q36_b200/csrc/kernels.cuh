// Internal launcher prototypes shared by the translation units of libq36moe.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace q36 {

// Expert-parallel hooks of the two decode-sized kernels (all pointers device memory; peers == nullptr: not used).
// Windows: peers[r] is rank r's exchange window as mapped on this device; offsets are the same on every rank and
// come in pairs indexed by the parity of the call number ctl[0] + 1.  slot_major: index the slot blocks by the
// OTHER rank instead of this one (local staging for the NCCL transport).
struct EpSendArgs {     // front end: quantised rows straight into the destination ranks' windows
    uint8_t *const *peers;
    uint64_t rows0, rows1, hdr0, hdr1;
    int *ctl, *ypos;
    int me, world, per, cap, slot_major;
};
struct EpReturnArgs {   // FFN: result rows of the sorted rows [0, n_map) straight into their home ranks' windows
    uint8_t *const *peers;
    uint64_t ret0, ret1, rhdr0, rhdr1;
    int *ctl;
    const int *rowmap;  // sorted row -> received slot (source rank * cap + j)
    int n_map, me, world, cap, slot_major;
};

constexpr int DISPATCH_MAX_GROUPS = 512;  // upper bound on expert groups per call

bool router_supports(int n_expert);   // moe_api.cu: expert counts the router kernels are built for

// moe_route.cu
int launch_router_topk(const float *logits, int n_expert, int k, int *idx, float *wt, float scale,
                       int renorm, int T, int row_stride, cudaStream_t st);
uint64_t dispatch_ws_bytes(int n_entries, int n_expert);
// soffs (optional): receives {s0, s1}, the row range of the shared expert's group
// plan (optional): the tensor-core work plan of the groups [se0, se1) (+ the group [s0, s1) when s1 > s0) is written by
// the scan kernel as well, for the launches of D x FF matrices with token tiles of plan_tile_rows (0: 112 / 128)
int launch_dispatch(const int *eid, int n, int n_expert, int se0, int se1, int *ecount, int *eoffs,
                    int *elist, int *pos, void *ws, int *soffs, int s0, int s1, cudaStream_t st, void *plan = nullptr, int D = 0,
                    int FF = 0, int plan_tile_rows = 0);
int launch_quant(const void *X, int bf16, uint8_t *Xq, uint8_t *Xs, int T, int K, const int *pos,
                 int k, int shared_row0, bool scatter, cudaStream_t st);

// Router + dispatch (+ tensor-core work plan when plan != NULL, + quantise-and-scatter of X when X != NULL)
// in one single-block launch; T * k <= 1024.
// decode front end as one thread-block cluster (router, dispatch, plan and the row quantiser in one launch);
// returns EINVAL without launching when the sizes are outside what it holds
int launch_front_decode(const float *logits, int n_expert, int k, float scale, int T, int row_stride, int *idx, float *wt,
                        int *ecount, int *eoffs, int *elist, int *pos, int *soffs, int s0, int s1, void *plan, int D, int FF,
                        int *status, const void *X, int x_is_bf16, uint8_t *Xq, uint8_t *Xs, int shared_row0, int put_k,
                        cudaStream_t st, const EpSendArgs *ep = nullptr);
// expert-parallel: wait (bounded) for every source rank's header of this call in the exchange window, bucket the
// received slots by local expert, write the work plan; counts_out[world] receives the per-source slot counts
int launch_ep_recv_plan(const void *win, uint64_t off_hdr0, uint64_t off_hdr1, uint64_t off_rows0, uint64_t off_rows1, const int *ctr,
                        int world, int cap, int row_bytes, int eid_off, unsigned limit, int *status, int n_expert, int se0, int se1,
                        int *ecount, int *eoffs, int *elist, int *pos, int *soffs, int s0, int s1, void *plan, int D, int FF,
                        int plan_tile_rows, int *counts_out, cudaStream_t st);
int launch_front_small(const float *logits, int n_expert, int k, float scale, int T, int row_stride, int se0, int se1,
                       int *idx, float *wt, int *ecount, int *eoffs, int *elist, int *pos, int *soffs, int s0, int s1,
                       void *plan, int D, int FF, int *status, const void *X, int x_is_bf16, uint8_t *Xq, uint8_t *Xs,
                       int shared_row0, int plan_tile_rows, cudaStream_t st);

// moe_gemv.cu
// Sg/Su/Sd + soffs[2]: one extra group (the shared expert) with its own planes and row range, or NULL
int launch_gateup_gemv(const void *Wg, const void *Wu, int n_group, const int *goffs, const void *Sg,
                       const void *Su, const int *soffs, const uint8_t *Xq, const uint8_t *Xs,
                       uint8_t *Hq, uint8_t *Hs, int D, int FF, cudaStream_t st);
int launch_down_gemv(const void *Wd, int n_group, const int *goffs, const void *Sd, const int *soffs,
                     const uint8_t *Hq, const uint8_t *Hs, float *Y, int D, int FF, cudaStream_t st);
int launch_combine(float *out, const float *Y, const int *pos, const float *wt, const float *SH,
                   const float *shgate, int shgate_stride, int D, int k, int T, bool early_meta, cudaStream_t st, int y_bf16 = 0);
int launch_gather_rows(const void *src, const int *index, void *dst, int n_rows, int row_bytes,
                       cudaStream_t st);
int launch_dequant_mxfp4(const void *W, int M, int K, float *out, cudaStream_t st);

// moe_block.cu: the steps before and after the expert computation
// h += a (a may be NULL); x = rmsnorm(h) * norm_w; logits[:, 0:n_rows) = router_w . x.  gate_row: index of the
// shared-gate row inside router_w (must be the last row, n_rows - 1) or -1.
int launch_pre_norm_router(float *h, const float *a, const float *norm_w, float eps, const float *router_w, int n_rows,
                           int gate_row, float *x, float *logits, int logit_stride, int T, int D, cudaStream_t st);
int launch_combine_add_rmsnorm(float *moe_out, const float *Y, const int *pos, const float *wt, const float *SH,
                               const float *shgate, int shgate_stride, float *h, const float *w_next, float eps, float *x_next,
                               int D, int k, int T, bool early_meta, cudaStream_t st, int y_bf16 = 0);

// moe_tc.cu
// One plan per grouped-FFN call (groups = n_group routed + the shared expert's when soffs != NULL), then the
// gate/up and the down launch read it.  status: 4 ints, [0] gate/up, [1] down.
uint64_t tc_ws_bytes();
// tile_rows: 0 for the two grouped-GEMM launches, 16 for the one-launch decode kernel
int launch_tc_plan(const int *goffs, int n_group, const int *soffs, int D, int FF, void *plan, int *status, int tile_rows,
                   cudaStream_t st);
int launch_gateup_tc(const void *Wg, const void *Wu, const void *Sg, const void *Su, int n_group, int R_max,
                     int max_group_rows, const uint8_t *Xq, const uint8_t *Xs, uint8_t *Hq, uint8_t *Hs, int D, int FF, const void *plan,
                     int *status, cudaStream_t st);
// a 32-thread kernel that waits (1024 polls) on a barrier nobody completes, records the give-up in status[0] and returns
int launch_wait_timeout(int *status, cudaStream_t st);
int launch_down_tc(const void *Wd, const void *Sd, int n_group, int R_max, int max_group_rows, const uint8_t *Hq, const uint8_t *Hs,
                   float *Y, int D, int FF, const void *plan, int *status, cudaStream_t st, int y_bf16 = 0);
// 1 when prefill-sized calls of the whole-layer entries stage their result rows as bf16 (Q36_Y_BF16=1 in the
// environment; the default is f32, which keeps the layer at 1e-7 of a float64 product instead of 1e-3)
int stage_y_bf16();

// host helpers of moe_tc.cu shared with moe_tc_fused.cu
int make_map_codes(CUtensorMap *m, const void *base, int M, int K, int n_group, uint64_t expert_stride);
int make_map_rows(CUtensorMap *m, const void *base, int R, int K, int box_rows);
// the same planes seen as [.., K / 128 steps, rows, 128 elements] so that ONE copy fetches `ksteps` consecutive
// K steps as consecutive 128-byte-swizzled tiles (coordinates: 0, row, K step [, expert])
int make_map_codes_ksteps(CUtensorMap *m, const void *base, int M, int K, int n_group, uint64_t expert_stride, int ksteps);
int make_map_rows_ksteps(CUtensorMap *m, const void *base, int R, int K, int box_rows, int ksteps);
int sm_count();            // of the CURRENT device
int current_device();      // -1 when it cannot be determined or is beyond MAX_DEVICES
constexpr int MAX_DEVICES = 64;   // per-device state of the library is kept for device ordinals below this
// once per (kernel, device): allow `bytes` of dynamic shared memory; done = 64 flags owned by the caller
int ensure_smem_attr(const void *kernel, int bytes, bool *done);

// moe_tc_fused.cu: gate/up and down of decode-sized groups (every group <= 16 rows) in ONE persistent launch
bool ffn_fused_small_fits(int R_max, int n_group, int D, int FF);   // does launch_ffn_fused_small take this call?
int ffn_fused_small_grid(int R_max, int n_group, int D, int FF);   // CTAs of that launch
int gateup_tile_rows();           // token rows per tile a two-launch call's plan must be cut in (0: defaults)
int fused_rows_limit();            // policy: rows up to which that kernel is preferred when groups may exceed 16 rows   // largest R_max launch_ffn_fused_small accepts
int launch_ffn_fused_small(const void *Wg, const void *Wu, const void *Wd, const void *Sg, const void *Su,
                           const void *Sd, int n_group, int R_max, const uint8_t *Xq, const uint8_t *Xs, uint8_t *Hq,
                           uint8_t *Hs, float *Y, int D, int FF, void *plan, int *status, const EpReturnArgs *ep, cudaStream_t st);

}  // namespace q36
