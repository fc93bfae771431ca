/* q36_moe.h -- C ABI of the B200 (sm_100a) MXFP4-weight / E4M3-activation
 * mixture-of-experts expert path.
 *
 * The q36 engine has no plugin registry: its MoE path is a fixed sequence of
 * kernel launches inside two static functions, moe_ffn (T = 1 decode,
 * q36_engine.cu:1592-1654) and pf_moe_block (batched / prefill,
 * q36_engine.cu:3423-3472), over weights laid out by upload()
 * (q36_engine.cu:202-228).  Each entry point below replaces one of those
 * launches (or one whole function) and keeps the conventions of the engine's
 * existing extern "C" launchers (q36_cuda.cu:226-292): raw device pointers,
 * int dimensions, no structs across the boundary, launch-only (no host
 * synchronisation, no allocation, capturable in a CUDA graph).  Differences:
 * every call takes an explicit stream (a cudaStream_t passed as void*; NULL
 * = the legacy default stream) and returns a status instead of exiting.
 *
 * Conventions
 *   - All pointers are DEVICE pointers unless the name starts with "host_".
 *   - Weights use the engine's "mxfp4-split" layout (`dw.elayout == 2`):
 *     per resident expert [codes: M*K/2 bytes, row-major, GGUF nibble order]
 *     [scales: M*K/32 E8M0 bytes, row-major]; expert stride M*K*17/32 bytes;
 *     only experts [se0, se1) are resident and expert `se0` sits at offset 0.
 *   - Activations are quantised per (row, 32-element block) to E4M3 codes
 *     plus one UE8M0 scale byte, value = e4m3(code) * 2^(scale-127).
 *   - "hw order": inside a 32-block, logical element j is stored at position
 *     2j (j < 16) or 2(j-16)+1 (j >= 16), the element order of the MXFP4 code
 *     bytes.  Buffers that only this library reads and writes use hw order;
 *     q36_moe_quant_e4m3 writes logical order like the engine's kernel.
 *   - Experts outside [se0, se1) contribute zeros (q36_engine.cu:763-766).
 *   - Weight scale bytes 0..254 are supported; byte 255 (NaN in the OCP MX
 *     convention, 2^127 in ggml's) is not and gives unspecified values.
 *   - The library keeps its per-device state (multiprocessor count, kernel
 *     attributes) for the device that is current at the call, so one host
 *     thread may drive several devices in turn with cudaSetDevice, as
 *     q36_multi_prefill does (q36_engine.cu:4261-4306).
 */
#ifndef Q36_MOE_H
#define Q36_MOE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define Q36_MOE_OK 0
#define Q36_MOE_EINVAL (-1)   /* bad argument (NULL, size not supported)        */
#define Q36_MOE_ECUDA (-2)    /* a CUDA call failed: q36_moe_last_cuda_error()  */
#define Q36_MOE_ENOSPACE (-3) /* workspace smaller than q36_moe_workspace_bytes */
#define Q36_MOE_EDEVICE (-4)  /* a bounded device-side wait gave up             */
#define Q36_MOE_EUNSUPPORTED (-5) /* well-formed input this path does not take (a tensor type, a shape) */
#define Q36_MOE_EIO (-6)      /* a file could not be opened, mapped or parsed: q36_gguf_last_error() */

/* Path selection for the grouped expert FFN. */
#define Q36_MOE_PATH_AUTO 0
#define Q36_MOE_PATH_GEMV 1   /* streaming SIMT GEMV (decode-sized groups)      */
#define Q36_MOE_PATH_TC 2     /* tcgen05 block-scaled grouped GEMM (prefill)    */

const char *q36_moe_strerror(int status);
int q36_moe_last_cuda_error(void);
/* Library ABI version; bumped when a signature changes. */
int q36_moe_abi_version(void);

/* ---- weights ------------------------------------------------------------
 * Replaces the MXFP4 branch of upload() (q36_engine.cu:202-228). */

/* Bytes per expert in the split layout: M*K/2 + M*K/32. */
uint64_t q36_moe_expert_stride(int M, int K);
/* Host -> host: GGUF block_mxfp4 array [n_expert][M][K/32] (17 B blocks,
 * q36.h:114) -> split planes of experts [e0, e1) in host_dst. */
int q36_moe_repack_mxfp4(const void *host_blocks, int K, int M, int e0, int e1, void *host_dst);
/* Host -> device: same, then copies into the caller's device buffer dev_dst
 * of (e1-e0)*q36_moe_expert_stride(M,K) bytes.  Synchronous, like upload(). */
int q36_moe_upload_mxfp4(const void *host_blocks, int K, int M, int e0, int e1, void *dev_dst);
/* Device: split planes -> f32 [n_rows][K] (row r of the expert at W).  The
 * on-device form of q36_deq_row(Q36_GGML_MXFP4, ...) (q36_dequant.cuh:168-181),
 * used to prove bit-exact dequantisation. */
int q36_moe_dequant_mxfp4(const void *W, int M, int K, float *out, void *stream);

/* ---- on-disk format in: GGUF ----------------------------------------------
 * Replaces, for this path, the engine's GGUF v3 reader (gguf.c:129-261), its
 * tensor binding by name (q36_model.c:62-75) and the MXFP4 branch of upload()
 * (q36_engine.cu:202-228).  The file is mapped read-only; nothing is copied
 * until a tensor is repacked for the device.  Messages for Q36_MOE_EIO /
 * Q36_MOE_EUNSUPPORTED come from q36_gguf_last_error() (per thread). */
int q36_gguf_open(const char *path, void **gguf_out);
int q36_gguf_close(void *gguf);
const char *q36_gguf_last_error(void);
/* Directory entry of one tensor: ggml type id (q36.h:133-141), dimensions
 * (fastest first, unused ones 1), pointer into the mapping, bytes on disk.
 * Any out pointer may be NULL. */
int q36_gguf_tensor(const void *gguf, const char *name, int *ggml_type, int *n_dims, uint64_t *dims4,
                    const void **host_data, uint64_t *nbytes);
/* Integer metadata value (u32/i32/u64/i64 keys such as "general.alignment"). */
int q36_gguf_meta_u32(const void *gguf, const char *key, uint32_t *out);
/* Shapes of blk.<layer>.ffn_{gate,up,down}_exps.weight: gate/up [K=D, M=FF, E],
 * down [K=FF, M=D, E] (q36_model.h:75-77); ggml_types3 (or NULL) receives the
 * three tensor types. */
int q36_moe_gguf_layer_shape(const void *gguf, int layer, int *n_expert, int *D, int *FF, int *ggml_types3);
/* Experts [e0, e1) of the three tensors -> split planes in the caller's
 * device buffers of (e1-e0)*q36_moe_expert_stride(...) bytes each.  MXFP4
 * tensors only: the published model's Q5_K / Q6_K down projections
 * (requantised to Q8 by the engine, q36_engine.cu:229-252) return
 * Q36_MOE_EUNSUPPORTED.  Synchronous. */
int q36_moe_gguf_upload_layer(const void *gguf, int layer, int e0, int e1, void *dev_Wg, void *dev_Wu,
                              void *dev_Wd);
/* blk.<layer>.ffn_{gate,up,down}_shexp.weight as one-expert split planes;
 * MXFP4 only (the published model stores them as Q8_0: Q36_MOE_EUNSUPPORTED). */
int q36_moe_gguf_upload_shared(const void *gguf, int layer, void *dev_Sg, void *dev_Su, void *dev_Sd);
/* Router rows and the shared-gate row as ONE f32 matrix [n_expert + 1][D], the
 * concatenation the engine makes at load (q36_engine.cu:1599-1601), from
 * blk.<layer>.ffn_gate_inp.weight [D, E] and ffn_gate_inp_shexp.weight [D]
 * (F32 or BF16, widened). */
int q36_moe_gguf_upload_router(const void *gguf, int layer, float *dev_router);
/* Any F32 / BF16 tensor of n elements (norm weights) -> f32 on the device. */
int q36_moe_gguf_upload_f32(const void *gguf, const char *name, float *dev_dst, uint64_t n);

/* ---- stages -------------------------------------------------------------- */

/* k_router_topk (q36_ops.cuh:397-431): per row softmax statistics over
 * n_expert (256, 128, 64 or 32; anything else is Q36_MOE_EINVAL here and in
 * the whole-layer entries) logits, top-k (k <= 8) on the raw logits in descending
 * order with ties to the lower index, weights exp(v-m)/s, renormalised to
 * sum `scale` when renorm != 0.  logits row t starts at t*row_stride. */
int q36_moe_router_topk(const float *logits, int n_expert, int k, int *idx, float *wt,
                        float scale, int renorm, int T, int row_stride, void *stream);

/* k_quant_e4m3 (q36_engine.cu:2412-2428): X [T][K] (f32, or bf16 when
 * x_is_bf16) -> Xq [T][K] E4M3 bytes in logical order, Xs [T][K/32] UE8M0.
 * The shared exponent is the exact integer ceil(log2(amax/448)). */
int q36_moe_quant_e4m3(const void *X, int x_is_bf16, uint8_t *Xq, uint8_t *Xs, int T, int K,
                       void *stream);

/* k_moe_dispatch (q36_engine.cu:3387-3392) made deterministic: buckets the
 * n_entries ids (entry i = t*k + s) by expert in ascending-id order.
 *   ecount[n_expert]   entries per expert (0 outside [se0,se1))
 *   eoffs[n_expert+1]  exclusive prefix sum of ecount
 *   elist[n_entries]   packed buckets: elist[eoffs[e] + p] = p-th entry of e
 *   pos[n_entries]     inverse: row of entry i in elist, -1 if not resident
 * 0 <= se0 <= se1 <= n_expert <= 512; ids outside [se0, se1) or negative are
 * not resident.  ws: q36_moe_dispatch_ws_bytes(n_entries, n_expert) bytes of scratch. */
uint64_t q36_moe_dispatch_ws_bytes(int n_entries, int n_expert);
int q36_moe_dispatch(const int *expert_of_entry, int n_entries, int n_expert, int se0, int se1,
                     int *ecount, int *eoffs, int *elist, int *pos, void *ws, uint64_t ws_bytes,
                     void *stream);

/* No counterpart in the reference.  q36_moe_dispatch for callers that have no
 * scratch to hand over and may not allocate any: code that runs in the
 * engine's per-step path, where every buffer was sized and allocated once at
 * engine creation (q36_engine.cu:1467-1512) and an allocation could
 * synchronise the device in the middle of a step (the engine caches its own
 * for that reason, q36_cuda.cu:285-287), or a host that only passes its input
 * and output arrays through a fixed plugin signature.  The scratch is a
 * 96 KiB array built into the library image (held by every GPU that loads the
 * library until the process exits); the call allocates and frees nothing.
 *   Limits: n_entries <= 16384, n_expert <= 512; larger sizes return
 *   Q36_MOE_ENOSPACE with a message on stderr.
 *   The first call on each device looks up the array's device address; make
 *   that first call before starting any stream capture.
 *   Every call shares the one array: two calls whose kernels overlap on the
 *   GPU (different streams, no ordering between them) race on it.  Calls on
 *   one stream, or otherwise ordered, are safe.  Nothing in the array needs
 *   clearing between calls.
 * Outputs are identical to q36_moe_dispatch's. */
#define Q36_MOE_NOALLOC_MAX_ENTRIES 16384
int q36_moe_dispatch_noalloc(const int *expert_of_entry, int n_entries, int n_expert, int se0,
                             int se1, int *ecount, int *eoffs, int *elist, int *pos, void *stream);

/* Quantises X [T][K] and writes every token's row to the rows of the sorted
 * space that its entries occupy: for s < k row pos[t*k+s] (skipped when
 * negative) and, when shared_row0 >= 0, row shared_row0 + t.  Rows are
 * written in hw order: Xq_rows [R][K], Xs_rows [R][K/32].  Fuses
 * k_quant_e4m3 with the gather the engine's GEMM does by `elist`
 * (q36_engine.cu:2475-2483). */
int q36_moe_quant_scatter(const void *X, int x_is_bf16, const int *pos, int k, int shared_row0,
                          uint8_t *Xq_rows, uint8_t *Xs_rows, int T, int K, void *stream);

/* The grouped expert FFN over rows already sorted by expert:
 *   for each group g (rows [goffs[g], goffs[g+1])), weights Wg/Wu/Wd of
 *   expert g:  h = silu(Wg x) * (Wu x); (hq,hs) = quant_e4m3(h);
 *   y = Wd dequant(hq,hs)
 * Replaces k_expert_gemv2 + k_silu_mul_slots + k_expert_gemv
 * (q36_engine.cu:752-783, 744-746, 711-742) for decode-sized groups and
 * k_gemm_expert_mma x2 + k_silu_mul + k_gemm_expert_tc (:2435-2524,
 * q36_ops.cuh:65, :2723-2766) for prefill-sized ones.
 *   Wg, Wu: [n_group] experts of [FF][D]; Wd: [n_group] of [D][FF]
 *   goffs[n_group+1]: row offsets (device); Xq_rows/Xs_rows: hw order
 *   Hq_rows [R][FF], Hs_rows [R][FF/32]: quantised SwiGLU output (hw order)
 *   Y_rows [R][D] f32
 * path: Q36_MOE_PATH_GEMV or Q36_MOE_PATH_TC.  ws (tensor-core path only):
 * q36_moe_ffn_ws_bytes(...) bytes; its first 256 bytes are the sticky device
 * status words (q36_moe_ws_reset once after allocation, q36_moe_ws_status). */
uint64_t q36_moe_ffn_ws_bytes(int n_group, int R_max, int D, int FF);
/* 1 when the one-launch decode kernel takes a call of R_max rows in n_group
 * (+ 1 shared) groups with these matrix sizes, else 0 (then the two
 * grouped-GEMM launches run): it needs D, FF <= 2048 and multiples of 512, and
 * a per-block tile table that holds the call. */
int q36_moe_one_launch_fits(int R_max, int n_group, int D, int FF);
/* The row count (sorted rows incl. the shared expert's) up to which the
 * whole-layer entries prefer that kernel when it fits: measured, 4096. */
int q36_moe_one_launch_rows(void);
/* Sg/Su/Sd (or NULL): one extra group, the shared expert, with its own planes
 * and the row range [soffs[0], soffs[1]) (device ints).  stages: bit 0 runs
 * gate/up + SwiGLU, bit 1 runs down; 3 = both (the intermediate Hq/Hs is the
 * hand-over, so the halves can be launched and timed separately); 4 alone
 * does only the set-up both halves share on the tensor-core path (status
 * words, work plan), so that a benchmark can take it out of a timing.
 * max_group_rows: an upper bound on the rows of any single group when the
 * caller knows one (decode: the number of tokens), else 0.  With the
 * tensor-core path, stages == 3 and a bound given, gate/up and down run as
 * ONE persistent launch (token tiles of 16 rows) up to 4096 rows in all,
 * where the two launches with their 112/128-row token tiles take over. */
int q36_moe_expert_ffn_sorted(const void *Wg, const void *Wu, const void *Wd, int n_group,
                              const int *goffs, const void *Sg, const void *Su, const void *Sd,
                              const int *soffs, int R_max, const uint8_t *Xq_rows,
                              const uint8_t *Xs_rows, uint8_t *Hq_rows, uint8_t *Hs_rows,
                              float *Y_rows, int D, int FF, int path, int stages, int max_group_rows,
                              void *ws, uint64_t ws_bytes, void *stream);

/* k_moe_combine / k_moe_combine_pf (q36_engine.cu:785-791, 3393-3401):
 *   out[t][i] = sum_{s<k} wt[t][s] * Y_rows[pos[t*k+s]][i]          (pos >= 0)
 *             + (SH_rows ? sigmoid(shgate[t*shgate_stride]) * SH_rows[t][i] : 0)
 * in slot order; shgate == NULL means gate 1.  1 <= k <= 8. */
int q36_moe_combine(float *out, const float *Y_rows, const int *pos, const float *wt,
                    const float *SH_rows, const float *shgate, int shgate_stride, int D, int k,
                    int T, void *stream);

/* ---- whole layer -----------------------------------------------------------
 * One call = moe_ffn (q36_engine.cu:1592-1654) or pf_moe_block (:3423-3472)
 * from the router logits on:
 *   route -> dispatch -> quantise -> gate/up + SwiGLU -> down -> combine.
 * logits [T][logit_stride] f32: columns [0,n_expert) are router logits;
 * column shgate_col (or < 0 for none: gate = 1) is the shared-expert gate
 * logit (the engine keeps it at column n_expert, q36_engine.cu:1599-1601).
 * Sg/Su/Sd: the shared expert's split planes, or NULL for no shared expert;
 * inc_shared == 0 suppresses its term (non-owner ranks, :3398-3400).
 * Optional outputs idx_out [T][k], wt_out [T][k] (may be NULL). */
uint64_t q36_moe_workspace_bytes(int T_max, int n_expert, int k, int D, int FF);
/* The first 256 bytes of every workspace hold device status words.  They are
 * STICKY: a kernel whose bounded wait gives up records where, and nothing but
 * q36_moe_ws_reset clears it, so one check after many launches that shared a
 * workspace (a 40-layer step, a benchmark loop) still sees a failure in any
 * of them.  Call q36_moe_ws_reset once after allocating a workspace (its
 * memory is not assumed to be zero) and again to clear a recorded failure. */
int q36_moe_ws_reset(void *ws, void *stream);
/* Synchronises `stream` and reports whether any launch that used the
 * workspace `ws` since the last reset gave up on a bounded wait
 * (Q36_MOE_EDEVICE; q36_moe_last_cuda_error() = 200000 + role * 256 + stage)
 * or not (Q36_MOE_OK).  The launch-only entry points cannot report this
 * themselves. */
int q36_moe_ws_status(const void *ws, void *stream);
/* Exercises the give-up path on its own: launches one warp that waits, with
 * a limit of 1024 polls, on a barrier that nothing completes, records the
 * give-up in ws like the tensor-core kernels do, and returns what
 * q36_moe_ws_status then reports (Q36_MOE_EDEVICE when the mechanism works).
 * The context stays usable; q36_moe_ws_reset clears the record. */
int q36_moe_selftest_wait_timeout(void *ws, void *stream);
int q36_moe_layer(const void *Wg, const void *Wu, const void *Wd, const void *Sg, const void *Su,
                  const void *Sd, int n_expert, int se0, int se1, int k, int D, int FF,
                  const void *X, int x_is_bf16, const float *logits, int logit_stride,
                  int shgate_col, float route_scale, int inc_shared, float *out, int *idx_out,
                  float *wt_out, int T, int path, void *ws, uint64_t ws_bytes, void *stream);
/* moe_ffn / pf_moe_block by name: q36_moe_layer with path = Q36_MOE_PATH_AUTO
 * (the fastest measured path for the call's size) and no routing outputs. */
int q36_moe_decode(const void *Wg, const void *Wu, const void *Wd, const void *Sg, const void *Su,
                   const void *Sd, int n_expert, int se0, int se1, int k, int D, int FF,
                   const void *X, int x_is_bf16, const float *logits, int logit_stride,
                   int shgate_col, float route_scale, int inc_shared, float *out, int T, void *ws,
                   uint64_t ws_bytes, void *stream);
int q36_moe_prefill(const void *Wg, const void *Wu, const void *Wd, const void *Sg, const void *Su,
                    const void *Sd, int n_expert, int se0, int se1, int k, int D, int FF,
                    const void *X, int x_is_bf16, const float *logits, int logit_stride,
                    int shgate_col, float route_scale, int inc_shared, float *out, int T, void *ws,
                    uint64_t ws_bytes, void *stream);

/* ---- the block from the residual stream -----------------------------------
 * The steps the engine runs either side of moe_ffn / pf_moe_block, so that a
 * caller can hand over the residual stream instead of pre-made logits.
 *
 * Before (k_add_rmsnorm, q36_engine.cu:696-706,1962, + k_matvec_f32_row,
 * q36_ops.cuh:331-342, at decode; k_rmsnorm_b + pf_gemm, q36_engine.cu:3426-3427,
 * 3469, when batched):
 *   h [T][D] f32 += a   (a == NULL: no add, as in the batched path)
 *   x [T][D] f32  = h * rsqrt(mean(h^2) + eps) * norm_w
 *   logits[t][r]  = router_w[r][:] . x[t][:]   for r < n_rows
 * router_w is [n_rows][D] f32; gate_row (n_rows - 1 or -1) names the
 * shared-gate row of the engine's concatenated router (q36_engine.cu:1599-1601).
 * f32 dot products at every T (the engine's batched path rounds to fp16). */
int q36_moe_pre_norm_router(float *h, const float *a, const float *norm_w, float eps, const float *router_w,
                            int n_rows, int gate_row, float *x, float *logits, int logit_stride, int T,
                            int D, void *stream);
/* After (k_moe_combine(_pf) + k_add_rmsnorm, q36_engine.cu:785-791,3393-3401,
 * 696-706,1966) as one launch: moe = q36_moe_combine(...) (written to moe_out
 * when not NULL), h += moe, x_next = rmsnorm(h) * next_norm_w.  D <= 4096. */
int q36_moe_combine_add_rmsnorm(float *moe_out, const float *Y_rows, const int *pos, const float *wt,
                                const float *SH_rows, const float *shgate, int shgate_stride, float *h,
                                const float *next_norm_w, float eps, float *x_next, int D, int k, int T,
                                void *stream);
/* One MoE block of the decode / prefill loop (q36_engine.cu:1962-1966) from
 * the residual stream: the step before, the layer (path AUTO; router_w has
 * n_expert + 1 rows, the last one the shared gate), the step after.
 * h [T][D] in/out; a [T][D] or NULL; x_next [T][D] out; moe_out or NULL.
 * ws: q36_moe_block_workspace_bytes(...) bytes (status words first, as for
 * q36_moe_layer). */
uint64_t q36_moe_block_workspace_bytes(int T_max, int n_expert, int k, int D, int FF);
int q36_moe_block(const void *Wg, const void *Wu, const void *Wd, const void *Sg, const void *Su,
                  const void *Sd, int n_expert, int se0, int se1, int k, int D, int FF,
                  const float *post_norm_w, const float *router_w, const float *next_norm_w, float eps,
                  float route_scale, int inc_shared, float *h, const float *a, float *x_next, float *moe_out,
                  int T, void *ws, uint64_t ws_bytes, void *stream);

/* Host-buffer form of q36_moe_layer: X, logits and out are HOST pointers
 * (pinned or pageable); the call copies in, runs the layer and copies out on
 * `stream`, then synchronises it.  dev_io: device staging of
 * q36_moe_host_io_bytes(T, D, logit_stride, x_is_bf16) bytes. */
uint64_t q36_moe_host_io_bytes(int T, int D, int logit_stride, int x_is_bf16);
int q36_moe_layer_host(const void *Wg, const void *Wu, const void *Wd, const void *Sg,
                       const void *Su, const void *Sd, int n_expert, int se0, int se1, int k,
                       int D, int FF, const void *host_X, int x_is_bf16, const float *host_logits,
                       int logit_stride, int shgate_col, float route_scale, int inc_shared,
                       float *host_out, int T, int path, void *dev_io, void *ws, uint64_t ws_bytes,
                       void *stream);

/* A stack of n_layers layers from HOST buffers in one call: host_X [L][T][D], host_logits [L][T][stride] in,
 * host_out [L][T][D] out (pinned or pageable); Wg..Sd are arrays of n_layers device pointers (Sg/Su/Sd may be
 * NULL).  Three copies per call (all X, all logits, all outputs) around the layer launches on `stream`, which is
 * synchronised before returning; reports the device status like q36_moe_layer_host.
 * dev_io: q36_moe_stack_host_io_bytes(...) bytes of device staging. */
uint64_t q36_moe_stack_host_io_bytes(int n_layers, int T, int D, int logit_stride, int x_is_bf16);
int q36_moe_stack_host(int n_layers, const void *const *Wg, const void *const *Wu, const void *const *Wd,
                       const void *const *Sg, const void *const *Su, const void *const *Sd, int n_expert, int se0,
                       int se1, int k, int D, int FF, const void *host_X, int x_is_bf16, const float *host_logits,
                       int logit_stride, int shgate_col, float route_scale, int inc_shared, float *host_out, int T,
                       int path, void *dev_io, void *ws, uint64_t ws_bytes, void *stream);

/* ---- expert-parallel helpers ----------------------------------------------
 * Row permutation used either side of the all-to-all: dst[i] = src[index[i]]
 * for rows of row_bytes bytes (row_bytes % 16 == 0); index[i] < 0 zero-fills. */
int q36_moe_gather_rows(const void *src, const int *index, void *dst, int n_rows, int row_bytes,
                        void *stream);

/* Expert-parallel layer step: the role of q36_multi_create / q36_multi_prefill (q36_engine.cu:4234-4306), with
 * the reference's gather + sum + broadcast through device 0 replaced by a dispatch and a combine that the
 * library's own kernels write straight into the destination rank's memory over NVLink.  Rank r owns experts
 * [r*n_expert/world, (r+1)*n_expert/world) (q36_engine.cu:4245) and passes ITS shard's planes as Wg/Wu/Wd; the
 * shared expert (Sg/Su/Sd, may be NULL) is replicated and runs on the rank's own tokens.
 *
 * Two ways to form the ranks:
 *   q36_moe_ep_unique_id + q36_moe_ep_init   one process per GPU; NCCL (looked up at run time, libnccl.so.2)
 *                          carries the bootstrap.  rank 0 fills 128 bytes that the caller gives to every rank.
 *   q36_moe_ep_init_local  one process, `world` ranks on the listed devices, as the engine's own driver runs
 *                          them from one host thread; a device may be listed several times (its ranks then take
 *                          turns on it, which is how a single GPU exercises the 2/4/8-rank data path).
 * q36_moe_ep_open_window (collective over the ranks of a process group; for local ranks one call on any of them
 * opens all) allocates each rank's exchange window for calls of at most T_max tokens per rank and maps the
 * others' windows (CUDA IPC, or peer access for local ranks).  cap_rows: rows one rank may send to one other rank
 * per call; 0 = T_max*k, which can never overflow; a smaller cap drops the rows beyond it and records 0xD00 in
 * the status words.  Not launch-only: it allocates and synchronises; the layer calls below allocate nothing.
 *
 * q36_moe_ep_layer is launch-only: X [T][D], logits [T][stride] of this rank's T tokens -> out [T][D].
 * q36_moe_ep_layer_phase issues one of its three phases (0 route + send, 1 expert work + return, 2 combine): a
 * host thread that drives several local ranks must issue phase p for EVERY rank before phase p + 1 of any, and a
 * caller may put phase 0 of the next call's tokens on another stream to overlap it with phase 1 of this one.
 * (such calls alternate between two workspaces).  T must be the same on every rank of a call.  Calls with more
 * rows on a rank than q36_moe_one_launch_rows() return one weighted partial row per (token, expert rank) when
 * cap_rows >= T_max, else one row per (token, expert) like the smaller calls.
 * Every cross-rank wait is bounded and reports through the status words (0xB00 + source, 0xC00 + source).
 * ws: q36_moe_ep_workspace_bytes(...) bytes with the T_max / cap_rows the window was opened with; its first 256
 * bytes are the status words (q36_moe_ws_reset, q36_moe_ws_status).
 * q36_moe_ep_set_transport: 0 = peer memory (default), 1 = the same kernels over local staging buffers moved
 * by grouped ncclSend/ncclRecv (process-per-GPU ranks only), kept for comparison. */
int q36_moe_ep_unique_id(void *out128);
int q36_moe_ep_init(const void *id128, int rank, int world, void **comm_out);
int q36_moe_ep_init_local(int world, const int *devices, void **comms_out);
int q36_moe_ep_destroy(void *comm);   /* local ranks: destroy rank 0 last */
int q36_moe_ep_open_window(void *comm, int T_max, int k, int D, int cap_rows);
int q36_moe_ep_set_transport(void *comm, int transport);
uint64_t q36_moe_ep_workspace_bytes(int T_max, int cap_rows, int world, int n_expert, int k, int D, int FF);
int q36_moe_ep_layer(void *comm, const void *Wg, const void *Wu, const void *Wd, const void *Sg,
                     const void *Su, const void *Sd, int n_expert, int k, int D, int FF, const void *X,
                     int x_is_bf16, const float *logits, int logit_stride, int shgate_col,
                     float route_scale, float *out, int T, void *ws, uint64_t ws_bytes, void *stream);
int q36_moe_ep_layer_phase(void *comm, int phase, const void *Wg, const void *Wu, const void *Wd, const void *Sg,
                           const void *Su, const void *Sd, int n_expert, int k, int D, int FF, const void *X,
                           int x_is_bf16, const float *logits, int logit_stride, int shgate_col,
                           float route_scale, float *out, int T, void *ws, uint64_t ws_bytes, void *stream);

/* q36_moe_stack_host for an expert-parallel stack: this rank's tokens of every layer in, its outputs out. */
int q36_moe_ep_stack_host(void *comm, int n_layers, const void *const *Wg, const void *const *Wu,
                          const void *const *Wd, const void *const *Sg, const void *const *Su,
                          const void *const *Sd, int n_expert, int k, int D, int FF, const void *host_X,
                          int x_is_bf16, const float *host_logits, int logit_stride, int shgate_col,
                          float route_scale, float *host_out, int T, void *dev_io, void *ws, uint64_t ws_bytes,
                          void *stream);

/* ---- tensor-core self-check (the role of test_mma_bs.cu:45-175) ----------
 * Runs 128 x N x K block-scaled tcgen05 tiles on caller data and returns the
 * f32 accumulators, so that the operand, scale-factor and descriptor mapping
 * can be proven against a CPU product on silicon.
 *   A: one 128-row matrix in the split layout: [128][K/2] MXFP4 code bytes
 *      (GGUF nibble order) followed by [128][K/32] E8M0 scale bytes
 *   B_q [N][K] E4M3 (hw order), B_s [N][K/32] UE8M0
 *   D [N][128] f32: D[n][m] = sum_k A[m][k] * B[n][k]
 * K % 512 == 0, 1 <= N <= 4096.  ws: 512 + q36_moe_ffn_ws_bytes(1,N,128,K)
 * bytes.  Synchronous; returns Q36_MOE_EDEVICE if a bounded wait gave up. */
int q36_moe_tc_selftest(const uint8_t *A, const uint8_t *B_q, const uint8_t *B_s, float *D, int N,
                        int K, void *ws, uint64_t ws_bytes, void *stream);

#ifdef __cplusplus
}
#endif
#endif /* Q36_MOE_H */
