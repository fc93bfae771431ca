// Expert-parallel MoE layer step, host orchestration in C with NCCL send/recv as the all-to-all.
//
// The reference's multi-GPU driver is native host code too (q36_multi_prefill, q36_engine.cu:4261-4306): every
// device runs the layer on its expert shard and device 0 gathers, sums and broadcasts the partial outputs with
// peer copies.  Here tokens stay on their home rank and only routed rows travel:
//   route + dispatch (all experts) -> quantise -> pack rows per destination rank (fixed capacity C = T*k per
//   peer, so no count ever reaches the host) -> all-to-all -> local dispatch of the received rows -> grouped
//   expert FFN on the local shard (+ the shared expert on the rank's own tokens) -> result rows back by
//   all-to-all -> weighted combine on the home rank.
// A packed row is [2048 E4M3 bytes | 64 UE8M0 scale bytes | expert id (int32, -1 = empty slot) | 12 B pad].
//
// NCCL is resolved at run time (dlopen of libnccl.so.2, the one the process already has loaded), so the library
// keeps loading on machines without it.  All kernels read local memory only; the transport is NCCL's.
#include <dlfcn.h>
#include <nccl.h>
#include <stdio.h>
#include <string.h>

#include "common.cuh"
#include "kernels.cuh"

namespace q36 {

struct NcclApi {
    ncclResult_t (*GetUniqueId)(ncclUniqueId *);
    ncclResult_t (*CommInitRank)(ncclComm_t *, int, ncclUniqueId, int);
    ncclResult_t (*CommDestroy)(ncclComm_t);
    ncclResult_t (*GroupStart)();
    ncclResult_t (*GroupEnd)();
    ncclResult_t (*Send)(const void *, size_t, ncclDataType_t, int, ncclComm_t, cudaStream_t);
    ncclResult_t (*Recv)(void *, size_t, ncclDataType_t, int, ncclComm_t, cudaStream_t);
    bool ok;
};
static NcclApi *nccl() {
    static NcclApi api = {};
    static bool tried = false;
    if (!tried) {
        tried = true;
        void *h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
        if (!h) h = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
        if (h) {
            api.GetUniqueId = (decltype(api.GetUniqueId))dlsym(h, "ncclGetUniqueId");
            api.CommInitRank = (decltype(api.CommInitRank))dlsym(h, "ncclCommInitRank");
            api.CommDestroy = (decltype(api.CommDestroy))dlsym(h, "ncclCommDestroy");
            api.GroupStart = (decltype(api.GroupStart))dlsym(h, "ncclGroupStart");
            api.GroupEnd = (decltype(api.GroupEnd))dlsym(h, "ncclGroupEnd");
            api.Send = (decltype(api.Send))dlsym(h, "ncclSend");
            api.Recv = (decltype(api.Recv))dlsym(h, "ncclRecv");
            api.ok = api.GetUniqueId && api.CommInitRank && api.CommDestroy && api.GroupStart && api.GroupEnd && api.Send && api.Recv;
        }
    }
    return api.ok ? &api : nullptr;
}

struct EpComm { ncclComm_t comm; int rank, world; };

constexpr int EP_PAD = 16;   // expert id + padding behind the quantised row

// ------------------------------------------------------------------ kernels
// One block per send slot.  Slot (r, j) of the block for rank r carries the j-th row (in expert order) routed to
// r: entry elist[base_r + j]; slots beyond the rank's count are marked empty.  Entry i comes back in slot
// ypos[i] = r*C + (pos[i] - base_r).
__global__ void __launch_bounds__(128)
k_ep_pack(const uint8_t *__restrict__ Xq, const uint8_t *__restrict__ Xs, const int *__restrict__ idx,
          const int *__restrict__ eoffs, const int *__restrict__ elist, const int *__restrict__ pos, int world, int E,
          int k, int T, int C, int D, uint8_t *__restrict__ send, int *__restrict__ ypos) {
    Q36_GDS();
    const int slot = blockIdx.x, r = slot / C, j = slot % C, per = E / world;
    const int nbs = D / Q36_QK, row_bytes = D + nbs + EP_PAD;
    const int base = eoffs[r * per], cnt = eoffs[(r + 1) * per] - base;
    uint8_t *dst = send + (size_t)slot * row_bytes;
    int eid = -1;
    if (j < cnt) {
        const int entry = elist[base + j], t = entry / k;
        eid = idx[entry];
        const uint4 *sq = reinterpret_cast<const uint4 *>(Xq + (size_t)t * D);
        for (int i = threadIdx.x; i < D / 16; i += blockDim.x) reinterpret_cast<uint4 *>(dst)[i] = sq[i];
        const uint4 *ss = reinterpret_cast<const uint4 *>(Xs + (size_t)t * nbs);
        for (int i = threadIdx.x; i < nbs / 16; i += blockDim.x) reinterpret_cast<uint4 *>(dst + D)[i] = ss[i];
    }
    if (threadIdx.x == 0) *reinterpret_cast<int4 *>(dst + D + nbs) = make_int4(eid, 0, 0, 0);
    // entries -> return slots (each entry handled once, by the blocks of slot index < T*k)
    const int i = slot * blockDim.x + threadIdx.x;
    if (i < T * k) {
        const int p = pos[i];
        const int rr = idx[i] / per;
        ypos[i] = (p >= 0) ? rr * C + (p - eoffs[rr * per]) : -1;
    }
}

__global__ void k_ep_eids(const uint8_t *__restrict__ recv, int n_slots, int row_bytes, int eid_off, int *__restrict__ eid) {
    Q36_GDS();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n_slots) eid[i] = *reinterpret_cast<const int *>(recv + (size_t)i * row_bytes + eid_off);
}

// Sorted row r (< R) <- received slot llist[r] (zeros when r is beyond the resident count: llist holds -1 there);
// rows [R, R+T) <- the rank's own tokens (the shared expert's group).
__global__ void __launch_bounds__(128)
k_ep_unpack(const uint8_t *__restrict__ recv, const int *__restrict__ llist, const int *__restrict__ loffs_end,
            const uint8_t *__restrict__ Xq, const uint8_t *__restrict__ Xs, int R, int T, int D,
            uint8_t *__restrict__ rows_q, uint8_t *__restrict__ rows_s) {
    Q36_GDS();
    const int r = blockIdx.x;
    const int nbs = D / Q36_QK, row_bytes = D + nbs + EP_PAD;
    const uint8_t *sq = nullptr, *ss = nullptr;
    if (r < R) {
        if (r < *loffs_end) {
            const uint8_t *src = recv + (size_t)llist[r] * row_bytes;
            sq = src;
            ss = src + D;
        }
    } else {
        sq = Xq + (size_t)(r - R) * D;
        ss = Xs + (size_t)(r - R) * nbs;
    }
    uint4 *dq = reinterpret_cast<uint4 *>(rows_q + (size_t)r * D), *ds = reinterpret_cast<uint4 *>(rows_s + (size_t)r * nbs);
    const uint4 z = make_uint4(0, 0, 0, 0);
    for (int i = threadIdx.x; i < D / 16; i += blockDim.x) dq[i] = sq ? reinterpret_cast<const uint4 *>(sq)[i] : z;
    for (int i = threadIdx.x; i < nbs / 16; i += blockDim.x) ds[i] = ss ? reinterpret_cast<const uint4 *>(ss)[i] : z;
}

static inline uint64_t al256(uint64_t x) { return (x + 255) & ~(uint64_t)255; }

struct EpWs {
    int *status, *idx, *ecount, *eoffs, *elist, *pos, *ypos, *reid, *lcount, *loffs, *llist, *lpos, *soffs;
    float *wt, *Y, *back, *recv_y;
    void *disp, *ldisp, *plan;
    uint8_t *Xq, *Xs, *send, *recv, *rows_q, *rows_s, *Hq, *Hs;
    uint64_t total;
};
static EpWs ep_carve(void *base, int T, int world, int E, int k, int D, int FF) {
    EpWs w;
    uint8_t *p = (uint8_t *)base;
    uint64_t o = 0;
    auto take = [&](uint64_t b) { uint8_t *r = p + o; o += al256(b); return (void *)r; };
    const uint64_t n = (uint64_t)T * k, C = n, S = (uint64_t)world * C, R = S, RT = R + T;
    const uint64_t nbs = D / Q36_QK, rowb = D + nbs + EP_PAD;
    w.status = (int *)take(256);
    w.idx = (int *)take(n * 4); w.wt = (float *)take(n * 4);
    w.ecount = (int *)take((uint64_t)E * 4); w.eoffs = (int *)take((uint64_t)(E + 1) * 4);
    w.elist = (int *)take(n * 4); w.pos = (int *)take(n * 4); w.ypos = (int *)take(n * 4);
    w.disp = take(dispatch_ws_bytes((int)n, E));
    w.Xq = (uint8_t *)take((uint64_t)T * D); w.Xs = (uint8_t *)take((uint64_t)T * nbs);
    w.send = (uint8_t *)take(S * rowb); w.recv = (uint8_t *)take(S * rowb);
    w.reid = (int *)take(S * 4);
    w.lcount = (int *)take((uint64_t)E * 4); w.loffs = (int *)take((uint64_t)(E + 1) * 4);
    w.llist = (int *)take(S * 4); w.lpos = (int *)take(S * 4); w.soffs = (int *)take(8);
    w.ldisp = take(dispatch_ws_bytes((int)S, E));
    w.rows_q = (uint8_t *)take(RT * D); w.rows_s = (uint8_t *)take(RT * nbs);
    w.Hq = (uint8_t *)take(RT * FF); w.Hs = (uint8_t *)take(RT * (FF / Q36_QK));
    w.Y = (float *)take(RT * D * 4);
    w.back = (float *)take(S * D * 4); w.recv_y = (float *)take(S * D * 4);
    w.plan = take(tc_ws_bytes());
    w.total = o;
    return w;
}

static int all_to_all(NcclApi *api, EpComm *c, const void *send, void *recv, size_t bytes_per_peer, cudaStream_t st) {
    ncclResult_t r = api->GroupStart();
    for (int p = 0; p < c->world && r == ncclSuccess; p++) {
        r = api->Send((const uint8_t *)send + (size_t)p * bytes_per_peer, bytes_per_peer, ncclUint8, p, c->comm, st);
        if (r == ncclSuccess) r = api->Recv((uint8_t *)recv + (size_t)p * bytes_per_peer, bytes_per_peer, ncclUint8, p, c->comm, st);
    }
    const ncclResult_t e = api->GroupEnd();
    if (r == ncclSuccess) r = e;
    if (r != ncclSuccess) { last_cuda_error() = 300000 + (int)r; return Q36_MOE_ECUDA; }
    return Q36_MOE_OK;
}

}  // namespace q36

using namespace q36;

extern "C" {

int q36_moe_ep_unique_id(void *out128) {
    NcclApi *api = nccl();
    if (!api || !out128) return Q36_MOE_EINVAL;
    ncclUniqueId id;
    if (api->GetUniqueId(&id) != ncclSuccess) return Q36_MOE_ECUDA;
    memcpy(out128, &id, sizeof id);
    return Q36_MOE_OK;
}

int q36_moe_ep_init(const void *id128, int rank, int world, void **comm_out) {
    NcclApi *api = nccl();
    if (!api || !id128 || !comm_out || world < 1 || rank < 0 || rank >= world) return Q36_MOE_EINVAL;
    ncclUniqueId id;
    memcpy(&id, id128, sizeof id);
    EpComm *c = new EpComm{nullptr, rank, world};
    const ncclResult_t r = api->CommInitRank(&c->comm, world, id, rank);
    if (r != ncclSuccess) { last_cuda_error() = 300000 + (int)r; delete c; return Q36_MOE_ECUDA; }
    *comm_out = c;
    return Q36_MOE_OK;
}

int q36_moe_ep_destroy(void *comm) {
    NcclApi *api = nccl();
    EpComm *c = (EpComm *)comm;
    if (!api || !c) return Q36_MOE_EINVAL;
    api->CommDestroy(c->comm);
    delete c;
    return Q36_MOE_OK;
}

uint64_t q36_moe_ep_workspace_bytes(int T, int world, int n_expert, int k, int D, int FF) {
    if (T <= 0 || world <= 0 || n_expert <= 0 || k <= 0) return 0;
    return ep_carve(nullptr, T, world, n_expert, k, D, FF).total;
}

int q36_moe_ep_layer(void *comm, const void *Wg, const void *Wu, const void *Wd, const void *Sg, const void *Su,
                     const void *Sd, int n_expert, int k, int D, int FF, const void *X, int x_is_bf16,
                     const float *logits, int logit_stride, int shgate_col, float route_scale, float *out, int T,
                     void *ws, uint64_t ws_bytes, void *stream) {
    NcclApi *api = nccl();
    EpComm *c = (EpComm *)comm;
    if (!api || !c || !Wg || !Wu || !Wd || !X || !logits || !out || !ws) return Q36_MOE_EINVAL;
    const int world = c->world, rank = c->rank, E = n_expert;
    if (T <= 0 || k <= 0 || k > 8 || E % world || E > DISPATCH_MAX_GROUPS || D % 512 || FF % 512 || logit_stride < E)
        return Q36_MOE_EINVAL;
    if (!router_supports(E)) return Q36_MOE_EINVAL;
    const EpWs w = ep_carve(ws, T, world, E, k, D, FF);
    if (w.total > ws_bytes) return Q36_MOE_ENOSPACE;
    cudaStream_t st = (cudaStream_t)stream;
    const int n = T * k, C = n, S = world * C, R = S, per = E / world, se0 = rank * per, se1 = se0 + per;
    const int nbs = D / Q36_QK, rowb = D + nbs + EP_PAD;
    const bool shared = Sg && Su && Sd;
    int rc;
    // 1. route + dispatch over ALL experts (their order is the destination-rank order), and
    // 2. quantise the rank's tokens once, in token order (hw order inside the blocks): one cluster launch at decode sizes
    const bool cluster_front = T <= 16 && n <= 128 && D % 1024 == 0 && D * T <= 32 * 1024;
    if (cluster_front) {
        if ((rc = launch_front_decode(logits, E, k, route_scale, T, logit_stride, w.idx, w.wt, w.ecount, w.eoffs, w.elist, w.pos,
                                      nullptr, 0, 0, nullptr, D, FF, w.status, X, x_is_bf16, w.Xq, w.Xs, 0, 0, st)))
            return rc;
    } else if (n <= 1024) {
        if ((rc = launch_front_small(logits, E, k, route_scale, T, logit_stride, 0, E, w.idx, w.wt, w.ecount, w.eoffs, w.elist,
                                     w.pos, nullptr, 0, 0, nullptr, D, FF, w.status, nullptr, 0, nullptr, nullptr, -1, 0, st)))
            return rc;
    } else {
        if ((rc = launch_router_topk(logits, E, k, w.idx, w.wt, route_scale, 1, T, logit_stride, st))) return rc;
        if ((rc = launch_dispatch(w.idx, n, E, 0, E, w.ecount, w.eoffs, w.elist, w.pos, w.disp, nullptr, 0, 0, st))) return rc;
    }
    if (!cluster_front && (rc = launch_quant(X, x_is_bf16, w.Xq, w.Xs, T, D, nullptr, 0, 0, true, st))) return rc;
    // 3. pack per destination rank and exchange
    launch_k(k_ep_pack, dim3(S), dim3(128), 0, st, (const uint8_t *)w.Xq, (const uint8_t *)w.Xs, (const int *)w.idx,
             (const int *)w.eoffs, (const int *)w.elist, (const int *)w.pos, world, E, k, T, C, D, w.send, w.ypos);
    if ((rc = check_launch())) return rc;
    if ((rc = all_to_all(api, c, w.send, w.recv, (size_t)C * rowb, st))) return rc;
    // 4. local plan over the received slots; empty slots (-1) and nothing else drop out
    const bool small_plan = S <= 1024;   // one block sorts the slots and writes the work plan
    // the one-launch decode kernel: always when no expert can receive more than 16 rows, else up to a row count
    const bool one_launch = ffn_fused_small_fits(R + T, per, D, FF) && (world * T <= 16 || R + T <= fused_rows_limit());
    if (small_plan) {
        if ((rc = launch_dispatch_plan_small(w.recv + (D + nbs), rowb, S, E, se0, se1, w.lcount, w.loffs, w.llist, w.lpos, w.soffs,
                                             R, shared ? R + T : R, w.plan, D, FF, w.status, one_launch ? 16 : 0, st)))
            return rc;
    } else {
        launch_k(k_ep_eids, dim3((S + 255) / 256), dim3(256), 0, st, (const uint8_t *)w.recv, S, rowb, D + nbs, w.reid);
        if ((rc = launch_dispatch(w.reid, S, E, se0, se1, w.lcount, w.loffs, w.llist, w.lpos, w.ldisp, w.soffs, R, shared ? R + T : R, st)))
            return rc;
    }
    launch_k(k_ep_unpack, dim3(R + T), dim3(128), 0, st, (const uint8_t *)w.recv, (const int *)w.llist,
             (const int *)(w.loffs + E), (const uint8_t *)w.Xq, (const uint8_t *)w.Xs, R, T, D, w.rows_q, w.rows_s);
    if ((rc = check_launch())) return rc;
    // 5. grouped expert FFN on the local shard (+ shared expert on the own tokens)
    const int *goffs = w.loffs + se0;
    if (!small_plan && (rc = launch_tc_plan(goffs, per, shared ? w.soffs : nullptr, D, FF, w.plan, w.status, one_launch ? 16 : 0, st)))
        return rc;
    // an expert receives at most one row per token of every rank: with at most 16 of them the decode kernel
    // (gate/up and down in one persistent launch) applies
    if (one_launch) {
        if ((rc = launch_ffn_fused_small(Wg, Wu, Wd, shared ? Sg : nullptr, shared ? Su : nullptr, shared ? Sd : nullptr, per,
                                         R + T, w.rows_q, w.rows_s, w.Hq, w.Hs, w.Y, D, FF, w.plan, w.status, w.llist, w.back, R, st)))
            return rc;   // (routed result rows land in the slots of the return exchange; the shared rows stay in Y)
    } else {
        if ((rc = launch_gateup_tc(Wg, Wu, shared ? Sg : nullptr, shared ? Su : nullptr, per, R + T, R + T, w.rows_q, w.rows_s,
                                   w.Hq, w.Hs, D, FF, w.plan, w.status, st)))
            return rc;
        if ((rc = launch_down_tc(Wd, shared ? Sd : nullptr, per, R + T, R + T, w.Hq, w.Hs, w.Y, D, FF, w.plan, w.status + 1, st)))
            return rc;
    }
    // 6. result rows back to their home ranks, then the weighted combine
    if (!one_launch && (rc = launch_gather_rows(w.Y, w.lpos, w.back, S, D * 4, st))) return rc;
    if ((rc = all_to_all(api, c, w.back, w.recv_y, (size_t)C * D * 4, st))) return rc;
    const float *shg = (shared && shgate_col >= 0) ? logits + shgate_col : nullptr;
    return launch_combine(out, w.recv_y, w.ypos, w.wt, shared ? w.Y + (size_t)R * D : nullptr, shg, logit_stride, D, k, T, false, st);
}

}  // extern "C"
