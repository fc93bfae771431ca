// Expert-parallel MoE layer step: dispatch and combine as the library's own kernels over peer memory.
//
// The reference's multi-GPU driver is native host code (q36_multi_create / q36_multi_prefill,
// q36_engine.cu:4234-4306): every device runs the layer on its expert shard and device 0 gathers, sums and
// broadcasts the partial outputs with peer copies.  Here tokens stay on their home rank and only routed rows
// travel, written by kernels STRAIGHT INTO THE DESTINATION RANK'S MEMORY over NVLink:
//
//   phase 0 (home)    route + dispatch over all experts, quantise the rank's rows once, then k_ep_send stores
//                     every routed row into the window of the rank that owns its expert and publishes
//                     (count, epoch) there
//   phase 1 (expert)  wait (bounded) for every source's header, bucket the received rows by local expert, run the
//                     grouped FFN on the shard (+ the shared expert on the rank's own tokens), then k_ep_return
//                     stores each result row into its home rank's window and publishes the epoch there
//   phase 2 (home)    wait (bounded) for every expert rank's header, weighted combine
//
// Each rank owns one "window" (device memory allocated once when the window is opened, mapped into the other
// ranks with CUDA IPC or, for ranks of one process, by peer access): [2 parities] x { headers, rows of every
// source, result rows of every expert rank }.  A call uses parity (call number & 1); a rank can run at most one
// call ahead of a peer because its combine needs that peer's results, so two parities suffice.  The call
// numbers live on the device (one counter per phase, advanced by the phase's last kernel), which makes a stack of
// calls capturable in a CUDA graph and lets phase 0 of the next call run beside phases 1 and 2 of this one.
//
// Every wait is bounded; a wait that gives up records 0xB00 + source (dispatch) or 0xC00 + source (results) in
// the status words and the step goes on (with garbage, but it ends and the host can see why).
// No TMA or bulk copy ever touches another GPU's memory: peers are reached by plain st.global only, and every
// tensor-core operand is read from local memory.
//
// NCCL carries the bootstrap (the IPC handles) and is kept as an alternative transport for comparison
// (q36_moe_ep_set_transport): the same kernels then fill local staging buffers that grouped ncclSend/ncclRecv move.
#include <dlfcn.h>
#include <nccl.h>
#include <stdio.h>
#include <stdlib.h>
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
    ncclResult_t (*AllGather)(const void *, void *, size_t, ncclDataType_t, ncclComm_t, cudaStream_t);
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
            api.AllGather = (decltype(api.AllGather))dlsym(h, "ncclAllGather");
            api.ok = api.GetUniqueId && api.CommInitRank && api.CommDestroy && api.GroupStart && api.GroupEnd && api.Send &&
                     api.Recv && api.AllGather;
        }
    }
    return api.ok ? &api : nullptr;
}

constexpr int EP_MAX_WORLD = 16;
constexpr int EP_TAIL = 16;   // behind the quantised row: expert id (int32) + 12 B pad
constexpr unsigned EP_SPIN_LIMIT = 1u << 22;

// Byte offsets inside a window, the same on every rank.
struct WinLayout {
    uint64_t hdr[2], rhdr[2], rows[2], ret[2], tslot[2], twt[2], ctl, bytes;
    int cap, D, world, row_bytes, n_max, tstride;
};
// n_max: entries (tokens x k) one rank routes per call at most
static WinLayout win_layout(int world, int cap, int D, int n_max) {
    WinLayout L;
    L.cap = cap; L.D = D; L.world = world; L.n_max = n_max;
    L.tstride = n_max + 4;               // ints per source in a token table: [n_max] = the source's token count of the call
    L.row_bytes = D + D / Q36_QK + EP_TAIL;
    uint64_t o = 0;
    auto take = [&](uint64_t b) { const uint64_t r = o; o += (b + 255) & ~(uint64_t)255; return r; };
    for (int p = 0; p < 2; p++) { L.hdr[p] = take(8 * EP_MAX_WORLD); L.rhdr[p] = take(8 * EP_MAX_WORLD); }
    L.ctl = take(256);   // ints: [0..2] calls whose phase 0 / 1 / 2 has finished on this rank, [3..6] tickets of the "last block" patterns, [8 + r] per destination
    for (int p = 0; p < 2; p++) L.rows[p] = take((uint64_t)world * cap * L.row_bytes);
    for (int p = 0; p < 2; p++) L.ret[p] = take((uint64_t)world * cap * D * 4);
    // token tables (reduced return): per source and entry (t, s) the slot its row went to on this rank (-1: another
    // rank, or dropped) and its combine weight
    for (int p = 0; p < 2; p++) { L.tslot[p] = take((uint64_t)world * L.tstride * 4); L.twt[p] = take((uint64_t)world * L.tstride * 4); }
    L.bytes = o;
    return L;
}

enum { EP_KIND_PROCS = 0, EP_KIND_LOCAL = 1 };
enum { EP_TRANSPORT_PEER = 0, EP_TRANSPORT_NCCL = 1 };

struct EpComm {
    ncclComm_t comm = nullptr;
    int rank = 0, world = 1, kind = EP_KIND_PROCS, device = 0, transport = EP_TRANSPORT_PEER;
    EpComm **group = nullptr;            // EP_KIND_LOCAL: all ranks of the process (shared array, owned by rank 0)
    bool open = false;
    WinLayout L{};
    int T_max = 0, k = 0;                // what the window was opened for
    uint8_t *win = nullptr;              // this rank's window
    uint8_t *peer[EP_MAX_WORLD] = {};    // every rank's window as mapped here (peer[rank] == win)
    bool ipc_opened[EP_MAX_WORLD] = {};
    uint8_t **d_peer = nullptr;          // device copy of peer[] (or of stage pointers for the NCCL transport)
    uint8_t *stage = nullptr;            // NCCL transport: local staging laid out like a window
    unsigned spin_limit = EP_SPIN_LIMIT;
    unsigned long long calls[3] = {0, 0, 0};   // host mirror of the device's per-phase call counters (NCCL transport only)
};

__device__ __forceinline__ void st_release_sys_u64(unsigned long long *p, unsigned long long v) {
    asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ unsigned long long ld_acq_sys_u64(const unsigned long long *p) {
    unsigned long long v;
    asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ int wait_hdr(const unsigned long long *hdr, unsigned epoch, unsigned limit, int *status, int where) {
    for (unsigned i = 0; i < limit; i++) {
        const unsigned long long v = ld_acq_sys_u64(hdr);
        if ((unsigned)(v >> 32) == epoch) return (int)(unsigned)v;
        if (i > 64) __nanosleep(i < 4096 ? 32 : 256);
    }
    atomicCAS(status, 0, where);
    return -1;
}

// ------------------------------------------------------------------ kernels
// Blocks (r, b), b < nb: block b of destination rank r copies the rows j = b, b + nb, ... that this rank routed to r
// (sorted rows eoffs[r * per] + j: entry elist[.], expert e) -- the quantised row of the entry's token + the expert
// id -- into slot (me, j) of r's window, then publishes (count_r, epoch) there: thread 0 after the block barrier
// with one system-scope fence (the barrier orders the other threads' stores before it).  With several blocks
// per destination the last one to arrive at the destination's ticket publishes.  ypos[entry] = r * cap + j: where
// the result row comes back.  slot_major_dst: NCCL transport, "peers" are local staging blocks indexed by
// DESTINATION instead.
__global__ void __launch_bounds__(1024)
k_ep_send(const uint8_t *__restrict__ Xq, const uint8_t *__restrict__ Xs, const int *__restrict__ idx,
          const int *__restrict__ eoffs, const int *__restrict__ elist, int world, int per, int k, int cap, int D,
          uint8_t *const *__restrict__ peers, int me, uint64_t rows0, uint64_t rows1, uint64_t hdr0, uint64_t hdr1, int *ctl,
          int *__restrict__ ypos, int slot_major_dst, int *status, int nb, const int *__restrict__ pos, const float *__restrict__ wt,
          int n, int T, uint64_t tslot0, uint64_t tslot1, uint64_t twt0, uint64_t twt1, int tstride, int tables) {
    Q36_GDS();
    Q36_TR_BEGIN(status, 1)
    const int r = blockIdx.x / nb, b = blockIdx.x % nb;
    const unsigned epoch = (unsigned)ctl[0] + 1u;
    const bool odd = epoch & 1u;
    const int nbs = D / Q36_QK, row_bytes = D + nbs + EP_TAIL;
    const int base = eoffs[r * per], cnt_all = eoffs[(r + 1) * per] - base, cnt = min(cap, cnt_all);
    uint8_t *dst0 = peers[r] + (odd ? rows1 : rows0) + (size_t)(slot_major_dst ? r : me) * cap * row_bytes;
    const int u4_row = D / 16, u4_all = u4_row + nbs / 16;
    // flat over the 16-byte units of this block's rows (codes, then scale bytes; the tail separately), four loads
    // in flight per thread before the (remote) stores
    const int my_rows = cnt > b ? (cnt - b + nb - 1) / nb : 0;      // rows j = b + nb * q, q < my_rows
    const int total = my_rows * u4_all;
    for (int x0 = threadIdx.x; x0 < total; x0 += 4 * blockDim.x) {
        uint4 v[4];
        uint4 *dptr[4];
#pragma unroll
        for (int u = 0; u < 4; u++) {
            const int x = x0 + u * blockDim.x;
            dptr[u] = nullptr;
            if (x < total) {
                const int q = x / u4_all, i = x - q * u4_all, j = b + nb * q;
                const int t = elist[base + j] / k;
                v[u] = (i < u4_row) ? reinterpret_cast<const uint4 *>(Xq + (size_t)t * D)[i]
                                    : reinterpret_cast<const uint4 *>(Xs + (size_t)t * nbs)[i - u4_row];
                dptr[u] = reinterpret_cast<uint4 *>(dst0 + (size_t)j * row_bytes) + i;
            }
        }
#pragma unroll
        for (int u = 0; u < 4; u++)
            if (dptr[u]) *dptr[u] = v[u];
    }
    for (int q = threadIdx.x; q * nb + b < cnt_all; q += blockDim.x) {   // per row: the tail and the return position
        const int j = b + nb * q, entry = elist[base + j];
        if (j < cnt) {
            *reinterpret_cast<int4 *>(dst0 + (size_t)j * row_bytes + D + nbs) = make_int4(idx[entry], 0, 0, 0);
            ypos[entry] = r * cap + j;
        } else {                                 // beyond the window's capacity: dropped, and reported
            ypos[entry] = -1;
            atomicCAS(status, 0, 0xD00);
        }
    }
    if (tables) {   // reduced return: entry i -> its slot on r (or -1) and its weight, + this rank's token count
        int *ts = reinterpret_cast<int *>(peers[r] + (odd ? tslot1 : tslot0)) + (size_t)me * tstride;
        float *tw = reinterpret_cast<float *>(peers[r] + (odd ? twt1 : twt0)) + (size_t)me * tstride;
        for (int i = b * blockDim.x + threadIdx.x; i < n; i += nb * blockDim.x) {
            const int j = pos[i] - base;
            const bool mine = idx[i] / per == r && j < cap;
            ts[i] = mine ? j : -1;
            tw[i] = wt[i];
        }
        if (b == 0 && threadIdx.x == 0) ts[tstride - 4] = T;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        bool publish = true;
        if (nb > 1) {
            __threadfence_system();
            publish = atomicAdd(ctl + 8 + r, 1) == nb - 1;
            if (publish) ctl[8 + r] = 0;
        }
        if (publish) {   // (a release store: one system-scope fence, ordered after the whole block's stores by the barrier)
            unsigned long long *h = reinterpret_cast<unsigned long long *>(peers[r] + (odd ? hdr1 : hdr0)) + (slot_major_dst ? r : me);
            st_release_sys_u64(h, (unsigned long long)(unsigned)cnt | ((unsigned long long)epoch << 32));
        }
        // the last block of the launch (every block has read the counter by then) ends phase 0 of this call
        if (atomicAdd(ctl + 5, 1) == (int)gridDim.x - 1) { ctl[5] = 0; ctl[0] = (int)epoch; }
    }
    Q36_TR_END(status, 1)
}

// Received slots beyond FRONT_MAX_ENTRIES: wait for the headers in every block, then list each slot's expert id
// (-1 for a slot its source did not fill) for the general dispatch kernels.
__global__ void __launch_bounds__(256)
k_ep_wait_eids(const uint8_t *__restrict__ win, uint64_t hdr0, uint64_t hdr1, uint64_t rows0, uint64_t rows1, const int *ctl,
               int world, int cap, int row_bytes, int eid_off, unsigned limit, int *status, int *__restrict__ eid,
               int *__restrict__ counts_out) {
    Q36_GDS();
    __shared__ int s_cnt[EP_MAX_WORLD];
    const unsigned epoch = (unsigned)ctl[1] + 1u;
    const bool odd = epoch & 1u;
    if (threadIdx.x < world) {
        const int c = wait_hdr(reinterpret_cast<const unsigned long long *>(win + (odd ? hdr1 : hdr0)) + threadIdx.x, epoch, limit,
                               status, 0xB00 + threadIdx.x);
        s_cnt[threadIdx.x] = max(0, min(c, cap));
        if (blockIdx.x == 0) counts_out[threadIdx.x] = s_cnt[threadIdx.x];
    }
    __syncthreads();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < world * cap)
        eid[i] = ((i % cap) < s_cnt[i / cap]) ? *reinterpret_cast<const int *>(win + (odd ? rows1 : rows0) + (size_t)i * row_bytes + eid_off) : -1;
}

// Sorted row r (< R) <- received slot llist[r] (zeros beyond the resident count); rows [R, R + T) <- the rank's
// own tokens (the shared expert's group).
__global__ void __launch_bounds__(256)
k_ep_unpack(const uint8_t *__restrict__ win, uint64_t rows0, uint64_t rows1, const int *ctl, const int *__restrict__ llist,
            const int *__restrict__ loffs_end, const uint8_t *__restrict__ Xq, const uint8_t *__restrict__ Xs, int R, int T, int D,
            uint8_t *__restrict__ rows_q, uint8_t *__restrict__ rows_s, int *status) {
    Q36_GDS();
    Q36_TR_BEGIN(status, 3)
    const int nbs = D / Q36_QK, row_bytes = D + nbs + EP_TAIL;
    const bool odd = ((unsigned)ctl[1] + 1u) & 1u;
    const uint8_t *recv = win + (odd ? rows1 : rows0);
    const int n_res = *loffs_end;          // rows that arrived; rows [n_res, R) belong to no group and are never used
    // a warp per row, several 16-byte loads in flight per lane (a block per row at a time, each thread one load after
    // a dependent index load, was bound by latency: 62 rows in turn per block at prefill sizes)
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, wpb = blockDim.x >> 5;
    const int uq = D / 16, us = nbs / 16;
    for (int x = blockIdx.x * wpb + warp; x < n_res + T; x += gridDim.x * wpb) {
        const int r = x < n_res ? x : R + (x - n_res);
        const uint8_t *sq, *ss;
        if (r < R) {
            sq = recv + (size_t)llist[r] * row_bytes;
            ss = sq + D;
        } else {
            sq = Xq + (size_t)(r - R) * D;
            ss = Xs + (size_t)(r - R) * nbs;
        }
        uint4 *dq = reinterpret_cast<uint4 *>(rows_q + (size_t)r * D), *ds = reinterpret_cast<uint4 *>(rows_s + (size_t)r * nbs);
        for (int i0 = lane; i0 < uq; i0 += 128) {
            uint4 v[4];
#pragma unroll
            for (int u = 0; u < 4; u++)
                if (i0 + 32 * u < uq) v[u] = reinterpret_cast<const uint4 *>(sq)[i0 + 32 * u];
#pragma unroll
            for (int u = 0; u < 4; u++)
                if (i0 + 32 * u < uq) dq[i0 + 32 * u] = v[u];
        }
        for (int i = lane; i < us; i += 32) ds[i] = reinterpret_cast<const uint4 *>(ss)[i];
    }
    Q36_TR_END(status, 3)
}

// Blocks (s, b), b < nb: block b of source rank s copies the result rows of the slots j = b, b + nb, ... that s
// filled (Y[lpos[s * cap + j]]) into slot (me, j) of the result area in s's window, then publishes the epoch there
// (same pattern as k_ep_send).
__global__ void __launch_bounds__(1024)
k_ep_return(const float *__restrict__ Y, const int *__restrict__ lpos, const int *__restrict__ counts, int world, int cap, int D,
            uint8_t *const *__restrict__ peers, int me, uint64_t ret0, uint64_t ret1, uint64_t rhdr0, uint64_t rhdr1, int *ctl,
            int slot_major_dst, int nb, int *status, int y_bf16) {
    Q36_GDS();
    Q36_TR_BEGIN(status, 5)
    const int s = blockIdx.x / nb, b = blockIdx.x % nb;
    const unsigned epoch = (unsigned)ctl[1] + 1u;
    const bool odd = epoch & 1u;
    const int cnt = counts[s];
    float4 *dst0 = reinterpret_cast<float4 *>(peers[s] + (odd ? ret1 : ret0) + (size_t)(slot_major_dst ? s : me) * cap * D * 4);
    const int f4 = D / 4;
    const int my_rows = cnt > b ? (cnt - b + nb - 1) / nb : 0;
    const int total = my_rows * f4;
    for (int x0 = threadIdx.x; x0 < total; x0 += 4 * blockDim.x) {
        float4 v[4];
        float4 *dptr[4];
#pragma unroll
        for (int u = 0; u < 4; u++) {
            const int x = x0 + u * blockDim.x;
            dptr[u] = nullptr;
            if (x < total) {
                const int q = x / f4, i = x - q * f4, j = b + nb * q;
                const int p = lpos[s * cap + j];
                v[u] = (p >= 0) ? ld_y4(Y, (size_t)p * D + 4 * (size_t)i, y_bf16) : make_float4(0.f, 0.f, 0.f, 0.f);
                dptr[u] = dst0 + (size_t)j * f4 + i;
            }
        }
#pragma unroll
        for (int u = 0; u < 4; u++)
            if (dptr[u]) *dptr[u] = v[u];
    }
    __syncthreads();
    if (threadIdx.x == 0) {   // one system-scope fence (the barrier ordered the block's stores before it), then count this block in at s
        __threadfence_system();
        unsigned *h = reinterpret_cast<unsigned *>(peers[s] + (odd ? rhdr1 : rhdr0) + 8 * (slot_major_dst ? s : me));
        asm volatile("red.relaxed.sys.global.add.u32 [%0], 1;" ::"l"(h) : "memory");
        if (atomicAdd(ctl + 6, 1) == (int)gridDim.x - 1) { ctl[6] = 0; ctl[1] = (int)epoch; }   // the last block ends phase 1 of this call
    }
    Q36_TR_END(status, 5)
}

// Reduced return.  Blocks (s, b), b < nb: for the tokens t = b, b + nb, ... of source rank s, the weighted sum over
// the token's entries that ran on this rank, in entry order (sum_s' wt * Y[lpos[slot]], slots and weights from the
// token table s wrote with its rows), goes into row t of this rank's block of the result area in s's window: one
// row per (token, expert rank) pair crosses the link instead of one per (token, expert).  Tokens without an entry
// here are skipped; the home rank knows which those are.  Then the block counts itself in at s (as k_ep_return).
__global__ void __launch_bounds__(512)
k_ep_reduce_return(const float *__restrict__ Y, const int *__restrict__ lpos, const uint8_t *__restrict__ win, uint64_t tslot0,
                   uint64_t tslot1, uint64_t twt0, uint64_t twt1, int tstride, int k, int world, int cap, int D,
                   uint8_t *const *__restrict__ peers, int me, uint64_t ret0, uint64_t ret1, uint64_t rhdr0, uint64_t rhdr1, int *ctl,
                   int nb, int *status, int y_bf16) {
    Q36_GDS();
    Q36_TR_BEGIN(status, 5)
    const int s = blockIdx.x / nb, b = blockIdx.x % nb;
    const unsigned epoch = (unsigned)ctl[1] + 1u;
    const bool odd = epoch & 1u;
    const int *ts = reinterpret_cast<const int *>(win + (odd ? tslot1 : tslot0)) + (size_t)s * tstride;
    const float *tw = reinterpret_cast<const float *>(win + (odd ? twt1 : twt0)) + (size_t)s * tstride;
    const int Ts = min(ts[tstride - 4], cap);
    float *dst0 = reinterpret_cast<float *>(peers[s] + (odd ? ret1 : ret0) + (size_t)me * cap * D * 4);
    constexpr int KMAX = 8;
    // a warp per token: the chain table -> row position -> rows is three dependent latencies, so a block that took its
    // tokens one after another was bound by latency; sixteen tokens per block are in flight here
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, wpb = blockDim.x >> 5;
    for (int t = b * wpb + warp; t < Ts; t += nb * wpb) {
        int p[KMAX];
        float w[KMAX];
        bool any = false;
#pragma unroll
        for (int q = 0; q < KMAX; q++) {
            const int j = (q < k) ? ts[(size_t)t * k + q] : -1;
            any |= j >= 0;
            p[q] = (j >= 0) ? lpos[s * cap + j] : -1;
            w[q] = (q < k) ? tw[(size_t)t * k + q] : 0.f;
        }
        if (!any) continue;
        for (int i = lane * 4; i < D; i += 128) {
            float4 y[KMAX];
#pragma unroll
            for (int q = 0; q < KMAX; q++)
                y[q] = (p[q] >= 0) ? ld_y4(Y, (size_t)p[q] * D + i, y_bf16) : make_float4(0.f, 0.f, 0.f, 0.f);
            float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
            for (int q = 0; q < KMAX; q++) {
                if (p[q] < 0) continue;
                acc.x = fmaf(w[q], y[q].x, acc.x); acc.y = fmaf(w[q], y[q].y, acc.y);
                acc.z = fmaf(w[q], y[q].z, acc.z); acc.w = fmaf(w[q], y[q].w, acc.w);
            }
            *reinterpret_cast<float4 *>(dst0 + (size_t)t * D + i) = acc;
        }
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence_system();
        unsigned *h = reinterpret_cast<unsigned *>(peers[s] + (odd ? rhdr1 : rhdr0) + 8 * me);
        asm volatile("red.relaxed.sys.global.add.u32 [%0], 1;" ::"l"(h) : "memory");
        if (atomicAdd(ctl + 6, 1) == (int)gridDim.x - 1) { ctl[6] = 0; ctl[1] = (int)epoch; }
    }
    Q36_TR_END(status, 5)
}

// k_moe_combine_pf (q36_engine.cu:3393-3401) on the home rank: waits (bounded) for every expert rank's results of
// this call, then out[t] = sum_s wt[t][s] * ret[ypos[t*k+s]] + sigmoid(gate) * SH[t] in slot order.  The last
// block to finish advances the call counter.  grid (D / 1024, T).
__global__ void __launch_bounds__(256)
k_ep_combine(float *__restrict__ out, const uint8_t *__restrict__ win, uint64_t ret0, uint64_t ret1, uint64_t rhdr0, uint64_t rhdr1,
             int *ctl, int world, unsigned limit, int *status, const int *__restrict__ ypos, const float *__restrict__ wt,
             const float *__restrict__ SH, const float *__restrict__ shgate, int shgate_stride, int D, int k, unsigned expected,
             int reduced, int cap, int sh_bf16) {
    // reduced: the expert ranks sent one weighted partial row per token (row r * cap + t for rank r): add those of
    // the ranks that ran an entry of the token, in rank order
    // expected: arrivals every expert rank counts in at this rank's result header per call (the CTAs of its FFN
    // launch, or the blocks per source of its return kernel: the same on every rank for equal sizes)
    Q36_GDS();
    Q36_TR_BEGIN(status, 6)
    const unsigned epoch = (unsigned)ctl[2] + 1u;
    const bool odd = epoch & 1u;
    if (threadIdx.x < world) {
        const unsigned *h = reinterpret_cast<const unsigned *>(win + (odd ? rhdr1 : rhdr0) + 8 * threadIdx.x);
        bool ok = false;
        for (unsigned i = 0; i < limit && !ok; i++) {
            unsigned v;
            asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(h) : "memory");
            ok = v >= expected;
            if (!ok && i > 64) __nanosleep(i < 4096 ? 32 : 256);
        }
        if (!ok) atomicCAS(status, 0, 0xC00 + threadIdx.x);
    }
    __syncthreads();
    const float *Y = reinterpret_cast<const float *>(win + (odd ? ret1 : ret0));
    const int t = blockIdx.y;
    const int i = (blockIdx.x * blockDim.x + threadIdx.x) * 4;
    if (i < D) {
        constexpr int KMAX = 8;
        int p[KMAX];
        float w[KMAX];
        float4 y[KMAX];
#pragma unroll
        for (int s = 0; s < KMAX; s++) {
            p[s] = (s < k) ? ypos[(size_t)t * k + s] : -1;
            w[s] = (s < k) ? wt[(size_t)t * k + s] : 0.f;
        }
        if (reduced) {
            unsigned mask = 0;
#pragma unroll
            for (int s = 0; s < KMAX; s++)
                if (p[s] >= 0) mask |= 1u << (p[s] / cap);
#pragma unroll
            for (int s = 0; s < KMAX; s++) {   // (world <= KMAX on this path: one candidate row per rank)
                p[s] = (s < world && ((mask >> s) & 1u)) ? s * cap + t : -1;
                w[s] = 1.f;
            }
        }
        const float gs = (SH && shgate) ? sigm_f(shgate[(size_t)t * shgate_stride]) : 1.f;
        float4 ysh = make_float4(0.f, 0.f, 0.f, 0.f);
        if (SH) ysh = ld_y4(SH, (size_t)t * D + i, sh_bf16);      // (the shared expert's rows come from this rank's own down launch)
#pragma unroll
        for (int s = 0; s < KMAX; s++)
            y[s] = (p[s] >= 0) ? *reinterpret_cast<const float4 *>(Y + (size_t)p[s] * D + i) : make_float4(0.f, 0.f, 0.f, 0.f);
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int s = 0; s < KMAX; s++) {
            if (p[s] < 0) continue;
            acc.x = fmaf(w[s], y[s].x, acc.x); acc.y = fmaf(w[s], y[s].y, acc.y);
            acc.z = fmaf(w[s], y[s].z, acc.z); acc.w = fmaf(w[s], y[s].w, acc.w);
        }
        if (SH) {
            acc.x = fmaf(gs, ysh.x, acc.x); acc.y = fmaf(gs, ysh.y, acc.y);
            acc.z = fmaf(gs, ysh.z, acc.z); acc.w = fmaf(gs, ysh.w, acc.w);
        }
        *reinterpret_cast<float4 *>(out + (size_t)t * D + i) = acc;
    }
    __syncthreads();
    __shared__ int s_last;
    if (threadIdx.x == 0) s_last = (atomicAdd(ctl + 3, 1) == (int)(gridDim.x * gridDim.y) - 1);
    __syncthreads();
    if (s_last) {   // the call is over: clear this parity's arrival counts (their next use is two calls away), next call
        if (threadIdx.x < world) *reinterpret_cast<unsigned long long *>(const_cast<uint8_t *>(win) + (odd ? rhdr1 : rhdr0) + 8 * threadIdx.x) = 0ull;
        __syncthreads();
        if (threadIdx.x == 0) { ctl[3] = 0; ctl[2] = (int)epoch; }
    }
    Q36_TR_END(status, 6)
}

static inline uint64_t al256(uint64_t x) { return (x + 255) & ~(uint64_t)255; }

struct EpWs {
    int *status, *idx, *ecount, *eoffs, *elist, *pos, *ypos, *reid, *lcount, *loffs, *llist, *lpos, *soffs, *counts;
    float *wt, *Y;
    void *disp, *ldisp, *plan;
    uint8_t *Xq, *Xs, *rows_q, *rows_s, *Hq, *Hs;
    uint64_t total;
};
// T: most tokens per call on this rank; cap: rows one rank may send to one other rank per call
static EpWs ep_carve(void *base, int T, int cap, int world, int E, int k, int D, int FF) {
    EpWs w;
    uint8_t *p = (uint8_t *)base;
    uint64_t o = 0;
    auto take = [&](uint64_t b) { uint8_t *r = p + o; o += al256(b); return (void *)r; };
    const uint64_t n = (uint64_t)T * k, C = (uint64_t)cap, S = (uint64_t)world * C, R = S, RT = R + T;
    const uint64_t nbs = D / Q36_QK;
    w.status = (int *)take(256);
    w.idx = (int *)take(n * 4); w.wt = (float *)take(n * 4);
    w.ecount = (int *)take((uint64_t)E * 4); w.eoffs = (int *)take((uint64_t)(E + 1) * 4);
    w.elist = (int *)take(n * 4); w.pos = (int *)take(n * 4); w.ypos = (int *)take(n * 4);
    w.disp = take(dispatch_ws_bytes((int)n, E));
    w.Xq = (uint8_t *)take((uint64_t)T * D); w.Xs = (uint8_t *)take((uint64_t)T * nbs);
    w.reid = (int *)take(S * 4);
    w.lcount = (int *)take((uint64_t)E * 4); w.loffs = (int *)take((uint64_t)(E + 1) * 4);
    w.llist = (int *)take(S * 4); w.lpos = (int *)take(S * 4); w.soffs = (int *)take(8); w.counts = (int *)take(4 * EP_MAX_WORLD);
    w.ldisp = take(dispatch_ws_bytes((int)S, E));
    w.rows_q = (uint8_t *)take(RT * D); w.rows_s = (uint8_t *)take(RT * nbs);
    w.Hq = (uint8_t *)take(RT * FF); w.Hs = (uint8_t *)take(RT * (FF / Q36_QK));
    w.Y = (float *)take(RT * D * 4);
    w.plan = take(tc_ws_bytes());
    w.total = o;
    return w;
}

static int ckc(cudaError_t e) {
    if (e != cudaSuccess) { last_cuda_error() = (int)e; return Q36_MOE_ECUDA; }
    return Q36_MOE_OK;
}
static int ckn(ncclResult_t r) {
    if (r != ncclSuccess) { last_cuda_error() = 300000 + (int)r; return Q36_MOE_ECUDA; }
    return Q36_MOE_OK;
}

// NCCL transport: block p of `send` (bytes_per_peer each) -> rank p's `recv` block of this rank
static int all_to_all(NcclApi *api, EpComm *c, const void *send, void *recv, size_t bytes_per_peer, cudaStream_t st) {
    ncclResult_t r = api->GroupStart();
    for (int p = 0; p < c->world && r == ncclSuccess; p++) {
        r = api->Send((const uint8_t *)send + (size_t)p * bytes_per_peer, bytes_per_peer, ncclUint8, p, c->comm, st);
        if (r == ncclSuccess) r = api->Recv((uint8_t *)recv + (size_t)p * bytes_per_peer, bytes_per_peer, ncclUint8, p, c->comm, st);
    }
    const ncclResult_t e = api->GroupEnd();
    return ckn(r == ncclSuccess ? e : r);
}

static void close_window(EpComm *c) {
    if (!c->open) return;
    cudaSetDevice(c->device);
    for (int r = 0; r < c->world; r++)
        if (c->ipc_opened[r]) { cudaIpcCloseMemHandle(c->peer[r]); c->ipc_opened[r] = false; }
    if (c->d_peer) cudaFree(c->d_peer);
    if (c->stage) cudaFree(c->stage);
    if (c->win) cudaFree(c->win);
    c->d_peer = nullptr; c->stage = nullptr; c->win = nullptr;
    c->open = false;
}

// device copy of the table the kernels index by rank: the ranks' windows, or (NCCL transport) the local staging
static int push_peer_table(EpComm *c) {
    uint8_t *tbl[EP_MAX_WORLD];
    for (int r = 0; r < EP_MAX_WORLD; r++) tbl[r] = (c->transport == EP_TRANSPORT_NCCL) ? c->stage : c->peer[r];
    return ckc(cudaMemcpy(c->d_peer, tbl, sizeof tbl, cudaMemcpyHostToDevice));
}

struct LayerArgs {
    const void *Wg, *Wu, *Wd, *Sg, *Su, *Sd;
    int E, k, D, FF;
    const void *X;
    int x_is_bf16;
    const float *logits;
    int logit_stride, shgate_col;
    float route_scale;
    float *out;
    int T;
    void *ws;
    uint64_t ws_bytes;
};

// Two-launch (prefill-sized) calls over the peer transport return one weighted partial row per (token, expert rank)
// instead of one row per (token, expert); the rows use the first T_max rows of each rank's block of the result area.
static bool ep_reduced_return(const EpComm *c, bool one_launch) {
    return !one_launch && c->transport != EP_TRANSPORT_NCCL && c->world <= 8 && c->T_max <= c->L.cap;
}
static int ep_reduce_blocks(const EpComm *c) { return max(1, min(512 / c->world, (c->T_max + 15) / 16)); }

static int ep_phase(EpComm *c, int phase, const LayerArgs &a, cudaStream_t st) {
    const int world = c->world, rank = c->rank, E = a.E, k = a.k, D = a.D, FF = a.FF, T = a.T;
    if (!c->open) return Q36_MOE_EINVAL;
    if (!a.Wg || !a.Wu || !a.Wd || !a.X || !a.logits || !a.out || !a.ws) return Q36_MOE_EINVAL;
    if (T <= 0 || k <= 0 || k > 8 || E % world || E > DISPATCH_MAX_GROUPS || D % 512 || FF % 512 || a.logit_stride < E) return Q36_MOE_EINVAL;
    if (!router_supports(E)) return Q36_MOE_EINVAL;
    const int n = T * k, C = c->L.cap, S = world * C, R = S, per = E / world, se0 = rank * per, se1 = se0 + per;
    if (D != c->L.D || k != c->k || T > c->T_max) return Q36_MOE_ENOSPACE;   // the window was opened for other sizes
    // the private workspace is carved for the window's sizes so that every call sees the same layout
    const EpWs w = ep_carve(a.ws, c->T_max, C, world, E, k, D, FF);
    if (w.total > a.ws_bytes) return Q36_MOE_ENOSPACE;
    const int nbs = D / Q36_QK, rowb = c->L.row_bytes;
    const bool shared = a.Sg && a.Su && a.Sd;
    const WinLayout &L = c->L;
    int *ctl = (int *)(c->win + L.ctl);
    const bool use_nccl = c->transport == EP_TRANSPORT_NCCL;
    NcclApi *api = use_nccl ? nccl() : nullptr;
    if (use_nccl && (!api || c->kind != EP_KIND_PROCS)) return Q36_MOE_EINVAL;
    const int par = (int)((c->calls[phase < 3 && phase >= 0 ? phase : 0] + 1) & 1);   // NCCL transport only (host mirror of the phase's call counter)
    // the one-launch decode kernel: always when no expert can receive more than 16 rows, else up to a row count (every
    // rank takes the same decision for equal T)
    const bool one_launch = ffn_fused_small_fits(R + T, per, D, FF) && (world * T <= 16 || R + T <= fused_rows_limit());
    const bool reduced = ep_reduced_return(c, one_launch);
    const int ybf = one_launch ? 0 : stage_y_bf16();     // the two grouped-GEMM launches stage their result rows as bf16
    int rc;
    if (phase == 0) {
        // route + dispatch over ALL experts (their order is the destination-rank order); quantise the rank's tokens
        // once, in token order (hw order inside the blocks): one cluster launch at decode sizes
        const bool cluster_front = !reduced && T <= 16 && n <= 128 && D % 1024 == 0 && D * T <= 32 * 1024;
        if (cluster_front) {
            // ... and the rows go straight from the quantising warps into the destination ranks' windows
            const EpSendArgs sa{(uint8_t *const *)c->d_peer, L.rows[0], L.rows[1], L.hdr[0], L.hdr[1], ctl, w.ypos, rank, world, per, C, use_nccl ? 1 : 0};
            if ((rc = launch_front_decode(a.logits, E, k, a.route_scale, T, a.logit_stride, w.idx, w.wt, w.ecount, w.eoffs, w.elist,
                                          w.pos, nullptr, 0, 0, nullptr, D, FF, w.status, a.X, a.x_is_bf16, w.Xq, w.Xs, 0, 0, st, &sa)))
                return rc;
        } else if (n <= 1024) {
            if ((rc = launch_front_small(a.logits, E, k, a.route_scale, T, a.logit_stride, 0, E, w.idx, w.wt, w.ecount, w.eoffs,
                                         w.elist, w.pos, nullptr, 0, 0, nullptr, D, FF, w.status, nullptr, 0, nullptr, nullptr, -1, 0, st)))
                return rc;
        } else {
            if ((rc = launch_router_topk(a.logits, E, k, w.idx, w.wt, a.route_scale, 1, T, a.logit_stride, st))) return rc;
            if ((rc = launch_dispatch(w.idx, n, E, 0, E, w.ecount, w.eoffs, w.elist, w.pos, w.disp, nullptr, 0, 0, st))) return rc;
        }
        if (!cluster_front && (rc = launch_quant(a.X, a.x_is_bf16, w.Xq, w.Xs, T, D, nullptr, 0, 0, true, st))) return rc;
        // (larger calls: a kernel of its own.)  Blocks per destination: one up to 256 rows, then one per 256 (at most 32)
        const int nb_send = max(1, min(32, (min(n, C) + 255) / 256));
        if (!cluster_front) launch_k(k_ep_send, dim3(world * nb_send), dim3(1024), 0, st, (const uint8_t *)w.Xq, (const uint8_t *)w.Xs, (const int *)w.idx,
                 (const int *)w.eoffs, (const int *)w.elist, world, per, k, C, D, (uint8_t *const *)c->d_peer, rank, L.rows[0], L.rows[1],
                 L.hdr[0], L.hdr[1], ctl, w.ypos, use_nccl ? 1 : 0, w.status, nb_send, (const int *)w.pos, (const float *)w.wt, n, T,
                 L.tslot[0], L.tslot[1], L.twt[0], L.twt[1], L.tstride, reduced ? 1 : 0);
        if ((rc = check_launch())) return rc;
        if (use_nccl) {   // staging blocks (indexed by destination) -> the destinations' windows (indexed by source)
            if ((rc = all_to_all(api, c, c->stage + L.rows[par], c->win + L.rows[par], (size_t)C * rowb, st))) return rc;
            if ((rc = all_to_all(api, c, c->stage + L.hdr[par], c->win + L.hdr[par], 8, st))) return rc;
        }
        c->calls[0]++;
        return Q36_MOE_OK;
    }
    if (phase == 1) {
        // local plan over the received slots
        const bool small_plan = S <= 1024;   // one block waits, sorts the slots and writes the work plan
        if (small_plan) {
            if ((rc = launch_ep_recv_plan(c->win, L.hdr[0], L.hdr[1], L.rows[0], L.rows[1], ctl, world, C, rowb, D + nbs, c->spin_limit,
                                          w.status, E, se0, se1, w.lcount, w.loffs, w.llist, w.lpos, w.soffs, R, shared ? R + T : R,
                                          w.plan, D, FF, one_launch ? 16 : gateup_tile_rows(), w.counts, st)))
                return rc;
        } else {
            launch_k(k_ep_wait_eids, dim3((S + 255) / 256), dim3(256), 0, st, (const uint8_t *)c->win, L.hdr[0], L.hdr[1], L.rows[0],
                     L.rows[1], (const int *)ctl, world, C, rowb, D + nbs, c->spin_limit, w.status, w.reid, w.counts);
            if ((rc = launch_dispatch(w.reid, S, E, se0, se1, w.lcount, w.loffs, w.llist, w.lpos, w.ldisp, w.soffs, R, shared ? R + T : R, st,
                                      w.plan, D, FF, one_launch ? 16 : gateup_tile_rows())))   // (+ the work plan)
                return rc;
        }
        launch_k(k_ep_unpack, dim3(min((R + T + 7) / 8, 16 * sm_count())), dim3(256), 0, st, (const uint8_t *)c->win, L.rows[0], L.rows[1], (const int *)ctl,
                 (const int *)w.llist, (const int *)(w.loffs + E), (const uint8_t *)w.Xq, (const uint8_t *)w.Xs, R, T, D, w.rows_q, w.rows_s, w.status);
        if ((rc = check_launch())) return rc;
        // grouped expert FFN on the local shard (+ shared expert on the own tokens)
        if (one_launch) {
            // its down epilogue stores the routed result rows straight into their home ranks' windows and its last CTA
            // publishes; the shared expert's rows stay in Y for the combine
            const EpReturnArgs ra{(uint8_t *const *)c->d_peer, L.ret[0], L.ret[1], L.rhdr[0], L.rhdr[1], ctl, w.llist, R, rank, world, C, use_nccl ? 1 : 0};
            if ((rc = launch_ffn_fused_small(a.Wg, a.Wu, a.Wd, shared ? a.Sg : nullptr, shared ? a.Su : nullptr, shared ? a.Sd : nullptr,
                                             per, R + T, w.rows_q, w.rows_s, w.Hq, w.Hs, w.Y, D, FF, w.plan, w.status, &ra, st)))
                return rc;
        } else {
            if ((rc = launch_gateup_tc(a.Wg, a.Wu, shared ? a.Sg : nullptr, shared ? a.Su : nullptr, per, R + T, R + T, w.rows_q, w.rows_s,
                                       w.Hq, w.Hs, D, FF, w.plan, w.status, st)))
                return rc;
            if ((rc = launch_down_tc(a.Wd, shared ? a.Sd : nullptr, per, R + T, R + T, w.Hq, w.Hs, w.Y, D, FF, w.plan, w.status + 1, st, ybf)))
                return rc;
        }
        // (two launches: a kernel of its own puts the result rows into their home ranks' windows)
        // blocks per source: one while a pair of ranks exchanges at most 64 rows (a single fence on the way), else one per 64
        const int nb_ret = max(1, min(32, (min(c->T_max * k, C) + 63) / 64));
        if (reduced) {
            const int nb = ep_reduce_blocks(c);
            launch_k(k_ep_reduce_return, dim3(world * nb), dim3(512), 0, st, (const float *)w.Y, (const int *)w.lpos, (const uint8_t *)c->win,
                     L.tslot[0], L.tslot[1], L.twt[0], L.twt[1], L.tstride, k, world, C, D, (uint8_t *const *)c->d_peer, rank, L.ret[0], L.ret[1],
                     L.rhdr[0], L.rhdr[1], ctl, nb, w.status, ybf);
        } else if (!one_launch) launch_k(k_ep_return, dim3(world * nb_ret), dim3(1024), 0, st, (const float *)w.Y, (const int *)w.lpos, (const int *)w.counts, world, C, D,
                 (uint8_t *const *)c->d_peer, rank, L.ret[0], L.ret[1], L.rhdr[0], L.rhdr[1], ctl, use_nccl ? 1 : 0, nb_ret, w.status, ybf);
        if ((rc = check_launch())) return rc;
        if (use_nccl) {
            if ((rc = all_to_all(api, c, c->stage + L.ret[par], c->win + L.ret[par], (size_t)C * D * 4, st))) return rc;
            if ((rc = all_to_all(api, c, c->stage + L.rhdr[par], c->win + L.rhdr[par], 8, st))) return rc;
            if ((rc = ckc(cudaMemsetAsync(c->stage + L.rhdr[par], 0, 8 * EP_MAX_WORLD, st)))) return rc;   // the staged arrival counts start at zero next time
        }
        c->calls[1]++;
        return Q36_MOE_OK;
    }
    if (phase == 2) {
        // what every expert rank counts in at this rank per call: the CTAs of its one-launch FFN, else its return blocks
        const unsigned expected = one_launch ? (unsigned)ffn_fused_small_grid(R + T, per, D, FF)
                                  : reduced        ? (unsigned)ep_reduce_blocks(c)
                                                   : (unsigned)max(1, min(32, (min(c->T_max * k, C) + 63) / 64));
        const float *shg = (shared && a.shgate_col >= 0) ? a.logits + a.shgate_col : nullptr;
        launch_k(k_ep_combine, dim3((D / 4 + 255) / 256, T), dim3(256), 0, st, a.out, (const uint8_t *)c->win, L.ret[0], L.ret[1],
                 L.rhdr[0], L.rhdr[1], ctl, world, c->spin_limit, w.status, (const int *)w.ypos, (const float *)w.wt,
                 shared ? y_row(w.Y, R, D, ybf) : (const float *)nullptr, shg, a.logit_stride, D, k, expected, reduced ? 1 : 0, C, ybf);
        c->calls[2]++;
        return check_launch();
    }
    return Q36_MOE_EINVAL;
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
    if (!api || !id128 || !comm_out || world < 1 || world > EP_MAX_WORLD || rank < 0 || rank >= world) return Q36_MOE_EINVAL;
    ncclUniqueId id;
    memcpy(&id, id128, sizeof id);
    EpComm *c = new EpComm;
    c->rank = rank; c->world = world; c->kind = EP_KIND_PROCS;
    cudaGetDevice(&c->device);
    const int rc = ckn(api->CommInitRank(&c->comm, world, id, rank));
    if (rc) { delete c; return rc; }
    *comm_out = c;
    return Q36_MOE_OK;
}

int q36_moe_ep_init_local(int world, const int *devices, void **comms_out) {
    if (!devices || !comms_out || world < 1 || world > EP_MAX_WORLD) return Q36_MOE_EINVAL;
    EpComm **group = new EpComm *[world];
    for (int r = 0; r < world; r++) {
        EpComm *c = new EpComm;
        c->rank = r; c->world = world; c->kind = EP_KIND_LOCAL; c->device = devices[r]; c->group = group;
        group[r] = c;
        comms_out[r] = c;
    }
    return Q36_MOE_OK;
}

int q36_moe_ep_destroy(void *comm) {
    EpComm *c = (EpComm *)comm;
    if (!c) return Q36_MOE_EINVAL;
    int dev = 0;
    cudaGetDevice(&dev);
    close_window(c);
    cudaSetDevice(dev);
    if (c->kind == EP_KIND_PROCS) {
        NcclApi *api = nccl();
        if (api && c->comm) api->CommDestroy(c->comm);
    } else if (c->rank == 0) {
        // rank 0 owns the shared array; the caller destroys rank 0 last
        delete[] c->group;
    }
    delete c;
    return Q36_MOE_OK;
}

int q36_moe_ep_set_transport(void *comm, int transport) {
    EpComm *c = (EpComm *)comm;
    if (!c || (transport != EP_TRANSPORT_PEER && transport != EP_TRANSPORT_NCCL)) return Q36_MOE_EINVAL;
    if (transport == EP_TRANSPORT_NCCL && c->kind != EP_KIND_PROCS) return Q36_MOE_EINVAL;
    c->transport = transport;
    if (!c->open) return Q36_MOE_OK;
    if (transport == EP_TRANSPORT_NCCL && !c->stage) {
        int rc = ckc(cudaMalloc((void **)&c->stage, c->L.bytes));
        if (rc) return rc;
        if ((rc = ckc(cudaMemset(c->stage, 0, c->L.bytes)))) return rc;
    }
    return push_peer_table(c);
}

int q36_moe_ep_open_window(void *comm, int T_max, int k, int D, int cap_rows) {
    EpComm *c0 = (EpComm *)comm;
    if (!c0 || T_max <= 0 || k <= 0 || k > 8 || D % 512 || cap_rows < 0 || cap_rows > T_max * k) return Q36_MOE_EINVAL;
    int dev0 = 0;
    cudaGetDevice(&dev0);
    const int world = c0->world;
    const WinLayout L = win_layout(world, cap_rows ? cap_rows : T_max * k, D, T_max * k);
    int rc = Q36_MOE_OK;
    auto alloc_one = [&](EpComm *c) -> int {
        close_window(c);
        int r;
        if ((r = ckc(cudaSetDevice(c->device)))) return r;
        c->L = L; c->T_max = T_max; c->k = k;
        if ((r = ckc(cudaMalloc((void **)&c->win, L.bytes)))) return r;
        if ((r = ckc(cudaMemset(c->win, 0, L.bytes)))) return r;
        if ((r = ckc(cudaMalloc((void **)&c->d_peer, sizeof(uint8_t *) * EP_MAX_WORLD)))) return r;
        c->calls[0] = c->calls[1] = c->calls[2] = 0;
        c->open = true;
        return Q36_MOE_OK;
    };
    if (c0->kind == EP_KIND_LOCAL) {
        // one process: every rank's window is plain device memory; ranks on different devices reach it by peer access
        for (int r = 0; r < world && !rc; r++) rc = alloc_one(c0->group[r]);
        for (int r = 0; r < world && !rc; r++) {
            EpComm *c = c0->group[r];
            cudaSetDevice(c->device);
            bool same_device_only = true;
            for (int p = 0; p < world; p++) {
                c->peer[p] = c0->group[p]->win;
                if (c0->group[p]->device != c->device) {
                    same_device_only = false;
                    const cudaError_t e = cudaDeviceEnablePeerAccess(c0->group[p]->device, 0);
                    if (e != cudaSuccess && e != cudaErrorPeerAccessAlreadyEnabled) rc = ckc(e);
                    cudaGetLastError();
                }
            }
            // ranks that take turns on ONE device run their phases in stream order: a header is there before the kernel
            // that reads it starts, so a wait never has to spin; keep the limit small so a wrong phase order ends at once
            if (same_device_only) c->spin_limit = 1024;
            if (!rc) rc = push_peer_table(c);
        }
        if (!rc) rc = ckc(cudaDeviceSynchronize());
        cudaSetDevice(dev0);
        return rc;
    }
    // one process per GPU: exchange CUDA IPC handles of the windows over NCCL
    NcclApi *api = nccl();
    if (!api) return Q36_MOE_EINVAL;
    if ((rc = alloc_one(c0))) return rc;
    cudaIpcMemHandle_t mine, all[EP_MAX_WORLD];
    if ((rc = ckc(cudaIpcGetMemHandle(&mine, c0->win)))) return rc;
    uint8_t *d_h = nullptr;
    if ((rc = ckc(cudaMalloc((void **)&d_h, sizeof(mine) * (world + 1))))) return rc;
    if (!rc) rc = ckc(cudaMemcpy(d_h, &mine, sizeof mine, cudaMemcpyHostToDevice));
    if (!rc) rc = ckn(api->AllGather(d_h, d_h + sizeof mine, sizeof mine, ncclUint8, c0->comm, (cudaStream_t)0));
    if (!rc) rc = ckc(cudaStreamSynchronize((cudaStream_t)0));
    if (!rc) rc = ckc(cudaMemcpy(all, d_h + sizeof mine, sizeof(mine) * world, cudaMemcpyDeviceToHost));
    cudaFree(d_h);
    for (int p = 0; p < world && !rc; p++) {
        if (p == c0->rank) { c0->peer[p] = c0->win; continue; }
        void *ptr = nullptr;
        rc = ckc(cudaIpcOpenMemHandle(&ptr, all[p], cudaIpcMemLazyEnablePeerAccess));
        if (!rc) { c0->peer[p] = (uint8_t *)ptr; c0->ipc_opened[p] = true; }
    }
    if (!rc && c0->transport == EP_TRANSPORT_NCCL) {
        rc = ckc(cudaMalloc((void **)&c0->stage, L.bytes));
        if (!rc) rc = ckc(cudaMemset(c0->stage, 0, L.bytes));
    }
    if (!rc) rc = push_peer_table(c0);
    if (!rc) rc = ckc(cudaDeviceSynchronize());
    return rc;
}

uint64_t q36_moe_ep_workspace_bytes(int T_max, int cap_rows, int world, int n_expert, int k, int D, int FF) {
    if (T_max <= 0 || world <= 0 || n_expert <= 0 || k <= 0 || cap_rows < 0) return 0;
    return ep_carve(nullptr, T_max, cap_rows ? cap_rows : T_max * k, world, n_expert, k, D, FF).total;
}

int q36_moe_ep_layer_phase(void *comm, int phase, const void *Wg, const void *Wu, const void *Wd, const void *Sg, const void *Su,
                           const void *Sd, int n_expert, int k, int D, int FF, const void *X, int x_is_bf16, const float *logits,
                           int logit_stride, int shgate_col, float route_scale, float *out, int T, void *ws, uint64_t ws_bytes,
                           void *stream) {
    EpComm *c = (EpComm *)comm;
    if (!c) return Q36_MOE_EINVAL;
    const LayerArgs a{Wg, Wu, Wd, Sg, Su, Sd, n_expert, k, D, FF, X, x_is_bf16, logits, logit_stride, shgate_col, route_scale, out, T, ws, ws_bytes};
    return ep_phase(c, phase, a, (cudaStream_t)stream);
}

int q36_moe_ep_layer(void *comm, const void *Wg, const void *Wu, const void *Wd, const void *Sg, const void *Su,
                     const void *Sd, int n_expert, int k, int D, int FF, const void *X, int x_is_bf16,
                     const float *logits, int logit_stride, int shgate_col, float route_scale, float *out, int T,
                     void *ws, uint64_t ws_bytes, void *stream) {
    EpComm *c = (EpComm *)comm;
    if (!c) return Q36_MOE_EINVAL;
    const LayerArgs a{Wg, Wu, Wd, Sg, Su, Sd, n_expert, k, D, FF, X, x_is_bf16, logits, logit_stride, shgate_col, route_scale, out, T, ws, ws_bytes};
    int rc;
    for (int phase = 0; phase < 3; phase++)
        if ((rc = ep_phase(c, phase, a, (cudaStream_t)stream))) return rc;
    return Q36_MOE_OK;
}

// The expert-parallel stack from host buffers (this rank's tokens of every layer): three copies per step around
// n_layers calls of the layer step.  dev_io: q36_moe_stack_host_io_bytes(...) bytes.
int q36_moe_ep_stack_host(void *comm, int n_layers, const void *const *Wg, const void *const *Wu, const void *const *Wd,
                          const void *const *Sg, const void *const *Su, const void *const *Sd, int n_expert, int k, int D, int FF,
                          const void *host_X, int x_is_bf16, const float *host_logits, int logit_stride, int shgate_col,
                          float route_scale, float *host_out, int T, void *dev_io, void *ws, uint64_t ws_bytes, void *stream) {
    EpComm *c = (EpComm *)comm;
    if (!c || n_layers <= 0 || !Wg || !Wu || !Wd || !host_X || !host_logits || !host_out || !dev_io || T <= 0) return Q36_MOE_EINVAL;
    cudaStream_t st = (cudaStream_t)stream;
    const uint64_t xb = (uint64_t)T * D * (x_is_bf16 ? 2 : 4), lb = (uint64_t)T * logit_stride * 4, ob = (uint64_t)T * D * 4;
    uint8_t *dX = (uint8_t *)dev_io, *dL = dX + al256(xb * n_layers), *dO = dL + al256(lb * n_layers);
    int rc;
    if ((rc = ckc(cudaMemcpyAsync(dX, host_X, xb * n_layers, cudaMemcpyHostToDevice, st)))) return rc;
    if ((rc = ckc(cudaMemcpyAsync(dL, host_logits, lb * n_layers, cudaMemcpyHostToDevice, st)))) return rc;
    for (int l = 0; l < n_layers; l++) {
        const LayerArgs a{Wg[l], Wu[l], Wd[l], Sg ? Sg[l] : nullptr, Su ? Su[l] : nullptr, Sd ? Sd[l] : nullptr, n_expert, k, D, FF,
                          dX + xb * l, x_is_bf16, (const float *)(dL + lb * l), logit_stride, shgate_col, route_scale,
                          (float *)(dO + ob * l), T, ws, ws_bytes};
        for (int phase = 0; phase < 3; phase++)
            if ((rc = ep_phase(c, phase, a, st))) return rc;
    }
    if ((rc = ckc(cudaMemcpyAsync(host_out, dO, ob * n_layers, cudaMemcpyDeviceToHost, st)))) return rc;
    if ((rc = ckc(cudaStreamSynchronize(st)))) return rc;
    return q36_moe_ws_status(ws, stream);
}

}  // extern "C"
