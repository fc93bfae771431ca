"""Expert-parallel MoE layer over the GPUs of one node.

The reference shards experts in contiguous blocks [r*E/N, (r+1)*E/N)
(q36_engine.cu:4245), replicates every token on every device and sum-reduces
the partial outputs through device 0 with peer copies (q36_engine.cu:4279-4293).
Here tokens stay data-parallel (each rank routes its own T tokens) and only the
routed rows travel: one all-to-all dispatches quantised activation rows
(2048 E4M3 bytes + 64 UE8M0 scale bytes + the expert id) to the ranks that own
the experts, the grouped expert FFN runs on the local shard, one all-to-all
brings the f32 result rows back, and the home rank does the weighted combine
and adds its shared expert (replicated on every rank).

The product path is the native one (`NativeEP`, `LocalEP` -> q36_moe_ep_layer):
the library's own kernels store the routed rows and the result rows straight
into the destination rank's exchange window over NVLink, with a capacity of
rows per pair of ranks fixed when the window is opened, so that no count ever
has to reach the host and the whole step stays launch-only.

`ep_layer` below is the same step written with torch.distributed collectives
over an `ops` object: `DeviceOps` binds the C-ABI kernels; the CPU tests
substitute an oracle-backed stand-in to exercise the slot arithmetic and the
exchange pattern on world-size-2 gloo ranks.
"""
from __future__ import annotations

import torch
import torch.distributed as dist


def slot_maps(idx: torch.Tensor, eoffs: torch.Tensor, elist: torch.Tensor, pos: torch.Tensor, world: int, E: int,
              k: int, C: int):
    """Index arithmetic of the fixed-capacity exchange (pure tensor ops, no host sync).

    idx [T,k] expert of entry; eoffs [E+1], elist [n], pos [n] from the dispatch over ALL E experts.
    Returns
      tok_of_slot [world*C]  source token of every send slot, -1 for an empty slot
      eid_of_slot [world*C]  global expert id of the row in that slot, -1 if empty
      ypos [n]               slot in which entry i's result row comes back
    """
    n = idx.numel()
    per = E // world
    dev = idx.device
    rank_base = eoffs[0:E:per].to(torch.int64)                       # first sorted row of each destination rank
    rank_end = eoffs[per:E + 1:per].to(torch.int64)
    cnt = rank_end - rank_base
    slots = torch.arange(world * C, device=dev, dtype=torch.int64)
    r, j = slots // C, slots % C
    valid = j < cnt[r]
    p = (rank_base[r] + j).clamp_(max=max(n - 1, 0))
    entry = elist.to(torch.int64)[p]
    flat = idx.reshape(-1).to(torch.int64)
    tok_of_slot = torch.where(valid, entry // k, torch.full_like(entry, -1)).to(torch.int32)
    eid_of_slot = torch.where(valid, flat[entry], torch.full_like(entry, -1)).to(torch.int32)
    dest = flat // per
    ypos = (dest * C + pos.to(torch.int64) - rank_base[dest]).to(torch.int32)
    return tok_of_slot, eid_of_slot, ypos


class DeviceOps:
    """The C-ABI kernels (q36_b200.moe) behind the small interface the EP step needs."""

    def __init__(self, moe):
        self.m = moe

    def router_topk(self, logits, E, k):
        return self.m.router_topk(logits, E, k)

    def dispatch(self, eid, E, se0=0, se1=None):
        return self.m.dispatch(eid, E, se0, se1)

    def quant_rows(self, X):
        """[T,D] -> (Xq [T,D] hw order, Xs [T,D/32]) in token order."""
        return self.m.quant_scatter(X, None, 0, 0, X.shape[0])

    def gather_rows(self, src, index):
        return self.m.gather_rows(src, index)

    def ffn(self, layer, goffs, Xq, Xs, soffs, path):
        return self.m.expert_ffn_sorted(layer.Wg, layer.Wu, layer.Wd, layer.se1 - layer.se0, goffs, Xq, Xs, layer.D,
                                        layer.FF, path, sync_check=False, shared=(layer.Sg, layer.Su, layer.Sd),
                                        soffs=soffs)[2]

    def combine(self, Y, ypos, wt, SH, shgate, stride, D, k, T):
        return self.m.combine(Y, ypos, wt, SH, shgate, stride, D, k, T)


_SOFFS_CACHE: dict = {}


def _soffs(R: int, T: int, device) -> torch.Tensor:
    """Row range of the shared expert's group, built once per shape (a host-to-device copy is not capturable)."""
    key = (R, T, str(device))
    if key not in _SOFFS_CACHE:
        _SOFFS_CACHE[key] = torch.tensor([R, R + T], dtype=torch.int32, device=device)
    return _SOFFS_CACHE[key]


def ep_layer(ops, layer, X, logits, world: int, rank: int, E: int, k: int, path: int, group=None, reduced: bool = False):
    """One expert-parallel layer step for this rank's T tokens (the same T on every rank).  Returns out [T,D] f32.
    reduced: the expert ranks sum a token's result rows with the combine weights and return one row per (token,
    expert rank) instead of one per (token, expert) -- what the native step does for prefill-sized calls."""
    T, D = X.shape
    C = T * k
    per = E // world
    idx, wt = ops.router_topk(logits, E, k)
    ecount, eoffs, elist, pos = ops.dispatch(idx.reshape(-1), E)
    Xq, Xs = ops.quant_rows(X)
    tok_of_slot, eid_of_slot, ypos = slot_maps(idx, eoffs, elist, pos, world, E, k, C)
    send_q = ops.gather_rows(Xq, tok_of_slot)                 # [world*C, D]
    send_s = ops.gather_rows(Xs, tok_of_slot)                 # [world*C, D/32]
    recv_q, recv_s, recv_e = torch.empty_like(send_q), torch.empty_like(send_s), torch.empty_like(eid_of_slot)
    dist.all_to_all_single(recv_q, send_q, group=group)
    dist.all_to_all_single(recv_s, send_s, group=group)
    dist.all_to_all_single(recv_e, eid_of_slot, group=group)
    # local plan: sort the received slots by (local) expert; empty slots carry -1 and drop out
    se0, se1 = rank * per, (rank + 1) * per
    lcount, loffs, llist, lpos = ops.dispatch(recv_e, E, se0, se1)
    R = world * C
    rows_q = torch.cat([ops.gather_rows(recv_q, _pad_index(llist, R)), Xq], 0)     # sorted rows, then own tokens
    rows_s = torch.cat([ops.gather_rows(recv_s, _pad_index(llist, R)), Xs], 0)
    soffs = _soffs(R, T, X.device)
    Y = ops.ffn(layer, loffs[se0:], rows_q, rows_s, soffs, path)                  # [R+T, D] f32
    back = ops.gather_rows(Y, lpos)                                               # result row of every received slot
    stride = logits.shape[1]
    shg = logits[:, E:] if stride > E else None
    if reduced:
        # the weight of every send slot travels with its token index; empty slots carry weight 0 and token -1
        wt_of_slot = torch.zeros(world * C, dtype=torch.float32, device=X.device)
        wt_of_slot[ypos.long()] = wt.reshape(-1).float()
        recv_t, recv_w = torch.empty_like(tok_of_slot), torch.empty_like(wt_of_slot)
        dist.all_to_all_single(recv_t, tok_of_slot, group=group)
        dist.all_to_all_single(recv_w, wt_of_slot, group=group)
        src = torch.arange(world * C, device=X.device) // C                       # source rank of every received slot
        row = (src * T + recv_t.long().clamp(min=0))                              # (source, token) -> row of the partial sums
        contrib = back.float() * torch.where(recv_t >= 0, recv_w, torch.zeros_like(recv_w))[:, None]
        partial = torch.zeros((world * T, D), dtype=torch.float32, device=X.device).index_add_(0, row, contrib)
        recv_p = torch.empty_like(partial)
        dist.all_to_all_single(recv_p, partial, group=group)                      # block r: what expert rank r summed for my tokens
        out = recv_p.reshape(world, T, D).sum(0)
        SH = Y[R:].float()
        gate = torch.sigmoid(shg[:, 0].float())[:, None] if shg is not None else 1.0
        return out + gate * SH
    recv_y = torch.empty_like(back)
    dist.all_to_all_single(recv_y, back, group=group)
    return ops.combine(recv_y, ypos, wt, Y[R:], shg, stride, D, k, T)


def _pad_index(llist: torch.Tensor, R: int) -> torch.Tensor:
    """dispatch() returns the packed list of resident entries followed by unwritten slots (-1)."""
    if llist.numel() == R:
        return llist
    out = torch.full((R,), -1, dtype=torch.int32, device=llist.device)
    out[:llist.numel()] = llist
    return out


TRANSPORT_PEER, TRANSPORT_NCCL = 0, 1


def _layer_args(m, ly, X, logits, out, ws):
    stride = logits.shape[1]
    return (ly.Wg.data_ptr(), ly.Wu.data_ptr(), ly.Wd.data_ptr(), m.ptr(ly.Sg), m.ptr(ly.Su), m.ptr(ly.Sd), ly.E, ly.k, ly.D,
            ly.FF, X.data_ptr(), int(X.dtype == torch.bfloat16), logits.data_ptr(), stride, ly.E if stride > ly.E else -1, 1.0,
            out.data_ptr(), X.shape[0], ws.data_ptr(), ws.numel(), m.stream_ptr())


class NativeEP:
    """One process per GPU.  The C entry point q36_moe_ep_layer issues the whole step from native code on the
    current stream: the library's kernels store routed rows and result rows straight into the peer ranks'
    exchange windows (CUDA IPC over NVLink).  torch.distributed only carries the 128-byte NCCL id at set-up; NCCL
    itself only carries the IPC handles, unless `transport=TRANSPORT_NCCL` asks for the comparison transport."""

    def __init__(self, layers, world: int, rank: int, T: int, transport: int = TRANSPORT_PEER, cap_rows: int = 0):
        import ctypes as C
        from . import moe
        self.moe, self.layers, self.world, self.rank, self.T = moe, layers, world, rank, T
        ly = layers[0]
        # kernels per layer step: front (cluster at decode sizes, else router + dispatch x3 + quantise), send, the
        # received slots' plan, unpack, FFN (one launch up to q36_moe_one_launch_rows() rows, else two), return, combine
        small_front = T <= 16 and T * ly.k <= 128
        S = world * (cap_rows or T * ly.k)
        one_launch = S + T <= moe.lib.q36_moe_one_launch_rows()
        self.launches_per_layer = (1 if small_front else (2 if T * ly.k <= 1024 else 6)) + 1 + (1 if S <= 1024 else 5) + 1 + \
            (1 if one_launch else 2) + 1 + 1
        dev = ly.device
        idt = torch.zeros(128, dtype=torch.uint8)
        if rank == 0:
            buf = (C.c_uint8 * 128)()
            moe.check(moe.lib.q36_moe_ep_unique_id(buf), "ep_unique_id")
            idt = torch.tensor(list(buf), dtype=torch.uint8)
        idt = idt.to(dev)
        dist.broadcast(idt, src=0)
        idb = bytes(idt.cpu().tolist())
        comm = C.c_void_p()
        moe.check(moe.lib.q36_moe_ep_init(idb, rank, world, C.byref(comm)), "ep_init")
        self.comm = comm
        moe.check(moe.lib.q36_moe_ep_set_transport(comm, transport), "ep_set_transport")
        moe.check(moe.lib.q36_moe_ep_open_window(comm, T, ly.k, ly.D, cap_rows), "ep_open_window")
        n = int(moe.lib.q36_moe_ep_workspace_bytes(T, cap_rows, world, ly.E, ly.k, ly.D, ly.FF))
        self.ws = torch.empty(n, dtype=torch.uint8, device=dev)
        moe.check(moe.lib.q36_moe_ws_reset(self.ws.data_ptr(), moe.stream_ptr()), "ws_reset")

    def layer(self, ly, X, logits, out):
        m = self.moe
        m.check(m.lib.q36_moe_ep_layer(self.comm, *_layer_args(m, ly, X, logits, out, self.ws)), "ep_layer")
        return out

    def second_workspace(self):
        """A second private workspace: calls whose phases overlap (phase 0 of the next call issued before phases 1 and
        2 of this one) must alternate between two."""
        w = torch.empty_like(self.ws)
        self.moe.check(self.moe.lib.q36_moe_ws_reset(w.data_ptr(), self.moe.stream_ptr()), "ws_reset")
        return w

    def phase(self, p: int, ly, X, logits, out, stream=None, ws=None):
        m = self.moe
        args = list(_layer_args(m, ly, X, logits, out, self.ws if ws is None else ws))
        if stream is not None:
            args[-1] = stream.cuda_stream
        m.check(m.lib.q36_moe_ep_layer_phase(self.comm, p, *args), f"ep_layer_phase {p}")

    def step(self, Xs, Ls, outs):
        for l, ly in enumerate(self.layers):
            self.layer(ly, Xs[l], Ls[l], outs[l])

    def check_device_status(self):
        self.moe.check(self.moe.lib.q36_moe_ws_status(self.ws.data_ptr(), self.moe.stream_ptr()), "device status")

    def close(self):
        if self.comm:
            self.moe.lib.q36_moe_ep_destroy(self.comm)
            self.comm = None


class LocalEP:
    """One process, `world` ranks on the listed devices (q36_moe_ep_init_local), driven from one host thread
    the way the engine's own multi-GPU driver works (q36_engine.cu:4261-4306).  Listing one device several
    times makes its ranks take turns on it: the full 2/4/8-rank data path on a single GPU."""

    def __init__(self, world: int, devices, T_max: int, E: int, k: int, D: int, FF: int, cap_rows: int = 0):
        import ctypes as C
        from . import moe
        self.moe, self.world, self.devices = moe, world, list(devices)
        comms = (C.c_void_p * world)()
        moe.check(moe.lib.q36_moe_ep_init_local(world, (C.c_int * world)(*self.devices), comms), "ep_init_local")
        self.comms = [C.c_void_p(c) for c in comms]
        moe.check(moe.lib.q36_moe_ep_open_window(self.comms[0], T_max, k, D, cap_rows), "ep_open_window")
        n = int(moe.lib.q36_moe_ep_workspace_bytes(T_max, cap_rows, world, E, k, D, FF))
        self.ws = []
        for r in range(world):
            with torch.cuda.device(self.devices[r]):
                w = torch.empty(n, dtype=torch.uint8, device=f"cuda:{self.devices[r]}")
                moe.check(moe.lib.q36_moe_ws_reset(w.data_ptr(), moe.stream_ptr()), "ws_reset")
            self.ws.append(w)

    def phase(self, p: int, r: int, ly, X, logits, out, ws=None):
        m = self.moe
        with torch.cuda.device(self.devices[r]):
            return m.lib.q36_moe_ep_layer_phase(self.comms[r], p, *_layer_args(m, ly, X, logits, out, self.ws[r] if ws is None else ws))

    def layer(self, shards, Xs, Ls, outs):
        """One call on every rank: phase p of all ranks before phase p + 1 of any."""
        for p in range(3):
            for r in range(self.world):
                self.moe.check(self.phase(p, r, shards[r], Xs[r], Ls[r], outs[r]), f"rank {r} phase {p}")
        return outs

    def status(self, r: int) -> int:
        with torch.cuda.device(self.devices[r]):
            return self.moe.lib.q36_moe_ws_status(self.ws[r].data_ptr(), self.moe.stream_ptr())

    def reset_status(self, r: int):
        with torch.cuda.device(self.devices[r]):
            self.moe.check(self.moe.lib.q36_moe_ws_reset(self.ws[r].data_ptr(), self.moe.stream_ptr()), "ws_reset")

    def close(self):
        for c in reversed(self.comms):      # rank 0 last
            self.moe.lib.q36_moe_ep_destroy(c)
        self.comms = []


class EPStack:
    """A stack of layers stepped expert-parallel; `step` runs every layer on this rank's tokens."""
    launches_per_layer = 17     # kernels of this library per layer step (dispatch x2, quant, gathers x5, FFN x2, combine)

    def __init__(self, layers, world: int, rank: int, T: int, path: int | None = None, group=None):
        from . import moe
        self.ops = DeviceOps(moe)
        self.layers, self.world, self.rank, self.T, self.group = layers, world, rank, T, group
        self.path = moe.PATH_TC if path is None else path

    def step(self, Xs, Ls, outs):
        for l, layer in enumerate(self.layers):
            o = ep_layer(self.ops, layer, Xs[l], Ls[l], self.world, self.rank, layer.E, layer.k, self.path, self.group)
            outs[l].copy_(o)
