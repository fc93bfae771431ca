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

Decode-sized steps use a FIXED capacity per peer (C = T*k rows, the worst
case) so that no count ever has to reach the host: the exchange is two
equal-split all-to-alls and the whole step stays launch-only.  Slot j of the
block sent to rank r holds the j-th row (in expert order) routed to r, or is
marked empty (expert id -1).

All device work goes through an `ops` object: `DeviceOps` binds the C-ABI
kernels; the CPU tests substitute an oracle-backed stand-in to exercise the
index arithmetic and the collectives with gloo.
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


def ep_layer(ops, layer, X, logits, world: int, rank: int, E: int, k: int, path: int, group=None):
    """One expert-parallel layer step for this rank's T tokens.  Returns out [T,D] f32.
    Launch-only (no host synchronisation), so a whole stack of these can be captured in one CUDA graph."""
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
    recv_y = torch.empty_like(back)
    dist.all_to_all_single(recv_y, back, group=group)
    stride = logits.shape[1]
    shg = logits[:, E:] if stride > E else None
    return ops.combine(recv_y, ypos, wt, Y[R:], shg, stride, D, k, T)


def _pad_index(llist: torch.Tensor, R: int) -> torch.Tensor:
    """dispatch() returns the packed list of resident entries followed by unwritten slots (-1)."""
    if llist.numel() == R:
        return llist
    out = torch.full((R,), -1, dtype=torch.int32, device=llist.device)
    out[:llist.numel()] = llist
    return out


class NativeEP:
    """The C entry point q36_moe_ep_layer: the whole step (kernels and NCCL send/recv) is issued from native
    code on the current stream; torch.distributed only carries the 128-byte NCCL id at set-up."""
    # front, quantise, pack, eids, dispatch x3, unpack, plan, gate/up, down, gather, combine (+2 exchanges);
    # gate/up and down are one launch when no expert can receive more than 16 rows (world * T <= 16)
    launches_per_layer = 14

    def __init__(self, layers, world: int, rank: int, T: int):
        import ctypes as C
        from . import moe
        self.moe, self.layers, self.world, self.rank, self.T = moe, layers, world, rank, T
        # decode sizes: front cluster (route, dispatch, quantise), pack, sort + plan of the received slots, unpack,
        # FFN (one launch when no expert can receive more than 16 rows, else two), gather, combine
        small = T <= 16 and world * T * layers[0].k <= 1024
        one_launch = world * T * layers[0].k + T <= 6300   # the library's switch to the two grouped-GEMM launches
        self.launches_per_layer = (6 if one_launch else 8) if small else 14   # (one launch: no gather either)
        dev = layers[0].device
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
        ly = layers[0]
        n = int(moe.lib.q36_moe_ep_workspace_bytes(T, world, ly.E, ly.k, ly.D, ly.FF))
        self.ws = torch.empty(n, dtype=torch.uint8, device=dev)
        moe.check(moe.lib.q36_moe_ws_reset(self.ws.data_ptr(), moe.stream_ptr()), "ws_reset")

    def layer(self, ly, X, logits, out):
        m = self.moe
        stride = logits.shape[1]
        m.check(m.lib.q36_moe_ep_layer(self.comm, ly.Wg.data_ptr(), ly.Wu.data_ptr(), ly.Wd.data_ptr(), m.ptr(ly.Sg),
                                       m.ptr(ly.Su), m.ptr(ly.Sd), ly.E, ly.k, ly.D, ly.FF, X.data_ptr(),
                                       int(X.dtype == torch.bfloat16), logits.data_ptr(), stride,
                                       ly.E if stride > ly.E else -1, 1.0, out.data_ptr(), X.shape[0], self.ws.data_ptr(),
                                       self.ws.numel(), m.stream_ptr()), "ep_layer")
        return out

    def step(self, Xs, Ls, outs):
        for l, ly in enumerate(self.layers):
            self.layer(ly, Xs[l], Ls[l], outs[l])

    def check_device_status(self):
        self.moe.check(self.moe.lib.q36_moe_ws_status(self.ws.data_ptr(), self.moe.stream_ptr()), "device status")

    def close(self):
        if self.comm:
            self.moe.lib.q36_moe_ep_destroy(self.comm)
            self.comm = None


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
