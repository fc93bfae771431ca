"""Expert-parallel step on CPU: two gloo ranks run q36_b200.ep.ep_layer with an oracle-backed stand-in for the
device kernels, so the index arithmetic of the fixed-capacity exchange, the all-to-alls and the combine are
exercised without a GPU.  The result must equal the single-process oracle layer."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from q36_b200 import ep, synth

D, FF, E, K = 256, 128, 8, 2
T = 5


def _to_hw(a):
    s = a.shape
    b = a.reshape(s[:-1] + (s[-1] // 32, 32))
    out = np.empty_like(b)
    out[..., 0::2] = b[..., :16]
    out[..., 1::2] = b[..., 16:]
    return out.reshape(s)


def _from_hw(a):
    s = a.shape
    b = a.reshape(s[:-1] + (s[-1] // 32, 32))
    out = np.empty_like(b)
    out[..., :16] = b[..., 0::2]
    out[..., 16:] = b[..., 1::2]
    return out.reshape(s)


class OracleOps:
    """Same interface as ep.DeviceOps, computed by the CPU oracle (test stand-in, not a product path)."""

    def __init__(self, O, w):
        self.O, self.w = O, w

    def router_topk(self, logits, n_expert, k):
        idx, wt = self.O.router_topk(logits.numpy(), k, n_expert=n_expert)
        return torch.from_numpy(idx), torch.from_numpy(wt)

    def dispatch(self, eid, n_expert, se0=0, se1=None):
        se1 = n_expert if se1 is None else se1
        e = eid.numpy().astype(np.int64)
        keep = (e >= se0) & (e < se1)
        ids = np.nonzero(keep)[0]
        order = ids[np.argsort(e[ids], kind="stable")]
        cnt = np.bincount(e[keep], minlength=n_expert).astype(np.int32)
        eoffs = np.concatenate([[0], np.cumsum(cnt)]).astype(np.int32)
        elist = np.full(e.size, -1, np.int32)
        elist[:order.size] = order
        pos = np.full(e.size, -1, np.int32)
        pos[order] = np.arange(order.size)
        return torch.from_numpy(cnt), torch.from_numpy(eoffs), torch.from_numpy(elist), torch.from_numpy(pos)

    def quant_rows(self, X):
        xq, xs = self.O.quant_e4m3(X.float().numpy())
        return torch.from_numpy(_to_hw(xq)), torch.from_numpy(xs)

    def gather_rows(self, src, index):
        i = index.long()
        out = src[i.clamp(min=0)].clone()
        out[i < 0] = 0
        return out

    def ffn(self, layer, goffs, Xq, Xs, soffs, path):
        O, w = self.O, self.w
        g = goffs.numpy()
        xd = O.dequant_e4m3(_from_hw(Xq.numpy()), Xs.numpy())
        Y = np.zeros((Xq.shape[0], D), np.float32)
        for j in range(layer.se1 - layer.se0):
            e = layer.se0 + j
            for r in range(g[j], g[j + 1]):
                Y[r] = O.expert_ffn(w["gate"][e], w["up"][e], w["down"][e], D, FF, xd[r])[0]
        s0, s1 = soffs.tolist()
        for r in range(s0, s1):
            Y[r] = O.expert_ffn(w["sgate"][0], w["sup"][0], w["sdown"][0], D, FF, xd[r])[0]
        return torch.from_numpy(Y)

    def combine(self, Y, ypos, wt, SH, shgate, stride, Dm, k, Tn):
        Yn, p, wn = Y.numpy().astype(np.float64), ypos.numpy().reshape(Tn, k), wt.numpy().astype(np.float64)
        out = np.zeros((Tn, Dm))
        for t in range(Tn):
            for s in range(k):
                if p[t, s] >= 0:
                    out[t] += wn[t, s] * Yn[p[t, s]]
            gate = 1.0 / (1.0 + np.exp(-float(shgate[t, 0]))) if shgate is not None else 1.0
            out[t] += gate * SH[t].numpy()
        return torch.from_numpy(out)


class _Shard:
    def __init__(self, se0, se1):
        self.se0, self.se1, self.E, self.k, self.D, self.FF = se0, se1, E, K, D, FF
        self.Wg = self.Wu = self.Wd = self.Sg = self.Su = self.Sd = None


def _worker(rank, world, port, q, reduced=False):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from oracle import oracle as O
    w = synth.layer(seed=5, n_expert=E, D=D, FF=FF)
    rng = np.random.default_rng(100 + rank)
    X = synth.activations(rng, T, D)
    L = synth.router_logits(rng, T, E)
    per = E // world
    out = ep.ep_layer(OracleOps(O, w), _Shard(rank * per, (rank + 1) * per), torch.from_numpy(X), torch.from_numpy(L),
                      world, rank, E, K, path=0, reduced=reduced)
    idx, wt = O.router_topk(L, K, n_expert=E)
    want = O.moe_layer(w["gate"], w["up"], w["down"], w["sgate"][0], w["sup"][0], w["sdown"][0], D, FF, X, idx, wt, L[:, E])
    err = float(np.linalg.norm(out.numpy() - want) / np.linalg.norm(want))
    q.put((rank, err))
    dist.destroy_process_group()


def test_slot_maps_roundtrip():
    """Every entry is sent in exactly one slot of its owner's block and comes back where ypos says."""
    rng = np.random.default_rng(0)
    world, k, Tn, En = 4, 3, 7, 16
    idx = torch.from_numpy(np.stack([rng.choice(En, size=k, replace=False) for _ in range(Tn)]).astype(np.int32))
    ops = OracleOps(None, None)
    cnt, eoffs, elist, pos = ops.dispatch(idx.reshape(-1), En)
    C = Tn * k
    tok, eid, ypos = ep.slot_maps(idx, eoffs, elist, pos, world, En, k, C)
    flat = idx.reshape(-1)
    for i in range(Tn * k):
        s = int(ypos[i])
        assert s // C == int(flat[i]) // (En // world)          # the slot lies in the owner's block
        assert int(tok[s]) == i // k and int(eid[s]) == int(flat[i])
    assert int((tok >= 0).sum()) == Tn * k                        # and nothing else is marked valid
    assert torch.equal(tok >= 0, eid >= 0)


@pytest.mark.timeout(300)
@pytest.mark.parametrize("reduced", [False, True])      # one row back per (token, expert) | per (token, expert rank)
def test_ep_layer_two_ranks_gloo(oracle, reduced):
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q, reduced)) for r in range(2)]
    for p in procs:
        p.start()
    res = [q.get(timeout=240) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, err in res:
        assert err < 1e-6, f"rank {rank}: rel-L2 {err}"
