"""The steps either side of the expert computation (residual add + RMSNorm + router logits in front; combine +
residual add + next RMSNorm behind) and the whole block from the residual stream, against the CPU oracle."""
import numpy as np
import pytest

from q36_b200 import synth

pytestmark = pytest.mark.gpu

D, FF, E, K8 = synth.D_MODEL, synth.EXPERT_FF, synth.N_EXPERT, synth.N_USED
EPS = 1e-6    # Q36_RMS_EPS (q36.h)


def rel_l2(a, b):
    a, b = np.asarray(a, np.float64), np.asarray(b, np.float64)
    return float(np.linalg.norm(a - b) / max(np.linalg.norm(b), 1e-300))


@pytest.fixture(scope="module")
def weights():
    return synth.layer(seed=0)


@pytest.fixture(scope="module")
def layer(moe, weights):
    w = weights
    return moe.MoELayer().load_gguf_blocks(w["gate"], w["up"], w["down"], w["sgate"], w["sup"], w["sdown"])


def _stream_inputs(rng, T):
    h = (rng.standard_normal((T, D), dtype=np.float32) * 3.0)
    a = rng.standard_normal((T, D), dtype=np.float32)
    w_post = (1.0 + 0.1 * rng.standard_normal(D, dtype=np.float32))
    w_next = (1.0 + 0.1 * rng.standard_normal(D, dtype=np.float32))
    router = rng.standard_normal((E + 1, D), dtype=np.float32) * 0.05
    return h, a, w_post, w_next, router


@pytest.mark.parametrize("T,with_add", [(1, True), (8, True), (16, False), (100, True), (300, False)])
def test_step_before_vs_oracle(moe, oracle, T, with_add):
    """h += a, x = rmsnorm(h) * w, logits = router . x: the decode-sized kernel (T <= 16, one warp per router row)
    and the batched one (tiled f32 GEMM + the gate row inside the norm kernel), ragged T and 257 rows included."""
    import torch
    rng = np.random.default_rng(700 + T)
    h, a, w_post, _, router = _stream_inputs(rng, T)
    ht = torch.from_numpy(h.copy()).cuda()
    at = torch.from_numpy(a).cuda() if with_add else None
    x, logits = moe.pre_norm_router(ht, at, torch.from_numpy(w_post).cuda(), torch.from_numpy(router).cuda(), EPS, gate_row=E)
    torch.cuda.synchronize()
    hn, xw = oracle.add_rmsnorm(h, a if with_add else None, w_post, EPS)
    np.testing.assert_array_equal(ht.cpu().numpy(), hn)                       # the f32 add is exact either way
    np.testing.assert_allclose(x.cpu().numpy(), xw, rtol=2e-6, atol=1e-7)
    lw = oracle.router_logits(x.cpu().numpy(), router)                        # the dot products of the GPU's own x
    np.testing.assert_allclose(logits.cpu().numpy(), lw, rtol=0, atol=2e-5 * np.abs(lw).max())


@pytest.mark.parametrize("T", [1, 8, 40, 300])
def test_step_after_vs_oracle(moe, oracle, T):
    """combine + residual add + next RMSNorm in one launch == q36_moe_combine followed by the oracle's add + norm."""
    import torch
    rng = np.random.default_rng(720 + T)
    n = T * K8
    Y = rng.standard_normal((n + T, D), dtype=np.float32)
    pos = rng.permutation(n).astype(np.int32)
    pos[rng.integers(0, n, size=max(1, n // 10))] = -1                          # non-resident entries contribute nothing
    wt = rng.random((T, K8), dtype=np.float32)
    shg = rng.standard_normal((T, 3), dtype=np.float32)                         # a strided gate column
    h, _, _, w_next, _ = _stream_inputs(rng, T)
    Yt, pt, wtt = torch.from_numpy(Y).cuda(), torch.from_numpy(pos).cuda(), torch.from_numpy(wt).cuda()
    sgt = torch.from_numpy(shg).cuda()
    ref_moe = moe.combine(Yt[:n], pt, wtt, Yt[n:], sgt[:, 1:], 3, D, K8, T)
    ht = torch.from_numpy(h.copy()).cuda()
    got_moe, x_next = moe.combine_add_rmsnorm(Yt[:n], pt, wtt, Yt[n:], sgt[:, 1:], 3, ht, torch.from_numpy(w_next).cuda(),
                                              EPS, D, K8, T)
    torch.cuda.synchronize()
    assert torch.equal(got_moe, ref_moe)                                        # same sum, same order
    hn, xw = oracle.add_rmsnorm(h, ref_moe.cpu().numpy(), w_next, EPS)
    np.testing.assert_array_equal(ht.cpu().numpy(), hn)
    np.testing.assert_allclose(x_next.cpu().numpy(), xw, rtol=2e-6, atol=1e-7)


@pytest.mark.parametrize("T", [4, 8, 150])
def test_block_from_the_residual_stream(moe, oracle, layer, weights, T):
    """q36_moe_block == the three pieces chained through the public entries (bit for bit), and the whole thing
    against the oracle: routing indices bit-exact on the block's own logits, layer output within 1e-2."""
    import torch
    rng = np.random.default_rng(740 + T)
    h, a, w_post, w_next, router = _stream_inputs(rng, T)
    cu = lambda v: torch.from_numpy(v).cuda()
    ht = cu(h.copy())
    x_next, moe_out = layer.block(ht, cu(a), cu(w_post), cu(router), cu(w_next), EPS)
    torch.cuda.synchronize()
    layer.check_device_status()
    # the same chain by hand
    h2 = cu(h.copy())
    x, logits = moe.pre_norm_router(h2, cu(a), cu(w_post), cu(router), EPS, gate_row=E)
    out, idx, wt = layer.forward(x, logits, path=moe.PATH_AUTO, want_routing=True)
    assert torch.equal(out, moe_out)
    hn, xw = oracle.add_rmsnorm(h2.cpu().numpy(), out.cpu().numpy(), w_next, EPS)
    np.testing.assert_array_equal(ht.cpu().numpy(), hn)
    np.testing.assert_allclose(x_next.cpu().numpy(), xw, rtol=2e-6, atol=1e-7)
    # against the oracle from the GPU's logits on
    L = logits.cpu().numpy()
    widx, wwt = oracle.router_topk(L, K8, n_expert=E)
    np.testing.assert_array_equal(idx.cpu().numpy(), widx)
    toks = rng.choice(T, size=min(T, 6), replace=False)
    w = weights
    want = oracle.moe_layer(w["gate"], w["up"], w["down"], w["sgate"][0], w["sup"][0], w["sdown"][0], D, FF,
                            x.cpu().numpy(), widx, wwt, L[:, E], tokens=toks)
    assert rel_l2(moe_out.cpu().numpy()[toks], want) < 1e-2
