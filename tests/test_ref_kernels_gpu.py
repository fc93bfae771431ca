"""The reference's OWN device kernels (q36_ops.cuh, compiled for sm_100a into oracle/_ref/libq36ref_gpu.so by
oracle/Makefile) run on the same GPU beside the library's and the oracle's restatement: this pins the router,
SwiGLU, RMSNorm, router matvec and the MXFP4 dot product to the reference itself, not only to a restatement of
its source.  Skipped when that file was never built (the reference tree was absent at build time)."""
import numpy as np
import pytest

from q36_b200 import synth

pytestmark = pytest.mark.gpu

D, FF, E, K8 = synth.D_MODEL, synth.EXPERT_FF, synth.N_EXPERT, synth.N_USED


@pytest.fixture(scope="module")
def G(oracle):
    g = oracle.ref_gpu()
    if g is None:
        pytest.skip("oracle/_ref/libq36ref_gpu.so not built")
    return g


@pytest.mark.parametrize("T,zipf,stride", [(1, False, 257), (8, False, 257), (64, True, 256), (257, True, 257)])
def test_router_against_the_reference_kernel(moe, oracle, G, T, zipf, stride):
    """k_router_topk (q36_ops.cuh:397-431) on the B200: indices bit-exact (library == reference == oracle), ties
    included; weights within the error of the reference's fast-math __expf."""
    import torch
    rng = np.random.default_rng(800 + T)
    L = synth.router_logits(rng, T, E, zipf=zipf, with_shared_gate=(stride == 257))
    if T > 4:
        L[3, 17] = L[3, 170] = L[3, :E].max() + 1      # an exact tie: the lower expert id wins
        L[4, :E] = 0.0                                   # all equal: experts 0..7 in order
    lt = torch.from_numpy(L).cuda()
    idx, wt = moe.router_topk(lt, E, K8)
    ridx = torch.empty_like(idx)
    rwt = torch.empty_like(wt)
    torch.cuda.synchronize()
    assert G.ref_gpu_router_topk(lt.data_ptr(), E, K8, ridx.data_ptr(), rwt.data_ptr(), 1.0, 1, T, stride) == 0
    np.testing.assert_array_equal(idx.cpu().numpy(), ridx.cpu().numpy())
    np.testing.assert_allclose(wt.cpu().numpy(), rwt.cpu().numpy(), rtol=1e-5)
    widx, wwt = oracle.router_topk(L, K8, n_expert=E)
    np.testing.assert_array_equal(ridx.cpu().numpy(), widx)
    np.testing.assert_allclose(rwt.cpu().numpy(), wwt, rtol=1e-5)
    # without renormalisation and with a scale
    idx2, wt2 = moe.router_topk(lt, E, K8, scale=2.5, renorm=False)
    torch.cuda.synchronize()
    assert G.ref_gpu_router_topk(lt.data_ptr(), E, K8, ridx.data_ptr(), rwt.data_ptr(), 2.5, 0, T, stride) == 0
    np.testing.assert_array_equal(idx2.cpu().numpy(), ridx.cpu().numpy())
    np.testing.assert_allclose(wt2.cpu().numpy(), rwt.cpu().numpy(), rtol=1e-5)


def test_swiglu_against_the_reference_kernel(oracle, G):
    """k_silu_mul (q36_ops.cuh:58,65) vs the oracle's SwiGLU in float64: the reference's own fast-math result sits
    within 2e-6 relative of it, which bounds what the library's epilogue (same formula, same intrinsics) may differ."""
    import torch
    rng = np.random.default_rng(3)
    g = (rng.standard_normal(1 << 16) * 4).astype(np.float32)
    u = rng.standard_normal(1 << 16).astype(np.float32)
    gt, ut = torch.from_numpy(g.copy()).cuda(), torch.from_numpy(u).cuda()
    torch.cuda.synchronize()
    assert G.ref_gpu_silu_mul(gt.data_ptr(), ut.data_ptr(), g.size) == 0
    g64 = g.astype(np.float64)
    want = g64 / (1.0 + np.exp(-g64)) * u
    np.testing.assert_allclose(gt.cpu().numpy(), want, rtol=2e-6, atol=1e-7)


def test_norm_and_router_matvec_against_the_reference_kernels(moe, oracle, G):
    """k_rmsnorm (q36_ops.cuh:69-79) + k_matvec_f32_row (:331-342), the engine's decode pair in front of the
    layer, vs q36_moe_pre_norm_router on the same row."""
    import torch
    rng = np.random.default_rng(4)
    h = (rng.standard_normal((1, D)) * 3).astype(np.float32)
    w = (1 + 0.1 * rng.standard_normal(D)).astype(np.float32)
    router = (rng.standard_normal((E + 1, D)) * 0.05).astype(np.float32)
    ht, wt_, rt = torch.from_numpy(h).cuda(), torch.from_numpy(w).cuda(), torch.from_numpy(router).cuda()
    x, logits = moe.pre_norm_router(ht, None, wt_, rt, 1e-6, gate_row=E)
    rx = torch.empty(D, dtype=torch.float32, device="cuda")
    rl = torch.empty(E + 1, dtype=torch.float32, device="cuda")
    torch.cuda.synchronize()
    assert G.ref_gpu_rmsnorm(ht.data_ptr(), wt_.data_ptr(), rx.data_ptr(), D, 1e-6) == 0
    assert G.ref_gpu_matvec_f32_row(rt.data_ptr(), rx.data_ptr(), rl.data_ptr(), E + 1, D) == 0
    np.testing.assert_allclose(x.cpu().numpy()[0], rx.cpu().numpy(), rtol=2e-6, atol=1e-7)
    np.testing.assert_allclose(logits.cpu().numpy()[0], rl.cpu().numpy(), rtol=0, atol=2e-5 * float(rl.abs().max()))


def test_mxfp4_dot_against_the_reference_and_the_dequantiser(moe, oracle, G):
    """dot_mxfp4_split (q36_ops.cuh:146-187), the reference's in-register MXFP4 decode + f32 FMA, against a float64
    product over the bit-exact dequantised weights: the decode the GEMV and tensor-core paths replace."""
    import torch
    rng = np.random.default_rng(6)
    M, K, T = 64, D, 3
    b = synth.mxfp4_blocks(rng, 1, M, K)
    W = moe.upload_mxfp4(b, K, M, 0, 1)
    x = synth.activations(rng, T, K)
    xt = torch.from_numpy(x).cuda()
    y = torch.empty((T, M), dtype=torch.float32, device="cuda")
    torch.cuda.synchronize()
    assert G.ref_gpu_dot_mxfp4_split(W.data_ptr(), xt.data_ptr(), y.data_ptr(), M, K, T) == 0
    Wd = oracle.deq_matrix(b[0], M, K).astype(np.float64)
    want = x.astype(np.float64) @ Wd.T
    got = y.cpu().numpy()
    assert np.linalg.norm(got - want) / np.linalg.norm(want) < 1e-6
    # and the library's on-device dequantiser gives exactly those weights
    np.testing.assert_array_equal(moe.dequant_mxfp4(W, M, K).cpu().numpy(), oracle.deq_matrix(b[0], M, K))
