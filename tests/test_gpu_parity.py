"""GPU parity tests: every stage of the CUDA path against the CPU oracle, through the C ABI.

Bit-exact: dequantised weights, quantised activations, routing indices, dispatch.
Outputs: within 1e-2 relative L2 of the float64 oracle (the tolerance of the
benchmark specification); the per-stage check that feeds the GPU's own quantised
intermediate to the oracle is held to 1e-4.
"""
import numpy as np
import pytest

from q36_b200 import synth

pytestmark = pytest.mark.gpu

D, FF, E, K8 = synth.D_MODEL, synth.EXPERT_FF, synth.N_EXPERT, synth.N_USED
TOL = 1e-2        # relative L2, end to end
TOL_STAGE = 1e-4  # relative L2, stage-wise (same quantised inputs on both sides)


def rel_l2(a, b):
    a = np.asarray(a, np.float64)
    b = np.asarray(b, np.float64)
    return float(np.linalg.norm(a - b) / max(np.linalg.norm(b), 1e-300))


def to_hw(a):
    """logical -> hw order inside every 32-block of the last axis"""
    s = a.shape
    b = a.reshape(s[:-1] + (s[-1] // 32, 32))
    out = np.empty_like(b)
    out[..., 0::2] = b[..., :16]
    out[..., 1::2] = b[..., 16:]
    return out.reshape(s)


def from_hw(a):
    s = a.shape
    b = a.reshape(s[:-1] + (s[-1] // 32, 32))
    out = np.empty_like(b)
    out[..., :16] = b[..., 0::2]
    out[..., 16:] = b[..., 1::2]
    return out.reshape(s)


@pytest.fixture(scope="module")
def torch_cuda():
    import torch
    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    return torch


@pytest.fixture(scope="module")
def weights():
    return synth.layer(seed=0)      # 256 + 1 experts as GGUF blocks


@pytest.fixture(scope="module")
def layer(moe, torch_cuda, weights):
    w = weights
    return moe.MoELayer().load_gguf_blocks(w["gate"], w["up"], w["down"], w["sgate"], w["sup"], w["sdown"])


def test_dequant_bit_exact(moe, oracle, torch_cuda, weights):
    """Device dequantisation of the split planes == reference dequantiser, bit for bit."""
    rng = np.random.default_rng(0)
    b = synth.mxfp4_blocks(rng, 1, 128, 512)
    b[0, :, :, 0] = rng.integers(0, 255, size=(128, 16), dtype=np.uint8)   # every scale byte but 255
    W = moe.upload_mxfp4(b, 512, 128, 0, 1)
    got = moe.dequant_mxfp4(W, 128, 512).cpu().numpy()
    want = oracle.deq_matrix(b[0], 128, 512, use_ref=oracle.ref() is not None)
    np.testing.assert_array_equal(got.view(np.uint32), want.view(np.uint32))
    # and one real-shaped gate matrix of the benchmark layer
    Wg = moe.upload_mxfp4(weights["gate"], D, FF, 3, 4)
    got = moe.dequant_mxfp4(Wg, FF, D).cpu().numpy()
    np.testing.assert_array_equal(got.view(np.uint32), oracle.deq_matrix(weights["gate"][3], FF, D).view(np.uint32))


@pytest.mark.parametrize("T", [1, 3, 64])
@pytest.mark.parametrize("bf16", [False, True])
def test_quant_bit_exact(moe, oracle, torch_cuda, T, bf16):
    torch = torch_cuda
    rng = np.random.default_rng(T)
    X = synth.activations(rng, T, D)
    X[0, :32] = 0.0
    X[0, 32:64] *= 1e-30
    X[0, 64:96] *= 1e30
    X[0, 96] = 448.0
    xt = torch.from_numpy(X).cuda()
    if bf16:
        xt = xt.to(torch.bfloat16)
        X = xt.float().cpu().numpy()
    Xq, Xs = moe.quant_e4m3(xt)
    wq, ws = oracle.quant_e4m3(X)
    np.testing.assert_array_equal(Xs.cpu().numpy(), ws)
    np.testing.assert_array_equal(Xq.cpu().numpy(), wq)


@pytest.mark.parametrize("T,zipf", [(1, False), (8, False), (257, True)])
def test_router_indices_bit_exact(moe, oracle, torch_cuda, T, zipf):
    torch = torch_cuda
    rng = np.random.default_rng(100 + T)
    L = synth.router_logits(rng, T, E, zipf=zipf)
    if T > 4:
        L[3, 17] = L[3, 170] = L[3].max() + 1      # tie
    idx, wt = moe.router_topk(torch.from_numpy(L).cuda(), E, K8)
    widx, wwt = oracle.router_topk(L, K8, n_expert=E)
    np.testing.assert_array_equal(idx.cpu().numpy(), widx)
    np.testing.assert_allclose(wt.cpu().numpy(), wwt, rtol=1e-5)


@pytest.mark.parametrize("n,se", [(8, (0, 256)), (1000, (0, 256)), (5000, (64, 128)), (40000, (0, 256))])
def test_dispatch_bit_exact(moe, oracle, torch_cuda, n, se):
    torch = torch_cuda
    rng = np.random.default_rng(n)
    p = 1.0 / np.arange(1, E + 1) ** 1.1
    eid = rng.choice(E, size=n, p=p / p.sum()).astype(np.int32)
    ec, eo, el, pos = moe.dispatch(torch.from_numpy(eid).cuda(), E, se[0], se[1])
    keep = (eid >= se[0]) & (eid < se[1])
    ids = np.nonzero(keep)[0]
    order = ids[np.argsort(eid[ids], kind="stable")]
    nres = order.size
    np.testing.assert_array_equal(el.cpu().numpy()[:nres], order)
    want_cnt = np.bincount(eid[keep], minlength=E)
    np.testing.assert_array_equal(ec.cpu().numpy(), want_cnt)
    np.testing.assert_array_equal(eo.cpu().numpy(), np.concatenate([[0], np.cumsum(want_cnt)]))
    wpos = np.full(n, -1, np.int32)
    wpos[order] = np.arange(nres)
    np.testing.assert_array_equal(pos.cpu().numpy(), wpos)


def _sorted_inputs(moe, oracle, torch, T, rng, zipf=False):
    X = synth.activations(rng, T, D)
    L = synth.router_logits(rng, T, E, zipf=zipf)
    xt, lt = torch.from_numpy(X).cuda(), torch.from_numpy(L).cuda()
    idx, wt = moe.router_topk(lt, E, K8)
    ec, eo, el, pos = moe.dispatch(idx.reshape(-1), E)
    R = T * (K8 + 1)
    Xq, Xs = moe.quant_scatter(xt, pos, K8, T * K8, R)
    return X, L, xt, lt, idx, wt, eo, el, pos, Xq, Xs


def test_quant_scatter_rows(moe, oracle, torch_cuda):
    """Every sorted row holds its token's quantised activation, in hw order."""
    torch = torch_cuda
    T = 5
    X, L, xt, lt, idx, wt, eo, el, pos, Xq, Xs = _sorted_inputs(moe, oracle, torch, T, np.random.default_rng(9))
    wq, ws = oracle.quant_e4m3(X)
    tok = np.concatenate([el.cpu().numpy() // K8, np.arange(T)])
    np.testing.assert_array_equal(from_hw(Xq.cpu().numpy()), wq[tok])
    np.testing.assert_array_equal(Xs.cpu().numpy(), ws[tok])


def _check_ffn(moe, oracle, torch, layer, weights, T, path, rng, zipf=False, sample=24):
    """Grouped FFN (routed groups) against the oracle, stage by stage."""
    X, L, xt, lt, idx, wt, eo, el, pos, Xq, Xs = _sorted_inputs(moe, oracle, torch, T, rng, zipf)
    n = T * K8
    Hq, Hs, Y = moe.expert_ffn_sorted(layer.Wg, layer.Wu, layer.Wd, E, eo, Xq[:n], Xs[:n], D, FF, path)
    Hq, Hs, Y = from_hw(Hq.cpu().numpy()), Hs.cpu().numpy(), Y.cpu().numpy()
    eln, idxn = el.cpu().numpy(), idx.cpu().numpy().reshape(-1)
    xq, xs = oracle.quant_e4m3(X)
    xd = oracle.dequant_e4m3(xq, xs)
    rows = rng.choice(n, size=min(sample, n), replace=False)
    worst_e2e = worst_stage = 0.0
    flips = total = 0
    for r in rows:
        entry = eln[r]
        t, e = entry // K8, idxn[entry]
        y, h, hq, hs = oracle.expert_ffn(weights["gate"][e], weights["up"][e], weights["down"][e], D, FF, xd[t])
        worst_e2e = max(worst_e2e, rel_l2(Y[r], y))
        # the GPU's own quantised intermediate must be what the quantiser gives for a
        # SwiGLU output within fp32 rounding of the oracle's: compare dequantised values
        hd_gpu = oracle.dequant_e4m3(Hq[r][None], Hs[r][None])[0]
        hd_orc = oracle.dequant_e4m3(hq[None], hs[None])[0]
        flips += int((hd_gpu != hd_orc).sum())
        total += FF
        assert rel_l2(hd_gpu, h) < 0.05
        y2, *_ = oracle.expert_ffn(weights["gate"][e], weights["up"][e], weights["down"][e], D, FF, xd[t],
                                   hq_in=Hq[r], hs_in=Hs[r])
        worst_stage = max(worst_stage, rel_l2(Y[r], y2))
    assert worst_stage < TOL_STAGE, f"down stage rel-L2 {worst_stage}"
    assert worst_e2e < TOL, f"end-to-end rel-L2 {worst_e2e}"
    assert flips <= max(2, total // 200), f"{flips}/{total} intermediate codes differ from the oracle"


@pytest.mark.parametrize("T", [1, 2, 7])
def test_ffn_gemv_vs_oracle(moe, oracle, torch_cuda, layer, weights, T):
    _check_ffn(moe, oracle, torch_cuda, layer, weights, T, moe.PATH_GEMV, np.random.default_rng(20 + T))


def _check_layer(moe, oracle, torch, layer, weights, T, path, rng, zipf=False, sample=6, bf16=True, spread=False, **kw):
    X = synth.activations(rng, T, D)
    L = synth.router_logits(rng, T, E, zipf=zipf)
    xt = torch.from_numpy(X).cuda()
    if bf16:
        xt = xt.to(torch.bfloat16)          # exact: the activations are bf16 values
    out, idx, wt = layer.forward(xt, torch.from_numpy(L).cuda(), path=path, want_routing=True, **kw)
    torch.cuda.synchronize()
    if path != moe.PATH_GEMV:
        layer.check_device_status()
    out, idx, wt = out.cpu().numpy(), idx.cpu().numpy(), wt.cpu().numpy()
    widx, wwt = oracle.router_topk(L, K8, n_expert=E)
    np.testing.assert_array_equal(idx, widx)
    toks = rng.choice(T, size=min(sample, T), replace=False)
    if spread and T > sample:
        # half of the sample from the tokens whose rarest chosen expert is rarest overall (the tail of a skewed load:
        # groups of a few rows), half at random (mostly the head: groups of thousands of rows)
        load = np.bincount(widx.reshape(-1), minlength=E)
        rare = np.argsort(load[widx].min(axis=1), kind="stable")[:sample // 2]
        toks = np.unique(np.concatenate([rare, toks[:sample - rare.size]]))
    w = weights
    want = oracle.moe_layer(w["gate"], w["up"], w["down"], w["sgate"][0], w["sup"][0], w["sdown"][0], D, FF, X, widx,
                            wwt, L[:, E], tokens=toks, se0=layer.se0, se1=layer.se1,
                            inc_shared=kw.get("inc_shared", True))
    assert np.isfinite(out).all()
    err = rel_l2(out[toks], want)
    assert err < TOL, f"layer rel-L2 {err}"
    return out


@pytest.mark.parametrize("T", [5, 16, 40])
def test_decode_layer_collisions_zero_rows_and_ties(moe, oracle, torch_cuda, layer, weights, T):
    """Edge cases of the decode path: every token routes to the SAME eight experts (groups of T rows: one full
    16-row token tile at T = 16, three token tiles at T = 40), some activation rows are all zero (block amax 0 ->
    the smallest exponent), and the logits hold exact ties (lower expert id wins)."""
    torch = torch_cuda
    rng = np.random.default_rng(300 + T)
    X = synth.activations(rng, T, D)
    X[0] = 0.0
    X[T - 1, 32:96] = 0.0                              # two whole 32-blocks of an otherwise normal row
    row = synth.router_logits(rng, 1, E)[0]
    row[[3, 40, 41, 200]] = row.max() + 1.0            # a four-way tie at the top, the rest distinct
    L = np.tile(row, (T, 1)).astype(np.float32)
    xt, lt = torch.from_numpy(X).cuda().to(torch.bfloat16), torch.from_numpy(L).cuda()
    out, idx, wt = layer.forward(xt, lt, path=moe.PATH_TC, want_routing=True)
    torch.cuda.synchronize()
    layer.check_device_status()
    widx, wwt = oracle.router_topk(L, K8, n_expert=E)
    np.testing.assert_array_equal(idx.cpu().numpy(), widx)
    assert list(widx[0][:4]) == [3, 40, 41, 200]
    w = weights
    want = oracle.moe_layer(w["gate"], w["up"], w["down"], w["sgate"][0], w["sup"][0], w["sdown"][0], D, FF, X, widx,
                            wwt, L[:, E], tokens=np.arange(T), se0=layer.se0, se1=layer.se1, inc_shared=True)
    got = out.cpu().numpy()
    assert np.isfinite(got).all()
    assert np.abs(got[0]).max() == 0.0                 # a zero token stays zero through every stage
    assert rel_l2(got, want) < TOL


@pytest.mark.parametrize("T", [24, 64])
def test_mid_size_layer_vs_oracle(moe, oracle, torch_cuda, layer, weights, T):
    """Token counts between decode and prefill: the one-launch kernel with the shared expert's group (and any
    routed group of more than 16 rows) cut into several 16-row token tiles."""
    _check_layer(moe, oracle, torch_cuda, layer, weights, T, moe.PATH_TC, np.random.default_rng(400 + T), sample=8)


@pytest.mark.parametrize("path", ["gemv", "tc"])
@pytest.mark.parametrize("T", [1, 2, 4, 8, 16])
def test_decode_layer_vs_oracle(moe, oracle, torch_cuda, layer, weights, T, path):
    """Config 1 of the benchmark: T = 1, 2, 4, 8 tokens, 256 + 1 experts, top-8 -- on the streaming GEMV and
    on the fused tcgen05 decode kernel (gate/up + down in one persistent launch)."""
    p = moe.PATH_GEMV if path == "gemv" else moe.PATH_TC
    _check_layer(moe, oracle, torch_cuda, layer, weights, T, p, np.random.default_rng(40 + T))


def test_decode_paths_agree_and_repeat(moe, oracle, torch_cuda, layer, weights):
    """The fused decode kernel hands its intermediate from SM to SM through global memory: run it many times
    on the same input; every run must give the same bits, and the GEMV path must agree closely."""
    torch = torch_cuda
    rng = np.random.default_rng(3)
    T = 8
    xt = torch.from_numpy(synth.activations(rng, T)).cuda().to(torch.bfloat16)
    lt = torch.from_numpy(synth.router_logits(rng, T, E)).cuda()
    ref = layer.forward(xt, lt, path=moe.PATH_TC).clone()
    for _ in range(20):
        out = layer.forward(xt, lt, path=moe.PATH_TC)
        assert torch.equal(out, ref)
    layer.check_device_status()
    g = layer.forward(xt, lt, path=moe.PATH_GEMV)
    assert rel_l2(g.cpu().numpy(), ref.cpu().numpy()) < 2e-3


@pytest.mark.parametrize("T", [1, 8])
def test_decode_entry_by_name(moe, oracle, torch_cuda, layer, weights, T):
    """q36_moe_decode (the drop-in for moe_ffn) takes the fastest path: bit-identical to q36_moe_layer with
    path AUTO, and within tolerance of the oracle."""
    torch = torch_cuda
    rng = np.random.default_rng(900 + T)
    X = synth.activations(rng, T, D)
    L = synth.router_logits(rng, T, E)
    xt, lt = torch.from_numpy(X).cuda().to(torch.bfloat16), torch.from_numpy(L).cuda()
    ref = layer.forward(xt, lt, path=moe.PATH_AUTO).clone()
    got = layer.decode(xt, lt)
    torch.cuda.synchronize()
    layer.check_device_status()
    assert torch.equal(got, ref)
    widx, wwt = oracle.router_topk(L, K8, n_expert=E)
    w = weights
    want = oracle.moe_layer(w["gate"], w["up"], w["down"], w["sgate"][0], w["sup"][0], w["sdown"][0], D, FF, X, widx, wwt,
                            L[:, E], tokens=np.arange(T))
    assert rel_l2(got.cpu().numpy(), want) < TOL


def test_prefill_entry_by_name(moe, oracle, torch_cuda, layer, weights):
    """q36_moe_prefill (the drop-in for pf_moe_block): bit-identical to q36_moe_layer with path AUTO at a
    prefill-sized call, and within tolerance of the oracle on sampled tokens."""
    torch = torch_cuda
    T = 600                                  # 5400 sorted rows: beyond the one-launch kernel's row limit
    rng = np.random.default_rng(901)
    X = synth.activations(rng, T, D)
    L = synth.router_logits(rng, T, E, zipf=True)
    xt, lt = torch.from_numpy(X).cuda().to(torch.bfloat16), torch.from_numpy(L).cuda()
    ref = layer.forward(xt, lt, path=moe.PATH_AUTO).clone()
    got = layer.prefill(xt, lt)
    torch.cuda.synchronize()
    layer.check_device_status()
    assert torch.equal(got, ref)
    widx, wwt = oracle.router_topk(L, K8, n_expert=E)
    toks = rng.choice(T, size=8, replace=False)
    w = weights
    want = oracle.moe_layer(w["gate"], w["up"], w["down"], w["sgate"][0], w["sup"][0], w["sdown"][0], D, FF, X, widx, wwt,
                            L[:, E], tokens=toks)
    assert rel_l2(got.cpu().numpy()[toks], want) < TOL


def test_bounded_wait_gives_up_and_the_status_is_sticky(moe, torch_cuda, layer):
    """A wait that nothing completes must end by itself: the kernel records where it gave up, returns, and the
    host reads Q36_MOE_EDEVICE; the context stays usable.  The record survives later launches on the same
    workspace (they never clear it) until q36_moe_ws_reset."""
    torch = torch_cuda
    rng = np.random.default_rng(5)
    T = 4
    xt = torch.from_numpy(synth.activations(rng, T, D)).cuda().to(torch.bfloat16)
    lt = torch.from_numpy(synth.router_logits(rng, T, E)).cuda()
    ref = layer.forward(xt, lt, path=moe.PATH_TC).clone()
    layer.check_device_status()                                   # clean so far
    ws = layer.workspace(T)
    rc = moe.lib.q36_moe_selftest_wait_timeout(ws.data_ptr(), moe.stream_ptr())
    assert rc == moe.EDEVICE
    assert moe.lib.q36_moe_last_cuda_error() == 200000 + 0xA00    # role 0xA, stage 0: the self-test's waiter
    out = layer.forward(xt, lt, path=moe.PATH_TC)                 # the device still works ...
    torch.cuda.synchronize()
    assert torch.equal(out, ref)
    with pytest.raises(moe.MoEError):                             # ... and the record is still there
        layer.check_device_status()
    layer.reset_device_status()
    layer.check_device_status()


def test_layer_host_buffers_and_f32_input(moe, oracle, torch_cuda, layer, weights):
    torch = torch_cuda
    rng = np.random.default_rng(77)
    T = 4
    X = synth.activations(rng, T, D)
    L = synth.router_logits(rng, T, E)
    ref = layer.forward(torch.from_numpy(X).cuda(), torch.from_numpy(L).cuda(), path=moe.PATH_GEMV).cpu().numpy()
    hx, hl = torch.from_numpy(X).pin_memory(), torch.from_numpy(L).pin_memory()
    ho = torch.empty((T, D), dtype=torch.float32).pin_memory()
    layer.forward_host(hx, hl, ho, path=moe.PATH_GEMV)
    np.testing.assert_array_equal(ho.numpy(), ref)       # same kernels, same order: bit-identical


def test_layer_loaded_from_a_gguf_file(moe, oracle, torch_cuda, weights, tmp_path):
    """On-disk format in: blk.N.ffn_*_exps.weight of a GGUF v3 file -> split planes on the device through the
    library's reader; the layer built that way gives the bits of the layer built from the same blocks in memory,
    on a shard, and the router matrix arrives as the engine's [E + 1][D] concatenation."""
    torch = torch_cuda
    rng = np.random.default_rng(41)
    w = weights
    router = rng.standard_normal((E, D), dtype=np.float32)
    sgate = rng.standard_normal(D, dtype=np.float32)
    path = str(tmp_path / "block7.gguf")
    synth.write_gguf(path, synth.layer_tensors(w, 7, router=router, shared_gate=sgate))
    T = 6
    xt = torch.from_numpy(synth.activations(rng, T, D)).cuda().to(torch.bfloat16)
    lt = torch.from_numpy(synth.router_logits(rng, T, E)).cuda()
    with moe.GgufFile(path) as g:
        assert g.layer_shape(7) == (E, D, FF, (39, 39, 39))
        for se0, se1 in ((0, E), (64, 192)):
            a = moe.MoELayer(se0=se0, se1=se1).load_gguf(g, 7)
            b = moe.MoELayer(se0=se0, se1=se1).load_gguf_blocks(w["gate"], w["up"], w["down"], w["sgate"], w["sup"], w["sdown"])
            for pa, pb in ((a.Wg, b.Wg), (a.Wu, b.Wu), (a.Wd, b.Wd), (a.Sg, b.Sg), (a.Su, b.Su), (a.Sd, b.Sd)):
                assert torch.equal(pa, pb)
            assert torch.equal(a.forward(xt, lt, path=moe.PATH_TC), b.forward(xt, lt, path=moe.PATH_TC))
            a.check_device_status()
        rt = torch.empty((E + 1, D), dtype=torch.float32, device="cuda")
        moe.check(moe.lib.q36_moe_gguf_upload_router(g.h, 7, rt.data_ptr()), "gguf_upload_router")
        np.testing.assert_array_equal(rt.cpu().numpy(), np.concatenate([router, sgate[None]], 0))


def test_shard_contract(moe, oracle, torch_cuda, weights):
    """Experts outside [se0,se1) contribute zeros; shards sum to the whole; only the owner adds the shared expert
    (q36_engine.cu:763-766, 3398-3400, 4245-4248)."""
    torch = torch_cuda
    rng = np.random.default_rng(5)
    T = 4
    X = synth.activations(rng, T, D)
    L = synth.router_logits(rng, T, E)
    xt, lt = torch.from_numpy(X).cuda(), torch.from_numpy(L).cuda()
    w = weights
    full = moe.MoELayer().load_gguf_blocks(w["gate"], w["up"], w["down"], w["sgate"], w["sup"], w["sdown"])
    whole = full.forward(xt, lt, path=moe.PATH_GEMV).cpu().numpy().astype(np.float64)
    acc = np.zeros_like(whole)
    for r in range(4):
        sh = moe.MoELayer(se0=r * 64, se1=(r + 1) * 64).load_gguf_blocks(w["gate"], w["up"], w["down"], w["sgate"],
                                                                         w["sup"], w["sdown"])
        acc += sh.forward(xt, lt, path=moe.PATH_GEMV, inc_shared=(r == 0)).cpu().numpy()
    assert rel_l2(acc, whole) < 1e-5


# ----------------------------------------------------------------- tensor cores
def _selftest_case(moe, oracle, torch, N, K, rng, scale_lo=118, scale_hi=131):
    b = synth.mxfp4_blocks(rng, 1, 128, K)
    b[..., 0] = rng.integers(scale_lo, scale_hi, size=b.shape[:-1], dtype=np.uint8)
    A = moe.upload_mxfp4(b, K, 128, 0, 1)
    Xb = synth.activations(rng, N, K) * np.exp2(rng.integers(-6, 7, size=(N, 1))).astype(np.float32)
    xq, xs = oracle.quant_e4m3(Xb)
    Dg = moe.tc_selftest(A, torch.from_numpy(to_hw(xq)).cuda(), torch.from_numpy(xs).cuda(), N, K).cpu().numpy()
    Wa = oracle.deq_matrix(b[0], 128, K).astype(np.float64)
    want = oracle.dequant_e4m3(xq, xs).astype(np.float64) @ Wa.T
    return Dg, want


@pytest.mark.parametrize("N,K", [(16, 512), (128, 512), (40, 2048), (300, 2048)])
def test_tcgen05_tile_vs_cpu(moe, oracle, torch_cuda, N, K):
    """The role of the reference's test_mma_bs.cu: operand, scale and descriptor mapping of the
    block-scaled MMA proven on silicon against a CPU product (its bound: max rel err < 1e-3)."""
    Dg, want = _selftest_case(moe, oracle, torch_cuda, N, K, np.random.default_rng(N + K))
    assert rel_l2(Dg, want) < 1e-5
    assert np.abs(Dg - want).max() <= 1e-3 * np.abs(want).max()


@pytest.mark.parametrize("T", [16, 100])
def test_ffn_tc_vs_oracle(moe, oracle, torch_cuda, layer, weights, T):
    _check_ffn(moe, oracle, torch_cuda, layer, weights, T, moe.PATH_TC, np.random.default_rng(60 + T))


@pytest.mark.parametrize("T", [3, 16])
def test_ffn_one_launch_matches_two_and_setup_only(moe, oracle, torch_cuda, layer, weights, T):
    """With a bound of at most 16 rows per group the tensor-core call is ONE persistent launch (gate/up and down);
    it must give what the two grouped-GEMM launches give, shared expert's group included.  The f32 sums differ in
    their order (four partial accumulators against one), so a code of the quantised intermediate may sit on the
    other side of a rounding boundary now and then.  stages = 4 alone builds the plan and touches no output."""
    torch = torch_cuda
    X, L, xt, lt, idx, wt, eo, el, pos, Xq, Xs = _sorted_inputs(moe, oracle, torch, T, np.random.default_rng(70 + T))
    n, R = T * K8, T * (K8 + 1)
    soffs = torch.tensor([n, n + T], dtype=torch.int32, device="cuda")
    shared = (layer.Sg, layer.Su, layer.Sd)
    two = moe.expert_ffn_sorted(layer.Wg, layer.Wu, layer.Wd, E, eo, Xq, Xs, D, FF, moe.PATH_TC, shared=shared, soffs=soffs)
    one = moe.expert_ffn_sorted(layer.Wg, layer.Wu, layer.Wd, E, eo, Xq, Xs, D, FF, moe.PATH_TC, shared=shared, soffs=soffs,
                                max_group_rows=T)
    hq1, hq2 = one[0].cpu().numpy(), two[0].cpu().numpy()
    assert (hq1 != hq2).sum() <= max(2, hq1.size // 2000)
    assert (one[1].cpu().numpy() != two[1].cpu().numpy()).sum() <= 2          # Hs
    assert rel_l2(one[2].cpu().numpy(), two[2].cpu().numpy()) < 1e-3
    bufs = tuple(torch.full_like(b, 7) for b in one)
    moe.expert_ffn_sorted(layer.Wg, layer.Wu, layer.Wd, E, eo, Xq, Xs, D, FF, moe.PATH_TC, shared=shared, soffs=soffs,
                          stages=4, bufs=bufs, max_group_rows=T)
    for b in bufs:
        assert bool((b == 7).all())


def test_tc_and_gemv_paths_agree(moe, oracle, torch_cuda, layer, weights):
    torch = torch_cuda
    rng = np.random.default_rng(8)
    T = 24
    X = synth.activations(rng, T, D)
    L = synth.router_logits(rng, T, E)
    xt, lt = torch.from_numpy(X).cuda().to(torch.bfloat16), torch.from_numpy(L).cuda()
    a = layer.forward(xt, lt, path=moe.PATH_GEMV).cpu().numpy()
    b = layer.forward(xt, lt, path=moe.PATH_TC).cpu().numpy()
    layer.check_device_status()
    assert rel_l2(b, a) < 2e-3


def test_prefill_layer_vs_oracle_small(moe, oracle, torch_cuda, layer, weights):
    _check_layer(moe, oracle, torch_cuda, layer, weights, 600, moe.PATH_TC, np.random.default_rng(70), zipf=True)


def test_prefill_layer_full_size_zipf(moe, oracle, torch_cuda, layer, weights):
    """Config 2 of the benchmark at full size (T = 4096, Zipf-skewed routing): sampled tokens against the
    oracle, plus size-independent properties over all tokens."""
    torch = torch_cuda
    rng = np.random.default_rng(71)
    T = 4096
    out = _check_layer(moe, oracle, torch, layer, weights, T, moe.PATH_TC, rng, zipf=True, sample=64, spread=True)
    # permutation invariance: the same tokens in another order give the same rows
    rng = np.random.default_rng(71)
    X = synth.activations(rng, T, D)
    L = synth.router_logits(rng, T, E, zipf=True)
    perm = np.random.default_rng(1).permutation(T)
    out_p = layer.forward(torch.from_numpy(X[perm]).cuda().to(torch.bfloat16), torch.from_numpy(L[perm]).cuda(),
                          path=moe.PATH_TC).cpu().numpy()
    layer.check_device_status()
    np.testing.assert_array_equal(out_p, out[perm])


@pytest.mark.parametrize("switches", [{"Q36_GATEUP_NARROW": "1", "Q36_OLD_DOWN": "1"}, {"Q36_Y_BF16": "1"}])
def test_the_selectable_variants_still_agree_with_the_oracle(switches):
    """k_grouped_mma<2> (gate/up with weights as the 128-row operand) and k_grouped_mma<1> (the generic down kernel),
    and bf16 staging of the result rows between down and combine, sit behind environment switches read once per
    process: run the prefill-sized oracle tests in a child process that selects them."""
    import os
    import subprocess
    import sys
    env = dict(os.environ, **switches)
    here = os.path.dirname(os.path.abspath(__file__))
    r = subprocess.run([sys.executable, "-m", "pytest", os.path.join(here, "test_gpu_parity.py"), "-x", "-q", "-m", "gpu", "-k",
                        "prefill_entry_by_name or prefill_layer_vs_oracle_small or ffn_tc_vs_oracle or ffn_one_launch_matches_two"],
                       env=env, capture_output=True, text=True, timeout=900, cwd=os.path.dirname(here))
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]


@pytest.mark.parametrize("path_name", ["gemv", "tc"])
def test_benchmark_configuration_0_single_expert_one_token(moe, oracle, torch_cuda, path_name):
    """The reference's own CPU-runnable case, at full size: ONE expert (gate and up [512 x 2048], down [2048 x 512],
    GGUF MXFP4 blocks with uniform codes and scale bytes in [118, 130], seed 0), ONE bf16 N(0,1) token.  Dequantised
    weights bit-exact against the reference's C dequantiser; the quantised activation bit-exact; the expert's output
    against the oracle's float64 product over those values."""
    torch = torch_cuda
    w = synth.layer(0, n_expert=1, D=D, FF=FF)
    rng = np.random.default_rng(0)
    x = synth.activations(rng, 1, D)
    Wg, Wu, Wd = (moe.upload_mxfp4(w[k], K, M, 0, 1) for k, K, M in (("gate", D, FF), ("up", D, FF), ("down", FF, D)))
    for name, W, M, K in (("gate", Wg, FF, D), ("up", Wu, FF, D), ("down", Wd, D, FF)):      # 3 x 32,768 blocks
        np.testing.assert_array_equal(moe.dequant_mxfp4(W, M, K).cpu().numpy(), oracle.deq_matrix(w[name][0], M, K))
    Xq, Xs = moe.quant_scatter(torch.from_numpy(x).cuda().to(torch.bfloat16), None, 0, 0, 1)
    xq, xs = oracle.quant_e4m3(x)
    np.testing.assert_array_equal(from_hw(Xq.cpu().numpy()), xq)
    np.testing.assert_array_equal(Xs.cpu().numpy(), xs)
    goffs = torch.tensor([0, 1], dtype=torch.int32, device="cuda")
    path = moe.PATH_GEMV if path_name == "gemv" else moe.PATH_TC
    Hq, Hs, Y = moe.expert_ffn_sorted(Wg, Wu, Wd, 1, goffs, Xq, Xs, D, FF, path)
    xd = oracle.dequant_e4m3(xq, xs)[0]
    y, h, hq, hs = oracle.expert_ffn(w["gate"][0], w["up"][0], w["down"][0], D, FF, xd)
    assert rel_l2(Y.cpu().numpy()[0], y) < TOL
    y2, *_ = oracle.expert_ffn(w["gate"][0], w["up"][0], w["down"][0], D, FF, xd, hq_in=from_hw(Hq.cpu().numpy())[0],
                               hs_in=Hs.cpu().numpy()[0])
    assert rel_l2(Y.cpu().numpy()[0], y2) < TOL_STAGE
