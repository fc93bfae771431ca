"""CPU tests: the oracle against the reference's known answers and golden vectors."""
import os
import subprocess

import numpy as np
import pytest

from q36_b200 import synth

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def test_reference_constants(oracle):
    """The known answers of the reference's test_dequant.c:46-62."""
    L = oracle.lib()
    assert L.orc_e8m0_half(127) == 0.5 and L.orc_e8m0_half(128) == 1.0 and L.orc_e8m0_half(129) == 2.0
    blk = np.zeros(17, np.uint8)
    blk[0] = 128
    blk[1:] = np.arange(16)
    out = oracle.deq_mxfp4(blk)
    np.testing.assert_array_equal(out[:8], np.array([0, 1, 2, 3, 4, 6, 8, 12], np.float32))
    # block_mxfp4 is 17 bytes (test_dequant.c:48): the planes of one 32-block are 16 + 1 bytes
    assert oracle.split_planes(np.zeros((1, 1, 1, 17), np.uint8), 32, 1, 0, 1).size == 17


def test_dequant_matches_reference_golden(oracle):
    """Bit-exact against vectors produced by the reference's own q36_deq_row."""
    g = np.load(os.path.join(GOLD, "dequant_ref.npz"))
    out = oracle.deq_mxfp4(g["blocks"])
    np.testing.assert_array_equal(out.view(np.uint32), g["out_bits"])
    e8 = np.array([oracle.lib().orc_e8m0_half(e) for e in range(256)], np.float32)
    np.testing.assert_array_equal(e8.view(np.uint32), g["e8m0_half_bits"])


def test_dequant_matches_reference_live(oracle):
    """Same, against oracle/_ref when it was built here (the reference tree is mounted)."""
    if oracle.ref() is None:
        pytest.skip("oracle/_ref not built")
    rng = np.random.default_rng(1)
    b = synth.mxfp4_blocks(rng, 2, 64, 256)
    b[..., 0] = rng.integers(0, 255, size=b.shape[:-1], dtype=np.uint8)
    a, r = oracle.deq_mxfp4(b), oracle.deq_mxfp4(b, use_ref=True)
    np.testing.assert_array_equal(a.view(np.uint32), r.view(np.uint32))
    assert oracle.ref().ref_sizeof_block_mxfp4() == 17


def test_e4m3_encoder_pinned_to_cuda_fp8(oracle):
    """pin_e4m3 compares the encoder with cuda_fp8.h's host conversion over ~4e8 floats."""
    exe = os.path.join(os.path.dirname(oracle.__file__), "_build", "pin_e4m3")
    if not os.path.exists(exe):
        r = subprocess.run(["make", "-s", "-C", os.path.dirname(oracle.__file__), "_build/pin_e4m3"],
                           capture_output=True, text=True)
        if r.returncode:
            pytest.skip("cuda_fp8.h / g++ not available to build pin_e4m3")
    r = subprocess.run([exe], capture_output=True, text=True)
    assert r.returncode == 0, r.stdout[-500:]


def test_e4m3_known_values(oracle):
    enc = oracle.e4m3_encode(np.array([1.0, 448.0, 500.0, -3.3, 0.0019, 1e-9, 464.0, 463.9, 0.0009765625], np.float32))
    np.testing.assert_array_equal(enc, np.array([0x38, 0x7E, 0x7E, 0xC5, 0x01, 0x00, 0x7E, 0x7E, 0x00], np.uint8))
    tab = oracle.e4m3_table()
    assert tab[0x7E] == 448.0 and tab[0x01] == 2.0 ** -9 and np.isnan(tab[0x7F])
    # encode(decode(b)) == b for every finite code
    fin = [b for b in range(256) if (b & 0x7F) != 0x7F]
    np.testing.assert_array_equal(oracle.e4m3_encode(tab[fin]), np.array(fin, np.uint8) & np.where(tab[fin] == 0, 0x80, 0xFF))


def test_quantiser_properties(oracle):
    rng = np.random.default_rng(2)
    X = synth.activations(rng, 16, 2048)
    X[0, :32] = 0
    Xq, Xs = oracle.quant_e4m3(X)
    Xd = oracle.dequant_e4m3(Xq, Xs)
    B = X.reshape(16, 64, 32)
    amax = np.abs(B).max(-1)
    e2 = Xs.astype(np.int32) - 127
    nz = amax > 0
    # smallest exponent with amax <= 448 * 2^e2
    assert np.all(amax[nz] <= 448.0 * np.exp2(e2[nz].astype(np.float64)))
    assert np.all(amax[nz] > 448.0 * np.exp2(e2[nz].astype(np.float64) - 1))
    assert np.all(e2[~nz] == -127)
    # E4M3 has 3 mantissa bits: relative error <= 2^-4 for normals of the scaled block
    err = np.abs(Xd - X).reshape(16, 64, 32)
    assert np.all(err <= np.maximum(np.abs(B) * 2.0 ** -4, np.exp2(e2.astype(np.float64))[..., None] * 2.0 ** -10))
    # idempotent: quantising the dequantised values changes nothing
    Xq2, Xs2 = oracle.quant_e4m3(Xd)
    Xd2 = oracle.dequant_e4m3(Xq2, Xs2)
    np.testing.assert_array_equal(Xd2, Xd)


def test_frozen_oracle_outputs(oracle):
    g = np.load(os.path.join(GOLD, "oracle_frozen.npz"))
    Xq, Xs = oracle.quant_e4m3(g["X"])
    np.testing.assert_array_equal(Xq, g["Xq"])
    np.testing.assert_array_equal(Xs, g["Xs"])
    idx, wt = oracle.router_topk(g["L"], 8, n_expert=256)
    np.testing.assert_array_equal(idx, g["idx"])
    np.testing.assert_allclose(wt, g["wt"], rtol=1e-6)
    assert idx[5, 0] == 10 and idx[5, 1] == 200      # tie goes to the lower expert id
    ec, eo, el = oracle.dispatch(idx, 256)
    np.testing.assert_array_equal(el, g["elist"])
    xd = oracle.dequant_e4m3(Xq, Xs)[0]
    y, h, hq, hs = oracle.expert_ffn(g["gate"], g["up"], g["down"], 256, 128, xd)
    np.testing.assert_array_equal(hq, g["hq"])
    np.testing.assert_allclose(y, g["y"], rtol=1e-12)


def test_router_against_numpy(oracle):
    rng = np.random.default_rng(3)
    L = synth.router_logits(rng, 64, 256, zipf=True)
    idx, wt = oracle.router_topk(L, 8, n_expert=256)
    r = L[:, :256].astype(np.float64)
    order = np.argsort(-r, axis=1, kind="stable")[:, :8]
    np.testing.assert_array_equal(idx, order)
    p = np.exp(r - r.max(1, keepdims=True))
    p /= p.sum(1, keepdims=True)
    w = np.take_along_axis(p, order, 1)
    w /= w.sum(1, keepdims=True)
    np.testing.assert_allclose(wt, w, rtol=2e-6)
    np.testing.assert_allclose(wt.sum(1), 1.0, rtol=1e-6)


def test_dispatch_is_stable_sort(oracle):
    rng = np.random.default_rng(4)
    tk = rng.integers(0, 256, size=(100, 8)).astype(np.int32)
    ec, eo, el = oracle.dispatch(tk, 256)
    flat = tk.reshape(-1)
    np.testing.assert_array_equal(el, np.argsort(flat, kind="stable"))
    np.testing.assert_array_equal(ec, np.bincount(flat, minlength=256))
    assert eo[-1] == 800


def test_expert_ffn_against_numpy(oracle):
    """The f64 expert against a plain numpy float64 product over the same dequantised values."""
    rng = np.random.default_rng(5)
    D, FF = 256, 128
    w = synth.layer(11, n_expert=1, D=D, FF=FF)
    x = synth.activations(rng, 1, D)
    Xq, Xs = oracle.quant_e4m3(x)
    xd = oracle.dequant_e4m3(Xq, Xs)[0]
    y, h, hq, hs = oracle.expert_ffn(w["gate"][0], w["up"][0], w["down"][0], D, FF, xd)
    Wg = oracle.deq_matrix(w["gate"][0], FF, D).astype(np.float64)
    Wu = oracle.deq_matrix(w["up"][0], FF, D).astype(np.float64)
    Wd = oracle.deq_matrix(w["down"][0], D, FF).astype(np.float64)
    g, u = Wg @ xd.astype(np.float64), Wu @ xd.astype(np.float64)
    hh = (g / (1 + np.exp(-g)) * u).astype(np.float32)
    np.testing.assert_allclose(h, hh, rtol=1e-6)
    hq2, hs2 = oracle.quant_e4m3(hh[None])
    hd = oracle.dequant_e4m3(hq2, hs2)[0].astype(np.float64)
    np.testing.assert_allclose(y, Wd @ hd, rtol=1e-9, atol=1e-6 * np.abs(y).max())


def test_linearity_of_down_stage(oracle):
    """With the quantised intermediate fixed, the down stage is linear in the routing weight."""
    rng = np.random.default_rng(6)
    D, FF = 256, 128
    w = synth.layer(12, n_expert=2, D=D, FF=FF)
    X = synth.activations(rng, 2, D)
    idx = np.array([[0, 1], [1, 0]], np.int32)
    wt = np.array([[0.25, 0.75], [0.5, 0.5]], np.float32)
    a = oracle.moe_layer(w["gate"], w["up"], w["down"], None, None, None, D, FF, X, idx, wt, None, inc_shared=False)
    b = oracle.moe_layer(w["gate"], w["up"], w["down"], None, None, None, D, FF, X, idx, 2 * wt, None, inc_shared=False)
    np.testing.assert_allclose(b, 2 * a, rtol=1e-12)
    # shard contract: the two half-shards sum to the whole (q36_engine.cu:763-766, 4286-4287)
    s0 = oracle.moe_layer(w["gate"], w["up"], w["down"], None, None, None, D, FF, X, idx, wt, None, se0=0, se1=1, inc_shared=False)
    s1 = oracle.moe_layer(w["gate"], w["up"], w["down"], None, None, None, D, FF, X, idx, wt, None, se0=1, se1=2, inc_shared=False)
    np.testing.assert_allclose(s0 + s1, a, rtol=1e-12)


def test_add_rmsnorm_and_router_logits_restatement(oracle):
    """The oracle's restatement of k_add_rmsnorm / k_matvec_f32_row on a case small enough to check by hand."""
    h = np.array([[3.0, 4.0, 0.0, 0.0]], np.float32)
    a = np.array([[0.0, 0.0, 0.0, 0.0]], np.float32)
    w = np.array([1.0, 2.0, 1.0, 1.0], np.float32)
    hn, y = oracle.add_rmsnorm(h, a, w, 0.0)
    np.testing.assert_array_equal(hn, h)
    np.testing.assert_allclose(y, [[3 / 2.5, 2 * 4 / 2.5, 0, 0]], rtol=1e-12)       # mean(h^2) = 25/4
    hn2, _ = oracle.add_rmsnorm(h, np.ones_like(h), w, 1e-6)
    np.testing.assert_array_equal(hn2, h + 1)
    W = np.array([[1, 0, 0, 0], [1, 1, 1, 1]], np.float32)
    np.testing.assert_allclose(oracle.router_logits(y, W), [[1.2, 1.2 + 3.2]], rtol=1e-12)
