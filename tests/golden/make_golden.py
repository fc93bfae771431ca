"""Regenerates tests/golden/*.npz.

dequant_ref.npz is produced by the REFERENCE's own dequantiser, compiled from
the reference tree by oracle/Makefile into oracle/_ref/libq36ref.so (so it can
only be regenerated where the reference tree is mounted).  The other fixtures
freeze the oracle's outputs on seeded inputs so that a change of the oracle
shows up as a diff.

Run from the repository root:  python tests/golden/make_golden.py
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from oracle import oracle as O  # noqa: E402
from q36_b200 import synth  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))


def main():
    rng = np.random.default_rng(20260101)
    # 1. reference dequantiser: every scale byte 0..254 once with random codes,
    #    plus the test_dequant.c block (e = 128, qs[i] = i)
    blocks = rng.integers(0, 256, size=(256, 17), dtype=np.uint8)
    blocks[:255, 0] = np.arange(255, dtype=np.uint8)
    blocks[255, 0] = 128
    blocks[255, 1:] = np.arange(16, dtype=np.uint8)
    assert O.ref() is not None, "oracle/_ref is not built (reference tree absent?)"
    out = O.deq_mxfp4(blocks, use_ref=True)
    e8 = np.array([O.ref().ref_e8m0_half(e) for e in range(256)], np.float32)
    np.savez_compressed(os.path.join(HERE, "dequant_ref.npz"), blocks=blocks, out_bits=out.view(np.uint32),
                        e8m0_half_bits=e8.view(np.uint32))
    # 2. quantiser / router / dispatch / one expert, frozen from the oracle
    X = synth.activations(rng, 4, 256)
    X[1, :32] = 0.0                     # an all-zero block
    X[2, 32:64] *= 1e-30                # tiny block
    X[3, 64:96] *= 1e30                 # huge block
    X[0, 0] = 448.0
    X[0, 33] = 464.0
    Xq, Xs = O.quant_e4m3(X)
    L = synth.router_logits(rng, 6, 256, zipf=True)
    L[5, 10] = L[5, 200] = L[5].max() + 1.0   # a tie for first place
    idx, wt = O.router_topk(L, 8, n_expert=256)
    ec, eo, el = O.dispatch(idx, 256)
    w = synth.layer(7, n_expert=1, D=256, FF=128)
    xd = O.dequant_e4m3(Xq, Xs)[0]
    y, h, hq, hs = O.expert_ffn(w["gate"][0], w["up"][0], w["down"][0], 256, 128, xd)
    np.savez_compressed(os.path.join(HERE, "oracle_frozen.npz"), X=X, Xq=Xq, Xs=Xs, L=L, idx=idx, wt=wt,
                        ecount=ec, eoffs=eo, elist=el, gate=w["gate"][0], up=w["up"][0], down=w["down"][0],
                        y=y, h=h, hq=hq, hs=hs)
    print("wrote", os.listdir(HERE))


if __name__ == "__main__":
    main()
