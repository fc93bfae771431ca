"""Seeded synthetic inputs with the shapes and value distributions of the
benchmark configurations (the reference's own bench is synthetic as well,
bench.c:28-33,66-73).

Weights: GGUF MXFP4 blocks, every nibble uniform over the 16 E2M1 codes, scale
byte uniform in [118, 130].  Activations: N(0,1) rounded to bf16.  Router
logits: N(0,1), optionally plus the Zipf-like per-expert bias
1.1 * ln(1/rank), rank = expert id + 1.
"""
from __future__ import annotations

import numpy as np

D_MODEL = 2048      # q36.h:62  Q36_D_MODEL
N_EXPERT = 256      # q36.h:82  Q36_N_EXPERT
N_USED = 8          # q36.h:83  Q36_N_EXPERT_USED
EXPERT_FF = 512     # q36.h:84  Q36_EXPERT_FF
BLK = 17            # q36.h:114 sizeof(block_mxfp4)


def mxfp4_blocks(rng: np.random.Generator, n_expert: int, M: int, K: int) -> np.ndarray:
    """uint8 [n_expert, M, K/32, 17] GGUF MXFP4 blocks."""
    b = rng.integers(0, 256, size=(n_expert, M, K // 32, BLK), dtype=np.uint8)
    b[..., 0] = rng.integers(118, 131, size=(n_expert, M, K // 32), dtype=np.uint8)
    return b


def bf16_round(x: np.ndarray) -> np.ndarray:
    """float32 -> nearest-even bf16 -> float32."""
    u = np.ascontiguousarray(x, np.float32).view(np.uint32)
    r = ((u >> 16) & 1) + 0x7FFF
    return ((u + r) & 0xFFFF0000).astype(np.uint32).view(np.float32)


def activations(rng: np.random.Generator, T: int, D: int = D_MODEL) -> np.ndarray:
    return bf16_round(rng.standard_normal((T, D), dtype=np.float32))


def router_logits(rng: np.random.Generator, T: int, n_expert: int = N_EXPERT, zipf: bool = False,
                  with_shared_gate: bool = True) -> np.ndarray:
    """float32 [T, n_expert (+1)]; the extra column is the shared-gate logit
    (the reference concatenates it as row 256 of the router,
    q36_engine.cu:1599-1601)."""
    L = rng.standard_normal((T, n_expert + (1 if with_shared_gate else 0)), dtype=np.float32)
    if zipf:
        L[:, :n_expert] += (1.1 * np.log(1.0 / np.arange(1, n_expert + 1))).astype(np.float32)
    return L


def layer(seed: int, n_expert: int = N_EXPERT, D: int = D_MODEL, FF: int = EXPERT_FF):
    """One layer's weights as GGUF blocks: dict gate/up/down [E,...] and the
    shared expert sgate/sup/sdown [1,...]."""
    rng = np.random.default_rng(seed)
    return {
        "gate": mxfp4_blocks(rng, n_expert, FF, D),
        "up": mxfp4_blocks(rng, n_expert, FF, D),
        "down": mxfp4_blocks(rng, n_expert, D, FF),
        "sgate": mxfp4_blocks(rng, 1, FF, D),
        "sup": mxfp4_blocks(rng, 1, FF, D),
        "sdown": mxfp4_blocks(rng, 1, D, FF),
    }
