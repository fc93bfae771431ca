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


# ---------------------------------------------------------------- GGUF out
# ggml tensor type ids used by the engine's model file (q36.h:133-141)
GGML_F32, GGML_BF16, GGML_Q8_0, GGML_MXFP4 = 0, 30, 8, 39


def write_gguf(path: str, tensors: dict, meta: dict | None = None, alignment: int = 32) -> None:
    """Writes a GGUF v3 file.  tensors: name -> (ggml_type, dims fastest-first, bytes-like data).
    meta: key -> int | float | str | list of int | list of str (written as u32 / f32 / string / arrays).
    Layout as the engine's reader expects it (gguf.c:129-190): header, metadata, tensor directory, padding to
    `general.alignment`, then each tensor's data at its aligned offset."""
    import struct

    def s(x: str) -> bytes:
        b = x.encode()
        return struct.pack("<Q", len(b)) + b

    meta = dict(meta or {})
    meta.setdefault("general.alignment", alignment)
    out = [b"GGUF", struct.pack("<IQQ", 3, len(tensors), len(meta))]
    for k, v in meta.items():
        out.append(s(k))
        if isinstance(v, bool):
            out.append(struct.pack("<IB", 7, int(v)))
        elif isinstance(v, int):
            out.append(struct.pack("<II", 4, v))
        elif isinstance(v, float):
            out.append(struct.pack("<If", 6, v))
        elif isinstance(v, str):
            out.append(struct.pack("<I", 8) + s(v))
        elif isinstance(v, (list, tuple)) and v and isinstance(v[0], str):
            out.append(struct.pack("<IIQ", 9, 8, len(v)) + b"".join(s(x) for x in v))
        elif isinstance(v, (list, tuple)):
            out.append(struct.pack("<IIQ", 9, 5, len(v)) + b"".join(struct.pack("<i", x) for x in v))
        else:
            raise TypeError(f"metadata value of {k}")
    off = 0
    blobs = []
    for name, (typ, dims, data) in tensors.items():
        data = bytes(data)
        out.append(s(name) + struct.pack("<I", len(dims)) + b"".join(struct.pack("<Q", d) for d in dims) +
                   struct.pack("<IQ", typ, off))
        pad = (-len(data)) % alignment
        blobs.append(data + b"\0" * pad)
        off += len(data) + pad
    head = b"".join(out)
    head += b"\0" * ((-len(head)) % alignment)
    with open(path, "wb") as f:
        f.write(head)
        for b in blobs:
            f.write(b)


def layer_tensors(w: dict, layer: int, router: np.ndarray | None = None, shared_gate: np.ndarray | None = None,
                  post_norm: np.ndarray | None = None) -> dict:
    """The tensors of one MoE block under the engine's names (q36_model.c:62-75) from `layer()`'s dict.
    GGUF dims are fastest-first: expert tensors [K, M, E], router [D, E]."""
    E, FF, nb, _ = w["gate"].shape
    D = nb * 32
    t = {
        f"blk.{layer}.ffn_gate_exps.weight": (GGML_MXFP4, (D, FF, E), w["gate"].tobytes()),
        f"blk.{layer}.ffn_up_exps.weight": (GGML_MXFP4, (D, FF, E), w["up"].tobytes()),
        f"blk.{layer}.ffn_down_exps.weight": (GGML_MXFP4, (FF, D, E), w["down"].tobytes()),
        f"blk.{layer}.ffn_gate_shexp.weight": (GGML_MXFP4, (D, FF), w["sgate"].tobytes()),
        f"blk.{layer}.ffn_up_shexp.weight": (GGML_MXFP4, (D, FF), w["sup"].tobytes()),
        f"blk.{layer}.ffn_down_shexp.weight": (GGML_MXFP4, (FF, D), w["sdown"].tobytes()),
    }
    if router is not None:
        t[f"blk.{layer}.ffn_gate_inp.weight"] = (GGML_F32, (D, E), np.ascontiguousarray(router, np.float32).tobytes())
    if shared_gate is not None:
        t[f"blk.{layer}.ffn_gate_inp_shexp.weight"] = (GGML_F32, (D,), np.ascontiguousarray(shared_gate, np.float32).tobytes())
    if post_norm is not None:
        t[f"blk.{layer}.post_attention_norm.weight"] = (GGML_F32, (D,), np.ascontiguousarray(post_norm, np.float32).tobytes())
    return t
