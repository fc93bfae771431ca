"""ctypes front-end of the CPU oracle (oracle/q36_oracle.c) and of the
reference's own dequantiser (oracle/_ref/libq36ref.so).

TEST INFRASTRUCTURE ONLY: imported by tests/, by __graft_entry__.smoke() and
by bench.py's CPU-baseline / reference arm.  The shipped package never imports
this module.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess
import time

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = os.path.join(_HERE, "_build", "libq36oracle.so")
_REF = os.path.join(_HERE, "_ref", "libq36ref.so")
_REF_GPU = os.path.join(_HERE, "_ref", "libq36ref_gpu.so")

u8p = C.POINTER(C.c_uint8)
f32p = C.POINTER(C.c_float)
f64p = C.POINTER(C.c_double)
i32p = C.POINTER(C.c_int)


def build(force: bool = False) -> None:
    """Compile the oracle (and, when the reference tree is present, _ref)."""
    if force or not os.path.exists(_LIB) or (
        os.path.getmtime(_LIB) < os.path.getmtime(os.path.join(_HERE, "q36_oracle.c"))
    ):
        subprocess.check_call(["make", "-s", "-C", _HERE, "_build/libq36oracle.so"])
    ref_dir = reference_dir()
    if ref_dir and (force or not os.path.exists(_REF)):
        subprocess.check_call(["make", "-s", "-C", _HERE, "ref", f"REF={ref_dir}"])
    if ref_dir and (force or not os.path.exists(_REF_GPU)):
        subprocess.check_call(["make", "-s", "-C", _HERE, "ref_gpu", f"REF={ref_dir}"])


def reference_dir() -> str | None:
    """Root of the reference source tree: the Q36_REFERENCE environment variable, else a `reference`
    directory beside the repository.  None when neither exists (then a prebuilt _ref is used as is)."""
    cand = [os.environ.get("Q36_REFERENCE"), os.path.join(os.path.dirname(os.path.dirname(_HERE)), "reference")]
    for c in cand:
        if c and os.path.isfile(os.path.join(c, "q36_dequant.cuh")):
            return c
    return None


def _p(a, t):
    return a.ctypes.data_as(t) if a is not None else None


_lib = None
_ref = None


def lib():
    global _lib
    if _lib is None:
        build()
        L = C.CDLL(_LIB)
        L.orc_e8m0_half.restype = C.c_float
        L.orc_e8m0_half.argtypes = [C.c_uint8]
        L.orc_e4m3_encode.restype = C.c_uint8
        L.orc_e4m3_encode.argtypes = [C.c_float]
        L.orc_e4m3_decode.restype = C.c_float
        L.orc_e4m3_decode.argtypes = [C.c_uint8]
        L.orc_num_threads.restype = C.c_int
        _lib = L
    return _lib


def ref():
    """The reference's dequantiser, or None when oracle/_ref was never built."""
    global _ref
    if _ref is None:
        build()
        if not os.path.exists(_REF):
            return None
        R = C.CDLL(_REF)
        R.ref_e8m0_half.restype = C.c_float
        R.ref_e8m0_half.argtypes = [C.c_uint8]
        R.ref_fp16.restype = C.c_float
        R.ref_fp16.argtypes = [C.c_uint16]
        R.ref_sizeof_block_mxfp4.restype = C.c_int
        if hasattr(R, "ref_gguf_probe"):
            R.ref_gguf_probe.restype = C.c_int
            R.ref_gguf_probe.argtypes = [C.c_char_p, C.c_char_p, C.POINTER(C.c_uint32), C.POINTER(C.c_uint32),
                                         C.POINTER(C.c_uint64), C.POINTER(C.c_uint64), C.POINTER(C.c_uint64),
                                         C.POINTER(C.c_uint32), C.POINTER(C.c_uint64)]
        _ref = R
    return _ref


# ------------------------------------------------------------------ dequant
def deq_mxfp4(blocks: np.ndarray, use_ref: bool = False) -> np.ndarray:
    """blocks: uint8 [..., 17] GGUF MXFP4 blocks -> float32 [..., 32]."""
    b = np.ascontiguousarray(blocks, dtype=np.uint8).reshape(-1, 17)
    out = np.empty((b.shape[0], 32), np.float32)
    fn = ref().ref_deq_mxfp4_row if use_ref else lib().orc_deq_mxfp4_row
    fn(_p(b, u8p), C.c_int64(b.shape[0] * 32), _p(out, f32p))
    return out.reshape(blocks.shape[:-1] + (32,))


def deq_matrix(blocks: np.ndarray, M: int, K: int, use_ref: bool = False) -> np.ndarray:
    """[M*K/32, 17] blocks of one matrix -> float32 [M, K]."""
    return deq_mxfp4(blocks.reshape(M * K // 32, 17), use_ref).reshape(M, K)


def split_planes(blocks: np.ndarray, K: int, M: int, e0: int, e1: int) -> np.ndarray:
    b = np.ascontiguousarray(blocks, dtype=np.uint8)
    stride = M * K // 2 + M * K // 32
    out = np.empty((e1 - e0) * stride, np.uint8)
    lib().orc_split_planes(_p(b, u8p), K, M, e0, e1, _p(out, u8p))
    return out


# --------------------------------------------------------------------- E4M3
def e4m3_encode(x: np.ndarray) -> np.ndarray:
    f = lib().orc_e4m3_encode
    return np.array([f(float(v)) for v in np.asarray(x, np.float32).ravel()], np.uint8).reshape(np.shape(x))


def e4m3_table() -> np.ndarray:
    f = lib().orc_e4m3_decode
    return np.array([f(b) for b in range(256)], np.float32)


def quant_e4m3(X: np.ndarray):
    X = np.ascontiguousarray(X, np.float32)
    T, K = X.shape
    Xq = np.empty((T, K), np.uint8)
    Xs = np.empty((T, K // 32), np.uint8)
    lib().orc_quant_e4m3(_p(X, f32p), _p(Xq, u8p), _p(Xs, u8p), T, K)
    return Xq, Xs


def dequant_e4m3(Xq: np.ndarray, Xs: np.ndarray) -> np.ndarray:
    Xq = np.ascontiguousarray(Xq, np.uint8)
    Xs = np.ascontiguousarray(Xs, np.uint8)
    T, K = Xq.shape
    X = np.empty((T, K), np.float32)
    lib().orc_dequant_e4m3(_p(Xq, u8p), _p(Xs, u8p), _p(X, f32p), T, K)
    return X


# ------------------------------------------------------------------- router
def router_topk(logits: np.ndarray, k: int = 8, scale: float = 1.0, renorm: bool = True,
                n_expert: int | None = None):
    L = np.ascontiguousarray(logits, np.float32)
    T, stride = L.shape
    n_expert = n_expert or stride
    idx = np.empty((T, k), np.int32)
    wt = np.empty((T, k), np.float32)
    lib().orc_router_topk(_p(L, f32p), n_expert, k, _p(idx, i32p), _p(wt, f32p),
                          C.c_float(scale), int(renorm), T, stride)
    return idx, wt


def dispatch(topk: np.ndarray, n_expert: int):
    tk = np.ascontiguousarray(topk, np.int32)
    T, k = tk.shape
    ecount = np.empty(n_expert, np.int32)
    eoffs = np.empty(n_expert + 1, np.int32)
    elist = np.empty(T * k, np.int32)
    lib().orc_dispatch(_p(tk, i32p), _p(ecount, i32p), _p(eoffs, i32p), _p(elist, i32p), T, k, n_expert)
    return ecount, eoffs, elist


# --------------------------------------------------------------- expert FFN
def expert_ffn(gate, up, down, D, FF, xd, hq_in=None, hs_in=None):
    """One expert, one token.  Returns (y f64[D], h f32[FF], hq u8[FF], hs u8[FF/32])."""
    g = np.ascontiguousarray(gate, np.uint8)
    u = np.ascontiguousarray(up, np.uint8)
    d = np.ascontiguousarray(down, np.uint8)
    xd = np.ascontiguousarray(xd, np.float32)
    y = np.empty(D, np.float64)
    h = np.empty(FF, np.float32)
    hq = np.empty(FF, np.uint8)
    hs = np.empty(FF // 32, np.uint8)
    hqi = np.ascontiguousarray(hq_in, np.uint8) if hq_in is not None else None
    hsi = np.ascontiguousarray(hs_in, np.uint8) if hs_in is not None else None
    lib().orc_expert_ffn(_p(g, u8p), _p(u, u8p), _p(d, u8p), D, FF, _p(xd, f32p),
                         _p(hqi, u8p), _p(hsi, u8p), _p(y, f64p), _p(h, f32p), _p(hq, u8p), _p(hs, u8p))
    return y, h, hq, hs


def moe_layer(Wg, Wu, Wd, Sg, Su, Sd, D, FF, X, idx, wt, shg, tokens=None,
              se0=0, se1=None, inc_shared=True):
    """Layer output (f64 [n_tok, D]) for the listed tokens (default: all)."""
    X = np.ascontiguousarray(X, np.float32)
    T = X.shape[0]
    idx = np.ascontiguousarray(idx, np.int32)
    wt = np.ascontiguousarray(wt, np.float32)
    k = idx.shape[1]
    shg = np.ascontiguousarray(shg if shg is not None else np.zeros(T), np.float32)
    tok = np.ascontiguousarray(np.arange(T) if tokens is None else tokens, np.int32)
    E = Wg.reshape(-1).shape[0] // (FF * (D // 32) * 17)
    se1 = E if se1 is None else se1
    out = np.empty((tok.shape[0], D), np.float64)
    a = [np.ascontiguousarray(w, np.uint8) if w is not None else None for w in (Wg, Wu, Wd, Sg, Su, Sd)]
    lib().orc_moe_layer(*[_p(w, u8p) for w in a], D, FF, k, se0, se1, int(inc_shared),
                        _p(X, f32p), _p(idx, i32p), _p(wt, f32p), _p(shg, f32p),
                        _p(tok, i32p), tok.shape[0], _p(out, f64p))
    return out


# ------------------------------------------------------------- CPU baseline
def add_rmsnorm(h: np.ndarray, a: np.ndarray | None, w: np.ndarray, eps: float):
    """k_add_rmsnorm (q36_engine.cu:696-706) / k_rmsnorm_b (:3230-3240) per row: h += a (f32), then
    y = h * rsqrt(mean(h^2) + eps) * w, the reduction in float64.  Returns (h_new f32, y f64)."""
    hn = np.asarray(h, np.float32) if a is None else (np.asarray(h, np.float32) + np.asarray(a, np.float32))
    h64 = hn.astype(np.float64)
    ss = 1.0 / np.sqrt((h64 * h64).mean(axis=-1, keepdims=True) + float(eps))
    return hn, h64 * ss * np.asarray(w, np.float64)


def router_logits(x: np.ndarray, router_w: np.ndarray) -> np.ndarray:
    """k_matvec_f32_row (q36_ops.cuh:331-342) over the concatenated router [n_rows][D]: float64 dot products."""
    return np.asarray(x, np.float64) @ np.asarray(router_w, np.float64).T


def cpu_expert_seconds(gate, up, down, D, FF, xd, reps: int, threads: int | None = None,
                       use_ref: bool = True):
    """Times `reps` runs of the reference's CPU path for one (token, expert)
    pair: C dequantiser over gate/up/down + plain fp32 matmul.  Returns
    (median seconds per run, y, kind, threads)."""
    L = lib()
    R = ref() if use_ref else None
    deq = C.cast(R.ref_deq_mxfp4_row if R is not None else L.orc_deq_mxfp4_row, C.c_void_p)
    kind = "reference" if R is not None else "port"
    if threads:
        L.orc_set_threads(int(threads))
    nthr = L.orc_num_threads()
    g = np.ascontiguousarray(gate, np.uint8)
    u = np.ascontiguousarray(up, np.uint8)
    d = np.ascontiguousarray(down, np.uint8)
    xd = np.ascontiguousarray(xd, np.float32)
    scratch = np.empty(3 * FF * D, np.float32)
    y = np.empty(D, np.float32)
    L.orc_cpu_expert_f32.argtypes = [C.c_void_p, u8p, u8p, u8p, C.c_int, C.c_int, f32p, f32p, f32p]
    ts = []
    for _ in range(reps):
        t0 = time.perf_counter()
        L.orc_cpu_expert_f32(deq, _p(g, u8p), _p(u, u8p), _p(d, u8p), D, FF, _p(xd, f32p),
                             _p(scratch, f32p), _p(y, f32p))
        ts.append(time.perf_counter() - t0)
    return float(np.median(ts)), y, kind, nthr


def ref_gguf_probe(path: str, name: str):
    """What the reference's own GGUF reader (gguf.c) reports for tensor `name` of the file at `path`:
    dict(type, dims, file_offset, nbytes, alignment, n_tensors), or None when oracle/_ref lacks the reader."""
    R = ref()
    if R is None or not hasattr(R, "ref_gguf_probe"):
        return None
    t, nd, al = C.c_uint32(), C.c_uint32(), C.c_uint32()
    off, nb, nt = C.c_uint64(), C.c_uint64(), C.c_uint64()
    dims = (C.c_uint64 * 4)()
    rc = R.ref_gguf_probe(os.fsencode(path), name.encode(), C.byref(t), C.byref(nd), dims, C.byref(off), C.byref(nb),
                          C.byref(al), C.byref(nt))
    if rc != 0:
        raise KeyError(f"reference reader: rc {rc} for {name}")
    return {"type": t.value, "dims": tuple(dims[d] for d in range(nd.value)), "file_offset": off.value,
            "nbytes": nb.value, "alignment": al.value, "n_tensors": nt.value}


_ref_gpu = None


def ref_gpu():
    """The reference's own device kernels compiled for sm_100a (oracle/_ref/libq36ref_gpu.so), or None when that
    file was never built.  Every function takes raw device pointers, runs on the legacy default stream,
    synchronises the device and returns the CUDA error code (0 = ok)."""
    global _ref_gpu
    if _ref_gpu is None:
        if not os.path.exists(_REF_GPU):
            return None
        G = C.CDLL(_REF_GPU)
        vp, i32, f32 = C.c_void_p, C.c_int, C.c_float
        G.ref_gpu_router_topk.argtypes = [vp, i32, i32, vp, vp, f32, i32, i32, i32]
        G.ref_gpu_silu_mul.argtypes = [vp, vp, i32]
        G.ref_gpu_rmsnorm.argtypes = [vp, vp, vp, i32, f32]
        G.ref_gpu_matvec_f32_row.argtypes = [vp, vp, vp, i32, i32]
        G.ref_gpu_dot_mxfp4_split.argtypes = [vp, vp, vp, i32, i32, i32]
        for fn in (G.ref_gpu_router_topk, G.ref_gpu_silu_mul, G.ref_gpu_rmsnorm, G.ref_gpu_matvec_f32_row, G.ref_gpu_dot_mxfp4_split):
            fn.restype = i32
        _ref_gpu = G
    return _ref_gpu
