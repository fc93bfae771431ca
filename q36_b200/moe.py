"""Host-side binding of libq36moe.so (the C ABI in include/q36_moe.h).

torch is used for device memory and streams only; every computation goes
through the C entry points.  The library must have been built
(`python -m q36_b200.build`): importing this module without it raises.

`MoELayer` mirrors what the q36 engine keeps per layer for this path: the
expert weights in the split-plane layout of upload() (q36_engine.cu:202-228),
the shared expert, the expert shard [se0, se1) (q36_engine.cu:57-60) and the
scratch that `moe_ffn` / `pf_moe_block` use (q36_engine.cu:1592-1654,
3423-3472).
"""
from __future__ import annotations

import ctypes as C
import os

import numpy as np
import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libq36moe.so")

PATH_AUTO, PATH_GEMV, PATH_TC = 0, 1, 2
OK, EINVAL, ECUDA, ENOSPACE, EDEVICE, EUNSUPPORTED, EIO = 0, -1, -2, -3, -4, -5, -6

if not os.path.exists(LIB_PATH):
    raise ImportError(
        f"{LIB_PATH} is missing: build it with `python -m q36_b200.build` "
        "(there is no CPU or PyTorch fallback for this path)")

lib = C.CDLL(LIB_PATH)
vp, i32, u64, f32 = C.c_void_p, C.c_int, C.c_uint64, C.c_float

_SIGS = {
    "q36_moe_strerror": (C.c_char_p, [i32]),
    "q36_moe_last_cuda_error": (i32, []),
    "q36_moe_abi_version": (i32, []),
    "q36_moe_expert_stride": (u64, [i32, i32]),
    "q36_moe_repack_mxfp4": (i32, [vp, i32, i32, i32, i32, vp]),
    "q36_moe_upload_mxfp4": (i32, [vp, i32, i32, i32, i32, vp]),
    "q36_gguf_open": (i32, [C.c_char_p, C.POINTER(vp)]),
    "q36_gguf_close": (i32, [vp]),
    "q36_gguf_last_error": (C.c_char_p, []),
    "q36_gguf_tensor": (i32, [vp, C.c_char_p, C.POINTER(i32), C.POINTER(i32), C.POINTER(u64), C.POINTER(vp), C.POINTER(u64)]),
    "q36_gguf_meta_u32": (i32, [vp, C.c_char_p, C.POINTER(C.c_uint32)]),
    "q36_moe_gguf_layer_shape": (i32, [vp, i32, C.POINTER(i32), C.POINTER(i32), C.POINTER(i32), C.POINTER(i32)]),
    "q36_moe_gguf_upload_layer": (i32, [vp, i32, i32, i32, vp, vp, vp]),
    "q36_moe_gguf_upload_shared": (i32, [vp, i32, vp, vp, vp]),
    "q36_moe_gguf_upload_router": (i32, [vp, i32, vp]),
    "q36_moe_gguf_upload_f32": (i32, [vp, C.c_char_p, vp, u64]),
    "q36_moe_dequant_mxfp4": (i32, [vp, i32, i32, vp, vp]),
    "q36_moe_router_topk": (i32, [vp, i32, i32, vp, vp, f32, i32, i32, i32, vp]),
    "q36_moe_quant_e4m3": (i32, [vp, i32, vp, vp, i32, i32, vp]),
    "q36_moe_dispatch_ws_bytes": (u64, [i32, i32]),
    "q36_moe_dispatch": (i32, [vp, i32, i32, i32, i32, vp, vp, vp, vp, vp, u64, vp]),
    "q36_moe_dispatch_noalloc": (i32, [vp, i32, i32, i32, i32, vp, vp, vp, vp, vp]),
    "q36_moe_quant_scatter": (i32, [vp, i32, vp, i32, i32, vp, vp, i32, i32, vp]),
    "q36_moe_ffn_ws_bytes": (u64, [i32, i32, i32, i32]),
    "q36_moe_one_launch_fits": (i32, [i32, i32, i32, i32]),
    "q36_moe_one_launch_rows": (i32, []),
    "q36_moe_expert_ffn_sorted": (i32, [vp, vp, vp, i32, vp, vp, vp, vp, vp, i32, vp, vp, vp, vp, vp, i32, i32, i32,
                                        i32, i32, vp, u64, vp]),
    "q36_moe_combine": (i32, [vp, vp, vp, vp, vp, vp, i32, i32, i32, i32, vp]),
    "q36_moe_workspace_bytes": (u64, [i32, i32, i32, i32, i32]),
    "q36_moe_ws_status": (i32, [vp, vp]),
    "q36_moe_ws_reset": (i32, [vp, vp]),
    "q36_moe_selftest_wait_timeout": (i32, [vp, vp]),
    "q36_moe_layer": (i32, [vp] * 6 + [i32] * 6 + [vp, i32, vp, i32, i32, f32, i32, vp, vp, vp, i32, i32, vp, u64, vp]),
    "q36_moe_decode": (i32, [vp] * 6 + [i32] * 6 + [vp, i32, vp, i32, i32, f32, i32, vp, i32, vp, u64, vp]),
    "q36_moe_prefill": (i32, [vp] * 6 + [i32] * 6 + [vp, i32, vp, i32, i32, f32, i32, vp, i32, vp, u64, vp]),
    "q36_moe_pre_norm_router": (i32, [vp, vp, vp, f32, vp, i32, i32, vp, vp, i32, i32, i32, vp]),
    "q36_moe_combine_add_rmsnorm": (i32, [vp, vp, vp, vp, vp, vp, i32, vp, vp, f32, vp, i32, i32, i32, vp]),
    "q36_moe_block_workspace_bytes": (u64, [i32, i32, i32, i32, i32]),
    "q36_moe_block": (i32, [vp] * 6 + [i32] * 6 + [vp, vp, vp, f32, f32, i32, vp, vp, vp, vp, i32, vp, u64, vp]),
    "q36_moe_host_io_bytes": (u64, [i32, i32, i32, i32]),
    "q36_moe_layer_host": (i32, [vp] * 6 + [i32] * 6 + [vp, i32, vp, i32, i32, f32, i32, vp, i32, i32, vp, vp, u64, vp]),
    "q36_moe_stack_host_io_bytes": (u64, [i32, i32, i32, i32, i32]),
    "q36_moe_stack_host": (i32, [i32] + [vp] * 6 + [i32] * 6 + [vp, i32, vp, i32, i32, f32, i32, vp, i32, i32, vp, vp, u64, vp]),
    "q36_moe_ep_stack_host": (i32, [vp, i32] + [vp] * 6 + [i32] * 4 + [vp, i32, vp, i32, i32, f32, vp, i32, vp, vp, u64, vp]),
    "q36_moe_gather_rows": (i32, [vp, vp, vp, i32, i32, vp]),
    "q36_moe_ep_unique_id": (i32, [vp]),
    "q36_moe_ep_init": (i32, [vp, i32, i32, C.POINTER(vp)]),
    "q36_moe_ep_destroy": (i32, [vp]),
    "q36_moe_ep_init_local": (i32, [i32, C.POINTER(i32), C.POINTER(vp)]),
    "q36_moe_ep_open_window": (i32, [vp, i32, i32, i32, i32]),
    "q36_moe_ep_set_transport": (i32, [vp, i32]),
    "q36_moe_ep_workspace_bytes": (u64, [i32, i32, i32, i32, i32, i32, i32]),
    "q36_moe_ep_layer_phase": (i32, [vp, i32] + [vp] * 6 + [i32] * 4 + [vp, i32, vp, i32, i32, f32, vp, i32, vp, u64, vp]),
    "q36_moe_ep_layer": (i32, [vp] * 7 + [i32] * 4 + [vp, i32, vp, i32, i32, f32, vp, i32, vp, u64, vp]),
    "q36_moe_tc_selftest": (i32, [vp, vp, vp, vp, i32, i32, vp, u64, vp]),
}
for _n, (_r, _a) in _SIGS.items():
    _f = getattr(lib, _n)
    _f.restype, _f.argtypes = _r, _a


class MoEError(RuntimeError):
    pass


def check(rc: int, what: str = "") -> None:
    if rc != OK:
        msg = lib.q36_moe_strerror(rc).decode()
        extra = f" (code {lib.q36_moe_last_cuda_error()})" if rc in (ECUDA, EDEVICE) else ""
        if rc in (EIO, EUNSUPPORTED):
            extra = f": {lib.q36_gguf_last_error().decode()}"
        raise MoEError(f"{what}: {msg}{extra}")


def ptr(t) -> int | None:
    return None if t is None else t.data_ptr()


def stream_ptr(stream=None) -> int:
    s = stream if stream is not None else torch.cuda.current_stream()
    return s.cuda_stream


def expert_stride(M: int, K: int) -> int:
    return int(lib.q36_moe_expert_stride(M, K))


def upload_mxfp4(blocks: np.ndarray, K: int, M: int, e0: int, e1: int, device="cuda") -> torch.Tensor:
    """GGUF blocks uint8 [E, M, K/32, 17] (host) -> split planes on the device."""
    b = np.ascontiguousarray(blocks, dtype=np.uint8)
    dst = torch.empty((e1 - e0) * expert_stride(M, K), dtype=torch.uint8, device=device)
    check(lib.q36_moe_upload_mxfp4(b.ctypes.data, K, M, e0, e1, dst.data_ptr()), "upload_mxfp4")
    return dst


def dequant_mxfp4(W: torch.Tensor, M: int, K: int) -> torch.Tensor:
    out = torch.empty((M, K), dtype=torch.float32, device=W.device)
    check(lib.q36_moe_dequant_mxfp4(W.data_ptr(), M, K, out.data_ptr(), stream_ptr()), "dequant_mxfp4")
    return out


def router_topk(logits: torch.Tensor, n_expert: int, k: int = 8, scale: float = 1.0, renorm: bool = True):
    T, stride = logits.shape
    idx = torch.empty((T, k), dtype=torch.int32, device=logits.device)
    wt = torch.empty((T, k), dtype=torch.float32, device=logits.device)
    check(lib.q36_moe_router_topk(logits.data_ptr(), n_expert, k, idx.data_ptr(), wt.data_ptr(), scale,
                                  int(renorm), T, stride, stream_ptr()), "router_topk")
    return idx, wt


def quant_e4m3(X: torch.Tensor):
    T, K = X.shape
    bf = X.dtype == torch.bfloat16
    assert bf or X.dtype == torch.float32
    Xq = torch.empty((T, K), dtype=torch.uint8, device=X.device)
    Xs = torch.empty((T, K // 32), dtype=torch.uint8, device=X.device)
    check(lib.q36_moe_quant_e4m3(X.data_ptr(), int(bf), Xq.data_ptr(), Xs.data_ptr(), T, K, stream_ptr()), "quant_e4m3")
    return Xq, Xs


def dispatch(eid: torch.Tensor, n_expert: int, se0: int = 0, se1: int | None = None):
    se1 = n_expert if se1 is None else se1
    n = eid.numel()
    dev = eid.device
    ecount = torch.empty(n_expert, dtype=torch.int32, device=dev)
    eoffs = torch.empty(n_expert + 1, dtype=torch.int32, device=dev)
    elist = torch.full((max(n, 1),), -1, dtype=torch.int32, device=dev)
    pos = torch.empty(max(n, 1), dtype=torch.int32, device=dev)
    wsb = int(lib.q36_moe_dispatch_ws_bytes(n, n_expert))
    ws = torch.empty(wsb, dtype=torch.uint8, device=dev)
    check(lib.q36_moe_dispatch(eid.data_ptr(), n, n_expert, se0, se1, ecount.data_ptr(), eoffs.data_ptr(),
                               elist.data_ptr(), pos.data_ptr(), ws.data_ptr(), wsb, stream_ptr()), "dispatch")
    return ecount, eoffs, elist[:n], pos[:n]


def quant_scatter(X: torch.Tensor, pos: torch.Tensor | None, k: int, shared_row0: int, R: int):
    T, K = X.shape
    bf = X.dtype == torch.bfloat16
    Xq = torch.zeros((R, K), dtype=torch.uint8, device=X.device)
    Xs = torch.full((R, K // 32), 127, dtype=torch.uint8, device=X.device)
    check(lib.q36_moe_quant_scatter(X.data_ptr(), int(bf), ptr(pos), k, shared_row0, Xq.data_ptr(), Xs.data_ptr(),
                                    T, K, stream_ptr()), "quant_scatter")
    return Xq, Xs


def expert_ffn_sorted(Wg, Wu, Wd, n_group: int, goffs: torch.Tensor, Xq: torch.Tensor, Xs: torch.Tensor,
                      D: int, FF: int, path: int, sync_check: bool = True, shared=None, soffs=None, stages: int = 3,
                      bufs=None, ws=None, max_group_rows: int = 0):
    """Grouped expert FFN over sorted rows.  shared = (Sg, Su, Sd) planes of the extra group whose rows are
    [soffs[0], soffs[1]).  bufs = (Hq, Hs, Y) to reuse; returns (Hq, Hs, Y)."""
    R = Xq.shape[0]
    dev = Xq.device
    if bufs is None:
        bufs = (torch.zeros((R, FF), dtype=torch.uint8, device=dev),
                torch.zeros((R, FF // 32), dtype=torch.uint8, device=dev),
                torch.zeros((R, D), dtype=torch.float32, device=dev))
    Hq, Hs, Y = bufs
    wsb = int(lib.q36_moe_ffn_ws_bytes(n_group, R, D, FF))
    if ws is None:
        ws = torch.zeros(wsb, dtype=torch.uint8, device=dev)
    Sg, Su, Sd = shared if shared is not None else (None, None, None)
    check(lib.q36_moe_expert_ffn_sorted(Wg.data_ptr(), Wu.data_ptr(), Wd.data_ptr(), n_group, goffs.data_ptr(),
                                        ptr(Sg), ptr(Su), ptr(Sd), ptr(soffs), R, Xq.data_ptr(), Xs.data_ptr(),
                                        Hq.data_ptr(), Hs.data_ptr(), Y.data_ptr(), D, FF, path, stages, max_group_rows,
                                        ws.data_ptr(), ws.numel(), stream_ptr()), "expert_ffn_sorted")
    if path == PATH_TC and sync_check:
        check(lib.q36_moe_ws_status(ws.data_ptr(), stream_ptr()), "expert_ffn_sorted (device status)")
    return Hq, Hs, Y


def combine(Y, pos, wt, SH, shgate, shgate_stride: int, D: int, k: int, T: int):
    out = torch.empty((T, D), dtype=torch.float32, device=Y.device)
    check(lib.q36_moe_combine(out.data_ptr(), Y.data_ptr(), pos.data_ptr(), wt.data_ptr(), ptr(SH), ptr(shgate),
                              shgate_stride, D, k, T, stream_ptr()), "combine")
    return out


def pre_norm_router(h, a, norm_w, router_w, eps=1e-6, gate_row=None):
    """h [T,D] f32 (updated in place when a is given) -> (x [T,D], logits [T, n_rows])."""
    T, D = h.shape
    n_rows = router_w.shape[0]
    x = torch.empty_like(h)
    logits = torch.empty((T, n_rows), dtype=torch.float32, device=h.device)
    check(lib.q36_moe_pre_norm_router(h.data_ptr(), ptr(a), norm_w.data_ptr(), eps, router_w.data_ptr(), n_rows,
                                      -1 if gate_row is None else gate_row, x.data_ptr(), logits.data_ptr(), n_rows, T, D,
                                      stream_ptr()), "pre_norm_router")
    return x, logits


def combine_add_rmsnorm(Y, pos, wt, SH, shgate, shgate_stride, h, next_norm_w, eps, D, k, T):
    """Returns (moe [T,D], x_next [T,D]); h is updated in place."""
    moe_out = torch.empty((T, D), dtype=torch.float32, device=Y.device)
    x_next = torch.empty((T, D), dtype=torch.float32, device=Y.device)
    check(lib.q36_moe_combine_add_rmsnorm(moe_out.data_ptr(), Y.data_ptr(), pos.data_ptr(), wt.data_ptr(), ptr(SH),
                                          ptr(shgate), shgate_stride, h.data_ptr(), next_norm_w.data_ptr(), eps,
                                          x_next.data_ptr(), D, k, T, stream_ptr()), "combine_add_rmsnorm")
    return moe_out, x_next


def gather_rows(src: torch.Tensor, index: torch.Tensor, n_rows: int | None = None) -> torch.Tensor:
    n_rows = index.numel() if n_rows is None else n_rows
    row_bytes = src.shape[1] * src.element_size()
    dst = torch.empty((n_rows, src.shape[1]), dtype=src.dtype, device=src.device)
    check(lib.q36_moe_gather_rows(src.data_ptr(), index.data_ptr(), dst.data_ptr(), n_rows, row_bytes, stream_ptr()),
          "gather_rows")
    return dst


def tc_selftest(A: torch.Tensor, Bq: torch.Tensor, Bs: torch.Tensor, N: int, K: int) -> torch.Tensor:
    """A: split layout of one 128-row matrix; returns D [N,128]; raises on a device-side timeout."""
    D = torch.zeros((N, 128), dtype=torch.float32, device=A.device)
    wsb = 512 + int(lib.q36_moe_ffn_ws_bytes(1, N, 128, K))
    ws = torch.zeros(wsb, dtype=torch.uint8, device=A.device)
    check(lib.q36_moe_tc_selftest(A.data_ptr(), Bq.data_ptr(), Bs.data_ptr(), D.data_ptr(), N, K, ws.data_ptr(), wsb,
                                  stream_ptr()), "tc_selftest")
    return D


class GgufFile:
    """A GGUF v3 file opened through the library's reader (the role of gguf.c in the engine)."""

    def __init__(self, path: str):
        self.h = vp()
        check(lib.q36_gguf_open(os.fsencode(path), C.byref(self.h)), "gguf_open")

    def close(self):
        if self.h:
            lib.q36_gguf_close(self.h)
            self.h = vp()

    def __enter__(self):
        return self

    def __exit__(self, *a):
        self.close()

    def tensor(self, name: str):
        """(ggml type, dims tuple, numpy uint8 view of the bytes in the mapping)."""
        t, nd, nb, data = i32(), i32(), u64(), vp()
        dims = (u64 * 4)()
        check(lib.q36_gguf_tensor(self.h, name.encode(), C.byref(t), C.byref(nd), dims, C.byref(data), C.byref(nb)), "gguf_tensor")
        buf = np.ctypeslib.as_array(C.cast(data, C.POINTER(C.c_uint8)), shape=(nb.value,)) if nb.value else np.zeros(0, np.uint8)
        return t.value, tuple(dims[d] for d in range(nd.value)), buf

    def meta_u32(self, key: str) -> int:
        v = C.c_uint32()
        check(lib.q36_gguf_meta_u32(self.h, key.encode(), C.byref(v)), "gguf_meta_u32")
        return v.value

    def layer_shape(self, layer: int):
        e, d, ff = i32(), i32(), i32()
        types = (i32 * 3)()
        check(lib.q36_moe_gguf_layer_shape(self.h, layer, C.byref(e), C.byref(d), C.byref(ff), types), "gguf_layer_shape")
        return e.value, d.value, ff.value, tuple(types)


class MoELayer:
    """One MoE layer resident on one GPU: routed experts [se0, se1) of n_expert,
    plus (optionally) the shared expert."""

    def __init__(self, n_expert=256, k=8, D=2048, FF=512, se0=0, se1=None, device="cuda"):
        self.E, self.k, self.D, self.FF = n_expert, k, D, FF
        self.se0, self.se1 = se0, (n_expert if se1 is None else se1)
        self.device = torch.device(device)
        self.Wg = self.Wu = self.Wd = None
        self.Sg = self.Su = self.Sd = None
        self._ws = None
        self._ws_T = 0
        self._io = None

    # ---- weights
    def load_gguf_blocks(self, gate, up, down, sgate=None, sup=None, sdown=None):
        """GGUF MXFP4 blocks (numpy uint8) for ALL n_expert experts; only the shard is uploaded."""
        D, FF = self.D, self.FF
        self.Wg = upload_mxfp4(gate, D, FF, self.se0, self.se1, self.device)
        self.Wu = upload_mxfp4(up, D, FF, self.se0, self.se1, self.device)
        self.Wd = upload_mxfp4(down, FF, D, self.se0, self.se1, self.device)
        if sgate is not None:
            self.Sg = upload_mxfp4(sgate, D, FF, 0, 1, self.device)
            self.Su = upload_mxfp4(sup, D, FF, 0, 1, self.device)
            self.Sd = upload_mxfp4(sdown, FF, D, 0, 1, self.device)
        return self

    def load_gguf(self, gguf: "GgufFile", layer: int, shared: bool = True):
        """Expert planes of block `layer` straight from a GGUF file (MXFP4 tensors); only the shard is uploaded."""
        E, D, FF, _ = gguf.layer_shape(layer)
        assert (E, D, FF) == (self.E, self.D, self.FF), f"file has E={E} D={D} FF={FF}"
        n = self.se1 - self.se0
        self.Wg = torch.empty(n * expert_stride(FF, D), dtype=torch.uint8, device=self.device)
        self.Wu = torch.empty_like(self.Wg)
        self.Wd = torch.empty(n * expert_stride(D, FF), dtype=torch.uint8, device=self.device)
        check(lib.q36_moe_gguf_upload_layer(gguf.h, layer, self.se0, self.se1, self.Wg.data_ptr(), self.Wu.data_ptr(),
                                            self.Wd.data_ptr()), "gguf_upload_layer")
        if shared:
            self.Sg = torch.empty(expert_stride(FF, D), dtype=torch.uint8, device=self.device)
            self.Su = torch.empty_like(self.Sg)
            self.Sd = torch.empty(expert_stride(D, FF), dtype=torch.uint8, device=self.device)
            check(lib.q36_moe_gguf_upload_shared(gguf.h, layer, self.Sg.data_ptr(), self.Su.data_ptr(), self.Sd.data_ptr()),
                  "gguf_upload_shared")
        return self

    def set_device_planes(self, Wg, Wu, Wd, Sg=None, Su=None, Sd=None):
        """Planes already on the device in the split layout (uint8 tensors)."""
        self.Wg, self.Wu, self.Wd, self.Sg, self.Su, self.Sd = Wg, Wu, Wd, Sg, Su, Sd
        return self

    def random_planes(self, seed: int, shared: bool = True):
        """Synthetic weights generated on the device: uniform code nibbles, scale bytes in [118,130]."""
        g = torch.Generator(device=self.device)
        g.manual_seed(seed)
        n = self.se1 - self.se0

        def planes(ne, M, K):
            t = torch.randint(0, 256, (ne, expert_stride(M, K)), dtype=torch.uint8, device=self.device, generator=g)
            t[:, M * K // 2:] = torch.randint(118, 131, (ne, M * K // 32), dtype=torch.uint8, device=self.device,
                                              generator=g)
            return t.reshape(-1)

        self.Wg, self.Wu, self.Wd = planes(n, self.FF, self.D), planes(n, self.FF, self.D), planes(n, self.D, self.FF)
        if shared:
            self.Sg, self.Su, self.Sd = planes(1, self.FF, self.D), planes(1, self.FF, self.D), planes(1, self.D, self.FF)
        return self

    # ---- scratch
    def workspace(self, T: int) -> torch.Tensor:
        if self._ws is None or T > self._ws_T:
            nbytes = int(lib.q36_moe_workspace_bytes(T, self.E, self.k, self.D, self.FF))
            self._ws = torch.empty(nbytes, dtype=torch.uint8, device=self.device)
            check(lib.q36_moe_ws_reset(self._ws.data_ptr(), stream_ptr()), "ws_reset")
            self._ws_T = T
        return self._ws

    # ---- compute
    def forward(self, X: torch.Tensor, logits: torch.Tensor, out: torch.Tensor | None = None, path: int = PATH_AUTO,
                shgate_col: int | None = None, route_scale: float = 1.0, inc_shared: bool = True,
                want_routing: bool = False, ws: torch.Tensor | None = None, stream=None):
        """X [T,D] f32|bf16, logits [T,stride] f32 (device).  Launch-only."""
        T = X.shape[0]
        bf = X.dtype == torch.bfloat16
        stride = logits.shape[1]
        if shgate_col is None:
            shgate_col = self.E if stride > self.E else -1
        if out is None:
            out = torch.empty((T, self.D), dtype=torch.float32, device=X.device)
        ws = self.workspace(T) if ws is None else ws
        idx = torch.empty((T, self.k), dtype=torch.int32, device=X.device) if want_routing else None
        wt = torch.empty((T, self.k), dtype=torch.float32, device=X.device) if want_routing else None
        check(lib.q36_moe_layer(self.Wg.data_ptr(), self.Wu.data_ptr(), self.Wd.data_ptr(), ptr(self.Sg), ptr(self.Su),
                                ptr(self.Sd), self.E, self.se0, self.se1, self.k, self.D, self.FF, X.data_ptr(), int(bf),
                                logits.data_ptr(), stride, shgate_col, route_scale, int(inc_shared), out.data_ptr(),
                                ptr(idx), ptr(wt), T, path, ws.data_ptr(), ws.numel(), stream_ptr(stream)), "moe_layer")
        return (out, idx, wt) if want_routing else out

    def _by_name(self, fn, name, X, logits, out, shgate_col, route_scale, inc_shared, stream):
        T = X.shape[0]
        stride = logits.shape[1]
        if shgate_col is None:
            shgate_col = self.E if stride > self.E else -1
        if out is None:
            out = torch.empty((T, self.D), dtype=torch.float32, device=X.device)
        ws = self.workspace(T)
        check(fn(self.Wg.data_ptr(), self.Wu.data_ptr(), self.Wd.data_ptr(), ptr(self.Sg), ptr(self.Su), ptr(self.Sd),
                 self.E, self.se0, self.se1, self.k, self.D, self.FF, X.data_ptr(), int(X.dtype == torch.bfloat16),
                 logits.data_ptr(), stride, shgate_col, route_scale, int(inc_shared), out.data_ptr(), T, ws.data_ptr(),
                 ws.numel(), stream_ptr(stream)), name)
        return out

    def decode(self, X, logits, out=None, shgate_col=None, route_scale=1.0, inc_shared=True, stream=None):
        """q36_moe_decode: the engine's moe_ffn by name (q36_engine.cu:1592-1654)."""
        return self._by_name(lib.q36_moe_decode, "moe_decode", X, logits, out, shgate_col, route_scale, inc_shared, stream)

    def prefill(self, X, logits, out=None, shgate_col=None, route_scale=1.0, inc_shared=True, stream=None):
        """q36_moe_prefill: the engine's pf_moe_block by name (q36_engine.cu:3423-3472)."""
        return self._by_name(lib.q36_moe_prefill, "moe_prefill", X, logits, out, shgate_col, route_scale, inc_shared, stream)

    def block(self, h, a, post_norm_w, router_w, next_norm_w, eps=1e-6, route_scale=1.0, inc_shared=True, stream=None):
        """q36_moe_block: the block from the residual stream.  h [T,D] f32 is updated in place; returns
        (x_next [T,D], moe [T,D])."""
        T = h.shape[0]
        need = int(lib.q36_moe_block_workspace_bytes(T, self.E, self.k, self.D, self.FF))
        if self._ws is None or self._ws.numel() < need:
            self._ws = torch.empty(need, dtype=torch.uint8, device=self.device)
            check(lib.q36_moe_ws_reset(self._ws.data_ptr(), stream_ptr()), "ws_reset")
            self._ws_T = T
        x_next = torch.empty((T, self.D), dtype=torch.float32, device=h.device)
        moe_out = torch.empty((T, self.D), dtype=torch.float32, device=h.device)
        check(lib.q36_moe_block(self.Wg.data_ptr(), self.Wu.data_ptr(), self.Wd.data_ptr(), ptr(self.Sg), ptr(self.Su),
                                ptr(self.Sd), self.E, self.se0, self.se1, self.k, self.D, self.FF, post_norm_w.data_ptr(),
                                router_w.data_ptr(), next_norm_w.data_ptr(), eps, route_scale, int(inc_shared), h.data_ptr(),
                                ptr(a), x_next.data_ptr(), moe_out.data_ptr(), T, self._ws.data_ptr(), self._ws.numel(),
                                stream_ptr(stream)), "moe_block")
        return x_next, moe_out

    def reset_device_status(self):
        if self._ws is not None:
            check(lib.q36_moe_ws_reset(self._ws.data_ptr(), stream_ptr()), "ws_reset")

    def check_device_status(self):
        if self._ws is not None:
            check(lib.q36_moe_ws_status(self._ws.data_ptr(), stream_ptr()), "device status")

    def forward_host(self, X: torch.Tensor, logits: torch.Tensor, out: torch.Tensor, path: int = PATH_AUTO,
                     shgate_col: int | None = None, route_scale: float = 1.0, inc_shared: bool = True, stream=None):
        """Host-buffer form: X, logits, out are CPU tensors (pinned for speed); synchronous."""
        T = X.shape[0]
        bf = X.dtype == torch.bfloat16
        stride = logits.shape[1]
        if shgate_col is None:
            shgate_col = self.E if stride > self.E else -1
        ws = self.workspace(T)
        need = int(lib.q36_moe_host_io_bytes(T, self.D, stride, int(bf)))
        if self._io is None or self._io.numel() < need:
            self._io = torch.empty(need, dtype=torch.uint8, device=self.device)
        check(lib.q36_moe_layer_host(self.Wg.data_ptr(), self.Wu.data_ptr(), self.Wd.data_ptr(), ptr(self.Sg),
                                     ptr(self.Su), ptr(self.Sd), self.E, self.se0, self.se1, self.k, self.D, self.FF,
                                     X.data_ptr(), int(bf), logits.data_ptr(), stride, shgate_col, route_scale,
                                     int(inc_shared), out.data_ptr(), T, path, self._io.data_ptr(), ws.data_ptr(),
                                     ws.numel(), stream_ptr(stream)), "moe_layer_host")
        return out


class HostStack:
    """q36_moe_stack_host / q36_moe_ep_stack_host: a stack of layers driven from pinned host buffers, one call
    per step (inputs copied in, results copied out, stream synchronised)."""

    def __init__(self, layers, T: int, x_is_bf16: bool = True, logit_stride: int | None = None, ep=None):
        self.layers, self.T, self.ep = layers, T, ep
        ly = layers[0]
        self.stride = (ly.E + 1) if logit_stride is None else logit_stride
        self.bf16 = x_is_bf16
        n = len(layers)
        arr = lambda ts: (vp * n)(*[ptr(t) for t in ts])
        self.planes = [arr([l.Wg for l in layers]), arr([l.Wu for l in layers]), arr([l.Wd for l in layers]),
                       arr([l.Sg for l in layers]), arr([l.Su for l in layers]), arr([l.Sd for l in layers])]
        self.has_shared = ly.Sg is not None
        io = int(lib.q36_moe_stack_host_io_bytes(n, T, ly.D, self.stride, int(x_is_bf16)))
        self.io = torch.empty(io, dtype=torch.uint8, device=ly.device)
        self.ws = ep.ws if ep is not None else ly.workspace(T)

    def step(self, hX: torch.Tensor, hL: torch.Tensor, hO: torch.Tensor, path: int = PATH_AUTO):
        """hX [L,T,D], hL [L,T,stride], hO [L,T,D]: CPU tensors (pinned for speed).  Synchronous."""
        ly, n = self.layers[0], len(self.layers)
        P = self.planes
        sh = P[3:] if self.has_shared else [None, None, None]
        gate_col = ly.E if self.stride > ly.E else -1
        if self.ep is None:
            check(lib.q36_moe_stack_host(n, P[0], P[1], P[2], sh[0], sh[1], sh[2], ly.E, ly.se0, ly.se1, ly.k, ly.D, ly.FF,
                                         hX.data_ptr(), int(self.bf16), hL.data_ptr(), self.stride, gate_col, 1.0, 1,
                                         hO.data_ptr(), self.T, path, self.io.data_ptr(), self.ws.data_ptr(), self.ws.numel(),
                                         stream_ptr()), "stack_host")
        else:
            check(lib.q36_moe_ep_stack_host(self.ep.comm, n, P[0], P[1], P[2], sh[0], sh[1], sh[2], ly.E, ly.k, ly.D, ly.FF,
                                            hX.data_ptr(), int(self.bf16), hL.data_ptr(), self.stride, gate_col, 1.0,
                                            hO.data_ptr(), self.T, self.io.data_ptr(), self.ws.data_ptr(), self.ws.numel(),
                                            stream_ptr()), "ep_stack_host")
        return hO
