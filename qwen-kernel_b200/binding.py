"""ctypes binding of include/qk_moe.h (libqkmoe.so) and a thin host-side mirror
of the reference engine's per-layer MoE interface.

There is no CPU path here: if the CUDA library is missing or no B200 is
present, loading or opening fails with an error.
"""
from __future__ import annotations

import ctypes as C
import os

import numpy as np

from . import synth

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libqkmoe.so")

OK, ERR_ARG, ERR_BUSY, ERR_BOUNDS, ERR_TYPE, ERR_MODE, ERR_CUDA, ERR_TIMEOUT = 0, -1, -2, -3, -4, -5, -6, -7


class Dims(C.Structure):
    _fields_ = [("n_embd", C.c_uint32), ("n_ff", C.c_uint32), ("n_expert", C.c_uint32), ("n_used", C.c_uint32)]


class Config(C.Structure):
    _fields_ = [("dims", Dims), ("n_layer", C.c_uint32), ("max_tokens", C.c_uint32), ("device", C.c_int32),
                ("flags", C.c_uint32), ("expert_first", C.c_uint32), ("expert_count", C.c_uint32)]


class LayerWeights(C.Structure):
    _fields_ = [("router_type", C.c_uint32), ("gateup_type", C.c_uint32), ("down_type", C.c_uint32),
                ("reserved", C.c_uint32), ("router", C.c_void_p), ("gate_inp_shexp", C.c_void_p),
                ("gate_exps", C.c_void_p), ("up_exps", C.c_void_p), ("down_exps", C.c_void_p),
                ("gate_shexp", C.c_void_p), ("up_shexp", C.c_void_p), ("down_shexp", C.c_void_p)]


EP_HANDLE_BYTES = 192   # QKM_EP_HANDLE_BYTES: three CUDA IPC handles
SEL_DTYPE = np.dtype([("ids", np.uint32, 16), ("w", np.float32, 16), ("w_shared", np.float32),
                      ("route_done", np.uint32), ("pad", np.float32, 6)])
assert SEL_DTYPE.itemsize == 160

_VP, _U32, _U64, _I, _SZ = C.c_void_p, C.c_uint32, C.c_uint64, C.c_int, C.c_size_t

# name -> (restype, argtypes); every symbol include/qk_moe.h declares
SIGNATURES = {
    "qkm_open": (_VP, [C.POINTER(Config), C.c_char_p, _SZ]),
    "qkm_close": (None, [_VP]),
    "qkm_last_error": (C.c_char_p, [_VP]),
    "qkm_version": (C.c_char_p, []),
    "qkm_n_embd": (_U32, [_VP]), "qkm_n_ff": (_U32, [_VP]), "qkm_n_expert": (_U32, [_VP]),
    "qkm_n_used": (_U32, [_VP]), "qkm_n_layer": (_U32, [_VP]), "qkm_max_tokens": (_U32, [_VP]),
    "qkm_row_bytes": (_SZ, [_U32, _U64]),
    "qkm_set_stream": (_I, [_VP, _VP]),
    "qkm_sync": (_I, [_VP]),
    "qkm_launch_count": (_U64, [_VP]),
    "qkm_dev_alloc": (_VP, [_VP, _SZ]),
    "qkm_dev_free": (_I, [_VP, _VP]),
    "qkm_h2d": (_I, [_VP, _VP, _VP, _SZ]),
    "qkm_d2h": (_I, [_VP, _VP, _VP, _SZ]),
    "qkm_upload_layer": (_I, [_VP, _U32, C.POINTER(LayerWeights)]),
    "qkm_layer_device_ptrs": (_I, [_VP, _U32, C.POINTER(LayerWeights)]),
    "qkm_moe_logits": (_I, [_VP, _U32, _VP, _VP, _VP, _U32]),
    "qkm_moe_select": (_I, [_VP, _VP, _VP, _VP, _VP, _U32]),
    "qkm_moe_route_select": (_I, [_VP, _U32, _VP, _VP, _VP, _VP, _U32]),
    "qkm_moe_group_pairs": (_I, [_VP, _VP, _U32, _VP, _VP]),
    "qkm_moe_gateup": (_I, [_VP, _U32, _VP, _VP, _VP, _VP, _VP, _U32]),
    "qkm_moe_gateup_grouped": (_I, [_VP, _U32, _VP, _VP, _VP, _VP, _VP, _VP, _U32]),
    "qkm_moe_shared_gateup": (_I, [_VP, _VP, _VP, _VP, _VP, _U32]),
    "qkm_moe_down": (_I, [_VP, _U32, _VP, _VP, _VP, _VP, _U32]),
    "qkm_moe_down_grouped": (_I, [_VP, _U32, _VP, _VP, _VP, _VP, _VP, _VP, _U32]),
    "qkm_moe_shared_down": (_I, [_VP, _VP, _VP, _VP, _VP, _U32]),
    "qkm_gemv": (_I, [_VP, _U32, _VP, _VP, _VP, _U32, _U32, _U32]),
    "qkm_dequant": (_I, [_VP, _U32, _VP, _VP, _U64]),
    "qkm_moe_decode": (_I, [_VP, _U32, _VP, _U32, _VP]),
    "qkm_moe_prefill": (_I, [_VP, _U32, _VP, _U32, _VP]),
    "qkm_moe_forward_host": (_I, [_VP, _U32, _I, _VP, _U32, _VP]),
    "qkm_moe_decode_stack": (_I, [_VP, _U32, _U32, _VP, _U32, _VP]),
    "qkm_moe_decode_stack_host": (_I, [_VP, _U32, _U32, _VP, _U32, _VP]),
    "qkm_profile_enable": (_I, [_VP, _I]),
    "qkm_profile_read": (_I, [_VP, _VP, _VP, _U32]),
    "qkm_last_sel": (_I, [_VP, _VP, _U32]),
    "qkm_sel_device": (_VP, [_VP]),
    "qkm_h_device": (_VP, [_VP]),
    "qkm_expert_range": (None, [_VP, C.POINTER(_U32), C.POINTER(_U32)]),
    "qkm_gguf_open": (_VP, [C.c_char_p, C.c_char_p, _SZ]),
    "qkm_gguf_close": (None, [_VP]),
    "qkm_gguf_last_error": (C.c_char_p, [_VP]),
    "qkm_gguf_tensor_count": (_U64, [_VP]),
    "qkm_gguf_find": (_I, [_VP, C.c_char_p, C.POINTER(_U32), C.POINTER(_U64), C.POINTER(_VP), C.POINTER(_U64)]),
    "qkm_gguf_kv_u64": (_U64, [_VP, C.c_char_p, _U64]),
    "qkm_gguf_kv_str": (_I, [_VP, C.c_char_p, C.c_char_p, _SZ]),
    "qkm_gguf_moe_layer": (_I, [_VP, _U32, C.POINTER(Dims), C.POINTER(LayerWeights)]),
    "qkm_upload_layer_gguf": (_I, [_VP, _U32, _VP, _U32]),
    "qkm_dense_upload": (_I, [_VP, _U32, _U32, _VP, _U32, _U32]),
    "qkm_dense_gemm": (_I, [_VP, _U32, _VP, _U32, _VP]),
    "qkm_argmax": (_I, [_VP, _VP, _U32, _U32, _VP]),
    "qkm_add_rmsnorm": (_I, [_VP, _VP, _VP, _VP, _VP, _VP, _U32, _U32, C.c_float]),
    "qkm_add_rms3": (_I, [_VP, _VP, _VP, _VP, _VP, _VP, _VP, _U32, _U32, C.c_float]),
    "qkm_add_rms3_grouped": (_I, [_VP, _VP, _VP, _VP, _VP, _VP, _VP, _U32, _U32, _U32, C.c_float]),
    "qkm_moe_layer_step": (_I, [_VP, _U32, _VP, _VP, _VP, _VP, _U32, C.c_float, _VP, _VP]),
    "qkm_ep_dispatch": (_I, [_VP, _U32, _VP, _U32, _U32, _VP, _VP, _VP]),
    "qkm_ep_dispatch_dev": (_I, [_VP, _U32, _VP, _U32, _U32, _VP, _VP, _VP]),
    "qkm_ep_shared": (_I, [_VP, _U32, _VP, _U32]),
    "qkm_ep_expert_forward": (_I, [_VP, _U32, _VP, _VP, _U32, _VP]),
    "qkm_ep_combine": (_I, [_VP, _U32, _U32, _VP, _VP]),
    "qkm_ep_peer_setup": (_I, [_VP, _U32, _U32, _U32]),
    "qkm_ep_peer_buffers": (_I, [_VP, C.POINTER(C.c_void_p), C.POINTER(C.c_void_p), C.POINTER(C.c_void_p)]),
    "qkm_ep_peer_set": (_I, [_VP, _U32, _VP, _VP, _VP]),
    "qkm_ep_peer_export": (_I, [_VP, C.c_char_p]),
    "qkm_ep_peer_import": (_I, [_VP, _U32, C.c_char_p]),
    "qkm_ep_push": (_I, [_VP, _U32, _VP, _U32, _U32]),
    "qkm_ep_forward_slots": (_I, [_VP, _U32, _U32, _U32]),
    "qkm_ep_pull": (_I, [_VP, _U32, _U32, _VP]),
    "qkm_ep_barrier": (_I, [_VP, _U32]),
    "qkm_ep_peer_layer": (_I, [_VP, _U32, _VP, _U32, _U32, _VP, _U32]),
    "qkm_route_select_static": (_I, [_I, _VP, C.POINTER(Dims), _U32, _VP, _VP, _VP, _VP, _U32, C.c_char_p, _SZ]),
}

_lib = None


def load_library(path: str = LIB_PATH) -> C.CDLL:
    """dlopen libqkmoe.so and declare every entry point.  Raises if it is missing."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(path):
        raise RuntimeError(f"{path} not found: build it with `python qwen-kernel_b200/build.py` "
                           "(there is no CPU fallback)")
    lib = C.CDLL(path)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError if the library lacks a declared symbol
        fn.restype, fn.argtypes = res, args
    _lib = lib
    return lib


class QkmError(RuntimeError):
    def __init__(self, code, msg):
        super().__init__(f"qkm error {code}: {msg}")
        self.code = code


class DevBuf:
    """Device memory owned through the C ABI (no torch needed)."""

    def __init__(self, ctx: "Context", nbytes: int):
        self.ctx, self.nbytes = ctx, int(nbytes)
        self.ptr = ctx.lib.qkm_dev_alloc(ctx.h, max(self.nbytes, 1))
        if not self.ptr:
            raise QkmError(ERR_CUDA, ctx.last_error())

    def upload(self, arr: np.ndarray) -> "DevBuf":
        arr = np.ascontiguousarray(arr)
        assert arr.nbytes <= self.nbytes
        self.ctx.check(self.ctx.lib.qkm_h2d(self.ctx.h, self.ptr, arr.ctypes.data, arr.nbytes))
        return self

    def download(self, dtype, shape) -> np.ndarray:
        out = np.empty(shape, dtype)
        assert out.nbytes <= self.nbytes
        self.ctx.check(self.ctx.lib.qkm_d2h(self.ctx.h, out.ctypes.data, self.ptr, out.nbytes))
        return out

    def free(self):
        if self.ptr and self.ctx.h:
            self.ctx.lib.qkm_dev_free(self.ctx.h, self.ptr)
        self.ptr = None


def _p(x):
    """Device pointer of a DevBuf / torch tensor / int."""
    if x is None:
        return None
    if isinstance(x, DevBuf):
        return x.ptr
    if hasattr(x, "data_ptr"):
        return x.data_ptr()
    return int(x)


class Context:
    """One GPU context (one host thread; calls are asynchronous on its stream)."""

    def __init__(self, dims: synth.Dims = None, n_layer=1, max_tokens=16, device=-1, expert_first=0,
                 expert_count=0):
        self.lib = load_library()
        dims = dims or synth.Dims()
        self.dims = dims
        cfg = Config(Dims(dims.n_embd, dims.n_ff, dims.n_expert, dims.n_used), n_layer, max_tokens, device, 0,
                     expert_first, expert_count)
        err = C.create_string_buffer(512)
        self.h = self.lib.qkm_open(C.byref(cfg), err, len(err))
        if not self.h:
            raise QkmError(ERR_CUDA, err.value.decode())
        self.n_layer, self.max_tokens = n_layer, max_tokens
        self.layer_types = {}

    # -- plumbing
    def close(self):
        if self.h:
            self.lib.qkm_close(self.h)
            self.h = None

    def __enter__(self):
        return self

    def __exit__(self, *a):
        self.close()

    def last_error(self) -> str:
        return self.lib.qkm_last_error(self.h).decode()

    def check(self, rc: int) -> int:
        if rc < 0:
            raise QkmError(rc, self.last_error())
        return rc

    def set_stream(self, cuda_stream: int):
        self.check(self.lib.qkm_set_stream(self.h, cuda_stream))

    def sync(self):
        self.check(self.lib.qkm_sync(self.h))

    def launch_count(self) -> int:
        return int(self.lib.qkm_launch_count(self.h))

    def alloc(self, nbytes: int) -> DevBuf:
        return DevBuf(self, nbytes)

    def to_device(self, arr: np.ndarray) -> DevBuf:
        arr = np.ascontiguousarray(arr)
        return DevBuf(self, arr.nbytes).upload(arr)

    # -- weights
    def upload_layer(self, layer_idx: int, layer: synth.Layer):
        w = LayerWeights()
        w.router_type, w.gateup_type, w.down_type = layer.router_type, layer.gateup_type, layer.down_type
        (w.router, w.gate_inp_shexp, w.gate_exps, w.up_exps, w.down_exps, w.gate_shexp, w.up_shexp,
         w.down_shexp) = [t.ctypes.data for t in layer.tensors()]
        self.check(self.lib.qkm_upload_layer(self.h, layer_idx, C.byref(w)))
        self.layer_types[layer_idx] = (layer.router_type, layer.gateup_type, layer.down_type)

    def layer_ptrs(self, layer_idx: int) -> LayerWeights:
        w = LayerWeights()
        self.check(self.lib.qkm_layer_device_ptrs(self.h, layer_idx, C.byref(w)))
        return w

    # -- op level (device pointers)
    def moe_logits(self, router_type, router, x, logits, n):
        self.check(self.lib.qkm_moe_logits(self.h, router_type, _p(router), _p(x), _p(logits), n))

    def moe_select(self, logits, gis, x, sel, n):
        self.check(self.lib.qkm_moe_select(self.h, _p(logits), _p(gis), _p(x), _p(sel), n))

    def moe_route_select(self, router_type, router, gis, x, sel, n):
        self.check(self.lib.qkm_moe_route_select(self.h, router_type, _p(router), _p(gis), _p(x), _p(sel), n))

    def moe_group_pairs(self, sel, n, offsets, pairs):
        self.check(self.lib.qkm_moe_group_pairs(self.h, _p(sel), n, _p(offsets), _p(pairs)))

    def moe_gateup(self, ttype, gate, up, x, sel, h, n):
        self.check(self.lib.qkm_moe_gateup(self.h, ttype, _p(gate), _p(up), _p(x), _p(sel), _p(h), n))

    def moe_gateup_grouped(self, ttype, gate, up, x, offsets, pairs, h, n):
        self.check(self.lib.qkm_moe_gateup_grouped(self.h, ttype, _p(gate), _p(up), _p(x), _p(offsets),
                                                   _p(pairs), _p(h), n))

    def moe_shared_gateup(self, gate, up, x, h, n):
        self.check(self.lib.qkm_moe_shared_gateup(self.h, _p(gate), _p(up), _p(x), _p(h), n))

    def moe_down(self, ttype, down, h, sel, y, n):
        self.check(self.lib.qkm_moe_down(self.h, ttype, _p(down), _p(h), _p(sel), _p(y), n))

    def moe_down_grouped(self, ttype, down, h, sel, offsets, pairs, contrib, n):
        self.check(self.lib.qkm_moe_down_grouped(self.h, ttype, _p(down), _p(h), _p(sel), _p(offsets),
                                                 _p(pairs), _p(contrib), n))

    def moe_shared_down(self, down, h, sel, y2, n):
        self.check(self.lib.qkm_moe_shared_down(self.h, _p(down), _p(h), _p(sel), _p(y2), n))

    def gemv(self, ttype, W, x, y, M, K, n=1):
        self.check(self.lib.qkm_gemv(self.h, ttype, _p(W), _p(x), _p(y), M, K, n))

    def dequant(self, ttype, blocks, y, n_elems):
        self.check(self.lib.qkm_dequant(self.h, ttype, _p(blocks), _p(y), n_elems))

    # -- fused
    def moe_decode(self, layer_idx, x, n, y):
        self.check(self.lib.qkm_moe_decode(self.h, layer_idx, _p(x), n, _p(y)))

    def moe_prefill(self, layer_idx, x, n, y):
        self.check(self.lib.qkm_moe_prefill(self.h, layer_idx, _p(x), n, _p(y)))

    def moe_decode_stack(self, first, count, x, n, y):
        self.check(self.lib.qkm_moe_decode_stack(self.h, first, count, _p(x), n, _p(y)))

    def moe_decode_stack_host(self, first, count, x_host_ptr, n, y_host_ptr):
        """x/y: host addresses (ints) of [count][n][n_embd] f32, ideally pinned."""
        self.check(self.lib.qkm_moe_decode_stack_host(self.h, first, count, x_host_ptr, n, y_host_ptr))

    def moe_forward_host(self, layer_idx, x: np.ndarray, mode=0) -> np.ndarray:
        """Host in, host out (copies inside): the call an engine with host-resident
        activations makes.  mode 0 = decode path, 1 = prefill path."""
        x = np.ascontiguousarray(x, np.float32).reshape(-1, self.dims.n_embd)
        y = np.empty_like(x)
        self.check(self.lib.qkm_moe_forward_host(self.h, layer_idx, mode, x.ctypes.data, x.shape[0], y.ctypes.data))
        return y

    # -- dense quantised GEMM
    def dense_upload(self, slot, ttype, W: np.ndarray, M, K):
        W = np.ascontiguousarray(W)
        self.check(self.lib.qkm_dense_upload(self.h, slot, ttype, W.ctypes.data, M, K))

    def dense_gemm(self, slot, x, n, y):
        self.check(self.lib.qkm_dense_gemm(self.h, slot, _p(x), n, _p(y)))

    # -- layer entry / tail
    def add_rmsnorm(self, a, b, w, y, xn, n_rows, n, eps=1e-6):
        self.check(self.lib.qkm_add_rmsnorm(self.h, _p(a), _p(b), _p(w), _p(y), _p(xn), n_rows, n, eps))

    def add_rms3(self, a, b, c2, w, s, xn, n_rows, n, eps=1e-6):
        self.check(self.lib.qkm_add_rms3(self.h, _p(a), _p(b), _p(c2), _p(w), _p(s), _p(xn), n_rows, n, eps))

    def add_rms3_grouped(self, a, routed, c2, w, s, xn, n_rows, n, n_used, eps=1e-6):
        self.check(self.lib.qkm_add_rms3_grouped(self.h, _p(a), _p(routed), _p(c2), _p(w), _p(s), _p(xn), n_rows, n, n_used, eps))

    def argmax(self, logits, n_rows, n, tok):
        self.check(self.lib.qkm_argmax(self.h, _p(logits), n_rows, n, _p(tok)))

    def moe_layer_step(self, layer_idx, resid, attn_out, w_post, w_next, n, resid_out, xn_next, eps=1e-6):
        self.check(self.lib.qkm_moe_layer_step(self.h, layer_idx, _p(resid), _p(attn_out), _p(w_post), _p(w_next), n, eps,
                                               _p(resid_out), _p(xn_next)))

    # -- expert parallel (this context is one shard; see include/qk_moe.h)
    def ep_dispatch(self, layer_idx, x, n, n_ranks, xsend, selsend) -> list:
        """Routes the n local tokens and packs the rows each rank needs; returns rows per rank."""
        counts = (C.c_uint32 * n_ranks)()
        self.check(self.lib.qkm_ep_dispatch(self.h, layer_idx, _p(x), n, n_ranks, _p(xsend), _p(selsend), counts))
        return list(counts)

    def ep_dispatch_dev(self, layer_idx, x, n, n_ranks, xsend, selsend, counts_dev):
        """Asynchronous form: counts_dev is a device int32 tensor of n_ranks entries."""
        self.check(self.lib.qkm_ep_dispatch_dev(self.h, layer_idx, _p(x), n, n_ranks, _p(xsend), _p(selsend), _p(counts_dev)))

    def ep_shared(self, layer_idx, x, n):
        self.check(self.lib.qkm_ep_shared(self.h, layer_idx, _p(x), n))

    def ep_expert_forward(self, layer_idx, xrecv, selrecv, n_recv, partial):
        self.check(self.lib.qkm_ep_expert_forward(self.h, layer_idx, _p(xrecv), _p(selrecv), n_recv, _p(partial)))

    def ep_combine(self, n, n_ranks, back, y):
        self.check(self.lib.qkm_ep_combine(self.h, n, n_ranks, _p(back), _p(y)))

    # -- expert parallel over peer memory
    def ep_peer_setup(self, n_ranks, rank, slot_cap):
        self.check(self.lib.qkm_ep_peer_setup(self.h, n_ranks, rank, slot_cap))

    def ep_peer_buffers(self):
        """Device addresses (xrecv, selrecv, partial) of this rank's receive buffers."""
        p = [C.c_void_p() for _ in range(3)]
        self.check(self.lib.qkm_ep_peer_buffers(self.h, *[C.byref(v) for v in p]))
        return tuple(int(v.value) for v in p)

    def ep_peer_set(self, peer, xrecv, selrecv, partial):
        self.check(self.lib.qkm_ep_peer_set(self.h, peer, _p(xrecv), _p(selrecv), _p(partial)))

    def ep_peer_export(self) -> bytes:
        buf = C.create_string_buffer(EP_HANDLE_BYTES)
        self.check(self.lib.qkm_ep_peer_export(self.h, buf))
        return buf.raw

    def ep_peer_import(self, peer, handles: bytes):
        if len(handles) != EP_HANDLE_BYTES:
            raise ValueError(f"expected {EP_HANDLE_BYTES} bytes of handles, got {len(handles)}")
        self.check(self.lib.qkm_ep_peer_import(self.h, peer, handles))

    def ep_push(self, layer_idx, x, n, slot_rows):
        self.check(self.lib.qkm_ep_push(self.h, layer_idx, _p(x), n, slot_rows))

    def ep_forward_slots(self, layer_idx, slot_rows, n_shared=None):
        """n_shared=None: the shared expert was a separate ep_shared call; else this rank's token
        count, and the shared expert runs beside the resident ones (no ep_shared call)."""
        self.check(self.lib.qkm_ep_forward_slots(self.h, layer_idx, slot_rows, 0xFFFFFFFF if n_shared is None else n_shared))

    def ep_pull(self, n, slot_rows, y):
        self.check(self.lib.qkm_ep_pull(self.h, n, slot_rows, _p(y)))

    def ep_barrier(self, timeout_ms=2000):
        self.check(self.lib.qkm_ep_barrier(self.h, timeout_ms))

    def ep_peer_layer(self, layer_idx, x, n, slot_rows, y, timeout_ms=2000):
        self.check(self.lib.qkm_ep_peer_layer(self.h, layer_idx, _p(x), n, slot_rows, _p(y), timeout_ms))

    def profile_enable(self, on=True):
        self.check(self.lib.qkm_profile_enable(self.h, int(on)))

    def profile_read(self) -> dict:
        """Stage label -> milliseconds of the last fused call (synchronises)."""
        labels = C.create_string_buffer(16 * 16)
        ms = (C.c_float * 16)()
        n = self.check(self.lib.qkm_profile_read(self.h, labels, ms, 16))
        return {labels.raw[16 * i:16 * i + 16].split(b"\0")[0].decode(): float(ms[i]) for i in range(n)}

    def last_sel(self, n) -> np.ndarray:
        sel = np.zeros(n, SEL_DTYPE)
        self.check(self.lib.qkm_last_sel(self.h, sel.ctypes.data, n))
        return sel
