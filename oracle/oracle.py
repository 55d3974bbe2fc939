"""ctypes front end of the CPU oracle (oracle/qkm_oracle.cpp) and, where it was
built, of the reference's own dequantisers (oracle/_ref/libqk_ref.so).

TEST INFRASTRUCTURE ONLY.  Importers: tests/, __graft_entry__.smoke() and the
cpu_baseline / reference legs of bench.py.  The product package never imports
this module.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ACC_F64, ACC_F32 = 0, 1


class Dims(C.Structure):
    _fields_ = [("n_embd", C.c_uint32), ("n_ff", C.c_uint32), ("n_expert", C.c_uint32), ("n_used", C.c_uint32)]


class LayerWeights(C.Structure):
    _fields_ = [("router_type", C.c_uint32), ("gateup_type", C.c_uint32), ("down_type", C.c_uint32),
                ("reserved", C.c_uint32), ("router", C.c_void_p), ("gate_inp_shexp", C.c_void_p),
                ("gate_exps", C.c_void_p), ("up_exps", C.c_void_p), ("down_exps", C.c_void_p),
                ("gate_shexp", C.c_void_p), ("up_shexp", C.c_void_p), ("down_shexp", C.c_void_p)]


SEL_DTYPE = np.dtype([("ids", np.uint32, 16), ("w", np.float32, 16), ("w_shared", np.float32),
                      ("route_done", np.uint32), ("pad", np.float32, 6)])
assert SEL_DTYPE.itemsize == 160


def build(ref: bool = True) -> None:
    """Compile the oracle (and oracle/_ref when the reference tree is present)."""
    targets = ["all"] + (["ref"] if ref else [])
    subprocess.run(["make", "-s", "-C", HERE] + targets, check=True, stdout=subprocess.DEVNULL)


def _ptr(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


class Oracle:
    def __init__(self):
        path = os.path.join(HERE, "libqkm_oracle.so")
        if not os.path.exists(path):
            build(ref=False)
        self.lib = L = C.CDLL(path)
        L.orc_f16_to_f32.restype = C.c_float
        L.orc_f16_to_f32.argtypes = [C.c_uint16]
        L.orc_f32_to_f16.restype = C.c_uint16
        L.orc_f32_to_f16.argtypes = [C.c_float]
        L.orc_row_bytes.restype = C.c_size_t
        L.orc_row_bytes.argtypes = [C.c_uint32, C.c_uint64]
        L.orc_signs8.restype = C.c_uint8
        L.orc_signs8.argtypes = [C.c_uint32]
        L.orc_f16_to_f32_n.argtypes = [C.c_void_p, C.c_void_p, C.c_uint64]
        L.orc_f32_to_f16_n.argtypes = [C.c_void_p, C.c_void_p, C.c_uint64]
        L.orc_dequant_row.argtypes = [C.c_uint32, C.c_void_p, C.c_void_p, C.c_int64]
        L.orc_gemv.argtypes = [C.c_uint32, C.c_void_p, C.c_void_p, C.c_void_p, C.c_uint32, C.c_uint32,
                               C.c_uint32, C.c_int, C.c_int]
        L.orc_moe_route.argtypes = [C.POINTER(Dims), C.c_uint32, C.c_void_p, C.c_void_p, C.c_void_p,
                                    C.c_uint32, C.c_void_p, C.c_void_p, C.c_int]
        L.orc_moe_logits.argtypes = [C.POINTER(Dims), C.c_uint32, C.c_void_p, C.c_void_p, C.c_uint32,
                                     C.c_void_p, C.c_int]
        L.orc_select_f32.argtypes = [C.POINTER(Dims), C.c_void_p, C.c_void_p, C.c_void_p, C.c_uint32, C.c_void_p]
        L.orc_group_pairs.argtypes = [C.c_void_p, C.c_uint32, C.c_uint32, C.c_uint32, C.c_void_p, C.c_void_p]
        L.orc_moe_layer.argtypes = [C.POINTER(Dims), C.POINTER(LayerWeights), C.c_void_p, C.c_uint32,
                                    C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                                    C.c_uint32, C.c_uint32, C.c_int, C.c_int, C.c_int]
        L.orc_hardware_threads.restype = C.c_int

    # -- scalar helpers
    def f16_to_f32(self, h: np.ndarray) -> np.ndarray:
        h = np.ascontiguousarray(h, dtype=np.uint16)
        out = np.empty(h.shape, np.float32)
        self.lib.orc_f16_to_f32_n(_ptr(h), _ptr(out), h.size)
        return out

    def f32_to_f16(self, f: np.ndarray) -> np.ndarray:
        f = np.ascontiguousarray(f, dtype=np.float32)
        out = np.empty(f.shape, np.uint16)
        self.lib.orc_f32_to_f16_n(_ptr(f), _ptr(out), f.size)
        return out

    def hardware_threads(self) -> int:
        return int(self.lib.orc_hardware_threads())

    # -- dequant / gemv
    def dequant(self, ttype: int, blocks: np.ndarray, n_elems: int) -> np.ndarray:
        out = np.empty(n_elems, np.float32)
        rc = self.lib.orc_dequant_row(ttype, _ptr(blocks), _ptr(out), n_elems)
        assert rc == 0, rc
        return out

    def gemv(self, ttype, W, x, M, K, acc=ACC_F64, threads=1) -> np.ndarray:
        x = np.ascontiguousarray(x, np.float32).reshape(-1, K)
        y = np.empty((x.shape[0], M), np.float32)
        rc = self.lib.orc_gemv(ttype, _ptr(W), _ptr(x), _ptr(y), M, K, x.shape[0], acc, threads)
        assert rc == 0, rc
        return y

    # -- MoE
    @staticmethod
    def _dims(d) -> Dims:
        return Dims(d.n_embd, d.n_ff, d.n_expert, d.n_used)

    @staticmethod
    def _weights(layer) -> LayerWeights:
        w = LayerWeights()
        w.router_type, w.gateup_type, w.down_type = layer.router_type, layer.gateup_type, layer.down_type
        (w.router, w.gate_inp_shexp, w.gate_exps, w.up_exps, w.down_exps, w.gate_shexp, w.up_shexp,
         w.down_shexp) = [t.ctypes.data for t in layer.tensors()]
        return w

    def route(self, layer, x, threads=1):
        d = layer.dims
        x = np.ascontiguousarray(x, np.float32).reshape(-1, d.n_embd)
        T = x.shape[0]
        sel = np.zeros(T, SEL_DTYPE)
        w64 = np.zeros((T, 17), np.float64)
        dd = self._dims(d)
        self.lib.orc_moe_route(C.byref(dd), layer.router_type, _ptr(layer.router), _ptr(layer.gate_inp_shexp),
                               _ptr(x), T, _ptr(sel), _ptr(w64), threads)
        return sel, w64

    def logits(self, layer, x, acc=ACC_F64) -> np.ndarray:
        d = layer.dims
        x = np.ascontiguousarray(x, np.float32).reshape(-1, d.n_embd)
        out = np.empty((x.shape[0], d.n_expert), np.float32)
        dd = self._dims(d)
        self.lib.orc_moe_logits(C.byref(dd), layer.router_type, _ptr(layer.router), _ptr(x), x.shape[0],
                                _ptr(out), acc)
        return out

    def select_f32(self, dims, logits, gis, x):
        x = np.ascontiguousarray(x, np.float32).reshape(-1, dims.n_embd)
        logits = np.ascontiguousarray(logits, np.float32)
        sel = np.zeros(x.shape[0], SEL_DTYPE)
        dd = self._dims(dims)
        self.lib.orc_select_f32(C.byref(dd), _ptr(logits), _ptr(gis), _ptr(x), x.shape[0], _ptr(sel))
        return sel

    def group_pairs(self, sel, n_expert, n_used):
        T = sel.shape[0]
        offsets = np.zeros(n_expert + 1, np.uint32)
        pairs = np.zeros(T * n_used, np.uint32)
        self.lib.orc_group_pairs(_ptr(sel), T, n_expert, n_used, _ptr(offsets), _ptr(pairs))
        return offsets, pairs

    def moe_layer(self, layer, x, acc=ACC_F64, threads=1, sel_in=None, want_h=False, want_contrib=False,
                  with_shared=True):
        """Returns dict(y, sel, h?, contrib?).  `layer` may be an expert-parallel
        slice (layer.expert_count > 0): only resident experts contribute."""
        d = layer.dims
        x = np.ascontiguousarray(x, np.float32).reshape(-1, d.n_embd)
        T = x.shape[0]
        y = np.zeros((T, d.n_embd), np.float32)
        sel = np.zeros(T, SEL_DTYPE)
        h = np.zeros((T, d.n_used + 1, d.n_ff), np.float32) if want_h else None
        contrib = np.zeros((T, d.n_used, d.n_embd), np.float32) if want_contrib else None
        dd, w = self._dims(d), self._weights(layer)
        rc = self.lib.orc_moe_layer(C.byref(dd), C.byref(w), _ptr(x), T, _ptr(y), _ptr(sel), _ptr(h),
                                    _ptr(contrib), _ptr(sel_in), layer.expert_first, layer.expert_count,
                                    int(with_shared), acc, threads)
        assert rc == 0, rc
        out = {"y": y, "sel": sel}
        if want_h:
            out["h"] = h
        if want_contrib:
            out["contrib"] = contrib
        return out


def _add_rms(self, mode, a, b, c2, w, n_used=0, eps=1e-6):
    a = np.ascontiguousarray(a, np.float32)
    n_rows, n = a.shape
    s, xn = np.empty_like(a), np.empty_like(a)
    b = np.ascontiguousarray(b, np.float32)
    c2 = None if c2 is None else np.ascontiguousarray(c2, np.float32)
    w = np.ascontiguousarray(w, np.float32)
    self.lib.orc_add_rms.argtypes = [C.c_int] + [C.c_void_p] * 6 + [C.c_uint32] * 3 + [C.c_float]
    rc = self.lib.orc_add_rms(mode, _ptr(a), _ptr(b), _ptr(c2), _ptr(w), _ptr(s), _ptr(xn), n_rows, n, n_used, eps)
    assert rc == 0
    return s, xn


Oracle.add_rms = _add_rms


class Reference:
    """The reference's own src/quants.h functions (oracle/_ref/libqk_ref.so)."""

    PATH = os.path.join(HERE, "_ref", "libqk_ref.so")

    @classmethod
    def available(cls) -> bool:
        return os.path.exists(cls.PATH)

    def __init__(self):
        self.lib = L = C.CDLL(self.PATH)
        L.ref_f16_to_f32_n.argtypes = [C.c_void_p, C.c_void_p, C.c_uint64]
        L.ref_f32_to_f16_n.argtypes = [C.c_void_p, C.c_void_p, C.c_uint64]
        L.ref_dequant_row.argtypes = [C.c_uint32, C.c_void_p, C.c_void_p, C.c_int64]
        L.ref_grid.restype = C.c_uint32
        L.ref_ksigns.restype = C.c_uint8
        L.ref_kvalues.restype = C.c_int8
        L.ref_block_bytes.restype = C.c_uint32

    def f16_to_f32(self, h):
        h = np.ascontiguousarray(h, dtype=np.uint16)
        out = np.empty(h.shape, np.float32)
        self.lib.ref_f16_to_f32_n(_ptr(h), _ptr(out), h.size)
        return out

    def f32_to_f16(self, f):
        f = np.ascontiguousarray(f, dtype=np.float32)
        out = np.empty(f.shape, np.uint16)
        self.lib.ref_f32_to_f16_n(_ptr(f), _ptr(out), f.size)
        return out

    def dequant(self, ttype, blocks, n_elems):
        out = np.empty(n_elems, np.float32)
        rc = self.lib.ref_dequant_row(ttype, _ptr(blocks), _ptr(out), n_elems)
        assert rc == 0, rc
        return out


class ReferenceLayer:
    """The reference's own CPU layer loop, `moeCpuRef` (src/main.cpp:1316-1387), compiled from
    the span oracle/Makefile cuts out of the reference's source (oracle/_ref/libqk_ref_layer.so).
    It accepts what `loadMoeT` accepts: F32 router and shared gate, IQ3_XXS / IQ4_XS gate/up,
    IQ4_XS / Q6_K down, Q8_0 shared expert.  Single-threaded, one token at a time."""

    PATH = os.path.join(HERE, "_ref", "libqk_ref_layer.so")

    @classmethod
    def available(cls) -> bool:
        return os.path.exists(cls.PATH)

    def __init__(self):
        self.lib = L = C.CDLL(self.PATH)
        L.ref_moe_layer.argtypes = [C.c_uint32] * 6 + [C.c_void_p] * 9 + [C.c_uint32] + [C.c_void_p] * 4

    def moe_layer(self, layer, x):
        """Returns dict(y f32 [T][n_embd], ids u32 [T][16], w f64 [T][16], w_shared f64 [T])."""
        d = layer.dims
        assert layer.router_type == 0, "the reference's loader accepts an F32 router only"
        x = np.ascontiguousarray(x, np.float32).reshape(-1, d.n_embd)
        T = x.shape[0]
        y = np.zeros((T, d.n_embd), np.float32)
        ids = np.zeros((T, 16), np.uint32)
        w = np.zeros((T, 16), np.float64)
        ws = np.zeros(T, np.float64)
        t = layer.tensors()
        rc = self.lib.ref_moe_layer(d.n_embd, d.n_ff, d.n_expert, d.n_used, layer.gateup_type, layer.down_type,
                                    *[_ptr(a) for a in t], _ptr(x), T, _ptr(y), _ptr(ids), _ptr(w), _ptr(ws))
        assert rc == 0, rc
        return {"y": y, "ids": ids, "w": w, "w_shared": ws}
