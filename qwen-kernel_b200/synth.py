"""Seeded synthetic ggml tensors and activations for the MoE path, plus the
byte/FLOP accounting used for roofline figures.

Real GGUF weights are not available to the tests and the bench, so every
tensor is generated from a seed with the distributions the reference's own
synthetic suite uses (src/main.cpp:637-767): uniformly random quant bytes and
an f16 block scale drawn from a small positive range.  Every byte pattern is a
valid block for all four quant formats.

Layouts are the raw ggml ones (src/quants.h:52-66, :107-119):
  Q8_0    34 B / 32:  d f16 | qs int8[32]
  Q6_K   210 B / 256: ql[128] | qh[64] | scales int8[16] | d f16
  IQ4_XS 136 B / 256: d f16 | scales_h u16 | scales_l[4] | qs[128]
  IQ3_XXS 98 B / 256: d f16 | qs[96] (64 grid indices, then 8 aux words)
"""
from __future__ import annotations

import zlib
from dataclasses import dataclass, field

import numpy as np

F32, F16, Q8_0, Q6_K, IQ3_XXS, IQ4_XS = 0, 1, 8, 14, 18, 23
TYPE_NAMES = {F32: "f32", F16: "f16", Q8_0: "q8_0", Q6_K: "q6_k", IQ3_XXS: "iq3_xxs", IQ4_XS: "iq4_xs"}
BLOCK = {F32: (1, 4), F16: (1, 2), Q8_0: (32, 34), Q6_K: (256, 210), IQ4_XS: (256, 136), IQ3_XXS: (256, 98)}


def row_bytes(ttype: int, ne0: int) -> int:
    """Bytes of one row of ne0 elements (ggmlRowBytes, src/gguf.h:36-46)."""
    elems, nbytes = BLOCK[ttype]
    assert ne0 % elems == 0
    return ne0 // elems * nbytes


def _rng(seed: int, *tags) -> np.random.Generator:
    h = zlib.crc32(repr(tags).encode()) & 0xFFFFFFFF
    return np.random.Generator(np.random.SFC64([seed & 0xFFFFFFFF, h]))


def _f16_scale(rng, n, lo, hi) -> np.ndarray:
    return rng.uniform(lo, hi, size=n).astype(np.float32).astype(np.float16).view(np.uint16)


def _put_u16(blocks: np.ndarray, off: int, vals: np.ndarray) -> None:
    blocks[:, off] = (vals & 0xFF).astype(np.uint8)
    blocks[:, off + 1] = (vals >> 8).astype(np.uint8)


def random_blocks(ttype: int, rows: int, k: int, seed: int, tag="w", scale=None) -> np.ndarray:
    """rows x k elements of `ttype` as a flat uint8 array of raw ggml bytes."""
    rng = _rng(seed, tag, ttype, rows, k)
    if ttype == F32:
        return (rng.standard_normal(rows * k, dtype=np.float32) * (scale or 0.02)).view(np.uint8)
    if ttype == F16:
        w = rng.standard_normal(rows * k, dtype=np.float32) * (scale or 0.05)
        return w.astype(np.float16).view(np.uint8)
    elems, nbytes = BLOCK[ttype]
    nb = rows * (k // elems)
    b = rng.integers(0, 256, size=(nb, nbytes), dtype=np.uint8)
    if ttype == Q8_0:
        lo, hi = scale or (1e-3, 1e-2)
        q = rng.integers(-127, 128, size=(nb, 32), dtype=np.int8)
        b[:, 2:] = q.view(np.uint8)
        _put_u16(b, 0, _f16_scale(rng, nb, lo, hi))
    elif ttype == Q6_K:
        lo, hi = scale or (2e-4, 1e-3)
        sc = rng.integers(-127, 128, size=(nb, 16), dtype=np.int8)
        b[:, 192:208] = sc.view(np.uint8)
        _put_u16(b, 208, _f16_scale(rng, nb, lo, hi))
    elif ttype in (IQ4_XS, IQ3_XXS):
        lo, hi = scale or (1e-3, 1e-2)
        _put_u16(b, 0, _f16_scale(rng, nb, lo, hi))
    else:
        raise ValueError(f"unsupported type {ttype}")
    return b.reshape(-1)


def random_x(n_tokens: int, k: int, seed: int, tag="x") -> np.ndarray:
    """f32 N(0,1) activation rows (randomX, src/main.cpp:619-625)."""
    return _rng(seed, tag, n_tokens, k).standard_normal((n_tokens, k), dtype=np.float32)


@dataclass
class Dims:
    n_embd: int = 2048
    n_ff: int = 512
    n_expert: int = 256
    n_used: int = 8


@dataclass
class Layer:
    """One layer's eight tensors as flat uint8 arrays (+ types)."""
    dims: Dims
    router_type: int
    gateup_type: int
    down_type: int
    router: np.ndarray
    gate_inp_shexp: np.ndarray  # f32 [n_embd]
    gate_exps: np.ndarray
    up_exps: np.ndarray
    down_exps: np.ndarray
    gate_shexp: np.ndarray
    up_shexp: np.ndarray
    down_shexp: np.ndarray
    expert_first: int = 0
    expert_count: int = 0  # 0 = all
    keep: list = field(default_factory=list)

    def tensors(self):
        return (self.router, self.gate_inp_shexp, self.gate_exps, self.up_exps, self.down_exps,
                self.gate_shexp, self.up_shexp, self.down_shexp)

    def expert_slice(self, first: int, count: int) -> "Layer":
        """The same layer holding only experts [first, first+count) (expert-parallel shard)."""
        d = self.dims
        gu = d.n_ff * row_bytes(self.gateup_type, d.n_embd)
        dn = d.n_embd * row_bytes(self.down_type, d.n_ff)
        return Layer(d, self.router_type, self.gateup_type, self.down_type, self.router,
                     self.gate_inp_shexp,
                     self.gate_exps[first * gu:(first + count) * gu],
                     self.up_exps[first * gu:(first + count) * gu],
                     self.down_exps[first * dn:(first + count) * dn],
                     self.gate_shexp, self.up_shexp, self.down_shexp, first, count)


def make_layer(dims: Dims, seed: int, layer: int = 0, router_type: int = F16,
               gateup_type: int = IQ3_XXS, down_type: int = IQ4_XS) -> Layer:
    """A seeded MoE layer.  Router ~N(0,0.02) (F16 as the bench configuration
    states, F32 as the reference engine loads it, src/main.cpp:1285); IQ3_XXS /
    IQ4_XS expert blocks with f16 scale ~U(1e-3,1e-2); Q8_0 shared expert."""
    d = dims
    s = seed * 1000003 + layer
    return Layer(
        d, router_type, gateup_type, down_type,
        router=random_blocks(router_type, d.n_expert, d.n_embd, s, "router", 0.02),
        gate_inp_shexp=random_blocks(F32, 1, d.n_embd, s, "gis", 0.02),
        gate_exps=random_blocks(gateup_type, d.n_expert * d.n_ff, d.n_embd, s, "ge"),
        up_exps=random_blocks(gateup_type, d.n_expert * d.n_ff, d.n_embd, s, "ue"),
        down_exps=random_blocks(down_type, d.n_expert * d.n_embd, d.n_ff, s, "de"),
        gate_shexp=random_blocks(Q8_0, d.n_ff, d.n_embd, s, "gs"),
        up_shexp=random_blocks(Q8_0, d.n_ff, d.n_embd, s, "us"),
        down_shexp=random_blocks(Q8_0, d.n_embd, d.n_ff, s, "ds"),
    )


# ---- accounting (weight bytes actually touched, as src/main.cpp:1238-1243 counts) ----

def layer_fixed_bytes(dims: Dims, router_type: int) -> int:
    """Router + shared-gate vector + the three shared-expert matrices."""
    d = dims
    return (d.n_expert * row_bytes(router_type, d.n_embd) + d.n_embd * 4 +
            2 * d.n_ff * row_bytes(Q8_0, d.n_embd) + d.n_embd * row_bytes(Q8_0, d.n_ff))


def expert_bytes(dims: Dims, gateup_type: int, down_type: int) -> int:
    d = dims
    return 2 * d.n_ff * row_bytes(gateup_type, d.n_embd) + d.n_embd * row_bytes(down_type, d.n_ff)


def layer_touched_bytes(dims: Dims, router_type: int, gateup_type: int, down_type: int,
                        n_distinct_experts: int) -> int:
    return layer_fixed_bytes(dims, router_type) + n_distinct_experts * expert_bytes(dims, gateup_type, down_type)


def flops_per_token(dims: Dims) -> int:
    """2*MACs of one token through one layer (router, shared gate dot, routed, shared)."""
    d = dims
    routed = d.n_used * (2 * 2 * d.n_ff * d.n_embd + 2 * d.n_embd * d.n_ff)
    shared = 2 * 2 * d.n_ff * d.n_embd + 2 * d.n_embd * d.n_ff
    router = 2 * d.n_expert * d.n_embd + 2 * d.n_embd
    return routed + shared + router


def gemv_bytes(ttype: int, m: int, k: int, n: int = 1) -> int:
    return m * row_bytes(ttype, k) + n * k * 4 + n * m * 4


# ---- error metrics ----

def rel_err_reference(got: np.ndarray, ref: np.ndarray) -> float:
    """The reference's scale-aware element error (src/main.cpp:548-560): each
    element is judged against max(|ref|, 1e-3, 1e-3*rms(ref))."""
    ref64 = ref.astype(np.float64).reshape(-1)
    rms = float(np.sqrt(np.mean(ref64 * ref64)))
    floor = max(1e-3, 1e-3 * rms)
    den = np.maximum(np.abs(ref64), floor)
    return float(np.max(np.abs(got.astype(np.float64).reshape(-1) - ref64) / den))


def rel_err_rows(got: np.ndarray, ref: np.ndarray) -> float:
    """Row-scaled relative error: |got-ref| / max(|ref|, rms(ref row)), max over
    all elements.  This is the "relative" figure the f32 (1e-5) and bf16 (2e-2)
    output tolerances are stated in."""
    g = got.astype(np.float64).reshape(ref.shape[0], -1) if ref.ndim > 1 else got.astype(np.float64).reshape(1, -1)
    r = ref.astype(np.float64).reshape(g.shape)
    rms = np.sqrt(np.mean(r * r, axis=1, keepdims=True))
    den = np.maximum(np.abs(r), np.maximum(rms, 1e-30))
    return float(np.max(np.abs(g - r) / den))
