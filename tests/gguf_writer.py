"""A minimal GGUF v3 writer for tests: metadata (u32 / string / array-of-string entries) and
raw tensors, data section aligned as `general.alignment` says."""
import struct

import numpy as np

T_U32, T_STR, T_ARR = 4, 8, 9


def _s(b: bytes) -> bytes:
    return struct.pack("<Q", len(b)) + b


def write_gguf(path, kv: dict, tensors: list, alignment=32, version=3):
    """tensors: (name, ggml_type, ne tuple (ne0 fastest), uint8 array of raw bytes)."""
    out = bytearray(b"GGUF" + struct.pack("<IQQ", version, len(tensors), len(kv) + 1))
    out += _s(b"general.alignment") + struct.pack("<II", T_U32, alignment)
    for k, v in kv.items():
        out += _s(k.encode())
        if isinstance(v, str):
            out += struct.pack("<I", T_STR) + _s(v.encode())
        elif isinstance(v, list):
            out += struct.pack("<IIQ", T_ARR, T_STR, len(v)) + b"".join(_s(x.encode()) for x in v)
        else:
            out += struct.pack("<II", T_U32, int(v))
    offs, off = [], 0
    for _, _, _, data in tensors:
        offs.append(off)
        off = (off + data.nbytes + alignment - 1) // alignment * alignment
    for (name, ttype, ne, _), o in zip(tensors, offs):
        out += _s(name.encode()) + struct.pack("<I", len(ne)) + b"".join(struct.pack("<Q", n) for n in ne)
        out += struct.pack("<IQ", ttype, o)
    out += b"\0" * ((-len(out)) % alignment)
    base = len(out)
    for (_, _, _, data), o in zip(tensors, offs):
        out += b"\0" * (base + o - len(out))
        out += np.ascontiguousarray(data).tobytes()
    with open(path, "wb") as f:
        f.write(out)


def moe_layer_tensors(layer, index: int):
    """The eight blk.<index>.ffn_* tensors of a synth.Layer, shaped as llama.cpp writes them."""
    d = layer.dims
    p = f"blk.{index}."
    return [
        (p + "ffn_gate_inp.weight", layer.router_type, (d.n_embd, d.n_expert), layer.router),
        (p + "ffn_gate_inp_shexp.weight", 0, (d.n_embd,), layer.gate_inp_shexp),
        (p + "ffn_gate_exps.weight", layer.gateup_type, (d.n_embd, d.n_ff, d.n_expert), layer.gate_exps),
        (p + "ffn_up_exps.weight", layer.gateup_type, (d.n_embd, d.n_ff, d.n_expert), layer.up_exps),
        (p + "ffn_down_exps.weight", layer.down_type, (d.n_ff, d.n_embd, d.n_expert), layer.down_exps),
        (p + "ffn_gate_shexp.weight", 8, (d.n_embd, d.n_ff), layer.gate_shexp),
        (p + "ffn_up_shexp.weight", 8, (d.n_embd, d.n_ff), layer.up_shexp),
        (p + "ffn_down_shexp.weight", 8, (d.n_ff, d.n_embd), layer.down_shexp),
    ]
