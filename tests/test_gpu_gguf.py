"""Weights taken from a GGUF file give the same results as the same blocks uploaded directly
(bit-identical: the bytes are the same), for a whole layer and for an expert-parallel shard."""
import ctypes as C

import numpy as np
import pytest

from gguf_writer import moe_layer_tensors, write_gguf

pytestmark = pytest.mark.gpu


def test_layer_from_gguf_equals_direct_upload(pkg, syn, tmp_path):
    dims = syn.Dims()
    layers = [syn.make_layer(dims, seed=91, layer=l) for l in range(2)]
    path = tmp_path / "two_layers.gguf"
    write_gguf(path, {"general.architecture": "qwen3moe", "qwen3moe.expert_used_count": dims.n_used},
               moe_layer_tensors(layers[0], 0) + moe_layer_tensors(layers[1], 1))
    lib = pkg.load_library()
    err = C.create_string_buffer(256)
    g = lib.qkm_gguf_open(str(path).encode(), err, 256)
    assert g, err.value
    x = syn.random_x(16, dims.n_embd, seed=92)
    with pkg.Context(dims, n_layer=2, max_tokens=16, device=0) as a, pkg.Context(dims, n_layer=2, max_tokens=16, device=0) as b:
        for l in range(2):
            a.upload_layer(l, layers[l])
            assert lib.qkm_upload_layer_gguf(b.h, l, g, l) == 0, lib.qkm_gguf_last_error(g)
        for l in range(2):
            assert np.array_equal(a.moe_forward_host(l, x), b.moe_forward_host(l, x))
        # a layer the file does not have, and a context of other dimensions
        assert lib.qkm_upload_layer_gguf(b.h, 0, g, 5) == -3
    with pkg.Context(syn.Dims(n_expert=128), n_layer=1, max_tokens=4, device=0) as c:
        assert lib.qkm_upload_layer_gguf(c.h, 0, g, 0) == -3
        assert b"differ" in lib.qkm_gguf_last_error(g)
    # an expert-parallel shard takes its slice of the expert tensors
    per = dims.n_expert // 4
    with pkg.Context(dims, n_layer=1, max_tokens=16, device=0, expert_first=2 * per, expert_count=per) as s1, \
            pkg.Context(dims, n_layer=1, max_tokens=16, device=0, expert_first=2 * per, expert_count=per) as s2:
        s1.upload_layer(0, layers[0].expert_slice(2 * per, per))
        assert lib.qkm_upload_layer_gguf(s2.h, 0, g, 0) == 0
        assert np.array_equal(s1.moe_forward_host(0, x), s2.moe_forward_host(0, x))
    lib.qkm_gguf_close(g)
