"""The C-ABI library builds, loads, and exports every symbol include/qk_moe.h declares;
without a GPU it refuses to open instead of falling back to the CPU."""
import ctypes as C
import os
import re

import pytest

from conftest import ROOT, has_gpu


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "qk_moe.h")).read()
    return sorted(set(re.findall(r"QKM_API[^;(]*?\b(qkm_\w+)\s*\(", text)))


def test_header_symbols_are_exported(pkg):
    pkg.build()
    lib = C.CDLL(pkg.LIB_PATH)
    names = declared_symbols()
    assert len(names) >= 35
    missing = [n for n in names if not hasattr(lib, n)]
    assert not missing, missing
    # and the binding declares a signature for each of them
    assert sorted(pkg.SIGNATURES) == names


def test_row_bytes_and_version(pkg):
    lib = pkg.load_library()
    assert b"sm_100a" in lib.qkm_version()
    # ggmlRowBytes (reference src/gguf.h:36-46)
    for ttype, k, want in ((0, 2048, 8192), (1, 2048, 4096), (8, 2048, 2176), (14, 2048, 1680),
                           (23, 2048, 1088), (18, 2048, 784), (14, 512, 420), (8, 33, 0), (99, 256, 0)):
        assert lib.qkm_row_bytes(ttype, k) == want


def test_null_handle_calls_fail_cleanly(pkg):
    lib = pkg.load_library()
    assert lib.qkm_sync(None) == -1
    assert lib.qkm_moe_decode(None, 0, None, 1, None) == -1
    assert lib.qkm_n_embd(None) == 0
    assert lib.qkm_last_error(None) == b"NULL context"
    lib.qkm_close(None)  # no-op


@pytest.mark.skipif(has_gpu(), reason="checks the no-GPU behaviour")
def test_open_without_gpu_fails_loudly(pkg):
    with pytest.raises(pkg.QkmError) as ei:
        pkg.Context(pkg.synth.Dims(), n_layer=1, max_tokens=1)
    assert "no CUDA device" in str(ei.value) or "CPU path" in str(ei.value)


def test_open_rejects_bad_config(pkg):
    lib = pkg.load_library()
    from qwen_kernel_b200.binding import Config, Dims
    err = C.create_string_buffer(256)
    for dims in ((2048, 512, 600, 8), (2048, 500, 256, 8), (2000, 512, 256, 8), (2048, 512, 256, 17), (2048, 512, 4, 8)):
        cfg = Config(Dims(*dims), 1, 1, -1, 0, 0, 0)
        assert not lib.qkm_open(C.byref(cfg), err, 256)
        assert b"unsupported dims" in err.value
    assert not lib.qkm_open(None, err, 256)
