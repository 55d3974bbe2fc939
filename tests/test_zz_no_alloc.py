"""The allocation-free router entry point against the context-based one.

qkm_route_select_static keeps its scratch in a fixed array inside the library instead of
memory taken from the driver.  It must select the same experts with the same weights as
qkm_moe_route_select, on repeated calls (the array is reused and never cleared), whether
or not other tests have used the device before.  This file sorts last on purpose.
"""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

MAX_LOGITS = 32768
MAX_EXPERTS = 512


@pytest.fixture(scope="module")
def ctx(pkg):
    c = pkg.Context(pkg.synth.Dims(), n_layer=1, max_tokens=128, device=0)
    yield c
    c.close()


def _static(pkg, dims, router_type, d_r, d_g, d_x, d_sel, n, device=0):
    from qwen_kernel_b200.binding import Dims
    lib = pkg.load_library()
    err = C.create_string_buffer(256)
    cd = Dims(dims.n_embd, dims.n_ff, dims.n_expert, dims.n_used)
    rc = lib.qkm_route_select_static(device, None, C.byref(cd), router_type, d_r.ptr, d_g.ptr, d_x.ptr,
                                     d_sel.ptr, n, err, 256)
    return rc, err.value.decode()


@pytest.mark.parametrize("router_type", [0, 1])
def test_static_matches_context_entry_point_twice(ctx, pkg, syn, router_type):
    from qwen_kernel_b200 import SEL_DTYPE
    dims = syn.Dims()
    layer = syn.make_layer(dims, seed=21, router_type=router_type)
    d_r, d_g = ctx.to_device(layer.router), ctx.to_device(layer.gate_inp_shexp)
    # two calls in a row with different inputs and token counts: the second reuses the
    # array the first left dirty
    for T, seed in ((128, 31), (37, 32)):
        x = syn.random_x(T, dims.n_embd, seed=seed)
        d_x = ctx.to_device(x)
        d_want, d_got = ctx.alloc(T * 160), ctx.alloc(T * 160)
        ctx.moe_route_select(router_type, d_r, d_g, d_x, d_want, T)
        want = d_want.download(SEL_DTYPE, T)
        rc, msg = _static(pkg, dims, router_type, d_r, d_g, d_x, d_got, T)
        assert rc == 0, msg
        got = d_got.download(SEL_DTYPE, T)
        assert np.array_equal(got["ids"], want["ids"])
        assert np.array_equal(got["w"].view(np.uint32), want["w"].view(np.uint32))
        assert np.array_equal(got["w_shared"].view(np.uint32), want["w_shared"].view(np.uint32))
        for b in (d_x, d_want, d_got):
            b.free()
    d_r.free(); d_g.free()


def test_static_takes_no_device_memory_and_keeps_the_device(ctx, pkg, syn):
    """What the entry point exists for: after its set-up call, a call takes no memory from
    the driver (free device memory is the same before and after, with the device idle at both
    readings) and leaves the caller's current device as it was."""
    import torch
    dims = syn.Dims()
    T = 32
    layer = syn.make_layer(dims, seed=23, router_type=syn.F16)
    x = syn.random_x(T, dims.n_embd, seed=34)
    d_r, d_g, d_x = ctx.to_device(layer.router), ctx.to_device(layer.gate_inp_shexp), ctx.to_device(x)
    d_sel = ctx.alloc(T * 160)
    rc, msg = _static(pkg, dims, syn.F16, d_r, d_g, d_x, d_sel, T)     # set-up call
    assert rc == 0, msg
    torch.cuda.synchronize(0)
    dev_before = torch.cuda.current_device()
    free_before, _ = torch.cuda.mem_get_info(0)
    for _ in range(3):
        rc, msg = _static(pkg, dims, syn.F16, d_r, d_g, d_x, d_sel, T)
        assert rc == 0, msg
    torch.cuda.synchronize(0)
    free_after, _ = torch.cuda.mem_get_info(0)
    assert free_after == free_before, (free_before, free_after)
    assert torch.cuda.current_device() == dev_before
    for b in (d_r, d_g, d_x, d_sel):
        b.free()


def test_static_wide_layer_takes_the_f32_path(pkg, syn, orc):
    """64 tokens x 512 experts: the f64 logits (256 KB) do not fit the static array, so this
    call ranks f32 logits and re-evaluates the boundary in f64 while the context call ranks f64
    logits outright.  Expert ids are still the f64 router's; weights agree to 1e-6."""
    from qwen_kernel_b200 import SEL_DTYPE
    dims = syn.Dims(n_embd=1024, n_ff=256, n_expert=512, n_used=10)
    T = 64
    rng = np.random.default_rng(3)
    router = (rng.standard_normal((512, 1024)) * 0.02).astype(np.float32)
    gis = (rng.standard_normal(1024) * 0.02).astype(np.float32)
    x = syn.random_x(T, dims.n_embd, seed=35)
    logits = x.astype(np.float64) @ router.astype(np.float64).T
    want_ids = np.argsort(-logits, axis=1, kind="stable")[:, :10]
    with pkg.Context(dims, n_layer=1, max_tokens=T, device=0) as c:
        d_r, d_g, d_x = c.to_device(router), c.to_device(gis), c.to_device(x)
        d_want, d_got = c.alloc(T * 160), c.alloc(T * 160)
        c.moe_route_select(0, d_r, d_g, d_x, d_want, T)
        want = d_want.download(SEL_DTYPE, T)
        rc, msg = _static(pkg, dims, 0, d_r, d_g, d_x, d_got, T)
        assert rc == 0, msg
        got = d_got.download(SEL_DTYPE, T)
        for b in (d_r, d_g, d_x, d_want, d_got):
            b.free()
    assert np.array_equal(want["ids"][:, :10], want_ids)
    assert np.array_equal(got["ids"], want["ids"])
    np.testing.assert_allclose(got["w"], want["w"], rtol=1e-6, atol=1e-9)
    np.testing.assert_allclose(got["w_shared"], want["w_shared"], rtol=1e-6)


def test_static_matches_oracle_ids(ctx, pkg, syn, orc):
    from qwen_kernel_b200 import SEL_DTYPE
    dims = syn.Dims()
    T = 16
    layer = syn.make_layer(dims, seed=22, router_type=syn.F32)
    x = syn.random_x(T, dims.n_embd, seed=33)
    want, _ = orc.route(layer, x)
    d_r, d_g, d_x = ctx.to_device(layer.router), ctx.to_device(layer.gate_inp_shexp), ctx.to_device(x)
    d_sel = ctx.alloc(T * 160)
    rc, msg = _static(pkg, dims, syn.F32, d_r, d_g, d_x, d_sel, T)
    assert rc == 0, msg
    assert np.array_equal(d_sel.download(SEL_DTYPE, T)["ids"], want["ids"])
    for b in (d_r, d_g, d_x, d_sel):
        b.free()


def test_static_rejects_sizes_beyond_the_array(ctx, pkg, syn):
    dims = syn.Dims()
    d = ctx.alloc(4096)
    too_many = MAX_LOGITS // dims.n_expert + 1
    rc, msg = _static(pkg, dims, 0, d, d, d, d, too_many)
    assert rc == -1 and "exceeds the static scratch" in msg
    wide = syn.Dims(n_expert=MAX_EXPERTS * 2)
    rc, msg = _static(pkg, wide, 0, d, d, d, d, 1)
    assert rc == -1 and "limits" in msg
    rc, msg = _static(pkg, dims, 8, d, d, d, d, 1)      # quantised router: not supported
    assert rc == -4
    rc, msg = _static(pkg, dims, 0, d, d, d, d, 1, device=999)
    assert rc == -1
    d.free()
