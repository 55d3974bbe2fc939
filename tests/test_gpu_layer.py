"""Whole-layer parity through the fused C-ABI calls, against the oracle and the golden
fixtures: ids positional-exact, weights 1e-4 (the reference's gate, src/main.cpp:1191-1194)
and tighter, outputs 1e-5 (f32 decode path) row-scaled relative, argmax of every output
row unchanged."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

TOL_F32 = 1e-5


def check_layer(syn, got_y, got_sel, ref, n_used, tol=TOL_F32):
    assert np.array_equal(got_sel["ids"][:, :n_used], ref["sel"]["ids"][:, :n_used])
    np.testing.assert_allclose(got_sel["w"][:, :n_used], ref["sel"]["w"][:, :n_used], rtol=1e-5, atol=1e-7)
    np.testing.assert_allclose(got_sel["w_shared"], ref["sel"]["w_shared"], rtol=1e-6)
    assert syn.rel_err_rows(got_y, ref["y"]) < tol
    assert syn.rel_err_reference(got_y, ref["y"]) < 1e-2
    assert np.array_equal(np.argmax(got_y, axis=1), np.argmax(ref["y"], axis=1))


@pytest.mark.parametrize("tag", ["a", "b", "c"])
def test_golden_small_layer(pkg, syn, golden, tag):
    g = golden(f"moe_small_{tag}.npz")
    rt, gt, dt = (int(v) for v in g["types"])
    dims = syn.Dims(*(int(v) for v in g["dims"]))
    layer = syn.make_layer(dims, seed=1234, layer=3, router_type=rt, gateup_type=gt, down_type=dt)
    with pkg.Context(dims, n_layer=1, max_tokens=4, device=0) as ctx:
        ctx.upload_layer(0, layer)
        for mode in (0, 1):
            y = ctx.moe_forward_host(0, g["x"], mode=mode)
            sel = ctx.last_sel(3)
            assert np.array_equal(sel["ids"], g["ids"])
            np.testing.assert_allclose(sel["w"], g["w"], rtol=1e-5, atol=1e-7)
            assert syn.rel_err_rows(y, g["y"]) < (TOL_F32 if mode == 0 else 2e-2)


@pytest.mark.parametrize("router_type,gt,dt", [(1, 18, 23), (0, 18, 14), (0, 23, 23)])
@pytest.mark.parametrize("T", [1, 5])
def test_decode_full_size_layer(pkg, orc, syn, router_type, gt, dt, T):
    """Bench configuration 0: 2048 / 512 / 256 experts / top-8."""
    dims = syn.Dims()
    layer = syn.make_layer(dims, seed=42, router_type=router_type, gateup_type=gt, down_type=dt)
    x = syn.random_x(T, dims.n_embd, seed=43)
    ref = orc.moe_layer(layer, x, threads=8)
    with pkg.Context(dims, n_layer=1, max_tokens=8, device=0) as ctx:
        ctx.upload_layer(0, layer)
        y = ctx.moe_forward_host(0, x, mode=0)
        check_layer(syn, y, ctx.last_sel(T), ref, 8)
        # determinism: a second run is bit-identical
        y2 = ctx.moe_forward_host(0, x, mode=0)
        assert np.array_equal(y, y2)


@pytest.mark.parametrize("T", [16, 64])
def test_decode_full_size_layer_batches(pkg, orc, syn, T):
    """The bench batch (16 slots) and the largest decode-sized batch (64 tokens: the last one on
    the streaming kernels; 65 is the first on the tensor cores, tests/test_gpu_prefill.py)."""
    dims = syn.Dims()
    layer = syn.make_layer(dims, seed=42)
    x = syn.random_x(T, dims.n_embd, seed=47)
    ref = orc.moe_layer(layer, x, threads=orc.hardware_threads())
    with pkg.Context(dims, n_layer=1, max_tokens=T, device=0) as ctx:
        ctx.upload_layer(0, layer)
        y = ctx.moe_forward_host(0, x, mode=0)
        check_layer(syn, y, ctx.last_sel(T), ref, 8)
        assert np.array_equal(y, ctx.moe_forward_host(0, x, mode=0))


@pytest.mark.parametrize("gt,dt", [(18, 14), (23, 23), (23, 14)])
@pytest.mark.parametrize("T", [3, 16, 64])
def test_decode_other_type_mixes_batches(pkg, orc, syn, T, gt, dt):
    """Layers whose routed down tensor is Q6_K (14) and / or whose gate/up tensors are IQ4_XS (23)
    take the fused decode sequence too, with the Q6_K form of the down kernel and the IQ4_XS form of
    the gate/up kernel (integer tensor-core arithmetic on their tiles): the decode tolerance holds,
    a row with a NaN stays confined to its token, and a second call is bit-identical."""
    dims = syn.Dims()
    layer = syn.make_layer(dims, seed=44, gateup_type=gt, down_type=dt)
    x = syn.random_x(T, dims.n_embd, seed=48)
    x[T // 2] *= 1e-3
    if T > 3:
        x[1, 7] = np.nan
    ref = orc.moe_layer(layer, x, threads=orc.hardware_threads())
    with pkg.Context(dims, n_layer=1, max_tokens=T, device=0) as ctx:
        ctx.upload_layer(0, layer)
        y = ctx.moe_forward_host(0, x, mode=0)
        sel = ctx.last_sel(T)
        assert np.array_equal(sel["ids"][:, :8], ref["sel"]["ids"][:, :8])
        ok = np.isfinite(x).all(axis=1)
        assert syn.rel_err_rows(y[ok], ref["y"][ok]) < TOL_F32
        assert np.isnan(y[~ok]).all()
        assert np.array_equal(y, ctx.moe_forward_host(0, x, mode=0), equal_nan=True)


@pytest.mark.parametrize("router_type", [0, 1])
def test_decode_router_ties_and_nonfinite(pkg, orc, syn, router_type):
    """The fused decode router (logits + ranking + grouping in one launch) on the hazards the
    reference's selection rules cover: identical router rows (lowest id wins), all-zero rows,
    NaN / Inf activations (logits at the floor: ids 0..7), an all-zero token.  Ids must equal the
    f64 router's; finite tokens' outputs stay within the decode tolerance, and a second call is
    bit-identical (the last-arriving block's ranking is deterministic)."""
    dims = syn.Dims()
    layer = syn.make_layer(dims, seed=9, router_type=router_type)
    if router_type == syn.F32:
        r = layer.router.view(np.float32).reshape(256, 2048).copy()
    else:
        r = layer.router.view(np.float16).reshape(256, 2048).copy()
    r[200] = r[17]; r[90] = r[17]            # three identical rows: exact ties
    r[3] = 0; r[4] = 0                       # two all-zero rows: logits exactly 0
    layer.router = r.reshape(-1).view(np.uint8)
    T = 12
    x = syn.random_x(T, 2048, seed=10)
    x[2] = r[17].astype(np.float32) * 50.0    # make the tied experts win for token 2
    x[5, 100] = np.nan                        # every logit NaN
    x[6, 7] = np.inf                          # logits +-inf / NaN
    x[7] = 0.0                                # every logit 0: ids 0..7
    x[T - 1] = x[2]
    want, w64 = orc.route(layer, x)
    finite = np.array([t for t in range(T) if t not in (5, 6)])
    ref = orc.moe_layer(layer, x[finite], threads=orc.hardware_threads())
    with pkg.Context(dims, n_layer=1, max_tokens=T, device=0) as ctx:
        ctx.upload_layer(0, layer)
        y = ctx.moe_forward_host(0, x, mode=0)
        sel = ctx.last_sel(T)
        y2 = ctx.moe_forward_host(0, x, mode=0)
        sel2 = ctx.last_sel(T)
    assert np.array_equal(sel["ids"][:, :8], want["ids"][:, :8])
    assert list(sel["ids"][2, :3]) == [17, 90, 200] and list(sel["ids"][T - 1, :3]) == [17, 90, 200]
    assert list(sel["ids"][5, :8]) == list(range(8)) and list(sel["ids"][7, :8]) == list(range(8))
    ok = np.isfinite(w64[:, :8]).all(axis=1)
    np.testing.assert_allclose(sel["w"][ok, :8], w64[ok, :8], rtol=1e-5, atol=1e-7)
    assert syn.rel_err_rows(y[finite], ref["y"]) < TOL_F32
    assert np.array_equal(sel["ids"], sel2["ids"]) and np.array_equal(y[finite], y2[finite])


@pytest.mark.parametrize("T", [3, 33])
def test_decode_512_experts(pkg, orc, syn, T):
    """More than 256 experts: the ranking keeps two sorted key lists per lane (the 512-expert
    variant of the model family); narrower rows (n_embd 1024: four column blocks per team)."""
    dims = syn.Dims(n_embd=1024, n_ff=512, n_expert=512, n_used=8)
    layer = syn.make_layer(dims, seed=14, router_type=syn.F32)
    x = syn.random_x(T, dims.n_embd, seed=15)
    ref = orc.moe_layer(layer, x, threads=orc.hardware_threads())
    with pkg.Context(dims, n_layer=1, max_tokens=T, device=0) as ctx:
        ctx.upload_layer(0, layer)
        y = ctx.moe_forward_host(0, x, mode=0)
        check_layer(syn, y, ctx.last_sel(T), ref, 8)
        assert np.array_equal(y, ctx.moe_forward_host(0, x, mode=0))


def test_decode_router_is_deterministic_over_many_calls(pkg, orc, syn):
    """200 calls of the fused decode sequence on the same 16 rows: ids, weights and outputs are the
    same bits every time (a last-arriving block ranks the logits; the reference removed such a
    fusion on one backend because relaxed atomics made it non-deterministic)."""
    dims = syn.Dims()
    layer = syn.make_layer(dims, seed=12)
    x = syn.random_x(16, dims.n_embd, seed=13)
    want, _ = orc.route(layer, x, threads=orc.hardware_threads())
    with pkg.Context(dims, n_layer=1, max_tokens=16, device=0) as ctx:
        ctx.upload_layer(0, layer)
        d_x, d_y = ctx.to_device(x), ctx.alloc(x.nbytes)
        ctx.moe_decode(0, d_x, 16, d_y)
        y0, s0 = d_y.download(np.float32, x.shape), ctx.last_sel(16)
        assert np.array_equal(s0["ids"][:, :8], want["ids"][:, :8])
        for _ in range(200):
            ctx.moe_decode(0, d_x, 16, d_y)
        y1, s1 = d_y.download(np.float32, x.shape), ctx.last_sel(16)
        for i in range(50):
            ctx.moe_decode(0, d_x, 16, d_y)
            if i % 10 == 0:
                s = ctx.last_sel(16)
                assert np.array_equal(s["ids"], s0["ids"]) and np.array_equal(s["w"].view(np.uint32), s0["w"].view(np.uint32))
    assert np.array_equal(s1["ids"], s0["ids"]) and np.array_equal(y1, y0)


def test_decode_stack_and_errors(pkg, orc, syn):
    dims = syn.Dims(n_embd=512, n_ff=256, n_expert=16, n_used=4)
    T, L = 6, 3
    layers = [syn.make_layer(dims, seed=50, layer=l) for l in range(L)]
    x = np.stack([syn.random_x(T, dims.n_embd, seed=60 + l) for l in range(L)])
    with pkg.Context(dims, n_layer=L, max_tokens=T, device=0) as ctx:
        with pytest.raises(pkg.QkmError) as ei:      # nothing uploaded yet
            ctx.moe_forward_host(0, x[0])
        assert ei.value.code == -2
        for l in range(L):
            ctx.upload_layer(l, layers[l])
        d_x, d_y = ctx.to_device(x), ctx.alloc(x.nbytes)
        ctx.moe_decode_stack(0, L, d_x, T, d_y)
        y = d_y.download(np.float32, x.shape)
        for l in range(L):
            ref = orc.moe_layer(layers[l], x[l])
            assert syn.rel_err_rows(y[l], ref["y"]) < TOL_F32
        with pytest.raises(pkg.QkmError) as ei:      # more tokens than the context was opened for
            ctx.moe_decode(0, d_x, T + 1, d_y)
        assert ei.value.code == -3
        with pytest.raises(pkg.QkmError):
            ctx.moe_decode(L, d_x, 1, d_y)
        assert ctx.launch_count() > 0


def test_decode_stack_host_buffers_in_chunks(pkg, orc, syn):
    """The host-buffer form of the stack (copies inside): nine layers run as chunks of layers, each
    its own graph, with the copies on their own streams; three layers take the plain form.  Both equal
    the layer-by-layer calls bit for bit, on a repeated call (graphs replayed) and after a call with
    another token count and with device buffers in between (more argument sets than one graph)."""
    import torch
    dims = syn.Dims(n_embd=512, n_ff=256, n_expert=16, n_used=4)
    T, L = 5, 9
    layers = [syn.make_layer(dims, seed=52, layer=l) for l in range(L)]
    x = np.stack([syn.random_x(T, dims.n_embd, seed=80 + l) for l in range(L)])
    with pkg.Context(dims, n_layer=L, max_tokens=T, device=0) as ctx:
        for l in range(L):
            ctx.upload_layer(l, layers[l])
        want = np.stack([ctx.moe_forward_host(l, x[l], mode=0) for l in range(L)])
        stream = torch.cuda.Stream(torch.device("cuda", 0))
        ctx.set_stream(stream.cuda_stream)
        y = np.zeros_like(x)
        for _ in range(3):
            y[:] = 0
            ctx.moe_decode_stack_host(0, L, x.ctypes.data, T, y.ctypes.data)
            assert np.array_equal(y, want)
        x3 = np.ascontiguousarray(x[:, :3])
        y3 = np.zeros_like(x3)
        ctx.moe_decode_stack_host(0, L, x3.ctypes.data, 3, y3.ctypes.data)
        assert max(syn.rel_err_rows(y3[l], want[l, :3]) for l in range(L)) < 1e-6   # (another batch: not held to the same bits)
        d_x, d_y = ctx.to_device(x), ctx.alloc(x.nbytes)
        ctx.moe_decode_stack(0, L, d_x, T, d_y)
        assert np.array_equal(d_y.download(np.float32, x.shape), want)
        y[:] = 0
        ctx.moe_decode_stack_host(0, L, x.ctypes.data, T, y.ctypes.data)
        assert np.array_equal(y, want)
        y2 = np.zeros_like(x[:3])
        ctx.moe_decode_stack_host(2, 3, x[2:5].ctypes.data, T, y2.ctypes.data)   # fewer layers than chunks: one copy each way
        assert np.array_equal(y2, want[2:5])
        ctx.set_stream(0)


def test_expert_parallel_view_partial_sums(pkg, orc, syn):
    """A context that holds experts [4,8) only returns that shard's partial sum."""
    dims = syn.Dims(n_embd=512, n_ff=256, n_expert=8, n_used=3)
    T = 7
    layer = syn.make_layer(dims, seed=70)
    x = syn.random_x(T, dims.n_embd, seed=71)
    full = orc.moe_layer(layer, x)
    total = np.zeros_like(full["y"])
    for first in (0, 4):
        shard = layer.expert_slice(first, 4)
        with pkg.Context(dims, n_layer=1, max_tokens=T, device=0, expert_first=first, expert_count=4) as ctx:
            ctx.upload_layer(0, shard)
            w = ctx.layer_ptrs(0)
            d_x, d_sel = ctx.to_device(x), ctx.to_device(full["sel"])
            d_h, d_y = ctx.to_device(np.zeros(T * 4 * 256, np.float32)), ctx.alloc(T * 512 * 4)
            ctx.moe_gateup(shard.gateup_type, w.gate_exps, w.up_exps, d_x, d_sel, d_h, T)
            ctx.moe_down(shard.down_type, w.down_exps, d_h, d_sel, d_y, T)
            part = d_y.download(np.float32, (T, 512))
            want = orc.moe_layer(shard, x, sel_in=full["sel"], with_shared=False)["y"]
            assert syn.rel_err_rows(part, want) < TOL_F32
            total += part
    routed = orc.moe_layer(layer, x, sel_in=full["sel"], with_shared=False)["y"]
    assert syn.rel_err_rows(total, routed) < TOL_F32
