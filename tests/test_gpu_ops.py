"""CUDA kernels against the CPU oracle, op by op, through the C ABI.

Tolerances: integer results (expert ids, pair grouping) and dequantised weights are
compared bit-for-bit.  f32 outputs: the reference's own element metric
(src/main.cpp:548-560) with its 1e-2 gate, and 1e-5 on the row-scaled relative error
|a-b| / max(|b|, rms(row)) against the f64-accumulating oracle.
"""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

TOL_F32 = 1e-5
TOL_REF_METRIC = 1e-2


@pytest.fixture(scope="module")
def ctx(pkg):
    c = pkg.Context(pkg.synth.Dims(), n_layer=1, max_tokens=64, device=0)
    yield c
    c.close()


@pytest.mark.parametrize("ttype", [0, 1, 8, 14, 23, 18])
def test_dequant_bit_exact(ctx, orc, syn, ttype):
    elems = syn.BLOCK[ttype][0]
    n = 256 * 600 if elems > 1 else 8 * 5000
    blocks = syn.random_blocks(ttype, 1, n, seed=100 + ttype)
    d_b, d_y = ctx.to_device(blocks), ctx.alloc(n * 4)
    ctx.dequant(ttype, d_b, d_y, n)
    got = d_y.download(np.float32, n)
    want = orc.dequant(ttype, blocks, n)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
    d_b.free(); d_y.free()


@pytest.mark.parametrize("name,ttype", [("q8_0", 8), ("q6_k", 14), ("iq4_xs", 23), ("iq3_xxs", 18)])
def test_dequant_golden(ctx, golden, name, ttype):
    g = golden(f"dequant_{name}.npz")
    d_b, d_y = ctx.to_device(g["blocks"]), ctx.alloc(g["y"].nbytes)
    ctx.dequant(ttype, d_b, d_y, g["y"].size)
    got = d_y.download(np.float32, g["y"].size)
    assert np.array_equal(got.view(np.uint32), g["y"].view(np.uint32))
    d_b.free(); d_y.free()


@pytest.mark.parametrize("ttype", [1, 8, 14, 23, 18])
@pytest.mark.parametrize("M,K,n", [(512, 2048, 1), (264, 4096, 3), (100, 256, 2), (7, 512, 1)])
def test_gemv(ctx, orc, syn, ttype, M, K, n):
    W = syn.random_blocks(ttype, M, K, seed=7 * ttype + M)
    x = syn.random_x(n, K, seed=43)
    d_w, d_x, d_y = ctx.to_device(W), ctx.to_device(x), ctx.alloc(n * M * 4)
    ctx.gemv(ttype, d_w, d_x, d_y, M, K, n)
    got = d_y.download(np.float32, (n, M))
    want = orc.gemv(ttype, W, x, M, K)
    assert syn.rel_err_reference(got, want) < TOL_REF_METRIC
    assert syn.rel_err_rows(got, want) < TOL_F32
    for b in (d_w, d_x, d_y):
        b.free()


@pytest.mark.parametrize("ttype,M,K", [(1, 65536, 2048), (8, 65536, 2048), (14, 65536, 2048), (23, 65536, 2048),
                                       (18, 65536, 2048), (14, 151936, 2048), (8, 32768, 4096), (18, 40000, 4096)])
def test_gemv_streamed_large_matrix(ctx, orc, syn, ttype, M, K):
    """Matrices above 48 MB at n = 1 take the streamed (bulk-copy ring) kernels, for K = 2048 the
    variant that keeps x in registers: the shapes the large-matrix bandwidth figures and the
    151,936 x 2048 Q6_K head are quoted on.  Same tolerances as the small shapes."""
    assert M * syn.row_bytes(ttype, K) > 48 << 20
    W = syn.random_blocks(ttype, M, K, seed=11 * ttype + 3)
    x = syn.random_x(1, K, seed=44)
    d_w, d_x, d_y = ctx.to_device(W), ctx.to_device(x), ctx.alloc(M * 4)
    ctx.gemv(ttype, d_w, d_x, d_y, M, K, 1)
    got = d_y.download(np.float32, (1, M))
    want = orc.gemv(ttype, W, x, M, K, threads=orc.hardware_threads())
    assert syn.rel_err_reference(got, want) < TOL_REF_METRIC
    assert syn.rel_err_rows(got, want) < TOL_F32
    for b in (d_w, d_x, d_y):
        b.free()


@pytest.mark.parametrize("ttype,M,K", [(14, 8192, 2048), (23, 8192, 2048), (14, 8200, 4096), (23, 8208, 1024), (8, 40000, 2048),
                                       (14, 40016, 512), (8, 30008, 3072)])
def test_gemv_tensor_core_forms(ctx, orc, syn, ttype, M, K):
    """The integer tensor-core GEMV kernels (digit planes x quantised weights): Q6_K and IQ4_XS from
    8192 rows on, Q8_0 above 48 MB; row counts that leave a tail of fewer than 16 rows, and other K."""
    W = syn.random_blocks(ttype, M, K, seed=7 * ttype + 1)
    x = syn.random_x(1, K, seed=45)
    x[0, 5] = 40.0          # one large element: the small ones keep fewer bits of the fixed-point planes
    d_w, d_x, d_y = ctx.to_device(W), ctx.to_device(x), ctx.alloc(M * 4)
    ctx.gemv(ttype, d_w, d_x, d_y, M, K, 1)
    got = d_y.download(np.float32, (1, M))
    want = orc.gemv(ttype, W, x, M, K, threads=orc.hardware_threads())
    assert syn.rel_err_reference(got, want) < TOL_REF_METRIC
    assert syn.rel_err_rows(got, want) < TOL_F32
    for b in (d_w, d_x, d_y):
        b.free()


def test_gemv_rejects_bad_shapes(ctx, pkg):
    d = ctx.alloc(4096)
    for ttype, K in ((8, 48), (14, 128), (18, 300), (99, 256)):
        with pytest.raises(pkg.QkmError):
            ctx.gemv(ttype, d, d, d, 1, K, 1)
    d.free()


def _upload_router(ctx, layer):
    return ctx.to_device(layer.router), ctx.to_device(layer.gate_inp_shexp)


@pytest.mark.parametrize("router_type", [0, 1])
def test_route_select_ids_exact(ctx, orc, syn, router_type):
    dims = syn.Dims()
    T = 64
    layer = syn.make_layer(dims, seed=5, router_type=router_type)
    x = syn.random_x(T, dims.n_embd, seed=6)
    want, w64 = orc.route(layer, x, threads=8)
    d_r, d_g = _upload_router(ctx, layer)
    d_x, d_sel = ctx.to_device(x), ctx.alloc(T * 160)
    ctx.moe_route_select(router_type, d_r, d_g, d_x, d_sel, T)
    got = d_sel.download(pkg_sel(ctx), T)
    assert np.array_equal(got["ids"], want["ids"])
    np.testing.assert_allclose(got["w"][:, :8], w64[:, :8], rtol=1e-5, atol=1e-7)
    np.testing.assert_allclose(got["w_shared"], w64[:, 16], rtol=1e-6)
    for b in (d_r, d_g, d_x, d_sel):
        b.free()


def pkg_sel(ctx):
    from qwen_kernel_b200 import SEL_DTYPE
    return SEL_DTYPE


def test_route_select_ties_and_nonfinite(ctx, orc, syn):
    dims = syn.Dims()
    layer = syn.make_layer(dims, seed=9, router_type=syn.F32)
    r = layer.router.view(np.float32).reshape(256, 2048).copy()
    r[200] = r[17]; r[90] = r[17]            # three identical rows: exact ties
    r[3] = 0.0; r[4] = 0.0                   # two all-zero rows: logits exactly 0
    layer.router = r.reshape(-1).view(np.uint8)
    T = 8
    x = syn.random_x(T, 2048, seed=10)
    x[2] = r[17] * 50.0                       # make the tied experts win for token 2
    x[5, 100] = np.nan                        # every logit NaN
    x[6, 7] = np.inf                          # logits +-inf / NaN
    x[7] = 0.0                                # every logit 0: ids 0..7
    want, w64 = orc.route(layer, x)
    d_r, d_g = _upload_router(ctx, layer)
    d_x, d_sel = ctx.to_device(x), ctx.alloc(T * 160)
    ctx.moe_route_select(syn.F32, d_r, d_g, d_x, d_sel, T)
    got = d_sel.download(pkg_sel(ctx), T)
    assert np.array_equal(got["ids"], want["ids"])
    assert list(got["ids"][2, :3]) == [17, 90, 200]
    assert list(got["ids"][5, :8]) == list(range(8)) and list(got["ids"][7, :8]) == list(range(8))
    ok = np.isfinite(w64[:, :8]).all(axis=1)
    np.testing.assert_allclose(got["w"][ok, :8], w64[ok, :8], rtol=1e-5, atol=1e-7)
    for b in (d_r, d_g, d_x, d_sel):
        b.free()


@pytest.mark.parametrize("T", [72, 160])
def test_route_select_ties_large_batch(pkg, orc, syn, T):
    """The same hazards on the large-batch paths (f32 logits below 128 tokens, tensor-core logits
    above), where the boundary is re-evaluated in f64: ids must still equal the f64 router's."""
    dims = syn.Dims()
    layer = syn.make_layer(dims, seed=9, router_type=syn.F32)
    r = layer.router.view(np.float32).reshape(256, 2048).copy()
    r[200] = r[17]; r[90] = r[17]
    r[3] = 0.0; r[4] = 0.0
    layer.router = r.reshape(-1).view(np.uint8)
    x = syn.random_x(T, 2048, seed=10)
    x[2] = r[17] * 50.0
    x[5, 100] = np.nan
    x[6, 7] = np.inf
    x[7] = 0.0
    x[T - 1] = x[2]
    want, w64 = orc.route(layer, x, threads=8)
    with pkg.Context(dims, n_layer=1, max_tokens=T, device=0) as c:
        c.upload_layer(0, layer)
        c.moe_forward_host(0, np.where(np.isfinite(x), x, 0.0).astype(np.float32), mode=1)   # allocates the tensor-core scratch
        d_r, d_g = c.to_device(layer.router), c.to_device(layer.gate_inp_shexp)
        d_x, d_sel = c.to_device(x), c.alloc(T * 160)
        c.moe_route_select(syn.F32, d_r, d_g, d_x, d_sel, T)
        got = d_sel.download(pkg_sel(c), T)
        for b in (d_r, d_g, d_x, d_sel):
            b.free()
        # and through the fused prefill call (tensor-core logits for T >= 128)
        c.moe_forward_host(0, x, mode=1)
        got_fused = c.last_sel(T)
    for g in (got, got_fused):
        assert np.array_equal(g["ids"], want["ids"])
        assert list(g["ids"][2, :3]) == [17, 90, 200] and list(g["ids"][T - 1, :3]) == [17, 90, 200]
        assert list(g["ids"][5, :8]) == list(range(8)) and list(g["ids"][7, :8]) == list(range(8))
        ok = np.isfinite(w64[:, :8]).all(axis=1)
        np.testing.assert_allclose(g["w"][ok, :8], w64[ok, :8], rtol=1e-5, atol=1e-7)


@pytest.mark.parametrize("T,router_type", [(1024, 0), (2048, 1)])
def test_route_select_op_large_batch(pkg, orc, syn, T, router_type):
    """The op-level call with >= 1024 tokens computes its f32 logits with the tiled GEMM kernel
    and re-evaluates the boundary in f64: ids equal the f64 router's for EVERY token, including
    tie / NaN / Inf / all-zero rows placed beyond row 1000."""
    dims = syn.Dims()
    layer = syn.make_layer(dims, seed=19, router_type=router_type)
    if router_type == syn.F32:
        r = layer.router.view(np.float32).reshape(256, 2048).copy()
        r[200] = r[17]; r[90] = r[17]; r[3] = 0.0; r[4] = 0.0
        layer.router = r.reshape(-1).view(np.uint8)
        tie_row = r[17] * 50.0
    else:
        r = layer.router.view(np.float16).reshape(256, 2048).copy()
        r[200] = r[17]; r[90] = r[17]; r[3] = 0.0; r[4] = 0.0
        layer.router = r.reshape(-1).view(np.uint8)
        tie_row = r[17].astype(np.float32) * 50.0
    x = syn.random_x(T, 2048, seed=20)
    x[1001] = tie_row; x[T - 1] = tie_row
    x[1005, 100] = np.nan
    x[1006, 7] = np.inf
    x[1007] = 0.0
    want, w64 = orc.route(layer, x, threads=orc.hardware_threads())
    with pkg.Context(dims, n_layer=1, max_tokens=T, device=0) as c:
        d_r, d_g = c.to_device(layer.router), c.to_device(layer.gate_inp_shexp)
        d_x, d_sel = c.to_device(x), c.alloc(T * 160)
        c.moe_route_select(router_type, d_r, d_g, d_x, d_sel, T)
        got = d_sel.download(pkg_sel(c), T)
        for b in (d_r, d_g, d_x, d_sel):
            b.free()
    assert np.array_equal(got["ids"], want["ids"])
    assert list(got["ids"][1001, :3]) == [17, 90, 200] and list(got["ids"][T - 1, :3]) == [17, 90, 200]
    assert list(got["ids"][1005, :8]) == list(range(8)) and list(got["ids"][1007, :8]) == list(range(8))
    ok = np.isfinite(w64[:, :8]).all(axis=1)
    np.testing.assert_allclose(got["w"][ok, :8], w64[ok, :8], rtol=1e-5, atol=1e-7)
    np.testing.assert_allclose(got["w_shared"][ok], w64[ok, 16], rtol=1e-6)


def test_logits_and_select_from_f32(ctx, orc, syn):
    dims = syn.Dims()
    T = 16
    layer = syn.make_layer(dims, seed=15, router_type=syn.F32)
    x = syn.random_x(T, 2048, seed=16)
    d_r, d_g = _upload_router(ctx, layer)
    d_x, d_l, d_sel = ctx.to_device(x), ctx.alloc(T * 256 * 4), ctx.alloc(T * 160)
    ctx.moe_logits(syn.F32, d_r, d_x, d_l, T)
    logits = d_l.download(np.float32, (T, 256))
    want_l = orc.logits(layer, x)
    assert syn.rel_err_rows(logits, want_l) < TOL_F32
    # selection is exact with respect to the f32 logits it was given, incl. floors and ties
    logits[1, 5] = np.nan; logits[1, 6] = np.inf; logits[2, :] = 1.0; logits[3, 10] = logits[3, 200] = 99.0
    d_l.upload(logits)
    ctx.moe_select(d_l, d_g, d_x, d_sel, T)
    got = d_sel.download(pkg_sel(ctx), T)
    want = orc.select_f32(dims, logits, layer.gate_inp_shexp.view(np.float32), x)
    assert np.array_equal(got["ids"], want["ids"])
    assert list(got["ids"][2, :8]) == list(range(8)) and list(got["ids"][3, :2]) == [10, 200]
    np.testing.assert_allclose(got["w"], want["w"], rtol=1e-6, atol=1e-9)
    np.testing.assert_allclose(got["w_shared"], want["w_shared"], rtol=1e-6)
    for b in (d_r, d_g, d_x, d_l, d_sel):
        b.free()


@pytest.mark.parametrize("T", [0, 1, 37, 64])
def test_group_pairs(ctx, orc, syn, T):
    dims = syn.Dims()
    layer = syn.make_layer(dims, seed=25)
    x = syn.random_x(max(T, 1), 2048, seed=26)[:T]
    sel, _ = orc.route(layer, x, threads=8) if T else (np.zeros(0, pkg_sel(ctx)), None)
    if T > 2:
        sel["ids"][1, :8] = 3          # a "hot" expert (uniform vs hot routing, as the reference's moegcmp)
        sel["ids"][2, 0] = 100000      # out-of-range id is clamped to n_expert-1
    d_sel = ctx.to_device(sel) if T else ctx.alloc(160)
    d_off, d_pairs = ctx.alloc(257 * 4), ctx.alloc(max(T, 1) * 8 * 4)
    ctx.moe_group_pairs(d_sel, T, d_off, d_pairs)
    off = d_off.download(np.uint32, 257)
    pairs = d_pairs.download(np.uint32, T * 8)
    want_off, want_pairs = orc.group_pairs(sel, 256, 8)
    assert np.array_equal(off, want_off)
    assert np.array_equal(pairs, want_pairs)   # same deterministic (token, slot) order inside a range
    for b in (d_sel, d_off, d_pairs):
        b.free()


@pytest.mark.parametrize("gt,dt", [(18, 23), (23, 14)])
def test_expert_ops_token_and_expert_major(pkg, orc, syn, gt, dt):
    """gate/up -> h and down -> y / contrib, token-major and expert-major, on a small layer."""
    dims = syn.Dims(n_embd=512, n_ff=256, n_expert=8, n_used=3)
    T = 9
    layer = syn.make_layer(dims, seed=35, gateup_type=gt, down_type=dt)
    x = syn.random_x(T, dims.n_embd, seed=36)
    ref = orc.moe_layer(layer, x, want_h=True, want_contrib=True)
    with pkg.Context(dims, n_layer=1, max_tokens=T, device=0) as ctx:
        ctx.upload_layer(0, layer)
        w = ctx.layer_ptrs(0)
        d_x, d_sel = ctx.to_device(x), ctx.to_device(ref["sel"])
        nh = T * 4 * 256
        d_h, d_y, d_y2 = ctx.to_device(np.zeros(nh, np.float32)), ctx.alloc(T * 512 * 4), ctx.alloc(T * 512 * 4)
        ctx.moe_gateup(gt, w.gate_exps, w.up_exps, d_x, d_sel, d_h, T)
        ctx.moe_shared_gateup(w.gate_shexp, w.up_shexp, d_x, d_h, T)
        h = d_h.download(np.float32, (T, 4, 256))
        assert syn.rel_err_rows(h.reshape(T * 4, 256), ref["h"].reshape(T * 4, 256)) < TOL_F32
        ctx.moe_down(dt, w.down_exps, d_h, d_sel, d_y, T)
        ctx.moe_shared_down(w.down_shexp, d_h, d_sel, d_y2, T)
        y = d_y.download(np.float32, (T, 512)) + d_y2.download(np.float32, (T, 512))
        assert syn.rel_err_rows(y, ref["y"]) < TOL_F32
        assert syn.rel_err_reference(y, ref["y"]) < TOL_REF_METRIC
        # expert-major
        d_off, d_pairs = ctx.alloc(9 * 4), ctx.alloc(T * 3 * 4)
        ctx.moe_group_pairs(d_sel, T, d_off, d_pairs)
        d_h2 = ctx.to_device(np.zeros(nh, np.float32))
        ctx.moe_gateup_grouped(gt, w.gate_exps, w.up_exps, d_x, d_off, d_pairs, d_h2, T)
        h2 = d_h2.download(np.float32, (T, 4, 256))
        assert np.array_equal(h2[:, :3], h[:, :3])   # same arithmetic, different traversal
        d_c = ctx.alloc(T * 3 * 512 * 4)
        ctx.moe_down_grouped(dt, w.down_exps, d_h, d_sel, d_off, d_pairs, d_c, T)
        contrib = d_c.download(np.float32, (T, 3, 512))
        assert syn.rel_err_rows(contrib.reshape(T * 3, 512), ref["contrib"].reshape(T * 3, 512)) < TOL_F32
