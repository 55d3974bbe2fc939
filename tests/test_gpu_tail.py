"""Residual add + RMS norm kernels and the layer step against the oracle.
The stored sums are bit-exact (same f32 additions in the same order); the normed rows are
held to 1e-5 relative (the mean of squares is f32 on the GPU, f64 in the oracle)."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu
TOL = 1e-5


@pytest.fixture(scope="module")
def ctx(pkg):
    c = pkg.Context(pkg.synth.Dims(), n_layer=1, max_tokens=96, device=0)
    yield c
    c.close()


def _rows(syn, n_rows, n, seed, scale=1.0):
    return syn.random_x(n_rows, n, seed) * np.float32(scale)


@pytest.mark.parametrize("mode", [0, 1, 2])
@pytest.mark.parametrize("n_rows,n", [(1, 2048), (16, 2048), (5, 1024), (3, 4096)])
def test_add_rms_kernels(ctx, orc, syn, mode, n_rows, n):
    n_used = 8
    a = _rows(syn, n_rows, n, 1, 3.0)
    b = _rows(syn, n_rows * (n_used if mode == 2 else 1), n, 2, 50.0)
    c2 = _rows(syn, n_rows, n, 3, 20.0)
    w = 1.0 + 0.1 * _rows(syn, 1, n, 4).reshape(-1)
    want_s, want_xn = orc.add_rms(mode, a, b, c2 if mode else None, w, n_used)
    d = [ctx.to_device(t) for t in (a, b, c2, w)]
    d_s, d_xn = ctx.alloc(a.nbytes), ctx.alloc(a.nbytes)
    if mode == 0:
        ctx.add_rmsnorm(d[0], d[1], d[3], d_s, d_xn, n_rows, n)
    elif mode == 1:
        ctx.add_rms3(d[0], d[1], d[2], d[3], d_s, d_xn, n_rows, n)
    else:
        ctx.add_rms3_grouped(d[0], d[1], d[2], d[3], d_s, d_xn, n_rows, n, n_used)
    got_s, got_xn = d_s.download(np.float32, a.shape), d_xn.download(np.float32, a.shape)
    assert np.array_equal(got_s.view(np.uint32), want_s.view(np.uint32))
    assert syn.rel_err_rows(got_xn, want_xn) < TOL
    for t in d + [d_s, d_xn]:
        t.free()


def test_add_rms_rejects_bad_width(ctx, pkg):
    d = ctx.alloc(1 << 16)
    with pytest.raises(pkg.QkmError):
        ctx.add_rmsnorm(d, d, d, d, d, 1, 2050)
    with pytest.raises(pkg.QkmError):
        ctx.add_rmsnorm(d, d, d, d, d, 1, 16384)
    d.free()


@pytest.mark.parametrize("T,tol", [(16, 1e-5), (80, 2e-2)])
def test_layer_step(ctx, orc, syn, T, tol):
    """resid + attn -> norm -> MoE -> + resid -> norm, decode kernels (T <= 64) or tensor cores."""
    dims = syn.Dims()
    layer = syn.make_layer(dims, seed=71)
    ctx.upload_layer(0, layer)
    E = dims.n_embd
    resid, attn = _rows(syn, T, E, 5, 2.0), _rows(syn, T, E, 6, 1.0)
    w_post = 1.0 + 0.1 * _rows(syn, 1, E, 7).reshape(-1)
    w_next = 1.0 + 0.1 * _rows(syn, 1, E, 8).reshape(-1)
    r2, xn2 = orc.add_rms(0, resid, attn, None, w_post)
    y = orc.moe_layer(layer, xn2, threads=orc.hardware_threads())["y"]
    want_r, want_xn = orc.add_rms(0, r2, y, None, w_next)
    d = [ctx.to_device(t) for t in (resid, attn, w_post, w_next)]
    d_r, d_xn = ctx.alloc(resid.nbytes), ctx.alloc(resid.nbytes)
    ctx.moe_layer_step(0, d[0], d[1], d[2], d[3], T, d_r, d_xn)
    got_r, got_xn = d_r.download(np.float32, resid.shape), d_xn.download(np.float32, resid.shape)
    assert syn.rel_err_rows(got_r, want_r) < tol
    assert syn.rel_err_rows(got_xn, want_xn) < tol
    for t in d + [d_r, d_xn]:
        t.free()


def _argmax_ref(rows):
    """argmax1/argmax2 semantics: largest value above -3.4e38, lowest index on ties, else 0."""
    out = []
    for r in rows:
        ok = r > np.float32(-3.4e38)          # False for NaN
        if not ok.any():
            out.append(0)
            continue
        m = r[ok].max()
        out.append(int(np.nonzero(ok & (r == m))[0][0]))
    return np.asarray(out, np.uint32)


@pytest.mark.parametrize("n", [1, 255, 4096, 151936])
def test_argmax(ctx, syn, n):
    rows = syn.random_x(6, n, seed=12).copy()
    if n > 300:
        rows[1, 77] = rows[1, 300] = rows[1].max() + 1.0     # tie: lower index wins
        rows[2, :] = -np.inf                                 # nothing above the floor
        rows[3, 5] = np.nan; rows[3, n - 1] = np.inf         # NaN ignored, +inf wins
        rows[4, :] = np.nan
        rows[5, n - 1] = 1e30                                # last element
    d_l, d_t = ctx.to_device(rows), ctx.alloc(4 * 6)
    ctx.argmax(d_l, 6, n, d_t)
    assert np.array_equal(d_t.download(np.uint32, 6), _argmax_ref(rows))
    d_l.free(); d_t.free()
