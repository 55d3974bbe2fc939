"""Batched prefill through the tensor-core path (bf16 operands, f32 accumulation) against the
f64-accumulating oracle.  Tolerance: 2e-2 on the row-scaled relative error (measured: about 4e-3), expert ids exact,
argmax of every output row unchanged (where the reference itself is not a near-tie)."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

TOL_BF16 = 2e-2


def run_prefill(pkg, orc, syn, dims, layer, x, tol=TOL_BF16):
    T = x.shape[0]
    ref = orc.moe_layer(layer, x, threads=orc.hardware_threads(), want_h=True)
    with pkg.Context(dims, n_layer=1, max_tokens=max(T, 1), device=0) as ctx:
        ctx.upload_layer(0, layer)
        y = ctx.moe_forward_host(0, x, mode=1)
        sel = ctx.last_sel(T)
        y_again = ctx.moe_forward_host(0, x, mode=1)
    assert np.array_equal(sel["ids"][:, :dims.n_used], ref["sel"]["ids"][:, :dims.n_used])
    err = syn.rel_err_rows(y, ref["y"])
    assert err < tol, err
    # argmax of every output row is unchanged wherever the reference's lead over the
    # runner-up is larger than twice the tolerated error (a closer call is a tie at this precision)
    r = ref["y"].astype(np.float64)
    top2 = np.sort(r, axis=1)[:, -2:]
    rms = np.sqrt(np.mean(r * r, axis=1))
    clear = (top2[:, 1] - top2[:, 0]) > 2 * tol * np.maximum(rms, np.abs(top2[:, 1]))
    assert np.array_equal(np.argmax(y, axis=1)[clear], np.argmax(r, axis=1)[clear])
    assert np.array_equal(y, y_again)   # deterministic
    return err


@pytest.mark.parametrize("T", [1, 17, 65, 130, 300])
def test_prefill_full_size(pkg, orc, syn, T):
    """Bench configuration 3 shapes (2048 / 512 / 256 experts / top-8) at small chunk sizes."""
    dims = syn.Dims()
    layer = syn.make_layer(dims, seed=42)
    x = syn.random_x(T, dims.n_embd, seed=77)
    run_prefill(pkg, orc, syn, dims, layer, x)


def test_prefill_operand_precision(pkg, orc, syn):
    """Both expert GEMMs run on f16 operands (x and the hidden rows scaled per row by a power of two,
    the dequantised weights rounded once or twice to f16), so the outputs sit well inside the 2e-2
    budget: a third of it at most on the full-size layer."""
    dims = syn.Dims()
    layer = syn.make_layer(dims, seed=42)
    x = syn.random_x(130, dims.n_embd, seed=78)
    x[3] *= 300.0      # rows of very different magnitude: the per-row scales keep their precision
    x[4] *= 1e-4
    err = run_prefill(pkg, orc, syn, dims, layer, x)
    assert err < 7e-3, err


@pytest.mark.parametrize("T", [512, 2048, 4096])
def test_prefill_bench_chunk_sizes(pkg, orc, syn, T):
    """The chunk sizes the prefill figures are quoted on.  Expert ids (tensor-core logits, boundary
    re-evaluated in f64) must equal the f64 router's for EVERY token - the oracle's router alone
    is cheap - including tie / NaN / all-zero rows placed beyond row 1024 where the chunk has
    them.  Outputs: the oracle's full layer on >= 64 sampled rows (selection given) that include
    the first and the last row, rows from every 128-pair N-tile of the busiest expert, and the
    special rows; 2e-2 row-scaled relative."""
    dims = syn.Dims()
    layer = syn.make_layer(dims, seed=42, router_type=syn.F32)
    r = layer.router.view(np.float32).reshape(256, 2048).copy()
    r[200] = r[17]; r[90] = r[17]; r[3] = 0.0; r[4] = 0.0
    r[40] *= 3.0                                    # a busy expert: several N-tiles at the larger chunks
    layer.router = r.reshape(-1).view(np.uint8)
    x = syn.random_x(T, dims.n_embd, seed=79)
    special = []
    if T > 1100:
        x[1030] = r[17] * 50.0; x[1031] = 0.0
        special = [1030, 1031]
    x[T - 1] = r[17] * 50.0
    nthr = orc.hardware_threads()
    want, w64 = orc.route(layer, x, threads=nthr)
    x_nan = None
    if T > 1100:                                    # a NaN row: ids must be 0..7; its output is not compared
        x_nan = 1040
        x[x_nan, 100] = np.nan
        want, w64 = orc.route(layer, x, threads=nthr)
    with pkg.Context(dims, n_layer=1, max_tokens=T, device=0) as ctx:
        ctx.upload_layer(0, layer)
        y = ctx.moe_forward_host(0, x, mode=1)
        sel = ctx.last_sel(T)
    assert np.array_equal(sel["ids"][:, :8], want["ids"][:, :8])
    assert list(sel["ids"][T - 1, :3]) == [17, 90, 200]
    if x_nan is not None:
        assert list(sel["ids"][x_nan, :8]) == list(range(8)) and list(sel["ids"][1031, :8]) == list(range(8))
    ok = np.isfinite(w64[:, :8]).all(axis=1)
    np.testing.assert_allclose(sel["w"][ok, :8], w64[ok, :8], rtol=1e-5, atol=1e-7)
    # rows to check through the whole layer
    ids = want["ids"][:, :8]
    counts = np.bincount(ids.reshape(-1), minlength=256)
    busiest = int(np.argmax(counts))
    toks_busy = np.nonzero((ids == busiest).any(axis=1))[0]      # ascending = pair order inside the expert
    rows = {0, T - 1, *special}
    for tile in range((len(toks_busy) + 127) // 128):            # first and last pair of every N-tile
        seg = toks_busy[tile * 128:(tile + 1) * 128]
        rows.update((int(seg[0]), int(seg[-1])))
    rng = np.random.default_rng(5)
    while len(rows) < 64:
        rows.add(int(rng.integers(0, T)))
    if x_nan is not None:
        rows.discard(x_nan)
    rows = np.array(sorted(rows))
    if T > 1100:
        assert counts[busiest] > 128, "the busy expert should span more than one N-tile"
    ref = orc.moe_layer(layer, x[rows], threads=nthr, sel_in=want[rows])
    err = syn.rel_err_rows(y[rows], ref["y"])
    assert err < TOL_BF16, err
    assert np.isfinite(y[np.setdiff1d(np.arange(T), [x_nan] if x_nan is not None else [])]).all()


def test_prefill_hot_expert(pkg, orc, syn):
    """Every token routed to the same experts: more pairs than one block holds (N tiles > 1)."""
    dims = syn.Dims(n_embd=1024, n_ff=512, n_expert=16, n_used=4)
    layer = syn.make_layer(dims, seed=5, router_type=syn.F32)
    r = layer.router.view(np.float32).reshape(16, 1024).copy()
    r[3] *= 40.0; r[7] *= 30.0                      # experts 3 and 7 dominate for most tokens
    layer.router = r.reshape(-1).view(np.uint8)
    x = syn.random_x(150, dims.n_embd, seed=6)
    x[:, :] = np.abs(x) * np.sign(r[3])[None, :] * 0.5 + x * 0.5   # push tokens towards expert 3
    run_prefill(pkg, orc, syn, dims, layer, x)


def test_prefill_matches_decode_path(pkg, syn):
    """The two fused paths agree to bf16 accuracy on the same inputs."""
    dims = syn.Dims()
    layer = syn.make_layer(dims, seed=8)
    x = syn.random_x(24, dims.n_embd, seed=9)
    with pkg.Context(dims, n_layer=1, max_tokens=24, device=0) as ctx:
        ctx.upload_layer(0, layer)
        yd = ctx.moe_forward_host(0, x, mode=0)
        yp = ctx.moe_forward_host(0, x, mode=1)
    assert syn.rel_err_rows(yp, yd) < TOL_BF16


@pytest.mark.parametrize("gt,dt", [(18, 14), (23, 23), (23, 14)])
@pytest.mark.parametrize("T", [70, 200])
def test_prefill_other_type_mixes(pkg, orc, syn, T, gt, dt):
    """Q6_K (14) down tensors and IQ4_XS (23) gate/up tensors: both expert GEMMs on the tensor cores
    (kernels that dequantise Q6_K / IQ4_XS tiles to f16 in shared memory)."""
    dims = syn.Dims()
    layer = syn.make_layer(dims, seed=46, router_type=syn.F32, gateup_type=gt, down_type=dt)
    x = syn.random_x(T, dims.n_embd, seed=78)
    run_prefill(pkg, orc, syn, dims, layer, x)
