"""Dense quantised GEMM (the reference's gemm_q8_0 / gemm_iq4_xs prefill projections) on the
tensor-core pipeline against the oracle's f64 GEMV, row by row.  bf16 operands: 2e-2 relative
(row-scaled), as for the expert GEMMs."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu
TOL = 2e-2


@pytest.fixture(scope="module")
def ctx(pkg):
    c = pkg.Context(pkg.synth.Dims(), n_layer=1, max_tokens=1, device=0)
    yield c
    c.close()


@pytest.mark.parametrize("ttype", [8, 23])
@pytest.mark.parametrize("M,K,n", [(512, 256, 1), (1024, 2048, 130), (4096, 2048, 300), (2048, 4096, 64)])
def test_dense_gemm(ctx, orc, syn, ttype, M, K, n):
    W = syn.random_blocks(ttype, M, K, seed=17, tag="dense")
    x = syn.random_x(n, K, seed=18)
    ctx.dense_upload(3, ttype, W, M, K)
    d_x, d_y = ctx.to_device(x), ctx.alloc(n * M * 4)
    ctx.dense_gemm(3, d_x, n, d_y)
    y = d_y.download(np.float32, (n, M))
    rows = sorted(set([0, n - 1, n // 2] + list(range(0, n, max(1, n // 6)))))
    want = np.stack([orc.gemv(ttype, W, x[r], M, K, threads=orc.hardware_threads()) for r in rows])
    assert syn.rel_err_rows(y[rows], want) < TOL
    # a second call with fewer rows reuses the scratch
    ctx.dense_gemm(3, d_x, 1, d_y)
    assert syn.rel_err_rows(d_y.download(np.float32, (1, M)), want[:1]) < TOL
    d_x.free(); d_y.free()


def test_dense_rejects(ctx, pkg, syn):
    W = syn.random_blocks(8, 128, 256, seed=1)
    d = ctx.alloc(1 << 16)
    with pytest.raises(pkg.QkmError):
        ctx.dense_upload(0, 14, W, 128, 256)          # Q6_K: not a GEMM type
    with pytest.raises(pkg.QkmError):
        ctx.dense_upload(0, 8, W, 100, 256)           # M not a multiple of 128
    with pytest.raises(pkg.QkmError):
        ctx.dense_upload(99, 8, W, 128, 256)
    with pytest.raises(pkg.QkmError):
        ctx.dense_gemm(5, d, 1, d)                    # empty slot
    d.free()
