"""Expert-parallel entry points (qkm_ep_*) on one GPU: G sharded contexts stand in for G
ranks, the all-to-all is done by copying rows between their buffers on the host.  No
kernel waits on another, so running the ranks one after the other is safe on one device.

Tolerance: the expert GEMMs run on the tensor cores (bf16/f16 operands), so outputs are held
to the prefill tolerance 2e-2 (row-scaled) against the f64 oracle; ids, send order and split
sizes are exact.  Shapes and type mixes outside the shard's tensor-core path take the f32 kernels and are
held to 1e-5."""
import numpy as np
import pytest

from ep_cpu_engine import plan_send

pytestmark = pytest.mark.gpu

TOL_BF16 = 2e-2
TOL_F32 = 1e-5


def run_ep(pkg, orc, syn, dims, layer, x_parts, G, tol):
    from qwen_kernel_b200 import SEL_DTYPE
    per = dims.n_expert // G
    fan = min(G, dims.n_used)
    T_all = sum(p.shape[0] for p in x_parts)
    ctxs = []
    for r in range(G):
        c = pkg.Context(dims, n_layer=1, max_tokens=max(T_all, 1), device=0, expert_first=r * per, expert_count=per)
        c.upload_layer(0, layer.expert_slice(r * per, per))
        ctxs.append(c)
    E = dims.n_embd
    st = []
    # phase 1: dispatch on every rank
    for r, (c, xp) in enumerate(zip(ctxs, x_parts)):
        n = xp.shape[0]
        d_x = c.to_device(xp) if n else c.alloc(16)
        d_xs, d_ss = c.alloc(max(n * fan, 1) * E * 4), c.alloc(max(n * fan, 1) * 160)
        counts = c.ep_dispatch(0, d_x, n, G, d_xs, d_ss)
        sel = c.last_sel(n) if n else np.zeros(0, SEL_DTYPE)
        want_sel, _ = orc.route(layer, xp) if n else (sel, None)
        assert np.array_equal(sel["ids"], want_sel["ids"])
        want_counts, send_tok, _ = plan_send(sel["ids"], dims.n_used, per, G)
        assert counts == want_counts
        k = sum(counts)
        xs = d_xs.download(np.float32, (k, E)) if k else np.zeros((0, E), np.float32)
        ss = d_ss.download(np.uint8, (k, 160)) if k else np.zeros((0, 160), np.uint8)
        assert np.array_equal(xs, xp[send_tok])
        assert np.array_equal(ss.reshape(-1).view(SEL_DTYPE)["ids"], sel["ids"][send_tok])
        # the asynchronous form leaves the same counts in device memory
        d_cnt = c.alloc(4 * G)
        c.ep_dispatch_dev(0, d_x, n, G, d_xs, d_ss, d_cnt)
        assert d_cnt.download(np.uint32, G).tolist() == counts
        d_cnt.free()
        c.ep_shared(0, d_x, n)
        st.append(dict(n=n, d_x=d_x, counts=counts, xs=xs, ss=ss, bufs=[d_x, d_xs, d_ss]))
    # phase 2: "all-to-all" on the host, expert forward on every rank
    partials = []
    for r, c in enumerate(ctxs):
        chunks_x, chunks_s = [], []
        for src in range(G):
            off = sum(st[src]["counts"][:r])
            cnt = st[src]["counts"][r]
            chunks_x.append(st[src]["xs"][off:off + cnt])
            chunks_s.append(st[src]["ss"][off:off + cnt])
        xr, sr = np.concatenate(chunks_x), np.concatenate(chunks_s)
        n_recv = xr.shape[0]
        if n_recv:
            d_xr, d_sr, d_p = c.to_device(xr), c.to_device(sr), c.alloc(n_recv * E * 4)
            c.ep_expert_forward(0, d_xr, d_sr, n_recv, d_p)
            partials.append(d_p.download(np.float32, (n_recv, E)))
            for b in (d_xr, d_sr, d_p):
                b.free()
        else:
            partials.append(np.zeros((0, E), np.float32))
    # phase 3: rows travel back, combine
    worst = 0.0
    for r, c in enumerate(ctxs):
        s = st[r]
        back = []
        for dst in range(G):   # rows this rank sent to dst come back in the same order
            off = sum(st[src]["counts"][dst] for src in range(r))
            back.append(partials[dst][off:off + s["counts"][dst]])
        back = np.concatenate(back) if back else np.zeros((0, E), np.float32)
        n = s["n"]
        if n:
            d_b = c.to_device(back) if back.shape[0] else c.alloc(16)
            d_y = c.alloc(n * E * 4)
            c.ep_combine(n, G, d_b, d_y)
            y = d_y.download(np.float32, (n, E))
            want = orc.moe_layer(layer, x_parts[r], threads=orc.hardware_threads())["y"]
            worst = max(worst, syn.rel_err_rows(y, want))
            d_b.free(); d_y.free()
        for b in s["bufs"]:
            b.free()
    for c in ctxs:
        c.close()
    assert worst < tol, worst
    return worst


@pytest.mark.parametrize("G,T", [(2, 24), (4, 40), (8, 200), (2, 200)])
def test_ep_full_size_shapes(pkg, orc, syn, G, T):
    dims = syn.Dims()
    layer = syn.make_layer(dims, seed=42)
    x = syn.random_x(T, dims.n_embd, seed=61)
    cuts = np.linspace(0, T, G + 1).astype(int)
    cuts[1] = min(T, cuts[1] + 3)                       # uneven shares
    parts = [x[cuts[r]:cuts[r + 1]] for r in range(G)]
    run_ep(pkg, orc, syn, dims, layer, parts, G, TOL_BF16)


def test_ep_rank_without_tokens(pkg, orc, syn):
    dims = syn.Dims()
    layer = syn.make_layer(dims, seed=43)
    x = syn.random_x(5, dims.n_embd, seed=62)
    run_ep(pkg, orc, syn, dims, layer, [x, x[:0]], 2, TOL_BF16)


def test_ep_generic_kernels_f32(pkg, orc, syn):
    """A shard's tensor-core path is wired for IQ3_XXS gate/up + IQ4_XS down tiles; a layer with a Q6_K
    down tensor is served by the f32 kernels, and 1e-5 applies."""
    dims = syn.Dims(n_embd=512, n_ff=256, n_expert=8, n_used=2)
    layer = syn.make_layer(dims, seed=44, down_type=syn.Q6_K)
    x = syn.random_x(10, dims.n_embd, seed=63)
    run_ep(pkg, orc, syn, dims, layer, [x[:6], x[6:]], 2, TOL_F32)


def test_ep_rejects_wrong_shard(pkg, syn):
    dims = syn.Dims()
    with pkg.Context(dims, n_layer=1, max_tokens=4, device=0, expert_first=0, expert_count=64) as c:
        c.upload_layer(0, syn.make_layer(dims, seed=45).expert_slice(0, 64))
        d = c.alloc(1 << 16)
        with pytest.raises(pkg.QkmError):
            c.ep_dispatch(0, d, 1, 8, d, d)      # 64 experts is a 4-way shard, not 8
        d.free()


# ---- the peer-memory form (qkm_ep_push / qkm_ep_forward_slots / qkm_ep_pull) -------------------------
def _download(c, ptr, dtype, shape):
    out = np.empty(shape, dtype)
    c.check(c.lib.qkm_d2h(c.h, out.ctypes.data, ptr, out.nbytes))
    return out


def run_ep_peer(pkg, orc, syn, dims, layer, x_parts, G, tol, slot_rows=None, cap_extra=0, merged=True):
    """G sharded contexts on one device; each has the others' receive buffers as raw pointers,
    which is what a peer mapping is to the kernels.  Phases are separated by a sync of every
    context (the barrier of the multi-GPU driver)."""
    from qwen_kernel_b200 import SEL_DTYPE
    per = dims.n_expert // G
    E = dims.n_embd
    most = max(p.shape[0] for p in x_parts)
    cap = most + cap_extra
    rows = cap if slot_rows is None else slot_rows
    ctxs = []
    for r in range(G):
        c = pkg.Context(dims, n_layer=1, max_tokens=G * cap, device=0, expert_first=r * per, expert_count=per)
        c.upload_layer(0, layer.expert_slice(r * per, per))
        c.ep_peer_setup(G, r, cap)
        ctxs.append(c)
    bufs = [c.ep_peer_buffers() for c in ctxs]
    for r, c in enumerate(ctxs):
        for q in range(G):
            if q != r:
                c.ep_peer_set(q, *bufs[q])
    d_xs, sels = [], []
    for r, (c, xp) in enumerate(zip(ctxs, x_parts)):
        n = xp.shape[0]
        d_x = c.to_device(xp) if n else c.alloc(16)
        c.ep_push(0, d_x, n, rows)
        if not merged:
            c.ep_shared(0, d_x, n)
        d_xs.append(d_x)
        sel = c.last_sel(n) if n else np.zeros(0, SEL_DTYPE)
        if n:
            assert np.array_equal(sel["ids"], orc.route(layer, xp)[0]["ids"])
        sels.append(sel)
    for c in ctxs:
        c.sync()
    # what landed: rank d holds source s's token i at row s * rows + i iff i selected an expert of d
    for d, c in enumerate(ctxs):
        xr = _download(c, bufs[d][0], np.float32, (G * rows, E))
        sr = _download(c, bufs[d][1], np.uint8, (G * rows, 160)).reshape(-1).view(SEL_DTYPE)
        for s in range(G):
            n = x_parts[s].shape[0]
            need = ((sels[s]["ids"][:, :dims.n_used] // per) == d).any(axis=1) if n else np.zeros(0, bool)
            got = sr[s * rows:(s + 1) * rows]
            assert np.array_equal(got["ids"][:n][need], sels[s]["ids"][need])
            if n and need.any():
                inv = got["pad"][:n, 0][need]
                if (inv != 0).all():
                    # rows travel as f16, scaled per row by a power of two (max|x| lands in [2^13, 2^14)), at the
                    # head of the row buffer; the scale that undoes it rides in the record's first padding word
                    xh = xr.view(np.float16).reshape(-1)[:G * rows * E].reshape(G * rows, E)[s * rows:s * rows + n][need]
                    xs = x_parts[s][need]
                    up = np.float32(2.0) ** (14 - (np.frexp(np.abs(xs).max(axis=1))[1]))
                    assert np.array_equal(inv, (1.0 / up).astype(np.float32))
                    assert np.array_equal(xh, (xs * up[:, None]).astype(np.float16))
                else:
                    assert np.array_equal(xr[s * rows:s * rows + n][need], x_parts[s][need])
            empty = np.ones(rows, bool)
            empty[:n] = ~need
            assert (got["ids"][empty][:, :dims.n_used] == 0xFFFFFFFF).all()
    for c, xp in zip(ctxs, x_parts):
        c.ep_forward_slots(0, rows, xp.shape[0] if merged else None)
    for c in ctxs:
        c.sync()
    worst = 0.0
    for r, c in enumerate(ctxs):
        n = x_parts[r].shape[0]
        if n:
            d_y = c.alloc(n * E * 4)
            c.ep_pull(n, rows, d_y)
            y = d_y.download(np.float32, (n, E))
            want = orc.moe_layer(layer, x_parts[r], threads=orc.hardware_threads())["y"]
            worst = max(worst, syn.rel_err_rows(y, want))
            d_y.free()
    for c, d_x in zip(ctxs, d_xs):
        d_x.free()
        c.close()
    assert worst < tol, worst


@pytest.mark.parametrize("merged", [True, False])
@pytest.mark.parametrize("G,T,extra", [(2, 24, 0), (4, 40, 5), (8, 200, 0), (2, 300, 0)])
def test_ep_peer_full_size_shapes(pkg, orc, syn, G, T, extra, merged):
    dims = syn.Dims()
    layer = syn.make_layer(dims, seed=46)
    x = syn.random_x(T, dims.n_embd, seed=64)
    cuts = np.linspace(0, T, G + 1).astype(int)
    cuts[1] = min(T, cuts[1] + 3)                       # uneven shares
    parts = [x[cuts[r]:cuts[r + 1]] for r in range(G)]
    run_ep_peer(pkg, orc, syn, dims, layer, parts, G, TOL_BF16, cap_extra=extra, merged=merged)


def test_ep_peer_rank_without_tokens_and_tight_slots(pkg, orc, syn):
    dims = syn.Dims()
    layer = syn.make_layer(dims, seed=47)
    x = syn.random_x(5, dims.n_embd, seed=65)
    run_ep_peer(pkg, orc, syn, dims, layer, [x, x[:0]], 2, TOL_BF16, slot_rows=5, cap_extra=3)


def test_ep_peer_generic_kernels_f32(pkg, orc, syn):
    dims = syn.Dims(n_embd=512, n_ff=256, n_expert=8, n_used=2)
    layer = syn.make_layer(dims, seed=48, down_type=syn.Q6_K)
    x = syn.random_x(10, dims.n_embd, seed=66)
    run_ep_peer(pkg, orc, syn, dims, layer, [x[:6], x[6:]], 2, TOL_F32)
    run_ep_peer(pkg, orc, syn, dims, layer, [x[:6], x[6:]], 2, TOL_F32, merged=False)


def test_ep_peer_argument_checks(pkg, syn):
    dims = syn.Dims()
    with pkg.Context(dims, n_layer=1, max_tokens=16, device=0, expert_first=64, expert_count=64) as c:
        c.upload_layer(0, syn.make_layer(dims, seed=45).expert_slice(64, 64))
        d = c.alloc(1 << 16)
        with pytest.raises(pkg.QkmError):
            c.ep_push(0, d, 1, 4)                  # before qkm_ep_peer_setup
        with pytest.raises(pkg.QkmError):
            c.ep_peer_setup(4, 0, 4)               # the context holds shard 1, not 0
        with pytest.raises(pkg.QkmError):
            c.ep_peer_setup(4, 1, 5)               # 4 x 5 rows exceed max_tokens
        c.ep_peer_setup(4, 1, 4)
        with pytest.raises(pkg.QkmError):
            c.ep_push(0, d, 1, 4)                  # peers not mapped yet
        with pytest.raises(pkg.QkmError):
            c.ep_peer_set(1, d, d, d)              # its own rank
        d.free()


def test_ep_peer_two_processes_over_ipc():
    """Two processes, one GPU each: buffers mapped through CUDA IPC handles, NCCL barriers."""
    import os
    import socket
    import subprocess
    import sys
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    here = os.path.dirname(os.path.abspath(__file__))
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    procs = [subprocess.Popen([sys.executable, os.path.join(here, "ep_gpu_worker.py"), "--rank", str(r), "--world", "2",
                               "--port", str(port)], stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
             for r in range(2)]
    outs = []
    for p in procs:
        try:
            out, _ = p.communicate(timeout=600)
        except subprocess.TimeoutExpired:
            for q in procs:
                q.kill()
            raise
        outs.append(out)
    for r, (p, out) in enumerate(zip(procs, outs)):
        assert p.returncode == 0, f"rank {r} failed:\n{out[-3000:]}"
    assert "EP_GPU" in outs[0]


def test_ep_peer_layer_single_rank_with_device_barrier(pkg, orc, syn):
    """One rank: the barrier kernel signals and polls its own words; the fused call is the layer."""
    dims = syn.Dims()
    layer = syn.make_layer(dims, seed=49)
    x = syn.random_x(140, dims.n_embd, seed=67)
    with pkg.Context(dims, n_layer=1, max_tokens=160, device=0, expert_first=0, expert_count=dims.n_expert) as c:
        c.upload_layer(0, layer)
        c.ep_peer_setup(1, 0, 160)
        d_x, d_y = c.to_device(x), c.alloc(x.nbytes)
        for rows in (140, 160):
            c.ep_peer_layer(0, d_x, 140, rows, d_y, timeout_ms=1000)
            c.sync()
            y = d_y.download(np.float32, x.shape)
            want = orc.moe_layer(layer, x, threads=orc.hardware_threads())["y"]
            assert syn.rel_err_rows(y, want) < TOL_BF16
        d_x.free(); d_y.free()


def test_ep_barrier_wait_runs_out(pkg, syn):
    """A peer that never arrives: the bounded wait gives up after its limit, the next sync
    reports QKM_ERR_TIMEOUT and the context keeps working."""
    dims = syn.Dims()
    layer = syn.make_layer(dims, seed=50)
    c0 = pkg.Context(dims, n_layer=1, max_tokens=16, device=0, expert_first=0, expert_count=128)
    c1 = pkg.Context(dims, n_layer=1, max_tokens=16, device=0, expert_first=128, expert_count=128)
    c0.upload_layer(0, layer.expert_slice(0, 128))
    c0.ep_peer_setup(2, 0, 8)
    c1.ep_peer_setup(2, 1, 8)
    c0.ep_peer_set(1, *c1.ep_peer_buffers())
    c0.ep_barrier(timeout_ms=20)                 # rank 1 never issues its barrier
    with pytest.raises(pkg.QkmError) as e:
        c0.sync()
    assert e.value.code == -7
    c0.sync()                                    # the flag was cleared; the context is usable
    x = syn.random_x(4, dims.n_embd, seed=68)
    d_x = c0.to_device(x)
    c0.ep_push(0, d_x, 4, 8)
    c0.sync()
    d_x.free()
    c0.close(); c1.close()
