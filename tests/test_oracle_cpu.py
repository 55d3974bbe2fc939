"""The CPU oracle against the reference: golden fixtures produced by the reference's
own src/quants.h (tests/golden/make_golden.py), and - where the reference tree is
present - the reference code itself, bit for bit."""
import numpy as np
import pytest

FORMATS = [("q8_0", 8), ("q6_k", 14), ("iq4_xs", 23), ("iq3_xxs", 18)]


@pytest.mark.parametrize("name,ttype", FORMATS)
def test_dequant_matches_golden(orc, golden, name, ttype):
    g = golden(f"dequant_{name}.npz")
    assert int(g["type"]) == ttype
    y = orc.dequant(ttype, g["blocks"], g["y"].size)
    assert np.array_equal(y.view(np.uint32), g["y"].view(np.uint32))


@pytest.mark.parametrize("name,ttype", FORMATS)
def test_dequant_matches_reference_code(orc, ref, syn, name, ttype):
    elems = syn.BLOCK[ttype][0]
    for seed in range(3):
        n = 4096 * elems // 32
        blocks = syn.random_blocks(ttype, 1, n, seed=seed, tag="cmp")
        a, b = orc.dequant(ttype, blocks, n), ref.dequant(ttype, blocks, n)
        assert np.array_equal(a.view(np.uint32), b.view(np.uint32))


def test_f16_tables(orc, golden):
    g = golden("f16.npz")
    f = orc.f16_to_f32(np.arange(65536, dtype=np.uint16))
    assert np.array_equal(f.view(np.uint32), g["f16_to_f32"])
    h = orc.f32_to_f16(g["f32_in"].view(np.float32))
    assert np.array_equal(h, g["f32_to_f16"])


def test_f16_matches_reference_code(orc, ref):
    h = np.arange(65536, dtype=np.uint16)
    assert np.array_equal(orc.f16_to_f32(h).view(np.uint32), ref.f16_to_f32(h).view(np.uint32))
    rng = np.random.default_rng(5)
    x = (rng.standard_normal(200000) * 10.0 ** rng.integers(-8, 6, 200000)).astype(np.float32)
    assert np.array_equal(orc.f32_to_f16(x), ref.f32_to_f16(x))


def test_codebooks(orc, golden, syn):
    t = golden("tables.npz")
    # sign byte i == i | parity(i) << 7  (reference shaders/iq_tables.glsl:2,43)
    assert [orc.lib.orc_signs8(i) for i in range(128)] == list(t["ksigns"])
    assert list(t["block_bytes"]) == [34, 210, 136, 98]
    for ttype, nbytes in ((8, 34), (14, 210), (23, 136), (18, 98)):
        assert syn.BLOCK[ttype][1] == nbytes
        assert orc.lib.orc_row_bytes(ttype, 2048) == 2048 // syn.BLOCK[ttype][0] * nbytes
    # one IQ3_XXS block whose 64 indices walk the grid: magnitudes must be the table's bytes
    for base in range(0, 256, 64):
        blk = np.zeros(98, np.uint8)
        blk[0:2] = np.frombuffer(np.float16(1.0).tobytes(), np.uint8)  # d = 1
        blk[2:66] = np.arange(base, base + 64, dtype=np.uint8)
        y = orc.dequant(18, blk, 256)  # aux = 0: scale (0.5+0)*0.5 = 0.25, all signs +
        mags = (y * 4).astype(np.uint32).reshape(64, 4)
        want = np.stack([(t["grid"][base:base + 64] >> (8 * j)) & 255 for j in range(4)], axis=1)
        assert np.array_equal(mags, want)
    # IQ4 value table through a block with d=1, scale code 33 (ls-32 = 1)
    blk = np.zeros(136, np.uint8)
    blk[0:2] = np.frombuffer(np.float16(1.0).tobytes(), np.uint8)
    blk[2:4] = np.frombuffer(np.uint16(0xAAAA).tobytes(), np.uint8)  # high bits 2 -> 32
    blk[4:8] = 0x11                                                   # low nibble 1 -> ls = 33
    blk[8:136] = np.tile(np.arange(16, dtype=np.uint8) * 17, 8)      # nibble i in both halves
    y = orc.dequant(23, blk, 256).reshape(8, 2, 16)
    assert np.array_equal(y[0, 0].astype(np.int8), t["kvalues"])
    assert np.array_equal(y[3, 1].astype(np.int8), t["kvalues"])


@pytest.mark.parametrize("tag", ["a", "b", "c"])
def test_moe_layer_matches_golden(orc, syn, golden, tag):
    g = golden(f"moe_small_{tag}.npz")
    rt, gt, dt = (int(v) for v in g["types"])
    dims = syn.Dims(*(int(v) for v in g["dims"]))
    layer = syn.make_layer(dims, seed=1234, layer=3, router_type=rt, gateup_type=gt, down_type=dt)
    x = syn.random_x(3, dims.n_embd, seed=4321)
    assert np.array_equal(x, g["x"]), "synthetic generator changed"
    out = orc.moe_layer(layer, x, want_h=True)
    assert np.array_equal(out["sel"]["ids"], g["ids"])
    assert np.array_equal(out["y"].view(np.uint32), g["y"].view(np.uint32))
    assert np.array_equal(out["h"].view(np.uint32), g["h"].view(np.uint32))
    np.testing.assert_allclose(out["sel"]["w"], g["w"], rtol=0, atol=0)
    np.testing.assert_allclose(out["sel"]["w_shared"], g["w_shared"], rtol=0, atol=0)
    # fixtures b and c were produced by the reference's own moeCpuRef, a by the oracle
    assert str(g["source"]) == ("oracle" if tag == "a" else "moeCpuRef")


@pytest.mark.parametrize("gt,dt", [(18, 23), (18, 14), (23, 23), (23, 14)])
def test_moe_layer_matches_reference_code(orc, ref_layer, syn, gt, dt):
    """The restated layer loop against the reference's own moeCpuRef (src/main.cpp:1316-1387),
    compiled from the reference's source: outputs, ids and selection weights bit for bit, for
    every tensor-type combination its loader accepts (F32 router)."""
    dims = syn.Dims(n_embd=512, n_ff=256, n_expert=32, n_used=8)
    for seed in (1, 2):
        layer = syn.make_layer(dims, seed=900 + seed, layer=seed, router_type=syn.F32, gateup_type=gt, down_type=dt)
        x = syn.random_x(4, dims.n_embd, seed=950 + seed)
        out = orc.moe_layer(layer, x, threads=2)
        r = ref_layer.moe_layer(layer, x)
        assert np.array_equal(out["sel"]["ids"], r["ids"])
        assert np.array_equal(out["y"].view(np.uint32), r["y"].view(np.uint32))
        assert np.array_equal(out["sel"]["w"], r["w"].astype(np.float32))
        assert np.array_equal(out["sel"]["w_shared"], r["w_shared"].astype(np.float32))


def test_moe_layer_properties(orc, syn):
    dims = syn.Dims(n_embd=256, n_ff=256, n_expert=8, n_used=3)
    layer = syn.make_layer(dims, seed=3)
    x = syn.random_x(5, dims.n_embd, seed=4)
    out = orc.moe_layer(layer, x, want_h=True, want_contrib=True)
    sel = out["sel"]
    # weights are a softmax over the selected logits: positive, descending, sum to 1
    w = sel["w"][:, :dims.n_used]
    assert np.all(w > 0) and np.all(np.diff(w, axis=1) <= 0)
    np.testing.assert_allclose(w.sum(axis=1), 1.0, rtol=1e-6)
    assert np.all((sel["w_shared"] > 0) & (sel["w_shared"] < 1))
    # ids agree with an independent f64 ranking of the f64 logits
    router = orc.dequant(layer.router_type, layer.router, dims.n_expert * dims.n_embd).reshape(dims.n_expert, -1)
    logits = x.astype(np.float64) @ router.astype(np.float64).T
    want = np.argsort(-logits, axis=1, kind="stable")[:, :dims.n_used]
    assert np.array_equal(sel["ids"][:, :dims.n_used], want)
    # the f32-accumulating CPU path agrees with the f64 one to f32 accuracy
    out32 = orc.moe_layer(layer, x, acc=1)
    assert syn.rel_err_rows(out32["y"], out["y"]) < 1e-5
    # expert-parallel partial sums add up to the whole layer
    parts = [orc.moe_layer(layer.expert_slice(f, 4), x, sel_in=sel, with_shared=(f == 0))["y"] for f in (0, 4)]
    assert syn.rel_err_rows(parts[0] + parts[1], out["y"]) < 1e-6
    # per-slot contributions fold back to the routed sum (slot order)
    r = orc.moe_layer(layer, x, sel_in=sel, with_shared=False, want_contrib=True)
    fold = np.zeros_like(r["y"])
    for s in range(dims.n_used):
        fold += r["contrib"][:, s]
    assert np.array_equal(fold, r["y"])
    # multi-threaded run is identical
    out_mt = orc.moe_layer(layer, x, threads=4)
    assert np.array_equal(out_mt["y"], out["y"])


def test_route_rules(orc, syn):
    """Non-finite logits rank at the floor; equal logits rank by ascending id."""
    dims = syn.Dims(n_embd=256, n_ff=256, n_expert=8, n_used=4)
    layer = syn.make_layer(dims, seed=11, router_type=syn.F32)
    r = layer.router.view(np.float32).reshape(8, 256).copy()
    r[5] = r[2]  # exact tie between experts 2 and 5
    layer.router = r.reshape(-1).view(np.uint8)
    x = syn.random_x(4, 256, seed=12)
    sel, _ = orc.route(layer, x)
    for t in range(4):
        ids = list(sel["ids"][t, :4])
        if 2 in ids and 5 in ids:
            assert ids.index(2) + 1 == ids.index(5)
    x[1, 7] = np.nan
    sel, _ = orc.route(layer, x)
    assert list(sel["ids"][1, :4]) == [0, 1, 2, 3]  # every logit NaN -> floor -> lowest ids


def test_group_pairs(orc, syn):
    dims = syn.Dims(n_embd=256, n_ff=256, n_expert=16, n_used=4)
    layer = syn.make_layer(dims, seed=21)
    x = syn.random_x(37, 256, seed=22)
    sel, _ = orc.route(layer, x)
    offsets, pairs = orc.group_pairs(sel, 16, 4)
    assert offsets[0] == 0 and offsets[-1] == 37 * 4 and np.all(np.diff(offsets.astype(np.int64)) >= 0)
    seen = set()
    for e in range(16):
        for p in pairs[offsets[e]:offsets[e + 1]]:
            t, s = int(p) >> 4, int(p) & 15
            assert sel["ids"][t, s] == e
            seen.add((t, s))
    assert len(seen) == 37 * 4
    # empty input
    off0, _ = orc.group_pairs(sel[:0], 16, 4)
    assert np.all(off0 == 0)


def test_gemv_oracle(orc, syn):
    for ttype in (syn.F16, syn.Q8_0, syn.Q6_K, syn.IQ4_XS, syn.IQ3_XXS):
        M, K = 24, 512
        W = syn.random_blocks(ttype, M, K, seed=31)
        x = syn.random_x(2, K, seed=32)
        y = orc.gemv(ttype, W, x, M, K)
        wf = orc.dequant(ttype, W, M * K).reshape(M, K).astype(np.float64)
        want = (x.astype(np.float64) @ wf.T).astype(np.float32)
        np.testing.assert_allclose(y, want, rtol=1e-6, atol=1e-6 * np.abs(want).max())
        y32 = orc.gemv(ttype, W, x, M, K, acc=1, threads=3)
        assert syn.rel_err_rows(y32, y) < 1e-5


def test_add_rms_oracle_matches_numpy(orc, syn):
    """Layer entry / tail arithmetic (add_rmsnorm.comp, add_rms3.comp, add_rms3_grouped.comp)."""
    n_rows, n, n_used = 4, 512, 3
    a, c2 = syn.random_x(n_rows, n, 1), syn.random_x(n_rows, n, 2)
    b3 = syn.random_x(n_rows * n_used, n, 3)
    w = 1.0 + 0.1 * syn.random_x(1, n, 4).reshape(-1)
    routed = b3.reshape(n_rows, n_used, n)
    for mode, b, want_s in (
        (0, b3[:n_rows], a + b3[:n_rows]),
        (1, b3[:n_rows], (a + b3[:n_rows]) + c2),
        (2, b3, (a + ((routed[:, 0] + routed[:, 1]) + routed[:, 2])) + c2),
    ):
        s, xn = orc.add_rms(mode, a, b, c2 if mode else None, w, n_used)
        assert np.array_equal(s, want_s.astype(np.float32))
        scale = 1.0 / np.sqrt((s.astype(np.float64) ** 2).mean(axis=1, keepdims=True) + 1e-6)
        np.testing.assert_allclose(xn, (s * scale * w).astype(np.float32), rtol=1e-6)
