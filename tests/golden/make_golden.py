"""Regenerates the golden fixtures in this directory.

    python tests/golden/make_golden.py

Needs the reference tree (it runs the reference's OWN src/quants.h through
oracle/_ref/libqk_ref.so); the fixtures it writes are what lets the same checks
run where the reference tree does not exist.

  dequant_<fmt>.npz   seeded random ggml blocks + the reference's dequantised f32
  f16.npz             reference f16->f32 of all 65536 patterns, and f32->f16 of a
                      spread of floats (normals, halfway cases, under/overflow)
  tables.npz          the reference's codebooks (grid, sign bytes, iq4 values)
  moe_small_a.npz     a small MoE layer with an F16 router (which the reference's loader
                      rejects) through the oracle's f64 path: a regression pin
  moe_small_b.npz,    small MoE layers with the tensor types the reference's loader accepts
  moe_small_c.npz     (F32 router; IQ4_XS + Q6_K and IQ3_XXS + IQ4_XS), outputs and selection
                      produced by the REFERENCE's own moeCpuRef (src/main.cpp:1316-1387,
                      compiled into oracle/_ref/libqk_ref_layer.so); h from the oracle after
                      its y matched the reference's bit for bit
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
import __graft_entry__ as entry  # noqa: E402


def main():
    pkg = entry.package()
    syn = pkg.synth
    om = entry.oracle_module()
    om.build(ref=True)
    assert om.Reference.available(), "reference tree not found: cannot regenerate golden vectors"
    ref, orc = om.Reference(), om.Oracle()

    for ttype, name, nblocks in ((syn.Q8_0, "q8_0", 256), (syn.Q6_K, "q6_k", 48), (syn.IQ4_XS, "iq4_xs", 64),
                                 (syn.IQ3_XXS, "iq3_xxs", 96)):
        elems = syn.BLOCK[ttype][0]
        blocks = syn.random_blocks(ttype, 1, nblocks * elems, seed=20250 + ttype, tag="golden")
        if ttype == syn.IQ3_XXS:  # make sure every grid index and every sign code occurs
            b = blocks.reshape(nblocks, 98)
            b[0:4, 2:66] = np.arange(256, dtype=np.uint8).reshape(4, 64)
            for i in range(128):
                blk, ib = 4 + i // 8, i % 8
                aux = (i | ((i ^ 0x55) & 127) << 7 | ((i * 3) & 127) << 14 | ((127 - i) & 127) << 21 | (i % 16) << 28)
                b[blk, 66 + 4 * ib:70 + 4 * ib] = np.frombuffer(np.uint32(aux).tobytes(), np.uint8)
        y = ref.dequant(ttype, blocks, nblocks * elems)
        assert np.array_equal(y.view(np.uint32), orc.dequant(ttype, blocks, nblocks * elems).view(np.uint32))
        np.savez_compressed(os.path.join(HERE, f"dequant_{name}.npz"), type=ttype, blocks=blocks, y=y)

    h = np.arange(65536, dtype=np.uint16)
    f = ref.f16_to_f32(h)
    rng = np.random.Generator(np.random.SFC64(99))
    xs = np.concatenate([
        rng.standard_normal(2048).astype(np.float32) * np.float32(10.0) ** rng.integers(-9, 6, 2048).astype(np.float32),
        (f[1:4096:7].astype(np.float64) + f[2:4097:7].astype(np.float64)).astype(np.float32) / np.float32(2),  # halfway
        np.array([0.0, -0.0, 65504.0, 65520.0, 65519.9, 1e5, -1e5, 6.1e-5, 6.0e-5, 5.96e-8, 1e-10, np.inf, -np.inf],
                 np.float32)])
    np.savez_compressed(os.path.join(HERE, "f16.npz"), f16_to_f32=f.view(np.uint32), f32_in=xs.view(np.uint32),
                        f32_to_f16=ref.f32_to_f16(xs))

    np.savez_compressed(os.path.join(HERE, "tables.npz"),
                        grid=np.array([ref.lib.ref_grid(i) for i in range(256)], np.uint32),
                        ksigns=np.array([ref.lib.ref_ksigns(i) for i in range(128)], np.uint8),
                        kvalues=np.array([ref.lib.ref_kvalues(i) for i in range(16)], np.int8),
                        block_bytes=np.array([ref.lib.ref_block_bytes(t) for t in (8, 14, 23, 18)], np.uint32))

    assert om.ReferenceLayer.available(), "reference layer loop not built: cannot regenerate the layer fixtures"
    ref_layer = om.ReferenceLayer()
    dims = syn.Dims(n_embd=512, n_ff=256, n_expert=16, n_used=4)
    for tag, rt, gt, dt in (("a", syn.F16, syn.IQ3_XXS, syn.IQ4_XS), ("b", syn.F32, syn.IQ4_XS, syn.Q6_K),
                            ("c", syn.F32, syn.IQ3_XXS, syn.IQ4_XS)):
        layer = syn.make_layer(dims, seed=1234, layer=3, router_type=rt, gateup_type=gt, down_type=dt)
        x = syn.random_x(3, dims.n_embd, seed=4321)
        out = orc.moe_layer(layer, x, want_h=True)
        y, ids, w, ws, source = out["y"], out["sel"]["ids"], out["sel"]["w"], out["sel"]["w_shared"], "oracle"
        if rt == syn.F32:   # what the reference's loader accepts: its own loop produces the fixture
            r = ref_layer.moe_layer(layer, x)
            assert np.array_equal(r["y"].view(np.uint32), y.view(np.uint32)), "oracle and moeCpuRef disagree"
            assert np.array_equal(r["ids"], ids)
            y, ids, w, ws, source = r["y"], r["ids"], r["w"].astype(np.float32), r["w_shared"].astype(np.float32), "moeCpuRef"
        np.savez_compressed(os.path.join(HERE, f"moe_small_{tag}.npz"), x=x, y=y, ids=ids, w=w, w_shared=ws, h=out["h"],
                            types=np.array([rt, gt, dt]), dims=np.array([512, 256, 16, 4]), source=source)
    print("golden fixtures written to", HERE)


if __name__ == "__main__":
    main()
