// Thin C wrapper around the REFERENCE's own CPU layer loop.  It contains no arithmetic of
// its own: oracle/Makefile cuts `struct MoeT` ... end of `moeCpuRef` out of the reference's
// src/main.cpp where it lies (that file as a whole needs <vulkan/vulkan.h>; this span needs
// only gguf.h, quants.h and the standard library) into oracle/_ref/moe_cpu_ref_span.inc, and
// this file #includes that span unchanged.  Tests compare the restated oracle with it bit for
// bit and tests/golden/make_golden.py generates the layer fixtures from it.  Built only
// where the reference tree exists; nothing under oracle/_ref/ is ever committed.
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <string>
#include <vector>

#include "gguf.h"    // reference: src/gguf.h
#include "quants.h"  // reference: src/quants.h

#include "moe_cpu_ref_span.inc"  // reference: src/main.cpp, struct MoeT .. moeCpuRef

#define REF_API extern "C" __attribute__((visibility("default")))

// Tensors as loadMoeT would find them in a file (router and shared gate F32, the only
// types it accepts).  ids[T][16], w[T][16] (f64), w_shared[T] (f64), y[T][n_embd].
REF_API int ref_moe_layer(uint32_t n_embd, uint32_t n_ff, uint32_t n_expert, uint32_t n_used,
                          uint32_t gateup_type, uint32_t down_type, const void* router, const void* gis,
                          const void* gate_exps, const void* up_exps, const void* down_exps,
                          const void* gate_shexp, const void* up_shexp, const void* down_shexp,
                          const float* x, uint32_t n_tokens, float* y, uint32_t* ids, double* w, double* w_shared) {
    if ((gateup_type != GGML_IQ3_XXS && gateup_type != GGML_IQ4_XS) || (down_type != GGML_IQ4_XS && down_type != GGML_Q6_K))
        return -4;
    GgufTensor t[8];
    const void* data[8] = {router, gis, gate_exps, up_exps, down_exps, gate_shexp, up_shexp, down_shexp};
    const uint32_t types[8] = {GGML_F32, GGML_F32, gateup_type, gateup_type, down_type, GGML_Q8_0, GGML_Q8_0, GGML_Q8_0};
    for (int i = 0; i < 8; ++i) { t[i].type = types[i]; t[i].data = (const uint8_t*)data[i]; }
    MoeT m{};
    m.gi = &t[0]; m.gis = &t[1]; m.ge = &t[2]; m.ue = &t[3]; m.de = &t[4]; m.gs = &t[5]; m.us = &t[6]; m.ds = &t[7];
    m.nEmbd = n_embd; m.nFf = n_ff; m.nExp = n_expert; m.nUsed = n_used;
    m.downQ6 = down_type == GGML_Q6_K;
    m.guIq4 = gateup_type == GGML_IQ4_XS;
    m.rbGE = ggmlRowBytes(gateup_type, n_embd);
    m.rbDE = ggmlRowBytes(down_type, n_ff);
    m.rbGS = ggmlRowBytes(GGML_Q8_0, n_embd);
    m.rbDS = ggmlRowBytes(GGML_Q8_0, n_ff);
    for (uint32_t tok = 0; tok < n_tokens; ++tok) {
        MoeRefSel sel{};
        moeCpuRef(m, x + (size_t)tok * n_embd, y + (size_t)tok * n_embd, &sel);
        for (uint32_t i = 0; i < 16; ++i) {
            ids[tok * 16 + i] = i < n_used ? sel.ids[i] : 0;
            w[tok * 16 + i] = i < n_used ? sel.w[i] : 0.0;
        }
        w_shared[tok] = sel.wShared;
    }
    return 0;
}
