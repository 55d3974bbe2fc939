// CPU oracle for the quantized MoE feed-forward path.  TEST INFRASTRUCTURE ONLY:
// nothing that ships may call into this file; it exists so the CUDA kernels can
// be checked against the reference's CPU semantics, and so the bench can time
// that CPU path on the host cores.
//
// Parity status: PINNED.  Every dequantiser here is compared bit-for-bit with
// the reference's own src/quants.h (compiled as oracle/_ref/libqk_ref.so by
// oracle/Makefile) over random blocks of every format and over all 65536 f16
// bit patterns; the outputs of that reference build are committed as fixtures
// under tests/golden/ so the same check runs where the reference tree is absent.
//
// What each function restates (file:line under the reference tree):
//   orc_f16_to_f32 / orc_f32_to_f16   src/quants.h:12-48
//   orc_dequant_row                   src/quants.h:70-165
//   orc_gemv                          src/main.cpp:627-635, :673-679
//   orc_moe_route                     src/main.cpp:1320-1344 (+ the non-finite
//                                     floor of shaders/moe_select.comp:28-34 and the
//                                     lowest-id tie rule of moe_select_256.comp:60-61)
//   orc_moe_layer                     src/main.cpp:1316-1387 (moeCpuRef)
//   orc_group_pairs                   shaders/moe_group_pairs.comp:19-50
//   orc_select_f32                    shaders/moe_select.comp:24-76
//
// Two accumulation modes: ORC_ACC_F64 is the reference's (double accumulators,
// float hrow, float y += (float)(w*a)); ORC_ACC_F32 is the "scalar f32 loop"
// CPU path that the bench times (same loops, float accumulators).

#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <functional>
#include <thread>
#include <vector>

#include "../include/qk_moe.h"

#define ORC_API extern "C" __attribute__((visibility("default")))

enum { ORC_ACC_F64 = 0, ORC_ACC_F32 = 1 };

namespace {

const uint32_t kGrid[256] = {
#define QKM_G(x) x,
#include "../qwen-kernel_b200/csrc/qkm_tables.inc"
};
const int8_t kIq4nl[16] = {-127, -104, -83, -65, -49, -35, -22, -10, 1, 13, 25, 38, 53, 69, 89, 113};

inline uint8_t signs8(uint32_t s7) { return (uint8_t)(s7 | ((__builtin_popcount(s7) & 1u) << 7)); }

inline float f16_to_f32(uint16_t h) {
    const uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    uint32_t e = (h >> 10) & 0x1Fu, m = h & 0x3FFu, bits;
    if (e == 0) {
        if (m == 0) {
            bits = sign;
        } else {  // subnormal: normalise
            int shift = 0;
            while (!(m & 0x400u)) { m <<= 1; ++shift; }
            bits = sign | ((uint32_t)(113 - shift) << 23) | ((m & 0x3FFu) << 13);
        }
    } else if (e == 31) {
        bits = sign | 0x7F800000u | (m << 13);
    } else {
        bits = sign | ((e + 112u) << 23) | (m << 13);
    }
    float f;
    memcpy(&f, &bits, 4);
    return f;
}

// Round-to-nearest-even; flushes results below the f16 normal range to signed
// zero and saturates overflow (and NaN) to infinity, as src/quants.h:36-48 does.
inline uint16_t f32_to_f16(float f) {
    uint32_t x;
    memcpy(&x, &f, 4);
    const uint32_t sign = (x >> 16) & 0x8000u;
    const int32_t e = (int32_t)((x >> 23) & 0xFF) - 112;
    const uint32_t m = x & 0x7FFFFFu;
    if (e <= 0) return (uint16_t)sign;
    if (e >= 31) return (uint16_t)(sign | 0x7C00u);
    uint32_t h = sign | ((uint32_t)e << 10) | (m >> 13);
    const uint32_t rest = m & 0x1FFFu;
    if (rest > 0x1000u || (rest == 0x1000u && (h & 1u))) ++h;
    return (uint16_t)h;
}

inline uint16_t rd16(const uint8_t* p) { uint16_t v; memcpy(&v, p, 2); return v; }
inline uint32_t rd32(const uint8_t* p) { uint32_t v; memcpy(&v, p, 4); return v; }

// ---- per-format row dequantisers (block byte layouts: src/quants.h:52-66, :107-119)

void dq_q8_0(const uint8_t* b, float* y, int64_t k) {
    for (int64_t i = 0; i < k / 32; ++i, b += 34) {
        const float d = f16_to_f32(rd16(b));
        const int8_t* q = (const int8_t*)(b + 2);
        for (int j = 0; j < 32; ++j) *y++ = d * q[j];
    }
}

void dq_q6_k(const uint8_t* b, float* y, int64_t k) {
    for (int64_t i = 0; i < k / 256; ++i, b += 210) {
        const uint8_t* ql = b;
        const uint8_t* qh = b + 128;
        const int8_t* sc = (const int8_t*)(b + 192);
        const float d = f16_to_f32(rd16(b + 208));
        for (int half = 0; half < 2; ++half) {
            for (int l = 0; l < 32; ++l) {
                const int is = l / 16;
                const int8_t q1 = (int8_t)((ql[l] & 0xF) | (((qh[l] >> 0) & 3) << 4)) - 32;
                const int8_t q2 = (int8_t)((ql[l + 32] & 0xF) | (((qh[l] >> 2) & 3) << 4)) - 32;
                const int8_t q3 = (int8_t)((ql[l] >> 4) | (((qh[l] >> 4) & 3) << 4)) - 32;
                const int8_t q4 = (int8_t)((ql[l + 32] >> 4) | (((qh[l] >> 6) & 3) << 4)) - 32;
                y[l] = d * sc[is] * q1;
                y[l + 32] = d * sc[is + 2] * q2;
                y[l + 64] = d * sc[is + 4] * q3;
                y[l + 96] = d * sc[is + 6] * q4;
            }
            y += 128; ql += 64; qh += 32; sc += 8;
        }
    }
}

void dq_iq4_xs(const uint8_t* b, float* y, int64_t k) {
    for (int64_t i = 0; i < k / 256; ++i, b += 136) {
        const float d = f16_to_f32(rd16(b));
        const uint32_t sh = rd16(b + 2);
        const uint8_t* sl = b + 4;
        const uint8_t* qs = b + 8;
        for (int ib = 0; ib < 8; ++ib, qs += 16, y += 32) {
            const int ls = (int)((sl[ib / 2] >> (4 * (ib % 2))) & 0xF) | (int)(((sh >> (2 * ib)) & 3) << 4);
            const float dl = d * (ls - 32);
            for (int j = 0; j < 16; ++j) {
                y[j] = dl * kIq4nl[qs[j] & 0xF];
                y[j + 16] = dl * kIq4nl[qs[j] >> 4];
            }
        }
    }
}

void dq_iq3_xxs(const uint8_t* b, float* y, int64_t k) {
    for (int64_t i = 0; i < k / 256; ++i, b += 98) {
        const float d = f16_to_f32(rd16(b));
        const uint8_t* qs = b + 2;
        const uint8_t* aux = b + 2 + 64;
        for (int ib = 0; ib < 8; ++ib, qs += 8) {
            const uint32_t a = rd32(aux + 4 * ib);
            const float db = d * (0.5f + (float)(a >> 28)) * 0.5f;
            for (int l = 0; l < 4; ++l, y += 8) {
                const uint8_t sg = signs8((a >> (7 * l)) & 127u);
                const uint32_t g1 = kGrid[qs[2 * l]], g2 = kGrid[qs[2 * l + 1]];
                for (int j = 0; j < 4; ++j) {
                    y[j] = db * (float)((g1 >> (8 * j)) & 255u) * ((sg >> j) & 1 ? -1.f : 1.f);
                    y[j + 4] = db * (float)((g2 >> (8 * j)) & 255u) * ((sg >> (j + 4)) & 1 ? -1.f : 1.f);
                }
            }
        }
    }
}

void dq_f16(const uint8_t* b, float* y, int64_t k) {
    for (int64_t i = 0; i < k; ++i) y[i] = f16_to_f32(rd16(b + 2 * i));
}
void dq_f32(const uint8_t* b, float* y, int64_t k) { memcpy(y, b, (size_t)k * 4); }

size_t row_bytes(uint32_t type, uint64_t ne0) {
    switch (type) {
        case QKM_TYPE_F32: return ne0 * 4;
        case QKM_TYPE_F16: return ne0 * 2;
        case QKM_TYPE_Q8_0: return ne0 / 32 * 34;
        case QKM_TYPE_Q6_K: return ne0 / 256 * 210;
        case QKM_TYPE_IQ4_XS: return ne0 / 256 * 136;
        case QKM_TYPE_IQ3_XXS: return ne0 / 256 * 98;
        default: return 0;
    }
}

bool dequant(uint32_t type, const void* blocks, float* y, int64_t k) {
    const uint8_t* b = (const uint8_t*)blocks;
    switch (type) {
        case QKM_TYPE_F32: dq_f32(b, y, k); return true;
        case QKM_TYPE_F16: dq_f16(b, y, k); return true;
        case QKM_TYPE_Q8_0: dq_q8_0(b, y, k); return true;
        case QKM_TYPE_Q6_K: dq_q6_k(b, y, k); return true;
        case QKM_TYPE_IQ4_XS: dq_iq4_xs(b, y, k); return true;
        case QKM_TYPE_IQ3_XXS: dq_iq3_xxs(b, y, k); return true;
        default: return false;
    }
}

template <class Acc>
inline Acc dot(const float* a, const float* b, uint32_t n) {
    Acc s = 0;
    for (uint32_t k = 0; k < n; ++k) s += (Acc)a[k] * (Acc)b[k];
    return s;
}

void parallel_for(uint32_t n, int threads, const std::function<void(uint32_t, uint32_t)>& body) {
    if (threads <= 1 || n < 2) { body(0, n); return; }
    const uint32_t nt = std::min<uint32_t>((uint32_t)threads, n);
    std::vector<std::thread> pool;
    for (uint32_t t = 0; t < nt; ++t) {
        const uint32_t lo = (uint64_t)n * t / nt, hi = (uint64_t)n * (t + 1) / nt;
        pool.emplace_back([=, &body] { body(lo, hi); });
    }
    for (auto& th : pool) th.join();
}

struct SelD { uint32_t ids[16]; double w[16]; double w_shared; };

// Router + selection in doubles (src/main.cpp:1320-1344).  A non-finite logit is
// replaced by the floor -3.4e38 before ranking (shaders/moe_select.comp:28-34);
// among equal logits the lower expert id ranks first (moe_select_256.comp:60-61).
void route_one(const qkm_dims& d, uint32_t router_type, const void* router, const float* gis,
               const float* x, SelD* out) {
    std::vector<double> logit(d.n_expert);
    std::vector<float> row(d.n_embd);
    const size_t rb = row_bytes(router_type, d.n_embd);
    for (uint32_t e = 0; e < d.n_expert; ++e) {
        const float* w;
        if (router_type == QKM_TYPE_F32) {
            w = (const float*)router + (size_t)e * d.n_embd;
        } else {
            dequant(router_type, (const uint8_t*)router + e * rb, row.data(), d.n_embd);
            w = row.data();
        }
        double a = dot<double>(w, x, d.n_embd);
        if (!std::isfinite(a)) a = -3.4e38;
        logit[e] = a;
    }
    std::vector<uint32_t> order(d.n_expert);
    for (uint32_t e = 0; e < d.n_expert; ++e) order[e] = e;
    std::stable_sort(order.begin(), order.end(),
                     [&](uint32_t a, uint32_t b) { return logit[a] > logit[b]; });
    const double mx = logit[order[0]];
    double sum = 0;
    for (uint32_t i = 0; i < d.n_used; ++i) {
        out->ids[i] = order[i];
        out->w[i] = std::exp(logit[order[i]] - mx);
        sum += out->w[i];
    }
    for (uint32_t i = 0; i < d.n_used; ++i) out->w[i] /= sum;
    const double sg = dot<double>(gis, x, d.n_embd);
    out->w_shared = 1.0 / (1.0 + std::exp(-sg));
}

template <class Acc>
inline Acc silu(Acc v) { return v / ((Acc)1 + std::exp(-v)); }

// One token through one layer (src/main.cpp:1346-1386).  `experts_first/count`
// restrict which selected experts contribute (expert-parallel partial sums);
// the shared expert is added only when `with_shared`.
template <class Acc>
void layer_one(const qkm_dims& d, const qkm_layer_weights& L, const float* x, const SelD& sel,
               float* y, float* h_out, uint32_t exp_first, uint32_t exp_count, bool with_shared,
               float* contrib) {
    const size_t rbGU = row_bytes(L.gateup_type, d.n_embd);
    const size_t rbD = row_bytes(L.down_type, d.n_ff);
    const size_t rbSG = row_bytes(QKM_TYPE_Q8_0, d.n_embd);
    const size_t rbSD = row_bytes(QKM_TYPE_Q8_0, d.n_ff);
    std::vector<float> tmpE(d.n_embd), tmpF(d.n_ff), hrow(d.n_ff);
    for (uint32_t o = 0; o < d.n_embd; ++o) y[o] = 0.f;
    for (uint32_t s = 0; s < d.n_used; ++s) {
        const uint32_t e = sel.ids[s];
        if (e < exp_first || e >= exp_first + exp_count) {
            if (h_out) for (uint32_t r = 0; r < d.n_ff; ++r) h_out[(size_t)s * d.n_ff + r] = 0.f;
            if (contrib) for (uint32_t o = 0; o < d.n_embd; ++o) contrib[(size_t)s * d.n_embd + o] = 0.f;
            continue;
        }
        const uint8_t* G = (const uint8_t*)L.gate_exps + (size_t)(e - exp_first) * d.n_ff * rbGU;
        const uint8_t* U = (const uint8_t*)L.up_exps + (size_t)(e - exp_first) * d.n_ff * rbGU;
        const uint8_t* D = (const uint8_t*)L.down_exps + (size_t)(e - exp_first) * d.n_embd * rbD;
        for (uint32_t r = 0; r < d.n_ff; ++r) {
            dequant(L.gateup_type, G + r * rbGU, tmpE.data(), d.n_embd);
            const Acc ga = dot<Acc>(tmpE.data(), x, d.n_embd);
            dequant(L.gateup_type, U + r * rbGU, tmpE.data(), d.n_embd);
            const Acc ua = dot<Acc>(tmpE.data(), x, d.n_embd);
            hrow[r] = (float)(silu<Acc>(ga) * ua);
        }
        if (h_out) memcpy(h_out + (size_t)s * d.n_ff, hrow.data(), d.n_ff * 4);
        for (uint32_t o = 0; o < d.n_embd; ++o) {
            dequant(L.down_type, D + o * rbD, tmpF.data(), d.n_ff);
            const Acc a = dot<Acc>(tmpF.data(), hrow.data(), d.n_ff);
            const float c = (float)((Acc)sel.w[s] * a);
            y[o] += c;
            if (contrib) contrib[(size_t)s * d.n_embd + o] = c;
        }
    }
    if (!with_shared) return;
    for (uint32_t r = 0; r < d.n_ff; ++r) {
        dequant(QKM_TYPE_Q8_0, (const uint8_t*)L.gate_shexp + r * rbSG, tmpE.data(), d.n_embd);
        const Acc ga = dot<Acc>(tmpE.data(), x, d.n_embd);
        dequant(QKM_TYPE_Q8_0, (const uint8_t*)L.up_shexp + r * rbSG, tmpE.data(), d.n_embd);
        const Acc ua = dot<Acc>(tmpE.data(), x, d.n_embd);
        hrow[r] = (float)(silu<Acc>(ga) * ua);
    }
    if (h_out) memcpy(h_out + (size_t)d.n_used * d.n_ff, hrow.data(), d.n_ff * 4);
    for (uint32_t o = 0; o < d.n_embd; ++o) {
        dequant(QKM_TYPE_Q8_0, (const uint8_t*)L.down_shexp + o * rbSD, tmpF.data(), d.n_ff);
        const Acc a = dot<Acc>(tmpF.data(), hrow.data(), d.n_ff);
        y[o] += (float)((Acc)sel.w_shared * a);
    }
}

}  // namespace

// ---------------------------------------------------------------- C entry points

ORC_API float orc_f16_to_f32(uint16_t h) { return f16_to_f32(h); }
ORC_API uint16_t orc_f32_to_f16(float f) { return f32_to_f16(f); }
ORC_API void orc_f16_to_f32_n(const uint16_t* h, float* f, uint64_t n) {
    for (uint64_t i = 0; i < n; ++i) f[i] = f16_to_f32(h[i]);
}
ORC_API void orc_f32_to_f16_n(const float* f, uint16_t* h, uint64_t n) {
    for (uint64_t i = 0; i < n; ++i) h[i] = f32_to_f16(f[i]);
}
ORC_API size_t orc_row_bytes(uint32_t type, uint64_t ne0) { return row_bytes(type, ne0); }
ORC_API uint8_t orc_signs8(uint32_t s7) { return signs8(s7 & 127u); }

// dequant_row_*: n_elems values from consecutive blocks.
ORC_API int orc_dequant_row(uint32_t type, const void* blocks, float* y, int64_t n_elems) {
    return dequant(type, blocks, y, n_elems) ? 0 : -4;
}

// y[n][M] = W[M][K] . x[n][K]: dequantise the row, accumulate in k order, cast.
ORC_API int orc_gemv(uint32_t type, const void* W, const float* x, float* y, uint32_t M,
                     uint32_t K, uint32_t n, int acc, int threads) {
    const size_t rb = row_bytes(type, K);
    if (!rb) return -4;
    parallel_for(M, threads, [&](uint32_t lo, uint32_t hi) {
        std::vector<float> row(K);
        for (uint32_t m = lo; m < hi; ++m) {
            dequant(type, (const uint8_t*)W + (size_t)m * rb, row.data(), K);
            for (uint32_t t = 0; t < n; ++t) {
                const float* xt = x + (size_t)t * K;
                y[(size_t)t * M + m] = acc == ORC_ACC_F64 ? (float)dot<double>(row.data(), xt, K)
                                                           : dot<float>(row.data(), xt, K);
            }
        }
    });
    return 0;
}

// Router + top-k for T tokens.  sel gets f32 copies of the double weights;
// sel_w64 (optional, [T][17]) gets the doubles: w[0..15], w_shared.
ORC_API int orc_moe_route(const qkm_dims* d, uint32_t router_type, const void* router,
                          const float* gis, const float* x, uint32_t T, qkm_sel* sel,
                          double* sel_w64, int threads) {
    parallel_for(T, threads, [&](uint32_t lo, uint32_t hi) {
        for (uint32_t t = lo; t < hi; ++t) {
            SelD s{};
            route_one(*d, router_type, router, gis, x + (size_t)t * d->n_embd, &s);
            memset(&sel[t], 0, sizeof(qkm_sel));
            for (uint32_t i = 0; i < d->n_used; ++i) {
                sel[t].ids[i] = s.ids[i];
                sel[t].w[i] = (float)s.w[i];
                if (sel_w64) sel_w64[(size_t)t * 17 + i] = s.w[i];
            }
            sel[t].w_shared = (float)s.w_shared;
            if (sel_w64) sel_w64[(size_t)t * 17 + 16] = s.w_shared;
        }
    });
    return 0;
}

// Logits only, f32 accumulation in k order per expert (the value a scalar CPU
// loop over shaders/moe_logits.comp's formula gives).
ORC_API int orc_moe_logits(const qkm_dims* d, uint32_t router_type, const void* router,
                           const float* x, uint32_t T, float* logits, int acc) {
    std::vector<float> row(d->n_embd);
    const size_t rb = row_bytes(router_type, d->n_embd);
    for (uint32_t e = 0; e < d->n_expert; ++e) {
        dequant(router_type, (const uint8_t*)router + e * rb, row.data(), d->n_embd);
        for (uint32_t t = 0; t < T; ++t) {
            const float* xt = x + (size_t)t * d->n_embd;
            logits[(size_t)t * d->n_expert + e] =
                acc == ORC_ACC_F64 ? (float)dot<double>(row.data(), xt, d->n_embd)
                                   : dot<float>(row.data(), xt, d->n_embd);
        }
    }
    return 0;
}

// Selection from given f32 logits: n_used rounds of argmax with the non-finite
// floor, lowest id on ties, softmax over the selected logits in f32, w_shared
// from an f64 dot rounded to f32.
ORC_API int orc_select_f32(const qkm_dims* d, const float* logits, const float* gis,
                           const float* x, uint32_t T, qkm_sel* sel) {
    for (uint32_t t = 0; t < T; ++t) {
        std::vector<float> l(d->n_expert);
        for (uint32_t e = 0; e < d->n_expert; ++e) {
            const float v = logits[(size_t)t * d->n_expert + e];
            l[e] = std::isfinite(v) ? v : -3.4e38f;
        }
        memset(&sel[t], 0, sizeof(qkm_sel));
        float picked[16];
        for (uint32_t i = 0; i < d->n_used; ++i) {
            uint32_t best = 0;
            for (uint32_t e = 1; e < d->n_expert; ++e)
                if (l[e] > l[best]) best = e;
            sel[t].ids[i] = best;
            picked[i] = l[best];
            l[best] = -3.4e38f;
        }
        double sum = 0, wv[16];
        for (uint32_t i = 0; i < d->n_used; ++i) { wv[i] = std::exp((double)picked[i] - (double)picked[0]); sum += wv[i]; }
        for (uint32_t i = 0; i < d->n_used; ++i) sel[t].w[i] = (float)(wv[i] / sum);
        const double sg = dot<double>(gis, x + (size_t)t * d->n_embd, d->n_embd);
        sel[t].w_shared = (float)(1.0 / (1.0 + std::exp(-sg)));
    }
    return 0;
}

// Counting sort of (expert, token, slot) into per-expert ranges.  The order of
// pairs inside a range is unspecified in the reference (atomic cursors); here it
// is ascending (token, slot), and tests compare ranges as sets.
ORC_API int orc_group_pairs(const qkm_sel* sel, uint32_t T, uint32_t n_expert, uint32_t n_used,
                            uint32_t* offsets, uint32_t* pairs) {
    std::vector<uint32_t> count(n_expert + 1, 0);
    for (uint32_t t = 0; t < T; ++t)
        for (uint32_t s = 0; s < n_used; ++s) count[std::min(sel[t].ids[s], n_expert - 1)]++;
    uint32_t off = 0;
    std::vector<uint32_t> cursor(n_expert);
    for (uint32_t e = 0; e < n_expert; ++e) { offsets[e] = off; cursor[e] = off; off += count[e]; }
    offsets[n_expert] = off;
    for (uint32_t t = 0; t < T; ++t)
        for (uint32_t s = 0; s < n_used; ++s) {
            const uint32_t e = std::min(sel[t].ids[s], n_expert - 1);
            pairs[cursor[e]++] = (t << 4) | s;
        }
    return 0;
}

// The whole layer for T tokens.  Outputs (any may be NULL except y):
//   y [T][n_embd]; sel [T]; h [T][n_used+1][n_ff]; contrib [T][n_used][n_embd].
// sel_in (optional) supplies the routing instead of computing it (used to time
// or check the expert math under a given selection).  exp_first/exp_count limit
// the routed sum to resident experts (L.*_exps then hold only those);
// with_shared=0 leaves the shared expert out.
ORC_API int orc_moe_layer(const qkm_dims* d, const qkm_layer_weights* L, const float* x, uint32_t T,
                          float* y, qkm_sel* sel, float* h, float* contrib, const qkm_sel* sel_in,
                          uint32_t exp_first, uint32_t exp_count, int with_shared, int acc,
                          int threads) {
    if (exp_count == 0) { exp_first = 0; exp_count = d->n_expert; }
    parallel_for(T, threads, [&](uint32_t lo, uint32_t hi) {
        for (uint32_t t = lo; t < hi; ++t) {
            const float* xt = x + (size_t)t * d->n_embd;
            SelD s{};
            if (sel_in) {
                for (uint32_t i = 0; i < d->n_used; ++i) { s.ids[i] = sel_in[t].ids[i]; s.w[i] = sel_in[t].w[i]; }
                s.w_shared = sel_in[t].w_shared;
            } else {
                route_one(*d, L->router_type, L->router, L->gate_inp_shexp, xt, &s);
            }
            if (sel) {
                memset(&sel[t], 0, sizeof(qkm_sel));
                for (uint32_t i = 0; i < d->n_used; ++i) { sel[t].ids[i] = s.ids[i]; sel[t].w[i] = (float)s.w[i]; }
                sel[t].w_shared = (float)s.w_shared;
            }
            float* ht = h ? h + (size_t)t * (d->n_used + 1) * d->n_ff : nullptr;
            float* ct = contrib ? contrib + (size_t)t * d->n_used * d->n_embd : nullptr;
            if (acc == ORC_ACC_F64)
                layer_one<double>(*d, *L, xt, s, y + (size_t)t * d->n_embd, ht, exp_first, exp_count, with_shared != 0, ct);
            else
                layer_one<float>(*d, *L, xt, s, y + (size_t)t * d->n_embd, ht, exp_first, exp_count, with_shared != 0, ct);
        }
    });
    return 0;
}

ORC_API int orc_hardware_threads(void) { return (int)std::thread::hardware_concurrency(); }

// ---- residual adds + RMS norm (layer entry / tail) ------------------------------------------
// shaders/add_rmsnorm.comp:22-40, add_rms3.comp:23-41, add_rms3_grouped.comp:22-50; the CPU
// check of the reference accumulates the mean of squares in double (src/main.cpp:1688).
// mode 0: s = a + b; 1: s = (a + b) + c2; 2: s = (a + sum_k routed[row][k][:]) + c2.
// The sums are f32 in the shaders' order of additions; xn = s * scale * w with
// scale = 1 / sqrt(mean(s^2) + eps), mean in double.
ORC_API int orc_add_rms(int mode, const float* a, const float* b, const float* c2, const float* w, float* s,
                        float* xn, uint32_t n_rows, uint32_t n, uint32_t n_used, float eps) {
    for (uint32_t r = 0; r < n_rows; ++r) {
        double ss = 0.0;
        for (uint32_t i = 0; i < n; ++i) {
            float v = a[(size_t)r * n + i];
            if (mode == 2) {
                float acc = 0.f;
                for (uint32_t k = 0; k < n_used; ++k) acc += b[((size_t)r * n_used + k) * n + i];
                v += acc;
            } else {
                v += b[(size_t)r * n + i];
            }
            if (mode >= 1) v += c2[(size_t)r * n + i];
            s[(size_t)r * n + i] = v;
            ss += (double)v * (double)v;
        }
        const double scale = 1.0 / std::sqrt(ss / (double)n + (double)eps);
        for (uint32_t i = 0; i < n; ++i) xn[(size_t)r * n + i] = (float)((double)s[(size_t)r * n + i] * scale * (double)w[i]);
    }
    return 0;
}
