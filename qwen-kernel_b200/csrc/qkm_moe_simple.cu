// Expert gate/up + SwiGLU and down projections, shape-generic form: one warp per
// output element, reading raw ggml blocks in place.
//
// These kernels accept every shape the ABI allows (any n_embd / n_ff that is a
// multiple of 256, n_expert <= 512, n_used <= 16) and every tensor type the
// reference loads (src/main.cpp:1283-1291).  They are the op-level entry points'
// implementation and the fall-back of the fused calls for shapes the streaming
// kernels do not cover.
//
// Reference kernels replaced: moe_gateup_iq3.comp / moe_gateup_iq4.comp (token
// major), moe_gateup_iq3_grouped.comp (expert major), moe_gateup_q8.comp (shared),
// moe_down_iq4.comp / moe_down_q6k.comp, moe_down_*_grouped.comp (contrib),
// moe_down_q8b.comp (shared), and the slot-order fold of add_rms3_grouped.comp:22-27.
#include "qkm_common.cuh"
#include "qkm_kernels.h"

namespace qkm {

// dot of one quantised row with one f32 vector, lane-strided over 8-element units
template <int TYPE>
__device__ __forceinline__ float row_dot(const uint8_t* __restrict__ row, const float* __restrict__ v,
                                         uint32_t K, uint32_t lane) {
    float acc = 0.f;
    for (uint32_t u = lane; u < K / 8; u += 32) {
        float w[8];
        dequant8<TYPE>(row, u * 8, w);
        const float4 a = *reinterpret_cast<const float4*>(v + u * 8);
        const float4 b = *reinterpret_cast<const float4*>(v + u * 8 + 4);
        acc += w[0] * a.x; acc += w[1] * a.y; acc += w[2] * a.z; acc += w[3] * a.w;
        acc += w[4] * b.x; acc += w[5] * b.y; acc += w[6] * b.z; acc += w[7] * b.w;
    }
    return acc;
}

// gate and up rows against the same vector (shares the x loads)
template <int TYPE>
__device__ __forceinline__ void row_dot2(const uint8_t* __restrict__ g, const uint8_t* __restrict__ u_,
                                         const float* __restrict__ v, uint32_t K, uint32_t lane,
                                         float& ag, float& au) {
    ag = 0.f; au = 0.f;
    for (uint32_t u = lane; u < K / 8; u += 32) {
        float wg[8], wu[8];
        dequant8<TYPE>(g, u * 8, wg);
        dequant8<TYPE>(u_, u * 8, wu);
        const float4 a = *reinterpret_cast<const float4*>(v + u * 8);
        const float4 b = *reinterpret_cast<const float4*>(v + u * 8 + 4);
        const float xv[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
#pragma unroll
        for (int i = 0; i < 8; ++i) { ag += wg[i] * xv[i]; au += wu[i] * xv[i]; }
    }
}

// ---- routed gate/up, token major: warp per (token, slot, row) -----------------------------
template <int TYPE>
__global__ void __launch_bounds__(256)
gateup_tokens_kernel(const uint8_t* __restrict__ gate, const uint8_t* __restrict__ up,
                     const float* __restrict__ x, const qkm_sel* __restrict__ sel, float* __restrict__ h,
                     qkm_dims d, uint32_t efirst, uint32_t ecount) {
    const uint32_t lane = threadIdx.x & 31u;
    const uint32_t r = blockIdx.x * 8u + (threadIdx.x >> 5);
    const uint32_t s = blockIdx.y, t = blockIdx.z;
    if (r >= d.n_ff) return;
    const uint32_t e = min(sel[t].ids[s], d.n_expert - 1) - efirst;
    float* out = h + ((size_t)t * (d.n_used + 1) + s) * d.n_ff + r;
    if (e >= ecount) { if (lane == 0) *out = 0.f; return; }
    const size_t rb = row_bytes(TYPE, d.n_embd);
    const size_t ro = ((size_t)e * d.n_ff + r) * rb;
    float ag, au;
    row_dot2<TYPE>(gate + ro, up + ro, x + (size_t)t * d.n_embd, d.n_embd, lane, ag, au);
    ag = warp_sum(ag); au = warp_sum(au);
    if (lane == 0) *out = swiglu(ag, au);
}

cudaError_t launch_gateup_tokens(const Launch& L, const qkm_dims& d, uint32_t type, const void* gate,
                                 const void* up, const float* x, const qkm_sel* sel, float* h,
                                 uint32_t n_tokens, uint32_t efirst, uint32_t ecount) {
    if (n_tokens == 0) return cudaSuccess;
    if (ecount == 0) { efirst = 0; ecount = d.n_expert; }
    const dim3 grid((d.n_ff + 7) / 8, d.n_used, n_tokens);
    const uint8_t *g = (const uint8_t*)gate, *u = (const uint8_t*)up;
    if (type == QKM_TYPE_IQ3_XXS)
        gateup_tokens_kernel<QKM_TYPE_IQ3_XXS><<<grid, 256, 0, L.stream>>>(g, u, x, sel, h, d, efirst, ecount);
    else if (type == QKM_TYPE_IQ4_XS)
        gateup_tokens_kernel<QKM_TYPE_IQ4_XS><<<grid, 256, 0, L.stream>>>(g, u, x, sel, h, d, efirst, ecount);
    else
        return cudaErrorInvalidValue;
    L.count();
    return cudaGetLastError();
}

// ---- routed gate/up, expert major: warp per (expert, row), loops the expert's pairs -----------
template <int TYPE>
__global__ void __launch_bounds__(256)
gateup_pairs_kernel(const uint8_t* __restrict__ gate, const uint8_t* __restrict__ up,
                    const float* __restrict__ x, const uint32_t* __restrict__ offsets,
                    const uint32_t* __restrict__ pairs, float* __restrict__ h, qkm_dims d) {
    const uint32_t lane = threadIdx.x & 31u;
    const uint32_t r = blockIdx.x * 8u + (threadIdx.x >> 5);
    const uint32_t e = blockIdx.y;
    if (r >= d.n_ff) return;
    const uint32_t p0 = offsets[e], p1 = offsets[e + 1];
    const size_t rb = row_bytes(TYPE, d.n_embd);
    const size_t ro = ((size_t)e * d.n_ff + r) * rb;
    for (uint32_t p = p0; p < p1; ++p) {
        const uint32_t pr = pairs[p], t = pr >> 4, s = pr & 15u;
        float ag, au;
        row_dot2<TYPE>(gate + ro, up + ro, x + (size_t)t * d.n_embd, d.n_embd, lane, ag, au);
        ag = warp_sum(ag); au = warp_sum(au);
        if (lane == 0) h[((size_t)t * (d.n_used + 1) + s) * d.n_ff + r] = swiglu(ag, au);
    }
}

cudaError_t launch_gateup_pairs(const Launch& L, const qkm_dims& d, uint32_t type, const void* gate,
                                const void* up, const float* x, const uint32_t* offsets,
                                const uint32_t* pairs, float* h, uint32_t n_tokens, uint32_t efirst,
                                uint32_t ecount) {
    (void)efirst;
    if (n_tokens == 0) return cudaSuccess;
    if (ecount == 0) ecount = d.n_expert;
    const dim3 grid((d.n_ff + 7) / 8, ecount);
    const uint8_t *g = (const uint8_t*)gate, *u = (const uint8_t*)up;
    if (type == QKM_TYPE_IQ3_XXS)
        gateup_pairs_kernel<QKM_TYPE_IQ3_XXS><<<grid, 256, 0, L.stream>>>(g, u, x, offsets, pairs, h, d);
    else if (type == QKM_TYPE_IQ4_XS)
        gateup_pairs_kernel<QKM_TYPE_IQ4_XS><<<grid, 256, 0, L.stream>>>(g, u, x, offsets, pairs, h, d);
    else
        return cudaErrorInvalidValue;
    L.count();
    return cudaGetLastError();
}

// ---- shared expert gate/up (Q8_0): warp per (token, row) -> h[t][n_used][r] ----------------------
__global__ void __launch_bounds__(256)
shared_gateup_kernel(const uint8_t* __restrict__ gate, const uint8_t* __restrict__ up,
                     const float* __restrict__ x, float* __restrict__ h, qkm_dims d) {
    const uint32_t lane = threadIdx.x & 31u;
    const uint32_t r = blockIdx.x * 8u + (threadIdx.x >> 5);
    const uint32_t t = blockIdx.y;
    if (r >= d.n_ff) return;
    const size_t ro = (size_t)r * row_bytes(QKM_TYPE_Q8_0, d.n_embd);
    float ag, au;
    row_dot2<QKM_TYPE_Q8_0>(gate + ro, up + ro, x + (size_t)t * d.n_embd, d.n_embd, lane, ag, au);
    ag = warp_sum(ag); au = warp_sum(au);
    if (lane == 0) h[((size_t)t * (d.n_used + 1) + d.n_used) * d.n_ff + r] = swiglu(ag, au);
}

cudaError_t launch_shared_gateup(const Launch& L, const qkm_dims& d, const void* gate, const void* up,
                                 const float* x, float* h, uint32_t n_tokens) {
    if (n_tokens == 0) return cudaSuccess;
    const dim3 grid((d.n_ff + 7) / 8, n_tokens);
    shared_gateup_kernel<<<grid, 256, 0, L.stream>>>((const uint8_t*)gate, (const uint8_t*)up, x, h, d);
    L.count();
    return cudaGetLastError();
}

// ---- routed down, token major: warp per (token, output) ---------------------------------------------
// y[t][o] = sum_s w_s * (D[ids_s][o] . h[t][s])  (+ w_shared * (DS[o] . h[t][n_used]) when
// down_shared is given).  The routing weight multiplies each lane's partial before the
// lane reduction, as moe_down_iq4.comp:70 does.
template <int TYPE>
__global__ void __launch_bounds__(256)
down_tokens_kernel(const uint8_t* __restrict__ down, const uint8_t* __restrict__ down_shared,
                   const float* __restrict__ h, const qkm_sel* __restrict__ sel, float* __restrict__ y,
                   qkm_dims d, uint32_t efirst, uint32_t ecount) {
    const uint32_t lane = threadIdx.x & 31u;
    const uint32_t o = blockIdx.x * 8u + (threadIdx.x >> 5);
    const uint32_t t = blockIdx.y;
    if (o >= d.n_embd) return;
    const size_t rb = row_bytes(TYPE, d.n_ff);
    const float* ht = h + (size_t)t * (d.n_used + 1) * d.n_ff;
    float acc = 0.f;
    for (uint32_t s = 0; s < d.n_used; ++s) {
        const uint32_t e = min(sel[t].ids[s], d.n_expert - 1) - efirst;
        if (e >= ecount) continue;
        const float part = row_dot<TYPE>(down + ((size_t)e * d.n_embd + o) * rb, ht + (size_t)s * d.n_ff, d.n_ff, lane);
        acc += sel[t].w[s] * part;
    }
    if (down_shared != nullptr) {
        const float part = row_dot<QKM_TYPE_Q8_0>(down_shared + (size_t)o * row_bytes(QKM_TYPE_Q8_0, d.n_ff),
                                                  ht + (size_t)d.n_used * d.n_ff, d.n_ff, lane);
        acc += sel[t].w_shared * part;
    }
    acc = warp_sum(acc);
    if (lane == 0) y[(size_t)t * d.n_embd + o] = acc;
}

cudaError_t launch_down_tokens(const Launch& L, const qkm_dims& d, uint32_t type, const void* down,
                               const float* h, const qkm_sel* sel, float* y, uint32_t n_tokens,
                               uint32_t efirst, uint32_t ecount, const void* down_shared) {
    if (n_tokens == 0) return cudaSuccess;
    if (ecount == 0) { efirst = 0; ecount = d.n_expert; }
    const dim3 grid((d.n_embd + 7) / 8, n_tokens);
    const uint8_t *w = (const uint8_t*)down, *ws = (const uint8_t*)down_shared;
    if (type == QKM_TYPE_IQ4_XS)
        down_tokens_kernel<QKM_TYPE_IQ4_XS><<<grid, 256, 0, L.stream>>>(w, ws, h, sel, y, d, efirst, ecount);
    else if (type == QKM_TYPE_Q6_K)
        down_tokens_kernel<QKM_TYPE_Q6_K><<<grid, 256, 0, L.stream>>>(w, ws, h, sel, y, d, efirst, ecount);
    else
        return cudaErrorInvalidValue;
    L.count();
    return cudaGetLastError();
}

// ---- routed down, expert major: per-(token, slot) contributions ----------------------------------------
template <int TYPE>
__global__ void __launch_bounds__(256)
down_pairs_kernel(const uint8_t* __restrict__ down, const float* __restrict__ h,
                  const qkm_sel* __restrict__ sel, const uint32_t* __restrict__ offsets,
                  const uint32_t* __restrict__ pairs, float* __restrict__ contrib, qkm_dims d) {
    const uint32_t lane = threadIdx.x & 31u;
    const uint32_t o = blockIdx.x * 8u + (threadIdx.x >> 5);
    const uint32_t e = blockIdx.y;
    if (o >= d.n_embd) return;
    const uint32_t p0 = offsets[e], p1 = offsets[e + 1];
    const uint8_t* row = down + ((size_t)e * d.n_embd + o) * row_bytes(TYPE, d.n_ff);
    for (uint32_t p = p0; p < p1; ++p) {
        const uint32_t pr = pairs[p], t = pr >> 4, s = pr & 15u;
        float part = row_dot<TYPE>(row, h + ((size_t)t * (d.n_used + 1) + s) * d.n_ff, d.n_ff, lane);
        part = warp_sum(part);
        // routing weight after the full K reduction (moe_down_iq4_grouped_coopmat.comp:160-161)
        if (lane == 0) contrib[((size_t)t * d.n_used + s) * d.n_embd + o] = sel[t].w[s] * part;
    }
}

cudaError_t launch_down_pairs(const Launch& L, const qkm_dims& d, uint32_t type, const void* down,
                              const float* h, const qkm_sel* sel, const uint32_t* offsets,
                              const uint32_t* pairs, float* contrib, uint32_t n_tokens, uint32_t efirst,
                              uint32_t ecount) {
    (void)efirst;
    if (n_tokens == 0) return cudaSuccess;
    if (ecount == 0) ecount = d.n_expert;
    const dim3 grid((d.n_embd + 7) / 8, ecount);
    const uint8_t* w = (const uint8_t*)down;
    if (type == QKM_TYPE_IQ4_XS)
        down_pairs_kernel<QKM_TYPE_IQ4_XS><<<grid, 256, 0, L.stream>>>(w, h, sel, offsets, pairs, contrib, d);
    else if (type == QKM_TYPE_Q6_K)
        down_pairs_kernel<QKM_TYPE_Q6_K><<<grid, 256, 0, L.stream>>>(w, h, sel, offsets, pairs, contrib, d);
    else
        return cudaErrorInvalidValue;
    L.count();
    return cudaGetLastError();
}

// ---- shared down: y2[t][o] = w_shared * (DS[o] . h[t][n_used]) ------------------------------------------------
// With `contrib` the routed per-slot contributions are folded in, slots in order, then the
// shared term: the sum add_rms3_grouped.comp:22-27 forms.
__global__ void __launch_bounds__(256)
shared_down_kernel(const uint8_t* __restrict__ down, const float* __restrict__ h,
                   const qkm_sel* __restrict__ sel, float* __restrict__ y2, qkm_dims d,
                   const float* __restrict__ contrib) {
    const uint32_t lane = threadIdx.x & 31u;
    const uint32_t o = blockIdx.x * 8u + (threadIdx.x >> 5);
    const uint32_t t = blockIdx.y;
    if (o >= d.n_embd) return;
    float part = row_dot<QKM_TYPE_Q8_0>(down + (size_t)o * row_bytes(QKM_TYPE_Q8_0, d.n_ff),
                                        h + ((size_t)t * (d.n_used + 1) + d.n_used) * d.n_ff, d.n_ff, lane);
    part = warp_sum(part);
    if (lane == 0) {
        const float shared = sel[t].w_shared * part;
        if (contrib != nullptr) {
            float v = 0.f;
            for (uint32_t s = 0; s < d.n_used; ++s) v += contrib[((size_t)t * d.n_used + s) * d.n_embd + o];
            y2[(size_t)t * d.n_embd + o] = v + shared;
        } else {
            y2[(size_t)t * d.n_embd + o] = shared;
        }
    }
}

cudaError_t launch_shared_down(const Launch& L, const qkm_dims& d, const void* down, const float* h,
                               const qkm_sel* sel, float* y2, uint32_t n_tokens, const float* contrib) {
    if (n_tokens == 0) return cudaSuccess;
    const dim3 grid((d.n_embd + 7) / 8, n_tokens);
    shared_down_kernel<<<grid, 256, 0, L.stream>>>((const uint8_t*)down, h, sel, y2, d, contrib);
    L.count();
    return cudaGetLastError();
}

// ---- fold: y[t][o] = (sum_s contrib[t][s][o]) + y2[t][o], slots in order ----------------------------------------
__global__ void fold_contrib_kernel(const float* __restrict__ contrib, const float* __restrict__ y2,
                                    float* __restrict__ y, uint32_t n_used, uint32_t n_embd, size_t n) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const size_t t = i / n_embd, o = i - t * n_embd;
    float v = 0.f;
    for (uint32_t s = 0; s < n_used; ++s) v += contrib[(t * n_used + s) * n_embd + o];
    y[i] = v + (y2 ? y2[i] : 0.f);
}

cudaError_t launch_fold_contrib(const Launch& L, const qkm_dims& d, const float* contrib, const float* y2,
                                float* y, uint32_t n_tokens) {
    if (n_tokens == 0) return cudaSuccess;
    const size_t n = (size_t)n_tokens * d.n_embd;
    fold_contrib_kernel<<<(unsigned)((n + 255) / 256), 256, 0, L.stream>>>(contrib, y2, y, d.n_used, d.n_embd, n);
    L.count();
    return cudaGetLastError();
}

}  // namespace qkm
