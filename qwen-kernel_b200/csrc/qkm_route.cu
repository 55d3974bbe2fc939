// Router: logits, top-k selection, and token-expert pair grouping.
//
// Replaces moe_logits.comp / moe_logits_gemm.comp (logits), moe_select.comp /
// moe_select_256.comp (selection from f32 logits), moe_route_select[_hier].comp
// (both in one call) and moe_group_pairs.comp.
//
// Selection rules kept from the reference: a non-finite logit ranks as -3.4e38
// (moe_select.comp:28-34); among equal logits the lowest expert id ranks first
// (moe_select_256.comp:60-61); weights are a softmax over the selected logits
// only (moe_select.comp:71-76); w_shared = sigmoid(gate_inp_shexp . x)
// (moe_select.comp:36-45).
//
// The fused path additionally guarantees that ids equal those of a router that
// accumulates in f64 (the CPU reference, src/main.cpp:1320-1341): f32 logits
// carry a provable error bound eps, every expert whose f32 logit lies within
// 2*eps of the k-th largest is a candidate, candidates are re-evaluated in f64
// and the final ranking uses those values.
#include <math.h>

#include "qkm_common.cuh"
#include "qkm_kernels.h"
#include "qkm_stream.cuh"

namespace qkm {

static constexpr float kFloor = -3.4e38f;

// ---- logits: two expert rows per block, four warps (column quarters) per row ----------------
// Every lane owns at most kMaxUnits 8-element units of its quarter, loads them and the
// matching x values of kTokPerBlock tokens up front (one memory round trip), adds its
// products in a fixed order, then the lanes meet in a 5-level tree and the four quarters
// in shared memory: fewer sequential additions than the error bound of the refined
// selection assumes.  Also writes |router row|^2 when row_norm2 != NULL.
static constexpr int kTokPerBlock = 4;
static constexpr int kMaxUnits = 2;  // K <= 2048 in one pass; longer rows loop

// With ACC = double the logits are those of an f64-accumulating router outright (the f64
// pipe does the 2 * K * n_expert flops of a decode batch in well under a microsecond), and
// the selection needs no error bound or re-evaluation.
template <int TYPE, typename ACC>
__global__ void __launch_bounds__(256)
logits_kernel(const uint8_t* __restrict__ router, const float* __restrict__ x, ACC* __restrict__ logits,
              float* __restrict__ row_norm2, uint32_t n_expert, uint32_t K, uint32_t n_tokens) {
    __shared__ ACC s_part[8][kTokPerBlock + 1];
    pdl_trigger();
    pdl_wait();   // the logits buffer is reused from layer to layer
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
    const uint32_t e = blockIdx.x * 2u + (warp >> 2), quarter = warp & 3u;
    const uint32_t t0 = blockIdx.y * kTokPerBlock;
    const uint32_t units_q = K / 32;  // units per quarter
    ACC acc[kTokPerBlock], nrm = 0;
#pragma unroll
    for (int j = 0; j < kTokPerBlock; ++j) acc[j] = 0;
    if (e < n_expert) {
        const uint8_t* row = router + (size_t)e * row_bytes(TYPE, K);
        for (uint32_t u0 = lane; u0 < units_q; u0 += 32 * kMaxUnits) {
            float w[kMaxUnits][8];
            float4 xa[kMaxUnits][kTokPerBlock], xb[kMaxUnits][kTokPerBlock];
#pragma unroll
            for (int i = 0; i < kMaxUnits; ++i) {
                const uint32_t u = u0 + 32 * i;
                if (u < units_q) {
                    const uint32_t k = (quarter * units_q + u) * 8;
                    dequant8<TYPE>(row, k, w[i]);
#pragma unroll
                    for (int j = 0; j < kTokPerBlock; ++j) {
                        const uint32_t tt = min(t0 + j, n_tokens - 1);
                        const float* xt = x + (size_t)tt * K + k;
                        xa[i][j] = *reinterpret_cast<const float4*>(xt);
                        xb[i][j] = *reinterpret_cast<const float4*>(xt + 4);
                    }
                }
            }
#pragma unroll
            for (int i = 0; i < kMaxUnits; ++i) {
                if (u0 + 32 * i < units_q) {
#pragma unroll
                    for (int q = 0; q < 8; ++q) nrm += (ACC)(w[i][q] * w[i][q]);
#pragma unroll
                    for (int j = 0; j < kTokPerBlock; ++j) {
                        ACC s = acc[j];
                        s += (ACC)w[i][0] * (ACC)xa[i][j].x; s += (ACC)w[i][1] * (ACC)xa[i][j].y;
                        s += (ACC)w[i][2] * (ACC)xa[i][j].z; s += (ACC)w[i][3] * (ACC)xa[i][j].w;
                        s += (ACC)w[i][4] * (ACC)xb[i][j].x; s += (ACC)w[i][5] * (ACC)xb[i][j].y;
                        s += (ACC)w[i][6] * (ACC)xb[i][j].z; s += (ACC)w[i][7] * (ACC)xb[i][j].w;
                        acc[j] = s;
                    }
                }
            }
        }
    }
#pragma unroll
    for (int j = 0; j < kTokPerBlock; ++j) {
        const ACC v = warp_sum(acc[j]);
        if (lane == 0) s_part[warp][j] = v;
    }
    nrm = warp_sum(nrm);
    if (lane == 0) s_part[warp][kTokPerBlock] = nrm;
    __syncthreads();
    if (quarter == 0 && e < n_expert && lane <= kTokPerBlock) {
        const ACC v = ((s_part[warp][lane] + s_part[warp + 1][lane]) + s_part[warp + 2][lane]) + s_part[warp + 3][lane];
        if (lane < kTokPerBlock) {
            if (t0 + lane < n_tokens) logits[(size_t)(t0 + lane) * n_expert + e] = v;
        } else if (row_norm2 != nullptr && blockIdx.y == 0) {
            row_norm2[e] = (float)v;
        }
    }
}

cudaError_t launch_logits(const Launch& L, const qkm_dims& d, uint32_t router_type, const void* router,
                          const float* x, float* logits, float* row_norm2, uint32_t n_tokens) {
    if (n_tokens == 0) return cudaSuccess;
    const dim3 grid((d.n_expert + 1) / 2, (n_tokens + kTokPerBlock - 1) / kTokPerBlock);
    const uint8_t* r = (const uint8_t*)router;
    if (router_type == QKM_TYPE_F32)
        logits_kernel<QKM_TYPE_F32, float><<<grid, 256, 0, L.stream>>>(r, x, logits, row_norm2, d.n_expert, d.n_embd, n_tokens);
    else if (router_type == QKM_TYPE_F16)
        logits_kernel<QKM_TYPE_F16, float><<<grid, 256, 0, L.stream>>>(r, x, logits, row_norm2, d.n_expert, d.n_embd, n_tokens);
    else
        return cudaErrorInvalidValue;
    L.count();
    return cudaGetLastError();
}

static cudaError_t launch_logits64(const Launch& L, const qkm_dims& d, uint32_t router_type, const void* router,
                                   const float* x, double* logits, uint32_t n_tokens) {
    const dim3 grid((d.n_expert + 1) / 2, (n_tokens + kTokPerBlock - 1) / kTokPerBlock);
    const uint8_t* r = (const uint8_t*)router;
    cudaError_t e;
    if (router_type == QKM_TYPE_F32)
        e = launch_kernel(L, logits_kernel<QKM_TYPE_F32, double>, grid, dim3(256), 0, r, x, logits, (float*)nullptr, d.n_expert, d.n_embd, n_tokens);
    else
        e = launch_kernel(L, logits_kernel<QKM_TYPE_F16, double>, grid, dim3(256), 0, r, x, logits, (float*)nullptr, d.n_expert, d.n_embd, n_tokens);
    L.count();
    return e != cudaSuccess ? e : cudaGetLastError();
}

// ---- logits for many tokens: 64 x 64 output tiles, f32 FMA -------------------------------------
// logits[t][e] = sum_k x[t][k] * w[e][k], k ascending in one chain per output (the refined
// selection is told the chain length).  Operands are staged through shared memory 16
// columns at a time; each thread owns a 4 x 4 block of outputs.
template <int TYPE>
__global__ void __launch_bounds__(256)
logits_gemm_kernel(const uint8_t* __restrict__ router, const float* __restrict__ x, float* __restrict__ logits,
                   uint32_t n_expert, uint32_t K, uint32_t n_tokens) {
    __shared__ __align__(16) float s_xt[16][64 + 4];   // [k][token]
    __shared__ __align__(16) float s_wt[16][64 + 4];   // [k][expert]
    const uint32_t tid = threadIdx.x, tx = tid & 15u, ty = tid >> 4;
    const uint32_t e0 = blockIdx.x * 64, t0 = blockIdx.y * 64;
    const size_t rb = row_bytes(TYPE, K);
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
    // loader role: thread -> (row = tid / 4, 4 columns at (tid % 4) * 4) of both operand tiles
    const uint32_t lr = tid >> 2, lc = (tid & 3u) * 4;
    auto fetch = [&](uint32_t k0, float4& xv, float4& wv) {
        xv = make_float4(0.f, 0.f, 0.f, 0.f); wv = xv;
        if (t0 + lr < n_tokens) xv = *reinterpret_cast<const float4*>(x + (size_t)(t0 + lr) * K + k0 + lc);
        if (e0 + lr < n_expert) {
            const uint8_t* row = router + (size_t)(e0 + lr) * rb;
            if (TYPE == QKM_TYPE_F32) {
                wv = *reinterpret_cast<const float4*>(row + (size_t)(k0 + lc) * 4);
            } else {
                const uint2 hv = *reinterpret_cast<const uint2*>(row + (size_t)(k0 + lc) * 2);
                wv = make_float4(f16_bits_to_f32(hv.x & 0xFFFFu), f16_bits_to_f32(hv.x >> 16),
                                 f16_bits_to_f32(hv.y & 0xFFFFu), f16_bits_to_f32(hv.y >> 16));
            }
        }
    };
    float4 xv, wv;
    fetch(0, xv, wv);
    for (uint32_t k0 = 0; k0 < K; k0 += 16) {
        __syncthreads();
        s_xt[lc + 0][lr] = xv.x; s_xt[lc + 1][lr] = xv.y; s_xt[lc + 2][lr] = xv.z; s_xt[lc + 3][lr] = xv.w;
        s_wt[lc + 0][lr] = wv.x; s_wt[lc + 1][lr] = wv.y; s_wt[lc + 2][lr] = wv.z; s_wt[lc + 3][lr] = wv.w;
        __syncthreads();
        if (k0 + 16 < K) fetch(k0 + 16, xv, wv);   // next tile's loads fly during this tile's math
#pragma unroll
        for (int k = 0; k < 16; ++k) {
            const float4 a = *reinterpret_cast<const float4*>(&s_xt[k][ty * 4]);
            const float4 b = *reinterpret_cast<const float4*>(&s_wt[k][tx * 4]);
            const float av[4] = {a.x, a.y, a.z, a.w}, bv[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] += av[i] * bv[j];
        }
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const uint32_t t = t0 + ty * 4 + i;
        if (t < n_tokens) {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const uint32_t e = e0 + tx * 4 + j;
                if (e < n_expert) logits[(size_t)t * n_expert + e] = acc[i][j];
            }
        }
    }
}

// |router row|^2, one warp per row
template <int TYPE>
__global__ void __launch_bounds__(256)
row_norm2_kernel(const uint8_t* __restrict__ router, float* __restrict__ row_norm2, uint32_t n_expert, uint32_t K) {
    const uint32_t e = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31u;
    if (e >= n_expert) return;
    const uint8_t* row = router + (size_t)e * row_bytes(TYPE, K);
    float nrm = 0.f;
    for (uint32_t u = lane; u < K / 8; u += 32) {
        float w[8];
        dequant8<TYPE>(row, u * 8, w);
#pragma unroll
        for (int i = 0; i < 8; ++i) nrm += w[i] * w[i];
    }
    nrm = warp_sum(nrm);
    if (lane == 0) row_norm2[e] = nrm;
}

// ---- helpers for block-wide (value, lowest id) argmax --------------------------------------
// Key orders by value first; among equal values the smaller id gives the larger key.
__device__ __forceinline__ unsigned long long rank_key(float v, uint32_t id) {
    v = v + 0.0f;  // -0 -> +0 so the two zeros tie
    uint32_t b = __float_as_uint(v);
    b = (b & 0x80000000u) ? ~b : (b | 0x80000000u);
    return ((unsigned long long)b << 32) | (unsigned long long)(0xFFFFFFFFu - id);
}
__device__ __forceinline__ float sane(float v) { return (isnan(v) || isinf(v)) ? kFloor : v; }

__device__ __forceinline__ unsigned long long warp_max_u64(unsigned long long k) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const unsigned long long other = __shfl_xor_sync(0xFFFFFFFFu, k, o);
        k = other > k ? other : k;
    }
    return k;
}

// Block-wide argmax over the (up to) 2 logits every one of 256 threads holds.
// Returns the winning key to every thread.
__device__ __forceinline__ unsigned long long block_argmax(float v0, uint32_t id0, float v1, uint32_t id1,
                                                           unsigned long long* s_warp /* [8] */) {
    const unsigned long long k0 = rank_key(v0, id0), k1 = rank_key(v1, id1);
    unsigned long long k = warp_max_u64(k0 > k1 ? k0 : k1);
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
    __syncthreads();  // s_warp reuse across rounds
    if (lane == 0) s_warp[warp] = k;
    __syncthreads();
    k = s_warp[0];
#pragma unroll
    for (int w = 1; w < 8; ++w) k = s_warp[w] > k ? s_warp[w] : k;
    return k;
}

// f64 dot of gate_inp_shexp with x over 256 threads; result valid in thread 0.
__device__ __forceinline__ double block_dot_f64(const float* __restrict__ a, const float* __restrict__ b,
                                                uint32_t K, double* s_red /* [8] */) {
    double acc = 0.0;
    for (uint32_t k = threadIdx.x; k < K; k += 256) acc += (double)a[k] * (double)b[k];
    acc = warp_sum(acc);
    __syncthreads();
    if ((threadIdx.x & 31u) == 0) s_red[threadIdx.x >> 5] = acc;
    __syncthreads();
    double tot = 0.0;
    if (threadIdx.x == 0)
        for (int w = 0; w < 8; ++w) tot += s_red[w];
    return tot;
}

// ---- selection from given f32 logits: one block per token --------------------------------
__global__ void __launch_bounds__(256)
select_kernel(const float* __restrict__ logits, const float* __restrict__ gis, const float* __restrict__ x,
              qkm_sel* __restrict__ sel, qkm_dims d) {
    __shared__ unsigned long long s_warp[8];
    __shared__ double s_red[8];
    __shared__ float s_pick[16];
    const uint32_t t = blockIdx.x, tid = threadIdx.x;
    const float* lt = logits + (size_t)t * d.n_expert;
    const uint32_t id0 = tid, id1 = tid + 256u;
    float v0 = id0 < d.n_expert ? sane(lt[id0]) : kFloor;
    float v1 = id1 < d.n_expert ? sane(lt[id1]) : kFloor;
    // padding lanes must never beat a real expert on a tie: give them the largest ids
    const uint32_t pid0 = id0 < d.n_expert ? id0 : 0xFFFFFFFEu;
    const uint32_t pid1 = id1 < d.n_expert ? id1 : 0xFFFFFFFEu;

    const double sg = block_dot_f64(gis, x + (size_t)t * d.n_embd, d.n_embd, s_red);
    if (tid == 0) {
        sel[t].w_shared = (float)(1.0 / (1.0 + exp(-sg)));
        sel[t].route_done = 0;
#pragma unroll
        for (int i = 0; i < 6; ++i) sel[t].pad[i] = 0.f;
    }
    for (uint32_t i = 0; i < 16; ++i) {
        if (i >= d.n_used) {
            if (tid == 0) { sel[t].ids[i] = 0; sel[t].w[i] = 0.f; }
            continue;
        }
        const unsigned long long k = block_argmax(v0, pid0, v1, pid1, s_warp);
        uint32_t id = 0xFFFFFFFFu - (uint32_t)(k & 0xFFFFFFFFull);
        if (id >= d.n_expert) id = d.n_expert - 1;  // clamp (moe_select.comp:61-63)
        if (tid == 0) {
            uint32_t b = (uint32_t)(k >> 32);
            b = (b & 0x80000000u) ? (b & 0x7FFFFFFFu) : ~b;
            sel[t].ids[i] = id;
            s_pick[i] = __uint_as_float(b);
        }
        if (id == id0) v0 = kFloor;
        if (id == id1) v1 = kFloor;
    }
    __syncthreads();
    if (tid == 0) {
        double w[16], sum = 0.0;
        for (uint32_t i = 0; i < d.n_used; ++i) { w[i] = exp((double)s_pick[i] - (double)s_pick[0]); sum += w[i]; }
        for (uint32_t i = 0; i < d.n_used; ++i) sel[t].w[i] = (float)(w[i] / sum);
    }
}

cudaError_t launch_select(const Launch& L, const qkm_dims& d, const float* logits, const float* gis,
                          const float* x, qkm_sel* sel, uint32_t n_tokens) {
    if (n_tokens == 0) return cudaSuccess;
    select_kernel<<<n_tokens, 256, 0, L.stream>>>(logits, gis, x, sel, d);
    L.count();
    return cudaGetLastError();
}

// ---- x rows as int8 digit planes (what the streaming expert kernels read) ---------------------
// One block per row: x * 2^p rounded to 28 bits, split into four balanced base-128 digits,
// layout [k-block][digit][256]; xscale = 2^-p.  A row with a non-finite value gets zero digits
// and a NaN scale.  (The selection kernel can write the same planes; doing it here lets the
// shared expert start before the routing is known.)
// With gis != NULL it also evaluates the shared expert's gate, w_shared = sigmoid(gis . x) in
// f64, into sel[t].w_shared - the selection kernel is then told to leave that field alone.
__global__ void __launch_bounds__(256)
xplanes_kernel(const float* __restrict__ x, uint32_t n_embd, int8_t* __restrict__ xplanes, float* __restrict__ xscale,
               const float* __restrict__ gis, qkm_sel* __restrict__ sel) {
    __shared__ float s_xm[8];
    __shared__ double s_sg[8];
    const uint32_t t = blockIdx.x, tid = threadIdx.x, lane = tid & 31u, warp = tid >> 5;
    const float* xt = x + (size_t)t * n_embd;
    float v[16];   // n_embd <= 4096
    float xm = 0.f;
    double dsg = 0.0;
    bool bad = false;
#pragma unroll
    for (int i = 0; i < 16; ++i) {
        const uint32_t k = tid + 256 * i;
        v[i] = k < n_embd ? xt[k] : 0.f;
        xm = fmaxf(xm, fabsf(v[i]));
        bad |= !(fabsf(v[i]) <= 3.0e38f);
        if (gis != nullptr && k < n_embd) dsg += (double)gis[k] * (double)v[i];
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) xm = fmaxf(xm, __shfl_xor_sync(0xFFFFFFFFu, xm, o));
    if (gis != nullptr) dsg = warp_sum(dsg);
    const int any_bad = __syncthreads_or(bad ? 1 : 0);
    if (lane == 0) { s_xm[warp] = xm; s_sg[warp] = dsg; }
    __syncthreads();
    if (gis != nullptr && tid == 0) {
        double sg = 0.0;
#pragma unroll
        for (int w = 0; w < 8; ++w) sg += s_sg[w];
        sel[t].w_shared = (float)(1.0 / (1.0 + exp(-sg)));
    }
    float xmax = 0.f;
#pragma unroll
    for (int w = 0; w < 8; ++w) xmax = fmaxf(xmax, s_xm[w]);
    const int p = digit_exponent(xmax);
    const float up = ldexpf(1.0f, p);
    int8_t* pl = xplanes + (size_t)t * 4 * n_embd;
#pragma unroll
    for (int i = 0; i < 16; ++i) {
        const uint32_t k = tid + 256 * i;
        if (k < n_embd) {
            const uint32_t dgt = any_bad ? 0u : digits4(__float2int_rn(v[i] * up));
            int8_t* q = pl + (size_t)(k >> 8) * 1024 + (k & 255u);
            q[0] = (int8_t)(dgt & 255u);
            q[256] = (int8_t)((dgt >> 8) & 255u);
            q[512] = (int8_t)((dgt >> 16) & 255u);
            q[768] = (int8_t)(dgt >> 24);
        }
    }
    if (tid == 0) xscale[t] = any_bad ? __int_as_float(0x7FC00000) : ldexpf(1.0f, -p);
}

cudaError_t launch_xplanes(const Launch& L, const float* x, uint32_t n_tokens, uint32_t n_embd, int8_t* xplanes, float* xscale,
                           const float* gis, qkm_sel* sel) {
    if (n_tokens == 0) return cudaSuccess;
    if (n_embd > 4096 || (gis != nullptr && sel == nullptr)) return cudaErrorInvalidValue;
    xplanes_kernel<<<n_tokens, 256, 0, L.stream>>>(x, n_embd, xplanes, xscale, gis, sel);
    L.count();
    return cudaGetLastError();
}

// ---- grouping of a decode-sized batch inside the selection kernel ------------------------------
// The block that finishes its token last (a ticket counter tells it) groups the pairs of all
// tokens and cuts the work list of the streaming kernels, which saves a launch on the layer's
// critical path.  At most 1024 pairs; same result as group_pairs_kernel.
struct GroupTail {
    uint32_t* counter;       // NULL: no grouping here
    uint32_t* offsets;
    uint32_t* pairs;
    StreamItem* items_gu;
    StreamItem* items_dn;
    uint32_t* n_items;       // [0] gate/up items, [1] down items
    uint32_t chunks_gu, chunks_dn, tok_per_item, n_tokens, expert_first, expert_count;
    uint32_t shared_gate_elsewhere;   // sel[t].w_shared is written by another kernel: neither x nor the gate is touched here
};
static constexpr uint32_t kTailMaxPairs = 1024;

__device__ void group_small_block(const qkm_sel* __restrict__ sel, uint32_t n_expert, uint32_t n_used, const GroupTail& g) {
    __shared__ uint16_t s_e[kTailMaxPairs];
    __shared__ uint32_t s_cnt[512], s_off[512];
    __shared__ unsigned long long s_wsum[8];
    const uint32_t tid = threadIdx.x, lane = tid & 31u, wrp = tid >> 5;
    const uint32_t np = g.n_tokens * n_used;
    for (uint32_t e = tid; e < 512; e += 256) s_cnt[e] = 0;
    for (uint32_t p = tid; p < np; p += 256) {
        const uint32_t t = p / n_used, s = p - t * n_used;
        const uint32_t e = min(__ldcg(&sel[t].ids[s]), n_expert - 1) - g.expert_first;
        s_e[p] = (uint16_t)(e < g.expert_count ? e : 0xFFFFu);
    }
    __syncthreads();
    for (uint32_t p = tid; p < np; p += 256)
        if (s_e[p] != 0xFFFFu) atomicAdd(&s_cnt[s_e[p]], 1u);
    __syncthreads();
    // exclusive scan over the experts, two per thread; pair counts low, token groups high
    const uint32_t c0 = s_cnt[2 * tid], c1 = s_cnt[2 * tid + 1];
    const uint32_t g0n = (c0 + g.tok_per_item - 1) / g.tok_per_item, g1n = (c1 + g.tok_per_item - 1) / g.tok_per_item;
    unsigned long long v = (unsigned long long)(c0 + c1) | ((unsigned long long)(g0n + g1n) << 32);
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const unsigned long long up = __shfl_up_sync(0xFFFFFFFFu, v, o);
        if (lane >= (uint32_t)o) v += up;
    }
    if (lane == 31) s_wsum[wrp] = v;
    __syncthreads();
    unsigned long long base = 0, total = 0;
    for (uint32_t w = 0; w < 8; ++w) { if (w < wrp) base += s_wsum[w]; total += s_wsum[w]; }
    const unsigned long long excl = base + v - ((unsigned long long)(c0 + c1) | ((unsigned long long)(g0n + g1n) << 32));
    const uint32_t off0 = (uint32_t)(excl & 0xFFFFFFFFull), grp0 = (uint32_t)(excl >> 32);
    s_off[2 * tid] = off0;
    s_off[2 * tid + 1] = off0 + c0;
    if (2 * tid < g.expert_count) g.offsets[2 * tid] = off0;
    if (2 * tid + 1 < g.expert_count) g.offsets[2 * tid + 1] = off0 + c0;
    if (tid == 0) {
        g.offsets[g.expert_count] = (uint32_t)(total & 0xFFFFFFFFull);
        g.n_items[0] = (uint32_t)(total >> 32) * g.chunks_gu;
        g.n_items[1] = (uint32_t)(total >> 32) * g.chunks_dn;
    }
#pragma unroll
    for (int k = 0; k < 2; ++k) {
        const uint32_t e = 2 * tid + k, cnt = k ? c1 : c0, off = k ? off0 + c0 : off0, gfirst = k ? grp0 + g0n : grp0;
        const uint32_t groups = k ? g1n : g0n;
        for (uint32_t gi = 0; gi < groups; ++gi) {
            StreamItem it;
            it.expert = (uint16_t)e;
            it.ntok = (uint8_t)min(g.tok_per_item, cnt - gi * g.tok_per_item);
            it.pair_off = off + gi * g.tok_per_item;
            for (uint32_t c = 0; c < g.chunks_gu; ++c) { it.chunk = (uint8_t)c; g.items_gu[(size_t)(gfirst + gi) * g.chunks_gu + c] = it; }
            for (uint32_t c = 0; c < g.chunks_dn; ++c) { it.chunk = (uint8_t)c; g.items_dn[(size_t)(gfirst + gi) * g.chunks_dn + c] = it; }
        }
    }
    __syncthreads();
    // place: rank among the earlier pairs of the same expert keeps (token, slot) order
    for (uint32_t p = tid; p < np; p += 256) {
        const uint32_t e = s_e[p];
        if (e == 0xFFFFu) continue;
        uint32_t rank = 0;
        for (uint32_t q = 0; q < p; ++q) rank += s_e[q] == e ? 1u : 0u;
        const uint32_t t = p / n_used, s = p - t * n_used;
        g.pairs[s_off[e] + rank] = (t << 4) | s;
    }
}

// ---- refined selection: f32 ranking, f64 re-evaluation of the boundary ---------------------
// One block per token.  Ranking is done by counting: every thread counts how many experts
// precede its own in the order (value descending, id ascending), which needs no rounds of
// block-wide argmax and no serial insertion.
static constexpr int kMaxCand = 128;

// the logit of a rank_key (keys of real experts are never 0, which pads)
__device__ __forceinline__ float rank_key_value(unsigned long long key) {
    const uint32_t b = (uint32_t)(key >> 32);
    return __uint_as_float((b & 0x80000000u) ? (b ^ 0x80000000u) : ~b);
}
// bitonic sort of one key per lane, descending: lane i ends with the i-th largest
__device__ __forceinline__ unsigned long long warp_sort_desc(unsigned long long key, uint32_t lane) {
#pragma unroll
    for (uint32_t k = 2; k <= 32; k <<= 1) {
#pragma unroll
        for (uint32_t j = k >> 1; j > 0; j >>= 1) {
            const unsigned long long other = __shfl_xor_sync(0xFFFFFFFFu, key, j);
            const bool take_max = ((lane & k) == 0) == ((lane & j) == 0);
            key = take_max ? (key > other ? key : other) : (key < other ? key : other);
        }
    }
    return key;
}

// EXACT: `logits_any` holds f64 logits of an f64-accumulating kernel; they are ranked as they
// are (no bound, no candidates).  Otherwise it holds f32 logits and the boundary is re-evaluated.
template <int TYPE, bool EXACT>
__global__ void __launch_bounds__(256)
refine_select_kernel(const uint8_t* __restrict__ router, const void* __restrict__ logits_any,
                     const float* __restrict__ row_norm2, const float* __restrict__ gis,
                     const float* __restrict__ x, qkm_sel* __restrict__ sel, qkm_dims d,
                     int8_t* __restrict__ xplanes, float* __restrict__ xscale, float eps_terms, float eps_abs,
                     GroupTail tail, uint32_t n_parts, size_t part_stride) {
    extern __shared__ float s_x[];  // n_embd floats
    __shared__ __align__(16) double s_val[512];   // f64 logit of every candidate, -inf elsewhere
    __shared__ __align__(16) float s_log[512];
    __shared__ double s_red[8];
    __shared__ float s_f[8], s_rn[8], s_xm[8];
    __shared__ uint32_t s_cand[kMaxCand];
    __shared__ uint32_t s_ncand;
    __shared__ float s_kth;
    __shared__ uint32_t s_best_id[16];
    __shared__ double s_best_val[16];
    const uint32_t t = blockIdx.x, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31u;
    pdl_trigger();
    pdl_wait();   // the logits come from the kernel before
    const float* xt = x + (size_t)t * d.n_embd;
    const uint32_t id0 = tid, id1 = tid + 256u;
    const double ninf = -__longlong_as_double(0x7FF0000000000000ll);
    float l0 = kFloor, l1 = kFloor;
    if (EXACT) {
        const double* lt = reinterpret_cast<const double*>(logits_any) + (size_t)t * d.n_expert;
        double v0 = ninf, v1 = ninf;
        if (id0 < d.n_expert) { v0 = lt[id0]; if (isnan(v0) || isinf(v0)) v0 = (double)kFloor; }
        if (id1 < d.n_expert) { v1 = lt[id1]; if (isnan(v1) || isinf(v1)) v1 = (double)kFloor; }
        s_val[id0] = v0;
        s_val[id1] = v1;
    } else {
        const float* lt = reinterpret_cast<const float*>(logits_any) + (size_t)t * d.n_expert;
        // the logits may arrive as n_parts partial sums over column ranges (split-K GEMM): added in order
        float a0 = 0.f, a1 = 0.f;
        for (uint32_t p = 0; p < n_parts; ++p) {
            if (id0 < d.n_expert) a0 += lt[p * part_stride + id0];
            if (id1 < d.n_expert) a1 += lt[p * part_stride + id1];
        }
        l0 = (id0 < d.n_expert ? sane(a0) : kFloor) + 0.0f;  // + 0: -0 and +0 tie
        l1 = (id1 < d.n_expert ? sane(a1) : kFloor) + 0.0f;
        s_log[id0] = l0;
        s_log[id1] = l1;
        s_val[id0] = ninf;
        s_val[id1] = ninf;
    }

    // One pass over the row: stage it in shared memory and gather everything that needs
    // it - |x|^2 and max|x| (error bound, digit exponent), the shared-gate dot in f64 -
    // together with max |router row|^2, so all global loads of this phase are in flight at once.
    float xs = 0.f, xm = 0.f, rn = 0.f;
    double dsg = 0.0;
    bool bad = false;
    // (skipped when the f64 logits are ranked as they are and the shared gate comes from
    // elsewhere: nothing below needs x then)
    const bool need_x = !EXACT || xplanes != nullptr || !tail.shared_gate_elsewhere;
    float x2 = 0.f, r2 = 0.f, xmax = 0.f;
    double sg = 0.0;
    int any_bad = 0;
    if (need_x) {
    for (uint32_t k = tid; k < d.n_embd; k += 256) {
        const float v = xt[k], gv = gis[k];
        s_x[k] = v;
        xs += v * v;
        xm = fmaxf(xm, fabsf(v));
        bad |= !(fabsf(v) <= 3.0e38f);
        dsg += (double)gv * (double)v;
    }
    if (!EXACT) {
        if (id0 < d.n_expert) rn = row_norm2[id0];
        if (id1 < d.n_expert) rn = fmaxf(rn, row_norm2[id1]);
    }
    xs = warp_sum(xs);
    dsg = warp_sum(dsg);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        rn = fmaxf(rn, __shfl_xor_sync(0xFFFFFFFFu, rn, o));
        xm = fmaxf(xm, __shfl_xor_sync(0xFFFFFFFFu, xm, o));
    }
    any_bad = __syncthreads_or(bad ? 1 : 0);
    if (lane == 0) { s_f[warp] = xs; s_red[warp] = dsg; s_rn[warp] = rn; s_xm[warp] = xm; }
    if (tid == 0) s_ncand = 0;
    __syncthreads();
#pragma unroll
    for (int w = 0; w < 8; ++w) { x2 += s_f[w]; sg += s_red[w]; r2 = fmaxf(r2, s_rn[w]); xmax = fmaxf(xmax, s_xm[w]); }
    } else {
        __syncthreads();   // s_val is complete
    }
    // the streaming expert kernels read x as int8 digit planes ([kb][digit][256] per row)
    if (xplanes != nullptr) {
        const int p = digit_exponent(xmax);
        const float up = ldexpf(1.0f, p);
        int8_t* pl = xplanes + (size_t)t * 4 * d.n_embd;
        for (uint32_t k = tid; k < d.n_embd; k += 256) {
            const uint32_t dgt = any_bad ? 0u : digits4(__float2int_rn(s_x[k] * up));
            int8_t* q = pl + (size_t)(k >> 8) * 1024 + (k & 255u);
            q[0] = (int8_t)(dgt & 255u);
            q[256] = (int8_t)((dgt >> 8) & 255u);
            q[512] = (int8_t)((dgt >> 16) & 255u);
            q[768] = (int8_t)(dgt >> 24);
        }
        if (tid == 0) xscale[t] = any_bad ? __int_as_float(0x7FC00000) : ldexpf(1.0f, -p);
    }

    bool listed_all = true;     // every expert holds an f64 value (s_val)
    uint32_t n_listed = 0;      // else: the candidates s_cand[0 .. n_listed)
    if (!EXACT) {
    // k-th largest f32 logit in the order (value descending, id ascending).  A logit and its id make one
    // 64-bit key (larger = earlier); every warp sorts its 32 keys with a bitonic network of shuffles and
    // only its first n_used survive to the next round, until one warp holds the rest: 2.5 k instructions per
    // token where ranking the survivors by counting took 12 k.
    {
        __shared__ unsigned long long s_keys[256];
        const bool two = d.n_expert > 256;       // the second expert of a thread exists only then
        const uint32_t sets = two ? 2u : 1u;
        const unsigned long long k0 = warp_sort_desc(id0 < d.n_expert ? rank_key(l0, id0) : 0ull, lane);
        if (lane < d.n_used) s_keys[warp * d.n_used + lane] = k0;
        if (two) {
            const unsigned long long k1 = warp_sort_desc(id1 < d.n_expert ? rank_key(l1, id1) : 0ull, lane);
            if (lane < d.n_used) s_keys[(8 + warp) * d.n_used + lane] = k1;
        }
        __syncthreads();
        uint32_t count = sets * 8u * d.n_used;    // <= 240
        while (true) {                            // block-uniform
            unsigned long long key = tid < count ? s_keys[tid] : 0ull;
            const bool active = warp * 32u < count;
            if (active) key = warp_sort_desc(key, lane);
            if (count <= 32u) {
                if (tid == d.n_used - 1) s_kth = rank_key_value(key);
                break;
            }
            __syncthreads();                      // every entry of this round has been read
            if (active && lane < d.n_used) s_keys[warp * d.n_used + lane] = key;
            count = ((count + 31u) / 32u) * d.n_used;
            __syncthreads();
        }
    }
    __syncthreads();
    const float kth = s_kth;
    // Error bound of one f32 logit whose longest chain of additions has eps_terms links:
    // |err| <= eps_terms * 2^-24 * sum|w_k x_k| <= that * |w| * |x|.
    // Doubled for safety, and doubled again because two logits are compared.
    const float eps = 5.9604645e-8f * (eps_terms * sqrtf(r2) + eps_abs) * sqrtf(x2);
    const float thresh = kth - 4.0f * eps;
    // candidates: every expert at or above the threshold
    // (written as !(l < thresh) so a NaN threshold - NaN in x - admits every expert)
    const bool k0 = id0 < d.n_expert && !(l0 < thresh), k1 = id1 < d.n_expert && !(l1 < thresh);
    if (k0) { const uint32_t p = atomicAdd(&s_ncand, 1u); if (p < kMaxCand) s_cand[p] = id0; }
    if (k1) { const uint32_t p = atomicAdd(&s_ncand, 1u); if (p < kMaxCand) s_cand[p] = id1; }
    __syncthreads();
    const uint32_t ncand = s_ncand;
    // too many near-ties (or non-finite input: everything at the floor): evaluate all experts
    const bool all = ncand > kMaxCand || ncand < d.n_used;
    const uint32_t total = all ? d.n_expert : ncand;
    listed_all = all;
    n_listed = ncand;

    // f64 re-evaluation, one warp per candidate, four independent partial sums per lane
    const size_t rb = row_bytes(TYPE, d.n_embd);
    for (uint32_t c = warp; c < total; c += 8) {
        const uint32_t e = all ? c : s_cand[c];
        const uint8_t* row = router + (size_t)e * rb;
        double a0 = 0.0, a1 = 0.0, a2 = 0.0, a3 = 0.0;
#pragma unroll 4
        for (uint32_t u = lane; u < d.n_embd / 8; u += 32) {
            float w[8];
            dequant8<TYPE>(row, u * 8, w);
            const float* xv = s_x + u * 8;
            a0 += (double)w[0] * (double)xv[0]; a1 += (double)w[1] * (double)xv[1];
            a2 += (double)w[2] * (double)xv[2]; a3 += (double)w[3] * (double)xv[3];
            a0 += (double)w[4] * (double)xv[4]; a1 += (double)w[5] * (double)xv[5];
            a2 += (double)w[6] * (double)xv[6]; a3 += (double)w[7] * (double)xv[7];
        }
        const double acc = warp_sum((a0 + a1) + (a2 + a3));
        if (lane == 0) s_val[e] = (isnan(acc) || isinf(acc)) ? (double)kFloor : acc;
    }
    }  // !EXACT
    __syncthreads();
    // final order among the candidates: (f64 value descending, id ascending)
    {
        const double v0 = s_val[id0], v1 = s_val[id1];
        const bool m0 = v0 > ninf, m1 = v1 > ninf;
        uint32_t c0 = d.n_used, c1 = d.n_used;   // "not among the first n_used" until shown otherwise
        if (EXACT || listed_all) {   // block-uniform: every thread takes part in the shuffles and the barrier
            // Two levels, as for the f32 k-th search: rank inside the warp's 32 experts by
            // shuffles, then only each warp's first n_used are ranked against each other.
            __shared__ double s_dv[2][8][16];
            __shared__ uint32_t s_di[2][8][16];
            const bool two = d.n_expert > 256;
            uint32_t q0 = 0, q1 = 0;
#pragma unroll 4
            for (uint32_t sft = 1; sft < 32; ++sft) {
                const uint32_t src = (lane + sft) & 31u;
                const double o0 = __shfl_sync(0xFFFFFFFFu, v0, src);
                q0 += (o0 > v0 || (o0 == v0 && src < lane)) ? 1u : 0u;
                if (two) {
                    const double o1 = __shfl_sync(0xFFFFFFFFu, v1, src);
                    q1 += (o1 > v1 || (o1 == v1 && src < lane)) ? 1u : 0u;
                }
            }
            if (q0 < d.n_used) { s_dv[0][warp][q0] = v0; s_di[0][warp][q0] = id0; }
            if (two && q1 < d.n_used) { s_dv[1][warp][q1] = v1; s_di[1][warp][q1] = id1; }
            __syncthreads();
            if (q0 < d.n_used || (two && q1 < d.n_used)) {
                uint32_t k0 = 0, k1 = 0;
                for (uint32_t st = 0; st < (two ? 2u : 1u); ++st)
                    for (uint32_t w = 0; w < 8; ++w)
                        for (uint32_t q = 0; q < d.n_used; ++q) {
                            const double vj = s_dv[st][w][q];
                            const uint32_t j = s_di[st][w][q];
                            k0 += (vj > v0 || (vj == v0 && j < id0)) ? 1u : 0u;
                            k1 += (vj > v1 || (vj == v1 && j < id1)) ? 1u : 0u;
                        }
                if (q0 < d.n_used) c0 = k0;
                if (two && q1 < d.n_used) c1 = k1;
            }
        } else if (m0 || m1) {   // only the listed candidates hold values
            uint32_t k0 = 0, k1 = 0;
            for (uint32_t q = 0; q < n_listed; ++q) {
                const uint32_t j = s_cand[q];
                const double vj = s_val[j];
                k0 += (vj > v0 || (vj == v0 && j < id0)) ? 1u : 0u;
                k1 += (vj > v1 || (vj == v1 && j < id1)) ? 1u : 0u;
            }
            c0 = k0; c1 = k1;
        }
        if (m0 && c0 < d.n_used) { s_best_id[c0] = id0; s_best_val[c0] = v0; }
        if (m1 && c1 < d.n_used) { s_best_id[c1] = id1; s_best_val[c1] = v1; }
    }
    __syncthreads();
    if (warp == 0) {
        // lane i < n_used: softmax term of pick i; lane 16: the shared gate
        double wv = 0.0;
        if (lane < d.n_used) wv = exp(s_best_val[lane] - s_best_val[0]);
        double sum = wv;
#pragma unroll
        for (int o = 8; o > 0; o >>= 1) sum += __shfl_xor_sync(0xFFFFFFFFu, sum, o);  // lanes 0..15
        if (lane < 16) {
            sel[t].ids[lane] = lane < d.n_used ? min(s_best_id[lane], d.n_expert - 1) : 0u;
            sel[t].w[lane] = lane < d.n_used ? (float)(wv / sum) : 0.f;
        } else if (lane == 16) {
            if (need_x) sel[t].w_shared = (float)(1.0 / (1.0 + exp(-sg)));
            sel[t].route_done = 0;
        } else if (lane < 23) {
            sel[t].pad[lane - 17] = 0.f;
        }
    }
    if (tail.counter != nullptr) {
        __shared__ uint32_t s_last;
        __threadfence();
        __syncthreads();
        if (tid == 0) s_last = atomicAdd(tail.counter, 1u) == gridDim.x - 1 ? 1u : 0u;
        __syncthreads();
        if (s_last) {
            if (tid == 0) *tail.counter = 0;   // ready for the next launch
            __threadfence();
            group_small_block(sel, d.n_expert, d.n_used, tail);
        }
    }
}

static constexpr uint32_t kExactMaxTokens = 64;   // decode-sized batches rank f64 logits directly

bool route_select_plans(const qkm_dims& d, uint32_t n_tokens, size_t scratch_bytes) {
    return n_tokens > 0 && n_tokens <= kExactMaxTokens && n_tokens * d.n_used <= kTailMaxPairs &&
           (size_t)n_tokens * d.n_expert * sizeof(double) <= scratch_bytes;
}

size_t route_scratch_bytes(uint32_t n_tokens, uint32_t n_expert) {
    // f32 logits (up to 8 partial sums over column ranges when the batch is small enough to split) + row norms
    const size_t parts = n_tokens >= 128 && n_tokens <= 4096 ? 8 : 1;
    const size_t f32_path = ((size_t)n_tokens * n_expert * parts + n_expert) * sizeof(float);
    const size_t f64_path = (size_t)(n_tokens < kExactMaxTokens ? n_tokens : kExactMaxTokens) * n_expert * sizeof(double);
    return f32_path > f64_path ? f32_path : f64_path;
}

cudaError_t launch_route_select(const Launch& L, const qkm_dims& d, uint32_t router_type,
                                const void* router, const float* gis, const float* x, qkm_sel* sel,
                                uint32_t n_tokens, void* scratch, size_t scratch_bytes, int8_t* xplanes, float* xscale,
                                const void* x_f16, const float* x_f16_inv, uint32_t* status, const RoutePlan* plan) {
    if (n_tokens == 0) return cudaSuccess;
    GroupTail tail{};
    if (plan && plan->counter && n_tokens <= kExactMaxTokens && n_tokens * d.n_used <= kTailMaxPairs) {
        uint32_t ef = plan->expert_first, ec = plan->expert_count;
        if (ec == 0) { ef = 0; ec = d.n_expert; }
        tail = GroupTail{plan->counter, plan->offsets, plan->pairs, plan->items_gu, plan->items_dn, plan->n_items,
                         plan->chunks_gu, plan->chunks_dn, plan->tok_per_item, n_tokens, ef, ec, plan->shared_gate_elsewhere};
    }
    if (router_type != QKM_TYPE_F32 && router_type != QKM_TYPE_F16) return cudaErrorInvalidValue;
    if (n_tokens <= kExactMaxTokens && (size_t)n_tokens * d.n_expert * sizeof(double) <= scratch_bytes) {
        // small batch: f64 logits, ranked as they are
        double* l64 = (double*)scratch;
        cudaError_t e = launch_logits64(L, d, router_type, router, x, l64, n_tokens);
        if (e != cudaSuccess) return e;
        if (router_type == QKM_TYPE_F32)
            e = launch_kernel(L, refine_select_kernel<QKM_TYPE_F32, true>, dim3(n_tokens), dim3(256), (size_t)d.n_embd * 4, (const uint8_t*)router, (const void*)l64, (const float*)nullptr, gis, x, sel, d, xplanes, xscale, 0.f, 0.f, tail, 1u, (size_t)0);
        else
            e = launch_kernel(L, refine_select_kernel<QKM_TYPE_F16, true>, dim3(n_tokens), dim3(256), (size_t)d.n_embd * 4, (const uint8_t*)router, (const void*)l64, (const float*)nullptr, gis, x, sel, d, xplanes, xscale, 0.f, 0.f, tail, 1u, (size_t)0);
        L.count();
        return e != cudaSuccess ? e : cudaGetLastError();
    }
    if (((size_t)n_tokens * d.n_expert + d.n_expert) * sizeof(float) > scratch_bytes) return cudaErrorInvalidValue;
    float* logits = (float*)scratch;
    float* norm2 = logits + (size_t)n_tokens * d.n_expert;
    const uint8_t* r = (const uint8_t*)router;
    float eps_terms, eps_abs = 0.f;
    uint32_t n_parts = 1;
    if (x_f16 && x_f16_inv && status && n_tokens >= 128 && d.n_expert % 128 == 0 && d.n_embd <= 4096) {
        // tensor cores, f16 operands: |error| <= 2^-9 |w| |x|, plus the flush of tiny router values.
        // Few output tiles: the columns are split over more blocks, partial logits side by side
        // (summed by the selection kernel).
        const uint32_t tiles = ((n_tokens + 127) / 128) * (d.n_expert / 128);
        uint32_t splits = 1;
        while (splits < 8 && tiles * splits * 2 <= 148u && (d.n_embd / 64) % (splits * 2) == 0 &&
               ((size_t)n_tokens * d.n_expert * (splits * 2) + d.n_expert) * sizeof(float) <= scratch_bytes) splits *= 2;
        norm2 = logits + (size_t)n_tokens * d.n_expert * splits;
        if (router_type == QKM_TYPE_F32)
            row_norm2_kernel<QKM_TYPE_F32><<<(d.n_expert + 7) / 8, 256, 0, L.stream>>>(r, norm2, d.n_expert, d.n_embd);
        else
            row_norm2_kernel<QKM_TYPE_F16><<<(d.n_expert + 7) / 8, 256, 0, L.stream>>>(r, norm2, d.n_expert, d.n_embd);
        L.count();
        cudaError_t e = launch_logits_mma(L, d, router_type, router, x_f16, x_f16_inv, logits, n_tokens, status, splits);
        if (e != cudaSuccess) return e;
        n_parts = splits;
        eps_terms = 32768.f + (float)splits;       // 2^-9 / 2^-24, plus the additions of the partial sums
        eps_abs = 2.f * sqrtf((float)d.n_embd);    // 2^-25 per router element that f16 flushes
    } else if (n_tokens >= 1024) {   // many tokens: tiled GEMM, one chain of n_embd additions per logit
        const dim3 grid((d.n_expert + 63) / 64, (n_tokens + 63) / 64);
        if (router_type == QKM_TYPE_F32) {
            row_norm2_kernel<QKM_TYPE_F32><<<(d.n_expert + 7) / 8, 256, 0, L.stream>>>(r, norm2, d.n_expert, d.n_embd);
            logits_gemm_kernel<QKM_TYPE_F32><<<grid, 256, 0, L.stream>>>(r, x, logits, d.n_expert, d.n_embd, n_tokens);
        } else {
            row_norm2_kernel<QKM_TYPE_F16><<<(d.n_expert + 7) / 8, 256, 0, L.stream>>>(r, norm2, d.n_expert, d.n_embd);
            logits_gemm_kernel<QKM_TYPE_F16><<<grid, 256, 0, L.stream>>>(r, x, logits, d.n_expert, d.n_embd, n_tokens);
        }
        L.count(2);
        cudaError_t e = cudaGetLastError();
        if (e != cudaSuccess) return e;
        eps_terms = (float)d.n_embd + 8.f;
    } else {
        cudaError_t e = launch_logits(L, d, router_type, router, x, logits, norm2, n_tokens);
        if (e != cudaSuccess) return e;
        eps_terms = (float)(d.n_embd / 32 + 8);
    }
    if (router_type == QKM_TYPE_F32)
        refine_select_kernel<QKM_TYPE_F32, false><<<n_tokens, 256, d.n_embd * 4, L.stream>>>(r, logits, norm2, gis, x, sel, d, xplanes, xscale, eps_terms, eps_abs, GroupTail{}, n_parts, (size_t)n_tokens * d.n_expert);
    else
        refine_select_kernel<QKM_TYPE_F16, false><<<n_tokens, 256, d.n_embd * 4, L.stream>>>(r, logits, norm2, gis, x, sel, d, xplanes, xscale, eps_terms, eps_abs, GroupTail{}, n_parts, (size_t)n_tokens * d.n_expert);
    L.count();
    return cudaGetLastError();
}

// ---- token-expert pair grouping: deterministic counting sort in one block --------------------
// offsets[e] .. offsets[e+1] delimit expert e's pairs; within a range pairs are in
// ascending (token, slot) order (the reference leaves the order unspecified,
// moe_group_pairs.comp:3-5).  With an expert-parallel view only resident experts
// get ranges, indexed from 0.
//
// When `plan` is given the same launch also cuts the work of the streaming kernels into
// items: for each expert with pairs, its tokens in groups of `tok_per_item`, times the
// row chunks of the gate/up matrices (items_gu) and of the down matrix (items_dn).
// The shared expert gets its own lists: every token is a "pair" (token, slot n_used)
// stored after the routed pairs, in groups of tok_per_item.
struct PlanArgs {
    StreamItem* items_gu;
    StreamItem* items_dn;
    StreamItem* items_sh_gu;
    StreamItem* items_sh_dn;
    uint32_t* n_items;   // [0] routed gate/up, [1] routed down, [2] shared gate/up, [3] shared down
    uint32_t chunks_gu, chunks_dn, tok_per_item;
};

// Expert id -> index inside the resident range [expert_first, expert_first + expert_count);
// a result >= expert_count means "not here" (the subtraction wraps for ids below the range).
// With every expert resident an id past the table is clamped to the last expert, as the
// reference's moe_group_pairs.comp does; on a shard it marks an empty record that no rank
// takes (the peer-memory exchange fills unused slots with such records).
__device__ __forceinline__ uint32_t local_expert_of(uint32_t id, uint32_t n_expert, uint32_t expert_first,
                                                    uint32_t expert_count) {
    if (expert_count >= n_expert) return min(id, n_expert - 1) - expert_first;
    return id < n_expert ? id - expert_first : 0xFFFFFFFFu;
}

__global__ void __launch_bounds__(512)
group_pairs_kernel(const qkm_sel* __restrict__ sel, uint32_t n_tokens, uint32_t n_expert, uint32_t n_used,
                   uint32_t expert_first, uint32_t expert_count, uint32_t n_chunks, uint32_t stage_ids,
                   uint32_t* __restrict__ offsets, uint32_t* __restrict__ pairs, PlanArgs plan) {
    extern __shared__ __align__(8) uint32_t s_dyn[];  // scan [512 x u64], counters [n_chunks][expert_count], totals
    uint32_t* s_scan = s_dyn;
    uint32_t* s_cnt = s_dyn + 1152;
    uint32_t* s_tot = s_cnt + (size_t)n_chunks * expert_count;
    const uint32_t tid = threadIdx.x;
    const uint32_t np = n_tokens * n_used;
    const uint32_t chunk = (np + n_chunks - 1) / n_chunks;
    for (uint32_t i = tid; i < n_chunks * expert_count; i += 512) s_cnt[i] = 0;
    // small inputs: fetch every id once, all loads in flight together, and walk them from
    // shared memory afterwards
    uint32_t* s_ids = s_tot + expert_count;
    if (stage_ids)
        for (uint32_t p = tid; p < np; p += 512) {
            const uint32_t t = p / n_used, s = p - t * n_used;
            s_ids[p] = local_expert_of(sel[t].ids[s], n_expert, expert_first, expert_count);
        }
    __syncthreads();
    auto local_expert = [&](uint32_t p) -> uint32_t {
        if (stage_ids) return s_ids[p];
        const uint32_t t = p / n_used, s = p - t * n_used;
        return local_expert_of(sel[t].ids[s], n_expert, expert_first, expert_count);
    };
    const uint32_t p0 = tid * chunk, p1 = min(np, p0 + chunk);
    if (tid < n_chunks) {
        for (uint32_t p = p0; p < p1; ++p) {
            const uint32_t e = local_expert(p);
            if (e < expert_count) s_cnt[(size_t)tid * expert_count + e]++;
        }
    }
    __syncthreads();
    for (uint32_t e = tid; e < expert_count; e += 512) {
        uint32_t run = 0;
        for (uint32_t c = 0; c < n_chunks; ++c) {
            const uint32_t v = s_cnt[(size_t)c * expert_count + e];
            s_cnt[(size_t)c * expert_count + e] = run;
            run += v;
        }
        s_tot[e] = run;
    }
    __syncthreads();
    // exclusive scan of the per-expert totals (expert_count <= 512: one element per thread)
    const uint32_t mine = tid < expert_count ? s_tot[tid] : 0u;
    const uint32_t groups = plan.n_items ? (mine + plan.tok_per_item - 1) / plan.tok_per_item : 0u;
    {
        // two scans at once: pair counts in the low half, token groups in the high half
        unsigned long long v = (unsigned long long)mine | ((unsigned long long)groups << 32);
        unsigned long long* s64 = reinterpret_cast<unsigned long long*>(s_scan);
        // inclusive scan over 512 threads: shuffles inside each warp, then the 16 warp totals
        const uint32_t lane = tid & 31u, wrp = tid >> 5;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const unsigned long long up = __shfl_up_sync(0xFFFFFFFFu, v, o);
            if (lane >= (uint32_t)o) v += up;
        }
        if (lane == 31) s64[wrp] = v;
        __syncthreads();
        if (wrp == 0) {
            unsigned long long w = lane < 16 ? s64[lane] : 0ull;
#pragma unroll
            for (int o = 1; o < 16; o <<= 1) {
                const unsigned long long up = __shfl_up_sync(0xFFFFFFFFu, w, o);
                if (lane >= (uint32_t)o) w += up;
            }
            if (lane < 16) s64[16 + lane] = w;  // inclusive totals of warps 0..lane
        }
        __syncthreads();
        if (wrp > 0) v += s64[16 + wrp - 1];
        s64[32 + tid] = v;
        __syncthreads();
        const unsigned long long incl = v;
        const unsigned long long last_incl = s64[32 + 511];
        const uint32_t off = (uint32_t)(incl & 0xFFFFFFFFull) - mine;
        const uint32_t g0 = (uint32_t)(incl >> 32) - groups;
        if (tid < expert_count) { offsets[tid] = off; s_tot[tid] = off; }
        if (tid == 511) offsets[expert_count] = (uint32_t)(last_incl & 0xFFFFFFFFull);
        if (plan.n_items) {
            if (tid == 511) {
                plan.n_items[0] = (uint32_t)(last_incl >> 32) * plan.chunks_gu;
                plan.n_items[1] = (uint32_t)(last_incl >> 32) * plan.chunks_dn;
            }
            for (uint32_t gi = 0; gi < groups; ++gi) {
                StreamItem it;
                it.expert = (uint16_t)tid;
                it.ntok = (uint8_t)min(plan.tok_per_item, mine - gi * plan.tok_per_item);
                it.pair_off = off + gi * plan.tok_per_item;
                for (uint32_t c = 0; c < plan.chunks_gu; ++c) { it.chunk = (uint8_t)c; plan.items_gu[(size_t)(g0 + gi) * plan.chunks_gu + c] = it; }
                for (uint32_t c = 0; c < plan.chunks_dn; ++c) { it.chunk = (uint8_t)c; plan.items_dn[(size_t)(g0 + gi) * plan.chunks_dn + c] = it; }
            }
        }
    }
    if (plan.n_items && plan.items_sh_gu) {
        const uint32_t sh_groups = (n_tokens + plan.tok_per_item - 1) / plan.tok_per_item;
        for (uint32_t t = tid; t < n_tokens; t += 512) pairs[np + t] = (t << 4) | n_used;
        for (uint32_t gi = tid; gi < sh_groups; gi += 512) {
            StreamItem it;
            it.expert = 0;
            it.ntok = (uint8_t)min(plan.tok_per_item, n_tokens - gi * plan.tok_per_item);
            it.pair_off = np + gi * plan.tok_per_item;
            for (uint32_t c = 0; c < plan.chunks_gu; ++c) { it.chunk = (uint8_t)c; plan.items_sh_gu[(size_t)gi * plan.chunks_gu + c] = it; }
            for (uint32_t c = 0; c < plan.chunks_dn; ++c) { it.chunk = (uint8_t)c; plan.items_sh_dn[(size_t)gi * plan.chunks_dn + c] = it; }
        }
        if (tid == 0) { plan.n_items[2] = sh_groups * plan.chunks_gu; plan.n_items[3] = sh_groups * plan.chunks_dn; }
    }
    __syncthreads();
    if (tid < n_chunks) {
        for (uint32_t p = p0; p < p1; ++p) {
            const uint32_t t = p / n_used, s = p - t * n_used;
            const uint32_t e = local_expert(p);
            if (e < expert_count) {
                const uint32_t dst = s_tot[e] + s_cnt[(size_t)tid * expert_count + e]++;
                pairs[dst] = (t << 4) | s;
            }
        }
    }
}

static cudaError_t group_pairs_launch(const Launch& L, const qkm_dims& d, const qkm_sel* sel, uint32_t n_tokens,
                                      uint32_t* offsets, uint32_t* pairs, uint32_t expert_first,
                                      uint32_t expert_count, const PlanArgs& plan) {
    if (expert_count == 0) { expert_first = 0; expert_count = d.n_expert; }
    if (expert_count > 512) return cudaErrorInvalidValue;
    // one chunk of pairs per thread: enough chunks to spread the pairs, no more counters
    // than 32768 words of shared memory hold
    const uint32_t np = n_tokens * d.n_used;
    uint32_t n_chunks = 32768u / expert_count;
    if (n_chunks > 512) n_chunks = 512;
    const uint32_t want = (np + 7) / 8;
    if (n_chunks > want) n_chunks = want ? want : 1;
    const uint32_t stage_ids = np <= 8192 ? 1u : 0u;
    const size_t smem = ((size_t)n_chunks * expert_count + expert_count + 1152 + (stage_ids ? np : 0)) * sizeof(uint32_t);
    cudaError_t e = cudaFuncSetAttribute(group_pairs_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)((32768 + 512 + 1152 + 8192) * sizeof(uint32_t)));
    if (e != cudaSuccess) return e;
    group_pairs_kernel<<<1, 512, smem, L.stream>>>(sel, n_tokens, d.n_expert, d.n_used, expert_first,
                                                   expert_count, n_chunks, stage_ids, offsets, pairs, plan);
    L.count();
    return cudaGetLastError();
}

// Work lists of the shared expert: every token is a "pair" (token, slot n_used) stored
// after the routed pairs, in groups of tok_per_item.  Depends on n_tokens only.
__global__ void shared_plan_kernel(uint32_t n_tokens, uint32_t n_used, uint32_t* __restrict__ pairs,
                                   StreamItem* __restrict__ items_gu, uint32_t chunks_gu,
                                   StreamItem* __restrict__ items_dn, uint32_t chunks_dn,
                                   uint32_t tok_per_item, uint32_t* __restrict__ n_items) {
    const uint32_t np = n_tokens * n_used, tid = threadIdx.x;
    const uint32_t groups = (n_tokens + tok_per_item - 1) / tok_per_item;
    for (uint32_t t = tid; t < n_tokens; t += blockDim.x) pairs[np + t] = (t << 4) | n_used;
    for (uint32_t gi = tid; gi < groups; gi += blockDim.x) {
        StreamItem it;
        it.expert = 0;
        it.ntok = (uint8_t)min(tok_per_item, n_tokens - gi * tok_per_item);
        it.pair_off = np + gi * tok_per_item;
        for (uint32_t c = 0; c < chunks_gu; ++c) { it.chunk = (uint8_t)c; items_gu[(size_t)gi * chunks_gu + c] = it; }
        for (uint32_t c = 0; c < chunks_dn; ++c) { it.chunk = (uint8_t)c; items_dn[(size_t)gi * chunks_dn + c] = it; }
    }
    if (tid == 0) { n_items[0] = groups * chunks_gu; n_items[1] = groups * chunks_dn; }
}

cudaError_t launch_shared_plan(const Launch& L, const qkm_dims& d, uint32_t n_tokens, uint32_t* pairs,
                               StreamItem* items_gu, uint32_t chunks_gu, StreamItem* items_dn,
                               uint32_t chunks_dn, uint32_t tok_per_item, uint32_t* n_items) {
    if (n_tokens == 0) return cudaSuccess;
    shared_plan_kernel<<<1, 256, 0, L.stream>>>(n_tokens, d.n_used, pairs, items_gu, chunks_gu, items_dn, chunks_dn,
                                                tok_per_item, n_items);
    L.count();
    return cudaGetLastError();
}

// ---- pair grouping for large batches: three launches over many blocks ---------------------------
// The pairs (token-major, slot-minor) are cut into runs of 128, one per warp.  (1) every warp
// counts its run per expert; (2) one block turns the counts into start positions (scan over the
// runs per expert, then over the experts); (3) every warp places its pairs: position = expert
// start + start of the run within the expert + rank within the run, which keeps each expert's
// pairs in ascending (token, slot) order without atomics on global memory.
namespace gw {
constexpr uint32_t kRun = 128;        // pairs per warp
constexpr uint32_t kWarps = 16;       // warps per block
constexpr uint32_t kInvalid = 0xFFFFFFFFu;
}  // namespace gw

__device__ __forceinline__ uint32_t gw_local_expert(const qkm_sel* __restrict__ sel, uint32_t p, uint32_t n_used,
                                                    uint32_t n_expert, uint32_t expert_first, uint32_t expert_count) {
    const uint32_t t = p / n_used, s = p - t * n_used;
    return local_expert_of(sel[t].ids[s], n_expert, expert_first, expert_count);
}

__global__ void __launch_bounds__(gw::kWarps * 32)
group_count_kernel(const qkm_sel* __restrict__ sel, uint32_t np, uint32_t n_used, uint32_t n_expert,
                   uint32_t expert_first, uint32_t expert_count, uint32_t n_runs, uint32_t* __restrict__ hist) {
    extern __shared__ uint32_t s_cnt[];   // [kWarps][expert_count]
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
    const uint32_t run = blockIdx.x * gw::kWarps + warp;
    uint32_t* mine = s_cnt + (size_t)warp * expert_count;
    for (uint32_t e = lane; e < expert_count; e += 32) mine[e] = 0;
    __syncwarp();
    const uint32_t p0 = run * gw::kRun;
    for (uint32_t i = 0; i < gw::kRun; i += 32) {
        const uint32_t p = p0 + i + lane;
        if (p < np) {
            const uint32_t e = gw_local_expert(sel, p, n_used, n_expert, expert_first, expert_count);
            if (e < expert_count) atomicAdd(&mine[e], 1u);
        }
    }
    __syncwarp();
    if (p0 < np)
        for (uint32_t e = lane; e < expert_count; e += 32) hist[(size_t)e * n_runs + run] = mine[e];
}

// hist is [expert][run]: one warp per expert turns its row of counts into exclusive prefix sums
// (32 runs per step, coalesced) and leaves the expert's total in totals[e].
__global__ void __launch_bounds__(256)
group_scan_kernel(uint32_t* __restrict__ hist, uint32_t n_runs, uint32_t expert_count, uint32_t* __restrict__ totals) {
    const uint32_t e = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31u;
    if (e >= expert_count) return;
    uint32_t* row = hist + (size_t)e * n_runs;
    uint32_t run_total = 0;
    for (uint32_t r0 = 0; r0 < n_runs; r0 += 32) {
        const uint32_t r = r0 + lane;
        const uint32_t v = r < n_runs ? row[r] : 0u;
        uint32_t inc = v;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const uint32_t up = __shfl_up_sync(0xFFFFFFFFu, inc, o);
            if (lane >= (uint32_t)o) inc += up;
        }
        if (r < n_runs) row[r] = run_total + inc - v;
        run_total += __shfl_sync(0xFFFFFFFFu, inc, 31);
    }
    if (lane == 0) totals[e] = run_total;
}

__global__ void __launch_bounds__(gw::kWarps * 32)
group_place_kernel(const qkm_sel* __restrict__ sel, uint32_t np, uint32_t n_used, uint32_t n_expert,
                   uint32_t expert_first, uint32_t expert_count, uint32_t n_runs, const uint32_t* __restrict__ hist,
                   const uint32_t* __restrict__ totals, uint32_t* __restrict__ offsets, uint32_t* __restrict__ pairs,
                   uint32_t* __restrict__ pos_of) {
    extern __shared__ uint32_t s_cnt[];   // [kWarps][expert_count]: pairs of the run placed so far, per expert
    __shared__ uint32_t s_off[513];       // exclusive scan of the expert totals (every block redoes it: 512 adds)
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
    const uint32_t run = blockIdx.x * gw::kWarps + warp;
    uint32_t* mine = s_cnt + (size_t)warp * expert_count;
    for (uint32_t e = lane; e < expert_count; e += 32) mine[e] = 0;
    {
        const uint32_t e = threadIdx.x;   // 512 threads, expert_count <= 512
        const uint32_t tot = e < expert_count ? totals[e] : 0u;
        uint32_t inc = tot;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const uint32_t up = __shfl_up_sync(0xFFFFFFFFu, inc, o);
            if (lane >= (uint32_t)o) inc += up;
        }
        __shared__ uint32_t s_wtot[16];
        if (lane == 31) s_wtot[warp] = inc;
        __syncthreads();
        uint32_t base = 0;
        for (uint32_t w = 0; w < warp; ++w) base += s_wtot[w];
        s_off[e] = base + inc - tot;
        if (e == 511) s_off[512] = base + inc;
        __syncthreads();
        if (blockIdx.x == 0) {
            if (e < expert_count) offsets[e] = s_off[e];
            if (e == 0) offsets[expert_count] = s_off[512];
        }
    }
    const uint32_t p0 = run * gw::kRun;
    for (uint32_t i = 0; i < gw::kRun; i += 32) {
        const uint32_t p = p0 + i + lane;
        uint32_t e = gw::kInvalid;
        if (p < np) {
            e = gw_local_expert(sel, p, n_used, n_expert, expert_first, expert_count);
            if (e >= expert_count) e = gw::kInvalid;
        }
        // lanes with the same expert: rank by lane, the lowest lane keeps the run's counter
        const uint32_t same = __match_any_sync(0xFFFFFFFFu, e);
        const uint32_t rank = __popc(same & ((1u << lane) - 1u));
        const uint32_t leader = __ffs(same) - 1;
        uint32_t before = 0;
        if (e != gw::kInvalid && lane == leader) { before = mine[e]; mine[e] = before + __popc(same); }
        before = __shfl_sync(0xFFFFFFFFu, before, leader);
        __syncwarp();
        if (p < np) {
            const uint32_t t = p / n_used, s = p - t * n_used;
            uint32_t pos = gw::kInvalid;
            if (e != gw::kInvalid) {
                pos = s_off[e] + hist[(size_t)e * n_runs + run] + before + rank;
                pairs[pos] = (t << 4) | s;
            }
            if (pos_of) pos_of[t * (n_used + 1) + s] = pos;
        }
    }
}

size_t group_wide_scratch_bytes(uint32_t n_tokens, uint32_t n_used, uint32_t expert_count) {
    const size_t runs = ((size_t)n_tokens * n_used + gw::kRun - 1) / gw::kRun;
    return ((runs + gw::kWarps) * expert_count + 512) * sizeof(uint32_t);   // [expert][run] counts, then the expert totals
}

cudaError_t launch_group_pairs_wide(const Launch& L, const qkm_dims& d, const qkm_sel* sel, uint32_t n_tokens,
                                    uint32_t* offsets, uint32_t* pairs, uint32_t expert_first, uint32_t expert_count,
                                    uint32_t* hist, uint32_t* pos_of) {
    if (expert_count == 0) { expert_first = 0; expert_count = d.n_expert; }
    if (expert_count > 512) return cudaErrorInvalidValue;
    const uint32_t np = n_tokens * d.n_used;
    const uint32_t n_runs = (np + gw::kRun - 1) / gw::kRun, blocks = (n_runs + gw::kWarps - 1) / gw::kWarps;
    const size_t smem = (size_t)gw::kWarps * expert_count * sizeof(uint32_t);
    if (np == 0) {
        cudaError_t e = cudaMemsetAsync(offsets, 0, (expert_count + 1) * sizeof(uint32_t), L.stream);
        return e;
    }
    uint32_t* totals = hist + (size_t)n_runs * expert_count;
    group_count_kernel<<<blocks, gw::kWarps * 32, smem, L.stream>>>(sel, np, d.n_used, d.n_expert, expert_first, expert_count, n_runs, hist);
    group_scan_kernel<<<(expert_count + 7) / 8, 256, 0, L.stream>>>(hist, n_runs, expert_count, totals);
    group_place_kernel<<<blocks, gw::kWarps * 32, smem, L.stream>>>(sel, np, d.n_used, d.n_expert, expert_first, expert_count, n_runs,
                                                                      hist, totals, offsets, pairs, pos_of);
    L.count(3);
    return cudaGetLastError();
}

cudaError_t launch_group_pairs(const Launch& L, const qkm_dims& d, const qkm_sel* sel, uint32_t n_tokens,
                               uint32_t* offsets, uint32_t* pairs, uint32_t expert_first,
                               uint32_t expert_count) {
    return group_pairs_launch(L, d, sel, n_tokens, offsets, pairs, expert_first, expert_count, PlanArgs{});
}

cudaError_t launch_group_plan(const Launch& L, const qkm_dims& d, const qkm_sel* sel, uint32_t n_tokens,
                              uint32_t* offsets, uint32_t* pairs, uint32_t expert_first, uint32_t expert_count,
                              StreamItem* items_gu, uint32_t chunks_gu, StreamItem* items_dn,
                              uint32_t chunks_dn, StreamItem* items_sh_gu, StreamItem* items_sh_dn,
                              uint32_t tok_per_item, uint32_t* n_items) {
    PlanArgs plan{items_gu, items_dn, items_sh_gu, items_sh_dn, n_items, chunks_gu, chunks_dn, tok_per_item};
    return group_pairs_launch(L, d, sel, n_tokens, offsets, pairs, expert_first, expert_count, plan);
}

}  // namespace qkm
