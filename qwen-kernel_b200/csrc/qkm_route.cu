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

// ---- logits: one warp per expert row, kTokPerWarp tokens per pass ---------------------------
// Each lane adds its K/32 products in a fixed order (8-element units lane, lane+32, ...)
// and the lanes meet in a 5-level tree: the order the error bound of the refined
// selection assumes.  Also writes |router row|^2 when row_norm2 != NULL.
static constexpr int kTokPerWarp = 4;

template <int TYPE>
__global__ void __launch_bounds__(256)
logits_kernel(const uint8_t* __restrict__ router, const float* __restrict__ x, float* __restrict__ logits,
              float* __restrict__ row_norm2, uint32_t n_expert, uint32_t K, uint32_t n_tokens) {
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
    const uint32_t e = blockIdx.x * 8u + warp;
    const uint32_t t0 = blockIdx.y * kTokPerWarp;
    if (e >= n_expert) return;
    const uint8_t* row = router + (size_t)e * row_bytes(TYPE, K);
    float acc[kTokPerWarp], nrm = 0.f;
#pragma unroll
    for (int j = 0; j < kTokPerWarp; ++j) acc[j] = 0.f;
    for (uint32_t u = lane; u < K / 8; u += 32) {
        float w[8];
        dequant8<TYPE>(row, u * 8, w);
#pragma unroll
        for (int i = 0; i < 8; ++i) nrm += w[i] * w[i];
#pragma unroll
        for (int j = 0; j < kTokPerWarp; ++j) {
            if (t0 + j < n_tokens) {
                const float* xt = x + (size_t)(t0 + j) * K + u * 8;
                const float4 a = *reinterpret_cast<const float4*>(xt);
                const float4 b = *reinterpret_cast<const float4*>(xt + 4);
                float s = acc[j];
                s += w[0] * a.x; s += w[1] * a.y; s += w[2] * a.z; s += w[3] * a.w;
                s += w[4] * b.x; s += w[5] * b.y; s += w[6] * b.z; s += w[7] * b.w;
                acc[j] = s;
            }
        }
    }
#pragma unroll
    for (int j = 0; j < kTokPerWarp; ++j) {
        const float v = warp_sum(acc[j]);
        if (lane == 0 && t0 + j < n_tokens) logits[(size_t)(t0 + j) * n_expert + e] = v;
    }
    if (row_norm2 != nullptr && blockIdx.y == 0) {
        nrm = warp_sum(nrm);
        if (lane == 0) row_norm2[e] = nrm;
    }
}

cudaError_t launch_logits(const Launch& L, const qkm_dims& d, uint32_t router_type, const void* router,
                          const float* x, float* logits, float* row_norm2, uint32_t n_tokens) {
    if (n_tokens == 0) return cudaSuccess;
    const dim3 grid((d.n_expert + 7) / 8, (n_tokens + kTokPerWarp - 1) / kTokPerWarp);
    const uint8_t* r = (const uint8_t*)router;
    if (router_type == QKM_TYPE_F32)
        logits_kernel<QKM_TYPE_F32><<<grid, 256, 0, L.stream>>>(r, x, logits, row_norm2, d.n_expert, d.n_embd, n_tokens);
    else if (router_type == QKM_TYPE_F16)
        logits_kernel<QKM_TYPE_F16><<<grid, 256, 0, L.stream>>>(r, x, logits, row_norm2, d.n_expert, d.n_embd, n_tokens);
    else
        return cudaErrorInvalidValue;
    L.count();
    return cudaGetLastError();
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

// ---- refined selection: f32 ranking, f64 re-evaluation of the boundary ---------------------
static constexpr int kMaxCand = 64;

template <int TYPE>
__global__ void __launch_bounds__(256)
refine_select_kernel(const uint8_t* __restrict__ router, const float* __restrict__ logits,
                     const float* __restrict__ row_norm2, const float* __restrict__ gis,
                     const float* __restrict__ x, qkm_sel* __restrict__ sel, qkm_dims d,
                     int8_t* __restrict__ xplanes, float* __restrict__ xscale) {
    __shared__ unsigned long long s_warp[8];
    __shared__ double s_red[8];
    __shared__ float s_f[8];
    __shared__ uint32_t s_cand[kMaxCand];
    __shared__ double s_val[kMaxCand];
    __shared__ uint32_t s_ncand;
    const uint32_t t = blockIdx.x, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31u;
    const float* xt = x + (size_t)t * d.n_embd;
    const float* lt = logits + (size_t)t * d.n_expert;
    const uint32_t id0 = tid, id1 = tid + 256u;
    const float l0 = id0 < d.n_expert ? sane(lt[id0]) : kFloor;
    const float l1 = id1 < d.n_expert ? sane(lt[id1]) : kFloor;
    const uint32_t pid0 = id0 < d.n_expert ? id0 : 0xFFFFFFFEu;
    const uint32_t pid1 = id1 < d.n_expert ? id1 : 0xFFFFFFFEu;

    // the streaming expert kernels read x as int8 digit planes: encode it here, where the
    // row is being read anyway
    if (xplanes != nullptr) {
        __shared__ float s_max[8];
        block_encode_digits(xt, xplanes + (size_t)t * 4 * d.n_embd, xscale + t, d.n_embd, s_max);
    }
    // |x|^2 and max |row|^2 for the error bound
    float xs = 0.f, rn = 0.f;
    for (uint32_t k = tid; k < d.n_embd; k += 256) xs += xt[k] * xt[k];
    if (id0 < d.n_expert) rn = row_norm2[id0];
    if (id1 < d.n_expert) rn = fmaxf(rn, row_norm2[id1]);
    xs = warp_sum(xs);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) rn = fmaxf(rn, __shfl_xor_sync(0xFFFFFFFFu, rn, o));
    if (lane == 0) { s_f[warp] = xs; s_red[warp] = (double)rn; }
    if (tid == 0) s_ncand = 0;
    __syncthreads();
    float x2 = 0.f, r2 = 0.f;
#pragma unroll
    for (int w = 0; w < 8; ++w) { x2 += s_f[w]; r2 = fmaxf(r2, (float)s_red[w]); }

    // k-th largest f32 logit
    float v0 = l0, v1 = l1, kth = kFloor;
    for (uint32_t i = 0; i < d.n_used; ++i) {
        const unsigned long long k = block_argmax(v0, pid0, v1, pid1, s_warp);
        const uint32_t id = 0xFFFFFFFFu - (uint32_t)(k & 0xFFFFFFFFull);
        uint32_t b = (uint32_t)(k >> 32);
        b = (b & 0x80000000u) ? (b & 0x7FFFFFFFu) : ~b;
        kth = __uint_as_float(b);
        if (id == id0) v0 = kFloor;
        if (id == id1) v1 = kFloor;
    }
    // Error bound of one f32 logit: each lane adds K/32 products in sequence, then a
    // 5-level tree; |err| <= (K/32 + 6) * 2^-24 * sum|w_k x_k| <= that * |w| * |x|.
    // Doubled for safety, and doubled again because two logits are compared.
    const float eps = (float)(d.n_embd / 32 + 6) * 5.9604645e-8f * sqrtf(r2) * sqrtf(x2);
    const float thresh = kth - 4.0f * eps;

    // candidates: every expert at or above the threshold
    // (written as !(l < thresh) so a NaN threshold - NaN in x - admits every expert)
    const bool c0 = id0 < d.n_expert && !(l0 < thresh), c1 = id1 < d.n_expert && !(l1 < thresh);
    if (c0) { const uint32_t p = atomicAdd(&s_ncand, 1u); if (p < kMaxCand) s_cand[p] = id0; }
    if (c1) { const uint32_t p = atomicAdd(&s_ncand, 1u); if (p < kMaxCand) s_cand[p] = id1; }
    __syncthreads();
    const uint32_t ncand_raw = s_ncand;
    __syncthreads();
    // Too many near-ties (or non-finite input: everything sits at the floor): fall
    // back to evaluating experts in id order, kMaxCand at a time is not enough, so
    // take the exact route of ranking ALL experts in f64 through the global pass below.
    const bool all = ncand_raw > kMaxCand || ncand_raw < d.n_used;
    const uint32_t total = all ? d.n_expert : ncand_raw;

    // f64 re-evaluation.  In the `all` case values stream through s_val in chunks and
    // a running top-k (ids, values) is kept by thread 0.
    __shared__ uint32_t s_best_id[16];
    __shared__ double s_best_val[16];
    __shared__ uint32_t s_nbest;
    if (tid == 0) s_nbest = 0;
    const size_t rb = row_bytes(TYPE, d.n_embd);
    for (uint32_t base = 0; base < total; base += kMaxCand) {
        const uint32_t n = min((uint32_t)kMaxCand, total - base);
        __syncthreads();
        for (uint32_t c = warp; c < n; c += 8) {
            const uint32_t e = all ? base + c : s_cand[c];
            const uint8_t* row = router + (size_t)e * rb;
            double acc = 0.0;
            for (uint32_t u = lane; u < d.n_embd / 8; u += 32) {
                float w[8];
                dequant8<TYPE>(row, u * 8, w);
#pragma unroll
                for (int i = 0; i < 8; ++i) acc += (double)w[i] * (double)xt[u * 8 + i];
            }
            acc = warp_sum(acc);
            if (lane == 0) {
                s_val[c] = (isnan(acc) || isinf(acc)) ? (double)kFloor : acc;
                if (all) s_cand[c] = e;
            }
        }
        __syncthreads();
        if (tid == 0) {
            // merge this chunk into the running top-k: (value desc, id asc)
            uint32_t nb = s_nbest;
            for (uint32_t c = 0; c < n; ++c) {
                const double v = s_val[c];
                const uint32_t e = s_cand[c];
                uint32_t pos = nb;
                while (pos > 0 && (s_best_val[pos - 1] < v || (s_best_val[pos - 1] == v && s_best_id[pos - 1] > e))) --pos;
                if (pos >= d.n_used) continue;
                const uint32_t last = nb < d.n_used ? nb : d.n_used - 1;
                for (uint32_t j = last; j > pos; --j) { s_best_val[j] = s_best_val[j - 1]; s_best_id[j] = s_best_id[j - 1]; }
                s_best_val[pos] = v;
                s_best_id[pos] = e;
                if (nb < d.n_used) ++nb;
            }
            s_nbest = nb;
        }
    }
    const double sg = block_dot_f64(gis, xt, d.n_embd, s_red);
    if (tid == 0) {
        double w[16], sum = 0.0;
        for (uint32_t i = 0; i < d.n_used; ++i) { w[i] = exp(s_best_val[i] - s_best_val[0]); sum += w[i]; }
        for (uint32_t i = 0; i < 16; ++i) {
            sel[t].ids[i] = i < d.n_used ? min(s_best_id[i], d.n_expert - 1) : 0u;
            sel[t].w[i] = i < d.n_used ? (float)(w[i] / sum) : 0.f;
        }
        sel[t].w_shared = (float)(1.0 / (1.0 + exp(-sg)));
        sel[t].route_done = 0;
#pragma unroll
        for (int i = 0; i < 6; ++i) sel[t].pad[i] = 0.f;
    }
}

size_t route_scratch_bytes(uint32_t n_tokens, uint32_t n_expert) {
    return ((size_t)n_tokens * n_expert + n_expert) * sizeof(float);
}

cudaError_t launch_route_select(const Launch& L, const qkm_dims& d, uint32_t router_type,
                                const void* router, const float* gis, const float* x, qkm_sel* sel,
                                uint32_t n_tokens, void* scratch, int8_t* xplanes, float* xscale) {
    if (n_tokens == 0) return cudaSuccess;
    float* logits = (float*)scratch;
    float* norm2 = logits + (size_t)n_tokens * d.n_expert;
    cudaError_t e = launch_logits(L, d, router_type, router, x, logits, norm2, n_tokens);
    if (e != cudaSuccess) return e;
    const uint8_t* r = (const uint8_t*)router;
    if (router_type == QKM_TYPE_F32)
        refine_select_kernel<QKM_TYPE_F32><<<n_tokens, 256, 0, L.stream>>>(r, logits, norm2, gis, x, sel, d, xplanes, xscale);
    else
        refine_select_kernel<QKM_TYPE_F16><<<n_tokens, 256, 0, L.stream>>>(r, logits, norm2, gis, x, sel, d, xplanes, xscale);
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

__global__ void __launch_bounds__(512)
group_pairs_kernel(const qkm_sel* __restrict__ sel, uint32_t n_tokens, uint32_t n_expert, uint32_t n_used,
                   uint32_t expert_first, uint32_t expert_count, uint32_t n_chunks,
                   uint32_t* __restrict__ offsets, uint32_t* __restrict__ pairs, PlanArgs plan) {
    extern __shared__ __align__(8) uint32_t s_dyn[];  // scan [512 x u64], counters [n_chunks][expert_count], totals
    uint32_t* s_scan = s_dyn;
    uint32_t* s_cnt = s_dyn + 1024;
    uint32_t* s_tot = s_cnt + (size_t)n_chunks * expert_count;
    const uint32_t tid = threadIdx.x;
    const uint32_t np = n_tokens * n_used;
    const uint32_t chunk = (np + n_chunks - 1) / n_chunks;
    for (uint32_t i = tid; i < n_chunks * expert_count; i += 512) s_cnt[i] = 0;
    __syncthreads();
    const uint32_t p0 = tid * chunk, p1 = min(np, p0 + chunk);
    if (tid < n_chunks) {
        for (uint32_t p = p0; p < p1; ++p) {
            const uint32_t t = p / n_used, s = p - t * n_used;
            const uint32_t e = min(sel[t].ids[s], n_expert - 1) - expert_first;  // wraps when below
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
        s64[tid] = v;
        __syncthreads();
        for (uint32_t o = 1; o < 512; o <<= 1) {
            const unsigned long long add = tid >= o ? s64[tid - o] : 0ull;
            __syncthreads();
            s64[tid] += add;
            __syncthreads();
        }
        const unsigned long long incl = s64[tid];
        const uint32_t off = (uint32_t)(incl & 0xFFFFFFFFull) - mine;
        const uint32_t g0 = (uint32_t)(incl >> 32) - groups;
        if (tid < expert_count) { offsets[tid] = off; s_tot[tid] = off; }
        if (tid == 511) offsets[expert_count] = (uint32_t)(incl & 0xFFFFFFFFull);
        if (plan.n_items) {
            if (tid == 511) {
                plan.n_items[0] = (uint32_t)(incl >> 32) * plan.chunks_gu;
                plan.n_items[1] = (uint32_t)(incl >> 32) * plan.chunks_dn;
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
            const uint32_t e = min(sel[t].ids[s], n_expert - 1) - expert_first;
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
    const size_t smem = ((size_t)n_chunks * expert_count + expert_count + 2 * 512) * sizeof(uint32_t);
    cudaError_t e = cudaFuncSetAttribute(group_pairs_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)((32768 + 512 + 1024) * sizeof(uint32_t)));
    if (e != cudaSuccess) return e;
    group_pairs_kernel<<<1, 512, smem, L.stream>>>(sel, n_tokens, d.n_expert, d.n_used, expert_first,
                                                   expert_count, n_chunks, offsets, pairs, plan);
    L.count();
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
