// Layer entry / tail around the MoE block: residual adds fused with the RMS norm that
// produces the next block's input.  One block per row; a row's sums stay in registers
// between the reduction and the scaling pass.
//
// Follows shaders/add_rmsnorm.comp:22-40 (y = a + b, xn = y * w / sqrt(mean(y^2) + eps)),
// shaders/add_rms3.comp:23-41 (three streams) and shaders/add_rms3_grouped.comp:22-50
// (the routed stream given as per-slot contributions [row][n_used][n], folded in slot
// order).  The stored sums use the shaders' order of additions, so they are bit-identical
// to an f32 evaluation of the same expression; the mean of squares is accumulated in f32
// per thread and combined in a fixed tree.
#include <cuda_runtime.h>
#include <stdint.h>

#include "qkm_common.cuh"
#include "qkm_kernels.h"

namespace qkm {

namespace {

constexpr int kTailThreads = 256;
constexpr int kTailMaxPerThread = 8;   // float4 units per thread: n <= 256 * 8 * 4 = 8192

// MODE 0: a + b;  1: a + b + c2;  2: a + (sum over slots of routed) + c2
template <int MODE>
__global__ void __launch_bounds__(kTailThreads)
add_rms_kernel(const float* __restrict__ a, const float* __restrict__ b, const float* __restrict__ c2,
               const float* __restrict__ w, float* __restrict__ s, float* __restrict__ xn, uint32_t n,
               uint32_t n_used, float eps) {
    __shared__ float s_red[kTailThreads / 32];
    const uint32_t row = blockIdx.x, tid = threadIdx.x, n4 = n / 4;
    const float4* a4 = reinterpret_cast<const float4*>(a + (size_t)row * n);
    const float4* c4 = MODE >= 1 ? reinterpret_cast<const float4*>(c2 + (size_t)row * n) : nullptr;
    float4 v[kTailMaxPerThread];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < kTailMaxPerThread; ++i) {
        const uint32_t u = tid + i * kTailThreads;
        if (u < n4) {
            float4 x = a4[u];
            if (MODE == 2) {
                float4 r = make_float4(0.f, 0.f, 0.f, 0.f);
                for (uint32_t k = 0; k < n_used; ++k) {
                    const float4 q = reinterpret_cast<const float4*>(b + ((size_t)row * n_used + k) * n)[u];
                    r.x += q.x; r.y += q.y; r.z += q.z; r.w += q.w;
                }
                x.x += r.x; x.y += r.y; x.z += r.z; x.w += r.w;
            } else {
                const float4 q = reinterpret_cast<const float4*>(b + (size_t)row * n)[u];
                x.x += q.x; x.y += q.y; x.z += q.z; x.w += q.w;
            }
            if (MODE >= 1) {
                const float4 q = c4[u];
                x.x += q.x; x.y += q.y; x.z += q.z; x.w += q.w;
            }
            reinterpret_cast<float4*>(s + (size_t)row * n)[u] = x;
            ss += x.x * x.x; ss += x.y * x.y; ss += x.z * x.z; ss += x.w * x.w;
            v[i] = x;
        }
    }
    ss = warp_sum(ss);
    if ((tid & 31u) == 0) s_red[tid >> 5] = ss;
    __syncthreads();
    float tot = 0.f;
#pragma unroll
    for (int i = 0; i < kTailThreads / 32; ++i) tot += s_red[i];
    const float scale = 1.0f / sqrtf(tot / (float)n + eps);
#pragma unroll
    for (int i = 0; i < kTailMaxPerThread; ++i) {
        const uint32_t u = tid + i * kTailThreads;
        if (u < n4) {
            const float4 g = reinterpret_cast<const float4*>(w)[u];
            float4 o;
            o.x = v[i].x * scale * g.x; o.y = v[i].y * scale * g.y; o.z = v[i].z * scale * g.z; o.w = v[i].w * scale * g.w;
            reinterpret_cast<float4*>(xn + (size_t)row * n)[u] = o;
        }
    }
}

}  // namespace

cudaError_t launch_add_rms(const Launch& L, int mode, const float* a, const float* b, const float* c2, const float* w,
                           float* s, float* xn, uint32_t n_rows, uint32_t n, uint32_t n_used, float eps) {
    if (n_rows == 0) return cudaSuccess;
    if (n == 0 || n % 4 || n > kTailThreads * kTailMaxPerThread * 4) return cudaErrorInvalidValue;
    switch (mode) {
        case 0: add_rms_kernel<0><<<n_rows, kTailThreads, 0, L.stream>>>(a, b, c2, w, s, xn, n, n_used, eps); break;
        case 1: add_rms_kernel<1><<<n_rows, kTailThreads, 0, L.stream>>>(a, b, c2, w, s, xn, n, n_used, eps); break;
        case 2: add_rms_kernel<2><<<n_rows, kTailThreads, 0, L.stream>>>(a, b, c2, w, s, xn, n, n_used, eps); break;
        default: return cudaErrorInvalidValue;
    }
    L.count();
    return cudaGetLastError();
}

}  // namespace qkm

// ---- greedy token: argmax over a row of logits ----------------------------------------------------
// shaders/argmax1.comp:17-40 + argmax2.comp:16-32: the largest value wins, the lower index on
// ties; a value must exceed -3.4e38 to be taken (so NaN never wins and an all-floor row gives 0).
// Two launches as in the reference: up to 64 spans per row, then one block per row.
namespace qkm {
namespace {

constexpr uint32_t kArgSpans = 64;

__device__ __forceinline__ void arg_better(float& bv, uint32_t& bi, float v, uint32_t i) {
    if (v > bv || (v == bv && i < bi)) { bv = v; bi = i; }
}

__device__ __forceinline__ void arg_block_reduce(float& bv, uint32_t& bi) {
    __shared__ float s_v[8];
    __shared__ uint32_t s_i[8];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float v = __shfl_xor_sync(0xFFFFFFFFu, bv, o);
        const uint32_t i = __shfl_xor_sync(0xFFFFFFFFu, bi, o);
        arg_better(bv, bi, v, i);
    }
    if ((threadIdx.x & 31u) == 0) { s_v[threadIdx.x >> 5] = bv; s_i[threadIdx.x >> 5] = bi; }
    __syncthreads();
    if (threadIdx.x == 0)
        for (int w = 1; w < 8; ++w) arg_better(bv, bi, s_v[w], s_i[w]);
}

__global__ void __launch_bounds__(256)
argmax_spans_kernel(const float* __restrict__ logits, uint32_t n, uint32_t span, float* __restrict__ vals,
                    uint32_t* __restrict__ idxs) {
    const uint32_t row = blockIdx.y, w = blockIdx.x;
    const float* l = logits + (size_t)row * n;
    const uint32_t start = w * span, end = min(start + span, n);
    float bv = -3.4e38f;
    uint32_t bi = 0xFFFFFFFFu;     // "nothing taken": loses every tie
    for (uint32_t i = start + threadIdx.x; i < end; i += 256) {
        const float v = l[i];
        if (v > bv) { bv = v; bi = i; }
    }
    arg_block_reduce(bv, bi);
    if (threadIdx.x == 0) { vals[row * kArgSpans + w] = bv; idxs[row * kArgSpans + w] = bi; }
}

__global__ void __launch_bounds__(256)
argmax_final_kernel(const float* __restrict__ vals, const uint32_t* __restrict__ idxs, uint32_t m, uint32_t* __restrict__ tok) {
    const uint32_t row = blockIdx.x, t = threadIdx.x;
    float bv = t < m ? vals[row * kArgSpans + t] : -3.4e38f;
    uint32_t bi = t < m ? idxs[row * kArgSpans + t] : 0xFFFFFFFFu;
    arg_block_reduce(bv, bi);
    if (t == 0) tok[row] = bi == 0xFFFFFFFFu ? 0u : bi;
}

}  // namespace

size_t argmax_scratch_bytes(uint32_t n_rows) { return (size_t)n_rows * kArgSpans * 8; }

cudaError_t launch_argmax(const Launch& L, const float* logits, uint32_t n_rows, uint32_t n, void* scratch, uint32_t* tok) {
    if (n_rows == 0) return cudaSuccess;
    if (n == 0) return cudaErrorInvalidValue;
    uint32_t spans = (n + 4095) / 4096;
    if (spans > kArgSpans) spans = kArgSpans;
    const uint32_t span = (n + spans - 1) / spans;
    float* vals = (float*)scratch;
    uint32_t* idxs = (uint32_t*)(vals + (size_t)n_rows * kArgSpans);
    argmax_spans_kernel<<<dim3(spans, n_rows), 256, 0, L.stream>>>(logits, n, span, vals, idxs);
    argmax_final_kernel<<<n_rows, 256, 0, L.stream>>>(vals, idxs, spans, tok);
    L.count(2);
    return cudaGetLastError();
}

}  // namespace qkm
