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
