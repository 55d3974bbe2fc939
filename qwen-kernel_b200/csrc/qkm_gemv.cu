// Dense dequant-GEMV and the dequantisation probe.
//
// Replaces the reference's gemv_{f16,q8_0,q6_k,iq4_xs,iq3_xxs}.comp
// (y[M] = W[M,K] . x[K] on raw ggml blocks, z-batched over n inputs,
// shaders/gemv_q8_0.comp:31-32) and exposes dequant_row_* (src/quants.h:70-165)
// on the GPU so dequantised weights can be compared bit-for-bit.
#include "qkm_common.cuh"
#include "qkm_kernels.h"

namespace qkm {

// ---- dequantisation probe: one thread per 8-element unit ---------------------------
template <int TYPE>
__global__ void dequant_kernel(const uint8_t* __restrict__ blocks, float* __restrict__ y, uint64_t n_units) {
    const uint64_t u = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (u >= n_units) return;
    // Treat the whole tensor as one long row: block addressing only depends on k.
    // Index in two levels so k stays within 32 bits per 2^24-unit chunk.
    constexpr uint64_t kChunkUnits = 1u << 24;  // 2^27 elements, a multiple of every block size
    const uint64_t chunk = u / kChunkUnits;
    const uint32_t k = (uint32_t)(u % kChunkUnits) * 8u;
    const uint64_t chunk_elems = kChunkUnits * 8u;
    const uint8_t* base = blocks + chunk * (chunk_elems / Fmt<TYPE>::kElems) * Fmt<TYPE>::kBytes;
    float w[8];
    dequant8<TYPE>(base, k, w);
    float4* out = reinterpret_cast<float4*>(y + u * 8u);
    out[0] = make_float4(w[0], w[1], w[2], w[3]);
    out[1] = make_float4(w[4], w[5], w[6], w[7]);
}

cudaError_t launch_dequant(const Launch& L, uint32_t type, const void* blocks, float* y, uint64_t n_elems) {
    if (n_elems == 0) return cudaSuccess;
    const uint64_t units = n_elems / 8;
    const unsigned grid = (unsigned)((units + 255) / 256);
    const uint8_t* b = (const uint8_t*)blocks;
    switch (type) {
        case QKM_TYPE_F32: dequant_kernel<QKM_TYPE_F32><<<grid, 256, 0, L.stream>>>(b, y, units); break;
        case QKM_TYPE_F16: dequant_kernel<QKM_TYPE_F16><<<grid, 256, 0, L.stream>>>(b, y, units); break;
        case QKM_TYPE_Q8_0: dequant_kernel<QKM_TYPE_Q8_0><<<grid, 256, 0, L.stream>>>(b, y, units); break;
        case QKM_TYPE_Q6_K: dequant_kernel<QKM_TYPE_Q6_K><<<grid, 256, 0, L.stream>>>(b, y, units); break;
        case QKM_TYPE_IQ4_XS: dequant_kernel<QKM_TYPE_IQ4_XS><<<grid, 256, 0, L.stream>>>(b, y, units); break;
        case QKM_TYPE_IQ3_XXS: dequant_kernel<QKM_TYPE_IQ3_XXS><<<grid, 256, 0, L.stream>>>(b, y, units); break;
        default: return cudaErrorInvalidValue;
    }
    L.count();
    return cudaGetLastError();
}

// ---- GEMV, generic shapes: one warp per (row, input) -----------------------------------
// Any M, any K that is a multiple of the block size (and of 8).  Lanes stride over
// 8-element units; f32 accumulation; one shuffle reduction per row.
template <int TYPE>
__global__ void __launch_bounds__(256)
gemv_warp_kernel(const uint8_t* __restrict__ W, const float* __restrict__ x, float* __restrict__ y,
                 uint32_t M, uint32_t K, size_t rb) {
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
    const uint32_t m = blockIdx.x * 8u + warp;
    const uint32_t t = blockIdx.y;
    if (m >= M) return;
    const uint8_t* row = W + (size_t)m * rb;
    const float* xt = x + (size_t)t * K;
    float acc = 0.f;
    for (uint32_t u = lane; u < K / 8; u += 32) {
        float w[8];
        dequant8<TYPE>(row, u * 8, w);
        const float4 a = *reinterpret_cast<const float4*>(xt + u * 8);
        const float4 b = *reinterpret_cast<const float4*>(xt + u * 8 + 4);
        acc += w[0] * a.x; acc += w[1] * a.y; acc += w[2] * a.z; acc += w[3] * a.w;
        acc += w[4] * b.x; acc += w[5] * b.y; acc += w[6] * b.z; acc += w[7] * b.w;
    }
    acc = warp_sum(acc);
    if (lane == 0) y[(size_t)t * M + m] = acc;
}

cudaError_t launch_gemv_generic(const Launch& L, uint32_t type, const void* W, const float* x, float* y,
                                uint32_t M, uint32_t K, uint32_t n) {
    const dim3 grid((M + 7) / 8, n);
    const uint8_t* w = (const uint8_t*)W;
    const size_t rb = row_bytes(type, K);
    switch (type) {
        case QKM_TYPE_F32: gemv_warp_kernel<QKM_TYPE_F32><<<grid, 256, 0, L.stream>>>(w, x, y, M, K, rb); break;
        case QKM_TYPE_F16: gemv_warp_kernel<QKM_TYPE_F16><<<grid, 256, 0, L.stream>>>(w, x, y, M, K, rb); break;
        case QKM_TYPE_Q8_0: gemv_warp_kernel<QKM_TYPE_Q8_0><<<grid, 256, 0, L.stream>>>(w, x, y, M, K, rb); break;
        case QKM_TYPE_Q6_K: gemv_warp_kernel<QKM_TYPE_Q6_K><<<grid, 256, 0, L.stream>>>(w, x, y, M, K, rb); break;
        case QKM_TYPE_IQ4_XS: gemv_warp_kernel<QKM_TYPE_IQ4_XS><<<grid, 256, 0, L.stream>>>(w, x, y, M, K, rb); break;
        case QKM_TYPE_IQ3_XXS: gemv_warp_kernel<QKM_TYPE_IQ3_XXS><<<grid, 256, 0, L.stream>>>(w, x, y, M, K, rb); break;
        default: return cudaErrorInvalidValue;
    }
    L.count();
    return cudaGetLastError();
}

cudaError_t launch_gemv(const Launch& L, uint32_t type, const void* W, const float* x, float* y,
                        uint32_t M, uint32_t K, uint32_t n) {
    if (M == 0 || n == 0) return cudaSuccess;
    return launch_gemv_generic(L, type, W, x, y, M, K, n);
}

}  // namespace qkm
