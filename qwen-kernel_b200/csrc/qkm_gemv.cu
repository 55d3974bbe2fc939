// Dense dequant-GEMV and the dequantisation probe.
//
// Replaces the reference's gemv_{f16,q8_0,q6_k,iq4_xs,iq3_xxs}.comp
// (y[M] = W[M,K] . x[K] on raw ggml blocks, z-batched over n inputs,
// shaders/gemv_q8_0.comp:31-32) and exposes dequant_row_* (src/quants.h:70-165)
// on the GPU so dequantised weights can be compared bit-for-bit.
#include "qkm_common.cuh"
#include "qkm_kernels.h"
#include "qkm_stream.cuh"

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
                 uint32_t M, uint32_t K, size_t rb, uint32_t y_stride) {
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
    if (lane == 0) y[(size_t)t * y_stride + m] = acc;
}

cudaError_t launch_gemv_tail(const Launch& L, uint32_t type, const void* W, const float* x, float* y,
                             uint32_t M, uint32_t K, uint32_t n, uint32_t y_stride) {
    const dim3 grid((M + 7) / 8, n);
    const uint8_t* w = (const uint8_t*)W;
    const size_t rb = row_bytes(type, K);
    switch (type) {
        case QKM_TYPE_F32: gemv_warp_kernel<QKM_TYPE_F32><<<grid, 256, 0, L.stream>>>(w, x, y, M, K, rb, y_stride); break;
        case QKM_TYPE_F16: gemv_warp_kernel<QKM_TYPE_F16><<<grid, 256, 0, L.stream>>>(w, x, y, M, K, rb, y_stride); break;
        case QKM_TYPE_Q8_0: gemv_warp_kernel<QKM_TYPE_Q8_0><<<grid, 256, 0, L.stream>>>(w, x, y, M, K, rb, y_stride); break;
        case QKM_TYPE_Q6_K: gemv_warp_kernel<QKM_TYPE_Q6_K><<<grid, 256, 0, L.stream>>>(w, x, y, M, K, rb, y_stride); break;
        case QKM_TYPE_IQ4_XS: gemv_warp_kernel<QKM_TYPE_IQ4_XS><<<grid, 256, 0, L.stream>>>(w, x, y, M, K, rb, y_stride); break;
        case QKM_TYPE_IQ3_XXS: gemv_warp_kernel<QKM_TYPE_IQ3_XXS><<<grid, 256, 0, L.stream>>>(w, x, y, M, K, rb, y_stride); break;
        default: return cudaErrorInvalidValue;
    }
    L.count();
    return cudaGetLastError();
}

cudaError_t launch_gemv_tail(const Launch& L, uint32_t type, const void* W, const float* x, float* y,
                             uint32_t M, uint32_t K, uint32_t n, uint32_t y_stride);

// ---- GEMV, streamed: persistent blocks, rows staged through shared memory by bulk copies ------
// Rows of a ggml tensor follow each other without padding, so a tile of R rows is one
// contiguous byte range; with R a multiple of 8 it starts and ends on 16-byte boundaries
// and one bulk copy (TMA) brings it into shared memory while the previous tile is being
// consumed.  Each warp then takes rows of the tile: lanes stride over 8-element units,
// decode them from shared memory (where the 2-byte alignment of ggml blocks costs nothing)
// and multiply with x held in shared memory; f32 accumulation, one shuffle tree per row.
namespace gv {
constexpr int kWarps = 8;
constexpr int kStages = 3;
constexpr int kStageBytes = 24 * 1024;
}  // namespace gv

template <int TYPE>
__global__ void __launch_bounds__(gv::kWarps * 32)
gemv_stream_kernel(const uint8_t* __restrict__ W, const float* __restrict__ x, float* __restrict__ y,
                   uint32_t M, uint32_t K, uint32_t n, uint32_t rows_per_tile, uint32_t* __restrict__ status) {
    extern __shared__ __align__(128) uint8_t smem_raw[];
    __shared__ __align__(8) unsigned long long s_bar[gv::kStages];
    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31u;
    const size_t rb = row_bytes(TYPE, K);
    float* s_x = reinterpret_cast<float*>(smem_raw);                 // n * K floats
    const uint32_t ring = smem_addr(smem_raw) + n * K * 4;           // kStages * kStageBytes
    uint8_t* ring_ptr = smem_raw + (size_t)n * K * 4;
    const uint32_t n_tiles = M / rows_per_tile;                      // whole tiles only; the caller handles the tail
    for (uint32_t i = tid; i < n * K; i += blockDim.x) s_x[i] = x[i];
    if (tid == 0) {
        for (int s = 0; s < gv::kStages; ++s) mbar_init(smem_addr(&s_bar[s]), 1);
        mbar_fence_init();
    }
    __syncthreads();
    const uint32_t tile_bytes_ = (uint32_t)(rows_per_tile * rb);
    uint32_t p_tile = blockIdx.x;
    auto issue = [&](uint32_t stage) {
        if (p_tile >= n_tiles) return;
        const uint32_t bar = smem_addr(&s_bar[stage]);
        mbar_expect_tx(bar, tile_bytes_);
        bulk_g2s(ring + stage * gv::kStageBytes, W + (size_t)p_tile * tile_bytes_, tile_bytes_, bar);
        p_tile += gridDim.x;
    };
    if (tid == 0)
        for (int s = 0; s < gv::kStages; ++s) issue(s);
    bool timed_out = false;
    uint32_t cnt = 0;
    for (uint32_t tile = blockIdx.x; tile < n_tiles; tile += gridDim.x, ++cnt) {
        const uint32_t stage = cnt % gv::kStages, parity = (cnt / gv::kStages) & 1u;
        if (!mbar_wait_bounded(smem_addr(&s_bar[stage]), parity)) timed_out = true;
        const uint8_t* tb = ring_ptr + (size_t)stage * gv::kStageBytes;
        for (uint32_t r = warp; r < rows_per_tile; r += gv::kWarps) {
            const uint8_t* row = tb + (size_t)r * rb;
            for (uint32_t t = 0; t < n; ++t) {
                const float* xt = s_x + (size_t)t * K;
                float acc = 0.f;
#pragma unroll 2
                for (uint32_t u = lane; u < K / 8; u += 32) {
                    float w[8];
                    dequant8<TYPE>(row, u * 8, w);
                    const float4 a = *reinterpret_cast<const float4*>(xt + u * 8);
                    const float4 b = *reinterpret_cast<const float4*>(xt + u * 8 + 4);
                    acc += w[0] * a.x; acc += w[1] * a.y; acc += w[2] * a.z; acc += w[3] * a.w;
                    acc += w[4] * b.x; acc += w[5] * b.y; acc += w[6] * b.z; acc += w[7] * b.w;
                }
                acc = warp_sum(acc);
                if (lane == 0) y[(size_t)t * M + (size_t)tile * rows_per_tile + r] = acc;
            }
        }
        __syncthreads();   // every warp is done with this stage
        if (tid == 0) issue(stage);
    }
    if (timed_out && tid == 0) atomicExch(status, (uint32_t)kStatusWaitTimeout);
}

template <int TYPE>
static cudaError_t gemv_stream_launch(const Launch& L, const uint8_t* W, const float* x, float* y, uint32_t M,
                                      uint32_t K, uint32_t n, uint32_t n_sms, uint32_t* status, uint32_t* rows_done) {
    const size_t rb = row_bytes(TYPE, K);
    uint32_t rows_per_tile = (uint32_t)(gv::kStageBytes / rb) & ~7u;
    *rows_done = 0;
    if (rows_per_tile == 0 || ((uintptr_t)W & 15u) || (size_t)n * K * 4 > 64 * 1024) return cudaSuccess;
    if (rows_per_tile > 64) rows_per_tile = 64;
    const uint32_t n_tiles = M / rows_per_tile;
    if (n_tiles == 0) return cudaSuccess;
    const size_t smem = (size_t)n * K * 4 + (size_t)gv::kStages * gv::kStageBytes;
    cudaError_t e = cudaFuncSetAttribute(gemv_stream_kernel<TYPE>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    const uint32_t blocks = n_tiles < 2 * n_sms ? n_tiles : 2 * n_sms;
    gemv_stream_kernel<TYPE><<<blocks, gv::kWarps * 32, smem, L.stream>>>(W, x, y, M, K, n, rows_per_tile, status);
    L.count();
    *rows_done = n_tiles * rows_per_tile;
    return cudaGetLastError();
}

cudaError_t launch_gemv_stream(const Launch& L, uint32_t type, const void* W, const float* x, float* y,
                               uint32_t M, uint32_t K, uint32_t n, uint32_t n_sms, uint32_t* status) {
    if (M == 0 || n == 0) return cudaSuccess;
    const uint8_t* w = (const uint8_t*)W;
    uint32_t done = 0;
    cudaError_t e;
    switch (type) {
        case QKM_TYPE_F32: e = gemv_stream_launch<QKM_TYPE_F32>(L, w, x, y, M, K, n, n_sms, status, &done); break;
        case QKM_TYPE_F16: e = gemv_stream_launch<QKM_TYPE_F16>(L, w, x, y, M, K, n, n_sms, status, &done); break;
        case QKM_TYPE_Q8_0: e = gemv_stream_launch<QKM_TYPE_Q8_0>(L, w, x, y, M, K, n, n_sms, status, &done); break;
        case QKM_TYPE_Q6_K: e = gemv_stream_launch<QKM_TYPE_Q6_K>(L, w, x, y, M, K, n, n_sms, status, &done); break;
        case QKM_TYPE_IQ4_XS: e = gemv_stream_launch<QKM_TYPE_IQ4_XS>(L, w, x, y, M, K, n, n_sms, status, &done); break;
        case QKM_TYPE_IQ3_XXS: e = gemv_stream_launch<QKM_TYPE_IQ3_XXS>(L, w, x, y, M, K, n, n_sms, status, &done); break;
        default: return cudaErrorInvalidValue;
    }
    if (e != cudaSuccess) return e;
    if (done < M) {  // tail rows (and shapes the streamed form does not take): one warp per row
        // y is [n][M]: the generic kernel indexes rows from its own origin, so it gets shifted
        // pointers and the full row stride through launch_gemv_tail
        return launch_gemv_tail(L, type, w + (size_t)done * row_bytes(type, K), x, y + done, M - done, K, n, M);
    }
    return cudaSuccess;
}

cudaError_t launch_gemv(const Launch& L, uint32_t type, const void* W, const float* x, float* y,
                        uint32_t M, uint32_t K, uint32_t n) {
    if (M == 0 || n == 0) return cudaSuccess;
    return launch_gemv_tail(L, type, W, x, y, M, K, n, M);
}

}  // namespace qkm
