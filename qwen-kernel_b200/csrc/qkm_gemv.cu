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
constexpr size_t kDirectMaxBytes = 48u << 20;   // above this the persistent, staged kernel wins

namespace gv {
constexpr int kWarps = 8;
constexpr int kStages = 3;
constexpr int kStageBytes = 36 * 1024;

// Codebooks in shared memory: lanes of a warp look up different entries, which constant
// memory would serve one lane at a time.
struct Luts {
    uint32_t grid[256];   // IQ3_XXS: four magnitudes per entry
    float iq4[16];        // IQ4_XS / IQ4_NL values
};

// Eight consecutive weights of a row held in shared memory, as f32 (same values as dequant8).
template <int TYPE>
__device__ __forceinline__ void unit8(const uint8_t* __restrict__ row, uint32_t k, float* w, const Luts& lut) {
    dequant8<TYPE>(row, k, w);
}
template <>
__device__ __forceinline__ void unit8<QKM_TYPE_IQ4_XS>(const uint8_t* __restrict__ row, uint32_t k, float* w, const Luts& lut) {
    const uint8_t* b = row + (size_t)(k >> 8) * 136;   // blocks are 8-byte aligned (136 = 8 * 17)
    const uint32_t n = k & 255u, ib = n >> 5, e = n & 31u;
    const uint32_t hdr = *reinterpret_cast<const uint32_t*>(b);           // d (f16) | scales_h
    const float d = f16_bits_to_f32(hdr & 0xFFFFu);
    const uint32_t sh = hdr >> 16;
    const uint32_t sl = b[4 + (ib >> 1)];
    const int ls = (int)(((sl >> (4 * (ib & 1u))) & 0xFu) | (((sh >> (2 * ib)) & 3u) << 4));
    const float dl = d * (float)(ls - 32);
    const uint2 q = *reinterpret_cast<const uint2*>(b + 8 + 16 * ib + (e & 15u));
    const uint32_t sft = (e >> 4) << 2;                 // 0: low nibbles, 4: high nibbles
    const uint32_t q0 = q.x >> sft, q1 = q.y >> sft;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        w[i] = dl * lut.iq4[(q0 >> (8 * i)) & 0xFu];
        w[i + 4] = dl * lut.iq4[(q1 >> (8 * i)) & 0xFu];
    }
}
template <>
__device__ __forceinline__ void unit8<QKM_TYPE_IQ3_XXS>(const uint8_t* __restrict__ row, uint32_t k, float* w, const Luts& lut) {
    const uint8_t* b = row + (size_t)(k >> 8) * 98;
    const uint32_t n = k & 255u, ib = n >> 5, l = (n >> 3) & 3u;
    const float d = f16_bits_to_f32(ld_u16(b));
    const uint32_t aux = ld_u32_a2(b + 2 + 64 + 4 * ib);
    const float db = d * (0.5f + (float)(aux >> 28)) * 0.5f;
    const uint32_t sg = signs8((aux >> (7 * l)) & 127u);
    const uint32_t idx = ld_u16(b + 2 + 8 * ib + 2 * l);
    const uint32_t g1 = lut.grid[idx & 0xFF], g2 = lut.grid[idx >> 8];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const float a = db * (float)((g1 >> (8 * j)) & 255u), c = db * (float)((g2 >> (8 * j)) & 255u);
        w[j] = __uint_as_float(__float_as_uint(a) ^ ((sg << (31 - j)) & 0x80000000u));
        w[j + 4] = __uint_as_float(__float_as_uint(c) ^ ((sg << (27 - j)) & 0x80000000u));
    }
}
}  // namespace gv

// XREG: K == 2048 and one activation row - a lane always meets the same eight 8-column units, so
// it keeps its 64 activation values in registers and shared memory carries weight bytes only.
template <int TYPE, bool XREG>
__global__ void __launch_bounds__(gv::kWarps * 32)
gemv_stream_kernel(const uint8_t* __restrict__ W, const float* __restrict__ x, float* __restrict__ y,
                   uint32_t M, uint32_t K, uint32_t n, uint32_t rows_per_tile, uint32_t stage_bytes,
                   uint32_t* __restrict__ status) {
    extern __shared__ __align__(128) uint8_t smem_raw[];
    __shared__ __align__(8) unsigned long long s_bar[gv::kStages];
    __shared__ gv::Luts s_lut;
    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31u;
    const size_t rb = row_bytes(TYPE, K);
    float* s_x = reinterpret_cast<float*>(smem_raw);                 // n * K floats
    const uint32_t ring = smem_addr(smem_raw) + n * K * 4;           // kStages * kStageBytes
    uint8_t* ring_ptr = smem_raw + (size_t)n * K * 4;
    const uint32_t n_tiles = M / rows_per_tile;                      // whole tiles only; the caller handles the tail
    const uint32_t tile_bytes_ = (uint32_t)(rows_per_tile * rb);
    uint32_t p_tile = blockIdx.x;
    auto issue = [&](uint32_t stage) {
        if (p_tile >= n_tiles) return;
        const uint32_t bar = smem_addr(&s_bar[stage]);
        mbar_expect_tx(bar, tile_bytes_);
        bulk_g2s(ring + stage * stage_bytes, W + (size_t)p_tile * tile_bytes_, tile_bytes_, bar);
        p_tile += gridDim.x;
    };
    if (tid == 0) {   // the first tiles are on their way while x and the codebooks are staged
        for (int s = 0; s < gv::kStages; ++s) mbar_init(smem_addr(&s_bar[s]), 1);
        mbar_fence_init();
        for (int s = 0; s < gv::kStages; ++s) issue(s);
    }
    for (uint32_t i = tid; i < n * K / 4; i += blockDim.x)
        reinterpret_cast<float4*>(s_x)[i] = reinterpret_cast<const float4*>(x)[i];
    if (TYPE == QKM_TYPE_IQ3_XXS) s_lut.grid[tid] = c_iq3_grid[tid];
    if (TYPE == QKM_TYPE_IQ4_XS && tid < 16) s_lut.iq4[tid] = (float)c_iq4_values[tid];
    __syncthreads();
    bool timed_out = false;
    uint32_t cnt = 0;
    float4 xr[XREG ? 16 : 1];
    if (XREG) {
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            xr[2 * i] = *reinterpret_cast<const float4*>(s_x + (lane + 32 * i) * 8);
            xr[2 * i + 1] = *reinterpret_cast<const float4*>(s_x + (lane + 32 * i) * 8 + 4);
        }
    }
    for (uint32_t tile = blockIdx.x; tile < n_tiles; tile += gridDim.x, ++cnt) {
        const uint32_t stage = cnt % gv::kStages, parity = (cnt / gv::kStages) & 1u;
        if (!mbar_wait_bounded(smem_addr(&s_bar[stage]), parity)) timed_out = true;
        const uint8_t* tb = ring_ptr + (size_t)stage * stage_bytes;
        for (uint32_t r = warp; r < rows_per_tile; r += gv::kWarps) {
            const uint8_t* row = tb + (size_t)r * rb;
            if (XREG) {
                float acc0 = 0.f, acc1 = 0.f;
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    float w[8];
                    gv::unit8<TYPE>(row, (lane + 32 * i) * 8, w, s_lut);
                    const float4 a = xr[2 * i], b = xr[2 * i + 1];
                    acc0 += w[0] * a.x; acc1 += w[1] * a.y; acc0 += w[2] * a.z; acc1 += w[3] * a.w;
                    acc0 += w[4] * b.x; acc1 += w[5] * b.y; acc0 += w[6] * b.z; acc1 += w[7] * b.w;
                }
                const float acc = warp_sum(acc0 + acc1);
                if (lane == 0) y[(size_t)tile * rows_per_tile + r] = acc;
                continue;
            }
            for (uint32_t t = 0; t < n; ++t) {
                const float* xt = s_x + (size_t)t * K;
                float acc0 = 0.f, acc1 = 0.f;
#pragma unroll 2
                for (uint32_t u = lane; u < K / 8; u += 32) {
                    float w[8];
                    gv::unit8<TYPE>(row, u * 8, w, s_lut);
                    const float4 a = *reinterpret_cast<const float4*>(xt + u * 8);
                    const float4 b = *reinterpret_cast<const float4*>(xt + u * 8 + 4);
                    acc0 += w[0] * a.x; acc1 += w[1] * a.y; acc0 += w[2] * a.z; acc1 += w[3] * a.w;
                    acc0 += w[4] * b.x; acc1 += w[5] * b.y; acc0 += w[6] * b.z; acc1 += w[7] * b.w;
                }
                const float acc = warp_sum(acc0 + acc1);
                if (lane == 0) y[(size_t)t * M + (size_t)tile * rows_per_tile + r] = acc;
            }
        }
        __syncthreads();   // every warp is done with this stage
        if (tid == 0) issue(stage);
    }
    if (timed_out && tid == 0) atomicExch(status, (uint32_t)kStatusWaitTimeout);
}

// ---- GEMV, direct: small matrices, one launch of M/8 blocks, one row per warp ---------------------
// For a matrix of a few megabytes the whole read fits in one wave of loads: every warp
// reads its row straight from global memory (all of its loads in flight at once) and x
// through L1; nothing is staged, so the kernel's duration is one memory round trip plus the
// decode of one row.
template <int TYPE>
__global__ void __launch_bounds__(256)
gemv_direct_kernel(const uint8_t* __restrict__ W, const float* __restrict__ x, float* __restrict__ y,
                   uint32_t M, uint32_t K, uint32_t split) {   // split = warps per row: 1, 2, 4 or 8
    __shared__ gv::Luts s_lut;
    __shared__ float s_part[8];
    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31u;
    if (TYPE == QKM_TYPE_IQ3_XXS) s_lut.grid[tid] = c_iq3_grid[tid];
    if (TYPE == QKM_TYPE_IQ4_XS && tid < 16) s_lut.iq4[tid] = (float)c_iq4_values[tid];
    if (TYPE == QKM_TYPE_IQ3_XXS || TYPE == QKM_TYPE_IQ4_XS) __syncthreads();
    const uint32_t rows_per_block = 8 / split;
    const uint32_t r = blockIdx.x * rows_per_block + warp / split, part = warp % split;
    float acc0 = 0.f, acc1 = 0.f;
    if (r < M) {
        const uint8_t* row = W + (size_t)r * row_bytes(TYPE, K);
        const uint32_t units = K / 8 / split;        // this warp's share of the row, contiguous
#pragma unroll 4
        for (uint32_t i = lane; i < units; i += 32) {
            const uint32_t u = part * units + i;
            float w[8];
            gv::unit8<TYPE>(row, u * 8, w, s_lut);
            const float4 a = __ldg(reinterpret_cast<const float4*>(x + u * 8));
            const float4 b = __ldg(reinterpret_cast<const float4*>(x + u * 8 + 4));
            acc0 += w[0] * a.x; acc1 += w[1] * a.y; acc0 += w[2] * a.z; acc1 += w[3] * a.w;
            acc0 += w[4] * b.x; acc1 += w[5] * b.y; acc0 += w[6] * b.z; acc1 += w[7] * b.w;
        }
    }
    const float acc = warp_sum(acc0 + acc1);
    if (split == 1) {
        if (lane == 0 && r < M) y[r] = acc;
        return;
    }
    if (lane == 0) s_part[warp] = acc;
    __syncthreads();
    if (part == 0 && lane == 0 && r < M) {
        float v = 0.f;
        for (uint32_t p = 0; p < split; ++p) v += s_part[warp + p];
        y[r] = v;
    }
}

template <int TYPE>
static cudaError_t gemv_direct_launch(const Launch& L, const uint8_t* W, const float* x, float* y, uint32_t M, uint32_t K) {
    // one wave: as many warps as the machine holds at once (148 SMs x 64 warps), a row shared by
    // up to eight warps when there are few rows
    uint32_t split = 1;
    while (split < 8 && (uint64_t)M * split * 2 <= 148u * 64u && (K / 8) % (split * 2 * 32) == 0) split *= 2;
    const uint32_t rows_per_block = 8 / split;
    gemv_direct_kernel<TYPE><<<(M + rows_per_block - 1) / rows_per_block, 256, 0, L.stream>>>(W, x, y, M, K, split);
    L.count();
    return cudaGetLastError();
}

template <int TYPE>
static cudaError_t gemv_stream_launch(const Launch& L, const uint8_t* W, const float* x, float* y, uint32_t M,
                                      uint32_t K, uint32_t n, uint32_t n_sms, uint32_t* status, uint32_t* rows_done) {
    const size_t rb = row_bytes(TYPE, K);
    *rows_done = 0;
    // a tile must start and end on 16-byte boundaries: whole multiples of `gran` rows
    uint32_t gran = 1;
    while ((gran * rb) % 16) gran *= 2;
    // whole rounds of the eight warps, about 20 KB per stage so that three blocks share an SM;
    // wide rows take one round per tile even when that is more
    uint32_t round = gran > 8 ? gran : 8;
    if ((size_t)round * rb > gv::kStageBytes) round = gran;          // very wide rows: fewer than eight per tile
    if (((uintptr_t)W & 15u) || ((uintptr_t)x & 15u) || (size_t)n * K * 4 > 64 * 1024 || (size_t)round * rb > gv::kStageBytes)
        return cudaSuccess;
    uint32_t rows_per_tile = (uint32_t)(20 * 1024 / rb) / round * round;
    if (rows_per_tile < round) rows_per_tile = round;
    if (rows_per_tile > 64) rows_per_tile = 64 / round * round;
    (void)n_sms;
    const uint32_t n_tiles = M / rows_per_tile;
    if (n_tiles == 0) return cudaSuccess;
    const uint32_t stage_bytes = (uint32_t)((rows_per_tile * rb + 127) / 128 * 128);
    const size_t smem = (size_t)n * K * 4 + (size_t)gv::kStages * stage_bytes;
    const bool xreg = K == 2048 && n == 1;
    cudaError_t e = xreg ? cudaFuncSetAttribute(gemv_stream_kernel<TYPE, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)
                         : cudaFuncSetAttribute(gemv_stream_kernel<TYPE, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    uint32_t per_sm = smem <= 72 * 1024 ? 3u : (smem <= 110 * 1024 ? 2u : 1u);
    if (xreg && per_sm > 2) per_sm = 2;   // about 100 registers per thread: two blocks fit
    const uint32_t blocks = n_tiles < per_sm * n_sms ? n_tiles : per_sm * n_sms;
    if (xreg)
        gemv_stream_kernel<TYPE, true><<<blocks, gv::kWarps * 32, smem, L.stream>>>(W, x, y, M, K, n, rows_per_tile, stage_bytes, status);
    else
        gemv_stream_kernel<TYPE, false><<<blocks, gv::kWarps * 32, smem, L.stream>>>(W, x, y, M, K, n, rows_per_tile, stage_bytes, status);
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
    const bool aligned = !((uintptr_t)W & 15u) && !((uintptr_t)x & 15u) && (type != QKM_TYPE_IQ4_XS || K % 256 == 0);
    // (the integer tensor-core kernels win from about 8192 rows on for the two formats whose unpacking is costly)
    const bool try_mma_small = M >= 8192 && (type == QKM_TYPE_Q6_K || type == QKM_TYPE_IQ4_XS);
    if (n == 1 && aligned && (size_t)M * row_bytes(type, K) <= kDirectMaxBytes && type != QKM_TYPE_F32 && !try_mma_small) {
        switch (type) {
            case QKM_TYPE_F16: return gemv_direct_launch<QKM_TYPE_F16>(L, w, x, y, M, K);
            case QKM_TYPE_Q8_0: return gemv_direct_launch<QKM_TYPE_Q8_0>(L, w, x, y, M, K);
            case QKM_TYPE_Q6_K: return gemv_direct_launch<QKM_TYPE_Q6_K>(L, w, x, y, M, K);
            case QKM_TYPE_IQ4_XS: return gemv_direct_launch<QKM_TYPE_IQ4_XS>(L, w, x, y, M, K);
            case QKM_TYPE_IQ3_XXS: return gemv_direct_launch<QKM_TYPE_IQ3_XXS>(L, w, x, y, M, K);
            default: return cudaErrorInvalidValue;
        }
    }
    if (n == 1 && aligned) {   // large matrices in the formats the integer tensor-core form takes
        e = launch_gemv_mma(L, type, w, x, y, M, K, n_sms, status, &done);
        if (e != cudaSuccess) return e;
        if (done == M) return cudaSuccess;
        if (done) return launch_gemv_tail(L, type, w + (size_t)done * row_bytes(type, K), x, y + done, M - done, K, n, M);
    }
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
