// Shared device/host definitions: ggml block geometry, exact dequantisation of
// one 8-element unit of any supported format, warp helpers, launch checks.
//
// "Exact" means the f32 value equals the reference CPU dequantiser's for the
// same bytes (src/quants.h:70-165): the same factors multiplied in the same
// order, with no fused multiply-add involved (only multiplications occur).
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/qk_moe.h"

namespace qkm {

// ---- block geometry (src/quants.h:52-66, :107-119) --------------------------
template <int TYPE> struct Fmt;
template <> struct Fmt<QKM_TYPE_F32>     { static constexpr int kElems = 8,   kBytes = 32;  };
template <> struct Fmt<QKM_TYPE_F16>     { static constexpr int kElems = 8,   kBytes = 16;  };
template <> struct Fmt<QKM_TYPE_Q8_0>    { static constexpr int kElems = 32,  kBytes = 34;  };
template <> struct Fmt<QKM_TYPE_Q6_K>    { static constexpr int kElems = 256, kBytes = 210; };
template <> struct Fmt<QKM_TYPE_IQ4_XS>  { static constexpr int kElems = 256, kBytes = 136; };
template <> struct Fmt<QKM_TYPE_IQ3_XXS> { static constexpr int kElems = 256, kBytes = 98;  };

__host__ __device__ inline size_t row_bytes(uint32_t type, uint64_t ne0) {
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
__host__ __device__ inline uint32_t block_elems(uint32_t type) {
    switch (type) {
        case QKM_TYPE_F32: case QKM_TYPE_F16: return 1;
        case QKM_TYPE_Q8_0: return 32;
        case QKM_TYPE_Q6_K: case QKM_TYPE_IQ4_XS: case QKM_TYPE_IQ3_XXS: return 256;
        default: return 0;
    }
}

// ---- codebooks -----------------------------------------------------------------
// 256-entry IQ3_XXS grid and 16-entry IQ4 value table in constant memory (for the
// simple kernels); the streaming kernels copy them to shared memory.
// (one copy per translation unit: the library is built without relocatable device code)
static __constant__ uint32_t c_iq3_grid[256] = {
#define QKM_G(x) x,
#include "qkm_tables.inc"
};
static __constant__ int8_t c_iq4_values[16] = {-127, -104, -83, -65, -49, -35, -22, -10,
                                               1,    13,   25,  38,  53,  69,  89,  113};
__device__ __forceinline__ float iq4_value(uint32_t nib) {
    return (float)c_iq4_values[nib & 15u];
}

// IQ2/IQ3 sign byte of a 7-bit code: bit 7 is the parity of the low seven
// (shaders/iq_tables.glsl:43; table form at src/quant_tables.h:40-49).
__host__ __device__ __forceinline__ uint32_t signs8(uint32_t s7) {
#ifdef __CUDA_ARCH__
    return s7 | ((__popc(s7) & 1u) << 7);
#else
    return s7 | ((uint32_t)(__builtin_popcount(s7) & 1) << 7);
#endif
}

// ---- unaligned little-endian loads (ggml blocks are only 2-byte aligned) --------
__device__ __forceinline__ uint32_t ld_u16(const uint8_t* p) {
    return *reinterpret_cast<const uint16_t*>(p);
}
__device__ __forceinline__ uint32_t ld_u32_a2(const uint8_t* p) {  // p 2-byte aligned
    return ld_u16(p) | (ld_u16(p + 2) << 16);
}
__device__ __forceinline__ float f16_bits_to_f32(uint32_t h) {
    return __half2float(__ushort_as_half((unsigned short)h));
}

// ---- exact dequantisation of 8 consecutive elements ---------------------------------
// `row` points at the first block of a row, `k` is the element index of the unit's
// first element (multiple of 8).  w[0..7] receive the reference's f32 values.
template <int TYPE>
__device__ __forceinline__ void dequant8(const uint8_t* __restrict__ row, uint32_t k, float* w);

template <>
__device__ __forceinline__ void dequant8<QKM_TYPE_F32>(const uint8_t* __restrict__ row, uint32_t k, float* w) {
    const float4* p = reinterpret_cast<const float4*>(row + (size_t)k * 4);
    const float4 a = p[0], b = p[1];
    w[0] = a.x; w[1] = a.y; w[2] = a.z; w[3] = a.w; w[4] = b.x; w[5] = b.y; w[6] = b.z; w[7] = b.w;
}
template <>
__device__ __forceinline__ void dequant8<QKM_TYPE_F16>(const uint8_t* __restrict__ row, uint32_t k, float* w) {
    const uint4 v = *reinterpret_cast<const uint4*>(row + (size_t)k * 2);
    const uint32_t u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        w[2 * i] = f16_bits_to_f32(u[i] & 0xFFFFu);
        w[2 * i + 1] = f16_bits_to_f32(u[i] >> 16);
    }
}
template <>
__device__ __forceinline__ void dequant8<QKM_TYPE_Q8_0>(const uint8_t* __restrict__ row, uint32_t k, float* w) {
    const uint8_t* b = row + (size_t)(k >> 5) * 34;
    const float d = f16_bits_to_f32(ld_u16(b));
    const uint8_t* q = b + 2 + (k & 31u);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const uint32_t v = ld_u16(q + 2 * i);
        w[2 * i] = d * (float)(int8_t)(v & 0xFF);
        w[2 * i + 1] = d * (float)(int8_t)(v >> 8);
    }
}
template <>
__device__ __forceinline__ void dequant8<QKM_TYPE_Q6_K>(const uint8_t* __restrict__ row, uint32_t k, float* w) {
    const uint8_t* b = row + (size_t)(k >> 8) * 210;   // blocks are 2-byte aligned
    const uint32_t n = k & 255u;          // element within the block
    const uint32_t half = n >> 7;         // which 128-element half
    const uint32_t quad = (n >> 5) & 3u;  // which 32-element quarter of the half
    const uint32_t l = n & 31u;           // multiple of 8
    const uint8_t* ql = b + 64 * half + 32 * (quad & 1u) + l;
    const uint8_t* qh = b + 128 + 32 * half + l;
    const float d = f16_bits_to_f32(ld_u16(b + 208));
    const float sc = (float)(int8_t)b[192 + (n >> 4)];
    const float ds = d * sc;  // (d * sc) * q, left to right as the reference writes it
    const uint32_t nib = (quad >> 1) << 2, hs = 2 * quad;
    // four values at a time: low nibbles (or high, for the upper quarters) and the two high
    // bits are isolated with word-wide masks, then each byte is one 6-bit value
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const uint32_t lo = (ld_u32_a2(ql + 4 * h) >> nib) & 0x0F0F0F0Fu;
        const uint32_t hi = ((ld_u32_a2(qh + 4 * h) >> hs) & 0x03030303u) << 4;
        const uint32_t q = lo | hi;
#pragma unroll
        for (int i = 0; i < 4; ++i) w[4 * h + i] = ds * (float)((int)((q >> (8 * i)) & 0xFFu) - 32);
    }
}
template <>
__device__ __forceinline__ void dequant8<QKM_TYPE_IQ4_XS>(const uint8_t* __restrict__ row, uint32_t k, float* w) {
    const uint8_t* b = row + (size_t)(k >> 8) * 136;
    const uint32_t n = k & 255u;
    const uint32_t ib = n >> 5;   // 32-element sub-block
    const uint32_t e = n & 31u;   // 0, 8, 16 or 24
    const float d = f16_bits_to_f32(ld_u16(b));
    const uint32_t sh = ld_u16(b + 2);
    const uint32_t sl = b[4 + (ib >> 1)];
    const int ls = (int)(((sl >> (4 * (ib & 1u))) & 0xFu) | (((sh >> (2 * ib)) & 3u) << 4));
    const float dl = d * (float)(ls - 32);
    const uint8_t* q = b + 8 + 16 * ib + (e & 15u);
    const bool hi = e >= 16;
#pragma unroll
    for (int i = 0; i < 8; ++i) w[i] = dl * iq4_value(hi ? (q[i] >> 4) : (q[i] & 0xF));
}
template <>
__device__ __forceinline__ void dequant8<QKM_TYPE_IQ3_XXS>(const uint8_t* __restrict__ row, uint32_t k, float* w) {
    const uint8_t* b = row + (size_t)(k >> 8) * 98;
    const uint32_t n = k & 255u;
    const uint32_t ib = n >> 5;        // 32-element sub-block
    const uint32_t l = (n >> 3) & 3u;  // 8-element group within it
    const float d = f16_bits_to_f32(ld_u16(b));
    const uint32_t aux = ld_u32_a2(b + 2 + 64 + 4 * ib);
    const float db = d * (0.5f + (float)(aux >> 28)) * 0.5f;
    const uint32_t sg = signs8((aux >> (7 * l)) & 127u);
    const uint32_t idx = ld_u16(b + 2 + 8 * ib + 2 * l);
    const uint32_t g1 = c_iq3_grid[idx & 0xFF], g2 = c_iq3_grid[idx >> 8];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        w[j] = db * (float)((g1 >> (8 * j)) & 255u) * (((sg >> j) & 1u) ? -1.f : 1.f);
        w[j + 4] = db * (float)((g2 >> (8 * j)) & 255u) * (((sg >> (j + 4)) & 1u) ? -1.f : 1.f);
    }
}

// ---- warp helpers ----------------------------------------------------------------------
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, o);
    return v;
}
__device__ __forceinline__ double warp_sum(double v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, o);
    return v;
}
// silu(g) * u in f32, written as the reference shader does (moe_gateup_iq3.comp:105)
__device__ __forceinline__ float swiglu(float g, float u) { return (g / (1.0f + expf(-g))) * u; }

}  // namespace qkm
