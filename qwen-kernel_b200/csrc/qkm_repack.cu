// Upload-time re-ordering of raw ggml tensors into the tile layout the streaming
// kernels read (see qkm_tiles.cuh).  Pure byte permutation: every output byte is a
// copy of one input byte, so dequantised values are unchanged and the byte count of
// a tensor stays what a GGUF file holds for it.
#include "qkm_common.cuh"
#include "qkm_kernels.h"
#include "qkm_tiles.cuh"

namespace qkm {

// One thread per output byte.  n_mats matrices of [rows][K] follow each other in both
// layouts (experts of a stacked tensor); rows % 16 == 0 and K % 256 == 0.
template <int TYPE>
__global__ void repack_kernel(const uint8_t* __restrict__ raw, uint8_t* __restrict__ out, uint32_t rows,
                              uint32_t K, uint64_t total_bytes) {
    constexpr int kTile = TYPE == QKM_TYPE_IQ3_XXS ? kTileIq3 : TYPE == QKM_TYPE_IQ4_XS ? kTileIq4 : TYPE == QKM_TYPE_Q6_K ? kTileQ6 : kTileQ8;
    const uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total_bytes) return;
    const uint32_t KB = K / 256, RT = rows / 16;
    const uint64_t tile = i / kTile;
    const uint32_t o = (uint32_t)(i - tile * kTile);
    const uint64_t mat = tile / ((uint64_t)KB * RT);
    const uint32_t tin = (uint32_t)(tile - mat * KB * RT);
    const uint32_t kb = tin / RT, rt = tin - kb * RT;
    const size_t rb = row_bytes(TYPE, K);
    const uint8_t* m = raw + mat * rows * rb;
    uint32_t row_in_tile, off;  // source: row (0..15) and byte offset inside that row's 256-column span
    if (TYPE == QKM_TYPE_IQ3_XXS) {
        if (o < 1024) {
            const uint32_t h = o >> 9, lane = (o >> 4) & 31u, b = o & 15u;
            const uint32_t g = lane >> 2, t = lane & 3u;
            const uint32_t ib = 2 * ((b & 7u) >> 1) + (b >> 3);   // even sub-blocks first, then the odd ones
            row_in_tile = g + 8 * h;
            off = 2 + 8 * ib + 2 * t + (b & 1u);
        } else if (o < 1536) {   // aux words: [parity of the sub-block][row][4 words]
            const uint32_t q = o - 1024;
            const uint32_t ib = 2 * ((q & 15u) >> 2) + (q >> 8);
            row_in_tile = (q >> 4) & 15u;
            off = 2 + 64 + 4 * ib + (q & 3u);
        } else {
            row_in_tile = (o - 1536) >> 1;
            off = (o - 1536) & 1u;
        }
        out[i] = m[(size_t)(rt * 16 + row_in_tile) * rb + (size_t)kb * 98 + off];
    } else if (TYPE == QKM_TYPE_IQ4_XS) {
        if (o < 128) {
            const uint32_t g = o >> 4, h = (o >> 3) & 1u;
            row_in_tile = g + 8 * h;
            off = o & 7u;
        } else {
            const uint32_t q = o - 128, c = q >> 9, lane = (q >> 4) & 31u, b = q & 15u;
            const uint32_t g = lane >> 2, t = lane & 3u;
            row_in_tile = g + 8 * (c >> 1);
            const uint32_t ib = 4 * (c & 1u) + (b >> 2);
            off = 8 + 16 * ib + 4 * t + (b & 3u);
        }
        out[i] = m[(size_t)(rt * 16 + row_in_tile) * rb + (size_t)kb * 136 + off];
    } else if (TYPE == QKM_TYPE_Q6_K) {
        if (o < 256) {
            const uint32_t b = o & 15u;
            row_in_tile = o >> 4;
            off = 192 + (b < 8 ? 2 * b : 2 * (b - 8) + 1);
        } else if (o < 3328) {
            const uint32_t q = o - 256, c = q >> 9, lane = (q >> 4) & 31u, b = q & 15u;
            const uint32_t g = lane >> 2, t = lane & 3u, h = c / 3, k = c - 3 * h, w = b >> 2;
            const uint32_t wm = (w & 1u) ? 4 + t : t;
            row_in_tile = g + 8 * h;
            off = k < 2 ? 64 * k + 32 * (w >> 1) + 4 * wm + (b & 3u) : 128 + 32 * (w >> 1) + 4 * wm + (b & 3u);
        } else {
            row_in_tile = (o - 3328) >> 1;
            off = 208 + (o & 1u);
        }
        out[i] = m[(size_t)(rt * 16 + row_in_tile) * rb + (size_t)kb * 210 + off];
    } else {  // Q8_0: per 32-column block, the 16 rows' d (32 B) then their quants (512 B)
        const uint32_t blk = o / 544u, q = o - blk * 544u;
        if (q < 32) {
            row_in_tile = q >> 1;
            off = q & 1u;
        } else {
            const uint32_t v = q - 32, h = (v >> 8) & 1u, lane = (v >> 3) & 31u, b = v & 7u;
            const uint32_t g = lane >> 2, t = lane & 3u;
            row_in_tile = g + 8 * h;
            off = 2 + (b < 4 ? 4 * t + b : 16 + 4 * t + (b - 4));
        }
        out[i] = m[(size_t)(rt * 16 + row_in_tile) * rb + (size_t)(kb * 8 + blk) * 34 + off];
    }
}

cudaError_t launch_repack(const Launch& L, uint32_t type, const void* raw, void* out, uint32_t n_mats,
                          uint32_t rows, uint32_t K) {
    if (rows % 16 || K % 256) return cudaErrorInvalidValue;
    const uint64_t total = (uint64_t)n_mats * rows * row_bytes(type, K);
    if (total == 0) return cudaSuccess;
    const unsigned grid = (unsigned)((total + 255) / 256);
    const uint8_t* r = (const uint8_t*)raw;
    uint8_t* o = (uint8_t*)out;
    switch (type) {
        case QKM_TYPE_IQ3_XXS: repack_kernel<QKM_TYPE_IQ3_XXS><<<grid, 256, 0, L.stream>>>(r, o, rows, K, total); break;
        case QKM_TYPE_IQ4_XS: repack_kernel<QKM_TYPE_IQ4_XS><<<grid, 256, 0, L.stream>>>(r, o, rows, K, total); break;
        case QKM_TYPE_Q6_K: repack_kernel<QKM_TYPE_Q6_K><<<grid, 256, 0, L.stream>>>(r, o, rows, K, total); break;
        case QKM_TYPE_Q8_0: repack_kernel<QKM_TYPE_Q8_0><<<grid, 256, 0, L.stream>>>(r, o, rows, K, total); break;
        default: return cudaErrorInvalidValue;
    }
    L.count();
    return cudaGetLastError();
}

}  // namespace qkm
