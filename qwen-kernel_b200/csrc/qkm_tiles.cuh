// Device-resident weight layout of the streaming kernels ("tiles") and the
// activation encoding they consume ("digit planes").
//
// TILES.  qkm_upload_layer keeps the raw ggml tensors and additionally stores a
// re-ordered copy: the same bytes, grouped so that one warp can fetch everything it
// needs for 16 rows x 256 columns with one bulk copy and read it back from shared
// memory with aligned, conflict-free 128-bit loads.  A tile holds exactly the bytes
// of its 16 row-blocks (no padding, nothing recomputed), so tile bytes = 16 x
// block bytes x (256 / block elements): IQ3_XXS 1568, IQ4_XS 2176, Q6_K 3360, Q8_0 4352.
// Tiles of one matrix [rows][K] are ordered [kb = K/256][rt = rows/16]: a warp that
// owns column block kb walks consecutive memory as it moves down the rows.
//
// Inside a tile, "lane" is the MMA lane 4*g + t (g = 0..7 row group, t = 0..3):
// lane (g,t) works on rows g and g+8 of the tile.
//
//   IQ3_XXS (block: d f16 | qs[64] grid indices | 8 aux words, src/quants.h:115-119)
//     [   0,1024)  index pairs: half h (row g + 8h), lane -> 16 B = for each of the 8
//                  sub-blocks the two grid indices of 8-element group t
//                  (raw qs[8*ib + 2*t], qs[8*ib + 2*t + 1]), the even sub-blocks 0,2,4,6 in
//                  the first 8 bytes and the odd ones in the last 8 (a prefill thread owns one
//                  32-column half of every 64-column k-step: one 8-byte load); address
//                  h*512 + lane*16
//     [1024,1536)  aux words (4 x 7 sign bits + 4 scale bits each), unchanged, as two halves:
//                  the words of sub-blocks par, 2+par, 4+par, 6+par of row r at
//                  1024 + 256*par + 16*r, so the 16-byte loads of eight rows g (or g+8) hit
//                  eight consecutive 16-byte slots
//     [1536,1568)  d[16] f16
//   IQ4_XS (block: d f16 | scales_h u16 | scales_l[4] | qs[128], src/quants.h:107-113)
//     [   0, 128)  headers: for g: 8 B of row g then 8 B of row g+8, each the raw first
//                  8 bytes of the block (d, scales_h, scales_l)
//     [ 128,2176)  quants: chunk c (0..3), lane -> 16 B at 128 + (c*32 + lane)*16;
//                  c = 2*h + q: row g + 8h, sub-blocks 4q..4q+3, for each the raw qs word t
//                  (bytes 4t..4t+3 of the sub-block's 16: low nibbles are elements
//                  4t..4t+3, high nibbles elements 16+4t..16+4t+3)
//   Q6_K (block: ql[128] | qh[64] | scales[16] int8 | d f16, src/quants.h:98-103).  A 128-column
//   half hf of a block packs element l + 32*qd (l < 32, qd < 4) as nibble (qd >> 1) of
//   ql[64*hf + 32*(qd & 1) + l] and bit pair qd of qh[32*hf + l]; its scale is scales[8*hf + 2*qd + l/16].
//   Word m (0..7) of a 32-byte run holds l = 4m..4m+3.  Lane (g,t) multiplies, for every (hf, qd),
//   the elements l = 4t..4t+3 (16-column group 2*(4*hf+qd)) and l = 16+4t..16+4t+3 (the group after it):
//     [   0, 256)  scales: row r at 16*r, the eight even groups 0,2,..,14 then the eight odd ones
//     [ 256,3328)  quants: chunk c (0..5), lane -> 16 B at 256 + (c*32 + lane)*16; c = 3*h + k, row g + 8h:
//                  k = 0, 1: half hf = k: ql words t and 4+t of the first 32-byte run, then of the second
//                  k = 2:    qh words t and 4+t of half 0, then of half 1
//     [3328,3360)  d[16] f16
//   Q8_0 (block: d f16 | qs[32], src/quants.h:53-57), 8 blocks per row per tile; block b of
//   the 16 rows is one 544-byte piece at 544*b (so a run of blocks is one bulk copy):
//     [  0, 32)  d: row r at 2*r
//     [ 32,544)  quants: half h (row g + 8h), lane -> 8 B at 32 + (h*32 + lane)*8
//                = raw qs[4t..4t+3] then qs[16+4t..16+4t+3]
//
// DIGIT PLANES.  An activation row x[K] is encoded as four int8 planes with one
// power-of-two scale per row (or per 128-element chunk for the expert hidden rows):
//   v = rint(x * 2^p),  |v| <= 2^26,  v = d0 + 128*d1 + 128^2*d2 + 128^3*d3,  d_j in [-64, 63]
// so x = 2^-p * sum_j 128^j d_j up to a rounding error of 2^-(p+1) <= 2^-27 * max|x|:
// finer than f32 for every element within 2^3 of the row maximum and exact integer
// arithmetic from there on (int8 x int8 -> int32 tensor-core MMAs).
#pragma once

#include <stdint.h>

namespace qkm {

static constexpr int kTileIq3 = 1568;
static constexpr int kTileIq4 = 2176;
static constexpr int kTileQ6 = 3360;
static constexpr int kTileQ8 = 4352;

__host__ __device__ inline int tile_bytes(uint32_t type) {
    switch (type) {
        case QKM_TYPE_IQ3_XXS: return kTileIq3;
        case QKM_TYPE_IQ4_XS: return kTileIq4;
        case QKM_TYPE_Q6_K: return kTileQ6;
        case QKM_TYPE_Q8_0: return kTileQ8;
        default: return 0;
    }
}

// digit planes of one activation row set: planes[(row * 4 + digit) * K + k], scale[row]
struct DigitRows {
    const int8_t* planes;
    const float* scale;  // 2^-p per row (per chunk where stated)
};

}  // namespace qkm
