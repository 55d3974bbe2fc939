// Dense dequant-GEMV of large matrices on the integer tensor-core path.
//
// Same contract as the other GEMV kernels (y[M] = W[M,K] . x[K] on raw ggml rows,
// shaders/gemv_q8_0.comp:31-32, gemv_q6_k.comp:48-73), for one input vector and matrices too large
// for the one-wave kernel.  The multiply-accumulate leaves the ALU pipe: x is encoded once per
// block as four int8 digit planes (27-bit fixed point relative to max|x|, qkm_stream.cuh) which are
// the B operand of mma.sync.m16n8k32.s8 (column n = digit plane), and the quantised weights are the
// A operand - for Q8_0 the raw bytes of a 32-column block as they lie in the row.
//
// A block has one warp per 256 columns of K, and every warp streams its own slice: for a tile of 16
// rows the 8 blocks x 34 bytes of each row that fall into its columns (272 contiguous bytes per
// row), fetched as one two-dimensional TMA copy (a tensor map over the matrix as [row][byte pair], box
// = 16 rows x 272 bytes; no multicast) into its own ring of stages.  A slice row is 68 words long, so the A-fragment loads of the eight row groups fall into
// different banks without padding, and no warp waits for another until the partial sums of eight
// tiles meet in shared memory.  (Bulk copies of whole rows into a padded block-wide stage moved
// 3.8 TB/s at most - sixteen 2 KB copies per tile - and 16-byte cp.async pieces 4.5 TB/s.)  A warp multiplies its 256 columns of the 16
// rows (eight MMAs), scales each 32-column block's integer sums by the block's f16 scale and keeps
// f32 partial sums.
#include <cuda.h>

#include "qkm_common.cuh"
#include "qkm_kernels.h"
#include "qkm_stream.cuh"

namespace qkm {

namespace gm {
constexpr int kRows = 16;          // rows per tile
constexpr int kGroup = 8;          // tiles between two reductions over the warps
constexpr int kMaxWarps = 16;      // K <= 4096
constexpr int kMaxStages = 6;
constexpr int kSlice = 8 * 34;     // bytes of one row inside a warp's 256 columns (Q8_0)
}  // namespace gm

// Q8_0: 16 rows x 32 columns of block `bi` of the tile at `st` (row stride S).  Loading a block's
// words and multiplying them are separate so that the next block's loads are in flight meanwhile.
struct Q8Frag { uint32_t w[8]; uint32_t d0, d1; };
template <bool EVEN>
__device__ __forceinline__ Q8Frag q8_block_load(uint32_t st, uint32_t S, uint32_t bi, uint32_t g, uint32_t t) {
    const uint32_t r0 = st + g * S + 34u * bi, r1 = r0 + 8u * S;
    Q8Frag f;
    if (EVEN) {   // the quants start two bytes into a word: two aligned words per fragment register
        f.w[0] = lds32(r0 + 4 * t);      f.w[1] = lds32(r0 + 4 * t + 4);
        f.w[2] = lds32(r1 + 4 * t);      f.w[3] = lds32(r1 + 4 * t + 4);
        f.w[4] = lds32(r0 + 16 + 4 * t); f.w[5] = lds32(r0 + 20 + 4 * t);
        f.w[6] = lds32(r1 + 16 + 4 * t); f.w[7] = lds32(r1 + 20 + 4 * t);
        f.d0 = lds32(r0); f.d1 = lds32(r1);             // the block scale (f16) sits in the low half
    } else {
        f.w[0] = lds32(r0 + 2 + 4 * t);  f.w[2] = lds32(r1 + 2 + 4 * t);
        f.w[4] = lds32(r0 + 18 + 4 * t); f.w[6] = lds32(r1 + 18 + 4 * t);
        f.w[1] = f.w[3] = f.w[5] = f.w[7] = 0;
        f.d0 = lds32(r0 - 2); f.d1 = lds32(r1 - 2);     // ... in the high half
    }
    return f;
}
// Adds to f0 / f1 the contribution to rows g / g+8 of this lane's two digit planes.
template <bool EVEN>
__device__ __forceinline__ void q8_block_mma(const Q8Frag& f, uint32_t b0, uint32_t b1, float plane_w, float& f0, float& f1) {
    uint32_t a0, a1, a2, a3;
    if (EVEN) {
        a0 = __funnelshift_r(f.w[0], f.w[1], 16); a1 = __funnelshift_r(f.w[2], f.w[3], 16);
        a2 = __funnelshift_r(f.w[4], f.w[5], 16); a3 = __funnelshift_r(f.w[6], f.w[7], 16);
    } else {
        a0 = f.w[0]; a1 = f.w[2]; a2 = f.w[4]; a3 = f.w[6];
    }
    int c[4] = {0, 0, 0, 0};
    mma_s8(c, a0, a1, a2, a3, b0, b1);
    const float d0 = f16_bits_to_f32(EVEN ? (f.d0 & 0xFFFFu) : (f.d0 >> 16));
    const float d1 = f16_bits_to_f32(EVEN ? (f.d1 & 0xFFFFu) : (f.d1 >> 16));
    // digits 2t (weight 1) and 2t+1 (weight 128) of this lane's pair, exact in int32
    f0 = fmaf((float)(c[0] + (c[1] << 7)) * plane_w, d0, f0);
    f1 = fmaf((float)(c[2] + (c[3] << 7)) * plane_w, d1, f1);
}

template <int TYPE>
__global__ void __launch_bounds__(gm::kMaxWarps * 32)
gemv_mma_kernel(const __grid_constant__ CUtensorMap tmap, const float* __restrict__ x, float* __restrict__ y,
                uint32_t n_tiles, uint32_t K, uint32_t n_stages, uint32_t* __restrict__ status) {
    static_assert(TYPE == QKM_TYPE_Q8_0, "formats: Q8_0");
    extern __shared__ __align__(128) uint8_t smem_raw[];
    __shared__ float s_max[gm::kMaxWarps];
    __shared__ float s_scale;
    __shared__ __align__(8) unsigned long long s_bar[gm::kMaxWarps][gm::kMaxStages];   // a stage of a warp's ring has landed
    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31u, g = lane >> 2, t = lane & 3u;
    const uint32_t KB = K / 256, n_threads = KB * 32;
    constexpr uint32_t S = gm::kSlice, kStage = gm::kRows * gm::kSlice;   // 272-byte slice rows, 4352 bytes per stage
    // layout: digit planes [KB][4][256] | partial sums [2][KB][kGroup * 16] | rings [KB][n_stages][4352]
    int8_t* planes = reinterpret_cast<int8_t*>(smem_raw);
    float* red = reinterpret_cast<float*>(smem_raw + (size_t)K * 4);
    const uint32_t red_floats = KB * gm::kGroup * gm::kRows;
    const uint32_t ring = ((smem_addr(smem_raw) + K * 4 + 2 * red_floats * 4 + 127u) & ~127u) + warp * n_stages * kStage;

    // this block's tiles: blockIdx.x, + gridDim.x, ...
    const uint32_t my_tiles = blockIdx.x < n_tiles ? (n_tiles - blockIdx.x + gridDim.x - 1) / gridDim.x : 0u;
    const uint32_t my_bar = smem_addr(&s_bar[warp][0]);
    bool timed_out = false;
    if (lane == 0) {
        for (uint32_t s = 0; s < n_stages; ++s) mbar_init(my_bar + 8 * s, 1);
        mbar_fence_init();
    }
    __syncwarp();
    auto issue = [&](uint32_t i) {   // tile number i of this block into stage i % n_stages of this warp's ring; lane 0
        const uint32_t s = i % n_stages, dst = ring + s * kStage, bar = my_bar + 8 * s;
        const uint32_t cx = warp * (S / 2), cy = (blockIdx.x + i * gridDim.x) * gm::kRows;   // byte pairs, rows
        mbar_expect_tx(bar, kStage);
        asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                     ::"r"(dst), "l"(&tmap), "r"(cx), "r"(cy), "r"(bar) : "memory");
    };
    if (lane == 0)
        for (uint32_t i = 0; i + 2 < n_stages && i < my_tiles; ++i) issue(i);   // n_stages - 2 tiles ahead; two more per pair below

    // x as digit planes (the first tiles are on their way meanwhile)
    {
        float m = 0.f;
        bool bad = false;
        for (uint32_t k = tid; k < K; k += n_threads) {
            const float v = x[k];
            bad |= !(fabsf(v) <= 3.0e38f);
            m = fmaxf(m, fabsf(v));
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xFFFFFFFFu, m, o));
        const int any_bad = __syncthreads_or(bad ? 1 : 0);
        if (lane == 0) s_max[warp] = m;
        __syncthreads();
        m = 0.f;
        for (uint32_t w = 0; w < KB; ++w) m = fmaxf(m, s_max[w]);
        const int p = digit_exponent(m);
        const float up = ldexpf(1.0f, p);
        for (uint32_t k = tid; k < K; k += n_threads) {
            const uint32_t dgt = any_bad ? 0u : digits4(__float2int_rn(x[k] * up));
            int8_t* q = planes + (size_t)(k >> 8) * 1024 + (k & 255u);
            q[0] = (int8_t)(dgt & 255u);
            q[256] = (int8_t)((dgt >> 8) & 255u);
            q[512] = (int8_t)((dgt >> 16) & 255u);
            q[768] = (int8_t)(dgt >> 24);
        }
        if (tid == 0) s_scale = any_bad ? __int_as_float(0x7FC00000) : ldexpf(1.0f, -p);
        __syncthreads();
    }
    // B operand of this warp's 256 columns: column n = g is digit plane g (g < 4), k = 4t..4t+3 and 16+4t..
    uint32_t b0[8], b1[8];
    {
        const uint32_t pl = smem_addr(planes) + warp * 1024u;
#pragma unroll
        for (int sb = 0; sb < 8; ++sb) {
            b0[sb] = g < 4 ? lds32(pl + g * 256 + sb * 32 + t * 4) : 0u;
            b1[sb] = g < 4 ? lds32(pl + g * 256 + sb * 32 + 16 + t * 4) : 0u;
        }
    }
    const float plane_w = t == 0 ? 1.f : (t == 1 ? 16384.f : 0.f);   // digits 2t, 2t+1 carry 128^(2t), 128^(2t+1)
    const float xscale = s_scale;

    uint32_t buf = 0;
    for (uint32_t i0 = 0; i0 < my_tiles; i0 += gm::kGroup) {
        const uint32_t in_group = min((uint32_t)gm::kGroup, my_tiles - i0);
        float acc[gm::kGroup][2];
#pragma unroll
        for (int q = 0; q < gm::kGroup; q += 2) {   // two tiles at a time: their dependent chains interleave
            acc[q][0] = acc[q][1] = acc[q + 1][0] = acc[q + 1][1] = 0.f;
            const uint32_t i = i0 + q;
            if (i < my_tiles) {   // block-uniform
                // refill the two stages this warp read one pair ago (its loads have returned), then wait for the pair
                __syncwarp();
                if (lane == 0) {
                    if (i + n_stages - 2 < my_tiles) issue(i + n_stages - 2);
                    if (i + n_stages - 1 < my_tiles) issue(i + n_stages - 1);
                }
                const bool two = i + 1 < my_tiles;
                if (!mbar_wait_bounded(my_bar + 8 * (i % n_stages), (i / n_stages) & 1u)) timed_out = true;
                if (two && !mbar_wait_bounded(my_bar + 8 * ((i + 1) % n_stages), ((i + 1) / n_stages) & 1u)) timed_out = true;
                const uint32_t sa = ring + (i % n_stages) * kStage, sb_ = two ? ring + ((i + 1) % n_stages) * kStage : sa;
                float fa0 = 0.f, fa1 = 0.f, fb0 = 0.f, fb1 = 0.f;
                Q8Frag ca = q8_block_load<true>(sa, S, 0, g, t), cb = q8_block_load<true>(sb_, S, 0, g, t);
#pragma unroll
                for (int sb = 0; sb < 8; ++sb) {   // block sb + 1 is loaded while block sb is multiplied
                    Q8Frag na = ca, nb = cb;
                    if (sb + 1 < 8) {
                        na = (sb & 1) ? q8_block_load<true>(sa, S, sb + 1, g, t) : q8_block_load<false>(sa, S, sb + 1, g, t);
                        nb = (sb & 1) ? q8_block_load<true>(sb_, S, sb + 1, g, t) : q8_block_load<false>(sb_, S, sb + 1, g, t);
                    }
                    if (sb & 1) { q8_block_mma<false>(ca, b0[sb], b1[sb], plane_w, fa0, fa1); q8_block_mma<false>(cb, b0[sb], b1[sb], plane_w, fb0, fb1); }
                    else { q8_block_mma<true>(ca, b0[sb], b1[sb], plane_w, fa0, fa1); q8_block_mma<true>(cb, b0[sb], b1[sb], plane_w, fb0, fb1); }
                    ca = na; cb = nb;
                }
                acc[q][0] = fa0; acc[q][1] = fa1;
                if (two) { acc[q + 1][0] = fb0; acc[q + 1][1] = fb1; }
            }
        }
        // the two digit-plane pairs of a row sit in lanes t = 0 and t = 1; then the warps' column blocks
        float* rw = red + (size_t)buf * red_floats + (size_t)warp * gm::kGroup * gm::kRows;
#pragma unroll
        for (int q = 0; q < gm::kGroup; ++q) {
            float v0 = acc[q][0], v1 = acc[q][1];
            v0 += __shfl_xor_sync(0xFFFFFFFFu, v0, 1); v1 += __shfl_xor_sync(0xFFFFFFFFu, v1, 1);
            if (t == 0) { rw[q * gm::kRows + g] = v0; rw[q * gm::kRows + g + 8] = v1; }
        }
        __syncthreads();
        for (uint32_t o = tid; o < in_group * gm::kRows; o += n_threads) {
            const float* rr = red + (size_t)buf * red_floats + o;
            float v = 0.f;
            for (uint32_t w = 0; w < KB; ++w) v += rr[(size_t)w * gm::kGroup * gm::kRows];
            const uint32_t q = o / gm::kRows, r = o - q * gm::kRows;
            const uint32_t tile = blockIdx.x + (i0 + q) * gridDim.x;
            y[(size_t)tile * gm::kRows + r] = v * xscale;
        }
        buf ^= 1u;
    }
    if (timed_out && lane == 0) atomicExch(status, (uint32_t)kStatusWaitTimeout);
}

// ---- Q6_K and IQ4_XS: a block-wide ring of whole tiles -----------------------------------------------------
// Rows of a Q6_K matrix are 210 bytes per 256 columns, so a warp's column block is not 16-byte
// aligned inside the row and cannot be fetched on its own; but a tile of 16 rows is one contiguous,
// 16-byte aligned run of the matrix, and for K = 2048 its row stride (420 words) spreads the eight row
// groups over different banks as it is.  So the whole tile comes in with ONE bulk copy into a
// block-wide ring, and every warp reads its block from there.  Inside a block the 6-bit values are
// put together from ql (low nibbles) and qh (two high bits) four at a time as int8 4 * (q - 32),
// and multiplied 32 columns at a time (mma.sync.m16n8k32.s8, the two 16-column groups of an MMA against
// different B columns: one int8 scale per 16 columns, applied to the integer sums), then by the
// block's f16 scale.
namespace gq {
constexpr int kRows = 16;
constexpr int kGroup = 4;          // tiles between two reductions over the warps
constexpr int kMaxStages = 8;
}  // namespace gq

// a 32-bit word at a 2-byte aligned shared address (ODD: the address is 2 mod 4)
template <bool ODD>
__device__ __forceinline__ uint32_t lds32_a2(uint32_t addr) {
    if (!ODD) return lds32(addr);
    return __funnelshift_r(lds32(addr - 2), lds32(addr + 2), 16);
}
__device__ __forceinline__ uint32_t prmt_q6(uint32_t a, uint32_t b, uint32_t sel) {
    uint32_t r;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(sel));
    return r;
}
// Sixteen Q6_K weights as four int8 A-operand registers, each 4 * (q - 32): the 6-bit value sits in the top
// six bits of its byte with its top bit flipped, so no sign extension is computed.  w1 / w2: the ql words
// of elements l..l+3 in the first / second 32-byte run of a 128-column half, hq: the qh word of the same l;
// r[qd] = elements l + 32 qd .. + 3  (src/quants.h:148-163).
__device__ __forceinline__ void q6_words_x4(uint32_t w1, uint32_t w2, uint32_t hq, uint32_t (&r)[4]) {
    const uint32_t hx = hq ^ 0xAAAAAAAAu;
    const uint32_t lo1 = w1 & 0x0F0F0F0Fu, hi1 = w1 & 0xF0F0F0F0u;
    const uint32_t lo2 = w2 & 0x0F0F0F0Fu, hi2 = w2 & 0xF0F0F0F0u;
    r[0] = ((hx << 6) & 0xC0C0C0C0u) | (lo1 << 2);
    r[1] = ((hx << 4) & 0xC0C0C0C0u) | (lo2 << 2);
    r[2] = ((hx << 2) & 0xC0C0C0C0u) | (hi1 >> 2);
    r[3] = (hx & 0xC0C0C0C0u) | (hi2 >> 2);
}

// One 16-row x 256-column tile.  MMA j = 4 hf + qd multiplies two 16-column groups at once (m16n8k32): the
// first against B columns 0..3 (the four digit planes; zero over the second group's k range), the second
// against columns 4..7, so lane t holds the sums of group 2j + t/2 for digits 2 (t & 1), 2 (t & 1) + 1 and
// multiplies them by that group's int8 scale as integers.  f0 / f1: rows g / g+8, this lane's share
// (the four lanes t of a row add up to the row's sum).
template <bool ODD>
__device__ __forceinline__ void q6k_tile(uint32_t blk0, uint32_t blk1, uint32_t t, const uint32_t (&b0)[8], const uint32_t (&b1)[8],
                                         float& f0, float& f1) {
    // blk0 / blk1: this warp's block of rows g / g+8 in the stage: ql[128] | qh[64] | scales[16] | d
    uint32_t sc0[4], sc1[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) { sc0[k] = lds32_a2<ODD>(blk0 + 192 + 4 * k); sc1[k] = lds32_a2<ODD>(blk1 + 192 + 4 * k); }
    const uint32_t sel_e = 0x8880u + (t >> 1) * 0x1111u, sel_o = sel_e + 0x2222u;   // byte t/2 (+2), sign-extended
    int acc[4] = {0, 0, 0, 0};
#pragma unroll
    for (int hf = 0; hf < 2; ++hf) {
        uint32_t a0[4], a1[4], a2[4], a3[4];
        {
            const uint32_t q0 = blk0 + 64 * hf + 4 * t, h0 = blk0 + 128 + 32 * hf + 4 * t;
            const uint32_t q1 = blk1 + 64 * hf + 4 * t, h1 = blk1 + 128 + 32 * hf + 4 * t;
            const uint32_t w0a = lds32_a2<ODD>(q0), w0b = lds32_a2<ODD>(q0 + 16), w0c = lds32_a2<ODD>(q0 + 32), w0d = lds32_a2<ODD>(q0 + 48);
            const uint32_t w1a = lds32_a2<ODD>(q1), w1b = lds32_a2<ODD>(q1 + 16), w1c = lds32_a2<ODD>(q1 + 32), w1d = lds32_a2<ODD>(q1 + 48);
            const uint32_t g0a = lds32_a2<ODD>(h0), g0b = lds32_a2<ODD>(h0 + 16), g1a = lds32_a2<ODD>(h1), g1b = lds32_a2<ODD>(h1 + 16);
            q6_words_x4(w0a, w0c, g0a, a0);   // row g, l = 4t ..
            q6_words_x4(w0b, w0d, g0b, a2);   // row g, l = 16 + 4t ..
            q6_words_x4(w1a, w1c, g1a, a1);   // row g + 8
            q6_words_x4(w1b, w1d, g1b, a3);
        }
#pragma unroll
        for (int qd = 0; qd < 4; ++qd) {
            const int j = 4 * hf + qd;
            int c[4] = {0, 0, 0, 0};
            mma_s8(c, a0[qd], a1[qd], a2[qd], a3[qd], b0[j], b1[j]);
            const uint32_t sel = (j & 1) ? sel_o : sel_e;
            const int sa = (int)prmt_q6(sc0[j >> 1], 0u, sel), sb = (int)prmt_q6(sc1[j >> 1], 0u, sel);
            acc[0] += sa * c[0]; acc[1] += sa * c[1]; acc[2] += sb * c[2]; acc[3] += sb * c[3];
        }
    }
    uint32_t d0, d1;
    asm volatile("ld.shared.u16 %0, [%1];" : "=r"(d0) : "r"(blk0 + 208));
    asm volatile("ld.shared.u16 %0, [%1];" : "=r"(d1) : "r"(blk1 + 208));
    const float dw0 = (t & 1u) ? 4096.f : 0.25f, dw1 = dw0 * 128.f;   // 128^(2 (t & 1)) / 4: the weights are 4 (q - 32)
    f0 = f16_bits_to_f32(d0) * ((float)acc[0] * dw0 + (float)acc[1] * dw1);
    f1 = f16_bits_to_f32(d1) * ((float)acc[2] * dw0 + (float)acc[3] * dw1);
}

// ---- IQ4_XS (in the same block-wide ring) -------------------------------------------------------------------
// A row is 136 bytes per 256 columns (d, scales_h, scales_l, 128 quant bytes), always word aligned.  A quant
// word holds elements 4t..4t+3 (low nibbles) and 16+4t..16+4t+3 (high nibbles) of a 32-column sub-block;
// the 16-entry codebook sits in four registers and is looked up with byte permutes, which leaves the
// values in the order (e, 16+e, e+1, 16+e+1 | e+2, ...): the B operand is loaded in that order too.
__device__ __forceinline__ uint32_t prmt_r(uint32_t a, uint32_t b, uint32_t sel) {
    uint32_t r;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(sel));
    return r;
}
__device__ __forceinline__ void iq4_codebook_word(uint32_t w, uint32_t& lo, uint32_t& hi) {
    const uint32_t T0 = 0xBFAD9881u, T1 = 0xF6EADDCFu, T2 = 0x26190D01u, T3 = 0x71594535u;   // kvalues_iq4nl as int8
    const uint32_t s = w & 0x77777777u, s2 = s >> 16, w4 = w << 4;
    // byte j of a mask is 0xFF when nibble j (of the low / high half-word) has its top bit set
    const uint32_t m_lo = prmt_r(w4, w, 0xD9C8u), m_hi = prmt_r(w4, w, 0xFBEAu);
    const uint32_t a_lo = prmt_r(T0, T1, s), b_lo = prmt_r(T2, T3, s);
    const uint32_t a_hi = prmt_r(T0, T1, s2), b_hi = prmt_r(T2, T3, s2);
    lo = (a_lo & ~m_lo) | (b_lo & m_lo);
    hi = (a_hi & ~m_hi) | (b_hi & m_hi);
}
// the eight sub-block scales ls - 32 of one row as int8: sub-blocks 0,2,4,6 in ev, 1,3,5,7 in od
// (scales_l: eight 4-bit fields, scales_h: eight 2-bit fields; src/quants.h:107-113, :139-146)
__device__ __forceinline__ void iq4_row_scales(uint32_t sl, uint32_t sh, uint32_t& ev, uint32_t& od) {
    const uint32_t r = prmt_r(sh, 0u, 0x1100u);                        // bytes (B0, B0, B1, B1) of scales_h
    const uint32_t he = ((r << 4) & 0x00300030u) | (r & 0x30003000u);  // top two bits of sub-blocks 0,2,4,6 at bits 4..5
    const uint32_t ho = ((r << 2) & 0x00300030u) | ((r >> 2) & 0x30003000u);
    const uint32_t te = ((sl & 0x0F0F0F0Fu) | he) ^ 0x20202020u;       // ls ^ 32 per byte
    const uint32_t to = (((sl >> 4) & 0x0F0F0F0Fu) | ho) ^ 0x20202020u;
    ev = (te & 0x20202020u) * 6u + te;                                 // ls - 32 as int8 (bit 5 extended into bits 6..7)
    od = (to & 0x20202020u) * 6u + to;
}
__device__ __forceinline__ void iq4_tile(uint32_t blk0, uint32_t blk1, uint32_t t, const uint32_t (&b0)[8], const uint32_t (&b1)[8],
                                         float plane_w, float& f0, float& f1) {
    const uint32_t h0 = lds32(blk0), h1 = lds32(blk1);   // d | scales_h << 16
    uint32_t ev0, od0, ev1, od1;
    iq4_row_scales(lds32(blk0 + 4), h0 >> 16, ev0, od0);
    iq4_row_scales(lds32(blk1 + 4), h1 >> 16, ev1, od1);
    uint32_t w0[8], w1[8];
#pragma unroll
    for (int sb = 0; sb < 8; ++sb) { w0[sb] = lds32(blk0 + 8 + 16 * sb + 4 * t); w1[sb] = lds32(blk1 + 8 + 16 * sb + 4 * t); }
    float s0 = 0.f, s1 = 0.f;
#pragma unroll
    for (int sb = 0; sb < 8; ++sb) {
        uint32_t a0, a1, a2, a3;
        iq4_codebook_word(w0[sb], a0, a2);
        iq4_codebook_word(w1[sb], a1, a3);
        int c[4] = {0, 0, 0, 0};
        mma_s8(c, a0, a1, a2, a3, b0[sb], b1[sb]);
        const int l0 = (int)(int8_t)(((sb & 1) ? od0 : ev0) >> (8 * (sb >> 1)));
        const int l1 = (int)(int8_t)(((sb & 1) ? od1 : ev1) >> (8 * (sb >> 1)));
        s0 += (float)((c[0] + (c[1] << 7)) * l0);
        s1 += (float)((c[2] + (c[3] << 7)) * l1);
    }
    f0 = s0 * plane_w * f16_bits_to_f32(h0 & 0xFFFFu);
    f1 = s1 * plane_w * f16_bits_to_f32(h1 & 0xFFFFu);
}

template <int TYPE>
__global__ void __launch_bounds__(gm::kMaxWarps * 32, 1)
gemv_tile_kernel(const uint8_t* __restrict__ W, const float* __restrict__ x, float* __restrict__ y, uint32_t n_tiles,
                uint32_t K, uint32_t rb, uint32_t n_stages, uint32_t* __restrict__ status) {
    extern __shared__ __align__(128) uint8_t smem_raw[];
    __shared__ __align__(8) unsigned long long s_bar[2 * gq::kMaxStages];   // full[stage], empty[stage]
    __shared__ float s_max[gm::kMaxWarps];
    __shared__ float s_scale;
    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31u, g = lane >> 2, t = lane & 3u;
    const uint32_t KB = K / 256, n_threads = KB * 32;
    // layout: digit planes [KB][4][256] | partial sums [2][KB][kGroup * 16] | stages [n_stages][16 rows][rb]
    int8_t* planes = reinterpret_cast<int8_t*>(smem_raw);
    float* red = reinterpret_cast<float*>(smem_raw + (size_t)K * 4);
    const uint32_t red_floats = KB * gq::kGroup * gq::kRows;
    const uint32_t stage0 = (smem_addr(smem_raw) + K * 4 + 2 * red_floats * 4 + 127u) & ~127u;
    const uint32_t stage_bytes = (gq::kRows * rb + 127u) & ~127u;
    const uint32_t bar_full = smem_addr(&s_bar[0]), bar_empty = smem_addr(&s_bar[gq::kMaxStages]);
    bool timed_out = false;

    if (tid == 0) {
        for (uint32_t s = 0; s < n_stages; ++s) { mbar_init(bar_full + 8 * s, 1); mbar_init(bar_empty + 8 * s, KB); }
        mbar_fence_init();
    }
    __syncthreads();
    const uint32_t my_tiles = blockIdx.x < n_tiles ? (n_tiles - blockIdx.x + gridDim.x - 1) / gridDim.x : 0u;
    auto issue = [&](uint32_t i) {   // tile number i of this block into stage i % n_stages: one copy; thread 0
        const uint32_t s = i % n_stages;
        mbar_expect_tx(bar_full + 8 * s, gq::kRows * rb);
        bulk_g2s(stage0 + s * stage_bytes, W + (size_t)(blockIdx.x + i * gridDim.x) * gq::kRows * rb, gq::kRows * rb, bar_full + 8 * s);
    };
    if (tid == 0)
        for (uint32_t i = 0; i + 1 < n_stages && i < my_tiles; ++i) issue(i);

    // x as digit planes (the first tiles are on their way meanwhile)
    {
        float m = 0.f;
        bool bad = false;
        for (uint32_t k = tid; k < K; k += n_threads) {
            const float v = x[k];
            bad |= !(fabsf(v) <= 3.0e38f);
            m = fmaxf(m, fabsf(v));
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xFFFFFFFFu, m, o));
        const int any_bad = __syncthreads_or(bad ? 1 : 0);
        if (lane == 0) s_max[warp] = m;
        __syncthreads();
        m = 0.f;
        for (uint32_t w = 0; w < KB; ++w) m = fmaxf(m, s_max[w]);
        const int p = digit_exponent(m);
        const float up = ldexpf(1.0f, p);
        for (uint32_t k = tid; k < K; k += n_threads) {
            const uint32_t dgt = any_bad ? 0u : digits4(__float2int_rn(x[k] * up));
            int8_t* q = planes + (size_t)(k >> 8) * 1024 + (k & 255u);
            q[0] = (int8_t)(dgt & 255u);
            q[256] = (int8_t)((dgt >> 8) & 255u);
            q[512] = (int8_t)((dgt >> 16) & 255u);
            q[768] = (int8_t)(dgt >> 24);
        }
        if (tid == 0) s_scale = any_bad ? __int_as_float(0x7FC00000) : ldexpf(1.0f, -p);
        __syncthreads();
    }
    static_assert(TYPE == QKM_TYPE_Q6_K || TYPE == QKM_TYPE_IQ4_XS, "formats: Q6_K, IQ4_XS");
    constexpr uint32_t kBlockBytes = TYPE == QKM_TYPE_Q6_K ? 210u : 136u;
    // B operands of this warp's 256 columns.  IQ4_XS: column n = g is digit plane g (g < 4), 32 columns each in the
    // codebook look-up's element order (see iq4_codebook_word).  Q6_K: see q6k_tile.
    uint32_t bq[16];
    {
        const uint32_t pl = smem_addr(planes) + warp * 1024u;
        if (TYPE == QKM_TYPE_Q6_K) {
#pragma unroll
            for (int j = 0; j < 8; ++j) {   // lanes g < 4: digit g of the first group of MMA j; g >= 4: digit g - 4 of the second
                const uint32_t v = lds32(pl + (g & 3u) * 256 + j * 32 + (g >> 2) * 16 + t * 4);
                bq[j] = g < 4 ? v : 0u;
                bq[8 + j] = g < 4 ? 0u : v;
            }
        } else {
#pragma unroll
            for (int sb = 0; sb < 8; ++sb) {
                const uint32_t wa = g < 4 ? lds32(pl + g * 256 + sb * 32 + t * 4) : 0u;        // elements 4t .. 4t+3
                const uint32_t wb = g < 4 ? lds32(pl + g * 256 + sb * 32 + 16 + t * 4) : 0u;   // elements 16+4t ..
                bq[sb] = prmt_r(wa, wb, 0x5140u);       // e, 16+e, e+1, 16+e+1
                bq[8 + sb] = prmt_r(wa, wb, 0x7362u);   // e+2, 16+e+2, e+3, 16+e+3
            }
        }
    }
    const float plane_w = t == 0 ? 1.f : (t == 1 ? 16384.f : 0.f);
    const float xscale = s_scale;
    const bool odd = TYPE == QKM_TYPE_Q6_K && (warp & 1u) != 0;   // 210 * warp is 2 mod 4 for odd warps (K / 256 is even: rows start on word boundaries)

    uint32_t buf = 0;
    for (uint32_t i0 = 0; i0 < my_tiles; i0 += gq::kGroup) {
        const uint32_t in_group = min((uint32_t)gq::kGroup, my_tiles - i0);
        float acc[gq::kGroup][2];
#pragma unroll
        for (int q = 0; q < gq::kGroup; ++q) {
            acc[q][0] = acc[q][1] = 0.f;
            const uint32_t i = i0 + q;
            if (i < my_tiles) {   // block-uniform
                const uint32_t s = i % n_stages;
                if (tid == 0 && i + n_stages - 1 < my_tiles) {   // refill the stage the block left one tile ago
                    const uint32_t j = i + n_stages - 1, sj = j % n_stages;
                    if (j >= n_stages && !mbar_wait_bounded(bar_empty + 8 * sj, ((j / n_stages) - 1) & 1u)) timed_out = true;
                    issue(j);
                }
                if (!mbar_wait_bounded(bar_full + 8 * s, (i / n_stages) & 1u)) timed_out = true;
                const uint32_t blk0 = stage0 + s * stage_bytes + g * rb + kBlockBytes * warp, blk1 = blk0 + 8u * rb;
                float f0, f1;
                uint32_t b0[8], b1[8];
#pragma unroll
                for (int sb = 0; sb < 8; ++sb) { b0[sb] = bq[sb]; b1[sb] = bq[8 + sb]; }
                if (TYPE == QKM_TYPE_IQ4_XS) {
                    iq4_tile(blk0, blk1, t, b0, b1, plane_w, f0, f1);
                } else if (odd) {
                    q6k_tile<true>(blk0, blk1, t, b0, b1, f0, f1);
                } else {
                    q6k_tile<false>(blk0, blk1, t, b0, b1, f0, f1);
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(bar_empty + 8 * s);
                acc[q][0] = f0; acc[q][1] = f1;
            }
        }
        float* rw = red + (size_t)buf * red_floats + (size_t)warp * gq::kGroup * gq::kRows;
#pragma unroll
        for (int q = 0; q < gq::kGroup; ++q) {
            float v0 = acc[q][0], v1 = acc[q][1];
            v0 += __shfl_xor_sync(0xFFFFFFFFu, v0, 1); v1 += __shfl_xor_sync(0xFFFFFFFFu, v1, 1);
            if (TYPE == QKM_TYPE_Q6_K) {   // all four lanes of a row hold a share
                v0 += __shfl_xor_sync(0xFFFFFFFFu, v0, 2); v1 += __shfl_xor_sync(0xFFFFFFFFu, v1, 2);
            }
            if (t == 0) { rw[q * gq::kRows + g] = v0; rw[q * gq::kRows + g + 8] = v1; }
        }
        __syncthreads();
        for (uint32_t o = tid; o < in_group * gq::kRows; o += n_threads) {
            const float* rr = red + (size_t)buf * red_floats + o;
            float v = 0.f;
            for (uint32_t w = 0; w < KB; ++w) v += rr[(size_t)w * gq::kGroup * gq::kRows];
            const uint32_t q = o / gq::kRows, r = o - q * gq::kRows;
            const uint32_t tile = blockIdx.x + (i0 + q) * gridDim.x;
            y[(size_t)tile * gq::kRows + r] = v * xscale;
        }
        buf ^= 1u;
    }
    if (timed_out && lane == 0) atomicExch(status, (uint32_t)kStatusWaitTimeout);
}

template <int TYPE>
static cudaError_t gemv_tile_launch(const Launch& L, const void* W, const float* x, float* y, uint32_t M, uint32_t K,
                                    uint32_t n_sms, uint32_t* status, uint32_t* rows_done) {
    const uint32_t KB = K / 256;
    if (K % 512 != 0 || KB > (uint32_t)gm::kMaxWarps || M < (uint32_t)gq::kRows) return cudaSuccess;   // an even number of blocks per row
    const uint32_t rb = (TYPE == QKM_TYPE_Q6_K ? 210u : 136u) * KB;
    const size_t fixed = (size_t)K * 4 + 2 * (size_t)KB * gq::kGroup * gq::kRows * 4 + 256;
    const size_t stage = ((size_t)gq::kRows * rb + 127) / 128 * 128;
    // two blocks per SM with three stages each where that fits (the kernel is bound by its own instructions,
    // so warps count), else one block with as many stages as fit
    uint32_t n_stages = 3;
    uint32_t per_sm = 2;
    if (fixed + 3 * stage > 110u * 1024u) {
        per_sm = 1;
        n_stages = gq::kMaxStages;
        while (n_stages > 2 && fixed + n_stages * stage > 200u * 1024u) --n_stages;
    }
    const size_t smem = fixed + n_stages * stage;
    if (smem > 220u * 1024u) return cudaSuccess;
    cudaError_t e = cudaFuncSetAttribute(gemv_tile_kernel<TYPE>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    const uint32_t n_tiles = M / gq::kRows;
    const uint32_t blocks = n_tiles < per_sm * n_sms ? n_tiles : per_sm * n_sms;
    gemv_tile_kernel<TYPE><<<blocks, KB * 32, smem, L.stream>>>((const uint8_t*)W, x, y, n_tiles, K, rb, n_stages, status);
    L.count();
    *rows_done = n_tiles * gq::kRows;
    return cudaGetLastError();
}

// Rows [0, *rows_done) are computed here; the caller finishes the rest.  Shapes this form does not take
// leave *rows_done at 0.
cudaError_t launch_gemv_mma(const Launch& L, uint32_t type, const void* W, const float* x, float* y, uint32_t M,
                            uint32_t K, uint32_t n_sms, uint32_t* status, uint32_t* rows_done) {
    *rows_done = 0;
    if (type == QKM_TYPE_Q6_K || type == QKM_TYPE_IQ4_XS) {
        if (((uintptr_t)W & 15u) || ((uintptr_t)x & 3u) || status == nullptr) return cudaSuccess;
        return type == QKM_TYPE_Q6_K ? gemv_tile_launch<QKM_TYPE_Q6_K>(L, W, x, y, M, K, n_sms, status, rows_done)
                                     : gemv_tile_launch<QKM_TYPE_IQ4_XS>(L, W, x, y, M, K, n_sms, status, rows_done);
    }
    if (type != QKM_TYPE_Q8_0 || K % 256 != 0 || K < 512 || K > 256u * gm::kMaxWarps || M < (uint32_t)gm::kRows) return cudaSuccess;
    if (((uintptr_t)W & 15u) || ((uintptr_t)x & 3u) || status == nullptr) return cudaSuccess;
    const uint32_t rb = (uint32_t)row_bytes(type, K);   // a multiple of 16 for K % 256 == 0
    if (rb % 16) return cudaSuccess;
    const uint32_t KB = K / 256;
    const size_t fixed = (size_t)K * 4 + 2 * (size_t)KB * gm::kGroup * gm::kRows * 4 + 128;
    const size_t stage = (size_t)KB * gm::kRows * gm::kSlice;   // one stage of every warp's ring
    // one block per SM with as deep a ring as fits: the bytes in flight, not the warps, carry the bandwidth
    uint32_t n_stages = gm::kMaxStages;
    while (n_stages > 3 && fixed + n_stages * stage > 200u * 1024u) --n_stages;
    const size_t smem = fixed + n_stages * stage;
    if (smem > 220u * 1024u || n_stages < 3) return cudaSuccess;
    // the matrix as [M rows][rb / 2 byte pairs]; a box is one warp's slice of a tile
    typedef CUresult (*EncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                 const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                 CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
    static EncodeFn encode = nullptr;
    if (!encode) {
        void* fn = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres) != cudaSuccess || !fn) return cudaSuccess;
        encode = (EncodeFn)fn;
    }
    CUtensorMap tmap;
    const cuuint64_t gdim[2] = {rb / 2, M}, gstride[1] = {rb};
    const cuuint32_t box[2] = {gm::kSlice / 2, gm::kRows}, estride[2] = {1, 1};
    if (encode(&tmap, CU_TENSOR_MAP_DATA_TYPE_UINT16, 2, const_cast<void*>(W), gdim, gstride, box, estride, CU_TENSOR_MAP_INTERLEAVE_NONE,
               CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
        return cudaSuccess;   // the other kernels take the call
    cudaError_t e = cudaFuncSetAttribute(gemv_mma_kernel<QKM_TYPE_Q8_0>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    const uint32_t n_tiles = M / gm::kRows;
    const uint32_t per_sm = smem <= 110u * 1024u ? 2u : 1u;
    const uint32_t blocks = n_tiles < per_sm * n_sms ? n_tiles : per_sm * n_sms;
    gemv_mma_kernel<QKM_TYPE_Q8_0><<<blocks, KB * 32, smem, L.stream>>>(tmap, x, y, n_tiles, K, n_stages, status);
    L.count();
    *rows_done = n_tiles * gm::kRows;
    return cudaGetLastError();
}

}  // namespace qkm
