// Down projection of the fused decode sequence, token major, routed experts (IQ4_XS) and the
// shared expert (Q8_0) and the final weighted sum in one persistent launch:
//   y[t] = sum_s w_s * D[ids_s] . h[t][s]  +  w_shared * DS . h[t][n_used].
//
// Replaces moe_down_iq4.comp + moe_down_q8b.comp + the "routed + shared" add.  A unit of work
// is (token, 16 output rows) and belongs to a whole block: warp (slot s, column block kb)
// streams the 16-row tile of expert ids_s through a private two-stage ring of bulk copies
// (TMA, no tensor map, no multicast), with the three bf16 pieces of h[t][s] for its 256 columns
// once per chunk of up to four tiles, so the eight slots of a token are worked on at once and
// are added in slot order by the block - no per-slot scratch in global memory, no atomics, the
// same bits on every run.  Tiles are cut evenly and contiguously over the blocks (one tile of
// imbalance in ~14).
//
// IQ4_XS inner step: a quant byte holds elements j and j+16 of a 32-column sub-block; a
// byte-permute drops it into bits 8..15 of a table address whose other bytes are lane
// constants (256-byte stride per entry, table at a 64 KB boundary), and the entry is the
// packed bf16 pair of the two codebook values = one MMA A-operand register.  Products with
// the bf16 pieces are exact, sums are f32 on the tensor cores, d * (ls - 32) multiplies each
// sub-block's partial sum.
//
// Shared expert: warp w also takes 32-column block w of the Q8_0 matrix for the tile's rows:
// raw int8 weights against h[t][n_used] as int8 digit planes, which the block encodes in shared
// memory whenever its token changes (an exact integer MMA, one f32 scale per block).
#include "qkm_kernels.h"
#include "qkm_stream.cuh"
#include "qkm_tiles.cuh"

namespace qkm {

namespace dd {
constexpr int kWarps = 16;
constexpr int kStages = 2;
constexpr int kBBytes = 3 * 512;                    // three pieces x 256 columns x bf16
constexpr int kShBlock = 32 + 512;                  // one Q8_0 block column of a 16-row tile: d, quants
constexpr int kStageBytes = kBBytes + kTileIq4 + kShBlock;   // 4256
constexpr int kRingBytes = kStages * kStageBytes;
constexpr uint32_t kTab = 65536, kTabBytes = 65536;
constexpr int kLowRingWarps = 7;
constexpr uint32_t kHigh = kTab + kTabBytes;
constexpr uint32_t kDl = kHigh + (kWarps - kLowRingWarps) * kRingBytes;   // 16 x 128 floats
constexpr int kChunk = 4;                                                 // tiles between two block-wide sums
constexpr uint32_t kRed = kDl + kWarps * 128 * 4;                         // [2 buffers][16 warps][kChunk tiles][16 rows]
constexpr uint32_t kHd = kRed + 2 * kWarps * kChunk * 16 * 4;             // 4 digit planes x 512 of h[t][n_used]
constexpr uint32_t kMisc = kHd + 4 * 512;                                 // 16 warp maxima, the row scale
constexpr uint32_t kEnd = kMisc + 128;
constexpr uint32_t kMaxFf = 512;
}  // namespace dd

size_t decode_down_lut_bytes() { return dd::kTabBytes; }

// row b (256 B) = for 32 lanes the packed bf16 pair (value of low nibble, value of high nibble)
__global__ void decode_down_lut_kernel(uint8_t* __restrict__ out) {
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= dd::kTabBytes / 4) return;
    const uint32_t b = i >> 6, w = i & 63u;
    uint32_t v = 0;
    if (w < 32) {
        const __nv_bfloat16 lo = __float2bfloat16_rn((float)c_iq4_values[b & 15u]);
        const __nv_bfloat16 hi = __float2bfloat16_rn((float)c_iq4_values[b >> 4]);
        v = (uint32_t)__bfloat16_as_ushort(lo) | ((uint32_t)__bfloat16_as_ushort(hi) << 16);
    }
    reinterpret_cast<uint32_t*>(out)[i] = v;
}

cudaError_t launch_decode_down_lut(const Launch& L, uint8_t* lut) {
    decode_down_lut_kernel<<<dd::kTabBytes / 4 / 256, 256, 0, L.stream>>>(lut);
    L.count();
    return cudaGetLastError();
}

__device__ __forceinline__ uint32_t prmt_dd(uint32_t a, uint32_t b, uint32_t sel) {
    uint32_t r;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(sel));
    return r;
}

__global__ void __launch_bounds__(dd::kWarps * 32, 1)
decode_down_kernel(DownDecodeArgs a) {
    extern __shared__ __align__(128) uint8_t smem_raw[];
    const uint32_t base = smem_addr(smem_raw);
    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31u, g = lane >> 2, t = lane & 3u;
    const qkm_dims d = a.d;
    const uint32_t KB = d.n_ff / 256;               // 2
    const uint32_t slot = warp / KB, kb = warp - slot * KB;
    const uint32_t RT = d.n_embd / 16;              // row tiles of the down matrix
    const uint32_t n_slots = d.n_used + 1;
    const bool with_shared = a.sh_tiles != nullptr;

    const uint32_t bar_base = (base + 15u) & ~15u;
    const uint32_t tab_bar = bar_base + dd::kWarps * dd::kStages * 8;
    const uint32_t low_ring = (tab_bar + 8 + 127u) & ~127u;
    if (low_ring + dd::kLowRingWarps * dd::kRingBytes > dd::kTab) {
        if (tid == 0) atomicExch(a.status, (uint32_t)kStatusBadLayout);
        return;
    }
    const uint32_t ring = warp < (uint32_t)dd::kLowRingWarps ? low_ring + warp * dd::kRingBytes
                                                             : dd::kHigh + (warp - dd::kLowRingWarps) * dd::kRingBytes;
    const uint32_t my_bar = bar_base + warp * dd::kStages * 8;
    const uint32_t my_dl = dd::kDl + warp * 128 * 4;
    float* dl = reinterpret_cast<float*>(smem_raw + (my_dl - base));
    float* red = reinterpret_cast<float*>(smem_raw + (dd::kRed - base));
    int8_t* s_hd = reinterpret_cast<int8_t*>(smem_raw + (dd::kHd - base));
    float* s_misc = reinterpret_cast<float*>(smem_raw + (dd::kMisc - base));
    bool timed_out = false;

    if (lane == 0) {
        for (int s = 0; s < dd::kStages; ++s) mbar_init(my_bar + 8 * s, 1);
        if (warp == 0) mbar_init(tab_bar, 1);
        mbar_fence_init();
    }
    __syncthreads();
    if (tid == 0) {
        mbar_expect_tx(tab_bar, dd::kTabBytes);
        for (uint32_t i = 0; i < 4; ++i) bulk_g2s(dd::kTab + i * 16384u, a.lut + i * 16384u, 16384u, tab_bar);
    }

    // Work: the flat list of (token, 16-row tile) is cut evenly and contiguously over the blocks; a
    // block walks its range in chunks of up to kChunk tiles of one token, sums once per chunk.
    const uint64_t tiles_total = (uint64_t)a.n_tokens * RT;
    const uint32_t t_lo = (uint32_t)(tiles_total * blockIdx.x / gridDim.x);
    const uint32_t t_hi = (uint32_t)(tiles_total * (blockIdx.x + 1) / gridDim.x);
    const size_t mat_tiles = (size_t)KB * RT;
    auto chunk_len = [&](uint32_t tile, uint32_t rt) -> uint32_t { return min((uint32_t)dd::kChunk, min(t_hi - tile, RT - rt)); };

    // producer cursor; lane 0 only.  The first stage of a chunk also carries the bf16 pieces of
    // h[t][slot] for the warp's 256 columns.
    uint32_t p_tile = t_lo, p_tok = t_lo / RT, p_rt = t_lo - p_tok * RT, p_left = 0;
    bool p_new_tok = true;
    const uint8_t* p_src = nullptr;     // next tile of expert ids[slot]
    const uint8_t* p_sh = nullptr;      // next tile of the shared matrix (column block warp / 8)
    auto issue = [&](uint32_t stage) {
        if (p_tile >= t_hi) return;
        if (p_new_tok) {
            p_new_tok = false;
            const uint32_t e = min(a.sel[p_tok].ids[slot], d.n_expert - 1);
            p_src = a.tiles + ((size_t)e * mat_tiles + (size_t)kb * RT + p_rt) * kTileIq4;
            if (with_shared) p_sh = a.sh_tiles + ((size_t)(warp >> 3) * RT + p_rt) * kTileQ8;
        }
        const bool first = p_left == 0;
        if (first) p_left = chunk_len(p_tile, p_rt);
        const uint32_t bar = my_bar + 8 * stage, dst = ring + stage * dd::kStageBytes;
        mbar_expect_tx(bar, kTileIq4 + (with_shared ? dd::kShBlock : 0) + (first ? dd::kBBytes : 0));
        if (first) {
            const __nv_bfloat16* hp = reinterpret_cast<const __nv_bfloat16*>(a.hpieces) + ((size_t)(p_tok * n_slots + slot) * 3) * d.n_ff + 256 * kb;
            bulk_g2s(dst, hp, 512, bar);
            bulk_g2s(dst + 512, hp + d.n_ff, 512, bar);
            bulk_g2s(dst + 1024, hp + 2 * (size_t)d.n_ff, 512, bar);
        }
        bulk_g2s(dst + dd::kBBytes, p_src, kTileIq4, bar);
        p_src += kTileIq4;
        if (with_shared) {   // block column `warp` of the shared matrix: column block warp / 8, block warp % 8
            bulk_g2s(dst + dd::kBBytes + kTileIq4, p_sh + 32 * (warp & 7u), 32, bar);
            bulk_g2s(dst + dd::kBBytes + kTileIq4 + 32, p_sh + 256 + 512 * (warp & 7u), 512, bar);
            p_sh += kTileQ8;
        }
        ++p_tile; --p_left;
        if (++p_rt == RT) { p_rt = 0; ++p_tok; p_new_tok = true; }
    };
    if (lane == 0)
        for (int s = 0; s < dd::kStages; ++s) issue(s);

    const uint32_t lut_c = dd::kTab + lane * 4;
    uint32_t cnt = 0, buf = 0;
    float w_s = 0.f, w_sh = 0.f;   // routing weight of this warp's slot; w_shared * 2^-p of the shared row's digits
    uint32_t bq[8][4];
    const bool b_lane = g < 3;   // column g = piece g of the token; other columns are zero
    // digit weights of the shared expert's integer MMA: C columns 2t, 2t+1 are digits 2t, 2t+1 (t < 2)
    const float dw0 = t == 0 ? 1.f : (t == 1 ? 16384.f : 0.f), dw1 = dw0 * 128.f;

    if (!mbar_wait_bounded(tab_bar, 0)) timed_out = true;

    uint32_t tok = t_lo / RT, rt = t_lo - tok * RT;
    bool new_tok = true;
    for (uint32_t tile = t_lo; tile < t_hi;) {
        if (new_tok) {   // block-uniform
            new_tok = false;
            w_s = a.sel[tok].w[slot];
            w_sh = a.sel[tok].w_shared;
            if (with_shared) {
                // h[t][n_used] as four int8 digit planes in shared memory, one power-of-two scale
                const float* hs = a.h + ((size_t)tok * n_slots + d.n_used) * d.n_ff;
                const float hv = tid < d.n_ff ? hs[tid] : 0.f;
                float m = fabsf(hv);
                const bool bad = !(m <= 3.0e38f);
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xFFFFFFFFu, m, o));
                const int any_bad = __syncthreads_or(bad ? 1 : 0);
                if (lane == 0) s_misc[warp] = m;
                __syncthreads();
                float mx = 0.f;
#pragma unroll
                for (int w = 0; w < dd::kWarps; ++w) mx = fmaxf(mx, s_misc[w]);
                const int p = digit_exponent(mx);
                if (tid < d.n_ff) {
                    const uint32_t dgt = any_bad ? 0u : digits4(__float2int_rn(hv * ldexpf(1.0f, p)));
                    s_hd[tid] = (int8_t)(dgt & 255u);
                    s_hd[dd::kMaxFf + tid] = (int8_t)((dgt >> 8) & 255u);
                    s_hd[2 * dd::kMaxFf + tid] = (int8_t)((dgt >> 16) & 255u);
                    s_hd[3 * dd::kMaxFf + tid] = (int8_t)(dgt >> 24);
                }
                w_sh *= any_bad ? __int_as_float(0x7FC00000) : ldexpf(1.0f, -p);
                __syncthreads();
            }
        }
        const uint32_t n_c = chunk_len(tile, rt);
        uint32_t hb0 = 0, hb1 = 0;   // the shared expert's B operand: digit g of block column `warp`
        if (with_shared && g < 4) {
            const int8_t* hp = s_hd + g * dd::kMaxFf + 32 * warp;
            hb0 = *reinterpret_cast<const uint32_t*>(hp + 4 * t);
            hb1 = *reinterpret_cast<const uint32_t*>(hp + 16 + 4 * t);
        }
#pragma unroll 1
        for (uint32_t i = 0; i < n_c; ++i, ++cnt) {
            const uint32_t stage = cnt % dd::kStages, parity = (cnt / dd::kStages) & 1u;
            if (!mbar_wait_bounded(my_bar + 8 * stage, parity)) timed_out = true;
            const uint32_t sb0 = ring + stage * dd::kStageBytes, tb = sb0 + dd::kBBytes, qb = tb + kTileIq4;
            if (i == 0) {
#pragma unroll
                for (int sb = 0; sb < 8; ++sb) {
                    uint4 v = make_uint4(0, 0, 0, 0);
                    if (b_lane) v = lds128(sb0 + g * 512 + (sb * 4 + t) * 16);
                    bq[sb][0] = v.x; bq[sb][1] = v.y; bq[sb][2] = v.z; bq[sb][3] = v.w;
                }
            }
            // sub-block scales d * (ls - 32): lane (g, t) computes rows g, g+8 x sub-blocks 2t, 2t+1
            {
                const uint4 hd = lds128(tb + 16 * g);
                const float da = f16_bits_to_f32(hd.x & 0xFFFFu), db = f16_bits_to_f32(hd.z & 0xFFFFu);
                const uint32_t sha = hd.x >> 16, shb = hd.z >> 16;
#pragma unroll
                for (int j = 0; j < 2; ++j) {
                    const uint32_t sb = 2 * t + j;
                    const int lsa = (int)(((hd.y >> (4 * sb)) & 0xFu) | (((sha >> (2 * sb)) & 3u) << 4)) - 32;
                    const int lsb = (int)(((hd.w >> (4 * sb)) & 0xFu) | (((shb >> (2 * sb)) & 3u) << 4)) - 32;
                    dl[g * 8 + sb] = da * (float)lsa;
                    dl[(g + 8) * 8 + sb] = db * (float)lsb;
                }
            }
            __syncwarp();
            float dla[8], dlb[8];
            {
                const uint4 a0 = lds128(my_dl + (g * 8) * 4), a1 = lds128(my_dl + (g * 8 + 4) * 4);
                const uint4 b0 = lds128(my_dl + ((g + 8) * 8) * 4), b1 = lds128(my_dl + ((g + 8) * 8 + 4) * 4);
                dla[0] = __uint_as_float(a0.x); dla[1] = __uint_as_float(a0.y); dla[2] = __uint_as_float(a0.z); dla[3] = __uint_as_float(a0.w);
                dla[4] = __uint_as_float(a1.x); dla[5] = __uint_as_float(a1.y); dla[6] = __uint_as_float(a1.z); dla[7] = __uint_as_float(a1.w);
                dlb[0] = __uint_as_float(b0.x); dlb[1] = __uint_as_float(b0.y); dlb[2] = __uint_as_float(b0.z); dlb[3] = __uint_as_float(b0.w);
                dlb[4] = __uint_as_float(b1.x); dlb[5] = __uint_as_float(b1.y); dlb[6] = __uint_as_float(b1.z); dlb[7] = __uint_as_float(b1.w);
            }
            float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int hf = 0; hf < 2; ++hf) {
                const uint4 qa4 = lds128(tb + 128 + (hf * 32 + lane) * 16);
                const uint4 qb4 = lds128(tb + 128 + ((2 + hf) * 32 + lane) * 16);
                const uint32_t wa[4] = {qa4.x, qa4.y, qa4.z, qa4.w}, wb[4] = {qb4.x, qb4.y, qb4.z, qb4.w};
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const int sb = 4 * hf + j;
                    const uint32_t x = wa[j], y = wb[j];
                    const uint32_t a0 = lds32(prmt_dd(x, lut_c, 0x7604u)), a1 = lds32(prmt_dd(x, lut_c, 0x7614u));
                    const uint32_t a2 = lds32(prmt_dd(x, lut_c, 0x7624u)), a3 = lds32(prmt_dd(x, lut_c, 0x7634u));
                    const uint32_t b0 = lds32(prmt_dd(y, lut_c, 0x7604u)), b1 = lds32(prmt_dd(y, lut_c, 0x7614u));
                    const uint32_t b2 = lds32(prmt_dd(y, lut_c, 0x7624u)), b3 = lds32(prmt_dd(y, lut_c, 0x7634u));
                    float c[4] = {0.f, 0.f, 0.f, 0.f};
                    mma_bf16(c, a0, b0, a1, b1, bq[sb][0], bq[sb][1]);
                    mma_bf16(c, a2, b2, a3, b3, bq[sb][2], bq[sb][3]);
                    acc[0] += dla[sb] * c[0]; acc[1] += dla[sb] * c[1];
                    acc[2] += dlb[sb] * c[2]; acc[3] += dlb[sb] * c[3];
                }
            }
            // shared expert: one Q8_0 block (32 columns) of the tile's 16 rows against the digit planes
            float sa = 0.f, sb_ = 0.f;
            if (with_shared) {
                const uint2 qa = lds64(qb + 32 + lane * 8);            // row g: qs[4t..4t+3], qs[16+4t..16+4t+3]
                const uint2 qc = lds64(qb + 32 + 256 + lane * 8);      // row g+8
                int c[4] = {0, 0, 0, 0};
                mma_s8(c, qa.x, qc.x, qa.y, qc.y, hb0, hb1);
                const uint32_t dw = lds32(qb + 2 * (g & ~1u)), dw8 = lds32(qb + 2 * (8 + (g & ~1u)));
                const float da = f16_bits_to_f32((dw >> (16 * (g & 1u))) & 0xFFFFu);
                const float db = f16_bits_to_f32((dw8 >> (16 * (g & 1u))) & 0xFFFFu);
                sa = da * ((float)c[0] * dw0 + (float)c[1] * dw1);
                sb_ = db * ((float)c[2] * dw0 + (float)c[3] * dw1);
            }
            __syncwarp();
            if (lane == 0) issue(stage);
            // pieces: columns 0, 1 in lane t = 0, column 2 in lane t = 1; digits: 0, 1 in t = 0 and 2, 3 in t = 1.
            // The routing weight multiplies the finished column sum of this warp's block.
            float va = w_s * (acc[0] + acc[1]) + w_sh * sa, vb = w_s * (acc[2] + acc[3]) + w_sh * sb_;
            va += __shfl_xor_sync(0xFFFFFFFFu, va, 1);
            vb += __shfl_xor_sync(0xFFFFFFFFu, vb, 1);
            if (t == 0) {
                float* r = red + ((buf * dd::kWarps + warp) * dd::kChunk + i) * 16;
                r[g] = va; r[g + 8] = vb;
            }
        }
        __syncthreads();
        if (tid < 16 * n_c) {
            const uint32_t i = tid >> 4, r = tid & 15u;
            float sum = 0.f;
#pragma unroll
            for (int w = 0; w < dd::kWarps; ++w)   // slot order, column blocks inside a slot
                sum += red[((buf * dd::kWarps + w) * dd::kChunk + i) * 16 + r];
            a.y[(size_t)tok * d.n_embd + (rt + i) * 16 + r] = sum;
        }
        buf ^= 1u;
        tile += n_c;
        rt += n_c;
        if (rt == RT) { rt = 0; ++tok; new_tok = true; }
    }
    if (timed_out && lane == 0) atomicExch(a.status, (uint32_t)kStatusWaitTimeout);
}

bool decode_down_ok(const qkm_dims& d) {
    return d.n_ff == dd::kMaxFf && d.n_used * (d.n_ff / 256) == dd::kWarps && d.n_embd % 32 == 0;
}

cudaError_t launch_decode_down(const Launch& L, const DownDecodeArgs& a, uint32_t n_blocks) {
    if (!decode_down_ok(a.d)) return cudaErrorInvalidValue;
    if (a.n_tokens == 0) return cudaSuccess;
    const size_t smem = dd::kEnd;
    cudaError_t e = cudaFuncSetAttribute(decode_down_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    e = launch_kernel(L, decode_down_kernel, dim3(n_blocks), dim3(dd::kWarps * 32), smem, a);
    L.count();
    return e != cudaSuccess ? e : cudaGetLastError();
}

}  // namespace qkm
