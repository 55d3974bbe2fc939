// Streaming gate/up + SwiGLU for small token counts (decode and short chunks).
//
// Replaces moe_gateup_iq3.comp / moe_gateup_iq3_rowtile.comp and, because each
// selected expert is streamed once for all tokens that chose it, the "live expert
// union" grouping of the reference's multi-slot decode.
//
// Work is cut into items = (expert, 128-row chunk of n_ff, up to 2 tokens).  A team of
// KB = n_embd/256 warps owns an item; warp kb streams the tiles of column block kb
// through a private two-stage bulk-copy ring, decodes IQ3_XXS straight into int8 MMA
// operands (a grid entry already is four packed magnitudes) and multiplies them with
// the int8 digit planes of x on the tensor cores.  Integer partial sums are exact; the
// sub-block scale (2s+1) is applied in integers, d*0.25 and the digit weights in f32
// once per 256 columns.  Column-block partials meet in shared memory, the team applies
// SwiGLU and writes h as f32 and as three bf16 pieces in the down kernel's operand order.
#include "qkm_kernels.h"
#include "qkm_stream.cuh"
#include "qkm_tiles.cuh"

namespace qkm {

// ---- x -> digit planes: one block per token ---------------------------------------------------
__global__ void __launch_bounds__(256)
encode_digits_kernel(const float* __restrict__ x, int8_t* __restrict__ planes, float* __restrict__ scale,
                     uint32_t K) {
    __shared__ float s_max[8];
    const uint32_t t = blockIdx.x, tid = threadIdx.x;
    const float* xt = x + (size_t)t * K;
    float m = 0.f;
    bool bad = false;
    for (uint32_t k = tid; k < K; k += 256) {
        const float v = xt[k];
        bad |= !(fabsf(v) <= 3.0e38f);
        m = fmaxf(m, fabsf(v));
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xFFFFFFFFu, m, o));
    const int any_bad = __syncthreads_or(bad ? 1 : 0);
    if ((tid & 31u) == 0) s_max[tid >> 5] = m;
    __syncthreads();
    m = s_max[0];
#pragma unroll
    for (int w = 1; w < 8; ++w) m = fmaxf(m, s_max[w]);
    const int p = digit_exponent(m);
    const float up = ldexpf(1.0f, p);
    int8_t* pl = planes + (size_t)t * 4 * K;
    for (uint32_t k = tid; k < K; k += 256) {
        const uint32_t d = any_bad ? 0u : digits4(__float2int_rn(xt[k] * up));
        pl[k] = (int8_t)(d & 255u);
        pl[K + k] = (int8_t)((d >> 8) & 255u);
        pl[2 * (size_t)K + k] = (int8_t)((d >> 16) & 255u);
        pl[3 * (size_t)K + k] = (int8_t)(d >> 24);
    }
    // a row holding NaN/Inf has no finite encoding: its outputs become NaN
    if (tid == 0) scale[t] = any_bad ? __int_as_float(0x7FC00000) : ldexpf(1.0f, -p);
}

cudaError_t launch_encode_digits(const Launch& L, const float* x, int8_t* planes, float* scale,
                                 uint32_t n_rows, uint32_t K) {
    if (n_rows == 0) return cudaSuccess;
    encode_digits_kernel<<<n_rows, 256, 0, L.stream>>>(x, planes, scale, K);
    L.count();
    return cudaGetLastError();
}

// ---- work list: (expert, chunk, token pair) items from the grouped pairs ----------------------------
__global__ void __launch_bounds__(512)
plan_items_kernel(const uint32_t* __restrict__ offsets, uint32_t n_expert_local, uint32_t n_chunks,
                  uint32_t tok_per_item, StreamItem* __restrict__ items, uint32_t* __restrict__ n_items) {
    __shared__ uint32_t s_scan[512];
    const uint32_t e = threadIdx.x;
    uint32_t groups = 0;
    if (e < n_expert_local) groups = (offsets[e + 1] - offsets[e] + tok_per_item - 1) / tok_per_item;
    s_scan[e] = groups;
    __syncthreads();
    for (uint32_t o = 1; o < 512; o <<= 1) {  // inclusive scan
        const uint32_t v = e >= o ? s_scan[e - o] : 0;
        __syncthreads();
        s_scan[e] += v;
        __syncthreads();
    }
    const uint32_t first = (s_scan[e] - groups) * n_chunks;
    if (e < n_expert_local) {
        const uint32_t p0 = offsets[e], n = offsets[e + 1] - p0;
        for (uint32_t gidx = 0; gidx < groups; ++gidx)
            for (uint32_t c = 0; c < n_chunks; ++c) {
                StreamItem it;
                it.expert = (uint16_t)e;
                it.chunk = (uint8_t)c;
                it.ntok = (uint8_t)min(tok_per_item, n - gidx * tok_per_item);
                it.pair_off = p0 + gidx * tok_per_item;
                // chunk-major inside an expert keeps the teams that share an expert close in time
                items[first + gidx * n_chunks + c] = it;
            }
    }
    if (e == 511) *n_items = s_scan[511] * n_chunks;
}

cudaError_t launch_plan_items(const Launch& L, const uint32_t* offsets, uint32_t n_expert_local,
                              uint32_t n_chunks, uint32_t tok_per_item, StreamItem* items, uint32_t* n_items) {
    if (n_expert_local > 512) return cudaErrorInvalidValue;
    plan_items_kernel<<<1, 512, 0, L.stream>>>(offsets, n_expert_local, n_chunks, tok_per_item, items, n_items);
    L.count();
    return cudaGetLastError();
}

// ---- the streaming kernel ----------------------------------------------------------------------------------
namespace gu {
constexpr int kWarps = 16;           // per block
constexpr int kStages = 2;           // ring depth per warp
constexpr int kRowsPerItem = 128;    // 8 tiles of 16 rows
constexpr int kTilesPerItem = kRowsPerItem / 16;
constexpr uint32_t kGridLut = 32768;   // absolute shared-window addresses: 32 KB aligned so that
constexpr uint32_t kSignLut = 65536;   // (index << shift) | lane offset needs no add
constexpr uint32_t kLutEnd = 98304;
constexpr int kStageBytes = 2 * kTileIq3;                  // gate tile + up tile
constexpr int kRingBytes = kStages * kStageBytes;          // per warp
constexpr int kRedFloats = kTilesPerItem * 16 * 2 * 2;     // per warp: tile,row,token,matrix
constexpr int kLowRingWarps = 4;                           // rings that fit below the tables
}  // namespace gu

// Shared memory map (absolute shared-window addresses; the block asks for enough dynamic
// shared memory that everything up to the end of the reduction scratch is covered):
//   [base, 32768)      barriers, then the rings of warps 0..3
//   [32768, 65536)     grid table, entry i lane l at 32768 + i*128 + l*4
//   [65536, 98304)     sign table, code c lane l at 65536 + c*256 + l*8: byte j of the
//                      64-bit entry is 0xFF when element j of the 8-group is negative
//   [98304, ...)       rings of warps 4..15, then the reduction scratch
__global__ void __launch_bounds__(gu::kWarps * 32, 1)
gateup_iq3_stream_kernel(const uint8_t* __restrict__ gate_tiles, const uint8_t* __restrict__ up_tiles,
                         const int8_t* __restrict__ xplanes, const float* __restrict__ xscale,
                         const uint32_t* __restrict__ pairs, const StreamItem* __restrict__ items,
                         const uint32_t* __restrict__ n_items_ptr, float* __restrict__ h,
                         __nv_bfloat16* __restrict__ hpieces, qkm_dims d, uint32_t* __restrict__ status) {
    extern __shared__ __align__(128) uint8_t smem_raw[];
    const uint32_t base = smem_addr(smem_raw);
    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31u, g = lane >> 2, t = lane & 3u;
    const uint32_t KB = d.n_embd / 256;          // warps per team (1, 2, 4, 8 or 16)
    const uint32_t n_teams = gu::kWarps / KB;
    const uint32_t team = warp / KB, kb = warp - team * KB;
    const uint32_t RT = d.n_ff / 16;             // row tiles per expert matrix
    const uint32_t n_items = *n_items_ptr;

    const uint32_t bar_base = (base + 15u) & ~15u;                      // kWarps * kStages barriers
    const uint32_t low_ring = (bar_base + gu::kWarps * gu::kStages * 8 + 127u) & ~127u;
    if (low_ring + gu::kLowRingWarps * gu::kRingBytes > gu::kGridLut) {  // layout assumption broken
        if (tid == 0) atomicExch(status, (uint32_t)kStatusBadLayout);
        return;
    }
    const uint32_t red_base = gu::kLutEnd + (gu::kWarps - gu::kLowRingWarps) * gu::kRingBytes;
    float* red = reinterpret_cast<float*>(smem_raw + (red_base - base));
    const uint32_t ring = warp < gu::kLowRingWarps ? low_ring + warp * gu::kRingBytes
                                                    : gu::kLutEnd + (warp - gu::kLowRingWarps) * gu::kRingBytes;
    const uint32_t my_bar = bar_base + warp * gu::kStages * 8;

    // tables
    for (uint32_t i = tid; i < 256 * 32; i += blockDim.x)
        *reinterpret_cast<uint32_t*>(smem_raw + (gu::kGridLut - base) + i * 4) = c_iq3_grid[i >> 5];
    for (uint32_t i = tid; i < 128 * 32; i += blockDim.x) {
        const uint32_t sg = signs8(i >> 5);
        uint32_t lo = 0, hi = 0;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            lo |= ((sg >> j) & 1u) ? (0xFFu << (8 * j)) : 0u;
            hi |= ((sg >> (j + 4)) & 1u) ? (0xFFu << (8 * j)) : 0u;
        }
        *reinterpret_cast<uint2*>(smem_raw + (gu::kSignLut - base) + i * 8) = make_uint2(lo, hi);
    }
    if (lane == 0) {
        for (int s = 0; s < gu::kStages; ++s) mbar_init(my_bar + 8 * s, 1);
        mbar_fence_init();
    }
    __syncthreads();

    const uint32_t team_global = blockIdx.x * n_teams + team, team_stride = gridDim.x * n_teams;
    const size_t mat_tiles = (size_t)KB * RT;  // tiles per expert matrix

    // producer cursor (lane 0 only uses it)
    uint32_t p_item = team_global, p_tile = 0;
    auto issue = [&](uint32_t stage) {
        if (p_item >= n_items) return;
        const StreamItem it = items[p_item];
        const size_t tile = ((size_t)it.expert * mat_tiles + (size_t)kb * RT + (size_t)it.chunk * gu::kTilesPerItem + p_tile);
        const uint32_t bar = my_bar + 8 * stage, dst = ring + stage * gu::kStageBytes;
        mbar_expect_tx(bar, gu::kStageBytes);
        bulk_g2s(dst, gate_tiles + tile * kTileIq3, kTileIq3, bar);
        bulk_g2s(dst + kTileIq3, up_tiles + tile * kTileIq3, kTileIq3, bar);
        if (++p_tile == gu::kTilesPerItem) { p_tile = 0; p_item += team_stride; }
    };
    if (lane == 0)
        for (int s = 0; s < gu::kStages; ++s) issue(s);

    const uint32_t grid_c = gu::kGridLut + lane * 4, sign_c = gu::kSignLut + lane * 8;
    uint32_t cnt = 0;  // tiles consumed by this warp
    bool timed_out = false;

    for (uint32_t item = team_global; item < n_items; item += team_stride) {
        const StreamItem it = items[item];
        // B operand: column g = (token slot g>>2, digit g&3); this warp's 256 columns
        uint32_t b0[8], b1[8], n0[8], n1[8];
        float wcol0 = 0.f, wcol1 = 0.f;  // digit weights of the two columns this lane's C holds (2t, 2t+1)
        {
            const uint32_t ts = g >> 2, dg = g & 3u;
            if (ts < it.ntok) {
                const uint32_t tok = pairs[it.pair_off + ts] >> 4;
                const int8_t* pl = xplanes + ((size_t)tok * 4 + dg) * d.n_embd + 256 * kb + 8 * t;
#pragma unroll
                for (int ib = 0; ib < 8; ++ib) {
                    const uint2 v = *reinterpret_cast<const uint2*>(pl + 32 * ib);
                    b0[ib] = v.x; b1[ib] = v.y;
                }
            } else {
#pragma unroll
                for (int ib = 0; ib < 8; ++ib) { b0[ib] = 0; b1[ib] = 0; }
            }
            // negated copies feed the "+1 per negative element" correction MMA
#pragma unroll
            for (int ib = 0; ib < 8; ++ib) {
                n0[ib] = __vneg4(b0[ib]);
                n1[ib] = __vneg4(b1[ib]);
            }
            const uint32_t cts = t >> 1;  // token slot of columns 2t, 2t+1
            if (cts < it.ntok) {
                const uint32_t tok = pairs[it.pair_off + cts] >> 4;
                const float sc = xscale[tok];
                const float w0 = (t & 1u) ? 16384.f : 1.f;  // 128^(2*(t&1))
                wcol0 = sc * w0;
                wcol1 = sc * w0 * 128.f;
            }
        }
        float* my_red = red + warp * gu::kRedFloats;

        for (int tile = 0; tile < gu::kTilesPerItem; ++tile, ++cnt) {
            const uint32_t stage = cnt % gu::kStages, parity = (cnt / gu::kStages) & 1u;
            if (!mbar_wait_bounded(my_bar + 8 * stage, parity)) timed_out = true;
            const uint32_t sbase = ring + stage * gu::kStageBytes;
            float part[4];  // (gate,row g) (gate,row g+8) (up,row g) (up,row g+8) for token slot t>>1
#pragma unroll
            for (int mat = 0; mat < 2; ++mat) {
                const uint32_t tb = sbase + mat * kTileIq3;
                const uint4 ia = lds128(tb + lane * 16);          // row g: 8 index pairs
                const uint4 ib_ = lds128(tb + 512 + lane * 16);   // row g+8
                const uint4 xa0 = lds128(tb + 1024 + 32 * g), xa1 = lds128(tb + 1024 + 32 * g + 16);
                const uint4 xb0 = lds128(tb + 1024 + 32 * (g + 8)), xb1 = lds128(tb + 1024 + 32 * (g + 8) + 16);
                const uint32_t idx_a[4] = {ia.x, ia.y, ia.z, ia.w}, idx_b[4] = {ib_.x, ib_.y, ib_.z, ib_.w};
                const uint32_t aux_a[8] = {xa0.x, xa0.y, xa0.z, xa0.w, xa1.x, xa1.y, xa1.z, xa1.w};
                const uint32_t aux_b[8] = {xb0.x, xb0.y, xb0.z, xb0.w, xb1.x, xb1.y, xb1.z, xb1.w};
                int acc[4] = {0, 0, 0, 0};
#pragma unroll
                for (int sb = 0; sb < 8; ++sb) {
                    const uint32_t wa = idx_a[sb >> 1], wb = idx_b[sb >> 1];
                    uint32_t a_lo, a_hi, b_lo, b_hi;  // table addresses of the two grid entries per row
                    if (sb & 1) {
                        a_lo = ((wa >> 9) & 0x7F80u) | grid_c;  a_hi = ((wa >> 17) & 0x7F80u) | grid_c;
                        b_lo = ((wb >> 9) & 0x7F80u) | grid_c;  b_hi = ((wb >> 17) & 0x7F80u) | grid_c;
                    } else {
                        a_lo = ((wa << 7) & 0x7F80u) | grid_c;  a_hi = ((wa >> 1) & 0x7F80u) | grid_c;
                        b_lo = ((wb << 7) & 0x7F80u) | grid_c;  b_hi = ((wb >> 1) & 0x7F80u) | grid_c;
                    }
                    const uint32_t ga0 = lds32(a_lo), ga1 = lds32(a_hi), gb0 = lds32(b_lo), gb1 = lds32(b_hi);
                    const uint32_t xa = aux_a[sb], xb = aux_b[sb];
                    const uint2 ma = lds64((((xa >> (7 * t)) & 127u) << 8) | sign_c);
                    const uint2 mb = lds64((((xb >> (7 * t)) & 127u) << 8) | sign_c);
                    int c[4] = {0, 0, 0, 0};
                    // m ^ 0xFF = -m-1 for negative elements; the second MMA adds the missing +1 * x
                    // (A = 0xFF = -1 where negative, B = -digits)
                    mma_s8(c, ga0 ^ ma.x, gb0 ^ mb.x, ga1 ^ ma.y, gb1 ^ mb.y, b0[sb], b1[sb]);
                    mma_s8(c, ma.x, mb.x, ma.y, mb.y, n0[sb], n1[sb]);
                    const int qa = (int)(2u * (xa >> 28) + 1u), qb = (int)(2u * (xb >> 28) + 1u);
                    acc[0] += qa * c[0]; acc[1] += qa * c[1];
                    acc[2] += qb * c[2]; acc[3] += qb * c[3];
                }
                const float da = f16_bits_to_f32(lds32(tb + 1536 + 2 * (g & ~1u)) >> (16 * (g & 1u)) & 0xFFFFu);
                const float db = f16_bits_to_f32(lds32(tb + 1536 + 2 * ((g + 8) & ~1u)) >> (16 * (g & 1u)) & 0xFFFFu);
                // d * 0.25 * (2s+1) * m  ==  d * (0.5 + s) * 0.5 * m
                float va = (da * 0.25f) * ((float)acc[0] * wcol0 + (float)acc[1] * wcol1);
                float vb = (db * 0.25f) * ((float)acc[2] * wcol0 + (float)acc[3] * wcol1);
                va += __shfl_xor_sync(0xFFFFFFFFu, va, 1);   // the token's other two digits
                vb += __shfl_xor_sync(0xFFFFFFFFu, vb, 1);
                part[2 * mat] = va; part[2 * mat + 1] = vb;
            }
            __syncwarp();
            if (lane == 0) issue(stage);
            if ((t & 1u) == 0) {
                const uint32_t ts = t >> 1;
                // [tile][row 16][token 2][matrix 2]
                float* r = my_red + (((tile * 16 + g) * 2 + ts) * 2);
                r[0] = part[0]; r[1] = part[2];
                float* r8 = my_red + (((tile * 16 + g + 8) * 2 + ts) * 2);
                r8[0] = part[1]; r8[1] = part[3];
            }
        }
        // team-wide: sum the KB column-block partials, SwiGLU, store
        const uint32_t team_threads = KB * 32;
        asm volatile("bar.sync %0, %1;" ::"r"(team + 1), "r"(team_threads) : "memory");
        const uint32_t lt = tid - team * team_threads;  // 0 .. team_threads-1
        for (uint32_t j = lt; j < gu::kTilesPerItem * 16 * 2; j += team_threads) {
            const uint32_t ts = j & 1u, row = j >> 1;  // row within the 128-row chunk
            if (ts < it.ntok) {
                float gsum = 0.f, usum = 0.f;
                for (uint32_t w = 0; w < KB; ++w) {
                    const float* r = red + (team * KB + w) * gu::kRedFloats + (row * 2 + ts) * 2;
                    gsum += r[0]; usum += r[1];
                }
                const float hv = swiglu(gsum, usum);
                const uint32_t pr = pairs[it.pair_off + ts], tok = pr >> 4, slot = pr & 15u;
                const uint32_t r_ff = it.chunk * gu::kRowsPerItem + row;
                h[((size_t)tok * (d.n_used + 1) + slot) * d.n_ff + r_ff] = hv;
                // bf16 pieces in the down kernel's B-operand order:
                // [pair][piece][kb][sub-block][t][8] with the 8 = elements (4t, 16+4t, 4t+1, 17+4t, ...)
                __nv_bfloat16 p0, p1, p2;
                bf16_pieces(hv, p0, p1, p2);
                const uint32_t e32 = r_ff & 31u, tt = (e32 & 15u) >> 2, pos = 2 * (e32 & 3u) + (e32 >> 4);
                const size_t o = ((((size_t)(it.pair_off + ts) * 3) * (d.n_ff / 32) + (r_ff >> 5)) * 4 + tt) * 8 + pos;
                const size_t piece_stride = (size_t)(d.n_ff / 32) * 32;
                hpieces[o] = p0; hpieces[o + piece_stride] = p1; hpieces[o + 2 * piece_stride] = p2;
            }
        }
        asm volatile("bar.sync %0, %1;" ::"r"(team + 1), "r"(team_threads) : "memory");
    }
    if (timed_out && lane == 0) atomicExch(status, (uint32_t)kStatusWaitTimeout);
}

uint32_t gateup_stream_rows_per_item() { return gu::kRowsPerItem; }

size_t gateup_stream_smem_bytes() {
    // the dynamic area must reach from wherever it starts (a few KB at most) to the end of
    // the reduction scratch
    return (size_t)gu::kLutEnd + (size_t)(gu::kWarps - gu::kLowRingWarps) * gu::kRingBytes +
           (size_t)gu::kWarps * gu::kRedFloats * 4;
}

cudaError_t launch_gateup_stream(const Launch& L, const qkm_dims& d, uint32_t type, const void* gate_tiles,
                                 const void* up_tiles, const int8_t* xplanes, const float* xscale,
                                 const uint32_t* pairs, const StreamItem* items, const uint32_t* n_items,
                                 float* h, void* hpieces, uint32_t n_sms, uint32_t* status) {
    if (type != QKM_TYPE_IQ3_XXS) return cudaErrorInvalidValue;
    const uint32_t KB = d.n_embd / 256;
    if (KB < 2 || KB > 16 || (KB & (KB - 1)) || d.n_ff % gu::kRowsPerItem) return cudaErrorInvalidValue;
    const size_t smem = gateup_stream_smem_bytes();
    cudaError_t e = cudaFuncSetAttribute(gateup_iq3_stream_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    gateup_iq3_stream_kernel<<<n_sms, gu::kWarps * 32, smem, L.stream>>>(
        (const uint8_t*)gate_tiles, (const uint8_t*)up_tiles, xplanes, xscale, pairs, items, n_items, h,
        (__nv_bfloat16*)hpieces, d, status);
    L.count();
    return cudaGetLastError();
}

}  // namespace qkm
