// Streaming gate/up + SwiGLU for small token counts (decode and short chunks).
//
// Replaces moe_gateup_iq3.comp / moe_gateup_iq3_rowtile.comp (routed experts, IQ3_XXS)
// and moe_gateup_q8.comp / moe_gateup_q8_64.comp (shared expert, Q8_0); because each
// selected expert is streamed once for all tokens that chose it, it also covers the
// "live expert union" grouping of the reference's multi-slot decode.
//
// Work is cut into items = (expert, 128-row chunk of n_ff, up to 2 tokens) and items
// into units of 32 rows.  The flat list of units is split evenly and contiguously over
// teams of KB = n_embd/256 warps; warp kb of a team streams the tiles of column block kb
// through a private bulk-copy ring, turns them into int8 MMA operands (an IQ3_XXS grid
// entry already is four packed magnitudes, Q8_0 bytes are used as they are) and
// multiplies them with the int8 digit planes of x on the tensor cores.  Integer partial
// sums are exact; sub-block scales are applied in integers (IQ3: 2s+1) or f32 (Q8_0: d),
// the digit weights in f32.  Column-block partials meet in shared memory, the team
// applies SwiGLU and writes h as f32 and as three bf16 pieces in the down kernel's
// operand order.
#include "qkm_kernels.h"
#include "qkm_stream.cuh"
#include "qkm_tiles.cuh"

namespace qkm {

// ---- x -> digit planes: one block per row (the fused router does this itself) ------------------
__global__ void __launch_bounds__(256)
encode_digits_kernel(const float* __restrict__ x, int8_t* __restrict__ planes, float* __restrict__ scale,
                     uint32_t K) {
    __shared__ float s_max[8];
    const uint32_t t = blockIdx.x;
    block_encode_digits(x + (size_t)t * K, planes + (size_t)t * 4 * K, scale + t, K, s_max);
}

cudaError_t launch_encode_digits(const Launch& L, const float* x, int8_t* planes, float* scale,
                                 uint32_t n_rows, uint32_t K) {
    if (n_rows == 0) return cudaSuccess;
    encode_digits_kernel<<<n_rows, 256, 0, L.stream>>>(x, planes, scale, K);
    L.count();
    return cudaGetLastError();
}

// ---- the streaming kernel ----------------------------------------------------------------------------------
namespace gu {
constexpr int kRowsPerItem = 128;
constexpr int kStages = 2;
constexpr uint32_t kGridLut = 32768;   // absolute shared-window addresses, 32 KB aligned so that
constexpr uint32_t kSignLut = 65536;   // (index << shift) | lane offset needs no add
constexpr uint32_t kLutEnd = 98304;

template <int FMT> struct Cfg;
// kUnitTiles: row tiles per unit of work.  The routed experts take 64-row units (fewer
// reductions and epilogues per weight); the shared expert has only n_ff rows per token pair and
// keeps 32-row units so that its work still spreads over the SMs.
template <> struct Cfg<QKM_TYPE_IQ3_XXS> {
    static constexpr int kWarps = 16, kTile = kTileIq3, kLowRingWarps = 4, kUnitTiles = 4;
    static constexpr bool kLuts = true;
};
template <> struct Cfg<QKM_TYPE_Q8_0> {
    static constexpr int kWarps = 8, kTile = kTileQ8, kLowRingWarps = 0, kUnitTiles = 2;
    static constexpr bool kLuts = false;
};
template <int FMT> constexpr int units_per_item() { return kRowsPerItem / (16 * Cfg<FMT>::kUnitTiles); }
template <int FMT> constexpr int red_floats() { return Cfg<FMT>::kUnitTiles * 16 * 2 * 2; }   // per warp: tile,row,token,matrix
}  // namespace gu

// One 16-row x 256-column tile of one matrix against the warp's B operand.
// Returns, for token slot t>>1, the partial dot of row g (va) and row g+8 (vb).
template <int FMT>
__device__ __forceinline__ void gu_tile(uint32_t tb, uint32_t lane, uint32_t g, uint32_t t, uint32_t grid_c,
                                        uint32_t sign_c, const uint32_t (&b0)[8], const uint32_t (&b1)[8],
                                        const uint32_t (&n0)[8], const uint32_t (&n1)[8], float wcol0,
                                        float wcol1, float& va, float& vb) {
    if (FMT == QKM_TYPE_IQ3_XXS) {
        const uint4 ia = lds128(tb + lane * 16);          // row g: 8 index pairs
        const uint4 ib_ = lds128(tb + 512 + lane * 16);   // row g+8
        const uint4 xa0 = lds128(tb + 1024 + 16 * g), xa1 = lds128(tb + 1280 + 16 * g);
        const uint4 xb0 = lds128(tb + 1152 + 16 * g), xb1 = lds128(tb + 1408 + 16 * g);
        const uint32_t idx_a[4] = {ia.x, ia.y, ia.z, ia.w}, idx_b[4] = {ib_.x, ib_.y, ib_.z, ib_.w};
        const uint32_t aux_a[8] = {xa0.x, xa0.y, xa0.z, xa0.w, xa1.x, xa1.y, xa1.z, xa1.w};
        const uint32_t aux_b[8] = {xb0.x, xb0.y, xb0.z, xb0.w, xb1.x, xb1.y, xb1.z, xb1.w};
        int acc[4] = {0, 0, 0, 0};
#pragma unroll
        for (int sb = 0; sb < 8; ++sb) {
            const uint32_t wa = idx_a[2 * (sb & 1) + (sb >> 2)], wb = idx_b[2 * (sb & 1) + (sb >> 2)];   // even sub-blocks in words 0,1; odd in 2,3
            uint32_t a_lo, a_hi, b_lo, b_hi;  // table addresses of the two grid entries per row
            if (sb & 2) {
                a_lo = ((wa >> 9) & 0x7F80u) | grid_c;  a_hi = ((wa >> 17) & 0x7F80u) | grid_c;
                b_lo = ((wb >> 9) & 0x7F80u) | grid_c;  b_hi = ((wb >> 17) & 0x7F80u) | grid_c;
            } else {
                a_lo = ((wa << 7) & 0x7F80u) | grid_c;  a_hi = ((wa >> 1) & 0x7F80u) | grid_c;
                b_lo = ((wb << 7) & 0x7F80u) | grid_c;  b_hi = ((wb >> 1) & 0x7F80u) | grid_c;
            }
            const uint32_t ga0 = lds32(a_lo), ga1 = lds32(a_hi), gb0 = lds32(b_lo), gb1 = lds32(b_hi);
            const uint32_t xa = aux_a[4 * (sb & 1) + (sb >> 1)], xb = aux_b[4 * (sb & 1) + (sb >> 1)];
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
        const float da = f16_bits_to_f32((lds32(tb + 1536 + 2 * (g & ~1u)) >> (16 * (g & 1u))) & 0xFFFFu);
        const float db = f16_bits_to_f32((lds32(tb + 1536 + 2 * ((g + 8) & ~1u)) >> (16 * (g & 1u))) & 0xFFFFu);
        // d * 0.25 * (2s+1) * m  ==  d * (0.5 + s) * 0.5 * m
        va = (da * 0.25f) * ((float)acc[0] * wcol0 + (float)acc[1] * wcol1);
        vb = (db * 0.25f) * ((float)acc[2] * wcol0 + (float)acc[3] * wcol1);
    } else {  // Q8_0: 8 blocks of 32 per row, raw int8 operands, one f16 scale per block
        float fa = 0.f, fb = 0.f;
#pragma unroll
        for (int blk = 0; blk < 8; ++blk) {
            const uint2 qa = lds64(tb + 544 * blk + 32 + lane * 8);
            const uint2 qb = lds64(tb + 544 * blk + 32 + 256 + lane * 8);
            int c[4] = {0, 0, 0, 0};
            mma_s8(c, qa.x, qb.x, qa.y, qb.y, b0[blk], b1[blk]);
            const uint32_t dw = lds32(tb + 544 * blk + 2 * (g & ~1u));       // d of rows g&~1, (g&~1)+1
            const uint32_t dw8 = lds32(tb + 544 * blk + 2 * (8 + (g & ~1u)));  // rows +8
            const float da = f16_bits_to_f32((dw >> (16 * (g & 1u))) & 0xFFFFu);
            const float db = f16_bits_to_f32((dw8 >> (16 * (g & 1u))) & 0xFFFFu);
            fa += da * ((float)c[0] * wcol0 + (float)c[1] * wcol1);
            fb += db * ((float)c[2] * wcol0 + (float)c[3] * wcol1);
        }
        va = fa; vb = fb;
    }
}

// Shared memory map (absolute shared-window addresses; the block asks for enough dynamic
// shared memory to cover everything up to the end of the reduction scratch).  IQ3_XXS:
//   [base, 32768)      barriers, then the rings of warps 0..3
//   [32768, 65536)     grid table, entry i lane l at 32768 + i*128 + l*4
//   [65536, 98304)     sign table, code c lane l at 65536 + c*256 + l*8: byte j of the
//                      64-bit entry is 0xFF when element j of the 8-group is negative
//   [98304, ...)       rings of warps 4..15, then the reduction scratch
// Q8_0 has no tables: barriers, rings, scratch follow each other from base.
template <int FMT>
__global__ void __launch_bounds__(gu::Cfg<FMT>::kWarps * 32, 1)
gateup_stream_kernel(const uint8_t* __restrict__ gate_tiles, const uint8_t* __restrict__ up_tiles,
                     const int8_t* __restrict__ xplanes, const float* __restrict__ xscale,
                     const uint32_t* __restrict__ pairs, const StreamItem* __restrict__ items,
                     const uint32_t* __restrict__ n_items_ptr, float* __restrict__ h,
                     __nv_bfloat16* __restrict__ hpieces, qkm_dims d, uint32_t* __restrict__ status) {
    using C = gu::Cfg<FMT>;
    constexpr int kStageBytes = 2 * C::kTile, kRingBytes = gu::kStages * kStageBytes;
    extern __shared__ __align__(128) uint8_t smem_raw[];
    const uint32_t base = smem_addr(smem_raw);
    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31u, g = lane >> 2, t = lane & 3u;
    const uint32_t KB = d.n_embd / 256;          // warps per team (2, 4 or 8)
    const uint32_t n_teams = C::kWarps / KB;
    const uint32_t team = warp / KB, kb = warp - team * KB;
    const uint32_t RT = d.n_ff / 16;             // row tiles per expert matrix
    pdl_trigger();

    const uint32_t bar_base = (base + 15u) & ~15u;                      // kWarps * kStages barriers
    const uint32_t low_ring = (bar_base + C::kWarps * gu::kStages * 8 + 127u) & ~127u;
    uint32_t ring, red_base;
    if (C::kLuts) {
        if (low_ring + C::kLowRingWarps * kRingBytes > gu::kGridLut) {  // layout assumption broken
            if (tid == 0) atomicExch(status, (uint32_t)kStatusBadLayout);
            return;
        }
        red_base = gu::kLutEnd + (C::kWarps - C::kLowRingWarps) * kRingBytes;
        ring = warp < (uint32_t)C::kLowRingWarps ? low_ring + warp * kRingBytes
                                                 : gu::kLutEnd + (warp - C::kLowRingWarps) * kRingBytes;
    } else {
        ring = low_ring + warp * kRingBytes;
        red_base = low_ring + C::kWarps * kRingBytes;
    }
    float* red = reinterpret_cast<float*>(smem_raw + (red_base - base));
    const uint32_t my_bar = bar_base + warp * gu::kStages * 8;

    if (C::kLuts) {
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
    }
    if (lane == 0) {
        for (int s = 0; s < gu::kStages; ++s) mbar_init(my_bar + 8 * s, 1);
        mbar_fence_init();
    }
    __syncthreads();
    pdl_wait();                                  // tables and barriers are set up; now the work lists may be read
    const uint32_t n_items = *n_items_ptr;

    // this team's contiguous share of the flat unit list
    const uint32_t teams_total = gridDim.x * n_teams, team_global = blockIdx.x * n_teams + team;
    const uint64_t units_total = (uint64_t)n_items * gu::units_per_item<FMT>();
    const uint32_t u_lo = (uint32_t)(units_total * team_global / teams_total);
    const uint32_t u_hi = (uint32_t)(units_total * (team_global + 1) / teams_total);
    const size_t mat_tiles = (size_t)KB * RT;

    // producer cursor over (unit, tile) of the same range; used by lane 0 only
    uint32_t p_unit = u_lo, p_tile = 0;
    auto issue = [&](uint32_t stage) {
        if (p_unit >= u_hi) return;
        const StreamItem it = items[p_unit / gu::units_per_item<FMT>()];
        const uint32_t rt = it.chunk * (gu::kRowsPerItem / 16) + (p_unit % gu::units_per_item<FMT>()) * gu::Cfg<FMT>::kUnitTiles + p_tile;
        const size_t tile = (size_t)it.expert * mat_tiles + (size_t)kb * RT + rt;
        const uint32_t bar = my_bar + 8 * stage, dst = ring + stage * kStageBytes;
        mbar_expect_tx(bar, kStageBytes);
        bulk_g2s(dst, gate_tiles + tile * C::kTile, C::kTile, bar);
        bulk_g2s(dst + C::kTile, up_tiles + tile * C::kTile, C::kTile, bar);
        if (++p_tile == gu::Cfg<FMT>::kUnitTiles) { p_tile = 0; ++p_unit; }
    };
    if (lane == 0)
        for (int s = 0; s < gu::kStages; ++s) issue(s);

    const uint32_t grid_c = gu::kGridLut + lane * 4, sign_c = gu::kSignLut + lane * 8;
    const uint32_t team_threads = KB * 32, lt = tid - team * team_threads;
    uint32_t cnt = 0;  // tiles consumed by this warp
    bool timed_out = false;
    uint32_t b0[8], b1[8], n0[8], n1[8];
    float wcol0 = 0.f, wcol1 = 0.f;  // digit weights of the two columns this lane's C holds (2t, 2t+1)
    uint32_t loaded_pair_off = 0xFFFFFFFFu, loaded_ntok = 0;

    for (uint32_t unit = u_lo; unit < u_hi; ++unit) {
        const StreamItem it = items[unit / gu::units_per_item<FMT>()];
        if (it.pair_off != loaded_pair_off || it.ntok != loaded_ntok) {
            // B operand: column g = (token slot g>>2, digit g&3); this warp's 256 columns
            loaded_pair_off = it.pair_off; loaded_ntok = it.ntok;
            const uint32_t ts = g >> 2, dg = g & 3u;
            if (ts < it.ntok) {
                const uint32_t tok = pairs[it.pair_off + ts] >> 4;
                const int8_t* pl = xplanes + (((size_t)tok * KB + kb) * 4 + dg) * 256;
#pragma unroll
                for (int sb = 0; sb < 8; ++sb) {
                    if (FMT == QKM_TYPE_IQ3_XXS) {   // lane t owns elements 8t..8t+7 of each sub-block
                        const uint2 v = *reinterpret_cast<const uint2*>(pl + 32 * sb + 8 * t);
                        b0[sb] = v.x; b1[sb] = v.y;
                    } else {                          // elements 4t..4t+3 and 16+4t..16+4t+3
                        b0[sb] = *reinterpret_cast<const uint32_t*>(pl + 32 * sb + 4 * t);
                        b1[sb] = *reinterpret_cast<const uint32_t*>(pl + 32 * sb + 16 + 4 * t);
                    }
                }
            } else {
#pragma unroll
                for (int sb = 0; sb < 8; ++sb) { b0[sb] = 0; b1[sb] = 0; }
            }
            if (FMT == QKM_TYPE_IQ3_XXS) {  // negated copies feed the "+1 per negative element" MMA
#pragma unroll
                for (int sb = 0; sb < 8; ++sb) { n0[sb] = __vneg4(b0[sb]); n1[sb] = __vneg4(b1[sb]); }
            }
            const uint32_t cts = t >> 1;  // token slot of columns 2t, 2t+1
            wcol0 = 0.f; wcol1 = 0.f;
            if (cts < it.ntok) {
                const float sc = xscale[pairs[it.pair_off + cts] >> 4];
                const float w0 = (t & 1u) ? 16384.f : 1.f;  // 128^(2*(t&1))
                wcol0 = sc * w0;
                wcol1 = sc * w0 * 128.f;
            }
        }
        float* my_red = red + warp * gu::red_floats<FMT>();
#pragma unroll 1
        for (int tile = 0; tile < gu::Cfg<FMT>::kUnitTiles; ++tile, ++cnt) {
            const uint32_t stage = cnt % gu::kStages, parity = (cnt / gu::kStages) & 1u;
            if (!mbar_wait_bounded(my_bar + 8 * stage, parity)) timed_out = true;
            const uint32_t sbase = ring + stage * kStageBytes;
            float ga, gb, ua, ub;
            gu_tile<FMT>(sbase, lane, g, t, grid_c, sign_c, b0, b1, n0, n1, wcol0, wcol1, ga, gb);
            gu_tile<FMT>(sbase + C::kTile, lane, g, t, grid_c, sign_c, b0, b1, n0, n1, wcol0, wcol1, ua, ub);
            __syncwarp();
            if (lane == 0) issue(stage);
            // the token's other two digits sit in lane t^1
            ga += __shfl_xor_sync(0xFFFFFFFFu, ga, 1); gb += __shfl_xor_sync(0xFFFFFFFFu, gb, 1);
            ua += __shfl_xor_sync(0xFFFFFFFFu, ua, 1); ub += __shfl_xor_sync(0xFFFFFFFFu, ub, 1);
            if ((t & 1u) == 0) {
                const uint32_t ts = t >> 1;  // [tile][row 16][token 2][matrix 2]
                float* r = my_red + (((tile * 16 + g) * 2 + ts) * 2);
                r[0] = ga; r[1] = ua;
                float* r8 = my_red + (((tile * 16 + g + 8) * 2 + ts) * 2);
                r8[0] = gb; r8[1] = ub;
            }
        }
        // team-wide: sum the KB column-block partials, SwiGLU, store
        asm volatile("bar.sync %0, %1;" ::"r"(team + 1), "r"(team_threads) : "memory");
        for (uint32_t j = lt; j < gu::Cfg<FMT>::kUnitTiles * 16 * 2; j += team_threads) {
            const uint32_t ts = j & 1u, row = j >> 1;  // row within the unit
            if (ts < it.ntok) {
                float gsum = 0.f, usum = 0.f;
                for (uint32_t w = 0; w < KB; ++w) {
                    const float* r = red + (team * KB + w) * gu::red_floats<FMT>() + (row * 2 + ts) * 2;
                    gsum += r[0]; usum += r[1];
                }
                const float hv = swiglu(gsum, usum);
                const uint32_t pr = pairs[it.pair_off + ts], tok = pr >> 4, slot = pr & 15u;
                const uint32_t r_ff = it.chunk * gu::kRowsPerItem + (unit % gu::units_per_item<FMT>()) * (16 * gu::Cfg<FMT>::kUnitTiles) + row;
                h[((size_t)tok * (d.n_used + 1) + slot) * d.n_ff + r_ff] = hv;
                // bf16 pieces in the down kernels' B-operand order: [token][slot][piece][sub-block][t][8]
                // with the 8 = elements (4t, 16+4t, 4t+1, 17+4t, 4t+2, 18+4t, 4t+3, 19+4t)
                __nv_bfloat16 p0, p1, p2;
                bf16_pieces(hv, p0, p1, p2);
                const uint32_t e32 = r_ff & 31u, tt = (e32 & 15u) >> 2, pos = 2 * (e32 & 3u) + (e32 >> 4);
                const size_t o = (((size_t)(tok * (d.n_used + 1) + slot) * 3) * (d.n_ff / 32) + (r_ff >> 5)) * 32 + tt * 8 + pos;
                hpieces[o] = p0; hpieces[o + d.n_ff] = p1; hpieces[o + 2 * (size_t)d.n_ff] = p2;
            }
        }
        asm volatile("bar.sync %0, %1;" ::"r"(team + 1), "r"(team_threads) : "memory");
    }
    if (timed_out && lane == 0) atomicExch(status, (uint32_t)kStatusWaitTimeout);
}

uint32_t gateup_stream_rows_per_item() { return gu::kRowsPerItem; }

template <int FMT>
static cudaError_t gateup_stream_launch(const Launch& L, const qkm_dims& d, const void* gate_tiles,
                                        const void* up_tiles, const int8_t* xplanes, const float* xscale,
                                        const uint32_t* pairs, const StreamItem* items, const uint32_t* n_items,
                                        float* h, void* hpieces, uint32_t n_blocks, uint32_t* status) {
    using C = gu::Cfg<FMT>;
    constexpr size_t kRings = (size_t)C::kWarps * gu::kStages * 2 * C::kTile;
    // the dynamic area must reach from wherever it starts (a few KB at most) to the end of
    // the reduction scratch
    const size_t smem = C::kLuts ? (size_t)gu::kLutEnd + (size_t)(C::kWarps - C::kLowRingWarps) * gu::kStages * 2 * C::kTile +
                                       (size_t)C::kWarps * gu::red_floats<FMT>() * 4
                                 : 1024 + kRings + (size_t)C::kWarps * gu::red_floats<FMT>() * 4;
    cudaError_t e = cudaFuncSetAttribute(gateup_stream_kernel<FMT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    e = launch_kernel(L, gateup_stream_kernel<FMT>, dim3(n_blocks), dim3(C::kWarps * 32), smem,
                      (const uint8_t*)gate_tiles, (const uint8_t*)up_tiles, xplanes, xscale, pairs, items, n_items, h,
                      (__nv_bfloat16*)hpieces, d, status);
    L.count();
    return e != cudaSuccess ? e : cudaGetLastError();
}

cudaError_t launch_gateup_stream(const Launch& L, const qkm_dims& d, uint32_t type, const void* gate_tiles,
                                 const void* up_tiles, const int8_t* xplanes, const float* xscale,
                                 const uint32_t* pairs, const StreamItem* items, const uint32_t* n_items,
                                 float* h, void* hpieces, uint32_t n_blocks, uint32_t* status) {
    const uint32_t KB = d.n_embd / 256;
    if (KB < 2 || KB > 8 || (KB & (KB - 1)) || d.n_ff % gu::kRowsPerItem || d.n_used > 15) return cudaErrorInvalidValue;
    if (type == QKM_TYPE_IQ3_XXS)
        return gateup_stream_launch<QKM_TYPE_IQ3_XXS>(L, d, gate_tiles, up_tiles, xplanes, xscale, pairs, items, n_items, h, hpieces, n_blocks, status);
    if (type == QKM_TYPE_Q8_0)
        return gateup_stream_launch<QKM_TYPE_Q8_0>(L, d, gate_tiles, up_tiles, xplanes, xscale, pairs, items, n_items, h, hpieces, n_blocks, status);
    return cudaErrorInvalidValue;
}

}  // namespace qkm
