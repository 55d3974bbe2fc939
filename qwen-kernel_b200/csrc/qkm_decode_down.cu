// Streaming down projection for small token counts, with the slot fold fused in.
//
// Replaces moe_down_iq4.comp (routed experts, IQ4_XS), moe_down_q8b.comp (shared
// expert, Q8_0) and the "routed slots in order, then shared" sum of
// add_rms3_grouped.comp:22-27.
//
// Items are (expert, 64-row chunk of n_embd, up to 2 tokens), cut into units of 32 rows;
// the flat unit list is split evenly over teams of n_ff/256 warps.  Each warp streams the
// tiles of its column block through a private bulk-copy ring.  A quant byte indexes a
// shared-memory table that returns MMA-ready bf16: for IQ4_XS the two codebook values of
// its nibbles (one A-operand register), for Q8_0 the value itself.  The expert's hidden
// row arrives as three bf16 pieces (an exact 24-bit split) in B-operand order, so products
// are exact and sums are f32 on the tensor cores.  Sub-block scales multiply each
// 32-column partial; the routing weight multiplies the finished sum (as
// moe_down_iq4_grouped_coopmat.comp:160-161).  Each (token, slot) contribution is written
// to contrib[token][slot][n_embd]; the team that delivers the last of a token's
// n_used + 1 contributions for a 32-row unit folds them, slots in order, into y.
#include "qkm_kernels.h"
#include "qkm_stream.cuh"
#include "qkm_tiles.cuh"

namespace qkm {

namespace dn {
constexpr int kWarps = 16;
constexpr int kRowsPerItem = 64;
constexpr int kUnitTiles = 2;
constexpr int kUnitRows = 16 * kUnitTiles;
constexpr int kUnitsPerItem = kRowsPerItem / kUnitRows;
constexpr uint32_t kLut = 32768;     // absolute shared-window address, 32 KB aligned
constexpr uint32_t kLutEnd = 65536;
constexpr int kLowRingWarps = 3;
constexpr int kRedFloats = kUnitTiles * 16 * 2;  // per warp: tile,row,token
template <int FMT> struct Cfg;
template <> struct Cfg<QKM_TYPE_IQ4_XS> { static constexpr int kTile = kTileIq4, kStages = 4; };
template <> struct Cfg<QKM_TYPE_Q8_0> { static constexpr int kTile = kTileQ8, kStages = 2; };
}  // namespace dn

template <int FMT>
__global__ void __launch_bounds__(dn::kWarps * 32, 1)
down_stream_kernel(const uint8_t* __restrict__ tiles, const __nv_bfloat16* __restrict__ hpieces,
                   const qkm_sel* __restrict__ sel, const uint32_t* __restrict__ pairs,
                   const StreamItem* __restrict__ items, const uint32_t* __restrict__ n_items_ptr,
                   float* __restrict__ contrib, float* __restrict__ y, uint32_t* __restrict__ arrivals,
                   qkm_dims d, uint32_t* __restrict__ status) {
    using C = dn::Cfg<FMT>;
    constexpr int kRingBytes = C::kStages * C::kTile;
    extern __shared__ __align__(128) uint8_t smem_raw[];
    const uint32_t base = smem_addr(smem_raw);
    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31u, g = lane >> 2, t = lane & 3u;
    const uint32_t KB = d.n_ff / 256;  // warps per team
    const uint32_t n_teams = dn::kWarps / KB;
    const uint32_t team = warp / KB, kb = warp - team * KB;
    const uint32_t RT = d.n_embd / 16;
    const uint32_t n_items = *n_items_ptr;
    const uint32_t n_slots = d.n_used + 1;  // routed slots + the shared expert

    const uint32_t bar_base = (base + 15u) & ~15u;
    const uint32_t low_ring = (bar_base + dn::kWarps * C::kStages * 8 + 127u) & ~127u;
    if (low_ring + dn::kLowRingWarps * kRingBytes > dn::kLut) {
        if (tid == 0) atomicExch(status, (uint32_t)kStatusBadLayout);
        return;
    }
    const uint32_t hi_ring = dn::kLutEnd;
    const uint32_t dl_base = hi_ring + (dn::kWarps - dn::kLowRingWarps) * kRingBytes;  // 16 x 128 floats
    const uint32_t red_base = dl_base + dn::kWarps * 128 * 4;
    const uint32_t flag_base = red_base + dn::kWarps * dn::kRedFloats * 4;             // per team: 2 flags
    float* red = reinterpret_cast<float*>(smem_raw + (red_base - base));
    uint32_t* flags = reinterpret_cast<uint32_t*>(smem_raw + (flag_base - base));
    const uint32_t ring = warp < (uint32_t)dn::kLowRingWarps ? low_ring + warp * kRingBytes
                                                             : hi_ring + (warp - dn::kLowRingWarps) * kRingBytes;
    const uint32_t my_bar = bar_base + warp * C::kStages * 8;
    const uint32_t my_dl = dl_base + warp * 128 * 4;

    // table, entry b lane l at kLut + b*128 + l*4.
    //   IQ4_XS: (codebook[b & 15], codebook[b >> 4]) as a packed bf16 pair
    //   Q8_0:   bf16(int8(b)) in both halves
    for (uint32_t i = tid; i < 256 * 32; i += blockDim.x) {
        const uint32_t b = i >> 5;
        uint32_t v;
        if (FMT == QKM_TYPE_IQ4_XS) {
            const __nv_bfloat16 lo = __float2bfloat16_rn((float)c_iq4_values[b & 15u]);
            const __nv_bfloat16 hi = __float2bfloat16_rn((float)c_iq4_values[b >> 4]);
            v = (uint32_t)__bfloat16_as_ushort(lo) | ((uint32_t)__bfloat16_as_ushort(hi) << 16);
        } else {
            const uint32_t q = __bfloat16_as_ushort(__float2bfloat16_rn((float)(int8_t)b));
            v = q | (q << 16);
        }
        *reinterpret_cast<uint32_t*>(smem_raw + (dn::kLut - base) + i * 4) = v;
    }
    if (lane == 0) {
        for (int s = 0; s < C::kStages; ++s) mbar_init(my_bar + 8 * s, 1);
        mbar_fence_init();
    }
    __syncthreads();

    const uint32_t teams_total = gridDim.x * n_teams, team_global = blockIdx.x * n_teams + team;
    const uint64_t units_total = (uint64_t)n_items * dn::kUnitsPerItem;
    const uint32_t u_lo = (uint32_t)(units_total * team_global / teams_total);
    const uint32_t u_hi = (uint32_t)(units_total * (team_global + 1) / teams_total);
    const size_t mat_tiles = (size_t)KB * RT;

    uint32_t p_unit = u_lo, p_tile = 0;
    auto issue = [&](uint32_t stage) {
        if (p_unit >= u_hi) return;
        const StreamItem it = items[p_unit / dn::kUnitsPerItem];
        const uint32_t rt = it.chunk * (dn::kRowsPerItem / 16) + (p_unit % dn::kUnitsPerItem) * dn::kUnitTiles + p_tile;
        const size_t tile = (size_t)it.expert * mat_tiles + (size_t)kb * RT + rt;
        const uint32_t bar = my_bar + 8 * stage;
        mbar_expect_tx(bar, C::kTile);
        bulk_g2s(ring + stage * C::kTile, tiles + tile * C::kTile, C::kTile, bar);
        if (++p_tile == dn::kUnitTiles) { p_tile = 0; ++p_unit; }
    };
    if (lane == 0)
        for (int s = 0; s < C::kStages; ++s) issue(s);

    const uint32_t lut_c = dn::kLut + lane * 4;
    const uint32_t team_threads = KB * 32, lt = tid - team * team_threads;
    uint32_t cnt = 0;
    bool timed_out = false;
    uint32_t bq[8][4];
    uint32_t loaded_pair_off = 0xFFFFFFFFu, loaded_ntok = 0;

    for (uint32_t unit = u_lo; unit < u_hi; ++unit) {
        const StreamItem it = items[unit / dn::kUnitsPerItem];
        if (it.pair_off != loaded_pair_off || it.ntok != loaded_ntok) {
            // B operand: column g = (token slot g>>2, piece g&3), piece 3 unused
            loaded_pair_off = it.pair_off; loaded_ntok = it.ntok;
            const uint32_t ts = g >> 2, piece = g & 3u;
            if (ts < it.ntok && piece < 3) {
                const uint32_t pr = pairs[it.pair_off + ts];
                const __nv_bfloat16* src = hpieces + ((size_t)((pr >> 4) * n_slots + (pr & 15u)) * 3 + piece) * d.n_ff +
                                           ((size_t)(8 * kb) * 4 + t) * 8;
#pragma unroll
                for (int sb = 0; sb < 8; ++sb) {
                    const uint4 v = __ldcg(reinterpret_cast<const uint4*>(src + (size_t)sb * 32));
                    bq[sb][0] = v.x; bq[sb][1] = v.y; bq[sb][2] = v.z; bq[sb][3] = v.w;
                }
            } else {
#pragma unroll
                for (int sb = 0; sb < 8; ++sb) { bq[sb][0] = 0; bq[sb][1] = 0; bq[sb][2] = 0; bq[sb][3] = 0; }
            }
        }
        float* my_red = red + warp * dn::kRedFloats;

#pragma unroll 1
        for (int tile = 0; tile < dn::kUnitTiles; ++tile, ++cnt) {
            const uint32_t stage = cnt % C::kStages, parity = (cnt / C::kStages) & 1u;
            if (!mbar_wait_bounded(my_bar + 8 * stage, parity)) timed_out = true;
            const uint32_t tb = ring + stage * C::kTile;
            float acc[4] = {0.f, 0.f, 0.f, 0.f};
            if (FMT == QKM_TYPE_IQ4_XS) {
                // sub-block scales d*(ls-32): lane (g,t) computes rows g, g+8 x sub-blocks 2t, 2t+1
                {
                    const uint4 hd = lds128(tb + 16 * g);  // row g: (d|sh<<16, sl), row g+8: same
                    const float da = f16_bits_to_f32(hd.x & 0xFFFFu), db = f16_bits_to_f32(hd.z & 0xFFFFu);
                    const uint32_t sha = hd.x >> 16, shb = hd.z >> 16;
                    float* dl = reinterpret_cast<float*>(smem_raw + (my_dl - base));
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
#pragma unroll
                for (int half = 0; half < 2; ++half) {
                    // chunk c = 2*rowhalf + half: row g (+8), sub-blocks 4*half .. 4*half+3, word t of each
                    const uint4 qa = lds128(tb + 128 + ((half)*32 + lane) * 16);
                    const uint4 qb = lds128(tb + 128 + ((2 + half) * 32 + lane) * 16);
                    const uint32_t wa[4] = {qa.x, qa.y, qa.z, qa.w}, wb[4] = {qb.x, qb.y, qb.z, qb.w};
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const int sb = 4 * half + j;
                        const uint32_t a = wa[j], b = wb[j];
                        const uint32_t a0 = lds32(((a << 7) & 0x7F80u) | lut_c), a1 = lds32(((a >> 1) & 0x7F80u) | lut_c);
                        const uint32_t a2 = lds32(((a >> 9) & 0x7F80u) | lut_c), a3 = lds32(((a >> 17) & 0x7F80u) | lut_c);
                        const uint32_t b0 = lds32(((b << 7) & 0x7F80u) | lut_c), b1 = lds32(((b >> 1) & 0x7F80u) | lut_c);
                        const uint32_t b2 = lds32(((b >> 9) & 0x7F80u) | lut_c), b3 = lds32(((b >> 17) & 0x7F80u) | lut_c);
                        float c[4] = {0.f, 0.f, 0.f, 0.f};
                        mma_bf16(c, a0, b0, a1, b1, bq[sb][0], bq[sb][1]);
                        mma_bf16(c, a2, b2, a3, b3, bq[sb][2], bq[sb][3]);
                        acc[0] += dla[sb] * c[0]; acc[1] += dla[sb] * c[1];
                        acc[2] += dlb[sb] * c[2]; acc[3] += dlb[sb] * c[3];
                    }
                }
            } else {  // Q8_0: 8 blocks of 32 per row
#pragma unroll
                for (int blk = 0; blk < 8; ++blk) {
                    const uint2 qa = lds64(tb + 544 * blk + 32 + lane * 8);  // row g: qs[4t..], qs[16+4t..]
                    const uint2 qb = lds64(tb + 544 * blk + 32 + 256 + lane * 8);  // row g+8
                    uint32_t ar[4], br[4];  // per byte j: (q[4t+j], q[16+4t+j]) as a bf16 pair
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const int sh = 8 * j - 7;
                        const uint32_t xa = sh < 0 ? (qa.x << 7) : (qa.x >> sh), ya = sh < 0 ? (qa.y << 7) : (qa.y >> sh);
                        const uint32_t xb = sh < 0 ? (qb.x << 7) : (qb.x >> sh), yb = sh < 0 ? (qb.y << 7) : (qb.y >> sh);
                        const uint32_t la = lds32((xa & 0x7F80u) | lut_c), ha = lds32((ya & 0x7F80u) | lut_c);
                        const uint32_t lb = lds32((xb & 0x7F80u) | lut_c), hb = lds32((yb & 0x7F80u) | lut_c);
                        ar[j] = (la & 0xFFFFu) | (ha & 0xFFFF0000u);
                        br[j] = (lb & 0xFFFFu) | (hb & 0xFFFF0000u);
                    }
                    float c[4] = {0.f, 0.f, 0.f, 0.f};
                    mma_bf16(c, ar[0], br[0], ar[1], br[1], bq[blk][0], bq[blk][1]);
                    mma_bf16(c, ar[2], br[2], ar[3], br[3], bq[blk][2], bq[blk][3]);
                    const uint32_t dw = lds32(tb + 544 * blk + 2 * (g & ~1u));
                    const uint32_t dw8 = lds32(tb + 544 * blk + 2 * (8 + (g & ~1u)));
                    const float da = f16_bits_to_f32((dw >> (16 * (g & 1u))) & 0xFFFFu);
                    const float db = f16_bits_to_f32((dw8 >> (16 * (g & 1u))) & 0xFFFFu);
                    acc[0] += da * c[0]; acc[1] += da * c[1];
                    acc[2] += db * c[2]; acc[3] += db * c[3];
                }
            }
            __syncwarp();
            if (lane == 0) issue(stage);
            // columns 2t, 2t+1 belong to token slot t>>1; the other pieces sit in lane t^1
            float va = acc[0] + acc[1], vb = acc[2] + acc[3];
            va += __shfl_xor_sync(0xFFFFFFFFu, va, 1);
            vb += __shfl_xor_sync(0xFFFFFFFFu, vb, 1);
            if ((t & 1u) == 0) {
                const uint32_t ts = t >> 1;
                my_red[(tile * 16 + g) * 2 + ts] = va;
                my_red[(tile * 16 + g + 8) * 2 + ts] = vb;
            }
        }
        // ---- unit epilogue: contributions out, then fold where this team delivered the last one
        const uint32_t row0 = it.chunk * dn::kRowsPerItem + (unit % dn::kUnitsPerItem) * dn::kUnitRows;
        const uint32_t unit_idx = row0 / dn::kUnitRows, units_per_row = d.n_embd / dn::kUnitRows;
        asm volatile("bar.sync %0, %1;" ::"r"(team + 1), "r"(team_threads) : "memory");
        for (uint32_t j = lt; j < dn::kUnitRows * 2; j += team_threads) {
            const uint32_t ts = j & 1u, row = j >> 1;
            if (ts < it.ntok) {
                float sum = 0.f;
                for (uint32_t w = 0; w < KB; ++w) sum += red[(team * KB + w) * dn::kRedFloats + row * 2 + ts];
                const uint32_t pr = pairs[it.pair_off + ts], tok = pr >> 4, slot = pr & 15u;
                // sel == NULL: the caller applies the weight (lets this kernel run before the routing is known)
                const float wgt = sel == nullptr ? 1.f : (slot < d.n_used ? sel[tok].w[slot] : sel[tok].w_shared);
                if (arrivals != nullptr) contrib[((size_t)tok * n_slots + slot) * d.n_embd + row0 + row] = wgt * sum;
                else y[(size_t)tok * d.n_embd + row0 + row] = wgt * sum;   // single-slot use: y is this slot's term
            }
        }
        if (arrivals != nullptr) {
            __threadfence();
            asm volatile("bar.sync %0, %1;" ::"r"(team + 1), "r"(team_threads) : "memory");
            if (lt < it.ntok) {
                const uint32_t tok = pairs[it.pair_off + lt] >> 4;
                const uint32_t old = atomicAdd(&arrivals[(size_t)tok * units_per_row + unit_idx], 1u);
                const bool last = old + 1 == n_slots;
                if (last) arrivals[(size_t)tok * units_per_row + unit_idx] = 0;  // ready for the next call
                flags[team * 2 + lt] = last ? 1u : 0u;
            }
            asm volatile("bar.sync %0, %1;" ::"r"(team + 1), "r"(team_threads) : "memory");
            for (uint32_t ts = 0; ts < it.ntok; ++ts) {
                if (flags[team * 2 + ts] == 0) continue;
                __threadfence();
                const uint32_t tok = pairs[it.pair_off + ts] >> 4;
                for (uint32_t row = lt; row < dn::kUnitRows; row += team_threads) {
                    const float* cp = contrib + (size_t)tok * n_slots * d.n_embd + row0 + row;
                    float part[16];
#pragma unroll
                    for (int s = 0; s < 16; ++s) part[s] = (uint32_t)s < n_slots ? __ldcg(cp + (size_t)s * d.n_embd) : 0.f;
                    float v = 0.f;
#pragma unroll
                    for (int s = 0; s < 16; ++s) v += part[s];  // slots in order, the shared expert last
                    y[(size_t)tok * d.n_embd + row0 + row] = v;
                }
            }
        }
        asm volatile("bar.sync %0, %1;" ::"r"(team + 1), "r"(team_threads) : "memory");
    }
    if (timed_out && lane == 0) atomicExch(status, (uint32_t)kStatusWaitTimeout);
}

uint32_t down_stream_rows_per_item() { return dn::kRowsPerItem; }
uint32_t down_stream_unit_rows() { return dn::kUnitRows; }

template <int FMT>
static cudaError_t down_stream_launch(const Launch& L, const qkm_dims& d, const void* tiles, const void* hpieces,
                                      const qkm_sel* sel, const uint32_t* pairs, const StreamItem* items,
                                      const uint32_t* n_items, float* contrib, float* y, uint32_t* arrivals,
                                      uint32_t n_blocks, uint32_t* status) {
    using C = dn::Cfg<FMT>;
    const size_t smem = (size_t)dn::kLutEnd + (size_t)(dn::kWarps - dn::kLowRingWarps) * C::kStages * C::kTile +
                        (size_t)dn::kWarps * 128 * 4 + (size_t)dn::kWarps * dn::kRedFloats * 4 + 256;
    cudaError_t e = cudaFuncSetAttribute(down_stream_kernel<FMT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    down_stream_kernel<FMT><<<n_blocks, dn::kWarps * 32, smem, L.stream>>>(
        (const uint8_t*)tiles, (const __nv_bfloat16*)hpieces, sel, pairs, items, n_items, contrib, y, arrivals, d, status);
    L.count();
    return cudaGetLastError();
}

cudaError_t launch_down_stream(const Launch& L, const qkm_dims& d, uint32_t type, const void* tiles,
                               const void* hpieces, const qkm_sel* sel, const uint32_t* pairs,
                               const StreamItem* items, const uint32_t* n_items, float* contrib, float* y,
                               uint32_t* arrivals, uint32_t n_blocks, uint32_t* status) {
    const uint32_t KB = d.n_ff / 256;
    if (KB < 2 || KB > 16 || (KB & (KB - 1)) || d.n_embd % dn::kRowsPerItem || d.n_used > 15) return cudaErrorInvalidValue;
    if (type == QKM_TYPE_IQ4_XS)
        return down_stream_launch<QKM_TYPE_IQ4_XS>(L, d, tiles, hpieces, sel, pairs, items, n_items, contrib, y, arrivals, n_blocks, status);
    if (type == QKM_TYPE_Q8_0)
        return down_stream_launch<QKM_TYPE_Q8_0>(L, d, tiles, hpieces, sel, pairs, items, n_items, contrib, y, arrivals, n_blocks, status);
    return cudaErrorInvalidValue;
}

}  // namespace qkm
