// Streaming routed down projection for small token counts.
//
// Replaces moe_down_iq4.comp (and its _128 / rowtile tunings).  Items are (expert,
// 64-row chunk of n_embd, up to 2 tokens).  A team of n_ff/256 warps owns an item; each
// warp streams IQ4_XS tiles of its column block through a private four-stage bulk-copy
// ring.  A quant byte indexes a shared-memory table that returns the two codebook
// values of its nibbles as a packed bf16 pair - exactly one MMA A-operand register - and
// the expert's hidden row arrives as three bf16 pieces (exact 24-bit split) in the
// B-operand order, so products are exact and sums are f32 on the tensor cores.  The
// per-sub-block scale d*(ls-32) multiplies each 32-column partial; the routing weight
// multiplies the finished sum (as moe_down_iq4_grouped_coopmat.comp:160-161).  Results go
// to contrib[token][slot][n_embd]; a fold pass adds slots in order plus the shared expert.
#include "qkm_kernels.h"
#include "qkm_stream.cuh"
#include "qkm_tiles.cuh"

namespace qkm {

namespace dn {
constexpr int kWarps = 16;
constexpr int kStages = 4;
constexpr int kRowsPerItem = 64;
constexpr int kTilesPerItem = kRowsPerItem / 16;
constexpr uint32_t kLut = 32768;     // absolute shared-window address, 32 KB aligned
constexpr uint32_t kLutEnd = 65536;
constexpr int kRingBytes = kStages * kTileIq4;
constexpr int kLowRingWarps = 3;
constexpr int kRedFloats = kTilesPerItem * 16 * 2;  // per warp: tile,row,token
}  // namespace dn

__global__ void __launch_bounds__(dn::kWarps * 32, 1)
down_iq4_stream_kernel(const uint8_t* __restrict__ tiles, const __nv_bfloat16* __restrict__ hpieces,
                       const qkm_sel* __restrict__ sel, const uint32_t* __restrict__ pairs,
                       const StreamItem* __restrict__ items, const uint32_t* __restrict__ n_items_ptr,
                       float* __restrict__ contrib, qkm_dims d, uint32_t* __restrict__ status) {
    extern __shared__ __align__(128) uint8_t smem_raw[];
    const uint32_t base = smem_addr(smem_raw);
    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31u, g = lane >> 2, t = lane & 3u;
    const uint32_t KB = d.n_ff / 256;  // warps per team
    const uint32_t n_teams = dn::kWarps / KB;
    const uint32_t team = warp / KB, kb = warp - team * KB;
    const uint32_t RT = d.n_embd / 16;
    const uint32_t n_items = *n_items_ptr;

    const uint32_t bar_base = (base + 15u) & ~15u;
    const uint32_t low_ring = (bar_base + dn::kWarps * dn::kStages * 8 + 127u) & ~127u;
    if (low_ring + dn::kLowRingWarps * dn::kRingBytes > dn::kLut) {
        if (tid == 0) atomicExch(status, (uint32_t)kStatusBadLayout);
        return;
    }
    const uint32_t hi_ring = dn::kLutEnd;
    const uint32_t dl_base = hi_ring + (dn::kWarps - dn::kLowRingWarps) * dn::kRingBytes;  // 16 x 128 floats
    const uint32_t red_base = dl_base + dn::kWarps * 128 * 4;
    float* red = reinterpret_cast<float*>(smem_raw + (red_base - base));
    const uint32_t ring = warp < dn::kLowRingWarps ? low_ring + warp * dn::kRingBytes
                                                   : hi_ring + (warp - dn::kLowRingWarps) * dn::kRingBytes;
    const uint32_t my_bar = bar_base + warp * dn::kStages * 8;
    const uint32_t my_dl = dl_base + warp * 128 * 4;

    // table: quant byte -> (codebook[low nibble], codebook[high nibble]) as packed bf16
    for (uint32_t i = tid; i < 256 * 32; i += blockDim.x) {
        const uint32_t b = i >> 5;
        const __nv_bfloat16 lo = __float2bfloat16_rn((float)c_iq4_values[b & 15u]);
        const __nv_bfloat16 hi = __float2bfloat16_rn((float)c_iq4_values[b >> 4]);
        const uint32_t v = (uint32_t)__bfloat16_as_ushort(lo) | ((uint32_t)__bfloat16_as_ushort(hi) << 16);
        *reinterpret_cast<uint32_t*>(smem_raw + (dn::kLut - base) + i * 4) = v;
    }
    if (lane == 0) {
        for (int s = 0; s < dn::kStages; ++s) mbar_init(my_bar + 8 * s, 1);
        mbar_fence_init();
    }
    __syncthreads();

    const uint32_t team_global = blockIdx.x * n_teams + team, team_stride = gridDim.x * n_teams;
    const size_t mat_tiles = (size_t)KB * RT;

    uint32_t p_item = team_global, p_tile = 0;
    auto issue = [&](uint32_t stage) {
        if (p_item >= n_items) return;
        const StreamItem it = items[p_item];
        const size_t tile = (size_t)it.expert * mat_tiles + (size_t)kb * RT + (size_t)it.chunk * dn::kTilesPerItem + p_tile;
        const uint32_t bar = my_bar + 8 * stage;
        mbar_expect_tx(bar, kTileIq4);
        bulk_g2s(ring + stage * kTileIq4, tiles + tile * kTileIq4, kTileIq4, bar);
        if (++p_tile == dn::kTilesPerItem) { p_tile = 0; p_item += team_stride; }
    };
    if (lane == 0)
        for (int s = 0; s < dn::kStages; ++s) issue(s);

    const uint32_t lut_c = dn::kLut + lane * 4;
    uint32_t cnt = 0;
    bool timed_out = false;

    for (uint32_t item = team_global; item < n_items; item += team_stride) {
        const StreamItem it = items[item];
        // B operand: column g = (token slot g>>2, piece g&3), piece 3 unused
        uint32_t bq[8][4];
        {
            const uint32_t ts = g >> 2, piece = g & 3u;
            if (ts < it.ntok && piece < 3) {
                const __nv_bfloat16* src = hpieces + ((size_t)(it.pair_off + ts) * 3 + piece) * d.n_ff +
                                           ((size_t)(8 * kb) * 4 + t) * 8;
#pragma unroll
                for (int sb = 0; sb < 8; ++sb) {
                    const uint4 v = *reinterpret_cast<const uint4*>(src + (size_t)sb * 32);
                    bq[sb][0] = v.x; bq[sb][1] = v.y; bq[sb][2] = v.z; bq[sb][3] = v.w;
                }
            } else {
#pragma unroll
                for (int sb = 0; sb < 8; ++sb) { bq[sb][0] = 0; bq[sb][1] = 0; bq[sb][2] = 0; bq[sb][3] = 0; }
            }
        }
        float* my_red = red + warp * dn::kRedFloats;

        for (int tile = 0; tile < dn::kTilesPerItem; ++tile, ++cnt) {
            const uint32_t stage = cnt % dn::kStages, parity = (cnt / dn::kStages) & 1u;
            if (!mbar_wait_bounded(my_bar + 8 * stage, parity)) timed_out = true;
            const uint32_t tb = ring + stage * kTileIq4;
            // sub-block scales d*(ls-32): lane (g,t) computes rows g, g+8 x sub-blocks 2t, 2t+1
            {
                const uint4 hd = lds128(tb + 16 * g);  // row g: (d|sh<<16, sl), row g+8: same
                const float da = f16_bits_to_f32(hd.x & 0xFFFFu), db = f16_bits_to_f32(hd.z & 0xFFFFu);
                const uint32_t sha = hd.x >> 16, shb = hd.z >> 16;
#pragma unroll
                for (int j = 0; j < 2; ++j) {
                    const uint32_t sb = 2 * t + j;
                    const int lsa = (int)(((hd.y >> (4 * sb)) & 0xFu) | (((sha >> (2 * sb)) & 3u) << 4)) - 32;
                    const int lsb = (int)(((hd.w >> (4 * sb)) & 0xFu) | (((shb >> (2 * sb)) & 3u) << 4)) - 32;
                    float* dl = reinterpret_cast<float*>(smem_raw + (my_dl - base));
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
        const uint32_t team_threads = KB * 32;
        asm volatile("bar.sync %0, %1;" ::"r"(team + 1), "r"(team_threads) : "memory");
        const uint32_t lt = tid - team * team_threads;
        for (uint32_t j = lt; j < dn::kTilesPerItem * 16 * 2; j += team_threads) {
            const uint32_t ts = j & 1u, row = j >> 1;
            if (ts < it.ntok) {
                float sum = 0.f;
                for (uint32_t w = 0; w < KB; ++w) sum += red[(team * KB + w) * dn::kRedFloats + row * 2 + ts];
                const uint32_t pr = pairs[it.pair_off + ts], tok = pr >> 4, slot = pr & 15u;
                const uint32_t o = it.chunk * dn::kRowsPerItem + row;
                contrib[((size_t)tok * d.n_used + slot) * d.n_embd + o] = sel[tok].w[slot] * sum;
            }
        }
        asm volatile("bar.sync %0, %1;" ::"r"(team + 1), "r"(team_threads) : "memory");
    }
    if (timed_out && lane == 0) atomicExch(status, (uint32_t)kStatusWaitTimeout);
}

cudaError_t launch_down_stream(const Launch& L, const qkm_dims& d, uint32_t type, const void* tiles,
                               const void* hpieces, const qkm_sel* sel, const uint32_t* pairs,
                               const StreamItem* items, const uint32_t* n_items, float* contrib,
                               uint32_t n_sms, uint32_t* status) {
    if (type != QKM_TYPE_IQ4_XS) return cudaErrorInvalidValue;
    const uint32_t KB = d.n_ff / 256;
    if (KB < 2 || KB > 16 || (KB & (KB - 1)) || d.n_embd % dn::kRowsPerItem) return cudaErrorInvalidValue;
    const size_t smem = (size_t)dn::kLutEnd + (size_t)(dn::kWarps - dn::kLowRingWarps) * dn::kRingBytes +
                        (size_t)dn::kWarps * 128 * 4 + (size_t)dn::kWarps * dn::kRedFloats * 4;
    cudaError_t e = cudaFuncSetAttribute(down_iq4_stream_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    down_iq4_stream_kernel<<<n_sms, dn::kWarps * 32, smem, L.stream>>>(
        (const uint8_t*)tiles, (const __nv_bfloat16*)hpieces, sel, pairs, items, n_items, contrib, d, status);
    L.count();
    return cudaGetLastError();
}

uint32_t down_stream_rows_per_item() { return dn::kRowsPerItem; }

}  // namespace qkm
