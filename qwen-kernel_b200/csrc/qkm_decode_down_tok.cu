// Streaming routed down projection, token major: y[t] = sum_s w_s * D[ids_s] . h[t][s] + w_shared * y2[t].
//
// Replaces moe_down_iq4.comp together with the final "routed + shared" add.  A unit of
// work is (token, 16 output rows): the team that owns it walks the token's n_used experts
// in slot order, so the weighted sum over slots stays in registers, is added in a fixed
// order and is written once - no per-slot scratch, no cross-block reduction.  An expert
// chosen by several tokens is streamed once per token; the second visit is served by L2.
//
// Per slot a warp's ring stage receives two bulk copies: the three bf16 pieces of
// h[t][s] for its 256 columns (1536 B, already in MMA B-operand order) and the IQ4_XS
// tile of its column block (2176 B).  A quant byte indexes a shared-memory table of
// packed bf16 codebook pairs (one A-operand register each); products are exact, sums are
// f32 on the tensor cores; d*(ls-32) multiplies each 32-column partial.
#include "qkm_kernels.h"
#include "qkm_stream.cuh"
#include "qkm_tiles.cuh"

namespace qkm {

namespace dt {
constexpr int kWarps = 16;
constexpr int kStages = 3;
constexpr int kBBytes = 3 * 512;                 // three pieces x 256 columns x bf16
constexpr int kStageBytes = kBBytes + kTileIq4;  // 3712
constexpr int kRingBytes = kStages * kStageBytes;
constexpr uint32_t kLut = 32768, kLutEnd = 65536;
constexpr int kLowRingWarps = 2;
}  // namespace dt

__global__ void __launch_bounds__(dt::kWarps * 32, 1)
down_tok_iq4_kernel(const uint8_t* __restrict__ tiles, const __nv_bfloat16* __restrict__ hpieces,
                    const qkm_sel* __restrict__ sel, const float* __restrict__ y2, float* __restrict__ y,
                    uint32_t n_tokens, qkm_dims d, uint32_t* __restrict__ status) {
    extern __shared__ __align__(128) uint8_t smem_raw[];
    const uint32_t base = smem_addr(smem_raw);
    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31u, g = lane >> 2, t = lane & 3u;
    const uint32_t KB = d.n_ff / 256, n_teams = dt::kWarps / KB;
    const uint32_t team = warp / KB, kb = warp - team * KB;
    const uint32_t RT = d.n_embd / 16;  // row tiles = units per token
    pdl_trigger();

    const uint32_t bar_base = (base + 15u) & ~15u;
    const uint32_t low_ring = (bar_base + dt::kWarps * dt::kStages * 8 + 127u) & ~127u;
    if (low_ring + dt::kLowRingWarps * dt::kRingBytes > dt::kLut) {
        if (tid == 0) atomicExch(status, (uint32_t)kStatusBadLayout);
        return;
    }
    const uint32_t hi_ring = dt::kLutEnd;
    const uint32_t dl_base = hi_ring + (dt::kWarps - dt::kLowRingWarps) * dt::kRingBytes;  // 16 x 128 floats
    const uint32_t red_base = dl_base + dt::kWarps * 128 * 4;                               // 16 x 16 floats
    float* red = reinterpret_cast<float*>(smem_raw + (red_base - base));
    const uint32_t ring = warp < (uint32_t)dt::kLowRingWarps ? low_ring + warp * dt::kRingBytes
                                                             : hi_ring + (warp - dt::kLowRingWarps) * dt::kRingBytes;
    const uint32_t my_bar = bar_base + warp * dt::kStages * 8;
    const uint32_t my_dl = dl_base + warp * 128 * 4;

    for (uint32_t i = tid; i < 256 * 32; i += blockDim.x) {
        const uint32_t b = i >> 5;
        const __nv_bfloat16 lo = __float2bfloat16_rn((float)c_iq4_values[b & 15u]);
        const __nv_bfloat16 hi = __float2bfloat16_rn((float)c_iq4_values[b >> 4]);
        *reinterpret_cast<uint32_t*>(smem_raw + (dt::kLut - base) + i * 4) =
            (uint32_t)__bfloat16_as_ushort(lo) | ((uint32_t)__bfloat16_as_ushort(hi) << 16);
    }
    if (lane == 0) {
        for (int s = 0; s < dt::kStages; ++s) mbar_init(my_bar + 8 * s, 1);
        mbar_fence_init();
    }
    __syncthreads();
    pdl_wait();                         // the gate/up kernel's pieces and the selection are complete

    const uint32_t teams_total = gridDim.x * n_teams, team_global = blockIdx.x * n_teams + team;
    const uint64_t units_total = (uint64_t)n_tokens * RT;
    const uint32_t u_lo = (uint32_t)(units_total * team_global / teams_total);
    const uint32_t u_hi = (uint32_t)(units_total * (team_global + 1) / teams_total);
    const size_t mat_tiles = (size_t)KB * RT;
    const uint32_t n_slots = d.n_used + 1;

    // producer cursor over (unit, slot); lane 0 only
    uint32_t p_unit = u_lo, p_slot = 0;
    auto issue = [&](uint32_t stage) {
        if (p_unit >= u_hi) return;
        const uint32_t tok = p_unit / RT, rt = p_unit - tok * RT;
        const uint32_t e = min(sel[tok].ids[p_slot], d.n_expert - 1);
        const uint32_t bar = my_bar + 8 * stage, dst = ring + stage * dt::kStageBytes;
        const __nv_bfloat16* hp = hpieces + ((size_t)(tok * n_slots + p_slot) * 3) * d.n_ff + 256 * kb;
        mbar_expect_tx(bar, dt::kStageBytes);
        bulk_g2s(dst, hp, 512, bar);
        bulk_g2s(dst + 512, hp + d.n_ff, 512, bar);
        bulk_g2s(dst + 1024, hp + 2 * (size_t)d.n_ff, 512, bar);
        bulk_g2s(dst + dt::kBBytes, tiles + ((size_t)e * mat_tiles + (size_t)kb * RT + rt) * kTileIq4, kTileIq4, bar);
        if (++p_slot == d.n_used) { p_slot = 0; ++p_unit; }
    };
    if (lane == 0)
        for (int s = 0; s < dt::kStages; ++s) issue(s);

    const uint32_t lut_c = dt::kLut + lane * 4;
    const uint32_t team_threads = KB * 32, lt = tid - team * team_threads;
    uint32_t cnt = 0;
    bool timed_out = false;
    const bool b_lane = g < 3;  // column g = piece g of the (single) token; other columns are zero

    for (uint32_t unit = u_lo; unit < u_hi; ++unit) {
        const uint32_t tok = unit / RT, rt = unit - tok * RT;
        float yacc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll 1
        for (uint32_t s = 0; s < d.n_used; ++s, ++cnt) {
            const uint32_t stage = cnt % dt::kStages, parity = (cnt / dt::kStages) & 1u;
            if (!mbar_wait_bounded(my_bar + 8 * stage, parity)) timed_out = true;
            const uint32_t sb0 = ring + stage * dt::kStageBytes, tb = sb0 + dt::kBBytes;
            const float wgt = sel[tok].w[s];
            uint32_t bq[8][4];
#pragma unroll
            for (int sb = 0; sb < 8; ++sb) {
                uint4 v = make_uint4(0, 0, 0, 0);
                if (b_lane) v = lds128(sb0 + g * 512 + (sb * 4 + t) * 16);
                bq[sb][0] = v.x; bq[sb][1] = v.y; bq[sb][2] = v.z; bq[sb][3] = v.w;
            }
            // sub-block scales d*(ls-32): lane (g,t) computes rows g, g+8 x sub-blocks 2t, 2t+1
            {
                const uint4 hd = lds128(tb + 16 * g);
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
            float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int half = 0; half < 2; ++half) {
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
            // routing weight after the full column reduction of this warp's block
            yacc[0] += wgt * acc[0]; yacc[1] += wgt * acc[1];
            yacc[2] += wgt * acc[2]; yacc[3] += wgt * acc[3];
        }
        // pieces: columns 0,1 in lane t=0, column 2 in lane t=1
        float va = yacc[0] + yacc[1], vb = yacc[2] + yacc[3];
        va += __shfl_xor_sync(0xFFFFFFFFu, va, 1);
        vb += __shfl_xor_sync(0xFFFFFFFFu, vb, 1);
        if (t == 0) { red[warp * 16 + g] = va; red[warp * 16 + g + 8] = vb; }
        asm volatile("bar.sync %0, %1;" ::"r"(team + 1), "r"(team_threads) : "memory");
        if (lt < 16) {
            float sum = 0.f;
            for (uint32_t w = 0; w < KB; ++w) sum += red[(team * KB + w) * 16 + lt];
            const size_t o = (size_t)tok * d.n_embd + rt * 16 + lt;
            // y2 holds the shared expert's down projection without its gate weight
            y[o] = sum + (y2 != nullptr ? sel[tok].w_shared * y2[o] : 0.f);
        }
        asm volatile("bar.sync %0, %1;" ::"r"(team + 1), "r"(team_threads) : "memory");
    }
    if (timed_out && lane == 0) atomicExch(status, (uint32_t)kStatusWaitTimeout);
}

cudaError_t launch_down_tok(const Launch& L, const qkm_dims& d, uint32_t type, const void* tiles,
                            const void* hpieces, const qkm_sel* sel, const float* y2, float* y,
                            uint32_t n_tokens, uint32_t n_blocks, uint32_t* status) {
    const uint32_t KB = d.n_ff / 256;
    if (type != QKM_TYPE_IQ4_XS || KB < 2 || KB > 16 || (KB & (KB - 1)) || d.n_used > 15) return cudaErrorInvalidValue;
    if (n_tokens == 0) return cudaSuccess;
    const size_t smem = (size_t)dt::kLutEnd + (size_t)(dt::kWarps - dt::kLowRingWarps) * dt::kRingBytes +
                        (size_t)dt::kWarps * 128 * 4 + (size_t)dt::kWarps * 16 * 4 + 256;
    cudaError_t e = cudaFuncSetAttribute(down_tok_iq4_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    e = launch_kernel(L, down_tok_iq4_kernel, dim3(n_blocks), dim3(dt::kWarps * 32), smem, (const uint8_t*)tiles,
                      (const __nv_bfloat16*)hpieces, sel, y2, y, n_tokens, d, status);
    L.count();
    return e != cudaSuccess ? e : cudaGetLastError();
}

}  // namespace qkm
