// Down projection of the fused decode sequence for layers whose routed down tensor is Q6_K
// (moe_down_q6k.comp + moe_down_q8b.comp + the "routed + shared" add in one persistent launch):
//   y[t] = sum_s w_s * D[ids_s] . h[t][s]  +  w_shared * DS . h[t][n_used].
//
// Same organisation as the IQ4_XS kernel: a unit of work is (token, 16 output rows) and belongs to
// the whole block; warp (slot s, column block kb) streams the 16-row tiles of expert ids_s through a
// private ring of bulk copies (TMA, no tensor map, no multicast); the block adds the eight slots in
// slot order.  A Q6_K tile is 3360 bytes, so a stage holds one tile (not two) and the ring has
// three stages; the flat list of (token, tile) is cut evenly and contiguously over the blocks.
//
// Arithmetic: exact integers until the last step.  h[t][s] becomes four int8 digit planes per
// 256-column block (28-bit fixed point, one power-of-two scale).  A 6-bit quant q goes into the
// top six bits of a byte, with its top bit flipped: as int8 that byte is 4 * (q - 32), so no sign
// extension is computed - three word operations per four weights (a shift of the nibbles, a shift
// of the bit pairs, one three-input logic op) plus five per sixteen for the masks.  The scales are
// per 16 columns: one m16n8k32 MMA multiplies two 16-column groups at once, the first against
// B columns 0..3 (the four digits; zero in the second group's k range) and the second against
// columns 4..7, so all eight B columns work and lane t multiplies its two sums by ONE int8 scale
// (group t / 2) as integers.  d, the digit weights, the plane scale, the factor 1/4 and the
// routing weight are applied once per tile in f32.
//
// Shared expert: warp w also takes 32-column block w of the Q8_0 matrix for the tile's rows.
#include "qkm_kernels.h"
#include "qkm_stream.cuh"
#include "qkm_tiles.cuh"

namespace qkm {

namespace dq {
constexpr int kWarps = 16;
constexpr int kStages = 3;
constexpr int kShBlock = 544;                       // one Q8_0 block column of a 16-row tile: d, quants
constexpr int kStageBytes = kTileQ6 + kShBlock;     // 3904
constexpr int kRingBytes = kStages * kStageBytes;
constexpr int kChunk = 4;                           // tiles between two block-wide sums
constexpr uint32_t kMaxFf = 512;
// dynamic shared memory, offsets from a 128-byte aligned base
constexpr uint32_t kBars = 0;                                              // kWarps * kStages mbarriers
constexpr uint32_t kRings = 1024;
constexpr uint32_t kDig = kRings + kWarps * kRingBytes;                    // per warp: 4 digit planes x 256 B, natural order
constexpr uint32_t kRed = kDig + kWarps * 1024;                            // [2 buffers][16 warps][kChunk tiles][16 rows]
constexpr uint32_t kHd = kRed + 2 * kWarps * kChunk * 16 * 4;              // 4 digit planes x 512 of h[t][n_used]
constexpr uint32_t kMisc = kHd + 4 * kMaxFf;                               // 16 warp maxima
constexpr uint32_t kEnd = kMisc + 128;
}  // namespace dq

__device__ __forceinline__ uint32_t prmt_dq(uint32_t a, uint32_t b, uint32_t sel) {
    uint32_t r;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(sel));
    return r;
}

// Sixteen Q6_K weights as four int8 MMA A-operand registers, each 4 * (q - 32): w1 / w2 are the ql
// words of elements l..l+3 in the first / second 32-byte run of a half, hq the qh word of the same
// l; r[qd] holds elements l + 32 * qd .. + 3  (src/quants.h:148-163).
__device__ __forceinline__ void q6k_words(uint32_t w1, uint32_t w2, uint32_t hq, uint32_t (&r)[4]) {
    const uint32_t hx = hq ^ 0xAAAAAAAAu;          // top bit of every pair flipped: the sign of q - 32
    const uint32_t lo1 = w1 & 0x0F0F0F0Fu, hi1 = w1 & 0xF0F0F0F0u;
    const uint32_t lo2 = w2 & 0x0F0F0F0Fu, hi2 = w2 & 0xF0F0F0F0u;
    r[0] = ((hx << 6) & 0xC0C0C0C0u) | (lo1 << 2);
    r[1] = ((hx << 4) & 0xC0C0C0C0u) | (lo2 << 2);
    r[2] = ((hx << 2) & 0xC0C0C0C0u) | (hi1 >> 2);
    r[3] = (hx & 0xC0C0C0C0u) | (hi2 >> 2);
}

__global__ void __launch_bounds__(dq::kWarps * 32, 1)
decode_down_q6k_kernel(DownDecodeArgs a) {
    extern __shared__ __align__(128) uint8_t smem_raw[];
    uint8_t* sm = reinterpret_cast<uint8_t*>(((uintptr_t)smem_raw + 127) & ~(uintptr_t)127);
    const uint32_t base = smem_addr(sm);
    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31u, g = lane >> 2, t = lane & 3u;
    const qkm_dims d = a.d;
    const uint32_t KB = d.n_ff / 256;               // 2
    const uint32_t slot = warp / KB, kb = warp - slot * KB;
    const uint32_t RT = d.n_embd / 16;              // row tiles of the down matrix
    const uint32_t n_slots = d.n_used + 1;
    const bool with_shared = a.sh_tiles != nullptr;

    const uint32_t ring = base + dq::kRings + warp * dq::kRingBytes;
    const uint32_t my_bar = base + dq::kBars + warp * dq::kStages * 8;
    const uint32_t my_dig = base + dq::kDig + warp * 1024;
    uint8_t* dig = sm + dq::kDig + warp * 1024;
    float* red = reinterpret_cast<float*>(sm + dq::kRed);
    int8_t* s_hd = reinterpret_cast<int8_t*>(sm + dq::kHd);
    float* s_misc = reinterpret_cast<float*>(sm + dq::kMisc);
    bool timed_out = false;

    if (lane == 0) {
        for (int s = 0; s < dq::kStages; ++s) mbar_init(my_bar + 8 * s, 1);
        mbar_fence_init();
    }
    __syncthreads();

    const uint64_t tiles_total = (uint64_t)a.n_tokens * RT;
    const uint32_t u_lo = (uint32_t)(tiles_total * blockIdx.x / gridDim.x);
    const uint32_t u_hi = (uint32_t)(tiles_total * (blockIdx.x + 1) / gridDim.x);
    const size_t mat_tiles = (size_t)KB * RT;

    // producer cursor; lane 0 only
    uint32_t p_u = u_lo, p_tok = u_lo / RT, p_rt = u_lo - p_tok * RT;
    bool p_new_tok = true;
    const uint8_t* p_src = nullptr;     // next tile of expert ids[slot]
    const uint8_t* p_sh = nullptr;      // block column `warp` of the next tile of the shared matrix
    auto issue = [&](uint32_t stage) {
        if (p_u >= u_hi) return;
        if (p_new_tok) {
            p_new_tok = false;
            const uint32_t e = min(__ldcg(&a.sel[p_tok].ids[slot]), d.n_expert - 1);
            p_src = a.tiles + ((size_t)e * mat_tiles + (size_t)kb * RT + p_rt) * kTileQ6;
            if (with_shared) p_sh = a.sh_tiles + ((size_t)(warp >> 3) * RT + p_rt) * kTileQ8 + dq::kShBlock * (warp & 7u);
        }
        const uint32_t bar = my_bar + 8 * stage, dst = ring + stage * dq::kStageBytes;
        mbar_expect_tx(bar, kTileQ6 + (with_shared ? dq::kShBlock : 0));
        bulk_g2s(dst, p_src, kTileQ6, bar);
        p_src += kTileQ6;
        if (with_shared) {
            bulk_g2s(dst + kTileQ6, p_sh, dq::kShBlock, bar);
            p_sh += kTileQ8;
        }
        ++p_u;
        if (++p_rt == RT) { p_rt = 0; ++p_tok; p_new_tok = true; }
    };
    if (lane == 0)
        for (int s = 0; s < dq::kStages; ++s) issue(s);
    // The first weight tiles are on their way (they depend on the selection only, which was final
    // before the gate/up kernel released this one); h is that kernel's output.
    pdl_wait();
    pdl_trigger();

    uint32_t cnt = 0, buf = 0;
    float w_s = 0.f, w_sh = 0.f;   // routing weight x plane scale / 4 of this warp's slot; w_shared x 2^-p of the shared row's digits
    // B operand of MMA j = 4 hf + qd: lanes g < 4 hold digit g of the first 16-column group in b0 (b1 = 0),
    // lanes g >= 4 digit g - 4 of the second group in b1 (b0 = 0)
    uint32_t b0[8], b1[8];
    // C columns 2t, 2t+1 are digits 2 (t & 1), 2 (t & 1) + 1 of group t / 2
    const float dw0 = (t & 1u) ? 16384.f : 1.f, dw1 = dw0 * 128.f;
    const float dws0 = t == 0 ? 1.f : (t == 1 ? 16384.f : 0.f), dws1 = dws0 * 128.f;   // the shared expert's MMA: digits in columns 0..3 only

    uint32_t tok = u_lo / RT, rt = u_lo - tok * RT;
    bool new_tok = true;
    for (uint32_t u = u_lo; u < u_hi;) {
        if (new_tok) {   // block-uniform
            new_tok = false;
            const float* hs = a.h + ((size_t)tok * n_slots + slot) * d.n_ff + 256 * kb + 8 * lane;
            const float4 v0 = *reinterpret_cast<const float4*>(hs), v1 = *reinterpret_cast<const float4*>(hs + 4);
            const float w_slot = a.sel[tok].w[slot];
            w_sh = a.sel[tok].w_shared;
            const float hv_sh = (with_shared && tid < d.n_ff) ? a.h[((size_t)tok * n_slots + d.n_used) * d.n_ff + tid] : 0.f;
            {
                const float hv[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
                float m = 0.f;
                bool bad = false;
#pragma unroll
                for (int i = 0; i < 8; ++i) { m = fmaxf(m, fabsf(hv[i])); bad |= !(fabsf(hv[i]) <= 3.0e38f); }
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xFFFFFFFFu, m, o));
                const bool any_bad = __any_sync(0xFFFFFFFFu, bad);
                const int p = digit_exponent(m);
                const float up = ldexpf(1.0f, p);
                uint32_t dg[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) dg[i] = any_bad ? 0u : digits4(__float2int_rn(hv[i] * up));
                __syncwarp();
                // plane j of elements 8 lane .. 8 lane + 7: byte j of each packed word
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const uint32_t sel = 0x4040u + 0x1111u * j;   // byte j of a, byte j of b, twice
                    const uint32_t p01 = prmt_dq(dg[0], dg[1], sel), p23 = prmt_dq(dg[2], dg[3], sel);
                    const uint32_t p45 = prmt_dq(dg[4], dg[5], sel), p67 = prmt_dq(dg[6], dg[7], sel);
                    *reinterpret_cast<uint2*>(dig + 256 * j + 8 * lane) =
                        make_uint2(prmt_dq(p01, p23, 0x5410u), prmt_dq(p45, p67, 0x5410u));
                }
                __syncwarp();
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const uint32_t v = lds32(my_dig + (g & 3u) * 256 + 32 * j + 16 * (g >> 2) + 4 * t);
                    b0[j] = g < 4 ? v : 0u;
                    b1[j] = g < 4 ? 0u : v;
                }
                w_s = w_slot * (any_bad ? __int_as_float(0x7FC00000) : ldexpf(0.25f, -p));
            }
            if (with_shared) {
                const float hv = hv_sh;
                float m = fabsf(hv);
                const bool bad = !(m <= 3.0e38f);
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xFFFFFFFFu, m, o));
                const int any_bad = __syncthreads_or(bad ? 1 : 0);
                if (lane == 0) s_misc[warp] = m;
                __syncthreads();
                float mx = 0.f;
#pragma unroll
                for (int w = 0; w < dq::kWarps; ++w) mx = fmaxf(mx, s_misc[w]);
                const int p = digit_exponent(mx);
                if (tid < d.n_ff) {
                    const uint32_t dgt = any_bad ? 0u : digits4(__float2int_rn(hv * ldexpf(1.0f, p)));
                    s_hd[tid] = (int8_t)(dgt & 255u);
                    s_hd[dq::kMaxFf + tid] = (int8_t)((dgt >> 8) & 255u);
                    s_hd[2 * dq::kMaxFf + tid] = (int8_t)((dgt >> 16) & 255u);
                    s_hd[3 * dq::kMaxFf + tid] = (int8_t)(dgt >> 24);
                }
                w_sh *= any_bad ? __int_as_float(0x7FC00000) : ldexpf(1.0f, -p);
                __syncthreads();
            }
        }
        const uint32_t n_c = min((uint32_t)dq::kChunk, min(u_hi - u, RT - rt));   // tiles of this chunk
        uint32_t hb0 = 0, hb1 = 0;   // the shared expert's B operand: digit g of block column `warp`
        if (with_shared && g < 4) {
            const int8_t* hp = s_hd + g * dq::kMaxFf + 32 * warp;
            hb0 = *reinterpret_cast<const uint32_t*>(hp + 4 * t);
            hb1 = *reinterpret_cast<const uint32_t*>(hp + 16 + 4 * t);
        }
#pragma unroll 1
        for (uint32_t i = 0; i < n_c; ++i, ++cnt) {
            const uint32_t stage = cnt % dq::kStages, parity = (cnt / dq::kStages) & 1u;
            if (!mbar_wait_bounded(my_bar + 8 * stage, parity)) timed_out = true;
            const uint32_t tb = ring + stage * dq::kStageBytes, qb = tb + kTileQ6;
            // the eight scales of this lane's groups (even groups for t < 2, odd for t >= 2), rows g and g+8
            const uint2 scA = lds64(tb + 16 * g + 8 * (t >> 1)), scB = lds64(tb + 16 * (g + 8) + 8 * (t >> 1));
            int acc[4] = {0, 0, 0, 0};
            const uint4 hA = lds128(tb + 256 + (2 * 32 + lane) * 16), hB = lds128(tb + 256 + (5 * 32 + lane) * 16);
#pragma unroll
            for (int hf = 0; hf < 2; ++hf) {
                const uint4 qA = lds128(tb + 256 + (hf * 32 + lane) * 16), qB = lds128(tb + 256 + ((3 + hf) * 32 + lane) * 16);
                uint32_t a0[4], a2[4], a1[4], a3[4];
                q6k_words(qA.x, qA.z, hf ? hA.z : hA.x, a0);   // row g, l = 4t..
                q6k_words(qA.y, qA.w, hf ? hA.w : hA.y, a2);   // row g, l = 16 + 4t..
                q6k_words(qB.x, qB.z, hf ? hB.z : hB.x, a1);   // row g + 8
                q6k_words(qB.y, qB.w, hf ? hB.w : hB.y, a3);
#pragma unroll
                for (int qd = 0; qd < 4; ++qd) {
                    const int j = 4 * hf + qd;
                    int c[4] = {0, 0, 0, 0};
                    mma_s8(c, a0[qd], a1[qd], a2[qd], a3[qd], b0[j], b1[j]);
                    const uint32_t sel = 0x8880u + (uint32_t)(j & 3) * 0x1111u;   // byte j & 3, sign-extended
                    const int sa = (int)prmt_dq(hf ? scA.y : scA.x, 0u, sel), sb = (int)prmt_dq(hf ? scB.y : scB.x, 0u, sel);
                    acc[0] += sa * c[0]; acc[1] += sa * c[1]; acc[2] += sb * c[2]; acc[3] += sb * c[3];
                }
            }
            const uint32_t dd2 = lds32(tb + 3328 + 2 * (g & ~1u)), dd8 = lds32(tb + 3328 + 16 + 2 * (g & ~1u));
            float va = w_s * (f16_bits_to_f32((dd2 >> (16 * (g & 1u))) & 0xFFFFu) * ((float)acc[0] * dw0 + (float)acc[1] * dw1));
            float vb = w_s * (f16_bits_to_f32((dd8 >> (16 * (g & 1u))) & 0xFFFFu) * ((float)acc[2] * dw0 + (float)acc[3] * dw1));
            if (with_shared) {
                const uint2 qa = lds64(qb + 32 + lane * 8);            // row g: qs[4t..4t+3], qs[16+4t..16+4t+3]
                const uint2 qc = lds64(qb + 32 + 256 + lane * 8);      // row g+8
                int c[4] = {0, 0, 0, 0};
                mma_s8(c, qa.x, qc.x, qa.y, qc.y, hb0, hb1);
                const uint32_t dw = lds32(qb + 2 * (g & ~1u)), dw8 = lds32(qb + 2 * (8 + (g & ~1u)));
                const float sda = f16_bits_to_f32((dw >> (16 * (g & 1u))) & 0xFFFFu);
                const float sdb = f16_bits_to_f32((dw8 >> (16 * (g & 1u))) & 0xFFFFu);
                va += w_sh * (sda * ((float)c[0] * dws0 + (float)c[1] * dws1));
                vb += w_sh * (sdb * ((float)c[2] * dws0 + (float)c[3] * dws1));
            }
            __syncwarp();
            if (lane == 0) issue(stage);
            va += __shfl_xor_sync(0xFFFFFFFFu, va, 1); vb += __shfl_xor_sync(0xFFFFFFFFu, vb, 1);
            va += __shfl_xor_sync(0xFFFFFFFFu, va, 2); vb += __shfl_xor_sync(0xFFFFFFFFu, vb, 2);
            if (t == 0) {
                float* r = red + ((buf * dq::kWarps + warp) * dq::kChunk + i) * 16;
                r[g] = va; r[g + 8] = vb;
            }
        }
        __syncthreads();
        if (tid < 16 * n_c) {
            const uint32_t i = tid >> 4, r = tid & 15u;   // tile i of the chunk
            float sum = 0.f;
#pragma unroll
            for (int w = 0; w < dq::kWarps; ++w)   // slot order, column blocks inside a slot
                sum += red[((buf * dq::kWarps + w) * dq::kChunk + i) * 16 + r];
            a.y[(size_t)tok * d.n_embd + (rt + i) * 16 + r] = sum;
        }
        buf ^= 1u;
        u += n_c;
        rt += n_c;
        if (rt == RT) { rt = 0; ++tok; new_tok = true; }
    }
    if (timed_out && lane == 0) atomicExch(a.status, (uint32_t)kStatusWaitTimeout);
}

cudaError_t launch_decode_down_q6k(const Launch& L, const DownDecodeArgs& a, uint32_t n_blocks) {
    if (!decode_down_ok(a.d)) return cudaErrorInvalidValue;
    if (a.n_tokens == 0) return cudaSuccess;
    const size_t smem = dq::kEnd + 128;
    cudaError_t e = cudaFuncSetAttribute(decode_down_q6k_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    e = launch_kernel(L, decode_down_q6k_kernel, dim3(n_blocks), dim3(dq::kWarps * 32), smem, a);
    L.count();
    return e != cudaSuccess ? e : cudaGetLastError();
}

}  // namespace qkm
