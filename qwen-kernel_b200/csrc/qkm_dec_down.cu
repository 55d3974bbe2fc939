// Down projection of the fused decode sequence, token major, routed experts (IQ4_XS) and the
// shared expert (Q8_0) and the final weighted sum in one persistent launch:
//   y[t] = sum_s w_s * D[ids_s] . h[t][s]  +  w_shared * DS . h[t][n_used].
//
// Replaces moe_down_iq4.comp + moe_down_q8b.comp + the "routed + shared" add.  A unit of work
// is (token, 16 output rows) and belongs to a whole block: warp (slot s, column block kb)
// streams the 16-row tiles of expert ids_s through a private three-stage ring of bulk copies
// (TMA, no tensor map, no multicast), so the eight slots of a token are worked on at once and
// are added in slot order by the block - no per-slot scratch in global memory, no atomics, the
// same bits on every run.  The flat list of (token, tile) is cut evenly and contiguously over
// the blocks; a block sums once per chunk of up to four tiles.
//
// Arithmetic: exact integers until the last step.  When its token changes, a warp encodes the
// 256 values of h[t][s] it multiplies with as four int8 digit planes (28-bit fixed point
// relative to the largest of the 256, one power-of-two scale) and keeps them in registers as
// the B operand of int8 MMAs.  IQ4_XS inner step: a quant byte holds two weights 16 columns
// apart; a 64 KB table image at shared address 0x10000 maps the byte to both codebook values
// (row = byte value, 256-byte stride, one 4-byte entry per lane: bank = lane, no conflicts),
// and a look-up address is one byte permute [lane * 4, byte, 0x01, 0x00].  Eight weights cost
// four permutes, four loads and one more permute that packs the operand register - the
// kernel is bound by the integer pipe, and this is half the work of looking the codebook up
// with permutes of four constant registers.  The 6-bit sub-block scales (ls - 32) are unpacked
// eight at a time with word-wide masks and multiply the int32 partial sums as integers; d, the
// digit weights, the plane scale and the routing weight are applied once per tile in f32.
//
// Shared expert: warp w also takes 32-column block w of the Q8_0 matrix for the tile's rows:
// raw int8 weights against h[t][n_used] as digit planes, which the block encodes in shared
// memory whenever its token changes.
//
// Shared memory: the table occupies [0x10000, 0x20000) of the shared window; barriers, the first
// rings and the shared row's planes lie below it, the other rings and the scratch above.
#include "qkm_kernels.h"
#include "qkm_stream.cuh"
#include "qkm_tiles.cuh"

namespace qkm {

namespace dd {
constexpr int kWarps = 16;
constexpr int kStages = 3;
constexpr int kShBlock = 544;                       // one Q8_0 block column of a 16-row tile: d, quants
constexpr int kStageBytes = kTileIq4 + kShBlock;    // 2720
constexpr int kRingBytes = kStages * kStageBytes;   // 8160
constexpr int kChunk = 4;                           // tiles between two block-wide sums
constexpr uint32_t kMaxFf = 512;
constexpr uint32_t kTab = 0x10000u, kTabBytes = 0x10000u;   // absolute shared-window address (64 KB aligned) and size
constexpr int kLowRingWarps = 7;                    // rings below the table; the others above it
// absolute shared-window addresses above the table
constexpr uint32_t kHigh = kTab + kTabBytes;
constexpr uint32_t kDig = kHigh + (kWarps - kLowRingWarps) * kRingBytes;   // per warp: 4 digit planes x 256 B, operand order
constexpr uint32_t kRed = kDig + kWarps * 1024;                            // [2 buffers][16 warps][kChunk tiles][16 rows]
constexpr uint32_t kEnd = kRed + 2 * kWarps * kChunk * 16 * 4;
// below the table, offsets from the (128-byte aligned) start of the dynamic area
constexpr uint32_t kBars = 0;                                              // kWarps * kStages ring barriers, then the table's
constexpr uint32_t kMisc = 512;                                            // 16 warp maxima
constexpr uint32_t kHd = 640;                                              // 4 digit planes x 512 of h[t][n_used]
constexpr uint32_t kLowRings = kHd + 4 * kMaxFf;                           // 2688
}  // namespace dd

size_t decode_down_lut_bytes() { return dd::kTabBytes; }

// The table image: row b (256 B) = for each of 32 lanes the 4-byte entry (kvalues[b & 15], kvalues[b >> 4], 0, 0)
// as int8 (src/quant_tables.h: kvalues_iq4nl); the upper 128 bytes of a row are unused.
__global__ void decode_down_lut_kernel(uint8_t* __restrict__ out) {
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;   // one 4-byte word each
    if (i >= dd::kTabBytes / 4) return;
    const uint32_t row = i >> 6, w = i & 63u;
    uint32_t v = 0;
    if (w < 32) v = (uint32_t)(uint8_t)c_iq4_values[row & 15u] | ((uint32_t)(uint8_t)c_iq4_values[row >> 4] << 8);
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

// The eight sub-block scales ls - 32 of one row as int8: even sub-blocks 0,2,4,6 in ev, odd 1,3,5,7 in od.
// sl: scales_l (eight 4-bit fields), sh: scales_h (eight 2-bit fields)  (src/quants.h:107-113, :139-146)
__device__ __forceinline__ void iq4_scales(uint32_t sl, uint32_t sh, uint32_t& ev, uint32_t& od) {
    const uint32_t r = prmt_dd(sh, 0u, 0x1100u);                       // bytes (B0, B0, B1, B1) of scales_h
    const uint32_t he = ((r << 4) & 0x00300030u) | (r & 0x30003000u);  // top two bits of sub-blocks 0,2,4,6 at bits 4..5
    const uint32_t ho = ((r << 2) & 0x00300030u) | ((r >> 2) & 0x30003000u);
    const uint32_t te = ((sl & 0x0F0F0F0Fu) | he) ^ 0x20202020u;       // ls ^ 32 per byte
    const uint32_t to = (((sl >> 4) & 0x0F0F0F0Fu) | ho) ^ 0x20202020u;
    // ls - 32 as int8: bit 5 of (ls ^ 32) extended into bits 6..7 (no carry leaves a byte)
    ev = (te & 0x20202020u) * 6u + te;
    od = (to & 0x20202020u) * 6u + to;
}

// Eight IQ4_XS weights of one quant word (bytes 4t..4t+3 of a sub-block's sixteen: the low nibbles are
// elements 4t..4t+3, the high nibbles elements 16+4t..16+4t+3) as two int8 MMA A-operand registers:
// lo = elements (4t, 16+4t, 4t+1, 17+4t), hi = elements (4t+2, 18+4t, 4t+3, 19+4t).
// tab_c: bytes (lane * 4, -, 0x01, 0x00): with a quant byte in byte 1 it is that byte's table entry for this lane.
__device__ __forceinline__ void iq4_word(uint32_t w, uint32_t tab_c, uint32_t& lo, uint32_t& hi) {
    const uint32_t e0 = lds32(prmt_dd(w, tab_c, 0x7604u)), e1 = lds32(prmt_dd(w, tab_c, 0x7614u));
    const uint32_t e2 = lds32(prmt_dd(w, tab_c, 0x7624u)), e3 = lds32(prmt_dd(w, tab_c, 0x7634u));
    lo = prmt_dd(e0, e1, 0x5410u);
    hi = prmt_dd(e2, e3, 0x5410u);
}

__global__ void __launch_bounds__(dd::kWarps * 32, 1)
decode_down_kernel(DownDecodeArgs a) {
    extern __shared__ __align__(128) uint8_t smem_raw[];
    const uint32_t win0 = smem_addr(smem_raw);                     // where the dynamic area starts in the shared window
    const uint32_t base = (win0 + 127u) & ~127u;
    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31u, g = lane >> 2, t = lane & 3u;
    const qkm_dims d = a.d;
    const uint32_t KB = d.n_ff / 256;               // 2
    const uint32_t slot = warp / KB, kb = warp - slot * KB;
    const uint32_t RT = d.n_embd / 16;              // row tiles of the down matrix
    const uint32_t n_slots = d.n_used + 1;
    const bool with_shared = a.sh_tiles != nullptr;

    if (base + dd::kLowRings + dd::kLowRingWarps * dd::kRingBytes > dd::kTab) {   // layout assumption broken
        if (tid == 0) atomicExch(a.status, (uint32_t)kStatusBadLayout);
        return;
    }
    auto at = [&](uint32_t window_addr) -> uint8_t* { return smem_raw + (window_addr - win0); };
    const uint32_t ring = warp < (uint32_t)dd::kLowRingWarps ? base + dd::kLowRings + warp * dd::kRingBytes
                                                             : dd::kHigh + (warp - dd::kLowRingWarps) * dd::kRingBytes;
    const uint32_t my_bar = base + dd::kBars + warp * dd::kStages * 8;
    const uint32_t tab_bar = base + dd::kBars + dd::kWarps * dd::kStages * 8;
    const uint32_t my_dig = dd::kDig + warp * 1024;
    uint8_t* dig = at(my_dig);
    float* red = reinterpret_cast<float*>(at(dd::kRed));
    int8_t* s_hd = reinterpret_cast<int8_t*>(at(base + dd::kHd));
    float* s_misc = reinterpret_cast<float*>(at(base + dd::kMisc));
    bool timed_out = false;

    if (lane == 0) {
        for (int s = 0; s < dd::kStages; ++s) mbar_init(my_bar + 8 * s, 1);
        if (warp == 0) mbar_init(tab_bar, 1);
        mbar_fence_init();
    }
    __syncthreads();
    if (tid == 0) {   // the 64 KB table image comes from global memory (L2 after the first block) in four bulk copies
        mbar_expect_tx(tab_bar, dd::kTabBytes);
        for (uint32_t i = 0; i < 4; ++i) bulk_g2s(dd::kTab + i * 16384u, a.lut + i * 16384u, 16384u, tab_bar);
    }

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
            p_src = a.tiles + ((size_t)e * mat_tiles + (size_t)kb * RT + p_rt) * kTileIq4;
            if (with_shared) p_sh = a.sh_tiles + ((size_t)(warp >> 3) * RT + p_rt) * kTileQ8 + dd::kShBlock * (warp & 7u);
        }
        const uint32_t bar = my_bar + 8 * stage, dst = ring + stage * dd::kStageBytes;
        mbar_expect_tx(bar, kTileIq4 + (with_shared ? dd::kShBlock : 0));
        bulk_g2s(dst, p_src, kTileIq4, bar);
        p_src += kTileIq4;
        if (with_shared) {
            bulk_g2s(dst + kTileIq4, p_sh, dd::kShBlock, bar);
            p_sh += kTileQ8;
        }
        ++p_u;
        if (++p_rt == RT) { p_rt = 0; ++p_tok; p_new_tok = true; }
    };
    if (lane == 0)
        for (int s = 0; s < dd::kStages; ++s) issue(s);
    // The first weight tiles are on their way (they depend on the selection only, which was final
    // before the gate/up kernel released this one); h is that kernel's output.
    pdl_wait();
    pdl_trigger();

    uint32_t cnt = 0, buf = 0;
    float w_s = 0.f, w_sh = 0.f;   // routing weight x plane scale of this warp's slot; w_shared x 2^-p of the shared row's digits
    uint32_t b0[8], b1[8];         // B operand: digit g (g < 4) of the token's h values, in the A operand's element order
    // digit weights: C columns 2t, 2t+1 are digits 2t, 2t+1 (t < 2); the other columns are zero
    const float dw0 = t == 0 ? 1.f : (t == 1 ? 16384.f : 0.f), dw1 = dw0 * 128.f;
    const uint32_t tab_c = dd::kTab + lane * 4;

    if (!mbar_wait_bounded(tab_bar, 0)) timed_out = true;   // every thread observes the table's arrival itself

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
                __syncwarp();
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    // element e = 8 * lane + i of the 256 -> sub-block lane / 4; inside it the order of iq4_word's
                    // registers: element 4tt + j -> register j / 2, byte 2 (j & 1); element 16 + 4tt + j one byte later
                    const uint32_t pos = (lane >> 2) * 32 + ((lane >> 1) & 1u) + (lane & 1u) * 8 + (i >> 2) * 4 + ((i & 3) >> 1) * 16 + (i & 1) * 2;
                    const uint32_t dgt = any_bad ? 0u : digits4(__float2int_rn(hv[i] * up));
                    dig[pos] = (uint8_t)(dgt & 255u);
                    dig[256 + pos] = (uint8_t)((dgt >> 8) & 255u);
                    dig[512 + pos] = (uint8_t)((dgt >> 16) & 255u);
                    dig[768 + pos] = (uint8_t)(dgt >> 24);
                }
                __syncwarp();
#pragma unroll
                for (int sb = 0; sb < 8; ++sb) {
                    b0[sb] = g < 4 ? lds32(my_dig + g * 256 + sb * 32 + t * 4) : 0u;
                    b1[sb] = g < 4 ? lds32(my_dig + g * 256 + sb * 32 + 16 + t * 4) : 0u;
                }
                w_s = w_slot * (any_bad ? __int_as_float(0x7FC00000) : ldexpf(1.0f, -p));
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
        const uint32_t n_c = min((uint32_t)dd::kChunk, min(u_hi - u, RT - rt));   // tiles of this chunk
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
            const uint32_t tb = ring + stage * dd::kStageBytes, qb = tb + kTileIq4;
            // headers: row g (x: d | scales_h << 16, y: scales_l), row g+8 (z, w)
            const uint4 hd = lds128(tb + 16 * g);
            uint32_t ea, oa, eb, ob;   // ls - 32 of the even / odd sub-blocks, rows g and g+8
            iq4_scales(hd.y, hd.x >> 16, ea, oa);
            iq4_scales(hd.w, hd.z >> 16, eb, ob);
            int acc[4] = {0, 0, 0, 0};
#pragma unroll
            for (int hf = 0; hf < 2; ++hf) {
                // quant word t of sub-blocks 4hf..4hf+3: rows g and g+8
                const uint4 qa4 = lds128(tb + 128 + (hf * 32 + lane) * 16), qb4 = lds128(tb + 128 + ((2 + hf) * 32 + lane) * 16);
                const uint32_t wa[4] = {qa4.x, qa4.y, qa4.z, qa4.w}, wb[4] = {qb4.x, qb4.y, qb4.z, qb4.w};
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const int sb = 4 * hf + j;
                    uint32_t a0, a1, a2, a3;
                    iq4_word(wa[j], tab_c, a0, a2);
                    iq4_word(wb[j], tab_c, a1, a3);
                    int c[4] = {0, 0, 0, 0};
                    mma_s8(c, a0, a1, a2, a3, b0[sb], b1[sb]);
                    const uint32_t sel = 0x8880u + (uint32_t)(sb >> 1) * 0x1111u;   // byte sb / 2, sign-extended
                    const int la = (int)prmt_dd((sb & 1) ? oa : ea, 0u, sel), lb = (int)prmt_dd((sb & 1) ? ob : eb, 0u, sel);
                    acc[0] += la * c[0]; acc[1] += la * c[1]; acc[2] += lb * c[2]; acc[3] += lb * c[3];
                }
            }
            float va = w_s * (f16_bits_to_f32(hd.x & 0xFFFFu) * ((float)acc[0] * dw0 + (float)acc[1] * dw1));
            float vb = w_s * (f16_bits_to_f32(hd.z & 0xFFFFu) * ((float)acc[2] * dw0 + (float)acc[3] * dw1));
            if (with_shared) {
                const uint2 qa = lds64(qb + 32 + lane * 8);            // row g: qs[4t..4t+3], qs[16+4t..16+4t+3]
                const uint2 qc = lds64(qb + 32 + 256 + lane * 8);      // row g+8
                int c[4] = {0, 0, 0, 0};
                mma_s8(c, qa.x, qc.x, qa.y, qc.y, hb0, hb1);
                const uint32_t dw = lds32(qb + 2 * (g & ~1u)), dw8 = lds32(qb + 2 * (8 + (g & ~1u)));
                const float sda = f16_bits_to_f32((dw >> (16 * (g & 1u))) & 0xFFFFu);
                const float sdb = f16_bits_to_f32((dw8 >> (16 * (g & 1u))) & 0xFFFFu);
                va += w_sh * (sda * ((float)c[0] * dw0 + (float)c[1] * dw1));
                vb += w_sh * (sdb * ((float)c[2] * dw0 + (float)c[3] * dw1));
            }
            __syncwarp();
            if (lane == 0) issue(stage);
            // digits 0, 1 sit in lane t = 0 and 2, 3 in t = 1
            va += __shfl_xor_sync(0xFFFFFFFFu, va, 1); vb += __shfl_xor_sync(0xFFFFFFFFu, vb, 1);
            if (t == 0) {
                float* r = red + ((buf * dd::kWarps + warp) * dd::kChunk + i) * 16;
                r[g] = va; r[g + 8] = vb;
            }
        }
        __syncthreads();
        if (tid < 16 * n_c) {
            const uint32_t i = tid >> 4, r = tid & 15u;   // tile i of the chunk
            float sum = 0.f;
#pragma unroll
            for (int w = 0; w < dd::kWarps; ++w)   // slot order, column blocks inside a slot
                sum += red[((buf * dd::kWarps + w) * dd::kChunk + i) * 16 + r];
            a.y[(size_t)tok * d.n_embd + (rt + i) * 16 + r] = sum;
        }
        buf ^= 1u;
        u += n_c;
        rt += n_c;
        if (rt == RT) { rt = 0; ++tok; new_tok = true; }
    }
    if (timed_out && lane == 0) atomicExch(a.status, (uint32_t)kStatusWaitTimeout);
}

bool decode_down_ok(const qkm_dims& d) {
    return d.n_ff == dd::kMaxFf && d.n_used * (d.n_ff / 256) == dd::kWarps && d.n_embd % 32 == 0;
}

cudaError_t launch_decode_down(const Launch& L, const DownDecodeArgs& a, uint32_t n_blocks) {
    if (!decode_down_ok(a.d) || !a.lut) return cudaErrorInvalidValue;
    if (a.n_tokens == 0) return cudaSuccess;
    const size_t smem = dd::kEnd;   // the dynamic area must reach from wherever it starts to the end of the scratch
    cudaError_t e = cudaFuncSetAttribute(decode_down_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    e = launch_kernel(L, decode_down_kernel, dim3(n_blocks), dim3(dd::kWarps * 32), smem, a);
    L.count();
    return e != cudaSuccess ? e : cudaGetLastError();
}

}  // namespace qkm
