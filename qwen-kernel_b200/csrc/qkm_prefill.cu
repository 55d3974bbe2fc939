// Batched prefill of the expert GEMMs on the 5th-generation tensor cores (tcgen05 + TMEM).
//
// Replaces moe_gateup_iq3_grouped_coopmat.comp / moe_gateup_q8_coopmat.comp (gate/up +
// SwiGLU), moe_down_{iq4}_grouped_coopmat.comp / moe_down_q8_coopmat.comp (down) and the
// slot-order fold of add_rms3_grouped.comp:22-27.
//
// Tokens are grouped by expert (moe_group_pairs).  One block owns (expert, 128 weight
// rows, up to 128 of the expert's pairs).  Weights are the M = 128 operand: every k-step
// the block's threads dequantise 128 x 64 weights from the tile-ordered quant blocks to
// bf16 (single rounding of the exact f32 value) straight into the 128-byte-swizzled
// K-major shared-memory layout, gather the matching 64 columns of the pairs' activation
// rows (bf16) as the N operand, and one thread issues tcgen05.mma (kind::f16, bf16 inputs,
// f32 accumulators in tensor memory).  Two shared-memory stages (two blocks per SM) let dequantisation of
// the next k-steps overlap the asynchronous MMAs.  Eight warps produce operands and later
// run the epilogue; a ninth warp only issues MMAs: producers arrive on a stage's "full"
// mbarrier, the issuer waits for it, issues the k-step's MMAs and commits them to the
// stage's "empty" mbarrier, which the producers wait on before refilling the stage.
// All waits are bounded.
//
// Operand types: the gate/up GEMM runs on f16 operands (11-bit significands; x is scaled
// per token by a power of two into f16 range and unscaled in the epilogue), the down GEMM
// on bf16 operands (the hidden rows need bf16's exponent range).  With bf16 on both GEMMs
// the worst element of a 2048-wide output row sits at the 2e-2 tolerance; f16 on the first
// GEMM leaves a 3x margin at the same tensor-core rate.
//
// gate/up: two accumulators (gate rows, up rows) share the B operand; the epilogue reads
//          both from TMEM, applies SwiGLU and stores h as bf16 [pair][n_ff] (the down
//          GEMM's N operand) and as f32 in the reference's h layout.
// down:    epilogue multiplies by the routing weight after the full K reduction
//          (moe_down_iq4_grouped_coopmat.comp:160-161) and stores contrib[pair][n_embd];
//          the fold adds a token's slots in order, then the shared expert.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "qkm_kernels.h"
#include "qkm_stream.cuh"
#include "qkm_tiles.cuh"
#include "qkm_umma.cuh"

namespace qkm {

namespace pf {
constexpr int kThreads = 256;                  // producer/epilogue threads; one more warp issues the MMAs
constexpr int kBlock = kThreads + 32;
constexpr int kStages = 2;
constexpr int kNT = 128;                       // pairs per block (N tile)
constexpr int kTileBytes = 128 * 128;          // 128 rows x 64 bf16
}  // namespace pf

// ---- x -> f16 rows, each scaled by a power of two so that max|x| lands in [2^13, 2^14) -----------
__global__ void __launch_bounds__(256)
to_f16_rows_kernel(const float* __restrict__ x, __half* __restrict__ xh, float* __restrict__ inv_scale, uint32_t K) {
    __shared__ float s_max[8];
    const uint32_t t = blockIdx.x, tid = threadIdx.x;
    const float* xt = x + (size_t)t * K;
    float m = 0.f;
    for (uint32_t k = tid; k < K; k += 256) m = fmaxf(m, fabsf(xt[k]));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xFFFFFFFFu, m, o));
    if ((tid & 31u) == 0) s_max[tid >> 5] = m;
    __syncthreads();
    m = s_max[0];
#pragma unroll
    for (int w = 1; w < 8; ++w) m = fmaxf(m, s_max[w]);
    int p = 0;
    if (m > 0.f && m <= 3.0e38f) { int e; frexpf(m, &e); p = 14 - e; }  // m * 2^p in [2^13, 2^14)
    const float up = ldexpf(1.0f, p);
    for (uint32_t k = tid * 2; k < K; k += 512) {
        const float2 v = *reinterpret_cast<const float2*>(xt + k);
        *reinterpret_cast<__half2*>(xh + (size_t)t * K + k) = __floats2half2_rn(v.x * up, v.y * up);
    }
    if (tid == 0) inv_scale[t] = ldexpf(1.0f, -p);
}

// The hidden rows for the down GEMM: f32 rows by pair position -> f16, each row scaled by a power of two so
// that max|h| lands in [2^13, 2^14) (exact), and the scale that undoes it.  Rows [first, first + count) with
// first = *first_ptr + first_add when first_ptr is given (the shared expert's rows start where the routed
// pairs end, a count only the device knows) and count = *count_ptr when count_ptr is given.  Persistent
// blocks: the row count is an upper bound on the host.
__global__ void __launch_bounds__(256)
h_rows_to_f16_kernel(const float* __restrict__ hp, __half* __restrict__ hh, float* __restrict__ inv_scale, uint32_t K,
                     const uint32_t* __restrict__ first_ptr, uint32_t first_add, const uint32_t* __restrict__ count_ptr,
                     uint32_t count_max) {
    // one warp per row, 4-element pieces: a row's values stay in registers between the maximum and the conversion
    const uint32_t lane = threadIdx.x & 31u, warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, n_warps = (gridDim.x * blockDim.x) >> 5;
    const uint32_t first = (first_ptr ? *first_ptr : 0u) + first_add;
    const uint32_t count = count_ptr ? min(*count_ptr, count_max) : count_max;
    constexpr int kPieces = 8;   // K <= 1024 in registers; wider rows are read twice
    for (uint32_t r = warp; r < count; r += n_warps) {
        const float4* src = reinterpret_cast<const float4*>(hp + (size_t)(first + r) * K);
        const uint32_t n4 = K / 4;
        float4 v[kPieces];
        float m = 0.f;
#pragma unroll
        for (int i = 0; i < kPieces; ++i) {
            const uint32_t c = lane + 32u * i;
            v[i] = c < n4 ? src[c] : make_float4(0.f, 0.f, 0.f, 0.f);
            m = fmaxf(m, fmaxf(fmaxf(fabsf(v[i].x), fabsf(v[i].y)), fmaxf(fabsf(v[i].z), fabsf(v[i].w))));
        }
        for (uint32_t c = lane + 32u * kPieces; c < n4; c += 32) {
            const float4 w = src[c];
            m = fmaxf(m, fmaxf(fmaxf(fabsf(w.x), fabsf(w.y)), fmaxf(fabsf(w.z), fabsf(w.w))));
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xFFFFFFFFu, m, o));
        int p = 0;
        if (m > 0.f && m <= 3.0e38f) { int e; frexpf(m, &e); p = 14 - e; }
        const float up = ldexpf(1.0f, p);
        uint2* dst = reinterpret_cast<uint2*>(hh + (size_t)(first + r) * K);
        auto pack = [&](const float4& w) -> uint2 {
            const __half2 a = __floats2half2_rn(w.x * up, w.y * up), b = __floats2half2_rn(w.z * up, w.w * up);
            return make_uint2(*reinterpret_cast<const uint32_t*>(&a), *reinterpret_cast<const uint32_t*>(&b));
        };
#pragma unroll
        for (int i = 0; i < kPieces; ++i) {
            const uint32_t c = lane + 32u * i;
            if (c < n4) dst[c] = pack(v[i]);
        }
        for (uint32_t c = lane + 32u * kPieces; c < n4; c += 32) dst[c] = pack(src[c]);
        if (lane == 0) inv_scale[first + r] = ldexpf(1.0f, -p);
    }
}

cudaError_t launch_h_rows_to_f16(const Launch& L, const float* hp, void* hh, float* inv_scale, uint32_t K,
                                 const uint32_t* first_ptr, uint32_t first_add, const uint32_t* count_ptr, uint32_t count_max) {
    if (count_max == 0) return cudaSuccess;
    if (K % 4) return cudaErrorInvalidValue;
    const uint32_t want = (count_max + 7) / 8;   // eight rows per block at a time
    const uint32_t blocks = want < 148u * 8u ? want : 148u * 8u;
    h_rows_to_f16_kernel<<<blocks, 256, 0, L.stream>>>(hp, (__half*)hh, inv_scale, K, first_ptr, first_add, count_ptr, count_max);
    L.count();
    return cudaGetLastError();
}

// ---- work list ------------------------------------------------------------------------------------------
// For every expert with pairs: its pairs in tiles of kNT, times the 128-row tiles of the
// gate/up matrices (items_gu) and of the down matrix (items_dn).  Index n_expert_local is
// the shared expert: its "pairs" are all tokens, stored after the routed pairs.
// Also pos_of[t * (n_used+1) + s] = position of pair (t, s) in the grouped order, or
// 0xFFFFFFFF when the pair is not in the lists (its expert lives on another GPU, or the
// shared expert is left out with with_shared == 0).
__global__ void __launch_bounds__(512)
mma_plan_kernel(const uint32_t* __restrict__ offsets, uint32_t* __restrict__ pairs, uint32_t n_expert_local,
                uint32_t n_tokens, uint32_t n_used, uint32_t rt_gu, uint32_t rt_dn, uint32_t with_shared,
                uint32_t routed_pos_done, uint32_t sh_first, uint32_t sh_count,
                MmaItem* __restrict__ items_gu, MmaItem* __restrict__ items_dn, MmaItem* __restrict__ items_sh_gu,
                MmaItem* __restrict__ items_sh_dn, uint32_t* __restrict__ n_items, uint32_t* __restrict__ pos_of) {
    __shared__ uint32_t s_scan[512];
    const uint32_t e = threadIdx.x;
    const uint32_t np = offsets[n_expert_local];
    if (!routed_pos_done)   // else the grouping kernels have written every routed (token, slot) entry
        for (uint32_t i = e; i < n_tokens * (n_used + 1); i += 512) pos_of[i] = 0xFFFFFFFFu;
    uint32_t tiles = 0, p0 = 0, n = 0;
    if (e < n_expert_local) { p0 = offsets[e]; n = offsets[e + 1] - p0; tiles = (n + pf::kNT - 1) / pf::kNT; }
    s_scan[e] = tiles;
    __syncthreads();
    for (uint32_t o = 1; o < 512; o <<= 1) {
        const uint32_t v = e >= o ? s_scan[e - o] : 0;
        __syncthreads();
        s_scan[e] += v;
        __syncthreads();
    }
    const uint32_t first = s_scan[e] - tiles;
    for (uint32_t ti = 0; ti < tiles; ++ti) {
        MmaItem it;
        it.expert = (uint16_t)e;
        it.pair_off = p0 + ti * pf::kNT;
        it.n = min((uint32_t)pf::kNT, n - ti * pf::kNT);
        for (uint32_t r = 0; r < rt_gu; ++r) { it.rt = (uint16_t)r; items_gu[(size_t)(first + ti) * rt_gu + r] = it; }
        for (uint32_t r = 0; r < rt_dn; ++r) { it.rt = (uint16_t)r; items_dn[(size_t)(first + ti) * rt_dn + r] = it; }
    }
    // the shared expert takes rows [sh_first, sh_first + sh_count): all rows of a single-GPU
    // chunk, this rank's own tokens among the received rows of an expert-parallel shard
    const uint32_t sh_n = with_shared ? sh_count : 0;
    const uint32_t sh_tiles = (sh_n + pf::kNT - 1) / pf::kNT;
    for (uint32_t ti = e; ti < sh_tiles; ti += 512) {
        MmaItem it;
        it.expert = 0;
        it.pair_off = np + ti * pf::kNT;
        it.n = min((uint32_t)pf::kNT, sh_n - ti * pf::kNT);
        for (uint32_t r = 0; r < rt_gu; ++r) { it.rt = (uint16_t)r; items_sh_gu[(size_t)ti * rt_gu + r] = it; }
        for (uint32_t r = 0; r < rt_dn; ++r) { it.rt = (uint16_t)r; items_sh_dn[(size_t)ti * rt_dn + r] = it; }
    }
    if (e == 511) {
        n_items[0] = s_scan[511] * rt_gu; n_items[1] = s_scan[511] * rt_dn;
        n_items[2] = sh_tiles * rt_gu;    n_items[3] = sh_tiles * rt_dn;
    }
    if (!routed_pos_done)
        for (uint32_t p = e; p < np; p += 512) {
            const uint32_t pr = pairs[p];
            pos_of[(pr >> 4) * (n_used + 1) + (pr & 15u)] = p;
        }
    for (uint32_t t = e; t < n_tokens; t += 512) {
        const uint32_t j = t - sh_first;          // wraps below the range
        const bool in = j < sh_n;
        if (in) pairs[np + j] = (t << 4) | n_used;
        pos_of[t * (n_used + 1) + n_used] = in ? np + j : 0xFFFFFFFFu;
    }
}

// ---- operand producers ----------------------------------------------------------------------------------
// Each fills, for one weight row and one 64-column k-step, the row's eight 16-byte chunks
// of the swizzled A tile.  `tile` points at the row's 16-row tile of the tile-ordered
// tensor (qkm_tiles.cuh), r16 is the row inside it, q = k-step within the 256-column block.

template <bool F16>
__device__ __forceinline__ uint32_t pack16(float a, float b) {
    if (F16) { __half2 v = __floats2half2_rn(a, b); return *reinterpret_cast<uint32_t*>(&v); }
    __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ uint32_t pack_bf16(float a, float b) { return pack16<false>(a, b); }

// IQ4_XS: a quant byte holds two weights 16 columns apart (low and high nibble).  The table
// maps a byte to both values as a bf16 pair; it is replicated per lane ([256][32] words, lane
// = bank) so lookups never conflict.  s_pair_lane already points at this lane's column.
// The sub-block scale is applied in two bf16 pieces (hi + lo), so the stored weight carries
// one bf16 rounding of the exact product, as before.
// the bytes one thread needs for (row, k-step, 32-column half j): fetched one k-step ahead
struct Iq4Raw { uint2 hd; uint32_t w[4]; };
__device__ __forceinline__ Iq4Raw load_iq4(const uint8_t* __restrict__ tile, uint32_t r16, uint32_t q, uint32_t j) {
    const uint32_t g = r16 & 7u, hf = r16 >> 3, sb = 2 * q + j;
    Iq4Raw r;
    r.hd = *reinterpret_cast<const uint2*>(tile + 16 * g + 8 * hf);  // d | scales_h << 16, scales_l
    // the sub-block's 16 quant bytes: word t sits in lane slot (g, t) of chunk 2*hf + sb/4
#pragma unroll
    for (int t = 0; t < 4; ++t)
        r.w[t] = *reinterpret_cast<const uint32_t*>(tile + 128 + ((2 * hf + (sb >> 2)) * 32 + 4 * g + t) * 16 + 4 * (sb & 3u));
    return r;
}

__device__ __forceinline__ void produce_iq4(const Iq4Raw& raw, uint32_t q, uint32_t j,
                                            const uint8_t* __restrict__ s_pair_lane, uint8_t* a_tile, uint32_t row) {
    const uint2 hd = raw.hd;
    const float d = f16_bits_to_f32(hd.x & 0xFFFFu);
    const uint32_t sh = hd.x >> 16;
    {
        const uint32_t sb = 2 * q + j;
        const int ls = (int)(((hd.y >> (4 * sb)) & 0xFu) | (((sh >> (2 * sb)) & 3u) << 4)) - 32;
        const float dl = d * (float)ls;
        const __nv_bfloat16 dhi = __float2bfloat16_rn(dl);
        const __nv_bfloat162 s_hi = __bfloat162bfloat162(dhi);
        const __nv_bfloat162 s_lo = __bfloat162bfloat162(__float2bfloat16_rn(dl - __bfloat162float(dhi)));
        const uint32_t* w = raw.w;
        uint32_t lo[8], hi[8];   // bf16 pairs: columns 2i, 2i+1 of the low-nibble half / of the high-nibble half
#pragma unroll
        for (int t = 0; t < 4; ++t) {
            const uint32_t l0 = *reinterpret_cast<const uint32_t*>(s_pair_lane + ((w[t] << 7) & 0x7F80u));
            const uint32_t l1 = *reinterpret_cast<const uint32_t*>(s_pair_lane + ((w[t] >> 1) & 0x7F80u));
            const uint32_t l2 = *reinterpret_cast<const uint32_t*>(s_pair_lane + ((w[t] >> 9) & 0x7F80u));
            const uint32_t l3 = *reinterpret_cast<const uint32_t*>(s_pair_lane + ((w[t] >> 17) & 0x7F80u));
            lo[2 * t] = __byte_perm(l0, l1, 0x5410); lo[2 * t + 1] = __byte_perm(l2, l3, 0x5410);
            hi[2 * t] = __byte_perm(l0, l1, 0x7632); hi[2 * t + 1] = __byte_perm(l2, l3, 0x7632);
        }
        auto scale = [&](uint32_t x) -> uint32_t {
            const __nv_bfloat162 v = *reinterpret_cast<const __nv_bfloat162*>(&x);
            const __nv_bfloat162 r = __hfma2(v, s_hi, __hmul2(v, s_lo));
            return *reinterpret_cast<const uint32_t*>(&r);
        };
#pragma unroll
        for (int p = 0; p < 4; ++p) {      // elements 8p .. 8p+7 of the sub-block -> chunk 4j + p
            const uint32_t* src = (p >> 1) ? hi : lo;
            const int o4 = 4 * (p & 1);
            uint4 o;
            o.x = scale(src[o4]); o.y = scale(src[o4 + 1]); o.z = scale(src[o4 + 2]); o.w = scale(src[o4 + 3]);
            *reinterpret_cast<uint4*>(a_tile + umma::sw128_chunk(row, 4 * j + p)) = o;
        }
    }
}

// IQ4_XS to f16 without the pair table (the gate/up kernel's form): the codebook times the sub-block
// scale as sixteen floats in shared memory (sixteen banks: look-ups of different entries never
// conflict, equal ones broadcast), one rounding of d * (ls - 32) * kvalue to f16.
__device__ __forceinline__ void produce_iq4_f16(const Iq4Raw& raw, uint32_t q, uint32_t j, const float* __restrict__ s_kv,
                                                uint8_t* a_tile, uint32_t row) {
    const uint32_t sb = 2 * q + j, sh = raw.hd.x >> 16;
    const int ls = (int)(((raw.hd.y >> (4 * sb)) & 0xFu) | (((sh >> (2 * sb)) & 3u) << 4)) - 32;
    const float dl = f16_bits_to_f32(raw.hd.x & 0xFFFFu) * (float)ls;
#pragma unroll
    for (int p = 0; p < 4; ++p) {      // elements 8p .. 8p+7: low nibbles of words 2p, 2p+1 (p < 2), high nibbles of words 2p-4, 2p-3
        const uint32_t sft = (p >> 1) ? 4u : 0u;
        const uint32_t a = raw.w[2 * (p & 1)] >> sft, b = raw.w[2 * (p & 1) + 1] >> sft;
        uint4 o;
        o.x = pack16<true>(dl * s_kv[a & 15u], dl * s_kv[(a >> 8) & 15u]);
        o.y = pack16<true>(dl * s_kv[(a >> 16) & 15u], dl * s_kv[(a >> 24) & 15u]);
        o.z = pack16<true>(dl * s_kv[b & 15u], dl * s_kv[(b >> 8) & 15u]);
        o.w = pack16<true>(dl * s_kv[(b >> 16) & 15u], dl * s_kv[(b >> 24) & 15u]);
        *reinterpret_cast<uint4*>(a_tile + umma::sw128_chunk(row, 4 * j + p)) = o;
    }
}

template <bool F16, int J0, int J1>
__device__ __forceinline__ void produce_q8(const uint8_t* __restrict__ tile, uint32_t r16, uint32_t q,
                                           uint8_t* a_tile, uint32_t row) {
    const uint32_t g = r16 & 7u, hf = r16 >> 3;
#pragma unroll
    for (int j = J0; j < J1; ++j) {
        const uint32_t blk = 2 * q + j;
        const float d = f16_bits_to_f32(*reinterpret_cast<const uint16_t*>(tile + 544 * blk + 2 * r16));
        // lane slot (g, t): qs[4t..4t+3] then qs[16+4t..16+4t+3]
        uint2 w[4];
#pragma unroll
        for (int t = 0; t < 4; ++t)
            w[t] = *reinterpret_cast<const uint2*>(tile + 544 * blk + 32 + (hf * 32 + 4 * g + t) * 8);
#pragma unroll
        for (int p = 0; p < 4; ++p) {      // elements 8p..8p+7: words (2(p&1), 2(p&1)+1), .x below 16, .y above
            const uint32_t a = (p >> 1) ? w[2 * (p & 1)].y : w[2 * (p & 1)].x;
            const uint32_t b = (p >> 1) ? w[2 * (p & 1) + 1].y : w[2 * (p & 1) + 1].x;
            uint4 o;
            o.x = pack16<F16>(d * (float)(int8_t)(a & 0xFF), d * (float)(int8_t)((a >> 8) & 0xFF));
            o.y = pack16<F16>(d * (float)(int8_t)((a >> 16) & 0xFF), d * (float)(int8_t)(a >> 24));
            o.z = pack16<F16>(d * (float)(int8_t)(b & 0xFF), d * (float)(int8_t)((b >> 8) & 0xFF));
            o.w = pack16<F16>(d * (float)(int8_t)((b >> 16) & 0xFF), d * (float)(int8_t)(b >> 24));
            *reinterpret_cast<uint4*>(a_tile + umma::sw128_chunk(row, 4 * j + p)) = o;
        }
    }
}

// Q6_K (tile layout of qkm_tiles.cuh): the 32 columns of 128-column half hf = q / 2, quarter
// qd = 2 (q & 1) + j - nibble qd / 2 of the (qd & 1)-th 32-byte run of ql, bit pair qd of qh, scales
// 2 (4 hf + qd) and the one after it (src/quants.h:148-163).  One rounding: d * scale * (q - 32) -> 16 bit.
template <bool F16>
__device__ __forceinline__ void produce_q6k(const uint8_t* __restrict__ tile, uint32_t r16, uint32_t q, uint32_t j,
                                            uint8_t* a_tile, uint32_t row) {
    const uint32_t g = r16 & 7u, h = r16 >> 3, hf = q >> 1, qd = 2 * (q & 1u) + j;
    const float d = f16_bits_to_f32(*reinterpret_cast<const uint16_t*>(tile + 3328 + 2 * r16));
    const float s0 = d * (float)(int8_t)tile[16 * r16 + 4 * hf + qd], s1 = d * (float)(int8_t)tile[16 * r16 + 8 + 4 * hf + qd];
    const uint8_t* ql = tile + 256 + ((3 * h + hf) * 32 + 4 * g) * 16 + 8 * (qd & 1u);
    const uint8_t* qh = tile + 256 + ((3 * h + 2) * 32 + 4 * g) * 16 + 8 * hf;
    uint32_t v[8];   // word m: elements 4m .. 4m+3 as bytes q (0..63)
#pragma unroll
    for (int m = 0; m < 8; ++m) {
        const uint32_t wl = *reinterpret_cast<const uint32_t*>(ql + 16 * (m & 3) + 4 * (m >> 2));
        const uint32_t wh = *reinterpret_cast<const uint32_t*>(qh + 16 * (m & 3) + 4 * (m >> 2));
        v[m] = (((qd >> 1) ? wl >> 4 : wl) & 0x0F0F0F0Fu) | (((wh >> (2 * qd)) & 0x03030303u) << 4);
    }
#pragma unroll
    for (int p = 0; p < 4; ++p) {      // elements 8p .. 8p+7
        const float s = p < 2 ? s0 : s1;
        const uint32_t a = v[2 * p], b = v[2 * p + 1];
        uint4 o;
        o.x = pack16<F16>(s * (float)((int)(a & 0xFF) - 32), s * (float)((int)((a >> 8) & 0xFF) - 32));
        o.y = pack16<F16>(s * (float)((int)((a >> 16) & 0xFF) - 32), s * (float)((int)(a >> 24) - 32));
        o.z = pack16<F16>(s * (float)((int)(b & 0xFF) - 32), s * (float)((int)((b >> 8) & 0xFF) - 32));
        o.w = pack16<F16>(s * (float)((int)((b >> 16) & 0xFF) - 32), s * (float)((int)(b >> 24) - 32));
        *reinterpret_cast<uint4*>(a_tile + umma::sw128_chunk(row, 4 * j + p)) = o;
    }
}

// N operand: rows [0, n_mma) of the block's pairs, 64 columns at k0; rows >= n are zero.
// Split in two so the global loads of the next k-step can be in flight during this one:
// fetch_b reads this thread's (at most 4) 16-byte chunks, store_b writes them swizzled.
// `row_ptr[i]` is the activation row of pair i (element type: 2 bytes).
struct BRegs { uint4 v[4]; };

template <class T, int PT = pf::kThreads>
__device__ __forceinline__ BRegs fetch_b(const T* const* row_ptr, uint32_t n, uint32_t n_mma, uint32_t k0) {
    BRegs b;
#pragma unroll
    for (int i = 0; i < 1024 / PT; ++i) {
        const uint32_t qd = threadIdx.x + i * PT, row = qd >> 3, c = qd & 7u;
        b.v[i] = make_uint4(0, 0, 0, 0);
        if (qd < n_mma * 8 && row < n) b.v[i] = *reinterpret_cast<const uint4*>(row_ptr[row] + k0 + 8 * c);
    }
    return b;
}
template <int PT = pf::kThreads>
__device__ __forceinline__ void store_b(uint8_t* b_tile, const BRegs& b, uint32_t n_mma) {
#pragma unroll
    for (int i = 0; i < 1024 / PT; ++i) {
        const uint32_t qd = threadIdx.x + i * PT, row = qd >> 3, c = qd & 7u;
        if (qd < n_mma * 8) *reinterpret_cast<uint4*>(b_tile + umma::sw128_chunk(row, c)) = b.v[i];
    }
}

// ---- gate/up + SwiGLU ------------------------------------------------------------------------------------
// FMT: QKM_TYPE_Q8_0 (shared expert) or QKM_TYPE_IQ4_XS (routed experts of layers whose gate/up tensors are
// IQ4_XS; 512 producers only).  IQ3_XXS routed experts have their own kernel below.
// PT: producer threads.  256: a thread dequantises both 32-column sub-blocks of its row's k-step, two
// blocks share an SM (big grids).  512: two threads share a row, one sub-block each, one block per
// SM - for grids that do not fill the machine (a shard of few experts, the shared expert), where a
// block's own speed is what counts.
template <int FMT, int PT>
__global__ void __launch_bounds__(PT + 32, PT == 256 ? 2 : 1)
gateup_mma_kernel(const uint8_t* __restrict__ gate_tiles, const uint8_t* __restrict__ up_tiles,
                  const __half* __restrict__ xb, const float* __restrict__ x_inv_scale,
                  const uint32_t* __restrict__ pairs, const MmaItem* __restrict__ items,
                  const uint32_t* __restrict__ n_items_ptr, float* __restrict__ h,
                  __nv_bfloat16* __restrict__ hb, float* __restrict__ hp, qkm_dims d, uint32_t* __restrict__ status) {
    if (blockIdx.x >= *n_items_ptr) return;
    constexpr int kSt = pf::kStages;
    static_assert(FMT == QKM_TYPE_Q8_0 || (FMT == QKM_TYPE_IQ4_XS && PT == 512), "IQ3_XXS has its own kernel (gateup_iq3_kernel)");
    constexpr int kTile = FMT == QKM_TYPE_IQ4_XS ? kTileIq4 : kTileQ8;
    __shared__ float s_kv[16];
    if (FMT == QKM_TYPE_IQ4_XS && threadIdx.x < 16) s_kv[threadIdx.x] = (float)c_iq4_values[threadIdx.x];
    extern __shared__ __align__(1024) uint8_t smem_dyn[];
    __shared__ __align__(8) unsigned long long s_bar[2 * kSt + 1];  // empty[stage], full[stage], done
    __shared__ uint32_t s_tmem;
    uint8_t* smem = reinterpret_cast<uint8_t*>(((uintptr_t)smem_dyn + 1023) & ~(uintptr_t)1023);
    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31u;
    const MmaItem it = items[blockIdx.x];
    const uint32_t n = it.n, n_mma = (n + 15u) & ~15u;
    const uint32_t KB = d.n_embd / 256, RT16 = d.n_ff / 16, KS = d.n_embd / 64;

    if (tid == 0) {
        for (int s = 0; s < kSt; ++s) {
            mbar_init(smem_addr(&s_bar[s]), 1);                            // empty: one commit
            mbar_init(smem_addr(&s_bar[kSt + s]), PT);   // full: every producer thread
        }
        mbar_init(smem_addr(&s_bar[2 * kSt]), 1);
        mbar_fence_init();
    }
    if (warp == 0) { umma::tmem_alloc(smem_addr(&s_tmem), 256); umma::tmem_relinquish(); }
    umma::fence_before_sync();
    __syncthreads();
    umma::fence_after_sync();
    const uint32_t tmem = s_tmem;
    const uint32_t idesc = umma::instr_desc_f16(n_mma);
    bool timed_out = false;

    // producer role of this thread: row r of the gate (threads 0..127 of each 256) or up (128..255) tile;
    // with 512 producers, threads 256.. take the second sub-block of the k-step
    const uint32_t r = tid & 127u, mat = (tid >> 7) & 1u, half = tid >> 8;
    const uint32_t rowidx = it.rt * 128u + r, rt16 = rowidx >> 4, r16 = rowidx & 15u;
    const uint8_t* wt = (mat ? up_tiles : gate_tiles) + (size_t)it.expert * KB * RT16 * kTile;

    // activation rows of this block's pairs (one dependent load less per k-step)
    // per column (pair) of this block: its x row, the scale that undoes the row's power-of-two
    // scaling, and where its h row goes in the [token][slot] layout
    __shared__ const __half* s_row[pf::kNT];
    __shared__ float s_inv[pf::kNT];
    __shared__ uint32_t s_hrow[pf::kNT];
    for (uint32_t i = tid; i < n; i += PT + 32) {
        const uint32_t pr = pairs[it.pair_off + i], tok = pr >> 4;
        s_row[i] = xb + (size_t)tok * d.n_embd;
        s_inv[i] = x_inv_scale[tok];
        s_hrow[i] = tok * (d.n_used + 1) + (pr & 15u);
    }
    __syncthreads();
    if (tid >= PT) {
        // ---- MMA issuer warp
        if (lane == 0) {
            for (uint32_t ks = 0; ks < KS; ++ks) {
                const uint32_t stage = ks % kSt;
                if (!mbar_wait_bounded(smem_addr(&s_bar[kSt + stage]), (ks / kSt) & 1u)) timed_out = true;
                umma::fence_after_sync();
                const uint32_t a_g = smem_addr(smem + stage * 3 * pf::kTileBytes), a_u = a_g + pf::kTileBytes, b = a_g + 2 * pf::kTileBytes;
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const bool acc = (ks | (uint32_t)j) != 0;
                    umma::mma_f16_ss(tmem, umma::smem_desc(a_g + 32 * j), umma::smem_desc(b + 32 * j), idesc, acc);
                    umma::mma_f16_ss(tmem + 128, umma::smem_desc(a_u + 32 * j), umma::smem_desc(b + 32 * j), idesc, acc);
                }
                umma::commit(smem_addr(&s_bar[stage]));
                if (ks + 1 == KS) umma::commit(smem_addr(&s_bar[2 * kSt]));
            }
        }
    } else {
    // ---- producer warps
    BRegs breg = fetch_b<__half, PT>(s_row, n, n_mma, 0);
    for (uint32_t ks = 0; ks < KS; ++ks) {
        const uint32_t stage = ks % kSt;
        BRegs bnext{};
        if (ks + 1 < KS) bnext = fetch_b<__half, PT>(s_row, n, n_mma, (ks + 1) * 64);
        if (ks >= (uint32_t)kSt)
            if (!mbar_wait_bounded(smem_addr(&s_bar[stage]), ((ks / kSt) - 1) & 1u)) timed_out = true;
        uint8_t* st = smem + stage * 3 * pf::kTileBytes;
        const uint8_t* tile = wt + ((size_t)(ks >> 2) * RT16 + rt16) * kTile;
        if (FMT == QKM_TYPE_IQ4_XS) produce_iq4_f16(load_iq4(tile, r16, ks & 3u, half), ks & 3u, half, s_kv, st + mat * pf::kTileBytes, r);
        else if (PT == 256) produce_q8<true, 0, 2>(tile, r16, ks & 3u, st + mat * pf::kTileBytes, r);
        else if (half == 0) produce_q8<true, 0, 1>(tile, r16, ks & 3u, st + mat * pf::kTileBytes, r);
        else produce_q8<true, 1, 2>(tile, r16, ks & 3u, st + mat * pf::kTileBytes, r);
        store_b<PT>(st + 2 * pf::kTileBytes, breg, n_mma);
        breg = bnext;
        umma::fence_smem_to_async();
        mbar_arrive(smem_addr(&s_bar[kSt + stage]));
    }
    if (!mbar_wait_bounded(smem_addr(&s_bar[2 * kSt]), 0)) timed_out = true;
    umma::fence_after_sync();

    // epilogue: warp w reads TMEM lanes 32*(w&3).. (rows) and every (PT/128)-th 16-column block
    {
        const uint32_t lg = warp & 3u, row = 32 * lg + lane;
        const uint32_t r_ff = it.rt * 128u + row;
        for (uint32_t cb = warp >> 2; cb < n_mma / 16; cb += PT / 128) {
            uint32_t vg[16], vu[16];
            umma::tmem_ld16(tmem + ((32 * lg) << 16) + cb * 16, vg);
            umma::tmem_ld16(tmem + ((32 * lg) << 16) + 128 + cb * 16, vu);
            umma::tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 16; ++i) {
                const uint32_t col = cb * 16 + i;
                if (col < n) {
                    const float us = s_inv[col];   // undo the per-token power-of-two scale of x
                    const float hv = swiglu(__uint_as_float(vg[i]) * us, __uint_as_float(vu[i]) * us);
                    if (hp) hp[(size_t)(it.pair_off + col) * d.n_ff + r_ff] = hv;   // f32 by pair position: converted to scaled f16 rows later
                    else hb[(size_t)(it.pair_off + col) * d.n_ff + r_ff] = __float2bfloat16_rn(hv);
                    if (h) h[(size_t)s_hrow[col] * d.n_ff + r_ff] = hv;
                }
            }
        }
    }
    }  // producer / epilogue warps
    umma::fence_before_sync();
    // any thread's wait that ran out counts (the MMA issuer's too, not only thread 0's)
    const int any_timed_out = __syncthreads_or(timed_out ? 1 : 0);
    if (warp == 0) umma::tmem_dealloc(tmem, 256);
    if (any_timed_out && tid == 0) atomicExch(status, (uint32_t)kStatusWaitTimeout);
}

// ---- gate/up + SwiGLU, IQ3_XXS, table-driven producers -------------------------------------------------
// The same GEMM as gateup_mma_kernel<QKM_TYPE_IQ3_XXS>, same operands and the same bits out, with the
// dequantisation cut to about two instructions per weight:
//   * one 64 KB table image at shared address 0x10000, 256 rows of 256 bytes.  Bytes [0,128) of row i:
//     the four magnitudes of grid entry i as f16, once per lane column (16 columns of 8 bytes: a
//     64-bit load of a half-warp never conflicts).  Bytes [128,256) of row i: the sign masks of the
//     8-weight sign code i & 127 - four words, bit 15 / bit 31 set for a negative weight - once per
//     lane column (8 columns of 16 bytes: a 128-bit load of a quarter-warp never conflicts).
//   * a look-up address is one byte permute: [column byte, index byte, 0x01, 0x00]; no shifts, masks
//     or adds (the sign code's eighth bit is whatever follows it in the aux word: rows 128..255
//     repeat the masks of rows 0..127).
//   * per 8 weights: 3 permutes, 3 loads, 4 packed multiplies by the sub-block scale, 4 XORs, 1 store.
//   * the dequantised weights never touch shared memory: a producer thread owns one weight row (one
//     tensor-memory lane) and writes its 32 columns of the k-step with two tcgen05.st; the MMA takes
//     its A operand from tensor memory (lane = row, two f16 per 32-bit column) and only the x tile
//     (B) from shared memory.  Shared-memory bandwidth is then spent on the table look-ups and on B,
//     not on writing and re-reading the 32 KB of A per k-step.
// 512 producer threads (row, matrix, 32-column half of the k-step), one block per SM, three stages
// of (gate and up weights: 64 tensor-memory columns; x tile: 16 KB of shared memory); a block walks
// items blockIdx.x, + gridDim.x, ... and keeps the table.  The accumulators of the next item are
// written only after every producer has read the previous item's (its arrival on the first
// k-step's barrier comes after its epilogue).
namespace pq {
constexpr int kProducers = 512;
constexpr int kBlock = kProducers + 32;
constexpr int kStages = 3;
constexpr uint32_t kTab = 0x10000u, kTabBytes = 0x10000u;
constexpr uint32_t kStage0 = 0x20000u;                                   // x tiles follow the table
constexpr uint32_t kEnd = kStage0 + kStages * pf::kTileBytes;
constexpr uint32_t kTmemCols = 512, kTmemA = 256;                        // accumulators [0,256), A stages [256,448)
__device__ __forceinline__ uint32_t stage_addr(uint32_t s) { return kStage0 + s * pf::kTileBytes; }
}  // namespace pq

size_t gateup_iq3_table_bytes() { return pq::kTabBytes; }

__global__ void gateup_iq3_table_kernel(uint8_t* __restrict__ out) {
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;   // one 4-byte word each
    if (i >= pq::kTabBytes / 4) return;
    const uint32_t row = i >> 6, w = i & 63u;
    uint32_t v;
    if (w < 32) {   // column w / 2, magnitudes 2 (w & 1) and 2 (w & 1) + 1
        const uint32_t g = c_iq3_grid[row] >> (16 * (w & 1u));
        const __half2 m = __floats2half2_rn((float)(g & 0xFFu), (float)((g >> 8) & 0xFFu));
        v = *reinterpret_cast<const uint32_t*>(&m);
    } else {        // column (w - 32) / 4, weights 2j and 2j + 1 of the group
        const uint32_t sg = signs8(row & 127u), j = w & 3u;
        v = (((sg >> (2 * j)) & 1u) ? 0x8000u : 0u) | (((sg >> (2 * j + 1)) & 1u) ? 0x80000000u : 0u);
    }
    reinterpret_cast<uint32_t*>(out)[i] = v;
}

cudaError_t launch_gateup_iq3_table(const Launch& L, uint8_t* out) {
    gateup_iq3_table_kernel<<<pq::kTabBytes / 4 / 256, 256, 0, L.stream>>>(out);
    L.count();
    return cudaGetLastError();
}

__device__ __forceinline__ uint32_t prmt_b32(uint32_t a, uint32_t b, uint32_t sel) {
    uint32_t r;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(sel));
    return r;
}
__device__ __forceinline__ void sts128(uint32_t addr, const uint4& v) {
    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}
__device__ __forceinline__ void named_sync(uint32_t id, uint32_t n_threads) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(n_threads) : "memory");
}
__device__ __forceinline__ uint32_t hmul2_bits(uint32_t a, __half2 b) {
    const __half2 v = __hmul2(*reinterpret_cast<const __half2*>(&a), b);
    return *reinterpret_cast<const uint32_t*>(&v);
}

// 32 lanes x 8 consecutive 32-bit columns of tensor memory: thread i of the warp writes lane (base lane + i)
__device__ __forceinline__ void tmem_st8(uint32_t taddr, const uint32_t (&v)[8]) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"r"(taddr), "r"(v[0]), "r"(v[1]),
                 "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7])
                 : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
// D[tmem] (+)= A[tmem] * B[smem]: A is 128 lanes (rows) x 8 columns (16 f16), B a K-major shared-memory tile
__device__ __forceinline__ void mma_f16_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t bdesc, uint32_t idesc, bool accumulate) {
    const uint32_t acc = accumulate ? 1u : 0u;
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n"
        "}\n" ::"r"(tmem_d), "r"(tmem_a), "l"(bdesc), "r"(idesc), "r"(acc)
        : "memory");
}

// The quant bytes one thread needs of its row's 256-column block, packed: ix[t][p] holds the index
// pairs of group t for k-steps 2p (low half) and 2p + 1 (high half) of the thread's 32-column
// half j; ax[q] is the aux word of sub-block 2q + j.
struct Iq3Block { uint32_t ix[4][2]; uint32_t ax[4]; uint32_t dbits; };
__device__ __forceinline__ Iq3Block load_iq3_block(const uint8_t* __restrict__ tile, uint32_t r16, uint32_t j) {
    const uint32_t g = r16 & 7u, hf = r16 >> 3;
    Iq3Block b;
#pragma unroll
    for (int t = 0; t < 4; ++t) {   // the tile keeps the even sub-blocks' pairs in the first 8 bytes, the odd ones' in the last 8
        const uint2 v = *reinterpret_cast<const uint2*>(tile + hf * 512 + (4 * g + t) * 16 + 8 * j);
        b.ix[t][0] = v.x; b.ix[t][1] = v.y;
    }
    const uint4 a = *reinterpret_cast<const uint4*>(tile + 1024 + 256 * j + 16 * r16);
    b.ax[0] = a.x; b.ax[1] = a.y; b.ax[2] = a.z; b.ax[3] = a.w;
    b.dbits = *reinterpret_cast<const uint16_t*>(tile + 1536 + 2 * r16);
    return b;
}
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, uint32_t src_bytes) {   // src_bytes 0: zero fill
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait_all_but_one() { asm volatile("cp.async.wait_group 1;" ::: "memory"); }

__global__ void __launch_bounds__(pq::kBlock, 1)
gateup_iq3_kernel(const uint8_t* __restrict__ gate_tiles, const uint8_t* __restrict__ up_tiles,
                  const __half* __restrict__ xb, const float* __restrict__ x_inv_scale,
                  const uint32_t* __restrict__ pairs, const MmaItem* __restrict__ items,
                  const uint32_t* __restrict__ n_items_ptr, float* __restrict__ h,
                  __nv_bfloat16* __restrict__ hb, float* __restrict__ hp, qkm_dims d, const uint8_t* __restrict__ table,
                  uint32_t* __restrict__ status) {
    constexpr int kSt = pq::kStages, PT = pq::kProducers;
    const uint32_t n_items = *n_items_ptr;
    if (blockIdx.x >= n_items) return;
    extern __shared__ __align__(1024) uint8_t smem_dyn[];
    __shared__ __align__(8) unsigned long long s_bar[2 * kSt + 2];  // empty[stage], full[stage], done, table
    __shared__ uint32_t s_tmem;
    __shared__ float s_inv[2][pf::kNT];
    __shared__ uint32_t s_hrow[2][pf::kNT];
    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31u;
    {   // the fixed addresses must lie inside the dynamic area
        const uint32_t dyn_base = smem_addr(smem_dyn);
        uint32_t dyn_size;
        asm("mov.u32 %0, %%dynamic_smem_size;" : "=r"(dyn_size));
        if (dyn_base > pq::kTab || dyn_base + dyn_size < pq::kEnd) {
            if (tid == 0) atomicExch(status, (uint32_t)kStatusBadLayout);
            return;
        }
    }
    const uint32_t KB = d.n_embd / 256, RT16 = d.n_ff / 16, KS = d.n_embd / 64;
    const uint32_t bar_empty = smem_addr(&s_bar[0]), bar_full = smem_addr(&s_bar[kSt]);
    const uint32_t bar_done = smem_addr(&s_bar[2 * kSt]), bar_tab = smem_addr(&s_bar[2 * kSt + 1]);

    if (tid == 0) {
        for (int s = 0; s < kSt; ++s) {
            mbar_init(bar_empty + 8 * s, 1);     // one commit
            mbar_init(bar_full + 8 * s, PT / 32); // one arrival per producer warp
        }
        mbar_init(bar_done, 1);
        mbar_init(bar_tab, 1);
        mbar_fence_init();
    }
    if (warp == 0) { umma::tmem_alloc(smem_addr(&s_tmem), pq::kTmemCols); umma::tmem_relinquish(); }
    umma::fence_before_sync();
    __syncthreads();
    umma::fence_after_sync();
    if (tid == 0) {
        mbar_expect_tx(bar_tab, pq::kTabBytes);
        for (uint32_t i = 0; i < 4; ++i) bulk_g2s(pq::kTab + i * 16384u, table + i * 16384u, 16384u, bar_tab);
    }
    const uint32_t tmem = s_tmem;
    bool timed_out = false;

    if (tid >= PT) {
        // ---- MMA issuer warp: the whole warp walks the loop (addresses stay warp-uniform), one
        // elected lane issues
        {
            const bool leader = umma::elect_one();
            uint32_t stage = 0, phase = 0;
            for (uint32_t item = blockIdx.x; item < n_items; item += gridDim.x) {
                const uint32_t idesc = umma::instr_desc_f16((items[item].n + 15u) & ~15u);
                for (uint32_t ks = 0; ks < KS; ++ks) {
                    if (!mbar_wait_bounded(bar_full + 8 * stage, phase)) timed_out = true;
                    umma::fence_after_sync();
                    const uint64_t d_b = umma::smem_desc(pq::stage_addr(stage));
                    const uint32_t t_g = tmem + pq::kTmemA + stage * 64u, t_u = t_g + 32u;
                    if (leader) {
#pragma unroll
                        for (int j = 0; j < 4; ++j) {   // 16 columns of K further: 8 tensor-memory columns, 32 bytes of the x tile
                            const bool acc = (ks | (uint32_t)j) != 0;
                            mma_f16_ts(tmem, t_g + 8 * j, d_b + 2 * j, idesc, acc);
                            mma_f16_ts(tmem + 128, t_u + 8 * j, d_b + 2 * j, idesc, acc);
                        }
                        umma::commit(bar_empty + 8 * stage);
                        if (ks + 1 == KS) umma::commit(bar_done);
                    }
                    __syncwarp();
                    if (++stage == (uint32_t)kSt) { stage = 0; phase ^= 1u; }
                }
            }
        }
    } else {
    // ---- producer warps: thread = (row r, matrix, 32-column half j of each k-step)
    const uint32_t r = tid & 127u, mat = (tid >> 7) & 1u, j = tid >> 8;
    const uint32_t mconst = 0x00010000u | ((lane & 15u) * 8u);
    const uint32_t sconst = 0x00010000u | (128u + (lane & 7u) * 16u);
    // this thread's 16 columns of its tensor-memory lane (row r): matrix, then the 32-column half
    const uint32_t a_lane = tmem + ((r & ~31u) << 16) + pq::kTmemA + mat * 32u + j * 16u;
    // N operand: chunks tid and tid + 512 of the x tile (row = chunk / 8), copied asynchronously
    const uint32_t b_row0 = tid >> 3, b_row1 = b_row0 + 64, b_c = tid & 7u;
    const uint32_t b_off0 = umma::sw128_chunk(b_row0, b_c), b_off1 = umma::sw128_chunk(b_row1, b_c);
    if (!mbar_wait_bounded(bar_tab, 0)) timed_out = true;

    // What an item needs before its first k-step - its record, the first weight bytes, the x rows of
    // this thread's two chunks, the per-column scale and h offset - is fetched while the item
    // before it drains (MMA tail and epilogue); s_inv / s_hrow are double-buffered for that.
    struct ItemHead {
        MmaItem it;
        Iq3Block blk;
        const uint8_t* wt;
        const __half* b_src0;
        const __half* b_src1;
        uint32_t r16;
    };
    auto fetch_head = [&](uint32_t item, uint32_t buf) -> ItemHead {
        ItemHead hd;
        hd.it = items[item];
        const uint32_t rowidx = hd.it.rt * 128u + r;
        hd.r16 = rowidx & 15u;
        hd.wt = (mat ? up_tiles : gate_tiles) + ((size_t)hd.it.expert * KB * RT16 + (rowidx >> 4)) * kTileIq3;
        hd.blk = load_iq3_block(hd.wt, hd.r16, j);
        // rows >= n are zero-filled, rows >= n_mma not written
        hd.b_src0 = xb + 8 * b_c;
        hd.b_src1 = hd.b_src0;
        if (b_row0 < hd.it.n) hd.b_src0 += (size_t)(pairs[hd.it.pair_off + b_row0] >> 4) * d.n_embd;
        if (b_row1 < hd.it.n) hd.b_src1 += (size_t)(pairs[hd.it.pair_off + b_row1] >> 4) * d.n_embd;
        for (uint32_t i = tid; i < hd.it.n; i += PT) {
            const uint32_t pr = pairs[hd.it.pair_off + i], tok = pr >> 4;
            s_inv[buf][i] = x_inv_scale[tok];
            s_hrow[buf][i] = (tok * (d.n_used + 1) + (pr & 15u)) * d.n_ff;   // element offset of the pair's h row
        }
        return hd;
    };
    uint32_t stage = 0, phase = 0, gs = 0, iter = 0;
    ItemHead head = fetch_head(blockIdx.x, 0);
    named_sync(1, PT);
    for (uint32_t item = blockIdx.x; item < n_items; item += gridDim.x, ++iter) {
        const MmaItem it = head.it;
        const uint32_t n = it.n, n_mma = (n + 15u) & ~15u;
        const uint32_t r16 = head.r16;
        const uint8_t* wt = head.wt;
        Iq3Block cur = head.blk;
        const __half* b_src0 = head.b_src0;
        const __half* b_src1 = head.b_src1;
        const uint32_t b_sz0 = b_row0 < n ? 16u : 0u, b_sz1 = b_row1 < n ? 16u : 0u;
        const bool b_do0 = b_row0 < n_mma, b_do1 = b_row1 < n_mma;
        const uint32_t buf = iter & 1u;
        // the first k-step's x tile
        if (gs >= (uint32_t)kSt)
            if (!mbar_wait_bounded(bar_empty + 8 * stage, phase ^ 1u)) timed_out = true;
        {
            const uint32_t st = pq::stage_addr(stage);
            if (b_do0) cp_async16(st + b_off0, b_src0, b_sz0);
            if (b_do1) cp_async16(st + b_off1, b_src1, b_sz1);
            cp_async_commit();
        }
        for (uint32_t kb = 0; kb < KB; ++kb) {
            Iq3Block nxt = cur;
            if (kb + 1 < KB) nxt = load_iq3_block(wt + (size_t)(kb + 1) * RT16 * kTileIq3, r16, j);
            const float dd = f16_bits_to_f32(cur.dbits);
            const float d2 = dd * 0.5f, d4 = dd * 0.25f;
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const uint32_t ks = kb * 4 + q;
                const uint32_t st = pq::stage_addr(stage);
                // the next k-step's x tile goes to the next stage, once the MMAs that read it are done
                uint32_t stage1 = stage + 1, phase1 = phase;
                if (stage1 == (uint32_t)kSt) { stage1 = 0; phase1 ^= 1u; }
                if (ks + 1 < KS) {
                    if (gs + 1 >= (uint32_t)kSt)
                        if (!mbar_wait_bounded(bar_empty + 8 * stage1, phase1 ^ 1u)) timed_out = true;
                    const uint32_t st1 = pq::stage_addr(stage1);
                    if (b_do0) cp_async16(st1 + b_off0, b_src0 + (ks + 1) * 64, b_sz0);
                    if (b_do1) cp_async16(st1 + b_off1, b_src1 + (ks + 1) * 64, b_sz1);
                }
                cp_async_commit();
                // sub-block 2q + j: scale d (2s + 1) / 4, exact in f32, one rounding to f16
                const uint32_t aux = cur.ax[q];
                const float sf = __uint_as_float(0x4B000000u | (aux >> 28)) - 8388608.f;
                const __half2 db2 = __float2half2_rn(fmaf(sf, d2, d4));
                const uint32_t sel_a = (q & 1) ? 0x7624u : 0x7604u, sel_b = (q & 1) ? 0x7634u : 0x7614u;
#pragma unroll
                for (int tp = 0; tp < 4; tp += 2) {   // two 8-weight groups at a time: all six look-ups first
                    uint2 m0[2], m1[2];
                    uint4 sg[2];
#pragma unroll
                    for (int u = 0; u < 2; ++u) {
                        const int t = tp + u;
                        const uint32_t w = cur.ix[t][q >> 1];
                        m0[u] = lds64(prmt_b32(w, mconst, sel_a));
                        m1[u] = lds64(prmt_b32(w, mconst, sel_b));
                        sg[u] = lds128(prmt_b32(t ? aux >> (7 * t) : aux, sconst, 0x7604u));
                    }
                    uint32_t o[8];   // groups tp, tp + 1 -> columns 4 tp .. 4 tp + 7 of the thread's 16
#pragma unroll
                    for (int u = 0; u < 2; ++u) {
                        o[4 * u + 0] = hmul2_bits(m0[u].x, db2) ^ sg[u].x;
                        o[4 * u + 1] = hmul2_bits(m0[u].y, db2) ^ sg[u].y;
                        o[4 * u + 2] = hmul2_bits(m1[u].x, db2) ^ sg[u].z;
                        o[4 * u + 3] = hmul2_bits(m1[u].y, db2) ^ sg[u].w;
                    }
                    tmem_st8(a_lane + stage * 64u + 4 * tp, o);
                }
                tmem_st_wait();
                cp_async_wait_all_but_one();   // this k-step's x tile has landed (the next one's may be in flight)
                umma::fence_smem_to_async();   // the x tile (generic-proxy writes) before the tensor core reads it
                umma::fence_before_sync();
                __syncwarp();
                if (lane == 0) mbar_arrive(bar_full + 8 * stage);
                ++gs;
                stage = stage1; phase = phase1;
            }
            cur = nxt;
        }
        if (item + gridDim.x < n_items) head = fetch_head(item + gridDim.x, buf ^ 1u);
        if (!mbar_wait_bounded(bar_done, iter & 1u)) timed_out = true;
        umma::fence_after_sync();

        // epilogue: warp w reads TMEM lanes 32*(w&3).. (rows) and every fourth 16-column block.
        // silu with the fast exponential and division: their error (a few ulp) is far below the f16
        // rounding of the operands, and the epilogue is a fifth of the kernel's instructions otherwise
        {
            const uint32_t lg = warp & 3u, row = 32 * lg + lane;
            const uint32_t r_ff = it.rt * 128u + row;
            for (uint32_t cb = warp >> 2; cb < n_mma / 16; cb += PT / 128) {
                uint32_t vg[16], vu[16];
                umma::tmem_ld16(tmem + ((32 * lg) << 16) + cb * 16, vg);
                umma::tmem_ld16(tmem + ((32 * lg) << 16) + 128 + cb * 16, vu);
                umma::tmem_ld_wait();
                const size_t hoff = (size_t)(it.pair_off + cb * 16) * d.n_ff + r_ff;
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    const uint32_t col = cb * 16 + i;
                    if (col < n) {
                        const float us = s_inv[buf][col];   // undo the per-token power-of-two scale of x
                        const float g = __uint_as_float(vg[i]) * us, u = __uint_as_float(vu[i]) * us;
                        const float hv = __fdividef(g, 1.0f + __expf(-g)) * u;
                        if (hp) hp[hoff + (size_t)i * d.n_ff] = hv;   // f32 by pair position: converted to scaled f16 rows later
                        else hb[hoff + (size_t)i * d.n_ff] = __float2bfloat16_rn(hv);
                        if (h) h[(size_t)s_hrow[buf][col] + r_ff] = hv;
                    }
                }
            }
            umma::fence_before_sync();   // the accumulators are read before this thread's next arrival
        }
        named_sync(1, PT);   // the next item's columns are written, this item's are read
    }
    }  // producer / epilogue warps
    umma::fence_before_sync();
    const int any_timed_out = __syncthreads_or(timed_out ? 1 : 0);
    if (warp == 0) umma::tmem_dealloc(tmem, pq::kTmemCols);
    if (any_timed_out && tid == 0) atomicExch(status, (uint32_t)kStatusWaitTimeout);
}

static cudaError_t gateup_iq3_launch(const Launch& L, const qkm_dims& d, const void* gate_tiles, const void* up_tiles,
                                     const void* xb, const float* x_inv_scale, const uint32_t* pairs, const MmaItem* items,
                                     const uint32_t* n_items, uint32_t max_items, float* h, void* hb, float* hp, const uint8_t* table,
                                     uint32_t* status) {
    static int n_sms = 0;
    if (n_sms == 0) {
        int dev = 0, v = 0;
        if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || v <= 0) v = 148;
        n_sms = v;
    }
    const size_t smem = pq::kEnd;   // reaches from wherever the dynamic area starts to the end of the fixed layout
    cudaError_t e = cudaFuncSetAttribute(gateup_iq3_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    const uint32_t grid = max_items < (uint32_t)n_sms ? max_items : (uint32_t)n_sms;
    gateup_iq3_kernel<<<grid, pq::kBlock, smem, L.stream>>>(
        (const uint8_t*)gate_tiles, (const uint8_t*)up_tiles, (const __half*)xb, x_inv_scale, pairs, items, n_items, h,
        (__nv_bfloat16*)hb, hp, d, table, status);
    L.count();
    return cudaGetLastError();
}

// ---- down -------------------------------------------------------------------------------------------------
// FMT: QKM_TYPE_IQ4_XS or QKM_TYPE_Q6_K (routed), QKM_TYPE_Q8_0 (shared).  contrib[pair position][n_embd].
// F16H: the hidden rows are f16, each scaled by a power of two (h_inv_scale undoes it in the epilogue), and the
// weights are dequantised to f16 as well (Q8_0, Q6_K); else both are bf16.
template <int FMT, bool F16H = false>
__global__ void __launch_bounds__(pf::kBlock, 2)
down_mma_kernel(const uint8_t* __restrict__ tiles, const __nv_bfloat16* __restrict__ hb,
                const qkm_sel* __restrict__ sel, const uint32_t* __restrict__ pairs,
                const MmaItem* __restrict__ items, const uint32_t* __restrict__ n_items_ptr,
                float* __restrict__ contrib, qkm_dims d, uint32_t row_tiles, uint32_t* __restrict__ status,
                const float* __restrict__ h_inv_scale = nullptr) {
    static_assert(!F16H || FMT != QKM_TYPE_IQ4_XS, "f16 hidden rows: Q8_0 / Q6_K weights here, IQ4_XS in down_iq4_kernel");
    if (blockIdx.x * row_tiles >= *n_items_ptr) return;
    constexpr int kTile = FMT == QKM_TYPE_IQ4_XS ? kTileIq4 : FMT == QKM_TYPE_Q6_K ? kTileQ6 : kTileQ8;
    extern __shared__ __align__(1024) uint8_t smem_dyn[];
    __shared__ __align__(8) unsigned long long s_bar[2 * pf::kStages + 1];  // empty[stage], full[stage], done
    __shared__ uint32_t s_tmem;
    uint8_t* smem = reinterpret_cast<uint8_t*>(((uintptr_t)smem_dyn + 1023) & ~(uintptr_t)1023);
    uint32_t* s_pair = reinterpret_cast<uint32_t*>(smem + pf::kStages * 2 * pf::kTileBytes);   // [256][32], IQ4_XS only
    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31u;
    const MmaItem it = items[blockIdx.x * row_tiles];   // items of one (expert, pair tile) are consecutive row tiles
    const uint32_t n = it.n, n_mma = (n + 15u) & ~15u;
    const uint32_t KB = d.n_ff / 256, RT16 = d.n_embd / 16, KS = d.n_ff / 64;

    if (FMT == QKM_TYPE_IQ4_XS)
        for (uint32_t i = tid; i < 256 * 32; i += pf::kThreads) {
            const uint32_t b = i >> 5;
            const __nv_bfloat162 v = __floats2bfloat162_rn((float)c_iq4_values[b & 15u], (float)c_iq4_values[b >> 4]);
            s_pair[i] = *reinterpret_cast<const uint32_t*>(&v);
        }
    const uint8_t* s_pair_lane = reinterpret_cast<const uint8_t*>(s_pair + lane);
    if (tid == 0) {
        for (int s = 0; s < pf::kStages; ++s) {
            mbar_init(smem_addr(&s_bar[s]), 1);                            // empty: one commit
            mbar_init(smem_addr(&s_bar[pf::kStages + s]), pf::kThreads);   // full: every producer thread
        }
        mbar_init(smem_addr(&s_bar[2 * pf::kStages]), 1);
        mbar_fence_init();
    }
    if (warp == 0) { umma::tmem_alloc(smem_addr(&s_tmem), 128); umma::tmem_relinquish(); }
    umma::fence_before_sync();
    __syncthreads();
    umma::fence_after_sync();
    const uint32_t tmem = s_tmem;
    const uint32_t idesc = F16H ? umma::instr_desc_f16(n_mma) : umma::instr_desc_bf16(n_mma);
    bool timed_out = false;

    // producer role: thread -> row (tid & 127), 32-column half (tid >> 7) of the A tile; all threads help with B
    const uint32_t r = tid & 127u;
    const uint8_t* wt = tiles + (size_t)it.expert * KB * RT16 * kTile;

    // per column (pair) of this block: its h row and its routing weight
    __shared__ const __nv_bfloat16* s_row[pf::kNT];
    __shared__ float s_wgt[pf::kNT];
    for (uint32_t i = tid; i < n; i += pf::kBlock) {
        s_row[i] = hb + (size_t)(it.pair_off + i) * d.n_ff;
        const uint32_t pr = pairs[it.pair_off + i], tok = pr >> 4, slot = pr & 15u;
        s_wgt[i] = (slot < d.n_used ? sel[tok].w[slot] : sel[tok].w_shared) * (F16H ? h_inv_scale[it.pair_off + i] : 1.0f);
    }
    __syncthreads();
    // The block walks `row_tiles` consecutive 128-row tiles of the same expert and pairs: tables,
    // barriers and tensor memory are set up once; gs counts k-steps across the tiles.
    if (tid >= pf::kThreads) {
        // ---- MMA issuer warp
        if (lane == 0) {
            for (uint32_t gs = 0; gs < row_tiles * KS; ++gs) {
                const uint32_t stage = gs % pf::kStages, ks = gs % KS;
                if (!mbar_wait_bounded(smem_addr(&s_bar[pf::kStages + stage]), (gs / pf::kStages) & 1u)) timed_out = true;
                umma::fence_after_sync();
                const uint32_t a = smem_addr(smem + stage * 2 * pf::kTileBytes), b = a + pf::kTileBytes;
#pragma unroll
                for (int j = 0; j < 4; ++j)
                    umma::mma_f16_ss(tmem, umma::smem_desc(a + 32 * j), umma::smem_desc(b + 32 * j), idesc, (ks | (uint32_t)j) != 0);
                umma::commit(smem_addr(&s_bar[stage]));
                if (ks + 1 == KS) umma::commit(smem_addr(&s_bar[2 * pf::kStages]));
            }
        }
    } else {
    // ---- producer warps
    const uint32_t jhalf = tid >> 7;   // which 32-column half of the k-step this thread expands
    for (uint32_t sub = 0; sub < row_tiles; ++sub) {
    const uint32_t rowidx = (it.rt + sub) * 128u + r, rt16 = rowidx >> 4, r16 = rowidx & 15u;
    BRegs breg = fetch_b(s_row, n, n_mma, 0);
    Iq4Raw raw{};
    if (FMT == QKM_TYPE_IQ4_XS) raw = load_iq4(wt + (size_t)rt16 * kTile, r16, 0, jhalf);
    for (uint32_t ks = 0; ks < KS; ++ks) {
        const uint32_t gs = sub * KS + ks, stage = gs % pf::kStages;
        BRegs bnext{};
        Iq4Raw next{};
        if (ks + 1 < KS) {
            bnext = fetch_b(s_row, n, n_mma, (ks + 1) * 64);
            if (FMT == QKM_TYPE_IQ4_XS)
                next = load_iq4(wt + ((size_t)((ks + 1) >> 2) * RT16 + rt16) * kTile, r16, (ks + 1) & 3u, jhalf);
        }
        if (gs >= (uint32_t)pf::kStages)
            if (!mbar_wait_bounded(smem_addr(&s_bar[stage]), ((gs / pf::kStages) - 1) & 1u)) timed_out = true;
        uint8_t* st = smem + stage * 2 * pf::kTileBytes;
        if (FMT == QKM_TYPE_IQ4_XS) {
            produce_iq4(raw, ks & 3u, jhalf, s_pair_lane, st, r);
            raw = next;
        } else if (FMT == QKM_TYPE_Q6_K) {
            produce_q6k<F16H>(wt + ((size_t)(ks >> 2) * RT16 + rt16) * kTile, r16, ks & 3u, jhalf, st, r);
        } else {
            const uint8_t* tile = wt + ((size_t)(ks >> 2) * RT16 + rt16) * kTile;
            if (tid < 128) produce_q8<F16H, 0, 1>(tile, r16, ks & 3u, st, r);
            else produce_q8<F16H, 1, 2>(tile, r16, ks & 3u, st, r);
        }
        store_b(st + pf::kTileBytes, breg, n_mma);
        breg = bnext;
        umma::fence_smem_to_async();
        mbar_arrive(smem_addr(&s_bar[pf::kStages + stage]));
    }
    if (!mbar_wait_bounded(smem_addr(&s_bar[2 * pf::kStages]), sub & 1u)) timed_out = true;
    umma::fence_after_sync();
    {
        const uint32_t lg = warp & 3u, row = 32 * lg + lane;
        const uint32_t o = (it.rt + sub) * 128u + row;
        for (uint32_t cb = warp >> 2; cb < n_mma / 16; cb += 2) {
            uint32_t v[16];
            umma::tmem_ld16(tmem + ((32 * lg) << 16) + cb * 16, v);
            umma::tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 16; ++i) {
                const uint32_t col = cb * 16 + i;
                // routing weight after the full K reduction
                if (col < n) contrib[(size_t)(it.pair_off + col) * d.n_embd + o] = s_wgt[col] * __uint_as_float(v[i]);
            }
        }
    }
    umma::fence_before_sync();   // the accumulator is read out before the next tile's first MMA overwrites it
    }  // row tiles
    }  // producer / epilogue warps
    umma::fence_before_sync();
    // any thread's wait that ran out counts (the MMA issuer's too, not only thread 0's)
    const int any_timed_out = __syncthreads_or(timed_out ? 1 : 0);
    if (warp == 0) umma::tmem_dealloc(tmem, 128);
    if (any_timed_out && tid == 0) atomicExch(status, (uint32_t)kStatusWaitTimeout);
}

// ---- router logits on the tensor cores -----------------------------------------------------------------
// logits[t][e] = router[e] . x[t] with f16 operands (the router as stored when it is F16, rounded
// from F32 otherwise; x rows as written by to_f16_rows_kernel) and f32 accumulation in tensor
// memory.  These logits only pre-select: the selection kernel re-evaluates every expert within
// its error bound of the k-th in f64, so the bound has to hold, not the last bits.
// Error per logit <= (2^-11 [x rounding] + 2^-11 [router rounding] + K * 2^-22 [accumulation])
// * |w| * |x|, below 2^-9 * |w| * |x| for K <= 4096.
// Block = 128 experts (M) x up to 128 tokens (N); 256 producer threads copy both operand tiles
// into the swizzled layout, the ninth warp issues the MMAs.
constexpr int kLgStages = 4;   // stages of the logits kernel (one block per SM: it is a small grid)
constexpr int kLgDepth = 3;    // k-steps of asynchronous copies in flight

__device__ __forceinline__ void cp_async16(uint32_t smem_dst, const void* gsrc) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_dst), "l"(gsrc) : "memory");
}
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

struct LgRegs { uint4 a[4], b[4]; };

template <int TYPE>
__device__ __forceinline__ void lg_fetch(LgRegs& r, const uint8_t* __restrict__ router, const __half* __restrict__ xh,
                                         uint32_t e0, uint32_t t0, uint32_t n, uint32_t n_mma, uint32_t K, uint32_t k0) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const uint32_t qd = threadIdx.x + i * pf::kThreads, row = qd >> 3, c = qd & 7u;
        if (TYPE == QKM_TYPE_F16) {
            r.a[i] = *reinterpret_cast<const uint4*>(router + ((size_t)(e0 + row) * K + k0 + 8 * c) * 2);
        } else {
            const float4* p = reinterpret_cast<const float4*>(router + ((size_t)(e0 + row) * K + k0 + 8 * c) * 4);
            const float4 lo = p[0], hi = p[1];
            r.a[i] = make_uint4(pack16<true>(lo.x, lo.y), pack16<true>(lo.z, lo.w), pack16<true>(hi.x, hi.y), pack16<true>(hi.z, hi.w));
        }
        r.b[i] = make_uint4(0, 0, 0, 0);
        if (qd < n_mma * 8 && row < n) r.b[i] = *reinterpret_cast<const uint4*>(xh + (size_t)(t0 + row) * K + k0 + 8 * c);
    }
}

template <int TYPE>
__global__ void __launch_bounds__(pf::kBlock, 1)
logits_mma_kernel(const uint8_t* __restrict__ router, const __half* __restrict__ xh, const float* __restrict__ x_inv_scale,
                  float* __restrict__ logits_all, uint32_t n_expert, uint32_t K_all, uint32_t n_tokens, uint32_t* __restrict__ status) {
    // blockIdx.z: the column range [z, z+1) * K_all / gridDim.z; its partial logits go to part z of the output
    const uint32_t K = K_all / gridDim.z;
    float* __restrict__ logits = logits_all + (size_t)blockIdx.z * n_tokens * n_expert;
    router += (size_t)blockIdx.z * K * (TYPE == QKM_TYPE_F16 ? 2 : 4);
    xh += (size_t)blockIdx.z * K;
    extern __shared__ __align__(1024) uint8_t smem_dyn[];
    __shared__ __align__(8) unsigned long long s_bar[2 * kLgStages + 1];  // empty[stage], full[stage], done
    __shared__ uint32_t s_tmem;
    uint8_t* smem = reinterpret_cast<uint8_t*>(((uintptr_t)smem_dyn + 1023) & ~(uintptr_t)1023);
    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31u;
    const uint32_t t0 = blockIdx.x * 128u, e0 = blockIdx.y * 128u;
    const uint32_t n = min(128u, n_tokens - t0), n_mma = (n + 15u) & ~15u, KS = K / 64;
    if (tid == 0) {
        for (int s = 0; s < kLgStages; ++s) {
            mbar_init(smem_addr(&s_bar[s]), 1);
            mbar_init(smem_addr(&s_bar[kLgStages + s]), pf::kThreads);
        }
        mbar_init(smem_addr(&s_bar[2 * kLgStages]), 1);
        mbar_fence_init();
    }
    if (warp == 0) { umma::tmem_alloc(smem_addr(&s_tmem), 128); umma::tmem_relinquish(); }
    umma::fence_before_sync();
    __syncthreads();
    umma::fence_after_sync();
    const uint32_t tmem = s_tmem;
    const uint32_t idesc = umma::instr_desc_f16(n_mma);
    bool timed_out = false;
    if (tid >= pf::kThreads) {
        if (lane == 0) {
            for (uint32_t ks = 0; ks < KS; ++ks) {
                const uint32_t stage = ks % kLgStages;
                if (!mbar_wait_bounded(smem_addr(&s_bar[kLgStages + stage]), (ks / kLgStages) & 1u)) timed_out = true;
                umma::fence_after_sync();
                const uint32_t a = smem_addr(smem + stage * 2 * pf::kTileBytes), b = a + pf::kTileBytes;
#pragma unroll
                for (int j = 0; j < 4; ++j)
                    umma::mma_f16_ss(tmem, umma::smem_desc(a + 32 * j), umma::smem_desc(b + 32 * j), idesc, (ks | (uint32_t)j) != 0);
                umma::commit(smem_addr(&s_bar[stage]));
                if (ks + 1 == KS) umma::commit(smem_addr(&s_bar[2 * kLgStages]));
            }
        }
    } else {
        if (TYPE == QKM_TYPE_F16) {
            // Both operands are plain copies: 16-byte asynchronous copies straight into the
            // swizzled tiles, kLgDepth k-steps in flight, so the global-load latency of a
            // block that has the SM almost to itself (small batches) is hidden.
            auto issue = [&](uint32_t ks) {
                const uint32_t stage = ks % kLgStages;
                if (ks >= (uint32_t)kLgStages)
                    if (!mbar_wait_bounded(smem_addr(&s_bar[stage]), ((ks / kLgStages) - 1) & 1u)) timed_out = true;
                const uint32_t st = smem_addr(smem + stage * 2 * pf::kTileBytes), k0 = ks * 64;
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const uint32_t qd = tid + i * pf::kThreads, row = qd >> 3, c = qd & 7u;
                    cp_async16(st + umma::sw128_chunk(row, c), router + ((size_t)(e0 + row) * K_all + k0 + 8 * c) * 2);
                    if (qd < n_mma * 8) {
                        const uint32_t src_row = row < n ? row : 0u;   // rows past n feed accumulator columns nobody reads
                        cp_async16(st + pf::kTileBytes + umma::sw128_chunk(row, c), xh + (size_t)(t0 + src_row) * K_all + k0 + 8 * c);
                    }
                }
                cp_async_commit();
            };
            for (uint32_t ks = 0; ks < (uint32_t)kLgDepth && ks < KS; ++ks) issue(ks);
            for (uint32_t ks = 0; ks < KS; ++ks) {
                if (ks + kLgDepth < KS) issue(ks + kLgDepth); else cp_async_commit();   // keep the group count in step
                cp_async_wait<kLgDepth>();          // the copies of step ks have landed
                umma::fence_smem_to_async();
                mbar_arrive(smem_addr(&s_bar[kLgStages + ks % kLgStages]));
            }
        } else {
        LgRegs cur;
        lg_fetch<TYPE>(cur, router, xh, e0, t0, n, n_mma, K_all, 0);
        for (uint32_t ks = 0; ks < KS; ++ks) {
            const uint32_t stage = ks % kLgStages;
            if (ks >= (uint32_t)kLgStages)
                if (!mbar_wait_bounded(smem_addr(&s_bar[stage]), ((ks / kLgStages) - 1) & 1u)) timed_out = true;
            uint8_t* st = smem + stage * 2 * pf::kTileBytes;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const uint32_t qd = tid + i * pf::kThreads, row = qd >> 3, c = qd & 7u;
                *reinterpret_cast<uint4*>(st + umma::sw128_chunk(row, c)) = cur.a[i];
                if (qd < n_mma * 8) *reinterpret_cast<uint4*>(st + pf::kTileBytes + umma::sw128_chunk(row, c)) = cur.b[i];
            }
            umma::fence_smem_to_async();
            mbar_arrive(smem_addr(&s_bar[kLgStages + stage]));
            if (ks + 1 < KS) lg_fetch<TYPE>(cur, router, xh, e0, t0, n, n_mma, K_all, (ks + 1) * 64);
        }
        }
        if (!mbar_wait_bounded(smem_addr(&s_bar[2 * kLgStages]), 0)) timed_out = true;
        umma::fence_after_sync();
        const uint32_t lg = warp & 3u, e = e0 + 32 * lg + lane;
        for (uint32_t cb = warp >> 2; cb < n_mma / 16; cb += 2) {
            uint32_t v[16];
            umma::tmem_ld16(tmem + ((32 * lg) << 16) + cb * 16, v);
            umma::tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 16; ++i) {
                const uint32_t col = cb * 16 + i;
                if (col < n) logits[(size_t)(t0 + col) * n_expert + e] = __uint_as_float(v[i]) * x_inv_scale[t0 + col];
            }
        }
    }
    umma::fence_before_sync();
    // any thread's wait that ran out counts (the MMA issuer's too, not only thread 0's)
    const int any_timed_out = __syncthreads_or(timed_out ? 1 : 0);
    if (warp == 0) umma::tmem_dealloc(tmem, 128);
    if (any_timed_out && tid == 0) atomicExch(status, (uint32_t)kStatusWaitTimeout);
}

cudaError_t launch_logits_mma(const Launch& L, const qkm_dims& d, uint32_t router_type, const void* router,
                              const void* x_f16, const float* x_inv_scale, float* logits, uint32_t n_tokens,
                              uint32_t* status, uint32_t splits) {
    if (n_tokens == 0) return cudaSuccess;
    if (d.n_expert % 128 || d.n_embd % 64 || d.n_embd > 4096 || splits == 0 || (d.n_embd / 64) % splits) return cudaErrorInvalidValue;
    const size_t smem = (size_t)kLgStages * 2 * pf::kTileBytes + 1024;
    const dim3 grid((n_tokens + 127) / 128, d.n_expert / 128, splits);
    cudaError_t e;
    if (router_type == QKM_TYPE_F16) {
        e = cudaFuncSetAttribute(logits_mma_kernel<QKM_TYPE_F16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return e;
        logits_mma_kernel<QKM_TYPE_F16><<<grid, pf::kBlock, smem, L.stream>>>((const uint8_t*)router, (const __half*)x_f16, x_inv_scale, logits, d.n_expert, d.n_embd, n_tokens, status);
    } else if (router_type == QKM_TYPE_F32) {
        e = cudaFuncSetAttribute(logits_mma_kernel<QKM_TYPE_F32>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return e;
        logits_mma_kernel<QKM_TYPE_F32><<<grid, pf::kBlock, smem, L.stream>>>((const uint8_t*)router, (const __half*)x_f16, x_inv_scale, logits, d.n_expert, d.n_embd, n_tokens, status);
    } else {
        return cudaErrorInvalidValue;
    }
    L.count();
    return cudaGetLastError();
}

// ---- dense quantised GEMM through the same pipeline ----------------------------------------------------
// Y[n][M] = X[n][K] . W^T for one tile-ordered Q8_0 / IQ4_XS matrix: the matrix plays the part of a
// single expert whose "pairs" are all n rows, so down_mma_kernel does the work.  These two kernels
// prepare its inputs: X as bf16 rows, the identity pair list with unit weights, and the work list
// (row tiles of one token tile are consecutive, as the kernel's row-tile walk expects).
__global__ void __launch_bounds__(256)
dense_prepare_kernel(const float* __restrict__ x, __nv_bfloat16* __restrict__ xb, uint64_t n_elems,
                     uint32_t n_rows, uint32_t* __restrict__ pairs, qkm_sel* __restrict__ unit_sel) {
    const uint64_t i = ((uint64_t)blockIdx.x * blockDim.x + threadIdx.x) * 2;
    if (i < n_elems) {
        const float2 v = *reinterpret_cast<const float2*>(x + i);
        *reinterpret_cast<__nv_bfloat162*>(xb + i) = __floats2bfloat162_rn(v.x, v.y);
    }
    const uint64_t t = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (t < n_rows) {
        pairs[t] = (uint32_t)t << 4;        // (row, slot 0)
        unit_sel[t].ids[0] = 0;
        unit_sel[t].w[0] = 1.0f;
    }
}

__global__ void dense_plan_kernel(uint32_t n_rows, uint32_t row_tiles_total, MmaItem* __restrict__ items,
                                  uint32_t* __restrict__ n_items) {
    const uint32_t tiles = (n_rows + pf::kNT - 1) / pf::kNT;
    for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < tiles * row_tiles_total; i += gridDim.x * blockDim.x) {
        MmaItem it;
        it.expert = 0;
        it.rt = (uint16_t)(i % row_tiles_total);
        it.pair_off = (i / row_tiles_total) * pf::kNT;
        it.n = min((uint32_t)pf::kNT, n_rows - it.pair_off);
        items[i] = it;
    }
    if (blockIdx.x == 0 && threadIdx.x == 0) *n_items = tiles * row_tiles_total;
}

cudaError_t launch_dense_gemm(const Launch& L, uint32_t type, const void* tiles, uint32_t M, uint32_t K, const float* x,
                              uint32_t n_rows, float* y, void* xb, uint32_t* pairs, qkm_sel* unit_sel, MmaItem* items,
                              uint32_t* n_items, uint32_t* status) {
    if (n_rows == 0) return cudaSuccess;
    if (M % 128 || K % 256 || M / 128 > 65535) return cudaErrorInvalidValue;
    const uint64_t n_elems = (uint64_t)n_rows * K;
    dense_prepare_kernel<<<(unsigned)((n_elems / 2 + 255) / 256), 256, 0, L.stream>>>(x, (__nv_bfloat16*)xb, n_elems, n_rows, pairs, unit_sel);
    const uint32_t total = (n_rows + pf::kNT - 1) / pf::kNT * (M / 128);
    dense_plan_kernel<<<(total + 255) / 256, 256, 0, L.stream>>>(n_rows, M / 128, items, n_items);
    L.count(2);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return e;
    qkm_dims d;
    d.n_embd = M; d.n_ff = K; d.n_expert = 1; d.n_used = 1;
    return launch_down_mma(L, d, type, tiles, xb, unit_sel, pairs, items, n_items, total, y, status);
}

// ---- fold: y[t] = sum over slots (in order) of contrib[pos(t,s)], then the shared expert -----------------
__global__ void fold_pairs_kernel(const float* __restrict__ contrib, const uint32_t* __restrict__ pos_of,
                                  float* __restrict__ y, uint32_t n_used, uint32_t n_embd) {
    const uint32_t t = blockIdx.y;
    const uint32_t o = (blockIdx.x * blockDim.x + threadIdx.x) * 4;
    if (o >= n_embd) return;
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    for (uint32_t s = 0; s <= n_used; ++s) {
        const uint32_t p = pos_of[t * (n_used + 1) + s];
        if (p == 0xFFFFFFFFu) continue;
        const float4 c = *reinterpret_cast<const float4*>(contrib + (size_t)p * n_embd + o);
        v.x += c.x; v.y += c.y; v.z += c.z; v.w += c.w;
    }
    *reinterpret_cast<float4*>(y + (size_t)t * n_embd + o) = v;
}

// The same sum for an expert-parallel shard whose rows are slots (source rank s, token i): the
// row goes straight into rank s's return buffer, at (this rank, i), over the peer mapping; a
// slot none of whose pairs ran here is not written (its owner does not read it).
__global__ void fold_pairs_peer_kernel(const float* __restrict__ contrib, const uint32_t* __restrict__ pos_of,
                                       EpPeerTable peers, uint32_t slot_rows, uint32_t rank, uint32_t n_used,
                                       uint32_t n_embd) {
    const uint32_t t = blockIdx.y;
    const uint32_t o = (blockIdx.x * blockDim.x + threadIdx.x) * 4;
    if (o >= n_embd) return;
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    bool any = false;
    for (uint32_t s = 0; s <= n_used; ++s) {
        const uint32_t p = pos_of[t * (n_used + 1) + s];
        if (p == 0xFFFFFFFFu) continue;
        any = true;
        const float4 c = *reinterpret_cast<const float4*>(contrib + (size_t)p * n_embd + o);
        v.x += c.x; v.y += c.y; v.z += c.z; v.w += c.w;
    }
    if (!any) return;
    const uint32_t src = t / slot_rows, i = t - src * slot_rows;
    *reinterpret_cast<float4*>(peers.back[src] + ((size_t)rank * slot_rows + i) * n_embd + o) = v;
}

// ---- launchers ---------------------------------------------------------------------------------------------
uint32_t prefill_pairs_per_block() { return pf::kNT; }

cudaError_t launch_to_f16_rows(const Launch& L, const float* x, void* xh, float* inv_scale, uint32_t n_rows, uint32_t K) {
    if (n_rows == 0) return cudaSuccess;
    to_f16_rows_kernel<<<n_rows, 256, 0, L.stream>>>(x, (__half*)xh, inv_scale, K);
    L.count();
    return cudaGetLastError();
}

cudaError_t launch_mma_plan(const Launch& L, const qkm_dims& d, const uint32_t* offsets, uint32_t* pairs,
                            uint32_t n_expert_local, uint32_t n_tokens, MmaItem* items_gu, MmaItem* items_dn,
                            MmaItem* items_sh_gu, MmaItem* items_sh_dn, uint32_t* n_items, uint32_t* pos_of,
                            bool with_shared, bool routed_pos_done, uint32_t sh_first, uint32_t sh_count) {
    if (n_expert_local > 512) return cudaErrorInvalidValue;
    if (sh_count == 0xFFFFFFFFu) { sh_first = 0; sh_count = n_tokens; }
    if (sh_first > n_tokens || sh_count > n_tokens - sh_first) return cudaErrorInvalidValue;
    mma_plan_kernel<<<1, 512, 0, L.stream>>>(offsets, pairs, n_expert_local, n_tokens, d.n_used, d.n_ff / 128,
                                             d.n_embd / 128, with_shared ? 1u : 0u, routed_pos_done ? 1u : 0u, sh_first, sh_count, items_gu, items_dn, items_sh_gu, items_sh_dn, n_items, pos_of);
    L.count();
    return cudaGetLastError();
}

template <int FMT, int PT>
static cudaError_t gateup_mma_launch(const Launch& L, const qkm_dims& d, const void* gate_tiles, const void* up_tiles,
                                     const void* xb, const float* x_inv_scale, const uint32_t* pairs, const MmaItem* items,
                                     const uint32_t* n_items, uint32_t max_items, float* h, void* hb, float* hp, uint32_t* status) {
    const size_t smem = (size_t)pf::kStages * 3 * pf::kTileBytes + 1024;
    cudaError_t e = cudaFuncSetAttribute(gateup_mma_kernel<FMT, PT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    gateup_mma_kernel<FMT, PT><<<max_items, PT + 32, smem, L.stream>>>(
        (const uint8_t*)gate_tiles, (const uint8_t*)up_tiles, (const __half*)xb, x_inv_scale, pairs, items, n_items, h,
        (__nv_bfloat16*)hb, hp, d, status);
    L.count();
    return cudaGetLastError();
}

cudaError_t launch_gateup_mma(const Launch& L, const qkm_dims& d, uint32_t type, const void* gate_tiles,
                              const void* up_tiles, const void* xb, const float* x_inv_scale, const uint32_t* pairs,
                              const MmaItem* items, const uint32_t* n_items, uint32_t max_items, float* h, void* hb,
                              uint32_t* status, bool few_blocks, const uint8_t* iq3_table, float* hp) {
    if (max_items == 0) return cudaSuccess;
    if (type == QKM_TYPE_IQ3_XXS) {
        if (!iq3_table) return cudaErrorInvalidValue;
        return gateup_iq3_launch(L, d, gate_tiles, up_tiles, xb, x_inv_scale, pairs, items, n_items, max_items, h, hb, hp, iq3_table, status);
    }
    if (type == QKM_TYPE_IQ4_XS)
        return gateup_mma_launch<QKM_TYPE_IQ4_XS, 512>(L, d, gate_tiles, up_tiles, xb, x_inv_scale, pairs, items, n_items, max_items, h, hb, hp, status);
    if (type == QKM_TYPE_Q8_0)
        return few_blocks ? gateup_mma_launch<QKM_TYPE_Q8_0, 512>(L, d, gate_tiles, up_tiles, xb, x_inv_scale, pairs, items, n_items, max_items, h, hb, hp, status)
                          : gateup_mma_launch<QKM_TYPE_Q8_0, 256>(L, d, gate_tiles, up_tiles, xb, x_inv_scale, pairs, items, n_items, max_items, h, hb, hp, status);
    return cudaErrorInvalidValue;
}

// ---- down, IQ4_XS, table-driven producers, A operand in tensor memory -------------------------------------
// The same GEMM, operands and bits as down_mma_kernel<QKM_TYPE_IQ4_XS>, built like gateup_iq3_kernel:
// 512 producer threads = (row of 128, row tile 2u or 2u+1 of the unit, 32-column half of the k-step);
// a unit is one (expert, pair tile) times two consecutive 128-row tiles of the down matrix, so the
// two accumulators share the h tile (B).  The table maps a quant byte to (kvalues[lo], kvalues[hi])
// as a bf16 pair, once per lane (a row of the 64 KB image is 32 x 4 bytes: a look-up never
// conflicts and its address is one byte permute).  The sub-block scale d * (ls - 32) is applied in
// two bf16 pieces, so a stored weight carries one bf16 rounding of the exact product.
namespace pd {
constexpr uint32_t kTab = pq::kTab, kTabBytes = pq::kTabBytes;
}
size_t down_iq4_table_bytes() { return pd::kTabBytes; }

__global__ void down_iq4_table_kernel(uint8_t* __restrict__ out) {
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;   // one 4-byte word each
    if (i >= pd::kTabBytes / 4) return;
    const uint32_t row = i >> 6, w = i & 63u;
    uint32_t v;
    if (w < 32) {    // bf16 pairs, one per lane
        const __nv_bfloat162 m = __floats2bfloat162_rn((float)c_iq4_values[row & 15u], (float)c_iq4_values[row >> 4]);
        v = *reinterpret_cast<const uint32_t*>(&m);
    } else {         // the same as f16 pairs
        const __half2 m = __floats2half2_rn((float)c_iq4_values[row & 15u], (float)c_iq4_values[row >> 4]);
        v = *reinterpret_cast<const uint32_t*>(&m);
    }
    reinterpret_cast<uint32_t*>(out)[i] = v;
}

cudaError_t launch_down_iq4_table(const Launch& L, uint8_t* out) {
    down_iq4_table_kernel<<<pd::kTabBytes / 4 / 256, 256, 0, L.stream>>>(out);
    L.count();
    return cudaGetLastError();
}

// the bytes one thread needs for (row, k-step q of the 256-column block, 32-column half j)
struct Iq4Step { uint32_t w[4]; };
__device__ __forceinline__ Iq4Step load_iq4_step(const uint8_t* __restrict__ tile, uint32_t r16, uint32_t q, uint32_t j) {
    const uint32_t g = r16 & 7u, hf = r16 >> 3, sb = 2 * q + j;
    Iq4Step r;
#pragma unroll
    for (int t = 0; t < 4; ++t)
        r.w[t] = *reinterpret_cast<const uint32_t*>(tile + 128 + ((2 * hf + (sb >> 2)) * 32 + 4 * g + t) * 16 + 4 * (sb & 3u));
    return r;
}

// F16H: the hidden rows are f16, each scaled by a power of two (h_inv_scale undoes it in the epilogue, with
// the routing weight), and the weights are dequantised to f16 with one multiply by the f16 sub-block scale
// (two roundings of 2^-12); else both operands are bf16 and the scale is applied in two bf16 pieces.
template <bool F16H>
__global__ void __launch_bounds__(pq::kBlock, 1)
down_iq4_kernel(const uint8_t* __restrict__ tiles, const __nv_bfloat16* __restrict__ hb,
                const qkm_sel* __restrict__ sel, const uint32_t* __restrict__ pairs,
                const MmaItem* __restrict__ items, const uint32_t* __restrict__ n_items_ptr,
                float* __restrict__ contrib, qkm_dims d, const uint8_t* __restrict__ table,
                uint32_t* __restrict__ status, const float* __restrict__ h_inv_scale) {
    constexpr int kSt = pq::kStages, PT = pq::kProducers;
    const uint32_t n_units = *n_items_ptr / 2;   // items of one (expert, pair tile) are consecutive row tiles, an even number
    if (blockIdx.x >= n_units) return;
    extern __shared__ __align__(1024) uint8_t smem_dyn[];
    __shared__ __align__(8) unsigned long long s_bar[2 * kSt + 2];  // empty[stage], full[stage], done, table
    __shared__ uint32_t s_tmem;
    __shared__ float s_wgt[2][pf::kNT];
    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31u;
    {   // the fixed addresses must lie inside the dynamic area
        const uint32_t dyn_base = smem_addr(smem_dyn);
        uint32_t dyn_size;
        asm("mov.u32 %0, %%dynamic_smem_size;" : "=r"(dyn_size));
        if (dyn_base > pq::kTab || dyn_base + dyn_size < pq::kEnd) {
            if (tid == 0) atomicExch(status, (uint32_t)kStatusBadLayout);
            return;
        }
    }
    const uint32_t KB = d.n_ff / 256, RT16 = d.n_embd / 16, KS = d.n_ff / 64;
    const uint32_t bar_empty = smem_addr(&s_bar[0]), bar_full = smem_addr(&s_bar[kSt]);
    const uint32_t bar_done = smem_addr(&s_bar[2 * kSt]), bar_tab = smem_addr(&s_bar[2 * kSt + 1]);

    if (tid == 0) {
        for (int s = 0; s < kSt; ++s) {
            mbar_init(bar_empty + 8 * s, 1);      // one commit
            mbar_init(bar_full + 8 * s, PT / 32); // one arrival per producer warp
        }
        mbar_init(bar_done, 1);
        mbar_init(bar_tab, 1);
        mbar_fence_init();
    }
    if (warp == 0) { umma::tmem_alloc(smem_addr(&s_tmem), pq::kTmemCols); umma::tmem_relinquish(); }
    umma::fence_before_sync();
    __syncthreads();
    umma::fence_after_sync();
    if (tid == 0) {
        mbar_expect_tx(bar_tab, pd::kTabBytes);
        for (uint32_t i = 0; i < 4; ++i) bulk_g2s(pd::kTab + i * 16384u, table + i * 16384u, 16384u, bar_tab);
    }
    const uint32_t tmem = s_tmem;
    bool timed_out = false;

    if (tid >= PT) {
        // ---- MMA issuer warp: the whole warp walks the loop, one elected lane issues
        const bool leader = umma::elect_one();
        uint32_t stage = 0, phase = 0;
        for (uint32_t unit = blockIdx.x; unit < n_units; unit += gridDim.x) {
            const uint32_t nn = (items[2 * unit].n + 15u) & ~15u;
            const uint32_t idesc = F16H ? umma::instr_desc_f16(nn) : umma::instr_desc_bf16(nn);
            for (uint32_t ks = 0; ks < KS; ++ks) {
                if (!mbar_wait_bounded(bar_full + 8 * stage, phase)) timed_out = true;
                umma::fence_after_sync();
                const uint64_t d_b = umma::smem_desc(pq::stage_addr(stage));
                const uint32_t t_0 = tmem + pq::kTmemA + stage * 64u, t_1 = t_0 + 32u;
                if (leader) {
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const bool acc = (ks | (uint32_t)j) != 0;
                        mma_f16_ts(tmem, t_0 + 8 * j, d_b + 2 * j, idesc, acc);
                        mma_f16_ts(tmem + 128, t_1 + 8 * j, d_b + 2 * j, idesc, acc);
                    }
                    umma::commit(bar_empty + 8 * stage);
                    if (ks + 1 == KS) umma::commit(bar_done);
                }
                __syncwarp();
                if (++stage == (uint32_t)kSt) { stage = 0; phase ^= 1u; }
            }
        }
    } else {
    // ---- producer warps: thread = (row r, row tile `mat` of the unit, 32-column half j of each k-step)
    const uint32_t r = tid & 127u, mat = (tid >> 7) & 1u, j = tid >> 8;
    const uint32_t tconst = 0x00010000u | ((F16H ? 128u : 0u) + lane * 4u);   // the f16 pairs sit in the upper half of a table row
    const uint32_t a_lane = tmem + ((r & ~31u) << 16) + pq::kTmemA + mat * 32u + j * 16u;
    // N operand: chunks tid and tid + 512 of the h tile (row = chunk / 8), copied asynchronously
    const uint32_t b_row0 = tid >> 3, b_row1 = b_row0 + 64, b_c = tid & 7u;
    const uint32_t b_off0 = umma::sw128_chunk(b_row0, b_c), b_off1 = umma::sw128_chunk(b_row1, b_c);
    if (!mbar_wait_bounded(bar_tab, 0)) timed_out = true;

    struct UnitHead {
        MmaItem it;            // the unit's first item (row tile it.rt, the second is it.rt + 1)
        const uint8_t* wt;     // this thread's 16-row tile of column block 0
        uint32_t r16;
        uint2 hd;              // block header of column block 0
        Iq4Step first;         // quant words of k-step 0
    };
    auto fetch_head = [&](uint32_t unit, uint32_t buf) -> UnitHead {
        UnitHead hd;
        hd.it = items[2 * unit];
        const uint32_t rowidx = (hd.it.rt + mat) * 128u + r;
        hd.r16 = rowidx & 15u;
        hd.wt = tiles + ((size_t)hd.it.expert * KB * RT16 + (rowidx >> 4)) * kTileIq4;
        hd.hd = *reinterpret_cast<const uint2*>(hd.wt + 16 * (hd.r16 & 7u) + 8 * (hd.r16 >> 3));
        hd.first = load_iq4_step(hd.wt, hd.r16, 0, j);
        for (uint32_t i = tid; i < hd.it.n; i += PT) {   // routing weight of the unit's columns (pairs)
            const uint32_t pr = pairs[hd.it.pair_off + i], tok = pr >> 4, slot = pr & 15u;
            s_wgt[buf][i] = (slot < d.n_used ? sel[tok].w[slot] : sel[tok].w_shared) * (F16H ? h_inv_scale[hd.it.pair_off + i] : 1.0f);
        }
        return hd;
    };
    uint32_t stage = 0, phase = 0, gs = 0, iter = 0;
    UnitHead head = fetch_head(blockIdx.x, 0);
    named_sync(1, PT);
    for (uint32_t unit = blockIdx.x; unit < n_units; unit += gridDim.x, ++iter) {
        const MmaItem it = head.it;
        const uint32_t n = it.n, n_mma = (n + 15u) & ~15u;
        const uint32_t r16 = head.r16;
        const uint8_t* wt = head.wt;
        uint2 hdr = head.hd;
        Iq4Step cur = head.first;
        const uint32_t buf = iter & 1u;
        // the h rows of this thread's two chunks: the unit's pairs are consecutive rows of hb
        const __nv_bfloat16* b_src0 = hb + (size_t)(it.pair_off + (b_row0 < n ? b_row0 : 0u)) * d.n_ff + 8 * b_c;
        const __nv_bfloat16* b_src1 = hb + (size_t)(it.pair_off + (b_row1 < n ? b_row1 : 0u)) * d.n_ff + 8 * b_c;
        const uint32_t b_sz0 = b_row0 < n ? 16u : 0u, b_sz1 = b_row1 < n ? 16u : 0u;
        const bool b_do0 = b_row0 < n_mma, b_do1 = b_row1 < n_mma;
        // the first k-step's h tile
        if (gs >= (uint32_t)kSt)
            if (!mbar_wait_bounded(bar_empty + 8 * stage, phase ^ 1u)) timed_out = true;
        {
            const uint32_t st = pq::stage_addr(stage);
            if (b_do0) cp_async16(st + b_off0, b_src0, b_sz0);
            if (b_do1) cp_async16(st + b_off1, b_src1, b_sz1);
            cp_async_commit();
        }
        for (uint32_t ks = 0; ks < KS; ++ks) {
            const uint32_t q = ks & 3u;
            // the next k-step's bytes (and the next column block's header) are fetched one step ahead
            Iq4Step nxt = cur;
            uint2 hdr_n = hdr;
            if (ks + 1 < KS) {
                const uint8_t* ntile = wt + (size_t)((ks + 1) >> 2) * RT16 * kTileIq4;
                nxt = load_iq4_step(ntile, r16, (ks + 1) & 3u, j);
                if (((ks + 1) & 3u) == 0) hdr_n = *reinterpret_cast<const uint2*>(ntile + 16 * (r16 & 7u) + 8 * (r16 >> 3));
            }
            // the next k-step's h tile goes to the next stage, once the MMAs that read it are done
            uint32_t stage1 = stage + 1, phase1 = phase;
            if (stage1 == (uint32_t)kSt) { stage1 = 0; phase1 ^= 1u; }
            if (ks + 1 < KS) {
                if (gs + 1 >= (uint32_t)kSt)
                    if (!mbar_wait_bounded(bar_empty + 8 * stage1, phase1 ^ 1u)) timed_out = true;
                const uint32_t st1 = pq::stage_addr(stage1);
                if (b_do0) cp_async16(st1 + b_off0, b_src0 + (ks + 1) * 64, b_sz0);
                if (b_do1) cp_async16(st1 + b_off1, b_src1 + (ks + 1) * 64, b_sz1);
            }
            cp_async_commit();
            // sub-block 2q + j: scale d * (ls - 32) in two bf16 pieces
            const uint32_t sb = 2 * q + j;
            const float dd = f16_bits_to_f32(hdr.x & 0xFFFFu);
            const int ls = (int)(((hdr.y >> (4 * sb)) & 0xFu) | ((((hdr.x >> 16) >> (2 * sb)) & 3u) << 4)) - 32;
            const float dl = dd * (float)ls;
            const __nv_bfloat16 dhi = __float2bfloat16_rn(dl);
            const __nv_bfloat162 s_hi = __bfloat162bfloat162(dhi);
            const __nv_bfloat162 s_lo = __bfloat162bfloat162(__float2bfloat16_rn(dl - __bfloat162float(dhi)));
            const __half2 s_h = __float2half2_rn(dl);
            auto scale = [&](uint32_t x) -> uint32_t {
                if (F16H) {
                    const __half2 o = __hmul2(*reinterpret_cast<const __half2*>(&x), s_h);
                    return *reinterpret_cast<const uint32_t*>(&o);
                }
                const __nv_bfloat162 v = *reinterpret_cast<const __nv_bfloat162*>(&x);
                const __nv_bfloat162 o = __hfma2(v, s_hi, __hmul2(v, s_lo));
                return *reinterpret_cast<const uint32_t*>(&o);
            };
            // all sixteen look-ups first: byte i of the sub-block -> (element i, element 16 + i)
            uint32_t l[16];
#pragma unroll
            for (int t = 0; t < 4; ++t) {
                l[4 * t + 0] = lds32(prmt_b32(cur.w[t], tconst, 0x7604u));
                l[4 * t + 1] = lds32(prmt_b32(cur.w[t], tconst, 0x7614u));
                l[4 * t + 2] = lds32(prmt_b32(cur.w[t], tconst, 0x7624u));
                l[4 * t + 3] = lds32(prmt_b32(cur.w[t], tconst, 0x7634u));
            }
            uint32_t lo[8], hi[8];   // columns 0..7: elements 0..15 (low nibbles); columns 8..15: elements 16..31
#pragma unroll
            for (int c = 0; c < 8; ++c) {
                lo[c] = scale(__byte_perm(l[2 * c], l[2 * c + 1], 0x5410));
                hi[c] = scale(__byte_perm(l[2 * c], l[2 * c + 1], 0x7632));
            }
            tmem_st8(a_lane + stage * 64u, lo);
            tmem_st8(a_lane + stage * 64u + 8, hi);
            tmem_st_wait();
            cp_async_wait<1>();            // this k-step's h tile has landed (the next one's may be in flight)
            umma::fence_smem_to_async();   // the h tile (generic-proxy writes) before the tensor core reads it
            umma::fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_full + 8 * stage);
            ++gs;
            stage = stage1; phase = phase1;
            cur = nxt; hdr = hdr_n;
        }
        if (unit + gridDim.x < n_units) head = fetch_head(unit + gridDim.x, buf ^ 1u);
        if (!mbar_wait_bounded(bar_done, iter & 1u)) timed_out = true;
        umma::fence_after_sync();

        // epilogue: warp w reads TMEM lanes 32*(w&3).. (rows) of accumulator (w >> 2) & 1 and every other
        // 16-column block; the routing weight is applied after the full K reduction
        {
            const uint32_t lg = warp & 3u, acc = (warp >> 2) & 1u;
            const uint32_t o = (it.rt + acc) * 128u + 32 * lg + lane;
            for (uint32_t cb = warp >> 3; cb < n_mma / 16; cb += 2) {
                uint32_t v[16];
                umma::tmem_ld16(tmem + ((32 * lg) << 16) + acc * 128u + cb * 16, v);
                umma::tmem_ld_wait();
                float* cp = contrib + (size_t)(it.pair_off + cb * 16) * d.n_embd + o;
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    const uint32_t col = cb * 16 + i;
                    if (col < n) cp[(size_t)i * d.n_embd] = s_wgt[buf][col] * __uint_as_float(v[i]);
                }
            }
            umma::fence_before_sync();   // the accumulators are read before this thread's next arrival
        }
        named_sync(1, PT);   // the next unit's columns are written, this unit's are read
    }
    }  // producer / epilogue warps
    umma::fence_before_sync();
    const int any_timed_out = __syncthreads_or(timed_out ? 1 : 0);
    if (warp == 0) umma::tmem_dealloc(tmem, pq::kTmemCols);
    if (any_timed_out && tid == 0) atomicExch(status, (uint32_t)kStatusWaitTimeout);
}

static cudaError_t down_iq4_launch(const Launch& L, const qkm_dims& d, const void* tiles, const void* hb,
                                   const qkm_sel* sel, const uint32_t* pairs, const MmaItem* items,
                                   const uint32_t* n_items, uint32_t max_items, float* contrib, const uint8_t* table,
                                   uint32_t* status, const float* h_inv_scale) {
    static int n_sms = 0;
    if (n_sms == 0) {
        int dev = 0, v = 0;
        if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || v <= 0) v = 148;
        n_sms = v;
    }
    const size_t smem = pq::kEnd;
    cudaError_t e = h_inv_scale ? cudaFuncSetAttribute(down_iq4_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)
                                : cudaFuncSetAttribute(down_iq4_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    const uint32_t units = max_items / 2;
    const uint32_t grid = units < (uint32_t)n_sms ? units : (uint32_t)n_sms;
    if (grid == 0) return cudaSuccess;
    if (h_inv_scale)
        down_iq4_kernel<true><<<grid, pq::kBlock, smem, L.stream>>>((const uint8_t*)tiles, (const __nv_bfloat16*)hb, sel, pairs, items,
                                                                    n_items, contrib, d, table, status, h_inv_scale);
    else
        down_iq4_kernel<false><<<grid, pq::kBlock, smem, L.stream>>>((const uint8_t*)tiles, (const __nv_bfloat16*)hb, sel, pairs, items,
                                                                     n_items, contrib, d, table, status, h_inv_scale);
    L.count();
    return cudaGetLastError();
}

template <int FMT, bool F16H = false>
static cudaError_t down_mma_launch(const Launch& L, const qkm_dims& d, const void* tiles, const void* hb,
                                   const qkm_sel* sel, const uint32_t* pairs, const MmaItem* items,
                                   const uint32_t* n_items, uint32_t max_items, float* contrib, uint32_t* status, bool few_blocks,
                                   const float* h_inv_scale = nullptr) {
    const size_t smem = (size_t)pf::kStages * 2 * pf::kTileBytes + (FMT == QKM_TYPE_IQ4_XS ? 256 * 32 * 4 : 0) + 1024;
    cudaError_t e = cudaFuncSetAttribute(down_mma_kernel<FMT, F16H>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    // routed experts: four row tiles per block (set-up amortised); the shared expert has few blocks, one each
    // (a shard of few experts: one row tile per block as well, so that its blocks fill the machine)
    uint32_t row_tiles = FMT == QKM_TYPE_Q8_0 ? 1u : 4u;
    (void)few_blocks;
    while (row_tiles > 1 && (d.n_embd / 128) % row_tiles) row_tiles >>= 1;
    down_mma_kernel<FMT, F16H><<<(max_items + row_tiles - 1) / row_tiles, pf::kBlock, smem, L.stream>>>(
        (const uint8_t*)tiles, (const __nv_bfloat16*)hb, sel, pairs, items, n_items, contrib, d, row_tiles, status, h_inv_scale);
    L.count();
    return cudaGetLastError();
}

cudaError_t launch_down_mma(const Launch& L, const qkm_dims& d, uint32_t type, const void* tiles, const void* hb,
                            const qkm_sel* sel, const uint32_t* pairs, const MmaItem* items, const uint32_t* n_items,
                            uint32_t max_items, float* contrib, uint32_t* status, bool few_blocks, const uint8_t* iq4_table,
                            const float* h_inv_scale) {
    if (max_items == 0) return cudaSuccess;
    if (type == QKM_TYPE_IQ4_XS && iq4_table && (d.n_embd / 128) % 2 == 0)   // row tiles in pairs
        return down_iq4_launch(L, d, tiles, hb, sel, pairs, items, n_items, max_items, contrib, iq4_table, status, h_inv_scale);
    if (h_inv_scale) {   // f16 hidden rows: only the two kernels above and below take them
        if (type == QKM_TYPE_Q6_K)
            return down_mma_launch<QKM_TYPE_Q6_K, true>(L, d, tiles, hb, sel, pairs, items, n_items, max_items, contrib, status, few_blocks, h_inv_scale);
        if (type != QKM_TYPE_Q8_0) return cudaErrorInvalidValue;
        return down_mma_launch<QKM_TYPE_Q8_0, true>(L, d, tiles, hb, sel, pairs, items, n_items, max_items, contrib, status, few_blocks, h_inv_scale);
    }
    if (type == QKM_TYPE_IQ4_XS)
        return down_mma_launch<QKM_TYPE_IQ4_XS>(L, d, tiles, hb, sel, pairs, items, n_items, max_items, contrib, status, few_blocks);
    if (type == QKM_TYPE_Q8_0)
        return down_mma_launch<QKM_TYPE_Q8_0>(L, d, tiles, hb, sel, pairs, items, n_items, max_items, contrib, status, few_blocks);
    return cudaErrorInvalidValue;
}

cudaError_t launch_fold_pairs(const Launch& L, const qkm_dims& d, const float* contrib, const uint32_t* pos_of,
                              float* y, uint32_t n_tokens) {
    if (n_tokens == 0) return cudaSuccess;
    const dim3 grid((d.n_embd / 4 + 255) / 256, n_tokens);
    fold_pairs_kernel<<<grid, 256, 0, L.stream>>>(contrib, pos_of, y, d.n_used, d.n_embd);
    L.count();
    return cudaGetLastError();
}

cudaError_t launch_fold_pairs_peer(const Launch& L, const qkm_dims& d, const float* contrib, const uint32_t* pos_of,
                                   const EpPeerTable& peers, uint32_t slot_rows, uint32_t rank, uint32_t n_ranks) {
    if (slot_rows == 0 || n_ranks == 0 || n_ranks > kMaxPeerRanks || rank >= n_ranks) return cudaErrorInvalidValue;
    const dim3 grid((d.n_embd / 4 + 255) / 256, n_ranks * slot_rows);
    fold_pairs_peer_kernel<<<grid, 256, 0, L.stream>>>(contrib, pos_of, peers, slot_rows, rank, d.n_used, d.n_embd);
    L.count();
    return cudaGetLastError();
}

}  // namespace qkm
