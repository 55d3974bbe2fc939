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
// row), copied asynchronously (cp.async, 16 bytes per lane and instruction) into its own ring of
// stages.  A slice row is 68 words long, so the A-fragment loads of the eight row groups fall into
// different banks without padding, and no warp waits for another until the partial sums of eight
// tiles meet in shared memory.  (Bulk copies of whole rows into a padded block-wide stage moved
// 3.8 TB/s at most: sixteen 2 KB copies per tile.)  A warp multiplies its 256 columns of the 16
// rows (eight MMAs), scales each 32-column block's integer sums by the block's f16 scale and keeps
// f32 partial sums.
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

// Q8_0: 16 rows x 32 columns of block `bi` of the tile at `st` (row stride S) against one k32 B operand.
// Returns in f0 / f1 the contribution to rows g / g+8 of this lane's two digit planes.
template <bool EVEN>
__device__ __forceinline__ void q8_block_mma(uint32_t st, uint32_t S, uint32_t bi, uint32_t g, uint32_t t, uint32_t b0,
                                             uint32_t b1, float plane_w, float& f0, float& f1) {
    const uint32_t r0 = st + g * S + 34u * bi, r1 = r0 + 8u * S;
    uint32_t a0, a1, a2, a3;
    if (EVEN) {   // the quants start two bytes into a word: two aligned words and a funnel shift each
        a0 = __funnelshift_r(lds32(r0 + 4 * t), lds32(r0 + 4 * t + 4), 16);
        a1 = __funnelshift_r(lds32(r1 + 4 * t), lds32(r1 + 4 * t + 4), 16);
        a2 = __funnelshift_r(lds32(r0 + 16 + 4 * t), lds32(r0 + 20 + 4 * t), 16);
        a3 = __funnelshift_r(lds32(r1 + 16 + 4 * t), lds32(r1 + 20 + 4 * t), 16);
    } else {
        a0 = lds32(r0 + 2 + 4 * t); a1 = lds32(r1 + 2 + 4 * t);
        a2 = lds32(r0 + 18 + 4 * t); a3 = lds32(r1 + 18 + 4 * t);
    }
    int c[4] = {0, 0, 0, 0};
    mma_s8(c, a0, a1, a2, a3, b0, b1);
    // the block scales (f16 at the head of each block); an even block's sits in the low half of its word
    const uint32_t w0 = lds32(EVEN ? r0 : r0 - 2), w1 = lds32(EVEN ? r1 : r1 - 2);
    const float d0 = f16_bits_to_f32(EVEN ? (w0 & 0xFFFFu) : (w0 >> 16));
    const float d1 = f16_bits_to_f32(EVEN ? (w1 & 0xFFFFu) : (w1 >> 16));
    // digits 2t (weight 1) and 2t+1 (weight 128) of this lane's pair, exact in int32
    f0 = fmaf((float)(c[0] + (c[1] << 7)) * plane_w, d0, f0);
    f1 = fmaf((float)(c[2] + (c[3] << 7)) * plane_w, d1, f1);
}

template <int N>
__device__ __forceinline__ void cp_async_wait_n() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ void cp_async_wait_dyn(uint32_t n) {   // at most n groups still in flight
    switch (n) {
        case 0: cp_async_wait_n<0>(); break;
        case 1: cp_async_wait_n<1>(); break;
        case 2: cp_async_wait_n<2>(); break;
        case 3: cp_async_wait_n<3>(); break;
        case 4: cp_async_wait_n<4>(); break;
        default: cp_async_wait_n<5>(); break;
    }
}

template <int TYPE>
__global__ void __launch_bounds__(gm::kMaxWarps * 32)
gemv_mma_kernel(const uint8_t* __restrict__ W, const float* __restrict__ x, float* __restrict__ y, uint32_t n_tiles,
                uint32_t K, uint32_t rb, uint32_t n_stages) {
    static_assert(TYPE == QKM_TYPE_Q8_0, "formats: Q8_0");
    extern __shared__ __align__(128) uint8_t smem_raw[];
    __shared__ float s_max[gm::kMaxWarps];
    __shared__ float s_scale;
    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31u, g = lane >> 2, t = lane & 3u;
    const uint32_t KB = K / 256, n_threads = KB * 32;
    constexpr uint32_t S = gm::kSlice, kStage = gm::kRows * gm::kSlice;   // 272-byte slice rows, 4352 bytes per stage
    // layout: digit planes [KB][4][256] | partial sums [2][KB][kGroup * 16] | rings [KB][n_stages][4352]
    int8_t* planes = reinterpret_cast<int8_t*>(smem_raw);
    float* red = reinterpret_cast<float*>(smem_raw + (size_t)K * 4);
    const uint32_t red_floats = KB * gm::kGroup * gm::kRows;
    const uint32_t ring = ((smem_addr(smem_raw) + K * 4 + 2 * red_floats * 4 + 127u) & ~127u) + warp * n_stages * kStage;

    // this block's tiles: blockIdx.x, + gridDim.x, ...; a lane's chunks of a tile: c = lane + 32 k < 272,
    // row c / 17, 16-byte piece c % 17 of the slice row - the same for every tile
    const uint32_t my_tiles = blockIdx.x < n_tiles ? (n_tiles - blockIdx.x + gridDim.x - 1) / gridDim.x : 0u;
    uint32_t c_src[9], c_dst[9];
#pragma unroll
    for (int k = 0; k < 9; ++k) {
        const uint32_t c = lane + 32u * k, row = c / 17u, j = c - row * 17u;
        c_src[k] = row * rb + warp * S + 16u * j;
        c_dst[k] = row * S + 16u * j;
    }
    auto issue = [&](uint32_t i) {   // tile number i of this block into stage i % n_stages of this warp's ring
        const uint32_t dst = ring + (i % n_stages) * kStage;
        const uint8_t* src = W + (size_t)(blockIdx.x + i * gridDim.x) * gm::kRows * rb;
#pragma unroll
        for (int k = 0; k < 9; ++k)
            if (k < 8 || lane < 16u) asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst + c_dst[k]), "l"(src + c_src[k]) : "memory");
    };
    for (uint32_t i = 0; i + 1 < n_stages; ++i) {
        if (i < my_tiles) issue(i);
        asm volatile("cp.async.commit_group;" ::: "memory");
    }

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
        for (int q = 0; q < gm::kGroup; ++q) {
            acc[q][0] = acc[q][1] = 0.f;
            const uint32_t i = i0 + q;
            if (i < my_tiles) {   // block-uniform
                // refill the stage this warp read one tile ago (its loads have returned), then wait for tile i
                __syncwarp();
                if (i + n_stages - 1 < my_tiles) issue(i + n_stages - 1);
                asm volatile("cp.async.commit_group;" ::: "memory");
                cp_async_wait_dyn(n_stages - 1);   // every lane's pieces of tile i
                __syncwarp();
                const uint32_t st = ring + (i % n_stages) * kStage;
                float f0 = 0.f, f1 = 0.f;
#pragma unroll
                for (int sb = 0; sb < 8; ++sb) {
                    if (sb & 1) q8_block_mma<false>(st, S, sb, g, t, b0[sb], b1[sb], plane_w, f0, f1);
                    else q8_block_mma<true>(st, S, sb, g, t, b0[sb], b1[sb], plane_w, f0, f1);
                }
                acc[q][0] = f0; acc[q][1] = f1;
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
}

// Rows [0, *rows_done) are computed here; the caller finishes the rest.  Shapes this form does not take
// leave *rows_done at 0.
cudaError_t launch_gemv_mma(const Launch& L, uint32_t type, const void* W, const float* x, float* y, uint32_t M,
                            uint32_t K, uint32_t n_sms, uint32_t* status, uint32_t* rows_done) {
    *rows_done = 0;
    if (type != QKM_TYPE_Q8_0 || K % 256 != 0 || K < 512 || K > 256u * gm::kMaxWarps || M < (uint32_t)gm::kRows) return cudaSuccess;
    (void)status;   // no device-side wait in this form
    if (((uintptr_t)W & 15u) || ((uintptr_t)x & 3u)) return cudaSuccess;
    const uint32_t rb = (uint32_t)row_bytes(type, K);   // a multiple of 16 for K % 256 == 0
    if (rb % 16) return cudaSuccess;
    const uint32_t KB = K / 256;
    const size_t fixed = (size_t)K * 4 + 2 * (size_t)KB * gm::kGroup * gm::kRows * 4 + 128;
    const size_t stage = (size_t)KB * gm::kRows * gm::kSlice;   // one stage of every warp's ring
    // one block per SM with as deep a ring as fits: the bytes in flight, not the warps, carry the bandwidth
    uint32_t n_stages = gm::kMaxStages;
    while (n_stages > 2 && fixed + n_stages * stage > 200u * 1024u) --n_stages;
    const size_t smem = fixed + n_stages * stage;
    if (smem > 220u * 1024u) return cudaSuccess;
    cudaError_t e = cudaFuncSetAttribute(gemv_mma_kernel<QKM_TYPE_Q8_0>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    const uint32_t n_tiles = M / gm::kRows;
    const uint32_t blocks = n_tiles < n_sms ? n_tiles : n_sms;
    gemv_mma_kernel<QKM_TYPE_Q8_0><<<blocks, KB * 32, smem, L.stream>>>((const uint8_t*)W, x, y, n_tiles, K, rb, n_stages);
    L.count();
    *rows_done = n_tiles * gm::kRows;
    return cudaGetLastError();
}

}  // namespace qkm
