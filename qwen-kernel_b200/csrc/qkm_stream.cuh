// Building blocks of the streaming kernels: bulk-copy (TMA) rings private to a warp,
// bounded mbarrier waits, tensor-core MMA wrappers, codebook tables in shared memory.
#pragma once

#include <cuda_bf16.h>
#include <stdint.h>

#include "qkm_common.cuh"

namespace qkm {

// status word values a kernel may leave in its error flag
enum : uint32_t { kStatusOk = 0, kStatusWaitTimeout = 1, kStatusBadLayout = 2 };

__device__ __forceinline__ uint32_t smem_addr(const void* p) {
    return (uint32_t)__cvta_generic_to_shared(p);
}

// ---- mbarrier + 1-D bulk copy global -> shared (no multicast anywhere) ----------------
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_fence_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
// dst/src 16-byte aligned, bytes a multiple of 16
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        "selp.u32 %0, 1, 0, p;\n"
        "}\n"
        : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
// Bounded wait: gives up after ~2^22 polls (each poll itself blocks for a
// hardware-defined interval), far beyond any legitimate copy latency.
__device__ __forceinline__ bool mbar_wait_bounded(uint32_t bar, uint32_t parity) {
    for (uint32_t i = 0; i < (1u << 22); ++i)
        if (mbar_try_wait(bar, parity)) return true;
    return false;
}

// ---- tensor-core MMAs (warp-level; operands in registers) -----------------------------
// D(16x8, s32) += A(16x32, s8, row) * B(32x8, s8, col)
__device__ __forceinline__ void mma_s8(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                       uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// unsigned A (magnitudes 0..255) with signed B
__device__ __forceinline__ void mma_u8s8(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// D(16x8, f32) += A(16x16, bf16, row) * B(16x8, bf16, col)
__device__ __forceinline__ void mma_bf16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t lds32(uint32_t addr) {
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint2 lds64(uint32_t addr) {
    uint2 v;
    asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint4 lds128(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}

// ---- activation encodings -----------------------------------------------------------------
// Exponent p with |x| * 2^p <= 2^26 for |x| <= m (m > 0 finite); 0 for m == 0.
__device__ __forceinline__ int digit_exponent(float m) {
    if (!(m > 0.f)) return 0;
    int e;
    frexpf(m, &e);  // m = f * 2^e, f in [0.5, 1)
    return 26 - e;
}
// four balanced base-128 digits of v (|v| <= 2^26), packed d0 | d1<<8 | d2<<16 | d3<<24
__device__ __forceinline__ uint32_t digits4(int v) {
    const int d0 = ((v + 64) & 127) - 64; v = (v - d0) >> 7;
    const int d1 = ((v + 64) & 127) - 64; v = (v - d1) >> 7;
    const int d2 = ((v + 64) & 127) - 64; v = (v - d2) >> 7;
    return (uint32_t)(d0 & 255) | ((uint32_t)(d1 & 255) << 8) | ((uint32_t)(d2 & 255) << 16) | ((uint32_t)(v & 255) << 24);
}
// Encodes one row x[K] into digit planes, called by all 256 threads of a block.
// Plane layout per row: [kb = k/256][digit 0..3][256], so the four planes of one
// 256-column block are 1 KB of consecutive memory.  scale receives 2^-p; a row that
// holds NaN/Inf gets all-zero planes and a NaN scale (its outputs become NaN).
__device__ __forceinline__ void block_encode_digits(const float* __restrict__ xt, int8_t* __restrict__ pl,
                                                    float* __restrict__ scale, uint32_t K, float* s_max /*[8]*/) {
    const uint32_t tid = threadIdx.x;
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
    for (uint32_t k = tid; k < K; k += 256) {
        const uint32_t dgt = any_bad ? 0u : digits4(__float2int_rn(xt[k] * up));
        int8_t* q = pl + (size_t)(k >> 8) * 1024 + (k & 255u);
        q[0] = (int8_t)(dgt & 255u);
        q[256] = (int8_t)((dgt >> 8) & 255u);
        q[512] = (int8_t)((dgt >> 16) & 255u);
        q[768] = (int8_t)(dgt >> 24);
    }
    if (tid == 0) *scale = any_bad ? __int_as_float(0x7FC00000) : ldexpf(1.0f, -p);
    __syncthreads();
}

// three bf16 pieces whose sum is x exactly (24 significant bits)
__device__ __forceinline__ void bf16_pieces(float x, __nv_bfloat16& p0, __nv_bfloat16& p1, __nv_bfloat16& p2) {
    p0 = __float2bfloat16_rn(x);
    const float r1 = x - __bfloat162float(p0);
    p1 = __float2bfloat16_rn(r1);
    const float r2 = r1 - __bfloat162float(p1);
    p2 = __float2bfloat16_rn(r2);
}

}  // namespace qkm
