// 5th-generation tensor core (tcgen05) building blocks for the batched-prefill GEMMs:
// tensor-memory allocation, shared-memory matrix descriptors for K-major bf16 tiles in
// the 128-byte swizzle layout, the MMA issue, commit-to-mbarrier, accumulator loads.
//
// Operand layout used throughout (both A and B are K-major, bf16, K extent 64 per tile):
//   a tile of R rows x 64 columns occupies R * 128 bytes; rows are grouped by 8 into
//   1024-byte atoms; inside an atom row r holds its eight 16-byte chunks at
//   chunk position (c ^ r): byte offset of element (row, k) =
//       (row / 8) * 1024 + (row % 8) * 128 + (((k / 8) ^ (row % 8)) * 16) + (k % 8) * 2.
//   The tile base must be 1024-byte aligned.  One MMA consumes 16 columns: the descriptor
//   start address advances by 32 bytes per 16-column step inside the 64-column tile.
#pragma once

#include <stdint.h>

namespace qkm {
namespace umma {

// byte offset of the 16-byte chunk holding columns [8*c, 8*c+8) of `row`
__device__ __forceinline__ uint32_t sw128_chunk(uint32_t row, uint32_t c) {
    return (row >> 3) * 1024u + (row & 7u) * 128u + ((c ^ (row & 7u)) << 4);
}

// shared-memory matrix descriptor: K-major, SWIZZLE_128B, 8-row groups 1024 bytes apart
__device__ __forceinline__ uint64_t smem_desc(uint32_t smem_byte_addr) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_byte_addr >> 4) & 0x3FFFu);   // start address, bits [0,14)
    d |= (uint64_t)1 << 16;                              // leading byte offset (unused for swizzled K-major)
    d |= (uint64_t)(1024u >> 4) << 32;                   // stride byte offset, bits [32,46)
    d |= (uint64_t)1 << 46;                              // descriptor version (Blackwell)
    d |= (uint64_t)2 << 61;                              // layout type: SWIZZLE_128B
    return d;
}

// true in exactly one lane of the (converged) warp
__device__ __forceinline__ bool elect_one() {
    uint32_t p;
    asm volatile(
        "{\n"
        ".reg .pred P1;\n"
        "elect.sync _|P1, 0xFFFFFFFF;\n"
        "selp.u32 %0, 1, 0, P1;\n"
        "}\n"
        : "=r"(p));
    return p != 0;
}

// instruction descriptor: bf16 x bf16 -> f32, both operands K-major, M = 128, N = n (multiple of 16)
__device__ __forceinline__ uint32_t instr_desc_bf16(uint32_t n) {
    uint32_t d = 0;
    d |= 1u << 4;            // D format: f32
    d |= 1u << 7;            // A format: bf16
    d |= 1u << 10;           // B format: bf16
    d |= (n >> 3) << 17;     // N / 8
    d |= (128u >> 4) << 24;  // M / 16
    return d;
}

// same with f16 inputs
__device__ __forceinline__ uint32_t instr_desc_f16(uint32_t n) {
    uint32_t d = 0;
    d |= 1u << 4;            // D format: f32; A and B formats 0 = f16
    d |= (n >> 3) << 17;
    d |= (128u >> 4) << 24;
    return d;
}

__device__ __forceinline__ void tmem_alloc(uint32_t smem_dst, uint32_t ncols) {  // whole warp
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_dst), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {  // whole warp
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}

// D[tmem] (+)= A[smem] * B[smem] (kind::f16: f16 or bf16 inputs per the instruction descriptor); issued by ONE thread
__device__ __forceinline__ void mma_f16_ss(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                            bool accumulate) {
    const uint32_t acc = accumulate ? 1u : 0u;
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n"
        "}\n" ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(acc)
        : "memory");
}
// all MMAs issued so far by this thread arrive on the mbarrier when they complete
__device__ __forceinline__ void commit(uint32_t mbar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(mbar) : "memory");
}
__device__ __forceinline__ void fence_before_sync() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void fence_after_sync() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
// make generic-proxy shared-memory writes visible to the async proxy (the tensor core reads)
__device__ __forceinline__ void fence_smem_to_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// 32 lanes x 16 consecutive 32-bit columns: thread i of the warp gets lane (base lane + i)
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&v)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
          "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
        : "r"(taddr));
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

}  // namespace umma
}  // namespace qkm
