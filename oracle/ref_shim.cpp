// Thin C wrapper around the REFERENCE's own CPU dequantisers.  It contains no
// arithmetic of its own: it #includes src/quants.h from the reference tree
// (path given with -I by oracle/Makefile) and re-exports the functions so tests
// can compare the restated oracle with them bit-for-bit and generate the golden
// fixtures under tests/golden/.  Built only where the reference tree exists;
// the resulting library goes to oracle/_ref/ and is never committed.
#include <cstdint>

#include "quants.h"  // reference: src/quants.h

#define REF_API extern "C" __attribute__((visibility("default")))

REF_API float ref_f16_to_f32(uint16_t h) { return qk_f16_to_f32(h); }
REF_API uint16_t ref_f32_to_f16(float f) { return qk_f32_to_f16(f); }
REF_API void ref_f16_to_f32_n(const uint16_t* h, float* f, uint64_t n) {
    for (uint64_t i = 0; i < n; ++i) f[i] = qk_f16_to_f32(h[i]);
}
REF_API void ref_f32_to_f16_n(const float* f, uint16_t* h, uint64_t n) {
    for (uint64_t i = 0; i < n; ++i) h[i] = qk_f32_to_f16(f[i]);
}
REF_API int ref_dequant_row(uint32_t type, const void* blocks, float* y, int64_t k) {
    switch (type) {
        case 8: dequant_row_q8_0((const block_q8_0*)blocks, y, k); return 0;
        case 14: dequant_row_q6_K((const block_q6_K*)blocks, y, k); return 0;
        case 23: dequant_row_iq4_xs((const block_iq4_xs*)blocks, y, k); return 0;
        case 18: dequant_row_iq3_xxs((const block_iq3_xxs*)blocks, y, k); return 0;
        default: return -4;
    }
}
REF_API uint32_t ref_grid(uint32_t i) { return iq3xxs_grid[i & 255u]; }
REF_API uint8_t ref_ksigns(uint32_t i) { return ksigns_iq2xs[i & 127u]; }
REF_API int8_t ref_kvalues(uint32_t i) { return kvalues_iq4nl[i & 15u]; }
REF_API uint32_t ref_block_bytes(uint32_t type) {
    switch (type) {
        case 8: return sizeof(block_q8_0);
        case 14: return sizeof(block_q6_K);
        case 23: return sizeof(block_iq4_xs);
        case 18: return sizeof(block_iq3_xxs);
        default: return 0;
    }
}
