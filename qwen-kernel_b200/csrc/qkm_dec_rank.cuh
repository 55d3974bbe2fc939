// Ranking of f64 router logits (one warp per token) and grouping of the (token, slot) pairs by
// expert (one thread block, in its own shared memory), for a decode-sized batch.
//
// The router kernel ranks a group of tokens in the block that finishes the group's logits last;
// the gate/up kernel groups the pairs in every block at its start (all blocks compute the same,
// deterministic lists), so the work list needs no launch of its own and never makes a round trip
// through global memory.
//
// Rules (the reference's): top n_used by raw logit, lowest id on ties
// (shaders/moe_select_256.comp:60-61), non-finite logits at the floor -3.4e38
// (shaders/moe_select.comp:28-34), softmax over the selected only
// (shaders/moe_select.comp:71-76); pairs grouped as shaders/moe_group_pairs.comp:19-50 does,
// ascending token inside an expert.
#pragma once

#include "qkm_kernels.h"

namespace qkm {

namespace rk {
constexpr uint32_t kMaxTokens = 64, kMaxExperts = 512;
constexpr uint32_t kMaxGroups = (kMaxTokens * 16 + kMaxExperts) / 2 + kMaxTokens / 2;   // 800
constexpr float kFloor = -3.4e38f;
}  // namespace rk

// Shared-memory working set and result of rank_and_group.
struct RankShared {
    unsigned long long mask[rk::kMaxExperts];   // tokens that chose expert e (bit t)
    unsigned long long wsum[32];                // warp totals of the scan
    uint32_t off[rk::kMaxExperts];
    DecodeGroup groups[rk::kMaxGroups];         // routed groups (ascending expert), then the shared expert's
    uint32_t pairs[rk::kMaxTokens * 17];        // (token << 4) | slot, grouped by expert; then the shared "pairs"
    uint16_t ids[rk::kMaxTokens * 16];
    uint32_t n_groups, n_routed;
};

// Ranks tokens [t_first, t_first + t_count): one warp per token, `n_warps` warps of the calling block.
// logits: [T][n_expert] f64 in global memory (complete and visible to this block).  Writes ids,
// weights, route_done and padding of each token's record (w_shared is not touched).
template <bool WIDE>   // WIDE: more than 256 experts (two sorted lists of eight keys per lane instead of one)
__device__ __forceinline__ void rank_tokens_impl(const double* __restrict__ logits, qkm_sel* __restrict__ sel_out, const qkm_dims& d,
                                                 uint32_t t_first, uint32_t t_count, uint32_t n_warps) {
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
    // Ranking with integer keys: an f64 maps to a 64-bit unsigned key whose order is the value's
    // (sign bit flipped for positives, all bits for negatives; -0 is turned into +0 first so the
    // two tie).  One warp per token.  A lane sorts its (up to 16) keys once, as two lists of
    // eight, with a sorting network; then each of the n_used rounds compares only list heads:
    // the warp finds the largest head with three hardware reductions (high word, low word among
    // the lanes that hold it, lowest id among those - lowest id wins ties) and the winning lane
    // pops its list.  Integer arithmetic only: a serial chain of f64 compares and selects is latency-
    // bound (f64 adds and multiplies run at half the f32 rate here, f32<->f64 conversions at an eighth).
    const uint32_t per_lane = (d.n_expert + 31) / 32;   // <= 16
    const unsigned long long kFloorBits = (unsigned long long)__double_as_longlong((double)rk::kFloor);
    for (uint32_t t = t_first + warp; t < t_first + t_count; t += n_warps) {
        const double* lt = logits + (size_t)t * d.n_expert;
        constexpr int NK = WIDE ? 16 : 8;
        uint32_t khi[NK], klo[NK], kid[NK];
#pragma unroll
        for (int j = 0; j < NK; ++j) {
            const uint32_t e = lane + 32u * j;
            khi[j] = 0; klo[j] = 0; kid[j] = e;   // key 0 is below every real key
            if ((uint32_t)j < per_lane && e < d.n_expert) {
                unsigned long long b = (unsigned long long)__ldcg(reinterpret_cast<const long long*>(lt) + e);
                if (((b >> 52) & 0x7FFull) == 0x7FFull) b = kFloorBits;      // NaN, +-Inf -> the floor
                if (b == 0x8000000000000000ull) b = 0ull;                    // -0 ties with +0
                const unsigned long long k = (b >> 63) ? ~b : (b | 0x8000000000000000ull);
                khi[j] = (uint32_t)(k >> 32); klo[j] = (uint32_t)k;
            }
        }
        // compare-exchange: afterwards position p holds the entry that ranks first (key descending, id ascending)
        auto cex = [&](int p, int q) {
            const bool swap = khi[q] > khi[p] || (khi[q] == khi[p] && (klo[q] > klo[p] || (klo[q] == klo[p] && kid[q] < kid[p])));
            const uint32_t h = swap ? khi[q] : khi[p], l = swap ? klo[q] : klo[p], i_ = swap ? kid[q] : kid[p];
            khi[q] = swap ? khi[p] : khi[q]; klo[q] = swap ? klo[p] : klo[q]; kid[q] = swap ? kid[p] : kid[q];
            khi[p] = h; klo[p] = l; kid[p] = i_;
        };
#pragma unroll
        for (int o = 0; o < NK; o += 8) {   // Batcher's 19-exchange network on each list of eight
            cex(o + 0, o + 1); cex(o + 2, o + 3); cex(o + 4, o + 5); cex(o + 6, o + 7);
            cex(o + 0, o + 2); cex(o + 1, o + 3); cex(o + 4, o + 6); cex(o + 5, o + 7);
            cex(o + 1, o + 2); cex(o + 5, o + 6);
            cex(o + 0, o + 4); cex(o + 1, o + 5); cex(o + 2, o + 6); cex(o + 3, o + 7);
            cex(o + 2, o + 4); cex(o + 3, o + 5);
            cex(o + 1, o + 2); cex(o + 3, o + 4); cex(o + 5, o + 6);
        }
        uint32_t my_id = 0, my_hi = 0, my_lo = 0;
        for (uint32_t i = 0; i < d.n_used; ++i) {
            // this lane's best remaining entry: the better of the two list heads
            bool second = false;
            if (WIDE) second = khi[NK - 8] > khi[0] || (khi[NK - 8] == khi[0] && (klo[NK - 8] > klo[0] || (klo[NK - 8] == klo[0] && kid[NK - 8] < kid[0])));
            const uint32_t bh = second ? khi[NK - 8] : khi[0], bl = second ? klo[NK - 8] : klo[0], bi = second ? kid[NK - 8] : kid[0];
            const uint32_t mh = __reduce_max_sync(0xFFFFFFFFu, bh);
            const uint32_t ml = __reduce_max_sync(0xFFFFFFFFu, bh == mh ? bl : 0u);
            const bool cand = bh == mh && bl == ml && (bh | bl) != 0u;
            const uint32_t id = __reduce_min_sync(0xFFFFFFFFu, cand ? bi : 0xFFFFFFFFu);
            const bool won = cand && id == bi;
            const bool pop0 = won && !second, pop8 = won && second;
#pragma unroll
            for (int j = 0; j < 7; ++j) {
                if (pop0) { khi[j] = khi[j + 1]; klo[j] = klo[j + 1]; kid[j] = kid[j + 1]; }
                if (WIDE && pop8) { khi[NK - 8 + j] = khi[NK - 7 + j]; klo[NK - 8 + j] = klo[NK - 7 + j]; kid[NK - 8 + j] = kid[NK - 7 + j]; }
            }
            if (pop0) { khi[7] = 0; klo[7] = 0; }
            if (WIDE && pop8) { khi[NK - 1] = 0; klo[NK - 1] = 0; }
            if (lane == i) { my_id = id; my_hi = mh; my_lo = ml; }
        }
        // Softmax over the selected: the differences to the top logit are formed in f64 (one
        // subtraction), the exponentials and their normalisation in f32 (relative error ~3e-7
        // against the reference's f64 weights).
        const unsigned long long k = ((unsigned long long)my_hi << 32) | my_lo;
        const unsigned long long b = (k >> 63) ? (k & 0x7FFFFFFFFFFFFFFFull) : ~k;
        const double my_val = __longlong_as_double((long long)b);
        const double top = __shfl_sync(0xFFFFFFFFu, my_val, 0);
        const float wv = lane < d.n_used ? expf((float)(my_val - top)) : 0.f;
        float sum = wv;
#pragma unroll
        for (int o = 8; o > 0; o >>= 1) sum += __shfl_xor_sync(0xFFFFFFFFu, sum, o);   // lanes 0..15
        if (lane < 16) {
            const uint32_t id = lane < d.n_used ? min(my_id, d.n_expert - 1) : 0u;
            sel_out[t].ids[lane] = id;
            sel_out[t].w[lane] = lane < d.n_used ? wv / sum : 0.f;
        } else if (lane == 16) {
            sel_out[t].route_done = 0;
        } else if (lane < 23) {
            sel_out[t].pad[lane - 17] = 0.f;
        }
    }
}

__device__ __forceinline__ void rank_tokens(const double* __restrict__ logits, qkm_sel* __restrict__ sel_out, const qkm_dims& d,
                                            uint32_t t_first, uint32_t t_count, uint32_t n_warps) {
    if (d.n_expert > 256) rank_tokens_impl<true>(logits, sel_out, d, t_first, t_count, n_warps);
    else rank_tokens_impl<false>(logits, sel_out, d, t_first, t_count, n_warps);
}

// Groups the (token, slot) pairs of a ranked batch by expert and cuts the gate/up kernel's work
// list, in the calling block's shared memory.  sel: the records rank_tokens wrote (complete and
// visible).  Called by all threads of a block of `n_warps` warps.
__device__ __forceinline__ void group_pairs_shared(RankShared& S, const qkm_sel* __restrict__ sel, const qkm_dims& d, uint32_t T,
                                                   uint32_t expert_first, uint32_t expert_count, bool with_shared, uint32_t n_warps) {
    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31u, n_threads = n_warps * 32;
    for (uint32_t e = tid; e < rk::kMaxExperts; e += n_threads) S.mask[e] = 0ull;
    for (uint32_t i = tid; i < T * 16; i += n_threads) S.ids[i] = (uint16_t)__ldcg(&sel[i >> 4].ids[i & 15u]);
    __syncthreads();
    // token masks per resident expert
    const uint32_t np = T * d.n_used;
    for (uint32_t p = tid; p < np; p += n_threads) {
        const uint32_t t = p / d.n_used, s = p - t * d.n_used;
        const uint32_t e = (uint32_t)S.ids[t * 16 + s] - expert_first;
        if (e < expert_count) atomicOr(&S.mask[e], 1ull << t);
    }
    __syncthreads();
    // exclusive scan over the experts: pair counts in the low word, token groups (of up to two) in the high word
    unsigned long long carry = 0;   // the same in every thread
    for (uint32_t e0 = 0; e0 < rk::kMaxExperts; e0 += n_threads) {   // one pass when the block has 512 threads
        const uint32_t e = e0 + tid;
        const uint32_t c = e < rk::kMaxExperts ? (uint32_t)__popcll(S.mask[e]) : 0u, gn = (c + 1) / 2;
        const unsigned long long mine = (unsigned long long)c | ((unsigned long long)gn << 32);
        unsigned long long v = mine;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const unsigned long long up = __shfl_up_sync(0xFFFFFFFFu, v, o);
            if (lane >= (uint32_t)o) v += up;
        }
        if (lane == 31) S.wsum[warp] = v;
        __syncthreads();
        unsigned long long base = 0, total = 0;
        for (uint32_t w = 0; w < n_warps; ++w) { if (w < warp) base += S.wsum[w]; total += S.wsum[w]; }
        const unsigned long long excl = carry + base + v - mine;
        const uint32_t off = (uint32_t)(excl & 0xFFFFFFFFull), gfirst = (uint32_t)(excl >> 32);
        if (e < rk::kMaxExperts) {
            S.off[e] = off;
            for (uint32_t gi = 0; gi < gn; ++gi) {
                DecodeGroup g;
                g.expert = (uint16_t)e;
                g.ntok = (uint8_t)min(2u, c - 2 * gi);
                g.kind = 0;
                g.pair_off = off + 2 * gi;
                S.groups[gfirst + gi] = g;
            }
        }
        carry += total;
        __syncthreads();   // wsum is rewritten by the next pass
    }
    const uint32_t n_routed = (uint32_t)(carry >> 32);
    // the shared expert: every token is a "pair" (token, slot n_used) stored after the routed pairs
    const uint32_t n_shared = with_shared ? (T + 1) / 2 : 0u;
    if (with_shared)
        for (uint32_t t = tid; t < T; t += n_threads) S.pairs[np + t] = (t << 4) | d.n_used;
    for (uint32_t gi = tid; gi < n_shared; gi += n_threads) {
        DecodeGroup g;
        g.expert = 0;
        g.ntok = (uint8_t)min(2u, T - 2 * gi);
        g.kind = 1;
        g.pair_off = np + 2 * gi;
        S.groups[n_routed + gi] = g;
    }
    if (tid == 0) { S.n_groups = n_routed + n_shared; S.n_routed = n_routed; }
    // place: a pair's rank inside its expert is the number of lower tokens that chose the expert
    for (uint32_t p = tid; p < np; p += n_threads) {
        const uint32_t t = p / d.n_used, s = p - t * d.n_used;
        const uint32_t e = (uint32_t)S.ids[t * 16 + s] - expert_first;
        if (e >= expert_count) continue;
        const uint32_t rank = (uint32_t)__popcll(S.mask[e] & ((1ull << t) - 1ull));
        S.pairs[S.off[e] + rank] = (t << 4) | s;
    }
    __syncthreads();
}

}  // namespace qkm
