// Gate/up + SwiGLU of the fused decode sequence: routed experts (IQ3_XXS) and the shared
// expert (Q8_0) in one persistent launch.
//
// Replaces moe_gateup_iq3.comp / moe_gateup_iq3_rowtile.comp and moe_gateup_q8.comp /
// moe_gateup_q8_64.comp for decode-sized batches; every selected expert is streamed once for
// up to two of the tokens that chose it (the reference's "live expert union" of multi-slot
// decode), and the shared expert rides in the same work list as groups of its own.
//
// Every block first groups the selection's (token, slot) pairs by expert in its own shared
// memory (qkm_dec_rank.cuh), so the work list needs no launch, no serial tail of a single block
// and no trip through global memory.
//
// Work: the flat list of (group, 16-row tile) pairs - a group is an expert with up to two
// tokens, n_ff / 16 tiles each - is cut evenly and contiguously over teams of KB = n_embd / 256
// warps; warp kb of a team streams column block kb of every tile of the team's range through
// a private two-stage ring of bulk copies (TMA, no tensor map, no multicast).
//
// IQ3_XXS inner step (one 32-column sub-block of 16 rows = one int8 MMA of weights):
//   * the lane's two grid indices are already bytes of one register; a byte-permute drops
//     each into bits 8..15 of a table address whose other bytes are lane constants (the grid
//     table has a 256-byte stride per entry and sits at a 64 KB boundary), so a lookup
//     address costs one instruction;
//   * the 7-bit sign code is rotated to bits 9..15 and masked into the address of the sign
//     table, which lives in the unused half of the same 256-byte rows;
//   * magnitudes ^ mask is -m-1 where the element is negative; a second MMA of the masks
//     (-1 / 0) with the negated digit planes adds the missing +1 * x, so no per-element
//     sign arithmetic remains;
//   * the 4-bit sub-block scale stays an integer (2s + 1) and multiplies the exact int32
//     partial sums; d * 0.25 and the digit weights are applied once per tile in f32.
// Q8_0 tiles are cut into quarters (two 32-column blocks) so that a stage of the same ring
// holds them.
//
// IQ4_XS gate/up tensors (moe_gateup_iq4.comp) take the same kernel, instantiated with the inner
// step of the decode down kernel: the 16-entry codebook in four registers, looked up with byte
// permutes, the 6-bit sub-block scales as integers.  No table image: the rings (4352 bytes per
// stage) lie in one run at the start of shared memory.
#include "qkm_dec_rank.cuh"
#include "qkm_kernels.h"
#include "qkm_stream.cuh"
#include "qkm_tiles.cuh"

namespace qkm {

namespace dg {
constexpr int kWarps = 16;
constexpr int kStages = 2;
constexpr int kStageBytes = 2 * kTileIq3;          // gate tile + up tile (3136); a Q8_0 quarter pair needs 2176
constexpr int kRingBytes = kStages * kStageBytes;
constexpr int kStageBytes4 = 2 * kTileIq4;         // the IQ4_XS form: 4352
constexpr int kRingBytes4 = kStages * kStageBytes4;
constexpr uint32_t kTab = 65536, kTabBytes = 65536;   // absolute shared-window address (64 KB aligned) and size
constexpr int kLowRingWarps = 10;                   // rings below the table; the others above it
constexpr int kGroupTiles = 4;                      // tiles between two team-wide reductions
constexpr int kRedFloats = kGroupTiles * 16 * 2 * 2;   // per warp and buffer: tile, row, token, matrix
constexpr uint32_t kHigh = kTab + kTabBytes;
constexpr uint32_t kRed = kHigh + (kWarps - kLowRingWarps) * kRingBytes;
constexpr uint32_t kRank = kRed + kWarps * 2 * kRedFloats * 4;   // RankShared: selection scratch, group list, pairs
constexpr uint32_t kEnd = kRank + ((sizeof(RankShared) + 127) / 128) * 128;
// IQ4_XS form, offsets from the (128-byte aligned) start of the dynamic area: barriers, rings, scratch
constexpr uint32_t kRings4 = 1024;
constexpr uint32_t kRed4 = kRings4 + kWarps * kRingBytes4;
constexpr uint32_t kRank4 = kRed4 + kWarps * 2 * kRedFloats * 4;
constexpr uint32_t kEnd4 = kRank4 + ((sizeof(RankShared) + 127) / 128) * 128 + 128;
constexpr int kQ8Quarter = 2 * 544;                 // two 32-column blocks of a Q8_0 tile: d and quants of 16 rows each
constexpr uint32_t kCostRouted = 8, kCostShared = 11;   // relative time of a routed / a shared tile (measured)
}  // namespace dg

size_t decode_gateup_lut_bytes() { return dg::kTabBytes; }

// The table image: row i (256 B) = grid entry i for 32 lanes (4 B each), then, in the upper 128 B,
// sign masks: row 2c + hl holds code c for lanes 16*hl .. 16*hl+15, 8 B each (byte j = 0xFF when
// element j of the 8-group is negative).
__global__ void decode_gateup_lut_kernel(uint8_t* __restrict__ out) {
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;   // one 4-byte word each
    if (i >= dg::kTabBytes / 4) return;
    const uint32_t row = i >> 6, w = i & 63u;
    uint32_t v;
    if (w < 32) {
        v = c_iq3_grid[row];
    } else {
        const uint32_t sg = signs8(row >> 1), hi = w & 1u;
        v = 0;
#pragma unroll
        for (int j = 0; j < 4; ++j) v |= ((sg >> (j + 4 * hi)) & 1u) ? (0xFFu << (8 * j)) : 0u;
    }
    reinterpret_cast<uint32_t*>(out)[i] = v;
}

cudaError_t launch_decode_gateup_luts(const Launch& L, uint8_t* luts) {
    decode_gateup_lut_kernel<<<dg::kTabBytes / 4 / 256, 256, 0, L.stream>>>(luts);
    L.count();
    return cudaGetLastError();
}

__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
    uint32_t r;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(sel));
    return r;
}

// One IQ3_XXS tile (16 rows x 256 columns) of one matrix against the warp's B operand.
// acc[0..1]: row g, columns 2t and 2t+1; acc[2..3]: row g+8.  Integer, exact.
__device__ __forceinline__ void iq3_tile(uint32_t tb, uint32_t lane, uint32_t g, uint32_t grid_c, uint32_t sign_c,
                                         uint32_t rot, const uint32_t (&b0)[8], const uint32_t (&b1)[8],
                                         const uint32_t (&n0)[8], const uint32_t (&n1)[8], int (&acc)[4]) {
    const uint4 ia = lds128(tb + lane * 16);          // row g: 8 index pairs
    const uint4 ib = lds128(tb + 512 + lane * 16);    // row g+8
    const uint4 xa0 = lds128(tb + 1024 + 16 * g), xa1 = lds128(tb + 1280 + 16 * g);
    const uint4 xb0 = lds128(tb + 1152 + 16 * g), xb1 = lds128(tb + 1408 + 16 * g);
    const uint32_t idx_a[4] = {ia.x, ia.y, ia.z, ia.w}, idx_b[4] = {ib.x, ib.y, ib.z, ib.w};
    const uint32_t aux_a[8] = {xa0.x, xa0.y, xa0.z, xa0.w, xa1.x, xa1.y, xa1.z, xa1.w};
    const uint32_t aux_b[8] = {xb0.x, xb0.y, xb0.z, xb0.w, xb1.x, xb1.y, xb1.z, xb1.w};
    acc[0] = acc[1] = acc[2] = acc[3] = 0;
#pragma unroll
    for (int sb = 0; sb < 8; ++sb) {
        const uint32_t wa = idx_a[2 * (sb & 1) + (sb >> 2)], wb = idx_b[2 * (sb & 1) + (sb >> 2)];   // even sub-blocks in words 0,1; odd in 2,3
        const uint32_t s_lo = (sb & 2) ? 0x7624u : 0x7604u, s_hi = (sb & 2) ? 0x7634u : 0x7614u;
        const uint32_t ga0 = lds32(prmt(wa, grid_c, s_lo)), ga1 = lds32(prmt(wa, grid_c, s_hi));
        const uint32_t gb0 = lds32(prmt(wb, grid_c, s_lo)), gb1 = lds32(prmt(wb, grid_c, s_hi));
        const uint32_t xa = aux_a[4 * (sb & 1) + (sb >> 1)], xb = aux_b[4 * (sb & 1) + (sb >> 1)];
        const uint2 ma = lds64((__funnelshift_l(xa, xa, rot) & 0xFE00u) | sign_c);
        const uint2 mb = lds64((__funnelshift_l(xb, xb, rot) & 0xFE00u) | sign_c);
        int c[4] = {0, 0, 0, 0};
        mma_s8(c, ga0 ^ ma.x, gb0 ^ mb.x, ga1 ^ ma.y, gb1 ^ mb.y, b0[sb], b1[sb]);
        mma_s8(c, ma.x, mb.x, ma.y, mb.y, n0[sb], n1[sb]);
        const int qa = (int)(2u * (xa >> 28) + 1u), qb = (int)(2u * (xb >> 28) + 1u);
        acc[0] += qa * c[0]; acc[1] += qa * c[1];
        acc[2] += qb * c[2]; acc[3] += qb * c[3];
    }
}

// Eight IQ4_XS weights of one quant word (low nibbles: elements 4t..4t+3, high nibbles: 16+4t..16+4t+3) as
// two int8 A-operand registers: lo = elements (4t, 16+4t, 4t+1, 17+4t), hi = (4t+2, 18+4t, 4t+3, 19+4t).
__device__ __forceinline__ void iq4_word_gu(uint32_t w, uint32_t& lo, uint32_t& hi) {
    const uint32_t T0 = 0xBFAD9881u, T1 = 0xF6EADDCFu, T2 = 0x26190D01u, T3 = 0x71594535u;   // kvalues_iq4nl as int8
    const uint32_t s = w & 0x77777777u, s2 = s >> 16, w4 = w << 4;
    const uint32_t m_lo = prmt(w4, w, 0xD9C8u), m_hi = prmt(w4, w, 0xFBEAu);   // 0xFF where a nibble's top bit is set
    const uint32_t a_lo = prmt(T0, T1, s), b_lo = prmt(T2, T3, s);
    const uint32_t a_hi = prmt(T0, T1, s2), b_hi = prmt(T2, T3, s2);
    lo = (a_lo & ~m_lo) | (b_lo & m_lo);
    hi = (a_hi & ~m_hi) | (b_hi & m_hi);
}
// the eight sub-block scales ls - 32 of one row as int8: sub-blocks 0,2,4,6 in ev, 1,3,5,7 in od
__device__ __forceinline__ void iq4_scales_gu(uint32_t sl, uint32_t sh, uint32_t& ev, uint32_t& od) {
    const uint32_t r = prmt(sh, 0u, 0x1100u);
    const uint32_t he = ((r << 4) & 0x00300030u) | (r & 0x30003000u);
    const uint32_t ho = ((r << 2) & 0x00300030u) | ((r >> 2) & 0x30003000u);
    const uint32_t te = ((sl & 0x0F0F0F0Fu) | he) ^ 0x20202020u;
    const uint32_t to = (((sl >> 4) & 0x0F0F0F0Fu) | ho) ^ 0x20202020u;
    ev = (te & 0x20202020u) * 6u + te;
    od = (to & 0x20202020u) * 6u + to;
}
// One IQ4_XS tile against the warp's B operand (elements in iq4_word_gu's order).  acc as in iq3_tile;
// hd: the headers of rows g (x: d | scales_h << 16, y: scales_l) and g+8 (z, w).
__device__ __forceinline__ void iq4_tile_gu(uint32_t tb, uint32_t lane, uint32_t g, const uint32_t (&b0)[8],
                                            const uint32_t (&b1)[8], int (&acc)[4], uint4& hd) {
    hd = lds128(tb + 16 * g);
    uint32_t ea, oa, eb, ob;
    iq4_scales_gu(hd.y, hd.x >> 16, ea, oa);
    iq4_scales_gu(hd.w, hd.z >> 16, eb, ob);
    acc[0] = acc[1] = acc[2] = acc[3] = 0;
#pragma unroll
    for (int hf = 0; hf < 2; ++hf) {
        const uint4 qa4 = lds128(tb + 128 + (hf * 32 + lane) * 16), qb4 = lds128(tb + 128 + ((2 + hf) * 32 + lane) * 16);
        const uint32_t wa[4] = {qa4.x, qa4.y, qa4.z, qa4.w}, wb[4] = {qb4.x, qb4.y, qb4.z, qb4.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int sb = 4 * hf + j;
            uint32_t a0, a1, a2, a3;
            iq4_word_gu(wa[j], a0, a2);
            iq4_word_gu(wb[j], a1, a3);
            int c[4] = {0, 0, 0, 0};
            mma_s8(c, a0, a1, a2, a3, b0[sb], b1[sb]);
            const uint32_t sel = 0x8880u + (uint32_t)(sb >> 1) * 0x1111u;   // byte sb / 2, sign-extended
            const int la = (int)prmt((sb & 1) ? oa : ea, 0u, sel), lb = (int)prmt((sb & 1) ? ob : eb, 0u, sel);
            acc[0] += la * c[0]; acc[1] += la * c[1]; acc[2] += lb * c[2]; acc[3] += lb * c[3];
        }
    }
}

// Two Q8_0 blocks (a quarter tile) of one matrix: q points at two 544-byte pieces [d 32 B][quants 512 B].
__device__ __forceinline__ void q8_quarter(uint32_t q, uint32_t lane, uint32_t g, uint32_t b0a, uint32_t b1a, uint32_t b0b,
                                           uint32_t b1b, float wcol0, float wcol1, float& fa, float& fb) {
#pragma unroll
    for (int bb = 0; bb < 2; ++bb) {
        const uint32_t pb = q + 544 * bb;
        const uint2 qa = lds64(pb + 32 + lane * 8);
        const uint2 qb = lds64(pb + 32 + 256 + lane * 8);
        int c[4] = {0, 0, 0, 0};
        mma_s8(c, qa.x, qb.x, qa.y, qb.y, bb ? b0b : b0a, bb ? b1b : b1a);
        const uint32_t dw = lds32(pb + 2 * (g & ~1u));
        const uint32_t dw8 = lds32(pb + 2 * (8 + (g & ~1u)));
        const float da = f16_bits_to_f32((dw >> (16 * (g & 1u))) & 0xFFFFu);
        const float db = f16_bits_to_f32((dw8 >> (16 * (g & 1u))) & 0xFFFFu);
        fa += da * ((float)c[0] * wcol0 + (float)c[1] * wcol1);
        fb += db * ((float)c[2] * wcol0 + (float)c[3] * wcol1);
    }
}

template <bool IQ4>
__global__ void __launch_bounds__(dg::kWarps * 32, 1)
decode_gateup_kernel(GateupDecodeArgs a) {
    constexpr int kTileR = IQ4 ? kTileIq4 : kTileIq3;                       // routed tile bytes
    constexpr int kStageB = IQ4 ? dg::kStageBytes4 : dg::kStageBytes, kRingB = IQ4 ? dg::kRingBytes4 : dg::kRingBytes;
    extern __shared__ __align__(128) uint8_t smem_raw[];
    const uint32_t base = smem_addr(smem_raw);
    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31u, g = lane >> 2, t = lane & 3u;
    const qkm_dims d = a.d;
    const uint32_t KB = d.n_embd / 256;           // warps per team (2, 4 or 8)
    const uint32_t n_teams = dg::kWarps / KB;
    const uint32_t team = warp / KB, kb = warp - team * KB;
    const uint32_t RT = d.n_ff / 16;              // tiles per group

    const uint32_t base4 = (base + 127u) & ~127u;                        // IQ4_XS form: everything relative to here
    const uint32_t bar_base = IQ4 ? base4 : (base + 15u) & ~15u;         // kWarps * kStages ring barriers, then the table's
    const uint32_t tab_bar = bar_base + dg::kWarps * dg::kStages * 8;
    const uint32_t low_ring = (tab_bar + 8 + 127u) & ~127u;
    if (!IQ4 && low_ring + dg::kLowRingWarps * dg::kRingBytes > dg::kTab) {   // layout assumption broken
        if (tid == 0) atomicExch(a.status, (uint32_t)kStatusBadLayout);
        return;
    }
    const uint32_t ring = IQ4 ? base4 + dg::kRings4 + warp * kRingB
                        : warp < (uint32_t)dg::kLowRingWarps ? low_ring + warp * dg::kRingBytes
                                                             : dg::kHigh + (warp - dg::kLowRingWarps) * dg::kRingBytes;
    float* red = reinterpret_cast<float*>(smem_raw + ((IQ4 ? base4 + dg::kRed4 : dg::kRed) - base));
    const uint32_t my_bar = bar_base + warp * dg::kStages * 8;
    bool timed_out = false;

    if (lane == 0) {
        for (int s = 0; s < dg::kStages; ++s) mbar_init(my_bar + 8 * s, 1);
        if (warp == 0) mbar_init(tab_bar, 1);
        mbar_fence_init();
    }
    __syncthreads();
    if (!IQ4 && tid == 0) {   // the 64 KB table image comes from global memory (L2 after the first block) in four bulk copies
        mbar_expect_tx(tab_bar, dg::kTabBytes);
        for (uint32_t i = 0; i < 4; ++i) bulk_g2s(dg::kTab + i * 16384u, a.luts + i * 16384u, 16384u, tab_bar);
    }

    // Up to here nothing depended on the router kernel, so a block scheduled early (programmatic
    // dependent launch) has its barriers and table copy under way while that kernel's tail runs.  The
    // next kernel is released only now: what it reads before its own wait (the selection) is then final.
    pdl_wait();
    pdl_trigger();

    // Every block groups the selection's pairs by expert itself (same lists everywhere).
    RankShared& S = *reinterpret_cast<RankShared*>(smem_raw + ((IQ4 ? base4 + dg::kRank4 : dg::kRank) - base));
    group_pairs_shared(S, a.sel, d, a.n_tokens, a.expert_first, a.expert_count, a.with_shared != 0, dg::kWarps);

    // This team's contiguous share of the flat tile list.  A shared-expert (Q8_0) tile takes longer
    // than a routed one (four ring stages, each a round trip), so the cut is made in cost units:
    // kCostRouted per routed tile, kCostShared per shared tile (the shared groups come last).
    const uint32_t n_groups = S.n_groups, n_routed = S.n_routed;
    const uint32_t teams_total = gridDim.x * n_teams, team_global = blockIdx.x * n_teams + team;
    const uint32_t tiles_routed = n_routed * RT, tiles_total = n_groups * RT;
    const uint64_t cost_routed = (uint64_t)tiles_routed * dg::kCostRouted;
    const uint64_t cost_total = cost_routed + (uint64_t)(tiles_total - tiles_routed) * dg::kCostShared;
    auto cut = [&](uint32_t i) -> uint32_t {
        const uint64_t c = cost_total * i / teams_total;
        return c <= cost_routed ? (uint32_t)(c / dg::kCostRouted) : tiles_routed + (uint32_t)((c - cost_routed) / dg::kCostShared);
    };
    const uint32_t t_lo = cut(team_global), t_hi = team_global + 1 == teams_total ? tiles_total : cut(team_global + 1);
    const size_t mat_tiles = (size_t)KB * RT;

    // producer cursor over (tile, quarter); lane 0 only.  A routed tile is one stage, a shared
    // tile four (its quarters).
    uint32_t p_tile = t_lo, p_q = 0, p_rt = RT;   // p_rt == RT: the group record must be (re)loaded
    uint32_t p_gi = t_lo / RT;
    const uint8_t* p_g = nullptr;                 // next tile of the gate (routed) / shared gate matrix
    const uint8_t* p_u = nullptr;
    uint32_t p_kind = 0;
    auto issue = [&](uint32_t stage) {
        if (p_tile >= t_hi) return;
        if (p_rt >= RT) {   // first call, or the previous group is finished
            p_rt = p_tile - p_gi * RT;
            const DecodeGroup r = S.groups[p_gi];
            p_kind = r.kind;
            if (p_kind == 0) {
                const size_t tile = (size_t)r.expert * mat_tiles + (size_t)kb * RT + p_rt;
                p_g = a.gate_tiles + tile * kTileR; p_u = a.up_tiles + tile * kTileR;
            } else {
                const size_t tile = (size_t)kb * RT + p_rt;
                p_g = a.sh_gate_tiles + tile * kTileQ8; p_u = a.sh_up_tiles + tile * kTileQ8;
            }
        }
        const uint32_t bar = my_bar + 8 * stage, dst = ring + stage * kStageB;
        if (p_kind == 0) {
            mbar_expect_tx(bar, 2 * kTileR);
            bulk_g2s(dst, p_g, kTileR, bar);
            bulk_g2s(dst + kTileR, p_u, kTileR, bar);
            p_g += kTileR; p_u += kTileR;
            ++p_tile; ++p_rt;
        } else {
            mbar_expect_tx(bar, 2 * dg::kQ8Quarter);   // a quarter = two 32-column blocks = one 1088-byte piece
            bulk_g2s(dst, p_g + dg::kQ8Quarter * p_q, dg::kQ8Quarter, bar);
            bulk_g2s(dst + dg::kQ8Quarter, p_u + dg::kQ8Quarter * p_q, dg::kQ8Quarter, bar);
            if (++p_q == 4) { p_q = 0; p_g += kTileQ8; p_u += kTileQ8; ++p_tile; ++p_rt; }
        }
        if (p_rt >= RT) ++p_gi;
    };
    if (lane == 0)
        for (int s = 0; s < dg::kStages; ++s) issue(s);

    const uint32_t grid_c = dg::kTab + lane * 4;
    const uint32_t sign_c = dg::kTab + (lane >> 4) * 256 + 128 + (lane & 15u) * 8;
    const uint32_t rot = (41u - 7u * t) & 31u;     // rotate-left that brings sign code t to bits 9..15
    const uint32_t team_threads = KB * 32, lt = tid - team * team_threads;
    uint32_t cnt = 0;   // stages consumed by this warp
    uint32_t b0[8], b1[8], n0[8], n1[8];
    float wcol0 = 0.f, wcol1 = 0.f;   // digit weights of the two C columns of this lane (2t, 2t+1)
    DecodeGroup rec{};
    uint32_t e_first = 0, e_n = 0, e_buf = 0;   // tiles waiting for the team-wide reduction: first rt, count, buffer
    uint32_t gi = t_lo / RT, rt = t_lo - gi * RT;
    bool new_group = true;
    // where this thread's reduction outputs of the current group go: (token, slot) of token slot lt & 1
    size_t h_base = 0;
    bool ts_live = false;

    if (!IQ4 && !mbar_wait_bounded(tab_bar, 0)) timed_out = true;   // every thread observes the table's arrival itself

    for (uint32_t tile = t_lo; tile < t_hi; ++tile) {
        if (new_group) {
            new_group = false;
            rec = S.groups[gi];
            {
                const uint32_t ets = lt & 1u;   // the reduction below gives this thread token slot (j & 1) == (lt & 1)
                ts_live = ets < rec.ntok;
                if (ts_live) {
                    const uint32_t pr = S.pairs[rec.pair_off + ets], tok = pr >> 4, slot = pr & 15u;
                    h_base = ((size_t)tok * (d.n_used + 1) + slot) * d.n_ff;
                }
            }
            // B operand: column g of the MMA = (token slot g >> 2, digit g & 3); this warp's 256 columns
            const uint32_t ts = g >> 2, dgt = g & 3u;
            if (ts < rec.ntok) {
                const uint32_t tok = S.pairs[rec.pair_off + ts] >> 4;
                const int8_t* pl = a.planes + (((size_t)tok * KB + kb) * 8 + dgt) * 256;
#pragma unroll
                for (int sb = 0; sb < 8; ++sb) {
                    if (IQ4 && rec.kind == 0) {   // iq4_word_gu's order: (4t, 16+4t, 4t+1, 17+4t | 4t+2, 18+4t, 4t+3, 19+4t)
                        const uint32_t v = *reinterpret_cast<const uint32_t*>(pl + 32 * sb + 4 * t);
                        const uint32_t u = *reinterpret_cast<const uint32_t*>(pl + 32 * sb + 16 + 4 * t);
                        b0[sb] = prmt(v, u, 0x5140u); b1[sb] = prmt(v, u, 0x7362u);
                    } else if (rec.kind == 0) {   // lane t owns elements 8t .. 8t+7 of each sub-block
                        const uint2 v = *reinterpret_cast<const uint2*>(pl + 32 * sb + 8 * t);
                        const uint2 n = *reinterpret_cast<const uint2*>(pl + 1024 + 32 * sb + 8 * t);
                        b0[sb] = v.x; b1[sb] = v.y; n0[sb] = n.x; n1[sb] = n.y;
                    } else {               // elements 4t .. 4t+3 and 16+4t .. 16+4t+3
                        b0[sb] = *reinterpret_cast<const uint32_t*>(pl + 32 * sb + 4 * t);
                        b1[sb] = *reinterpret_cast<const uint32_t*>(pl + 32 * sb + 16 + 4 * t);
                    }
                }
            } else {
#pragma unroll
                for (int sb = 0; sb < 8; ++sb) { b0[sb] = 0; b1[sb] = 0; n0[sb] = 0; n1[sb] = 0; }
            }
            const uint32_t cts = t >> 1;   // token slot of C columns 2t, 2t+1
            wcol0 = 0.f; wcol1 = 0.f;
            if (cts < rec.ntok) {
                const float sc = a.xscale[S.pairs[rec.pair_off + cts] >> 4];
                const float w0 = (t & 1u) ? 16384.f : 1.f;   // 128^(2 * (t & 1))
                wcol0 = sc * w0;
                wcol1 = sc * w0 * 128.f;
            }
        }
        if (e_n == 0) e_first = rt;
        float ga, gb, ua, ub;
        if (rec.kind == 0) {
            const uint32_t stage = cnt % dg::kStages, parity = (cnt / dg::kStages) & 1u;
            if (!mbar_wait_bounded(my_bar + 8 * stage, parity)) timed_out = true;
            const uint32_t sbase = ring + stage * kStageB;
            int ig[4], iu[4];
            if (IQ4) {
                uint4 hg, hu;
                iq4_tile_gu(sbase, lane, g, b0, b1, ig, hg);
                iq4_tile_gu(sbase + kTileIq4, lane, g, b0, b1, iu, hu);
                __syncwarp();
                if (lane == 0) issue(stage);
                ++cnt;
                ga = f16_bits_to_f32(hg.x & 0xFFFFu) * ((float)ig[0] * wcol0 + (float)ig[1] * wcol1);
                gb = f16_bits_to_f32(hg.z & 0xFFFFu) * ((float)ig[2] * wcol0 + (float)ig[3] * wcol1);
                ua = f16_bits_to_f32(hu.x & 0xFFFFu) * ((float)iu[0] * wcol0 + (float)iu[1] * wcol1);
                ub = f16_bits_to_f32(hu.z & 0xFFFFu) * ((float)iu[2] * wcol0 + (float)iu[3] * wcol1);
            } else {
            iq3_tile(sbase, lane, g, grid_c, sign_c, rot, b0, b1, n0, n1, ig);
            iq3_tile(sbase + kTileIq3, lane, g, grid_c, sign_c, rot, b0, b1, n0, n1, iu);
            const uint32_t dwa = lds32(sbase + 1536 + 2 * (g & ~1u)), dwb = lds32(sbase + 1536 + 2 * ((g + 8) & ~1u));
            const uint32_t uwa = lds32(sbase + kTileIq3 + 1536 + 2 * (g & ~1u)), uwb = lds32(sbase + kTileIq3 + 1536 + 2 * ((g + 8) & ~1u));
            __syncwarp();
            if (lane == 0) issue(stage);
            ++cnt;
            const uint32_t sh = 16 * (g & 1u);
            // d * 0.25 * (2s+1) * m  ==  d * (0.5 + s) * 0.5 * m
            ga = (f16_bits_to_f32((dwa >> sh) & 0xFFFFu) * 0.25f) * ((float)ig[0] * wcol0 + (float)ig[1] * wcol1);
            gb = (f16_bits_to_f32((dwb >> sh) & 0xFFFFu) * 0.25f) * ((float)ig[2] * wcol0 + (float)ig[3] * wcol1);
            ua = (f16_bits_to_f32((uwa >> sh) & 0xFFFFu) * 0.25f) * ((float)iu[0] * wcol0 + (float)iu[1] * wcol1);
            ub = (f16_bits_to_f32((uwb >> sh) & 0xFFFFu) * 0.25f) * ((float)iu[2] * wcol0 + (float)iu[3] * wcol1);
            }
        } else {
            ga = gb = ua = ub = 0.f;
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const uint32_t stage = cnt % dg::kStages, parity = (cnt / dg::kStages) & 1u;
                if (!mbar_wait_bounded(my_bar + 8 * stage, parity)) timed_out = true;
                const uint32_t sbase = ring + stage * kStageB;
                q8_quarter(sbase, lane, g, b0[2 * q], b1[2 * q], b0[2 * q + 1], b1[2 * q + 1], wcol0, wcol1, ga, gb);
                q8_quarter(sbase + dg::kQ8Quarter, lane, g, b0[2 * q], b1[2 * q], b0[2 * q + 1], b1[2 * q + 1], wcol0, wcol1, ua, ub);
                __syncwarp();
                if (lane == 0) issue(stage);
                ++cnt;
            }
        }
        // the token's other two digits sit in lane t^1
        ga += __shfl_xor_sync(0xFFFFFFFFu, ga, 1); gb += __shfl_xor_sync(0xFFFFFFFFu, gb, 1);
        ua += __shfl_xor_sync(0xFFFFFFFFu, ua, 1); ub += __shfl_xor_sync(0xFFFFFFFFu, ub, 1);
        float* my_red = red + (warp * 2 + e_buf) * dg::kRedFloats;
        if ((t & 1u) == 0) {
            const uint32_t ts = t >> 1;   // [tile][row 16][token 2][matrix 2]
            *reinterpret_cast<float2*>(my_red + (((e_n * 16 + g) * 2 + ts) * 2)) = make_float2(ga, ua);
            *reinterpret_cast<float2*>(my_red + (((e_n * 16 + g + 8) * 2 + ts) * 2)) = make_float2(gb, ub);
        }
        ++e_n;
        if (e_n == dg::kGroupTiles || (rt & (dg::kGroupTiles - 1)) == dg::kGroupTiles - 1 || tile + 1 == t_hi) {
            // team-wide: sum the KB column-block partials, SwiGLU, store.  The scratch is double
            // buffered, so one barrier per reduction is enough.
            asm volatile("bar.sync %0, %1;" ::"r"(team + 1), "r"(team_threads) : "memory");
            for (uint32_t j = lt; j < e_n * 32; j += team_threads) {   // team_threads is even: j & 1 == lt & 1
                const uint32_t ts = j & 1u, row = j >> 1;   // row within the waiting tiles
                if (ts_live) {
                    float gsum = 0.f, usum = 0.f;
                    for (uint32_t w = 0; w < KB; ++w) {
                        const float2 r = *reinterpret_cast<const float2*>(red + ((team * KB + w) * 2 + e_buf) * dg::kRedFloats + (row * 2 + ts) * 2);
                        gsum += r.x; usum += r.y;
                    }
                    const float hv = swiglu(gsum, usum);
                    const uint32_t r_ff = e_first * 16 + row;
                    a.h[h_base + r_ff] = hv;
                }
            }
            e_n = 0;
            e_buf ^= 1u;
        }
        if (++rt == RT) { rt = 0; ++gi; new_group = true; }
    }
    if (timed_out && lane == 0) atomicExch(a.status, (uint32_t)kStatusWaitTimeout);
}

bool decode_gateup_ok(const qkm_dims& d) {
    const uint32_t KB = d.n_embd / 256;
    return d.n_embd % 256 == 0 && KB >= 2 && KB <= 8 && (KB & (KB - 1)) == 0 && d.n_ff % 64 == 0 && d.n_used <= 15;
}

cudaError_t launch_decode_gateup(const Launch& L, const GateupDecodeArgs& a, uint32_t n_blocks) {
    if (!decode_gateup_ok(a.d)) return cudaErrorInvalidValue;
    if (a.gateup_type == QKM_TYPE_IQ4_XS) {
        const size_t smem4 = dg::kEnd4;
        cudaError_t e4 = cudaFuncSetAttribute(decode_gateup_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem4);
        if (e4 != cudaSuccess) return e4;
        e4 = launch_kernel(L, decode_gateup_kernel<true>, dim3(n_blocks), dim3(dg::kWarps * 32), smem4, a);
        L.count();
        return e4 != cudaSuccess ? e4 : cudaGetLastError();
    }
    if (a.gateup_type != QKM_TYPE_IQ3_XXS) return cudaErrorInvalidValue;
    const size_t smem = dg::kEnd;   // the dynamic area must reach from wherever it starts to the end of the scratch
    cudaError_t e = cudaFuncSetAttribute(decode_gateup_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    e = launch_kernel(L, decode_gateup_kernel<false>, dim3(n_blocks), dim3(dg::kWarps * 32), smem, a);
    L.count();
    return e != cudaSuccess ? e : cudaGetLastError();
}

}  // namespace qkm
