// Host-side launchers of the sm_100a kernels.  Every launcher enqueues on the
// given stream and returns the CUDA error of the launch (cudaSuccess on success);
// none of them synchronises.  `launches` (may be NULL) is incremented once per
// kernel launched.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/qk_moe.h"

namespace qkm {

struct Launch {
    cudaStream_t stream;
    uint64_t* launches;
    // programmatic dependent launch: the kernel may be scheduled while the previous kernel of the
    // stream is still running; it runs its set-up, then waits (pdl_wait) for that kernel's results
    bool pdl = false;
    void count(int n = 1) const { if (launches) *launches += (uint64_t)n; }
};

// Launch with or without the programmatic-serialization attribute.
template <typename... KArgs, typename... Args>
inline cudaError_t launch_kernel(const Launch& L, void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = L.stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr; cfg.numAttrs = L.pdl ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

#ifdef __CUDACC__
// Both are no-ops in a kernel launched without the attribute.  pdl_wait: every kernel this one
// depends on has finished and its stores are visible.  pdl_trigger: the next kernel of the
// stream may be scheduled now (it still waits for this one's end in its own pdl_wait).
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
#endif

// One unit of work of a streaming kernel: an expert, a chunk of its rows and up to
// tok_per_item of the tokens routed to it (pairs[pair_off .. pair_off + ntok)).
struct StreamItem {
    uint16_t expert;   // resident-expert index
    uint8_t chunk;     // row chunk within the expert's matrix
    uint8_t ntok;
    uint32_t pair_off;
};

// One block of the prefill GEMMs: an expert, a 128-row tile of its matrix and up to 128
// of its pairs (pairs[pair_off .. pair_off + n)).
struct MmaItem {
    uint16_t expert;
    uint16_t rt;
    uint32_t pair_off;
    uint32_t n;
};

// ---- fused decode sequence (qkm_dec_route.cu, qkm_dec_gateup.cu, qkm_dec_down.cu) ---------------
// One expert (or the shared expert) with up to two of the tokens routed to it:
// pairs[pair_off .. pair_off + ntok).  The gate/up kernel walks all n_ff rows of a group.
struct DecodeGroup {
    uint16_t expert;   // resident-expert index (kind 0)
    uint8_t ntok;      // 1 or 2
    uint8_t kind;      // 0 routed expert, 1 shared expert
    uint32_t pair_off;
};
struct RouteDecodeArgs {
    const uint8_t* router;     // [n_expert][n_embd] F32 or F16
    const float* gis;          // [n_embd]
    const float* x;            // [n_tokens][n_embd]
    qkm_sel* sel;              // out [n_tokens]
    double* logits;            // scratch [n_tokens][n_expert]
    uint32_t* counter;         // ceil(n_tokens / 8) zero words; left at zero
    int8_t* planes;            // out [n_tokens][n_embd/256][8][256]: digit planes 0..3 and their negatives 4..7
    float* xscale;             // out [n_tokens] 2^-p
    uint32_t n_tokens;
    qkm_dims d;
};
bool route_decode_ok(const qkm_dims& d, uint32_t n_tokens, size_t scratch_bytes);
cudaError_t launch_route_decode(const Launch& L, uint32_t router_type, const RouteDecodeArgs& a);
// routed (IQ3_XXS) and shared (Q8_0) gate/up + SwiGLU over the groups
struct GateupDecodeArgs {
    const uint8_t* gate_tiles;      // routed experts, IQ3_XXS or IQ4_XS tiles (gateup_type)
    const uint8_t* up_tiles;
    const uint8_t* sh_gate_tiles;   // shared expert, Q8_0 tiles (may be NULL when no group has kind 1)
    const uint8_t* sh_up_tiles;
    const uint8_t* luts;            // decode_gateup_lut_bytes() bytes written by launch_decode_gateup_luts
    const int8_t* planes;
    const float* xscale;
    const qkm_sel* sel;             // the selection (its pairs are grouped by expert in every block at its start)
    uint32_t n_tokens, expert_first, expert_count, with_shared;
    uint32_t gateup_type;           // QKM_TYPE_IQ3_XXS or QKM_TYPE_IQ4_XS
    float* h;                       // out [T][n_used+1][n_ff]
    uint32_t* status;
    qkm_dims d;
};
size_t decode_gateup_lut_bytes();
cudaError_t launch_decode_gateup_luts(const Launch& L, uint8_t* luts);
bool decode_gateup_ok(const qkm_dims& d);
cudaError_t launch_decode_gateup(const Launch& L, const GateupDecodeArgs& a, uint32_t n_blocks);
// routed (IQ4_XS) down + shared (Q8_0) down + weighted sum: y[t] = sum_s w_s D[ids_s] h[t][s] + w_shared DS h[t][n_used]
struct DownDecodeArgs {
    const uint8_t* tiles;           // routed experts, IQ4_XS tiles
    const uint8_t* sh_tiles;        // shared expert, Q8_0 tiles (NULL: no shared term)
    const uint8_t* lut;             // IQ4_XS form: decode_down_lut_bytes() bytes written by launch_decode_down_lut
    const float* h;                 // [T][n_used+1][n_ff] f32 (encoded as int8 digit planes inside the kernel)
    const qkm_sel* sel;
    float* y;
    uint32_t n_tokens;
    uint32_t* status;
    qkm_dims d;
};
bool decode_down_ok(const qkm_dims& d);
size_t decode_down_lut_bytes();
cudaError_t launch_decode_down_lut(const Launch& L, uint8_t* lut);
cudaError_t launch_decode_down(const Launch& L, const DownDecodeArgs& a, uint32_t n_blocks);
// the same with the routed experts as Q6_K tiles
cudaError_t launch_decode_down_q6k(const Launch& L, const DownDecodeArgs& a, uint32_t n_blocks);

// ---- qkm_prefill.cu : tcgen05 expert GEMMs for batched prefill
uint32_t prefill_pairs_per_block();
// x rows as f16 scaled per row by a power of two (inv_scale[row] undoes it)
cudaError_t launch_to_f16_rows(const Launch& L, const float* x, void* xh, float* inv_scale, uint32_t n_rows, uint32_t K);
cudaError_t launch_mma_plan(const Launch& L, const qkm_dims& d, const uint32_t* offsets, uint32_t* pairs,
                            uint32_t n_expert_local, uint32_t n_tokens, MmaItem* items_gu, MmaItem* items_dn,
                            MmaItem* items_sh_gu, MmaItem* items_sh_dn, uint32_t* n_items, uint32_t* pos_of,
                            bool with_shared = true, bool routed_pos_done = false, uint32_t sh_first = 0,
                            uint32_t sh_count = 0xFFFFFFFFu /* all rows */);
cudaError_t launch_gateup_mma(const Launch& L, const qkm_dims& d, uint32_t type, const void* gate_tiles,
                              const void* up_tiles, const void* xb, const float* x_inv_scale, const uint32_t* pairs,
                              const MmaItem* items, const uint32_t* n_items, uint32_t max_items, float* h, void* hb,
                              uint32_t* status, bool few_blocks = false,   // few_blocks: the grid will not fill the machine
                              const uint8_t* iq3_table = nullptr,          // IQ3_XXS: the table image (launch_gateup_iq3_table) selects the table-driven kernel
                              float* hp = nullptr);                        // f32 rows by pair position instead of the bf16 rows in hb (see launch_h_rows_to_f16)
// rows [first, first + count) of hp (f32, K wide) -> f16 rows scaled per row by a power of two + the inverse scales;
// first = *first_ptr + first_add (first_ptr may be null), count = min(*count_ptr, count_max) (count_ptr may be null)
cudaError_t launch_h_rows_to_f16(const Launch& L, const float* hp, void* hh, float* inv_scale, uint32_t K,
                                 const uint32_t* first_ptr, uint32_t first_add, const uint32_t* count_ptr, uint32_t count_max);
size_t gateup_iq3_table_bytes();
cudaError_t launch_gateup_iq3_table(const Launch& L, uint8_t* out);
cudaError_t launch_down_mma(const Launch& L, const qkm_dims& d, uint32_t type, const void* tiles, const void* hb,
                            const qkm_sel* sel, const uint32_t* pairs, const MmaItem* items, const uint32_t* n_items,
                            uint32_t max_items, float* contrib, uint32_t* status, bool few_blocks = false,
                            const uint8_t* iq4_table = nullptr,    // IQ4_XS: the table image (launch_down_iq4_table) selects the table-driven kernel
                            const float* h_inv_scale = nullptr);   // hb holds scaled f16 rows (launch_h_rows_to_f16): f16 operands
size_t down_iq4_table_bytes();
cudaError_t launch_down_iq4_table(const Launch& L, uint8_t* out);
cudaError_t launch_fold_pairs(const Launch& L, const qkm_dims& d, const float* contrib, const uint32_t* pos_of,
                              float* y, uint32_t n_tokens);

// ---- qkm_repack.cu : raw ggml -> tile layout (same bytes, see qkm_tiles.cuh)
cudaError_t launch_repack(const Launch& L, uint32_t type, const void* raw, void* out, uint32_t n_mats,
                          uint32_t rows, uint32_t K);

// ---- qkm_decode_gateup.cu / qkm_decode_down.cu : streaming kernels for small token counts
cudaError_t launch_encode_digits(const Launch& L, const float* x, int8_t* planes, float* scale,
                                 uint32_t n_rows, uint32_t K);
cudaError_t launch_gateup_stream(const Launch& L, const qkm_dims& d, uint32_t type, const void* gate_tiles,
                                 const void* up_tiles, const int8_t* xplanes, const float* xscale,
                                 const uint32_t* pairs, const StreamItem* items, const uint32_t* n_items,
                                 float* h, void* hpieces, uint32_t n_blocks, uint32_t* status);
// contrib [T][n_used+1][n_embd]; arrivals [T][n_embd/unit rows] zero before the first call
cudaError_t launch_down_stream(const Launch& L, const qkm_dims& d, uint32_t type, const void* tiles,
                               const void* hpieces, const qkm_sel* sel, const uint32_t* pairs,
                               const StreamItem* items, const uint32_t* n_items, float* contrib, float* y,
                               uint32_t* arrivals, uint32_t n_blocks, uint32_t* status);
uint32_t down_stream_unit_rows();
// token-major routed down: y[t] = sum_s w_s * D[ids_s].h[t][s] + y2[t] (y2 may be NULL)
cudaError_t launch_down_tok(const Launch& L, const qkm_dims& d, uint32_t type, const void* tiles,
                            const void* hpieces, const qkm_sel* sel, const float* y2, float* y,
                            uint32_t n_tokens, uint32_t n_blocks, uint32_t* status);
uint32_t gateup_stream_rows_per_item();
uint32_t down_stream_rows_per_item();

// ---- qkm_gemv.cu
cudaError_t launch_dequant(const Launch& L, uint32_t type, const void* blocks, float* y, uint64_t n_elems);
cudaError_t launch_gemv(const Launch& L, uint32_t type, const void* W, const float* x, float* y,
                        uint32_t M, uint32_t K, uint32_t n);

// streamed form (bulk-copy ring) with the generic kernel for tail rows / unaligned tensors
cudaError_t launch_gemv_mma(const Launch& L, uint32_t type, const void* W, const float* x, float* y, uint32_t M,
                            uint32_t K, uint32_t n_sms, uint32_t* status, uint32_t* rows_done);
cudaError_t launch_gemv_stream(const Launch& L, uint32_t type, const void* W, const float* x, float* y,
                               uint32_t M, uint32_t K, uint32_t n, uint32_t n_sms, uint32_t* status);

// ---- qkm_route.cu
// x rows as int8 digit planes + per-row scale (the selection kernel can write the same).
cudaError_t launch_xplanes(const Launch& L, const float* x, uint32_t n_tokens, uint32_t n_embd, int8_t* xplanes, float* xscale,
                           const float* gis = nullptr, qkm_sel* sel = nullptr);   // gis given: also sel[t].w_shared = sigmoid(gis . x)
// Optional tail of launch_route_select for decode-sized batches (<= 64 tokens, <= 1024 pairs,
// f64-logit path): the selection kernel's last block also groups the pairs and cuts the
// streaming kernels' work lists (what launch_group_plan does), saving a launch.  `counter` is a
// zero-initialised device word the kernel leaves at zero.  route_select_plans() tells whether
// a call with these sizes takes that path.
struct RoutePlan {
    uint32_t* counter;
    uint32_t* offsets;
    uint32_t* pairs;
    StreamItem* items_gu;
    StreamItem* items_dn;
    uint32_t* n_items;
    uint32_t chunks_gu, chunks_dn, tok_per_item, expert_first, expert_count;
    uint32_t shared_gate_elsewhere;   // 1: sel[t].w_shared is written by launch_xplanes (given gis); the selection kernel skips x
};
bool route_select_plans(const qkm_dims& d, uint32_t n_tokens, size_t scratch_bytes);
// Scratch the refined router needs: n_tokens * n_expert f32 logits + n_expert f32 row norms,
// or n_tokens * n_expert f64 logits for the small batches that are ranked in f64 directly.
size_t route_scratch_bytes(uint32_t n_tokens, uint32_t n_expert);
cudaError_t launch_logits(const Launch& L, const qkm_dims& d, uint32_t router_type, const void* router,
                          const float* x, float* logits, float* row_norm2, uint32_t n_tokens);
cudaError_t launch_select(const Launch& L, const qkm_dims& d, const float* logits, const float* gis,
                          const float* x, qkm_sel* sel, uint32_t n_tokens);
cudaError_t launch_route_select(const Launch& L, const qkm_dims& d, uint32_t router_type,
                                const void* router, const float* gis, const float* x, qkm_sel* sel,
                                uint32_t n_tokens, void* scratch, size_t scratch_bytes, int8_t* xplanes = nullptr,
                                float* xscale = nullptr, const void* x_f16 = nullptr, const float* x_f16_inv = nullptr,
                                uint32_t* status = nullptr, const RoutePlan* plan = nullptr);
// f32 logits from f16 operands on the tensor cores (x_f16 / x_inv_scale as written by launch_to_f16_rows);
// |error| <= 2^-9 * |router row| * |x|.  Needs n_expert % 128 == 0 and n_embd <= 4096.
cudaError_t launch_logits_mma(const Launch& L, const qkm_dims& d, uint32_t router_type, const void* router,
                              const void* x_f16, const float* x_inv_scale, float* logits, uint32_t n_tokens,
                              uint32_t* status, uint32_t splits = 1)   /* splits > 1: partial logits over column ranges, [splits][n_tokens][n_expert] */;
cudaError_t launch_group_pairs(const Launch& L, const qkm_dims& d, const qkm_sel* sel, uint32_t n_tokens,
                               uint32_t* offsets, uint32_t* pairs, uint32_t expert_first,
                               uint32_t expert_count);
// The same grouping spread over many blocks (large batches).  `hist` is scratch of
// group_wide_scratch_bytes(); pos_of (optional) gets, for every (token, slot), the position of
// the pair in `pairs`, or 0xFFFFFFFF when its expert is not resident.
size_t group_wide_scratch_bytes(uint32_t n_tokens, uint32_t n_used, uint32_t expert_count);
cudaError_t launch_group_pairs_wide(const Launch& L, const qkm_dims& d, const qkm_sel* sel, uint32_t n_tokens,
                                    uint32_t* offsets, uint32_t* pairs, uint32_t expert_first, uint32_t expert_count,
                                    uint32_t* hist, uint32_t* pos_of);
// group_pairs plus, in the same launch, the work lists of the streaming kernels
cudaError_t launch_group_plan(const Launch& L, const qkm_dims& d, const qkm_sel* sel, uint32_t n_tokens,
                              uint32_t* offsets, uint32_t* pairs, uint32_t expert_first, uint32_t expert_count,
                              StreamItem* items_gu, uint32_t chunks_gu, StreamItem* items_dn,
                              uint32_t chunks_dn, StreamItem* items_sh_gu, StreamItem* items_sh_dn,
                              uint32_t tok_per_item, uint32_t* n_items);

// shared-expert work lists: n_items[0] gate/up, n_items[1] down; pairs[n_tokens*n_used + t] = (t<<4)|n_used
cudaError_t launch_shared_plan(const Launch& L, const qkm_dims& d, uint32_t n_tokens, uint32_t* pairs,
                               StreamItem* items_gu, uint32_t chunks_gu, StreamItem* items_dn,
                               uint32_t chunks_dn, uint32_t tok_per_item, uint32_t* n_items);

// ---- qkm_moe_simple.cu : one warp per output element, raw ggml layout
cudaError_t launch_gateup_tokens(const Launch& L, const qkm_dims& d, uint32_t type, const void* gate,
                                 const void* up, const float* x, const qkm_sel* sel, float* h,
                                 uint32_t n_tokens, uint32_t expert_first, uint32_t expert_count);
cudaError_t launch_gateup_pairs(const Launch& L, const qkm_dims& d, uint32_t type, const void* gate,
                                const void* up, const float* x, const uint32_t* offsets,
                                const uint32_t* pairs, float* h, uint32_t n_tokens,
                                uint32_t expert_first, uint32_t expert_count);
cudaError_t launch_shared_gateup(const Launch& L, const qkm_dims& d, const void* gate, const void* up,
                                 const float* x, float* h, uint32_t n_tokens);
cudaError_t launch_down_tokens(const Launch& L, const qkm_dims& d, uint32_t type, const void* down,
                               const float* h, const qkm_sel* sel, float* y, uint32_t n_tokens,
                               uint32_t expert_first, uint32_t expert_count,
                               const void* down_shared /* NULL: routed only */);
cudaError_t launch_down_pairs(const Launch& L, const qkm_dims& d, uint32_t type, const void* down,
                              const float* h, const qkm_sel* sel, const uint32_t* offsets,
                              const uint32_t* pairs, float* contrib, uint32_t n_tokens,
                              uint32_t expert_first, uint32_t expert_count);
// y2 = w_shared * shared down; with contrib != NULL: y2 = sum_s contrib[.][s][.] + that
cudaError_t launch_shared_down(const Launch& L, const qkm_dims& d, const void* down, const float* h,
                               const qkm_sel* sel, float* y2, uint32_t n_tokens,
                               const float* contrib = nullptr);
// y[t][o] = sum over slots (in order) of contrib[t][s][o], plus y2[t][o] when y2 != NULL
cudaError_t launch_fold_contrib(const Launch& L, const qkm_dims& d, const float* contrib, const float* y2,
                                float* y, uint32_t n_tokens);

// Dense quantised GEMM Y[n][M] = X[n][K] . W^T on the tcgen05 pipeline (W tile-ordered Q8_0 / IQ4_XS,
// M % 128 == 0, K % 256 == 0).  Scratch: xb n*K bf16, pairs n words, unit_sel n records,
// items ceil(n/128) * M/128 entries, n_items one word.
cudaError_t launch_dense_gemm(const Launch& L, uint32_t type, const void* tiles, uint32_t M, uint32_t K, const float* x,
                              uint32_t n_rows, float* y, void* xb, uint32_t* pairs, qkm_sel* unit_sel, MmaItem* items,
                              uint32_t* n_items, uint32_t* status);

// ---- residual adds fused with the RMS norm (qkm_tail.cu) ---------------------------------------
// mode 0: s = a + b; 1: s = a + b + c2; 2: s = a + sum_k b[row][k][:] + c2 (b = per-slot contributions).
// xn = s * w / sqrt(mean(s^2) + eps).
cudaError_t launch_add_rms(const Launch& L, int mode, const float* a, const float* b, const float* c2, const float* w,
                           float* s, float* xn, uint32_t n_rows, uint32_t n, uint32_t n_used, float eps);

// greedy token per row of logits: largest value, lowest index on ties (scratch: argmax_scratch_bytes)
size_t argmax_scratch_bytes(uint32_t n_rows);
cudaError_t launch_argmax(const Launch& L, const float* logits, uint32_t n_rows, uint32_t n, void* scratch, uint32_t* tok);

// ---- expert-parallel exchange helpers (qkm_ep.cu) --------------------------------------------
// counts[0..n_ranks) rows per destination rank and counts[n_ranks] their sum; send_tok the
// tokens in send order; send_pos[t][r] the row of token t among the rows sent (to rank r).
// Receive buffers of every rank as this rank sees them (its own, and the peers' mapped ones).
constexpr uint32_t kMaxPeerRanks = 16;
struct EpPeerTable {
    float* x[kMaxPeerRanks];          // [n_ranks * slot_rows][n_embd] rows pushed by the sources
    qkm_sel* sel[kMaxPeerRanks];      // their selection records
    float* back[kMaxPeerRanks];       // [n_ranks * slot_rows][n_embd] partial rows returned by the owners
    uint32_t* flags[kMaxPeerRanks];   // [n_ranks] barrier words, word s written by rank s
};
cudaError_t launch_ep_barrier(const Launch& L, const EpPeerTable& peers, uint32_t rank, uint32_t n_ranks, uint32_t epoch,
                              uint64_t limit_ns, uint32_t* status);
// xh / x_inv_scale: the rows as scaled f16 (to_f16_rows_kernel) - then those travel instead of the f32 rows
cudaError_t launch_ep_push(const Launch& L, const qkm_dims& d, const float* x, const qkm_sel* sel, const EpPeerTable& peers,
                           uint32_t n_tokens, uint32_t slot_rows, uint32_t rank, uint32_t n_ranks, const void* xh = nullptr,
                           const float* x_inv_scale = nullptr);
cudaError_t launch_ep_row_scales(const Launch& L, const qkm_sel* selrecv, float* x_inv_scale, uint32_t n_rows);
constexpr uint32_t kSelScaleWord = 34;   // first padding word of a selection record (ids 0-15, w 16-31, w_shared, route_done, pad)
cudaError_t launch_fold_pairs_peer(const Launch& L, const qkm_dims& d, const float* contrib, const uint32_t* pos_of,
                                   const EpPeerTable& peers, uint32_t slot_rows, uint32_t rank, uint32_t n_ranks);
cudaError_t launch_ep_return(const Launch& L, const qkm_dims& d, const float* partial, const qkm_sel* selrecv,
                             const EpPeerTable& peers, uint32_t slot_rows, uint32_t rank, uint32_t n_ranks, uint32_t n_shared);
cudaError_t launch_ep_pull(const Launch& L, const qkm_dims& d, const qkm_sel* sel, const EpPeerTable& peers, const float* y2,
                           float* y, uint32_t n_tokens, uint32_t slot_rows, uint32_t rank, uint32_t n_ranks,
                           bool own_always);
cudaError_t launch_ep_plan(const Launch& L, const qkm_dims& d, const qkm_sel* sel, uint32_t n_tokens, uint32_t n_ranks,
                           uint32_t* counts, uint32_t* send_tok, uint32_t* send_pos);
cudaError_t launch_ep_pack(const Launch& L, const qkm_dims& d, const float* x, const qkm_sel* sel,
                           const uint32_t* send_tok, const uint32_t* total, uint32_t max_rows, float* xsend,
                           qkm_sel* selsend);
cudaError_t launch_ep_combine(const Launch& L, const qkm_dims& d, const float* back, const uint32_t* send_pos,
                              const float* y2, float* y, uint32_t n_tokens, uint32_t n_ranks);

}  // namespace qkm
