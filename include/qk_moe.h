/* qk_moe.h — C ABI of the B200 (sm_100a) quantized MoE feed-forward path.
 *
 * This is the boundary a qk engine binds instead of its per-layer MoE / GEMV
 * shader dispatches.  It keeps the conventions of the engine ABI
 * (reference include/qk.h:18-29): an opaque handle, an open call that returns
 * NULL and fills a NUL-terminated error string, every other call returning 0
 * (or a non-negative count) on success and a negative code on failure, the
 * caller owning every output buffer, inputs copied at upload, and ALL calls on
 * one context made from a single thread (reference include/qk.h:3-7).
 *
 * Differences a caller must know:
 *   - calls that launch GPU work are asynchronous on the context's CUDA
 *     stream; qkm_sync() (or a *_host call, which synchronises itself) makes
 *     results visible;
 *   - there is no CPU fallback: without a CUDA device qkm_open fails.
 *
 * Buffer layouts are the reference's (file:line under the reference tree):
 *   x        [T][n_embd] f32                       shaders/moe_logits.comp:12
 *   logits   [T][n_expert] f32                     shaders/moe_logits.comp:13
 *   sel      qkm_sel[T], 160 B each                shaders/moe_select.comp:15
 *   h        [T][n_used+1][n_ff] f32, slot n_used = shared expert
 *                                                  shaders/moe_gateup_iq3.comp:42
 *   y, y2    [T][n_embd] f32                       shaders/moe_down_iq4.comp:29
 *   offsets  [n_expert+1] u32, pairs [T*n_used] u32 = (token<<4)|slot
 *                                                  shaders/moe_group_pairs.comp:24-50
 *   contrib  [T][n_used][n_embd] f32               shaders/moe_down_iq4_grouped.comp
 * Weight tensors are raw ggml blocks (reference src/quants.h:52-119), row-major
 * [n_expert][rows][K/blk] exactly as they sit in a GGUF file.
 */
#ifndef QK_MOE_H
#define QK_MOE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(_WIN32)
#define QKM_API
#else
#define QKM_API __attribute__((visibility("default")))
#endif

/* ggml tensor type ids (reference src/gguf.h:17-21). */
enum {
    QKM_TYPE_F32 = 0,
    QKM_TYPE_F16 = 1,
    QKM_TYPE_Q8_0 = 8,
    QKM_TYPE_Q6_K = 14,
    QKM_TYPE_IQ3_XXS = 18,
    QKM_TYPE_IQ4_XS = 23
};

/* Error codes (negative).  -1..-5 keep the meaning they have in the reference
 * engine (src/main.cpp:5447-5453, :5530). */
enum {
    QKM_OK = 0,
    QKM_ERR_ARG = -1,      /* NULL handle / bad argument                    */
    QKM_ERR_BUSY = -2,     /* layer not uploaded / context in wrong state    */
    QKM_ERR_BOUNDS = -3,   /* size beyond the limits given at open           */
    QKM_ERR_TYPE = -4,     /* unsupported ggml type for this operand         */
    QKM_ERR_MODE = -5,     /* call not valid in this mode (e.g. EP not set)  */
    QKM_ERR_CUDA = -6,     /* a CUDA runtime call failed; see qkm_last_error */
    QKM_ERR_TIMEOUT = -7   /* a bounded device-side wait gave up             */
};

/* Selection record, one per token (reference shaders/moe_select.comp:15 and
 * shaders/moe_route_select.comp:17-23: the fused variant uses the first pad
 * word as its arrival counter).  ids are in descending-logit order; w is the
 * softmax over the selected logits only; w_shared = sigmoid(gate_inp_shexp.x). */
typedef struct qkm_sel {
    uint32_t ids[16];
    float    w[16];
    float    w_shared;
    uint32_t route_done;
    float    pad[6];
} qkm_sel;

/* The 4xu32 push constant every MoE shader receives (src/main.cpp:4202). */
typedef struct qkm_dims {
    uint32_t n_embd;   /* hidden width, multiple of 256                      */
    uint32_t n_ff;     /* expert FFN width, multiple of 256 (main.cpp:3620)  */
    uint32_t n_expert; /* 1..512 (main.cpp:955)                              */
    uint32_t n_used;   /* 1..16, <= n_expert (main.cpp:1298)                 */
} qkm_dims;

typedef struct qkm_config {
    qkm_dims dims;
    uint32_t n_layer;     /* number of layer slots that can be uploaded, >= 1 */
    uint32_t max_tokens;  /* largest T any call will pass, >= 1               */
    int32_t  device;      /* CUDA device ordinal; -1 = current device         */
    uint32_t flags;       /* QKM_FLAG_*                                       */
    /* Expert parallel view (0/0 = all experts local).  Experts
     * [expert_first, expert_first+expert_count) are resident on this GPU. */
    uint32_t expert_first;
    uint32_t expert_count;
} qkm_config;

enum {
    QKM_FLAG_NONE = 0
};

/* One layer's eight MoE tensors (the set loadMoeT reads, src/main.cpp:1265-1308).
 * Pointers are HOST pointers for qkm_upload_layer and DEVICE pointers when the
 * struct is filled by qkm_layer_device_ptrs.  With an expert-parallel view the
 * three *_exps tensors hold only the resident experts, first resident expert
 * first. */
typedef struct qkm_layer_weights {
    uint32_t router_type;   /* QKM_TYPE_F32 (reference) or QKM_TYPE_F16        */
    uint32_t gateup_type;   /* QKM_TYPE_IQ3_XXS or QKM_TYPE_IQ4_XS             */
    uint32_t down_type;     /* QKM_TYPE_IQ4_XS or QKM_TYPE_Q6_K                */
    uint32_t reserved;
    const void  *router;          /* ffn_gate_inp        [n_expert][n_embd]      */
    const float *gate_inp_shexp;  /* ffn_gate_inp_shexp  [n_embd] f32            */
    const void  *gate_exps;       /* ffn_gate_exps       [n_expert][n_ff][n_embd] */
    const void  *up_exps;         /* ffn_up_exps         [n_expert][n_ff][n_embd] */
    const void  *down_exps;       /* ffn_down_exps       [n_expert][n_embd][n_ff] */
    const void  *gate_shexp;      /* ffn_gate_shexp      [n_ff][n_embd] Q8_0      */
    const void  *up_shexp;        /* ffn_up_shexp        [n_ff][n_embd] Q8_0      */
    const void  *down_shexp;      /* ffn_down_shexp      [n_embd][n_ff] Q8_0      */
} qkm_layer_weights;

typedef struct qkm_ctx qkm_ctx;

/* ---- lifecycle (shape of qk_open/qk_close, include/qk.h:26-29) ---------- */
QKM_API qkm_ctx *qkm_open(const qkm_config *cfg, char *err, size_t err_len);
QKM_API void     qkm_close(qkm_ctx *c);
QKM_API const char *qkm_last_error(const qkm_ctx *c);
QKM_API const char *qkm_version(void);

/* getters (include/qk.h:31-36 style) */
QKM_API uint32_t qkm_n_embd(const qkm_ctx *c);
QKM_API uint32_t qkm_n_ff(const qkm_ctx *c);
QKM_API uint32_t qkm_n_expert(const qkm_ctx *c);
QKM_API uint32_t qkm_n_used(const qkm_ctx *c);
QKM_API uint32_t qkm_n_layer(const qkm_ctx *c);
QKM_API uint32_t qkm_max_tokens(const qkm_ctx *c);
/* resident experts [first, first + count) of this context (all of them when unsharded) */
QKM_API void     qkm_expert_range(const qkm_ctx *c, uint32_t *first, uint32_t *count);
/* bytes per row of ne0 elements of a ggml type, 0 if unsupported
 * (ggmlRowBytes, src/gguf.h:36-46) */
QKM_API size_t   qkm_row_bytes(uint32_t type, uint64_t ne0);

/* Stream the context launches on (a cudaStream_t passed as void*; NULL = the
 * legacy default stream).  qkm_sync waits for it. */
QKM_API int qkm_set_stream(qkm_ctx *c, void *cuda_stream);
QKM_API int qkm_sync(qkm_ctx *c);
/* Number of kernels this context has launched since open (bench accounting). */
QKM_API uint64_t qkm_launch_count(const qkm_ctx *c);

/* Plain device memory for callers that do not link the CUDA runtime. */
QKM_API void *qkm_dev_alloc(qkm_ctx *c, size_t bytes);
QKM_API int   qkm_dev_free(qkm_ctx *c, void *p);
QKM_API int   qkm_h2d(qkm_ctx *c, void *dst_dev, const void *src_host, size_t bytes);
QKM_API int   qkm_d2h(qkm_ctx *c, void *dst_host, const void *src_dev, size_t bytes);

/* ---- weights ------------------------------------------------------------ */
/* Copy one layer's tensors to the GPU (replaces the per-layer upload in
 * qk_engine::open, src/main.cpp:4031-4067).  The caller keeps ownership. */
QKM_API int qkm_upload_layer(qkm_ctx *c, uint32_t layer, const qkm_layer_weights *host);
/* Device addresses of an uploaded layer, for the op-level calls below. */
QKM_API int qkm_layer_device_ptrs(const qkm_ctx *c, uint32_t layer, qkm_layer_weights *out);

/* ---- op-level entry points: one per reference shader group ---------------
 * All pointers are DEVICE pointers.  n_tokens is the reference's grid-z. */

/* moe_logits.comp:18-36 / moe_logits_gemm.comp:34-73 */
QKM_API int qkm_moe_logits(qkm_ctx *c, uint32_t router_type, const void *router,
                           const float *x, float *logits, uint32_t n_tokens);
/* moe_select.comp:24-76 / moe_select_256.comp:31-96: top-n_used of the given
 * f32 logits (non-finite -> -3.4e38, lowest id wins ties), softmax over the
 * selected, w_shared. */
QKM_API int qkm_moe_select(qkm_ctx *c, const float *logits, const float *gate_inp_shexp,
                           const float *x, qkm_sel *sel, uint32_t n_tokens);
/* moe_route_select.comp:41-130 (+_hier): logits and selection in one call.
 * This is the path the fused layer calls use: candidates near the selection
 * boundary are re-evaluated in f64 so ids equal an f64-accumulating CPU router
 * (src/main.cpp:1320-1341). */
QKM_API int qkm_moe_route_select(qkm_ctx *c, uint32_t router_type, const void *router,
                                 const float *gate_inp_shexp, const float *x,
                                 qkm_sel *sel, uint32_t n_tokens);
/* moe_group_pairs.comp:19-50 */
QKM_API int qkm_moe_group_pairs(qkm_ctx *c, const qkm_sel *sel, uint32_t n_tokens,
                                uint32_t *offsets, uint32_t *pairs);
/* moe_gateup_iq3.comp:34-106 / moe_gateup_iq4.comp (+_rowtile): token-major */
QKM_API int qkm_moe_gateup(qkm_ctx *c, uint32_t type, const void *gate_exps,
                           const void *up_exps, const float *x, const qkm_sel *sel,
                           float *h, uint32_t n_tokens);
/* moe_gateup_iq3_grouped*.comp: expert-major over offsets/pairs */
QKM_API int qkm_moe_gateup_grouped(qkm_ctx *c, uint32_t type, const void *gate_exps,
                                   const void *up_exps, const float *x,
                                   const uint32_t *offsets, const uint32_t *pairs,
                                   float *h, uint32_t n_tokens);
/* moe_gateup_q8.comp:30-62 (+_64, _coopmat): shared expert -> h[t][n_used][:] */
QKM_API int qkm_moe_shared_gateup(qkm_ctx *c, const void *gate_shexp, const void *up_shexp,
                                  const float *x, float *h, uint32_t n_tokens);
/* moe_down_iq4.comp:35-81 / moe_down_q6k.comp:33-84: token-major weighted sum */
QKM_API int qkm_moe_down(qkm_ctx *c, uint32_t type, const void *down_exps, const float *h,
                         const qkm_sel *sel, float *y, uint32_t n_tokens);
/* moe_down_{iq4,q6k}_grouped*.comp: expert-major, per-(token,slot) contributions */
QKM_API int qkm_moe_down_grouped(qkm_ctx *c, uint32_t type, const void *down_exps,
                                 const float *h, const qkm_sel *sel,
                                 const uint32_t *offsets, const uint32_t *pairs,
                                 float *contrib, uint32_t n_tokens);
/* moe_down_q8b.comp:31-57 (+_32, moe_down_q8_coopmat.comp) */
QKM_API int qkm_moe_shared_down(qkm_ctx *c, const void *down_shexp, const float *h,
                                const qkm_sel *sel, float *y2, uint32_t n_tokens);
/* gemv_{f16,q8_0,q6_k,iq4_xs,iq3_xxs}.comp; n = grid-z batch (gemv_q8_0.comp:31-32):
 * y[n][M] = W[M][K] . x[n][K] */
QKM_API int qkm_gemv(qkm_ctx *c, uint32_t type, const void *W, const float *x, float *y,
                     uint32_t M, uint32_t K, uint32_t n);
/* dequant_row_* (src/quants.h:70-165) on the GPU: the bit-exactness probe. */
QKM_API int qkm_dequant(qkm_ctx *c, uint32_t type, const void *blocks, float *y,
                        uint64_t n_elems);

/* ---- fused layer calls --------------------------------------------------- */
/* Decode sequence of one layer (src/main.cpp:4375-4404) for T tokens/slots:
 * router -> top-k -> routed gate/up + shared gate/up -> routed + shared down,
 * y = sum_s w_s*down_s + w_shared*down_shared.  x, y: device [T][n_embd]. */
QKM_API int qkm_moe_decode(qkm_ctx *c, uint32_t layer, const float *x, uint32_t n_tokens,
                           float *y);
/* Batched-prefill sequence (src/main.cpp:5050-5198): grouped by expert, expert
 * GEMMs on the tensor cores with f16 operands (x and h rows scaled per row by a power of
 * two) and f32 accumulation. */
QKM_API int qkm_moe_prefill(qkm_ctx *c, uint32_t layer, const float *x, uint32_t n_tokens,
                            float *y);
/* Same two calls with HOST buffers: copies x in, runs, copies y out, syncs.
 * mode 0 = decode path, 1 = prefill path. */
QKM_API int qkm_moe_forward_host(qkm_ctx *c, uint32_t layer, int mode, const float *x_host,
                                 uint32_t n_tokens, float *y_host);
/* Decode through layers [0, n_layer) in sequence, feeding each layer the same
 * per-layer input rows x[l] (device [n_layer][T][n_embd]); y likewise. */
QKM_API int qkm_moe_decode_stack(qkm_ctx *c, uint32_t layer_first, uint32_t layer_count,
                                 const float *x, uint32_t n_tokens, float *y);
/* The same with HOST buffers [layer_count][T][n_embd], then a stream synchronise.  From eight
 * layers on (and on a stream of the caller's) the stack runs in four chunks of layers (two layers,
 * two halves of the rest, two layers): all input
 * copies are queued at once on a copy stream, a chunk starts when its rows have arrived and its
 * outputs leave on a third stream while the next chunk computes.  Pinned host memory makes the
 * copies asynchronous. */
QKM_API int qkm_moe_decode_stack_host(qkm_ctx *c, uint32_t layer_first, uint32_t layer_count,
                                      const float *x_host, uint32_t n_tokens, float *y_host);
/* Per-stage device timing of the fused calls (the reference's QK_STEP_PROF,
 * src/main.cpp:4173-4185, :4591-4632: a timestamp after every stage of the decode
 * sequence, reported per label).  While enabled, qkm_moe_decode / qkm_moe_prefill
 * record a CUDA event on the context's stream after each stage; qkm_profile_read
 * synchronises and returns, for the LAST fused call, the number of stages, their
 * labels (16 bytes each, NUL-terminated) and their durations in milliseconds. */
QKM_API int qkm_profile_enable(qkm_ctx *c, int on);
QKM_API int qkm_profile_read(qkm_ctx *c, char *labels, float *ms, uint32_t max_stages);
/* Selection records of the last fused call (device -> host copy, syncs). */
QKM_API int qkm_last_sel(qkm_ctx *c, qkm_sel *sel_host, uint32_t n_tokens);
/* Device address of the context's selection / h scratch of the last fused call (h in f32 is
 * written by the decode calls and by the prefill calls that take the f32 kernels; the tensor-core
 * prefill writes f32 rows by pair position there, not [T][slot]). */
QKM_API const qkm_sel *qkm_sel_device(const qkm_ctx *c);
QKM_API const float   *qkm_h_device(const qkm_ctx *c);

/* ---- dense quantised GEMM (gemm_q8_0*.comp, gemm_iq4_xs.comp; src/main.cpp:4806-4835) -----
 * Y[n][M] = X[n][K] . W^T for a Q8_0 or IQ4_XS matrix W [M][K] (ggml rows), M % 128 == 0,
 * K % 256 == 0.  qkm_dense_upload copies W (host pointer) into one of 16 slots; qkm_dense_gemm
 * takes device x [n][K] / y [n][M] f32 and runs on the tensor cores with bf16 operands
 * (the prefill tolerance applies).  Scratch grows to the largest n seen. */
QKM_API int qkm_dense_upload(qkm_ctx *c, uint32_t slot, uint32_t type, const void *w_host,
                             uint32_t M, uint32_t K);
QKM_API int qkm_dense_gemm(qkm_ctx *c, uint32_t slot, const float *x, uint32_t n, float *y);

/* ---- GGUF files (src/gguf.h:54-198; tensor set and checks of loadMoeT, src/main.cpp:1265-1308)
 * Read-only, memory-mapped; a split model is opened by its first shard
 * ("<prefix>-00001-of-000NN.gguf").  Every length in the file is bounds-checked; failures
 * return NULL / a negative code with a message, they never abort. */
typedef struct qkm_gguf qkm_gguf;
QKM_API qkm_gguf *qkm_gguf_open(const char *path, char *err, size_t err_len);
QKM_API void      qkm_gguf_close(qkm_gguf *g);
QKM_API const char *qkm_gguf_last_error(const qkm_gguf *g);
QKM_API uint64_t  qkm_gguf_tensor_count(const qkm_gguf *g);
/* tensor by name: ggml type, ne[4], pointer into the mapping, bytes left in its shard */
QKM_API int qkm_gguf_find(const qkm_gguf *g, const char *name, uint32_t *type, uint64_t ne[4],
                          const void **data, uint64_t *nbytes);
QKM_API uint64_t qkm_gguf_kv_u64(const qkm_gguf *g, const char *key, uint64_t def);
QKM_API int qkm_gguf_kv_str(const qkm_gguf *g, const char *key, char *out, size_t out_len);
/* the eight blk.<layer>.ffn_* tensors, validated: dims for qkm_open, host pointers for
 * qkm_upload_layer */
QKM_API int qkm_gguf_moe_layer(qkm_gguf *g, uint32_t layer, qkm_dims *dims, qkm_layer_weights *w);
/* file layer -> context layer; a sharded context takes its slice of the expert tensors */
QKM_API int qkm_upload_layer_gguf(qkm_ctx *c, uint32_t layer, qkm_gguf *g, uint32_t file_layer);

/* ---- layer entry / tail around the MoE block ------------------------------------------
 * add_rmsnorm.comp:22-40: y = a + b, xn = y * w / sqrt(mean(y^2) + eps); rows of n f32. */
QKM_API int qkm_add_rmsnorm(qkm_ctx *c, const float *a, const float *b, const float *w, float *y,
                            float *xn, uint32_t n_rows, uint32_t n, float eps);
/* add_rms3.comp:23-41: s = a + b + c2 (residual + routed + shared), xn = rmsnorm(s) * w */
QKM_API int qkm_add_rms3(qkm_ctx *c, const float *a, const float *b, const float *c2, const float *w,
                         float *s, float *xn, uint32_t n_rows, uint32_t n, float eps);
/* add_rms3_grouped.comp:22-50: the routed stream as contrib [row][n_used][n], folded in
 * slot order before the shared stream is added */
QKM_API int qkm_add_rms3_grouped(qkm_ctx *c, const float *a, const float *routed, const float *c2,
                                 const float *w, float *s, float *xn, uint32_t n_rows, uint32_t n,
                                 uint32_t n_used, float eps);
/* argmax1.comp:17-40 + argmax2.comp:16-32 (after the head GEMV, src/main.cpp:4406-4412): per row
 * of n logits the index of the largest value, the lower index on ties; values must exceed
 * -3.4e38 to count (NaN never wins; a row with nothing above the floor gives 0).  tok: device u32[n_rows]. */
QKM_API int qkm_argmax(qkm_ctx *c, const float *logits, uint32_t n_rows, uint32_t n, uint32_t *tok);
/* The feed-forward half of a decoder layer as the engine sequences it (src/main.cpp:4375-4404:
 * add_rmsnorm, the MoE dispatches, add_rms3): resid_out = resid + attn_out + MoE(rmsnorm(resid +
 * attn_out) * w_post); xn_next = rmsnorm(resid_out) * w_next.  resid_out may alias resid.
 * n_tokens <= 64 takes the decode kernels, more the tensor-core path. */
QKM_API int qkm_moe_layer_step(qkm_ctx *c, uint32_t layer, const float *resid, const float *attn_out,
                               const float *w_post, const float *w_next, uint32_t n_tokens, float eps,
                               float *resid_out, float *xn_next);

/* ---- expert parallel (one context per GPU; no counterpart in the reference, which is
 * single-GPU: the arithmetic per (token, expert) is that of src/main.cpp:1351-1369) -------
 * Rank r of n_ranks is a context opened with expert_first = r * n_expert / n_ranks and
 * expert_count = n_expert / n_ranks; router and shared-expert weights are replicated, the
 * three *_exps tensors hold the shard.  Tokens are data-parallel.  Per layer and rank:
 *
 *   qkm_ep_dispatch        route the n local tokens; for every rank that owns at least one
 *                          of a token's experts, one row of xsend (the token's x) and of
 *                          selsend (its selection record), rank by rank, ascending token
 *                          within a rank.  counts_host[r] = rows for rank r.  Blocks until
 *                          the counts are on the host.  xsend / selsend must hold
 *                          n * min(n_ranks, n_used) rows.
 *   (caller)               all-to-all-v of xsend and selsend by counts -> xrecv, selrecv
 *   qkm_ep_shared          shared expert of the local tokens; overlaps the exchange
 *   qkm_ep_expert_forward  resident experts over the n_recv received rows: partial[i] =
 *                          sum over the slots of row i whose expert is resident of
 *                          w_slot * down(silu(gate x) * up x); n_recv <= max_tokens
 *   (caller)               all-to-all-v of partial back (the reverse split) -> back, which
 *                          then has one row per row of xsend, in the same order
 *   qkm_ep_combine         y[t] = shared(t) + sum of t's rows of back in rank order
 */
QKM_API int qkm_ep_dispatch(qkm_ctx *c, uint32_t layer, const float *x, uint32_t n_tokens,
                            uint32_t n_ranks, float *xsend, qkm_sel *selsend,
                            uint32_t *counts_host);
/* As qkm_ep_dispatch, but asynchronous: counts_dev (DEVICE memory, n_ranks 32-bit words)
 * receives the row counts on the context's stream; nothing is copied to the host. */
QKM_API int qkm_ep_dispatch_dev(qkm_ctx *c, uint32_t layer, const float *x, uint32_t n_tokens,
                                uint32_t n_ranks, float *xsend, qkm_sel *selsend,
                                uint32_t *counts_dev);
QKM_API int qkm_ep_shared(qkm_ctx *c, uint32_t layer, const float *x, uint32_t n_tokens);
QKM_API int qkm_ep_expert_forward(qkm_ctx *c, uint32_t layer, const float *xrecv,
                                  const qkm_sel *selrecv, uint32_t n_recv, float *partial);
QKM_API int qkm_ep_combine(qkm_ctx *c, uint32_t n_tokens, uint32_t n_ranks, const float *back,
                           float *y);

/* Expert parallel over peer memory (NVLink loads and stores), NO COUNTERPART IN THE
 * REFERENCE.  The same layer without an all-to-all: each rank keeps receive buffers of
 * n_ranks * slot_cap rows and has every peer's buffers mapped.  A token's row and record
 * are stored by the push kernel straight into the buffers of the ranks that own its
 * experts, at row (source rank * slot_rows + token), so no counts travel and nothing is
 * packed; the owners store their partial rows into the source's return buffer the same
 * way, and the pull kernel sums them from local memory.
 *   qkm_ep_peer_setup(c, n_ranks, rank, slot_cap)  once; n_ranks * slot_cap <= max_tokens,
 *                          n_ranks <= 16, the context opened on shard `rank`
 *   qkm_ep_peer_export / qkm_ep_peer_import  QKM_EP_HANDLE_BYTES of CUDA IPC handles per
 *                          rank, exchanged by the caller (processes of one node), or
 *   qkm_ep_peer_buffers / qkm_ep_peer_set    raw device pointers (one process, several
 *                          GPUs with peer access enabled)
 * Per layer, all ranks with the same slot_rows (>= every rank's n_tokens, <= slot_cap):
 *   qkm_ep_push(c, layer, x, n_tokens, slot_rows)   route + store rows into the owners
 *   qkm_ep_shared(c, layer, x, n_tokens)
 *   (caller)  barrier: any collective of the ranks enqueued on the context's stream
 *   qkm_ep_forward_slots(c, layer, slot_rows, n_shared)  resident experts over all slots;
 *             n_shared = QKM_EP_NO_SHARED after a qkm_ep_shared call, or n_tokens INSTEAD
 *             of that call: the shared expert of this rank's tokens then runs beside the
 *             resident experts and arrives with this rank's partial rows
 *   (caller)  barrier
 *   qkm_ep_pull(c, n_tokens, slot_rows, y)          y = shared + the returned partial rows
 * The two barriers are all the ordering the buffers need from one layer to the next.
 * No kernel waits on another GPU, nothing is read by the host. */
#define QKM_EP_HANDLE_BYTES 192
#define QKM_EP_NO_SHARED 0xFFFFFFFFu
QKM_API int qkm_ep_peer_setup(qkm_ctx *c, uint32_t n_ranks, uint32_t rank, uint32_t slot_cap);
QKM_API int qkm_ep_peer_buffers(qkm_ctx *c, void **xrecv, void **selrecv, void **back);
QKM_API int qkm_ep_peer_set(qkm_ctx *c, uint32_t peer, void *xrecv, void *selrecv, void *back);
QKM_API int qkm_ep_peer_export(qkm_ctx *c, void *handles);
QKM_API int qkm_ep_peer_import(qkm_ctx *c, uint32_t peer, const void *handles);
QKM_API int qkm_ep_push(qkm_ctx *c, uint32_t layer, const float *x, uint32_t n_tokens,
                        uint32_t slot_rows);
QKM_API int qkm_ep_forward_slots(qkm_ctx *c, uint32_t layer, uint32_t slot_rows,
                                 uint32_t n_shared);
QKM_API int qkm_ep_pull(qkm_ctx *c, uint32_t n_tokens, uint32_t slot_rows, float *y);
/* The barrier as a kernel of the library: each rank stores a barrier number into a word of
 * every peer's buffer and polls its own words.  Every rank issues the same sequence of
 * barriers, each rank on its own GPU (two ranks' barriers on one device would wait on each
 * other's launch).  The wait is bounded: after timeout_ms (> 0) the kernel gives up and the
 * next qkm_sync returns QKM_ERR_TIMEOUT; the context stays usable.  slot_cap must be the
 * same on all ranks.  qkm_ep_peer_layer is the whole per-layer sequence above with these
 * barriers, one call per layer, nothing read by the host. */
QKM_API int qkm_ep_barrier(qkm_ctx *c, uint32_t timeout_ms);
QKM_API int qkm_ep_peer_layer(qkm_ctx *c, uint32_t layer, const float *x, uint32_t n_tokens,
                              uint32_t slot_rows, float *y, uint32_t timeout_ms);

/* Router logits + selection WITHOUT any device allocation and without a context.
 * NO COUNTERPART IN THE REFERENCE: it exists for hosts that may not take memory from
 * the driver while they run (a server that already owns all free HBM through its own
 * pool, a latency-bound loop in which an allocation may stall the device, a plugin in
 * a process with externally accounted memory).  Same selection rules as
 * qkm_moe_route_select and the same expert ids.  Up to 64 tokens the context call ranks
 * f64 logits; this call does the same while n_tokens * n_expert * 8 bytes fit the array
 * (then the weights are bit-identical), and otherwise ranks f32 logits and re-evaluates
 * the boundary in f64 (e.g. 64 tokens x 512 experts: ids still equal, softmax weights
 * equal to about 1e-6 relative).  Scratch is a fixed array inside the library image, one
 * per device, shared by all calls on that device:
 *   - limits: n_tokens * n_expert <= QKM_STATIC_ROUTE_MAX_LOGITS and
 *     n_expert <= QKM_STATIC_ROUTE_MAX_EXPERTS; larger calls return QKM_ERR_ARG and
 *     write the reason to `err`;
 *   - nothing in the array needs to start at zero (each call writes all it reads);
 *   - calls that overlap in time on one device race on the array: keep them on one
 *     stream or order them with events;
 *   - the first call on a device looks up the array's address (and lets the runtime
 *     initialise the device if the process has not used it): make it during start-up,
 *     before any stream capture.  The address is cached for the life of the process
 *     and does not survive a cudaDeviceReset;
 *   - the caller's current device is left as it was.
 * `stream` is a cudaStream_t (NULL = default stream); all pointers are device memory. */
#define QKM_STATIC_ROUTE_MAX_LOGITS  32768u
#define QKM_STATIC_ROUTE_MAX_EXPERTS 512u
QKM_API int qkm_route_select_static(int device, void *stream, const qkm_dims *dims,
                                    uint32_t router_type, const void *router,
                                    const float *gate_inp_shexp, const float *x, qkm_sel *sel,
                                    uint32_t n_tokens, char *err, size_t err_len);

#ifdef __cplusplus
}
#endif

#endif /* QK_MOE_H */
