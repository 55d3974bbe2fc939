// The C ABI of include/qk_moe.h: context, weight upload, op-level entry points and
// the fused per-layer sequences.  Host-side C++; every kernel lives in the other
// translation units and is reached through qkm_kernels.h.
//
// The call sequences mirror the reference engine's dispatch order: decode
// src/main.cpp:4375-4404, batched prefill src/main.cpp:5050-5198.
#include <cuda_runtime.h>

#include <cstdarg>
#include <cstdlib>
#include <cstdio>
#include <cstring>
#include <new>
#include <vector>

#include "qkm_common.cuh"
#include "qkm_kernels.h"

using namespace qkm;

struct qkm_layer_dev {
    bool uploaded = false;
    qkm_layer_weights w{};  // device pointers, raw ggml layout
    void* allocs[8] = {nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr};
    // tile-ordered copies for the streaming kernels (NULL where the type has none)
    void* tiles[8] = {nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr};
    bool tiles_ok = false;   // routed gate/up and down both have tiles
    bool stream_ok = false;  // tiles, and every expert resident: the fused decode / prefill sequences apply
    bool gu_only = false;    // as stream_ok for gate/up and the shared expert; the down tensor is Q6_K (tiles[4] holds Q6_K tiles)
    bool fused_ok = false;   // every tensor has tiles and every expert is resident (any supported type mix): the
                             // three-kernel decode sequence and the tensor-core prefill apply
};

struct qkm_ctx {
    qkm_config cfg{};
    int device = 0;
    cudaStream_t stream = nullptr;
    uint64_t launches = 0;
    char err[512] = {0};
    std::vector<qkm_layer_dev> layers;
    uint32_t efirst = 0, ecount = 0;  // resident experts (ecount == n_expert when unsharded)
    // scratch, sized for max_tokens
    qkm_sel* sel = nullptr;
    float* h = nullptr;
    void* route_scratch = nullptr;
    size_t route_scratch_bytes = 0;
    uint32_t* offsets = nullptr;
    uint32_t* pairs = nullptr;
    float* contrib = nullptr;  // allocated on first use
    float* y2 = nullptr;
    float* x_stage = nullptr;
    float* y_stage = nullptr;
    float* stack_x = nullptr;  // [n_layer][max_tokens][n_embd], allocated on first use
    float* stack_y = nullptr;
    // streaming path scratch
    int n_sms = 0;
    int8_t* xplanes = nullptr;        // [max_tokens][4][n_embd]
    float* xscale = nullptr;          // [max_tokens]
    void* hpieces = nullptr;          // [max_tokens*n_used][3][n_ff] bf16
    StreamItem* items_gu = nullptr;
    StreamItem* items_dn = nullptr;
    StreamItem* items_sh_gu = nullptr;
    StreamItem* items_sh_dn = nullptr;
    uint32_t* n_items = nullptr;      // [0] gate/up, [1] down, [2] shared gate/up, [3] shared down
    float* contrib_s = nullptr;       // [max_tokens][n_used+1][n_embd]
    uint32_t* arrivals = nullptr;     // [max_tokens][n_embd / unit rows]
    uint32_t* status = nullptr;       // kernel status word (device)
    uint32_t shared_plan_n = 0;        // token count the shared expert's decode work lists were last cut for (0: stale)
    uint32_t* route_counter = nullptr; // ticket counter of the selection kernel's grouping tail (device, stays zero)
    // fused decode sequence (router + grouping + planes -> gate/up -> down, three launches)
    bool dec_ok = false;               // dims fit the fused decode kernels
    int8_t* planes8 = nullptr;         // [max_tokens][n_embd/256][8][256]
    uint8_t* lut_gu = nullptr;         // table images the decode kernels copy to shared memory
    uint8_t* lut_dd = nullptr;         // table image of the decode IQ4_XS down kernel
    uint8_t* lut_pf = nullptr;         // table image of the prefill IQ3_XXS gate/up kernel
    uint8_t* lut_dn = nullptr;         // table image of the prefill IQ4_XS down kernel
    uint32_t* status_host = nullptr;  // pinned mirror
    bool shapes_stream_ok = false;
    // prefill (tcgen05) scratch, allocated on first use
    void* xb = nullptr;               // [max_tokens][n_embd] f16, rows scaled by powers of two (xscale undoes it)
    void* hb = nullptr;               // [max_tokens*(n_used+1)][n_ff] hidden rows by pair position: f16 scaled per row (bf16 on the f32-down path)
    float* hscale = nullptr;          // [max_tokens*(n_used+1)] the scales that undo the rows' scaling
    float* contrib_p = nullptr;       // [max_tokens*(n_used+1)][n_embd]
    MmaItem* mma_items[4] = {nullptr, nullptr, nullptr, nullptr};  // gate/up, down, shared gate/up, shared down
    uint32_t* pos_of = nullptr;       // [max_tokens*(n_used+1)]
    uint32_t* group_hist = nullptr;   // scratch of the multi-block grouping
    void* argmax_scratch = nullptr; uint32_t argmax_rows = 0;
    // dense matrices for qkm_dense_gemm (tile-ordered copies) and its scratch, sized on demand
    static constexpr int kDenseSlots = 16;
    struct Dense { uint32_t type = 0, M = 0, K = 0; void* tiles = nullptr; } dense[kDenseSlots];
    void* dense_xb = nullptr; uint32_t* dense_pairs = nullptr; qkm_sel* dense_sel = nullptr; MmaItem* dense_items = nullptr;
    uint32_t* dense_n_items = nullptr;
    size_t dense_cap_elems = 0, dense_cap_rows = 0, dense_cap_items = 0;
    // expert-parallel exchange plan of the last qkm_ep_dispatch, allocated on first use
    uint32_t ep_ranks = 0;
    uint32_t* ep_counts = nullptr;       // [n_ranks + 1] rows per destination rank, then their sum
    uint32_t* ep_counts_host = nullptr;  // pinned mirror
    uint32_t* ep_send_tok = nullptr;     // [max_tokens * min(n_ranks, n_used)]
    uint32_t* ep_send_pos = nullptr;     // [max_tokens][n_ranks]
    // peer-memory form of the exchange: this rank's receive buffers and every rank's as mapped here
    uint32_t pm_ranks = 0, pm_rank = 0, pm_cap = 0;   // slot_cap rows per source rank
    uint32_t pm_epoch = 0;                            // barriers issued so far (qkm_ep_barrier)
    bool pm_shared_in_partial = false;                // the last qkm_ep_forward_slots included the shared expert
    bool pm_rows_f16 = false;                         // the last qkm_ep_push sent f16 rows (layers on the tensor-core path)
    float* pm_xrecv = nullptr; qkm_sel* pm_selrecv = nullptr; float* pm_back = nullptr;   // mapped by the peers
    float* pm_partial = nullptr;                      // local partial rows where the fold does not store to the peers
    float* pm_xscale = nullptr;                       // [slot_cap] scales of the local rows sent as f16 (small batches)
    EpPeerTable pm_peers{};
    void* pm_opened[kMaxPeerRanks][3] = {};           // mappings this context opened from handles
    // the shared expert's kernels run on a side stream, beside the routing/grouping kernels
    cudaStream_t side = nullptr;
    cudaEvent_t ev_fork = nullptr, ev_join = nullptr, ev_planes = nullptr;
    // the decode stack as CUDA graphs: captured on first use of an argument set, a few sets kept
    // (the host-buffer form runs the stack in chunks of layers, each its own graph)
    static constexpr int kStackGraphs = 8;
    struct StackGraph {
        cudaGraphExec_t exec = nullptr;
        uint32_t first = 0, count = 0, n = 0;
        const float* x = nullptr;
        float* y = nullptr;
        cudaStream_t stream = nullptr;
        uint64_t launches = 0;       // kernels one replay launches
        uint32_t plan_after = 0;     // shared_plan_n once the sequence has run
        uint64_t used = 0;           // for least-recently-used replacement
    } stack_graphs[kStackGraphs];
    uint64_t stack_clock = 0;
    // the host-buffer form of the stack copies chunk k+1 in and chunk k-1 out while chunk k computes
    static constexpr int kStackChunks = 4;
    cudaStream_t copy_in = nullptr, copy_out = nullptr;
    cudaEvent_t ev_in[kStackChunks] = {}, ev_out[kStackChunks] = {}, ev_copies = nullptr;
    void drop_stack_graphs() {
        for (auto& g : stack_graphs) if (g.exec) { cudaGraphExecDestroy(g.exec); g.exec = nullptr; }
    }
    // per-stage profiling of the fused calls
    static constexpr int kMaxStages = 16;
    bool profiling = false;
    cudaEvent_t prof_ev[kMaxStages + 1] = {};
    char prof_label[kMaxStages][16] = {};
    int prof_n = 0;
    void prof_begin() {
        prof_n = 0;
        if (profiling) cudaEventRecord(prof_ev[0], stream);
    }
    void prof_mark(const char* label) {
        if (!profiling || prof_n >= kMaxStages) return;
        snprintf(prof_label[prof_n], 16, "%s", label);
        cudaEventRecord(prof_ev[++prof_n], stream);
    }
    Launch L() { return Launch{stream, &launches}; }
    // decode chain (logits -> selection -> gate/up -> down -> next layer's logits): each kernel is
    // launched as a programmatic dependent of the one before, so its scheduling and set-up overlap
    // that kernel's tail.  Off unless QKM_PDL=1 is in the environment when the context is opened:
    // inside the captured decode graph the kernels already follow one another without a gap, and the
    // persistent blocks leave an early block no room on an SM, so it measured no gain (75.5 us per
    // layer at 16 slots either way).
    bool use_pdl = false;
    Launch Lchain() { return Launch{stream, &launches, use_pdl && !profiling}; }
};

namespace {

int fail(qkm_ctx* c, int code, const char* fmt, ...) {
    if (c) {
        va_list ap;
        va_start(ap, fmt);
        vsnprintf(c->err, sizeof c->err, fmt, ap);
        va_end(ap);
    }
    return code;
}

#define QKM_CUDA(c, call)                                                                       \
    do {                                                                                        \
        cudaError_t e_ = (call);                                                                \
        if (e_ != cudaSuccess)                                                                  \
            return fail((c), QKM_ERR_CUDA, "%s failed: %s (%s:%d)", #call, cudaGetErrorString(e_), \
                        __FILE__, __LINE__);                                                    \
    } while (0)

bool dims_ok(const qkm_dims& d) {
    // limits the reference enforces: src/main.cpp:955, :1298, :3620-3621
    return d.n_embd >= 256 && d.n_embd % 256 == 0 && d.n_ff >= 256 && d.n_ff % 256 == 0 &&
           d.n_expert >= 1 && d.n_expert <= 512 && d.n_used >= 1 && d.n_used <= 16 &&
           d.n_used <= d.n_expert;
}

size_t tensor_bytes(const qkm_ctx* c, int idx, const qkm_layer_weights& w) {
    const qkm_dims& d = c->cfg.dims;
    const size_t ne = c->ecount;
    switch (idx) {
        case 0: return (size_t)d.n_expert * row_bytes(w.router_type, d.n_embd);
        case 1: return (size_t)d.n_embd * 4;
        case 2: case 3: return ne * d.n_ff * row_bytes(w.gateup_type, d.n_embd);
        case 4: return ne * d.n_embd * row_bytes(w.down_type, d.n_ff);
        case 5: case 6: return (size_t)d.n_ff * row_bytes(QKM_TYPE_Q8_0, d.n_embd);
        case 7: return (size_t)d.n_embd * row_bytes(QKM_TYPE_Q8_0, d.n_ff);
    }
    return 0;
}

int check_tokens(qkm_ctx* c, uint32_t n) {
    if (!c) return QKM_ERR_ARG;
    if (n > c->cfg.max_tokens) return fail(c, QKM_ERR_BOUNDS, "n_tokens %u exceeds max_tokens %u", n, c->cfg.max_tokens);
    return QKM_OK;
}

int layer_ready(qkm_ctx* c, uint32_t layer) {
    if (!c) return QKM_ERR_ARG;
    if (layer >= c->cfg.n_layer) return fail(c, QKM_ERR_BOUNDS, "layer %u out of range (n_layer %u)", layer, c->cfg.n_layer);
    if (!c->layers[layer].uploaded) return fail(c, QKM_ERR_BUSY, "layer %u has no weights uploaded", layer);
    return QKM_OK;
}

}  // namespace

// ---------------------------------------------------------------- lifecycle

extern "C" QKM_API const char* qkm_version(void) { return "qk-moe-b200 0.1 (sm_100a)"; }

extern "C" QKM_API qkm_ctx* qkm_open(const qkm_config* cfg, char* err, size_t err_len) {
    auto bail = [&](const char* msg, const char* detail) -> qkm_ctx* {
        if (err && err_len) snprintf(err, err_len, "%s%s%s", msg, detail ? ": " : "", detail ? detail : "");
        return nullptr;
    };
    if (!cfg) return bail("qkm_open: NULL config", nullptr);
    if (!dims_ok(cfg->dims)) return bail("qkm_open: unsupported dims (n_embd,n_ff multiples of 256; n_expert<=512; n_used<=16)", nullptr);
    if (cfg->n_layer < 1 || cfg->max_tokens < 1) return bail("qkm_open: n_layer and max_tokens must be >= 1", nullptr);
    if (cfg->max_tokens >= (1u << 28)) return bail("qkm_open: max_tokens too large for the pair encoding", nullptr);
    uint32_t efirst = cfg->expert_first, ecount = cfg->expert_count;
    if (ecount == 0) { efirst = 0; ecount = cfg->dims.n_expert; }
    if ((uint64_t)efirst + ecount > cfg->dims.n_expert) return bail("qkm_open: expert range exceeds n_expert", nullptr);

    int ndev = 0;
    cudaError_t e = cudaGetDeviceCount(&ndev);
    if (e != cudaSuccess || ndev == 0) return bail("qkm_open: no CUDA device (this library has no CPU path)", cudaGetErrorString(e));
    int dev = cfg->device;
    if (dev < 0) { if (cudaGetDevice(&dev) != cudaSuccess) dev = 0; }
    if (dev >= ndev) return bail("qkm_open: device ordinal out of range", nullptr);
    if ((e = cudaSetDevice(dev)) != cudaSuccess) return bail("qkm_open: cudaSetDevice", cudaGetErrorString(e));
    cudaDeviceProp prop{};
    if ((e = cudaGetDeviceProperties(&prop, dev)) != cudaSuccess) return bail("qkm_open: cudaGetDeviceProperties", cudaGetErrorString(e));
    if (prop.major != 10) return bail("qkm_open: kernels are built for sm_100a only; device is", prop.name);

    qkm_ctx* c = new (std::nothrow) qkm_ctx();
    if (!c) return bail("qkm_open: out of host memory", nullptr);
    c->cfg = *cfg;
    c->device = dev;
    if (const char* v = getenv("QKM_PDL")) c->use_pdl = v[0] == '1';
    c->efirst = efirst;
    c->ecount = ecount;
    c->layers.resize(cfg->n_layer);
    const qkm_dims& d = cfg->dims;
    const size_t T = cfg->max_tokens;
    c->route_scratch_bytes = qkm::route_scratch_bytes((uint32_t)T, d.n_expert);
    struct { void** p; size_t bytes; } allocs[] = {
        {(void**)&c->sel, T * sizeof(qkm_sel)},
        {(void**)&c->h, T * (d.n_used + 1) * d.n_ff * sizeof(float)},
        {(void**)&c->route_scratch, qkm::route_scratch_bytes((uint32_t)T, d.n_expert)},
        {(void**)&c->offsets, (d.n_expert + 1) * sizeof(uint32_t)},
        {(void**)&c->pairs, T * (d.n_used + 1) * sizeof(uint32_t)},
        {(void**)&c->y2, T * d.n_embd * sizeof(float)},
        {(void**)&c->x_stage, T * d.n_embd * sizeof(float)},
        {(void**)&c->y_stage, T * d.n_embd * sizeof(float)},
    };
    for (auto& a : allocs) {
        if ((e = cudaMalloc(a.p, a.bytes)) != cudaSuccess) {
            bail("qkm_open: cudaMalloc of scratch", cudaGetErrorString(e));
            qkm_close(c);
            return nullptr;
        }
    }
    c->n_sms = prop.multiProcessorCount;
    // Streaming kernels: column blocks per row must be a power of two in [2,16] (one warp
    // each) and rows must split into whole items.  (The fused decode / prefill sequences
    // also need every expert resident; a sharded context uses the tiles through qkm_ep_*.)
    auto pow2_2_16 = [](uint32_t v) { return v >= 2 && v <= 16 && (v & (v - 1)) == 0; };
    c->shapes_stream_ok = pow2_2_16(d.n_embd / 256) && d.n_embd / 256 <= 8 && pow2_2_16(d.n_ff / 256) && d.n_used <= 15 &&
                          d.n_ff % gateup_stream_rows_per_item() == 0 &&
                          d.n_embd % down_stream_rows_per_item() == 0;
    if (c->shapes_stream_ok) {
        const size_t max_groups = (T * d.n_used + 1) / 2 + d.n_expert;  // token pairs per expert, rounded up
        const size_t sh_groups = (T + 1) / 2;
        const size_t chunks_gu = d.n_ff / gateup_stream_rows_per_item(), chunks_dn = d.n_embd / down_stream_rows_per_item();
        struct { void** p; size_t bytes; } more[] = {
            {(void**)&c->xplanes, T * 4 * d.n_embd},
            {(void**)&c->xscale, T * sizeof(float)},
            {(void**)&c->hpieces, T * (d.n_used + 1) * 3 * d.n_ff * 2},
            {(void**)&c->items_gu, max_groups * chunks_gu * sizeof(StreamItem)},
            {(void**)&c->items_dn, max_groups * chunks_dn * sizeof(StreamItem)},
            {(void**)&c->items_sh_gu, sh_groups * chunks_gu * sizeof(StreamItem)},
            {(void**)&c->items_sh_dn, sh_groups * chunks_dn * sizeof(StreamItem)},
            {(void**)&c->n_items, 4 * sizeof(uint32_t)},
            {(void**)&c->contrib_s, T * (d.n_used + 1) * d.n_embd * sizeof(float)},
            {(void**)&c->arrivals, T * (d.n_embd / down_stream_unit_rows()) * sizeof(uint32_t)},
        };
        for (auto& a : more) {
            if ((e = cudaMalloc(a.p, a.bytes)) != cudaSuccess) {
                bail("qkm_open: cudaMalloc of streaming scratch", cudaGetErrorString(e));
                qkm_close(c);
                return nullptr;
            }
        }
        cudaMemset(c->arrivals, 0, T * (d.n_embd / down_stream_unit_rows()) * sizeof(uint32_t));
        c->dec_ok = decode_gateup_ok(d) && d.n_embd <= 4096;
        if (c->dec_ok) {
            struct { void** p; size_t bytes; } dec[] = {
                {(void**)&c->planes8, T * 8 * d.n_embd},
                {(void**)&c->lut_gu, decode_gateup_lut_bytes()},
                {(void**)&c->lut_dd, decode_down_lut_bytes()},
            };
            for (auto& a : dec) {
                if ((e = cudaMalloc(a.p, a.bytes)) != cudaSuccess) {
                    bail("qkm_open: cudaMalloc of decode scratch", cudaGetErrorString(e));
                    qkm_close(c);
                    return nullptr;
                }
            }
            const Launch L0{nullptr, nullptr};
            if ((e = launch_decode_gateup_luts(L0, c->lut_gu)) != cudaSuccess ||
                (e = launch_decode_down_lut(L0, c->lut_dd)) != cudaSuccess ||
                (e = cudaDeviceSynchronize()) != cudaSuccess) {
                bail("qkm_open: decode tables", cudaGetErrorString(e));
                qkm_close(c);
                return nullptr;
            }
        }
    }
    if ((e = cudaMalloc((void**)&c->status, sizeof(uint32_t))) != cudaSuccess ||
        (e = cudaMemset(c->status, 0, sizeof(uint32_t))) != cudaSuccess ||
        (e = cudaMalloc((void**)&c->route_counter, 16 * sizeof(uint32_t))) != cudaSuccess ||
        (e = cudaMemset(c->route_counter, 0, 16 * sizeof(uint32_t))) != cudaSuccess ||
        (e = cudaMallocHost((void**)&c->status_host, sizeof(uint32_t))) != cudaSuccess) {
        bail("qkm_open: status word", cudaGetErrorString(e));
        qkm_close(c);
        return nullptr;
    }
    *c->status_host = 0;
    {
        const Launch L0{nullptr, nullptr};
        if ((e = cudaMalloc((void**)&c->lut_pf, gateup_iq3_table_bytes())) != cudaSuccess ||
            (e = launch_gateup_iq3_table(L0, c->lut_pf)) != cudaSuccess ||
            (e = cudaMalloc((void**)&c->lut_dn, down_iq4_table_bytes())) != cudaSuccess ||
            (e = launch_down_iq4_table(L0, c->lut_dn)) != cudaSuccess || (e = cudaDeviceSynchronize()) != cudaSuccess) {
            bail("qkm_open: prefill tables", cudaGetErrorString(e));
            qkm_close(c);
            return nullptr;
        }
    }
    if (cudaStreamCreateWithFlags(&c->side, cudaStreamNonBlocking) != cudaSuccess ||
        cudaEventCreateWithFlags(&c->ev_fork, cudaEventDisableTiming) != cudaSuccess ||
        cudaEventCreateWithFlags(&c->ev_join, cudaEventDisableTiming) != cudaSuccess ||
        cudaEventCreateWithFlags(&c->ev_planes, cudaEventDisableTiming) != cudaSuccess) {
        bail("qkm_open: side stream", nullptr);
        qkm_close(c);
        return nullptr;
    }
    if (err && err_len) err[0] = 0;
    return c;
}

extern "C" QKM_API void qkm_close(qkm_ctx* c) {
    if (!c) return;
    cudaSetDevice(c->device);
    cudaDeviceSynchronize();
    for (auto& l : c->layers) {
        for (void* p : l.allocs) if (p) cudaFree(p);
        for (void* p : l.tiles) if (p) cudaFree(p);
    }
    for (auto& dm : c->dense) if (dm.tiles) cudaFree(dm.tiles);
    void* scratch[] = {c->argmax_scratch, c->dense_xb, c->dense_pairs, c->dense_sel, c->dense_items, c->dense_n_items, c->sel, c->h, c->route_scratch, c->offsets, c->pairs, c->contrib, c->y2, c->x_stage, c->y_stage,
                       c->stack_x, c->stack_y, c->xplanes, c->xscale, c->hpieces, c->items_gu, c->items_dn,
                       c->items_sh_gu, c->items_sh_dn, c->n_items, c->contrib_s, c->arrivals, c->status, c->route_counter,
                       c->planes8, c->lut_gu, c->lut_dd, c->lut_pf, c->lut_dn,
                       c->xb, c->hb, c->hscale, c->contrib_p, c->mma_items[0], c->mma_items[1], c->mma_items[2], c->mma_items[3],
                       c->pos_of, c->group_hist, c->ep_counts, c->ep_send_tok, c->ep_send_pos};
    for (void* p : scratch) if (p) cudaFree(p);
    for (auto& o : c->pm_opened) for (void* p : o) if (p) cudaIpcCloseMemHandle(p);
    for (void* p : {(void*)c->pm_xrecv, (void*)c->pm_selrecv, (void*)c->pm_back, (void*)c->pm_partial, (void*)c->pm_xscale}) if (p) cudaFree(p);
    if (c->status_host) cudaFreeHost(c->status_host);
    if (c->ep_counts_host) cudaFreeHost(c->ep_counts_host);
    c->drop_stack_graphs();
    for (cudaEvent_t ev : c->ev_in) if (ev) cudaEventDestroy(ev);
    for (cudaEvent_t ev : c->ev_out) if (ev) cudaEventDestroy(ev);
    if (c->ev_copies) cudaEventDestroy(c->ev_copies);
    if (c->copy_in) cudaStreamDestroy(c->copy_in);
    if (c->copy_out) cudaStreamDestroy(c->copy_out);
    if (c->ev_fork) cudaEventDestroy(c->ev_fork);
    if (c->ev_join) cudaEventDestroy(c->ev_join);
    if (c->ev_planes) cudaEventDestroy(c->ev_planes);
    if (c->side) cudaStreamDestroy(c->side);
    for (cudaEvent_t ev : c->prof_ev) if (ev) cudaEventDestroy(ev);
    delete c;
}

extern "C" QKM_API const char* qkm_last_error(const qkm_ctx* c) { return c ? c->err : "NULL context"; }
extern "C" QKM_API uint32_t qkm_n_embd(const qkm_ctx* c) { return c ? c->cfg.dims.n_embd : 0; }
extern "C" QKM_API uint32_t qkm_n_ff(const qkm_ctx* c) { return c ? c->cfg.dims.n_ff : 0; }
extern "C" QKM_API uint32_t qkm_n_expert(const qkm_ctx* c) { return c ? c->cfg.dims.n_expert : 0; }
extern "C" QKM_API uint32_t qkm_n_used(const qkm_ctx* c) { return c ? c->cfg.dims.n_used : 0; }
extern "C" QKM_API uint32_t qkm_n_layer(const qkm_ctx* c) { return c ? c->cfg.n_layer : 0; }
extern "C" QKM_API uint32_t qkm_max_tokens(const qkm_ctx* c) { return c ? c->cfg.max_tokens : 0; }
extern "C" QKM_API void qkm_expert_range(const qkm_ctx* c, uint32_t* first, uint32_t* count) {
    if (first) *first = c ? c->efirst : 0;
    if (count) *count = c ? c->ecount : 0;
}
extern "C" QKM_API size_t qkm_row_bytes(uint32_t type, uint64_t ne0) {
    const uint32_t be = block_elems(type);
    if (be == 0 || ne0 % be) return 0;
    return row_bytes(type, ne0);
}

extern "C" QKM_API int qkm_set_stream(qkm_ctx* c, void* s) {
    if (!c) return QKM_ERR_ARG;
    c->stream = (cudaStream_t)s;
    return QKM_OK;
}
// Copies the kernels' status word back after a synchronise; a bounded device-side wait
// that gave up (or a broken layout assumption) surfaces here as an error code.
static int check_status(qkm_ctx* c) {
    QKM_CUDA(c, cudaMemcpyAsync(c->status_host, c->status, sizeof(uint32_t), cudaMemcpyDeviceToHost, c->stream));
    QKM_CUDA(c, cudaStreamSynchronize(c->stream));
    if (*c->status_host != 0) {
        const uint32_t st = *c->status_host;
        cudaMemsetAsync(c->status, 0, sizeof(uint32_t), c->stream);
        return fail(c, QKM_ERR_TIMEOUT, "a kernel reported status %u (1 = bounded wait gave up, 2 = shared-memory layout)", st);
    }
    return QKM_OK;
}

extern "C" QKM_API int qkm_sync(qkm_ctx* c) {
    if (!c) return QKM_ERR_ARG;
    return check_status(c);
}
extern "C" QKM_API uint64_t qkm_launch_count(const qkm_ctx* c) { return c ? c->launches : 0; }

extern "C" QKM_API void* qkm_dev_alloc(qkm_ctx* c, size_t bytes) {
    if (!c) return nullptr;
    void* p = nullptr;
    cudaSetDevice(c->device);
    cudaError_t e = cudaMalloc(&p, bytes ? bytes : 1);
    if (e != cudaSuccess) { fail(c, QKM_ERR_CUDA, "cudaMalloc(%zu): %s", bytes, cudaGetErrorString(e)); return nullptr; }
    return p;
}
extern "C" QKM_API int qkm_dev_free(qkm_ctx* c, void* p) {
    if (!c) return QKM_ERR_ARG;
    QKM_CUDA(c, cudaFree(p));
    return QKM_OK;
}
extern "C" QKM_API int qkm_h2d(qkm_ctx* c, void* dst, const void* src, size_t bytes) {
    if (!c || (!dst && bytes) || (!src && bytes)) return QKM_ERR_ARG;
    QKM_CUDA(c, cudaMemcpyAsync(dst, src, bytes, cudaMemcpyHostToDevice, c->stream));
    QKM_CUDA(c, cudaStreamSynchronize(c->stream));
    return QKM_OK;
}
extern "C" QKM_API int qkm_d2h(qkm_ctx* c, void* dst, const void* src, size_t bytes) {
    if (!c || (!dst && bytes) || (!src && bytes)) return QKM_ERR_ARG;
    QKM_CUDA(c, cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToHost, c->stream));
    QKM_CUDA(c, cudaStreamSynchronize(c->stream));
    return QKM_OK;
}

// ---------------------------------------------------------------- weights

extern "C" QKM_API int qkm_upload_layer(qkm_ctx* c, uint32_t layer, const qkm_layer_weights* w) {
    if (!c || !w) return QKM_ERR_ARG;
    if (layer >= c->cfg.n_layer) return fail(c, QKM_ERR_BOUNDS, "layer %u out of range", layer);
    // the types loadMoeT accepts (src/main.cpp:1283-1291), plus an F16 router
    if (w->router_type != QKM_TYPE_F32 && w->router_type != QKM_TYPE_F16)
        return fail(c, QKM_ERR_TYPE, "router type %u unsupported (F32 or F16)", w->router_type);
    if (w->gateup_type != QKM_TYPE_IQ3_XXS && w->gateup_type != QKM_TYPE_IQ4_XS)
        return fail(c, QKM_ERR_TYPE, "gate/up type %u unsupported (IQ3_XXS or IQ4_XS)", w->gateup_type);
    if (w->down_type != QKM_TYPE_IQ4_XS && w->down_type != QKM_TYPE_Q6_K)
        return fail(c, QKM_ERR_TYPE, "down type %u unsupported (IQ4_XS or Q6_K)", w->down_type);
    const void* src[8] = {w->router, w->gate_inp_shexp, w->gate_exps, w->up_exps, w->down_exps,
                          w->gate_shexp, w->up_shexp, w->down_shexp};
    for (const void* p : src) if (!p) return fail(c, QKM_ERR_ARG, "layer %u: NULL tensor pointer", layer);
    QKM_CUDA(c, cudaSetDevice(c->device));
    c->drop_stack_graphs();
    qkm_layer_dev& l = c->layers[layer];
    for (int i = 0; i < 8; ++i) {
        const size_t bytes = tensor_bytes(c, i, *w);
        if (l.allocs[i]) { QKM_CUDA(c, cudaFree(l.allocs[i])); l.allocs[i] = nullptr; }
        // 256 spare bytes: streaming kernels may read a few bytes past a tensor's end
        QKM_CUDA(c, cudaMalloc(&l.allocs[i], bytes + 256));
        QKM_CUDA(c, cudaMemcpyAsync(l.allocs[i], src[i], bytes, cudaMemcpyHostToDevice, c->stream));
        QKM_CUDA(c, cudaMemsetAsync((uint8_t*)l.allocs[i] + bytes, 0, 256, c->stream));
    }
    // tile-ordered copies for the streaming kernels (same bytes, re-ordered on the device)
    for (void*& p : l.tiles) { if (p) { QKM_CUDA(c, cudaFree(p)); p = nullptr; } }
    l.stream_ok = l.tiles_ok = l.gu_only = l.fused_ok = false;
    if (c->shapes_stream_ok) {
        const qkm_dims& d = c->cfg.dims;
        struct { int idx; uint32_t type, mats, rows, K; } plan[] = {
            {2, w->gateup_type, c->ecount, d.n_ff, d.n_embd}, {3, w->gateup_type, c->ecount, d.n_ff, d.n_embd},
            {4, w->down_type, c->ecount, d.n_embd, d.n_ff},
            {5, QKM_TYPE_Q8_0, 1, d.n_ff, d.n_embd}, {6, QKM_TYPE_Q8_0, 1, d.n_ff, d.n_embd},
            {7, QKM_TYPE_Q8_0, 1, d.n_embd, d.n_ff},
        };
        const bool gu = w->gateup_type == QKM_TYPE_IQ3_XXS, dn = w->down_type == QKM_TYPE_IQ4_XS;
        for (auto& t : plan) {
            const size_t bytes = tensor_bytes(c, t.idx, *w);
            QKM_CUDA(c, cudaMalloc(&l.tiles[t.idx], bytes + 256));
            cudaError_t e = launch_repack(c->L(), t.type, l.allocs[t.idx], l.tiles[t.idx], t.mats, t.rows, t.K);
            if (e != cudaSuccess) return fail(c, QKM_ERR_CUDA, "repack: %s", cudaGetErrorString(e));
        }
        const bool all_resident = c->ecount == c->cfg.dims.n_expert;
        l.tiles_ok = gu && dn;
        l.stream_ok = gu && dn && all_resident;
        l.gu_only = gu && !dn && all_resident;
        l.fused_ok = all_resident;
    }
    QKM_CUDA(c, cudaStreamSynchronize(c->stream));
    l.w = *w;
    l.w.router = l.allocs[0];
    l.w.gate_inp_shexp = (const float*)l.allocs[1];
    l.w.gate_exps = l.allocs[2];
    l.w.up_exps = l.allocs[3];
    l.w.down_exps = l.allocs[4];
    l.w.gate_shexp = l.allocs[5];
    l.w.up_shexp = l.allocs[6];
    l.w.down_shexp = l.allocs[7];
    l.uploaded = true;
    return QKM_OK;
}

extern "C" QKM_API int qkm_layer_device_ptrs(const qkm_ctx* c, uint32_t layer, qkm_layer_weights* out) {
    if (!c || !out) return QKM_ERR_ARG;
    if (layer >= c->cfg.n_layer) return QKM_ERR_BOUNDS;
    if (!c->layers[layer].uploaded) return QKM_ERR_BUSY;
    *out = c->layers[layer].w;
    return QKM_OK;
}

// ---------------------------------------------------------------- op-level entry points

#define QKM_LAUNCH(c, call)                                                                          \
    do {                                                                                             \
        cudaError_t e_ = (call);                                                                     \
        if (e_ == cudaErrorInvalidValue) return fail((c), QKM_ERR_TYPE, "%s: unsupported type or shape", #call); \
        if (e_ != cudaSuccess) return fail((c), QKM_ERR_CUDA, "%s: %s", #call, cudaGetErrorString(e_)); \
    } while (0)

extern "C" QKM_API int qkm_moe_logits(qkm_ctx* c, uint32_t router_type, const void* router, const float* x,
                                      float* logits, uint32_t n) {
    if (!c || !router || !x || !logits) return QKM_ERR_ARG;
    QKM_LAUNCH(c, launch_logits(c->L(), c->cfg.dims, router_type, router, x, logits, nullptr, n));
    return QKM_OK;
}

extern "C" QKM_API int qkm_moe_select(qkm_ctx* c, const float* logits, const float* gis, const float* x,
                                      qkm_sel* sel, uint32_t n) {
    if (!c || !logits || !gis || !x || !sel) return QKM_ERR_ARG;
    QKM_LAUNCH(c, launch_select(c->L(), c->cfg.dims, logits, gis, x, sel, n));
    return QKM_OK;
}

extern "C" QKM_API int qkm_moe_route_select(qkm_ctx* c, uint32_t router_type, const void* router,
                                            const float* gis, const float* x, qkm_sel* sel, uint32_t n) {
    if (!c || !router || !gis || !x || !sel) return QKM_ERR_ARG;
    if (int rc = check_tokens(c, n)) return rc;
    if (router_type != QKM_TYPE_F32 && router_type != QKM_TYPE_F16) return fail(c, QKM_ERR_TYPE, "router type %u", router_type);
    QKM_LAUNCH(c, launch_route_select(c->L(), c->cfg.dims, router_type, router, gis, x, sel, n, c->route_scratch, c->route_scratch_bytes));
    return QKM_OK;
}

extern "C" QKM_API int qkm_moe_group_pairs(qkm_ctx* c, const qkm_sel* sel, uint32_t n, uint32_t* offsets,
                                           uint32_t* pairs) {
    if (!c || !sel || !offsets || !pairs) return QKM_ERR_ARG;
    QKM_LAUNCH(c, launch_group_pairs(c->L(), c->cfg.dims, sel, n, offsets, pairs, c->efirst, c->ecount));
    return QKM_OK;
}

extern "C" QKM_API int qkm_moe_gateup(qkm_ctx* c, uint32_t type, const void* gate, const void* up,
                                      const float* x, const qkm_sel* sel, float* h, uint32_t n) {
    if (!c || !gate || !up || !x || !sel || !h) return QKM_ERR_ARG;
    QKM_LAUNCH(c, launch_gateup_tokens(c->L(), c->cfg.dims, type, gate, up, x, sel, h, n, c->efirst, c->ecount));
    return QKM_OK;
}

extern "C" QKM_API int qkm_moe_gateup_grouped(qkm_ctx* c, uint32_t type, const void* gate, const void* up,
                                              const float* x, const uint32_t* offsets, const uint32_t* pairs,
                                              float* h, uint32_t n) {
    if (!c || !gate || !up || !x || !offsets || !pairs || !h) return QKM_ERR_ARG;
    QKM_LAUNCH(c, launch_gateup_pairs(c->L(), c->cfg.dims, type, gate, up, x, offsets, pairs, h, n, c->efirst, c->ecount));
    return QKM_OK;
}

extern "C" QKM_API int qkm_moe_shared_gateup(qkm_ctx* c, const void* gate, const void* up, const float* x,
                                             float* h, uint32_t n) {
    if (!c || !gate || !up || !x || !h) return QKM_ERR_ARG;
    QKM_LAUNCH(c, launch_shared_gateup(c->L(), c->cfg.dims, gate, up, x, h, n));
    return QKM_OK;
}

extern "C" QKM_API int qkm_moe_down(qkm_ctx* c, uint32_t type, const void* down, const float* h,
                                    const qkm_sel* sel, float* y, uint32_t n) {
    if (!c || !down || !h || !sel || !y) return QKM_ERR_ARG;
    QKM_LAUNCH(c, launch_down_tokens(c->L(), c->cfg.dims, type, down, h, sel, y, n, c->efirst, c->ecount, nullptr));
    return QKM_OK;
}

extern "C" QKM_API int qkm_moe_down_grouped(qkm_ctx* c, uint32_t type, const void* down, const float* h,
                                            const qkm_sel* sel, const uint32_t* offsets, const uint32_t* pairs,
                                            float* contrib, uint32_t n) {
    if (!c || !down || !h || !sel || !offsets || !pairs || !contrib) return QKM_ERR_ARG;
    QKM_LAUNCH(c, launch_down_pairs(c->L(), c->cfg.dims, type, down, h, sel, offsets, pairs, contrib, n, c->efirst, c->ecount));
    return QKM_OK;
}

extern "C" QKM_API int qkm_moe_shared_down(qkm_ctx* c, const void* down, const float* h, const qkm_sel* sel,
                                           float* y2, uint32_t n) {
    if (!c || !down || !h || !sel || !y2) return QKM_ERR_ARG;
    QKM_LAUNCH(c, launch_shared_down(c->L(), c->cfg.dims, down, h, sel, y2, n));
    return QKM_OK;
}

extern "C" QKM_API int qkm_gemv(qkm_ctx* c, uint32_t type, const void* W, const float* x, float* y,
                                uint32_t M, uint32_t K, uint32_t n) {
    if (!c || !W || !x || !y) return QKM_ERR_ARG;
    const uint32_t be = block_elems(type);
    if (be == 0) return fail(c, QKM_ERR_TYPE, "qkm_gemv: type %u unsupported", type);
    if (K == 0 || K % be || K % 8) return fail(c, QKM_ERR_ARG, "qkm_gemv: K=%u must be a multiple of the block size %u and of 8", K, be);
    if (n > 65535) return fail(c, QKM_ERR_BOUNDS, "qkm_gemv: n=%u exceeds 65535", n);
    QKM_LAUNCH(c, launch_gemv_stream(c->L(), type, W, x, y, M, K, n, (uint32_t)c->n_sms, c->status));
    return QKM_OK;
}

extern "C" QKM_API int qkm_dequant(qkm_ctx* c, uint32_t type, const void* blocks, float* y, uint64_t n_elems) {
    if (!c || !blocks || !y) return QKM_ERR_ARG;
    const uint32_t be = block_elems(type);
    if (be == 0) return fail(c, QKM_ERR_TYPE, "qkm_dequant: type %u unsupported", type);
    if (n_elems % be || n_elems % 8) return fail(c, QKM_ERR_ARG, "qkm_dequant: n_elems must be whole blocks and a multiple of 8");
    QKM_LAUNCH(c, launch_dequant(c->L(), type, blocks, y, n_elems));
    return QKM_OK;
}

// ---------------------------------------------------------------- fused layer calls

extern "C" QKM_API int qkm_moe_decode(qkm_ctx* c, uint32_t layer, const float* x, uint32_t n, float* y) {
    if (int rc = layer_ready(c, layer)) return rc;
    if (!x || !y) return QKM_ERR_ARG;
    if (int rc = check_tokens(c, n)) return rc;
    const qkm_layer_dev& ld = c->layers[layer];
    const qkm_layer_weights& w = ld.w;
    const qkm_dims& d = c->cfg.dims;
    c->prof_begin();
    const bool fused = ld.fused_ok && c->dec_ok && route_decode_ok(d, n, c->route_scratch_bytes) && decode_down_ok(d);
    if (!fused && !ld.stream_ok && !ld.gu_only) {  // generic kernels on the raw layout
        QKM_LAUNCH(c, launch_route_select(c->L(), d, w.router_type, w.router, w.gate_inp_shexp, x, c->sel, n, c->route_scratch, c->route_scratch_bytes));
        c->prof_mark("moe.route");
        QKM_LAUNCH(c, launch_shared_gateup(c->L(), d, w.gate_shexp, w.up_shexp, x, c->h, n));
        c->prof_mark("moe.shared_gu");
        QKM_LAUNCH(c, launch_gateup_tokens(c->L(), d, w.gateup_type, w.gate_exps, w.up_exps, x, c->sel, c->h, n, c->efirst, c->ecount));
        c->prof_mark("moe.gu");
        QKM_LAUNCH(c, launch_down_tokens(c->L(), d, w.down_type, w.down_exps, c->h, c->sel, y, n, c->efirst, c->ecount, w.down_shexp));
        c->prof_mark("moe.dn");
        return QKM_OK;
    }
    const uint32_t nb = (uint32_t)c->n_sms;
    // Three launches for the whole layer: (1) router logits, selection and digit planes; (2) pair
    // grouping (in every block's shared memory), then gate/up + SwiGLU of the routed experts and of
    // the shared expert; (3) down
    // projections of both and the weighted sum.  The shared expert rides inside (2) and (3): no
    // side stream, and nothing runs beside the two persistent kernels that they would have to
    // share the SMs with.
    if (fused) {
        RouteDecodeArgs ra{};
        ra.router = (const uint8_t*)w.router; ra.gis = w.gate_inp_shexp; ra.x = x; ra.sel = c->sel;
        ra.logits = (double*)c->route_scratch; ra.counter = c->route_counter; ra.planes = c->planes8; ra.xscale = c->xscale; ra.n_tokens = n; ra.d = d;
        QKM_LAUNCH(c, launch_route_decode(c->Lchain(), w.router_type, ra));
        c->prof_mark("moe.route");
        GateupDecodeArgs ga{};
        ga.gate_tiles = (const uint8_t*)ld.tiles[2]; ga.up_tiles = (const uint8_t*)ld.tiles[3];
        ga.sh_gate_tiles = (const uint8_t*)ld.tiles[5]; ga.sh_up_tiles = (const uint8_t*)ld.tiles[6];
        ga.luts = c->lut_gu; ga.planes = c->planes8; ga.xscale = c->xscale; ga.sel = c->sel;
        ga.n_tokens = n; ga.expert_first = c->efirst; ga.expert_count = c->ecount; ga.with_shared = 1;
        ga.gateup_type = w.gateup_type;
        ga.h = c->h; ga.status = c->status; ga.d = d;
        QKM_LAUNCH(c, launch_decode_gateup(c->Lchain(), ga, nb));
        c->prof_mark("moe.gu");
        if (w.down_type == QKM_TYPE_IQ4_XS) {
            DownDecodeArgs da{};
            da.tiles = (const uint8_t*)ld.tiles[4]; da.sh_tiles = (const uint8_t*)ld.tiles[7]; da.lut = c->lut_dd;
            da.h = c->h; da.sel = c->sel; da.y = y; da.n_tokens = n; da.status = c->status; da.d = d;
            QKM_LAUNCH(c, launch_decode_down(c->Lchain(), da, nb));
        } else {   // Q6_K down
            DownDecodeArgs da{};
            da.tiles = (const uint8_t*)ld.tiles[4]; da.sh_tiles = (const uint8_t*)ld.tiles[7];
            da.h = c->h; da.sel = c->sel; da.y = y; da.n_tokens = n; da.status = c->status; da.d = d;
            QKM_LAUNCH(c, launch_decode_down_q6k(c->Lchain(), da, nb));
        }
        c->prof_mark("moe.dn");
        c->shared_plan_n = 0;   // pairs / work lists of the older sequence are overwritten
        return QKM_OK;
    }
    // Shared expert: depends on x only (as digit planes), so the whole of it - planes, gate/up,
    // down - runs on the side stream from the start of the layer, beside the router.  The main
    // stream needs the planes before the routed gate/up (ev_planes) and y2 before the routed
    // down kernel (ev_join).  (Sequential while profiling.)
    const bool fork = !c->profiling;
    Launch S{fork ? c->side : c->stream, &c->launches};
    if (fork) {
        QKM_CUDA(c, cudaEventRecord(c->ev_fork, c->stream));
        QKM_CUDA(c, cudaStreamWaitEvent(c->side, c->ev_fork, 0));
    }
    // the shared gate too, when the selection kernel will not touch it (same condition as below)
    const bool fused_plan = route_select_plans(d, n, c->route_scratch_bytes);
    QKM_LAUNCH(c, launch_xplanes(S, x, n, d.n_embd, c->xplanes, c->xscale, fused_plan ? w.gate_inp_shexp : nullptr, c->sel));
    if (fork) QKM_CUDA(c, cudaEventRecord(c->ev_planes, c->side));
    // the shared expert's work lists depend on the token count only and live in parts of the
    // scratch the decode kernels never write: cut once, reused until another kind of call intervenes
    if (c->shared_plan_n != n) {
        QKM_LAUNCH(c, launch_shared_plan(S, d, n, c->pairs, c->items_sh_gu, d.n_ff / gateup_stream_rows_per_item(),
                                         c->items_sh_dn, d.n_embd / down_stream_rows_per_item(), 2, c->n_items + 2));
        c->shared_plan_n = n;
    }
    QKM_LAUNCH(c, launch_gateup_stream(S, d, QKM_TYPE_Q8_0, ld.tiles[5], ld.tiles[6], c->xplanes, c->xscale, c->pairs,
                                       c->items_sh_gu, c->n_items + 2, c->h, c->hpieces, nb, c->status));
    if (!fork) c->prof_mark("moe.shared_gu");
    if (ld.stream_ok) {
        QKM_LAUNCH(c, launch_down_stream(S, d, QKM_TYPE_Q8_0, ld.tiles[7], c->hpieces, nullptr, c->pairs, c->items_sh_dn,
                                         c->n_items + 3, nullptr, c->y2, nullptr, nb, c->status));   // unweighted: w_shared is applied by the routed down kernel
        if (!fork) c->prof_mark("moe.shared_dn");
    }
    if (fork) QKM_CUDA(c, cudaEventRecord(c->ev_join, c->side));
    // Router.  Decode-sized batches: the selection kernel's last block also groups the pairs and
    // cuts the work lists; otherwise a grouping launch follows.
    const RoutePlan rplan{c->route_counter, c->offsets, c->pairs, c->items_gu, c->items_dn, c->n_items,
                          d.n_ff / gateup_stream_rows_per_item(), d.n_embd / down_stream_rows_per_item(), 2, c->efirst, c->ecount, 1};
    QKM_LAUNCH(c, launch_route_select(c->Lchain(), d, w.router_type, w.router, w.gate_inp_shexp, x, c->sel, n, c->route_scratch, c->route_scratch_bytes,
                                      nullptr, nullptr, nullptr, nullptr, nullptr, fused_plan ? &rplan : nullptr));
    c->prof_mark("moe.route");
    if (!fused_plan) {
        QKM_LAUNCH(c, launch_group_plan(c->L(), d, c->sel, n, c->offsets, c->pairs, c->efirst, c->ecount, c->items_gu,
                                        d.n_ff / gateup_stream_rows_per_item(), c->items_dn,
                                        d.n_embd / down_stream_rows_per_item(), nullptr, nullptr, 2, c->n_items));
        c->prof_mark("moe.pairs");
    }
    if (fork) QKM_CUDA(c, cudaStreamWaitEvent(c->stream, c->ev_planes, 0));
    QKM_LAUNCH(c, launch_gateup_stream(fused_plan ? c->Lchain() : c->L(), d, w.gateup_type, ld.tiles[2], ld.tiles[3], c->xplanes, c->xscale, c->pairs,
                                       c->items_gu, c->n_items, c->h, c->hpieces, nb, c->status));
    c->prof_mark("moe.gu");
    if (fork) QKM_CUDA(c, cudaStreamWaitEvent(c->stream, c->ev_join, 0));
    if (ld.stream_ok) {
        QKM_LAUNCH(c, launch_down_tok(c->Lchain(), d, w.down_type, ld.tiles[4], c->hpieces, c->sel, c->y2, y, n, nb, c->status));
    } else {   // Q6_K down: f32 kernel over h, routed slots and the shared expert in one pass
        QKM_LAUNCH(c, launch_down_tokens(c->L(), d, w.down_type, w.down_exps, c->h, c->sel, y, n, c->efirst, c->ecount, w.down_shexp));
    }
    c->prof_mark("moe.dn");
    return QKM_OK;
}

// Generic prefill sequence on the raw layout (any supported shape and type).
static int prefill_generic(qkm_ctx* c, const qkm_layer_dev& ld, const float* x, uint32_t n, float* y) {
    const qkm_layer_weights& w = ld.w;
    const qkm_dims& d = c->cfg.dims;
    if (!c->contrib) {
        QKM_CUDA(c, cudaMalloc((void**)&c->contrib, (size_t)c->cfg.max_tokens * d.n_used * d.n_embd * sizeof(float)));
    }
    QKM_LAUNCH(c, launch_route_select(c->L(), d, w.router_type, w.router, w.gate_inp_shexp, x, c->sel, n, c->route_scratch, c->route_scratch_bytes));
    QKM_LAUNCH(c, launch_group_pairs(c->L(), d, c->sel, n, c->offsets, c->pairs, c->efirst, c->ecount));
    QKM_LAUNCH(c, launch_shared_gateup(c->L(), d, w.gate_shexp, w.up_shexp, x, c->h, n));
    QKM_LAUNCH(c, launch_gateup_pairs(c->L(), d, w.gateup_type, w.gate_exps, w.up_exps, x, c->offsets, c->pairs, c->h, n, c->efirst, c->ecount));
    QKM_CUDA(c, cudaMemsetAsync(c->contrib, 0, (size_t)n * d.n_used * d.n_embd * sizeof(float), c->stream));
    QKM_LAUNCH(c, launch_down_pairs(c->L(), d, w.down_type, w.down_exps, c->h, c->sel, c->offsets, c->pairs, c->contrib, n, c->efirst, c->ecount));
    QKM_LAUNCH(c, launch_shared_down(c->L(), d, w.down_shexp, c->h, c->sel, c->y2, n));
    QKM_LAUNCH(c, launch_fold_contrib(c->L(), d, c->contrib, c->y2, y, n));
    return QKM_OK;
}

// Scratch of the tensor-core (tcgen05) sequences, allocated on first use.
static int ensure_prefill_scratch(qkm_ctx* c) {
    if (c->xb) return QKM_OK;
    const qkm_dims& d = c->cfg.dims;
    const size_t T = c->cfg.max_tokens, rows = T * (d.n_used + 1);
    const uint32_t NT = prefill_pairs_per_block();
    const uint32_t rt_gu = d.n_ff / 128, rt_dn = d.n_embd / 128;
    const size_t max_tiles = d.n_expert + (T * d.n_used + NT - 1) / NT, max_sh = (T + NT - 1) / NT;
    QKM_CUDA(c, cudaMalloc(&c->xb, T * d.n_embd * 2));
    QKM_CUDA(c, cudaMalloc(&c->hb, rows * d.n_ff * 2));
    QKM_CUDA(c, cudaMalloc((void**)&c->hscale, rows * sizeof(float)));
    QKM_CUDA(c, cudaMalloc((void**)&c->contrib_p, rows * d.n_embd * sizeof(float)));
    QKM_CUDA(c, cudaMalloc((void**)&c->mma_items[0], max_tiles * rt_gu * sizeof(MmaItem)));
    QKM_CUDA(c, cudaMalloc((void**)&c->mma_items[1], max_tiles * rt_dn * sizeof(MmaItem)));
    QKM_CUDA(c, cudaMalloc((void**)&c->mma_items[2], max_sh * rt_gu * sizeof(MmaItem)));
    QKM_CUDA(c, cudaMalloc((void**)&c->mma_items[3], max_sh * rt_dn * sizeof(MmaItem)));
    QKM_CUDA(c, cudaMalloc((void**)&c->pos_of, rows * sizeof(uint32_t)));
    QKM_CUDA(c, cudaMalloc((void**)&c->group_hist, group_wide_scratch_bytes((uint32_t)T, d.n_used, c->ecount)));
    return QKM_OK;
}

extern "C" QKM_API int qkm_moe_prefill(qkm_ctx* c, uint32_t layer, const float* x, uint32_t n, float* y) {
    if (int rc = layer_ready(c, layer)) return rc;
    if (!x || !y) return QKM_ERR_ARG;
    if (int rc = check_tokens(c, n)) return rc;
    const qkm_layer_dev& ld = c->layers[layer];
    const qkm_layer_weights& w = ld.w;
    const qkm_dims& d = c->cfg.dims;
    c->shared_plan_n = 0;   // this call rewrites the scratch the decode work lists live in
    if (!ld.fused_ok || n == 0) return prefill_generic(c, ld, x, n, y);
    // tensor-core path: tokens grouped by expert, expert GEMMs on tcgen05 with bf16 operands
    const uint32_t NT = prefill_pairs_per_block();
    const uint32_t rt_gu = d.n_ff / 128, rt_dn = d.n_embd / 128;
    if (int rc = ensure_prefill_scratch(c)) return rc;
    const uint32_t tiles_now = d.n_expert < n * d.n_used ? d.n_expert + (n * d.n_used + NT - 1) / NT : n * d.n_used;
    const uint32_t sh_now = (n + NT - 1) / NT;
    c->prof_begin();
    QKM_LAUNCH(c, launch_to_f16_rows(c->L(), x, c->xb, c->xscale, n, d.n_embd));
    QKM_LAUNCH(c, launch_route_select(c->L(), d, w.router_type, w.router, w.gate_inp_shexp, x, c->sel, n, c->route_scratch, c->route_scratch_bytes,
                                      nullptr, nullptr, c->xb, c->xscale, c->status));
    c->prof_mark("moe.route");
    QKM_LAUNCH(c, launch_group_pairs_wide(c->L(), d, c->sel, n, c->offsets, c->pairs, c->efirst, c->ecount, c->group_hist, c->pos_of));
    QKM_LAUNCH(c, launch_mma_plan(c->L(), d, c->offsets, c->pairs, c->ecount, n, c->mma_items[0], c->mma_items[1],
                                  c->mma_items[2], c->mma_items[3], c->n_items, c->pos_of, true, true));
    c->prof_mark("moe.pairs");
    // the shared expert's two GEMMs (few, long blocks) run beside the routed ones
    const bool fork = !c->profiling;
    Launch S{fork ? c->side : c->stream, &c->launches};
    if (fork) {
        QKM_CUDA(c, cudaEventRecord(c->ev_fork, c->stream));
        QKM_CUDA(c, cudaStreamWaitEvent(c->side, c->ev_fork, 0));
    }
    // Tensor-core down GEMMs take the hidden rows as f16 scaled per row by a power of two: the gate/up kernels
    // store them in f32 by pair position (in c->h), a conversion pass finds each row's scale.
    QKM_LAUNCH(c, launch_gateup_mma(S, d, QKM_TYPE_Q8_0, ld.tiles[5], ld.tiles[6], c->xb, c->xscale, c->pairs, c->mma_items[2],
                                    c->n_items + 2, sh_now * rt_gu, nullptr, c->hb, c->status, sh_now * rt_gu <= 2u * (uint32_t)c->n_sms, nullptr, c->h));
    if (!fork) c->prof_mark("moe.shared_gu");
    // the shared expert's rows follow the routed pairs (their number is offsets[ecount], known on the device)
    QKM_LAUNCH(c, launch_h_rows_to_f16(S, c->h, c->hb, c->hscale, d.n_ff, c->offsets + c->ecount, 0, nullptr, n));
    QKM_LAUNCH(c, launch_down_mma(S, d, QKM_TYPE_Q8_0, ld.tiles[7], c->hb, c->sel, c->pairs, c->mma_items[3],
                                  c->n_items + 3, sh_now * rt_dn, c->contrib_p, c->status, false, nullptr, c->hscale));
    if (!fork) c->prof_mark("moe.shared_dn");
    if (fork) QKM_CUDA(c, cudaEventRecord(c->ev_join, c->side));
    QKM_LAUNCH(c, launch_gateup_mma(c->L(), d, w.gateup_type, ld.tiles[2], ld.tiles[3], c->xb, c->xscale, c->pairs, c->mma_items[0],
                                    c->n_items, tiles_now * rt_gu, nullptr, c->hb, c->status, false, c->lut_pf, c->h));
    c->prof_mark("moe.gu");
    QKM_LAUNCH(c, launch_h_rows_to_f16(c->L(), c->h, c->hb, c->hscale, d.n_ff, nullptr, 0, c->offsets + c->ecount, n * d.n_used));
    QKM_LAUNCH(c, launch_down_mma(c->L(), d, w.down_type, ld.tiles[4], c->hb, c->sel, c->pairs, c->mma_items[1],
                                  c->n_items + 1, tiles_now * rt_dn, c->contrib_p, c->status, false, c->lut_dn, c->hscale));
    c->prof_mark("moe.dn");
    if (fork) QKM_CUDA(c, cudaStreamWaitEvent(c->stream, c->ev_join, 0));
    QKM_LAUNCH(c, launch_fold_pairs(c->L(), d, c->contrib_p, c->pos_of, y, n));
    c->prof_mark("moe.fold");
    return QKM_OK;
}

extern "C" QKM_API int qkm_moe_forward_host(qkm_ctx* c, uint32_t layer, int mode, const float* x_host,
                                            uint32_t n, float* y_host) {
    if (!c || !x_host || !y_host) return QKM_ERR_ARG;
    if (int rc = check_tokens(c, n)) return rc;
    const size_t bytes = (size_t)n * c->cfg.dims.n_embd * sizeof(float);
    QKM_CUDA(c, cudaMemcpyAsync(c->x_stage, x_host, bytes, cudaMemcpyHostToDevice, c->stream));
    const int rc = mode == 0 ? qkm_moe_decode(c, layer, c->x_stage, n, c->y_stage)
                             : qkm_moe_prefill(c, layer, c->x_stage, n, c->y_stage);
    if (rc) return rc;
    QKM_CUDA(c, cudaMemcpyAsync(y_host, c->y_stage, bytes, cudaMemcpyDeviceToHost, c->stream));
    return check_status(c);
}

static int decode_stack_eager(qkm_ctx* c, uint32_t first, uint32_t count, const float* x, uint32_t n, float* y) {
    const size_t stride = (size_t)n * c->cfg.dims.n_embd;
    for (uint32_t l = 0; l < count; ++l)
        if (int rc = qkm_moe_decode(c, first + l, x + l * stride, n, y + l * stride)) return rc;
    return QKM_OK;
}

// The per-layer launches of the stack are captured into a CUDA graph the first time an
// argument set is seen and replayed afterwards (a launch-bound inner loop: each layer is a
// handful of short kernels).  Capture needs a real stream: on the legacy default stream,
// while profiling, or after an upload, the launches are issued one by one.
extern "C" QKM_API int qkm_moe_decode_stack(qkm_ctx* c, uint32_t first, uint32_t count, const float* x,
                                            uint32_t n, float* y) {
    if (!c || !x || !y) return QKM_ERR_ARG;
    if ((uint64_t)first + count > c->cfg.n_layer) return fail(c, QKM_ERR_BOUNDS, "layers [%u,%u) out of range", first, first + count);
    if (int rc = check_tokens(c, n)) return rc;
    for (uint32_t l = 0; l < count; ++l)
        if (int rc = layer_ready(c, first + l)) return rc;
    if (c->stream == nullptr || c->profiling || count < 2) return decode_stack_eager(c, first, count, x, n, y);
    // A captured sequence always cuts the shared expert's work lists itself (shared_plan_n is cleared
    // before the capture), so a replay never depends on what ran in between.
    qkm_ctx::StackGraph* g = nullptr;
    for (auto& e : c->stack_graphs)
        if (e.exec && e.first == first && e.count == count && e.n == n && e.x == x && e.y == y && e.stream == c->stream) g = &e;
    if (!g) {
        qkm_ctx::StackGraph* slot = &c->stack_graphs[0];
        for (auto& e : c->stack_graphs) {
            if (!e.exec) { slot = &e; break; }
            if (e.used < slot->used) slot = &e;
        }
        if (slot->exec) { cudaGraphExecDestroy(slot->exec); slot->exec = nullptr; }
        c->shared_plan_n = 0;   // the captured sequence must cut the list itself
        const uint64_t before = c->launches;
        if (cudaStreamBeginCapture(c->stream, cudaStreamCaptureModeThreadLocal) != cudaSuccess) {
            cudaGetLastError();
            return decode_stack_eager(c, first, count, x, n, y);
        }
        const int rc = decode_stack_eager(c, first, count, x, n, y);
        cudaGraph_t graph = nullptr;
        const cudaError_t e = cudaStreamEndCapture(c->stream, &graph);
        slot->launches = c->launches - before;
        slot->plan_after = c->shared_plan_n;
        c->launches = before;
        c->shared_plan_n = 0;   // nothing captured has run
        if (rc != QKM_OK || e != cudaSuccess || !graph) {
            if (graph) cudaGraphDestroy(graph);
            cudaGetLastError();
            return rc != QKM_OK ? rc : decode_stack_eager(c, first, count, x, n, y);
        }
        const cudaError_t ei = cudaGraphInstantiate(&slot->exec, graph, 0);
        cudaGraphDestroy(graph);
        if (ei != cudaSuccess) {
            slot->exec = nullptr;
            cudaGetLastError();
            return decode_stack_eager(c, first, count, x, n, y);
        }
        slot->first = first; slot->count = count; slot->n = n; slot->x = x; slot->y = y; slot->stream = c->stream;
        g = slot;
    }
    g->used = ++c->stack_clock;
    QKM_CUDA(c, cudaGraphLaunch(g->exec, c->stream));
    c->launches += g->launches;
    c->shared_plan_n = g->plan_after;
    return QKM_OK;
}

extern "C" QKM_API int qkm_moe_decode_stack_host(qkm_ctx* c, uint32_t first, uint32_t count,
                                                 const float* x_host, uint32_t n, float* y_host) {
    if (!c || !x_host || !y_host) return QKM_ERR_ARG;
    if (int rc = check_tokens(c, n)) return rc;
    if ((uint64_t)first + count > c->cfg.n_layer) return fail(c, QKM_ERR_BOUNDS, "layers [%u,%u) out of range", first, first + count);
    if (!c->stack_x) {
        const size_t cap = (size_t)c->cfg.n_layer * c->cfg.max_tokens * c->cfg.dims.n_embd * sizeof(float);
        QKM_CUDA(c, cudaMalloc((void**)&c->stack_x, cap));
        QKM_CUDA(c, cudaMalloc((void**)&c->stack_y, cap));
    }
    const size_t layer_elems = (size_t)n * c->cfg.dims.n_embd;
    const size_t bytes = (size_t)count * layer_elems * sizeof(float);
    if (c->stream == nullptr || c->profiling || count < 2u * qkm_ctx::kStackChunks) {
        QKM_CUDA(c, cudaMemcpyAsync(c->stack_x, x_host, bytes, cudaMemcpyHostToDevice, c->stream));
        if (int rc = qkm_moe_decode_stack(c, first, count, c->stack_x, n, c->stack_y)) return rc;
        QKM_CUDA(c, cudaMemcpyAsync(y_host, c->stack_y, bytes, cudaMemcpyDeviceToHost, c->stream));
        return check_status(c);
    }
    // Chunks of layers: all input copies are queued on their own stream at once, chunk k computes as soon
    // as its rows are there, and its outputs leave on a third stream while chunk k+1 computes.  Only the
    // first chunk's copy in and the last chunk's copy out are not hidden, so these two chunks are short.
    if (!c->copy_in) {
        QKM_CUDA(c, cudaStreamCreateWithFlags(&c->copy_in, cudaStreamNonBlocking));
        QKM_CUDA(c, cudaStreamCreateWithFlags(&c->copy_out, cudaStreamNonBlocking));
        for (cudaEvent_t& ev : c->ev_in) QKM_CUDA(c, cudaEventCreateWithFlags(&ev, cudaEventDisableTiming));
        for (cudaEvent_t& ev : c->ev_out) QKM_CUDA(c, cudaEventCreateWithFlags(&ev, cudaEventDisableTiming));
        QKM_CUDA(c, cudaEventCreateWithFlags(&c->ev_copies, cudaEventDisableTiming));
    }
    constexpr uint32_t K = qkm_ctx::kStackChunks;
    // two layers first and two last (what is not hidden is their copy in and copy out), the rest in halves
    static_assert(K == 4, "chunk boundaries below are written for four chunks");
    const uint32_t lo[K + 1] = {0u, 2u, 2u + (count - 4u) / 2u, count - 2u, count};
    // whatever the stream still holds (it reads or writes the staging buffers) comes first
    QKM_CUDA(c, cudaEventRecord(c->ev_copies, c->stream));
    QKM_CUDA(c, cudaStreamWaitEvent(c->copy_in, c->ev_copies, 0));
    for (uint32_t k = 0; k < K; ++k) {
        const size_t off = lo[k] * layer_elems, len = (size_t)(lo[k + 1] - lo[k]) * layer_elems * sizeof(float);
        QKM_CUDA(c, cudaMemcpyAsync(c->stack_x + off, x_host + off, len, cudaMemcpyHostToDevice, c->copy_in));
        QKM_CUDA(c, cudaEventRecord(c->ev_in[k], c->copy_in));
    }
    for (uint32_t k = 0; k < K; ++k) {
        const size_t off = lo[k] * layer_elems, len = (size_t)(lo[k + 1] - lo[k]) * layer_elems * sizeof(float);
        QKM_CUDA(c, cudaStreamWaitEvent(c->stream, c->ev_in[k], 0));
        if (int rc = qkm_moe_decode_stack(c, first + lo[k], lo[k + 1] - lo[k], c->stack_x + off, n, c->stack_y + off)) return rc;
        QKM_CUDA(c, cudaEventRecord(c->ev_out[k], c->stream));
        QKM_CUDA(c, cudaStreamWaitEvent(c->copy_out, c->ev_out[k], 0));
        QKM_CUDA(c, cudaMemcpyAsync(y_host + off, c->stack_y + off, len, cudaMemcpyDeviceToHost, c->copy_out));
    }
    QKM_CUDA(c, cudaEventRecord(c->ev_copies, c->copy_out));
    QKM_CUDA(c, cudaStreamWaitEvent(c->stream, c->ev_copies, 0));   // the stream's synchronise below covers the copies
    return check_status(c);
}

extern "C" QKM_API int qkm_profile_enable(qkm_ctx* c, int on) {
    if (!c) return QKM_ERR_ARG;
    if (on && !c->prof_ev[0])
        for (cudaEvent_t& ev : c->prof_ev) QKM_CUDA(c, cudaEventCreate(&ev));
    c->profiling = on != 0;
    c->prof_n = 0;
    return QKM_OK;
}

extern "C" QKM_API int qkm_profile_read(qkm_ctx* c, char* labels, float* ms, uint32_t max_stages) {
    if (!c || !labels || !ms) return QKM_ERR_ARG;
    if (!c->profiling) return fail(c, QKM_ERR_MODE, "profiling is not enabled");
    QKM_CUDA(c, cudaStreamSynchronize(c->stream));
    const int n = c->prof_n < (int)max_stages ? c->prof_n : (int)max_stages;
    for (int i = 0; i < n; ++i) {
        memcpy(labels + 16 * i, c->prof_label[i], 16);
        QKM_CUDA(c, cudaEventElapsedTime(&ms[i], c->prof_ev[i], c->prof_ev[i + 1]));
    }
    return n;
}

extern "C" QKM_API int qkm_last_sel(qkm_ctx* c, qkm_sel* sel_host, uint32_t n) {
    if (!c || !sel_host) return QKM_ERR_ARG;
    if (int rc = check_tokens(c, n)) return rc;
    return qkm_d2h(c, sel_host, c->sel, (size_t)n * sizeof(qkm_sel));
}
extern "C" QKM_API const qkm_sel* qkm_sel_device(const qkm_ctx* c) { return c ? c->sel : nullptr; }
extern "C" QKM_API const float* qkm_h_device(const qkm_ctx* c) { return c ? c->h : nullptr; }

// ---------------------------------------------------------------- dense quantised GEMM
// The reference's batched-prefill projections (gemm_q8_0*.comp, gemm_iq4_xs.comp; dispatched at
// src/main.cpp:4806-4835): Y[n][M] = X[n][K] . W^T with W a Q8_0 or IQ4_XS matrix.  The matrix is
// uploaded once into a slot (copied and tile-ordered on the device); the GEMM runs on the same
// dequantise-to-shared-memory + tcgen05 pipeline as the experts' down projection, bf16 operands.

extern "C" QKM_API int qkm_dense_upload(qkm_ctx* c, uint32_t slot, uint32_t type, const void* w_host, uint32_t M, uint32_t K) {
    if (!c || !w_host) return QKM_ERR_ARG;
    if (slot >= qkm_ctx::kDenseSlots) return fail(c, QKM_ERR_BOUNDS, "dense slot %u out of range", slot);
    if (type != QKM_TYPE_Q8_0 && type != QKM_TYPE_IQ4_XS) return fail(c, QKM_ERR_TYPE, "qkm_dense_upload: type %u (Q8_0 or IQ4_XS)", type);
    if (M == 0 || M % 128 || K == 0 || K % 256) return fail(c, QKM_ERR_ARG, "qkm_dense_upload: M %% 128 and K %% 256 must be 0 (M=%u K=%u)", M, K);
    auto& dm = c->dense[slot];
    if (dm.tiles) { QKM_CUDA(c, cudaFree(dm.tiles)); dm = qkm_ctx::Dense{}; }
    const size_t bytes = (size_t)M * row_bytes(type, K);
    void* raw = nullptr;
    QKM_CUDA(c, cudaMalloc(&raw, bytes + 256));
    cudaError_t e = cudaMalloc(&dm.tiles, bytes + 256);
    if (e == cudaSuccess) e = cudaMemcpyAsync(raw, w_host, bytes, cudaMemcpyHostToDevice, c->stream);
    if (e == cudaSuccess) e = cudaMemsetAsync((uint8_t*)dm.tiles + bytes, 0, 256, c->stream);
    if (e == cudaSuccess) e = launch_repack(c->L(), type, raw, dm.tiles, 1, M, K);
    if (e == cudaSuccess) e = cudaStreamSynchronize(c->stream);
    cudaFree(raw);
    if (e != cudaSuccess) {
        if (dm.tiles) cudaFree(dm.tiles);
        dm = qkm_ctx::Dense{};
        return fail(c, QKM_ERR_CUDA, "qkm_dense_upload: %s", cudaGetErrorString(e));
    }
    dm.type = type; dm.M = M; dm.K = K;
    return QKM_OK;
}

extern "C" QKM_API int qkm_dense_gemm(qkm_ctx* c, uint32_t slot, const float* x, uint32_t n, float* y) {
    if (!c || !x || !y) return QKM_ERR_ARG;
    if (slot >= qkm_ctx::kDenseSlots || !c->dense[slot].tiles) return fail(c, QKM_ERR_BUSY, "dense slot %u holds no matrix", slot);
    if (n == 0) return QKM_OK;
    const auto& dm = c->dense[slot];
    const uint32_t NT = prefill_pairs_per_block();
    const size_t elems = (size_t)n * dm.K, items = (size_t)((n + NT - 1) / NT) * (dm.M / 128);
    if (elems > c->dense_cap_elems) {
        if (c->dense_xb) QKM_CUDA(c, cudaFree(c->dense_xb));
        c->dense_xb = nullptr; c->dense_cap_elems = 0;
        QKM_CUDA(c, cudaMalloc(&c->dense_xb, elems * 2));
        c->dense_cap_elems = elems;
    }
    if (n > c->dense_cap_rows) {
        if (c->dense_pairs) { cudaFree(c->dense_pairs); cudaFree(c->dense_sel); }
        c->dense_pairs = nullptr; c->dense_sel = nullptr; c->dense_cap_rows = 0;
        QKM_CUDA(c, cudaMalloc((void**)&c->dense_pairs, (size_t)n * sizeof(uint32_t)));
        QKM_CUDA(c, cudaMalloc((void**)&c->dense_sel, (size_t)n * sizeof(qkm_sel)));
        c->dense_cap_rows = n;
    }
    if (items > c->dense_cap_items) {
        if (c->dense_items) cudaFree(c->dense_items);
        c->dense_items = nullptr; c->dense_cap_items = 0;
        QKM_CUDA(c, cudaMalloc((void**)&c->dense_items, items * sizeof(MmaItem)));
        c->dense_cap_items = items;
    }
    if (!c->dense_n_items) QKM_CUDA(c, cudaMalloc((void**)&c->dense_n_items, sizeof(uint32_t)));
    QKM_LAUNCH(c, launch_dense_gemm(c->L(), dm.type, dm.tiles, dm.M, dm.K, x, n, y, c->dense_xb, c->dense_pairs, c->dense_sel,
                                    c->dense_items, c->dense_n_items, c->status));
    return QKM_OK;
}

// ---------------------------------------------------------------- layer entry / tail

extern "C" QKM_API int qkm_add_rmsnorm(qkm_ctx* c, const float* a, const float* b, const float* w, float* y, float* xn,
                                       uint32_t n_rows, uint32_t n, float eps) {
    if (!c || !a || !b || !w || !y || !xn) return QKM_ERR_ARG;
    QKM_LAUNCH(c, launch_add_rms(c->L(), 0, a, b, nullptr, w, y, xn, n_rows, n, 0, eps));
    return QKM_OK;
}

extern "C" QKM_API int qkm_add_rms3(qkm_ctx* c, const float* a, const float* b, const float* c2, const float* w,
                                    float* s, float* xn, uint32_t n_rows, uint32_t n, float eps) {
    if (!c || !a || !b || !c2 || !w || !s || !xn) return QKM_ERR_ARG;
    QKM_LAUNCH(c, launch_add_rms(c->L(), 1, a, b, c2, w, s, xn, n_rows, n, 0, eps));
    return QKM_OK;
}

extern "C" QKM_API int qkm_add_rms3_grouped(qkm_ctx* c, const float* a, const float* routed, const float* c2,
                                            const float* w, float* s, float* xn, uint32_t n_rows, uint32_t n,
                                            uint32_t n_used, float eps) {
    if (!c || !a || !routed || !c2 || !w || !s || !xn) return QKM_ERR_ARG;
    if (n_used == 0 || n_used > 16) return fail(c, QKM_ERR_ARG, "qkm_add_rms3_grouped: n_used %u", n_used);
    QKM_LAUNCH(c, launch_add_rms(c->L(), 2, a, routed, c2, w, s, xn, n_rows, n, n_used, eps));
    return QKM_OK;
}

extern "C" QKM_API int qkm_argmax(qkm_ctx* c, const float* logits, uint32_t n_rows, uint32_t n, uint32_t* tok) {
    if (!c || !logits || !tok) return QKM_ERR_ARG;
    if (n_rows > c->argmax_rows) {
        if (c->argmax_scratch) QKM_CUDA(c, cudaFree(c->argmax_scratch));
        c->argmax_scratch = nullptr; c->argmax_rows = 0;
        QKM_CUDA(c, cudaMalloc(&c->argmax_scratch, argmax_scratch_bytes(n_rows)));
        c->argmax_rows = n_rows;
    }
    QKM_LAUNCH(c, launch_argmax(c->L(), logits, n_rows, n, c->argmax_scratch, tok));
    return QKM_OK;
}

// One decoder layer's feed-forward half as the engine runs it (src/main.cpp:4375-4404):
// resid2 = resid + attn_out, xn2 = rmsnorm(resid2) * w_post; y = MoE(xn2);
// resid_out = resid2 + y, xn_next = rmsnorm(resid_out) * w_next.
extern "C" QKM_API int qkm_moe_layer_step(qkm_ctx* c, uint32_t layer, const float* resid, const float* attn_out,
                                          const float* w_post, const float* w_next, uint32_t n, float eps,
                                          float* resid_out, float* xn_next) {
    if (int rc = layer_ready(c, layer)) return rc;
    if (!resid || !attn_out || !w_post || !w_next || !resid_out || !xn_next) return QKM_ERR_ARG;
    if (int rc = check_tokens(c, n)) return rc;
    const qkm_dims& d = c->cfg.dims;
    // x_stage / y_stage double as resid2 / MoE output scratch ([max_tokens][n_embd] each)
    float* xn2 = c->x_stage;
    QKM_LAUNCH(c, launch_add_rms(c->L(), 0, resid, attn_out, nullptr, w_post, resid_out, xn2, n, d.n_embd, 0, eps));
    const int rc = n <= 64 ? qkm_moe_decode(c, layer, xn2, n, c->y_stage) : qkm_moe_prefill(c, layer, xn2, n, c->y_stage);
    if (rc) return rc;
    QKM_LAUNCH(c, launch_add_rms(c->L(), 0, resid_out, c->y_stage, nullptr, w_next, resid_out, xn_next, n, d.n_embd, 0, eps));
    return QKM_OK;
}

// ---------------------------------------------------------------- expert parallel
// One context per GPU, opened with expert_first/expert_count naming its shard.  Per layer:
//   qkm_ep_dispatch  : route the local tokens, decide which rows go to which rank, pack them
//   (host: all-to-all of the rows and their selection records)
//   qkm_ep_shared    : the shared expert of the local tokens (runs while the rows travel)
//   qkm_ep_expert_forward : resident experts over the received rows -> one partial row each
//   (host: all-to-all of the partial rows back)
//   qkm_ep_combine   : y = shared + partials, summed in rank order
// The reference has no multi-GPU path; the sequence keeps its single-GPU arithmetic
// (src/main.cpp:1316-1387) and only changes the order in which a token's slots are summed.

static int ep_check(qkm_ctx* c, uint32_t n_ranks) {
    const qkm_dims& d = c->cfg.dims;
    c->shared_plan_n = 0;
    if (n_ranks == 0 || n_ranks > 64 || d.n_expert % n_ranks) return fail(c, QKM_ERR_ARG, "n_ranks %u does not divide n_expert %u", n_ranks, d.n_expert);
    if (c->ecount != d.n_expert / n_ranks || c->efirst % c->ecount)
        return fail(c, QKM_ERR_MODE, "context holds experts [%u,%u): not one of %u equal shards", c->efirst, c->efirst + c->ecount, n_ranks);
    if (c->ep_ranks != n_ranks) {
        if (c->ep_counts) { cudaFree(c->ep_counts); cudaFree(c->ep_send_tok); cudaFree(c->ep_send_pos); cudaFreeHost(c->ep_counts_host); }
        c->ep_counts = c->ep_send_tok = c->ep_send_pos = c->ep_counts_host = nullptr;
        c->ep_ranks = 0;
        const size_t T = c->cfg.max_tokens, fan = n_ranks < d.n_used ? n_ranks : d.n_used;
        QKM_CUDA(c, cudaMalloc((void**)&c->ep_counts, (n_ranks + 1) * sizeof(uint32_t)));
        QKM_CUDA(c, cudaMalloc((void**)&c->ep_send_tok, T * fan * sizeof(uint32_t)));
        QKM_CUDA(c, cudaMalloc((void**)&c->ep_send_pos, T * n_ranks * sizeof(uint32_t)));
        QKM_CUDA(c, cudaMallocHost((void**)&c->ep_counts_host, (n_ranks + 1) * sizeof(uint32_t)));
        c->ep_ranks = n_ranks;
    }
    return QKM_OK;
}

// router logits and selection of the n local tokens into c->sel (digit planes / f16 rows as the
// shared-expert kernels of that size want them)
static int ep_route_local(qkm_ctx* c, uint32_t layer, const float* x, uint32_t n) {
    const qkm_layer_dev& ld = c->layers[layer];
    const qkm_layer_weights& w = ld.w;
    const qkm_dims& d = c->cfg.dims;
    const bool planes = ld.tiles_ok && n <= 64;   // the streamed shared-expert kernels read digit planes
    const bool tc = ld.tiles_ok && n >= 128;      // tensor-core logits from f16 rows
    if (tc) {
        if (int rc = ensure_prefill_scratch(c)) return rc;
        QKM_LAUNCH(c, launch_to_f16_rows(c->L(), x, c->xb, c->xscale, n, d.n_embd));
    }
    QKM_LAUNCH(c, launch_route_select(c->L(), d, w.router_type, w.router, w.gate_inp_shexp, x, c->sel, n, c->route_scratch, c->route_scratch_bytes,
                                      planes ? c->xplanes : nullptr, planes ? c->xscale : nullptr, tc ? c->xb : nullptr,
                                      tc ? c->xscale : nullptr, c->status));
    return QKM_OK;
}

static int ep_dispatch_launch(qkm_ctx* c, uint32_t layer, const float* x, uint32_t n, uint32_t n_ranks,
                              float* xsend, qkm_sel* selsend) {
    if (int rc = layer_ready(c, layer)) return rc;
    if (!x || !xsend || !selsend) return QKM_ERR_ARG;
    if (int rc = check_tokens(c, n)) return rc;
    if (int rc = ep_check(c, n_ranks)) return rc;
    if (int rc = ep_route_local(c, layer, x, n)) return rc;
    const qkm_dims& d = c->cfg.dims;
    QKM_LAUNCH(c, launch_ep_plan(c->L(), d, c->sel, n, n_ranks, c->ep_counts, c->ep_send_tok, c->ep_send_pos));
    const uint32_t fan = n_ranks < d.n_used ? n_ranks : d.n_used;
    QKM_LAUNCH(c, launch_ep_pack(c->L(), d, x, c->sel, c->ep_send_tok, c->ep_counts + n_ranks, n * fan, xsend, selsend));
    return QKM_OK;
}

extern "C" QKM_API int qkm_ep_dispatch(qkm_ctx* c, uint32_t layer, const float* x, uint32_t n, uint32_t n_ranks,
                                       float* xsend, qkm_sel* selsend, uint32_t* counts_host) {
    if (!counts_host) return QKM_ERR_ARG;
    if (int rc = ep_dispatch_launch(c, layer, x, n, n_ranks, xsend, selsend)) return rc;
    QKM_CUDA(c, cudaMemcpyAsync(c->ep_counts_host, c->ep_counts, (n_ranks + 1) * sizeof(uint32_t), cudaMemcpyDeviceToHost, c->stream));
    QKM_CUDA(c, cudaStreamSynchronize(c->stream));
    memcpy(counts_host, c->ep_counts_host, n_ranks * sizeof(uint32_t));
    return QKM_OK;
}

// The same without touching the host: the row counts go to a device buffer of the caller
// (n_ranks 32-bit words), so they can feed the collective that exchanges them directly.
extern "C" QKM_API int qkm_ep_dispatch_dev(qkm_ctx* c, uint32_t layer, const float* x, uint32_t n, uint32_t n_ranks,
                                           float* xsend, qkm_sel* selsend, uint32_t* counts_dev) {
    if (!counts_dev) return QKM_ERR_ARG;
    if (int rc = ep_dispatch_launch(c, layer, x, n, n_ranks, xsend, selsend)) return rc;
    QKM_CUDA(c, cudaMemcpyAsync(counts_dev, c->ep_counts, n_ranks * sizeof(uint32_t), cudaMemcpyDeviceToDevice, c->stream));
    return QKM_OK;
}

extern "C" QKM_API int qkm_ep_shared(qkm_ctx* c, uint32_t layer, const float* x, uint32_t n) {
    if (int rc = layer_ready(c, layer)) return rc;
    c->shared_plan_n = 0;
    if (!x) return QKM_ERR_ARG;
    if (int rc = check_tokens(c, n)) return rc;
    if (n == 0) return QKM_OK;
    const qkm_layer_dev& ld = c->layers[layer];
    const qkm_layer_weights& w = ld.w;
    const qkm_dims& d = c->cfg.dims;
    if (!ld.tiles_ok) {
        QKM_LAUNCH(c, launch_shared_gateup(c->L(), d, w.gate_shexp, w.up_shexp, x, c->h, n));
        QKM_LAUNCH(c, launch_shared_down(c->L(), d, w.down_shexp, c->h, c->sel, c->y2, n));
        return QKM_OK;
    }
    if (n <= 64) {   // streamed kernels of the decode sequence (digit planes written by qkm_ep_dispatch)
        const uint32_t nb = (uint32_t)c->n_sms;
        QKM_LAUNCH(c, launch_shared_plan(c->L(), d, n, c->pairs, c->items_sh_gu, d.n_ff / gateup_stream_rows_per_item(),
                                         c->items_sh_dn, d.n_embd / down_stream_rows_per_item(), 2, c->n_items + 2));
        QKM_LAUNCH(c, launch_gateup_stream(c->L(), d, QKM_TYPE_Q8_0, ld.tiles[5], ld.tiles[6], c->xplanes, c->xscale, c->pairs,
                                           c->items_sh_gu, c->n_items + 2, c->h, c->hpieces, nb, c->status));
        QKM_LAUNCH(c, launch_down_stream(c->L(), d, QKM_TYPE_Q8_0, ld.tiles[7], c->hpieces, c->sel, c->pairs, c->items_sh_dn,
                                         c->n_items + 3, nullptr, c->y2, nullptr, nb, c->status));
        return QKM_OK;
    }
    // tensor-core kernels with an empty routed list: only the shared expert's tiles
    if (int rc = ensure_prefill_scratch(c)) return rc;
    const uint32_t NT = prefill_pairs_per_block(), sh_now = (n + NT - 1) / NT;
    QKM_CUDA(c, cudaMemsetAsync(c->offsets, 0, sizeof(uint32_t), c->stream));
    QKM_LAUNCH(c, launch_mma_plan(c->L(), d, c->offsets, c->pairs, 0, n, c->mma_items[0], c->mma_items[1], c->mma_items[2],
                                  c->mma_items[3], c->n_items, c->pos_of, true));
    QKM_LAUNCH(c, launch_to_f16_rows(c->L(), x, c->xb, c->xscale, n, d.n_embd));
    QKM_LAUNCH(c, launch_gateup_mma(c->L(), d, QKM_TYPE_Q8_0, ld.tiles[5], ld.tiles[6], c->xb, c->xscale, c->pairs, c->mma_items[2],
                                    c->n_items + 2, sh_now * (d.n_ff / 128), nullptr, c->hb, c->status, sh_now * (d.n_ff / 128) <= 2u * (uint32_t)c->n_sms,
                                    nullptr, c->h));
    QKM_LAUNCH(c, launch_h_rows_to_f16(c->L(), c->h, c->hb, c->hscale, d.n_ff, nullptr, 0, nullptr, n));   // the routed list is empty: rows 0 .. n-1
    QKM_LAUNCH(c, launch_down_mma(c->L(), d, QKM_TYPE_Q8_0, ld.tiles[7], c->hb, c->sel, c->pairs, c->mma_items[3],
                                  c->n_items + 3, sh_now * (d.n_embd / 128), c->contrib_p, c->status, false, nullptr, c->hscale));
    QKM_LAUNCH(c, launch_fold_pairs(c->L(), d, c->contrib_p, c->pos_of, c->y2, n));
    return QKM_OK;
}

// Resident experts over n_recv rows -> partial.  with_shared: rows [sh_first, sh_first + sh_count)
// are this rank's own tokens and also get the shared expert (its two GEMMs run beside the routed
// ones on the side stream, as in qkm_moe_prefill), so their partial rows carry shared + routed.
// slot_rows_peer != 0: the rows are slots of the peer-memory form and every live partial row is
// stored into its source rank's return buffer instead of staying in `partial`.
static int ep_expert_forward_impl(qkm_ctx* c, uint32_t layer, const float* xrecv, const qkm_sel* selrecv, uint32_t n_recv,
                                  float* partial, bool with_shared, uint32_t sh_first, uint32_t sh_count,
                                  uint32_t slot_rows_peer = 0, bool rows_f16 = false) {
    if (int rc = layer_ready(c, layer)) return rc;
    c->shared_plan_n = 0;
    if (n_recv == 0) return QKM_OK;
    if (!xrecv || !selrecv || !partial) return QKM_ERR_ARG;
    if (int rc = check_tokens(c, n_recv)) return rc;
    const qkm_layer_dev& ld = c->layers[layer];
    const qkm_layer_weights& w = ld.w;
    const qkm_dims& d = c->cfg.dims;
    if (!ld.tiles_ok) {   // generic kernels on the raw layout
        const float* y2 = nullptr;
        if (with_shared && sh_count) {   // shared expert of the own rows first (it uses h too), added by the fold
            const float* xo = xrecv + (size_t)sh_first * d.n_embd;
            QKM_CUDA(c, cudaMemsetAsync(c->y2, 0, (size_t)n_recv * d.n_embd * sizeof(float), c->stream));
            QKM_LAUNCH(c, launch_shared_gateup(c->L(), d, w.gate_shexp, w.up_shexp, xo, c->h, sh_count));
            QKM_LAUNCH(c, launch_shared_down(c->L(), d, w.down_shexp, c->h, selrecv + sh_first, c->y2 + (size_t)sh_first * d.n_embd, sh_count));
            y2 = c->y2;
        }
        QKM_LAUNCH(c, launch_group_pairs(c->L(), d, selrecv, n_recv, c->offsets, c->pairs, c->efirst, c->ecount));
        if (!c->contrib) QKM_CUDA(c, cudaMalloc((void**)&c->contrib, (size_t)c->cfg.max_tokens * d.n_used * d.n_embd * sizeof(float)));
        QKM_LAUNCH(c, launch_gateup_pairs(c->L(), d, w.gateup_type, w.gate_exps, w.up_exps, xrecv, c->offsets, c->pairs, c->h, n_recv, c->efirst, c->ecount));
        QKM_CUDA(c, cudaMemsetAsync(c->contrib, 0, (size_t)n_recv * d.n_used * d.n_embd * sizeof(float), c->stream));
        QKM_LAUNCH(c, launch_down_pairs(c->L(), d, w.down_type, w.down_exps, c->h, selrecv, c->offsets, c->pairs, c->contrib, n_recv, c->efirst, c->ecount));
        QKM_LAUNCH(c, launch_fold_contrib(c->L(), d, c->contrib, y2, partial, n_recv));
        if (slot_rows_peer)
            QKM_LAUNCH(c, launch_ep_return(c->L(), d, partial, selrecv, c->pm_peers, slot_rows_peer, c->pm_rank, c->pm_ranks,
                                           with_shared ? sh_count : 0));
        return QKM_OK;
    }
    if (int rc = ensure_prefill_scratch(c)) return rc;
    const uint32_t NT = prefill_pairs_per_block();
    const uint32_t np_max = n_recv * d.n_used;
    const uint32_t tiles_now = c->ecount < np_max ? c->ecount + (np_max + NT - 1) / NT : np_max;
    const uint32_t rt_gu = d.n_ff / 128, rt_dn = d.n_embd / 128;
    QKM_LAUNCH(c, launch_group_pairs_wide(c->L(), d, selrecv, n_recv, c->offsets, c->pairs, c->efirst, c->ecount, c->group_hist, c->pos_of));
    QKM_LAUNCH(c, launch_mma_plan(c->L(), d, c->offsets, c->pairs, c->ecount, n_recv, c->mma_items[0], c->mma_items[1],
                                  c->mma_items[2], c->mma_items[3], c->n_items, c->pos_of, with_shared, true, sh_first,
                                  with_shared ? sh_count : 0));
    // the rows as scaled f16: converted here, or already so on arrival (then only their scales are gathered)
    const void* xb_rows = c->xb;
    if (rows_f16) {
        xb_rows = xrecv;
        QKM_LAUNCH(c, launch_ep_row_scales(c->L(), selrecv, c->xscale, n_recv));
    } else {
        QKM_LAUNCH(c, launch_to_f16_rows(c->L(), xrecv, c->xb, c->xscale, n_recv, d.n_embd));
    }
    const bool fork = with_shared && sh_count;
    if (fork) {
        const uint32_t sh_now = (sh_count + NT - 1) / NT;
        Launch S{c->side, &c->launches};
        QKM_CUDA(c, cudaEventRecord(c->ev_fork, c->stream));
        QKM_CUDA(c, cudaStreamWaitEvent(c->side, c->ev_fork, 0));
        QKM_LAUNCH(c, launch_gateup_mma(S, d, QKM_TYPE_Q8_0, ld.tiles[5], ld.tiles[6], xb_rows, c->xscale, c->pairs, c->mma_items[2],
                                        c->n_items + 2, sh_now * rt_gu, nullptr, c->hb, c->status, sh_now * rt_gu <= 2u * (uint32_t)c->n_sms,
                                        nullptr, c->h));
        QKM_LAUNCH(c, launch_h_rows_to_f16(S, c->h, c->hb, c->hscale, d.n_ff, c->offsets + c->ecount, 0, nullptr, sh_count));
        QKM_LAUNCH(c, launch_down_mma(S, d, QKM_TYPE_Q8_0, ld.tiles[7], c->hb, selrecv, c->pairs, c->mma_items[3],
                                      c->n_items + 3, sh_now * rt_dn, c->contrib_p, c->status, false, nullptr, c->hscale));
        QKM_CUDA(c, cudaEventRecord(c->ev_join, c->side));
    }
    // a shard of few experts launches fewer blocks than the machine holds: faster blocks instead (see the launchers)
    const bool few_gu = c->ecount * rt_gu <= 2u * (uint32_t)c->n_sms, few_dn = c->ecount * rt_dn / 4 <= 2u * (uint32_t)c->n_sms;
    QKM_LAUNCH(c, launch_gateup_mma(c->L(), d, w.gateup_type, ld.tiles[2], ld.tiles[3], xb_rows, c->xscale, c->pairs, c->mma_items[0],
                                    c->n_items, tiles_now * rt_gu, nullptr, c->hb, c->status, few_gu, c->lut_pf, c->h));
    QKM_LAUNCH(c, launch_h_rows_to_f16(c->L(), c->h, c->hb, c->hscale, d.n_ff, nullptr, 0, c->offsets + c->ecount, n_recv * d.n_used));
    QKM_LAUNCH(c, launch_down_mma(c->L(), d, w.down_type, ld.tiles[4], c->hb, selrecv, c->pairs, c->mma_items[1],
                                  c->n_items + 1, tiles_now * rt_dn, c->contrib_p, c->status, few_dn, c->lut_dn, c->hscale));
    if (fork) QKM_CUDA(c, cudaStreamWaitEvent(c->stream, c->ev_join, 0));
    if (slot_rows_peer)
        QKM_LAUNCH(c, launch_fold_pairs_peer(c->L(), d, c->contrib_p, c->pos_of, c->pm_peers, slot_rows_peer, c->pm_rank, c->pm_ranks));
    else
        QKM_LAUNCH(c, launch_fold_pairs(c->L(), d, c->contrib_p, c->pos_of, partial, n_recv));
    return QKM_OK;
}

extern "C" QKM_API int qkm_ep_expert_forward(qkm_ctx* c, uint32_t layer, const float* xrecv, const qkm_sel* selrecv,
                                             uint32_t n_recv, float* partial) {
    return ep_expert_forward_impl(c, layer, xrecv, selrecv, n_recv, partial, false, 0, 0);
}

extern "C" QKM_API int qkm_ep_combine(qkm_ctx* c, uint32_t n, uint32_t n_ranks, const float* back, float* y) {
    if (!c || !y || (!back && n)) return QKM_ERR_ARG;
    if (int rc = check_tokens(c, n)) return rc;
    if (c->ep_ranks != n_ranks || !c->ep_send_pos) return fail(c, QKM_ERR_MODE, "qkm_ep_combine without a matching qkm_ep_dispatch");
    QKM_LAUNCH(c, launch_ep_combine(c->L(), c->cfg.dims, back, c->ep_send_pos, c->y2, y, n, n_ranks));
    return QKM_OK;
}

// ---------------------------------------------------------------- expert parallel over peer memory
// The same layer without an all-to-all.  Every rank keeps three receive buffers of
// n_ranks * slot_cap rows (x rows, selection records, returned partial rows) and maps every peer's:
//   qkm_ep_peer_setup   : allocate this rank's buffers
//   qkm_ep_peer_export / qkm_ep_peer_import : CUDA IPC handles between processes of one node,
//   or qkm_ep_peer_buffers / qkm_ep_peer_set  : raw pointers (one process driving several GPUs)
// and per layer, with slot_rows (>= every rank's token count, the same on all ranks):
//   qkm_ep_push         : route the local tokens, store rows + records into the owners' buffers
//   qkm_ep_shared       : the shared expert (no dependence on the peers)
//   (host: barrier)     : all pushes have landed
//   qkm_ep_forward_slots: resident experts over the n_ranks * slot_rows rows; each partial row is
//                         stored into its source rank's return buffer
//   (host: barrier)     : all partial rows have landed
//   qkm_ep_pull         : y = shared + the partial rows the owners returned
// The two barriers also order the reuse of the buffers by the next layer: a rank pushes layer
// l+1 after the second barrier of layer l, when every rank has finished reading the rows of l,
// and stores partial rows of l+1 after the first barrier of l+1, which every rank enters after
// its pull of l.  Kernels only store to and load from peer memory; none waits.

constexpr size_t kPmFlagBytes = 256;
static uint32_t* pm_flags_of(const qkm_ctx* c, void* selrecv) {
    return (uint32_t*)((char*)selrecv + (size_t)c->pm_ranks * c->pm_cap * sizeof(qkm_sel));
}

static int pm_check(qkm_ctx* c, uint32_t slot_rows) {
    if (!c) return QKM_ERR_ARG;
    if (!c->pm_ranks) return fail(c, QKM_ERR_MODE, "qkm_ep_peer_setup has not been called");
    if (slot_rows == 0 || slot_rows > c->pm_cap) return fail(c, QKM_ERR_BOUNDS, "slot_rows %u outside 1..%u", slot_rows, c->pm_cap);
    for (uint32_t r = 0; r < c->pm_ranks; ++r)
        if (!c->pm_peers.x[r] || !c->pm_peers.sel[r] || !c->pm_peers.back[r] || !c->pm_peers.flags[r])
            return fail(c, QKM_ERR_MODE, "buffers of rank %u are not mapped (qkm_ep_peer_import / qkm_ep_peer_set)", r);
    return QKM_OK;
}

extern "C" QKM_API int qkm_ep_peer_setup(qkm_ctx* c, uint32_t n_ranks, uint32_t rank, uint32_t slot_cap) {
    if (!c) return QKM_ERR_ARG;
    const qkm_dims& d = c->cfg.dims;
    if (c->pm_ranks) return fail(c, QKM_ERR_MODE, "qkm_ep_peer_setup was already called on this context");
    if (n_ranks == 0 || n_ranks > kMaxPeerRanks || d.n_expert % n_ranks || rank >= n_ranks)
        return fail(c, QKM_ERR_ARG, "rank %u of %u ranks (at most %u, dividing n_expert %u)", rank, n_ranks, kMaxPeerRanks, d.n_expert);
    if (c->ecount != d.n_expert / n_ranks || c->efirst != rank * c->ecount)
        return fail(c, QKM_ERR_MODE, "context holds experts [%u,%u): not shard %u of %u", c->efirst, c->efirst + c->ecount, rank, n_ranks);
    if (slot_cap == 0 || (uint64_t)slot_cap * n_ranks > c->cfg.max_tokens)
        return fail(c, QKM_ERR_BOUNDS, "%u ranks x %u rows exceed max_tokens %u", n_ranks, slot_cap, c->cfg.max_tokens);
    const size_t rows = (size_t)n_ranks * slot_cap;
    QKM_CUDA(c, cudaSetDevice(c->device));
    // all five buffers or none: a failure part way frees what was taken, so a retry starts clean
    cudaError_t e = cudaMalloc((void**)&c->pm_xrecv, rows * d.n_embd * sizeof(float));
    // the barrier words of qkm_ep_barrier sit behind the records, so three mappings carry everything
    if (e == cudaSuccess) e = cudaMalloc((void**)&c->pm_selrecv, rows * sizeof(qkm_sel) + kPmFlagBytes);
    if (e == cudaSuccess) e = cudaMemset((char*)c->pm_selrecv + rows * sizeof(qkm_sel), 0, kPmFlagBytes);
    if (e == cudaSuccess) e = cudaMalloc((void**)&c->pm_partial, rows * d.n_embd * sizeof(float));
    if (e == cudaSuccess) e = cudaMalloc((void**)&c->pm_back, rows * d.n_embd * sizeof(float));
    if (e == cudaSuccess) e = cudaMalloc((void**)&c->pm_xscale, (size_t)slot_cap * sizeof(float));
    if (e == cudaSuccess) e = cudaMemset(c->pm_back, 0, rows * d.n_embd * sizeof(float));
    if (e == cudaSuccess) e = cudaMemset(c->pm_xrecv, 0, rows * d.n_embd * sizeof(float));
    if (e == cudaSuccess) e = cudaMemset(c->pm_selrecv, 0xFF, rows * sizeof(qkm_sel));   // every record empty
    if (e == cudaSuccess) e = cudaMemset(c->pm_partial, 0, rows * d.n_embd * sizeof(float));
    if (e != cudaSuccess) {
        for (void** p : {(void**)&c->pm_xrecv, (void**)&c->pm_selrecv, (void**)&c->pm_partial, (void**)&c->pm_back, (void**)&c->pm_xscale}) {
            if (*p) cudaFree(*p);
            *p = nullptr;
        }
        return fail(c, QKM_ERR_CUDA, "qkm_ep_peer_setup: %s", cudaGetErrorString(e));
    }
    c->pm_ranks = n_ranks; c->pm_rank = rank; c->pm_cap = slot_cap; c->pm_epoch = 0;
    c->pm_peers.x[rank] = c->pm_xrecv; c->pm_peers.sel[rank] = c->pm_selrecv; c->pm_peers.back[rank] = c->pm_back;
    c->pm_peers.flags[rank] = pm_flags_of(c, c->pm_selrecv);
    return QKM_OK;
}

extern "C" QKM_API int qkm_ep_peer_buffers(qkm_ctx* c, void** xrecv, void** selrecv, void** back) {
    if (!c || !xrecv || !selrecv || !back) return QKM_ERR_ARG;
    if (!c->pm_ranks) return fail(c, QKM_ERR_MODE, "qkm_ep_peer_setup has not been called");
    *xrecv = c->pm_xrecv; *selrecv = c->pm_selrecv; *back = c->pm_back;
    return QKM_OK;
}

extern "C" QKM_API int qkm_ep_peer_set(qkm_ctx* c, uint32_t peer, void* xrecv, void* selrecv, void* back) {
    if (!c || !xrecv || !selrecv || !back) return QKM_ERR_ARG;
    if (!c->pm_ranks) return fail(c, QKM_ERR_MODE, "qkm_ep_peer_setup has not been called");
    if (peer >= c->pm_ranks || peer == c->pm_rank) return fail(c, QKM_ERR_ARG, "peer %u is not another rank of %u", peer, c->pm_ranks);
    c->pm_peers.x[peer] = (float*)xrecv; c->pm_peers.sel[peer] = (qkm_sel*)selrecv; c->pm_peers.back[peer] = (float*)back;
    c->pm_peers.flags[peer] = pm_flags_of(c, selrecv);   // every rank uses the same slot_cap, hence the same offset
    return QKM_OK;
}

extern "C" QKM_API int qkm_ep_peer_export(qkm_ctx* c, void* handles) {
    if (!c || !handles) return QKM_ERR_ARG;
    if (!c->pm_ranks) return fail(c, QKM_ERR_MODE, "qkm_ep_peer_setup has not been called");
    static_assert(sizeof(cudaIpcMemHandle_t) == QKM_EP_HANDLE_BYTES / 3, "handle size");
    cudaIpcMemHandle_t h[3];
    QKM_CUDA(c, cudaIpcGetMemHandle(&h[0], c->pm_xrecv));
    QKM_CUDA(c, cudaIpcGetMemHandle(&h[1], c->pm_selrecv));
    QKM_CUDA(c, cudaIpcGetMemHandle(&h[2], c->pm_back));
    memcpy(handles, h, sizeof h);
    return QKM_OK;
}

extern "C" QKM_API int qkm_ep_peer_import(qkm_ctx* c, uint32_t peer, const void* handles) {
    if (!c || !handles) return QKM_ERR_ARG;
    if (!c->pm_ranks) return fail(c, QKM_ERR_MODE, "qkm_ep_peer_setup has not been called");
    if (peer >= c->pm_ranks || peer == c->pm_rank) return fail(c, QKM_ERR_ARG, "peer %u is not another rank of %u", peer, c->pm_ranks);
    if (c->pm_opened[peer][0]) return fail(c, QKM_ERR_MODE, "buffers of rank %u are already mapped", peer);
    cudaIpcMemHandle_t h[3];
    memcpy(h, handles, sizeof h);
    QKM_CUDA(c, cudaSetDevice(c->device));   // the mappings belong to this context's device
    void* p[3] = {};
    for (int i = 0; i < 3; ++i) {
        const cudaError_t e = cudaIpcOpenMemHandle(&p[i], h[i], cudaIpcMemLazyEnablePeerAccess);
        if (e != cudaSuccess) {
            for (int j = 0; j < i; ++j) cudaIpcCloseMemHandle(p[j]);
            cudaGetLastError();
            return fail(c, QKM_ERR_CUDA, "mapping buffer %d of rank %u failed: %s", i, peer, cudaGetErrorString(e));
        }
    }
    for (int i = 0; i < 3; ++i) c->pm_opened[peer][i] = p[i];
    return qkm_ep_peer_set(c, peer, p[0], p[1], p[2]);
}

extern "C" QKM_API int qkm_ep_push(qkm_ctx* c, uint32_t layer, const float* x, uint32_t n, uint32_t slot_rows) {
    if (int rc = layer_ready(c, layer)) return rc;
    if (int rc = pm_check(c, slot_rows)) return rc;
    if (!x && n) return QKM_ERR_ARG;
    if (n > slot_rows) return fail(c, QKM_ERR_BOUNDS, "%u tokens exceed slot_rows %u", n, slot_rows);
    c->shared_plan_n = 0;
    if (n) if (int rc = ep_route_local(c, layer, x, n)) return rc;
    // Layers whose resident experts run on the tensor cores consume the rows as scaled f16: then those
    // travel (half the bytes; every rank decides the same from the layer's types).  The router above
    // has made them already for 128 tokens and more.
    const qkm_layer_dev& ld = c->layers[layer];
    c->pm_rows_f16 = ld.tiles_ok && c->cfg.dims.n_embd % 8 == 0;
    if (c->pm_rows_f16 && n) {
        const float* inv = c->xscale;
        if (n < 128) {   // (the router made digit planes, whose scales sit in xscale for the streamed shared expert)
            if (int rc = ensure_prefill_scratch(c)) return rc;
            QKM_LAUNCH(c, launch_to_f16_rows(c->L(), x, c->xb, c->pm_xscale, n, c->cfg.dims.n_embd));
            inv = c->pm_xscale;
        }
        QKM_LAUNCH(c, launch_ep_push(c->L(), c->cfg.dims, x, c->sel, c->pm_peers, n, slot_rows, c->pm_rank, c->pm_ranks, c->xb, inv));
    } else {
        QKM_LAUNCH(c, launch_ep_push(c->L(), c->cfg.dims, x, c->sel, c->pm_peers, n, slot_rows, c->pm_rank, c->pm_ranks));
    }
    return QKM_OK;
}

extern "C" QKM_API int qkm_ep_forward_slots(qkm_ctx* c, uint32_t layer, uint32_t slot_rows, uint32_t n_shared) {
    if (int rc = pm_check(c, slot_rows)) return rc;
    if (n_shared != QKM_EP_NO_SHARED && n_shared > slot_rows) return fail(c, QKM_ERR_BOUNDS, "%u shared rows exceed slot_rows %u", n_shared, slot_rows);
    const bool with_shared = n_shared != QKM_EP_NO_SHARED;
    c->pm_shared_in_partial = with_shared;
    return ep_expert_forward_impl(c, layer, c->pm_xrecv, c->pm_selrecv, c->pm_ranks * slot_rows, c->pm_partial, with_shared,
                                  c->pm_rank * slot_rows, with_shared ? n_shared : 0, slot_rows,
                                  c->pm_rows_f16 && c->layers[layer].tiles_ok);
}

extern "C" QKM_API int qkm_ep_pull(qkm_ctx* c, uint32_t n, uint32_t slot_rows, float* y) {
    if (int rc = pm_check(c, slot_rows)) return rc;
    if (!y && n) return QKM_ERR_ARG;
    if (n > slot_rows) return fail(c, QKM_ERR_BOUNDS, "%u tokens exceed slot_rows %u", n, slot_rows);
    const bool own = c->pm_shared_in_partial;   // the shared expert came with this rank's partial rows
    QKM_LAUNCH(c, launch_ep_pull(c->L(), c->cfg.dims, c->sel, c->pm_peers, own ? nullptr : c->y2, y, n, slot_rows, c->pm_rank, c->pm_ranks, own));
    return QKM_OK;
}

// Barrier of the ranks as a kernel on the context's stream (ep_barrier_kernel): every rank must
// issue the same sequence of barriers, each rank on its own GPU.  timeout_ms bounds the wait on
// the device; a wait that ran out shows as QKM_ERR_TIMEOUT at the next qkm_sync.
extern "C" QKM_API int qkm_ep_barrier(qkm_ctx* c, uint32_t timeout_ms) {
    if (int rc = pm_check(c, 1)) return rc;
    if (timeout_ms == 0) return fail(c, QKM_ERR_ARG, "the barrier needs a time limit");
    QKM_LAUNCH(c, launch_ep_barrier(c->L(), c->pm_peers, c->pm_rank, c->pm_ranks, ++c->pm_epoch, (uint64_t)timeout_ms * 1000000ull, c->status));
    return QKM_OK;
}

// The whole layer in one call: push, barrier, resident + shared experts, barrier, pull.
extern "C" QKM_API int qkm_ep_peer_layer(qkm_ctx* c, uint32_t layer, const float* x, uint32_t n, uint32_t slot_rows, float* y,
                                         uint32_t timeout_ms) {
    if (int rc = qkm_ep_push(c, layer, x, n, slot_rows)) return rc;
    if (int rc = qkm_ep_barrier(c, timeout_ms)) return rc;
    if (int rc = qkm_ep_forward_slots(c, layer, slot_rows, n)) return rc;   // the shared expert rides with the resident ones
    if (int rc = qkm_ep_barrier(c, timeout_ms)) return rc;
    return qkm_ep_pull(c, n, slot_rows, y);
}
