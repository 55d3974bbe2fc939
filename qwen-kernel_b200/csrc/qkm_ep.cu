// Expert-parallel exchange helpers: which of this GPU's tokens go to which peer, packing
// the rows to send, and summing the partial results that come back.
//
// Experts are sharded contiguously: rank r of G owns experts [r * n_expert / G, (r + 1) * n_expert / G).
// A token is sent ONCE to every rank that owns at least one of its selected experts (not
// once per expert), together with its selection record; the receiving rank runs its resident
// experts over the received rows and returns one weighted partial row per received token.
// The all-to-all itself is the host's (NCCL); these kernels only prepare and consume its
// buffers, so nothing here waits on another GPU.
//
// Second form, without an all-to-all: every rank's receive buffers are mapped on every rank
// (peer memory over NVLink).  The push kernel stores a token's row and selection record straight
// into the buffers of each rank that owns one of its experts, at a row that depends only on
// (source rank, token), so no counts are exchanged and nothing is packed; the owners store the
// partial rows straight into the source's return buffer the same way (stores are posted, loads
// from a peer are round trips), and the pull kernel sums them from local memory.  Only plain stores and
// loads touch peer memory.  The host orders the phases with a barrier (any collective on the
// stream); these kernels do not wait on anything either.
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "qkm_kernels.h"
#include "qkm_stream.cuh"

namespace qkm {

namespace {

constexpr uint32_t kInvalid = 0xFFFFFFFFu;
constexpr int kPlanThreads = 1024;

// One block.  counts[r] = tokens sent to rank r; send_tok = those tokens, rank by rank, each
// rank's in ascending token order; send_pos[t][r] = row of token t in the send order for
// rank r (kInvalid if t needs nothing from r).  total[0] = sum of counts.
__global__ void __launch_bounds__(kPlanThreads)
ep_plan_kernel(const qkm_sel* __restrict__ sel, uint32_t n_tokens, uint32_t n_used, uint32_t experts_per_rank,
               uint32_t n_ranks, uint32_t* __restrict__ counts, uint32_t* __restrict__ send_tok,
               uint32_t* __restrict__ send_pos) {
    __shared__ uint32_t s_warp[kPlanThreads / 32];
    __shared__ uint32_t s_base;
    const uint32_t tid = threadIdx.x, lane = tid & 31u, warp = tid >> 5;
    if (tid == 0) s_base = 0;
    __syncthreads();
    for (uint32_t r = 0; r < n_ranks; ++r) {
        uint32_t rank_count = 0;
        for (uint32_t t0 = 0; t0 < n_tokens; t0 += kPlanThreads) {
            const uint32_t t = t0 + tid;
            bool need = false;
            if (t < n_tokens)
                for (uint32_t s = 0; s < n_used; ++s) need |= (sel[t].ids[s] / experts_per_rank) == r;
            const uint32_t bal = __ballot_sync(0xFFFFFFFFu, need);
            if (lane == 0) s_warp[warp] = __popc(bal);
            __syncthreads();
            uint32_t before = 0, all = 0;
            for (uint32_t w = 0; w < kPlanThreads / 32; ++w) {
                const uint32_t c = s_warp[w];
                if (w < warp) before += c;
                all += c;
            }
            const uint32_t base = s_base;
            if (t < n_tokens) {
                if (need) {
                    const uint32_t pos = base + rank_count + before + __popc(bal & ((1u << lane) - 1u));
                    send_tok[pos] = t;
                    send_pos[(size_t)t * n_ranks + r] = pos;
                } else {
                    send_pos[(size_t)t * n_ranks + r] = kInvalid;
                }
            }
            rank_count += all;
            __syncthreads();
        }
        if (tid == 0) { counts[r] = rank_count; s_base += rank_count; }
        __syncthreads();
    }
    if (tid == 0) counts[n_ranks] = s_base;
}

// One block per send row (blocks past the total leave): x row and selection record.
__global__ void __launch_bounds__(256)
ep_pack_kernel(const float* __restrict__ x, const qkm_sel* __restrict__ sel, const uint32_t* __restrict__ send_tok,
               const uint32_t* __restrict__ total, float* __restrict__ xsend, qkm_sel* __restrict__ selsend,
               uint32_t n_embd) {
    const uint32_t p = blockIdx.x;
    if (p >= *total) return;
    const uint32_t t = send_tok[p];
    const float4* src = reinterpret_cast<const float4*>(x + (size_t)t * n_embd);
    float4* dst = reinterpret_cast<float4*>(xsend + (size_t)p * n_embd);
    for (uint32_t i = threadIdx.x; i < n_embd / 4; i += blockDim.x) dst[i] = src[i];
    const uint32_t* ss = reinterpret_cast<const uint32_t*>(sel + t);
    uint32_t* sd = reinterpret_cast<uint32_t*>(selsend + p);
    if (threadIdx.x < sizeof(qkm_sel) / 4) sd[threadIdx.x] = ss[threadIdx.x];
}

// y[t] = y2[t] + sum over ranks, in rank order, of the partial row that rank returned for t
__global__ void __launch_bounds__(256)
ep_combine_kernel(const float* __restrict__ back, const uint32_t* __restrict__ send_pos,
                  const float* __restrict__ y2, float* __restrict__ y, uint32_t n_ranks, uint32_t n_embd) {
    const uint32_t t = blockIdx.y;
    const uint32_t o = (blockIdx.x * blockDim.x + threadIdx.x) * 4;
    if (o >= n_embd) return;
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    for (uint32_t r = 0; r < n_ranks; ++r) {
        const uint32_t p = send_pos[(size_t)t * n_ranks + r];
        if (p == kInvalid) continue;
        const float4 c = *reinterpret_cast<const float4*>(back + (size_t)p * n_embd + o);
        v.x += c.x; v.y += c.y; v.z += c.z; v.w += c.w;
    }
    if (y2) {
        const float4 c = *reinterpret_cast<const float4*>(y2 + (size_t)t * n_embd + o);
        v.x += c.x; v.y += c.y; v.z += c.z; v.w += c.w;
    }
    *reinterpret_cast<float4*>(y + (size_t)t * n_embd + o) = v;
}

// One block per slot row i of this rank's region (slot_rows rows on every rank).  Rank d's
// buffers get, at row rank * slot_rows + i: the selection record of token i and its x row if
// token i selected an expert of d; otherwise a record whose ids are all past the expert table,
// which the grouping kernels skip (rows i >= n_tokens are such records on every rank).  This
// rank's own buffers always get the x row, and the weights of the record even when its ids are
// blanked: the shared expert of the local tokens is computed from there.
// With xh (the rows as f16, each scaled by a power of two) the f16 row travels instead - half the
// bytes; it lands at the head of the same row buffer (row r at byte r * n_embd * 2) and the scale
// that undoes the scaling rides in the record's first padding word.  The owner would make exactly
// this conversion from the f32 row, so its results do not change.
__global__ void __launch_bounds__(256)
ep_push_kernel(const float* __restrict__ x, const __half* __restrict__ xh, const float* __restrict__ x_inv_scale,
               const qkm_sel* __restrict__ sel, EpPeerTable peers, uint32_t n_tokens,
               uint32_t slot_rows, uint32_t rank, uint32_t n_ranks, uint32_t n_used, uint32_t experts_per_rank,
               uint32_t n_embd) {
    const uint32_t i = blockIdx.x, tid = threadIdx.x;
    uint32_t need = 0;
    if (i < n_tokens)
        for (uint32_t s = 0; s < n_used; ++s) {
            const uint32_t r = __ldg(&sel[i].ids[s]) / experts_per_rank;
            if (r < n_ranks) need |= 1u << r;
        }
    const size_t row = (size_t)rank * slot_rows + i;
    constexpr uint32_t kWords = sizeof(qkm_sel) / 4;
    if (tid < kWords) {
        uint32_t mine = i < n_tokens ? reinterpret_cast<const uint32_t*>(sel + i)[tid] : 0u;
        if (xh != nullptr && tid == kSelScaleWord && i < n_tokens) mine = __float_as_uint(x_inv_scale[i]);
        const uint32_t empty = tid < 16 ? kInvalid : 0u;
        for (uint32_t d = 0; d < n_ranks; ++d)
            reinterpret_cast<uint32_t*>(peers.sel[d] + row)[tid] = (need >> d & 1u) ? mine : (d == rank && tid >= 16) ? mine : empty;
    }
    if (i >= n_tokens) return;
    const uint32_t dest = need | (1u << rank);
    if (xh != nullptr) {
        const uint4* src = reinterpret_cast<const uint4*>(xh + (size_t)i * n_embd);
        for (uint32_t c = tid; c < n_embd / 8; c += blockDim.x) {
            const uint4 v = __ldg(src + c);
            for (uint32_t d = 0; d < n_ranks; ++d)
                if (dest >> d & 1u) reinterpret_cast<uint4*>(reinterpret_cast<__half*>(peers.x[d]) + row * n_embd)[c] = v;
        }
        return;
    }
    const float4* src = reinterpret_cast<const float4*>(x + (size_t)i * n_embd);
    for (uint32_t c = tid; c < n_embd / 4; c += blockDim.x) {
        const float4 v = __ldg(src + c);
        for (uint32_t d = 0; d < n_ranks; ++d)
            if (dest >> d & 1u) reinterpret_cast<float4*>(peers.x[d] + row * n_embd)[c] = v;
    }
}

// x_inv_scale[r] = the scale that came with row r's record (f16 rows on the wire)
__global__ void ep_row_scales_kernel(const qkm_sel* __restrict__ selrecv, float* __restrict__ x_inv_scale, uint32_t n_rows) {
    const uint32_t r = blockIdx.x * blockDim.x + threadIdx.x;
    if (r < n_rows) x_inv_scale[r] = __uint_as_float(reinterpret_cast<const uint32_t*>(selrecv + r)[kSelScaleWord]);
}

// Slot row (source s, token i) of the local partial rows goes to rank s's return buffer at
// (this rank, i), if a resident expert (or, for the first n_shared own rows, the shared expert)
// contributed to it.  Used where the fold kernel does not store to the peers itself.
__global__ void __launch_bounds__(256)
ep_return_kernel(const float* __restrict__ partial, const qkm_sel* __restrict__ selrecv, EpPeerTable peers,
                 uint32_t slot_rows, uint32_t rank, uint32_t n_used, uint32_t expert_first, uint32_t expert_count,
                 uint32_t n_shared, uint32_t n_embd) {
    const uint32_t r = blockIdx.x, src = r / slot_rows, i = r - src * slot_rows;
    bool live = src == rank && i < n_shared;
    for (uint32_t s = 0; s < n_used; ++s) live |= (__ldg(&selrecv[r].ids[s]) - expert_first) < expert_count;
    if (!live) return;
    const float4* from = reinterpret_cast<const float4*>(partial + (size_t)r * n_embd);
    float4* to = reinterpret_cast<float4*>(peers.back[src] + ((size_t)rank * slot_rows + i) * n_embd);
    for (uint32_t c = threadIdx.x; c < n_embd / 4; c += blockDim.x) to[c] = from[c];
}

// y[t] = y2[t] + sum over the ranks that own one of t's experts, in rank order, of the partial
// row that rank returned for t (row rank d * slot_rows + t of this rank's return buffer).
__global__ void __launch_bounds__(256)
ep_pull_kernel(const qkm_sel* __restrict__ sel, EpPeerTable peers, const float* __restrict__ y2, float* __restrict__ y,
               uint32_t slot_rows, uint32_t rank, uint32_t n_ranks, uint32_t n_used, uint32_t experts_per_rank,
               uint32_t n_embd, uint32_t own_always) {
    const uint32_t t = blockIdx.y;
    const uint32_t o = (blockIdx.x * blockDim.x + threadIdx.x) * 4;
    if (o >= n_embd) return;
    uint32_t need = 0;
    for (uint32_t s = 0; s < n_used; ++s) {
        const uint32_t r = __ldg(&sel[t].ids[s]) / experts_per_rank;
        if (r < n_ranks) need |= 1u << r;
    }
    if (own_always) need |= 1u << rank;   // this rank's partial row carries the shared expert
    const float* back = peers.back[rank];
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    for (uint32_t d = 0; d < n_ranks; ++d) {
        if (!(need >> d & 1u)) continue;
        const float4 c = *reinterpret_cast<const float4*>(back + ((size_t)d * slot_rows + t) * n_embd + o);
        v.x += c.x; v.y += c.y; v.z += c.z; v.w += c.w;
    }
    if (y2) {
        const float4 c = *reinterpret_cast<const float4*>(y2 + (size_t)t * n_embd + o);
        v.x += c.x; v.y += c.y; v.z += c.z; v.w += c.w;
    }
    *reinterpret_cast<float4*>(y + (size_t)t * n_embd + o) = v;
}

// Barrier of the ranks, one launch per rank, each on its own GPU (never two of them on one
// device: they wait for one another).  Barriers are numbered 1, 2, ... in the order every rank
// issues them.  Lane d stores the number into word `rank` of rank d's flag array (release,
// system scope: everything this rank's earlier kernels stored is visible before it); lane s
// then polls word s of this rank's OWN array until rank s has reached the same barrier.  A
// rank that has already gone on to a later barrier leaves a larger number, which also passes.
// The wait is bounded by the device's nanosecond timer: when it runs out the kernel leaves
// kStatusWaitTimeout in the status word and returns.
__global__ void __launch_bounds__(32)
ep_barrier_kernel(EpPeerTable peers, uint32_t rank, uint32_t n_ranks, uint32_t epoch, unsigned long long limit_ns,
                  uint32_t* __restrict__ status) {
    const uint32_t lane = threadIdx.x;
    if (lane >= n_ranks) return;
    __threadfence_system();
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(peers.flags[lane] + rank), "r"(epoch) : "memory");
    const uint32_t* mine = peers.flags[rank] + lane;
    unsigned long long t0, t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
    for (uint32_t polls = 0;; ++polls) {
        uint32_t v;
        asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(mine) : "memory");
        if ((int32_t)(v - epoch) >= 0) break;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
        if (t - t0 > limit_ns) {
            atomicExch(status, (uint32_t)kStatusWaitTimeout);
            break;
        }
        __nanosleep(polls < 64 ? 32 : 256);
    }
}

}  // namespace

cudaError_t launch_ep_barrier(const Launch& L, const EpPeerTable& peers, uint32_t rank, uint32_t n_ranks, uint32_t epoch,
                              uint64_t limit_ns, uint32_t* status) {
    if (n_ranks == 0 || n_ranks > kMaxPeerRanks || rank >= n_ranks || !status) return cudaErrorInvalidValue;
    ep_barrier_kernel<<<1, 32, 0, L.stream>>>(peers, rank, n_ranks, epoch, (unsigned long long)limit_ns, status);
    L.count();
    return cudaGetLastError();
}

cudaError_t launch_ep_row_scales(const Launch& L, const qkm_sel* selrecv, float* x_inv_scale, uint32_t n_rows) {
    if (n_rows == 0) return cudaSuccess;
    ep_row_scales_kernel<<<(n_rows + 255) / 256, 256, 0, L.stream>>>(selrecv, x_inv_scale, n_rows);
    L.count();
    return cudaGetLastError();
}

cudaError_t launch_ep_push(const Launch& L, const qkm_dims& d, const float* x, const qkm_sel* sel, const EpPeerTable& peers,
                           uint32_t n_tokens, uint32_t slot_rows, uint32_t rank, uint32_t n_ranks, const void* xh,
                           const float* x_inv_scale) {
    if (n_ranks == 0 || n_ranks > kMaxPeerRanks || d.n_expert % n_ranks || rank >= n_ranks || n_tokens > slot_rows)
        return cudaErrorInvalidValue;
    if (slot_rows == 0) return cudaSuccess;
    if ((xh != nullptr) != (x_inv_scale != nullptr) || (xh && d.n_embd % 8)) return cudaErrorInvalidValue;
    ep_push_kernel<<<slot_rows, 256, 0, L.stream>>>(x, (const __half*)xh, x_inv_scale, sel, peers, n_tokens, slot_rows, rank, n_ranks, d.n_used,
                                                    d.n_expert / n_ranks, d.n_embd);
    L.count();
    return cudaGetLastError();
}

cudaError_t launch_ep_return(const Launch& L, const qkm_dims& d, const float* partial, const qkm_sel* selrecv,
                             const EpPeerTable& peers, uint32_t slot_rows, uint32_t rank, uint32_t n_ranks, uint32_t n_shared) {
    if (slot_rows == 0 || n_ranks == 0 || n_ranks > kMaxPeerRanks || rank >= n_ranks || d.n_expert % n_ranks) return cudaErrorInvalidValue;
    const uint32_t per = d.n_expert / n_ranks;
    ep_return_kernel<<<n_ranks * slot_rows, 256, 0, L.stream>>>(partial, selrecv, peers, slot_rows, rank, d.n_used, rank * per, per,
                                                                n_shared, d.n_embd);
    L.count();
    return cudaGetLastError();
}

cudaError_t launch_ep_pull(const Launch& L, const qkm_dims& d, const qkm_sel* sel, const EpPeerTable& peers, const float* y2,
                           float* y, uint32_t n_tokens, uint32_t slot_rows, uint32_t rank, uint32_t n_ranks, bool own_always) {
    if (n_ranks == 0 || n_ranks > kMaxPeerRanks || d.n_expert % n_ranks || rank >= n_ranks || n_tokens > slot_rows)
        return cudaErrorInvalidValue;
    if (n_tokens == 0) return cudaSuccess;
    const dim3 grid((d.n_embd / 4 + 255) / 256, n_tokens);
    ep_pull_kernel<<<grid, 256, 0, L.stream>>>(sel, peers, y2, y, slot_rows, rank, n_ranks, d.n_used, d.n_expert / n_ranks,
                                               d.n_embd, own_always ? 1u : 0u);
    L.count();
    return cudaGetLastError();
}

cudaError_t launch_ep_plan(const Launch& L, const qkm_dims& d, const qkm_sel* sel, uint32_t n_tokens, uint32_t n_ranks,
                           uint32_t* counts, uint32_t* send_tok, uint32_t* send_pos) {
    if (n_ranks == 0 || d.n_expert % n_ranks) return cudaErrorInvalidValue;
    ep_plan_kernel<<<1, kPlanThreads, 0, L.stream>>>(sel, n_tokens, d.n_used, d.n_expert / n_ranks, n_ranks, counts,
                                                     send_tok, send_pos);
    L.count();
    return cudaGetLastError();
}

cudaError_t launch_ep_pack(const Launch& L, const qkm_dims& d, const float* x, const qkm_sel* sel,
                           const uint32_t* send_tok, const uint32_t* total, uint32_t max_rows, float* xsend,
                           qkm_sel* selsend) {
    if (max_rows == 0) return cudaSuccess;
    ep_pack_kernel<<<max_rows, 256, 0, L.stream>>>(x, sel, send_tok, total, xsend, selsend, d.n_embd);
    L.count();
    return cudaGetLastError();
}

cudaError_t launch_ep_combine(const Launch& L, const qkm_dims& d, const float* back, const uint32_t* send_pos,
                              const float* y2, float* y, uint32_t n_tokens, uint32_t n_ranks) {
    if (n_tokens == 0) return cudaSuccess;
    const dim3 grid((d.n_embd / 4 + 255) / 256, n_tokens);
    ep_combine_kernel<<<grid, 256, 0, L.stream>>>(back, send_pos, y2, y, n_ranks, d.n_embd);
    L.count();
    return cudaGetLastError();
}

}  // namespace qkm
