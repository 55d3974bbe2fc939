// Decode-sized batches (<= 64 tokens): router logits, top-k selection and the activation rows as
// int8 digit planes, in one launch.  (The token-expert grouping happens at the start of the
// gate/up kernel, in every block's own shared memory: qkm_dec_rank.cuh.)
//
// Replaces, for the fused decode sequence, moe_logits.comp + moe_select_256.comp, i.e. their
// fused form moe_route_select.comp.  Two kinds of blocks share the grid:
//   * logits blocks: two router rows and eight tokens each, f64 accumulation - the logits are
//     those of the CPU reference's f64 router (src/main.cpp:1320-1324) up to the order of the
//     f64 additions, so they are ranked as they are, without an error bound; the block that
//     finishes a group of eight tokens last ranks them, one warp per token;
//   * one block per token encodes x as digit planes (and their negatives, which the IQ3_XXS
//     kernel multiplies with its sign masks) and evaluates the shared expert's gate
//     sigmoid(gis . x) in f64 (moe_select.comp's wShared).
#include "qkm_common.cuh"
#include "qkm_dec_rank.cuh"
#include "qkm_kernels.h"
#include "qkm_stream.cuh"

namespace qkm {

namespace rd {
constexpr int kThreads = 256;
constexpr int kTok = 8;           // tokens per logits block
}  // namespace rd

// digit planes of one row, layout [kb][8][256]: planes 0..3 the digits, 4..7 their negatives
__device__ __forceinline__ void store_planes8(int8_t* __restrict__ pl, uint32_t k, uint32_t dgt) {
    int8_t* q = pl + (size_t)(k >> 8) * 2048 + (k & 255u);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const int dj = (int)(int8_t)((dgt >> (8 * j)) & 255u);
        q[256 * j] = (int8_t)dj;
        q[256 * (j + 4)] = (int8_t)(-dj);
    }
}

template <int TYPE>
__global__ void __launch_bounds__(rd::kThreads, 2)
route_decode_kernel(RouteDecodeArgs a) {
    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31u;
    const qkm_dims d = a.d;
    const uint32_t T = a.n_tokens;
    const uint32_t n_pair_blocks = (d.n_expert + 1) / 2;                              // blocks along the experts
    const uint32_t n_logit_blocks = n_pair_blocks * ((T + rd::kTok - 1) / rd::kTok);  // times the token groups

    // x is the output of the kernel before; the selection, planes and logits written here are still
    // read by the previous layer's kernels until that kernel has ended
    pdl_wait();
    pdl_trigger();

    if (blockIdx.x >= n_logit_blocks) {
        // ---- one token: digit planes + shared gate ----------------------------------------------
        __shared__ float s_xm[8];
        __shared__ double s_sg[8];
        const uint32_t t = blockIdx.x - n_logit_blocks;
        const float* xt = a.x + (size_t)t * d.n_embd;
        float v[16];   // n_embd <= 4096
        float xm = 0.f;
        double dsg = 0.0;
        bool bad = false;
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            const uint32_t k = tid + 256 * i;
            v[i] = k < d.n_embd ? xt[k] : 0.f;
            xm = fmaxf(xm, fabsf(v[i]));
            bad |= !(fabsf(v[i]) <= 3.0e38f);
            if (k < d.n_embd) dsg += (double)a.gis[k] * (double)v[i];
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) xm = fmaxf(xm, __shfl_xor_sync(0xFFFFFFFFu, xm, o));
        dsg = warp_sum(dsg);
        const int any_bad = __syncthreads_or(bad ? 1 : 0);
        if (lane == 0) { s_xm[warp] = xm; s_sg[warp] = dsg; }
        __syncthreads();
        if (tid == 0) {
            double sg = 0.0;
#pragma unroll
            for (int w = 0; w < 8; ++w) sg += s_sg[w];
            a.sel[t].w_shared = (float)(1.0 / (1.0 + exp(-sg)));
        }
        float xmax = 0.f;
#pragma unroll
        for (int w = 0; w < 8; ++w) xmax = fmaxf(xmax, s_xm[w]);
        const int p = digit_exponent(xmax);
        const float up = ldexpf(1.0f, p);
        int8_t* pl = a.planes + (size_t)t * 8 * d.n_embd;
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            const uint32_t k = tid + 256 * i;
            if (k < d.n_embd) store_planes8(pl, k, any_bad ? 0u : digits4(__float2int_rn(v[i] * up)));
        }
        if (tid == 0) a.xscale[t] = any_bad ? __int_as_float(0x7FC00000) : ldexpf(1.0f, -p);
        return;
    }

    // ---- logits of two experts for kTok tokens ------------------------------------------------------
    // warp w owns the w-th eighth of the columns; a lane loads one 8-element unit of both router
    // rows and the matching x values of the block's tokens in one go
    __shared__ double s_part[8][2 * rd::kTok];
    const uint32_t e0 = (blockIdx.x % n_pair_blocks) * 2u, t0 = (blockIdx.x / n_pair_blocks) * rd::kTok;
    const bool two = e0 + 1 < d.n_expert;
    const size_t rb = row_bytes(TYPE, d.n_embd);
    const uint8_t* row0 = a.router + (size_t)e0 * rb;
    const uint8_t* row1 = a.router + (size_t)(two ? e0 + 1 : e0) * rb;
    const uint32_t units_w = d.n_embd / 64;   // 8-element units per warp
    {
        double acc[2 * rd::kTok];   // [expert 0: tokens][expert 1: tokens]
#pragma unroll
        for (int j = 0; j < 2 * rd::kTok; ++j) acc[j] = 0.0;
        for (uint32_t u = lane; u < units_w; u += 32) {
            const uint32_t k = (warp * units_w + u) * 8;
            float w0[8], w1[8];
            dequant8<TYPE>(row0, k, w0);
            dequant8<TYPE>(row1, k, w1);
            float4 xa[rd::kTok], xb[rd::kTok];
#pragma unroll
            for (int j = 0; j < rd::kTok; ++j) {
                const uint32_t tt = min(t0 + j, T - 1);
                const float* xt = a.x + (size_t)tt * d.n_embd + k;
                xa[j] = *reinterpret_cast<const float4*>(xt);
                xb[j] = *reinterpret_cast<const float4*>(xt + 4);
            }
#pragma unroll
            for (int j = 0; j < rd::kTok; ++j) {
                const double x0 = xa[j].x, x1 = xa[j].y, x2 = xa[j].z, x3 = xa[j].w;
                const double x4 = xb[j].x, x5 = xb[j].y, x6 = xb[j].z, x7 = xb[j].w;
                double s = acc[j];
                s += (double)w0[0] * x0; s += (double)w0[1] * x1; s += (double)w0[2] * x2; s += (double)w0[3] * x3;
                s += (double)w0[4] * x4; s += (double)w0[5] * x5; s += (double)w0[6] * x6; s += (double)w0[7] * x7;
                acc[j] = s;
                s = acc[rd::kTok + j];
                s += (double)w1[0] * x0; s += (double)w1[1] * x1; s += (double)w1[2] * x2; s += (double)w1[3] * x3;
                s += (double)w1[4] * x4; s += (double)w1[5] * x5; s += (double)w1[6] * x6; s += (double)w1[7] * x7;
                acc[rd::kTok + j] = s;
            }
        }
        // reduce-scatter over the warp: after the step with distance o a lane keeps the half of its
        // values selected by (lane & o); 16 values, distances 16..2 halve them to one, distance 1 finishes it
#pragma unroll
        for (int o = 16, n = 2 * rd::kTok; o >= 2; o >>= 1, n >>= 1) {
            const bool up = (lane & o) != 0;
#pragma unroll
            for (int j = 0; j < n / 2; ++j) {
                const double send = up ? acc[j] : acc[j + n / 2];
                const double keep = up ? acc[j + n / 2] : acc[j];
                acc[j] = keep + __shfl_xor_sync(0xFFFFFFFFu, send, o);
            }
        }
        const double v = acc[0] + __shfl_xor_sync(0xFFFFFFFFu, acc[0], 1);
        // lane l holds value index: bit 3 from (l & 16), bit 2 from (l & 8), bit 1 from (l & 4), bit 0 from (l & 2)
        if ((lane & 1u) == 0) s_part[warp][(lane >> 1) & 15u] = v;
    }
    __syncthreads();
    if (tid < 2 * rd::kTok) {
        const uint32_t r = tid / rd::kTok, j = tid % rd::kTok;
        double v = 0.0;
#pragma unroll
        for (int w = 0; w < 8; ++w) v += s_part[w][tid];
        if (t0 + j < T && (r == 0 || two)) a.logits[(size_t)(t0 + j) * d.n_expert + e0 + r] = v;
    }

    // ---- the block that finishes a token group's logits last ranks the group's tokens ---------------
    // (a ticket counter per group; writes are fenced before the ticket, reads after it - the
    // device-scope release/acquire the reference's fused router relies on, moe_route_select.comp:56-67)
    __shared__ uint32_t s_last;
    uint32_t* counter = a.counter + blockIdx.x / n_pair_blocks;
    __threadfence();
    __syncthreads();
    if (tid == 0) s_last = atomicAdd(counter, 1u) == n_pair_blocks - 1 ? 1u : 0u;
    __syncthreads();
    if (!s_last) return;
    if (tid == 0) *counter = 0;   // ready for the next launch
    __threadfence();
    rank_tokens(a.logits, a.sel, d, t0, min((uint32_t)rd::kTok, T - t0), rd::kThreads / 32);
}

bool route_decode_ok(const qkm_dims& d, uint32_t n_tokens, size_t scratch_bytes) {
    return n_tokens > 0 && n_tokens <= 64 && d.n_expert <= 512 && d.n_used <= 16 && d.n_embd <= 4096 && d.n_embd % 64 == 0 &&
           (size_t)n_tokens * d.n_expert * sizeof(double) <= scratch_bytes;
}

cudaError_t launch_route_decode(const Launch& L, uint32_t router_type, const RouteDecodeArgs& a) {
    if (router_type != QKM_TYPE_F32 && router_type != QKM_TYPE_F16) return cudaErrorInvalidValue;
    if (a.n_tokens == 0 || a.n_tokens > 64 || a.d.n_expert > 512 || a.d.n_embd > 4096) return cudaErrorInvalidValue;
    const dim3 grid((a.d.n_expert + 1) / 2 * ((a.n_tokens + rd::kTok - 1) / rd::kTok) + a.n_tokens);
    cudaError_t e;
    if (router_type == QKM_TYPE_F32)
        e = launch_kernel(L, route_decode_kernel<QKM_TYPE_F32>, grid, dim3(rd::kThreads), 0, a);
    else
        e = launch_kernel(L, route_decode_kernel<QKM_TYPE_F16>, grid, dim3(rd::kThreads), 0, a);
    L.count();
    return e != cudaSuccess ? e : cudaGetLastError();
}

}  // namespace qkm
