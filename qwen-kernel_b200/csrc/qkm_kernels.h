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
    void count(int n = 1) const { if (launches) *launches += (uint64_t)n; }
};

// ---- qkm_gemv.cu
cudaError_t launch_dequant(const Launch& L, uint32_t type, const void* blocks, float* y, uint64_t n_elems);
cudaError_t launch_gemv(const Launch& L, uint32_t type, const void* W, const float* x, float* y,
                        uint32_t M, uint32_t K, uint32_t n);

// ---- qkm_route.cu
// Scratch the refined router needs: n_tokens * n_expert f32 logits + n_expert f32 row norms.
size_t route_scratch_bytes(uint32_t n_tokens, uint32_t n_expert);
cudaError_t launch_logits(const Launch& L, const qkm_dims& d, uint32_t router_type, const void* router,
                          const float* x, float* logits, float* row_norm2, uint32_t n_tokens);
cudaError_t launch_select(const Launch& L, const qkm_dims& d, const float* logits, const float* gis,
                          const float* x, qkm_sel* sel, uint32_t n_tokens);
cudaError_t launch_route_select(const Launch& L, const qkm_dims& d, uint32_t router_type,
                                const void* router, const float* gis, const float* x, qkm_sel* sel,
                                uint32_t n_tokens, void* scratch);
cudaError_t launch_group_pairs(const Launch& L, const qkm_dims& d, const qkm_sel* sel, uint32_t n_tokens,
                               uint32_t* offsets, uint32_t* pairs, uint32_t expert_first,
                               uint32_t expert_count);

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
cudaError_t launch_shared_down(const Launch& L, const qkm_dims& d, const void* down, const float* h,
                               const qkm_sel* sel, float* y2, uint32_t n_tokens);
// y[t][o] = sum over slots (in order) of contrib[t][s][o], plus y2[t][o] when y2 != NULL
cudaError_t launch_fold_contrib(const Launch& L, const qkm_dims& d, const float* contrib, const float* y2,
                                float* y, uint32_t n_tokens);

}  // namespace qkm
