// Router logits + top-k selection for callers that may not allocate device memory.
//
// Some hosts hand a library a fixed set of device buffers and forbid anything that takes
// memory from the driver while they run: an inference server that has already given all
// free HBM to its own pool allocator, a real-time loop in which an allocation (which can
// synchronise the whole device) would break its latency bound, or a plugin running inside
// a process whose memory is accounted by someone else.  The context-based entry points
// allocate their scratch when the context is opened.  This one needs no context and takes
// no memory from the driver at all: its scratch is an array that is part of the library
// image and is placed on the device when the library's module is loaded.
//
// Limits: n_tokens * n_expert <= QKM_STATIC_ROUTE_MAX_LOGITS (32768) and
// n_expert <= QKM_STATIC_ROUTE_MAX_EXPERTS (512), e.g. 64 tokens of a 512-expert layer or
// 128 tokens of a 256-expert one.  Larger calls are refused with QKM_ERR_ARG.
//
// The array is one per device and is shared by every call on that device.  Nothing in it
// has to start at zero: each call writes every logit and every row norm it later reads.
// Two calls that overlap in time on one device (different streams, or different host
// threads) race on the array and give wrong selections; callers put such calls on one
// stream or order them with events.
//
// The first call on a device looks the array's address up (and, if the process has not
// used the device yet, lets the runtime create its context and load the module).  That is
// set-up work: make one call per device during start-up, before any stream capture.
// The address is cached per device for the life of the process; a cudaDeviceReset
// invalidates it (a process that resets a device must not call this entry point again).
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include <mutex>

#include "../../include/qk_moe.h"
#include "qkm_kernels.h"

namespace {

constexpr size_t kScratchFloats = (size_t)QKM_STATIC_ROUTE_MAX_LOGITS + QKM_STATIC_ROUTE_MAX_EXPERTS;

// [n_tokens][n_expert] f32 logits followed by [n_expert] squared row norms of the router
static __device__ __align__(256) float g_route_scratch[kScratchFloats];

constexpr int kMaxDevices = 64;
std::mutex g_mu;
void* g_scratch_addr[kMaxDevices] = {};

void put_error(char* err, size_t err_len, const char* what, const char* detail) {
    if (err && err_len) snprintf(err, err_len, "%s%s%s", what, detail ? ": " : "", detail ? detail : "");
}

}  // namespace

extern "C" QKM_API int qkm_route_select_static(int device, void* stream, const qkm_dims* dims,
                                               uint32_t router_type, const void* router,
                                               const float* gate_inp_shexp, const float* x, qkm_sel* sel,
                                               uint32_t n_tokens, char* err, size_t err_len) {
    if (err && err_len) err[0] = 0;
    if (!dims || !router || !gate_inp_shexp || !x || !sel) {
        put_error(err, err_len, "null argument", nullptr);
        return QKM_ERR_ARG;
    }
    if (device < 0 || device >= kMaxDevices) {
        put_error(err, err_len, "device index out of range", nullptr);
        return QKM_ERR_ARG;
    }
    if (router_type != QKM_TYPE_F32 && router_type != QKM_TYPE_F16) {
        put_error(err, err_len, "router must be f32 or f16", nullptr);
        return QKM_ERR_TYPE;
    }
    if (dims->n_expert == 0 || dims->n_expert > QKM_STATIC_ROUTE_MAX_EXPERTS || dims->n_used == 0 ||
        dims->n_used > 16 || dims->n_used > dims->n_expert || dims->n_embd == 0 || dims->n_embd % 256 != 0) {
        put_error(err, err_len, "dimensions outside the static scratch limits (n_expert <= 512, n_embd % 256 == 0)", nullptr);
        return QKM_ERR_ARG;
    }
    if ((uint64_t)n_tokens * dims->n_expert > QKM_STATIC_ROUTE_MAX_LOGITS) {
        put_error(err, err_len, "n_tokens * n_expert exceeds the static scratch (32768 logits)", nullptr);
        return QKM_ERR_ARG;
    }
    if (n_tokens == 0) return QKM_OK;

    int prev = -1;
    cudaError_t e = cudaGetDevice(&prev);
    if (e == cudaSuccess && prev != device) e = cudaSetDevice(device);
    if (e != cudaSuccess) {
        put_error(err, err_len, "selecting the device failed", cudaGetErrorString(e));
        return QKM_ERR_CUDA;
    }
    void* scratch = nullptr;
    {
        std::lock_guard<std::mutex> lk(g_mu);
        if (!g_scratch_addr[device]) {
            void* p = nullptr;
            e = cudaGetSymbolAddress((void**)&p, g_route_scratch);
            if (e == cudaSuccess) g_scratch_addr[device] = p;
        }
        scratch = g_scratch_addr[device];
    }
    int rc = QKM_OK;
    if (e != cudaSuccess || !scratch) {
        put_error(err, err_len, "looking up the static scratch failed", cudaGetErrorString(e));
        rc = QKM_ERR_CUDA;
    } else {
        const qkm::Launch L{(cudaStream_t)stream, nullptr};
        e = qkm::launch_route_select(L, *dims, router_type, router, gate_inp_shexp, x, sel, n_tokens, scratch, kScratchFloats * sizeof(float));
        if (e != cudaSuccess) {
            put_error(err, err_len, "launch failed", cudaGetErrorString(e));
            rc = QKM_ERR_CUDA;
        }
    }
    if (prev >= 0 && prev != device) cudaSetDevice(prev);
    return rc;
}
