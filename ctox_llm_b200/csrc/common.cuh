// Shared host-side plumbing of libctox_b200: context object, error reporting,
// tracked device allocations.
#pragma once

#include <cuda_runtime.h>
#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <string>
#include <utility>
#include <vector>

#include "../../include/ctox_b200.h"

namespace ctox {
struct TpPeer;
}
struct ctox_ctx {
    int device = 0;
    cudaStream_t stream = nullptr;
    bool owns_stream = false;
    int sm_count = 0;
    int max_smem_optin = 0;
    uint64_t allocated = 0;
    int32_t *dev_error = nullptr;   // device error word (kernels set, host reads)
    int32_t *host_error = nullptr;  // pinned mirror
    void *pinned = nullptr;         // pinned staging for the host-form calls
    size_t pinned_bytes = 0;
    void *scratch = nullptr;        // context-owned device scratch of the selection kernels
    size_t scratch_bytes = 0;
    std::string last_error;
    // tensor parallelism: NCCL communicator over the GPUs of one box (tp.cu); world 1 = none
    int tp_rank = 0, tp_world = 1;
    void *nccl_comm = nullptr;
    ctox::TpPeer *tp_peer = nullptr;  // peer-memory all-reduce state (tp.cu); null = NCCL only
    // Limit of the bounded device waits on a peer, in SM clock cycles (~1 s by default).
    long long wait_limit_cycles = 2000000000ll;
    // Test mode: a group whose other ranks never answer (ctox_tp_debug_silent_peers).
    bool tp_silent = false;
    // optional per-kernel timing of the dominant kernel (benchmark support)
    bool timing = false;
    std::vector<std::pair<cudaEvent_t, cudaEvent_t>> timing_events;
};

namespace ctox {

extern thread_local std::string g_create_error;

inline ctox_status fail(ctox_ctx *ctx, ctox_status code, const char *fmt, ...) {
    char buf[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof buf, fmt, ap);
    va_end(ap);
    if (ctx)
        ctx->last_error = buf;
    else
        g_create_error = buf;
    return code;
}

#define CTOX_CUDA(ctx, expr)                                                              \
    do {                                                                                  \
        cudaError_t e_ = (expr);                                                          \
        if (e_ != cudaSuccess)                                                            \
            return ctox::fail((ctx), CTOX_INVALID_STATE, "%s failed: %s", #expr,          \
                              cudaGetErrorString(e_));                                    \
    } while (0)

// Tracked allocation: every byte is accounted on the context so that a caller
// can assert "nothing left" after destroying its handles.
ctox_status dev_alloc(ctox_ctx *ctx, void **ptr, size_t bytes);
void dev_free(ctox_ctx *ctx, void *ptr, size_t bytes);
ctox_status ensure_pinned(ctox_ctx *ctx, size_t bytes);
// Context-owned device scratch (not counted as a caller-visible allocation); grows on demand.
ctox_status ensure_scratch(ctox_ctx *ctx, size_t bytes);
// Collectives over the tensor-parallel group, enqueued on the context's stream (tp.cu).
ctox_status tp_all_reduce_sum_f32(ctox_ctx *ctx, float *buf, size_t n);
ctox_status tp_all_gather(ctox_ctx *ctx, const void *send, void *recv, size_t bytes_per_rank);
// Sets up the peer-memory all-reduce for vectors of up to `elems` floats per rank (buffers and
// flags every rank can address); falls back to NCCL (returns CTOX_OK with ctx->tp_peer null) when
// peer mapping is unavailable or CTOX_TP_P2P=0.
ctox_status tp_peer_init(ctox_ctx *ctx, size_t elems);
void tp_peer_destroy(ctox_ctx *ctx);
// When timing is enabled, brackets the next launches with a CUDA event pair on
// the context's stream; both are no-ops otherwise.
void timing_begin(ctox_ctx *ctx);
void timing_end(ctox_ctx *ctx);

// Programmatic dependent launch. A kernel launched through launch_pdl may begin while the kernel
// before it in the stream is still running; it must execute pdl_wait() before it touches memory
// that earlier work writes or reads (the wait returns once everything earlier in the stream has
// completed and is visible), and EVERY kernel launched this way must execute it, so that
// completion stays transitive along the stream. What a kernel does before the wait (staging its
// own constant weights into shared memory) overlaps the tail of its predecessors.
// pdl_launch() lets the next kernel in the stream be scheduled. CTOX_PDL=0 in the environment
// turns the early start off (every launch then serialises as usual).
bool pdl_enabled();
// Kernels enqueued through launch_pdl / launch_pdl_cluster by this process (every kernel of the
// decode path goes through them); read by ctox_kernel_launches().
void count_launch();
#ifdef __CUDACC__
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st,
                              Args &&...args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = pdl_enabled() ? 1 : 0;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    count_launch();
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// The same with the grid cut into thread-block clusters of cluster_x CTAs along x (the CTAs of a
// cluster can read each other's shared memory).
template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl_cluster(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st,
                                      unsigned cluster_x, Args &&...args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = pdl_enabled() ? 1 : 0;
    attr[1].id = cudaLaunchAttributeClusterDimension;
    attr[1].val.clusterDim.x = cluster_x;
    attr[1].val.clusterDim.y = 1;
    attr[1].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 2;
    count_launch();
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}
#endif

// Device error codes written by kernels into ctx->dev_error.
enum : int32_t {
    DEV_ERR_NONE = 0,
    DEV_ERR_WAIT_TIMEOUT = 1,   // a bounded mbarrier wait ran out
    DEV_ERR_NONFINITE_SCALE = 2,
    DEV_ERR_NONFINITE_VALUE = 3,
};

inline float f16_bits_to_f32(uint16_t h) {
    uint32_t sign = (uint32_t)(h & 0x8000u) << 16, exp = (h >> 10) & 0x1fu, man = h & 0x3ffu, bits;
    if (exp == 0) {
        if (man == 0) {
            bits = sign;
        } else {
            int shift = 0;
            while (!(man & 0x400u)) {
                man <<= 1;
                shift++;
            }
            bits = sign | ((uint32_t)(113 - shift) << 23) | ((man & 0x3ffu) << 13);
        }
    } else if (exp == 31) {
        bits = sign | 0x7f800000u | (man << 13);
    } else {
        bits = sign | ((exp + 112) << 23) | (man << 13);
    }
    float f;
    memcpy(&f, &bits, 4);
    return f;
}

}  // namespace ctox
