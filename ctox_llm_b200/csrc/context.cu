// Context lifecycle and allocation accounting of libctox_b200.
#include <atomic>
#include "common.cuh"

#include <cmath>

namespace ctox {
thread_local std::string g_create_error;

ctox_status dev_alloc(ctox_ctx *ctx, void **ptr, size_t bytes) {
    *ptr = nullptr;
    if (bytes == 0) return CTOX_OK;
    cudaError_t e = cudaMalloc(ptr, bytes);
    if (e != cudaSuccess) {
        cudaGetLastError();
        return fail(ctx, CTOX_MEMORY_BUDGET, "cudaMalloc(%zu) failed: %s", bytes,
                    cudaGetErrorString(e));
    }
    ctx->allocated += bytes;
    return CTOX_OK;
}

void dev_free(ctox_ctx *ctx, void *ptr, size_t bytes) {
    if (!ptr) return;
    cudaFree(ptr);
    ctx->allocated -= bytes;
}

ctox_status ensure_pinned(ctox_ctx *ctx, size_t bytes) {
    if (bytes <= ctx->pinned_bytes) return CTOX_OK;
    if (ctx->pinned) cudaFreeHost(ctx->pinned);
    ctx->pinned = nullptr;
    ctx->pinned_bytes = 0;
    size_t want = bytes < (1u << 20) ? (1u << 20) : bytes;
    CTOX_CUDA(ctx, cudaMallocHost(&ctx->pinned, want));
    ctx->pinned_bytes = want;
    return CTOX_OK;
}
ctox_status ensure_scratch(ctox_ctx *ctx, size_t bytes) {
    if (bytes <= ctx->scratch_bytes) return CTOX_OK;
    if (ctx->scratch) {
        CTOX_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
        cudaFree(ctx->scratch);
    }
    ctx->scratch = nullptr;
    ctx->scratch_bytes = 0;
    const size_t want = bytes < (1u << 20) ? (1u << 20) : bytes;
    cudaError_t e = cudaMalloc(&ctx->scratch, want);
    if (e != cudaSuccess) {
        cudaGetLastError();
        return fail(ctx, CTOX_MEMORY_BUDGET, "cudaMalloc(%zu) failed: %s", want, cudaGetErrorString(e));
    }
    ctx->scratch_bytes = want;
    return CTOX_OK;
}

void timing_begin(ctox_ctx *ctx) {
    if (!ctx->timing) return;
    cudaEvent_t a = nullptr, b = nullptr;
    if (cudaEventCreate(&a) != cudaSuccess || cudaEventCreate(&b) != cudaSuccess) return;
    cudaEventRecord(a, ctx->stream);
    ctx->timing_events.emplace_back(a, b);
}

void timing_end(ctox_ctx *ctx) {
    if (!ctx->timing || ctx->timing_events.empty()) return;
    cudaEventRecord(ctx->timing_events.back().second, ctx->stream);
}
}  // namespace ctox

using namespace ctox;

namespace ctox {
bool pdl_enabled() {
    static const bool on = [] {
        const char *v = getenv("CTOX_PDL");
        return !(v && v[0] == '0');
    }();
    return on;
}
static std::atomic<uint64_t> g_kernel_launches{0};
void count_launch() { g_kernel_launches.fetch_add(1, std::memory_order_relaxed); }
}  // namespace ctox

extern "C" uint64_t ctox_kernel_launches(void) { return ctox::g_kernel_launches.load(std::memory_order_relaxed); }

extern "C" {

uint32_t ctox_abi_version(void) { return 1; }

const char *ctox_backend_profile(void) { return "cuda-sm100a-b200"; }

const char *ctox_last_error_message(const ctox_ctx *ctx) {
    return ctx ? ctx->last_error.c_str() : g_create_error.c_str();
}

ctox_status ctox_ctx_create(int32_t device, void *stream, ctox_ctx **out) {
    if (!out) return fail(nullptr, CTOX_SHAPE, "ctox_ctx_create: out is NULL");
    *out = nullptr;
    int count = 0;
    cudaError_t e = cudaGetDeviceCount(&count);
    if (e != cudaSuccess || count == 0) {
        cudaGetLastError();
        return fail(nullptr, CTOX_UNSUPPORTED_OPERATION,
                    "no CUDA device available (%s); this library has no CPU fallback",
                    e == cudaSuccess ? "device count is 0" : cudaGetErrorString(e));
    }
    if (device < 0 || device >= count)
        return fail(nullptr, CTOX_SHAPE, "device %d out of range (0..%d)", device, count - 1);
    cudaDeviceProp prop;
    CTOX_CUDA(nullptr, cudaGetDeviceProperties(&prop, device));
    if (prop.major != 10)
        return fail(nullptr, CTOX_UNSUPPORTED_OPERATION,
                    "device %d is compute capability %d.%d; this library is built for sm_100a only",
                    device, prop.major, prop.minor);
    CTOX_CUDA(nullptr, cudaSetDevice(device));
    ctox_ctx *ctx = new ctox_ctx();
    ctx->device = device;
    ctx->sm_count = prop.multiProcessorCount;
    ctx->max_smem_optin = (int)prop.sharedMemPerBlockOptin;
    if (stream) {
        ctx->stream = (cudaStream_t)stream;
    } else {
        e = cudaStreamCreateWithFlags(&ctx->stream, cudaStreamNonBlocking);
        if (e != cudaSuccess) {
            delete ctx;
            return fail(nullptr, CTOX_INVALID_STATE, "cudaStreamCreate failed: %s",
                        cudaGetErrorString(e));
        }
        ctx->owns_stream = true;
    }
    if (cudaMalloc(&ctx->dev_error, sizeof(int32_t)) != cudaSuccess ||
        cudaMallocHost(&ctx->host_error, sizeof(int32_t)) != cudaSuccess ||
        cudaMemset(ctx->dev_error, 0, sizeof(int32_t)) != cudaSuccess) {
        ctox_ctx_destroy(ctx);
        return fail(nullptr, CTOX_MEMORY_BUDGET, "context allocation failed");
    }
    *out = ctx;
    return CTOX_OK;
}

ctox_status ctox_ctx_destroy(ctox_ctx *ctx) {
    if (!ctx) return CTOX_OK;
    cudaSetDevice(ctx->device);
    if (ctx->stream) cudaStreamSynchronize(ctx->stream);
    ctox_tp_destroy(ctx);
    for (auto &ev : ctx->timing_events) {
        cudaEventDestroy(ev.first);
        cudaEventDestroy(ev.second);
    }
    if (ctx->dev_error) cudaFree(ctx->dev_error);
    if (ctx->host_error) cudaFreeHost(ctx->host_error);
    if (ctx->pinned) cudaFreeHost(ctx->pinned);
    if (ctx->scratch) cudaFree(ctx->scratch);
    if (ctx->owns_stream && ctx->stream) cudaStreamDestroy(ctx->stream);
    delete ctx;
    return CTOX_OK;
}

ctox_status ctox_ctx_synchronize(ctox_ctx *ctx) {
    if (!ctx) return CTOX_INVALID_STATE;
    CTOX_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    return CTOX_OK;
}

ctox_status ctox_ctx_allocated_bytes(const ctox_ctx *ctx, uint64_t *bytes) {
    if (!ctx || !bytes) return CTOX_INVALID_STATE;
    *bytes = ctx->allocated;
    return CTOX_OK;
}

ctox_status ctox_ctx_kernel_timing(ctox_ctx *ctx, int32_t enable) {
    if (!ctx) return CTOX_INVALID_STATE;
    ctx->timing = enable != 0;
    return CTOX_OK;
}

ctox_status ctox_ctx_kernel_timing_read(ctox_ctx *ctx, double *total_ms, uint64_t *launches) {
    if (!ctx || !total_ms || !launches) return CTOX_INVALID_STATE;
    CTOX_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    double sum = 0.0;
    uint64_t n = 0;
    for (auto &ev : ctx->timing_events) {
        float ms = 0.f;
        if (cudaEventElapsedTime(&ms, ev.first, ev.second) == cudaSuccess) {
            sum += ms;
            ++n;
        }
        cudaEventDestroy(ev.first);
        cudaEventDestroy(ev.second);
    }
    ctx->timing_events.clear();
    *total_ms = sum;
    *launches = n;
    return CTOX_OK;
}

ctox_status ctox_ctx_device_error(ctox_ctx *ctx, int32_t *code) {
    if (!ctx || !code) return CTOX_INVALID_STATE;
    CTOX_CUDA(ctx, cudaMemcpyAsync(ctx->host_error, ctx->dev_error, sizeof(int32_t),
                                   cudaMemcpyDeviceToHost, ctx->stream));
    CTOX_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    *code = *ctx->host_error;
    if (*code != 0)
        CTOX_CUDA(ctx, cudaMemsetAsync(ctx->dev_error, 0, sizeof(int32_t), ctx->stream));
    return CTOX_OK;
}

}  // extern "C"
