// Tensor-parallel plumbing: one process per GPU, an NCCL communicator over the GPUs of one
// NVSwitch box. The reference has no multi-GPU code; this is new work behind the same executor
// interface. NCCL is loaded at run time (dlopen) so that the single-GPU library has no
// dependency on it; the rendezvous (sharing the unique id) is the caller's, e.g.
// torch.distributed.
#include "common.cuh"

#include <dlfcn.h>

namespace {

struct Id128 {  // ncclUniqueId: 128 opaque bytes, passed by value
    char bytes[128];
};
struct NcclApi {
    void *lib = nullptr;
    int (*GetUniqueId)(void *) = nullptr;
    int (*CommInitRank)(void **, int, Id128, int) = nullptr;
    int (*AllReduce)(const void *, void *, size_t, int, int, void *, cudaStream_t) = nullptr;
    int (*AllGather)(const void *, void *, size_t, int, void *, cudaStream_t) = nullptr;
    int (*CommDestroy)(void *) = nullptr;
    const char *(*GetErrorString)(int) = nullptr;
};
NcclApi g_nccl;

ctox_status load_nccl(ctox_ctx *ctx, const char *path) {
    if (g_nccl.lib) return CTOX_OK;
    void *lib = dlopen(path && path[0] ? path : "libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
    if (!lib) return ctox::fail(ctx, CTOX_UNSUPPORTED_OPERATION, "cannot load NCCL (%s): %s", path ? path : "libnccl.so.2", dlerror());
#define SYM(field, name)                                                                     \
    *(void **)(&g_nccl.field) = dlsym(lib, name);                                            \
    if (!g_nccl.field) return ctox::fail(ctx, CTOX_UNSUPPORTED_OPERATION, "NCCL symbol %s missing", name)
    SYM(GetUniqueId, "ncclGetUniqueId");
    SYM(CommInitRank, "ncclCommInitRank");
    SYM(AllReduce, "ncclAllReduce");
    SYM(AllGather, "ncclAllGather");
    SYM(CommDestroy, "ncclCommDestroy");
    SYM(GetErrorString, "ncclGetErrorString");
#undef SYM
    g_nccl.lib = lib;
    return CTOX_OK;
}

constexpr int kNcclFloat32 = 7, kNcclInt8 = 0, kNcclSum = 0;

}  // namespace

namespace ctox {

ctox_status tp_all_reduce_sum_f32(ctox_ctx *ctx, float *buf, size_t n) {
    if (ctx->tp_world <= 1) return CTOX_OK;
    const int rc = g_nccl.AllReduce(buf, buf, n, kNcclFloat32, kNcclSum, ctx->nccl_comm, ctx->stream);
    if (rc) return fail(ctx, CTOX_INVALID_STATE, "ncclAllReduce failed: %s", g_nccl.GetErrorString(rc));
    return CTOX_OK;
}

ctox_status tp_all_gather(ctox_ctx *ctx, const void *send, void *recv, size_t bytes_per_rank) {
    if (ctx->tp_world <= 1) {
        if (send != recv) CTOX_CUDA(ctx, cudaMemcpyAsync(recv, send, bytes_per_rank, cudaMemcpyDeviceToDevice, ctx->stream));
        return CTOX_OK;
    }
    const int rc = g_nccl.AllGather(send, recv, bytes_per_rank, kNcclInt8, ctx->nccl_comm, ctx->stream);
    if (rc) return fail(ctx, CTOX_INVALID_STATE, "ncclAllGather failed: %s", g_nccl.GetErrorString(rc));
    return CTOX_OK;
}

}  // namespace ctox

using namespace ctox;

extern "C" {

ctox_status ctox_tp_unique_id(ctox_ctx *ctx, const char *nccl_path, uint8_t *id128) {
    if (!ctx || !id128) return CTOX_INVALID_STATE;
    ctox_status rc = load_nccl(ctx, nccl_path);
    if (rc) return rc;
    const int e = g_nccl.GetUniqueId(id128);
    if (e) return fail(ctx, CTOX_INVALID_STATE, "ncclGetUniqueId failed: %s", g_nccl.GetErrorString(e));
    return CTOX_OK;
}

ctox_status ctox_tp_init(ctox_ctx *ctx, const char *nccl_path, int32_t rank, int32_t world, const uint8_t *id128) {
    if (!ctx || !id128) return CTOX_INVALID_STATE;
    if (world < 1 || rank < 0 || rank >= world) return fail(ctx, CTOX_SHAPE, "tp: rank %d of %d", rank, world);
    if (ctx->nccl_comm) return fail(ctx, CTOX_INVALID_STATE, "tp: communicator already initialised");
    if (world == 1) {
        ctx->tp_rank = 0;
        ctx->tp_world = 1;
        return CTOX_OK;
    }
    ctox_status rc = load_nccl(ctx, nccl_path);
    if (rc) return rc;
    CTOX_CUDA(ctx, cudaSetDevice(ctx->device));
    Id128 id;
    memcpy(id.bytes, id128, 128);
    void *comm = nullptr;
    const int e = g_nccl.CommInitRank(&comm, world, id, rank);
    if (e) return fail(ctx, CTOX_INVALID_STATE, "ncclCommInitRank failed: %s", g_nccl.GetErrorString(e));
    ctx->nccl_comm = comm;
    ctx->tp_rank = rank;
    ctx->tp_world = world;
    return CTOX_OK;
}

ctox_status ctox_tp_destroy(ctox_ctx *ctx) {
    if (!ctx) return CTOX_OK;
    if (ctx->nccl_comm) {
        cudaStreamSynchronize(ctx->stream);
        g_nccl.CommDestroy(ctx->nccl_comm);
        ctx->nccl_comm = nullptr;
    }
    ctx->tp_rank = 0;
    ctx->tp_world = 1;
    return CTOX_OK;
}

/* Device-buffer all-reduce (sum, fp32) over the group: the collective the executor uses,
 * exposed for tests and for callers that shard an operation themselves. */
ctox_status ctox_tp_all_reduce_f32(ctox_ctx *ctx, float *buf_dev, uint64_t n) {
    if (!ctx || !buf_dev) return CTOX_INVALID_STATE;
    return tp_all_reduce_sum_f32(ctx, buf_dev, n);
}

}  // extern "C"
