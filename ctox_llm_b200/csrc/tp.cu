// Tensor-parallel plumbing: one process per GPU, an NCCL communicator over the GPUs of one
// NVSwitch box. The reference has no multi-GPU code; this is new work behind the same executor
// interface. NCCL is loaded at run time (dlopen) so that the single-GPU library has no
// dependency on it; the rendezvous (sharing the unique id) is the caller's, e.g.
// torch.distributed.
#include "common.cuh"
#include "layers.cuh"

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
    if (ctx->tp_world <= 1 || ctx->tp_silent) return CTOX_OK;
    const int rc = g_nccl.AllReduce(buf, buf, n, kNcclFloat32, kNcclSum, ctx->nccl_comm, ctx->stream);
    if (rc) return fail(ctx, CTOX_INVALID_STATE, "ncclAllReduce failed: %s", g_nccl.GetErrorString(rc));
    return CTOX_OK;
}

ctox_status tp_all_gather(ctox_ctx *ctx, const void *send, void *recv, size_t bytes_per_rank) {
    if (ctx->tp_silent) {  // the other ranks never answer: their slots read as zeros
        uint8_t *own = (uint8_t *)recv + (size_t)ctx->tp_rank * bytes_per_rank;
        if (send != own) CTOX_CUDA(ctx, cudaMemcpyAsync(own, send, bytes_per_rank, cudaMemcpyDeviceToDevice, ctx->stream));
        for (int r = 0; r < ctx->tp_world; ++r)
            if (r != ctx->tp_rank)
                CTOX_CUDA(ctx, cudaMemsetAsync((uint8_t *)recv + (size_t)r * bytes_per_rank, 0, bytes_per_rank, ctx->stream));
        return CTOX_OK;
    }
    if (ctx->tp_world <= 1) {
        if (send != recv) CTOX_CUDA(ctx, cudaMemcpyAsync(recv, send, bytes_per_rank, cudaMemcpyDeviceToDevice, ctx->stream));
        return CTOX_OK;
    }
    const int rc = g_nccl.AllGather(send, recv, bytes_per_rank, kNcclInt8, ctx->nccl_comm, ctx->stream);
    if (rc) return fail(ctx, CTOX_INVALID_STATE, "ncclAllGather failed: %s", g_nccl.GetErrorString(rc));
    return CTOX_OK;
}

}  // namespace ctox

// ------------------------------------------------------------------ one-shot all-reduce over peer memory
// The sum of a column-split projection over the group without a library collective, in the
// low-latency style: every rank PUSHES its finished partial vector into a receive buffer in each
// peer's memory as 8-byte words {value, sequence number}; an 8-byte store is single-copy atomic,
// so the word itself says when it has arrived and no fence or separate flag is needed. The
// residual kernel of every rank polls its own (local) receive buffer, one word per source rank and
// element, and adds the W values in rank order: all ranks get identical bits, and the residual add,
// the sum over the group and the partial sums of squares are one kernel. Plain peer stores over
// NVLink only (no multicast, no reads of peer memory). Waits are bounded: a peer that never
// delivers makes the kernel set the device error word and carry on.
namespace ctox {

constexpr uint32_t kTpChunk = 256, kTpMaxWorld = 8;

struct TpPeer {
    uint32_t world = 0, rank = 0, seq = 0;
    size_t elems = 0;          // floats per vector
    uint2 *recv = nullptr;     // own: [2 parities][world sources][elems] of {value bits, seq}
    uint2 *peer_recv[kTpMaxWorld] = {nullptr};
    uint2 *sink = nullptr;     // test mode only: where pushes to the silent peers go
};
struct TpPeerPtrs {  // by value into the kernels: where each rank receives THIS rank's vector
    uint2 *dst[kTpMaxWorld];
};

// One aligned 64-bit scalar access (single-copy atomic): low word = value bits, high word = seq.
__device__ __forceinline__ void st_word_sys(uint2 *p, uint32_t value, uint32_t seq) {
    const unsigned long long w = ((unsigned long long)seq << 32) | value;
    asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(p), "l"(w) : "memory");
}
__device__ __forceinline__ uint2 ld_word_sys(const uint2 *p) {
    unsigned long long w;
    asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(w) : "l"(p) : "memory");
    return make_uint2((uint32_t)w, (uint32_t)(w >> 32));
}

// One kernel per sum: y[pos][row] of this rank's partial result goes to every PEER's receive slot
// for this rank; then the same thread collects the peers' values for its (row, position) from this
// rank's own receive buffer and adds all W values to h in rank order (its own from the register:
// the same bits the peers receive). Pushes never wait, so two ranks cannot wait on each other
// without one of them having pushed. Partial sums of squares of the result per 256-column part,
// like k_residual_add.
// This thread's (column c, position m): push the rank's own partial value to every peer, collect the
// peers' values and return h + the sum over the group in rank order (h is rewritten).
__device__ __forceinline__ float tp_push_collect(const MvOut &o, const OutRef &oref, float *__restrict__ h,
                                                 const TpPeerPtrs &peers,
                                                 const uint2 *recv, size_t source_stride, uint32_t rank,
                                                 uint32_t world, uint32_t seq, uint32_t hidden, uint32_t c, int m,
                                                 int32_t *error_flag, long long wait_limit) {
    const float mine = out_at(o, oref, c, m);
    const size_t at = (size_t)m * hidden + c;
    // (unrolled with predicates: a run-time index into the by-value pointer table would copy it
    // to the local-memory stack first)
#pragma unroll
    for (uint32_t r = 0; r < kTpMaxWorld; ++r)
        if (r < world && r != rank) st_word_sys(peers.dst[r] + at, __float_as_uint(mine), seq);
    float v = h[at];
    const long long t0 = clock64();
    // once a wait has run out anywhere (this kernel or an earlier one of the same call), nobody
    // waits again: the call is lost anyway and the kernels behind it must not each spend the limit
    bool gave_up = *reinterpret_cast<volatile int32_t *>(error_flag) != 0;
    for (uint32_t r = 0; r < world; ++r) {
        if (r == rank) {
            v += mine;
            continue;
        }
        const uint2 *p = recv + r * source_stride + at;
        uint2 word = ld_word_sys(p);
        while (word.y != seq && !gave_up) {
            if (clock64() - t0 > wait_limit) {  // a peer is gone
                atomicExch(error_flag, DEV_ERR_WAIT_TIMEOUT);
                gave_up = true;
                break;
            }
            if (*reinterpret_cast<volatile int32_t *>(error_flag) != 0) gave_up = true;
            word = ld_word_sys(p);
        }
        v += __uint_as_float(word.x);
    }
    h[at] = v;
    return v;
}

__global__ void __launch_bounds__(kTpChunk) k_tp_reduce_residual(MvOut o, float *__restrict__ h, TpPeerPtrs peers,
                                                               const uint2 *recv, size_t source_stride,
                                                               uint32_t rank, uint32_t world, uint32_t seq,
                                                               uint32_t hidden, float *__restrict__ sumsq,
                                                               int32_t *error_flag, long long wait_limit) {
    pdl_launch();
    __shared__ float red[kTpChunk / 32];
    const int m = blockIdx.y;
    const uint32_t c = blockIdx.x * kTpChunk + threadIdx.x;
    const OutRef oref = c < hidden ? out_ref(o, c) : OutRef{nullptr, 0, 0, 1.0f, false};
    pdl_wait();
    float v = 0.f;
    if (c < hidden)
        v = tp_push_collect(o, oref, h, peers, recv, source_stride, rank, world, seq, hidden, c, m, error_flag, wait_limit);
    float s = v * v;
#pragma unroll
    for (int o2 = 16; o2 > 0; o2 >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o2);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = s;
    __syncthreads();
    if (threadIdx.x == 0) {
        float t = 0.f;
        for (unsigned w = 0; w < kTpChunk / 32; ++w) t += red[w];  // fixed order
        sumsq[m * gridDim.x + blockIdx.x] = t;
    }
}

// The same, then the RMS norm of the new residual and the next projection's fragments without a
// kernel boundary: a thread-block cluster of kRnCluster CTAs per position (residual_norm_finish).
// A wait that runs out leaves v undefined but every thread still reaches the cluster barriers.
__global__ void __launch_bounds__(kRnColumns / kRnCluster, 1) k_tp_reduce_residual_norm_prep(
    MvOut o, float *__restrict__ h, TpPeerPtrs peers, const uint2 *recv, size_t source_stride, uint32_t rank,
    uint32_t world, uint32_t seq, uint32_t hidden, int32_t *error_flag, long long wait_limit,
    const float *__restrict__ w, float eps, int npos, float *__restrict__ xn_out, MvIn next, int has_next,
    uint32_t nblocks) {
    pdl_launch();
    const int m = blockIdx.y;
    const uint32_t c = blockIdx.x * (kRnColumns / kRnCluster) + threadIdx.x;
    const float wc = c < hidden ? w[c] : 0.f;  // constants first: they do not depend on earlier kernels
    const float sc = (has_next && next.s_in && c < hidden) ? next.s_in[c] : 1.0f;
    const OutRef oref = c < hidden ? out_ref(o, c) : OutRef{nullptr, 0, 0, 1.0f, false};
    pdl_wait();
    float v = 0.f;
    if (c < hidden)
        v = tp_push_collect(o, oref, h, peers, recv, source_stride, rank, world, seq, hidden, c, m, error_flag, wait_limit);
    residual_norm_finish<kRnCluster>(v, hidden, wc, sc, eps, m, npos, xn_out, next, has_next, nblocks);
}

ctox_status tp_peer_init(ctox_ctx *ctx, size_t elems) {
    if (ctx->tp_world <= 1 || ctx->tp_peer) return CTOX_OK;
    const char *env = getenv("CTOX_TP_P2P");
    if (env && env[0] == '0') return CTOX_OK;
    const uint32_t W = (uint32_t)ctx->tp_world, R = (uint32_t)ctx->tp_rank;
    if (W > kTpMaxWorld) return CTOX_OK;
    TpPeer *tp = new TpPeer();
    tp->world = W;
    tp->rank = R;
    tp->elems = elems;
    const size_t bytes = 2 * (size_t)W * elems * sizeof(uint2);
    if (ctx->tp_silent) {
        // test mode: this rank's pushes land in a local sink, nothing is ever pushed to it
        uint2 *sink = nullptr;
        if (cudaMalloc((void **)&tp->recv, bytes) != cudaSuccess || cudaMemset(tp->recv, 0, bytes) != cudaSuccess ||
            cudaMalloc((void **)&sink, bytes) != cudaSuccess) {
            cudaFree(tp->recv);
            delete tp;
            cudaGetLastError();
            return fail(ctx, CTOX_MEMORY_BUDGET, "tp: no memory for the silent-peer buffers");
        }
        for (uint32_t r = 0; r < W; ++r) tp->peer_recv[r] = r == R ? tp->recv : sink;
        tp->sink = sink;
        ctx->tp_peer = tp;
        return CTOX_OK;
    }
    struct Card {
        cudaIpcMemHandle_t recv;
        int ok;
    } mine{}, all[kTpMaxWorld];
    bool ok = cudaMalloc((void **)&tp->recv, bytes) == cudaSuccess && cudaMemset(tp->recv, 0, bytes) == cudaSuccess &&
              cudaIpcGetMemHandle(&mine.recv, tp->recv) == cudaSuccess;
    mine.ok = ok ? 1 : 0;
    // exchange the cards through the communicator the group already has
    Card *dev = nullptr;
    ctox_status rc = CTOX_OK;
    if (cudaMalloc((void **)&dev, sizeof(Card) * (W + 1)) != cudaSuccess) {
        rc = fail(ctx, CTOX_MEMORY_BUDGET, "tp: no memory for the peer exchange");
    } else {
        if (cudaMemcpyAsync(dev + W, &mine, sizeof(Card), cudaMemcpyHostToDevice, ctx->stream) != cudaSuccess)
            rc = fail(ctx, CTOX_INVALID_STATE, "tp: peer exchange failed (upload)");
        if (!rc) rc = tp_all_gather(ctx, dev + W, dev, sizeof(Card));
        if (!rc && (cudaMemcpyAsync(all, dev, sizeof(Card) * W, cudaMemcpyDeviceToHost, ctx->stream) != cudaSuccess ||
                    cudaStreamSynchronize(ctx->stream) != cudaSuccess))
            rc = fail(ctx, CTOX_INVALID_STATE, "tp: peer exchange failed (download)");
        cudaFree(dev);
    }
    if (rc) {
        cudaFree(tp->recv);
        delete tp;
        return rc;
    }
    for (uint32_t r = 0; r < W && ok; ++r) ok = all[r].ok != 0;
    for (uint32_t r = 0; r < W && ok; ++r) {
        if (r == R) {
            tp->peer_recv[r] = tp->recv;
            continue;
        }
        ok = cudaIpcOpenMemHandle((void **)&tp->peer_recv[r], all[r].recv, cudaIpcMemLazyEnablePeerAccess) == cudaSuccess;
    }
    // every rank must take the same path: agree through one more exchange
    int agree = ok ? 1 : 0, *agree_dev = nullptr, votes[kTpMaxWorld] = {0};
    if (cudaMalloc((void **)&agree_dev, sizeof(int) * (W + 1)) == cudaSuccess) {
        // a failed copy leaves the votes at zero: every rank then falls back to NCCL together
        if (cudaMemcpyAsync(agree_dev + W, &agree, sizeof(int), cudaMemcpyHostToDevice, ctx->stream) == cudaSuccess &&
            !tp_all_gather(ctx, agree_dev + W, agree_dev, sizeof(int))) {
            int got[kTpMaxWorld] = {0};
            if (cudaMemcpyAsync(got, agree_dev, sizeof(int) * W, cudaMemcpyDeviceToHost, ctx->stream) == cudaSuccess &&
                cudaStreamSynchronize(ctx->stream) == cudaSuccess)
                memcpy(votes, got, sizeof(int) * W);
        }
        cudaFree(agree_dev);
    }
    for (uint32_t r = 0; r < W; ++r) ok = ok && votes[r] == 1;
    cudaGetLastError();  // a refused mapping is not an error of the context: NCCL serves instead
    ctx->tp_peer = tp;
    if (!ok) tp_peer_destroy(ctx);
    return CTOX_OK;
}

void tp_peer_destroy(ctox_ctx *ctx) {
    TpPeer *tp = ctx->tp_peer;
    if (!tp) return;
    cudaStreamSynchronize(ctx->stream);
    for (uint32_t r = 0; r < tp->world; ++r)
        if (!tp->sink && r != tp->rank && tp->peer_recv[r]) cudaIpcCloseMemHandle(tp->peer_recv[r]);
    if (tp->sink) cudaFree(tp->sink);
    if (tp->recv) cudaFree(tp->recv);
    delete tp;
    ctx->tp_peer = nullptr;
}

// Enqueues "h += sum over the group of this matvec's output" for m positions through peer memory.
// Receive buffers alternate with the parity of the sequence number: a rank's next-but-one push runs
// after its own next residual kernel, which has consumed every peer's next push, which those peers
// issued after consuming the current one.
ctox_status tp_peer_reduce_add(ctox_ctx *ctx, const MvOut &o, uint32_t rows, uint32_t m, float *h, float *sumsq) {
    TpPeer *tp = ctx->tp_peer;
    if (!tp) return fail(ctx, CTOX_INVALID_STATE, "tp: peer all-reduce is not set up");
    if ((size_t)m * rows > tp->elems) return fail(ctx, CTOX_SHAPE, "tp: vector of %u x %u exceeds the peer buffer", m, rows);
    const uint32_t seq = ++tp->seq, parity = seq & 1;
    if (seq == 0) return fail(ctx, CTOX_INVALID_STATE, "tp: sequence numbers exhausted");
    const uint32_t chunks = (rows + kTpChunk - 1) / kTpChunk;
    const size_t parity_off = (size_t)parity * tp->world * tp->elems;
    TpPeerPtrs pp{};
    for (uint32_t r = 0; r < tp->world; ++r) pp.dst[r] = tp->peer_recv[r] + parity_off + (size_t)tp->rank * tp->elems;
    launch_pdl(k_tp_reduce_residual, dim3(chunks, m), dim3(kTpChunk), 0, ctx->stream, o, h, pp, tp->recv + parity_off,
               tp->elems, tp->rank, tp->world, seq, rows, sumsq, ctx->dev_error, ctx->wait_limit_cycles);
    CTOX_CUDA(ctx, cudaGetLastError());
    return CTOX_OK;
}

bool tp_peer_reduce_add_norm_fits(uint32_t rows, const MvIn *next) {
    static const bool merged = [] {
        const char *v = getenv("CTOX_MERGED_NORM");
        return !(v && v[0] == '0');
    }();
    const uint32_t nblocks = next ? next->blocks_padded : (rows + 63) / 64;
    return merged && rows <= (uint32_t)kRnColumns && nblocks <= (uint32_t)kRnColumns / 64;
}

ctox_status tp_peer_reduce_add_norm(ctox_ctx *ctx, const MvOut &o, uint32_t rows, uint32_t m, float *h,
                                    const float *w, float eps, float *xn_out, const MvIn *next) {
    TpPeer *tp = ctx->tp_peer;
    if (!tp) return fail(ctx, CTOX_INVALID_STATE, "tp: peer all-reduce is not set up");
    if ((size_t)m * rows > tp->elems) return fail(ctx, CTOX_SHAPE, "tp: vector of %u x %u exceeds the peer buffer", m, rows);
    if (!tp_peer_reduce_add_norm_fits(rows, next)) return fail(ctx, CTOX_SHAPE, "tp: %u rows do not fit the merged kernel", rows);
    const uint32_t seq = ++tp->seq, parity = seq & 1;
    if (seq == 0) return fail(ctx, CTOX_INVALID_STATE, "tp: sequence numbers exhausted");
    const size_t parity_off = (size_t)parity * tp->world * tp->elems;
    TpPeerPtrs pp{};
    for (uint32_t r = 0; r < tp->world; ++r) pp.dst[r] = tp->peer_recv[r] + parity_off + (size_t)tp->rank * tp->elems;
    const MvIn n = next ? *next : MvIn{nullptr, nullptr, nullptr, 0, 0, 0};
    const uint32_t nblocks = next ? next->blocks_padded : (rows + 63) / 64;
    launch_pdl_cluster(k_tp_reduce_residual_norm_prep, dim3(kRnCluster, m), dim3(kRnColumns / kRnCluster), 0, ctx->stream,
                       kRnCluster, o, h, pp, tp->recv + parity_off, tp->elems, tp->rank, tp->world, seq, rows,
                       ctx->dev_error, ctx->wait_limit_cycles, w, eps, (int)m, xn_out, n, next != nullptr, nblocks);
    CTOX_CUDA(ctx, cudaGetLastError());
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

ctox_status ctox_tp_debug_silent_peers(ctox_ctx *ctx, int32_t world, uint64_t wait_limit_cycles) {
    if (!ctx) return CTOX_INVALID_STATE;
    if (world < 2 || world > (int32_t)kTpMaxWorld) return fail(ctx, CTOX_SHAPE, "silent peers: world %d", world);
    if (ctx->nccl_comm || ctx->tp_world > 1) return fail(ctx, CTOX_INVALID_STATE, "tp: the context already belongs to a group");
    ctx->tp_rank = 0;
    ctx->tp_world = world;
    ctx->tp_silent = true;
    if (wait_limit_cycles) ctx->wait_limit_cycles = (long long)wait_limit_cycles;
    return CTOX_OK;
}

ctox_status ctox_tp_collective(const ctox_ctx *ctx, const char **name) {
    if (!ctx || !name) return CTOX_INVALID_STATE;
    *name = ctx->tp_world <= 1 ? "none" : (ctx->tp_peer ? "p2p_push" : "nccl");
    return CTOX_OK;
}

ctox_status ctox_tp_destroy(ctox_ctx *ctx) {
    if (!ctx) return CTOX_OK;
    tp_peer_destroy(ctx);
    ctx->tp_silent = false;
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
