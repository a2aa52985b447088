// Element-wise and attention kernels of the decode executor (layers.cu), as host launchers.
// Every tensor is device memory; `m` counts the positions of the current pass (1..8).
#pragma once
#include <cuda_runtime.h>

#include <cstdint>

#include "matvec.cuh"

namespace ctox {

// Output of a streamed matvec, still as partial sums (consumers add them up themselves).
struct MvOut {
    const float *partial;
    const uint8_t *pieces;
    const float *s_out;
    uint32_t slices, max_pieces;
    // When set, the output is this finished vector instead ([position][plain_stride]): the form a
    // column-split matvec has after its partial results were summed over the tensor-parallel group.
    const float *plain;
    uint32_t plain_stride;
    // The work split that produced the partial sums (units of a slice = pairs * kst_s, warps per
    // slice): consumers compute the piece count of a row pair instead of loading it.
    // warps_per_slice == 0: use the table.
    uint32_t kst_s, warps_per_slice, pairs;
};
// Input of the next matvec: where to write the activation fragments.
struct MvIn {
    uint8_t *xfrag;
    float2 *meta;
    const float *s_in;
    uint32_t columns, blocks_padded;
    int dt;
};

MvOut mv_out(ctox_matvec *mv, uint32_t npos);
MvIn mv_in(ctox_matvec *mv);

// Most context splits a query head's partial outputs can be merged from (k_attn_combine_prep).
constexpr int kAttnMaxSplits = 160;

struct AttnGeom {
    uint32_t q_heads, kv_heads, head_dim, rotary_dim;
    float theta, eps;
};

// h[m] (+= matvec output) ; xn = rmsnorm_1p(h[m], w) ; optional copy of xn ; fragments of xn * s_in.
// scratch: m * ceil(hidden / 256) floats.
void launch_residual_norm_prep(cudaStream_t st, float *h, const MvOut *add, const float *w, float eps,
                               uint32_t hidden, uint32_t m, float *xn_out, const MvIn *next, float *scratch);
// h[m] (+= matvec output) and the partial sums of squares of the result: scratch[m][ceil(hidden/256)],
// the form launch_norm_prep reads.
void launch_residual_add(cudaStream_t st, float *h, const MvOut *add, uint32_t hidden, uint32_t m, float *scratch);
inline uint32_t residual_parts(uint32_t hidden) { return (hidden + 255) / 256; }
// The norm half of launch_residual_norm_prep alone (scratch already holds the sums of squares of h).
void launch_norm_prep(cudaStream_t st, const float *h, const float *w, float eps, uint32_t hidden, uint32_t m,
                      float *xn_out, const MvIn *next, const float *scratch);
// h += sum over the tensor-parallel group of a matvec's output, through peer memory (tp.cu);
// scratch receives the partial sums of squares like launch_residual_add.
ctox_status tp_peer_reduce_add(ctox_ctx *ctx, const MvOut &o, uint32_t rows, uint32_t m, float *h, float *scratch);
// The same followed, in the same kernel, by the RMS norm (weight w) and the fragments of `next`
// (null: xn_out only). False when the shape does not fit the merged kernel (the caller then uses
// tp_peer_reduce_add + launch_norm_prep).
bool tp_peer_reduce_add_norm_fits(uint32_t rows, const MvIn *next);
ctox_status tp_peer_reduce_add_norm(ctox_ctx *ctx, const MvOut &o, uint32_t rows, uint32_t m, float *h,
                                    const float *w, float eps, float *xn_out, const MvIn *next);
// MTP input: fragments of concat(rmsnorm_1p(embed(tok[m])), rmsnorm_1p(prev_hidden[m])) * s_in.
void launch_mtp_pre(cudaStream_t st, const float *embed_rows, const float *prev_hidden, const float *w_embed,
                    const float *w_hidden, float eps, uint32_t hidden, uint32_t m, const MvIn *next);
// silu(gate) * up of a fused [gate; up] projection -> fragments for the down projection.
void launch_swiglu_prep(cudaStream_t st, const MvOut &gate_up, uint32_t inter, uint32_t m, const MvIn &next);
// conv_state <- conv_state shifted by the first n inputs of the pass (commit of n positions).
void launch_conv_commit(cudaStream_t st, float *conv_state, const float *conv_in, uint32_t channels,
                        uint32_t conv_kernel, uint32_t n);
// Full attention, before the cache: split q/gate, per-head norms, partial RoPE, K/V append.
void launch_attn_pre(cudaStream_t st, const MvOut &fan, const AttnGeom &g, const float *q_norm,
                     const float *k_norm, uint64_t rope_position, uint64_t cache_slot, uint32_t m, float *q,
                     float *gate, void *k_cache, void *v_cache, int kv_bf16, const uint32_t *page_table,
                     uint32_t page_tokens);
// Causal GQA over the paged cache for m query positions, split over the context; then the
// sigmoid gate and the fragments for o_proj.
size_t attn_workspace_bytes(const AttnGeom &g, uint32_t m, uint32_t max_splits);
void launch_attention(cudaStream_t st, const AttnGeom &g, const float *q, const float *gate,
                      const void *k_cache, const void *v_cache, int kv_bf16, const uint32_t *page_table,
                      uint32_t page_tokens, uint64_t cache_slot, uint32_t m, uint32_t splits, float *workspace,
                      const MvIn &next);

// Linear attention of one layer in one kernel: causal conv + SiLU over this head's channels of the
// fused projection, decay/beta, the gated-delta recurrence over the m positions, rms_norm_gated and
// the fragments for out_proj. One CTA per value head. The pass's conv inputs and (q, k, v, g,
// beta) are kept so that a commit of any accepted prefix can re-scan (delta.cu).
struct LinearAttnArgs {
    MvOut fan;
    uint32_t key_width, value_width, value_heads, qk_heads, conv_kernel;
    const float *conv_state, *conv_w, *a_log, *dt_bias, *norm_w;
    float eps;
    const float *state_in;
    float *state_out, *conv_in, *q, *k, *v, *log_decay, *beta;
    MvIn next;
};
void launch_linear_attention(cudaStream_t st, const LinearAttnArgs &a, uint32_t m);

// Commit of an accepted prefix for all linear-attention layers in one launch (delta.cu).
struct CommitLayer {
    const float *q, *k, *v, *g, *beta;  // kept inputs of the last pass
    float *state[2];                    // recurrent state double buffer
    float *conv_state;
    const float *conv_in;
};
struct CommitCur {
    uint64_t lo, hi;  // bit j: index (0 / 1) of the committed state buffer of linear layer j < 128
};
void launch_commit_batch(cudaStream_t st, const CommitLayer *layers_dev, const CommitCur &cur, uint32_t n_layers,
                         uint32_t n, bool rescan, uint32_t heads, uint32_t qk_heads, uint32_t channels,
                         uint32_t conv_kernel);

}  // namespace ctox

#ifdef __CUDACC__
#include <cooperative_groups.h>

#include "prep.cuh"
namespace ctox {
// One output value of an earlier matvec.
__device__ __forceinline__ float out_of(const MvOut &o, uint32_t row, uint32_t pos) {
    if (o.plain) return o.plain[(size_t)pos * o.plain_stride + row];
    if (o.warps_per_slice)
        return matvec_output_n(o.partial, piece_count(row >> 5, o.kst_s, o.warps_per_slice, o.pairs), o.slices,
                               o.max_pieces, o.s_out, row, pos);
    return matvec_output(o.partial, o.pieces, o.slices, o.max_pieces, o.s_out, row, pos);
}
// The part of the merged residual + norm kernels after this thread's new residual value v of column
// c = blockIdx.x * kRnThreads + threadIdx.x of position m is known (and stored): the kRnCluster
// CTAs of a thread-block cluster share a position; the partial sums of squares meet through
// distributed shared memory (one cluster barrier instead of a kernel boundary), then each CTA
// normalises its kRnThreads columns and writes its kRnBlocks 64-column blocks of the next projection's
// fragments. wc = norm weight, sc = s_in of column c. Every thread of the cluster must call it.
// (measured per speculative block of four verify positions: 5 CTAs of 1024 threads 6.24 ms, 8 of 640
// 6.18, 10 of 512 6.22, 16 of 320 6.24; one CTA of 1024 threads with five columns per thread 7.74. With
// one position 16 CTAs are the fastest: 196.5 against 194.8 tokens/s of plain decode.)
constexpr int kRnCluster = 8, kRnClusterWide = 16, kRnColumns = 5120;
template <int CL>
__device__ __forceinline__ void residual_norm_finish(float v, uint32_t hidden, float wc, float sc, float eps, int m,
                                                     int npos, float *__restrict__ xn_out, const MvIn &next,
                                                     int has_next, uint32_t nblocks) {
    constexpr int kRnThreads = kRnColumns / CL, kRnBlocks = kRnThreads / 64;
    static_assert(kRnThreads % 64 == 0 && kRnThreads <= 1024, "whole 64-column blocks per CTA");
    namespace cg = cooperative_groups;
    cg::cluster_group cluster = cg::this_cluster();
    __shared__ float red[kRnThreads / 32];
    __shared__ float part;  // this CTA's sum of squares, read by the whole cluster
    __shared__ float vals[kRnThreads];
    const uint32_t tid = threadIdx.x, rank = blockIdx.x;
    const uint32_t c = rank * kRnThreads + tid;
    float s = v * v;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    if ((tid & 31) == 0) red[tid >> 5] = s;
    __syncthreads();
    if (tid < 32) {  // the 32 warp sums, by one warp (a fixed tree: the same bits in every run)
        float t = tid < kRnThreads / 32 ? red[tid] : 0.f;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
        if (tid == 0) part = t;
    }
    cluster.sync();
    float total = 0.f;
    for (int r = 0; r < CL; ++r) total += *cluster.map_shared_rank(&part, r);  // rank order
    // nobody may leave while its `part` can still be read: every thread arrives here and waits for
    // the others only at the very end, behind its stores
    cluster.barrier_arrive();
    const float inv = 1.0f / sqrtf(total / (float)hidden + eps);
    float xn = 0.f;
    if (c < hidden) {
        xn = v * inv * (1.0f + wc);
        if (xn_out) xn_out[(size_t)m * hidden + c] = xn;
    }
    if (has_next) {
        vals[tid] = xn * sc;
        __syncthreads();
        if (tid < kRnBlocks * 16) {  // groups of 16 lanes, one 64-column block each
            const int i = tid & 15;
            const uint32_t grp = tid >> 4, b = rank * kRnBlocks + grp;
            if (b < nblocks) {
                const float x[4] = {vals[grp * 64 + i * 4], vals[grp * 64 + i * 4 + 1], vals[grp * 64 + i * 4 + 2],
                                    vals[grp * 64 + i * 4 + 3]};
                const unsigned gmask = (tid & 16) ? 0xffff0000u : 0x0000ffffu;
                prep_block(x, i, gmask, (int)b, m, npos, next.dt, next.xfrag, next.meta);
            }
        }
    }
    cluster.barrier_wait();
}
// out_of in two halves for kernels launched ahead of their producer: out_ref is arithmetic on the
// launch arguments plus the constant s_out[row] and may run BEFORE the dependency wait; out_at does
// the loads. Same additions in the same order as out_of.
struct OutRef {
    const float *first;
    uint32_t n, total;
    float so;
    bool pieces;  // false: out_at falls back to out_of
};
__device__ __forceinline__ OutRef out_ref(const MvOut &o, uint32_t row) {
    OutRef r{nullptr, 0, 0, 1.0f, false};
    if (!o.plain && o.warps_per_slice) {
        r.pieces = true;
        r.n = piece_count(row >> 5, o.kst_s, o.warps_per_slice, o.pairs);
        r.total = o.slices * r.n;
        r.first = o.partial + (size_t)(row >> 5) * o.slices * o.max_pieces * 256 + (row & 31);
        if (o.s_out) r.so = o.s_out[row];
    }
    return r;
}
__device__ __forceinline__ float out_at(const MvOut &o, const OutRef &r, uint32_t row, uint32_t pos) {
    if (!r.pieces) return out_of(o, row, pos);
    const float *first = r.first + pos * 32;
    float v = 0.f;
    uint32_t sl = 0, q = 0;
    for (uint32_t k0 = 0; k0 < r.total; k0 += 8) {
        float buf[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            buf[j] = 0.f;
            if (k0 + j < r.total) {
                buf[j] = first[((size_t)sl * o.max_pieces + q) * 256];
                if (++q == r.n) {
                    q = 0;
                    ++sl;
                }
            }
        }
#pragma unroll
        for (int j = 0; j < 8; ++j)
            if (k0 + j < r.total) v += buf[j];
    }
    return o.s_out ? v * r.so : v;
}
__device__ __forceinline__ float silu_f(float v) { return v / (1.0f + expf(-v)); }
// Two output values of the same matvec and position with the loads of both issued together
// (each up to four pieces per trip; same order of additions as out_of).
__device__ __forceinline__ void out_of2(const MvOut &o, uint32_t row_a, uint32_t row_b, uint32_t pos, float &a,
                                        float &b) {
    if (o.plain || !o.warps_per_slice) {
        a = out_of(o, row_a, pos);
        b = out_of(o, row_b, pos);
        return;
    }
    const uint32_t na = piece_count(row_a >> 5, o.kst_s, o.warps_per_slice, o.pairs);
    const uint32_t nb = piece_count(row_b >> 5, o.kst_s, o.warps_per_slice, o.pairs);
    const float *fa = o.partial + (size_t)(row_a >> 5) * o.slices * o.max_pieces * 256 + pos * 32 + (row_a & 31);
    const float *fb = o.partial + (size_t)(row_b >> 5) * o.slices * o.max_pieces * 256 + pos * 32 + (row_b & 31);
    const uint32_t ta = o.slices * na, tb = o.slices * nb;
    float va = 0.f, vb = 0.f;
    uint32_t sla = 0, qa = 0, slb = 0, qb = 0;
    for (uint32_t k0 = 0; k0 < max(ta, tb); k0 += 4) {
        float ba[4], bb[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            ba[j] = bb[j] = 0.f;
            if (k0 + j < ta) {
                ba[j] = fa[((size_t)sla * o.max_pieces + qa) * 256];
                if (++qa == na) {
                    qa = 0;
                    ++sla;
                }
            }
            if (k0 + j < tb) {
                bb[j] = fb[((size_t)slb * o.max_pieces + qb) * 256];
                if (++qb == nb) {
                    qb = 0;
                    ++slb;
                }
            }
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            if (k0 + j < ta) va += ba[j];
            if (k0 + j < tb) vb += bb[j];
        }
    }
    a = o.s_out ? va * o.s_out[row_a] : va;
    b = o.s_out ? vb * o.s_out[row_b] : vb;
}
}  // namespace ctox
#endif
