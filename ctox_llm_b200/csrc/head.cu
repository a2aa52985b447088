// Selection over the vocabulary: multi-CTA argmax, and the fused
// lm_head -> softmax statistics -> speculative acceptance path.
//
// Reference semantics: greedy = last maximal index under f32::total_cmp
// (sampler.rs:76-82, engine.rs:906-913; CUDA candidate ctox_argmax_f32_sm86,
// kernels/cuda/q2q4_fused_matvec_sm86.cu:2568-2620, which scans 248 077 logits
// with ONE CTA); greedy MTP verification engine.rs:915-963 and the one-thread
// accept kernel vendor/cuda/tensorrt_llm_mtp/mtp_accept_draft_token_sm86.cu:64-80.
// The reference has no stochastic acceptance (engine.rs:583-590 fails closed);
// the rule implemented here is stated in k_spec_accept.
//
// The lm_head logits are never written out: the streaming matvec leaves raw
// per-piece sums, and k_head_stats turns them into per-position (argmax, max,
// sum of exp, Gumbel-argmax, logits of the candidate tokens) in one sweep.
#include "common.cuh"
#include "head.cuh"
#include "matvec.cuh"

#include <cmath>
#include <cstddef>

namespace ctox {

constexpr int kMaxNodes = 16;     // verify positions (tree nodes incl. the root)
constexpr int kHeadThreads = 256;

struct NodeStat {
    unsigned long long argmax;  // pack_key_index(logit, row)
    unsigned long long gumbel;  // pack_key_index(z + noise, row) over rows that are not children
    float max;                  // max of z = logit / T
    float sum;                  // sum of exp(z - max)
    uint32_t nonfinite;
    uint32_t pad;
};

// parent[] travels by value; the node tokens stay in device memory because the drafts
// of a speculative block are produced on the device and never visit the host.
struct TreeDesc {
    int32_t parent[kMaxNodes];
    const uint32_t *token;  // device, [n_nodes]
    uint32_t n_nodes;
};

__device__ __forceinline__ void merge_stat(NodeStat &a, const NodeStat &b) {
    a.argmax = a.argmax > b.argmax ? a.argmax : b.argmax;
    a.gumbel = a.gumbel > b.gumbel ? a.gumbel : b.gumbel;
    a.nonfinite |= b.nonfinite;
    if (b.sum > 0.f) {
        if (a.sum > 0.f) {
            const float m = fmaxf(a.max, b.max);
            a.sum = a.sum * expf(a.max - m) + b.sum * expf(b.max - m);
            a.max = m;
        } else {
            a.max = b.max;
            a.sum = b.sum;
        }
    }
}

// One sweep over the vocabulary rows for the `npos` positions of the current pass.
__global__ void __launch_bounds__(kHeadThreads) k_head_stats(
    const float *__restrict__ partial, const uint8_t *__restrict__ pieces, const float *__restrict__ s_out,
    const float *__restrict__ bias, uint32_t rows, uint32_t slices, uint32_t max_pieces, uint32_t node0,
    uint32_t npos,
    float inv_temperature, unsigned long long seed, unsigned long long step, TreeDesc tree,
    NodeStat *__restrict__ cta_stats, float *__restrict__ child_z, float *__restrict__ logits_out,
    unsigned long long logits_stride, uint32_t row_offset) {
    pdl_launch();
    pdl_wait();
    __shared__ NodeStat sh[kHeadThreads / 32][kMaxPosPerPass];
    NodeStat st[kMaxPosPerPass];
#pragma unroll
    for (int m = 0; m < kMaxPosPerPass; ++m) st[m] = NodeStat{0ull, 0ull, 0.f, 0.f, 0u, 0u};
    for (uint32_t row = blockIdx.x * blockDim.x + threadIdx.x; row < rows; row += gridDim.x * blockDim.x) {
        const uint32_t pr = row / kPairRows, rl = row % kPairRows;
        float lg[kMaxPosPerPass];
#pragma unroll
        for (int m = 0; m < kMaxPosPerPass; ++m) lg[m] = 0.f;
        for (uint32_t sl = 0; sl < slices; ++sl) {
            // a slot is [position][32 rows]: the 32 rows of a pair are one coalesced line per position
            const float *base = partial + ((size_t)pr * slices + sl) * max_pieces * (kPairRows * kMaxPosPerPass) + rl;
            const uint32_t n = pieces[pr * slices + sl];
            for (uint32_t q = 0; q < n; ++q) {
                const float *sl_q = base + q * (kPairRows * kMaxPosPerPass);
#pragma unroll
                for (int m = 0; m < kMaxPosPerPass; ++m)
                    if ((uint32_t)m < npos) lg[m] += sl_q[m * kPairRows];
            }
        }
        const float so = s_out ? s_out[row] : 1.0f, bi = bias ? bias[row] : 0.0f;
#pragma unroll
        for (int m = 0; m < kMaxPosPerPass; ++m) lg[m] = (lg[m] + bi) * so;
#pragma unroll
        for (int m = 0; m < kMaxPosPerPass; ++m) {
            if ((uint32_t)m >= npos) break;
            const uint32_t node = node0 + m;
            const float logit = lg[m];
            if (logits_out) logits_out[(size_t)node * logits_stride + row] = logit;
            if (!isfinite(logit)) {
                st[m].nonfinite = 1;
                continue;
            }
            const uint32_t token = row + row_offset;  // rows of a vocabulary shard start at row_offset
            const unsigned long long pk = pack_key_index(logit, token);
            st[m].argmax = pk > st[m].argmax ? pk : st[m].argmax;
            if (inv_temperature > 0.f) {
                const float z = logit * inv_temperature;
                if (st[m].sum > 0.f) {
                    if (z > st[m].max) {
                        st[m].sum = st[m].sum * expf(st[m].max - z) + 1.0f;
                        st[m].max = z;
                    } else {
                        st[m].sum += expf(z - st[m].max);
                    }
                } else {
                    st[m].max = z;
                    st[m].sum = 1.0f;
                }
                bool is_child = false;
                for (uint32_t c = node + 1; c < tree.n_nodes; ++c)
                    if ((uint32_t)tree.parent[c] == node && tree.token[c] == token) {
                        is_child = true;
                        child_z[c] = z;  // one writer: the row is unique
                    }
                if (!is_child) {
                    const unsigned long long gk = pack_key_index(z + gumbel_noise(seed, step, node, token), token);
                    st[m].gumbel = gk > st[m].gumbel ? gk : st[m].gumbel;
                }
            }
        }
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int m = 0; m < kMaxPosPerPass; ++m) {
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            NodeStat other;
            other.argmax = __shfl_xor_sync(0xffffffffu, st[m].argmax, o);
            other.gumbel = __shfl_xor_sync(0xffffffffu, st[m].gumbel, o);
            other.max = __shfl_xor_sync(0xffffffffu, st[m].max, o);
            other.sum = __shfl_xor_sync(0xffffffffu, st[m].sum, o);
            other.nonfinite = __shfl_xor_sync(0xffffffffu, st[m].nonfinite, o);
            merge_stat(st[m], other);
        }
        if (lane == 0) sh[warp][m] = st[m];
    }
    __syncthreads();
    if (threadIdx.x < kMaxPosPerPass) {
        NodeStat a = sh[0][threadIdx.x];
        for (int w = 1; w < kHeadThreads / 32; ++w) merge_stat(a, sh[w][threadIdx.x]);
        cta_stats[(size_t)blockIdx.x * kMaxPosPerPass + threadIdx.x] = a;
    }
}

// Merges the per-CTA statistics of one pass into node_stats[node0 .. node0+npos): one warp per
// position, lanes stride over the CTAs, then a butterfly (max/sum merges are order-insensitive up
// to rounding; the lane order is fixed, so the result is reproducible).
__global__ void k_head_merge(const NodeStat *__restrict__ cta_stats, uint32_t n_ctas, uint32_t node0,
                             uint32_t npos, NodeStat *__restrict__ node_stats) {
    pdl_launch();
    pdl_wait();
    const uint32_t m = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (m >= npos) return;
    NodeStat a{0ull, 0ull, 0.f, 0.f, 0u, 0u};
    for (uint32_t c = lane; c < n_ctas; c += 32) merge_stat(a, cta_stats[(size_t)c * kMaxPosPerPass + m]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        NodeStat other;
        other.argmax = __shfl_xor_sync(0xffffffffu, a.argmax, o);
        other.gumbel = __shfl_xor_sync(0xffffffffu, a.gumbel, o);
        other.max = __shfl_xor_sync(0xffffffffu, a.max, o);
        other.sum = __shfl_xor_sync(0xffffffffu, a.sum, o);
        other.nonfinite = __shfl_xor_sync(0xffffffffu, a.nonfinite, o);
        merge_stat(a, other);
    }
    if (lane == 0) node_stats[node0 + m] = a;
}

// Tensor-parallel vocabulary: every rank holds the statistics of its shard and the logit of the
// children whose token lies in its shard. gathered = [world][kMaxNodes stats | kMaxNodes child_z];
// the merge runs in rank order on every rank, so all ranks resolve the same record.
struct RankStats {
    NodeStat node[kMaxNodes];
    float child_z[kMaxNodes];
};
__global__ void k_head_merge_ranks(const RankStats *__restrict__ gathered, uint32_t world, uint32_t shard_rows,
                                   TreeDesc tree, RankStats *__restrict__ out) {
    pdl_launch();
    pdl_wait();
    const uint32_t n = threadIdx.x;
    if (n >= tree.n_nodes) return;
    NodeStat a = gathered[0].node[n];
    for (uint32_t r = 1; r < world; ++r) merge_stat(a, gathered[r].node[n]);
    out->node[n] = a;
    uint32_t owner = tree.token[n] / shard_rows;
    if (owner >= world) owner = world - 1;
    out->child_z[n] = gathered[owner].child_z[n];
}

// Walks the draft tree with the statistics of every node. One thread: the walk is
// a dependent chain of at most kMaxNodes steps.
//
// Node 0 is the root (the current position). At node n with children c1..cm in
// index order: with temperature 0, child c is accepted iff its token equals
// argmax of n's logits (engine.rs:939-962); otherwise c is accepted with
// probability p_n(c) / (1 - mass of its rejected elder siblings) on the draw
// accept_draw(seed, step, c). The drafter is deterministic, so this is speculative
// sampling with a point-mass proposal and the emitted token is distributed as
// softmax(logits / T). When no child is accepted the token is the Gumbel-max
// sample of p_n restricted to non-children (greedy: the argmax).
__global__ void k_spec_accept(const NodeStat *__restrict__ node_stats, const float *__restrict__ child_z,
                              TreeDesc tree, float inv_temperature, unsigned long long seed,
                              unsigned long long step, int force_accept, ctox_spec_record *__restrict__ rec) {
    pdl_launch();
    pdl_wait();
    if (threadIdx.x != 0 || blockIdx.x != 0) return;
    uint32_t count = 0, node = 0, status = 0;
    for (uint32_t n = 0; n < tree.n_nodes; ++n) rec->node_token[n] = tree.token[n];
    for (uint32_t n = 0; n < tree.n_nodes; ++n) {
        rec->node_argmax[n] = (uint32_t)(node_stats[n].argmax & 0xffffffffull);
        if (node_stats[n].nonfinite) status = 1;
    }
    for (uint32_t n = tree.n_nodes; n < kMaxNodes; ++n) rec->node_argmax[n] = 0;
    for (uint32_t i = 0; i < kMaxNodes; ++i) rec->path[i] = -1;
    if (status == 0 && force_accept >= 0) {
        // throughput buckets: accept exactly force_accept drafts of the chain, then the target's token
        while (count < (uint32_t)force_accept && node + 1 < tree.n_nodes) {
            rec->path[count] = (int32_t)(node + 1);
            rec->emitted[count++] = tree.token[node + 1];
            ++node;
        }
        rec->emitted[count++] = (uint32_t)(node_stats[node].argmax & 0xffffffffull);
    } else if (status == 0) {
        for (;;) {
            const NodeStat st = node_stats[node];
            bool moved = false;
            if (!(inv_temperature > 0.f)) {
                const uint32_t target = (uint32_t)(st.argmax & 0xffffffffull);
                for (uint32_t c = node + 1; c < tree.n_nodes; ++c)
                    if ((uint32_t)tree.parent[c] == node && tree.token[c] == target) {
                        rec->path[count] = (int32_t)c;
                        rec->emitted[count++] = target;
                        node = c;
                        moved = true;
                        break;
                    }
                if (!moved) {
                    rec->emitted[count++] = target;
                    break;
                }
                continue;
            }
            float residual = 1.0f;
            for (uint32_t c = node + 1; c < tree.n_nodes; ++c) {
                if ((uint32_t)tree.parent[c] != node) continue;
                const float p = expf(child_z[c] - st.max) / st.sum;
                const float u = accept_draw(seed, step, c);
                if (u * residual < p) {
                    rec->path[count] = (int32_t)c;
                    rec->emitted[count++] = tree.token[c];
                    node = c;
                    moved = true;
                    break;
                }
                residual -= p;
                if (residual < 0.f) residual = 0.f;
            }
            if (moved) continue;
            rec->emitted[count++] = (uint32_t)(st.gumbel & 0xffffffffull);
            break;
        }
    }
    for (uint32_t i = count; i < kMaxNodes + 1; ++i) rec->emitted[i] = 0;
    rec->n_emitted = count;
    rec->status = status;
}

// ------------------------------------------------------------------ plain argmax
struct ArgmaxPartial {
    unsigned long long best;
    uint32_t nonfinite;
    uint32_t pad;
};

__global__ void __launch_bounds__(kHeadThreads) k_argmax_partial(const float *__restrict__ logits, uint32_t n,
                                                               ArgmaxPartial *__restrict__ out) {
    pdl_launch();
    pdl_wait();
    __shared__ ArgmaxPartial sh[kHeadThreads / 32];
    unsigned long long best = 0ull;
    uint32_t bad = 0;
    for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
        const float v = logits[i];
        if (!isfinite(v)) bad = 1;
        const unsigned long long pk = pack_key_index(v, i);
        best = pk > best ? pk : best;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const unsigned long long ob = __shfl_xor_sync(0xffffffffu, best, o);
        best = ob > best ? ob : best;
        bad |= __shfl_xor_sync(0xffffffffu, bad, o);
    }
    if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = ArgmaxPartial{best, bad, 0};
    __syncthreads();
    if (threadIdx.x == 0) {
        ArgmaxPartial a = sh[0];
        for (int w = 1; w < kHeadThreads / 32; ++w) {
            a.best = sh[w].best > a.best ? sh[w].best : a.best;
            a.nonfinite |= sh[w].nonfinite;
        }
        out[blockIdx.x] = a;
    }
}

// result[0] = token (mapped through row_ids when given, engine.rs:203-217), result[1] = status
// (1 = a logit is not finite, kernels/cuda/q2q4_fused_matvec_sm86.cu:2583-2585).
// With packed_out the (key, token) pair is stored as well, for the merge over a tensor-parallel group.
__global__ void k_argmax_final(const ArgmaxPartial *__restrict__ parts, uint32_t n_parts,
                               const uint32_t *__restrict__ row_ids, uint32_t row_offset,
                               uint32_t *__restrict__ token_out, uint32_t *__restrict__ status_out,
                               ArgmaxPartial *__restrict__ packed_out) {
    pdl_launch();
    pdl_wait();
    if (threadIdx.x != 0) return;
    ArgmaxPartial a = parts[0];
    for (uint32_t i = 1; i < n_parts; ++i) {
        a.best = parts[i].best > a.best ? parts[i].best : a.best;
        a.nonfinite |= parts[i].nonfinite;
    }
    const uint32_t row = (uint32_t)(a.best & 0xffffffffull);
    const uint32_t token = row_ids ? row_ids[row] : row + row_offset;
    if (token_out) *token_out = token;
    if (status_out) *status_out = a.nonfinite;
    if (packed_out) *packed_out = ArgmaxPartial{(a.best & 0xffffffff00000000ull) | token, a.nonfinite, 0};
}

// Greatest (key, token) over the ranks' local results; an empty shard contributes best == 0.
__global__ void k_argmax_ranks(const ArgmaxPartial *__restrict__ gathered, uint32_t world,
                               uint32_t *__restrict__ token_out, uint32_t *__restrict__ status_out) {
    pdl_launch();
    pdl_wait();
    if (threadIdx.x != 0) return;
    ArgmaxPartial a = gathered[0];
    for (uint32_t r = 1; r < world; ++r) {
        a.best = gathered[r].best > a.best ? gathered[r].best : a.best;
        a.nonfinite |= gathered[r].nonfinite;
    }
    *token_out = (uint32_t)(a.best & 0xffffffffull);
    if (status_out) *status_out = a.nonfinite;
}

// ------------------------------------------------------------------ top-k / top-p sampling with a supplied draw
// Sampler::sample_with_draw (sampler.rs:65-144): z = logit / T; candidates ordered by z descending,
// ties by token id descending; the first top_k; weights exp(z - z_max); the nucleus ends at the first
// candidate whose running sum reaches top_p * total; the token is the first whose running sum
// reaches draw * nucleus_total. All sums are sequential fp32 in candidate order, as in the
// reference. The reference's CUDA sampler takes top_k in 1..=256
// (backend/cuda_runtime.rs:2828, kernels/cuda/q2q4_fused_matvec_sm86.cu:2648-2667); this one 1..=1024.
// One CTA: radix select of the top_k-th largest key (then of the largest ids among equal keys),
// gather, bitonic sort of the <= 1024 candidates, one thread for the sequential part.
constexpr uint32_t kSampleMaxTopK = 1024, kSampleThreads = 1024;

// result: [0] token, [1] status (0 ok, 1 invalid arguments, 2 non-finite value), [2] nucleus size
__global__ void __launch_bounds__(kSampleThreads) k_sample_topk_topp(const float *__restrict__ logits, uint32_t n,
                                                                    uint32_t top_k, float inv_t, float top_p,
                                                                    float draw, uint32_t *__restrict__ result) {
    pdl_launch();
    pdl_wait();
    __shared__ uint32_t hist[256];
    __shared__ unsigned long long cand[kSampleMaxTopK];  // (key << 32) | id, sorted descending
    __shared__ uint32_t sh_prefix, sh_need, sh_count, sh_bad;
    const uint32_t tid = threadIdx.x;
    if (tid == 0) {
        sh_bad = 0;
        sh_count = 0;
    }
    __syncthreads();
    if (n == 0 || top_k == 0 || top_k > kSampleMaxTopK || !isfinite(inv_t) || inv_t <= 0.f || !isfinite(top_p) ||
        top_p <= 0.f || top_p > 1.f || !isfinite(draw) || draw < 0.f || draw >= 1.f) {
        if (tid == 0) {
            result[0] = 0;
            result[1] = 1;
            result[2] = 0;
        }
        return;
    }
    const uint32_t k = top_k < n ? top_k : n;
    auto key_of = [&](uint32_t i) {
        const float z = logits[i] * inv_t;
        if (!isfinite(logits[i]) || !isfinite(z)) sh_bad = 1;
        return total_order_key(z);
    };
    // ---- the k-th largest key, 8 bits at a time from the top
    uint32_t prefix = 0, need = k;  // among keys matching `prefix` on the bits fixed so far, `need` more
    for (int shift = 24; shift >= 0; shift -= 8) {
        if (tid < 256) hist[tid] = 0;
        __syncthreads();
        const uint32_t mask_hi = shift == 24 ? 0u : (0xffffffffu << (shift + 8));
        for (uint32_t i = tid; i < n; i += kSampleThreads) {
            const uint32_t key = key_of(i);
            if ((key & mask_hi) == (prefix & mask_hi)) atomicAdd(&hist[(key >> shift) & 0xff], 1u);
        }
        __syncthreads();
        if (tid == 0) {
            uint32_t acc = 0, b = 255;
            for (;; --b) {  // from the largest digit down
                if (acc + hist[b] >= need || b == 0) break;
                acc += hist[b];
            }
            sh_prefix = prefix | (b << shift);
            sh_need = need - acc;
        }
        __syncthreads();
        prefix = sh_prefix;
        need = sh_need;
        __syncthreads();
    }
    const uint32_t kth_key = prefix;  // `need` of the candidates carry exactly this key: the largest ids
    // ---- among keys == kth_key, the need-th largest id (same select over the ids)
    uint32_t id_prefix = 0, id_need = need;
    for (int shift = 24; shift >= 0; shift -= 8) {
        if (tid < 256) hist[tid] = 0;
        __syncthreads();
        const uint32_t mask_hi = shift == 24 ? 0u : (0xffffffffu << (shift + 8));
        for (uint32_t i = tid; i < n; i += kSampleThreads)
            if (key_of(i) == kth_key && (i & mask_hi) == (id_prefix & mask_hi)) atomicAdd(&hist[(i >> shift) & 0xff], 1u);
        __syncthreads();
        if (tid == 0) {
            uint32_t acc = 0, b = 255;
            for (;; --b) {
                if (acc + hist[b] >= id_need || b == 0) break;
                acc += hist[b];
            }
            sh_prefix = id_prefix | (b << shift);
            sh_need = id_need - acc;
        }
        __syncthreads();
        id_prefix = sh_prefix;
        id_need = sh_need;
        __syncthreads();
    }
    const uint32_t min_tie_id = id_prefix;
    // ---- gather the k candidates, pad, sort descending
    for (uint32_t i = tid; i < kSampleMaxTopK; i += kSampleThreads) cand[i] = 0ull;
    __syncthreads();
    for (uint32_t i = tid; i < n; i += kSampleThreads) {
        const uint32_t key = key_of(i);
        if (key > kth_key || (key == kth_key && i >= min_tie_id)) {
            const uint32_t slot = atomicAdd(&sh_count, 1u);
            if (slot < kSampleMaxTopK) cand[slot] = ((unsigned long long)key << 32) | i;
        }
    }
    __syncthreads();
    for (uint32_t size = 2; size <= kSampleMaxTopK; size <<= 1) {
        for (uint32_t stride = size >> 1; stride > 0; stride >>= 1) {
            const uint32_t partner = tid ^ stride;
            if (partner > tid) {
                const bool descending = (tid & size) == 0;
                const unsigned long long a = cand[tid], b = cand[partner];
                if ((a < b) == descending) {
                    cand[tid] = b;
                    cand[partner] = a;
                }
            }
            __syncthreads();
        }
    }
    // ---- the sequential part (sampler.rs:108-143)
    if (tid == 0) {
        uint32_t status = sh_bad ? 2u : 0u, token = 0, nucleus = 0;
        if (status == 0 && sh_count != k) status = 2;  // cannot happen for finite input
        if (status == 0) {
            const float maximum = logits[(uint32_t)(cand[0] & 0xffffffffull)] * inv_t;
            float normalization = 0.f;
            for (uint32_t i = 0; i < k; ++i)
                normalization += expf(logits[(uint32_t)(cand[i] & 0xffffffffull)] * inv_t - maximum);
            if (!isfinite(normalization) || normalization <= 0.f) {
                status = 2;
            } else {
                float cumulative = 0.f;
                nucleus = k;
                for (uint32_t i = 0; i < k; ++i) {
                    cumulative += expf(logits[(uint32_t)(cand[i] & 0xffffffffull)] * inv_t - maximum);
                    if (cumulative >= top_p * normalization) {
                        nucleus = i + 1;
                        break;
                    }
                }
                float nucleus_total = 0.f;
                for (uint32_t i = 0; i < nucleus; ++i)
                    nucleus_total += expf(logits[(uint32_t)(cand[i] & 0xffffffffull)] * inv_t - maximum);
                const float threshold = draw * nucleus_total;
                cumulative = 0.f;
                token = (uint32_t)(cand[nucleus - 1] & 0xffffffffull);
                for (uint32_t i = 0; i < nucleus; ++i) {
                    cumulative += expf(logits[(uint32_t)(cand[i] & 0xffffffffull)] * inv_t - maximum);
                    if (threshold <= cumulative) {
                        token = (uint32_t)(cand[i] & 0xffffffffull);
                        break;
                    }
                }
            }
        }
        result[0] = token;
        result[1] = status;
        result[2] = nucleus;
    }
}

}  // namespace ctox

using namespace ctox;

namespace {
constexpr uint32_t kHeadGridMax = 592;  // 4 CTAs per SM on 148 SMs

constexpr uint32_t kMaxTpWorld = 8;

struct HeadScratch {
    NodeStat *cta_stats;   // [grid][kMaxPosPerPass]
    NodeStat *node_stats;  // [kMaxNodes]   } one RankStats: what a rank contributes to the
    float *child_z;        // [kMaxNodes]   } tensor-parallel merge
    RankStats *gathered;   // [kMaxTpWorld]
    ArgmaxPartial *argmax_send, *argmax_gathered;  // [1], [kMaxTpWorld]
    ctox_spec_record *record;
    ArgmaxPartial *argmax_parts;  // [grid]
    uint32_t *argmax_result;      // [2]
    uint32_t *tokens;             // [kMaxNodes] node tokens of the host-form verify call
};

ctox_status head_scratch(ctox_ctx *ctx, HeadScratch &hs) {
    size_t off = 0;
    auto take = [&](size_t bytes) {
        const size_t o = off;
        off += (bytes + 255) & ~(size_t)255;
        return o;
    };
    const size_t o_cta = take(sizeof(NodeStat) * kHeadGridMax * kMaxPosPerPass);
    const size_t o_node = take(sizeof(RankStats));
    const size_t o_child = o_node + offsetof(RankStats, child_z);
    const size_t o_gath = take(sizeof(RankStats) * kMaxTpWorld);
    const size_t o_as = take(sizeof(ArgmaxPartial));
    const size_t o_ag = take(sizeof(ArgmaxPartial) * kMaxTpWorld);
    const size_t o_rec = take(sizeof(ctox_spec_record));
    const size_t o_ap = take(sizeof(ArgmaxPartial) * kHeadGridMax);
    const size_t o_ar = take(sizeof(uint32_t) * 2);
    const size_t o_tok = take(sizeof(uint32_t) * kMaxNodes);
    ctox_status rc = ensure_scratch(ctx, off);
    if (rc) return rc;
    uint8_t *b = (uint8_t *)ctx->scratch;
    hs.cta_stats = (NodeStat *)(b + o_cta);
    hs.node_stats = (NodeStat *)(b + o_node);
    hs.child_z = (float *)(b + o_child);
    hs.gathered = (RankStats *)(b + o_gath);
    hs.argmax_send = (ArgmaxPartial *)(b + o_as);
    hs.argmax_gathered = (ArgmaxPartial *)(b + o_ag);
    hs.record = (ctox_spec_record *)(b + o_rec);
    hs.argmax_parts = (ArgmaxPartial *)(b + o_ap);
    hs.argmax_result = (uint32_t *)(b + o_ar);
    hs.tokens = (uint32_t *)(b + o_tok);
    return CTOX_OK;
}
}  // namespace

extern "C" {

ctox_status ctox_argmax_f32(ctox_ctx *ctx, const float *logits_dev, uint32_t n, const uint32_t *row_ids_dev,
                            uint32_t *result_dev) {
    if (!ctx) return CTOX_INVALID_STATE;
    if (!logits_dev || !result_dev || n == 0) return fail(ctx, CTOX_INVALID_ARTIFACT, "greedy logits are empty");
    CTOX_CUDA(ctx, cudaSetDevice(ctx->device));
    HeadScratch hs;
    ctox_status rc = head_scratch(ctx, hs);
    if (rc) return rc;
    uint32_t grid = (n + kHeadThreads * 4 - 1) / (kHeadThreads * 4);
    if (grid > kHeadGridMax) grid = kHeadGridMax;
    if (grid == 0) grid = 1;
    launch_pdl(k_argmax_partial, dim3(grid), dim3(kHeadThreads), 0, ctx->stream, logits_dev, n, hs.argmax_parts);
    launch_pdl(k_argmax_final, dim3(1), dim3(32), 0, ctx->stream, hs.argmax_parts, grid, row_ids_dev, 0, result_dev, result_dev + 1,
                                              nullptr);
    CTOX_CUDA(ctx, cudaGetLastError());
    return CTOX_OK;
}

ctox_status ctox_argmax_f32_host(ctox_ctx *ctx, const float *logits_dev, uint32_t n, const uint32_t *row_ids_dev,
                                 uint32_t *token) {
    if (!ctx || !token) return CTOX_INVALID_STATE;
    HeadScratch hs;
    ctox_status rc = head_scratch(ctx, hs);
    if (rc) return rc;
    rc = ctox_argmax_f32(ctx, logits_dev, n, row_ids_dev, hs.argmax_result);
    if (rc) return rc;
    rc = ensure_pinned(ctx, 8);
    if (rc) return rc;
    CTOX_CUDA(ctx, cudaMemcpyAsync(ctx->pinned, hs.argmax_result, 8, cudaMemcpyDeviceToHost, ctx->stream));
    CTOX_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    const uint32_t *r = (const uint32_t *)ctx->pinned;
    if (r[1]) return fail(ctx, CTOX_INVALID_STATE, "argmax input contains a non-finite logit");
    *token = r[0];
    return CTOX_OK;
}

ctox_status ctox_sample_topk_topp(ctox_ctx *ctx, const float *logits_dev, uint32_t n, float temperature,
                                  uint32_t top_k, float top_p, float draw, uint32_t *token) {
    if (!ctx || !token) return CTOX_INVALID_STATE;
    if (!logits_dev || n == 0) return fail(ctx, CTOX_INVALID_ARTIFACT, "sampler logits are empty");
    if (!std::isfinite(draw) || !(draw >= 0.f && draw < 1.f))
        return fail(ctx, CTOX_INVALID_ARTIFACT, "sampler draw must lie in [0, 1)");
    if (!std::isfinite(temperature) || temperature < 0.f)
        return fail(ctx, CTOX_INVALID_ARTIFACT, "temperature must be finite and non-negative");
    if (!(std::isfinite(top_p) && top_p > 0.f && top_p <= 1.f))
        return fail(ctx, CTOX_INVALID_ARTIFACT, "top_p must lie in (0, 1]");
    if (temperature == 0.f) return ctox_argmax_f32_host(ctx, logits_dev, n, nullptr, token);  // sampler.rs:76-82
    if (top_k == 0 || top_k > kSampleMaxTopK)
        return fail(ctx, CTOX_UNSUPPORTED_OPERATION, "device sampler takes top_k in 1..=%u", kSampleMaxTopK);
    const float inv_t = 1.0f / temperature;
    if (!std::isfinite(inv_t)) return fail(ctx, CTOX_INVALID_ARTIFACT, "temperature is too small");
    CTOX_CUDA(ctx, cudaSetDevice(ctx->device));
    HeadScratch hs;
    ctox_status rc = head_scratch(ctx, hs);
    if (rc) return rc;
    launch_pdl(k_sample_topk_topp, dim3(1), dim3(kSampleThreads), 0, ctx->stream, logits_dev, n, top_k, inv_t, top_p,
               draw, hs.tokens);
    CTOX_CUDA(ctx, cudaGetLastError());
    rc = ensure_pinned(ctx, 16);
    if (rc) return rc;
    CTOX_CUDA(ctx, cudaMemcpyAsync(ctx->pinned, hs.tokens, 12, cudaMemcpyDeviceToHost, ctx->stream));
    CTOX_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    const uint32_t *r = (const uint32_t *)ctx->pinned;
    if (r[1] == 2) return fail(ctx, CTOX_INVALID_ARTIFACT, "sampler input or normalisation is not finite");
    if (r[1]) return fail(ctx, CTOX_INVALID_ARTIFACT, "sampler arguments rejected on the device");
    *token = r[0];
    return CTOX_OK;
}

}  // extern "C"

namespace ctox {

ctox_status head_verify_enqueue(ctox_matvec *mv, uint32_t node0, uint32_t npos, uint32_t n_nodes,
                                const int32_t *parent, const uint32_t *tokens_dev, float inv_t, uint64_t seed,
                                uint64_t step, uint32_t rows, float *logits_out_dev, uint32_t row_offset) {
    ctox_ctx *ctx = mv->ctx;
    HeadScratch hs;
    ctox_status rc = head_scratch(ctx, hs);
    if (rc) return rc;
    TreeDesc tree;
    memset(&tree, 0, sizeof tree);
    tree.n_nodes = n_nodes;
    tree.token = tokens_dev;
    for (uint32_t i = 0; i < n_nodes; ++i) tree.parent[i] = parent[i];
    MatvecPart &p = mv->parts[0];
    uint32_t grid = (rows + kHeadThreads - 1) / kHeadThreads;
    if (grid > kHeadGridMax) grid = kHeadGridMax;
    launch_pdl(k_head_stats, dim3(grid), dim3(kHeadThreads), 0, ctx->stream, p.partial, p.split[npos > 4 ? 1 : 0].pieces, mv->s_out,
                                                        mv->bias, rows, p.slices, p.max_pieces, node0, npos,
                                                        inv_t, seed, step, tree, hs.cta_stats, hs.child_z,
                                                        logits_out_dev, (unsigned long long)mv->rows, row_offset);
    launch_pdl(k_head_merge, dim3(1), dim3(32 * kMaxPosPerPass), 0, ctx->stream, hs.cta_stats, grid, node0, npos, hs.node_stats);
    CTOX_CUDA(ctx, cudaGetLastError());
    return CTOX_OK;
}

ctox_status head_accept_enqueue(ctox_ctx *ctx, uint32_t n_nodes, const int32_t *parent,
                                const uint32_t *tokens_dev, float inv_t, uint64_t seed, uint64_t step,
                                int force_accept, ctox_spec_record **record_dev) {
    HeadScratch hs;
    ctox_status rc = head_scratch(ctx, hs);
    if (rc) return rc;
    TreeDesc tree;
    memset(&tree, 0, sizeof tree);
    tree.n_nodes = n_nodes;
    tree.token = tokens_dev;
    for (uint32_t i = 0; i < n_nodes; ++i) tree.parent[i] = parent[i];
    launch_pdl(k_spec_accept, dim3(1), dim3(32), 0, ctx->stream, hs.node_stats, hs.child_z, tree, inv_t, seed, step, force_accept,
                                            hs.record);
    CTOX_CUDA(ctx, cudaGetLastError());
    *record_dev = hs.record;
    return CTOX_OK;
}

ctox_status argmax_enqueue(ctox_ctx *ctx, const float *logits_dev, uint32_t n, const uint32_t *row_ids_dev,
                           uint32_t row_offset, uint32_t *token_dev, uint32_t *status_dev) {
    HeadScratch hs;
    ctox_status rc = head_scratch(ctx, hs);
    if (rc) return rc;
    const bool tp = ctx->tp_world > 1;
    if (n == 0) {  // an empty shard of a tensor-parallel draft head
        if (!tp) return fail(ctx, CTOX_INVALID_ARTIFACT, "greedy logits are empty");
        CTOX_CUDA(ctx, cudaMemsetAsync(hs.argmax_send, 0, sizeof(ArgmaxPartial), ctx->stream));
    } else {
        uint32_t grid = (n + kHeadThreads * 4 - 1) / (kHeadThreads * 4);
        if (grid > kHeadGridMax) grid = kHeadGridMax;
        if (grid == 0) grid = 1;
        launch_pdl(k_argmax_partial, dim3(grid), dim3(kHeadThreads), 0, ctx->stream, logits_dev, n, hs.argmax_parts);
        launch_pdl(k_argmax_final, dim3(1), dim3(32), 0, ctx->stream, hs.argmax_parts, grid, row_ids_dev, row_offset,
                                                  tp ? nullptr : token_dev, tp ? nullptr : status_dev,
                                                  tp ? hs.argmax_send : nullptr);
    }
    if (tp) {
        rc = tp_all_gather(ctx, hs.argmax_send, hs.argmax_gathered, sizeof(ArgmaxPartial));
        if (rc) return rc;
        launch_pdl(k_argmax_ranks, dim3(1), dim3(32), 0, ctx->stream, hs.argmax_gathered, (uint32_t)ctx->tp_world, token_dev, status_dev);
    }
    CTOX_CUDA(ctx, cudaGetLastError());
    return CTOX_OK;
}

// Tensor-parallel vocabulary: exchanges the per-rank statistics and leaves the merged ones where
// head_accept_enqueue reads them. shard_rows = vocabulary rows per rank.
ctox_status head_tp_merge_enqueue(ctox_ctx *ctx, uint32_t n_nodes, const int32_t *parent,
                                  const uint32_t *tokens_dev, uint32_t shard_rows) {
    if (ctx->tp_world <= 1) return CTOX_OK;
    if ((uint32_t)ctx->tp_world > kMaxTpWorld) return fail(ctx, CTOX_SHAPE, "tensor-parallel group larger than %u", kMaxTpWorld);
    HeadScratch hs;
    ctox_status rc = head_scratch(ctx, hs);
    if (rc) return rc;
    rc = tp_all_gather(ctx, hs.node_stats, hs.gathered, sizeof(RankStats));
    if (rc) return rc;
    TreeDesc tree;
    memset(&tree, 0, sizeof tree);
    tree.n_nodes = n_nodes;
    tree.token = tokens_dev;
    for (uint32_t i = 0; i < n_nodes; ++i) tree.parent[i] = parent[i];
    launch_pdl(k_head_merge_ranks, dim3(1), dim3(32), 0, ctx->stream, hs.gathered, (uint32_t)ctx->tp_world, shard_rows, tree,
                                                  (RankStats *)hs.node_stats);
    CTOX_CUDA(ctx, cudaGetLastError());
    return CTOX_OK;
}

}  // namespace ctox

extern "C" {

ctox_status ctox_lmhead_verify(ctox_matvec *mv, const void *hidden_dev, uint32_t hidden_dtype,
                               uint64_t hidden_stride, uint32_t n_nodes, const int32_t *parent,
                               const uint32_t *token, float temperature, uint64_t seed, uint64_t step,
                               uint32_t vocab, float *logits_out_dev, ctox_spec_record *record) {
    if (!mv) return CTOX_INVALID_STATE;
    ctox_ctx *ctx = mv->ctx;
    if (!hidden_dev || !parent || !token || !record) return fail(ctx, CTOX_SHAPE, "lmhead_verify: null pointer");
    if (n_nodes == 0 || n_nodes > kMaxNodes)
        return fail(ctx, CTOX_SHAPE, "lmhead_verify: n_nodes must be 1..%d, got %u", kMaxNodes, n_nodes);
    if (mv->parts.size() != 1)
        return fail(ctx, CTOX_UNSUPPORTED_OPERATION, "lmhead_verify needs a pure Q2 or Q4 lm_head");
    if (hidden_dtype != CTOX_F32 && hidden_dtype != CTOX_BF16)
        return fail(ctx, CTOX_UNSUPPORTED_DTYPE, "lmhead_verify: hidden dtype %u", hidden_dtype);
    if (hidden_stride < mv->columns) return fail(ctx, CTOX_SHAPE, "lmhead_verify: stride shorter than a row");
    if (!std::isfinite(temperature) || temperature < 0.f)
        return fail(ctx, CTOX_INVALID_ARTIFACT, "temperature must be finite and non-negative");
    const uint32_t rows = vocab ? vocab : (uint32_t)mv->rows;
    if (rows > mv->rows) return fail(ctx, CTOX_SHAPE, "lmhead_verify: vocab %u exceeds %llu rows", vocab,
                                     (unsigned long long)mv->rows);
    if (parent[0] != -1) return fail(ctx, CTOX_SHAPE, "lmhead_verify: node 0 must be the root");
    for (uint32_t i = 1; i < n_nodes; ++i) {
        if (parent[i] < 0 || (uint32_t)parent[i] >= i)
            return fail(ctx, CTOX_SHAPE, "lmhead_verify: parent[%u] = %d is not an earlier node", i, parent[i]);
        if (token[i] >= rows) return fail(ctx, CTOX_SHAPE, "lmhead_verify: draft token %u out of range", token[i]);
    }
    const float inv_t = temperature > 0.f ? 1.0f / temperature : 0.f;
    if (temperature > 0.f && !std::isfinite(inv_t))
        return fail(ctx, CTOX_INVALID_ARTIFACT, "inverse temperature must be finite");
    CTOX_CUDA(ctx, cudaSetDevice(ctx->device));
    HeadScratch hs;
    ctox_status rc = head_scratch(ctx, hs);
    if (rc) return rc;
    rc = ensure_pinned(ctx, sizeof(ctox_spec_record) + kMaxNodes * sizeof(uint32_t));
    if (rc) return rc;
    uint32_t *tok_pinned = (uint32_t *)((uint8_t *)ctx->pinned + sizeof(ctox_spec_record));
    memcpy(tok_pinned, token, n_nodes * sizeof(uint32_t));
    CTOX_CUDA(ctx, cudaMemcpyAsync(hs.tokens, tok_pinned, n_nodes * sizeof(uint32_t), cudaMemcpyHostToDevice,
                                   ctx->stream));
    const uint32_t per_pass = matvec_positions_per_pass(mv);
    if (per_pass == 0) return fail(ctx, CTOX_MEMORY_BUDGET, "lm_head columns exceed the streaming kernel's budget");
    const size_t esz = hidden_dtype == CTOX_BF16 ? 2 : 4;
    for (uint32_t n0 = 0; n0 < n_nodes; n0 += per_pass) {
        const uint32_t npos = n_nodes - n0 < per_pass ? n_nodes - n0 : per_pass;
        rc = matvec_stream_pass(mv, 0, (const uint8_t *)hidden_dev + (size_t)n0 * hidden_stride * esz,
                                hidden_dtype, npos, hidden_stride);
        if (rc) return rc;
        rc = head_verify_enqueue(mv, n0, npos, n_nodes, parent, hs.tokens, inv_t, seed, step, rows,
                                 logits_out_dev, 0);
        if (rc) return rc;
    }
    ctox_spec_record *rec_dev = nullptr;
    rc = head_accept_enqueue(ctx, n_nodes, parent, hs.tokens, inv_t, seed, step, -1, &rec_dev);
    if (rc) return rc;
    CTOX_CUDA(ctx, cudaMemcpyAsync(ctx->pinned, rec_dev, sizeof(ctox_spec_record), cudaMemcpyDeviceToHost,
                                   ctx->stream));
    CTOX_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    memcpy(record, ctx->pinned, sizeof(ctox_spec_record));
    if (record->status) return fail(ctx, CTOX_INVALID_STATE, "lm_head produced a non-finite logit");
    return CTOX_OK;
}

}  // extern "C"
