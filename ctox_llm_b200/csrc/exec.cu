// Decode executor: the target model pass, the MTP draft chain, verification and the
// speculative state transaction, as one sequence of kernels on the context's stream.
//
// Reference behaviour: trait ModelExecutor (engine.rs:322-362); CPU oracle executor
// decoder.rs:1278-1458 (draft, verify, commit by replay); CUDA candidate
// backend/cuda_executor.rs:797-1073 over backend/cuda_graph.rs (4 chained MTP drafts, one
// 5-row verify pass, acceptance on the device, one small host read per block,
// restore + replay on a partial acceptance, cuda_graph.rs:3166-3292,4962-5003).
//
// What is different here: a verify pass keeps everything it needs to commit ANY accepted
// prefix without re-running projections. Attention layers only advance a token count; linear
// layers write the recurrent state of the whole pass into a second buffer (flip on full
// acceptance) and keep the pass's conv inputs and (q, k, v, g, beta), so a partial acceptance
// re-scans the recurrence alone (~6 MB per layer) instead of replaying whole model passes.
//
// Tensor parallelism (no counterpart in the reference): when the context belongs to a group of W
// GPUs, every rank holds 1/W of the heads, of the FFN width and of the vocabulary. Fan-out
// matrices are split by rows, the projections back to the hidden width by columns; their partial
// results are summed over the group (2 all-reduces of m x hidden floats per layer). The residual
// stream, the norms, the embedding and the small MTP input projection are replicated. The head
// exchanges per-rank statistics (one all-gather per block), never logits.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <algorithm>
#include <chrono>
#include <cmath>
#include <cstdlib>
#include <vector>

#include "common.cuh"
#include "layers.cuh"
#include "matvec.cuh"

namespace ctox {
constexpr uint32_t kMaxPass = 8;  // positions per pass (verify rows / prefill chunk)

struct LayerW {
    bool full = false;
    float *in_ln = nullptr, *post_ln = nullptr;
    ctox_matvec *in_fan = nullptr, *out = nullptr, *gate_up = nullptr, *down = nullptr;
    float *conv_w = nullptr, *a_log = nullptr, *dt_bias = nullptr, *lin_norm = nullptr;
    float *q_norm = nullptr, *k_norm = nullptr;
};

struct LayerS {
    float *conv_state = nullptr;                  // [channels][kernel], committed
    float *delta[2] = {nullptr, nullptr};         // [heads][128][128]; delta[cur] is committed
    int cur = 0;
    float *conv_in = nullptr;                     // [kMaxPass][channels] inputs of the last pass
    float *q = nullptr, *k = nullptr, *v = nullptr, *g = nullptr, *beta = nullptr;  // last pass
    void *k_cache = nullptr, *v_cache = nullptr;  // [slots][kv_heads][head_dim]
};
}  // namespace ctox

using namespace ctox;

struct ctox_exec {
    ctox_ctx *ctx = nullptr;
    ctox_model_config cfg{};  // this rank's shard: heads and FFN width divided by the group size
    uint32_t tp_world = 1, tp_rank = 0;
    uint32_t vocab_l = 0, vocab_off = 0;      // rows of lm_head on this rank
    uint32_t kv_heads_global = 0;             // KV heads of the unsharded model
    uint32_t draft_lo = 0, draft_n = 0;       // this rank's range of the draft id table
    std::vector<uint32_t> draft_ids_host;
    float *tp_buf = nullptr;                  // [kMaxPass][hidden] vector being summed over the group
    uint32_t n_layers = 0;  // target layers; index n_layers is the MTP layer when present
    uint32_t key_width = 0, value_width = 0, channels = 0, q_width = 0, kv_width = 0;
    std::vector<LayerW> w;
    std::vector<LayerS> s;
    ctox_matvec *embed = nullptr, *lm_head = nullptr, *mtp_fc = nullptr, *draft_head = nullptr;
    float *final_norm = nullptr, *mtp_norm_e = nullptr, *mtp_norm_h = nullptr, *mtp_norm = nullptr;
    uint32_t *draft_ids = nullptr;  // device, [draft_vocab]
    CommitLayer *commit_table = nullptr;  // device, one entry per linear-attention layer
    uint32_t n_linear = 0;
    bool lm_head_is_embed = false;
    // session
    uint64_t position = 0;     // tokens consumed by the target so far
    bool have_hidden = false;  // hist_hidden[0 .. hist_n) holds the final hidden of the last hist_n positions
    uint32_t hist_n = 0;       // committed positions of the last block (1..kMaxPass)
    uint32_t hist_tokens[kMaxPass] = {0};  // tokens at positions position-hist_n+1 .. position-1 (drafts accepted)
    uint64_t step_counter = 0;
    bool warmed = false, keep_logits = false;
    // Speculative transaction (engine.rs:322-362): an MTP decode resolves and commits its accepted
    // prefix on the device and leaves the count here until commit_speculative confirms it.
    int32_t pending = -1;
    double last_enqueue_us = 0.0;  // host time the last decode spent enqueuing before it waited for the device
    // Optional device times of the phases of a decode call (events at the phase boundaries):
    // drafting, target pass, head + acceptance, commit.
    bool phase_timing = false;
    cudaEvent_t phase_ev[6] = {};
    float phase_ms[4] = {0.f, 0.f, 0.f, 0.f};
    bool commit_timed = false;
    // A device error or a failed call after work was enqueued leaves the session state undefined:
    // every call fails until reset_session (engine.rs:594-611 invalidates the session the same way).
    bool poisoned = false;
    // evidence of the last decode call (with keep_logits): the MTP layer's final hidden of every
    // (token, hidden) pair it ran, in order, and the logits of every draft
    float *mtp_trace = nullptr, *draft_trace = nullptr;
    uint32_t mtp_trace_n = 0, draft_trace_n = 0, draft_rows = 0;
    // buffers ([kMaxPass] rows each)
    float *h = nullptr, *final_hidden = nullptr, *hist_hidden = nullptr, *embed_rows = nullptr;
    float *mtp_h = nullptr, *mtp_hidden = nullptr;
    float *aq = nullptr, *agate = nullptr, *attn_ws = nullptr;
    float *lz = nullptr, *lcore = nullptr, *norm_scratch = nullptr;
    float *draft_logits = nullptr, *logits = nullptr;
    uint32_t *tokens_dev = nullptr;  // [kMaxPass + 1]: verify inputs = [token, drafts...]
    uint32_t *mtp_tokens_dev = nullptr;
    uint32_t *page_table = nullptr, *mtp_page_table = nullptr;
    uint32_t attn_splits_max = kAttnMaxSplits;
    uint64_t model_bytes = 0, session_bytes = 0;
    std::vector<std::pair<void *, size_t>> owned;  // tracked raw allocations (vectors, buffers, states)
};

namespace {

ctox_status xalloc(ctox_exec *e, void **p, size_t bytes, bool session, bool zero = true) {
    ctox_status rc = dev_alloc(e->ctx, p, bytes);
    if (rc) return rc;
    e->owned.emplace_back(*p, bytes);
    (session ? e->session_bytes : e->model_bytes) += bytes;
    if (zero) CTOX_CUDA(e->ctx, cudaMemsetAsync(*p, 0, bytes, e->ctx->stream));
    return CTOX_OK;
}

bool layer_is_full(const ctox_exec *e, uint32_t l) {
    if (l >= e->n_layers) return true;  // the MTP layer is a full-attention layer
    return (l + 1) % e->cfg.full_attention_interval == 0;
}

size_t kv_elem(const ctox_exec *e) { return e->cfg.kv_dtype == CTOX_BF16 ? 2 : 4; }

}  // namespace

extern "C" {

ctox_status ctox_exec_create(ctox_ctx *ctx, const ctox_model_config *c_global, ctox_exec **out) {
    if (!ctx || !c_global || !out) return CTOX_INVALID_STATE;
    *out = nullptr;
    const uint32_t W = (uint32_t)ctx->tp_world, R = (uint32_t)ctx->tp_rank;
    ctox_model_config local = *c_global;
    if (W > 1) {
        const ctox_model_config &g = *c_global;
        if (g.num_attention_heads % W || g.linear_num_key_heads % W || g.linear_num_value_heads % W ||
            g.intermediate_size % (64 * W) || g.vocab_size % W || g.num_key_value_heads == 0 ||
            (g.num_key_value_heads % W && W % g.num_key_value_heads))
            return fail(ctx, CTOX_SHAPE, "executor: the model does not split over %u GPUs", W);
        local.num_attention_heads /= W;
        // fewer KV heads than ranks: neighbouring ranks hold a copy of the same KV head
        local.num_key_value_heads = g.num_key_value_heads >= W ? g.num_key_value_heads / W : 1;
        local.linear_num_key_heads /= W;
        local.linear_num_value_heads /= W;
        local.intermediate_size /= W;
    }
    const ctox_model_config *c = &local;
    if (c->hidden_size == 0 || c->hidden_size % 64 || c->intermediate_size % 64 || c->vocab_size == 0 ||
        c->num_hidden_layers == 0 || c->full_attention_interval == 0)
        return fail(ctx, CTOX_SHAPE, "executor: hidden/intermediate sizes must be non-zero multiples of 64");
    if (c->num_key_value_heads == 0 || c->num_attention_heads % c->num_key_value_heads || c->head_dim % 64 ||
        c->head_dim > 256 || c->rotary_dim > c->head_dim || c->rotary_dim % 2 ||
        (c->num_attention_heads * c->head_dim) % 256 ||
        c->num_attention_heads / c->num_key_value_heads * kMaxPass > 48)
        return fail(ctx, CTOX_SHAPE, "executor: unsupported attention geometry");
    if (c->linear_key_head_dim != 128 || c->linear_value_head_dim != 128 || c->linear_num_key_heads == 0 ||
        c->linear_num_value_heads % c->linear_num_key_heads || (c->linear_num_value_heads * 128) % 256 ||
        c->linear_conv_kernel_dim == 0 || c->linear_conv_kernel_dim > 8)
        return fail(ctx, CTOX_SHAPE, "executor: unsupported linear-attention geometry");
    if (c->kv_dtype != CTOX_F32 && c->kv_dtype != CTOX_BF16)
        return fail(ctx, CTOX_UNSUPPORTED_DTYPE, "executor: kv dtype %u", c->kv_dtype);
    if (c->max_draft_tokens + 1 > kMaxPass || c->mtp_num_hidden_layers > 1 || c->kv_page_tokens == 0 ||
        c->max_context_tokens < 2 * kMaxPass || c->draft_vocab > c->vocab_size)
        return fail(ctx, CTOX_SHAPE, "executor: unsupported draft, page or context configuration");
    CTOX_CUDA(ctx, cudaSetDevice(ctx->device));
    ctox_exec *e = new ctox_exec();
    e->ctx = ctx;
    e->cfg = *c;
    e->n_layers = c->num_hidden_layers;
    e->tp_world = W;
    e->tp_rank = R;
    e->kv_heads_global = c_global->num_key_value_heads;
    e->vocab_l = c->vocab_size / W;
    e->vocab_off = R * e->vocab_l;
    e->key_width = c->linear_num_key_heads * 128;
    e->value_width = c->linear_num_value_heads * 128;
    e->channels = 2 * e->key_width + e->value_width;
    e->q_width = c->num_attention_heads * c->head_dim;
    e->kv_width = c->num_key_value_heads * c->head_dim;
    // one CTA per (KV head, context split): fill the SMs once
    e->attn_splits_max = (uint32_t)ctx->sm_count / c->num_key_value_heads;
    if (e->attn_splits_max < 1) e->attn_splits_max = 1;
    if (e->attn_splits_max > (uint32_t)kAttnMaxSplits) e->attn_splits_max = kAttnMaxSplits;
    if (const char *cap = getenv("CTOX_ATTN_SPLITS_MAX")) {  // fewer, longer splits (tests: many tiles per CTA)
        const long v = strtol(cap, nullptr, 10);
        if (v >= 1 && (uint32_t)v < e->attn_splits_max) e->attn_splits_max = (uint32_t)v;
    }
    const uint32_t total_layers = e->n_layers + c->mtp_num_hidden_layers;
    e->w.resize(total_layers);
    e->s.resize(total_layers);
    for (uint32_t l = 0; l < total_layers; ++l) e->w[l].full = layer_is_full(e, l);
    *out = e;
    return CTOX_OK;
}

ctox_status ctox_exec_destroy(ctox_exec *e) {
    if (!e) return CTOX_OK;
    cudaSetDevice(e->ctx->device);
    cudaStreamSynchronize(e->ctx->stream);
    for (auto &lw : e->w) {
        ctox_matvec_destroy(lw.in_fan);
        ctox_matvec_destroy(lw.out);
        ctox_matvec_destroy(lw.gate_up);
        ctox_matvec_destroy(lw.down);
    }
    if (!e->lm_head_is_embed) ctox_matvec_destroy(e->lm_head);
    ctox_matvec_destroy(e->embed);
    ctox_matvec_destroy(e->mtp_fc);
    ctox_matvec_destroy(e->draft_head);
    for (auto &o : e->owned) dev_free(e->ctx, o.first, o.second);
    for (auto &ev : e->phase_ev)
        if (ev) cudaEventDestroy(ev);
    delete e;
    return CTOX_OK;
}

ctox_status ctox_exec_allocated_bytes(const ctox_exec *e, uint64_t *model, uint64_t *session) {
    if (!e) return CTOX_INVALID_STATE;
    uint64_t mats = 0;
    auto add = [&](ctox_matvec *mv) {
        if (mv) mats += mv->device_bytes;
    };
    for (auto &lw : e->w) {
        add(lw.in_fan);
        add(lw.out);
        add(lw.gate_up);
        add(lw.down);
    }
    add(e->embed);
    if (!e->lm_head_is_embed) add(e->lm_head);
    add(e->mtp_fc);
    add(e->draft_head);
    if (model) *model = e->model_bytes + mats;
    if (session) *session = e->session_bytes;
    return CTOX_OK;
}

}  // extern "C"

namespace {

struct Shape {
    uint64_t rows, cols;
};

bool matrix_slot(ctox_exec *e, uint32_t layer, uint32_t tensor, ctox_matvec ***slot, Shape *shape) {
    const ctox_model_config &c = e->cfg;
    const uint64_t H = c.hidden_size, F = c.intermediate_size;
    if (layer == CTOX_LAYER_GLOBAL) {
        switch (tensor) {
            case CTOX_T_EMBED: *slot = &e->embed; *shape = {c.vocab_size, H}; return true;
            case CTOX_T_LM_HEAD: *slot = &e->lm_head; *shape = {e->vocab_l, H}; return true;
            case CTOX_T_MTP_FC:
                if (!c.mtp_num_hidden_layers) return false;
                *slot = &e->mtp_fc; *shape = {H, 2 * H}; return true;
            default: return false;
        }
    }
    if (layer >= e->w.size()) return false;
    LayerW &lw = e->w[layer];
    switch (tensor) {
        case CTOX_T_ATTN_QKV:
            if (!lw.full) return false;
            *slot = &lw.in_fan; *shape = {2ull * e->q_width + 2ull * e->kv_width, H}; return true;
        case CTOX_T_ATTN_O:
            if (!lw.full) return false;
            *slot = &lw.out; *shape = {H, e->q_width}; return true;
        case CTOX_T_LIN_IN:
            if (lw.full) return false;
            *slot = &lw.in_fan;
            *shape = {(uint64_t)e->channels + e->value_width + 2ull * c.linear_num_value_heads, H};
            return true;
        case CTOX_T_LIN_OUT:
            if (lw.full) return false;
            *slot = &lw.out; *shape = {H, e->value_width}; return true;
        case CTOX_T_MLP_GATE_UP: *slot = &lw.gate_up; *shape = {2 * F, H}; return true;
        case CTOX_T_MLP_DOWN: *slot = &lw.down; *shape = {H, F}; return true;
        default: return false;
    }
}

bool vector_slot(ctox_exec *e, uint32_t layer, uint32_t tensor, float ***slot, uint64_t *n) {
    const ctox_model_config &c = e->cfg;
    if (layer == CTOX_LAYER_GLOBAL) {
        switch (tensor) {
            case CTOX_T_FINAL_NORM: *slot = &e->final_norm; *n = c.hidden_size; return true;
            case CTOX_T_MTP_NORM_E: *slot = &e->mtp_norm_e; *n = c.hidden_size; return true;
            case CTOX_T_MTP_NORM_H: *slot = &e->mtp_norm_h; *n = c.hidden_size; return true;
            case CTOX_T_MTP_NORM: *slot = &e->mtp_norm; *n = c.hidden_size; return true;
            default: return false;
        }
    }
    if (layer >= e->w.size()) return false;
    LayerW &lw = e->w[layer];
    switch (tensor) {
        case CTOX_T_INPUT_NORM: *slot = &lw.in_ln; *n = c.hidden_size; return true;
        case CTOX_T_POST_NORM: *slot = &lw.post_ln; *n = c.hidden_size; return true;
        case CTOX_T_Q_NORM: if (!lw.full) return false; *slot = &lw.q_norm; *n = c.head_dim; return true;
        case CTOX_T_K_NORM: if (!lw.full) return false; *slot = &lw.k_norm; *n = c.head_dim; return true;
        case CTOX_T_CONV_W:
            if (lw.full) return false;
            *slot = &lw.conv_w; *n = (uint64_t)e->channels * c.linear_conv_kernel_dim; return true;
        case CTOX_T_A_LOG: if (lw.full) return false; *slot = &lw.a_log; *n = c.linear_num_value_heads; return true;
        case CTOX_T_DT_BIAS: if (lw.full) return false; *slot = &lw.dt_bias; *n = c.linear_num_value_heads; return true;
        case CTOX_T_LIN_NORM: if (lw.full) return false; *slot = &lw.lin_norm; *n = 128; return true;
        default: return false;
    }
}

}  // namespace

extern "C" {

ctox_status ctox_exec_load_matrix(ctox_exec *e, uint32_t layer, uint32_t tensor, const ctox_fused_matvec_op *op) {
    if (!e || !op) return CTOX_INVALID_STATE;
    ctox_ctx *ctx = e->ctx;
    ctox_matvec **slot = nullptr;
    Shape shape{};
    if (!matrix_slot(e, layer, tensor, &slot, &shape))
        return fail(ctx, CTOX_INVALID_ARTIFACT, "tensor %u is not a matrix of layer %u", tensor, layer);
    if (op->rows != shape.rows || op->columns != shape.cols)
        return fail(ctx, CTOX_SHAPE, "tensor %u of layer %u is %llux%llu, expected %llux%llu", tensor, layer,
                    (unsigned long long)op->rows, (unsigned long long)op->columns,
                    (unsigned long long)shape.rows, (unsigned long long)shape.cols);
    if (op->dtype != CTOX_Q2B64 && op->dtype != CTOX_Q4B64)
        return fail(ctx, CTOX_UNSUPPORTED_DTYPE, "executor matrices must be pure Q2_B64 or Q4_B64");
    if (op->activation != CTOX_ACT_IDENTITY || op->bias)
        return fail(ctx, CTOX_UNSUPPORTED_OPERATION, "executor matrices carry no bias or activation");
    if (*slot) {
        ctox_matvec_destroy(*slot);
        *slot = nullptr;
    }
    const bool keep = tensor == CTOX_T_EMBED || (tensor == CTOX_T_LM_HEAD && e->cfg.draft_vocab);
    e->warmed = false;
    return ctox_matvec_prepare(ctx, op, keep ? CTOX_PREPARE_KEEP_CANONICAL : 0, slot);
}

ctox_status ctox_exec_load_vector(ctox_exec *e, uint32_t layer, uint32_t tensor, const float *values, uint64_t n) {
    if (!e || !values) return CTOX_INVALID_STATE;
    ctox_ctx *ctx = e->ctx;
    if (layer == CTOX_LAYER_GLOBAL && tensor == CTOX_T_DRAFT_IDS) {
        if (n != e->cfg.draft_vocab || n == 0)
            return fail(ctx, CTOX_SHAPE, "draft id table has %llu entries, expected %u", (unsigned long long)n,
                        e->cfg.draft_vocab);
        const uint32_t *ids = reinterpret_cast<const uint32_t *>(values);
        for (uint64_t i = 0; i < n; ++i)
            if (ids[i] >= e->cfg.vocab_size || (i && ids[i] <= ids[i - 1]))
                return fail(ctx, CTOX_INVALID_ARTIFACT, "draft token ids must be strictly increasing and in range");
        if (!e->draft_ids) {
            ctox_status rc = xalloc(e, (void **)&e->draft_ids, n * 4, false);
            if (rc) return rc;
        }
        CTOX_CUDA(ctx, cudaMemcpyAsync(e->draft_ids, ids, n * 4, cudaMemcpyHostToDevice, ctx->stream));
        CTOX_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
        e->draft_ids_host.assign(ids, ids + n);
        e->warmed = false;
        return CTOX_OK;
    }
    float **slot = nullptr;
    uint64_t expect = 0;
    if (!vector_slot(e, layer, tensor, &slot, &expect))
        return fail(ctx, CTOX_INVALID_ARTIFACT, "tensor %u is not a vector of layer %u", tensor, layer);
    if (n != expect)
        return fail(ctx, CTOX_SHAPE, "tensor %u of layer %u has %llu values, expected %llu", tensor, layer,
                    (unsigned long long)n, (unsigned long long)expect);
    for (uint64_t i = 0; i < n; ++i)
        if (!std::isfinite(values[i])) return fail(ctx, CTOX_INVALID_ARTIFACT, "tensor %u has a non-finite value", tensor);
    if (!*slot) {
        ctox_status rc = xalloc(e, (void **)slot, n * sizeof(float), false);
        if (rc) return rc;
    }
    CTOX_CUDA(ctx, cudaMemcpyAsync(*slot, values, n * sizeof(float), cudaMemcpyHostToDevice, ctx->stream));
    CTOX_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    e->warmed = false;
    return CTOX_OK;
}

}  // extern "C"

// ------------------------------------------------------------------ synthetic tensors, draft head
namespace ctox {

__device__ __forceinline__ uint64_t mix64(uint64_t x) {
    x += 0x9E3779B97F4A7C15ull;
    x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
    x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
    return x ^ (x >> 31);
}

// Where the rows of a rank's shard sit in the unsharded matrix: up to 6 runs of consecutive rows
// (fan-out groups are several matrices, each split by heads). A single GPU uses one identity run.
struct RowMap {
    uint32_t n;
    uint64_t local_start[6], global_start[6];
};
__device__ __forceinline__ uint64_t global_row(const RowMap &map, uint64_t row) {
    uint32_t seg = 0;
    for (uint32_t i = 1; i < map.n; ++i)
        if (row >= map.local_start[i]) seg = i;
    return map.global_start[seg] + (row - map.local_start[seg]);
}

// Canonical blocks [f16 scale][codes]: codes uniform, scale drawn from a 4096-entry quantile table.
// Every block is a function of its position in the UNSHARDED matrix (global row, global column
// block), so the shards of a tensor-parallel group are slices of the one-GPU model.
__global__ void k_fill_canonical(uint8_t *__restrict__ out, uint64_t blocks, uint32_t block_bytes,
                                 const uint16_t *__restrict__ table, uint64_t seed, uint32_t blocks_per_row,
                                 uint32_t global_blocks_per_row, uint32_t col_block0, RowMap map) {
    const uint64_t b = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (b >= blocks) return;
    uint8_t *p = out + b * block_bytes;
    const uint64_t gid = global_row(map, b / blocks_per_row) * global_blocks_per_row + col_block0 + b % blocks_per_row;
    uint64_t r = mix64(seed ^ (gid * 0x100000001B3ull));
    const uint16_t sc = table[r & 4095];
    p[0] = (uint8_t)(sc & 0xff);
    p[1] = (uint8_t)(sc >> 8);
    for (uint32_t i = 2; i < block_bytes; i += 8) {
        r = mix64(r + i);
        for (uint32_t j = 0; j < 8 && i + j < block_bytes; ++j) p[i + j] = (uint8_t)(r >> (8 * j));
    }
}

// out[i] for the global index offset + i (columns) or the mapped row (rows, use_map).
__global__ void k_fill_uniform_f16(float *__restrict__ out, uint64_t n, float lo, float hi, uint64_t seed,
                                   uint64_t offset, int use_map, RowMap map) {
    const uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const uint64_t gi = use_map ? global_row(map, i) : offset + i;
    const float u = (float)(mix64(seed ^ (gi * 0x9E3779B1ull)) >> 40) * (1.0f / 16777216.0f);
    out[i] = __half2float(__float2half_rn(lo + (hi - lo) * u));  // what an f16 payload would hold
}

template <typename T>
__global__ void k_fill_normal(T *__restrict__ out, uint64_t n, float mean, float std, uint64_t seed) {
    const uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const uint64_t r = mix64(seed ^ (i * 0xD6E8FEB86659FD93ull));
    const float u1 = ((float)(r >> 40) + 0.5f) * (1.0f / 16777216.0f);
    const float u2 = (float)((r >> 16) & 0xffffff) * (1.0f / 16777216.0f);
    const float z = sqrtf(-2.0f * logf(u1)) * cosf(6.28318530718f * u2);
    const float v = mean + std * z;
    if (sizeof(T) == 2)
        reinterpret_cast<__nv_bfloat16 *>(out)[i] = __float2bfloat16_rn(v);
    else
        reinterpret_cast<float *>(out)[i] = v;
}

// Values of a per-item vector (per_item values per row of `map`), a function of the global index.
__global__ void k_fill_normal_mapped(float *__restrict__ out, uint64_t n, uint32_t per_item, float mean, float std,
                                     uint64_t seed, RowMap map) {
    const uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const uint64_t gi = global_row(map, i / per_item) * per_item + i % per_item;
    const uint64_t r = mix64(seed ^ (gi * 0xD6E8FEB86659FD93ull));
    const float u1 = ((float)(r >> 40) + 0.5f) * (1.0f / 16777216.0f);
    const float u2 = (float)((r >> 16) & 0xffffff) * (1.0f / 16777216.0f);
    out[i] = mean + std * sqrtf(-2.0f * logf(u1)) * cosf(6.28318530718f * u2);
}

__global__ void k_gather_rows(const uint8_t *__restrict__ src, const uint32_t *__restrict__ ids,
                              uint32_t id_offset, uint32_t row_bytes, uint32_t n, uint8_t *__restrict__ dst) {
    const uint32_t r = blockIdx.x;
    if (r >= n) return;
    const uint8_t *s = src + (size_t)(ids[r] - id_offset) * row_bytes;
    uint8_t *d = dst + (size_t)r * row_bytes;
    for (uint32_t i = threadIdx.x * 2; i < row_bytes; i += blockDim.x * 2)
        *reinterpret_cast<uint16_t *>(d + i) = *reinterpret_cast<const uint16_t *>(s + i);
}

__global__ void k_gather_f32(const float *__restrict__ src, const uint32_t *__restrict__ ids,
                             uint32_t id_offset, uint32_t n, float *__restrict__ dst) {
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) dst[i] = src[ids[i] - id_offset];
}

__global__ void k_iota_u32(uint32_t *out, uint32_t n, uint32_t stride) {
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = i * stride;
}

}  // namespace ctox

namespace {

// Inverse normal CDF (Acklam's rational approximation, |error| < 1.2e-9).
double inv_norm_cdf(double p) {
    static const double a[] = {-3.969683028665376e+01, 2.209460984245205e+02, -2.759285104469687e+02,
                               1.383577518672690e+02, -3.066479806614716e+01, 2.506628277459239e+00};
    static const double b[] = {-5.447609879822406e+01, 1.615858368580409e+02, -1.556989798598866e+02,
                               6.680131188771972e+01, -1.328068155288572e+01};
    static const double c[] = {-7.784894002430293e-03, -3.223964580411365e-01, -2.400758277161838e+00,
                               -2.549732539343734e+00, 4.374664141464968e+00, 2.938163982698783e+00};
    static const double d[] = {7.784695709041462e-03, 3.224671290700398e-01, 2.445134137142996e+00,
                               3.754408661907416e+00};
    if (p < 0.02425) {
        const double q = std::sqrt(-2 * std::log(p));
        return (((((c[0] * q + c[1]) * q + c[2]) * q + c[3]) * q + c[4]) * q + c[5]) /
               ((((d[0] * q + d[1]) * q + d[2]) * q + d[3]) * q + 1);
    }
    if (p > 1 - 0.02425) return -inv_norm_cdf(1 - p);
    const double q = p - 0.5, r = q * q;
    return (((((a[0] * r + a[1]) * r + a[2]) * r + a[3]) * r + a[4]) * r + a[5]) * q /
           (((((b[0] * r + b[1]) * r + b[2]) * r + b[3]) * r + b[4]) * r + 1);
}

uint16_t f32_to_f16_bits(float f) {
    __half h = __float2half_rn(f);
    uint16_t u;
    memcpy(&u, &h, 2);
    return u;
}

// One run of rows: local rows [.., ..+count) are global rows [global, global+count).
struct RowRun {
    uint64_t global, count;
};

// A matrix of `rows` x `cols` that is the slice (row runs, columns [col0, col0 + cols)) of an unsharded
// matrix with global_cols columns: codes and recovery scales follow the global indices.
ctox_status synth_matrix(ctox_exec *e, int dt, uint64_t cols, uint64_t global_cols, uint64_t col0,
                         std::initializer_list<RowRun> runs, const uint16_t *table_dev, uint64_t seed, uint32_t flags,
                         ctox_matvec **out) {
    ctox_ctx *ctx = e->ctx;
    RowMap map{};
    uint64_t rows = 0;
    for (const RowRun &r : runs) {
        if (map.n >= 6) return fail(ctx, CTOX_SHAPE, "synthetic matrix: too many row runs");
        map.local_start[map.n] = rows;
        map.global_start[map.n] = r.global;
        rows += r.count;
        ++map.n;
    }
    const uint32_t bb = dt ? 34 : 18;
    const uint64_t blocks = rows * (cols / 64);
    uint8_t *canon = nullptr;
    float *s_in = nullptr, *s_out = nullptr;
    ctox_status rc = dev_alloc(ctx, (void **)&canon, blocks * bb);
    if (!rc) rc = dev_alloc(ctx, (void **)&s_in, cols * 4);
    if (!rc) rc = dev_alloc(ctx, (void **)&s_out, rows * 4);
    if (rc) return rc;
    k_fill_canonical<<<(unsigned)((blocks + 255) / 256), 256, 0, ctx->stream>>>(
        canon, blocks, bb, table_dev, seed, (uint32_t)(cols / 64), (uint32_t)(global_cols / 64), (uint32_t)(col0 / 64), map);
    k_fill_uniform_f16<<<(unsigned)((cols + 255) / 256), 256, 0, ctx->stream>>>(s_in, cols, 0.75f, 1.25f,
                                                                             seed ^ 0x5151, col0, 0, map);
    k_fill_uniform_f16<<<(unsigned)((rows + 255) / 256), 256, 0, ctx->stream>>>(s_out, rows, 0.75f, 1.25f,
                                                                             seed ^ 0xA0A0, 0, 1, map);
    CTOX_CUDA(ctx, cudaGetLastError());
    return matvec_create_device(ctx, dt, rows, cols, canon, blocks * bb, s_in, s_out, flags, out);
}

ctox_status synth_vector(ctox_exec *e, float **slot, uint64_t n, float mean, float std, uint64_t seed) {
    if (!*slot) {
        ctox_status rc = xalloc(e, (void **)slot, n * 4, false);
        if (rc) return rc;
    }
    k_fill_normal<float><<<(unsigned)((n + 255) / 256), 256, 0, e->ctx->stream>>>(*slot, n, mean, std, seed);
    return CTOX_OK;
}

ctox_status synth_vector_sharded(ctox_exec *e, float **slot, uint32_t per_item, std::initializer_list<RowRun> runs,
                                 float mean, float std, uint64_t seed) {
    RowMap map{};
    uint64_t items = 0;
    for (const RowRun &r : runs) {
        map.local_start[map.n] = items;
        map.global_start[map.n] = r.global;
        items += r.count;
        ++map.n;
    }
    const uint64_t n = items * per_item;
    if (!*slot) {
        ctox_status rc = xalloc(e, (void **)slot, n * 4, false);
        if (rc) return rc;
    }
    k_fill_normal_mapped<<<(unsigned)((n + 255) / 256), 256, 0, e->ctx->stream>>>(*slot, n, per_item, mean, std, seed, map);
    return CTOX_OK;
}

ctox_status build_draft_head(ctox_exec *e) {
    ctox_ctx *ctx = e->ctx;
    if (e->draft_head) {
        ctox_matvec_destroy(e->draft_head);
        e->draft_head = nullptr;
    }
    if (!e->cfg.draft_vocab) return CTOX_OK;
    if (!e->draft_ids) return fail(ctx, CTOX_INVALID_STATE, "draft vocabulary configured but no id table loaded");
    MatvecPart &p = e->lm_head->parts[0];
    if (!p.canon) return fail(ctx, CTOX_INVALID_STATE, "lm_head canonical bytes are not resident");
    // this rank's rows: the draft ids that fall into its vocabulary shard (ids ascend)
    const auto &ids = e->draft_ids_host;
    if (ids.size() != e->cfg.draft_vocab) return fail(ctx, CTOX_INVALID_STATE, "draft id table is incomplete");
    const uint32_t lo = (uint32_t)(std::lower_bound(ids.begin(), ids.end(), e->vocab_off) - ids.begin());
    const uint32_t hi = (uint32_t)(std::lower_bound(ids.begin(), ids.end(), e->vocab_off + e->vocab_l) - ids.begin());
    e->draft_lo = lo;
    e->draft_n = hi - lo;
    const uint32_t n = e->draft_n;
    if (n == 0) return CTOX_OK;  // no draft token in this shard: the rank only takes part in the merge
    const uint32_t row_bytes = (uint32_t)(e->lm_head->columns / 64) * (p.dt ? 34 : 18);
    uint8_t *canon = nullptr;
    float *s_in = nullptr, *s_out = nullptr;
    ctox_status rc = dev_alloc(ctx, (void **)&canon, (size_t)n * row_bytes);
    if (!rc) rc = dev_alloc(ctx, (void **)&s_in, e->lm_head->columns * 4);
    if (!rc) rc = dev_alloc(ctx, (void **)&s_out, (size_t)n * 4);
    if (rc) return rc;
    k_gather_rows<<<n, 128, 0, ctx->stream>>>(p.canon, e->draft_ids + lo, e->vocab_off, row_bytes, n, canon);
    CTOX_CUDA(ctx, cudaMemcpyAsync(s_in, e->lm_head->s_in, e->lm_head->columns * 4, cudaMemcpyDeviceToDevice,
                                   ctx->stream));
    k_gather_f32<<<(n + 255) / 256, 256, 0, ctx->stream>>>(e->lm_head->s_out, e->draft_ids + lo, e->vocab_off, n,
                                                           s_out);
    CTOX_CUDA(ctx, cudaGetLastError());
    return matvec_create_device(ctx, p.dt, n, e->lm_head->columns, canon, (size_t)n * row_bytes, s_in, s_out, 0,
                                &e->draft_head);
}

}  // namespace

extern "C" {

ctox_status ctox_exec_fill_synthetic(ctox_exec *e, uint64_t seed, float mu, float sigma) {
    if (!e) return CTOX_INVALID_STATE;
    ctox_ctx *ctx = e->ctx;
    CTOX_CUDA(ctx, cudaSetDevice(ctx->device));
    const ctox_model_config &c = e->cfg;
    // f16 block-scale quantile table of the log-normal(mu, sigma)
    std::vector<uint16_t> table(4096);
    for (int i = 0; i < 4096; ++i)
        table[i] = f32_to_f16_bits((float)std::exp(mu + sigma * inv_norm_cdf((i + 0.5) / 4096.0)));
    uint16_t *table_dev = nullptr;
    ctox_status rc = xalloc(e, (void **)&table_dev, 4096 * 2, false, false);
    if (rc) return rc;
    CTOX_CUDA(ctx, cudaMemcpyAsync(table_dev, table.data(), 4096 * 2, cudaMemcpyHostToDevice, ctx->stream));
    CTOX_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    const uint64_t H = c.hidden_size, F = c.intermediate_size;
    uint64_t sd = seed * 1000003ull + 17;
    auto next_seed = [&]() { return sd = sd * 6364136223846793005ull + 1442695040888963407ull; };
#define SYNTH(expr)    \
    do {               \
        rc = (expr);   \
        if (rc) return rc; \
    } while (0)
    auto replace = [&](ctox_matvec **slot) {
        if (*slot) ctox_matvec_destroy(*slot);
        *slot = nullptr;
    };
    if (e->lm_head && !e->lm_head_is_embed) replace(&e->lm_head);
    replace(&e->embed);
    // Shard geometry: this rank's heads, FFN columns and vocabulary rows inside the unsharded model
    // (world 1: everything). Seeds are drawn in the same order on every rank, and every tensor is a
    // function of (seed, global index), so a group's shards are slices of the one-GPU model.
    const uint64_t W = e->tp_world, R = e->tp_rank;
    const uint64_t hd = c.head_dim, QWl = e->q_width, KVl = e->kv_width, QW = QWl * W;
    const uint64_t kv_heads_global = e->kv_heads_global, KV = kv_heads_global * hd;
    const uint64_t kv_head0 = kv_heads_global >= W ? R * c.num_key_value_heads : R * kv_heads_global / W;
    const uint64_t KWl = e->key_width, VWl = e->value_width, KW = KWl * W, VW = VWl * W;
    const uint64_t VHl = c.linear_num_value_heads, VH = VHl * W, CH = 2 * KW + VW, Fl = F, FG = F * W;
    // attention / embedding weights Q4, FFN weights Q2 (the benchmark configuration)
    const uint64_t embed_seed = next_seed();
    SYNTH(synth_matrix(e, 1, H, H, 0, {{0, c.vocab_size}}, table_dev, embed_seed, CTOX_PREPARE_KEEP_CANONICAL,
                       &e->embed));
    if (e->tp_world == 1) {
        e->lm_head = e->embed;  // tied: one resident copy serves row gathers and the head
        e->lm_head_is_embed = true;
    } else {  // the embedding is replicated, the head holds this rank's vocabulary rows of the same matrix
        e->lm_head = nullptr;
        e->lm_head_is_embed = false;
        SYNTH(synth_matrix(e, 1, H, H, 0, {{e->vocab_off, e->vocab_l}}, table_dev, embed_seed,
                           CTOX_PREPARE_KEEP_CANONICAL, &e->lm_head));
    }
    SYNTH(synth_vector(e, &e->final_norm, H, 0.f, 0.02f, next_seed()));
    for (uint32_t l = 0; l < e->w.size(); ++l) {
        LayerW &lw = e->w[l];
        replace(&lw.in_fan);
        replace(&lw.out);
        replace(&lw.gate_up);
        replace(&lw.down);
        SYNTH(synth_vector(e, &lw.in_ln, H, 0.f, 0.02f, next_seed()));
        SYNTH(synth_vector(e, &lw.post_ln, H, 0.f, 0.02f, next_seed()));
        if (lw.full) {
            // [q + gate per head | k | v]: this rank's query heads and its KV head(s)
            SYNTH(synth_matrix(e, 1, H, H, 0,
                               {{R * 2 * QWl, 2 * QWl}, {2 * QW + kv_head0 * hd, KVl}, {2 * QW + KV + kv_head0 * hd, KVl}},
                               table_dev, next_seed(), 0, &lw.in_fan));
            SYNTH(synth_matrix(e, 1, QWl, QW, R * QWl, {{0, H}}, table_dev, next_seed(), 0, &lw.out));
            SYNTH(synth_vector(e, &lw.q_norm, c.head_dim, 0.f, 0.02f, next_seed()));
            SYNTH(synth_vector(e, &lw.k_norm, c.head_dim, 0.f, 0.02f, next_seed()));
        } else {
            // [q | k | v] conv channels, z, a, b: this rank's key heads and value heads
            SYNTH(synth_matrix(e, 1, H, H, 0,
                               {{R * KWl, KWl}, {KW + R * KWl, KWl}, {2 * KW + R * VWl, VWl}, {CH + R * VWl, VWl},
                                {CH + VW + R * VHl, VHl}, {CH + VW + VH + R * VHl, VHl}},
                               table_dev, next_seed(), 0, &lw.in_fan));
            SYNTH(synth_matrix(e, 1, VWl, VW, R * VWl, {{0, H}}, table_dev, next_seed(), 0, &lw.out));
            // per-channel / per-head vectors: generated for the whole model, this rank keeps its part
            SYNTH(synth_vector_sharded(e, &lw.conv_w, c.linear_conv_kernel_dim,
                                       {{R * KWl, KWl}, {KW + R * KWl, KWl}, {2 * KW + R * VWl, VWl}}, 0.f, 0.3f,
                                       next_seed()));
            SYNTH(synth_vector_sharded(e, &lw.a_log, 1, {{R * VHl, VHl}}, 0.f, 0.5f, next_seed()));
            SYNTH(synth_vector_sharded(e, &lw.dt_bias, 1, {{R * VHl, VHl}}, 0.f, 0.5f, next_seed()));
            SYNTH(synth_vector(e, &lw.lin_norm, 128, 1.f, 0.02f, next_seed()));
        }
        SYNTH(synth_matrix(e, 0, H, H, 0, {{R * Fl, Fl}, {FG + R * Fl, Fl}}, table_dev, next_seed(), 0, &lw.gate_up));
        SYNTH(synth_matrix(e, 0, Fl, FG, R * Fl, {{0, H}}, table_dev, next_seed(), 0, &lw.down));
    }
    if (c.mtp_num_hidden_layers) {
        replace(&e->mtp_fc);
        SYNTH(synth_matrix(e, 1, 2 * H, 2 * H, 0, {{0, H}}, table_dev, next_seed(), 0, &e->mtp_fc));
        SYNTH(synth_vector(e, &e->mtp_norm_e, H, 0.f, 0.02f, next_seed()));
        SYNTH(synth_vector(e, &e->mtp_norm_h, H, 0.f, 0.02f, next_seed()));
        SYNTH(synth_vector(e, &e->mtp_norm, H, 0.f, 0.02f, next_seed()));
    }
    if (c.draft_vocab) {
        if (!e->draft_ids) SYNTH(xalloc(e, (void **)&e->draft_ids, (size_t)c.draft_vocab * 4, false));
        const uint32_t stride = c.vocab_size / c.draft_vocab;
        k_iota_u32<<<(c.draft_vocab + 255) / 256, 256, 0, ctx->stream>>>(e->draft_ids, c.draft_vocab, stride);
        e->draft_ids_host.resize(c.draft_vocab);
        for (uint32_t i = 0; i < c.draft_vocab; ++i) e->draft_ids_host[i] = i * stride;
    }
#undef SYNTH
    CTOX_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    e->warmed = false;
    return CTOX_OK;
}

ctox_status ctox_exec_warmup(ctox_exec *e) {
    if (!e) return CTOX_INVALID_STATE;
    ctox_ctx *ctx = e->ctx;
    const ctox_model_config &c = e->cfg;
    CTOX_CUDA(ctx, cudaSetDevice(ctx->device));
    if (!e->embed || !e->lm_head || !e->final_norm)
        return fail(ctx, CTOX_INVALID_STATE, "warmup: embedding, lm_head or final norm missing");
    if (!e->embed->parts[0].canon) return fail(ctx, CTOX_INVALID_STATE, "warmup: embedding rows not resident");
    if (!e->lm_head->s_in || !e->lm_head->s_out || !e->embed->s_in || !e->embed->s_out)
        return fail(ctx, CTOX_INVALID_STATE, "warmup: embedding and lm_head need recovery scales");
    for (uint32_t l = 0; l < e->w.size(); ++l) {
        LayerW &lw = e->w[l];
        bool ok = lw.in_ln && lw.post_ln && lw.in_fan && lw.out && lw.gate_up && lw.down;
        ok = ok && (lw.full ? (lw.q_norm && lw.k_norm) : (lw.conv_w && lw.a_log && lw.dt_bias && lw.lin_norm));
        if (!ok) return fail(ctx, CTOX_INVALID_STATE, "warmup: layer %u has missing tensors", l);
        for (ctox_matvec *mv : {lw.in_fan, lw.out, lw.gate_up, lw.down})
            if (mv->parts.size() != 1 || matvec_positions_per_pass(mv) < kMaxPass)
                return fail(ctx, CTOX_MEMORY_BUDGET, "warmup: layer %u matrix cannot take %u positions per pass", l,
                            kMaxPass);
    }
    if (c.mtp_num_hidden_layers && !(e->mtp_fc && e->mtp_norm_e && e->mtp_norm_h && e->mtp_norm))
        return fail(ctx, CTOX_INVALID_STATE, "warmup: MTP tensors missing");
    ctox_status rc = build_draft_head(e);
    if (rc) return rc;
    if (e->h) {  // buffers exist from an earlier warmup
        e->warmed = true;
        return ctox_exec_reset_session(e);
    }
    const uint64_t H = c.hidden_size, P = kMaxPass;
#define WALLOC(ptr, bytes)                                  \
    do {                                                    \
        rc = xalloc(e, (void **)&(ptr), (bytes), true);     \
        if (rc) return rc;                                  \
    } while (0)
    WALLOC(e->h, P * H * 4);
    WALLOC(e->final_hidden, P * H * 4);
    WALLOC(e->hist_hidden, P * H * 4);
    WALLOC(e->embed_rows, P * H * 4);
    WALLOC(e->mtp_h, P * H * 4);
    WALLOC(e->mtp_hidden, P * H * 4);
    WALLOC(e->aq, P * e->q_width * 4);
    WALLOC(e->agate, P * e->q_width * 4);
    AttnGeom g{c.num_attention_heads, c.num_key_value_heads, c.head_dim, c.rotary_dim, c.rope_theta,
               c.rms_norm_epsilon};
    WALLOC(e->attn_ws, attn_workspace_bytes(g, kMaxPass, e->attn_splits_max));
    WALLOC(e->lz, P * e->value_width * 4);
    WALLOC(e->lcore, P * e->value_width * 4);
    WALLOC(e->norm_scratch, P * ((H + 255) / 256) * 4);
    WALLOC(e->draft_logits, (size_t)(c.draft_vocab ? (e->draft_n ? e->draft_n : 1) : e->vocab_l) * 4);
    if (e->tp_world > 1) {
        WALLOC(e->tp_buf, P * H * 4);
        rc = tp_peer_init(ctx, (size_t)P * H);
        if (rc) return rc;
    }
    WALLOC(e->tokens_dev, (P + 1) * 4);
    WALLOC(e->mtp_tokens_dev, (P + 1) * 4);
    const uint32_t slots = (c.max_context_tokens + c.kv_page_tokens - 1) / c.kv_page_tokens * c.kv_page_tokens;
    const uint32_t pages = slots / c.kv_page_tokens;
    WALLOC(e->page_table, pages * 4);
    WALLOC(e->mtp_page_table, pages * 4);
    k_iota_u32<<<(pages + 255) / 256, 256, 0, ctx->stream>>>(e->page_table, pages, 1);
    k_iota_u32<<<(pages + 255) / 256, 256, 0, ctx->stream>>>(e->mtp_page_table, pages, 1);
    for (uint32_t l = 0; l < e->w.size(); ++l) {
        LayerS &ls = e->s[l];
        if (e->w[l].full) {
            const size_t kvb = (size_t)slots * e->kv_width * kv_elem(e);
            WALLOC(ls.k_cache, kvb);
            WALLOC(ls.v_cache, kvb);
        } else {
            WALLOC(ls.conv_state, (size_t)e->channels * c.linear_conv_kernel_dim * 4);
            WALLOC(ls.delta[0], (size_t)c.linear_num_value_heads * 128 * 128 * 4);
            WALLOC(ls.delta[1], (size_t)c.linear_num_value_heads * 128 * 128 * 4);
            WALLOC(ls.conv_in, P * e->channels * 4);
            WALLOC(ls.q, P * e->key_width * 4);
            WALLOC(ls.k, P * e->key_width * 4);
            WALLOC(ls.v, P * e->value_width * 4);
            WALLOC(ls.g, P * c.linear_num_value_heads * 4);
            WALLOC(ls.beta, P * c.linear_num_value_heads * 4);
        }
    }
    {   // pointer table of the batched commit kernel
        std::vector<CommitLayer> table;
        for (uint32_t l = 0; l < e->n_layers; ++l) {
            if (e->w[l].full) continue;
            LayerS &ls = e->s[l];
            table.push_back(CommitLayer{ls.q, ls.k, ls.v, ls.g, ls.beta, {ls.delta[0], ls.delta[1]}, ls.conv_state,
                                        ls.conv_in});
        }
        e->n_linear = (uint32_t)table.size();
        if (e->n_linear && e->n_linear <= 128) {
            WALLOC(e->commit_table, table.size() * sizeof(CommitLayer));
            CTOX_CUDA(ctx, cudaMemcpyAsync(e->commit_table, table.data(), table.size() * sizeof(CommitLayer),
                                           cudaMemcpyHostToDevice, ctx->stream));
            CTOX_CUDA(ctx, cudaStreamSynchronize(ctx->stream));  // `table` is a local
        }
    }
#undef WALLOC
    CTOX_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    e->warmed = true;
    e->position = 0;
    e->have_hidden = false;
    e->hist_n = 0;
    return CTOX_OK;
}

ctox_status ctox_exec_reset_session(ctox_exec *e) {
    if (!e) return CTOX_INVALID_STATE;
    ctox_ctx *ctx = e->ctx;
    if (!e->h) return fail(ctx, CTOX_INVALID_STATE, "reset: executor is not warm");
    const ctox_model_config &c = e->cfg;
    for (uint32_t l = 0; l < e->w.size(); ++l) {
        LayerS &ls = e->s[l];
        if (e->w[l].full) continue;  // cache slots are rewritten before they are read
        CTOX_CUDA(ctx, cudaMemsetAsync(ls.conv_state, 0, (size_t)e->channels * c.linear_conv_kernel_dim * 4,
                                       ctx->stream));
        CTOX_CUDA(ctx, cudaMemsetAsync(ls.delta[0], 0, (size_t)c.linear_num_value_heads * 128 * 128 * 4,
                                       ctx->stream));
        ls.cur = 0;
    }
    e->position = 0;
    e->have_hidden = false;
    e->hist_n = 0;
    e->step_counter = 0;
    e->pending = -1;
    if (e->poisoned) {  // the error word may still be set by kernels that ran after the failure
        CTOX_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
        CTOX_CUDA(ctx, cudaMemsetAsync(ctx->dev_error, 0, sizeof(int32_t), ctx->stream));
        e->poisoned = false;
    }
    return CTOX_OK;
}

ctox_status ctox_exec_prefill_synthetic(ctox_exec *e, uint64_t n, uint64_t seed) {
    if (!e) return CTOX_INVALID_STATE;
    ctox_ctx *ctx = e->ctx;
    if (!e->warmed) return fail(ctx, CTOX_INVALID_STATE, "prefill: executor is not warm");
    const ctox_model_config &c = e->cfg;
    if (n == 0 || n + 2 * kMaxPass > c.max_context_tokens)
        return fail(ctx, CTOX_SHAPE, "prefill: %llu tokens do not fit the context", (unsigned long long)n);
    ctox_status rc = ctox_exec_reset_session(e);
    if (rc) return rc;
    uint64_t sd = seed;
    for (uint32_t l = 0; l < e->w.size(); ++l) {
        LayerS &ls = e->s[l];
        if (e->w[l].full) {
            const uint64_t cnt = n * e->kv_width;
            for (void *buf : {ls.k_cache, ls.v_cache}) {
                sd = sd * 6364136223846793005ull + 1442695040888963407ull;
                if (c.kv_dtype == CTOX_BF16)
                    k_fill_normal<__nv_bfloat16><<<(unsigned)((cnt + 255) / 256), 256, 0, ctx->stream>>>(
                        (__nv_bfloat16 *)buf, cnt, 0.f, 1.f, sd);
                else
                    k_fill_normal<float><<<(unsigned)((cnt + 255) / 256), 256, 0, ctx->stream>>>((float *)buf, cnt,
                                                                                              0.f, 1.f, sd);
            }
        } else {
            const uint64_t cnt = (uint64_t)c.linear_num_value_heads * 128 * 128;
            sd = sd * 6364136223846793005ull + 1442695040888963407ull;
            k_fill_normal<float><<<(unsigned)((cnt + 255) / 256), 256, 0, ctx->stream>>>(ls.delta[0], cnt, 0.f, 0.02f,
                                                                                      sd);
            ls.cur = 0;
        }
    }
    // a plausible previous hidden state so that the first block can draft
    sd = sd * 6364136223846793005ull + 1442695040888963407ull;
    k_fill_normal<float><<<(unsigned)((c.hidden_size + 255) / 256), 256, 0, ctx->stream>>>(e->hist_hidden,
                                                                                        c.hidden_size, 0.f, 1.f, sd);
    CTOX_CUDA(ctx, cudaGetLastError());
    e->position = n;
    e->have_hidden = true;
    e->hist_n = 1;
    return CTOX_OK;
}

ctox_status ctox_exec_position(const ctox_exec *e, uint64_t *position) {
    if (!e || !position) return CTOX_INVALID_STATE;
    *position = e->position;
    return CTOX_OK;
}

ctox_status ctox_exec_keep_logits(ctox_exec *e, int32_t enable) {
    if (!e) return CTOX_INVALID_STATE;
    e->keep_logits = enable != 0;
    if (e->keep_logits && !e->logits) {
        ctox_status rc = xalloc(e, (void **)&e->logits, (size_t)kMaxPass * e->vocab_l * 4, true);
        if (rc) return rc;
    }
    if (e->keep_logits && e->cfg.mtp_num_hidden_layers && !e->mtp_trace) {
        ctox_status rc = xalloc(e, (void **)&e->mtp_trace, (size_t)2 * kMaxPass * e->cfg.hidden_size * 4, true);
        if (rc) return rc;
        e->draft_rows = e->cfg.draft_vocab ? (e->draft_n ? e->draft_n : 1) : e->vocab_l;
        rc = xalloc(e, (void **)&e->draft_trace, (size_t)kMaxPass * e->draft_rows * 4, true);
        if (rc) return rc;
    }
    return CTOX_OK;
}

}  // extern "C"

// ------------------------------------------------------------------ passes
namespace {

#define EX(expr)               \
    do {                       \
        ctox_status rc_ = (expr); \
        if (rc_) return rc_;   \
    } while (0)

AttnGeom attn_geom(const ctox_exec *e) {
    const ctox_model_config &c = e->cfg;
    return AttnGeom{c.num_attention_heads, c.num_key_value_heads, c.head_dim, c.rotary_dim, c.rope_theta,
                    c.rms_norm_epsilon};
}

// Column-split projection in a tensor-parallel group: finish this rank's partial result, sum it
// over the group and hand the sum on as a plain vector. A single GPU passes the raw sums through.
ctox_status group_sum(ctox_exec *e, ctox_matvec *mv, uint32_t m, MvOut *o) {
    if (e->tp_world <= 1) return CTOX_OK;
    const uint32_t H = e->cfg.hidden_size;
    matvec_finish_enqueue(mv, m, e->tp_buf, H);
    EX(tp_all_reduce_sum_f32(e->ctx, e->tp_buf, (size_t)m * H));
    o->plain = e->tp_buf;
    o->plain_stride = H;
    return CTOX_OK;
}

// h += output of a projection back to the hidden width (summed over the tensor-parallel group when
// there is one: through peer memory, else NCCL), with the partial sums of squares in norm_scratch;
// then, unless `add_only`, the RMS norm (weight norm_w) into xn_out and / or the fragments of `next`.
// (The norm used to run inside the next projection's prologue for passes of one or two positions:
// measured slower than the merged kernel at every position count, and removed.)
ctox_status add_and_norm(ctox_exec *e, float *h, ctox_matvec *mv, uint32_t m, const float *norm_w, float *xn_out,
                         ctox_matvec *next, bool add_only) {
    ctox_ctx *ctx = e->ctx;
    const ctox_model_config &c = e->cfg;
    MvOut o = mv_out(mv, m);
    if (ctx->tp_peer) {
        const MvIn nin = next ? mv_in(next) : MvIn{};
        if (!add_only && tp_peer_reduce_add_norm_fits(c.hidden_size, next ? &nin : nullptr)) {
            // group sum, residual add, norm and fragments as one cluster kernel
            EX(tp_peer_reduce_add_norm(ctx, o, c.hidden_size, m, h, norm_w, c.rms_norm_epsilon, xn_out,
                                       next ? &nin : nullptr));
            return CTOX_OK;
        }
        EX(tp_peer_reduce_add(ctx, o, c.hidden_size, m, h, e->norm_scratch));
    } else {
        EX(group_sum(e, mv, m, &o));
        if (!add_only) {  // residual add, norm and fragments as one cluster kernel
            const MvIn nin = next ? mv_in(next) : MvIn{};
            launch_residual_norm_prep(ctx->stream, h, &o, norm_w, c.rms_norm_epsilon, c.hidden_size, m, xn_out,
                                      next ? &nin : nullptr, e->norm_scratch);
            return CTOX_OK;
        }
        launch_residual_add(ctx->stream, h, &o, c.hidden_size, m, e->norm_scratch);
    }
    if (!add_only) {
        const MvIn nin = next ? mv_in(next) : MvIn{};
        launch_norm_prep(ctx->stream, h, norm_w, c.rms_norm_epsilon, c.hidden_size, m, xn_out, next ? &nin : nullptr,
                         e->norm_scratch);
    }
    return CTOX_OK;
}

// One decoder layer for m positions. The fragments of the layer's input projection are in place on
// entry; next_norm / next name the norm and projection that follow the layer (xn_out also receives
// the normalised vector); with neither, the layer ends with the residual add alone.
ctox_status layer_body(ctox_exec *e, uint32_t l, float *h, uint32_t m, uint64_t rope_pos0, uint64_t slot0,
                       const uint32_t *page_table, const float *next_norm, float *xn_out, ctox_matvec *next) {
    ctox_ctx *ctx = e->ctx;
    cudaStream_t st = ctx->stream;
    const ctox_model_config &c = e->cfg;
    LayerW &lw = e->w[l];
    LayerS &ls = e->s[l];
    EX(matvec_stream_prepared(lw.in_fan, 0, m));
    const MvOut fan = mv_out(lw.in_fan, m);
    const MvIn out_in = mv_in(lw.out);
    if (!lw.full) {
        LinearAttnArgs la{fan, e->key_width, e->value_width, c.linear_num_value_heads, c.linear_num_key_heads,
                          c.linear_conv_kernel_dim, ls.conv_state, lw.conv_w, lw.a_log, lw.dt_bias, lw.lin_norm,
                          c.rms_norm_epsilon, ls.delta[ls.cur], ls.delta[ls.cur ^ 1], ls.conv_in, ls.q, ls.k, ls.v,
                          ls.g, ls.beta, out_in};
        launch_linear_attention(st, la, m);
    } else {
        const AttnGeom g = attn_geom(e);
        launch_attn_pre(st, fan, g, lw.q_norm, lw.k_norm, rope_pos0, slot0, m, e->aq, e->agate, ls.k_cache,
                        ls.v_cache, c.kv_dtype == CTOX_BF16, page_table, c.kv_page_tokens);
        const uint64_t tiles = (slot0 + m + 63) / 64;
        const uint32_t splits = (uint32_t)(tiles < e->attn_splits_max ? (tiles ? tiles : 1) : e->attn_splits_max);
        launch_attention(st, g, e->aq, e->agate, ls.k_cache, ls.v_cache, c.kv_dtype == CTOX_BF16, page_table,
                         c.kv_page_tokens, slot0, m, splits, e->attn_ws, out_in);
    }
    EX(matvec_stream_prepared(lw.out, 0, m));
    EX(add_and_norm(e, h, lw.out, m, lw.post_ln, nullptr, lw.gate_up, false));
    EX(matvec_stream_prepared(lw.gate_up, 0, m));
    launch_swiglu_prep(st, mv_out(lw.gate_up, m), c.intermediate_size, m, mv_in(lw.down));
    EX(matvec_stream_prepared(lw.down, 0, m));
    EX(add_and_norm(e, h, lw.down, m, next_norm, xn_out, next, !(xn_out || next)));
    CTOX_CUDA(ctx, cudaGetLastError());
    return CTOX_OK;
}

// Target model over the m tokens in tokens_dev at positions pos0 ...: final_hidden[m] and the
// lm_head fragments on return. Linear layers leave their new state in the spare buffer.
ctox_status target_pass(ctox_exec *e, uint32_t m, uint64_t pos0) {
    ctox_ctx *ctx = e->ctx;
    const ctox_model_config &c = e->cfg;
    EX(matvec_embed_rows(e->embed, e->tokens_dev, m, e->h));
    const MvIn first = mv_in(e->w[0].in_fan);
    launch_residual_norm_prep(ctx->stream, e->h, nullptr, e->w[0].in_ln, c.rms_norm_epsilon, c.hidden_size, m, nullptr,
                              &first, e->norm_scratch);
    for (uint32_t l = 0; l < e->n_layers; ++l) {
        const bool last = l + 1 == e->n_layers;
        const float *next_norm = last ? e->final_norm : e->w[l + 1].in_ln;
        ctox_matvec *next = last ? e->lm_head : e->w[l + 1].in_fan;
        EX(layer_body(e, l, e->h, m, pos0, pos0, e->page_table, next_norm, last ? e->final_hidden : nullptr, next));
    }
    return CTOX_OK;
}

// Commits the first n of the m positions of the last target pass.
ctox_status commit_positions(ctox_exec *e, uint32_t m, uint32_t n) {
    ctox_ctx *ctx = e->ctx;
    const ctox_model_config &c = e->cfg;
    if (e->commit_table) {  // all linear-attention layers in one launch
        CommitCur cur{};
        uint32_t j = 0;
        for (uint32_t l = 0; l < e->n_layers; ++l)
            if (!e->w[l].full) {
                if (e->s[l].cur) (j < 64 ? cur.lo : cur.hi) |= 1ull << (j & 63);
                ++j;
            }
        // partial acceptance: re-scan the recurrence alone from the committed state
        launch_commit_batch(ctx->stream, e->commit_table, cur, e->n_linear, n, n < m, c.linear_num_value_heads,
                            c.linear_num_key_heads, e->channels, c.linear_conv_kernel_dim);
        for (uint32_t l = 0; l < e->n_layers; ++l)
            if (!e->w[l].full) e->s[l].cur ^= 1;
    } else {
        for (uint32_t l = 0; l < e->n_layers; ++l) {
            if (e->w[l].full) continue;
            LayerS &ls = e->s[l];
            if (n < m)
                EX(ctox_gated_delta_scan(ctx, ls.q, ls.k, ls.v, ls.g, ls.beta, ls.delta[ls.cur], ls.delta[ls.cur ^ 1],
                                         e->lcore, n, c.linear_num_value_heads, c.linear_num_key_heads, 128, 128));
            ls.cur ^= 1;
            launch_conv_commit(ctx->stream, ls.conv_state, ls.conv_in, e->channels, c.linear_conv_kernel_dim, n);
        }
    }
    CTOX_CUDA(ctx, cudaMemcpyAsync(e->hist_hidden, e->final_hidden, (size_t)n * c.hidden_size * 4,
                                   cudaMemcpyDeviceToDevice, ctx->stream));
    e->hist_n = n;
    e->have_hidden = true;
    e->position += n;
    return CTOX_OK;
}

// MTP layer over m (token, previous final hidden) pairs; tokens in device memory, the pair of
// absolute position p uses cache slot p - 1 (decoder.rs:1009-1046). With draft_slot >= 0 the greedy
// draft of the last pair goes to tokens_dev[draft_slot].
ctox_status mtp_pass(ctox_exec *e, uint32_t m, uint64_t abs_pos0, const uint32_t *tokens, const float *hidden_rows,
                     int draft_slot) {
    ctox_ctx *ctx = e->ctx;
    const ctox_model_config &c = e->cfg;
    const uint32_t L = e->n_layers;
    EX(matvec_embed_rows(e->embed, tokens, m, e->embed_rows));
    const MvIn fc_in = mv_in(e->mtp_fc);
    launch_mtp_pre(ctx->stream, e->embed_rows, hidden_rows, e->mtp_norm_e, e->mtp_norm_h, c.rms_norm_epsilon,
                   c.hidden_size, m, &fc_in);
    EX(matvec_stream_prepared(e->mtp_fc, 0, m));
    CTOX_CUDA(ctx, cudaMemsetAsync(e->mtp_h, 0, (size_t)m * c.hidden_size * 4, ctx->stream));
    const MvOut fc = mv_out(e->mtp_fc, m);
    const MvIn lin = mv_in(e->w[L].in_fan);
    launch_residual_norm_prep(ctx->stream, e->mtp_h, &fc, e->w[L].in_ln, c.rms_norm_epsilon, c.hidden_size, m, nullptr,
                              &lin, e->norm_scratch);
    EX(layer_body(e, L, e->mtp_h, m, abs_pos0, abs_pos0 - 1, e->mtp_page_table, e->mtp_norm, e->mtp_hidden,
                  nullptr));
    if (e->keep_logits && e->mtp_trace && e->mtp_trace_n + m <= 2 * kMaxPass) {
        CTOX_CUDA(ctx, cudaMemcpyAsync(e->mtp_trace + (size_t)e->mtp_trace_n * c.hidden_size, e->mtp_hidden,
                                       (size_t)m * c.hidden_size * 4, cudaMemcpyDeviceToDevice, ctx->stream));
        e->mtp_trace_n += m;
    }
    if (draft_slot >= 0) {
        const bool restricted = c.draft_vocab != 0;
        ctox_matvec *head = restricted ? e->draft_head : e->lm_head;  // null: no draft row on this rank
        if (head) {
            EX(matvec_stream_pass(head, 0, e->mtp_hidden + (size_t)(m - 1) * c.hidden_size, CTOX_F32, 1,
                                  c.hidden_size));
            matvec_finish_enqueue(head, 1, e->draft_logits, head->rows);
            if (e->keep_logits && e->draft_trace && e->draft_trace_n < kMaxPass && head->rows <= e->draft_rows) {
                CTOX_CUDA(ctx, cudaMemcpyAsync(e->draft_trace + (size_t)e->draft_trace_n * e->draft_rows,
                                               e->draft_logits, (size_t)head->rows * 4, cudaMemcpyDeviceToDevice,
                                               ctx->stream));
                e->draft_trace_n += 1;
            }
        }
        EX(argmax_enqueue(ctx, e->draft_logits, head ? (uint32_t)head->rows : 0,
                          restricted ? e->draft_ids + e->draft_lo : nullptr, e->vocab_off,
                          e->tokens_dev + draft_slot, nullptr));
    }
    return CTOX_OK;
}

ctox_status upload_u32(ctox_exec *e, uint32_t *dst, const uint32_t *src, uint32_t n) {
    ctox_ctx *ctx = e->ctx;
    // pageable source: the copy is staged by the runtime before the call returns
    CTOX_CUDA(ctx, cudaMemcpyAsync(dst, src, n * 4, cudaMemcpyHostToDevice, ctx->stream));
    return CTOX_OK;
}

bool cancelled(const volatile int32_t *cancel) { return cancel && *cancel != 0; }

ctox_status session_usable(ctox_exec *e, const char *what) {
    if (e->poisoned)
        return fail(e->ctx, CTOX_INVALID_STATE,
                    "%s: the session was invalidated by an earlier device error; reset_session first", what);
    return CTOX_OK;
}

ctox_status prefill_impl(ctox_exec *e, const uint32_t *tokens, uint64_t n, const volatile int32_t *cancel,
                         bool *began) {
    ctox_ctx *ctx = e->ctx;
    EX(ctox_exec_reset_session(e));
    const uint64_t consume = n - 1;  // the last token is the input of the first decode
    for (uint64_t a = 0; a < consume; a += kMaxPass) {
        if (cancelled(cancel)) return fail(ctx, CTOX_CANCELLED, "prefill cancelled at token %llu", (unsigned long long)a);
        const uint32_t m = (uint32_t)(consume - a < kMaxPass ? consume - a : kMaxPass);
        *began = true;
        EX(upload_u32(e, e->tokens_dev, tokens + a, m));
        EX(target_pass(e, m, a));
        EX(commit_positions(e, m, m));
        for (uint32_t j = 0; j + 1 < m; ++j) e->hist_tokens[j] = tokens[a + 1 + j];
        const bool last_chunk = a + m >= consume;
        if (e->cfg.mtp_num_hidden_layers && !last_chunk) {
            // keep the MTP cache exact: pairs (token p+1, final hidden p) of this chunk
            EX(upload_u32(e, e->mtp_tokens_dev, tokens + a + 1, m));
            EX(mtp_pass(e, m, a + 1, e->mtp_tokens_dev, e->hist_hidden, -1));
        }
        // `tokens` may be pageable host memory: finish the chunk, and read the device error word
        int32_t dev_err = 0;
        EX(ctox_ctx_device_error(ctx, &dev_err));
        if (dev_err)
            return fail(ctx, CTOX_INVALID_STATE,
                        dev_err == DEV_ERR_WAIT_TIMEOUT ? "prefill: a bounded device wait ran out (device error %d)"
                                                        : "prefill: device error %d",
                        dev_err);
    }
    return CTOX_OK;
}

ctox_status decode_impl(ctox_exec *e, uint32_t token, int32_t mtp_enabled, float temperature, uint64_t seed,
                        int32_t force_accept, const volatile int32_t *cancel, ctox_exec_step *step, bool *began) {
    ctox_ctx *ctx = e->ctx;
    const ctox_model_config &c = e->cfg;
    memset(step, 0, sizeof *step);
    const uint32_t k = (mtp_enabled && e->have_hidden && e->position > 0) ? c.max_draft_tokens : 0;
    const uint64_t P = e->position;
    uint32_t host_tokens[kMaxPass + 1] = {0};
    host_tokens[0] = token;
    e->mtp_trace_n = e->draft_trace_n = 0;
    const auto t_begin = std::chrono::steady_clock::now();
    // Nothing below changes the committed session before the acceptance is known: a cancellation
    // between passes leaves the session where it was (the MTP cache slots written so far belong to
    // committed positions or lie beyond them and are rewritten by the next call).
    *began = true;
    EX(upload_u32(e, e->tokens_dev, host_tokens, 1));
    if (e->phase_timing) {
        if (e->commit_timed) {  // the commit of the block before: its events have long completed
            cudaEventSynchronize(e->phase_ev[5]);
            cudaEventElapsedTime(&e->phase_ms[3], e->phase_ev[4], e->phase_ev[5]);
            e->commit_timed = false;
        }
        cudaEventRecord(e->phase_ev[0], ctx->stream);
    }
    if (k > 0) {
        // catch-up over the pairs of the last block (true target hiddens), then the chained drafts
        const uint32_t n = e->hist_n;
        uint32_t mt[kMaxPass];
        for (uint32_t j = 0; j + 1 < n; ++j) mt[j] = e->hist_tokens[j];
        mt[n - 1] = token;
        EX(upload_u32(e, e->mtp_tokens_dev, mt, n));
        EX(mtp_pass(e, n, P - n + 1, e->mtp_tokens_dev, e->hist_hidden, 1));
        for (uint32_t i = 1; i < k; ++i) {
            if (cancelled(cancel)) return fail(ctx, CTOX_CANCELLED, "decode cancelled while drafting");
            // the draft just written to tokens_dev[i] and the MTP's own hidden of the last pair, in
            // place: the pass reads both in its first kernels and rewrites mtp_hidden in its last
            const uint32_t prev_rows = i == 1 ? n : 1;
            EX(mtp_pass(e, 1, P + i, e->tokens_dev + i, e->mtp_hidden + (size_t)(prev_rows - 1) * c.hidden_size,
                        (int)(1 + i)));
        }
    }
    if (cancelled(cancel)) return fail(ctx, CTOX_CANCELLED, "decode cancelled before the target pass");
    const uint32_t m = k + 1;
    if (e->phase_timing) cudaEventRecord(e->phase_ev[1], ctx->stream);
    EX(target_pass(e, m, P));
    if (e->phase_timing) cudaEventRecord(e->phase_ev[2], ctx->stream);
    EX(matvec_stream_prepared(e->lm_head, 0, m));
    int32_t parent[kMaxPass];
    for (uint32_t i = 0; i < m; ++i) parent[i] = (int32_t)i - 1;
    const float inv_t = temperature > 0.f ? 1.0f / temperature : 0.f;
    const uint64_t step_id = e->step_counter++;
    EX(head_verify_enqueue(e->lm_head, 0, m, m, parent, e->tokens_dev, inv_t, seed, step_id, e->vocab_l,
                           e->keep_logits ? e->logits : nullptr, e->vocab_off));
    EX(head_tp_merge_enqueue(ctx, m, parent, e->tokens_dev, e->vocab_l));
    ctox_spec_record *rec_dev = nullptr;
    EX(head_accept_enqueue(ctx, m, parent, e->tokens_dev, inv_t, seed, step_id,
                           force_accept < 0 ? -1 : (force_accept > (int32_t)k ? (int32_t)k : force_accept),
                           &rec_dev));
    if (e->phase_timing) cudaEventRecord(e->phase_ev[3], ctx->stream);
    EX(ensure_pinned(ctx, sizeof(ctox_spec_record) + 16));
    CTOX_CUDA(ctx, cudaMemcpyAsync(ctx->pinned, rec_dev, sizeof(ctox_spec_record), cudaMemcpyDeviceToHost,
                                   ctx->stream));
    CTOX_CUDA(ctx, cudaMemcpyAsync((uint8_t *)ctx->pinned + sizeof(ctox_spec_record), ctx->dev_error, 4,
                                   cudaMemcpyDeviceToHost, ctx->stream));
    e->last_enqueue_us = std::chrono::duration<double, std::micro>(std::chrono::steady_clock::now() - t_begin).count();
    CTOX_CUDA(ctx, cudaStreamSynchronize(ctx->stream));  // the one host read of the block
    if (e->phase_timing)
        for (int i = 0; i < 3; ++i) cudaEventElapsedTime(&e->phase_ms[i], e->phase_ev[i], e->phase_ev[i + 1]);
    ctox_spec_record rec;
    memcpy(&rec, ctx->pinned, sizeof rec);
    int32_t dev_err;
    memcpy(&dev_err, (uint8_t *)ctx->pinned + sizeof(ctox_spec_record), 4);
    if (dev_err) {
        cudaMemsetAsync(ctx->dev_error, 0, 4, ctx->stream);
        e->poisoned = true;  // kernels carried on past the failure: the residual stream and caches are undefined
        return fail(ctx, CTOX_INVALID_STATE,
                    dev_err == DEV_ERR_WAIT_TIMEOUT ? "decode: a bounded device wait ran out (device error %d)"
                                                    : "decode: device error %d",
                    dev_err);
    }
    if (rec.status) return fail(ctx, CTOX_INVALID_STATE, "decode: the target produced a non-finite logit");
    if (rec.n_emitted == 0 || rec.n_emitted > m)
        return fail(ctx, CTOX_INVALID_STATE, "decode: malformed acceptance record");
    const uint32_t n_acc = rec.n_emitted - 1;
    if (e->phase_timing) cudaEventRecord(e->phase_ev[4], ctx->stream);
    EX(commit_positions(e, m, n_acc + 1));
    if (e->phase_timing) {
        cudaEventRecord(e->phase_ev[5], ctx->stream);
        e->commit_timed = true;
    }
    for (uint32_t j = 0; j < n_acc; ++j) e->hist_tokens[j] = rec.emitted[j];
    step->proposed_drafts = k;
    step->n_accepted = n_acc;
    step->verified_drafts = k == 0 ? 0 : (n_acc == k ? k : n_acc + 1);  // engine.rs:118-136
    for (uint32_t j = 0; j < n_acc; ++j) step->accepted_draft_tokens[j] = rec.emitted[j];
    step->next_token = rec.emitted[n_acc];
    for (uint32_t j = 0; j < k; ++j) step->draft_tokens[j] = rec.node_token[1 + j];
    for (uint32_t j = 0; j < m; ++j) step->target_tokens[j] = rec.node_argmax[j];
    if (k > 0) e->pending = (int32_t)n_acc;
    return CTOX_OK;
}

}  // namespace

extern "C" {

ctox_status ctox_exec_prefill(ctox_exec *e, const uint32_t *tokens, uint64_t n, const volatile int32_t *cancel) {
    if (!e || !tokens) return CTOX_INVALID_STATE;
    ctox_ctx *ctx = e->ctx;
    if (cancelled(cancel)) return fail(ctx, CTOX_CANCELLED, "prefill cancelled");
    if (!e->warmed) return fail(ctx, CTOX_INVALID_STATE, "prefill: executor is not warm");
    if (n == 0 || n + 2 * kMaxPass > e->cfg.max_context_tokens)
        return fail(ctx, CTOX_SHAPE, "prefill: %llu tokens do not fit the context", (unsigned long long)n);
    for (uint64_t i = 0; i < n; ++i)
        if (tokens[i] >= e->cfg.vocab_size) return fail(ctx, CTOX_SHAPE, "prefill: token %u out of range", tokens[i]);
    CTOX_CUDA(ctx, cudaSetDevice(ctx->device));
    bool began = false;
    const ctox_status rc = prefill_impl(e, tokens, n, cancel, &began);
    // a prefill that stopped half way (cancelled or failed) leaves no usable session
    if (rc && began) e->poisoned = true;
    return rc;
}

ctox_status ctox_exec_decode(ctox_exec *e, uint32_t token, int32_t mtp_enabled, float temperature, uint64_t seed,
                             int32_t force_accept, const volatile int32_t *cancel, ctox_exec_step *step) {
    if (!e || !step) return CTOX_INVALID_STATE;
    ctox_ctx *ctx = e->ctx;
    const ctox_model_config &c = e->cfg;
    if (cancelled(cancel)) return fail(ctx, CTOX_CANCELLED, "decode cancelled");  // decoder.rs:1284-1292
    if (!e->warmed) return fail(ctx, CTOX_INVALID_STATE, "decode: executor is not warm");
    EX(session_usable(e, "decode"));
    if (e->pending >= 0)  // decoder.rs:1293-1297
        return fail(ctx, CTOX_INVALID_STATE, "decode requires the previous speculative branch to be committed");
    if (token >= c.vocab_size) return fail(ctx, CTOX_SHAPE, "decode: token %u out of range", token);
    if (!std::isfinite(temperature) || temperature < 0.f)
        return fail(ctx, CTOX_INVALID_ARTIFACT, "temperature must be finite and non-negative");
    if (e->position + 2 * kMaxPass >= c.max_context_tokens)
        return fail(ctx, CTOX_SHAPE, "decode: context capacity exhausted at position %llu",
                    (unsigned long long)e->position);
    if (mtp_enabled && !c.mtp_num_hidden_layers)
        return fail(ctx, CTOX_INVALID_STATE, "decode enabled MTP but the model has no MTP layer");
    CTOX_CUDA(ctx, cudaSetDevice(ctx->device));
    bool began = false;
    const ctox_status rc = decode_impl(e, token, mtp_enabled, temperature, seed, force_accept, cancel, step, &began);
    if (rc && rc != CTOX_CANCELLED && began) e->poisoned = true;
    return rc;
}

ctox_status ctox_exec_commit_speculative(ctox_exec *e, uint32_t accepted_drafts, const volatile int32_t *cancel) {
    if (!e) return CTOX_INVALID_STATE;
    ctox_ctx *ctx = e->ctx;
    EX(session_usable(e, "commit_speculative"));
    if (e->pending < 0)  // decoder.rs:1401-1403
        return fail(ctx, CTOX_INVALID_STATE, "executor has no pending speculative branch");
    if (cancelled(cancel)) return fail(ctx, CTOX_CANCELLED, "commit_speculative cancelled");
    // The device resolved the acceptance and committed exactly that prefix (the resolved form,
    // engine.rs:110-136); any other depth would name a state this executor does not hold.
    if ((int32_t)accepted_drafts != e->pending)
        return fail(ctx, CTOX_INVALID_STATE, "accepted MTP depth %u differs from the device-resolved prefix %d",
                    accepted_drafts, e->pending);
    e->pending = -1;
    return CTOX_OK;
}

ctox_status ctox_exec_session_state(const ctox_exec *e, int32_t *pending_accepted, int32_t *poisoned) {
    if (!e) return CTOX_INVALID_STATE;
    if (pending_accepted) *pending_accepted = e->pending;
    if (poisoned) *poisoned = e->poisoned ? 1 : 0;
    return CTOX_OK;
}

ctox_status ctox_exec_phase_timing(ctox_exec *e, int32_t enable) {
    if (!e) return CTOX_INVALID_STATE;
    ctox_ctx *ctx = e->ctx;
    CTOX_CUDA(ctx, cudaSetDevice(ctx->device));
    if (enable)
        for (auto &ev : e->phase_ev)
            if (!ev) CTOX_CUDA(ctx, cudaEventCreate(&ev));
    e->phase_timing = enable != 0;
    e->commit_timed = false;
    return CTOX_OK;
}

ctox_status ctox_exec_last_phase_ms(ctox_exec *e, float *ms4) {
    if (!e || !ms4) return CTOX_INVALID_STATE;
    if (e->commit_timed) {
        cudaEventSynchronize(e->phase_ev[5]);
        cudaEventElapsedTime(&e->phase_ms[3], e->phase_ev[4], e->phase_ev[5]);
        e->commit_timed = false;
    }
    for (int i = 0; i < 4; ++i) ms4[i] = e->phase_ms[i];
    return CTOX_OK;
}

ctox_status ctox_exec_last_enqueue_us(const ctox_exec *e, double *microseconds) {
    if (!e || !microseconds) return CTOX_INVALID_STATE;
    *microseconds = e->last_enqueue_us;
    return CTOX_OK;
}

ctox_status ctox_exec_last_mtp_hidden(ctox_exec *e, uint32_t index, float *out, uint32_t *count) {
    if (!e) return CTOX_INVALID_STATE;
    ctox_ctx *ctx = e->ctx;
    if (count) *count = e->mtp_trace_n;
    if (!out) return CTOX_OK;
    if (!e->keep_logits || !e->mtp_trace || index >= e->mtp_trace_n)
        return fail(ctx, CTOX_INVALID_STATE, "MTP hidden states are not kept (ctox_exec_keep_logits) or index out of range");
    CTOX_CUDA(ctx, cudaMemcpyAsync(out, e->mtp_trace + (size_t)index * e->cfg.hidden_size,
                                   (size_t)e->cfg.hidden_size * 4, cudaMemcpyDeviceToHost, ctx->stream));
    CTOX_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    return CTOX_OK;
}

ctox_status ctox_exec_last_draft_logits(ctox_exec *e, uint32_t draft, float *out, uint32_t *rows, uint32_t *count) {
    if (!e) return CTOX_INVALID_STATE;
    ctox_ctx *ctx = e->ctx;
    if (rows) *rows = e->draft_rows;
    if (count) *count = e->draft_trace_n;
    if (!out) return CTOX_OK;
    if (!e->keep_logits || !e->draft_trace || draft >= e->draft_trace_n)
        return fail(ctx, CTOX_INVALID_STATE, "draft logits are not kept (ctox_exec_keep_logits) or index out of range");
    CTOX_CUDA(ctx, cudaMemcpyAsync(out, e->draft_trace + (size_t)draft * e->draft_rows, (size_t)e->draft_rows * 4,
                                   cudaMemcpyDeviceToHost, ctx->stream));
    CTOX_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    return CTOX_OK;
}

ctox_status ctox_exec_last_hidden(ctox_exec *e, float *out) {
    if (!e || !out) return CTOX_INVALID_STATE;
    ctox_ctx *ctx = e->ctx;
    if (!e->have_hidden || e->hist_n == 0) return fail(ctx, CTOX_INVALID_STATE, "no committed hidden state");
    CTOX_CUDA(ctx, cudaMemcpyAsync(out, e->hist_hidden + (size_t)(e->hist_n - 1) * e->cfg.hidden_size,
                                   (size_t)e->cfg.hidden_size * 4, cudaMemcpyDeviceToHost, ctx->stream));
    CTOX_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    return CTOX_OK;
}

ctox_status ctox_exec_last_logits(ctox_exec *e, uint32_t position, float *out) {
    if (!e || !out) return CTOX_INVALID_STATE;
    ctox_ctx *ctx = e->ctx;
    if (!e->keep_logits || !e->logits || position >= kMaxPass)
        return fail(ctx, CTOX_INVALID_STATE, "logits are not kept (ctox_exec_keep_logits) or position out of range");
    CTOX_CUDA(ctx, cudaMemcpyAsync(out, e->logits + (size_t)position * e->vocab_l, (size_t)e->vocab_l * 4,
                                   cudaMemcpyDeviceToHost, ctx->stream));
    CTOX_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    return CTOX_OK;
}

ctox_status ctox_exec_select_target(ctox_exec *e, uint32_t position, float temperature, uint32_t top_k,
                                    float top_p, float draw, uint32_t *token) {
    if (!e || !token) return CTOX_INVALID_STATE;
    ctox_ctx *ctx = e->ctx;
    if (!e->keep_logits || !e->logits || position >= kMaxPass)
        return fail(ctx, CTOX_INVALID_STATE, "logits are not kept (ctox_exec_keep_logits) or position out of range");
    if (e->tp_world > 1)
        return fail(ctx, CTOX_UNSUPPORTED_OPERATION, "select_target: the kept logits are a vocabulary shard");
    return ctox_sample_topk_topp(ctx, e->logits + (size_t)position * e->vocab_l, e->vocab_l, temperature, top_k, top_p,
                                 draw, token);
}

}  // extern "C"
