/*
 * libctox_b200 — C ABI of the B200 (sm_100a) decode hot path for CTOX-LLM's
 * Qwen3.8-27B integration.
 *
 * Every entry point is what a foreign-function binding of the reference crate
 * (models/qwen38_27b/src/) would bind for this path; the reference interface
 * each one replaces is cited as file:line relative to that directory.
 *
 * Conventions
 *  - All functions return a ctox_status; 0 is success. Codes map 1:1 to the
 *    variants of EngineError (error.rs:5-29). ctox_last_error_message() gives
 *    the text of the last failure on a context.
 *  - Host pointers are borrowed for the duration of the call. `*_prepare`
 *    copies what it needs into library-owned device memory.
 *  - Device pointers passed in are borrowed and must belong to the context's
 *    device. Work is enqueued on the context's stream; functions documented as
 *    "host form" synchronise before returning.
 *  - A context and everything created from it are thread-affine, like the
 *    reference's CudaCandidateRuntime (backend/cuda_runtime.rs:298-300): call
 *    from one thread at a time. There is no CPU fallback: without a usable
 *    CUDA device every call fails with CTOX_UNSUPPORTED_OPERATION.
 */
#ifndef CTOX_B200_H
#define CTOX_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef int32_t ctox_status;

/* error.rs:5-29 */
enum {
    CTOX_OK = 0,
    CTOX_SHAPE = 1,
    CTOX_INVALID_ARTIFACT = 2,
    CTOX_UNSUPPORTED_DTYPE = 3,
    CTOX_UNSUPPORTED_OPERATION = 4,
    CTOX_MEMORY_BUDGET = 5,
    CTOX_INVALID_STATE = 6,
    CTOX_CANCELLED = 7
};

/* format.rs:26-32 (TensorDType) plus the activation element types the device
 * entry points accept. */
enum {
    CTOX_Q2B64 = 0,
    CTOX_Q4B64 = 1,
    CTOX_MIXED_Q2Q4B64 = 2,
    CTOX_F16 = 3,
    CTOX_F32 = 4,
    CTOX_BF16 = 5
};

/* backend/mod.rs:54-57 (Activation); the kernel ABI uses the same codes
 * (backend/cuda_runtime.rs:8370-8373). */
enum { CTOX_ACT_IDENTITY = 0, CTOX_ACT_SILU = 1 };

/* backend/mod.rs:74-77 (ScaleSlice) */
enum { CTOX_SCALE_NONE = 0, CTOX_SCALE_F32 = 1, CTOX_SCALE_F16LE = 2 };

/* Kernel choice for ctox_matvec_dispatch. AUTO is the production path. */
enum {
    CTOX_KERNEL_AUTO = 0,
    CTOX_KERNEL_STREAM = 1, /* bulk-copy staged, tensor-core dot products, repacked weights */
    CTOX_KERNEL_ROWWARP = 2 /* one warp per row over canonical bytes, fp32 FMA */
};

/* ctox_matvec_prepare flags */
enum {
    CTOX_PREPARE_KEEP_CANONICAL = 1u /* keep the canonical bytes resident (row gathers, ROWWARP) */
};

typedef struct ctox_ctx ctox_ctx;
typedef struct ctox_matvec ctox_matvec;

/* format.rs:56-64 (QuantSegment) */
typedef struct {
    uint32_t group_index;
    uint32_t dtype;
    uint64_t row_start;
    uint64_t row_end;
    uint64_t offset;
    uint64_t length;
} ctox_segment;

/* backend/mod.rs:115-128 (FusedMatVec<'a>) with host slices as pointer+length. */
typedef struct {
    uint32_t dtype;
    uint32_t activation;
    const uint8_t *weights;
    uint64_t weights_len;
    const ctox_segment *segments;
    uint64_t n_segments;
    uint64_t rows;
    uint64_t columns;
    const float *input;
    uint64_t input_len;
    uint32_t s_in_kind;
    uint32_t s_out_kind;
    const void *s_in;
    uint64_t s_in_len; /* values, not bytes */
    const void *s_out;
    uint64_t s_out_len;
    const float *bias;
    uint64_t bias_len;
} ctox_fused_matvec_op;

/* ---- context (backend/cuda_runtime.rs:352-417: private context + one stream) ---- */

/* `stream` is a cudaStream_t to borrow, or NULL to let the context own one. */
ctox_status ctox_ctx_create(int32_t device, void *stream, ctox_ctx **out);
ctox_status ctox_ctx_destroy(ctox_ctx *ctx);
ctox_status ctox_ctx_synchronize(ctox_ctx *ctx);

/* ---- tensor-parallel group (no counterpart in the reference, which runs on one GPU) ----
 * One process per GPU of an NVSwitch box. Rank 0 draws an id, the caller carries its 128 bytes
 * to the other ranks (any rendezvous, e.g. torch.distributed), then every rank joins. NCCL is
 * loaded at run time from nccl_path (NULL or "" = "libnccl.so.2" on the loader's search path).
 * An executor created on a context that has joined a group holds this rank's shard of the model
 * (include/ctox_b200.h: ctox_exec_create). Collectives are enqueued on the context's stream;
 * every rank must make the same executor calls in the same order. */
ctox_status ctox_tp_unique_id(ctox_ctx *ctx, const char *nccl_path, uint8_t *id128);
ctox_status ctox_tp_init(ctox_ctx *ctx, const char *nccl_path, int32_t rank, int32_t world,
                         const uint8_t *id128);
ctox_status ctox_tp_destroy(ctox_ctx *ctx);
/* Sum of an fp32 device buffer over the group, in place (the collective the executor uses). */
ctox_status ctox_tp_all_reduce_f32(ctox_ctx *ctx, float *buf_dev, uint64_t n);
/* Which collective sums the column-split projections: "none" (one GPU), "p2p_push" (one-shot
 * all-reduce through peer memory, set up at warmup) or "nccl" (the fall-back). Static string. */
ctox_status ctox_tp_collective(const ctox_ctx *ctx, const char **name);
/* Failure-detection test support (no counterpart in the reference): makes the context rank 0 of a
 * group of `world` ranks whose other ranks never answer, without NCCL or a second GPU, and sets the
 * limit of the bounded device waits on a peer (SM clock cycles; 0 keeps the default of ~1 s). An
 * executor created afterwards holds rank 0's shard; its first group sum runs out of time, the
 * kernels set the device error word and return, and the call reports CTOX_INVALID_STATE. Nothing
 * hangs: every later wait of the same call is skipped once the word is set. */
ctox_status ctox_tp_debug_silent_peers(ctox_ctx *ctx, int32_t world, uint64_t wait_limit_cycles);
/* Never NULL; empty when no call has failed. ctx may be NULL (creation errors). */
const char *ctox_last_error_message(const ctox_ctx *ctx);
/* Bytes of device memory currently owned through this context
 * (engine.rs:46-74 AllocationSnapshot; must be 0 after everything is destroyed,
 * engine.rs:818-824). */
ctox_status ctox_ctx_allocated_bytes(const ctox_ctx *ctx, uint64_t *bytes);
/* Returns (and clears) the device-side error word: 0 = none. Kernels set it
 * instead of trapping, e.g. when a bounded wait ran out. */
ctox_status ctox_ctx_device_error(ctox_ctx *ctx, int32_t *code);
/* Kernels this library has enqueued in this process so far (all contexts): the count behind the
 * benchmark's `gpu_launches` (difference over the timed region). No counterpart in the reference. */
uint64_t ctox_kernel_launches(void);
/* Benchmark support (the reference's verify/bench binaries time dispatches the
 * same way, src/bin/cuda_bench.rs): when enabled, every launch of the dominant
 * kernel (the streaming / row-warp matvec) is bracketed by a CUDA event pair on
 * the context's stream. _read synchronises, returns the
 * summed duration and the number of launches since the last read, and clears. */
ctox_status ctox_ctx_kernel_timing(ctox_ctx *ctx, int32_t enable);
ctox_status ctox_ctx_kernel_timing_read(ctox_ctx *ctx, double *total_ms, uint64_t *launches);
/* backend/mod.rs:153-156: kind()/promotion_state()/profile() */
const char *ctox_backend_profile(void);
uint32_t ctox_abi_version(void);

/* ---- Backend trait, host form (backend/mod.rs:153-169; CPU implementation
 * backend/cpu.rs:432-497). Inputs and outputs are host memory; the call
 * uploads, runs on the GPU, downloads and synchronises. Validation and error
 * kinds follow backend/cpu.rs:41-173. ---- */
ctox_status ctox_fused_matvec(ctox_ctx *ctx, const ctox_fused_matvec_op *op, float *out);
ctox_status ctox_fused_matvec_fanout(ctox_ctx *ctx, const ctox_fused_matvec_op *ops, uint64_t n,
                                     float *const *outs);
/* RecoveredRow (backend/mod.rs:131-141, backend/cpu.rs:312-370) */
ctox_status ctox_recovered_row(ctox_ctx *ctx, uint32_t dtype, const uint8_t *weights,
                               uint64_t weights_len, uint64_t columns, uint32_t s_in_kind,
                               const void *s_in, uint64_t s_in_len, float s_out, float *out);
/* RecoveredRowMatVec (backend/mod.rs:143-151, backend/cpu.rs:478-497) */
ctox_status ctox_recovered_row_matvec(ctox_ctx *ctx, uint32_t dtype, const uint8_t *weights,
                                      uint64_t weights_len, const float *corrected_input,
                                      uint64_t columns, float s_out, float *out);

/* ---- resident form (backend/cuda_runtime.rs:8341-8382 prepare_fused_matvec,
 * :10560 dispatch_prepared*, :423-468 device views) ---- */

/* Validates like ctox_fused_matvec (op->input may be NULL), uploads weights and
 * scales once and repacks them for the streaming kernel. */
ctox_status ctox_matvec_prepare(ctox_ctx *ctx, const ctox_fused_matvec_op *op, uint32_t flags,
                                ctox_matvec **out);
ctox_status ctox_matvec_destroy(ctox_matvec *mv);
/* Y[m][r] = act((sum_c W[r][c] * X[m][c] * s_in[c] + bias[r]) * s_out[r]) for
 * m < positions. x_dev: positions rows of `columns` elements (CTOX_F32 or
 * CTOX_BF16), row stride x_stride elements; y_dev: float, row stride y_stride.
 * positions = 1 is the decode matvec (kernel ABI backend/cuda.rs:73-122); 2..16
 * is the verify-batched projection (backend/cuda_runtime.rs:9764-9816). */
ctox_status ctox_matvec_dispatch(ctox_matvec *mv, const void *x_dev, uint32_t x_dtype,
                                 uint32_t positions, uint64_t x_stride, float *y_dev,
                                 uint64_t y_stride, uint32_t kernel);
/* Same, with host x and y (pinned staging inside the library); synchronises. */
ctox_status ctox_matvec_dispatch_host(ctox_matvec *mv, const float *x_host, uint32_t positions,
                                      float *y_host, uint32_t kernel);
/* No counterpart in the reference. Same result as ctox_matvec_dispatch (kernel
 * AUTO) for callers that may not allocate device memory around a dispatch - a
 * serving loop that has given every free byte to its cache, a plug-in inside a
 * foreign memory pool, code where an allocation's implicit synchronisation is
 * not acceptable. The kernel's scratch (activation fragments, block metadata,
 * partial sums) is an 8 MiB array built into the library image; every GPU that
 * loads the library keeps it until exit. Operations that need more scratch than
 * that (for example a 248320-row head) fail with CTOX_MEMORY_BUDGET. The call
 * makes no cudaMalloc/cudaFree and calls no allocating routine. The first call
 * on a device looks the array's address up (cudaGetSymbolAddress) and should
 * therefore come before any stream capture. All calls on a device share the one
 * array and nothing in it has to start at zero, but two calls whose kernels
 * overlap on the GPU (different streams or contexts) race on it: keep them on
 * one stream or order them yourself. */
ctox_status ctox_matvec_dispatch_static(ctox_matvec *mv, const void *x_dev, uint32_t x_dtype,
                                        uint32_t positions, uint64_t x_stride, float *y_dev,
                                        uint64_t y_stride);
/* Backend::fused_matvec_fanout on prepared, device-resident matrices (backend/cpu.rs:444-472;
 * policy fanout.rs:31-70: members read the same input and carry identical s_in). The activation
 * fragments are built once and every member streams against them. Members must be pure (one code
 * format, the same for all) and have the same column count; otherwise CTOX_SHAPE /
 * CTOX_UNSUPPORTED_OPERATION. y_devs[i] receives [positions][y_strides[i]] like
 * ctox_matvec_dispatch. */
ctox_status ctox_matvec_fanout_dispatch(ctox_matvec *const *mvs, uint64_t n, const void *x_dev,
                                        uint32_t x_dtype, uint32_t positions, uint64_t x_stride,
                                        float *const *y_devs, const uint64_t *y_strides);
/* Device form of recovered rows (backend/cpu.rs:312-370; CUDA candidate
 * ctox_q{2,4}_b64_recovered_rows_sm86): out_dev[i][c] = W[row_ids[i]][c] * s_in[c] *
 * s_out[row_ids[i]] for n row ids in device memory. Needs CTOX_PREPARE_KEEP_CANONICAL and both
 * recovery scales; a row id out of range sets the device error word. */
ctox_status ctox_matvec_recovered_rows(ctox_matvec *mv, const uint32_t *row_ids_dev, uint32_t n,
                                       float *out_dev);
/* Geometry of the prepared operation. */
ctox_status ctox_matvec_info(const ctox_matvec *mv, uint64_t *rows, uint64_t *columns,
                             uint64_t *packed_bytes, uint64_t *device_bytes);

/* ---- gated-delta recurrence (reference.rs:230-297,377-415; CUDA candidate
 * backend/cuda_runtime.rs:3514-3900 prepare_gated_delta_f16 /
 * dispatch_gated_delta_f16[_scan]_device, kernel ABI backend/cuda.rs:266-387).
 * All pointers are device memory, fp32. q, k: [tokens][qk_heads][key_dim]; when
 * qk_heads < heads, head h reads source head h / (heads / qk_heads), which is
 * repeat_heads (decoder.rs:47-65). v, out: [tokens][heads][value_dim];
 * log_decay, beta: [tokens][heads]; state: [heads][key_dim][value_dim].
 * state_out may equal state_in (in place) or be a second buffer, which leaves
 * state_in untouched for a speculative pass. Enqueued on the context's stream. */
ctox_status ctox_gated_delta_scan(ctox_ctx *ctx, const float *q, const float *k, const float *v,
                                  const float *log_decay, const float *beta, const float *state_in,
                                  float *state_out, float *out, uint32_t tokens, uint32_t heads,
                                  uint32_t qk_heads, uint32_t key_dim, uint32_t value_dim);
/* The scan of `layers` independent layers in ONE launch: every array holds the layers back to back
 * in the single-layer layout above (q, k: [layers][tokens][qk_heads][128], state: [layers][heads][128][128],
 * ...); out may be NULL (state only). 128 x 128 heads. This is the form in which the executor
 * re-scans an accepted prefix over all linear-attention layers (the reference replays whole passes
 * instead, backend/cuda_graph.rs:4962-5003); results equal `layers` calls of ctox_gated_delta_scan. */
ctox_status ctox_gated_delta_scan_layers(ctox_ctx *ctx, const float *q, const float *k, const float *v,
                                         const float *log_decay, const float *beta, const float *state_in,
                                         float *state_out, float *out, uint32_t layers, uint32_t tokens,
                                         uint32_t heads, uint32_t qk_heads);
/* The same scan with the FP16-resident state of the reference's CUDA candidate
 * (recurrent_gated_delta_step_f16_state, reference.rs:299-373; backend/cuda_runtime.rs:3514-3900
 * dispatch_gated_delta_f16[_scan]_device): state_in / state_out are [heads][128][128] binary16;
 * dot products and update arithmetic stay fp32, every state element is rounded to binary16 when
 * it is written (after the decay and after the update of every token). 128 x 128 heads only. */
ctox_status ctox_gated_delta_scan_f16_state(ctox_ctx *ctx, const float *q, const float *k, const float *v,
                                            const float *log_decay, const float *beta,
                                            const void *state_in, void *state_out, float *out,
                                            uint32_t tokens, uint32_t heads, uint32_t qk_heads,
                                            uint32_t key_dim, uint32_t value_dim);
/* ---- K/V rows as packed blocks: the steps of the reference's paged KV cache (kv_cache.rs:22-73
 * QuantizedKvToken::quantize / dequantize / requantize over quant.rs:74-105,144-168; reference CUDA
 * kernels ctox_pack_paged_kv_q4_f32_sm86 and ctox_demote_paged_kv_q4_to_q2_sm86,
 * kernels/cuda/q2q4_fused_matvec_sm86.cu:1675-1835). All pointers are device memory; values are
 * [n_blocks][64] floats, blocks the canonical 34-byte Q4_B64 / 18-byte Q2_B64 encodings back to
 * back. The bytes equal the scalar code's for the same floats. A non-finite value or scale sets the
 * device error word (ctox_ctx_device_error). The executor's cache does not use these yet (it keeps
 * bf16 / f32 rows). */
ctox_status ctox_kv_pack_q4(ctox_ctx *ctx, const float *values, uint64_t n_blocks, uint8_t *q4_bytes);
/* Every block decoded and re-quantized to Q2_B64: what a page undergoes when it leaves the recent
 * window (kv_cache.rs:67-73,461-478). */
ctox_status ctox_kv_demote_q4_to_q2(ctox_ctx *ctx, const uint8_t *q4_bytes, uint64_t n_blocks, uint8_t *q2_bytes);
/* dtype: CTOX_Q2B64 or CTOX_Q4B64. */
ctox_status ctox_kv_unpack(ctox_ctx *ctx, uint32_t dtype, const uint8_t *bytes, uint64_t n_blocks, float *values);
/* beta = sigmoid(b), log_decay = -exp(A_log) * softplus(a + dt_bias)
 * (decoder.rs:29-35,881,897-902). a, b, log_decay, beta: [tokens][heads]. */
ctox_status ctox_gated_delta_prepare(ctox_ctx *ctx, const float *a, const float *b,
                                     const float *a_log, const float *dt_bias, float *log_decay,
                                     float *beta, uint32_t tokens, uint32_t heads);

/* ---- selection (sampler.rs:65-144, engine.rs:203-217,906-963; CUDA candidate
 * backend/cuda_runtime.rs:2376-2917: prepare_argmax_f32 / dispatch_argmax_f32_device,
 * prepare_mtp_compact_result / enqueue_mtp_accept_from_device_drafts /
 * verifier_read_mtp_compact_result) ---- */

#define CTOX_MAX_VERIFY_NODES 16

/* Result of one speculative verification, the counterpart of the reference's
 * CudaMtpCompactResultRecord (backend/cuda_runtime.rs:775-779) and of
 * ResolvedGreedyMtpVerification (engine.rs:110-116): emitted[0 .. n_emitted-2]
 * are the accepted draft tokens, emitted[n_emitted-1] is the next token (the
 * target's correction, or the bonus token when every draft was accepted);
 * path[i] is the tree node of the i-th accepted draft. */
typedef struct {
    uint32_t status; /* 0 = ok, 1 = a logit was not finite */
    uint32_t n_emitted;
    uint32_t emitted[CTOX_MAX_VERIFY_NODES + 1];
    int32_t path[CTOX_MAX_VERIFY_NODES];
    uint32_t node_argmax[CTOX_MAX_VERIFY_NODES]; /* greedy token of every node's distribution */
    uint32_t node_token[CTOX_MAX_VERIFY_NODES];  /* the draft token of every node, as verified */
} ctox_spec_record;

/* Greedy selection over device logits: the LAST maximal index under the IEEE
 * total order. row_ids (device, may be NULL) maps a local row to a token id
 * (restricted draft vocabulary). result_dev: two uint32 {token, status};
 * status 1 = non-finite logit. Enqueued on the context's stream. */
ctox_status ctox_argmax_f32(ctox_ctx *ctx, const float *logits_dev, uint32_t n,
                            const uint32_t *row_ids_dev, uint32_t *result_dev);
/* Host form of the same: synchronises and returns the token; a non-finite
 * logit is CTOX_INVALID_STATE (backend/cuda_runtime.rs:2790-2794). */
ctox_status ctox_argmax_f32_host(ctox_ctx *ctx, const float *logits_dev, uint32_t n,
                                 const uint32_t *row_ids_dev, uint32_t *token);
/* Sampler::sample_with_draw (sampler.rs:65-144; CUDA candidate ctox_topk_topp_sample_f32_sm86,
 * kernels/cuda/q2q4_fused_matvec_sm86.cu:2648, prepared by backend/cuda_runtime.rs:2728-2910):
 * temperature, top-k, top-p over n device logits with the caller's uniform draw in [0, 1).
 * temperature 0 = greedy. The device path takes top_k in 1..=1024 (the reference's 1..=256);
 * other values are CTOX_UNSUPPORTED_OPERATION. Host form: synchronises, returns the token.
 * Invalid draw / temperature / top_p and non-finite logits are CTOX_INVALID_ARTIFACT like the
 * reference's fail-closed sampler (sampler.rs:66-99). */
ctox_status ctox_sample_topk_topp(ctox_ctx *ctx, const float *logits_dev, uint32_t n,
                                  float temperature, uint32_t top_k, float top_p, float draw,
                                  uint32_t *token);
/* Fused lm_head -> softmax statistics -> acceptance for the n_nodes verify
 * positions of a draft tree (a chain is the tree parent[i] = i-1). hidden_dev:
 * n_nodes rows of the lm_head's input (CTOX_F32 or CTOX_BF16), row i being the
 * final hidden state after node i's token; node 0 is the current position.
 * parent[0] = -1, parent[i] < i; token[i] is node i's draft token (token[0]
 * unused). temperature 0 is greedy verification (engine.rs:939-962); otherwise
 * rejection sampling against softmax(logits/temperature) with Philox4x32-10
 * draws keyed by (seed, step) - no counterpart in the reference. vocab limits
 * selection to the first `vocab` rows (0 = all rows). logits_out_dev (may be
 * NULL): [n_nodes][rows] materialised logits for evidence paths. The weight
 * matrix is streamed once per pass of up to sixteen positions. Synchronises; one small
 * device-to-host read, like backend/cuda_runtime.rs:2707-2726. */
ctox_status ctox_lmhead_verify(ctox_matvec *lm_head, const void *hidden_dev, uint32_t hidden_dtype,
                               uint64_t hidden_stride, uint32_t n_nodes, const int32_t *parent,
                               const uint32_t *token, float temperature, uint64_t seed,
                               uint64_t step, uint32_t vocab, float *logits_out_dev,
                               ctox_spec_record *record);

/* ---- executor (engine.rs:322-362 trait ModelExecutor; CPU oracle executor
 * decoder.rs:1278-1458; CUDA candidate backend/cuda_executor.rs:797-1073 and the
 * graph backend/cuda_graph.rs:3166-3292,3763-5003) ---- */

typedef struct ctox_exec ctox_exec;

/* Qwen38Config (config.rs:12-58) plus deployment choices. */
typedef struct {
    uint32_t vocab_size, hidden_size, intermediate_size, num_hidden_layers;
    uint32_t num_attention_heads, num_key_value_heads, head_dim, rotary_dim;
    float rope_theta, rms_norm_epsilon;
    uint32_t full_attention_interval; /* layer l is full attention iff (l+1) % interval == 0 */
    uint32_t linear_num_key_heads, linear_num_value_heads, linear_key_head_dim, linear_value_head_dim;
    uint32_t linear_conv_kernel_dim;
    uint32_t mtp_num_hidden_layers; /* 0 or 1 */
    uint32_t max_context_tokens;
    uint32_t kv_page_tokens;    /* tokens per KV page */
    uint32_t kv_dtype;          /* CTOX_F32 or CTOX_BF16 */
    uint32_t max_draft_tokens;  /* k: drafts per speculative block, 0..7 */
    uint32_t draft_vocab;       /* rows of the restricted draft head, 0 = full vocabulary */
} ctox_model_config;

/* Tensors of the model. Fan-out groups are single matrices whose rows are the
 * members' rows in the listed order; they share one s_in (fanout.rs:31-70). */
enum {
    CTOX_T_EMBED = 0,          /* global, matrix vocab x hidden (tensor_contract.rs:70-249) */
    CTOX_T_LM_HEAD = 1,        /* global, matrix vocab x hidden */
    CTOX_T_FINAL_NORM = 2,     /* global, vector hidden */
    CTOX_T_INPUT_NORM = 3,     /* layer, vector hidden */
    CTOX_T_POST_NORM = 4,      /* layer, vector hidden */
    CTOX_T_ATTN_QKV = 5,       /* full layer, matrix [q+gate interleaved per head | k | v] x hidden */
    CTOX_T_ATTN_O = 6,         /* full layer, matrix hidden x (heads*head_dim) */
    CTOX_T_Q_NORM = 7,         /* full layer, vector head_dim */
    CTOX_T_K_NORM = 8,         /* full layer, vector head_dim */
    CTOX_T_LIN_IN = 9,         /* linear layer, matrix [in_proj_qkv | in_proj_z | in_proj_a | in_proj_b] x hidden */
    CTOX_T_LIN_OUT = 10,       /* linear layer, matrix hidden x (value_heads*value_dim) */
    CTOX_T_CONV_W = 11,        /* linear layer, vector channels*kernel */
    CTOX_T_A_LOG = 12,         /* linear layer, vector value_heads */
    CTOX_T_DT_BIAS = 13,       /* linear layer, vector value_heads */
    CTOX_T_LIN_NORM = 14,      /* linear layer, vector value_dim */
    CTOX_T_MLP_GATE_UP = 15,   /* layer, matrix [gate | up] x hidden */
    CTOX_T_MLP_DOWN = 16,      /* layer, matrix hidden x intermediate */
    CTOX_T_MTP_FC = 17,        /* global, matrix hidden x 2*hidden */
    CTOX_T_MTP_NORM_E = 18,    /* global, vector hidden (pre_fc_norm_embedding) */
    CTOX_T_MTP_NORM_H = 19,    /* global, vector hidden (pre_fc_norm_hidden) */
    CTOX_T_MTP_NORM = 20,      /* global, vector hidden (mtp.norm) */
    CTOX_T_DRAFT_IDS = 21      /* global, draft_vocab strictly increasing token ids (as uint32) */
};
#define CTOX_LAYER_GLOBAL 0xffffffffu
/* layer index of the MTP decoder layer = num_hidden_layers */

/* One speculative block (engine.rs:110-116 ResolvedGreedyMtpVerification). */
typedef struct {
    uint32_t proposed_drafts;
    uint32_t verified_drafts;
    uint32_t n_accepted;
    uint32_t accepted_draft_tokens[CTOX_MAX_VERIFY_NODES];
    uint32_t next_token;
    uint32_t draft_tokens[CTOX_MAX_VERIFY_NODES];
    uint32_t target_tokens[CTOX_MAX_VERIFY_NODES + 1]; /* greedy token after each verify position */
} ctox_exec_step;

ctox_status ctox_exec_create(ctox_ctx *ctx, const ctox_model_config *config, ctox_exec **out);
ctox_status ctox_exec_destroy(ctox_exec *exec); /* unload: frees every allocation */
/* load(): one tensor at a time, host memory. Matrices are FusedMatVec descriptions
 * without input (weights, s_in, s_out, optional bias). */
ctox_status ctox_exec_load_matrix(ctox_exec *exec, uint32_t layer, uint32_t tensor,
                                  const ctox_fused_matvec_op *op);
ctox_status ctox_exec_load_vector(ctox_exec *exec, uint32_t layer, uint32_t tensor, const float *values,
                                  uint64_t n);
/* Random-init weights of the configured shapes, generated on the device: codes
 * uniform, f16 block scales log-normal(mu, sigma) from a quantile table, recovery
 * scales U(0.75, 1.25), norm weights ~ N(0, 0.02). */
ctox_status ctox_exec_fill_synthetic(ctox_exec *exec, uint64_t seed, float scale_mu, float scale_sigma);
/* warmup(): checks that every tensor is present and builds launch plans. */
ctox_status ctox_exec_warmup(ctox_exec *exec);
ctox_status ctox_exec_reset_session(ctox_exec *exec);
/* Cancellation (engine.rs:364-377 CancellationToken = Arc<AtomicBool>): `cancel` points to a
 * word another thread may set to non-zero at any time, or is NULL. It is read on the host at
 * entry and between passes; a call that sees it returns CTOX_CANCELLED (error.rs:5-29). A
 * cancelled decode leaves the session as it was before the call; a cancelled prefill leaves no
 * usable session (reset_session or a new prefill). */

/* prefill(): runs the tokens through the target (and the MTP cache) in chunks;
 * the last token is NOT consumed: it is the input of the first decode. */
ctox_status ctox_exec_prefill(ctox_exec *exec, const uint32_t *tokens, uint64_t n,
                              const volatile int32_t *cancel);
/* Benchmark prefill: fills `n` cache positions with random K/V ~ N(0,1) and random
 * recurrent state instead of running the model, and sets the position. */
ctox_status ctox_exec_prefill_synthetic(ctox_exec *exec, uint64_t n, uint64_t seed);
/* decode(): consumes `token` at the current position. With mtp_enabled, drafts
 * max_draft_tokens tokens, verifies them in one target pass and resolves the
 * acceptance on the device (temperature 0: engine.rs:939-962). The state is
 * committed on the device for the accepted prefix before returning, and the block
 * stays pending until ctox_exec_commit_speculative confirms it (a second decode
 * before that is CTOX_INVALID_STATE, like decoder.rs:1293-1297). force_accept >= 0
 * accepts exactly that many drafts regardless of the target (throughput buckets).
 *
 * The three forms of ExecutorStep (engine.rs:77-150,240-319) map onto the result so:
 *  - resolved (ResolvedGreedyMtpVerification): proposed_drafts, verified_drafts,
 *    accepted_draft_tokens[0..n_accepted), next_token: the form this executor reports;
 *  - compact (GreedyMtpVerification): draft_tokens[0..k), target_tokens[0..k) and
 *    bonus_token = target_tokens[k], k = proposed_drafts;
 *  - logit form: with ctox_exec_keep_logits on, target_logits / target_verification_logits[i] /
 *    bonus_logits are ctox_exec_last_logits(i) for i = 0 / 0..k-1 / k, and the restricted
 *    draft distributions are ctox_exec_last_draft_logits(i) over the draft id table.
 * A device error (a bounded wait that ran out, a non-finite scale) invalidates the session:
 * every later call fails with CTOX_INVALID_STATE until ctox_exec_reset_session or a prefill
 * (engine.rs:594-611). */
ctox_status ctox_exec_decode(ctox_exec *exec, uint32_t token, int32_t mtp_enabled, float temperature,
                             uint64_t seed, int32_t force_accept, const volatile int32_t *cancel,
                             ctox_exec_step *step);
/* commit_speculative() (engine.rs:322-362, decoder.rs:1396-1458): resolves the branch an MTP
 * decode left pending. accepted_drafts must equal the n_accepted the decode reported: the
 * device already holds exactly that state; any other depth is CTOX_INVALID_STATE, as is a call
 * with no pending branch. */
ctox_status ctox_exec_commit_speculative(ctox_exec *exec, uint32_t accepted_drafts,
                                         const volatile int32_t *cancel);
/* pending_accepted: -1, or the accepted depth of the block awaiting commit_speculative;
 * poisoned: 1 after a device error until reset_session. Either pointer may be NULL. */
ctox_status ctox_exec_session_state(const ctox_exec *exec, int32_t *pending_accepted, int32_t *poisoned);
/* Host time, in microseconds, that the last decode call spent enqueuing its kernels before it
 * waited for the device: the launch path's cost, which bounds a block when the shards are small
 * (the reference bench reports the same split, src/bin/cuda_target_mtp4_graph_bench.rs:36-64). */
ctox_status ctox_exec_last_enqueue_us(const ctox_exec *exec, double *microseconds);
/* Device time of the phases of a decode call, measured with events at the phase boundaries when
 * enabled (off by default: an event between two kernels ends their overlap there): ms4 = {MTP
 * catch-up + chained drafts, target pass, lm_head + statistics + acceptance, commit of the accepted
 * prefix} of the last call. The reference's loop bench reports the same split
 * (src/bin/cuda_target_mtp4_graph_bench.rs:36-64,124-136). */
ctox_status ctox_exec_phase_timing(ctox_exec *exec, int32_t enable);
ctox_status ctox_exec_last_phase_ms(ctox_exec *exec, float *ms4);
ctox_status ctox_exec_position(const ctox_exec *exec, uint64_t *position);
/* Final hidden state of the last committed position (device -> host), for parity tests. */
ctox_status ctox_exec_last_hidden(ctox_exec *exec, float *out);
/* Logits of the verify positions of the last decode: [positions][vocab] (evidence path;
 * enabled with ctox_exec_keep_logits). */
ctox_status ctox_exec_keep_logits(ctox_exec *exec, int32_t enable);
ctox_status ctox_exec_last_logits(ctox_exec *exec, uint32_t position, float *out);
/* Evidence of the MTP layer (decoder.rs:1009-1046), kept while ctox_exec_keep_logits is on: the
 * final hidden state (after mtp.norm) of every (token, previous hidden) pair the last decode ran,
 * in order (first the pairs of the previous block with the target's own hidden states, then the
 * chained drafts), and the logits of draft `draft` over the rows of the draft head (the draft id
 * table's entries on this rank, or the vocabulary shard when draft_vocab is 0). `count` receives
 * how many are held; `out` may be NULL to query the counts only. */
ctox_status ctox_exec_last_mtp_hidden(ctox_exec *exec, uint32_t index, float *out, uint32_t *count);
ctox_status ctox_exec_last_draft_logits(ctox_exec *exec, uint32_t draft, float *out, uint32_t *rows,
                                        uint32_t *count);
/* ModelExecutor::select_target_token (engine.rs:322-362): samples the target token of verify
 * position `position` of the last decode call from the logits the executor kept on the device
 * (ctox_exec_keep_logits must be on), with the same rules as ctox_sample_topk_topp. In a
 * tensor-parallel group the kept logits are a vocabulary shard: CTOX_UNSUPPORTED_OPERATION. */
ctox_status ctox_exec_select_target(ctox_exec *exec, uint32_t position, float temperature,
                                    uint32_t top_k, float top_p, float draw, uint32_t *token);
ctox_status ctox_exec_allocated_bytes(const ctox_exec *exec, uint64_t *model, uint64_t *session);

#ifdef __cplusplus
}
#endif
#endif
