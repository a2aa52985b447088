/*
 * CPU oracle for the CTOX-LLM Qwen3.8-27B decode hot path.
 *
 * TEST INFRASTRUCTURE ONLY. This is a plain-C restatement of the reference
 * crate's scalar arithmetic (models/qwen38_27b/src/{quant,reference,sampler,
 * engine}.rs and backend/cpu.rs). It is the checker for the CUDA library and
 * the timed CPU baseline; no product code path links, loads or calls it.
 *
 * Status codes mirror the variants of the reference's EngineError
 * (models/qwen38_27b/src/error.rs:5-29).
 */
#ifndef CTOX_ORACLE_H
#define CTOX_ORACLE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum {
    ORC_OK = 0,
    ORC_SHAPE = 1,
    ORC_INVALID_ARTIFACT = 2,
    ORC_UNSUPPORTED_DTYPE = 3,
    ORC_UNSUPPORTED_OPERATION = 4,
    ORC_MEMORY_BUDGET = 5,
    ORC_INVALID_STATE = 6,
    ORC_CANCELLED = 7
};

/* TensorDType (models/qwen38_27b/src/format.rs:26-32). */
enum { ORC_Q2B64 = 0, ORC_Q4B64 = 1, ORC_MIXED_Q2Q4B64 = 2, ORC_F16 = 3, ORC_F32 = 4 };
/* Activation (models/qwen38_27b/src/backend/mod.rs:54-57). */
enum { ORC_ACT_IDENTITY = 0, ORC_ACT_SILU = 1 };
/* ScaleSlice kinds (backend/mod.rs:74-77). */
enum { ORC_SCALE_NONE = 0, ORC_SCALE_F32 = 1, ORC_SCALE_F16LE = 2 };

/* QuantSegment (models/qwen38_27b/src/format.rs:56-64). */
typedef struct {
    uint32_t group_index;
    uint32_t dtype;
    uint64_t row_start;
    uint64_t row_end;
    uint64_t offset;
    uint64_t length;
} orc_segment;

/* FusedMatVec (backend/mod.rs:115-128). */
typedef struct {
    uint32_t dtype;
    uint32_t activation;
    const uint8_t *weights;
    uint64_t weights_len;
    const orc_segment *segments;
    uint64_t n_segments;
    uint64_t rows;
    uint64_t columns;
    const float *input;
    uint64_t input_len;
    uint32_t s_in_kind;
    uint32_t s_out_kind;
    const void *s_in;
    uint64_t s_in_len; /* values */
    const void *s_out;
    uint64_t s_out_len; /* values */
    const float *bias;
    uint64_t bias_len;
} orc_fused_matvec;

/* f16 helpers (the `half` crate: IEEE binary16, round to nearest even). */
float orc_f16_to_f32(uint16_t bits);
uint16_t orc_f32_to_f16(float value);

/* quant.rs:73-205 */
int orc_q2_quantize_block(const float *values64, uint8_t *out18);
int orc_q4_quantize_block(const float *values64, uint8_t *out34);
int orc_q2_dequantize_block(const uint8_t *in18, float *out64);
int orc_q4_dequantize_block(const uint8_t *in34, float *out64);
int orc_quantize_matrix(uint32_t dtype, const float *values, uint64_t rows, uint64_t columns,
                        uint8_t *out);
/* quant.rs:46-61 */
int orc_a8_quantize_block(const float *values64, float *scale, int8_t *codes64);

/* backend/cpu.rs:41-310,432-497 (ScalarVerifier arm). */
int orc_fused_matvec_run(const orc_fused_matvec *op, float *out);
/* Same arithmetic, rows partitioned over `threads` host threads (bit-identical
 * to the single-threaded call because rows are independent). */
int orc_fused_matvec_run_mt(const orc_fused_matvec *op, float *out, int threads);
int orc_fused_matvec_fanout(const orc_fused_matvec *ops, uint64_t n, float *const *outs);
int orc_recovered_row(uint32_t dtype, const uint8_t *weights, uint64_t weights_len,
                      uint64_t columns, uint32_t s_in_kind, const void *s_in, uint64_t s_in_len,
                      float s_out, float *out);
int orc_recovered_row_matvec(uint32_t dtype, const uint8_t *weights, uint64_t weights_len,
                             const float *corrected_input, uint64_t columns, float s_out,
                             float *out);
/* x86-64 AVX2 arm (backend/cpu.rs:595-658); returns ORC_UNSUPPORTED_OPERATION
 * when the build or the CPU lacks AVX2. */
int orc_fused_matvec_run_avx2(const orc_fused_matvec *op, float *out, int threads);

/* reference.rs */
float orc_silu(float value);
int orc_rms_norm_1p_weight(const float *values, uint64_t rows, uint64_t columns,
                           const float *weight, float epsilon, float *out);
int orc_rms_norm_gated(const float *values, const float *gate, uint64_t rows, uint64_t columns,
                       const float *weight, float epsilon, float *out);
int orc_swiglu(const float *gate, const float *up, uint64_t n, float *out);
int orc_apply_partial_rope(float *query, float *key, uint64_t query_heads, uint64_t key_heads,
                           uint64_t head_dim, uint64_t rotary_dim, uint64_t position, float theta);
int orc_causal_conv_silu_update(const float *input, float *state, const float *weight,
                                uint64_t channels, uint64_t kernel, float *out);
int orc_causal_conv_silu_update_f16_state(const float *input, uint16_t *state, const float *weight,
                                          uint64_t channels, uint64_t kernel, float *out);
int orc_recurrent_gated_delta_step(const float *query, const float *key, const float *value,
                                   const float *log_decay, const float *beta, float *state,
                                   uint64_t heads, uint64_t key_dim, uint64_t value_dim,
                                   float *out);
int orc_recurrent_gated_delta_step_f16_state(const float *query, const float *key,
                                             const float *value, const float *log_decay,
                                             const float *beta, uint16_t *state, uint64_t heads,
                                             uint64_t key_dim, uint64_t value_dim, float *out);
int orc_recurrent_gated_delta_sequence(const float *query, const float *key, const float *value,
                                       const float *log_decay, const float *beta, float *state,
                                       uint64_t tokens, uint64_t heads, uint64_t key_dim,
                                       uint64_t value_dim, float *out);
int orc_grouped_query_attention(const float *query, const float *key, const float *value,
                                uint64_t query_heads, uint64_t key_value_heads,
                                uint64_t query_tokens, uint64_t key_value_tokens,
                                uint64_t head_dim, uint64_t query_start_position, float *out);
int orc_sigmoid_gate(float *values, const float *gate, uint64_t n);

/* decoder.rs:29-65,881,897-902 */
float orc_softplus(float value);
int orc_repeat_heads(const float *in, uint64_t source_heads, uint64_t target_heads,
                     uint64_t head_dim, float *out);
int orc_gated_delta_prepare(const float *a, const float *b, const float *a_log,
                            const float *dt_bias, uint64_t heads, float *log_decay, float *beta);

/* sampler.rs */
int orc_greedy_token(const float *logits, uint64_t n, uint32_t *token);
int orc_sample_with_draw(const float *logits, uint64_t n, float temperature, uint64_t top_k,
                         float top_p, float draw, uint32_t *token);
void orc_pcg32_new(uint64_t seed, uint64_t *state);
uint32_t orc_pcg32_next_u32(uint64_t *state);
float orc_pcg32_next_f32(uint64_t *state);

/* engine.rs:915-963 */
int orc_verify_greedy_mtp_tokens(const uint32_t *draft_tokens, const uint32_t *target_tokens,
                                 uint64_t k, uint32_t bonus_token, uint32_t *next_token,
                                 uint32_t *verified, uint32_t *accepted, uint32_t *n_accepted);
int orc_verify_greedy_mtp_logits(const float *const *draft_logits, const uint64_t *draft_len,
                                 const uint32_t *const *draft_token_ids,
                                 const float *const *target_logits, uint64_t vocab, uint64_t k,
                                 const float *bonus_logits, uint32_t *next_token,
                                 uint32_t *verified, uint32_t *accepted, uint32_t *n_accepted);

/* Philox4x32-10 (Salmon et al. 2011), counter-based; no reference counterpart
 * (the reference has no device RNG). */
void orc_philox4x32_10(const uint32_t counter[4], const uint32_t key[2], uint32_t out[4]);
float orc_u32_to_unit_f32(uint32_t bits);

/* Speculative sampling over a draft tree; no reference counterpart (the
 * reference fails closed on stochastic MTP, engine.rs:583-590, and drafts a
 * chain only). Node 0 is the root (the position of the current token); node n
 * carries draft token node_token[n] and parent[n] < n. target_logits[n] is the
 * target distribution after consuming node n's path. The drafter is
 * deterministic (q is a point mass), so child c of node n is accepted with
 * probability p_n(c) / (1 - sum of p_n over its earlier, rejected siblings);
 * when no child is accepted the emitted token is drawn from p_n restricted to
 * tokens that are not children of n (Gumbel-max with Philox noise). With
 * temperature 0 the rule degenerates to verify_greedy_mtp (engine.rs:939-962).
 * emitted[] receives the accepted draft tokens followed by the final token. */
float orc_gumbel_from_bits(uint32_t bits);
float orc_accept_draw(uint64_t seed, uint64_t step, uint32_t node);
float orc_gumbel_noise(uint64_t seed, uint64_t step, uint32_t node, uint32_t token);
int orc_softmax_stats(const float *logits, uint64_t n, float inv_temperature, float *max_out,
                      float *sum_out);
int orc_spec_tree_accept(const float *target_logits, uint64_t vocab, const int32_t *parent,
                         const uint32_t *node_token, uint64_t n_nodes, float temperature,
                         uint64_t seed, uint64_t step, uint32_t *emitted, uint32_t *n_emitted,
                         int32_t *path_nodes);

#ifdef __cplusplus
}
#endif
#endif
