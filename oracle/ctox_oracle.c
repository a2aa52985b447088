/*
 * CPU oracle for the CTOX-LLM Qwen3.8-27B decode hot path (plain C).
 *
 * TEST INFRASTRUCTURE ONLY: the checker for the CUDA library and the timed CPU
 * baseline. Nothing in the product path links, loads or calls this file.
 *
 * Every function restates the scalar arithmetic of the reference crate in the
 * same evaluation order; the reference file:line it follows is cited above it
 * (paths relative to models/qwen38_27b/src/). Build with
 *   gcc -O2 -ffp-contract=off -fno-fast-math
 * so that no multiply-add is contracted (Rust never contracts).
 */
#include "ctox_oracle.h"

#include <math.h>
#include <pthread.h>
#include <stdlib.h>
#include <string.h>

#define BLOCK_LEN 64
#define Q2_BLOCK_BYTES 18
#define Q4_BLOCK_BYTES 34

/* quant.rs:8 */
static const float Q2_CODEBOOK[4] = {-1.0f, -1.0f / 3.0f, 1.0f / 3.0f, 1.0f};

/* ---- binary16 <-> binary32 (the `half` crate: f16::to_f32 / f16::from_f32,
 * round to nearest even, subnormals preserved) ---- */
float orc_f16_to_f32(uint16_t h) {
    uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1fu;
    uint32_t man = h & 0x3ffu;
    uint32_t bits;
    if (exp == 0) {
        if (man == 0) {
            bits = sign;
        } else {
            int shift = 0;
            while ((man & 0x400u) == 0) {
                man <<= 1;
                shift++;
            }
            man &= 0x3ffu;
            bits = sign | ((uint32_t)(127 - 15 - shift + 1) << 23) | (man << 13);
        }
    } else if (exp == 31) {
        bits = sign | 0x7f800000u | (man << 13);
    } else {
        bits = sign | ((exp + 127 - 15) << 23) | (man << 13);
    }
    float out;
    memcpy(&out, &bits, 4);
    return out;
}

uint16_t orc_f32_to_f16(float value) {
    uint32_t x;
    memcpy(&x, &value, 4);
    uint32_t sign = (x >> 16) & 0x8000u;
    uint32_t exp = (x >> 23) & 0xffu;
    uint32_t man = x & 0x7fffffu;
    if (exp == 0xff) {
        if (man == 0) return (uint16_t)(sign | 0x7c00u);
        return (uint16_t)(sign | 0x7e00u | (man >> 13));
    }
    int32_t e = (int32_t)exp - 127 + 15;
    if (e >= 31) return (uint16_t)(sign | 0x7c00u);
    if (e <= 0) {
        if (e < -10) return (uint16_t)sign;
        man |= 0x800000u;
        uint32_t shift = (uint32_t)(14 - e);
        uint32_t half_man = man >> shift;
        uint32_t rem = man & ((1u << shift) - 1u);
        uint32_t halfway = 1u << (shift - 1);
        if (rem > halfway || (rem == halfway && (half_man & 1u))) half_man++;
        return (uint16_t)(sign | half_man);
    }
    uint32_t half = sign | ((uint32_t)e << 10) | (man >> 13);
    uint32_t rem = man & 0x1fffu;
    if (rem > 0x1000u || (rem == 0x1000u && (half & 1u))) half++;
    return (uint16_t)half;
}

static int is_finite_f(float v) { return isfinite(v) ? 1 : 0; }

/* f32::total_cmp key: monotone map of the IEEE bit pattern to a signed order. */
static int32_t total_key(float v) {
    int32_t b;
    memcpy(&b, &v, 4);
    b ^= (int32_t)(((uint32_t)(b >> 31)) >> 1);
    return b;
}

/* quant.rs:31-44 */
static int require_block(const float *values) {
    for (int i = 0; i < BLOCK_LEN; i++)
        if (!is_finite_f(values[i])) return ORC_INVALID_ARTIFACT;
    return ORC_OK;
}

/* Rust f32::round: half away from zero. */
static float round_half_away(float v) { return roundf(v); }

/* quant.rs:74-105 */
int orc_q2_quantize_block(const float *values, uint8_t *out) {
    int rc = require_block(values);
    if (rc) return rc;
    float scale = 0.0f;
    for (int i = 0; i < BLOCK_LEN; i++) {
        float a = fabsf(values[i]);
        scale = a > scale ? a : scale; /* f32::max */
    }
    memset(out, 0, Q2_BLOCK_BYTES);
    if (scale == 0.0f) return ORC_OK;
    for (int i = 0; i < BLOCK_LEN; i++) {
        float normalized = values[i] / scale;
        /* Iterator::min_by keeps the first minimal element. */
        int best = 0;
        float best_d = fabsf(normalized - Q2_CODEBOOK[0]);
        for (int c = 1; c < 4; c++) {
            float d = fabsf(normalized - Q2_CODEBOOK[c]);
            if (total_key(d) < total_key(best_d)) {
                best = c;
                best_d = d;
            }
        }
        out[2 + i / 4] |= (uint8_t)(best << ((i % 4) * 2));
    }
    uint16_t bits = orc_f32_to_f16(scale);
    out[0] = (uint8_t)(bits & 0xff);
    out[1] = (uint8_t)(bits >> 8);
    return ORC_OK;
}

/* quant.rs:144-168 */
int orc_q4_quantize_block(const float *values, uint8_t *out) {
    int rc = require_block(values);
    if (rc) return rc;
    float scale = 0.0f;
    for (int i = 0; i < BLOCK_LEN; i++) {
        float a = fabsf(values[i]);
        scale = a > scale ? a : scale;
    }
    memset(out, 0, Q4_BLOCK_BYTES);
    if (scale == 0.0f) return ORC_OK;
    for (int i = 0; i < BLOCK_LEN; i++) {
        float normalized = values[i] / scale;
        if (normalized < -1.0f) normalized = -1.0f;
        if (normalized > 1.0f) normalized = 1.0f;
        float r = round_half_away((normalized * 7.5f) + 7.5f);
        if (r < 0.0f) r = 0.0f;
        if (r > 15.0f) r = 15.0f;
        uint8_t code = (uint8_t)r;
        out[2 + i / 2] |= (uint8_t)(code << ((i % 2) * 4));
    }
    uint16_t bits = orc_f32_to_f16(scale);
    out[0] = (uint8_t)(bits & 0xff);
    out[1] = (uint8_t)(bits >> 8);
    return ORC_OK;
}

static float block_scale(const uint8_t *block) {
    return orc_f16_to_f32((uint16_t)(block[0] | ((uint16_t)block[1] << 8)));
}

/* quant.rs:107-115,124-140 */
int orc_q2_dequantize_block(const uint8_t *in, float *out) {
    float scale = block_scale(in);
    if (!is_finite_f(scale)) return ORC_INVALID_ARTIFACT;
    for (int i = 0; i < BLOCK_LEN; i++) {
        unsigned code = (in[2 + i / 4] >> ((i % 4) * 2)) & 0x3u;
        out[i] = scale * Q2_CODEBOOK[code];
    }
    return ORC_OK;
}

/* quant.rs:170-179,188-204 */
int orc_q4_dequantize_block(const uint8_t *in, float *out) {
    float scale = block_scale(in);
    if (!is_finite_f(scale)) return ORC_INVALID_ARTIFACT;
    for (int i = 0; i < BLOCK_LEN; i++) {
        unsigned code = (in[2 + i / 2] >> ((i % 2) * 4)) & 0xfu;
        float normalized = ((float)code - 7.5f) / 7.5f;
        out[i] = scale * normalized;
    }
    return ORC_OK;
}

int orc_quantize_matrix(uint32_t dtype, const float *values, uint64_t rows, uint64_t columns,
                        uint8_t *out) {
    if (columns == 0 || rows == 0 || columns % BLOCK_LEN) return ORC_SHAPE;
    uint64_t blocks = rows * (columns / BLOCK_LEN);
    for (uint64_t b = 0; b < blocks; b++) {
        int rc;
        if (dtype == ORC_Q2B64)
            rc = orc_q2_quantize_block(values + b * BLOCK_LEN, out + b * Q2_BLOCK_BYTES);
        else if (dtype == ORC_Q4B64)
            rc = orc_q4_quantize_block(values + b * BLOCK_LEN, out + b * Q4_BLOCK_BYTES);
        else
            return ORC_UNSUPPORTED_DTYPE;
        if (rc) return rc;
    }
    return ORC_OK;
}

/* quant.rs:46-61 (f32::round_ties_even == rintf under the default mode) */
int orc_a8_quantize_block(const float *values, float *scale_out, int8_t *codes) {
    int rc = require_block(values);
    if (rc) return rc;
    float maximum = 0.0f;
    for (int i = 0; i < BLOCK_LEN; i++) {
        float a = fabsf(values[i]);
        maximum = a > maximum ? a : maximum;
    }
    memset(codes, 0, BLOCK_LEN);
    if (maximum == 0.0f) {
        *scale_out = 0.0f;
        return ORC_OK;
    }
    float scale = maximum / 127.0f;
    for (int i = 0; i < BLOCK_LEN; i++) {
        float r = rintf(values[i] / scale);
        if (r < -127.0f) r = -127.0f;
        if (r > 127.0f) r = 127.0f;
        codes[i] = (int8_t)r;
    }
    *scale_out = scale;
    return ORC_OK;
}

/* ---- backend/mod.rs:79-112 ScaleSlice ---- */
static int scale_value(uint32_t kind, const void *data, uint64_t len, uint64_t index, float *out) {
    if (index >= len) return ORC_SHAPE;
    float v;
    if (kind == ORC_SCALE_F32) {
        v = ((const float *)data)[index];
    } else {
        const uint8_t *bytes = (const uint8_t *)data;
        v = orc_f16_to_f32((uint16_t)(bytes[2 * index] | ((uint16_t)bytes[2 * index + 1] << 8)));
    }
    if (!is_finite_f(v)) return ORC_INVALID_ARTIFACT;
    *out = v;
    return ORC_OK;
}

/* backend/mod.rs:59-66 and reference.rs:14-16 */
float orc_silu(float value) { return value / (1.0f + expf(-value)); }

static float apply_activation(uint32_t activation, float v) {
    return activation == ORC_ACT_SILU ? orc_silu(v) : v;
}

/* backend/cpu.rs:558-565 */
static float scalar_packed_q2_dot(float scale, const uint8_t *codes, const float *input) {
    float sum = 0.0f;
    for (int i = 0; i < BLOCK_LEN; i++) {
        unsigned code = (codes[i / 4] >> ((i % 4) * 2)) & 0x3u;
        sum += scale * Q2_CODEBOOK[code] * input[i];
    }
    return sum;
}

/* backend/cpu.rs:567-575 */
static float scalar_packed_q4_dot(float scale, const uint8_t *codes, const float *input) {
    float sum = 0.0f;
    for (int i = 0; i < BLOCK_LEN; i++) {
        unsigned code = (codes[i / 2] >> ((i % 2) * 4)) & 0xfu;
        float normalized = ((float)code - 7.5f) / 7.5f;
        sum += scale * normalized * input[i];
    }
    return sum;
}

/* backend/cpu.rs:180-226 */
static int row_sum(uint32_t dtype, const uint8_t *row, uint64_t blocks, const float *input,
                   float *out) {
    float sum = 0.0f;
    uint64_t bb = dtype == ORC_Q2B64 ? Q2_BLOCK_BYTES : Q4_BLOCK_BYTES;
    for (uint64_t b = 0; b < blocks; b++) {
        const uint8_t *block = row + b * bb;
        float scale = block_scale(block);
        if (!is_finite_f(scale)) return ORC_INVALID_ARTIFACT;
        if (dtype == ORC_Q2B64)
            sum += scalar_packed_q2_dot(scale, block + 2, input + b * BLOCK_LEN);
        else
            sum += scalar_packed_q4_dot(scale, block + 2, input + b * BLOCK_LEN);
    }
    *out = sum;
    return ORC_OK;
}

/* backend/cpu.rs:41-173 */
static int validate(const orc_fused_matvec *op, uint64_t *blocks_per_row) {
    if (op->columns == 0 || op->rows == 0 || op->columns % BLOCK_LEN) return ORC_SHAPE;
    if (op->input_len != op->columns) return ORC_SHAPE;
    if (op->s_in_kind != ORC_SCALE_NONE && op->s_in_len != op->columns) return ORC_SHAPE;
    if (op->s_out_kind != ORC_SCALE_NONE && op->s_out_len != op->rows) return ORC_SHAPE;
    if (op->bias && op->bias_len != op->rows) return ORC_SHAPE;
    uint64_t bpr = op->columns / BLOCK_LEN;
    uint64_t block_bytes = 0;
    if (op->dtype == ORC_Q2B64)
        block_bytes = Q2_BLOCK_BYTES;
    else if (op->dtype == ORC_Q4B64)
        block_bytes = Q4_BLOCK_BYTES;
    else if (op->dtype != ORC_MIXED_Q2Q4B64)
        return ORC_UNSUPPORTED_DTYPE;
    if (block_bytes) {
        if (op->n_segments) return ORC_INVALID_ARTIFACT;
        uint64_t blocks, expected;
        if (__builtin_mul_overflow(op->rows, bpr, &blocks) ||
            __builtin_mul_overflow(blocks, block_bytes, &expected))
            return ORC_SHAPE;
        if (op->weights_len != expected) return ORC_SHAPE;
        *blocks_per_row = bpr;
        return ORC_OK;
    }
    if (op->n_segments == 0) return ORC_INVALID_ARTIFACT;
    uint64_t expected_row = 0, expected_offset = 0;
    for (uint64_t g = 0; g < op->n_segments; g++) {
        const orc_segment *s = &op->segments[g];
        if (s->group_index != g || s->row_start != expected_row || s->row_end <= s->row_start ||
            s->row_end > op->rows || s->offset != expected_offset)
            return ORC_INVALID_ARTIFACT;
        uint64_t sbb;
        if (s->dtype == ORC_Q2B64)
            sbb = Q2_BLOCK_BYTES;
        else if (s->dtype == ORC_Q4B64)
            sbb = Q4_BLOCK_BYTES;
        else
            return ORC_INVALID_ARTIFACT;
        uint64_t blocks, expected_length;
        if (__builtin_mul_overflow(s->row_end - s->row_start, bpr, &blocks) ||
            __builtin_mul_overflow(blocks, sbb, &expected_length))
            return ORC_SHAPE;
        if (s->length != expected_length) return ORC_INVALID_ARTIFACT;
        expected_row = s->row_end;
        if (__builtin_add_overflow(expected_offset, s->length, &expected_offset)) return ORC_SHAPE;
    }
    if (expected_row != op->rows || expected_offset != op->weights_len) return ORC_SHAPE;
    *blocks_per_row = bpr;
    return ORC_OK;
}

/* backend/cpu.rs:228-240 */
static int corrected_input(const orc_fused_matvec *op, float **owned, const float **input) {
    *owned = NULL;
    *input = op->input;
    if (op->s_in_kind == ORC_SCALE_NONE) return ORC_OK;
    float *buf = (float *)malloc(sizeof(float) * op->columns);
    if (!buf) return ORC_MEMORY_BUDGET;
    for (uint64_t i = 0; i < op->columns; i++) {
        float s;
        int rc = scale_value(op->s_in_kind, op->s_in, op->s_in_len, i, &s);
        if (rc) {
            free(buf);
            return rc;
        }
        buf[i] = op->input[i] * s;
    }
    *owned = buf;
    *input = buf;
    return ORC_OK;
}

/* backend/cpu.rs:249-257 */
static int finish_row(const orc_fused_matvec *op, uint64_t row, float sum, float *out) {
    sum += op->bias ? op->bias[row] : 0.0f;
    float s = 1.0f;
    if (op->s_out_kind != ORC_SCALE_NONE) {
        int rc = scale_value(op->s_out_kind, op->s_out, op->s_out_len, row, &s);
        if (rc) return rc;
    }
    sum *= s;
    *out = apply_activation(op->activation, sum);
    return ORC_OK;
}

/* Locate the packed bytes of one logical row (pure or mixed layout). */
static int locate_row(const orc_fused_matvec *op, uint64_t bpr, uint64_t row,
                      const uint8_t **bytes, uint32_t *dtype) {
    if (op->dtype != ORC_MIXED_Q2Q4B64) {
        uint64_t bb = op->dtype == ORC_Q2B64 ? Q2_BLOCK_BYTES : Q4_BLOCK_BYTES;
        *bytes = op->weights + row * bpr * bb;
        *dtype = op->dtype;
        return ORC_OK;
    }
    for (uint64_t g = 0; g < op->n_segments; g++) {
        const orc_segment *s = &op->segments[g];
        if (row >= s->row_start && row < s->row_end) {
            uint64_t bb = s->dtype == ORC_Q2B64 ? Q2_BLOCK_BYTES : Q4_BLOCK_BYTES;
            *bytes = op->weights + s->offset + (row - s->row_start) * bpr * bb;
            *dtype = s->dtype;
            return ORC_OK;
        }
    }
    return ORC_SHAPE;
}

/* backend/cpu.rs:242-310 over a row range */
static int execute_rows(const orc_fused_matvec *op, uint64_t bpr, const float *input,
                        uint64_t row_begin, uint64_t row_end, float *out) {
    for (uint64_t row = row_begin; row < row_end; row++) {
        const uint8_t *bytes;
        uint32_t dtype;
        int rc = locate_row(op, bpr, row, &bytes, &dtype);
        if (rc) return rc;
        float sum;
        rc = row_sum(dtype, bytes, bpr, input, &sum);
        if (rc) return rc;
        rc = finish_row(op, row, sum, &out[row]);
        if (rc) return rc;
    }
    return ORC_OK;
}

/* backend/cpu.rs:432-442 */
int orc_fused_matvec_run(const orc_fused_matvec *op, float *out) {
    uint64_t bpr;
    int rc = validate(op, &bpr);
    if (rc) return rc;
    float *owned;
    const float *input;
    rc = corrected_input(op, &owned, &input);
    if (rc) return rc;
    rc = execute_rows(op, bpr, input, 0, op->rows, out);
    free(owned);
    return rc;
}

typedef struct {
    const orc_fused_matvec *op;
    uint64_t bpr;
    const float *input;
    uint64_t row_begin, row_end;
    float *out;
    int rc;
    int avx2;
} mt_job;

static int execute_rows_avx2(const orc_fused_matvec *op, uint64_t bpr, const float *input,
                             uint64_t row_begin, uint64_t row_end, float *out);

static void *mt_worker(void *arg) {
    mt_job *job = (mt_job *)arg;
    job->rc = job->avx2 ? execute_rows_avx2(job->op, job->bpr, job->input, job->row_begin,
                                            job->row_end, job->out)
                        : execute_rows(job->op, job->bpr, job->input, job->row_begin,
                                       job->row_end, job->out);
    return NULL;
}

static int run_mt(const orc_fused_matvec *op, float *out, int threads, int avx2) {
    uint64_t bpr;
    int rc = validate(op, &bpr);
    if (rc) return rc;
    float *owned;
    const float *input;
    rc = corrected_input(op, &owned, &input);
    if (rc) return rc;
    if (threads < 1) threads = 1;
    if ((uint64_t)threads > op->rows) threads = (int)op->rows;
    pthread_t *tids = (pthread_t *)malloc(sizeof(pthread_t) * (size_t)threads);
    mt_job *jobs = (mt_job *)malloc(sizeof(mt_job) * (size_t)threads);
    uint64_t per = (op->rows + (uint64_t)threads - 1) / (uint64_t)threads;
    for (int t = 0; t < threads; t++) {
        uint64_t b = per * (uint64_t)t, e = b + per;
        if (b > op->rows) b = op->rows;
        if (e > op->rows) e = op->rows;
        jobs[t] = (mt_job){op, bpr, input, b, e, out, ORC_OK, avx2};
        pthread_create(&tids[t], NULL, mt_worker, &jobs[t]);
    }
    for (int t = 0; t < threads; t++) {
        pthread_join(tids[t], NULL);
        if (jobs[t].rc && !rc) rc = jobs[t].rc;
    }
    free(tids);
    free(jobs);
    free(owned);
    return rc;
}

int orc_fused_matvec_run_mt(const orc_fused_matvec *op, float *out, int threads) {
    return run_mt(op, out, threads, 0);
}

/* ---- AVX2 arm: backend/cpu.rs:577-658. Eight f32 lanes, multiply then add
 * (no FMA), horizontal sum in lane order. ---- */
#if defined(__x86_64__)
#include <immintrin.h>

__attribute__((target("avx2"))) static float avx2_hsum(__m256 v) {
    float lanes[8];
    _mm256_storeu_ps(lanes, v);
    float s = 0.0f;
    for (int i = 0; i < 8; i++) s += lanes[i];
    return s;
}

/* cpu.rs:595-626: (scale/3) * (2*code-3), codes extracted by per-lane shifts. */
__attribute__((target("avx2"))) static float avx2_packed_q2_dot(float scale, const uint8_t *codes,
                                                                const float *input) {
    __m256 factor = _mm256_set1_ps(scale / 3.0f);
    __m256i shifts = _mm256_setr_epi32(0, 2, 4, 6, 8, 10, 12, 14);
    __m256i mask = _mm256_set1_epi32(3);
    __m256 acc = _mm256_setzero_ps();
    for (int w = 0; w < 4; w++) {
        uint32_t word;
        memcpy(&word, codes + 4 * w, 4);
        for (int half = 0; half < 2; half++) {
            __m256i v = _mm256_set1_epi32((int)(word >> (16 * half)));
            __m256i c = _mm256_and_si256(_mm256_srlv_epi32(v, shifts), mask);
            __m256i centered =
                _mm256_sub_epi32(_mm256_add_epi32(c, c), _mm256_set1_epi32(3));
            __m256 wv = _mm256_mul_ps(_mm256_cvtepi32_ps(centered), factor);
            __m256 x = _mm256_loadu_ps(input + 16 * w + 8 * half);
            acc = _mm256_add_ps(acc, _mm256_mul_ps(wv, x));
        }
    }
    return avx2_hsum(acc);
}

/* cpu.rs:623-658: (scale/15) * (2*code-15); per 8 code bytes the low nibbles
 * pair with even inputs and the high nibbles with odd inputs. */
__attribute__((target("avx2"))) static float avx2_packed_q4_dot(float scale, const uint8_t *codes,
                                                                const float *input) {
    __m256 factor = _mm256_set1_ps(scale / 15.0f);
    __m128i nibble_mask = _mm_set1_epi8(0x0f);
    __m256i offset = _mm256_set1_epi32(15);
    __m256i lane_fix = _mm256_setr_epi32(0, 1, 4, 5, 2, 3, 6, 7);
    __m256 acc = _mm256_setzero_ps();
    for (int group = 0; group < 4; group++) {
        __m128i bytes = _mm_loadl_epi64((const __m128i *)(codes + 8 * group));
        __m256i even_codes = _mm256_cvtepu8_epi32(_mm_and_si128(bytes, nibble_mask));
        __m256i odd_codes =
            _mm256_cvtepu8_epi32(_mm_and_si128(_mm_srli_epi16(bytes, 4), nibble_mask));
        __m256 lower = _mm256_loadu_ps(input + group * 16);
        __m256 upper = _mm256_loadu_ps(input + group * 16 + 8);
        __m256 even_inputs =
            _mm256_permutevar8x32_ps(_mm256_shuffle_ps(lower, upper, 0x88), lane_fix);
        __m256 odd_inputs =
            _mm256_permutevar8x32_ps(_mm256_shuffle_ps(lower, upper, 0xDD), lane_fix);
        __m256i cv[2] = {even_codes, odd_codes};
        __m256 xv[2] = {even_inputs, odd_inputs};
        for (int j = 0; j < 2; j++) {
            __m256i centered = _mm256_sub_epi32(_mm256_slli_epi32(cv[j], 1), offset);
            __m256 value = _mm256_mul_ps(_mm256_cvtepi32_ps(centered), factor);
            acc = _mm256_add_ps(acc, _mm256_mul_ps(value, xv[j]));
        }
    }
    return avx2_hsum(acc);
}

__attribute__((target("avx2"))) static int execute_rows_avx2(const orc_fused_matvec *op,
                                                             uint64_t bpr, const float *input,
                                                             uint64_t row_begin, uint64_t row_end,
                                                             float *out) {
    for (uint64_t row = row_begin; row < row_end; row++) {
        const uint8_t *bytes;
        uint32_t dtype;
        int rc = locate_row(op, bpr, row, &bytes, &dtype);
        if (rc) return rc;
        uint64_t bb = dtype == ORC_Q2B64 ? Q2_BLOCK_BYTES : Q4_BLOCK_BYTES;
        float sum = 0.0f;
        for (uint64_t b = 0; b < bpr; b++) {
            const uint8_t *block = bytes + b * bb;
            float scale = block_scale(block);
            if (!is_finite_f(scale)) return ORC_INVALID_ARTIFACT;
            sum += dtype == ORC_Q2B64
                       ? avx2_packed_q2_dot(scale, block + 2, input + b * BLOCK_LEN)
                       : avx2_packed_q4_dot(scale, block + 2, input + b * BLOCK_LEN);
        }
        rc = finish_row(op, row, sum, &out[row]);
        if (rc) return rc;
    }
    return ORC_OK;
}

int orc_fused_matvec_run_avx2(const orc_fused_matvec *op, float *out, int threads) {
    if (!__builtin_cpu_supports("avx2")) return ORC_UNSUPPORTED_OPERATION;
    return run_mt(op, out, threads, 1);
}
#else
static int execute_rows_avx2(const orc_fused_matvec *op, uint64_t bpr, const float *input,
                             uint64_t row_begin, uint64_t row_end, float *out) {
    (void)op; (void)bpr; (void)input; (void)row_begin; (void)row_end; (void)out;
    return ORC_UNSUPPORTED_OPERATION;
}
int orc_fused_matvec_run_avx2(const orc_fused_matvec *op, float *out, int threads) {
    (void)op; (void)out; (void)threads;
    return ORC_UNSUPPORTED_OPERATION;
}
#endif

/* backend/cpu.rs:373-380 */
static int same_scale_slice(const orc_fused_matvec *a, const orc_fused_matvec *b) {
    if (a->s_in_kind != b->s_in_kind) return 0;
    if (a->s_in_kind == ORC_SCALE_NONE) return 1;
    if (a->s_in_len != b->s_in_len) return 0;
    size_t bytes = a->s_in_kind == ORC_SCALE_F32 ? 4 * a->s_in_len : 2 * a->s_in_len;
    return memcmp(a->s_in, b->s_in, bytes) == 0;
}

/* backend/cpu.rs:444-472 */
int orc_fused_matvec_fanout(const orc_fused_matvec *ops, uint64_t n, float *const *outs) {
    if (n == 0) return ORC_SHAPE;
    int can_share = 1;
    for (uint64_t i = 0; i < n; i++)
        if (ops[i].input_len != ops[0].input_len || ops[i].input != ops[0].input ||
            !same_scale_slice(&ops[i], &ops[0]))
            can_share = 0;
    if (!can_share) {
        for (uint64_t i = 0; i < n; i++) {
            int rc = orc_fused_matvec_run(&ops[i], outs[i]);
            if (rc) return rc;
        }
        return ORC_OK;
    }
    uint64_t *bprs = (uint64_t *)malloc(sizeof(uint64_t) * n);
    for (uint64_t i = 0; i < n; i++) {
        int rc = validate(&ops[i], &bprs[i]);
        if (rc) {
            free(bprs);
            return rc;
        }
    }
    float *owned;
    const float *input;
    int rc = corrected_input(&ops[0], &owned, &input);
    for (uint64_t i = 0; i < n && !rc; i++)
        rc = execute_rows(&ops[i], bprs[i], input, 0, ops[i].rows, outs[i]);
    free(owned);
    free(bprs);
    return rc;
}

/* backend/cpu.rs:312-370 */
int orc_recovered_row(uint32_t dtype, const uint8_t *weights, uint64_t weights_len,
                      uint64_t columns, uint32_t s_in_kind, const void *s_in, uint64_t s_in_len,
                      float s_out, float *out) {
    if (columns == 0 || columns % BLOCK_LEN) return ORC_SHAPE;
    if (s_in_kind == ORC_SCALE_NONE || s_in_len != columns || !is_finite_f(s_out))
        return ORC_SHAPE;
    uint64_t bb;
    if (dtype == ORC_Q2B64)
        bb = Q2_BLOCK_BYTES;
    else if (dtype == ORC_Q4B64)
        bb = Q4_BLOCK_BYTES;
    else
        return ORC_UNSUPPORTED_DTYPE;
    if (weights_len != columns / BLOCK_LEN * bb) return ORC_SHAPE;
    for (uint64_t b = 0; b < columns / BLOCK_LEN; b++) {
        const uint8_t *block = weights + b * bb;
        float scale = block_scale(block);
        if (!is_finite_f(scale)) return ORC_INVALID_ARTIFACT;
        for (int lc = 0; lc < BLOCK_LEN; lc++) {
            float normalized;
            if (dtype == ORC_Q2B64) {
                normalized = Q2_CODEBOOK[(block[2 + lc / 4] >> ((lc % 4) * 2)) & 0x3u];
            } else {
                uint8_t packed = block[2 + lc / 2];
                unsigned code = (lc % 2 == 0) ? (packed & 0x0fu) : (packed >> 4);
                normalized = ((float)code - 7.5f) / 7.5f;
            }
            uint64_t column = b * BLOCK_LEN + (uint64_t)lc;
            float si;
            int rc = scale_value(s_in_kind, s_in, s_in_len, column, &si);
            if (rc) return rc;
            out[column] = scale * normalized * si * s_out;
        }
    }
    return ORC_OK;
}

/* backend/cpu.rs:478-497 */
int orc_recovered_row_matvec(uint32_t dtype, const uint8_t *weights, uint64_t weights_len,
                             const float *corrected, uint64_t columns, float s_out, float *out) {
    if (columns == 0 || columns % BLOCK_LEN || !is_finite_f(s_out)) return ORC_SHAPE;
    for (uint64_t i = 0; i < columns; i++)
        if (!is_finite_f(corrected[i])) return ORC_SHAPE;
    if (dtype != ORC_Q2B64 && dtype != ORC_Q4B64) return ORC_UNSUPPORTED_DTYPE;
    uint64_t bb = dtype == ORC_Q2B64 ? Q2_BLOCK_BYTES : Q4_BLOCK_BYTES;
    if (weights_len != columns / BLOCK_LEN * bb) return ORC_SHAPE;
    float sum;
    int rc = row_sum(dtype, weights, columns / BLOCK_LEN, corrected, &sum);
    if (rc) return rc;
    *out = sum * s_out;
    return ORC_OK;
}

/* ---- reference.rs ---- */

/* reference.rs:18-34 */
static int matrix_contract(const float *values, uint64_t n_values, uint64_t rows,
                           uint64_t columns) {
    uint64_t expected;
    if (__builtin_mul_overflow(rows, columns, &expected)) return ORC_SHAPE;
    if (rows == 0 || columns == 0 || n_values != expected) return ORC_SHAPE;
    for (uint64_t i = 0; i < n_values; i++)
        if (!is_finite_f(values[i])) return ORC_INVALID_ARTIFACT;
    return ORC_OK;
}

/* reference.rs:38-62 */
int orc_rms_norm_1p_weight(const float *values, uint64_t rows, uint64_t columns,
                           const float *weight, float epsilon, float *out) {
    int rc = matrix_contract(values, rows * columns, rows, columns);
    if (rc) return rc;
    if (!is_finite_f(epsilon) || epsilon <= 0.0f) return ORC_SHAPE;
    for (uint64_t r = 0; r < rows; r++) {
        const float *row = values + r * columns;
        float sum = 0.0f;
        for (uint64_t c = 0; c < columns; c++) sum += row[c] * row[c];
        float variance = sum / (float)columns;
        float inverse = 1.0f / sqrtf(variance + epsilon);
        for (uint64_t c = 0; c < columns; c++)
            out[r * columns + c] = row[c] * inverse * (1.0f + weight[c]);
    }
    return ORC_OK;
}

/* reference.rs:66-93 */
int orc_rms_norm_gated(const float *values, const float *gate, uint64_t rows, uint64_t columns,
                       const float *weight, float epsilon, float *out) {
    int rc = matrix_contract(values, rows * columns, rows, columns);
    if (rc) return rc;
    rc = matrix_contract(gate, rows * columns, rows, columns);
    if (rc) return rc;
    if (!is_finite_f(epsilon) || epsilon <= 0.0f) return ORC_SHAPE;
    for (uint64_t r = 0; r < rows; r++) {
        const float *row = values + r * columns;
        const float *grow = gate + r * columns;
        float sum = 0.0f;
        for (uint64_t c = 0; c < columns; c++) sum += row[c] * row[c];
        float variance = sum / (float)columns;
        float inverse = 1.0f / sqrtf(variance + epsilon);
        for (uint64_t c = 0; c < columns; c++)
            out[r * columns + c] = row[c] * inverse * weight[c] * orc_silu(grow[c]);
    }
    return ORC_OK;
}

/* reference.rs:96-110 */
int orc_swiglu(const float *gate, const float *up, uint64_t n, float *out) {
    if (n == 0) return ORC_SHAPE;
    for (uint64_t i = 0; i < n; i++)
        if (!is_finite_f(gate[i]) || !is_finite_f(up[i])) return ORC_SHAPE;
    for (uint64_t i = 0; i < n; i++) out[i] = orc_silu(gate[i]) * up[i];
    return ORC_OK;
}

/* reference.rs:115-155 */
int orc_apply_partial_rope(float *query, float *key, uint64_t query_heads, uint64_t key_heads,
                           uint64_t head_dim, uint64_t rotary_dim, uint64_t position,
                           float theta) {
    int rc = matrix_contract(query, query_heads * head_dim, query_heads, head_dim);
    if (rc) return rc;
    rc = matrix_contract(key, key_heads * head_dim, key_heads, head_dim);
    if (rc) return rc;
    if (rotary_dim == 0 || rotary_dim > head_dim || rotary_dim % 2 || !is_finite_f(theta) ||
        theta <= 0.0f)
        return ORC_SHAPE;
    uint64_t half = rotary_dim / 2;
    float *cosine = (float *)malloc(sizeof(float) * half);
    float *sine = (float *)malloc(sizeof(float) * half);
    for (uint64_t i = 0; i < half; i++) {
        float inverse_frequency = powf(theta, -((float)(2 * i)) / (float)rotary_dim);
        float angle = (float)position * inverse_frequency;
        cosine[i] = cosf(angle);
        sine[i] = sinf(angle);
    }
    float *sets[2] = {query, key};
    uint64_t heads[2] = {query_heads, key_heads};
    for (int s = 0; s < 2; s++)
        for (uint64_t h = 0; h < heads[s]; h++) {
            float *head = sets[s] + h * head_dim;
            for (uint64_t i = 0; i < half; i++) {
                float left = head[i];
                float right = head[i + half];
                head[i] = left * cosine[i] - right * sine[i];
                head[i + half] = right * cosine[i] + left * sine[i];
            }
        }
    free(cosine);
    free(sine);
    return ORC_OK;
}

/* reference.rs:159-187 */
int orc_causal_conv_silu_update(const float *input, float *state, const float *weight,
                                uint64_t channels, uint64_t kernel, float *out) {
    int rc = matrix_contract(state, channels * kernel, channels, kernel);
    if (rc) return rc;
    rc = matrix_contract(weight, channels * kernel, channels, kernel);
    if (rc) return rc;
    for (uint64_t c = 0; c < channels; c++)
        if (!is_finite_f(input[c])) return ORC_SHAPE;
    for (uint64_t c = 0; c < channels; c++) {
        float *local = state + c * kernel;
        memmove(local, local + 1, sizeof(float) * (kernel - 1));
        local[kernel - 1] = input[c];
        float sum = 0.0f;
        for (uint64_t j = 0; j < kernel; j++) sum += local[j] * weight[c * kernel + j];
        out[c] = orc_silu(sum);
    }
    return ORC_OK;
}

/* reference.rs:191-225 */
int orc_causal_conv_silu_update_f16_state(const float *input, uint16_t *state,
                                          const float *weight, uint64_t channels, uint64_t kernel,
                                          float *out) {
    int rc = matrix_contract(weight, channels * kernel, channels, kernel);
    if (rc) return rc;
    for (uint64_t c = 0; c < channels; c++)
        if (!is_finite_f(input[c])) return ORC_SHAPE;
    for (uint64_t i = 0; i < channels * kernel; i++)
        if (!is_finite_f(orc_f16_to_f32(state[i]))) return ORC_SHAPE;
    for (uint64_t c = 0; c < channels; c++) {
        uint16_t *local = state + c * kernel;
        memmove(local, local + 1, sizeof(uint16_t) * (kernel - 1));
        local[kernel - 1] = orc_f32_to_f16(input[c]);
        float sum = 0.0f;
        for (uint64_t j = 0; j < kernel; j++)
            sum += orc_f16_to_f32(local[j]) * weight[c * kernel + j];
        out[c] = orc_silu(sum);
    }
    return ORC_OK;
}

static int delta_contract(const float *query, const float *key, const float *value,
                          const float *log_decay, const float *beta, uint64_t heads,
                          uint64_t key_dim, uint64_t value_dim) {
    int rc = matrix_contract(query, heads * key_dim, heads, key_dim);
    if (rc) return rc;
    rc = matrix_contract(key, heads * key_dim, heads, key_dim);
    if (rc) return rc;
    rc = matrix_contract(value, heads * value_dim, heads, value_dim);
    if (rc) return rc;
    for (uint64_t h = 0; h < heads; h++)
        if (!is_finite_f(log_decay[h]) || !is_finite_f(beta[h])) return ORC_SHAPE;
    return ORC_OK;
}

/* reference.rs:230-297 */
int orc_recurrent_gated_delta_step(const float *query, const float *key, const float *value,
                                   const float *log_decay, const float *beta, float *state,
                                   uint64_t heads, uint64_t key_dim, uint64_t value_dim,
                                   float *out) {
    int rc = delta_contract(query, key, value, log_decay, beta, heads, key_dim, value_dim);
    if (rc) return rc;
    for (uint64_t i = 0; i < heads * key_dim * value_dim; i++)
        if (!is_finite_f(state[i])) return ORC_SHAPE;
    float query_scale = 1.0f / sqrtf((float)key_dim);
    for (uint64_t head = 0; head < heads; head++) {
        const float *q = query + head * key_dim;
        const float *k = key + head * key_dim;
        const float *v = value + head * value_dim;
        float qs = 0.0f, ks = 0.0f;
        for (uint64_t i = 0; i < key_dim; i++) qs += q[i] * q[i];
        for (uint64_t i = 0; i < key_dim; i++) ks += k[i] * k[i];
        float q_inverse = 1.0f / sqrtf(qs + 1e-6f);
        float k_inverse = 1.0f / sqrtf(ks + 1e-6f);
        float *local = state + head * key_dim * value_dim;
        float decay = expf(log_decay[head]);
        for (uint64_t i = 0; i < key_dim * value_dim; i++) local[i] *= decay;
        for (uint64_t vi = 0; vi < value_dim; vi++) {
            float memory = 0.0f;
            for (uint64_t i = 0; i < key_dim; i++)
                memory += local[i * value_dim + vi] * k[i] * k_inverse;
            float delta = (v[vi] - memory) * beta[head];
            for (uint64_t ki = 0; ki < key_dim; ki++)
                local[ki * value_dim + vi] += k[ki] * k_inverse * delta;
        }
        for (uint64_t vi = 0; vi < value_dim; vi++) {
            float acc = 0.0f;
            for (uint64_t i = 0; i < key_dim; i++)
                acc += local[i * value_dim + vi] * q[i] * q_inverse * query_scale;
            out[head * value_dim + vi] = acc;
        }
    }
    return ORC_OK;
}

/* reference.rs:302-373 */
int orc_recurrent_gated_delta_step_f16_state(const float *query, const float *key,
                                             const float *value, const float *log_decay,
                                             const float *beta, uint16_t *state, uint64_t heads,
                                             uint64_t key_dim, uint64_t value_dim, float *out) {
    int rc = delta_contract(query, key, value, log_decay, beta, heads, key_dim, value_dim);
    if (rc) return rc;
    for (uint64_t i = 0; i < heads * key_dim * value_dim; i++)
        if (!is_finite_f(orc_f16_to_f32(state[i]))) return ORC_SHAPE;
    float query_scale = 1.0f / sqrtf((float)key_dim);
    for (uint64_t head = 0; head < heads; head++) {
        const float *q = query + head * key_dim;
        const float *k = key + head * key_dim;
        const float *v = value + head * value_dim;
        float qs = 0.0f, ks = 0.0f;
        for (uint64_t i = 0; i < key_dim; i++) qs += q[i] * q[i];
        for (uint64_t i = 0; i < key_dim; i++) ks += k[i] * k[i];
        float q_inverse = 1.0f / sqrtf(qs + 1e-6f);
        float k_inverse = 1.0f / sqrtf(ks + 1e-6f);
        uint16_t *local = state + head * key_dim * value_dim;
        float decay = expf(log_decay[head]);
        for (uint64_t i = 0; i < key_dim * value_dim; i++)
            local[i] = orc_f32_to_f16(orc_f16_to_f32(local[i]) * decay);
        for (uint64_t vi = 0; vi < value_dim; vi++) {
            float memory = 0.0f;
            for (uint64_t i = 0; i < key_dim; i++)
                memory += orc_f16_to_f32(local[i * value_dim + vi]) * k[i] * k_inverse;
            float delta = (v[vi] - memory) * beta[head];
            for (uint64_t ki = 0; ki < key_dim; ki++) {
                uint64_t index = ki * value_dim + vi;
                float updated = orc_f16_to_f32(local[index]) + k[ki] * k_inverse * delta;
                local[index] = orc_f32_to_f16(updated);
            }
        }
        for (uint64_t vi = 0; vi < value_dim; vi++) {
            float acc = 0.0f;
            for (uint64_t i = 0; i < key_dim; i++)
                acc += orc_f16_to_f32(local[i * value_dim + vi]) * q[i] * q_inverse * query_scale;
            out[head * value_dim + vi] = acc;
        }
    }
    return ORC_OK;
}

/* reference.rs:377-415 */
int orc_recurrent_gated_delta_sequence(const float *query, const float *key, const float *value,
                                       const float *log_decay, const float *beta, float *state,
                                       uint64_t tokens, uint64_t heads, uint64_t key_dim,
                                       uint64_t value_dim, float *out) {
    if (tokens == 0) return ORC_SHAPE;
    uint64_t qk = heads * key_dim, vv = heads * value_dim;
    for (uint64_t t = 0; t < tokens; t++) {
        int rc = orc_recurrent_gated_delta_step(query + t * qk, key + t * qk, value + t * vv,
                                                log_decay + t * heads, beta + t * heads, state,
                                                heads, key_dim, value_dim, out + t * vv);
        if (rc) return rc;
    }
    return ORC_OK;
}

/* reference.rs:420-499 */
int orc_grouped_query_attention(const float *query, const float *key, const float *value,
                                uint64_t query_heads, uint64_t key_value_heads,
                                uint64_t query_tokens, uint64_t key_value_tokens,
                                uint64_t head_dim, uint64_t query_start_position, float *out) {
    if (query_heads == 0 || query_tokens == 0 || head_dim == 0 || key_value_tokens == 0)
        return ORC_SHAPE;
    if (key_value_heads == 0 || query_heads % key_value_heads ||
        query_start_position + query_tokens > key_value_tokens)
        return ORC_SHAPE;
    uint64_t groups = query_heads / key_value_heads;
    float scale = 1.0f / sqrtf((float)head_dim);
    float *scores = (float *)malloc(sizeof(float) * key_value_tokens);
    memset(out, 0, sizeof(float) * query_tokens * query_heads * head_dim);
    for (uint64_t token = 0; token < query_tokens; token++) {
        uint64_t available = query_start_position + token + 1;
        for (uint64_t qh = 0; qh < query_heads; qh++) {
            uint64_t kvh = qh / groups;
            const float *qrow = query + (qh * query_tokens + token) * head_dim;
            for (uint64_t kt = 0; kt < available; kt++) {
                const float *krow = key + (kvh * key_value_tokens + kt) * head_dim;
                float s = 0.0f;
                for (uint64_t d = 0; d < head_dim; d++) s += qrow[d] * krow[d];
                scores[kt] = s * scale;
            }
            float maximum = -INFINITY;
            for (uint64_t kt = 0; kt < available; kt++)
                maximum = scores[kt] > maximum ? scores[kt] : maximum;
            float denominator = 0.0f;
            for (uint64_t kt = 0; kt < available; kt++) {
                scores[kt] = expf(scores[kt] - maximum);
                denominator += scores[kt];
            }
            if (!is_finite_f(denominator) || denominator <= 0.0f) {
                free(scores);
                return ORC_INVALID_ARTIFACT;
            }
            float *orow = out + (token * query_heads + qh) * head_dim;
            for (uint64_t kt = 0; kt < available; kt++) {
                const float *vrow = value + (kvh * key_value_tokens + kt) * head_dim;
                for (uint64_t d = 0; d < head_dim; d++)
                    orow[d] += scores[kt] / denominator * vrow[d];
            }
        }
    }
    free(scores);
    return ORC_OK;
}

/* reference.rs:502-515 */
int orc_sigmoid_gate(float *values, const float *gate, uint64_t n) {
    if (n == 0) return ORC_SHAPE;
    for (uint64_t i = 0; i < n; i++)
        if (!is_finite_f(values[i]) || !is_finite_f(gate[i])) return ORC_SHAPE;
    for (uint64_t i = 0; i < n; i++) values[i] *= 1.0f / (1.0f + expf(-gate[i]));
    return ORC_OK;
}

/* decoder.rs:29-35 */
float orc_softplus(float value) { return value > 20.0f ? value : log1pf(expf(value)); }

/* decoder.rs:47-65: target head h reads source head h / (target/source). */
int orc_repeat_heads(const float *in, uint64_t source_heads, uint64_t target_heads,
                     uint64_t head_dim, float *out) {
    if (source_heads == 0 || target_heads % source_heads) return ORC_SHAPE;
    uint64_t repeat = target_heads / source_heads;
    for (uint64_t h = 0; h < target_heads; h++)
        memcpy(out + h * head_dim, in + (h / repeat) * head_dim, sizeof(float) * head_dim);
    return ORC_OK;
}

/* decoder.rs:881,897-902 */
int orc_gated_delta_prepare(const float *a, const float *b, const float *a_log,
                            const float *dt_bias, uint64_t heads, float *log_decay, float *beta) {
    for (uint64_t h = 0; h < heads; h++) {
        beta[h] = 1.0f / (1.0f + expf(-b[h]));
        log_decay[h] = -expf(a_log[h]) * orc_softplus(a[h] + dt_bias[h]);
    }
    return ORC_OK;
}

/* ---- sampler.rs ---- */

/* sampler.rs:76-82 and engine.rs:906-913: Iterator::max_by keeps the LAST
 * maximal element under f32::total_cmp. */
int orc_greedy_token(const float *logits, uint64_t n, uint32_t *token) {
    if (n == 0) return ORC_INVALID_ARTIFACT;
    uint64_t best = 0;
    int32_t best_key = total_key(logits[0]);
    for (uint64_t i = 1; i < n; i++) {
        int32_t k = total_key(logits[i]);
        if (k >= best_key) {
            best = i;
            best_key = k;
        }
    }
    *token = (uint32_t)best;
    return ORC_OK;
}

typedef struct {
    uint32_t token;
    float value;
} candidate;

/* sampler.rs:101-106: value descending, ties by token id descending. */
static int candidate_cmp(const void *a, const void *b) {
    const candidate *l = (const candidate *)a, *r = (const candidate *)b;
    int32_t lk = total_key(l->value), rk = total_key(r->value);
    if (lk != rk) return rk > lk ? 1 : -1;
    if (l->token != r->token) return r->token > l->token ? 1 : -1;
    return 0;
}

/* sampler.rs:65-144 */
int orc_sample_with_draw(const float *logits, uint64_t n, float temperature, uint64_t top_k,
                         float top_p, float draw, uint32_t *token) {
    if (n == 0) return ORC_INVALID_ARTIFACT;
    for (uint64_t i = 0; i < n; i++)
        if (!is_finite_f(logits[i])) return ORC_INVALID_ARTIFACT;
    if (!is_finite_f(draw) || !(draw >= 0.0f && draw < 1.0f)) return ORC_INVALID_ARTIFACT;
    if (!is_finite_f(temperature) || temperature < 0.0f) return ORC_INVALID_ARTIFACT;
    if (!(is_finite_f(top_p) && 0.0f < top_p && top_p <= 1.0f)) return ORC_INVALID_ARTIFACT;
    if (temperature == 0.0f) return orc_greedy_token(logits, n, token);
    float inverse_temperature = 1.0f / temperature;
    if (!is_finite_f(inverse_temperature)) return ORC_INVALID_ARTIFACT;
    candidate *c = (candidate *)malloc(sizeof(candidate) * n);
    for (uint64_t i = 0; i < n; i++) {
        c[i].token = (uint32_t)i;
        c[i].value = logits[i] * inverse_temperature;
        if (!is_finite_f(c[i].value)) {
            free(c);
            return ORC_INVALID_ARTIFACT;
        }
    }
    qsort(c, n, sizeof(candidate), candidate_cmp);
    uint64_t len = n;
    if (top_k > 0 && top_k < len) len = top_k;
    float maximum = c[0].value;
    float normalization = 0.0f;
    for (uint64_t i = 0; i < len; i++) {
        c[i].value = expf(c[i].value - maximum);
        normalization += c[i].value;
    }
    if (!is_finite_f(normalization) || normalization <= 0.0f) {
        free(c);
        return ORC_INVALID_ARTIFACT;
    }
    float cumulative = 0.0f;
    uint64_t nucleus = len;
    for (uint64_t i = 0; i < len; i++) {
        cumulative += c[i].value;
        if (cumulative >= top_p * normalization) {
            nucleus = i + 1;
            break;
        }
    }
    float nucleus_total = 0.0f;
    for (uint64_t i = 0; i < nucleus; i++) nucleus_total += c[i].value;
    float threshold = draw * nucleus_total;
    cumulative = 0.0f;
    uint32_t chosen = c[nucleus - 1].token;
    for (uint64_t i = 0; i < nucleus; i++) {
        cumulative += c[i].value;
        if (threshold <= cumulative) {
            chosen = c[i].token;
            break;
        }
    }
    free(c);
    *token = chosen;
    return ORC_OK;
}

/* sampler.rs:149-174 */
uint32_t orc_pcg32_next_u32(uint64_t *state) {
    uint64_t old = *state;
    *state = old * 6364136223846793005ull + 1442695040888963407ull;
    uint32_t shifted = (uint32_t)(((old >> 18) ^ old) >> 27);
    uint32_t rot = (uint32_t)(old >> 59);
    return (shifted >> rot) | (shifted << ((32 - rot) & 31));
}

void orc_pcg32_new(uint64_t seed, uint64_t *state) {
    *state = seed + 0x853c49e6748fea9bull;
    (void)orc_pcg32_next_u32(state);
}

float orc_pcg32_next_f32(uint64_t *state) {
    return (float)((double)orc_pcg32_next_u32(state) / ((double)UINT32_MAX + 1.0));
}

/* ---- engine.rs ---- */

/* engine.rs:923-938 (compact form) */
int orc_verify_greedy_mtp_tokens(const uint32_t *draft_tokens, const uint32_t *target_tokens,
                                 uint64_t k, uint32_t bonus_token, uint32_t *next_token,
                                 uint32_t *verified, uint32_t *accepted, uint32_t *n_accepted) {
    uint32_t v = 0, na = 0;
    for (uint64_t i = 0; i < k; i++) {
        v++;
        if (draft_tokens[i] != target_tokens[i]) {
            *next_token = target_tokens[i];
            *verified = v;
            *n_accepted = na;
            return ORC_OK;
        }
        accepted[na++] = draft_tokens[i];
    }
    *next_token = bonus_token;
    *verified = v;
    *n_accepted = na;
    return ORC_OK;
}

/* engine.rs:939-962 with DraftDistribution::greedy_token (engine.rs:203-217):
 * draft_token_ids[i] == NULL means a Full distribution. */
int orc_verify_greedy_mtp_logits(const float *const *draft_logits, const uint64_t *draft_len,
                                 const uint32_t *const *draft_token_ids,
                                 const float *const *target_logits, uint64_t vocab, uint64_t k,
                                 const float *bonus_logits, uint32_t *next_token,
                                 uint32_t *verified, uint32_t *accepted, uint32_t *n_accepted) {
    uint32_t v = 0, na = 0;
    for (uint64_t i = 0; i < k; i++) {
        uint32_t local, target;
        int rc = orc_greedy_token(draft_logits[i], draft_len[i], &local);
        if (rc) return rc;
        uint32_t draft = draft_token_ids[i] ? draft_token_ids[i][local] : local;
        rc = orc_greedy_token(target_logits[i], vocab, &target);
        if (rc) return rc;
        v++;
        if (draft != target) {
            *next_token = target;
            *verified = v;
            *n_accepted = na;
            return ORC_OK;
        }
        accepted[na++] = draft;
    }
    if (!bonus_logits) return ORC_INVALID_ARTIFACT;
    uint32_t bonus;
    int rc = orc_greedy_token(bonus_logits, vocab, &bonus);
    if (rc) return rc;
    *next_token = bonus;
    *verified = v;
    *n_accepted = na;
    return ORC_OK;
}

/* ---- Philox4x32-10 (Salmon, Moraes, Dror, Shaw: "Parallel random numbers:
 * as easy as 1, 2, 3", SC'11). No reference counterpart. ---- */
void orc_philox4x32_10(const uint32_t counter[4], const uint32_t key[2], uint32_t out[4]) {
    uint32_t c0 = counter[0], c1 = counter[1], c2 = counter[2], c3 = counter[3];
    uint32_t k0 = key[0], k1 = key[1];
    for (int round = 0; round < 10; round++) {
        uint64_t p0 = (uint64_t)0xD2511F53u * c0;
        uint64_t p1 = (uint64_t)0xCD9E8D57u * c2;
        uint32_t n0 = (uint32_t)(p1 >> 32) ^ c1 ^ k0;
        uint32_t n1 = (uint32_t)p1;
        uint32_t n2 = (uint32_t)(p0 >> 32) ^ c3 ^ k1;
        uint32_t n3 = (uint32_t)p0;
        c0 = n0; c1 = n1; c2 = n2; c3 = n3;
        k0 += 0x9E3779B9u;
        k1 += 0xBB67AE85u;
    }
    out[0] = c0; out[1] = c1; out[2] = c2; out[3] = c3;
}

/* 24 random bits -> [0, 1), exactly representable. */
float orc_u32_to_unit_f32(uint32_t bits) { return (float)(bits >> 8) * (1.0f / 16777216.0f); }

/* Natural logarithm from +, * and bit operations only, so that a device
 * implementation can reproduce it bit for bit (no libm, no contraction).
 * x = m * 2^e with m in [sqrt(1/2), sqrt(2)); ln m = 2 atanh(s), s=(m-1)/(m+1). */
static float det_ln(float x) {
    uint32_t bits;
    memcpy(&bits, &x, 4);
    int32_t e = (int32_t)(bits >> 23) - 127;
    uint32_t mb = (bits & 0x7fffffu) | 0x3f800000u;
    float m;
    memcpy(&m, &mb, 4);
    if (m > 1.41421356f) {
        m = m * 0.5f;
        e += 1;
    }
    float s = (m - 1.0f) / (m + 1.0f);
    float s2 = s * s;
    float poly = 0.11111111f;
    poly = poly * s2 + 0.14285715f;
    poly = poly * s2 + 0.2f;
    poly = poly * s2 + 0.33333334f;
    poly = poly * s2 + 1.0f;
    float ln_m = 2.0f * s * poly;
    return (float)e * 0.69314718f + ln_m;
}

/* Standard Gumbel noise -ln(-ln u) from 32 random bits; u in (0, 1). */
float orc_gumbel_from_bits(uint32_t bits) {
    float u = ((float)(bits >> 8) + 0.5f) * (1.0f / 16777216.0f);
    float inner = -det_ln(u);
    return -det_ln(inner);
}

/* Counter layout: (token or 0xffffffff, node, step lo, step hi), key = seed. */
float orc_accept_draw(uint64_t seed, uint64_t step, uint32_t node) {
    uint32_t ctr[4] = {0xffffffffu, node, (uint32_t)step, (uint32_t)(step >> 32)};
    uint32_t key[2] = {(uint32_t)seed, (uint32_t)(seed >> 32)};
    uint32_t out[4];
    orc_philox4x32_10(ctr, key, out);
    return orc_u32_to_unit_f32(out[0]);
}

float orc_gumbel_noise(uint64_t seed, uint64_t step, uint32_t node, uint32_t token) {
    /* One Philox call yields the noise of four consecutive tokens. */
    uint32_t ctr[4] = {token >> 2, node, (uint32_t)step, (uint32_t)(step >> 32)};
    uint32_t key[2] = {(uint32_t)seed, (uint32_t)(seed >> 32)};
    uint32_t out[4];
    orc_philox4x32_10(ctr, key, out);
    return orc_gumbel_from_bits(out[token & 3u]);
}

int orc_softmax_stats(const float *logits, uint64_t n, float inv_temperature, float *max_out,
                      float *sum_out) {
    if (n == 0) return ORC_SHAPE;
    float maximum = -INFINITY;
    for (uint64_t i = 0; i < n; i++) {
        float z = logits[i] * inv_temperature;
        if (!is_finite_f(z)) return ORC_INVALID_ARTIFACT;
        maximum = z > maximum ? z : maximum;
    }
    double sum = 0.0;
    for (uint64_t i = 0; i < n; i++) sum += (double)expf(logits[i] * inv_temperature - maximum);
    *max_out = maximum;
    *sum_out = (float)sum;
    return ORC_OK;
}

int orc_spec_tree_accept(const float *target_logits, uint64_t vocab, const int32_t *parent,
                         const uint32_t *node_token, uint64_t n_nodes, float temperature,
                         uint64_t seed, uint64_t step, uint32_t *emitted, uint32_t *n_emitted,
                         int32_t *path_nodes) {
    if (n_nodes == 0 || vocab == 0 || parent[0] != -1) return ORC_SHAPE;
    for (uint64_t n = 1; n < n_nodes; n++)
        if (parent[n] < 0 || (uint64_t)parent[n] >= n || node_token[n] >= vocab) return ORC_SHAPE;
    if (!is_finite_f(temperature) || temperature < 0.0f) return ORC_INVALID_ARTIFACT;
    uint32_t count = 0;
    uint64_t node = 0;
    for (;;) {
        const float *logits = target_logits + node * vocab;
        int moved = 0;
        if (temperature == 0.0f) {
            uint32_t target;
            int rc = orc_greedy_token(logits, vocab, &target);
            if (rc) return rc;
            for (uint64_t c = node + 1; c < n_nodes; c++)
                if ((uint64_t)parent[c] == node && node_token[c] == target) {
                    if (path_nodes) path_nodes[count] = (int32_t)c;
                    emitted[count++] = target;
                    node = c;
                    moved = 1;
                    break;
                }
            if (!moved) {
                emitted[count++] = target;
                *n_emitted = count;
                return ORC_OK;
            }
            continue;
        }
        float inv_t = 1.0f / temperature;
        float maximum, sum;
        int rc = orc_softmax_stats(logits, vocab, inv_t, &maximum, &sum);
        if (rc) return rc;
        float residual = 1.0f;
        for (uint64_t c = node + 1; c < n_nodes; c++) {
            if ((uint64_t)parent[c] != node) continue;
            float p = expf(logits[node_token[c]] * inv_t - maximum) / sum;
            float u = orc_accept_draw(seed, step, (uint32_t)c);
            if (u * residual < p) {
                if (path_nodes) path_nodes[count] = (int32_t)c;
                emitted[count++] = node_token[c];
                node = c;
                moved = 1;
                break;
            }
            residual -= p;
            if (residual < 0.0f) residual = 0.0f;
        }
        if (moved) continue;
        /* Gumbel-max over tokens that are not children of this node; ties keep
         * the later index, like the greedy rule. */
        uint32_t best = 0;
        int have = 0;
        float best_key = 0.0f;
        for (uint64_t t = 0; t < vocab; t++) {
            int excluded = 0;
            for (uint64_t c = node + 1; c < n_nodes; c++)
                if ((uint64_t)parent[c] == node && node_token[c] == t) excluded = 1;
            if (excluded) continue;
            float key = logits[t] * inv_t + orc_gumbel_noise(seed, step, (uint32_t)node, (uint32_t)t);
            if (!have || total_key(key) >= total_key(best_key)) {
                best = (uint32_t)t;
                best_key = key;
                have = 1;
            }
        }
        if (!have) return ORC_INVALID_ARTIFACT;
        emitted[count++] = best;
        *n_emitted = count;
        return ORC_OK;
    }
}
