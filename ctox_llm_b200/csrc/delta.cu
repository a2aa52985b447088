// Gated-delta (linear attention) recurrence over a chunk of T tokens for sm_100a.
//
// Reference semantics: recurrent_gated_delta_step / _sequence (reference.rs:230-297,377-415);
// CUDA candidate kernels/cuda/q2q4_fused_matvec_sm86.cu:937-1110, which keeps the
// state as FP16 in global memory and sweeps it twice per token with 48 CTAs.
//
// Per value head h the state S[key i][value j] (fp32, 128 x 128) evolves per token as
//   S *= exp(g);  m_j = sum_i S[i][j] k^_i;  d_j = (v_j - m_j) beta;
//   S[i][j] += k^_i d_j;  o_j = sum_i S[i][j] q^_i / sqrt(128)
// with k^ = k / sqrt(sum k^2 + 1e-6), q^ likewise. Value columns never mix, so a
// head is cut into 4 slices of 32 columns: 48 x 4 = 192 CTAs. Each CTA loads its
// 128 x 32 slice once (coalesced 128-byte rows), keeps it on chip for all T
// tokens (one column per lane, 32 key rows per warp, in registers, with the
// cross-warp sums going through shared memory) and writes it back once: the
// state crosses HBM exactly once per direction per call, whatever T is.
// state_in and state_out may differ, which is how a speculative verify pass
// leaves the committed state untouched.
#include "common.cuh"

#include <cmath>

namespace ctox {

constexpr int kDeltaDim = 128;    // key_dim == value_dim of the fast path
constexpr int kDeltaSlice = 32;   // value columns per CTA
constexpr float kL2Eps = 1e-6f;   // reference.rs:11

__global__ void __launch_bounds__(128) k_gated_delta_scan128(
    const float *__restrict__ q, const float *__restrict__ k, const float *__restrict__ v,
    const float *__restrict__ log_decay, const float *__restrict__ beta,
    const float *__restrict__ state_in, float *__restrict__ state_out, float *__restrict__ out,
    int tokens, int heads, int qk_heads) {
    pdl_launch();
    pdl_wait();
    const int head = blockIdx.x >> 2, slice = blockIdx.x & 3;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int col = slice * kDeltaSlice + lane;
    const int src = head / (heads / qk_heads);  // repeat_heads: decoder.rs:47-65
    __shared__ float qs[kDeltaDim], ks[kDeltaDim];
    __shared__ float red[2][4][kDeltaSlice];
    __shared__ float norms[2];

    float s[32];
    const float *sin_ = state_in + ((size_t)head * kDeltaDim + warp * 32) * kDeltaDim + col;
#pragma unroll
    for (int i = 0; i < 32; ++i) s[i] = sin_[(size_t)i * kDeltaDim];

    const float query_scale = 1.0f / sqrtf((float)kDeltaDim);
    for (int tok = 0; tok < tokens; ++tok) {
        const float *qt = q + ((size_t)tok * qk_heads + src) * kDeltaDim;
        const float *kt = k + ((size_t)tok * qk_heads + src) * kDeltaDim;
        const float qv = qt[threadIdx.x], kv = kt[threadIdx.x];
        qs[threadIdx.x] = qv;
        ks[threadIdx.x] = kv;
        float q2 = qv * qv, k2 = kv * kv;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            q2 += __shfl_xor_sync(0xffffffffu, q2, o);
            k2 += __shfl_xor_sync(0xffffffffu, k2, o);
        }
        if (lane == 0) {
            red[0][warp][0] = q2;
            red[0][warp][1] = k2;
        }
        __syncthreads();
        if (threadIdx.x == 0) {
            const float sq = red[0][0][0] + red[0][1][0] + red[0][2][0] + red[0][3][0];
            const float sk = red[0][0][1] + red[0][1][1] + red[0][2][1] + red[0][3][1];
            norms[0] = 1.0f / sqrtf(sq + kL2Eps);
            norms[1] = 1.0f / sqrtf(sk + kL2Eps);
        }
        __syncthreads();
        const float q_inv = norms[0], k_inv = norms[1];
        const float decay = expf(log_decay[(size_t)tok * heads + head]);
        const float b = beta[(size_t)tok * heads + head];
        const float vj = v[((size_t)tok * heads + head) * kDeltaDim + col];
        float mem = 0.f;
#pragma unroll
        for (int i = 0; i < 32; ++i) {
            s[i] *= decay;
            mem += s[i] * ks[warp * 32 + i] * k_inv;
        }
        red[1][warp][lane] = mem;
        __syncthreads();
        const float delta = (vj - (red[1][0][lane] + red[1][1][lane] + red[1][2][lane] + red[1][3][lane])) * b;
        float o = 0.f;
#pragma unroll
        for (int i = 0; i < 32; ++i) {
            s[i] += ks[warp * 32 + i] * k_inv * delta;
            o += s[i] * qs[warp * 32 + i] * q_inv * query_scale;
        }
        red[0][warp][lane] = o;
        __syncthreads();
        if (warp == 0)
            out[((size_t)tok * heads + head) * kDeltaDim + col] =
                red[0][0][lane] + red[0][1][lane] + red[0][2][lane] + red[0][3][lane];
        // red[0] is rewritten by the next token's norm partials only after the
        // barrier that follows the qs/ks stores, which every warp reaches after this read
        __syncthreads();
    }
    float *sout = state_out + ((size_t)head * kDeltaDim + warp * 32) * kDeltaDim + col;
#pragma unroll
    for (int i = 0; i < 32; ++i) sout[(size_t)i * kDeltaDim] = s[i];
}

// Any head geometry: one thread per (head, value column), the reference's loop order.
__global__ void k_gated_delta_scan_generic(const float *__restrict__ q, const float *__restrict__ k,
                                           const float *__restrict__ v, const float *__restrict__ log_decay,
                                           const float *__restrict__ beta, const float *__restrict__ state_in,
                                           float *__restrict__ state_out, float *__restrict__ out, int tokens,
                                           int heads, int qk_heads, int key_dim, int value_dim) {
    pdl_launch();
    pdl_wait();
    const int idx = blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= heads * value_dim) return;
    const int head = idx / value_dim, col = idx % value_dim;
    const int src = head / (heads / qk_heads);
    const float *si = state_in + (size_t)head * key_dim * value_dim + col;
    float *so = state_out + (size_t)head * key_dim * value_dim + col;
    if (si != so)
        for (int i = 0; i < key_dim; ++i) so[(size_t)i * value_dim] = si[(size_t)i * value_dim];
    const float query_scale = 1.0f / sqrtf((float)key_dim);
    for (int tok = 0; tok < tokens; ++tok) {
        const float *qt = q + ((size_t)tok * qk_heads + src) * key_dim;
        const float *kt = k + ((size_t)tok * qk_heads + src) * key_dim;
        float q2 = 0.f, k2 = 0.f;
        for (int i = 0; i < key_dim; ++i) {
            q2 += qt[i] * qt[i];
            k2 += kt[i] * kt[i];
        }
        const float q_inv = 1.0f / sqrtf(q2 + kL2Eps), k_inv = 1.0f / sqrtf(k2 + kL2Eps);
        const float decay = expf(log_decay[(size_t)tok * heads + head]);
        float mem = 0.f;
        for (int i = 0; i < key_dim; ++i) {
            const float sv = so[(size_t)i * value_dim] * decay;
            so[(size_t)i * value_dim] = sv;
            mem += sv * kt[i] * k_inv;
        }
        const float delta = (v[((size_t)tok * heads + head) * value_dim + col] - mem) *
                            beta[(size_t)tok * heads + head];
        float o = 0.f;
        for (int i = 0; i < key_dim; ++i) {
            const float sv = so[(size_t)i * value_dim] + kt[i] * k_inv * delta;
            so[(size_t)i * value_dim] = sv;
            o += sv * qt[i] * q_inv * query_scale;
        }
        out[((size_t)tok * heads + head) * value_dim + col] = o;
    }
}

// beta = sigmoid(b), log_decay = -exp(A_log) * softplus(a + dt_bias) (decoder.rs:29-35,881,897-902;
// CUDA candidate kernels/cuda/q2q4_fused_matvec_sm86.cu:837-926).
__global__ void k_gated_delta_prepare(const float *__restrict__ a, const float *__restrict__ b,
                                      const float *__restrict__ a_log, const float *__restrict__ dt_bias,
                                      float *__restrict__ log_decay, float *__restrict__ beta, int tokens,
                                      int heads) {
    pdl_launch();
    pdl_wait();
    const int idx = blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= tokens * heads) return;
    const int h = idx % heads;
    beta[idx] = 1.0f / (1.0f + expf(-b[idx]));
    const float x = a[idx] + dt_bias[h];
    const float sp = x > 20.0f ? x : log1pf(expf(x));
    log_decay[idx] = -expf(a_log[h]) * sp;
}

}  // namespace ctox

using namespace ctox;

extern "C" {

ctox_status ctox_gated_delta_scan(ctox_ctx *ctx, const float *q, const float *k, const float *v,
                                  const float *log_decay, const float *beta, const float *state_in,
                                  float *state_out, float *out, uint32_t tokens, uint32_t heads,
                                  uint32_t qk_heads, uint32_t key_dim, uint32_t value_dim) {
    if (!ctx) return CTOX_INVALID_STATE;
    if (!q || !k || !v || !log_decay || !beta || !state_in || !state_out || !out)
        return fail(ctx, CTOX_SHAPE, "gated delta: null device pointer");
    if (tokens == 0 || heads == 0 || key_dim == 0 || value_dim == 0 || qk_heads == 0 || heads % qk_heads)
        return fail(ctx, CTOX_SHAPE, "gated delta: tokens %u heads %u qk_heads %u key_dim %u value_dim %u",
                    tokens, heads, qk_heads, key_dim, value_dim);
    CTOX_CUDA(ctx, cudaSetDevice(ctx->device));
    if (key_dim == kDeltaDim && value_dim == kDeltaDim) {
        launch_pdl(k_gated_delta_scan128, dim3(heads * 4), dim3(128), 0, ctx->stream, q, k, v, log_decay, beta, state_in, state_out,
                                                                 out, (int)tokens, (int)heads, (int)qk_heads);
    } else {
        const unsigned n = heads * value_dim;
        launch_pdl(k_gated_delta_scan_generic, dim3((n + 127) / 128), dim3(128), 0, ctx->stream, 
            q, k, v, log_decay, beta, state_in, state_out, out, (int)tokens, (int)heads, (int)qk_heads,
            (int)key_dim, (int)value_dim);
    }
    CTOX_CUDA(ctx, cudaGetLastError());
    return CTOX_OK;
}

ctox_status ctox_gated_delta_prepare(ctox_ctx *ctx, const float *a, const float *b, const float *a_log,
                                     const float *dt_bias, float *log_decay, float *beta, uint32_t tokens,
                                     uint32_t heads) {
    if (!ctx) return CTOX_INVALID_STATE;
    if (!a || !b || !a_log || !dt_bias || !log_decay || !beta || tokens == 0 || heads == 0)
        return fail(ctx, CTOX_SHAPE, "gated delta prepare: bad arguments");
    CTOX_CUDA(ctx, cudaSetDevice(ctx->device));
    const unsigned n = tokens * heads;
    launch_pdl(k_gated_delta_prepare, dim3((n + 127) / 128), dim3(128), 0, ctx->stream, a, b, a_log, dt_bias, log_decay, beta,
                                                                   (int)tokens, (int)heads);
    CTOX_CUDA(ctx, cudaGetLastError());
    return CTOX_OK;
}

}  // extern "C"
