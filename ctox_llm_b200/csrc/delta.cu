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
#include "layers.cuh"

#include <cuda_fp16.h>

#include <cmath>

namespace ctox {

constexpr int kDeltaDim = 128;    // key_dim == value_dim of the fast path
constexpr int kDeltaSlice = 32;   // value columns per CTA
constexpr float kL2Eps = 1e-6f;   // reference.rs:11

// State element types: fp32, or FP16-resident (reference.rs:299-373: dot products and update
// arithmetic stay fp32, every persistent state element is rounded to binary16 when it is written,
// i.e. after the decay and after the delta update of every token).
template <typename S>
__device__ __forceinline__ float state_load(const S *p);
template <>
__device__ __forceinline__ float state_load<float>(const float *p) { return *p; }
template <>
__device__ __forceinline__ float state_load<__half>(const __half *p) { return __half2float(*p); }
template <typename S>
__device__ __forceinline__ float state_round(float v);
template <>
__device__ __forceinline__ float state_round<float>(float v) { return v; }
template <>
__device__ __forceinline__ float state_round<__half>(float v) { return __half2float(__float2half_rn(v)); }
template <typename S>
__device__ __forceinline__ void state_store(S *p, float v);
template <>
__device__ __forceinline__ void state_store<float>(float *p, float v) { *p = v; }
template <>
__device__ __forceinline__ void state_store<__half>(__half *p, float v) { *p = __float2half_rn(v); }

// The scan of one (head, 32-column slice) by one CTA of 128 threads; out may be null (state only).
// kWaitAfterState: the dependency wait comes after the state loads (for a caller whose state_in
// nothing in flight can write; the inputs of the tokens are read after the wait).
template <typename S, bool kWaitAfterState = false>
__device__ __forceinline__ void delta_scan128_body(
    const float *__restrict__ q, const float *__restrict__ k, const float *__restrict__ v,
    const float *__restrict__ log_decay, const float *__restrict__ beta,
    const S *__restrict__ state_in, S *__restrict__ state_out, float *__restrict__ out,
    int tokens, int heads, int qk_heads, int head, int slice) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int col = slice * kDeltaSlice + lane;
    const int src = head / (heads / qk_heads);  // repeat_heads: decoder.rs:47-65
    __shared__ float qs[kDeltaDim], ks[kDeltaDim];
    __shared__ float red[2][4][kDeltaSlice];

    float s[32];
    const S *sin_ = state_in + ((size_t)head * kDeltaDim + warp * 32) * kDeltaDim + col;
#pragma unroll
    for (int i = 0; i < 32; ++i) s[i] = state_load<S>(sin_ + (size_t)i * kDeltaDim);
    if (kWaitAfterState) pdl_wait();

    const float query_scale = 1.0f / sqrtf((float)kDeltaDim);
    for (int tok = 0; tok < tokens; ++tok) {
        const float *qt = q + ((size_t)tok * qk_heads + src) * kDeltaDim;
        const float *kt = k + ((size_t)tok * qk_heads + src) * kDeltaDim;
        const float qv = qt[threadIdx.x], kv = kt[threadIdx.x];
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
        const float q_inv = 1.0f / sqrtf(red[0][0][0] + red[0][1][0] + red[0][2][0] + red[0][3][0] + kL2Eps);
        const float k_inv = 1.0f / sqrtf(red[0][0][1] + red[0][1][1] + red[0][2][1] + red[0][3][1] + kL2Eps);
        ks[threadIdx.x] = kv * k_inv;
        qs[threadIdx.x] = qv * q_inv * query_scale;
        const float decay = expf(log_decay[(size_t)tok * heads + head]);
        const float b = beta[(size_t)tok * heads + head];
        const float vj = v[((size_t)tok * heads + head) * kDeltaDim + col];
        __syncthreads();
        float mem = 0.f;
#pragma unroll
        for (int i = 0; i < 32; ++i) {
            s[i] = state_round<S>(s[i] * decay);
            mem += s[i] * ks[warp * 32 + i];
        }
        red[1][warp][lane] = mem;
        __syncthreads();
        const float delta = (vj - (red[1][0][lane] + red[1][1][lane] + red[1][2][lane] + red[1][3][lane])) * b;
        float o = 0.f;
#pragma unroll
        for (int i = 0; i < 32; ++i) {
            s[i] = state_round<S>(s[i] + ks[warp * 32 + i] * delta);
            o += s[i] * qs[warp * 32 + i];
        }
        red[0][warp][lane] = o;
        __syncthreads();
        if (warp == 0 && out)
            out[((size_t)tok * heads + head) * kDeltaDim + col] =
                red[0][0][lane] + red[0][1][lane] + red[0][2][lane] + red[0][3][lane];
        // red[0] is rewritten by the next token's norm partials only after the
        // barrier that follows the qs/ks stores, which every warp reaches after this read
        __syncthreads();
    }
    S *sout = state_out + ((size_t)head * kDeltaDim + warp * 32) * kDeltaDim + col;
#pragma unroll
    for (int i = 0; i < 32; ++i) state_store<S>(sout + (size_t)i * kDeltaDim, s[i]);
}

template <typename S>
__global__ void __launch_bounds__(128) k_gated_delta_scan128(
    const float *__restrict__ q, const float *__restrict__ k, const float *__restrict__ v,
    const float *__restrict__ log_decay, const float *__restrict__ beta,
    const S *__restrict__ state_in, S *__restrict__ state_out, float *__restrict__ out,
    int tokens, int heads, int qk_heads) {
    pdl_launch();
    pdl_wait();
    delta_scan128_body<S>(q, k, v, log_decay, beta, state_in, state_out, out, tokens, heads, qk_heads,
                          blockIdx.x >> 2, blockIdx.x & 3);
}

// The scan of `layers` independent layers in one launch (blockIdx.y = layer): every array holds the
// layers back to back in the layout of the single-layer scan.
__global__ void __launch_bounds__(128) k_gated_delta_scan128_layers(
    const float *__restrict__ q, const float *__restrict__ k, const float *__restrict__ v,
    const float *__restrict__ log_decay, const float *__restrict__ beta, const float *__restrict__ state_in,
    float *__restrict__ state_out, float *__restrict__ out, int tokens, int heads, int qk_heads) {
    pdl_launch();
    pdl_wait();
    const size_t l = blockIdx.y;
    const size_t qk_n = (size_t)tokens * qk_heads * kDeltaDim, v_n = (size_t)tokens * heads * kDeltaDim;
    const size_t g_n = (size_t)tokens * heads, s_n = (size_t)heads * kDeltaDim * kDeltaDim;
    delta_scan128_body<float>(q + l * qk_n, k + l * qk_n, v + l * v_n, log_decay + l * g_n, beta + l * g_n,
                              state_in + l * s_n, state_out + l * s_n, out ? out + l * v_n : nullptr, tokens, heads,
                              qk_heads, blockIdx.x >> 2, blockIdx.x & 3);
}

// Commit of the first n positions of a pass for ALL linear-attention layers in one launch:
// blockIdx.y = layer; the first heads * 4 CTAs of a layer re-scan the recurrence from the committed
// state over the kept (q, k, v, g, beta) when only a prefix was accepted, the others shift the first
// n kept conv inputs into the conv state. `cur` says which state buffer of a layer is committed.
__global__ void __launch_bounds__(128) k_commit_batch(const CommitLayer *__restrict__ layers, CommitCur cur, int n,
                                                    int rescan, int heads, int qk_heads, uint32_t channels,
                                                    uint32_t conv_kernel) {
    pdl_launch();
    // The layer table and the committed buffers do not change while a pass is in flight (the state a
    // re-scan starts from was written by the commit before): pointers and state before the wait.
    const CommitLayer *L = layers + blockIdx.y;
    const int scan_ctas = heads * 4;
    if ((int)blockIdx.x < scan_ctas) {
        if (!rescan) return;
        const int c = (int)(((blockIdx.y < 64 ? cur.lo : cur.hi) >> (blockIdx.y & 63)) & 1);
        const float *sin_ = c ? L->state[1] : L->state[0];
        float *sout = c ? L->state[0] : L->state[1];
        delta_scan128_body<float, true>(L->q, L->k, L->v, L->g, L->beta, sin_, sout, nullptr, n, heads, qk_heads,
                                        blockIdx.x >> 2, blockIdx.x & 3);
        return;
    }
    const uint32_t r = (blockIdx.x - scan_ctas) * blockDim.x + threadIdx.x;
    float *cs = L->conv_state;
    const float *ci = L->conv_in;
    // taps in registers for any kernel width <= 8 (loops fully unrolled with predicates)
    float st[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) st[j] = (r < channels && (uint32_t)j < conv_kernel) ? cs[(size_t)r * conv_kernel + j] : 0.f;
    pdl_wait();
    if (r >= channels) return;
    for (int m = 0; m < n; ++m) {
        const float x = ci[(size_t)m * channels + r];
#pragma unroll
        for (int j = 0; j < 7; ++j)
            if ((uint32_t)j + 1 < conv_kernel) st[j] = st[j + 1];
#pragma unroll
        for (int j = 0; j < 8; ++j)
            if ((uint32_t)j + 1 == conv_kernel) st[j] = x;
    }
#pragma unroll
    for (int j = 0; j < 8; ++j)
        if ((uint32_t)j < conv_kernel) cs[(size_t)r * conv_kernel + j] = st[j];
}

void launch_commit_batch(cudaStream_t st, const CommitLayer *layers_dev, const CommitCur &cur, uint32_t n_layers,
                         uint32_t n, bool rescan, uint32_t heads, uint32_t qk_heads, uint32_t channels,
                         uint32_t conv_kernel) {
    const uint32_t conv_ctas = (channels + 127) / 128;
    launch_pdl(k_commit_batch, dim3(heads * 4 + conv_ctas, n_layers), dim3(128), 0, st, layers_dev, cur, (int)n,
               rescan ? 1 : 0, (int)heads, (int)qk_heads, channels, conv_kernel);
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


// ------------------------------------------------------------------ one kernel per linear-attention layer
// Everything between the fused input projection and out_proj of a linear-attention layer
// (decoder.rs:806-938) for one value head per CTA, 512 threads:
//   1. causal conv + SiLU (reference.rs:159-187) over the head's 128 q, 128 k and 128 v channels for
//      the m positions, the head's z, and decay / beta from a, b (decoder.rs:29-35,881,897-902);
//   2. the recurrence above, four 32-column slices side by side (warp = slice * 4 + row group), with
//      exactly the arithmetic and the order of k_gated_delta_scan128, so that a later re-scan of an
//      accepted prefix from the kept (q, k, v, g, beta) reproduces this pass bit for bit;
//   3. rms_norm_gated (reference.rs:66-93) and the two 64-column fragments of out_proj's input.
// The q and k channels are shared by the value heads of a key head; the first of them stores them.
constexpr int kLaMaxPos = 8;

__global__ void __launch_bounds__(512, 1) k_linear_attention(LinearAttnArgs a, int npos) {
    pdl_launch();
    __shared__ float qs[kLaMaxPos][kDeltaDim], ks[kLaMaxPos][kDeltaDim], vs[kLaMaxPos][kDeltaDim];
    __shared__ float zs[kLaMaxPos][kDeltaDim];
    __shared__ float gs[kLaMaxPos], bs[kLaMaxPos];
    __shared__ float nred[kLaMaxPos][2][4];
    __shared__ float redm[2][4][4][kDeltaSlice];
    __shared__ float redo[kLaMaxPos][4][4][kDeltaSlice];
    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t head = blockIdx.x, rep = a.value_heads / a.qk_heads, khead = head / rep;
    const bool owns_qk = head % rep == 0;
    const uint32_t channels = 2 * a.key_width + a.value_width;

    // Before the dependency wait: what the pass itself does not write. The committed recurrent
    // state and conv state were last written by the commit of the previous block, which a host
    // copy separates from this pass; the weights never change. These loads overlap the tail of
    // the input projection.
    const uint32_t slice = warp >> 2, rg = warp & 3, col = slice * kDeltaSlice + lane;
    float s[32];  // rows rg * 32 .. + 32 of column slice * 32 + lane
    {
        const float *sin_ = a.state_in + ((size_t)head * kDeltaDim + rg * 32) * kDeltaDim + col;
#pragma unroll
        for (int i = 0; i < 32; ++i) s[i] = sin_[(size_t)i * kDeltaDim];
    }
    const uint32_t part = tid >> 7, cd = tid & 127;
    const uint32_t ch = part == 0 ? khead * kDeltaDim + cd
                        : part == 1 ? a.key_width + khead * kDeltaDim + cd
                                    : 2 * a.key_width + head * kDeltaDim + cd;
    // taps in registers for any kernel width <= 8: every loop over them is fully unrolled with
    // predicates (a run-time trip count would put the arrays on the local-memory stack)
    const uint32_t K = a.conv_kernel;
    float st[8], cw[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        st[j] = cw[j] = 0.f;
        if (tid < 384 && (uint32_t)j < K) {
            st[j] = a.conv_state[(size_t)ch * K + j];
            cw[j] = a.conv_w[(size_t)ch * K + j];
        }
    }
    // One row of the input projection per thread: conv threads their channel, the last 128 their
    // gate column. Where the projection left stream-K pieces (at most eight per value), their
    // offsets are the same for every position: they are formed once, and the pieces of position
    // m + 1 are in flight while position m is worked on. Same additions in the same order as out_of.
    const uint32_t row = tid < 384 ? ch : channels + head * kDeltaDim + (tid - 384);
    const MvOut &o = a.fan;
    uint32_t total = 0, off[8];
    const float *first = nullptr;
    if (!o.plain && o.warps_per_slice) {
        const uint32_t n = piece_count(row >> 5, o.kst_s, o.warps_per_slice, o.pairs);
        total = o.slices * n;
        first = o.partial + (size_t)(row >> 5) * o.slices * o.max_pieces * 256 + (row & 31);
        uint32_t sl = 0, q = 0;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            off[j] = (sl * o.max_pieces + q) * 256;
            if (++q == n) {
                q = 0;
                ++sl;
            }
        }
    }
    const bool pieces = total >= 1 && total <= 8;  // otherwise the general fetch per position
    const float so = pieces && o.s_out ? o.s_out[row] : 1.0f;
    pdl_wait();

    // ---- 1. conv + SiLU, z, decay, beta
    {
        float buf[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) buf[j] = (pieces && (uint32_t)j < total) ? first[off[j]] : 0.f;
        const bool store = part == 2 || owns_qk;
        for (int m = 0; m < npos; ++m) {
            float x = 0.f;
            if (pieces) {
#pragma unroll
                for (int j = 0; j < 8; ++j)
                    if ((uint32_t)j < total) x += buf[j];
                if (o.s_out) x *= so;
                if (m + 1 < npos) {
#pragma unroll
                    for (int j = 0; j < 8; ++j) buf[j] = (uint32_t)j < total ? first[off[j] + (m + 1) * 32] : 0.f;
                }
            } else {
                x = out_of(o, row, m);
            }
            if (tid < 384) {
                const uint32_t d = cd;
                if (store) a.conv_in[(size_t)m * channels + ch] = x;
#pragma unroll
                for (int j = 0; j < 7; ++j)
                    if ((uint32_t)j + 1 < K) st[j] = st[j + 1];
#pragma unroll
                for (int j = 0; j < 8; ++j)
                    if ((uint32_t)j + 1 == K) st[j] = x;
                float sum = 0.f;
#pragma unroll
                for (int j = 0; j < 8; ++j)
                    if ((uint32_t)j < K) sum += st[j] * cw[j];
                const float y = silu_f(sum);
                if (part == 0) {
                    qs[m][d] = y;
                    if (store) a.q[(size_t)m * a.key_width + khead * kDeltaDim + d] = y;
                } else if (part == 1) {
                    ks[m][d] = y;
                    if (store) a.k[(size_t)m * a.key_width + khead * kDeltaDim + d] = y;
                } else {
                    vs[m][d] = y;
                    a.v[(size_t)m * a.value_width + head * kDeltaDim + d] = y;
                }
            } else {
                zs[m][tid - 384] = x;
            }
        }
        if (tid >= 384) {
            const uint32_t d = tid - 384;
            if (d < (uint32_t)npos) {
                const float x = out_of(a.fan, channels + a.value_width + head, d) + a.dt_bias[head];
                const float sp = x > 20.0f ? x : log1pf(expf(x));  // decoder.rs:29-35
                const float g = -expf(a.a_log[head]) * sp;
                gs[d] = g;
                a.log_decay[(size_t)d * a.value_heads + head] = g;
            } else if (d >= 32 && d < 32 + (uint32_t)npos) {
                const uint32_t m = d - 32;
                const float b = 1.0f / (1.0f + expf(-out_of(a.fan, channels + a.value_width + a.value_heads + head, m)));
                bs[m] = b;
                a.beta[(size_t)m * a.value_heads + head] = b;
            }
        }
    }
    __syncthreads();
    // L2 norms of q and k for all positions at once, with the reduction tree of the stand-alone scan
    // (value d in lane d % 32 of warp d / 32, butterfly, then the four warp sums in order); then the
    // normalised key and the scaled query replace q and k in shared memory, as in the scan
    if (warp < 8) {
        for (int m = 0; m < npos; ++m) {
            const float x = warp < 4 ? qs[m][warp * 32 + lane] : ks[m][(warp - 4) * 32 + lane];
            float x2 = x * x;
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) x2 += __shfl_xor_sync(0xffffffffu, x2, o);
            if (lane == 0) nred[m][warp >> 2][warp & 3] = x2;
        }
    }
    __syncthreads();
    const float query_scale = 1.0f / sqrtf((float)kDeltaDim);
    if (tid < 256) {  // thread d < 128: q element d of every position; 128..255: k element d - 128
        const uint32_t d = tid & 127;
        for (int m = 0; m < npos; ++m) {
            if (tid < 128) {
                const float qi = 1.0f / sqrtf(nred[m][0][0] + nred[m][0][1] + nred[m][0][2] + nred[m][0][3] + kL2Eps);
                qs[m][d] = qs[m][d] * qi * query_scale;
            } else {
                const float ki = 1.0f / sqrtf(nred[m][1][0] + nred[m][1][1] + nred[m][1][2] + nred[m][1][3] + kL2Eps);
                ks[m][d] = ks[m][d] * ki;
            }
        }
    }
    __syncthreads();

    // ---- 2. recurrence: one barrier per position (redm double-buffered by parity, the output
    // partial sums kept per position and added up in phase 3)
    for (int m = 0; m < npos; ++m) {
        const float decay = expf(gs[m]), b = bs[m], vj = vs[m][col];
        float mem = 0.f;
#pragma unroll
        for (int i = 0; i < 32; ++i) {
            s[i] *= decay;
            mem += s[i] * ks[m][rg * 32 + i];
        }
        redm[m & 1][slice][rg][lane] = mem;
        __syncthreads();
        const float delta = (vj - (redm[m & 1][slice][0][lane] + redm[m & 1][slice][1][lane] +
                                   redm[m & 1][slice][2][lane] + redm[m & 1][slice][3][lane])) * b;
        float o = 0.f;
#pragma unroll
        for (int i = 0; i < 32; ++i) {
            s[i] += ks[m][rg * 32 + i] * delta;
            o += s[i] * qs[m][rg * 32 + i];
        }
        redo[m][slice][rg][lane] = o;
    }
    __syncthreads();
    {
        float *sout = a.state_out + ((size_t)head * kDeltaDim + rg * 32) * kDeltaDim + col;
#pragma unroll
        for (int i = 0; i < 32; ++i) sout[(size_t)i * kDeltaDim] = s[i];
    }

    // ---- 3. gated norm and fragments: warp m takes position m, four values per lane
    if (warp < (uint32_t)npos) {
        const int m = warp;
        // columns lane * 4 .. + 3 lie in slice lane / 8; the four row groups in order
        float4 c = *reinterpret_cast<const float4 *>(&redo[m][lane >> 3][0][(lane & 7) * 4]);
#pragma unroll
        for (int r = 1; r < 4; ++r) {
            const float4 t = *reinterpret_cast<const float4 *>(&redo[m][lane >> 3][r][(lane & 7) * 4]);
            c.x += t.x;
            c.y += t.y;
            c.z += t.z;
            c.w += t.w;
        }
        const float4 g = *reinterpret_cast<const float4 *>(&zs[m][lane * 4]);
        float sq = c.x * c.x + c.y * c.y + c.z * c.z + c.w * c.w;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
        const float inv = 1.0f / sqrtf(sq / 128.0f + a.eps);
        const uint32_t ocol = head * kDeltaDim + lane * 4;
        const float cs[4] = {c.x, c.y, c.z, c.w}, gz[4] = {g.x, g.y, g.z, g.w};
        float v[4];
#pragma unroll
        for (int j = 0; j < 4; ++j)
            v[j] = cs[j] * inv * a.norm_w[lane * 4 + j] * silu_f(gz[j]) * (a.next.s_in ? a.next.s_in[ocol + j] : 1.0f);
        const unsigned gmask = (lane & 16) ? 0xffff0000u : 0x0000ffffu;
        prep_block(v, lane & 15, gmask, (int)(head * 2 + (lane >> 4)), m, npos, a.next.dt, a.next.xfrag, a.next.meta);
    }
}

void launch_linear_attention(cudaStream_t st, const LinearAttnArgs &a, uint32_t m) {
    launch_pdl(k_linear_attention, dim3(a.value_heads), dim3(512), 0, st, a, (int)m);
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
        launch_pdl(k_gated_delta_scan128<float>, dim3(heads * 4), dim3(128), 0, ctx->stream, q, k, v, log_decay, beta,
                   state_in, state_out, out, (int)tokens, (int)heads, (int)qk_heads);
    } else {
        const unsigned n = heads * value_dim;
        launch_pdl(k_gated_delta_scan_generic, dim3((n + 127) / 128), dim3(128), 0, ctx->stream, 
            q, k, v, log_decay, beta, state_in, state_out, out, (int)tokens, (int)heads, (int)qk_heads,
            (int)key_dim, (int)value_dim);
    }
    CTOX_CUDA(ctx, cudaGetLastError());
    return CTOX_OK;
}

ctox_status ctox_gated_delta_scan_layers(ctox_ctx *ctx, const float *q, const float *k, const float *v,
                                         const float *log_decay, const float *beta, const float *state_in,
                                         float *state_out, float *out, uint32_t layers, uint32_t tokens,
                                         uint32_t heads, uint32_t qk_heads) {
    if (!ctx) return CTOX_INVALID_STATE;
    if (!q || !k || !v || !log_decay || !beta || !state_in || !state_out)
        return fail(ctx, CTOX_SHAPE, "gated delta (layers): null device pointer");
    if (layers == 0 || layers > 65535 || tokens == 0 || heads == 0 || qk_heads == 0 || heads % qk_heads)
        return fail(ctx, CTOX_SHAPE, "gated delta (layers): layers %u tokens %u heads %u qk_heads %u", layers, tokens,
                    heads, qk_heads);
    CTOX_CUDA(ctx, cudaSetDevice(ctx->device));
    launch_pdl(k_gated_delta_scan128_layers, dim3(heads * 4, layers), dim3(128), 0, ctx->stream, q, k, v, log_decay,
               beta, state_in, state_out, out, (int)tokens, (int)heads, (int)qk_heads);
    CTOX_CUDA(ctx, cudaGetLastError());
    return CTOX_OK;
}

ctox_status ctox_gated_delta_scan_f16_state(ctox_ctx *ctx, const float *q, const float *k, const float *v,
                                            const float *log_decay, const float *beta, const void *state_in,
                                            void *state_out, float *out, uint32_t tokens, uint32_t heads,
                                            uint32_t qk_heads, uint32_t key_dim, uint32_t value_dim) {
    if (!ctx) return CTOX_INVALID_STATE;
    if (!q || !k || !v || !log_decay || !beta || !state_in || !state_out || !out)
        return fail(ctx, CTOX_SHAPE, "gated delta (f16 state): null device pointer");
    if (tokens == 0 || heads == 0 || qk_heads == 0 || heads % qk_heads)
        return fail(ctx, CTOX_SHAPE, "gated delta (f16 state): tokens %u heads %u qk_heads %u", tokens, heads, qk_heads);
    if (key_dim != kDeltaDim || value_dim != kDeltaDim)
        return fail(ctx, CTOX_UNSUPPORTED_OPERATION, "gated delta (f16 state): only 128 x 128 heads, got %u x %u", key_dim,
                    value_dim);
    CTOX_CUDA(ctx, cudaSetDevice(ctx->device));
    launch_pdl(k_gated_delta_scan128<__half>, dim3(heads * 4), dim3(128), 0, ctx->stream, q, k, v, log_decay, beta,
               (const __half *)state_in, (__half *)state_out, out, (int)tokens, (int)heads, (int)qk_heads);
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
