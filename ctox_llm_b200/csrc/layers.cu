// Element-wise and attention kernels of the decode executor.
//
// Reference semantics: the scalar operators of reference.rs composed in the order of
// decoder.rs (ArtifactDecoder::{decoder_mlp_residual :636-670, full_attention_residual_at
// :687-800, linear_attention_residual :806-938, mtp_final_hidden :1009-1046}). Each kernel
// consumes the raw partial sums of the preceding streamed matvec and emits the activation
// fragments of the next one, so a matvec output never makes a round trip as a plain vector
// unless a later step needs it.
#include "layers.cuh"

#include <cooperative_groups.h>
#include <cuda_bf16.h>

#include <cstdlib>

#include "prep.cuh"

namespace ctox {

MvOut mv_out(ctox_matvec *mv, uint32_t npos) {
    MatvecPart &p = mv->parts[0];
    const MatvecPart::Split &sp = p.split[npos > 4 ? 1 : 0];
    const uint64_t units = (uint64_t)p.pairs * p.kst_s;
    const bool fits = (units + 1) * sp.warps_per_slice + units < (1ull << 32);  // piece_count() in 32 bits
    return MvOut{p.partial, sp.pieces, mv->s_out, p.slices, p.max_pieces, nullptr, 0,
                 p.kst_s, fits ? sp.warps_per_slice : 0, p.pairs};
}
MvIn mv_in(ctox_matvec *mv) {
    return MvIn{mv->xfrag, mv->meta, mv->s_in, (uint32_t)mv->columns, mv->blocks_padded, mv->parts[0].dt};
}

__device__ __forceinline__ float block_sum(float v, float *red) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
    __syncthreads();
    float s = 0.f;
    for (unsigned w = 0; w < blockDim.x / 32; ++w) s += red[w];  // fixed order
    return s;
}

// h[m][c] (+= matvec output); per-CTA partial sums of squares go to sumsq[m][blockIdx.x].
__global__ void __launch_bounds__(256) k_residual_add(float *__restrict__ h, MvOut add, int has_add,
                                                    uint32_t hidden, float *__restrict__ sumsq) {
    pdl_launch();
    pdl_wait();
    __shared__ float red[8];
    const int m = blockIdx.y;
    const uint32_t c = blockIdx.x * blockDim.x + threadIdx.x;
    float v = 0.f;
    if (c < hidden) {
        v = h[(size_t)m * hidden + c];
        if (has_add) {
            v += out_of(add, c, m);
            h[(size_t)m * hidden + c] = v;
        }
    }
    const float s = block_sum(v * v, red);
    if (threadIdx.x == 0) sumsq[m * gridDim.x + blockIdx.x] = s;
}

// xn = h * rsqrt(mean(h^2) + eps) * (1 + w); optional copy; fragments of xn * s_in. One 16-lane
// group per (position, 64-column block); every group adds the partial sums in the same order.
__global__ void k_norm_prep(const float *__restrict__ h, const float *__restrict__ sumsq, uint32_t nparts,
                            const float *__restrict__ w, float eps, uint32_t hidden, int npos,
                            float *__restrict__ xn_out, MvIn next, int has_next, uint32_t nblocks) {
    pdl_launch();
    pdl_wait();
    const uint32_t gid = (blockIdx.x * blockDim.x + threadIdx.x) >> 4;
    const int i = threadIdx.x & 15;
    if (gid >= nblocks * (uint32_t)npos) return;
    const uint32_t b = gid / npos;
    const int m = gid % npos;
    float sq = 0.f;
    for (uint32_t q = 0; q < nparts; ++q) sq += sumsq[m * nparts + q];
    const float inv = 1.0f / sqrtf(sq / (float)hidden + eps);
    float v[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const uint32_t c = b * 64 + i * 4 + j;
        v[j] = 0.f;
        if (c < hidden) {
            const float xn = h[(size_t)m * hidden + c] * inv * (1.0f + w[c]);
            if (xn_out) xn_out[(size_t)m * hidden + c] = xn;
            v[j] = has_next ? xn * (next.s_in ? next.s_in[c] : 1.0f) : 0.f;
        }
    }
    if (has_next) {
        const unsigned gmask = (threadIdx.x & 16) ? 0xffff0000u : 0x0000ffffu;
        prep_block(v, i, gmask, (int)b, m, npos, next.dt, next.xfrag, next.meta);
    }
}

void launch_residual_add(cudaStream_t st, float *h, const MvOut *add, uint32_t hidden, uint32_t m, float *scratch) {
    MvOut a = add ? *add : MvOut{};
    launch_pdl(k_residual_add, dim3(residual_parts(hidden), m), dim3(256), 0, st, h, a, add != nullptr, hidden, scratch);
}

void launch_norm_prep(cudaStream_t st, const float *h, const float *w, float eps, uint32_t hidden, uint32_t m,
                      float *xn_out, const MvIn *next, const float *scratch) {
    MvIn n = next ? *next : MvIn{nullptr, nullptr, nullptr, 0, 0, 0};
    const uint32_t nparts = (hidden + 255) / 256;
    const uint32_t nblocks = next ? next->blocks_padded : (hidden + 63) / 64;
    const uint32_t groups = nblocks * m;
    launch_pdl(k_norm_prep, dim3((groups * 16 + 127) / 128), dim3(128), 0, st, h, scratch, nparts, w, eps, hidden,
               (int)m, xn_out, n, next != nullptr, nblocks);
}

// Residual add, RMS norm and the next projection's fragments in ONE kernel (the shared part is
// residual_norm_finish, layers.cuh). For hidden <= kRnColumns.
template <int CL>
__global__ void __launch_bounds__(kRnColumns / CL, 1) k_residual_norm_prep(float *__restrict__ h, MvOut add, int has_add,
                                                                    uint32_t hidden, const float *__restrict__ w,
                                                                    float eps, int npos, float *__restrict__ xn_out,
                                                                    MvIn next, int has_next, uint32_t nblocks) {
    pdl_launch();
    const uint32_t tid = threadIdx.x, rank = blockIdx.x;  // gridDim.x == cluster size
    const int m = blockIdx.y;
    const uint32_t c = rank * (kRnColumns / CL) + tid;
    const float wc = c < hidden ? w[c] : 0.f;  // constants first: they do not depend on earlier kernels
    const float sc = (has_next && next.s_in && c < hidden) ? next.s_in[c] : 1.0f;
    const OutRef ar = (has_add && c < hidden) ? out_ref(add, c) : OutRef{nullptr, 0, 0, 1.0f, false};
    pdl_wait();
    float v = 0.f;
    if (c < hidden) {
        v = h[(size_t)m * hidden + c];
        if (has_add) {
            v += out_at(add, ar, c, m);
            h[(size_t)m * hidden + c] = v;
        }
    }
    residual_norm_finish<CL>(v, hidden, wc, sc, eps, m, npos, xn_out, next, has_next, nblocks);
}

void launch_residual_norm_prep(cudaStream_t st, float *h, const MvOut *add, const float *w, float eps,
                               uint32_t hidden, uint32_t m, float *xn_out, const MvIn *next, float *scratch) {
    static const bool merged = [] {
        const char *v = getenv("CTOX_MERGED_NORM");
        return !(v && v[0] == '0');
    }();
    const uint32_t nblocks = next ? next->blocks_padded : (hidden + 63) / 64;
    if (merged && hidden <= kRnColumns && nblocks <= kRnColumns / 64) {
        MvOut a = add ? *add : MvOut{};
        MvIn n = next ? *next : MvIn{nullptr, nullptr, nullptr, 0, 0, 0};
        // one or two positions: 16 CTAs per cluster (more than the portable size: the kernel opts in,
        // once per device); more positions: 8
        static thread_local unsigned long long wide_ok = 0, wide_tried = 0;
        int dev = 0;
        cudaGetDevice(&dev);
        if (m <= 2 && dev < 64 && !(wide_tried >> dev & 1ull)) {
            wide_tried |= 1ull << dev;
            if (cudaFuncSetAttribute(k_residual_norm_prep<kRnClusterWide>, cudaFuncAttributeNonPortableClusterSizeAllowed,
                                     1) == cudaSuccess)
                wide_ok |= 1ull << dev;
            else
                cudaGetLastError();
        }
        if (m <= 2 && dev < 64 && (wide_ok >> dev & 1ull))
            launch_pdl_cluster(k_residual_norm_prep<kRnClusterWide>, dim3(kRnClusterWide, m),
                               dim3(kRnColumns / kRnClusterWide), 0, st, kRnClusterWide, h, a, add != nullptr, hidden, w,
                               eps, (int)m, xn_out, n, next != nullptr, nblocks);
        else
            launch_pdl_cluster(k_residual_norm_prep<kRnCluster>, dim3(kRnCluster, m), dim3(kRnColumns / kRnCluster), 0, st,
                               kRnCluster, h, a, add != nullptr, hidden, w, eps, (int)m, xn_out, n, next != nullptr,
                               nblocks);
        return;
    }
    launch_residual_add(st, h, add, hidden, m, scratch);
    launch_norm_prep(st, h, w, eps, hidden, m, xn_out, next, scratch);
}

// [rmsnorm(embed) | rmsnorm(prev_hidden)] -> fragments (2 * hidden columns). One CTA per
// (16 blocks of 64 columns, position); every CTA adds up both sums of squares itself (40 KB from L2),
// then each 16-lane group writes one block.
__global__ void __launch_bounds__(256) k_mtp_pre(const float *__restrict__ embed_rows,
                                               const float *__restrict__ prev_hidden,
                                               const float *__restrict__ w_embed,
                                               const float *__restrict__ w_hidden, float eps, uint32_t hidden,
                                               int npos, MvIn next) {
    pdl_launch();
    pdl_wait();
    __shared__ float red[8];
    const int m = blockIdx.y;
    const float *e = embed_rows + (size_t)m * hidden, *h = prev_hidden + (size_t)m * hidden;
    float sq_e = 0.f, sq_h = 0.f;
    for (uint32_t c = threadIdx.x; c < hidden; c += blockDim.x) {
        const float a = e[c], b = h[c];
        sq_e += a * a;
        sq_h += b * b;
    }
    const float inv_e = 1.0f / sqrtf(block_sum(sq_e, red) / (float)hidden + eps);
    const float inv_h = 1.0f / sqrtf(block_sum(sq_h, red) / (float)hidden + eps);
    const uint32_t b = blockIdx.x * 16 + (threadIdx.x >> 4);
    if (b >= next.blocks_padded) return;
    const int i = threadIdx.x & 15;
    float v[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const uint32_t c = b * 64 + i * 4 + j;
        v[j] = 0.f;
        if (c < 2 * hidden) {
            const bool second = c >= hidden;
            const uint32_t cc = second ? c - hidden : c;
            const float xn = second ? h[cc] * inv_h * (1.0f + w_hidden[cc]) : e[cc] * inv_e * (1.0f + w_embed[cc]);
            v[j] = xn * (next.s_in ? next.s_in[c] : 1.0f);
        }
    }
    const unsigned gmask = (threadIdx.x & 16) ? 0xffff0000u : 0x0000ffffu;
    prep_block(v, i, gmask, (int)b, m, npos, next.dt, next.xfrag, next.meta);
}

void launch_mtp_pre(cudaStream_t st, const float *embed_rows, const float *prev_hidden, const float *w_embed,
                    const float *w_hidden, float eps, uint32_t hidden, uint32_t m, const MvIn *next) {
    launch_pdl(k_mtp_pre, dim3((next->blocks_padded + 15) / 16, m), dim3(256), 0, st, embed_rows, prev_hidden,
               w_embed, w_hidden, eps, hidden, (int)m, *next);
}

// One CTA per (position, 256 columns of the intermediate width): every thread finishes one
// column (two matvec outputs), then four 16-lane groups write the four 64-column blocks.
constexpr int kSwThreads = 512;  // one column per thread (measured per block: 128 / 256 threads 6.155 ms, 512 6.143, 1024 6.227)
__global__ void __launch_bounds__(kSwThreads) k_swiglu_prep(MvOut gu, uint32_t inter, int npos, MvIn next) {
    pdl_launch();
    __shared__ float vals[kSwThreads];
    const int m = blockIdx.y;
    const uint32_t c = blockIdx.x * kSwThreads + threadIdx.x;
    const float sc = (next.s_in && c < inter) ? next.s_in[c] : 1.0f;  // a constant: before the wait
    const OutRef gr = c < inter ? out_ref(gu, c) : OutRef{nullptr, 0, 0, 1.0f, false};
    const OutRef ur = c < inter ? out_ref(gu, inter + c) : OutRef{nullptr, 0, 0, 1.0f, false};
    pdl_wait();
    float v = 0.f;
    if (c < inter) {
        float gate, up;
        if (gr.pieces && gr.total <= 8 && ur.total <= 8) {
            // both values' pieces requested before the first addition (same additions as out_of)
            float bg[8], bu[8];
            const float *fg = gr.first + m * 32, *fu = ur.first + m * 32;
            uint32_t sg = 0, qg = 0, su = 0, qu = 0;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                bg[j] = bu[j] = 0.f;
                if ((uint32_t)j < gr.total) {
                    bg[j] = fg[((size_t)sg * gu.max_pieces + qg) * 256];
                    if (++qg == gr.n) {
                        qg = 0;
                        ++sg;
                    }
                }
                if ((uint32_t)j < ur.total) {
                    bu[j] = fu[((size_t)su * gu.max_pieces + qu) * 256];
                    if (++qu == ur.n) {
                        qu = 0;
                        ++su;
                    }
                }
            }
            gate = up = 0.f;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                if ((uint32_t)j < gr.total) gate += bg[j];
                if ((uint32_t)j < ur.total) up += bu[j];
            }
            if (gu.s_out) {
                gate *= gr.so;
                up *= ur.so;
            }
        } else {
            out_of2(gu, c, inter + c, m, gate, up);
        }
        v = silu_f(gate) * up * sc;
    }
    vals[threadIdx.x] = v;
    __syncthreads();
    if (threadIdx.x < kSwThreads / 4) {
        const int i = threadIdx.x & 15, grp = threadIdx.x >> 4;
        const uint32_t b = blockIdx.x * (kSwThreads / 64) + grp;
        if (b < next.blocks_padded) {
            const float x[4] = {vals[grp * 64 + i * 4], vals[grp * 64 + i * 4 + 1], vals[grp * 64 + i * 4 + 2],
                                vals[grp * 64 + i * 4 + 3]};
            const unsigned gmask = (threadIdx.x & 16) ? 0xffff0000u : 0x0000ffffu;
            prep_block(x, i, gmask, (int)b, m, npos, next.dt, next.xfrag, next.meta);
        }
    }
}

void launch_swiglu_prep(cudaStream_t st, const MvOut &gate_up, uint32_t inter, uint32_t m, const MvIn &next) {
    launch_pdl(k_swiglu_prep, dim3((next.blocks_padded + kSwThreads / 64 - 1) / (kSwThreads / 64), m), dim3(kSwThreads), 0, st,
               gate_up, inter, (int)m, next);
}

// ------------------------------------------------------------------ linear attention
// conv_state <- conv_state shifted by the first n kept inputs of a pass (causal_conv_silu_update,
// reference.rs:159-187: shift left, append): the commit of n positions when the batched commit
// kernel is not in use.
__global__ void k_conv_commit(float *__restrict__ conv_state, const float *__restrict__ conv_in,
                              uint32_t channels, uint32_t conv_kernel, uint32_t n) {
    pdl_launch();
    pdl_wait();
    const uint32_t r = blockIdx.x * blockDim.x + threadIdx.x;
    if (r >= channels) return;
    float st[8];
    for (uint32_t j = 0; j < conv_kernel; ++j) st[j] = conv_state[(size_t)r * conv_kernel + j];
    for (uint32_t m = 0; m < n; ++m) {
        for (uint32_t j = 0; j + 1 < conv_kernel; ++j) st[j] = st[j + 1];
        st[conv_kernel - 1] = conv_in[(size_t)m * channels + r];
    }
    for (uint32_t j = 0; j < conv_kernel; ++j) conv_state[(size_t)r * conv_kernel + j] = st[j];
}

void launch_conv_commit(cudaStream_t st, float *conv_state, const float *conv_in, uint32_t channels,
                        uint32_t conv_kernel, uint32_t n) {
    launch_pdl(k_conv_commit, dim3((channels + 127) / 128), dim3(128), 0, st, conv_state, conv_in, channels, conv_kernel, n);
}

// ------------------------------------------------------------------ full attention
template <typename T>
__device__ __forceinline__ float kv_load(const T *p);
template <>
__device__ __forceinline__ float kv_load<float>(const float *p) { return *p; }
template <>
__device__ __forceinline__ float kv_load<__nv_bfloat16>(const __nv_bfloat16 *p) { return __bfloat162float(*p); }
template <typename T>
__device__ __forceinline__ void kv_store(T *p, float v);
template <>
__device__ __forceinline__ void kv_store<float>(float *p, float v) { *p = v; }
template <>
__device__ __forceinline__ void kv_store<__nv_bfloat16>(__nv_bfloat16 *p, float v) { *p = __float2bfloat16_rn(v); }

__device__ __forceinline__ size_t kv_slot(const uint32_t *page_table, uint32_t page_tokens, uint64_t t) {
    return (size_t)page_table[t / page_tokens] * page_tokens + (size_t)(t % page_tokens);
}

// One CTA per (position, head) and one thread per head dimension over the fused [q+gate | k | v]
// projection (decoder.rs:717-772): q rows are [query(hd), gate(hd)] per head; q and k get the
// (1+w) RMS norm per head and the non-interleaved partial RoPE (reference.rs:115-155); k and v go
// to the cache slot of the position. One element per thread keeps the chain of dependent loads
// (piece count, then the partial sums) one deep.
template <typename T>
__global__ void __launch_bounds__(256) k_attn_pre(MvOut fan, AttnGeom g, const float *__restrict__ q_norm,
                                                  const float *__restrict__ k_norm, uint64_t rope_position,
                                                  uint64_t cache_slot, int npos, float *__restrict__ q,
                                                  float *__restrict__ gate, T *__restrict__ k_cache,
                                                  T *__restrict__ v_cache, const uint32_t *__restrict__ page_table,
                                                  uint32_t page_tokens) {
    pdl_launch();
    pdl_wait();
    __shared__ float buf[256];
    __shared__ float red[8];
    const uint32_t heads_total = g.q_heads + 2 * g.kv_heads;
    const uint32_t hi = blockIdx.x % heads_total;
    const int m = blockIdx.x / heads_total;
    const uint32_t hd = g.head_dim, d = threadIdx.x;  // blockDim.x == head_dim
    const uint32_t k_row0 = g.q_heads * 2 * hd, v_row0 = k_row0 + g.kv_heads * hd;
    const size_t slot = kv_slot(page_table, page_tokens, cache_slot + m);
    if (hi >= g.q_heads + g.kv_heads) {  // value head: plain copy into the cache
        const uint32_t kh = hi - g.q_heads - g.kv_heads;
        kv_store(v_cache + (slot * g.kv_heads + kh) * hd + d, out_of(fan, v_row0 + kh * hd + d, m));
        return;
    }
    const bool is_q = hi < g.q_heads;
    const uint32_t head = is_q ? hi : hi - g.q_heads;
    const uint32_t row0 = is_q ? head * 2 * hd : k_row0 + head * hd;
    const float v = out_of(fan, row0 + d, m);
    if (is_q) gate[((size_t)m * g.q_heads + head) * hd + d] = out_of(fan, row0 + hd + d, m);
    const float sq = block_sum(v * v, red);
    const float inv = 1.0f / sqrtf(sq / (float)hd + g.eps);
    const float xn = v * inv * (1.0f + (is_q ? q_norm : k_norm)[d]);
    buf[d] = xn;
    __syncthreads();
    float out = xn;
    if (d < g.rotary_dim) {
        const uint32_t half = g.rotary_dim / 2;
        const uint32_t i = d < half ? d : d - half;
        const float pos = (float)(rope_position + (uint64_t)m);
        const float inv_freq = powf(g.theta, -((float)(2 * i)) / (float)g.rotary_dim);
        const float ang = pos * inv_freq, cs = cosf(ang), sn = sinf(ang);
        out = d < half ? xn * cs - buf[d + half] * sn : xn * cs + buf[d - half] * sn;
    }
    if (is_q)
        q[((size_t)m * g.q_heads + head) * hd + d] = out;
    else
        kv_store(k_cache + (slot * g.kv_heads + head) * hd + d, out);
}

void launch_attn_pre(cudaStream_t st, const MvOut &fan, const AttnGeom &g, const float *q_norm,
                     const float *k_norm, uint64_t rope_position, uint64_t cache_slot, uint32_t m, float *q,
                     float *gate, void *k_cache, void *v_cache, int kv_bf16, const uint32_t *page_table,
                     uint32_t page_tokens) {
    const uint32_t grid = (g.q_heads + 2 * g.kv_heads) * m;
    if (kv_bf16)
        launch_pdl(k_attn_pre<__nv_bfloat16>, dim3(grid), dim3(g.head_dim), 0, st, fan, g, q_norm, k_norm,
                   rope_position, cache_slot, (int)m, q, gate, (__nv_bfloat16 *)k_cache, (__nv_bfloat16 *)v_cache,
                   page_table, page_tokens);
    else
        launch_pdl(k_attn_pre<float>, dim3(grid), dim3(g.head_dim), 0, st, fan, g, q_norm, k_norm, rope_position,
                   cache_slot, (int)m, q, gate, (float *)k_cache, (float *)v_cache, page_table, page_tokens);
}

constexpr int kAttnTile = 32;      // tokens per tile
constexpr int kAttnThreads = 256;

// grouped_query_attention (reference.rs:420-499) for the m query positions of one KV head over
// one split of the context, flash-decoding style: per tile of 32 tokens the K rows are staged in
// shared memory, every warp scores its queries against the 32 tokens (lane = token), keeps the
// running max / sum per query, and each thread then owns one output dimension of all queries.
// Partial (max, sum, unnormalised output) go to the workspace; k_attn_combine_prep merges them.
template <typename T, int NQMAX>
__global__ void __launch_bounds__(kAttnThreads) k_attention(
    AttnGeom g, const float *__restrict__ q, const T *__restrict__ k_cache, const T *__restrict__ v_cache,
    const uint32_t *__restrict__ page_table, uint32_t page_tokens, uint64_t cache_slot, int npos,
    uint32_t splits, float *__restrict__ ws) {
    pdl_launch();
    pdl_wait();
    extern __shared__ __align__(128) uint8_t smraw[];
    const uint32_t hd = g.head_dim, G = g.q_heads / g.kv_heads, NQ = G * npos;
    const uint32_t kh = blockIdx.x / splits, sp = blockIdx.x % splits;
    const uint32_t kstride = hd + 16 / sizeof(T);  // padded row: conflict-free 16-byte reads
    float *q_s = reinterpret_cast<float *>(smraw);                       // [NQ][hd]
    float *p_s = q_s + NQMAX * hd;                                        // [NQ][tile]
    float *m_run = p_s + NQMAX * kAttnTile, *l_run = m_run + NQMAX, *alpha = l_run + NQMAX;
    T *k_s = reinterpret_cast<T *>(alpha + NQMAX);                        // [tile][kstride]
    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint64_t total = cache_slot + (uint64_t)npos;  // tokens visible to the last query
    const uint64_t tiles = (total + kAttnTile - 1) / kAttnTile;
    const uint64_t tile_beg = tiles * sp / splits, tile_end = tiles * (sp + 1) / splits;
    for (uint32_t i = tid; i < NQ * hd; i += kAttnThreads) {
        const uint32_t qi = i / hd, d = i % hd, mi = qi / G, gq = qi % G;
        q_s[i] = q[((size_t)mi * g.q_heads + kh * G + gq) * hd + d];
    }
    if (tid < NQMAX) {
        m_run[tid] = -INFINITY;
        l_run[tid] = 0.f;
    }
    float o[NQMAX];
#pragma unroll
    for (int i = 0; i < NQMAX; ++i) o[i] = 0.f;
    const float scale = 1.0f / sqrtf((float)hd);
    __syncthreads();
    for (uint64_t tile = tile_beg; tile < tile_end; ++tile) {
        const uint64_t t0 = tile * kAttnTile;
        // stage K rows (16-byte chunks, coalesced)
        const uint32_t chunks_per_row = hd * sizeof(T) / 16;
        for (uint32_t c = tid; c < kAttnTile * chunks_per_row; c += kAttnThreads) {
            const uint32_t r = c / chunks_per_row, cc = c % chunks_per_row;
            uint4 v = make_uint4(0, 0, 0, 0);
            if (t0 + r < total) {
                const size_t slot = kv_slot(page_table, page_tokens, t0 + r);
                v = *reinterpret_cast<const uint4 *>(reinterpret_cast<const uint8_t *>(
                        k_cache + (slot * g.kv_heads + kh) * hd) + cc * 16);
            }
            *reinterpret_cast<uint4 *>(reinterpret_cast<uint8_t *>(k_s + r * kstride) + cc * 16) = v;
        }
        __syncthreads();
        // scores + running softmax: warp w takes queries w, w+8, ...; lane = token of the tile
        const uint64_t t = t0 + lane;
        for (uint32_t qi = warp; qi < NQ; qi += kAttnThreads / 32) {
            const uint32_t mi = qi / G;
            float s = 0.f;
            const T *kr = k_s + lane * kstride;
            const float *qr = q_s + qi * hd;
            for (uint32_t d = 0; d < hd; ++d) s += qr[d] * kv_load(kr + d);
            s *= scale;
            const bool valid = t < total && t <= cache_slot + mi;  // causal inside the pass
            if (!valid) s = -INFINITY;
            float tmax = s;
#pragma unroll
            for (int of = 16; of > 0; of >>= 1) tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, of));
            const float m_old = m_run[qi], m_new = fmaxf(m_old, tmax);
            const float p = (valid && m_new > -INFINITY) ? expf(s - m_new) : 0.f;
            float psum = p;
#pragma unroll
            for (int of = 16; of > 0; of >>= 1) psum += __shfl_xor_sync(0xffffffffu, psum, of);
            p_s[qi * kAttnTile + lane] = p;
            if (lane == 0) {
                const float a = m_old > -INFINITY ? expf(m_old - m_new) : 0.f;
                alpha[qi] = a;
                l_run[qi] = l_run[qi] * a + psum;
                m_run[qi] = m_new;
            }
        }
        __syncthreads();
        // output: thread d owns dimension d of every query
        if (tid < hd) {
#pragma unroll
            for (int qi = 0; qi < NQMAX; ++qi)
                if ((uint32_t)qi < NQ) o[qi] *= alpha[qi];
            for (uint32_t r = 0; r < (uint32_t)kAttnTile && t0 + r < total; ++r) {
                const size_t slot = kv_slot(page_table, page_tokens, t0 + r);
                const float vv = kv_load(v_cache + (slot * g.kv_heads + kh) * hd + tid);
#pragma unroll
                for (int qi = 0; qi < NQMAX; ++qi)
                    if ((uint32_t)qi < NQ) o[qi] += p_s[qi * kAttnTile + r] * vv;
            }
        }
        __syncthreads();
    }
    // workspace: [kv head][split][query][hd + 2]
    float *out = ws + ((size_t)(kh * splits + sp) * NQ) * (hd + 2);
    if (tid < hd) {
#pragma unroll
        for (int qi = 0; qi < NQMAX; ++qi)
            if ((uint32_t)qi < NQ) out[(size_t)qi * (hd + 2) + tid] = o[qi];
    }
    if (tid < NQ) {
        out[(size_t)tid * (hd + 2) + hd] = m_run[tid];
        out[(size_t)tid * (hd + 2) + hd + 1] = l_run[tid];
    }
}

// ------------------------------------------------------------------ tensor-core attention (bf16 cache)
// Same contract as k_attention for a bf16 cache and head_dim 256, built for HBM speed:
//  * 64-token K and V tiles are staged in shared memory with 16-byte cp.async, double buffered;
//  * each warp owns 16 tokens of a tile and 16 queries (warps 0-3: queries 0-15, warps 4-7:
//    queries 16-31) and runs flash-attention on mma.sync.m16n8k16 (bf16 in, fp32 accumulate):
//    S = Q K^T with Q split as bf16 hi + lo (16 significant bits, K exact), online softmax in the
//    accumulator layout, O += P V with P split the same way and V read through ldmatrix.trans;
//  * no barrier between the four warps of a group inside a tile: each keeps its own running
//    max / sum / O and the four are merged once at the end, like the context splits.
// Q rows are padded (conflict-free ldmatrix). With two query groups the K / V tile rows are 512 bytes
// with their 16-byte chunks XOR-swizzled by the row (chunk c of row r sits at c ^ (r & 7)):
// conflict-free too, and three tile buffers fit beside Q. With one group: two buffers of padded rows.
constexpr int kFaTile = 64, kFaHd = 256, kFaStride = kFaHd + 8;
// Tile buffers: three (two tiles in flight) for two query groups, two for one (measured: the third
// buffer costs the 4-warp kernel 5 us per launch).
__host__ __device__ constexpr int fa_buffers(int groups) { return groups == 2 ? 3 : 2; }

__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void cp_async16(uint32_t dst, const void *src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const uint32_t *>(&v);
}
// hi and lo parts of two floats as packed bf16 pairs
__device__ __forceinline__ void split_bf16(float x, float y, uint32_t &hi, uint32_t &lo) {
    const __nv_bfloat16 xh = __float2bfloat16_rn(x), yh = __float2bfloat16_rn(y);
    hi = pack_bf16(__bfloat162float(xh), __bfloat162float(yh));
    lo = pack_bf16(x - __bfloat162float(xh), y - __bfloat162float(yh));
}

template <int GROUPS>  // 1: up to 16 queries (4 warps), 2: up to 32 queries (8 warps)
__global__ void __launch_bounds__(GROUPS * 128, 1) k_attention_mma(
    AttnGeom g, const float *__restrict__ q, const __nv_bfloat16 *__restrict__ k_cache,
    const __nv_bfloat16 *__restrict__ v_cache, const uint32_t *__restrict__ page_table, uint32_t page_tokens,
    uint64_t cache_slot, int npos, uint32_t splits, float *__restrict__ ws) {
    pdl_launch();
    extern __shared__ __align__(128) uint8_t smraw[];
    constexpr int NT = GROUPS * 128, kFaBuffers = fa_buffers(GROUPS);
    const uint32_t G = g.q_heads / g.kv_heads, NQ = G * npos;
    const uint32_t kh = blockIdx.x / splits, sp = blockIdx.x % splits;
    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, gq = lane >> 2, tq = lane & 3;
    const uint32_t grp = warp >> 2, wg = warp & 3;  // query group, warp inside the group
    // shared memory: Q [2 terms][32 queries][stride], then kFaBuffers buffers of (K tile, V tile)
    __nv_bfloat16 *q_s = reinterpret_cast<__nv_bfloat16 *>(smraw);
    // tile rows: swizzled 512-byte rows where three buffers must fit, padded rows otherwise (their
    // ldmatrix offsets are compile-time constants)
    constexpr bool kSwz = kFaBuffers == 3;
    constexpr uint32_t kRowB = kSwz ? kFaHd * 2 : kFaStride * 2;
    constexpr uint32_t kQBytes = 2 * 32 * kFaStride * 2, kTileBytes = kFaTile * kRowB;
    const uint32_t q_a = (uint32_t)__cvta_generic_to_shared(q_s);
    const uint32_t buf_a = q_a + kQBytes;  // buffer b: K at buf_a + b*2*kTileBytes, V right after
    const uint64_t total = cache_slot + (uint64_t)npos;
    const uint64_t tiles = (total + kFaTile - 1) / kFaTile;
    const uint64_t tile_beg = tiles * sp / splits, tile_end = tiles * (sp + 1) / splits;
    const float scale = 1.0f / sqrtf((float)kFaHd);
    // Tile loads. Thread (warp, lane) copies the 16-byte chunk `lane` of rows warp, warp + NT/32, ...
    // of the K and of the V tile. The cache slots of a tile (page-table lookups) are fetched one
    // tile ahead of the copies that use them, so the lookups never sit between two copies.
    constexpr int kRowStep = NT / 32, kRowsPerThread = kFaTile / kRowStep;
    constexpr uint32_t kNoSlot = 0xffffffffu;
    const int page_shift = (page_tokens & (page_tokens - 1)) == 0 ? 31 - __clz(page_tokens) : -1;
    uint32_t slots[kRowsPerThread];
    // a tile is 2..32 whole pages: one lookup per lane
    const bool tile_pages = page_shift >= 1 && page_tokens <= (uint32_t)kFaTile;
    auto fetch_slots = [&](uint64_t tile) {
        if (tile_pages) {
            // lane l reads the l-th page of the tile; the rows pick theirs with a shuffle
            const uint32_t first_page = (uint32_t)(tile * kFaTile) >> page_shift;
            const uint32_t pages_per_tile = (uint32_t)kFaTile >> page_shift;
            const uint32_t last_page = (uint32_t)(total - 1) >> page_shift;
            uint32_t mine = 0;
            if (lane < pages_per_tile && first_page + lane <= last_page) mine = page_table[first_page + lane];
#pragma unroll
            for (int j = 0; j < kRowsPerThread; ++j) {
                const uint32_t r = warp + j * kRowStep;
                const uint32_t pg = __shfl_sync(0xffffffffu, mine, r >> page_shift);
                const uint64_t t = tile * kFaTile + r;
                slots[j] = t < total ? (pg << page_shift) + (r & (page_tokens - 1)) : kNoSlot;
            }
            return;
        }
#pragma unroll
        for (int j = 0; j < kRowsPerThread; ++j) {
            const uint64_t t = tile * kFaTile + warp + j * kRowStep;
            const uint32_t t32 = (uint32_t)t;
            slots[j] = t < total ? page_table[t32 / page_tokens] * page_tokens + t32 % page_tokens : kNoSlot;
        }
    };
    auto issue_tile = [&](uint32_t b) {
#pragma unroll
        for (int j = 0; j < kRowsPerThread; ++j) {
            const uint32_t r = warp + j * kRowStep;
            const uint32_t dst = buf_a + b * 2 * kTileBytes + r * kRowB + ((kSwz ? lane ^ (r & 7) : lane) * 16);
            if (slots[j] != kNoSlot) {
                const size_t off = ((size_t)slots[j] * g.kv_heads + kh) * kFaHd + lane * 8;
                cp_async16(dst, k_cache + off);
                cp_async16(dst + kTileBytes, v_cache + off);
            } else {
                asm volatile("st.shared.v4.u32 [%0], {%1,%1,%1,%1};" ::"r"(dst), "r"(0u) : "memory");
                asm volatile("st.shared.v4.u32 [%0], {%1,%1,%1,%1};" ::"r"(dst + kTileBytes), "r"(0u) : "memory");
            }
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    float oacc[32][4];
#pragma unroll
    for (int i = 0; i < 32; ++i) oacc[i][0] = oacc[i][1] = oacc[i][2] = oacc[i][3] = 0.f;
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
    const uint32_t qrow[2] = {grp * 16 + gq, grp * 16 + gq + 8};
    uint64_t limit[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) limit[r] = cache_slot + (qrow[r] < NQ ? qrow[r] / G : 0);
    // The page table does not change after warm-up: the lookups of the first tile go out before the
    // wait for the kernels in front (which write q and the new K/V rows).
    if (tile_beg < tile_end) fetch_slots(tile_beg);
    pdl_wait();
    if (tile_beg < tile_end) {
        issue_tile(0);
        if (tile_beg + 1 < tile_end) fetch_slots(tile_beg + 1);  // lands while Q is staged below
    }
    {   // Q as bf16 hi + lo: 8 float4 per thread, all loads issued before the first conversion
        constexpr int kQRows = 16 * GROUPS, kVec = kQRows * kFaHd / 4 / NT;
        float4 qv[kVec];
#pragma unroll
        for (int it = 0; it < kVec; ++it) {
            const uint32_t i = (tid + it * NT) * 4, qi = i / kFaHd, d = i % kFaHd;
            qv[it] = make_float4(0.f, 0.f, 0.f, 0.f);
            if (qi < NQ)
                qv[it] = *reinterpret_cast<const float4 *>(
                    q + ((size_t)(qi / G) * g.q_heads + kh * G + qi % G) * kFaHd + d);
        }
#pragma unroll
        for (int it = 0; it < kVec; ++it) {
            const uint32_t i = (tid + it * NT) * 4, qi = i / kFaHd, d = i % kFaHd;
            const float v[4] = {qv[it].x * scale, qv[it].y * scale, qv[it].z * scale, qv[it].w * scale};
            uint32_t hi[2], lo[2];
            split_bf16(v[0], v[1], hi[0], lo[0]);
            split_bf16(v[2], v[3], hi[1], lo[1]);
            *reinterpret_cast<uint2 *>(q_s + qi * kFaStride + d) = make_uint2(hi[0], hi[1]);
            *reinterpret_cast<uint2 *>(q_s + (32 + qi) * kFaStride + d) = make_uint2(lo[0], lo[1]);
        }
    }
    if (kFaBuffers == 3 && tile_beg + 1 < tile_end) {  // the second tile in flight before the first is worked on
        issue_tile(1);
        if (tile_beg + 2 < tile_end) fetch_slots(tile_beg + 2);
    }
    for (uint64_t tile = tile_beg; tile < tile_end; ++tile) {
        const uint32_t b = (uint32_t)((tile - tile_beg) % kFaBuffers);
        if (kFaBuffers == 2) {
            // two buffers: the next tile is requested before this one is waited for (both in flight
            // during the wait); a barrier at the end of the iteration frees this buffer
            if (tile + 1 < tile_end) {
                issue_tile(b ^ 1);
                if (tile + 2 < tile_end) fetch_slots(tile + 2);
                asm volatile("cp.async.wait_group 1;" ::: "memory");
            } else {
                asm volatile("cp.async.wait_group 0;" ::: "memory");
            }
            __syncthreads();
        } else {
            // three buffers: this tile's copies have landed (the group issued after it may still be in
            // flight) for every thread, and every thread is done with the tile before, whose buffer
            // takes the tile after next: one barrier per tile, two tiles in flight
            if (tile + 1 < tile_end)
                asm volatile("cp.async.wait_group 1;" ::: "memory");
            else
                asm volatile("cp.async.wait_group 0;" ::: "memory");
            __syncthreads();
            if (tile + 2 < tile_end) {
                issue_tile((b + 2) % kFaBuffers);
                if (tile + 3 < tile_end) fetch_slots(tile + 3);
            }
        }
        const uint32_t k_a = buf_a + b * 2 * kTileBytes, v_a = k_a + kTileBytes;
        const uint32_t tok0 = wg * 16;
        // ---- S = Q K^T for this warp's 16 queries x 16 tokens
        float sacc[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
        float slo[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};  // the lo term's own chains
#pragma unroll 4
        for (int ks = 0; ks < kFaHd / 16; ++ks) {
            uint32_t bk[4], aq[4];
            // K matrices: (tokens 0-7, k 0-7), (tokens 0-7, k 8-15), (tokens 8-15, k 0-7), (tokens 8-15, k 8-15)
            ldsm_x4(bk, k_a + (tok0 + (lane & 7) + 8 * (lane >> 4)) * kRowB +
                            ((kSwz ? (ks * 2 + ((lane >> 3) & 1)) ^ (lane & 7) : ks * 2 + ((lane >> 3) & 1)) * 16));
#pragma unroll
            for (int term = 0; term < 2; ++term) {
                // Q matrices: (rows 0-7, k 0-7), (rows 8-15, k 0-7), (rows 0-7, k 8-15), (rows 8-15, k 8-15)
                ldsm_x4(aq, q_a + ((term * 32 + grp * 16 + (lane & 7) + 8 * ((lane >> 3) & 1)) * kFaStride +
                                   ks * 16 + 8 * (lane >> 4)) * 2);
                mma_bf16(term ? slo[0] : sacc[0], aq, bk[0], bk[1]);
                mma_bf16(term ? slo[1] : sacc[1], aq, bk[2], bk[3]);
            }
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            sacc[0][i] += slo[0][i];
            sacc[1][i] += slo[1][i];
        }
        // ---- online softmax; this lane holds rows gq, gq+8 and tokens tok0 + {2tq, 2tq+1, 8+2tq, 9+2tq}
        const uint64_t tbase = tile * kFaTile + tok0;
        uint32_t p_hi[4], p_lo[4];
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            float sv[4] = {sacc[0][2 * r], sacc[0][2 * r + 1], sacc[1][2 * r], sacc[1][2 * r + 1]};
            const uint32_t toff[4] = {2 * tq, 2 * tq + 1, 8 + 2 * tq, 9 + 2 * tq};
            float tmax = -INFINITY;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                if (tbase + toff[j] > limit[r] || tbase + toff[j] >= total) sv[j] = -INFINITY;
                tmax = fmaxf(tmax, sv[j]);
            }
            tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, 1));
            tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, 2));
            const float m_new = fmaxf(m_run[r], tmax);
            const float alpha = m_run[r] > -INFINITY ? expf(m_run[r] - m_new) : 0.f;
            float ps[4], sum = 0.f;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                ps[j] = sv[j] > -INFINITY ? expf(sv[j] - m_new) : 0.f;
                sum += ps[j];
            }
            sum += __shfl_xor_sync(0xffffffffu, sum, 1);
            sum += __shfl_xor_sync(0xffffffffu, sum, 2);
            l_run[r] = l_run[r] * alpha + sum;
            m_run[r] = m_new;
            if (alpha != 1.0f) {  // the running maximum settles after the first tiles
#pragma unroll
                for (int i = 0; i < 32; ++i) {
                    oacc[i][2 * r] *= alpha;
                    oacc[i][2 * r + 1] *= alpha;
                }
            }
            // A fragment of P: a0 (row g, k 2t..) / a1 (row g+8) from n-tile 0, a2 / a3 from n-tile 1
            split_bf16(ps[0], ps[1], p_hi[r], p_lo[r]);
            split_bf16(ps[2], ps[3], p_hi[2 + r], p_lo[2 + r]);
        }
        // ---- O += P V: V matrices (trans): (tokens 0-7, dims n0..), (tokens 8-15, dims n0..),
        //      (tokens 0-7, dims n0+8..), (tokens 8-15, dims n0+8..)
#pragma unroll
        for (int dn = 0; dn < kFaHd / 16; ++dn) {
            uint32_t bv[4];
            ldsm_x4_trans(bv, v_a + (tok0 + (lane & 7) + 8 * ((lane >> 3) & 1)) * kRowB +
                                  ((kSwz ? (dn * 2 + (lane >> 4)) ^ (lane & 7) : dn * 2 + (lane >> 4)) * 16));
            mma_bf16(oacc[2 * dn], p_hi, bv[0], bv[1]);
            mma_bf16(oacc[2 * dn], p_lo, bv[0], bv[1]);
            mma_bf16(oacc[2 * dn + 1], p_hi, bv[2], bv[3]);
            mma_bf16(oacc[2 * dn + 1], p_lo, bv[2], bv[3]);
        }
        if (kFaBuffers == 2) __syncthreads();  // everyone is done with buffer b before it is refilled
    }
    __syncthreads();  // the merge below reuses the tile buffers
    // ---- merge the four warps of each group through shared memory (reusing the tile buffers)
    float *mo = reinterpret_cast<float *>(smraw + kQBytes);  // [warp][16 rows][hd + 2]
    float *mine = mo + (size_t)warp * 16 * (kFaHd + 2);
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        float *row = mine + (gq + 8 * r) * (kFaHd + 2);
#pragma unroll
        for (int i = 0; i < 32; ++i) {
            row[i * 8 + 2 * tq] = oacc[i][2 * r];
            row[i * 8 + 2 * tq + 1] = oacc[i][2 * r + 1];
        }
        if (tq == 0) {
            row[kFaHd] = m_run[r];
            row[kFaHd + 1] = l_run[r];
        }
    }
    __syncthreads();
    float *out = ws + ((size_t)(kh * splits + sp) * NQ) * (kFaHd + 2);
    // weights of the four warps per query row, once; they go where the rows kept (max, sum)
    if (tid < 16 * GROUPS && tid < NQ) {
        const uint32_t gg = tid / 16, rr = tid % 16;
        float mx = -INFINITY, den = 0.f, wgt[4];
        for (int w = 0; w < 4; ++w) mx = fmaxf(mx, mo[((size_t)(gg * 4 + w) * 16 + rr) * (kFaHd + 2) + kFaHd]);
        for (int w = 0; w < 4; ++w) {
            float *row = mo + ((size_t)(gg * 4 + w) * 16 + rr) * (kFaHd + 2);
            wgt[w] = row[kFaHd] > -INFINITY ? expf(row[kFaHd] - mx) : 0.f;
            den += row[kFaHd + 1] * wgt[w];
        }
        for (int w = 0; w < 4; ++w) mo[((size_t)(gg * 4 + w) * 16 + rr) * (kFaHd + 2) + kFaHd] = wgt[w];
        out[(size_t)tid * (kFaHd + 2) + kFaHd] = mx;
        out[(size_t)tid * (kFaHd + 2) + kFaHd + 1] = den;
    }
    __syncthreads();
#pragma unroll 4
    for (uint32_t i = tid; i < 16 * GROUPS * (kFaHd / 2); i += NT) {
        const uint32_t qi = i / (kFaHd / 2), d = (i % (kFaHd / 2)) * 2;
        if (qi >= NQ) continue;
        const uint32_t gg = qi / 16, rr = qi % 16;
        float2 acc = make_float2(0.f, 0.f);
#pragma unroll
        for (int w = 0; w < 4; ++w) {
            const float *row = mo + ((size_t)(gg * 4 + w) * 16 + rr) * (kFaHd + 2);
            const float wgt = row[kFaHd];
            const float2 v = *reinterpret_cast<const float2 *>(row + d);
            acc.x += v.x * wgt;
            acc.y += v.y * wgt;
        }
        *reinterpret_cast<float2 *>(out + (size_t)qi * (kFaHd + 2) + d) = acc;
    }
}

// Merge of the splits, sigmoid gate (reference.rs:502-515) and fragments for o_proj: one CTA per
// (position, query head), one thread per head dimension. The weights of the splits are formed once
// per CTA; every thread then adds its dimension over the splits, eight loads at a time.
__global__ void __launch_bounds__(256) k_attn_combine_prep(AttnGeom g, const float *__restrict__ ws,
                                                         const float *__restrict__ gate, int npos, uint32_t splits,
                                                         MvIn next) {
    pdl_launch();
    pdl_wait();
    __shared__ float wgt[kAttnMaxSplits];  // per split: exp(max_s - max) / denominator
    __shared__ float vals[256];  // the head's output, gated and scaled
    const uint32_t hd = g.head_dim, G = g.q_heads / g.kv_heads, NQ = G * npos;
    const uint32_t hq = blockIdx.x % g.q_heads;
    const int m = blockIdx.x / g.q_heads;
    const uint32_t kh = hq / G, qi = m * G + hq % G, d = threadIdx.x;  // blockDim.x == head_dim
    const float *base = ws + ((size_t)kh * splits * NQ + qi) * (hd + 2);
    const size_t split_stride = (size_t)NQ * (hd + 2);
    // this thread's dimension of the first sixteen splits and its gate value: requested before the
    // weights are formed (they do not depend on them), sixteen loads per trip afterwards
    float buf[16];
#pragma unroll
    for (int j = 0; j < 16; ++j) buf[j] = (uint32_t)j < splits ? base[j * split_stride + d] : 0.f;
    const float gt = gate[((size_t)m * g.q_heads + hq) * hd + d];
    if (threadIdx.x < 32) {  // splits <= kAttnMaxSplits: up to kPerLane per lane
        constexpr int kPerLane = kAttnMaxSplits / 32;
        float ms[kPerLane], ls[kPerLane];
#pragma unroll
        for (int j = 0; j < kPerLane; ++j) {
            const uint32_t sp = threadIdx.x + 32 * j;
            ms[j] = sp < splits ? base[sp * split_stride + hd] : -INFINITY;
            ls[j] = sp < splits ? base[sp * split_stride + hd + 1] : 0.f;
        }
        float mx = ms[0];
#pragma unroll
        for (int j = 1; j < kPerLane; ++j) mx = fmaxf(mx, ms[j]);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
        float w[kPerLane], den = 0.f;
#pragma unroll
        for (int j = 0; j < kPerLane; ++j) {
            w[j] = ms[j] > -INFINITY ? expf(ms[j] - mx) : 0.f;
            den += ls[j] * w[j];
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) den += __shfl_xor_sync(0xffffffffu, den, o);
#pragma unroll
        for (int j = 0; j < kPerLane; ++j)
            if (threadIdx.x + 32 * j < splits) wgt[threadIdx.x + 32 * j] = w[j] / den;
    }
    __syncthreads();
    float acc = 0.f;
    for (uint32_t s0 = 0; s0 < splits; s0 += 16) {
        float nxt[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) nxt[j] = s0 + 16 + j < splits ? base[(s0 + 16 + j) * split_stride + d] : 0.f;
#pragma unroll
        for (int j = 0; j < 16; ++j)
            if (s0 + j < splits) acc += buf[j] * wgt[s0 + j];
#pragma unroll
        for (int j = 0; j < 16; ++j) buf[j] = nxt[j];
    }
    const uint32_t col = hq * hd + d;
    vals[d] = acc * (1.0f / (1.0f + expf(-gt))) * (next.s_in ? next.s_in[col] : 1.0f);
    __syncthreads();
    const uint32_t bph = hd / 64;
    if (threadIdx.x < bph * 16) {
        const int i = threadIdx.x & 15;
        const uint32_t blk = threadIdx.x >> 4;
        const float v[4] = {vals[blk * 64 + i * 4], vals[blk * 64 + i * 4 + 1], vals[blk * 64 + i * 4 + 2],
                            vals[blk * 64 + i * 4 + 3]};
        const unsigned gmask = (threadIdx.x & 16) ? 0xffff0000u : 0x0000ffffu;
        prep_block(v, i, gmask, (int)(hq * bph + blk), m, npos, next.dt, next.xfrag, next.meta);
    }
}

size_t attn_workspace_bytes(const AttnGeom &g, uint32_t m, uint32_t max_splits) {
    return (size_t)g.q_heads * m * max_splits * (g.head_dim + 2) * sizeof(float);
}

template <typename T, int NQMAX>
static void launch_attention_t(cudaStream_t st, const AttnGeom &g, const float *q, const void *k_cache,
                               const void *v_cache, const uint32_t *page_table, uint32_t page_tokens,
                               uint64_t cache_slot, uint32_t m, uint32_t splits, float *ws) {
    const size_t smem = (size_t)NQMAX * g.head_dim * 4 + (size_t)NQMAX * kAttnTile * 4 + 3 * NQMAX * 4 +
                        (size_t)kAttnTile * (g.head_dim + 16 / sizeof(T)) * sizeof(T) + 16;
    // the attribute belongs to the device, not to the process: once per device
    static thread_local unsigned long long attr_devices = 0;
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 64 && !(attr_devices >> dev & 1ull) &&
        cudaFuncSetAttribute(k_attention<T, NQMAX>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024) ==
            cudaSuccess)
        attr_devices |= 1ull << dev;
    launch_pdl(k_attention<T, NQMAX>, dim3(g.kv_heads * splits), dim3(kAttnThreads), smem, st, 
        g, q, (const T *)k_cache, (const T *)v_cache, page_table, page_tokens, cache_slot, (int)m, splits, ws);
}

void launch_attention(cudaStream_t st, const AttnGeom &g, const float *q, const float *gate,
                      const void *k_cache, const void *v_cache, int kv_bf16, const uint32_t *page_table,
                      uint32_t page_tokens, uint64_t cache_slot, uint32_t m, uint32_t splits, float *workspace,
                      const MvIn &next) {
    const uint32_t nq = g.q_heads / g.kv_heads * m;
    if (kv_bf16 && g.head_dim == kFaHd && nq <= 32) {
        const size_t smem1 = 2 * 32 * kFaStride * 2 + (size_t)fa_buffers(1) * 2 * kFaTile * kFaStride * 2;
        const size_t smem2 = 2 * 32 * kFaStride * 2 + (size_t)fa_buffers(2) * 2 * kFaTile * kFaHd * 2;
        static thread_local unsigned long long attr_devices = 0;  // per device, like above
        int dev = 0;
        cudaGetDevice(&dev);
        if (dev < 64 && !(attr_devices >> dev & 1ull) &&
            cudaFuncSetAttribute(k_attention_mma<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem1) ==
                cudaSuccess &&
            cudaFuncSetAttribute(k_attention_mma<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem2) ==
                cudaSuccess)
            attr_devices |= 1ull << dev;
        if (nq <= 16)
            launch_pdl(k_attention_mma<1>, dim3(g.kv_heads * splits), dim3(128), smem1, st, 
                g, q, (const __nv_bfloat16 *)k_cache, (const __nv_bfloat16 *)v_cache, page_table, page_tokens,
                cache_slot, (int)m, splits, workspace);
        else
            launch_pdl(k_attention_mma<2>, dim3(g.kv_heads * splits), dim3(256), smem2, st, 
                g, q, (const __nv_bfloat16 *)k_cache, (const __nv_bfloat16 *)v_cache, page_table, page_tokens,
                cache_slot, (int)m, splits, workspace);
        launch_pdl(k_attn_combine_prep, dim3(m * g.q_heads), dim3(g.head_dim), 0, st, g, workspace, gate, (int)m, splits,
                   next);
        return;
    }
#define CTOX_ATTN(T)                                                                                        \
    do {                                                                                                    \
        if (nq <= 8)                                                                                        \
            launch_attention_t<T, 8>(st, g, q, k_cache, v_cache, page_table, page_tokens, cache_slot, m,    \
                                     splits, workspace);                                                    \
        else if (nq <= 24)                                                                                  \
            launch_attention_t<T, 24>(st, g, q, k_cache, v_cache, page_table, page_tokens, cache_slot, m,   \
                                      splits, workspace);                                                   \
        else                                                                                                \
            launch_attention_t<T, 48>(st, g, q, k_cache, v_cache, page_table, page_tokens, cache_slot, m,   \
                                      splits, workspace);                                                   \
    } while (0)
    if (kv_bf16)
        CTOX_ATTN(__nv_bfloat16);
    else
        CTOX_ATTN(float);
#undef CTOX_ATTN
    launch_pdl(k_attn_combine_prep, dim3(m * g.q_heads), dim3(g.head_dim), 0, st, g, workspace, gate, (int)m, splits, next);
}

}  // namespace ctox
