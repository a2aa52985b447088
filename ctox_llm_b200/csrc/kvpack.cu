// K/V rows as Q4_B64 / Q2_B64 blocks: the pieces of the reference's paged KV cache policy
// (kv_cache.rs:22-73: QuantizedKvToken::quantize / dequantize / requantize; quant.rs:74-105 and
// 144-168 for the two block quantizers; the reference's CUDA kernels for the same steps are
// ctox_pack_paged_kv_q4_f32_sm86 and ctox_demote_paged_kv_q4_to_q2_sm86, kernels/cuda/
// q2q4_fused_matvec_sm86.cu:1675-1835). One warp per 64-value block, two values per lane; every
// operation is the reference's own (IEEE division, a separate multiply and add, round half away
// from zero, binary16 scale rounded to nearest even), so the bytes equal the scalar code's.
#include <cuda_fp16.h>

#include "common.cuh"

namespace ctox {
namespace {

constexpr int kWarpsPerCta = 8;

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// quant.rs:144-168. lane l holds values 2l, 2l+1 and writes code byte l.
__device__ __forceinline__ void q4_quantize_block(float v0, float v1, uint8_t *out, uint32_t lane, int32_t *error_flag) {
    if (!isfinite(v0) || !isfinite(v1)) atomicExch(error_flag, DEV_ERR_NONFINITE_VALUE);
    const float scale = warp_max(fmaxf(fabsf(v0), fabsf(v1)));
    uint32_t byte = 0;
    if (scale != 0.0f) {
        const float in[2] = {v0, v1};
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            float n = __fdiv_rn(in[j], scale);
            n = fminf(fmaxf(n, -1.0f), 1.0f);
            float r = roundf(__fadd_rn(__fmul_rn(n, 7.5f), 7.5f));  // f32::round: half away from zero
            r = fminf(fmaxf(r, 0.0f), 15.0f);
            byte |= (uint32_t)r << (4 * j);
        }
    }
    out[2 + lane] = (uint8_t)byte;
    if (lane == 0) {
        // block strides (34 and 18 bytes) and bases are even: the little-endian scale is one 16-bit store
        *reinterpret_cast<__half *>(out) = __float2half_rn(scale);
    }
}

__global__ void __launch_bounds__(kWarpsPerCta * 32) k_kv_pack_q4(const float *__restrict__ values, uint64_t n_blocks,
                                                                  uint8_t *__restrict__ out, int32_t *error_flag) {
    pdl_launch();
    pdl_wait();
    const uint32_t lane = threadIdx.x & 31;
    const uint64_t stride = (uint64_t)gridDim.x * kWarpsPerCta;
    for (uint64_t b = (uint64_t)blockIdx.x * kWarpsPerCta + (threadIdx.x >> 5); b < n_blocks; b += stride) {
        const float2 v = *reinterpret_cast<const float2 *>(values + b * 64 + 2 * lane);
        q4_quantize_block(v.x, v.y, out + b * 34, lane, error_flag);
    }
}

__device__ __forceinline__ float block_scale_f32(const uint8_t *block) {
    return __half2float(__ushort_as_half((unsigned short)(block[0] | (block[1] << 8))));
}

// Q4 block -> values (quant.rs:170-175), then Q2Block64::quantize of them (quant.rs:74-105): what
// QuantizedKvToken::requantize does to every block of a page that leaves the recent window.
__global__ void __launch_bounds__(kWarpsPerCta * 32) k_kv_demote_q4_to_q2(const uint8_t *__restrict__ q4,
                                                                          uint64_t n_blocks,
                                                                          uint8_t *__restrict__ q2,
                                                                          int32_t *error_flag) {
    pdl_launch();
    pdl_wait();
    const uint32_t lane = threadIdx.x & 31;
    const uint64_t stride = (uint64_t)gridDim.x * kWarpsPerCta;
    for (uint64_t b = (uint64_t)blockIdx.x * kWarpsPerCta + (threadIdx.x >> 5); b < n_blocks; b += stride) {
    const uint8_t *in = q4 + b * 34;
    const float s4 = block_scale_f32(in);
    if (!isfinite(s4)) atomicExch(error_flag, DEV_ERR_NONFINITE_SCALE);
    const uint32_t byte = in[2 + lane];
    float v[2];
#pragma unroll
    for (int j = 0; j < 2; ++j) {
        const float code = (float)((byte >> (4 * j)) & 0xfu);
        v[j] = __fmul_rn(s4, __fdiv_rn(__fsub_rn(code, 7.5f), 7.5f));
    }
    const float scale = warp_max(fmaxf(fabsf(v[0]), fabsf(v[1])));
    uint32_t pair = 0;  // two 2-bit codes: values 2 * lane and 2 * lane + 1
    if (scale != 0.0f) {
        const float third = __fdiv_rn(1.0f, 3.0f);
        const float book[4] = {-1.0f, -third, third, 1.0f};  // -1.0 / 3.0 is the negation of 1.0 / 3.0
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            const float n = __fdiv_rn(v[j], scale);
            uint32_t best = 0;
            float best_d = fabsf(__fsub_rn(n, book[0]));
#pragma unroll
            for (uint32_t c = 1; c < 4; ++c) {  // Iterator::min_by keeps the first minimum
                const float d = fabsf(__fsub_rn(n, book[c]));
                if (d < best_d) {
                    best = c;
                    best_d = d;
                }
            }
            pair |= best << (2 * j);
        }
    }
    // byte j of the codes holds values 4j .. 4j + 3: lanes 2j (low nibble) and 2j + 1 (high)
    const uint32_t other = __shfl_down_sync(0xffffffffu, pair, 1);
    uint8_t *out = q2 + b * 18;
    if ((lane & 1) == 0) out[2 + (lane >> 1)] = (uint8_t)(pair | (other << 4));
    if (lane == 0) {
        // block strides (34 and 18 bytes) and bases are even: the little-endian scale is one 16-bit store
        *reinterpret_cast<__half *>(out) = __float2half_rn(scale);
    }
    }
}

// Block decode (quant.rs:107-115, 170-175).
__global__ void __launch_bounds__(kWarpsPerCta * 32) k_kv_unpack(const uint8_t *__restrict__ bytes, int q4,
                                                                 uint64_t n_blocks, float *__restrict__ values,
                                                                 int32_t *error_flag) {
    pdl_launch();
    pdl_wait();
    const uint32_t lane = threadIdx.x & 31;
    const uint64_t stride = (uint64_t)gridDim.x * kWarpsPerCta;
    for (uint64_t b = (uint64_t)blockIdx.x * kWarpsPerCta + (threadIdx.x >> 5); b < n_blocks; b += stride) {
    const uint8_t *in = bytes + b * (q4 ? 34 : 18);
    const float scale = block_scale_f32(in);
    if (!isfinite(scale)) atomicExch(error_flag, DEV_ERR_NONFINITE_SCALE);
    float2 v;
    if (q4) {
        const uint32_t byte = in[2 + lane];
        v.x = __fmul_rn(scale, __fdiv_rn(__fsub_rn((float)(byte & 0xfu), 7.5f), 7.5f));
        v.y = __fmul_rn(scale, __fdiv_rn(__fsub_rn((float)(byte >> 4), 7.5f), 7.5f));
    } else {
        const float third = __fdiv_rn(1.0f, 3.0f);
        const float book[4] = {-1.0f, -third, third, 1.0f};
        const uint32_t byte = in[2 + (lane >> 1)] >> (4 * (lane & 1));
        v.x = __fmul_rn(scale, book[byte & 3u]);
        v.y = __fmul_rn(scale, book[(byte >> 2) & 3u]);
    }
    *reinterpret_cast<float2 *>(values + b * 64 + 2 * lane) = v;
    }
}

// 8 CTAs of 8 warps per SM (full occupancy); each warp walks the blocks with the grid's stride.
unsigned kv_grid(const ctox_ctx *ctx, uint64_t n_blocks) {
    const uint64_t want = (n_blocks + kWarpsPerCta - 1) / kWarpsPerCta, cap = (uint64_t)ctx->sm_count * 8;
    return (unsigned)(want < cap ? want : cap);
}

ctox_status check(ctox_ctx *ctx, const void *a, const void *b, uint64_t n_blocks, const char *what) {
    if (!ctx) return CTOX_INVALID_STATE;
    if (!a || !b) return fail(ctx, CTOX_SHAPE, "%s: null device pointer", what);
    if (n_blocks == 0 || n_blocks > (1ull << 34)) return fail(ctx, CTOX_SHAPE, "%s: %llu blocks", what, (unsigned long long)n_blocks);
    return CTOX_OK;
}

}  // namespace
}  // namespace ctox

using namespace ctox;

extern "C" {

ctox_status ctox_kv_pack_q4(ctox_ctx *ctx, const float *values, uint64_t n_blocks, uint8_t *q4_bytes) {
    ctox_status rc = check(ctx, values, q4_bytes, n_blocks, "kv pack");
    if (rc) return rc;
    CTOX_CUDA(ctx, cudaSetDevice(ctx->device));
    launch_pdl(k_kv_pack_q4, dim3(kv_grid(ctx, n_blocks)), dim3(kWarpsPerCta * 32), 0,
               ctx->stream, values, n_blocks, q4_bytes, ctx->dev_error);
    CTOX_CUDA(ctx, cudaGetLastError());
    return CTOX_OK;
}

ctox_status ctox_kv_demote_q4_to_q2(ctox_ctx *ctx, const uint8_t *q4_bytes, uint64_t n_blocks, uint8_t *q2_bytes) {
    ctox_status rc = check(ctx, q4_bytes, q2_bytes, n_blocks, "kv demote");
    if (rc) return rc;
    CTOX_CUDA(ctx, cudaSetDevice(ctx->device));
    launch_pdl(k_kv_demote_q4_to_q2, dim3(kv_grid(ctx, n_blocks)),
               dim3(kWarpsPerCta * 32), 0, ctx->stream, q4_bytes, n_blocks, q2_bytes, ctx->dev_error);
    CTOX_CUDA(ctx, cudaGetLastError());
    return CTOX_OK;
}

ctox_status ctox_kv_unpack(ctox_ctx *ctx, uint32_t dtype, const uint8_t *bytes, uint64_t n_blocks, float *values) {
    ctox_status rc = check(ctx, bytes, values, n_blocks, "kv unpack");
    if (rc) return rc;
    if (dtype != CTOX_Q2B64 && dtype != CTOX_Q4B64) return fail(ctx, CTOX_UNSUPPORTED_DTYPE, "kv unpack: dtype %u", dtype);
    CTOX_CUDA(ctx, cudaSetDevice(ctx->device));
    launch_pdl(k_kv_unpack, dim3(kv_grid(ctx, n_blocks)), dim3(kWarpsPerCta * 32), 0,
               ctx->stream, bytes, dtype == CTOX_Q4B64 ? 1 : 0, n_blocks, values, ctx->dev_error);
    CTOX_CUDA(ctx, cudaGetLastError());
    return CTOX_OK;
}

}  // extern "C"
