// Device helpers of the selection kernels: IEEE total-order keys, Philox4x32-10,
// a transcendental-free logarithm, and the record the acceptance kernel writes.
#pragma once
#include <cstdint>

namespace ctox {

// f32::total_cmp as an unsigned key: larger key == greater under the total order
// (sampler.rs:76-82 uses max_by(total_cmp); the CUDA candidate builds the same
// key at kernels/cuda/q2q4_fused_matvec_sm86.cu:2587-2596).
__device__ __forceinline__ uint32_t total_order_key(float v) {
    const uint32_t b = __float_as_uint(v);
    return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}
// (key, index) packed so that an unsigned max picks the greatest value and, among
// equal values, the LATER index, which is what Iterator::max_by returns.
__device__ __forceinline__ unsigned long long pack_key_index(float v, uint32_t index) {
    return ((unsigned long long)total_order_key(v) << 32) | index;
}

// Philox4x32-10 (Salmon et al., SC'11), counter-based: no state to carry.
__device__ __forceinline__ uint4 philox4x32_10(uint4 ctr, uint2 key) {
#pragma unroll
    for (int round = 0; round < 10; ++round) {
        const uint32_t hi0 = __umulhi(0xD2511F53u, ctr.x), lo0 = 0xD2511F53u * ctr.x;
        const uint32_t hi1 = __umulhi(0xCD9E8D57u, ctr.z), lo1 = 0xCD9E8D57u * ctr.z;
        ctr = make_uint4(hi1 ^ ctr.y ^ key.x, lo1, hi0 ^ ctr.w ^ key.y, lo0);
        key.x += 0x9E3779B9u;
        key.y += 0xBB67AE85u;
    }
    return ctr;
}

// Natural logarithm from +, *, / and bit operations only (each correctly rounded,
// nothing contracted), so that host and device agree bit for bit.
// x = m * 2^e with m in [sqrt(1/2), sqrt(2)); ln m = 2 atanh((m-1)/(m+1)).
__device__ __forceinline__ float det_ln(float x) {
    const uint32_t bits = __float_as_uint(x);
    int e = (int)(bits >> 23) - 127;
    float m = __uint_as_float((bits & 0x7fffffu) | 0x3f800000u);
    if (m > 1.41421356f) {
        m = __fmul_rn(m, 0.5f);
        e += 1;
    }
    const float s = __fdiv_rn(__fadd_rn(m, -1.0f), __fadd_rn(m, 1.0f));
    const float s2 = __fmul_rn(s, s);
    float poly = 0.11111111f;
    poly = __fadd_rn(__fmul_rn(poly, s2), 0.14285715f);
    poly = __fadd_rn(__fmul_rn(poly, s2), 0.2f);
    poly = __fadd_rn(__fmul_rn(poly, s2), 0.33333334f);
    poly = __fadd_rn(__fmul_rn(poly, s2), 1.0f);
    const float ln_m = __fmul_rn(__fmul_rn(2.0f, s), poly);
    return __fadd_rn(__fmul_rn((float)e, 0.69314718f), ln_m);
}

// Standard Gumbel noise -ln(-ln u), u in (0, 1) from the top 24 bits.
__device__ __forceinline__ float gumbel_from_bits(uint32_t bits) {
    const float u = __fmul_rn(__fadd_rn((float)(bits >> 8), 0.5f), 1.0f / 16777216.0f);
    return -det_ln(-det_ln(u));
}
// Counter layout: (token / 4 or 0xffffffff, node, step lo, step hi), key = seed.
__device__ __forceinline__ float gumbel_noise(uint64_t seed, uint64_t step, uint32_t node, uint32_t token) {
    const uint4 r = philox4x32_10(make_uint4(token >> 2, node, (uint32_t)step, (uint32_t)(step >> 32)),
                                  make_uint2((uint32_t)seed, (uint32_t)(seed >> 32)));
    const uint32_t w = (token & 3u) == 0 ? r.x : (token & 3u) == 1 ? r.y : (token & 3u) == 2 ? r.z : r.w;
    return gumbel_from_bits(w);
}
__device__ __forceinline__ float accept_draw(uint64_t seed, uint64_t step, uint32_t node) {
    const uint4 r = philox4x32_10(make_uint4(0xffffffffu, node, (uint32_t)step, (uint32_t)(step >> 32)),
                                  make_uint2((uint32_t)seed, (uint32_t)(seed >> 32)));
    return (float)(r.x >> 8) * (1.0f / 16777216.0f);
}

}  // namespace ctox
