// Writing activations in the fragment form the streaming matvec consumes.
//
// Every kernel that produces the input of a matvec (norms, SwiGLU, gates ...)
// ends with prep_block(): 16 consecutive lanes hold one 64-column block, four
// consecutive columns each, already multiplied by s_in. The block is scaled by
// a power of two so that its maximum lies in [2^E, 2^(E+1)), split as fp16
// hi + lo, multiplied by the column's power of two (layout.cuh) and stored as
//   xfrag[block][half 0|1][column n = 2*pos + (hi|lo)][lane quarter t][8 fp16]
//   meta[block][pos] = (-offset * code_scale * sum(x~), unit / (factor * code_scale)).
#pragma once
#include <cuda_fp16.h>

#include "layout.cuh"

namespace ctox {

// v: this lane's four columns (4*i .. 4*i+3 of block b), i = lane index within the 16-lane
// group, gmask = the shuffle mask of the group (0x0000ffff or 0xffff0000).
__device__ __forceinline__ void prep_block(const float (&v)[4], int i, unsigned gmask, int b, int m, int npos,
                                           int dt, uint8_t *__restrict__ xfrag, float2 *__restrict__ meta) {
    const int nc = 2 * npos;
    float amax = fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3])));
#pragma unroll
    for (int o = 1; o < 16; o <<= 1) amax = fmaxf(amax, __shfl_xor_sync(gmask, amax, o));
    const int ne = norm_exponent(dt);
    int e = (int)((__float_as_uint(amax) >> 23) & 0xff) - 127;
    if (!(amax > 0.f) || e > 127) e = ne;  // zero block or non-finite input: factor 1
    e = max(e, -100);
    const float f = __uint_as_float((uint32_t)(ne - e + 127) << 23);
    const float inv = __uint_as_float((uint32_t)(e - ne + 127) << 23);
    float sum = 0.f;
    uint8_t *base = xfrag + (size_t)b * nc * 128;
    const int t = i >> 2;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const int q = (i & 3) * 4 + j;
        const float sv = v[j] * f;
        const __half hi = __float2half_rn(sv);
        const __half lo = __float2half_rn(sv - __half2float(hi));
        sum += __half2float(hi) + __half2float(lo);
        const float mul = column_multiplier(dt, q);  // power of two: exact
        const int pos = inv_perm(dt, q);
        uint8_t *p = base + (pos >> 3) * (nc * 64) + t * 16 + (pos & 7) * 2;
        *reinterpret_cast<__half *>(p + (2 * m) * 64) = __float2half_rn(__half2float(hi) * mul);
        *reinterpret_cast<__half *>(p + (2 * m + 1) * 64) = __float2half_rn(__half2float(lo) * mul);
    }
#pragma unroll
    for (int o = 1; o < 16; o <<= 1) sum += __shfl_xor_sync(gmask, sum, o);
    if (i == 0)
        meta[b * npos + m] =
            make_float2(-code_offset(dt) * code_scale(dt) * sum, inv * code_unit(dt) / code_scale(dt));
}

// Pieces of row pair pr of a streamed matvec: the warps (warps_per_slice of them, over
// units = pairs * kst_s per slice) whose ranges [w * units / nw, (w + 1) * units / nw) meet the
// pair's units. Same formula as the host's table (matvec.cu, prepare_part); computing it saves the
// consumer a dependent load. 32-bit: the caller checks that (units + 1) * nw + units fits.
__device__ __forceinline__ uint32_t piece_count(uint32_t pr, uint32_t kst_s, uint32_t nw, uint32_t pairs) {
    const uint32_t units = pairs * kst_s;
    const uint32_t u_first = pr * kst_s, u_last = u_first + kst_s - 1;
    const uint32_t w_first = ((u_first + 1) * nw + units - 1) / units - 1;
    const uint32_t w_last = ((u_last + 1) * nw + units - 1) / units - 1;
    return w_last - w_first + 1;
}

// Sum of the raw partial sums the streaming kernel left for (row, pos), times s_out (+ bias):
// the value of one matvec output. pieces: [pair][slice].
__device__ __forceinline__ float matvec_output(const float *__restrict__ partial,
                                               const uint8_t *__restrict__ pieces, uint32_t slices,
                                               uint32_t max_pieces, const float *__restrict__ s_out,
                                               uint32_t row, uint32_t pos) {
    const uint32_t pr = row >> 5, rl = row & 31;
    float v = 0.f;
    for (uint32_t sl = 0; sl < slices; ++sl) {
        const float *base = partial + ((size_t)pr * slices + sl) * max_pieces * (32 * 8) + pos * 32 + rl;
        const uint32_t n = pieces[pr * slices + sl];
        for (uint32_t q = 0; q < n; ++q) v += base[q * (32 * 8)];
    }
    return s_out ? v * s_out[row] : v;
}

// The same value with the piece count computed (n pieces in every slice) and the loads of up to
// eight pieces issued before the first addition: one trip to L2 instead of one per piece plus the
// table lookup. Same order of additions.
__device__ __forceinline__ float matvec_output_n(const float *__restrict__ partial, uint32_t n, uint32_t slices,
                                                 uint32_t max_pieces, const float *__restrict__ s_out,
                                                 uint32_t row, uint32_t pos) {
    const uint32_t pr = row >> 5, rl = row & 31;
    const float *first = partial + (size_t)pr * slices * max_pieces * (32 * 8) + pos * 32 + rl;
    const float so = s_out ? s_out[row] : 1.0f;
    const uint32_t total = slices * n;
    float v = 0.f;
    uint32_t sl = 0, q = 0;
    for (uint32_t k0 = 0; k0 < total; k0 += 8) {
        float buf[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            buf[j] = 0.f;
            if (k0 + j < total) {
                buf[j] = first[((size_t)sl * max_pieces + q) * (32 * 8)];
                if (++q == n) {
                    q = 0;
                    ++sl;
                }
            }
        }
#pragma unroll
        for (int j = 0; j < 8; ++j)
            if (k0 + j < total) v += buf[j];
    }
    return s_out ? v * so : v;
}

}  // namespace ctox
