// Fused Q2_B64 / Q4_B64 dequantize-matvec for sm_100a, decode (1 position) and
// verify (2..16 positions) forms.
//
//   y[m][r] = act((sum_c W[r][c] * x[m][c] * s_in[c] + bias[r]) * s_out[r])
//
// Reference semantics: CpuBackend::fused_matvec (backend/cpu.rs:228-310,432-442),
// CUDA candidate kernels kernels/cuda/q2q4_fused_matvec_sm86.cu:87-195. The
// reference kernel is one warp per row with byte loads and scalar FMAs and is
// instruction-bound; this one is built around HBM bandwidth:
//
//  * weights are repacked once (layout.cuh) so that every lane reads its codes
//    as one 16-byte vector and the bytes of any contiguous work range are one
//    contiguous byte range;
//  * each warp owns a private ring of shared-memory stages that it fills with
//    bulk async copies (cp.async.bulk + mbarrier, no cross-warp barrier in the
//    steady state), so ~140 KB per SM are in flight;
//  * the work list (16-row x 256-column super-tiles) is split evenly over all
//    warps of a persistent grid (stream-K); a row tile cut by a split is summed
//    from per-piece partials in fixed piece order by whichever warp arrives
//    last, so the result does not depend on timing;
//  * codes become fp16 operands with one AND per two codes: the masked code
//    bits, read as an fp16 subnormal, are exactly code * 2^(p-24), and the
//    dot products run on mma.sync.m16n8k16 with fp32 accumulation. The
//    activation is split into fp16 hi + lo parts (two B columns per position)
//    after a per-block power of two normalisation, which keeps ~22 bits of
//    each activation; the code offset (7.5 / 1.5) enters through the
//    accumulator's initial value -offset * sum(x).
#include "common.cuh"
#include "layout.cuh"
#include "matvec.cuh"
#include "prep.cuh"

#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <cmath>
#include <cstdlib>
#include <vector>

namespace ctox {


// ------------------------------------------------------------------ PTX helpers
__device__ __forceinline__ uint32_t smem_u32(const void *p) {
    return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void fence_barrier_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ bool mbar_test(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
__device__ __forceinline__ bool mbar_try(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait: gives up after ~0.3 s so that a lost copy can never hang the GPU.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
    if (mbar_test(bar, parity)) return true;
    const long long t0 = clock64();
    for (int i = 0; i < (1 << 24); ++i) {
        if (mbar_try(bar, parity)) return true;  // blocks for a bounded, hardware-defined time
        if ((i & 255) == 255 && clock64() - t0 > 600000000ll) break;
    }
    return false;
}
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void *src, uint32_t bytes,
                                         uint32_t bar) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
        ::"r"(dst), "l"(src), "r"(bytes), "r"(bar)
        : "memory");
}
__device__ __forceinline__ void mma_f16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                        uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
        "{%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// d = a * b + (c0, c1, c0, c1): first MMA of a chain, no register copies for the initial value
__device__ __forceinline__ void mma_f16_init(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                             uint32_t a3, uint32_t b0, uint32_t b1, float c0, float c1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
        "{%8,%9}, {%10,%11,%10,%11};"
        : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(c0), "f"(c1));
}
// Four f16 values packed in two 32-bit words -> four floats, in registers.
__device__ __forceinline__ void h2x2_to_f32(uint32_t a, uint32_t b, float (&out)[4]) {
    asm("{\n\t.reg .b16 l0, h0, l1, h1;\n\t"
        "mov.b32 {l0, h0}, %4;\n\tmov.b32 {l1, h1}, %5;\n\t"
        "cvt.f32.f16 %0, l0;\n\tcvt.f32.f16 %1, h0;\n\tcvt.f32.f16 %2, l1;\n\tcvt.f32.f16 %3, h1;\n\t}"
        : "=f"(out[0]), "=f"(out[1]), "=f"(out[2]), "=f"(out[3])
        : "r"(a), "r"(b));
}
__device__ __forceinline__ uint4 lds128(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "r"(addr));
    return v;
}
__device__ __forceinline__ float2 lds64f(uint32_t addr) {
    float2 v;
    asm volatile("ld.shared.v2.f32 {%0,%1}, [%2];" : "=f"(v.x), "=f"(v.y) : "r"(addr));
    return v;
}

// ------------------------------------------------------------------ repack
// One warp per super-tile; lane (g, t) gathers its own code bytes.
template <int DT>
__global__ void k_repack(const uint8_t *__restrict__ canon, uint8_t *__restrict__ prep,
                         uint32_t rows, uint32_t blocks, uint32_t pairs, uint32_t kst_s, uint32_t slices,
                         int32_t *error_flag) {
    pdl_launch();
    pdl_wait();
    using F = Fmt<DT>;
    const uint64_t s = (uint64_t)blockIdx.x * (blockDim.x / 32) + threadIdx.x / 32;
    if (s >= (uint64_t)slices * pairs * kst_s * 2) return;
    const uint32_t lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    // s = (((slice * pairs + pair) * kst_s) + ks_in_slice) * 2 + tile_of_pair
    const uint64_t per_slice = (uint64_t)pairs * kst_s * 2;
    const uint32_t slice = (uint32_t)(s / per_slice);
    const uint64_t rem = s % per_slice;
    const uint32_t rt = (uint32_t)(rem / (2ull * kst_s)) * 2 + (uint32_t)(rem & 1);
    const uint32_t ks = slice * kst_s + (uint32_t)((rem >> 1) % kst_s);
    uint8_t *out = prep + s * F::kSuperTileBytes;
    const uint64_t row_bytes = (uint64_t)blocks * F::kBlockBytes;
    // scales: lane t == 0 writes the 8 halfs of (row g, row g+8) x 4 blocks
    if (t == 0) {
        uint16_t sc[8];
        for (int hh = 0; hh < 2; ++hh)
            for (int j = 0; j < 4; ++j) {
                uint32_t row = rt * 16 + g + 8 * hh, blk = ks * 4 + j;
                uint16_t v = 0;
                if (row < rows && blk < blocks) {
                    const uint8_t *b = canon + row * row_bytes + (uint64_t)blk * F::kBlockBytes;
                    v = (uint16_t)(b[0] | (b[1] << 8));
                    if ((v & 0x7c00u) == 0x7c00u) atomicExch(error_flag, DEV_ERR_NONFINITE_SCALE);
                }
                sc[hh * 4 + j] = v;
            }
        uint4 pk;
        pk.x = sc[0] | ((uint32_t)sc[1] << 16);
        pk.y = sc[2] | ((uint32_t)sc[3] << 16);
        pk.z = sc[4] | ((uint32_t)sc[5] << 16);
        pk.w = sc[6] | ((uint32_t)sc[7] << 16);
        *reinterpret_cast<uint4 *>(out + g * 16) = pk;
    }
    constexpr int kPerLane = F::kCodeBytes / 4;  // code bytes per (row, block, lane quarter)
    for (int j = 0; j < 4; ++j) {
        for (int hh = 0; hh < 2; ++hh) {
            uint32_t row = rt * 16 + g + 8 * hh, blk = ks * 4 + j;
            uint8_t bytes[kPerLane];
            for (int i = 0; i < kPerLane; ++i) bytes[i] = 0;
            if (row < rows && blk < blocks) {
                const uint8_t *b =
                    canon + row * row_bytes + (uint64_t)blk * F::kBlockBytes + 2 + t * kPerLane;
                for (int i = 0; i < kPerLane; ++i) bytes[i] = b[i];
            }
            uint8_t *dst;
            if (DT == 1)  // Q4: one 16 B vector per block: [row g: 8 B][row g+8: 8 B]
                dst = out + kScaleBytes + j * 512 + lane * 16 + hh * 8;
            else  // Q2: one vector per block pair: [g,b0][g+8,b0][g,b1][g+8,b1], 4 B each
                dst = out + kScaleBytes + (j >> 1) * 512 + lane * 16 + (j & 1) * 8 + hh * 4;
            for (int i = 0; i < kPerLane; ++i) dst[i] = bytes[i];
        }
    }
}

// ------------------------------------------------------------------ activation preparation
// Turns positions x columns activations into the B-operand fragments of the
// streaming kernel: x' = x * s_in, per 64-column block scaled by a power of two
// so that the block maximum lies in [2^E, 2^(E+1)) (E = norm_exponent), split
// as fp16 hi + lo and pre-multiplied by the column's power of two.
// Layout per block: [half 0|1][column n = 2*pos + (hi|lo)][lane quarter t][8 fp16].
// meta[block][pos] = (-offset * code_scale * sum of the block's x~, unit / (scale factor * code_scale)).
__global__ void k_prep_x(const void *__restrict__ x, int x_is_bf16, long long x_stride,
                         const float *__restrict__ s_in, int columns, int blocks_padded, int npos,
                         int dt, uint8_t *__restrict__ xfrag, float2 *__restrict__ meta) {
    pdl_launch();
    pdl_wait();
    const int gid = (blockIdx.x * blockDim.x + threadIdx.x) >> 4;
    const int i = threadIdx.x & 15;
    if (gid >= blocks_padded * npos) return;  // whole 16-lane groups leave together
    const int b = gid / npos, m = gid % npos;
    float v[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        int k = b * 64 + i * 4 + j;
        float xv = 0.f;
        if (k < columns) {
            if (x_is_bf16)
                xv = __bfloat162float(((const __nv_bfloat16 *)x)[(long long)m * x_stride + k]);
            else
                xv = ((const float *)x)[(long long)m * x_stride + k];
            if (s_in) xv *= s_in[k];
        }
        v[j] = xv;
    }
    // the 16 lanes of a group are lanes 0-15 or 16-31 of a warp
    const unsigned gmask = (threadIdx.x & 16) ? 0xffff0000u : 0x0000ffffu;
    prep_block(v, i, gmask, b, m, npos, dt, xfrag, meta);
}

// ------------------------------------------------------------------ streaming kernel
struct StreamParams {
    const uint8_t *wprep;
    const uint8_t *xfrag;   // prepared activations (k_prep_x), [block][half][column][quarter][8 fp16]
    const float2 *meta;     // [block][position]
    float *partial;         // [pair][slice][piece][kMaxPosPerPass][32 rows] raw sums
    int32_t *error_flag;
    uint32_t pairs;            // 32-row tile pairs
    uint32_t kst_s;            // 256-column super-tiles per column slice
    uint32_t slices;           // column slices (each CTA works inside one slice)
    uint32_t ctas_per_slice;
    uint32_t warps_per_slice;  // warps that take work (<= units per slice)
    uint32_t npos, max_pieces;
};

// Four MMAs of one 16-row x 64-column block; cw = this lane's code vector(s).
template <int DT>
__device__ __forceinline__ void block_mma(float (&c)[4], uint32_t w0, uint32_t w0h, uint32_t w1,
                                          uint32_t w1h, const uint4 &bA, const uint4 &bB, float c0) {
    // w0/w1: first/second code word of row g, w0h/w1h: of row g+8 (Q2 uses w0, w0h only)
    if (DT == 1) {
        constexpr uint32_t kLo = 0x000f000fu, kHi = 0x00f000f0u;
        const uint32_t t0 = w0 >> 8, t0h = w0h >> 8, t1 = w1 >> 8, t1h = w1h >> 8;
        mma_f16_init(c, w0 & kLo, w0h & kLo, w0 & kHi, w0h & kHi, bA.x, bA.y, c0, 0.f);
        mma_f16(c, t0 & kLo, t0h & kLo, t0 & kHi, t0h & kHi, bA.z, bA.w);
        mma_f16(c, w1 & kLo, w1h & kLo, w1 & kHi, w1h & kHi, bB.x, bB.y);
        mma_f16(c, t1 & kLo, t1h & kLo, t1 & kHi, t1h & kHi, bB.z, bB.w);
    } else {
        const uint32_t t = w0 >> 10, th = w0h >> 10;
        mma_f16_init(c, w0 & 0x00030003u, w0h & 0x00030003u, w0 & 0x000c000cu, w0h & 0x000c000cu, bA.x,
                     bA.y, c0, 0.f);
        mma_f16(c, w0 & 0x00300030u, w0h & 0x00300030u, w0 & 0x00c000c0u, w0h & 0x00c000c0u, bA.z, bA.w);
        mma_f16(c, w0 & 0x03000300u, w0h & 0x03000300u, t & 0x00030003u, th & 0x00030003u, bB.x, bB.y);
        mma_f16(c, t & 0x000c000cu, th & 0x000c000cu, t & 0x00300030u, th & 0x00300030u, bB.z, bB.w);
    }
}

template <int DT, int WARPS, int STAGES, int NT>
__global__ void __launch_bounds__(WARPS * 32, 1) k_matvec_stream(const StreamParams p) {
    pdl_launch();
    using F = Fmt<DT>;
    constexpr uint32_t kST = F::kSuperTileBytes;
    constexpr uint32_t kUnitBytes = 2 * kST;                      // one tile pair
    constexpr uint32_t kChunkBytes = F::kChunkPairs * kUnitBytes;  // one bulk copy
    extern __shared__ __align__(128) uint8_t smem[];
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const uint32_t nc = 2 * p.npos;
    const uint32_t slice_blocks = p.kst_s * 4;
    const uint32_t xfrag_bytes = slice_blocks * nc * 128, meta_bytes = slice_blocks * p.npos * 8;

    uint8_t *stages = smem;
    uint8_t *xs = smem + WARPS * STAGES * kChunkBytes;
    uint8_t *ms = xs + xfrag_bytes;
    uint8_t *zero = ms + ((meta_bytes + 15) & ~15u);  // 16 zero bytes for lanes without operands
    uint64_t *bars = reinterpret_cast<uint64_t *>(zero + 16);
    const uint32_t xbar = smem_u32(&bars[WARPS * STAGES]);
    const uint32_t my_bars = smem_u32(&bars[warp * STAGES]);
    const uint32_t my_stage = smem_u32(stages + warp * STAGES * kChunkBytes);

    // This CTA works inside one column slice; its warps split the slice's units
    // (tile pair x super-tile of the slice, pair-major) evenly: [beg, end).
    const uint32_t slice = blockIdx.x / p.ctas_per_slice;
    const uint32_t lw = (blockIdx.x % p.ctas_per_slice) * WARPS + warp;
    const uint64_t total = (uint64_t)p.pairs * p.kst_s;
    const bool active = lw < p.warps_per_slice;
    uint64_t beg = 0, end = 0;
    if (active) {
        beg = ((uint64_t)lw * total) / p.warps_per_slice;
        end = ((uint64_t)(lw + 1) * total) / p.warps_per_slice;
    }
    const uint32_t nchunks = (uint32_t)((end - beg + F::kChunkPairs - 1) / F::kChunkPairs);
    const uint8_t *wsrc = p.wprep + (uint64_t)slice * total * kUnitBytes;

    if (threadIdx.x == 0) {
        mbar_init(xbar, 1);
        *reinterpret_cast<uint4 *>(zero) = make_uint4(0, 0, 0, 0);
    }
    if (lane == 0) {
        for (int s = 0; s < STAGES; ++s) mbar_init(my_bars + 8 * s, 1);
        fence_barrier_init();
        fence_proxy_async();
        // weights do not depend on the activations: start streaming at once
        for (uint32_t c = 0; c < (uint32_t)STAGES && c < nchunks; ++c) {
            const uint64_t u0 = beg + (uint64_t)c * F::kChunkPairs;
            const uint32_t n = (uint32_t)min((uint64_t)F::kChunkPairs, end - u0);
            mbar_expect_tx(my_bars + 8 * c, n * kUnitBytes);
            bulk_g2s(my_stage + c * kChunkBytes, wsrc + u0 * kUnitBytes, n * kUnitBytes, my_bars + 8 * c);
        }
    }
    __syncthreads();  // xbar and the zero bytes are initialised
    // Everything above touched only this matrix's weights, which nothing in the stream writes.
    // The activations come from the kernels before this one: wait for them here, with the first
    // STAGES chunks of every warp already on their way.
    pdl_wait();
    if (threadIdx.x == 0) {
        fence_proxy_async();
        mbar_expect_tx(xbar, xfrag_bytes + meta_bytes);
        const uint8_t *xsrc = p.xfrag + (size_t)slice * xfrag_bytes;
        uint32_t off = 0;
        while (off < xfrag_bytes) {
            const uint32_t n = min(xfrag_bytes - off, 32768u);
            bulk_g2s(smem_u32(xs) + off, xsrc + off, n, xbar);
            off += n;
        }
        bulk_g2s(smem_u32(ms), reinterpret_cast<const uint8_t *>(p.meta) + (size_t)slice * meta_bytes,
                 meta_bytes, xbar);
    }
    if (!active || nchunks == 0) return;  // warp 0 of every CTA is active and waits for xbar below
    bool ok = mbar_wait(xbar, 0);

    // lanes whose B column / position does not exist read zeros with stride 0
    uint32_t b_base[NT], b_stride[NT], b_half[NT], m_base[NT], m_stride[NT];
    bool has_m[NT];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
        const bool hb = 8 * nt + g < nc;
        has_m[nt] = 4 * nt + t < p.npos;
        b_stride[nt] = hb ? nc * 128 : 0;
        b_base[nt] = hb ? smem_u32(xs) + nt * 512 + lane * 16 : smem_u32(zero);
        b_half[nt] = hb ? nc * 64 : 0;
        m_stride[nt] = has_m[nt] ? p.npos * 8 : 0;
        m_base[nt] = has_m[nt] ? smem_u32(ms) + (4 * nt + t) * 8 : smem_u32(zero);
    }

    float acc[NT][8];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[nt][i] = 0.f;
    uint32_t cur_pair = (uint32_t)(beg / p.kst_s), cur_ks = (uint32_t)(beg % p.kst_s);

    const uint32_t rloc[4] = {g, g + 8, 16 + g, 24 + g};  // rows of this lane inside a pair
    // Raw sums go to the slot (pair, slice, piece): piece = rank of this warp among the
    // consecutive warps of the slice whose ranges intersect the pair. A pair that lies wholly
    // inside this warp's range has one piece; only the first and the last pair of a range can be
    // cut. The finish kernels add slices and pieces in index order, so the result does not
    // depend on timing and the stream needs no atomics, counters or fences.
    auto close_pair = [&](uint32_t pr, bool reached_end_of_pair) {
        uint32_t piece = 0;
        if ((uint64_t)pr * p.kst_s < beg || !reached_end_of_pair) {
            const uint64_t u_first = (uint64_t)pr * p.kst_s;
            const uint32_t w_first =
                (uint32_t)(((u_first + 1) * p.warps_per_slice + total - 1) / total - 1);
            piece = lw - w_first;
        }
        float *slot = p.partial + (((size_t)pr * p.slices + slice) * p.max_pieces + piece) *
                                      (kPairRows * kMaxPosPerPass);
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
            if (has_m[nt]) {  // hi + lo columns of position 4*nt + t
                float *col = slot + (4 * nt + t) * kPairRows;  // a slot is [position][32 rows]
                col[rloc[0]] = acc[nt][0] + acc[nt][1];
                col[rloc[1]] = acc[nt][2] + acc[nt][3];
                col[rloc[2]] = acc[nt][4] + acc[nt][5];
                col[rloc[3]] = acc[nt][6] + acc[nt][7];
            }
        }
    };

    uint32_t waited = 0;  // chunks whose barrier we have passed (for the drain on failure)
    for (uint32_t c = 0; c < nchunks && ok; ++c) {
        const uint32_t st = c % STAGES, parity = (c / STAGES) & 1;
        ok = mbar_wait(my_bars + 8 * st, parity);
        if (!ok) break;
        waited = c + 1;
        const uint64_t u0 = beg + (uint64_t)c * F::kChunkPairs;
        const uint32_t n = (uint32_t)min((uint64_t)F::kChunkPairs, end - u0);
        for (uint32_t i = 0; i < n; ++i) {
            if (cur_ks == p.kst_s) {  // crossed into the next tile pair
                close_pair(cur_pair, true);
#pragma unroll
                for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                    for (int k = 0; k < 8; ++k) acc[nt][k] = 0.f;
                ++cur_pair;
                cur_ks = 0;
            }
            const uint32_t b0 = (cur_ks++) * 4;
            const uint32_t tile0 = my_stage + st * kChunkBytes + i * kUnitBytes, tile1 = tile0 + kST;
            // scales of both tiles: rows g, g+8 (tile 0) and 16+g, 24+g (tile 1), blocks 0..3
            const uint4 sv0 = lds128(tile0 + g * 16), sv1 = lds128(tile1 + g * 16);
            // row r of the pair: two words = four f16 block scales (no address is taken of a register
            // array here: that would put it on the local-memory stack, a round trip per unit)
            float sc[4][4];
            h2x2_to_f32(sv0.x, sv0.y, sc[0]);
            h2x2_to_f32(sv0.z, sv0.w, sc[1]);
            h2x2_to_f32(sv1.x, sv1.y, sc[2]);
            h2x2_to_f32(sv1.z, sv1.w, sc[3]);
            uint4 q0 = make_uint4(0, 0, 0, 0), q1 = make_uint4(0, 0, 0, 0);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                uint32_t w0, w0h, w1, w1h, v0, v0h, v1, v1h;  // tile 0 / tile 1 code words
                if (DT == 1) {
                    const uint4 a0 = lds128(tile0 + kScaleBytes + j * 512 + lane * 16);
                    const uint4 a1 = lds128(tile1 + kScaleBytes + j * 512 + lane * 16);
                    w0 = a0.x, w0h = a0.z, w1 = a0.y, w1h = a0.w;
                    v0 = a1.x, v0h = a1.z, v1 = a1.y, v1h = a1.w;
                } else {
                    if ((j & 1) == 0) {
                        q0 = lds128(tile0 + kScaleBytes + (j >> 1) * 512 + lane * 16);
                        q1 = lds128(tile1 + kScaleBytes + (j >> 1) * 512 + lane * 16);
                    }
                    w0 = (j & 1) ? q0.z : q0.x, w0h = (j & 1) ? q0.w : q0.y, w1 = 0, w1h = 0;
                    v0 = (j & 1) ? q1.z : q1.x, v0h = (j & 1) ? q1.w : q1.y, v1 = 0, v1h = 0;
                }
#pragma unroll
                for (int nt = 0; nt < NT; ++nt) {
                    const uint32_t xb = b_base[nt] + (b0 + j) * b_stride[nt];
                    const uint4 bA = lds128(xb), bB = lds128(xb + b_half[nt]);
                    const float2 mt = lds64f(m_base[nt] + (b0 + j) * m_stride[nt]);
                    float c0[4], c1[4];
                    block_mma<DT>(c0, w0, w0h, w1, w1h, bA, bB, mt.x);
                    block_mma<DT>(c1, v0, v0h, v1, v1h, bA, bB, mt.x);
                    const float f0 = sc[0][j] * mt.y, f1 = sc[1][j] * mt.y;
                    const float f2 = sc[2][j] * mt.y, f3 = sc[3][j] * mt.y;
                    acc[nt][0] = fmaf(f0, c0[0], acc[nt][0]);
                    acc[nt][1] = fmaf(f0, c0[1], acc[nt][1]);
                    acc[nt][2] = fmaf(f1, c0[2], acc[nt][2]);
                    acc[nt][3] = fmaf(f1, c0[3], acc[nt][3]);
                    acc[nt][4] = fmaf(f2, c1[0], acc[nt][4]);
                    acc[nt][5] = fmaf(f2, c1[1], acc[nt][5]);
                    acc[nt][6] = fmaf(f3, c1[2], acc[nt][6]);
                    acc[nt][7] = fmaf(f3, c1[3], acc[nt][7]);
                }
            }
        }
        __syncwarp();
        if (lane == 0 && c + STAGES < nchunks) {
            // refill the stage we just drained
            const uint32_t cn = c + STAGES;
            const uint64_t un = beg + (uint64_t)cn * F::kChunkPairs;
            const uint32_t nn = (uint32_t)min((uint64_t)F::kChunkPairs, end - un);
            fence_proxy_async();
            mbar_expect_tx(my_bars + 8 * st, nn * kUnitBytes);
            bulk_g2s(my_stage + st * kChunkBytes, wsrc + un * kUnitBytes, nn * kUnitBytes, my_bars + 8 * st);
        }
    }
    if (!ok) {
        if (lane == 0) atomicExch(p.error_flag, DEV_ERR_WAIT_TIMEOUT);
        // let copies already issued into our stages land before the CTA can retire
        const uint32_t issued = min(nchunks, waited + (uint32_t)STAGES);
        for (uint32_t c = waited; c < issued; ++c)
            mbar_wait(my_bars + 8 * (c % STAGES), (c / STAGES) & 1);
        return;
    }
    close_pair(cur_pair, cur_ks == p.kst_s);
}

// y[pos][row] = act((sum over slices and pieces + bias[row]) * s_out[row]); one thread per (row, pos).
// pieces: [pair][slice] number of pieces.
__global__ void k_matvec_finish(const float *__restrict__ partial, const uint8_t *__restrict__ pieces,
                                const float *__restrict__ s_out, const float *__restrict__ bias,
                                float *__restrict__ y, long long y_stride, uint32_t rows, uint32_t npos,
                                uint32_t slices, uint32_t max_pieces, uint32_t activation) {
    pdl_launch();
    pdl_wait();
    const uint32_t idx = blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= rows * npos) return;
    const uint32_t row = idx / npos, pos = idx % npos;
    const uint32_t pr = row / kPairRows, rl = row % kPairRows;
    float v = 0.f;
    for (uint32_t sl = 0; sl < slices; ++sl) {
        const float *base = partial + ((size_t)pr * slices + sl) * max_pieces * (kPairRows * kMaxPosPerPass) +
                            pos * kPairRows + rl;
        const uint32_t n = pieces[pr * slices + sl];
        for (uint32_t q = 0; q < n; ++q) v += base[q * (kPairRows * kMaxPosPerPass)];
    }
    if (bias) v += bias[row];
    if (s_out) v *= s_out[row];
    if (activation == CTOX_ACT_SILU) v = v / (1.0f + expf(-v));
    y[(long long)pos * y_stride + row] = v;
}

// ------------------------------------------------------------------ row-per-warp kernel
// One warp per row over the canonical bytes, scalar fp32 FMAs, shuffle
// reduction: the shape of the reference's sm_86 kernel
// (kernels/cuda/q2q4_fused_matvec_sm86.cu:87-195). Kept as the comparison
// point for the streaming kernel and for operations that keep canonical bytes.
template <int DT>
__global__ void k_matvec_rowwarp(const uint8_t *__restrict__ canon, const float *__restrict__ x,
                                 const float *__restrict__ s_in, const float *__restrict__ s_out,
                                 const float *__restrict__ bias, float *__restrict__ y,
                                 uint32_t rows, uint32_t blocks, uint32_t activation) {
    pdl_launch();
    pdl_wait();
    using F = Fmt<DT>;
    const uint32_t row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const uint32_t lane = threadIdx.x & 31;
    if (row >= rows) return;
    const uint8_t *rp = canon + (uint64_t)row * blocks * F::kBlockBytes;
    float sum = 0.f;
    for (uint32_t b = lane; b < blocks; b += 32) {
        const uint16_t *bp = reinterpret_cast<const uint16_t *>(rp + (uint64_t)b * F::kBlockBytes);
        const float scale = __half2float(__ushort_as_half(bp[0]));
        float part = 0.f;
        const float *xb = x + b * 64;
        const float *sb = s_in ? s_in + b * 64 : nullptr;
#pragma unroll 4
        for (int h = 0; h < F::kCodeBytes / 2; ++h) {
            const uint32_t w = bp[1 + h];
            if (DT == 1) {
#pragma unroll
                for (int n = 0; n < 4; ++n) {
                    const int k = h * 4 + n;
                    const float xv = sb ? xb[k] * sb[k] : xb[k];
                    part = fmaf(((float)((w >> (4 * n)) & 15u) - 7.5f) * (1.0f / 7.5f), xv, part);
                }
            } else {
#pragma unroll
                for (int n = 0; n < 8; ++n) {
                    const int k = h * 8 + n;
                    const float xv = sb ? xb[k] * sb[k] : xb[k];
                    part = fmaf((2.0f * (float)((w >> (2 * n)) & 3u) - 3.0f) * (1.0f / 3.0f), xv, part);
                }
            }
        }
        sum = fmaf(scale, part, sum);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    if (lane == 0) {
        if (bias) sum += bias[row];
        if (s_out) sum *= s_out[row];
        if (activation == CTOX_ACT_SILU) sum = sum / (1.0f + expf(-sum));
        y[row] = sum;
    }
}

// Embedding-row decode: out[i][c] = scale * norm(code) * s_in[c] * s_out_i for the
// rows picked by row_ids (backend/cpu.rs:312-370; CUDA candidate
// kernels/cuda/q2q4_fused_matvec_sm86.cu:711-830). One thread per two columns.
template <int DT>
__global__ void k_recovered_rows(const uint8_t *__restrict__ canon, const uint32_t *__restrict__ row_ids,
                                 const float *__restrict__ s_in, const float *__restrict__ s_out,
                                 float s_out_scalar, float *__restrict__ out, uint32_t columns,
                                 uint32_t n_rows, uint32_t matrix_rows, int32_t *error_flag) {
    pdl_launch();
    pdl_wait();
    using F = Fmt<DT>;
    const uint32_t i = blockIdx.y;
    const uint32_t c = (blockIdx.x * blockDim.x + threadIdx.x) * 2;
    if (i >= n_rows || c >= columns) return;
    const uint32_t row = row_ids ? row_ids[i] : i;
    if (row >= matrix_rows) {
        atomicExch(error_flag, DEV_ERR_NONFINITE_VALUE);
        return;
    }
    const uint32_t blocks = columns / 64;
    const uint8_t *bp = canon + ((uint64_t)row * blocks + c / 64) * F::kBlockBytes;
    const float scale = __half2float(__ushort_as_half(*reinterpret_cast<const uint16_t *>(bp)));
    const uint32_t lc = c & 63;
    float n0, n1;
    if (DT == 1) {
        const uint32_t byte = bp[2 + lc / 2];
        n0 = ((float)(byte & 15u) - 7.5f) / 7.5f;
        n1 = ((float)(byte >> 4) - 7.5f) / 7.5f;
    } else {
        const uint32_t byte = bp[2 + lc / 4] >> ((lc & 3) * 2);
        const float cb[4] = {-1.0f, -1.0f / 3.0f, 1.0f / 3.0f, 1.0f};
        n0 = cb[byte & 3u];
        n1 = cb[(byte >> 2) & 3u];
    }
    const float so = s_out ? s_out[row] : s_out_scalar;
    const float a = s_in ? s_in[c] : 1.0f, b = s_in ? s_in[c + 1] : 1.0f;
    out[(size_t)i * columns + c] = scale * n0 * a * so;
    out[(size_t)i * columns + c + 1] = scale * n1 * b * so;
}

__global__ void k_bf16_to_f32(const __nv_bfloat16 *in, float *out, long long n) {
    pdl_launch();
    pdl_wait();
    long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = __bfloat162float(in[i]);
}

}  // namespace ctox

using namespace ctox;

namespace {

// backend/cpu.rs:41-173
ctox_status validate_op(ctox_ctx *ctx, const ctox_fused_matvec_op *op, bool need_input) {
    if (!op) return fail(ctx, CTOX_SHAPE, "operation is NULL");
    if (op->columns == 0 || op->rows == 0 || op->columns % kBlockLen)
        return fail(ctx, CTOX_SHAPE,
                    "Q2/Q4 fused matvec dimensions must be non-zero and columns divisible by 64");
    if (need_input && (!op->input || op->input_len != op->columns))
        return fail(ctx, CTOX_SHAPE, "input has %llu, expected %llu values",
                    (unsigned long long)op->input_len, (unsigned long long)op->columns);
    if (op->s_in_kind != CTOX_SCALE_NONE && op->s_in_len != op->columns)
        return fail(ctx, CTOX_SHAPE, "s_in length differs from columns");
    if (op->s_out_kind != CTOX_SCALE_NONE && op->s_out_len != op->rows)
        return fail(ctx, CTOX_SHAPE, "s_out length differs from rows");
    if (op->bias && op->bias_len != op->rows)
        return fail(ctx, CTOX_SHAPE, "bias length differs from rows");
    if (op->s_in_kind > CTOX_SCALE_F16LE || op->s_out_kind > CTOX_SCALE_F16LE)
        return fail(ctx, CTOX_SHAPE, "unknown scale slice kind");
    if (op->activation > CTOX_ACT_SILU) return fail(ctx, CTOX_SHAPE, "unknown activation");
    const uint64_t bpr = op->columns / kBlockLen;
    uint64_t bb = 0;
    if (op->dtype == CTOX_Q2B64)
        bb = kQ2BlockBytes;
    else if (op->dtype == CTOX_Q4B64)
        bb = kQ4BlockBytes;
    else if (op->dtype != CTOX_MIXED_Q2Q4B64)
        return fail(ctx, CTOX_UNSUPPORTED_DTYPE, "dtype %u", op->dtype);
    if (op->rows > 0x7fffffffull || op->columns > 0x7fffffffull)
        return fail(ctx, CTOX_SHAPE, "matrix dimension exceeds the device index range");
    if (bb) {
        if (op->n_segments)
            return fail(ctx, CTOX_INVALID_ARTIFACT, "pure Q2/Q4 operation declares mixed row segments");
        uint64_t blocks, expected;
        if (__builtin_mul_overflow(op->rows, bpr, &blocks) || __builtin_mul_overflow(blocks, bb, &expected))
            return fail(ctx, CTOX_SHAPE, "weight buffer size overflows");
        if (op->weights_len != expected || !op->weights)
            return fail(ctx, CTOX_SHAPE, "weight buffer has %llu bytes, expected %llu",
                        (unsigned long long)op->weights_len, (unsigned long long)expected);
        return CTOX_OK;
    }
    if (op->n_segments == 0 || !op->segments)
        return fail(ctx, CTOX_INVALID_ARTIFACT, "mixed Q2/Q4 operation has no row segments");
    uint64_t expected_row = 0, expected_offset = 0;
    for (uint64_t gidx = 0; gidx < op->n_segments; ++gidx) {
        const ctox_segment &s = op->segments[gidx];
        if (s.group_index != gidx || s.row_start != expected_row || s.row_end <= s.row_start ||
            s.row_end > op->rows || s.offset != expected_offset)
            return fail(ctx, CTOX_INVALID_ARTIFACT, "mixed Q2/Q4 operation has non-contiguous segment %u",
                        s.group_index);
        uint64_t sbb;
        if (s.dtype == CTOX_Q2B64)
            sbb = kQ2BlockBytes;
        else if (s.dtype == CTOX_Q4B64)
            sbb = kQ4BlockBytes;
        else
            return fail(ctx, CTOX_INVALID_ARTIFACT, "mixed Q2/Q4 segment %u has invalid dtype %u",
                        s.group_index, s.dtype);
        uint64_t blocks, expected_length;
        if (__builtin_mul_overflow(s.row_end - s.row_start, bpr, &blocks) ||
            __builtin_mul_overflow(blocks, sbb, &expected_length))
            return fail(ctx, CTOX_SHAPE, "mixed segment size overflows");
        if (s.length != expected_length)
            return fail(ctx, CTOX_INVALID_ARTIFACT, "mixed Q2/Q4 segment %u has %llu bytes, expected %llu",
                        s.group_index, (unsigned long long)s.length, (unsigned long long)expected_length);
        expected_row = s.row_end;
        if (__builtin_add_overflow(expected_offset, s.length, &expected_offset))
            return fail(ctx, CTOX_SHAPE, "mixed weight buffer size overflows");
    }
    if (expected_row != op->rows || expected_offset != op->weights_len || !op->weights)
        return fail(ctx, CTOX_SHAPE, "mixed segments cover %llu/%llu rows and %llu/%llu bytes",
                    (unsigned long long)expected_row, (unsigned long long)op->rows,
                    (unsigned long long)expected_offset, (unsigned long long)op->weights_len);
    return CTOX_OK;
}

// backend/mod.rs:91-111: widen a recovery-scale slice, rejecting non-finite values.
ctox_status widen_scales(ctox_ctx *ctx, uint32_t kind, const void *data, uint64_t n,
                         std::vector<float> &out) {
    out.resize(n);
    for (uint64_t i = 0; i < n; ++i) {
        float v;
        if (kind == CTOX_SCALE_F32) {
            v = ((const float *)data)[i];
        } else {
            const uint8_t *b = (const uint8_t *)data + 2 * i;
            v = f16_bits_to_f32((uint16_t)(b[0] | (b[1] << 8)));
        }
        if (!std::isfinite(v))
            return fail(ctx, CTOX_INVALID_ARTIFACT, "recovery scale %llu is non-finite",
                        (unsigned long long)i);
        out[i] = v;
    }
    return CTOX_OK;
}

ctox_status upload_f32(ctox_ctx *ctx, const float *src, uint64_t n, float **dst, ctox_matvec *mv) {
    ctox_status rc = dev_alloc(ctx, (void **)dst, n * sizeof(float));
    if (rc) return rc;
    mv->device_bytes += n * sizeof(float);
    CTOX_CUDA(ctx, cudaMemcpyAsync(*dst, src, n * sizeof(float), cudaMemcpyHostToDevice, ctx->stream));
    CTOX_CUDA(ctx, cudaStreamSynchronize(ctx->stream));  // src may be a temporary
    return CTOX_OK;
}

// Launch shapes of the streaming kernel: warps per CTA x bulk-copy stages per warp. More warps
// hide the unpack/MMA latency better (16x2 measured fastest on B200); fewer leave shared memory
// for the activation fragments of wide matrices and many positions.
struct StreamCfg {
    int warps, stages;
};

size_t stream_smem_bytes(int dt, StreamCfg cfg, uint32_t slice_blocks, uint32_t npos) {
    const size_t chunk = dt ? (size_t)Fmt<1>::kChunkPairs * 2 * Fmt<1>::kSuperTileBytes
                            : (size_t)Fmt<0>::kChunkPairs * 2 * Fmt<0>::kSuperTileBytes;
    const size_t stage = (size_t)cfg.warps * cfg.stages * chunk;
    const size_t xfrag = (size_t)slice_blocks * 2 * npos * 128;
    const size_t meta = ((size_t)slice_blocks * npos * 8 + 15) & ~(size_t)15;
    return stage + xfrag + meta + 16 + ((size_t)cfg.warps * cfg.stages + 1) * 8;
}

// The widest launch shape whose shared memory fits; warps == 0 when none does.
StreamCfg pick_stream_cfg(ctox_ctx *ctx, int dt, uint32_t slice_blocks, uint32_t npos) {
    static const int forced = [] {
        const char *e = getenv("CTOX_MATVEC_CFG");
        if (e && !strcmp(e, "8x4")) return 1;
        if (e && !strcmp(e, "8x2")) return 2;
        return 0;
    }();
    const StreamCfg order[] = {{16, 2}, {8, 4}, {8, 2}};
    for (int i = forced; i < 3; ++i)
        if (stream_smem_bytes(dt, order[i], slice_blocks, npos) <= (size_t)ctx->max_smem_optin) return order[i];
    return StreamCfg{0, 0};
}

template <int DT, int NT>
void launch_stream_nt(StreamCfg cfg, unsigned grid, size_t smem, cudaStream_t st, const StreamParams &sp) {
    if (cfg.warps == 16)
        launch_pdl(k_matvec_stream<DT, 16, 2, NT>, dim3(grid), dim3(512), smem, st, sp);
    else if (cfg.stages == 4)
        launch_pdl(k_matvec_stream<DT, 8, 4, NT>, dim3(grid), dim3(256), smem, st, sp);
    else
        launch_pdl(k_matvec_stream<DT, 8, 2, NT>, dim3(grid), dim3(256), smem, st, sp);
}

template <int DT>
void launch_stream(StreamCfg cfg, unsigned grid, size_t smem, cudaStream_t st, const StreamParams &sp) {
    if (sp.npos > 4)
        launch_stream_nt<DT, 2>(cfg, grid, smem, st, sp);
    else
        launch_stream_nt<DT, 1>(cfg, grid, smem, st, sp);
}

void free_matvec(ctox_matvec *mv) {
    ctox_ctx *ctx = mv->ctx;
    for (auto &p : mv->parts) {
        dev_free(ctx, p.prep, p.prep_bytes);
        dev_free(ctx, p.canon, p.canon_bytes);
        dev_free(ctx, p.partial, p.partial_bytes);
        for (auto &sp : p.split) dev_free(ctx, sp.pieces, sp.pieces_bytes);
    }
    dev_free(ctx, mv->s_in, mv->columns * sizeof(float));
    dev_free(ctx, mv->s_out, mv->rows * sizeof(float));
    dev_free(ctx, mv->bias, mv->rows * sizeof(float));
    dev_free(ctx, mv->xfrag, mv->xfrag_bytes);
    dev_free(ctx, mv->meta, mv->meta_bytes);
    dev_free(ctx, mv->xtmp, mv->xtmp_bytes);
    dev_free(ctx, mv->ytmp, mv->ytmp_bytes);
    delete mv;
}

// Column slices: the streaming kernel keeps the activation fragments of one slice in shared
// memory (2 KB per 64-column block at 8 positions), so wide matrices are cut until a slice has
// at most 72 blocks (4608 columns), which leaves room for the 8-warp bulk-copy ring.
uint32_t choose_slices(uint32_t kst) {
    for (uint32_t sl : {1u, 2u, 4u, 8u})
        if (kst % sl == 0 && kst / sl <= 18) return sl;
    for (uint32_t sl : {8u, 4u, 2u})
        if (kst % sl == 0) return sl;
    return 1;
}

// host_bytes != NULL: the canonical bytes are uploaded; otherwise part.canon already holds them
// on the device (tracked allocation of nbytes, ownership taken).
ctox_status prepare_part(ctox_ctx *ctx, ctox_matvec *mv, MatvecPart &part, const uint8_t *host_bytes,
                         size_t nbytes, uint32_t flags) {
    const int stb = part.dt ? Fmt<1>::kSuperTileBytes : Fmt<0>::kSuperTileBytes;
    const uint32_t row_tiles = (uint32_t)((part.rows + kTileRows - 1) / kTileRows);
    const uint32_t kst = mv->blocks_padded / kTileBlocks;
    part.pairs = (row_tiles + 1) / 2;
    part.slices = choose_slices(kst);
    part.kst_s = kst / part.slices;
    part.canon_bytes = nbytes;
    ctox_status rc = CTOX_OK;
    if (host_bytes) {
        rc = dev_alloc(ctx, (void **)&part.canon, nbytes);
        if (rc) return rc;
        CTOX_CUDA(ctx, cudaMemcpyAsync(part.canon, host_bytes, nbytes, cudaMemcpyHostToDevice, ctx->stream));
    }
    const uint64_t tiles = (uint64_t)part.pairs * 2 * kst;
    part.prep_bytes = (size_t)tiles * stb;
    rc = dev_alloc(ctx, (void **)&part.prep, part.prep_bytes);
    if (rc) return rc;
    const uint32_t grid = (uint32_t)((tiles + 3) / 4);
    if (part.dt)
        launch_pdl(k_repack<1>, dim3(grid), dim3(128), 0, ctx->stream, part.canon, part.prep, (uint32_t)part.rows, mv->blocks,
                                                   part.pairs, part.kst_s, part.slices, ctx->dev_error);
    else
        launch_pdl(k_repack<0>, dim3(grid), dim3(128), 0, ctx->stream, part.canon, part.prep, (uint32_t)part.rows, mv->blocks,
                                                   part.pairs, part.kst_s, part.slices, ctx->dev_error);
    CTOX_CUDA(ctx, cudaGetLastError());
    // work split of the streaming kernel, per launch-shape class, and the pieces each
    // (pair, slice) is cut into
    const uint64_t units = (uint64_t)part.pairs * part.kst_s;  // per slice
    part.max_pieces = 1;
    for (int cls = 0; cls < 2; ++cls) {
        MatvecPart::Split &sp = part.split[cls];
        const StreamCfg cfg = pick_stream_cfg(ctx, part.dt, part.kst_s * 4, cls ? kMaxPosPerPass : 4);
        sp.warps = cfg.warps;
        sp.stages = cfg.stages;
        if (cfg.warps == 0) continue;
        sp.ctas_per_slice = (uint32_t)ctx->sm_count / part.slices;
        if (sp.ctas_per_slice == 0) sp.ctas_per_slice = 1;
        uint64_t nw = (uint64_t)sp.ctas_per_slice * cfg.warps;
        if (nw > units) nw = units;
        sp.warps_per_slice = (uint32_t)nw;
        sp.ctas_per_slice = (uint32_t)((nw + cfg.warps - 1) / cfg.warps);
        std::vector<uint8_t> pieces((size_t)part.pairs * part.slices);
        uint32_t mp = 1;
        for (uint32_t pr = 0; pr < part.pairs; ++pr) {
            const uint64_t u_first = (uint64_t)pr * part.kst_s, u_last = u_first + part.kst_s - 1;
            const uint64_t w_first = ((u_first + 1) * nw + units - 1) / units - 1;
            const uint64_t w_last = ((u_last + 1) * nw + units - 1) / units - 1;
            const uint64_t n = w_last - w_first + 1;
            if (n > 255) return fail(ctx, CTOX_SHAPE, "row pair split into %llu pieces", (unsigned long long)n);
            for (uint32_t sl = 0; sl < part.slices; ++sl) pieces[(size_t)pr * part.slices + sl] = (uint8_t)n;
            if (n > mp) mp = (uint32_t)n;
        }
        sp.max_pieces = mp;
        if (mp > part.max_pieces) part.max_pieces = mp;
        sp.pieces_bytes = pieces.size();
        rc = dev_alloc(ctx, (void **)&sp.pieces, sp.pieces_bytes);
        if (rc) return rc;
        CTOX_CUDA(ctx, cudaMemcpyAsync(sp.pieces, pieces.data(), sp.pieces_bytes, cudaMemcpyHostToDevice,
                                       ctx->stream));
        CTOX_CUDA(ctx, cudaStreamSynchronize(ctx->stream));  // `pieces` is a temporary
        mv->device_bytes += sp.pieces_bytes;
    }
    part.partial_bytes = (size_t)part.pairs * part.slices * part.max_pieces * kPairRows * kMaxPosPerPass *
                         sizeof(float);
    rc = dev_alloc(ctx, (void **)&part.partial, part.partial_bytes);
    if (rc) return rc;
    CTOX_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    if (!(flags & CTOX_PREPARE_KEEP_CANONICAL)) {
        dev_free(ctx, part.canon, part.canon_bytes);
        part.canon = nullptr;
        part.canon_bytes = 0;
    }
    mv->device_bytes += part.prep_bytes + part.canon_bytes + part.partial_bytes;
    return CTOX_OK;
}

ctox_status set_smem_attr(ctox_ctx *ctx) {
    static thread_local int done_device = -1;
    if (done_device == ctx->device) return CTOX_OK;
#define CTOX_SMEM_ATTR(...)                                                                        \
    CTOX_CUDA(ctx, cudaFuncSetAttribute(k_matvec_stream<__VA_ARGS__>,                              \
                                        cudaFuncAttributeMaxDynamicSharedMemorySize, ctx->max_smem_optin))
    CTOX_SMEM_ATTR(0, 16, 2, 1);
    CTOX_SMEM_ATTR(1, 16, 2, 1);
    CTOX_SMEM_ATTR(0, 8, 4, 1);
    CTOX_SMEM_ATTR(1, 8, 4, 1);
    CTOX_SMEM_ATTR(0, 8, 2, 1);
    CTOX_SMEM_ATTR(1, 8, 2, 1);
    CTOX_SMEM_ATTR(0, 16, 2, 2);
    CTOX_SMEM_ATTR(1, 16, 2, 2);
    CTOX_SMEM_ATTR(0, 8, 4, 2);
    CTOX_SMEM_ATTR(1, 8, 4, 2);
    CTOX_SMEM_ATTR(0, 8, 2, 2);
    CTOX_SMEM_ATTR(1, 8, 2, 2);
#undef CTOX_SMEM_ATTR
    done_device = ctx->device;
    return CTOX_OK;
}

ctox_status check_device_error(ctox_ctx *ctx, const char *what) {
    int32_t code = 0;
    ctox_status rc = ctox_ctx_device_error(ctx, &code);
    if (rc) return rc;
    if (code == DEV_ERR_NONFINITE_SCALE)
        return fail(ctx, CTOX_INVALID_ARTIFACT, "%s: block scale is non-finite", what);
    if (code == DEV_ERR_WAIT_TIMEOUT)
        return fail(ctx, CTOX_INVALID_STATE, "%s: a bounded device wait ran out", what);
    if (code) return fail(ctx, CTOX_INVALID_STATE, "%s: device error %d", what, code);
    return CTOX_OK;
}

}  // namespace

namespace ctox {

uint32_t matvec_positions_per_pass(ctox_matvec *mv) {
    // every part must fit: 8 positions if the wide class fits, else up to 4 (shrinking if needed)
    bool wide = true, narrow = true;
    for (auto &p : mv->parts) {
        wide = wide && p.split[1].warps != 0;
        narrow = narrow && p.split[0].warps != 0;
    }
    if (wide) return kMaxPosPerPass;
    if (narrow) return 4;
    uint32_t per_pass = 3;
    for (; per_pass > 0; --per_pass) {
        bool fits = true;
        for (auto &p : mv->parts)
            fits = fits && pick_stream_cfg(mv->ctx, p.dt, p.kst_s * 4, per_pass).warps != 0;
        if (fits) break;
    }
    return per_pass;
}

// fragments_of: another matrix of the same fan-out group whose fragment buffers hold the activations.
ctox_status matvec_stream_prepared(ctox_matvec *mv, size_t part_index, uint32_t npos, const ctox_matvec *fragments_of) {
    ctox_ctx *ctx = mv->ctx;
    MatvecPart &p = mv->parts[part_index];
    const MatvecPart::Split &split = p.split[npos > 4 ? 1 : 0];
    StreamCfg cfg{split.warps, split.stages};
    if (cfg.warps == 0) {
        // the class shape does not fit; a smaller position count may (same work split as class 0
        // only if the shape is the same, so recompute nothing: refuse instead)
        return fail(ctx, CTOX_MEMORY_BUDGET, "streaming kernel: %u positions of %llu columns exceed shared memory",
                    npos, (unsigned long long)mv->columns);
    }
    StreamParams sp;
    sp.wprep = p.prep;
    sp.xfrag = fragments_of ? fragments_of->xfrag : mv->xfrag;
    sp.meta = fragments_of ? fragments_of->meta : mv->meta;
    sp.partial = p.partial;
    sp.error_flag = ctx->dev_error;
    sp.pairs = p.pairs;
    sp.kst_s = p.kst_s;
    sp.slices = p.slices;
    sp.ctas_per_slice = split.ctas_per_slice;
    sp.warps_per_slice = split.warps_per_slice;
    sp.npos = npos;
    sp.max_pieces = p.max_pieces;
    const size_t smem = stream_smem_bytes(p.dt, cfg, p.kst_s * 4, npos);
    const unsigned grid = split.ctas_per_slice * p.slices;
    timing_begin(ctx);
    if (p.dt)
        launch_stream<1>(cfg, grid, smem, ctx->stream, sp);
    else
        launch_stream<0>(cfg, grid, smem, ctx->stream, sp);
    timing_end(ctx);
    CTOX_CUDA(ctx, cudaGetLastError());
    return CTOX_OK;
}

ctox_status matvec_stream_pass(ctox_matvec *mv, size_t part_index, const void *x, uint32_t x_dtype,
                               uint32_t npos, uint64_t x_stride) {
    MatvecPart &p = mv->parts[part_index];
    // the activation fragments depend on the code format (column multipliers)
    const int groups = (int)(mv->blocks_padded * npos);
    launch_pdl(k_prep_x, dim3((groups * 16 + 255) / 256), dim3(256), 0, mv->ctx->stream, 
        x, x_dtype == CTOX_BF16, (long long)x_stride, mv->s_in, (int)mv->columns, (int)mv->blocks_padded,
        (int)npos, p.dt, mv->xfrag, mv->meta);
    return matvec_stream_prepared(mv, part_index, npos);
}

ctox_status matvec_create_device(ctox_ctx *ctx, int dt, uint64_t rows, uint64_t columns, uint8_t *canon,
                                 size_t canon_bytes, float *s_in, float *s_out, uint32_t flags,
                                 ctox_matvec **out) {
    *out = nullptr;
    ctox_status rc = set_smem_attr(ctx);
    if (rc) return rc;
    ctox_matvec *mv = new ctox_matvec();
    mv->ctx = ctx;
    mv->rows = rows;
    mv->columns = columns;
    mv->packed_bytes = canon_bytes;
    mv->blocks = (uint32_t)(columns / kBlockLen);
    mv->blocks_padded = (mv->blocks + kTileBlocks - 1) / kTileBlocks * kTileBlocks;
    mv->activation = CTOX_ACT_IDENTITY;
    mv->s_in = s_in;
    mv->s_out = s_out;
    mv->device_bytes += (s_in ? columns * 4 : 0) + (s_out ? rows * 4 : 0);
    MatvecPart part;
    part.dt = dt;
    part.rows = rows;
    part.canon = canon;
    mv->parts.push_back(part);
    rc = prepare_part(ctx, mv, mv->parts.back(), nullptr, canon_bytes, flags);
    if (!rc) {
        mv->xfrag_bytes = (size_t)mv->blocks_padded * 2 * kMaxPosPerPass * 128;
        rc = dev_alloc(ctx, (void **)&mv->xfrag, mv->xfrag_bytes);
    }
    if (!rc) {
        mv->meta_bytes = (size_t)mv->blocks_padded * kMaxPosPerPass * sizeof(float2);
        rc = dev_alloc(ctx, (void **)&mv->meta, mv->meta_bytes);
    }
    if (!rc) {
        mv->device_bytes += mv->xfrag_bytes + mv->meta_bytes;
        rc = check_device_error(ctx, "prepare");
    }
    if (rc) {
        free_matvec(mv);
        return rc;
    }
    *out = mv;
    return CTOX_OK;
}

ctox_status matvec_embed_rows(ctox_matvec *mv, const uint32_t *row_ids_dev, uint32_t n, float *out) {
    ctox_ctx *ctx = mv->ctx;
    MatvecPart &p = mv->parts[0];
    if (!p.canon)
        return fail(ctx, CTOX_UNSUPPORTED_OPERATION, "row gather needs CTOX_PREPARE_KEEP_CANONICAL at prepare");
    dim3 grid((unsigned)((mv->columns / 2 + 127) / 128), n);
    if (p.dt)
        launch_pdl(k_recovered_rows<1>, dim3(grid), dim3(128), 0, ctx->stream, p.canon, row_ids_dev, mv->s_in, mv->s_out, 1.0f, out,
                                                           (uint32_t)mv->columns, n, (uint32_t)mv->rows,
                                                           ctx->dev_error);
    else
        launch_pdl(k_recovered_rows<0>, dim3(grid), dim3(128), 0, ctx->stream, p.canon, row_ids_dev, mv->s_in, mv->s_out, 1.0f, out,
                                                           (uint32_t)mv->columns, n, (uint32_t)mv->rows,
                                                           ctx->dev_error);
    CTOX_CUDA(ctx, cudaGetLastError());
    return CTOX_OK;
}

void matvec_finish_enqueue(ctox_matvec *mv, uint32_t npos, float *y, uint64_t y_stride) {
    MatvecPart &p = mv->parts[0];
    const unsigned n_out = (unsigned)(p.rows * npos);
    launch_pdl(k_matvec_finish, dim3((n_out + 255) / 256), dim3(256), 0, mv->ctx->stream, 
        p.partial, p.split[npos > 4 ? 1 : 0].pieces, mv->s_out, mv->bias, y, (long long)y_stride,
        (uint32_t)p.rows, npos, p.slices, p.max_pieces, mv->activation);
}

}  // namespace ctox

extern "C" {

ctox_status ctox_matvec_prepare(ctox_ctx *ctx, const ctox_fused_matvec_op *op, uint32_t flags,
                                ctox_matvec **out) {
    if (!ctx || !out) return CTOX_INVALID_STATE;
    *out = nullptr;
    ctox_status rc = validate_op(ctx, op, false);
    if (rc) return rc;
    std::vector<float> s_in, s_out;
    if (op->s_in_kind != CTOX_SCALE_NONE) {
        rc = widen_scales(ctx, op->s_in_kind, op->s_in, op->s_in_len, s_in);
        if (rc) return rc;
    }
    if (op->s_out_kind != CTOX_SCALE_NONE) {
        rc = widen_scales(ctx, op->s_out_kind, op->s_out, op->s_out_len, s_out);
        if (rc) return rc;
    }
    uint64_t s_in_digest = 0;
    if (!s_in.empty()) {
        s_in_digest = 1469598103934665603ull;  // FNV-1a over the widened values
        const uint8_t *b = reinterpret_cast<const uint8_t *>(s_in.data());
        for (size_t i = 0; i < s_in.size() * sizeof(float); ++i) s_in_digest = (s_in_digest ^ b[i]) * 1099511628211ull;
        if (s_in_digest == 0) s_in_digest = 1;
    }
    CTOX_CUDA(ctx, cudaSetDevice(ctx->device));
    rc = set_smem_attr(ctx);
    if (rc) return rc;
    ctox_matvec *mv = new ctox_matvec();
    mv->ctx = ctx;
    mv->rows = op->rows;
    mv->columns = op->columns;
    mv->packed_bytes = op->weights_len;
    mv->blocks = (uint32_t)(op->columns / kBlockLen);
    mv->blocks_padded = (mv->blocks + kTileBlocks - 1) / kTileBlocks * kTileBlocks;
    mv->activation = op->activation;
    mv->s_in_digest = s_in_digest;
#define PREP_TRY(expr)          \
    do {                        \
        rc = (expr);            \
        if (rc) {               \
            free_matvec(mv);    \
            return rc;          \
        }                       \
    } while (0)
    if (!s_in.empty()) PREP_TRY(upload_f32(ctx, s_in.data(), s_in.size(), &mv->s_in, mv));
    if (!s_out.empty()) PREP_TRY(upload_f32(ctx, s_out.data(), s_out.size(), &mv->s_out, mv));
    if (op->bias) PREP_TRY(upload_f32(ctx, op->bias, op->rows, &mv->bias, mv));
    if (op->dtype == CTOX_MIXED_Q2Q4B64) {
        for (uint64_t i = 0; i < op->n_segments; ++i) {
            const ctox_segment &s = op->segments[i];
            MatvecPart part;
            part.dt = s.dtype == CTOX_Q4B64;
            part.row_start = s.row_start;
            part.rows = s.row_end - s.row_start;
            mv->parts.push_back(part);
            PREP_TRY(prepare_part(ctx, mv, mv->parts.back(), op->weights + s.offset, s.length, flags));
        }
    } else {
        MatvecPart part;
        part.dt = op->dtype == CTOX_Q4B64;
        part.rows = op->rows;
        mv->parts.push_back(part);
        PREP_TRY(prepare_part(ctx, mv, mv->parts.back(), op->weights, op->weights_len, flags));
    }
    mv->xfrag_bytes = (size_t)mv->blocks_padded * 2 * kMaxPosPerPass * 128;
    PREP_TRY(dev_alloc(ctx, (void **)&mv->xfrag, mv->xfrag_bytes));
    mv->meta_bytes = (size_t)mv->blocks_padded * kMaxPosPerPass * sizeof(float2);
    PREP_TRY(dev_alloc(ctx, (void **)&mv->meta, mv->meta_bytes));
    mv->device_bytes += mv->xfrag_bytes + mv->meta_bytes;
    PREP_TRY(check_device_error(ctx, "prepare"));
#undef PREP_TRY
    *out = mv;
    return CTOX_OK;
}

ctox_status ctox_matvec_destroy(ctox_matvec *mv) {
    if (!mv) return CTOX_OK;
    cudaSetDevice(mv->ctx->device);
    cudaStreamSynchronize(mv->ctx->stream);
    free_matvec(mv);
    return CTOX_OK;
}

ctox_status ctox_matvec_info(const ctox_matvec *mv, uint64_t *rows, uint64_t *columns,
                             uint64_t *packed_bytes, uint64_t *device_bytes) {
    if (!mv) return CTOX_INVALID_STATE;
    if (rows) *rows = mv->rows;
    if (columns) *columns = mv->columns;
    if (packed_bytes) *packed_bytes = mv->packed_bytes;
    if (device_bytes) *device_bytes = mv->device_bytes;
    return CTOX_OK;
}

ctox_status ctox_matvec_dispatch(ctox_matvec *mv, const void *x_dev, uint32_t x_dtype,
                                 uint32_t positions, uint64_t x_stride, float *y_dev,
                                 uint64_t y_stride, uint32_t kernel) {
    if (!mv) return CTOX_INVALID_STATE;
    ctox_ctx *ctx = mv->ctx;
    if (!x_dev || !y_dev) return fail(ctx, CTOX_SHAPE, "dispatch: null device pointer");
    if (positions == 0 || positions > 16)
        return fail(ctx, CTOX_SHAPE, "dispatch: positions must be 1..16, got %u", positions);
    if (x_dtype != CTOX_F32 && x_dtype != CTOX_BF16)
        return fail(ctx, CTOX_UNSUPPORTED_DTYPE, "dispatch: activation dtype %u", x_dtype);
    if (x_stride < mv->columns || y_stride < mv->rows)
        return fail(ctx, CTOX_SHAPE, "dispatch: stride shorter than a row");
    if (kernel == CTOX_KERNEL_AUTO) kernel = CTOX_KERNEL_STREAM;
    cudaStream_t st = ctx->stream;

    if (kernel == CTOX_KERNEL_ROWWARP) {
        const float *xf = (const float *)x_dev;
        if (x_dtype == CTOX_BF16) {
            size_t need = (size_t)positions * x_stride * sizeof(float);
            if (need > mv->xtmp_bytes) {
                dev_free(ctx, mv->xtmp, mv->xtmp_bytes);
                mv->xtmp = nullptr;
                mv->xtmp_bytes = 0;
                ctox_status rc = dev_alloc(ctx, (void **)&mv->xtmp, need);
                if (rc) return rc;
                mv->xtmp_bytes = need;
            }
            long long n = (long long)positions * x_stride;
            launch_pdl(k_bf16_to_f32, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, st, (const __nv_bfloat16 *)x_dev,
                                                                       mv->xtmp, n);
            xf = mv->xtmp;
        }
        for (auto &p : mv->parts) {
            if (!p.canon)
                return fail(ctx, CTOX_UNSUPPORTED_OPERATION,
                            "row-warp kernel needs CTOX_PREPARE_KEEP_CANONICAL at prepare");
            for (uint32_t m = 0; m < positions; ++m) {
                const unsigned grid = (unsigned)((p.rows + 3) / 4);
                const float *so = mv->s_out ? mv->s_out + p.row_start : nullptr;
                const float *bi = mv->bias ? mv->bias + p.row_start : nullptr;
                float *yy = y_dev + m * y_stride + p.row_start;
                timing_begin(ctx);
                if (p.dt)
                    launch_pdl(k_matvec_rowwarp<1>, dim3(grid), dim3(128), 0, st, p.canon, xf + m * x_stride, mv->s_in, so, bi,
                                                              yy, (uint32_t)p.rows, mv->blocks, mv->activation);
                else
                    launch_pdl(k_matvec_rowwarp<0>, dim3(grid), dim3(128), 0, st, p.canon, xf + m * x_stride, mv->s_in, so, bi,
                                                              yy, (uint32_t)p.rows, mv->blocks, mv->activation);
                timing_end(ctx);
            }
        }
        CTOX_CUDA(ctx, cudaGetLastError());
        return CTOX_OK;
    }
    if (kernel != CTOX_KERNEL_STREAM) return fail(ctx, CTOX_SHAPE, "dispatch: unknown kernel %u", kernel);

    const uint32_t per_pass = matvec_positions_per_pass(mv);
    if (per_pass == 0)
        return fail(ctx, CTOX_MEMORY_BUDGET, "columns %llu exceed the shared-memory budget of the streaming kernel",
                    (unsigned long long)mv->columns);
    const size_t esz = x_dtype == CTOX_BF16 ? 2 : 4;
    for (uint32_t m0 = 0; m0 < positions; m0 += per_pass) {
        const uint32_t npos = positions - m0 < per_pass ? positions - m0 : per_pass;
        const uint8_t *xp = (const uint8_t *)x_dev + (size_t)m0 * x_stride * esz;
        for (size_t pi = 0; pi < mv->parts.size(); ++pi) {
            ctox_status rc = matvec_stream_pass(mv, pi, xp, x_dtype, npos, x_stride);
            if (rc) return rc;
            MatvecPart &p = mv->parts[pi];
            const unsigned n_out = (unsigned)(p.rows * npos);
            launch_pdl(k_matvec_finish, dim3((n_out + 255) / 256), dim3(256), 0, st, 
                p.partial, p.split[npos > 4 ? 1 : 0].pieces, mv->s_out ? mv->s_out + p.row_start : nullptr,
                mv->bias ? mv->bias + p.row_start : nullptr, y_dev + (size_t)m0 * y_stride + p.row_start,
                (long long)y_stride, (uint32_t)p.rows, npos, p.slices, p.max_pieces, mv->activation);
        }
    }
    CTOX_CUDA(ctx, cudaGetLastError());
    return CTOX_OK;
}

ctox_status ctox_matvec_fanout_dispatch(ctox_matvec *const *mvs, uint64_t n, const void *x_dev, uint32_t x_dtype,
                                        uint32_t positions, uint64_t x_stride, float *const *y_devs,
                                        const uint64_t *y_strides) {
    if (!mvs || n == 0 || !mvs[0]) return CTOX_INVALID_STATE;
    ctox_matvec *first = mvs[0];
    ctox_ctx *ctx = first->ctx;
    if (!x_dev || !y_devs || !y_strides) return fail(ctx, CTOX_SHAPE, "fan-out: null pointer");
    if (positions == 0 || positions > 16) return fail(ctx, CTOX_SHAPE, "fan-out: positions must be 1..16, got %u", positions);
    if (x_dtype != CTOX_F32 && x_dtype != CTOX_BF16) return fail(ctx, CTOX_UNSUPPORTED_DTYPE, "fan-out: activation dtype %u", x_dtype);
    if (x_stride < first->columns) return fail(ctx, CTOX_SHAPE, "fan-out: stride shorter than a row");
    // fanout.rs:31-70: one corrected input serves matrices with the same input and identical s_in;
    // here also the same code format, which fixes the fragment layout
    uint32_t per_pass = kMaxPosPerPass;
    for (uint64_t i = 0; i < n; ++i) {
        ctox_matvec *mv = mvs[i];
        if (!mv || mv->ctx != ctx || !y_devs[i]) return fail(ctx, CTOX_INVALID_STATE, "fan-out: member %llu is unusable", (unsigned long long)i);
        if (mv->parts.size() != 1 || mv->parts[0].dt != first->parts[0].dt)
            return fail(ctx, CTOX_UNSUPPORTED_OPERATION, "fan-out: members must be pure and of one code format");
        if (mv->columns != first->columns || mv->s_in_digest != first->s_in_digest)
            return fail(ctx, CTOX_SHAPE, "fan-out: members must share the input width and s_in");
        if (y_strides[i] < mv->rows) return fail(ctx, CTOX_SHAPE, "fan-out: output stride shorter than a row");
        const uint32_t pp = matvec_positions_per_pass(mv);
        if (pp == 0) return fail(ctx, CTOX_MEMORY_BUDGET, "fan-out: columns exceed the shared-memory budget");
        per_pass = pp < per_pass ? pp : per_pass;
    }
    const size_t esz = x_dtype == CTOX_BF16 ? 2 : 4;
    for (uint32_t m0 = 0; m0 < positions; m0 += per_pass) {
        const uint32_t npos = positions - m0 < per_pass ? positions - m0 : per_pass;
        const uint8_t *xp = (const uint8_t *)x_dev + (size_t)m0 * x_stride * esz;
        const int groups = (int)(first->blocks_padded * npos);
        launch_pdl(k_prep_x, dim3((groups * 16 + 255) / 256), dim3(256), 0, ctx->stream, (const void *)xp,
                   (int)(x_dtype == CTOX_BF16), (long long)x_stride, (const float *)first->s_in, (int)first->columns,
                   (int)first->blocks_padded, (int)npos, first->parts[0].dt, first->xfrag, first->meta);
        for (uint64_t i = 0; i < n; ++i) {
            ctox_matvec *mv = mvs[i];
            ctox_status rc = matvec_stream_prepared(mv, 0, npos, first);
            if (rc) return rc;
            float *y = y_devs[i] + (size_t)m0 * y_strides[i];
            MatvecPart &p = mv->parts[0];
            const unsigned n_out = (unsigned)(p.rows * npos);
            launch_pdl(k_matvec_finish, dim3((n_out + 255) / 256), dim3(256), 0, ctx->stream, p.partial,
                       p.split[npos > 4 ? 1 : 0].pieces, mv->s_out, mv->bias, y, (long long)y_strides[i],
                       (uint32_t)p.rows, npos, p.slices, p.max_pieces, mv->activation);
        }
    }
    CTOX_CUDA(ctx, cudaGetLastError());
    return CTOX_OK;
}

ctox_status ctox_matvec_recovered_rows(ctox_matvec *mv, const uint32_t *row_ids_dev, uint32_t n, float *out_dev) {
    if (!mv) return CTOX_INVALID_STATE;
    ctox_ctx *ctx = mv->ctx;
    if (!row_ids_dev || !out_dev || n == 0) return fail(ctx, CTOX_SHAPE, "recovered rows: null pointer or no rows");
    if (mv->parts.size() != 1) return fail(ctx, CTOX_UNSUPPORTED_OPERATION, "recovered rows: mixed matrices are served by the host form");
    if (!mv->s_in || !mv->s_out) return fail(ctx, CTOX_SHAPE, "recovered rows need both recovery scales (backend/cpu.rs:312-370)");
    CTOX_CUDA(ctx, cudaSetDevice(ctx->device));
    return matvec_embed_rows(mv, row_ids_dev, n, out_dev);
}

ctox_status ctox_matvec_dispatch_host(ctox_matvec *mv, const float *x_host, uint32_t positions,
                                      float *y_host, uint32_t kernel) {
    if (!mv) return CTOX_INVALID_STATE;
    ctox_ctx *ctx = mv->ctx;
    if (!x_host || !y_host) return fail(ctx, CTOX_SHAPE, "dispatch_host: null pointer");
    if (positions == 0 || positions > 16)
        return fail(ctx, CTOX_SHAPE, "dispatch_host: positions must be 1..16, got %u", positions);
    CTOX_CUDA(ctx, cudaSetDevice(ctx->device));
    const size_t xb = (size_t)positions * mv->columns * sizeof(float);
    const size_t yb = (size_t)positions * mv->rows * sizeof(float);
    ctox_status rc = ensure_pinned(ctx, xb + yb);
    if (rc) return rc;
    if (xb > mv->xtmp_bytes) {
        dev_free(ctx, mv->xtmp, mv->xtmp_bytes);
        mv->xtmp = nullptr;
        mv->xtmp_bytes = 0;
        rc = dev_alloc(ctx, (void **)&mv->xtmp, xb);
        if (rc) return rc;
        mv->xtmp_bytes = xb;
    }
    if (yb > mv->ytmp_bytes) {
        dev_free(ctx, mv->ytmp, mv->ytmp_bytes);
        mv->ytmp = nullptr;
        mv->ytmp_bytes = 0;
        rc = dev_alloc(ctx, (void **)&mv->ytmp, yb);
        if (rc) return rc;
        mv->ytmp_bytes = yb;
    }
    float *px = (float *)ctx->pinned;
    float *py = (float *)((uint8_t *)ctx->pinned + xb);
    memcpy(px, x_host, xb);
    CTOX_CUDA(ctx, cudaMemcpyAsync(mv->xtmp, px, xb, cudaMemcpyHostToDevice, ctx->stream));
    rc = ctox_matvec_dispatch(mv, mv->xtmp, CTOX_F32, positions, mv->columns, mv->ytmp, mv->rows, kernel);
    if (rc) return rc;
    CTOX_CUDA(ctx, cudaMemcpyAsync(py, mv->ytmp, yb, cudaMemcpyDeviceToHost, ctx->stream));
    CTOX_CUDA(ctx, cudaMemcpyAsync(ctx->host_error, ctx->dev_error, sizeof(int32_t), cudaMemcpyDeviceToHost,
                                   ctx->stream));
    CTOX_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    if (*ctx->host_error) {
        rc = check_device_error(ctx, "dispatch");
        if (rc) return rc;
    }
    memcpy(y_host, py, yb);
    return CTOX_OK;
}

ctox_status ctox_fused_matvec(ctox_ctx *ctx, const ctox_fused_matvec_op *op, float *out) {
    if (!ctx) return CTOX_INVALID_STATE;
    ctox_status rc = validate_op(ctx, op, true);
    if (rc) return rc;
    if (!out) return fail(ctx, CTOX_SHAPE, "output is NULL");
    ctox_matvec *mv = nullptr;
    rc = ctox_matvec_prepare(ctx, op, 0, &mv);
    if (rc) return rc;
    rc = ctox_matvec_dispatch_host(mv, op->input, 1, out, CTOX_KERNEL_AUTO);
    ctox_matvec_destroy(mv);
    if (rc) return rc;
    // a non-finite output is an invalid state, as in backend/cuda_runtime.rs:10626-10630
    for (uint64_t i = 0; i < op->rows; ++i)
        if (!std::isfinite(out[i]))
            return fail(ctx, CTOX_INVALID_STATE, "fused matvec produced a non-finite output at row %llu",
                        (unsigned long long)i);
    return CTOX_OK;
}

ctox_status ctox_fused_matvec_fanout(ctox_ctx *ctx, const ctox_fused_matvec_op *ops, uint64_t n,
                                     float *const *outs) {
    if (!ctx) return CTOX_INVALID_STATE;
    if (n == 0 || !ops || !outs) return fail(ctx, CTOX_SHAPE, "fan-out requires at least one projection");
    for (uint64_t i = 0; i < n; ++i) {
        ctox_status rc = validate_op(ctx, &ops[i], true);
        if (rc) return rc;
    }
    for (uint64_t i = 0; i < n; ++i) {
        ctox_status rc = ctox_fused_matvec(ctx, &ops[i], outs[i]);
        if (rc) return rc;
    }
    return CTOX_OK;
}

ctox_status ctox_recovered_row(ctox_ctx *ctx, uint32_t dtype, const uint8_t *weights,
                               uint64_t weights_len, uint64_t columns, uint32_t s_in_kind,
                               const void *s_in, uint64_t s_in_len, float s_out, float *out) {
    if (!ctx) return CTOX_INVALID_STATE;
    // backend/cpu.rs:313-338
    if (columns == 0 || columns % kBlockLen)
        return fail(ctx, CTOX_SHAPE, "recovered row columns must be non-zero and divisible by 64");
    if (s_in_kind == CTOX_SCALE_NONE || s_in_kind > CTOX_SCALE_F16LE || s_in_len != columns ||
        !std::isfinite(s_out))
        return fail(ctx, CTOX_SHAPE, "recovered row scale contract differs");
    uint64_t bb;
    if (dtype == CTOX_Q2B64)
        bb = kQ2BlockBytes;
    else if (dtype == CTOX_Q4B64)
        bb = kQ4BlockBytes;
    else
        return fail(ctx, CTOX_UNSUPPORTED_DTYPE, "dtype %u", dtype);
    const uint64_t expected = columns / kBlockLen * bb;
    if (weights_len != expected || !weights || !out)
        return fail(ctx, CTOX_SHAPE, "recovered row has %llu packed bytes, expected %llu",
                    (unsigned long long)weights_len, (unsigned long long)expected);
    for (uint64_t b = 0; b < columns / kBlockLen; ++b) {
        const uint8_t *blk = weights + b * bb;
        if (!std::isfinite(f16_bits_to_f32((uint16_t)(blk[0] | (blk[1] << 8)))))
            return fail(ctx, CTOX_INVALID_ARTIFACT, "recovered row block scale is non-finite");
    }
    std::vector<float> si;
    ctox_status rc = widen_scales(ctx, s_in_kind, s_in, s_in_len, si);
    if (rc) return rc;
    CTOX_CUDA(ctx, cudaSetDevice(ctx->device));
    uint8_t *dw = nullptr;
    float *dsi = nullptr, *dout = nullptr;
    const size_t fb = columns * sizeof(float);
    rc = dev_alloc(ctx, (void **)&dw, weights_len);
    if (!rc) rc = dev_alloc(ctx, (void **)&dsi, fb);
    if (!rc) rc = dev_alloc(ctx, (void **)&dout, fb);
    if (!rc) rc = ensure_pinned(ctx, fb);
    cudaError_t e = cudaSuccess;
    if (!rc) {
        e = cudaMemcpyAsync(dw, weights, weights_len, cudaMemcpyHostToDevice, ctx->stream);
        if (e == cudaSuccess)
            e = cudaMemcpyAsync(dsi, si.data(), fb, cudaMemcpyHostToDevice, ctx->stream);
        if (e == cudaSuccess) {
            dim3 grid((unsigned)((columns / 2 + 127) / 128), 1);
            if (dtype == CTOX_Q4B64)
                launch_pdl(k_recovered_rows<1>, dim3(grid), dim3(128), 0, ctx->stream, dw, nullptr, dsi, nullptr, s_out, dout,
                                                                   (uint32_t)columns, 1, 1, ctx->dev_error);
            else
                launch_pdl(k_recovered_rows<0>, dim3(grid), dim3(128), 0, ctx->stream, dw, nullptr, dsi, nullptr, s_out, dout,
                                                                   (uint32_t)columns, 1, 1, ctx->dev_error);
            e = cudaGetLastError();
        }
        if (e == cudaSuccess)
            e = cudaMemcpyAsync(ctx->pinned, dout, fb, cudaMemcpyDeviceToHost, ctx->stream);
        if (e == cudaSuccess) e = cudaStreamSynchronize(ctx->stream);
        if (e == cudaSuccess) memcpy(out, ctx->pinned, fb);
    }
    dev_free(ctx, dw, weights_len);
    dev_free(ctx, dsi, fb);
    dev_free(ctx, dout, fb);
    if (rc) return rc;
    if (e != cudaSuccess) return fail(ctx, CTOX_INVALID_STATE, "recovered row: %s", cudaGetErrorString(e));
    return CTOX_OK;
}

ctox_status ctox_recovered_row_matvec(ctox_ctx *ctx, uint32_t dtype, const uint8_t *weights,
                                      uint64_t weights_len, const float *corrected_input,
                                      uint64_t columns, float s_out, float *out) {
    if (!ctx) return CTOX_INVALID_STATE;
    // backend/cpu.rs:478-497
    bool bad = columns == 0 || columns % kBlockLen || !std::isfinite(s_out) || !corrected_input || !out;
    for (uint64_t i = 0; !bad && i < columns; ++i) bad = !std::isfinite(corrected_input[i]);
    if (bad) return fail(ctx, CTOX_SHAPE, "recovered row matvec input or output scale is invalid");
    if (dtype != CTOX_Q2B64 && dtype != CTOX_Q4B64) return fail(ctx, CTOX_UNSUPPORTED_DTYPE, "dtype %u", dtype);
    ctox_fused_matvec_op op;
    memset(&op, 0, sizeof op);
    op.dtype = dtype;
    op.weights = weights;
    op.weights_len = weights_len;
    op.rows = 1;
    op.columns = columns;
    op.input = corrected_input;
    op.input_len = columns;
    op.s_out_kind = CTOX_SCALE_F32;
    op.s_out = &s_out;
    op.s_out_len = 1;
    return ctox_fused_matvec(ctx, &op, out);
}

}  // extern "C"

// ------------------------------------------------------------------ dispatch without allocation
// Some callers must not allocate device memory around a dispatch: a real-time serving loop that
// has handed every free byte to its KV cache, a plug-in running inside another framework's
// memory pool, or code between two points where cudaMalloc's implicit device synchronisation
// would stall other streams. For them the scratch of the streaming kernel (activation fragments,
// per-block metadata and the partial sums) lives in one fixed array inside the library image
// instead of buffers owned by the handle. Every GPU that loads the library carries the array
// until the process exits.
namespace {

constexpr size_t kStaticScratchBytes = 8u << 20;  // 8 MiB
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

// The array's name is only a host-side stand-in; kernels need its device address, which is looked
// up once per device with that device current.
ctox_status static_scratch_address(ctox_ctx *ctx, unsigned char **out) {
    constexpr int kMaxDevices = 64;
    static unsigned char *cached[kMaxDevices] = {nullptr};
    if (ctx->device < 0 || ctx->device >= kMaxDevices)
        return fail(ctx, CTOX_SHAPE, "device index %d has no static scratch slot", ctx->device);
    if (!cached[ctx->device]) {
        CTOX_CUDA(ctx, cudaSetDevice(ctx->device));
        void *ptr = nullptr;
        const cudaError_t e = cudaGetSymbolAddress(&ptr, g_static_scratch);
        if (e != cudaSuccess || !ptr)
            return fail(ctx, CTOX_INVALID_STATE, "cudaGetSymbolAddress(static scratch) failed: %s",
                        cudaGetErrorString(e));
        cached[ctx->device] = static_cast<unsigned char *>(ptr);
    }
    *out = cached[ctx->device];
    return CTOX_OK;
}

size_t align256(size_t v) { return (v + 255) & ~(size_t)255; }

}  // namespace

extern "C" ctox_status ctox_matvec_dispatch_static(ctox_matvec *mv, const void *x_dev, uint32_t x_dtype,
                                                   uint32_t positions, uint64_t x_stride, float *y_dev,
                                                   uint64_t y_stride) {
    if (!mv) return CTOX_INVALID_STATE;
    ctox_ctx *ctx = mv->ctx;
    if (!x_dev || !y_dev) return fail(ctx, CTOX_SHAPE, "dispatch_static: null device pointer");
    if (positions == 0 || positions > 16)
        return fail(ctx, CTOX_SHAPE, "dispatch_static: positions must be 1..16, got %u", positions);
    if (x_dtype != CTOX_F32 && x_dtype != CTOX_BF16)
        return fail(ctx, CTOX_UNSUPPORTED_DTYPE, "dispatch_static: activation dtype %u", x_dtype);
    if (x_stride < mv->columns || y_stride < mv->rows)
        return fail(ctx, CTOX_SHAPE, "dispatch_static: stride shorter than a row");
    const uint32_t per_pass = matvec_positions_per_pass(mv);
    if (per_pass == 0)
        return fail(ctx, CTOX_MEMORY_BUDGET, "dispatch_static: columns %llu exceed the streaming kernel's budget",
                    (unsigned long long)mv->columns);
    // scratch layout: [fragments][metadata][partial sums of the largest part]
    const uint32_t pass_max = positions < per_pass ? positions : per_pass;
    const size_t frag_bytes = align256((size_t)mv->blocks_padded * 2 * pass_max * 128);
    const size_t meta_bytes = align256((size_t)mv->blocks_padded * pass_max * sizeof(float2));
    size_t partial_bytes = 0;
    for (auto &p : mv->parts) partial_bytes = partial_bytes > p.partial_bytes ? partial_bytes : p.partial_bytes;
    const size_t need = frag_bytes + meta_bytes + align256(partial_bytes);
    if (need > kStaticScratchBytes)
        return fail(ctx, CTOX_MEMORY_BUDGET,
                    "dispatch_static: this %llux%llu operation needs %zu bytes of scratch, the built-in array "
                    "holds %zu; use ctox_matvec_dispatch",
                    (unsigned long long)mv->rows, (unsigned long long)mv->columns, need, kStaticScratchBytes);
    CTOX_CUDA(ctx, cudaSetDevice(ctx->device));  // every call: the launches below go to the current device
    unsigned char *base = nullptr;
    ctox_status rc = static_scratch_address(ctx, &base);
    if (rc) return rc;
    uint8_t *xfrag = base;
    float2 *meta = reinterpret_cast<float2 *>(base + frag_bytes);
    float *partial = reinterpret_cast<float *>(base + frag_bytes + meta_bytes);
    cudaStream_t st = ctx->stream;
    const size_t esz = x_dtype == CTOX_BF16 ? 2 : 4;
    for (uint32_t m0 = 0; m0 < positions; m0 += per_pass) {
        const uint32_t npos = positions - m0 < per_pass ? positions - m0 : per_pass;
        const uint8_t *xp = (const uint8_t *)x_dev + (size_t)m0 * x_stride * esz;
        for (auto &p : mv->parts) {
            const MatvecPart::Split &split = p.split[npos > 4 ? 1 : 0];
            if (split.warps == 0)
                return fail(ctx, CTOX_MEMORY_BUDGET, "dispatch_static: %u positions do not fit shared memory", npos);
            const int groups = (int)(mv->blocks_padded * npos);
            launch_pdl(k_prep_x, dim3((groups * 16 + 255) / 256), dim3(256), 0, st, xp, x_dtype == CTOX_BF16, (long long)x_stride,
                                                               mv->s_in, (int)mv->columns,
                                                               (int)mv->blocks_padded, (int)npos, p.dt, xfrag, meta);
            StreamParams sp;
            sp.wprep = p.prep;
            sp.xfrag = xfrag;
            sp.meta = meta;
            sp.partial = partial;
            sp.error_flag = ctx->dev_error;
            sp.pairs = p.pairs;
            sp.kst_s = p.kst_s;
            sp.slices = p.slices;
            sp.ctas_per_slice = split.ctas_per_slice;
            sp.warps_per_slice = split.warps_per_slice;
            sp.npos = npos;
            sp.max_pieces = p.max_pieces;
            const StreamCfg cfg{split.warps, split.stages};
            const size_t smem = stream_smem_bytes(p.dt, cfg, p.kst_s * 4, npos);
            const unsigned grid = split.ctas_per_slice * p.slices;
            timing_begin(ctx);
            if (p.dt)
                launch_stream<1>(cfg, grid, smem, st, sp);
            else
                launch_stream<0>(cfg, grid, smem, st, sp);
            timing_end(ctx);
            const unsigned n_out = (unsigned)(p.rows * npos);
            launch_pdl(k_matvec_finish, dim3((n_out + 255) / 256), dim3(256), 0, st, 
                partial, split.pieces, mv->s_out ? mv->s_out + p.row_start : nullptr,
                mv->bias ? mv->bias + p.row_start : nullptr, y_dev + (size_t)m0 * y_stride + p.row_start,
                (long long)y_stride, (uint32_t)p.rows, npos, p.slices, p.max_pieces, mv->activation);
        }
    }
    CTOX_CUDA(ctx, cudaGetLastError());
    return CTOX_OK;
}
