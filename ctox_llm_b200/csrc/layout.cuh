// Prepared ("streaming") weight layout of the Q2_B64 / Q4_B64 matvec kernels.
//
// The canonical CTOXQ payload is row-major blocks of [f16 scale][codes]
// (34 B for Q4, 18 B for Q2; quant.rs:5-8,117-122,181-186). Neither stride is a
// multiple of 16 bytes, so a kernel cannot fetch canonical blocks with 128-bit
// loads or bulk copies. `prepare` therefore repacks once, on the device, into
// super-tiles of 16 rows x 4 blocks (256 columns) whose bytes are exactly the
// canonical bytes, regrouped so that one warp reads a super-tile as
//   [128 B scales][code vectors: 32 lanes x 16 B each]
// and every lane's 16-byte vector holds the codes it feeds to
// mma.sync.m16n8k16 (rows g and g+8, 16 consecutive columns of lane quarter t).
// The size is unchanged: 16*4*34 = 2176 B (Q4), 16*4*18 = 1152 B (Q2); rows pad
// to 16 and blocks to 4 with zero-scale blocks.
//
// Super-tiles are ordered (row-tile pair, column super-tile, tile of the pair):
// the two row tiles of a pair share one column range, so a warp that takes a
// pair loads the activation fragments once for 32 rows, and any contiguous
// range of the work list (in pair units) is one contiguous byte range.
#pragma once
#include <cstdint>

namespace ctox {

constexpr int kBlockLen = 64;
constexpr int kQ2BlockBytes = 18;
constexpr int kQ4BlockBytes = 34;
constexpr int kTileRows = 16;
constexpr int kTileBlocks = 4;
constexpr int kScaleBytes = 128;  // 16 rows x 4 blocks x f16

template <int DT>
struct Fmt;
template <>
struct Fmt<0> {  // Q2_B64
    static constexpr int kBlockBytes = kQ2BlockBytes;
    static constexpr int kCodeBytes = 16;
    static constexpr int kSuperTileBytes = kScaleBytes + 2 * 512;  // 1152
    static constexpr int kChunkPairs = 2;                          // tile pairs per bulk copy
};
template <>
struct Fmt<1> {  // Q4_B64
    static constexpr int kBlockBytes = kQ4BlockBytes;
    static constexpr int kCodeBytes = 32;
    static constexpr int kSuperTileBytes = kScaleBytes + 4 * 512;  // 2176
    static constexpr int kChunkPairs = 1;
};

// Column order in which a lane's 16 consecutive columns are fed to the four
// MMAs of a block (two columns per A/B register), as the inverse map
// column -> slot.
//   Q4: registers are the nibble pairs (0,4)(1,5)(2,6)(3,7) of each 8-code word.
//   Q2: registers are the field pairs (0,8)(1,9)...(7,15) of the 16-code word.
__host__ __device__ inline int inv_perm(int dt, int q) {
    // Q4 {0,2,4,6,1,3,5,7, 8,10,12,14,9,11,13,15}; Q2 {0,2,..,14, 1,3,..,15}: as arithmetic, so that a
    // run-time q does not turn a table into a local-memory array
    return dt ? ((q & 8) | ((q & 3) << 1) | ((q >> 2) & 1)) : (((q & 7) << 1) | (q >> 3));
}

// The kernels feed the tensor cores the masked code bits themselves: a code at
// mantissa bit p of an otherwise zero fp16 is the subnormal  code * 2^(p-24),
// exact, with no exponent to OR in. Codes at different bit positions carry
// different powers of two; the activation of that column is pre-multiplied by
// the inverse power so that every product is  code * x * kCodeScale.
//   Q4: low nibble p=0 (x16), high nibble p=4 (x1); product scale 2^-20.
//   Q2: fields at p = 0,2,4,6,8 -> x256,x64,x16,x4,x1; product scale 2^-16.
__host__ __device__ inline float column_multiplier(int dt, int column) {
    if (dt) return (column & 1) ? 1.0f : 16.0f;
    // Q2 {256, 64, 16, 4, 1, 256, 64, 16}: 2^(8 - 2 k), k = position of the field in its half word
    const int idx = column & 7, k = idx >= 5 ? idx - 5 : idx;
    return (float)(1 << (8 - 2 * k));
}
__host__ __device__ inline float code_scale(int dt) { return dt ? 9.5367431640625e-07f /* 2^-20 */
                                                               : 1.52587890625e-05f /* 2^-16 */; }
// Exponent to which a block's largest |activation| is normalised, so that the
// largest pre-multiplied fp16 stays below 2^15.
__host__ __device__ inline int norm_exponent(int dt) { return dt ? 10 : 6; }
// value = unit * (code - offset): Q4 (code-7.5)/7.5, Q2 (2*code-3)/3.
__host__ __device__ inline float code_offset(int dt) { return dt ? 7.5f : 1.5f; }
__host__ __device__ inline float code_unit(int dt) { return dt ? (1.0f / 7.5f) : (2.0f / 3.0f); }

}  // namespace ctox
