// Host-side objects of the prepared matvec, shared by the selection kernels and the
// decode executor, which drive the streaming kernel pass by pass and read its partial sums.
#pragma once
#include <cuda_runtime.h>

#include <cstdint>
#include <vector>

#include "common.cuh"

namespace ctox {
constexpr int kMaxPosPerPass = 8;  // positions per pass of the streaming kernel (hi/lo => 16 columns)
constexpr int kPairRows = 32;      // rows of a tile pair (the unit of work and of the partial sums)
}  // namespace ctox

struct MatvecPart {
    int dt = 0;  // 0 Q2, 1 Q4
    uint64_t row_start = 0, rows = 0;
    uint32_t pairs = 0;   // 32-row tile pairs
    uint32_t slices = 1;  // column slices; a CTA of the streaming kernel works inside one
    uint32_t kst_s = 0;   // 256-column super-tiles per slice
    uint8_t *prep = nullptr;
    size_t prep_bytes = 0;
    uint8_t *canon = nullptr;
    size_t canon_bytes = 0;
    float *partial = nullptr;
    size_t partial_bytes = 0;
    // The work split depends on the launch shape, which depends on the number of positions
    // (shared memory); one table per shape class: [0] 1..4 positions, [1] 5..8 positions.
    struct Split {
        int warps = 0, stages = 0;       // launch shape; warps == 0: does not fit
        uint32_t ctas_per_slice = 0, warps_per_slice = 0, max_pieces = 1;
        uint8_t *pieces = nullptr;       // [pairs][slices] partial-sum pieces
        size_t pieces_bytes = 0;
    } split[2];
    uint32_t max_pieces = 1;  // slot stride of `partial`: max over both splits
};

struct ctox_matvec {
    ctox_ctx *ctx = nullptr;
    uint64_t rows = 0, columns = 0, packed_bytes = 0;
    uint32_t blocks = 0, blocks_padded = 0, activation = 0;
    std::vector<MatvecPart> parts;
    float *s_in = nullptr, *s_out = nullptr, *bias = nullptr;
    uint8_t *xfrag = nullptr;  // [blocks_padded][2*kMaxPosPerPass][128]
    size_t xfrag_bytes = 0;
    float2 *meta = nullptr;
    size_t meta_bytes = 0;
    float *xtmp = nullptr;  // f32 staging (bf16 input to the row-warp kernel, host form)
    size_t xtmp_bytes = 0;
    float *ytmp = nullptr;
    size_t ytmp_bytes = 0;
    uint64_t device_bytes = 0;
};

namespace ctox {
// Positions one pass of the streaming kernel can take for this matrix (shared-memory bound).
uint32_t matvec_positions_per_pass(ctox_matvec *mv);
// Enqueues activation preparation + streaming kernel for `npos` positions of one part; raw sums
// land in part.partial ([pairs][max_pieces][32][kMaxPosPerPass]); no finish kernel is run.
ctox_status matvec_stream_pass(ctox_matvec *mv, size_t part_index, const void *x, uint32_t x_dtype,
                               uint32_t npos, uint64_t x_stride);
// Same, for activations that are already in fragment form in mv->xfrag / mv->meta.
ctox_status matvec_stream_prepared(ctox_matvec *mv, size_t part_index, uint32_t npos);
}  // namespace ctox
