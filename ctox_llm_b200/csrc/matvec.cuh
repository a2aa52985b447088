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
    uint64_t s_in_digest = 0;  // FNV-1a of the widened s_in values (0 = none): fan-out groups must agree
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
// land in part.partial ([pairs][slices][max_pieces][kMaxPosPerPass][32 rows]); no finish kernel is run.
ctox_status matvec_stream_pass(ctox_matvec *mv, size_t part_index, const void *x, uint32_t x_dtype,
                               uint32_t npos, uint64_t x_stride);
// Same, for activations that are already in fragment form in mv->xfrag / mv->meta (or in those of
// fragments_of, another matrix of the same fan-out group).
ctox_status matvec_stream_prepared(ctox_matvec *mv, size_t part_index, uint32_t npos,
                                   const ctox_matvec *fragments_of = nullptr);
// Takes ownership of tracked device buffers: canonical bytes, widened s_in [columns], s_out [rows].
ctox_status matvec_create_device(ctox_ctx *ctx, int dt, uint64_t rows, uint64_t columns, uint8_t *canon,
                                 size_t canon_bytes, float *s_in, float *s_out, uint32_t flags,
                                 ctox_matvec **out);
// out[i][c] = W[row_ids[i]][c] * s_in[c] * s_out[row] (embedding rows, backend/cpu.rs:312-370).
ctox_status matvec_embed_rows(ctox_matvec *mv, const uint32_t *row_ids_dev, uint32_t n, float *out);
// y[pos][row] from the partial sums of the last streamed pass.
void matvec_finish_enqueue(ctox_matvec *mv, uint32_t npos, float *y, uint64_t y_stride);
// Selection over the partial sums of an lm_head pass (head.cu). Statistics of verify nodes
// node0 .. node0+npos; then the acceptance walk over all nodes, whose record stays on the device.
ctox_status head_verify_enqueue(ctox_matvec *mv, uint32_t node0, uint32_t npos, uint32_t n_nodes,
                                const int32_t *parent, const uint32_t *tokens_dev, float inv_t, uint64_t seed,
                                uint64_t step, uint32_t rows, float *logits_out_dev, uint32_t row_offset);
// Tensor-parallel vocabulary: merges the ranks' statistics (all-gather) before the acceptance walk.
ctox_status head_tp_merge_enqueue(ctox_ctx *ctx, uint32_t n_nodes, const int32_t *parent,
                                  const uint32_t *tokens_dev, uint32_t shard_rows);
ctox_status head_accept_enqueue(ctox_ctx *ctx, uint32_t n_nodes, const int32_t *parent,
                                const uint32_t *tokens_dev, float inv_t, uint64_t seed, uint64_t step,
                                int force_accept, ctox_spec_record **record_dev);
// Greedy token of a logit vector; token = row_ids[row] or row + row_offset. In a tensor-parallel
// group every rank passes its shard and all ranks receive the group's token.
ctox_status argmax_enqueue(ctox_ctx *ctx, const float *logits_dev, uint32_t n, const uint32_t *row_ids_dev,
                           uint32_t row_offset, uint32_t *token_dev, uint32_t *status_dev);
}  // namespace ctox
