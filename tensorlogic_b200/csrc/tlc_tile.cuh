// Device layout of Q4_0 / Q8_0 weights: the GGUF blocks of a [N, K] tensor, bit
// for bit, regrouped into tiles of 16 rows so that both matrix kernels fetch
// them with aligned 16-byte accesses and no byte shuffling:
//
//   tensor = [slab = row / 16][k-tile] tiles, each 1024 bytes of quants + the scales
//
//   Q4_0 tile: 16 rows x 4 blocks (128 columns), 1152 bytes (= 16 x 4 x 18)
//     quants  [h = r / 8][g = r % 8][t = 0..3] 16 bytes = word t of the qs of blocks 0, 1, 2, 3 of row r
//     scales  [r = 0..15][block 0..3] f16                                    at byte 1024
//   Q8_0 tile: 16 rows x 2 blocks (64 columns), 1088 bytes (= 16 x 2 x 34)
//     quants  [h][g][t = 0..3] 16 bytes = words 2t, 2t+1 of block 0, words 2t, 2t+1 of block 1 of row r
//     scales  [r][block 0..1] f16                                            at byte 1024
//
// (word w of a block = its quant bytes 4w .. 4w+3, little endian.)
//   * the GEMV's lane (g, t) of a warp reads the 16 bytes [h = 0][g][t] and
//     [h = 1][g][t]: the A-fragment words of rows g and g + 8 for every block of
//     the tile, conflict-free, and a whole ring stage is ONE contiguous bulk copy;
//   * a GEMM producer thread that owns row r reads the 64 contiguous bytes
//     [h][g][0..3]: every quant of the row's blocks in the tile.
// Rows past N and blocks past K / 32 are zero (scale 0): they add nothing.
// Replaces the row-major Vec<f16> the reference's loader builds
// (src/model/formats/gguf.rs:377-450) as the resident form of a weight.
#pragma once

#include <cstddef>
#include <cstdint>

#include "tlcuda.h"

namespace tlc_tile {

constexpr int kSlabRows = 16;
constexpr int kQuantBytes = 1024;  // quant bytes of a tile, either type

__host__ __device__ constexpr int tile_blocks(int type) { return type == TLC_TYPE_Q4_0 ? 4 : 2; }
__host__ __device__ constexpr int tile_bytes(int type) { return type == TLC_TYPE_Q4_0 ? 1152 : 1088; }
__host__ __device__ constexpr int block_words(int type) { return type == TLC_TYPE_Q4_0 ? 4 : 8; }
__host__ __device__ constexpr int block_bytes(int type) { return type == TLC_TYPE_Q4_0 ? 18 : 34; }

// Byte offset inside a tile of word w of block j (of the tile) of row r (of the slab).
__host__ __device__ inline uint32_t word_offset(int type, int r, int j, int w) {
    const uint32_t base = (uint32_t)((r >> 3) * 512 + (r & 7) * 64);
    if (type == TLC_TYPE_Q4_0) return base + (uint32_t)(w * 16 + j * 4);
    return base + (uint32_t)((w >> 1) * 16 + (j * 2 + (w & 1)) * 4);
}
__host__ __device__ inline uint32_t scale_offset(int type, int r, int j) {
    return (uint32_t)kQuantBytes + (uint32_t)((r * tile_blocks(type) + j) * 2);
}

// Tiles along K and slabs along N of a [rows, cols] tensor.
__host__ __device__ inline int64_t k_tiles(int type, int64_t cols) {
    const int64_t per = 32 * tile_blocks(type);
    return (cols + per - 1) / per;
}
__host__ __device__ inline int64_t slabs(int64_t rows) { return (rows + kSlabRows - 1) / kSlabRows; }

// Start of the tile that holds block bc of row `row`.
__host__ __device__ inline size_t tile_start(int type, int64_t ktiles, int64_t row, int64_t bc) {
    return (size_t)((row / kSlabRows) * ktiles + bc / tile_blocks(type)) * (size_t)tile_bytes(type);
}

// Scatters one verbatim GGUF block (`blk`: d, then the quant bytes) to its place
// (32-bit stores: every word of a tile is 4-byte aligned).
__host__ __device__ inline void store_block(uint8_t *data, int type, int64_t ktiles, int64_t row, int64_t bc,
                                            const uint8_t *blk) {
    uint8_t *tile = data + tile_start(type, ktiles, row, bc);
    const int r = (int)(row % kSlabRows), j = (int)(bc % tile_blocks(type));
    *reinterpret_cast<uint16_t *>(tile + scale_offset(type, r, j)) = (uint16_t)(blk[0] | (blk[1] << 8));
    for (int w = 0; w < block_words(type); w++) {
        const uint8_t *b = blk + 2 + 4 * w;
        *reinterpret_cast<uint32_t *>(tile + word_offset(type, r, j, w)) =
            (uint32_t)b[0] | ((uint32_t)b[1] << 8) | ((uint32_t)b[2] << 16) | ((uint32_t)b[3] << 24);
    }
}

// Gathers the block back into its verbatim GGUF bytes.
__host__ __device__ inline void load_block(const uint8_t *data, int type, int64_t ktiles, int64_t row, int64_t bc,
                                           uint8_t *blk) {
    const uint8_t *tile = data + tile_start(type, ktiles, row, bc);
    const int r = (int)(row % kSlabRows), j = (int)(bc % tile_blocks(type));
    const uint16_t d = *reinterpret_cast<const uint16_t *>(tile + scale_offset(type, r, j));
    blk[0] = (uint8_t)d;
    blk[1] = (uint8_t)(d >> 8);
    for (int w = 0; w < block_words(type); w++) {
        const uint32_t v = *reinterpret_cast<const uint32_t *>(tile + word_offset(type, r, j, w));
        for (int i = 0; i < 4; i++) blk[2 + 4 * w + i] = (uint8_t)(v >> (8 * i));
    }
}

}  // namespace tlc_tile
