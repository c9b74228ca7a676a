// Quantized weights kept in HBM as their GGUF blocks (regrouped into 16-row
// tiles, tlc_tile.cuh), the device-side dequantizer, and the counter-based
// synthetic weight generator.
//
// Replaces the load-time CPU dequantization of the TensorLogic loaders
// (src/model/formats/gguf.rs:22-112, :377-450; mmap_gguf.rs:383-439).
#include <cstring>

#include "tlc_internal.h"
#include "tlc_synth.cuh"
#include "tlc_tile.cuh"

// ---------------------------------------------------------------------------
// Dequantization: one thread per block of 32.  Bit-exact with
// GGUFLoader::dequantize_q4_0 (gguf.rs:68-112): value = f16_rne((nib-8)*f32(d));
// low nibbles -> elements 0..15, high nibbles -> 16..31.  And with
// dequantize_q8_0 (gguf.rs:22-53): f16_rne(float(q)*float(d)).
// ---------------------------------------------------------------------------
__global__ void dequant_q4_0_kernel(const uint8_t *__restrict__ data, int64_t ktiles,
                                    int blocks_per_row, int64_t n_rows, __half *__restrict__ out) {
    int64_t gb = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    int64_t total = n_rows * blocks_per_row;
    if (gb >= total) return;
    int64_t row = gb / blocks_per_row;
    int bc = (int)(gb % blocks_per_row);
    uint8_t blk[18];
    tlc_tile::load_block(data, TLC_TYPE_Q4_0, ktiles, row, bc, blk);
    uint16_t dbits = (uint16_t)(blk[0] | (blk[1] << 8));
    float d = __half2float(__ushort_as_half(dbits));
    __half *o = out + (row * blocks_per_row + bc) * 32;
#pragma unroll
    for (int j = 0; j < 16; j++) {
        uint8_t b = blk[2 + j];
        o[j] = __float2half_rn(__fmul_rn((float)((int)(b & 0x0F) - 8), d));
        o[j + 16] = __float2half_rn(__fmul_rn((float)((int)(b >> 4) - 8), d));
    }
}

__global__ void dequant_q8_0_kernel(const uint8_t *__restrict__ data, int64_t ktiles,
                                    int blocks_per_row, int64_t n_rows, __half *__restrict__ out) {
    int64_t gb = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    int64_t total = n_rows * blocks_per_row;
    if (gb >= total) return;
    int64_t row = gb / blocks_per_row;
    int bc = (int)(gb % blocks_per_row);
    uint8_t blk[34];
    tlc_tile::load_block(data, TLC_TYPE_Q8_0, ktiles, row, bc, blk);
    uint16_t dbits = (uint16_t)(blk[0] | (blk[1] << 8));
    float d = __half2float(__ushort_as_half(dbits));
    __half *o = out + (row * blocks_per_row + bc) * 32;
#pragma unroll
    for (int j = 0; j < 32; j++) {
        int8_t q = (int8_t)blk[2 + j];
        o[j] = __float2half_rn(__fmul_rn((float)q, d));
    }
}

// Regrouping of row-major GGUF blocks (`src`, rows src_pitch apart) into tiles
// and back: one thread per block.
__global__ void tile_blocks_kernel(const uint8_t *__restrict__ src, size_t src_pitch, int type, int blocks_per_row,
                                   int64_t n_rows, int64_t ktiles, uint8_t *__restrict__ dst) {
    int64_t gb = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (gb >= n_rows * blocks_per_row) return;
    int64_t row = gb / blocks_per_row;
    int bc = (int)(gb % blocks_per_row);
    const int bb = tlc_tile::block_bytes(type);
    const uint16_t *s16 = reinterpret_cast<const uint16_t *>(src + row * src_pitch + (size_t)bc * bb);
    __align__(4) uint8_t blk[36];
    for (int i = 0; i < bb / 2; i++) reinterpret_cast<uint16_t *>(blk)[i] = s16[i];
    tlc_tile::store_block(dst, type, ktiles, row, bc, blk);
}

__global__ void untile_blocks_kernel(const uint8_t *__restrict__ data, int type, int blocks_per_row, int64_t n_rows,
                                     int64_t ktiles, uint8_t *__restrict__ out) {
    int64_t gb = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (gb >= n_rows * blocks_per_row) return;
    int64_t row = gb / blocks_per_row;
    int bc = (int)(gb % blocks_per_row);
    const int bb = tlc_tile::block_bytes(type);
    __align__(4) uint8_t blk[36];
    tlc_tile::load_block(data, type, ktiles, row, bc, blk);
    uint16_t *o16 = reinterpret_cast<uint16_t *>(out + (size_t)gb * bb);
    for (int i = 0; i < bb / 2; i++) o16[i] = reinterpret_cast<const uint16_t *>(blk)[i];
}

// Q6_K (GGUFLoader::dequantize_q6_k, gguf.rs:128-218, the llama.cpp order): one
// thread per (row, super-block, half, l) produces the four values l, l+32, l+64,
// l+96 of its half: q = 4 bits of ql | 2 bits of qh, value = f16_rne((d*sc)*(q-32)).
// Writes columns [col0, col0 + out_cols) of the row into a dense-pitch f16 tensor.
__global__ void dequant_q6_k_kernel(const uint8_t *__restrict__ data, int sb_per_row, int sb_bytes, int64_t n_rows,
                                    int64_t col0, int64_t out_cols, __half *__restrict__ out, size_t out_pitch) {
    const int64_t gi = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const int64_t total = n_rows * sb_per_row * 64;
    if (gi >= total) return;
    const int l = (int)(gi & 31), half = (int)((gi >> 5) & 1);
    const int64_t sbi = gi >> 6;
    const int64_t row = sbi / sb_per_row;
    const int sb = (int)(sbi % sb_per_row);
    const uint8_t *blk = data + (size_t)sbi * sb_bytes;  // 210 as in the file, 224 in the resident (padded) form
    const uint8_t *ql = blk + 64 * half, *qh = blk + 128 + 32 * half;
    const int8_t *sc = reinterpret_cast<const int8_t *>(blk + 192 + 8 * half);
    const float d = __half2float(__ushort_as_half((unsigned short)(blk[208] | (blk[209] << 8))));
    const int is = l >> 4;
    const int h = qh[l];
    int q[4];
    q[0] = ((ql[l] & 0xF) | (((h >> 0) & 3) << 4)) - 32;
    q[1] = ((ql[l + 32] & 0xF) | (((h >> 2) & 3) << 4)) - 32;
    q[2] = ((ql[l] >> 4) | (((h >> 4) & 3) << 4)) - 32;
    q[3] = ((ql[l + 32] >> 4) | (((h >> 6) & 3) << 4)) - 32;
    __half *orow = reinterpret_cast<__half *>(reinterpret_cast<uint8_t *>(out) + (size_t)row * out_pitch);
#pragma unroll
    for (int j = 0; j < 4; j++) {
        const int64_t col = (int64_t)sb * 256 + 128 * half + l + 32 * j - col0;
        if (col >= 0 && col < out_cols)
            orow[col] = __float2half_rn(__fmul_rn(__fmul_rn(d, (float)sc[is + 2 * j]), (float)q[j]));
    }
}

// Resident Q6_K: the file's 210-byte super-blocks, each padded to 224 bytes (ql 128 | qh 64 |
// scales 16 | d 2 | 14 zero bytes) so that every piece starts on a 16-byte boundary.  No byte
// of a super-block is changed.  pad = true: 210 -> 224; false: back to the file's form.
__global__ void q6k_repad_kernel(const uint8_t *__restrict__ src, uint8_t *__restrict__ dst, int64_t n_sb, bool pad) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;  // one thread per 2 bytes
    if (i >= n_sb * 112) return;
    const int64_t sb = i / 112;
    const int w = (int)(i % 112);
    if (pad) {
        const uint16_t v = w < 105 ? *reinterpret_cast<const uint16_t *>(src + sb * 210 + 2 * w) : (uint16_t)0;
        *reinterpret_cast<uint16_t *>(dst + sb * 224 + 2 * w) = v;
    } else if (w < 105) {
        *reinterpret_cast<uint16_t *>(dst + sb * 210 + 2 * w) = *reinterpret_cast<const uint16_t *>(src + sb * 224 + 2 * w);
    }
}

__global__ void copy_rows_f16_kernel(const uint8_t *__restrict__ data, size_t row_pitch, int64_t n_cols,
                                     int64_t n_rows, __half *__restrict__ out) {
    int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n_rows * n_cols) return;
    int64_t r = i / n_cols, c = i % n_cols;
    out[i] = reinterpret_cast<const __half *>(data + r * row_pitch)[c];
}

// ---------------------------------------------------------------------------
// Synthetic blocks generated in place (one thread per block).  The byte
// stream is defined by tlc_synth.cuh and restated in numpy by the Python
// package so that host- and device-generated weights are identical.
// ---------------------------------------------------------------------------
__global__ void synth_blocks_kernel(uint8_t *__restrict__ data, int64_t ktiles, int type,
                                    int blocks_per_row, int64_t n_rows, int64_t row0, int64_t bc0,
                                    int64_t full_blocks_per_row, uint64_t key, int scale_log2) {
    int64_t lb = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (lb >= n_rows * blocks_per_row) return;
    int64_t row = lb / blocks_per_row;
    int bc = (int)(lb % blocks_per_row);
    uint64_t gb = (uint64_t)((row0 + row) * full_blocks_per_row + bc0 + bc);
    __align__(8) uint8_t blk[40];
    if (type == TLC_TYPE_Q4_0)
        tlc_synth_q4_0_block(key, gb, scale_log2, blk);
    else
        tlc_synth_q8_0_block(key, gb, scale_log2, blk);
    tlc_tile::store_block(data, type, ktiles, row, bc, blk);
}

// ---------------------------------------------------------------------------

static int32_t shard_shape(int32_t type, int64_t n_rows, int64_t n_cols, int32_t tp_rank, int32_t tp_size,
                           int32_t split, int64_t *rows, int64_t *cols, int64_t *row0, int64_t *col0) {
    TLC_REQUIRE(type == TLC_TYPE_F16 || type == TLC_TYPE_F32 || type == TLC_TYPE_Q4_0 || type == TLC_TYPE_Q8_0 ||
                    type == TLC_TYPE_Q6_K,
                TLC_ERR_LOAD, "unsupported GGUF tensor type %d (supported: F32, F16, Q4_0, Q8_0, Q6_K)", type);
    TLC_REQUIRE(n_rows > 0 && n_cols > 0, TLC_ERR_INVALID_DIMENSION, "tensor shape [%lld, %lld] is empty",
                (long long)n_rows, (long long)n_cols);
    bool quant = type == TLC_TYPE_Q4_0 || type == TLC_TYPE_Q8_0;
    TLC_REQUIRE(!quant || n_cols % 32 == 0, TLC_ERR_LOAD,
                "quantized tensor needs columns in multiples of 32 (got %lld)", (long long)n_cols);
    TLC_REQUIRE(tp_size >= 1 && tp_rank >= 0 && tp_rank < tp_size, TLC_ERR_INVALID_OPERATION,
                "bad tensor-parallel rank %d of %d", tp_rank, tp_size);
    *rows = n_rows;
    *cols = n_cols;
    *row0 = 0;
    *col0 = 0;
    if (tp_size > 1 && split == TLC_SPLIT_ROWS) {
        TLC_REQUIRE(n_rows % tp_size == 0, TLC_ERR_SHAPE_MISMATCH,
                    "rows %lld do not divide over %d ranks", (long long)n_rows, tp_size);
        *rows = n_rows / tp_size;
        *row0 = *rows * tp_rank;
    } else if (tp_size > 1 && split == TLC_SPLIT_COLS) {
        int64_t unit = quant ? 32 : 1;
        TLC_REQUIRE((n_cols / unit) % tp_size == 0, TLC_ERR_SHAPE_MISMATCH,
                    "columns %lld do not divide over %d ranks in units of %lld", (long long)n_cols, tp_size,
                    (long long)unit);
        *cols = n_cols / tp_size;
        *col0 = *cols * tp_rank;
    } else {
        TLC_REQUIRE(tp_size == 1 || split == TLC_SPLIT_NONE, TLC_ERR_INVALID_OPERATION, "bad split mode %d",
                    split);
    }
    return TLC_OK;
}

static size_t bytes_per_row(int32_t type, int64_t cols) {
    if (type == TLC_TYPE_Q4_0) return (size_t)(cols / 32) * 18;
    if (type == TLC_TYPE_Q8_0) return (size_t)(cols / 32) * 34;
    if (type == TLC_TYPE_Q6_K) return (size_t)(cols / 256) * 210;
    return (size_t)cols * 2;  // F16 (F32 is converted on the host first)
}

static int32_t alloc_qtensor(tlc_ctx *ctx, int32_t type, int64_t rows, int64_t cols, int64_t full_rows,
                             int64_t full_cols, int32_t tp_rank, int32_t tp_size, int32_t split,
                             tlc_qtensor **out) {
    tlc_qtensor *qt = new tlc_qtensor();
    qt->ctx = ctx;
    qt->type = type == TLC_TYPE_F32 ? TLC_TYPE_F16 : type;
    qt->n_rows = rows;
    qt->n_cols = cols;
    qt->full_rows = full_rows;
    qt->full_cols = full_cols;
    qt->row_bytes = bytes_per_row(qt->type, cols);
    if (qt->type == TLC_TYPE_Q4_0 || qt->type == TLC_TYPE_Q8_0) {
        // Tiles of 16 rows; rows past N and blocks past K stay zero.
        qt->row_pitch = 0;
        qt->k_tiles = tlc_tile::k_tiles(qt->type, cols);
        qt->slab_pitch = (size_t)qt->k_tiles * tlc_tile::tile_bytes(qt->type);
        qt->bytes = qt->slab_pitch * (size_t)tlc_tile::slabs(rows);
    } else if (qt->type == TLC_TYPE_Q6_K) {
        // Resident Q6_K: rows of 224-byte padded super-blocks (q6k_repad_kernel).
        qt->row_pitch = (size_t)(cols / 256) * 224;
        qt->k_tiles = 0;
        qt->slab_pitch = 0;
        qt->bytes = qt->row_pitch * (size_t)rows;
    } else {
        // Dense rows start on 16-byte boundaries.
        qt->row_pitch = (qt->row_bytes + 15) & ~(size_t)15;
        qt->k_tiles = 0;
        qt->slab_pitch = 0;
        qt->bytes = qt->row_pitch * (size_t)rows;
    }
    qt->tp_rank = tp_rank;
    qt->tp_size = tp_size;
    qt->split = split;
    cudaError_t e = cudaMalloc(&qt->data, qt->bytes + 16);
    if (e != cudaSuccess) {
        cudaGetLastError();
        size_t want = qt->bytes;
        delete qt;
        return tlc_fail(TLC_ERR_ALLOCATION, "weight allocation of %zu bytes failed: %s", want,
                        cudaGetErrorString(e));
    }
    *out = qt;
    return TLC_OK;
}

extern "C" int32_t tlc_qtensor_create(tlc_ctx *ctx, int32_t type, int64_t n_rows, int64_t n_cols,
                                      const void *blocks, size_t bytes, int32_t tp_rank, int32_t tp_size,
                                      int32_t split, tlc_qtensor **out) {
    if (int32_t rc = tlc_enter(ctx)) return rc;
    TLC_REQUIRE(out && blocks, TLC_ERR_INVALID_OPERATION, "tlc_qtensor_create: null pointer");
    *out = nullptr;
    int64_t rows, cols, row0, col0;
    if (int32_t rc = shard_shape(type, n_rows, n_cols, tp_rank, tp_size, split, &rows, &cols, &row0, &col0))
        return rc;
    size_t src_row_bytes = type == TLC_TYPE_F32 ? (size_t)n_cols * 4 : bytes_per_row(type, n_cols);
    {
        size_t need = 0;
        TLC_REQUIRE(!__builtin_mul_overflow(src_row_bytes, (size_t)n_rows, &need), TLC_ERR_INVALID_DIMENSION,
                    "qtensor_create: [%lld, %lld] overflows the byte count", (long long)n_rows, (long long)n_cols);
    }
    TLC_REQUIRE(type == TLC_TYPE_Q6_K || bytes >= src_row_bytes * (size_t)n_rows, TLC_ERR_LOAD,
                "tensor data too short: %zu bytes for shape [%lld, %lld] (need %zu)", bytes, (long long)n_rows,
                (long long)n_cols, src_row_bytes * (size_t)n_rows);
    if (type == TLC_TYPE_Q6_K) {
        TLC_REQUIRE(n_cols % 256 == 0, TLC_ERR_LOAD, "Q6_K tensor needs columns in multiples of 256 (got %lld)",
                    (long long)n_cols);
        const int sb_per_row = (int)(n_cols / 256);
        const size_t q_row_bytes = (size_t)sb_per_row * 210;
        TLC_REQUIRE(bytes >= q_row_bytes * (size_t)n_rows, TLC_ERR_LOAD,
                    "tensor data too short: %zu bytes for Q6_K shape [%lld, %lld] (need %zu)", bytes, (long long)n_rows,
                    (long long)n_cols, q_row_bytes * (size_t)n_rows);
        if (ctx->q6k_resident && cols == n_cols) {
            // Whole rows (no column shard): the super-blocks stay quantized in HBM, 0.875 bytes per
            // weight instead of the 2 of an f16 copy; linear() runs on them directly.
            tlc_qtensor *qt = nullptr;
            if (int32_t rc = alloc_qtensor(ctx, TLC_TYPE_Q6_K, rows, cols, n_rows, n_cols, tp_rank, tp_size, split, &qt))
                return rc;
            void *tmp = nullptr;
            const int64_t n_sb = rows * sb_per_row;
            cudaError_t e = cudaMalloc(&tmp, q_row_bytes * (size_t)rows);
            if (e == cudaSuccess)
                e = cudaMemcpyAsync(tmp, static_cast<const uint8_t *>(blocks) + (size_t)row0 * q_row_bytes,
                                    q_row_bytes * (size_t)rows, cudaMemcpyHostToDevice, ctx->stream);
            if (e == cudaSuccess) {
                q6k_repad_kernel<<<(unsigned)((n_sb * 112 + 255) / 256), 256, 0, ctx->stream>>>(
                    static_cast<const uint8_t *>(tmp), static_cast<uint8_t *>(qt->data), n_sb, true);
                ctx->launches++;
                e = cudaGetLastError();
            }
            if (e == cudaSuccess) e = cudaStreamSynchronize(ctx->stream);
            cudaFree(tmp);
            if (e != cudaSuccess) {
                cudaGetLastError();
                cudaFree(qt->data);
                delete qt;
                return tlc_fail(TLC_ERR_CUDA, "Q6_K upload failed: %s", cudaGetErrorString(e));
            }
            *out = qt;
            return TLC_OK;
        }
        // A column shard (or option "q6k_resident" = 0): dequantized on the device into an F16
        // tensor, which is what the reference's loader keeps in memory.
        tlc_qtensor *qt = nullptr;
        if (int32_t rc = alloc_qtensor(ctx, TLC_TYPE_F16, rows, cols, n_rows, n_cols, tp_rank, tp_size, split, &qt))
            return rc;
        void *tmp = nullptr;
        cudaError_t e = cudaMalloc(&tmp, q_row_bytes * (size_t)rows);
        if (e == cudaSuccess) e = cudaMemsetAsync(qt->data, 0, qt->bytes + 16, ctx->stream);
        if (e == cudaSuccess)
            e = cudaMemcpyAsync(tmp, static_cast<const uint8_t *>(blocks) + (size_t)row0 * q_row_bytes,
                                q_row_bytes * (size_t)rows, cudaMemcpyHostToDevice, ctx->stream);
        if (e == cudaSuccess) {
            const int64_t total = rows * sb_per_row * 64;
            dequant_q6_k_kernel<<<(unsigned)((total + 255) / 256), 256, 0, ctx->stream>>>(
                static_cast<const uint8_t *>(tmp), sb_per_row, 210, rows, col0, cols, static_cast<__half *>(qt->data),
                qt->row_pitch);
            ctx->launches++;
            e = cudaGetLastError();
        }
        if (e == cudaSuccess) e = cudaStreamSynchronize(ctx->stream);
        cudaFree(tmp);
        if (e != cudaSuccess) {
            cudaGetLastError();
            cudaFree(qt->data);
            delete qt;
            return tlc_fail(TLC_ERR_CUDA, "Q6_K upload failed: %s", cudaGetErrorString(e));
        }
        *out = qt;
        return TLC_OK;
    }
    tlc_qtensor *qt = nullptr;
    if (int32_t rc = alloc_qtensor(ctx, type, rows, cols, n_rows, n_cols, tp_rank, tp_size, split, &qt)) return rc;

    const uint8_t *src = static_cast<const uint8_t *>(blocks);
    std::vector<__half> conv;
    size_t src_pitch = src_row_bytes;
    size_t col_off;
    if (type == TLC_TYPE_F32) {
        // f32 -> f16 with round-to-nearest-even (half::f16::from_f32, gguf.rs:384-395).
        conv.resize((size_t)rows * cols);
        const float *f = reinterpret_cast<const float *>(src);
        for (int64_t r = 0; r < rows; r++)
            for (int64_t c = 0; c < cols; c++)
                conv[(size_t)r * cols + c] = __float2half_rn(f[(size_t)(row0 + r) * n_cols + col0 + c]);
        src = reinterpret_cast<const uint8_t *>(conv.data());
        src_pitch = (size_t)cols * 2;
        row0 = 0;
        col_off = 0;
    } else if (type == TLC_TYPE_F16) {
        col_off = (size_t)col0 * 2;
    } else {
        col_off = (size_t)(col0 / 32) * tlc_block_bytes(type);
    }
    cudaError_t e = cudaMemsetAsync(qt->data, 0, qt->bytes + 16, ctx->stream);
    void *tmp = nullptr;
    if (qt->slab_pitch) {
        // The shard's rows go to a staging buffer as the file has them; a kernel regroups them.
        if (e == cudaSuccess) e = cudaMalloc(&tmp, qt->row_bytes * (size_t)rows);
        if (e == cudaSuccess)
            e = cudaMemcpy2DAsync(tmp, qt->row_bytes, src + (size_t)row0 * src_pitch + col_off, src_pitch,
                                  qt->row_bytes, (size_t)rows, cudaMemcpyHostToDevice, ctx->stream);
        if (e == cudaSuccess) {
            const int bpr = (int)(cols / 32);
            const int64_t total = rows * bpr;
            tile_blocks_kernel<<<(unsigned)((total + 255) / 256), 256, 0, ctx->stream>>>(
                static_cast<const uint8_t *>(tmp), qt->row_bytes, qt->type, bpr, rows, qt->k_tiles,
                static_cast<uint8_t *>(qt->data));
            ctx->launches++;
            e = cudaGetLastError();
        }
    } else if (e == cudaSuccess) {
        e = cudaMemcpy2DAsync(qt->data, qt->row_pitch, src + (size_t)row0 * src_pitch + col_off, src_pitch,
                              qt->row_bytes, (size_t)rows, cudaMemcpyHostToDevice, ctx->stream);
    }
    if (e == cudaSuccess) e = cudaStreamSynchronize(ctx->stream);  // `blocks`/`conv` may go away
    if (tmp) cudaFree(tmp);
    if (e != cudaSuccess) {
        cudaGetLastError();
        cudaFree(qt->data);
        delete qt;
        return tlc_fail(TLC_ERR_CUDA, "weight upload failed: %s", cudaGetErrorString(e));
    }
    *out = qt;
    return TLC_OK;
}

extern "C" int32_t tlc_qtensor_create_synthetic(tlc_ctx *ctx, int32_t type, int64_t n_rows, int64_t n_cols,
                                                uint64_t seed, uint64_t tensor_id, int32_t scale_log2,
                                                int32_t tp_rank, int32_t tp_size, int32_t split,
                                                tlc_qtensor **out) {
    if (int32_t rc = tlc_enter(ctx)) return rc;
    TLC_REQUIRE(out, TLC_ERR_INVALID_OPERATION, "tlc_qtensor_create_synthetic: null pointer");
    *out = nullptr;
    TLC_REQUIRE(type == TLC_TYPE_Q4_0 || type == TLC_TYPE_Q8_0, TLC_ERR_INVALID_OPERATION,
                "synthetic weights exist for Q4_0 and Q8_0 only (got type %d)", type);
    int64_t rows, cols, row0, col0;
    if (int32_t rc = shard_shape(type, n_rows, n_cols, tp_rank, tp_size, split, &rows, &cols, &row0, &col0))
        return rc;
    tlc_qtensor *qt = nullptr;
    if (int32_t rc = alloc_qtensor(ctx, type, rows, cols, n_rows, n_cols, tp_rank, tp_size, split, &qt)) return rc;
    cudaError_t e = cudaMemsetAsync(qt->data, 0, qt->bytes + 16, ctx->stream);
    if (e != cudaSuccess) {
        cudaFree(qt->data);
        delete qt;
        return tlc_fail(TLC_ERR_CUDA, "memset failed: %s", cudaGetErrorString(e));
    }
    int bpr = (int)(cols / 32);
    int64_t total = rows * bpr;
    int threads = 256;
    int64_t grid = (total + threads - 1) / threads;
    synth_blocks_kernel<<<(unsigned)grid, threads, 0, ctx->stream>>>(
        static_cast<uint8_t *>(qt->data), qt->k_tiles, type, bpr, rows, row0, col0 / 32, n_cols / 32,
        tlc_synth_key(seed, tensor_id), scale_log2);
    ctx->launches++;
    e = cudaGetLastError();
    if (e != cudaSuccess) {
        cudaFree(qt->data);
        delete qt;
        return tlc_fail(TLC_ERR_CUDA, "generator launch failed: %s", cudaGetErrorString(e));
    }
    *out = qt;
    return TLC_OK;
}

extern "C" int32_t tlc_synth_blocks_host(int32_t type, uint64_t seed, uint64_t tensor_id, int32_t scale_log2,
                                         int64_t first_block, int64_t n_blocks, void *out_host) {
    TLC_REQUIRE(type == TLC_TYPE_Q4_0 || type == TLC_TYPE_Q8_0, TLC_ERR_INVALID_OPERATION,
                "synthetic weights exist for Q4_0 and Q8_0 only (got type %d)", type);
    TLC_REQUIRE(out_host && first_block >= 0 && n_blocks >= 0, TLC_ERR_INVALID_OPERATION,
                "tlc_synth_blocks_host: bad arguments");
    const uint64_t key = tlc_synth_key(seed, tensor_id);
    uint8_t *o = static_cast<uint8_t *>(out_host);
    const size_t bb = tlc_block_bytes(type);
    for (int64_t i = 0; i < n_blocks; i++) {
        if (type == TLC_TYPE_Q4_0)
            tlc_synth_q4_0_block(key, (uint64_t)(first_block + i), scale_log2, o + (size_t)i * bb);
        else
            tlc_synth_q8_0_block(key, (uint64_t)(first_block + i), scale_log2, o + (size_t)i * bb);
    }
    return TLC_OK;
}

// f16 N(mean, std) from the same counter-based uniforms (Box-Muller); used for
// device-side filling of large f16 tensors of the benchmark configurations
// (embedding tables, a pre-filled KV cache).  Not bit-matched with the host
// generator's f64 Box-Muller: parity tests always upload host-generated f16 data.
__global__ void fill_normal_f16_kernel(__half *__restrict__ out, size_t n, uint64_t key, float mean, float std) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const uint64_t r1 = tlc_mix64(key + 2 * i), r2 = tlc_mix64(key + 2 * i + 1);
    const float u1 = ((float)(r1 >> 40) + 0.5f) * (1.0f / 16777216.0f);
    const float u2 = ((float)(r2 >> 40) + 0.5f) * (1.0f / 16777216.0f);
    const float z = sqrtf(-2.0f * logf(u1)) * cospif(2.0f * u2);
    out[i] = __float2half_rn(mean + std * z);
}

extern "C" int32_t tlc_fill_normal_f16(tlc_ctx *ctx, void *dst_dev, size_t n, uint64_t seed, uint64_t tensor_id,
                                       float mean, float std) {
    if (int32_t rc = tlc_enter(ctx)) return rc;
    TLC_REQUIRE(dst_dev, TLC_ERR_INVALID_OPERATION, "fill_normal_f16: null pointer");
    if (n == 0) return TLC_OK;
    fill_normal_f16_kernel<<<(unsigned)((n + 255) / 256), 256, 0, ctx->stream>>>(
        static_cast<__half *>(dst_dev), n, tlc_synth_key(seed, tensor_id), mean, std);
    TLC_CHECK_LAUNCH(ctx);
    return TLC_OK;
}

extern "C" int32_t tlc_qtensor_create_normal_f16(tlc_ctx *ctx, int64_t n_rows, int64_t n_cols, uint64_t seed,
                                                 uint64_t tensor_id, float mean, float std, tlc_qtensor **out) {
    if (int32_t rc = tlc_enter(ctx)) return rc;
    TLC_REQUIRE(out, TLC_ERR_INVALID_OPERATION, "qtensor_create_normal_f16: null pointer");
    *out = nullptr;
    TLC_REQUIRE(n_rows > 0 && n_cols > 0 && n_cols % 8 == 0, TLC_ERR_INVALID_DIMENSION,
                "f16 tensor shape [%lld, %lld] (columns must be a multiple of 8)", (long long)n_rows, (long long)n_cols);
    tlc_qtensor *qt = nullptr;
    if (int32_t rc = alloc_qtensor(ctx, TLC_TYPE_F16, n_rows, n_cols, n_rows, n_cols, 0, 1, TLC_SPLIT_NONE, &qt)) return rc;
    // n_cols % 8 == 0 makes the row pitch equal to the row size: one flat fill.
    if (int32_t rc = tlc_fill_normal_f16(ctx, qt->data, (size_t)n_rows * n_cols, seed, tensor_id, mean, std)) {
        cudaFree(qt->data);
        delete qt;
        return rc;
    }
    *out = qt;
    return TLC_OK;
}

extern "C" int32_t tlc_qtensor_destroy(tlc_qtensor *qt) {
    if (!qt) return TLC_OK;
    cudaSetDevice(qt->ctx->device);
    cudaFree(qt->data);  // waits for queued work that still reads it
    delete qt;
    return TLC_OK;
}

extern "C" int32_t tlc_qtensor_info(tlc_qtensor *qt, int32_t *type, int64_t *n_rows, int64_t *n_cols,
                                    size_t *row_pitch, const void **dev_ptr) {
    TLC_REQUIRE(qt != nullptr, TLC_ERR_INVALID_OPERATION, "tlc_qtensor_info: null tensor");
    if (type) *type = qt->type;
    if (n_rows) *n_rows = qt->n_rows;
    if (n_cols) *n_cols = qt->n_cols;
    if (row_pitch) *row_pitch = qt->slab_pitch ? qt->row_bytes : qt->row_pitch;
    if (dev_ptr) *dev_ptr = qt->data;
    return TLC_OK;
}

// A dense F16 copy of a quantized tensor (same shape and shard).
int32_t tlc_qtensor_to_f16(tlc_ctx *ctx, tlc_qtensor *qt, tlc_qtensor **out) {
    TLC_REQUIRE(qt && out, TLC_ERR_INVALID_OPERATION, "qtensor_to_f16: null pointer");
    TLC_REQUIRE(qt->n_cols % 8 == 0, TLC_ERR_INVALID_DIMENSION, "qtensor_to_f16: %lld columns are not a multiple of 8",
                (long long)qt->n_cols);
    tlc_qtensor *dense = nullptr;
    if (int32_t rc = alloc_qtensor(ctx, TLC_TYPE_F16, qt->n_rows, qt->n_cols, qt->full_rows, qt->full_cols,
                                   qt->tp_rank, qt->tp_size, qt->split, &dense))
        return rc;
    int32_t rc = tlc_dequant(ctx, qt, dense->data);  // pitch == 2 * cols: the dense layout tlc_dequant writes
    if (!rc) rc = tlc_synchronize(ctx);
    if (rc) {
        cudaFree(dense->data);
        delete dense;
        return rc;
    }
    *out = dense;
    return TLC_OK;
}

extern "C" int32_t tlc_dequant(tlc_ctx *ctx, tlc_qtensor *qt, void *out_f16_dev) {
    if (int32_t rc = tlc_enter(ctx)) return rc;
    TLC_REQUIRE(qt && out_f16_dev, TLC_ERR_INVALID_OPERATION, "tlc_dequant: null pointer");
    TLC_REQUIRE(qt->ctx->device == ctx->device, TLC_ERR_DEVICE, "tlc_dequant: tensor lives on device %d, context on %d",
                qt->ctx->device, ctx->device);
    const int threads = 256;
    const uint8_t *data = static_cast<const uint8_t *>(qt->data);
    __half *out = static_cast<__half *>(out_f16_dev);
    if (qt->type == TLC_TYPE_F16) {
        int64_t total = qt->n_rows * qt->n_cols;
        copy_rows_f16_kernel<<<(unsigned)((total + threads - 1) / threads), threads, 0, ctx->stream>>>(
            data, qt->row_pitch, qt->n_cols, qt->n_rows, out);
    } else if (qt->type == TLC_TYPE_Q6_K) {
        const int sb_per_row = (int)(qt->n_cols / 256);
        const int64_t total = qt->n_rows * sb_per_row * 64;
        dequant_q6_k_kernel<<<(unsigned)((total + threads - 1) / threads), threads, 0, ctx->stream>>>(
            data, sb_per_row, 224, qt->n_rows, 0, qt->n_cols, out, (size_t)qt->n_cols * 2);
    } else {
        int bpr = (int)(qt->n_cols / 32);
        int64_t total = qt->n_rows * bpr;
        unsigned grid = (unsigned)((total + threads - 1) / threads);
        if (qt->type == TLC_TYPE_Q4_0)
            dequant_q4_0_kernel<<<grid, threads, 0, ctx->stream>>>(data, qt->k_tiles, bpr, qt->n_rows, out);
        else
            dequant_q8_0_kernel<<<grid, threads, 0, ctx->stream>>>(data, qt->k_tiles, bpr, qt->n_rows, out);
    }
    TLC_CHECK_LAUNCH(ctx);
    return TLC_OK;
}

extern "C" int32_t tlc_qtensor_blocks(tlc_ctx *ctx, tlc_qtensor *qt, void *out_dev) {
    if (int32_t rc = tlc_enter(ctx)) return rc;
    TLC_REQUIRE(qt && out_dev, TLC_ERR_INVALID_OPERATION, "tlc_qtensor_blocks: null pointer");
    TLC_REQUIRE(qt->ctx->device == ctx->device, TLC_ERR_DEVICE, "tlc_qtensor_blocks: tensor lives on device %d, context on %d",
                qt->ctx->device, ctx->device);
    if (qt->type == TLC_TYPE_Q6_K) {
        const int64_t n_sb = qt->n_rows * (qt->n_cols / 256);
        q6k_repad_kernel<<<(unsigned)((n_sb * 112 + 255) / 256), 256, 0, ctx->stream>>>(
            static_cast<const uint8_t *>(qt->data), static_cast<uint8_t *>(out_dev), n_sb, false);
        TLC_CHECK_LAUNCH(ctx);
        return TLC_OK;
    }
    if (!qt->slab_pitch) {
        TLC_CUDA(cudaMemcpy2DAsync(out_dev, qt->row_bytes, qt->data, qt->row_pitch, qt->row_bytes, (size_t)qt->n_rows,
                                   cudaMemcpyDeviceToDevice, ctx->stream));
        return TLC_OK;
    }
    const int bpr = (int)(qt->n_cols / 32);
    const int64_t total = qt->n_rows * bpr;
    untile_blocks_kernel<<<(unsigned)((total + 255) / 256), 256, 0, ctx->stream>>>(
        static_cast<const uint8_t *>(qt->data), qt->type, bpr, qt->n_rows, qt->k_tiles, static_cast<uint8_t *>(out_dev));
    TLC_CHECK_LAUNCH(ctx);
    return TLC_OK;
}

extern "C" size_t tlc_tiled_bytes(int32_t type, int64_t n_rows, int64_t n_cols) {
    if ((type != TLC_TYPE_Q4_0 && type != TLC_TYPE_Q8_0) || n_rows <= 0 || n_cols <= 0) return 0;
    return (size_t)tlc_tile::slabs(n_rows) * (size_t)tlc_tile::k_tiles(type, n_cols) * tlc_tile::tile_bytes(type);
}

extern "C" int32_t tlc_tile_blocks_host(int32_t type, int64_t n_rows, int64_t n_cols, const void *blocks,
                                        void *tiles_out) {
    TLC_REQUIRE(type == TLC_TYPE_Q4_0 || type == TLC_TYPE_Q8_0, TLC_ERR_INVALID_OPERATION,
                "tile_blocks_host: type %d is not stored in tiles", type);
    TLC_REQUIRE(blocks && tiles_out && n_rows > 0 && n_cols > 0 && n_cols % 32 == 0, TLC_ERR_INVALID_OPERATION,
                "tile_blocks_host: bad arguments");
    const int64_t bpr = n_cols / 32, ktiles = tlc_tile::k_tiles(type, n_cols);
    const int bb = tlc_tile::block_bytes(type);
    uint8_t *dst = static_cast<uint8_t *>(tiles_out);
    memset(dst, 0, tlc_tiled_bytes(type, n_rows, n_cols));
    const uint8_t *src = static_cast<const uint8_t *>(blocks);
    for (int64_t r = 0; r < n_rows; r++)
        for (int64_t b = 0; b < bpr; b++) tlc_tile::store_block(dst, type, ktiles, r, b, src + (size_t)(r * bpr + b) * bb);
    return TLC_OK;
}
