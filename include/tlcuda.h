/*
 * tlcuda.h -- C ABI of libtlcuda, the CUDA (sm_100a) device layer that takes
 * the place of TensorLogic's Metal device layer for the quantized-LLM path.
 *
 * TensorLogic has no FFI for this path: its ops call Rust methods on
 * MetalDevice / MetalBuffer / BufferPool / Commands / KernelExecutor
 * (the files of src/device).  Each entry point below names the Rust item it replaces,
 * by path within the TensorLogic project.
 *
 * Conventions
 *  - plain C, opaque handles, every call returns an int32_t status
 *    (0 = TLC_OK, negative = error); tlc_last_error() gives the message of the
 *    calling thread's last failing call.
 *  - "device pointer" arguments are raw CUDA device addresses (from
 *    tlc_buf_ptr, or any other allocation of the same device);
 *    f16 data is IEEE binary16, row-major.
 *  - ops are asynchronous: they are enqueued on the context's stream and
 *    return at once, like the reference's command-buffer encoding
 *    (src/ops/matmul.rs:414-438 returns without waiting).  tlc_download and
 *    tlc_synchronize are the blocking points (src/tensor/tensor_io.rs:103-135).
 *  - one tlc_ctx per GPU per host thread; handles are not thread-safe (the
 *    interpreter above is single-threaded).
 *  - there is no CPU fallback: without a CUDA device tlc_init fails.
 */
#ifndef TLCUDA_H
#define TLCUDA_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(_WIN32)
#define TLC_API
#else
#define TLC_API __attribute__((visibility("default")))
#endif

/* Status codes; the negative ones map 1:1 onto TensorError variants
 * (src/error.rs:9-49). */
enum {
    TLC_OK = 0,
    TLC_ERR_SHAPE_MISMATCH = -1,    /* TensorError::ShapeMismatch          */
    TLC_ERR_INVALID_OPERATION = -2, /* TensorError::InvalidOperation       */
    TLC_ERR_DEVICE = -3,            /* TensorError::DeviceConversionError  */
    TLC_ERR_CUDA = -4,              /* TensorError::MetalError             */
    TLC_ERR_ALLOCATION = -5,        /* TensorError::AllocationError        */
    TLC_ERR_LOAD = -6,              /* TensorError::LoadError              */
    TLC_ERR_BUFFER_EXHAUSTED = -7,  /* TensorError::BufferExhausted        */
    TLC_ERR_INDEX = -8,             /* TensorError::IndexOutOfBounds       */
    TLC_ERR_INVALID_DIMENSION = -9, /* TensorError::InvalidDimension       */
    TLC_ERR_TIMEOUT = -10,          /* a bounded device-side wait ran out  */
    TLC_ERR_COMM = -11              /* collective / communicator failure   */
};

/* GGUF tensor type ids (src/model/formats/mmap_gguf.rs:30-45). */
enum { TLC_TYPE_F32 = 0, TLC_TYPE_F16 = 1, TLC_TYPE_Q4_0 = 2, TLC_TYPE_Q8_0 = 8 };

/* How a weight is split across tensor-parallel ranks. */
enum {
    TLC_SPLIT_NONE = 0,
    TLC_SPLIT_ROWS = 1, /* column-parallel linear: rank keeps N/tp output rows       */
    TLC_SPLIT_COLS = 2  /* row-parallel linear: rank keeps K/tp input columns per row */
};

typedef struct tlc_ctx tlc_ctx;
typedef struct tlc_buf tlc_buf;
typedef struct tlc_qtensor tlc_qtensor;
typedef struct tlc_model tlc_model;
typedef struct tlc_llama tlc_llama;

TLC_API const char *tlc_last_error(void);
TLC_API const char *tlc_version(void);

/* ---- device ------------------------------------------------------------ */

/* Replaces MetalDevice::new (src/device/metal_device.rs:36-74).  Creates a
 * context on CUDA device `ordinal` with its own stream.  Fails with
 * TLC_ERR_DEVICE when no CUDA device is present. */
TLC_API int32_t tlc_init(int32_t ordinal, tlc_ctx **out);
TLC_API int32_t tlc_destroy(tlc_ctx *ctx);
/* MetalDevice::name (metal_device.rs:89). */
TLC_API int32_t tlc_device_name(tlc_ctx *ctx, char *buf, size_t buflen);
/* recommended_max_working_set_size / current_allocated_size and the pre-load
 * check check_memory_available (metal_device.rs:279-333). */
TLC_API int32_t tlc_mem_info(tlc_ctx *ctx, size_t *free_bytes, size_t *total_bytes);
TLC_API int32_t tlc_sm_count(tlc_ctx *ctx, int32_t *out);
/* MetalDevice::wait_until_completed (metal_device.rs:195, commands.rs:189-289).
 * Also reports a device-side bounded wait that ran out as TLC_ERR_TIMEOUT. */
TLC_API int32_t tlc_synchronize(tlc_ctx *ctx);
/* The CUDA stream (cudaStream_t) all ops of this context are enqueued on. */
TLC_API void *tlc_stream(tlc_ctx *ctx);
/* Number of kernels this context has launched since creation (TL_PERF-style
 * accounting, src/device/kernel_executor.rs:33-41). */
TLC_API uint64_t tlc_launch_count(tlc_ctx *ctx);

/* ---- allocator --------------------------------------------------------- */

/* Mirrors PoolStats (src/device/buffer_pool.rs:15-29). */
typedef struct tlc_pool_stats {
    uint64_t total_pooled;     /* buffers idle in the pool            */
    uint64_t size_classes;     /* distinct sizes with an idle buffer  */
    uint64_t total_memory;     /* bytes held idle                     */
    uint64_t reuse_count;      /* allocations served from the pool    */
    uint64_t allocation_count; /* allocations that hit cudaMalloc     */
    uint64_t eviction_count;   /* idle buffers released to the driver */
    uint64_t live_bytes;       /* bytes currently handed out          */
} tlc_pool_stats;

/* BufferPool::allocate (buffer_pool.rs:137): size-class pool, 14 power-of-two
 * classes 2 KiB..16 MiB, exact size above (buffer_pool.rs:78-101).  Memory is
 * not zeroed on reuse (buffer_pool.rs:222-230). */
TLC_API int32_t tlc_alloc(tlc_ctx *ctx, size_t bytes, tlc_buf **out);
/* BufferPool::try_return_buffer (buffer_pool.rs:426-499).  Stream-ordered:
 * safe to call while kernels using the buffer are still queued. */
TLC_API int32_t tlc_free(tlc_buf *buf);
TLC_API void *tlc_buf_ptr(tlc_buf *buf);
TLC_API size_t tlc_buf_size(tlc_buf *buf);
/* BufferPool::stats (buffer_pool.rs:514-534). */
TLC_API int32_t tlc_pool_stats_get(tlc_ctx *ctx, tlc_pool_stats *out);
/* BufferPool::shrink_to_fit / clear: release idle buffers until at most
 * max_idle_bytes stay pooled. */
TLC_API int32_t tlc_pool_trim(tlc_ctx *ctx, size_t max_idle_bytes);

/* ---- transfer ---------------------------------------------------------- */

/* MetalBuffer::from_vec_pooled / from_slice (src/device/metal_buffer.rs:226,
 * :37): host -> device, enqueued on the stream. */
TLC_API int32_t tlc_upload(tlc_ctx *ctx, void *dst_dev, const void *src_host, size_t bytes);
/* MetalBuffer::to_vec (metal_buffer.rs:113-134): waits for the stream, then
 * device -> host. */
TLC_API int32_t tlc_download(tlc_ctx *ctx, void *dst_host, const void *src_dev, size_t bytes);
/* Page-locked host staging memory for the end-to-end path. */
TLC_API int32_t tlc_host_alloc(size_t bytes, void **out);
TLC_API int32_t tlc_host_free(void *p);

/* ---- quantized weights -------------------------------------------------- */

/* Replaces the load-time CPU dequantization (GGUFLoader::dequantize_q4_0 /
 * dequantize_q8_0, src/model/formats/gguf.rs:22-112, and the upload at
 * gguf.rs:450): the GGUF blocks of W [n_rows, n_cols] (row-major, n_cols
 * fastest; 18-byte Q4_0 / 34-byte Q8_0 blocks of 32 along a row) are copied to
 * HBM unchanged.  `blocks` is a HOST pointer to the FULL tensor; with
 * tp_size > 1 only this rank's shard is kept (rows [r*N/tp, (r+1)*N/tp) for
 * TLC_SPLIT_ROWS; block columns [r*K/tp, (r+1)*K/tp) of every row for
 * TLC_SPLIT_COLS).  F16 and F32 tensors are accepted too (F32 is converted
 * to f16 with round-to-nearest-even as Tensor::from_vec_gpu does after the
 * loader's f32 -> f16 cast, gguf.rs:384-395). */
TLC_API int32_t tlc_qtensor_create(tlc_ctx *ctx, int32_t type, int64_t n_rows, int64_t n_cols,
                                   const void *blocks, size_t bytes, int32_t tp_rank,
                                   int32_t tp_size, int32_t split, tlc_qtensor **out);
/* Same, but the shard is filled on the device from the counter-based
 * generator of the benchmark configurations (weights too large to stage on
 * the host).  Only Q4_0 / Q8_0. */
TLC_API int32_t tlc_qtensor_create_synthetic(tlc_ctx *ctx, int32_t type, int64_t n_rows,
                                             int64_t n_cols, uint64_t seed, uint64_t tensor_id,
                                             int32_t tp_rank, int32_t tp_size, int32_t split,
                                             tlc_qtensor **out);
/* The same generator on the host (no GPU needed): writes n_blocks consecutive
 * blocks of the full tensor, starting at block index first_block (row-major
 * block order), into out_host.  No counterpart upstream: the reference has no
 * synthetic weights; this exists so that benchmark inputs are reproducible. */
TLC_API int32_t tlc_synth_blocks_host(int32_t type, uint64_t seed, uint64_t tensor_id,
                                      int64_t first_block, int64_t n_blocks, void *out_host);
TLC_API int32_t tlc_qtensor_destroy(tlc_qtensor *qt);
/* Local (per-rank) shape and storage.  row_pitch is the distance in bytes
 * between rows in HBM: the GGUF row size rounded up to 16 (equal to it, i.e.
 * a verbatim copy of the file's bytes, whenever n_cols is a multiple of 256). */
TLC_API int32_t tlc_qtensor_info(tlc_qtensor *qt, int32_t *type, int64_t *n_rows,
                                 int64_t *n_cols, size_t *row_pitch, const void **dev_ptr);
/* Device-side GGUFLoader::dequantize_q4_0 / _q8_0: writes the n_rows*n_cols
 * f16 values of the local shard; bit-exact with the reference. */
TLC_API int32_t tlc_dequant(tlc_ctx *ctx, tlc_qtensor *qt, void *out_f16_dev);

/* ---- ops ---------------------------------------------------------------- */

/* linear(x, W[, bias]) = Tensor::matmul_transposed_b (src/ops/matmul.rs:241-311,
 * builtin src/interpreter/builtin_math.rs:76-199): y[M,N] = x[M,K] . W[N,K]^T,
 * f16 in/out, f32 accumulation, one rounding; optional bias [N] added as a
 * separate f16 add like the builtin does (builtin_math.rs:109-117).
 * x_cols is the caller's K and must equal W's columns
 * (TLC_ERR_INVALID_OPERATION otherwise, matmul.rs:266-273). */
TLC_API int32_t tlc_linear(tlc_ctx *ctx, tlc_qtensor *w, const void *x_dev, int32_t m,
                           int64_t x_cols, void *y_dev, const void *bias_dev);
/* Host-buffer variant: uploads x, runs, downloads y, waits. */
TLC_API int32_t tlc_linear_host(tlc_ctx *ctx, tlc_qtensor *w, const void *x_host, int32_t m,
                                int64_t x_cols, void *y_host, const void *bias_host);

/* rms_norm(x, w[, eps]) = Tensor::rms_norm (src/ops/normalization.rs:42-248;
 * builtin default eps 1e-6, src/interpreter/builtin_nn.rs:83-92). */
TLC_API int32_t tlc_rms_norm(tlc_ctx *ctx, const void *x_dev, const void *w_dev, void *y_dev,
                             int32_t rows, int32_t d, float eps);
/* rope(x[, position_offset]) = Tensor::rope (src/ops/rope.rs:71-118, :215-312):
 * x [seq, heads, d], interleaved pairs, integer base (10000 upstream).
 * positions_dev (nullable, int32[seq]) overrides pos = s + pos_offset. */
TLC_API int32_t tlc_rope(tlc_ctx *ctx, const void *x_dev, void *y_dev, int32_t seq,
                         int32_t heads, int32_t d, int32_t pos_offset, uint32_t base,
                         const int32_t *positions_dev);
/* sigmoid / mul / add (src/ops/activations.rs:239-266, elementwise.rs:232-330,
 * :48-140). */
TLC_API int32_t tlc_sigmoid(tlc_ctx *ctx, const void *x_dev, void *y_dev, size_t n);
TLC_API int32_t tlc_mul(tlc_ctx *ctx, const void *a_dev, const void *b_dev, void *y_dev, size_t n);
TLC_API int32_t tlc_add(tlc_ctx *ctx, const void *a_dev, const void *b_dev, void *y_dev, size_t n);
/* silu(gate) * up as the scripts compose it from sigmoid and mul
 * (debug/chat_demo_with_kvcache.tl:26-41), one kernel. */
TLC_API int32_t tlc_swiglu(tlc_ctx *ctx, const void *gate_dev, const void *up_dev, void *y_dev,
                           size_t n);
/* softmax over the last dim = Tensor::softmax (src/ops/activations.rs:107-229). */
TLC_API int32_t tlc_softmax(tlc_ctx *ctx, const void *x_dev, void *y_dev, int32_t rows,
                            int32_t last_dim);
/* embedding(table, ids) (src/interpreter/builtin_nn.rs:627-909): row gather
 * from an f16 [vocab, d] table; ids are checked on the host first
 * (builtin_nn.rs:681-688) so they are passed as a HOST array. */
TLC_API int32_t tlc_embedding(tlc_ctx *ctx, const void *table_dev, int32_t vocab, int32_t d,
                              const int32_t *ids_host, int32_t m, void *y_dev);

/* ---- fused per-token ops around the linears ------------------------------ */

/* y = linear(rms_norm(x, norm_w, eps), W) for up to 3 weights sharing x (q/k/v
 * or gate/up), one launch.  norm_w_dev may be NULL (no norm).  rope_heads[i] > 0
 * applies rope to output i viewed as [m, rope_heads[i], N_i/rope_heads[i]] with
 * position pos_offset + row (or positions_dev[row]). */
TLC_API int32_t tlc_norm_linear_multi(tlc_ctx *ctx, int32_t n_weights, tlc_qtensor *const *w,
                                      void *const *y_dev, const int32_t *rope_heads,
                                      const void *x_dev, int32_t m, const void *norm_w_dev,
                                      float eps, int32_t pos_offset, uint32_t rope_base,
                                      const int32_t *positions_dev);
/* act = silu(linear(xn, W_gate)) * linear(xn, W_up), xn = rms_norm(x) when
 * norm_w_dev != NULL; one launch. */
TLC_API int32_t tlc_swiglu_gate_up(tlc_ctx *ctx, tlc_qtensor *w_gate, tlc_qtensor *w_up,
                                   const void *x_dev, int32_t m, const void *norm_w_dev,
                                   float eps, void *act_dev);
/* y = residual + linear(x, W) (f16 add after the f16 rounding of the linear). */
TLC_API int32_t tlc_linear_residual(tlc_ctx *ctx, tlc_qtensor *w, const void *x_dev, int32_t m,
                                    const void *residual_dev, void *y_dev);

#ifdef __cplusplus
}
#endif
#endif /* TLCUDA_H */
