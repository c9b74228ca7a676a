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

/* GGUF tensor type ids (src/model/formats/mmap_gguf.rs:30-45).  Q4_0 and Q8_0
 * stay quantized in device memory; Q6_K (210-byte super-blocks of 256 values) and
 * F32 are accepted on upload and become F16 tensors, which is what the reference's
 * loader makes of every type (src/model/formats/gguf.rs:128-253, :413-440). */
enum { TLC_TYPE_F32 = 0, TLC_TYPE_F16 = 1, TLC_TYPE_Q4_0 = 2, TLC_TYPE_Q8_0 = 8, TLC_TYPE_Q6_K = 14 };

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
/* Runtime switches the reference reads from the environment (TL_PERF, TL_DEBUG,
 * src/device/kernel_executor.rs:33-41); here by name:
 *   "gemm_min_m"  activation rows from which quantized linears run as the
 *                 tcgen05 GEMM (0 = decide from the shape);
 *   "gemm_tile"   0 = pick the GEMM tile from the shape; 11, 12, 22 force
 *                 128x128, 128x256 or 256x256 (activation rows x weight rows);
 *   "wait_limit_ms" how long a device-side wait (mbarrier, peer flag) may last before the
 *                 kernel gives up and the next tlc_synchronize returns TLC_ERR_TIMEOUT;
 *   "pdl"         programmatic dependent launch on (1) / off (0);
 *   "pdl_mode"    when a GEMV lets the next kernel of the stream be scheduled: 1 = at once,
 *                 2 = after its last slab, 3 = after its own dependency wait, 4 (default) = 3 for
 *                 kernels that stream 40 MB of weights or more and 2 for shorter ones;
 *   "l2_hint"     the GEMV's weight copies carry the evict-first L2 hint (1, default) or none (0);
 *   "host_graph"  tlc_llama_decode_host runs as one graph launch with copy nodes (1, default)
 *                 or as copy + graph + copy (0);
 *   "host_poll"   with host_graph: the host watches the pinned result words (1, default)
 *                 instead of synchronizing the stream (0).
 *   "step_kernel" single-sequence greedy decode steps run as ONE persistent kernel (1)
 *                 or kernel by kernel, five launches per layer (0, default: faster on a B200).
 *   "gemm_tma"    the GEMM's activation tiles arrive by TMA (1, default) or through cp.async
 *                 loader warps (0);
 *   "gemm_pg"     weight-producer groups of the GEMM: 0 (default) = two groups taking alternate K
 *                 steps where the K steps of a tile are shared out ("gemm_splitk"), one group
 *                 otherwise; 1 = one group and no sharing; 2 = two groups wherever possible;
 *   "perf"        per-op timing on (1) / off (0, default): see tlc_perf_report;
 *   "comm_ll"     peer-memory all-reduces of up to 262144 values send data and flag in one word and
 *                 poll the data (1, default) or use stores + fences + flags (0);
 *   "gemm_splitk" GEMMs of up to 128 activation rows whose weight gives fewer tiles than SMs share
 *                 the K steps over several CTAs per tile where a cost model says it pays, one finishing
 *                 kernel adds (1, default); 2 = wherever possible; 0 = off;
 *   "gemm_pair"   from 129 activation rows on, the GEMM runs on CTA pairs (tcgen05 cta_group::2,
 *                 persistent, two accumulators in tensor memory) (1) or on single CTAs (0,
 *                 default: faster on a B200);
 *   "gemv_splitk" 2 to 16 activation rows whose fragments crowd the shared memory: K is cut into
 *                 windows, one pass over the weights (2, default: windows sized for one CTA per
 *                 SM; 1: for two CTAs per SM) or several passes (0);
 *   "gemv_f8"     one activation row of a Q4_0 weight on the FP8 tensor-core form (1) or the
 *                 f16 form (0, default: faster);
 *   "q6k_resident" Q6_K tensors stay quantized in HBM (1, default) or become f16 at upload (0);
 *   "attn_wide"   decode attention of one sequence with at most four KV heads over a long
 *                 context runs on clusters of sixteen key splits (1) or eight (0, default: no slower).
 * Unknown names fail with TLC_ERR_INVALID_OPERATION. */
TLC_API int32_t tlc_set_option(tlc_ctx *ctx, const char *name, int64_t value);
/* Failure-detection self-test.  Enqueues a kernel whose device-side wait can never be
 * satisfied -- kind 0: an mbarrier nothing arrives on (the wait of the GEMV / GEMM
 * pipelines); kind 1: the peer flags of the all-reduce with no peer present; kind 2: the
 * flagged words of its short-vector form.  The wait
 * gives up after the "wait_limit_ms" option (default 2000), the kernel returns, and the
 * next tlc_synchronize reports TLC_ERR_TIMEOUT once; the context stays usable. */
TLC_API int32_t tlc_selftest_wait_timeout(tlc_ctx *ctx, int32_t kind);
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
/* Per-op timing, the counterpart of the reference's TL_PERF environment switch
 * (src/interpreter/builtin_math.rs:190-197, builtin_nn.rs:119, ops/elementwise.rs:274-299): with
 * the option "perf" set (tlc_set_option, TLC_PERF=1, or TL_PERF in the environment) every op entry
 * point times its launches with CUDA events, waits for them, prints "[PERF] op(shape): x.xxxms" to
 * stderr and adds to per-op totals.  tlc_perf_report writes those totals as text, one line per op:
 * "name calls total_ms"; needed_out (optional) receives the report's length; reset != 0 clears
 * the totals.  A measuring mode: every timed op synchronizes; nothing is timed inside a stream
 * capture. */
TLC_API int32_t tlc_perf_report(tlc_ctx *ctx, char *buf, size_t buflen, int32_t reset, size_t *needed_out);

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
 * fastest; 18-byte Q4_0 / 34-byte Q8_0 blocks of 32 along a row) are kept in
 * HBM bit for bit, regrouped on the device into tiles of 16 rows (the order the
 * matrix kernels fetch them in; tlc_qtensor_blocks gives the file's order
 * back).  `blocks` is a HOST pointer to the FULL tensor; with
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
 * the host).  Only Q4_0 / Q8_0.  Block scales are U[0.002, 0.02] * 2^scale_log2. */
TLC_API int32_t tlc_qtensor_create_synthetic(tlc_ctx *ctx, int32_t type, int64_t n_rows,
                                             int64_t n_cols, uint64_t seed, uint64_t tensor_id,
                                             int32_t scale_log2, int32_t tp_rank, int32_t tp_size,
                                             int32_t split, tlc_qtensor **out);
/* The same generator on the host (no GPU needed): writes n_blocks consecutive
 * blocks of the full tensor, starting at block index first_block (row-major
 * block order), into out_host.  No counterpart upstream: the reference has no
 * synthetic weights; this exists so that benchmark inputs are reproducible. */
TLC_API int32_t tlc_synth_blocks_host(int32_t type, uint64_t seed, uint64_t tensor_id,
                                      int32_t scale_log2, int64_t first_block, int64_t n_blocks,
                                      void *out_host);
/* Device-side f16 N(mean, std) fill from the same generator (embedding tables
 * and pre-filled KV caches of the large benchmark shapes).  No counterpart in
 * the reference. */
TLC_API int32_t tlc_fill_normal_f16(tlc_ctx *ctx, void *dst_dev, size_t n, uint64_t seed,
                                    uint64_t tensor_id, float mean, float std);
TLC_API int32_t tlc_qtensor_create_normal_f16(tlc_ctx *ctx, int64_t n_rows, int64_t n_cols,
                                              uint64_t seed, uint64_t tensor_id, float mean,
                                              float std, tlc_qtensor **out);
TLC_API int32_t tlc_qtensor_destroy(tlc_qtensor *qt);
/* Local (per-rank) shape and storage.  For F16 tensors row_pitch is the
 * distance in bytes between rows in HBM (the row size rounded up to 16); for
 * Q4_0 / Q8_0 tensors, whose storage is tiled, it is the GGUF size of one row. */
TLC_API int32_t tlc_qtensor_info(tlc_qtensor *qt, int32_t *type, int64_t *n_rows,
                                 int64_t *n_cols, size_t *row_pitch, const void **dev_ptr);
/* Writes the local shard's GGUF blocks in the file's order (row-major,
 * n_rows * n_cols/32 blocks, no padding) to device memory: the inverse of the
 * regrouping done at upload, bit for bit.  F16 tensors are copied row by row. */
TLC_API int32_t tlc_qtensor_blocks(tlc_ctx *ctx, tlc_qtensor *qt, void *out_dev);
/* The regrouping on the host (no GPU needed): bytes a Q4_0 / Q8_0 tensor of this shape
 * occupies in HBM, and the tiled image of row-major GGUF blocks (what tlc_qtensor_create
 * stores: dev_ptr of tlc_qtensor_info points at exactly these bytes).  Tiles of 16 rows,
 * [slab = row / 16][k-tile]; a Q4_0 tile is 16 rows x 4 blocks = 1152 bytes: 16-byte groups
 * [row / 8 % 2][row % 8][t] holding quant word t (bytes 4t..4t+3 of qs) of the row's four
 * blocks, then [row][block] f16 scales at byte 1024; a Q8_0 tile is 16 rows x 2 blocks =
 * 1088 bytes: group [..][..][t] holds words 2t, 2t+1 of block 0, then of block 1; scales at
 * byte 1024.  Rows past n_rows and blocks past n_cols / 32 are zero.  No counterpart
 * upstream (the reference keeps dequantized f16 rows). */
TLC_API size_t tlc_tiled_bytes(int32_t type, int64_t n_rows, int64_t n_cols);
TLC_API int32_t tlc_tile_blocks_host(int32_t type, int64_t n_rows, int64_t n_cols,
                                     const void *blocks, void *tiles_out);
/* Device-side GGUFLoader::dequantize_q4_0 / _q8_0: writes the n_rows*n_cols
 * f16 values of the local shard; bit-exact with the reference. */
TLC_API int32_t tlc_dequant(tlc_ctx *ctx, tlc_qtensor *qt, void *out_f16_dev);

/* ---- ops ---------------------------------------------------------------- */

/* matmul(a, b) builtin (src/interpreter/builtin_math.rs:39-66, Tensor::matmul
 * src/ops/matmul.rs:13-75; kernels shaders/unified.metal:33-478): dense
 * y[m, n] = a[m, k] . b[k2, n], f16 in, f32 accumulate, one rounding to f16.
 * k != k2 fails with TLC_ERR_INVALID_OPERATION "matmul shape mismatch: [m, k] @ [k2, n]"
 * (matmul.rs:41-46).  A general-purpose builtin; quantized weights go through tlc_linear. */
TLC_API int32_t tlc_matmul(tlc_ctx *ctx, const void *a_dev, const void *b_dev, void *y_dev, int32_t m,
                           int32_t k, int32_t k2, int32_t n);

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

/* rope(x, cos, sin): the arm of the rope builtin with precomputed f16 tables
 * (src/interpreter/builtin_tensor.rs:634-722, Tensor::rope_candle src/ops/rope.rs:18-65,
 * kernel rope_candle_f16 shaders/unified.metal:5122-5184).  x, y [seq, heads, head_dim];
 * cos/sin tables of table_rows (>= seq) rows whose rows lie `pitch` elements apart; the
 * rotary pair p of position s uses cos[s * pitch + p], sin[s * pitch + p].  A table with one
 * column per pair ([max_seq, head_dim / 2], pitch = head_dim / 2) rotates like tlc_rope.  The
 * reference's builtin stores each frequency twice in rows of head_dim values while its kernel
 * indexes by pair: passing such a table with pitch = head_dim reproduces what the reference
 * computes (pair p gets frequency p / 2). */
TLC_API int32_t tlc_rope_table(tlc_ctx *ctx, const void *x_dev, const void *cos_dev, const void *sin_dev,
                               void *y_dev, int32_t seq, int32_t heads, int32_t head_dim,
                               int32_t table_rows, int32_t pitch);
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

/* ---- KV cache and attention ----------------------------------------------- */

typedef struct tlc_kvcache tlc_kvcache;

/* KVCache::new_f16(n_layers) (src/model/llama.rs:51-76) with the storage
 * pre-allocated the way src/ops/cache_ops.rs:28-60 does it: per layer
 * K and V [max_batch, max_seq, n_kv_heads, head_dim] f16, zero-filled. */
TLC_API int32_t tlc_kvcache_create(tlc_ctx *ctx, int32_t n_layers, int32_t max_batch,
                                   int32_t max_seq, int32_t n_kv_heads, int32_t head_dim,
                                   tlc_kvcache **out);
TLC_API int32_t tlc_kvcache_destroy(tlc_kvcache *cache);
TLC_API int32_t tlc_kvcache_layer_ptrs(tlc_kvcache *cache, int32_t layer, void **k_dev,
                                       void **v_dev);
/* cache.append(layer, K, V) (src/model/llama.rs:78-99; kernel cache_append_f16,
 * shaders/unified.metal:4189-4197) without the O(T) concat: rows of k/v
 * [m, n_kv_heads*head_dim] are written in place.  positions_dev == NULL: the m
 * rows are consecutive tokens of sequence 0 starting at pos_offset (prefill);
 * otherwise row r is the new token of sequence r at positions_dev[r] (decode). */
TLC_API int32_t tlc_kvcache_append(tlc_ctx *ctx, tlc_kvcache *cache, int32_t layer,
                                   const void *k_dev, const void *v_dev, int32_t m,
                                   int32_t pos_offset, const int32_t *positions_dev);
/* Grouped-query causal attention over the cache; replaces the script-level
 * chain reshape/broadcast_to/einsum/scale/causal_mask/apply_attention_mask/
 * softmax/einsum (debug/chat_demo_with_kvcache.tl:44-88, :247-282; kernels at
 * shaders/unified.metal:2524-2683, :4474-4488, :2057-2200).
 * q, out: [batch * n_queries, n_heads, head_dim] f16.  Query i of a sequence
 * sits at position q_pos0 + i and sees keys 0 .. q_pos0 + i; the cache must
 * already hold the keys of these positions.  With positions_dev (int32[batch],
 * n_queries must be 1) each sequence's query sits at positions_dev[b] and
 * max_keys bounds positions_dev[b] + 1.  KV head of query head h is
 * h / (n_heads / n_kv_heads). */
TLC_API int32_t tlc_attention(tlc_ctx *ctx, tlc_kvcache *cache, int32_t layer, const void *q_dev,
                              void *out_dev, int32_t batch, int32_t n_queries, int32_t n_heads,
                              int32_t q_pos0, const int32_t *positions_dev, int32_t max_keys,
                              float scale);

/* Decode attention that allocates nothing (no counterpart in the reference: it
 * exists for hosts of this library that cannot request device memory while
 * they decode -- a CUDA-graph capture in progress, a serving loop that must
 * not hit the device-wide synchronisation of cudaMalloc, or a process whose
 * memory manager owns all of HBM).  Same computation as tlc_attention with
 * positions_dev (one query per sequence), on caller-owned buffers:
 *   q, out        [batch, n_heads, head_dim] f16
 *   k/v_cache_dev [batch, max_seq, n_kv_heads, head_dim] f16 (one layer)
 * launched on `stream` (a cudaStream_t) of the CURRENT device (a stream of
 * another device is refused with TLC_ERR_DEVICE).  The split-key partial
 * results, ticket counters and one status word live in a 2 MiB + 4.25 KiB array
 * inside the library image, per GPU, for the life of the process; a call is rejected
 * (TLC_ERR_BUFFER_EXHAUSTED) when batch * n_heads * splits * (head_dim + 2) * 4
 * bytes exceed 2 MiB (splits = key splits the launch uses, about 2 * SMs /
 * (batch * n_kv_heads), at most max_keys / 64) or batch * n_kv_heads exceeds 1024.  The first call on a
 * device looks the array's address up (cudaGetSymbolAddress) and sets kernel
 * attributes; make that first call before any stream capture.  All calls on a
 * device share the array: two calls that overlap on the GPU (different
 * streams) race; calls on one stream are safe.  The first-call set-up is
 * guarded by a mutex, so host threads may race to make it.  positions_dev[b] + 1
 * keys are read per sequence, never more than max_keys: a larger position is cut
 * there and tlc_attention_decode_static_status reports it.  Never calls
 * cudaMalloc / cudaFree or any allocating routine. */
TLC_API int32_t tlc_attention_decode_static(void *stream, const void *q_dev, const void *k_cache_dev,
                                            const void *v_cache_dev, void *out_dev, int32_t batch,
                                            int32_t n_heads, int32_t n_kv_heads, int32_t head_dim,
                                            int32_t max_seq, const int32_t *positions_dev,
                                            int32_t max_keys, float scale);

/* Companion of tlc_attention_decode_static (no counterpart in the reference):
 * waits for `stream`, then sets *clamped_out to 1 if, since the last query on the
 * current device, a call met a position at or beyond its max_keys and cut the
 * keys there, else 0; the note is cleared.  Allocates nothing. */
TLC_API int32_t tlc_attention_decode_static_status(void *stream, int32_t *clamped_out);

/* ---- GGUF models ----------------------------------------------------------- */

/* load_model(path) (src/interpreter/builtin_model.rs:106-131 -> Model::load,
 * src/model/mod.rs:165-184 -> GGUFLoader::load, src/model/formats/gguf.rs:256;
 * header walk of src/model/formats/mmap_gguf.rs:187-275): reads a GGUF v2/v3
 * file and uploads every tensor; Q4_0/Q8_0 tensors keep their blocks, F32 is
 * rounded to f16.  Rank >= 2 dims are reversed to [out, in] (gguf.rs:288-291).
 * With tp_size > 1 the LLaMA projections are sharded by name (q/k/v/gate/up/
 * output: rows; attn_output/ffn_down: columns). */
TLC_API int32_t tlc_model_load_gguf(tlc_ctx *ctx, const char *path, int32_t tp_rank,
                                    int32_t tp_size, tlc_model **out);
/* Lazy weight cache: GGUFWeightCache (src/model/gguf_weight_cache.rs:45-262, :418-441;
 * builtins load_weight_cache_gguf_f16 / _f32 and get_weight, builtin_model.rs:330-414).
 * Opens the file and reads its tensor table; tlc_weight_cache_get uploads a tensor on
 * first use and keeps at most `capacity` tensors, least recently used evicted first.
 * Cached tensors keep their GGUF quantization; a tensor returned by _get belongs to
 * the cache and stays valid until it is evicted, or the cache is cleared or closed.
 * Unknown names fail with TLC_ERR_LOAD "Weight not found: <name>". */
typedef struct tlc_weight_cache tlc_weight_cache;
TLC_API int32_t tlc_weight_cache_open(tlc_ctx *ctx, const char *path, int64_t capacity, tlc_weight_cache **out);
TLC_API int32_t tlc_weight_cache_close(tlc_weight_cache *cache);
TLC_API int32_t tlc_weight_cache_get(tlc_weight_cache *cache, const char *name, tlc_qtensor **out);
TLC_API int32_t tlc_weight_cache_contains(tlc_weight_cache *cache, const char *name);
TLC_API int32_t tlc_weight_cache_clear(tlc_weight_cache *cache);
TLC_API int32_t tlc_weight_cache_stats(tlc_weight_cache *cache, int64_t *len, int64_t *capacity, uint64_t *hits,
                                       uint64_t *misses, uint64_t *evictions);
/* MmapGGUFLoader::new (src/model/formats/mmap_gguf.rs:120, header walk
 * :187-275): parses header, metadata and tensor table only -- no device needed.
 * Per tensor: reversed [rows, cols], GGUF type id, absolute file offset and
 * byte size (n/32*18 for Q4_0, n/32*34 for Q8_0, mmap_gguf.rs:361-379). */
typedef struct tlc_gguf tlc_gguf;
TLC_API int32_t tlc_gguf_open(const char *path, tlc_gguf **out);
TLC_API int32_t tlc_gguf_close(tlc_gguf *g);
TLC_API int32_t tlc_gguf_tensor_count(tlc_gguf *g);
TLC_API int32_t tlc_gguf_tensor_info(tlc_gguf *g, int32_t index, const char **name, int32_t *type,
                                     int64_t *rows, int64_t *cols, uint64_t *file_offset,
                                     uint64_t *nbytes);
TLC_API int32_t tlc_gguf_meta_num(tlc_gguf *g, const char *key, double *out);
TLC_API const char *tlc_gguf_meta_str(tlc_gguf *g, const char *key);
TLC_API uint64_t tlc_gguf_data_start(tlc_gguf *g);
/* Model::new / insert for weights that do not come from a file (synthetic). */
TLC_API int32_t tlc_model_create(tlc_ctx *ctx, tlc_model **out);
TLC_API int32_t tlc_model_add(tlc_model *m, const char *name, tlc_qtensor *qt); /* takes ownership */
TLC_API int32_t tlc_model_destroy(tlc_model *m);
/* get_tensor(model, name) (src/interpreter/builtin_model.rs:203-246); the
 * handle stays owned by the model.  TLC_ERR_LOAD when the name is unknown. */
TLC_API int32_t tlc_model_get(tlc_model *m, const char *name, tlc_qtensor **out);
TLC_API int32_t tlc_model_tensor_count(tlc_model *m);
TLC_API const char *tlc_model_tensor_name(tlc_model *m, int32_t index);
/* GGUF metadata (numeric and bool keys as double; "<key>.length" for arrays). */
TLC_API int32_t tlc_model_meta_num(tlc_model *m, const char *key, double *out);
TLC_API const char *tlc_model_meta_str(tlc_model *m, const char *key);

/* ---- LLaMA forward pass ----------------------------------------------------- */

/* LlamaConfig (src/model/llama.rs:14-42; defaults there are TinyLlama's). */
typedef struct tlc_llama_config {
    int32_t n_layers, d_model, n_heads, n_kv_heads, head_dim, ffn_dim, vocab;
    float rms_eps;
    uint32_t rope_base;
    int32_t max_seq;         /* KV cache positions per sequence                */
    int32_t max_batch;       /* sequences decoded together (<= 64)              */
    int32_t max_prefill;     /* longest prompt chunk one prefill call may take  */
    int32_t tp_rank, tp_size;
    int32_t logits_all_rows; /* keep logits of every prompt row (parity checks) */
    int32_t no_graph;        /* launch kernels one by one, no CUDA graph replay */
} tlc_llama_config;

/* The forward pass the TL scripts spell out builtin by builtin
 * (debug/chat_demo_with_kvcache.tl:136-181 prefill, :213-296 decode;
 * LlamaModel::forward itself is a stub, src/model/llama.rs:257-266), bound to
 * the GGUF tensor names token_embd / blk.N.* / output_norm / output. */
TLC_API int32_t tlc_llama_create(tlc_ctx *ctx, tlc_model *model, const tlc_llama_config *cfg,
                                 tlc_llama **out);
TLC_API int32_t tlc_llama_destroy(tlc_llama *l);
/* Prompt tokens ids_host[0..n) of sequence 0 at positions pos0.. : fills the
 * cache, returns the greedy next token (last-index-wins ties,
 * src/interpreter/builtin_sampling.rs:176-181) and optionally the f16 logits
 * of the last row (or of all n rows when all_rows != 0). */
TLC_API int32_t tlc_llama_prefill(tlc_llama *l, const int32_t *ids_host, int32_t n, int32_t pos0,
                                  void *logits_host, int32_t all_rows, int32_t *next_id_host);
/* Sets the pending token and position of `batch` sequences (batched decode). */
TLC_API int32_t tlc_llama_set_state(tlc_llama *l, int32_t batch, const int32_t *ids_host,
                                    const int32_t *positions_host);
/* One greedy decode step through host buffers: ids_host (NULL = continue with
 * the tokens sampled by the previous step) is uploaded, the step runs, the
 * sampled tokens (and the f16 logits [batch, vocab] if logits_host != NULL)
 * are downloaded. */
TLC_API int32_t tlc_llama_decode_host(tlc_llama *l, int32_t batch, const int32_t *ids_host,
                                      int32_t *next_ids_host, void *logits_host);
/* Enqueues `steps` greedy decode steps back to back on the device; nothing is
 * read back (use tlc_llama_read_state). */
TLC_API int32_t tlc_llama_decode_enqueue(tlc_llama *l, int32_t batch, int32_t steps);
TLC_API int32_t tlc_llama_read_state(tlc_llama *l, int32_t batch, int32_t *next_ids_host,
                                     int32_t *positions_host);
/* Per-phase device timing of `steps` decode steps of sequence 0 (the counterpart of the
 * per-op times the reference prints under TL_PERF, src/interpreter/builtin_math.rs:190-197,
 * src/device/kernel_executor.rs:33-41).  With option "step_kernel" = 1 single-sequence greedy
 * decode runs as one persistent kernel; with this call its first CTA records the device clock (ns) at the
 * end of each phase: per layer A norm + q/k/v + rope, B attention, C o + residual,
 * D norm + gate/up + SiLU.mul, E down + residual, then F norm + lm_head, G sample.
 * out_ns receives [steps][n_layers * 5 + 2][3] values (capacity in elements): per phase the
 * time its input was complete, its dot products were done and its outputs were stored
 * (0 where a phase has no such point).  The steps
 * advance the sequence like tlc_llama_decode_enqueue.  TLC_ERR_INVALID_OPERATION when the
 * model does not run on that kernel (tensor parallel, temperature sampling, mixed or dense
 * weight types, option "step_kernel" = 0). */
TLC_API int32_t tlc_llama_step_trace(tlc_llama *l, int32_t steps, uint64_t *out_ns, size_t capacity);
/* Sampling of the runner (src/interpreter/builtin_sampling.rs:66-250).  temperature
 * <= 1e-4 is greedy, the default.  Otherwise every step draws the next token as
 * temperature_sample does -- f32 logits / temperature, softmax, first index whose
 * running probability sum exceeds a uniform draw -- on the device; the draw is a
 * pure function of (seed, position of the token fed to the step, sequence index),
 * tlc_sample_uniform_host gives the same number on the host. */
TLC_API int32_t tlc_llama_set_sampling(tlc_llama *l, float temperature, uint64_t seed);
TLC_API float tlc_sample_uniform_host(uint64_t seed, uint32_t position, uint32_t sequence);
/* The temperature_sample builtin on its own: logits_dev [rows, vocab] f16, one
 * uniform draw in [0, 1) per row from the caller (upstream: rand::thread_rng()),
 * sampled ids to the host.  uniforms_host may be NULL when temperature <= 1e-4. */
TLC_API int32_t tlc_temperature_sample(tlc_ctx *ctx, const void *logits_dev, int32_t rows, int32_t vocab,
                                       float temperature, const float *uniforms_host, int32_t *ids_host);
/* The same, replaying only some of the step's launches, for per-kernel timing:
 * parts is a mask of 1 (the quantized linears), 2 (attention), 4 (embedding
 * gather + sampling); tokens and positions are left untouched unless parts == 7. */
TLC_API int32_t tlc_llama_decode_enqueue_parts(tlc_llama *l, int32_t batch, int32_t steps,
                                               int32_t parts);
/* ---- tensor parallelism ----------------------------------------------------- */

/* No counterpart in the reference (it has no multi-GPU code).  One process per
 * GPU; the 128-byte id made by rank 0 (tlc_comm_unique_id) is handed to the
 * other ranks by the caller (a file, MPI, torch.distributed ...).  NCCL is
 * loaded at run time; TLC_ERR_COMM if it is missing or a call fails. */
typedef struct tlc_comm tlc_comm;
TLC_API int32_t tlc_comm_unique_id(void *out128);
TLC_API int32_t tlc_comm_init(tlc_ctx *ctx, const void *id128, int32_t rank, int32_t world,
                              tlc_comm **out);
TLC_API int32_t tlc_comm_destroy(tlc_comm *comm);
TLC_API int32_t tlc_comm_rank(tlc_comm *comm);
TLC_API int32_t tlc_comm_size(tlc_comm *comm);
/* In-place sum of `count` f16 values over the ranks (after the row-parallel
 * attn_output / ffn_down projections), enqueued on the context's stream. */
TLC_API int32_t tlc_allreduce_f16(tlc_ctx *ctx, tlc_comm *comm, void *buf_dev, size_t count);
/* recv[rank * count ...] = every rank's `count` f16 values (logit shards). */
TLC_API int32_t tlc_allgather_f16(tlc_ctx *ctx, tlc_comm *comm, const void *send_dev,
                                  void *recv_dev, size_t count);
/* Joins a runner created with tp_size > 1 to its communicator; required before
 * the first prefill / decode of a sharded model.  Logits handed back to the
 * host are full [rows, vocab] rows on every rank. */
/* Peer-memory exchange for small all-reduces (one process per GPU on one host,
 * GPUs connected by NVLink): every rank exports an exchange block
 * (tlc_comm_p2p_export -> a CUDA IPC handle of TLC_IPC_HANDLE_BYTES bytes), the
 * host gathers the handles of all ranks in rank order and gives them to
 * tlc_comm_p2p_import.  From then on tlc_allreduce_residual_f16 runs as ONE
 * kernel that pushes the partial sums to the peers over NVLink, waits (bounded:
 * a wait that runs out reports TLC_ERR_TIMEOUT at the next tlc_synchronize) and
 * sums in rank order, for vectors of up to max_elems values; larger ones, and
 * communicators without the exchange, use NCCL all-reduce + an add kernel. */
#define TLC_IPC_HANDLE_BYTES 64
TLC_API int32_t tlc_comm_p2p_export(tlc_comm *comm, size_t max_elems, void *handle_out);
TLC_API int32_t tlc_comm_p2p_import(tlc_comm *comm, const void *handles);
TLC_API int32_t tlc_comm_p2p_ready(tlc_comm *comm);
/* out = residual + sum over ranks of partial; residual may be null (out = the sum);
 * partial_dev may be overwritten.  count f16 values on every rank. */
TLC_API int32_t tlc_allreduce_residual_f16(tlc_ctx *ctx, tlc_comm *comm, void *partial_dev,
                                           const void *residual_dev, void *out_dev, size_t count);
TLC_API int32_t tlc_llama_set_comm(tlc_llama *l, tlc_comm *comm);

/* Kernels one decode step launches for a parts mask (7 = whole step), known
 * once such a step has been enqueued. */
TLC_API int32_t tlc_llama_launches_per_step(tlc_llama *l, int32_t parts);
TLC_API tlc_kvcache *tlc_llama_cache(tlc_llama *l);

#ifdef __cplusplus
}
#endif
#endif /* TLCUDA_H */
