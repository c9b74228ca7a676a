// Internal declarations shared by the translation units of libtlcuda.
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <map>
#include <string>
#include <vector>

#include "tlcuda.h"

// Device-side status word polled by tlc_synchronize: kernels with bounded
// waits store a non-zero code here instead of spinning forever.
struct tlc_dev_status {
    int code;   // 0 = fine
    int where;  // kernel-specific location id of the wait that gave up
};
// Status codes below TLC_DEV_INDEX mean a bounded wait that ran out (TLC_ERR_TIMEOUT);
// TLC_DEV_INDEX means a kernel met a sequence position outside its cache and skipped the
// access (TLC_ERR_INDEX).
#define TLC_DEV_INDEX 16

struct tlc_pool {
    // idle buffers by class size
    std::map<size_t, std::vector<void *>> idle;
    size_t max_per_class = 10;  // BufferPool::new, buffer_pool.rs:106
    tlc_pool_stats stats{};
};

struct tlc_ctx {
    int device = 0;
    cudaStream_t stream = nullptr;
    cudaDeviceProp prop{};
    int sm_count = 0;
    tlc_pool pool;
    uint64_t launches = 0;
    // Option "perf" / TLC_PERF=1 (or the reference's TL_PERF in the environment): every op entry
    // point times its launches with CUDA events, prints "[PERF] op: x.xxxms" to stderr as the
    // reference's builtins do (src/interpreter/builtin_math.rs:190-197) and adds to these totals
    // (tlc_perf_report).  Each timed op waits for its own launches: a measuring mode, not a fast one.
    bool perf = false;
    struct perf_total { uint64_t calls = 0; double ms = 0.0; };
    std::map<std::string, perf_total> perf_totals;
    tlc_dev_status *dev_status = nullptr;   // device memory
    tlc_dev_status *host_status = nullptr;  // pinned mirror
    // Reusable scratch for kernels that need global workspace (grows on demand).
    void *scratch = nullptr;
    size_t scratch_bytes = 0;
    // Zero-initialised ticket counters for kernels whose last CTA merges
    // partial results; every user leaves them at zero again.
    int *tickets = nullptr;
    size_t n_tickets = 0;
    // Launch kernels with programmatic stream serialization (the kernels call
    // griddepcontrol.wait before they touch a predecessor's output); the
    // environment variable TLC_NO_PDL=1 turns it off.
    bool use_pdl = true;
    int pdl_mode = 4;      // TLC_PDL_MODE: when the GEMV lets its successor be scheduled (1 at once, 2 after its last slab, 3 after its own dependency wait, 4 = 3 for long kernels and 2 for short ones; measured on TinyLlama decode: 2 is 9 % faster than no PDL, 1 is 10 % slower than 2)
    bool pdl_small = true; // TLC_PDL_SMALL=0: keep PDL off for the non-GEMV kernels
    // TLC_GEMM_MIN_M: activation rows from which quantized linears run as the
    // tensor-core GEMM (0: decide from the shape; a huge value keeps the GEMV).
    int gemm_min_m = 0;
    // Decode attention with few (sequence, KV head) tiles and a long context: clusters of sixteen
    // key splits (a non-portable cluster size) instead of eight.  Off: measured no faster (one
    // rank's share of the 70B-shape decode at TP8, 2048 keys: 3.79 ms per step against 3.73 ms).
    int attn_wide = 0;
    int l2_hint = 1;         // GEMV weight copies marked evict-first in the L2 (measured: +3 % on the decode step)
    bool host_graph = true;  // decode_host: ids up, the step, results down as ONE graph launch
    bool host_poll = true;   // ... and the host watches the pinned result words instead of a stream sync
    // How long a device-side wait (mbarrier, peer flag) may last before the kernel gives up,
    // sets the status word and drains; option "wait_limit_ms".
    uint64_t wait_ns = 2000000000ull;
    bool gemm_pair = false;  // GEMM tiles of 256 x 256 on CTA pairs (tcgen05 cta_group::2) from 129 rows on; measured slower
    bool comm_ll = true;  // peer-memory all-reduces of up to 256 Ki values use flagged words instead of fences + flags
    int gemm_splitk = 1;  // GEMMs of up to 128 rows and few weight tiles share K over several CTAs per tile: 0 off, 1 where a cost model says it pays, 2 wherever possible
    int gemm_pg = 0;  // producer groups of the GEMM: 0 = two where K is shared out over CTAs, else one; 1 / 2 = forced
    bool gemm_tma = true;  // activation tiles of the GEMM by TMA (false: cp.async loader warps)
    int gemm_tile = 0;  // 0: pick the GEMM tile from the shape; 11, 12, 22: force 128x128, 128x256, 256x256
    // Option "gemv_f8" / TLC_GEMV_F8=1: one activation row against a Q4_0 weight takes the FP8-limb
    // form of the fused GEMV (tlc_gemv_kernel.cuh).  Off by default: fewer instructions per block,
    // but measured slower on a B200 (35.3 vs 30.5 us on a 132 MB weight, 7.1 vs 5.5 us on 6.5 MB).
    bool gemv_f8 = false;
    // Option "gemv_splitk" / TLC_GEMV_SPLITK=0: 2..16 activation rows whose fragments crowd the
    // shared memory take further passes over the weights instead of one pass with K cut into windows.
    int gemv_splitk = 2;  // 0: off; 1: windows sized for two CTAs per SM first; 2: for one CTA per SM first (measured faster)
    // Option "q6k_resident" / TLC_Q6K_RESIDENT=0: Q6_K tensors are expanded to f16 at upload (what
    // the reference's loader keeps) instead of staying quantized in HBM.
    bool q6k_resident = true;
    // Option "step_kernel" / TLC_STEP_KERNEL=1: single-sequence greedy decode steps run as one
    // persistent kernel (tlc_step.cu) when the model allows it.  Off by default: on a B200 the
    // TinyLlama step takes 0.79 ms that way against 0.61 ms kernel by kernel (its hand-overs
    // between phases cost more than the launches they replace).
    bool step_kernel = false;
};

struct tlc_buf {
    tlc_ctx *ctx;
    void *ptr;
    size_t class_bytes;
    size_t requested;
};

struct tlc_qtensor {
    tlc_ctx *ctx;
    int32_t type;        // TLC_TYPE_*
    int64_t n_rows;      // local rows (N of this rank)
    int64_t n_cols;      // local cols (K of this rank)
    int64_t full_rows;   // unsharded shape
    int64_t full_cols;
    size_t row_bytes;    // bytes of one local row as GGUF stores it (no padding)
    size_t row_pitch;    // F16: distance between rows in HBM (row_bytes rounded up to 16); Q4_0 / Q8_0: 0
    int64_t k_tiles;     // Q4_0 / Q8_0: tiles along K (tlc_tile.cuh); F16: 0
    size_t slab_pitch;   // Q4_0 / Q8_0: bytes of one 16-row slab = k_tiles * tile bytes
    size_t bytes;        // allocation: n_rows * row_pitch, or slabs * slab_pitch
    void *data;          // device
    int32_t tp_rank, tp_size, split;
};

// ---- error plumbing -------------------------------------------------------
int32_t tlc_fail(int32_t code, const char *fmt, ...);
void tlc_clear_error();

#define TLC_CUDA(expr)                                                                     \
    do {                                                                                   \
        cudaError_t _e = (expr);                                                           \
        if (_e != cudaSuccess)                                                             \
            return tlc_fail(TLC_ERR_CUDA, "%s failed: %s (%s:%d)", #expr,                  \
                            cudaGetErrorString(_e), __FILE__, __LINE__);                   \
    } while (0)

#define TLC_CHECK_LAUNCH(ctx)                                                              \
    do {                                                                                   \
        (ctx)->launches++;                                                                 \
        cudaError_t _e = cudaGetLastError();                                               \
        if (_e != cudaSuccess)                                                             \
            return tlc_fail(TLC_ERR_CUDA, "kernel launch failed: %s (%s:%d)",              \
                            cudaGetErrorString(_e), __FILE__, __LINE__);                   \
    } while (0)

#define TLC_REQUIRE(cond, code, ...)                                                       \
    do {                                                                                   \
        if (!(cond)) return tlc_fail((code), __VA_ARGS__);                                 \
    } while (0)

static inline size_t tlc_block_bytes(int32_t type) {
    return type == TLC_TYPE_Q4_0 ? 18 : type == TLC_TYPE_Q8_0 ? 34 : 0;
}

// A dense F16 copy of a quantized tensor (device-side dequantization).
int32_t tlc_qtensor_to_f16(tlc_ctx *ctx, tlc_qtensor *qt, tlc_qtensor **out);
// Failure-detection self-tests: launch a kernel whose bounded wait must run out.
int32_t tlc_selftest_mbarrier_wait(tlc_ctx *ctx);
int32_t tlc_selftest_peer_wait(tlc_ctx *ctx, bool flagged_words);
// Makes the context's device current; every entry point calls it first.
int32_t tlc_enter(tlc_ctx *ctx);
// After a stream synchronize that followed a copy of the status word to host_status.
int32_t tlc_status_after_sync(tlc_ctx *ctx);
// Ensures ctx->scratch holds at least `bytes`.
int32_t tlc_scratch_reserve(tlc_ctx *ctx, size_t bytes);

// Launches `kernel` on the context's stream, with programmatic stream
// serialization when the context allows it: the kernel may then be scheduled
// before its predecessor has finished and must execute griddepcontrol.wait
// before it reads or overwrites anything the predecessor touches.
template <typename... KArgs, typename... Args>
inline cudaError_t tlc_launch_pdl(tlc_ctx *ctx, void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                  Args &&...args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = ctx->stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = ctx->use_pdl && ctx->pdl_small ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// Times the launches an op entry point makes between its construction and destruction when the
// context's "perf" option is on (never inside a stream capture).
struct tlc_perf_scope {
    tlc_ctx *ctx;
    char name[96];
    cudaEvent_t e0 = nullptr, e1 = nullptr;
    bool on = false;
    tlc_perf_scope(tlc_ctx *c, const char *fmt, ...);
    ~tlc_perf_scope();
    tlc_perf_scope(const tlc_perf_scope &) = delete;
    tlc_perf_scope &operator=(const tlc_perf_scope &) = delete;
};

#ifdef __CUDACC__
__device__ __forceinline__ uint64_t tlc_globaltimer_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
// Device side of the above: let the successor be scheduled, then wait for the
// predecessor's results.  Both are no-ops for a kernel launched the plain way.
__device__ __forceinline__ void tlc_pdl_prologue() {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
}
#endif

// ---- launchers implemented in the kernel translation units ----------------

// One weight of a fused multi-GEMV launch.
struct tlc_gemv_out {
    const tlc_qtensor *w;
    void *y;             // f16 [m, N]
    int32_t rope_heads;  // >0: apply rope over [m, heads, N/heads]
    // Output addressing: element (row r, output n) lands at
    //   y[r * row_stride + pos(r) * pos_stride + n],
    // pos(r) = positions[r] or pos_offset + r.  Defaults give dense [m, N].
    int64_t row_stride = -1;  // < 0: N
    int64_t pos_stride = 0;
};

enum tlc_gemv_epilogue {
    TLC_EPI_STORE = 0,     // y = f16(acc) [+ bias]
    TLC_EPI_RESIDUAL = 1,  // y = f16(acc) + residual
    TLC_EPI_SWIGLU = 2,    // outs[0]=gate, outs[1]=up -> act = silu(g)*u into outs[0].y
};

struct tlc_gemv_args {
    int32_t n_out = 0;
    tlc_gemv_out outs[3]{};
    const void *x = nullptr;  // f16 [m, K]
    int32_t m = 0;
    const void *norm_w = nullptr;  // f16 [K] or null
    float eps = 0.f;
    int32_t epilogue = TLC_EPI_STORE;
    const void *bias = nullptr;      // f16 [N] (STORE, single output)
    const void *residual = nullptr;  // f16 [m, N] (RESIDUAL)
    int32_t pos_offset = 0;
    uint32_t rope_base = 10000;
    const int32_t *positions = nullptr;  // device int32 [m] or null
    // Outputs addressed by position (pos_stride != 0, a KV cache): a position outside [0, max_pos)
    // never reaches memory outside the cache -- the one-pass GEMV stores at the last row instead (the
    // attention kernel that follows reports the position), the split-K finish and the GEMM drop the
    // row and raise TLC_DEV_INDEX themselves.  0: no limit.
    int32_t max_pos = 0;
};

int32_t tlc_launch_gemv(tlc_ctx *ctx, const tlc_gemv_args &a);

// Tensor-core (tcgen05) path of the same contract for many activation rows;
// tlc_launch_gemv forwards to it when tlc_gemm_eligible says so.
bool tlc_gemm_eligible(const tlc_ctx *ctx, const tlc_gemv_args &a);
int32_t tlc_launch_gemm(tlc_ctx *ctx, const tlc_gemv_args &a);
// Scratch the GEMM path needs for m rows of width k with a fused RMSNorm and a
// SiLU.mul pair of n_swiglu outputs (reserve it before capturing a graph).
size_t tlc_gemm_scratch_bytes(const tlc_ctx *ctx, int m, int64_t k, int64_t n_total);
// Adds the ksplit f32 shares in partial[ksplit][m][sum of N] and applies the epilogue of `a` (tlc_gemv.cu).
int32_t tlc_gemv_splitk_finish(tlc_ctx *ctx, const tlc_gemv_args &a, int ksplit, float *partial);
// Scratch the fused GEMV may need for m rows (split-K partial sums; 0 when it does not split).
size_t tlc_gemv_scratch_bytes(tlc_ctx *ctx, int type, int64_t k, int m, int64_t n_total);

struct tlc_kvcache;
int32_t tlc_launch_attention(tlc_ctx *ctx, tlc_kvcache *cache, int layer, const void *q_dev, void *out_dev,
                             int batch, int n_queries, int n_heads, int q_pos0, const int *positions_dev,
                             int max_keys, float scale, bool positions_settled);
