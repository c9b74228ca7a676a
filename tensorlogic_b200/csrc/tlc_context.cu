// Device context, size-class buffer pool and host<->device transfers.
//
// Takes the place of MetalDevice (src/device/metal_device.rs), BufferPool
// (src/device/buffer_pool.rs) and MetalBuffer's copies
// (src/device/metal_buffer.rs) of the TensorLogic project.
#include <cstdlib>
#include <cstring>

#include "tlc_internal.h"

static thread_local std::string g_last_error;

int32_t tlc_fail(int32_t code, const char *fmt, ...) {
    char buf[1024];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof(buf), fmt, ap);
    va_end(ap);
    g_last_error = buf;
    return code;
}
void tlc_clear_error() { g_last_error.clear(); }

extern "C" const char *tlc_last_error(void) { return g_last_error.c_str(); }
extern "C" const char *tlc_version(void) { return "tlcuda 0.1 (sm_100a)"; }

int32_t tlc_enter(tlc_ctx *ctx) {
    TLC_REQUIRE(ctx != nullptr, TLC_ERR_INVALID_OPERATION, "null context");
    TLC_CUDA(cudaSetDevice(ctx->device));
    return TLC_OK;
}

extern "C" int32_t tlc_init(int32_t ordinal, tlc_ctx **out) {
    TLC_REQUIRE(out != nullptr, TLC_ERR_INVALID_OPERATION, "tlc_init: null out pointer");
    *out = nullptr;
    int count = 0;
    cudaError_t e = cudaGetDeviceCount(&count);
    if (e != cudaSuccess || count == 0) {
        cudaGetLastError();
        return tlc_fail(TLC_ERR_DEVICE, "no CUDA device available (%s); this library has no CPU path",
                        e == cudaSuccess ? "device count is 0" : cudaGetErrorString(e));
    }
    TLC_REQUIRE(ordinal >= 0 && ordinal < count, TLC_ERR_DEVICE,
                "device ordinal %d out of range (have %d)", ordinal, count);
    TLC_CUDA(cudaSetDevice(ordinal));
    tlc_ctx *ctx = new tlc_ctx();
    ctx->device = ordinal;
    cudaError_t pe = cudaGetDeviceProperties(&ctx->prop, ordinal);
    if (pe != cudaSuccess) {
        delete ctx;
        return tlc_fail(TLC_ERR_CUDA, "cudaGetDeviceProperties: %s", cudaGetErrorString(pe));
    }
    if (ctx->prop.major < 10) {
        int major = ctx->prop.major, minor = ctx->prop.minor;
        delete ctx;
        return tlc_fail(TLC_ERR_DEVICE, "device %d is sm_%d%d; this library is built for sm_100a only",
                        ordinal, major, minor);
    }
    ctx->sm_count = ctx->prop.multiProcessorCount;
    if (cudaStreamCreateWithFlags(&ctx->stream, cudaStreamNonBlocking) != cudaSuccess ||
        cudaMalloc(&ctx->dev_status, sizeof(tlc_dev_status)) != cudaSuccess ||
        cudaMemset(ctx->dev_status, 0, sizeof(tlc_dev_status)) != cudaSuccess ||
        cudaMalloc(&ctx->tickets, 16384 * sizeof(int)) != cudaSuccess ||
        cudaMemset(ctx->tickets, 0, 16384 * sizeof(int)) != cudaSuccess ||
        cudaMallocHost(&ctx->host_status, sizeof(tlc_dev_status)) != cudaSuccess) {
        const char *msg = cudaGetErrorString(cudaGetLastError());
        if (ctx->stream) cudaStreamDestroy(ctx->stream);
        if (ctx->dev_status) cudaFree(ctx->dev_status);
        if (ctx->tickets) cudaFree(ctx->tickets);
        delete ctx;
        return tlc_fail(TLC_ERR_CUDA, "context set-up failed: %s", msg);
    }
    memset(ctx->host_status, 0, sizeof(tlc_dev_status));
    ctx->n_tickets = 16384;
    const char *no_pdl = getenv("TLC_NO_PDL");
    ctx->use_pdl = !(no_pdl && no_pdl[0] == '1');
    if (const char *e = getenv("TLC_PDL_MODE")) ctx->pdl_mode = atoi(e);
    if (const char *e = getenv("TLC_PDL_SMALL")) ctx->pdl_small = atoi(e) != 0;
    if (const char *e = getenv("TLC_GEMM_MIN_M")) ctx->gemm_min_m = atoi(e);
    if (const char *e = getenv("TLC_GEMM_PAIR")) ctx->gemm_pair = atoi(e) != 0;
    if (const char *e = getenv("TLC_PERF")) ctx->perf = atoi(e) != 0;
    else if (getenv("TL_PERF")) ctx->perf = true;  // the reference's own switch
    if (const char *e = getenv("TLC_COMM_LL")) ctx->comm_ll = atoi(e) != 0;
    if (const char *e = getenv("TLC_GEMM_SPLITK")) ctx->gemm_splitk = atoi(e);
    if (const char *e = getenv("TLC_GEMM_PG")) ctx->gemm_pg = atoi(e);
    if (const char *e = getenv("TLC_GEMM_TMA")) ctx->gemm_tma = atoi(e) != 0;
    if (const char *e = getenv("TLC_ATTN_WIDE")) ctx->attn_wide = atoi(e);
    if (const char *e = getenv("TLC_L2_HINT")) ctx->l2_hint = atoi(e);
    if (const char *e = getenv("TLC_HOST_GRAPH")) ctx->host_graph = atoi(e) != 0;
    if (const char *e = getenv("TLC_HOST_POLL")) ctx->host_poll = atoi(e) != 0;
    if (const char *e = getenv("TLC_STEP_KERNEL")) ctx->step_kernel = atoi(e) != 0;
    if (const char *e = getenv("TLC_GEMV_F8")) ctx->gemv_f8 = atoi(e) != 0;
    if (const char *e = getenv("TLC_GEMV_SPLITK")) ctx->gemv_splitk = atoi(e);
    if (const char *e = getenv("TLC_Q6K_RESIDENT")) ctx->q6k_resident = atoi(e) != 0;
    *out = ctx;
    return TLC_OK;
}

extern "C" int32_t tlc_set_option(tlc_ctx *ctx, const char *name, int64_t value) {
    TLC_REQUIRE(ctx && name, TLC_ERR_INVALID_OPERATION, "set_option: null pointer");
    const std::string n(name);
    if (n == "gemm_min_m")
        ctx->gemm_min_m = (int)value;
    else if (n == "wait_limit_ms") {
        TLC_REQUIRE(value >= 1 && value <= 60000, TLC_ERR_INVALID_OPERATION, "set_option: wait_limit_ms must be 1..60000");
        ctx->wait_ns = (uint64_t)value * 1000000ull;
    } else if (n == "gemm_tile") {
        TLC_REQUIRE(value == 0 || value == 11 || value == 12 || value == 22, TLC_ERR_INVALID_OPERATION,
                    "set_option: gemm_tile must be 0, 11, 12 or 22");
        ctx->gemm_tile = (int)value;
    } else if (n == "gemm_pair")
        ctx->gemm_pair = value != 0;
    else if (n == "perf")
        ctx->perf = value != 0;
    else if (n == "comm_ll")
        ctx->comm_ll = value != 0;
    else if (n == "gemm_splitk")
        ctx->gemm_splitk = (int)value;
    else if (n == "gemm_pg") {
        TLC_REQUIRE(value >= 0 && value <= 2, TLC_ERR_INVALID_OPERATION, "set_option: gemm_pg must be 0, 1 or 2");
        ctx->gemm_pg = (int)value;
    } else if (n == "gemm_tma")
        ctx->gemm_tma = value != 0;
    else if (n == "pdl")
        ctx->use_pdl = value != 0;
    else if (n == "pdl_mode") {
        TLC_REQUIRE(value >= 0 && value <= 4, TLC_ERR_INVALID_OPERATION, "set_option: pdl_mode must be 0..4");
        ctx->pdl_mode = (int)value;
    } else if (n == "attn_wide")
        ctx->attn_wide = (int)value;
    else if (n == "l2_hint")
        ctx->l2_hint = value != 0;
    else if (n == "host_graph")
        ctx->host_graph = value != 0;
    else if (n == "host_poll")
        ctx->host_poll = value != 0;
    else if (n == "step_kernel")
        ctx->step_kernel = value != 0;
    else if (n == "gemv_f8")
        ctx->gemv_f8 = value != 0;
    else if (n == "gemv_splitk")
        ctx->gemv_splitk = (int)value;
    else if (n == "q6k_resident")
        ctx->q6k_resident = value != 0;
    else
        return tlc_fail(TLC_ERR_INVALID_OPERATION, "set_option: unknown option '%s'", name);
    return TLC_OK;
}

tlc_perf_scope::tlc_perf_scope(tlc_ctx *c, const char *fmt, ...) : ctx(c) {
    name[0] = 0;
    if (!c || !c->perf) return;
    cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(c->stream, &cap) != cudaSuccess || cap != cudaStreamCaptureStatusNone) {
        cudaGetLastError();
        return;
    }
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(name, sizeof name, fmt, ap);
    va_end(ap);
    if (cudaEventCreate(&e0) != cudaSuccess || cudaEventCreate(&e1) != cudaSuccess ||
        cudaEventRecord(e0, c->stream) != cudaSuccess) {
        cudaGetLastError();
        if (e0) cudaEventDestroy(e0);
        if (e1) cudaEventDestroy(e1);
        e0 = e1 = nullptr;
        return;
    }
    on = true;
}

tlc_perf_scope::~tlc_perf_scope() {
    if (!on) return;
    float ms = 0.f;
    if (cudaEventRecord(e1, ctx->stream) == cudaSuccess && cudaEventSynchronize(e1) == cudaSuccess &&
        cudaEventElapsedTime(&ms, e0, e1) == cudaSuccess) {
        fprintf(stderr, "[PERF] %s: %.3fms\n", name, ms);
        // totals by op name without its shape: "linear(q4_0, ...)" counts under "linear"
        std::string key(name);
        const size_t paren = key.find('(');
        if (paren != std::string::npos) key.resize(paren);
        tlc_ctx::perf_total &t = ctx->perf_totals[key];
        t.calls++;
        t.ms += ms;
    } else {
        cudaGetLastError();
    }
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
}

// Per-op totals of the "perf" option as text, one line per op: "name calls total_ms".  Returns the
// number of bytes the whole report needs (excluding the terminating zero); `reset` clears the totals.
extern "C" int32_t tlc_perf_report(tlc_ctx *ctx, char *buf, size_t buflen, int32_t reset, size_t *needed_out) {
    if (int32_t rc = tlc_enter(ctx)) return rc;
    std::string out;
    char line[160];
    for (const auto &kv : ctx->perf_totals) {
        snprintf(line, sizeof line, "%s %llu %.3f\n", kv.first.c_str(), (unsigned long long)kv.second.calls, kv.second.ms);
        out += line;
    }
    if (needed_out) *needed_out = out.size();
    if (buf && buflen > 0) {
        const size_t n = out.size() < buflen - 1 ? out.size() : buflen - 1;
        memcpy(buf, out.data(), n);
        buf[n] = 0;
    }
    if (reset) ctx->perf_totals.clear();
    return TLC_OK;
}

extern "C" int32_t tlc_selftest_wait_timeout(tlc_ctx *ctx, int32_t kind) {
    if (int32_t rc = tlc_enter(ctx)) return rc;
    TLC_REQUIRE(kind >= 0 && kind <= 2, TLC_ERR_INVALID_OPERATION, "selftest_wait_timeout: kind %d (0, 1 or 2)", kind);
    return kind == 0 ? tlc_selftest_mbarrier_wait(ctx) : tlc_selftest_peer_wait(ctx, kind == 2);
}

extern "C" int32_t tlc_destroy(tlc_ctx *ctx) {
    if (!ctx) return TLC_OK;
    cudaSetDevice(ctx->device);
    cudaStreamSynchronize(ctx->stream);
    for (auto &kv : ctx->pool.idle)
        for (void *p : kv.second) cudaFree(p);
    if (ctx->scratch) cudaFree(ctx->scratch);
    cudaFree(ctx->dev_status);
    cudaFree(ctx->tickets);
    cudaFreeHost(ctx->host_status);
    cudaStreamDestroy(ctx->stream);
    delete ctx;
    return TLC_OK;
}

extern "C" int32_t tlc_device_name(tlc_ctx *ctx, char *buf, size_t buflen) {
    TLC_REQUIRE(ctx && buf && buflen > 0, TLC_ERR_INVALID_OPERATION, "tlc_device_name: bad arguments");
    snprintf(buf, buflen, "%s", ctx->prop.name);
    return TLC_OK;
}

extern "C" int32_t tlc_mem_info(tlc_ctx *ctx, size_t *free_bytes, size_t *total_bytes) {
    if (int32_t rc = tlc_enter(ctx)) return rc;
    size_t f = 0, t = 0;
    TLC_CUDA(cudaMemGetInfo(&f, &t));
    if (free_bytes) *free_bytes = f;
    if (total_bytes) *total_bytes = t;
    return TLC_OK;
}

extern "C" int32_t tlc_sm_count(tlc_ctx *ctx, int32_t *out) {
    TLC_REQUIRE(ctx && out, TLC_ERR_INVALID_OPERATION, "tlc_sm_count: bad arguments");
    *out = ctx->sm_count;
    return TLC_OK;
}

extern "C" void *tlc_stream(tlc_ctx *ctx) { return ctx ? (void *)ctx->stream : nullptr; }
extern "C" uint64_t tlc_launch_count(tlc_ctx *ctx) { return ctx ? ctx->launches : 0; }

extern "C" int32_t tlc_synchronize(tlc_ctx *ctx) {
    if (int32_t rc = tlc_enter(ctx)) return rc;
    TLC_CUDA(cudaMemcpyAsync(ctx->host_status, ctx->dev_status, sizeof(tlc_dev_status),
                             cudaMemcpyDeviceToHost, ctx->stream));
    TLC_CUDA(cudaStreamSynchronize(ctx->stream));
    return tlc_status_after_sync(ctx);
}

// The status word has just been copied to its pinned mirror and the stream is idle:
// report (once) a bounded wait that gave up, and clear the word.
int32_t tlc_status_after_sync(tlc_ctx *ctx) {
    if (ctx->host_status->code != 0) {
        int code = ctx->host_status->code, where = ctx->host_status->where;
        cudaMemsetAsync(ctx->dev_status, 0, sizeof(tlc_dev_status), ctx->stream);
        cudaStreamSynchronize(ctx->stream);
        if (code == TLC_DEV_INDEX)
            return tlc_fail(TLC_ERR_INDEX, "Index out of bounds: a sequence position lies outside the KV cache "
                            "(site %d); the access was skipped", where);
        return tlc_fail(TLC_ERR_TIMEOUT, "a device-side bounded wait gave up (code %d at site %d)", code,
                        where);
    }
    return TLC_OK;
}

int32_t tlc_scratch_reserve(tlc_ctx *ctx, size_t bytes) {
    if (bytes <= ctx->scratch_bytes) return TLC_OK;
    // Growing replaces the allocation; earlier kernels may still be using it.
    TLC_CUDA(cudaStreamSynchronize(ctx->stream));
    if (ctx->scratch) TLC_CUDA(cudaFree(ctx->scratch));
    ctx->scratch = nullptr;
    ctx->scratch_bytes = 0;
    size_t want = (bytes + ((size_t)1 << 20) - 1) & ~(((size_t)1 << 20) - 1);
    cudaError_t e = cudaMalloc(&ctx->scratch, want);
    if (e != cudaSuccess) {
        cudaGetLastError();
        return tlc_fail(TLC_ERR_ALLOCATION, "scratch allocation of %zu bytes failed: %s", want,
                        cudaGetErrorString(e));
    }
    ctx->scratch_bytes = want;
    return TLC_OK;
}

// ---- pool -----------------------------------------------------------------

// Size classes of BufferPool::get_size_class (buffer_pool.rs:78-101), in
// bytes: 1 Ki .. 8 Mi f16 elements = 2 KiB .. 16 MiB; larger requests keep
// their exact size (rounded up to 256 B so every buffer stays 256-B aligned
// in size as well as in address).
static size_t size_class(size_t bytes) {
    size_t c = 2048;
    while (c < bytes && c < ((size_t)16 << 20)) c <<= 1;
    if (c >= bytes) return c;
    return (bytes + 255) & ~(size_t)255;
}

extern "C" int32_t tlc_alloc(tlc_ctx *ctx, size_t bytes, tlc_buf **out) {
    if (int32_t rc = tlc_enter(ctx)) return rc;
    TLC_REQUIRE(out != nullptr, TLC_ERR_INVALID_OPERATION, "tlc_alloc: null out pointer");
    *out = nullptr;
    size_t cls = size_class(bytes == 0 ? 1 : bytes);
    void *p = nullptr;
    auto it = ctx->pool.idle.find(cls);
    if (it != ctx->pool.idle.end() && !it->second.empty()) {
        p = it->second.back();
        it->second.pop_back();
        if (it->second.empty()) ctx->pool.idle.erase(it);
        ctx->pool.stats.reuse_count++;
    } else {
        cudaError_t e = cudaMalloc(&p, cls);
        if (e != cudaSuccess) {
            cudaGetLastError();
            // Give idle memory back to the driver and retry once.
            tlc_pool_trim(ctx, 0);
            e = cudaMalloc(&p, cls);
        }
        if (e != cudaSuccess) {
            cudaGetLastError();
            size_t f = 0, t = 0;
            cudaMemGetInfo(&f, &t);
            return tlc_fail(TLC_ERR_BUFFER_EXHAUSTED,
                            "Buffer exhausted: requested %zu bytes, available %zu bytes", cls, f);
        }
        ctx->pool.stats.allocation_count++;
    }
    ctx->pool.stats.live_bytes += cls;
    *out = new tlc_buf{ctx, p, cls, bytes};
    return TLC_OK;
}

extern "C" int32_t tlc_free(tlc_buf *buf) {
    if (!buf) return TLC_OK;
    tlc_ctx *ctx = buf->ctx;
    if (int32_t rc = tlc_enter(ctx)) return rc;
    ctx->pool.stats.live_bytes -= buf->class_bytes;
    auto &vec = ctx->pool.idle[buf->class_bytes];
    if (vec.size() < ctx->pool.max_per_class) {
        // All work is ordered on ctx->stream, so a later user of this memory
        // cannot overtake kernels already queued on it.
        vec.push_back(buf->ptr);
    } else {
        // cudaFree waits for outstanding work on the memory.
        cudaFree(buf->ptr);
        ctx->pool.stats.eviction_count++;
        if (vec.empty()) ctx->pool.idle.erase(buf->class_bytes);
    }
    delete buf;
    return TLC_OK;
}

extern "C" void *tlc_buf_ptr(tlc_buf *buf) { return buf ? buf->ptr : nullptr; }
extern "C" size_t tlc_buf_size(tlc_buf *buf) { return buf ? buf->class_bytes : 0; }

extern "C" int32_t tlc_pool_stats_get(tlc_ctx *ctx, tlc_pool_stats *out) {
    TLC_REQUIRE(ctx && out, TLC_ERR_INVALID_OPERATION, "tlc_pool_stats_get: bad arguments");
    tlc_pool_stats s = ctx->pool.stats;
    s.total_pooled = 0;
    s.total_memory = 0;
    s.size_classes = 0;
    for (auto &kv : ctx->pool.idle) {
        if (kv.second.empty()) continue;
        s.size_classes++;
        s.total_pooled += kv.second.size();
        s.total_memory += kv.first * kv.second.size();
    }
    *out = s;
    return TLC_OK;
}

extern "C" int32_t tlc_pool_trim(tlc_ctx *ctx, size_t max_idle_bytes) {
    if (int32_t rc = tlc_enter(ctx)) return rc;
    size_t idle = 0;
    for (auto &kv : ctx->pool.idle) idle += kv.first * kv.second.size();
    // Largest classes go first.
    for (auto it = ctx->pool.idle.rbegin(); it != ctx->pool.idle.rend() && idle > max_idle_bytes; ++it) {
        while (!it->second.empty() && idle > max_idle_bytes) {
            cudaFree(it->second.back());
            it->second.pop_back();
            idle -= it->first;
            ctx->pool.stats.eviction_count++;
        }
    }
    for (auto it = ctx->pool.idle.begin(); it != ctx->pool.idle.end();)
        it = it->second.empty() ? ctx->pool.idle.erase(it) : std::next(it);
    return TLC_OK;
}

// ---- transfers --------------------------------------------------------------

extern "C" int32_t tlc_upload(tlc_ctx *ctx, void *dst_dev, const void *src_host, size_t bytes) {
    if (int32_t rc = tlc_enter(ctx)) return rc;
    TLC_REQUIRE(dst_dev && src_host, TLC_ERR_INVALID_OPERATION, "tlc_upload: null pointer");
    TLC_CUDA(cudaMemcpyAsync(dst_dev, src_host, bytes, cudaMemcpyHostToDevice, ctx->stream));
    return TLC_OK;
}

extern "C" int32_t tlc_download(tlc_ctx *ctx, void *dst_host, const void *src_dev, size_t bytes) {
    if (int32_t rc = tlc_enter(ctx)) return rc;
    TLC_REQUIRE(dst_host && src_dev, TLC_ERR_INVALID_OPERATION, "tlc_download: null pointer");
    TLC_CUDA(cudaMemcpyAsync(dst_host, src_dev, bytes, cudaMemcpyDeviceToHost, ctx->stream));
    return tlc_synchronize(ctx);
}

extern "C" int32_t tlc_host_alloc(size_t bytes, void **out) {
    TLC_REQUIRE(out != nullptr, TLC_ERR_INVALID_OPERATION, "tlc_host_alloc: null out pointer");
    cudaError_t e = cudaMallocHost(out, bytes == 0 ? 1 : bytes);
    if (e != cudaSuccess) {
        cudaGetLastError();
        return tlc_fail(TLC_ERR_ALLOCATION, "pinned host allocation of %zu bytes failed: %s", bytes,
                        cudaGetErrorString(e));
    }
    return TLC_OK;
}

extern "C" int32_t tlc_host_free(void *p) {
    if (p) cudaFreeHost(p);
    return TLC_OK;
}
