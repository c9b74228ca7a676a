// Stand-alone per-token ops of the builtin surface (rms_norm, rope, sigmoid,
// mul, add, softmax, embedding) and the C-ABI entry points of the linear
// family.  The TL scripts call these builtins one by one
// (debug/chat_demo_with_kvcache.tl:219-290); the fused entry points in
// tlc_gemv.cu fold them into the GEMV launches.
#include <cmath>
#include <vector>

#include "tlc_internal.h"

namespace {

// rms_norm_f16 (shaders/unified.metal:1785-1831) / Tensor::rms_norm_cpu
// (src/ops/normalization.rs:199-248): one CTA per row.
__global__ void rms_norm_kernel(const __half *__restrict__ x, const __half *__restrict__ w,
                                __half *__restrict__ y, int d, float eps) {
    __shared__ float warp_sums[32];
    __shared__ float inv_s;
    const __half *xr = x + (size_t)blockIdx.x * d;
    __half *yr = y + (size_t)blockIdx.x * d;
    // 16-byte accesses when the row allows it (d a multiple of 8, 16-byte aligned pointers)
    const bool vec = (d & 7) == 0 && ((((uintptr_t)x | (uintptr_t)w | (uintptr_t)y) & 15) == 0);
    float sq = 0.f;
    if (vec) {
        for (int i = threadIdx.x; i < (d >> 3); i += blockDim.x) {
            const uint4 raw = reinterpret_cast<const uint4 *>(xr)[i];
            const __half2 *h = reinterpret_cast<const __half2 *>(&raw);
#pragma unroll
            for (int j = 0; j < 4; j++) {
                const float2 v = __half22float2(h[j]);
                sq = fmaf(v.x, v.x, sq);
                sq = fmaf(v.y, v.y, sq);
            }
        }
    } else {
        for (int i = threadIdx.x; i < d; i += blockDim.x) {
            float v = __half2float(xr[i]);
            sq = fmaf(v, v, sq);
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
    if ((threadIdx.x & 31) == 0) warp_sums[threadIdx.x >> 5] = sq;
    __syncthreads();
    if (threadIdx.x < 32) {
        float v = threadIdx.x < (blockDim.x >> 5) ? warp_sums[threadIdx.x] : 0.f;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
        if (threadIdx.x == 0) inv_s = 1.0f / sqrtf(v / (float)d + eps);
    }
    __syncthreads();
    const float inv = inv_s;
    if (vec) {
        for (int i = threadIdx.x; i < (d >> 3); i += blockDim.x) {
            const uint4 raw = reinterpret_cast<const uint4 *>(xr)[i], wraw = reinterpret_cast<const uint4 *>(w)[i];
            const __half *xh = reinterpret_cast<const __half *>(&raw), *wh = reinterpret_cast<const __half *>(&wraw);
            __align__(16) __half o[8];
#pragma unroll
            for (int j = 0; j < 8; j++)
                o[j] = __float2half_rn(__fmul_rn(__fmul_rn(__half2float(xh[j]), inv), __half2float(wh[j])));
            reinterpret_cast<uint4 *>(yr)[i] = *reinterpret_cast<const uint4 *>(o);
        }
    } else {
        for (int i = threadIdx.x; i < d; i += blockDim.x) {
            float nrm = __fmul_rn(__half2float(xr[i]), inv);
            yr[i] = __float2half_rn(__fmul_rn(nrm, __half2float(w[i])));
        }
    }
}

// rope_f16 (shaders/unified.metal:2355-2417): one thread per pair.
__global__ void rope_kernel(const __half *__restrict__ x, __half *__restrict__ y, int seq, int heads, int d,
                            int pos_offset, float base, const int *__restrict__ positions) {
    const int half_d = d >> 1;
    const size_t total = (size_t)seq * heads * half_d;
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const int pair = (int)(i % half_d);
    const size_t sh = i / half_d;
    const int s = (int)(sh / heads);
    const unsigned pos = positions ? (unsigned)positions[s] : (unsigned)(s + pos_offset);
    const float exponent = (float)(2 * pair) / (float)d;
    const float freq = 1.0f / powf(base, exponent);
    const float theta = (float)pos * freq;
    const float cs = cosf(theta), sn = sinf(theta);
    const size_t o = sh * d + 2 * pair;
    const float x0 = __half2float(x[o]), x1 = __half2float(x[o + 1]);
    y[o] = __float2half_rn(__fsub_rn(__fmul_rn(x0, cs), __fmul_rn(x1, sn)));
    y[o + 1] = __float2half_rn(__fadd_rn(__fmul_rn(x0, sn), __fmul_rn(x1, cs)));
}

// rope_candle_f16 (shaders/unified.metal:5122-5184): the same interleaved rotation with the
// cosines and sines read from f16 tables instead of being worked out.  Pair p of position s
// reads table[s * pitch + p] -- exactly the shader's index arithmetic (`seq_idx * head_dim +
// dim_pair_idx`, i.e. pitch = head_dim there).  One thread per pair.
__global__ void rope_table_kernel(const __half *__restrict__ x, const __half *__restrict__ cos_t,
                                  const __half *__restrict__ sin_t, __half *__restrict__ y, int seq, int heads, int d,
                                  int pitch) {
    const int half_d = d >> 1;
    const size_t total = (size_t)seq * heads * half_d;
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const int pair = (int)(i % half_d);
    const size_t sh = i / half_d;
    const int s = (int)(sh / heads);
    const float cs = __half2float(cos_t[(size_t)s * pitch + pair]), sn = __half2float(sin_t[(size_t)s * pitch + pair]);
    const size_t o = sh * d + 2 * pair;
    const float x0 = __half2float(x[o]), x1 = __half2float(x[o + 1]);
    y[o] = __float2half_rn(__fsub_rn(__fmul_rn(x0, cs), __fmul_rn(x1, sn)));
    y[o + 1] = __float2half_rn(__fadd_rn(__fmul_rn(x0, sn), __fmul_rn(x1, cs)));
}

// Dense C[M, N] = A[M, K] . B[K, N], f16 in, f32 accumulate, one rounding to f16 (the matmul
// builtin: Tensor::matmul, src/ops/matmul.rs:13-75; kernels matmul_f16 / matmul_tiled_f16,
// shaders/unified.metal:33-478).  64 x 64 output tile per CTA of 256 threads, 4 x 4 outputs per
// thread, K in steps of 16 through shared memory.  A general-purpose builtin, not a tuned path:
// the model's linears never come here (they are quantized or go through tlc_linear).
__global__ void __launch_bounds__(256) matmul_f16_kernel(const __half *__restrict__ a, const __half *__restrict__ b,
                                                         __half *__restrict__ c, int m, int k, int n) {
    __shared__ float as[16][64 + 1], bs[16][64 + 1];
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    const int row0 = blockIdx.y * 64, col0 = blockIdx.x * 64;
    float acc[4][4] = {};
    for (int k0 = 0; k0 < k; k0 += 16) {
        for (int i = threadIdx.x; i < 64 * 16; i += 256) {
            const int r = i >> 4, kk = i & 15;  // A tile: 64 rows x 16 k
            as[kk][r] = row0 + r < m && k0 + kk < k ? __half2float(a[(size_t)(row0 + r) * k + k0 + kk]) : 0.f;
            const int kb = i >> 6, cc = i & 63;  // B tile: 16 k x 64 columns
            bs[kb][cc] = k0 + kb < k && col0 + cc < n ? __half2float(b[(size_t)(k0 + kb) * n + col0 + cc]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < 16; kk++) {
            float av[4], bv[4];
#pragma unroll
            for (int i = 0; i < 4; i++) {
                av[i] = as[kk][ty * 4 + i];
                bv[i] = bs[kk][tx * 4 + i];
            }
#pragma unroll
            for (int i = 0; i < 4; i++)
#pragma unroll
                for (int j = 0; j < 4; j++) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; i++)
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const int r = row0 + ty * 4 + i, cc = col0 + tx * 4 + j;
            if (r < m && cc < n) c[(size_t)r * n + cc] = __float2half_rn(acc[i][j]);
        }
}

// sigmoid: f32 math, RNE to f16 (Tensor::sigmoid_cpu, src/ops/activations.rs:252-266).
__global__ void sigmoid_kernel(const __half *__restrict__ x, __half *__restrict__ y, size_t n) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) y[i] = __float2half_rn(1.0f / (1.0f + expf(-__half2float(x[i]))));
}
__global__ void mul_kernel(const __half *__restrict__ a, const __half *__restrict__ b, __half *__restrict__ y,
                           size_t n) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) y[i] = __hmul(a[i], b[i]);
}
__global__ void add_kernel(const __half *__restrict__ a, const __half *__restrict__ b, __half *__restrict__ y,
                           size_t n) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) y[i] = __hadd(a[i], b[i]);
}
__global__ void swiglu_kernel(const __half *__restrict__ g, const __half *__restrict__ u,
                              __half *__restrict__ y, size_t n) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const __half gv = g[i];
    const __half s = __float2half_rn(1.0f / (1.0f + expf(-__half2float(gv))));
    y[i] = __hmul(__hmul(gv, s), u[i]);
}

// softmax over the last dim, one warp per row; arithmetic of
// softmax_simple_f16 (shaders/unified.metal:2150-2200): finite-only f32 max and
// sum, exponentials rounded to f16 before the divide, uniform row when the sum
// degenerates.
__global__ void softmax_kernel(const __half *__restrict__ x, __half *__restrict__ y, int rows, int last) {
    const int row = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (row >= rows) return;
    const __half *xr = x + (size_t)row * last;
    __half *yr = y + (size_t)row * last;
    float mx = -INFINITY;
    for (int i = lane; i < last; i += 32) {
        float v = __half2float(xr[i]);
        if (isfinite(v)) mx = fmaxf(mx, v);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    if (!isfinite(mx)) mx = 0.f;
    float sum = 0.f;
    for (int i = lane; i < last; i += 32) {
        float v = __half2float(xr[i]);
        sum += isfinite(v) ? expf(v - mx) : 0.f;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    if (sum > 0.f && isfinite(sum)) {
        for (int i = lane; i < last; i += 32) {
            float v = __half2float(xr[i]);
            float e = isfinite(v) ? expf(v - mx) : 0.f;
            yr[i] = __float2half_rn(__half2float(__float2half_rn(e)) / sum);
        }
    } else {
        const __half u = __float2half_rn(1.0f / (float)last);
        for (int i = lane; i < last; i += 32) yr[i] = u;
    }
}

// embedding_lookup_f16 (shaders/unified.metal:658-675): 16-byte vector gather.
__global__ void embedding_kernel(const __half *__restrict__ table, const int *__restrict__ ids, int d,
                                 int m, __half *__restrict__ y) {
    const int vec_per_row = d >> 3;
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (size_t)m * vec_per_row) return;
    const int r = (int)(i / vec_per_row), c = (int)(i % vec_per_row);
    reinterpret_cast<uint4 *>(y + (size_t)r * d)[c] =
        reinterpret_cast<const uint4 *>(table + (size_t)ids[r] * d)[c];
}
__global__ void embedding_scalar_kernel(const __half *__restrict__ table, const int *__restrict__ ids, int d,
                                        int m, __half *__restrict__ y) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (size_t)m * d) return;
    const int r = (int)(i / d), c = (int)(i % d);
    y[i] = table[(size_t)ids[r] * d + c];
}

// Eight elements per thread (16-byte accesses) for the large element-wise passes of a prefill.
__global__ void swiglu_vec8_kernel(const uint4 *__restrict__ g, const uint4 *__restrict__ u, uint4 *__restrict__ y,
                                   size_t n8) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n8) return;
    const uint4 gv = g[i], uv = u[i];
    const __half *gh = reinterpret_cast<const __half *>(&gv), *uh = reinterpret_cast<const __half *>(&uv);
    __align__(16) __half o[8];
#pragma unroll
    for (int j = 0; j < 8; j++) {
        const __half s = __float2half_rn(1.0f / (1.0f + expf(-__half2float(gh[j]))));
        o[j] = __hmul(__hmul(gh[j], s), uh[j]);
    }
    y[i] = *reinterpret_cast<const uint4 *>(o);
}

inline unsigned blocks_for(size_t n, int threads) { return (unsigned)((n + threads - 1) / threads); }

}  // namespace

extern "C" int32_t tlc_rms_norm(tlc_ctx *ctx, const void *x_dev, const void *w_dev, void *y_dev, int32_t rows,
                                int32_t d, float eps) {
    if (int32_t rc = tlc_enter(ctx)) return rc;
    tlc_perf_scope perf(ctx, "rms_norm(rows=%d, d=%d)", rows, d);
    TLC_REQUIRE(x_dev && w_dev && y_dev, TLC_ERR_INVALID_OPERATION, "rms_norm: null pointer");
    TLC_REQUIRE(rows >= 0 && d > 0, TLC_ERR_INVALID_DIMENSION, "rms_norm: bad shape [%d, %d]", rows, d);
    if (rows == 0) return TLC_OK;
    rms_norm_kernel<<<rows, 256, 0, ctx->stream>>>(static_cast<const __half *>(x_dev),
                                                   static_cast<const __half *>(w_dev),
                                                   static_cast<__half *>(y_dev), d, eps);
    TLC_CHECK_LAUNCH(ctx);
    return TLC_OK;
}

extern "C" int32_t tlc_rope(tlc_ctx *ctx, const void *x_dev, void *y_dev, int32_t seq, int32_t heads,
                            int32_t d, int32_t pos_offset, uint32_t base, const int32_t *positions_dev) {
    if (int32_t rc = tlc_enter(ctx)) return rc;
    tlc_perf_scope perf(ctx, "rope(seq=%d, heads=%d, d=%d)", seq, heads, d);
    TLC_REQUIRE(x_dev && y_dev, TLC_ERR_INVALID_OPERATION, "rope: null pointer");
    // Tensor::rope rejects an odd head_dim (src/ops/rope.rs:90-96).
    TLC_REQUIRE(d > 0 && d % 2 == 0, TLC_ERR_INVALID_OPERATION, "RoPE requires even head_dim, got %d", d);
    TLC_REQUIRE(seq >= 0 && heads > 0, TLC_ERR_INVALID_DIMENSION, "rope: bad shape [%d, %d, %d]", seq, heads, d);
    if (seq == 0) return TLC_OK;
    const size_t total = (size_t)seq * heads * (d / 2);
    rope_kernel<<<blocks_for(total, 256), 256, 0, ctx->stream>>>(
        static_cast<const __half *>(x_dev), static_cast<__half *>(y_dev), seq, heads, d, pos_offset, (float)base,
        positions_dev);
    TLC_CHECK_LAUNCH(ctx);
    return TLC_OK;
}

// rope(x, cos, sin): the arm of the rope builtin that takes precomputed tables
// (src/interpreter/builtin_tensor.rs:634-722 -> Tensor::rope_candle, src/ops/rope.rs:18-65).
// x, y: [seq, heads, d] f16; cos/sin: f16 tables of table_rows rows, `pitch` elements apart;
// pair p of position s uses cos[s * pitch + p], sin[s * pitch + p].
//   * A table of head_dim / 2 columns (pitch = head_dim / 2, one column per rotary pair) is what
//     the kernel's index arithmetic is written for, and gives the same rotation as tlc_rope.
//   * The reference's own builtin stores every frequency twice in rows of head_dim values and
//     passes pitch = head_dim in effect: pair p then reads column p of a row laid out
//     c0 c0 c1 c1 ..., i.e. frequency p / 2 -- its result, quirk included, is reproduced by
//     passing that table with pitch = head_dim.
extern "C" int32_t tlc_rope_table(tlc_ctx *ctx, const void *x_dev, const void *cos_dev, const void *sin_dev,
                                  void *y_dev, int32_t seq, int32_t heads, int32_t d, int32_t table_rows,
                                  int32_t pitch) {
    if (int32_t rc = tlc_enter(ctx)) return rc;
    tlc_perf_scope perf(ctx, "rope_table(seq=%d, heads=%d, d=%d)", seq, heads, d);
    TLC_REQUIRE(x_dev && cos_dev && sin_dev && y_dev, TLC_ERR_INVALID_OPERATION, "rope: null pointer");
    TLC_REQUIRE(d > 0 && d % 2 == 0, TLC_ERR_INVALID_OPERATION, "RoPE requires even head_dim, got %d", d);
    TLC_REQUIRE(seq >= 0 && heads > 0, TLC_ERR_INVALID_DIMENSION, "rope: bad shape [%d, %d, %d]", seq, heads, d);
    TLC_REQUIRE(pitch >= d / 2, TLC_ERR_INVALID_OPERATION,
                "cos/sin last dim must hold head_dim / 2 = %d pairs, got %d", d / 2, pitch);
    TLC_REQUIRE(table_rows >= seq, TLC_ERR_INVALID_OPERATION,
                "cos/sin first dim must be >= seq_len = %d, got cos: %d, sin: %d", seq, table_rows, table_rows);
    if (seq == 0) return TLC_OK;
    const size_t total = (size_t)seq * heads * (d / 2);
    rope_table_kernel<<<blocks_for(total, 256), 256, 0, ctx->stream>>>(
        static_cast<const __half *>(x_dev), static_cast<const __half *>(cos_dev), static_cast<const __half *>(sin_dev),
        static_cast<__half *>(y_dev), seq, heads, d, pitch);
    TLC_CHECK_LAUNCH(ctx);
    return TLC_OK;
}

// matmul(a, b): a [m, k] . b [k2, n] -> y [m, n], all f16 on the device.  Shape rule and message
// of Tensor::matmul (src/ops/matmul.rs:36-46).
extern "C" int32_t tlc_matmul(tlc_ctx *ctx, const void *a_dev, const void *b_dev, void *y_dev, int32_t m, int32_t k,
                              int32_t k2, int32_t n) {
    if (int32_t rc = tlc_enter(ctx)) return rc;
    tlc_perf_scope perf(ctx, "matmul(m=%d, k=%d, n=%d)", m, k, n);
    TLC_REQUIRE(a_dev && b_dev && y_dev, TLC_ERR_INVALID_OPERATION, "matmul: null pointer");
    TLC_REQUIRE(m >= 0 && k >= 0 && k2 >= 0 && n >= 0, TLC_ERR_INVALID_DIMENSION, "matmul: bad shape");
    TLC_REQUIRE(k == k2, TLC_ERR_INVALID_OPERATION, "matmul shape mismatch: [%d, %d] @ [%d, %d]", m, k, k2, n);
    if (m == 0 || n == 0) return TLC_OK;
    const dim3 grid((unsigned)((n + 63) / 64), (unsigned)((m + 63) / 64));
    matmul_f16_kernel<<<grid, 256, 0, ctx->stream>>>(static_cast<const __half *>(a_dev), static_cast<const __half *>(b_dev),
                                                     static_cast<__half *>(y_dev), m, k, n);
    TLC_CHECK_LAUNCH(ctx);
    return TLC_OK;
}

#define TLC_ELEMENTWISE_1(name, kernel)                                                                  \
    extern "C" int32_t name(tlc_ctx *ctx, const void *x_dev, void *y_dev, size_t n) {                    \
        if (int32_t rc = tlc_enter(ctx)) return rc;                                                      \
        TLC_REQUIRE(x_dev && y_dev, TLC_ERR_INVALID_OPERATION, #name ": null pointer");                  \
        if (n == 0) return TLC_OK;                                                                       \
        tlc_perf_scope perf(ctx, "%s(n=%zu)", #name + 4, n);                                             \
        kernel<<<blocks_for(n, 256), 256, 0, ctx->stream>>>(static_cast<const __half *>(x_dev),          \
                                                            static_cast<__half *>(y_dev), n);            \
        TLC_CHECK_LAUNCH(ctx);                                                                           \
        return TLC_OK;                                                                                   \
    }
#define TLC_ELEMENTWISE_2(name, kernel)                                                                  \
    extern "C" int32_t name(tlc_ctx *ctx, const void *a_dev, const void *b_dev, void *y_dev, size_t n) { \
        if (int32_t rc = tlc_enter(ctx)) return rc;                                                      \
        TLC_REQUIRE(a_dev && b_dev && y_dev, TLC_ERR_INVALID_OPERATION, #name ": null pointer");         \
        if (n == 0) return TLC_OK;                                                                       \
        tlc_perf_scope perf(ctx, "%s(n=%zu)", #name + 4, n);                                             \
        kernel<<<blocks_for(n, 256), 256, 0, ctx->stream>>>(static_cast<const __half *>(a_dev),          \
                                                            static_cast<const __half *>(b_dev),          \
                                                            static_cast<__half *>(y_dev), n);            \
        TLC_CHECK_LAUNCH(ctx);                                                                           \
        return TLC_OK;                                                                                   \
    }

TLC_ELEMENTWISE_1(tlc_sigmoid, sigmoid_kernel)
TLC_ELEMENTWISE_2(tlc_mul, mul_kernel)
TLC_ELEMENTWISE_2(tlc_add, add_kernel)
extern "C" int32_t tlc_swiglu(tlc_ctx *ctx, const void *a_dev, const void *b_dev, void *y_dev, size_t n) {
    if (int32_t rc = tlc_enter(ctx)) return rc;
    tlc_perf_scope perf(ctx, "swiglu(n=%zu)", n);
    TLC_REQUIRE(a_dev && b_dev && y_dev, TLC_ERR_INVALID_OPERATION, "tlc_swiglu: null pointer");
    if (n == 0) return TLC_OK;
    if (n % 8 == 0 && (((uintptr_t)a_dev | (uintptr_t)b_dev | (uintptr_t)y_dev) & 15) == 0)
        swiglu_vec8_kernel<<<blocks_for(n / 8, 256), 256, 0, ctx->stream>>>(
            static_cast<const uint4 *>(a_dev), static_cast<const uint4 *>(b_dev), static_cast<uint4 *>(y_dev), n / 8);
    else
        swiglu_kernel<<<blocks_for(n, 256), 256, 0, ctx->stream>>>(
            static_cast<const __half *>(a_dev), static_cast<const __half *>(b_dev), static_cast<__half *>(y_dev), n);
    TLC_CHECK_LAUNCH(ctx);
    return TLC_OK;
}

extern "C" int32_t tlc_softmax(tlc_ctx *ctx, const void *x_dev, void *y_dev, int32_t rows, int32_t last_dim) {
    if (int32_t rc = tlc_enter(ctx)) return rc;
    tlc_perf_scope perf(ctx, "softmax(rows=%d, d=%d)", rows, last_dim);
    TLC_REQUIRE(x_dev && y_dev, TLC_ERR_INVALID_OPERATION, "softmax: null pointer");
    TLC_REQUIRE(rows >= 0 && last_dim > 0, TLC_ERR_INVALID_DIMENSION, "softmax: bad shape [%d, %d]", rows, last_dim);
    if (rows == 0) return TLC_OK;
    softmax_kernel<<<blocks_for((size_t)rows * 32, 256), 256, 0, ctx->stream>>>(
        static_cast<const __half *>(x_dev), static_cast<__half *>(y_dev), rows, last_dim);
    TLC_CHECK_LAUNCH(ctx);
    return TLC_OK;
}

extern "C" int32_t tlc_embedding(tlc_ctx *ctx, const void *table_dev, int32_t vocab, int32_t d,
                                 const int32_t *ids_host, int32_t m, void *y_dev) {
    if (int32_t rc = tlc_enter(ctx)) return rc;
    tlc_perf_scope perf(ctx, "embedding(d=%d)", d);
    TLC_REQUIRE(table_dev && ids_host && y_dev, TLC_ERR_INVALID_OPERATION, "embedding: null pointer");
    TLC_REQUIRE(vocab > 0 && d > 0 && m >= 0, TLC_ERR_INVALID_DIMENSION, "embedding: bad shape");
    // Host-side bounds check as in src/interpreter/builtin_nn.rs:681-688.
    for (int i = 0; i < m; i++)
        TLC_REQUIRE(ids_host[i] >= 0 && ids_host[i] < vocab, TLC_ERR_INDEX,
                    "Index out of bounds: index %d, size %d", ids_host[i], vocab);
    if (m == 0) return TLC_OK;
    tlc_buf *ids = nullptr;
    if (int32_t rc = tlc_alloc(ctx, (size_t)m * sizeof(int32_t), &ids)) return rc;
    cudaError_t e = cudaMemcpyAsync(ids->ptr, ids_host, (size_t)m * sizeof(int32_t), cudaMemcpyHostToDevice,
                                    ctx->stream);
    if (e != cudaSuccess) {
        tlc_free(ids);
        return tlc_fail(TLC_ERR_CUDA, "embedding: id upload failed: %s", cudaGetErrorString(e));
    }
    const bool vec = d % 8 == 0 && ((uintptr_t)table_dev % 16 == 0) && ((uintptr_t)y_dev % 16 == 0);
    if (vec)
        embedding_kernel<<<blocks_for((size_t)m * (d / 8), 256), 256, 0, ctx->stream>>>(
            static_cast<const __half *>(table_dev), static_cast<const int *>(ids->ptr), d, m,
            static_cast<__half *>(y_dev));
    else
        embedding_scalar_kernel<<<blocks_for((size_t)m * d, 256), 256, 0, ctx->stream>>>(
            static_cast<const __half *>(table_dev), static_cast<const int *>(ids->ptr), d, m,
            static_cast<__half *>(y_dev));
    ctx->launches++;
    e = cudaGetLastError();
    tlc_free(ids);  // stream-ordered: the gather above is already queued
    if (e != cudaSuccess) return tlc_fail(TLC_ERR_CUDA, "embedding launch failed: %s", cudaGetErrorString(e));
    return TLC_OK;
}

// ---- linear family -----------------------------------------------------------

static int32_t check_linear(tlc_ctx *ctx, tlc_qtensor *w, const void *x, int32_t m, int64_t x_cols,
                            const void *y) {
    TLC_REQUIRE(w && x && y, TLC_ERR_INVALID_OPERATION, "linear: null pointer");
    TLC_REQUIRE(m >= 1, TLC_ERR_INVALID_OPERATION, "matmul_transposed_b requires 2D tensors (m = %d)", m);
    // Same message shape as src/ops/matmul.rs:266-273.
    TLC_REQUIRE(x_cols == w->n_cols, TLC_ERR_INVALID_OPERATION,
                "matmul_transposed_b shape mismatch: [%d, %lld] @ [%lld, %lld].T", m, (long long)x_cols,
                (long long)w->n_rows, (long long)w->n_cols);
    TLC_REQUIRE(w->ctx->device == ctx->device, TLC_ERR_DEVICE,
                "matmul_transposed_b requires tensors on same device");
    return TLC_OK;
}

static const char *type_name(const tlc_qtensor *w) {
    return !w ? "?" : w->type == TLC_TYPE_Q4_0 ? "q4_0" : w->type == TLC_TYPE_Q8_0 ? "q8_0" : w->type == TLC_TYPE_Q6_K ? "q6_k" : "f16";
}

extern "C" int32_t tlc_linear(tlc_ctx *ctx, tlc_qtensor *w, const void *x_dev, int32_t m, int64_t x_cols,
                              void *y_dev, const void *bias_dev) {
    if (int32_t rc = tlc_enter(ctx)) return rc;
    if (int32_t rc = check_linear(ctx, w, x_dev, m, x_cols, y_dev)) return rc;
    tlc_perf_scope perf(ctx, "linear(%s, m=%d, n=%lld, k=%lld)", type_name(w), m, (long long)w->n_rows, (long long)w->n_cols);
    tlc_gemv_args a;
    a.n_out = 1;
    a.outs[0] = {w, y_dev, 0};
    a.x = x_dev;
    a.m = m;
    a.bias = bias_dev;
    return tlc_launch_gemv(ctx, a);
}

extern "C" int32_t tlc_linear_host(tlc_ctx *ctx, tlc_qtensor *w, const void *x_host, int32_t m,
                                   int64_t x_cols, void *y_host, const void *bias_host) {
    if (int32_t rc = tlc_enter(ctx)) return rc;
    if (int32_t rc = check_linear(ctx, w, x_host, m, x_cols, y_host)) return rc;
    const size_t xb = (size_t)m * x_cols * 2, yb = (size_t)m * w->n_rows * 2, bb = (size_t)w->n_rows * 2;
    tlc_buf *xd = nullptr, *yd = nullptr, *bd = nullptr;
    int32_t rc = tlc_alloc(ctx, xb, &xd);
    if (!rc) rc = tlc_alloc(ctx, yb, &yd);
    if (!rc && bias_host) rc = tlc_alloc(ctx, bb, &bd);
    if (!rc) rc = tlc_upload(ctx, xd->ptr, x_host, xb);
    if (!rc && bias_host) rc = tlc_upload(ctx, bd->ptr, bias_host, bb);
    if (!rc) rc = tlc_linear(ctx, w, xd->ptr, m, x_cols, yd->ptr, bd ? bd->ptr : nullptr);
    if (!rc) rc = tlc_download(ctx, y_host, yd->ptr, yb);
    tlc_free(xd);
    tlc_free(yd);
    tlc_free(bd);
    return rc;
}

extern "C" int32_t tlc_norm_linear_multi(tlc_ctx *ctx, int32_t n_weights, tlc_qtensor *const *w,
                                         void *const *y_dev, const int32_t *rope_heads, const void *x_dev,
                                         int32_t m, const void *norm_w_dev, float eps, int32_t pos_offset,
                                         uint32_t rope_base, const int32_t *positions_dev) {
    if (int32_t rc = tlc_enter(ctx)) return rc;
    TLC_REQUIRE(n_weights >= 1 && n_weights <= 3 && w && y_dev, TLC_ERR_INVALID_OPERATION,
                "norm_linear_multi: 1..3 weights expected, got %d", n_weights);
    tlc_gemv_args a;
    a.n_out = n_weights;
    for (int i = 0; i < n_weights; i++) {
        if (int32_t rc = check_linear(ctx, w[i], x_dev, m, w[0] ? w[0]->n_cols : 0, y_dev[i])) return rc;
        a.outs[i] = {w[i], y_dev[i], rope_heads ? rope_heads[i] : 0};
    }
    a.x = x_dev;
    a.m = m;
    a.norm_w = norm_w_dev;
    a.eps = eps;
    a.pos_offset = pos_offset;
    a.rope_base = rope_base;
    a.positions = positions_dev;
    tlc_perf_scope perf(ctx, "norm_linear_multi(%s, %d weights, m=%d, k=%lld)", type_name(w[0]), n_weights, m,
                        (long long)w[0]->n_cols);
    return tlc_launch_gemv(ctx, a);
}

extern "C" int32_t tlc_swiglu_gate_up(tlc_ctx *ctx, tlc_qtensor *w_gate, tlc_qtensor *w_up, const void *x_dev,
                                      int32_t m, const void *norm_w_dev, float eps, void *act_dev) {
    if (int32_t rc = tlc_enter(ctx)) return rc;
    if (int32_t rc = check_linear(ctx, w_gate, x_dev, m, w_gate ? w_gate->n_cols : 0, act_dev)) return rc;
    if (int32_t rc = check_linear(ctx, w_up, x_dev, m, w_gate->n_cols, act_dev)) return rc;
    tlc_gemv_args a;
    a.n_out = 2;
    a.outs[0] = {w_gate, act_dev, 0};
    a.outs[1] = {w_up, act_dev, 0};
    a.x = x_dev;
    a.m = m;
    a.norm_w = norm_w_dev;
    a.eps = eps;
    a.epilogue = TLC_EPI_SWIGLU;
    tlc_perf_scope perf(ctx, "swiglu_gate_up(%s, m=%d, n=%lld, k=%lld)", type_name(w_gate), m, (long long)w_gate->n_rows,
                        (long long)w_gate->n_cols);
    return tlc_launch_gemv(ctx, a);
}

extern "C" int32_t tlc_linear_residual(tlc_ctx *ctx, tlc_qtensor *w, const void *x_dev, int32_t m,
                                       const void *residual_dev, void *y_dev) {
    if (int32_t rc = tlc_enter(ctx)) return rc;
    if (int32_t rc = check_linear(ctx, w, x_dev, m, w ? w->n_cols : 0, y_dev)) return rc;
    TLC_REQUIRE(residual_dev, TLC_ERR_INVALID_OPERATION, "linear_residual: null residual");
    tlc_gemv_args a;
    a.n_out = 1;
    a.outs[0] = {w, y_dev, 0};
    a.x = x_dev;
    a.m = m;
    a.epilogue = TLC_EPI_RESIDUAL;
    a.residual = residual_dev;
    tlc_perf_scope perf(ctx, "linear_residual(%s, m=%d, n=%lld, k=%lld)", type_name(w), m, (long long)w->n_rows,
                        (long long)w->n_cols);
    return tlc_launch_gemv(ctx, a);
}
