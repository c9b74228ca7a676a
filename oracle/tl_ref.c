/*
 * tl_ref.c -- CPU oracle for the quantized-LLM hot path.
 *
 * TEST INFRASTRUCTURE ONLY.  This file restates, in plain C, the arithmetic of
 * the reference's Rust/Metal implementation so that the CUDA library can be
 * checked against it.  Nothing in the shipped library links, loads or calls it;
 * only the test-suite, the smoke check and the benchmark's CPU-baseline leg do.
 *
 * Every function cites the reference source (path within the TensorLogic
 * project) whose behaviour it follows.
 *
 * Parity pins: the dequantizers and the f16 conversion are pinned against the
 * reference's own known-answer tests (src/model/formats/gguf.rs:622-718), the
 * reference's Python dequantizer (scripts/reference_with_gguf.py:12-55) and
 * the `gguf` Python package; rms_norm / matmul are pinned against
 * src/ops/normalization.rs:736-957 and src/ops/matmul.rs:466-576; rope and
 * attention against scripts/reference_impl.py.  Rounding of inexact f16
 * products inside the `half` crate (v2.7.1, not vendored upstream) is not
 * pinned by any upstream vector; IEEE-754 round-to-nearest-even is assumed.
 *
 * All tensors are row-major.  f16 values travel as uint16_t bit patterns.
 */
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define TLREF_API __attribute__((visibility("default")))

/* ------------------------------------------------------------------------- */
/* f16 <-> f32.  Software conversion, round-to-nearest-even, subnormals kept. */
/* Matches half::f16::from_f32 / to_f32 (half crate 2.7.1) used at            */
/* src/model/formats/gguf.rs:46,100,106 and src/ops/matmul.rs:218-222.        */
/* ------------------------------------------------------------------------- */

static inline float h2f_sw(uint16_t h) {
    uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1Fu;
    uint32_t man = h & 0x3FFu;
    uint32_t bits;
    if (exp == 0) {
        if (man == 0) {
            bits = sign;
        } else { /* subnormal: normalise */
            int e = -1;
            do { man <<= 1; e++; } while (!(man & 0x400u));
            man &= 0x3FFu;
            bits = sign | ((uint32_t)(127 - 15 - e) << 23) | (man << 13);
        }
    } else if (exp == 31) {
        bits = sign | 0x7F800000u | (man << 13);
    } else {
        bits = sign | ((exp + 127 - 15) << 23) | (man << 13);
    }
    float f;
    memcpy(&f, &bits, 4);
    return f;
}

static inline uint16_t f2h_sw(float f) {
    uint32_t x;
    memcpy(&x, &f, 4);
    uint16_t sign = (uint16_t)((x >> 16) & 0x8000u);
    uint32_t absx = x & 0x7FFFFFFFu;
    if (absx >= 0x7F800000u) { /* inf / nan */
        if (absx > 0x7F800000u) return (uint16_t)(sign | 0x7E00u | ((absx >> 13) & 0x3FFu));
        return (uint16_t)(sign | 0x7C00u);
    }
    if (absx >= 0x477FF000u) { /* >= 65520 rounds to inf */
        return (uint16_t)(sign | 0x7C00u);
    }
    if (absx < 0x33000001u) { /* < 2^-25 (or exactly 2^-25: ties to even -> 0) */
        return sign;
    }
    int32_t e = (int32_t)(absx >> 23) - 127;
    uint32_t m = (absx & 0x7FFFFFu) | 0x800000u;
    uint32_t shift, hexp;
    if (e < -14) { /* subnormal result */
        shift = (uint32_t)(13 + (-14 - e));
        hexp = 0;
    } else {
        shift = 13;
        hexp = (uint32_t)(e + 15);
    }
    uint32_t q = m >> shift;
    uint32_t rem = m & ((1u << shift) - 1u);
    uint32_t half = 1u << (shift - 1);
    if (rem > half || (rem == half && (q & 1u))) q++;
    /* q holds the implicit bit for normals; adding hexp-1 lets a mantissa
       carry propagate into the exponent field. */
    uint32_t h = (hexp == 0) ? q : (((hexp - 1) << 10) + q);
    return (uint16_t)(sign | h);
}

TLREF_API float tlref_f16_to_f32(uint16_t h) { return h2f_sw(h); }
TLREF_API uint16_t tlref_f32_to_f16(float f) { return f2h_sw(f); }

/* Bulk helpers used by the tests to pin the conversion against numpy. */
TLREF_API void tlref_f16_to_f32_n(const uint16_t *h, float *f, size_t n) {
    for (size_t i = 0; i < n; i++) f[i] = h2f_sw(h[i]);
}
TLREF_API void tlref_f32_to_f16_n(const float *f, uint16_t *h, size_t n) {
    for (size_t i = 0; i < n; i++) h[i] = f2h_sw(f[i]);
}

#define h2f h2f_sw
#define f2h f2h_sw

/* ------------------------------------------------------------------------- */
/* GGUF block dequantizers (bit-exact targets).                               */
/* ------------------------------------------------------------------------- */

/* Q4_0: follows GGUFLoader::dequantize_q4_0, src/model/formats/gguf.rs:68-112
 * (same arithmetic as src/model/formats/mmap_gguf.rs:383-414).  18-byte block:
 * f16 scale, then 16 bytes; low nibble of byte j -> element j, high nibble ->
 * element j+16 ("grouped" layout); value = f16_rne((nibble-8) * f32(scale)).
 * Stops at the first block that does not fit in `nbytes`; the rest stays 0. */
TLREF_API void tlref_dequant_q4_0(const uint8_t *data, size_t nbytes, size_t n_elem,
                                  uint16_t *out) {
    const size_t BS = 32, BB = 18;
    size_t nblocks = (n_elem + BS - 1) / BS;
    memset(out, 0, n_elem * sizeof(uint16_t));
    for (size_t b = 0; b < nblocks; b++) {
        size_t off = b * BB;
        if (off + BB > nbytes) break;
        uint16_t dbits = (uint16_t)(data[off] | ((uint16_t)data[off + 1] << 8));
        float d = h2f(dbits);
        size_t base = b * BS;
        for (size_t j = 0; j < 16; j++) {
            if (base + j >= n_elem) break;
            uint8_t byte = data[off + 2 + j];
            float x0 = (float)((int)(byte & 0x0F) - 8);
            out[base + j] = f2h(x0 * d);
            if (base + j + 16 < n_elem) {
                float x1 = (float)((int)(byte >> 4) - 8);
                out[base + j + 16] = f2h(x1 * d);
            }
        }
    }
}

/* Q8_0: follows GGUFLoader::dequantize_q8_0, src/model/formats/gguf.rs:22-53
 * (= mmap_gguf.rs:417-439).  34-byte block: f16 scale + 32 int8;
 * value = f16(q) * scale as an f16 multiply = f16_rne(float(q) * float(scale))
 * (the f32 product of two f16 values is exact, so one rounding).
 * Returns the number of elements produced (the reference truncates its Vec). */
TLREF_API size_t tlref_dequant_q8_0(const uint8_t *data, size_t nbytes, size_t n_elem,
                                    uint16_t *out) {
    const size_t BS = 32, BB = 34;
    size_t nblocks = (n_elem + BS - 1) / BS;
    size_t produced = 0;
    for (size_t b = 0; b < nblocks; b++) {
        size_t off = b * BB;
        if (off + BB > nbytes) break;
        uint16_t dbits = (uint16_t)(data[off] | ((uint16_t)data[off + 1] << 8));
        float d = h2f(dbits);
        for (size_t i = 0; i < BS; i++) {
            if (produced >= n_elem) break;
            int8_t q = (int8_t)data[off + 2 + i];
            uint16_t qh = f2h((float)q); /* exact */
            out[produced++] = f2h(h2f(qh) * d);
        }
    }
    for (size_t i = produced; i < n_elem; i++) out[i] = 0;
    return produced;
}

/* Q6_K: follows GGUFLoader::dequantize_q6_k, src/model/formats/gguf.rs:128-218
 * (the llama.cpp element order; NOT gguf_weight_cache.rs:340-415, which differs).
 * 210-byte super-block of 256 values: ql[128] low nibbles, qh[64] two high bits,
 * sc[16] int8 scales, d f16.  Per half of 128 values and l in 0..31:
 *   q1 = (ql[l] & 15)    | ((qh[l] >> 0) & 3) << 4   -> y[l],      scale sc[l/16 + 0]
 *   q2 = (ql[l+32] & 15) | ((qh[l] >> 2) & 3) << 4   -> y[l + 32], scale sc[l/16 + 2]
 *   q3 = (ql[l] >> 4)    | ((qh[l] >> 4) & 3) << 4   -> y[l + 64], scale sc[l/16 + 4]
 *   q4 = (ql[l+32] >> 4) | ((qh[l] >> 6) & 3) << 4   -> y[l + 96], scale sc[l/16 + 6]
 * value = f16_rne((d * sc) * (q - 32)) in f32 (both products are exact: 11 + 7 + 6 bits). */
TLREF_API size_t tlref_dequant_q6_k(const uint8_t *data, size_t nbytes, size_t n_elem,
                                    uint16_t *out) {
    const size_t QK = 256, BB = 210;
    size_t nblocks = (n_elem + QK - 1) / QK;
    for (size_t i = 0; i < n_elem; i++) out[i] = 0;
    size_t produced = 0;
    for (size_t b = 0; b < nblocks; b++) {
        size_t off = b * BB;
        if (off + BB > nbytes) break;
        const uint8_t *ql = data + off, *qh = data + off + 128;
        const int8_t *sc = (const int8_t *)(data + off + 192);
        float d = h2f((uint16_t)(data[off + 208] | ((uint16_t)data[off + 209] << 8)));
        for (size_t n = 0; n < QK; n += 128) {
            for (size_t l = 0; l < 32; l++) {
                size_t base = b * QK + n + l;
                size_t is = l / 16;
                int q[4];
                q[0] = (int)((ql[l] & 0xF) | (((qh[l] >> 0) & 3) << 4)) - 32;
                q[1] = (int)((ql[l + 32] & 0xF) | (((qh[l] >> 2) & 3) << 4)) - 32;
                q[2] = (int)((ql[l] >> 4) | (((qh[l] >> 4) & 3) << 4)) - 32;
                q[3] = (int)((ql[l + 32] >> 4) | (((qh[l] >> 6) & 3) << 4)) - 32;
                for (int j = 0; j < 4; j++) {
                    size_t idx = base + 32 * (size_t)j;
                    if (idx < n_elem) {
                        float v = d * (float)sc[is + 2 * (size_t)j];
                        out[idx] = f2h(v * (float)q[j]);
                        if (idx + 1 > produced) produced = idx + 1;
                    }
                }
            }
            ql += 64;
            qh += 32;
            sc += 8;
        }
    }
    return produced;
}

/* ------------------------------------------------------------------------- */
/* Matmul / linear.                                                           */
/* ------------------------------------------------------------------------- */

/* The same loop with the CPU's F16C conversion instructions, which the `half`
 * crate also uses on x86-64 when the CPU has them (runtime detection); results
 * are bit-identical to the software conversions above (the tests check). */
#if defined(__x86_64__)
#include <immintrin.h>
__attribute__((target("f16c"))) static void matmul_f16acc_f16c(const uint16_t *a, const uint16_t *b,
                                                                uint16_t *c, int m, int k, int n) {
    for (int i = 0; i < m; i++) {
        for (int j = 0; j < n; j++) {
            uint16_t sum = 0;
            for (int p = 0; p < k; p++) {
                float fa = _cvtsh_ss(a[(size_t)i * k + p]), fb = _cvtsh_ss(b[(size_t)p * n + j]);
                uint16_t prod = _cvtss_sh(fa * fb, _MM_FROUND_TO_NEAREST_INT);
                sum = _cvtss_sh(_cvtsh_ss(sum) + _cvtsh_ss(prod), _MM_FROUND_TO_NEAREST_INT);
            }
            c[(size_t)i * n + j] = sum;
        }
    }
}
static int have_f16c(void) { return __builtin_cpu_supports("f16c"); }
#else
static int have_f16c(void) { return 0; }
#endif

static int g_allow_f16c = 1;
/* Tests switch the hardware path off to compare it with the software one. */
TLREF_API void tlref_set_f16c(int enable) { g_allow_f16c = enable; }
TLREF_API int tlref_uses_f16c(void) { return g_allow_f16c && have_f16c(); }

/* Literal CPU matmul: follows Tensor::matmul_cpu, src/ops/matmul.rs:201-228.
 * C[m,n] = A[m,k] * B[k,n]; the running sum is an f16: every step rounds the
 * product to f16, then the sum to f16.  Single thread, as upstream. */
TLREF_API void tlref_matmul_f16acc(const uint16_t *a, const uint16_t *b, uint16_t *c,
                                   int m, int k, int n) {
#if defined(__x86_64__)
    if (g_allow_f16c && have_f16c()) {
        matmul_f16acc_f16c(a, b, c, m, k, n);
        return;
    }
#endif
    for (int i = 0; i < m; i++) {
        for (int j = 0; j < n; j++) {
            uint16_t sum = 0;
            for (int p = 0; p < k; p++) {
                uint16_t prod = f2h(h2f(a[(size_t)i * k + p]) * h2f(b[(size_t)p * n + j]));
                sum = f2h(h2f(sum) + h2f(prod));
            }
            c[(size_t)i * n + j] = sum;
        }
    }
}

/* Literal CPU linear: the CPU arm of Tensor::matmul_transposed_b,
 * src/ops/matmul.rs:293-297: materialise W^T ([K,N]) and call matmul_cpu.
 * `scratch` must hold k*n f16 values. */
TLREF_API void tlref_linear_literal(const uint16_t *x, const uint16_t *w, uint16_t *y,
                                    int m, int k, int n, uint16_t *scratch) {
    for (int i = 0; i < n; i++)
        for (int j = 0; j < k; j++) scratch[(size_t)j * n + i] = w[(size_t)i * k + j];
    tlref_matmul_f16acc(x, scratch, y, m, k, n);
}

/* Parity target for linear: f16 inputs, f32 accumulation over K in index
 * order, one round-to-nearest-even to f16 -- the arithmetic of the Metal
 * kernels matmul_transposed_b_tiled_f16, shaders/unified.metal:4226-4288
 * (f32 `sum`, `half(sum)` on store).  y[m,n] = x[m,k] * W[n,k]^T.
 * Threads over output rows of W; `threads` <= 0 means all available. */
TLREF_API void tlref_linear_f32acc(const uint16_t *x, const uint16_t *w, uint16_t *y, int m,
                                   int k, int n, int threads) {
    float *xf = (float *)malloc((size_t)m * k * sizeof(float));
    for (size_t i = 0; i < (size_t)m * k; i++) xf[i] = h2f(x[i]);
#ifdef _OPENMP
    if (threads <= 0) threads = omp_get_max_threads();
#pragma omp parallel num_threads(threads)
#endif
    {
        float *wf = (float *)malloc((size_t)k * sizeof(float));
#ifdef _OPENMP
#pragma omp for schedule(static)
#endif
        for (int j = 0; j < n; j++) {
            for (int p = 0; p < k; p++) wf[p] = h2f(w[(size_t)j * k + p]);
            for (int i = 0; i < m; i++) {
                const float *xr = xf + (size_t)i * k;
                float sum = 0.0f;
                for (int p = 0; p < k; p++) sum += xr[p] * wf[p];
                y[(size_t)i * n + j] = f2h(sum);
            }
        }
        free(wf);
    }
    free(xf);
}

/* Same parity target, taking the weight as native GGUF blocks: each row is
 * dequantized with the bit-exact dequantizer above (so the f16 weight values
 * are exactly the reference loader's) and contracted with f32 accumulation.
 * qtype: 2 = Q4_0, 8 = Q8_0, 14 = Q6_K (GGUF type ids, mmap_gguf.rs:30-45), 1 = F16. */
TLREF_API int tlref_linear_q_f32acc(int qtype, const uint8_t *wq, const uint16_t *x,
                                    uint16_t *y, int m, int k, int n, int threads) {
    if (k % 32 != 0 && qtype != 1) return -1;
    size_t row_bytes = qtype == 2 ? (size_t)(k / 32) * 18
                     : qtype == 8 ? (size_t)(k / 32) * 34
                     : qtype == 14 ? (k % 256 == 0 ? (size_t)(k / 256) * 210 : 0)
                     : qtype == 1 ? (size_t)k * 2 : 0;
    if (!row_bytes) return -2;
    float *xf = (float *)malloc((size_t)m * k * sizeof(float));
    for (size_t i = 0; i < (size_t)m * k; i++) xf[i] = h2f(x[i]);
    /* rows in groups of eight, transposed to [group][p][8] for the blocked loop below */
    float *xt = m >= 8 ? (float *)malloc((size_t)(m / 8) * k * 8 * sizeof(float)) : NULL;
    if (xt)
        for (int gI = 0; gI < m / 8; gI++)
            for (int p = 0; p < k; p++)
                for (int v = 0; v < 8; v++) xt[((size_t)gI * k + p) * 8 + v] = xf[(size_t)(gI * 8 + v) * k + p];
#ifdef _OPENMP
    if (threads <= 0) threads = omp_get_max_threads();
#pragma omp parallel num_threads(threads)
#endif
    {
        uint16_t *wh = (uint16_t *)malloc((size_t)k * sizeof(uint16_t));
        float *wf = (float *)malloc((size_t)k * sizeof(float));
#ifdef _OPENMP
#pragma omp for schedule(static)
#endif
        for (int j = 0; j < n; j++) {
            const uint8_t *row = wq + (size_t)j * row_bytes;
            if (qtype == 2) tlref_dequant_q4_0(row, row_bytes, (size_t)k, wh);
            else if (qtype == 8) tlref_dequant_q8_0(row, row_bytes, (size_t)k, wh);
            else if (qtype == 14) tlref_dequant_q6_k(row, row_bytes, (size_t)k, wh);
            else memcpy(wh, row, row_bytes);
            for (int p = 0; p < k; p++) wf[p] = h2f(wh[p]);
            int i = 0;
            /* Eight activation rows at a time, one SIMD lane each: every output is still
             * its own f32 sum over p in index order (separate multiply and add, no
             * contraction), so the bits are those of the plain loop below -- only the
             * eight sums advance together instead of one after the other. */
            for (; xt && i + 8 <= m; i += 8) {
                const float *xb = xt + (size_t)(i / 8) * k * 8;
                float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
                for (int p = 0; p < k; p++) {
                    const float wv = wf[p];
#pragma omp simd
                    for (int v = 0; v < 8; v++) acc[v] += xb[(size_t)p * 8 + v] * wv;
                }
                for (int v = 0; v < 8; v++) y[(size_t)(i + v) * n + j] = f2h(acc[v]);
            }
            for (; i < m; i++) {
                const float *xr = xf + (size_t)i * k;
                float sum = 0.0f;
                for (int p = 0; p < k; p++) sum += xr[p] * wf[p];
                y[(size_t)i * n + j] = f2h(sum);
            }
        }
        free(wh);
        free(wf);
    }
    free(xf);
    free(xt);
    return 0;
}

/* ------------------------------------------------------------------------- */
/* Per-token ops.                                                             */
/* ------------------------------------------------------------------------- */

/* RMSNorm: follows Tensor::rms_norm_cpu, src/ops/normalization.rs:199-248.
 * f32 sum of squares in index order, inv = 1/sqrt(mean+eps) with an f32 eps,
 * y = f16((x*inv)*w).  (The Metal path passes eps through an f16 buffer,
 * normalization.rs:133-137; the CPU path restated here does not.) */
TLREF_API void tlref_rms_norm(const uint16_t *x, const uint16_t *w, uint16_t *y, int rows,
                              int d, float eps) {
    for (int r = 0; r < rows; r++) {
        const uint16_t *xr = x + (size_t)r * d;
        float sq = 0.0f;
        for (int i = 0; i < d; i++) {
            float v = h2f(xr[i]);
            sq += v * v;
        }
        float mean_sq = sq / (float)d;
        float rms = sqrtf(mean_sq + eps);
        float inv = 1.0f / rms;
        for (int i = 0; i < d; i++) {
            float nrm = h2f(xr[i]) * inv;
            y[(size_t)r * d + i] = f2h(nrm * h2f(w[i]));
        }
    }
}

/* RoPE: restates kernel rope_f16, shaders/unified.metal:2355-2417 (there is
 * no CPU implementation upstream).  Input [seq, heads, d]; interleaved pairs
 * (2i, 2i+1); freq = 1/pow(base, 2i/d) with base a float made from an
 * unsigned integer (src/ops/rope.rs:244-245); theta = float(pos)*freq; f32
 * trig; RNE to f16.  `positions` (nullable) overrides pos = s + pos_offset
 * per sequence row, which is what a batched decode step needs. */
TLREF_API void tlref_rope(const uint16_t *x, uint16_t *y, int seq, int heads, int d,
                          int pos_offset, unsigned base, const int32_t *positions) {
    float fbase = (float)base;
    for (int s = 0; s < seq; s++) {
        unsigned pos = positions ? (unsigned)positions[s] : (unsigned)(s + pos_offset);
        for (int h = 0; h < heads; h++) {
            size_t o = ((size_t)s * heads + h) * d;
            for (int p = 0; p < d / 2; p++) {
                float exponent = (float)(2 * p) / (float)d;
                float freq = 1.0f / powf(fbase, exponent);
                float theta = (float)pos * freq;
                float c = cosf(theta), sn = sinf(theta);
                float x0 = h2f(x[o + 2 * p]), x1 = h2f(x[o + 2 * p + 1]);
                y[o + 2 * p] = f2h(x0 * c - x1 * sn);
                y[o + 2 * p + 1] = f2h(x0 * sn + x1 * c);
            }
        }
    }
}

/* RoPE from precomputed tables: restates kernel rope_candle_f16,
 * shaders/unified.metal:5122-5184 (dispatched by Tensor::rope_candle,
 * src/ops/rope.rs:18-65, :121-212).  Pair p of position s reads
 * table[s * pitch + p]; the shader's own arithmetic is pitch = head_dim
 * (`seq_idx * head_dim + dim_pair_idx`), a table with one column per pair is
 * pitch = head_dim / 2.  f32 products, f32 difference / sum, RNE to f16. */
TLREF_API void tlref_rope_table(const uint16_t *x, const uint16_t *cos_t, const uint16_t *sin_t, uint16_t *y,
                                int seq, int heads, int d, int pitch) {
    for (int s = 0; s < seq; s++)
        for (int h = 0; h < heads; h++) {
            size_t o = ((size_t)s * heads + h) * d;
            for (int p = 0; p < d / 2; p++) {
                float c = h2f(cos_t[(size_t)s * pitch + p]), sn = h2f(sin_t[(size_t)s * pitch + p]);
                float x0 = h2f(x[o + 2 * p]), x1 = h2f(x[o + 2 * p + 1]);
                y[o + 2 * p] = f2h(x0 * c - x1 * sn);
                y[o + 2 * p + 1] = f2h(x0 * sn + x1 * c);
            }
        }
}

/* sigmoid: follows Tensor::sigmoid_cpu, src/ops/activations.rs:252-266:
 * 1/(1+exp(-x)) in f32, RNE to f16. */
TLREF_API void tlref_sigmoid(const uint16_t *x, uint16_t *y, size_t n) {
    for (size_t i = 0; i < n; i++) {
        float v = h2f(x[i]);
        y[i] = f2h(1.0f / (1.0f + expf(-v)));
    }
}

/* mul / add: follow the CPU arms of Tensor::mul / Tensor::add,
 * src/ops/elementwise.rs:309-330 and :122-140: an f16 op = f32 op + RNE. */
TLREF_API void tlref_mul(const uint16_t *a, const uint16_t *b, uint16_t *y, size_t n) {
    for (size_t i = 0; i < n; i++) y[i] = f2h(h2f(a[i]) * h2f(b[i]));
}
TLREF_API void tlref_add(const uint16_t *a, const uint16_t *b, uint16_t *y, size_t n) {
    for (size_t i = 0; i < n; i++) y[i] = f2h(h2f(a[i]) + h2f(b[i]));
}

/* SiLU(gate)*up exactly as the TL scripts compose it
 * (debug/chat_demo_with_kvcache.tl:26-41): s = sigmoid(g); a = g*s; y = a*u;
 * three f16 roundings in sequence. */
TLREF_API void tlref_swiglu(const uint16_t *gate, const uint16_t *up, uint16_t *y, size_t n) {
    for (size_t i = 0; i < n; i++) {
        float g = h2f(gate[i]);
        uint16_t s = f2h(1.0f / (1.0f + expf(-g)));
        uint16_t a = f2h(g * h2f(s));
        y[i] = f2h(h2f(a) * h2f(up[i]));
    }
}

/* softmax over the last dim: restates softmax_simple_f16,
 * shaders/unified.metal:2150-2200 (no CPU path upstream,
 * src/ops/activations.rs:232-236).  f32 max and sum over finite inputs,
 * non-finite -> 0, degenerate row -> uniform.  With round_exp != 0 the
 * exponentials are rounded to f16 before the divide, as the shader does by
 * storing them into the f16 output first; the sum still uses the f32 values. */
TLREF_API void tlref_softmax(const uint16_t *x, uint16_t *y, int rows, int last,
                             int round_exp) {
    for (int r = 0; r < rows; r++) {
        const uint16_t *xr = x + (size_t)r * last;
        uint16_t *yr = y + (size_t)r * last;
        float mx = -INFINITY;
        for (int i = 0; i < last; i++) {
            float v = h2f(xr[i]);
            if (isfinite(v)) mx = fmaxf(mx, v);
        }
        if (!isfinite(mx)) mx = 0.0f;
        float sum = 0.0f;
        float *e = (float *)malloc((size_t)last * sizeof(float));
        for (int i = 0; i < last; i++) {
            float v = h2f(xr[i]);
            float ev = isfinite(v) ? expf(v - mx) : 0.0f;
            e[i] = round_exp ? h2f(f2h(ev)) : ev;
            sum += ev;
        }
        if (sum > 0.0f && isfinite(sum)) {
            for (int i = 0; i < last; i++) yr[i] = f2h(e[i] / sum);
        } else {
            float u = 1.0f / (float)last;
            for (int i = 0; i < last; i++) yr[i] = f2h(u);
        }
        free(e);
    }
}

/* embedding: row gather, restates embedding_lookup_f16,
 * shaders/unified.metal:658-675; ids are bounds-checked on the host upstream
 * (src/interpreter/builtin_nn.rs:681-688) -- returns -1 on a bad id. */
TLREF_API int tlref_embedding(const uint16_t *table, int vocab, int d, const int32_t *ids,
                              int m, uint16_t *y) {
    for (int i = 0; i < m; i++) {
        if (ids[i] < 0 || ids[i] >= vocab) return -1;
        memcpy(y + (size_t)i * d, table + (size_t)ids[i] * d, (size_t)d * 2);
    }
    return 0;
}

/* Grouped-query attention as the TL scripts build it from builtins
 * (debug/chat_demo_with_kvcache.tl:44-88 prefill, :247-282 decode):
 *   scores[i,h,j] = sum_d q[i,h,d]*k[j,h/g,d]       f32 acc -> f16
 *                    (einsum_ihd_jhd_ihj_f16, shaders/unified.metal:2524-2563)
 *   scores *= scale                                  f16 multiply
 *   masked (j > q_pos0+i) -> -10000                  (unified.metal:4474-4488)
 *   softmax over j                                   (unified.metal:2150-2200)
 *   out[i,h,d] = sum_j p[i,h,j]*v[j,h/g,d]           (unified.metal:2646-2683)
 * KV head for query head h is h / (H/Hkv): each KV head repeated consecutively
 * (reshape -> broadcast_to -> reshape in the script).
 * flags bit0: round exp to f16 inside softmax (shader behaviour).
 * flags bit1: accumulate P.V in f16 (shader behaviour); otherwise f32 with one
 *             rounding, which is the documented parity target.
 * q: [I,H,D], k/v: [J,Hkv,D], out: [I,H,D]. */
TLREF_API void tlref_attention(const uint16_t *q, const uint16_t *k, const uint16_t *v,
                               uint16_t *out, int I, int J, int H, int Hkv, int D,
                               float scale, int q_pos0, int flags) {
    int g = H / Hkv;
    uint16_t hscale = f2h(scale);
#ifdef _OPENMP
#pragma omp parallel for collapse(2) schedule(static)
#endif
    for (int i = 0; i < I; i++) {
        for (int h = 0; h < H; h++) {
            uint16_t *sc = (uint16_t *)malloc((size_t)J * 2);
            uint16_t *pr = (uint16_t *)malloc((size_t)J * 2);
            int kvh = h / g;
            const uint16_t *qr = q + ((size_t)i * H + h) * D;
            for (int j = 0; j < J; j++) {
                const uint16_t *kr = k + ((size_t)j * Hkv + kvh) * D;
                float s = 0.0f;
                for (int d = 0; d < D; d++) s += h2f(qr[d]) * h2f(kr[d]);
                uint16_t sh = f2h(s);
                sh = f2h(h2f(sh) * h2f(hscale));
                if (j > q_pos0 + i) sh = f2h(-10000.0f);
                sc[j] = sh;
            }
            tlref_softmax(sc, pr, 1, J, flags & 1);
            for (int d = 0; d < D; d++) {
                if (flags & 2) {
                    uint16_t acc = 0;
                    for (int j = 0; j < J; j++) {
                        uint16_t pv = f2h(h2f(pr[j]) * h2f(v[((size_t)j * Hkv + kvh) * D + d]));
                        acc = f2h(h2f(acc) + h2f(pv));
                    }
                    out[((size_t)i * H + h) * D + d] = acc;
                } else {
                    float acc = 0.0f;
                    for (int j = 0; j < J; j++)
                        acc += h2f(pr[j]) * h2f(v[((size_t)j * Hkv + kvh) * D + d]);
                    out[((size_t)i * H + h) * D + d] = f2h(acc);
                }
            }
            free(sc);
            free(pr);
        }
    }
}

/* Greedy sample: follows temperature_sample's greedy arm,
 * src/interpreter/builtin_sampling.rs:176-181: logits widened to f32, then
 * Iterator::max_by, which returns the LAST maximal element on ties. */
TLREF_API int tlref_argmax_last(const uint16_t *logits, int n) {
    int best = 0;
    float bv = h2f(logits[0]);
    for (int i = 1; i < n; i++) {
        float v = h2f(logits[i]);
        if (!(v < bv)) { /* v >= bv, or unordered -> treated as Equal upstream */
            best = i;
            bv = v;
        }
    }
    return best;
}

/* Temperature sample: follows temperature_sample_cpu,
 * src/interpreter/builtin_sampling.rs:131-220, with the uniform draw passed in
 * (upstream: rand::thread_rng().gen::<f32>()).  Logits widened to f32; T <= 1e-4
 * is the greedy arm; otherwise scaled = x / T, softmax with the maximum
 * subtracted (f32, sums in index order), probabilities divided by the sum, then
 * the first index whose running sum exceeds u; the last index if none does.
 * cdf_out (optional, n floats) receives the running sums. */
TLREF_API int tlref_temperature_sample(const uint16_t *logits, int n, float temperature, float u,
                                       float *cdf_out) {
    if (temperature <= 0.0001f) return tlref_argmax_last(logits, n);
    float *p = (float *)malloc((size_t)n * sizeof(float));
    float mx = -INFINITY;
    for (int i = 0; i < n; i++) {
        p[i] = h2f(logits[i]) / temperature;
        if (p[i] > mx) mx = p[i];  /* f32::max fold */
    }
    float sum = 0.0f;
    for (int i = 0; i < n; i++) {
        p[i] = expf(p[i] - mx);
        sum += p[i];
    }
    int idx = n - 1;
    int found = 0;
    float cum = 0.0f;
    for (int i = 0; i < n; i++) {
        cum += p[i] / sum;
        if (cdf_out) cdf_out[i] = cum;
        if (!found && u < cum) {
            idx = i;
            found = 1;
            if (!cdf_out) break;
        }
    }
    free(p);
    return idx;
}

TLREF_API int tlref_num_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}
