// Fused dequant-GEMV for decode-sized activations (M <= 16) over weights kept
// in their native GGUF Q4_0 / Q8_0 block layout.
//
// Takes the place of the dense f16 kernels the reference runs after
// dequantizing at load time (matmul_transposed_b_tiled_f16,
// shaders/unified.metal:4226-4347, dispatched from src/ops/matmul.rs:314-458)
// and of the separate rms_norm / rope / sigmoid / mul / add launches around
// them in the TL scripts (debug/chat_demo_with_kvcache.tl:219-290).
//
// Design (memory-bound; the weight bytes are read from HBM exactly once):
//   * persistent CTAs, one per SM, each walking 16-row slabs of the weight(s);
//   * a producer warp streams the raw block bytes of a slab into a shared
//     memory ring with 16-byte-granular bulk async copies (one per row per
//     stage) that complete on mbarriers -- no thread ever issues a narrow
//     global load for weight data, and the ring keeps tens of KB per SM in
//     flight independent of occupancy;
//   * four consumer warps unpack nibbles / bytes in registers straight into
//     f16 tensor-core fragments: a 4-bit (8-bit) integer n placed in the low
//     mantissa bits of a binary16 is the subnormal n * 2^-24, so one AND per
//     pair of weights yields an exact A fragment; the -8 (-128) offset is
//     carried by the accumulator's initial value (-8 * sum of the 32
//     activations of the block) and the block scale d multiplies the 16x8 block
//     result in f32;  mma.sync m16n8k16 with f32 accumulation does the dot
//     products for up to 8 activation rows at no extra cost;
//   * the K range of a slab is split over the four warps, reduced through
//     shared memory, and the epilogue (f16 rounding, bias / residual add,
//     SiLU(gate)*up, interleaved RoPE) is applied before the single store.
// The activation vector(s) are optionally RMS-normalised on the way into
// shared memory, where they are kept pre-permuted in fragment order.
#include <cuda_fp16.h>

#include "tlc_internal.h"

namespace {

constexpr int kRows = 16;           // rows of W per slab (the M of m16n8k16)
constexpr int kConsumerWarps = 8;
constexpr int kConsumerThreads = kConsumerWarps * 32;
constexpr int kThreads = (kConsumerWarps + 1) * 32;
constexpr int kMaxStages = 8;
constexpr uint32_t kWaitLimit = 1u << 22;

template <int QT> struct QTraits;
template <> struct QTraits<TLC_TYPE_Q4_0> {
    static constexpr int BB = 18;        // bytes per block
    static constexpr int KCB = 64;       // blocks per ring stage and row (1152 B)
    static constexpr int PAIR_WORDS = 9; // 32-bit words per (even, odd) block pair
    static constexpr float OFFSET = 8.0f;
};
template <> struct QTraits<TLC_TYPE_Q8_0> {
    static constexpr int BB = 34;
    static constexpr int KCB = 32;       // 1088 B
    static constexpr int PAIR_WORDS = 17;
    static constexpr float OFFSET = 128.0f;
};

// Shared-memory distance between the rows of a stage: the smallest odd
// multiple of 16 bytes that holds a row segment, so that the 8 row groups of a
// warp-wide 32-bit load fall into 8 different bank quads.
__host__ __device__ constexpr int stage_pitch(int seg_bytes) {
    int units = (seg_bytes + 15) / 16;
    return (units | 1) * 16;
}

struct GemvTensor {
    const uint8_t *w;
    size_t pitch;
    int n;          // rows of W (outputs)
    __half *y;
    int rope_heads;
    int head_dim;
    long long row_stride;  // elements between the outputs of consecutive activation rows
    long long pos_stride;  // elements per position (0 unless the destination is a KV cache)
};

struct GemvParams {
    GemvTensor t[3];
    int n_out;
    int slabs[3];
    int total_units;
    int subs;        // slabs per unit (2 for the gate/up pair)
    int k;
    int nblk;        // k / 32
    int nblk_pad;    // rounded up to even
    int nchunks;     // ring stages per slab
    int m;
    const __half *x;
    const __half *norm_w;
    float eps;
    int epilogue;
    const __half *bias;
    const __half *residual;
    int pos_offset;
    float rope_base;
    const int *positions;
    int nstages;
    tlc_dev_status *status;
};

__device__ __forceinline__ uint32_t smem_u32(const void *p) {
    return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void mbar_init(uint64_t *bar, int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t *bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t *bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t *bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n"
        " .reg .pred p;\n"
        " mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        " selp.u32 %0, 1, 0, p;\n"
        "}\n"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait: gives up after kWaitLimit polls, records where, and raises the
// CTA's abort flag; once that flag is up every later wait only polls briefly
// (long enough for copies already in flight to land) so the kernel drains and
// returns instead of hanging.  The result is made warp-uniform by the callers.
__device__ __forceinline__ bool mbar_wait(uint64_t *bar, uint32_t parity, volatile int *abort_flag,
                                          tlc_dev_status *status, int where) {
    if (mbar_try_wait(bar, parity)) return true;
    const uint32_t limit = *abort_flag ? 4096u : kWaitLimit;
    for (uint32_t i = 0; i < limit; i++) {
        if (mbar_try_wait(bar, parity)) return true;
    }
    *abort_flag = 1;
    if (atomicCAS(&status->code, 0, 1) == 0) status->where = where;
    return false;
}
__device__ __forceinline__ void bulk_g2s(void *dst, const void *src, uint32_t bytes, uint64_t *bar) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
            smem_u32(dst)),
        "l"(src), "r"(bytes), "r"(smem_u32(bar))
        : "memory");
}
__device__ __forceinline__ void consumer_bar() {
    asm volatile("bar.sync 1, %0;" ::"n"(kConsumerThreads) : "memory");
}

__device__ __forceinline__ void mma16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1,
                                         const float (&c)[4]) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%10,%11,%12,%13};"
        : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1), "f"(c[0]), "f"(c[1]), "f"(c[2]),
          "f"(c[3]));
}

__device__ __forceinline__ float half_bits_to_float(uint32_t bits16) {
    return __half2float(__ushort_as_half((unsigned short)bits16));
}

// One block of 32 along K for 16 rows x (8*NT) activation rows.
//   wg / wg8  : this lane's qs word(s) of the block for rows g and g+8
//               (Q4_0: 1 word = word t of the 16 qs bytes;
//                Q8_0: 2 words = words 2t, 2t+1 of the 32 qs bytes)
//   dg / dg8  : block scales of the two rows
//   xp        : fragment-ordered activations of this block, per n-tile
//   cinit     : accumulator start (-OFFSET * 2^-24 * sum of the block's x)
template <int QT, int NT>
__device__ __forceinline__ void block_mma(const uint32_t *wg, const uint32_t *wg8, float dg, float dg8,
                                          const uint4 (&xp)[NT], const float2 (&cinit)[NT],
                                          float (&acc)[4 * NT]) {
    uint32_t a1[4], a2[4];
    if (QT == TLC_TYPE_Q4_0) {
        const uint32_t w0 = wg[0], w1 = wg8[0];
        // Every nibble is moved to the lowest mantissa bits, so all fragments
        // carry the same 2^-24 and the activations need no per-slot scaling
        // (scaling them down instead would push small activations into the
        // f16 subnormal range and lose bits).
        a1[0] = w0 & 0x000F000Fu;           // elems 4t, 4t+2
        a1[1] = w1 & 0x000F000Fu;
        a1[2] = (w0 >> 4) & 0x000F000Fu;    // elems 16+4t, 18+4t
        a1[3] = (w1 >> 4) & 0x000F000Fu;
        a2[0] = (w0 >> 8) & 0x000F000Fu;    // elems 4t+1, 4t+3
        a2[1] = (w1 >> 8) & 0x000F000Fu;
        a2[2] = (w0 >> 12) & 0x000F000Fu;   // elems 17+4t, 19+4t
        a2[3] = (w1 >> 12) & 0x000F000Fu;
    } else {
        const uint32_t u0 = wg[0] ^ 0x80808080u, v0 = wg8[0] ^ 0x80808080u;
        const uint32_t u1 = wg[1] ^ 0x80808080u, v1 = wg8[1] ^ 0x80808080u;
        a1[0] = __byte_perm(u0, 0, 0x4140);  // elems 8t, 8t+1   (q+128) x 2^-24
        a1[1] = __byte_perm(v0, 0, 0x4140);
        a1[2] = __byte_perm(u0, 0, 0x4342);  // elems 8t+2, 8t+3
        a1[3] = __byte_perm(v0, 0, 0x4342);
        a2[0] = __byte_perm(u1, 0, 0x4140);  // elems 8t+4, 8t+5
        a2[1] = __byte_perm(v1, 0, 0x4140);
        a2[2] = __byte_perm(u1, 0, 0x4342);  // elems 8t+6, 8t+7
        a2[3] = __byte_perm(v1, 0, 0x4342);
    }
#pragma unroll
    for (int nt = 0; nt < NT; nt++) {
        float c[4] = {cinit[nt].x, cinit[nt].y, cinit[nt].x, cinit[nt].y};
        float d1[4], d2[4];
        mma16816(d1, a1, xp[nt].x, xp[nt].y, c);
        mma16816(d2, a2, xp[nt].z, xp[nt].w, d1);
        acc[nt * 4 + 0] = fmaf(dg, d2[0], acc[nt * 4 + 0]);
        acc[nt * 4 + 1] = fmaf(dg, d2[1], acc[nt * 4 + 1]);
        acc[nt * 4 + 2] = fmaf(dg8, d2[2], acc[nt * 4 + 2]);
        acc[nt * 4 + 3] = fmaf(dg8, d2[3], acc[nt * 4 + 3]);
    }
}

// Loads the (even, odd) block pair `p` of one row segment from the ring and
// returns this lane's qs words and the two scales.  Pair p starts at word
// PAIR_WORDS*p of the (4-byte aligned) segment; the even block's qs bytes sit
// 2 bytes past a word boundary, hence the funnel shifts.
template <int QT>
__device__ __forceinline__ void load_pair(const uint32_t *seg, int p, int t, uint32_t (&we)[2],
                                          uint32_t (&wo)[2], float &de, float &dod) {
    constexpr int PW = QTraits<QT>::PAIR_WORDS;
    const uint32_t *q = seg + PW * p;
    if (QT == TLC_TYPE_Q4_0) {
        uint32_t lo = q[t], hi = q[t + 1];
        we[0] = __funnelshift_r(lo, hi, 16);
        wo[0] = q[5 + t];
        de = half_bits_to_float(q[0] & 0xFFFFu);
        dod = half_bits_to_float(q[4] >> 16);
    } else {
        uint32_t r0 = q[2 * t], r1 = q[2 * t + 1], r2 = q[2 * t + 2];
        we[0] = __funnelshift_r(r0, r1, 16);
        we[1] = __funnelshift_r(r1, r2, 16);
        wo[0] = q[9 + 2 * t];
        wo[1] = q[10 + 2 * t];
        de = half_bits_to_float(q[0] & 0xFFFFu);
        dod = half_bits_to_float(q[8] >> 16);
    }
}

template <int QT, int NT>
__global__ void __launch_bounds__(kThreads, 2) gemv_mma_kernel(const GemvParams p) {
    using T = QTraits<QT>;
    constexpr int MP = 8 * NT;  // padded activation rows
    constexpr int PITCH = stage_pitch(T::KCB * T::BB);
    constexpr int STAGE_BYTES = kRows * PITCH;

    extern __shared__ __align__(128) uint8_t smem[];
    uint64_t *full = reinterpret_cast<uint64_t *>(smem);
    uint64_t *empty = full + kMaxStages;
    volatile int *abort_flag = reinterpret_cast<volatile int *>(smem + 128);
    float *inv_rms = reinterpret_cast<float *>(smem + 192);                // 16 floats
    float *red = reinterpret_cast<float *>(smem + 256);                     // [2][4][16][MP]
    float *xs8 = red + 2 * kConsumerWarps * kRows * MP;                     // [nblk_pad][MP]
    uint4 *xperm = reinterpret_cast<uint4 *>(xs8 + (size_t)p.nblk_pad * MP);  // [nblk_pad][m][4]
    uint8_t *stages = reinterpret_cast<uint8_t *>(xperm + (size_t)p.nblk_pad * p.m * 4);
    stages = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(stages) + 127) & ~(uintptr_t)127);

    const int tid = threadIdx.x;
    const int warp = tid >> 5, lane = tid & 31;
    const int S = p.nstages;

    if (tid == 0) {
        for (int s = 0; s < S; s++) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], kConsumerWarps);
        }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    __syncthreads();

    if (warp == kConsumerWarps) {
        // ------------------------------ producer ------------------------------
        uint32_t it = 0;
        for (int unit = blockIdx.x; unit < p.total_units; unit += gridDim.x) {
            for (int sub = 0; sub < p.subs; sub++) {
                int ti, sl;
                if (p.subs == 2) {
                    ti = sub;
                    sl = unit;
                } else {
                    ti = 0;
                    sl = unit;
                    while (sl >= p.slabs[ti]) {
                        sl -= p.slabs[ti];
                        ti++;
                    }
                }
                const GemvTensor &gt = p.t[ti];
                const int rows_valid = min(kRows, gt.n - sl * kRows);
                for (int c = 0; c < p.nchunks; c++, it++) {
                    const int s = it % S;
                    const uint32_t par = ((it / S) & 1u) ^ 1u;
                    // On a timeout the producer stops issuing copies; the consumers'
                    // own bounded waits then end the CTA.
                    if (!__all_sync(0xffffffffu, mbar_wait(&empty[s], par, abort_flag, p.status, 1))) return;
                    const int kcb = min(T::KCB, p.nblk - c * T::KCB);
                    const uint32_t bytes_row = (uint32_t)((kcb * T::BB + 15) & ~15);
                    if (lane == 0) mbar_expect_tx(&full[s], bytes_row * (uint32_t)rows_valid);
                    __syncwarp();
                    if (lane < rows_valid) {
                        const uint8_t *src =
                            gt.w + (size_t)(sl * kRows + lane) * gt.pitch + (size_t)c * (T::KCB * T::BB);
                        bulk_g2s(stages + (size_t)s * STAGE_BYTES + lane * PITCH, src, bytes_row, &full[s]);
                    }
                }
            }
        }
        return;
    }

    // -------------------------------- consumers --------------------------------
    const int ctid = tid;  // 0..kConsumerThreads-1
    const bool do_norm = p.norm_w != nullptr;

    // (a) RMS statistics: warp w owns activation rows w, w+4, ...
    if (do_norm) {
        for (int m = warp; m < p.m; m += kConsumerWarps) {
            const __half *xr = p.x + (size_t)m * p.k;
            float sq = 0.f;
            for (int k = lane * 2; k < p.k; k += 64) {
                float2 v = __half22float2(*reinterpret_cast<const __half2 *>(xr + k));
                sq = fmaf(v.x, v.x, sq);
                sq = fmaf(v.y, v.y, sq);
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
            if (lane == 0) {
                float mean_sq = sq / (float)p.k;
                inv_rms[m] = 1.0f / sqrtf(mean_sq + p.eps);
            }
        }
    }
    for (int i = ctid; i < p.nblk_pad * MP; i += kConsumerThreads) xs8[i] = 0.f;
    consumer_bar();

    // (b) activations into fragment order + per-block sums.  Item = (block b,
    // activation row m, quad lane t); the 4 t-items of a (b, m) are adjacent
    // lanes, so a 2-step shuffle gives the block sum.
    {
        const int items = p.nblk_pad * p.m * 4;
        const int rounds = (items + kConsumerThreads - 1) / kConsumerThreads;
        for (int r = 0; r < rounds; r++) {
            const int idx = ctid + r * kConsumerThreads;
            const bool live = idx < items;
            const int t = idx & 3;
            const int bm = idx >> 2;
            const int b = live ? bm / p.m : 0;
            const int m = live ? bm % p.m : 0;
            float v[8];
#pragma unroll
            for (int j = 0; j < 8; j++) v[j] = 0.f;
            if (live && b < p.nblk) {
                // Fragment order of the 8 activations this lane supplies for block b:
                //   Q4_0: {4t, 4t+2, 16+4t, 18+4t | 4t+1, 4t+3, 17+4t, 19+4t}
                //   Q8_0: {8t .. 8t+7}
                const __half *xr = p.x + (size_t)m * p.k + b * 32;
                const float inv = do_norm ? inv_rms[m] : 1.f;
                __half raw[8], nw[8];
                if (QT == TLC_TYPE_Q4_0) {
                    *reinterpret_cast<uint2 *>(&raw[0]) = *reinterpret_cast<const uint2 *>(xr + 4 * t);
                    *reinterpret_cast<uint2 *>(&raw[4]) = *reinterpret_cast<const uint2 *>(xr + 16 + 4 * t);
                    if (do_norm) {
                        const __half *wr = p.norm_w + b * 32;
                        *reinterpret_cast<uint2 *>(&nw[0]) = *reinterpret_cast<const uint2 *>(wr + 4 * t);
                        *reinterpret_cast<uint2 *>(&nw[4]) = *reinterpret_cast<const uint2 *>(wr + 16 + 4 * t);
                    }
                } else {
                    *reinterpret_cast<uint4 *>(&raw[0]) = *reinterpret_cast<const uint4 *>(xr + 8 * t);
                    if (do_norm)
                        *reinterpret_cast<uint4 *>(&nw[0]) =
                            *reinterpret_cast<const uint4 *>(p.norm_w + b * 32 + 8 * t);
                }
                float f[8];
#pragma unroll
                for (int j = 0; j < 8; j++) {
                    f[j] = __half2float(raw[j]);
                    // f16((x * inv) * w): two separately rounded f32 multiplies, then RNE
                    // (Tensor::rms_norm_cpu, src/ops/normalization.rs:236-240).
                    if (do_norm)
                        f[j] = __half2float(
                            __float2half_rn(__fmul_rn(__fmul_rn(f[j], inv), __half2float(nw[j]))));
                }
                if (QT == TLC_TYPE_Q4_0) {
                    v[0] = f[0]; v[1] = f[2]; v[2] = f[4]; v[3] = f[6];
                    v[4] = f[1]; v[5] = f[3]; v[6] = f[5]; v[7] = f[7];
                } else {
#pragma unroll
                    for (int j = 0; j < 8; j++) v[j] = f[j];
                }
            }
            float s = ((v[0] + v[1]) + (v[2] + v[3])) + ((v[4] + v[5]) + (v[6] + v[7]));
            s += __shfl_xor_sync(0xffffffffu, s, 1);
            s += __shfl_xor_sync(0xffffffffu, s, 2);
            if (live) {
                __half2 h0 = __floats2half2_rn(v[0], v[1]);  // exact: v[] are f16 values
                __half2 h1 = __floats2half2_rn(v[2], v[3]);
                __half2 h2 = __floats2half2_rn(v[4], v[5]);
                __half2 h3 = __floats2half2_rn(v[6], v[7]);
                uint4 o;
                o.x = *reinterpret_cast<uint32_t *>(&h0);
                o.y = *reinterpret_cast<uint32_t *>(&h1);
                o.z = *reinterpret_cast<uint32_t *>(&h2);
                o.w = *reinterpret_cast<uint32_t *>(&h3);
                xperm[idx] = o;
                if (t == 0) xs8[b * MP + m] = -T::OFFSET * 5.9604644775390625e-08f * s;  // * 2^-24
            }
        }
    }
    consumer_bar();

    // (c) main loop
    const int g = lane >> 2, t = lane & 3;
    uint32_t it = 0;
    int slab_count = 0;
    __half hold[1] = {__float2half(0.f)};  // gate value kept between the two slabs of a gate/up unit

    for (int unit = blockIdx.x; unit < p.total_units; unit += gridDim.x) {
        for (int sub = 0; sub < p.subs; sub++, slab_count++) {
            int ti, sl;
            if (p.subs == 2) {
                ti = sub;
                sl = unit;
            } else {
                ti = 0;
                sl = unit;
                while (sl >= p.slabs[ti]) {
                    sl -= p.slabs[ti];
                    ti++;
                }
            }
            const GemvTensor &gt = p.t[ti];
            float acc[4 * NT];
#pragma unroll
            for (int i = 0; i < 4 * NT; i++) acc[i] = 0.f;

            for (int c = 0; c < p.nchunks; c++, it++) {
                const int s = it % S;
                const uint32_t par = (it / S) & 1u;
                // A wait that ran out skips the math but keeps the barrier protocol
                // going, so every warp still reaches the same bar.sync calls.
                const bool ready = __all_sync(0xffffffffu, mbar_wait(&full[s], par, abort_flag, p.status, 2));
                const int kcb = min(T::KCB, p.nblk - c * T::KCB);
                const int npairs = ready ? (kcb + 1) >> 1 : 0;
                const uint8_t *st = stages + (size_t)s * STAGE_BYTES;
                const uint32_t *seg_g = reinterpret_cast<const uint32_t *>(st + g * PITCH);
                const uint32_t *seg_g8 = reinterpret_cast<const uint32_t *>(st + (g + 8) * PITCH);
                for (int pr = warp; pr < npairs; pr += kConsumerWarps) {
                    uint32_t we_g[2], wo_g[2], we_g8[2], wo_g8[2];
                    float de_g, do_g, de_g8, do_g8;
                    load_pair<QT>(seg_g, pr, t, we_g, wo_g, de_g, do_g);
                    load_pair<QT>(seg_g8, pr, t, we_g8, wo_g8, de_g8, do_g8);
                    const int b0 = c * T::KCB + 2 * pr;
                    if (2 * pr + 1 >= kcb) {  // odd tail block does not exist
                        do_g = 0.f;
                        do_g8 = 0.f;
                    }
#pragma unroll
                    for (int e = 0; e < 2; e++) {
                        const int b = b0 + e;
                        uint4 xp[NT];
                        float2 ci[NT];
#pragma unroll
                        for (int nt = 0; nt < NT; nt++) {
                            const int mrow = nt * 8 + g;
                            xp[nt] = mrow < p.m ? xperm[((size_t)b * p.m + mrow) * 4 + t] : make_uint4(0, 0, 0, 0);
                            ci[nt] = *reinterpret_cast<const float2 *>(&xs8[b * MP + nt * 8 + 2 * t]);
                        }
                        if (e == 0)
                            block_mma<QT, NT>(we_g, we_g8, de_g, de_g8, xp, ci, acc);
                        else
                            block_mma<QT, NT>(wo_g, wo_g8, do_g, do_g8, xp, ci, acc);
                    }
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(&empty[s]);
            }

            // (d) cross-warp reduction and epilogue
            float *rbuf = red + (size_t)(slab_count & 1) * (kConsumerWarps * kRows * MP);
            float *mine = rbuf + warp * (kRows * MP);
#pragma unroll
            for (int nt = 0; nt < NT; nt++) {
                mine[g * MP + nt * 8 + 2 * t] = acc[nt * 4 + 0];
                mine[g * MP + nt * 8 + 2 * t + 1] = acc[nt * 4 + 1];
                mine[(g + 8) * MP + nt * 8 + 2 * t] = acc[nt * 4 + 2];
                mine[(g + 8) * MP + nt * 8 + 2 * t + 1] = acc[nt * 4 + 3];
            }
            consumer_bar();
            if (ctid < kRows * MP) {
                const int oi = 0;
                const int o = ctid;
                const int col = o >> 4, row = o & 15;
                const int n = sl * kRows + row;
                auto total = [&](int r_) {
                    float v = 0.f;
#pragma unroll
                    for (int w = 0; w < kConsumerWarps; w++) v += rbuf[w * (kRows * MP) + r_ * MP + col];
                    return v * 16777216.0f;  // undo the 2^-24 of the integer fragments
                };
                if (col < p.m && n < gt.n) {
                    __half h = __float2half_rn(total(row));
                    const size_t oidx = (size_t)col * gt.n + n;  // dense [m, N] index (residual, act)
                    const int pos = p.positions ? p.positions[col] : p.pos_offset + col;
                    // Where this output goes: dense rows by default; a KV-cache destination
                    // addresses rows by (sequence, position) instead.
                    const size_t yidx = (size_t)((long long)col * gt.row_stride + (long long)pos * gt.pos_stride) + n;
                    if (gt.rope_heads > 0) {
                        // Interleaved RoPE on the f16-rounded projection
                        // (rope_f16, shaders/unified.metal:2355-2417).
                        __half hp = __float2half_rn(total(row ^ 1));
                        const int dim = n % gt.head_dim;
                        const int pair = dim >> 1;
                        const float x0 = __half2float((dim & 1) ? hp : h);
                        const float x1 = __half2float((dim & 1) ? h : hp);
                        const float exponent = (float)(2 * pair) / (float)gt.head_dim;
                        const float freq = 1.0f / powf(p.rope_base, exponent);
                        const float theta = (float)(unsigned)pos * freq;
                        const float cs = cosf(theta), sn = sinf(theta);
                        const float r = (dim & 1) ? __fadd_rn(__fmul_rn(x0, sn), __fmul_rn(x1, cs))
                                                  : __fsub_rn(__fmul_rn(x0, cs), __fmul_rn(x1, sn));
                        gt.y[yidx] = __float2half_rn(r);
                    } else if (p.epilogue == TLC_EPI_RESIDUAL) {
                        gt.y[yidx] = __hadd(h, p.residual[oidx]);
                    } else if (p.epilogue == TLC_EPI_SWIGLU) {
                        if (sub == 0) {
                            hold[oi] = h;
                        } else {
                            // s = sigmoid(g) (f32, RNE); a = g*s; act = a*u: three
                            // f16 roundings as in debug/chat_demo_with_kvcache.tl:26-41.
                            const float gf = __half2float(hold[oi]);
                            const __half sg = __float2half_rn(1.0f / (1.0f + expf(-gf)));
                            const __half a = __hmul(hold[oi], sg);
                            p.t[0].y[oidx] = __hmul(a, h);
                        }
                    } else {
                        if (p.bias) h = __hadd(h, p.bias[n]);
                        gt.y[yidx] = h;
                    }
                }
            }
        }
    }
}

// ---------------------------------------------------------------------------
// Generic path: any type (F16 included), any M, no alignment assumptions.  One
// warp per output row; used for f16 weights only (embedding-tied heads, norms
// never go through linear) -- it is correct but far from the roofline.
// ---------------------------------------------------------------------------
__global__ void linear_generic_kernel(const uint8_t *__restrict__ w, size_t pitch, int type, int n_rows,
                                      int k, const __half *__restrict__ x, int m, __half *__restrict__ y,
                                      const __half *__restrict__ bias) {
    const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (warp >= n_rows) return;
    const uint8_t *row = w + (size_t)warp * pitch;
    for (int mm = 0; mm < m; mm++) {
        const __half *xr = x + (size_t)mm * k;
        float acc = 0.f;
        if (type == TLC_TYPE_F16) {
            const __half *wr = reinterpret_cast<const __half *>(row);
            for (int i = lane; i < k; i += 32) acc = fmaf(__half2float(wr[i]), __half2float(xr[i]), acc);
        } else {
            const int bb = type == TLC_TYPE_Q4_0 ? 18 : 34;
            for (int b = lane; b < k / 32; b += 32) {
                const uint8_t *blk = row + (size_t)b * bb;
                const float d = half_bits_to_float((uint32_t)blk[0] | ((uint32_t)blk[1] << 8));
                float s = 0.f;
                if (type == TLC_TYPE_Q4_0) {
                    for (int j = 0; j < 16; j++) {
                        const uint8_t q = blk[2 + j];
                        // dequantized weight rounded to f16 first, as the reference's loader does
                        const float w0 = __half2float(__float2half_rn(__fmul_rn((float)((int)(q & 15) - 8), d)));
                        const float w1 = __half2float(__float2half_rn(__fmul_rn((float)((int)(q >> 4) - 8), d)));
                        s = fmaf(w0, __half2float(xr[b * 32 + j]), s);
                        s = fmaf(w1, __half2float(xr[b * 32 + j + 16]), s);
                    }
                } else {
                    for (int j = 0; j < 32; j++) {
                        const float wv = __half2float(__float2half_rn(__fmul_rn((float)(int8_t)blk[2 + j], d)));
                        s = fmaf(wv, __half2float(xr[b * 32 + j]), s);
                    }
                }
                acc += s;
            }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
        if (lane == 0) {
            __half h = __float2half_rn(acc);
            if (bias) h = __hadd(h, bias[warp]);
            y[(size_t)mm * n_rows + warp] = h;
        }
    }
}

template <int QT, int NT>
int32_t launch_mma(tlc_ctx *ctx, GemvParams &p, size_t smem_fixed) {
    using T = QTraits<QT>;
    constexpr int PITCH = stage_pitch(T::KCB * T::BB);
    constexpr size_t STAGE_BYTES = (size_t)kRows * PITCH;
    const size_t budget = (size_t)ctx->prop.sharedMemPerBlockOptin;
    TLC_REQUIRE(smem_fixed + 2 * STAGE_BYTES <= budget, TLC_ERR_INVALID_OPERATION,
                "gemv: activations of %d x %d do not fit in shared memory", p.m, p.k);
    // Two CTAs per SM (16 consumer warps hide the shared-memory and MMA latency
    // of the unpack loop) whenever the activations leave room for at least
    // three ring stages in half of the SM's shared memory.
    const size_t half = (size_t)ctx->prop.sharedMemPerMultiprocessor / 2 - 1024;
    const bool two = smem_fixed + 3 * STAGE_BYTES <= half;
    const size_t cap = two ? half : budget;
    const int max_ctas = two ? 2 * ctx->sm_count : ctx->sm_count;
    int grid = p.total_units < max_ctas ? p.total_units : max_ctas;
    // No more stages than this CTA will ever fill.
    long per_cta = ((long)(p.total_units + grid - 1) / grid) * p.subs * p.nchunks;
    int stages = (int)((cap - smem_fixed) / STAGE_BYTES);
    if (stages > kMaxStages) stages = kMaxStages;
    if (stages > per_cta) stages = per_cta < 2 ? 2 : (int)per_cta;
    p.nstages = stages;
    size_t smem = smem_fixed + (size_t)stages * STAGE_BYTES;
    static bool configured[64] = {};
    if (!configured[ctx->device & 63]) {
        TLC_CUDA(cudaFuncSetAttribute(gemv_mma_kernel<QT, NT>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      (int)budget));
        TLC_CUDA(cudaFuncSetAttribute(gemv_mma_kernel<QT, NT>, cudaFuncAttributePreferredSharedMemoryCarveout,
                                      cudaSharedmemCarveoutMaxShared));
        configured[ctx->device & 63] = true;
    }
    gemv_mma_kernel<QT, NT><<<grid, kThreads, smem, ctx->stream>>>(p);
    TLC_CHECK_LAUNCH(ctx);
    return TLC_OK;
}

size_t gemv_fixed_smem(int nblk_pad, int m, int nt) {
    const int mp = 8 * nt;
    size_t s = 256;                                              // barriers, flags, inv_rms
    s += (size_t)2 * kConsumerWarps * kRows * mp * sizeof(float);  // red
    s += (size_t)nblk_pad * mp * sizeof(float);                  // xs8
    s += (size_t)nblk_pad * m * 4 * sizeof(uint4);               // xperm
    s += 128;                                                    // stage alignment slack
    return s;
}

}  // namespace

// Largest number of activation rows one launch can take for this K.
static int gemv_max_m(tlc_ctx *ctx, int type, int k) {
    const int nblk_pad = ((k / 32) + 1) & ~1;
    const size_t budget = (size_t)ctx->prop.sharedMemPerBlockOptin;
    const size_t stage = type == TLC_TYPE_Q4_0 ? (size_t)kRows * stage_pitch(64 * 18) : (size_t)kRows * stage_pitch(32 * 34);
    for (int m = 16; m >= 1; m--) {
        int nt = m > 8 ? 2 : 1;
        if (gemv_fixed_smem(nblk_pad, m, nt) + 3 * stage <= budget) return m;
    }
    return 0;
}

int32_t tlc_launch_gemv(tlc_ctx *ctx, const tlc_gemv_args &a) {
    TLC_REQUIRE(a.n_out >= 1 && a.n_out <= 3, TLC_ERR_INVALID_OPERATION, "gemv: %d outputs", a.n_out);
    TLC_REQUIRE(a.m >= 1, TLC_ERR_INVALID_OPERATION, "gemv: m = %d", a.m);
    const tlc_qtensor *w0 = a.outs[0].w;
    const int type = w0->type;
    const int64_t k = w0->n_cols;
    for (int i = 0; i < a.n_out; i++) {
        const tlc_qtensor *w = a.outs[i].w;
        TLC_REQUIRE(w && a.outs[i].y, TLC_ERR_INVALID_OPERATION, "gemv: null weight or output");
        TLC_REQUIRE(w->ctx->device == ctx->device, TLC_ERR_DEVICE,
                    "linear requires tensors on same device (weight on %d, context on %d)", w->ctx->device,
                    ctx->device);
        TLC_REQUIRE(w->type == type && w->n_cols == k, TLC_ERR_INVALID_OPERATION,
                    "fused linears must share type and input width");
        if (a.outs[i].rope_heads > 0)
            TLC_REQUIRE(w->n_rows % a.outs[i].rope_heads == 0 && (w->n_rows / a.outs[i].rope_heads) % 2 == 0,
                        TLC_ERR_INVALID_OPERATION, "rope needs an even head_dim (rows %lld, heads %d)",
                        (long long)w->n_rows, a.outs[i].rope_heads);
    }
    if (a.epilogue == TLC_EPI_SWIGLU)
        TLC_REQUIRE(a.n_out == 2 && a.outs[0].w->n_rows == a.outs[1].w->n_rows, TLC_ERR_INVALID_OPERATION,
                    "gate and up projections must have the same shape");

    if (type == TLC_TYPE_F16) {
        TLC_REQUIRE(a.epilogue == TLC_EPI_STORE && !a.norm_w && a.n_out == 1 && a.outs[0].rope_heads == 0,
                    TLC_ERR_INVALID_OPERATION, "fused epilogues need a quantized weight");
        const int threads = 256;
        const int64_t warps = w0->n_rows;
        unsigned grid = (unsigned)((warps * 32 + threads - 1) / threads);
        linear_generic_kernel<<<grid, threads, 0, ctx->stream>>>(
            static_cast<const uint8_t *>(w0->data), w0->row_pitch, type, (int)w0->n_rows, (int)k,
            static_cast<const __half *>(a.x), a.m, static_cast<__half *>(a.outs[0].y),
            static_cast<const __half *>(a.bias));
        TLC_CHECK_LAUNCH(ctx);
        return TLC_OK;
    }

    const int max_m = gemv_max_m(ctx, type, (int)k);
    TLC_REQUIRE(max_m >= 1, TLC_ERR_INVALID_OPERATION, "gemv: K = %lld too large for the shared-memory staging",
                (long long)k);
    // Activation rows beyond what one launch can hold are processed in
    // further passes over the weights.
    for (int m0 = 0; m0 < a.m; m0 += max_m) {
        const int mc = a.m - m0 < max_m ? a.m - m0 : max_m;
        GemvParams p{};
        p.n_out = a.n_out;
        p.total_units = 0;
        for (int i = 0; i < a.n_out; i++) {
            const tlc_qtensor *w = a.outs[i].w;
            p.t[i].w = static_cast<const uint8_t *>(w->data);
            p.t[i].pitch = w->row_pitch;
            p.t[i].n = (int)w->n_rows;
            // Outputs are [m, N] row-major: a pass over rows m0.. writes at y + m0*N.
            const long long rs = a.outs[i].row_stride >= 0 ? a.outs[i].row_stride : (long long)w->n_rows;
            p.t[i].row_stride = rs;
            p.t[i].pos_stride = a.outs[i].pos_stride;
            p.t[i].y = static_cast<__half *>(a.outs[i].y) + (size_t)m0 * rs;
            p.t[i].rope_heads = a.outs[i].rope_heads;
            p.t[i].head_dim = a.outs[i].rope_heads > 0 ? (int)(w->n_rows / a.outs[i].rope_heads) : 0;
            p.slabs[i] = (int)((w->n_rows + kRows - 1) / kRows);
            p.total_units += p.slabs[i];
        }
        p.subs = 1;
        if (a.epilogue == TLC_EPI_SWIGLU) {
            p.subs = 2;
            p.total_units = p.slabs[0];
        }
        p.k = (int)k;
        p.nblk = (int)(k / 32);
        p.nblk_pad = (p.nblk + 1) & ~1;
        const int kcb = type == TLC_TYPE_Q4_0 ? 64 : 32;
        p.nchunks = (p.nblk + kcb - 1) / kcb;
        p.m = mc;
        p.x = static_cast<const __half *>(a.x) + (size_t)m0 * k;
        p.norm_w = static_cast<const __half *>(a.norm_w);
        p.eps = a.eps;
        p.epilogue = a.epilogue;
        p.bias = static_cast<const __half *>(a.bias);
        p.residual = a.residual ? static_cast<const __half *>(a.residual) + (size_t)m0 * w0->n_rows : nullptr;
        p.pos_offset = a.pos_offset + m0;
        p.rope_base = (float)a.rope_base;
        p.positions = a.positions ? a.positions + m0 : nullptr;
        p.status = ctx->dev_status;
        const int nt = mc > 8 ? 2 : 1;
        const size_t fixed = gemv_fixed_smem(p.nblk_pad, mc, nt);
        int32_t rc;
        if (type == TLC_TYPE_Q4_0)
            rc = nt == 1 ? launch_mma<TLC_TYPE_Q4_0, 1>(ctx, p, fixed) : launch_mma<TLC_TYPE_Q4_0, 2>(ctx, p, fixed);
        else
            rc = nt == 1 ? launch_mma<TLC_TYPE_Q8_0, 1>(ctx, p, fixed) : launch_mma<TLC_TYPE_Q8_0, 2>(ctx, p, fixed);
        if (rc) return rc;
    }
    return TLC_OK;
}
