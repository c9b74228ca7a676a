// The fused dequant-GEMV kernel.  See tlc_gemv.cu for the design notes.
#pragma once

#include "tlc_gemv_common.cuh"

namespace tlc_gemv {

// Shared-memory layout (bytes from the start of dynamic shared memory):
//   0    full[12] mbarriers      128  empty[12] mbarriers      256  abort flag
//   512  sum-of-squares partials [16 activation rows][consumer warps]
//   1536 red   [2][AS sets][consumer warps][16 rows][MP] f32   cross-warp reduction, double buffered
//   ...  cinit [nblk_pad][NT][4 quad lanes] float2  accumulator start per block (columns 2t, 2t+1);
//              with one activation row: [nblk_pad] float4, the start value four times (a whole
//              C fragment in one load; columns past the first are never read back)
//   ...  xzero one zero uint4 (B fragment of activation rows that do not exist)
//   ...  xperm [nblk_pad][m][4 quad lanes] uint4    activations in fragment order
//   ...  ring  [stages][16 tiles]                   weight tiles as they lie in HBM (128-byte aligned)
//              F8 (below): [nblk_pad][4 limbs][32] bytes, the activations as FP8 limbs
__host__ __device__ inline size_t fixed_smem_bytes(int nblk_pad, int m, int nt, int as, int cw = 8, bool f8 = false) {
    size_t s = kHeaderBytes;
    s += (size_t)2 * as * cw * kRows * (8 * nt) * sizeof(float);
    s += m == 1 ? (size_t)nblk_pad * sizeof(float4) : (size_t)nblk_pad * nt * 4 * sizeof(float2);
    s += sizeof(uint4);
    s += f8 ? (size_t)nblk_pad * 128 : (size_t)nblk_pad * m * 4 * sizeof(uint4);
    s += 128;  // ring alignment slack
    return s;
}

// M1: exactly one activation row (the decode step of one sequence).  Columns 1-7
// of the 16x8 tensor-core tile are then never read back, so every lane may load
// the same B fragments and accumulator start values: their shared-memory
// addresses become warp-uniform with compile-time strides.
// CW: consumer warps, 8 (two CTAs per SM) or 16 (one CTA per SM, for launches whose
// activations leave no room for two).
// F8 (one activation row, Q4_0): the dot products run on the FP8 tensor-core path.  A nibble n in
// a byte of its own IS the e4m3 number n * 2^-9 (exponent fields 0 and 1 share one scale, as
// with the f16 subnormals above), so `w & 0x0F0F0F0F` and `(w >> 4) & 0x0F0F0F0F` are finished A
// fragments of m16n8k32: three integer operations per eight weights instead of seven, one MMA
// per block instead of two.  The activation row, scaled by a power of two so that its largest
// value lies in [64, 256), is split into four e4m3 limbs x' = l0 + l1 + l2 + l3 (each the e4m3
// rounding of what the earlier ones left: 16 significant bits, absolute error <= 2^-10, i.e.
// <= 2^-16 of the row's largest value); the limbs are four columns of the B operand, every
// product and every 32-term sum is exact in the f32 accumulator, and the four columns are added
// once per slab.  A row with a non-finite value yields NaN outputs.
template <int QT, int NT, int AS, bool M1, int CW, bool F8 = false>
__global__ void __launch_bounds__((CW + 1) * 32, CW == 8 ? 2 : 1) gemv_mma_kernel(const GemvParams p) {
    static_assert(!M1 || NT == 1, "one activation row needs one column tile");
    static_assert(!F8 || (M1 && QT == TLC_TYPE_Q4_0), "the FP8 path is for one activation row of Q4_0");
    static_assert(CW == 8 || CW == 16, "8 or 16 consumer warps");
    constexpr int CT = CW * 32;  // consumer threads
    using T = QTraits<QT>;
    constexpr int MP = 8 * NT;  // padded activation rows
    constexpr int TILE = T::TILE_BYTES;
    constexpr int STAGE_BYTES = kTilesPerStage * TILE;

    extern __shared__ __align__(128) uint8_t smem[];
    uint64_t *full = reinterpret_cast<uint64_t *>(smem);
    uint64_t *empty = reinterpret_cast<uint64_t *>(smem + 128);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(smem + 256);
    float *sq_part = reinterpret_cast<float *>(smem + 512);
    float *red = reinterpret_cast<float *>(smem + kHeaderBytes);
    static_assert(kMaxStages * 8 <= 128 && 512 + 16 * CW * 4 <= kHeaderBytes, "header layout");
    float2 *cinit = reinterpret_cast<float2 *>(red + 2 * AS * CW * kRows * MP);
    uint4 *xzero = M1 ? reinterpret_cast<uint4 *>(reinterpret_cast<float4 *>(cinit) + p.nblk_pad)
                      : reinterpret_cast<uint4 *>(cinit + (size_t)p.nblk_pad * NT * 4);
    uint4 *xperm = xzero + 1;
    uint8_t *stages = F8 ? reinterpret_cast<uint8_t *>(xperm) + (size_t)p.nblk_pad * 128
                         : reinterpret_cast<uint8_t *>(xperm + (size_t)p.nblk_pad * p.m * 4);
    float *f8_scale = reinterpret_cast<float *>(smem + 260);  // F8: 2^9 / (the row's power-of-two scale), NaN for a non-finite row
    float *mx_part = sq_part + CW;                            // F8: per-warp maxima of |x| and |norm weight| (rows 1, 2 of sq_part: one activation row uses row 0 only)
    stages = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(stages) + 127) & ~(uintptr_t)127);

    const int tid = threadIdx.x;
    const int warp = tid >> 5, lane = tid & 31;
    const int S = p.nstages;
    // Split K (p.ksplit > 1): CTA b works on K window b % ksplit -- tiles [kt0, kt0 + p.ktiles) of
    // every slab it owns, p.nblk blocks of the activation rows starting at block kb0 -- and shares
    // the slabs with the other CTAs of the same window.
    // (One activation row never splits: its instantiation folds all of this away.)
    const bool split = !M1 && p.ksplit > 1;
    const int ks = split ? (int)blockIdx.x % p.ksplit : 0;
    const int cta_i = split ? (int)blockIdx.x / p.ksplit : (int)blockIdx.x;
    const int cta_n = split ? (int)gridDim.x / p.ksplit : (int)gridDim.x;
    const int kt0 = split ? ks * p.ktiles_win : 0;
    const int kb0 = kt0 * T::TB;
    const int my_ktiles = split ? max(0, min(p.ktiles_win, p.ktiles_full - kt0)) : p.ktiles;
    const int my_nchunks = split ? (my_ktiles + kTilesPerStage - 1) / kTilesPerStage : p.nchunks;
    const int my_nblk = split ? max(0, min(p.ktiles_win * T::TB, p.k / 32 - kb0)) : p.nblk;

    if (tid == 0) {
        for (int s = 0; s < S; s++) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], CW);
        }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    __syncthreads();
    // The next kernel of the stream may be scheduled from here on: its producer
    // warps only read weights, everything else waits for this grid to finish.
    if (p.pdl_mode == 1) pdl_launch_dependents();

    // Units of this CTA (see the main loop below).  Worked out here, before anything waits for the
    // previous kernel: the divisions are then off the critical path of the decode step.
    const int u_lo = p.contig ? (int)((long long)cta_i * p.total_units / cta_n) : 0;
    const int u_hi = p.contig ? (int)((long long)(cta_i + 1) * p.total_units / cta_n) : 0;
    const int n_mine = p.contig ? u_hi - u_lo : ((int)p.total_units - cta_i + cta_n - 1) / cta_n;

    if (warp == CW) {
        // ------------------------------ producer ------------------------------
        // Weights are never written by a kernel, so the ring starts filling
        // before the previous kernel of the stream has finished.
        int rs = 0;
        uint32_t rpar = 1;
        const uint64_t policy = l2_evict_first_policy();
        const int pu_lo = u_lo, pcount = n_mine;
        for (int ui = 0; ui < pcount; ui++) {
            const int unit = p.contig ? pu_lo + ui : cta_i + ui * cta_n;
            for (int sub = 0; sub < p.subs; sub++) {
                int ti = 0, sl = unit;
                if (p.subs == 2) {
                    ti = sub;
                } else {
                    if (sl >= p.slabs[0]) { sl -= p.slabs[0]; ti = 1; }
                    if (ti == 1 && sl >= p.slabs[1]) { sl -= p.slabs[1]; ti = 2; }
                }
                const uint8_t *wbase = ti == 0 ? p.t[0].w : ti == 1 ? p.t[1].w : p.t[2].w;
                const size_t spitch = ti == 0 ? p.t[0].slab_pitch : ti == 1 ? p.t[1].slab_pitch : p.t[2].slab_pitch;
                for (int c = 0; c < my_nchunks; c++) {
                    const int s = rs;
                    // On a timeout the producer stops issuing copies; the consumers'
                    // own bounded waits then end the CTA.
                    if (!__all_sync(0xffffffffu, mbar_wait(&empty[s], rpar, abort_flag, p.status, 1, p.wait_ns))) return;
                    if (++rs == S) {
                        rs = 0;
                        rpar ^= 1u;
                    }
                    // The stage's tiles are contiguous in HBM: one bulk copy.
                    const int ntiles = min(kTilesPerStage, my_ktiles - c * kTilesPerStage);
                    const uint32_t bytes = (uint32_t)(ntiles * TILE);
                    if (lane == 0) {
                        const uint8_t *src = wbase + (size_t)sl * spitch + (size_t)(kt0 + c * kTilesPerStage) * TILE;
                        mbar_expect_tx(&full[s], bytes);
                        if (p.l2_hint)
                            bulk_g2s_hint(stages + (size_t)s * STAGE_BYTES, src, bytes, &full[s], policy);
                        else
                            bulk_g2s(stages + (size_t)s * STAGE_BYTES, src, bytes, &full[s]);
                    }
                }
            }
        }
        return;
    }

    // -------------------------------- consumers --------------------------------
    const int ctid = tid;  // 0..CT-1
    const bool do_norm = p.norm_w != nullptr;
    // The norm weights do not come from the previous kernel: the first round's are fetched
    // (the later rounds' brought into the cache) while that kernel is still running.
    uint4 nw_first = make_uint4(0, 0, 0, 0);
    if (do_norm) {
        const int items = p.nblk_pad * p.m * 4;
        for (int idx = ctid; idx < items; idx += CT) {
            const int t = idx & 3, b = M1 ? idx >> 2 : (idx >> 2) / p.m;
            if (b >= my_nblk) continue;
            const __half *wr = p.norm_w + (kb0 + b) * 32;
            if (idx == ctid) {
                if (QT == TLC_TYPE_Q4_0) {
                    const uint2 lo = *reinterpret_cast<const uint2 *>(wr + 4 * t);
                    const uint2 hi = *reinterpret_cast<const uint2 *>(wr + 16 + 4 * t);
                    nw_first = make_uint4(lo.x, lo.y, hi.x, hi.y);
                } else {
                    nw_first = *reinterpret_cast<const uint4 *>(wr + 8 * t);
                }
            } else {
                asm volatile("prefetch.global.L2 [%0];" ::"l"(wr));
            }
        }
    }
    // (nothing of the previous kernel is needed to clear the accumulator start values)
    for (int i = ctid; i < (M1 ? p.nblk_pad * 2 : p.nblk_pad * NT * 4); i += CT)
        cinit[i] = make_float2(0.f, 0.f);
    if (ctid == 0) *xzero = make_uint4(0, 0, 0, 0);
    pdl_wait();  // the activations (and residual) come from the previous kernel
    // Mode 3: the successor may be scheduled while this CTA does its own work, but not before the
    // predecessor is done (its CTAs then never wait behind two grids).
    if (p.pdl_mode == 3) pdl_launch_dependents();

    // (a) sum of squares per activation row: every thread takes 8-element chunks.
    if (F8) {
        // also the largest |x| and |norm weight|: their product (times the normalisation factor)
        // bounds the normalised row, which fixes its power-of-two scale without another pass
        float sq = 0.f, mx = 0.f, mw = do_norm ? 0.f : 1.f;
        bool bad = false;
        for (int k = ctid * 8; k < p.k; k += CT * 8) {
            const uint4 raw = *reinterpret_cast<const uint4 *>(p.x + k);
            const __half2 *h = reinterpret_cast<const __half2 *>(&raw);
#pragma unroll
            for (int j = 0; j < 4; j++) {
                const float2 v = __half22float2(h[j]);
                sq = fmaf(v.x, v.x, sq);
                sq = fmaf(v.y, v.y, sq);
                mx = fmaxf(mx, fmaxf(fabsf(v.x), fabsf(v.y)));
                bad = bad || !(fabsf(v.x) <= 65504.f) || !(fabsf(v.y) <= 65504.f);
            }
            if (do_norm) {
                const uint4 wraw = *reinterpret_cast<const uint4 *>(p.norm_w + k);
                const __half2 *wh = reinterpret_cast<const __half2 *>(&wraw);
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    const float2 v = __half22float2(wh[j]);
                    mw = fmaxf(mw, fmaxf(fabsf(v.x), fabsf(v.y)));
                    bad = bad || !(fabsf(v.x) <= 65504.f) || !(fabsf(v.y) <= 65504.f);
                }
            }
        }
        if (bad) mx = INFINITY;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            sq += __shfl_xor_sync(0xffffffffu, sq, o);
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
            mw = fmaxf(mw, __shfl_xor_sync(0xffffffffu, mw, o));
        }
        if (lane == 0) {
            sq_part[warp] = sq;
            mx_part[warp] = mx;
            mx_part[CW + warp] = mw;
        }
    } else if (do_norm) {
        for (int m = 0; m < p.m; m++) {
            const __half *xr = p.x + (size_t)m * p.k;
            float sq = 0.f;
            for (int k = ctid * 8; k < p.k; k += CT * 8) {
                const uint4 raw = *reinterpret_cast<const uint4 *>(xr + k);
                const __half2 *h = reinterpret_cast<const __half2 *>(&raw);
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    const float2 v = __half22float2(h[j]);
                    sq = fmaf(v.x, v.x, sq);
                    sq = fmaf(v.y, v.y, sq);
                }
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
            if (lane == 0) sq_part[m * CW + warp] = sq;
        }
    }
    consumer_bar<CT>();

    // (b) activations into fragment order + accumulator start values.  Item =
    // (block b, activation row m, quad lane t); the 4 t-items of a (b, m) are
    // adjacent lanes, so a 2-step shuffle gives the block sum.
    //   Q4_0 fragment order: {4t, 4t+2, 16+4t, 18+4t | 4t+1, 4t+3, 17+4t, 19+4t}
    //   Q8_0 fragment order: {8t .. 8t+7}
    {
        const int items = p.nblk_pad * p.m * 4;
        const int rounds = (items + CT - 1) / CT;
        float f8_s = 1.f;  // F8: the row's power-of-two scale
        if (F8) {
            float ss = 0.f, mxv = 0.f, mwv = 0.f;
#pragma unroll
            for (int w = 0; w < CW; w++) {
                ss += sq_part[w];
                mxv = fmaxf(mxv, mx_part[w]);
                mwv = fmaxf(mwv, mx_part[CW + w]);
            }
            // |f16((x * inv) * w)| <= bound * (1 + 2^-10): the scaled row stays below 256
            const float bound = do_norm ? mxv * (1.0f / sqrtf(ss / (float)p.k + p.eps)) * mwv * 1.001f : mxv;
            const bool bad = !(bound <= 3.0e38f);
            int e = bound > 0.f && !bad ? 7 - ilogbf(bound) : 0;
            e = e < -100 ? -100 : e > 100 ? 100 : e;
            f8_s = exp2f((float)e);
            if (ctid == 0) *f8_scale = bad ? __int_as_float(0x7fc00000) : 512.0f / f8_s;  // 2^9 undoes the e4m3 nibbles
        }
        for (int r = 0; r < rounds; r++) {
            const int idx = ctid + r * CT;
            const bool live = idx < items;
            const int t = idx & 3;
            const int bm = idx >> 2;
            const int b = !live ? 0 : M1 ? bm : bm / p.m;
            const int m = !live || M1 ? 0 : bm % p.m;
            float v[8];
#pragma unroll
            for (int j = 0; j < 8; j++) v[j] = 0.f;
            if (live && b < my_nblk) {
                const __half *xr = p.x + (size_t)m * p.k + (kb0 + b) * 32;
                float inv = 1.f;
                if (do_norm) {
                    float ss = 0.f;
#pragma unroll
                    for (int w = 0; w < CW; w++) ss += sq_part[m * CW + w];
                    inv = 1.0f / sqrtf(ss / (float)p.k + p.eps);
                }
                __align__(16) __half raw[8], nw[8];
                if (QT == TLC_TYPE_Q4_0) {
                    *reinterpret_cast<uint2 *>(&raw[0]) = *reinterpret_cast<const uint2 *>(xr + 4 * t);
                    *reinterpret_cast<uint2 *>(&raw[4]) = *reinterpret_cast<const uint2 *>(xr + 16 + 4 * t);
                    if (do_norm && r > 0) {
                        const __half *wr = p.norm_w + (kb0 + b) * 32;
                        *reinterpret_cast<uint2 *>(&nw[0]) = *reinterpret_cast<const uint2 *>(wr + 4 * t);
                        *reinterpret_cast<uint2 *>(&nw[4]) = *reinterpret_cast<const uint2 *>(wr + 16 + 4 * t);
                    }
                } else {
                    *reinterpret_cast<uint4 *>(&raw[0]) = *reinterpret_cast<const uint4 *>(xr + 8 * t);
                    if (do_norm && r > 0)
                        *reinterpret_cast<uint4 *>(&nw[0]) = *reinterpret_cast<const uint4 *>(p.norm_w + (kb0 + b) * 32 + 8 * t);
                }
                if (do_norm && r == 0) *reinterpret_cast<uint4 *>(&nw[0]) = nw_first;
                float f[8];
#pragma unroll
                for (int j = 0; j < 8; j++) {
                    f[j] = __half2float(raw[j]);
                    // f16((x * inv) * w): two separately rounded f32 multiplies, then RNE
                    // (Tensor::rms_norm_cpu, src/ops/normalization.rs:236-240).
                    if (do_norm)
                        f[j] = __half2float(__float2half_rn(__fmul_rn(__fmul_rn(f[j], inv), __half2float(nw[j]))));
                }
                if (F8) {
#pragma unroll
                    for (int j = 0; j < 8; j++) v[j] = f[j] * f8_s;  // natural order: 4t .. 4t+3, 16+4t .. 19+4t
                } else if (QT == TLC_TYPE_Q4_0) {
                    v[0] = f[0]; v[1] = f[2]; v[2] = f[4]; v[3] = f[6];
                    v[4] = f[1]; v[5] = f[3]; v[6] = f[5]; v[7] = f[7];
                } else {
#pragma unroll
                    for (int j = 0; j < 8; j++) v[j] = f[j];
                }
            }
            if (F8) {
                // Four e4m3 limbs per value, each the rounding of what the earlier ones left; limb c
                // of the item's eight values is eight bytes of column c of the B operand, and the
                // column's sum over the block (exact in f32) gives the accumulator its start
                // value -8 * 2^-9 * sum: the -8 of (q - 8) for that column.
                float cs[4];
#pragma unroll
                for (int c = 0; c < 4; c++) {
                    uint32_t wd[2];
                    float sum = 0.f;
#pragma unroll
                    for (int hw = 0; hw < 2; hw++) {
                        uint16_t p01, p23;
                        asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(p01) : "f"(v[4 * hw + 1]), "f"(v[4 * hw + 0]));
                        asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(p23) : "f"(v[4 * hw + 3]), "f"(v[4 * hw + 2]));
                        uint32_t h01, h23;
                        asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(h01) : "h"(p01));
                        asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(h23) : "h"(p23));
                        const float2 q01 = __half22float2(*reinterpret_cast<const __half2 *>(&h01));
                        const float2 q23 = __half22float2(*reinterpret_cast<const __half2 *>(&h23));
                        v[4 * hw + 0] -= q01.x;
                        v[4 * hw + 1] -= q01.y;
                        v[4 * hw + 2] -= q23.x;
                        v[4 * hw + 3] -= q23.y;
                        sum += (q01.x + q01.y) + (q23.x + q23.y);
                        wd[hw] = (uint32_t)p01 | ((uint32_t)p23 << 16);
                    }
                    sum += __shfl_xor_sync(0xffffffffu, sum, 1);
                    sum += __shfl_xor_sync(0xffffffffu, sum, 2);
                    cs[c] = -8.0f * 0.001953125f * sum;
                    if (live)
                        *reinterpret_cast<uint2 *>(reinterpret_cast<uint8_t *>(xperm) + ((size_t)(b * 4 + c) * 32 + t * 8)) =
                            make_uint2(wd[0], wd[1]);
                }
                if (live && t == 0) reinterpret_cast<float4 *>(cinit)[b] = make_float4(cs[0], cs[1], cs[2], cs[3]);
                continue;
            }
            float s = ((v[0] + v[1]) + (v[2] + v[3])) + ((v[4] + v[5]) + (v[6] + v[7]));
            s += __shfl_xor_sync(0xffffffffu, s, 1);
            s += __shfl_xor_sync(0xffffffffu, s, 2);
            if (live) {
                const __half2 h0 = __floats2half2_rn(v[0], v[1]);  // exact: v[] are f16 values
                const __half2 h1 = __floats2half2_rn(v[2], v[3]);
                const __half2 h2 = __floats2half2_rn(v[4], v[5]);
                const __half2 h3 = __floats2half2_rn(v[6], v[7]);
                uint4 o;
                o.x = *reinterpret_cast<const uint32_t *>(&h0);
                o.y = *reinterpret_cast<const uint32_t *>(&h1);
                o.z = *reinterpret_cast<const uint32_t *>(&h2);
                o.w = *reinterpret_cast<const uint32_t *>(&h3);
                xperm[idx] = o;
                if (t == 0) {
                    // Column m of the 16x8 tile sits in the C fragment of quad lane (m%8)/2,
                    // components m%2 (row g) and m%2 + 2 (row g+8).
                    const float cv = -T::OFFSET * 5.9604644775390625e-08f * s;  // * 2^-24
                    if (M1) {
                        reinterpret_cast<float4 *>(cinit)[b] = make_float4(cv, cv, cv, cv);
                    } else {
                        float *cf = reinterpret_cast<float *>(&cinit[(b * NT + (m >> 3)) * 4 + ((m & 7) >> 1)]);
                        cf[m & 1] = cv;  // rows g and g+8 of the tile start from the same value
                    }
                }
            }
        }
    }
    consumer_bar<CT>();

    // (c) main loop
    const int g = lane >> 2, t = lane & 3;
    // Loop-invariant shared-memory addresses (32-bit, explicit ld.shared: a generic
    // load would go through the global-memory path).  B fragments of activation
    // row nt*8+g: xperm[(block*m + row)*4 + t]; rows that do not exist read xzero.
    uint32_t xp_addr[NT], xp_stride[NT];
#pragma unroll
    for (int nt = 0; nt < NT; nt++) {
        const bool has = nt * 8 + g < p.m;
        xp_addr[nt] = M1 ? smem_u32(xperm + t) : has ? smem_u32(xperm + (nt * 8 + g) * 4 + t) : smem_u32(xzero);
        xp_stride[nt] = M1 ? 64u : has ? (uint32_t)p.m * 64u : 0u;
    }
    const uint32_t ci_addr = M1 ? smem_u32(cinit) : smem_u32(cinit + t);
    const uint32_t stages_addr = smem_u32(stages);

    // Units of this CTA: with only a few per CTA a balanced contiguous range
    // (1.5 % faster on the TinyLlama decode step), otherwise blockIdx.x,
    // blockIdx.x + gridDim.x, ... so that neighbouring CTAs stream neighbouring
    // rows (9 % faster on a 132 MB weight).  They are processed in batches of AS
    // accumulator sets (one set = one 16-row slab; a gate/up unit takes two) with
    // ONE cross-warp reduction per batch.
    const int ub = AS >> (p.subs - 1);  // units per batch (subs is 1 or 2)
    // The first output of this thread (item `ctid` of the first batch) adds a residual value and / or
    // is addressed by a position that earlier kernels wrote: both are fetched now, so that their
    // latency runs beside the dot products instead of after the reduction at the very end of the
    // kernel (the tail of every kernel is on the critical path of a decode step).
    __half res_first = __ushort_as_half((unsigned short)0);
    int pos_first = 0;
    bool have_first = false;
    if (!split) {
        const int pu = M1 ? kRows : kRows * p.m;
        const int ui = M1 ? ctid >> 4 : ctid / pu, rc = M1 ? ctid & 15 : ctid % pu;
        const int col = rc >> 4, row = rc & 15;
        if (ui < min(ub, n_mine)) {
            int ti = 0, sl = p.contig ? u_lo + ui : cta_i + ui * cta_n;
            if (p.subs == 1) {
                if (sl >= p.slabs[0]) { sl -= p.slabs[0]; ti = 1; }
                if (ti == 1 && sl >= p.slabs[1]) { sl -= p.slabs[1]; ti = 2; }
            }
            const int n = sl * kRows + row;
            const int wn = ti == 0 ? p.t[0].n : ti == 1 ? p.t[1].n : p.t[2].n;
            if (n < wn) {
                have_first = true;
                pos_first = p.positions ? p.positions[col] : p.pos_offset + col;
                if (p.epilogue == TLC_EPI_RESIDUAL) res_first = p.residual[(size_t)col * wn + n];
            }
        }
    }
    int rs = 0;           // ring position and its parity, carried from stage to stage
    uint32_t rpar = 0;
    int batch_count = 0;

    // Words and scales of one tile for this lane: rows g (lo) and g + 8 (hi).
    struct TileRegs {
        uint4 vlo, vhi;
        uint32_t slo[2], shi[2];
    };
    auto load_tile = [&](TileRegs &r, uint32_t tb) {
        r.vlo = lds_u128(tb + lane * 16);
        r.vhi = lds_u128(tb + 512 + lane * 16);
        if (QT == TLC_TYPE_Q4_0) {
            const uint2 a = lds_u64(tb + 1024 + g * 8), b = lds_u64(tb + 1024 + (g + 8) * 8);
            r.slo[0] = a.x; r.slo[1] = a.y;
            r.shi[0] = b.x; r.shi[1] = b.y;
        } else {
            r.slo[0] = lds_u32(tb + 1024 + g * 4);
            r.shi[0] = lds_u32(tb + 1024 + (g + 8) * 4);
            r.slo[1] = r.shi[1] = 0;
        }
    };

    for (int i0 = 0; i0 < n_mine; i0 += ub, batch_count++) {
        const int nsets = min(ub, n_mine - i0) * p.subs;
        float acc[AS][4 * NT];
#pragma unroll
        for (int a = 0; a < AS; a++)
#pragma unroll
            for (int i = 0; i < 4 * NT; i++) acc[a][i] = 0.f;

#pragma unroll
        for (int a = 0; a < AS; a++) {
            if (a >= nsets) break;
            // The math of one tile, block by block; B fragments and accumulator
            // start values of block j + 1 are fetched while block j is in the
            // tensor cores.  b0: first block of the tile.
            auto do_tile = [&](const TileRegs &r, uint32_t b0) {
                const uint32_t lo[4] = {r.vlo.x, r.vlo.y, r.vlo.z, r.vlo.w};
                const uint32_t hi[4] = {r.vhi.x, r.vhi.y, r.vhi.z, r.vhi.w};
                float dlo[4], dhi[4];
#pragma unroll
                for (int h = 0; h < T::TB / 2; h++) {
                    const float2 l = __half22float2(*reinterpret_cast<const __half2 *>(&r.slo[h]));
                    const float2 u = __half22float2(*reinterpret_cast<const __half2 *>(&r.shi[h]));
                    dlo[2 * h] = l.x; dlo[2 * h + 1] = l.y;
                    dhi[2 * h] = u.x; dhi[2 * h + 1] = u.y;
                }
                if (F8) {
                    // B fragment: limb column g & 3 (columns 4-7 repeat 0-3 and are never read back),
                    // 128 bytes per block; start values of columns 2(t&1), 2(t&1)+1, 16 bytes per block
                    const uint32_t xa = smem_u32(xperm) + (uint32_t)((g & 3) * 32 + t * 8) + b0 * 128u;
                    const uint32_t ca = smem_u32(cinit) + (uint32_t)((t & 1) * 8) + b0 * 16u;
                    uint2 bf = lds_u64(xa);
                    float2 ci = lds_f32x2(ca);
#pragma unroll
                    for (int j = 0; j < 4; j++) {
                        const uint32_t fa[4] = {lo[j] & 0x0F0F0F0Fu, hi[j] & 0x0F0F0F0Fu, (lo[j] >> 4) & 0x0F0F0F0Fu,
                                                (hi[j] >> 4) & 0x0F0F0F0Fu};
                        const uint2 bc = bf;
                        const float2 cc = ci;
                        if (j + 1 < 4) {
                            bf = lds_u64(xa + (j + 1) * 128);
                            ci = lds_f32x2(ca + (j + 1) * 16);
                        }
                        float d[4] = {cc.x, cc.y, cc.x, cc.y};
                        mma16832_e4m3(d, fa, bc.x, bc.y);
                        acc[a][0] = fmaf(dlo[j], d[0] + d[1], acc[a][0]);
                        acc[a][2] = fmaf(dhi[j], d[2] + d[3], acc[a][2]);
                    }
                    return;
                }
                if (M1) {
                    // B fragments 64 bytes and start values 16 bytes apart from block to block
                    const uint32_t xa = xp_addr[0] + b0 * 64u, ca = ci_addr + b0 * 16u;
                    uint4 xp = lds_u128(xa);
                    uint4 ci = lds_u128(ca);
#pragma unroll
                    for (int j = 0; j < T::TB; j++) {
                        uint32_t w0[2], w1[2], a1[4], a2[4];
                        if (QT == TLC_TYPE_Q4_0) {
                            w0[0] = lo[j];
                            w1[0] = hi[j];
                            w0[1] = w1[1] = 0;
                        } else {
                            w0[0] = lo[2 * j];
                            w0[1] = lo[2 * j + 1];
                            w1[0] = hi[2 * j];
                            w1[1] = hi[2 * j + 1];
                        }
                        unpack<QT>(w0, w1, a1, a2);
                        const uint4 xc = xp, cq = ci;
                        if (j + 1 < T::TB) {
                            xp = lds_u128(xa + (j + 1) * 64);
                            ci = lds_u128(ca + (j + 1) * 16);
                        }
                        const float cc[4] = {__uint_as_float(cq.x), __uint_as_float(cq.y), __uint_as_float(cq.z),
                                             __uint_as_float(cq.w)};
                        float d1[4], d2[4];
                        mma16816(d1, a1, xc.x, xc.y, cc);
                        mma16816(d2, a2, xc.z, xc.w, d1);
                        // only column 0 of the tile (d2[0], d2[2] of quad lane 0) is ever read back
                        acc[a][0] = fmaf(dlo[j], d2[0], acc[a][0]);
                        acc[a][2] = fmaf(dhi[j], d2[2], acc[a][2]);
                    }
                    return;
                }
                uint32_t xa[NT], ca = ci_addr + b0 * (NT * 32);
                uint4 xp[NT];
                float2 ci[NT];
#pragma unroll
                for (int nt = 0; nt < NT; nt++) {
                    xa[nt] = xp_addr[nt] + b0 * xp_stride[nt];
                    xp[nt] = lds_u128(xa[nt]);
                    ci[nt] = lds_f32x2(ca + nt * 32);
                }
#pragma unroll
                for (int j = 0; j < T::TB; j++) {
                    uint32_t w0[2], w1[2], a1[4], a2[4];
                    if (QT == TLC_TYPE_Q4_0) {
                        w0[0] = lo[j];
                        w1[0] = hi[j];
                        w0[1] = w1[1] = 0;
                    } else {
                        w0[0] = lo[2 * j];
                        w0[1] = lo[2 * j + 1];
                        w1[0] = hi[2 * j];
                        w1[1] = hi[2 * j + 1];
                    }
                    unpack<QT>(w0, w1, a1, a2);
                    uint4 xc[NT];
                    float2 cc2[NT];
#pragma unroll
                    for (int nt = 0; nt < NT; nt++) {
                        xc[nt] = xp[nt];
                        cc2[nt] = ci[nt];
                        if (j + 1 < T::TB) {
                            xa[nt] += xp_stride[nt];
                            xp[nt] = lds_u128(xa[nt]);
                            ci[nt] = lds_f32x2(ca + ((j + 1) * NT + nt) * 32);
                        }
                    }
#pragma unroll
                    for (int nt = 0; nt < NT; nt++) {
                        const float cc[4] = {cc2[nt].x, cc2[nt].y, cc2[nt].x, cc2[nt].y};
                        float d1[4], d2[4];
                        mma16816(d1, a1, xc[nt].x, xc[nt].y, cc);
                        mma16816(d2, a2, xc[nt].z, xc[nt].w, d1);
                        acc[a][nt * 4 + 0] = fmaf(dlo[j], d2[0], acc[a][nt * 4 + 0]);
                        acc[a][nt * 4 + 1] = fmaf(dlo[j], d2[1], acc[a][nt * 4 + 1]);
                        acc[a][nt * 4 + 2] = fmaf(dhi[j], d2[2], acc[a][nt * 4 + 2]);
                        acc[a][nt * 4 + 3] = fmaf(dhi[j], d2[3], acc[a][nt * 4 + 3]);
                    }
                }
            };
            for (int c = 0; c < my_nchunks; c++) {
                // A wait that ran out skips the math but keeps the barrier protocol
                // going, so every warp still reaches the same bar.sync calls.
                const bool ready = __all_sync(0xffffffffu, mbar_wait(&full[rs], rpar, abort_flag, p.status, 2, p.wait_ns));
                const int ntiles = ready ? min(kTilesPerStage, my_ktiles - c * kTilesPerStage) : 0;
                const uint32_t sbase = stages_addr + (uint32_t)rs * STAGE_BYTES;
                const uint32_t cb0 = (uint32_t)(c * kTilesPerStage * T::TB);  // first block of the stage
                if (ntiles == kTilesPerStage) {
                    // Lane (g, t) reads the words of rows g and g + 8 of its warp's two tiles
                    // up front (four 16-byte loads), then runs the blocks.
                    constexpr int TPW = kTilesPerStage / CW;  // tiles per warp and stage
                    static_assert(TPW * CW == kTilesPerStage && TPW >= 1, "whole tiles per warp");
                    TileRegs r[TPW];
#pragma unroll
                    for (int i = 0; i < TPW; i++) load_tile(r[i], sbase + (uint32_t)(warp + i * CW) * TILE);
#pragma unroll
                    for (int i = 0; i < TPW; i++) do_tile(r[i], cb0 + (uint32_t)(warp + i * CW) * T::TB);
                } else {
                    for (int ti = warp; ti < ntiles; ti += CW) {
                        TileRegs r0;
                        load_tile(r0, sbase + (uint32_t)ti * TILE);
                        do_tile(r0, cb0 + (uint32_t)ti * T::TB);
                    }
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(&empty[rs]);
                if (++rs == S) {
                    rs = 0;
                    rpar ^= 1u;
                }
            }
        }

        // (d) cross-warp reduction and epilogue of the batch
        if (F8) {  // quad lanes 0 and 1 hold limb columns 0-1 and 2-3: lane 0 gets their sum
#pragma unroll
            for (int a = 0; a < AS; a++) {
                acc[a][0] += __shfl_xor_sync(0xffffffffu, acc[a][0], 1);
                acc[a][2] += __shfl_xor_sync(0xffffffffu, acc[a][2], 1);
            }
        }
        if (p.pdl_mode == 2 && i0 + ub >= n_mine) pdl_launch_dependents();
        float *rbuf = red + (size_t)(batch_count & 1) * (AS * CW * kRows * MP);
#pragma unroll
        for (int a = 0; a < AS; a++) {
            if (a >= nsets) break;
            float *mine = rbuf + (a * CW + warp) * (kRows * MP);
#pragma unroll
            for (int nt = 0; nt < NT; nt++) {
                *reinterpret_cast<float2 *>(&mine[g * MP + nt * 8 + 2 * t]) = make_float2(acc[a][nt * 4 + 0], acc[a][nt * 4 + 1]);
                *reinterpret_cast<float2 *>(&mine[(g + 8) * MP + nt * 8 + 2 * t]) =
                    make_float2(acc[a][nt * 4 + 2], acc[a][nt * 4 + 3]);
            }
        }
        consumer_bar<CT>();
        // Outputs of the batch: (unit, row, activation row) items over the consumer threads.
        const int per_unit = M1 ? kRows : kRows * p.m;  // one activation row: a constant, shifts instead of divisions below
        for (int item = ctid; item < (nsets >> (p.subs - 1)) * per_unit; item += CT) {  // subs is 1 or 2
            const int ui = item / per_unit, rc = item % per_unit;
            const int col = rc >> 4, row = rc & 15;
            const int a0 = ui * p.subs;
            int ti = 0, sl = p.contig ? u_lo + i0 + ui : cta_i + (i0 + ui) * cta_n;
            if (p.subs == 1) {
                if (sl >= p.slabs[0]) { sl -= p.slabs[0]; ti = 1; }
                if (ti == 1 && sl >= p.slabs[1]) { sl -= p.slabs[1]; ti = 2; }
            }
            const int n = sl * kRows + row;
            const int wn = ti == 0 ? p.t[0].n : ti == 1 ? p.t[1].n : p.t[2].n;
            if (n >= wn) continue;
            auto total = [&](int set, int r_) {
                const float *base = rbuf + (size_t)set * CW * (kRows * MP) + r_ * MP + col;
                float v = 0.f;
#pragma unroll
                for (int w = 0; w < CW; w++) v += base[w * (kRows * MP)];
                if (F8) return v * *f8_scale;  // undo the row's scale and the 2^-9 of the e4m3 nibbles
                return v * 16777216.0f;  // undo the 2^-24 of the integer fragments
            };
            if (split) {
                // Split K: this window's f32 share of the dot product; gemv_splitk_finish_kernel adds
                // the windows and applies the epilogue.  Outputs of the fused weights lie side by side.
                const int noff = ti == 0 ? 0 : ti == 1 ? p.t[0].n : p.t[0].n + p.t[1].n;
                float *dst = p.partial + ((size_t)ks * p.m + col) * p.ntot + noff + n;
                *dst = total(a0, row);
                if (p.subs == 2) dst[p.t[0].n] = total(a0 + 1, row);
                continue;
            }
            __half *yout = ti == 0 ? p.t[0].y : ti == 1 ? p.t[1].y : p.t[2].y;
            const long long rstride = ti == 0 ? p.t[0].row_stride : ti == 1 ? p.t[1].row_stride : p.t[2].row_stride;
            const long long pstride = ti == 0 ? p.t[0].pos_stride : ti == 1 ? p.t[1].pos_stride : p.t[2].pos_stride;
            const int rheads = ti == 0 ? p.t[0].rope_heads : ti == 1 ? p.t[1].rope_heads : p.t[2].rope_heads;
            const int hdim = ti == 0 ? p.t[0].head_dim : ti == 1 ? p.t[1].head_dim : p.t[2].head_dim;
            __half h = __float2half_rn(total(a0, row));
            const size_t oidx = (size_t)col * wn + n;  // dense [m, N] index (residual, act)
            const bool first = have_first && i0 == 0 && item == ctid;
            int pos = first ? pos_first : p.positions ? p.positions[col] : p.pos_offset + col;
            // Second line of defence behind the host-side bound of the positions: a position outside
            // the cache is brought back to its last row, so the store stays inside the allocation; the
            // attention kernel of the same layer meets the same position, cuts it and raises the status
            // word (TLC_ERR_INDEX).  A clamp, not a test: a branch with a status update in this loop
            // cost the TinyLlama decode step 1.5 %.
            if (p.max_pos > 0) pos = min(max(pos, 0), p.max_pos - 1);
            // Where this output goes: dense rows by default; a KV-cache destination
            // addresses rows by (sequence, position) instead.
            const size_t yidx = (size_t)((long long)col * rstride + (long long)pos * pstride) + n;
            if (rheads > 0) {
                // Interleaved RoPE on the f16-rounded projection
                // (rope_f16, shaders/unified.metal:2355-2417).
                const __half hp = __float2half_rn(total(a0, row ^ 1));
                const int dim = n % hdim;
                const int pair = dim >> 1;
                const float x0 = __half2float((dim & 1) ? hp : h);
                const float x1 = __half2float((dim & 1) ? h : hp);
                const float exponent = (float)(2 * pair) / (float)hdim;
                const float freq = 1.0f / powf(p.rope_base, exponent);
                const float theta = (float)(unsigned)pos * freq;
                const float cs = cosf(theta), sn = sinf(theta);
                const float r = (dim & 1) ? __fadd_rn(__fmul_rn(x0, sn), __fmul_rn(x1, cs))
                                          : __fsub_rn(__fmul_rn(x0, cs), __fmul_rn(x1, sn));
                yout[yidx] = __float2half_rn(r);
            } else if (p.epilogue == TLC_EPI_RESIDUAL) {
                yout[yidx] = __hadd(h, first ? res_first : p.residual[oidx]);
            } else if (p.epilogue == TLC_EPI_SWIGLU) {
                // h = gate; s = sigmoid(g) (f32, RNE); a = g*s; act = a*u: three
                // f16 roundings as in debug/chat_demo_with_kvcache.tl:26-41.
                const __half up = __float2half_rn(total(a0 + 1, row));
                const float gf = __half2float(h);
                const __half sg = __float2half_rn(1.0f / (1.0f + expf(-gf)));
                const __half av = __hmul(h, sg);
                p.t[0].y[oidx] = __hmul(av, up);
            } else {
                if (p.bias) h = __hadd(h, p.bias[n]);
                yout[yidx] = h;
            }
        }
    }
}

}  // namespace tlc_gemv
