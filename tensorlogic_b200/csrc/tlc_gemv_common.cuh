// Shared pieces of the fused dequant-GEMV: launch parameters, block-format
// traits and the PTX wrappers (mbarrier, bulk async copy, mma.sync, programmatic
// dependent launch).
#pragma once

#include <cuda_fp16.h>

#include "tlc_internal.h"

namespace tlc_gemv {

constexpr int kRows = 16;  // rows of W per slab (the M of m16n8k16)
// Eight consumer warps per CTA and two CTAs per SM wherever two CTAs fit: sixteen
// warps in one CTA per SM measured 14 % slower on a 132 MB weight (one barrier and
// one reduction over twice the warps).  Launches whose activations leave room for
// one CTA only (several rows of a long K) take the sixteen-warp form.
constexpr int kMaxStages = 12;
constexpr int kHeaderBytes = 1536;  // mbarriers, abort flag, sum-of-squares partials

// Weights arrive in the tiled layout of tlc_tile.cuh: a ring stage is 16
// consecutive tiles of one 16-row slab (Q4_0: 64 blocks, Q8_0: 32 blocks of K).
constexpr int kTilesPerStage = 16;
template <int QT> struct QTraits;
template <> struct QTraits<TLC_TYPE_Q4_0> {
    static constexpr int TB = 4;             // blocks per tile
    static constexpr int TILE_BYTES = 1152;  // 1024 quant bytes + 16 rows x 4 f16 scales
    static constexpr float OFFSET = 8.0f;
};
template <> struct QTraits<TLC_TYPE_Q8_0> {
    static constexpr int TB = 2;
    static constexpr int TILE_BYTES = 1088;  // 1024 quant bytes + 16 rows x 2 f16 scales
    static constexpr float OFFSET = 128.0f;
};

struct GemvTensor {
    const uint8_t *w;   // tiles, [slab][k-tile]
    size_t slab_pitch;  // bytes of one 16-row slab
    int n;  // rows of W (outputs)
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
    int subs;      // slabs per unit (2 for the gate/up pair)
    int k;
    int nblk;      // k / 32
    int nblk_pad;  // rounded up to whole tiles
    int ktiles;    // tiles per slab
    int nchunks;   // ring stages per slab
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
    int max_pos;   // > 0: positions of outputs addressed by position are brought into [0, max_pos) (the one-pass
                   // kernel; the attention kernel reports them) or dropped with status TLC_DEV_INDEX (split-K finish)
    int nstages;
    int contig;    // 1: each CTA takes a contiguous range of units, 0: units blockIdx.x, + gridDim.x, ...
    int l2_hint;   // 1: weight copies carry the evict-first L2 hint
    int pdl_mode;  // 1: let the next kernel be scheduled at once, 2: only when this CTA's last slab is done, 3: after this CTA's own dependency wait
    tlc_dev_status *status;
    uint64_t wait_ns;  // how long a wait may last before the kernel gives up
    // Split K (ksplit > 1): the K range is cut into ksplit windows of ktiles_win tiles (nblk_pad is
    // then a window's padded block count); CTA b takes window b % ksplit and writes its f32 share of
    // every output to partial[window][activation row][ntot outputs] instead of running the epilogue.
    int ksplit, ktiles_win, ktiles_full, ntot;
    float *partial;
};

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
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
// Bounded wait: gives up after wait_ns nanoseconds, records where, and raises the
// CTA's abort flag; once that flag is up every later wait only polls briefly
// (long enough for copies already in flight to land) so the kernel drains and
// returns instead of hanging.  The result is made warp-uniform by the callers.
__device__ __forceinline__ bool mbar_wait(uint64_t *bar, uint32_t parity, volatile int *abort_flag,
                                          tlc_dev_status *status, int where, uint64_t wait_ns) {
    if (mbar_try_wait(bar, parity)) return true;
    const uint64_t limit = *abort_flag ? 20000ull : wait_ns;
    const uint64_t t0 = tlc_globaltimer_ns();
    do {
        if (mbar_try_wait(bar, parity)) return true;
    } while (tlc_globaltimer_ns() - t0 < limit);
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
// The same copy with an L2 eviction hint: weight tiles are read once per launch, so they
// are marked evict-first and leave the L2 to activations, norm weights and the KV cache.
__device__ __forceinline__ uint64_t l2_evict_first_policy() {
    uint64_t pol;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(pol));
    return pol;
}
__device__ __forceinline__ void bulk_g2s_hint(void *dst, const void *src, uint32_t bytes, uint64_t *bar,
                                              uint64_t policy) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;" ::
            "r"(smem_u32(dst)),
        "l"(src), "r"(bytes), "r"(smem_u32(bar)), "l"(policy)
        : "memory");
}
template <int N>
__device__ __forceinline__ void consumer_bar() {
    asm volatile("bar.sync 1, %0;" ::"n"(N) : "memory");
}
// Programmatic dependent launch: let the next kernel of the stream be scheduled
// now (it may start fetching its weights), and wait for the previous kernel's
// results before touching anything it wrote.
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// Explicit shared-memory loads by 32-bit address.
__device__ __forceinline__ uint32_t lds_u32(uint32_t a) {
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(a));
    return v;
}
__device__ __forceinline__ uint2 lds_u64(uint32_t a) {
    uint2 v;
    asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(a));
    return v;
}
__device__ __forceinline__ uint4 lds_u128(uint32_t a) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(a));
    return v;
}
__device__ __forceinline__ float2 lds_f32x2(uint32_t a) {
    float2 v;
    asm volatile("ld.shared.v2.f32 {%0,%1}, [%2];" : "=f"(v.x), "=f"(v.y) : "r"(a));
    return v;
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

// FP8 (e4m3) tensor-core step: 16 rows x 32 k of A, 32 k x 8 columns of B, f32 accumulate in place.
__device__ __forceinline__ void mma16832_e4m3(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k32.row.col.f32.e4m3.e4m3.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// Integer fragments of one block for rows g (w0*) and g+8 (w1*).
//   Q4_0: one 32-bit word of nibbles per row; every nibble ends up in the
//   lowest mantissa bits, so all fragments carry the same 2^-24 and the
//   activations need no per-slot scaling.
//     a1: elems {4t, 4t+2 | 16+4t, 18+4t}   a2: elems {4t+1, 4t+3 | 17+4t, 19+4t}
//   Q8_0: two words of int8 per row, biased to unsigned ((q+128) * 2^-24).
//     a1: elems {8t, 8t+1 | 8t+2, 8t+3}     a2: elems {8t+4, 8t+5 | 8t+6, 8t+7}
template <int QT>
__device__ __forceinline__ void unpack(const uint32_t (&w0)[2], const uint32_t (&w1)[2], uint32_t (&a1)[4],
                                       uint32_t (&a2)[4]) {
    if (QT == TLC_TYPE_Q4_0) {
        // A nibble in bits 4-7 of a half is the subnormal 16n * 2^-24: one f16
        // multiply by 1/16 (exact) moves it down -- on the FMA pipe, which idles,
        // instead of a shift on the integer pipe, which is the busy one.
        const __half2 sixteenth = __float2half2_rn(0.0625f);
        auto down = [&](uint32_t v) {
            const __half2 h = __hmul2(*reinterpret_cast<const __half2 *>(&v), sixteenth);
            return *reinterpret_cast<const uint32_t *>(&h);
        };
        const uint32_t s0 = w0[0] >> 8, s1 = w1[0] >> 8;
        a1[0] = w0[0] & 0x000F000Fu;
        a1[1] = w1[0] & 0x000F000Fu;
        a1[2] = down(w0[0] & 0x00F000F0u);
        a1[3] = down(w1[0] & 0x00F000F0u);
        a2[0] = s0 & 0x000F000Fu;
        a2[1] = s1 & 0x000F000Fu;
        a2[2] = down(s0 & 0x00F000F0u);
        a2[3] = down(s1 & 0x00F000F0u);
    } else {
        const uint32_t u0 = w0[0] ^ 0x80808080u, v0 = w1[0] ^ 0x80808080u;
        const uint32_t u1 = w0[1] ^ 0x80808080u, v1 = w1[1] ^ 0x80808080u;
        a1[0] = __byte_perm(u0, 0, 0x4140);
        a1[1] = __byte_perm(v0, 0, 0x4140);
        a1[2] = __byte_perm(u0, 0, 0x4342);
        a1[3] = __byte_perm(v0, 0, 0x4342);
        a2[0] = __byte_perm(u1, 0, 0x4140);
        a2[1] = __byte_perm(v1, 0, 0x4140);
        a2[2] = __byte_perm(u1, 0, 0x4342);
        a2[3] = __byte_perm(v1, 0, 0x4342);
    }
}

}  // namespace tlc_gemv
