// Prefill dequant-GEMM on the 5th-generation tensor cores (tcgen05 + TMEM).
//
//   y[M, N] = x[M, K] . W[N, K]^T,  W in GGUF Q4_0 / Q8_0 blocks, x and y f16.
//
// Takes the place of matmul_transposed_b_tiled_32x32_f16 (shaders/unified.metal:
// 4291-4347, chosen by src/ops/matmul.rs:377-381 for large shapes) applied to
// weights the reference dequantized at load time.  Here the blocks are
// dequantized on the way into shared memory: the B operand tile holds exactly
// the f16 values GGUFLoader::dequantize_q4_0 / _q8_0 produce
// (src/model/formats/gguf.rs:22-112: f16_rne((q - 8) * d), computed as an exact
// integer in f16 times the f16 scale, one rounding), and tcgen05.mma
// (kind::f16) accumulates in f32 in tensor memory -- the arithmetic of the
// Metal kernel (f16 inputs, f32 sum, one rounding on store).
//
// One CTA computes a (128*MT) x (128*NT) tile of y: MT sub-tiles of 128
// activation rows (the M of the MMA, one per 128 tensor-memory lanes x 128*NT
// columns) against 128*NT weight rows (the N of the MMA).  Wide tiles matter:
// every CTA streams its activation tile from L2, and at 128 x 128 that traffic
// (16 KB per 64-wide K step and SM) saturates the L2 long before the tensor
// cores; 256 x 256 halves it per MMA.  Per 64-wide K step:
//   warps 0-3   A loaders: cp.async of the activation rows into the 128-byte
//               swizzled K-major tile, several steps ahead;
//   warps 4-11  B producers (4*NT of them work): thread r dequantizes row r of
//               the weight tile (2 blocks = 64 values) into the same layout; the
//               row's quants (64 contiguous bytes per tile of the tiled weight
//               layout) are fetched a group of K steps ahead into registers;
//   warp 12     allocates tensor memory and issues the MMAs: four K=16
//               tcgen05.mma per sub-tile and stage, tcgen05.commit to hand the
//               stage back.
// All twelve worker warps share the epilogue: tcgen05.ld of the accumulator,
// f16 rounding, optional RoPE / bias / residual, store.
// All waits are bounded; a wait that runs out sets the status word and lets the
// CTA drain, free its tensor memory and return.
#pragma once

#include <cuda.h>
#include <cuda_fp16.h>

#include "tlc_internal.h"

namespace tlc_gemm {

constexpr int kBK = 64;  // K elements per stage (one 128-byte swizzle row)
// Threads of a CTA: 4 warps at the activation tile (one TMA issuer, or four cp.async loaders),
// 4*nt*pg weight-producer warps, the MMA warp.
__host__ __device__ constexpr int gemm_threads(int nt, int pg) { return 32 * (4 + 4 * nt * pg + 1); }

struct GemmParams {
    const uint8_t *w;   // weight tiles [slab of 16 rows][k-tile] (tlc_tile.cuh)
    const uint8_t *w2;  // second weight of the SiLU.mul pair (same shape) or null
    size_t w_pitch;     // bytes of one 16-row slab
    int k_tiles;        // tiles per slab
    const __half *x;         // [M, K]
    __half *y;               // [M, N]
    const __half *residual;  // [M, N] or null: y = f16(acc) + residual
    const __half *bias;      // [N] or null
    int m, n, k;
    // element (row r, output n) lands at y[r * row_stride + pos(r) * pos_stride + n],
    // pos(r) = positions[r] or pos_offset + r
    long long row_stride, pos_stride;
    int head_dim;  // > 0: interleaved RoPE over heads of this width
    int pos_offset;
    const int *positions;
    int max_pos;  // > 0: rows addressed by position are dropped from this position on (status TLC_DEV_INDEX)
    float rope_base;
    int vec_ok;  // strides, N and pointers allow 16-byte stores
    // Split K (up to 128 activation rows, few weight tiles): CTA z of gridDim.z = ksplit takes a
    // share of the K steps and stores its f32 accumulators to partial[z][row][noff + n] (rows of
    // ntot floats; the SiLU.mul pair: gate at n, up at N + n); gemv_splitk_finish_kernel adds
    // the shares and applies the epilogue.
    float *partial;
    int ksplit, ntot, noff;
    int a_tma;   // the activation tile arrives by TMA (tensor map in the second kernel argument)
    tlc_dev_status *status;
    uint64_t wait_ns;  // how long a wait may last before the kernel gives up
};

// Ring depth for a tile of 128*mt x 128*nt: stages of 16 KB per sub-tile.
__host__ __device__ constexpr int stages_for(int mt, int nt) { return 12 / (mt + nt); }
__host__ __device__ constexpr size_t smem_bytes(int mt, int nt) {
    return 1024 /*align*/ + (size_t)stages_for(mt, nt) * (size_t)(mt + nt) * 128 * 128 + 256;
}

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint64_t *bar, int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(uint64_t *bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t *bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
// One box of a 2-D tensor map into shared memory; its bytes count on `bar`.  x is the inner
// (contiguous) coordinate and must be a multiple of 16 bytes' worth of elements.
__device__ __forceinline__ void tma_load_2d(uint32_t smem_dst, const void *map, int x, int y, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(
            smem_dst),
        "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(bar)
        : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t *bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}\n"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
__device__ __forceinline__ bool mbar_wait(uint64_t *bar, uint32_t parity, volatile int *abort_flag,
                                          tlc_dev_status *status, int where, uint64_t wait_ns) {
    if (mbar_try_wait(bar, parity)) return true;
    const uint64_t limit = *abort_flag ? 20000ull : wait_ns;
    const uint64_t t0 = tlc_globaltimer_ns();
    do {
        if (mbar_try_wait(bar, parity)) return true;
    } while (tlc_globaltimer_ns() - t0 < limit);
    *abort_flag = 1;
    if (atomicCAS(&status->code, 0, 2) == 0) status->where = where;
    return false;
}
__device__ __forceinline__ void fence_async_proxy() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }

// Shared-memory matrix descriptor of a K-major tile with 128-byte swizzle:
// rows are 128 bytes (64 f16), 8-row groups are 1024 bytes apart.
__device__ __forceinline__ uint64_t make_desc(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr & 0x3FFFF) >> 4);  // start address
    d |= (uint64_t)1 << 16;                       // leading byte offset (unused with swizzle)
    d |= (uint64_t)(1024 >> 4) << 32;             // stride byte offset: 8 rows x 128 B
    d |= (uint64_t)1 << 46;                       // descriptor version of sm_100
    d |= (uint64_t)2 << 61;                       // SWIZZLE_128B
    return d;
}
// Instruction descriptor: f16 x f16 -> f32, both operands K-major, M = 128, N = n.
__host__ __device__ constexpr uint32_t idesc_for(int n) {
    return (1u << 4) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
}

__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                         uint32_t accumulate) {
    asm volatile(
        "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
        " tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n" ::"r"(tmem_d),
        "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t *bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
                 : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,"
        "%29,%30,%31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void cp_async16(uint32_t smem_dst, const void *gsrc, bool valid) {
    const int sz = valid ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_dst), "l"(gsrc), "r"(sz) : "memory");
}

// (1024 + a, 1024 + b) as f16 pair from two bytes: the byte goes into the low
// mantissa bits of 0x6400 (= 1024.0), so value - 1024 is the byte, exactly.
__device__ __forceinline__ __half2 bytes_to_half2(uint32_t x, uint32_t sel) {
    const uint32_t v = __byte_perm(x, 0x64646464u, sel);
    return *reinterpret_cast<const __half2 *>(&v);
}

// Dequantizes 8 consecutive values given as the 8 integer bytes of (lo, hi)
// words (already reduced to one value per byte) and returns one 16-byte chunk.
//   value = (byte - bias) * d, both steps exact/rounded exactly like the
//   reference: the integer is exact in f16 and the f16 product is correctly rounded.
__device__ __forceinline__ uint4 dequant8(uint32_t w0, uint32_t w1, __half2 bias, __half2 d2) {
    __half2 h[4];
    h[0] = __hmul2(__hsub2(bytes_to_half2(w0, 0x4140), bias), d2);
    h[1] = __hmul2(__hsub2(bytes_to_half2(w0, 0x4342), bias), d2);
    h[2] = __hmul2(__hsub2(bytes_to_half2(w1, 0x4140), bias), d2);
    h[3] = __hmul2(__hsub2(bytes_to_half2(w1, 0x4342), bias), d2);
    return *reinterpret_cast<const uint4 *>(h);
}

// Dequantizes one block of a weight row -- `q`: its quant words (4 for Q4_0, 8
// for Q8_0), `d`: its scale -- into four 16-byte pieces of the swizzled tile at
// `bt` (`piece`: the byte offsets of the row's pieces, `e`: which half of the K step).
template <int QT>
__device__ __forceinline__ void dequant_block(const uint32_t *q, __half d, uint8_t *bt, const uint32_t (&piece)[8],
                                              int e) {
    const __half2 d2 = __half2half2(d);
    uint4 c[4];
    if (QT == TLC_TYPE_Q4_0) {
        const __half2 bias = __float2half2_rn(1032.f);  // 1024 (magic) + 8
        c[0] = dequant8(q[0] & 0x0F0F0F0Fu, q[1] & 0x0F0F0F0Fu, bias, d2);                // elems 0..7
        c[1] = dequant8(q[2] & 0x0F0F0F0Fu, q[3] & 0x0F0F0F0Fu, bias, d2);                // 8..15
        c[2] = dequant8((q[0] >> 4) & 0x0F0F0F0Fu, (q[1] >> 4) & 0x0F0F0F0Fu, bias, d2);  // 16..23
        c[3] = dequant8((q[2] >> 4) & 0x0F0F0F0Fu, (q[3] >> 4) & 0x0F0F0F0Fu, bias, d2);  // 24..31
    } else {
        const __half2 bias = __float2half2_rn(1152.f);  // 1024 (magic) + 128 (sign flip)
#pragma unroll
        for (int j = 0; j < 4; j++) c[j] = dequant8(q[2 * j] ^ 0x80808080u, q[2 * j + 1] ^ 0x80808080u, bias, d2);
    }
#pragma unroll
    for (int j = 0; j < 4; j++) *reinterpret_cast<uint4 *>(bt + piece[4 * e + j]) = c[j];
}

// One 32-column piece of the epilogue for one activation row: f16 rounding of
// the accumulators `r`, then RoPE / bias / residual as the launch asks, store.
__device__ __forceinline__ void epilogue_piece(const GemmParams &p, const uint32_t (&r)[32], int row, int pos, int nb,
                                               __half *ybase) {
    __align__(16) __half h[32];
#pragma unroll
    for (int e = 0; e < 32; e++) h[e] = __float2half_rn(__uint_as_float(r[e]));
    if (p.head_dim > 0) {
        // Interleaved RoPE on the f16-rounded projection (rope_f16,
        // shaders/unified.metal:2355-2417); a pair never straddles this
        // thread's 32 columns because heads start at even columns.
#pragma unroll
        for (int e = 0; e < 32; e += 2) {
            const int pair = ((nb + e) % p.head_dim) >> 1;
            const float exponent = (float)(2 * pair) / (float)p.head_dim;
            const float freq = 1.0f / powf(p.rope_base, exponent);
            const float theta = (float)(unsigned)pos * freq;
            const float cs = cosf(theta), sn = sinf(theta);
            const float x0 = __half2float(h[e]), x1 = __half2float(h[e + 1]);
            h[e] = __float2half_rn(__fsub_rn(__fmul_rn(x0, cs), __fmul_rn(x1, sn)));
            h[e + 1] = __float2half_rn(__fadd_rn(__fmul_rn(x0, sn), __fmul_rn(x1, cs)));
        }
    }
    const bool whole = nb + 32 <= p.n;
    const bool vec_ok = p.vec_ok != 0;
    if (p.bias) {
#pragma unroll
        for (int e = 0; e < 32; e++)
            if (whole || nb + e < p.n) h[e] = __hadd(h[e], p.bias[nb + e]);
    }
    if (p.residual) {
        const __half *rrow = p.residual + (size_t)row * p.n + nb;
        if (whole && vec_ok) {
#pragma unroll
            for (int v = 0; v < 4; v++) {
                const uint4 rv = *reinterpret_cast<const uint4 *>(rrow + 8 * v);
                const __half *rh = reinterpret_cast<const __half *>(&rv);
#pragma unroll
                for (int e = 0; e < 8; e++) h[8 * v + e] = __hadd(h[8 * v + e], rh[e]);
            }
        } else {
#pragma unroll
            for (int e = 0; e < 32; e++)
                if (nb + e < p.n) h[e] = __hadd(h[e], rrow[e]);
        }
    }
    if (whole && vec_ok) {
#pragma unroll
        for (int v = 0; v < 4; v++)
            *reinterpret_cast<uint4 *>(ybase + nb + 8 * v) = *reinterpret_cast<const uint4 *>(h + 8 * v);
    } else {
#pragma unroll
        for (int e = 0; e < 32; e++)
            if (nb + e < p.n) ybase[nb + e] = h[e];
    }
}

// The SiLU.mul epilogue of one 32-column piece: `r` the gate accumulators, `ru` the up
// accumulators.  s = sigmoid(g) (f32, RNE); a = g*s; act = a*u: three f16 roundings as in
// debug/chat_demo_with_kvcache.tl:26-41 (the GEMV's SiLU.mul epilogue does the same).
__device__ __forceinline__ void epilogue_piece_swiglu(const GemmParams &p, const uint32_t (&r)[32],
                                                      const uint32_t (&ru)[32], int nb, __half *ybase) {
    __align__(16) __half h[32];
#pragma unroll
    for (int e = 0; e < 32; e++) {
        const __half gate = __float2half_rn(__uint_as_float(r[e]));
        const __half up = __float2half_rn(__uint_as_float(ru[e]));
        const __half sg = __float2half_rn(1.0f / (1.0f + expf(-__half2float(gate))));
        h[e] = __hmul(__hmul(gate, sg), up);
    }
    if (nb + 32 <= p.n && p.vec_ok) {
#pragma unroll
        for (int v = 0; v < 4; v++)
            *reinterpret_cast<uint4 *>(ybase + nb + 8 * v) = *reinterpret_cast<const uint4 *>(h + 8 * v);
    } else {
#pragma unroll
        for (int e = 0; e < 32; e++)
            if (nb + e < p.n) ybase[nb + e] = h[e];
    }
}

// Tensor map of activations for the TMA-fed A tile (defined in tlc_gemm_sm100.cu).
bool encode_x_map(CUtensorMap *map, const GemmParams &p);

// The CTA-pair form of the GEMM (tlc_gemm_pair.cu): persistent clusters of two CTAs, one
// tcgen05.mma.cta_group::2 tile of 256 activation rows x 256 weight rows per cluster.
// `sw`: the SiLU.mul pair (w = gate, w2 = up).  TLC_ERR_INVALID_OPERATION when the shape
// cannot take this form; the caller then uses the single-CTA kernel.
bool cta_pair_eligible(const tlc_ctx *ctx, const GemmParams &p);
int32_t launch_cta_pair(tlc_ctx *ctx, const GemmParams &p, int type, bool sw);

}  // namespace tlc_gemm
