// Fused dequant-GEMV for decode-sized activations (M <= 16) over weights kept
// as GGUF Q4_0 / Q8_0 blocks in 16-row tiles (tlc_tile.cuh).
//
// Takes the place of the dense f16 kernels the reference runs after
// dequantizing at load time (matmul_transposed_b_tiled_f16,
// shaders/unified.metal:4226-4347, dispatched from src/ops/matmul.rs:314-458)
// and of the separate rms_norm / rope / sigmoid / mul / add launches around
// them in the TL scripts (debug/chat_demo_with_kvcache.tl:219-290).
//
// Design (the weight bytes are read from HBM exactly once):
//   * persistent CTAs, up to two per SM, each walking 16-row slabs of the weight(s);
//   * a producer warp streams the tiles of a slab into a shared memory ring,
//     ONE bulk async copy of up to 18 KB per stage (a stage's 16 tiles are
//     contiguous in HBM), completing on mbarriers -- no thread ever issues a
//     narrow global load for weight data, and the ring keeps tens of KB per SM
//     in flight independent of occupancy;
//   * eight consumer warps read their fragment words with two conflict-free
//     16-byte shared loads per tile and unpack nibbles / bytes in registers
//     straight into f16 tensor-core fragments: a 4-bit (8-bit) integer n placed
//     in the low mantissa bits of a binary16 is the subnormal n * 2^-24, so one
//     AND per pair of weights yields an exact A fragment; the -8 (-128) offset is
//     carried by the accumulator's initial value (-8 * sum of the 32
//     activations of the block) and the block scale d multiplies the 16x8 block
//     result in f32;  mma.sync m16n8k16 with f32 accumulation does the dot
//     products for up to 8 activation rows at no extra cost;
//   * the K range of a slab is split over the eight warps, reduced through
//     shared memory (up to four slabs per reduction), and the epilogue (f16 rounding, bias / residual add,
//     SiLU(gate)*up, interleaved RoPE) is applied before the single store.
// The activation vector(s) are optionally RMS-normalised on the way into
// shared memory, where they are kept pre-permuted in fragment order.
#include <cuda_fp16.h>

#include "tlc_gemv_kernel.cuh"
#include "tlc_internal.h"
#include "tlc_tile.cuh"

using namespace tlc_gemv;

namespace {

// ---------------------------------------------------------------------------
// Generic path for dense f16 weights: any M, no alignment assumptions.  One
// warp per output row -- correct but far from the roofline.
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

// ---------------------------------------------------------------------------
// Dense f16 weights (F16 / F32 files, Q6_K after its load-time dequantization,
// tied embeddings): one warp per output row, 16-byte loads of the row and of up
// to 8 activation rows, f32 accumulation, optional bias / residual.  HBM-bound
// on the 2 bytes per weight; K must be a multiple of 8 and rows 16-byte aligned.
// ---------------------------------------------------------------------------
template <int MR>
__global__ void __launch_bounds__(256) linear_f16_kernel(const uint8_t *__restrict__ w, size_t pitch, int n_rows,
                                                         int k, const __half *__restrict__ x, int m,
                                                         __half *__restrict__ y, const __half *__restrict__ bias,
                                                         const __half *__restrict__ residual) {
    tlc_pdl_prologue();
    const int row = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (row >= n_rows) return;
    const uint4 *wr = reinterpret_cast<const uint4 *>(w + (size_t)row * pitch);
    const int steps = k >> 3;  // 16-byte pieces per row
    float acc[MR];
#pragma unroll
    for (int i = 0; i < MR; i++) acc[i] = 0.f;
#pragma unroll 4
    for (int s = lane; s < steps; s += 32) {
        const uint4 wv = __ldg(wr + s);
        const __half2 *wh = reinterpret_cast<const __half2 *>(&wv);
        float2 wf[4];
#pragma unroll
        for (int j = 0; j < 4; j++) wf[j] = __half22float2(wh[j]);
#pragma unroll
        for (int i = 0; i < MR; i++) {
            if (i < m) {
                const uint4 xv = *(reinterpret_cast<const uint4 *>(x + (size_t)i * k) + s);
                const __half2 *xh = reinterpret_cast<const __half2 *>(&xv);
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    const float2 xf = __half22float2(xh[j]);
                    acc[i] = fmaf(wf[j].x, xf.x, acc[i]);
                    acc[i] = fmaf(wf[j].y, xf.y, acc[i]);
                }
            }
        }
    }
#pragma unroll
    for (int i = 0; i < MR; i++) {
        if (i < m) {
            float v = acc[i];
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
            if (lane == 0) {
                __half h = __float2half_rn(v);
                if (bias) h = __hadd(h, bias[row]);
                if (residual) h = __hadd(h, residual[(size_t)i * n_rows + row]);
                y[(size_t)i * n_rows + row] = h;
            }
        }
    }
}

// ---------------------------------------------------------------------------
// Q6_K weights kept quantized (stock Q4_0 GGUF files store output.weight, the largest
// linear of a decode step, as Q6_K: GGUFLoader::dequantize_q6_k, src/model/formats/gguf.rs:
// 128-218).  One warp per output row over rows of 224-byte padded super-blocks (tlc_qtensor.cu);
// sixteen lanes share a super-block: lane (half h, quarter q) takes l = 4q .. 4q+3 of half h,
// i.e. one 32-bit word each of ql[l], ql[l+32], qh[l] and from them the sixteen weights
// l, l+32, l+64, l+96.  The four 6-bit values of a word are put together with byte-wise integer
// operations, turned into exact f16 (1024 + q, minus 1056) and accumulated in f32 against up to
// MR activation rows held in shared memory; the group's scale d * sc multiplies the group's sum.
// HBM-bound on 0.875 bytes per weight (the f16 copy the reference keeps costs 2).
// ---------------------------------------------------------------------------
template <int MR>
__global__ void __launch_bounds__(256) linear_q6k_kernel(const uint8_t *__restrict__ w, size_t pitch, int n_rows, int k,
                                                         const __half *__restrict__ x, int m, __half *__restrict__ y,
                                                         const __half *__restrict__ bias,
                                                         const __half *__restrict__ residual) {
    extern __shared__ __align__(16) uint8_t q6_smem[];
    __half *xs = reinterpret_cast<__half *>(q6_smem);  // [m][k]
    tlc_pdl_prologue();
    for (int i = threadIdx.x * 8; i < m * k; i += blockDim.x * 8)
        *reinterpret_cast<uint4 *>(xs + i) = *reinterpret_cast<const uint4 *>(x + i);
    __syncthreads();
    const int row = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (row >= n_rows) return;
    const int sub = lane & 15, h = sub >> 3, q = sub & 7, is = q >> 2;
    const int n_sb = k >> 8;
    float acc[MR];
#pragma unroll
    for (int i = 0; i < MR; i++) acc[i] = 0.f;
    const __half2 bias1056 = __float2half2_rn(1056.0f);  // 1024 (the magic exponent) + 32 (the offset of q)
    for (int sb = lane >> 4; sb < n_sb; sb += 2) {
        const uint8_t *blk = w + (size_t)row * pitch + (size_t)sb * 224;
        const uint32_t qa = *reinterpret_cast<const uint32_t *>(blk + 64 * h + 4 * q);
        const uint32_t qb = *reinterpret_cast<const uint32_t *>(blk + 64 * h + 32 + 4 * q);
        const uint32_t qh = *reinterpret_cast<const uint32_t *>(blk + 128 + 32 * h + 4 * q);
        const uint2 scw = *reinterpret_cast<const uint2 *>(blk + 192 + 8 * h);
        const float d = __half2float(*reinterpret_cast<const __half *>(blk + 208));
        // group j (elements l + 32 j): four 6-bit values in the four bytes of a word
        uint32_t qv[4];
        qv[0] = (qa & 0x0F0F0F0Fu) | ((qh & 0x03030303u) << 4);
        qv[1] = (qb & 0x0F0F0F0Fu) | (((qh >> 2) & 0x03030303u) << 4);
        qv[2] = ((qa >> 4) & 0x0F0F0F0Fu) | (((qh >> 4) & 0x03030303u) << 4);
        qv[3] = ((qb >> 4) & 0x0F0F0F0Fu) | (((qh >> 6) & 0x03030303u) << 4);
        const uint32_t scs[2] = {scw.x, scw.y};
#pragma unroll
        for (int j = 0; j < 4; j++) {
            // bytes (b0, b1 | b2, b3) -> f16 pairs 1024 + b, then - 1056: exactly q - 32
            const uint32_t p01 = __byte_perm(qv[j], 0x64646464u, 0x4140), p23 = __byte_perm(qv[j], 0x64646464u, 0x4342);
            const float2 w01 = __half22float2(__hsub2(*reinterpret_cast<const __half2 *>(&p01), bias1056));
            const float2 w23 = __half22float2(__hsub2(*reinterpret_cast<const __half2 *>(&p23), bias1056));
            const int sidx = is + 2 * j;  // scale of this group: byte sidx of the half's eight
            const float scale = d * (float)(int8_t)((scs[sidx >> 2] >> (8 * (sidx & 3))) & 0xFF);
            const int e0 = sb * 256 + 128 * h + 4 * q + 32 * j;
#pragma unroll
            for (int i = 0; i < MR; i++) {
                if (i < m) {
                    const uint2 xr = *reinterpret_cast<const uint2 *>(xs + (size_t)i * k + e0);
                    const float2 x01 = __half22float2(*reinterpret_cast<const __half2 *>(&xr.x));
                    const float2 x23 = __half22float2(*reinterpret_cast<const __half2 *>(&xr.y));
                    const float s = fmaf(w01.x, x01.x, fmaf(w01.y, x01.y, fmaf(w23.x, x23.x, w23.y * x23.y)));
                    acc[i] = fmaf(scale, s, acc[i]);
                }
            }
        }
    }
#pragma unroll
    for (int i = 0; i < MR; i++) {
        if (i < m) {
            float v = acc[i];
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
            if (lane == 0) {
                __half hv = __float2half_rn(v);
                if (bias) hv = __hadd(hv, bias[row]);
                if (residual) hv = __hadd(hv, residual[(size_t)i * n_rows + row]);
                y[(size_t)i * n_rows + row] = hv;
            }
        }
    }
}

// Second half of a split-K launch (GemvParams::ksplit > 1): one thread per output adds the K
// windows' f32 shares in window order (so the result does not depend on scheduling) and applies
// the epilogue of gemv_mma_kernel -- f16 rounding, then bias / residual / SiLU(gate)*up /
// interleaved RoPE, dense or (sequence, position) addressing.
__global__ void __launch_bounds__(256) gemv_splitk_finish_kernel(const GemvParams p) {
    tlc_pdl_prologue();
    const int nout = p.subs == 2 ? p.t[0].n : p.ntot;
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (size_t)p.m * nout) return;
    const int col = (int)(i / nout), nn = (int)(i % nout);
    int ti = 0, n = nn;
    if (p.subs == 1) {
        if (n >= p.t[0].n) { n -= p.t[0].n; ti = 1; }
        if (ti == 1 && n >= p.t[1].n) { n -= p.t[1].n; ti = 2; }
    }
    const int noff = nn - n;
    auto sum = [&](int off) {
        float v = 0.f;
#pragma unroll 4
        for (int w = 0; w < p.ksplit; w++) v += p.partial[((size_t)w * p.m + col) * p.ntot + off];
        return v;
    };
    const int wn = ti == 0 ? p.t[0].n : ti == 1 ? p.t[1].n : p.t[2].n;
    __half *yout = ti == 0 ? p.t[0].y : ti == 1 ? p.t[1].y : p.t[2].y;
    const long long rstride = ti == 0 ? p.t[0].row_stride : ti == 1 ? p.t[1].row_stride : p.t[2].row_stride;
    const long long pstride = ti == 0 ? p.t[0].pos_stride : ti == 1 ? p.t[1].pos_stride : p.t[2].pos_stride;
    const int rheads = ti == 0 ? p.t[0].rope_heads : ti == 1 ? p.t[1].rope_heads : p.t[2].rope_heads;
    const int hdim = ti == 0 ? p.t[0].head_dim : ti == 1 ? p.t[1].head_dim : p.t[2].head_dim;
    __half h = __float2half_rn(sum(noff + n));
    const size_t oidx = (size_t)col * wn + n;
    const int pos = p.positions ? p.positions[col] : p.pos_offset + col;
    const size_t yidx = (size_t)((long long)col * rstride + (long long)pos * pstride) + n;
    if (pstride != 0 && p.max_pos > 0 && (pos < 0 || pos >= p.max_pos)) {
        if (atomicCAS(&p.status->code, 0, TLC_DEV_INDEX) == 0) p.status->where = 302;
        return;
    }
    if (rheads > 0) {
        const __half hp = __float2half_rn(sum(noff + (n ^ 1)));
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
        yout[yidx] = __hadd(h, p.residual[oidx]);
    } else if (p.epilogue == TLC_EPI_SWIGLU) {
        const __half up = __float2half_rn(sum(p.t[0].n + n));
        const __half sg = __float2half_rn(1.0f / (1.0f + expf(-__half2float(h))));
        p.t[0].y[oidx] = __hmul(__hmul(h, sg), up);
    } else {
        if (p.bias) h = __hadd(h, p.bias[n]);
        yout[yidx] = h;
    }
}

template <int QT, int NT, int AS, bool M1, int CW, bool F8 = false>
int32_t launch_mma_as(tlc_ctx *ctx, GemvParams &p, int grid, size_t smem) {
    static bool configured[64] = {};
    if (!configured[ctx->device & 63]) {
        TLC_CUDA(cudaFuncSetAttribute(gemv_mma_kernel<QT, NT, AS, M1, CW, F8>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      (int)ctx->prop.sharedMemPerBlockOptin));
        TLC_CUDA(cudaFuncSetAttribute(gemv_mma_kernel<QT, NT, AS, M1, CW, F8>,
                                      cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared));
        configured[ctx->device & 63] = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)grid);
    cfg.blockDim = dim3((CW + 1) * 32);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = ctx->stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = ctx->use_pdl ? 1 : 0;
    cudaError_t le = cudaLaunchKernelEx(&cfg, gemv_mma_kernel<QT, NT, AS, M1, CW, F8>, p);
    if (le != cudaSuccess) {
        cudaGetLastError();
        return tlc_fail(TLC_ERR_CUDA, "gemv launch failed: %s", cudaGetErrorString(le));
    }
    TLC_CHECK_LAUNCH(ctx);
    return TLC_OK;
}

template <int QT, int NT, int CW>
int32_t launch_mma_cw(tlc_ctx *ctx, GemvParams &p, int grid, size_t smem, int as, bool f8) {
    if constexpr (NT == 1 && QT == TLC_TYPE_Q4_0) {
        if (p.m == 1 && f8) {  // one sequence, Q4_0: the FP8-limb form of the dot products
            if (as == 1) return launch_mma_as<QT, 1, 1, true, CW, true>(ctx, p, grid, smem);
            if (as == 2) return launch_mma_as<QT, 1, 2, true, CW, true>(ctx, p, grid, smem);
            return launch_mma_as<QT, 1, 4, true, CW, true>(ctx, p, grid, smem);
        }
    }
    if constexpr (NT == 1) {
        if (p.m == 1) {  // the decode step of one sequence
            if (as == 1) return launch_mma_as<QT, 1, 1, true, CW>(ctx, p, grid, smem);
            if (as == 2) return launch_mma_as<QT, 1, 2, true, CW>(ctx, p, grid, smem);
            return launch_mma_as<QT, 1, 4, true, CW>(ctx, p, grid, smem);
        }
    }
    if (as == 1) return launch_mma_as<QT, NT, 1, false, CW>(ctx, p, grid, smem);
    if (as == 2) return launch_mma_as<QT, NT, 2, false, CW>(ctx, p, grid, smem);
    return launch_mma_as<QT, NT, 4, false, CW>(ctx, p, grid, smem);
}

template <int QT, int NT>
int32_t launch_mma(tlc_ctx *ctx, GemvParams &p) {
    using T = QTraits<QT>;
    constexpr size_t STAGE_BYTES = (size_t)kTilesPerStage * T::TILE_BYTES;
    const size_t budget = (size_t)ctx->prop.sharedMemPerBlockOptin;
    // One activation row of a Q4_0 weight runs on the FP8 form (option "gemv_f8"), as long as its
    // limbs (128 bytes per block) leave room for the ring.
    bool f8 = QT == TLC_TYPE_Q4_0 && NT == 1 && p.m == 1 && ctx->gemv_f8;
    if (f8 && fixed_smem_bytes(p.nblk_pad, p.m, NT, p.subs, 8, true) + 3 * STAGE_BYTES > budget) f8 = false;
    auto fixed_smem_bytes = [f8](int nblk_pad, int m, int nt, int as, int cw = 8) {
        return tlc_gemv::fixed_smem_bytes(nblk_pad, m, nt, as, cw, f8);
    };
    const size_t fixed1 = fixed_smem_bytes(p.nblk_pad, p.m, NT, p.subs);
    TLC_REQUIRE(fixed1 + 2 * STAGE_BYTES <= budget, TLC_ERR_INVALID_OPERATION,
                "gemv: activations of %d x %d do not fit in shared memory", p.m, p.k);
    // Two CTAs per SM (16 consumer warps hide the shared-memory and MMA latency
    // of the unpack loop) whenever the activations leave room for at least
    // three ring stages in half of the SM's shared memory.
    const size_t half = (size_t)ctx->prop.sharedMemPerMultiprocessor / 2 - 1024;
    const bool fits_half = fixed1 + 3 * STAGE_BYTES <= half;
    // (Measured on the TinyLlama decode step: keeping small launches at one CTA per
    // SM, to leave room for the next kernel's early CTAs, costs 8 % against
    // letting them spread over two CTAs per SM.)
    const bool two = fits_half;
    // One CTA per SM: sixteen consumer warps instead of eight, if the larger reduction
    // buffers still leave three ring stages.
    const int cw = !two && fixed_smem_bytes(p.nblk_pad, p.m, NT, p.subs, 16) + 3 * STAGE_BYTES <= budget ? 16 : 8;
    const size_t cap = two ? half : budget;
    const int max_ctas = two ? 2 * ctx->sm_count : ctx->sm_count;
    const int ks = p.ksplit > 1 ? p.ksplit : 1;
    // Split K: the CTAs come in groups of ks (one per window); a group shares the slabs.
    int grid = p.total_units * ks < max_ctas ? p.total_units * ks : max_ctas;
    grid -= grid % ks;
    if (grid < ks) grid = ks;
    // Accumulator sets per reduction: enough units for about four ring stages
    // between two cross-warp reductions, as far as this CTA has units and the
    // shared memory (reduction buffers grow with the sets) allows.
    const int units_per_cta = (p.total_units + grid / ks - 1) / (grid / ks);
    const int iters_per_unit = p.subs * p.nchunks;
    int ub = (4 + iters_per_unit - 1) / iters_per_unit;
    if (ub > units_per_cta) ub = units_per_cta;
    int as = p.subs;
    while (as < ub * p.subs && as < (NT == 2 ? 2 : 4)) as *= 2;
    while (as > p.subs && fixed_smem_bytes(p.nblk_pad, p.m, NT, as, cw) + 3 * STAGE_BYTES > cap) as /= 2;
    const size_t smem_fixed = fixed_smem_bytes(p.nblk_pad, p.m, NT, as, cw);
    // No more stages than this CTA will ever fill.
    const long per_cta = (long)units_per_cta * p.subs * p.nchunks;
    int stages = (int)((cap - smem_fixed) / STAGE_BYTES);
    if (stages > kMaxStages) stages = kMaxStages;
    if (stages > per_cta) stages = per_cta < 2 ? 2 : (int)per_cta;
    p.nstages = stages;
    // Mode 4 decides per launch.  A kernel whose CTAs stream eight or more ring stages (40 MB over the
    // grid, about 6 us of HBM time) lets its successor in right after its own dependency wait: the
    // successor is then resident with its ring filled when this grid ends (Llama-70B decode: 10.07 ->
    // 9.74 ms per token).  Shorter kernels keep the late trigger (TinyLlama decode: 2.2 % slower with
    // the early one from three stages on, 0.5 % slower with it everywhere).
    p.pdl_mode = ctx->pdl_mode == 4 ? (per_cta >= 8 ? 3 : 2) : ctx->pdl_mode;
    p.l2_hint = ctx->l2_hint;
    p.contig = units_per_cta <= 4 ? 1 : 0;
    const size_t smem = smem_fixed + (size_t)stages * STAGE_BYTES;
    return cw == 16 ? launch_mma_cw<QT, NT, 16>(ctx, p, grid, smem, as, f8) : launch_mma_cw<QT, NT, 8>(ctx, p, grid, smem, as, f8);
}

size_t gemv_fixed_smem(int nblk_pad, int m, int nt) { return fixed_smem_bytes(nblk_pad, m, nt, 2); }

}  // namespace

// Failure-detection self-test: a CTA waits on an mbarrier that nothing ever
// completes, through the same bounded wait the GEMV uses.  The wait runs out
// after the context's limit, the status word is set and the kernel returns.
namespace {
__global__ void selftest_mbarrier_wait_kernel(tlc_dev_status *status, uint64_t wait_ns) {
    __shared__ uint64_t bar;
    __shared__ int abort_flag;
    if (threadIdx.x == 0) {
        mbar_init(&bar, 1);
        abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    mbar_wait(&bar, 0, &abort_flag, status, 99, wait_ns);
}
}  // namespace

int32_t tlc_selftest_mbarrier_wait(tlc_ctx *ctx) {
    selftest_mbarrier_wait_kernel<<<1, 32, 0, ctx->stream>>>(ctx->dev_status, ctx->wait_ns);
    TLC_CHECK_LAUNCH(ctx);
    return TLC_OK;
}

// Largest number of activation rows one launch can take for this K.
static int gemv_max_m(tlc_ctx *ctx, int type, int k) {
    const int nblk_pad = (int)tlc_tile::k_tiles(type, k) * tlc_tile::tile_blocks(type);
    const size_t budget = (size_t)ctx->prop.sharedMemPerBlockOptin;
    const size_t stage = (size_t)kTilesPerStage * tlc_tile::tile_bytes(type);
    for (int m = 16; m >= 1; m--) {
        int nt = m > 8 ? 2 : 1;
        if (gemv_fixed_smem(nblk_pad, m, nt) + 3 * stage <= budget) return m;
    }
    return 0;
}

// Split K for several activation rows.  The rows sit in shared memory in fragment order, 64 bytes
// per block and row: 8 rows of K = 8192 already take half an SM's shared memory, 16 rows of
// K = 28672 eight times an SM's.  Instead of passing over the weights once per group of rows that
// fits, the K range is cut into windows: every CTA keeps only its window of the rows, the windows'
// f32 partial sums meet in gemv_splitk_finish_kernel.  The weights are read once.
// Returns the number of windows (1: no split) for m rows, of which max_m fit in one unsplit launch.
//  - A launch that runs two CTAs per SM without a split is left alone.
//  - More than four rows that fit one launch at one CTA per SM stay unsplit (sixteen consumer
//    warps; 8 rows of K = 8192: 44 us against 50 us split).
//  - Otherwise the windows are sized for one CTA per SM with sixteen consumer warps (option
//    gemv_splitk = 2, the default: 16 rows of K = 8192 take 76 us, against 120 us with windows
//    for two CTAs per SM and 87 us in two passes), else, or first with gemv_splitk = 1, for two
//    CTAs per SM; a window holds at least eight tiles.
static int gemv_choose_ksplit(tlc_ctx *ctx, int type, int64_t ktiles, int m, int n_sub, int max_m, int mode) {
    const int tb = tlc_tile::tile_blocks(type);
    const size_t stage = (size_t)kTilesPerStage * tlc_tile::tile_bytes(type);
    const size_t half = (size_t)ctx->prop.sharedMemPerMultiprocessor / 2 - 1024;
    const size_t budget = (size_t)ctx->prop.sharedMemPerBlockOptin;
    const int nt = m > 8 ? 2 : 1;
    auto fits = [&](int64_t win, bool two) {
        return fixed_smem_bytes((int)win * tb, m, nt, n_sub, two ? 8 : 16) + 3 * stage <= (two ? half : budget);
    };
    if (fits(ktiles, true)) return 1;
    const bool multi_pass = m > max_m;
    if (!multi_pass && m > 4) return 1;
    static const int cand[] = {2, 3, 4, 6, 8, 12, 16, 24, 32};
    for (int round = 0; round < 2; round++) {
        const bool two = (round == 0) != (mode == 2);
        if (!two && !multi_pass) continue;  // one CTA per SM is what the unsplit launch already does
        for (int ks : cand) {
            const int64_t win = (ktiles + ks - 1) / ks;
            if (win < 8) break;
            if (fits(win, two)) return ks;
        }
    }
    return 1;
}

// Bytes of context scratch a fused linear over m rows of width k with n_total outputs may need
// (the split-K partial sums); callers that capture graphs reserve it up front.
size_t tlc_gemv_scratch_bytes(tlc_ctx *ctx, int type, int64_t k, int m, int64_t n_total) {
    if ((type != TLC_TYPE_Q4_0 && type != TLC_TYPE_Q8_0) || m < 2 || m > 16) return 0;
    const int max_m = gemv_max_m(ctx, type, (int)k);
    int ks = 1;
    for (int mode = 1; mode <= 2; mode++)  // whatever the option says at launch time
        for (int n_sub = 1; n_sub <= 2; n_sub++) {
            const int c = gemv_choose_ksplit(ctx, type, tlc_tile::k_tiles(type, k), m, n_sub, max_m, mode);
            ks = c > ks ? c : ks;
        }
    return ks > 1 ? (size_t)ks * m * (size_t)n_total * sizeof(float) : 0;
}

int32_t tlc_gemv_splitk_finish(tlc_ctx *ctx, const tlc_gemv_args &a, int ksplit, float *partial) {
    GemvParams p{};
    p.n_out = a.n_out;
    p.ntot = 0;
    for (int i = 0; i < a.n_out; i++) {
        const tlc_qtensor *w = a.outs[i].w;
        p.t[i].n = (int)w->n_rows;
        p.t[i].row_stride = a.outs[i].row_stride >= 0 ? a.outs[i].row_stride : (long long)w->n_rows;
        p.t[i].pos_stride = a.outs[i].pos_stride;
        p.t[i].y = static_cast<__half *>(a.outs[i].y);
        p.t[i].rope_heads = a.outs[i].rope_heads;
        p.t[i].head_dim = a.outs[i].rope_heads > 0 ? (int)(w->n_rows / a.outs[i].rope_heads) : 0;
        p.ntot += p.t[i].n;
    }
    p.subs = a.epilogue == TLC_EPI_SWIGLU ? 2 : 1;
    p.m = a.m;
    p.epilogue = a.epilogue;
    p.bias = static_cast<const __half *>(a.bias);
    p.residual = static_cast<const __half *>(a.residual);
    p.pos_offset = a.pos_offset;
    p.rope_base = (float)a.rope_base;
    p.positions = a.positions;
    p.max_pos = a.max_pos;
    p.status = ctx->dev_status;
    p.ksplit = ksplit;
    p.partial = partial;
    const int nout = p.subs == 2 ? p.t[0].n : p.ntot;
    const size_t total = (size_t)a.m * nout;
    cudaError_t le = tlc_launch_pdl(ctx, gemv_splitk_finish_kernel, dim3((unsigned)((total + 255) / 256)), dim3(256), 0, p);
    if (le != cudaSuccess) {
        cudaGetLastError();
        return tlc_fail(TLC_ERR_CUDA, "split-K finish launch failed: %s", cudaGetErrorString(le));
    }
    TLC_CHECK_LAUNCH(ctx);
    return TLC_OK;
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
        // Dense weights: RMSNorm (if asked for) runs as its own kernel, bias and
        // residual are applied in the store; RoPE, SiLU.mul and cache addressing
        // exist on the quantized path only.
        TLC_REQUIRE(a.epilogue != TLC_EPI_SWIGLU && a.n_out == 1 && a.outs[0].rope_heads == 0 &&
                        a.outs[0].row_stride < 0 && a.outs[0].pos_stride == 0,
                    TLC_ERR_INVALID_OPERATION, "fused RoPE / SiLU.mul / cache epilogues need a quantized weight");
        const __half *x = static_cast<const __half *>(a.x);
        if (a.norm_w) {
            if (int32_t rc = tlc_scratch_reserve(ctx, (size_t)a.m * k * 2)) return rc;
            if (int32_t rc = tlc_rms_norm(ctx, a.x, a.norm_w, ctx->scratch, a.m, (int32_t)k, a.eps)) return rc;
            x = static_cast<const __half *>(ctx->scratch);
        }
        const int threads = 256;
        const unsigned grid = (unsigned)((w0->n_rows * 32 + threads - 1) / threads);
        const __half *residual = a.epilogue == TLC_EPI_RESIDUAL ? static_cast<const __half *>(a.residual) : nullptr;
        const bool vec = k % 8 == 0 && w0->row_pitch % 16 == 0 && ((uintptr_t)x % 16) == 0 && ((uintptr_t)w0->data % 16) == 0;
        if (!vec) {
            TLC_REQUIRE(!residual, TLC_ERR_INVALID_OPERATION, "residual epilogue needs 16-byte aligned f16 rows");
            linear_generic_kernel<<<grid, threads, 0, ctx->stream>>>(
                static_cast<const uint8_t *>(w0->data), w0->row_pitch, type, (int)w0->n_rows, (int)k, x, a.m,
                static_cast<__half *>(a.outs[0].y), static_cast<const __half *>(a.bias));
            TLC_CHECK_LAUNCH(ctx);
            return TLC_OK;
        }
        for (int m0 = 0; m0 < a.m; m0 += 8) {
            const int mc = a.m - m0 < 8 ? a.m - m0 : 8;
            cudaError_t le = tlc_launch_pdl(
                ctx, mc <= 2 ? linear_f16_kernel<2> : linear_f16_kernel<8>, dim3(grid), dim3(threads), 0,
                static_cast<const uint8_t *>(w0->data), w0->row_pitch, (int)w0->n_rows, (int)k, x + (size_t)m0 * k, mc,
                static_cast<__half *>(a.outs[0].y) + (size_t)m0 * w0->n_rows, static_cast<const __half *>(a.bias),
                residual ? residual + (size_t)m0 * w0->n_rows : nullptr);
            if (le != cudaSuccess) {
                cudaGetLastError();
                return tlc_fail(TLC_ERR_CUDA, "f16 linear launch failed: %s", cudaGetErrorString(le));
            }
            TLC_CHECK_LAUNCH(ctx);
        }
        return TLC_OK;
    }

    if (type == TLC_TYPE_Q6_K) {
        // Resident Q6_K (one weight per launch; RMSNorm, if asked for, as its own kernel; bias
        // and residual in the store).  More than eight activation rows take further passes.
        TLC_REQUIRE(a.epilogue != TLC_EPI_SWIGLU && a.n_out == 1 && a.outs[0].rope_heads == 0 &&
                        a.outs[0].row_stride < 0 && a.outs[0].pos_stride == 0,
                    TLC_ERR_INVALID_OPERATION, "fused RoPE / SiLU.mul / cache epilogues need a Q4_0 or Q8_0 weight");
        const __half *x = static_cast<const __half *>(a.x);
        if (a.norm_w) {
            if (int32_t rc = tlc_scratch_reserve(ctx, (size_t)a.m * k * 2)) return rc;
            if (int32_t rc = tlc_rms_norm(ctx, a.x, a.norm_w, ctx->scratch, a.m, (int32_t)k, a.eps)) return rc;
            x = static_cast<const __half *>(ctx->scratch);
        }
        TLC_REQUIRE(((uintptr_t)x & 15) == 0, TLC_ERR_INVALID_OPERATION, "linear: activations must be 16-byte aligned");
        const __half *residual = a.epilogue == TLC_EPI_RESIDUAL ? static_cast<const __half *>(a.residual) : nullptr;
        // rows per pass: up to eight, fewer if the activation rows would not fit in shared memory
        int per = 8;
        while (per > 1 && (size_t)per * k * 2 > (size_t)ctx->prop.sharedMemPerBlockOptin - 1024) per >>= 1;
        TLC_REQUIRE((size_t)per * k * 2 <= (size_t)ctx->prop.sharedMemPerBlockOptin - 1024, TLC_ERR_INVALID_OPERATION,
                    "linear: K = %lld too large for the shared-memory staging", (long long)k);
        static bool configured[64] = {};
        if (!configured[ctx->device & 63]) {
            TLC_CUDA(cudaFuncSetAttribute(linear_q6k_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                          (int)ctx->prop.sharedMemPerBlockOptin));
            TLC_CUDA(cudaFuncSetAttribute(linear_q6k_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                          (int)ctx->prop.sharedMemPerBlockOptin));
            TLC_CUDA(cudaFuncSetAttribute(linear_q6k_kernel<8>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                          (int)ctx->prop.sharedMemPerBlockOptin));
            configured[ctx->device & 63] = true;
        }
        const unsigned grid = (unsigned)((w0->n_rows * 32 + 255) / 256);
        for (int m0 = 0; m0 < a.m; m0 += per) {
            const int mc = a.m - m0 < per ? a.m - m0 : per;
            auto kern = mc == 1 ? linear_q6k_kernel<1> : mc <= 4 ? linear_q6k_kernel<4> : linear_q6k_kernel<8>;
            cudaError_t le = tlc_launch_pdl(
                ctx, kern, dim3(grid), dim3(256), (size_t)mc * k * 2, static_cast<const uint8_t *>(w0->data), w0->row_pitch,
                (int)w0->n_rows, (int)k, x + (size_t)m0 * k, mc, static_cast<__half *>(a.outs[0].y) + (size_t)m0 * w0->n_rows,
                static_cast<const __half *>(a.bias), residual ? residual + (size_t)m0 * w0->n_rows : nullptr);
            if (le != cudaSuccess) {
                cudaGetLastError();
                return tlc_fail(TLC_ERR_CUDA, "Q6_K linear launch failed: %s", cudaGetErrorString(le));
            }
            TLC_CHECK_LAUNCH(ctx);
        }
        return TLC_OK;
    }

    if (tlc_gemm_eligible(ctx, a)) return tlc_launch_gemm(ctx, a);

    int max_m = gemv_max_m(ctx, type, (int)k);
    TLC_REQUIRE(max_m >= 1, TLC_ERR_INVALID_OPERATION, "gemv: K = %lld too large for the shared-memory staging",
                (long long)k);
    // Up to 16 rows whose fragments do not leave two CTAs per SM room: one pass with K cut into windows.
    int ksplit = 1;
    if (a.m >= 2 && a.m <= 16 && ctx->gemv_splitk) {
        ksplit = gemv_choose_ksplit(ctx, type, w0->k_tiles, a.m, a.epilogue == TLC_EPI_SWIGLU ? 2 : 1, max_m,
                                    ctx->gemv_splitk);
        if (ksplit > 1) max_m = a.m;
    }
    // Otherwise activation rows beyond what one launch can hold are processed in
    // further passes over the weights.
    for (int m0 = 0; m0 < a.m; m0 += max_m) {
        const int mc = a.m - m0 < max_m ? a.m - m0 : max_m;
        GemvParams p{};
        p.n_out = a.n_out;
        p.total_units = 0;
        for (int i = 0; i < a.n_out; i++) {
            const tlc_qtensor *w = a.outs[i].w;
            p.t[i].w = static_cast<const uint8_t *>(w->data);
            p.t[i].slab_pitch = w->slab_pitch;
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
        p.ktiles = (int)w0->k_tiles;
        p.nblk_pad = p.ktiles * tlc_tile::tile_blocks(type);
        p.nchunks = (p.ktiles + kTilesPerStage - 1) / kTilesPerStage;
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
        p.max_pos = a.max_pos;
        p.status = ctx->dev_status;
        p.wait_ns = ctx->wait_ns;
        if (ksplit > 1) {
            p.ksplit = ksplit;
            p.ktiles_full = p.ktiles;
            p.ktiles_win = (p.ktiles + ksplit - 1) / ksplit;
            p.ntot = 0;
            for (int i = 0; i < a.n_out; i++) p.ntot += p.t[i].n;
            // what the launcher sizes shared memory, stages and batches by: one window
            p.ktiles = p.ktiles_win;
            p.nblk_pad = p.ktiles_win * tlc_tile::tile_blocks(type);
            p.nblk = p.nblk_pad;
            p.nchunks = (p.ktiles_win + kTilesPerStage - 1) / kTilesPerStage;
            const size_t need = (size_t)ksplit * mc * (size_t)p.ntot * sizeof(float);
            if (int32_t rc = tlc_scratch_reserve(ctx, need)) return rc;
            p.partial = static_cast<float *>(ctx->scratch);
        }
        const int nt = mc > 8 ? 2 : 1;
        int32_t rc;
        if (type == TLC_TYPE_Q4_0)
            rc = nt == 1 ? launch_mma<TLC_TYPE_Q4_0, 1>(ctx, p) : launch_mma<TLC_TYPE_Q4_0, 2>(ctx, p);
        else
            rc = nt == 1 ? launch_mma<TLC_TYPE_Q8_0, 1>(ctx, p) : launch_mma<TLC_TYPE_Q8_0, 2>(ctx, p);
        if (rc) return rc;
        if (ksplit > 1) {
            const int nout = p.subs == 2 ? p.t[0].n : p.ntot;
            const size_t total = (size_t)mc * nout;
            cudaError_t le = tlc_launch_pdl(ctx, gemv_splitk_finish_kernel, dim3((unsigned)((total + 255) / 256)), dim3(256), 0, p);
            if (le != cudaSuccess) {
                cudaGetLastError();
                return tlc_fail(TLC_ERR_CUDA, "split-K finish launch failed: %s", cudaGetErrorString(le));
            }
            TLC_CHECK_LAUNCH(ctx);
        }
    }
    return TLC_OK;
}
