// CTA-pair form of the tcgen05 dequant-GEMM: y[M, N] = x[M, K] . W[N, K]^T with W in GGUF
// Q4_0 / Q8_0 blocks (same arithmetic and operand layout as tlc_gemm_kernel.cuh describes).
//
// A cluster of two CTAs (two SMs) computes one 256 x 256 tile with
// tcgen05.mma.cta_group::2: CTA r of the pair holds 128 activation rows (its half of M)
// and 128 weight rows (its half of N) of every K step in its own shared memory, and the
// accumulator of its 128 activation rows x 256 columns in its own tensor memory.  Against
// the single-CTA kernel each SM dequantizes and stores half as many weight rows per MMA
// and the tensor core reads a third less shared memory per flop.
//
// The kernel is persistent: a cluster walks tiles cluster_id, cluster_id + n_clusters, ...
// (activation-row tiles fastest, so clusters that run together share weight rows in L2).
// Tensor memory holds two accumulators of 256 columns; the MMAs of tile j+1 run while the
// epilogue warps drain tile j.  Roles of the 14 warps of a CTA:
//   warp 0       one thread issues the TMA copies of the CTA's activation tile
//                (128 rows x 64 columns, 128-byte swizzle, zero fill outside);
//   warp 1       tensor-memory allocation; in the leader CTA (rank 0) one thread issues
//                the MMAs and commits; in the peer CTA the warp forwards "stage full" to
//                the leader;
//   warps 2-9    weight producers: thread r of a group dequantizes row r of the CTA's
//                128 weight rows; warps 2-5 fill the even K steps, warps 6-9 the odd ones;
//   warps 10-13  epilogue: tcgen05.ld, f16 rounding, RoPE / bias / residual / SiLU.mul, store.
// Hand-overs are mbarriers: full[s] (TMA bytes + 4 producer warps, per CTA), pfull[s]
// (peer -> leader), empty[s] and acc_full[b] (tcgen05.commit, multicast to both CTAs),
// acc_empty[b] (the eight epilogue warps of the pair -> leader).  Every wait is bounded; a
// wait that runs out sets the status word, the role leaves its loop, and both CTAs meet at
// the cluster barrier before tensor memory is freed.
//
// Measured (B200, Q4_0, 8192 x 8192, M = 2048): 378 us = 728 TFLOP/s, against 220 us = 1246
// TFLOP/s of the single-CTA 256 x 256 kernel with TMA-fed activation tiles, so the option
// "gemm_pair" is OFF by default.  Both forms move the same bytes from L2 per flop (128 + 128
// operand rows per 128 x 256 outputs and SM against 256 + 256 per 256 x 256); what the pair
// adds is a hand-over chain across two SMs per ring stage (commit -> both CTAs' producers ->
// forwarder -> leader) that six stages of 0.3 us do not cover: with the weight math compiled
// out the time does not move (395 us), without the activation copies 287 us, without both
// 254 us; polling the barriers without suspending changes nothing.  TMA copies signal the barrier of the CTA they write to (the .cta_group::2 form of
// the copy, which would signal the leader directly, is not used in this code base).
#include <cuda.h>

#include "tlc_gemm_kernel.cuh"

using namespace tlc_gemm;

namespace {

constexpr int kPairThreads = 448;
constexpr int kPairStages = 6;
constexpr int kTileBytes = 128 * 128;                 // 128 rows of one 64-wide K step
constexpr int kPairStageBytes = 2 * kTileBytes;       // activation tile + weight tile
constexpr size_t kPairSmem = 1024 + (size_t)kPairStages * kPairStageBytes + 512;
constexpr uint32_t kAccCols = 256;

__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// Arrive on the barrier at the same shared-memory offset in CTA `cta` of the cluster.
__device__ __forceinline__ void mbar_arrive_remote(uint64_t *bar, uint32_t cta) {
    asm volatile(
        "{\n .reg .b32 ra;\n mapa.shared::cluster.u32 ra, %0, %1;\n"
        " mbarrier.arrive.release.cluster.shared::cluster.b64 _, [ra];\n}\n" ::"r"(smem_u32(bar)),
        "r"(cta)
        : "memory");
}
__device__ __forceinline__ bool mbar_try_wait_cluster(uint64_t *bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n .reg .pred p;\n mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n"
        " selp.u32 %0, 1, 0, p;\n}\n"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait on a barrier another CTA of the cluster arrives on.
__device__ __forceinline__ bool mbar_wait_cluster(uint64_t *bar, uint32_t parity, volatile int *abort_flag,
                                                  tlc_dev_status *status, int where, uint64_t wait_ns) {
    if (mbar_try_wait_cluster(bar, parity)) return true;
    const uint64_t limit = *abort_flag ? 20000ull : wait_ns;
    const uint64_t t0 = tlc_globaltimer_ns();
    do {
        if (mbar_try_wait_cluster(bar, parity)) return true;
    } while (tlc_globaltimer_ns() - t0 < limit);
    *abort_flag = 1;
    if (atomicCAS(&status->code, 0, 2) == 0) status->where = where;
    return false;
}
// M = 256 over the CTA pair, N = n, f16 x f16 -> f32, both operands K-major.
__host__ __device__ constexpr uint32_t idesc_pair(int n) {
    return (1u << 4) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(256 >> 4) << 24);
}
__device__ __forceinline__ void umma_f16_pair(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                              uint32_t accumulate) {
    asm volatile(
        "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
        " tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n}\n" ::"r"(tmem_d),
        "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// Arrives on `bar` (same offset) in both CTAs of the pair once the MMAs issued so far are done.
__device__ __forceinline__ void umma_commit_pair(uint64_t *bar) {
    const uint16_t mask = 3;
    asm volatile(
        "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(
            smem_u32(bar)),
        "h"(mask)
        : "memory");
}

template <int QT, bool SW>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kPairThreads, 1)
    gemm_pair_kernel(const GemmParams p, const __grid_constant__ CUtensorMap x_map) {
    constexpr int S = kPairStages;
    constexpr int OUT_COLS = SW ? 128 : 256;  // output columns of a cluster tile
    constexpr uint32_t IDESC = idesc_pair(256);
    constexpr int TILE = QT == TLC_TYPE_Q4_0 ? 1152 : 1088;

    extern __shared__ uint8_t smem_raw[];
    uint8_t *tiles = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint64_t *full = reinterpret_cast<uint64_t *>(tiles + (size_t)S * kPairStageBytes);
    uint64_t *pfull = full + S;
    uint64_t *empty = pfull + S;
    uint64_t *acc_full = empty + S;
    uint64_t *acc_empty = acc_full + 2;
    uint64_t *done_bar = acc_empty + 2;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(done_bar + 1);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t rank = cluster_ctarank();
    const int cluster_id = blockIdx.x >> 1, n_clusters = gridDim.x >> 1;
    const int KT = (p.k + kBK - 1) / kBK;
    const int m_tiles = (p.m + 255) / 256, n_tiles = (p.n + OUT_COLS - 1) / OUT_COLS;
    const int total = m_tiles * n_tiles;
    const int my_tiles = cluster_id < total ? (total - cluster_id + n_clusters - 1) / n_clusters : 0;

    if (tid == 0) {
        for (int s = 0; s < S; s++) {
            mbar_init(&full[s], 1 + 4);  // arrive.expect_tx of the TMA issuer + the four producer warps of the step
            mbar_init(&pfull[s], 1);
            mbar_init(&empty[s], 1);
        }
        for (int b = 0; b < 2; b++) {
            mbar_init(&acc_full[b], 1);
            mbar_init(&acc_empty[b], 8);  // four epilogue warps in each CTA of the pair
        }
        mbar_init(done_bar, 1);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                     "r"(512u)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();  // the peer's barriers exist before anything arrives on them
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    tlc_pdl_prologue();  // x (and residual) come from the previous kernel of the stream

    if (warp == 0) {
        // ------------------------------ activation tile by TMA ------------------------------
        if (lane == 0) {
            asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&x_map)) : "memory");
            int s = 0;
            uint32_t ph = 0;
            bool ok = true;
            for (int j = 0; j < my_tiles && ok; j++) {
                const int t = cluster_id + j * n_clusters;
                const int m0 = (t % m_tiles) * 256 + 128 * (int)rank;
                for (int kt = 0; kt < KT; kt++) {
                    if (!mbar_wait(&empty[s], ph ^ 1u, abort_flag, p.status, 21, p.wait_ns)) {
                        ok = false;
                        break;
                    }
                    mbar_arrive_expect_tx(&full[s], kTileBytes);
                    tma_load_2d(smem_u32(tiles + (size_t)s * kPairStageBytes), &x_map, kt * kBK, m0,
                                smem_u32(&full[s]));
                    if (++s == S) {
                        s = 0;
                        ph ^= 1u;
                    }
                }
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        // ------------------------------ MMA issuer / forwarder ------------------------------
        int s = 0;
        uint32_t ph = 0;
        bool ok = true;
        if (rank == 0) {
            for (int j = 0; j < my_tiles && ok; j++) {
                const int b = j & 1;
                // the epilogue warps of both CTAs have drained this accumulator (two tiles ago)
                ok = __all_sync(0xffffffffu, mbar_wait_cluster(&acc_empty[b], (((uint32_t)j >> 1) & 1u) ^ 1u, abort_flag,
                                                               p.status, 22, p.wait_ns));
                if (!ok) break;
                tc_fence_after();
                for (int kt = 0; kt < KT; kt++) {
                    const bool mine = mbar_wait(&full[s], ph, abort_flag, p.status, 23, p.wait_ns);
                    const bool theirs = mine && mbar_wait_cluster(&pfull[s], ph, abort_flag, p.status, 24, p.wait_ns);
                    ok = __all_sync(0xffffffffu, mine && theirs);
                    if (!ok) break;
                    tc_fence_after();
                    if (lane == 0) {
                        const uint32_t a_addr = smem_u32(tiles + (size_t)s * kPairStageBytes);
                        const uint32_t b_addr = a_addr + kTileBytes;
#pragma unroll
                        for (int k16 = 0; k16 < kBK / 16; k16++)
                            umma_f16_pair(tmem_base + kAccCols * b, make_desc(a_addr + k16 * 32),
                                          make_desc(b_addr + k16 * 32), IDESC, (kt > 0 || k16 > 0) ? 1u : 0u);
                        umma_commit_pair(&empty[s]);  // both CTAs may refill the stage once these MMAs have read it
                    }
                    __syncwarp();
                    if (++s == S) {
                        s = 0;
                        ph ^= 1u;
                    }
                }
                if (ok && lane == 0) umma_commit_pair(&acc_full[b]);
                __syncwarp();
            }
            if (lane == 0) umma_commit_pair(done_bar);
            __syncwarp();
        } else {
            const int steps = my_tiles * KT;
            for (int q = 0; q < steps; q++) {
                ok = __all_sync(0xffffffffu, mbar_wait(&full[s], ph, abort_flag, p.status, 25, p.wait_ns));
                if (!ok) break;
                if (lane == 0) mbar_arrive_remote(&pfull[s], 0);
                __syncwarp();
                if (++s == S) {
                    s = 0;
                    ph ^= 1u;
                }
            }
        }
    } else if (warp < 10) {
        // ------------------------------ weight producers ------------------------------
        const int group = (warp - 2) >> 2;      // 0: even K steps of the cluster's walk, 1: odd
        const int row = (tid - 64) & 127;       // row of the CTA's weight tile
        const int r16 = row & 15;
        const uint8_t *wbase = SW && rank == 1 ? p.w2 : p.w;
        const int row_in_tile = SW ? row : 128 * (int)rank + row;
        const uint32_t qoff = (uint32_t)((r16 >> 3) * 512 + (r16 & 7) * 64);
        const uint32_t soff = 1024u + (uint32_t)r16 * (QT == TLC_TYPE_Q4_0 ? 8u : 4u);
        uint32_t piece[8];
#pragma unroll
        for (int j = 0; j < 8; j++) piece[j] = (uint32_t)(row * 128 + ((j ^ (row & 7)) << 4));
        const int steps = my_tiles * KT;
        constexpr int PF = 2;                            // own steps fetched ahead
        constexpr int QW = QT == TLC_TYPE_Q4_0 ? 8 : 16;  // quant words of a row per K step
        uint32_t qn[PF][QW], sn[PF];
        // quants and scales of this thread's row for step q of the walk
        auto fetch = [&](int q, uint32_t (&qw)[QW], uint32_t &sc) {
            const int j = q / KT, kt = q - j * KT;
            const int t = cluster_id + j * n_clusters;
            const int wrow = (t / m_tiles) * OUT_COLS + row_in_tile;
            const int wt = QT == TLC_TYPE_Q4_0 ? kt >> 1 : kt;
            const bool ok = q < steps && wrow < p.n && wt < p.k_tiles;
            const uint8_t *tile = wbase + (size_t)(ok ? wrow >> 4 : 0) * p.w_pitch + (size_t)(ok ? wt : 0) * TILE;
            if (QT == TLC_TYPE_Q4_0) {
                const int half = kt & 1;  // which pair of the tile's four blocks
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    const uint2 v = ok ? __ldg(reinterpret_cast<const uint2 *>(tile + qoff + 16 * i + 8 * half))
                                       : make_uint2(0, 0);
                    qw[2 * i] = v.x;
                    qw[2 * i + 1] = v.y;
                }
                sc = ok ? __ldg(reinterpret_cast<const uint32_t *>(tile + soff + 4 * half)) : 0u;
            } else {
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    const uint4 v = ok ? __ldg(reinterpret_cast<const uint4 *>(tile + qoff) + i) : make_uint4(0, 0, 0, 0);
                    qw[4 * i] = v.x;
                    qw[4 * i + 1] = v.y;
                    qw[4 * i + 2] = v.z;
                    qw[4 * i + 3] = v.w;
                }
                sc = ok ? __ldg(reinterpret_cast<const uint32_t *>(tile + soff)) : 0u;
            }
        };
#pragma unroll
        for (int u = 0; u < PF; u++) fetch(group + 2 * u, qn[u], sn[u]);
        bool ok = true;
#pragma unroll 1
        for (int base = group; base < steps && ok; base += 2 * PF) {
#pragma unroll
            for (int u = 0; u < PF; u++) {
                const int q = base + 2 * u;
                if (q >= steps || !ok) break;
                uint32_t cw[QW];
#pragma unroll
                for (int i = 0; i < QW; i++) cw[i] = qn[u][i];
                const uint32_t scw = sn[u];
                fetch(q + 2 * PF, qn[u], sn[u]);
                const int s = q % S;
                const uint32_t ph = (uint32_t)(q / S) & 1u;
                if (!mbar_wait(&empty[s], ph ^ 1u, abort_flag, p.status, 26, p.wait_ns)) {
                    ok = false;
                    break;
                }
                uint8_t *bt = tiles + (size_t)s * kPairStageBytes + kTileBytes;
#pragma unroll
                for (int e = 0; e < 2; e++) {
                    const __half d = __ushort_as_half((unsigned short)(e == 0 ? scw & 0xFFFFu : scw >> 16));
                    if (QT == TLC_TYPE_Q4_0) {
                        uint32_t qb[4];
#pragma unroll
                        for (int i = 0; i < 4; i++) qb[i] = cw[2 * i + e];
                        dequant_block<QT>(qb, d, bt, piece, e);
                    } else {
                        uint32_t qb[8];
#pragma unroll
                        for (int i = 0; i < 4; i++) {
                            qb[2 * i] = cw[4 * i + 2 * e];
                            qb[2 * i + 1] = cw[4 * i + 2 * e + 1];
                        }
                        dequant_block<QT>(qb, d, bt, piece, e);
                    }
                }
                fence_async_proxy();
                __syncwarp();
                if (lane == 0) mbar_arrive(&full[s]);
            }
        }
    } else {
        // ------------------------------ epilogue ------------------------------
        // Warp w reads tensor-memory lanes 32*(w%4) .. +31: activation rows of this CTA's half.
        const int wq = warp & 3;
        for (int j = 0; j < my_tiles; j++) {
            const int b = j & 1;
            if (!__all_sync(0xffffffffu,
                            mbar_wait(&acc_full[b], ((uint32_t)j >> 1) & 1u, abort_flag, p.status, 27, p.wait_ns)))
                break;
            tc_fence_after();
            const int t = cluster_id + j * n_clusters;
            const int n0 = (t / m_tiles) * OUT_COLS;
            const int row = (t % m_tiles) * 256 + 128 * (int)rank + 32 * wq + lane;
            bool row_ok = row < p.m;
            const int pos = !row_ok ? 0 : p.positions ? p.positions[row] : p.pos_offset + row;
            if (row_ok && p.pos_stride != 0 && p.max_pos > 0 && (pos < 0 || pos >= p.max_pos)) {
                // a cache row that does not exist: nothing is written, the host hears about it
                if (atomicCAS(&p.status->code, 0, TLC_DEV_INDEX) == 0) p.status->where = 303;
                row_ok = false;
            }
            __half *ybase = p.y + (size_t)((long long)row * p.row_stride + (long long)pos * p.pos_stride);
            const uint32_t taddr = tmem_base + ((uint32_t)(32 * wq) << 16) + kAccCols * (uint32_t)b;
#pragma unroll 1
            for (int c0 = 0; c0 < OUT_COLS; c0 += 32) {
                uint32_t r[32];
                tmem_ld32(taddr + (uint32_t)c0, r);
                if (SW) {
                    uint32_t ru[32];
                    tmem_ld32(taddr + 128u + (uint32_t)c0, ru);
                    if (row_ok && n0 + c0 < p.n) epilogue_piece_swiglu(p, r, ru, n0 + c0, ybase);
                } else if (row_ok && n0 + c0 < p.n) {
                    epilogue_piece(p, r, row, pos, n0 + c0, ybase);
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) {
                if (rank == 0)
                    mbar_arrive(&acc_empty[b]);
                else
                    mbar_arrive_remote(&acc_empty[b], 0);
            }
            __syncwarp();
        }
    }

    // Tensor memory goes back when every MMA has finished and both CTAs are done with it.
    if (warp == 1) {
        __all_sync(0xffffffffu, mbar_wait(done_bar, 0, abort_flag, p.status, 28, my_tiles > 0 ? p.wait_ns : 20000ull));
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u) : "memory");
    }
}

template <int QT, bool SW>
int32_t launch_cta_pair_t(tlc_ctx *ctx, const GemmParams &p) {
    static int clusters[64] = {};
    int &nc = clusters[ctx->device & 63];
    if (nc == 0) {
        TLC_CUDA(cudaFuncSetAttribute(gemm_pair_kernel<QT, SW>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      (int)kPairSmem));
        TLC_CUDA(cudaFuncSetAttribute(gemm_pair_kernel<QT, SW>, cudaFuncAttributePreferredSharedMemoryCarveout,
                                      cudaSharedmemCarveoutMaxShared));
        // clusters of two that can be resident at once: an even share of tiles per cluster
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3((unsigned)(ctx->sm_count & ~1));
        cfg.blockDim = dim3(kPairThreads);
        cfg.dynamicSmemBytes = kPairSmem;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = 2;
        attr[0].val.clusterDim.y = 1;
        attr[0].val.clusterDim.z = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        int n = 0;
        if (cudaOccupancyMaxActiveClusters(&n, gemm_pair_kernel<QT, SW>, &cfg) != cudaSuccess || n <= 0) {
            cudaGetLastError();
            n = ctx->sm_count / 2;
        }
        nc = n < ctx->sm_count / 2 ? n : ctx->sm_count / 2;
    }
    const int out_cols = SW ? 128 : 256;
    const long total = (long)((p.m + 255) / 256) * ((p.n + out_cols - 1) / out_cols);
    const int n_clusters = (int)(total < nc ? total : nc);
    GemmParams q = p;
    CUtensorMap x_map;
    memset(&x_map, 0, sizeof x_map);
    if (!encode_x_map(&x_map, p)) return tlc_fail(TLC_ERR_INVALID_OPERATION, "gemm: no tensor map for the activations");
    q.a_tma = 1;
    cudaError_t le = tlc_launch_pdl(ctx, gemm_pair_kernel<QT, SW>, dim3((unsigned)(2 * n_clusters)), dim3(kPairThreads),
                                    kPairSmem, q, x_map);
    if (le != cudaSuccess) {
        cudaGetLastError();
        return tlc_fail(TLC_ERR_CUDA, "gemm (CTA pair) launch failed: %s", cudaGetErrorString(le));
    }
    TLC_CHECK_LAUNCH(ctx);
    return TLC_OK;
}

}  // namespace

bool tlc_gemm::cta_pair_eligible(const tlc_ctx *ctx, const GemmParams &p) {
    // Below 129 activation rows the peer CTA would multiply zeros; a forced single-CTA tile
    // shape keeps the single-CTA kernel; the tensor map needs 16-byte aligned rows.
    return ctx->gemm_pair && ctx->gemm_tile == 0 && p.m > 128 && ((uintptr_t)p.x & 15) == 0 && (p.k & 7) == 0;
}

int32_t tlc_gemm::launch_cta_pair(tlc_ctx *ctx, const GemmParams &p, int type, bool sw) {
    if (type == TLC_TYPE_Q4_0)
        return sw ? launch_cta_pair_t<TLC_TYPE_Q4_0, true>(ctx, p) : launch_cta_pair_t<TLC_TYPE_Q4_0, false>(ctx, p);
    return sw ? launch_cta_pair_t<TLC_TYPE_Q8_0, true>(ctx, p) : launch_cta_pair_t<TLC_TYPE_Q8_0, false>(ctx, p);
}
