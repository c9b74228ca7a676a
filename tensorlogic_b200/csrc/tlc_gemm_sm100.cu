// Kernel body and launcher of the tcgen05 dequant-GEMM (see tlc_gemm_kernel.cuh).
#include <cuda.h>
#include <cudaTypedefs.h>

#include <type_traits>

#include "tlc_gemm_kernel.cuh"

using namespace tlc_gemm;

// Tensor map of the activations [M, K] (f16, rows K elements apart): boxes of 128 rows
// x 64 columns, 128-byte swizzle, zero fill outside.  False when the driver entry point
// is missing or refuses the shape; the cp.async loaders take over then.
bool tlc_gemm::encode_x_map(CUtensorMap *map, const GemmParams &p) {
    static PFN_cuTensorMapEncodeTiled_v12000 encode = [] {
        void *fn = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres) != cudaSuccess ||
            qres != cudaDriverEntryPointSuccess)
            fn = nullptr;
        cudaGetLastError();
        return reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(fn);
    }();
    if (!encode || ((uintptr_t)p.x & 15) != 0 || (p.k & 7) != 0) return false;
    const cuuint64_t dims[2] = {(cuuint64_t)p.k, (cuuint64_t)p.m};
    const cuuint64_t strides[1] = {(cuuint64_t)p.k * 2};
    const cuuint32_t box[2] = {(cuuint32_t)kBK, 128};
    const cuuint32_t estr[2] = {1, 1};
    return encode(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<__half *>(p.x), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

namespace {

// B producer of one weight row.  The row's share of a weight tile (64 bytes of
// quants: four 16-byte pieces, plus its block scales) covers two K steps for
// Q4_0 and one for Q8_0; shares are fetched in groups of two tiles, one group
// ahead of their use, so the global-memory latency is spread over a group's
// worth of K steps.
template <int QT, int STAGES, int STAGE_BYTES>
__device__ __forceinline__ void produce_b(const GemmParams &p, uint8_t *btiles, uint64_t *full, uint64_t *empty,
                                          volatile int *abort_flag, const uint8_t *wbase, int wrow, int row, int KT,
                                          int lane) {
    constexpr int TILE = QT == TLC_TYPE_Q4_0 ? 1152 : 1088;
    constexpr int TS = QT == TLC_TYPE_Q4_0 ? 2 : 1;  // K steps per tile
    constexpr int GT = 2;                             // tiles per group
    // `row`: row of the smem tile this thread fills; `wrow`: the weight row it holds (of `wbase`).
    // Rows past N load nothing: a zero scale makes every value of the tile row zero.
    const bool row_ok = wrow < p.n;
    const int r16 = wrow & 15;
    const uint8_t *slab = wbase + (size_t)(row_ok ? wrow >> 4 : 0) * p.w_pitch;
    const uint32_t qoff = (uint32_t)((r16 >> 3) * 512 + (r16 & 7) * 64);
    const uint32_t soff = 1024u + (uint32_t)r16 * (QT == TLC_TYPE_Q4_0 ? 8u : 4u);
    uint4 nxt4[GT * 4], cur4[GT * 4];
    uint32_t nxts[GT * TS], curs[GT * TS];
    auto load_group = [&](int g) {
#pragma unroll
        for (int i = 0; i < GT; i++) {
            const int kt = g * GT + i;
            const bool ok = row_ok && kt < p.k_tiles;
            const uint8_t *tile = slab + (size_t)(ok ? kt : 0) * TILE;
#pragma unroll
            for (int t = 0; t < 4; t++)
                nxt4[i * 4 + t] = ok ? __ldg(reinterpret_cast<const uint4 *>(tile + qoff) + t) : make_uint4(0, 0, 0, 0);
            if (QT == TLC_TYPE_Q4_0) {
                const uint2 sc = ok ? __ldg(reinterpret_cast<const uint2 *>(tile + soff)) : make_uint2(0, 0);
                nxts[i * TS] = sc.x;
                nxts[i * TS + TS - 1] = sc.y;
            } else {
                nxts[i * TS] = ok ? __ldg(reinterpret_cast<const uint32_t *>(tile + soff)) : 0u;
            }
        }
    };
    // byte offsets of the eight 16-byte pieces of this row under the 128-byte swizzle
    uint32_t piece[8];
#pragma unroll
    for (int j = 0; j < 8; j++) piece[j] = (uint32_t)(row * 128 + ((j ^ (row & 7)) << 4));
    constexpr int SPG = GT * TS;  // K steps per group
    const int n_groups = (KT + SPG - 1) / SPG;
    auto comp = [](const uint4 &v, int i) { return i == 0 ? v.x : i == 1 ? v.y : i == 2 ? v.z : v.w; };
    auto process = [&](int g) {
#pragma unroll
        for (int st = 0; st < SPG; st++) {
            const int kt = g * SPG + st;
            if (kt >= KT) break;
            const int ti = st / TS;        // tile of the group
            const int half = st % TS;      // Q4_0: which pair of the tile's four blocks
            const uint32_t scw = curs[ti * TS + half];  // the two scales of this K step
            const int s = kt % STAGES;
            mbar_wait(&empty[s], ((kt / STAGES) & 1u) ^ 1u, abort_flag, p.status, 11, p.wait_ns);
            uint8_t *bt = btiles + (size_t)s * STAGE_BYTES;
#pragma unroll
            for (int e = 0; e < 2; e++) {
                const __half d = __ushort_as_half((unsigned short)(e == 0 ? scw & 0xFFFFu : scw >> 16));
                if (QT == TLC_TYPE_Q4_0) {
                    uint32_t q[4];
#pragma unroll
                    for (int t = 0; t < 4; t++) q[t] = comp(cur4[ti * 4 + t], 2 * half + e);
                    dequant_block<QT>(q, d, bt, piece, e);
                } else {
                    uint32_t q[8];
#pragma unroll
                    for (int t = 0; t < 4; t++) {
                        q[2 * t] = comp(cur4[ti * 4 + t], 2 * e);
                        q[2 * t + 1] = comp(cur4[ti * 4 + t], 2 * e + 1);
                    }
                    dequant_block<QT>(q, d, bt, piece, e);
                }
            }
            fence_async_proxy();
            __syncwarp();
            if (lane == 0) mbar_arrive(&full[s]);
        }
    };
    load_group(0);
#pragma unroll 1
    for (int g = 0; g < n_groups; g++) {
#pragma unroll
        for (int i = 0; i < GT * 4; i++) cur4[i] = nxt4[i];
#pragma unroll
        for (int i = 0; i < GT * TS; i++) curs[i] = nxts[i];
        if (g + 1 < n_groups) load_group(g + 1);
        process(g);
    }
}

// B producer for the form with two producer groups (PG = 2): the warps of group g fill the K
// steps kt = g, g + 2, ...  A thread still owns one weight row, but only every other ring stage,
// so twice as many warps share the dequantization of a K step sequence: the per-step latency of
// the producers, which bounds the GEMM when the tensor cores have little to do (one sub-tile of
// activation rows), halves.  Per own step a thread fetches its row's quants (32 bytes of Q4_0 in
// four 8-byte loads, 64 bytes of Q8_0) and scale word two own steps ahead.
template <int QT, int STAGES, int STAGE_BYTES>
__device__ __forceinline__ void produce_b_alt(const GemmParams &p, uint8_t *btiles, uint64_t *full, uint64_t *empty,
                                              volatile int *abort_flag, const uint8_t *wbase, int wrow, int row, int KT,
                                              int lane, int group, int kt0) {
    // KT: K steps of this CTA, the first one being step kt0 of the weight (split K)
    constexpr int TILE = QT == TLC_TYPE_Q4_0 ? 1152 : 1088;
    constexpr int PF = 2;                             // own steps fetched ahead
    constexpr int QW = QT == TLC_TYPE_Q4_0 ? 8 : 16;  // quant words of a row per K step
    const bool row_ok = wrow < p.n;
    const int r16 = wrow & 15;
    const uint8_t *slab = wbase + (size_t)(row_ok ? wrow >> 4 : 0) * p.w_pitch;
    const uint32_t qoff = (uint32_t)((r16 >> 3) * 512 + (r16 & 7) * 64);
    const uint32_t soff = 1024u + (uint32_t)r16 * (QT == TLC_TYPE_Q4_0 ? 8u : 4u);
    uint32_t piece[8];
#pragma unroll
    for (int j = 0; j < 8; j++) piece[j] = (uint32_t)(row * 128 + ((j ^ (row & 7)) << 4));
    uint32_t qn[PF][QW], sn[PF];
    auto fetch = [&](int kl, uint32_t (&qw)[QW], uint32_t &sc) {
        const int kt = kt0 + kl;
        const int wt = QT == TLC_TYPE_Q4_0 ? kt >> 1 : kt;
        const bool ok = row_ok && kl < KT && wt < p.k_tiles;
        const uint8_t *tile = slab + (size_t)(ok ? wt : 0) * TILE;
        if (QT == TLC_TYPE_Q4_0) {
            const int half = kt & 1;  // which pair of the tile's four blocks
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const uint2 v = ok ? __ldg(reinterpret_cast<const uint2 *>(tile + qoff + 16 * i + 8 * half)) : make_uint2(0, 0);
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
#pragma unroll 1
    for (int base = group; base < KT; base += 2 * PF) {
#pragma unroll
        for (int u = 0; u < PF; u++) {
            const int kt = base + 2 * u;
            if (kt >= KT) break;
            uint32_t cw[QW];
#pragma unroll
            for (int i = 0; i < QW; i++) cw[i] = qn[u][i];
            const uint32_t scw = sn[u];
            fetch(kt + 2 * PF, qn[u], sn[u]);
            const int s = kt % STAGES;
            mbar_wait(&empty[s], ((kt / STAGES) & 1u) ^ 1u, abort_flag, p.status, 15, p.wait_ns);
            uint8_t *bt = btiles + (size_t)s * STAGE_BYTES;
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
}

// SW: the SiLU.mul pair.  The weight tile holds 128 rows of the gate weight (tile rows
// 0-127) and the same 128 rows of the up weight (tile rows 128-255); the epilogue reads
// both accumulators and stores silu(gate) * up for the 128 output columns of the CTA.
// 32 consecutive f32 accumulators of one activation row to the split-K partial sums.
__device__ __forceinline__ void store_partial(float *dst, const uint32_t (&r)[32], bool ok, bool vec, int left) {
    if (!ok) return;
    if (vec) {
#pragma unroll
        for (int v = 0; v < 8; v++)
            *reinterpret_cast<uint4 *>(dst + 4 * v) = make_uint4(r[4 * v], r[4 * v + 1], r[4 * v + 2], r[4 * v + 3]);
    } else {
#pragma unroll
        for (int e = 0; e < 32; e++)
            if (e < left) dst[e] = __uint_as_float(r[e]);
    }
}

// PG: producer groups.  1: the 4*NT producer warps fill every K step.  2: twice the warps, each
// group every other step (produce_b_alt) -- for tiles of one activation sub-tile, where the
// producers and not the MMAs set the pace.
template <int QT, int MT, int NT, bool SW, int PG>
__global__ void __launch_bounds__(gemm_threads(NT, PG), 1)
    gemm_tcgen05_kernel(const GemmParams p, const __grid_constant__ CUtensorMap x_map) {
    static_assert(!SW || NT == 2, "the gate/up pair fills a 256-row weight tile");
    constexpr int BN = 128 * NT;
    constexpr int A_BYTES = 128 * MT * 128, B_BYTES = BN * 128;
    constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
    constexpr int kStages = stages_for(MT, NT);
    constexpr uint32_t TMEM_COLS = MT * BN;  // 128, 256 or 512: a power of two
    constexpr uint32_t IDESC = idesc_for(BN);
    constexpr int MMA_WARP = 4 + 4 * NT * PG;  // 12 with NT = 2, PG = 1 (eight producer warps) or NT = 1, PG = 2

    extern __shared__ uint8_t smem_raw[];
    uint8_t *tiles = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint64_t *full = reinterpret_cast<uint64_t *>(tiles + (size_t)kStages * STAGE_BYTES);
    uint64_t *empty = full + kStages;
    uint64_t *accum_bar = empty + kStages;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(accum_bar + 1);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int n0 = blockIdx.x * (SW ? 128 : BN), m0 = blockIdx.y * 128 * MT;
    const int KT_all = (p.k + kBK - 1) / kBK;  // K is a multiple of 32: the last step may hold one block only
    // split K (two-group form only): this CTA's share of the K steps, never empty
    int kt0 = 0, KT = KT_all;
    const bool split = PG == 2 && p.ksplit > 1;
    if (split) {
        const int per = (KT_all + p.ksplit - 1) / p.ksplit;
        kt0 = (int)blockIdx.z * per;
        KT = KT_all - kt0 < per ? KT_all - kt0 : per;
    }

    if (tid == 0) {
        for (int s = 0; s < kStages; s++) {
            // the activation tile arrives by TMA (one arrive.expect_tx) or from the four
            // cp.async loader warps; the working B-producer warps arrive once each
            mbar_init(&full[s], (p.a_tma ? 1 : 4) + 4 * NT);
            mbar_init(&empty[s], 1);          // tcgen05.commit
        }
        mbar_init(accum_bar, 1);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == MMA_WARP) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                     "r"(TMEM_COLS)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    tlc_pdl_prologue();  // x (and residual) come from the previous kernel of the stream

    if (warp >= 4 && warp < 4 + 4 * NT * PG) {
        const int trow = (tid - 128) % BN;  // row of the weight tile
        const uint8_t *wbase = SW && trow >= 128 ? p.w2 : p.w;
        const int wrow = SW ? n0 + (trow & 127) : n0 + trow;
        if (PG == 1)
            produce_b<QT, kStages, STAGE_BYTES>(p, tiles + A_BYTES, full, empty, abort_flag, wbase, wrow, trow, KT, lane);
        else
            produce_b_alt<QT, kStages, STAGE_BYTES>(p, tiles + A_BYTES, full, empty, abort_flag, wbase, wrow, trow, KT,
                                                    lane, (tid - 128) / BN, kt0);
    } else if (warp < 4 && p.a_tma) {
        // ------------------------------ A tile by TMA ------------------------------
        // One thread issues, per K step, MT boxes of 128 rows x 64 columns with the 128-byte
        // swizzle of the tile; rows past M and columns past K read the zero fill.  The
        // inner coordinate is a multiple of 64 elements (128 bytes).
        if (tid == 0) {
            asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&x_map)) : "memory");
            for (int j = 0; j < KT; j++) {
                const int s = j % kStages;
                if (!mbar_wait(&empty[s], ((j / kStages) & 1u) ^ 1u, abort_flag, p.status, 12, p.wait_ns)) break;
                const uint32_t bar = smem_u32(&full[s]);
                const uint32_t abase = smem_u32(tiles + (size_t)s * STAGE_BYTES);
                mbar_arrive_expect_tx(&full[s], A_BYTES);
#pragma unroll
                for (int i = 0; i < MT; i++)
                    tma_load_2d(abase + i * (128 * 128), &x_map, (kt0 + j) * kBK, m0 + 128 * i, bar);
            }
        }
        __syncwarp();  // the other lanes of warp 0 sleep here instead of polling beside the issuer
    } else if (warp < 4) {
        // ------------------------------ A loaders (cp.async) ------------------------------
        auto issue = [&](int j) {
            const int s = j % kStages;
            mbar_wait(&empty[s], ((j / kStages) & 1u) ^ 1u, abort_flag, p.status, 12, p.wait_ns);
            const uint32_t abase = smem_u32(tiles + (size_t)s * STAGE_BYTES);
            // 8 consecutive threads copy the 128 bytes of one row.
#pragma unroll
            for (int it = 0; it < 8 * MT; it++) {
                const int row = it * 16 + (tid >> 3), c = tid & 7;
                // rows past M and, in a last step of one block, columns past K are zero-filled
                const bool ok = m0 + row < p.m && (kt0 + j) * kBK + c * 8 < p.k;
                const __half *src = p.x + (ok ? (size_t)(m0 + row) * p.k + (size_t)(kt0 + j) * kBK + c * 8 : 0);
                cp_async16(abase + row * 128 + ((c ^ (row & 7)) << 4), src, ok);
            }
        };
        constexpr int kAhead = kStages - 1;
        for (int j = 0; j < kAhead; j++) {
            if (j < KT) issue(j);
            asm volatile("cp.async.commit_group;" ::: "memory");
        }
        for (int kt = 0; kt < KT; kt++) {
            // Hand over stage kt first, then refill the stage the MMA of step
            // kt-1 is about to free: the hand-over must not wait for that MMA.
            asm volatile("cp.async.wait_group %0;" ::"n"(kAhead - 1) : "memory");
            fence_async_proxy();
            __syncwarp();
            if (lane == 0) mbar_arrive(&full[kt % kStages]);
            const int j = kt + kAhead;
            if (j < KT) issue(j);
            asm volatile("cp.async.commit_group;" ::: "memory");
        }
    } else if (warp == MMA_WARP) {
        // ------------------------------ MMA issuer ------------------------------
        for (int kt = 0; kt < KT; kt++) {
            const int s = kt % kStages;
            const bool ready = __all_sync(0xffffffffu, mbar_wait(&full[s], (kt / kStages) & 1u, abort_flag, p.status, 14, p.wait_ns));
            tc_fence_after();
            if (lane == 0 && ready) {
                const uint32_t a_addr = smem_u32(tiles + (size_t)s * STAGE_BYTES);
                const uint32_t b_addr = a_addr + A_BYTES;
#pragma unroll
                for (int k16 = 0; k16 < kBK / 16; k16++) {
                    const uint64_t bdesc = make_desc(b_addr + k16 * 32);
#pragma unroll
                    for (int i = 0; i < MT; i++)
                        umma_f16(tmem_base + BN * i, make_desc(a_addr + i * (128 * 128) + k16 * 32), bdesc, IDESC,
                                 (kt > 0 || k16 > 0) ? 1u : 0u);
                }
            }
            if (lane == 0) umma_commit(&empty[s]);  // arrives when the MMAs above have read the stage
            __syncwarp();
        }
        if (lane == 0) umma_commit(accum_bar);
        __syncwarp();
    }

    // ------------------------------ epilogue ------------------------------
    // Warp w reads tensor-memory lanes 32*(w%4) .. +31 (= activation rows of a
    // sub-tile); the warps of a lane quarter (three, or five with two producer groups of a
    // 256-row weight tile) take the 32-column pieces in turn.
    if (warp < MMA_WARP) {
        mbar_wait(accum_bar, 0, abort_flag, p.status, 13, p.wait_ns);
        tc_fence_after();
        const int wq = warp & 3;
        constexpr int OUT_COLS = SW ? 128 : BN;  // output columns of the CTA
        constexpr int PIECES = MT * OUT_COLS / 32;
#pragma unroll 1
        for (int pc = warp >> 2; pc < PIECES; pc += MMA_WARP / 4) {
            const int i = pc / (OUT_COLS / 32), c0 = (pc % (OUT_COLS / 32)) * 32;
            const int row = m0 + 128 * i + 32 * wq + lane;
            bool row_ok = row < p.m;
            const int pos = !row_ok ? 0 : p.positions ? p.positions[row] : p.pos_offset + row;
            if (row_ok && p.pos_stride != 0 && p.max_pos > 0 && (pos < 0 || pos >= p.max_pos)) {
                // a cache row that does not exist: nothing is written, the host hears about it
                if (atomicCAS(&p.status->code, 0, TLC_DEV_INDEX) == 0) p.status->where = 301;
                row_ok = false;
            }
            // Dense rows by default; a KV-cache destination addresses rows by (sequence, position).
            __half *ybase = p.y + (size_t)((long long)row * p.row_stride + (long long)pos * p.pos_stride);
            uint32_t r[32];
            tmem_ld32(tmem_base + ((uint32_t)(32 * wq) << 16) + (uint32_t)(BN * i + c0), r);
            if (split) {
                // this CTA's f32 share; the finishing kernel rounds and applies the epilogue
                float *dst = p.partial + ((size_t)blockIdx.z * p.m + (row < p.m ? row : 0)) * p.ntot + p.noff + n0 + c0;
                const bool ok = row < p.m && n0 + c0 < p.n;
                const bool vec = ok && n0 + c0 + 32 <= p.n && ((p.ntot | p.noff | p.n) & 3) == 0;
                store_partial(dst, r, ok, vec, p.n - (n0 + c0));
                if (SW) {
                    tmem_ld32(tmem_base + ((uint32_t)(32 * wq) << 16) + (uint32_t)(BN * i + 128 + c0), r);
                    store_partial(dst + p.n, r, ok, vec, p.n - (n0 + c0));
                }
                continue;
            }
            if (SW) {
                // s = sigmoid(g) (f32, RNE); a = g*s; act = a*u: three f16 roundings as in
                // debug/chat_demo_with_kvcache.tl:26-41 (the GEMV's SiLU.mul epilogue does the same)
                uint32_t ru[32];
                tmem_ld32(tmem_base + ((uint32_t)(32 * wq) << 16) + (uint32_t)(BN * i + 128 + c0), ru);
                if (row_ok && n0 + c0 < p.n) epilogue_piece_swiglu(p, r, ru, n0 + c0, ybase);
            } else if (row_ok && n0 + c0 < p.n) {
                epilogue_piece(p, r, row, pos, n0 + c0, ybase);
            }
        }
        tc_fence_before();
    }

    __syncthreads();
    if (warp == MMA_WARP) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
    }
}

template <int QT, int MT, int NT, bool SW, int PG>
int32_t launch_tile_pg(tlc_ctx *ctx, const GemmParams &p) {
    const size_t smem = smem_bytes(MT, NT);
    static bool configured[64] = {};
    if (!configured[ctx->device & 63]) {
        TLC_CUDA(cudaFuncSetAttribute(gemm_tcgen05_kernel<QT, MT, NT, SW, PG>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      (int)smem));
        TLC_CUDA(cudaFuncSetAttribute(gemm_tcgen05_kernel<QT, MT, NT, SW, PG>,
                                      cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared));
        configured[ctx->device & 63] = true;
    }
    const int out_cols = SW ? 128 : 128 * NT;  // output columns per CTA
    GemmParams q = p;
    if (PG != 2 || q.ksplit < 2) {  // split K exists in the two-group form only
        q.ksplit = 1;
        q.partial = nullptr;
    }
    const dim3 grid((unsigned)((p.n + out_cols - 1) / out_cols), (unsigned)((p.m + 128 * MT - 1) / (128 * MT)),
                    (unsigned)q.ksplit);
    CUtensorMap x_map;
    memset(&x_map, 0, sizeof x_map);
    q.a_tma = ctx->gemm_tma && encode_x_map(&x_map, p) ? 1 : 0;
    cudaError_t le = tlc_launch_pdl(ctx, gemm_tcgen05_kernel<QT, MT, NT, SW, PG>, grid, dim3(gemm_threads(NT, PG)), smem, q,
                                    x_map);
    if (le != cudaSuccess) {
        cudaGetLastError();
        return tlc_fail(TLC_ERR_CUDA, "gemm launch failed: %s", cudaGetErrorString(le));
    }
    TLC_CHECK_LAUNCH(ctx);
    return TLC_OK;
}

// Two producer groups (the form split K exists in) when the K steps of a tile are shared out, or
// when option "gemm_pg" = 2 forces them; one group otherwise (1 = forced, and no split K).  On
// unsplit launches two groups measured no faster (8192 -> 28672, 32 rows: 86 against 80 us).
template <int QT, int MT, int NT, bool SW = false>
int32_t launch_tile(tlc_ctx *ctx, const GemmParams &p) {
    const bool two = MT == 1 && (ctx->gemm_pg == 2 || (ctx->gemm_pg == 0 && p.ksplit > 1));
    if (two) return launch_tile_pg<QT, 1, NT, SW, 2>(ctx, p);
    return launch_tile_pg<QT, MT, NT, SW, 1>(ctx, p);
}

template <int QT>
int32_t launch_one_t(tlc_ctx *ctx, const GemmParams &p) {
    // Tile choice: 256 x 256 halves the activation traffic from L2 per MMA against 128 x 128
    // (measured on wide weights: about 930 / 760 / 580 TFLOP/s for 256x256 / 128x256 / 128x128),
    // but a tile shape only pays if its CTAs fill the SMs: score = relative tile speed x the
    // fraction of SM slots the last wave leaves busy.
    auto ctas = [&](int mt, int nt) {
        return (long)((p.n + 128 * nt - 1) / (128 * nt)) * ((p.m + 128 * mt - 1) / (128 * mt));
    };
    auto score = [&](int mt, int nt, double speed) {
        const long c = ctas(mt, nt), sms = ctx->sm_count;
        return speed * (double)c / (double)(((c + sms - 1) / sms) * sms);
    };
    int tile = ctx->gemm_tile;  // 0: choose; 11 / 12 / 22: forced (tests)
    if (tile == 0) {
        const double s22 = p.m > 128 ? score(2, 2, 1.0) : 0.0, s12 = score(1, 2, 0.8), s11 = score(1, 1, 0.6);
        tile = s22 >= s12 && s22 >= s11 ? 22 : s12 >= s11 ? 12 : 11;
    }
    if (tile == 22) return launch_tile<QT, 2, 2>(ctx, p);
    if (tile == 12) return launch_tile<QT, 1, 2>(ctx, p);
    return launch_tile<QT, 1, 1>(ctx, p);
}

// The gate/up pair: 128 output columns per CTA (a 256-row weight tile), one or two token sub-tiles.
template <int QT>
int32_t launch_pair_t(tlc_ctx *ctx, const GemmParams &p) {
    auto ctas = [&](int mt) { return (long)((p.n + 127) / 128) * ((p.m + 128 * mt - 1) / (128 * mt)); };
    auto score = [&](int mt, double speed) {
        const long c = ctas(mt), sms = ctx->sm_count;
        return speed * (double)c / (double)(((c + sms - 1) / sms) * sms);
    };
    const bool two = ctx->gemm_tile == 22 || (ctx->gemm_tile == 0 && p.m > 128 && score(2, 1.0) >= score(1, 0.8));
    return two ? launch_tile<QT, 2, 2, true>(ctx, p) : launch_tile<QT, 1, 2, true>(ctx, p);
}

int32_t launch_one(tlc_ctx *ctx, const GemmParams &p, int type) {
    // From 129 activation rows on, two SMs share a 256 x 256 tile (tlc_gemm_pair.cu).
    if (cta_pair_eligible(ctx, p)) return launch_cta_pair(ctx, p, type, p.w2 != nullptr);
    if (p.w2) return type == TLC_TYPE_Q4_0 ? launch_pair_t<TLC_TYPE_Q4_0>(ctx, p) : launch_pair_t<TLC_TYPE_Q8_0>(ctx, p);
    return type == TLC_TYPE_Q4_0 ? launch_one_t<TLC_TYPE_Q4_0>(ctx, p) : launch_one_t<TLC_TYPE_Q8_0>(ctx, p);
}

inline size_t align256(size_t v) { return (v + 255) & ~(size_t)255; }

}  // namespace

// Split K for the GEMM: with at most 128 activation rows a weight of few rows gives few CTAs (a
// 2048-row projection: eight), each walking all of K at the producers' pace.  The K steps are
// then shared out over gridDim.z CTAs per tile, at most enough to fill the SMs, at least eight
// steps each; f32 shares go to scratch and gemv_splitk_finish_kernel finishes.  `tiles`: weight
// tiles of 256 rows over all outputs of the call, `n_total`: their output columns.  1: no split.
static int gemm_choose_ksplit(const tlc_ctx *ctx, int m, int64_t k, int64_t tiles, int64_t n_total) {
    if (!ctx->gemm_splitk || m > 128 || ctx->gemm_pg == 1 || ctx->gemm_tile == 22 || tiles < 1) return 1;
    const int KT = (int)((k + kBK - 1) / kBK);
    int64_t ks_max = ctx->sm_count / tiles;
    if (ks_max > KT / 8) ks_max = KT / 8;
    if (ks_max > 16) ks_max = 16;
    // Cost in microseconds: K steps of a CTA at 0.45 us, plus, when split, the finishing launch and
    // the f32 shares written and read back (about 3 TB/s through the L2).  128 rows of a
    // 2048 -> 8192 projection are faster unsplit (18 against 28 us), 32 rows split (18 against 30 us).
    int best = 1;
    double best_t = KT * 0.45;
    for (int ks = 2; ks <= ks_max; ks++) {
        const int per = (KT + ks - 1) / ks;
        if ((KT + per - 1) / per != ks) continue;  // a share would be empty
        const double t = per * 0.45 + 4.0 + (double)ks * m * (double)n_total * 8.0 / 3.0e6;
        if (t < best_t || ctx->gemm_splitk == 2) {  // 2: the most shares, whatever they cost (tests)
            best_t = t;
            best = ks;
        }
    }
    return best;
}
static int64_t gemm_tiles(const tlc_gemv_args &a) {
    if (a.epilogue == TLC_EPI_SWIGLU) return (a.outs[0].w->n_rows + 127) / 128;
    int64_t t = 0;
    for (int i = 0; i < a.n_out; i++) t += (a.outs[i].w->n_rows + 255) / 256;
    return t;
}

// Context scratch the GEMM form of a linear over m rows of width k with n_total outputs (all
// outputs of a fused call; the SiLU.mul pair counts twice) may need: the normalized rows and
// the split-K partial sums.  Callers that capture graphs reserve it up front.
size_t tlc_gemm_scratch_bytes(const tlc_ctx *ctx, int m, int64_t k, int64_t n_total) {
    const int mp = m < 128 ? m : 128;
    // the most shares any row count and any tiling of n_total outputs can get, whatever the options
    // say when the launch comes
    int ks = 1;
    {
        const int KT = (int)((k + kBK - 1) / kBK);
        const int64_t tiles = (n_total + 255) / 256 > 0 ? (n_total + 255) / 256 : 1;
        int64_t ks_max = ctx->sm_count / tiles;
        if (ks_max > KT / 8) ks_max = KT / 8;
        if (ks_max > 16) ks_max = 16;
        if (ks_max > 1) ks = (int)ks_max;
    }
    return align256((size_t)m * k * 2) + (ks > 1 ? align256((size_t)ks * mp * (size_t)n_total * sizeof(float)) : 0);
}

bool tlc_gemm_eligible(const tlc_ctx *ctx, const tlc_gemv_args &a) {
    const tlc_qtensor *w0 = a.outs[0].w;
    if (w0->type != TLC_TYPE_Q4_0 && w0->type != TLC_TYPE_Q8_0) return false;
    // K in whole blocks; an odd block count ends in a K step whose second block is the row's
    // zero padding (rows are padded to 16 bytes with zeros at upload) against zero-filled activations
    if (w0->n_cols % 32 != 0 || w0->n_cols < kBK) return false;
    if (ctx->gemm_min_m > 0) return a.m >= ctx->gemm_min_m;
    // Below 17 rows one GEMV pass reads the weights once.
    if (a.m <= 16) return false;
    // With split K the few CTAs of a narrow weight share K, and the GEMM wins from 17 rows on.
    int64_t n_total = 0;
    for (int i = 0; i < a.n_out; i++) n_total += a.outs[i].w->n_rows;
    if (gemm_choose_ksplit(ctx, a.m, w0->n_cols, gemm_tiles(a), n_total) > 1) return true;
    // Without it, up to 48 rows the GEMV's few passes still win unless the weight has enough
    // 128-row tiles to occupy half of the SMs.
    int64_t tiles = 0;
    for (int i = 0; i < a.n_out; i++) tiles = tiles < (a.outs[i].w->n_rows + 128 - 1) / 128 ? (a.outs[i].w->n_rows + 128 - 1) / 128 : tiles;
    return a.m > (tiles * 2 >= ctx->sm_count ? 16 : 48);
}

// Same contract as tlc_launch_gemv for m activation rows on the tensor cores:
// the RMSNorm prologue runs as its own kernel into scratch, every output of a
// fused multi-projection is its own GEMM, and the SiLU.mul pair is one GEMM whose
// weight tile holds gate and up rows side by side.
int32_t tlc_launch_gemm(tlc_ctx *ctx, const tlc_gemv_args &a) {
    const tlc_qtensor *w0 = a.outs[0].w;
    const int64_t k = w0->n_cols;
    const bool swiglu = a.epilogue == TLC_EPI_SWIGLU;
    const size_t norm_bytes = a.norm_w ? align256((size_t)a.m * k * 2) : 0;
    int64_t ntot = 0;
    for (int i = 0; i < a.n_out; i++) ntot += a.outs[i].w->n_rows;
    const int ksplit = gemm_choose_ksplit(ctx, a.m, k, gemm_tiles(a), ntot);
    const size_t part_bytes = ksplit > 1 ? align256((size_t)ksplit * a.m * (size_t)ntot * sizeof(float)) : 0;
    if (norm_bytes + part_bytes > 0)
        if (int32_t rc = tlc_scratch_reserve(ctx, norm_bytes + part_bytes)) return rc;
    uint8_t *scratch = static_cast<uint8_t *>(ctx->scratch);
    float *partial = ksplit > 1 ? reinterpret_cast<float *>(scratch + norm_bytes) : nullptr;
    int noff = 0;
    const __half *x = static_cast<const __half *>(a.x);
    if (a.norm_w) {
        if (int32_t rc = tlc_rms_norm(ctx, a.x, a.norm_w, scratch, a.m, (int32_t)k, a.eps)) return rc;
        x = reinterpret_cast<const __half *>(scratch);
    }
    TLC_REQUIRE(((uintptr_t)x & 15) == 0, TLC_ERR_INVALID_OPERATION, "gemm: activations must be 16-byte aligned");
    // The SiLU.mul pair is ONE launch: gate and up rows share the weight tile of a CTA.
    const int n_launch = swiglu ? 1 : a.n_out;
    for (int i = 0; i < n_launch; i++) {
        const tlc_qtensor *w = a.outs[i].w;
        GemmParams p{};
        p.w = static_cast<const uint8_t *>(w->data);
        p.w_pitch = w->slab_pitch;
        p.k_tiles = (int)w->k_tiles;
        p.x = x;
        p.m = a.m;
        p.n = (int)w->n_rows;
        p.k = (int)k;
        p.status = ctx->dev_status;
        p.wait_ns = ctx->wait_ns;
        p.y = static_cast<__half *>(a.outs[i].y);
        if (swiglu) {
            TLC_REQUIRE(a.outs[1].w->slab_pitch == w->slab_pitch, TLC_ERR_SHAPE_MISMATCH,
                        "gate and up projections must have the same layout");
            p.w2 = static_cast<const uint8_t *>(a.outs[1].w->data);
            p.row_stride = p.n;
        } else {
            p.row_stride = a.outs[i].row_stride >= 0 ? a.outs[i].row_stride : (long long)w->n_rows;
            p.pos_stride = a.outs[i].pos_stride;
            p.head_dim = a.outs[i].rope_heads > 0 ? (int)(w->n_rows / a.outs[i].rope_heads) : 0;
            p.residual = a.epilogue == TLC_EPI_RESIDUAL ? static_cast<const __half *>(a.residual) : nullptr;
            p.bias = a.epilogue == TLC_EPI_STORE ? static_cast<const __half *>(a.bias) : nullptr;
        }
        p.pos_offset = a.pos_offset;
        p.positions = a.positions;
        p.max_pos = a.max_pos;
        p.rope_base = (float)a.rope_base;
        p.vec_ok = ((p.row_stride | p.pos_stride | (long long)p.n) & 7) == 0 && ((uintptr_t)p.y & 15) == 0 &&
                   ((uintptr_t)p.residual & 15) == 0;
        p.partial = partial;
        p.ksplit = ksplit;
        p.ntot = (int)ntot;
        p.noff = noff;
        noff += p.n;
        if (int32_t rc = launch_one(ctx, p, w->type)) return rc;
    }
    if (ksplit > 1) return tlc_gemv_splitk_finish(ctx, a, ksplit, partial);
    return TLC_OK;
}
