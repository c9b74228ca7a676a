// One decode step of a LLaMA-architecture model as ONE persistent kernel.
//
// The TL scripts run a decode step as about 28 builtin dispatches per layer plus a
// host read-back of the logits (debug/chat_demo_with_kvcache.tl:213-296,
// src/interpreter/builtin_sampling.rs:131-140); launched kernel by kernel even the fused
// form (five launches per layer) spends most of a small model's step between kernels:
// the weights of a TinyLlama layer stream from HBM in under 4 us, five launches cost 25 us.
// Here the whole step -- every layer's
//
//   A  rms_norm + q/k/v linears + rope + cache append
//   B  grouped-query attention over the cache
//   C  o projection + residual
//   D  rms_norm + gate/up linears + silu*mul
//   E  down projection + residual
//
// then  F  rms_norm + lm_head  and  G  greedy sample + bookkeeping -- runs in one
// cooperative grid of one CTA per SM.  Phases are separated by a grid-wide barrier (one
// atomic per CTA on a monotonic counter); activations cross it through global memory and
// are re-read with L1-bypassing loads.  In every CTA one producer warp walks the CTA's
// share of ALL the step's weight tiles in schedule order and streams them into a shared
// memory ring with bulk async copies; weights are immutable, so it never waits for a
// barrier and the ring already holds the next phase's tiles when the consumers get there.
// Eight consumer warps do the math of tlc_gemv_kernel.cuh (one activation row): nibbles
// and bytes become exact f16 tensor-core fragments, the K range of a 16-row slab is split
// over the warps, one cross-warp reduction per batch of slabs, epilogue, store.
// The attention phase is the flash-decoding of tlc_attention.cu: (KV head, key split)
// items over the CTAs, partial (max, sum, O) to global scratch, the last CTA of a head
// (atomic ticket) merges.
//
// One sequence, greedy sampling, no tensor parallelism, all quantized linears of one
// type; anything else takes the kernel-by-kernel path of tlc_llama.cu.  `steps` decode
// steps can run inside one launch.  Every wait (mbarrier, grid barrier) is bounded in
// time: a wait that runs out raises the device status word, every CTA sees it at its next
// barrier, drains its copies and returns; the host reports TLC_ERR_TIMEOUT.
#include <cuda_fp16.h>

#include "tlc_gemv_common.cuh"
#include "tlc_internal.h"
#include "tlc_step.h"

namespace tlc_step {

using namespace tlc_gemv;

constexpr int CW = 8;                 // consumer warps
constexpr int CT = CW * 32;           // consumer threads
constexpr int kThreads = CT + 32;     // + the producer warp
constexpr int kBatchSlabs = 8;        // slabs per cross-warp reduction
constexpr int kTileKeys = 64;

// ---- shared memory layout ---------------------------------------------------------------
//   0     full[12]   128  empty[12]   256 abort flag, 260 issued stages, 264 scratch ints
//   512   sq_part[CW] + misc floats
//   1024  red [2][CW][kBatchSlabs][16] f32
//   ...   cand_v[CW] / cand_i[CW], sm_m / sm_l [4][16] (attention merge)
//   ...   xres  f16 [d]           raw input of the last normalised phase (the residual)
//   ...   xin   f16 [kmax]        the current phase's input as it came from global memory
//   ...   cinit float4 [kmax/32 padded]
//   ...   xperm uint4 [kmax/32 padded][4]
//   ...   attention K/V tiles [2][2][64][D+8] f16 (reused as the 4 warps' O partials)
//   ...   ring [stages][16 tiles]
constexpr size_t kOffRed = 1024;
constexpr size_t kOffSmall = kOffRed + (size_t)2 * CW * kBatchSlabs * 16 * sizeof(float);
constexpr size_t kOffXres = kOffSmall + 1024;

__host__ __device__ inline size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

struct SmemPlan {
    size_t xres, xin, cinit, xperm, attn, ring, total;
    int stages;
};

__host__ __device__ inline SmemPlan plan_smem(int d, int kmax, int head_dim, int stage_bytes, int tb, size_t budget) {
    SmemPlan s{};
    const int nblk_pad = (kmax / 32 + tb - 1) / tb * tb;
    s.xres = kOffXres;
    s.xin = align_up(s.xres + (size_t)d * 2, 16);
    s.cinit = align_up(s.xin + (size_t)kmax * 2, 16);
    s.xperm = s.cinit + (size_t)nblk_pad * 16;
    s.attn = align_up(s.xperm + (size_t)nblk_pad * 64, 128);
    const size_t kv = (size_t)4 * kTileKeys * (head_dim + 8) * 2, so = (size_t)4 * 16 * head_dim * 4;
    s.ring = align_up(s.attn + (kv > so ? kv : so), 128);
    long st = budget > s.ring ? (long)((budget - s.ring) / (size_t)stage_bytes) : 0;
    if (st > kMaxStages) st = kMaxStages;
    s.stages = (int)st;
    s.total = s.ring + (size_t)s.stages * stage_bytes;
    return s;
}

// ---- device helpers ---------------------------------------------------------------------

__device__ __forceinline__ uint4 ldcg_u128(const void *p) {
    uint4 v;
    asm volatile("ld.global.cg.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
__device__ __forceinline__ int ldcg_i32(const int *p) {
    int v;
    asm volatile("ld.global.cg.s32 %0, [%1];" : "=r"(v) : "l"(p));
    return v;
}
__device__ __forceinline__ float ldcg_f32(const float *p) {
    float v;
    asm volatile("ld.global.cg.f32 %0, [%1];" : "=f"(v) : "l"(p));
    return v;
}
__device__ __forceinline__ uint32_t ld_acquire_gpu(const uint32_t *p) {
    uint32_t v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void red_release_gpu_add(uint32_t *p, uint32_t v) {
    asm volatile("red.release.gpu.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void cp_async16(void *smem_dst, const void *gsrc, bool valid) {
    const uint32_t d = (uint32_t)__cvta_generic_to_shared(smem_dst);
    const int sz = valid ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(gsrc), "r"(sz) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], const void *p) {
    const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(a));
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t (&r)[4], const void *p) {
    const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(a));
}
__device__ __forceinline__ void mma16816_acc(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_half2(float a, float b) {
    __half2 h = __floats2half2_rn(a, b);
    return *reinterpret_cast<uint32_t *>(&h);
}
template <int N>
__device__ __forceinline__ void named_bar(int id) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "n"(N) : "memory");
}

// One GEMV phase as both the producer and the consumers see it.
struct Phase {
    const uint8_t *w[3];
    size_t pitch[3];
    int slabs[3];
    int n[3];      // rows of each weight
    int subs;      // 2: units are (gate slab, up slab) pairs of w[0], w[1]
    int units;
    int ktiles, nchunks, nblk, k;
};

__device__ __forceinline__ Phase make_phase(const StepParams &P, const StepLayer *L, int ph) {
    Phase f{};
    f.subs = 1;
    int k = P.d;
    if (ph == 0) {  // A: q, k, v
        f.w[0] = L->wq; f.w[1] = L->wk; f.w[2] = L->wv;
        f.n[0] = P.qd; f.n[1] = P.kvd; f.n[2] = P.kvd;
    } else if (ph == 2) {  // C: o
        f.w[0] = L->wo; f.n[0] = P.d; k = P.qd;
    } else if (ph == 3) {  // D: gate / up
        f.w[0] = L->wg; f.w[1] = L->wu; f.n[0] = f.n[1] = P.ffn; f.subs = 2;
    } else if (ph == 4) {  // E: down
        f.w[0] = L->wd; f.n[0] = P.d; k = P.ffn;
    } else {  // F: lm_head
        f.w[0] = P.w_out; f.n[0] = P.vocab;
    }
    f.k = k;
    f.nblk = k / 32;
    f.ktiles = (f.nblk + P.tb - 1) / P.tb;
    f.nchunks = (f.ktiles + kTilesPerStage - 1) / kTilesPerStage;
    const size_t pitch = (size_t)f.ktiles * P.tile_bytes;
    f.units = 0;
    for (int i = 0; i < 3; i++) {
        f.pitch[i] = pitch;
        f.slabs[i] = f.w[i] ? (f.n[i] + kRows - 1) / kRows : 0;
        f.units += f.slabs[i];
    }
    if (f.subs == 2) f.units = f.slabs[0];
    return f;
}

// Which weight and slab unit `u`, sub-unit `sub` is.
__device__ __forceinline__ void unit_slab(const Phase &f, int u, int sub, int &ti, int &sl) {
    ti = 0;
    sl = u;
    if (f.subs == 2) {
        ti = sub;
        return;
    }
    if (sl >= f.slabs[0]) { sl -= f.slabs[0]; ti = 1; }
    if (ti == 1 && sl >= f.slabs[1]) { sl -= f.slabs[1]; ti = 2; }
}

struct Ctl {
    uint64_t *full, *empty;
    volatile int *abort_flag;
    volatile int *issued;  // stages the producer has started copies for
    tlc_dev_status *status;
    uint64_t wait_ns;
};

// Bounded wait on an mbarrier phase; gives up at once when the CTA is aborting.
__device__ __forceinline__ bool wait_bar(const Ctl &c, uint64_t *bar, uint32_t parity, int where) {
    if (*c.abort_flag) return false;  // once aborting, no stage is taken any more (the drain counts on it)
    if (mbar_try_wait(bar, parity)) return true;
    const uint64_t t0 = tlc_globaltimer_ns();
    for (;;) {
        for (int i = 0; i < 64; i++)
            if (mbar_try_wait(bar, parity)) return true;
        if (*c.abort_flag) return false;
        if (tlc_globaltimer_ns() - t0 > c.wait_ns) break;
    }
    *c.abort_flag = 1;
    if (atomicCAS(&c.status->code, 0, 1) == 0) c.status->where = where;
    return false;
}

__device__ __forceinline__ uint32_t ldcg_u32(const void *p) {
    uint32_t v;
    asm volatile("ld.global.cg.u32 %0, [%1];" : "=r"(v) : "l"(p));
    return v;
}

// One (KV head, key split) item of the decode attention, run by warps 0-3 of a CTA (tid =
// 0..127): the arithmetic of attention_kernel in tlc_attention.cu for one query per sequence.
// The tile of 16 rows holds the Gq query heads of the group (rows past Gq are padding).
// Tile 0 is already on its way into stage 0 when this is called.
template <int D, typename LoadTile>
__device__ __forceinline__ void attention_item(const StepParams &P, const __half *ks, const __half *vs, float *sm_m,
                                               float *sm_l, int hk, int split, int nsplit, int Gq, int pos,
                                               int k_begin, int k_end, int ntiles, LoadTile &&load_tile, int tid,
                                               int *sm_flag) {
    constexpr int PITCH = D + 8;
    constexpr int TILE = kTileKeys * PITCH;
    constexpr int KSTEPS = D / 16;
    constexpr int NDT = D / 8;
    const int warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, t = lane & 3;
    const bool valid_lo = g < Gq, valid_hi = g + 8 < Gq;
    const int head_lo = hk * Gq + (valid_lo ? g : 0), head_hi = hk * Gq + (valid_hi ? g + 8 : 0);

    uint32_t qa[KSTEPS][4];
    {
        const __half *q_lo = P.q + (size_t)head_lo * D, *q_hi = P.q + (size_t)head_hi * D;
#pragma unroll
        for (int kk = 0; kk < KSTEPS; kk++) {
            qa[kk][0] = valid_lo ? ldcg_u32(q_lo + 16 * kk + 2 * t) : 0u;
            qa[kk][1] = valid_hi ? ldcg_u32(q_hi + 16 * kk + 2 * t) : 0u;
            qa[kk][2] = valid_lo ? ldcg_u32(q_lo + 16 * kk + 8 + 2 * t) : 0u;
            qa[kk][3] = valid_hi ? ldcg_u32(q_hi + 16 * kk + 8 + 2 * t) : 0u;
        }
    }
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
    float o[NDT][4];
#pragma unroll
    for (int i = 0; i < NDT; i++) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    const __half scale_h = __float2half_rn(P.attn_scale);

    for (int tile = 0; tile < ntiles; tile++) {
        const int stage = tile & 1;
        if (tile + 1 < ntiles) {
            load_tile(tile + 1, stage ^ 1);
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        named_bar<128>(2);
        const int j0 = k_begin + tile * kTileKeys;
        const int kw0 = warp * 16;  // this warp's 16 keys of the tile
        if (j0 + kw0 < k_end) {
            const __half *kt = ks + stage * TILE;
            const __half *vt = vs + stage * TILE;
            float s[2][4];
#pragma unroll
            for (int i = 0; i < 2; i++) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
#pragma unroll
            for (int kk = 0; kk < KSTEPS; kk++) {
                uint32_t r[4];
                const int mi = lane >> 3;
                ldsm_x4(r, kt + (kw0 + (mi >> 1) * 8 + (lane & 7)) * PITCH + 16 * kk + (mi & 1) * 8);
                mma16816_acc(s[0], qa[kk], r[0], r[1]);
                mma16816_acc(s[1], qa[kk], r[2], r[3]);
            }
            // Scores: f16 rounding of the einsum output, f16 multiply by the scale (the scripts
            // multiply the f16 score tensor by 0.125), then the causal mask (key <= pos).
            float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
            for (int nt = 0; nt < 2; nt++)
#pragma unroll
                for (int e = 0; e < 4; e++) {
                    const int key = j0 + kw0 + nt * 8 + 2 * t + (e & 1);
                    float v = __half2float(__hmul(__float2half_rn(s[nt][e]), scale_h));
                    if (key >= k_end || key > pos) v = -INFINITY;
                    s[nt][e] = v;
                    mx[e >> 1] = fmaxf(mx[e >> 1], v);
                }
            float corr[2], msafe[2];
#pragma unroll
            for (int h = 0; h < 2; h++) {
                mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 1));
                mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 2));
                const float m_new = fmaxf(m_run[h], mx[h]);
                msafe[h] = m_new == -INFINITY ? 0.f : m_new;
                corr[h] = expf(m_run[h] - msafe[h]);
                m_run[h] = m_new;
            }
            float psum[2] = {0.f, 0.f};
#pragma unroll
            for (int nt = 0; nt < 2; nt++)
#pragma unroll
                for (int e = 0; e < 4; e++) {
                    const float pv = expf(s[nt][e] - msafe[e >> 1]);
                    s[nt][e] = pv;
                    psum[e >> 1] += pv;
                }
            l_run[0] = l_run[0] * corr[0] + psum[0];
            l_run[1] = l_run[1] * corr[1] + psum[1];
#pragma unroll
            for (int i = 0; i < NDT; i++) {
                o[i][0] *= corr[0];
                o[i][1] *= corr[0];
                o[i][2] *= corr[1];
                o[i][3] *= corr[1];
            }
            uint32_t pa[4];
            pa[0] = pack_half2(s[0][0], s[0][1]);
            pa[1] = pack_half2(s[0][2], s[0][3]);
            pa[2] = pack_half2(s[1][0], s[1][1]);
            pa[3] = pack_half2(s[1][2], s[1][3]);
#pragma unroll
            for (int jd = 0; jd < KSTEPS; jd++) {
                uint32_t r[4];
                const int mi = lane >> 3;
                ldsm_x4_trans(r, vt + (kw0 + (mi & 1) * 8 + (lane & 7)) * PITCH + 16 * jd + (mi >> 1) * 8);
                mma16816_acc(o[2 * jd], pa, r[0], r[1]);
                mma16816_acc(o[2 * jd + 1], pa, r[2], r[3]);
            }
        }
        named_bar<128>(2);
    }

    // ---- merge the 4 warps (each saw a different quarter of every tile) ----
#pragma unroll
    for (int h = 0; h < 2; h++) {
        l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 1);
        l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 2);
    }
    float *so = reinterpret_cast<float *>(const_cast<__half *>(ks));  // [4][16][D], reuses the K/V tiles
    if (t == 0) {
        sm_m[warp * 16 + g] = m_run[0];
        sm_m[warp * 16 + g + 8] = m_run[1];
        sm_l[warp * 16 + g] = l_run[0];
        sm_l[warp * 16 + g + 8] = l_run[1];
    }
#pragma unroll
    for (int i = 0; i < NDT; i++) {
        float *base = so + (size_t)warp * 16 * D;
        *reinterpret_cast<float2 *>(base + g * D + 8 * i + 2 * t) = make_float2(o[i][0], o[i][1]);
        *reinterpret_cast<float2 *>(base + (g + 8) * D + 8 * i + 2 * t) = make_float2(o[i][2], o[i][3]);
    }
    named_bar<128>(2);

    // thread -> (row, D/8 consecutive dims)
    constexpr int DPT = D / 8;
    const int row = tid >> 3, d0 = (tid & 7) * DPT;
    const bool row_valid = row < Gq;
    const int head = hk * Gq + (row_valid ? row : 0);
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < 4; w++) M = fmaxf(M, sm_m[w * 16 + row]);
    float Lsum = 0.f, acc[DPT];
#pragma unroll
    for (int j = 0; j < DPT; j++) acc[j] = 0.f;
#pragma unroll
    for (int w = 0; w < 4; w++) {
        const float wgt = sm_m[w * 16 + row] == -INFINITY ? 0.f : expf(sm_m[w * 16 + row] - M);
        Lsum += sm_l[w * 16 + row] * wgt;
#pragma unroll
        for (int j = 0; j < DPT; j++) acc[j] += so[((size_t)w * 16 + row) * D + d0 + j] * wgt;
    }
    if (nsplit == 1) {
        if (row_valid) {
            const float inv = Lsum > 0.f ? 1.0f / Lsum : 0.f;
#pragma unroll
            for (int j = 0; j < DPT; j++) P.attn[(size_t)head * D + d0 + j] = __float2half_rn(acc[j] * inv);
        }
        return;
    }
    // ---- split keys: publish the partial, the last CTA of the KV head merges ----
    if (row_valid) {
        const size_t pi = (size_t)head * nsplit + split;
        if ((tid & 7) == 0) {
            P.part_ml[pi * 2] = M;
            P.part_ml[pi * 2 + 1] = Lsum;
        }
#pragma unroll
        for (int j = 0; j < DPT; j++) P.part_o[pi * D + d0 + j] = acc[j];
    }
    __threadfence();
    named_bar<128>(2);
    if (tid == 0) {
        const int ticket = atomicAdd(P.tickets + hk, 1);
        const int last = ticket == nsplit - 1;
        if (last) P.tickets[hk] = 0;  // ready for the next layer
        *sm_flag = last;
    }
    named_bar<128>(2);
    if (!*reinterpret_cast<volatile int *>(sm_flag)) return;
    __threadfence();
    if (row_valid) {
        float Mg = -INFINITY;
        for (int sp = 0; sp < nsplit; sp++) Mg = fmaxf(Mg, ldcg_f32(&P.part_ml[((size_t)head * nsplit + sp) * 2]));
        float Lg = 0.f;
#pragma unroll
        for (int j = 0; j < DPT; j++) acc[j] = 0.f;
        for (int sp = 0; sp < nsplit; sp++) {
            const size_t pi = (size_t)head * nsplit + sp;
            const float ms = ldcg_f32(&P.part_ml[pi * 2]);
            const float wgt = ms == -INFINITY ? 0.f : expf(ms - Mg);
            Lg += ldcg_f32(&P.part_ml[pi * 2 + 1]) * wgt;
#pragma unroll
            for (int j = 0; j < DPT; j++) acc[j] += ldcg_f32(&P.part_o[pi * D + d0 + j]) * wgt;
        }
        const float inv = Lg > 0.f ? 1.0f / Lg : 0.f;
#pragma unroll
        for (int j = 0; j < DPT; j++) P.attn[(size_t)head * D + d0 + j] = __float2half_rn(acc[j] * inv);
    }
}

template <int QT>
__global__ void __launch_bounds__(kThreads, 1) decode_step_kernel(const StepParams P) {
    using T = QTraits<QT>;
    constexpr int TILE = T::TILE_BYTES;
    constexpr int STAGE_BYTES = kTilesPerStage * TILE;

    extern __shared__ __align__(128) uint8_t smem[];
    Ctl ctl;
    ctl.full = reinterpret_cast<uint64_t *>(smem);
    ctl.empty = reinterpret_cast<uint64_t *>(smem + 128);
    ctl.abort_flag = reinterpret_cast<volatile int *>(smem + 256);
    ctl.issued = reinterpret_cast<volatile int *>(smem + 260);
    ctl.status = P.status;
    ctl.wait_ns = P.wait_ns;
    int *scratch_i = reinterpret_cast<int *>(smem + 264);
    float *sq_part = reinterpret_cast<float *>(smem + 512);
    float *red = reinterpret_cast<float *>(smem + kOffRed);
    float *cand_v = reinterpret_cast<float *>(smem + kOffSmall);
    int *cand_i = reinterpret_cast<int *>(smem + kOffSmall + 64);
    float *sm_m = reinterpret_cast<float *>(smem + kOffSmall + 128);  // [4][16]
    float *sm_l = sm_m + 64;                                          // [4][16]
    __half *xres = reinterpret_cast<__half *>(smem + P.off_xres);
    __half *xin = reinterpret_cast<__half *>(smem + P.off_xin);
    float4 *cinit = reinterpret_cast<float4 *>(smem + P.off_cinit);
    uint4 *xperm = reinterpret_cast<uint4 *>(smem + P.off_xperm);
    uint8_t *attn_smem = smem + P.off_attn;
    uint8_t *stages = smem + P.off_ring;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int S = P.nstages;
    const int G = (int)gridDim.x, cta = (int)blockIdx.x;

    if (tid == 0) {
        for (int s = 0; s < S; s++) {
            mbar_init(&ctl.full[s], 1);
            mbar_init(&ctl.empty[s], CW);
        }
        *ctl.abort_flag = 0;
        *ctl.issued = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    __syncthreads();

    if (warp == CW) {
        // ================================ producer ================================
        int rs = 0, issued = 0;
        uint32_t rpar = 1;
        const uint64_t policy = l2_evict_first_policy();
        bool alive = true;
        for (int step = 0; step < P.steps && alive; step++) {
            for (int l = 0; l <= P.n_layers && alive; l++) {
                for (int ph = (l < P.n_layers ? 0 : 5); ph <= (l < P.n_layers ? 4 : 5) && alive; ph++) {
                    if (ph == 1) continue;
                    const Phase f = make_phase(P, P.layers + (l < P.n_layers ? l : 0), ph);
                    const int u_lo = (int)((long long)cta * f.units / G), u_hi = (int)((long long)(cta + 1) * f.units / G);
                    for (int u = u_lo; u < u_hi && alive; u++) {
                        for (int sub = 0; sub < f.subs && alive; sub++) {
                            int ti, sl;
                            unit_slab(f, u, sub, ti, sl);
                            const uint8_t *src = f.w[ti] + (size_t)sl * f.pitch[ti];
                            for (int c = 0; c < f.nchunks; c++) {
                                if (!__all_sync(0xffffffffu, wait_bar(ctl, &ctl.empty[rs], rpar, 1))) {
                                    alive = false;
                                    break;
                                }
                                const int ntiles = min(kTilesPerStage, f.ktiles - c * kTilesPerStage);
                                const uint32_t bytes = (uint32_t)(ntiles * TILE);
                                if (lane == 0) {
                                    mbar_expect_tx(&ctl.full[rs], bytes);
                                    bulk_g2s_hint(stages + (size_t)rs * STAGE_BYTES,
                                                  src + (size_t)c * (kTilesPerStage * TILE), bytes, &ctl.full[rs], policy);
                                    *ctl.issued = ++issued;
                                }
                                if (++rs == S) {
                                    rs = 0;
                                    rpar ^= 1u;
                                }
                            }
                        }
                    }
                }
            }
        }
        __syncwarp();
        named_bar<kThreads>(3);  // meet the consumers at the exit (they drain what is in flight)
        return;
    }

    // ================================== consumers ==================================
    const int ctid = tid;
    const int g = lane >> 2, t = lane & 3;
    int rs = 0, consumed = 0;
    uint32_t rpar = 0;
    uint32_t bar_target = ld_acquire_gpu(P.bar_base);  // the counter's value when this launch began
    bool ok = true;

    // Grid-wide barrier: every consumer thread's global stores, then one release-add per CTA on
    // the monotonic counter; thread 0 spins (bounded) until all CTAs of this round have arrived.
    auto grid_barrier = [&](int where) -> bool {
        bar_target += (uint32_t)G;
        consumer_bar<CT>();
        if (ctid == 0) {
            red_release_gpu_add(P.bar_counter, 1u);
            const uint64_t t0 = tlc_globaltimer_ns();
            bool done = false;
            for (long it = 0;; it++) {
                if ((int32_t)(ld_acquire_gpu(P.bar_counter) - bar_target) >= 0) {
                    done = true;
                    break;
                }
                if ((it & 63) == 63) {
                    if (*reinterpret_cast<volatile int *>(&P.status->code) != 0) break;  // another CTA gave up
                    if (tlc_globaltimer_ns() - t0 > P.wait_ns) {
                        if (atomicCAS(&P.status->code, 0, 2) == 0) P.status->where = where;
                        break;
                    }
                }
            }
            if (!done) *ctl.abort_flag = 1;
        }
        consumer_bar<CT>();
        return *ctl.abort_flag == 0;
    };

    // Input vector of a phase: K f16 values from global memory (written by other CTAs: loads
    // bypass the L1), optionally RMS-normalised, into fragment order + accumulator start values.
    auto load_input = [&](const __half *src, int k, int nblk, int nblk_pad, const __half *norm_w, bool keep) {
        float sq = 0.f;
        for (int i = ctid * 8; i < k; i += CT * 8) {
            const uint4 raw = ldcg_u128(src + i);
            *reinterpret_cast<uint4 *>(xin + i) = raw;
            if (keep) *reinterpret_cast<uint4 *>(xres + i) = raw;
            if (norm_w) {
                const __half2 *h = reinterpret_cast<const __half2 *>(&raw);
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    const float2 v = __half22float2(h[j]);
                    sq = fmaf(v.x, v.x, sq);
                    sq = fmaf(v.y, v.y, sq);
                }
            }
        }
        if (norm_w) {
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
            if (lane == 0) sq_part[warp] = sq;
        }
        consumer_bar<CT>();
        float inv = 1.f;
        if (norm_w) {
            float ss = 0.f;
#pragma unroll
            for (int w = 0; w < CW; w++) ss += sq_part[w];
            inv = 1.0f / sqrtf(ss / (float)k + P.eps);
        }
        const int items = nblk_pad * 4;
        for (int idx = ctid; idx < ((items + 31) & ~31); idx += CT) {
            const bool live = idx < items;
            const int tt = idx & 3, b = idx >> 2;
            float v[8];
#pragma unroll
            for (int j = 0; j < 8; j++) v[j] = 0.f;
            if (live && b < nblk) {
                const __half *xr = xin + b * 32;
                __align__(16) __half raw[8], nw[8];
                if (QT == TLC_TYPE_Q4_0) {
                    *reinterpret_cast<uint2 *>(&raw[0]) = *reinterpret_cast<const uint2 *>(xr + 4 * tt);
                    *reinterpret_cast<uint2 *>(&raw[4]) = *reinterpret_cast<const uint2 *>(xr + 16 + 4 * tt);
                    if (norm_w) {
                        *reinterpret_cast<uint2 *>(&nw[0]) = *reinterpret_cast<const uint2 *>(norm_w + b * 32 + 4 * tt);
                        *reinterpret_cast<uint2 *>(&nw[4]) = *reinterpret_cast<const uint2 *>(norm_w + b * 32 + 16 + 4 * tt);
                    }
                } else {
                    *reinterpret_cast<uint4 *>(&raw[0]) = *reinterpret_cast<const uint4 *>(xr + 8 * tt);
                    if (norm_w) *reinterpret_cast<uint4 *>(&nw[0]) = *reinterpret_cast<const uint4 *>(norm_w + b * 32 + 8 * tt);
                }
                float f[8];
#pragma unroll
                for (int j = 0; j < 8; j++) {
                    f[j] = __half2float(raw[j]);
                    // f16((x * inv) * w): two separately rounded f32 multiplies, then RNE
                    // (Tensor::rms_norm_cpu, src/ops/normalization.rs:236-240).
                    if (norm_w) f[j] = __half2float(__float2half_rn(__fmul_rn(__fmul_rn(f[j], inv), __half2float(nw[j]))));
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
                uint4 o;
                o.x = pack_half2(v[0], v[1]);  // exact: v[] are f16 values
                o.y = pack_half2(v[2], v[3]);
                o.z = pack_half2(v[4], v[5]);
                o.w = pack_half2(v[6], v[7]);
                xperm[idx] = o;
                if (tt == 0) {
                    const float cv = -T::OFFSET * 5.9604644775390625e-08f * s;  // * 2^-24
                    cinit[b] = make_float4(cv, cv, cv, cv);
                }
            }
        }
        consumer_bar<CT>();
    };

    const uint32_t xp_base = smem_u32(xperm) + (uint32_t)t * 16u;
    const uint32_t ci_base = smem_u32(cinit);
    const uint32_t stages_addr = smem_u32(stages);

    // Dot products of one 16-row slab with the activation vector: this warp's share of the
    // slab's tiles, summed into (row g, row g + 8).  A wait that ran out (the CTA's abort flag
    // is then up) skips the math but keeps walking the schedule, so that every warp still
    // reaches the same bar.sync calls; the callers test the flag right after those.
    auto slab_dot = [&](const Phase &f, float &acc_lo, float &acc_hi) {
        acc_lo = 0.f;
        acc_hi = 0.f;
        for (int c = 0; c < f.nchunks; c++) {
            const bool ready = __all_sync(0xffffffffu, wait_bar(ctl, &ctl.full[rs], rpar, 2));
            const int ntiles = ready ? min(kTilesPerStage, f.ktiles - c * kTilesPerStage) : 0;
            const uint32_t sbase = stages_addr + (uint32_t)rs * STAGE_BYTES;
            for (int ti = warp; ti < ntiles; ti += CW) {
                const uint32_t tb = sbase + (uint32_t)ti * TILE;
                const uint4 vlo = lds_u128(tb + lane * 16), vhi = lds_u128(tb + 512 + lane * 16);
                uint32_t slo[2], shi[2];
                if (QT == TLC_TYPE_Q4_0) {
                    const uint2 a = lds_u64(tb + 1024 + g * 8), b = lds_u64(tb + 1024 + (g + 8) * 8);
                    slo[0] = a.x; slo[1] = a.y; shi[0] = b.x; shi[1] = b.y;
                } else {
                    slo[0] = lds_u32(tb + 1024 + g * 4);
                    shi[0] = lds_u32(tb + 1024 + (g + 8) * 4);
                    slo[1] = shi[1] = 0;
                }
                const uint32_t lo[4] = {vlo.x, vlo.y, vlo.z, vlo.w};
                const uint32_t hi[4] = {vhi.x, vhi.y, vhi.z, vhi.w};
                float dlo[4], dhi[4];
#pragma unroll
                for (int h = 0; h < T::TB / 2; h++) {
                    const float2 l2 = __half22float2(*reinterpret_cast<const __half2 *>(&slo[h]));
                    const float2 u2 = __half22float2(*reinterpret_cast<const __half2 *>(&shi[h]));
                    dlo[2 * h] = l2.x; dlo[2 * h + 1] = l2.y;
                    dhi[2 * h] = u2.x; dhi[2 * h + 1] = u2.y;
                }
                const uint32_t b0 = (uint32_t)((c * kTilesPerStage + ti) * T::TB);  // first block of the tile
                const uint32_t xa = xp_base + b0 * 64u, ca = ci_base + b0 * 16u;
                uint4 xp = lds_u128(xa);
                uint4 ci = lds_u128(ca);
#pragma unroll
                for (int j = 0; j < T::TB; j++) {
                    uint32_t w0[2], w1[2], a1[4], a2[4];
                    if (QT == TLC_TYPE_Q4_0) {
                        w0[0] = lo[j]; w1[0] = hi[j]; w0[1] = w1[1] = 0;
                    } else {
                        w0[0] = lo[2 * j]; w0[1] = lo[2 * j + 1];
                        w1[0] = hi[2 * j]; w1[1] = hi[2 * j + 1];
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
                    acc_lo = fmaf(dlo[j], d2[0], acc_lo);  // column 0 of the tile: rows g and g + 8
                    acc_hi = fmaf(dhi[j], d2[2], acc_hi);
                }
            }
            __syncwarp();
            if (ready) {
                if (lane == 0) mbar_arrive(&ctl.empty[rs]);
                consumed++;
            }
            if (++rs == S) {
                rs = 0;
                rpar ^= 1u;
            }
        }
    };

    // A whole GEMV phase: this CTA's units in batches of up to kBatchSlabs slabs, one cross-warp
    // reduction per batch, then `epilogue(unit, sub-slab index in batch, row, total...)`.
    // epi(u, row, v0, v0_pair, v1): v0 = row's dot product of sub 0 (already * 2^24), v0_pair =
    // the one of row ^ 1, v1 = sub 1's (gate/up pairs only).
    auto gemv_phase = [&](const Phase &f, auto &&epi) -> bool {
        const int u_lo = (int)((long long)cta * f.units / G), u_hi = (int)((long long)(cta + 1) * f.units / G);
        const int ub = kBatchSlabs / f.subs;
        int batch_no = 0;
        for (int u0 = u_lo; u0 < u_hi; u0 += ub, batch_no++) {
            const int nu = min(ub, u_hi - u0);
            float *rbuf = red + (size_t)(batch_no & 1) * (CW * kBatchSlabs * 16);
            for (int a = 0; a < nu * f.subs; a++) {
                float lo, hi;
                slab_dot(f, lo, hi);
                if (t == 0) {
                    rbuf[(warp * kBatchSlabs + a) * 16 + g] = lo;
                    rbuf[(warp * kBatchSlabs + a) * 16 + g + 8] = hi;
                }
            }
            consumer_bar<CT>();
            // Same answer in every warp: a flag raised after this barrier needs a full wait
            // limit (milliseconds at least) to come up, the reads below take nanoseconds.
            if (*ctl.abort_flag) return false;
            for (int item = ctid; item < nu * 16; item += CT) {
                const int ui = item >> 4, row = item & 15;
                auto total = [&](int set, int r_) {
                    float v = 0.f;
#pragma unroll
                    for (int w = 0; w < CW; w++) v += rbuf[(w * kBatchSlabs + set) * 16 + r_];
                    return v * 16777216.0f;  // undo the 2^-24 of the integer fragments
                };
                const int a0 = ui * f.subs;
                epi(u0 + ui, row, total(a0, row), total(a0, row ^ 1), f.subs == 2 ? total(a0 + 1, row) : 0.f);
            }
        }
        return true;
    };

    for (int step = 0; step < P.steps && ok; step++) {
        // The token to feed and its position: written by the previous step's phase G
        // (or by the host before the launch).
        const int *ids = P.ids_src ? P.ids_src : P.ids;
        int tok = ldcg_i32(ids);
        tok = tok < 0 ? 0 : (tok >= P.vocab ? P.vocab - 1 : tok);  // validated on the host; never read outside
        const int pos = ldcg_i32(P.positions);
        const bool pos_ok = pos >= 0 && pos < P.Tmax;
        if (!pos_ok && ctid == 0 && atomicCAS(&P.status->code, 0, TLC_DEV_INDEX) == 0) P.status->where = 310;
        const int T_keys = pos_ok ? pos + 1 : 1;

        for (int l = 0; l < P.n_layers && ok; l++) {
            const StepLayer *L = P.layers + l;
            // ---- A: rms_norm + q/k/v + rope + cache append ----
            {
                const Phase f = make_phase(P, L, 0);
                const __half *src = l == 0 ? reinterpret_cast<const __half *>(P.embd + (size_t)tok * P.embd_pitch) : P.x;
                load_input(src, f.k, f.nblk, f.ktiles * P.tb, L->attn_norm, true);
                const int hd = P.D;
                ok = gemv_phase(f, [&](int u, int row, float v0, float vp, float) {
                    int ti, sl;
                    unit_slab(f, u, 0, ti, sl);
                    const int n = sl * kRows + row;
                    if (n >= f.n[ti]) return;
                    __half h = __float2half_rn(v0);
                    if (ti < 2) {
                        // Interleaved RoPE on the f16-rounded projection (rope_f16,
                        // shaders/unified.metal:2355-2417), at the token's true position.
                        const __half hp = __float2half_rn(vp);
                        const int dim = n % hd, pair = dim >> 1;
                        const float x0 = __half2float((dim & 1) ? hp : h), x1 = __half2float((dim & 1) ? h : hp);
                        const float freq = 1.0f / powf(P.rope_base, (float)(2 * pair) / (float)hd);
                        const float theta = (float)(unsigned)pos * freq;
                        const float cs = cosf(theta), sn = sinf(theta);
                        const float r = (dim & 1) ? __fadd_rn(__fmul_rn(x0, sn), __fmul_rn(x1, cs))
                                                  : __fsub_rn(__fmul_rn(x0, cs), __fmul_rn(x1, sn));
                        h = __float2half_rn(r);
                    }
                    if (ti == 0)
                        P.q[n] = h;
                    else if (pos_ok)
                        (ti == 1 ? L->kc : L->vc)[(size_t)pos * P.kvd + n] = h;
                });
                if (!ok) break;
            }
            // ---- B: attention ----
            // (KV head, key split) items over the CTAs; warps 0-3 of an item's CTA do the work.
            const int tiles_total = (T_keys + kTileKeys - 1) / kTileKeys;
            int nsplit = G / P.Hkv;
            nsplit = nsplit < 1 ? 1 : nsplit > tiles_total ? tiles_total : nsplit;
            nsplit = nsplit > P.max_splits ? P.max_splits : nsplit;
            const int keys_per_split = ((tiles_total + nsplit - 1) / nsplit) * kTileKeys;
            const bool has_item = cta < P.Hkv * nsplit;
            const int hk = cta / nsplit, split = cta % nsplit;
            const int k_begin = split * keys_per_split;
            const int k_end = min(T_keys, k_begin + keys_per_split);
            const int ntiles = has_item && k_end > k_begin ? (k_end - k_begin + kTileKeys - 1) / kTileKeys : 0;
            const int D = P.D;
            const int PITCH = D + 8, TILEH = kTileKeys * PITCH;
            __half *ks = reinterpret_cast<__half *>(attn_smem), *vs = ks + 2 * TILEH;
            const __half *kbase = L->kc + (size_t)hk * D, *vbase = L->vc + (size_t)hk * D;
            const size_t key_stride = (size_t)P.kvd;
            auto load_kv_tile = [&](int tile, int stage) {
                const int j0 = k_begin + tile * kTileKeys;
                const int chunks = kTileKeys * (D / 8);
                for (int c = ctid; c < chunks; c += 128) {
                    const int key = c / (D / 8), part = c % (D / 8);
                    const bool in = j0 + key < k_end;
                    const size_t off = (size_t)(in ? j0 + key : 0) * key_stride + part * 8;
                    cp_async16(ks + stage * TILEH + key * PITCH + part * 8, kbase + off, in);
                    cp_async16(vs + stage * TILEH + key * PITCH + part * 8, vbase + off, in);
                }
                cp_async_commit();
            };
            // A first tile made of rows of earlier steps only does not depend on phase A: it is
            // fetched before the barrier.
            const bool early = ntiles > 0 && warp < 4 && k_begin + kTileKeys <= pos;
            if (early) load_kv_tile(0, 0);
            if (!(ok = grid_barrier(10))) break;
            if (has_item && warp < 4) {
                const int Gq = P.H / P.Hkv;  // query heads per KV head (rows of the tile that are real)
                if (ntiles > 0 && !early) load_kv_tile(0, 0);
                if (D == 64)
                    attention_item<64>(P, ks, vs, sm_m, sm_l, hk, split, nsplit, Gq, pos, k_begin, k_end, ntiles,
                                       load_kv_tile, ctid, scratch_i);
                else
                    attention_item<128>(P, ks, vs, sm_m, sm_l, hk, split, nsplit, Gq, pos, k_begin, k_end, ntiles,
                                        load_kv_tile, ctid, scratch_i);
            }
            if (!(ok = grid_barrier(11))) break;
            // ---- C: o projection + residual ----
            {
                const Phase f = make_phase(P, L, 2);
                load_input(P.attn, f.k, f.nblk, f.ktiles * P.tb, nullptr, false);
                ok = gemv_phase(f, [&](int u, int row, float v0, float, float) {
                    const int n = u * kRows + row;
                    if (n < f.n[0]) P.x1[n] = __hadd(__float2half_rn(v0), xres[n]);
                });
                if (!ok || !(ok = grid_barrier(12))) break;
            }
            // ---- D: rms_norm + gate/up + silu*mul ----
            {
                const Phase f = make_phase(P, L, 3);
                load_input(P.x1, f.k, f.nblk, f.ktiles * P.tb, L->ffn_norm, true);
                ok = gemv_phase(f, [&](int u, int row, float v0, float, float v1) {
                    const int n = u * kRows + row;
                    if (n >= f.n[0]) return;
                    // h = gate; s = sigmoid(g) (f32, RNE); a = g*s; act = a*u: three f16
                    // roundings as in debug/chat_demo_with_kvcache.tl:26-41.
                    const __half gate = __float2half_rn(v0), up = __float2half_rn(v1);
                    const __half sg = __float2half_rn(1.0f / (1.0f + expf(-__half2float(gate))));
                    P.act[n] = __hmul(__hmul(gate, sg), up);
                });
                if (!ok || !(ok = grid_barrier(13))) break;
            }
            // ---- E: down projection + residual ----
            {
                const Phase f = make_phase(P, L, 4);
                load_input(P.act, f.k, f.nblk, f.ktiles * P.tb, nullptr, false);
                ok = gemv_phase(f, [&](int u, int row, float v0, float, float) {
                    const int n = u * kRows + row;
                    if (n < f.n[0]) P.x[n] = __hadd(__float2half_rn(v0), xres[n]);
                });
                if (!ok || !(ok = grid_barrier(14))) break;
            }
        }
        if (!ok) break;
        // ---- F: rms_norm + lm_head, local argmax ----
        {
            const Phase f = make_phase(P, P.layers, 5);
            load_input(P.x, f.k, f.nblk, f.ktiles * P.tb, P.out_norm, false);
            float best = -INFINITY;
            int bi = -1;
            ok = gemv_phase(f, [&](int u, int row, float v0, float, float) {
                const int n = u * kRows + row;
                if (n >= f.n[0]) return;
                const __half h = __float2half_rn(v0);
                P.logits[n] = h;
                const float v = __half2float(h);
                if (bi < 0 || !(v < best)) {  // a thread meets its rows in increasing order: later index wins ties
                    best = v;
                    bi = n;
                }
            });
            if (!ok) break;
            // Ties go to the LAST maximal index, like Iterator::max_by in temperature_sample's
            // greedy arm (src/interpreter/builtin_sampling.rs:176-181).
            auto better = [](float v, int i, float bv, int bidx) {
                if (bidx < 0) return i >= 0;
                if (i < 0) return false;
                if (v > bv) return true;
                if (v < bv) return false;
                return i > bidx;
            };
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                const float ov = __shfl_xor_sync(0xffffffffu, best, o);
                const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
                if (better(ov, oi, best, bi)) { best = ov; bi = oi; }
            }
            if (lane == 0) { cand_v[warp] = best; cand_i[warp] = bi; }
            consumer_bar<CT>();
            if (ctid == 0) {
                for (int w = 1; w < CW; w++)
                    if (better(cand_v[w], cand_i[w], best, bi)) { best = cand_v[w]; bi = cand_i[w]; }
                P.cand_val[cta] = best;
                P.cand_idx[cta] = bi;
            }
            if (!(ok = grid_barrier(15))) break;
            // ---- G: the token, the bookkeeping, the report to the host ----
            if (cta == 0) {
                best = -INFINITY;
                bi = -1;
                for (int i = ctid; i < G; i += CT) {
                    const float v = ldcg_f32(P.cand_val + i);
                    const int idx = ldcg_i32(P.cand_idx + i);
                    if (better(v, idx, best, bi)) { best = v; bi = idx; }
                }
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) {
                    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
                    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
                    if (better(ov, oi, best, bi)) { best = ov; bi = oi; }
                }
                consumer_bar<CT>();  // cand_v / cand_i of phase F have been read
                if (lane == 0) { cand_v[warp] = best; cand_i[warp] = bi; }
                consumer_bar<CT>();
                if (ctid == 0) {
                    for (int w = 1; w < CW; w++)
                        if (better(cand_v[w], cand_i[w], best, bi)) { best = cand_v[w]; bi = cand_i[w]; }
                    if (bi < 0) bi = 0;
                    P.next_ids[0] = bi;
                    if (P.advance) {
                        P.ids[0] = bi;
                        P.positions[0] = pos + 1;
                    }
                    if (P.host_next && step == P.steps - 1) {
                        if (P.host_status) {
                            P.host_status->code = *reinterpret_cast<volatile int *>(&P.status->code);
                            P.host_status->where = *reinterpret_cast<volatile int *>(&P.status->where);
                        }
                        __threadfence_system();
                        *reinterpret_cast<volatile int *>(P.host_next) = bi;
                    }
                }
            }
            if (step + 1 < P.steps)
                if (!(ok = grid_barrier(16))) break;
        }
    }

    // The next launch starts counting where this one stopped (the host zeroes both words
    // after a launch that gave up).
    if (ok && cta == 0 && ctid == 0) *P.bar_base = bar_target;
    if (!ok) *ctl.abort_flag = 1;  // the producer stops at its next wait
    named_bar<kThreads>(3);
    if (!ok && ctid == 0) {
        // Copies the producer started and nobody consumed must land before this CTA's shared
        // memory goes away.
        const int issued = *ctl.issued;
        for (int i = consumed; i < issued; i++) {
            const int s = i % S;
            const uint32_t par = (uint32_t)((i / S) & 1);
            const uint64_t t0 = tlc_globaltimer_ns();
            while (!mbar_try_wait(&ctl.full[s], par) && tlc_globaltimer_ns() - t0 < 1000000ull) {
            }
        }
    }
}

}  // namespace tlc_step

// ---- host side ----------------------------------------------------------------------------

namespace tlc_step {

StepWorkspace step_workspace(int n_heads, int head_dim, int n_kv_heads, int max_splits, int grid) {
    StepWorkspace w{};
    size_t off = 0;
    auto take = [&](size_t bytes) {
        const size_t at = off;
        off = align_up(off + bytes, 256);
        return at;
    };
    w.part_ml = take((size_t)n_heads * max_splits * 2 * sizeof(float));
    w.part_o = take((size_t)n_heads * max_splits * head_dim * sizeof(float));
    w.tickets = take((size_t)n_kv_heads * sizeof(int));
    w.cand_val = take((size_t)grid * sizeof(float));
    w.cand_idx = take((size_t)grid * sizeof(int));
    w.bar = take(2 * sizeof(uint32_t));
    w.total = off;
    return w;
}

template <int QT>
static int32_t configure(tlc_ctx *ctx, int *blocks_per_sm, size_t smem) {
    static bool configured[64] = {};
    if (!configured[ctx->device & 63]) {
        TLC_CUDA(cudaFuncSetAttribute(decode_step_kernel<QT>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      (int)ctx->prop.sharedMemPerBlockOptin));
        TLC_CUDA(cudaFuncSetAttribute(decode_step_kernel<QT>, cudaFuncAttributePreferredSharedMemoryCarveout,
                                      cudaSharedmemCarveoutMaxShared));
        configured[ctx->device & 63] = true;
    }
    TLC_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(blocks_per_sm, decode_step_kernel<QT>, kThreads, smem));
    return TLC_OK;
}

static SmemPlan plan_for(tlc_ctx *ctx, int qtype, int d, int kmax, int head_dim) {
    const int tb = qtype == TLC_TYPE_Q4_0 ? QTraits<TLC_TYPE_Q4_0>::TB : QTraits<TLC_TYPE_Q8_0>::TB;
    const int tile = qtype == TLC_TYPE_Q4_0 ? QTraits<TLC_TYPE_Q4_0>::TILE_BYTES : QTraits<TLC_TYPE_Q8_0>::TILE_BYTES;
    return plan_smem(d, kmax, head_dim, kTilesPerStage * tile, tb, (size_t)ctx->prop.sharedMemPerBlockOptin);
}

bool step_supported(tlc_ctx *ctx, int qtype, int d, int kmax, int head_dim, int *grid_out) {
    if (qtype != TLC_TYPE_Q4_0 && qtype != TLC_TYPE_Q8_0) return false;
    if (head_dim != 64 && head_dim != 128) return false;
    if (d % 32 != 0 || kmax % 32 != 0) return false;
    int coop = 0;
    if (cudaDeviceGetAttribute(&coop, cudaDevAttrCooperativeLaunch, ctx->device) != cudaSuccess || !coop) return false;
    const SmemPlan s = plan_for(ctx, qtype, d, kmax, head_dim);
    if (s.stages < 3) return false;
    int per_sm = 0;
    const int32_t rc = qtype == TLC_TYPE_Q4_0 ? configure<TLC_TYPE_Q4_0>(ctx, &per_sm, s.total)
                                              : configure<TLC_TYPE_Q8_0>(ctx, &per_sm, s.total);
    if (rc != TLC_OK) {
        tlc_clear_error();
        return false;
    }
    if (per_sm < 1) return false;
    if (grid_out) *grid_out = ctx->sm_count;
    return true;
}

int32_t step_launch(tlc_ctx *ctx, int qtype, int grid, int kmax, StepParams &p) {
    const SmemPlan s = plan_for(ctx, qtype, p.d, kmax, p.D);
    TLC_REQUIRE(s.stages >= 3, TLC_ERR_INVALID_OPERATION, "decode step kernel: shared memory too small for K = %d", kmax);
    p.nstages = s.stages;
    p.off_xres = (uint32_t)s.xres;
    p.off_xin = (uint32_t)s.xin;
    p.off_cinit = (uint32_t)s.cinit;
    p.off_xperm = (uint32_t)s.xperm;
    p.off_attn = (uint32_t)s.attn;
    p.off_ring = (uint32_t)s.ring;
    p.tb = qtype == TLC_TYPE_Q4_0 ? QTraits<TLC_TYPE_Q4_0>::TB : QTraits<TLC_TYPE_Q8_0>::TB;
    p.tile_bytes = qtype == TLC_TYPE_Q4_0 ? QTraits<TLC_TYPE_Q4_0>::TILE_BYTES : QTraits<TLC_TYPE_Q8_0>::TILE_BYTES;
    p.status = ctx->dev_status;
    p.wait_ns = ctx->wait_ns;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)grid);
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = s.total;
    cfg.stream = ctx->stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeCooperative;  // all CTAs resident at once: they wait on one another
    attr[0].val.cooperative = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    const cudaError_t le = qtype == TLC_TYPE_Q4_0 ? cudaLaunchKernelEx(&cfg, decode_step_kernel<TLC_TYPE_Q4_0>, p)
                                                  : cudaLaunchKernelEx(&cfg, decode_step_kernel<TLC_TYPE_Q8_0>, p);
    if (le != cudaSuccess) {
        cudaGetLastError();
        return tlc_fail(TLC_ERR_CUDA, "decode step launch failed: %s", cudaGetErrorString(le));
    }
    TLC_CHECK_LAUNCH(ctx);
    return TLC_OK;
}

}  // namespace tlc_step
