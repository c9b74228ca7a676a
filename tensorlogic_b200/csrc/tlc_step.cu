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
// then  F  rms_norm + lm_head  and  G  greedy sample + bookkeeping -- runs in one grid of
// one CTA per SM, all resident at once (a cooperative launch).
//
// Data flow instead of barriers.  What one phase hands to the next (2 to 11 KB) travels as
// flagged words: 4 bytes of data and a 32-bit epoch number in one 8-byte store (tlc_step.h).
// A consumer polls exactly the words it needs until they carry the epoch of the current
// (step, layer, phase); there is no grid barrier, no atomic and no fence on that path, so a
// hand-over costs one store to L2 and one load from it.  Write-after-read is safe by
// construction: a CTA that writes buffer X in phase P+2 has seen every output of phase P+1,
// whose writers had all finished reading X in phase P.
//
// Weights.  In every CTA one producer warp walks the CTA's share of ALL the step's weight
// tiles in schedule order and streams them into a shared-memory ring with bulk async
// copies; weights are immutable, so it never waits for data and the ring already holds the
// next phase's tiles when the consumers get there.  Eight consumer warps do the math of
// tlc_gemv_kernel.cuh (one activation row): nibbles and bytes become exact f16 tensor-core
// fragments, the K range of a 16-row slab is split over the warps, one cross-warp reduction
// per batch of slabs, epilogue, flagged store.
//
// Attention is the flash-decoding of tlc_attention.cu: (KV head, key split) items on the
// first CTAs, which read q and the newest K/V row as flagged words (older rows from the
// cache) and publish partial (max, sum, O) as flagged f32 words; one merger CTA per query
// head (taken from the end of the grid) polls them and publishes the head's output.
//
// One sequence, greedy sampling, no tensor parallelism, all quantized linears of one
// type; anything else takes the kernel-by-kernel path of tlc_llama.cu.  `steps` decode
// steps can run inside one launch.  Every wait (mbarrier, flagged word) is bounded in
// time: a wait that runs out raises the device status word, every CTA sees it in its own
// polls, drains its copies and returns; the host reports TLC_ERR_TIMEOUT.
#include <cuda_fp16.h>

#include <cstdlib>

#include "tlc_gemv_common.cuh"
#include "tlc_internal.h"
#include "tlc_step.h"

namespace tlc_step {

using namespace tlc_gemv;

constexpr int kMaxCW = 16;            // most consumer warps a variant uses (shared-memory layout is sized for it)
constexpr int kBatchSlabs = 8;        // slabs per cross-warp reduction
constexpr int kTileKeys = 64;

// Epoch slots inside a layer's block of 8, and after the last layer.
enum { kSlotQKV = 1, kSlotPart = 2, kSlotAttn = 3, kSlotX1 = 4, kSlotAct = 5, kSlotX = 6, kSlotCand = 1, kSlotTok = 2 };

// ---- shared memory layout ---------------------------------------------------------------
//   0     full[12]   128  empty[12]   256 abort flag, 260 issued stages, 264 token, 268 scratch
//   512   sq_part[CW]
//   1024  red [2][CW][kBatchSlabs][16] f32
//   ...   cand_v[CW] / cand_i[CW], sm_m / sm_l [4][16] (attention merge), rope (cos, sin) [D/2]
//   ...   xres  f16 [d]           raw input of the last normalised phase (the residual)
//   ...   cinit float4 [kmax/32 padded]
//   ...   xperm uint4 [kmax/32 padded][4]
//   ...   attention K/V tiles [2][2][64][D+8] f16 (reused as the 4 warps' O partials)
//   ...   ring [stages][16 tiles]
constexpr size_t kOffRed = 1024;
constexpr size_t kOffSmall = kOffRed + (size_t)2 * kMaxCW * kBatchSlabs * 16 * sizeof(float);
constexpr size_t kOffRope = kOffSmall + 1024;  // float2 [64]
constexpr size_t kOffXres = kOffSmall + 2048;

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
    s.cinit = s.xin;  // (no staging copy of the input any more: it stays in registers)
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


// ---- flagged words --------------------------------------------------------------------------
__device__ __forceinline__ void fw_store(uint2 *p, uint32_t data, uint32_t epoch) {
    asm volatile("st.volatile.global.v2.u32 [%0], {%1,%2};" ::"l"(p), "r"(data), "r"(epoch) : "memory");
}
__device__ __forceinline__ void fw_store2(uint4 *p, uint32_t a, uint32_t b, uint32_t epoch) {
    asm volatile("st.volatile.global.v4.u32 [%0], {%1,%2,%3,%2};" ::"l"(p), "r"(a), "r"(epoch), "r"(b) : "memory");
}
__device__ __forceinline__ uint2 fw_load(const uint2 *p) {
    uint2 v;
    asm volatile("ld.volatile.global.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ uint4 fw_load2(const void *p) {  // two adjacent words (16-byte aligned)
    uint4 v;
    asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ uint32_t half2_bits(__half a, __half b) {
    __half2 h = __halves2half2(a, b);
    return *reinterpret_cast<uint32_t *>(&h);
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
    // Wait limit in SM clock cycles (the limit in ns times two: the SM clock stays below
    // 2 GHz, so a wait lasts at least the limit).  Waits are timed with the SM's own cycle
    // counter: reading the global nanosecond timer costs far more than a poll.
    long long wait_cycles;
    unsigned backoff;  // ns to sleep between two polls of a flagged word (0: none)
};

// Bounded wait on an mbarrier phase; gives up at once when the CTA is aborting.
__device__ __forceinline__ bool wait_bar(const Ctl &c, uint64_t *bar, uint32_t parity, int where) {
    if (*c.abort_flag) return false;  // once aborting, no stage is taken any more (the drain counts on it)
    if (mbar_try_wait(bar, parity)) return true;
    const long long t0 = clock64();
    for (;;) {
        for (int i = 0; i < 64; i++)
            if (mbar_try_wait(bar, parity)) return true;
        if (*c.abort_flag) return false;
        if (clock64() - t0 > c.wait_cycles) break;
    }
    *c.abort_flag = 1;
    if (atomicCAS(&c.status->code, 0, 1) == 0) c.status->where = where;
    return false;
}


// Polls a flagged word (pair of words) until it carries `epoch`.  Gives up -- raising the CTA's
// abort flag -- when the CTA is already aborting, when another CTA has reported a failure, or
// after the wait limit.  The value returned after a failure is meaningless; the callers test
// the abort flag at their next CTA-wide barrier.
__device__ __forceinline__ bool fw_giveup(const Ctl &c, long long t0, int where) {
    if (*c.abort_flag) return true;
    if (*reinterpret_cast<volatile int *>(&c.status->code) != 0) {  // another CTA gave up
        *c.abort_flag = 1;
        return true;
    }
    if (clock64() - t0 > c.wait_cycles) {
        *c.abort_flag = 1;
        if (atomicCAS(&c.status->code, 0, 2) == 0) c.status->where = where;
        return true;
    }
    return false;
}
__device__ __noinline__ uint2 fw_wait_slow(const Ctl &c, const uint2 *p, uint32_t epoch, int where) {
    const long long t0 = clock64();
    uint2 v;
    for (int it = 0;; it++) {
        v = fw_load(p);
        if (v.y == epoch) break;
        if (c.backoff) __nanosleep(c.backoff);
        if ((it & 63) == 63 && fw_giveup(c, t0, where)) break;
    }
    return v;
}
__device__ __noinline__ uint4 fw_wait2_slow(const Ctl &c, const void *p, uint32_t epoch, int where) {
    const long long t0 = clock64();
    uint4 v;
    for (int it = 0;; it++) {
        v = fw_load2(p);
        if (v.y == epoch && v.w == epoch) break;
        if (c.backoff) __nanosleep(c.backoff);
        if ((it & 63) == 63 && fw_giveup(c, t0, where)) break;
    }
    return v;
}
__device__ __forceinline__ uint32_t fw_wait(const Ctl &c, const uint2 *p, uint32_t epoch, int where) {
    uint2 v = fw_load(p);
    if (v.y != epoch) v = fw_wait_slow(c, p, epoch, where);
    return v.x;
}

// One (KV head, key split) item of the decode attention, run by warps 0-3 of a CTA (tid =
// 0..127): the arithmetic of attention_kernel in tlc_attention.cu for one query per sequence.
// The tile of 16 rows holds the Gq query heads of the group (rows past Gq are padding).
// q and the newest K/V row (position `pos`) arrive as flagged words of epoch e_in; tile 0 is
// already on its way into stage 0 when this is called.  The result goes out as flagged words:
// with several splits the partial (max, sum, O) of every head, epoch e_part; with one split
// the finished head outputs, epoch e_out.
template <int D, typename LoadTile>
__device__ __forceinline__ void attention_item(const StepParams &P, const Ctl &ctl, __half *ks, __half *vs, float *sm_m,
                                               float *sm_l, int hk, int split, int nsplit, int Gq, int pos, int k_begin,
                                               int k_end, int ntiles, LoadTile &&load_tile, int tid, uint32_t e_in,
                                               uint32_t e_part, uint32_t e_out) {
    constexpr int PITCH = D + 8;
    constexpr int TILE = kTileKeys * PITCH;
    constexpr int KSTEPS = D / 16;
    constexpr int NDT = D / 8;
    const int warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, t = lane & 3;
    const bool valid_lo = g < Gq, valid_hi = g + 8 < Gq;
    const int head_lo = hk * Gq + (valid_lo ? g : 0), head_hi = hk * Gq + (valid_hi ? g + 8 : 0);

    // Q fragments: one flagged word is one 32-bit fragment element (two adjacent f16).
    uint32_t qa[KSTEPS][4];
    {
        const uint2 *q_lo = P.q_w + (size_t)head_lo * (D / 2) + t, *q_hi = P.q_w + (size_t)head_hi * (D / 2) + t;
        uint2 raw[KSTEPS][4];
#pragma unroll
        for (int kk = 0; kk < KSTEPS; kk++) {  // all loads first, then the checks
            raw[kk][0] = valid_lo ? fw_load(q_lo + 8 * kk) : make_uint2(0u, e_in);
            raw[kk][1] = valid_hi ? fw_load(q_hi + 8 * kk) : make_uint2(0u, e_in);
            raw[kk][2] = valid_lo ? fw_load(q_lo + 8 * kk + 4) : make_uint2(0u, e_in);
            raw[kk][3] = valid_hi ? fw_load(q_hi + 8 * kk + 4) : make_uint2(0u, e_in);
        }
#pragma unroll
        for (int kk = 0; kk < KSTEPS; kk++)
#pragma unroll
            for (int i = 0; i < 4; i++) {
                if (raw[kk][i].y != e_in) {
                    const uint2 *p = ((i & 1) ? q_hi : q_lo) + 8 * kk + ((i >> 1) ? 4 : 0);
                    raw[kk][i] = fw_wait_slow(ctl, p, e_in, 20);
                }
                qa[kk][i] = raw[kk][i].x;
            }
    }
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
    float o[NDT][4];
#pragma unroll
    for (int i = 0; i < NDT; i++) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    const __half scale_h = __float2half_rn(P.attn_scale);
    // The tile and row of the newest key, if this split holds it.
    const bool has_new = pos >= k_begin && pos < k_end;
    const int new_tile = has_new ? (pos - k_begin) / kTileKeys : -1, new_row = has_new ? (pos - k_begin) % kTileKeys : 0;

    for (int tile = 0; tile < ntiles; tile++) {
        const int stage = tile & 1;
        if (tile + 1 < ntiles) {
            load_tile(tile + 1, stage ^ 1);
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        named_bar<128>(2);
        if (tile == new_tile) {
            // This step's K and V rows come straight from phase A's flagged words: the copy of
            // the cache row above may or may not have seen phase A's plain store.
            if (tid < D) {
                const int which = tid / (D / 2), w = tid % (D / 2);  // 0: K, 1: V
                const uint32_t v = fw_wait(ctl, P.kv_w + (size_t)which * (P.kvd / 2) + (size_t)hk * (D / 2) + w, e_in, 21);
                *reinterpret_cast<uint32_t *>((which ? vs : ks) + stage * TILE + new_row * PITCH + 2 * w) = v;
            }
            named_bar<128>(2);
        }
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
    float *so = reinterpret_cast<float *>(ks);  // [4][16][D], reuses the K/V tiles
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
    if (!row_valid) return;
    if (nsplit == 1) {
        const float inv = Lsum > 0.f ? 1.0f / Lsum : 0.f;
        uint2 *dst = P.attn_w + ((size_t)head * D + d0) / 2;
#pragma unroll
        for (int j = 0; j < DPT; j += 2) fw_store(dst + j / 2, pack_half2(acc[j] * inv, acc[j + 1] * inv), e_out);
        return;
    }
    // several splits: publish the partial; the head's merger CTA polls for it
    uint2 *dst = P.part_w + ((size_t)head * P.max_splits + split) * (D + 2);
    if ((tid & 7) == 0) {
        fw_store(dst, __float_as_uint(M), e_part);
        fw_store(dst + 1, __float_as_uint(Lsum), e_part);
    }
#pragma unroll
    for (int j = 0; j < DPT; j++) fw_store(dst + 2 + d0 + j, __float_as_uint(acc[j]), e_part);
}

// Merger of one query head: polls the head's nsplit partials and publishes its output.
// Threads 0 .. D-1 of the CTA, one output dimension each.
__device__ __forceinline__ void attention_merge(const StepParams &P, const Ctl &ctl, int head, int nsplit, int tid,
                                                uint32_t e_part, uint32_t e_out) {
    const int D = P.D;
    const uint2 *src = P.part_w + (size_t)head * P.max_splits * (D + 2);
    float Mg = -INFINITY, Lg = 0.f, acc = 0.f;
    for (int sp0 = 0; sp0 < nsplit; sp0 += 4) {
        uint2 m[4], l[4], o[4];
#pragma unroll
        for (int u = 0; u < 4; u++)  // all loads first, then the checks
            if (sp0 + u < nsplit) {
                const uint2 *p = src + (size_t)(sp0 + u) * (D + 2);
                m[u] = fw_load(p);
                l[u] = fw_load(p + 1);
                o[u] = fw_load(p + 2 + tid);
            }
#pragma unroll
        for (int u = 0; u < 4; u++)
            if (sp0 + u < nsplit) {
                const uint2 *p = src + (size_t)(sp0 + u) * (D + 2);
                if (m[u].y != e_part) m[u] = fw_wait_slow(ctl, p, e_part, 22);
                if (l[u].y != e_part) l[u] = fw_wait_slow(ctl, p + 1, e_part, 22);
                if (o[u].y != e_part) o[u] = fw_wait_slow(ctl, p + 2 + tid, e_part, 22);
                const float ms = __uint_as_float(m[u].x);
                const float Mn = fmaxf(Mg, ms);
                const float keep = Mg == -INFINITY ? 0.f : expf(Mg - Mn), wgt = ms == -INFINITY ? 0.f : expf(ms - Mn);
                Lg = Lg * keep + __uint_as_float(l[u].x) * wgt;
                acc = acc * keep + __uint_as_float(o[u].x) * wgt;
                Mg = Mn;
            }
    }
    const float out = Lg > 0.f ? acc / Lg : 0.f;
    const float nxt = __shfl_down_sync(0xffffffffu, out, 1);
    if ((tid & 1) == 0) fw_store(P.attn_w + ((size_t)head * D + tid) / 2, pack_half2(out, nxt), e_out);
}

// CW consumer warps + the producer warp.  Eight is the default; sixteen (96 registers per
// thread, spills in the attention) measured slower.
template <int QT, int HD, int CW>
__global__ void __launch_bounds__((CW + 1) * 32, 1) decode_step_kernel(const StepParams P) {
    constexpr int CT = CW * 32;
    constexpr int kThreads = CT + 32;
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
    ctl.wait_cycles = (long long)(P.wait_ns * 2ull);
    ctl.backoff = (unsigned)P.poll_backoff_ns;
    volatile int *sm_tok = reinterpret_cast<volatile int *>(smem + 264);
    float *sq_part = reinterpret_cast<float *>(smem + 512);
    float *red = reinterpret_cast<float *>(smem + kOffRed);
    float *cand_v = reinterpret_cast<float *>(smem + kOffSmall);
    int *cand_i = reinterpret_cast<int *>(smem + kOffSmall + 64);
    float *sm_m = reinterpret_cast<float *>(smem + kOffSmall + 128);  // [4][16]
    float *sm_l = sm_m + 64;                                          // [4][16]
    __half *xres = reinterpret_cast<__half *>(smem + P.off_xres);
    float2 *rope_cs = reinterpret_cast<float2 *>(smem + kOffRope);
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
    bool ok = true;
    const uint32_t stride = (uint32_t)P.n_layers * 8u + 8u;  // epochs per step

    // Input vector of a phase -- K f16 values, as flagged words of epoch `e` (or plain f16 from
    // an immutable table when e == 0) -- optionally RMS-normalised, into fragment order +
    // accumulator start values.  `keep`: also keep the raw values as the residual.
    // Item (block b, quad lane tt) owns the eight values of one B fragment: a thread polls
    // exactly the two 16-byte pieces its items need and keeps them in registers across the
    // one barrier the sum of squares costs; the norm weights are fetched before the wait.
    //   Q4_0 fragment order: {4t, 4t+2, 16+4t, 18+4t | 4t+1, 4t+3, 17+4t, 19+4t}
    //   Q8_0 fragment order: {8t .. 8t+7}
    constexpr int kRounds = 2;  // items a thread holds at once; a normalised input is at most kRounds * CT items (host-checked)
    auto load_input = [&](const void *src, uint32_t e, int k, int nblk, int nblk_pad, const __half *norm_w, bool keep,
                          int where) {
        const int items = nblk_pad * 4;
#pragma unroll 1
      for (int base = 0; base < items; base += kRounds * CT) {  // one trip for a normalised input
        uint32_t raw[kRounds][4], nwr[kRounds][4];
        // halves of the two pieces of item (b, tt)
        auto piece0 = [](int b, int tt) { return QT == TLC_TYPE_Q4_0 ? b * 32 + 4 * tt : b * 32 + 8 * tt; };
        auto piece1 = [](int b, int tt) { return QT == TLC_TYPE_Q4_0 ? b * 32 + 16 + 4 * tt : b * 32 + 8 * tt + 4; };
#pragma unroll
        for (int r = 0; r < kRounds; r++) {
            const int idx = base + ctid + r * CT, tt = idx & 3, b = idx >> 2;
            nwr[r][0] = nwr[r][1] = nwr[r][2] = nwr[r][3] = 0u;
            if (norm_w && idx < items && b < nblk) {
                const uint2 w0 = *reinterpret_cast<const uint2 *>(norm_w + piece0(b, tt));
                const uint2 w1 = *reinterpret_cast<const uint2 *>(norm_w + piece1(b, tt));
                nwr[r][0] = w0.x; nwr[r][1] = w0.y; nwr[r][2] = w1.x; nwr[r][3] = w1.y;
            }
        }
        if (e != 0) {
            const uint2 *w = static_cast<const uint2 *>(src);  // word i holds halves 2i, 2i + 1
            uint4 v[kRounds][2];
#pragma unroll
            for (int r = 0; r < kRounds; r++) {  // all loads first, then the checks
                const int idx = base + ctid + r * CT, tt = idx & 3, b = idx >> 2;
                if (idx < items && b < nblk) {
                    v[r][0] = fw_load2(w + piece0(b, tt) / 2);
                    v[r][1] = fw_load2(w + piece1(b, tt) / 2);
                }
            }
#pragma unroll
            for (int r = 0; r < kRounds; r++) {
                const int idx = base + ctid + r * CT, tt = idx & 3, b = idx >> 2;
                raw[r][0] = raw[r][1] = raw[r][2] = raw[r][3] = 0u;
                if (idx < items && b < nblk) {
                    if (v[r][0].y != e || v[r][0].w != e) v[r][0] = fw_wait2_slow(ctl, w + piece0(b, tt) / 2, e, where);
                    if (v[r][1].y != e || v[r][1].w != e) v[r][1] = fw_wait2_slow(ctl, w + piece1(b, tt) / 2, e, where);
                    raw[r][0] = v[r][0].x; raw[r][1] = v[r][0].z; raw[r][2] = v[r][1].x; raw[r][3] = v[r][1].z;
                }
            }
        } else {
            const __half *h = static_cast<const __half *>(src);
#pragma unroll
            for (int r = 0; r < kRounds; r++) {
                const int idx = base + ctid + r * CT, tt = idx & 3, b = idx >> 2;
                raw[r][0] = raw[r][1] = raw[r][2] = raw[r][3] = 0u;
                if (idx < items && b < nblk) {
                    const uint2 a = *reinterpret_cast<const uint2 *>(h + piece0(b, tt));
                    const uint2 c = *reinterpret_cast<const uint2 *>(h + piece1(b, tt));
                    raw[r][0] = a.x; raw[r][1] = a.y; raw[r][2] = c.x; raw[r][3] = c.y;
                }
            }
        }
        float sq = 0.f;
#pragma unroll
        for (int r = 0; r < kRounds; r++) {
            const int idx = base + ctid + r * CT, tt = idx & 3, b = idx >> 2;
            if (idx < items && b < nblk) {
                if (keep) {
                    *reinterpret_cast<uint2 *>(xres + piece0(b, tt)) = make_uint2(raw[r][0], raw[r][1]);
                    *reinterpret_cast<uint2 *>(xres + piece1(b, tt)) = make_uint2(raw[r][2], raw[r][3]);
                }
                if (norm_w) {
#pragma unroll
                    for (int j = 0; j < 4; j++) {
                        const float2 f = __half22float2(*reinterpret_cast<const __half2 *>(&raw[r][j]));
                        sq = fmaf(f.x, f.x, sq);
                        sq = fmaf(f.y, f.y, sq);
                    }
                }
            }
        }
        float inv = 1.f;
        if (norm_w) {
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
            if (lane == 0) sq_part[warp] = sq;
            consumer_bar<CT>();
            float ss = 0.f;
#pragma unroll
            for (int w = 0; w < CW; w++) ss += sq_part[w];
            inv = 1.0f / sqrtf(ss / (float)k + P.eps);
        }
#pragma unroll
        for (int r = 0; r < kRounds; r++) {
            const int idx = base + ctid + r * CT;
            const bool live = idx < items;
            const int b = idx >> 2;
            float f[8], v[8];
#pragma unroll
            for (int j = 0; j < 4; j++) {
                const float2 x2 = __half22float2(*reinterpret_cast<const __half2 *>(&raw[r][j]));
                f[2 * j] = x2.x;
                f[2 * j + 1] = x2.y;
                if (norm_w) {
                    // f16((x * inv) * w): two separately rounded f32 multiplies, then RNE
                    // (Tensor::rms_norm_cpu, src/ops/normalization.rs:236-240).
                    const float2 w2 = __half22float2(*reinterpret_cast<const __half2 *>(&nwr[r][j]));
                    f[2 * j] = __half2float(__float2half_rn(__fmul_rn(__fmul_rn(x2.x, inv), w2.x)));
                    f[2 * j + 1] = __half2float(__float2half_rn(__fmul_rn(__fmul_rn(x2.y, inv), w2.y)));
                }
            }
            if (QT == TLC_TYPE_Q4_0) {
                v[0] = f[0]; v[1] = f[2]; v[2] = f[4]; v[3] = f[6];
                v[4] = f[1]; v[5] = f[3]; v[6] = f[5]; v[7] = f[7];
            } else {
#pragma unroll
                for (int j = 0; j < 8; j++) v[j] = f[j];
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
                if ((idx & 3) == 0) {
                    const float cv = -T::OFFSET * 5.9604644775390625e-08f * s;  // * 2^-24
                    cinit[b] = make_float4(cv, cv, cv, cv);
                }
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
    // reduction per batch, then the epilogue on pairs of adjacent rows:
    // epi(unit, pr, a0, a1, b0, b1): a0, a1 = dot products (already * 2^24) of rows 2pr and
    // 2pr + 1 of the unit's slab, b0, b1 the same for the second slab of a gate/up pair.
    uint64_t *tslot = nullptr;  // tracing: the three stamps of the current phase (CTA 0, thread 0)
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
            if (tslot) tslot[1] = tlc_globaltimer_ns();  // dot products done
            for (int item = ctid; item < nu * 8; item += CT) {
                const int ui = item >> 3, pr = item & 7;
                auto total2 = [&](int set, float &v0, float &v1) {
                    float s0 = 0.f, s1 = 0.f;
#pragma unroll
                    for (int w = 0; w < CW; w++) {
                        const float2 p = *reinterpret_cast<const float2 *>(&rbuf[(w * kBatchSlabs + set) * 16 + 2 * pr]);
                        s0 += p.x;
                        s1 += p.y;
                    }
                    v0 = s0 * 16777216.0f;  // undo the 2^-24 of the integer fragments
                    v1 = s1 * 16777216.0f;
                };
                float a0, a1, b0 = 0.f, b1 = 0.f;
                total2(ui * f.subs, a0, a1);
                if (f.subs == 2) total2(ui * f.subs + 1, b0, b1);
                epi(u0 + ui, pr, a0, a1, b0, b1);
            }
        }
        return true;
    };

    // The first token and its position come from memory; later steps of the same launch get
    // the token as a flagged word and count the position themselves.
    if (ctid == 0) {
        const int *ids = P.ids_src ? P.ids_src : P.ids;
        int tk = ldcg_i32(ids);
        *sm_tok = tk < 0 ? 0 : (tk >= P.vocab ? P.vocab - 1 : tk);  // validated on the host; never read outside
    }
    int pos = ldcg_i32(P.positions);
    consumer_bar<CT>();

    for (int step = 0; step < P.steps && ok; step++, pos++) {
        const uint32_t e_step = P.epoch_base + (uint32_t)step * stride;
        const int tok = *sm_tok;
        const bool pos_ok = pos >= 0 && pos < P.Tmax;
        if (!pos_ok && ctid == 0 && atomicCAS(&P.status->code, 0, TLC_DEV_INDEX) == 0) P.status->where = 310;
        const int T_keys = pos_ok ? pos + 1 : 1;
        // Rotary angles of this position, one (cos, sin) per pair of the head: computed while
        // the first input is still on its way (they become visible with phase A's barriers).
        if (ctid < HD / 2) {
            const float freq = 1.0f / powf(P.rope_base, (float)(2 * ctid) / (float)HD);
            const float theta = (float)(unsigned)pos * freq;
            rope_cs[ctid] = make_float2(cosf(theta), sinf(theta));
        }
        uint64_t *trace = P.trace && cta == 0 && ctid == 0 ? P.trace + (size_t)step * (P.n_layers * 5 + 2) * 3 : nullptr;

        for (int l = 0; l < P.n_layers && ok; l++) {
            const StepLayer *L = P.layers + l;
            const uint32_t e_l = e_step + (uint32_t)l * 8u;
            // ---- A: rms_norm + q/k/v + rope + cache append ----
            {
                const Phase f = make_phase(P, L, 0);
                if (l == 0)
                    load_input(P.embd + (size_t)tok * P.embd_pitch, 0u, f.k, f.nblk, f.ktiles * P.tb, L->attn_norm, true, 30);
                else
                    load_input(P.x_w, e_l - 8u + kSlotX, f.k, f.nblk, f.ktiles * P.tb, L->attn_norm, true, 30);
                const int hd = P.D;
                if ((tslot = trace ? trace + (l * 5 + 0) * 3 : nullptr)) tslot[0] = tlc_globaltimer_ns();
                ok = gemv_phase(f, [&](int u, int pr, float a0, float a1, float, float) {
                    int ti, sl;
                    unit_slab(f, u, 0, ti, sl);
                    const int n = sl * kRows + 2 * pr;  // even: the pair (n, n + 1) is a rotary pair
                    if (n >= f.n[ti]) return;
                    __half h0 = __float2half_rn(a0), h1 = __float2half_rn(a1);
                    if (ti < 2) {
                        // Interleaved RoPE on the f16-rounded projection (rope_f16,
                        // shaders/unified.metal:2355-2417), at the token's true position.
                        const float2 rot = rope_cs[(n % hd) >> 1];
                        const float x0 = __half2float(h0), x1 = __half2float(h1);
                        const float cs = rot.x, sn = rot.y;
                        h0 = __float2half_rn(__fsub_rn(__fmul_rn(x0, cs), __fmul_rn(x1, sn)));
                        h1 = __float2half_rn(__fadd_rn(__fmul_rn(x0, sn), __fmul_rn(x1, cs)));
                    }
                    const uint32_t bits = half2_bits(h0, h1);
                    if (ti == 0) {
                        fw_store(P.q_w + n / 2, bits, e_l + kSlotQKV);
                    } else {
                        // the cache row for later steps, the flagged copy for this step's attention
                        if (pos_ok) *reinterpret_cast<uint32_t *>((ti == 1 ? L->kc : L->vc) + (size_t)pos * P.kvd + n) = bits;
                        fw_store(P.kv_w + (size_t)(ti - 1) * (P.kvd / 2) + n / 2, bits, e_l + kSlotQKV);
                    }
                });
                if (!ok) break;
                if (trace) trace[(l * 5 + 0) * 3 + 2] = tlc_globaltimer_ns();
            }
            // ---- B: attention ----
            // (KV head, key split) items on the first CTAs (warps 0-3 do the work); with several
            // splits, one merger CTA per query head at the end of the grid.
            {
                const int tiles_total = (T_keys + kTileKeys - 1) / kTileKeys;
                int nsplit = tiles_total < P.max_splits ? tiles_total : P.max_splits;
                nsplit = nsplit < 1 ? 1 : nsplit;
                const int keys_per_split = ((tiles_total + nsplit - 1) / nsplit) * kTileKeys;
                const bool has_item = cta < P.Hkv * nsplit;
                const int hk = cta / nsplit, split = cta % nsplit;
                const int k_begin = split * keys_per_split;
                const int k_end = min(T_keys, k_begin + keys_per_split);
                const int ntiles = has_item && k_end > k_begin ? (k_end - k_begin + kTileKeys - 1) / kTileKeys : 0;
                constexpr int D = HD;
                constexpr int PITCH = D + 8, TILEH = kTileKeys * PITCH;
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
                if (has_item && warp < 4) {
                    const int Gq = P.H / P.Hkv;  // query heads per KV head (rows of the tile that are real)
                    if (ntiles > 0) load_kv_tile(0, 0);
                    attention_item<HD>(P, ctl, ks, vs, sm_m, sm_l, hk, split, nsplit, Gq, pos, k_begin, k_end, ntiles,
                                       load_kv_tile, ctid, e_l + kSlotQKV, e_l + kSlotPart, e_l + kSlotAttn);
                }
                if (nsplit > 1 && cta >= G - P.H && ctid < D)
                    attention_merge(P, ctl, cta - (G - P.H), nsplit, ctid, e_l + kSlotPart, e_l + kSlotAttn);
                if (trace) trace[(l * 5 + 1) * 3 + 2] = tlc_globaltimer_ns();
            }
            // ---- C: o projection + residual ----
            {
                const Phase f = make_phase(P, L, 2);
                load_input(P.attn_w, e_l + kSlotAttn, f.k, f.nblk, f.ktiles * P.tb, nullptr, false, 32);
                if ((tslot = trace ? trace + (l * 5 + 2) * 3 : nullptr)) tslot[0] = tlc_globaltimer_ns();
                ok = gemv_phase(f, [&](int u, int pr, float a0, float a1, float, float) {
                    const int n = u * kRows + 2 * pr;
                    if (n >= f.n[0]) return;
                    const __half2 r = *reinterpret_cast<const __half2 *>(xres + n);
                    fw_store(P.x1_w + n / 2, half2_bits(__hadd(__float2half_rn(a0), __low2half(r)),
                                                        __hadd(__float2half_rn(a1), __high2half(r))), e_l + kSlotX1);
                });
                if (!ok) break;
                if (trace) trace[(l * 5 + 2) * 3 + 2] = tlc_globaltimer_ns();
            }
            // ---- D: rms_norm + gate/up + silu*mul ----
            {
                const Phase f = make_phase(P, L, 3);
                load_input(P.x1_w, e_l + kSlotX1, f.k, f.nblk, f.ktiles * P.tb, L->ffn_norm, true, 33);
                if ((tslot = trace ? trace + (l * 5 + 3) * 3 : nullptr)) tslot[0] = tlc_globaltimer_ns();
                ok = gemv_phase(f, [&](int u, int pr, float a0, float a1, float b0, float b1) {
                    const int n = u * kRows + 2 * pr;
                    if (n >= f.n[0]) return;
                    // h = gate; s = sigmoid(g) (f32, RNE); a = g*s; act = a*u: three f16
                    // roundings as in debug/chat_demo_with_kvcache.tl:26-41.
                    auto swiglu = [](float gv, float uv) {
                        const __half gate = __float2half_rn(gv), up = __float2half_rn(uv);
                        const __half sg = __float2half_rn(1.0f / (1.0f + expf(-__half2float(gate))));
                        return __hmul(__hmul(gate, sg), up);
                    };
                    fw_store(P.act_w + n / 2, half2_bits(swiglu(a0, b0), swiglu(a1, b1)), e_l + kSlotAct);
                });
                if (!ok) break;
                if (trace) trace[(l * 5 + 3) * 3 + 2] = tlc_globaltimer_ns();
            }
            // ---- E: down projection + residual ----
            {
                const Phase f = make_phase(P, L, 4);
                load_input(P.act_w, e_l + kSlotAct, f.k, f.nblk, f.ktiles * P.tb, nullptr, false, 34);
                if ((tslot = trace ? trace + (l * 5 + 4) * 3 : nullptr)) tslot[0] = tlc_globaltimer_ns();
                ok = gemv_phase(f, [&](int u, int pr, float a0, float a1, float, float) {
                    const int n = u * kRows + 2 * pr;
                    if (n >= f.n[0]) return;
                    const __half2 r = *reinterpret_cast<const __half2 *>(xres + n);
                    fw_store(P.x_w + n / 2, half2_bits(__hadd(__float2half_rn(a0), __low2half(r)),
                                                       __hadd(__float2half_rn(a1), __high2half(r))), e_l + kSlotX);
                });
                if (!ok) break;
                if (trace) trace[(l * 5 + 4) * 3 + 2] = tlc_globaltimer_ns();
            }
        }
        if (!ok) break;
        // ---- F: rms_norm + lm_head, local argmax ----
        const uint32_t e_fin = e_step + (uint32_t)P.n_layers * 8u;
        {
            const Phase f = make_phase(P, P.layers, 5);
            load_input(P.x_w, e_fin - 8u + kSlotX, f.k, f.nblk, f.ktiles * P.tb, P.out_norm, false, 35);
            if ((tslot = trace ? trace + (P.n_layers * 5 + 0) * 3 : nullptr)) tslot[0] = tlc_globaltimer_ns();
            float best = -INFINITY;
            int bi = -1;
            ok = gemv_phase(f, [&](int u, int pr, float a0, float a1, float, float) {
                const int n = u * kRows + 2 * pr;
                if (n >= f.n[0]) return;
                const __half h0 = __float2half_rn(a0), h1 = __float2half_rn(a1);
                const float v0 = __half2float(h0), v1 = __half2float(h1);
                // a thread meets its rows in increasing order: the later index wins ties
                if (bi < 0 || !(v0 < best)) { best = v0; bi = n; }
                if (n + 1 < f.n[0]) {
                    *reinterpret_cast<__half2 *>(P.logits + n) = __halves2half2(h0, h1);
                    if (!(v1 < best)) { best = v1; bi = n + 1; }
                } else {
                    P.logits[n] = h0;
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
            // This CTA's plain stores of the step (cache rows, logits) are made visible before
            // its candidate word: whoever sees the next token may read them.
            __threadfence();
            consumer_bar<CT>();
            if (ctid == 0) {
                for (int w = 1; w < CW; w++)
                    if (better(cand_v[w], cand_i[w], best, bi)) { best = cand_v[w]; bi = cand_i[w]; }
                fw_store2(P.cand_w + cta, __float_as_uint(best), (uint32_t)bi, e_fin + kSlotCand);
            }
            if (trace) trace[(P.n_layers * 5 + 0) * 3 + 2] = tlc_globaltimer_ns();
            // ---- G: the token, the bookkeeping, the report to the host ----
            if (cta == 0) {
                best = -INFINITY;
                bi = -1;
                for (int i = ctid; i < G; i += CT) {
                    uint4 v = fw_load2(P.cand_w + i);
                    if (v.y != e_fin + kSlotCand || v.w != e_fin + kSlotCand)
                        v = fw_wait2_slow(ctl, P.cand_w + i, e_fin + kSlotCand, 36);
                    const float cv = __uint_as_float(v.x);
                    const int idx = (int)v.z;
                    if (better(cv, idx, best, bi)) { best = cv; bi = idx; }
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
                if (*ctl.abort_flag) {
                    ok = false;
                    break;
                }
                if (ctid == 0) {
                    for (int w = 1; w < CW; w++)
                        if (better(cand_v[w], cand_i[w], best, bi)) { best = cand_v[w]; bi = cand_i[w]; }
                    if (bi < 0) bi = 0;
                    __threadfence();  // every CTA's stores of this step, seen through its candidate word
                    P.next_ids[0] = bi;
                    P.ids[0] = bi;
                    P.positions[0] = pos + 1;
                    if (step + 1 < P.steps) fw_store(P.tok_w, (uint32_t)bi, e_fin + kSlotTok);
                    if (trace) trace[(P.n_layers * 5 + 1) * 3 + 2] = tlc_globaltimer_ns();
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
            if (step + 1 < P.steps) {
                if (ctid == 0) {
                    const int tk = (int)fw_wait(ctl, P.tok_w, e_fin + kSlotTok, 37);
                    __threadfence();
                    *sm_tok = tk < 0 ? 0 : (tk >= P.vocab ? P.vocab - 1 : tk);
                }
                consumer_bar<CT>();
                if (*ctl.abort_flag) ok = false;
            }
        }
    }

    if (!ok) *ctl.abort_flag = 1;  // the producer stops at its next wait
    named_bar<kThreads>(3);
    if (!ok && ctid == 0) {
        // Copies the producer started and nobody consumed must land before this CTA's shared
        // memory goes away.
        const int issued = *ctl.issued;
        for (int i = consumed; i < issued; i++) {
            const int s = i % S;
            const uint32_t par = (uint32_t)((i / S) & 1);
            const long long t0 = clock64();
            while (!mbar_try_wait(&ctl.full[s], par) && clock64() - t0 < 2000000ll) {
            }
        }
    }
}

}  // namespace tlc_step

// ---- host side ----------------------------------------------------------------------------

namespace tlc_step {

int step_max_splits(int grid, int n_heads, int n_kv_heads) {
    // split workers and one merger per head must be different CTAs
    int s = grid > n_heads ? (grid - n_heads) / n_kv_heads : 1;
    s = s < 1 ? 1 : s > 64 ? 64 : s;
    return s;
}

StepWorkspace step_workspace(int d, int qd, int kvd, int ffn, int n_heads, int head_dim, int max_splits, int grid) {
    StepWorkspace w{};
    size_t off = 0;
    auto take = [&](size_t bytes) {
        const size_t at = off;
        off = align_up(off + bytes, 256);
        return at;
    };
    w.x = take((size_t)d / 2 * 8);
    w.x1 = take((size_t)d / 2 * 8);
    w.q = take((size_t)qd / 2 * 8);
    w.kv = take((size_t)kvd * 8);
    w.attn = take((size_t)qd / 2 * 8);
    w.act = take((size_t)ffn / 2 * 8);
    w.part = take((size_t)n_heads * max_splits * (head_dim + 2) * 8);
    w.cand = take((size_t)grid * 16);
    w.tok = take(16);
    w.total = off;
    return w;
}

// The variant for a weight type and head width, as (kernel, threads per CTA).
typedef void (*StepKernel)(const StepParams);
static int wide_variant() {  // TLC_STEP_CW=16: sixteen consumer warps for head_dim 64 (measured: 0.91 ms vs 0.79 ms per TinyLlama step)
    static int v = -1;
    if (v < 0) {
        const char *e = getenv("TLC_STEP_CW");
        v = e && atoi(e) == 16 ? 1 : 0;
    }
    return v;
}
static StepKernel pick_kernel(int qtype, int head_dim, int *threads) {
    if (head_dim == 64 && !wide_variant()) {
        *threads = 9 * 32;
        return qtype == TLC_TYPE_Q4_0 ? decode_step_kernel<TLC_TYPE_Q4_0, 64, 8> : decode_step_kernel<TLC_TYPE_Q8_0, 64, 8>;
    }
    if (head_dim == 64) {
        *threads = 17 * 32;
        return qtype == TLC_TYPE_Q4_0 ? decode_step_kernel<TLC_TYPE_Q4_0, 64, 16> : decode_step_kernel<TLC_TYPE_Q8_0, 64, 16>;
    }
    *threads = 9 * 32;
    return qtype == TLC_TYPE_Q4_0 ? decode_step_kernel<TLC_TYPE_Q4_0, 128, 8> : decode_step_kernel<TLC_TYPE_Q8_0, 128, 8>;
}

static int32_t configure(tlc_ctx *ctx, int qtype, int head_dim, int *blocks_per_sm, size_t smem) {
    static bool configured[64][2][2] = {};
    int threads = 0;
    StepKernel k = pick_kernel(qtype, head_dim, &threads);
    bool &done = configured[ctx->device & 63][qtype == TLC_TYPE_Q4_0 ? 0 : 1][head_dim == 64 ? 0 : 1];
    if (!done) {
        TLC_CUDA(cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)ctx->prop.sharedMemPerBlockOptin));
        TLC_CUDA(cudaFuncSetAttribute(k, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared));
        done = true;
    }
    TLC_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(blocks_per_sm, k, threads, smem));
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
    // a normalised input (d values) must fit the registers of one pass: 2 items of 8 values per thread
    if (d / 8 > 2 * (head_dim == 64 && wide_variant() ? 16 : 8) * 32) return false;
    int coop = 0;
    if (cudaDeviceGetAttribute(&coop, cudaDevAttrCooperativeLaunch, ctx->device) != cudaSuccess || !coop) return false;
    const SmemPlan s = plan_for(ctx, qtype, d, kmax, head_dim);
    if (s.stages < 3) return false;
    int per_sm = 0;
    const int32_t rc = configure(ctx, qtype, head_dim, &per_sm, s.total);
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
    {
        static int backoff = -1;
        if (backoff < 0) {
            const char *e = getenv("TLC_STEP_BACKOFF_NS");
            backoff = e ? atoi(e) : 0;
        }
        p.poll_backoff_ns = backoff;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)grid);
    int threads = 0;
    StepKernel kernel = pick_kernel(qtype, p.D, &threads);
    cfg.blockDim = dim3((unsigned)threads);
    cfg.dynamicSmemBytes = s.total;
    cfg.stream = ctx->stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeCooperative;  // all CTAs resident at once: they wait on one another
    attr[0].val.cooperative = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    const cudaError_t le = cudaLaunchKernelEx(&cfg, kernel, p);
    if (le != cudaSuccess) {
        cudaGetLastError();
        return tlc_fail(TLC_ERR_CUDA, "decode step launch failed: %s", cudaGetErrorString(le));
    }
    TLC_CHECK_LAUNCH(ctx);
    return TLC_OK;
}

}  // namespace tlc_step
