// Pre-allocated f16 KV cache and fused grouped-query attention over it.
//
// Takes the place of the builtin chain the TL scripts run per layer
// (debug/chat_demo_with_kvcache.tl:44-88 prefill, :247-282 decode):
//   cache.append (a concat of the whole cache, src/model/llama.rs:85-99)
//   reshape -> broadcast_to -> reshape            (GQA expansion, 8x copies)
//   einsum("ihd,jhd->ihj") -> * 0.125 -> causal_mask -> apply_attention_mask
//   softmax -> einsum("ihj,jhd->ihd")
// (kernels einsum_ihd_jhd_ihj_f16, apply_attention_mask_f16, softmax_f16,
// einsum_ihj_jhd_ihd_f16 of shaders/unified.metal:2524-2683, :4474-4488,
// :2057-2200) by one kernel that never materialises the [I, H, J] scores.
//
// One CTA owns a tile of 16 (query, head) rows that share a KV head -- the G
// query heads of the group times 16/G query positions -- and a range of keys.
// K/V tiles of 64 keys are staged in shared memory with 16-byte cp.async
// (zero-filled past the end), each of the 4 warps takes 16 keys of a tile:
// S = Q.K^T with m16n8k16 (f32 accumulate), the two f16 roundings the reference
// applies to the scores (einsum output, then the f16 multiply by the scale),
// online softmax in f32, P rounded to f16 as the reference stores it, and
// O += P.V with f32 accumulation.  The 4 warps' partial (max, sum, O) are merged
// through shared memory.  For decode the key range of a sequence is split over
// several CTAs; each writes its partial to global scratch and the last one to
// finish (atomic ticket) merges them, so no second launch is needed.
#include <cooperative_groups.h>
#include <cuda_fp16.h>

#include <mutex>

#include "tlc_internal.h"

struct tlc_kvcache {
    tlc_ctx *ctx;
    int n_layers, max_batch, max_seq, n_kv_heads, head_dim;
    __half *k;  // [layer][batch][max_seq][n_kv_heads][head_dim]
    __half *v;
    size_t layer_stride;  // elements
};

namespace {

constexpr int kTileKeys = 64;
constexpr int kAttnThreads = 128;

struct AttnParams {
    const __half *q;   // [B*I, H, D]
    const __half *kc;  // this layer's K cache [B][Tmax][Hkv][D]
    const __half *vc;
    __half *out;       // [B*I, H, D]
    int I, H, Hkv, G, Tmax;
    int q_pos0;            // position of query 0 (prefill); ignored when positions != null
    const int *positions;  // device int32[B]: position of each sequence's single query (decode)
    float scale;
    int nsplit;
    int keys_per_split;  // multiple of kTileKeys
    int q_tiles;
    float *part_ml;  // [rows][nsplit][2]
    float *part_o;   // [rows][nsplit][D]
    int *counters;   // [B][q_tiles][Hkv], zero between launches
    int push_offset; // cluster mode: byte offset of the merge area in dynamic shared memory
    int push_splits; // cluster mode: splits the merge area of rank 0 is laid out for (8 or 16)
    int cluster;     // 1: the nsplit CTAs of a tile form a thread-block cluster and merge through
                     // distributed shared memory instead of global scratch
    int pos_settled; // 1: the launcher vouches that positions[] was final before this kernel could start
                     // (see tlc_launch_attention); the kernel then reads it once, before the wait
    int key_limit;   // keys the launch was sized for (<= Tmax): a sequence whose position says it
                     // holds more is cut there and the status word (when given) says so
    tlc_dev_status *status;  // device word or null
};

__device__ __forceinline__ void cp_async16(void *smem_dst, const void *gsrc, bool valid) {
    const uint32_t d = (uint32_t)__cvta_generic_to_shared(smem_dst);
    const int sz = valid ? 16 : 0;  // src-size 0: the 16 bytes are zero-filled
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
__device__ __forceinline__ void mma16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
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

template <int D>
__global__ void __launch_bounds__(kAttnThreads) attention_kernel(const AttnParams p) {
    constexpr int PITCH = D + 8;             // halves; +16 B keeps ldmatrix rows on distinct banks
    constexpr int TILE = kTileKeys * PITCH;  // halves per K (or V) tile
    constexpr int KSTEPS = D / 16;
    constexpr int NDT = D / 8;               // n8 tiles of the output
    extern __shared__ __align__(128) uint8_t smem_raw[];
    __half *ks = reinterpret_cast<__half *>(smem_raw);  // [2][TILE]
    __half *vs = ks + 2 * TILE;                         // [2][TILE]
    __shared__ float sm_m[4][16], sm_l[4][16];
    __shared__ int sm_last;

    // Cluster mode: tell the peers this CTA is running (its shared memory may be written from
    // now on); the matching wait comes just before the first remote store.
    if (p.cluster) asm volatile("barrier.cluster.arrive.relaxed.aligned;" ::: "memory");
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, t = lane & 3;
    const int b = blockIdx.z, hk = blockIdx.y;
    const int qt = blockIdx.x / p.nsplit, split = blockIdx.x % p.nsplit;
    // the group size is a power of two (1 .. 16, checked by the launcher): shifts, not divisions
    const int G = p.G, gsh = 31 - __clz(p.G), RQ = 16 >> gsh;

    // A decode step's query, its newest cache row AND its position come from earlier kernels
    // of the stream.  Before griddepcontrol.wait the position word may still hold the previous
    // step's value; positions only grow while kernels are in flight (the host resets them
    // after a stream synchronize), so that value is a lower bound of the true one.  It is used
    // for one thing only: a first K/V tile that lies entirely below it holds rows of earlier
    // steps, whatever the true position turns out to be, and is fetched while the previous
    // kernel is still running.  k_begin does not depend on the position at all.
    const int k_begin = split * p.keys_per_split;
    const __half *kbase = p.kc + ((size_t)b * p.Tmax * p.Hkv + hk) * D;
    const __half *vbase = p.vc + ((size_t)b * p.Tmax * p.Hkv + hk) * D;
    const size_t key_stride = (size_t)p.Hkv * D;
    int k_end = 0;  // set below; the early tile is whole, so every key of it passes `< k_end`
    auto load_tile = [&](int tile, int stage) {
        const int j0 = k_begin + tile * kTileKeys;
        constexpr int CHUNKS = kTileKeys * (D / 8);
#pragma unroll
        for (int c = tid; c < CHUNKS; c += kAttnThreads) {
            const int key = c / (D / 8), part = c % (D / 8);
            const bool ok = j0 + key < k_end;
            const size_t off = (size_t)(ok ? j0 + key : 0) * key_stride + part * 8;
            cp_async16(ks + stage * TILE + key * PITCH + part * 8, kbase + off, ok);
            cp_async16(vs + stage * TILE + key * PITCH + part * 8, vbase + off, ok);
        }
        cp_async_commit();
    };
    // Rows of the tile: r -> (query qt*RQ + r/G, head hk*G + r%G).
    const int qi_lo = qt * RQ + (g >> gsh), qi_hi = qt * RQ + ((g + 8) >> gsh);
    const int head_lo = hk * G + (g & (G - 1)), head_hi = hk * G + ((g + 8) & (G - 1));
    const bool valid_lo = qi_lo < p.I, valid_hi = qi_hi < p.I;
    const int last_q = min(p.I, (qt + 1) * RQ) - 1;
    // Everything that depends on the position of query 0.
    int pos0 = 0, rpos_lo = 0, rpos_hi = 0, ntiles = 0;
    auto derive = [&](int pos_raw, bool final_value) {
        pos0 = pos_raw < 0 ? 0 : pos_raw;
        if (pos0 + p.I > p.key_limit) {  // more keys than the launch (or the cache) holds: cut, and say so
            pos0 = p.key_limit - p.I;
            if (final_value && p.status && tid == 0 && atomicCAS(&p.status->code, 0, TLC_DEV_INDEX) == 0)
                p.status->where = 200 + b;
        }
        const int T = pos0 + p.I;  // keys in the cache (incl. the new ones)
        rpos_lo = pos0 + qi_lo;    // last visible key of the row
        rpos_hi = pos0 + qi_hi;
        // Keys this CTA covers: its split, cut at the last key any row of the tile may see.
        const int visible_end = min(T, pos0 + last_q + 1);
        k_end = min(visible_end, k_begin + p.keys_per_split);
        ntiles = k_end > k_begin ? (k_end - k_begin + kTileKeys - 1) / kTileKeys : 0;
    };
    // A launch argument is final; a device word is final before the wait only if the launcher vouches
    // for it (tlc_launch_attention).  Then all of the above is worked out while the previous kernel
    // still runs; otherwise the word is a lower bound, good for the early tile only, and is read
    // again after the wait (an L2 round trip on the critical path of the layer).
    const bool settled = !p.positions || p.pos_settled;
    const int pos_seen = p.positions ? *reinterpret_cast<const volatile int *>(p.positions + b) : p.q_pos0;
    derive(pos_seen, settled);
    const bool early = p.I == 1 && ntiles > 0 && k_begin + kTileKeys <= pos0;
    if (early) {
        if (!settled) k_end = k_begin + kTileKeys;  // the tile is whole whatever the final position is
        load_tile(0, 0);
    }
    asm volatile("griddepcontrol.wait;" ::: "memory");
    // The next kernel of the stream (a GEMV: its producer warp streams weights, the rest waits) may be
    // scheduled from here on; letting it in before this wait was 0.2 % slower on the decode step.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    if (!settled) derive(*reinterpret_cast<const volatile int *>(p.positions + b), true);

    // Q fragments (A operand), straight from global memory.
    uint32_t qa[KSTEPS][4];
    {
        const __half *q_lo = p.q + ((size_t)(b * p.I + (valid_lo ? qi_lo : 0)) * p.H + head_lo) * D;
        const __half *q_hi = p.q + ((size_t)(b * p.I + (valid_hi ? qi_hi : 0)) * p.H + head_hi) * D;
#pragma unroll
        for (int kk = 0; kk < KSTEPS; kk++) {
            qa[kk][0] = valid_lo ? *reinterpret_cast<const uint32_t *>(q_lo + 16 * kk + 2 * t) : 0u;
            qa[kk][1] = valid_hi ? *reinterpret_cast<const uint32_t *>(q_hi + 16 * kk + 2 * t) : 0u;
            qa[kk][2] = valid_lo ? *reinterpret_cast<const uint32_t *>(q_lo + 16 * kk + 8 + 2 * t) : 0u;
            qa[kk][3] = valid_hi ? *reinterpret_cast<const uint32_t *>(q_hi + 16 * kk + 8 + 2 * t) : 0u;
        }
    }

    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
    float o[NDT][4];
#pragma unroll
    for (int i = 0; i < NDT; i++) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    const __half scale_h = __float2half_rn(p.scale);

    if (ntiles > 0 && !early) load_tile(0, 0);
    for (int tile = 0; tile < ntiles; tile++) {
        const int stage = tile & 1;
        if (tile + 1 < ntiles) {
            load_tile(tile + 1, stage ^ 1);
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();

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
                mma16816(s[0], qa[kk], r[0], r[1]);
                mma16816(s[1], qa[kk], r[2], r[3]);
            }
            // Scores: f16 rounding of the einsum output, f16 multiply by the scale
            // (scripts multiply the f16 score tensor by 0.125), then the causal mask.
            float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
            for (int nt = 0; nt < 2; nt++)
#pragma unroll
                for (int e = 0; e < 4; e++) {
                    const int key = j0 + kw0 + nt * 8 + 2 * t + (e & 1);
                    const int rpos = e < 2 ? rpos_lo : rpos_hi;
                    float v = __half2float(__hmul(__float2half_rn(s[nt][e]), scale_h));
                    if (key >= k_end || key > rpos) v = -INFINITY;
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
                corr[h] = expf(m_run[h] - msafe[h]);  // exp(-inf) = 0 on the first tile
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
                mma16816(o[2 * jd], pa, r[0], r[1]);
                mma16816(o[2 * jd + 1], pa, r[2], r[3]);
            }
        }
        __syncthreads();
    }

    // ---- merge the 4 warps (each saw a different quarter of every tile) ----
#pragma unroll
    for (int h = 0; h < 2; h++) {
        l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 1);
        l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 2);
    }
    float *so = reinterpret_cast<float *>(smem_raw);  // [4][16][D], reuses the K/V tiles
    if (t == 0) {
        sm_m[warp][g] = m_run[0];
        sm_m[warp][g + 8] = m_run[1];
        sm_l[warp][g] = l_run[0];
        sm_l[warp][g + 8] = l_run[1];
    }
#pragma unroll
    for (int i = 0; i < NDT; i++) {
        float *base = so + (size_t)warp * 16 * D;
        *reinterpret_cast<float2 *>(base + g * D + 8 * i + 2 * t) = make_float2(o[i][0], o[i][1]);
        *reinterpret_cast<float2 *>(base + (g + 8) * D + 8 * i + 2 * t) = make_float2(o[i][2], o[i][3]);
    }
    __syncthreads();

    // thread -> (row, D/8 consecutive dims)
    constexpr int DPT = D / 8;
    const int row = tid >> 3, d0 = (tid & 7) * DPT;
    const int qi = qt * RQ + (row >> gsh), head = hk * G + (row & (G - 1));
    const bool row_valid = qi < p.I;
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < 4; w++) M = fmaxf(M, sm_m[w][row]);
    float L = 0.f, acc[DPT];
#pragma unroll
    for (int j = 0; j < DPT; j++) acc[j] = 0.f;
#pragma unroll
    for (int w = 0; w < 4; w++) {
        const float wgt = sm_m[w][row] == -INFINITY ? 0.f : expf(sm_m[w][row] - M);
        L += sm_l[w][row] * wgt;
#pragma unroll
        for (int j = 0; j < DPT; j++) acc[j] += so[((size_t)w * 16 + row) * D + d0 + j] * wgt;
    }
    const size_t out_row = (size_t)(b * p.I + (row_valid ? qi : 0)) * p.H + head;

    if (p.nsplit == 1) {
        if (row_valid) {
            const float inv = L > 0.f ? 1.0f / L : 0.f;
#pragma unroll
            for (int j = 0; j < DPT; j++) p.out[out_row * D + d0 + j] = __float2half_rn(acc[j] * inv);
        }
        return;
    }

    if (p.cluster) {
        // ---- split keys inside a cluster: every CTA stores its partial (max, sum, O) into
        // rank 0's shared memory through distributed shared memory, one cluster barrier, and
        // rank 0 merges from its own memory; the peers are free to leave at once ----
        namespace cg = cooperative_groups;
        cg::cluster_group cl = cg::this_cluster();
        // [nsplit][16] max, [nsplit][16] sum, [nsplit][16][D] O, behind the K/V tiles
        float *push = reinterpret_cast<float *>(smem_raw + p.push_offset);
        float *r0 = cl.map_shared_rank(push, 0);
        const int PS = p.push_splits;
        float *pm = r0, *pl = r0 + PS * 16, *po = r0 + 2 * PS * 16;
        asm volatile("barrier.cluster.wait.aligned;" ::: "memory");  // every CTA of the cluster has started
        if ((tid & 7) == 0) {
            pm[split * 16 + row] = M;
            pl[split * 16 + row] = L;
        }
#pragma unroll
        for (int j = 0; j < DPT; j += 4)
            *reinterpret_cast<float4 *>(po + ((size_t)split * 16 + row) * D + d0 + j) =
                make_float4(acc[j], acc[j + 1], acc[j + 2], acc[j + 3]);
        asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
        asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
        if (cl.block_rank() == 0 && row_valid) {
            const float *lm = push, *ll = push + PS * 16, *lo = push + 2 * PS * 16;
            float Mg = -INFINITY;
#pragma unroll 4
            for (int sp = 0; sp < p.nsplit; sp++) Mg = fmaxf(Mg, lm[sp * 16 + row]);
            float Lg = 0.f;
#pragma unroll
            for (int j = 0; j < DPT; j++) acc[j] = 0.f;
#pragma unroll 4
            for (int sp = 0; sp < p.nsplit; sp++) {
                const float ms = lm[sp * 16 + row];
                const float wgt = ms == -INFINITY ? 0.f : expf(ms - Mg);
                Lg += ll[sp * 16 + row] * wgt;
                const float *ro = lo + ((size_t)sp * 16 + row) * D + d0;
#pragma unroll
                for (int j = 0; j < DPT; j += 4) {
                    const float4 v = *reinterpret_cast<const float4 *>(ro + j);
                    acc[j] += v.x * wgt;
                    acc[j + 1] += v.y * wgt;
                    acc[j + 2] += v.z * wgt;
                    acc[j + 3] += v.w * wgt;
                }
            }
            const float inv = Lg > 0.f ? 1.0f / Lg : 0.f;
#pragma unroll
            for (int j = 0; j < DPT; j++) p.out[out_row * D + d0 + j] = __float2half_rn(acc[j] * inv);
        }
        return;
    }

    // ---- split keys: publish the partial, last CTA of the tile merges ----
    if (row_valid) {
        const size_t pi = out_row * p.nsplit + split;
        if ((tid & 7) == 0) {
            p.part_ml[pi * 2] = M;
            p.part_ml[pi * 2 + 1] = L;
        }
#pragma unroll
        for (int j = 0; j < DPT; j += 4)
            *reinterpret_cast<float4 *>(p.part_o + pi * D + d0 + j) = make_float4(acc[j], acc[j + 1], acc[j + 2], acc[j + 3]);
    }
    __threadfence();
    __syncthreads();
    if (tid == 0) {
        int *ctr = p.counters + ((size_t)b * p.q_tiles + qt) * p.Hkv + hk;
        const int ticket = atomicAdd(ctr, 1);
        sm_last = ticket == p.nsplit - 1;
        if (sm_last) *ctr = 0;  // ready for the next launch
    }
    __syncthreads();
    if (!sm_last) return;
    __threadfence();
    if (row_valid) {
        // loads of several splits in flight at once: a merge of 64 splits is a chain of L2 round trips otherwise
        float Mg = -INFINITY;
#pragma unroll 8
        for (int sp = 0; sp < p.nsplit; sp++) Mg = fmaxf(Mg, __ldcg(&p.part_ml[(out_row * p.nsplit + sp) * 2]));
        float Lg = 0.f;
#pragma unroll
        for (int j = 0; j < DPT; j++) acc[j] = 0.f;
#pragma unroll 4
        for (int sp = 0; sp < p.nsplit; sp++) {
            const size_t pi = out_row * p.nsplit + sp;
            const float2 ml = __ldcg(reinterpret_cast<const float2 *>(p.part_ml + pi * 2));
            const float wgt = ml.x == -INFINITY ? 0.f : expf(ml.x - Mg);
            Lg += ml.y * wgt;
#pragma unroll
            for (int j = 0; j < DPT; j += 4) {
                const float4 v = __ldcg(reinterpret_cast<const float4 *>(p.part_o + pi * D + d0 + j));
                acc[j] += v.x * wgt;
                acc[j + 1] += v.y * wgt;
                acc[j + 2] += v.z * wgt;
                acc[j + 3] += v.w * wgt;
            }
        }
        const float inv = Lg > 0.f ? 1.0f / Lg : 0.f;
#pragma unroll
        for (int j = 0; j < DPT; j++) p.out[out_row * D + d0 + j] = __float2half_rn(acc[j] * inv);
    }
}

// Prefill variant: one CTA owns 64 (query, head) rows that share a KV head -- the G
// query heads of the group times 64/G query positions -- and walks the keys in tiles
// of 64.  Each of the 4 warps takes 16 ROWS against the whole tile (the decode kernel
// above gives each warp 16 KEYS of the tile instead): a K/V tile fetched from L2 now
// serves 64 rows, a quarter of the traffic of the 16-row tiling, and a row's softmax
// statistics stay inside one warp, so there is nothing to merge at the end.  Same
// arithmetic: f16 roundings of the scores (einsum output, then the f16 multiply by the
// scale) and of P, online softmax and O accumulation in f32.
template <int D>
__global__ void __launch_bounds__(kAttnThreads) attention_prefill_kernel(const AttnParams p) {
    constexpr int PITCH = D + 8;
    constexpr int TILE = kTileKeys * PITCH;
    constexpr int KSTEPS = D / 16;
    constexpr int NDT = D / 8;
    extern __shared__ __align__(128) uint8_t smem_raw[];
    __half *ks = reinterpret_cast<__half *>(smem_raw);  // [2][TILE]
    __half *vs = ks + 2 * TILE;                         // [2][TILE]

    tlc_pdl_prologue();
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, t = lane & 3;
    const int b = blockIdx.z, hk = blockIdx.y, qt = blockIdx.x;
    const int G = p.G, RQ = 64 / G;
    const int pos0 = p.q_pos0;
    const int T = min(pos0 + p.I, p.key_limit);  // the host checks pos0 + I <= Tmax; never read past the cache
    // rows of this warp: r_lo = 16*warp + g, r_hi = r_lo + 8; r -> (query qt*RQ + r/G, head hk*G + r%G)
    const int r_lo = 16 * warp + g, r_hi = r_lo + 8;
    const int qi_lo = qt * RQ + r_lo / G, qi_hi = qt * RQ + r_hi / G;
    const int head_lo = hk * G + r_lo % G, head_hi = hk * G + r_hi % G;
    const bool valid_lo = qi_lo < p.I, valid_hi = qi_hi < p.I;
    const int rpos_lo = pos0 + qi_lo, rpos_hi = pos0 + qi_hi;
    // last key any row of this warp may see (warp-uniform): rows 16*warp .. 16*warp+15
    const int warp_last_q = min(p.I - 1, qt * RQ + (16 * warp + 15) / G);
    const int warp_end = pos0 + warp_last_q + 1;
    const int last_q = min(p.I, (qt + 1) * RQ) - 1;
    const int k_end = min(T, pos0 + last_q + 1);
    const int ntiles = (k_end + kTileKeys - 1) / kTileKeys;

    uint32_t qa[KSTEPS][4];
    {
        const __half *q_lo = p.q + ((size_t)(b * p.I + (valid_lo ? qi_lo : 0)) * p.H + head_lo) * D;
        const __half *q_hi = p.q + ((size_t)(b * p.I + (valid_hi ? qi_hi : 0)) * p.H + head_hi) * D;
#pragma unroll
        for (int kk = 0; kk < KSTEPS; kk++) {
            qa[kk][0] = valid_lo ? *reinterpret_cast<const uint32_t *>(q_lo + 16 * kk + 2 * t) : 0u;
            qa[kk][1] = valid_hi ? *reinterpret_cast<const uint32_t *>(q_hi + 16 * kk + 2 * t) : 0u;
            qa[kk][2] = valid_lo ? *reinterpret_cast<const uint32_t *>(q_lo + 16 * kk + 8 + 2 * t) : 0u;
            qa[kk][3] = valid_hi ? *reinterpret_cast<const uint32_t *>(q_hi + 16 * kk + 8 + 2 * t) : 0u;
        }
    }
    const __half *kbase = p.kc + ((size_t)b * p.Tmax * p.Hkv + hk) * D;
    const __half *vbase = p.vc + ((size_t)b * p.Tmax * p.Hkv + hk) * D;
    const size_t key_stride = (size_t)p.Hkv * D;
    auto load_tile = [&](int tile, int stage) {
        const int j0 = tile * kTileKeys;
        constexpr int CHUNKS = kTileKeys * (D / 8);
#pragma unroll
        for (int c = tid; c < CHUNKS; c += kAttnThreads) {
            const int key = c / (D / 8), part = c % (D / 8);
            const bool ok = j0 + key < k_end;
            const size_t off = (size_t)(ok ? j0 + key : 0) * key_stride + part * 8;
            cp_async16(ks + stage * TILE + key * PITCH + part * 8, kbase + off, ok);
            cp_async16(vs + stage * TILE + key * PITCH + part * 8, vbase + off, ok);
        }
        cp_async_commit();
    };

    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
    float o[NDT][4];
#pragma unroll
    for (int i = 0; i < NDT; i++) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    const __half scale_h = __float2half_rn(p.scale);

    if (ntiles > 0) load_tile(0, 0);
    for (int tile = 0; tile < ntiles; tile++) {
        const int stage = tile & 1;
        if (tile + 1 < ntiles) {
            load_tile(tile + 1, stage ^ 1);
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();
        const int j0 = tile * kTileKeys;
        if (j0 < warp_end) {  // causal: tiles past this warp's last row are skipped
            const __half *kt = ks + stage * TILE;
            const __half *vt = vs + stage * TILE;
            float s[8][4];
#pragma unroll
            for (int i = 0; i < 8; i++) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
#pragma unroll
            for (int kk = 0; kk < KSTEPS; kk++) {
#pragma unroll
                for (int np = 0; np < 4; np++) {  // two n8 tiles (16 keys) per ldmatrix.x4
                    uint32_t r[4];
                    const int mi = lane >> 3;
                    ldsm_x4(r, kt + (16 * np + (mi >> 1) * 8 + (lane & 7)) * PITCH + 16 * kk + (mi & 1) * 8);
                    mma16816(s[2 * np], qa[kk], r[0], r[1]);
                    mma16816(s[2 * np + 1], qa[kk], r[2], r[3]);
                }
            }
            float mx[2] = {-INFINITY, -INFINITY};
            // a tile wholly below the diagonal of this warp's rows and inside the context needs no mask
            const bool unmasked = j0 + kTileKeys <= k_end && j0 + kTileKeys - 1 <= pos0 + qt * RQ + (16 * warp) / G;
            const __half2 scale_h2 = __half2half2(scale_h);
#pragma unroll
            for (int nt = 0; nt < 8; nt++)
#pragma unroll
                for (int e = 0; e < 4; e += 2) {
                    // two roundings as the reference does: the score to f16, then its product with the scale
                    const float2 v2 = __half22float2(__hmul2(__floats2half2_rn(s[nt][e], s[nt][e + 1]), scale_h2));
                    float v0 = v2.x, v1 = v2.y;
                    if (!unmasked) {
                        const int key = j0 + nt * 8 + 2 * t;
                        const int rpos = e < 2 ? rpos_lo : rpos_hi;
                        if (key >= k_end || key > rpos) v0 = -INFINITY;
                        if (key + 1 >= k_end || key + 1 > rpos) v1 = -INFINITY;
                    }
                    s[nt][e] = v0;
                    s[nt][e + 1] = v1;
                    mx[e >> 1] = fmaxf(mx[e >> 1], fmaxf(v0, v1));
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
            for (int nt = 0; nt < 8; nt++)
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
#pragma unroll
            for (int kp = 0; kp < 4; kp++) {  // 16 keys of the tile per step
                uint32_t pa[4];
                pa[0] = pack_half2(s[2 * kp][0], s[2 * kp][1]);
                pa[1] = pack_half2(s[2 * kp][2], s[2 * kp][3]);
                pa[2] = pack_half2(s[2 * kp + 1][0], s[2 * kp + 1][1]);
                pa[3] = pack_half2(s[2 * kp + 1][2], s[2 * kp + 1][3]);
#pragma unroll
                for (int jd = 0; jd < KSTEPS; jd++) {
                    uint32_t r[4];
                    const int mi = lane >> 3;
                    ldsm_x4_trans(r, vt + (16 * kp + (mi & 1) * 8 + (lane & 7)) * PITCH + 16 * jd + (mi >> 1) * 8);
                    mma16816(o[2 * jd], pa, r[0], r[1]);
                    mma16816(o[2 * jd + 1], pa, r[2], r[3]);
                }
            }
        }
        __syncthreads();
    }
#pragma unroll
    for (int h = 0; h < 2; h++) {
        l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 1);
        l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 2);
    }
    const float inv_lo = l_run[0] > 0.f ? 1.0f / l_run[0] : 0.f, inv_hi = l_run[1] > 0.f ? 1.0f / l_run[1] : 0.f;
    __half *out_lo = p.out + ((size_t)(b * p.I + (valid_lo ? qi_lo : 0)) * p.H + head_lo) * D;
    __half *out_hi = p.out + ((size_t)(b * p.I + (valid_hi ? qi_hi : 0)) * p.H + head_hi) * D;
#pragma unroll
    for (int i = 0; i < NDT; i++) {
        if (valid_lo)
            *reinterpret_cast<__half2 *>(out_lo + 8 * i + 2 * t) = __floats2half2_rn(o[i][0] * inv_lo, o[i][1] * inv_lo);
        if (valid_hi)
            *reinterpret_cast<__half2 *>(out_hi + 8 * i + 2 * t) = __floats2half2_rn(o[i][2] * inv_hi, o[i][3] * inv_hi);
    }
}

// cache.append for the unfused surface: rows of K/V [m, Hkv*D] go to position
// pos(row) of sequence seq(row).
// Dynamic shared memory an attention_kernel<D> launch may ask for: the K/V tiles plus, in
// cluster mode, the merge area of rank 0.  Every place that sets the kernel's limit uses this
// value, so one launcher never lowers the limit another one needs.
static constexpr size_t attention_smem_limit(int D) {
    return (size_t)4 * kTileKeys * (D + 8) * sizeof(__half) + 128 + (size_t)16 * 16 * (D + 2) * sizeof(float);
}

__global__ void kv_append_kernel(const __half *__restrict__ k, const __half *__restrict__ v,
                                 __half *__restrict__ kc, __half *__restrict__ vc, int m, int row_elems,
                                 int tmax, int pos_offset, const int *__restrict__ positions, int batched) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (size_t)m * row_elems) return;
    const int r = (int)(i / row_elems), c = (int)(i % row_elems);
    const int pos = positions ? positions[r] : pos_offset + (batched ? 0 : r);
    const size_t seq = batched ? r : 0;
    const size_t dst = (seq * tmax + pos) * row_elems + c;
    kc[dst] = k[i];
    vc[dst] = v[i];
}

}  // namespace

// How many clusters of sixteen attention CTAs (with the merge area for sixteen splits) the
// device can hold at once; 0 when it cannot place one.  Allows the non-portable cluster size
// on first use.
static int attention_wide_clusters(tlc_ctx *ctx, int D) {
    static int cached[2][64];
    static bool known[2][64] = {};
    const int di = D == 64 ? 0 : 1, dev = ctx->device & 63;
    if (known[di][dev]) return cached[di][dev];
    known[di][dev] = true;
    cached[di][dev] = 0;
    const void *fn = D == 64 ? (const void *)attention_kernel<64> : (const void *)attention_kernel<128>;
    if (cudaFuncSetAttribute(fn, cudaFuncAttributeNonPortableClusterSizeAllowed, 1) != cudaSuccess ||
        cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)attention_smem_limit(D)) != cudaSuccess) {
        cudaGetLastError();
        return 0;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(16, 1, 1);
    cfg.blockDim = dim3(kAttnThreads);
    cfg.dynamicSmemBytes = attention_smem_limit(D);
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 16;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    int n = 0;
    cudaError_t e = D == 64 ? cudaOccupancyMaxActiveClusters(&n, attention_kernel<64>, &cfg)
                            : cudaOccupancyMaxActiveClusters(&n, attention_kernel<128>, &cfg);
    if (e != cudaSuccess) {
        cudaGetLastError();
        n = 0;
    }
    cached[di][dev] = n;
    return n;
}

// Host-side launcher shared by the ABI entry point and the decode runner.
//   batch sequences, I queries each (I == 1 when positions_dev is given).
//   nsplit_hint <= 0: choose from the key count; with positions_dev the key
//   count is only known on the device, so max_keys bounds it.
//   positions_settled: the caller vouches that positions_dev[] is final before this kernel can
//   be scheduled, not merely before its dependency wait returns.  A kernel can be scheduled once
//   every CTA of its predecessor has let dependents in, so this holds when some kernel between
//   the writer of the positions and this one does that only after its own dependency wait, or is
//   launched the plain way: that kernel's wait returns when its predecessor is complete, and a
//   grid is complete only when its threads have passed their own waits, back to the writer.  In
//   the decode runner the writer is the previous step's sampling kernel and the kernel in between
//   is the q/k/v GEMV (pdl_mode 2, 3 or 4) or, from 17 rows on, the plain-launched RMSNorm in
//   front of the q/k/v GEMM; with pdl_mode 0 or 1 the runner passes false, and so does the
//   builtin, whose caller may have written the positions with the kernel right before.
int32_t tlc_launch_attention(tlc_ctx *ctx, tlc_kvcache *cache, int layer, const void *q_dev, void *out_dev,
                             int batch, int I, int n_heads, int q_pos0, const int *positions_dev, int max_keys,
                             float scale, bool positions_settled) {
    TLC_REQUIRE(cache && q_dev && out_dev, TLC_ERR_INVALID_OPERATION, "attention: null pointer");
    TLC_REQUIRE(layer >= 0 && layer < cache->n_layers, TLC_ERR_INDEX, "Index out of bounds: index %d, size %d",
                layer, cache->n_layers);
    TLC_REQUIRE(batch >= 1 && batch <= cache->max_batch, TLC_ERR_SHAPE_MISMATCH,
                "attention: batch %d exceeds the cache's %d sequences", batch, cache->max_batch);
    const int D = cache->head_dim, Hkv = cache->n_kv_heads;
    TLC_REQUIRE(n_heads % Hkv == 0, TLC_ERR_SHAPE_MISMATCH, "attention: %d query heads over %d KV heads", n_heads,
                Hkv);
    const int G = n_heads / Hkv;
    TLC_REQUIRE(G == 1 || G == 2 || G == 4 || G == 8 || G == 16, TLC_ERR_INVALID_OPERATION,
                "attention: group size %d unsupported (1, 2, 4, 8, 16)", G);
    TLC_REQUIRE(D == 64 || D == 128, TLC_ERR_INVALID_OPERATION, "attention: head_dim %d unsupported (64, 128)", D);
    TLC_REQUIRE(I >= 1 && (positions_dev == nullptr || I == 1), TLC_ERR_INVALID_OPERATION,
                "attention: per-sequence positions need one query per sequence");
    const int T = positions_dev ? max_keys : q_pos0 + I;
    TLC_REQUIRE(T >= 1 && T <= cache->max_seq, TLC_ERR_INDEX, "Index out of bounds: index %d, size %d", T,
                cache->max_seq);

    AttnParams p{};
    p.q = static_cast<const __half *>(q_dev);
    p.kc = cache->k + (size_t)layer * cache->layer_stride;
    p.vc = cache->v + (size_t)layer * cache->layer_stride;
    p.out = static_cast<__half *>(out_dev);
    p.I = I;
    p.H = n_heads;
    p.Hkv = Hkv;
    p.G = G;
    p.Tmax = cache->max_seq;
    p.q_pos0 = q_pos0;
    p.positions = positions_dev;
    p.scale = scale;
    p.pos_settled = positions_settled ? 1 : 0;
    p.key_limit = T;  // <= max_seq (checked above); a position beyond it is cut on the device
    p.status = ctx->dev_status;
    if (I > 1) {
        // Prefill: 64-row tiles, the warps split the rows (attention_prefill_kernel).
        p.nsplit = 1;
        const int RQ64 = 64 / G;
        p.q_tiles = (I + RQ64 - 1) / RQ64;
        const size_t smem_pf = (size_t)4 * kTileKeys * (D + 8) * sizeof(__half);
        static bool configured_pf[2][64] = {};
        const int dj = D == 64 ? 0 : 1;
        if (!configured_pf[dj][ctx->device & 63]) {
            if (D == 64) {
                TLC_CUDA(cudaFuncSetAttribute(attention_prefill_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                              (int)smem_pf));
                TLC_CUDA(cudaFuncSetAttribute(attention_prefill_kernel<64>,
                                              cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared));
            } else {
                TLC_CUDA(cudaFuncSetAttribute(attention_prefill_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                              (int)smem_pf));
                TLC_CUDA(cudaFuncSetAttribute(attention_prefill_kernel<128>,
                                              cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared));
            }
            configured_pf[dj][ctx->device & 63] = true;
        }
        const dim3 grid_pf(p.q_tiles, Hkv, batch);
        cudaError_t le = D == 64 ? tlc_launch_pdl(ctx, attention_prefill_kernel<64>, grid_pf, dim3(kAttnThreads), smem_pf, p)
                                 : tlc_launch_pdl(ctx, attention_prefill_kernel<128>, grid_pf, dim3(kAttnThreads), smem_pf, p);
        if (le != cudaSuccess) {
            cudaGetLastError();
            return tlc_fail(TLC_ERR_CUDA, "attention launch failed: %s", cudaGetErrorString(le));
        }
        TLC_CHECK_LAUNCH(ctx);
        return TLC_OK;
    }
    const int RQ = 16 / G;
    p.q_tiles = (I + RQ - 1) / RQ;
    // Decode: split the keys so that about two CTAs per SM are busy.
    int nsplit = 1;
    if (I == 1) {
        const int tiles = (T + kTileKeys - 1) / kTileKeys;
        const int want = (2 * ctx->sm_count + batch * Hkv - 1) / (batch * Hkv);
        nsplit = tiles < want ? tiles : want;
        if (nsplit < 1) nsplit = 1;
        if (nsplit > 64) nsplit = 64;
    }
    // Up to 128 key tiles (8192 keys) the splits of a tile form one thread-block cluster
    // (8 CTAs, up to 16 tiles each, walked with the double-buffered tile loop) and merge
    // through distributed shared memory; beyond that, up to 64 independent splits and the
    // global-memory merge.
    // A portable cluster holds eight splits.  With few (sequence, KV head) tiles -- one KV head
    // per rank of a tensor-parallel model, one sequence -- eight CTAs would walk a long context
    // alone on an otherwise idle GPU: such launches use clusters of sixteen (option attn_wide).
    const bool cluster = I == 1 && nsplit > 1 && (T + kTileKeys - 1) / kTileKeys <= 128;
    const bool wide = cluster && ctx->attn_wide && nsplit >= 16 && (T + kTileKeys - 1) / kTileKeys >= 24 &&
                      (long)batch * Hkv * 32 <= ctx->sm_count && attention_wide_clusters(ctx, D) > 0;
    if (cluster && nsplit > (wide ? 16 : 8)) nsplit = wide ? 16 : 8;
    p.push_splits = wide ? 16 : 8;
    p.nsplit = nsplit;
    p.cluster = cluster ? 1 : 0;
    const int tiles_total = (T + kTileKeys - 1) / kTileKeys;
    p.keys_per_split = ((tiles_total + nsplit - 1) / nsplit) * kTileKeys;
    if (nsplit > 1 && !cluster) {
        const size_t rows = (size_t)batch * I * n_heads;
        const size_t ml = (rows * nsplit * 2 * sizeof(float) + 15) & ~(size_t)15, po = rows * nsplit * D * sizeof(float);
        // Ticket counters (one per tile, zero between launches: the merging
        // CTA resets its own) live in a small zero-initialised context buffer.
        TLC_REQUIRE((size_t)batch * p.q_tiles * Hkv <= ctx->n_tickets, TLC_ERR_INVALID_OPERATION,
                    "attention: %d x %d tiles exceed the ticket area", batch, Hkv);
        if (int32_t rc = tlc_scratch_reserve(ctx, ml + po)) return rc;
        p.part_ml = static_cast<float *>(ctx->scratch);
        p.part_o = reinterpret_cast<float *>(static_cast<uint8_t *>(ctx->scratch) + ml);
        p.counters = ctx->tickets;
    }
    dim3 grid(p.q_tiles * nsplit, Hkv, batch);
    const size_t smem = (size_t)4 * kTileKeys * (D + 8) * sizeof(__half);
    const size_t smem_o = (size_t)4 * 16 * D * sizeof(float);
    size_t smem_bytes = smem > smem_o ? smem : smem_o;
    if (cluster) {  // the merge area of rank 0 (every CTA of the launch has the same layout)
        p.push_offset = (int)((smem_bytes + 127) & ~(size_t)127);
        smem_bytes = (size_t)p.push_offset + (size_t)p.push_splits * 16 * (D + 2) * sizeof(float);
    }
    // All kernels of a decode step ask for the same (maximal) shared-memory
    // carve-out: switching the L1/shared split between consecutive launches
    // makes the SMs drain first.
    static bool configured[2][64] = {};
    const int di = D == 64 ? 0 : 1;
    if (!configured[di][ctx->device & 63]) {
        if (D == 64) {
            TLC_CUDA(cudaFuncSetAttribute(attention_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                          (int)attention_smem_limit(64)));
            TLC_CUDA(cudaFuncSetAttribute(attention_kernel<64>, cudaFuncAttributePreferredSharedMemoryCarveout,
                                          cudaSharedmemCarveoutMaxShared));
        } else {
            TLC_CUDA(cudaFuncSetAttribute(attention_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                          (int)attention_smem_limit(128)));
            TLC_CUDA(cudaFuncSetAttribute(attention_kernel<128>, cudaFuncAttributePreferredSharedMemoryCarveout,
                                          cudaSharedmemCarveoutMaxShared));
        }
        configured[di][ctx->device & 63] = true;
    }
    cudaError_t le;
    if (cluster) {
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = grid;
        cfg.blockDim = dim3(kAttnThreads);
        cfg.dynamicSmemBytes = smem_bytes;
        cfg.stream = ctx->stream;
        cudaLaunchAttribute attr[2];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = (unsigned)nsplit;
        attr[0].val.clusterDim.y = 1;
        attr[0].val.clusterDim.z = 1;
        attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[1].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = ctx->use_pdl && ctx->pdl_small ? 2 : 1;
        le = D == 64 ? cudaLaunchKernelEx(&cfg, attention_kernel<64>, p) : cudaLaunchKernelEx(&cfg, attention_kernel<128>, p);
    } else {
        le = D == 64 ? tlc_launch_pdl(ctx, attention_kernel<64>, grid, dim3(kAttnThreads), smem_bytes, p)
                     : tlc_launch_pdl(ctx, attention_kernel<128>, grid, dim3(kAttnThreads), smem_bytes, p);
    }
    if (le != cudaSuccess) {
        cudaGetLastError();
        return tlc_fail(TLC_ERR_CUDA, "attention launch failed: %s", cudaGetErrorString(le));
    }
    TLC_CHECK_LAUNCH(ctx);
    return TLC_OK;
}

extern "C" int32_t tlc_kvcache_create(tlc_ctx *ctx, int32_t n_layers, int32_t max_batch, int32_t max_seq,
                                      int32_t n_kv_heads, int32_t head_dim, tlc_kvcache **out) {
    if (int32_t rc = tlc_enter(ctx)) return rc;
    TLC_REQUIRE(out, TLC_ERR_INVALID_OPERATION, "kvcache_create: null out pointer");
    *out = nullptr;
    TLC_REQUIRE(n_layers > 0 && max_batch > 0 && max_seq > 0 && n_kv_heads > 0 && head_dim > 0 && head_dim % 8 == 0,
                TLC_ERR_INVALID_DIMENSION, "kvcache_create: bad shape");
    tlc_kvcache *c = new tlc_kvcache();
    c->ctx = ctx;
    c->n_layers = n_layers;
    c->max_batch = max_batch;
    c->max_seq = max_seq;
    c->n_kv_heads = n_kv_heads;
    c->head_dim = head_dim;
    c->layer_stride = (size_t)max_batch * max_seq * n_kv_heads * head_dim;
    const size_t bytes = c->layer_stride * n_layers * sizeof(__half);
    cudaError_t e = cudaMalloc(&c->k, bytes);
    if (e == cudaSuccess) e = cudaMalloc(&c->v, bytes);
    if (e == cudaSuccess) e = cudaMemsetAsync(c->k, 0, bytes, ctx->stream);
    if (e == cudaSuccess) e = cudaMemsetAsync(c->v, 0, bytes, ctx->stream);
    if (e != cudaSuccess) {
        cudaGetLastError();
        if (c->k) cudaFree(c->k);
        if (c->v) cudaFree(c->v);
        delete c;
        return tlc_fail(TLC_ERR_ALLOCATION, "KV cache allocation of 2 x %zu bytes failed: %s", bytes,
                        cudaGetErrorString(e));
    }
    *out = c;
    return TLC_OK;
}

extern "C" int32_t tlc_kvcache_destroy(tlc_kvcache *cache) {
    if (!cache) return TLC_OK;
    cudaSetDevice(cache->ctx->device);
    cudaFree(cache->k);
    cudaFree(cache->v);
    delete cache;
    return TLC_OK;
}

extern "C" int32_t tlc_kvcache_layer_ptrs(tlc_kvcache *cache, int32_t layer, void **k_dev, void **v_dev) {
    TLC_REQUIRE(cache && layer >= 0 && layer < cache->n_layers, TLC_ERR_INDEX, "kvcache: bad layer %d", layer);
    if (k_dev) *k_dev = cache->k + (size_t)layer * cache->layer_stride;
    if (v_dev) *v_dev = cache->v + (size_t)layer * cache->layer_stride;
    return TLC_OK;
}

extern "C" int32_t tlc_kvcache_append(tlc_ctx *ctx, tlc_kvcache *cache, int32_t layer, const void *k_dev,
                                      const void *v_dev, int32_t m, int32_t pos_offset,
                                      const int32_t *positions_dev) {
    if (int32_t rc = tlc_enter(ctx)) return rc;
    TLC_REQUIRE(cache && k_dev && v_dev, TLC_ERR_INVALID_OPERATION, "kvcache_append: null pointer");
    TLC_REQUIRE(layer >= 0 && layer < cache->n_layers, TLC_ERR_INDEX, "Index out of bounds: index %d, size %d",
                layer, cache->n_layers);
    const bool batched = positions_dev != nullptr;
    if (batched)
        TLC_REQUIRE(m <= cache->max_batch, TLC_ERR_SHAPE_MISMATCH, "kvcache_append: %d rows for %d sequences", m,
                    cache->max_batch);
    else
        TLC_REQUIRE(pos_offset >= 0 && pos_offset + m <= cache->max_seq, TLC_ERR_INDEX,
                    "Index out of bounds: index %d, size %d", pos_offset + m, cache->max_seq);
    if (m <= 0) return TLC_OK;
    const int row_elems = cache->n_kv_heads * cache->head_dim;
    const size_t total = (size_t)m * row_elems;
    kv_append_kernel<<<(unsigned)((total + 255) / 256), 256, 0, ctx->stream>>>(
        static_cast<const __half *>(k_dev), static_cast<const __half *>(v_dev),
        cache->k + (size_t)layer * cache->layer_stride, cache->v + (size_t)layer * cache->layer_stride, m, row_elems,
        cache->max_seq, pos_offset, positions_dev, batched ? 1 : 0);
    TLC_CHECK_LAUNCH(ctx);
    return TLC_OK;
}

extern "C" int32_t tlc_attention(tlc_ctx *ctx, tlc_kvcache *cache, int32_t layer, const void *q_dev,
                                 void *out_dev, int32_t batch, int32_t n_queries, int32_t n_heads,
                                 int32_t q_pos0, const int32_t *positions_dev, int32_t max_keys, float scale) {
    if (int32_t rc = tlc_enter(ctx)) return rc;
    tlc_perf_scope perf(ctx, "attention(batch=%d, queries=%d, heads=%d)", batch, n_queries, n_heads);
    return tlc_launch_attention(ctx, cache, layer, q_dev, out_dev, batch, n_queries, n_heads, q_pos0,
                                positions_dev, max_keys, scale, false);
}

// ---------------------------------------------------------------------------
// Decode attention for callers that must not allocate.
//
// Some hosts of this library run the decode step from places where device
// memory cannot be requested: inside a CUDA-graph capture or a latency-critical
// serving loop (cudaMalloc synchronises the device and is illegal while
// capturing), or under a memory manager that owns every byte of HBM and hands
// the library nothing.  tlc_attention() above grows a scratch block with
// cudaMalloc when the split-key partials do not fit.  This variant keeps the
// partials and the ticket counters in a fixed array inside the library image
// instead: kStaticScratchBytes of device memory per GPU that loads the library,
// held until the process exits.
// ---------------------------------------------------------------------------
namespace {

constexpr size_t kStaticPartialBytes = (size_t)2 << 20;  // split-key partials (max, sum, O)
constexpr size_t kStaticTicketBytes = 4096;              // one int per (sequence, KV head)
constexpr size_t kStaticStatusBytes = 256;               // a tlc_dev_status: "a position was cut at max_keys"
constexpr size_t kStaticScratchBytes = kStaticPartialBytes + kStaticTicketBytes + kStaticStatusBytes;

static __device__ __align__(256) unsigned char g_static_attention_scratch[kStaticScratchBytes];

struct StaticSetup {
    bool done = false;
    unsigned char *scratch = nullptr;  // device address of g_static_attention_scratch on that device
    int sm_count = 0;
};
StaticSetup g_static_setup[64];
std::mutex g_static_setup_mutex;  // two host threads may make the first call on a device at once

}  // namespace

extern "C" int32_t tlc_attention_decode_static(void *stream, const void *q_dev, const void *k_cache_dev,
                                               const void *v_cache_dev, void *out_dev, int32_t batch,
                                               int32_t n_heads, int32_t n_kv_heads, int32_t head_dim,
                                               int32_t max_seq, const int32_t *positions_dev, int32_t max_keys,
                                               float scale) {
    TLC_REQUIRE(q_dev && k_cache_dev && v_cache_dev && out_dev && positions_dev, TLC_ERR_INVALID_OPERATION,
                "attention_decode_static: null pointer");
    TLC_REQUIRE(batch >= 1 && n_heads >= 1 && n_kv_heads >= 1 && n_heads % n_kv_heads == 0, TLC_ERR_SHAPE_MISMATCH,
                "attention_decode_static: batch %d, %d query heads over %d KV heads", batch, n_heads, n_kv_heads);
    const int G = n_heads / n_kv_heads, D = head_dim;
    TLC_REQUIRE(G == 1 || G == 2 || G == 4 || G == 8 || G == 16, TLC_ERR_INVALID_OPERATION,
                "attention: group size %d unsupported (1, 2, 4, 8, 16)", G);
    TLC_REQUIRE(D == 64 || D == 128, TLC_ERR_INVALID_OPERATION, "attention: head_dim %d unsupported (64, 128)", D);
    TLC_REQUIRE(max_keys >= 1 && max_keys <= max_seq, TLC_ERR_INDEX, "Index out of bounds: index %d, size %d", max_keys,
                max_seq);
    int device = 0;
    TLC_CUDA(cudaGetDevice(&device));
    TLC_REQUIRE(device >= 0 && device < 64, TLC_ERR_DEVICE, "device ordinal %d out of range", device);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (st != nullptr && st != cudaStreamLegacy && st != cudaStreamPerThread) {
        // the scratch address below belongs to the current device; a stream of another one would
        // run the kernel there with this device's pointers
        int sdev = -1;
        TLC_CUDA(cudaStreamGetDevice(st, &sdev));
        TLC_REQUIRE(sdev == device, TLC_ERR_DEVICE,
                    "attention_decode_static: the stream belongs to device %d, the current device is %d", sdev, device);
    }
    StaticSetup &su = g_static_setup[device];
    const size_t smem = (size_t)4 * kTileKeys * (D + 8) * sizeof(__half);
    const size_t smem_o = (size_t)4 * 16 * D * sizeof(float);
    const size_t smem_bytes = smem > smem_o ? smem : smem_o;
    std::lock_guard<std::mutex> setup_lock(g_static_setup_mutex);
    if (!su.done) {
        // First call on this device (which is the current one): in host code the
        // array's name is only a stand-in, the kernel needs its device address.
        void *p = nullptr;
        cudaError_t e = cudaGetSymbolAddress(&p, g_static_attention_scratch);
        if (e != cudaSuccess || p == nullptr) {
            cudaGetLastError();
            return tlc_fail(TLC_ERR_CUDA, "cudaGetSymbolAddress(static attention scratch) failed on device %d: %s",
                            device, cudaGetErrorString(e));
        }
        TLC_CUDA(cudaDeviceGetAttribute(&su.sm_count, cudaDevAttrMultiProcessorCount, device));
        TLC_CUDA(cudaFuncSetAttribute(attention_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      (int)attention_smem_limit(64)));
        TLC_CUDA(cudaFuncSetAttribute(attention_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      (int)attention_smem_limit(128)));
        su.scratch = static_cast<unsigned char *>(p);
        // the status word starts at zero like every __device__ array; later calls leave it alone
        su.done = true;
    }

    AttnParams p{};
    p.q = static_cast<const __half *>(q_dev);
    p.kc = static_cast<const __half *>(k_cache_dev);
    p.vc = static_cast<const __half *>(v_cache_dev);
    p.out = static_cast<__half *>(out_dev);
    p.I = 1;
    p.H = n_heads;
    p.Hkv = n_kv_heads;
    p.G = G;
    p.Tmax = max_seq;
    p.q_pos0 = 0;
    p.positions = positions_dev;
    p.scale = scale;
    // positions_dev[b] + 1 keys are read, but never more than max_keys: a larger position is cut
    // there (the newest keys are dropped) and the status word below records it.
    p.key_limit = max_keys;
    p.status = reinterpret_cast<tlc_dev_status *>(su.scratch + kStaticPartialBytes + kStaticTicketBytes);
    p.q_tiles = 1;
    const int tiles = (max_keys + kTileKeys - 1) / kTileKeys;
    const int want = (2 * su.sm_count + batch * n_kv_heads - 1) / (batch * n_kv_heads);
    int nsplit = tiles < want ? tiles : want;
    if (nsplit < 1) nsplit = 1;
    if (nsplit > 64) nsplit = 64;
    p.nsplit = nsplit;
    p.keys_per_split = ((tiles + nsplit - 1) / nsplit) * kTileKeys;
    const size_t rows = (size_t)batch * n_heads;
    const size_t ml = (rows * nsplit * 2 * sizeof(float) + 15) & ~(size_t)15, po = rows * nsplit * D * sizeof(float);
    TLC_REQUIRE(nsplit == 1 || ml + po <= kStaticPartialBytes, TLC_ERR_BUFFER_EXHAUSTED,
                "attention_decode_static: %d sequences x %d heads x %d key splits need %zu bytes of partials, the "
                "built-in scratch holds %zu; use tlc_attention or a smaller batch",
                batch, n_heads, nsplit, ml + po, kStaticPartialBytes);
    TLC_REQUIRE((size_t)batch * n_kv_heads * sizeof(int) <= kStaticTicketBytes, TLC_ERR_BUFFER_EXHAUSTED,
                "attention_decode_static: %d x %d (sequence, KV head) pairs exceed the %zu built-in tickets", batch,
                n_kv_heads, kStaticTicketBytes / sizeof(int));
    p.part_ml = reinterpret_cast<float *>(su.scratch);
    p.part_o = reinterpret_cast<float *>(su.scratch + ml);
    p.counters = reinterpret_cast<int *>(su.scratch + kStaticPartialBytes);
    // The array keeps whatever the previous call left; only the tickets must start at zero.
    TLC_CUDA(cudaMemsetAsync(p.counters, 0, (size_t)batch * n_kv_heads * sizeof(int), st));
    dim3 grid(nsplit, n_kv_heads, batch);
    if (D == 64)
        attention_kernel<64><<<grid, kAttnThreads, smem_bytes, st>>>(p);
    else
        attention_kernel<128><<<grid, kAttnThreads, smem_bytes, st>>>(p);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return tlc_fail(TLC_ERR_CUDA, "kernel launch failed: %s", cudaGetErrorString(e));
    return TLC_OK;
}

// Reads (and clears) the note tlc_attention_decode_static leaves when a sequence's position
// was at or beyond max_keys and its keys were cut there: *clamped_out = 1 if that happened
// since the last query on the current device, else 0.  Waits for `stream`; allocates nothing.
extern "C" int32_t tlc_attention_decode_static_status(void *stream, int32_t *clamped_out) {
    TLC_REQUIRE(clamped_out, TLC_ERR_INVALID_OPERATION, "attention_decode_static_status: null pointer");
    *clamped_out = 0;
    int device = 0;
    TLC_CUDA(cudaGetDevice(&device));
    TLC_REQUIRE(device >= 0 && device < 64, TLC_ERR_DEVICE, "device ordinal %d out of range", device);
    unsigned char *scratch = nullptr;
    {
        std::lock_guard<std::mutex> setup_lock(g_static_setup_mutex);
        if (!g_static_setup[device].done) return TLC_OK;  // never called here: nothing was cut
        scratch = g_static_setup[device].scratch;
    }
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    tlc_dev_status h{};
    void *word = scratch + kStaticPartialBytes + kStaticTicketBytes;
    TLC_CUDA(cudaMemcpyAsync(&h, word, sizeof(h), cudaMemcpyDeviceToHost, st));
    TLC_CUDA(cudaStreamSynchronize(st));
    if (h.code != 0) {
        TLC_CUDA(cudaMemsetAsync(word, 0, sizeof(h), st));
        TLC_CUDA(cudaStreamSynchronize(st));
        *clamped_out = 1;
    }
    return TLC_OK;
}
