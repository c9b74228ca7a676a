// LLaMA-architecture forward pass over quantized-resident weights.
//
// The reference has no compiled model: LlamaModel::forward is a stub
// (src/model/llama.rs:257-266) and the forward pass is a TL script that calls
// builtins one by one (debug/chat_demo_with_kvcache.tl:136-181 prefill,
// :213-296 decode), about 28 dispatches per layer plus a host read-back of all
// logits per token (src/interpreter/builtin_sampling.rs:131-140).  This runner
// executes the same sequence of operations with 5 launches per layer:
//
//   [rms_norm + q/k/v linears + rope(q), rope(k) + cache append]   1 launch
//   [grouped-query attention over the cache]                        1 launch
//   [o projection + residual add]                                   1 launch
//   [rms_norm + gate/up linears + silu*mul]                         1 launch
//   [down projection + residual add]                                1 launch
//
// then [rms_norm + lm_head] and an on-device sample (greedy, or temperature
// sampling with counter-based draws).  Token ids, positions and the sampled
// token live in device memory, so a decode step has no host-dependent kernel
// argument and is replayed as a CUDA graph.  A prompt of many tokens takes the
// same path with the linears on the tcgen05 GEMM (norms and SiLU.mul then run
// as their own kernels).  With tensor parallelism the o and down projections
// produce partial sums that one peer-memory kernel all-reduces and adds to the
// residual, and the vocabulary shards of the logits are all-gathered.
// RoPE takes the true position of every token (the reference's decode branch
// calls rope() with its default offset 0, chat_demo_with_kvcache.tl:236,:244).
#include <chrono>
#include <cmath>
#include <cstring>
#include <memory>

#include "tlc_internal.h"
#include "tlc_step.h"
#include "tlc_synth.cuh"

struct tlc_kvcache;
extern "C" int32_t tlc_kvcache_create(tlc_ctx *, int32_t, int32_t, int32_t, int32_t, int32_t, tlc_kvcache **);
extern "C" int32_t tlc_kvcache_destroy(tlc_kvcache *);
extern "C" int32_t tlc_kvcache_layer_ptrs(tlc_kvcache *, int32_t, void **, void **);
struct tlc_model;
extern "C" int32_t tlc_model_get(tlc_model *, const char *, tlc_qtensor **);
struct tlc_comm;
extern "C" int32_t tlc_allreduce_f16(tlc_ctx *, tlc_comm *, void *, size_t);
extern "C" int32_t tlc_allgather_f16(tlc_ctx *, tlc_comm *, const void *, void *, size_t);
extern "C" int32_t tlc_comm_size(tlc_comm *);
extern "C" int32_t tlc_comm_rank(tlc_comm *);

struct LayerWeights {
    tlc_qtensor *attn_norm, *wq, *wk, *wv, *wo, *ffn_norm, *w_gate, *w_up, *w_down;
};

// Where a decode step that runs as one graph reports to the host without copy nodes:
// pinned host words the sampling kernel writes directly (status first, then the token).
struct HostReport {
    int *host_next;                      // [batch] pinned, or null
    tlc_dev_status *host_status;         // pinned mirror of the status word
    const tlc_dev_status *dev_status;
};

struct tlc_llama {
    tlc_ctx *ctx;
    tlc_llama_config cfg;
    std::vector<LayerWeights> layers;
    tlc_qtensor *tok_embd, *out_norm, *out_w;
    tlc_kvcache *cache;
    int max_rows;  // rows of the activation buffers
    __half *x, *x1, *q, *attn, *act, *logits;
    __half *part = nullptr;         // tensor parallel: this rank's partial [rows, d] before the all-reduce
    __half *logits_full = nullptr;  // tensor parallel: gathered logits [rank][rows][vocab / tp]
    tlc_comm *comm = nullptr;
    int last_logit_rows = 1;
    int32_t *ids, *positions, *next_ids;
    int32_t *host_ids;  // pinned staging
    int32_t *host_next;
    std::map<int, cudaGraphExec_t> graph;  // decode graphs keyed by batch * 8 + parts (1000 + batch: the host step)
    const int *ids_src = nullptr;          // set while the host step is captured: token ids read from pinned memory
    HostReport report{};                   //   and results reported straight to pinned memory
    int launches_in[8] = {0, 0, 0, 0, 0, 0, 0, 0};  // kernels per step, by parts mask
    int heads_local, kv_heads_local, ffn_local, vocab_local;
    // Host-side upper bound of every sequence's position (the device copy advances by itself
    // during graph replays): no step is enqueued that would write cache row max_seq.
    std::vector<int> pos_hi;
    // The persistent decode-step kernel (tlc_step.cu): one sequence, greedy, no tensor parallelism.
    bool step_ok = false;
    int step_grid = 0, step_qtype = 0, step_kmax = 0, step_splits = 1;
    uint8_t *step_ws = nullptr;                 // global workspace: the flagged-word buffers
    tlc_step::StepWorkspace step_wsl{};
    uint32_t step_epoch = 1;                    // first epoch of the next launch (0 is never used)
    uint64_t *step_trace = nullptr;             // device buffer of the last traced launch
    size_t step_trace_words = 0;
    tlc_step::StepLayer *step_layers = nullptr;  // device copy of the per-layer pointers
    float temperature = 0.f;   // <= 1e-4: greedy
    uint64_t sample_seed = 0;  // uniform draws: counter-based, keyed by (seed, position, sequence)
};

namespace {

__device__ __forceinline__ void report_to_host(const HostReport &hr, int b, int tok) {
    if (!hr.host_next) return;
    if (b == 0 && hr.host_status) {
        hr.host_status->code = hr.dev_status->code;
        hr.host_status->where = hr.dev_status->where;
    }
    __threadfence_system();
    *reinterpret_cast<volatile int *>(hr.host_next + b) = tok;
}

__global__ void embed_kernel(const uint8_t *__restrict__ table, size_t pitch, int vocab, int d,
                             const int *__restrict__ ids, int m, __half *__restrict__ y) {
    tlc_pdl_prologue();  // ids are written by the previous step's sampling kernel
    const int vec = d >> 3;
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (size_t)m * vec) return;
    const int r = (int)(i / vec), c = (int)(i % vec);
    int id = ids[r];
    id = id < 0 ? 0 : (id >= vocab ? vocab - 1 : id);  // ids are validated on the host; never read outside
    reinterpret_cast<uint4 *>(y + (size_t)r * d)[c] = reinterpret_cast<const uint4 *>(table + (size_t)id * pitch)[c];
}

// Greedy sample + step bookkeeping, one CTA per sequence.  Ties go to the LAST
// maximal index, like Iterator::max_by in temperature_sample's greedy arm
// (src/interpreter/builtin_sampling.rs:176-181).  Also feeds the sampled token
// back as the next input and advances the sequence position.
// With tensor parallelism the logits arrive as gathered vocabulary shards
// [shard][row][vocab_per_shard]; token index = shard * vocab_per_shard + i.
__global__ void argmax_advance_kernel(const __half *__restrict__ logits, int vocab, int shards, int rows,
                                      int *__restrict__ next_ids, int *__restrict__ ids,
                                      int *__restrict__ positions, int advance, HostReport hr) {
    __shared__ float sv[32];
    __shared__ int si[32];
    tlc_pdl_prologue();  // the logits come from the previous kernel
    const int b = blockIdx.x;
    float best = -INFINITY;
    int bi = -1;
    for (int sh = 0; sh < shards; sh++) {
        const __half *row = logits + ((size_t)sh * rows + b) * vocab;
        if (vocab % 8 == 0 && (reinterpret_cast<uintptr_t>(row) & 15) == 0) {
            // 16-byte loads; a thread still meets its elements in increasing index order
            for (int c = threadIdx.x; c < vocab / 8; c += blockDim.x) {
                const uint4 raw = *reinterpret_cast<const uint4 *>(row + 8 * c);
                const __half *h = reinterpret_cast<const __half *>(&raw);
#pragma unroll
                for (int j = 0; j < 8; j++) {
                    const float v = __half2float(h[j]);
                    if (bi < 0 || !(v < best)) {
                        best = v;
                        bi = sh * vocab + 8 * c + j;
                    }
                }
            }
            continue;
        }
        for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
            const float v = __half2float(row[i]);
            if (bi < 0 || !(v < best)) {  // v >= best (or unordered): later index wins
                best = v;
                bi = sh * vocab + i;
            }
        }
    }
    auto better = [](float v, int i, float bv, int bidx) {
        if (bidx < 0) return true;
        if (i < 0) return false;
        if (v > bv) return true;
        if (v < bv) return false;
        return i > bidx;
    };
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (better(ov, oi, best, bi)) {
            best = ov;
            bi = oi;
        }
    }
    if ((threadIdx.x & 31) == 0) {
        sv[threadIdx.x >> 5] = best;
        si[threadIdx.x >> 5] = bi;
    }
    __syncthreads();
    if (threadIdx.x < 32) {
        const int nw = blockDim.x >> 5;
        best = threadIdx.x < nw ? sv[threadIdx.x] : -INFINITY;
        bi = threadIdx.x < nw ? si[threadIdx.x] : -1;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (better(ov, oi, best, bi)) {
                best = ov;
                bi = oi;
            }
        }
        if (threadIdx.x == 0) {
            next_ids[b] = bi;
            if (advance) {
                ids[b] = bi;
                positions[b] += 1;
            }
            report_to_host(hr, b, bi);
        }
    }
}

}  // namespace

// Uniform draw in [0, 1) with 24 bits, a pure function of (seed, position, sequence).
__host__ __device__ inline float tlc_sample_uniform(uint64_t seed, uint32_t pos, uint32_t seq) {
    const uint64_t r = tlc_mix64(tlc_mix64(seed ^ 0x73616d706c65ull) + ((uint64_t)pos << 20) + seq);
    return (float)(r >> 40) * (1.0f / 16777216.0f);
}

// Temperature sample + step bookkeeping, one CTA per sequence: the arithmetic of
// temperature_sample_cpu (src/interpreter/builtin_sampling.rs:185-217) -- logits
// widened to f32 and divided by the temperature, softmax with the maximum
// subtracted, first index whose running probability sum exceeds the uniform
// draw, the last index if none does -- with the sums formed in parallel: every
// thread owns a contiguous run of the vocabulary, a block-wide scan gives each
// run its starting sum, and the comparison is made against u * total instead of
// dividing every probability (the f32 rounding differs from the sequential sum
// only for draws within ~1e-6 of a boundary).
// u comes from `uniforms[b]` when given, else from tlc_sample_uniform.
__global__ void __launch_bounds__(1024) sample_advance_kernel(const __half *__restrict__ logits, int vocab, int shards,
                                                              int rows, float temperature, uint64_t seed,
                                                              const float *__restrict__ uniforms, int fixed_pos,
                                                              int *__restrict__ next_ids, int *__restrict__ ids,
                                                              int *__restrict__ positions, int advance, HostReport hr) {
    __shared__ float red[32];
    __shared__ float warp_sum[32];
    __shared__ int found_min;
    tlc_pdl_prologue();  // the logits come from the previous kernel
    const int b = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int V = vocab * shards;
    const int seg = (V + (int)blockDim.x - 1) / (int)blockDim.x;
    const int lo = min(V, tid * seg), hi = min(V, lo + seg);
    auto logit = [&](int j) {  // token j of the gathered shards
        const int sh = j / vocab, i = j - sh * vocab;
        return __half2float(logits[((size_t)sh * rows + b) * vocab + i]) / temperature;
    };
    float mx = -INFINITY;
    for (int j = lo; j < hi; j++) mx = fmaxf(mx, logit(j));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    if (lane == 0) red[warp] = mx;
    if (tid == 0) found_min = V - 1;  // "default to last token"
    __syncthreads();
    mx = red[lane];  // blockDim.x == 1024: 32 warps
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    float local = 0.f;
    for (int j = lo; j < hi; j++) local += expf(logit(j) - mx);
    // inclusive scan of the per-thread sums: within the warp, then across warps
    float incl = local;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const float t = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += t;
    }
    if (lane == 31) warp_sum[warp] = incl;
    __syncthreads();
    float wbase = 0.f, total = 0.f;
    {
        float w = warp_sum[lane], wi = w;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const float t = __shfl_up_sync(0xffffffffu, wi, o);
            if (lane >= o) wi += t;
        }
        total = __shfl_sync(0xffffffffu, wi, 31);
        wbase = __shfl_sync(0xffffffffu, wi - w, warp);  // exclusive sum of the warps before this one
    }
    const int pos = fixed_pos >= 0 ? fixed_pos : positions ? positions[b] : 0;  // position of the token fed to this step
    const float u = uniforms ? uniforms[b] : tlc_sample_uniform(seed, (uint32_t)pos, (uint32_t)b);
    const float target = u * total;
    float run = wbase + incl - local;  // sum of everything before this thread's run
    if (target < run + local) {
        for (int j = lo; j < hi; j++) {
            run += expf(logit(j) - mx);
            if (target < run) {
                atomicMin(&found_min, j);
                break;
            }
        }
    }
    __syncthreads();
    if (tid == 0) {
        const int tok = found_min;
        next_ids[b] = tok;
        if (advance) {
            ids[b] = tok;
            positions[b] += 1;
        }
        report_to_host(hr, b, tok);
    }
}

namespace {

int32_t get(tlc_model *m, const std::string &name, tlc_qtensor **out) { return tlc_model_get(m, name.c_str(), out); }

}  // namespace

// Decides whether single-sequence greedy decode steps of this model can run as the
// persistent step kernel, and if so builds its device-side tables.
static int32_t step_setup(tlc_llama *L) {
    const tlc_llama_config &c = L->cfg;
    L->step_ok = false;
    if (c.tp_size != 1) return TLC_OK;
    const int qt = L->out_w->type;
    if (qt != TLC_TYPE_Q4_0 && qt != TLC_TYPE_Q8_0) return TLC_OK;
    for (const LayerWeights &w : L->layers)
        for (const tlc_qtensor *t : {w.wq, w.wk, w.wv, w.wo, w.w_gate, w.w_up, w.w_down})
            if (t->type != qt) return TLC_OK;
    const int gq = c.n_heads / c.n_kv_heads;
    if (gq != 1 && gq != 2 && gq != 4 && gq != 8 && gq != 16) return TLC_OK;
    const int qd = c.n_heads * c.head_dim;
    int kmax = c.d_model > qd ? c.d_model : qd;
    kmax = kmax > c.ffn_dim ? kmax : c.ffn_dim;
    if (qd % 32 != 0 || c.ffn_dim % 32 != 0 || (c.n_kv_heads * c.head_dim) % 16 != 0) return TLC_OK;
    int grid = 0;
    if (!tlc_step::step_supported(L->ctx, qt, c.d_model, kmax, c.head_dim, &grid)) return TLC_OK;
    if (grid < c.n_kv_heads) return TLC_OK;
    const int splits = tlc_step::step_max_splits(grid, c.n_heads, c.n_kv_heads);
    L->step_wsl = tlc_step::step_workspace(c.d_model, qd, c.n_kv_heads * c.head_dim, c.ffn_dim, c.n_heads, c.head_dim,
                                           splits, grid);
    cudaError_t e = cudaMalloc(&L->step_ws, L->step_wsl.total);
    if (e == cudaSuccess) e = cudaMemset(L->step_ws, 0, L->step_wsl.total);
    if (e == cudaSuccess) e = cudaMalloc(&L->step_layers, sizeof(tlc_step::StepLayer) * (size_t)c.n_layers);
    if (e != cudaSuccess) {
        cudaGetLastError();
        return tlc_fail(TLC_ERR_ALLOCATION, "decode step workspace failed: %s", cudaGetErrorString(e));
    }
    std::vector<tlc_step::StepLayer> host((size_t)c.n_layers);
    for (int l = 0; l < c.n_layers; l++) {
        const LayerWeights &w = L->layers[(size_t)l];
        void *kc = nullptr, *vc = nullptr;
        tlc_kvcache_layer_ptrs(L->cache, l, &kc, &vc);
        auto u8 = [](const tlc_qtensor *t) { return static_cast<const uint8_t *>(t->data); };
        host[(size_t)l] = {u8(w.wq), u8(w.wk), u8(w.wv), u8(w.wo), u8(w.w_gate), u8(w.w_up), u8(w.w_down),
                           static_cast<const __half *>(w.attn_norm->data), static_cast<const __half *>(w.ffn_norm->data),
                           static_cast<__half *>(kc), static_cast<__half *>(vc)};
    }
    TLC_CUDA(cudaMemcpy(L->step_layers, host.data(), sizeof(tlc_step::StepLayer) * host.size(), cudaMemcpyHostToDevice));
    L->step_ok = true;
    L->step_grid = grid;
    L->step_qtype = qt;
    L->step_kmax = kmax;
    L->step_splits = splits;
    return TLC_OK;
}

static bool step_usable(const tlc_llama *L, int batch) {
    return L->step_ok && L->ctx->step_kernel && batch == 1 && !(L->temperature > 0.0001f);
}

// Launches `steps` decode steps of sequence 0 as one persistent kernel.  ids_src: where the
// first step reads its token (pinned host memory) or null for L->ids; host_next /
// host_status: pinned words the last step reports to, or null.
static int32_t step_launch(tlc_llama *L, int steps, const int *ids_src, int *host_next, tlc_dev_status *host_status,
                           uint64_t *trace = nullptr) {
    const tlc_llama_config &c = L->cfg;
    tlc_step::StepParams p{};
    p.layers = L->step_layers;
    p.n_layers = c.n_layers;
    p.d = c.d_model;
    p.qd = c.n_heads * c.head_dim;
    p.kvd = c.n_kv_heads * c.head_dim;
    p.ffn = c.ffn_dim;
    p.vocab = c.vocab;
    p.H = c.n_heads;
    p.Hkv = c.n_kv_heads;
    p.D = c.head_dim;
    p.Tmax = c.max_seq;
    p.eps = c.rms_eps;
    p.rope_base = (float)c.rope_base;
    p.attn_scale = 1.0f / sqrtf((float)c.head_dim);
    p.w_out = static_cast<const uint8_t *>(L->out_w->data);
    p.out_norm = static_cast<const __half *>(L->out_norm->data);
    p.embd = static_cast<const uint8_t *>(L->tok_embd->data);
    p.embd_pitch = L->tok_embd->row_pitch;
    p.logits = L->logits;
    const tlc_step::StepWorkspace &w = L->step_wsl;
    p.x_w = reinterpret_cast<uint2 *>(L->step_ws + w.x);
    p.x1_w = reinterpret_cast<uint2 *>(L->step_ws + w.x1);
    p.q_w = reinterpret_cast<uint2 *>(L->step_ws + w.q);
    p.kv_w = reinterpret_cast<uint2 *>(L->step_ws + w.kv);
    p.attn_w = reinterpret_cast<uint2 *>(L->step_ws + w.attn);
    p.act_w = reinterpret_cast<uint2 *>(L->step_ws + w.act);
    p.part_w = reinterpret_cast<uint2 *>(L->step_ws + w.part);
    p.cand_w = reinterpret_cast<uint4 *>(L->step_ws + w.cand);
    p.tok_w = reinterpret_cast<uint2 *>(L->step_ws + w.tok);
    p.max_splits = L->step_splits;
    p.trace = trace;
    // Epochs grow from launch to launch; before the 32-bit counter wraps the flagged words
    // are cleared and counting starts again.
    const uint64_t need = (uint64_t)steps * tlc_step::epochs_per_step(c.n_layers);
    if ((uint64_t)L->step_epoch + need >= 0xfffffff0ull) {
        TLC_CUDA(cudaMemsetAsync(L->step_ws, 0, L->step_wsl.total, L->ctx->stream));
        L->step_epoch = 1;
    }
    p.epoch_base = L->step_epoch;
    L->step_epoch += (uint32_t)need;
    p.ids = L->ids;
    p.positions = L->positions;
    p.next_ids = L->next_ids;
    p.ids_src = ids_src;
    p.host_next = host_next;
    p.host_status = host_status;
    p.steps = steps;
    L->last_logit_rows = 1;
    return tlc_step::step_launch(L->ctx, L->step_qtype, L->step_grid, L->step_kmax, p);
}

extern "C" int32_t tlc_llama_create(tlc_ctx *ctx, tlc_model *model, const tlc_llama_config *cfg, tlc_llama **out) {
    if (int32_t rc = tlc_enter(ctx)) return rc;
    TLC_REQUIRE(model && cfg && out, TLC_ERR_INVALID_OPERATION, "llama_create: null pointer");
    *out = nullptr;
    const tlc_llama_config &c = *cfg;
    TLC_REQUIRE(c.n_layers > 0 && c.d_model > 0 && c.n_heads > 0 && c.n_kv_heads > 0 && c.head_dim > 0 &&
                    c.ffn_dim > 0 && c.vocab > 0 && c.max_seq > 0 && c.max_batch > 0 && c.max_batch <= 64,
                TLC_ERR_INVALID_DIMENSION, "llama_create: bad configuration");
    const int tp = c.tp_size < 1 ? 1 : c.tp_size;
    TLC_REQUIRE(c.n_heads % c.n_kv_heads == 0 && c.n_heads % tp == 0 && c.n_kv_heads % tp == 0 && c.ffn_dim % tp == 0,
                TLC_ERR_SHAPE_MISMATCH, "heads %d / kv heads %d / ffn %d do not divide over %d ranks", c.n_heads,
                c.n_kv_heads, c.ffn_dim, tp);
    std::unique_ptr<tlc_llama> L(new tlc_llama());
    L->ctx = ctx;
    L->cfg = c;
    L->cfg.tp_size = tp;
    L->heads_local = c.n_heads / tp;
    L->kv_heads_local = c.n_kv_heads / tp;
    L->ffn_local = c.ffn_dim / tp;
    L->layers.resize(c.n_layers);
    L->pos_hi.assign(64, 0);
    auto expect = [&](tlc_qtensor *t, int64_t rows, int64_t cols, const std::string &name) -> int32_t {
        TLC_REQUIRE(t->n_rows == rows && t->n_cols == cols, TLC_ERR_SHAPE_MISMATCH,
                    "tensor '%s' is [%lld, %lld], expected [%lld, %lld]", name.c_str(), (long long)t->n_rows,
                    (long long)t->n_cols, (long long)rows, (long long)cols);
        return TLC_OK;
    };
    const int64_t d = c.d_model, qd = (int64_t)L->heads_local * c.head_dim, kvd = (int64_t)L->kv_heads_local * c.head_dim;
    for (int l = 0; l < c.n_layers; l++) {
        const std::string p = "blk." + std::to_string(l) + ".";
        LayerWeights &w = L->layers[l];
        struct { tlc_qtensor **t; const char *n; int64_t r, cc; } want[] = {
            {&w.attn_norm, "attn_norm.weight", 1, d},   {&w.wq, "attn_q.weight", qd, d},
            {&w.wk, "attn_k.weight", kvd, d},           {&w.wv, "attn_v.weight", kvd, d},
            {&w.wo, "attn_output.weight", d, qd},       {&w.ffn_norm, "ffn_norm.weight", 1, d},
            {&w.w_gate, "ffn_gate.weight", L->ffn_local, d}, {&w.w_up, "ffn_up.weight", L->ffn_local, d},
            {&w.w_down, "ffn_down.weight", d, L->ffn_local}};
        for (auto &e : want) {
            if (int32_t rc = get(model, p + e.n, e.t)) return rc;
            if (int32_t rc = expect(*e.t, e.r, e.cc, p + e.n)) return rc;
        }
        TLC_REQUIRE(w.attn_norm->type == TLC_TYPE_F16 && w.ffn_norm->type == TLC_TYPE_F16, TLC_ERR_LOAD,
                    "norm weights of layer %d must be f16/f32", l);
    }
    if (int32_t rc = get(model, "token_embd.weight", &L->tok_embd)) return rc;
    if (int32_t rc = get(model, "output_norm.weight", &L->out_norm)) return rc;
    if (int32_t rc = get(model, "output.weight", &L->out_w)) return rc;
    TLC_REQUIRE(L->tok_embd->type == TLC_TYPE_F16 && L->tok_embd->n_cols == d && d % 8 == 0, TLC_ERR_LOAD,
                "token_embd.weight must be f16 [vocab, %lld]", (long long)d);
    TLC_REQUIRE(c.vocab % tp == 0, TLC_ERR_SHAPE_MISMATCH, "vocab %d does not divide over %d ranks", c.vocab, tp);
    L->vocab_local = c.vocab / tp;
    if (int32_t rc = expect(L->out_w, L->vocab_local, d, "output.weight")) return rc;
    if (int32_t rc = expect(L->out_norm, 1, d, "output_norm.weight")) return rc;

    if (int32_t rc = tlc_kvcache_create(ctx, c.n_layers, c.max_batch, c.max_seq, L->kv_heads_local, c.head_dim, &L->cache))
        return rc;
    L->max_rows = c.max_prefill > c.max_batch ? c.max_prefill : c.max_batch;
    if (L->max_rows < 16) L->max_rows = 16;
    const size_t R = (size_t)L->max_rows;
    const size_t logits_rows = (size_t)(c.max_batch > 1 ? c.max_batch : 1);
    struct { void **p; size_t bytes; } bufs[] = {
        {(void **)&L->x, R * d * 2},      {(void **)&L->x1, R * d * 2},          {(void **)&L->q, R * qd * 2},
        {(void **)&L->attn, R * qd * 2},  {(void **)&L->act, R * L->ffn_local * 2},
        {(void **)&L->logits, (c.logits_all_rows ? R : logits_rows) * L->vocab_local * 2},
        {(void **)&L->ids, R * 4},        {(void **)&L->positions, 64 * 4},      {(void **)&L->next_ids, 64 * 4},
        {(void **)&L->part, tp > 1 ? R * d * 2 : 0},
        {(void **)&L->logits_full, tp > 1 ? (c.logits_all_rows ? R : logits_rows) * (size_t)c.vocab * 2 : 0}};
    for (auto &b : bufs) {
        if (b.bytes == 0) continue;
        cudaError_t e = cudaMalloc(b.p, b.bytes);
        if (e != cudaSuccess) {
            cudaGetLastError();
            return tlc_fail(TLC_ERR_ALLOCATION, "activation buffer of %zu bytes failed: %s", b.bytes, cudaGetErrorString(e));
        }
    }
    // The tensor-core path of the linears (many rows) works through scratch;
    // reserve it now so that no allocation happens inside a graph capture.
    {
        const int64_t kmax = d > qd ? d : qd;
        {
            const int64_t shapes[][2] = {{d, qd + 2 * kvd}, {qd, d}, {d, 2 * (int64_t)L->ffn_local}, {L->ffn_local, d},
                                         {d, L->vocab_local}};
            size_t need = tlc_gemm_scratch_bytes(ctx, L->max_rows, kmax, 0);
            for (auto &sh : shapes) {
                const size_t b = tlc_gemm_scratch_bytes(ctx, L->max_rows, sh[0], sh[1]);
                need = b > need ? b : need;
            }
            if (int32_t rc = tlc_scratch_reserve(ctx, need)) return rc;
        }
        // ... and the split-K partial sums of the batched decode GEMVs
        const int qt0 = L->layers[0].wq->type;
        size_t need = 0;
        for (int m = 2; m <= c.max_batch && m <= 16; m++) {
            const size_t cand[] = {tlc_gemv_scratch_bytes(ctx, qt0, d, m, qd + 2 * kvd), tlc_gemv_scratch_bytes(ctx, qt0, qd, m, d),
                                   tlc_gemv_scratch_bytes(ctx, qt0, d, m, 2 * (int64_t)L->ffn_local),
                                   tlc_gemv_scratch_bytes(ctx, qt0, L->ffn_local, m, d),
                                   tlc_gemv_scratch_bytes(ctx, L->out_w->type, d, m, L->vocab_local)};
            for (size_t b : cand) need = b > need ? b : need;
        }
        if (int32_t rc = tlc_scratch_reserve(ctx, need)) return rc;
    }
    // Same shared-memory carve-out as the GEMV and attention kernels they run between.
    TLC_CUDA(cudaFuncSetAttribute(embed_kernel, cudaFuncAttributePreferredSharedMemoryCarveout,
                                  cudaSharedmemCarveoutMaxShared));
    TLC_CUDA(cudaFuncSetAttribute(argmax_advance_kernel, cudaFuncAttributePreferredSharedMemoryCarveout,
                                  cudaSharedmemCarveoutMaxShared));
    TLC_CUDA(cudaMemsetAsync(L->positions, 0, 64 * 4, ctx->stream));
    if (int32_t rc = step_setup(L.get())) return rc;
    TLC_CUDA(cudaMallocHost(&L->host_ids, R * 4));
    TLC_CUDA(cudaMallocHost(&L->host_next, 64 * 4));
    *out = L.release();
    return TLC_OK;
}

extern "C" int32_t tlc_llama_destroy(tlc_llama *L) {
    if (!L) return TLC_OK;
    cudaSetDevice(L->ctx->device);
    cudaStreamSynchronize(L->ctx->stream);
    for (auto &g : L->graph)
        if (g.second) cudaGraphExecDestroy(g.second);
    tlc_kvcache_destroy(L->cache);
    void *bufs[] = {L->x, L->x1, L->q, L->attn, L->act, L->logits, L->ids, L->positions, L->next_ids,
                    L->part, L->logits_full, L->step_ws, L->step_layers, L->step_trace};
    for (void *b : bufs) cudaFree(b);
    cudaFreeHost(L->host_ids);
    cudaFreeHost(L->host_next);
    delete L;
    return TLC_OK;
}

// Enqueues one forward pass over m activation rows whose token ids are already
// in L->ids.  decode == false: the rows are consecutive tokens of sequence 0
// starting at pos0 (prefill).  decode == true: row r is the next token of
// sequence r at L->positions[r].
// `parts` selects which launches are issued (1: the quantized linears, 2: the
// attention, 4: embedding gather and sampling); 7 is the whole step.
static int32_t forward(tlc_llama *L, int m, bool decode, int pos0, bool all_logits, bool sample, bool advance,
                       int parts = 7) {
    tlc_ctx *ctx = L->ctx;
    const tlc_llama_config &c = L->cfg;
    const bool tp = c.tp_size > 1;
    TLC_REQUIRE(!tp || L->comm, TLC_ERR_COMM, "tensor-parallel model (tp_size = %d) has no communicator: call "
                "tlc_llama_set_comm first", c.tp_size);
    const int d = c.d_model, D = c.head_dim;
    const int64_t kv_row = (int64_t)L->kv_heads_local * D;
    if (parts & 4) {
        const size_t total = (size_t)m * (d / 8);
        cudaError_t le = tlc_launch_pdl(ctx, embed_kernel, dim3((unsigned)((total + 255) / 256)), dim3(256), 0,
                                        static_cast<const uint8_t *>(L->tok_embd->data), L->tok_embd->row_pitch,
                                        (int)L->tok_embd->n_rows, d, L->ids_src ? L->ids_src : (const int *)L->ids, m, L->x);
        if (le != cudaSuccess) return tlc_fail(TLC_ERR_CUDA, "embedding launch failed: %s", cudaGetErrorString(le));
        TLC_CHECK_LAUNCH(ctx);
    }
    const int *positions = decode ? L->positions : nullptr;
    const float scale = 1.0f / sqrtf((float)D);
    for (int l = 0; l < c.n_layers; l++) {
        const LayerWeights &w = L->layers[l];
        void *kc = nullptr, *vc = nullptr;
        tlc_kvcache_layer_ptrs(L->cache, l, &kc, &vc);
        if (parts & 1) {
            tlc_gemv_args a;
            a.n_out = 3;
            a.outs[0] = {w.wq, L->q, L->heads_local};
            a.outs[1] = {w.wk, kc, L->kv_heads_local};
            a.outs[2] = {w.wv, vc, 0};
            for (int i = 1; i < 3; i++) {
                a.outs[i].row_stride = decode ? (int64_t)c.max_seq * kv_row : 0;
                a.outs[i].pos_stride = kv_row;
            }
            a.x = L->x;
            a.m = m;
            a.norm_w = w.attn_norm->data;
            a.eps = c.rms_eps;
            a.pos_offset = pos0;
            a.rope_base = c.rope_base;
            a.positions = positions;
            a.max_pos = c.max_seq;  // second line of defence behind the host-side bound (pos_hi)
            if (int32_t rc = tlc_launch_gemv(ctx, a)) return rc;
        }
        if (parts & 2)
            // positions[] is written by the previous step's sampling kernel (or by set_state / prefill);
            // the embedding gather and the q/k/v kernels lie between it and this launch.  The q/k/v GEMV
            // lets its successor in only after its own dependency wait (pdl_mode 2 and up), and the
            // q/k/v GEMM of 17 rows and more comes behind a plain-launched RMSNorm: either way the
            // positions are final before this kernel can be scheduled
            if (int32_t rc = tlc_launch_attention(ctx, L->cache, l, L->q, L->attn, decode ? m : 1, decode ? 1 : m,
                                                  L->heads_local, pos0, positions, c.max_seq, scale,
                                                  !ctx->use_pdl || ctx->pdl_mode >= 2))
                return rc;
        if (parts & 1) {
            tlc_gemv_args a;
            a.n_out = 1;
            a.outs[0] = {w.wo, tp ? L->part : L->x1, 0};
            a.x = L->attn;
            a.m = m;
            if (!tp) {
                a.epilogue = TLC_EPI_RESIDUAL;
                a.residual = L->x;
            }
            if (int32_t rc = tlc_launch_gemv(ctx, a)) return rc;
            if (tp) {
                // Row-parallel projection: sum the ranks' partial products, then the residual add.
                if (int32_t rc = tlc_allreduce_residual_f16(ctx, L->comm, L->part, L->x, L->x1, (size_t)m * d)) return rc;
            }
        }
        if (parts & 1) {
            tlc_gemv_args a;
            a.n_out = 2;
            a.outs[0] = {w.w_gate, L->act, 0};
            a.outs[1] = {w.w_up, L->act, 0};
            a.x = L->x1;
            a.m = m;
            a.norm_w = w.ffn_norm->data;
            a.eps = c.rms_eps;
            a.epilogue = TLC_EPI_SWIGLU;
            if (int32_t rc = tlc_launch_gemv(ctx, a)) return rc;
        }
        if (parts & 1) {
            tlc_gemv_args a;
            a.n_out = 1;
            a.outs[0] = {w.w_down, tp ? L->part : L->x, 0};
            a.x = L->act;
            a.m = m;
            if (!tp) {
                a.epilogue = TLC_EPI_RESIDUAL;
                a.residual = L->x1;
            }
            if (int32_t rc = tlc_launch_gemv(ctx, a)) return rc;
            if (tp) {
                if (int32_t rc = tlc_allreduce_residual_f16(ctx, L->comm, L->part, L->x1, L->x, (size_t)m * d)) return rc;
            }
        }
    }
    {
        // Logits: every row for a batched decode step, otherwise only the last
        // prompt token (all rows on request, for parity checks).
        const int rows = (decode || all_logits) ? m : 1;
        tlc_gemv_args a;
        a.n_out = 1;
        a.outs[0] = {L->out_w, L->logits, 0};
        a.x = L->x + (size_t)(m - rows) * d;
        a.m = rows;
        a.norm_w = L->out_norm->data;
        a.eps = c.rms_eps;
        if (parts & 1) {
            if (int32_t rc = tlc_launch_gemv(ctx, a)) return rc;
            // Column-parallel lm_head: gather the vocabulary shards [rank][rows][vocab / tp].
            if (tp)
                if (int32_t rc = tlc_allgather_f16(ctx, L->comm, L->logits, L->logits_full, (size_t)rows * L->vocab_local))
                    return rc;
        }
        L->last_logit_rows = rows;
        if (sample && (parts & 4)) {
            const int srows = decode ? m : 1;
            const __half *lg = (tp ? L->logits_full : L->logits) + (size_t)(rows - srows) * L->vocab_local;
            cudaError_t le =
                L->temperature > 0.0001f
                    ? tlc_launch_pdl(ctx, sample_advance_kernel, dim3(srows), dim3(1024), 0, lg, L->vocab_local,
                                     c.tp_size, rows, L->temperature, L->sample_seed, (const float *)nullptr,
                                     decode ? -1 : pos0 + m - 1, (int *)L->next_ids, (int *)L->ids, (int *)L->positions, advance ? 1 : 0,
                                     L->report)
                    : tlc_launch_pdl(ctx, argmax_advance_kernel, dim3(srows), dim3(1024), 0, lg, L->vocab_local,
                                     c.tp_size, rows, (int *)L->next_ids, (int *)L->ids, (int *)L->positions,
                                     advance ? 1 : 0, L->report);
            if (le != cudaSuccess) return tlc_fail(TLC_ERR_CUDA, "sampling launch failed: %s", cudaGetErrorString(le));
            TLC_CHECK_LAUNCH(ctx);
        }
    }
    return TLC_OK;
}

// Enqueues the copy of the last forward's logits to host memory as [rows, vocab]
// (with tensor parallelism the gathered shards are interleaved into full rows).
static int32_t copy_logits(tlc_llama *L, void *logits_host, int rows) {
    const size_t vl = (size_t)L->vocab_local;
    if (L->cfg.tp_size == 1) {
        TLC_CUDA(cudaMemcpyAsync(logits_host, L->logits, (size_t)rows * vl * 2, cudaMemcpyDeviceToHost, L->ctx->stream));
        return TLC_OK;
    }
    const size_t vocab = (size_t)L->cfg.vocab;
    for (int r = 0; r < L->cfg.tp_size; r++)
        TLC_CUDA(cudaMemcpy2DAsync(static_cast<char *>(logits_host) + r * vl * 2, vocab * 2,
                                   L->logits_full + (size_t)r * rows * vl, vl * 2, vl * 2, (size_t)rows,
                                   cudaMemcpyDeviceToHost, L->ctx->stream));
    return TLC_OK;
}

// Tensor parallelism: the communicator that joins this rank's runner to the
// others (tlc_comm_init).  Must be set before the first prefill / decode.
extern "C" int32_t tlc_llama_set_comm(tlc_llama *L, tlc_comm *comm) {
    TLC_REQUIRE(L && comm, TLC_ERR_INVALID_OPERATION, "llama_set_comm: null pointer");
    TLC_REQUIRE(tlc_comm_size(comm) == L->cfg.tp_size && tlc_comm_rank(comm) == L->cfg.tp_rank, TLC_ERR_COMM,
                "communicator is rank %d of %d, the model is shard %d of %d", tlc_comm_rank(comm), tlc_comm_size(comm),
                L->cfg.tp_rank, L->cfg.tp_size);
    L->comm = comm;
    return TLC_OK;
}

static int32_t check_ids(const tlc_llama *L, const int32_t *ids, int n) {
    for (int i = 0; i < n; i++)
        TLC_REQUIRE(ids[i] >= 0 && ids[i] < L->cfg.vocab, TLC_ERR_INDEX, "Index out of bounds: index %d, size %d",
                    ids[i], L->cfg.vocab);
    return TLC_OK;
}

extern "C" int32_t tlc_llama_prefill(tlc_llama *L, const int32_t *ids_host, int32_t n, int32_t pos0,
                                     void *logits_host, int32_t all_rows, int32_t *next_id_host) {
    TLC_REQUIRE(L && ids_host, TLC_ERR_INVALID_OPERATION, "llama_prefill: null pointer");
    if (int32_t rc = tlc_enter(L->ctx)) return rc;
    tlc_perf_scope perf(L->ctx, "llama_prefill(tokens=%d)", n);
    TLC_REQUIRE(n >= 1 && n <= L->max_rows, TLC_ERR_SHAPE_MISMATCH, "prefill of %d tokens (buffers hold %d)", n,
                L->max_rows);
    TLC_REQUIRE(pos0 >= 0 && pos0 + n <= L->cfg.max_seq, TLC_ERR_INDEX, "Index out of bounds: index %d, size %d",
                pos0 + n, L->cfg.max_seq);
    TLC_REQUIRE(!all_rows || L->cfg.logits_all_rows, TLC_ERR_INVALID_OPERATION,
                "all-row logits need logits_all_rows in the configuration");
    if (int32_t rc = check_ids(L, ids_host, n)) return rc;
    memcpy(L->host_ids, ids_host, (size_t)n * 4);
    TLC_CUDA(cudaMemcpyAsync(L->ids, L->host_ids, (size_t)n * 4, cudaMemcpyHostToDevice, L->ctx->stream));
    if (int32_t rc = forward(L, n, false, pos0, all_rows != 0, true, false)) return rc;
    // Sequence 0 continues after the prompt with the sampled token.
    const int32_t next_pos = pos0 + n;
    L->pos_hi[0] = next_pos;
    L->host_next[32] = next_pos;
    TLC_CUDA(cudaMemcpyAsync(L->positions, &L->host_next[32], 4, cudaMemcpyHostToDevice, L->ctx->stream));
    TLC_CUDA(cudaMemcpyAsync(L->ids, L->next_ids, 4, cudaMemcpyDeviceToDevice, L->ctx->stream));
    const int rows = all_rows ? n : 1;
    if (logits_host)
        if (int32_t rc = copy_logits(L, logits_host, rows)) return rc;
    TLC_CUDA(cudaMemcpyAsync(L->host_next, L->next_ids, 4, cudaMemcpyDeviceToHost, L->ctx->stream));
    if (int32_t rc = tlc_synchronize(L->ctx)) return rc;
    if (next_id_host) *next_id_host = L->host_next[0];
    return TLC_OK;
}

extern "C" int32_t tlc_llama_set_state(tlc_llama *L, int32_t batch, const int32_t *ids_host,
                                       const int32_t *positions_host) {
    TLC_REQUIRE(L && ids_host && positions_host, TLC_ERR_INVALID_OPERATION, "llama_set_state: null pointer");
    if (int32_t rc = tlc_enter(L->ctx)) return rc;
    TLC_REQUIRE(batch >= 1 && batch <= L->cfg.max_batch, TLC_ERR_SHAPE_MISMATCH, "batch %d (max %d)", batch,
                L->cfg.max_batch);
    if (int32_t rc = check_ids(L, ids_host, batch)) return rc;
    for (int i = 0; i < batch; i++)
        TLC_REQUIRE(positions_host[i] >= 0 && positions_host[i] < L->cfg.max_seq, TLC_ERR_INDEX,
                    "Index out of bounds: index %d, size %d", positions_host[i], L->cfg.max_seq);
    TLC_CUDA(cudaStreamSynchronize(L->ctx->stream));  // earlier steps may still read ids/positions
    TLC_CUDA(cudaMemcpy(L->ids, ids_host, (size_t)batch * 4, cudaMemcpyHostToDevice));
    TLC_CUDA(cudaMemcpy(L->positions, positions_host, (size_t)batch * 4, cudaMemcpyHostToDevice));
    for (int i = 0; i < batch; i++) L->pos_hi[i] = positions_host[i];
    return TLC_OK;
}

// A decode step at position p writes cache row p: `steps` more steps need
// p + steps <= max_seq for every sequence of the batch.  The reference's cache.append
// concatenates and cannot overflow; a pre-allocated cache has to refuse instead.
static int32_t reserve_positions(tlc_llama *L, int batch, int steps) {
    int hi = 0;
    for (int i = 0; i < batch; i++) hi = L->pos_hi[i] > hi ? L->pos_hi[i] : hi;
    TLC_REQUIRE((int64_t)hi + steps <= L->cfg.max_seq, TLC_ERR_INDEX, "Index out of bounds: index %d, size %d",
                hi + steps, L->cfg.max_seq);
    for (int i = 0; i < batch; i++) L->pos_hi[i] += steps;
    return TLC_OK;
}

// Enqueues `steps` greedy decode steps for `batch` sequences (graph replay);
// nothing is read back.  parts != 7 replays only some of the step's launches
// (for per-kernel timing) and leaves tokens and positions untouched.
static int32_t decode_enqueue(tlc_llama *L, int32_t batch, int32_t steps, int parts) {
    TLC_REQUIRE(L, TLC_ERR_INVALID_OPERATION, "llama_decode: null handle");
    if (int32_t rc = tlc_enter(L->ctx)) return rc;
    TLC_REQUIRE(batch >= 1 && batch <= L->cfg.max_batch, TLC_ERR_SHAPE_MISMATCH, "batch %d (max %d)", batch,
                L->cfg.max_batch);
    TLC_REQUIRE(parts >= 1 && parts <= 7, TLC_ERR_INVALID_OPERATION, "decode parts mask %d", parts);
    TLC_REQUIRE(steps >= 0, TLC_ERR_INVALID_OPERATION, "decode of %d steps", steps);
    tlc_ctx *ctx = L->ctx;
    const bool advance = parts == 7;
    if (advance)
        if (int32_t rc = reserve_positions(L, batch, steps)) return rc;
    if (advance && step_usable(L, batch)) {
        // the whole run of steps is one launch of the persistent kernel
        L->launches_in[7] = 1;
        if (steps == 0) return TLC_OK;
        return step_launch(L, steps, nullptr, nullptr, nullptr);
    }
    const int key = batch * 8 + parts;
    if (!L->graph.count(key) && !L->cfg.no_graph) {
        // Warm every kernel configuration (function attributes, scratch growth)
        // outside the capture, on a throw-away step that does not advance.
        if (int32_t rc = forward(L, batch, true, 0, false, true, false, parts)) return rc;
        TLC_CUDA(cudaStreamSynchronize(ctx->stream));
        const uint64_t launches_before = ctx->launches;
        TLC_CUDA(cudaStreamBeginCapture(ctx->stream, cudaStreamCaptureModeThreadLocal));
        int32_t rc = forward(L, batch, true, 0, false, true, advance, parts);
        cudaGraph_t g = nullptr;
        cudaError_t e = cudaStreamEndCapture(ctx->stream, &g);
        L->launches_in[parts] = (int)(ctx->launches - launches_before);
        ctx->launches = launches_before;
        if (rc) {
            if (g) cudaGraphDestroy(g);
            return rc;
        }
        if (e != cudaSuccess) return tlc_fail(TLC_ERR_CUDA, "graph capture failed: %s", cudaGetErrorString(e));
        cudaGraphExec_t ge = nullptr;
        e = cudaGraphInstantiate(&ge, g, 0);
        cudaGraphDestroy(g);
        if (e != cudaSuccess) return tlc_fail(TLC_ERR_CUDA, "graph instantiate failed: %s", cudaGetErrorString(e));
        L->graph[key] = ge;
    }
    for (int s = 0; s < steps; s++) {
        if (L->cfg.no_graph) {
            const uint64_t before = ctx->launches;
            if (int32_t rc = forward(L, batch, true, 0, false, true, advance, parts)) return rc;
            L->launches_in[parts] = (int)(ctx->launches - before);
        } else {
            TLC_CUDA(cudaGraphLaunch(L->graph[key], ctx->stream));
            ctx->launches += (uint64_t)L->launches_in[parts];
        }
    }
    return TLC_OK;
}

extern "C" int32_t tlc_llama_decode_enqueue(tlc_llama *L, int32_t batch, int32_t steps) {
    return decode_enqueue(L, batch, steps, 7);
}

extern "C" int32_t tlc_llama_decode_enqueue_parts(tlc_llama *L, int32_t batch, int32_t steps, int32_t parts) {
    return decode_enqueue(L, batch, steps, parts);
}

// One decode step through host buffers: uploads the token ids (NULL: continue
// with the tokens sampled by the previous step), runs the step, and returns the
// sampled tokens and, on request, the logits [batch, vocab].
extern "C" int32_t tlc_llama_decode_host(tlc_llama *L, int32_t batch, const int32_t *ids_host,
                                         int32_t *next_ids_host, void *logits_host) {
    TLC_REQUIRE(L && next_ids_host, TLC_ERR_INVALID_OPERATION, "llama_decode_host: null pointer");
    if (int32_t rc = tlc_enter(L->ctx)) return rc;
    tlc_perf_scope perf(L->ctx, "llama_decode(batch=%d)", batch);
    TLC_REQUIRE(batch >= 1 && batch <= L->cfg.max_batch, TLC_ERR_SHAPE_MISMATCH, "batch %d (max %d)", batch,
                L->cfg.max_batch);
    if (ids_host) {
        if (int32_t rc = check_ids(L, ids_host, batch)) return rc;
        memcpy(L->host_ids, ids_host, (size_t)batch * 4);
    }
    if (step_usable(L, batch)) {
        // One launch: the kernel reads the token id from pinned memory and writes the status
        // word, then the sampled id, to pinned memory; the host watches that word.
        tlc_ctx *ctx = L->ctx;
        if (int32_t rc = reserve_positions(L, batch, 1)) return rc;  // before anything is launched
        volatile int32_t *landed = L->host_next;
        landed[0] = -1;  // no token id is negative
        L->launches_in[7] = 1;
        if (int32_t rc = step_launch(L, 1, ids_host ? L->host_ids : nullptr, L->host_next, ctx->host_status)) return rc;
        if (logits_host)
            if (int32_t rc = copy_logits(L, logits_host, batch)) return rc;
        bool seen = false;
        if (ctx->host_poll && !logits_host) {
            const auto t0 = std::chrono::steady_clock::now();
            for (long spin = 0; !seen; spin++) {
                seen = landed[0] >= 0;
                if (!seen && (spin & 1023) == 1023 &&
                    std::chrono::steady_clock::now() - t0 > std::chrono::milliseconds(50))
                    break;
            }
        }
        if (!seen) {
            if (int32_t rc = tlc_synchronize(ctx)) return rc;  // also copies and checks the status word
        } else if (int32_t rc = tlc_status_after_sync(ctx)) {
            return rc;
        }
        next_ids_host[0] = L->host_next[0];
        return TLC_OK;
    }
    if (ids_host && !logits_host && !L->cfg.no_graph && L->ctx->host_graph) {
        // The common call: token ids up, one step, sampled ids and the status word down --
        // all of it one graph (copy nodes around the step's kernels), one launch, one wait.
        tlc_ctx *ctx = L->ctx;
        if (int32_t rc = reserve_positions(L, batch, 1)) return rc;  // before anything is launched
        const int key = 1000 + batch;
        if (!L->graph.count(key)) {
            if (int32_t rc = decode_enqueue(L, batch, 0, 7)) return rc;  // warms the kernels, captures the plain step
            TLC_CUDA(cudaStreamSynchronize(ctx->stream));
            const uint64_t launches_before = ctx->launches;
            TLC_CUDA(cudaStreamBeginCapture(ctx->stream, cudaStreamCaptureModeThreadLocal));
            // No copy nodes: the embedding gather reads the ids from pinned host memory and the
            // sampling kernel writes the status word, then the sampled ids, to pinned host memory.
            cudaError_t ce = cudaSuccess;
            L->ids_src = L->host_ids;
            L->report = HostReport{L->host_next, ctx->host_status, ctx->dev_status};
            int32_t rc = forward(L, batch, true, 0, false, true, true, 7);
            L->ids_src = nullptr;
            L->report = HostReport{};
            cudaGraph_t g = nullptr;
            cudaError_t e = cudaStreamEndCapture(ctx->stream, &g);
            ctx->launches = launches_before;
            if (rc || ce != cudaSuccess || e != cudaSuccess) {
                if (g) cudaGraphDestroy(g);
                cudaGetLastError();
                if (rc) return rc;
                return tlc_fail(TLC_ERR_CUDA, "graph capture of the host step failed: %s",
                                cudaGetErrorString(ce != cudaSuccess ? ce : e));
            }
            cudaGraphExec_t ge = nullptr;
            e = cudaGraphInstantiate(&ge, g, 0);
            cudaGraphDestroy(g);
            if (e != cudaSuccess) return tlc_fail(TLC_ERR_CUDA, "graph instantiate failed: %s", cudaGetErrorString(e));
            L->graph[key] = ge;
        }
        volatile int32_t *landed = L->host_next;
        for (int i = 0; i < batch; i++) landed[i] = -1;  // no token id is negative
        TLC_CUDA(cudaGraphLaunch(L->graph[key], ctx->stream));
        ctx->launches += (uint64_t)L->launches_in[7];
        bool seen = false;
        if (ctx->host_poll) {
            // Watch the pinned words the last copy node writes; after 50 ms without them
            // (an error, a very long step) fall back to the stream synchronize below.
            const auto t0 = std::chrono::steady_clock::now();
            for (long spin = 0; !seen; spin++) {
                seen = true;
                for (int i = 0; i < batch; i++) seen = seen && landed[i] >= 0;
                if (!seen && (spin & 1023) == 1023 &&
                    std::chrono::steady_clock::now() - t0 > std::chrono::milliseconds(50))
                    break;
            }
        }
        if (!seen) TLC_CUDA(cudaStreamSynchronize(ctx->stream));
        if (int32_t rc = tlc_status_after_sync(ctx)) return rc;
        memcpy(next_ids_host, L->host_next, (size_t)batch * 4);
        return TLC_OK;
    }
    if (ids_host)
        TLC_CUDA(cudaMemcpyAsync(L->ids, L->host_ids, (size_t)batch * 4, cudaMemcpyHostToDevice, L->ctx->stream));
    if (int32_t rc = tlc_llama_decode_enqueue(L, batch, 1)) return rc;
    if (logits_host)
        if (int32_t rc = copy_logits(L, logits_host, batch)) return rc;
    TLC_CUDA(cudaMemcpyAsync(L->host_next, L->next_ids, (size_t)batch * 4, cudaMemcpyDeviceToHost, L->ctx->stream));
    if (int32_t rc = tlc_synchronize(L->ctx)) return rc;
    memcpy(next_ids_host, L->host_next, (size_t)batch * 4);
    return TLC_OK;
}

extern "C" int32_t tlc_llama_read_state(tlc_llama *L, int32_t batch, int32_t *next_ids_host,
                                        int32_t *positions_host) {
    TLC_REQUIRE(L, TLC_ERR_INVALID_OPERATION, "llama_read_state: null handle");
    if (int32_t rc = tlc_enter(L->ctx)) return rc;
    TLC_REQUIRE(batch >= 1 && batch <= 64, TLC_ERR_SHAPE_MISMATCH, "batch %d", batch);
    if (next_ids_host) {
        if (int32_t rc = tlc_download(L->ctx, next_ids_host, L->next_ids, (size_t)batch * 4)) return rc;
    }
    if (positions_host) {
        if (int32_t rc = tlc_download(L->ctx, positions_host, L->positions, (size_t)batch * 4)) return rc;
    }
    return TLC_OK;
}

// Sampling of prefill / decode: temperature <= 1e-4 is greedy (the default).
// Otherwise tokens are drawn as temperature_sample does, with uniform draws that
// are a pure function of (seed, position of the sampled token, sequence index):
// a run is reproducible and tensor-parallel ranks draw the same tokens.
extern "C" int32_t tlc_llama_set_sampling(tlc_llama *L, float temperature, uint64_t seed) {
    TLC_REQUIRE(L, TLC_ERR_INVALID_OPERATION, "llama_set_sampling: null pointer");
    TLC_REQUIRE(temperature >= 0.f && temperature == temperature, TLC_ERR_INVALID_OPERATION,
                "temperature must be >= 0 (got %f)", (double)temperature);
    if (int32_t rc = tlc_enter(L->ctx)) return rc;
    TLC_CUDA(cudaStreamSynchronize(L->ctx->stream));
    // captured decode graphs hold the old sampling kernel and its arguments
    for (auto &g : L->graph)
        if (g.second) cudaGraphExecDestroy(g.second);
    L->graph.clear();
    L->temperature = temperature;
    L->sample_seed = seed;
    return TLC_OK;
}

extern "C" float tlc_sample_uniform_host(uint64_t seed, uint32_t position, uint32_t sequence) {
    return tlc_sample_uniform(seed, position, sequence);
}

// temperature_sample(logits, T) as a builtin: logits_dev [rows, vocab] f16, one
// uniform draw per row from the caller (upstream draws rand::thread_rng().gen::<f32>()),
// the sampled ids come back to the host (the builtin returns an Integer).
extern "C" int32_t tlc_temperature_sample(tlc_ctx *ctx, const void *logits_dev, int32_t rows, int32_t vocab,
                                          float temperature, const float *uniforms_host, int32_t *ids_host) {
    if (int32_t rc = tlc_enter(ctx)) return rc;
    TLC_REQUIRE(logits_dev && ids_host && (uniforms_host || temperature <= 0.0001f), TLC_ERR_INVALID_OPERATION,
                "temperature_sample: null pointer");
    TLC_REQUIRE(rows >= 1 && vocab >= 1, TLC_ERR_INVALID_DIMENSION, "temperature_sample: bad shape [%d, %d]", rows, vocab);
    tlc_buf *ub = nullptr, *ib = nullptr;
    int32_t rc = tlc_alloc(ctx, (size_t)rows * 4, &ib);
    if (!rc) rc = tlc_alloc(ctx, (size_t)rows * 4, &ub);
    if (!rc && temperature > 0.0001f) rc = tlc_upload(ctx, tlc_buf_ptr(ub), uniforms_host, (size_t)rows * 4);
    if (!rc) {
        if (temperature > 0.0001f)
            sample_advance_kernel<<<rows, 1024, 0, ctx->stream>>>(
                static_cast<const __half *>(logits_dev), vocab, 1, rows, temperature, 0, (const float *)tlc_buf_ptr(ub),
                -1, (int *)tlc_buf_ptr(ib), nullptr, nullptr, 0, HostReport{});
        else
            argmax_advance_kernel<<<rows, 1024, 0, ctx->stream>>>(static_cast<const __half *>(logits_dev), vocab, 1, rows,
                                                                   (int *)tlc_buf_ptr(ib), nullptr, nullptr, 0, HostReport{});
        ctx->launches++;
        if (cudaGetLastError() != cudaSuccess) rc = tlc_fail(TLC_ERR_CUDA, "sampling launch failed");
    }
    if (!rc) rc = tlc_download(ctx, ids_host, tlc_buf_ptr(ib), (size_t)rows * 4);
    tlc_free(ub);
    tlc_free(ib);
    return rc;
}

extern "C" int32_t tlc_llama_launches_per_step(tlc_llama *L, int32_t parts) {
    return L && parts >= 1 && parts <= 7 ? L->launches_in[parts] : 0;
}
extern "C" tlc_kvcache *tlc_llama_cache(tlc_llama *L) { return L ? L->cache : nullptr; }

// Per-phase timing of the persistent decode step (the counterpart of the per-op timing the
// reference prints under TL_PERF, src/interpreter/builtin_math.rs:190-197): runs `steps`
// decode steps of sequence 0 with CTA 0 recording the device time (ns) at the end of each of
// its phases -- per layer A (norm + q/k/v + rope), B (attention), C (o + residual), D (norm +
// gate/up + SiLU.mul), E (down + residual), then F (norm + lm_head) and G (sample) -- and
// copies the stamps to out_ns as [steps][n_layers * 5 + 2][3]: for each phase the time its input
// was complete in shared memory, the time its dot products were done and the time its outputs
// were stored (phases B and G record only the last).  TLC_ERR_INVALID_OPERATION when the
// model does not run on the persistent kernel.
extern "C" int32_t tlc_llama_step_trace(tlc_llama *L, int32_t steps, uint64_t *out_ns, size_t capacity) {
    TLC_REQUIRE(L && out_ns, TLC_ERR_INVALID_OPERATION, "llama_step_trace: null pointer");
    if (int32_t rc = tlc_enter(L->ctx)) return rc;
    TLC_REQUIRE(step_usable(L, 1), TLC_ERR_INVALID_OPERATION,
                "llama_step_trace: this model / configuration does not run as the persistent step kernel");
    const size_t per_step = ((size_t)L->cfg.n_layers * 5 + 2) * 3, words = per_step * (size_t)steps;
    TLC_REQUIRE(steps >= 1 && capacity >= words, TLC_ERR_SHAPE_MISMATCH, "llama_step_trace: %d steps need %zu words (got %zu)",
                steps, words, capacity);
    if (int32_t rc = reserve_positions(L, 1, steps)) return rc;
    if (L->step_trace_words < words) {
        TLC_CUDA(cudaStreamSynchronize(L->ctx->stream));
        if (L->step_trace) cudaFree(L->step_trace);
        L->step_trace = nullptr;
        L->step_trace_words = 0;
        TLC_CUDA(cudaMalloc(&L->step_trace, words * sizeof(uint64_t)));
        L->step_trace_words = words;
    }
    TLC_CUDA(cudaMemsetAsync(L->step_trace, 0, words * sizeof(uint64_t), L->ctx->stream));
    if (int32_t rc = step_launch(L, steps, nullptr, nullptr, nullptr, L->step_trace)) return rc;
    TLC_CUDA(cudaMemcpyAsync(out_ns, L->step_trace, words * sizeof(uint64_t), cudaMemcpyDeviceToHost, L->ctx->stream));
    return tlc_synchronize(L->ctx);
}
