// Parameters of the persistent decode-step kernel (tlc_step.cu), filled by the LLaMA
// runner (tlc_llama.cu).
#pragma once

#include <cuda_fp16.h>

#include <cstddef>
#include <cstdint>

#include "tlc_internal.h"

namespace tlc_step {

// Device pointers of one layer: tiled quantized weights (tlc_tile.cuh), f16 norm weights,
// this layer's K and V cache [max_seq][kv_heads * head_dim] of sequence 0.
struct StepLayer {
    const uint8_t *wq, *wk, *wv, *wo, *wg, *wu, *wd;
    const __half *attn_norm, *ffn_norm;
    __half *kc, *vc;
};

struct StepParams {
    const StepLayer *layers;  // device array [n_layers]
    int n_layers;
    int d, qd, kvd, ffn, vocab;  // model width, heads*head_dim, kv_heads*head_dim, FFN width, vocabulary
    int H, Hkv, D, Tmax;
    int tb, tile_bytes;  // blocks per weight tile and its bytes (Q4_0: 4 / 1152, Q8_0: 2 / 1088)
    float eps, rope_base, attn_scale;
    const uint8_t *w_out;    // lm_head tiles
    const __half *out_norm;
    const uint8_t *embd;     // f16 embedding table
    size_t embd_pitch;       // bytes per row
    // activations in global memory (they cross the grid barriers)
    __half *x, *x1, *q, *attn, *act, *logits;
    float *part_ml, *part_o;  // split-key partials [H][max_splits][2], [H][max_splits][D]
    int *tickets;             // [Hkv], zero between phases
    int max_splits;
    float *cand_val;          // per-CTA best logit and its index
    int *cand_idx;
    uint32_t *bar_counter;    // monotonic arrival counter of the grid barrier
    uint32_t *bar_base;       // its value at the start of the next launch
    int *ids, *positions, *next_ids;  // device: pending token, its position, sampled token (sequence 0)
    const int *ids_src;       // where the first step reads its token (pinned host memory) or null = ids
    int *host_next;           // pinned host word for the last step's token, or null
    tlc_dev_status *host_status;  // pinned mirror of the status word, written before host_next
    int steps;
    int advance;  // 1: feed the sampled token back and advance the position
    int nstages;
    uint32_t off_xres, off_xin, off_cinit, off_xperm, off_attn, off_ring;
    tlc_dev_status *status;
    uint64_t wait_ns;
};

// Bytes of global workspace the kernel needs besides the runner's activation buffers, and
// where each piece sits in it.
struct StepWorkspace {
    size_t part_ml, part_o, tickets, cand_val, cand_idx, bar, total;
};
StepWorkspace step_workspace(int n_heads, int head_dim, int n_kv_heads, int max_splits, int grid);

// Whether the kernel can run this model on this device (shared memory for the widest input
// plus at least three ring stages; one CTA per SM resident).  On success *grid_out is the
// cooperative grid size.
bool step_supported(tlc_ctx *ctx, int qtype, int d, int kmax, int head_dim, int *grid_out);

// Launches the kernel on the context's stream (cooperative launch).  The smem plan fields
// and nstages of `p` are filled here.
int32_t step_launch(tlc_ctx *ctx, int qtype, int grid, int kmax, StepParams &p);

}  // namespace tlc_step
