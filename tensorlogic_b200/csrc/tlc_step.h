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

// Activations cross from CTA to CTA as "flagged words": 8 bytes = 4 bytes of data (two f16
// values, or one f32 / int32) + a 32-bit epoch number, written with one 8-byte store.  A reader
// polls the word until the epoch is the one it expects; no barrier, no fence, no atomic.
// Every (decode step, layer, buffer) has its own epoch, and epochs grow from launch to launch
// (the host passes the first one), so a word of an earlier step never matches.
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
    // flagged-word buffers (global workspace)
    uint2 *x_w, *x1_w, *q_w, *kv_w, *attn_w, *act_w;  // [d/2] [d/2] [qd/2] [kvd: k then v] [qd/2] [ffn/2]
    uint2 *part_w;   // split-key partials [H][max_splits][D + 2] f32: max, sum, O
    uint4 *cand_w;   // per CTA {best logit, epoch, its index, epoch}
    uint2 *tok_w;    // the sampled token, for the next step inside the same launch
    int max_splits;
    __half *logits;  // [vocab] plain f16 (read by the host after the launch)
    int *ids, *positions, *next_ids;  // device: pending token, its position, sampled token (sequence 0)
    const int *ids_src;       // where the first step reads its token (pinned host memory) or null = ids
    int *host_next;           // pinned host word for the last step's token, or null
    tlc_dev_status *host_status;  // pinned mirror of the status word, written before host_next
    uint64_t *trace;          // null, or [steps][n_layers * 5 + 2][3] device times (ns) of CTA 0: a phase's
                              // input ready, dot products done, outputs stored (0 where a phase has no such point)
    uint32_t epoch_base;      // first epoch of this launch
    int steps;
    int poll_backoff_ns;      // sleep between two polls of a flagged word that is not there yet (0: none)
    int nstages;
    uint32_t off_xres, off_xin, off_cinit, off_xperm, off_attn, off_ring;
    tlc_dev_status *status;
    uint64_t wait_ns;
};

// Epochs one decode step uses (the host advances its counter by steps * this).
inline uint32_t epochs_per_step(int n_layers) { return (uint32_t)n_layers * 8u + 8u; }

// Bytes of global workspace the kernel needs besides the runner's buffers, and where each
// piece sits in it.  Must be zero before the first launch (epoch 0 is never used).
struct StepWorkspace {
    size_t x, x1, q, kv, attn, act, part, cand, tok, total;
};
StepWorkspace step_workspace(int d, int qd, int kvd, int ffn, int n_heads, int head_dim, int max_splits, int grid);

// Key splits the attention phase may use at most on a grid of `grid` CTAs.
int step_max_splits(int grid, int n_heads, int n_kv_heads);

// Whether the kernel can run this model on this device (shared memory for the widest input
// plus at least three ring stages; one CTA per SM resident).  On success *grid_out is the grid size.
bool step_supported(tlc_ctx *ctx, int qtype, int d, int kmax, int head_dim, int *grid_out);

// Launches the kernel on the context's stream.  The smem plan fields and nstages of `p` are
// filled here.
int32_t step_launch(tlc_ctx *ctx, int qtype, int grid, int kmax, StepParams &p);

}  // namespace tlc_step
