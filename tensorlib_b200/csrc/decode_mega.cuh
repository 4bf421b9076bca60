// Argument structures of the one-kernel decode step (decode_mega.cu), shared with the host
// plumbing that fills them (engine.cu).
#pragma once

#include "kernels.cuh"

namespace tlb {

struct FlowLayer {
    const __half *attn_norm, *wq, *wk, *wv, *wo, *ffn_norm, *w1, *w3, *w2;
    __half *cache_k, *cache_v;   // (max_seq, local heads, head_dim)
};

// Activation vectors that one phase hands to the next travel through L2 as 32-bit words
// (fp16 value in the low half, the low 16 bits of the producing phase's epoch in the high half).
struct FlowWords {
    unsigned int *x;     // [dim]   residual stream entering a layer (after w2 of the previous one)
    unsigned int *h;     // [dim]   residual stream after attention
    unsigned int *q, *k, *v;   // [dim_local] this step's query / key / value rows
    unsigned int *att;   // [dim_local] attention output
    unsigned int *g;     // [hidden_local] silu(gate) * up
};

struct FlowArgs {
    const FlowLayer* layers; int n_layers;
    const __half* emb; const __half* final_norm; const __half* wcls;
    int dim, dl, hl, vocab, vocab_local, H, hd, splits, max_seq;
    FlowWords w;
    float* attn_scratch; unsigned int* attn_counters;
    const __half* cos_t; const __half* sin_t; const __half* silu_tab;
    __half* logits;                         // [vocab] fp16 logits of this step (what the host reads)
    unsigned long long* cand;               // [grid] per-CTA best (value, index) of the classifier rows
    unsigned int* cand_counter;
    int* d_next; int* d_pos; int* d_generated;
    unsigned int* step;                     // decode steps done so far (epoch base), same on every rank
    int* status; float eps;
    int x_bytes;                            // shared-memory bytes reserved for the activation vector / attention scratch
    // tensor parallelism: fp32 partial sums of wo (0) and w2 (1) and the fp16 logit slices are pushed
    // into slot [rank] of these regions in every rank's memory as (payload, epoch) 8-byte words
    int world, rank;
    const unsigned long long* local_part[2];        // [world][dim]
    unsigned long long* peer_part[2][TL_MAX_TP];    // slot [rank] in rank d's memory
    const unsigned long long* local_logits;         // [vocab / 2]
    unsigned long long* peer_logits[TL_MAX_TP];     // slot [rank] (vocab_local / 2 words) in rank d's memory
    unsigned int exchange_tries;
    unsigned long long* prof;  // optional [phases][3] %globaltimer stamps written by CTA prof_cta
    int prof_cta;
};

inline int flow_phases(int n_layers) { return 5 * n_layers + 1; }
int mega_smem_bytes(int max_k);
int mega_x_bytes(int max_k);
int mega_attn_splits(int H, int grid);
// cooperative launch of the step kernel on `st`
int launch_decode_flow(const FlowArgs& args, int grid, int smem, cudaStream_t st);

}  // namespace tlb
