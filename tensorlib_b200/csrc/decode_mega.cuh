// Argument structures of the one-kernel decode step (decode_mega.cu), shared with the host
// plumbing that fills them (engine.cu).
#pragma once

#include "kernels.cuh"

namespace tlb {

struct MegaPhase {
    int kind, epilogue;
    const __half* x;        // nullptr: the embedding row of the current token
    const __half* norm_w;   // nullptr: no RMSNorm prologue
    const __half* W0; const __half* W1; const __half* W2;
    int N_each, K, total_units;
    __half* y;
    const __half* residual; // EPI_RESIDUAL; nullptr: the embedding row of the current token
    float* y32;
    __half* k_cache; __half* v_cache;
};

struct MegaArgs {
    const MegaPhase* phases; int n_phases;
    const __half* emb; int dim, vocab;
    int H, hd, splits, max_seq; long long kv_pitch;
    float* attn_scratch; unsigned int* attn_counters;
    const __half* cos_t; const __half* sin_t; const __half* silu_tab;
    const __half* logits; int* d_next; int* d_pos; int* d_generated;
    unsigned int* grid_bar; int* status; float eps;
    int x_bytes;            // shared-memory bytes reserved for the activation vector / attention scratch
    unsigned long long* prof;  // optional [n_phases][3] globaltimer stamps written by CTA prof_cta
    int prof_cta;
};


int mega_smem_bytes(int max_k);
int mega_x_bytes(int max_k);
int mega_attn_splits(int H, int grid);
// memset of the grid-barrier word + cooperative launch of the step kernel on `st`
int launch_decode_mega(const MegaArgs& args, int grid, int smem, cudaStream_t st);

}  // namespace tlb
