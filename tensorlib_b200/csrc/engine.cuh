// Host-side plumbing of the Llama2 forward: weights, KV caches, activation buffers, the per-layer
// launch sequence and the CUDA graph of one decode step. Mirrors Transformer<half> / Attention /
// FeedForward / TransformerBlock (model/llama2_7b/src/Transformer.cpp) and ActivationBuffer
// (model/llama2_7b/include/ActivationBuffer.hpp) of the reference.
#pragma once
#include <cstdio>

#include <vector>

#include "kernels.cuh"

namespace tlb {

struct LayerWeights {
    __half *attn_norm, *wq, *wk, *wv, *wo, *ffn_norm, *w1, *w2, *w3;
    __half *cache_k, *cache_v;  // (max_seq, H_local, hd)
};

// Hook the tensor-parallel build installs: sum `n` halfs in place across ranks, enqueued on `st`.
struct Collective {
    virtual ~Collective() = default;
    virtual int allreduce_sum_f16(__half* buf, size_t n, cudaStream_t st) = 0;
    virtual int allreduce_sum_f32(float* buf, size_t n, cudaStream_t st) = 0;
    virtual int allgather_f16(const __half* send, __half* recv, size_t n_per_rank, cudaStream_t st) = 0;
    virtual bool graph_capturable() const = 0;
};

class Llama2Engine {
public:
    explicit Llama2Engine(const tl_llama2_config& cfg);
    ~Llama2Engine();
    int allocate();
    int load_payload_host(const __half* payload, bool shared_classifier);
    // stream a llama2.c checkpoint (positioned after its 28-byte header) through two pinned staging
    // buffers: the read of chunk i+1 overlaps the host-to-device copy of chunk i
    int load_payload_stream(FILE* f, long long payload_offset_bytes, bool shared_classifier);
    int init_random(uint64_t seed, float std);

    // Transformer::forward. Token ids must already be in d_tokens_[0..T) (see set_tokens).
    // all_logits: compute logits for every position (what the reference returns) or only the last.
    int forward(int T, int start_pos, bool all_logits, cudaStream_t st);
    int set_tokens(const int* tokens_host, int T, cudaStream_t st);
    int sample_last(int T, cudaStream_t st);  // greedy argmax of the last position -> d_next_

    // One decode step replayed from a CUDA graph: token = *d_next_, position = *d_pos_; writes the
    // sampled id to d_next_ and d_generated_[pos], then increments *d_pos_.
    int decode_steps(int start_pos, int steps, cudaStream_t st);
    int align_ranks(cudaStream_t st);
    int ensure_decode_graph(cudaStream_t st);

    const tl_llama2_config& cfg() const { return cfg_; }
    __half* logits() const { return logits_; }
    int* d_next() const { return d_next_; }
    int* d_pos() const { return d_pos_; }
    int* d_generated() const { return d_generated_; }
    long long launches() const { return launches_; }
    long long weight_bytes() const { return weight_bytes_; }
    int vocab_local() const { return vocab_local_; }
    void set_collective(Collective* c) { coll_ = c; }
    // Fused tensor-parallel exchange (see PeerExchange): allocate this rank's receive region and
    // export it; then map every rank's region. After xch_open the decode step needs no collective
    // library call.
    int xch_export(cudaIpcMemHandle_t* out);
    int xch_open(const cudaIpcMemHandle_t* handles, int world);
    int xch_close();
    const __half* last_logits() const { return last_logits_; }
    int tensor(const char* name, int layer, void** dptr, int* rows, int* cols) const;
    // one decode step with per-phase device timestamps of CTA `cta`: out_host[n_phases][3] in ns
    int decode_profile(int start_pos, int cta, unsigned long long* out_host, int capacity, int* n_phases);

private:
    int ensure_activations(int T, int S);
    int linear(const __half* x, const __half* W, __half* y, int T, int N, int K, cudaStream_t st);
    int forward_reference_order(int T, int pos, bool all_logits, cudaStream_t st);
    int forward_fast_prefill(int T, int pos, bool all_logits, cudaStream_t st);
    int decode_step_fast(cudaStream_t st, bool pdl);  // position-indirect (reads *d_pos_)
    int free_all();

    tl_llama2_config cfg_;
    int hd_, H_local_, dim_local_, hidden_local_, vocab_local_;
    bool shared_classifier_ = true;
    __half *emb_ = nullptr, *final_norm_ = nullptr, *wcls_ = nullptr;
    std::vector<LayerWeights> layers_;
    std::vector<void*> allocs_;
    long long weight_bytes_ = 0;

    // activations
    int act_T_ = 0, act_S_ = 0;
    __half *x_ = nullptr, *xn_ = nullptr, *h_ = nullptr, *q_ = nullptr, *k_ = nullptr, *v_ = nullptr,
           *att_ = nullptr, *ao_ = nullptr, *g_ = nullptr, *u_ = nullptr, *logits_ = nullptr,
           *scores_ = nullptr, *probs_ = nullptr, *vt_ = nullptr;
    std::vector<void*> act_allocs_;
    float* attn_scratch_ = nullptr;
    float* ao32_ = nullptr;  // [dim] fp32 partial sums of the K-split matmuls (tensor parallel decode)
    __half* cls_local_ = nullptr;  // [vocab/world] this rank's slice of the logits before the gather
    unsigned int* attn_counters_ = nullptr;
    int attn_splits_ = 1;
    int *d_tokens_ = nullptr, *d_next_ = nullptr, *d_pos_ = nullptr, *d_generated_ = nullptr;
    const __half *cos_t_ = nullptr, *sin_t_ = nullptr;

    // one-kernel decode step (single GPU, fast numerics): phase list in device memory
    // the persistent step kernel: single GPU, or tensor parallel once the fused exchange is open
    bool use_mega() const { return cfg_.one_kernel_decode != 0 && (coll_ == nullptr || xch_ready_) && cfg_.numerics == TL_NUMERICS_FAST; }
    int ensure_mega();
    int decode_step_mega(cudaStream_t st, unsigned long long* prof = nullptr, int prof_cta = 0);
    void* mega_phases_ = nullptr;
    unsigned int* flow_words_ = nullptr;          // the vectors the phases hand over, as (value, epoch) words
    unsigned long long* flow_cand_ = nullptr;     // [grid] per-CTA sampling candidates
    unsigned int* flow_counters_ = nullptr;       // [0] candidate arrivals, [1] decode steps done (epoch base)
    int mega_n_phases_ = 0, mega_grid_ = 0, mega_smem_ = 0, mega_splits_ = 1, mega_x_bytes_ = 0;
    float* mega_attn_scratch_ = nullptr;
    bool mega_ready_ = false;

    cudaGraphExec_t decode_graph_ = nullptr;
    long long launches_ = 0;
    long long decode_step_launches_ = 0;
    Collective* coll_ = nullptr;
    // exchange region, all payloads as 8-byte (payload, epoch) words:
    // [part0: world*dim words][part1: world*dim words][logits: vocab/2 words][step u32]
    int decode_step_tp_fused(cudaStream_t st, bool pdl);
    PeerExchange make_exchange(int buf, int phase_id) const;
    unsigned char* xch_base_ = nullptr;
    unsigned char* xch_peer_[TL_MAX_TP] = {};
    size_t xch_off_part_[2] = {0, 0}, xch_off_pub_[2] = {0, 0}, xch_off_logits_ = 0, xch_off_step_ = 0, xch_bytes_ = 0;
    unsigned long long* prof_ = nullptr;   // device buffer for %globaltimer stamps while decode_profile runs a step
    bool xch_ready_ = false;
    // prefill part of the exchange region (tp_prefill.cu) and the exchange counter every rank advances in step
    size_t pf_off_recv_ = 0, pf_off_xn_ = 0, pf_off_aflags_ = 0, pf_off_gflags_ = 0;
    int pf_rpo_max_ = 0;
    unsigned int pf_epoch_ = 0;
    __half* align_buf_ = nullptr;       // operand of the rank-aligning allreduce (align_ranks)
    const __half* last_logits_ = nullptr;
};

// Which block of a [rows, cols] checkpoint tensor rank `rank` of `world` keeps.
// kind: 0 replicated, 1 split by rows (wq, wk, wv, w1, w3, classifier), 2 split by columns (wo, w2).
int shard_block(int kind, int rows, int cols, int rank, int world, int* row0, int* nrows, int* col0, int* ncols);

}  // namespace tlb

// the opaque handle of the C ABI
struct tl_llama2 {
    tlb::Llama2Engine* eng;
    int* pinned;  // [max_seq + 8] staging for token ids
};
