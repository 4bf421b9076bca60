// Llama2 forward plumbing. See engine.cuh.
#include "engine.cuh"
#include "decode_mega.cuh"

#include <algorithm>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <vector>
#include <string>

namespace tlb {

namespace {

// seeded N(0, std^2) fill on the device (splitmix64 counter hash + Box-Muller)
__device__ __forceinline__ unsigned long long mix64(unsigned long long x) {
    x += 0x9E3779B97F4A7C15ull;
    x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
    x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
    return x ^ (x >> 31);
}
__global__ void k_fill_normal(__half* out, size_t n, unsigned long long key, float std) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    unsigned long long b = mix64(i * 0xD1342543DE82EF95ull + key);
    float u1 = ((float)(b >> 40) + 1.0f) * (1.0f / 16777216.0f);
    float u2 = (float)((b >> 8) & 0xFFFFFF) * (1.0f / 16777216.0f);
    out[i] = __float2half_rn(sqrtf(-2.0f * logf(u1)) * cospif(2.0f * u2) * std);
}
__global__ void k_fill_const(__half* out, size_t n, float v) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = __float2half_rn(v);
}
// bookkeeping at the end of a decode step: record the sampled id, advance the position
__global__ void k_advance(int* pos, const int* next, int* generated, int max_seq) {
    int p = *pos;
    if (p >= 0 && p < max_seq) generated[p] = *next;
    *pos = p + 1;
}

}  // namespace

Llama2Engine::Llama2Engine(const tl_llama2_config& cfg) : cfg_(cfg) {
    hd_ = cfg.dim / cfg.n_heads;
    H_local_ = cfg.n_heads / cfg.tp_world;
    dim_local_ = H_local_ * hd_;
    hidden_local_ = cfg.hidden_dim / cfg.tp_world;
    vocab_local_ = cfg.vocab_size / cfg.tp_world;
}

Llama2Engine::~Llama2Engine() { free_all(); }

int Llama2Engine::free_all() {
    xch_close();
    if (decode_graph_) { cudaGraphExecDestroy(decode_graph_); decode_graph_ = nullptr; }
    mega_ready_ = false;
    for (void* p : allocs_) cudaFree(p);
    for (void* p : act_allocs_) cudaFree(p);
    allocs_.clear();
    act_allocs_.clear();
    return TL_OK;
}

int Llama2Engine::allocate() {
    const size_t dim = cfg_.dim, L = cfg_.n_layers, V = cfg_.vocab_size, S = cfg_.max_seq_len;
    auto alloc = [&](__half** p, size_t elems, bool weight) -> int {
        void* d = nullptr;
        TL_CUDA(cudaMalloc(&d, elems * sizeof(__half)));
        allocs_.push_back(d);
        *p = static_cast<__half*>(d);
        if (weight) weight_bytes_ += (long long)(elems * sizeof(__half));
        return TL_OK;
    };
    // one allocation per tensor kind, layers consecutive, like the checkpoint groups them
    __half *an, *wq, *wk, *wv, *wo, *fn, *w1, *w2, *w3, *ck, *cv;
    TL_PROPAGATE(alloc(&emb_, V * dim, true));
    TL_PROPAGATE(alloc(&an, L * dim, true));
    TL_PROPAGATE(alloc(&wq, L * dim_local_ * dim, true));
    TL_PROPAGATE(alloc(&wk, L * dim_local_ * dim, true));
    TL_PROPAGATE(alloc(&wv, L * dim_local_ * dim, true));
    TL_PROPAGATE(alloc(&wo, L * dim * dim_local_, true));
    TL_PROPAGATE(alloc(&fn, L * dim, true));
    TL_PROPAGATE(alloc(&w1, L * hidden_local_ * dim, true));
    TL_PROPAGATE(alloc(&w2, L * dim * hidden_local_, true));
    TL_PROPAGATE(alloc(&w3, L * hidden_local_ * dim, true));
    TL_PROPAGATE(alloc(&final_norm_, dim, true));
    TL_PROPAGATE(alloc(&wcls_, (size_t)vocab_local_ * dim, true));  // unused (aliased) when shared on 1 GPU
    TL_PROPAGATE(alloc(&ck, L * S * dim_local_, false));
    TL_PROPAGATE(alloc(&cv, L * S * dim_local_, false));
    TL_CUDA(cudaMemset(ck, 0, L * S * dim_local_ * sizeof(__half)));
    TL_CUDA(cudaMemset(cv, 0, L * S * dim_local_ * sizeof(__half)));
    layers_.resize(L);
    for (size_t l = 0; l < L; l++) {
        LayerWeights& w = layers_[l];
        w.attn_norm = an + l * dim;
        w.wq = wq + l * dim_local_ * dim;
        w.wk = wk + l * dim_local_ * dim;
        w.wv = wv + l * dim_local_ * dim;
        w.wo = wo + l * dim * dim_local_;
        w.ffn_norm = fn + l * dim;
        w.w1 = w1 + l * hidden_local_ * dim;
        w.w2 = w2 + l * dim * hidden_local_;
        w.w3 = w3 + l * hidden_local_ * dim;
        w.cache_k = ck + l * S * dim_local_;
        w.cache_v = cv + l * S * dim_local_;
    }
    void* d = nullptr;
    TL_CUDA(cudaMalloc(&d, (2 * S + 8) * sizeof(int)));
    allocs_.push_back(d);
    d_tokens_ = static_cast<int*>(d);
    d_generated_ = d_tokens_ + S;
    d_next_ = d_generated_ + S;
    d_pos_ = d_next_ + 1;
    TL_CUDA(cudaMemset(d, 0, (2 * S + 8) * sizeof(int)));
    TL_PROPAGATE(rope_table(hd_, (int)S, &cos_t_, &sin_t_));
    // decode attention: enough CTAs to cover the SMs
    attn_splits_ = 1;
    while (H_local_ * attn_splits_ < sm_count() && attn_splits_ < 8) attn_splits_ *= 2;  // <= 8: one cluster per head
    if (const char* e = getenv("TL_ATTN_SPLITS")) {   // experiments: 1, 2, 4 or 8
        const int v = atoi(e);
        if (v == 1 || v == 2 || v == 4 || v == 8) attn_splits_ = v;
    }
    TL_CUDA(cudaMalloc(&d, (size_t)H_local_ * 16 * (hd_ + 2) * sizeof(float)));
    allocs_.push_back(d);
    attn_scratch_ = static_cast<float*>(d);
    TL_CUDA(cudaMalloc(&d, (size_t)H_local_ * sizeof(unsigned int)));
    allocs_.push_back(d);
    attn_counters_ = static_cast<unsigned int*>(d);
    TL_CUDA(cudaMemset(d, 0, (size_t)H_local_ * sizeof(unsigned int)));
    TL_CUDA(cudaMalloc(&d, dim * sizeof(float)));
    allocs_.push_back(d);
    ao32_ = static_cast<float*>(d);
    TL_CUDA(cudaMalloc(&d, (size_t)vocab_local_ * sizeof(__half)));
    allocs_.push_back(d);
    cls_local_ = static_cast<__half*>(d);
    return ensure_activations(1, 0);
}

// ActivationBuffer (model/llama2_7b/include/ActivationBuffer.hpp:8-57): buffers for T tokens;
// the (H,T,S) score buffers only exist for multi-token passes.
int Llama2Engine::ensure_activations(int T, int S) {
    // score buffers are sized for the whole context once they are needed at all
    const bool need_scores = S > 0 && (vt_ == nullptr || T > act_T_);
    if (T <= act_T_ && !need_scores) return TL_OK;
    if (S > 0 || act_S_ > 0) S = cfg_.max_seq_len;
    TL_CUDA(cudaDeviceSynchronize());
    if (decode_graph_) { cudaGraphExecDestroy(decode_graph_); decode_graph_ = nullptr; }
    mega_ready_ = false;
    for (void* p : act_allocs_) cudaFree(p);
    act_allocs_.clear();
    const int Tn = std::max(T, act_T_), Sn = std::max(S, act_S_);
    auto alloc = [&](__half** p, size_t elems) -> int {
        void* d = nullptr;
        TL_CUDA(cudaMalloc(&d, std::max<size_t>(elems, 8) * sizeof(__half)));
        act_allocs_.push_back(d);
        *p = static_cast<__half*>(d);
        return TL_OK;
    };
    const size_t dim = cfg_.dim;
    TL_PROPAGATE(alloc(&x_, Tn * dim));
    TL_PROPAGATE(alloc(&xn_, Tn * dim));
    TL_PROPAGATE(alloc(&h_, Tn * dim));
    TL_PROPAGATE(alloc(&q_, (size_t)Tn * dim_local_));
    TL_PROPAGATE(alloc(&k_, (size_t)Tn * dim_local_));
    TL_PROPAGATE(alloc(&v_, (size_t)Tn * dim_local_));
    TL_PROPAGATE(alloc(&att_, (size_t)Tn * dim_local_));
    TL_PROPAGATE(alloc(&ao_, Tn * dim));
    TL_PROPAGATE(alloc(&g_, (size_t)Tn * hidden_local_));
    TL_PROPAGATE(alloc(&u_, (size_t)Tn * hidden_local_));
    TL_PROPAGATE(alloc(&logits_, (size_t)Tn * cfg_.vocab_size));
    scores_ = probs_ = vt_ = nullptr;
    if (Sn > 0) {
        // the fused prefill attention (fast numerics, head_dim 128) keeps the scores on the SM
        const bool fused_attn = cfg_.numerics != TL_NUMERICS_REFERENCE_ORDER && hd_ == 128 &&
                                tensor_map_encode_available();
        if (!fused_attn) {
            TL_PROPAGATE(alloc(&scores_, (size_t)H_local_ * Tn * Sn));
            TL_PROPAGATE(alloc(&probs_, (size_t)H_local_ * Tn * Sn));
        }
        TL_PROPAGATE(alloc(&vt_, (size_t)dim_local_ * (Sn + 8)));
    }
    act_T_ = Tn;
    act_S_ = Sn;
    return TL_OK;
}

// read_weights (model/llama2_7b/src/main.cpp:36-190): same tensor order; each rank keeps its
// tensor-parallel slice (row blocks of wq/wk/wv/w1/w3 and of the classifier, column blocks of
// wo/w2).
int Llama2Engine::load_payload_host(const __half* payload, bool shared_classifier) {
    const size_t dim = cfg_.dim, hid = cfg_.hidden_dim, L = cfg_.n_layers, V = cfg_.vocab_size;
    const int r = cfg_.tp_rank;
    shared_classifier_ = shared_classifier;
    const __half* cur = payload;
    // copy this rank's block of a [nrows_full, ncols_full] checkpoint tensor (kind: see shard_block)
    auto put = [&](__half* dst, const __half* src, int kind, size_t nrows_full, size_t ncols_full) -> int {
        int r0, nr, c0, nc;
        TL_PROPAGATE(shard_block(kind, (int)nrows_full, (int)ncols_full, r, cfg_.tp_world, &r0, &nr, &c0, &nc));
        TL_CUDA(cudaMemcpy2D(dst, (size_t)nc * sizeof(__half), src + (size_t)r0 * ncols_full + c0,
                             ncols_full * sizeof(__half), (size_t)nc * sizeof(__half), nr, cudaMemcpyHostToDevice));
        return TL_OK;
    };
    const __half* emb_host = cur;
    TL_PROPAGATE(put(emb_, cur, 0, V, dim)); cur += V * dim;
    for (size_t l = 0; l < L; l++) { TL_PROPAGATE(put(layers_[l].attn_norm, cur, 0, 1, dim)); cur += dim; }
    for (size_t l = 0; l < L; l++) { TL_PROPAGATE(put(layers_[l].wq, cur, 1, dim, dim)); cur += dim * dim; }
    for (size_t l = 0; l < L; l++) { TL_PROPAGATE(put(layers_[l].wk, cur, 1, dim, dim)); cur += dim * dim; }
    for (size_t l = 0; l < L; l++) { TL_PROPAGATE(put(layers_[l].wv, cur, 1, dim, dim)); cur += dim * dim; }
    for (size_t l = 0; l < L; l++) { TL_PROPAGATE(put(layers_[l].wo, cur, 2, dim, dim)); cur += dim * dim; }
    for (size_t l = 0; l < L; l++) { TL_PROPAGATE(put(layers_[l].ffn_norm, cur, 0, 1, dim)); cur += dim; }
    for (size_t l = 0; l < L; l++) { TL_PROPAGATE(put(layers_[l].w1, cur, 1, hid, dim)); cur += hid * dim; }
    for (size_t l = 0; l < L; l++) { TL_PROPAGATE(put(layers_[l].w2, cur, 2, dim, hid)); cur += hid * dim; }
    for (size_t l = 0; l < L; l++) { TL_PROPAGATE(put(layers_[l].w3, cur, 1, hid, dim)); cur += hid * dim; }
    TL_PROPAGATE(put(final_norm_, cur, 0, 1, dim)); cur += dim;
    if (shared_classifier) {
        TL_PROPAGATE(put(wcls_, emb_host, 1, V, dim));
    } else {
        cur += (size_t)cfg_.max_seq_len * hd_;  // RoPE values the reference skips (main.cpp:175-177)
        TL_PROPAGATE(put(wcls_, cur, 1, V, dim));
    }
    return TL_OK;
}

// The same tensor order read from a file without holding the checkpoint in host memory
// (read_weights, main.cpp:36-190, freads every tensor group into one pageable buffer and copies it
// with a blocking cudaMemcpy). Two pinned 64 MB staging buffers: while chunk i travels to the
// device (cudaMemcpy2DAsync, which also cuts this rank's column block out of wo / w2 rows), chunk
// i+1 is read from the file. Row-split tensors only read their own rows.
int Llama2Engine::load_payload_stream(FILE* f, long long payload_offset_bytes, bool shared_classifier) {
    const size_t dim = cfg_.dim, hid = cfg_.hidden_dim, L = cfg_.n_layers, V = cfg_.vocab_size;
    shared_classifier_ = shared_classifier;
    constexpr size_t CAP = (size_t)64 << 20;
    __half* stage[2] = {nullptr, nullptr};
    cudaEvent_t done[2] = {nullptr, nullptr};
    cudaStream_t st = nullptr;
    int rc = TL_OK;
    auto cleanup = [&]() {
        if (st) { cudaStreamSynchronize(st); cudaStreamDestroy(st); }
        for (int i = 0; i < 2; i++) { if (done[i]) cudaEventDestroy(done[i]); if (stage[i]) cudaFreeHost(stage[i]); }
    };
    for (int i = 0; i < 2 && rc == TL_OK; i++) {
        if (cudaMallocHost(&stage[i], CAP) != cudaSuccess) rc = set_error(TL_ERR_OUT_OF_MEMORY, "pinned staging buffer of %zu bytes", CAP);
        else if (cudaEventCreateWithFlags(&done[i], cudaEventDisableTiming) != cudaSuccess) rc = set_error(TL_ERR_CUDA, "event creation failed");
    }
    if (rc == TL_OK && cudaStreamCreateWithFlags(&st, cudaStreamNonBlocking) != cudaSuccess) rc = set_error(TL_ERR_CUDA, "stream creation failed");
    int cur = 0;
    // copy this rank's block of the [nrows_full, ncols_full] tensor that starts `elem_off` elements into the payload
    auto put = [&](__half* dst, size_t elem_off, int kind, size_t nrows_full, size_t ncols_full) -> int {
        int r0, nr, c0, nc;
        TL_PROPAGATE(shard_block(kind, (int)nrows_full, (int)ncols_full, cfg_.tp_rank, cfg_.tp_world, &r0, &nr, &c0, &nc));
        const size_t rows_per_chunk = std::max<size_t>(1, CAP / (ncols_full * sizeof(__half)));
        TL_REQUIRE(ncols_full * sizeof(__half) <= CAP, "checkpoint row of %zu bytes exceeds the staging buffer", ncols_full * sizeof(__half));
        for (size_t row = 0; row < (size_t)nr; row += rows_per_chunk) {
            const size_t rows = std::min(rows_per_chunk, (size_t)nr - row);
            TL_CUDA(cudaEventSynchronize(done[cur]));            // the previous copy out of this buffer has finished
            const long long pos = payload_offset_bytes + (long long)((elem_off + ((size_t)r0 + row) * ncols_full) * sizeof(__half));
            if (fseeko(f, pos, SEEK_SET) != 0) return set_error(TL_ERR_IO, "seek to %lld failed", pos);
            const size_t want = rows * ncols_full;
            if (fread(stage[cur], sizeof(__half), want, f) != want) return set_error(TL_ERR_IO, "checkpoint is truncated (tensor at element %zu)", elem_off);
            TL_CUDA(cudaMemcpy2DAsync(dst + row * (size_t)nc, (size_t)nc * sizeof(__half), stage[cur] + c0,
                                      ncols_full * sizeof(__half), (size_t)nc * sizeof(__half), rows, cudaMemcpyHostToDevice, st));
            TL_CUDA(cudaEventRecord(done[cur], st));
            cur ^= 1;
        }
        return TL_OK;
    };
    auto run = [&]() -> int {
        size_t off = 0;
        const size_t emb_off = off;
        TL_PROPAGATE(put(emb_, off, 0, V, dim)); off += V * dim;
        for (size_t l = 0; l < L; l++) { TL_PROPAGATE(put(layers_[l].attn_norm, off, 0, 1, dim)); off += dim; }
        for (size_t l = 0; l < L; l++) { TL_PROPAGATE(put(layers_[l].wq, off, 1, dim, dim)); off += dim * dim; }
        for (size_t l = 0; l < L; l++) { TL_PROPAGATE(put(layers_[l].wk, off, 1, dim, dim)); off += dim * dim; }
        for (size_t l = 0; l < L; l++) { TL_PROPAGATE(put(layers_[l].wv, off, 1, dim, dim)); off += dim * dim; }
        for (size_t l = 0; l < L; l++) { TL_PROPAGATE(put(layers_[l].wo, off, 2, dim, dim)); off += dim * dim; }
        for (size_t l = 0; l < L; l++) { TL_PROPAGATE(put(layers_[l].ffn_norm, off, 0, 1, dim)); off += dim; }
        for (size_t l = 0; l < L; l++) { TL_PROPAGATE(put(layers_[l].w1, off, 1, hid, dim)); off += hid * dim; }
        for (size_t l = 0; l < L; l++) { TL_PROPAGATE(put(layers_[l].w2, off, 2, dim, hid)); off += hid * dim; }
        for (size_t l = 0; l < L; l++) { TL_PROPAGATE(put(layers_[l].w3, off, 1, hid, dim)); off += hid * dim; }
        TL_PROPAGATE(put(final_norm_, off, 0, 1, dim)); off += dim;
        if (shared_classifier) return put(wcls_, emb_off, 1, V, dim);
        off += (size_t)cfg_.max_seq_len * hd_;  // RoPE values the reference skips (main.cpp:175-177)
        return put(wcls_, off, 1, V, dim);
    };
    if (rc == TL_OK) rc = run();
    if (rc == TL_OK && cudaStreamSynchronize(st) != cudaSuccess) rc = set_error(TL_ERR_CUDA, "checkpoint upload failed");
    cleanup();
    return rc;
}

int Llama2Engine::init_random(uint64_t seed, float std) {
    const size_t dim = cfg_.dim, L = cfg_.n_layers;
    unsigned long long id = 0;
    auto fill = [&](__half* p, size_t n) -> int {
        unsigned long long key = seed * 0x9E3779B97F4A7C15ull + (++id) * 0xD6E8FEB86659FD93ull +
                                 (unsigned long long)cfg_.tp_rank * 0xA0761D6478BD642Full;
        k_fill_normal<<<(unsigned)ceil_div(n, 256), 256>>>(p, n, key, std);
        TL_LAUNCH_CHECK();
        return TL_OK;
    };
    auto ones = [&](__half* p, size_t n) -> int {
        k_fill_const<<<(unsigned)ceil_div(n, 256), 256>>>(p, n, 1.0f);
        TL_LAUNCH_CHECK();
        return TL_OK;
    };
    shared_classifier_ = false;
    TL_PROPAGATE(fill(emb_, (size_t)cfg_.vocab_size * dim));
    TL_PROPAGATE(fill(wcls_, (size_t)vocab_local_ * dim));
    TL_PROPAGATE(ones(final_norm_, dim));
    for (size_t l = 0; l < L; l++) {
        LayerWeights& w = layers_[l];
        TL_PROPAGATE(ones(w.attn_norm, dim));
        TL_PROPAGATE(ones(w.ffn_norm, dim));
        TL_PROPAGATE(fill(w.wq, (size_t)dim_local_ * dim));
        TL_PROPAGATE(fill(w.wk, (size_t)dim_local_ * dim));
        TL_PROPAGATE(fill(w.wv, (size_t)dim_local_ * dim));
        TL_PROPAGATE(fill(w.wo, dim * dim_local_));
        TL_PROPAGATE(fill(w.w1, (size_t)hidden_local_ * dim));
        TL_PROPAGATE(fill(w.w2, dim * hidden_local_));
        TL_PROPAGATE(fill(w.w3, (size_t)hidden_local_ * dim));
    }
    TL_CUDA(cudaDeviceSynchronize());
    return TL_OK;
}

int shard_block(int kind, int rows, int cols, int rank, int world, int* row0, int* nrows, int* col0, int* ncols) {
    TL_REQUIRE(row0 && nrows && col0 && ncols && world >= 1 && rank >= 0 && rank < world, "bad argument");
    *row0 = 0; *nrows = rows; *col0 = 0; *ncols = cols;
    if (kind == 1) {
        TL_REQUIRE(rows % world == 0, "%d rows do not divide by %d ranks", rows, world);
        *nrows = rows / world; *row0 = rank * *nrows;
    } else if (kind == 2) {
        TL_REQUIRE(cols % world == 0, "%d columns do not divide by %d ranks", cols, world);
        *ncols = cols / world; *col0 = rank * *ncols;
    } else {
        TL_REQUIRE(kind == 0, "unknown shard kind %d", kind);
    }
    return TL_OK;
}

int Llama2Engine::tensor(const char* name, int layer, void** dptr, int* rows, int* cols) const {
    const std::string n(name);
    auto set = [&](const __half* p, int r, int c) { *dptr = const_cast<__half*>(p); *rows = r; *cols = c; return TL_OK; };
    if (n == "tok_embeddings") return set(emb_, cfg_.vocab_size, cfg_.dim);
    if (n == "norm") return set(final_norm_, 1, cfg_.dim);
    if (n == "output") return set((shared_classifier_ && cfg_.tp_world == 1) ? emb_ : wcls_, vocab_local_, cfg_.dim);
    TL_REQUIRE(layer >= 0 && layer < cfg_.n_layers, "layer %d out of range", layer);
    const LayerWeights& w = layers_[layer];
    if (n == "attention_norm") return set(w.attn_norm, 1, cfg_.dim);
    if (n == "ffn_norm") return set(w.ffn_norm, 1, cfg_.dim);
    if (n == "wq") return set(w.wq, dim_local_, cfg_.dim);
    if (n == "wk") return set(w.wk, dim_local_, cfg_.dim);
    if (n == "wv") return set(w.wv, dim_local_, cfg_.dim);
    if (n == "wo") return set(w.wo, cfg_.dim, dim_local_);
    if (n == "w1") return set(w.w1, hidden_local_, cfg_.dim);
    if (n == "w3") return set(w.w3, hidden_local_, cfg_.dim);
    if (n == "w2") return set(w.w2, cfg_.dim, hidden_local_);
    return set_error(TL_ERR_INVALID_ARGUMENT, "unknown tensor name '%s'", name);
}

int Llama2Engine::set_tokens(const int* tokens_host, int T, cudaStream_t st) {
    TL_REQUIRE(T > 0 && T <= cfg_.max_seq_len, "token count %d out of range", T);
    TL_CUDA(cudaMemcpyAsync(d_tokens_, tokens_host, (size_t)T * sizeof(int), cudaMemcpyHostToDevice, st));
    return TL_OK;
}

// nn::Linear::forward -> Tensor::matmul -> Device::matmul2d (linear.cpp:43-49, matmul.cpp:313-320)
int Llama2Engine::linear(const __half* x, const __half* W, __half* y, int T, int N, int K, cudaStream_t st) {
    if (cfg_.numerics == TL_NUMERICS_REFERENCE_ORDER) {
        SeqMatmul p{x, W, y, 1, T, N, K, K, 1, K, 1, N, 0, 0, 0};
        launches_++;
        return launch_matmul_seq(p, st);
    }
    if (gemv_ring_rows_supported(x, W, T, N, K, K, K)) {
        launches_++;
        return launch_gemv(x, W, y, T, N, K, K, K, N, st, true);
    }
    if (T > 8 && T <= 128 && hgemm_supported(x, W, y, T, N, K, K, K, N) && (reinterpret_cast<uintptr_t>(y) & 15) == 0 &&
        hgemm_splitk_preferred(T, N, K)) {
        launches_++;
        return launch_hgemm(x, W, y, 1, T, N, K, K, K, N, 0, 0, 0, st, true);
    }
    if (T >= 2 && T <= 128 && skinny_supported(x, W, T, N, K, K, K)) {
        launches_++;
        return launch_skinny(x, W, y, T, N, K, K, K, N, st, true);     // model weights are constants
    }
    if (T > 8 && hgemm_supported(x, W, y, T, N, K, K, K, N)) {
        launches_++;
        return launch_hgemm(x, W, y, 1, T, N, K, K, K, N, 0, 0, 0, st, true);
    }
    if (gemv_supported(x, W, T <= 8 ? T : 8, N, K, K)) {
        for (int t0 = 0; t0 < T; t0 += 8) {  // skinny batches: stream the weights once per 8 rows
            int m = std::min(8, T - t0);
            launches_++;
            TL_PROPAGATE(launch_gemv(x + (size_t)t0 * K, W, y + (size_t)t0 * N, m, N, K, K, K, N, st));
        }
        return TL_OK;
    }
    SeqMatmul p{x, W, y, 1, T, N, K, K, 1, K, 1, N, 0, 0, 0};
    launches_++;
    return launch_matmul_seq(p, st);
}

int Llama2Engine::forward(int T, int start_pos, bool all_logits, cudaStream_t st) {
    TL_REQUIRE(T > 0 && start_pos >= 0 && start_pos + T <= cfg_.max_seq_len,
               "forward: T=%d start_pos=%d exceeds max_seq_len=%d", T, start_pos, cfg_.max_seq_len);
    const bool exact = cfg_.numerics == TL_NUMERICS_REFERENCE_ORDER;
    TL_PROPAGATE(ensure_activations(T, (exact || T > 1) ? start_pos + T : 0));
    last_logits_ = logits_ + (size_t)(T - 1) * cfg_.vocab_size;
    if (exact) return forward_reference_order(T, start_pos, all_logits, st);
    if (T == 1) {
        // same launch sequence as the graph, position passed through *d_pos_
        TL_CUDA(cudaMemcpyAsync(d_pos_, &start_pos, sizeof(int), cudaMemcpyHostToDevice, st));
        TL_CUDA(cudaMemcpyAsync(d_next_, d_tokens_, sizeof(int), cudaMemcpyDeviceToDevice, st));
        if (use_mega()) {
            TL_PROPAGATE(ensure_mega());
            return decode_step_mega(st);
        }
        return decode_step_fast(st, false);
    }
    return forward_fast_prefill(T, start_pos, all_logits, st);
}

// The reference's op sequence, one kernel per op, reference-order numerics throughout:
// Transformer::forward (Transformer.cpp:264-299), TransformerBlock::forward (:162-178),
// Attention::forward (:28-112), FeedForward::forward (:133-145).
int Llama2Engine::forward_reference_order(int T, int pos, bool all_logits, cudaStream_t st) {
    const int dim = cfg_.dim, S = pos + T, H = H_local_;
    TL_REQUIRE(cfg_.tp_world == 1, "reference-order numerics is single-GPU");
    launches_++;
    TL_PROPAGATE(launch_embedding(x_, emb_, d_tokens_, T, dim, cfg_.vocab_size, st));
    for (int l = 0; l < cfg_.n_layers; l++) {
        const LayerWeights& w = layers_[l];
        launches_ += 16;
        TL_PROPAGATE(launch_rmsnorm_seq(xn_, x_, w.attn_norm, 1e-5f, dim, T, st));
        TL_PROPAGATE(linear(xn_, w.wq, q_, T, dim, dim, st));
        TL_PROPAGATE(linear(xn_, w.wk, k_, T, dim, dim, st));
        TL_PROPAGATE(linear(xn_, w.wv, v_, T, dim, dim, st));
        TL_PROPAGATE(launch_rope(q_, q_, pos, T, T, H, hd_, cos_t_, sin_t_, st));
        TL_PROPAGATE(launch_rope(k_, k_, pos, T, T, H, hd_, cos_t_, sin_t_, st));
        TL_PROPAGATE(launch_copy_rows(w.cache_k + (size_t)pos * dim, k_, T, dim, dim, st));
        TL_PROPAGATE(launch_copy_rows(w.cache_v + (size_t)pos * dim, v_, T, dim, dim, st));
        // scores[h] (T x S) = q[:, h, :] . K[:, h, :]^T
        SeqMatmul qk{q_, w.cache_k, scores_, H, T, S, hd_, dim, 1, dim, 1, S, hd_, hd_, (long long)T * S};
        TL_PROPAGATE(launch_matmul_seq(qk, st));
        TL_PROPAGATE(launch_scale_mask(scores_, H, T, S, pos, hd_, st));
        TL_PROPAGATE(launch_softmax_seq(probs_, scores_, (size_t)H * T, S, st));
        // att[:, h, :] (T x hd) = P[h] (T x S) . V[:, h, :]
        SeqMatmul pv{probs_, w.cache_v, att_, H, T, hd_, S, S, 1, 1, dim, dim, (long long)T * S, hd_, hd_};
        TL_PROPAGATE(launch_matmul_seq(pv, st));
        TL_PROPAGATE(linear(att_, w.wo, ao_, T, dim, dim, st));
        TL_PROPAGATE(launch_binary(h_, x_, ao_, (size_t)T * dim, 0, st));
        TL_PROPAGATE(launch_rmsnorm_seq(xn_, h_, w.ffn_norm, 1e-5f, dim, T, st));
        TL_PROPAGATE(linear(xn_, w.w1, g_, T, cfg_.hidden_dim, dim, st));
        TL_PROPAGATE(launch_silu(g_, g_, (size_t)T * cfg_.hidden_dim, cfg_.silu_via_float, st));
        TL_PROPAGATE(linear(xn_, w.w3, u_, T, cfg_.hidden_dim, dim, st));
        TL_PROPAGATE(launch_binary(g_, g_, u_, (size_t)T * cfg_.hidden_dim, 1, st));
        TL_PROPAGATE(linear(g_, w.w2, ao_, T, dim, cfg_.hidden_dim, st));
        TL_PROPAGATE(launch_binary(x_, h_, ao_, (size_t)T * dim, 0, st));
    }
    launches_ += 1;
    const int t0 = all_logits ? 0 : T - 1, tn = all_logits ? T : 1;
    TL_PROPAGATE(launch_rmsnorm_seq(xn_ + (size_t)t0 * dim, x_ + (size_t)t0 * dim, final_norm_, 1e-5f, dim, tn, st));
    const __half* cls = shared_classifier_ ? emb_ : wcls_;
    return linear(xn_ + (size_t)t0 * dim, cls, logits_ + (size_t)t0 * cfg_.vocab_size, tn, cfg_.vocab_size, dim, st);
}

// Multi-token pass, fast numerics. With 32-column-aligned shapes the operators next to a matmul run
// in its epilogue: [norm] [wq|wk|wv + RoPE + KV-cache write] [attention] [wo + residual] [norm]
// [w1|w3 + SiLU*up] [w2 + residual] = 7 launches per layer (+1 for the V transpose the fused
// attention reads). Other shapes (and the K-split matmuls under tensor parallelism, which need the
// allreduce between matmul and residual) take the operator-by-operator sequence.
int Llama2Engine::forward_fast_prefill(int T, int pos, bool all_logits, cudaStream_t st) {
    const int dim = cfg_.dim, S = pos + T, H = H_local_, dl = dim_local_, hl = hidden_local_;
    const float scale = 1.0f / sqrtf((float)hd_);
    // up to 128 rows the matmuls are bound by the weight stream and run on the skinny kernel
    const bool fused = T > 128 && tensor_map_encode_available() && hd_ % 32 == 0 && dl % 64 == 0 && hl % 32 == 0 &&
                       dim % 32 == 0;
    const bool fused_residual = fused && coll_ == nullptr;
    // Tensor parallel with the exchange region open: the K-split matmuls push their partial rows to the ranks
    // that own them and the owner's add + RMSNorm kernel hands the normalised rows to every rank
    // (tp_prefill.cu); no collective library call in the layer loop. TL_TP_PREFILL=nccl keeps the allreduce form.
    const int world = cfg_.tp_world;
    static const bool force_nccl = [] { const char* e = getenv("TL_TP_PREFILL"); return e && !strcmp(e, "nccl"); }();
    const bool tp_fused = fused && coll_ != nullptr && xch_ready_ && !force_nccl && T % (128 * world) == 0 && dim <= 8192 &&
                          (world == 2 || world == 4 || world == 8) &&
                          T / world <= pf_rpo_max_;
    const int rpo = tp_fused ? T / world : 0, row0 = cfg_.tp_rank * rpo;
    __half* xn = tp_fused ? reinterpret_cast<__half*>(xch_base_ + pf_off_xn_) : xn_;
    // TL_PREFILL_TIMING=<layer>: stage-by-stage device times of that layer on stderr (the event records
    // serialise the stages, so the sum exceeds the layer's share of an untimed run)
    static const int timing_layer = [] { const char* e = getenv("TL_PREFILL_TIMING"); return e ? atoi(e) : -1; }();
    std::vector<std::pair<const char*, cudaEvent_t>> marks;
    bool timing = false;
    auto mark = [&](const char* name) {
        if (!timing) return;
        cudaEvent_t e; cudaEventCreate(&e); cudaEventRecord(e, st); marks.emplace_back(name, e);
    };
    auto exchange = [&](const __half* A, const __half* Wk, int K, const __half* resid, __half* resid_out, const __half* norm_w) -> int {
        // one fused compute + collective: push GEMM, owner-side reduce + norm + gather, wait for every owner's rows
        HgemmPush push{};
        push.world = world; push.rows_per_owner = rpo; push.epoch = ++pf_epoch_;
        const size_t fslot = (size_t)(pf_rpo_max_ / 128) * 64;
        for (int d = 0; d < world; d++)
            push.flags[d] = reinterpret_cast<unsigned int*>(xch_peer_[d] + pf_off_aflags_) + (size_t)cfg_.tp_rank * fslot;
        int col_tiles = 0;
        launches_ += 3;
        TL_PROPAGATE(launch_hgemm_push(A, Wk, reinterpret_cast<__half*>(xch_base_ + pf_off_recv_), T, dim, K, K, K, push, &col_tiles, st));
        TpReduceNorm rn{};
        rn.world = world; rn.rank = cfg_.tp_rank; rn.rows = rpo; rn.row0 = row0; rn.dim = dim; rn.col_tiles = col_tiles; rn.epoch = push.epoch;
        for (int d = 0; d < world; d++) rn.partial[d] = reinterpret_cast<const __half*>(xch_peer_[d] + pf_off_recv_);
        rn.arrive_flags = reinterpret_cast<const unsigned int*>(xch_base_ + pf_off_aflags_); rn.flags_slot_stride = (int)fslot;
        rn.residual = resid + (size_t)row0 * dim; rn.residual_out = resid_out + (size_t)row0 * dim;
        rn.norm_w = norm_w; rn.eps = 1e-5f;
        for (int d = 0; d < world; d++) {
            rn.xn_dst[d] = reinterpret_cast<__half*>(xch_peer_[d] + pf_off_xn_);
            rn.owner_done[d] = reinterpret_cast<unsigned int*>(xch_peer_[d] + pf_off_gflags_);
        }
        mark("  k-split matmul");
        rn.rows_done = reinterpret_cast<unsigned int*>(xch_base_ + pf_off_gflags_) + 64;
        TL_PROPAGATE(launch_tp_reduce_norm(rn, st));
        mark("  owner reduce + norm + gather");
        TL_PROPAGATE(launch_tp_wait_owners(reinterpret_cast<const unsigned int*>(xch_base_ + pf_off_gflags_), world, push.epoch, st));
        mark("  wait for all owners");
        return TL_OK;
    };
    if (tp_fused) TL_PROPAGATE(align_ranks(st));
    launches_++;
    TL_PROPAGATE(launch_embedding(x_, emb_, d_tokens_, T, dim, cfg_.vocab_size, st));
    for (int l = 0; l < cfg_.n_layers; l++) {
        const LayerWeights& w = layers_[l];
        timing = l == timing_layer && T > 128;
        mark("start");
        // (under the fused exchange the norm of layers > 0 was applied by the owner of each row at the end of the previous layer)
        if (!tp_fused || l == 0) TL_PROPAGATE(launch_rmsnorm_fast(xn, x_, w.attn_norm, 1e-5f, dim, T, st));
        if (fused) {
            launches_ += 2;
            const size_t half_hd = (size_t)hd_ / 2;
            TL_PROPAGATE(launch_hgemm_qkv_rope(xn, w.wq, w.wk, w.wv, q_, w.cache_k + (size_t)pos * dl,
                                               w.cache_v + (size_t)pos * dl, T, dl, dim, dim, dim, dl, dl,
                                               cos_t_ + (size_t)pos * half_hd, sin_t_ + (size_t)pos * half_hd, hd_, st));
        } else {
            launches_ += 5;   // linear() counts its own launches
            TL_PROPAGATE(linear(xn, w.wq, q_, T, dl, dim, st));
            TL_PROPAGATE(linear(xn, w.wk, k_, T, dl, dim, st));
            TL_PROPAGATE(linear(xn, w.wv, v_, T, dl, dim, st));
            TL_PROPAGATE(launch_rope(q_, q_, pos, T, T, H, hd_, cos_t_, sin_t_, st));
            TL_PROPAGATE(launch_rope(k_, k_, pos, T, T, H, hd_, cos_t_, sin_t_, st));
            TL_PROPAGATE(launch_copy_rows(w.cache_k + (size_t)pos * dl, k_, T, dl, dl, st));
            TL_PROPAGATE(launch_copy_rows(w.cache_v + (size_t)pos * dl, v_, T, dl, dl, st));
        }
        mark("norm + qkv + rope");
        // scores[h] = q_h . K_h^T ; softmax (scale + causal mask inside) ; att_h = P_h . V_h
        if (flash_prefill_supported(q_, w.cache_k, w.cache_v, att_, T, S, pos, H, hd_, dl, dl, dl, dl)) {
            // one kernel, scores stay in tensor memory / registers, K and V read in place from the caches
            launches_ += 1;
            TL_PROPAGATE(launch_flash_prefill(q_, w.cache_k, w.cache_v, att_, T, S, pos, H, hd_, dl, dl, dl, dl, st));
        } else if (hgemm_supported(q_, w.cache_k, scores_, T, S, hd_, dl, dl, S) &&
                   hgemm_supported(scores_, vt_, att_, T, hd_, S, S, S, dl)) {
            launches_ += 4;
            TL_PROPAGATE(launch_hgemm(q_, w.cache_k, scores_, H, T, S, hd_, dl, dl, S, hd_, hd_, (long long)T * S, st));
            TL_PROPAGATE(launch_softmax_causal_fast(scores_, H, T, S, pos, scale, st));
            TL_PROPAGATE(launch_transpose_v(vt_, w.cache_v, S, H, hd_, dl, S, st));
            TL_PROPAGATE(launch_hgemm(scores_, vt_, att_, H, T, hd_, S, S, S, dl, (long long)T * S, (long long)hd_ * S, hd_, st));
        } else {
            launches_ += 3;
            SeqMatmul qk{q_, w.cache_k, scores_, H, T, S, hd_, dl, 1, dl, 1, S, hd_, hd_, (long long)T * S};
            TL_PROPAGATE(launch_matmul_seq(qk, st));
            TL_PROPAGATE(launch_softmax_causal_fast(scores_, H, T, S, pos, scale, st));
            SeqMatmul pv{scores_, w.cache_v, att_, H, T, hd_, S, S, 1, 1, dl, dl, (long long)T * S, hd_, hd_};
            TL_PROPAGATE(launch_matmul_seq(pv, st));
        }
        mark("attention");
        if (tp_fused) {
            TL_PROPAGATE(exchange(att_, w.wo, dl, x_, h_, w.ffn_norm));          // h = x + wo(att); xn = norm(h) * ffn_norm
        } else if (fused_residual) {
            launches_++;
            TL_PROPAGATE(launch_hgemm_residual(att_, w.wo, x_, h_, T, dim, dl, dl, dl, dim, dim, st, true));
        } else {
            launches_++;
            TL_PROPAGATE(linear(att_, w.wo, ao_, T, dim, dl, st));
            if (coll_) TL_PROPAGATE(coll_->allreduce_sum_f16(ao_, (size_t)T * dim, st));
            TL_PROPAGATE(launch_binary(h_, x_, ao_, (size_t)T * dim, 0, st));
        }
        mark("wo + exchange + residual");
        if (!tp_fused) {
            launches_++;
            TL_PROPAGATE(launch_rmsnorm_fast(xn, h_, w.ffn_norm, 1e-5f, dim, T, st));
        }
        if (fused) {
            launches_++;
            TL_PROPAGATE(launch_hgemm_swiglu(xn, w.w1, w.w3, g_, T, hl, dim, dim, dim, hl, st));
        } else {
            launches_++;
            TL_PROPAGATE(linear(xn, w.w1, g_, T, hl, dim, st));
            TL_PROPAGATE(linear(xn, w.w3, u_, T, hl, dim, st));
            TL_PROPAGATE(launch_swiglu_fast(g_, g_, u_, (size_t)T * hl, st));
        }
        mark("norm + gate/up");
        if (tp_fused) {
            const __half* next_norm = l + 1 < cfg_.n_layers ? layers_[l + 1].attn_norm : final_norm_;
            TL_PROPAGATE(exchange(g_, w.w2, hl, h_, x_, next_norm));             // x = h + w2(g); xn = norm(x) * next norm
        } else if (fused_residual) {
            launches_++;
            TL_PROPAGATE(launch_hgemm_residual(g_, w.w2, h_, x_, T, dim, hl, hl, hl, dim, dim, st, true));
        } else {
            launches_++;
            TL_PROPAGATE(linear(g_, w.w2, ao_, T, dim, hl, st));
            if (coll_) TL_PROPAGATE(coll_->allreduce_sum_f16(ao_, (size_t)T * dim, st));
            TL_PROPAGATE(launch_binary(x_, h_, ao_, (size_t)T * dim, 0, st));
        }
        mark("w2 + exchange + residual");
        if (timing && !marks.empty()) {
            cudaStreamSynchronize(st);
            for (size_t i = 1; i < marks.size(); i++) {
                float ms = 0.f;
                cudaEventElapsedTime(&ms, marks[i - 1].second, marks[i].second);
                fprintf(stderr, "[prefill timing rank %d layer %d T %d] %-34s %8.1f us\n", cfg_.tp_rank, l, T, marks[i].first, ms * 1e3f);
            }
            for (auto& m : marks) cudaEventDestroy(m.second);
            marks.clear();
        }
    }
    timing = false;
    launches_ += 1;
    const int t0 = all_logits ? 0 : T - 1, tn = all_logits ? T : 1;
    // (fused exchange: the last layer's owner-side kernel already applied the final norm to every row)
    if (!tp_fused) TL_PROPAGATE(launch_rmsnorm_fast(xn + (size_t)t0 * dim, x_ + (size_t)t0 * dim, final_norm_, 1e-5f, dim, tn, st));
    const __half* cls = (shared_classifier_ && cfg_.tp_world == 1) ? emb_ : wcls_;
    if (cfg_.tp_world == 1)
        return linear(xn + (size_t)t0 * dim, cls, logits_ + (size_t)t0 * cfg_.vocab_size, tn, cfg_.vocab_size, dim, st);
    // vocabulary-split classifier: local slice, then gather the slices of every rank
    for (int t = t0; t < t0 + tn; t++) {
        TL_PROPAGATE(linear(xn + (size_t)t * dim, cls, cls_local_, 1, vocab_local_, dim, st));
        TL_PROPAGATE(coll_->allgather_f16(cls_local_, logits_ + (size_t)t * cfg_.vocab_size, vocab_local_, st));
    }
    return TL_OK;
}

// One decode step, fast numerics, 5 kernels per layer:
//   [RMSNorm + wq|wk|wv GEMV + RoPE + KV-cache write] -> [attention over the cache in place] ->
//   [wo GEMV + residual] -> [RMSNorm + w1|w3 GEMV + SiLU*up] -> [w2 GEMV + residual]
// then [RMSNorm + classifier GEMV] -> argmax -> advance. Token and position are read from device
// memory so the same launches can be replayed from a CUDA graph.
// ---- fused tensor-parallel exchange -----------------------------------------------------------------
namespace {
// greedy sampling over logits that the ranks pushed slice by slice as (two fp16 logits, epoch)
// words: wait (bounded) for every word of this step, unpack into the plain logits row, then the
// usual lowest-index argmax
__global__ void k_argmax_after_exchange(int* out_idx, const unsigned long long* words, __half* logits, int cols,
                                        const unsigned int* step_ptr, int phases_per_step, int phase_id, int* status) {
    __shared__ float sv[32];
    __shared__ int si[32];
    const unsigned int epoch = __ldcg(step_ptr) * (unsigned)phases_per_step + (unsigned)phase_id + 1u;
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    bool timed_out = false;
    for (int j = threadIdx.x; 2 * j < cols; j += blockDim.x) {
        unsigned int data = 0, flag = 0;
        bool here = false;
        for (unsigned i = 0; i < 2 * TL_EXCHANGE_TRIES && !here; i++) {
            asm volatile("ld.volatile.global.v2.u32 {%0, %1}, [%2];" : "=r"(data), "=r"(flag) : "l"(words + j) : "memory");
            here = flag == epoch;
        }
        timed_out |= !here;
        *reinterpret_cast<unsigned int*>(logits + 2 * j) = data;
        const __half2 h = *reinterpret_cast<const __half2*>(&data);
        const float v0 = __low2float(h), v1 = __high2float(h);
        if (bi == 0x7fffffff || v0 > bv) { bv = v0; bi = 2 * j; }
        if (2 * j + 1 < cols && v1 > bv) { bv = v1; bi = 2 * j + 1; }
    }
    if (timed_out) atomicExch(status, TL_ERR_TIMEOUT);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
    }
    if ((threadIdx.x & 31) == 0) { sv[threadIdx.x >> 5] = bv; si[threadIdx.x >> 5] = bi; }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < (int)(blockDim.x >> 5); w++)
            if (sv[w] > bv || (sv[w] == bv && si[w] < bi)) { bv = sv[w]; bi = si[w]; }
        out_idx[0] = bi == 0x7fffffff ? 0 : bi;
    }
}
__global__ void k_advance_tp(int* pos, const int* next, int* generated, int max_seq, unsigned int* step) {
    int p = *pos;
    if (p >= 0 && p < max_seq) generated[p] = *next;
    *pos = p + 1;
    *step = *step + 1;
}
}  // namespace

int Llama2Engine::xch_export(cudaIpcMemHandle_t* out) {
    TL_REQUIRE(out && cfg_.tp_world > 1 && cfg_.tp_world <= TL_MAX_TP, "exchange needs 2..%d ranks", TL_MAX_TP);
    TL_REQUIRE(vocab_local_ % 2 == 0 && cfg_.dim % 8 == 0, "exchange needs an even vocabulary slice and dim %% 8 == 0");
    if (!xch_base_) {
        const size_t dim = cfg_.dim, W = cfg_.tp_world;
        size_t off = 0;
        auto take = [&](size_t bytes) { size_t o = off; off = (off + bytes + 255) & ~(size_t)255; return o; };
        // every payload travels as an 8-byte (payload, epoch) word
        xch_off_part_[0] = take(W * dim * sizeof(unsigned long long));
        xch_off_part_[1] = take(W * dim * sizeof(unsigned long long));
        xch_off_logits_ = take(((size_t)cfg_.vocab_size / 2 + 1) * sizeof(unsigned long long));
        // local only: the reduced vector of each exchange, published once per GPU as (two halfs, epoch) words
        xch_off_pub_[0] = take(dim / 2 * sizeof(unsigned long long));
        xch_off_pub_[1] = take(dim / 2 * sizeof(unsigned long long));
        xch_off_step_ = take(sizeof(unsigned int));
        // prefill: this rank's partial result of a K-split matmul [max_seq][dim] (fetched by the row owners), the gathered normalised
        // rows [max_seq][dim], arrival flags [source][row block][64 column tiles], gather flags [max_seq]
        const size_t S = cfg_.max_seq_len;
        pf_rpo_max_ = (int)(((S + W - 1) / W + 127) / 128 * 128);
        pf_off_recv_ = take(S * dim * sizeof(__half));
        pf_off_xn_ = take(S * dim * sizeof(__half));
        pf_off_aflags_ = take(W * (size_t)(pf_rpo_max_ / 128) * 64 * sizeof(unsigned int));
        pf_off_gflags_ = take(128 * sizeof(unsigned int));   // [0, world): owner flags; [64]: this rank's finished-row counter
        xch_bytes_ = off;
        void* d = nullptr;
        TL_CUDA(cudaMalloc(&d, xch_bytes_));
        TL_CUDA(cudaMemset(d, 0, xch_bytes_));
        TL_CUDA(cudaDeviceSynchronize());
        allocs_.push_back(d);
        xch_base_ = static_cast<unsigned char*>(d);
    }
    TL_CUDA(cudaIpcGetMemHandle(out, xch_base_));
    return TL_OK;
}

int Llama2Engine::xch_open(const cudaIpcMemHandle_t* handles, int world) {
    TL_REQUIRE(handles && world == cfg_.tp_world && xch_base_, "exchange: export first, then open with %d handles", cfg_.tp_world);
    for (int r = 0; r < world; r++) {
        if (r == cfg_.tp_rank) { xch_peer_[r] = xch_base_; continue; }
        void* p = nullptr;
        TL_CUDA(cudaIpcOpenMemHandle(&p, handles[r], cudaIpcMemLazyEnablePeerAccess));
        xch_peer_[r] = static_cast<unsigned char*>(p);
    }
    if (decode_graph_) { cudaGraphExecDestroy(decode_graph_); decode_graph_ = nullptr; }
    xch_ready_ = true;
    return TL_OK;
}

int Llama2Engine::xch_close() {
    if (!xch_ready_) return TL_OK;
    cudaDeviceSynchronize();
    if (decode_graph_) { cudaGraphExecDestroy(decode_graph_); decode_graph_ = nullptr; }
    for (int r = 0; r < cfg_.tp_world; r++)
        if (r != cfg_.tp_rank && xch_peer_[r]) cudaIpcCloseMemHandle(xch_peer_[r]);
    xch_ready_ = false;
    return TL_OK;
}

// buf 0: wo partials, 1: w2 partials (fp32, dim per rank); 2: classifier slices (fp16, vocab/world per rank)
PeerExchange Llama2Engine::make_exchange(int buf, int phase_id) const {
    PeerExchange e{};
    e.world = cfg_.tp_world; e.rank = cfg_.tp_rank;
    // words per rank slot: one per fp32 partial sum, one per pair of fp16 logits
    const size_t slot_words = buf < 2 ? (size_t)cfg_.dim : (size_t)vocab_local_ / 2;
    const size_t base_off = buf < 2 ? xch_off_part_[buf] : xch_off_logits_;
    e.n = buf < 2 ? cfg_.dim : vocab_local_;
    e.local_slots = reinterpret_cast<const unsigned long long*>(xch_base_ + base_off);
    e.local_pub = buf < 2 ? reinterpret_cast<unsigned long long*>(xch_base_ + xch_off_pub_[buf]) : nullptr;
    for (int d = 0; d < e.world; d++)
        e.peer_slot[d] = reinterpret_cast<unsigned long long*>(xch_peer_[d] + base_off) + (size_t)e.rank * slot_words;
    e.step_ptr = reinterpret_cast<const unsigned int*>(xch_base_ + xch_off_step_);
    e.phases_per_step = 2 * cfg_.n_layers + 1;
    e.phase_id = phase_id;
    // up to four ranks every CTA sums the slots itself (at most 128 KB of L2 reads per CTA, one on-chip hop fewer:
    // 1.656 against ~1.70 ms per token at two GPUs, 1.319 against 1.346 at four); TL_TP_REDUCE=direct|slice overrides
    static const int forced = [] { const char* v = getenv("TL_TP_REDUCE"); return !v ? 0 : (!strcmp(v, "direct") ? 1 : (!strcmp(v, "slice") ? 2 : 0)); }();
    e.direct = forced == 1 || (forced == 0 && e.world <= 4) ? 1 : 0;
    return e;
}

// The tensor-parallel decode step with the exchanges fused into the GEMV kernels: same five
// kernels per layer as on one GPU, no collective launches. wo and w2 push fp32 partial sums to
// every rank; the next GEMV's prologue waits for all ranks, sums in rank order and adds the
// residual. The classifier pushes its logit slice; the sampling kernel waits for all slices.
int Llama2Engine::decode_step_tp_fused(cudaStream_t st, bool pdl) {
    const int dim = cfg_.dim, dl = dim_local_, hl = hidden_local_, L = cfg_.n_layers;
    long long n = 0;
    // Three launches per layer: [attention] [wo -> exchange -> norm + w1|w3 + SiLU*up] [w2 -> exchange ->
    // norm + next layer's wq|wk|wv + RoPE + KV write]; the last pair ends in the classifier instead.
    // prof_ (tl_llama2_decode_profile): three %globaltimer stamps per GEMV phase, in launch order.
    unsigned long long* prof = prof_;
    auto next_prof = [&]() { unsigned long long* p = prof; if (prof) prof += 3; return p; };
    auto qkv_phase = [&](int l, FusedGemv& a, PeerExchange& in) {
        const LayerWeights& w = layers_[l];
        a.x = x_; a.norm_w = w.attn_norm; a.eps = 1e-5f;
        a.W[0] = w.wq; a.W[1] = w.wk; a.W[2] = w.wv; a.n_mats = 3; a.N_each = dl; a.K = dim;
        a.epilogue = EPI_QKV_ROPE; a.y = q_; a.k_out = w.cache_k; a.v_out = w.cache_v;
        a.cos_row = cos_t_; a.sin_row = sin_t_; a.head_dim = hd_; a.pos_ptr = d_pos_; a.kv_pitch = dl;
        a.pdl = pdl;
        if (l > 0) {  // x = h + sum of the previous layer's w2 partials
            in = make_exchange(1, 2 * (l - 1) + 1);
            in.residual = h_; in.sum_out = x_;
            a.xin = &in;
        }
    };
    TL_PROPAGATE(launch_embedding(x_, emb_, d_next_, 1, dim, cfg_.vocab_size, st)); n++;
    {
        FusedGemv a{}; PeerExchange in{};
        qkv_phase(0, a, in);
        a.prof = next_prof();
        TL_PROPAGATE(launch_fused_gemv(a, st)); n++;
    }
    for (int l = 0; l < L; l++) {
        const LayerWeights& w = layers_[l];
        DecodeAttn at{q_, w.cache_k, w.cache_v, att_, attn_scratch_, attn_counters_, H_local_, hd_, 0,
                      attn_splits_, d_pos_, dl, pdl};
        TL_PROPAGATE(launch_decode_attn_cluster(at, st)); n++;

        PeerExchange out_wo = make_exchange(0, 2 * l), in_wo = make_exchange(0, 2 * l);
        in_wo.residual = x_; in_wo.sum_out = h_;
        FusedGemv o{}, f{};
        o.x = att_; o.W[0] = w.wo; o.n_mats = 1; o.N_each = dim; o.K = dl; o.pdl = pdl;
        o.epilogue = EPI_PUSH_F32; o.xout = &out_wo; o.prof = next_prof();
        f.x = x_; f.norm_w = w.ffn_norm; f.eps = 1e-5f; f.xin = &in_wo;
        f.W[0] = w.w1; f.W[1] = w.w3; f.n_mats = 2; f.N_each = hl; f.K = dim;
        f.epilogue = EPI_SWIGLU; f.y = g_; f.pdl = pdl; f.prof = next_prof();
        TL_PROPAGATE(launch_fused_gemv_pair(o, f, st)); n++;

        PeerExchange out_w2 = make_exchange(1, 2 * l + 1), in_next{}, out_cls{};
        FusedGemv d{}, c{};
        d.x = g_; d.W[0] = w.w2; d.n_mats = 1; d.N_each = dim; d.K = hl; d.pdl = pdl;
        d.epilogue = EPI_PUSH_F32; d.xout = &out_w2; d.prof = next_prof();
        if (l + 1 < L) {
            qkv_phase(l + 1, c, in_next);
        } else {
            in_next = make_exchange(1, 2 * (L - 1) + 1);
            in_next.residual = h_; in_next.sum_out = x_;
            out_cls = make_exchange(2, 2 * L);
            c.x = x_; c.norm_w = final_norm_; c.eps = 1e-5f; c.xin = &in_next;
            c.W[0] = wcls_; c.n_mats = 1; c.N_each = vocab_local_; c.K = dim; c.epilogue = EPI_PUSH_F16; c.xout = &out_cls;
            c.pdl = pdl;
        }
        c.prof = next_prof();
        TL_PROPAGATE(launch_fused_gemv_pair(d, c, st)); n++;
    }
    const PeerExchange out_cls = make_exchange(2, 2 * L);
    k_argmax_after_exchange<<<1, 1024, 0, st>>>(d_next_, out_cls.local_slots, logits_, cfg_.vocab_size, out_cls.step_ptr,
                                                out_cls.phases_per_step, out_cls.phase_id, device_status_word()); n++;
    TL_LAUNCH_CHECK();
    k_advance_tp<<<1, 1, 0, st>>>(d_pos_, d_next_, d_generated_, cfg_.max_seq_len,
                                  reinterpret_cast<unsigned int*>(xch_base_ + xch_off_step_)); n++;
    TL_LAUNCH_CHECK();
    last_logits_ = logits_;
    decode_step_launches_ = n;
    launches_ += n;
    return TL_OK;
}

int Llama2Engine::decode_step_fast(cudaStream_t st, bool pdl) {
    if (xch_ready_) return decode_step_tp_fused(st, pdl);
    const int dim = cfg_.dim, dl = dim_local_, hl = hidden_local_;
    long long n = 0;
    last_logits_ = logits_;
    unsigned long long* prof = prof_;
    auto next_prof = [&]() { unsigned long long* p = prof; if (prof) prof += 3; return p; };
    TL_PROPAGATE(launch_embedding(x_, emb_, d_next_, 1, dim, cfg_.vocab_size, st)); n++;
    for (int l = 0; l < cfg_.n_layers; l++) {
        const LayerWeights& w = layers_[l];
        FusedGemv a{};
        a.x = x_; a.norm_w = w.attn_norm; a.eps = 1e-5f;
        a.W[0] = w.wq; a.W[1] = w.wk; a.W[2] = w.wv; a.n_mats = 3; a.N_each = dl; a.K = dim;
        a.epilogue = EPI_QKV_ROPE; a.y = q_; a.k_out = w.cache_k; a.v_out = w.cache_v;
        a.cos_row = cos_t_; a.sin_row = sin_t_; a.head_dim = hd_; a.pos_ptr = d_pos_; a.kv_pitch = dl;
        a.pdl = pdl; a.prof = next_prof();
        TL_PROPAGATE(launch_fused_gemv(a, st)); n++;

        DecodeAttn at{q_, w.cache_k, w.cache_v, att_, attn_scratch_, attn_counters_, H_local_, hd_, 0,
                      attn_splits_, d_pos_, dl, pdl};
        TL_PROPAGATE(launch_decode_attn_cluster(at, st)); n++;

        FusedGemv o{};
        o.x = att_; o.W[0] = w.wo; o.n_mats = 1; o.N_each = dim; o.K = dl; o.pdl = pdl; o.prof = next_prof();
        if (coll_) {
            o.epilogue = EPI_STORE_F32; o.y32 = ao32_;
            TL_PROPAGATE(launch_fused_gemv(o, st)); n++;
            TL_PROPAGATE(coll_->allreduce_sum_f32(ao32_, dim, st)); n++;
            TL_PROPAGATE(launch_residual_add_f32(h_, x_, ao32_, dim, st)); n++;
        } else {
            o.epilogue = EPI_RESIDUAL; o.y = h_; o.residual = x_;
            TL_PROPAGATE(launch_fused_gemv(o, st)); n++;
        }

        FusedGemv f{};
        f.x = h_; f.norm_w = w.ffn_norm; f.eps = 1e-5f;
        f.W[0] = w.w1; f.W[1] = w.w3; f.n_mats = 2; f.N_each = hl; f.K = dim;
        f.epilogue = EPI_SWIGLU; f.y = g_; f.pdl = pdl; f.prof = next_prof();
        TL_PROPAGATE(launch_fused_gemv(f, st)); n++;

        FusedGemv d{};
        d.x = g_; d.W[0] = w.w2; d.n_mats = 1; d.N_each = dim; d.K = hl; d.pdl = pdl; d.prof = next_prof();
        if (coll_) {
            d.epilogue = EPI_STORE_F32; d.y32 = ao32_;
            TL_PROPAGATE(launch_fused_gemv(d, st)); n++;
            TL_PROPAGATE(coll_->allreduce_sum_f32(ao32_, dim, st)); n++;
            TL_PROPAGATE(launch_residual_add_f32(x_, h_, ao32_, dim, st)); n++;
        } else {
            d.epilogue = EPI_RESIDUAL; d.y = x_; d.residual = h_;
            TL_PROPAGATE(launch_fused_gemv(d, st)); n++;
        }
    }
    FusedGemv c{};
    c.x = x_; c.norm_w = final_norm_; c.eps = 1e-5f;
    c.W[0] = (shared_classifier_ && cfg_.tp_world == 1) ? emb_ : wcls_;
    c.n_mats = 1; c.N_each = vocab_local_; c.K = dim; c.epilogue = EPI_STORE; c.pdl = pdl; c.prof = next_prof();
    if (coll_) {
        c.y = cls_local_;
        TL_PROPAGATE(launch_fused_gemv(c, st)); n++;
        TL_PROPAGATE(coll_->allgather_f16(cls_local_, logits_, vocab_local_, st)); n++;
    } else {
        c.y = logits_;
        TL_PROPAGATE(launch_fused_gemv(c, st)); n++;
    }
    TL_PROPAGATE(launch_argmax(d_next_, logits_, 1, cfg_.vocab_size, st)); n++;
    k_advance<<<1, 1, 0, st>>>(d_pos_, d_next_, d_generated_, cfg_.max_seq_len); n++;
    TL_LAUNCH_CHECK();
    decode_step_launches_ = n;
    launches_ += n;
    return TL_OK;
}

int Llama2Engine::sample_last(int T, cudaStream_t st) {
    launches_++;
    (void)T;
    return launch_argmax(d_next_, last_logits_, 1, cfg_.vocab_size, st);
}

int Llama2Engine::ensure_decode_graph(cudaStream_t st) {
    if (decode_graph_) return TL_OK;
    TL_REQUIRE(cfg_.numerics == TL_NUMERICS_FAST, "the decode graph exists for fast numerics only");
    if (use_mega()) return ensure_mega();  // the one-kernel step needs no graph
    TL_REQUIRE(!coll_ || coll_->graph_capturable(), "collective is not capturable");
    TL_PROPAGATE(ensure_activations(1, 0));
    cudaStream_t cap = st;
    bool own = false;
    if (cap == nullptr) {  // the legacy default stream cannot be captured
        TL_CUDA(cudaStreamCreateWithFlags(&cap, cudaStreamNonBlocking));
        own = true;
    }
    cudaGraph_t graph = nullptr;
    const long long before = launches_;
    TL_CUDA(cudaStreamBeginCapture(cap, cudaStreamCaptureModeThreadLocal));
    int rc = decode_step_fast(cap, true);
    cudaError_t e = cudaStreamEndCapture(cap, &graph);
    launches_ = before;  // capture enqueues nothing
    if (own) cudaStreamDestroy(cap);
    if (rc != TL_OK) { if (graph) cudaGraphDestroy(graph); return rc; }
    if (e != cudaSuccess) return set_error(TL_ERR_CUDA, "graph capture failed: %s", cudaGetErrorString(e));
    e = cudaGraphInstantiate(&decode_graph_, graph, 0);
    cudaGraphDestroy(graph);
    if (e != cudaSuccess) { decode_graph_ = nullptr; return set_error(TL_ERR_CUDA, "graph instantiate failed: %s", cudaGetErrorString(e)); }
    return TL_OK;
}

// Set-up of the one-kernel decode step: the per-layer weight table, the word vectors the phases hand
// to one another, the sampling scratch. Under tensor parallelism the exchange region must be open.
int Llama2Engine::ensure_mega() {
    if (mega_ready_) return TL_OK;
    TL_PROPAGATE(ensure_activations(1, 0));
    TL_REQUIRE(vocab_local_ % 2 == 0 && cfg_.dim % 16 == 0 && dim_local_ % 16 == 0 && hidden_local_ % 16 == 0,
               "one-kernel decode needs an even vocabulary slice and widths that are multiples of 16");
    TL_REQUIRE(cfg_.tp_world == 1 || xch_ready_, "one-kernel decode under tensor parallelism needs the fused exchange (tl_tp_exchange_open)");
    const int dim = cfg_.dim, dl = dim_local_, hl = hidden_local_;
    std::vector<FlowLayer> lay(cfg_.n_layers);
    for (int l = 0; l < cfg_.n_layers; l++) {
        const LayerWeights& w = layers_[l];
        lay[l] = FlowLayer{w.attn_norm, w.wq, w.wk, w.wv, w.wo, w.ffn_norm, w.w1, w.w3, w.w2, w.cache_k, w.cache_v};
    }
    mega_grid_ = sm_count();
    if (!mega_phases_) {
        TL_CUDA(cudaMalloc(&mega_phases_, lay.size() * sizeof(FlowLayer)));
        allocs_.push_back(mega_phases_);
        // words: x, h [dim]; q, k, v, att [dl]; g [hl]; then the sampling candidates, their counter and the step counter
        const size_t n_words = 2 * (size_t)dim + 4 * (size_t)dl + (size_t)hl;
        const size_t bytes = n_words * sizeof(unsigned int) + 256 + (size_t)mega_grid_ * sizeof(unsigned long long) + 256;
        void* d = nullptr;
        TL_CUDA(cudaMalloc(&d, bytes));
        TL_CUDA(cudaMemset(d, 0, bytes));
        allocs_.push_back(d);
        flow_words_ = static_cast<unsigned int*>(d);
        unsigned char* tail = reinterpret_cast<unsigned char*>(flow_words_ + n_words);
        tail = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(tail) + 255) & ~(uintptr_t)255);
        flow_cand_ = reinterpret_cast<unsigned long long*>(tail);
        flow_counters_ = reinterpret_cast<unsigned int*>(tail + (size_t)mega_grid_ * sizeof(unsigned long long));
    }
    TL_CUDA(cudaMemcpy(mega_phases_, lay.data(), lay.size() * sizeof(FlowLayer), cudaMemcpyHostToDevice));
    const int max_k = std::max(std::max(dim, dl), hl);
    mega_smem_ = mega_smem_bytes(max_k);
    mega_x_bytes_ = mega_x_bytes(max_k);
    TL_REQUIRE(mega_smem_ <= 227 * 1024, "decode step kernel needs %d bytes of shared memory", mega_smem_);
    mega_splits_ = 16;    // scratch slots per head: the kernel picks ceil(context / 128) splits, at most 16
    if (!mega_attn_scratch_) {
        void* d = nullptr;
        TL_CUDA(cudaMalloc(&d, (size_t)H_local_ * 16 * (hd_ + 2) * sizeof(float)));
        allocs_.push_back(d);
        mega_attn_scratch_ = static_cast<float*>(d);
    }
    mega_n_phases_ = flow_phases(cfg_.n_layers);
    mega_ready_ = true;
    return TL_OK;
}

int Llama2Engine::decode_profile(int start_pos, int cta, unsigned long long* out_host, int capacity, int* n_phases) {
    TL_REQUIRE(out_host && n_phases, "null argument");
    TL_PROPAGATE(align_ranks(nullptr));
    if (!use_mega()) {
        // the step as plain launches (programmatic dependent launch, no graph), CTA 0 of every GEMV phase stamping
        // %globaltimer at its first instruction, when its activation vector is staged and when it is done
        TL_REQUIRE(cfg_.numerics == TL_NUMERICS_FAST, "phase timestamps exist for fast numerics only");
        const int phases = 4 * cfg_.n_layers + 1;   // GEMV phases in launch order: qkv, wo, gate/up, w2 per layer, then the classifier (attention is not stamped)
        TL_REQUIRE(capacity >= 3 * phases, "timestamp buffer needs %d entries", 3 * phases);
        TL_PROPAGATE(ensure_activations(1, 0));
        unsigned long long* d = nullptr;
        TL_CUDA(cudaMalloc(&d, (size_t)3 * phases * sizeof(unsigned long long)));
        TL_CUDA(cudaMemset(d, 0, (size_t)3 * phases * sizeof(unsigned long long)));
        TL_CUDA(cudaMemcpy(d_pos_, &start_pos, sizeof(int), cudaMemcpyHostToDevice));
        prof_ = d;
        int rc = decode_step_fast(nullptr, true);
        prof_ = nullptr;
        if (rc == TL_OK && cudaMemcpy(out_host, d, (size_t)3 * phases * sizeof(unsigned long long), cudaMemcpyDeviceToHost) != cudaSuccess)
            rc = set_error(TL_ERR_CUDA, "timestamp copy failed");
        cudaFree(d);
        *n_phases = phases;
        return rc;
    }
    TL_PROPAGATE(ensure_mega());
    TL_REQUIRE(capacity >= 3 * mega_n_phases_, "timestamp buffer needs %d entries", 3 * mega_n_phases_);
    unsigned long long* d = nullptr;
    TL_CUDA(cudaMalloc(&d, (size_t)3 * mega_n_phases_ * sizeof(unsigned long long)));
    TL_CUDA(cudaMemcpy(d_pos_, &start_pos, sizeof(int), cudaMemcpyHostToDevice));
    int rc = decode_step_mega(nullptr, d, cta);
    if (rc == TL_OK && cudaMemcpy(out_host, d, (size_t)3 * mega_n_phases_ * sizeof(unsigned long long), cudaMemcpyDeviceToHost) != cudaSuccess)
        rc = set_error(TL_ERR_CUDA, "timestamp copy failed");
    cudaFree(d);
    *n_phases = mega_n_phases_;
    return rc;
}

int Llama2Engine::decode_step_mega(cudaStream_t st, unsigned long long* prof, int prof_cta) {
    FlowArgs a{};
    a.prof = prof; a.prof_cta = prof_cta;
    last_logits_ = logits_;
    const int dim = cfg_.dim, dl = dim_local_, hl = hidden_local_;
    a.layers = static_cast<const FlowLayer*>(mega_phases_); a.n_layers = cfg_.n_layers;
    a.emb = emb_; a.final_norm = final_norm_;
    a.wcls = (shared_classifier_ && cfg_.tp_world == 1) ? emb_ : wcls_;
    a.dim = dim; a.dl = dl; a.hl = hl; a.vocab = cfg_.vocab_size; a.vocab_local = vocab_local_;
    a.H = H_local_; a.hd = hd_; a.splits = mega_splits_; a.max_seq = cfg_.max_seq_len;
    unsigned int* w = flow_words_;
    a.w.x = w; w += dim; a.w.h = w; w += dim;
    a.w.q = w; w += dl; a.w.k = w; w += dl; a.w.v = w; w += dl; a.w.att = w; w += dl;
    a.w.g = w;
    a.attn_scratch = mega_attn_scratch_; a.attn_counters = attn_counters_;
    a.cos_t = cos_t_; a.sin_t = sin_t_; a.silu_tab = tables().silu_float_tab;
    a.logits = logits_; a.cand = flow_cand_; a.cand_counter = flow_counters_;
    a.d_next = d_next_; a.d_pos = d_pos_; a.d_generated = d_generated_;
    a.step = flow_counters_ + 1;
    a.status = device_status_word(); a.eps = 1e-5f; a.x_bytes = mega_x_bytes_;
    a.world = cfg_.tp_world; a.rank = cfg_.tp_rank;
    a.exchange_tries = TL_EXCHANGE_TRIES;
    if (cfg_.tp_world > 1) {
        TL_REQUIRE(xch_ready_, "one-kernel decode under tensor parallelism needs the fused exchange");
        a.step = reinterpret_cast<unsigned int*>(xch_base_ + xch_off_step_);     // the counter every rank advances in step
        for (int buf = 0; buf < 2; buf++) {
            a.local_part[buf] = reinterpret_cast<const unsigned long long*>(xch_base_ + xch_off_part_[buf]);
            for (int d = 0; d < cfg_.tp_world; d++)
                a.peer_part[buf][d] = reinterpret_cast<unsigned long long*>(xch_peer_[d] + xch_off_part_[buf]) + (size_t)cfg_.tp_rank * dim;
        }
        a.local_logits = reinterpret_cast<const unsigned long long*>(xch_base_ + xch_off_logits_);
        for (int d = 0; d < cfg_.tp_world; d++)
            a.peer_logits[d] = reinterpret_cast<unsigned long long*>(xch_peer_[d] + xch_off_logits_) + (size_t)cfg_.tp_rank * (vocab_local_ / 2);
    }
    launches_ += 1;
    return launch_decode_flow(a, mega_grid_, mega_smem_, st);
}

// The waits of the fused exchange are bounded (about two seconds), the skew between the ranks' host threads is
// not: a tiny allreduce through the collective library, which waits as long as it takes, lines the ranks up
// before a call enters the kernels that wait for one another. Once per call, never inside the layer loop.
int Llama2Engine::align_ranks(cudaStream_t st) {
    if (!coll_ || !xch_ready_) return TL_OK;
    if (!align_buf_) {
        void* d = nullptr;
        TL_CUDA(cudaMalloc(&d, 256));
        TL_CUDA(cudaMemset(d, 0, 256));
        allocs_.push_back(d);
        align_buf_ = static_cast<__half*>(d);
    }
    return coll_->allreduce_sum_f16(align_buf_, 8, st);
}

int Llama2Engine::decode_steps(int start_pos, int steps, cudaStream_t st) {
    TL_REQUIRE(steps >= 0 && start_pos >= 0 && start_pos + steps <= cfg_.max_seq_len,
               "decode: positions [%d,%d) exceed max_seq_len=%d", start_pos, start_pos + steps, cfg_.max_seq_len);
    TL_CUDA(cudaMemcpyAsync(d_pos_, &start_pos, sizeof(int), cudaMemcpyHostToDevice, st));
    if (use_mega()) {
        // single GPU: the whole step is one persistent kernel
        TL_PROPAGATE(ensure_mega());
        for (int i = 0; i < steps; i++) TL_PROPAGATE(decode_step_mega(st));
        return TL_OK;
    }
    if (cfg_.numerics == TL_NUMERICS_FAST) {
        TL_PROPAGATE(ensure_decode_graph(st));
        for (int i = 0; i < steps; i++) {
            TL_CUDA(cudaGraphLaunch(decode_graph_, st));
            launches_ += decode_step_launches_;
        }
        return TL_OK;
    }
    // reference-order numerics: plain launches, token fed back on the device
    for (int i = 0; i < steps; i++) {
        TL_CUDA(cudaMemcpyAsync(d_tokens_, d_next_, sizeof(int), cudaMemcpyDeviceToDevice, st));
        TL_PROPAGATE(forward(1, start_pos + i, false, st));
        TL_PROPAGATE(sample_last(1, st));
        k_advance<<<1, 1, 0, st>>>(d_pos_, d_next_, d_generated_, cfg_.max_seq_len);
        TL_LAUNCH_CHECK();
        launches_++;
    }
    return TL_OK;
}

}  // namespace tlb
