// C++ host mirror of the reference's user-visible API for the matmul -> Llama2 forward path, over
// the C ABI of tensorlib_b200.h. Header-only, C++17, no CUDA headers needed by the includer.
//
//   reference (DavidZyy/tensorLib)                              here (namespace tlb200)
//   Tensor<half>::matmul(other, result_opt)   Tensor.hpp:90     Tensor::matmul(other, result_opt)
//   Tensor<half>::transpose(0, 1) view        Tensor.cpp:277+   Tensor::transpose()  (last two dims)
//   nn::Linear<half>::forward(x, result_opt)  nn/linear.hpp:13  nn::Linear::forward(x, result_opt)
//   ModelArgs                                 Transformer.hpp:13 ModelArgs
//   Transformer<half>::forward(tokens, start_pos, buf)  Transformer.hpp:80
//                                                               Transformer::forward(tokens, start_pos)
//   Llama2<half>::generate(prompt_tokens)     llama2.hpp:19     Llama2::generate(prompt_tokens, max_new)
//   Tokenizer::encode / decode                Tokenizer.hpp:33  Tokenizer::encode / decode (host only)
//   Llama2<half>::text_completion(prompt)     llama2.hpp:20     Llama2::text_completion(tokenizer, prompt)
//   Llama2<half>::chat()                      llama2.hpp:21     Llama2::chat(tokenizer, in, out)
//
// Error behaviour follows the reference: argument/shape errors throw std::invalid_argument
// (matmul.cpp:209-221); CUDA failures, which the reference answers with exit(1) (CUDA.cuh:131-151),
// throw tlb200::Error so that an embedding application can decide.
// Tensors live in device memory ("cuda" is the only device type: there is no CPU path).
#pragma once

#include <cstdint>
#include <cstdio>
#include <fstream>
#include <istream>
#include <ostream>
#include <memory>
#include <optional>
#include <stdexcept>
#include <string>
#include <unordered_map>
#include <vector>

#include "tensorlib_b200.h"

namespace tlb200 {

class Error : public std::runtime_error {
public:
    Error(int status, const std::string& what) : std::runtime_error(what), status(status) {}
    int status;
};

inline void check(int status) {
    if (status == TL_OK) return;
    const std::string msg = tl_last_error();
    if (status == TL_ERR_INVALID_ARGUMENT) throw std::invalid_argument(msg);
    throw Error(status, msg);
}

inline void init(int device = 0) { check(tl_init(device)); }

// fp16 tensor in device memory: contiguous row-major storage, plus an optional "last two
// dimensions swapped" view (what the reference's transpose(0,1) of a 2-D weight produces).
class Tensor {
public:
    Tensor() = default;
    explicit Tensor(const std::vector<int>& shape) : shape_(shape) {
        void* p = nullptr;
        check(tl_malloc(&p, bytes()));
        data_ = std::shared_ptr<void>(p, [](void* q) { tl_free(q); });
    }
    // copy `numel()` fp16 values (raw 16-bit patterns) from host memory
    Tensor(const std::vector<int>& shape, const uint16_t* host) : Tensor(shape) {
        check(tl_memcpy_h2d(data_.get(), host, bytes(), nullptr));
        check(tl_stream_synchronize(nullptr));
    }
    const std::vector<int>& shape() const { return shape_; }
    size_t numel() const {
        size_t n = 1;
        for (int d : shape_) n *= (size_t)d;
        return n;
    }
    size_t bytes() const { return numel() * sizeof(uint16_t); }
    tl_half* data() const { return static_cast<tl_half*>(data_.get()); }
    bool is_transposed_view() const { return transposed_; }
    std::vector<uint16_t> to_host() const {
        if (transposed_) throw std::invalid_argument("to_host: make the view contiguous first");
        std::vector<uint16_t> out(numel());
        check(tl_memcpy_d2h(out.data(), data_.get(), bytes(), nullptr));
        check(tl_stream_synchronize(nullptr));
        return out;
    }
    // view with the last two dimensions swapped; shares storage (Tensor.cpp:277-304)
    Tensor transpose() const {
        if (shape_.size() < 2) throw std::invalid_argument("transpose: needs at least 2 dimensions");
        Tensor v = *this;
        std::swap(v.shape_[v.shape_.size() - 1], v.shape_[v.shape_.size() - 2]);
        v.transposed_ = !transposed_;
        return v;
    }
    // this: (..., M, K) contiguous; other: a transposed view of (..., N, K) storage, i.e. logical
    // (..., K, N) — the form every matmul on the Llama2 path has (Linear: x . W^T,
    // attention: q . k^T). Leading dimensions of `other` broadcast when it has none.
    // result_opt: caller-owned output of shape (..., M, N), returned (Tensor.hpp:90).
    Tensor matmul(const Tensor& other, std::optional<Tensor> result_opt = std::nullopt,
                  int numerics = TL_NUMERICS_FAST) const {
        if (transposed_) throw std::invalid_argument("matmul: left operand must be contiguous");
        if (!other.transposed_)
            throw std::invalid_argument("matmul: right operand must be a transposed view of (N, K) row-major storage");
        if (shape_.size() < 2 || other.shape_.size() < 2) throw std::invalid_argument("matmul: operands need 2 dimensions");
        const size_t M = (size_t)shape_[shape_.size() - 2], K = (size_t)shape_.back();
        const size_t Kb = (size_t)other.shape_[other.shape_.size() - 2], N = (size_t)other.shape_.back();
        if (K != Kb) throw std::invalid_argument("matmul: inner dimensions differ");   // matmul.cpp:209-221
        size_t batch = 1, batch_b = 1;
        for (size_t i = 0; i + 2 < shape_.size(); i++) batch *= (size_t)shape_[i];
        for (size_t i = 0; i + 2 < other.shape_.size(); i++) batch_b *= (size_t)other.shape_[i];
        if (batch_b != 1 && batch_b != batch) throw std::invalid_argument("matmul: batch dimensions do not broadcast");
        std::vector<int> out_shape(shape_.begin(), shape_.end() - 1);
        out_shape.push_back((int)N);
        Tensor out = result_opt ? *result_opt : Tensor(out_shape);
        if (out.transposed_ || out.numel() != batch * M * N) throw std::invalid_argument("matmul: result has the wrong size");
        check(tl_matmul_batched_f16(data(), other.data(), out.data(), batch, M, N, K, K, K, N, M * K,
                                    batch_b == 1 ? 0 : N * K, M * N, numerics, nullptr));
        out.shape_ = out_shape;
        return out;
    }

private:
    std::vector<int> shape_;
    std::shared_ptr<void> data_;
    bool transposed_ = false;
};

namespace nn {
// weight [out_features, in_features] as in the checkpoint (linear.cpp:10-14)
class Linear {
public:
    Linear() = default;
    Linear(int in_features, int out_features, Tensor weight)
        : in_features(in_features), out_features(out_features), weight(std::move(weight)) {
        if (this->weight.shape() != std::vector<int>{out_features, in_features})
            throw std::invalid_argument("Linear: weight must be (out_features, in_features)");
    }
    // x.matmul(weight.transpose(0, 1), result_opt)   (linear.cpp:43-49)
    Tensor forward(const Tensor& input, std::optional<Tensor> result_opt = std::nullopt) const {
        return input.matmul(weight.transpose(), std::move(result_opt));
    }
    int in_features = 0, out_features = 0;
    Tensor weight;
};
}  // namespace nn

struct ModelArgs {          // Transformer.hpp:13-24
    int dim = 0, hidden_dim = 0, n_layers = 0, n_heads = 0, vocab_size = 0, n_kv_heads = 0;
    int max_batch_size = 1, max_seq_len = 0;
};

// Llama2 decoder. forward() takes token ids on the host and returns the logits of every position
// (T, vocab) on the host, like the reference's Transformer::forward followed by the caller's copy
// (Transformer.cpp:264-299); activation buffers are owned by the model, not passed in.
class Transformer {
public:
    explicit Transformer(const ModelArgs& args, int numerics = TL_NUMERICS_FAST, bool silu_via_float = true) : args(args) {
        tl_llama2_config c{};
        c.dim = args.dim; c.hidden_dim = args.hidden_dim; c.n_layers = args.n_layers; c.n_heads = args.n_heads;
        c.n_kv_heads = args.n_kv_heads ? args.n_kv_heads : args.n_heads; c.vocab_size = args.vocab_size;
        c.max_seq_len = args.max_seq_len; c.numerics = numerics; c.silu_via_float = silu_via_float ? 1 : 0;
        c.tp_rank = 0; c.tp_world = 1; c.one_kernel_decode = 0;
        tl_llama2* h = nullptr;
        check(tl_llama2_create(&c, &h));
        handle_ = std::shared_ptr<tl_llama2>(h, [](tl_llama2* q) { tl_llama2_destroy(q); });
    }
    // read_checkpoint + read_weights (main.cpp:195-228, :36-190): a llama2.c file, header included
    void load_checkpoint(const std::string& path) { check(tl_llama2_load_file(handle_.get(), path.c_str())); }
    std::vector<uint16_t> forward(const std::vector<int>& tokens, int start_pos) const {
        std::vector<uint16_t> logits(tokens.size() * (size_t)args.vocab_size);
        check(tl_llama2_forward(handle_.get(), tokens.data(), (int)tokens.size(), start_pos,
                                reinterpret_cast<tl_half*>(logits.data()), nullptr));
        return logits;
    }
    tl_llama2* handle() const { return handle_.get(); }
    ModelArgs args;

private:
    std::shared_ptr<tl_llama2> handle_;
};

// Byte-pair tokenizer over a llama2.c `tokenizer.bin` (int32 max_token_length, then per entry:
// float score, int32 length, bytes), the format and algorithm of the reference's Tokenizer
// (model/llama2_7b/src/Tokenizer.cpp, itself a restatement of llama2.c's): optional BOS (id 1), a
// " " prefix token for non-empty text, one lookup per UTF-8 code point with byte fallback (byte + 3),
// then repeatedly merging the adjacent pair whose concatenation has the highest score; optional
// EOS (id 2). Host only. Two deliberate differences from the reference: decode() does not edit
// the vocabulary in place (Tokenizer.cpp:155-167 assigns through a reference, so a piece decoded
// once after BOS loses its leading space for good), and an empty token list does not underflow
// the merge loop's bound (Tokenizer.cpp:131).
class Tokenizer {
public:
    Tokenizer(const std::string& tokenizer_file, int vocab_size) : vocab_(vocab_size), scores_(vocab_size) {
        std::ifstream f(tokenizer_file, std::ios::binary);
        if (!f) throw std::runtime_error("couldn't load " + tokenizer_file);
        int32_t max_len = 0;
        f.read(reinterpret_cast<char*>(&max_len), sizeof max_len);
        for (int i = 0; i < vocab_size; i++) {
            int32_t len = 0;
            f.read(reinterpret_cast<char*>(&scores_[i]), sizeof(float));
            f.read(reinterpret_cast<char*>(&len), sizeof len);
            if (!f || len < 0 || len > (1 << 20)) throw std::runtime_error("tokenizer file is truncated or corrupt");
            vocab_[i].resize((size_t)len);
            f.read(&vocab_[i][0], len);
            if (!f) throw std::runtime_error("tokenizer file is truncated");
            index_.emplace(vocab_[i], i);          // first id wins for a repeated piece
        }
    }
    int vocab_size() const { return (int)vocab_.size(); }

    std::vector<int> encode(const std::string& text, bool bos, bool eos) const {
        std::vector<int> tokens;
        if (bos) tokens.push_back(1);
        if (!text.empty()) {
            const int space = lookup(" ");
            if (space < 0) throw std::invalid_argument("tokenizer vocabulary has no \" \" piece");
            tokens.push_back(space);
        }
        std::string cp;                               // bytes of the current code point
        for (size_t i = 0; i < text.size(); i++) {
            const unsigned char c = (unsigned char)text[i];
            if ((c & 0xC0) != 0x80) cp.clear();       // a lead byte starts a new code point
            cp.push_back((char)c);
            const unsigned char next = i + 1 < text.size() ? (unsigned char)text[i + 1] : 0;
            if ((next & 0xC0) == 0x80 && cp.size() < 4) continue;
            const int id = lookup(cp);
            if (id >= 0) tokens.push_back(id);
            else for (unsigned char b : cp) tokens.push_back((int)b + 3);
            cp.clear();
        }
        while (tokens.size() >= 2) {
            float best_score = -1e10f;
            int best_id = -1;
            size_t best_at = 0;
            for (size_t i = 0; i + 1 < tokens.size(); i++) {
                const int id = lookup(vocab_[(size_t)tokens[i]] + vocab_[(size_t)tokens[i + 1]]);
                if (id >= 0 && scores_[(size_t)id] > best_score) { best_score = scores_[(size_t)id]; best_id = id; best_at = i; }
            }
            if (best_id < 0) break;
            tokens[best_at] = best_id;
            tokens.erase(tokens.begin() + (long)best_at + 1);
        }
        if (eos) tokens.push_back(2);
        return tokens;
    }

    // the text of `token` given its predecessor: no leading space right after BOS; <0xHH> pieces
    // are the raw byte (byte 0 decodes to the empty string, as a C string would)
    std::string decode(int prev_token, int token) const {
        if (token < 0 || token >= (int)vocab_.size()) throw std::invalid_argument("token id out of range");
        std::string piece = vocab_[(size_t)token];
        if (prev_token == 1 && !piece.empty() && piece[0] == ' ') piece.erase(0, 1);
        unsigned int byte = 0;
        int digits = 0;
        if (piece.size() >= 4 && piece.compare(0, 3, "<0x") == 0) {
            for (size_t i = 3; i < piece.size() && digits < 2; i++, digits++) {
                const char ch = piece[i];
                const int v = ch >= '0' && ch <= '9' ? ch - '0' : ch >= 'a' && ch <= 'f' ? ch - 'a' + 10 : ch >= 'A' && ch <= 'F' ? ch - 'A' + 10 : -1;
                if (v < 0) break;
                byte = byte * 16 + (unsigned)v;
            }
        }
        if (digits > 0) return byte == 0 ? std::string() : std::string(1, (char)byte);
        return piece;
    }

private:
    int lookup(const std::string& s) const {
        auto it = index_.find(s);
        return it == index_.end() ? -1 : it->second;
    }
    std::vector<std::string> vocab_;
    std::vector<float> scores_;
    std::unordered_map<std::string, int> index_;
};

struct GenerateResult {
    std::vector<int> tokens;          // generated ids (without the prompt)
    double prefill_seconds = 0, decode_seconds = 0;
    double tokens_per_second() const { return decode_seconds > 0 ? (tokens.size() - 1) / decode_seconds : 0; }
};

// Llama2::generate (llama2.cpp:15-101): prefill, then greedy steps; stops early on id 1 or 2 when
// stop_on_eos is set (llama2.cpp:88-91); text_completion and the chat loop sit on top of it.
class Llama2 {
public:
    Llama2(const ModelArgs& args, const std::string& checkpoint_path, int numerics = TL_NUMERICS_FAST)
        : model(args, numerics) {
        model.load_checkpoint(checkpoint_path);
    }
    GenerateResult generate(const std::vector<int>& prompt_tokens, int max_new = 256, bool stop_on_eos = true) {
        GenerateResult r;
        r.tokens.resize((size_t)max_new);
        int n_out = 0;
        check(tl_llama2_generate(model.handle(), prompt_tokens.data(), (int)prompt_tokens.size(), max_new,
                                 stop_on_eos ? 1 : 0, r.tokens.data(), &n_out, &r.prefill_seconds, &r.decode_seconds));
        r.tokens.resize((size_t)n_out);
        return r;
    }
    // Llama2::text_completion (llama2.cpp:104-107): encode with BOS, generate, decode piece by piece
    std::string text_completion(const Tokenizer& tokenizer, const std::string& prompt, int max_new = 256) {
        const std::vector<int> ids = tokenizer.encode(prompt, true, false);
        const GenerateResult r = generate(ids, max_new, true);
        std::string out;
        int prev = ids.empty() ? 1 : ids.back();
        for (int t : r.tokens) {
            if (t == 1 || t == 2) break;
            out += tokenizer.decode(prev, t);
            prev = t;
        }
        return out;
    }
    // One turn continuing at position `start_pos` over the KV cache of earlier turns (the reference keeps that
    // position in the global total_len, llama2.cpp:13, :51-52, :79).
    GenerateResult generate_at(int start_pos, const std::vector<int>& prompt_tokens, int max_new = 256, bool stop_on_eos = true) {
        GenerateResult r;
        r.tokens.resize((size_t)max_new);
        int n_out = 0;
        check(tl_llama2_generate_at(model.handle(), start_pos, prompt_tokens.data(), (int)prompt_tokens.size(), max_new,
                                    stop_on_eos ? 1 : 0, r.tokens.data(), &n_out, &r.prefill_seconds, &r.decode_seconds));
        r.tokens.resize((size_t)n_out);
        return r;
    }
    // Llama2::chat (llama2.cpp:119-146): every line read from `in` is one user turn (at most 511 characters, the
    // reference's buffer), rendered as "[INST] %s [/INST]", encoded with BOS and answered by a generation that
    // continues at the running position, so earlier turns stay in the KV cache; every piece is written to `out` as
    // decode(-1, token), like the reference prints it. A turn generates at most 1 + 256 tokens (the reference's
    // first token from the prefill and generate_len = 256 steps) and stops on id 1 or 2. The reference loops for
    // ever; this loop ends at end of input or when the context cannot hold another turn. Returns the turns answered.
    int chat(const Tokenizer& tokenizer, std::istream& in, std::ostream& out, int max_new = 257) {
        int turns = 0;
        std::string line;
        while (true) {
            out << "> " << std::flush;
            if (!std::getline(in, line)) break;
            if (line.size() > 511) line.resize(511);
            const std::vector<int> ids = tokenizer.encode("[INST] " + line + " [/INST]", true, false);
            const int room = model.args.max_seq_len - total_len_ - (int)ids.size();     // positions left after the prompt
            if (ids.empty() || room < 0) break;
            const GenerateResult r = generate_at(total_len_, ids, max_new < room + 1 ? max_new : room + 1, true);
            total_len_ += (int)ids.size() + (int)r.tokens.size() - 1;                 // one decode step per token after the first
            for (int t : r.tokens) {
                if (t == 1 || t == 2) break;
                out << tokenizer.decode(-1, t) << std::flush;
            }
            out << std::endl;
            turns++;
        }
        return turns;
    }
    int total_len() const { return total_len_; }
    Transformer model;

private:
    int total_len_ = 0;     // running position of chat(): prompt and generated tokens of all turns so far
};

}  // namespace tlb200
