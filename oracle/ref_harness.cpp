// TEST INFRASTRUCTURE — not part of the product.
//
// C entry points around the UNMODIFIED reference sources (compiled where they lie, see
// oracle/Makefile). Every arithmetic step below is executed by the reference's own classes on
// "cpu" tensors; this file only holds
//   * pointer-in / pointer-out wrappers so Python tests can drive single operators, and
//   * the ~40 lines of block/model glue of the reference's Llama2 forward that cannot be used as
//     shipped on "cpu":
//       - TransformerBlock::forward (model/llama2_7b/src/Transformer.cpp:162-178) discards the
//         return value of RMSNorm::forward, and RMSNorm::forward_plain
//         (tensorLib/src/nn/rmsNorm.cpp:37-56) ignores result_opt, so activation_buffer.x_norm is
//         never written on "cpu". The glue here stores the norm result into x_norm.
//       - FeedForward::forward (Transformer.cpp:133-145) uses the fp16 SiLU of the CPU backend,
//         which evaluates 1/(1+exp(x)) (tensorLib/src/device/cpu/CPU.cpp:216-219) instead of
//         1/(1+exp(-x)) (CPU.cpp:220-222 for float, tensorLib/src/device/cuda/CUDA.cu:334-342 for
//         every dtype). silu_mode 0 ("A") keeps that as is; silu_mode 1 ("B") takes SiLU through
//         the reference's own float route (Tensor<float>(x).silu() -> Tensor<half>), which is the
//         formula and the single rounding of the reference's CUDA kernel.
// Everything else (Attention::forward, Linear::forward, Embedding::forward, get_mask, argmax) is
// called unchanged.
#include "Tensor.hpp"
// The reference defines the Attention / FeedForward / TransformerBlock member templates in
// Transformer.cpp and instantiates only Transformer<half> explicitly, so their symbols are not
// reliably exported by that object file. The file is therefore compiled as part of this
// translation unit, from where it lies in the reference tree (oracle/Makefile passes its folder
// with -I); nothing of it is copied.
#include "Transformer.cpp"
#include "nn/linear.hpp"
#include "nn/rmsNorm.hpp"
#include "nn/embedding.hpp"
#include "device/cpu/CPU.hpp"

#include <cstdint>
#include <cstring>
#include <exception>
#include <memory>
#include <string>
#include <vector>
#include <omp.h>
#include <cuda_runtime.h>
#include "device/cuda/CUDA.cuh"

namespace {

thread_local std::string g_err;

template <typename F>
int guarded(F&& f) {
    try {
        f();
        return 0;
    } catch (const std::exception& e) {
        g_err = e.what();
        return 1;
    } catch (...) {
        g_err = "unknown exception";
        return 1;
    }
}

Tensor<half> make_tensor(const std::vector<int>& shape, const uint16_t* src) {
    Tensor<half> t(shape, "cpu");
    if (src) std::memcpy(t.device->getDataPtr(), src, sizeof(half) * (size_t)t.num_elements);
    return t;
}

void copy_out(const Tensor<half>& t, uint16_t* dst) {
    Tensor<half> c = t.contiguous();
    std::memcpy(dst, c.device->getDataPtr() + c.offset_, sizeof(half) * (size_t)c.num_elements);
}

struct RefModel {
    ModelArgs args;
    std::unique_ptr<Transformer<half>> model;
};

void set_weight(Tensor<half>& w, const uint16_t* src, size_t n) {
    std::memcpy(w.device->getDataPtr(), src, n * sizeof(half));
}

}  // namespace

extern "C" {

const char* ref_last_error() { return g_err.c_str(); }

int ref_omp_max_threads() { return omp_get_max_threads(); }
void ref_omp_set_threads(int n) { omp_set_num_threads(n); }

// Device<half>::matmul2d on the CPU backend (tensorLib/src/device/cpu/CPU.cpp:76-89).
int ref_matmul2d_f16(const uint16_t* A, const uint16_t* B, uint16_t* C, int M, int N, int K) {
    return guarded([&] {
        CPU<half> dev;  // no storage of its own: matmul2d only uses its arguments
        dev.matmul2d(reinterpret_cast<const half*>(A), reinterpret_cast<const half*>(B),
                     reinterpret_cast<half*>(C), (size_t)M, (size_t)N, (size_t)K);
    });
}

// Device<half>::matmul, the strided batched form (CPU.cpp:18-68), on the reference's CPU device object.
int ref_matmul_strided_f16(const uint16_t* lhs, const uint16_t* rhs, uint16_t* result, const int* lhs_stride,
                           const int* rhs_stride, size_t lhs_offset, size_t rhs_offset, const int* result_shape, int ndim,
                           size_t result_elements, size_t K) {
    return guarded([&] {
        CPU<half> dev;
        dev.matmul(reinterpret_cast<const half*>(lhs), reinterpret_cast<const half*>(rhs), reinterpret_cast<half*>(result),
                   std::vector<int>(lhs_stride, lhs_stride + ndim), std::vector<int>(rhs_stride, rhs_stride + ndim), lhs_offset,
                   rhs_offset, std::vector<int>(result_shape, result_shape + ndim), result_elements, K);
    });
}

// nn::Linear<half>::forward == x.matmul(W.transpose(0,1)) through Tensor::matmul / call2
// (tensorLib/src/nn/linear.cpp:43-49, tensorLib/src/ops/matmul.cpp:206-324). x is (1,T,in).
int ref_linear_f16(const uint16_t* x, const uint16_t* W, uint16_t* y, int T, int in_f, int out_f) {
    return guarded([&] {
        nn::Linear<half> lin(in_f, out_f, "cpu");
        set_weight(lin.weight, W, (size_t)in_f * out_f);
        Tensor<half> xt = make_tensor({1, T, in_f}, x);
        Tensor<half> out = lin.forward(xt);
        copy_out(out, y);
    });
}

// Batched Tensor<half>::matmul: a is (B,M,K), b is (B,K,N) given as its (B,N,K) storage, i.e.
// the call is a.matmul(bt.transpose(1,2)). Exercises the per-batch loop of call2.
int ref_bmm_nt_f16(const uint16_t* a, const uint16_t* bt, uint16_t* c, int B, int M, int N, int K) {
    return guarded([&] {
        Tensor<half> at = make_tensor({B, M, K}, a);
        Tensor<half> btt = make_tensor({B, N, K}, bt);
        Tensor<half> out = at.matmul(btt.transpose(1, 2));
        copy_out(out, c);
    });
}

// nn::RMSNorm<half>::forward_plain (tensorLib/src/nn/rmsNorm.cpp:15-56). x is (1,T,dim).
int ref_rmsnorm_f16(const uint16_t* x, const uint16_t* w, uint16_t* y, int T, int dim, float eps) {
    return guarded([&] {
        nn::RMSNorm<half> norm(dim, eps, "cpu");
        set_weight(norm.weight, w, (size_t)dim);
        Tensor<half> xt = make_tensor({1, T, dim}, x);
        Tensor<half> out = norm.forward_plain(xt);
        copy_out(out, y);
    });
}

// apply_rotary_emb (tensorLib/include/Tensor.hpp:427-466 -> CPU.cpp:427-461). x is (1,T,H,hd).
int ref_rope_f16(const uint16_t* x, uint16_t* y, int start_pos, int T, int H, int hd) {
    return guarded([&] {
        Tensor<half> xt = make_tensor({1, T, H, hd}, x);
        Tensor<half> out = apply_rotary_emb(xt, start_pos);
        copy_out(out, y);
    });
}

// Tensor<half>::softmax over the last dim (tensorLib/src/device/cpu/softmax.cpp:10-31).
int ref_softmax_f16(const uint16_t* x, uint16_t* y, int rows, int cols) {
    return guarded([&] {
        Tensor<half> xt = make_tensor({rows, cols}, x);
        Tensor<half> out = xt.softmax(1);
        copy_out(out, y);
    });
}

// SiLU. via_float == 0: Tensor<half>::silu as is (CPU.cpp:216-219, sign defect).
// via_float == 1: Tensor<half>(Tensor<float>(x).silu()) (CPU.cpp:220-222, Tensor.hpp:289-312).
int ref_silu_f16(const uint16_t* x, uint16_t* y, int n, int via_float) {
    return guarded([&] {
        Tensor<half> xt = make_tensor({n}, x);
        if (via_float) {
            Tensor<float> xf(xt);
            Tensor<float> sf = xf.silu();
            Tensor<half> out(sf);
            copy_out(out, y);
        } else {
            Tensor<half> out = xt.silu();
            copy_out(out, y);
        }
    });
}

// Binary / scalar elementwise ops used by the forward: 0 add, 1 mul, 2 scalar-div.
int ref_ewise_f16(const uint16_t* a, const uint16_t* b, uint16_t* y, int n, int op, double scalar) {
    return guarded([&] {
        Tensor<half> at = make_tensor({n}, a);
        Tensor<half> out;
        if (op == 0) {
            Tensor<half> bt = make_tensor({n}, b);
            out = at.EwiseAdd(bt);
        } else if (op == 1) {
            Tensor<half> bt = make_tensor({n}, b);
            out = at.EwiseMul(bt);
        } else {
            out = at.ScalarDiv(scalar);  // double -> half conversion of the scalar, as at Transformer.cpp:94
        }
        copy_out(out, y);
    });
}

// Tensor<half>::argmax(-1) (CPU.cpp:358-372): strict '>' so the lowest index wins ties.
int ref_argmax_f16(const uint16_t* x, int* idx, int rows, int cols) {
    return guarded([&] {
        Tensor<half> xt = make_tensor({rows, cols}, x);
        Tensor<int> out = xt.argmax(-1, false);
        std::memcpy(idx, out.device->getDataPtr(), sizeof(int) * (size_t)rows);
    });
}

// ---------------------------------------------------------------------------------------------
// The rest of the Device<half> surface, straight on the reference's CPU<half> device object
// (tensorLib/include/device/cpu/CPU.hpp): the virtuals a Tensor<half> program ends up calling.
// ---------------------------------------------------------------------------------------------
namespace {
std::vector<int> ivec(const int* p, int n) { return std::vector<int>(p, p + n); }
}

int ref_contiguous_f16(uint16_t* result, const uint16_t* data, size_t data_elems, const int* shape, const int* stride,
                       int ndim, size_t offset, size_t n) {
    return guarded([&] {
        CPU<half> dev(data_elems);
        std::memcpy(dev.getDataPtr(), data, data_elems * sizeof(half));
        dev.contiguous(reinterpret_cast<half*>(result), ivec(shape, ndim), ivec(stride, ndim), offset, n);
    });
}
// value_or_src: a pointer to n source values (scalar == 0) or to one value (scalar != 0); `data` is updated in place
int ref_set_item_f16(uint16_t* data, size_t data_elems, const uint16_t* value_or_src, int scalar, const int* shape,
                     const int* stride, int ndim, size_t offset, size_t n) {
    return guarded([&] {
        CPU<half> dev(data_elems);
        std::memcpy(dev.getDataPtr(), data, data_elems * sizeof(half));
        if (scalar) {
            half v;
            std::memcpy(&v, value_or_src, sizeof v);
            dev.setItemScalar(v, ivec(shape, ndim), ivec(stride, ndim), offset, n);
        } else {
            std::vector<half> src(n);
            std::memcpy(src.data(), value_or_src, n * sizeof(half));
            dev.setItemEwise(src.data(), ivec(shape, ndim), ivec(stride, ndim), offset, n);
        }
        std::memcpy(data, dev.getDataPtr(), data_elems * sizeof(half));
    });
}
// op codes: TL_UNARY_* of include/tensorlib_b200.h. Inputs that make the reference throw inside its
// OpenMP loop (sqrt / rsqrt of a value <= 0) must not be passed: that ends the process.
int ref_unary_f16(const uint16_t* x, uint16_t* y, int n, int op) {
    return guarded([&] {
        if (op == 7) {                      // SiLU through the float route, as ref_silu_f16 does
            Tensor<half> xt = make_tensor({n}, x);
            Tensor<float> xf(xt);
            Tensor<half> out(xf.silu());
            copy_out(out, y);
            return;
        }
        CPU<half> dev((size_t)n);
        std::memcpy(dev.getDataPtr(), x, (size_t)n * sizeof(half));
        half* r = reinterpret_cast<half*>(y);
        switch (op) {
            case 0: dev.neg(r, n); break;
            case 1: dev.sin(r, n); break;
            case 2: dev.cos(r, n); break;
            case 3: dev.exp(r, n); break;
            case 4: dev.log(r, n); break;
            case 5: dev.abs(r, n); break;
            case 6: dev.tanh(r, n); break;
            case 8: dev.sqrt(r, n); break;
            case 9: dev.rsqrt(r, n); break;
            case 10: dev.silu(r, n); break;
            default: throw std::invalid_argument("unknown unary op");
        }
    });
}
// 0 add, 1 sub, 2 mul, 3 div (no zero divisors: see above), 4 pow (scalar only)
int ref_binary_f16(const uint16_t* a, const uint16_t* b, uint16_t* y, int n, int op) {
    return guarded([&] {
        CPU<half> dev((size_t)n);
        std::memcpy(dev.getDataPtr(), a, (size_t)n * sizeof(half));
        std::vector<half> other(n);
        std::memcpy(other.data(), b, (size_t)n * sizeof(half));
        half* r = reinterpret_cast<half*>(y);
        switch (op) {
            case 0: dev.add(r, other.data(), n); break;
            case 1: dev.sub(r, other.data(), n); break;
            case 2: dev.mul(r, other.data(), n); break;
            case 3: dev.div(r, other.data(), n); break;
            default: throw std::invalid_argument("unknown binary op");
        }
    });
}
int ref_binary_scalar_f16(const uint16_t* a, uint16_t s, uint16_t* y, int n, int op) {
    return guarded([&] {
        CPU<half> dev((size_t)n);
        std::memcpy(dev.getDataPtr(), a, (size_t)n * sizeof(half));
        half v;
        std::memcpy(&v, &s, sizeof v);
        half* r = reinterpret_cast<half*>(y);
        switch (op) {
            case 0: dev.add(r, v, n); break;
            case 1: dev.sub(r, v, n); break;
            case 2: dev.mul(r, v, n); break;
            case 3: dev.div(r, v, n); break;
            case 4: dev.pow(r, v, n); break;
            default: throw std::invalid_argument("unknown binary op");
        }
    });
}
int ref_reduce_f16(const uint16_t* x, uint16_t* y, size_t reduce_size, size_t n, int op) {
    return guarded([&] {
        CPU<half> dev(n);
        std::memcpy(dev.getDataPtr(), x, n * sizeof(half));
        half* r = reinterpret_cast<half*>(y);
        switch (op) {
            case 0: dev.max(r, reduce_size, n); break;
            case 1: dev.min(r, reduce_size, n); break;
            case 2: dev.sum(r, reduce_size, n); break;
            case 3: dev.mean(r, reduce_size, n); break;
            default: throw std::invalid_argument("unknown reduce op");
        }
    });
}
int ref_argreduce_f16(const uint16_t* x, int* idx, size_t reduce_size, size_t n, int want_min) {
    return guarded([&] {
        CPU<half> dev(n);
        std::memcpy(dev.getDataPtr(), x, n * sizeof(half));
        if (want_min) dev.argmin(idx, reduce_size, n);
        else dev.argmax(idx, reduce_size, n);
    });
}
// 0 half->float, 1 float->half, 2 half->int, 3 int->half
int ref_cast(const void* in, void* out, size_t n, int kind) {
    return guarded([&] {
        if (kind == 0) { CPU<float> d(0, nullptr); d.type_cast(static_cast<float*>(out), static_cast<const half*>(in), n); }
        else if (kind == 1) { CPU<half> d(0, nullptr); d.type_cast(static_cast<half*>(out), static_cast<const float*>(in), n); }
        else if (kind == 2) { CPU<int> d(0, nullptr); d.type_cast(static_cast<int*>(out), static_cast<const half*>(in), n); }
        else if (kind == 3) { CPU<half> d(0, nullptr); d.type_cast(static_cast<half*>(out), static_cast<const int*>(in), n); }
        else throw std::invalid_argument("unknown cast");
    });
}

// ---------------------------------------------------------------------------------------------
// Llama2 model: Transformer<half> on "cpu".
// ---------------------------------------------------------------------------------------------

void* ref_llama2_create(int dim, int hidden_dim, int n_layers, int n_heads, int vocab_size,
                        int max_seq_len) {
    RefModel* m = nullptr;
    int rc = guarded([&] {
        m = new RefModel();
        m->args.dim = dim;
        m->args.hidden_dim = hidden_dim;
        m->args.n_layers = n_layers;
        m->args.n_heads = n_heads;
        m->args.n_kv_heads = n_heads;
        m->args.vocab_size = vocab_size;
        m->args.max_batch_size = 1;
        m->args.max_seq_len = max_seq_len;
        m->model = std::make_unique<Transformer<half>>(m->args, "cpu");
    });
    if (rc) {
        delete m;
        return nullptr;
    }
    return m;
}

void ref_llama2_destroy(void* h) { delete static_cast<RefModel*>(h); }

// Fill the weights from a llama2.c legacy-v0 fp16 payload (the bytes after the 28-byte header),
// in the order model/llama2_7b/src/main.cpp:36-190 reads them. `shared` != 0: the classifier
// aliases the embedding table (main.cpp:172-173); otherwise seq_len*head_size values are skipped
// and wcls follows (main.cpp:174-187).
int ref_llama2_load(void* h, const uint16_t* payload, int shared) {
    return guarded([&] {
        RefModel* m = static_cast<RefModel*>(h);
        const ModelArgs& p = m->args;
        Transformer<half>& t = *m->model;
        const size_t dim = p.dim, hid = p.hidden_dim, L = p.n_layers, V = p.vocab_size;
        const uint16_t* cur = payload;
        auto block = [&](int l) { return std::dynamic_pointer_cast<TransformerBlock<half>>(t.layers[l]); };
        set_weight(t.tok_embeddings.weight, cur, V * dim); cur += V * dim;
        for (size_t l = 0; l < L; l++) { set_weight(block(l)->attention_norm.weight, cur, dim); cur += dim; }
        for (size_t l = 0; l < L; l++) { set_weight(block(l)->attention.wq.weight, cur, dim * dim); cur += dim * dim; }
        for (size_t l = 0; l < L; l++) { set_weight(block(l)->attention.wk.weight, cur, dim * dim); cur += dim * dim; }
        for (size_t l = 0; l < L; l++) { set_weight(block(l)->attention.wv.weight, cur, dim * dim); cur += dim * dim; }
        for (size_t l = 0; l < L; l++) { set_weight(block(l)->attention.wo.weight, cur, dim * dim); cur += dim * dim; }
        for (size_t l = 0; l < L; l++) { set_weight(block(l)->ffn_norm.weight, cur, dim); cur += dim; }
        for (size_t l = 0; l < L; l++) { set_weight(block(l)->feed_forward.w1.weight, cur, hid * dim); cur += hid * dim; }
        for (size_t l = 0; l < L; l++) { set_weight(block(l)->feed_forward.w2.weight, cur, hid * dim); cur += hid * dim; }
        for (size_t l = 0; l < L; l++) { set_weight(block(l)->feed_forward.w3.weight, cur, hid * dim); cur += hid * dim; }
        set_weight(t.norm.weight, cur, dim); cur += dim;
        if (shared) {
            t.output.weight.device = t.tok_embeddings.weight.device;
        } else {
            cur += (size_t)p.max_seq_len * (dim / p.n_heads);
            set_weight(t.output.weight, cur, V * dim);
        }
    });
}

// One forward pass: tokens (1,T) at start_pos -> logits (1,T,vocab) copied to logits_out.
// hidden_out (optional): the residual stream after every block, (n_layers, T, dim).
int ref_llama2_forward(void* h, const int* tokens, int T, int start_pos, int silu_mode,
                       uint16_t* logits_out, uint16_t* hidden_out) {
    return guarded([&] {
        RefModel* m = static_cast<RefModel*>(h);
        const ModelArgs& p = m->args;
        Transformer<half>& model = *m->model;
        const int dim = p.dim, H = p.n_heads;
        if (silu_mode != 0 && silu_mode != 1)
            throw std::invalid_argument("silu_mode must be 0 or 1: the reference's CPU code has one RMSNorm");

        Tensor<int> tok({1, T}, "cpu");
        for (int i = 0; i < T; i++) tok.setData({0, i}, tokens[i]);

        // a fresh buffer per call, like the reference allocates one per stage (llama2.cpp:40-49, :69-78)
        ActivationBuffer<half> buf(1, T, dim, p.hidden_dim, H, p.max_seq_len, p.vocab_size, "cpu");
        buf.bsz = 1; buf.seq_len = T; buf.dim = dim;                       // Transformer.cpp:271-273
        model.tok_embeddings.forward(tok, buf.x);                          // :276
        auto freqs = model.freqs.slice(start_pos, start_pos + T, 0);       // :278 (unused by Attention)

        std::vector<std::vector<int>> mask_slices = {{0, H * T * (start_pos + T)}};
        auto mask_buffer = buf.mask.getItem(mask_slices).view({1, H, T, start_pos + T});
        auto mask = model.get_mask(T, start_pos, mask_buffer);             // :280-285

        std::vector<std::vector<int>> all = {{0, 1}, {0, T}, {0, dim}};
        Tensor<half> out;
        for (int l = 0; l < p.n_layers; l++) {
            auto layer = std::dynamic_pointer_cast<TransformerBlock<half>>(model.layers[l]);
            // TransformerBlock::forward with the norm result stored (Transformer.cpp:165-177)
            Tensor<half> n1 = layer->attention_norm.forward_plain(buf.x);
            { auto s = all; buf.x_norm.setItem(s, n1.contiguous()); }
            Tensor<half> att = layer->attention.forward(buf, start_pos, freqs, mask);
            Tensor<half> hres = buf.x.EwiseAdd(att, buf.x_residual);       // :169
            Tensor<half> n2 = layer->ffn_norm.forward_plain(hres);
            { auto s = all; buf.x_norm.setItem(s, n2.contiguous()); }
            Tensor<half> ff;
            if (silu_mode == 0) {
                ff = layer->feed_forward.forward(buf);                     // :175, fp16 SiLU as is
            } else {
                const FeedForward<half>& f = layer->feed_forward;          // :133-145 with SiLU via float
                Tensor<half> x1 = f.w1.forward(buf.x_norm, buf.x1);
                Tensor<float> x1f(x1);
                Tensor<half> x1s(x1f.silu());
                Tensor<half> x3 = f.w3.forward(buf.x_norm, buf.x3);
                Tensor<half> x2 = x1s.EwiseMul(x3, buf.x2);
                ff = f.w2.forward(x2, buf.x);
            }
            out = hres.EwiseAdd(ff, buf.x_residual);                       // :175
            { auto s = all; buf.x.setItem(s, out); }                       // :291
            if (hidden_out) copy_out(out, hidden_out + (size_t)l * T * dim);
        }
        Tensor<half> hn = model.norm.forward_plain(out);                   // :295
        Tensor<half> logits = model.output.forward(hn, buf.logical);       // :296
        copy_out(logits, logits_out);
    });
}

// ---------------------------------------------------------------------------------------------
// The reference's CUDA backend, driven through its own classes on "cuda" tensors. These entry
// points need a GPU; they exist so that (a) the oracle's restatement of the CUDA RMSNorm can be
// compared with the real kernel and (b) the reference's own matmul route (gemv_v6 / gemv_v4 /
// hgemm_cublas behind CUDA<half>::matmul2d, tensorLib/src/device/cuda/gemm.cu:153-172) can be
// timed on the same GPU as a baseline. Host arrays in, host arrays out.
// ---------------------------------------------------------------------------------------------
int ref_cuda_device_count() {
    int n = 0;
    return cudaGetDeviceCount(&n) == cudaSuccess ? n : 0;
}

// nn::RMSNorm<half>::forward on "cuda" tensors -> CUDA<half>::rms_norm -> rms_norm_kernel_v1
// (tensorLib/src/nn/rmsNorm.cpp:62-106, tensorLib/src/device/cuda/rms_norm.cu:138-184).
int ref_cuda_rms_norm_f16(const uint16_t* x, const uint16_t* w, uint16_t* y, int T, int dim, float eps) {
    return guarded([&] {
        nn::RMSNorm<half> norm(dim, eps, "cuda");
        Tensor<half> xt({1, T, dim}, "cuda");
        const size_t n = (size_t)T * dim;
        if (cudaMemcpy(norm.weight.device->getDataPtr(), w, (size_t)dim * sizeof(half), cudaMemcpyHostToDevice) != cudaSuccess ||
            cudaMemcpy(xt.device->getDataPtr(), x, n * sizeof(half), cudaMemcpyHostToDevice) != cudaSuccess)
            throw std::runtime_error("cudaMemcpy to the device failed");
        Tensor<half> out = norm.forward(xt);
        if (cudaDeviceSynchronize() != cudaSuccess ||
            cudaMemcpy(y, out.device->getDataPtr(), n * sizeof(half), cudaMemcpyDeviceToHost) != cudaSuccess)
            throw std::runtime_error(std::string("reference rms_norm failed: ") + cudaGetErrorString(cudaGetLastError()));
    });
}

// CUDA<half>::matmul2d (gemm.cu:153-172) on device copies of A[M,K], B[N,K]; `reps` timed calls
// rotate over `b_copies` copies of B so that no call finds its weights in L2; the mean time per
// call (CUDA events on the legacy stream, which is where the reference launches) goes to *us and
// the result of the last call to C. reps == 0 runs it once untimed.
int ref_cuda_matmul2d_f16(const uint16_t* A, const uint16_t* B, uint16_t* C, int M, int N, int K, int reps,
                          int b_copies, double* us) {
    return guarded([&] {
        half *dA = nullptr, *dB = nullptr, *dC = nullptr;
        const size_t na = (size_t)M * K, nb = (size_t)N * K, nc = (size_t)M * N;
        if (b_copies < 1) b_copies = 1;
        cudaEvent_t e0 = nullptr, e1 = nullptr;
        auto cleanup = [&] {
            cudaFree(dA); cudaFree(dB); cudaFree(dC);
            if (e0) cudaEventDestroy(e0);
            if (e1) cudaEventDestroy(e1);
        };
        if (cudaMalloc(&dA, na * 2) != cudaSuccess || cudaMalloc(&dB, nb * 2 * b_copies) != cudaSuccess ||
            cudaMalloc(&dC, nc * 2) != cudaSuccess) { cleanup(); throw std::runtime_error("cudaMalloc failed"); }
        cudaMemcpy(dA, A, na * 2, cudaMemcpyHostToDevice);
        for (int c = 0; c < b_copies; c++) cudaMemcpy(dB + (size_t)c * nb, B, nb * 2, cudaMemcpyHostToDevice);
        CUDA<half> dev;   // no storage of its own: matmul2d only uses its arguments
        dev.matmul2d(dA, dB, dC, (size_t)M, (size_t)N, (size_t)K);
        if (cudaDeviceSynchronize() != cudaSuccess) { cleanup(); throw std::runtime_error("reference matmul2d failed"); }
        if (reps > 0) {
            cudaEventCreate(&e0); cudaEventCreate(&e1);
            for (int i = 0; i < 3; i++) dev.matmul2d(dA, dB + (size_t)(i % b_copies) * nb, dC, (size_t)M, (size_t)N, (size_t)K);
            cudaEventRecord(e0, 0);
            for (int i = 0; i < reps; i++) dev.matmul2d(dA, dB + (size_t)(i % b_copies) * nb, dC, (size_t)M, (size_t)N, (size_t)K);
            cudaEventRecord(e1, 0);
            if (cudaEventSynchronize(e1) != cudaSuccess) { cleanup(); throw std::runtime_error("reference matmul2d failed"); }
            float ms = 0.f;
            cudaEventElapsedTime(&ms, e0, e1);
            if (us) *us = (double)ms * 1e3 / reps;
        }
        cudaMemcpy(C, dC, nc * 2, cudaMemcpyDeviceToHost);
        cleanup();
    });
}

}  // extern "C"
