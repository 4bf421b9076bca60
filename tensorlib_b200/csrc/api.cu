// extern "C" entry points declared in include/tensorlib_b200.h: argument checks with the
// reference's error behaviour (invalid shapes -> TL_ERR_INVALID_ARGUMENT where the reference
// throws std::invalid_argument), dispatch on numerics and shape, launch.
#include <chrono>
#include <cstdio>
#include <cstring>
#include <new>
#include <vector>

#include <algorithm>

#include "engine.cuh"

using namespace tlb;

namespace {
inline const __half* H(const tl_half* p) { return reinterpret_cast<const __half*>(p); }
inline __half* H(tl_half* p) { return reinterpret_cast<__half*>(p); }
bool valid_numerics(int n) { return n == TL_NUMERICS_REFERENCE_ORDER || n == TL_NUMERICS_FAST; }
// pinned word behind the token staging area: the device status word is copied here at every point
// where a model call synchronises anyway, so a timed-out wait turns into an error return
int* status_slot(tl_llama2* m) { return m->pinned + m->eng->cfg().max_seq_len + 4; }
}  // namespace

extern "C" {

int tl_matmul_batched_f16(const tl_half* A, const tl_half* B, tl_half* C, size_t batch, size_t M,
                          size_t N, size_t K, size_t lda, size_t ldb, size_t ldc, size_t strideA,
                          size_t strideB, size_t strideC, int numerics, tl_stream stream) {
    TL_CHECK_INIT();
    TL_REQUIRE(valid_numerics(numerics), "unknown numerics %d", numerics);
    if (batch == 0 || M == 0 || N == 0) return TL_OK;
    TL_REQUIRE(A && B && C, "null matrix pointer");
    TL_REQUIRE(lda >= K && ldb >= K && ldc >= N, "row pitch smaller than the row");
    TL_REQUIRE(M < (1u << 31) && N < (1u << 31) && K < (1u << 31) && batch < (1u << 31), "dimension too large");
    cudaStream_t st = as_stream(stream);
    if (numerics == TL_NUMERICS_FAST && K > 0) {
        if (batch == 1 && gemv_ring_rows_supported(A, B, M, N, K, ldb, lda))
            return launch_gemv(H(A), H(B), H(C), (int)M, (int)N, (int)K, ldb, lda, ldc, st);
        if (batch == 1 && M > 8 && M <= 128 && hgemm_supported(A, B, C, M, N, K, lda, ldb, ldc) && ldc % 8 == 0 &&
            (reinterpret_cast<uintptr_t>(C) & 15) == 0 && hgemm_splitk_preferred((int)M, (int)N, (int)K))
            return launch_hgemm(H(A), H(B), H(C), 1, (int)M, (int)N, (int)K, lda, ldb, ldc, 0, 0, 0, st);
        if (batch == 1 && M >= 2 && M <= 128 && skinny_supported(A, B, M, N, K, lda, ldb))
            return launch_skinny(H(A), H(B), H(C), (int)M, (int)N, (int)K, lda, ldb, ldc, st);
        if (M > 8 && strideA % 8 == 0 && strideB % 8 == 0 && hgemm_supported(A, B, C, M, N, K, lda, ldb, ldc))
            return launch_hgemm(H(A), H(B), H(C), (int)batch, (int)M, (int)N, (int)K, lda, ldb, ldc,
                                strideA, strideB, strideC, st);
        if (gemv_supported(A, B, M < 8 ? M : 8, N, K, ldb) && lda % 8 == 0 && strideA % 8 == 0 && strideB % 8 == 0) {
            for (size_t b = 0; b < batch; b++)
                for (size_t m0 = 0; m0 < M; m0 += 8) {
                    int m = (int)(M - m0 < 8 ? M - m0 : 8);
                    TL_PROPAGATE(launch_gemv(H(A) + b * strideA + m0 * lda, H(B) + b * strideB,
                                             H(C) + b * strideC + m0 * ldc, m, (int)N, (int)K, ldb, lda, ldc, st));
                }
            return TL_OK;
        }
    }
    // reference-order kernel: any shape, any alignment (also the fast path's fallback for those)
    SeqMatmul p{H(A), H(B), H(C), (int)batch, (int)M, (int)N, (int)K, (long long)lda, 1,
                (long long)ldb, 1, (long long)ldc, (long long)strideA, (long long)strideB, (long long)strideC};
    for (size_t m0 = 0; m0 < M; m0 += 65535) {  // grid.y limit
        SeqMatmul q = p;
        q.A = p.A + m0 * lda;
        q.C = p.C + m0 * ldc;
        q.M = (int)(M - m0 < 65535 ? M - m0 : 65535);
        TL_PROPAGATE(launch_matmul_seq(q, st));
    }
    return TL_OK;
}

// Host-only: which kernel tl_matmul2d_f16 picks in fast numerics for aligned operands on a device
// with `sm_count` SMs, and how it cuts the work. No device is touched.
int tl_matmul_plan(size_t M, size_t N, size_t K, int sm_count, int* kernel, int* grid, int* tile_n, int* k_blocks_per_cta,
                   int* cluster) {
    TL_REQUIRE(kernel && grid && tile_n && k_blocks_per_cta && cluster, "null output");
    TL_REQUIRE(M >= 1 && N >= 1 && K >= 8 && sm_count >= 1 && M < (1u << 31) && N < (1u << 31) && K < (1u << 31), "bad shape");
    *grid = *tile_n = *k_blocks_per_cta = *cluster = 0;
    if (M == 1 && N % 2 == 0 && K % 16 == 0 && K <= 12288) { *kernel = TL_PLAN_GEMV_RING; return TL_OK; }
    if (M >= 2 && M <= 8 && N % 2 == 0 && K % 16 == 0) {   // the same ring with the M rows as columns of the MMA's B operand
        *kernel = TL_PLAN_GEMV_RING; *grid = (int)std::min<size_t>((size_t)sm_count, (N / 2 + 7) / 8);
        return TL_OK;
    }
    auto splitk = [&]() -> bool {      // few 128-row tiles, long K: one tile per cluster, K split over its CTAs
        if (M <= 8 || K % 8 != 0) return false;
        int kind = 0, bn = 0, ks = 0;
        hgemm_plan((int)M, (int)N, (int)K, 1, sm_count, &kind, &bn, &ks);
        if (kind != 3) return false;
        const size_t tile_m = 128;
        *kernel = TL_PLAN_HGEMM_SPLITK; *tile_n = bn; *cluster = ks;
        *grid = (int)(((M + tile_m - 1) / tile_m) * ((N + bn - 1) / bn)) * ks;
        *k_blocks_per_cta = (int)(((K + 63) / 64 + ks - 1) / ks);
        return true;
    };
    if (M >= 2 && M <= 128 && K % 8 == 0) {
        if (M > 32 && splitk()) return TL_OK;       // up to 32 rows the skinny kernel measured faster
        const SkinnyPlan pl = skinny_plan((int)M, (int)N, (int)K, sm_count);
        *kernel = pl.cluster_splits >= 2 ? TL_PLAN_SKINNY_CLUSTER : TL_PLAN_SKINNY_STREAMK;
        *grid = pl.grid; *tile_n = pl.nb; *k_blocks_per_cta = pl.per; *cluster = pl.cluster_splits;
        return TL_OK;
    }
    if (M > 8 && K % 8 == 0) {
        if (splitk()) return TL_OK;
        int kind = 0, bn = 0, sk_per = 0;
        hgemm_plan((int)M, (int)N, (int)K, 1, sm_count, &kind, &bn, &sk_per);
        *kernel = kind == 2 ? TL_PLAN_HGEMM_PAIR512 : (kind == 1 ? TL_PLAN_HGEMM_PAIR : TL_PLAN_HGEMM);
        *tile_n = bn; *cluster = kind >= 1 ? 2 : 0;
        const long long tile_m = kind == 2 ? 512 : (kind == 1 ? 256 : 128);
        const long long tiles = (long long)((M + tile_m - 1) / tile_m) * ((N + bn - 1) / bn);
        *grid = (int)std::min<long long>(tiles * (kind >= 1 ? 2 : 1), kind >= 1 ? (sm_count / 2) * 2 : sm_count);
        if (sk_per > 0) {    // stream-K ranges of sk_per k-blocks per CTA pair
            *k_blocks_per_cta = sk_per;
            *grid = 2 * (int)((tiles * (long long)((K + 63) / 64) + sk_per - 1) / sk_per);
        }
        return TL_OK;
    }
    *kernel = M <= 8 && K % 8 == 0 ? TL_PLAN_GEMV_SMALL : TL_PLAN_REFERENCE_ORDER;
    return TL_OK;
}

// Device::matmul (Device.hpp:13-20): every batch dimension may have its own stride in either operand.
// The innermost batch dimension becomes the batch of one launch; outer batch dimensions are walked
// on the host. Operands whose reduction dimension is contiguous take the kernels tl_matmul_batched_f16
// dispatches to; anything else takes the any-stride kernel.
int tl_matmul_strided_f16(const tl_half* lhs, const tl_half* rhs, tl_half* result, const int* lhs_stride_host,
                          const int* rhs_stride_host, size_t lhs_offset, size_t rhs_offset, const int* result_shape_host,
                          int ndim, size_t result_elements, size_t K, int numerics, tl_stream stream) {
    TL_CHECK_INIT();
    TL_REQUIRE(valid_numerics(numerics), "unknown numerics %d", numerics);
    TL_REQUIRE(ndim >= 2 && ndim <= 8 && lhs_stride_host && rhs_stride_host && result_shape_host, "matmul: 2..8 dimensions");
    size_t total = 1;
    for (int i = 0; i < ndim; i++) {
        TL_REQUIRE(result_shape_host[i] >= 0, "matmul: negative extent");
        total *= (size_t)result_shape_host[i];
    }
    TL_REQUIRE(total == result_elements, "matmul: result_elements %zu is not the product of result_shape (%zu)", result_elements, total);
    if (total == 0) return TL_OK;
    TL_REQUIRE(lhs && rhs && result, "null matrix pointer");
    const int* sh = result_shape_host;
    const size_t M = (size_t)sh[ndim - 2], N = (size_t)sh[ndim - 1];
    const long long a_m = lhs_stride_host[ndim - 2], a_k = lhs_stride_host[ndim - 1];
    const long long b_k = rhs_stride_host[ndim - 2], b_n = rhs_stride_host[ndim - 1];
    const int nb = ndim - 2;                                  // batch dimensions
    const size_t inner = nb > 0 ? (size_t)sh[nb - 1] : 1;     // innermost batch dimension = one launch
    const long long sA = nb > 0 ? lhs_stride_host[nb - 1] : 0, sB = nb > 0 ? rhs_stride_host[nb - 1] : 0;
    size_t outer = 1;
    for (int i = 0; i + 1 < nb; i++) outer *= (size_t)sh[i];
    const bool k_contiguous = (K <= 1 || (a_k == 1 && b_k == 1)) && a_m >= (long long)K && b_n >= (long long)K && sA >= 0 && sB >= 0;
    cudaStream_t st = as_stream(stream);
    for (size_t o = 0; o < outer; o++) {
        long long ao = (long long)lhs_offset, bo = (long long)rhs_offset;
        size_t rem = o;
        for (int i = nb - 2; i >= 0; i--) {                   // digits of o over the outer batch dimensions
            const size_t d = rem % (size_t)sh[i];
            rem /= (size_t)sh[i];
            ao += (long long)d * lhs_stride_host[i];
            bo += (long long)d * rhs_stride_host[i];
        }
        const tl_half* A = lhs + ao;
        const tl_half* B = rhs + bo;
        tl_half* C = result + o * inner * M * N;
        if (k_contiguous && numerics == TL_NUMERICS_FAST) {
            TL_PROPAGATE(tl_matmul_batched_f16(A, B, C, inner, M, N, K, (size_t)a_m, (size_t)b_n, N, (size_t)sA, (size_t)sB, M * N,
                                               numerics, stream));
        } else {
            TL_REQUIRE(M < 65536, "matmul: more than 65535 rows with a strided reduction dimension");
            SeqMatmul p{H(A), H(B), H(C), (int)inner, (int)M, (int)N, (int)K, a_m, a_k, b_n, b_k, (long long)N, sA, sB, (long long)(M * N)};
            TL_PROPAGATE(launch_matmul_seq(p, st));
        }
    }
    return TL_OK;
}

int tl_matmul2d_f16(const tl_half* A, const tl_half* B, tl_half* C, size_t M, size_t N, size_t K,
                    int numerics, tl_stream stream) {
    return tl_matmul_batched_f16(A, B, C, 1, M, N, K, K, K, N, 0, 0, 0, numerics, stream);
}

// nn::Linear<half>::forward (tensorLib/src/nn/linear.cpp:43-49): y[T, out] = x[T, in] * W[out, in]^T.
int tl_linear_f16(const tl_half* x, const tl_half* W, tl_half* y, size_t T, size_t in_features, size_t out_features,
                  tl_stream stream) {
    TL_CHECK_INIT();
    if (T == 0 || out_features == 0) return TL_OK;
    TL_REQUIRE(x && W && y, "null pointer");
    TL_REQUIRE(T < (1u << 31) && in_features < (1u << 31) && out_features < (1u << 31), "dimension too large");
    const size_t K = in_features, N = out_features;
    cudaStream_t st = as_stream(stream);
    // 1..8 rows ride the weight-streaming ring, whose producer may run ahead of the previous kernel: W is a parameter
    if (T == 1 && gemv_supported(x, W, 1, N, K, K) && N % 2 == 0 && K % 16 == 0 && K <= 12288)
        return launch_gemv(H(x), H(W), H(y), 1, (int)N, (int)K, K, K, N, st, true);
    if (gemv_ring_rows_supported(x, W, T, N, K, K, K))
        return launch_gemv(H(x), H(W), H(y), (int)T, (int)N, (int)K, K, K, N, st, true);
    if (T > 8 && T <= 128 && hgemm_supported(x, W, y, T, N, K, K, K, N) && (reinterpret_cast<uintptr_t>(y) & 15) == 0 &&
        hgemm_splitk_preferred((int)T, (int)N, (int)K))
        return launch_hgemm(H(x), H(W), H(y), 1, (int)T, (int)N, (int)K, K, K, N, 0, 0, 0, st, true);
    if (T >= 2 && T <= 128 && skinny_supported(x, W, T, N, K, K, K))
        return launch_skinny(H(x), H(W), H(y), (int)T, (int)N, (int)K, K, K, N, st, true);
    if (T > 8 && hgemm_supported(x, W, y, T, N, K, K, K, N))
        return launch_hgemm(H(x), H(W), H(y), 1, (int)T, (int)N, (int)K, K, K, N, 0, 0, 0, st, true);
    return tl_matmul2d_f16(x, W, y, T, N, K, TL_NUMERICS_FAST, stream);
}

int tl_matmul2d_f16_host(const tl_half* A_host, const tl_half* B_host, tl_half* C_host, size_t M,
                         size_t N, size_t K, int numerics) {
    TL_CHECK_INIT();
    TL_REQUIRE(A_host && B_host && C_host, "null host pointer");
    __half *dA = nullptr, *dB = nullptr, *dC = nullptr;
    const size_t ba = M * K * 2, bb = N * K * 2, bc = M * N * 2;
    int rc = TL_OK;
    cudaError_t e;
    if ((e = cudaMalloc(&dA, ba ? ba : 2)) != cudaSuccess || (e = cudaMalloc(&dB, bb ? bb : 2)) != cudaSuccess ||
        (e = cudaMalloc(&dC, bc ? bc : 2)) != cudaSuccess) {
        rc = set_error(TL_ERR_OUT_OF_MEMORY, "cudaMalloc: %s", cudaGetErrorString(e));
    } else {
        cudaMemcpyAsync(dA, A_host, ba, cudaMemcpyHostToDevice, nullptr);
        cudaMemcpyAsync(dB, B_host, bb, cudaMemcpyHostToDevice, nullptr);
        rc = tl_matmul2d_f16(reinterpret_cast<tl_half*>(dA), reinterpret_cast<tl_half*>(dB),
                             reinterpret_cast<tl_half*>(dC), M, N, K, numerics, nullptr);
        if (rc == TL_OK) {
            e = cudaMemcpy(C_host, dC, bc, cudaMemcpyDeviceToHost);
            if (e != cudaSuccess) rc = set_error(TL_ERR_CUDA, "copy back failed: %s", cudaGetErrorString(e));
        }
    }
    cudaFree(dA); cudaFree(dB); cudaFree(dC);
    return rc;
}

int tl_rms_norm_f16(tl_half* out, const tl_half* in, const tl_half* weight, float eps, int hidden,
                    int tokens, int numerics, tl_stream stream) {
    TL_CHECK_INIT();
    TL_REQUIRE(valid_numerics(numerics), "unknown numerics %d", numerics);
    TL_REQUIRE(hidden > 0 && tokens >= 0 && out && in && weight, "rms_norm: bad arguments");
    if (numerics == TL_NUMERICS_REFERENCE_ORDER)
        return launch_rmsnorm_seq(H(out), H(in), H(weight), eps, hidden, tokens, as_stream(stream));
    return launch_rmsnorm_fast(H(out), H(in), H(weight), eps, hidden, tokens, as_stream(stream));
}

int tl_apply_rotary_emb_f16(const tl_half* in, tl_half* out, int start_pos, int B, int T,
                            int n_heads, int head_dim, tl_stream stream) {
    TL_CHECK_INIT();
    TL_REQUIRE(in && out && start_pos >= 0 && B >= 0 && T >= 0 && n_heads > 0 && head_dim > 0 && head_dim % 2 == 0,
               "apply_rotary_emb: bad arguments");
    if (B == 0 || T == 0) return TL_OK;
    const __half *c, *s;
    TL_PROPAGATE(rope_table(head_dim, start_pos + T, &c, &s));
    return launch_rope(H(in), H(out), start_pos, B * T, T, n_heads, head_dim, c, s, as_stream(stream));
}

int tl_softmax_f16(tl_half* out, const tl_half* in, size_t rows, size_t cols, int numerics,
                   tl_stream stream) {
    TL_CHECK_INIT();
    TL_REQUIRE(valid_numerics(numerics), "unknown numerics %d", numerics);
    TL_REQUIRE(out && in, "softmax: null pointer");
    if (numerics == TL_NUMERICS_REFERENCE_ORDER) return launch_softmax_seq(H(out), H(in), rows, cols, as_stream(stream));
    return launch_softmax_fast(H(out), H(in), rows, cols, as_stream(stream));
}

int tl_silu_f16(tl_half* out, const tl_half* in, size_t n, int via_float, tl_stream stream) {
    TL_CHECK_INIT();
    TL_REQUIRE(out && in, "silu: null pointer");
    return launch_silu(H(out), H(in), n, via_float, as_stream(stream));
}
int tl_add_f16(tl_half* out, const tl_half* a, const tl_half* b, size_t n, tl_stream stream) {
    TL_CHECK_INIT();
    TL_REQUIRE(out && a && b, "add: null pointer");
    return launch_binary(H(out), H(a), H(b), n, 0, as_stream(stream));
}
int tl_mul_f16(tl_half* out, const tl_half* a, const tl_half* b, size_t n, tl_stream stream) {
    TL_CHECK_INIT();
    TL_REQUIRE(out && a && b, "mul: null pointer");
    return launch_binary(H(out), H(a), H(b), n, 1, as_stream(stream));
}
int tl_div_scalar_f16(tl_half* out, const tl_half* a, double scalar, size_t n, tl_stream stream) {
    TL_CHECK_INIT();
    TL_REQUIRE(out && a, "div: null pointer");
    __half hs(scalar);  // double -> fp16 like the reference's dtype scalar parameter
    TL_REQUIRE(__half2float(hs) != 0.0f, "Division by zero.");  // divFunc, CPU.cpp:280-293
    return launch_div_scalar(H(out), H(a), hs, n, as_stream(stream));
}
int tl_argmax_f16(int* out_idx, const tl_half* in, size_t rows, size_t cols, tl_stream stream) {
    TL_CHECK_INIT();
    TL_REQUIRE(out_idx && in, "argmax: null pointer");
    return launch_argmax(out_idx, H(in), rows, cols, as_stream(stream));
}
int tl_embedding_f16(tl_half* out, const tl_half* table, const int* tokens, int n_tokens, int dim,
                     int vocab, tl_stream stream) {
    TL_CHECK_INIT();
    TL_REQUIRE(out && table && tokens && dim > 0 && vocab > 0 && n_tokens >= 0, "embedding: bad arguments");
    return launch_embedding(H(out), H(table), tokens, n_tokens, dim, vocab, as_stream(stream));
}

// ---------------------------------------------------------------------------------------------
// The rest of the Device<half> surface (device_ops.cu)
// ---------------------------------------------------------------------------------------------
int tl_contiguous_f16(tl_half* result, const tl_half* data, const int* shape_host, const int* stride_host, int ndim,
                      size_t offset, size_t n, tl_stream stream) {
    TL_CHECK_INIT();
    return launch_contiguous(H(result), H(data), shape_host, stride_host, ndim, offset, n, as_stream(stream));
}
int tl_set_item_f16(tl_half* data, const tl_half* src, const int* shape_host, const int* stride_host, int ndim,
                    size_t offset, size_t n, tl_stream stream) {
    TL_CHECK_INIT();
    return launch_set_item(H(data), H(src), shape_host, stride_host, ndim, offset, n, as_stream(stream));
}
int tl_set_item_scalar_f16(tl_half* data, tl_half value, const int* shape_host, const int* stride_host, int ndim,
                           size_t offset, size_t n, tl_stream stream) {
    TL_CHECK_INIT();
    __half_raw r;
    r.x = value;
    return launch_set_item_scalar(H(data), __half(r), shape_host, stride_host, ndim, offset, n, as_stream(stream));
}
int tl_unary_f16(tl_half* out, const tl_half* in, size_t n, int op, tl_stream stream) {
    TL_CHECK_INIT();
    TL_REQUIRE(n == 0 || (out && in), "unary: null pointer");
    return launch_unary(H(out), H(in), n, op, as_stream(stream));
}
int tl_binary_f16(tl_half* out, const tl_half* a, const tl_half* b, size_t n, int op, tl_stream stream) {
    TL_CHECK_INIT();
    TL_REQUIRE(n == 0 || (out && a && b), "binary: null pointer");
    TL_REQUIRE(op >= TL_BINARY_ADD && op <= TL_BINARY_DIV, "binary: op %d needs a scalar second operand or is unknown", op);
    return launch_binary_op(H(out), H(a), H(b), n, op, as_stream(stream));
}
int tl_binary_scalar_f16(tl_half* out, const tl_half* a, tl_half scalar, size_t n, int op, tl_stream stream) {
    TL_CHECK_INIT();
    TL_REQUIRE(n == 0 || (out && a), "binary: null pointer");
    TL_REQUIRE(op >= TL_BINARY_ADD && op <= TL_BINARY_POW, "unknown binary op %d", op);
    __half_raw r;
    r.x = scalar;
    const __half s(r);
    if (op == TL_BINARY_DIV) TL_REQUIRE(__half2float(s) != 0.0f, "Division by zero.");   // divFunc, CPU.cpp:280-293
    return launch_binary_scalar(H(out), H(a), s, n, op, as_stream(stream));
}
int tl_reduce_f16(tl_half* out, const tl_half* in, size_t reduce_size, size_t n, int op, int numerics, tl_stream stream) {
    TL_CHECK_INIT();
    TL_REQUIRE(valid_numerics(numerics), "unknown numerics %d", numerics);
    TL_REQUIRE(n == 0 || (out && in), "reduce: null pointer");
    return launch_reduce(H(out), H(in), reduce_size, n, op, numerics, as_stream(stream));
}
int tl_argreduce_f16(int* out_idx, const tl_half* in, size_t reduce_size, size_t n, int want_min, tl_stream stream) {
    TL_CHECK_INIT();
    TL_REQUIRE(n == 0 || (out_idx && in), "argreduce: null pointer");
    return launch_argreduce(out_idx, H(in), reduce_size, n, want_min, as_stream(stream));
}
int tl_cast(void* out, const void* in, size_t n, int kind, tl_stream stream) {
    TL_CHECK_INIT();
    TL_REQUIRE(n == 0 || (out && in), "cast: null pointer");
    return launch_cast(out, in, n, kind, as_stream(stream));
}

// ---------------------------------------------------------------------------------------------
// Llama2
// ---------------------------------------------------------------------------------------------
int tl_llama2_create(const tl_llama2_config* cfg, tl_llama2** out) {
    TL_CHECK_INIT();
    TL_REQUIRE(cfg && out, "null argument");
    tl_llama2_config c = *cfg;
    if (c.tp_world <= 0) { c.tp_world = 1; c.tp_rank = 0; }
    if (c.n_kv_heads <= 0) c.n_kv_heads = c.n_heads;
    TL_REQUIRE(c.dim > 0 && c.hidden_dim > 0 && c.n_layers > 0 && c.n_heads > 0 && c.vocab_size > 0 && c.max_seq_len > 0,
               "model dimensions must be positive");
    TL_REQUIRE(c.dim % c.n_heads == 0 && (c.dim / c.n_heads) % 2 == 0, "dim must split into even-sized heads");
    TL_REQUIRE(c.n_kv_heads == c.n_heads, "n_kv_heads != n_heads is not supported (nor by the reference, Transformer.hpp:21)");
    TL_REQUIRE(valid_numerics(c.numerics), "unknown numerics %d", c.numerics);
    TL_REQUIRE(c.tp_rank >= 0 && c.tp_rank < c.tp_world, "tp_rank out of range");
    TL_REQUIRE(c.n_heads % c.tp_world == 0 && c.hidden_dim % c.tp_world == 0 && c.vocab_size % c.tp_world == 0,
               "heads, hidden_dim and vocab_size must divide by tp_world");
    TL_REQUIRE(c.tp_world == 1 || c.numerics == TL_NUMERICS_FAST, "tensor parallelism needs fast numerics");
    TL_REQUIRE(!c.one_kernel_decode || c.numerics == TL_NUMERICS_FAST, "one_kernel_decode needs fast numerics");
    if (c.numerics == TL_NUMERICS_FAST) {
        TL_REQUIRE(c.dim % 16 == 0 && (c.hidden_dim / c.tp_world) % 16 == 0 && ((c.dim / c.n_heads) * (c.n_heads / c.tp_world)) % 16 == 0,
                   "fast numerics needs dim, local hidden_dim and local attention width to be multiples of 16");
        TL_REQUIRE(c.dim <= 12288 && c.hidden_dim / c.tp_world <= 12288, "fast numerics: reduction length above 12288");
        TL_REQUIRE(c.dim / c.n_heads <= 256, "fast numerics: head_dim above 256");
    }
    tl_llama2* m = new (std::nothrow) tl_llama2{nullptr, nullptr};
    if (!m) return set_error(TL_ERR_OUT_OF_MEMORY, "host allocation failed");
    m->eng = new (std::nothrow) Llama2Engine(c);
    if (!m->eng) { delete m; return set_error(TL_ERR_OUT_OF_MEMORY, "host allocation failed"); }
    int rc = m->eng->allocate();
    if (rc == TL_OK && cudaMallocHost(&m->pinned, (size_t)(c.max_seq_len + 8) * sizeof(int)) != cudaSuccess)
        rc = set_error(TL_ERR_OUT_OF_MEMORY, "pinned allocation failed");
    if (rc != TL_OK) { delete m->eng; delete m; return rc; }
    *out = m;
    return TL_OK;
}

int tl_llama2_destroy(tl_llama2* m) {
    if (!m) return TL_OK;
    cudaDeviceSynchronize();
    delete m->eng;
    if (m->pinned) cudaFreeHost(m->pinned);
    delete m;
    return TL_OK;
}

int tl_llama2_load_payload_host(tl_llama2* m, const tl_half* payload_host, int shared_classifier) {
    TL_CHECK_INIT();
    TL_REQUIRE(m && payload_host, "null argument");
    return m->eng->load_payload_host(H(payload_host), shared_classifier != 0);
}

// read_checkpoint + read_weights (model/llama2_7b/src/main.cpp:195-228, :36-190)
int tl_llama2_load_file(tl_llama2* m, const char* path) {
    TL_CHECK_INIT();
    TL_REQUIRE(m && path, "null argument");
    FILE* f = fopen(path, "rb");
    if (!f) return set_error(TL_ERR_IO, "Couldn't open file %s", path);
    int hdr[7];
    if (fread(hdr, sizeof(int), 7, f) != 7) { fclose(f); return set_error(TL_ERR_IO, "short header in %s", path); }
    const tl_llama2_config& c = m->eng->cfg();
    const bool shared = hdr[5] > 0;
    const int vocab = hdr[5] > 0 ? hdr[5] : -hdr[5];
    if (hdr[0] != c.dim || hdr[1] != c.hidden_dim || hdr[2] != c.n_layers || hdr[3] != c.n_heads ||
        vocab != c.vocab_size || hdr[6] != c.max_seq_len) {
        fclose(f);
        return set_error(TL_ERR_INVALID_ARGUMENT, "checkpoint header (%d,%d,%d,%d,%d,%d) does not match the model",
                         hdr[0], hdr[1], hdr[2], hdr[3], vocab, hdr[6]);
    }
    const size_t d = c.dim, h = c.hidden_dim, L = c.n_layers, V = c.vocab_size;
    size_t n = V * d + L * (2 * d + 4 * d * d + 3 * d * h) + d;
    if (!shared) n += (size_t)c.max_seq_len * (d / c.n_heads) + V * d;
    // refuse a truncated file before anything is uploaded
    if (fseeko(f, 0, SEEK_END) != 0) { fclose(f); return set_error(TL_ERR_IO, "cannot seek in %s", path); }
    const long long size = ftello(f);
    if (size < (long long)(7 * sizeof(int) + n * sizeof(tl_half))) {
        fclose(f);
        return set_error(TL_ERR_IO, "checkpoint %s is truncated: %lld of %zu bytes", path, size, 7 * sizeof(int) + n * sizeof(tl_half));
    }
    const int rc = m->eng->load_payload_stream(f, (long long)(7 * sizeof(int)), shared);
    fclose(f);
    return rc;
}

int tl_llama2_init_random(tl_llama2* m, uint64_t seed, float std) {
    TL_CHECK_INIT();
    TL_REQUIRE(m, "null model");
    return m->eng->init_random(seed, std);
}

int tl_llama2_forward(tl_llama2* m, const int* tokens_host, int T, int start_pos,
                      tl_half* logits_host, tl_half* last_logits_host) {
    TL_CHECK_INIT();
    TL_REQUIRE(m && tokens_host, "null argument");
    Llama2Engine& e = *m->eng;
    const int V = e.cfg().vocab_size;
    TL_REQUIRE(T > 0 && T <= e.cfg().max_seq_len, "T=%d out of range", T);
    for (int i = 0; i < T; i++)
        TL_REQUIRE(tokens_host[i] >= 0 && tokens_host[i] < V, "token id %d out of range", tokens_host[i]);
    memcpy(m->pinned, tokens_host, (size_t)T * sizeof(int));
    TL_PROPAGATE(e.set_tokens(m->pinned, T, nullptr));
    TL_PROPAGATE(e.forward(T, start_pos, logits_host != nullptr, nullptr));
    TL_PROPAGATE(e.sample_last(T, nullptr));
    if (logits_host)
        TL_CUDA(cudaMemcpyAsync(logits_host, T == 1 ? e.last_logits() : e.logits(), (size_t)T * V * 2, cudaMemcpyDeviceToHost, nullptr));
    if (last_logits_host)
        TL_CUDA(cudaMemcpyAsync(last_logits_host, e.last_logits(), (size_t)V * 2, cudaMemcpyDeviceToHost, nullptr));
    int* stat = status_slot(m);
    TL_CUDA(cudaMemcpyAsync(stat, device_status_word(), sizeof(int), cudaMemcpyDeviceToHost, nullptr));
    TL_CUDA(cudaStreamSynchronize(nullptr));
    return consume_device_status(*stat);
}

int tl_llama2_set_next_token(tl_llama2* m, int token) {
    TL_CHECK_INIT();
    TL_REQUIRE(m && token >= 0 && token < m->eng->cfg().vocab_size, "bad token");
    m->pinned[0] = token;
    TL_CUDA(cudaMemcpy(m->eng->d_next(), m->pinned, sizeof(int), cudaMemcpyHostToDevice));
    return TL_OK;
}

int tl_llama2_generate(tl_llama2* m, const int* prompt_host, int n_prompt, int max_new,
                       int stop_on_eos, int* out_tokens_host, int* n_out, double* prefill_seconds,
                       double* decode_seconds) {
    return tl_llama2_generate_at(m, 0, prompt_host, n_prompt, max_new, stop_on_eos, out_tokens_host, n_out,
                                 prefill_seconds, decode_seconds);
}

int tl_llama2_generate_at(tl_llama2* m, int start_pos, const int* prompt_host, int n_prompt, int max_new,
                          int stop_on_eos, int* out_tokens_host, int* n_out, double* prefill_seconds,
                          double* decode_seconds) {
    TL_CHECK_INIT();
    TL_REQUIRE(m && prompt_host && out_tokens_host && n_out, "null argument");
    Llama2Engine& e = *m->eng;
    const int V = e.cfg().vocab_size;
    TL_REQUIRE(start_pos >= 0 && n_prompt > 0 && max_new > 0 && start_pos + n_prompt + max_new - 1 <= e.cfg().max_seq_len,
               "start (%d) + prompt (%d) + generation (%d) exceeds max_seq_len", start_pos, n_prompt, max_new);
    for (int i = 0; i < n_prompt; i++) TL_REQUIRE(prompt_host[i] >= 0 && prompt_host[i] < V, "token id out of range");
    using clk = std::chrono::high_resolution_clock;
    cudaStream_t st = nullptr;
    int* tok = m->pinned;
    *n_out = 0;
    // prefill + first argmax, timed together like llama2.cpp:35-61
    auto t0 = clk::now();
    memcpy(tok, prompt_host, (size_t)n_prompt * sizeof(int));
    TL_PROPAGATE(e.set_tokens(tok, n_prompt, st));
    TL_PROPAGATE(e.forward(n_prompt, start_pos, false, st));
    TL_PROPAGATE(e.sample_last(n_prompt, st));
    int* stat = status_slot(m);
    TL_CUDA(cudaMemcpyAsync(tok, e.d_next(), sizeof(int), cudaMemcpyDeviceToHost, st));
    TL_CUDA(cudaMemcpyAsync(stat, device_status_word(), sizeof(int), cudaMemcpyDeviceToHost, st));
    TL_CUDA(cudaStreamSynchronize(st));
    TL_PROPAGATE(consume_device_status(*stat));
    int next = tok[0];
    if (prefill_seconds) *prefill_seconds = std::chrono::duration<double>(clk::now() - t0).count();
    out_tokens_host[(*n_out)++] = next;
    // decode loop (llama2.cpp:67-99): every step the id goes host -> device -> host
    const bool fast = e.cfg().numerics == TL_NUMERICS_FAST;
    if (fast && max_new > 1) TL_PROPAGATE(e.ensure_decode_graph(st));
    auto t1 = clk::now();
    int pos = start_pos + n_prompt;
    while (*n_out < max_new) {
        if (stop_on_eos && (next == 1 || next == 2)) break;
        tok[0] = next;
        if (fast) {
            TL_CUDA(cudaMemcpyAsync(e.d_next(), tok, sizeof(int), cudaMemcpyHostToDevice, st));
            TL_PROPAGATE(e.decode_steps(pos, 1, st));
        } else {
            TL_PROPAGATE(e.set_tokens(tok, 1, st));
            TL_PROPAGATE(e.forward(1, pos, false, st));
            TL_PROPAGATE(e.sample_last(1, st));
        }
        TL_CUDA(cudaMemcpyAsync(tok, e.d_next(), sizeof(int), cudaMemcpyDeviceToHost, st));
        TL_CUDA(cudaMemcpyAsync(stat, device_status_word(), sizeof(int), cudaMemcpyDeviceToHost, st));
        TL_CUDA(cudaStreamSynchronize(st));
        TL_PROPAGATE(consume_device_status(*stat));
        next = tok[0];
        out_tokens_host[(*n_out)++] = next;
        pos++;
    }
    if (decode_seconds) *decode_seconds = std::chrono::duration<double>(clk::now() - t1).count();
    return TL_OK;
}

int tl_llama2_decode_device(tl_llama2* m, int start_pos, int steps, int* out_tokens_host, tl_stream stream) {
    TL_CHECK_INIT();
    TL_REQUIRE(m && steps >= 0, "bad argument");
    Llama2Engine& e = *m->eng;
    cudaStream_t st = as_stream(stream);
    TL_PROPAGATE(e.align_ranks(st));
    TL_PROPAGATE(e.decode_steps(start_pos, steps, st));
    if (out_tokens_host && steps > 0) {
        int* stat = status_slot(m);
        TL_CUDA(cudaMemcpyAsync(out_tokens_host, e.d_generated() + start_pos, (size_t)steps * sizeof(int),
                                cudaMemcpyDeviceToHost, st));
        TL_CUDA(cudaMemcpyAsync(stat, device_status_word(), sizeof(int), cudaMemcpyDeviceToHost, st));
        TL_CUDA(cudaStreamSynchronize(st));
        return consume_device_status(*stat);
    }
    return TL_OK;
}

int tl_llama2_kernel_launches(tl_llama2* m, long long* launches) {
    TL_REQUIRE(m && launches, "null argument");
    *launches = m->eng->launches();
    return TL_OK;
}
int tl_llama2_weight_bytes(tl_llama2* m, long long* bytes) {
    TL_REQUIRE(m && bytes, "null argument");
    *bytes = m->eng->weight_bytes();
    return TL_OK;
}

}  // extern "C"

// ---------------------------------------------------------------------------------------------
// Fused decode stages as stand-alone entry points
// ---------------------------------------------------------------------------------------------
extern "C" {

int tl_rmsnorm_qkv_rope_f16(const tl_half* x, const tl_half* norm_w, float eps, const tl_half* wq,
                            const tl_half* wk, const tl_half* wv, tl_half* q_out, tl_half* k_cache,
                            tl_half* v_cache, int dim, int n_q, int head_dim, int pos, tl_stream stream) {
    TL_CHECK_INIT();
    TL_REQUIRE(x && norm_w && wq && wk && wv && q_out && k_cache && v_cache, "null pointer");
    TL_REQUIRE(dim > 0 && n_q > 0 && head_dim > 0 && pos >= 0, "bad shape");
    const __half *c, *s;
    TL_PROPAGATE(rope_table(head_dim, pos + 1, &c, &s));
    FusedGemv a{};
    a.x = H(x); a.norm_w = H(norm_w); a.eps = eps;
    a.W[0] = H(wq); a.W[1] = H(wk); a.W[2] = H(wv); a.n_mats = 3; a.N_each = n_q; a.K = dim;
    a.epilogue = EPI_QKV_ROPE; a.y = H(q_out);
    a.k_out = H(k_cache) + (size_t)pos * n_q; a.v_out = H(v_cache) + (size_t)pos * n_q;
    a.cos_row = c + (size_t)pos * (head_dim / 2); a.sin_row = s + (size_t)pos * (head_dim / 2);
    a.head_dim = head_dim; a.pos_ptr = nullptr; a.kv_pitch = n_q; a.pdl = false;
    return launch_fused_gemv(a, as_stream(stream));
}

int tl_attn_decode_f16(const tl_half* q, const tl_half* k_cache, const tl_half* v_cache, tl_half* out,
                       float* scratch, unsigned int* counters, int n_heads, int head_dim, int seq_len,
                       int splits, tl_stream stream) {
    TL_CHECK_INIT();
    TL_REQUIRE(q && k_cache && v_cache && out && scratch && counters, "null pointer");
    TL_REQUIRE(n_heads > 0 && seq_len > 0 && splits > 0, "bad shape");
    DecodeAttn a{H(q), H(k_cache), H(v_cache), H(out), scratch, counters, n_heads, head_dim, seq_len,
                 splits, nullptr, (long long)n_heads * head_dim, false};
    return launch_decode_attn(a, as_stream(stream));
}

int tl_attn_prefill_f16(const tl_half* q, const tl_half* k_cache, const tl_half* v_cache, tl_half* out, int T,
                        int start_pos, int n_heads, int head_dim, tl_stream stream) {
    TL_CHECK_INIT();
    TL_REQUIRE(q && k_cache && v_cache && out, "null pointer");
    TL_REQUIRE(T > 0 && start_pos >= 0 && n_heads > 0 && head_dim > 0, "bad shape");
    const int S = start_pos + T;
    const long long pitch = (long long)n_heads * head_dim;
    if (!flash_prefill_supported(q, k_cache, v_cache, out, T, S, start_pos, n_heads, head_dim, pitch, pitch, pitch, pitch))
        return set_error(TL_ERR_UNSUPPORTED, "tl_attn_prefill_f16: head_dim %d (128 only) or unaligned pointers", head_dim);
    return launch_flash_prefill(H(q), H(k_cache), H(v_cache), H(out), T, S, start_pos, n_heads, head_dim, pitch,
                                pitch, pitch, pitch, as_stream(stream));
}

int tl_gemv_residual_f16(const tl_half* x, const tl_half* W, const tl_half* residual, tl_half* y,
                         int N, int K, tl_stream stream) {
    TL_CHECK_INIT();
    TL_REQUIRE(x && W && residual && y && N > 0 && K > 0, "bad argument");
    FusedGemv a{};
    a.x = H(x); a.W[0] = H(W); a.n_mats = 1; a.N_each = N; a.K = K;
    a.epilogue = EPI_RESIDUAL; a.y = H(y); a.residual = H(residual); a.pdl = false;
    return launch_fused_gemv(a, as_stream(stream));
}

int tl_rmsnorm_gateup_swiglu_f16(const tl_half* x, const tl_half* norm_w, float eps, const tl_half* w1,
                                 const tl_half* w3, tl_half* out, int hidden, int dim, tl_stream stream) {
    TL_CHECK_INIT();
    TL_REQUIRE(x && norm_w && w1 && w3 && out && hidden > 0 && dim > 0, "bad argument");
    FusedGemv a{};
    a.x = H(x); a.norm_w = H(norm_w); a.eps = eps;
    a.W[0] = H(w1); a.W[1] = H(w3); a.n_mats = 2; a.N_each = hidden; a.K = dim;
    a.epilogue = EPI_SWIGLU; a.y = H(out); a.pdl = false;
    return launch_fused_gemv(a, as_stream(stream));
}

// Self-test of the bounded wait of the tensor-parallel exchange (see the header).
int tl_selftest_unposted_exchange(int max_polls, tl_stream stream) {
    TL_CHECK_INIT();
    TL_REQUIRE(max_polls >= 1 && max_polls <= (1 << 20), "max_polls must be in [1, 2^20]");
    constexpr int K = 256, N = 64, WORLD = 2;
    cudaStream_t st = as_stream(stream);
    // [slots: WORLD x K words, all zero = epoch 0][step counter = 0][published vector: K/2 words]
    // [x, residual: K halfs each][W: N x K][y: N]
    const size_t slot_bytes = (size_t)WORLD * K * sizeof(unsigned long long);
    const size_t pub_bytes = (size_t)K / 2 * sizeof(unsigned long long);
    const size_t bytes = slot_bytes + 256 + pub_bytes + (size_t)(2 * K + N * K + N) * sizeof(__half);
    unsigned char* base = nullptr;
    TL_CUDA(cudaMalloc(&base, bytes));
    cudaError_t e = cudaMemsetAsync(base, 0, bytes, st);
    int rc = e == cudaSuccess ? TL_OK : set_error(TL_ERR_CUDA, "memset failed: %s", cudaGetErrorString(e));
    if (rc == TL_OK) {
        __half* vec = reinterpret_cast<__half*>(base + slot_bytes + 256 + pub_bytes);
        PeerExchange in{};
        in.world = WORLD; in.rank = 0; in.n = K;
        in.local_slots = reinterpret_cast<const unsigned long long*>(base);
        in.step_ptr = reinterpret_cast<const unsigned int*>(base + slot_bytes);
        in.local_pub = reinterpret_cast<unsigned long long*>(base + slot_bytes + 256);
        in.phases_per_step = 1; in.phase_id = 0;          // expected epoch 1; the slots hold epoch 0 for ever
        in.residual = vec + K; in.sum_out = nullptr;
        FusedGemv f{};
        f.x = vec; f.xin = &in; f.xin_tries = (unsigned)max_polls;
        f.W[0] = vec + 2 * K; f.n_mats = 1; f.N_each = N; f.K = K; f.epilogue = EPI_STORE; f.y = vec + 2 * K + N * K;
        f.pdl = false;
        rc = launch_fused_gemv(f, st);
    }
    cudaStreamSynchronize(st);      // the kernel must come back on its own; its only trace is the status word
    cudaFree(base);
    return rc;
}

int tl_selftest_tp_prefill_exchange(const tl_half* A, const tl_half* B, const tl_half* residual, const tl_half* norm_w,
                                    tl_half* residual_out, tl_half* xn_out, int M, int dim, int K, int world, int owner,
                                    float eps, tl_stream stream) {
    TL_CHECK_INIT();
    TL_REQUIRE(A && B && residual && norm_w && residual_out && xn_out, "null pointer");
    TL_REQUIRE((world == 2 || world == 4 || world == 8) && owner >= 0 && owner < world && M > 0 && M % (128 * world) == 0 &&
               dim % 32 == 0 && dim <= 8192 && K % 8 == 0, "self-test: M a multiple of 128 x world, world 2, 4 or 8, dim %% 32 == 0");
    cudaStream_t st = as_stream(stream);
    const int rpo = M / world;
    const size_t fslot = (size_t)(rpo / 128) * 64;          // flag words per source rank
    // [P: M x dim halfs][arrival flags: world x fslot][owner flags + row counter: 128 words]
    const size_t p_bytes = (size_t)M * dim * sizeof(__half), f_bytes = (size_t)world * fslot * sizeof(unsigned int);
    unsigned char* base = nullptr;
    TL_CUDA(cudaMalloc(&base, p_bytes + f_bytes + 512));
    __half* P = reinterpret_cast<__half*>(base);
    unsigned int* aflags = reinterpret_cast<unsigned int*>(base + p_bytes);
    unsigned int* gflags = reinterpret_cast<unsigned int*>(base + p_bytes + f_bytes);
    const unsigned int epoch = 1;
    int rc = TL_OK;
    {   // every source but `owner` has "already signalled"; the matmul below signals as source `owner`
        std::vector<unsigned int> h((size_t)world * fslot, epoch);
        for (size_t i = 0; i < fslot; i++) h[(size_t)owner * fslot + i] = 0;
        cudaError_t e = cudaMemcpyAsync(aflags, h.data(), f_bytes, cudaMemcpyHostToDevice, st);
        if (e == cudaSuccess) e = cudaMemsetAsync(gflags, 0, 512, st);
        if (e == cudaSuccess) e = cudaStreamSynchronize(st);
        if (e != cudaSuccess) rc = set_error(TL_ERR_CUDA, "self-test set-up failed: %s", cudaGetErrorString(e));
    }
    if (rc == TL_OK) {
        HgemmPush push{};
        push.world = world; push.rows_per_owner = rpo; push.epoch = epoch;
        // the matmul raises the flags of every owner; only `owner`'s block is read back, the others land in a scratch slot
        unsigned int* scratch = nullptr;
        if (cudaMalloc(&scratch, fslot * sizeof(unsigned int)) != cudaSuccess) rc = set_error(TL_ERR_OUT_OF_MEMORY, "self-test scratch");
        if (rc == TL_OK) {
            for (int d = 0; d < world; d++) push.flags[d] = d == owner ? aflags + (size_t)owner * fslot : scratch;
            int col_tiles = 0;
            rc = launch_hgemm_push(H(A), H(B), P, M, dim, K, K, K, push, &col_tiles, st);
            if (rc == TL_OK) {
                TpReduceNorm rn{};
                rn.world = world; rn.rank = owner; rn.rows = rpo; rn.row0 = owner * rpo; rn.dim = dim; rn.col_tiles = col_tiles; rn.epoch = epoch;
                for (int d = 0; d < world; d++) {
                    rn.partial[d] = P;
                    rn.xn_dst[d] = reinterpret_cast<__half*>(xn_out) + (size_t)d * M * dim;
                    rn.owner_done[d] = gflags + 8 * d;       // a separate flag block per emulated destination
                }
                rn.arrive_flags = aflags; rn.flags_slot_stride = (int)fslot;
                rn.residual = H(residual); rn.residual_out = reinterpret_cast<__half*>(residual_out);
                rn.norm_w = H(norm_w); rn.eps = eps;
                rn.rows_done = gflags + 64;
                rc = launch_tp_reduce_norm(rn, st);
                // this rank's view as a destination: the flag of owner `owner` in block 0
                if (rc == TL_OK) rc = launch_tp_wait_owners(gflags + owner, 1, epoch, st);
            }
        }
        cudaStreamSynchronize(st);
        if (scratch) cudaFree(scratch);
    }
    cudaFree(base);
    return rc;
}

int tl_llama2_decode_profile(tl_llama2* m, int start_pos, int cta, unsigned long long* stamps_host, int capacity,
                             int* n_phases) {
    TL_CHECK_INIT();
    TL_REQUIRE(m, "null model");
    return m->eng->decode_profile(start_pos, cta, stamps_host, capacity, n_phases);
}

int tl_llama2_tensor(tl_llama2* m, const char* name, int layer, void** dptr, int* rows, int* cols) {
    TL_REQUIRE(m && name && dptr && rows && cols, "null argument");
    return m->eng->tensor(name, layer, dptr, rows, cols);
}

}  // extern "C"
