// B200 : CUDA<half> — the reference-side binding of libtensorlib_b200.so.
//
// A maintainer of DavidZyy/tensorLib adds this header to the reference tree (for example as
// tensorLib/include/device/cuda/B200.hpp), links the library, and constructs B200 where
// Tensor<half> constructs CUDA<half> today (tensorLib/src/Tensor.cpp:46-52). Storage, getData and
// setData stay the reference's (CUDA<half> owns data_); every compute virtual of Device<half>
// (tensorLib/include/device/Device.hpp:13-98) forwards to the C ABI, on the legacy default stream
// like the reference, and keeps the reference's error behaviour: std::invalid_argument where the
// op layer throws it, print-and-exit for everything else (CUDA_CHECK, CUDA.cuh:131-151).
//
// This file needs the reference's headers on the include path; it is not used by the library itself.
#pragma once

#include <cstdlib>
#include <cstring>
#include <iostream>
#include <stdexcept>
#include <vector>

#include "device/cuda/CUDA.cuh"
#include "tensorlib_b200.h"

namespace tlb200 {
inline void check(int s) {
    if (s == TL_ERR_INVALID_ARGUMENT) throw std::invalid_argument(tl_last_error());
    if (s != TL_OK) {
        std::cerr << "tensorlib_b200: " << tl_last_error() << std::endl;
        std::exit(1);
    }
}
inline const tl_half* th(const half* p) { return reinterpret_cast<const tl_half*>(p); }
inline tl_half* th(half* p) { return reinterpret_cast<tl_half*>(p); }
inline tl_half bits(half v) {
    tl_half b;
    static_assert(sizeof(half) == sizeof(tl_half), "half is 16 bits");
    std::memcpy(&b, &v, sizeof b);
    return b;
}
}  // namespace tlb200

class B200 : public CUDA<half> {
public:
    using CUDA<half>::CUDA;
    int numerics = TL_NUMERICS_FAST;   // TL_NUMERICS_REFERENCE_ORDER reproduces the CPU backend bit for bit

    // ---- matmul: Device.hpp:13-22; was gemm.cu:28-85 (one thread per output, half accumulator) and
    //      gemm.cu:153-172 (gemv_v6 / gemv_v4 / cublasHgemm with a handle per call) -----------------------
    void matmul(const half* lhs, const half* rhs, half* result, const std::vector<int>& lhs_stride,
                const std::vector<int>& rhs_stride, size_t lhs_offset, size_t rhs_offset,
                const std::vector<int>& result_shape, size_t result_elements, size_t K) override {
        tlb200::check(tl_matmul_strided_f16(tlb200::th(lhs), tlb200::th(rhs), tlb200::th(result), lhs_stride.data(),
                                            rhs_stride.data(), lhs_offset, rhs_offset, result_shape.data(),
                                            (int)result_shape.size(), result_elements, K, numerics, nullptr));
    }
    void matmul2d(const half* A, const half* B, half* C, size_t M, size_t N, size_t K) override {
        tlb200::check(tl_matmul2d_f16(tlb200::th(A), tlb200::th(B), tlb200::th(C), M, N, K, numerics, nullptr));
    }

    // ---- strided copies: Device.hpp:30-47; were CUDA.cu:83-186 ---------------------------------------------
    void contiguous(half* result, const std::vector<int>& shape, const std::vector<int>& stride, size_t offset,
                    size_t num_elements) override {
        tlb200::check(tl_contiguous_f16(tlb200::th(result), tlb200::th(this->data_), shape.data(), stride.data(),
                                        (int)shape.size(), offset, num_elements, nullptr));
    }
    void setItemEwise(half* src, const std::vector<int>& shape, const std::vector<int>& stride, size_t offset,
                      size_t num_elements) override {
        tlb200::check(tl_set_item_f16(tlb200::th(this->data_), tlb200::th(src), shape.data(), stride.data(),
                                      (int)shape.size(), offset, num_elements, nullptr));
    }
    void setItemScalar(half value, const std::vector<int>& shape, const std::vector<int>& stride, size_t offset,
                       size_t num_elements) override {
        tlb200::check(tl_set_item_scalar_f16(tlb200::th(this->data_), tlb200::bits(value), shape.data(), stride.data(),
                                             (int)shape.size(), offset, num_elements, nullptr));
    }

    // ---- unary family: Device.hpp:49-58; were CUDA.cu:194-402 ---------------------------------------------
    void neg(half* r, size_t n) override { unary(r, n, TL_UNARY_NEG); }
    void sin(half* r, size_t n) override { unary(r, n, TL_UNARY_SIN); }
    void cos(half* r, size_t n) override { unary(r, n, TL_UNARY_COS); }
    void exp(half* r, size_t n) override { unary(r, n, TL_UNARY_EXP); }
    void log(half* r, size_t n) override { unary(r, n, TL_UNARY_LOG); }
    void abs(half* r, size_t n) override { unary(r, n, TL_UNARY_ABS); }
    void tanh(half* r, size_t n) override { unary(r, n, TL_UNARY_TANH); }
    void silu(half* r, size_t n) override { unary(r, n, TL_UNARY_SILU); }
    void sqrt(half* r, size_t n) override { unary(r, n, TL_UNARY_SQRT); }
    void rsqrt(half* r, size_t n) override { unary(r, n, TL_UNARY_RSQRT); }

    // ---- binary and scalar arithmetic: Device.hpp:61-70; were binary.cuh:42-75 ----------------------------
    void add(half* r, half* o, size_t n) const override { binary(r, o, n, TL_BINARY_ADD); }
    void sub(half* r, half* o, size_t n) const override { binary(r, o, n, TL_BINARY_SUB); }
    void mul(half* r, half* o, size_t n) const override { binary(r, o, n, TL_BINARY_MUL); }
    void div(half* r, half* o, size_t n) const override { binary(r, o, n, TL_BINARY_DIV); }
    void add(half* r, half s, size_t n) const override { scalar(r, s, n, TL_BINARY_ADD); }
    void sub(half* r, half s, size_t n) const override { scalar(r, s, n, TL_BINARY_SUB); }
    void mul(half* r, half s, size_t n) const override { scalar(r, s, n, TL_BINARY_MUL); }
    void div(half* r, half s, size_t n) const override { scalar(r, s, n, TL_BINARY_DIV); }
    void pow(half* r, half s, size_t n) const override { scalar(r, s, n, TL_BINARY_POW); }

    // ---- reductions over the last dimension: Device.hpp:73-79; were reduce.cuh:18-39, reduceArg.cu, softmax.cu
    void max(half* r, size_t reduce_size, size_t n) const override { reduce(r, reduce_size, n, TL_REDUCE_MAX); }
    void min(half* r, size_t reduce_size, size_t n) const override { reduce(r, reduce_size, n, TL_REDUCE_MIN); }
    void sum(half* r, size_t reduce_size, size_t n) const override { reduce(r, reduce_size, n, TL_REDUCE_SUM); }
    void mean(half* r, size_t reduce_size, size_t n) const override { reduce(r, reduce_size, n, TL_REDUCE_MEAN); }
    void argmax(int* r, size_t reduce_size, size_t n) const override {
        tlb200::check(tl_argreduce_f16(r, tlb200::th(this->data_), reduce_size, n, 0, nullptr));
    }
    void argmin(int* r, size_t reduce_size, size_t n) const override {
        tlb200::check(tl_argreduce_f16(r, tlb200::th(this->data_), reduce_size, n, 1, nullptr));
    }
    void softmax(half* out, size_t rows, size_t cols) const override {
        tlb200::check(tl_softmax_f16(tlb200::th(out), tlb200::th(this->data_), rows, cols, numerics, nullptr));
    }

    // ---- Device.hpp:91-98; was CUDA.cu:405-437 -------------------------------------------------------------
    void apply_rotary_emb(const half* in, half* out, int start_pos, int B, int T, int n_heads, int head_dim) const override {
        tlb200::check(tl_apply_rotary_emb_f16(tlb200::th(in), tlb200::th(out), start_pos, B, T, n_heads, head_dim, nullptr));
    }
    // ---- CUDA.cuh:108 (not virtual: nn::RMSNorm reaches it by dynamic_pointer_cast<CUDA<half>>, so a
    //      maintainer casts to B200 there, rmsNorm.cpp:85-91); was rms_norm.cu:181-184 ----------------------------
    void rms_norm(half* out, half* in, half* w, float eps, int hidden, int tokens) {
        tlb200::check(tl_rms_norm_f16(tlb200::th(out), tlb200::th(in), tlb200::th(w), eps, hidden, tokens, numerics, nullptr));
    }
    // ---- type_cast into half (CUDA.cu:440-464; a template, hence not virtual either) -------------------------
    void type_cast_from_float(half* result, const float* src, size_t n) {
        tlb200::check(tl_cast(result, src, n, TL_CAST_F32_TO_F16, nullptr));
    }
    void type_cast_from_int(half* result, const int* src, size_t n) {
        tlb200::check(tl_cast(result, src, n, TL_CAST_I32_TO_F16, nullptr));
    }

private:
    void unary(half* r, size_t n, int op) { tlb200::check(tl_unary_f16(tlb200::th(r), tlb200::th(this->data_), n, op, nullptr)); }
    void binary(half* r, half* o, size_t n, int op) const {
        tlb200::check(tl_binary_f16(tlb200::th(r), tlb200::th(this->data_), tlb200::th(o), n, op, nullptr));
    }
    void scalar(half* r, half s, size_t n, int op) const {
        tlb200::check(tl_binary_scalar_f16(tlb200::th(r), tlb200::th(this->data_), tlb200::bits(s), n, op, nullptr));
    }
    void reduce(half* r, size_t reduce_size, size_t n, int op) const {
        tlb200::check(tl_reduce_f16(tlb200::th(r), tlb200::th(this->data_), reduce_size, n, op, numerics, nullptr));
    }
};
