// Shared helpers of the tensorlib_b200 kernels: status plumbing, fp16 arithmetic that mirrors the
// reference's host `half` operators, small device utilities.
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdarg>
#include <cstddef>
#include <cstdint>
#include <cstdio>

#include "../../include/tensorlib_b200.h"

namespace tlb {

// ---- status / error text -------------------------------------------------------------------
int set_error(int status, const char* fmt, ...);
bool initialized();
int sm_count();

// Kernel attributes (opt-in shared-memory size) belong to a device: a process that moves between
// devices with tl_init must set them once on each. One of these per kernel instantiation.
struct PerDeviceOnce {
    unsigned long long done = 0;   // bit d: configured on device d (d < 64)
    bool needed() {
        int dev = 0;
        if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return true;
        if (done & (1ull << dev)) return false;
        done |= 1ull << dev;
        return true;
    }
};

#define TL_REQUIRE(cond, ...)                                              \
    do {                                                                   \
        if (!(cond)) return ::tlb::set_error(TL_ERR_INVALID_ARGUMENT, __VA_ARGS__); \
    } while (0)

#define TL_CUDA(expr)                                                                        \
    do {                                                                                     \
        cudaError_t _e = (expr);                                                             \
        if (_e != cudaSuccess)                                                               \
            return ::tlb::set_error(_e == cudaErrorMemoryAllocation ? TL_ERR_OUT_OF_MEMORY   \
                                                                    : TL_ERR_CUDA,           \
                                    "%s failed: %s (%s:%d)", #expr, cudaGetErrorString(_e),  \
                                    __FILE__, __LINE__);                                     \
    } while (0)

#define TL_CHECK_INIT()                                                                      \
    do {                                                                                     \
        if (!::tlb::initialized())                                                           \
            return ::tlb::set_error(TL_ERR_NOT_INITIALIZED, "tl_init() has not succeeded");  \
    } while (0)

#define TL_LAUNCH_CHECK()                                                                    \
    do {                                                                                     \
        cudaError_t _e = cudaGetLastError();                                                 \
        if (_e != cudaSuccess)                                                               \
            return ::tlb::set_error(TL_ERR_CUDA, "kernel launch failed: %s (%s:%d)",         \
                                    cudaGetErrorString(_e), __FILE__, __LINE__);             \
    } while (0)

#define TL_PROPAGATE(expr)            \
    do {                              \
        int _s = (expr);              \
        if (_s != TL_OK) return _s;   \
    } while (0)

inline cudaStream_t as_stream(tl_stream s) { return reinterpret_cast<cudaStream_t>(s); }
inline size_t ceil_div(size_t a, size_t b) { return (a + b - 1) / b; }

// ---- fp16 arithmetic with the reference's rounding -------------------------------------------
// The reference's host operators on `half` convert to float, operate, and round once to half
// (host branches of __hadd/__hsub/__hmul/__hdiv in cuda_fp16.hpp). Because float carries
// 24 >= 2*11+2 significand bits, that double rounding is innocuous for + - * /, so these equal
// the correctly rounded fp16 result; they are spelled out in float so no FMA contraction or
// approximate division can sneak in.
__device__ __forceinline__ __half hadd_ref(__half a, __half b) {
    return __float2half_rn(__fadd_rn(__half2float(a), __half2float(b)));
}
__device__ __forceinline__ __half hsub_ref(__half a, __half b) {
    return __float2half_rn(__fsub_rn(__half2float(a), __half2float(b)));
}
__device__ __forceinline__ __half hmul_ref(__half a, __half b) {
    return __float2half_rn(__fmul_rn(__half2float(a), __half2float(b)));
}
__device__ __forceinline__ __half hdiv_ref(__half a, __half b) {
    return __float2half_rn(__fdiv_rn(__half2float(a), __half2float(b)));
}
// SiLU through float, one rounding (tensorLib/src/device/cuda/CUDA.cu:334-342 and the CPU float
// route CPU.cpp:220-222). exp is taken in double and rounded to float so that it agrees with a
// correctly rounded host expf in all but astronomically rare cases.
__device__ __forceinline__ float expf_cr(float x) { return (float)exp((double)x); }
__device__ __forceinline__ __half silu_via_float(__half x) {
    float xf = __half2float(x);
    float sig = __fdiv_rn(1.0f, __fadd_rn(1.0f, expf_cr(-xf)));
    return __float2half_rn(__fmul_rn(xf, sig));
}
// The CPU backend's fp16 SiLU as shipped (CPU.cpp:216-219): sigmoid evaluated as 1/(1+exp(x)).
__device__ __forceinline__ __half silu_half_as_shipped(__half x) {
    __half sig = __float2half_rn(__fdiv_rn(1.0f, __fadd_rn(1.0f, expf_cr(__half2float(x)))));
    return hmul_ref(x, sig);
}

// ---- warp / block reductions ------------------------------------------------------------------
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Programmatic dependent launch: let the next kernel in the stream start its weight prefetch
// while this one drains, and wait for the previous kernel's results before touching activations.
__device__ __forceinline__ void pdl_launch_dependents() {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// Launch with programmatic stream serialization: the grid may be scheduled while the previous
// kernel of the stream is still draining; the kernel itself executes griddepcontrol.wait before it
// touches anything another kernel may have written.
template <typename Kern, typename... Args>
int launch_pdl(Kern kern, dim3 grid, dim3 block, size_t smem, cudaStream_t st, bool pdl, Args... args) {
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 1 : 0;
    TL_CUDA(cudaLaunchKernelEx(&cfg, kern, args...));
    return TL_OK;
}

}  // namespace tlb
