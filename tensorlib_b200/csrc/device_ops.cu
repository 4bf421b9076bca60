// The rest of the Device<half> surface on fp16 device memory: strided copies (contiguous /
// setItemEwise / setItemScalar), the unary family, binary and scalar arithmetic, row reductions
// and type casts. Replaces tensorLib/src/device/cuda/CUDA.cu:83-210, :440-464,
// tensorLib/include/device/cuda/binary.cuh:42-75 and reduce.cuh:18-39; the arithmetic follows the
// reference's CPU backend (tensorLib/src/device/cpu/CPU.cpp:127-402) bit for bit:
//   * functions half -> half that go through libm (sin, cos, exp, log, tanh, SiLU, pow by a
//     scalar) are 65536-entry tables evaluated on the host with the calls the reference makes, so
//     the device cannot disagree with it in the last place;
//   * + - * / are "both operands to float, one operation, one rounding" (the reference's host half
//     operators), sqrt and 1/sqrt use the correctly rounded float instructions;
//   * reductions come in the reference's sequential fp16 order and in a parallel fp32 form.
// All of it is HBM-bound byte shuffling: 16-byte accesses wherever alignment allows, grids sized
// in multiples of the SM count, and no index division in the inner loop (the mixed-radix split of
// a linear index uses multiply-high by constants prepared on the host).
#include <algorithm>
#include <cmath>
#include <cstring>
#include <mutex>
#include <vector>

#include "kernels.cuh"

namespace tlb {

namespace {

inline bool al16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }
inline unsigned grid_for(size_t work_items, int threads) {
    const size_t blocks = ceil_div(work_items, (size_t)threads);
    const size_t cap = (size_t)std::max(1, sm_count()) * 16;      // grid-stride loops: a few CTAs per SM
    return (unsigned)std::max<size_t>(1, std::min(blocks, cap));
}

// ---------------------------------------------------------------------------------------------
// Strided copies. Element i of the logical (contiguous) order sits at
// offset + sum_d idx_d * stride_d with idx the mixed-radix digits of i over `shape`
// (convertIdx, tensorLib/include/device/cuda/CUDA.cuh:186-202; CPU.cpp:127-167).
// ---------------------------------------------------------------------------------------------
constexpr int MAX_DIMS = 8;
struct StridedDesc {
    int ndim;
    unsigned int shape[MAX_DIMS];
    long long stride[MAX_DIMS];
    unsigned long long magic[MAX_DIMS];   // ceil(2^64 / shape): q = umul64hi(n, magic) is n / shape for n < 2^32
    long long offset;
};

__device__ __forceinline__ long long strided_offset(const StridedDesc& d, unsigned int i) {
    long long off = d.offset;
#pragma unroll
    for (int k = MAX_DIMS - 1; k >= 0; k--) {
        if (k < d.ndim) {
            const unsigned int s = d.shape[k];
            const unsigned int q = s == 1 ? i : (unsigned int)__umul64hi((unsigned long long)i, d.magic[k]);
            off += (long long)(i - q * s) * d.stride[k];
            i = q;
        }
    }
    return off;
}

// MODE 0: dst[i] = src[strided(i)]   (contiguous)
// MODE 1: dst[strided(i)] = src[i]   (setItemEwise)
// MODE 2: dst[strided(i)] = value    (setItemScalar)
template <int MODE, typename T>
__global__ void k_strided(T* __restrict__ dst, const T* __restrict__ src, T value, StridedDesc d, unsigned int n) {
    for (unsigned long long i0 = (unsigned long long)blockIdx.x * blockDim.x + threadIdx.x; i0 < n;
         i0 += (unsigned long long)gridDim.x * blockDim.x) {
        const unsigned int i = (unsigned int)i0;
        const long long off = strided_offset(d, i);
        if (MODE == 0) dst[i] = src[off];
        else if (MODE == 1) dst[off] = src[i];
        else dst[off] = value;
    }
}

// Merge neighbouring dimensions that are contiguous with respect to each other and drop size-1
// dimensions, so that the common cases (a slice of the leading dimension, a transposed pair of
// large blocks) decompose into one or two digits.
int collapse(const int* shape, const int* stride, int ndim, StridedDesc* out) {
    long long sh[MAX_DIMS], st[MAX_DIMS];
    int m = 0;
    for (int k = 0; k < ndim; k++) {
        if (shape[k] == 1) continue;
        if (m > 0 && st[m - 1] == (long long)stride[k] * shape[k]) {
            sh[m - 1] *= shape[k];
            st[m - 1] = stride[k];
        } else {
            sh[m] = shape[k];
            st[m] = stride[k];
            m++;
        }
    }
    if (m == 0) { sh[0] = 1; st[0] = 1; m = 1; }
    out->ndim = m;
    for (int k = 0; k < m; k++) {
        if (sh[k] >= (1ll << 32)) return -1;
        out->shape[k] = (unsigned int)sh[k];
        out->stride[k] = st[k];
        out->magic[k] = sh[k] <= 1 ? 0ull : (~0ull / (unsigned long long)sh[k]) + 1ull;   // ceil(2^64 / s), s >= 2, s not a power of two or exact either way
    }
    return 0;
}

template <int MODE>
int launch_strided(__half* dst, const __half* src, __half value, const int* shape, const int* stride, int ndim,
                   size_t offset, size_t n, cudaStream_t st) {
    TL_REQUIRE(ndim >= 0 && ndim <= MAX_DIMS && (ndim == 0 || (shape && stride)), "strided copy: 0..%d dimensions", MAX_DIMS);
    size_t total = 1;
    for (int k = 0; k < ndim; k++) {
        TL_REQUIRE(shape[k] >= 0, "strided copy: negative extent");
        total *= (size_t)shape[k];
    }
    TL_REQUIRE(total == n, "strided copy: num_elements %zu is not the product of the shape (%zu)", n, total);
    if (n == 0) return TL_OK;
    TL_REQUIRE(n < (1ull << 32), "strided copy: more than 2^32 - 1 elements");
    TL_REQUIRE(dst && (MODE == 2 || src), "strided copy: null pointer");
    StridedDesc d{};
    TL_REQUIRE(collapse(shape, stride, ndim, &d) == 0, "strided copy: a merged dimension exceeds 2^32");
    d.offset = (long long)offset;
    // 16-byte path: the innermost digit runs over contiguous memory in multiples of eight halfs and
    // every other term of the address is a multiple of eight too
    const int in = d.ndim - 1;
    const __half* strided_ptr = MODE == 0 ? src : dst;
    const __half* linear_ptr = MODE == 0 ? dst : src;
    bool vec = d.stride[in] == 1 && d.shape[in] % 8 == 0 && offset % 8 == 0 && al16(strided_ptr) && (MODE == 2 || al16(linear_ptr));
    for (int k = 0; k < in && vec; k++) vec = d.stride[k] % 8 == 0;
    if (vec) {
        StridedDesc v = d;
        v.shape[in] = d.shape[in] / 8;
        v.magic[in] = v.shape[in] <= 1 ? 0ull : (~0ull / (unsigned long long)v.shape[in]) + 1ull;
        for (int k = 0; k < in; k++) v.stride[k] = d.stride[k] / 8;
        v.offset = d.offset / 8;
        const unsigned int n8 = (unsigned int)(n / 8);
        uint4 vv;
        __half* hv = reinterpret_cast<__half*>(&vv);
        for (int j = 0; j < 8; j++) hv[j] = value;
        k_strided<MODE, uint4><<<grid_for(n8, 256), 256, 0, st>>>(reinterpret_cast<uint4*>(dst), reinterpret_cast<const uint4*>(src), vv, v, n8);
    } else {
        k_strided<MODE, __half><<<grid_for(n, 256), 256, 0, st>>>(dst, src, value, d, (unsigned int)n);
    }
    TL_LAUNCH_CHECK();
    return TL_OK;
}

// ---------------------------------------------------------------------------------------------
// Unary family (Device.hpp:49-58; CPU.cpp:169-276). Table ops: out = tab[bits(in)].
// ---------------------------------------------------------------------------------------------
// Large inputs: every CTA copies the 128 KB table into shared memory once and then streams its
// share of the input through it with 16-byte loads and stores; the lookups hit shared memory
// instead of issuing one global gather per element.
__global__ void __launch_bounds__(1024, 1) k_lookup_smem(uint4* __restrict__ out, const uint4* __restrict__ in, size_t n8,
                                                         const uint4* __restrict__ tab) {
    extern __shared__ uint4 stab4[];
    for (int i = threadIdx.x; i < 65536 / 8; i += blockDim.x) stab4[i] = tab[i];
    __syncthreads();
    const unsigned short* stab = reinterpret_cast<const unsigned short*>(stab4);
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n8; i += (size_t)gridDim.x * blockDim.x) {
        uint4 v = in[i], o;
        const unsigned short* hv = reinterpret_cast<const unsigned short*>(&v);
        unsigned short* ho = reinterpret_cast<unsigned short*>(&o);
#pragma unroll
        for (int j = 0; j < 8; j++) ho[j] = stab[hv[j]];
        out[i] = o;
    }
}
__global__ void k_lookup_gmem(unsigned short* out, const unsigned short* in, size_t n, const unsigned short* tab) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
        out[i] = __ldg(tab + in[i]);
}

// direct ops: 0 neg, 1 abs, 2 sqrt, 3 rsqrt
template <int OP>
__device__ __forceinline__ __half unary_direct(__half x) {
    if (OP == 0) return __float2half_rn(-__half2float(x));              // host operator-: through float
    if (OP == 1) return __float2half_rn(fabsf(__half2float(x)));
    const float f = __half2float(x);
    if (OP == 2) return __float2half_rn(__fsqrt_rn(f));
    return __float2half_rn(__fdiv_rn(1.0f, __fsqrt_rn(f)));
}
template <int OP>
__global__ void k_unary_direct(__half* out, const __half* in, size_t n, bool vec) {
    if (vec) {
        const size_t n8 = n / 8;
        for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n8; i += (size_t)gridDim.x * blockDim.x) {
            uint4 v = reinterpret_cast<const uint4*>(in)[i], o;
            const __half* hv = reinterpret_cast<const __half*>(&v);
            __half* ho = reinterpret_cast<__half*>(&o);
#pragma unroll
            for (int j = 0; j < 8; j++) ho[j] = unary_direct<OP>(hv[j]);
            reinterpret_cast<uint4*>(out)[i] = o;
        }
    } else {
        for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
            out[i] = unary_direct<OP>(in[i]);
    }
}

// Host-evaluated tables, built on first use of an op and kept for the life of the process.
struct OpTable { __half* dev = nullptr; };
std::mutex g_tab_mu;
OpTable g_unary_tab[16];

float unary_host(int op, float x) {
    switch (op) {
        case TL_UNARY_SIN: return std::sin(x);      // sinFunc ... tanhFunc, CPU.cpp:170-211
        case TL_UNARY_COS: return std::cos(x);
        case TL_UNARY_EXP: return std::exp(x);
        case TL_UNARY_LOG: return std::log(x);
        case TL_UNARY_TANH: return std::tanh(x);
        default: return x;
    }
}

int table_for_unary(int op, const __half** out) {
    std::lock_guard<std::mutex> lk(g_tab_mu);
    OpTable& t = g_unary_tab[op];
    if (!t.dev) {
        std::vector<__half> h(65536);
        for (unsigned i = 0; i < 65536; i++) {
            __half_raw r;
            r.x = (unsigned short)i;
            h[i] = __float2half(unary_host(op, __half2float(__half(r))));
        }
        __half* d = nullptr;
        TL_CUDA(cudaMalloc(&d, 65536 * sizeof(__half)));
        TL_CUDA(cudaMemcpy(d, h.data(), 65536 * sizeof(__half), cudaMemcpyHostToDevice));
        t.dev = d;
    }
    *out = t.dev;
    return TL_OK;
}

int launch_lookup(__half* out, const __half* in, size_t n, const __half* tab, cudaStream_t st) {
    if (n >= (1u << 20) && n % 8 == 0 && al16(out) && al16(in)) {
        static PerDeviceOnce once;
        if (once.needed())
            TL_CUDA(cudaFuncSetAttribute(k_lookup_smem, cudaFuncAttributeMaxDynamicSharedMemorySize, 65536 * 2));
        k_lookup_smem<<<std::max(1, sm_count()), 1024, 65536 * 2, st>>>(reinterpret_cast<uint4*>(out), reinterpret_cast<const uint4*>(in),
                                                                        n / 8, reinterpret_cast<const uint4*>(tab));
    } else {
        k_lookup_gmem<<<grid_for(n, 256), 256, 0, st>>>(reinterpret_cast<unsigned short*>(out), reinterpret_cast<const unsigned short*>(in), n,
                                                        reinterpret_cast<const unsigned short*>(tab));
    }
    TL_LAUNCH_CHECK();
    return TL_OK;
}

// ---------------------------------------------------------------------------------------------
// Binary and scalar arithmetic (Device.hpp:61-70; CPU.cpp:277-340).
// ---------------------------------------------------------------------------------------------
template <int OP>
__device__ __forceinline__ __half binary_op(__half a, __half b) {
    if (OP == TL_BINARY_ADD) return hadd_ref(a, b);
    if (OP == TL_BINARY_SUB) return hsub_ref(a, b);
    if (OP == TL_BINARY_MUL) return hmul_ref(a, b);
    return hdiv_ref(a, b);
}
// SCALAR: b is one value; otherwise an array
template <int OP, bool SCALAR>
__global__ void k_binary_any(__half* out, const __half* a, const __half* b, __half s, size_t n, bool vec) {
    if (vec) {
        const size_t n8 = n / 8;
        for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n8; i += (size_t)gridDim.x * blockDim.x) {
            const uint4 va = reinterpret_cast<const uint4*>(a)[i];
            uint4 vb = va, vo;
            if (!SCALAR) vb = reinterpret_cast<const uint4*>(b)[i];
            const __half* ha = reinterpret_cast<const __half*>(&va);
            const __half* hb = reinterpret_cast<const __half*>(&vb);
            __half* ho = reinterpret_cast<__half*>(&vo);
#pragma unroll
            for (int j = 0; j < 8; j++) ho[j] = binary_op<OP>(ha[j], SCALAR ? s : hb[j]);
            reinterpret_cast<uint4*>(out)[i] = vo;
        }
    } else {
        for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
            out[i] = binary_op<OP>(a[i], SCALAR ? s : b[i]);
    }
}

template <bool SCALAR>
int launch_binary_any(__half* out, const __half* a, const __half* b, __half s, size_t n, int op, cudaStream_t st) {
    const bool vec = n % 8 == 0 && al16(out) && al16(a) && (SCALAR || al16(b));
    const unsigned grid = grid_for(vec ? n / 8 : n, 256);
    switch (op) {
        case TL_BINARY_ADD: k_binary_any<TL_BINARY_ADD, SCALAR><<<grid, 256, 0, st>>>(out, a, b, s, n, vec); break;
        case TL_BINARY_SUB: k_binary_any<TL_BINARY_SUB, SCALAR><<<grid, 256, 0, st>>>(out, a, b, s, n, vec); break;
        case TL_BINARY_MUL: k_binary_any<TL_BINARY_MUL, SCALAR><<<grid, 256, 0, st>>>(out, a, b, s, n, vec); break;
        case TL_BINARY_DIV: k_binary_any<TL_BINARY_DIV, SCALAR><<<grid, 256, 0, st>>>(out, a, b, s, n, vec); break;
        default: return set_error(TL_ERR_INVALID_ARGUMENT, "unknown binary op %d", op);
    }
    TL_LAUNCH_CHECK();
    return TL_OK;
}

// pow by a scalar: half(powf(float(a), float(s))) (powFunc, CPU.cpp:295-309) as a table over a,
// evaluated on the host for this s. The last few exponents are kept (an RMSNorm squares).
struct PowTable { unsigned short s_bits = 0; bool used = false; __half* dev = nullptr; unsigned long long age = 0; };
PowTable g_pow[4];
unsigned long long g_pow_clock = 0;

int table_for_pow(__half s, const __half** out, cudaStream_t st) {
    std::lock_guard<std::mutex> lk(g_tab_mu);
    const unsigned short bits = __half_as_ushort(s);
    PowTable* victim = &g_pow[0];
    for (PowTable& t : g_pow) {
        if (t.used && t.s_bits == bits) { t.age = ++g_pow_clock; *out = t.dev; return TL_OK; }
        if (!t.used || t.age < victim->age || (victim->used && !t.used)) victim = &t;
    }
    std::vector<__half> h(65536);
    const float sf = __half2float(s);
    for (unsigned i = 0; i < 65536; i++) {
        __half_raw r;
        r.x = (unsigned short)i;
        h[i] = __float2half(std::pow(__half2float(__half(r)), sf));
    }
    if (!victim->dev) TL_CUDA(cudaMalloc(&victim->dev, 65536 * sizeof(__half)));
    // a table that is being replaced may still be read by a launch in flight on another stream
    if (victim->used) TL_CUDA(cudaDeviceSynchronize());
    TL_CUDA(cudaMemcpyAsync(victim->dev, h.data(), 65536 * sizeof(__half), cudaMemcpyHostToDevice, st));
    TL_CUDA(cudaStreamSynchronize(st));      // h goes out of scope
    victim->used = true;
    victim->s_bits = bits;
    victim->age = ++g_pow_clock;
    *out = victim->dev;
    return TL_OK;
}

// ---------------------------------------------------------------------------------------------
// Reductions over the last dimension (Device.hpp:73-78; CPU.cpp:342-402).
// ---------------------------------------------------------------------------------------------
// Reference order: temp = x[0]; temp = op(temp, x[j]) for j = 1.. in fp16, one thread per row.
template <int OP>
__global__ void k_reduce_seq(__half* out, const __half* in, size_t rows, size_t cols, __half hcols) {
    const size_t r = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (r >= rows) return;
    const __half* x = in + r * cols;
    __half t = x[0];
    for (size_t j = 1; j < cols; j++) {
        const __half v = x[j];
        if (OP == TL_REDUCE_MAX) t = (__half2float(t) < __half2float(v)) ? v : t;        // std::max(a, b) = a < b ? b : a
        else if (OP == TL_REDUCE_MIN) t = (__half2float(v) < __half2float(t)) ? v : t;   // std::min(a, b) = b < a ? b : a
        else t = hadd_ref(t, v);
    }
    if (OP == TL_REDUCE_MEAN) t = hdiv_ref(t, hcols);                                    // result[i] /= dtype(reduce_size)
    out[r] = t;
}

// Parallel form, one warp per row: max / min carry the index so that the first of several equal
// values wins, like the sequential scan (it matters only for the sign of a zero); sum / mean
// accumulate in fp32 and round once.
template <int OP>
__global__ void k_reduce_warp(__half* out, int* out_idx, const __half* in, size_t rows, size_t cols) {
    const size_t r = (size_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (r >= rows) return;
    const int lane = threadIdx.x & 31;
    const __half* x = in + r * cols;
    if (OP == TL_REDUCE_SUM || OP == TL_REDUCE_MEAN) {
        float s = 0.f;
        for (size_t j = lane; j < cols; j += 32) s += __half2float(x[j]);
        s = warp_sum(s);
        if (lane == 0) out[r] = __float2half_rn(OP == TL_REDUCE_MEAN ? s / (float)cols : s);
    } else {
        const float sign = OP == TL_REDUCE_MAX ? 1.f : -1.f;    // min(x) = -max(-x); negation is exact
        float bv = 0.f;
        long long bi = -1;
        for (size_t j = lane; j < cols; j += 32) {
            const float v = sign * __half2float(x[j]);
            if (bi < 0 || v > bv) { bv = v; bi = (long long)j; }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
            const long long oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (oi >= 0 && (bi < 0 || ov > bv || (ov == bv && oi < bi))) { bv = ov; bi = oi; }
        }
        if (lane == 0) {
            if (out) out[r] = x[bi];
            if (out_idx) out_idx[r] = (int)bi;
        }
    }
}

// ---------------------------------------------------------------------------------------------
// Type casts (CPU.cpp:462-486, CUDA.cu:440-464)
// ---------------------------------------------------------------------------------------------
template <typename D, typename S>
__global__ void k_cast(D* out, const S* in, size_t n) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        if constexpr (std::is_same<D, __half>::value) out[i] = __float2half_rn(static_cast<float>(in[i]));   // through float, also from int
        else if constexpr (std::is_same<S, __half>::value && std::is_same<D, int>::value) out[i] = __half2int_rz(in[i]);
        else out[i] = static_cast<D>(in[i]);
    }
}

}  // namespace

int launch_contiguous(__half* result, const __half* data, const int* shape, const int* stride, int ndim, size_t offset,
                      size_t n, cudaStream_t st) {
    return launch_strided<0>(result, data, __half(), shape, stride, ndim, offset, n, st);
}
int launch_set_item(__half* data, const __half* src, const int* shape, const int* stride, int ndim, size_t offset,
                    size_t n, cudaStream_t st) {
    return launch_strided<1>(data, src, __half(), shape, stride, ndim, offset, n, st);
}
int launch_set_item_scalar(__half* data, __half value, const int* shape, const int* stride, int ndim, size_t offset,
                           size_t n, cudaStream_t st) {
    return launch_strided<2>(data, nullptr, value, shape, stride, ndim, offset, n, st);
}

int launch_unary(__half* out, const __half* in, size_t n, int op, cudaStream_t st) {
    if (n == 0) return TL_OK;
    const bool vec = n % 8 == 0 && al16(out) && al16(in);
    const unsigned grid = grid_for(vec ? n / 8 : n, 256);
    switch (op) {
        case TL_UNARY_NEG: k_unary_direct<0><<<grid, 256, 0, st>>>(out, in, n, vec); break;
        case TL_UNARY_ABS: k_unary_direct<1><<<grid, 256, 0, st>>>(out, in, n, vec); break;
        case TL_UNARY_SQRT: k_unary_direct<2><<<grid, 256, 0, st>>>(out, in, n, vec); break;
        case TL_UNARY_RSQRT: k_unary_direct<3><<<grid, 256, 0, st>>>(out, in, n, vec); break;
        case TL_UNARY_SILU: return launch_lookup(out, in, n, tables().silu_float_tab, st);
        case TL_UNARY_SILU_CPU_HALF: return launch_lookup(out, in, n, tables().silu_half_tab, st);
        case TL_UNARY_SIN: case TL_UNARY_COS: case TL_UNARY_EXP: case TL_UNARY_LOG: case TL_UNARY_TANH: {
            const __half* tab;
            TL_PROPAGATE(table_for_unary(op, &tab));
            return launch_lookup(out, in, n, tab, st);
        }
        default: return set_error(TL_ERR_INVALID_ARGUMENT, "unknown unary op %d", op);
    }
    TL_LAUNCH_CHECK();
    return TL_OK;
}

int launch_binary_op(__half* out, const __half* a, const __half* b, size_t n, int op, cudaStream_t st) {
    if (n == 0) return TL_OK;
    return launch_binary_any<false>(out, a, b, __half(), n, op, st);
}

int launch_binary_scalar(__half* out, const __half* a, __half s, size_t n, int op, cudaStream_t st) {
    if (n == 0) return TL_OK;
    if (op == TL_BINARY_POW) {
        const __half* tab;
        TL_PROPAGATE(table_for_pow(s, &tab, st));
        return launch_lookup(out, a, n, tab, st);
    }
    return launch_binary_any<true>(out, a, nullptr, s, n, op, st);
}

int launch_reduce(__half* out, const __half* in, size_t reduce_size, size_t n, int op, int numerics, cudaStream_t st) {
    TL_REQUIRE(reduce_size > 0 && n % reduce_size == 0, "reduce: %zu elements do not split into rows of %zu", n, reduce_size);
    TL_REQUIRE(op >= TL_REDUCE_MAX && op <= TL_REDUCE_MEAN, "unknown reduce op %d", op);
    const size_t rows = n / reduce_size;
    if (rows == 0) return TL_OK;
    const bool exact_either_way = op == TL_REDUCE_MAX || op == TL_REDUCE_MIN;   // the parallel form keeps the first of equal values
    if (numerics == TL_NUMERICS_REFERENCE_ORDER && !exact_either_way) {
        const __half hcols = __float2half((float)reduce_size);                  // static_cast<dtype>(reduce_size), CPU.cpp:393
        const unsigned grid = (unsigned)ceil_div(rows, 128);
        if (op == TL_REDUCE_SUM) k_reduce_seq<TL_REDUCE_SUM><<<grid, 128, 0, st>>>(out, in, rows, reduce_size, hcols);
        else k_reduce_seq<TL_REDUCE_MEAN><<<grid, 128, 0, st>>>(out, in, rows, reduce_size, hcols);
    } else {
        const unsigned grid = (unsigned)ceil_div(rows, 8);
        switch (op) {
            case TL_REDUCE_MAX: k_reduce_warp<TL_REDUCE_MAX><<<grid, 256, 0, st>>>(out, nullptr, in, rows, reduce_size); break;
            case TL_REDUCE_MIN: k_reduce_warp<TL_REDUCE_MIN><<<grid, 256, 0, st>>>(out, nullptr, in, rows, reduce_size); break;
            case TL_REDUCE_SUM: k_reduce_warp<TL_REDUCE_SUM><<<grid, 256, 0, st>>>(out, nullptr, in, rows, reduce_size); break;
            default: k_reduce_warp<TL_REDUCE_MEAN><<<grid, 256, 0, st>>>(out, nullptr, in, rows, reduce_size); break;
        }
    }
    TL_LAUNCH_CHECK();
    return TL_OK;
}

int launch_argreduce(int* out_idx, const __half* in, size_t reduce_size, size_t n, int want_min, cudaStream_t st) {
    TL_REQUIRE(reduce_size > 0 && reduce_size < 0x7fffffffu && n % reduce_size == 0, "argreduce: bad shape");
    const size_t rows = n / reduce_size;
    if (rows == 0) return TL_OK;
    const unsigned grid = (unsigned)ceil_div(rows, 8);
    if (want_min) k_reduce_warp<TL_REDUCE_MIN><<<grid, 256, 0, st>>>(nullptr, out_idx, in, rows, reduce_size);
    else k_reduce_warp<TL_REDUCE_MAX><<<grid, 256, 0, st>>>(nullptr, out_idx, in, rows, reduce_size);
    TL_LAUNCH_CHECK();
    return TL_OK;
}

int launch_cast(void* out, const void* in, size_t n, int kind, cudaStream_t st) {
    if (n == 0) return TL_OK;
    const unsigned grid = grid_for(n, 256);
    switch (kind) {
        case TL_CAST_F16_TO_F32: k_cast<float, __half><<<grid, 256, 0, st>>>(static_cast<float*>(out), static_cast<const __half*>(in), n); break;
        case TL_CAST_F32_TO_F16: k_cast<__half, float><<<grid, 256, 0, st>>>(static_cast<__half*>(out), static_cast<const float*>(in), n); break;
        case TL_CAST_F16_TO_I32: k_cast<int, __half><<<grid, 256, 0, st>>>(static_cast<int*>(out), static_cast<const __half*>(in), n); break;
        case TL_CAST_I32_TO_F16: k_cast<__half, int><<<grid, 256, 0, st>>>(static_cast<__half*>(out), static_cast<const int*>(in), n); break;
        default: return set_error(TL_ERR_INVALID_ARGUMENT, "unknown cast %d", kind);
    }
    TL_LAUNCH_CHECK();
    return TL_OK;
}

}  // namespace tlb
