// Reference-order kernels: every rounding point and every accumulation order of the reference's
// CPU backend, so results are bit-identical to it. Parallelism is only across independent
// outputs; each dependent chain (a dot product, a running fp16 sum) stays sequential.
// Also the elementwise / gather / argmax kernels that are the same in both numerics.
#include "kernels.cuh"

namespace tlb {

// ---------------------------------------------------------------------------------------------
// Device::matmul2d on the CPU (tensorLib/src/device/cpu/CPU.cpp:76-89) and the strided batched
// Device::matmul (CPU.cpp:18-68): float sum = 0; for k ascending: sum += float(a)*float(b);
// one cast. fp16 x fp16 products are exact in fp32, so fmaf(a, b, sum) rounds exactly like the
// reference's separate multiply and add.
// ---------------------------------------------------------------------------------------------
template <bool VEC>
__global__ void k_matmul_seq(SeqMatmul p) {
    const int n = blockIdx.x * blockDim.x + threadIdx.x;
    const int m = blockIdx.y;
    const int b = blockIdx.z;
    if (n >= p.N) return;
    const __half* a = p.A + (long long)b * p.sA + (long long)m * p.a_m;
    const __half* w = p.B + (long long)b * p.sB + (long long)n * p.b_n;
    float sum = 0.0f;
    if (VEC) {  // unit k-strides, K % 8 == 0, 16-byte aligned rows
        const uint4* a4 = reinterpret_cast<const uint4*>(a);
        const uint4* w4 = reinterpret_cast<const uint4*>(w);
        for (int k8 = 0; k8 < p.K / 8; k8++) {
            uint4 av = a4[k8], wv = w4[k8];
            const __half* ah = reinterpret_cast<const __half*>(&av);
            const __half* wh = reinterpret_cast<const __half*>(&wv);
#pragma unroll
            for (int i = 0; i < 8; i++) sum = fmaf(__half2float(ah[i]), __half2float(wh[i]), sum);
        }
    } else {
        for (int k = 0; k < p.K; k++)
            sum = fmaf(__half2float(a[(long long)k * p.a_k]), __half2float(w[(long long)k * p.b_k]), sum);
    }
    p.C[(long long)b * p.sC + (long long)m * p.c_m + n] = __float2half_rn(sum);
}

int launch_matmul_seq(const SeqMatmul& p, cudaStream_t st) {
    if (p.batch <= 0 || p.M <= 0 || p.N <= 0) return TL_OK;
    TL_REQUIRE(p.M <= 65535 && p.batch <= 65535, "reference-order matmul: M and batch must be <= 65535");
    auto al16 = [](const void* q) { return (reinterpret_cast<uintptr_t>(q) & 15) == 0; };
    bool vec = p.a_k == 1 && p.b_k == 1 && p.K % 8 == 0 && p.K > 0 && al16(p.A) && al16(p.B) &&
               p.a_m % 8 == 0 && p.b_n % 8 == 0 && p.sA % 8 == 0 && p.sB % 8 == 0;
    dim3 block(128), grid((unsigned)ceil_div(p.N, 128), p.M, p.batch);
    if (vec) k_matmul_seq<true><<<grid, block, 0, st>>>(p);
    else k_matmul_seq<false><<<grid, block, 0, st>>>(p);
    TL_LAUNCH_CHECK();
    return TL_OK;
}

// ---------------------------------------------------------------------------------------------
// nn::RMSNorm::forward_plain (tensorLib/src/nn/rmsNorm.cpp:15-56): pow(2) -> fp16; mean = fp16
// SEQUENTIAL running sum (reduceOperation, CPU.cpp:342-353) / half(dim) (CPU.cpp:389-395);
// + half(eps); rsqrt through float (CPU.cpp:240-254); x*r -> fp16; *weight -> fp16.
// One block per token; thread 0 owns the sequential sum.
// ---------------------------------------------------------------------------------------------
__global__ void k_rmsnorm_seq(__half* out, const __half* in, const __half* w, float eps, int hidden) {
    extern __shared__ __half sq[];
    __shared__ __half r_sh;
    const __half* x = in + (size_t)blockIdx.x * hidden;
    for (int j = threadIdx.x; j < hidden; j += blockDim.x) {
        float xf = __half2float(x[j]);
        sq[j] = __float2half_rn(__fmul_rn(xf, xf));  // powf(x, 2) is exact for fp16 inputs
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        __half s = sq[0];
        for (int j = 1; j < hidden; j++) s = hadd_ref(s, sq[j]);
        __half mean = hdiv_ref(s, __float2half_rn((float)hidden));
        __half v = hadd_ref(mean, __float2half_rn(eps));
        // the reference throws for v <= 0; here that yields NaN/inf outputs instead
        r_sh = __float2half_rn(__fdiv_rn(1.0f, __fsqrt_rn(__half2float(v))));
    }
    __syncthreads();
    const __half r = r_sh;
    for (int j = threadIdx.x; j < hidden; j += blockDim.x)
        out[(size_t)blockIdx.x * hidden + j] = hmul_ref(hmul_ref(x[j], r), w[j]);
}

int launch_rmsnorm_seq(__half* out, const __half* in, const __half* w, float eps, int hidden,
                       int tokens, cudaStream_t st) {
    if (tokens <= 0) return TL_OK;
    TL_REQUIRE(hidden > 0 && hidden <= 24576, "rms_norm: hidden %d out of range", hidden);
    k_rmsnorm_seq<<<tokens, 256, (size_t)hidden * sizeof(__half), st>>>(out, in, w, eps, hidden);
    TL_LAUNCH_CHECK();
    return TL_OK;
}

// ---------------------------------------------------------------------------------------------
// softmax over the last dim (tensorLib/src/device/cpu/softmax.cpp:10-31): fp16 max (strict '>'),
// e = half(exp(double(x - max))) via the host-built table, fp16 SEQUENTIAL sum starting from 0,
// fp16 divide. One block per row; thread 0 owns the running sum.
// ---------------------------------------------------------------------------------------------
__global__ void k_softmax_seq(__half* out, const __half* in, size_t cols, const __half* exp_tab) {
    __shared__ float red[32];
    __shared__ __half sum_sh;
    const __half* x = in + (size_t)blockIdx.x * cols;
    __half* y = out + (size_t)blockIdx.x * cols;
    // max: order-independent (ties and signed zeros give the same exp argument)
    float mx = -INFINITY;
    for (size_t j = threadIdx.x; j < cols; j += blockDim.x) mx = fmaxf(mx, __half2float(x[j]));
    mx = warp_max(mx);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = mx;
    __syncthreads();
    if (threadIdx.x < 32) {
        float v = threadIdx.x < (blockDim.x >> 5) ? red[threadIdx.x] : -INFINITY;
        v = warp_max(v);
        if (threadIdx.x == 0) red[0] = v;
    }
    __syncthreads();
    const __half hmx = __float2half_rn(red[0]);  // exact: the max is one of the fp16 inputs
    for (size_t j = threadIdx.x; j < cols; j += blockDim.x) {
        __half d = hsub_ref(x[j], hmx);
        y[j] = exp_tab[__half_as_ushort(d)];
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        __half s = __float2half_rn(0.0f);
        for (size_t j = 0; j < cols; j++) s = hadd_ref(s, y[j]);
        sum_sh = s;
    }
    __syncthreads();
    const __half s = sum_sh;
    for (size_t j = threadIdx.x; j < cols; j += blockDim.x) y[j] = hdiv_ref(y[j], s);
}

int launch_softmax_seq(__half* out, const __half* in, size_t rows, size_t cols, cudaStream_t st) {
    if (rows == 0 || cols == 0) return TL_OK;
    TL_REQUIRE(rows <= 0x7fffffffu, "softmax: too many rows");
    k_softmax_seq<<<(unsigned)rows, 128, 0, st>>>(out, in, cols, tables().exp_tab);
    TL_LAUNCH_CHECK();
    return TL_OK;
}

// scores.ScalarDiv(sqrt(head_dim)) then EwiseAdd(mask) (model/llama2_7b/src/Transformer.cpp:94,
// :99-102; mask values from get_mask :233-261). sqrt is taken in double and converted to fp16.
__global__ void k_scale_mask(__half* sc, int T, int S, int pos, __half hscale, size_t total) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    __half e = hdiv_ref(sc[i], hscale);
    if (T > 1) {
        int s = (int)(i % S);
        int t = (int)((i / S) % T);
        __half mk = __ushort_as_half(s > pos + t ? (unsigned short)0xFC00u : (unsigned short)0);
        e = hadd_ref(e, mk);
    }
    sc[i] = e;
}
int launch_scale_mask(__half* scores, int H, int T, int S, int pos, int head_dim, cudaStream_t st) {
    size_t total = (size_t)H * T * S;
    if (total == 0) return TL_OK;
    __half hscale = __half(sqrt((double)head_dim));
    k_scale_mask<<<(unsigned)ceil_div(total, 256), 256, 0, st>>>(scores, T, S, pos, hscale, total);
    TL_LAUNCH_CHECK();
    return TL_OK;
}

// ---------------------------------------------------------------------------------------------
// apply_rotary_emb (CPU.cpp:427-461): (v0,v1) -> (v0*c - v1*s, v0*s + v1*c), every product and
// the final add/sub rounded to fp16; cos/sin from the host table.
// ---------------------------------------------------------------------------------------------
__global__ void k_rope(const __half* in, __half* out, int start_pos, int T, int n_heads, int head_dim,
                       const __half* cos_t, const __half* sin_t, size_t pairs) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= pairs) return;
    const int half_dim = head_dim / 2;
    int d2 = (int)(i % half_dim);
    size_t row = i / half_dim;                 // (b*T + t)*n_heads + h
    int t = (int)((row / n_heads) % T);
    size_t off = row * head_dim + 2 * (size_t)d2;
    __half c = cos_t[(size_t)(start_pos + t) * half_dim + d2];
    __half s = sin_t[(size_t)(start_pos + t) * half_dim + d2];
    __half v0 = in[off], v1 = in[off + 1];
    out[off] = hsub_ref(hmul_ref(v0, c), hmul_ref(v1, s));
    out[off + 1] = hadd_ref(hmul_ref(v0, s), hmul_ref(v1, c));
}
int launch_rope(const __half* in, __half* out, int start_pos, int rows_bt, int T, int n_heads,
                int head_dim, const __half* cos_t, const __half* sin_t, cudaStream_t st) {
    size_t pairs = (size_t)rows_bt * n_heads * (head_dim / 2);
    if (pairs == 0) return TL_OK;
    k_rope<<<(unsigned)ceil_div(pairs, 256), 256, 0, st>>>(in, out, start_pos, T, n_heads, head_dim,
                                                          cos_t, sin_t, pairs);
    TL_LAUNCH_CHECK();
    return TL_OK;
}

__global__ void k_lookup(__half* out, const __half* in, size_t n, const __half* tab) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = tab[__half_as_ushort(in[i])];
}
int launch_silu(__half* out, const __half* in, size_t n, int via_float, cudaStream_t st) {
    if (n == 0) return TL_OK;
    const __half* tab = via_float ? tables().silu_float_tab : tables().silu_half_tab;
    k_lookup<<<(unsigned)ceil_div(n, 256), 256, 0, st>>>(out, in, n, tab);
    TL_LAUNCH_CHECK();
    return TL_OK;
}

// Device::add / mul (CPU.cpp:277-279): fp16 result of the float operation
__global__ void k_binary(__half* out, const __half* a, const __half* b, size_t n, int op) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = op == 0 ? hadd_ref(a[i], b[i]) : hmul_ref(a[i], b[i]);
}
// the same arithmetic, eight elements per thread (16-byte aligned operands, n % 8 == 0)
__global__ void k_binary_vec(uint4* out, const uint4* a, const uint4* b, size_t n8, int op) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n8) return;
    const uint4 va = a[i], vb = b[i];
    uint4 vo;
    const __half* ha = reinterpret_cast<const __half*>(&va);
    const __half* hb = reinterpret_cast<const __half*>(&vb);
    __half* ho = reinterpret_cast<__half*>(&vo);
#pragma unroll
    for (int j = 0; j < 8; j++) ho[j] = op == 0 ? hadd_ref(ha[j], hb[j]) : hmul_ref(ha[j], hb[j]);
    out[i] = vo;
}
int launch_binary(__half* out, const __half* a, const __half* b, size_t n, int op, cudaStream_t st) {
    if (n == 0) return TL_OK;
    if (n % 8 == 0 && ((reinterpret_cast<uintptr_t>(out) | reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(b)) & 15) == 0) {
        k_binary_vec<<<(unsigned)ceil_div(n / 8, 256), 256, 0, st>>>(reinterpret_cast<uint4*>(out), reinterpret_cast<const uint4*>(a),
                                                                    reinterpret_cast<const uint4*>(b), n / 8, op);
        TL_LAUNCH_CHECK();
        return TL_OK;
    }
    k_binary<<<(unsigned)ceil_div(n, 256), 256, 0, st>>>(out, a, b, n, op);
    TL_LAUNCH_CHECK();
    return TL_OK;
}
__global__ void k_div_scalar(__half* out, const __half* a, __half s, size_t n) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = hdiv_ref(a[i], s);
}
int launch_div_scalar(__half* out, const __half* a, __half scalar, size_t n, cudaStream_t st) {
    if (n == 0) return TL_OK;
    k_div_scalar<<<(unsigned)ceil_div(n, 256), 256, 0, st>>>(out, a, scalar, n);
    TL_LAUNCH_CHECK();
    return TL_OK;
}

// ---------------------------------------------------------------------------------------------
// argmax over the last dim (CPU.cpp:358-372): first element wins unless a later one is strictly
// greater, i.e. the lowest index among equal maxima. One block per row.
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void argmax_merge(float& bv, int& bi, float ov, int oi) {
    if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
}
__global__ void k_argmax(int* out_idx, const __half* in, size_t cols) {
    __shared__ float sv[32];
    __shared__ int si[32];
    const __half* x = in + (size_t)blockIdx.x * cols;
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    for (size_t j = threadIdx.x; j < cols; j += blockDim.x) {
        float v = __half2float(x[j]);
        if (bi == 0x7fffffff || v > bv) { bv = v; bi = (int)j; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        argmax_merge(bv, bi, ov, oi);
    }
    if ((threadIdx.x & 31) == 0) { sv[threadIdx.x >> 5] = bv; si[threadIdx.x >> 5] = bi; }
    __syncthreads();
    if (threadIdx.x < 32) {
        bool has = threadIdx.x < (blockDim.x >> 5);
        bv = has ? sv[threadIdx.x] : -INFINITY;
        bi = has ? si[threadIdx.x] : 0x7fffffff;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            float ov = __shfl_xor_sync(0xffffffffu, bv, o);
            int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            argmax_merge(bv, bi, ov, oi);
        }
        if (threadIdx.x == 0) out_idx[blockIdx.x] = bi == 0x7fffffff ? 0 : bi;
    }
}
int launch_argmax(int* out_idx, const __half* in, size_t rows, size_t cols, cudaStream_t st) {
    if (rows == 0) return TL_OK;
    TL_REQUIRE(cols > 0 && cols < 0x7fffffffu && rows <= 0x7fffffffu, "argmax: bad shape");
    k_argmax<<<(unsigned)rows, 1024, 0, st>>>(out_idx, in, cols);
    TL_LAUNCH_CHECK();
    return TL_OK;
}

// nn::Embedding::forward (tensorLib/src/nn/embedding.cpp:48-81) as a row gather. Ids outside
// [0, vocab) produce a zero row instead of the reference's out-of-bounds read.
__global__ void k_embedding(__half* out, const __half* table, const int* tokens, int dim, int vocab) {
    int tok = tokens[blockIdx.x];
    bool ok = tok >= 0 && tok < vocab;
    const __half* src = table + (size_t)(ok ? tok : 0) * dim;
    for (int j = threadIdx.x; j < dim; j += blockDim.x)
        out[(size_t)blockIdx.x * dim + j] = ok ? src[j] : __float2half_rn(0.0f);
}
int launch_embedding(__half* out, const __half* table, const int* tokens, int n_tokens, int dim,
                     int vocab, cudaStream_t st) {
    if (n_tokens <= 0) return TL_OK;
    k_embedding<<<n_tokens, 256, 0, st>>>(out, table, tokens, dim, vocab);
    TL_LAUNCH_CHECK();
    return TL_OK;
}

__global__ void k_residual_add_f32(__half* out, const __half* a, const float* s, size_t n) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = hadd_ref(a[i], __float2half_rn(s[i]));
}
int launch_residual_add_f32(__half* out, const __half* a, const float* sum32, size_t n, cudaStream_t st) {
    if (n == 0) return TL_OK;
    k_residual_add_f32<<<(unsigned)ceil_div(n, 256), 256, 0, st>>>(out, a, sum32, n);
    TL_LAUNCH_CHECK();
    return TL_OK;
}

__global__ void k_copy_rows(__half* dst, const __half* src, int dim, long long dst_pitch) {
    for (int j = threadIdx.x; j < dim; j += blockDim.x)
        dst[(long long)blockIdx.x * dst_pitch + j] = src[(size_t)blockIdx.x * dim + j];
}
int launch_copy_rows(__half* dst, const __half* src, int rows, int dim, long long dst_pitch,
                     cudaStream_t st) {
    if (rows <= 0) return TL_OK;
    k_copy_rows<<<rows, 256, 0, st>>>(dst, src, dim, dst_pitch);
    TL_LAUNCH_CHECK();
    return TL_OK;
}

}  // namespace tlb
