/* TEST INFRASTRUCTURE — not part of the product, never linked into it.
 *
 * Plain-C restatement of the reference's CPU ("cpu" device, OpenMP) arithmetic for the
 * Tensor::matmul -> Llama2 forward path. Every function names the reference lines it follows.
 * fp16 values travel as uint16_t bit patterns; the reference's host `half` arithmetic is
 * "convert both operands to float, operate in float, round once to half" (cuda_fp16.hpp host
 * branches of __hadd/__hsub/__hmul/__hdiv), which is what hadd()/hmul()/... below do.
 *
 * Pinning: the reference holds no golden vectors for this path; this file is pinned against the
 * reference's own code run in the build container (oracle/_ref, built by oracle/Makefile from the
 * unmodified sources) by tests/test_oracle.py and against the fixtures under tests/golden/
 * that were generated from that same library (tests/golden/make_golden.py).
 *
 * Known reference behaviour kept on purpose:
 *   - RMSNorm sums x^2 sequentially IN FP16 (reduceOperation, CPU.cpp:342-353).
 *   - softmax: fp16 max, exp evaluated in DOUBLE and rounded straight to fp16, fp16 sequential
 *     sum, fp16 divide (softmax.cpp:10-31).
 *   - argmax keeps the lowest index on ties (strict '>', CPU.cpp:358-372).
 *   - silu_mode 0 keeps the CPU fp16 SiLU's sign defect 1/(1+exp(x)) (CPU.cpp:216-219);
 *     silu_mode 1 is the float route x*(1/(1+expf(-x))) rounded once (CPU.cpp:220-222).
 *
 * One operator exists in two restatements. The CPU RMSNorm's fp16 running sum stops growing once
 * it reaches 2048 (an addend below half an ulp of the sum is rounded away), so at dim 4096 the
 * CPU result carries a 3-5 % scale error against exact arithmetic; at dim <= 512 it is below
 * 0.2 %. The reference's CUDA backend computes the same operator with an fp32 sum
 * (rms_norm_kernel_v1, tensorLib/src/device/cuda/rms_norm.cu:138-167). rmsnorm() below is the CPU
 * form (bit-identical to the reference CPU code); rmsnorm_cuda_route() restates the CUDA kernel
 * and is what the Llama2 forward uses when bit 1 of silu_mode is set. That second form cannot be
 * pinned in a GPU-less container: tests/test_gpu_ref_cuda.py compares it on the GPU with the
 * reference's own kernel (compiled into oracle/_ref) to within one fp16 ulp.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#include <stdio.h>
#include <omp.h>

typedef uint16_t h16;

static _Thread_local char g_err[256];
static int fail(const char* msg) { snprintf(g_err, sizeof g_err, "%s", msg); return 1; }
const char* orc_last_error(void) { return g_err; }
int orc_omp_max_threads(void) { return omp_get_max_threads(); }
void orc_omp_set_threads(int n) { omp_set_num_threads(n); }

/* ---- fp16 <-> fp32/fp64 ------------------------------------------------------------------- */
static inline float h2f(h16 h) {
    uint32_t s = (uint32_t)(h & 0x8000u) << 16, e = (h >> 10) & 0x1Fu, m = h & 0x3FFu, u;
    if (e == 0) {
        if (m == 0) u = s;
        else { /* subnormal: normalise */
            int sh = 0;
            while (!(m & 0x400u)) { m <<= 1; sh++; }
            u = s | ((uint32_t)(113 - sh) << 23) | ((m & 0x3FFu) << 13);
        }
    } else if (e == 31) u = s | 0x7F800000u | (m << 13);
    else u = s | ((e + 112u) << 23) | (m << 13);
    float f; memcpy(&f, &u, 4); return f;
}

/* round-to-nearest-even of a double to fp16 in ONE rounding step */
static inline h16 d2h(double d) {
    uint64_t u; memcpy(&u, &d, 8);
    h16 s = (h16)((u >> 48) & 0x8000u);
    uint64_t a = u & 0x7FFFFFFFFFFFFFFFull;
    if (a >= 0x7FF0000000000000ull) return (h16)(s | (a > 0x7FF0000000000000ull ? 0x7FFFu : 0x7C00u));
    int e = (int)(a >> 52) - 1023;               /* unbiased exponent */
    uint64_t m = (a & 0xFFFFFFFFFFFFFull) | (1ull << 52);
    if (a == 0) return s;
    if (e > 15) return (h16)(s | 0x7C00u);       /* overflow (65520 rounds to inf as well, below) */
    int shift;                                   /* bits of m dropped */
    int he;
    if (e >= -14) { shift = 42; he = e + 15; }   /* normal half: keep 11 significant bits */
    else { shift = 42 + (-14 - e); he = 0; }     /* subnormal half */
    if (shift > 63) return s;                    /* far below the smallest subnormal */
    uint64_t keep = m >> shift, rem = m & ((1ull << shift) - 1), halfway = 1ull << (shift - 1);
    if (rem > halfway || (rem == halfway && (keep & 1))) keep++;
    uint32_t r;
    if (he == 0) r = (uint32_t)keep;             /* may carry into the first normal, which is right */
    else r = ((uint32_t)he << 10) + (uint32_t)(keep - 0x400u); /* carry bumps the exponent */
    if (r >= 0x7C00u) r = 0x7C00u;
    return (h16)(s | r);
}
/* float -> half: a float is exactly a double, so one rounding */
static inline h16 f2h(float f) { return d2h((double)f); }

static inline h16 hadd(h16 a, h16 b) { return f2h(h2f(a) + h2f(b)); }
static inline h16 hsub(h16 a, h16 b) { return f2h(h2f(a) - h2f(b)); }
static inline h16 hmul(h16 a, h16 b) { return f2h(h2f(a) * h2f(b)); }
static inline h16 hdiv(h16 a, h16 b) { return f2h(h2f(a) / h2f(b)); }

/* ---- Device::matmul2d, CPU.cpp:76-89 -------------------------------------------------------- */
static void matmul2d(const h16* A, const h16* B, h16* C, int M, int N, int K) {
    #pragma omp parallel for collapse(2)
    for (int i = 0; i < M; i++)
        for (int j = 0; j < N; j++) {
            float sum = 0.0f;
            const h16* a = A + (size_t)i * K;
            const h16* b = B + (size_t)j * K;
            for (int k = 0; k < K; k++) sum += h2f(a[k]) * h2f(b[k]);
            C[(size_t)i * N + j] = f2h(sum);
        }
}
int orc_matmul2d_f16(const h16* A, const h16* B, h16* C, int M, int N, int K) {
    matmul2d(A, B, C, M, N, K); return 0;
}
/* nn::Linear::forward (linear.cpp:43-49) reaches matmul2d(M=T,N=out,K=in) through call2
 * (matmul.cpp:206-324) with B = the [out,in] weight as stored. */
int orc_linear_f16(const h16* x, const h16* W, h16* y, int T, int in_f, int out_f) {
    matmul2d(x, W, y, T, out_f, in_f); return 0;
}
/* call2's batch loop (matmul.cpp:297-321): one matmul2d per batch matrix */
int orc_bmm_nt_f16(const h16* a, const h16* bt, h16* c, int B, int M, int N, int K) {
    for (int b = 0; b < B; b++)
        matmul2d(a + (size_t)b * M * K, bt + (size_t)b * N * K, c + (size_t)b * M * N, M, N, K);
    return 0;
}

/* Device::matmul, the strided batched form, CPU.cpp:18-68: one sequential fp32 dot product per
 * result element, operands addressed through per-dimension strides. */
int orc_matmul_strided_f16(const h16* lhs, const h16* rhs, h16* result, const int* lhs_stride, const int* rhs_stride,
                           size_t lhs_offset, size_t rhs_offset, const int* result_shape, int ndim,
                           size_t result_elements, size_t K) {
    #pragma omp parallel for
    for (size_t idx = 0; idx < result_elements; idx++) {
        size_t lin = idx;
        long long Aoff = (long long)lhs_offset, Boff = (long long)rhs_offset;
        for (int i = ndim - 1; i >= 0; i--) {
            int cur = (int)(lin % (size_t)result_shape[i]);
            lin /= (size_t)result_shape[i];
            if (i != ndim - 1) Aoff += (long long)cur * lhs_stride[i];
            if (i != ndim - 2) Boff += (long long)cur * rhs_stride[i];
        }
        float sum = 0.0f;
        const int t1 = lhs_stride[ndim - 1], t2 = rhs_stride[ndim - 2];
        for (size_t k = 0; k < K; k++) sum += h2f(lhs[Aoff + (long long)k * t1]) * h2f(rhs[Boff + (long long)k * t2]);
        result[idx] = f2h(sum);
    }
    return 0;
}

/* ---- nn::RMSNorm::forward_plain, rmsNorm.cpp:15-56 ------------------------------------------ */
static int rmsnorm(const h16* x, const h16* w, h16* y, int T, int dim, float eps) {
    h16 heps = f2h(eps);                       /* float eps -> dtype scalar of operator+ */
    h16 hdim = f2h((float)dim);                /* static_cast<dtype>(reduce_size), CPU.cpp:393 */
    for (int t = 0; t < T; t++) {
        const h16* xr = x + (size_t)t * dim;
        h16 s = f2h(powf(h2f(xr[0]), 2.0f));    /* pow(2): powFunc, CPU.cpp:295-300 */
        for (int j = 1; j < dim; j++)          /* sequential fp16 running sum, CPU.cpp:346-351 */
            s = hadd(s, f2h(powf(h2f(xr[j]), 2.0f)));
        h16 mean = hdiv(s, hdim);              /* CPU.cpp:389-395 */
        h16 v = hadd(mean, heps);              /* temp + eps */
        float vf = h2f(v);
        if (!(vf > 0.0f)) return fail("Cannot take sqrt of non-positive values."); /* CPU.cpp:242-246 */
        h16 r = f2h(1 / sqrtf(vf));            /* rsqrtFunc */
        for (int j = 0; j < dim; j++)
            y[(size_t)t * dim + j] = hmul(hmul(xr[j], r), w[j]);   /* x*temp, then *weight */
    }
    return 0;
}
int orc_rmsnorm_f16(const h16* x, const h16* w, h16* y, int T, int dim, float eps) {
    return rmsnorm(x, w, y, T, dim, eps);
}

/* ---- CUDA<half>::rms_norm = rms_norm_kernel_v1 (tensorLib/src/device/cuda/rms_norm.cu:138-167):
 * one warp per token row; lane i adds float(x[j])*float(x[j]) for j = i, i+32, ... in fp32 (the
 * product of two halves is exact in fp32, so a fused multiply-add rounds like multiply-then-add),
 * the 32 lane sums are added across the warp (cg::reduce; taken here as a butterfly over lane
 * distances 16, 8, 4, 2, 1 - the order is not documented, which is why the comparison with the
 * real kernel allows one ulp), rms = half(sqrtf(sum / hidden + eps)), and
 * out[j] = (x[j] * w[j]) / rms with every half operation rounded once. */
static int rmsnorm_cuda_route(const h16* x, const h16* w, h16* y, int T, int dim, float eps) {
    for (int t = 0; t < T; t++) {
        const h16* xr = x + (size_t)t * dim;
        float lane[32];
        for (int i = 0; i < 32; i++) {
            float s = 0.0f;
            for (int j = i; j < dim; j += 32) s += h2f(xr[j]) * h2f(xr[j]);
            lane[i] = s;
        }
        for (int o = 16; o > 0; o >>= 1)
            for (int i = 0; i < o; i++) lane[i] = lane[i] + lane[i + o];
        h16 rms = f2h(sqrtf(lane[0] / (float)dim + eps));
        for (int j = 0; j < dim; j++) y[(size_t)t * dim + j] = hdiv(hmul(xr[j], w[j]), rms);
    }
    return 0;
}
int orc_rmsnorm_cuda_route_f16(const h16* x, const h16* w, h16* y, int T, int dim, float eps) {
    return rmsnorm_cuda_route(x, w, y, T, dim, eps);
}

/* ---- apply_rotary_emb, CPU.cpp:427-461 ------------------------------------------------------- */
static void rope(const h16* x, h16* y, int start_pos, int T, int H, int hd) {
    for (int t = 0; t < T; t++)
        for (int h = 0; h < H; h++)
            for (int d = 0; d < hd; d += 2) {
                size_t off = ((size_t)t * H + h) * hd + d;
                float theta = (start_pos + t) * 1.0f / powf(10000.0f, (float)d / (float)hd);
                h16 c = f2h(cosf(theta)), s = f2h(sinf(theta));
                h16 v0 = x[off], v1 = x[off + 1];
                y[off] = hsub(hmul(v0, c), hmul(v1, s));
                y[off + 1] = hadd(hmul(v0, s), hmul(v1, c));
            }
}
int orc_rope_f16(const h16* x, h16* y, int start_pos, int T, int H, int hd) {
    rope(x, y, start_pos, T, H, hd); return 0;
}

/* ---- softmax over the last dim, softmax.cpp:10-31 -------------------------------------------- */
static void softmax(const h16* x, h16* y, int rows, int cols) {
    #pragma omp parallel for
    for (int i = 0; i < rows; i++) {
        const h16* in = x + (size_t)i * cols;
        h16* out = y + (size_t)i * cols;
        h16 mx = in[0];
        for (int j = 1; j < cols; j++) if (h2f(in[j]) > h2f(mx)) mx = in[j];
        h16 sum = 0;
        for (int j = 0; j < cols; j++) {
            out[j] = d2h(exp((double)h2f(hsub(in[j], mx))));   /* ::exp(double), half(double) */
            sum = hadd(sum, out[j]);
        }
        for (int j = 0; j < cols; j++) out[j] = hdiv(out[j], sum);
    }
}
int orc_softmax_f16(const h16* x, h16* y, int rows, int cols) { softmax(x, y, rows, cols); return 0; }

/* ---- SiLU ------------------------------------------------------------------------------------ */
static inline h16 silu_half_as_is(h16 x) {      /* CPU.cpp:216-219 */
    h16 sig = f2h(1 / (1 + expf(h2f(x))));
    return hmul(x, sig);
}
static inline h16 silu_via_float(h16 x) {       /* type_cast -> CPU.cpp:220-222 -> type_cast */
    float xf = h2f(x);
    float sig = 1 / (1 + expf(-xf));
    return f2h(xf * sig);
}
int orc_silu_f16(const h16* x, h16* y, int n, int via_float) {
    for (int i = 0; i < n; i++) y[i] = via_float ? silu_via_float(x[i]) : silu_half_as_is(x[i]);
    return 0;
}

/* ---- elementwise add / mul / scalar-div (CPU.cpp:277-293) ------------------------------------- */
int orc_ewise_f16(const h16* a, const h16* b, h16* y, int n, int op, double scalar) {
    if (op == 2) {
        h16 hs = d2h(scalar);                   /* double -> dtype scalar */
        if (h2f(hs) == 0) return fail("Division by zero.");
        for (int i = 0; i < n; i++) y[i] = hdiv(a[i], hs);
    } else if (op == 0) for (int i = 0; i < n; i++) y[i] = hadd(a[i], b[i]);
    else for (int i = 0; i < n; i++) y[i] = hmul(a[i], b[i]);
    return 0;
}

/* ---- argmax over the last dim, CPU.cpp:358-372 ------------------------------------------------ */
static void argmax(const h16* x, int* idx, int rows, int cols) {
    for (int i = 0; i < rows; i++) {
        const h16* r = x + (size_t)i * cols;
        h16 best = r[0]; int bi = 0;
        for (int j = 1; j < cols; j++) if (h2f(r[j]) > h2f(best)) { best = r[j]; bi = j; }
        idx[i] = bi;
    }
}
int orc_argmax_f16(const h16* x, int* idx, int rows, int cols) { argmax(x, idx, rows, cols); return 0; }


/* ==== the rest of the Device<half> surface (Device.hpp:30-78) ===================================== */
/* convertIdx (CPU.cpp / CUDA.cuh:186-202): digits of i over shape, innermost last */
static size_t convert_idx(size_t i, const int* shape, const int* stride, int ndim, size_t offset) {
    long long off = 0;
    for (int d = ndim - 1; d >= 0; d--) {
        int cur = (int)(i % (size_t)shape[d]);
        i /= (size_t)shape[d];
        off += (long long)cur * stride[d];
    }
    return (size_t)(off + (long long)offset);
}
/* CPU::contiguous / setItemEwise / setItemScalar, CPU.cpp:127-167 */
int orc_contiguous_f16(h16* result, const h16* data, const int* shape, const int* stride, int ndim, size_t offset, size_t n) {
    for (size_t i = 0; i < n; i++) result[i] = data[convert_idx(i, shape, stride, ndim, offset)];
    return 0;
}
int orc_set_item_f16(h16* data, const h16* src, const int* shape, const int* stride, int ndim, size_t offset, size_t n) {
    for (size_t i = 0; i < n; i++) data[convert_idx(i, shape, stride, ndim, offset)] = src[i];
    return 0;
}
int orc_set_item_scalar_f16(h16* data, h16 value, const int* shape, const int* stride, int ndim, size_t offset, size_t n) {
    for (size_t i = 0; i < n; i++) data[convert_idx(i, shape, stride, ndim, offset)] = value;
    return 0;
}
/* unary family, CPU.cpp:169-276. op codes as in include/tensorlib_b200.h (TL_UNARY_*). sqrt / rsqrt of
 * a non-positive value make the reference throw; here they fail the call. */
int orc_unary_f16(const h16* x, h16* y, int n, int op) {
    for (int i = 0; i < n; i++) {
        float f = h2f(x[i]);
        switch (op) {
            case 0: y[i] = f2h(-f); break;                       /* operator- of the host half: through float */
            case 1: y[i] = f2h(sinf(f)); break;
            case 2: y[i] = f2h(cosf(f)); break;
            case 3: y[i] = f2h(expf(f)); break;
            case 4: y[i] = f2h(logf(f)); break;
            case 5: y[i] = f2h(fabsf(f)); break;
            case 6: y[i] = f2h(tanhf(f)); break;
            case 7: y[i] = silu_via_float(x[i]); break;
            case 8: if (!(f > 0.0f)) return fail("Cannot take sqrt of non-positive values."); y[i] = f2h(sqrtf(f)); break;
            case 9: if (!(f > 0.0f)) return fail("Cannot take sqrt of non-positive values."); y[i] = f2h(1 / sqrtf(f)); break;
            case 10: y[i] = silu_half_as_is(x[i]); break;
            default: return fail("unknown unary op");
        }
    }
    return 0;
}
/* binary / scalar arithmetic, CPU.cpp:277-340: 0 add, 1 sub, 2 mul, 3 div, 4 pow */
static int binop(h16 a, h16 b, int op, h16* out) {
    switch (op) {
        case 0: *out = hadd(a, b); return 0;
        case 1: *out = hsub(a, b); return 0;
        case 2: *out = hmul(a, b); return 0;
        case 3: if (h2f(b) == 0) return fail("Division by zero."); *out = hdiv(a, b); return 0;
        case 4: if (h2f(a) == 0 && h2f(b) < 0) return fail("Cannot take negative power of zero.");
                *out = f2h(powf(h2f(a), h2f(b))); return 0;
        default: return fail("unknown binary op");
    }
}
int orc_binary_f16(const h16* a, const h16* b, h16* y, int n, int op) {
    if (op == 4) return fail("pow takes a scalar exponent");
    for (int i = 0; i < n; i++) if (binop(a[i], b[i], op, &y[i])) return 1;
    return 0;
}
int orc_binary_scalar_f16(const h16* a, h16 s, h16* y, int n, int op) {
    for (int i = 0; i < n; i++) if (binop(a[i], s, op, &y[i])) return 1;
    return 0;
}
/* reductions over runs of reduce_size, CPU.cpp:342-402: 0 max, 1 min, 2 sum, 3 mean; sequential in fp16 */
int orc_reduce_f16(const h16* x, h16* y, size_t reduce_size, size_t n, int op) {
    h16 hsize = f2h((float)reduce_size);
    for (size_t i = 0; i < n; i += reduce_size) {
        h16 t = x[i];
        for (size_t j = 1; j < reduce_size; j++) {
            h16 v = x[i + j];
            if (op == 0) t = (h2f(t) < h2f(v)) ? v : t;          /* std::max(a, b) */
            else if (op == 1) t = (h2f(v) < h2f(t)) ? v : t;     /* std::min(a, b) */
            else t = hadd(t, v);
        }
        if (op == 3) t = hdiv(t, hsize);
        y[i / reduce_size] = t;
    }
    return 0;
}
int orc_argreduce_f16(const h16* x, int* idx, size_t reduce_size, size_t n, int want_min) {
    for (size_t i = 0; i < n; i += reduce_size) {
        h16 best = x[i]; int bi = 0;
        for (size_t j = 1; j < reduce_size; j++) {
            int better = want_min ? (h2f(x[i + j]) < h2f(best)) : (h2f(x[i + j]) > h2f(best));
            if (better) { best = x[i + j]; bi = (int)j; }
        }
        idx[i / reduce_size] = bi;
    }
    return 0;
}
/* type_cast, CPU.cpp:462-486: 0 half->float, 1 float->half, 2 half->int (truncation), 3 int->half (through float) */
int orc_cast(const void* in, void* out, size_t n, int kind) {
    for (size_t i = 0; i < n; i++) {
        if (kind == 0) ((float*)out)[i] = h2f(((const h16*)in)[i]);
        else if (kind == 1) ((h16*)out)[i] = f2h(((const float*)in)[i]);
        else if (kind == 2) ((int*)out)[i] = (int)h2f(((const h16*)in)[i]);
        else if (kind == 3) ((h16*)out)[i] = f2h((float)((const int*)in)[i]);
        else return fail("unknown cast");
    }
    return 0;
}

/* ---- Llama2 forward ---------------------------------------------------------------------------
 * Transformer::forward (Transformer.cpp:264-299) with TransformerBlock::forward (:162-178),
 * Attention::forward (:28-112) and FeedForward::forward (:133-145). The norm result is used as
 * the block input (what the reference's CUDA path does; its CPU path forgets the store). */
typedef struct {
    int dim, hidden, L, H, V, S, hd;
    h16 *emb, *attn_norm, *wq, *wk, *wv, *wo, *ffn_norm, *w1, *w2, *w3, *norm, *wcls;
    h16 *cache_k, *cache_v;                    /* (L, S, H, hd) like the reference's per-layer caches */
} Model;

void* orc_llama2_create(int dim, int hidden, int n_layers, int n_heads, int vocab, int max_seq) {
    Model* m = (Model*)calloc(1, sizeof(Model));
    m->dim = dim; m->hidden = hidden; m->L = n_layers; m->H = n_heads; m->V = vocab; m->S = max_seq;
    m->hd = dim / n_heads;
    size_t c = (size_t)n_layers * max_seq * dim;
    m->cache_k = (h16*)calloc(c, 2); m->cache_v = (h16*)calloc(c, 2);
    return m;
}
void orc_llama2_destroy(void* h) {
    Model* m = (Model*)h; if (!m) return;
    free(m->emb); free(m->cache_k); free(m->cache_v); free(m);
}
/* payload order: main.cpp:36-190 */
int orc_llama2_load(void* h, const h16* payload, int shared) {
    Model* m = (Model*)h;
    size_t d = m->dim, hid = m->hidden, L = m->L, V = m->V;
    size_t n = V * d + L * (2 * d + 4 * d * d + 3 * d * hid) + d;
    if (!shared) n += (size_t)m->S * m->hd + V * d;
    free(m->emb);
    h16* p = (h16*)malloc(n * 2);
    if (!p) return fail("out of memory");
    memcpy(p, payload, n * 2);
    m->emb = p; p += V * d;
    m->attn_norm = p; p += L * d;
    m->wq = p; p += L * d * d;  m->wk = p; p += L * d * d;
    m->wv = p; p += L * d * d;  m->wo = p; p += L * d * d;
    m->ffn_norm = p; p += L * d;
    m->w1 = p; p += L * d * hid; m->w2 = p; p += L * d * hid; m->w3 = p; p += L * d * hid;
    m->norm = p; p += d;
    if (shared) m->wcls = m->emb;
    else { p += (size_t)m->S * m->hd; m->wcls = p; }
    return 0;
}

/* silu_mode bit 0: SiLU route (see the header); bit 1: RMSNorm as the reference's CUDA backend
 * computes it (fp32 sum) instead of the CPU's fp16 running sum. */
int orc_llama2_forward(void* hmodel, const int* tokens, int T, int pos, int silu_mode,
                       h16* logits_out, h16* hidden_out) {
    Model* m = (Model*)hmodel;
    int (*const norm)(const h16*, const h16*, h16*, int, int, float) = (silu_mode & 2) ? rmsnorm_cuda_route : rmsnorm;
    silu_mode &= 1;
    const int dim = m->dim, hid = m->hidden, H = m->H, hd = m->hd, S = pos + T;
    if (S > m->S) return fail("sequence exceeds max_seq_len");
    size_t td = (size_t)T * dim;
    h16 *x = malloc(td * 2), *xn = malloc(td * 2), *q = malloc(td * 2), *k = malloc(td * 2),
        *v = malloc(td * 2), *att = malloc(td * 2), *hres = malloc(td * 2), *ao = malloc(td * 2),
        *g = malloc((size_t)T * hid * 2), *u = malloc((size_t)T * hid * 2),
        *sc = malloc((size_t)H * T * S * 2), *pr = malloc((size_t)H * T * S * 2);
    h16 hscale = d2h(sqrt((double)hd));       /* ScalarDiv(sqrt(head_dim)), Transformer.cpp:94 */
    int rc = 0;
    for (int t = 0; t < T; t++) {             /* Embedding::forward, embedding.cpp:48-81 */
        if (tokens[t] < 0 || tokens[t] >= m->V) { rc = fail("token id out of range"); goto done; }
        memcpy(x + (size_t)t * dim, m->emb + (size_t)tokens[t] * dim, dim * 2);
    }
    for (int l = 0; l < m->L; l++) {
        size_t wo2 = (size_t)l * dim * dim, wf = (size_t)l * dim * hid;
        h16* ck = m->cache_k + (size_t)l * m->S * dim;
        h16* cv = m->cache_v + (size_t)l * m->S * dim;
        if ((rc = norm(x, m->attn_norm + (size_t)l * dim, xn, T, dim, 1e-5f))) goto done;
        matmul2d(xn, m->wq + wo2, q, T, dim, dim);
        matmul2d(xn, m->wk + wo2, k, T, dim, dim);
        matmul2d(xn, m->wv + wo2, v, T, dim, dim);
        rope(q, q, pos, T, H, hd);
        rope(k, k, pos, T, H, hd);
        memcpy(ck + (size_t)pos * dim, k, td * 2);   /* cache (1,S,H,hd), Transformer.cpp:51-53 */
        memcpy(cv + (size_t)pos * dim, v, td * 2);
        /* scores[h,t,s] = q[t,h,:].k[s,h,:] -> fp16, / sqrt(hd), + mask (:92-102) */
        #pragma omp parallel for collapse(2)
        for (int h = 0; h < H; h++)
            for (int t = 0; t < T; t++)
                for (int s = 0; s < S; s++) {
                    float sum = 0.0f;
                    const h16* qq = q + ((size_t)t * H + h) * hd;
                    const h16* kk = ck + ((size_t)s * H + h) * hd;
                    for (int d = 0; d < hd; d++) sum += h2f(qq[d]) * h2f(kk[d]);
                    h16 e = hdiv(f2h(sum), hscale);
                    if (T > 1) e = hadd(e, (s > pos + t) ? (h16)0xFC00u : (h16)0);  /* get_mask :233-261 */
                    sc[((size_t)h * T + t) * S + s] = e;
                }
        softmax(sc, pr, H * T, S);                   /* :105 */
        /* out[t,h,d] = sum_s p[h,t,s] v[s,h,d] (:107-109) */
        #pragma omp parallel for collapse(2)
        for (int h = 0; h < H; h++)
            for (int t = 0; t < T; t++)
                for (int d = 0; d < hd; d++) {
                    float sum = 0.0f;
                    const h16* pp = pr + ((size_t)h * T + t) * S;
                    for (int s = 0; s < S; s++) sum += h2f(pp[s]) * h2f(cv[((size_t)s * H + h) * hd + d]);
                    att[((size_t)t * H + h) * hd + d] = f2h(sum);
                }
        matmul2d(att, m->wo + wo2, ao, T, dim, dim);            /* :111 */
        for (size_t i = 0; i < td; i++) hres[i] = hadd(x[i], ao[i]);   /* :169 */
        if ((rc = norm(hres, m->ffn_norm + (size_t)l * dim, xn, T, dim, 1e-5f))) goto done;
        matmul2d(xn, m->w1 + wf, g, T, hid, dim);               /* :136 */
        for (size_t i = 0; i < (size_t)T * hid; i++)
            g[i] = silu_mode ? silu_via_float(g[i]) : silu_half_as_is(g[i]);   /* :137 */
        matmul2d(xn, m->w3 + wf, u, T, hid, dim);               /* :139 */
        for (size_t i = 0; i < (size_t)T * hid; i++) g[i] = hmul(g[i], u[i]);  /* :141 */
        matmul2d(g, m->w2 + wf, ao, T, dim, hid);               /* :143 */
        for (size_t i = 0; i < td; i++) x[i] = hadd(hres[i], ao[i]);   /* :175, :291 */
        if (hidden_out) memcpy(hidden_out + (size_t)l * td, x, td * 2);
    }
    if ((rc = norm(x, m->norm, xn, T, dim, 1e-5f))) goto done;         /* :295 */
    matmul2d(xn, m->wcls, logits_out, T, m->V, dim);                   /* :296, all positions */
done:
    free(x); free(xn); free(q); free(k); free(v); free(att); free(hres); free(ao);
    free(g); free(u); free(sc); free(pr);
    return rc;
}
