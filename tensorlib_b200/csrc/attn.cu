// Fast-numerics attention and the small row-wise operators of the prefill path.
//
// Decode attention replaces, for one new token, the reference's chain
//   contiguous copies of the whole K/V prefix -> n_heads GEMVs q.K^T -> ScalarDiv -> softmax ->
//   n_heads GEMVs P.V -> transpose copy        (model/llama2_7b/src/Transformer.cpp:56-109)
// with one kernel that reads the (S, H, hd) caches in place: grid (H, splits); each CTA keeps an
// online-softmax state (max, sum, acc[hd]) in fp32 for its slice of the sequence, writes it to a
// scratch slot, and the last CTA to finish a head merges the slots. HBM-bound on the KV bytes:
// 2 * S * H * hd * 2 bytes per call.
#include <cooperative_groups.h>

#include <mutex>

#include "kernels.cuh"

namespace cg = cooperative_groups;

namespace tlb {

namespace {

constexpr int ATT_WARPS = 4;
constexpr int ATT_THREADS = ATT_WARPS * 32;
constexpr int MAX_HD = 256;   // head_dim <= 256, even
constexpr int HD_ITERS = MAX_HD / 64;

struct AttnArgs {
    const __half* q; const __half* kc; const __half* vc; __half* out;
    float* scratch; unsigned int* counters;
    int H, hd, seq_len, splits;
    const int* pos_ptr; long long pitch; float scale;
};

// Each lane owns the half2 slices d = 2*lane + 64*i of the head dimension.
__global__ void __launch_bounds__(ATT_THREADS) k_decode_attn(AttnArgs p) {
    __shared__ float sm_m[ATT_WARPS], sm_l[ATT_WARPS];
    __shared__ float sm_acc[ATT_WARPS][MAX_HD];
    __shared__ bool is_last;
    const int h = blockIdx.x, split = blockIdx.y;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int hd = p.hd;

    pdl_launch_dependents();
    pdl_wait();
    const int S = p.pos_ptr ? (*p.pos_ptr + 1) : p.seq_len;
    const int per = (S + p.splits - 1) / p.splits;
    const int s_begin = split * per, s_end = min(S, s_begin + per);

    float2 qf[HD_ITERS];
#pragma unroll
    for (int i = 0; i < HD_ITERS; i++) {
        int d = 2 * lane + 64 * i;
        qf[i] = d < hd ? __half22float2(*reinterpret_cast<const __half2*>(p.q + (size_t)h * hd + d))
                       : make_float2(0.f, 0.f);
    }
    float m = -INFINITY, l = 0.f;
    float2 acc[HD_ITERS];
#pragma unroll
    for (int i = 0; i < HD_ITERS; i++) acc[i] = make_float2(0.f, 0.f);

    constexpr int U = 4;  // positions per warp iteration, loads issued together
    for (int s0 = s_begin + warp * U; s0 < s_end; s0 += ATT_WARPS * U) {
        __half2 kv[U][HD_ITERS], vv[U][HD_ITERS];
#pragma unroll
        for (int u = 0; u < U; u++) {
            const int s = s0 + u;
            const size_t base = (size_t)s * p.pitch + (size_t)h * hd;
#pragma unroll
            for (int i = 0; i < HD_ITERS; i++) {
                int d = 2 * lane + 64 * i;
                bool ok = s < s_end && d < hd;
                kv[u][i] = ok ? *reinterpret_cast<const __half2*>(p.kc + base + d) : __half2half2(__float2half(0.f));
                vv[u][i] = ok ? *reinterpret_cast<const __half2*>(p.vc + base + d) : __half2half2(__float2half(0.f));
            }
        }
        float sc[U];
#pragma unroll
        for (int u = 0; u < U; u++) {
            float d = 0.f;
#pragma unroll
            for (int i = 0; i < HD_ITERS; i++) {
                float2 kf = __half22float2(kv[u][i]);
                d = fmaf(qf[i].x, kf.x, d);
                d = fmaf(qf[i].y, kf.y, d);
            }
            sc[u] = d;
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1)
#pragma unroll
            for (int u = 0; u < U; u++) sc[u] += __shfl_xor_sync(0xffffffffu, sc[u], o);
#pragma unroll
        for (int u = 0; u < U; u++) {
            if (s0 + u < s_end) {
                const float x = sc[u] * p.scale;
                const float mn = fmaxf(m, x);
                const float corr = __expf(m - mn), pe = __expf(x - mn);
                l = l * corr + pe;
#pragma unroll
                for (int i = 0; i < HD_ITERS; i++) {
                    float2 vf = __half22float2(vv[u][i]);
                    acc[i].x = fmaf(pe, vf.x, acc[i].x * corr);
                    acc[i].y = fmaf(pe, vf.y, acc[i].y * corr);
                }
                m = mn;
            }
        }
    }
    // merge the warps of this CTA
    if (lane == 0) { sm_m[warp] = m; sm_l[warp] = l; }
#pragma unroll
    for (int i = 0; i < HD_ITERS; i++) {
        int d = 2 * lane + 64 * i;
        if (d < hd) { sm_acc[warp][d] = acc[i].x; sm_acc[warp][d + 1] = acc[i].y; }
    }
    __syncthreads();
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < ATT_WARPS; w++) M = fmaxf(M, sm_m[w]);
    float L = 0.f;
#pragma unroll
    for (int w = 0; w < ATT_WARPS; w++) L += sm_m[w] == -INFINITY ? 0.f : sm_l[w] * __expf(sm_m[w] - M);
    float* slot = p.scratch + ((size_t)h * p.splits + split) * (hd + 2);
    for (int d = threadIdx.x; d < hd; d += ATT_THREADS) {
        float a = 0.f;
#pragma unroll
        for (int w = 0; w < ATT_WARPS; w++)
            a += sm_m[w] == -INFINITY ? 0.f : sm_acc[w][d] * __expf(sm_m[w] - M);
        slot[2 + d] = a;
    }
    if (threadIdx.x == 0) { slot[0] = M; slot[1] = L; }
    // last CTA of this head merges the splits
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
        unsigned int prev = atomicAdd(&p.counters[h], 1u);
        is_last = prev == (unsigned)p.splits - 1;
        if (is_last) p.counters[h] = 0;  // ready for the next launch
    }
    __syncthreads();
    if (!is_last) return;
    __threadfence();
    const float* base = p.scratch + (size_t)h * p.splits * (hd + 2);
    float GM = -INFINITY;
    for (int sp = 0; sp < p.splits; sp++) GM = fmaxf(GM, __ldcg(base + (size_t)sp * (hd + 2)));
    float GL = 0.f;
    for (int sp = 0; sp < p.splits; sp++) {
        float ms = __ldcg(base + (size_t)sp * (hd + 2));
        if (ms != -INFINITY) GL += __ldcg(base + (size_t)sp * (hd + 2) + 1) * __expf(ms - GM);
    }
    for (int d = threadIdx.x; d < hd; d += ATT_THREADS) {
        float a = 0.f;
        for (int sp = 0; sp < p.splits; sp++) {
            float ms = __ldcg(base + (size_t)sp * (hd + 2));
            if (ms != -INFINITY) a += __ldcg(base + (size_t)sp * (hd + 2) + 2 + d) * __expf(ms - GM);
        }
        p.out[(size_t)h * hd + d] = __float2half_rn(a / GL);
    }
}

// RMSNorm, fp32 sum, one rounding: out = half(x * rsqrt(mean(x^2) + eps) * w). One warp per token
// like the reference's rms_norm_kernel_v1 (tensorLib/src/device/cuda/rms_norm.cu:140-167).
__global__ void k_rmsnorm_fast(__half* out, const __half* in, const __half* w, float eps, int hidden, int tokens) {
    const int t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (t >= tokens) return;
    const __half* x = in + (size_t)t * hidden;
    float ss = 0.f;
    for (int j = lane; j < hidden; j += 32) { float v = __half2float(x[j]); ss = fmaf(v, v, ss); }
    ss = warp_sum(ss);
    const float rinv = rsqrtf(ss / (float)hidden + eps);
    for (int j = lane; j < hidden; j += 32)
        out[(size_t)t * hidden + j] = __float2half_rn(__half2float(x[j]) * rinv * __half2float(w[j]));
}

// The same arithmetic with one 128-thread block per token and 16-byte loads (hidden % 8 == 0,
// 16-byte aligned rows): the multi-token (prefill) form, bound by HBM at 4 bytes per element.
__global__ void __launch_bounds__(128) k_rmsnorm_fast_vec(__half* out, const __half* in, const __half* w, float eps, int hidden) {
    __shared__ float red[4];
    pdl_launch_dependents();
    pdl_wait();
    const size_t t = blockIdx.x;
    const uint4* x4 = reinterpret_cast<const uint4*>(in + t * hidden);
    const uint4* w4 = reinterpret_cast<const uint4*>(w);
    uint4* o4 = reinterpret_cast<uint4*>(out + t * hidden);
    const int n8 = hidden >> 3;
    float ss = 0.f;
    for (int j = threadIdx.x; j < n8; j += 128) {
        const uint4 v = x4[j];
        const __half2* h = reinterpret_cast<const __half2*>(&v);
#pragma unroll
        for (int i = 0; i < 4; i++) { const float2 f = __half22float2(h[i]); ss = fmaf(f.x, f.x, ss); ss = fmaf(f.y, f.y, ss); }
    }
    ss = warp_sum(ss);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
    __syncthreads();
    const float rinv = rsqrtf((red[0] + red[1] + red[2] + red[3]) / (float)hidden + eps);
    for (int j = threadIdx.x; j < n8; j += 128) {
        const uint4 v = x4[j], wv = w4[j];
        const __half2* h = reinterpret_cast<const __half2*>(&v);
        const __half2* wh = reinterpret_cast<const __half2*>(&wv);
        uint4 o;
        __half2* oh = reinterpret_cast<__half2*>(&o);
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const float2 f = __half22float2(h[i]), g = __half22float2(wh[i]);
            oh[i] = __floats2half2_rn(f.x * rinv * g.x, f.y * rinv * g.y);
        }
        o4[j] = o;
    }
}

// softmax over the last dim with fp32 internals; optional scale and causal mask (col > pos + t)
__global__ void k_softmax_fast(__half* out, const __half* in, size_t cols, int T, int pos, float scale, bool causal) {
    __shared__ float red[32];
    const size_t row = blockIdx.x;
    const __half* x = in + row * cols;
    __half* y = out + row * cols;
    const int t = causal ? (int)(row % T) : 0;
    const size_t lim = causal ? min(cols, (size_t)(pos + t + 1)) : cols;
    float mx = -INFINITY;
    for (size_t j = threadIdx.x; j < lim; j += blockDim.x) mx = fmaxf(mx, __half2float(x[j]) * scale);
    mx = warp_max(mx);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = mx;
    __syncthreads();
    if (threadIdx.x < 32) {
        float v = threadIdx.x < (blockDim.x >> 5) ? red[threadIdx.x] : -INFINITY;
        v = warp_max(v);
        if (threadIdx.x == 0) red[0] = v;
    }
    __syncthreads();
    mx = red[0];
    __syncthreads();
    float sum = 0.f;
    for (size_t j = threadIdx.x; j < lim; j += blockDim.x) sum += __expf(__half2float(x[j]) * scale - mx);
    sum = warp_sum(sum);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = sum;
    __syncthreads();
    if (threadIdx.x < 32) {
        float v = threadIdx.x < (blockDim.x >> 5) ? red[threadIdx.x] : 0.f;
        v = warp_sum(v);
        if (threadIdx.x == 0) red[0] = v;
    }
    __syncthreads();
    const float inv = 1.f / red[0];
    for (size_t j = threadIdx.x; j < cols; j += blockDim.x)
        y[j] = j < lim ? __float2half_rn(__expf(__half2float(x[j]) * scale - mx) * inv) : __float2half_rn(0.f);
}

__global__ void k_swiglu_fast(__half* out, const __half* gate, const __half* up, size_t n) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    float g = __half2float(gate[i]);
    __half s = __float2half_rn(g / (1.f + __expf(-g)));
    out[i] = __hmul(s, up[i]);
}

// vt[h][d][s] = v[s][h][d]
__global__ void k_transpose_v(__half* vt, const __half* v, int S, int H, int hd, long long v_pitch, long long vt_pitch_s) {
    __shared__ __half tile[32][34];
    const int h = blockIdx.z;
    const int s0 = blockIdx.x * 32, d0 = blockIdx.y * 32;
    for (int i = threadIdx.y; i < 32; i += blockDim.y) {
        int s = s0 + i, d = d0 + threadIdx.x;
        if (s < S && d < hd) tile[i][threadIdx.x] = v[(long long)s * v_pitch + (long long)h * hd + d];
    }
    __syncthreads();
    for (int i = threadIdx.y; i < 32; i += blockDim.y) {
        int d = d0 + i, s = s0 + threadIdx.x;
        if (s < S && d < hd) vt[((long long)h * hd + d) * vt_pitch_s + s] = tile[threadIdx.x][i];
    }
}

}  // namespace

// Same attention, splits merged through distributed shared memory: the `splits` CTAs of a head
// form one thread-block cluster; each leaves its (max, sum, acc) in its own shared memory, and
// after a cluster barrier the first CTA of the cluster reads its peers' partials over DSMEM and
// writes the head's output. No scratch buffer, no atomics, no global-memory round trips in the
// merge, which is most of the kernel's latency at decode-sized contexts.
namespace {
constexpr int CL_WARPS = 8;
constexpr int CL_THREADS = CL_WARPS * 32;

__global__ void __launch_bounds__(CL_THREADS) k_decode_attn_cluster(AttnArgs p) {
    __shared__ float sm_m[CL_WARPS], sm_l[CL_WARPS];
    __shared__ float sm_acc[CL_WARPS][MAX_HD];
    __shared__ float cta_out[MAX_HD + 2];
    cg::cluster_group cluster = cg::this_cluster();
    const int h = blockIdx.x, split = blockIdx.y;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int hd = p.hd;

    pdl_launch_dependents();
    // In the decode step (pos_ptr set) the position counter and every cache row below the current
    // position were written by kernels of EARLIER steps, long finished; only the newest row (and q)
    // come from the kernel just before this one. So the first chunk of old rows is fetched before
    // the dependency wait and its L2 latency overlaps that kernel's tail.
    const bool early = p.pos_ptr != nullptr;
    if (!early) pdl_wait();
    const int S = p.pos_ptr ? (*p.pos_ptr + 1) : p.seq_len;
    const int newest = early ? S - 1 : -1;
    const int per = (S + p.splits - 1) / p.splits;
    const int s_begin = split * per, s_end = min(S, s_begin + per);

    constexpr int U = 4;
    auto load_rows = [&](__half2 (&kv)[U][HD_ITERS], __half2 (&vv)[U][HD_ITERS], int s0, bool skip_newest) {
#pragma unroll
        for (int u = 0; u < U; u++) {
            const int s = s0 + u;
            const size_t base = (size_t)s * p.pitch + (size_t)h * hd;
#pragma unroll
            for (int i = 0; i < HD_ITERS; i++) {
                const int d = 2 * lane + 64 * i;
                const bool ok = s < s_end && d < hd && !(skip_newest && s == newest);
                kv[u][i] = ok ? *reinterpret_cast<const __half2*>(p.kc + base + d) : __half2half2(__float2half(0.f));
                vv[u][i] = ok ? *reinterpret_cast<const __half2*>(p.vc + base + d) : __half2half2(__float2half(0.f));
            }
        }
    };
    __half2 kv[U][HD_ITERS], vv[U][HD_ITERS];
    const int s_first = s_begin + warp * U;
    if (early) {
        if (s_first < s_end) load_rows(kv, vv, s_first, true);
        pdl_wait();
    }

    float2 qf[HD_ITERS];
#pragma unroll
    for (int i = 0; i < HD_ITERS; i++) {
        int d = 2 * lane + 64 * i;
        qf[i] = d < hd ? __half22float2(*reinterpret_cast<const __half2*>(p.q + (size_t)h * hd + d))
                       : make_float2(0.f, 0.f);
    }
    float m = -INFINITY, l = 0.f;
    float2 acc[HD_ITERS];
#pragma unroll
    for (int i = 0; i < HD_ITERS; i++) acc[i] = make_float2(0.f, 0.f);

    for (int s0 = s_first; s0 < s_end; s0 += CL_WARPS * U) {
        if (!early || s0 != s_first) {
            load_rows(kv, vv, s0, false);
        } else if (newest >= s0 && newest < s0 + U && newest < s_end) {
            // the one row the previous kernel wrote, if it falls into the prefetched chunk
#pragma unroll
            for (int u = 0; u < U; u++) {
                if (s0 + u == newest) {
                    const size_t base = (size_t)newest * p.pitch + (size_t)h * hd;
#pragma unroll
                    for (int i = 0; i < HD_ITERS; i++) {
                        const int d = 2 * lane + 64 * i;
                        if (d < hd) {
                            kv[u][i] = *reinterpret_cast<const __half2*>(p.kc + base + d);
                            vv[u][i] = *reinterpret_cast<const __half2*>(p.vc + base + d);
                        }
                    }
                }
            }
        }
        float sc[U];
#pragma unroll
        for (int u = 0; u < U; u++) {
            float d = 0.f;
#pragma unroll
            for (int i = 0; i < HD_ITERS; i++) {
                float2 kf = __half22float2(kv[u][i]);
                d = fmaf(qf[i].x, kf.x, d);
                d = fmaf(qf[i].y, kf.y, d);
            }
            sc[u] = d;
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1)
#pragma unroll
            for (int u = 0; u < U; u++) sc[u] += __shfl_xor_sync(0xffffffffu, sc[u], o);
#pragma unroll
        for (int u = 0; u < U; u++) {
            if (s0 + u < s_end) {
                const float x = sc[u] * p.scale;
                const float mn = fmaxf(m, x);
                const float corr = __expf(m - mn), pe = __expf(x - mn);
                l = l * corr + pe;
#pragma unroll
                for (int i = 0; i < HD_ITERS; i++) {
                    float2 vf = __half22float2(vv[u][i]);
                    acc[i].x = fmaf(pe, vf.x, acc[i].x * corr);
                    acc[i].y = fmaf(pe, vf.y, acc[i].y * corr);
                }
                m = mn;
            }
        }
    }
    if (lane == 0) { sm_m[warp] = m; sm_l[warp] = l; }
#pragma unroll
    for (int i = 0; i < HD_ITERS; i++) {
        int d = 2 * lane + 64 * i;
        if (d < hd) { sm_acc[warp][d] = acc[i].x; sm_acc[warp][d + 1] = acc[i].y; }
    }
    __syncthreads();
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < CL_WARPS; w++) M = fmaxf(M, sm_m[w]);
    float L = 0.f;
#pragma unroll
    for (int w = 0; w < CL_WARPS; w++) L += sm_m[w] == -INFINITY ? 0.f : sm_l[w] * __expf(sm_m[w] - M);
    for (int d = threadIdx.x; d < hd; d += CL_THREADS) {
        float a = 0.f;
#pragma unroll
        for (int w = 0; w < CL_WARPS; w++)
            a += sm_m[w] == -INFINITY ? 0.f : sm_acc[w][d] * __expf(sm_m[w] - M);
        cta_out[2 + d] = a;
    }
    if (threadIdx.x == 0) { cta_out[0] = M; cta_out[1] = L; }
    cluster.sync();   // every split's partial is in its CTA's shared memory
    if (cluster.block_rank() == 0) {
        const int n = (int)cluster.num_blocks();
        float GM = -INFINITY;
        for (int r = 0; r < n; r++) GM = fmaxf(GM, cluster.map_shared_rank(cta_out, r)[0]);
        float GL = 0.f;
        for (int r = 0; r < n; r++) {
            const float* rem = cluster.map_shared_rank(cta_out, r);
            if (rem[0] != -INFINITY) GL += rem[1] * __expf(rem[0] - GM);
        }
        for (int d = threadIdx.x; d < hd; d += CL_THREADS) {
            float a = 0.f;
            for (int r = 0; r < n; r++) {
                const float* rem = cluster.map_shared_rank(cta_out, r);
                if (rem[0] != -INFINITY) a += rem[2 + d] * __expf(rem[0] - GM);
            }
            p.out[(size_t)h * hd + d] = __float2half_rn(a / GL);
        }
    }
    cluster.sync();   // peers keep their shared memory alive until the reader is done
}
}  // namespace

int launch_decode_attn_cluster(const DecodeAttn& q, cudaStream_t st) {
    TL_REQUIRE(q.head_dim > 0 && q.head_dim <= MAX_HD && q.head_dim % 2 == 0, "decode attention: head_dim %d unsupported", q.head_dim);
    TL_REQUIRE(q.H > 0 && q.splits >= 1 && q.splits <= 8, "decode attention (cluster): splits must be 1..8");
    AttnArgs a{q.q, q.k_cache, q.v_cache, q.out, nullptr, nullptr, q.H, q.head_dim, q.seq_len,
               q.splits, q.pos_ptr, q.kv_pitch, 1.0f / sqrtf((float)q.head_dim)};
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(q.H, q.splits);
    cfg.blockDim = dim3(CL_THREADS);
    cfg.stream = st;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 1;
    attr[0].val.clusterDim.y = q.splits;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = q.pdl ? 2 : 1;
    TL_CUDA(cudaLaunchKernelEx(&cfg, k_decode_attn_cluster, a));
    return TL_OK;
}

int launch_decode_attn(const DecodeAttn& q, cudaStream_t st) {
    TL_REQUIRE(q.head_dim > 0 && q.head_dim <= MAX_HD && q.head_dim % 2 == 0, "decode attention: head_dim %d unsupported", q.head_dim);
    TL_REQUIRE(q.H > 0 && q.splits > 0 && q.splits <= 65535, "decode attention: bad grid");
    AttnArgs a{q.q, q.k_cache, q.v_cache, q.out, q.scratch, q.counters, q.H, q.head_dim, q.seq_len,
               q.splits, q.pos_ptr, q.kv_pitch, 1.0f / sqrtf((float)q.head_dim)};
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(q.H, q.splits);
    cfg.blockDim = dim3(ATT_THREADS);
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = q.pdl ? 1 : 0;
    TL_CUDA(cudaLaunchKernelEx(&cfg, k_decode_attn, a));
    return TL_OK;
}

}  // namespace tlb

// ---------------------------------------------------------------------------------------------
// Decode attention for callers that must not allocate.
//
// Some hosts of this library cannot call cudaMalloc at the point where they need attention: code
// running inside a CUDA-graph capture, a plugin that was handed a fixed memory budget by its
// embedding application, or a latency-critical serving loop that forbids allocator calls after
// start-up. tl_attn_decode_f16 asks such a caller for a scratch buffer and a counter array it may
// have no way to provide. This variant keeps both in a fixed array that is part of the loaded
// library image instead: every GPU that loads the library holds NOALLOC_BYTES (about 0.5 MB) of
// device memory for it until the process exits.
//
// The array's name is only a host-side handle in host code; the device address is looked up with
// cudaGetSymbolAddress once per device (on the first call made while that device is current) and
// handed to the kernel like any other pointer.
// ---------------------------------------------------------------------------------------------
namespace {
constexpr size_t NOALLOC_MAX_HEADS = 128;
constexpr size_t NOALLOC_MAX_PARTIAL_FLOATS = 128 * 1024;  // n_heads * splits * (head_dim + 2) at most
constexpr size_t NOALLOC_COUNTER_BYTES = NOALLOC_MAX_HEADS * sizeof(unsigned int);
constexpr size_t NOALLOC_BYTES = NOALLOC_COUNTER_BYTES + NOALLOC_MAX_PARTIAL_FLOATS * sizeof(float);
static __device__ __align__(256) unsigned char g_noalloc_scratch[NOALLOC_BYTES];

constexpr int NOALLOC_MAX_DEVICES = 64;
unsigned char* g_noalloc_ptr[NOALLOC_MAX_DEVICES] = {};
std::mutex g_noalloc_mu;
}  // namespace

extern "C" int tl_attn_decode_f16_noalloc(const tl_half* q, const tl_half* k_cache, const tl_half* v_cache,
                                          tl_half* out, int n_heads, int head_dim, int seq_len, int splits,
                                          tl_stream stream) {
    using namespace tlb;
    TL_CHECK_INIT();
    TL_REQUIRE(q && k_cache && v_cache && out, "null pointer");
    TL_REQUIRE(n_heads > 0 && head_dim > 0 && seq_len > 0 && splits > 0, "bad shape");
    TL_REQUIRE((size_t)n_heads <= NOALLOC_MAX_HEADS,
               "tl_attn_decode_f16_noalloc: n_heads=%d exceeds the built-in scratch (max %zu heads); "
               "use tl_attn_decode_f16 with your own scratch", n_heads, NOALLOC_MAX_HEADS);
    // bound every factor before forming the product, so that it cannot wrap below the limit
    TL_REQUIRE(head_dim <= 256 && head_dim % 2 == 0 && splits <= 65535,
               "tl_attn_decode_f16_noalloc: head_dim=%d (even, at most 256) or splits=%d (at most 65535) "
               "exceeds the built-in scratch", head_dim, splits);
    const size_t partial_floats = (size_t)n_heads * (size_t)splits * ((size_t)head_dim + 2);
    TL_REQUIRE(partial_floats <= NOALLOC_MAX_PARTIAL_FLOATS,
               "tl_attn_decode_f16_noalloc: n_heads*splits*(head_dim+2)=%zu floats exceeds the built-in scratch "
               "(max %zu); use fewer splits or tl_attn_decode_f16 with your own scratch",
               partial_floats, NOALLOC_MAX_PARTIAL_FLOATS);
    int dev = -1;
    TL_CUDA(cudaGetDevice(&dev));
    TL_REQUIRE(dev >= 0 && dev < NOALLOC_MAX_DEVICES, "device index %d out of range", dev);
    unsigned char* base;
    {
        std::lock_guard<std::mutex> lk(g_noalloc_mu);
        if (!g_noalloc_ptr[dev]) {  // first call on this device: resolve the symbol (not capturable)
            unsigned char* p = nullptr;
            TL_CUDA(cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_noalloc_scratch));
            g_noalloc_ptr[dev] = p;
        }
        base = g_noalloc_ptr[dev];
    }
    unsigned int* counters = reinterpret_cast<unsigned int*>(base);
    float* partials = reinterpret_cast<float*>(base + NOALLOC_COUNTER_BYTES);
    cudaStream_t st = as_stream(stream);
    // The array keeps whatever the previous call left behind. The per-head arrival counters must
    // start at zero; the partial-result slots are fully rewritten before they are read.
    TL_CUDA(cudaMemsetAsync(counters, 0, (size_t)n_heads * sizeof(unsigned int), st));
    DecodeAttn a{reinterpret_cast<const __half*>(q), reinterpret_cast<const __half*>(k_cache),
                 reinterpret_cast<const __half*>(v_cache), reinterpret_cast<__half*>(out), partials, counters,
                 n_heads, head_dim, seq_len, splits, nullptr, (long long)n_heads * head_dim, false};
    return launch_decode_attn(a, st);
}

namespace tlb {

int launch_rmsnorm_fast(__half* out, const __half* in, const __half* w, float eps, int hidden,
                        int tokens, cudaStream_t st) {
    if (tokens <= 0) return TL_OK;
    const bool vec = hidden % 8 == 0 && ((reinterpret_cast<uintptr_t>(out) | reinterpret_cast<uintptr_t>(in) |
                                          reinterpret_cast<uintptr_t>(w)) & 15) == 0;
    if (vec && tokens >= 16) {
        return launch_pdl(k_rmsnorm_fast_vec, dim3((unsigned)tokens), dim3(128), 0, st, true, out, in, w, eps, hidden);
    }
    k_rmsnorm_fast<<<(unsigned)ceil_div(tokens, 8), 256, 0, st>>>(out, in, w, eps, hidden, tokens);
    TL_LAUNCH_CHECK();
    return TL_OK;
}
int launch_softmax_fast(__half* out, const __half* in, size_t rows, size_t cols, cudaStream_t st) {
    if (rows == 0 || cols == 0) return TL_OK;
    k_softmax_fast<<<(unsigned)rows, 256, 0, st>>>(out, in, cols, 1, 0, 1.0f, false);
    TL_LAUNCH_CHECK();
    return TL_OK;
}
int launch_softmax_causal_fast(__half* scores, int H, int T, int S, int pos, float scale, cudaStream_t st) {
    if ((size_t)H * T == 0 || S == 0) return TL_OK;
    k_softmax_fast<<<(unsigned)((size_t)H * T), 256, 0, st>>>(scores, scores, (size_t)S, T, pos, scale, true);
    TL_LAUNCH_CHECK();
    return TL_OK;
}
int launch_swiglu_fast(__half* out, const __half* gate, const __half* up, size_t n, cudaStream_t st) {
    if (n == 0) return TL_OK;
    k_swiglu_fast<<<(unsigned)ceil_div(n, 256), 256, 0, st>>>(out, gate, up, n);
    TL_LAUNCH_CHECK();
    return TL_OK;
}
int launch_transpose_v(__half* vt, const __half* v, int S, int H, int hd, long long v_pitch,
                       long long vt_pitch_s, cudaStream_t st) {
    if (S <= 0) return TL_OK;
    dim3 grid((unsigned)ceil_div(S, 32), (unsigned)ceil_div(hd, 32), H), block(32, 8);
    k_transpose_v<<<grid, block, 0, st>>>(vt, v, S, H, hd, v_pitch, vt_pitch_s);
    TL_LAUNCH_CHECK();
    return TL_OK;
}

}  // namespace tlb
