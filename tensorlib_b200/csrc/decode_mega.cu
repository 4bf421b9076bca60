// One decode step of the Llama2 forward as ONE persistent kernel (fast numerics, batch 1), with
// DATAFLOW synchronisation between its phases.
//
// Replaces, per token, the reference's ~2.8 k launches (model/llama2_7b/src/Transformer.cpp:264-299
// and everything it calls) and this library's own graph of ~130 kernels. One CTA per SM stays
// resident for the whole token and walks the phases
//     per layer:  [RMSNorm + wq|wk|wv GEMV + RoPE + KV write] | [attention] | [wo GEMV + residual] |
//                 [RMSNorm + w1|w3 GEMV + SiLU*up] | [w2 GEMV + residual]
//     then        [RMSNorm + classifier GEMV + greedy sampling]
// Two things keep HBM busy across phase boundaries:
//   * the weight stream: the producer warp of every CTA pushes the weight rows of ALL phases, in
//     order, through the shared-memory ring with TMA bulk copies and never waits for a phase to end
//     (weights do not depend on activations); it only waits for ring slots. The ring holds 190 KB
//     per SM (28 MB per GPU, ~4 us of HBM time);
//   * no barriers: the activation vector a phase produces travels through L2 as 32-bit words that
//     carry their fp16 value AND the low 16 bits of the producing phase's epoch (a counter that
//     advances with every phase of every step), written with one store per word (or pair). A
//     consumer polls the words it needs until their epoch is the one it expects, so a hand-over costs
//     one L2 round trip after the LAST producer finished instead of a grid-wide barrier or a kernel
//     boundary (measured ~5 us each), and words never need resetting: the value a word held before
//     is one step (5 L + 1 epochs) older, which no 16-bit comparison confuses with the current one.
// Under tensor parallelism the partial sums of wo and w2 are pushed into every rank's memory as
// (fp32, epoch) words like in the multi-kernel step; each CTA adds the ranks' partials for its own
// slice of the vector, adds the residual, and publishes the slice as ordinary words, so the sum is
// formed once per GPU and the consumers are the same code as on one GPU.
//
// Consumers: 16 warps. In a GEMV phase warp w multiplies the k16 steps [4w, 4w+4) of every 1024-wide
// chunk for the 32 rows of a stage on the tensor cores (mma.sync, the activation vector in column
// 0 of B); in the attention phase they form 4 groups of 4 warps, each working on one (head, split)
// item. Every wait (mbarrier, word poll, peer slot poll) is bounded and reports TL_ERR_TIMEOUT
// through the device status word instead of hanging. The CTAs wait on one another, so the launch
// is cooperative (all CTAs co-resident).
#include <cuda.h>

#include <vector>

#include "decode_mega.cuh"
#include "engine.cuh"

namespace tlb {

namespace {

// ---- small device helpers -----------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}\n"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
constexpr uint32_t WAIT_LIMIT = 1u << 22;
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
    for (uint32_t i = 0; i < WAIT_LIMIT; i++)
        if (mbar_try_wait(bar, parity)) return true;
    return false;
}
__device__ __forceinline__ void tma_load_1d(uint32_t dst_smem, const void* src, uint32_t bytes, uint32_t bar,
                                            uint64_t policy) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;"
        ::"r"(dst_smem), "l"(src), "r"(bytes), "r"(bar), "l"(policy)
        : "memory");
}
__device__ __forceinline__ uint64_t policy_evict_first() {
    uint64_t p;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
    return p;
}
__device__ __forceinline__ void named_bar_sync(int id, int threads) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}
__device__ __forceinline__ unsigned int ld_acquire_u32(const unsigned int* p) {
    unsigned int v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ __half ldcg_half(const __half* p) {
    unsigned short v = __ldcg(reinterpret_cast<const unsigned short*>(p));
    return __ushort_as_half(v);
}
__device__ __forceinline__ float dot8(const uint4& w, const uint4& x, float acc) {
    const __half2* wh = reinterpret_cast<const __half2*>(&w);
    const __half2* xh = reinterpret_cast<const __half2*>(&x);
#pragma unroll
    for (int i = 0; i < 4; i++) {
        float2 wf = __half22float2(wh[i]);
        float2 xf = __half22float2(xh[i]);
        acc = fmaf(wf.x, xf.x, acc);
        acc = fmaf(wf.y, xf.y, acc);
    }
    return acc;
}
__device__ __forceinline__ float sumsq8(const uint4& v) {
    const __half2* h = reinterpret_cast<const __half2*>(&v);
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < 4; i++) {
        float2 f = __half22float2(h[i]);
        s = fmaf(f.x, f.x, s);
        s = fmaf(f.y, f.y, s);
    }
    return s;
}

// ---- geometry -------------------------------------------------------------------------------------
constexpr int CONSUMERS = 16;
constexpr int CONSUMER_THREADS = CONSUMERS * 32;
constexpr int MEGA_THREADS = CONSUMER_THREADS + 32;   // + one producer warp
constexpr int KC = 1024;                              // halfs per row-chunk
constexpr int CHUNK_BYTES = KC * 2;
constexpr int ROW_STRIDE = CHUNK_BYTES + 16;          // +16 B: conflict-free ldmatrix row addresses
constexpr int STAGE_ROWS = CONSUMERS * 2;
constexpr int STAGE_BYTES = STAGE_ROWS * ROW_STRIDE;  // 66,048 B
constexpr int NSTAGES = 3;
constexpr int STEPS_PER_WARP = KC / 16 / CONSUMERS;   // k16 steps of a chunk each warp multiplies

__device__ __forceinline__ void ldmatrix_x4(uint32_t saddr, uint32_t& a0, uint32_t& a1, uint32_t& a2, uint32_t& a3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(a0), "=r"(a1), "=r"(a2), "=r"(a3)
                 : "r"(saddr));
}
__device__ __forceinline__ void mma_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                          uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
constexpr int ATT_GROUPS = 4, ATT_WARPS = 4;          // 4 groups x 4 warps
constexpr int MAX_HD = 256, HD_ITERS = MAX_HD / 64;
constexpr int ATT_SMEM_PER_GROUP = (2 * ATT_WARPS + ATT_WARPS * MAX_HD + 4) * 4;

}  // namespace

namespace {

__device__ __forceinline__ unsigned long long globaltimer_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

// ---- words: (fp16 value, 16-bit epoch) in 32 bits -----------------------------------------------------
constexpr uint32_t POLL_LIMIT = 1u << 22;     // L2 polls (~0.5 us each) before a consumer gives up
__device__ __forceinline__ uint32_t make_word(__half v, uint32_t e16) { return (uint32_t)__half_as_ushort(v) | (e16 << 16); }
__device__ __forceinline__ void st_word1(uint32_t* p, uint32_t w) {
    asm volatile("st.volatile.global.u32 [%0], %1;" ::"l"(p), "r"(w) : "memory");
}
__device__ __forceinline__ void st_word_pair(uint32_t* p, uint32_t w0, uint32_t w1) {
    asm volatile("st.volatile.global.v2.u32 [%0], {%1, %2};" ::"l"(p), "r"(w0), "r"(w1) : "memory");
}
__device__ __forceinline__ uint4 ld_word4(const uint32_t* p) {
    uint4 v;
    asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ uint2 ld_word2(const uint32_t* p) {
    uint2 v;
    asm volatile("ld.volatile.global.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ bool epochs_ok(const uint4& w, uint32_t e16) {
    return ((w.x >> 16) == e16) & ((w.y >> 16) == e16) & ((w.z >> 16) == e16) & ((w.w >> 16) == e16);
}
// eight consecutive values of a word vector as eight packed halfs, waiting (bounded) for their epoch
__device__ __forceinline__ uint4 gather8(const uint32_t* words, uint32_t e16, int* status) {
    uint4 a, b;
    bool here = false;
    for (uint32_t i = 0; i < POLL_LIMIT && !here; i++) {
        a = ld_word4(words);
        b = ld_word4(words + 4);
        here = epochs_ok(a, e16) & epochs_ok(b, e16);
    }
    if (!here) atomicExch(status, TL_ERR_TIMEOUT);
    return make_uint4((a.x & 0xffffu) | (a.y << 16), (a.z & 0xffffu) | (a.w << 16), (b.x & 0xffffu) | (b.y << 16),
                      (b.z & 0xffffu) | (b.w << 16));
}
// two consecutive values as one packed half2
__device__ __forceinline__ uint32_t gather2(const uint32_t* words, uint32_t e16, int* status) {
    uint2 w;
    bool here = false;
    for (uint32_t i = 0; i < POLL_LIMIT && !here; i++) {
        w = ld_word2(words);
        here = ((w.x >> 16) == e16) & ((w.y >> 16) == e16);
    }
    if (!here) atomicExch(status, TL_ERR_TIMEOUT);
    return (w.x & 0xffffu) | (w.y << 16);
}
// (payload, epoch) 8-byte words of the cross-GPU exchange (see PeerExchange in kernels.cuh)
__device__ __forceinline__ uint4 ld_xwords2(const unsigned long long* p) {
    uint4 v;
    asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_xwords2(unsigned long long* p, unsigned int d0, unsigned int d1, unsigned int epoch) {
    asm volatile("st.volatile.global.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(p), "r"(d0), "r"(epoch), "r"(d1), "r"(epoch) : "memory");
}
__device__ __forceinline__ void st_xword(unsigned long long* p, unsigned int d, unsigned int epoch) {
    asm volatile("st.volatile.global.v2.u32 [%0], {%1, %2};" ::"l"(p), "r"(d), "r"(epoch) : "memory");
}

// ---- phases -----------------------------------------------------------------------------------------------
enum { PH_QKV = 0, PH_ATTN = 1, PH_WO = 2, PH_GATEUP = 3, PH_W2 = 4, PH_CLS = 5 };

struct GemvDesc {
    const __half *W0, *W1, *W2;
    int N_each, K, total_units;
    bool swiglu;
};
// the weight side of phase `kind` of layer l: what the producer streams and the consumers multiply
__device__ __forceinline__ GemvDesc gemv_desc(const FlowArgs& a, int kind, int l) {
    GemvDesc d{};
    if (kind == PH_CLS) { d.W0 = a.wcls; d.N_each = a.vocab_local; d.K = a.dim; d.total_units = a.vocab_local / 2; return d; }
    const FlowLayer& w = a.layers[l];
    if (kind == PH_QKV) { d.W0 = w.wq; d.W1 = w.wk; d.W2 = w.wv; d.N_each = a.dl; d.K = a.dim; d.total_units = 3 * a.dl / 2; }
    else if (kind == PH_WO) { d.W0 = w.wo; d.N_each = a.dim; d.K = a.dl; d.total_units = a.dim / 2; }
    else if (kind == PH_GATEUP) { d.W0 = w.w1; d.W1 = w.w3; d.N_each = a.hl; d.K = a.dim; d.total_units = a.hl; d.swiglu = true; }
    else { d.W0 = w.w2; d.N_each = a.dim; d.K = a.hl; d.total_units = a.dim / 2; }
    return d;
}
// unit u of a phase = the two weight rows one lane pair finishes: rows (2u, 2u+1) of one of up to three
// matrices, or row u of w1 and of w3
__device__ __forceinline__ void unit_rows(const GemvDesc& p, int unit, const __half*& ra, const __half*& rb, int& mat, int& r) {
    if (p.swiglu) {
        mat = 0; r = unit;
        ra = p.W0 + (long long)unit * p.K;
        rb = p.W1 + (long long)unit * p.K;
    } else {
        const int row = unit * 2;
        mat = row / p.N_each;
        r = row - mat * p.N_each;
        const __half* Wm = mat == 0 ? p.W0 : (mat == 1 ? p.W1 : p.W2);
        ra = Wm + (long long)r * p.K;
        rb = ra + p.K;
    }
}

struct Ctx {
    unsigned char* stages; uint4* xs; float* red; float* partials; uint32_t full0, empty0;
    int warp, lane, ctid, tile_parity;
    int tok, pos;
    unsigned int epoch0;   // step * phases: epoch of phase p of this step is epoch0 + p + 1
    float rinv;            // 1/rms of the current phase's input (1 when the phase has no RMSNorm)
    int it;                // ring iteration counter of this role
    bool ok;
    float best_v; int best_i;   // classifier: this lane's best logit so far
};
__device__ __forceinline__ uint32_t e16_of(const Ctx& c, int phase) { return (c.epoch0 + (unsigned)phase + 1u) & 0xffffu; }
__device__ __forceinline__ uint32_t e32_of(const Ctx& c, int phase) { return c.epoch0 + (unsigned)phase + 1u; }

// ---- staging the activation vector of a GEMV phase ------------------------------------------------------------
// RMSNorm in one pass: the vector staged is x * w (fp16); the scalar 1/rms is applied to the finished
// dot products instead (sum_k rinv*x_k*w_k*W_nk = rinv * sum_k (x_k*w_k)*W_nk), so no second pass over
// x has to wait for the reduction.
template <typename Load>
__device__ __forceinline__ void stage_vector(const FlowArgs& a, Ctx& c, int K, const __half* norm_w, Load load8) {
    const int K8 = K >> 3;
    if (norm_w) {
        float ss = 0.f;
        const uint4* nw4 = reinterpret_cast<const uint4*>(norm_w);
        for (int i = c.ctid; i < K8; i += CONSUMER_THREADS) {
            uint4 v = load8(i), g = nw4[i];
            ss += sumsq8(v);
            __half2* vh = reinterpret_cast<__half2*>(&v);
            const __half2* gh = reinterpret_cast<const __half2*>(&g);
#pragma unroll
            for (int j = 0; j < 4; j++) {
                float2 vf = __half22float2(vh[j]), gf = __half22float2(gh[j]);
                vh[j] = __floats2half2_rn(vf.x * gf.x, vf.y * gf.y);
            }
            c.xs[i] = v;
        }
        ss = warp_sum(ss);
        if (c.lane == 0) c.red[c.warp] = ss;
        named_bar_sync(1, CONSUMER_THREADS);
        float tot = 0.f;
#pragma unroll
        for (int w = 0; w < CONSUMERS; w++) tot += c.red[w];
        c.rinv = rsqrtf(tot / (float)K + a.eps);
    } else {
        for (int i = c.ctid; i < K8; i += CONSUMER_THREADS) c.xs[i] = load8(i);
        c.rinv = 1.0f;
        named_bar_sync(1, CONSUMER_THREADS);
    }
}

// Tensor parallelism: this CTA's slice of (residual + sum over ranks of the pushed partial sums),
// published as words with the epoch of the phase that produced the partials. buf 0: wo, 1: w2.
__device__ __forceinline__ void reduce_slice_and_publish(const FlowArgs& a, Ctx& c, int buf, int src_phase,
                                                         const uint32_t* residual_words, uint32_t* out_words) {
    const int K8 = a.dim >> 3;
    const int g_begin = (int)((long long)K8 * blockIdx.x / gridDim.x), g_end = (int)((long long)K8 * (blockIdx.x + 1) / gridDim.x);
    const unsigned int epoch = e32_of(c, src_phase);
    const uint32_t e16 = e16_of(c, src_phase);
    for (int g = g_begin + c.ctid; g < g_end; g += CONSUMER_THREADS) {
        // the residual of these eight elements: the embedding row in layer 0, else words this CTA verified when it staged them
        __half res[8];
        if (residual_words) {
            const uint4 r0 = ld_word4(residual_words + 8 * g), r1 = ld_word4(residual_words + 8 * g + 4);
            res[0] = __ushort_as_half(r0.x & 0xffff); res[1] = __ushort_as_half(r0.y & 0xffff);
            res[2] = __ushort_as_half(r0.z & 0xffff); res[3] = __ushort_as_half(r0.w & 0xffff);
            res[4] = __ushort_as_half(r1.x & 0xffff); res[5] = __ushort_as_half(r1.y & 0xffff);
            res[6] = __ushort_as_half(r1.z & 0xffff); res[7] = __ushort_as_half(r1.w & 0xffff);
        } else {
            const uint4 r = __ldg(reinterpret_cast<const uint4*>(a.emb + (long long)c.tok * a.dim) + g);
            *reinterpret_cast<uint4*>(res) = r;
        }
        float s[8];
        bool all_here = false;
        for (uint32_t tries = 0; tries < a.exchange_tries && !all_here; tries++) {
            all_here = true;
#pragma unroll
            for (int i = 0; i < 8; i++) s[i] = 0.f;
            for (int r = 0; r < a.world; r++) {   // rank order: every rank adds the same values in the same order
                const unsigned long long* src = a.local_part[buf] + (size_t)r * a.dim + 8 * g;
#pragma unroll
                for (int q = 0; q < 4; q++) {
                    const uint4 w = ld_xwords2(src + 2 * q);
                    s[2 * q] += __uint_as_float(w.x);
                    s[2 * q + 1] += __uint_as_float(w.z);
                    all_here &= (w.y == epoch) & (w.w == epoch);
                }
            }
        }
        if (!all_here) atomicExch(a.status, TL_ERR_TIMEOUT);
        uint32_t w[8];
#pragma unroll
        for (int i = 0; i < 8; i++) w[i] = make_word(hadd_ref(res[i], __float2half_rn(s[i])), e16);
        asm volatile("st.volatile.global.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(out_words + 8 * g), "r"(w[0]), "r"(w[1]), "r"(w[2]), "r"(w[3]) : "memory");
        asm volatile("st.volatile.global.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(out_words + 8 * g + 4), "r"(w[4]), "r"(w[5]), "r"(w[6]), "r"(w[7]) : "memory");
    }
}

// ---- one GEMV phase: multiply the stages as they arrive, hand each finished row pair to `epi` ---------------------
// epi(mat, r, sa, sb, unit): called by the even lanes of warp 0 for their unit: rows (r, r+1) of matrix `mat`
// (or row r of w1 and w3 for SiLU*up), sa / sb the two fp32 dot products already scaled by 1/rms.
template <typename Epi>
__device__ __forceinline__ void gemv_consume(const FlowArgs& a, const GemvDesc& p, Ctx& c, Epi epi) {
    const int u_begin = (int)((long long)p.total_units * blockIdx.x / gridDim.x);
    const int u_end = (int)((long long)p.total_units * (blockIdx.x + 1) / gridDim.x);
    const int n_units = u_end - u_begin;
    const int n_tiles = (n_units + CONSUMERS - 1) / CONSUMERS;
    const int nk = (p.K + KC - 1) / KC;
    const int lane = c.lane, g = lane >> 2, t = lane & 3;
    const uint32_t lm_off = (uint32_t)(((lane & 7) + ((lane >> 3) & 1) * 8) * ROW_STRIDE + (lane >> 4) * 16);
    const __half* xh = reinterpret_cast<const __half*>(c.xs);
    for (int tile = 0; tile < n_tiles && c.ok; tile++) {
        const int units_here = min(CONSUMERS, n_units - tile * CONSUMERS);
        float acc0[4] = {0.f, 0.f, 0.f, 0.f}, acc1[4] = {0.f, 0.f, 0.f, 0.f};
        for (int chunk = 0; chunk < nk; chunk++, c.it++) {
            const int s = c.it % NSTAGES, use = c.it / NSTAGES;
            c.ok = mbar_wait(c.full0 + 8 * s, use & 1);
            c.ok = __all_sync(0xffffffffu, c.ok);
            if (!c.ok) break;
            const int steps = min(KC, p.K - chunk * KC) >> 4;
            const uint32_t sbase = smem_u32(c.stages + (size_t)s * STAGE_BYTES) + lm_off;
#pragma unroll
            for (int kk = 0; kk < STEPS_PER_WARP; kk++) {
                const int step = c.warp * STEPS_PER_WARP + kk;
                if (step < steps) {
                    uint32_t a0, a1, a2, a3, e0, e1, e2, e3;
                    ldmatrix_x4(sbase + step * 32, a0, a1, a2, a3);
                    ldmatrix_x4(sbase + 16 * ROW_STRIDE + step * 32, e0, e1, e2, e3);
                    const __half* xk = xh + chunk * KC + step * 16 + 2 * t;
                    const uint32_t b0 = *reinterpret_cast<const uint32_t*>(xk);
                    const uint32_t b1 = *reinterpret_cast<const uint32_t*>(xk + 8);
                    mma_16816(acc0, a0, a1, a2, a3, b0, b1);
                    mma_16816(acc1, e0, e1, e2, e3, b0, b1);
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(c.empty0 + 8 * s);
        }
        if (!c.ok) break;
        float* part = c.partials + (c.tile_parity & 1) * (CONSUMERS * STAGE_ROWS);
        c.tile_parity ^= 1;
        if (t == 0) {
            part[c.warp * STAGE_ROWS + g] = acc0[0];
            part[c.warp * STAGE_ROWS + g + 8] = acc0[2];
            part[c.warp * STAGE_ROWS + 16 + g] = acc1[0];
            part[c.warp * STAGE_ROWS + 24 + g] = acc1[2];
        }
        named_bar_sync(1, CONSUMER_THREADS);
        if (c.warp != 0) continue;
        float rowsum = 0.f;   // lane = row slot of the stage: slots 2u, 2u+1 are the rows of unit u
#pragma unroll
        for (int w = 0; w < CONSUMERS; w++) rowsum += part[w * STAGE_ROWS + lane];
        const float other = __shfl_xor_sync(0xffffffffu, rowsum, 1);
        if ((lane & 1) || (lane >> 1) >= units_here) continue;
        const __half *ra, *rb; int mat, r;
        unit_rows(p, u_begin + tile * CONSUMERS + (lane >> 1), ra, rb, mat, r);
        epi(mat, r, rowsum * c.rinv, other * c.rinv);
    }
}

// Attention of the new token over positions [0, pos] of the caches, read in place; the newest row
// (position pos) and the query come from this step's words. A work item is (head, split) and is taken
// by a whole CTA: 16 warps x ATT_U positions each = 128 positions per pass, all loads of a pass in
// flight together, so an item of up to 128 positions costs one memory latency. The number of splits
// follows the context (ceil(S / 128), at most ATT_MAX_SPLITS): with one split the warps' partial
// (max, sum, acc) meet in shared memory and the head's output words are published at once; with
// several, partials go to a scratch slot and the last CTA to finish a head merges them.
constexpr int ATT_U = 8;                        // positions per warp and pass
constexpr int ATT_MAX_SPLITS = 16;
__device__ __forceinline__ int attn_splits_for(int S) { return min(ATT_MAX_SPLITS, max(1, (S + 16 * ATT_U - 1) / (16 * ATT_U))); }

// L2 prefetch of the cache rows this CTA will read in the attention phase of layer l (they do not depend
// on this step, so the request can go out a whole phase early)
__device__ __forceinline__ void attn_prefetch(const FlowArgs& a, const Ctx& c, int l) {
    const FlowLayer& lw = a.layers[l];
    const int hd = a.hd, S = c.pos + 1, splits = attn_splits_for(S), per = (S + splits - 1) / splits;
    const int lines = (hd * 2 + 127) / 128;     // 128-byte lines per row
    for (int item = blockIdx.x; item < a.H * splits; item += gridDim.x) {
        const int h = item / splits, split = item - h * splits;
        const int s_begin = split * per, s_end = min(c.pos, s_begin + per);      // rows below pos only
        for (int i = c.ctid; i < (s_end - s_begin) * lines * 2; i += CONSUMER_THREADS) {
            const int row = i / (2 * lines), rem = i - row * 2 * lines;
            const __half* base = (rem < lines ? lw.cache_k : lw.cache_v) + (size_t)(s_begin + row) * a.dl + (size_t)h * hd;
            asm volatile("prefetch.global.L2 [%0];" ::"l"(reinterpret_cast<const char*>(base) + (rem % lines) * 128));
        }
    }
}

template <int HDI>      // head_dim <= 64 * HDI
__device__ __forceinline__ void attn_phase(const FlowArgs& a, Ctx& c, int l, int phase) {
    constexpr int U = HDI <= 2 ? ATT_U : ATT_U / 2;         // fewer rows in flight for wide heads: registers
    const FlowLayer& lw = a.layers[l];
    const int lane = c.lane, warp = c.warp;
    float* sm_m = reinterpret_cast<float*>(c.xs);          // [16]
    float* sm_l = sm_m + CONSUMERS;                          // [16]
    float* sm_acc = sm_l + CONSUMERS;                        // [16][MAX_HD]
    int* is_last = reinterpret_cast<int*>(sm_acc + CONSUMERS * MAX_HD);
    const int hd = a.hd, S = c.pos + 1;
    const int splits = attn_splits_for(S), per = (S + splits - 1) / splits;
    const float scale = rsqrtf((float)hd);
    const uint32_t e_qkv = e16_of(c, phase - 1), e_out = e16_of(c, phase);
    for (int item = blockIdx.x; item < a.H * splits; item += gridDim.x) {
        const int h = item / splits, split = item - h * splits;
        const int s_begin = split * per, s_end = min(S, s_begin + per);
        float m = -INFINITY, l_sum = 0.f;
        float2 acc[HDI], qf[HDI];
#pragma unroll
        for (int i = 0; i < HDI; i++) {
            acc[i] = make_float2(0.f, 0.f);
            const int d = 2 * lane + 64 * i;
            if (d < hd) {
                uint32_t raw = gather2(a.w.q + (size_t)h * hd + d, e_qkv, a.status);
                qf[i] = __half22float2(*reinterpret_cast<__half2*>(&raw));
            } else qf[i] = make_float2(0.f, 0.f);
        }
        for (int s0 = s_begin + warp * U; s0 < s_end; s0 += CONSUMERS * U) {
            unsigned int kv[U][HDI], vv[U][HDI];
#pragma unroll
            for (int u = 0; u < U; u++) {
                const int s = s0 + u;
                const size_t base = (size_t)s * a.dl + (size_t)h * hd;
#pragma unroll
                for (int i = 0; i < HDI; i++) {
                    const int d = 2 * lane + 64 * i;
                    const bool okk = s < s_end && d < hd;
                    if (okk && s == c.pos) {      // this step's row: still on its way through L2
                        kv[u][i] = gather2(a.w.k + (size_t)h * hd + d, e_qkv, a.status);
                        vv[u][i] = gather2(a.w.v + (size_t)h * hd + d, e_qkv, a.status);
                    } else {
                        kv[u][i] = okk ? __ldcg(reinterpret_cast<const unsigned int*>(lw.cache_k + base + d)) : 0u;
                        vv[u][i] = okk ? __ldcg(reinterpret_cast<const unsigned int*>(lw.cache_v + base + d)) : 0u;
                    }
                }
            }
            float sc[U];
#pragma unroll
            for (int u = 0; u < U; u++) {
                float d = 0.f;
#pragma unroll
                for (int i = 0; i < HDI; i++) {
                    float2 kf = __half22float2(*reinterpret_cast<__half2*>(&kv[u][i]));
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
                    const float x = sc[u] * scale;
                    const float mn = fmaxf(m, x);
                    const float corr = __expf(m - mn), pe = __expf(x - mn);
                    l_sum = l_sum * corr + pe;
#pragma unroll
                    for (int i = 0; i < HDI; i++) {
                        float2 vf = __half22float2(*reinterpret_cast<__half2*>(&vv[u][i]));
                        acc[i].x = fmaf(pe, vf.x, acc[i].x * corr);
                        acc[i].y = fmaf(pe, vf.y, acc[i].y * corr);
                    }
                    m = mn;
                }
            }
        }
        if (lane == 0) { sm_m[warp] = m; sm_l[warp] = l_sum; }
#pragma unroll
        for (int i = 0; i < HDI; i++) {
            const int d = 2 * lane + 64 * i;
            if (d < hd) { sm_acc[warp * MAX_HD + d] = acc[i].x; sm_acc[warp * MAX_HD + d + 1] = acc[i].y; }
        }
        named_bar_sync(1, CONSUMER_THREADS);
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < CONSUMERS; w++) M = fmaxf(M, sm_m[w]);
        float Lsum = 0.f;
#pragma unroll
        for (int w = 0; w < CONSUMERS; w++) Lsum += sm_m[w] == -INFINITY ? 0.f : sm_l[w] * __expf(sm_m[w] - M);
        float v = 0.f;
        if (c.ctid < hd) {
#pragma unroll
            for (int w = 0; w < CONSUMERS; w++)
                v += sm_m[w] == -INFINITY ? 0.f : sm_acc[w * MAX_HD + c.ctid] * __expf(sm_m[w] - M);
        }
        if (splits == 1) {
            if (c.ctid < hd) st_word1(a.w.att + (size_t)h * hd + c.ctid, make_word(__float2half_rn(v / Lsum), e_out));
        } else {
            float* slot = a.attn_scratch + ((size_t)h * ATT_MAX_SPLITS + split) * (hd + 2);
            if (c.ctid < hd) slot[2 + c.ctid] = v;
            if (c.ctid == 0) { slot[0] = M; slot[1] = Lsum; }
            __threadfence();
            named_bar_sync(1, CONSUMER_THREADS);
            if (c.ctid == 0) {
                const unsigned int prev = atomicAdd(&a.attn_counters[h], 1u);
                *is_last = prev == (unsigned)splits - 1;
                if (*is_last) a.attn_counters[h] = 0;
            }
            named_bar_sync(1, CONSUMER_THREADS);
            if (*is_last && c.ctid < hd) {
                __threadfence();
                const float* base = a.attn_scratch + (size_t)h * ATT_MAX_SPLITS * (hd + 2);
                float GM = -INFINITY;
                for (int sp = 0; sp < splits; sp++) GM = fmaxf(GM, __ldcg(base + (size_t)sp * (hd + 2)));
                float GL = 0.f, out = 0.f;
                for (int sp = 0; sp < splits; sp++) {
                    const float ms = __ldcg(base + (size_t)sp * (hd + 2));
                    if (ms != -INFINITY) {
                        const float w = __expf(ms - GM);
                        GL += __ldcg(base + (size_t)sp * (hd + 2) + 1) * w;
                        out += __ldcg(base + (size_t)sp * (hd + 2) + 2 + c.ctid) * w;
                    }
                }
                st_word1(a.w.att + (size_t)h * hd + c.ctid, make_word(__float2half_rn(out / GL), e_out));
            }
        }
        named_bar_sync(1, CONSUMER_THREADS);  // the shared scratch is reused by the CTA's next item
    }
}

__global__ void __launch_bounds__(MEGA_THREADS, 1) k_decode_flow(FlowArgs a) {
    extern __shared__ __align__(128) unsigned char smem[];
    Ctx c;
    c.stages = smem;
    c.xs = reinterpret_cast<uint4*>(smem + NSTAGES * STAGE_BYTES);
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + NSTAGES * STAGE_BYTES + a.x_bytes);
    c.red = reinterpret_cast<float*>(bars + 2 * NSTAGES);
    c.partials = c.red + CONSUMERS;   // [2][CONSUMERS][STAGE_ROWS]
    c.tile_parity = 0;
    c.full0 = smem_u32(bars);
    c.empty0 = smem_u32(bars + NSTAGES);
    c.warp = threadIdx.x >> 5; c.lane = threadIdx.x & 31; c.ctid = threadIdx.x;
    c.it = 0; c.ok = true;
    c.best_v = -INFINITY; c.best_i = 0x7fffffff;
    const int L = a.n_layers, n_phases = 5 * L + 1;

    if (threadIdx.x == 0) {
        for (int s = 0; s < NSTAGES; s++) {
            mbar_init(c.full0 + 8 * s, 1);
            mbar_init(c.empty0 + 8 * s, CONSUMERS);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();

    if (c.warp == CONSUMERS) {
        // ---------------- producer: every phase's weights, in order ------------------------------
        const uint64_t pol = policy_evict_first();
        const int lane = c.lane;
        bool ok = true;
        int it = 0;
        for (int ph = 0; ph < n_phases && ok; ph++) {
            const int kind = ph == 5 * L ? PH_CLS : ph % 5;
            if (kind == PH_ATTN) continue;
            const GemvDesc p = gemv_desc(a, kind, ph / 5);
            const int u_begin = (int)((long long)p.total_units * blockIdx.x / gridDim.x);
            const int u_end = (int)((long long)p.total_units * (blockIdx.x + 1) / gridDim.x);
            const int n_units = u_end - u_begin;
            const int n_tiles = (n_units + CONSUMERS - 1) / CONSUMERS;
            const int nk = (p.K + KC - 1) / KC;
            for (int tile = 0; tile < n_tiles && ok; tile++) {
                const int rows_in_tile = min(CONSUMERS, n_units - tile * CONSUMERS) * 2;
                const __half* row_ptr = nullptr;
                if (lane < rows_in_tile) {
                    const __half *ra, *rb; int mat, r;
                    unit_rows(p, u_begin + tile * CONSUMERS + (lane >> 1), ra, rb, mat, r);
                    row_ptr = (lane & 1) ? rb : ra;
                }
                for (int chunk = 0; chunk < nk; chunk++, it++) {
                    const int s = it % NSTAGES, use = it / NSTAGES;
                    if (use > 0) ok = mbar_wait(c.empty0 + 8 * s, (use - 1) & 1);
                    ok = __all_sync(0xffffffffu, ok);
                    if (!ok) break;
                    const int kc = min(KC, p.K - chunk * KC);
                    if (lane == 0) mbar_arrive_expect_tx(c.full0 + 8 * s, (uint32_t)(rows_in_tile * kc * 2));
                    __syncwarp();
                    if (lane < rows_in_tile)
                        tma_load_1d(smem_u32(c.stages + (size_t)s * STAGE_BYTES + (size_t)lane * ROW_STRIDE),
                                    row_ptr + (size_t)chunk * KC, (uint32_t)(kc * 2), c.full0 + 8 * s, pol);
                }
            }
        }
        if (!ok && lane == 0) atomicExch(a.status, TL_ERR_TIMEOUT);
        return;
    }

    // ---------------- consumers ----------------------------------------------------------------------
    c.tok = __ldcg(a.d_next);
    c.pos = __ldcg(a.d_pos);
    c.epoch0 = __ldcg(a.step) * (unsigned)n_phases;
    if (c.tok < 0 || c.tok >= a.vocab) c.tok = 0;
    const bool tp = a.world > 1;
    const __half* emb_row = a.emb + (long long)c.tok * a.dim;
    const int half_dim = a.hd >> 1;
    // optional per-phase timestamps (ns) of one CTA: [phase][0] phase start, [1] activation vector staged,
    // [2] phase work done
    const bool prof = a.prof != nullptr && blockIdx.x == a.prof_cta && c.ctid == 0;
    for (int l = 0; l < L; l++) {
        const FlowLayer& lw = a.layers[l];
        const int p0 = 5 * l;
        // ---- [RMSNorm + wq|wk|wv + RoPE + KV write] ------------------------------------------------------
        if (prof) a.prof[3 * p0] = globaltimer_ns();
        attn_prefetch(a, c, l);
        if (l == 0) {
            stage_vector(a, c, a.dim, lw.attn_norm, [&](int i) { return __ldg(reinterpret_cast<const uint4*>(emb_row) + i); });
        } else {
            if (tp) reduce_slice_and_publish(a, c, 1, p0 - 1, a.w.h, a.w.x);     // x = h + sum of the w2 partials
            const uint32_t e = e16_of(c, p0 - 1);
            stage_vector(a, c, a.dim, lw.attn_norm, [&](int i) { return gather8(a.w.x + 8 * i, e, a.status); });
        }
        if (prof) a.prof[3 * p0 + 1] = globaltimer_ns();
        {
            const uint32_t e = e16_of(c, p0);
            const __half* cs_row = a.cos_t + (long long)c.pos * half_dim;
            const __half* sn_row = a.sin_t + (long long)c.pos * half_dim;
            __half* krow = lw.cache_k + (long long)c.pos * a.dl;
            __half* vrow = lw.cache_v + (long long)c.pos * a.dl;
            gemv_consume(a, gemv_desc(a, PH_QKV, l), c, [&](int mat, int r, float sa, float sb) {
                const __half ha = __float2half_rn(sa), hb = __float2half_rn(sb);
                if (mat == 2) {                       // v: the cache row for later steps, words for this one
                    *reinterpret_cast<__half2*>(vrow + r) = __halves2half2(ha, hb);
                    st_word_pair(a.w.v + r, make_word(ha, e), make_word(hb, e));
                } else {                              // q, k: interleaved-pair rotation, fp16 rounding per op
                    const int d2 = (r % a.hd) >> 1;
                    const __half cs = cs_row[d2], sn = sn_row[d2];
                    const __half o0 = hsub_ref(hmul_ref(ha, cs), hmul_ref(hb, sn));
                    const __half o1 = hadd_ref(hmul_ref(ha, sn), hmul_ref(hb, cs));
                    if (mat == 1) *reinterpret_cast<__half2*>(krow + r) = __halves2half2(o0, o1);
                    st_word_pair((mat == 0 ? a.w.q : a.w.k) + r, make_word(o0, e), make_word(o1, e));
                }
            });
        }
        if (prof) a.prof[3 * p0 + 2] = globaltimer_ns();
        // ---- [attention] ----------------------------------------------------------------------------------
        named_bar_sync(1, CONSUMER_THREADS);      // the attention scratch shares the activation vector's shared memory
        if (prof) a.prof[3 * (p0 + 1)] = a.prof[3 * (p0 + 1) + 1] = globaltimer_ns();
        if (a.hd <= 64) attn_phase<1>(a, c, l, p0 + 1);
        else if (a.hd <= 128) attn_phase<2>(a, c, l, p0 + 1);
        else attn_phase<4>(a, c, l, p0 + 1);
        named_bar_sync(1, CONSUMER_THREADS);
        if (prof) a.prof[3 * (p0 + 1) + 2] = globaltimer_ns();
        // ---- [wo + residual] ------------------------------------------------------------------------------
        if (prof) a.prof[3 * (p0 + 2)] = globaltimer_ns();
        {
            const uint32_t e_in = e16_of(c, p0 + 1);
            stage_vector(a, c, a.dl, nullptr, [&](int i) { return gather8(a.w.att + 8 * i, e_in, a.status); });
        }
        if (prof) a.prof[3 * (p0 + 2) + 1] = globaltimer_ns();
        {
            const uint32_t e = e16_of(c, p0 + 2);
            const unsigned int e32 = e32_of(c, p0 + 2);
            gemv_consume(a, gemv_desc(a, PH_WO, l), c, [&](int mat, int r, float sa, float sb) {
                if (tp) {                              // K-split: fp32 partial sums into slot [rank] on every rank
#pragma unroll 1
                    for (int d = 0; d < a.world; d++) st_xwords2(a.peer_part[0][d] + r, __float_as_uint(sa), __float_as_uint(sb), e32);
                    return;
                }
                __half r0, r1;                         // h = x + wo(att), fp16 add like Tensor::EwiseAdd
                if (l == 0) { const __half2 rr = *reinterpret_cast<const __half2*>(emb_row + r); r0 = __low2half(rr); r1 = __high2half(rr); }
                else { const uint2 rw = ld_word2(a.w.x + r); r0 = __ushort_as_half(rw.x & 0xffff); r1 = __ushort_as_half(rw.y & 0xffff); }
                st_word_pair(a.w.h + r, make_word(hadd_ref(r0, __float2half_rn(sa)), e), make_word(hadd_ref(r1, __float2half_rn(sb)), e));
            });
        }
        if (prof) a.prof[3 * (p0 + 2) + 2] = globaltimer_ns();
        // ---- [RMSNorm + w1|w3 + SiLU*up] -------------------------------------------------------------------
        named_bar_sync(1, CONSUMER_THREADS);
        if (prof) a.prof[3 * (p0 + 3)] = globaltimer_ns();
        {
            if (tp) reduce_slice_and_publish(a, c, 0, p0 + 2, l == 0 ? nullptr : a.w.x, a.w.h);
            const uint32_t e_in = e16_of(c, p0 + 2);
            stage_vector(a, c, a.dim, lw.ffn_norm, [&](int i) { return gather8(a.w.h + 8 * i, e_in, a.status); });
        }
        if (prof) a.prof[3 * (p0 + 3) + 1] = globaltimer_ns();
        {
            const uint32_t e = e16_of(c, p0 + 3);
            gemv_consume(a, gemv_desc(a, PH_GATEUP, l), c, [&](int mat, int r, float sa, float sb) {
                const __half gate = a.silu_tab[__half_as_ushort(__float2half_rn(sa))];
                st_word1(a.w.g + r, make_word(hmul_ref(gate, __float2half_rn(sb)), e));
            });
        }
        if (prof) a.prof[3 * (p0 + 3) + 2] = globaltimer_ns();
        // ---- [w2 + residual] ------------------------------------------------------------------------------
        named_bar_sync(1, CONSUMER_THREADS);
        if (prof) a.prof[3 * (p0 + 4)] = globaltimer_ns();
        {
            const uint32_t e_in = e16_of(c, p0 + 3);
            stage_vector(a, c, a.hl, nullptr, [&](int i) { return gather8(a.w.g + 8 * i, e_in, a.status); });
        }
        if (prof) a.prof[3 * (p0 + 4) + 1] = globaltimer_ns();
        {
            const uint32_t e = e16_of(c, p0 + 4);
            const unsigned int e32 = e32_of(c, p0 + 4);
            gemv_consume(a, gemv_desc(a, PH_W2, l), c, [&](int mat, int r, float sa, float sb) {
                if (tp) {
#pragma unroll 1
                    for (int d = 0; d < a.world; d++) st_xwords2(a.peer_part[1][d] + r, __float_as_uint(sa), __float_as_uint(sb), e32);
                    return;
                }
                const uint2 rw = ld_word2(a.w.h + r);
                const __half r0 = __ushort_as_half(rw.x & 0xffff), r1 = __ushort_as_half(rw.y & 0xffff);
                st_word_pair(a.w.x + r, make_word(hadd_ref(r0, __float2half_rn(sa)), e), make_word(hadd_ref(r1, __float2half_rn(sb)), e));
            });
        }
        if (prof) a.prof[3 * (p0 + 4) + 2] = globaltimer_ns();
        named_bar_sync(1, CONSUMER_THREADS);
    }
    // ---- [RMSNorm + classifier] + greedy sampling -------------------------------------------------------------
    const int pc = 5 * L;
    if (prof) a.prof[3 * pc] = globaltimer_ns();
    {
        if (tp) reduce_slice_and_publish(a, c, 1, pc - 1, a.w.h, a.w.x);
        const uint32_t e_in = e16_of(c, pc - 1);
        stage_vector(a, c, a.dim, a.final_norm, [&](int i) { return gather8(a.w.x + 8 * i, e_in, a.status); });
    }
    if (prof) a.prof[3 * pc + 1] = globaltimer_ns();
    {
        const unsigned int e32 = e32_of(c, pc);
        gemv_consume(a, gemv_desc(a, PH_CLS, 0), c, [&](int mat, int r, float sa, float sb) {
            const __half ha = __float2half_rn(sa), hb = __float2half_rn(sb);
            if (tp) {                                  // this rank's slice of the logits onto every rank
                const __half2 pair = __halves2half2(ha, hb);
#pragma unroll 1
                for (int d = 0; d < a.world; d++) st_xword(a.peer_logits[d] + (r >> 1), *reinterpret_cast<const unsigned int*>(&pair), e32);
                return;
            }
            *reinterpret_cast<__half2*>(a.logits + r) = __halves2half2(ha, hb);
            const float va = __half2float(ha), vb = __half2float(hb);      // rows ascend within a lane: '>' keeps the lowest index
            if (va > c.best_v || c.best_i == 0x7fffffff) { c.best_v = va; c.best_i = r; }
            if (vb > c.best_v) { c.best_v = vb; c.best_i = r + 1; }
        });
    }
    if (prof) a.prof[3 * pc + 2] = globaltimer_ns();
    if (!c.ok && c.lane == 0) atomicExch(a.status, TL_ERR_TIMEOUT);

    // Greedy sampling (lowest index wins ties, CPU.cpp:358-372) and the bookkeeping of the step.
    int chosen = -1;
    if (tp) {
        // every rank holds all slices once the words of this step have arrived; CTA 0 unpacks and scans them
        if (blockIdx.x != 0) return;
        float bv = -INFINITY;
        int bi = 0x7fffffff;
        const unsigned int e32 = e32_of(c, pc);
        for (int j = c.ctid; 2 * j < a.vocab; j += CONSUMER_THREADS) {
            unsigned int data = 0, flag = 0;
            bool here = false;
            for (unsigned i = 0; i < 2 * a.exchange_tries && !here; i++) {
                asm volatile("ld.volatile.global.v2.u32 {%0, %1}, [%2];" : "=r"(data), "=r"(flag) : "l"(a.local_logits + j) : "memory");
                here = flag == e32;
            }
            if (!here) atomicExch(a.status, TL_ERR_TIMEOUT);
            *reinterpret_cast<unsigned int*>(a.logits + 2 * j) = data;
            const __half2 hh = *reinterpret_cast<const __half2*>(&data);
            const float v0 = __low2float(hh), v1 = __high2float(hh);
            if (bi == 0x7fffffff || v0 > bv) { bv = v0; bi = 2 * j; }
            if (v1 > bv) { bv = v1; bi = 2 * j + 1; }
        }
        c.best_v = bv; c.best_i = bi;
    } else if (c.warp != 0) {
        return;                                        // only warp 0 finished rows; the other warps are done
    }
    // reduce (value, index) over the lanes (and, under tensor parallelism, over the warps of CTA 0)
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, c.best_v, o);
        const int oi = __shfl_xor_sync(0xffffffffu, c.best_i, o);
        if (ov > c.best_v || (ov == c.best_v && oi < c.best_i)) { c.best_v = ov; c.best_i = oi; }
    }
    if (tp) {
        float* sv = c.red;
        int* si = reinterpret_cast<int*>(c.xs);
        named_bar_sync(1, CONSUMER_THREADS);           // everyone is done with the staged vector
        if (c.lane == 0) { sv[c.warp] = c.best_v; si[c.warp] = c.best_i; }
        named_bar_sync(1, CONSUMER_THREADS);
        if (c.ctid == 0) {
            float bv = sv[0]; int bi = si[0];
            for (int w = 1; w < CONSUMERS; w++)
                if (sv[w] > bv || (sv[w] == bv && si[w] < bi)) { bv = sv[w]; bi = si[w]; }
            chosen = bi == 0x7fffffff ? 0 : bi;
        }
    } else if (c.lane == 0) {
        // one candidate per CTA; the last CTA to arrive picks among them
        const unsigned long long cand = ((unsigned long long)__float_as_uint(c.best_v) << 32) | (unsigned int)c.best_i;
        asm volatile("st.volatile.global.u64 [%0], %1;" ::"l"(a.cand + blockIdx.x), "l"(cand) : "memory");
        __threadfence();
        const unsigned int prev = atomicAdd(a.cand_counter, 1u);
        if (prev == gridDim.x - 1) {
            __threadfence();
            *a.cand_counter = 0;
            float bv = -INFINITY; int bi = 0x7fffffff;
            for (unsigned b = 0; b < gridDim.x; b++) {
                const unsigned long long v = __ldcg(a.cand + b);
                const float fv = __uint_as_float((unsigned int)(v >> 32));
                const int iv = (int)(unsigned int)(v & 0xffffffffu);
                if (iv != 0x7fffffff && (fv > bv || (fv == bv && iv < bi) || bi == 0x7fffffff)) { bv = fv; bi = iv; }
            }
            chosen = bi == 0x7fffffff ? 0 : bi;
        }
    }
    if (chosen >= 0) {
        *a.d_next = chosen;
        if (c.pos >= 0 && c.pos < a.max_seq) a.d_generated[c.pos] = chosen;
        *a.d_pos = c.pos + 1;
        *a.step = __ldcg(a.step) + 1u;
    }
}

}  // namespace

// ---------------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------------
int mega_smem_bytes(int max_k) {
    int x_bytes = std::max((max_k * 2 + 127) & ~127, ATT_GROUPS * ATT_SMEM_PER_GROUP);
    x_bytes = (x_bytes + 127) & ~127;
    return NSTAGES * STAGE_BYTES + x_bytes + 2 * NSTAGES * 8 + CONSUMERS * 4 + 2 * CONSUMERS * STAGE_ROWS * 4 + 64;
}

int launch_decode_flow(const FlowArgs& args, int grid, int smem, cudaStream_t st) {
    static PerDeviceOnce once;
    if (once.needed()) {
        TL_CUDA(cudaFuncSetAttribute(k_decode_flow, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
    }
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(MEGA_THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeCooperative;   // all CTAs must be co-resident: they wait on each other
    attr[0].val.cooperative = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    TL_CUDA(cudaLaunchKernelEx(&cfg, k_decode_flow, args));
    return TL_OK;
}

int mega_x_bytes(int max_k) {
    int x_bytes = std::max((max_k * 2 + 127) & ~127, ATT_GROUPS * ATT_SMEM_PER_GROUP);
    return (x_bytes + 127) & ~127;
}

int mega_attn_splits(int H, int grid) {
    int s = 1;
    while (s < 16 && H * s * 2 <= grid * ATT_GROUPS) s *= 2;
    return s;
}

}  // namespace tlb
