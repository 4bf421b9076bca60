// Decode-path GEMV, M = 1..8, fast numerics: y[m,n] = sum_k x[m,k] * W[n,k] with W in the
// llama2.c [out,in] fp16 layout the reference keeps (nn::Linear, tensorLib/src/nn/linear.cpp:10-14).
// Replaces gemv_v6 / gemv_v4 (tensorLib/src/device/cuda/gemv.cu:379-450, :260-306).
//
// The kernels:
//
//  k_gemv_ring (M = 1, the decode step). One persistent CTA per SM. A producer warp streams the
//  CTA's weight rows through a 3-stage shared-memory ring with TMA bulk copies
//  (cp.async.bulk global -> shared, completion on an mbarrier): a stage holds 32 row-chunks of
//  1024 halfs (64 KB), so ~190 KB per SM are in flight independent of what the consumers do.
//  Sixteen consumer warps multiply a stage on the tensor cores: the 32 weight rows are the M side
//  of mma.sync.m16n8k16 (ldmatrix.x4 from the ring), the activation vector staged once in shared
//  memory is column 0 of the B operand, and warp w owns the k16 steps [4w, 4w+4) of every chunk.
//  The 16 per-warp partial sums of each row meet in shared memory at the end of a tile and warp 0
//  applies the epilogue. HBM-bound; algorithmic bytes = 2*(rows*K) + small vectors.
//  The neighbouring operators of the Llama2 block ride along: RMSNorm in the prologue (computed
//  by the consumers while the producer is already streaming: weights never depend on the
//  previous kernel, so the producer does not wait for it), RoPE + KV-cache write / residual add /
//  SiLU*up in the epilogue.
//
//  k_gemv_ring_rows (M = 2..8, tl_matmul2d_f16 / tl_linear_f16): the same ring; the activation rows are
//  columns 0..M-1 of the B fragment the M = 1 kernel fills with one column, so the weights are
//  streamed once for all rows.
//
//  k_gemv_ring2 (tensor-parallel decode): two ring phases in one launch (wo -> gate/up, w2 -> next
//  QKV or classifier); the first phase's epilogue pushes its fp32 partial sums to every rank as
//  (payload, epoch) words, the second phase's prologue sums the ranks' words (every CTA by itself up
//  to four ranks; one slice per CTA, published once per GPU, at eight) behind a bounded wait.
//
//  k_gemv (M = 1..8 for shapes the ring does not take: odd N, K not a multiple of 16): activations
//  staged in shared memory, each warp owns two rows and streams them with 128-bit non-allocating
//  loads, 16 of them in flight per lane.
#include <cstdlib>
#include <cstring>

#include "kernels.cuh"

namespace tlb {

namespace {

// ---------------------------------------------------------------------------------------------
// shared helpers
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ uint4 ldg_stream(const uint4* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
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

// ---- mbarrier / TMA bulk copy (sm_90+ PTX) -------------------------------------------------------
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
// Bounded wait: gives up after WAIT_LIMIT polls (each poll may itself block for a hardware time
// slice), so a logic error shows up as a status word instead of a hung GPU.
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
__device__ __forceinline__ void consumer_bar_sync(int threads) {  // the consumer warps only
    asm volatile("bar.sync 1, %0;" ::"r"(threads) : "memory");
}

// ---------------------------------------------------------------------------------------------
// k_gemv_ring
// ---------------------------------------------------------------------------------------------
constexpr int KC = 1024;                           // halfs per row-chunk
constexpr int CHUNK_BYTES = KC * 2;                // 2 KB: the smallest copy that keeps the TMA request rate off the critical path
// rows sit 2 KB + 16 B apart so that the 8 row addresses of an ldmatrix phase fall into
// different banks
constexpr int ROW_STRIDE = CHUNK_BYTES + 16;
// Two shapes of the same kernel. CW = consumer warps, NST = ring stages; a stage holds CW units =
// 2*CW weight rows (CW/8 m16 MMA tiles).
//   <16, 3>  one CTA per SM, 3 x 64.5 KB ring
//   <8, 3>, <8, 2>  two CTAs per SM (3 or 2 stages of 32 KB, by the size of the staged vector):
//            the same 16 consumer warps and ~190 KB of ring per SM, but a CTA that finishes
//            hands its half of the SM to a CTA of the NEXT kernel, which starts streaming its
//            weights while the other half is still working: the weight stream does not pause at
//            kernel boundaries.
template <int CW, int NST> struct RingCfg {
    static constexpr int THREADS = (CW + 1) * 32;          // + one producer warp
    static constexpr int STAGE_ROWS = CW * 2;
    static constexpr int STAGE_BYTES = STAGE_ROWS * ROW_STRIDE;
    static constexpr int STEPS_PER_WARP = KC / 16 / CW;    // k16 steps of a chunk each warp multiplies
    static constexpr int M16 = STAGE_ROWS / 16;            // m16 tiles per stage
    static constexpr int CTAS_PER_SM = CW == 16 ? 1 : 2;
    static size_t smem_bytes(int K) {
        return (size_t)NST * STAGE_BYTES + (((size_t)K * 2 + 127) & ~(size_t)127) + 2 * NST * sizeof(uint64_t) +
               CW * sizeof(float) + 2 * CW * STAGE_ROWS * sizeof(float) + 64;
    }
};

__device__ __forceinline__ void ldmatrix_x4(uint32_t saddr, uint32_t& a0, uint32_t& a1, uint32_t& a2, uint32_t& a3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(a0), "=r"(a1), "=r"(a2), "=r"(a3)
                 : "r"(saddr));
}
// D(16x8, fp32) += A(16x16 fp16, row) * B(16x8 fp16, col)
__device__ __forceinline__ void mma_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                          uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

struct RingArgs {
    const __half* x; const __half* norm_w; float eps;
    const __half* W0; const __half* W1; const __half* W2;
    int N_each, K, total_units;   // a unit = the two weight rows one consumer warp owns
    __half* y; const __half* residual; float* y32;
    __half* k_out; __half* v_out; const __half* cos_t; const __half* sin_t; int head_dim;
    const int* pos_ptr; long long kv_pitch;
    const __half* silu_tab;
    int* status;                  // device status word: set on a timed-out wait
    int wait_weights;             // the weight stream also waits for the previous kernel (generic entry point)
    int has_xin;                  // the activation vector is residual + sum of pushed partials
    PeerExchange xin, xout;
    unsigned int xin_tries;       // polls of the slots before the tensor-parallel input wait gives up
    unsigned long long* prof;     // optional: CTA 0 stamps %globaltimer at [0] start, [1] vector staged, [2] done
    int m_rows; long long ldx, ldy;   // k_gemv_ring_rows only: activation rows (2..8) and the pitches of x and y
};

// 16 bytes = two (payload, epoch) words, one volatile access (served by L2, where peer stores land)
__device__ __forceinline__ uint4 ld_words2(const unsigned long long* p) {
    uint4 v;
    asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_words2(unsigned long long* p, unsigned int d0, unsigned int d1, unsigned int epoch) {
    asm volatile("st.volatile.global.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(p), "r"(d0), "r"(epoch), "r"(d1), "r"(epoch) : "memory");
}
__device__ __forceinline__ void st_word(unsigned long long* p, unsigned int d, unsigned int epoch) {
    asm volatile("st.volatile.global.v2.u32 [%0], {%1, %2};" ::"l"(p), "r"(d), "r"(epoch) : "memory");
}
__device__ __forceinline__ unsigned int exchange_epoch(const PeerExchange& e) {
    return __ldcg(e.step_ptr) * (unsigned)e.phases_per_step + (unsigned)e.phase_id + 1u;
}

template <int EPI>
__device__ __forceinline__ void unit_rows(const RingArgs& p, int unit, const __half*& ra, const __half*& rb,
                                          int& mat, int& r) {
    if (EPI == EPI_SWIGLU) {  // row `unit` of w1 (gate) and of w3 (up)
        mat = 0; r = unit;
        ra = p.W0 + (long long)unit * p.K;
        rb = p.W1 + (long long)unit * p.K;
    } else {                  // rows 2u, 2u+1 of one of up to three matrices
        int row = unit * 2;
        mat = row / p.N_each;
        r = row - mat * p.N_each;
        const __half* Wm = mat == 0 ? p.W0 : (mat == 1 ? p.W1 : p.W2);
        ra = Wm + (long long)r * p.K;
        rb = ra + p.K;
    }
}

__device__ __forceinline__ unsigned long long globaltimer_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

// Shared-memory view of a ring kernel and the ring position of the calling role. A kernel may run
// several GEMV phases back to back through the same ring (k_gemv_ring2): `it` keeps counting, so
// the producer streams the next phase's weights while the consumers still finish the previous one.
struct RingSmem {
    unsigned char* stages; uint4* xs; float* red; float* partials; uint32_t full0, empty0;
};

// The producer warp of the ring kernels: streams this CTA's weight rows, a stage (2*CW rows x one
// 1024-half chunk) at a time, lane l copying row l of the stage with one bulk copy. Weights only:
// in the model they never depend on the previous kernel; a caller of the plain matmul entry point
// may have just written them (wait_weights). Returns false after a timed-out wait.
template <int EPI, int CW, int NST>
__device__ __forceinline__ bool ring_produce(const RingArgs& p, const RingSmem& sm, int& it, int lane, uint64_t pol) {
    constexpr int CONSUMERS = CW, NSTAGES = NST, STAGE_BYTES = RingCfg<CW, NST>::STAGE_BYTES;
    const int u_begin = (int)((long long)p.total_units * blockIdx.x / gridDim.x);
    const int u_end = (int)((long long)p.total_units * (blockIdx.x + 1) / gridDim.x);
    const int n_units = u_end - u_begin;
    const int n_tiles = (n_units + CONSUMERS - 1) / CONSUMERS;
    const int nk = (p.K + KC - 1) / KC;
    bool ok = true;
    for (int tile = 0; tile < n_tiles && ok; tile++) {
        const int rows_in_tile = min(CONSUMERS, n_units - tile * CONSUMERS) * 2;
        const __half* row_ptr = nullptr;
        if (lane < rows_in_tile) {
            const __half *ra, *rb; int mat, r;
            unit_rows<EPI>(p, u_begin + tile * CONSUMERS + (lane >> 1), ra, rb, mat, r);
            row_ptr = (lane & 1) ? rb : ra;
        }
        for (int chunk = 0; chunk < nk; chunk++, it++) {
            const int s = it % NSTAGES, use = it / NSTAGES;
            if (use > 0) ok = mbar_wait(sm.empty0 + 8 * s, (use - 1) & 1);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            const int kc = min(KC, p.K - chunk * KC);
            if (lane == 0) mbar_arrive_expect_tx(sm.full0 + 8 * s, (uint32_t)(rows_in_tile * kc * 2));
            __syncwarp();
            if (lane < rows_in_tile)
                tma_load_1d(smem_u32(sm.stages + (size_t)s * STAGE_BYTES + (size_t)lane * ROW_STRIDE),
                            row_ptr + (size_t)chunk * KC, (uint32_t)(kc * 2), sm.full0 + 8 * s, pol);
        }
    }
    if (!ok && lane == 0) atomicExch(p.status, TL_ERR_TIMEOUT);
    return ok;
}

// Tensor-parallel input of a GEMV: x = residual + sum over ranks of the partial vectors the ranks
// pushed into this GPU's slots. The sum is formed ONCE per GPU, not once per CTA: CTA c waits for
// (bounded) and adds the slots of its own slice of the vector only (K / gridDim elements: a few
// 16-byte groups), adds the residual, and publishes the fp16 result as (two halfs, epoch) words in a
// local buffer; then every CTA gathers the whole published vector (K/2 words) from L2, retrying
// words whose epoch is not this step's yet. A CTA therefore reads world * K / grid * 8 + K * 4 bytes
// instead of world * K * 8. The CTAs of the grid wait on one another here; that is safe because the
// grid has at most one CTA per SM and the next kernel of the stream cannot start before every CTA
// of this one has been scheduled (it is released by their launch_dependents).
// Returns the 16-byte group c of the vector; all consumer threads must have called
// exchange_reduce_slice first.
template <int CW>
__device__ __forceinline__ void exchange_reduce_slice(const RingArgs& p, unsigned int epoch, int ctid) {
    const PeerExchange& e = p.xin;
    const int K8 = p.K >> 3;
    const int g_begin = (int)((long long)K8 * blockIdx.x / gridDim.x), g_end = (int)((long long)K8 * (blockIdx.x + 1) / gridDim.x);
    for (int c = g_begin + ctid; c < g_end; c += CW * 32) {
        float s[8];
        bool all_here = false;
        for (uint32_t tries = 0; tries < p.xin_tries && !all_here; tries++) {
            all_here = true;
#pragma unroll
            for (int i = 0; i < 8; i++) s[i] = 0.f;
            for (int r = 0; r < e.world; r++) {   // no branch inside: the loads of all ranks are in flight together
                const unsigned long long* src = e.local_slots + (size_t)r * e.n + 8 * c;
#pragma unroll
                for (int q = 0; q < 4; q++) {
                    const uint4 w = ld_words2(src + 2 * q);
                    s[2 * q] += __uint_as_float(w.x);
                    s[2 * q + 1] += __uint_as_float(w.z);
                    all_here &= (w.y == epoch) & (w.w == epoch);
                }
            }
        }
        if (!all_here) atomicExch(p.status, TL_ERR_TIMEOUT);
        uint4 res = __ldcg(reinterpret_cast<const uint4*>(e.residual) + c), out;
        const __half* rh = reinterpret_cast<const __half*>(&res);
        __half* oh = reinterpret_cast<__half*>(&out);
#pragma unroll
        for (int i = 0; i < 8; i++) oh[i] = hadd_ref(rh[i], __float2half_rn(s[i]));
        if (e.sum_out) reinterpret_cast<uint4*>(e.sum_out)[c] = out;
        st_words2(e.local_pub + 4 * c, out.x, out.y, epoch);        // four (half2, epoch) words = one group
        st_words2(e.local_pub + 4 * c + 2, out.z, out.w, epoch);
    }
}
// direct form: this thread sums group c (8 elements) of every rank's slot itself; the CTA whose slice holds c also
// writes the sum to sum_out
__device__ __forceinline__ uint4 exchange_reduce_group(const RingArgs& p, unsigned int epoch, int c, int g_begin, int g_end) {
    const PeerExchange& e = p.xin;
    float s[8];
    bool all_here = false;
    for (uint32_t tries = 0; tries < p.xin_tries && !all_here; tries++) {
        all_here = true;
#pragma unroll
        for (int i = 0; i < 8; i++) s[i] = 0.f;
        for (int r = 0; r < e.world; r++) {
            const unsigned long long* src = e.local_slots + (size_t)r * e.n + 8 * c;
#pragma unroll
            for (int q = 0; q < 4; q++) {
                const uint4 w = ld_words2(src + 2 * q);
                s[2 * q] += __uint_as_float(w.x);
                s[2 * q + 1] += __uint_as_float(w.z);
                all_here &= (w.y == epoch) & (w.w == epoch);
            }
        }
    }
    if (!all_here) atomicExch(p.status, TL_ERR_TIMEOUT);
    uint4 res = __ldcg(reinterpret_cast<const uint4*>(e.residual) + c), out;
    const __half* rh = reinterpret_cast<const __half*>(&res);
    __half* oh = reinterpret_cast<__half*>(&out);
#pragma unroll
    for (int i = 0; i < 8; i++) oh[i] = hadd_ref(rh[i], __float2half_rn(s[i]));
    if (e.sum_out && c >= g_begin && c < g_end) reinterpret_cast<uint4*>(e.sum_out)[c] = out;
    return out;
}
__device__ __forceinline__ uint4 exchange_gather_group(const RingArgs& p, unsigned int epoch, int c) {
    const unsigned long long* src = p.xin.local_pub + 4 * c;
    uint4 lo, hi;
    bool here = false;
    for (uint32_t tries = 0; tries < p.xin_tries && !here; tries++) {
        lo = ld_words2(src);
        hi = ld_words2(src + 2);
        here = (lo.y == epoch) & (lo.w == epoch) & (hi.y == epoch) & (hi.w == epoch);
    }
    if (!here) atomicExch(p.status, TL_ERR_TIMEOUT);
    return make_uint4(lo.x, lo.z, hi.x, hi.z);
}

// The consumer warps' share of one GEMV phase: stage the activation vector (optionally reduced over
// the ranks, optionally RMS-normalised), multiply the stages as they arrive, apply the epilogue.
template <int EPI, bool NORM, int CW, int NST>
__device__ __forceinline__ bool ring_consume(const RingArgs& p, const RingSmem& sm, int& it, int& tile_parity) {
    using Cfg = RingCfg<CW, NST>;
    constexpr int CONSUMERS = CW, NSTAGES = NST, STAGE_ROWS = Cfg::STAGE_ROWS, STAGE_BYTES = Cfg::STAGE_BYTES;
    constexpr int STEPS_PER_WARP = Cfg::STEPS_PER_WARP;
    unsigned char* stages = sm.stages;
    uint4* xs = sm.xs;
    float* red = sm.red;
    float* partials = sm.partials;
    const uint32_t full0 = sm.full0, empty0 = sm.empty0;
    const int K8 = p.K >> 3;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // this CTA's contiguous share of the units, balanced to +-1
    const int u_begin = (int)((long long)p.total_units * blockIdx.x / gridDim.x);
    const int u_end = (int)((long long)p.total_units * (blockIdx.x + 1) / gridDim.x);
    const int n_units = u_end - u_begin;
    const int n_tiles = (n_units + CONSUMERS - 1) / CONSUMERS;
    const int nk = (p.K + KC - 1) / KC;
    const int ctid = threadIdx.x;  // 0 .. 32 * CW - 1
    const uint4* x4 = reinterpret_cast<const uint4*>(p.x);
    float rinv = 1.0f;
    const unsigned int xin_epoch = p.has_xin ? exchange_epoch(p.xin) : 0u;
    const unsigned int xout_epoch = (EPI == EPI_PUSH_F32 || EPI == EPI_PUSH_F16) ? exchange_epoch(p.xout) : 0u;
    const bool xin_direct = p.has_xin && p.xin.direct;
    if (p.has_xin && !xin_direct) exchange_reduce_slice<CW>(p, xin_epoch, ctid);
    const int xg_begin = (int)((long long)K8 * blockIdx.x / gridDim.x), xg_end = (int)((long long)K8 * (blockIdx.x + 1) / gridDim.x);
    // one 16-byte group of the activation vector (plain, or reduced over the ranks)
    auto load_x = [&](int c) -> uint4 {
        if (!p.has_xin) return x4[c];
        return xin_direct ? exchange_reduce_group(p, xin_epoch, c, xg_begin, xg_end) : exchange_gather_group(p, xin_epoch, c);
    };
    if (NORM) {
        // RMSNorm in one pass: the staged vector is x * w (fp16); the scalar 1/rms multiplies the
        // finished dot products instead (sum_k rinv*x_k*w_k*W_nk = rinv * sum_k (x_k*w_k)*W_nk), so
        // no second pass over x has to wait for the block-wide sum of squares.
        float ss = 0.f;
        const uint4* nw4 = reinterpret_cast<const uint4*>(p.norm_w);
        for (int c = ctid; c < K8; c += CONSUMERS * 32) {
            uint4 v = load_x(c), g = nw4[c];
            ss += sumsq8(v);
            __half2* vh = reinterpret_cast<__half2*>(&v);
            const __half2* gh = reinterpret_cast<const __half2*>(&g);
#pragma unroll
            for (int i = 0; i < 4; i++) {
                float2 vf = __half22float2(vh[i]), gf = __half22float2(gh[i]);
                vh[i] = __floats2half2_rn(vf.x * gf.x, vf.y * gf.y);
            }
            xs[c] = v;
        }
        ss = warp_sum(ss);
        if (lane == 0) red[warp] = ss;
        consumer_bar_sync(CONSUMERS * 32);
        float tot = 0.f;
#pragma unroll
        for (int w = 0; w < CONSUMERS; w++) tot += red[w];
        rinv = rsqrtf(tot / (float)p.K + p.eps);
    } else {
        for (int c = ctid; c < K8; c += CONSUMERS * 32) xs[c] = load_x(c);
        consumer_bar_sync(CONSUMERS * 32);
    }
    if (p.prof && blockIdx.x == 0 && ctid == 0) p.prof[1] = globaltimer_ns();

    // Main loop. A stage is a 32-row x 1024-k slab of weights. The dot products run on the tensor
    // cores (mma.sync m16n8k16, fp32 accumulate): the slab's rows are the M dimension (two m16
    // tiles), the activation vector is column 0 of the B operand. Warp w multiplies the k16 steps
    // [w*STEPS_PER_WARP, +STEPS_PER_WARP) of every chunk for all 32 rows; at the end of a tile the
    // 16 per-warp partial sums of each row meet in shared memory and warp 0 finishes the rows.
    // This keeps the consumers' instruction count ~8x below a SIMT FMA loop, so they outrun HBM and
    // the ring can absorb prologue and barrier time.
    // QKV epilogue: the rotary factors of this lane's rows depend only on the position and the row,
    // so warp 0 fetches them now (up to ROPE_PRE tiles) instead of on the critical path of each tile
    constexpr int ROPE_PRE = 4;
    __half2 rope_cs[ROPE_PRE];
    int rope_pos = 0;
    if (EPI == EPI_QKV_ROPE && warp == 0) {
        rope_pos = p.pos_ptr ? *p.pos_ptr : 0;
        const int half_dim = p.head_dim >> 1;
#pragma unroll
        for (int tt = 0; tt < ROPE_PRE; tt++) {
            rope_cs[tt] = __half2half2(__float2half(0.f));
            const int unit = u_begin + tt * CONSUMERS + (lane >> 1);
            if (tt < n_tiles && !(lane & 1) && unit < u_end) {
                const __half *ra, *rb; int mat, r;
                unit_rows<EPI>(p, unit, ra, rb, mat, r);
                if (mat < 2) {
                    const int d2 = (r % p.head_dim) >> 1;
                    rope_cs[tt] = __halves2half2(p.cos_t[(long long)rope_pos * half_dim + d2],
                                                 p.sin_t[(long long)rope_pos * half_dim + d2]);
                }
            }
        }
    }
    // residual epilogue: the two residual values of this lane's rows, fetched ahead the same way
    __half2 res_pre[ROPE_PRE];
    if (EPI == EPI_RESIDUAL && warp == 0) {
#pragma unroll
        for (int tt = 0; tt < ROPE_PRE; tt++) {
            res_pre[tt] = __half2half2(__float2half(0.f));
            const int unit = u_begin + tt * CONSUMERS + (lane >> 1);
            if (tt < n_tiles && !(lane & 1) && unit < u_end)
                res_pre[tt] = *reinterpret_cast<const __half2*>(p.residual + 2 * unit);   // rows 2u, 2u+1 of the single matrix
        }
    }
    bool ok = true;
    const int g = lane >> 2, t = lane & 3;
    // ldmatrix row addresses: lanes 0-7 rows 0-7 (k 0-7), 8-15 rows 8-15, 16-23 rows 0-7 (k 8-15), 24-31 rows 8-15
    const uint32_t lm_off = (uint32_t)(((lane & 7) + ((lane >> 3) & 1) * 8) * ROW_STRIDE + (lane >> 4) * 16);
    const __half* xh = reinterpret_cast<const __half*>(xs);
    for (int tile = 0; tile < n_tiles && ok; tile++) {
        const int units_here = min(CONSUMERS, n_units - tile * CONSUMERS);
        float acc0[4] = {0.f, 0.f, 0.f, 0.f}, acc1[4] = {0.f, 0.f, 0.f, 0.f};   // acc1: second m16 tile (CW = 16 only)
        for (int chunk = 0; chunk < nk; chunk++, it++) {
            const int s = it % NSTAGES, use = it / NSTAGES;
            ok = mbar_wait(full0 + 8 * s, use & 1);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            const int steps = min(KC, p.K - chunk * KC) >> 4;
            const uint32_t sbase = smem_u32(stages + (size_t)s * STAGE_BYTES) + lm_off;
#pragma unroll
            for (int kk = 0; kk < STEPS_PER_WARP; kk++) {
                const int step = warp * STEPS_PER_WARP + kk;
                if (step < steps) {
                    uint32_t a0, a1, a2, a3;
                    ldmatrix_x4(sbase + step * 32, a0, a1, a2, a3);
                    const __half* xk = xh + chunk * KC + step * 16 + 2 * t;
                    const uint32_t b0 = *reinterpret_cast<const uint32_t*>(xk);
                    const uint32_t b1 = *reinterpret_cast<const uint32_t*>(xk + 8);
                    mma_16816(acc0, a0, a1, a2, a3, b0, b1);
                    if (Cfg::M16 == 2) {
                        uint32_t c0, c1, c2, c3;
                        ldmatrix_x4(sbase + 16 * ROW_STRIDE + step * 32, c0, c1, c2, c3);
                        mma_16816(acc1, c0, c1, c2, c3, b0, b1);
                    }
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(empty0 + 8 * s);
        }
        if (!ok) break;
        // column 0 of the accumulators lives in the lanes with t == 0: rows g and g+8 of each m16 tile
        float* part = partials + (tile_parity & 1) * (CONSUMERS * STAGE_ROWS);
        tile_parity ^= 1;
        if (t == 0) {
            part[warp * STAGE_ROWS + g] = acc0[0];
            part[warp * STAGE_ROWS + g + 8] = acc0[2];
            if (Cfg::M16 == 2) {
                part[warp * STAGE_ROWS + 16 + g] = acc1[0];
                part[warp * STAGE_ROWS + 24 + g] = acc1[2];
            }
        }
        consumer_bar_sync(CONSUMERS * 32);
        if (warp != 0) continue;
        float rowsum = 0.f;   // lane = row slot of the stage: slots 2u, 2u+1 are the two rows of unit u
#pragma unroll
        for (int w = 0; w < CONSUMERS; w++) rowsum += part[w * STAGE_ROWS + (lane & (STAGE_ROWS - 1))];
        const float other = __shfl_xor_sync(0xffffffffu, rowsum, 1);
        if ((lane & 1) || (lane >> 1) >= units_here) continue;
        const float sa = rowsum * rinv, sb = other * rinv;
        const __half ha = __float2half_rn(sa), hb = __float2half_rn(sb);
        const __half *ra, *rb; int mat, r;
        unit_rows<EPI>(p, u_begin + tile * CONSUMERS + (lane >> 1), ra, rb, mat, r);
        if (EPI == EPI_STORE) {
            p.y[(long long)mat * p.N_each + r] = ha;
            p.y[(long long)mat * p.N_each + r + 1] = hb;
        } else if (EPI == EPI_STORE_F32) {
            p.y32[(long long)mat * p.N_each + r] = sa;
            p.y32[(long long)mat * p.N_each + r + 1] = sb;
        } else if (EPI == EPI_PUSH_F32) {  // K-split partial sums into slot [rank] on every rank
#pragma unroll 1
            for (int d = 0; d < p.xout.world; d++)
                st_words2(p.xout.peer_slot[d] + r, __float_as_uint(sa), __float_as_uint(sb), xout_epoch);
        } else if (EPI == EPI_PUSH_F16) {  // row-split results (classifier slice) onto every rank
#pragma unroll 1
            const __half2 pair = __halves2half2(ha, hb);
            for (int d = 0; d < p.xout.world; d++)
                st_word(p.xout.peer_slot[d] + (r >> 1), *reinterpret_cast<const unsigned int*>(&pair), xout_epoch);
        } else if (EPI == EPI_RESIDUAL) {  // h = x + linear(...), fp16 add like Tensor::EwiseAdd
            __half r0, r1;
            if (tile < ROPE_PRE) {
                __half2 rr = res_pre[0];
#pragma unroll
                for (int tt = 1; tt < ROPE_PRE; tt++) if (tile == tt) rr = res_pre[tt];
                r0 = __low2half(rr); r1 = __high2half(rr);
            } else {
                r0 = p.residual[r]; r1 = p.residual[r + 1];
            }
            p.y[r] = hadd_ref(r0, ha);
            p.y[r + 1] = hadd_ref(r1, hb);
        } else if (EPI == EPI_QKV_ROPE) {
            const int pos = rope_pos;
            if (mat == 2) {                // v: straight into the cache row of this position
                __half* vo = p.v_out + (long long)pos * p.kv_pitch;
                vo[r] = ha; vo[r + 1] = hb;
            } else {                       // q, k: interleaved-pair rotation, fp16 rounding per op
                const int half_dim = p.head_dim >> 1;
                const int d2 = (r % p.head_dim) >> 1;
                __half c, s;
                if (tile < ROPE_PRE) {
                    __half2 cs = rope_cs[0];
#pragma unroll
                    for (int tt = 1; tt < ROPE_PRE; tt++) if (tile == tt) cs = rope_cs[tt];
                    c = __low2half(cs); s = __high2half(cs);
                } else {
                    c = p.cos_t[(long long)pos * half_dim + d2];
                    s = p.sin_t[(long long)pos * half_dim + d2];
                }
                const __half o0 = hsub_ref(hmul_ref(ha, c), hmul_ref(hb, s));
                const __half o1 = hadd_ref(hmul_ref(ha, s), hmul_ref(hb, c));
                __half* dst = mat == 0 ? p.y : p.k_out + (long long)pos * p.kv_pitch;
                dst[r] = o0; dst[r + 1] = o1;
            }
        } else {                           // EPI_SWIGLU: silu(gate) * up, each rounded to fp16
            const __half g = p.silu_tab[__half_as_ushort(ha)];
            p.y[r] = hmul_ref(g, hb);
        }
    }
    if (!ok && lane == 0) atomicExch(p.status, TL_ERR_TIMEOUT);
    return ok;
}

template <int CW, int NST>
__device__ __forceinline__ RingSmem ring_smem_init(unsigned char* smem, int max_k) {
    using Cfg = RingCfg<CW, NST>;
    // layout: [NST stages][x: max_k halfs][full barriers][empty barriers][reduction scratch]
    RingSmem sm;
    sm.stages = smem;
    sm.xs = reinterpret_cast<uint4*>(smem + NST * Cfg::STAGE_BYTES);
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + NST * Cfg::STAGE_BYTES + (((size_t)max_k * 2 + 127) & ~(size_t)127));
    sm.red = reinterpret_cast<float*>(bars + 2 * NST);
    sm.partials = sm.red + CW;  // [2][CW][STAGE_ROWS] per-warp partial row sums, double buffered
    sm.full0 = smem_u32(bars);
    sm.empty0 = smem_u32(bars + NST);
    if (threadIdx.x == 0) {
        for (int s = 0; s < NST; s++) {
            mbar_init(sm.full0 + 8 * s, 1);
            mbar_init(sm.empty0 + 8 * s, CW);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    return sm;
}

template <int EPI, bool NORM, int CW, int NST>
__global__ void __launch_bounds__(RingCfg<CW, NST>::THREADS, RingCfg<CW, NST>::CTAS_PER_SM) k_gemv_ring(RingArgs p) {
    extern __shared__ __align__(128) unsigned char smem[];
    const bool stamp = p.prof && blockIdx.x == 0 && threadIdx.x == 0;
    if (stamp) p.prof[0] = globaltimer_ns();
    const RingSmem sm = ring_smem_init<CW, NST>(smem, p.K);
    pdl_launch_dependents();
    int it = 0;
    if ((threadIdx.x >> 5) == CW) {
        if (p.wait_weights) pdl_wait();
        ring_produce<EPI, CW, NST>(p, sm, it, threadIdx.x & 31, policy_evict_first());
        return;
    }
    pdl_wait();  // activations written by the previous kernel are visible from here on
    int tile_parity = 0;
    ring_consume<EPI, NORM, CW, NST>(p, sm, it, tile_parity);
    if (stamp) p.prof[2] = globaltimer_ns();
}

// Two GEMV phases of the tensor-parallel decode step in one launch, through one ring:
//   phase A  a K-split matmul (wo or w2) whose fp32 partial sums are pushed to every rank, then
//   phase B  the matmul that consumes the exchanged sum: RMSNorm + w1|w3 + SiLU*up after wo,
//            RMSNorm + wq|wk|wv + RoPE + KV write (next layer) or RMSNorm + classifier after w2.
// Between the two the consumers only wait for what phase B needs anyway, the partial sums of all
// ranks; the producer warp does not wait at all and fills the ring with phase B's weights while the
// partial sums travel. This takes one launch and one kernel boundary out of every exchange.
template <int EPI_B>
__global__ void __launch_bounds__(RingCfg<16, 3>::THREADS, 1) k_gemv_ring2(RingArgs pa, RingArgs pb) {
    extern __shared__ __align__(128) unsigned char smem[];
    const bool stamp = pa.prof && blockIdx.x == 0 && threadIdx.x == 0;
    if (stamp) pa.prof[0] = globaltimer_ns();
    const RingSmem sm = ring_smem_init<16, 3>(smem, max(pa.K, pb.K));
    pdl_launch_dependents();
    int it = 0;
    if ((threadIdx.x >> 5) == 16) {
        const uint64_t pol = policy_evict_first();
        if (ring_produce<EPI_PUSH_F32, 16, 3>(pa, sm, it, threadIdx.x & 31, pol))
            ring_produce<EPI_B, 16, 3>(pb, sm, it, threadIdx.x & 31, pol);
        return;
    }
    pdl_wait();
    int tile_parity = 0;
    if (!ring_consume<EPI_PUSH_F32, false, 16, 3>(pa, sm, it, tile_parity)) return;
    if (stamp) pa.prof[2] = globaltimer_ns();
    consumer_bar_sync(16 * 32);        // every warp is done with phase A's activation vector
    if (stamp) pb.prof[0] = globaltimer_ns();
    ring_consume<EPI_B, true, 16, 3>(pb, sm, it, tile_parity);
    if (stamp) pb.prof[2] = globaltimer_ns();
}

// ---------------------------------------------------------------------------------------------
// k_gemv_ring_rows<G>: the same ring for 2..8 G activation rows (used with G = 1: tl_matmul2d_f16 with M = 2..8).
// The B operand of mma.sync.m16n8k16 has eight columns; the M = 1 kernel fills column 0 only. Here
// column m of column group j is activation row 8 j + m, so up to 8 G rows cost the weight stream of
// one: the kernel stays HBM-bound at 2*N*K bytes. The 16 consumer warps form a (16 / G) x G grid:
// warp (kq, cg) multiplies the k16 steps [kq * 4 G, (kq + 1) * 4 G) of every chunk against column
// group cg for all 32 rows of a stage, so a stage is read from shared memory G times (G = 4:
// 256 KB per 64 KB stage, ~1 us at 128 B/clk against the ~1.5 us a stage takes to arrive from HBM).
// The activation rows (up to 32 x K halfs) do not fit beside the 3 x 64.5 KB ring, so they are not
// staged: every lane fetches its B fragments (row 8 cg + lane/4, two 4-byte words per k16 step) for
// the coming chunk straight from global memory BEFORE it waits for the chunk's weights, which hides
// the L1/L2 latency behind the HBM latency of the stage. Per-warp partial sums [32 rows x 8 columns]
// meet in shared memory (16 KB whatever G is); warp w finishes the two rows of unit w.
// ---------------------------------------------------------------------------------------------
struct RowsCfg {
    using Ring = RingCfg<16, 3>;
    static constexpr int PART_FLOATS = 16 * Ring::STAGE_ROWS * 8;   // per buffer: [kq][row][8 G columns] = 16 warps x 32 rows x 8
    static size_t smem_bytes() {
        return (size_t)3 * Ring::STAGE_BYTES + 2 * 3 * sizeof(uint64_t) + 16 + 2 * PART_FLOATS * sizeof(float);
    }
};

__device__ __forceinline__ uint32_t ldg_u32(const __half* p) {
    return __ldg(reinterpret_cast<const unsigned int*>(p));
}

template <int G>
__global__ void __launch_bounds__(RingCfg<16, 3>::THREADS, 1) k_gemv_ring_rows(RingArgs p) {
    using Cfg = RingCfg<16, 3>;
    constexpr int CONSUMERS = 16, NSTAGES = 3, STAGE_ROWS = Cfg::STAGE_ROWS, STAGE_BYTES = Cfg::STAGE_BYTES;
    constexpr int KQ = CONSUMERS / G;            // ways the k16 steps of a chunk are split
    constexpr int STEPS = (KC / 16) / KQ;        // steps per warp and chunk
    constexpr int COLS = 8 * G;
    extern __shared__ __align__(128) unsigned char smem[];
    // layout: [3 stages][full barriers][empty barriers][pad][partials: 2 buffers]
    unsigned char* stages = smem;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + NSTAGES * STAGE_BYTES);
    float* partials = reinterpret_cast<float*>(smem + NSTAGES * STAGE_BYTES + 2 * NSTAGES * sizeof(uint64_t) + 16);
    const uint32_t full0 = smem_u32(bars), empty0 = smem_u32(bars + NSTAGES);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int u_begin = (int)((long long)p.total_units * blockIdx.x / gridDim.x);
    const int u_end = (int)((long long)p.total_units * (blockIdx.x + 1) / gridDim.x);
    const int n_units = u_end - u_begin;
    const int n_tiles = (n_units + CONSUMERS - 1) / CONSUMERS;
    const int nk = (p.K + KC - 1) / KC;

    if (threadIdx.x == 0) {
        for (int s = 0; s < NSTAGES; s++) {
            mbar_init(full0 + 8 * s, 1);
            mbar_init(empty0 + 8 * s, CONSUMERS);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    pdl_launch_dependents();

    if (warp == CONSUMERS) {
        if (p.wait_weights) pdl_wait();
        const RingSmem sm{stages, nullptr, nullptr, nullptr, full0, empty0};
        int pit = 0;
        ring_produce<EPI_STORE, 16, 3>(p, sm, pit, lane, policy_evict_first());
        return;
    }

    pdl_wait();  // the activation rows may have been written by the previous kernel
    const int kq = warp / G, cg = warp % G;
    const int g = lane >> 2, t = lane & 3;
    const int xrow_idx = 8 * cg + g;                           // column g of this warp's B = activation row 8 cg + g
    const bool col_ok = xrow_idx < p.m_rows;
    const __half* xrow = p.x + (long long)(col_ok ? xrow_idx : 0) * p.ldx + 2 * t;
    const uint32_t lm_off = (uint32_t)(((lane & 7) + ((lane >> 3) & 1) * 8) * ROW_STRIDE + (lane >> 4) * 16);
    bool ok = true;
    int it = 0;
    for (int tile = 0; tile < n_tiles && ok; tile++) {
        const int units_here = min(CONSUMERS, n_units - tile * CONSUMERS);
        float acc0[4] = {0.f, 0.f, 0.f, 0.f}, acc1[4] = {0.f, 0.f, 0.f, 0.f};
        for (int chunk = 0; chunk < nk; chunk++, it++) {
            const int s = it % NSTAGES, use = it / NSTAGES;
            const int steps = min(KC, p.K - chunk * KC) >> 4;
            // this warp's B fragments of the chunk, in flight while the weights arrive
            uint32_t b0[STEPS], b1[STEPS];
#pragma unroll
            for (int kk = 0; kk < STEPS; kk++) {
                const int step = kq * STEPS + kk;
                b0[kk] = b1[kk] = 0u;
                if (col_ok && step < steps) {
                    const __half* xk = xrow + chunk * KC + step * 16;
                    b0[kk] = ldg_u32(xk);
                    b1[kk] = ldg_u32(xk + 8);
                }
            }
            ok = mbar_wait(full0 + 8 * s, use & 1);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            const uint32_t sbase = smem_u32(stages + (size_t)s * STAGE_BYTES) + lm_off;
#pragma unroll
            for (int kk = 0; kk < STEPS; kk++) {
                const int step = kq * STEPS + kk;
                if (step < steps) {
                    uint32_t a0, a1, a2, a3, c0, c1, c2, c3;
                    ldmatrix_x4(sbase + step * 32, a0, a1, a2, a3);
                    mma_16816(acc0, a0, a1, a2, a3, b0[kk], b1[kk]);
                    ldmatrix_x4(sbase + 16 * ROW_STRIDE + step * 32, c0, c1, c2, c3);
                    mma_16816(acc1, c0, c1, c2, c3, b0[kk], b1[kk]);
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(empty0 + 8 * s);
        }
        if (!ok) break;
        // accumulator layout: d[0], d[1] = (row g, columns 2t, 2t+1); d[2], d[3] = (row g + 8, same columns).
        // partials[kq][row][8 cg + column]
        float* part = partials + (tile & 1) * RowsCfg::PART_FLOATS + kq * (STAGE_ROWS * COLS) + 8 * cg;
        *reinterpret_cast<float2*>(part + g * COLS + 2 * t) = make_float2(acc0[0], acc0[1]);
        *reinterpret_cast<float2*>(part + (g + 8) * COLS + 2 * t) = make_float2(acc0[2], acc0[3]);
        *reinterpret_cast<float2*>(part + (g + 16) * COLS + 2 * t) = make_float2(acc1[0], acc1[1]);
        *reinterpret_cast<float2*>(part + (g + 24) * COLS + 2 * t) = make_float2(acc1[2], acc1[3]);
        consumer_bar_sync(CONSUMERS * 32);
        // warp w finishes unit w of the tile: 2 rows x 8 G columns, each the sum of KQ partials
        const float* src = partials + (tile & 1) * RowsCfg::PART_FLOATS + (2 * warp) * COLS;
#pragma unroll
        for (int o = lane; o < 2 * COLS; o += 32) {
            float sum = 0.f;
#pragma unroll
            for (int q = 0; q < KQ; q++) sum += src[q * (STAGE_ROWS * COLS) + o];
            const int col = o % COLS;
            if (warp < units_here && col < p.m_rows) {
                const int n = (u_begin + tile * CONSUMERS + warp) * 2 + o / COLS;
                p.y[(long long)col * p.ldy + n] = __float2half_rn(sum);
            }
        }
    }
    if (!ok && lane == 0) atomicExch(p.status, TL_ERR_TIMEOUT);
}

// ---------------------------------------------------------------------------------------------
// Plain GEMV for M rows of x (tl_matmul2d_f16 with M <= 8).
// x is staged in K-tiles of KT halfs so that M*KT*2 bytes fit a 32 KB shared buffer.
// ---------------------------------------------------------------------------------------------
constexpr int WARPS = 8;
constexpr int THREADS = WARPS * 32;
constexpr int UNROLL = 8;  // 16-byte chunks per row kept in flight per lane

template <int M>
__global__ void __launch_bounds__(THREADS) k_gemv(const __half* __restrict__ x, const __half* __restrict__ W,
                                                  __half* __restrict__ y, int N, int K, long long ldw,
                                                  long long ldx, long long ldy, int KT) {
    extern __shared__ uint4 xsm[];  // [M][KT/8]
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int row0 = (blockIdx.x * WARPS + warp) * 2;
    const bool has0 = row0 < N, has1 = row0 + 1 < N;
    const uint4* w0 = reinterpret_cast<const uint4*>(W + (long long)(has0 ? row0 : 0) * ldw);
    const uint4* w1 = reinterpret_cast<const uint4*>(W + (long long)(has1 ? row0 + 1 : 0) * ldw);
    float acc0[M], acc1[M];
#pragma unroll
    for (int m = 0; m < M; m++) acc0[m] = acc1[m] = 0.f;

    for (int k0 = 0; k0 < K; k0 += KT) {
        const int kt8 = (min(KT, K - k0)) >> 3;  // 16-byte chunks in this tile
        if (k0) __syncthreads();
        for (int i = threadIdx.x; i < M * kt8; i += THREADS) {
            int m = i / kt8, c = i - m * kt8;
            xsm[m * (KT >> 3) + c] = reinterpret_cast<const uint4*>(x + (long long)m * ldx + k0)[c];
        }
        __syncthreads();
        if (has0) {
            const uint4* a0 = w0 + (k0 >> 3);
            const uint4* a1 = w1 + (k0 >> 3);
            for (int c0 = lane; c0 < kt8; c0 += 32 * UNROLL) {
                uint4 v0[UNROLL], v1[UNROLL];
#pragma unroll
                for (int u = 0; u < UNROLL; u++) {
                    int c = c0 + u * 32;
                    if (c < kt8) { v0[u] = ldg_stream(a0 + c); v1[u] = ldg_stream(a1 + c); }
                }
#pragma unroll
                for (int u = 0; u < UNROLL; u++) {
                    int c = c0 + u * 32;
                    if (c < kt8) {
#pragma unroll
                        for (int m = 0; m < M; m++) {
                            uint4 xv = xsm[m * (KT >> 3) + c];
                            acc0[m] = dot8(v0[u], xv, acc0[m]);
                            acc1[m] = dot8(v1[u], xv, acc1[m]);
                        }
                    }
                }
            }
        }
    }
    if (!has0) return;
#pragma unroll
    for (int m = 0; m < M; m++) {
        float s0 = warp_sum(acc0[m]), s1 = warp_sum(acc1[m]);
        if (lane == 0) {
            y[(long long)m * ldy + row0] = __float2half_rn(s0);
            if (has1) y[(long long)m * ldy + row0 + 1] = __float2half_rn(s1);
        }
    }
}

template <int EPI, bool NORM, int CW, int NST>
int launch_ring_cfg(const RingArgs& a, cudaStream_t st, bool pdl) {
    using Cfg = RingCfg<CW, NST>;
    static PerDeviceOnce once;
    if (once.needed()) {
        TL_CUDA(cudaFuncSetAttribute(k_gemv_ring<EPI, NORM, CW, NST>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     CW == 16 ? 227 * 1024 : 113 * 1024));
        if (CW != 16)
            TL_CUDA(cudaFuncSetAttribute(k_gemv_ring<EPI, NORM, CW, NST>, cudaFuncAttributePreferredSharedMemoryCarveout,
                                         (int)cudaSharedmemCarveoutMaxShared));
    }
    // persistent CTAs, each with a contiguous share of the units balanced to +-1; a CTA's last stage may
    // be partly filled (it streams only its own rows), so every SM gets work as soon as there is half
    // a stage of units per CTA: N = 4096 spreads over all 148 SMs instead of 128 full stages
    const int grid = std::max(1, std::min(sm_count() * Cfg::CTAS_PER_SM, (a.total_units + CW / 2 - 1) / (CW / 2)));
    return launch_pdl(k_gemv_ring<EPI, NORM, CW, NST>, dim3(grid), dim3(Cfg::THREADS), Cfg::smem_bytes(a.K), st, pdl, a);
}

// 0: one CTA per SM (default); 1: two half-size CTAs per SM (TL_RING=half). Measured on the 7B decode
// step with both shapes spreading N = 4096 over all SMs: 2.459 ms per token for the full shape,
// 2.483 ms for the half shape on one GPU, and -13 % for the half shape under 2-GPU tensor
// parallelism (every CTA sums all ranks' partial vectors in its prologue, and there are twice as
// many CTAs). The half shape stays selectable for experiments.
int ring_shape_choice() {
    static const int forced = [] {
        const char* e = getenv("TL_RING");
        return !e ? 0 : (!strcmp(e, "half") ? 1 : 0);
    }();
    return forced;
}

template <int EPI, bool NORM>
int launch_ring(const RingArgs& a, cudaStream_t st, bool pdl) {
    if (ring_shape_choice() == 1) {
        if (RingCfg<8, 3>::smem_bytes(a.K) <= 113 * 1024) return launch_ring_cfg<EPI, NORM, 8, 3>(a, st, pdl);
        if (RingCfg<8, 2>::smem_bytes(a.K) <= 113 * 1024) return launch_ring_cfg<EPI, NORM, 8, 2>(a, st, pdl);
    }
    return launch_ring_cfg<EPI, NORM, 16, 3>(a, st, pdl);
}

}  // namespace

bool gemv_supported(const void* x, const void* W, size_t M, size_t N, size_t K, size_t ldw) {
    auto al16 = [](const void* q) { return (reinterpret_cast<uintptr_t>(q) & 15) == 0; };
    return M >= 1 && M <= 8 && N >= 1 && K >= 8 && K % 8 == 0 && ldw % 8 == 0 && al16(x) && al16(W);
}

bool gemv_ring_rows_supported(const void* x, const void* W, size_t M, size_t N, size_t K, size_t ldw, size_t ldx) {
    auto al16 = [](const void* q) { return (reinterpret_cast<uintptr_t>(q) & 15) == 0; };
    // More than eight rows (G = 2, 4 column groups) measured slower than the skinny tensor-core kernel: 16 or 32
    // activation rows no longer fit the ~28 KB of L1 left beside the ring, so the B fragments come from L2 at two to
    // four times the bytes of the weight stream (M = 16: 27.3 us against 22.7 us at 4096 x 11008; M = 32: 51.8 against 23.8).
    return M >= 2 && M <= 8 && N >= 2 && K >= 16 && al16(x) && al16(W) && ldx % 8 == 0 && ldw == K && N % 2 == 0 && K % 16 == 0;
}

int launch_gemv(const __half* x, const __half* W, __half* y, int M, int N, int K, long long ldw,
                long long ldx, long long ldy, cudaStream_t st, bool weights_constant) {
    TL_REQUIRE((gemv_supported(x, W, M, N, K, ldw) && ldx % 8 == 0) || gemv_ring_rows_supported(x, W, M, N, K, ldw, ldx),
               "gemv: unsupported shape or alignment");
    if (M == 1 && ldw == K && N % 2 == 0 && K % 16 == 0 && K <= 12288) {  // the decode kernel, plain store epilogue
        FusedGemv f{};
        f.x = x; f.W[0] = W; f.n_mats = 1; f.N_each = N; f.K = K; f.epilogue = EPI_STORE; f.y = y;
        f.pdl = true; f.weights_may_change = !weights_constant;
        return launch_fused_gemv(f, st);
    }
    if (gemv_ring_rows_supported(x, W, M, N, K, ldw, ldx)) {   // up to eight rows at the weight traffic of one
        static PerDeviceOnce once;
        if (once.needed())
            TL_CUDA(cudaFuncSetAttribute(k_gemv_ring_rows<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)RowsCfg::smem_bytes()));
        RingArgs a{};
        a.x = x; a.W0 = W; a.N_each = N; a.K = K; a.total_units = N / 2; a.y = y;
        a.status = device_status_word(); a.wait_weights = weights_constant ? 0 : 1;
        a.m_rows = M; a.ldx = ldx; a.ldy = ldy;
        const int grid = std::max(1, std::min(sm_count(), (a.total_units + 7) / 8));
        return launch_pdl(k_gemv_ring_rows<1>, dim3(grid), dim3(RingCfg<16, 3>::THREADS), RowsCfg::smem_bytes(), st, true, a);
    }
    int KT = 16384 / M;                 // halfs per tile so that M*KT*2 <= 32 KB
    KT &= ~255;
    if (KT > K) KT = (K + 7) & ~7;
    size_t smem = (size_t)M * KT * sizeof(__half);
    dim3 grid((unsigned)ceil_div(ceil_div(N, 2), WARPS)), block(THREADS);
#define TL_GEMV_CASE(MM) \
    case MM: k_gemv<MM><<<grid, block, smem, st>>>(x, W, y, N, K, ldw, ldx, ldy, KT); break;
    switch (M) {
        TL_GEMV_CASE(1) TL_GEMV_CASE(2) TL_GEMV_CASE(3) TL_GEMV_CASE(4)
        TL_GEMV_CASE(5) TL_GEMV_CASE(6) TL_GEMV_CASE(7) TL_GEMV_CASE(8)
    }
#undef TL_GEMV_CASE
    TL_LAUNCH_CHECK();
    return TL_OK;
}

namespace {
int build_ring_args(const FusedGemv& q, RingArgs* out) {
    auto al16 = [](const void* v) { return (reinterpret_cast<uintptr_t>(v) & 15) == 0; };
    TL_REQUIRE(q.K >= 16 && q.K % 16 == 0 && q.K <= 12288, "fused gemv: K=%d must be a multiple of 16, <= 12288", q.K);
    TL_REQUIRE(q.N_each > 0 && q.N_each % 2 == 0, "fused gemv: N must be even");
    TL_REQUIRE(al16(q.x) && al16(q.W[0]) && (!q.norm_w || al16(q.norm_w)), "fused gemv: 16-byte alignment required");
    for (int i = 1; i < q.n_mats; i++) TL_REQUIRE(al16(q.W[i]), "fused gemv: 16-byte alignment required");
    RingArgs a{};
    a.x = q.x; a.norm_w = q.norm_w; a.eps = q.eps;
    a.W0 = q.W[0]; a.W1 = q.n_mats > 1 ? q.W[1] : nullptr; a.W2 = q.n_mats > 2 ? q.W[2] : nullptr;
    a.N_each = q.N_each; a.K = q.K;
    a.y = q.y; a.residual = q.residual; a.y32 = q.y32;
    a.k_out = q.k_out; a.v_out = q.v_out; a.cos_t = q.cos_row; a.sin_t = q.sin_row; a.head_dim = q.head_dim;
    a.pos_ptr = q.pos_ptr; a.kv_pitch = q.kv_pitch;
    a.silu_tab = tables().silu_float_tab;
    a.status = device_status_word();
    a.wait_weights = q.weights_may_change ? 1 : 0;
    a.has_xin = q.xin != nullptr;
    a.prof = q.prof;
    if (q.xin) {
        TL_REQUIRE(q.xin->world >= 1 && q.xin->world <= TL_MAX_TP && q.xin->n == q.K && q.xin->residual && q.xin->local_pub &&
                   q.K % 8 == 0, "fused gemv: bad exchange input");
        a.xin = *q.xin;
        a.xin_tries = q.xin_tries ? q.xin_tries : TL_EXCHANGE_TRIES;
    }
    if (q.epilogue == EPI_PUSH_F32 || q.epilogue == EPI_PUSH_F16) {
        TL_REQUIRE(q.xout && q.n_mats == 1 && q.xout->world >= 1 && q.xout->world <= TL_MAX_TP, "fused gemv: bad exchange output");
        a.xout = *q.xout;
    }
    if (q.epilogue == EPI_SWIGLU) {
        TL_REQUIRE(q.n_mats == 2, "swiglu epilogue needs w1 and w3");
        a.total_units = q.N_each;
    } else {
        if (q.epilogue == EPI_QKV_ROPE)
            TL_REQUIRE(q.n_mats == 3 && q.head_dim % 2 == 0 && q.N_each % q.head_dim == 0, "qkv epilogue: bad shape");
        if (q.epilogue == EPI_RESIDUAL) TL_REQUIRE(q.n_mats == 1 && q.residual, "residual epilogue: one matrix and a residual");
        a.total_units = q.n_mats * q.N_each / 2;
    }
    *out = a;
    return TL_OK;
}

template <int EPI_B>
int launch_ring2(const RingArgs& a, const RingArgs& b, cudaStream_t st, bool pdl) {
    using Cfg = RingCfg<16, 3>;
    static PerDeviceOnce once;
    if (once.needed())
        TL_CUDA(cudaFuncSetAttribute(k_gemv_ring2<EPI_B>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
    const int units = std::max(a.total_units, b.total_units);
    const int grid = std::max(1, std::min(sm_count(), (units + 7) / 8));
    return launch_pdl(k_gemv_ring2<EPI_B>, dim3(grid), dim3(Cfg::THREADS), Cfg::smem_bytes(std::max(a.K, b.K)), st, pdl, a, b);
}
}  // namespace

int launch_fused_gemv(const FusedGemv& q, cudaStream_t st) {
    RingArgs a{};
    TL_PROPAGATE(build_ring_args(q, &a));
    const bool norm = q.norm_w != nullptr;
#define TL_FUSED(E) (norm ? launch_ring<E, true>(a, st, q.pdl) : launch_ring<E, false>(a, st, q.pdl))
    switch (q.epilogue) {
        case EPI_STORE: return TL_FUSED(EPI_STORE);
        case EPI_STORE_F32: return TL_FUSED(EPI_STORE_F32);
        case EPI_PUSH_F32: return TL_FUSED(EPI_PUSH_F32);
        case EPI_PUSH_F16: return TL_FUSED(EPI_PUSH_F16);
        case EPI_RESIDUAL: return TL_FUSED(EPI_RESIDUAL);
        case EPI_QKV_ROPE: return TL_FUSED(EPI_QKV_ROPE);
        case EPI_SWIGLU: return TL_FUSED(EPI_SWIGLU);
        default: return set_error(TL_ERR_INVALID_ARGUMENT, "fused gemv: unknown epilogue %d", q.epilogue);
    }
#undef TL_FUSED
}

// Phase A: a K-split matmul pushing fp32 partial sums (EPI_PUSH_F32, no norm); phase B: the matmul
// fed by that exchange (xin set, RMSNorm prologue) with one of the three epilogues that follow an
// exchange in the decode step.
int launch_fused_gemv_pair(const FusedGemv& qa, const FusedGemv& qb, cudaStream_t st) {
    TL_REQUIRE(qa.epilogue == EPI_PUSH_F32 && !qa.norm_w && !qa.xin && qb.xin && qb.norm_w,
               "fused gemv pair: phase A pushes partial sums, phase B consumes an exchange behind an RMSNorm");
    RingArgs a{}, b{};
    TL_PROPAGATE(build_ring_args(qa, &a));
    TL_PROPAGATE(build_ring_args(qb, &b));
    switch (qb.epilogue) {
        case EPI_SWIGLU: return launch_ring2<EPI_SWIGLU>(a, b, st, qa.pdl);
        case EPI_QKV_ROPE: return launch_ring2<EPI_QKV_ROPE>(a, b, st, qa.pdl);
        case EPI_PUSH_F16: return launch_ring2<EPI_PUSH_F16>(a, b, st, qa.pdl);
        default: return set_error(TL_ERR_INVALID_ARGUMENT, "fused gemv pair: phase B epilogue %d is not one that follows an exchange", qb.epilogue);
    }
}

}  // namespace tlb
