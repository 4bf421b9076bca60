// One decode step of the Llama2 forward as ONE persistent kernel (fast numerics, batch 1).
//
// Replaces, per token, the reference's ~2.8 k launches (model/llama2_7b/src/Transformer.cpp:264-299
// and everything it calls) and this library's own 164-launch graph. One CTA per SM stays resident
// for the whole token and walks a list of phases:
//     per layer:  [RMSNorm + wq|wk|wv GEMV + RoPE + KV write] | [attention] | [wo GEMV + residual] |
//                 [RMSNorm + w1|w3 GEMV + SiLU*up] | [w2 GEMV + residual]
//     then        [RMSNorm + classifier GEMV] | argmax + position bookkeeping (CTA 0)
// separated by grid-wide barriers. The point of fusing the phases is the weight stream: the
// producer warp of every CTA pushes the weight rows of ALL phases, in order, through the
// shared-memory ring with TMA bulk copies and never waits for a barrier (weights do not depend on
// activations); it only waits for ring slots. While the consumers sit in a barrier or compute
// attention, the ring (190 KB per SM, 28 MB per GPU) fills with the next phase's weights, so HBM
// does not idle at phase boundaries the way it does at kernel boundaries.
//
// Consumers: 16 warps. In a GEMV phase each owns one unit (two weight rows) of a stage; in the
// attention phase they form 4 groups of 4 warps, each group working on one (head, split) item.
// Activations exchanged between CTAs are read with ld.global.cg (L2) because L1 is not coherent
// across SMs within a kernel. Every wait (mbarrier, grid barrier) is bounded and reports
// TL_ERR_TIMEOUT through the device status word instead of hanging.
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

enum { PH_GEMV = 0, PH_ATTN = 1 };

}  // namespace

namespace {

template <int EPI>
__device__ __forceinline__ void unit_rows(const MegaPhase& p, int unit, const __half*& ra, const __half*& rb,
                                          int& mat, int& r) {
    if (EPI == EPI_SWIGLU) {
        mat = 0; r = unit;
        ra = p.W0 + (long long)unit * p.K;
        rb = p.W1 + (long long)unit * p.K;
    } else {
        int row = unit * 2;
        mat = row / p.N_each;
        r = row - mat * p.N_each;
        const __half* Wm = mat == 0 ? p.W0 : (mat == 1 ? p.W1 : p.W2);
        ra = Wm + (long long)r * p.K;
        rb = ra + p.K;
    }
}
__device__ __forceinline__ void unit_rows_rt(const MegaPhase& p, int unit, const __half*& ra, const __half*& rb) {
    int mat, r;
    if (p.epilogue == EPI_SWIGLU) unit_rows<EPI_SWIGLU>(p, unit, ra, rb, mat, r);
    else unit_rows<EPI_STORE>(p, unit, ra, rb, mat, r);
}

struct Ctx {
    unsigned char* stages; uint4* xs; float* red; float* partials; uint32_t full0, empty0;
    int warp, lane, ctid, tile_parity;
    int tok, pos;
    float rinv;            // 1/rms of the current phase's input (1 when the phase has no RMSNorm)
    int it;                // ring iteration counter of this role
    unsigned int bar_target;
    bool ok;
};

// Grid-wide barrier among the consumer warps of all CTAs (the producers never join it).
__device__ __forceinline__ void grid_barrier(const MegaArgs& a, Ctx& c) {
    // bar.sync orders every consumer thread's stores before thread 0's release-add (cumulative at
    // gpu scope); the acquire-load that sees the last arrival orders the other CTAs' stores before
    // everything after the second bar.sync. No return value is needed from the add, so it is a
    // fire-and-forget reduction rather than an atomic round trip.
    named_bar_sync(1, CONSUMER_THREADS);
    if (c.ctid == 0) {
        c.bar_target += gridDim.x;
        asm volatile("red.release.gpu.global.add.u32 [%0], 1;" ::"l"(a.grid_bar) : "memory");
        bool done = false;
        for (uint32_t i = 0; i < (1u << 24); i++)
            if (ld_acquire_u32(a.grid_bar) >= c.bar_target) { done = true; break; }
        if (!done) atomicExch(a.status, TL_ERR_TIMEOUT);
    }
    named_bar_sync(1, CONSUMER_THREADS);
}

// stage the activation vector of a GEMV phase in shared memory (optionally RMS-normalised)
__device__ __forceinline__ void stage_x(const MegaArgs& a, const MegaPhase& p, Ctx& c) {
    const int K8 = p.K >> 3;
    const __half* xsrc = p.x ? p.x : a.emb + (long long)c.tok * a.dim;
    const uint4* x4 = reinterpret_cast<const uint4*>(xsrc);
    if (p.norm_w) {
        // RMSNorm in one pass: the vector staged is x * w (fp16); the scalar 1/rms is applied to
        // the finished dot products instead (sum_k rinv*x_k*w_k*W_nk = rinv * sum_k (x_k*w_k)*W_nk),
        // so no second pass over x has to wait for the reduction.
        float ss = 0.f;
        const uint4* nw4 = reinterpret_cast<const uint4*>(p.norm_w);
        for (int i = c.ctid; i < K8; i += CONSUMER_THREADS) {
            uint4 v = __ldcg(x4 + i), g = nw4[i];
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
        c.rinv = rsqrtf(tot / (float)p.K + a.eps);
    } else {
        for (int i = c.ctid; i < K8; i += CONSUMER_THREADS) c.xs[i] = __ldcg(x4 + i);
        c.rinv = 1.0f;
        named_bar_sync(1, CONSUMER_THREADS);
    }
}

template <int EPI>
__device__ __forceinline__ void gemv_consume(const MegaArgs& a, const MegaPhase& p, Ctx& c) {
    const int u_begin = (int)((long long)p.total_units * blockIdx.x / gridDim.x);
    const int u_end = (int)((long long)p.total_units * (blockIdx.x + 1) / gridDim.x);
    const int n_units = u_end - u_begin;
    const int n_tiles = (n_units + CONSUMERS - 1) / CONSUMERS;
    const int nk = (p.K + KC - 1) / KC;
    // Tensor-core dot products (mma.sync m16n8k16, fp32 accumulate): the 32 rows of a stage are two
    // m16 tiles, the activation vector is column 0 of B; warp w multiplies k16 steps
    // [w*STEPS_PER_WARP, +STEPS_PER_WARP) of every chunk for all rows; the per-warp partial row
    // sums meet in shared memory at the end of a tile and warp 0 finishes the rows.
    const int lane = c.lane, g = lane >> 2, t = lane & 3;
    const uint32_t lm_off = (uint32_t)(((lane & 7) + ((lane >> 3) & 1) * 8) * ROW_STRIDE + (lane >> 4) * 16);
    const __half* xh = reinterpret_cast<const __half*>(c.xs);
    for (int tile = 0; tile < n_tiles && c.ok; tile++) {
        const int units_here = min(CONSUMERS, n_units - tile * CONSUMERS);
        float acc0[4] = {0.f, 0.f, 0.f, 0.f}, acc1[4] = {0.f, 0.f, 0.f, 0.f};
        // warp 0 finishes the rows of this tile: fetch what its epilogue needs from L2 now, so the
        // latency overlaps the multiply instead of following it
        __half res_a = __float2half_rn(0.f), res_b = res_a;
        if (EPI == EPI_RESIDUAL && c.warp == 0 && !(lane & 1) && (lane >> 1) < units_here) {
            const __half *ra, *rb; int mat, r;
            unit_rows<EPI>(p, u_begin + tile * CONSUMERS + (lane >> 1), ra, rb, mat, r);
            const __half* res = p.residual ? p.residual : a.emb + (long long)c.tok * a.dim;
            res_a = ldcg_half(res + r);
            res_b = ldcg_half(res + r + 1);
        }
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
        const float sa = rowsum * c.rinv, sb = other * c.rinv;
        const __half ha = __float2half_rn(sa), hb = __float2half_rn(sb);
        const __half *ra, *rb; int mat, r;
        unit_rows<EPI>(p, u_begin + tile * CONSUMERS + (lane >> 1), ra, rb, mat, r);
        if (EPI == EPI_STORE) {
            p.y[(long long)mat * p.N_each + r] = ha;
            p.y[(long long)mat * p.N_each + r + 1] = hb;
        } else if (EPI == EPI_STORE_F32) {
            p.y32[(long long)mat * p.N_each + r] = sa;
            p.y32[(long long)mat * p.N_each + r + 1] = sb;
        } else if (EPI == EPI_RESIDUAL) {
            p.y[r] = hadd_ref(res_a, ha);
            p.y[r + 1] = hadd_ref(res_b, hb);
        } else if (EPI == EPI_QKV_ROPE) {
            if (mat == 2) {
                __half* vo = p.v_cache + (long long)c.pos * a.kv_pitch;
                vo[r] = ha; vo[r + 1] = hb;
            } else {
                const int half_dim = a.hd >> 1;
                const int d2 = (r % a.hd) >> 1;
                const __half cs = a.cos_t[(long long)c.pos * half_dim + d2];
                const __half sn = a.sin_t[(long long)c.pos * half_dim + d2];
                const __half o0 = hsub_ref(hmul_ref(ha, cs), hmul_ref(hb, sn));
                const __half o1 = hadd_ref(hmul_ref(ha, sn), hmul_ref(hb, cs));
                __half* dst = mat == 0 ? p.y : p.k_cache + (long long)c.pos * a.kv_pitch;
                dst[r] = o0; dst[r + 1] = o1;
            }
        } else {  // EPI_SWIGLU
            const __half g = a.silu_tab[__half_as_ushort(ha)];
            p.y[r] = hmul_ref(g, hb);
        }
    }
}

// Attention of the new token over positions [0, pos] of the caches, read in place. Work items are
// (head, split) pairs; a group of 4 warps takes one item at a time; partial (max, sum, acc) go to
// a scratch slot; the last group to finish a head merges its splits.
__device__ __forceinline__ void attn_phase(const MegaArgs& a, const MegaPhase& p, Ctx& c) {
    const int g = c.warp / ATT_WARPS, gw = c.warp % ATT_WARPS, lane = c.lane;
    float* gs = reinterpret_cast<float*>(c.xs) + (size_t)g * (ATT_SMEM_PER_GROUP / 4);
    float* sm_m = gs; float* sm_l = gs + ATT_WARPS; float* sm_acc = gs + 2 * ATT_WARPS;
    int* is_last = reinterpret_cast<int*>(gs + 2 * ATT_WARPS + ATT_WARPS * MAX_HD);
    const int hd = a.hd, S = c.pos + 1;
    const int per = (S + a.splits - 1) / a.splits;
    const float scale = rsqrtf((float)hd);
    const int n_items = a.H * a.splits;
    const int gtid = gw * 32 + lane;
    for (int item = blockIdx.x * ATT_GROUPS + g; item < n_items; item += gridDim.x * ATT_GROUPS) {
        const int h = item / a.splits, split = item - h * a.splits;
        const int s_begin = split * per, s_end = min(S, s_begin + per);
        float2 qf[HD_ITERS];
#pragma unroll
        for (int i = 0; i < HD_ITERS; i++) {
            int d = 2 * lane + 64 * i;
            if (d < hd) {
                unsigned int raw = __ldcg(reinterpret_cast<const unsigned int*>(p.x + (size_t)h * hd + d));
                qf[i] = __half22float2(*reinterpret_cast<__half2*>(&raw));
            } else qf[i] = make_float2(0.f, 0.f);
        }
        float m = -INFINITY, l = 0.f;
        float2 acc[HD_ITERS];
#pragma unroll
        for (int i = 0; i < HD_ITERS; i++) acc[i] = make_float2(0.f, 0.f);
        constexpr int U = 4;
        for (int s0 = s_begin + gw * U; s0 < s_end; s0 += ATT_WARPS * U) {
            unsigned int kv[U][HD_ITERS], vv[U][HD_ITERS];
#pragma unroll
            for (int u = 0; u < U; u++) {
                const int s = s0 + u;
                const size_t base = (size_t)s * a.kv_pitch + (size_t)h * hd;
#pragma unroll
                for (int i = 0; i < HD_ITERS; i++) {
                    int d = 2 * lane + 64 * i;
                    bool okk = s < s_end && d < hd;
                    kv[u][i] = okk ? __ldcg(reinterpret_cast<const unsigned int*>(p.k_cache + base + d)) : 0u;
                    vv[u][i] = okk ? __ldcg(reinterpret_cast<const unsigned int*>(p.v_cache + base + d)) : 0u;
                }
            }
            float sc[U];
#pragma unroll
            for (int u = 0; u < U; u++) {
                float d = 0.f;
#pragma unroll
                for (int i = 0; i < HD_ITERS; i++) {
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
                    l = l * corr + pe;
#pragma unroll
                    for (int i = 0; i < HD_ITERS; i++) {
                        float2 vf = __half22float2(*reinterpret_cast<__half2*>(&vv[u][i]));
                        acc[i].x = fmaf(pe, vf.x, acc[i].x * corr);
                        acc[i].y = fmaf(pe, vf.y, acc[i].y * corr);
                    }
                    m = mn;
                }
            }
        }
        if (lane == 0) { sm_m[gw] = m; sm_l[gw] = l; }
#pragma unroll
        for (int i = 0; i < HD_ITERS; i++) {
            int d = 2 * lane + 64 * i;
            if (d < hd) { sm_acc[gw * MAX_HD + d] = acc[i].x; sm_acc[gw * MAX_HD + d + 1] = acc[i].y; }
        }
        named_bar_sync(2 + g, ATT_WARPS * 32);
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < ATT_WARPS; w++) M = fmaxf(M, sm_m[w]);
        float L = 0.f;
#pragma unroll
        for (int w = 0; w < ATT_WARPS; w++) L += sm_m[w] == -INFINITY ? 0.f : sm_l[w] * __expf(sm_m[w] - M);
        float* slot = a.attn_scratch + ((size_t)h * a.splits + split) * (hd + 2);
        for (int d = gtid; d < hd; d += ATT_WARPS * 32) {
            float v = 0.f;
#pragma unroll
            for (int w = 0; w < ATT_WARPS; w++)
                v += sm_m[w] == -INFINITY ? 0.f : sm_acc[w * MAX_HD + d] * __expf(sm_m[w] - M);
            slot[2 + d] = v;
        }
        if (gtid == 0) { slot[0] = M; slot[1] = L; }
        __threadfence();
        named_bar_sync(2 + g, ATT_WARPS * 32);
        if (gtid == 0) {
            unsigned int prev = atomicAdd(&a.attn_counters[h], 1u);
            *is_last = prev == (unsigned)a.splits - 1;
            if (*is_last) a.attn_counters[h] = 0;
        }
        named_bar_sync(2 + g, ATT_WARPS * 32);
        if (*is_last) {
            __threadfence();
            const float* base = a.attn_scratch + (size_t)h * a.splits * (hd + 2);
            float GM = -INFINITY;
            for (int sp = 0; sp < a.splits; sp++) GM = fmaxf(GM, __ldcg(base + (size_t)sp * (hd + 2)));
            float GL = 0.f;
            for (int sp = 0; sp < a.splits; sp++) {
                float ms = __ldcg(base + (size_t)sp * (hd + 2));
                if (ms != -INFINITY) GL += __ldcg(base + (size_t)sp * (hd + 2) + 1) * __expf(ms - GM);
            }
            for (int d = gtid; d < hd; d += ATT_WARPS * 32) {
                float v = 0.f;
                for (int sp = 0; sp < a.splits; sp++) {
                    float ms = __ldcg(base + (size_t)sp * (hd + 2));
                    if (ms != -INFINITY) v += __ldcg(base + (size_t)sp * (hd + 2) + 2 + d) * __expf(ms - GM);
                }
                p.y[(size_t)h * hd + d] = __float2half_rn(v / GL);
            }
        }
        named_bar_sync(2 + g, ATT_WARPS * 32);  // the group's shared scratch is reused by its next item
    }
}

__global__ void __launch_bounds__(MEGA_THREADS, 1) k_decode_mega(MegaArgs a) {
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
    c.it = 0; c.bar_target = 0; c.ok = true;

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
        // (An L2 prefetch running ahead of the ring with cp.async.bulk.prefetch.L2 was measured and
        // dropped: phase times grew by ~50 %, the extra bulk requests compete with the ring's own.)
        for (int ph = 0; ph < a.n_phases && ok; ph++) {
            const MegaPhase& p = a.phases[ph];
            if (p.kind != PH_GEMV) continue;
            const int u_begin = (int)((long long)p.total_units * blockIdx.x / gridDim.x);
            const int u_end = (int)((long long)p.total_units * (blockIdx.x + 1) / gridDim.x);
            const int n_units = u_end - u_begin;
            const int n_tiles = (n_units + CONSUMERS - 1) / CONSUMERS;
            const int nk = (p.K + KC - 1) / KC;
            for (int tile = 0; tile < n_tiles && ok; tile++) {
                const int rows_in_tile = min(CONSUMERS, n_units - tile * CONSUMERS) * 2;
                const __half* row_ptr = nullptr;
                if (lane < rows_in_tile) {
                    const __half *ra, *rb;
                    unit_rows_rt(p, u_begin + tile * CONSUMERS + (lane >> 1), ra, rb);
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
    if (c.tok < 0 || c.tok >= a.vocab) c.tok = 0;
    // optional per-phase timestamps (ns) of one CTA: [phase][0] work start (barrier passed),
    // [1] activation vector staged, [2] phase work done
    const bool prof = a.prof != nullptr && blockIdx.x == a.prof_cta && c.ctid == 0;
    auto now = []() { unsigned long long t; asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t)); return t; };
    for (int ph = 0; ph < a.n_phases; ph++) {
        const MegaPhase& p = a.phases[ph];
        if (ph > 0) grid_barrier(a, c);
        if (prof) a.prof[3 * ph] = now();
        if (p.kind == PH_ATTN) {
            attn_phase(a, p, c);
            if (prof) a.prof[3 * ph + 1] = a.prof[3 * ph + 2] = now();
            continue;
        }
        stage_x(a, p, c);
        if (prof) a.prof[3 * ph + 1] = now();
        switch (p.epilogue) {
            case EPI_STORE: gemv_consume<EPI_STORE>(a, p, c); break;
            case EPI_STORE_F32: gemv_consume<EPI_STORE_F32>(a, p, c); break;
            case EPI_RESIDUAL: gemv_consume<EPI_RESIDUAL>(a, p, c); break;
            case EPI_QKV_ROPE: gemv_consume<EPI_QKV_ROPE>(a, p, c); break;
            default: gemv_consume<EPI_SWIGLU>(a, p, c); break;
        }
        if (prof) a.prof[3 * ph + 2] = now();
    }
    if (!c.ok && c.lane == 0) atomicExch(a.status, TL_ERR_TIMEOUT);
    grid_barrier(a, c);
    if (blockIdx.x != 0) return;
    // greedy sampling (lowest index wins ties, CPU.cpp:358-372) and position bookkeeping by CTA 0
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    for (int j = c.ctid; j < a.vocab; j += CONSUMER_THREADS) {
        float v = __half2float(ldcg_half(a.logits + j));
        if (bi == 0x7fffffff || v > bv) { bv = v; bi = j; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
    }
    float* sv = c.red;
    int* si = reinterpret_cast<int*>(c.xs);
    if (c.lane == 0) { sv[c.warp] = bv; si[c.warp] = bi; }
    named_bar_sync(1, CONSUMER_THREADS);
    if (c.ctid == 0) {
        for (int w = 1; w < CONSUMERS; w++)
            if (sv[w] > bv || (sv[w] == bv && si[w] < bi)) { bv = sv[w]; bi = si[w]; }
        if (bi == 0x7fffffff) bi = 0;
        *a.d_next = bi;
        if (c.pos >= 0 && c.pos < a.max_seq) a.d_generated[c.pos] = bi;
        *a.d_pos = c.pos + 1;
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

int launch_decode_mega(const MegaArgs& args, int grid, int smem, cudaStream_t st) {
    static PerDeviceOnce once;
    if (once.needed()) {
        TL_CUDA(cudaFuncSetAttribute(k_decode_mega, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
    }
    TL_CUDA(cudaMemsetAsync(args.grid_bar, 0, sizeof(unsigned int), st));
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
    TL_CUDA(cudaLaunchKernelEx(&cfg, k_decode_mega, args));
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
