// Skinny matmul for sm_100a: C[M,N] = A[M,K] * W[N,K]^T with 2 <= M <= 128 (decode batches, short
// prompts, the M = 8 / 32 / 128 points of the matmul sweep). Same entry point as the other matmul
// kernels (Device::matmul2d, tensorLib/include/device/Device.hpp:22); replaces the reference's loop
// of one GEMV launch per row (tensorLib/src/ops/matmul.cpp:297-320 -> gemv_v6).
//
// Bound by HBM: 2*N*K weight bytes must be streamed once, the activations fit in L2. So the
// operands are swapped: the 128-row side of the tcgen05 MMA is a block of W rows, its N side is
// the (zero-padded) batch of activation rows, and the fp32 accumulator in TMEM is a 128 x NB tile
// of C^T. Work is split stream-K fashion: the (W-row tile, k-block) space is cut into equal
// contiguous ranges, one per SM, so every SM streams the same number of weight bytes whatever
// N and K are. A tile whose k-range is shared by several CTAs is finished by the LAST CTA to
// arrive (atomic counter per tile): every sharer leaves its fp32 partial in a workspace slot,
// the last one adds the slots in CTA order, a fixed order, so results do not depend on timing,
// and nobody ever waits for another CTA.
//
// Roles as in the HGEMM: warp 0 TMA producer (8-10 stages of 16 KB of W + NB*128 B of A, tiled
// TMA, 128-byte swizzle, zero fill past M / K), warp 1 tcgen05.mma issuer, warp 2 TMEM
// allocation, warps 4-7 epilogue. Every mbarrier wait is bounded (TL_ERR_TIMEOUT in the device
// status word).
#include <cuda.h>

#include <cstdlib>
#include <mutex>
#include <unordered_map>

#include "kernels.cuh"
#include "sm100.cuh"

namespace tlb {

namespace {

using namespace sm100;

constexpr int TW = 128, BK = 64;           // W rows per tile, k-block
constexpr int SK_THREADS = 256;
constexpr int W_BYTES = TW * BK * 2;

struct SkinnyArgs {
    __half* C;
    long long ldc;
    int M, N, K;
    int tiles, nkb, per;        // W-row tiles, k-blocks per tile, k-blocks per CTA
    int per_cluster;            // cluster variant: CTAs (k-splits) per tile
    float* ws;                  // [2 * grid][NB][TW] fp32 partial tiles
    unsigned int* counters;     // [tiles], zero between launches
    int* status;
    int w_const;                // W is a parameter nobody in flight writes: its copies may start before the previous kernel ends
};

template <int NB> struct SkinnyCfg {
    static constexpr int STAGES = NB <= 32 ? 10 : (NB <= 64 ? 8 : 6);
    static constexpr int STAGE_BYTES = W_BYTES + NB * BK * 2;
    static constexpr uint32_t TMEM_COLS = 2 * NB < 32 ? 32 : 2 * NB;
    static constexpr size_t SMEM = (size_t)STAGES * STAGE_BYTES + 1024 + 512;
};

template <int NB>
__global__ void __launch_bounds__(SK_THREADS, 1)
k_skinny(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmX, SkinnyArgs p) {
    using Cfg = SkinnyCfg<NB>;
    constexpr int STAGES = Cfg::STAGES, STAGE_BYTES = Cfg::STAGE_BYTES;
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES);
    const uint32_t full0 = smem_u32(bars), empty0 = smem_u32(bars + STAGES);
    const uint32_t tfull0 = smem_u32(bars + 2 * STAGES), tempty0 = smem_u32(bars + 2 * STAGES + 2);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    volatile int* last_flag = reinterpret_cast<volatile int*>(tmem_slot + 2);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long total = (long long)p.tiles * p.nkb;
    const long long g_begin = (long long)blockIdx.x * p.per;
    const long long g_end = g_begin + p.per < total ? g_begin + p.per : total;   // may be <= g_begin: nothing to do

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; s++) { mbar_init(full0 + 8 * s, 1); mbar_init(empty0 + 8 * s, 1); }
        for (int b = 0; b < 2; b++) { mbar_init(tfull0 + 8 * b, 1); mbar_init(tempty0 + 8 * b, 4); }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 2) tmem_alloc<Cfg::TMEM_COLS>(tmem_slot);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    // set-up done (barriers, TMEM): let the next kernel of the stream start its own set-up, then wait
    // for the previous one before any operand is read or any result written
    pdl_launch_dependents();
    const bool producer = warp == 0 && lane == 0;
    int w_ahead = 0;       // stages whose weight half is already on its way (constant weights only)
    if (producer && p.w_const) {
        // the weight halves of the first ring-full of stages do not depend on the previous kernel
        asm volatile("prefetch.tensormap [%0];" ::"l"(&tmW) : "memory");
        for (long long g = g_begin; g < g_end && w_ahead < STAGES; g++, w_ahead++) {
            const int t = (int)(g / p.nkb), kb = (int)(g - (long long)t * p.nkb);
            mbar_arrive_expect_tx(full0 + 8 * w_ahead, STAGE_BYTES);
            tma_load_3d(smem_u32(smem + w_ahead * STAGE_BYTES), &tmW, kb * BK, t * TW, 0, full0 + 8 * w_ahead);
        }
    }
    pdl_wait();

    if (producer) {
        // ---------------- TMA producer ---------------------------------------------------------
        asm volatile("prefetch.tensormap [%0];" ::"l"(&tmW) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&tmX) : "memory");
        int it = 0;
        bool ok = true;
        for (long long g = g_begin; g < g_end && ok; g++, it++) {
            const int t = (int)(g / p.nkb), kb = (int)(g - (long long)t * p.nkb);
            const int s = it % STAGES, use = it / STAGES;
            if (use > 0 && !(ok = mbar_wait(empty0 + 8 * s, (use - 1) & 1, abort_flag))) break;
            const uint32_t sw = smem_u32(smem + s * STAGE_BYTES), sx = sw + W_BYTES;
            if (it >= w_ahead) {
                mbar_arrive_expect_tx(full0 + 8 * s, STAGE_BYTES);
                tma_load_3d(sw, &tmW, kb * BK, t * TW, 0, full0 + 8 * s);
            }
            tma_load_3d(sx, &tmX, kb * BK, 0, 0, full0 + 8 * s);
        }
        if (!ok) {  // let copies already in flight land before the CTA goes away
            for (int j = max(0, it - STAGES); j < it; j++)
                for (uint32_t i = 0; i < (1u << 16); i++)
                    if (mbar_try_wait(full0 + 8 * (j % STAGES), (j / STAGES) & 1)) break;
        }
    } else if (warp == 1 && lane == 0) {
        // ---------------- MMA issuer: D[W row, token] += W[rows, k] * A[tokens, k]^T ----------------
        constexpr uint32_t idesc = make_idesc(NB);
        int it = 0, seg = 0;
        bool ok = true;
        long long g = g_begin;
        while (g < g_end && ok) {
            const int t = (int)(g / p.nkb), kb0 = (int)(g - (long long)t * p.nkb);
            const int len = (int)min((long long)(p.nkb - kb0), g_end - g);
            const int buf = seg & 1, use = seg >> 1;
            if (use > 0 && !(ok = mbar_wait(tempty0 + 8 * buf, (use - 1) & 1, abort_flag))) break;
            tc_fence_after();
            const uint32_t d_tmem = tmem_base + (uint32_t)(buf * NB);
            for (int i = 0; i < len; i++, it++) {
                const int s = it % STAGES, use_s = it / STAGES;
                if (!(ok = mbar_wait(full0 + 8 * s, use_s & 1, abort_flag))) break;
                tc_fence_after();
                const uint32_t sw = smem_u32(smem + s * STAGE_BYTES), sx = sw + W_BYTES;
#pragma unroll
                for (int k = 0; k < BK / 16; k++)
                    umma(d_tmem, make_desc(sw + k * 32), make_desc(sx + k * 32), idesc, (i > 0 || k > 0) ? 1u : 0u);
                umma_commit(empty0 + 8 * s);
            }
            if (ok) umma_commit(tfull0 + 8 * buf);
            g += len;
            seg++;
        }
    } else if (warp >= 4) {
        // ---------------- epilogue ---------------------------------------------------------------------
        const int q = warp & 3;
        const int r = q * 32 + lane;                 // W row inside the tile = TMEM lane
        int seg = 0;
        bool ok = true;
        long long g = g_begin;
        while (g < g_end) {
            const int t = (int)(g / p.nkb), kb0 = (int)(g - (long long)t * p.nkb);
            const int len = (int)min((long long)(p.nkb - kb0), g_end - g);
            const bool whole = kb0 == 0 && len == p.nkb;
            const int buf = seg & 1, use = seg >> 1;
            ok = mbar_wait(tfull0 + 8 * buf, use & 1, abort_flag);
            {   // one decision for all four epilogue warps (they share named barrier 1 below): this
                // reducing barrier is reached by every epilogue thread because the wait above is bounded
                uint32_t all_ok;
                asm volatile("{\n .reg .pred p, q;\n setp.ne.u32 q, %1, 0;\n bar.red.and.pred p, 1, 128, q;\n selp.u32 %0, 1, 0, p;\n}\n"
                             : "=r"(all_ok) : "r"((uint32_t)ok) : "memory");
                ok = all_ok != 0;
            }
            if (!ok) break;
            tc_fence_after();
            const int n = t * TW + r;
            const uint32_t tbase = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(buf * NB);
            const int slot = kb0 > 0 ? 2 * (int)blockIdx.x : 2 * (int)blockIdx.x + 1;
            float* wrow = p.ws + (size_t)slot * NB * TW + r;
#pragma unroll 1
            for (int c = 0; c < NB; c += 32) {
                uint32_t v[32];
                tmem_ld32(tbase + (uint32_t)c, v);
                tmem_ld_wait();
                if (whole) {
                    if (n < p.N) {
#pragma unroll
                        for (int j = 0; j < 32; j++)
                            if (c + j < p.M) p.C[(long long)(c + j) * p.ldc + n] = __float2half_rn(__uint_as_float(v[j]));
                    }
                } else {
#pragma unroll
                    for (int j = 0; j < 32; j++)
                        if (c + j < p.M) wrow[(size_t)(c + j) * TW] = __uint_as_float(v[j]);
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(tempty0 + 8 * buf);     // the accumulator may be overwritten
            if (!whole) {
                // publish the partial, count arrivals; the last sharer of the tile adds all partials
                __threadfence();
                asm volatile("bar.sync 1, 128;" ::: "memory");
                const int first = (int)(((long long)t * p.nkb) / p.per);
                const int last = (int)((((long long)(t + 1)) * p.nkb - 1) / p.per);
                if (r == 0) {
                    const unsigned int old = atomicAdd(p.counters + t, 1u);
                    const int is_last = old == (unsigned)(last - first) ? 1 : 0;
                    if (is_last) p.counters[t] = 0;            // ready for the next launch
                    *last_flag = is_last;
                }
                asm volatile("bar.sync 1, 128;" ::: "memory");
                const bool is_last = *last_flag != 0;
                asm volatile("bar.sync 1, 128;" ::: "memory");  // flag read by all before the next segment rewrites it
                if (is_last) {
                    __threadfence();
                    if (n < p.N) {
                        // 32 token columns at a time, two sharers per trip: 64 independent L2 loads in
                        // flight per thread (the stores could alias them as far as the compiler knows,
                        // so they come after the group's loads)
                        const float* __restrict__ wsr = p.ws;
                        auto slot_of = [&](int c) { return ((long long)c * p.per > (long long)t * p.nkb) ? 2 * c : 2 * c + 1; };
                        for (int m0 = 0; m0 < p.M; m0 += 32) {
                            float acc[32];
#pragma unroll
                            for (int i = 0; i < 32; i++) acc[i] = 0.f;
                            for (int c = first; c <= last; c += 2) {
                                const float* s0 = wsr + ((size_t)slot_of(c) * NB + m0) * TW + r;
                                const bool two = c + 1 <= last;
                                const float* s1 = wsr + ((size_t)slot_of(two ? c + 1 : c) * NB + m0) * TW + r;
                                float v0[32], v1[32];
#pragma unroll
                                for (int i = 0; i < 32; i++) v0[i] = (m0 + i < p.M) ? __ldcg(s0 + (size_t)i * TW) : 0.f;
#pragma unroll
                                for (int i = 0; i < 32; i++) v1[i] = (two && m0 + i < p.M) ? __ldcg(s1 + (size_t)i * TW) : 0.f;
#pragma unroll
                                for (int i = 0; i < 32; i++) acc[i] = (acc[i] + v0[i]) + v1[i];   // CTA order
                            }
#pragma unroll
                            for (int i = 0; i < 32; i++)
                                if (m0 + i < p.M) p.C[(long long)(m0 + i) * p.ldc + n] = __float2half_rn(acc[i]);
                        }
                    }
                }
            }
            g += len;
            seg++;
        }
    }
    // ---------------- teardown ---------------------------------------------------------------------
    tc_fence_before();
    __syncthreads();
    if (warp == 2) {
        tc_fence_after();
        tmem_dealloc<Cfg::TMEM_COLS>(tmem_base);
    }
    if (threadIdx.x == 0 && *abort_flag) atomicExch(p.status, TL_ERR_TIMEOUT);
}

// ---- cluster variant: the sharers of a W tile are one thread-block cluster -------------------------
// When a whole number of CTAs per tile fills the GPU (few W tiles, e.g. N = 4096), the k-range of a
// tile is split evenly over the `splits` CTAs of a cluster. Each leaves its fp32 partial tile in
// its own shared memory (the drained operand ring); after one cluster barrier every CTA adds up
// its share of the token columns from all sharers over distributed shared memory, in rank order,
// and writes fp16. No workspace, no atomics, no global-memory round trip, and the reduction is
// spread over all sharers instead of falling on the last one to arrive.
template <int NB>
__global__ void __launch_bounds__(SK_THREADS, 1)
k_skinny_cluster(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmX, SkinnyArgs p) {
    using Cfg = SkinnyCfg<NB>;
    constexpr int STAGES = Cfg::STAGES, STAGE_BYTES = Cfg::STAGE_BYTES;
    constexpr uint32_t TMEM_COLS = NB < 32 ? 32 : NB;
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES);
    const uint32_t full0 = smem_u32(bars), empty0 = smem_u32(bars + STAGES);
    const uint32_t tfull = smem_u32(bars + 2 * STAGES);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    float* part = reinterpret_cast<float*>(smem);       // [NB][TW] once the ring has drained

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int splits = p.per_cluster;                    // cluster size = sharers per tile
    const int rank = (int)cluster_ctarank();
    const int t = (int)blockIdx.x / splits;
    const int kb0 = min(p.nkb, rank * p.per), kb1 = min(p.nkb, kb0 + p.per), len = kb1 - kb0;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; s++) { mbar_init(full0 + 8 * s, 1); mbar_init(empty0 + 8 * s, 1); }
        mbar_init(tfull, 1);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 2) tmem_alloc<TMEM_COLS>(tmem_slot);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    pdl_launch_dependents();
    const bool producer = warp == 0 && lane == 0;
    int w_ahead = 0;       // stages whose weight half is already on its way (constant weights only)
    if (producer && p.w_const) {
        asm volatile("prefetch.tensormap [%0];" ::"l"(&tmW) : "memory");
        for (int kb = kb0; kb < kb1 && w_ahead < STAGES; kb++, w_ahead++) {
            mbar_arrive_expect_tx(full0 + 8 * w_ahead, STAGE_BYTES);
            tma_load_3d(smem_u32(smem + w_ahead * STAGE_BYTES), &tmW, kb * BK, t * TW, 0, full0 + 8 * w_ahead);
        }
    }
    pdl_wait();

    if (producer) {
        asm volatile("prefetch.tensormap [%0];" ::"l"(&tmW) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&tmX) : "memory");
        bool ok = true;
        int it = 0;
        for (int kb = kb0; kb < kb1 && ok; kb++, it++) {
            const int s = it % STAGES, use = it / STAGES;
            if (use > 0 && !(ok = mbar_wait(empty0 + 8 * s, (use - 1) & 1, abort_flag))) break;
            const uint32_t sw = smem_u32(smem + s * STAGE_BYTES), sx = sw + W_BYTES;
            if (it >= w_ahead) {
                mbar_arrive_expect_tx(full0 + 8 * s, STAGE_BYTES);
                tma_load_3d(sw, &tmW, kb * BK, t * TW, 0, full0 + 8 * s);
            }
            tma_load_3d(sx, &tmX, kb * BK, 0, 0, full0 + 8 * s);
        }
        if (!ok) {
            for (int j = max(0, it - STAGES); j < it; j++)
                for (uint32_t i = 0; i < (1u << 16); i++)
                    if (mbar_try_wait(full0 + 8 * (j % STAGES), (j / STAGES) & 1)) break;
        }
    } else if (warp == 1 && lane == 0) {
        constexpr uint32_t idesc = make_idesc(NB);
        bool ok = true;
        for (int i = 0; i < len && ok; i++) {
            const int s = i % STAGES, use_s = i / STAGES;
            if (!(ok = mbar_wait(full0 + 8 * s, use_s & 1, abort_flag))) break;
            tc_fence_after();
            const uint32_t sw = smem_u32(smem + s * STAGE_BYTES), sx = sw + W_BYTES;
#pragma unroll
            for (int k = 0; k < BK / 16; k++)
                umma(tmem_base, make_desc(sw + k * 32), make_desc(sx + k * 32), idesc, (i > 0 || k > 0) ? 1u : 0u);
            umma_commit(empty0 + 8 * s);
        }
        if (ok && len > 0) umma_commit(tfull);
    } else if (warp >= 4) {
        // this CTA's partial tile: TMEM -> registers -> own shared memory, [token][W row]
        const int q = warp & 3, r = q * 32 + lane;
        bool ok = true;
        if (len > 0) {
            ok = mbar_wait(tfull, 0, abort_flag);       // all MMAs done: the ring is drained too
            ok = __all_sync(0xffffffffu, ok);
        }
        if (ok && len > 0) {
            tc_fence_after();
            const uint32_t tbase = tmem_base + ((uint32_t)(q * 32) << 16);
#pragma unroll 1
            for (int c = 0; c < NB; c += 32) {
                uint32_t v[32];
                tmem_ld32(tbase + (uint32_t)c, v);
                tmem_ld_wait();
#pragma unroll
                for (int j = 0; j < 32; j++) part[(c + j) * TW + r] = __uint_as_float(v[j]);
            }
        } else {
            for (int m = 0; m < NB; m++) part[m * TW + r] = 0.f;   // empty k-range (or gave up): contributes nothing
        }
    }
    // every thread of every sharer: partials are complete and visible cluster-wide
    tc_fence_before();
    __syncthreads();
    __syncwarp();
    cluster_sync_all();
    if (warp >= 4) {
        const int r = (warp & 3) * 32 + lane, n = t * TW + r;
        const int mper = (p.M + splits - 1) / splits;
        const int m0 = rank * mper, m1 = min(p.M, m0 + mper);
        if (n < p.N) {
            const uint32_t my_part = smem_u32(part);
            for (int mb = m0; mb < m1; mb += 16) {
                float acc[16];
#pragma unroll
                for (int i = 0; i < 16; i++) acc[i] = 0.f;
                for (int c = 0; c < splits; c++) {           // rank order: a fixed summation order
                    const uint32_t remote = map_to_cta(my_part, (uint32_t)c);
                    float v[16];
#pragma unroll
                    for (int i = 0; i < 16; i++) {
                        v[i] = 0.f;
                        if (mb + i < m1)
                            asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v[i]) : "r"(remote + (uint32_t)(((mb + i) * TW + r) * 4)) : "memory");
                    }
#pragma unroll
                    for (int i = 0; i < 16; i++) acc[i] += v[i];
                }
#pragma unroll
                for (int i = 0; i < 16; i++)
                    if (mb + i < m1) p.C[(long long)(mb + i) * p.ldc + n] = __float2half_rn(acc[i]);
            }
        }
    }
    // nobody leaves (and frees its shared memory) while a sharer may still read it
    __syncwarp();
    cluster_sync_all();
    if (warp == 2) {
        tc_fence_after();
        tmem_dealloc<TMEM_COLS>(tmem_base);
    }
    if (threadIdx.x == 0 && *abort_flag) atomicExch(p.status, TL_ERR_TIMEOUT);
}

// ---- host side ------------------------------------------------------------------------------------
// One workspace per (device, stream): calls on different streams may overlap on the GPU.
struct Workspace { float* ws = nullptr; unsigned int* counters = nullptr; };
constexpr int MAX_GRID = 256, MAX_TILES = 1 << 16;
std::mutex g_ws_mutex;
std::unordered_map<unsigned long long, Workspace> g_ws;

int workspace_for(cudaStream_t st, Workspace* out) {
    int dev = 0;
    TL_CUDA(cudaGetDevice(&dev));
    const unsigned long long key = (unsigned long long)reinterpret_cast<uintptr_t>(st) * 64ull + (unsigned long long)dev;
    std::lock_guard<std::mutex> lock(g_ws_mutex);
    auto it = g_ws.find(key);
    if (it == g_ws.end()) {
        Workspace w;
        TL_CUDA(cudaMalloc(&w.ws, (size_t)2 * MAX_GRID * 128 * TW * sizeof(float)));
        TL_CUDA(cudaMalloc(&w.counters, (size_t)MAX_TILES * sizeof(unsigned int)));
        TL_CUDA(cudaMemset(w.counters, 0, (size_t)MAX_TILES * sizeof(unsigned int)));
        TL_CUDA(cudaDeviceSynchronize());
        it = g_ws.emplace(key, w).first;
    }
    *out = it->second;
    return TL_OK;
}

template <int NB>
int launch_nb(const CUtensorMap& mw, const CUtensorMap& mx, const SkinnyArgs& a, int grid, cudaStream_t st) {
    static PerDeviceOnce once;
    if (once.needed()) {
        TL_CUDA(cudaFuncSetAttribute(k_skinny<NB>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SkinnyCfg<NB>::SMEM));
    }
    return launch_pdl(k_skinny<NB>, dim3(grid), dim3(SK_THREADS), SkinnyCfg<NB>::SMEM, st, true, mw, mx, a);
}

template <int NB>
int launch_cluster(const CUtensorMap& mw, const CUtensorMap& mx, const SkinnyArgs& a, int grid, int cluster, cudaStream_t st) {
    static PerDeviceOnce once;
    if (once.needed()) {
        TL_CUDA(cudaFuncSetAttribute(k_skinny_cluster<NB>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SkinnyCfg<NB>::SMEM));
    }
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3((unsigned)grid);
    cfg.blockDim = dim3(SK_THREADS);
    cfg.dynamicSmemBytes = SkinnyCfg<NB>::SMEM;
    cfg.stream = st;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = (unsigned)cluster; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 2;
    TL_CUDA(cudaLaunchKernelEx(&cfg, k_skinny_cluster<NB>, mw, mx, a));
    return TL_OK;
}

}  // namespace

bool skinny_supported(const void* A, const void* W, size_t M, size_t N, size_t K, size_t lda, size_t ldw) {
    auto al16 = [](const void* q) { return (reinterpret_cast<uintptr_t>(q) & 15) == 0; };
    return M >= 2 && M <= 128 && N >= 1 && K >= 8 && lda % 8 == 0 && ldw % 8 == 0 && al16(A) && al16(W) &&
           (N + TW - 1) / TW <= (size_t)MAX_TILES && tensor_map_encode_available();
}

// Host-side planning (no device needed): how the (W tile, k-block) space of an M x N x K problem is
// cut for `sms` SMs.
SkinnyPlan skinny_plan(int M, int N, int K, int sms) {
    SkinnyPlan pl{};
    pl.nb = M <= 32 ? 32 : (M <= 64 ? 64 : 128);
    pl.tiles = (N + TW - 1) / TW;
    pl.nkb = (K + BK - 1) / BK;
    const long long total = (long long)pl.tiles * pl.nkb;
    // equal contiguous k-block ranges, one per SM; at least 4 k-blocks each so that tiny problems
    // do not pay a partial-tile exchange per k-block
    const int max_grid = std::max(1, std::min(sms, MAX_GRID));
    int per = (int)((total + max_grid - 1) / max_grid);
    if (per < 4) per = (int)std::min<long long>(4, total);
    // few W tiles: give every tile the same whole number of sharers when that still fills enough of
    // the SMs; two or more sharers form a cluster and reduce over distributed shared memory
    pl.cluster_splits = 0;
    if (pl.tiles <= max_grid) {
        const int sp = std::max(1, std::min(std::min(max_grid / pl.tiles, 8), std::max(1, pl.nkb / 4)));
        // measured at N = 11008 (86 tiles on 148 SMs): whole tiles beat the stream-K ranges once the
        // fp32 partial tiles are large (M = 128: 30.2 against 33.9 us; M = 64: 26.5 against 27.4) and
        // lose for narrow ones (M = 8: 23.6 against 22.0)
        const int fill_pct = pl.nb >= 64 ? 55 : 85;
        if ((long long)pl.tiles * sp * 100 >= (long long)max_grid * fill_pct) {
            per = (pl.nkb + sp - 1) / sp;
            if (sp >= 2) pl.cluster_splits = sp;
        }
    }
    pl.per = per;
    pl.grid = pl.cluster_splits >= 2 ? pl.tiles * pl.cluster_splits : (int)((total + per - 1) / per);
    return pl;
}

int launch_skinny(const __half* A, const __half* W, __half* C, int M, int N, int K, long long lda, long long ldw,
                  long long ldc, cudaStream_t st, bool weights_constant) {
    TL_REQUIRE(skinny_supported(A, W, M, N, K, lda, ldw), "skinny matmul: unsupported shape or alignment");
    const SkinnyPlan pl = skinny_plan(M, N, K, sm_count());
    const int nb = pl.nb, tiles = pl.tiles, nkb = pl.nkb, per = pl.per, cluster_splits = pl.cluster_splits, grid = pl.grid;
    Workspace w;
    TL_PROPAGATE(workspace_for(st, &w));
    CUtensorMap mw, mx;
    TL_PROPAGATE(make_tensor_map_f16(&mw, W, N, K, ldw, 0, 1, TW));
    TL_PROPAGATE(make_tensor_map_f16(&mx, A, M, K, lda, 0, 1, nb));
    SkinnyArgs a{C, ldc, M, N, K, tiles, nkb, per, cluster_splits, w.ws, w.counters, device_status_word(), weights_constant ? 1 : 0};
    if (cluster_splits >= 2) {
        if (nb == 32) return launch_cluster<32>(mw, mx, a, tiles * cluster_splits, cluster_splits, st);
        if (nb == 64) return launch_cluster<64>(mw, mx, a, tiles * cluster_splits, cluster_splits, st);
        return launch_cluster<128>(mw, mx, a, tiles * cluster_splits, cluster_splits, st);
    }
    if (nb == 32) return launch_nb<32>(mw, mx, a, grid, st);
    if (nb == 64) return launch_nb<64>(mw, mx, a, grid, st);
    return launch_nb<128>(mw, mx, a, grid, st);
}

}  // namespace tlb
