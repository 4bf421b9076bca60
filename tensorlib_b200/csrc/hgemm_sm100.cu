// Prefill HGEMM for sm_100a: C[M,N] = A[M,K] * B[N,K]^T, fp16 operands, fp32 accumulation in
// tensor memory, fp16 result. Replaces hgemm_cublas (tensorLib/src/device/cuda/hgemm.cu:20-38) and
// the mma.sync kernel next to it (:45-105) behind Device::matmul2d for M > 8.
//
// Both operands are K-major as stored (activations [M,K] and llama2.c weights [N,K] are row-major),
// so no transposes: TMA tensor maps (128-byte swizzle, no multicast) bring 128x64 A tiles and
// BNx64 B tiles into a 4-stage shared-memory ring; one elected thread issues tcgen05.mma
// (kind::f16, M=128, N=BN, K=16) with shared-memory descriptors; the fp32 accumulator (128 lanes x
// BN columns) lives in TMEM, double buffered, so the epilogue warps (tcgen05.ld -> fp16 -> global)
// drain tile i while the tensor core already works on tile i+1. Persistent: one CTA per SM walks
// the (batch, m-tile, n-tile) list. Warp roles: 0 TMA producer, 1 MMA issuer, 2 TMEM allocator,
// 4-7 epilogue. Bound: tensor pipe for M >= ~512 (2*M*N*K flops), HBM (the B operand) below.
//
// Epilogues fused for the Llama2 block (the operators the reference launches right after the
// matmul, model/llama2_7b/src/Transformer.cpp):
//   RESIDUAL  C = half(A B^T) + R                 wo / w2 matmul + EwiseAdd            (:111+:169, :143+:175)
//   SWIGLU    C = silu(A W1^T) * (A W3^T)         w1, w3 matmuls + silu + EwiseMul     (:136-141)
//             the B tile is 128 rows of W1 next to the same 128 rows of W3 (two TMA loads), so
//             gate and up of one output column sit in one accumulator row
//   QKV_ROPE  q, k, v = A [Wq|Wk|Wv]^T; rotary embedding on q and k; k, v written straight into
//             the KV cache rows of their positions                                    (:35-53)
//
// Every mbarrier wait is bounded; when one gives up the CTA raises an abort flag, every role
// leaves its loop, TMEM is freed and TL_ERR_TIMEOUT is recorded in the device status word.
#include <cuda.h>

#include <unordered_map>

#include <cstdlib>
#include <cstring>
#include <mutex>

#include "kernels.cuh"
#include "sm100.cuh"

namespace tlb {

namespace {

constexpr int BM = 128, BK = 64, STAGES = 4;
constexpr int GEMM_THREADS = 256;
constexpr int A_BYTES = BM * BK * 2;

using namespace sm100;

enum { GEPI_STORE = 0, GEPI_RESIDUAL = 1, GEPI_SWIGLU = 2, GEPI_QKV_ROPE = 3 };

struct GemmArgs {
    __half* C;
    int M, N, K, batch;
    long long ldc, sC;
    int a_batched, b_batched;   // 0: the operand is shared by all batches (batch coordinate 0)
    int b_const;                // cluster split-K kernel: B is a constant (a weight), its first tiles may be fetched before the dependency wait
    int* status;
    // RESIDUAL
    const __half* R; long long ldr;
    // QKV_ROPE: N = n_each columns per matrix; q -> C, k -> kc, v -> vc (row t = position pos0 + t,
    // the pointers already point at position pos0); cos/sin rows [t][head_dim / 2] likewise
    __half* kc; __half* vc; long long ld_kv;
    const __half* cos_t; const __half* sin_t;
    int head_dim;
    // CTA-pair kernel, stream-K mode (sk_per > 0): the flattened (tile, k-block) space is cut into ranges
    // of sk_per k-blocks, one per pair; partial tiles go through sk_ws, arrivals are counted in sk_counters
    int sk_per;
    float* sk_ws;
    unsigned int* sk_counters;
    // Tensor-parallel signalling (STORE epilogue of a K-split matmul): row m of the partial result is owned by
    // rank m / push_rows, which will fetch it from C (this rank's memory) once it is complete: when the 128 rows x
    // BN columns a CTA finished are stored, flag word push_flags[owner][(m0 % push_rows) / 128 *
    // PUSH_MAX_COL_TILES + column tile] in the OWNER's memory is set to push_epoch (one 4-byte peer store; the
    // tile itself stays local, because a thread's share of a tile is 64 contiguous bytes per row, far too small a
    // unit to send over NVLink). push_rows = 0: no signalling.
    unsigned int* push_flags[8];
    int push_rows;
    unsigned int push_epoch;
};
constexpr int PUSH_MAX_COL_TILES = 64;

// after the epilogue threads of one 128-row sub-tile have stored their rows: meet, and let one thread raise the
// flag of (row block, column tile) in the owner's memory. The barrier orders the other threads' stores before the
// writer's release store, which is cumulative at system scope (one fence per tile instead of one per thread).
__device__ __forceinline__ void push_signal(const GemmArgs& p, int row0, int col_tile, int bar_id, bool writer) {
    asm volatile("bar.sync %0, 128;" ::"r"(bar_id) : "memory");
    if (writer && row0 < p.M) {
        __threadfence_system();
        const int owner = row0 / p.push_rows, rb = (row0 - owner * p.push_rows) >> 7;
        asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p.push_flags[owner] + rb * PUSH_MAX_COL_TILES + col_tile), "r"(p.push_epoch) : "memory");
    }
}


// 32 consecutive columns of one output row: fp32 accumulators -> fp16 -> 64 bytes
__device__ __forceinline__ void store32(__half* dst, const uint32_t* r) {
#pragma unroll
    for (int v = 0; v < 4; v++) {
        uint4 o;
        __half2* oh = reinterpret_cast<__half2*>(&o);
#pragma unroll
        for (int j = 0; j < 4; j++)
            oh[j] = __floats2half2_rn(__uint_as_float(r[v * 8 + 2 * j]), __uint_as_float(r[v * 8 + 2 * j + 1]));
        *reinterpret_cast<uint4*>(dst + v * 8) = o;
    }
}
// The operands of the fused epilogues are loaded first and all together: the destination may alias
// them as far as the compiler knows (the residual add runs in place), so loads placed between the
// stores would each wait for a full L2 round trip.
__device__ __forceinline__ void store32_residual_pre(__half* dst, const uint4* rr, const uint32_t* r) {
#pragma unroll
    for (int v = 0; v < 4; v++) {
        uint4 o;
        __half2* oh = reinterpret_cast<__half2*>(&o);
        const __half2* rh = reinterpret_cast<const __half2*>(&rr[v]);
#pragma unroll
        for (int j = 0; j < 4; j++)   // the matmul result is rounded to fp16 first, then added in fp16
            oh[j] = __hadd2(__floats2half2_rn(__uint_as_float(r[v * 8 + 2 * j]), __uint_as_float(r[v * 8 + 2 * j + 1])), rh[j]);
        *reinterpret_cast<uint4*>(dst + v * 8) = o;
    }
}
__device__ __forceinline__ void load32_residual(uint4* rr, const __half* res) {
#pragma unroll
    for (int v = 0; v < 4; v++) rr[v] = *reinterpret_cast<const uint4*>(res + v * 8);
}
__device__ __forceinline__ void store32_residual(__half* dst, const __half* res, const uint32_t* r) {
    uint4 rr[4];
    load32_residual(rr, res);
    store32_residual_pre(dst, rr, r);
}
// interleaved-pair rotation (x0, x1) -> (x0 c - x1 s, x0 s + x1 c), every product and sum rounded
// to fp16 like the reference's apply_rotary_emb (tensorLib/src/device/CPU.cpp:427-461)
__device__ __forceinline__ void store32_rope_pre(__half* dst, const uint2* cc, const uint2* ss, const uint32_t* r) {
#pragma unroll
    for (int v = 0; v < 4; v++) {
        const __half* ch = reinterpret_cast<const __half*>(&cc[v]);
        const __half* sh = reinterpret_cast<const __half*>(&ss[v]);
        uint4 o;
        __half2* oh = reinterpret_cast<__half2*>(&o);
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const __half2 x = __floats2half2_rn(__uint_as_float(r[v * 8 + 2 * j]), __uint_as_float(r[v * 8 + 2 * j + 1]));
            const __half2 t1 = __hmul2(x, __half2half2(ch[j]));                          // (x0 c, x1 c)
            const __half2 t2 = __hmul2(__lowhigh2highlow(x), __half2half2(sh[j]));       // (x1 s, x0 s)
            oh[j] = __halves2half2(__hsub(__low2half(t1), __low2half(t2)), __hadd(__high2half(t2), __high2half(t1)));
        }
        *reinterpret_cast<uint4*>(dst + v * 8) = o;
    }
}
__device__ __forceinline__ void load32_rope(uint2* cc, uint2* ss, const __half* cosr, const __half* sinr) {
#pragma unroll
    for (int v = 0; v < 4; v++) {
        cc[v] = *reinterpret_cast<const uint2*>(cosr + v * 4);
        ss[v] = *reinterpret_cast<const uint2*>(sinr + v * 4);
    }
}
__device__ __forceinline__ void store32_rope(__half* dst, const __half* cosr, const __half* sinr, const uint32_t* r) {
    uint2 cc[4], ss[4];
    load32_rope(cc, ss, cosr, sinr);
    store32_rope_pre(dst, cc, ss, r);
}
// silu(gate) * up with the gate through float: g / (1 + exp(-g)), rounded to fp16, then an fp16 product
__device__ __forceinline__ void store32_swiglu(__half* dst, const uint32_t* g, const uint32_t* u) {
#pragma unroll
    for (int v = 0; v < 4; v++) {
        uint4 o;
        __half* oh = reinterpret_cast<__half*>(&o);
#pragma unroll
        for (int j = 0; j < 8; j++) {
            const float gf = __half2float(__float2half_rn(__uint_as_float(g[v * 8 + j])));
            const __half s = __float2half_rn(gf / (1.f + __expf(-gf)));
            oh[j] = __hmul(s, __float2half_rn(__uint_as_float(u[v * 8 + j])));
        }
        *reinterpret_cast<uint4*>(dst + v * 8) = o;
    }
}

template <int BN, int EPI>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
k_hgemm(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
        const __grid_constant__ CUtensorMap tmB2, const __grid_constant__ CUtensorMap tmB3, GemmArgs p) {
    constexpr int B_BYTES = BN * BK * 2;
    constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
    constexpr uint32_t TMEM_COLS = 2 * BN;      // two accumulator buffers
    constexpr int OUT_COLS = EPI == GEPI_SWIGLU ? BN / 2 : BN;   // output columns per tile
    extern __shared__ unsigned char smem_raw[];
    // the swizzled tiles need 1024-byte alignment
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES);
    const uint32_t full0 = smem_u32(bars), empty0 = smem_u32(bars + STAGES);
    const uint32_t tfull0 = smem_u32(bars + 2 * STAGES), tempty0 = smem_u32(bars + 2 * STAGES + 2);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int mt_count = (p.M + BM - 1) / BM;
    const int nt_each = (p.N + OUT_COLS - 1) / OUT_COLS;                 // column tiles per weight matrix
    const int nt_count = EPI == GEPI_QKV_ROPE ? 3 * nt_each : nt_each;
    const int tiles_per_batch = mt_count * nt_count;
    const int total_tiles = tiles_per_batch * p.batch;
    const int nkb = (p.K + BK - 1) / BK;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; s++) { mbar_init(full0 + 8 * s, 1); mbar_init(empty0 + 8 * s, 1); }
        for (int b = 0; b < 2; b++) { mbar_init(tfull0 + 8 * b, 1); mbar_init(tempty0 + 8 * b, 4); }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 2) tmem_alloc<TMEM_COLS>(tmem_slot);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    // set-up done (barriers, TMEM): let the next kernel of the stream start its own set-up, then wait
    // for the previous one before any operand is read or any result written
    pdl_launch_dependents();
    pdl_wait();

    if (warp == 0 && lane == 0) {
        // ---------------- TMA producer ---------------------------------------------------------
        asm volatile("prefetch.tensormap [%0];" ::"l"(&tmA) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&tmB) : "memory");
        if (EPI == GEPI_SWIGLU || EPI == GEPI_QKV_ROPE) asm volatile("prefetch.tensormap [%0];" ::"l"(&tmB2) : "memory");
        if (EPI == GEPI_QKV_ROPE) asm volatile("prefetch.tensormap [%0];" ::"l"(&tmB3) : "memory");
        int it = 0;
        bool ok = true;
        for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
            const int b = tile / tiles_per_batch, idx = tile - b * tiles_per_batch;
            const int mt = idx % mt_count, nt = idx / mt_count;
            const int which = EPI == GEPI_QKV_ROPE ? nt / nt_each : 0, ntl = nt - which * nt_each;
            const CUtensorMap* mb = which == 0 ? &tmB : (which == 1 ? &tmB2 : &tmB3);
            for (int kb = 0; kb < nkb; kb++, it++) {
                const int s = it % STAGES, use = it / STAGES;
                if (use > 0 && !(ok = mbar_wait(empty0 + 8 * s, (use - 1) & 1, abort_flag))) break;
                const uint32_t sa = smem_u32(smem + s * STAGE_BYTES), sb = sa + A_BYTES;
                mbar_arrive_expect_tx(full0 + 8 * s, STAGE_BYTES);
                tma_load_3d(sa, &tmA, kb * BK, mt * BM, p.a_batched ? b : 0, full0 + 8 * s);
                if (EPI == GEPI_SWIGLU) {   // rows [0, BN/2): W1, rows [BN/2, BN): the same rows of W3
                    tma_load_3d(sb, &tmB, kb * BK, ntl * OUT_COLS, 0, full0 + 8 * s);
                    tma_load_3d(sb + B_BYTES / 2, &tmB2, kb * BK, ntl * OUT_COLS, 0, full0 + 8 * s);
                } else {
                    tma_load_3d(sb, mb, kb * BK, ntl * BN, p.b_batched ? b : 0, full0 + 8 * s);
                }
            }
        }
        if (!ok) {  // let copies already in flight land before the CTA goes away
            const int issued = it;
            for (int j = max(0, issued - STAGES); j < issued; j++)
                for (uint32_t i = 0; i < (1u << 16); i++)
                    if (mbar_try_wait(full0 + 8 * (j % STAGES), (j / STAGES) & 1)) break;
        }
    } else if (warp == 1 && lane == 0) {
        // ---------------- MMA issuer ------------------------------------------------------------
        constexpr uint32_t idesc = make_idesc(BN);
        int it = 0, tcount = 0;
        bool ok = true;
        for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x, tcount++) {
            const int buf = tcount & 1, use = tcount >> 1;
            if (use > 0 && !(ok = mbar_wait(tempty0 + 8 * buf, (use - 1) & 1, abort_flag))) break;
            tc_fence_after();
            const uint32_t d_tmem = tmem_base + (uint32_t)(buf * BN);
            for (int kb = 0; kb < nkb; kb++, it++) {
                const int s = it % STAGES, use_s = it / STAGES;
                if (!(ok = mbar_wait(full0 + 8 * s, use_s & 1, abort_flag))) break;
                tc_fence_after();
                const uint32_t sa = smem_u32(smem + s * STAGE_BYTES), sb = sa + A_BYTES;
#pragma unroll
                for (int k = 0; k < BK / 16; k++)
                    umma(d_tmem, make_desc(sa + k * 32), make_desc(sb + k * 32), idesc, (kb > 0 || k > 0) ? 1u : 0u);
                umma_commit(empty0 + 8 * s);      // stage reusable once these MMAs have read it
            }
            if (ok) umma_commit(tfull0 + 8 * buf);  // accumulator complete
        }
    } else if (warp >= 4) {
        // ---------------- epilogue: TMEM -> registers -> fp16 (+ fused operator) -> global -------------
        const int q = warp & 3;                   // TMEM lane quarter this warp may access
        int tcount = 0;
        bool ok = true;
        const bool vec_ok = (p.ldc % 8 == 0) && (p.sC % 8 == 0) && ((reinterpret_cast<uintptr_t>(p.C) & 15) == 0);
        for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x, tcount++) {
            const int b = tile / tiles_per_batch, idx = tile - b * tiles_per_batch;
            const int mt = idx % mt_count, nt = idx / mt_count;
            const int which = EPI == GEPI_QKV_ROPE ? nt / nt_each : 0, ntl = nt - which * nt_each;
            const int buf = tcount & 1, use = tcount >> 1;
            ok = mbar_wait(tfull0 + 8 * buf, use & 1, abort_flag);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            tc_fence_after();
            const int row = mt * BM + q * 32 + lane;
            const uint32_t tbase = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(buf * BN);
            __half* crow = p.C + (long long)b * p.sC + (long long)row * p.ldc;
            if (EPI == GEPI_SWIGLU) {
#pragma unroll 1
                for (int c = 0; c < OUT_COLS; c += 32) {
                    uint32_t g[32], u[32];
                    tmem_ld32(tbase + (uint32_t)c, g);
                    tmem_ld32(tbase + (uint32_t)(OUT_COLS + c), u);
                    tmem_ld_wait();
                    const int col0 = ntl * OUT_COLS + c;
                    if (row < p.M && col0 < p.N) store32_swiglu(crow + col0, g, u);
                }
            } else {
#pragma unroll 1
                for (int c = 0; c < BN; c += 32) {
                    uint32_t r[32];
                    tmem_ld32(tbase + (uint32_t)c, r);
                    tmem_ld_wait();
                    const int col0 = ntl * BN + c;
                    if (row >= p.M || col0 >= p.N) continue;
                    if (EPI == GEPI_RESIDUAL) {
                        store32_residual(crow + col0, p.R + (long long)row * p.ldr + col0, r);
                    } else if (EPI == GEPI_QKV_ROPE) {
                        if (which == 2) {
                            store32(p.vc + (long long)row * p.ld_kv + col0, r);
                        } else {
                            const int half_dim = p.head_dim >> 1, d2 = (col0 % p.head_dim) >> 1;
                            __half* dst = which == 0 ? crow + col0 : p.kc + (long long)row * p.ld_kv + col0;
                            store32_rope(dst, p.cos_t + (long long)row * half_dim + d2, p.sin_t + (long long)row * half_dim + d2, r);
                        }
                    } else if (vec_ok && col0 + 32 <= p.N) {
                        store32(crow + col0, r);
                    } else {
                        for (int j = 0; j < 32 && col0 + j < p.N; j++)
                            crow[col0 + j] = __float2half_rn(__uint_as_float(r[j]));
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(tempty0 + 8 * buf);
            if (EPI == GEPI_STORE && p.push_rows > 0) push_signal(p, mt * BM, ntl, 2, warp == 4 && lane == 0);
        }
    }
    // ---------------- teardown ---------------------------------------------------------------------
    tc_fence_before();
    __syncthreads();
    if (warp == 2) {
        tc_fence_after();
        tmem_dealloc<TMEM_COLS>(tmem_base);
    }
    if (threadIdx.x == 0 && *abort_flag) atomicExch(p.status, TL_ERR_TIMEOUT);
}

// ---- one tile per cluster, K split over its CTAs ---------------------------------------------------------
// Few output tiles and a long K (M <= 512 against the 7B weights, or any M <= 128): whole tiles on a persistent
// grid leave most SMs idle, and splitting K through global memory costs a round trip of fp32 partial tiles plus
// a counter. Here the KS CTAs of a cluster each run the TMA -> tcgen05 pipeline over their K / KS share of the
// SAME (128 MSUB) x BN tile (accumulators in their own TMEM) and then exchange partial sums over distributed
// shared memory as a reduce-scatter: CTA r finishes columns [r BN/KS, (r+1) BN/KS) of the tile, every other CTA
// writes its fp32 partial of those columns into r's pipeline stages, idle by then (st.shared::cluster, a warp
// writes 512 contiguous bytes) and arrives on r's mbarrier (release at cluster scope); r adds the parts in rank
// order, converts and stores. No workspace, no atomics, the order of the additions is fixed, and the epilogue
// itself is spread over all KS CTAs. MSUB = 2 gives one CTA a 256 x 256 tile (two 128-row A boxes against one
// B box, all 512 TMEM columns): 64 KB of shared-memory fill per 1024 MMA cycles instead of 48 KB per 512, which
// takes a single CTA off the fill limit; with KS = 1 that is a plain one-wave kernel for shapes of up to one
// 256 x 256 tile per SM. The launcher uses the family only when tiles x KS fits the SMs.
template <int BN, int KS, int MSUB>
struct SplitCfg {
    static constexpr int B_BYTES = BN * BK * 2;
    static constexpr int STAGE_BYTES = MSUB * A_BYTES + B_BYTES;
    static constexpr int SLICE = BN / KS;                               // output columns one CTA finishes
    static constexpr int PART_BYTES = MSUB * BM * SLICE * 4;            // one sender's partial of my slice
    static constexpr int RECV_BYTES = (KS - 1) * PART_BYTES;            // received over the pipeline stages, once they are idle
    static constexpr int NST = (216 * 1024) / STAGE_BYTES > 8 ? 8 : (216 * 1024) / STAGE_BYTES;
    static constexpr size_t SMEM = (size_t)NST * STAGE_BYTES + 1024 + 256;
    static constexpr uint32_t TMEM_COLS = MSUB * BN;
    static_assert(SLICE % 32 == 0 && NST >= 2 && RECV_BYTES <= NST * STAGE_BYTES, "slice of whole 32-column chunks; the parts fit the stages");
    static_assert(TMEM_COLS == 128 || TMEM_COLS == 256 || TMEM_COLS == 512, "tensor-memory columns: a power of two");
};

template <int BN, int KS, int MSUB, int EPI>
__global__ void __cluster_dims__(KS, 1, 1) __launch_bounds__(GEMM_THREADS, 1)
k_hgemm_splitk(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, GemmArgs p) {
    using Cfg = SplitCfg<BN, KS, MSUB>;
    constexpr int NST = Cfg::NST, STAGE_BYTES = Cfg::STAGE_BYTES, SLICE = Cfg::SLICE;
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    unsigned char* recv = smem;                                          // [sender slot][sub-tile][column / 4][row][4 floats], over the idle stages
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + NST * STAGE_BYTES);
    const uint32_t full0 = smem_u32(bars), empty0 = smem_u32(bars + NST);
    const uint32_t tfull = smem_u32(bars + 2 * NST), recv_full = smem_u32(bars + 2 * NST + 1), peers_idle = smem_u32(bars + 2 * NST + 2);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * NST + 3);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int rank = KS > 1 ? (int)cluster_ctarank() : 0;
    const int tile = blockIdx.x / KS;
    const int mt_count = (p.M + MSUB * BM - 1) / (MSUB * BM);
    const int mt = tile % mt_count, nt = tile / mt_count;
    const int nkb = (p.K + BK - 1) / BK;
    const int kb0 = (int)((long long)nkb * rank / KS), kb1 = (int)((long long)nkb * (rank + 1) / KS);

    if (threadIdx.x == 0) {
        for (int s = 0; s < NST; s++) { mbar_init(full0 + 8 * s, 1); mbar_init(empty0 + 8 * s, 1); }
        mbar_init(tfull, 1);
        mbar_init(recv_full, KS > 1 ? (KS - 1) * 128 : 1);   // every epilogue thread of every other CTA arrives once
        mbar_init(peers_idle, KS > 1 ? KS - 1 : 1);          // one thread of every other CTA, when its stages are idle
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 2) tmem_alloc<Cfg::TMEM_COLS>(tmem_slot);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    if (KS > 1) cluster_sync_all();                  // nobody arrives on a barrier that is not initialised yet
    pdl_launch_dependents();

    if (warp == 0 && lane == 0) {
        // ---------------- TMA producer ---------------------------------------------------------
        asm volatile("prefetch.tensormap [%0];" ::"l"(&tmA) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&tmB) : "memory");
        // B a constant (a model weight): its first tiles are requested while the previous kernel of the
        // stream is still running; A, which that kernel may have written, only after the dependency wait
        const int early = p.b_const ? min(NST, kb1 - kb0) : 0;
        for (int it = 0; it < early; it++) {
            mbar_arrive_expect_tx(full0 + 8 * it, STAGE_BYTES);
            tma_load_3d(smem_u32(smem + it * STAGE_BYTES) + MSUB * A_BYTES, &tmB, (kb0 + it) * BK, nt * BN, 0, full0 + 8 * it);
        }
        pdl_wait();
        bool ok = true;
        int it = 0;
        for (int kb = kb0; kb < kb1; kb++, it++) {
            const int s = it % NST, use = it / NST;
            if (use > 0 && !(ok = mbar_wait(empty0 + 8 * s, (use - 1) & 1, abort_flag))) break;
            const uint32_t sa = smem_u32(smem + s * STAGE_BYTES), sb = sa + MSUB * A_BYTES;
            if (it >= early) mbar_arrive_expect_tx(full0 + 8 * s, STAGE_BYTES);
#pragma unroll
            for (int ms = 0; ms < MSUB; ms++)       // rows beyond M read as zero
                tma_load_3d(sa + ms * A_BYTES, &tmA, kb * BK, (mt * MSUB + ms) * BM, 0, full0 + 8 * s);
            if (it >= early) tma_load_3d(sb, &tmB, kb * BK, nt * BN, 0, full0 + 8 * s);
        }
        if (!ok) {  // let copies already in flight land before the CTA goes away
            for (int j = max(0, it - NST); j < it; j++)
                for (uint32_t i = 0; i < (1u << 16); i++)
                    if (mbar_try_wait(full0 + 8 * (j % NST), (j / NST) & 1)) break;
        }
    } else if (warp == 1 && lane == 0) {
        // ---------------- MMA issuer ------------------------------------------------------------
        pdl_wait();
        constexpr uint32_t idesc = make_idesc(BN);
        bool ok = true;
        int it = 0;
        for (int kb = kb0; kb < kb1; kb++, it++) {
            const int s = it % NST, use_s = it / NST;
            if (!(ok = mbar_wait(full0 + 8 * s, use_s & 1, abort_flag))) break;
            tc_fence_after();
            const uint32_t sa = smem_u32(smem + s * STAGE_BYTES), sb = sa + MSUB * A_BYTES;
#pragma unroll
            for (int k = 0; k < BK / 16; k++)
#pragma unroll
                for (int ms = 0; ms < MSUB; ms++)
                    umma(tmem_base + (uint32_t)(ms * BN), make_desc(sa + ms * A_BYTES + k * 32), make_desc(sb + k * 32), idesc,
                         (kb > kb0 || k > 0) ? 1u : 0u);
            umma_commit(empty0 + 8 * s);
        }
        if (ok) umma_commit(tfull);
    } else if (warp >= 4) {
        // ---------------- epilogue: send the foreign slices, finish the own one -------------------------
        pdl_wait();
        const int q = warp & 3, rl = q * 32 + lane;                       // row of a sub-tile = TMEM lane
        bool ok = mbar_wait(tfull, 0, abort_flag);
        ok = __all_sync(0xffffffffu, ok);
        tc_fence_after();
        const uint32_t tbase = tmem_base + ((uint32_t)(q * 32) << 16);
        if (KS > 1 && ok) {
            // all my MMAs are done, so my stages are idle: the other CTAs may write their parts over them
            if (warp == 4 && lane == 0) {
#pragma unroll 1
                for (int o = 0; o < KS; o++)
                    if (o != rank) mbar_arrive_cluster(map_to_cta(peers_idle, (uint32_t)o));
            }
            ok = mbar_wait_cluster(peers_idle, 0, abort_flag);
            ok = __all_sync(0xffffffffu, ok);
        }
        if (KS > 1 && ok) {
#pragma unroll 1
            for (int o = 0; o < KS; o++) {
                if (o == rank) continue;
                const int slot = rank < o ? rank : rank - 1;              // senders in rank order, the owner left out
                const uint32_t dst = map_to_cta(smem_u32(recv), (uint32_t)o) + (uint32_t)(slot * Cfg::PART_BYTES + rl * 16);
#pragma unroll 1
                for (int ms = 0; ms < MSUB; ms++) {
#pragma unroll 1
                    for (int c = 0; c < SLICE; c += 32) {
                        uint32_t r[32];
                        tmem_ld32(tbase + (uint32_t)(ms * BN + o * SLICE + c), r);
                        tmem_ld_wait();
#pragma unroll
                        for (int v = 0; v < 8; v++)
                            st_cluster_f4(dst + (uint32_t)(((ms * SLICE + c) / 4 + v) * BM * 16), __uint_as_float(r[4 * v]),
                                          __uint_as_float(r[4 * v + 1]), __uint_as_float(r[4 * v + 2]), __uint_as_float(r[4 * v + 3]));
                    }
                }
                mbar_arrive_cluster(map_to_cta(recv_full, (uint32_t)o));
            }
            ok = mbar_wait_cluster(recv_full, 0, abort_flag);
            ok = __all_sync(0xffffffffu, ok);
        }
        if (ok) {
            const float4* mine = reinterpret_cast<const float4*>(recv) + rl;
#pragma unroll 1
            for (int ms = 0; ms < MSUB; ms++) {
                const int row = (mt * MSUB + ms) * BM + rl;
                __half* crow = p.C + (long long)row * p.ldc;
#pragma unroll 1
                for (int c = 0; c < SLICE; c += 32) {
                    uint32_t r[32];
                    tmem_ld32(tbase + (uint32_t)(ms * BN + rank * SLICE + c), r);
                    tmem_ld_wait();
                    if (KS > 1) {
                        float acc[32];
#pragma unroll
                        for (int i = 0; i < 32; i++) acc[i] = 0.f;
#pragma unroll
                        for (int s = 0; s < KS; s++) {                    // parts in k order = rank order
                            if (s == rank) {
#pragma unroll
                                for (int i = 0; i < 32; i++) acc[i] += __uint_as_float(r[i]);
                            } else {
                                const float4* src = mine + (size_t)(s < rank ? s : s - 1) * (Cfg::PART_BYTES / 16) + (size_t)((ms * SLICE + c) / 4) * BM;
#pragma unroll
                                for (int v = 0; v < 8; v++) {
                                    const float4 f = src[(size_t)v * BM];
                                    acc[4 * v] += f.x; acc[4 * v + 1] += f.y; acc[4 * v + 2] += f.z; acc[4 * v + 3] += f.w;
                                }
                            }
                        }
#pragma unroll
                        for (int i = 0; i < 32; i++) r[i] = __float_as_uint(acc[i]);
                    }
                    const int col0 = nt * BN + rank * SLICE + c;
                    if (row >= p.M || col0 >= p.N) continue;
                    if (EPI == GEPI_RESIDUAL) store32_residual(crow + col0, p.R + (long long)row * p.ldr + col0, r);
                    else store32(crow + col0, r);
                }
            }
        }
    }
    // ---------------- teardown: nobody leaves while a CTA of the cluster may still write to it ---------
    tc_fence_before();
    __syncthreads();
    __syncwarp();
    if (KS > 1) cluster_sync_all();
    if (warp == 2) {
        tc_fence_after();
        tmem_dealloc<Cfg::TMEM_COLS>(tmem_base);
    }
    if (threadIdx.x == 0 && *abort_flag) atomicExch(p.status, TL_ERR_TIMEOUT);
}

// ---- CTA-pair variant: 256 x 256 tile per 2-CTA cluster ------------------------------------------
// The 128x256 tile above is limited by the rate at which one SM can fill its shared memory
// (48 KB per 512 MMA cycles: the tensor pipe measures 69 % active). With cta_group::2 the two CTAs
// of a cluster share one MMA of M = 256: each CTA loads its own 128 rows of A and only HALF of the
// B tile (128 of the 256 weight rows), 32 KB per 512 MMA cycles, and keeps its 128 rows of the
// accumulator in its own TMEM. The leader CTA (cluster rank 0) issues the MMAs and owns the "full"
// barriers (the loads of both CTAs complete there); "empty" and "accumulator ready" are
// signalled to each CTA's own barrier by a separate commit; the peer's epilogue warps release
// the accumulator on the leader's barrier with a remote arrive. No multicast anywhere.
// For SWIGLU the split of B by halves is exactly W1 | W3: rank 0 loads the W1 rows, rank 1 the
// W3 rows of the same output columns.
// MSUB = 2 gives every CTA TWO 128-row sub-tiles of A against the same half B tile (a 512 x 256 tile per
// pair, two accumulators = all 512 TMEM columns, so no accumulator double buffering): 48 KB of
// operands per CTA for twice the MMA work, i.e. 24 KB per 512 MMA cycles. That moves the kernel
// from the shared-memory fill limit (measured ~72 B/clk per SM) to the tensor pipe.
constexpr int PAIR_BN = 256;
constexpr int PAIR_B_BYTES = (PAIR_BN / 2) * BK * 2;                  // this CTA's half of the B tile
template <int MSUB> struct PairCfg {
    static constexpr int STAGE_BYTES = MSUB * A_BYTES + PAIR_B_BYTES;   // 32 KB / 48 KB
    static constexpr int STAGES = MSUB == 1 ? 6 : 4;
    static constexpr size_t SMEM = (size_t)STAGES * STAGE_BYTES + 1024 + 256;
    static constexpr int THREADS = GEMM_THREADS + (MSUB - 1) * 128;     // four epilogue warps per sub-tile
};

// The work of one pair as a list of segments (tile, k-blocks [kb0, kb1)). Whole-tile mode: tiles pair,
// pair + n_pairs, ... each with all its k-blocks. Stream-K mode: the contiguous range
// [pair * per, (pair + 1) * per) of the flattened (tile, k-block) space, so a pair may start in the
// middle of one tile and end in the middle of another. The partial pieces come FIRST (the one at the
// start of the range, then the one at its end), the whole tiles after them: every tile's parts are
// then finished early in the launch and the last arriver adds them up while its whole tiles run,
// instead of at the very end. `first` marks the piece at the start of the range (workspace slot 0).
struct PairSegments {
    int mode_per, nkb, n_pairs, total_tiles;
    int tile_next;                 // whole-tile mode cursor; stream-K: next whole tile
    int stage;                     // stream-K: 0 start piece, 1 end piece, 2 whole tiles
    int t_first, kb_first0, t_last, kb_last1, w_end;
    bool empty;
    __device__ PairSegments(int per, int nkb_, int pair, int n_pairs_, int total_tiles_)
        : mode_per(per), nkb(nkb_), n_pairs(n_pairs_), total_tiles(total_tiles_), tile_next(pair), stage(0) {
        if (per > 0) {
            const long long total = (long long)total_tiles_ * nkb_;
            const long long begin = min(total, (long long)pair * per), end = min(total, begin + per);
            empty = begin >= end;
            if (!empty) {
                t_first = (int)(begin / nkb_); kb_first0 = (int)(begin - (long long)t_first * nkb_);
                t_last = (int)((end - 1) / nkb_); kb_last1 = (int)(end - (long long)t_last * nkb_);
                // whole tiles: t_first if it starts at k-block 0 (and is not cut at the end), ... , t_last if it ends at nkb
                tile_next = (kb_first0 == 0 && (t_last > t_first || kb_last1 == nkb_)) ? t_first : t_first + 1;
                w_end = (kb_last1 == nkb_) ? t_last + 1 : t_last;
            }
        }
    }
    __device__ bool next(int& tile, int& kb0, int& kb1, bool& first) {
        if (mode_per > 0) {
            if (empty) return false;
            if (stage == 0) {      // the piece at the start of the range, if it is not a whole tile
                stage = 1;
                const int e = t_last == t_first ? kb_last1 : nkb;
                if (kb_first0 > 0 || e < nkb) { tile = t_first; kb0 = kb_first0; kb1 = e; first = true; return true; }
            }
            if (stage == 1) {      // the piece at the end of the range, if it is a different, cut tile
                stage = 2;
                if (t_last > t_first && kb_last1 < nkb) { tile = t_last; kb0 = 0; kb1 = kb_last1; first = false; return true; }
            }
            if (tile_next >= w_end) return false;
            tile = tile_next++; kb0 = 0; kb1 = nkb; first = false;
            return true;
        }
        if (tile_next >= total_tiles) return false;
        tile = tile_next; kb0 = 0; kb1 = nkb; first = false;
        tile_next += n_pairs;
        return true;
    }
};

template <int EPI, int MSUB>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(PairCfg<MSUB>::THREADS, 1)
k_hgemm_pair(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
             const __grid_constant__ CUtensorMap tmB2, const __grid_constant__ CUtensorMap tmB3, GemmArgs p) {
    constexpr int BN = PAIR_BN, STAGES = PairCfg<MSUB>::STAGES, STAGE_BYTES = PairCfg<MSUB>::STAGE_BYTES;
    constexpr uint32_t TMEM_COLS = 2 * BN;      // MSUB 1: two buffers of one accumulator; MSUB 2: one buffer of two
    constexpr int OUT_COLS = EPI == GEPI_SWIGLU ? BN / 2 : BN;
    constexpr int EPI_THREADS = 128 * MSUB;
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES);
    const uint32_t full0 = smem_u32(bars), empty0 = smem_u32(bars + STAGES);
    const uint32_t tfull0 = smem_u32(bars + 2 * STAGES), tempty0 = smem_u32(bars + 2 * STAGES + 2);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    volatile int* last_flag = reinterpret_cast<volatile int*>(tmem_slot + 2);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();                              // 0: leader
    const int pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;
    const int mt_count = (p.M + 2 * MSUB * BM - 1) / (2 * MSUB * BM);     // 256- or 512-row tiles
    const int nt_each = (p.N + OUT_COLS - 1) / OUT_COLS;
    const int nt_count = EPI == GEPI_QKV_ROPE ? 3 * nt_each : nt_each;
    const int tiles_per_batch = mt_count * nt_count;
    const int total_tiles = tiles_per_batch * p.batch;
    const int nkb = (p.K + BK - 1) / BK;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; s++) { mbar_init(full0 + 8 * s, 1); mbar_init(empty0 + 8 * s, 1); }
        for (int b = 0; b < 2; b++) { mbar_init(tfull0 + 8 * b, 1); mbar_init(tempty0 + 8 * b, 8 * MSUB); }   // epilogue warps x 2 CTAs
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 2) tmem_alloc_pair<TMEM_COLS>(tmem_slot);
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();          // both CTAs' barriers exist before anything is signalled across the pair
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    // set-up done (barriers, TMEM): let the next kernel of the stream start its own set-up, then wait
    // for the previous one before any operand is read or any result written
    pdl_launch_dependents();
    pdl_wait();

    if (warp == 0 && lane == 0) {
        // ---------------- TMA producer (both CTAs) ----------------------------------------------
        asm volatile("prefetch.tensormap [%0];" ::"l"(&tmA) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&tmB) : "memory");
        if (EPI == GEPI_SWIGLU || EPI == GEPI_QKV_ROPE) asm volatile("prefetch.tensormap [%0];" ::"l"(&tmB2) : "memory");
        if (EPI == GEPI_QKV_ROPE) asm volatile("prefetch.tensormap [%0];" ::"l"(&tmB3) : "memory");
        int it = 0;
        bool ok = true;
        PairSegments segs(p.sk_per, nkb, pair, n_pairs, total_tiles);
        int tile, kb0, kb1; bool first;
        while (ok && segs.next(tile, kb0, kb1, first)) {
            const int b = tile / tiles_per_batch, idx = tile - b * tiles_per_batch;
            const int mt = idx % mt_count, nt = idx / mt_count;
            const int which = EPI == GEPI_QKV_ROPE ? nt / nt_each : 0, ntl = nt - which * nt_each;
            const CUtensorMap* mb = EPI == GEPI_SWIGLU ? (rank == 0 ? &tmB : &tmB2)
                                                       : (which == 0 ? &tmB : (which == 1 ? &tmB2 : &tmB3));
            const int brow = EPI == GEPI_SWIGLU ? ntl * OUT_COLS : ntl * BN + (int)rank * (BN / 2);
            for (int kb = kb0; kb < kb1; kb++, it++) {
                const int s = it % STAGES, use = it / STAGES;
                if (use > 0 && !(ok = mbar_wait(empty0 + 8 * s, (use - 1) & 1, abort_flag))) break;
                const uint32_t sa = smem_u32(smem + s * STAGE_BYTES), sb = sa + MSUB * A_BYTES;
                const uint32_t leader_full = map_to_cta(full0 + 8 * s, 0);
                if (rank == 0) mbar_arrive_expect_tx(full0 + 8 * s, 2 * STAGE_BYTES);   // both CTAs' bytes
#pragma unroll
                for (int ms = 0; ms < MSUB; ms++)   // sub-tile ms of this CTA: rows ((mt * 2 + rank) * MSUB + ms) * 128 ...
                    tma_load_3d_pair(sa + ms * A_BYTES, &tmA, kb * BK, ((mt * 2 + (int)rank) * MSUB + ms) * BM,
                                     p.a_batched ? b : 0, leader_full);
                tma_load_3d_pair(sb, mb, kb * BK, brow, p.b_batched ? b : 0, leader_full);
            }
        }
        // Copies in flight complete on the leader's barrier; before leaving, wait (bounded) until
        // the MMAs that read this CTA's last stages are done: its "empty" barriers say so.
        if (ok) {
            for (int j = max(0, it - STAGES); j < it; j++)
                if (!mbar_wait(empty0 + 8 * (j % STAGES), (j / STAGES) & 1, abort_flag)) break;
        }
    } else if (warp == 1 && lane == 0 && rank == 0) {
        // ---------------- MMA issuer (leader only) ------------------------------------------------
        constexpr uint32_t idesc = make_idesc_pair(BN);
        int it = 0, tcount = 0;
        bool ok = true;
        PairSegments segs(p.sk_per, nkb, pair, n_pairs, total_tiles);
        int tile, kb0, kb1; bool first;
        for (; ok && segs.next(tile, kb0, kb1, first); tcount++) {
            // MSUB 1: accumulator buffers alternate; MSUB 2: both accumulators form the single buffer 0
            const int buf = MSUB == 1 ? (tcount & 1) : 0, use = MSUB == 1 ? (tcount >> 1) : tcount;
            if (use > 0 && !(ok = mbar_wait(tempty0 + 8 * buf, (use - 1) & 1, abort_flag))) break;
            tc_fence_after();
            const uint32_t d_tmem = tmem_base + (uint32_t)(buf * BN);
            for (int kb = kb0; kb < kb1; kb++, it++) {
                const int s = it % STAGES, use_s = it / STAGES;
                if (!(ok = mbar_wait(full0 + 8 * s, use_s & 1, abort_flag))) break;
                tc_fence_after();
                const uint32_t sa = smem_u32(smem + s * STAGE_BYTES), sb = sa + MSUB * A_BYTES;
#pragma unroll
                for (int k = 0; k < BK / 16; k++)
#pragma unroll
                    for (int ms = 0; ms < MSUB; ms++)
                        umma_pair(d_tmem + (uint32_t)(ms * BN), make_desc(sa + ms * A_BYTES + k * 32), make_desc(sb + k * 32), idesc,
                                  (kb > kb0 || k > 0) ? 1u : 0u);
                umma_commit_pair(empty0 + 8 * s);                   // my stage is reusable
                umma_commit_pair(map_to_cta(empty0 + 8 * s, 1));    // and the peer's
            }
            if (ok) {
                umma_commit_pair(tfull0 + 8 * buf);
                umma_commit_pair(map_to_cta(tfull0 + 8 * buf, 1));
            }
        }
    } else if (warp >= 4) {
        // ---------------- epilogue (both CTAs, own 128 rows per sub-tile) ----------------------------
        const int q = warp & 3;
        const int ms = (warp - 4) >> 2;            // warps 4..7 drain sub-tile 0, warps 8..11 sub-tile 1
        const int rl = q * 32 + lane;              // row inside the sub-tile
        int tcount = 0;
        bool ok = true;
        const uint32_t leader_tempty0 = map_to_cta(tempty0, 0);
        PairSegments segs(p.sk_per, nkb, pair, n_pairs, total_tiles);
        int tile, kb0, kb1; bool first;
        for (; ok && segs.next(tile, kb0, kb1, first); tcount++) {
            const int b = tile / tiles_per_batch, idx = tile - b * tiles_per_batch;
            const int mt = idx % mt_count, nt = idx / mt_count;
            const int which = EPI == GEPI_QKV_ROPE ? nt / nt_each : 0, ntl = nt - which * nt_each;
            const int buf = MSUB == 1 ? (tcount & 1) : 0, use = MSUB == 1 ? (tcount >> 1) : tcount;
            ok = mbar_wait(tfull0 + 8 * buf, use & 1, abort_flag);
            if (p.sk_per > 0) {
                // one decision for all epilogue warps of the CTA (they meet at named barrier 1 below); every
                // epilogue thread reaches this reducing barrier because the wait above is bounded
                uint32_t all_ok;
                asm volatile("{\n .reg .pred p, q;\n setp.ne.u32 q, %1, 0;\n bar.red.and.pred p, 1, %2, q;\n selp.u32 %0, 1, 0, p;\n}\n"
                             : "=r"(all_ok) : "r"((uint32_t)ok), "n"(EPI_THREADS) : "memory");
                ok = all_ok != 0;
            } else {
                ok = __all_sync(0xffffffffu, ok);
            }
            if (!ok) break;
            tc_fence_after();
            const int row = ((mt * 2 + (int)rank) * MSUB + ms) * BM + rl;
            const uint32_t tbase = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)((buf + ms) * BN);
            __half* crow = p.C + (long long)b * p.sC + (long long)row * p.ldc;
            // 32 finished accumulator columns of this thread's row -> the fused epilogue
            auto emit = [&](int c, const uint32_t* r) {
                const int col0 = ntl * BN + c;
                if (row >= p.M || col0 >= p.N) return;
                if (EPI == GEPI_RESIDUAL) {
                    store32_residual(crow + col0, p.R + (long long)row * p.ldr + col0, r);
                } else if (EPI == GEPI_QKV_ROPE) {
                    if (which == 2) {
                        store32(p.vc + (long long)row * p.ld_kv + col0, r);
                    } else {
                        const int half_dim = p.head_dim >> 1, d2 = (col0 % p.head_dim) >> 1;
                        __half* dst = which == 0 ? crow + col0 : p.kc + (long long)row * p.ld_kv + col0;
                        store32_rope(dst, p.cos_t + (long long)row * half_dim + d2, p.sin_t + (long long)row * half_dim + d2, r);
                    }
                } else {
                    store32(crow + col0, r);
                }
            };
            auto emit_swiglu = [&](int c, const uint32_t* g, const uint32_t* u) {
                const int col0 = ntl * OUT_COLS + c;
                if (row < p.M && col0 < p.N) store32_swiglu(crow + col0, g, u);
            };
            if (kb0 == 0 && kb1 == nkb) {
                if (EPI == GEPI_SWIGLU) {
#pragma unroll 1
                    for (int c = 0; c < OUT_COLS; c += 32) {
                        uint32_t g[32], u[32];
                        tmem_ld32(tbase + (uint32_t)c, g);
                        tmem_ld32(tbase + (uint32_t)(OUT_COLS + c), u);
                        tmem_ld_wait();
                        emit_swiglu(c, g, u);
                    }
                } else if (EPI == GEPI_RESIDUAL || (EPI == GEPI_QKV_ROPE && which < 2)) {
                    // the epilogue's own operands (residual row / rotary factors) of chunk c + 1 are fetched
                    // while chunk c is converted and stored
                    uint4 pre[4];                  // RESIDUAL: 64 bytes of the residual row; ROPE: 4 x (cos, sin) as uint2 pairs
                    const int half_dim = p.head_dim >> 1;
                    auto prefetch = [&](int c) {
                        const int col0 = ntl * BN + c;
                        if (row >= p.M || col0 >= p.N) return;
                        if (EPI == GEPI_RESIDUAL) {
                            load32_residual(pre, p.R + (long long)row * p.ldr + col0);
                        } else {
                            const int d2 = (col0 % p.head_dim) >> 1;
                            load32_rope(reinterpret_cast<uint2*>(pre), reinterpret_cast<uint2*>(pre) + 4,
                                        p.cos_t + (long long)row * half_dim + d2, p.sin_t + (long long)row * half_dim + d2);
                        }
                    };
                    prefetch(0);
#pragma unroll 1
                    for (int c = 0; c < BN; c += 32) {
                        uint32_t r[32];
                        tmem_ld32(tbase + (uint32_t)c, r);
                        uint4 cur[4] = {pre[0], pre[1], pre[2], pre[3]};
                        if (c + 32 < BN) prefetch(c + 32);
                        tmem_ld_wait();
                        const int col0 = ntl * BN + c;
                        if (row >= p.M || col0 >= p.N) continue;
                        if (EPI == GEPI_RESIDUAL) {
                            store32_residual_pre(crow + col0, cur, r);
                        } else {
                            __half* dst = which == 0 ? crow + col0 : p.kc + (long long)row * p.ld_kv + col0;
                            store32_rope_pre(dst, reinterpret_cast<const uint2*>(cur), reinterpret_cast<const uint2*>(cur) + 4, r);
                        }
                    }
                } else {
#pragma unroll 1
                    for (int c = 0; c < BN; c += 32) {
                        uint32_t r[32];
                        tmem_ld32(tbase + (uint32_t)c, r);
                        tmem_ld_wait();
                        emit(c, r);
                    }
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive_cluster(leader_tempty0 + 8 * buf);
                if (EPI == GEPI_STORE && p.push_rows > 0)
                    push_signal(p, ((mt * 2 + (int)rank) * MSUB + ms) * BM, ntl, 2 + ms, q == 0 && lane == 0);
                continue;
            }
            // ---- partial tile: fp32 partial to the workspace, last arriver of the tile half adds them up ----
            // slot layout [pair][first segment of the range ? 0 : 1][rank][sub-tile][column / 4][row][4 floats]:
            // a warp writes 512 contiguous bytes per instruction
            constexpr long long PART = (long long)BM * BN;      // floats of one sub-tile partial
            auto part_base = [&](int pr, int slot) { return p.sk_ws + ((((long long)pr * 2 + slot) * 2 + (long long)rank) * MSUB + ms) * PART; };
            {
                float4* dst = reinterpret_cast<float4*>(part_base(pair, first ? 0 : 1)) + rl;
#pragma unroll 1
                for (int c = 0; c < BN; c += 32) {
                    uint32_t r[32];
                    tmem_ld32(tbase + (uint32_t)c, r);
                    tmem_ld_wait();
#pragma unroll
                    for (int v = 0; v < 8; v++)
                        dst[(long long)(c / 4 + v) * BM] = make_float4(__uint_as_float(r[4 * v]), __uint_as_float(r[4 * v + 1]),
                                                                        __uint_as_float(r[4 * v + 2]), __uint_as_float(r[4 * v + 3]));
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(leader_tempty0 + 8 * buf);
            __threadfence();
            asm volatile("bar.sync 1, %0;" ::"n"(EPI_THREADS) : "memory");
            const int first_pair = (int)(((long long)tile * nkb) / p.sk_per);
            const int last_pair = (int)((((long long)tile + 1) * nkb - 1) / p.sk_per);
            if (warp == 4 && lane == 0) {
                unsigned int* cnt = p.sk_counters + (long long)tile * 2 + rank;
                const unsigned int old = atomicAdd(cnt, 1u);
                const int is_last = old == (unsigned)(last_pair - first_pair) ? 1 : 0;
                if (is_last) *cnt = 0;            // ready for the next launch
                *last_flag = is_last;
            }
            asm volatile("bar.sync 1, %0;" ::"n"(EPI_THREADS) : "memory");
            const bool is_last = *last_flag != 0;
            asm volatile("bar.sync 1, %0;" ::"n"(EPI_THREADS) : "memory");   // flag read by all before the next segment rewrites it
            if (!is_last) continue;
            __threadfence();
            // parts in k order (= pair order), each pair's slot by whether the tile holds the start of its range
            auto slot_of = [&](int pr) { return ((long long)pr * p.sk_per) / nkb == tile ? 0 : 1; };
            auto sum32 = [&](int c, uint32_t* r) {
                float acc[32];
#pragma unroll
                for (int i = 0; i < 32; i++) acc[i] = 0.f;
                // two parts per trip (one for SWIGLU, which holds two result chunks at once): 16 independent
                // 16-byte loads in flight per thread; the additions follow the part order either way
                constexpr int TRIP = EPI == GEPI_SWIGLU ? 1 : 2;
                for (int pr = first_pair; pr <= last_pair; pr += TRIP) {
                    const bool two = TRIP == 2 && pr + 1 <= last_pair;
                    const float4* src0 = reinterpret_cast<const float4*>(part_base(pr, slot_of(pr))) + rl;
                    const float4* src1 = two ? reinterpret_cast<const float4*>(part_base(pr + 1, slot_of(pr + 1))) + rl : src0;
                    float4 v0[8], v1[8];
#pragma unroll
                    for (int j = 0; j < 8; j++) v0[j] = __ldcg(src0 + (long long)(c / 4 + j) * BM);
                    if (two) {
#pragma unroll
                        for (int j = 0; j < 8; j++) v1[j] = __ldcg(src1 + (long long)(c / 4 + j) * BM);
                    }
#pragma unroll
                    for (int j = 0; j < 8; j++) { acc[4 * j] += v0[j].x; acc[4 * j + 1] += v0[j].y; acc[4 * j + 2] += v0[j].z; acc[4 * j + 3] += v0[j].w; }
                    if (two) {
#pragma unroll
                        for (int j = 0; j < 8; j++) { acc[4 * j] += v1[j].x; acc[4 * j + 1] += v1[j].y; acc[4 * j + 2] += v1[j].z; acc[4 * j + 3] += v1[j].w; }
                    }
                }
#pragma unroll
                for (int i = 0; i < 32; i++) r[i] = __float_as_uint(acc[i]);
            };
            if (EPI == GEPI_SWIGLU) {
#pragma unroll 1
                for (int c = 0; c < OUT_COLS; c += 32) {
                    uint32_t g[32], u[32];
                    sum32(c, g);
                    sum32(OUT_COLS + c, u);
                    emit_swiglu(c, g, u);
                }
            } else {
#pragma unroll 1
                for (int c = 0; c < BN; c += 32) {
                    uint32_t r[32];
                    sum32(c, r);
                    emit(c, r);
                }
            }
            if (EPI == GEPI_STORE && p.push_rows > 0)
                push_signal(p, ((mt * 2 + (int)rank) * MSUB + ms) * BM, ntl, 2 + ms, q == 0 && lane == 0);
        }
    }
    // ---------------- teardown: nobody frees TMEM or leaves while the pair may still use it -----------
    tc_fence_before();
    __syncthreads();
    __syncwarp();
    cluster_sync_all();
    if (warp == 2) {
        tc_fence_after();
        tmem_dealloc_pair<TMEM_COLS>(tmem_base);
    }
    if (threadIdx.x == 0 && *abort_flag) atomicExch(p.status, TL_ERR_TIMEOUT);
}

// ---- host side: tensor maps --------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn g_encode = nullptr;
std::once_flag g_encode_once;

EncodeTiledFn encode_fn() {
    std::call_once(g_encode_once, [] {
        void* fn = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            g_encode = reinterpret_cast<EncodeTiledFn>(fn);
    });
    return g_encode;
}

}  // namespace

bool tensor_map_encode_available() { return encode_fn() != nullptr; }

namespace {
int encode_tensor_map_f16(CUtensorMap* map, const __half* base, int rows, int K, long long ld, long long stride,
                          int batch, int box_rows) {
    EncodeTiledFn enc = encode_fn();
    if (!enc) return set_error(TL_ERR_UNSUPPORTED, "cuTensorMapEncodeTiled is not available from this driver");
    const bool batched = stride != 0 && batch > 1;
    cuuint64_t dims[3] = {(cuuint64_t)K, (cuuint64_t)rows, (cuuint64_t)(batched ? batch : 1)};
    cuuint64_t strides[2] = {(cuuint64_t)ld * 2, (cuuint64_t)(batched ? stride : (long long)rows * ld) * 2};
    cuuint32_t box[3] = {(cuuint32_t)BK, (cuuint32_t)box_rows, 1};
    cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, const_cast<__half*>(base), dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return set_error(TL_ERR_CUDA, "cuTensorMapEncodeTiled failed with code %d", (int)r);
    return TL_OK;
}

// Encoded maps are kept per (address, shape, pitches, box): a descriptor is a pure function of those, so a hit is
// always valid, and the model's weights, caches and activation buffers are encoded once instead of on every launch
// (an encode costs the host about a microsecond, two or three per launch).
struct MapKey {
    const void* base; long long ld, stride; int rows, K, batch, box_rows;
    bool operator==(const MapKey& o) const {
        return base == o.base && ld == o.ld && stride == o.stride && rows == o.rows && K == o.K && batch == o.batch && box_rows == o.box_rows;
    }
};
struct MapKeyHash {
    size_t operator()(const MapKey& k) const {
        size_t h = reinterpret_cast<uintptr_t>(k.base) * 0x9E3779B97F4A7C15ull;
        auto mix = [&](unsigned long long v) { h ^= v + 0x9E3779B97F4A7C15ull + (h << 6) + (h >> 2); };
        mix((unsigned long long)k.ld); mix((unsigned long long)k.stride); mix((unsigned long long)k.rows);
        mix((unsigned long long)k.K); mix((unsigned long long)k.batch); mix((unsigned long long)k.box_rows);
        return h;
    }
};
std::mutex g_map_mutex;
std::unordered_map<MapKey, CUtensorMap, MapKeyHash> g_map_cache;
constexpr size_t MAP_CACHE_LIMIT = 8192;      // entries; the cache is simply emptied when it gets there

}  // namespace

int make_tensor_map_f16(CUtensorMap* map, const __half* base, int rows, int K, long long ld, long long stride,
                        int batch, int box_rows) {
    const MapKey key{base, ld, stride, rows, K, batch, box_rows};
    {
        std::lock_guard<std::mutex> lock(g_map_mutex);
        auto it = g_map_cache.find(key);
        if (it != g_map_cache.end()) { *map = it->second; return TL_OK; }
    }
    TL_PROPAGATE(encode_tensor_map_f16(map, base, rows, K, ld, stride, batch, box_rows));
    std::lock_guard<std::mutex> lock(g_map_mutex);
    if (g_map_cache.size() >= MAP_CACHE_LIMIT) g_map_cache.clear();
    g_map_cache.emplace(key, *map);
    return TL_OK;
}


namespace {

template <int BN, int EPI>
int launch_k(const CUtensorMap& ma, const CUtensorMap& mb, const CUtensorMap& mb2, const CUtensorMap& mb3,
             const GemmArgs& a, int tiles, cudaStream_t st) {
    constexpr size_t smem = (size_t)STAGES * (A_BYTES + BN * BK * 2) + 1024 + 256;
    static PerDeviceOnce once;
    if (once.needed()) {
        TL_CUDA(cudaFuncSetAttribute(k_hgemm<BN, EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    }
    const int grid = std::max(1, std::min(tiles, sm_count()));
    return launch_pdl(k_hgemm<BN, EPI>, dim3(grid), dim3(GEMM_THREADS), smem, st, true, ma, mb, mb2, mb3, a);
}
template <int EPI>
int launch_any_bn(int bn, const CUtensorMap& ma, const CUtensorMap& mb, const CUtensorMap& mb2, const CUtensorMap& mb3,
                  const GemmArgs& a, int tiles, cudaStream_t st) {
    if (bn == 256) return launch_k<256, EPI>(ma, mb, mb2, mb3, a, tiles, st);
    if (bn == 128) return launch_k<128, EPI>(ma, mb, mb2, mb3, a, tiles, st);
    return launch_k<64, EPI>(ma, mb, mb2, mb3, a, tiles, st);
}

template <int BN, int KS, int MSUB, int EPI>
int launch_splitk_cfg(const CUtensorMap& ma, const CUtensorMap& mb, const GemmArgs& a, int tiles, cudaStream_t st) {
    static PerDeviceOnce once;
    if (once.needed()) {
        TL_CUDA(cudaFuncSetAttribute(k_hgemm_splitk<BN, KS, MSUB, EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SplitCfg<BN, KS, MSUB>::SMEM));
    }
    return launch_pdl(k_hgemm_splitk<BN, KS, MSUB, EPI>, dim3(tiles * KS), dim3(GEMM_THREADS), SplitCfg<BN, KS, MSUB>::SMEM, st, true, ma, mb, a);
}
template <int EPI>
int launch_splitk(int bn, int ks, int msub, const CUtensorMap& ma, const CUtensorMap& mb, const GemmArgs& a, int tiles, cudaStream_t st) {
    if (msub == 1) {
        if (bn == 128 && ks == 4) return launch_splitk_cfg<128, 4, 1, EPI>(ma, mb, a, tiles, st);
        if (bn == 128 && ks == 2) return launch_splitk_cfg<128, 2, 1, EPI>(ma, mb, a, tiles, st);
        if (bn == 256 && ks == 2) return launch_splitk_cfg<256, 2, 1, EPI>(ma, mb, a, tiles, st);
    }
    TL_REQUIRE(false, "hgemm split-K: no kernel for tile %d x %d, split %d", 128 * msub, bn, ks);
    return TL_ERR_UNSUPPORTED;
}

template <int EPI, int MSUB>
int launch_pair_cfg(const CUtensorMap& ma, const CUtensorMap& mb, const CUtensorMap& mb2, const CUtensorMap& mb3,
                    const GemmArgs& a, int pair_tiles, cudaStream_t st) {
    static PerDeviceOnce once;
    if (once.needed()) {
        TL_CUDA(cudaFuncSetAttribute(k_hgemm_pair<EPI, MSUB>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)PairCfg<MSUB>::SMEM));
    }
    const int grid = 2 * std::max(1, std::min(pair_tiles, sm_count() / 2));
    return launch_pdl(k_hgemm_pair<EPI, MSUB>, dim3(grid), dim3(PairCfg<MSUB>::THREADS), PairCfg<MSUB>::SMEM, st, true, ma, mb, mb2, mb3, a);
}
// estimated plan of the CTA-pair kernel: tile height (msub x 256 rows), whole tiles (sk_per = 0) or stream-K
// ranges of sk_per k-blocks per pair, and the estimated cycles of the launch
struct PairPlan { int msub, sk_per; long long cost; };
PairPlan pair_plan(int sms, int M, long long n_col_tiles, int nkb, int epi);

// workspace of the stream-K mode per (device, stream): partial tiles of every pair (two per pair, fp32)
// and the arrival counters (zero between launches: the last arriver of a tile resets its counter)
struct SkWorkspace { float* ws; unsigned int* counters; };
constexpr int SK_MAX_PAIRS = 128, SK_MAX_TILES = 1 << 16;
std::mutex g_sk_mutex;
std::unordered_map<unsigned long long, SkWorkspace> g_sk_ws;
int sk_workspace_for(cudaStream_t st, SkWorkspace* out) {
    int dev = 0;
    TL_CUDA(cudaGetDevice(&dev));
    const unsigned long long key = (unsigned long long)reinterpret_cast<uintptr_t>(st) * 64ull + (unsigned long long)dev;
    std::lock_guard<std::mutex> lock(g_sk_mutex);
    auto it = g_sk_ws.find(key);
    if (it == g_sk_ws.end()) {
        SkWorkspace w;
        // [pair][2 slots][2 ranks][up to 2 sub-tiles][128 x 256] floats
        TL_CUDA(cudaMalloc(&w.ws, (size_t)SK_MAX_PAIRS * 2 * 2 * 2 * BM * PAIR_BN * sizeof(float)));
        TL_CUDA(cudaMalloc(&w.counters, (size_t)2 * SK_MAX_TILES * sizeof(unsigned int)));
        TL_CUDA(cudaMemset(w.counters, 0, (size_t)2 * SK_MAX_TILES * sizeof(unsigned int)));
        TL_CUDA(cudaDeviceSynchronize());
        it = g_sk_ws.emplace(key, w).first;
    }
    *out = it->second;
    return TL_OK;
}

// `n_col_tiles` = column tiles per batch
template <int EPI>
int launch_pair(const CUtensorMap& ma, const CUtensorMap& mb, const CUtensorMap& mb2, const CUtensorMap& mb3,
                const GemmArgs& a_in, int n_col_tiles, cudaStream_t st) {
    GemmArgs a = a_in;
    const long long nt = (long long)n_col_tiles * a.batch;
    const int nkb = (a.K + BK - 1) / BK;
    PairPlan pl = pair_plan(sm_count(), a.M, nt, nkb, EPI);
    const long long tiles = (long long)((a.M + 256 * pl.msub - 1) / (256 * pl.msub)) * nt;
    int pair_ctas = (int)std::min<long long>(tiles, sm_count() / 2);
    if (pl.sk_per > 0) {
        SkWorkspace w;
        TL_PROPAGATE(sk_workspace_for(st, &w));
        a.sk_per = pl.sk_per; a.sk_ws = w.ws; a.sk_counters = w.counters;
        pair_ctas = (int)((tiles * nkb + pl.sk_per - 1) / pl.sk_per);
    }
    if (pl.msub == 2) return launch_pair_cfg<EPI, 2>(ma, mb, mb2, mb3, a, pair_ctas, st);
    return launch_pair_cfg<EPI, 1>(ma, mb, mb2, mb3, a, pair_ctas, st);
}

inline bool al16(const void* q) { return (reinterpret_cast<uintptr_t>(q) & 15) == 0; }

// the planning functions below take the SM count they plan for: the device's for a launch, the caller's for a
// host-only plan query

// Estimated cycles of the CTA-pair kernel. Per k-block a 256 x 256 pair tile measures ~590 cycles (512 of
// MMA stretched by the shared-memory fill running at its limit beside them), a 512 x 256 tile ~1090
// (1024 of MMA, the fill no longer the limit). Whole tiles cost rounds-of-tiles-over-the-pairs x k-blocks
// x that; stream-K ranges cost ceil(tiles x k-blocks / pairs) x that plus the exchange of the partial
// tiles (~4000 cycles per part and 256 rows of tile height: a partial goes out to L2 and the last
// arriver reads every part back).
// The 512-row tile has no second accumulator buffer, so its epilogue is not hidden behind the next
// tile's MMAs. The rotary epilogue (per-row factor loads, three destinations) is long enough that the
// 256-row tile with its hidden epilogue wins for the fused QKV projection (2048 tokens of the 7B model:
// 1.7 ms of 24.5 over 32 layers); the other epilogues gain from the larger tile.
// TL_HGEMM_PAIR=always|always512|streamk|streamk512|never overrides the estimate (tests force every
// kernel onto small shapes)
int pair_forced() {
    static const int forced = [] {
        const char* e = getenv("TL_HGEMM_PAIR");
        if (!e) return 0;
        if (!strcmp(e, "always")) return 1;
        if (!strcmp(e, "never")) return 2;
        if (!strcmp(e, "always512")) return 3;
        if (!strcmp(e, "streamk")) return 4;
        if (!strcmp(e, "streamk512")) return 5;
        return 0;
    }();
    return forced;
}
PairPlan pair_plan(int sms, int M, long long n_col_tiles, int nkb, int epi) {
    const long long pairs = std::max(1, sms / 2);
    const int forced = pair_forced();
    PairPlan best{1, 0, -1};
    for (int msub = 1; msub <= 2; msub++) {
        if (forced == 1 || forced == 4) { if (msub != 1) continue; }
        else if (forced == 3 || forced == 5) { if (msub != 2) continue; }
        else if (epi == GEPI_QKV_ROPE && msub == 2) continue;
        const long long tiles = (long long)((M + 256 * msub - 1) / (256 * msub)) * n_col_tiles;
        const long long c = msub == 1 ? 590 : 1090;
        if (forced != 4 && forced != 5) {
            // epilogues the MMAs cannot hide: the last tile's (~4000 cycles for 256 rows, ~8000 for 512), and for the
            // 512-row tile, which has no second accumulator buffer, ~3500 more per earlier round. Measured at
            // M = 2048, N = 4096: 256-row tiles win up to K ~ 2700 (K = 1024: 19.2 against 21.1 us), 512-row above
            // (K = 5504: 67.3 against 70.8 us).
            const long long rounds = (tiles + pairs - 1) / pairs;
            const long long cost = rounds * nkb * c + (msub == 2 ? (rounds - 1) * 3500 + 8000 : 4000);
            if (best.cost < 0 || cost < best.cost) best = PairPlan{msub, 0, cost};
        }
        if (tiles <= SK_MAX_TILES && pairs <= SK_MAX_PAIRS && forced != 1 && forced != 3) {
            const long long per = (tiles * nkb + pairs - 1) / pairs;
            const long long parts = (nkb + per - 1) / per + 1;
            const long long cost = per * c + 4000 * msub * (parts + 1);
            // Stream-K only where whole tiles leave most pairs idle for a long K loop (or where a test asks
            // for it). On the Llama2-7B shapes it measured slower than whole tiles: the fp32 partial tiles
            // (256 to 512 KB each) add ~150 MB of traffic to a 50 MB problem at M = 2048, 4096 x 4096
            // (70 us against 52 us), and M = 512 came out between -10 % and +8 %.
            const bool regime = 2 * tiles <= pairs && nkb >= 256 && best.cost >= 0 && cost * 100 < best.cost * 70;
            if (forced == 4 || forced == 5 || regime) best = PairPlan{msub, (int)per, cost};
        }
    }
    return best;
}
// estimated cycles of the pair kernel for the choice between it and the single-CTA kernel
long long pair_cost(int sms, int M, int n_tiles_256, int batch, int K, int epi = GEPI_STORE) {
    const int forced = pair_forced();
    if (forced == 2) return (1ll << 60);
    if (forced != 0) return -1;
    return pair_plan(sms, M, (long long)n_tiles_256 * batch, (K + BK - 1) / BK, epi).cost;
}
// estimated cycles of the single-CTA kernel
long long single_cost(int sms, int mt, int N, int batch, int bn, int K) {
    const long long tiles = (long long)mt * ((N + bn - 1) / bn) * batch;
    const long long waves = (tiles + sms - 1) / sms;
    return waves * std::max<long long>(2 * bn, (16384 + bn * 128) / 64) * ((K + BK - 1) / BK);
}

// Estimated plan of the one-tile-per-cluster kernel ((128 msub) x bn tile, K split over ks CTAs): only where
// every cluster is resident at once; cost = k-blocks per CTA x the cost of a k-block (the larger of MMA time and
// shared-memory fill, as for the single-CTA kernel; the 256 x 256 tile is MMA-bound at 1024 cycles) + the exchange
// of the partial slices over distributed shared memory and the cluster barriers + the unhidden epilogue.
// TL_HGEMM_SPLITK=never|always overrides the comparison with the other kernels.
struct SplitPlan { int bn, ks, msub; long long cost; };
int splitk_forced() {
    static const int forced = [] {
        const char* e = getenv("TL_HGEMM_SPLITK");
        if (!e) return 0;
        return !strcmp(e, "never") ? 2 : (!strcmp(e, "always") ? 1 : 0);
    }();
    return forced;
}
SplitPlan splitk_plan(int sms, int M, int N, int K, int batch) {
    SplitPlan best{0, 0, 0, -1};
    if (batch != 1 || splitk_forced() == 2 || N % 32 != 0) return best;
    const int nkb = (K + BK - 1) / BK;
    // (the 256 x 256 tile per CTA, msub = 2, measured slower: 28.3 us against 20.1 us at M = 512, 4096 x 4096 with the
    // split 4 against 128 x 256 tiles with the split 2 - the exchange moves 192 KB per CTA through four epilogue warps)
    static const int cand[3][3] = {{128, 4, 1}, {128, 2, 1}, {256, 2, 1}};
    for (const auto& c : cand) {
        const int bn = c[0], ks = c[1], msub = c[2];
        if (msub == 2 && M <= BM) continue;
        const long long tiles = (long long)((M + BM * msub - 1) / (BM * msub)) * ((N + bn - 1) / bn);
        if (tiles * ks > sms || nkb / ks < 4) continue;
        const long long per_kb = msub == 2 ? 1040 : std::max<long long>(2 * bn, (16384 + bn * 128) / 64);
        const long long cost = (long long)((nkb + ks - 1) / ks) * per_kb + (ks > 1 ? 3000 * msub : 0) + 1500 * msub;
        if (best.cost < 0 || cost < best.cost) best = SplitPlan{bn, ks, msub, cost};
    }
    return best;
}

int pick_bn(int sms, int mt, int N, int batch);
// the cluster split-K kernel where it has a plan and the estimate beats the whole-tile kernels
bool splitk_wins(int sms, int M, int N, int K, int batch, int epi, SplitPlan* out) {
    const SplitPlan sp = splitk_plan(sms, M, N, K, batch);
    *out = sp;
    if (sp.cost < 0) return false;
    if (splitk_forced() == 1) return true;
    const int mt = (M + BM - 1) / BM;
    // the whole-tile estimates leave out their last tile's epilogue: ask for a clear margin before displacing them
    if (sp.cost * 10 >= single_cost(sms, mt, N, batch, pick_bn(sms, mt, N, batch), K) * 9) return false;
    return M <= BM || sp.cost * 10 < pair_cost(sms, M, (N + 255) / 256, batch, K, epi) * 9;
}

// N-tile width with the smallest estimated time: waves of tiles over the SMs times the cost of one
// k-block of a tile, which is the larger of its MMA time (2 cycles per accumulator column) and
// the time to bring its operands into shared memory (16 KB of A + BN * 128 B of B at the roughly
// 64 bytes per cycle one SM sustains from L2; measured: the 128x256 tile runs the tensor pipe
// at 69 %, i.e. it is fill-bound, 48 KB per 512 MMA cycles).
int pick_bn(int sms, int mt, int N, int batch) {
    int best = 256;
    long long best_cost = -1;
    for (int bn = 256; bn >= 64; bn >>= 1) {
        const long long tiles = (long long)mt * ((N + bn - 1) / bn) * batch;
        const long long waves = (tiles + sms - 1) / sms;
        const long long per_kb = std::max<long long>(2 * bn, (16384 + bn * 128) / 64);
        const long long cost = waves * per_kb;
        if (best_cost < 0 || cost < best_cost) { best = bn; best_cost = cost; }
    }
    return best;
}

}  // namespace

// Up to 32 rows the skinny kernel (32-row tiles, mma.sync, no tensor-memory set-up) measured 0.6 to 2.5 us faster
// on the 7B shapes; from 33 rows on the cluster kernel wins (128 rows: 13.6 / 26.1 / 23.0 us against 15.7 / 30.1 / 25.6).
bool hgemm_splitk_preferred(int M, int N, int K) {
    SplitPlan sp;
    return (M > 32 || splitk_forced() == 1) && splitk_wins(sm_count(), M, N, K, 1, GEPI_STORE, &sp);
}

void hgemm_plan(int M, int N, int K, int batch, int sms, int* kind, int* bn, int* sk_per) {
    const int mt = (M + BM - 1) / BM;
    *bn = pick_bn(sms, mt, N, batch);
    *sk_per = 0;
    SplitPlan sp;
    if (N % 32 == 0 && splitk_wins(sms, M, N, K, batch, GEPI_STORE, &sp)) {
        *kind = 3;                        // one 128-row tile per cluster; sk_per = CTAs sharing the tile's K
        *bn = sp.bn;
        *sk_per = sp.ks;
        return;
    }
    *kind = (M > BM && N % 32 == 0 && pair_cost(sms, M, (N + 255) / 256, batch, K) < single_cost(sms, mt, N, batch, *bn, K)) ? 1 : 0;
    if (*kind == 1) {                     // 1: 256-row pair tiles, 2: 512-row pair tiles
        const PairPlan pl = pair_plan(sms, M, (long long)((N + 255) / 256) * batch, (K + BK - 1) / BK, GEPI_STORE);
        *bn = 256;
        *kind = pl.msub;
        *sk_per = pl.sk_per;
    }
}

bool hgemm_supported(const void* A, const void* B, const void* C, size_t M, size_t N, size_t K, size_t lda,
                     size_t ldb, size_t ldc) {
    (void)C; (void)ldc;
    return M >= 1 && N >= 1 && K >= 8 && lda % 8 == 0 && ldb % 8 == 0 && al16(A) && al16(B) && encode_fn() != nullptr;
}

int launch_hgemm(const __half* A, const __half* B, __half* C, int batch, int M, int N, int K, long long lda,
                 long long ldb, long long ldc, long long sA, long long sB, long long sC, cudaStream_t st, bool weights_constant) {
    TL_REQUIRE(hgemm_supported(A, B, C, M, N, K, lda, ldb, ldc), "hgemm: unsupported shape or alignment");
    TL_REQUIRE(sA % 8 == 0 && sB % 8 == 0, "hgemm: batch strides must be multiples of 8 elements");
    if (batch <= 0) return TL_OK;
    const int mt = (M + BM - 1) / BM;
    const int bn = pick_bn(sm_count(), mt, N, batch);
    GemmArgs a{};
    a.C = C; a.M = M; a.N = N; a.K = K; a.batch = batch; a.ldc = ldc; a.sC = sC;
    a.a_batched = (sA != 0 && batch > 1) ? 1 : 0; a.b_batched = (sB != 0 && batch > 1) ? 1 : 0;
    a.b_const = weights_constant ? 1 : 0;
    a.status = device_status_word();
    CUtensorMap ma, mb;
    TL_PROPAGATE(make_tensor_map_f16(&ma, A, M, K, lda, sA, batch, BM));
    const bool vec_c = ldc % 8 == 0 && sC % 8 == 0 && al16(C) && N % 32 == 0;   // the pair epilogue stores 64-byte chunks
    SplitPlan sp;
    if (vec_c && splitk_wins(sm_count(), M, N, K, batch, GEPI_STORE, &sp)) {
        TL_PROPAGATE(make_tensor_map_f16(&mb, B, N, K, ldb, 0, 1, sp.bn));
        return launch_splitk<GEPI_STORE>(sp.bn, sp.ks, sp.msub, ma, mb, a, ((M + BM * sp.msub - 1) / (BM * sp.msub)) * ((N + sp.bn - 1) / sp.bn), st);
    }
    if (M > BM && vec_c && pair_cost(sm_count(), M, (N + 255) / 256, batch, K) < single_cost(sm_count(), mt, N, batch, bn, K)) {
        TL_PROPAGATE(make_tensor_map_f16(&mb, B, N, K, ldb, sB, batch, 128));
        return launch_pair<GEPI_STORE>(ma, mb, mb, mb, a, (N + 255) / 256, st);
    }
    TL_PROPAGATE(make_tensor_map_f16(&mb, B, N, K, ldb, sB, batch, bn));
    const int tiles = mt * ((N + bn - 1) / bn) * batch;
    return launch_any_bn<GEPI_STORE>(bn, ma, mb, mb, mb, a, tiles, st);
}

// K-split matmul of the tensor-parallel prefill: C is this rank's partial result; the rank that owns a block of
// rows (m / rows_per_owner) is told through a flag per (128-row block, column tile) when it may fetch it.
int launch_hgemm_push(const __half* A, const __half* B, __half* C, int M, int N, int K, long long lda, long long ldb,
                      const HgemmPush& push, int* col_tiles, cudaStream_t st) {
    TL_REQUIRE(hgemm_supported(A, B, C, M, N, K, lda, ldb, N) && N % 32 == 0 && al16(C), "hgemm push: unsupported shape or alignment");
    TL_REQUIRE(push.world >= 2 && push.world <= 8 && push.rows_per_owner > 0 && push.rows_per_owner % 128 == 0 &&
               (long long)push.rows_per_owner * push.world >= M, "hgemm push: rows per owner must be a multiple of 128 covering M");
    const int mt = (M + BM - 1) / BM;
    const int bn = pick_bn(sm_count(), mt, N, 1);
    GemmArgs a{};
    a.C = C; a.M = M; a.N = N; a.K = K; a.batch = 1; a.ldc = N; a.sC = 0;
    a.status = device_status_word();
    a.push_rows = push.rows_per_owner; a.push_epoch = push.epoch;
    for (int r = 0; r < 8; r++) {
        a.push_flags[r] = r < push.world ? push.flags[r] : nullptr;
        if (r < push.world) TL_REQUIRE(push.flags[r] != nullptr, "hgemm push: bad destination");
    }
    CUtensorMap ma, mb;
    TL_PROPAGATE(make_tensor_map_f16(&ma, A, M, K, lda, 0, 1, BM));
    if (M > BM && pair_cost(sm_count(), M, (N + 255) / 256, 1, K) < single_cost(sm_count(), mt, N, 1, bn, K)) {
        TL_PROPAGATE(make_tensor_map_f16(&mb, B, N, K, ldb, 0, 1, 128));
        *col_tiles = (N + 255) / 256;
        TL_REQUIRE(*col_tiles <= PUSH_MAX_COL_TILES, "hgemm push: too many column tiles");
        return launch_pair<GEPI_STORE>(ma, mb, mb, mb, a, (N + 255) / 256, st);
    }
    TL_PROPAGATE(make_tensor_map_f16(&mb, B, N, K, ldb, 0, 1, bn));
    *col_tiles = (N + bn - 1) / bn;
    TL_REQUIRE(*col_tiles <= PUSH_MAX_COL_TILES, "hgemm push: too many column tiles");
    return launch_any_bn<GEPI_STORE>(bn, ma, mb, mb, mb, a, mt * *col_tiles, st);
}

// The fused forms need full 32-column chunks and 16-byte aligned rows everywhere.
bool hgemm_fused_supported(const void* A, const void* B, const void* C, size_t M, size_t N, size_t K, size_t lda,
                           size_t ldb, size_t ldc) {
    return hgemm_supported(A, B, C, M, N, K, lda, ldb, ldc) && N % 32 == 0 && ldc % 8 == 0 && al16(C);
}

// C = half(A B^T) + R
int launch_hgemm_residual(const __half* A, const __half* B, const __half* R, __half* C, int M, int N, int K,
                          long long lda, long long ldb, long long ldr, long long ldc, cudaStream_t st, bool weights_constant) {
    TL_REQUIRE(hgemm_fused_supported(A, B, C, M, N, K, lda, ldb, ldc) && R && al16(R) && ldr % 8 == 0,
               "hgemm+residual: unsupported shape or alignment");
    const int mt = (M + BM - 1) / BM;
    const int bn = pick_bn(sm_count(), mt, N, 1);
    CUtensorMap ma, mb;
    TL_PROPAGATE(make_tensor_map_f16(&ma, A, M, K, lda, 0, 1, BM));
    GemmArgs a{};
    a.C = C; a.M = M; a.N = N; a.K = K; a.batch = 1; a.ldc = ldc; a.status = device_status_word();
    a.R = R; a.ldr = ldr; a.b_const = weights_constant ? 1 : 0;
    SplitPlan sp;
    if (splitk_wins(sm_count(), M, N, K, 1, GEPI_RESIDUAL, &sp)) {
        TL_PROPAGATE(make_tensor_map_f16(&mb, B, N, K, ldb, 0, 1, sp.bn));
        return launch_splitk<GEPI_RESIDUAL>(sp.bn, sp.ks, sp.msub, ma, mb, a, ((M + BM * sp.msub - 1) / (BM * sp.msub)) * ((N + sp.bn - 1) / sp.bn), st);
    }
    if (M > BM && pair_cost(sm_count(), M, (N + 255) / 256, 1, K, GEPI_RESIDUAL) < single_cost(sm_count(), mt, N, 1, bn, K)) {
        TL_PROPAGATE(make_tensor_map_f16(&mb, B, N, K, ldb, 0, 1, 128));
        return launch_pair<GEPI_RESIDUAL>(ma, mb, mb, mb, a, (N + 255) / 256, st);
    }
    TL_PROPAGATE(make_tensor_map_f16(&mb, B, N, K, ldb, 0, 1, bn));
    return launch_any_bn<GEPI_RESIDUAL>(bn, ma, mb, mb, mb, a, mt * ((N + bn - 1) / bn), st);
}

// C[M, N] = silu(A W1^T) * (A W3^T); W1, W3: [N, K]
int launch_hgemm_swiglu(const __half* A, const __half* W1, const __half* W3, __half* C, int M, int N, int K,
                        long long lda, long long ldb, long long ldc, cudaStream_t st) {
    TL_REQUIRE(hgemm_fused_supported(A, W1, C, M, N, K, lda, ldb, ldc) && W3 && al16(W3),
               "hgemm+swiglu: unsupported shape or alignment");
    const int mt = (M + BM - 1) / BM, nt = (N + 127) / 128;
    CUtensorMap ma, m1, m3;
    TL_PROPAGATE(make_tensor_map_f16(&ma, A, M, K, lda, 0, 1, BM));
    TL_PROPAGATE(make_tensor_map_f16(&m1, W1, N, K, ldb, 0, 1, 128));
    TL_PROPAGATE(make_tensor_map_f16(&m3, W3, N, K, ldb, 0, 1, 128));
    GemmArgs a{};
    a.C = C; a.M = M; a.N = N; a.K = K; a.batch = 1; a.ldc = ldc; a.status = device_status_word();
    if (M > BM && pair_cost(sm_count(), M, nt, 1, K, GEPI_SWIGLU) < single_cost(sm_count(), mt, N, 1, 128, K) * 768 / 512)   // single: 128 output columns per 256-wide tile
        return launch_pair<GEPI_SWIGLU>(ma, m1, m3, m3, a, nt, st);
    return launch_k<256, GEPI_SWIGLU>(ma, m1, m3, m3, a, mt * nt, st);
}

// q[M, n_each] = rope(A Wq^T) -> q_out; rope(A Wk^T) -> k_rows; A Wv^T -> v_rows. Row t of k_rows /
// v_rows / cos_rows / sin_rows belongs to the position of token t (the caller offsets the bases).
int launch_hgemm_qkv_rope(const __half* A, const __half* Wq, const __half* Wk, const __half* Wv, __half* q_out,
                          __half* k_rows, __half* v_rows, int M, int n_each, int K, long long lda, long long ldb,
                          long long ldq, long long ld_kv, const __half* cos_rows, const __half* sin_rows,
                          int head_dim, cudaStream_t st) {
    TL_REQUIRE(hgemm_fused_supported(A, Wq, q_out, M, n_each, K, lda, ldb, ldq) && al16(Wk) && al16(Wv) &&
                   al16(k_rows) && al16(v_rows) && ld_kv % 8 == 0 && head_dim % 32 == 0 && n_each % head_dim == 0 &&
                   n_each % 64 == 0 && cos_rows && sin_rows && (reinterpret_cast<uintptr_t>(cos_rows) & 7) == 0 &&
                   (reinterpret_cast<uintptr_t>(sin_rows) & 7) == 0,
               "hgemm+qkv+rope: unsupported shape or alignment");
    const int mt = (M + BM - 1) / BM;
    int bn = 256;
    while (bn > 64 && (n_each % bn != 0 || (long long)mt * 3 * (n_each / bn) < sm_count())) bn >>= 1;
    CUtensorMap ma, mq, mk, mv;
    TL_PROPAGATE(make_tensor_map_f16(&ma, A, M, K, lda, 0, 1, BM));
    if (M > BM && n_each % 256 == 0 && pair_cost(sm_count(), M, 3 * (n_each / 256), 1, K, GEPI_QKV_ROPE) < single_cost(sm_count(), mt, 3 * n_each, 1, bn, K)) {
        TL_PROPAGATE(make_tensor_map_f16(&mq, Wq, n_each, K, ldb, 0, 1, 128));
        TL_PROPAGATE(make_tensor_map_f16(&mk, Wk, n_each, K, ldb, 0, 1, 128));
        TL_PROPAGATE(make_tensor_map_f16(&mv, Wv, n_each, K, ldb, 0, 1, 128));
        GemmArgs a2{};
        a2.C = q_out; a2.M = M; a2.N = n_each; a2.K = K; a2.batch = 1; a2.ldc = ldq; a2.status = device_status_word();
        a2.kc = k_rows; a2.vc = v_rows; a2.ld_kv = ld_kv; a2.cos_t = cos_rows; a2.sin_t = sin_rows; a2.head_dim = head_dim;
        return launch_pair<GEPI_QKV_ROPE>(ma, mq, mk, mv, a2, 3 * (n_each / 256), st);
    }
    TL_PROPAGATE(make_tensor_map_f16(&mq, Wq, n_each, K, ldb, 0, 1, bn));
    TL_PROPAGATE(make_tensor_map_f16(&mk, Wk, n_each, K, ldb, 0, 1, bn));
    TL_PROPAGATE(make_tensor_map_f16(&mv, Wv, n_each, K, ldb, 0, 1, bn));
    GemmArgs a{};
    a.C = q_out; a.M = M; a.N = n_each; a.K = K; a.batch = 1; a.ldc = ldq; a.status = device_status_word();
    a.kc = k_rows; a.vc = v_rows; a.ld_kv = ld_kv; a.cos_t = cos_rows; a.sin_t = sin_rows; a.head_dim = head_dim;
    return launch_any_bn<GEPI_QKV_ROPE>(bn, ma, mq, mk, mv, a, mt * 3 * (n_each / bn), st);
}

}  // namespace tlb
