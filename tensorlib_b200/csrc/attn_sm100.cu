// Prefill attention for sm_100a: softmax(Q K^T / sqrt(hd) + causal mask) V in one kernel, scores
// never leave the SM. Replaces, for T > 1, the run of launches in Attention::forward
// (model/llama2_7b/src/Transformer.cpp:56-109): per-head matmul -> ScalarDiv -> mask add -> softmax
// -> per-head matmul, which the unfused path executes as two batched HGEMMs around a softmax over
// a materialised (heads, T, S) score tensor.
//
// One CTA per (head, 128 query rows); two CTAs per SM so that one CTA's softmax overlaps the
// other's MMAs. Inside a CTA, per 64-column KV tile j:
//   warp 0   TMA: Q once, K tiles (2 stages), V tiles (2 stages), 128-byte swizzle, zero fill
//   warp 1   tcgen05.mma: S[j&1] = Q K_j^T (TMEM, 64 fp32 columns), up to two tiles ahead of the softmax
//   warps 2-5  one query row per thread: tcgen05.ld the S row, mask, running max and sum (exp2
//            domain, scale folded into the exponent's FFMA), P as fp16 back into the first 32 columns
//            of the same S buffer (tcgen05.st). The accumulator is rescaled (tcgen05.ld/st) only
//            when the running max grew by more than 2^8 since the last rescale; P stays below 2^8.
//   warp 6   tcgen05.mma with the A operand in tensor memory: O += P_j V_j (TMEM, 128 columns); its
//            completion frees the V stage and the S/P buffer
// Two issuing threads because one thread's barrier waits, commits and fences per tile cost more
// than the tile's MMAs take, and an MMA issue blocks while the tensor core's short queue is full
// (measured: one issuer 49.5 us per 7B layer at T = 2048, two issuers 41.3 us).
// V is read in place from the cache: (kv, head_dim) rows are the N x K operand of the second MMA in
// MN-major form (head_dim contiguous), so no transposed copy exists.
// Bound: tensor pipe / MUFU (exp2), not HBM: 4 * T * S * hd flops per head against
// 2 * (T + 2 S) * hd bytes.
//
// Every mbarrier wait is bounded; on a timeout the CTA raises an abort flag, all roles leave
// their loops, TMEM is freed and TL_ERR_TIMEOUT is recorded in the device status word.
#include <cuda.h>

#include "kernels.cuh"
#include "sm100.cuh"

namespace tlb {

namespace {

using namespace sm100;

constexpr int BQ = 128, BKV = 64, HD = 128;
constexpr int FA_THREADS = 224;     // TMA, S issuer, 4 softmax warps, P.V issuer
constexpr int Q_BYTES = BQ * HD * 2;          // two swizzle atoms of 64 columns
constexpr int K_BYTES = BKV * HD * 2;         // two atoms, 64 rows each
constexpr int V_BYTES = BKV * HD * 2;         // V tile as stored: 64 kv rows, two 64-column halves
constexpr int K_STAGES = 2, V_STAGES = 2;
constexpr uint32_t TMEM_COLS = 256;           // S0 | S1 (64 each) | O (128)
constexpr uint32_t S_COL = 0, O_COL = 128;
constexpr float RESCALE_THRESHOLD = 8.0f;     // log2 units

struct FlashArgs {
    __half* out;            // (T, heads * hd) row pitch ldo
    long long ldo;
    int T, S, pos0, heads;
    float scale_log2;       // log2(e) / sqrt(hd)
    int* status;
};

__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

__global__ void __launch_bounds__(FA_THREADS, 2)
k_flash_prefill(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                const __grid_constant__ CUtensorMap tmV, FlashArgs p) {
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    unsigned char* sQ = smem;
    unsigned char* sK = sQ + Q_BYTES;
    unsigned char* sV = sK + K_STAGES * K_BYTES;
    uint64_t* bars = reinterpret_cast<uint64_t*>(sV + V_STAGES * V_BYTES);
    // barriers: 0 q_full | 1,2 k_full | 3,4 k_empty | 5,6 v_full | 7,8 pv_done | 9,10 s_full | 11,12 p_full
    const uint32_t bar0 = smem_u32(bars);
    auto BAR = [&](int i) { return bar0 + 8u * (uint32_t)i; };
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 13);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int head = blockIdx.x;
    const int qt = (int)gridDim.y - 1 - (int)blockIdx.y;      // heaviest (latest) query tiles first
    const int q0 = qt * BQ;
    // causal: the last row of the tile sees columns 0 .. pos0 + min(q0 + BQ, T) - 1
    const int last_col = min(p.S, p.pos0 + min(q0 + BQ, p.T)) - 1;
    const int n_tiles = last_col / BKV + 1;

    if (threadIdx.x == 0) {
        mbar_init(BAR(0), 1);
        mbar_init(BAR(1), 1); mbar_init(BAR(2), 1); mbar_init(BAR(3), 1); mbar_init(BAR(4), 1);
        mbar_init(BAR(5), 1); mbar_init(BAR(6), 1); mbar_init(BAR(7), 1); mbar_init(BAR(8), 1);
        mbar_init(BAR(9), 1); mbar_init(BAR(10), 1);
        mbar_init(BAR(11), 4); mbar_init(BAR(12), 4);       // one arrival per softmax warp, after all its lanes stored their P rows
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) tmem_alloc<TMEM_COLS>(tmem_slot);
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
        asm volatile("prefetch.tensormap [%0];" ::"l"(&tmQ) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&tmK) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&tmV) : "memory");
        mbar_arrive_expect_tx(BAR(0), Q_BYTES);
        tma_load_3d(smem_u32(sQ), &tmQ, 0, q0, head, BAR(0));
        tma_load_3d(smem_u32(sQ) + Q_BYTES / 2, &tmQ, 64, q0, head, BAR(0));
        bool ok = true;
        int k_issued = 0, v_issued = 0;
        auto issue_k = [&](int t) -> bool {
            const int ks = t & 1;
            if (t >= K_STAGES && !mbar_wait(BAR(3 + ks), ((t >> 1) - 1) & 1, abort_flag)) return false;
            const uint32_t dk = smem_u32(sK + ks * K_BYTES);
            mbar_arrive_expect_tx(BAR(1 + ks), K_BYTES);
            tma_load_3d(dk, &tmK, 0, t * BKV, head, BAR(1 + ks));
            tma_load_3d(dk + K_BYTES / 2, &tmK, 64, t * BKV, head, BAR(1 + ks));
            k_issued++;
            return true;
        };
        ok = issue_k(0);
        for (int j = 0; j < n_tiles && ok; j++) {
            // K runs one tile ahead of V: its stage frees as soon as the scores of tile j-1 exist
            if (j + 1 < n_tiles && !(ok = issue_k(j + 1))) break;
            const int vs = j & 1;
            if (j >= V_STAGES && !(ok = mbar_wait(BAR(7 + vs), ((j >> 1) - 1) & 1, abort_flag))) break;   // P.V of tile j-2 has read this stage
            const uint32_t dv = smem_u32(sV + vs * V_BYTES);
            mbar_arrive_expect_tx(BAR(5 + vs), V_BYTES);
            tma_load_3d(dv, &tmV, 0, j * BKV, head, BAR(5 + vs));
            tma_load_3d(dv + V_BYTES / 2, &tmV, 64, j * BKV, head, BAR(5 + vs));
            v_issued++;
        }
        if (!ok) {  // let copies already in flight land before the CTA goes away
            for (uint32_t i = 0; i < (1u << 16); i++) if (mbar_try_wait(BAR(0), 0)) break;
            for (int j = max(0, k_issued - K_STAGES); j < k_issued; j++)
                for (uint32_t i = 0; i < (1u << 16); i++) if (mbar_try_wait(BAR(1 + (j & 1)), (j >> 1) & 1)) break;
            for (int j = max(0, v_issued - V_STAGES); j < v_issued; j++)
                for (uint32_t i = 0; i < (1u << 16); i++) if (mbar_try_wait(BAR(5 + (j & 1)), (j >> 1) & 1)) break;
        }
    } else if (warp == 1 && lane == 0) {
        // ---------------- MMA issuer 1: S_j = Q K_j^T -----------------------------------------------
        // Two issuing threads (this one and the P.V issuer below): the barrier waits, commits and
        // fences of a tile cost one thread more time than its MMAs take to execute, and an MMA issue
        // blocks while the tensor core's short queue is full.
        constexpr uint32_t idesc_s = make_idesc(BKV);
        bool ok = mbar_wait(BAR(0), 0, abort_flag);
        const uint32_t aQ = smem_u32(sQ);
        for (int j = 0; j < n_tiles && ok; j++) {
            const int b = j & 1;
            if (!(ok = mbar_wait(BAR(1 + b), (j >> 1) & 1, abort_flag))) break;
            if (j >= 2 && !(ok = mbar_wait(BAR(7 + b), ((j >> 1) - 1) & 1, abort_flag))) break;   // P.V of tile j-2 has read P from this buffer
            tc_fence_after();
            const uint32_t aK = smem_u32(sK + b * K_BYTES);
#pragma unroll
            for (int k = 0; k < HD / 16; k++)
                umma(tmem_base + S_COL + (uint32_t)(b * BKV),
                     make_desc(aQ + (k >> 2) * (Q_BYTES / 2) + (k & 3) * 32),
                     make_desc(aK + (k >> 2) * (K_BYTES / 2) + (k & 3) * 32), idesc_s, k > 0 ? 1u : 0u);
            umma_commit(BAR(9 + b));   // scores ready
            umma_commit(BAR(3 + b));   // K stage reusable
        }
    } else if (warp == 6 && lane == 0) {
        // ---------------- MMA issuer 2: O += P_t V_t, P_t read from the tensor-memory columns of S_t ----
        constexpr uint32_t idesc_o = make_idesc(HD) | IDESC_B_MN_MAJOR;
        bool ok = true;
        for (int t = 0; t < n_tiles && ok; t++) {
            const int tb = t & 1;
            if (!(ok = mbar_wait(BAR(5 + tb), (t >> 1) & 1, abort_flag))) break;
            if (!(ok = mbar_wait(BAR(11 + tb), (t >> 1) & 1, abort_flag))) break;
            tc_fence_after();
            const uint32_t aV = smem_u32(sV + tb * V_BYTES);
#pragma unroll
            for (int k = 0; k < BKV / 16; k++)
                umma_ts(tmem_base + O_COL, tmem_base + S_COL + (uint32_t)(tb * BKV + k * 8),
                        make_desc_mn(aV + k * 2048, V_BYTES / 2, 1024), idesc_o, (t > 0 || k > 0) ? 1u : 0u);
            umma_commit(BAR(7 + tb));   // V stage and score/P buffer tb reusable, accumulator updated
        }
    } else if (warp >= 2 && warp < 6) {
        // ---------------- softmax: one query row per thread -------------------------------------
        const int q = warp & 3;                         // TMEM lane quarter this warp may access
        const int r = q * 32 + lane;
        const int rowpos = p.pos0 + q0 + r;
        const uint32_t lane_addr = tmem_base + ((uint32_t)(q * 32) << 16);
        float m_ref = -INFINITY, l = 0.f;
        bool ok = true;
        for (int j = 0; j < n_tiles; j++) {
            const int b = j & 1;
            ok = mbar_wait(BAR(9 + b), (j >> 1) & 1, abort_flag);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            tc_fence_after();
            uint32_t s[BKV];
            tmem_ld32(lane_addr + S_COL + (uint32_t)(b * BKV), s);
            tmem_ld32(lane_addr + S_COL + (uint32_t)(b * BKV + 32), s + 32);
            tmem_ld_wait();
            const int c0 = j * BKV;
            const bool need_mask = c0 + BKV - 1 > p.pos0 + q0;
            // running maximum on the raw scores (the scale is positive); the scale is applied inside
            // the exponent's FFMA: p = 2^(s * scale - m)
            if (need_mask) {
#pragma unroll
                for (int c = 0; c < BKV; c++)
                    if (c0 + c > rowpos) s[c] = 0xff800000u;   // -inf
            }
            float mx[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};     // four independent chains
#pragma unroll
            for (int c = 0; c < BKV; c += 4) {
#pragma unroll
                for (int i = 0; i < 4; i++) mx[i] = fmaxf(mx[i], __uint_as_float(s[c + i]));
            }
            const float mraw = fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3]));
            const float mloc = mraw * p.scale_log2;
            const bool grow = mloc > m_ref + RESCALE_THRESHOLD;   // always true for the first tile
            const float alpha = grow ? ex2(m_ref - mloc) : 1.0f;
            if (grow) m_ref = mloc;
            const float neg_m = -m_ref;
            uint32_t pk[BKV / 2];
            float sum0 = 0.f, sum1 = 0.f;
#pragma unroll
            for (int c = 0; c < BKV; c += 2) {
                const float p0 = ex2(fmaf(__uint_as_float(s[c]), p.scale_log2, neg_m));
                const float p1 = ex2(fmaf(__uint_as_float(s[c + 1]), p.scale_log2, neg_m));
                sum0 += p0;
                sum1 += p1;
                __half2 h = __floats2half2_rn(p0, p1);
                pk[c >> 1] = *reinterpret_cast<uint32_t*>(&h);
            }
            l = l * alpha + (sum0 + sum1);
            if (j > 0 && __any_sync(0xffffffffu, grow)) {
                // rescaling the accumulator: the previous P.V must have finished writing it
                ok = mbar_wait(BAR(7 + ((j - 1) & 1)), ((j - 1) >> 1) & 1, abort_flag);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                tc_fence_after();
                {
#pragma unroll 1
                    for (int cc = 0; cc < HD; cc += 32) {
                        uint32_t o[32];
                        tmem_ld32(lane_addr + O_COL + (uint32_t)cc, o);
                        tmem_ld_wait();
#pragma unroll
                        for (int i = 0; i < 32; i++) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
                        tmem_st32(lane_addr + O_COL + (uint32_t)cc, o);
                    }
                    tmem_st_wait();
                }
            }
            // P_j as the A operand of the second MMA, in place of the first 32 columns of S_j: this
            // thread's row, two fp16 per column
            tmem_st32(lane_addr + S_COL + (uint32_t)(b * BKV), pk);
            tmem_st_wait();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(BAR(11 + b));
        }
        if (ok) {
            ok = mbar_wait(BAR(7 + ((n_tiles - 1) & 1)), ((n_tiles - 1) >> 1) & 1, abort_flag);
            ok = __all_sync(0xffffffffu, ok);
        }
        if (ok) {
            tc_fence_after();
            const float inv = 1.0f / l;
            const bool valid = q0 + r < p.T;
            __half* orow = p.out + (long long)(q0 + r) * p.ldo + (long long)head * HD;
#pragma unroll 1
            for (int cc = 0; cc < HD; cc += 32) {
                uint32_t o[32];
                tmem_ld32(lane_addr + O_COL + (uint32_t)cc, o);
                tmem_ld_wait();
                if (valid) {
#pragma unroll
                    for (int v = 0; v < 4; v++) {
                        uint4 w;
                        __half2* wh = reinterpret_cast<__half2*>(&w);
#pragma unroll
                        for (int i = 0; i < 4; i++)
                            wh[i] = __floats2half2_rn(__uint_as_float(o[v * 8 + 2 * i]) * inv, __uint_as_float(o[v * 8 + 2 * i + 1]) * inv);
                        *reinterpret_cast<uint4*>(orow + cc + v * 8) = w;
                    }
                }
            }
        }
    }
    // ---------------- teardown ---------------------------------------------------------------------
    tc_fence_before();
    __syncthreads();
    if (warp == 0) {
        __syncwarp();
        tc_fence_after();
        tmem_dealloc<TMEM_COLS>(tmem_base);
    }
    if (threadIdx.x == 0 && *abort_flag) atomicExch(p.status, TL_ERR_TIMEOUT);
}

constexpr size_t FA_SMEM = (size_t)Q_BYTES + K_STAGES * K_BYTES + V_STAGES * V_BYTES + 256 + 1024;

}  // namespace

bool flash_prefill_supported(const void* q, const void* k, const void* v, const void* out, int T, int S, int pos0,
                             int heads, int head_dim, long long ldq, long long ldk, long long ldv, long long ldo) {
    auto al16 = [](const void* x) { return (reinterpret_cast<uintptr_t>(x) & 15) == 0; };
    return head_dim == HD && T >= 1 && S >= 1 && pos0 >= 0 && pos0 + T <= S && heads >= 1 && ldq % 8 == 0 &&
           ldk % 8 == 0 && ldv % 8 == 0 && ldo % 8 == 0 && al16(q) && al16(k) && al16(v) && al16(out) &&
           tensor_map_encode_available();
}

// q: (T, heads, hd) pitch ldq; k, v: (S, heads, hd) pitch ldk / ldv (the caches, positions 0..S-1);
// out: (T, heads, hd) pitch ldo. Query row t sits at position pos0 + t and attends to cache
// positions 0 .. pos0 + t.
int launch_flash_prefill(const __half* q, const __half* k, const __half* v, __half* out, int T, int S, int pos0,
                         int heads, int head_dim, long long ldq, long long ldk, long long ldv, long long ldo,
                         cudaStream_t st) {
    TL_REQUIRE(flash_prefill_supported(q, k, v, out, T, S, pos0, heads, head_dim, ldq, ldk, ldv, ldo),
               "flash prefill: unsupported shape or alignment (head_dim must be %d)", HD);
    static PerDeviceOnce once;
    if (once.needed()) {
        TL_CUDA(cudaFuncSetAttribute(k_flash_prefill, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)FA_SMEM));
        TL_CUDA(cudaFuncSetAttribute(k_flash_prefill, cudaFuncAttributePreferredSharedMemoryCarveout,
                                     (int)cudaSharedmemCarveoutMaxShared));
    }
    CUtensorMap mq, mk, mv;
    TL_PROPAGATE(make_tensor_map_f16(&mq, q, T, HD, ldq, HD, heads, BQ));
    TL_PROPAGATE(make_tensor_map_f16(&mk, k, S, HD, ldk, HD, heads, BKV));
    TL_PROPAGATE(make_tensor_map_f16(&mv, v, S, HD, ldv, HD, heads, BKV));
    FlashArgs a{out, ldo, T, S, pos0, heads, 1.4426950408889634f / sqrtf((float)head_dim), device_status_word()};
    dim3 grid((unsigned)heads, (unsigned)((T + BQ - 1) / BQ));
    return launch_pdl(k_flash_prefill, grid, dim3(FA_THREADS), FA_SMEM, st, true, mq, mk, mv, a);
}

}  // namespace tlb
