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
// Every mbarrier wait is bounded; when one gives up the CTA raises an abort flag, every role
// leaves its loop, TMEM is freed and TL_ERR_TIMEOUT is recorded in the device status word.
#include <cuda.h>

#include <mutex>

#include "kernels.cuh"

namespace tlb {

namespace {

constexpr int BM = 128, BK = 64, STAGES = 4;
constexpr int GEMM_THREADS = 256;
constexpr int A_BYTES = BM * BK * 2;

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
// Bounded wait that also gives up as soon as another role of the CTA has raised the abort flag.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
    for (uint32_t i = 0; i < WAIT_LIMIT; i++) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((i & 63) == 63 && *abort_flag) return false;
    }
    *abort_flag = 1;
    return false;
}

__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* map, int c0, int c1, int c2, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
        ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1), "r"(c2)
        : "memory");
}

// Shared-memory matrix descriptor, K-major operand, 128-byte swizzle: rows are 128 bytes apart,
// groups of 8 rows (one swizzle atom) 1024 bytes apart.
__device__ __forceinline__ uint64_t make_desc(uint32_t saddr) {
    uint64_t d = 0;
    d |= (uint64_t)((saddr & 0x3FFFF) >> 4);   // start address
    d |= (uint64_t)1 << 16;                     // leading byte offset (unused for swizzled K-major)
    d |= (uint64_t)(1024 >> 4) << 32;           // stride byte offset between 8-row groups
    d |= (uint64_t)1 << 46;                     // descriptor version (sm_100)
    d |= (uint64_t)2 << 61;                     // SWIZZLE_128B
    return d;
}
// Instruction descriptor, kind::f16: A, B fp16 K-major, D fp32, M=128, N=n
__host__ __device__ constexpr uint32_t make_idesc(int n) {
    return (1u << 4) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
}
__device__ __forceinline__ void umma(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
        " tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n"
        ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t* r) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

struct GemmArgs {
    __half* C;
    int M, N, K, batch;
    long long ldc, sC;
    int a_batched, b_batched;   // 0: the operand is shared by all batches (batch coordinate 0)
    int* status;
};

template <int BN>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
k_hgemm(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, GemmArgs p) {
    constexpr int B_BYTES = BN * BK * 2;
    constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
    constexpr uint32_t TMEM_COLS = 2 * BN;      // two accumulator buffers
    extern __shared__ unsigned char smem_raw[];
    // the swizzled tiles need 1024-byte alignment
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES);
    const uint32_t full0 = smem_u32(bars), empty0 = smem_u32(bars + STAGES);
    const uint32_t tfull0 = smem_u32(bars + 2 * STAGES), tempty0 = smem_u32(bars + 2 * STAGES + 2);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int mt_count = (p.M + BM - 1) / BM, nt_count = (p.N + BN - 1) / BN;
    const int tiles_per_batch = mt_count * nt_count;
    const int total_tiles = tiles_per_batch * p.batch;
    const int nkb = (p.K + BK - 1) / BK;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; s++) { mbar_init(full0 + 8 * s, 1); mbar_init(empty0 + 8 * s, 1); }
        for (int b = 0; b < 2; b++) { mbar_init(tfull0 + 8 * b, 1); mbar_init(tempty0 + 8 * b, 4); }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 2) {  // TMEM allocation: one warp, result written to shared memory
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0 && lane == 0) {
        // ---------------- TMA producer ---------------------------------------------------------
        asm volatile("prefetch.tensormap [%0];" ::"l"(&tmA) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&tmB) : "memory");
        int it = 0;
        bool ok = true;
        for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
            const int b = tile / tiles_per_batch, idx = tile - b * tiles_per_batch;
            const int mt = idx % mt_count, nt = idx / mt_count;
            for (int kb = 0; kb < nkb; kb++, it++) {
                const int s = it % STAGES, use = it / STAGES;
                if (use > 0 && !(ok = mbar_wait(empty0 + 8 * s, (use - 1) & 1, abort_flag))) break;
                const uint32_t sa = smem_u32(smem + s * STAGE_BYTES), sb = sa + A_BYTES;
                mbar_arrive_expect_tx(full0 + 8 * s, STAGE_BYTES);
                tma_load_3d(sa, &tmA, kb * BK, mt * BM, p.a_batched ? b : 0, full0 + 8 * s);
                tma_load_3d(sb, &tmB, kb * BK, nt * BN, p.b_batched ? b : 0, full0 + 8 * s);
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
        // ---------------- epilogue: TMEM -> registers -> fp16 -> global -----------------------------
        const int q = warp & 3;                   // TMEM lane quarter this warp may access
        int tcount = 0;
        bool ok = true;
        const bool vec_ok = (p.ldc % 8 == 0) && (p.sC % 8 == 0) && ((reinterpret_cast<uintptr_t>(p.C) & 15) == 0);
        for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x, tcount++) {
            const int b = tile / tiles_per_batch, idx = tile - b * tiles_per_batch;
            const int mt = idx % mt_count, nt = idx / mt_count;
            const int buf = tcount & 1, use = tcount >> 1;
            ok = mbar_wait(tfull0 + 8 * buf, use & 1, abort_flag);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            tc_fence_after();
            const int row = mt * BM + q * 32 + lane;
            __half* crow = p.C + (long long)b * p.sC + (long long)row * p.ldc;
#pragma unroll 1
            for (int c = 0; c < BN; c += 32) {
                uint32_t r[32];
                tmem_ld32(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(buf * BN + c), r);
                tmem_ld_wait();
                const int col0 = nt * BN + c;
                if (row < p.M && col0 < p.N) {
                    if (vec_ok && col0 + 32 <= p.N) {
#pragma unroll
                        for (int v = 0; v < 4; v++) {
                            uint4 o;
                            __half2* oh = reinterpret_cast<__half2*>(&o);
#pragma unroll
                            for (int j = 0; j < 4; j++)
                                oh[j] = __floats2half2_rn(__uint_as_float(r[v * 8 + 2 * j]), __uint_as_float(r[v * 8 + 2 * j + 1]));
                            *reinterpret_cast<uint4*>(crow + col0 + v * 8) = o;
                        }
                    } else {
                        for (int j = 0; j < 32 && col0 + j < p.N; j++)
                            crow[col0 + j] = __float2half_rn(__uint_as_float(r[j]));
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(tempty0 + 8 * buf);
        }
    }
    // ---------------- teardown ---------------------------------------------------------------------
    tc_fence_before();
    __syncthreads();
    if (warp == 2) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
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

// rows x K fp16 operand with row pitch `ld` and batch stride `stride` (elements), box 64 x box_rows
int make_map(CUtensorMap* map, const __half* base, int rows, int K, long long ld, long long stride, int batch,
             int box_rows) {
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

template <int BN>
int launch_bn(const CUtensorMap& ma, const CUtensorMap& mb, const GemmArgs& a, int tiles, cudaStream_t st) {
    constexpr size_t smem = (size_t)STAGES * (A_BYTES + BN * BK * 2) + 1024 + 256;
    static bool configured = false;
    if (!configured) {
        TL_CUDA(cudaFuncSetAttribute(k_hgemm<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        configured = true;
    }
    const int grid = std::max(1, std::min(tiles, sm_count()));
    k_hgemm<BN><<<grid, GEMM_THREADS, smem, st>>>(ma, mb, a);
    TL_LAUNCH_CHECK();
    return TL_OK;
}

}  // namespace

bool hgemm_supported(const void* A, const void* B, const void* C, size_t M, size_t N, size_t K, size_t lda,
                     size_t ldb, size_t ldc) {
    auto al16 = [](const void* q) { return (reinterpret_cast<uintptr_t>(q) & 15) == 0; };
    (void)C; (void)ldc;
    return M >= 1 && N >= 1 && K >= 8 && lda % 8 == 0 && ldb % 8 == 0 && al16(A) && al16(B) && encode_fn() != nullptr;
}

int launch_hgemm(const __half* A, const __half* B, __half* C, int batch, int M, int N, int K, long long lda,
                 long long ldb, long long ldc, long long sA, long long sB, long long sC, cudaStream_t st) {
    TL_REQUIRE(hgemm_supported(A, B, C, M, N, K, lda, ldb, ldc), "hgemm: unsupported shape or alignment");
    TL_REQUIRE(sA % 8 == 0 && sB % 8 == 0, "hgemm: batch strides must be multiples of 8 elements");
    if (batch <= 0) return TL_OK;
    // widest N tile that still gives every SM a tile
    const int mt = (M + BM - 1) / BM;
    int bn = 256;
    while (bn > 64 && (long long)mt * ((N + bn - 1) / bn) * batch < sm_count()) bn >>= 1;
    CUtensorMap ma, mb;
    TL_PROPAGATE(make_map(&ma, A, M, K, lda, sA, batch, BM));
    TL_PROPAGATE(make_map(&mb, B, N, K, ldb, sB, batch, bn));
    GemmArgs a{C, M, N, K, batch, ldc, sC, (sA != 0 && batch > 1) ? 1 : 0, (sB != 0 && batch > 1) ? 1 : 0,
               device_status_word()};
    const int tiles = mt * ((N + bn - 1) / bn) * batch;
    if (bn == 256) return launch_bn<256>(ma, mb, a, tiles, st);
    if (bn == 128) return launch_bn<128>(ma, mb, a, tiles, st);
    return launch_bn<64>(ma, mb, a, tiles, st);
}

}  // namespace tlb
