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
#include "sm100.cuh"

namespace tlb {

namespace {

constexpr int BM = 128, BK = 64, STAGES = 4;
constexpr int GEMM_THREADS = 256;
constexpr int A_BYTES = BM * BK * 2;

using namespace sm100;

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
    return make_tensor_map_f16(map, base, rows, K, ld, stride, batch, box_rows);
}

}  // namespace

bool tensor_map_encode_available() { return encode_fn() != nullptr; }

int make_tensor_map_f16(CUtensorMap* map, const __half* base, int rows, int K, long long ld, long long stride,
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

namespace {

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
