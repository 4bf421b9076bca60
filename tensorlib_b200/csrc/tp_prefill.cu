// Tensor-parallel prefill: the owner's half of the fused compute + collective of the K-split
// matmuls (wo, w2). The reference is single-GPU; on one GPU this stage is the fused residual
// epilogue of the HGEMM followed by the RMSNorm kernel.
//
// Token rows are dealt out in contiguous slices, one per rank (the owner of a row). The matmul
// (hgemm_sm100.cu, push mode) keeps its partial result in its own memory and raises a flag in the
// OWNER's memory for every finished (128-row block, column tile) while its other tiles are still
// being computed. k_tp_reduce_norm below runs on the owner, one CTA per row: it waits for the flags
// of its row block from every source rank, fetches the partial rows from the sources' memory with
// plain peer loads (a warp reads 512 contiguous bytes: the reduce-scatter), adds them in rank order
// in fp32, rounds once, adds the residual in fp16 (the arithmetic of the single-GPU path up to the
// fp32 summation order), writes the new residual row locally, applies the RMSNorm of the operator
// that follows and stores the normalised row into every rank's activation buffer (the all-gather,
// 512-byte peer stores), then sets that row's flag on every rank. k_tp_wait_rows holds the stream
// until all rows of all owners have arrived, after which the next matmul reads them like any local
// buffer. No collective library call, no multicast, every wait is bounded.
// (Pushing the tiles from the matmul's epilogue instead was measured first: a thread owns 64
// contiguous bytes of a row there, and half a million such stores per matmul cost more NVLink time
// than the allreduce they replace: 18.9 ms against 15.7 ms for the 2048-token prefill on two GPUs.)
#include "kernels.cuh"

namespace tlb {

namespace {

constexpr int RN_THREADS = 256;

__device__ __forceinline__ unsigned int ld_acquire_sys(const unsigned int* p) {
    unsigned int v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

__global__ void __launch_bounds__(RN_THREADS) k_tp_reduce_norm(TpReduceNorm p, int* status) {
    __shared__ float red[RN_THREADS / 32];
    __shared__ int timed_out;
    const int r = blockIdx.x;                       // row of this rank's slice
    const int rb = r >> 7;
    if (threadIdx.x == 0) timed_out = 0;
    pdl_launch_dependents();
    pdl_wait();
    __syncthreads();
    // every (source, column tile) flag of this row block
    for (int i = threadIdx.x; i < p.world * p.col_tiles; i += RN_THREADS) {
        const int src = i / p.col_tiles, ct = i - src * p.col_tiles;
        const unsigned int* f = p.arrive_flags + (size_t)src * p.flags_slot_stride + rb * 64 + ct;
        bool here = false;
        for (unsigned int t = 0; t < TL_EXCHANGE_TRIES && !here; t++) here = ld_acquire_sys(f) == p.epoch;
        if (!here) timed_out = 1;
    }
    __syncthreads();
    if (timed_out) {
        if (threadIdx.x == 0) atomicExch(status, TL_ERR_TIMEOUT);
        return;
    }
    // h = residual + half(sum over ranks), kept in registers for the norm; dim / 8 16-byte groups per row
    const int groups = p.dim >> 3;
    const uint4* res4 = reinterpret_cast<const uint4*>(p.residual + (size_t)r * p.dim);
    uint4* out4 = reinterpret_cast<uint4*>(p.residual_out + (size_t)r * p.dim);
    constexpr int MAXG = 4;                          // groups per thread: dim <= 8 * 256 * 4 = 8192
    uint4 hval[MAXG];
    float ss = 0.f;
#pragma unroll
    for (int k = 0; k < MAXG; k++) {
        const int g = threadIdx.x + k * RN_THREADS;
        if (g >= groups) break;
        float s[8];
#pragma unroll
        for (int j = 0; j < 8; j++) s[j] = 0.f;
        for (int src = 0; src < p.world; src++) {
            uint4 v;     // straight from the source rank's memory; volatile: never served from a stale local cache line
            const uint4* ptr = reinterpret_cast<const uint4*>(p.partial[src] + (size_t)(p.row0 + r) * p.dim) + g;
            asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(ptr) : "memory");
            const __half2* vh = reinterpret_cast<const __half2*>(&v);
#pragma unroll
            for (int j = 0; j < 4; j++) { const float2 f = __half22float2(vh[j]); s[2 * j] += f.x; s[2 * j + 1] += f.y; }
        }
        const uint4 rv = res4[g];
        const __half* rh = reinterpret_cast<const __half*>(&rv);
        uint4 hv;
        __half* hh = reinterpret_cast<__half*>(&hv);
#pragma unroll
        for (int j = 0; j < 8; j++) {
            hh[j] = hadd_ref(rh[j], __float2half_rn(s[j]));
            const float f = __half2float(hh[j]);
            ss = fmaf(f, f, ss);
        }
        hval[k] = hv;
        out4[g] = hv;
    }
    ss = warp_sum(ss);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
    __syncthreads();
    float tot = 0.f;
#pragma unroll
    for (int w = 0; w < RN_THREADS / 32; w++) tot += red[w];
    const float rinv = rsqrtf(tot / (float)p.dim + p.eps);
    const uint4* nw4 = reinterpret_cast<const uint4*>(p.norm_w);
    const size_t grow = (size_t)(p.row0 + r);
#pragma unroll
    for (int k = 0; k < MAXG; k++) {
        const int g = threadIdx.x + k * RN_THREADS;
        if (g >= groups) break;
        const uint4 wv = nw4[g];
        const __half2* wh = reinterpret_cast<const __half2*>(&wv);
        const __half2* hh = reinterpret_cast<const __half2*>(&hval[k]);
        uint4 o;
        __half2* oh = reinterpret_cast<__half2*>(&o);
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const float2 hf = __half22float2(hh[j]), wf = __half22float2(wh[j]);
            oh[j] = __floats2half2_rn(hf.x * rinv * wf.x, hf.y * rinv * wf.y);
        }
        for (int d = 0; d < p.world; d++) reinterpret_cast<uint4*>(p.xn_dst[d] + grow * p.dim)[g] = o;
    }
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x < p.world)
        asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p.gather_flags[threadIdx.x] + grow), "r"(p.epoch) : "memory");
}

__global__ void __launch_bounds__(1024) k_tp_wait_rows(const unsigned int* flags, int rows, unsigned int epoch, int* status) {
    pdl_launch_dependents();
    pdl_wait();
    bool all = true;
    for (int i = threadIdx.x; i < rows; i += blockDim.x) {
        bool here = false;
        for (unsigned int t = 0; t < TL_EXCHANGE_TRIES && !here; t++) here = ld_acquire_sys(flags + i) == epoch;
        all &= here;
    }
    if (!all) atomicExch(status, TL_ERR_TIMEOUT);
}

}  // namespace

int launch_tp_reduce_norm(const TpReduceNorm& p, cudaStream_t st) {
    TL_REQUIRE(p.world >= 2 && p.world <= TL_MAX_TP && p.rows > 0 && p.dim % 8 == 0 && p.dim <= 8 * RN_THREADS * 4 &&
               p.col_tiles >= 1 && p.col_tiles <= 64, "tp reduce: bad shape");
    return launch_pdl(k_tp_reduce_norm, dim3((unsigned)p.rows), dim3(RN_THREADS), 0, st, true, p, device_status_word());
}

int launch_tp_wait_rows(const unsigned int* flags, int rows, unsigned int epoch, cudaStream_t st) {
    if (rows <= 0) return TL_OK;
    return launch_pdl(k_tp_wait_rows, dim3(1), dim3(1024), 0, st, true, flags, rows, epoch, device_status_word());
}

}  // namespace tlb
