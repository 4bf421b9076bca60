// Tensor-parallel prefill: the owner's half of the fused compute + collective of the K-split
// matmuls (wo, w2). The reference is single-GPU; on one GPU this stage is the fused residual
// epilogue of the HGEMM followed by the RMSNorm kernel.
//
// Token rows are dealt out in contiguous slices, one per rank (the owner of a row). The matmul
// (hgemm_sm100.cu, push mode) keeps its partial result in its own memory and raises a flag in the
// OWNER's memory for every finished (128-row block, column tile) while its other tiles are still
// being computed. k_tp_reduce_norm below runs on the owner, four warps per row: it waits for the flags
// of its row block from every source rank, fetches the partial rows from the sources' memory with
// plain peer loads (a warp reads 512 contiguous bytes: the reduce-scatter), adds them in rank order
// in fp32, rounds once, adds the residual in fp16 (the arithmetic of the single-GPU path up to the
// fp32 summation order), writes the new residual row locally, applies the RMSNorm of the operator
// that follows and stores the normalised row into every rank's activation buffer (the all-gather,
// 512-byte peer stores); the CTA that finishes the slice's last row sets this owner's flag on every
// rank. k_tp_wait_owners holds the stream until every owner's flag is up, after which the next
// matmul reads the rows like any local buffer. No collective library call, no multicast, every wait is bounded.
// (Pushing the tiles from the matmul's epilogue instead was measured first: a thread owns 64
// contiguous bytes of a row there, and half a million such stores per matmul cost more NVLink time
// than the allreduce they replace: 18.9 ms against 15.7 ms for the 2048-token prefill on two GPUs.)
#include "kernels.cuh"

namespace tlb {

namespace {

constexpr int RN_ROW_THREADS = 128;                // four warps share a row
constexpr int RN_ROWS = 2;                         // rows per CTA
constexpr int RN_THREADS = RN_ROW_THREADS * RN_ROWS;

__device__ __forceinline__ unsigned int ld_acquire_sys(const unsigned int* p) {
    unsigned int v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// barrier among the four warps of row `rsub` of the CTA (named barriers 1, 2; 0 is __syncthreads)
__device__ __forceinline__ void row_bar_sync(int rsub) {
    asm volatile("bar.sync %0, %1;" ::"r"(rsub + 1), "n"(RN_ROW_THREADS) : "memory");
}
__device__ __forceinline__ uint4 ld_peer16(const uint4* ptr) {
    uint4 v;     // relaxed system-scope load: straight from the source rank's memory, never a stale local cache line
    asm volatile("ld.relaxed.sys.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(ptr));
    return v;
}

// Four warps per row, two rows per CTA. Everything on a row's chain is a round trip over NVLink or a
// system-scope fence, so the kernel is built to have few of them in sequence: every lane holds GPT 16-byte groups
// of the row and issues the loads of all ranks for up to 16 of them before it uses any (one round trip for dim
// 4096 on up to four ranks; the first form, one warp per row with 16 groups per lane in batches of 4 / world,
// took 55 us for 512 rows on four GPUs where this one needs one batch), the row's sum of squares meets in shared
// memory across the four warps, and one thread per CTA fences. W = number of ranks, GPT = groups per thread.
template <int W, int GPT>
__global__ void __launch_bounds__(RN_THREADS) k_tp_reduce_norm(TpReduceNorm p, int* status) {
    constexpr int CH = GPT * W <= 16 ? GPT : (16 / W >= 1 ? 16 / W : 1);      // groups per thread whose loads are issued together
    __shared__ float red[RN_THREADS / 32];
    __shared__ int rows_here;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int rsub = threadIdx.x / RN_ROW_THREADS;                       // which of the CTA's rows
    const int t = threadIdx.x - rsub * RN_ROW_THREADS;                   // thread within the row
    const int r = blockIdx.x * RN_ROWS + rsub;                           // row of this rank's slice
    if (threadIdx.x == 0) rows_here = 0;
    pdl_launch_dependents();
    pdl_wait();
    __syncthreads();
    const int rb = min(r, p.rows - 1) >> 7;
    // every (source, column tile) flag of this row block, polled by the row's first warp
    bool ok = r < p.rows;
    if (ok && t < 32) {
        for (int i = lane; i < W * p.col_tiles; i += 32) {
            const int src = i / p.col_tiles, ct = i - src * p.col_tiles;
            const unsigned int* f = p.arrive_flags + (size_t)src * p.flags_slot_stride + rb * 64 + ct;
            bool here = false;
            for (unsigned int tr = 0; tr < TL_EXCHANGE_TRIES && !here; tr++) here = ld_acquire_sys(f) == p.epoch;
            ok &= here;
        }
        ok = __all_sync(0xffffffffu, ok);
        if (!ok && lane == 0) atomicExch(status, TL_ERR_TIMEOUT);     // the row is never counted: the waiting kernels give up as well
        if (lane == 0) red[warp] = ok ? 1.f : 0.f;
    }
    row_bar_sync(rsub);
    ok = r < p.rows && red[rsub * (RN_ROW_THREADS / 32)] != 0.f;
    row_bar_sync(rsub);                                                  // red is reused for the sums below
    // h = residual + half(sum over ranks), kept in registers for the norm; dim / 8 16-byte groups per row
    const int groups = p.dim >> 3;
    const size_t grow = (size_t)(p.row0 + min(r, p.rows - 1));
    const uint4* res4 = reinterpret_cast<const uint4*>(p.residual + (size_t)min(r, p.rows - 1) * p.dim);
    uint4* out4 = reinterpret_cast<uint4*>(p.residual_out + (size_t)min(r, p.rows - 1) * p.dim);
    uint4 hval[GPT];
    float ss = 0.f;
    if (ok) {
#pragma unroll
        for (int c0 = 0; c0 < GPT; c0 += CH) {
            if (c0 * RN_ROW_THREADS >= groups) break;
            uint4 v[CH][W], rv[CH];
#pragma unroll
            for (int cc = 0; cc < CH; cc++) {
                const int g = min(t + (c0 + cc) * RN_ROW_THREADS, groups - 1);
#pragma unroll
                for (int src = 0; src < W; src++) v[cc][src] = ld_peer16(reinterpret_cast<const uint4*>(p.partial[src] + grow * p.dim) + g);
                rv[cc] = res4[g];
            }
#pragma unroll
            for (int cc = 0; cc < CH; cc++) {
                const int g = t + (c0 + cc) * RN_ROW_THREADS;
                float s[8];
#pragma unroll
                for (int j = 0; j < 8; j++) s[j] = 0.f;
#pragma unroll
                for (int src = 0; src < W; src++) {
                    const __half2* vh = reinterpret_cast<const __half2*>(&v[cc][src]);
#pragma unroll
                    for (int j = 0; j < 4; j++) { const float2 f = __half22float2(vh[j]); s[2 * j] += f.x; s[2 * j + 1] += f.y; }
                }
                const __half* rh = reinterpret_cast<const __half*>(&rv[cc]);
                uint4 hv;
                __half* hh = reinterpret_cast<__half*>(&hv);
                float part = 0.f;
#pragma unroll
                for (int j = 0; j < 8; j++) {
                    hh[j] = hadd_ref(rh[j], __float2half_rn(s[j]));
                    const float f = __half2float(hh[j]);
                    part = fmaf(f, f, part);
                }
                hval[c0 + cc] = hv;
                if (g < groups) { out4[g] = hv; ss += part; }
            }
        }
    }
    ss = warp_sum(ss);
    if (lane == 0) red[warp] = ss;
    row_bar_sync(rsub);
    if (ok) {
        float tot = 0.f;
#pragma unroll
        for (int w = 0; w < RN_ROW_THREADS / 32; w++) tot += red[rsub * (RN_ROW_THREADS / 32) + w];
        const float rinv = rsqrtf(tot / (float)p.dim + p.eps);
        const uint4* nw4 = reinterpret_cast<const uint4*>(p.norm_w);
#pragma unroll
        for (int c = 0; c < GPT; c++) {
            const int g = t + c * RN_ROW_THREADS;
            if (g >= groups) break;
            const uint4 wv = nw4[g];
            const __half2* wh = reinterpret_cast<const __half2*>(&wv);
            const __half2* hh = reinterpret_cast<const __half2*>(&hval[c]);
            uint4 o;
            __half2* oh = reinterpret_cast<__half2*>(&o);
#pragma unroll
            for (int j = 0; j < 4; j++) {
                const float2 hf = __half22float2(hh[j]), wf = __half22float2(wh[j]);
                oh[j] = __floats2half2_rn(hf.x * rinv * wf.x, hf.y * rinv * wf.y);
            }
#pragma unroll
            for (int d = 0; d < W; d++) reinterpret_cast<uint4*>(p.xn_dst[d] + grow * p.dim)[g] = o;
        }
        if (t == 0) atomicAdd(&rows_here, 1);
    }
    // The CTA barrier orders every warp's stores before thread 0's fence (cumulative at system scope: one fence
    // per CTA; a fence per row measured 8 us more over 1024 rows, and it is the only system-scope fence on the
    // chain). The CTA that counts the last row of the slice then tells every rank that this owner's rows are all
    // in place: every other row's stores were performed system-wide before its count was added, and the flag
    // stores are issued after the count was read.
    __syncthreads();
    if (threadIdx.x == 0 && rows_here > 0) {
        __threadfence_system();
        if (atomicAdd(p.rows_done, (unsigned int)rows_here) + (unsigned int)rows_here == (unsigned int)p.rows) {
            *p.rows_done = 0;           // the next exchange's kernel starts after this one has finished
            __threadfence();
#pragma unroll
            for (int d = 0; d < W; d++)
                asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(p.owner_done[d] + p.rank), "r"(p.epoch) : "memory");
        }
    }
}

// holds the stream until every owner has announced its rows (one flag per owner)
__global__ void __launch_bounds__(32) k_tp_wait_owners(const unsigned int* flags, int owners, unsigned int epoch, int* status) {
    pdl_launch_dependents();
    pdl_wait();
    bool all = true;
    for (int i = threadIdx.x; i < owners; i += blockDim.x) {
        bool here = false;
        for (unsigned int t = 0; t < TL_EXCHANGE_TRIES && !here; t++) here = ld_acquire_sys(flags + i) == epoch;
        all &= here;
    }
    if (!all) atomicExch(status, TL_ERR_TIMEOUT);
}

}  // namespace

template <int W>
int launch_reduce_w(const TpReduceNorm& p, cudaStream_t st) {
    const dim3 grid((unsigned)((p.rows + RN_ROWS - 1) / RN_ROWS)), block(RN_THREADS);
    const int groups = p.dim / 8;
    if (groups <= RN_ROW_THREADS) return launch_pdl(k_tp_reduce_norm<W, 1>, grid, block, 0, st, true, p, device_status_word());
    if (groups <= 4 * RN_ROW_THREADS) return launch_pdl(k_tp_reduce_norm<W, 4>, grid, block, 0, st, true, p, device_status_word());
    return launch_pdl(k_tp_reduce_norm<W, 8>, grid, block, 0, st, true, p, device_status_word());
}

int launch_tp_reduce_norm(const TpReduceNorm& p, cudaStream_t st) {
    TL_REQUIRE(p.rows > 0 && p.dim % 8 == 0 && p.dim <= 8192 && p.col_tiles >= 1 && p.col_tiles <= 64, "tp reduce: bad shape");
    switch (p.world) {
        case 2: return launch_reduce_w<2>(p, st);
        case 4: return launch_reduce_w<4>(p, st);
        case 8: return launch_reduce_w<8>(p, st);
    }
    TL_REQUIRE(false, "tp reduce: 2, 4 or 8 ranks");
    return TL_ERR_UNSUPPORTED;
}

int launch_tp_wait_owners(const unsigned int* flags, int owners, unsigned int epoch, cudaStream_t st) {
    if (owners <= 0) return TL_OK;
    return launch_pdl(k_tp_wait_owners, dim3(1), dim3(32), 0, st, true, flags, owners, epoch, device_status_word());
}

}  // namespace tlb
