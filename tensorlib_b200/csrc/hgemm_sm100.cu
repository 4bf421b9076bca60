// Prefill HGEMM on tcgen05 / TMEM / TMA (placeholder until the kernel lands: reports every shape
// as unsupported so callers take the skinny-GEMV route).
#include "kernels.cuh"

namespace tlb {

bool hgemm_supported(const void*, const void*, const void*, size_t, size_t, size_t, size_t, size_t, size_t) {
    return false;
}

int launch_hgemm(const __half*, const __half*, __half*, int, int, int, int, long long, long long,
                 long long, long long, long long, long long, cudaStream_t) {
    return set_error(TL_ERR_UNSUPPORTED, "hgemm: not built");
}

}  // namespace tlb
