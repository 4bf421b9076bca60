// Library state: device selection, error text, device memory helpers, and the host-computed
// lookup tables that make transcendental functions agree bit for bit with the reference CPU code.
#include <cmath>
#include <cstring>
#include <mutex>
#include <string>
#include <vector>

#include "kernels.cuh"

namespace tlb {

namespace {
thread_local char g_err[512] = "";
bool g_init = false;
int g_device = -1;
int g_sms = 0;
Tables g_tables{};
int* g_status = nullptr;
std::mutex g_mu;

struct RopeTable {
    int head_dim = 0, rows = 0;
    __half* cos_t = nullptr;
    __half* sin_t = nullptr;
};
std::vector<RopeTable> g_rope;
// Tables that were replaced by a larger one. Their pointers may still be held by a model (and be
// baked into its decode graph), so they stay allocated until the process exits; a generation is
// rows * head_dim * 2 bytes, and the row count doubles, so all retired generations together are
// smaller than the live one.
std::vector<__half*> g_rope_retired;
}  // namespace

int set_error(int status, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof g_err, fmt, ap);
    va_end(ap);
    return status;
}
bool initialized() { return g_init; }
int sm_count() { return g_sms; }
const Tables& tables() { return g_tables; }
int* device_status_word() { return g_status; }

// `value` is a copy of the status word fetched at a synchronisation point. Non-zero: clear the
// word on the device and report the failure to the caller instead of returning results computed
// from partial or stale data.
int consume_device_status(int value) {
    if (value == 0) return TL_OK;
    cudaMemset(g_status, 0, sizeof(int));
    return set_error(value == TL_ERR_TIMEOUT ? TL_ERR_TIMEOUT : TL_ERR_CUDA,
                     "a kernel gave up on a bounded device-side wait (status word %d): the results of this call are not valid",
                     value);
}

// The three tables are functions half -> half, so 65536 entries each describe them completely.
// They are evaluated with the same libm calls and the same conversions the reference's CPU
// backend uses (tensorLib/src/device/cpu/softmax.cpp:22 for exp, CPU.cpp:216-222 for SiLU), which
// is what makes the reference-order kernels bit-identical to it without re-implementing libm.
static void compute_lookup_tables(__half* e, __half* sf, __half* sh) {
    for (unsigned i = 0; i < 65536; i++) {
        __half_raw r;
        r.x = (unsigned short)i;
        __half h(r);
        float x = __half2float(h);
        e[i] = __half(std::exp((double)x));                 // ::exp(double), then half(double)
        float sig = 1 / (1 + std::exp(-x));                 // float route
        sf[i] = __float2half(x * sig);
        __half sigh = __float2half(1 / (1 + std::exp(x)));  // fp16 route as shipped (sign defect)
        sh[i] = __float2half(__half2float(h) * __half2float(sigh));
    }
}

static int build_tables() {
    std::vector<__half> e(65536), sf(65536), sh(65536);
    compute_lookup_tables(e.data(), sf.data(), sh.data());
    __half* d = nullptr;
    TL_CUDA(cudaMalloc(&d, 3 * 65536 * sizeof(__half)));
    TL_CUDA(cudaMemcpy(d, e.data(), 65536 * 2, cudaMemcpyHostToDevice));
    TL_CUDA(cudaMemcpy(d + 65536, sf.data(), 65536 * 2, cudaMemcpyHostToDevice));
    TL_CUDA(cudaMemcpy(d + 2 * 65536, sh.data(), 65536 * 2, cudaMemcpyHostToDevice));
    g_tables.exp_tab = d;
    g_tables.silu_float_tab = d + 65536;
    g_tables.silu_half_tab = d + 2 * 65536;
    return TL_OK;
}

// cos/sin exactly as apply_rotary_emb evaluates them on the CPU (CPU.cpp:444-447): theta in
// float from powf, cosf/sinf, one rounding to half.
static void compute_rope_table(int head_dim, int rows, __half* c, __half* s) {
    const int half_dim = head_dim / 2;
    for (int p = 0; p < rows; p++)
        for (int d = 0; d < head_dim; d += 2) {
            float theta = p * 1.0f / std::pow(10000.0f, static_cast<float>(d) / static_cast<float>(head_dim));
            c[(size_t)p * half_dim + d / 2] = __float2half(std::cos(theta));
            s[(size_t)p * half_dim + d / 2] = __float2half(std::sin(theta));
        }
}

int rope_table(int head_dim, int min_rows, const __half** cos_t, const __half** sin_t) {
    std::lock_guard<std::mutex> lk(g_mu);
    RopeTable* t = nullptr;
    for (auto& r : g_rope)
        if (r.head_dim == head_dim) t = &r;
    if (!t) {
        g_rope.push_back(RopeTable{});
        t = &g_rope.back();
        t->head_dim = head_dim;
    }
    if (t->rows < min_rows) {
        int rows = 256;
        while (rows < min_rows) rows *= 2;
        const int half_dim = head_dim / 2;
        std::vector<__half> c((size_t)rows * half_dim), s((size_t)rows * half_dim);
        compute_rope_table(head_dim, rows, c.data(), s.data());
        __half *dc = nullptr, *ds = nullptr;
        TL_CUDA(cudaMalloc(&dc, c.size() * 2));
        if (cudaMalloc(&ds, s.size() * 2) != cudaSuccess) {
            cudaFree(dc);
            return set_error(TL_ERR_OUT_OF_MEMORY, "rope table of %d rows", rows);
        }
        TL_CUDA(cudaMemcpy(dc, c.data(), c.size() * 2, cudaMemcpyHostToDevice));
        TL_CUDA(cudaMemcpy(ds, s.data(), s.size() * 2, cudaMemcpyHostToDevice));
        // a table that was handed out is never freed: earlier callers keep reading their generation
        // (the first `rows` rows of every generation hold the same values)
        if (t->cos_t) g_rope_retired.push_back(t->cos_t);
        if (t->sin_t) g_rope_retired.push_back(t->sin_t);
        t->cos_t = dc;
        t->sin_t = ds;
        t->rows = rows;
    }
    *cos_t = t->cos_t;
    *sin_t = t->sin_t;
    return TL_OK;
}

}  // namespace tlb

using namespace tlb;

extern "C" {

const char* tl_strerror(int status) {
    switch (status) {
        case TL_OK: return "ok";
        case TL_ERR_INVALID_ARGUMENT: return "invalid argument";
        case TL_ERR_NOT_INITIALIZED: return "library not initialised (tl_init failed or was not called)";
        case TL_ERR_CUDA: return "CUDA error";
        case TL_ERR_UNSUPPORTED: return "unsupported";
        case TL_ERR_OUT_OF_MEMORY: return "out of device memory";
        case TL_ERR_TIMEOUT: return "device-side wait timed out";
        case TL_ERR_COMM: return "communication error";
        case TL_ERR_IO: return "I/O error";
        default: return "unknown status";
    }
}
const char* tl_last_error(void) { return g_err; }
int tl_version(void) { return 100; }

int tl_device_count(int* count) {
    TL_REQUIRE(count != nullptr, "count is null");
    int n = 0;
    cudaError_t e = cudaGetDeviceCount(&n);
    if (e != cudaSuccess) {
        *count = 0;
        return set_error(TL_ERR_NOT_INITIALIZED, "no CUDA device: %s", cudaGetErrorString(e));
    }
    *count = n;
    return TL_OK;
}

int tl_init(int device) {
    std::lock_guard<std::mutex> lk(g_mu);
    int n = 0;
    cudaError_t e = cudaGetDeviceCount(&n);
    if (e != cudaSuccess || n == 0)
        return set_error(TL_ERR_NOT_INITIALIZED, "no CUDA device available (%s); this library has no CPU path",
                         cudaGetErrorString(e));
    TL_REQUIRE(device >= 0 && device < n, "device %d out of range [0,%d)", device, n);
    if (g_init) {
        if (device != g_device)
            return set_error(TL_ERR_INVALID_ARGUMENT, "already initialised on device %d", g_device);
        TL_CUDA(cudaSetDevice(device));
        return TL_OK;
    }
    cudaDeviceProp prop;
    TL_CUDA(cudaGetDeviceProperties(&prop, device));
    if (prop.major != 10)
        return set_error(TL_ERR_UNSUPPORTED, "device %d is sm_%d%d; this library is built for sm_100a only",
                         device, prop.major, prop.minor);
    TL_CUDA(cudaSetDevice(device));
    g_device = device;
    g_sms = prop.multiProcessorCount;
    TL_PROPAGATE(build_tables());
    TL_CUDA(cudaMalloc(&g_status, sizeof(int)));
    TL_CUDA(cudaMemset(g_status, 0, sizeof(int)));
    g_init = true;
    return TL_OK;
}

// Synchronises the device, then reports (and clears) the status word kernels set when a bounded
// device-side wait gave up.
int tl_device_status(int* status) {
    TL_CHECK_INIT();
    TL_REQUIRE(status != nullptr, "status is null");
    TL_CUDA(cudaDeviceSynchronize());
    TL_CUDA(cudaMemcpy(status, g_status, sizeof(int), cudaMemcpyDeviceToHost));
    if (*status != 0) TL_CUDA(cudaMemset(g_status, 0, sizeof(int)));
    return TL_OK;
}

// Host-only: the tables above, written to caller memory. No device is touched.
int tl_host_lookup_tables(tl_half* exp_tab, tl_half* silu_float_tab, tl_half* silu_half_tab) {
    TL_REQUIRE(exp_tab && silu_float_tab && silu_half_tab, "null output");
    compute_lookup_tables(reinterpret_cast<__half*>(exp_tab), reinterpret_cast<__half*>(silu_float_tab),
                          reinterpret_cast<__half*>(silu_half_tab));
    return TL_OK;
}
int tl_host_rope_table(int head_dim, int rows, tl_half* cos_out, tl_half* sin_out) {
    TL_REQUIRE(head_dim > 0 && head_dim % 2 == 0 && rows > 0 && cos_out && sin_out, "bad rope table request");
    compute_rope_table(head_dim, rows, reinterpret_cast<__half*>(cos_out), reinterpret_cast<__half*>(sin_out));
    return TL_OK;
}

int tl_malloc(void** dptr, size_t bytes) {
    TL_CHECK_INIT();
    TL_REQUIRE(dptr != nullptr, "dptr is null");
    TL_CUDA(cudaMalloc(dptr, bytes ? bytes : 1));
    return TL_OK;
}
int tl_free(void* dptr) {
    TL_CHECK_INIT();
    TL_CUDA(cudaFree(dptr));
    return TL_OK;
}
int tl_memcpy_h2d(void* dst, const void* src_host, size_t bytes, tl_stream stream) {
    TL_CHECK_INIT();
    TL_CUDA(cudaMemcpyAsync(dst, src_host, bytes, cudaMemcpyHostToDevice, as_stream(stream)));
    return TL_OK;
}
int tl_memcpy_d2h(void* dst_host, const void* src, size_t bytes, tl_stream stream) {
    TL_CHECK_INIT();
    TL_CUDA(cudaMemcpyAsync(dst_host, src, bytes, cudaMemcpyDeviceToHost, as_stream(stream)));
    return TL_OK;
}
int tl_memcpy_d2d(void* dst, const void* src, size_t bytes, tl_stream stream) {
    TL_CHECK_INIT();
    TL_CUDA(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToDevice, as_stream(stream)));
    return TL_OK;
}
int tl_memset(void* dst, int value, size_t bytes, tl_stream stream) {
    TL_CHECK_INIT();
    TL_CUDA(cudaMemsetAsync(dst, value, bytes, as_stream(stream)));
    return TL_OK;
}
int tl_stream_synchronize(tl_stream stream) {
    TL_CHECK_INIT();
    TL_CUDA(cudaStreamSynchronize(as_stream(stream)));
    return TL_OK;
}
int tl_malloc_host(void** hptr, size_t bytes) {
    TL_CHECK_INIT();
    TL_REQUIRE(hptr != nullptr, "hptr is null");
    TL_CUDA(cudaMallocHost(hptr, bytes ? bytes : 1));
    return TL_OK;
}
int tl_free_host(void* hptr) {
    TL_CHECK_INIT();
    TL_CUDA(cudaFreeHost(hptr));
    return TL_OK;
}

}  // extern "C"
