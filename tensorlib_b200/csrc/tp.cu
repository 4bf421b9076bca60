// Tensor parallelism for the Llama2 forward: one process per GPU, NCCL over NVLink.
//
// The reference has no multi-GPU code at all. The split follows the Megatron scheme its export
// script undoes when it concatenates Meta's shards (script/export.py:444-460): wq/wk/wv/w1/w3 by
// output rows (heads / hidden slice per rank, no communication after them), wo/w2 by input
// columns (each rank produces a full-width partial sum -> allreduce), classifier by vocabulary
// rows (allgather of the logit slices). Decode partial sums travel as fp32 and are rounded to
// fp16 once after the sum, so a p-GPU run differs from the 1-GPU run only by fp32 summation order.
//
// NCCL is bound at run time (dlopen in the first tl_tp_* call), not at link time: a single-GPU
// process never maps it, and in a process that already holds an NCCL (PyTorch bundles its own,
// newer than the system copy) the loader hands back that same library instead of a second one
// with the same soname, which would otherwise shadow the symbols of whoever loads it later.
#include <dlfcn.h>
#include <nccl.h>

#include <cstring>
#include <mutex>

#include "engine.cuh"

namespace tlb {
namespace {

struct NcclApi {
    decltype(&::ncclGetUniqueId) GetUniqueId = nullptr;
    decltype(&::ncclCommInitRank) CommInitRank = nullptr;
    decltype(&::ncclCommDestroy) CommDestroy = nullptr;
    decltype(&::ncclAllReduce) AllReduce = nullptr;
    decltype(&::ncclAllGather) AllGather = nullptr;
    decltype(&::ncclGetErrorString) GetErrorString = nullptr;
    bool ok = false;
    char why[256] = {0};
};
NcclApi g_nccl;
std::once_flag g_nccl_once;

const NcclApi& nccl() {
    std::call_once(g_nccl_once, [] {
        void* h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_LOCAL);
        if (!h) h = dlopen("libnccl.so", RTLD_NOW | RTLD_LOCAL);
        if (!h) { snprintf(g_nccl.why, sizeof g_nccl.why, "libnccl.so.2 not found: %s", dlerror()); return; }
        auto sym = [&](const char* name) { void* p = dlsym(h, name); if (!p) snprintf(g_nccl.why, sizeof g_nccl.why, "%s missing in libnccl", name); return p; };
        g_nccl.GetUniqueId = reinterpret_cast<decltype(g_nccl.GetUniqueId)>(sym("ncclGetUniqueId"));
        g_nccl.CommInitRank = reinterpret_cast<decltype(g_nccl.CommInitRank)>(sym("ncclCommInitRank"));
        g_nccl.CommDestroy = reinterpret_cast<decltype(g_nccl.CommDestroy)>(sym("ncclCommDestroy"));
        g_nccl.AllReduce = reinterpret_cast<decltype(g_nccl.AllReduce)>(sym("ncclAllReduce"));
        g_nccl.AllGather = reinterpret_cast<decltype(g_nccl.AllGather)>(sym("ncclAllGather"));
        g_nccl.GetErrorString = reinterpret_cast<decltype(g_nccl.GetErrorString)>(sym("ncclGetErrorString"));
        g_nccl.ok = g_nccl.GetUniqueId && g_nccl.CommInitRank && g_nccl.CommDestroy && g_nccl.AllReduce &&
                    g_nccl.AllGather && g_nccl.GetErrorString;
    });
    return g_nccl;
}

#define TL_NCCL_READY()                                                                       \
    do {                                                                                      \
        if (!nccl().ok) return ::tlb::set_error(TL_ERR_COMM, "NCCL is not available: %s", nccl().why); \
    } while (0)
#define TL_NCCL(call, ...)                                                                    \
    do {                                                                                      \
        ncclResult_t _r = nccl().call(__VA_ARGS__);                                           \
        if (_r != ncclSuccess)                                                                \
            return ::tlb::set_error(TL_ERR_COMM, "nccl%s failed: %s (%s:%d)", #call,          \
                                    nccl().GetErrorString(_r), __FILE__, __LINE__);           \
    } while (0)

class NcclCollective : public Collective {
public:
    ncclComm_t comm = nullptr;
    int rank = 0, world = 1;
    int allreduce_sum_f16(__half* buf, size_t n, cudaStream_t st) override {
        TL_NCCL(AllReduce, buf, buf, n, ncclHalf, ncclSum, comm, st);
        return TL_OK;
    }
    int allreduce_sum_f32(float* buf, size_t n, cudaStream_t st) override {
        TL_NCCL(AllReduce, buf, buf, n, ncclFloat, ncclSum, comm, st);
        return TL_OK;
    }
    int allgather_f16(const __half* send, __half* recv, size_t n_per_rank, cudaStream_t st) override {
        TL_NCCL(AllGather, send, recv, n_per_rank, ncclHalf, comm, st);
        return TL_OK;
    }
    bool graph_capturable() const override { return true; }
};

NcclCollective g_coll;

}  // namespace
}  // namespace tlb

using namespace tlb;

extern "C" {

int tl_tp_unique_id(void* out, int nbytes) {
    TL_REQUIRE(out && nbytes >= (int)sizeof(ncclUniqueId), "unique id buffer needs %zu bytes", sizeof(ncclUniqueId));
    TL_NCCL_READY();
    ncclUniqueId id;
    TL_NCCL(GetUniqueId, &id);
    memcpy(out, &id, sizeof id);
    return TL_OK;
}

int tl_tp_init(const void* unique_id, int nbytes, int rank, int world) {
    TL_CHECK_INIT();
    TL_REQUIRE(unique_id && nbytes >= (int)sizeof(ncclUniqueId) && world >= 1 && rank >= 0 && rank < world, "bad argument");
    TL_REQUIRE(g_coll.comm == nullptr, "tensor-parallel group already initialised");
    ncclUniqueId id;
    memcpy(&id, unique_id, sizeof id);
    TL_NCCL_READY();
    TL_NCCL(CommInitRank, &g_coll.comm, world, id, rank);
    g_coll.rank = rank;
    g_coll.world = world;
    return TL_OK;
}

int tl_tp_attach(tl_llama2* m) {
    TL_REQUIRE(m && g_coll.comm, "no model or no tensor-parallel group");
    TL_REQUIRE(m->eng->cfg().tp_world == g_coll.world && m->eng->cfg().tp_rank == g_coll.rank,
               "model shard (%d of %d) does not match the group (%d of %d)", m->eng->cfg().tp_rank,
               m->eng->cfg().tp_world, g_coll.rank, g_coll.world);
    m->eng->set_collective(&g_coll);
    return TL_OK;
}

int tl_tp_allreduce_f32(float* buf, size_t n, tl_stream stream) {
    TL_REQUIRE(g_coll.comm, "no tensor-parallel group");
    return g_coll.allreduce_sum_f32(buf, n, as_stream(stream));
}

// Fused exchange: every rank exports its receive region (64-byte IPC handle), the handles travel
// out of band, every rank opens all of them. From then on the decode step pushes partial sums
// with peer stores from inside the GEMV kernels instead of calling ncclAllReduce.
int tl_tp_exchange_export(tl_llama2* m, void* handle64, int nbytes) {
    TL_CHECK_INIT();
    TL_REQUIRE(m && handle64 && nbytes >= (int)sizeof(cudaIpcMemHandle_t), "handle buffer needs %zu bytes", sizeof(cudaIpcMemHandle_t));
    cudaIpcMemHandle_t h;
    TL_PROPAGATE(m->eng->xch_export(&h));
    memcpy(handle64, &h, sizeof h);
    return TL_OK;
}
int tl_tp_exchange_open(tl_llama2* m, const void* handles, int world) {
    TL_CHECK_INIT();
    TL_REQUIRE(m && handles && world >= 2 && world <= TL_MAX_TP, "bad argument");
    cudaIpcMemHandle_t h[TL_MAX_TP];
    memcpy(h, handles, sizeof(cudaIpcMemHandle_t) * world);
    return m->eng->xch_open(h, world);
}
int tl_tp_exchange_close(tl_llama2* m) {
    TL_REQUIRE(m, "null model");
    return m->eng->xch_close();
}

int tl_tp_destroy(void) {
    if (g_coll.comm) {
        if (nccl().ok) nccl().CommDestroy(g_coll.comm);
        g_coll.comm = nullptr;
    }
    return TL_OK;
}

// Host-only view of the sharding rule the loader applies (see shard_block in engine.cu).
int tl_tp_shard(int kind, int rows, int cols, int rank, int world, int* row0, int* nrows, int* col0, int* ncols) {
    return shard_block(kind, rows, cols, rank, world, row0, nrows, col0, ncols);
}

}  // extern "C"
