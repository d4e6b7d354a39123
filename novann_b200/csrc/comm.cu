// NCCL communicator for the gradient all-reduce of the data-parallel training step.
// NovaNN is single process, so there is no reference counterpart; one process per GPU,
// the unique id travels over whatever side channel the launcher has (a store, a file).
// Everything else in the library shards by rows and needs no collective.
//
// NCCL is bound at run time (dlopen), not at link time: a process that also imports PyTorch
// must end up with ONE libnccl.so.2, and PyTorch insists on the version it ships.  The
// library named by NVQ_NCCL_LIB is tried first (the Python binding points it at the copy
// bundled with PyTorch when there is one), then whatever "libnccl.so.2" resolves to.
#include <dlfcn.h>
#include <nccl.h>
#include <stdlib.h>
#include <string.h>

#include <chrono>
#include <mutex>
#include <thread>

#include "nvq_common.cuh"

namespace {
struct Nccl {
    ncclResult_t (*GetUniqueId)(ncclUniqueId*);
    ncclResult_t (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int);
    ncclResult_t (*CommDestroy)(ncclComm_t);
    ncclResult_t (*AllReduce)(const void*, void*, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t,
                              cudaStream_t);
    const char* (*GetErrorString)(ncclResult_t);
    ncclResult_t (*CommGetAsyncError)(ncclComm_t, ncclResult_t*);
    ncclResult_t (*CommAbort)(ncclComm_t);
    bool ok = false;
} g_nccl;
std::mutex g_nccl_mu;

nvq_status load_nccl() {
    std::lock_guard<std::mutex> lock(g_nccl_mu);
    if (g_nccl.ok) return NVQ_OK;
    void* h = nullptr;
    if (const char* path = getenv("NVQ_NCCL_LIB")) h = dlopen(path, RTLD_NOW | RTLD_GLOBAL);
    if (!h) h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
    if (!h) NVQ_FAIL(NVQ_ERR_NCCL, "cannot load NCCL: %s", dlerror());
    g_nccl.GetUniqueId = (decltype(g_nccl.GetUniqueId))dlsym(h, "ncclGetUniqueId");
    g_nccl.CommInitRank = (decltype(g_nccl.CommInitRank))dlsym(h, "ncclCommInitRank");
    g_nccl.CommDestroy = (decltype(g_nccl.CommDestroy))dlsym(h, "ncclCommDestroy");
    g_nccl.AllReduce = (decltype(g_nccl.AllReduce))dlsym(h, "ncclAllReduce");
    g_nccl.GetErrorString = (decltype(g_nccl.GetErrorString))dlsym(h, "ncclGetErrorString");
    g_nccl.CommGetAsyncError = (decltype(g_nccl.CommGetAsyncError))dlsym(h, "ncclCommGetAsyncError");
    g_nccl.CommAbort = (decltype(g_nccl.CommAbort))dlsym(h, "ncclCommAbort");
    if (!g_nccl.GetUniqueId || !g_nccl.CommInitRank || !g_nccl.CommDestroy || !g_nccl.AllReduce ||
        !g_nccl.GetErrorString || !g_nccl.CommGetAsyncError || !g_nccl.CommAbort)
        NVQ_FAIL(NVQ_ERR_NCCL, "NCCL library lacks a required symbol");
    g_nccl.ok = true;
    return NVQ_OK;
}
}  // namespace

#define NVQ_NCCL_LOAD()                 \
    do {                                \
        nvq_status _s = load_nccl();    \
        if (_s != NVQ_OK) return _s;    \
    } while (0)

#define NVQ_NCCL(expr)                                                                  \
    do {                                                                                \
        ncclResult_t _r = (expr);                                                       \
        if (_r != ncclSuccess)                                                          \
            NVQ_FAIL(NVQ_ERR_NCCL, "%s failed: %s (%s:%d)", #expr, g_nccl.GetErrorString(_r), \
                     __FILE__, __LINE__);                                               \
    } while (0)

static_assert(sizeof(ncclUniqueId) == NVQ_UNIQUE_ID_BYTES, "unique id size");

extern "C" nvq_status nvq_comm_unique_id(uint8_t id[NVQ_UNIQUE_ID_BYTES]) {
    NVQ_REQUIRE(id, "null id");
    NVQ_NCCL_LOAD();
    ncclUniqueId u;
    NVQ_NCCL(g_nccl.GetUniqueId(&u));
    memcpy(id, &u, sizeof(u));
    return NVQ_OK;
}

extern "C" nvq_status nvq_comm_init(const uint8_t id[NVQ_UNIQUE_ID_BYTES], int rank, int world,
                                    int device, void** comm) {
    NVQ_REQUIRE(id && comm && world > 0 && rank >= 0 && rank < world, "nvq_comm_init: bad argument");
    NVQ_NCCL_LOAD();
    nvq_status s = nvq_use_device(device);
    if (s != NVQ_OK) return s;
    ncclUniqueId u;
    memcpy(&u, id, sizeof(u));
    ncclComm_t c;
    NVQ_NCCL(g_nccl.CommInitRank(&c, world, u, rank));
    *comm = (void*)c;
    return NVQ_OK;
}

extern "C" nvq_status nvq_comm_destroy(void* comm) {
    if (!comm) return NVQ_OK;
    NVQ_NCCL_LOAD();
    NVQ_NCCL(g_nccl.CommDestroy((ncclComm_t)comm));
    return NVQ_OK;
}

extern "C" nvq_status nvq_allreduce_sum_f32(void* comm, float* d_buf, size_t n, int device,
                                            void* stream) {
    NVQ_REQUIRE(comm && (n == 0 || d_buf), "nvq_allreduce_sum_f32: bad argument");
    if (n == 0) return NVQ_OK;
    nvq_status s = nvq_use_device(device);
    if (s != NVQ_OK) return s;
    NVQ_NCCL_LOAD();
    NVQ_NCCL(g_nccl.AllReduce(d_buf, d_buf, n, ncclFloat, ncclSum, (ncclComm_t)comm, (cudaStream_t)stream));
    return NVQ_OK;
}

// Host-side watchdog: the stream is polled with cudaStreamQuery (never a blocking wait, so a
// collective whose partner is missing cannot hold this thread) and the communicator's
// asynchronous error state is read between polls.
extern "C" nvq_status nvq_comm_wait(void* comm, int device, void* stream, uint32_t timeout_ms) {
    NVQ_REQUIRE(comm, "nvq_comm_wait: null communicator");
    NVQ_NCCL_LOAD();
    NVQ_CUDA(cudaSetDevice(device));
    const auto t0 = std::chrono::steady_clock::now();
    for (;;) {
        cudaError_t q = cudaStreamQuery((cudaStream_t)stream);
        if (q == cudaSuccess) return NVQ_OK;
        if (q != cudaErrorNotReady)
            NVQ_FAIL(NVQ_ERR_CUDA, "nvq_comm_wait: stream failed: %s", cudaGetErrorString(q));
        ncclResult_t async = ncclSuccess;
        NVQ_NCCL(g_nccl.CommGetAsyncError((ncclComm_t)comm, &async));
        if (async != ncclSuccess && async != ncclInProgress)
            NVQ_FAIL(NVQ_ERR_NCCL, "nvq_comm_wait: NCCL reported %s", g_nccl.GetErrorString(async));
        const auto ms = std::chrono::duration_cast<std::chrono::milliseconds>(
                            std::chrono::steady_clock::now() - t0).count();
        if ((uint64_t)ms >= timeout_ms)
            NVQ_FAIL(NVQ_ERR_TIMEOUT, "nvq_comm_wait: collective still pending after %u ms", timeout_ms);
        std::this_thread::sleep_for(std::chrono::microseconds(ms < 2 ? 20 : 200));
    }
}

extern "C" nvq_status nvq_comm_abort(void* comm) {
    if (!comm) return NVQ_OK;
    NVQ_NCCL_LOAD();
    NVQ_NCCL(g_nccl.CommAbort((ncclComm_t)comm));
    return NVQ_OK;
}
