// NCCL communicator for the gradient all-reduce of the data-parallel training step.
// NovaNN is single process, so there is no reference counterpart; one process per GPU,
// the unique id travels over whatever side channel the launcher has (a store, a file).
// Everything else in the library shards by rows and needs no collective.
#include <nccl.h>
#include <string.h>

#include "nvq_common.cuh"

#define NVQ_NCCL(expr)                                                                  \
    do {                                                                                \
        ncclResult_t _r = (expr);                                                       \
        if (_r != ncclSuccess)                                                          \
            NVQ_FAIL(NVQ_ERR_NCCL, "%s failed: %s (%s:%d)", #expr, ncclGetErrorString(_r), \
                     __FILE__, __LINE__);                                               \
    } while (0)

static_assert(sizeof(ncclUniqueId) == NVQ_UNIQUE_ID_BYTES, "unique id size");

extern "C" nvq_status nvq_comm_unique_id(uint8_t id[NVQ_UNIQUE_ID_BYTES]) {
    NVQ_REQUIRE(id, "null id");
    ncclUniqueId u;
    NVQ_NCCL(ncclGetUniqueId(&u));
    memcpy(id, &u, sizeof(u));
    return NVQ_OK;
}

extern "C" nvq_status nvq_comm_init(const uint8_t id[NVQ_UNIQUE_ID_BYTES], int rank, int world,
                                    int device, void** comm) {
    NVQ_REQUIRE(id && comm && world > 0 && rank >= 0 && rank < world, "nvq_comm_init: bad argument");
    nvq_status s = nvq_use_device(device);
    if (s != NVQ_OK) return s;
    ncclUniqueId u;
    memcpy(&u, id, sizeof(u));
    ncclComm_t c;
    NVQ_NCCL(ncclCommInitRank(&c, world, u, rank));
    *comm = (void*)c;
    return NVQ_OK;
}

extern "C" nvq_status nvq_comm_destroy(void* comm) {
    if (!comm) return NVQ_OK;
    NVQ_NCCL(ncclCommDestroy((ncclComm_t)comm));
    return NVQ_OK;
}

extern "C" nvq_status nvq_allreduce_sum_f32(void* comm, float* d_buf, size_t n, int device,
                                            void* stream) {
    NVQ_REQUIRE(comm && (n == 0 || d_buf), "nvq_allreduce_sum_f32: bad argument");
    if (n == 0) return NVQ_OK;
    nvq_status s = nvq_use_device(device);
    if (s != NVQ_OK) return s;
    NVQ_NCCL(ncclAllReduce(d_buf, d_buf, n, ncclFloat, ncclSum, (ncclComm_t)comm, (cudaStream_t)stream));
    return NVQ_OK;
}
