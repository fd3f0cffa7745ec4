// Data-parallel gradient exchange: one NCCL communicator per context (one
// process per GPU), a single in-place sum all-reduce of the flat gradient
// bucket on the context's stream.  NCCL is resolved at run time with dlopen so
// that the library loads (and every single-GPU entry point works) on machines
// without it; a missing NCCL surfaces as KATSU_ERR_NCCL from these calls only.
#include <dlfcn.h>
#include <string.h>

#include "common.cuh"

namespace {

// Minimal mirror of the NCCL declarations used here (stable since NCCL 2.x).
typedef struct ncclComm *ncclComm_t;
typedef struct { char internal[128]; } ncclUniqueId;
typedef int ncclResult_t;  // 0 == ncclSuccess
const int kNcclFloat32 = 7;
const int kNcclSum = 0;

struct NcclApi {
    void *handle;
    ncclResult_t (*GetUniqueId)(ncclUniqueId *);
    ncclResult_t (*CommInitRank)(ncclComm_t *, int, ncclUniqueId, int);
    ncclResult_t (*CommDestroy)(ncclComm_t);
    ncclResult_t (*AllReduce)(const void *, void *, size_t, int, int, ncclComm_t, cudaStream_t);
    const char *(*GetErrorString)(ncclResult_t);
};

NcclApi g_nccl = {nullptr, nullptr, nullptr, nullptr, nullptr, nullptr};

int32_t load_nccl() {
    if (g_nccl.handle != nullptr) return KATSU_OK;
    // RTLD_NOLOAD first: reuse the copy a host framework already mapped.
    void *h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_NOLOAD);
    if (h == nullptr) h = dlopen("libnccl.so.2", RTLD_NOW);
    if (h == nullptr) h = dlopen("libnccl.so", RTLD_NOW);
    if (h == nullptr) return katsu_set_error(KATSU_ERR_NCCL, "libnccl.so.2 not found: %s", dlerror());
    NcclApi api;
    api.handle = h;
    api.GetUniqueId = (ncclResult_t(*)(ncclUniqueId *))dlsym(h, "ncclGetUniqueId");
    api.CommInitRank = (ncclResult_t(*)(ncclComm_t *, int, ncclUniqueId, int))dlsym(h, "ncclCommInitRank");
    api.CommDestroy = (ncclResult_t(*)(ncclComm_t))dlsym(h, "ncclCommDestroy");
    api.AllReduce = (ncclResult_t(*)(const void *, void *, size_t, int, int, ncclComm_t, cudaStream_t))dlsym(
        h, "ncclAllReduce");
    api.GetErrorString = (const char *(*)(ncclResult_t))dlsym(h, "ncclGetErrorString");
    if (!api.GetUniqueId || !api.CommInitRank || !api.CommDestroy || !api.AllReduce || !api.GetErrorString)
        return katsu_set_error(KATSU_ERR_NCCL, "libnccl.so.2 lacks an expected symbol");
    g_nccl = api;
    return KATSU_OK;
}

int32_t nccl_fail(const char *what, ncclResult_t rc) {
    return katsu_set_error(KATSU_ERR_NCCL, "%s: %s", what, g_nccl.GetErrorString(rc));
}

}  // namespace

extern "C" int32_t katsu_cuda_comm_unique_id(uint8_t out_id[KATSU_COMM_ID_BYTES]) {
    KATSU_REQUIRE(out_id != nullptr, "out_id is null");
    KATSU_TRY(load_nccl());
    ncclUniqueId id;
    ncclResult_t rc = g_nccl.GetUniqueId(&id);
    if (rc != 0) return nccl_fail("ncclGetUniqueId", rc);
    static_assert(sizeof(id) == KATSU_COMM_ID_BYTES, "unique id size");
    memcpy(out_id, &id, sizeof(id));
    return KATSU_OK;
}

extern "C" int32_t katsu_cuda_comm_init(katsu_cuda_ctx *ctx, const uint8_t id_bytes[KATSU_COMM_ID_BYTES],
                                        int32_t n_ranks, int32_t rank) {
    KATSU_TRY(katsu_bind(ctx));
    KATSU_REQUIRE(id_bytes != nullptr, "id is null");
    KATSU_REQUIRE(n_ranks >= 1 && rank >= 0 && rank < n_ranks, "bad rank / world size");
    KATSU_REQUIRE(ctx->comm == nullptr, "communicator already initialised");
    KATSU_TRY(load_nccl());
    ncclUniqueId id;
    memcpy(&id, id_bytes, sizeof(id));
    ncclComm_t comm = nullptr;
    ncclResult_t rc = g_nccl.CommInitRank(&comm, n_ranks, id, rank);
    if (rc != 0) return nccl_fail("ncclCommInitRank", rc);
    ctx->comm = comm;
    ctx->comm_ranks = n_ranks;
    ctx->comm_rank = rank;
    return KATSU_OK;
}

int32_t katsu_comm_destroy_impl(katsu_cuda_ctx *ctx) {
    if (ctx->comm != nullptr && g_nccl.handle != nullptr) g_nccl.CommDestroy((ncclComm_t)ctx->comm);
    ctx->comm = nullptr;
    ctx->comm_ranks = 0;
    return KATSU_OK;
}

extern "C" int32_t katsu_cuda_comm_destroy(katsu_cuda_ctx *ctx) {
    KATSU_TRY(katsu_bind(ctx));
    cudaStreamSynchronize(ctx->stream);
    return katsu_comm_destroy_impl(ctx);
}

extern "C" int32_t katsu_cuda_allreduce_sum(katsu_cuda_ctx *ctx, float *buf, size_t count) {
    KATSU_TRY(katsu_bind(ctx));
    KATSU_REQUIRE(ctx->comm != nullptr, "no communicator: call katsu_cuda_comm_init first");
    if (count == 0) return KATSU_OK;
    KATSU_REQUIRE(buf != nullptr, "buf is null");
    ncclResult_t rc = g_nccl.AllReduce(buf, buf, count, kNcclFloat32, kNcclSum, (ncclComm_t)ctx->comm, ctx->stream);
    if (rc != 0) return nccl_fail("ncclAllReduce", rc);
    return KATSU_OK;
}
