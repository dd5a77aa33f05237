// Tensor-parallel plumbing: one process per GPU, NCCL over NVLink.  The
// reference has no collective of any kind; this is the exchange step a
// K-sharded (row-parallel) palettized matmul needs.  NCCL is bound at run time
// (dlopen) so a single-GPU user needs no NCCL at all, and a process that
// already loaded NCCL (e.g. through torch) shares that copy.
#include <dlfcn.h>
#include <nccl.h>

#include <cstring>

#include "common.cuh"

struct prism_nccl_api {
    void *lib = nullptr;
    ncclResult_t (*GetUniqueId)(ncclUniqueId *) = nullptr;
    ncclResult_t (*CommInitRank)(ncclComm_t *, int, ncclUniqueId, int) = nullptr;
    ncclResult_t (*AllReduce)(const void *, void *, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t,
                              cudaStream_t) = nullptr;
    ncclResult_t (*AllGather)(const void *, void *, size_t, ncclDataType_t, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
    const char *(*GetErrorString)(ncclResult_t) = nullptr;
};

namespace prism {

static prism_nccl_api *load_nccl(std::string &err) {
    static prism_nccl_api api;
    static bool tried = false;
    if (tried) return api.lib ? &api : nullptr;
    tried = true;
    const char *names[] = {"libnccl.so.2", "libnccl.so"};
    void *lib = nullptr;
    for (const char *n : names) {
        lib = dlopen(n, RTLD_NOW | RTLD_NOLOAD | RTLD_GLOBAL);  // a copy the process already holds
        if (lib) break;
    }
    for (int i = 0; !lib && i < 2; i++) lib = dlopen(names[i], RTLD_NOW | RTLD_GLOBAL);
    if (!lib) {
        err = std::string("NCCL not found: ") + dlerror();
        return nullptr;
    }
#define LOAD(field, sym)                                                 \
    api.field = reinterpret_cast<decltype(api.field)>(dlsym(lib, sym)); \
    if (!api.field) {                                                    \
        err = std::string("NCCL symbol missing: ") + sym;                \
        return nullptr;                                                  \
    }
    LOAD(GetUniqueId, "ncclGetUniqueId");
    LOAD(CommInitRank, "ncclCommInitRank");
    LOAD(AllReduce, "ncclAllReduce");
    LOAD(AllGather, "ncclAllGather");
    LOAD(CommDestroy, "ncclCommDestroy");
    LOAD(GetErrorString, "ncclGetErrorString");
#undef LOAD
    api.lib = lib;
    return &api;
}

int tp_all_reduce_f32(prism_cuda_ctx *ctx, float *buf, size_t n) {
    if (ctx->tp_world <= 1) return PRISM_OK;
    ncclResult_t r = ctx->nccl->AllReduce(buf, buf, n, ncclFloat32, ncclSum, (ncclComm_t)ctx->nccl_comm, ctx->stream);
    if (r != ncclSuccess) return fail(ctx, PRISM_E_COMM, std::string("ncclAllReduce: ") + ctx->nccl->GetErrorString(r));
    ctx->launches++;
    return PRISM_OK;
}

int tp_all_gather_bytes(prism_cuda_ctx *ctx, const void *send, void *recv, size_t bytes_per_rank) {
    if (ctx->tp_world <= 1) return PRISM_OK;
    ncclResult_t r = ctx->nccl->AllGather(send, recv, bytes_per_rank, ncclUint8, (ncclComm_t)ctx->nccl_comm, ctx->stream);
    if (r != ncclSuccess) return fail(ctx, PRISM_E_COMM, std::string("ncclAllGather: ") + ctx->nccl->GetErrorString(r));
    ctx->launches++;
    return PRISM_OK;
}

}  // namespace prism

using namespace prism;

extern "C" void prism_tp_shutdown(prism_cuda_ctx *ctx) {
    if (ctx->nccl_comm && ctx->nccl) {
        ctx->nccl->CommDestroy((ncclComm_t)ctx->nccl_comm);
        ctx->nccl_comm = nullptr;
    }
}

extern "C" {

int prism_cuda_tp_unique_id(uint8_t id[PRISM_NCCL_ID_BYTES]) {
    if (!id) return PRISM_E_NULL;
    std::string err;
    prism_nccl_api *api = load_nccl(err);
    if (!api) return fail(nullptr, PRISM_E_COMM, err);
    static_assert(sizeof(ncclUniqueId) == PRISM_NCCL_ID_BYTES, "ncclUniqueId size");
    ncclUniqueId uid;
    ncclResult_t r = api->GetUniqueId(&uid);
    if (r != ncclSuccess) return fail(nullptr, PRISM_E_COMM, std::string("ncclGetUniqueId: ") + api->GetErrorString(r));
    memcpy(id, &uid, PRISM_NCCL_ID_BYTES);
    return PRISM_OK;
}

int prism_cuda_tp_init(prism_cuda_ctx *ctx, int world, int rank, const uint8_t id[PRISM_NCCL_ID_BYTES]) {
    if (!ctx || !id) return fail(ctx, PRISM_E_NULL, "null argument");
    if (world < 1 || rank < 0 || rank >= world) return fail(ctx, PRISM_E_ARG, "bad world/rank");
    if (ctx->nccl_comm) return fail(ctx, PRISM_E_STATE, "tensor parallel group already initialised");
    ctx->tp_world = world;
    ctx->tp_rank = rank;
    if (world == 1) return PRISM_OK;
    std::string err;
    prism_nccl_api *api = load_nccl(err);
    if (!api) return fail(ctx, PRISM_E_COMM, err);
    PRISM_CUDA_TRY(ctx, cudaSetDevice(ctx->device));
    ncclUniqueId uid;
    memcpy(&uid, id, PRISM_NCCL_ID_BYTES);
    ncclComm_t comm;
    ncclResult_t r = api->CommInitRank(&comm, world, uid, rank);
    if (r != ncclSuccess) {
        ctx->tp_world = 1;
        ctx->tp_rank = 0;
        return fail(ctx, PRISM_E_COMM, std::string("ncclCommInitRank: ") + api->GetErrorString(r));
    }
    ctx->nccl = api;
    ctx->nccl_comm = comm;
    return PRISM_OK;
}

int prism_cuda_tp_world(prism_cuda_ctx *ctx, int *world, int *rank) {
    if (!ctx) return PRISM_E_NULL;
    if (world) *world = ctx->tp_world;
    if (rank) *rank = ctx->tp_rank;
    return PRISM_OK;
}

int prism_cuda_tp_all_reduce_dev(prism_cuda_ctx *ctx, void *buf_dev, size_t n_halfs) {
    if (!ctx || !buf_dev) return fail(ctx, PRISM_E_NULL, "null argument");
    if (ctx->tp_world <= 1) return PRISM_OK;
    ncclResult_t r = ctx->nccl->AllReduce(buf_dev, buf_dev, n_halfs, ncclFloat16, ncclSum,
                                          (ncclComm_t)ctx->nccl_comm, ctx->stream);
    if (r != ncclSuccess) return fail(ctx, PRISM_E_COMM, std::string("ncclAllReduce: ") + ctx->nccl->GetErrorString(r));
    ctx->launches++;
    return PRISM_OK;
}

}  // extern "C"
