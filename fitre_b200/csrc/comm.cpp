// Data-parallel plumbing: NCCL sum all-reduce of batch statistics, gradients and
// Hessian-vector products.  The reference is single-GPU (its only multi-device code is the
// disabled cudaMemcpyPeer offload of solvers/kfac_thread.cu:94-134), so this layer has no
// counterpart there.  NCCL is loaded at run time (dlopen) the first time a communicator is
// requested, so single-GPU users need no NCCL installation.
#include <dlfcn.h>

#include <cstring>

#include "common.h"

namespace fitre {

namespace {
// the slice of the NCCL C API used here (nccl.h, stable since NCCL 2.0)
typedef struct ncclComm *ncclComm_t;
typedef struct { char internal[128]; } ncclUniqueId;
typedef int ncclResult_t;
enum { ncclSuccess = 0 };
enum { ncclFloat64 = 8 };
enum { ncclSum = 0 };

struct Api {
    void *handle = nullptr;
    ncclResult_t (*GetUniqueId)(ncclUniqueId *) = nullptr;
    ncclResult_t (*CommInitRank)(ncclComm_t *, int, ncclUniqueId, int) = nullptr;
    ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
    ncclResult_t (*AllReduce)(const void *, void *, size_t, int, int, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*Reduce)(const void *, void *, size_t, int, int, int, ncclComm_t, cudaStream_t) = nullptr;
    const char *(*GetErrorString)(ncclResult_t) = nullptr;
};

Api &api() {
    static Api a;
    if (a.handle) return a;
    const char *names[] = {"libnccl.so.2", "libnccl.so"};
    for (const char *n : names) {
        a.handle = dlopen(n, RTLD_NOW | RTLD_GLOBAL);
        if (a.handle) break;
    }
    FITRE_REQUIRE(a.handle != nullptr, FITRE_ERR_COMM, "cannot load libnccl.so.2");
    a.GetUniqueId = (decltype(a.GetUniqueId))dlsym(a.handle, "ncclGetUniqueId");
    a.CommInitRank = (decltype(a.CommInitRank))dlsym(a.handle, "ncclCommInitRank");
    a.CommDestroy = (decltype(a.CommDestroy))dlsym(a.handle, "ncclCommDestroy");
    a.AllReduce = (decltype(a.AllReduce))dlsym(a.handle, "ncclAllReduce");
    a.Reduce = (decltype(a.Reduce))dlsym(a.handle, "ncclReduce");
    a.GetErrorString = (decltype(a.GetErrorString))dlsym(a.handle, "ncclGetErrorString");
    FITRE_REQUIRE(a.GetUniqueId && a.CommInitRank && a.CommDestroy && a.AllReduce && a.Reduce,
                  FITRE_ERR_COMM, "libnccl lacks a required symbol");
    return a;
}

void check(ncclResult_t r, const char *what) {
    if (r != ncclSuccess) {
        const char *s = api().GetErrorString ? api().GetErrorString(r) : "?";
        throw Error(FITRE_ERR_COMM, std::string(what) + ": " + s);
    }
}
}  // namespace

struct Comm {
    ncclComm_t comm = nullptr;
};

void comm_allreduce_sum(fitre_context *ctx, double *dev_buf, size_t n) {
    if (ctx->world <= 1 || !ctx->comm || n == 0) return;
    check(api().AllReduce(dev_buf, dev_buf, n, ncclFloat64, ncclSum, ctx->comm->comm, ctx->stream),
          "ncclAllReduce");
    ctx->launches += 1;  // NCCL's kernel; counted so the launch figure covers the whole step
}

// sum over the ranks, result on `root` only (the buffers of the other ranks are left as they were)
void comm_reduce_sum(fitre_context *ctx, double *dev_buf, size_t n, int root) {
    if (ctx->world <= 1 || !ctx->comm || n == 0) return;
    check(api().Reduce(dev_buf, dev_buf, n, ncclFloat64, ncclSum, root, ctx->comm->comm, ctx->stream), "ncclReduce");
    ctx->launches += 1;
}

void comm_destroy(fitre_context *ctx) {
    if (ctx->comm) {
        if (ctx->comm->comm) api().CommDestroy(ctx->comm->comm);
        delete ctx->comm;
        ctx->comm = nullptr;
    }
    ctx->world = 1;
    ctx->rank = 0;
}

void comm_unique_id(void *out128) {
    ncclUniqueId id;
    check(api().GetUniqueId(&id), "ncclGetUniqueId");
    std::memcpy(out128, &id, sizeof(id));
}

void comm_init(fitre_context *ctx, const void *id128, int rank, int world) {
    FITRE_REQUIRE(world >= 1 && rank >= 0 && rank < world, FITRE_ERR_BAD_ARG, "bad rank/world");
    comm_destroy(ctx);
    if (world == 1) return;
    ncclUniqueId id;
    std::memcpy(&id, id128, sizeof(id));
    FITRE_CUDA(cudaSetDevice(ctx->device));
    ctx->comm = new Comm();
    check(api().CommInitRank(&ctx->comm->comm, world, id, rank), "ncclCommInitRank");
    ctx->rank = rank;
    ctx->world = world;
}

}  // namespace fitre
