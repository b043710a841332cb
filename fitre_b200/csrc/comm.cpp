// Data-parallel plumbing: NCCL sum all-reduce of batch statistics, gradients and
// Hessian-vector products.  The reference is single-GPU (its only multi-device code is the
// disabled cudaMemcpyPeer offload of solvers/kfac_thread.cu:94-134), so this layer has no
// counterpart there.  NCCL is loaded at run time (dlopen) the first time a communicator is
// requested, so single-GPU users need no NCCL installation.
//
// Failure handling is on the host.  The communicator is created by a helper thread so that a
// peer that never joins costs a bounded wait and a status, not a hang.  With a communicator,
// every host wait on the context's stream polls the stream and ncclCommGetAsyncError; a
// reported error or an expired deadline aborts the communicator (ncclCommAbort stops NCCL's
// kernels, the CUDA context stays usable) and the call returns FITRE_ERR_COMM.
#include <dlfcn.h>

#include <chrono>
#include <condition_variable>
#include <cstdlib>
#include <cstring>
#include <memory>
#include <mutex>
#include <climits>
#include <thread>
#include <vector>

#include "common.h"

namespace fitre {

namespace {
// the slice of the NCCL C API used here (nccl.h, stable since NCCL 2.4)
typedef struct ncclComm *ncclComm_t;
typedef struct { char internal[128]; } ncclUniqueId;
typedef int ncclResult_t;
enum { ncclSuccess = 0, ncclInProgress = 7 };
enum { ncclChar = 0, ncclFloat64 = 8 };
enum { ncclSum = 0 };

// Leading fields of ncclConfig_t as published with NCCL 2.17 (nccl.h); the library reads `version`
// and gives every field that a newer layout adds its default.
struct CommConfig {
    size_t size;
    unsigned int magic, version;
    int blocking, cgaClusterSize, minCTAs, maxCTAs;
    const char *netName;
};
constexpr int kConfigUndef = INT_MIN;  // NCCL_CONFIG_UNDEF_INT

struct Api {
    void *handle = nullptr;
    ncclResult_t (*CommInitRankConfig)(ncclComm_t *, int, ncclUniqueId, int, CommConfig *) = nullptr;  // optional
    ncclResult_t (*GetUniqueId)(ncclUniqueId *) = nullptr;
    ncclResult_t (*CommInitRank)(ncclComm_t *, int, ncclUniqueId, int) = nullptr;
    ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
    ncclResult_t (*CommAbort)(ncclComm_t) = nullptr;
    ncclResult_t (*CommGetAsyncError)(ncclComm_t, ncclResult_t *) = nullptr;
    ncclResult_t (*AllReduce)(const void *, void *, size_t, int, int, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*Reduce)(const void *, void *, size_t, int, int, int, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*Broadcast)(const void *, void *, size_t, int, int, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*AllGather)(const void *, void *, size_t, int, ncclComm_t, cudaStream_t) = nullptr;  // optional
    const char *(*GetErrorString)(ncclResult_t) = nullptr;
};

Api &api() {
    static Api a;
    if (a.handle) return a;
    // FITRE_NCCL_LIBRARY names the library to load instead of the system's libnccl.so.2
    const char *over = std::getenv("FITRE_NCCL_LIBRARY");
    const char *names[] = {over && *over ? over : "libnccl.so.2", "libnccl.so"};
    for (const char *n : names) {
        a.handle = dlopen(n, RTLD_NOW | RTLD_GLOBAL);
        if (a.handle || (over && *over)) break;
    }
    FITRE_REQUIRE(a.handle != nullptr, FITRE_ERR_COMM, "cannot load the NCCL library (libnccl.so.2)");
    a.GetUniqueId = (decltype(a.GetUniqueId))dlsym(a.handle, "ncclGetUniqueId");
    a.CommInitRank = (decltype(a.CommInitRank))dlsym(a.handle, "ncclCommInitRank");
    a.CommInitRankConfig = (decltype(a.CommInitRankConfig))dlsym(a.handle, "ncclCommInitRankConfig");
    a.CommDestroy = (decltype(a.CommDestroy))dlsym(a.handle, "ncclCommDestroy");
    a.CommAbort = (decltype(a.CommAbort))dlsym(a.handle, "ncclCommAbort");
    a.CommGetAsyncError = (decltype(a.CommGetAsyncError))dlsym(a.handle, "ncclCommGetAsyncError");
    a.AllReduce = (decltype(a.AllReduce))dlsym(a.handle, "ncclAllReduce");
    a.Reduce = (decltype(a.Reduce))dlsym(a.handle, "ncclReduce");
    a.Broadcast = (decltype(a.Broadcast))dlsym(a.handle, "ncclBroadcast");
    a.AllGather = (decltype(a.AllGather))dlsym(a.handle, "ncclAllGather");
    a.GetErrorString = (decltype(a.GetErrorString))dlsym(a.handle, "ncclGetErrorString");
    const bool ok = a.GetUniqueId && a.CommInitRank && a.CommDestroy && a.CommAbort && a.CommGetAsyncError &&
                    a.AllReduce && a.Reduce && a.Broadcast;
    if (!ok) {
        a.handle = nullptr;
        throw Error(FITRE_ERR_COMM, "the NCCL library lacks a required symbol");
    }
    return a;
}

std::string nccl_text(ncclResult_t r) {
    const char *s = api().GetErrorString ? api().GetErrorString(r) : nullptr;
    return s ? s : ("NCCL result " + std::to_string(r));
}

void check(ncclResult_t r, const char *what) {
    if (r != ncclSuccess) throw Error(FITRE_ERR_COMM, std::string(what) + ": " + nccl_text(r));
}

// State shared with the set-up thread; it outlives the context when the set-up never returns.
struct InitJob {
    std::mutex mu;
    std::condition_variable cv;
    bool done = false, abandoned = false;
    ncclResult_t result = ncclSuccess;
    ncclComm_t comm = nullptr;
};
}  // namespace

struct Comm {
    ncclComm_t comm = nullptr;    // collectives on the context's stream (batch statistics, scalars, factors)
    // A second communicator on a stream of its own carries the all-reduces of finished slices of
    // the gradient / Hessian-vector product while the backward sweep goes on; two communicators,
    // because collectives of one communicator run in issue order whatever their streams.
    ncclComm_t side = nullptr;
    cudaStream_t side_stream = nullptr;
    cudaEvent_t ev_ready[32] = {};  // "slice is written" (context stream -> side stream)
    cudaEvent_t ev_done = nullptr;  // "all slices are reduced" (side stream -> context stream)
    int next_ev = 0;
    bool pending = false;
    bool aborted = false;
};

namespace {
// Stops NCCL's work on this communicator and marks it unusable; later collectives fail fast.
void abort_comm(fitre_context *ctx) {
    if (!ctx->comm || ctx->comm->aborted) return;
    ctx->comm->aborted = true;
    if (ctx->comm->comm) api().CommAbort(ctx->comm->comm);
    if (ctx->comm->side) api().CommAbort(ctx->comm->side);
    ctx->comm->comm = ctx->comm->side = nullptr;
    ctx->peer.enabled = false;
}

ncclComm_t live_comm(fitre_context *ctx) {
    FITRE_REQUIRE(ctx->comm && !ctx->comm->aborted && ctx->comm->comm, FITRE_ERR_COMM,
                  "the communicator was aborted after an error; create a new one with fitre_comm_init");
    return ctx->comm->comm;
}
}  // namespace

void comm_allreduce_sum(fitre_context *ctx, double *dev_buf, size_t n) {
    if (ctx->world <= 1 || !ctx->comm || n == 0) return;
    check(api().AllReduce(dev_buf, dev_buf, n, ncclFloat64, ncclSum, live_comm(ctx), ctx->stream), "ncclAllReduce");
    ctx->launches += 1;  // NCCL's kernel; counted so the launch figure covers the whole step
}

bool comm_has_allgather() { return api().AllGather != nullptr; }

bool comm_allgather_inplace(fitre_context *ctx, double *dev_buf, size_t chunk, cudaStream_t stream) {
    if (ctx->world <= 1 || !ctx->comm || chunk == 0) return true;
    if (!api().AllGather) return false;
    check(api().AllGather(dev_buf + (size_t)ctx->rank * chunk, dev_buf, chunk, ncclFloat64, live_comm(ctx), stream),
          "ncclAllGather");
    ctx->launches += 1;
    return true;
}

// sum over the ranks, result on `root` only (the buffers of the other ranks are left as they were)
void comm_reduce_sum(fitre_context *ctx, double *dev_buf, size_t n, int root) {
    if (ctx->world <= 1 || !ctx->comm || n == 0) return;
    check(api().Reduce(dev_buf, dev_buf, n, ncclFloat64, ncclSum, root, live_comm(ctx), ctx->stream), "ncclReduce");
    ctx->launches += 1;
}

void comm_allreduce_small(fitre_context *ctx, double *dev_buf, size_t n) {
    if (ctx->world <= 1 || !ctx->comm || n == 0) return;
    if (peer_allreduce_ready(ctx, (long)n)) {
        live_comm(ctx);
        peer_allreduce(ctx, nullptr, 0, 1, dev_buf, (int)n);
    } else {
        comm_allreduce_sum(ctx, dev_buf, n);
    }
}

// All-reduce of dev_buf[0, n) on the side communicator and stream, ordered after everything queued
// on the context's stream so far; the context's stream does not wait for it until comm_async_join.
void comm_allreduce_async(fitre_context *ctx, double *dev_buf, size_t n) {
    if (ctx->world <= 1 || !ctx->comm || n == 0) return;
    live_comm(ctx);
    Comm *c = ctx->comm;
    if (!c->side) {  // no side communicator: the plain ordered all-reduce
        comm_allreduce_sum(ctx, dev_buf, n);
        return;
    }
    cudaEvent_t &ev = c->ev_ready[c->next_ev++ & 31];
    if (!ev) FITRE_CUDA(cudaEventCreateWithFlags(&ev, cudaEventDisableTiming));
    FITRE_CUDA(cudaEventRecord(ev, ctx->stream));
    FITRE_CUDA(cudaStreamWaitEvent(c->side_stream, ev, 0));
    check(api().AllReduce(dev_buf, dev_buf, n, ncclFloat64, ncclSum, c->side, c->side_stream), "ncclAllReduce");
    c->pending = true;
    ctx->launches += 1;
}

// The stream that carries the asynchronous slice all-reduces (NULL without one).
cudaStream_t comm_async_stream(fitre_context *ctx) {
    return (ctx->world > 1 && ctx->comm && ctx->comm->side) ? ctx->comm->side_stream : nullptr;
}

// Makes the context's stream wait for every all-reduce started by comm_allreduce_async.
void comm_async_join(fitre_context *ctx) {
    if (ctx->world <= 1 || !ctx->comm || !ctx->comm->pending) return;
    Comm *c = ctx->comm;
    c->pending = false;
    if (c->aborted || !c->side) return;
    FITRE_CUDA(cudaEventRecord(c->ev_done, c->side_stream));
    FITRE_CUDA(cudaStreamWaitEvent(ctx->stream, c->ev_done, 0));
}

// Host wait for everything queued on `stream` (the context's stream, or another stream whose
// work depends on it).  Without a communicator this is cudaStreamSynchronize.  With one, the
// stream is polled together with the communicator's asynchronous error state, for at most
// ctx->comm_timeout_s seconds: a lost peer leaves NCCL's kernel spinning on the device, which a
// plain synchronize would wait for without end.
void stream_wait(fitre_context *ctx, cudaStream_t stream) {
    if (ctx->world <= 1 || !ctx->comm || ctx->comm->aborted) {
        FITRE_CUDA(cudaStreamSynchronize(stream));
        return;
    }
    using clock = std::chrono::steady_clock;
    const auto deadline = clock::now() + std::chrono::duration<double>(ctx->comm_timeout_s);
    long spins = 0;
    for (;;) {
        const cudaError_t e = cudaStreamQuery(stream);
        if (e == cudaSuccess) return;
        if (e != cudaErrorNotReady)
            throw Error(FITRE_ERR_CUDA, std::string("cudaStreamQuery: ") + cudaGetErrorString(e));
        ++spins;
        if ((spins & 63) == 0) {
            ncclResult_t state = ncclSuccess;
            ncclResult_t q = api().CommGetAsyncError(ctx->comm->comm, &state);
            if (q == ncclSuccess && (state == ncclSuccess || state == ncclInProgress) && ctx->comm->side)
                q = api().CommGetAsyncError(ctx->comm->side, &state);
            if (q != ncclSuccess || (state != ncclSuccess && state != ncclInProgress)) {
                const std::string why = nccl_text(q != ncclSuccess ? q : state);
                abort_comm(ctx);
                throw Error(FITRE_ERR_COMM, "NCCL reported an asynchronous error: " + why);
            }
            if (clock::now() > deadline) {
                abort_comm(ctx);
                throw Error(FITRE_ERR_COMM, "a collective did not finish within " +
                                                std::to_string(ctx->comm_timeout_s) +
                                                " s (lost peer?); the communicator was aborted");
            }
        }
        if (spins > 4096)
            std::this_thread::sleep_for(std::chrono::microseconds(20));
        else
            std::this_thread::yield();
    }
}

namespace {
void peer_teardown(fitre_context *ctx) {
    ctx->peer.enabled = false;
    for (int r = 0; r < FITRE_PEER_MAX_RANKS; ++r) {
        if (!ctx->peer.inbox[r]) continue;
        if (r == ctx->rank) cudaFree(ctx->peer.inbox[r]);
        else cudaIpcCloseMemHandle(ctx->peer.inbox[r]);
        ctx->peer.inbox[r] = nullptr;
    }
    cudaGetLastError();
}

// Mailboxes of the peer-memory all-reduce (peer.cu): every rank allocates one, the IPC handles go
// round through NCCL, every rank maps every other mailbox.  Best effort and all-or-nothing: the
// ranks agree (one all-reduce of a success flag) and use NCCL for the short vectors otherwise.
// FITRE_PEER_REDUCE=0 switches it off.
void peer_setup(fitre_context *ctx) {
    Api &a = api();
    const char *sw = std::getenv("FITRE_PEER_REDUCE");
    if ((sw && sw[0] == '0') || !a.AllGather || ctx->world > FITRE_PEER_MAX_RANKS) return;
    const int W = ctx->world, me = ctx->rank;
    const size_t doubles = 2 * (size_t)W * FITRE_PEER_MAX_DOUBLES + 2 * (size_t)W;
    bool ok = true;
    double *own = nullptr;
    char *stage = nullptr;  // [W + 1] handles of 64 bytes: gathered ones, then this rank's
    cudaIpcMemHandle_t mine;
    std::vector<cudaIpcMemHandle_t> all(W);
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
    FITRE_CUDA(cudaMalloc((void **)&own, doubles * sizeof(double)));
    ctx->peer.inbox[me] = own;
    FITRE_CUDA(cudaMemsetAsync(own, 0, doubles * sizeof(double), ctx->stream));
    FITRE_CUDA(cudaMalloc((void **)&stage, (size_t)(W + 1) * 64));
    std::memset(&mine, 0, sizeof(mine));
    if (cudaIpcGetMemHandle(&mine, own) != cudaSuccess) {
        cudaGetLastError();
        ok = false;
    }
    FITRE_CUDA(cudaMemcpyAsync(stage + (size_t)W * 64, &mine, 64, cudaMemcpyHostToDevice, ctx->stream));
    check(a.AllGather(stage + (size_t)W * 64, stage, 64, ncclChar, ctx->comm->comm, ctx->stream), "ncclAllGather");
    FITRE_CUDA(cudaMemcpyAsync(all.data(), stage, (size_t)W * 64, cudaMemcpyDeviceToHost, ctx->stream));
    stream_wait(ctx, ctx->stream);
    for (int r = 0; r < W && ok; ++r) {
        if (r == me) continue;
        void *p = nullptr;
        if (cudaIpcOpenMemHandle(&p, all[r], cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) {
            cudaGetLastError();
            ok = false;
        } else {
            ctx->peer.inbox[r] = (double *)p;
        }
    }
    double flag = ok ? 1.0 : 0.0;
    FITRE_CUDA(cudaMemcpyAsync(ctx->dscal + 3990, &flag, sizeof(double), cudaMemcpyHostToDevice, ctx->stream));
    comm_allreduce_sum(ctx, ctx->dscal + 3990, 1);
    FITRE_CUDA(cudaMemcpyAsync(&flag, ctx->dscal + 3990, sizeof(double), cudaMemcpyDeviceToHost, ctx->stream));
    stream_wait(ctx, ctx->stream);
    cudaFree(stage);
    if (flag == (double)W) {
        ctx->peer.enabled = true;
        ctx->peer.epoch = 0;
        const double lim = ctx->comm_timeout_s < 30.0 ? ctx->comm_timeout_s : 30.0;
        ctx->peer.wait_ns = (long long)(lim * 1e9);
    } else {
        peer_teardown(ctx);
    }
}
}  // namespace

void comm_destroy(fitre_context *ctx) {
    peer_teardown(ctx);
    if (ctx->comm) {
        if (ctx->comm->side && !ctx->comm->aborted) api().CommDestroy(ctx->comm->side);
        if (ctx->comm->comm && !ctx->comm->aborted) api().CommDestroy(ctx->comm->comm);
        if (ctx->comm->side_stream) cudaStreamDestroy(ctx->comm->side_stream);
        for (cudaEvent_t e : ctx->comm->ev_ready)
            if (e) cudaEventDestroy(e);
        if (ctx->comm->ev_done) cudaEventDestroy(ctx->comm->ev_done);
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

namespace {
// ncclCommInitRank blocks until every rank has joined.  It runs on a helper thread; the caller
// waits for it at most comm_timeout_s seconds.  If the time runs out the job is abandoned: should
// the set-up ever return, the helper aborts the communicator it got.
// max_ctas > 0 caps the thread blocks this communicator's kernels may occupy (ncclConfig_t's
// maxCTAs) when the library has ncclCommInitRankConfig.
ncclComm_t bounded_init(fitre_context *ctx, const ncclUniqueId &id, int rank, int world, int max_ctas = 0) {
    Api &a = api();
    auto job = std::make_shared<InitJob>();
    const int device = ctx->device;
    std::thread([job, id, rank, world, device, max_ctas, &a]() {
        cudaSetDevice(device);
        ncclComm_t c = nullptr;
        ncclResult_t r;
        if (max_ctas > 0 && a.CommInitRankConfig) {
            CommConfig cfg{sizeof(CommConfig), 0xcafebeefu, 21700u, kConfigUndef, kConfigUndef, 1, max_ctas, nullptr};
            r = a.CommInitRankConfig(&c, world, id, rank, &cfg);
        } else {
            r = a.CommInitRank(&c, world, id, rank);
        }
        std::unique_lock<std::mutex> lk(job->mu);
        job->result = r;
        job->comm = c;
        job->done = true;
        if (job->abandoned && r == ncclSuccess && c) a.CommAbort(c);
        lk.unlock();
        job->cv.notify_all();
    }).detach();
    {
        std::unique_lock<std::mutex> lk(job->mu);
        const bool in_time = job->cv.wait_for(lk, std::chrono::duration<double>(ctx->comm_timeout_s),
                                              [&] { return job->done; });
        if (!in_time) {
            job->abandoned = true;
            throw Error(FITRE_ERR_COMM, "communicator set-up did not finish within " +
                                            std::to_string(ctx->comm_timeout_s) +
                                            " s: a rank did not join");
        }
    }
    check(job->result, "ncclCommInitRank");
    return job->comm;
}
}  // namespace

void comm_init(fitre_context *ctx, const void *id128, int rank, int world) {
    FITRE_REQUIRE(world >= 1 && rank >= 0 && rank < world, FITRE_ERR_BAD_ARG, "bad rank/world");
    comm_destroy(ctx);
    if (world == 1) return;
    Api &a = api();
    ncclUniqueId id;
    std::memcpy(&id, id128, sizeof(id));
    FITRE_CUDA(cudaSetDevice(ctx->device));
    ctx->comm = new Comm();
    ctx->comm->comm = bounded_init(ctx, id, rank, world);
    ctx->rank = rank;
    ctx->world = world;
    // The side communicator: rank 0 draws a second id and hands it round through the first one.
    // FITRE_SIDE_COMM=0 keeps a single communicator (slices are then reduced in stream order).
    const char *sw = std::getenv("FITRE_SIDE_COMM");
    try {
        if (sw && sw[0] == '0') {
            peer_setup(ctx);
            return;
        }
        ncclUniqueId id2;
        std::memset(&id2, 0, sizeof(id2));
        if (rank == 0) check(a.GetUniqueId(&id2), "ncclGetUniqueId");
        char *dev = reinterpret_cast<char *>(ctx->dscal + 3900);  // 128 bytes of the scalar slab
        FITRE_CUDA(cudaMemcpyAsync(dev, &id2, sizeof(id2), cudaMemcpyHostToDevice, ctx->stream));
        check(a.Broadcast(dev, dev, sizeof(id2), ncclChar, 0, ctx->comm->comm, ctx->stream), "ncclBroadcast");
        FITRE_CUDA(cudaMemcpyAsync(&id2, dev, sizeof(id2), cudaMemcpyDeviceToHost, ctx->stream));
        stream_wait(ctx, ctx->stream);
        FITRE_CUDA(cudaMemsetAsync(dev, 0, sizeof(id2), ctx->stream));
        // Its all-reduces run under the backward sweep, whose convolution kernels want every SM:
        // a few thread blocks are enough for 74 MB per pass (FITRE_SIDE_COMM_CTAS, 0 = NCCL's choice).
        int side_ctas = 4;
        if (const char *e = std::getenv("FITRE_SIDE_COMM_CTAS")) side_ctas = std::atoi(e);
        ctx->comm->side = bounded_init(ctx, id2, rank, world, side_ctas);
        FITRE_CUDA(cudaStreamCreateWithFlags(&ctx->comm->side_stream, cudaStreamNonBlocking));
        FITRE_CUDA(cudaEventCreateWithFlags(&ctx->comm->ev_done, cudaEventDisableTiming));
        peer_setup(ctx);
    } catch (...) {
        comm_destroy(ctx);
        throw;
    }
}

}  // namespace fitre
