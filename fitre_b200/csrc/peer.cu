// Small sum all-reduce over peer memory (NVLink / NVSwitch loads and stores, no library call).
//
// The data-parallel passes exchange about forty vectors of 2C..7C doubles per step (batch-norm
// statistics between the reduce and the apply pass of each fused kernel, the loss).  Each is far
// below the size at which a collective is bandwidth-bound: its cost is latency, and it sits on the
// critical path.  Every rank owns a mailbox in its own HBM that all peers have mapped
// (cudaIpcOpenMemHandle, set up in comm.cpp).  One kernel, the same launch that sums the slice
// partials of a channel pass, then
//   1. writes this rank's vector into its row of EVERY rank's mailbox (plain stores through the
//      peer mappings), fences, and raises its flag in every mailbox to the call's epoch;
//   2. waits until all flags of its OWN mailbox show the epoch (volatile loads of local memory);
//   3. adds the rows of its own mailbox in rank order, so every rank forms the same bits.
// Two mailbox halves alternate by epoch parity: a rank can be at most one call ahead of a peer,
// because finishing call e needs the peer's flag of call e.  The wait is bounded by a time limit;
// when it runs out the kernel records an error word and returns, and the host reports
// FITRE_ERR_COMM (no trap, no endless loop).  No TMA, no multicast: plain loads and stores.
#include "common.h"

namespace fitre {
namespace {

constexpr int kPeerThreads = 512;

struct PeerArgs {
    double *inbox[FITRE_PEER_MAX_RANKS];
    int rank, world;
    unsigned long long epoch;
    long long wait_ns;
    int *err;
};

__device__ __forceinline__ unsigned long long globaltimer_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

// partials != nullptr: value i = sum_j partials[((i / NS) * S + j) * NS + i % NS]  (slice sums of a
// channel pass); otherwise value i = io[i].  Result (sum over ranks) in io[0, n).
__global__ void __launch_bounds__(kPeerThreads)
peer_allreduce_kernel(const double *partials, int S, int NS, double *io, int n, PeerArgs p) {
    __shared__ int timed_out;
    const int tid = threadIdx.x;
    const int half = (int)(p.epoch & 1ull);
    const long row = (long)FITRE_PEER_MAX_DOUBLES;
    const long flags_at = 2L * p.world * row;  // doubles in front of the flag words
    if (tid == 0) timed_out = 0;
    for (int i = tid; i < n; i += kPeerThreads) {
        double s;
        if (partials) {
            const int c = i / NS, k = i - c * NS;
            s = 0.0;
            for (int j = 0; j < S; ++j) s += partials[((long)c * S + j) * NS + k];
        } else {
            s = io[i];
        }
        for (int r = 0; r < p.world; ++r) p.inbox[r][((long)half * p.world + p.rank) * row + i] = s;
    }
    __threadfence_system();
    __syncthreads();
    if (tid < p.world) {
        volatile unsigned long long *theirs =
            reinterpret_cast<volatile unsigned long long *>(p.inbox[tid] + flags_at) + half * p.world + p.rank;
        *theirs = p.epoch;
        volatile unsigned long long *mine =
            reinterpret_cast<volatile unsigned long long *>(p.inbox[p.rank] + flags_at) + half * p.world + tid;
        const unsigned long long t0 = globaltimer_ns();
        while (*mine != p.epoch) {
            if ((long long)(globaltimer_ns() - t0) > p.wait_ns) {
                timed_out = 1;
                break;
            }
            __nanosleep(64);
        }
    }
    __threadfence_system();
    __syncthreads();
    if (timed_out) {
        if (tid == 0) atomicExch(p.err, 2);
        return;
    }
    const double *own = p.inbox[p.rank] + (long)half * p.world * row;
    for (int i = tid; i < n; i += kPeerThreads) {
        double s = 0.0;
        for (int r = 0; r < p.world; ++r) s += __ldcg(own + r * row + i);  // peers wrote these: bypass L1
        io[i] = s;
    }
}

}  // namespace

bool peer_allreduce_ready(const fitre_context *ctx, long n) {
    return ctx->world > 1 && ctx->peer.enabled && n > 0 && n <= FITRE_PEER_MAX_DOUBLES;
}

// Sum over the ranks of a short vector: `io` (n doubles) or, with partials, the slice sums of a
// channel pass (C x S x NS partials -> C x NS values).  Caller checked peer_allreduce_ready.
void peer_allreduce(fitre_context *ctx, const double *partials, int S, int NS, double *io, int n) {
    PeerArgs a{};
    for (int r = 0; r < ctx->world; ++r) a.inbox[r] = ctx->peer.inbox[r];
    a.rank = ctx->rank;
    a.world = ctx->world;
    a.epoch = ++ctx->peer.epoch;
    a.wait_ns = ctx->peer.wait_ns;
    a.err = (int *)(ctx->dscal + 4000);
    peer_allreduce_kernel<<<1, kPeerThreads, 0, ctx->stream>>>(partials, S, NS, io, n, a);
    check_launch(ctx, "peer_allreduce_kernel");
}

// Self-test of the bounded wait on ONE GPU: a two-rank mailbox in this device's memory whose second
// flag nothing ever raises.  The kernel must come back after about wait_ms and leave the error word
// set; returns that word (2 = the wait ran out).  The context stays usable.
int peer_wait_selftest(fitre_context *ctx, double wait_ms) {
    double *box = nullptr;
    const size_t doubles = 2 * 2 * (size_t)FITRE_PEER_MAX_DOUBLES + 2 * 2;
    FITRE_CUDA(cudaMalloc((void **)&box, doubles * sizeof(double)));
    FITRE_CUDA(cudaMemsetAsync(box, 0, doubles * sizeof(double), ctx->stream));
    double *io = ctx->dscal + 3000;
    PeerArgs a{};
    a.inbox[0] = box;
    a.inbox[1] = box;   // "rank 1" never runs: its flag stays 0
    a.rank = 0;
    a.world = 2;
    a.epoch = 1;
    a.wait_ns = (long long)(wait_ms * 1e6);
    a.err = (int *)(ctx->dscal + 4000);
    peer_allreduce_kernel<<<1, kPeerThreads, 0, ctx->stream>>>(nullptr, 0, 1, io, 4, a);
    check_launch(ctx, "peer_allreduce_kernel");
    int word = 0;
    FITRE_CUDA(cudaMemcpyAsync(ctx->pinned + 204, ctx->dscal + 4000, sizeof(double), cudaMemcpyDeviceToHost, ctx->stream));
    FITRE_CUDA(cudaStreamSynchronize(ctx->stream));
    std::memcpy(&word, ctx->pinned + 204, sizeof(int));
    FITRE_CUDA(cudaMemsetAsync(ctx->dscal + 4000, 0, sizeof(double), ctx->stream));
    FITRE_CUDA(cudaStreamSynchronize(ctx->stream));
    cudaFree(box);
    return word;
}

}  // namespace fitre
