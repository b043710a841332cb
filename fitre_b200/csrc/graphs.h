// CUDA-graph replay of fixed launch sequences (shared by the KFAC calls and the network passes).
#pragma once

#include <cstring>
#include <vector>

#include "common.h"

namespace fitre {

inline long long ptr_key(const void *p) { return (long long)(uintptr_t)p; }
inline long long bits_key(double v) {
    long long b;
    std::memcpy(&b, &v, sizeof b);
    return b;
}
// Runs enqueue() -- which issues work on ctx->stream and on the side streams forked from it --
// through a CUDA graph: captured on first use (from a stream of the library's own, because the
// caller's may be the legacy default stream, which cannot be captured), replayed on ctx->stream
// while `key` is unchanged.  If capture or instantiation is refused the sequence is launched
// directly and `*enabled` (default: the context's graph switch) is cleared.
template <class F>
void run_graphed(fitre_context *ctx, fitre_context::CapturedGraph &g, const std::vector<long long> &key,
                 F &&enqueue, int *enabled = nullptr) {
    if (!enabled) enabled = &ctx->use_graphs;
    if (!ctx->use_graphs || !*enabled) {
        enqueue();
        return;
    }
    if (g.exec && g.key == key) {
        FITRE_CUDA(cudaGraphLaunch(g.exec, ctx->stream));
        ctx->launches += g.launches;
        return;
    }
    if (g.exec) {
        cudaGraphExecDestroy(g.exec);
        g.exec = nullptr;
    }
    if (!ctx->graph_stream) FITRE_CUDA(cudaStreamCreateWithFlags(&ctx->graph_stream, cudaStreamNonBlocking));
    const long long l0 = ctx->launches;
    cudaStream_t user = ctx->stream;
    cudaGraph_t graph = nullptr;
    cudaError_t e = cudaStreamBeginCapture(ctx->graph_stream, cudaStreamCaptureModeRelaxed);
    if (e == cudaSuccess) {
        ctx->stream = ctx->graph_stream;
        try {
            enqueue();
        } catch (...) {
            ctx->stream = user;
            cudaStreamEndCapture(ctx->graph_stream, &graph);
            if (graph) cudaGraphDestroy(graph);
            cudaGetLastError();
            throw;
        }
        ctx->stream = user;
        e = cudaStreamEndCapture(ctx->graph_stream, &graph);
        if (e == cudaSuccess) e = cudaGraphInstantiate(&g.exec, graph, 0);
        if (graph) cudaGraphDestroy(graph);
    }
    if (e != cudaSuccess) {
        cudaGetLastError();
        g.exec = nullptr;
        *enabled = 0;
        ctx->launches = l0;
        enqueue();
        return;
    }
    g.key = key;
    g.launches = ctx->launches - l0;
    FITRE_CUDA(cudaGraphLaunch(g.exec, ctx->stream));
}

}  // namespace fitre
