// Internal declarations shared by the library's translation units.
#pragma once

#include <cuda_runtime.h>

#include <cstdint>
#include <cstdio>
#include <stdexcept>
#include <cstring>
#include <string>
#include <utility>
#include <vector>

#include "../../include/fitre_b200.h"

namespace fitre {

constexpr double kBnEps = 1e-5;  // functions/dev_batch_norm.h:10

// Error carrying a C-ABI status code; caught at the extern "C" boundary.
struct Error : std::runtime_error {
    int code;
    Error(int c, const std::string &what) : std::runtime_error(what), code(c) {}
};

#define FITRE_CUDA(call)                                                                   \
    do {                                                                                   \
        cudaError_t e_ = (call);                                                           \
        if (e_ != cudaSuccess)                                                             \
            throw ::fitre::Error(FITRE_ERR_CUDA, std::string(#call) + ": " +               \
                                                     cudaGetErrorString(e_));              \
    } while (0)

#define FITRE_REQUIRE(cond, code, msg)                         \
    do {                                                       \
        if (!(cond)) throw ::fitre::Error((code), (msg));      \
    } while (0)

struct Comm;  // NCCL state (comm.cpp)

// Mailbox all-reduce over peer memory (set up in comm.cpp, used by peer.cu)
#define FITRE_PEER_MAX_RANKS 8
#define FITRE_PEER_MAX_DOUBLES 3584   // 7 sums x 512 channels
struct PeerBox {
    bool enabled = false;
    double *inbox[FITRE_PEER_MAX_RANKS] = {};  // inbox[r]: rank r's mailbox mapped here (own rank: local)
    unsigned long long epoch = 0;
    long long wait_ns = 30000000000ll;          // bound of the device-side wait for the peers' flags
};

}  // namespace fitre

// One context per GPU and host thread.  Owns only small fixed buffers (pinned scalars and a
// device scalar slab); every tensor-sized buffer belongs to the caller.
struct fitre_context {
    int device = 0;
    cudaStream_t stream = nullptr;
    long long launches = 0;
    std::string err;
    int ref_softmax = 1;
    long scratch_limit = 0;     // doubles behind the caller's scratch pointer (0 = unknown, unchecked)
    int ref_quadratic = 1;      // quadratic model damps with lambda * weights (reference) or lambda * vector
    int precision = 0;          // FITRE_PRECISION_* (convolution products)
    int kfac_solver = 0;        // FITRE_KFAC_SOLVER_* (what the A-factor slots hold)
    int kfac_owned = 0;         // FITRE_KFAC_LAYER_OWNED: with ranks, each layer's factors live on one rank
    bool use_tma = true;        // TMA-fed convolution kernels where shape and alignment allow
    double *pinned = nullptr;   // 256 pinned host doubles (scalar read-back)
    double *dscal = nullptr;    // 4096 device doubles (scalar reductions)
    fitre::Comm *comm = nullptr;
    fitre::PeerBox peer;
    int rank = 0, world = 1;
    double comm_timeout_s = 300.0;  // bound of communicator set-up and of every host wait on a collective
    // workspace of the host-buffer entry point (allocated on first use, reused)
    double *host_ws = nullptr;
    size_t host_ws_doubles = 0;
    double *host_pinned = nullptr;
    size_t host_pinned_doubles = 0;
    cudaStream_t copy_stream = nullptr;   // second stream of the host-buffer entry point
    cudaEvent_t ev_up = nullptr, ev_down = nullptr;
    // hooks of the host-buffer entry point: the forward pass waits for `fwd_wait_event` before conv
    // layer `fwd_wait_layer` (late weights still uploading), and the R-backward pass sends finished
    // slices of hv to `hv_host_dst` on the copy stream as the layers complete
    cudaEvent_t fwd_wait_event = nullptr, ev_w2 = nullptr, chunk_ev[24] = {};
    int fwd_wait_layer = -1;
    double *hv_host_dst = nullptr;
    int host_shared = 0;                  // result buffers of the host entry point are shared by all ranks
    int host_replicated = 0;              // ... and its weights / vector inputs hold the same values on all ranks
    long hv_sent_from = 0;
    // set around a backward sweep whose result vector is a batch sum wanted on every rank: the
    // sweep then all-reduces each layer's finished slice while it computes the next layer
    bool reduce_slices = false;
    long reduced_from = 0;
    double *staging_buf = nullptr;        // staging of the opt-in tensor-core modes (operand copies, digit
    long staging_cap = 0;                 // planes, split slabs), owned by the context, grown on demand
    cudaStream_t inv_streams[8] = {};     // side streams of the batched factor inversion
    cudaEvent_t inv_fork = nullptr, inv_join[8] = {};
    // The launch sequences of the factor inverses and of the natural gradient are fixed by the
    // model and the buffers; each is captured once into a CUDA graph and replayed while its key
    // (pointers, sizes, damping, solver) stays the same.
    struct CapturedGraph {
        std::vector<long long> key;
        cudaGraphExec_t exec = nullptr;
        long long launches = 0;
    };
    CapturedGraph graph_invert, graph_natgrad, graph_factors, graph_factors_a, graph_factors_g;
    // Launch sequences of the network passes (one Hessian-vector product, one gradient): a few
    // recently used (model, buffer set) pairs each, so that a solver that alternates between two
    // direction vectors replays both.  Only where launch latency is what the call costs: one
    // rank, fp64 kernels, no host-buffer streaming, no event timing.
    CapturedGraph graph_hv[4], graph_grad[2];
    int graph_hv_next = 0, graph_grad_next = 0;
    int use_pass_graphs = 1;
    // two-call form of the factor step: the A side runs on a stream of its own between the calls
    cudaStream_t phase_stream = nullptr;
    cudaEvent_t phase_fork = nullptr, phase_done = nullptr;
    bool phase_open = false;
    std::vector<cudaEvent_t> layer_ev;    // "factor of layer l is ready" (fused factors + inverses)
    cudaStream_t graph_stream = nullptr;  // origin stream of the captures
    int use_graphs = 1;
    // optional per-kernel timing (CUDA events on the launch stream), see fitre_profile_*
    bool prof_on = false;
    struct ProfRec { cudaEvent_t beg, end; int kind; double flops; };
    std::vector<ProfRec> prof;
    std::vector<std::pair<cudaEvent_t, cudaEvent_t>> prof_pool;
    // launches per kernel name (the literal handed to check_launch; a name may appear under
    // several pointers, one per translation unit), read by fitre_kernel_launches
    std::vector<std::pair<const char *, long long>> launch_names;
};

namespace fitre {

inline void count_launch(fitre_context *ctx, int n = 1) { ctx->launches += n; }

// After a kernel launch: pick up launch-configuration errors.
inline void check_launch(fitre_context *ctx, const char *name) {
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess)
        throw Error(FITRE_ERR_CUDA, std::string("launch of ") + name + ": " + cudaGetErrorString(e));
    ctx->launches += 1;
    for (auto &r : ctx->launch_names)
        if (r.first == name) {
            r.second += 1;
            return;
        }
    ctx->launch_names.emplace_back(name, 1);
}

// A call that needs `need` doubles of caller scratch: refused when the caller declared fewer.
inline void require_scratch(const fitre_context *ctx, long need, const char *what) {
    if (ctx->scratch_limit > 0 && need > ctx->scratch_limit)
        throw Error(FITRE_ERR_WORKSPACE, std::string(what) + " needs " + std::to_string(need) +
                                             " doubles of scratch, the caller declared " +
                                             std::to_string(ctx->scratch_limit));
}

// Kernel classes the optional event timing distinguishes.
enum { PROF_CONV_IGEMM = 0, PROF_CONV_WGRAD = 1, PROF_KINDS = 2 };
// Brackets one launch with events when profiling is on (no-op otherwise).
struct ProfScope {
    fitre_context *ctx;
    int idx = -1;
    ProfScope(fitre_context *c, int kind, double flops);
    ~ProfScope();
};

// ---- comm.cpp: all-reduce hooks (no-ops when world == 1) ----
void comm_allreduce_sum(fitre_context *ctx, double *dev_buf, size_t n);
// In place: every rank contributes dev_buf[rank * chunk, +chunk) and receives all world chunks.
// False (nothing done) when the NCCL library at hand has no ncclAllGather.
bool comm_allgather_inplace(fitre_context *ctx, double *dev_buf, size_t chunk, cudaStream_t stream);
bool comm_has_allgather();
void comm_reduce_sum(fitre_context *ctx, double *dev_buf, size_t n, int root);
void comm_destroy(fitre_context *ctx);
// all-reduce of a finished slice on the side communicator / stream; join = the context's stream
// waits for all of them (no-ops on one rank)
void comm_allreduce_async(fitre_context *ctx, double *dev_buf, size_t n);
void comm_async_join(fitre_context *ctx);
cudaStream_t comm_async_stream(fitre_context *ctx);
// short vectors (batch statistics, scalars): one kernel over peer memory when the mailboxes are
// up, NCCL otherwise
void comm_allreduce_small(fitre_context *ctx, double *dev_buf, size_t n);
// peer.cu
bool peer_allreduce_ready(const fitre_context *ctx, long n);
void peer_allreduce(fitre_context *ctx, const double *partials, int S, int NS, double *io, int n);
int peer_wait_selftest(fitre_context *ctx, double wait_ms);
// host wait on a stream; with a communicator it also watches NCCL's error state and a deadline
void stream_wait(fitre_context *ctx, cudaStream_t stream);

// ---- model.cpp ----
struct ConvGeom {
    int Cin, Cout, H, W, Ho, Wo, k, pad;
    int bn, act;
    int poolType, pk, ps, pp, Hp, Wp;
    long zoff;                      // start of this layer's block in z / dx / rz
    long actOff, poolOff, bnOff, outOff;  // relative to zoff
    long meanOff, varOff;           // relative to zoff + bnOff
};
ConvGeom conv_geom(const CNN_MODEL *m, int l);
void model_check_batch(const CNN_MODEL *m, int curBatchSize);
long max_delta_elems(const CNN_MODEL *m);  // largest errors tensor incl. conv inputs

// ---- gemm.cu ----
struct ConvSeg {            // one (input tensor, weight matrix) pair of a K-/M-concatenated product
    const double *x;        // [Cin][N][W][H]
    const double *w;        // K x Cout column-major
};
// Y[M x Cout] (+= bias[c]) = sum_seg im2col(x_seg) * w_seg      (fprop and its R-op form)
// `split` = conv_fprop_scratch() doubles of scratch for split-K slabs (may be NULL).
long conv_fprop_scratch(int N, int Cin, int H, int W, int k, int pad, int Cout);
void conv_fprop(fitre_context *ctx, int nseg, const ConvSeg *segs, const double *bias, double *y,
                int N, int Cin, int H, int W, int k, int pad, int Cout, double *split);
// dX[(N H W) x Cin] = sum_seg im2colT(delta_seg) * perm(w_seg)  (dgrad and its R-op form);
// `wscratch` receives the permuted weights (nseg * K * Cout doubles).
long conv_dgrad_scratch(int N, int Cin, int H, int W, int k, int pad, int Cout);
void conv_dgrad(fitre_context *ctx, int nseg, const ConvSeg *segs, double *dx, int N, int Cin,
                int H, int W, int k, int pad, int Cout, double *wscratch, double *split);
// dW[K x Cout] = sum_seg im2col(x_seg)' * delta_seg ; segs[i].w is delta_seg (M x Cout).
// `partials` needs conv_wgrad_scratch() doubles.
long conv_wgrad_scratch(int N, int Cin, int H, int W, int k, int pad, int Cout);
void conv_wgrad(fitre_context *ctx, int nseg, const ConvSeg *segs, double *dw, int N, int Cin,
                int H, int W, int k, int pad, int Cout, double *partials);
// C (m x n, ldc) = alpha op(A) op(B) + beta C, column-major (cublasDgemm semantics)
void dgemm(fitre_context *ctx, bool tA, bool tB, int m, int n, int k, double alpha,
           const double *A, int lda, const double *B, int ldb, double beta, double *C, int ldc);
// the same with a structure hint (see gemm.cu): terms known to be zero are skipped
enum { GEMM_FULL = 0, GEMM_K_LE_COL = 1, GEMM_K_GE_COL = 2, GEMM_K_LE_ROW = 3, GEMM_LOWER_C = 4 };
void dgemm_structured(fitre_context *ctx, bool tA, bool tB, int m, int n, int k, double alpha,
                      const double *A, int lda, const double *B, int ldb, double beta, double *C, int ldc,
                      int kmode);
// C (n x n) = alpha * A' A  where A is rows x n column-major (lda); both triangles written.
long syrk_scratch(long rows, int n);
void syrk_tn(fitre_context *ctx, long rows, int n, double alpha, const double *A, long lda,
             double *C, double *partials);

long conv_patch_syrk_scratch(int N, int Cin, int H, int W, int k, int pad, bool bias);
long conv_patch_syrk_tma_scratch(int N, int Cin, int H, int W, int k, int pad);
int conv_patch_syrk_tma(fitre_context *ctx, const double *x, double *slabs, int N, int Cin, int H, int W,
                        int k, int pad);
// A = alpha * S (P~' P~) S over implicit im2col patches P~ = [im2col(x), 1], S = diag(patch_scale.., 1)
void conv_patch_syrk(fitre_context *ctx, const double *x, double *A, int N, int Cin, int H, int W,
                     int k, int pad, bool bias, double alpha, double patch_scale, double *partials);
void gemm_init_attributes();
void kfac_init_attributes();
// conv_tma.cu
void conv_tma_init_attributes();
long conv_fprop_tma_scratch(int N, int Cin, int H, int W, int k, int pad, int Cout);
bool conv_fprop_tma(fitre_context *ctx, int nseg, const ConvSeg *segs, const double *bias,
                    double *y, int N, int Cin, int H, int W, int k, int pad, int Cout,
                    double *split_scratch);
long conv_wgrad_tma_scratch(int N, int Cin, int H, int W, int k, int pad, int Cout);
bool conv_wgrad_tma(fitre_context *ctx, int nseg, const ConvSeg *segs, double *dw, int N, int Cin,
                    int H, int W, int k, int pad, int Cout, double *partials);
// conv_tf32.cu
void conv_tf32_init_attributes();
long conv_fprop_tf32_scratch(int N, int Cin, int H, int W, int k, int pad, int Cout);
// conv_i8.cu
void conv_i8_init_attributes();
bool conv_fprop_i8(fitre_context *ctx, int nseg, const ConvSeg *segs, const double *bias, double *y, int N,
                   int Cin, int H, int W, int k, int pad, int Cout);
bool conv_wgrad_i8(fitre_context *ctx, int nseg, const ConvSeg *segs, double *dw, int N, int Cin, int H, int W,
                   int k, int pad, int Cout);
long conv_wgrad_tf32_scratch(int N, int Cin, int H, int W, int k, int pad, int Cout);
bool conv_wgrad_tf32(fitre_context *ctx, int nseg, const ConvSeg *segs, double *dw, int N, int Cin, int H,
                     int W, int k, int pad, int Cout, double *scratch);
bool conv_fprop_tf32(fitre_context *ctx, int nseg, const ConvSeg *segs, const double *bias, double *y,
                     int N, int Cin, int H, int W, int k, int pad, int Cout, double *scratch);
// Device-side error word (set by a kernel whose bounded wait ran out): dscal[4000] as int.
void check_device_error(fitre_context *ctx);

// ---- layers.cu ----
long bn_scratch(int C);   // doubles of scratch any batch-norm / reduction helper may use
void add_channel_bias(fitre_context *ctx, double *x, const double *bias, long rows, int C);
void add_column_bias(fitre_context *ctx, double *x, const double *bias, int rows, int cols);
void apply_activation(fitre_context *ctx, int act, const double *in, double *out, long n);
// conv-out -> (bn out, mean, var) -> act out [-> pool out]
void conv_post_forward(fitre_context *ctx, const ConvGeom &g, int N, double *zl, double *scratch,
                       bool running_stats = false);
// R-op of the same chain: rz conv-out -> R bn -> R act -> R pool
void conv_post_rop_forward(fitre_context *ctx, const ConvGeom &g, int N, const double *zl,
                           double *rzl, double *scratch);
// pooled errors -> dx_P, dx_A, dx_BN (written into dxl); returns pointer to the errors the
// convolution consumes (dx_BN or dx_A).  db (may be NULL) receives the bias gradient.
// `pool_map` (pool_map_doubles(g, N) doubles of scratch, may be NULL): room for the arg-max map of
// the layer's pooling windows, which the backward gather of a general max pool then reads
long pool_map_doubles(const ConvGeom &g, int N);
// The part [lo, hi) of a finished range [a, b) of a result vector that this rank sends to the
// host: all of it, or its 1/world share when every rank's host buffer is the same memory.
inline void host_share(const fitre_context *ctx, long a, long b, long &lo, long &hi) {
    lo = a;
    hi = b;
    if (!ctx->host_shared || ctx->world <= 1) return;
    const long len = b - a;
    lo = a + len * ctx->rank / ctx->world;
    hi = a + len * (ctx->rank + 1) / ctx->world;
}
const double *conv_post_backward(fitre_context *ctx, const ConvGeom &g, int N, const double *zl,
                                 double *dxl, const double *delta_pool, double *db,
                                 double *scratch, unsigned char *pool_map = nullptr);
// R-op of the backward chain: Rdelta_pool -> Rdelta for the convolution (written to `rout`).
void conv_post_rop_backward(fitre_context *ctx, const ConvGeom &g, int N, const double *zl,
                            const double *rzl, const double *dxl, const double *rdelta_pool,
                            double *rout, double *rdb, double *scratch, unsigned char *pool_map = nullptr);
void conv_to_fc(fitre_context *ctx, double *buf, int C, int N, int Hp, int Wp, double *tmp);
void fc_to_conv(fitre_context *ctx, double *buf, int C, int N, int Hp, int Wp, double *tmp);
void act_backward(fitre_context *ctx, int act, double *delta, const double *zin,
                  const double *zout, long n);
void act_rop_backward(fitre_context *ctx, int act, double *rdelta, const double *delta_in,
                      const double *rzin, const double *zin, const double *zout, long n);
void row_sums(fitre_context *ctx, const double *x, int rows, int cols, double *out);
// softmax cross-entropy: probs, errors (p - y)/Nglobal; the batch loss sum lands in dscal[0]
void softmax_loss(fitre_context *ctx, const double *logits, const double *labels, int N,
                  int classes, double *probs, double *errors, double inv_n_global);
void softmax_rop_error(fitre_context *ctx, const double *rz, const double *probs, int N,
                       int classes, double *rerr, double inv_n_global);
void distribution_errors(fitre_context *ctx, const double *probs, const double *uniforms, int N,
                         int classes, double *target, double *errors, double inv_n_global);
// vector helpers on pSize-long vectors
void vec_axpy(fitre_context *ctx, long n, double a, const double *x, double *y);
void vec_scale(fitre_context *ctx, long n, double a, double *x);
void vec_copy(fitre_context *ctx, long n, const double *x, double *y);
void vec_axpby(fitre_context *ctx, long n, double a, const double *x, double b, double *y);
void vec_fill(fitre_context *ctx, long n, double v, double *x);
// up to 3 dot products in one pass; results in ctx->pinned[0..2] after a stream sync
void vec_dots(fitre_context *ctx, long n, const double *a0, const double *b0, const double *a1,
              const double *b1, const double *a2, const double *b2, double *host_out);

// ---- passes.cu ----
double cnn_forward(fitre_context *ctx, const CNN_MODEL *m, const DEVICE_DATASET *data,
                   double *scratch, double *z, double *probs, double *errors, int n,
                   bool want_loss, bool running_stats = false);
void cnn_backward(fitre_context *ctx, const CNN_MODEL *m, const DEVICE_DATASET *data,
                  double *scratch, double *z, double *gradient, double *dx, double *delta,
                  double *delta_new, int n);
void cnn_rop_forward(fitre_context *ctx, const CNN_MODEL *m, const DEVICE_DATASET *data,
                     const double *z, const double *vector, double *rz, int n, double *scratch);
void cnn_rop_backward(fitre_context *ctx, const CNN_MODEL *m, const DEVICE_DATASET *data,
                      const double *z, const double *dx, const double *lossErrors, double *rError,
                      const double *rz, const double *vector, double *hv, int n, double *scratch);
void cnn_hv(fitre_context *ctx, const CNN_MODEL *m, const DEVICE_DATASET *data, const double *z,
            const double *probs, const double *lossErrors, const double *dx, const double *vector,
            double *hv, int n, double *devPtr);
// forward + backward + slice all-reduces + weight decay of computeCNNGradient (the loss sum stays in
// ctx->dscal[0]); errors / errors1: the two error buffers, ws: scratch of the passes
void cnn_gradient(fitre_context *ctx, const CNN_MODEL *m, const DEVICE_DATASET *data, double *ws, double *z,
                  double *dx, double *probs, double *lossErrors, double *gradient, double *errors,
                  double *errors1, int n, double weightDecay);
long forward_scratch(const CNN_MODEL *m);
long backward_scratch(const CNN_MODEL *m);
long rop_forward_scratch(const CNN_MODEL *m);
long rop_backward_scratch(const CNN_MODEL *m);

}  // namespace fitre
