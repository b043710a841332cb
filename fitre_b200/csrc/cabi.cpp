// extern "C" surface: context management, the reference-named entry points, the solvers that
// sit directly on the Hessian-vector product, and the host-buffer entry point.
#include <cmath>
#include <cstring>

#include "common.h"

namespace fitre {
void comm_unique_id(void *out128);
void comm_init(fitre_context *ctx, const void *id128, int rank, int world);
void gemm_init_attributes();
}  // namespace fitre

using namespace fitre;

namespace fitre {
ProfScope::ProfScope(fitre_context *c, int kind, double flops) : ctx(c) {
    if (!c->prof_on) return;
    std::pair<cudaEvent_t, cudaEvent_t> ev;
    if (!c->prof_pool.empty()) {
        ev = c->prof_pool.back();
        c->prof_pool.pop_back();
    } else {
        FITRE_CUDA(cudaEventCreate(&ev.first));
        FITRE_CUDA(cudaEventCreate(&ev.second));
    }
    c->prof.push_back({ev.first, ev.second, kind, flops});
    idx = (int)c->prof.size() - 1;
    cudaEventRecord(ev.first, c->stream);
}
ProfScope::~ProfScope() {
    if (idx >= 0) cudaEventRecord(ctx->prof[idx].end, ctx->stream);
}
}  // namespace fitre

namespace fitre {
// Reads the device error word together with a scalar read-back; call after a stream sync
// point has been queued.  A non-zero word means a bounded wait inside a kernel gave up.
void check_device_error(fitre_context *ctx) {
    FITRE_CUDA(cudaMemcpyAsync(ctx->pinned + 200, ctx->dscal + 4000, sizeof(double),
                               cudaMemcpyDeviceToHost, ctx->stream));
    stream_wait(ctx, ctx->stream);
    int word;
    std::memcpy(&word, ctx->pinned + 200, sizeof(int));
    if (word != 0) {
        FITRE_CUDA(cudaMemsetAsync(ctx->dscal + 4000, 0, sizeof(double), ctx->stream));
        if (word == 2)
            throw Error(FITRE_ERR_COMM, "the peer all-reduce kernel's bounded wait for another rank's flag ran out");
        throw Error(FITRE_ERR_CUDA, "a kernel's bounded wait on a TMA transfer ran out");
    }
}
}  // namespace fitre

namespace {

long align32(long n) { return (n + 31) / 32 * 32; }

template <class F>
int guarded(fitre_context *ctx, F &&f) {
    try {
        if (!ctx) return FITRE_ERR_BAD_ARG;
        FITRE_CUDA(cudaSetDevice(ctx->device));
        f();
        return FITRE_OK;
    } catch (const Error &e) {
        if (ctx) ctx->err = e.what();
        return e.code;
    } catch (const std::exception &e) {
        if (ctx) ctx->err = e.what();
        return FITRE_ERR_CUDA;
    }
}

void require_ptrs(std::initializer_list<const void *> ps) {
    for (const void *p : ps) FITRE_REQUIRE(p != nullptr, FITRE_ERR_BAD_ARG, "NULL pointer argument");
}

}  // namespace

extern "C" {

int fitre_context_create(fitre_context **out, int device, void *stream) {
    if (!out) return FITRE_ERR_BAD_ARG;
    *out = nullptr;
    int count = 0;
    if (cudaGetDeviceCount(&count) != cudaSuccess || device < 0 || device >= count) {
        cudaGetLastError();
        return FITRE_ERR_CUDA;  // no CPU fallback: without a CUDA device there is no context
    }
    fitre_context *ctx = new fitre_context();
    ctx->device = device;
    ctx->stream = (cudaStream_t)stream;
    int rc = guarded(ctx, [&] {
        FITRE_CUDA(cudaMallocHost((void **)&ctx->pinned, 256 * sizeof(double)));
        FITRE_CUDA(cudaMalloc((void **)&ctx->dscal, 4096 * sizeof(double)));
        FITRE_CUDA(cudaMemsetAsync(ctx->dscal, 0, 4096 * sizeof(double), ctx->stream));
        gemm_init_attributes();
    });
    if (rc != FITRE_OK) {
        fitre_context_destroy(ctx);
        return rc;
    }
    *out = ctx;
    return FITRE_OK;
}

int fitre_context_destroy(fitre_context *ctx) {
    if (!ctx) return FITRE_OK;
    cudaSetDevice(ctx->device);
    try {
        stream_wait(ctx, ctx->stream);  // bounded when a communicator exists
    } catch (...) {
    }
    try {
        comm_destroy(ctx);
    } catch (...) {
    }
    if (ctx->pinned) cudaFreeHost(ctx->pinned);
    if (ctx->dscal) cudaFree(ctx->dscal);
    if (ctx->host_ws) cudaFree(ctx->host_ws);
    if (ctx->host_pinned) cudaFreeHost(ctx->host_pinned);
    if (ctx->staging_buf) cudaFree(ctx->staging_buf);
    if (ctx->copy_stream) cudaStreamDestroy(ctx->copy_stream);
    for (int s = 0; s < 8; ++s) {
        if (ctx->inv_streams[s]) cudaStreamDestroy(ctx->inv_streams[s]);
        if (ctx->inv_join[s]) cudaEventDestroy(ctx->inv_join[s]);
    }
    if (ctx->inv_fork) cudaEventDestroy(ctx->inv_fork);
    if (ctx->graph_invert.exec) cudaGraphExecDestroy(ctx->graph_invert.exec);
    if (ctx->graph_natgrad.exec) cudaGraphExecDestroy(ctx->graph_natgrad.exec);
    if (ctx->graph_factors.exec) cudaGraphExecDestroy(ctx->graph_factors.exec);
    if (ctx->graph_factors_a.exec) cudaGraphExecDestroy(ctx->graph_factors_a.exec);
    if (ctx->graph_factors_g.exec) cudaGraphExecDestroy(ctx->graph_factors_g.exec);
    for (auto &g : ctx->graph_hv)
        if (g.exec) cudaGraphExecDestroy(g.exec);
    for (auto &g : ctx->graph_grad)
        if (g.exec) cudaGraphExecDestroy(g.exec);
    if (ctx->phase_stream) cudaStreamDestroy(ctx->phase_stream);
    if (ctx->phase_fork) cudaEventDestroy(ctx->phase_fork);
    if (ctx->phase_done) cudaEventDestroy(ctx->phase_done);
    for (cudaEvent_t e : ctx->layer_ev) cudaEventDestroy(e);
    if (ctx->graph_stream) cudaStreamDestroy(ctx->graph_stream);
    if (ctx->ev_up) cudaEventDestroy(ctx->ev_up);
    if (ctx->ev_w2) cudaEventDestroy(ctx->ev_w2);
    for (int i = 0; i < 24; ++i)
        if (ctx->chunk_ev[i]) cudaEventDestroy(ctx->chunk_ev[i]);
    if (ctx->ev_down) cudaEventDestroy(ctx->ev_down);
    for (auto &r : ctx->prof) {
        cudaEventDestroy(r.beg);
        cudaEventDestroy(r.end);
    }
    for (auto &e : ctx->prof_pool) {
        cudaEventDestroy(e.first);
        cudaEventDestroy(e.second);
    }
    delete ctx;
    return FITRE_OK;
}

const char *fitre_last_error(const fitre_context *ctx) { return ctx ? ctx->err.c_str() : "no context"; }
long long fitre_launch_count(const fitre_context *ctx) { return ctx ? ctx->launches : 0; }
int fitre_set_reference_softmax(fitre_context *ctx, int on) {
    if (!ctx) return FITRE_ERR_BAD_ARG;
    ctx->ref_softmax = on ? 1 : 0;
    return FITRE_OK;
}

int fitre_set_scratch_limit(fitre_context *ctx, long doubles) {
    if (!ctx || doubles < 0) return FITRE_ERR_BAD_ARG;
    ctx->scratch_limit = doubles;
    return FITRE_OK;
}

int fitre_set_reference_quadratic_damping(fitre_context *ctx, int on) {
    if (!ctx) return FITRE_ERR_BAD_ARG;
    ctx->ref_quadratic = on ? 1 : 0;
    return FITRE_OK;
}

long long fitre_kernel_launches(const fitre_context *ctx, const char *name) {
    if (!ctx || !name) return -1;
    long long n = 0;
    for (const auto &r : ctx->launch_names)
        if (std::strcmp(r.first, name) == 0) n += r.second;
    return n;
}

int fitre_set_precision(fitre_context *ctx, int precision) {
    if (!ctx || (precision != FITRE_PRECISION_FP64 && precision != FITRE_PRECISION_TF32 &&
                 precision != FITRE_PRECISION_TF32X3 && precision != FITRE_PRECISION_FP64_I8))
        return FITRE_ERR_BAD_ARG;
    ctx->precision = precision;
    return FITRE_OK;
}

int fitre_set_kfac_solver(fitre_context *ctx, int solver) {
    if (!ctx || (solver != FITRE_KFAC_SOLVER_INVERSE && solver != FITRE_KFAC_SOLVER_CHOLESKY))
        return FITRE_ERR_BAD_ARG;
    ctx->kfac_solver = solver;
    return FITRE_OK;
}

int fitre_set_kfac_distribution(fitre_context *ctx, int mode) {
    if (!ctx || (mode != FITRE_KFAC_REPLICATED && mode != FITRE_KFAC_LAYER_OWNED)) return FITRE_ERR_BAD_ARG;
    ctx->kfac_owned = mode;
    return FITRE_OK;
}

int fitre_get_kfac_solver(const fitre_context *ctx) { return ctx ? ctx->kfac_solver : -1; }

int fitre_set_host_results_shared(fitre_context *ctx, int on) {
    if (!ctx) return FITRE_ERR_BAD_ARG;
    ctx->host_shared = on ? 1 : 0;
    return FITRE_OK;
}

int fitre_set_host_inputs_replicated(fitre_context *ctx, int on) {
    if (!ctx) return FITRE_ERR_BAD_ARG;
    ctx->host_replicated = on ? 1 : 0;
    return FITRE_OK;
}

int fitre_set_graphs(fitre_context *ctx, int on) {
    if (!ctx) return FITRE_ERR_BAD_ARG;
    ctx->use_graphs = on ? 1 : 0;
    return FITRE_OK;
}

int fitre_set_tma(fitre_context *ctx, int on) {
    if (!ctx) return FITRE_ERR_BAD_ARG;
    ctx->use_tma = on != 0;
    return FITRE_OK;
}

int fitre_profile_enable(fitre_context *ctx, int on) {
    if (!ctx) return FITRE_ERR_BAD_ARG;
    ctx->prof_on = on != 0;
    return FITRE_OK;
}

int fitre_profile_read(fitre_context *ctx, int kind, double *ms, double *flops, long *launches) {
    return guarded(ctx, [&] {
        FITRE_REQUIRE(kind >= 0 && kind < PROF_KINDS, FITRE_ERR_BAD_ARG, "bad kernel class");
        stream_wait(ctx, ctx->stream);
        double t = 0.0, f = 0.0;
        long n = 0;
        std::vector<fitre_context::ProfRec> keep;
        for (auto &r : ctx->prof) {
            if (r.kind != kind) {
                keep.push_back(r);
                continue;
            }
            float e = 0.f;
            FITRE_CUDA(cudaEventElapsedTime(&e, r.beg, r.end));
            t += e;
            f += r.flops;
            ++n;
            ctx->prof_pool.push_back({r.beg, r.end});
        }
        ctx->prof.swap(keep);
        if (ms) *ms = t;
        if (flops) *flops = f;
        if (launches) *launches = n;
    });
}

int fitre_comm_unique_id(void *id) {
    try {
        if (!id) return FITRE_ERR_BAD_ARG;
        comm_unique_id(id);
        return FITRE_OK;
    } catch (const Error &e) {
        return e.code;
    }
}
int fitre_comm_init(fitre_context *ctx, const void *id, int rank, int world) {
    return guarded(ctx, [&] {
        require_ptrs({id});
        comm_init(ctx, id, rank, world);
    });
}
int fitre_comm_world(const fitre_context *ctx) { return ctx ? ctx->world : 0; }
int fitre_peer_wait_selftest(fitre_context *ctx, double wait_ms) {
    return guarded(ctx, [&] {
        FITRE_REQUIRE(wait_ms > 0.0 && wait_ms <= 5000.0, FITRE_ERR_BAD_ARG, "wait_ms must be in (0, 5000]");
        const int word = peer_wait_selftest(ctx, wait_ms);
        FITRE_REQUIRE(word == 0, FITRE_ERR_COMM, "the bounded wait for a peer's flag ran out (error word " +
                                                     std::to_string(word) + ")");
    });
}
int fitre_peer_reduce_enabled(const fitre_context *ctx) { return ctx ? (ctx->peer.enabled ? 1 : 0) : 0; }
int fitre_set_comm_timeout(fitre_context *ctx, double seconds) {
    if (!ctx || !(seconds > 0.0)) return FITRE_ERR_BAD_ARG;
    ctx->comm_timeout_s = seconds;
    return FITRE_OK;
}

long fitre_cnn_forward_mem_required(const CNN_MODEL *m) { return m ? forward_scratch(m) : -1; }
long fitre_cnn_backward_mem_required(const CNN_MODEL *m) { return m ? backward_scratch(m) : -1; }
long fitre_cnn_rop_forward_mem_required(const CNN_MODEL *m) { return m ? rop_forward_scratch(m) : -1; }
long fitre_cnn_rop_backward_mem_required(const CNN_MODEL *m) { return m ? rop_backward_scratch(m) : -1; }
long fitre_cnn_gradient_mem_required(const CNN_MODEL *m) {
    if (!m) return -1;
    return 2 * align32(max_delta_elems(m)) + std::max(forward_scratch(m), backward_scratch(m));
}
long fitre_cnn_hv_mem_required(const CNN_MODEL *m) {
    if (!m) return -1;
    return align32(m->zSize) + align32(max_delta_elems(m)) +
           std::max(rop_forward_scratch(m), rop_backward_scratch(m));
}

int fitre_cnn_forward(fitre_context *ctx, const CNN_MODEL *m, const DEVICE_DATASET *data,
                      SCRATCH_AREA *scratch, real *z, real *probs, real *errors, int s,
                      int curBatchSize, int evalType, real *loss_host) {
    (void)s;
    return guarded(ctx, [&] {
        require_ptrs({m, data, scratch, z, probs, errors});
        require_ptrs({data->weights, data->currentBatch, data->sampledTrainY, scratch->nextDevPtr});
        FITRE_REQUIRE(evalType == FITRE_MODEL_TRAIN || evalType == FITRE_MODEL_TRAIN_ACCURACY ||
                          evalType == FITRE_MODEL_TEST_ACCURACY,
                      FITRE_ERR_BAD_ARG, "unknown EVAL_TYPE");
        model_check_batch(m, curBatchSize);
        require_scratch(ctx, forward_scratch(m), "fitre_cnn_forward");
        // the two accuracy modes normalise with the running statistics (functions/dev_batch_norm.cu:386-392)
        double loss = cnn_forward(ctx, m, data, scratch->nextDevPtr, z, probs, errors, curBatchSize, true,
                                  evalType != FITRE_MODEL_TRAIN);
        if (loss_host) *loss_host = loss;
        FITRE_REQUIRE(std::isfinite(loss), FITRE_ERR_NOT_FINITE, "the loss is not finite (NaN or Inf in the batch or the weights)");
    });
}

int fitre_cnn_backward(fitre_context *ctx, const CNN_MODEL *m, const DEVICE_DATASET *data,
                       real *devPtr, real *z, real *gradient, real *dx, real *delta,
                       real *delta_new, int offset, int batchSize, real *hostPtr) {
    (void)offset;
    (void)hostPtr;
    return guarded(ctx, [&] {
        require_ptrs({m, data, devPtr, z, gradient, dx, delta, delta_new});
        model_check_batch(m, batchSize);
        require_scratch(ctx, backward_scratch(m), "fitre_cnn_backward");
        cnn_backward(ctx, m, data, devPtr, z, gradient, dx, delta, delta_new, batchSize);
    });
}

int fitre_compute_cnn_gradient(fitre_context *ctx, const CNN_MODEL *m, const DEVICE_DATASET *data,
                               SCRATCH_AREA *scratch, real *z, real *dx, real *probs,
                               real *lossFuncErrors, real *gradient, int offset, int curBatchSize,
                               real weightDecay, real *loss_host) {
    (void)offset;
    return guarded(ctx, [&] {
        require_ptrs({m, data, scratch, z, dx, probs, lossFuncErrors, gradient});
        require_ptrs({data->weights, data->currentBatch, data->sampledTrainY, scratch->nextDevPtr});
        model_check_batch(m, curBatchSize);
        require_scratch(ctx, fitre_cnn_gradient_mem_required(m), "fitre_compute_cnn_gradient");
        // functions/cnn_gradient.cu:24-31: two error buffers in front of the pass scratch
        const long md = align32(max_delta_elems(m));
        double *errors = scratch->nextDevPtr;
        double *errors1 = errors + md;
        double *ws = errors1 + md;
        cnn_gradient(ctx, m, data, ws, z, dx, probs, lossFuncErrors, gradient, errors, errors1, curBatchSize,
                     weightDecay);
        comm_allreduce_small(ctx, ctx->dscal, 1);
        FITRE_CUDA(cudaMemcpyAsync(ctx->pinned, ctx->dscal, sizeof(double), cudaMemcpyDeviceToHost,
                                   ctx->stream));
        check_device_error(ctx);
        const double loss = ctx->pinned[0] / ((double)curBatchSize * ctx->world);
        if (loss_host) *loss_host = loss;
        FITRE_REQUIRE(std::isfinite(loss), FITRE_ERR_NOT_FINITE, "the loss is not finite (NaN or Inf in the batch or the weights)");
    });
}

int fitre_cnn_rop_forward(fitre_context *ctx, const CNN_MODEL *m, const DEVICE_DATASET *data,
                          SCRATCH_AREA *scratch, real *z, real *vector, real *rz, int s,
                          int curBatchSize, real *devPtr, real *hostPtr) {
    (void)scratch; (void)s; (void)hostPtr;
    return guarded(ctx, [&] {
        require_ptrs({m, data, z, vector, rz, devPtr});
        model_check_batch(m, curBatchSize);
        require_scratch(ctx, rop_forward_scratch(m), "fitre_cnn_rop_forward");
        cnn_rop_forward(ctx, m, data, z, vector, rz, curBatchSize, devPtr);
    });
}

int fitre_cnn_rop_backward(fitre_context *ctx, const CNN_MODEL *m, const DEVICE_DATASET *data,
                           SCRATCH_AREA *scratch, real *z, real *dx, real *lossFuncErrors,
                           real *rError, real *rz, real *vector, real *hv, int s,
                           int curBatchSize, real *devPtr, real *hostPtr) {
    (void)scratch; (void)s; (void)hostPtr;
    return guarded(ctx, [&] {
        require_ptrs({m, data, z, dx, lossFuncErrors, rError, rz, vector, hv, devPtr});
        model_check_batch(m, curBatchSize);
        require_scratch(ctx, rop_backward_scratch(m), "fitre_cnn_rop_backward");
        cnn_rop_backward(ctx, m, data, z, dx, lossFuncErrors, rError, rz, vector, hv, curBatchSize, devPtr);
    });
}

int fitre_cnn_hv(fitre_context *ctx, const CNN_MODEL *m, const DEVICE_DATASET *data, real *z,
                 real *probs, real *lossFuncErrors, real *dx, real *vector, real *hv, int s,
                 int curBatchSize, real *devPtr, real *hostPtr, real weightDecay) {
    (void)s; (void)hostPtr; (void)weightDecay;
    return guarded(ctx, [&] {
        require_ptrs({m, data, z, probs, lossFuncErrors, dx, vector, hv, devPtr});
        model_check_batch(m, curBatchSize);
        require_scratch(ctx, fitre_cnn_hv_mem_required(m), "fitre_cnn_hv");
        cnn_hv(ctx, m, data, z, probs, lossFuncErrors, dx, vector, hv, curBatchSize, devPtr);
        check_device_error(ctx);
    });
}

// functions/model_reduction.cu:20-93.  The damping term added to Hv is weightDecay * weights as
// in the C reference (model_reduction.cu:50-52) or, with fitre_set_reference_quadratic_damping(0),
// weightDecay * vector (what the reference's PyTorch twin adds, pytorch/peng/utils.py:77); both
// vanish at weightDecay == 0.
long fitre_quadratic_model_mem_required(const CNN_MODEL *m) {
    if (!m) return -1;
    return align32(m->pSize) + fitre_cnn_hv_mem_required(m);
}

int fitre_compute_quadratic_model(fitre_context *ctx, const CNN_MODEL *m,
                                  const DEVICE_DATASET *data, real *z, real *probs,
                                  real *lossFuncErrors, real *dx, real *gradient, real *vector,
                                  real delta, int offset, int curBatchSize, real weightDecay,
                                  real *devPtr, real *hostPtr, real *pageLckPtr, real *m_host) {
    (void)offset; (void)hostPtr; (void)pageLckPtr;
    return guarded(ctx, [&] {
        require_ptrs({m, data, z, probs, lossFuncErrors, dx, gradient, vector, devPtr});
        model_check_batch(m, curBatchSize);
        require_scratch(ctx, fitre_quadratic_model_mem_required(m), "fitre_compute_quadratic_model");
        const long P = m->pSize;
        double *hv = devPtr;
        double *next = hv + align32(P);
        cnn_hv(ctx, m, data, z, probs, lossFuncErrors, dx, vector, hv, curBatchSize, next);
        vec_axpy(ctx, P, weightDecay, ctx->ref_quadratic ? data->weights : vector, hv);
        double d[3];
        vec_dots(ctx, P, hv, vector, vector, vector, gradient, vector, d);
        check_device_error(ctx);
        const double vHv = d[0], nrm = std::sqrt(d[1]), gv = d[2];
        double alpha, val;
        if (vHv < 0) {
            alpha = delta / nrm;
            val = 0.5 * vHv * alpha * alpha - gv * alpha;
        } else {
            const double step = gv / (vHv + 1e-6);
            alpha = std::min(step, delta / (nrm + 1e-16));
            val = vHv * 0.5 * alpha * alpha - gv * alpha;
        }
        vec_scale(ctx, P, alpha, vector);
        if (m_host) *m_host = val;
    });
}

// Steihaug-CG (solvers/cg_steihaug.c:28-260; constants of pytorch/peng/utils.py:104-165).
int fitre_cg_steihaug(fitre_context *ctx, const CNN_MODEL *m, const DEVICE_DATASET *data,
                      real *z, real *probs, real *lossFuncErrors, real *dx, real *gradient,
                      real *p, int curBatchSize, real *devPtr, FITRE_CG_PARAMS *prm) {
    return guarded(ctx, [&] {
        require_ptrs({m, data, z, probs, lossFuncErrors, dx, gradient, p, devPtr, prm});
        model_check_batch(m, curBatchSize);
        FITRE_REQUIRE(prm->maxIterations >= 1 && prm->delta > 0, FITRE_ERR_BAD_ARG, "bad CG parameters");
        const long P = m->pSize, Pa = align32(P);
        require_scratch(ctx, 4 * Pa + fitre_cnn_hv_mem_required(m), "fitre_cg_steihaug");
        double *zs = devPtr, *rs = zs + Pa, *ds = rs + Pa, *Hd = ds + Pa, *ws = Hd + Pa;
        const double delta = prm->delta, wd = prm->weightDecay;
        vec_fill(ctx, P, 0.0, zs);
        vec_copy(ctx, P, gradient, rs);
        vec_axpby(ctx, P, -1.0, gradient, 0.0, ds);
        double d[3];
        int flag = FITRE_CG_MAX_ITERS, it = 0, hvc = 0;
        bool done = false;
        auto to_boundary = [&]() {  // p = zs + tau ds with ||p|| = delta
            vec_dots(ctx, P, ds, ds, zs, ds, zs, zs, d);
            const double ac = d[0], bc = 2 * d[1], cc = d[2] - delta * delta;
            const double tau = (-bc + std::sqrt(bc * bc - 4 * ac * cc)) / (2 * ac + 1e-6);
            vec_copy(ctx, P, zs, p);
            vec_axpy(ctx, P, tau, ds, p);
        };
        for (it = 0; it < prm->maxIterations; ++it) {
            cnn_hv(ctx, m, data, z, probs, lossFuncErrors, dx, ds, Hd, curBatchSize, ws);
            ++hvc;
            vec_axpy(ctx, P, wd, ds, Hd);
            vec_dots(ctx, P, Hd, ds, rs, rs, nullptr, nullptr, d);
            const double dHd = d[0], rr = d[1];
            if (dHd <= 0.0) {
                to_boundary();
                flag = FITRE_CG_NEG_CURVATURE;
                done = true;
                break;
            }
            const double alpha = rr / (dHd + 1e-6);
            // ||zs + alpha ds||^2 from three dots (no trial vector needed)
            vec_dots(ctx, P, zs, zs, zs, ds, ds, ds, d);
            const double nn2 = d[0] + 2 * alpha * d[1] + alpha * alpha * d[2];
            if (std::sqrt(std::max(nn2, 0.0)) >= delta) {
                to_boundary();
                flag = FITRE_CG_HIT_BOUNDARY;
                done = true;
                break;
            }
            vec_axpy(ctx, P, alpha, ds, zs);
            vec_axpy(ctx, P, alpha, Hd, rs);
            vec_dots(ctx, P, rs, rs, nullptr, nullptr, nullptr, nullptr, d);
            const double rn = d[0];
            if (rn < prm->tolerance) {
                vec_copy(ctx, P, zs, p);
                flag = FITRE_CG_CONVERGED;
                done = true;
                break;
            }
            const double beta = rn / (rr + 1e-6);
            vec_axpby(ctx, P, -1.0, rs, beta, ds);
        }
        // an exit taken on the very last iteration is reported as "maximum iterations" and
        // returns the last accepted iterate (pytorch/peng/utils.py:156-158)
        if (!done) it = prm->maxIterations - 1;
        if (it == prm->maxIterations - 1) {
            vec_copy(ctx, P, zs, p);
            flag = FITRE_CG_MAX_ITERS;
        }
        cnn_hv(ctx, m, data, z, probs, lossFuncErrors, dx, p, Hd, curBatchSize, ws);
        ++hvc;
        vec_dots(ctx, P, Hd, p, p, gradient, p, p, d);
        check_device_error(ctx);
        prm->modelValue = 0.5 * d[0] + d[1] + 0.5 * wd * d[2];
        prm->iterations = it + 1;
        prm->flag = flag;
        prm->hvCalls = hvc;
    });
}

// ---- host-buffer entry point --------------------------------------------------------------
int fitre_gradient_hv_host(fitre_context *ctx, const CNN_MODEL *m, const real *batch_host,
                           const real *labels_host, const real *weights_host,
                           const real *vector_host, int n, int numClasses, real weightDecay,
                           real *loss_host, real *gradient_host, real *hv_host) {
    return guarded(ctx, [&] {
        require_ptrs({m, batch_host, labels_host, weights_host, vector_host, gradient_host, hv_host});
        model_check_batch(m, n);
        FITRE_REQUIRE(numClasses == m->fcLayer[m->lLayers - 1].out, FITRE_ERR_BAD_ARG,
                      "numClasses differs from the last layer");
        const CONV_LAYER &c0 = m->convLayer[0];
        const long P = align32(m->pSize + 64), Z = align32(m->zSize);  // room for world equal chunks
        const long X = align32((long)n * c0.inChannels * c0.height * c0.width);
        const long Y = align32(n), PR = align32((long)n * numClasses);
        const long work = std::max(fitre_cnn_gradient_mem_required(m), fitre_cnn_hv_mem_required(m));
        const long total = X + Y + 4 * P + 2 * Z + 2 * PR + work;
        if (ctx->host_ws_doubles < (size_t)total) {
            if (ctx->host_ws) FITRE_CUDA(cudaFree(ctx->host_ws));
            ctx->host_ws = nullptr;
            ctx->host_ws_doubles = 0;
            FITRE_CUDA(cudaMalloc((void **)&ctx->host_ws, sizeof(double) * total));
            ctx->host_ws_doubles = total;
        }
        double *x = ctx->host_ws, *y = x + X, *w = y + Y, *v = w + P, *g = v + P, *hv = g + P;
        double *z = hv + P, *dx = z + Z, *probs = dx + Z, *errs = probs + PR, *ws = errs + PR;
        cudaStream_t st = ctx->stream;
        if (!ctx->copy_stream) {
            FITRE_CUDA(cudaStreamCreateWithFlags(&ctx->copy_stream, cudaStreamNonBlocking));
            FITRE_CUDA(cudaEventCreateWithFlags(&ctx->ev_up, cudaEventDisableTiming));
            FITRE_CUDA(cudaEventCreateWithFlags(&ctx->ev_down, cudaEventDisableTiming));
        }
        cudaStream_t cs = ctx->copy_stream;
        if (!ctx->ev_w2) FITRE_CUDA(cudaEventCreateWithFlags(&ctx->ev_w2, cudaEventDisableTiming));
        // Uploads.  The forward pass needs the batch and the first layers' weights at once; the late
        // layers' weights (most of the vector) and the direction vector travel on the copy stream
        // underneath the first layers' compute, in that order so that they do not share the link
        // with what the forward pass is waiting for.
        int split_layer = -1;
        for (int l = 1; l < m->cLayers; ++l)
            if ((long)m->wOffsets[l] * 8 >= (4L << 20)) {
                split_layer = l;
                break;
            }
        const long head = split_layer > 0 ? m->wOffsets[split_layer] : m->pSize;
        FITRE_CUDA(cudaMemcpyAsync(x, batch_host, sizeof(double) * (long)n * c0.inChannels * c0.height * c0.width,
                                   cudaMemcpyHostToDevice, st));
        FITRE_CUDA(cudaMemcpyAsync(y, labels_host, sizeof(double) * n, cudaMemcpyHostToDevice, st));
        // The head of the weights goes up at once on every rank.  The rest, and the direction vector,
        // travel on the copy stream underneath the first layers' compute: in full, or -- replicated
        // inputs, i.e. the same weights and direction on every rank, as data parallelism has them --
        // one of `world` equal chunks per rank, exchanged by an all-gather over NVLink queued on the
        // copy stream, so that the node reads each vector from host memory once.
        FITRE_CUDA(cudaMemcpyAsync(w, weights_host, sizeof(double) * head, cudaMemcpyHostToDevice, st));
        const bool gather = ctx->host_replicated && ctx->world > 1 && ctx->world <= 64 && comm_has_allgather();
        auto upload = [&](double *dst, const double *src, long first, long count) {  // on the copy stream
            if (count <= 0) return;
            if (!gather) {
                FITRE_CUDA(cudaMemcpyAsync(dst + first, src + first, sizeof(double) * (size_t)count,
                                           cudaMemcpyHostToDevice, cs));
                return;
            }
            const long chunk = (count + ctx->world - 1) / ctx->world;
            const long lo = std::min<long>(count, (long)ctx->rank * chunk), hi = std::min<long>(count, lo + chunk);
            if (hi > lo)
                FITRE_CUDA(cudaMemcpyAsync(dst + first + lo, src + first + lo, sizeof(double) * (size_t)(hi - lo),
                                           cudaMemcpyHostToDevice, cs));
            comm_allgather_inplace(ctx, dst + first, (size_t)chunk, cs);
        };
        if (head < m->pSize) {
            upload(w, weights_host, head, m->pSize - head);
            FITRE_CUDA(cudaEventRecord(ctx->ev_w2, cs));
            ctx->fwd_wait_event = ctx->ev_w2;
            ctx->fwd_wait_layer = split_layer;
        }
        upload(v, vector_host, 0, m->pSize);
        FITRE_CUDA(cudaEventRecord(ctx->ev_up, cs));
        DEVICE_DATASET data;
        std::memset(&data, 0, sizeof(data));
        data.weights = w;
        data.currentBatch = x;
        data.sampledTrainY = y;
        data.numClasses = numClasses;
        SCRATCH_AREA sa;
        std::memset(&sa, 0, sizeof(sa));
        sa.devWorkspace = sa.nextDevPtr = ws;
        double loss = 0.0;
        int rc = fitre_compute_cnn_gradient(ctx, m, &data, &sa, z, dx, probs, errs, g, 0, n,
                                            weightDecay, &loss);
        ctx->fwd_wait_event = nullptr;
        ctx->fwd_wait_layer = -1;
        FITRE_REQUIRE(rc == FITRE_OK, rc, ctx->err);
        // the gradient call returned after a stream sync (loss read-back): g is complete and
        // travels back on the copy stream while the Hessian-vector product runs
        {
            long lo, hi;
            host_share(ctx, 0, m->pSize, lo, hi);
            FITRE_CUDA(cudaMemcpyAsync(gradient_host + lo, g + lo, sizeof(double) * (size_t)(hi - lo),
                                       cudaMemcpyDeviceToHost, cs));
        }
        FITRE_CUDA(cudaStreamWaitEvent(st, ctx->ev_up, 0));
        // finished slices of hv follow the gradient on the copy stream as the backward sweep completes
        // its layers (with ranks: as each layer's slice has been all-reduced on the side stream)
        ctx->hv_host_dst = (ctx->world == 1 || comm_async_stream(ctx)) ? hv_host : nullptr;
        ctx->hv_sent_from = m->pSize;
        rc = fitre_cnn_hv(ctx, m, &data, z, probs, errs, dx, v, hv, 0, n, ws, nullptr, weightDecay);
        const long sent_from = ctx->hv_host_dst ? ctx->hv_sent_from : m->pSize;
        ctx->hv_host_dst = nullptr;
        FITRE_REQUIRE(rc == FITRE_OK, rc, ctx->err);
        if (sent_from > 0) {
            long lo, hi;
            host_share(ctx, 0, sent_from, lo, hi);
            if (hi > lo)
                FITRE_CUDA(cudaMemcpyAsync(hv_host + lo, hv + lo, sizeof(double) * (size_t)(hi - lo),
                                           cudaMemcpyDeviceToHost, st));
        }
        FITRE_CUDA(cudaEventRecord(ctx->ev_down, cs));
        if (ctx->host_shared && ctx->world > 1) {
            // every rank wrote its share of the one buffer: a one-element all-reduce queued behind
            // this rank's copies completes only when all ranks have queued theirs, i.e. sent their shares
            FITRE_CUDA(cudaStreamWaitEvent(st, ctx->ev_down, 0));
            comm_allreduce_sum(ctx, ctx->dscal + 3890, 1);
        }
        stream_wait(ctx, st);
        FITRE_CUDA(cudaEventSynchronize(ctx->ev_down));
        if (loss_host) *loss_host = loss;
    });
}

}  // extern "C"
