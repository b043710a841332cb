// Pieces of the training loop either side of the gradient / Hessian-vector path: minibatch
// assembly on the device (gather + layout change + augmentation + normalisation in one kernel),
// running batch-norm statistics set-up, accuracy, and the generalisation-error sweeps over a
// whole train or test set.
#include <algorithm>
#include <chrono>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <utility>
#include <vector>

#include "common.h"

namespace fitre {
namespace {

constexpr int kThreads = 256;
inline long align32(long n) { return (n + 31) / 32 * 32; }

// solvers/kfac_trust_region.cu:66-77 + functions/dev_batch_norm.cu:235-255
__global__ void init_running_stats_kernel(double *run_mean, double *run_var, int C) {
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c < C) {
        run_mean[c] = 0.0;
        run_var[c] = 1.0;
    }
}

// functions/cnn_accuracy.cu:16-37: one thread per sample scans the classes with a strict `<`
// against a running maximum that starts at 0; hit when class + 1 equals the label.  One block,
// fixed-order tree reduction (bit-reproducible, and the count is an integer anyway).
__global__ void accuracy_kernel(const double *probs, const double *target, int rows, int classes,
                                double *hits_out) {
    __shared__ double red[kThreads];
    double hits = 0.0;
    for (int i = threadIdx.x; i < rows; i += kThreads) {
        double best = 0.0;
        int cls = 0;
        for (int c = 0; c < classes; ++c) {
            const double p = probs[(long)i * classes + c];
            if (best < p) {
                best = p;
                cls = c;
            }
        }
        if ((double)(cls + 1) == target[i]) hits += 1.0;
    }
    red[threadIdx.x] = hits;
    __syncthreads();
    for (int s = kThreads / 2; s > 0; s >>= 1) {
        if (threadIdx.x < s) red[threadIdx.x] += red[threadIdx.x + s];
        __syncthreads();
    }
    if (threadIdx.x == 0) *hits_out = red[0];
}

struct NormConst {
    double mean[3], sd[3];
};

// One thread per element of the assembled batch [C][N][W][H] (h fastest, so writes coalesce and
// reads run along image columns).  Source image = column `indices[offset + im]` (or offset + im)
// of the features x samples matrix, stored per image as [C][W][H].
// utilities/sample_matrix.cu:70-92, solvers/kfac_da.cu:22-89, augmentation/dev_crop.cu:14-62,
// augmentation/dev_flip.cu:61-92, augmentation/dev_normalize.cu:12-36.
__global__ void prepare_minibatch_kernel(const double *__restrict__ setX, const double *__restrict__ setY,
                                         const int *__restrict__ indices, long offset, int n, int C,
                                         int H, int W, const double *__restrict__ uniforms,
                                         NormConst nc, double *__restrict__ batch,
                                         double *__restrict__ labels) {
    const long plane = (long)H * W, total = plane * C * n;
    for (long idx = blockIdx.x * (long)blockDim.x + threadIdx.x; idx < total;
         idx += (long)gridDim.x * blockDim.x) {
        const int row = (int)(idx % H);
        long t = idx / H;
        const int col = (int)(t % W);
        t /= W;
        const int im = (int)(t % n);
        const int c = (int)(t / n);
        const long src = indices ? (long)indices[offset + im] : offset + im;
        int dr = 0, dc = 0, ccol = col;
        if (uniforms) {
            dr = __double2int_rz(uniforms[im] * 100.) % 9 - 4;
            dc = __double2int_rz(uniforms[n + im] * 100.) % 9 - 4;
            if (uniforms[2 * n + im] < 0.5) ccol = W - 1 - col;
        }
        const int sr = row + dr, sc = ccol + dc;
        double v = 0.0;
        if (sr >= 0 && sc >= 0 && sr < H && sc < W) v = setX[src * plane * C + c * plane + (long)sc * H + sr];
        v /= 255.;
        v = (v - nc.mean[c % 3]) / nc.sd[c % 3];
        batch[idx] = v;
        if (c == 0 && col == 0 && row == 0) labels[im] = setY[src];
    }
}

// utilities/sample_matrix.cu:12-30 (kerExtractColumns): dst column j = src column indices[j]
__global__ void select_columns_kernel(const double *__restrict__ src, const int *__restrict__ indices,
                                      long rows, long total, double *__restrict__ dst) {
    for (long idx = blockIdx.x * (long)blockDim.x + threadIdx.x; idx < total;
         idx += (long)gridDim.x * blockDim.x) {
        const long col = idx / rows, r = idx - col * rows;
        dst[idx] = src[(long)indices[col] * rows + r];
    }
}

NormConst norm_constants(int datasetType) {
    // augmentation/dev_normalize.cu:52-83; DATASET_TYPE values core/structdefs.h:17-21
    switch (datasetType) {
        case 20: return NormConst{{0.5071, 0.4865, 0.4409}, {0.2673, 0.2564, 0.2762}};
        case 30: return NormConst{{0.4799, 0.4478, 0.3972}, {0.2769, 0.2690, 0.2820}};
        case 10: return NormConst{{0.4914, 0.4822, 0.4465}, {0.2470, 0.2435, 0.2616}};
        default: throw Error(FITRE_ERR_BAD_ARG, "datasetType must be CIFAR10 (10), CIFAR100 (20) or IMAGENET (30)");
    }
}

}  // namespace

void init_batch_norm_data(fitre_context *ctx, const CNN_MODEL *m, double *z) {
    for (int l = 0; l < m->cLayers; ++l) {
        const CONV_LAYER &c = m->convLayer[l];
        if (c.batchNorm == FITRE_NO_BATCH_NORM) continue;
        double *bn = z + m->zOffsets[l + 1] + c.batchNormOffset;
        init_running_stats_kernel<<<(c.outChannels + 127) / 128, 128, 0, ctx->stream>>>(
            bn + c.runningMeansOffset, bn + c.runningVariancesOffset, c.outChannels);
        check_launch(ctx, "init_running_stats_kernel");
    }
}

// hits over the global batch (all ranks), left in ctx->pinned[0] after a stream synchronise
double compute_hits(fitre_context *ctx, const double *probs, const double *target, int rows, int classes) {
    accuracy_kernel<<<1, kThreads, 0, ctx->stream>>>(probs, target, rows, classes, ctx->dscal);
    check_launch(ctx, "accuracy_kernel");
    comm_allreduce_small(ctx, ctx->dscal, 1);
    FITRE_CUDA(cudaMemcpyAsync(ctx->pinned, ctx->dscal, sizeof(double), cudaMemcpyDeviceToHost, ctx->stream));
    stream_wait(ctx, ctx->stream);
    return ctx->pinned[0];
}

void prepare_minibatch(fitre_context *ctx, const CNN_MODEL *m, DEVICE_DATASET *data, const double *setX,
                       const double *setY, const int *indices, long offset, int n,
                       const double *uniforms) {
    const CONV_LAYER &c0 = m->convLayer[0];
    const int C = c0.inChannels, H = c0.height, W = c0.width;
    FITRE_REQUIRE((long)C * H * W == data->features, FITRE_ERR_BAD_ARG,
                  "data->features must equal channels*height*width of the first layer");
    const NormConst nc = norm_constants(data->datasetType);
    // the assembled batch goes where the reference leaves it: the second half of sampledTrainX
    double *batch = data->sampledTrainX + (long)n * data->features;
    const long total = (long)n * data->features;
    const int grid = (int)std::min<long>((total + kThreads - 1) / kThreads, 148 * 16);
    prepare_minibatch_kernel<<<grid, kThreads, 0, ctx->stream>>>(setX, setY, indices, offset, n, C, H, W,
                                                                 uniforms, nc, batch, data->sampledTrainY);
    check_launch(ctx, "prepare_minibatch_kernel");
    data->currentBatch = batch;
}

}  // namespace fitre

using namespace fitre;

#define FITRE_ENTRY_BEGIN              \
    if (!ctx) return FITRE_ERR_BAD_ARG; \
    try {                               \
        FITRE_CUDA(cudaSetDevice(ctx->device));
#define FITRE_ENTRY_END          \
    return FITRE_OK;             \
    }                            \
    catch (const Error &e) {     \
        ctx->err = e.what();     \
        return e.code;           \
    }

extern "C" int fitre_init_batch_norm_data(fitre_context *ctx, const CNN_MODEL *m, real *z) {
    FITRE_ENTRY_BEGIN
    FITRE_REQUIRE(m && z, FITRE_ERR_BAD_ARG, "NULL pointer argument");
    init_batch_norm_data(ctx, m, z);
    FITRE_ENTRY_END
}

extern "C" int fitre_compute_accuracy(fitre_context *ctx, const real *probs, const real *target, int rows,
                                      int numClasses, real *hits_host, real *accuracy_host) {
    FITRE_ENTRY_BEGIN
    FITRE_REQUIRE(probs && target && rows > 0 && numClasses > 0, FITRE_ERR_BAD_ARG, "bad argument");
    const double hits = compute_hits(ctx, probs, target, rows, numClasses);
    if (hits_host) *hits_host = hits;
    if (accuracy_host) *accuracy_host = hits * 100. / ((double)rows * ctx->world);
    FITRE_ENTRY_END
}

extern "C" int fitre_select_column_matrix(fitre_context *ctx, DEVICE_DATASET *data, int sampleSize,
                                          const int *indices, int offset) {
    FITRE_ENTRY_BEGIN
    FITRE_REQUIRE(data && indices && sampleSize > 0 && offset >= 0 && data->trainSetX && data->trainSetY &&
                      data->sampledTrainX && data->sampledTrainY && data->features > 0,
                  FITRE_ERR_BAD_ARG, "bad argument");
    const long total = (long)sampleSize * data->features;
    select_columns_kernel<<<(int)std::min<long>((total + kThreads - 1) / kThreads, 148 * 16), kThreads, 0,
                            ctx->stream>>>(data->trainSetX, indices + offset, data->features, total,
                                           data->sampledTrainX);
    check_launch(ctx, "select_columns_kernel");
    select_columns_kernel<<<(sampleSize + kThreads - 1) / kThreads, kThreads, 0, ctx->stream>>>(
        data->trainSetY, indices + offset, 1, sampleSize, data->sampledTrainY);
    check_launch(ctx, "select_columns_kernel");
    FITRE_ENTRY_END
}

extern "C" int fitre_prepare_minibatch(fitre_context *ctx, const CNN_MODEL *m, DEVICE_DATASET *data,
                                       const real *setX, const real *setY, const int *indices,
                                       long offset, int n, const real *uniforms) {
    FITRE_ENTRY_BEGIN
    FITRE_REQUIRE(m && data && setX && setY && data->sampledTrainX && data->sampledTrainY && n > 0 &&
                      offset >= 0,
                  FITRE_ERR_BAD_ARG, "bad argument");
    prepare_minibatch(ctx, m, data, setX, setY, indices, offset, n, uniforms);
    FITRE_ENTRY_END
}

extern "C" int fitre_evaluate_cnn_model(fitre_context *ctx, const CNN_MODEL *m, const DEVICE_DATASET *data,
                                        SCRATCH_AREA *scratch, real *z, real *probs, real *lossFuncErrors,
                                        int offset, int curBatchSize, real *loss_host) {
    return fitre_cnn_forward(ctx, m, data, scratch, z, probs, lossFuncErrors, offset, curBatchSize,
                             FITRE_MODEL_TRAIN, loss_host);
}

// ---------------------------------------------------------------------------------------------
// generalisation sweeps
namespace fitre {
namespace {

#define FITRE_RC(call)                                                        \
    do {                                                                      \
        int rc_ = (call);                                                     \
        if (rc_ != FITRE_OK) throw Error(rc_, ctx->err.empty() ? #call : ctx->err); \
    } while (0)

long running_stat_doubles(const CNN_MODEL *m) {
    long n = 0;
    for (int l = 0; l < m->cLayers; ++l)
        if (m->convLayer[l].batchNorm != FITRE_NO_BATCH_NORM) n += 2L * m->convLayer[l].outChannels;
    return n;
}

// copy every layer's running mean/variance pair between `z` (laid out for model `m`) and a packed array
void move_running_stats(fitre_context *ctx, const CNN_MODEL *m, double *z, double *packed, bool to_packed) {
    long o = 0;
    for (int l = 0; l < m->cLayers; ++l) {
        const CONV_LAYER &c = m->convLayer[l];
        if (c.batchNorm == FITRE_NO_BATCH_NORM) continue;
        double *rs = z + m->zOffsets[l + 1] + c.batchNormOffset + c.runningMeansOffset;
        // running variances follow the running means directly (nn/read_vgg.c:77-101)
        if (to_packed)
            vec_copy(ctx, 2L * c.outChannels, rs, packed + o);
        else
            vec_copy(ctx, 2L * c.outChannels, packed + o, rs);
        o += 2L * c.outChannels;
    }
}

struct SweepTotals {
    double likelihood = 0, hits = 0;
};

// one evaluation batch of `n` images starting at image `first` of the set; returns through totals
void eval_batch(fitre_context *ctx, const CNN_MODEL *m, DEVICE_DATASET *data, double *fwd_scratch,
                const double *setX, const double *setY, long first, int n, long weight, double *z,
                double *probs, double *errors, SweepTotals &t) {
    prepare_minibatch(ctx, m, data, setX, setY, nullptr, first, n, nullptr);
    const double loss = cnn_forward(ctx, m, data, fwd_scratch, z, probs, errors, n, true, true);
    t.likelihood += loss * (double)weight;
    t.hits += compute_hits(ctx, probs, data->sampledTrainY, n, data->numClasses);
}

}  // namespace
}  // namespace fitre

extern "C" long fitre_generalization_mem_required(const CNN_MODEL *m) {
    if (!m) return -1;
    return align32(forward_scratch(m)) + align32(running_stat_doubles(m)) + 64;
}

extern "C" int fitre_compute_generalization_errors(fitre_context *ctx, const CNN_MODEL *m,
                                                   DEVICE_DATASET *data, SCRATCH_AREA *scratch, real *z,
                                                   real *probs, real *errors, int evalType,
                                                   real *likelihood, real *accuracy) {
    FITRE_ENTRY_BEGIN
    FITRE_REQUIRE(m && data && scratch && scratch->nextDevPtr && z && probs && errors && likelihood && accuracy,
                  FITRE_ERR_BAD_ARG, "NULL pointer argument");
    FITRE_REQUIRE(evalType == FITRE_MODEL_TEST_ACCURACY || evalType == FITRE_MODEL_TRAIN_ACCURACY,
                  FITRE_ERR_BAD_ARG, "evalType must be one of the two accuracy modes");
    const bool test = evalType == FITRE_MODEL_TEST_ACCURACY;
    const double *setX = test ? data->testSetX : data->trainSetX;
    const double *setY = test ? data->testSetY : data->trainSetY;
    const long size = test ? data->testSizeX : data->trainSizeX;
    FITRE_REQUIRE(setX && setY && size > 0, FITRE_ERR_BAD_ARG, "empty data set");
    FITRE_RC(fitre_model_validate(m));
    const int B = m->batchSize, W = ctx->world;
    double *fwd = scratch->nextDevPtr;
    double *packed = fwd + align32(forward_scratch(m));
    real *const saved_batch = data->currentBatch;

    // the batches of the reference's loop (functions/cnn_accuracy.cu:76-108 and :138-170)
    SweepTotals tot;
    long cur_idx = 0;
    int cur = B;
    std::vector<std::pair<long, int>> batches;
    while (cur_idx < size) {
        batches.push_back({cur_idx, cur});
        cur_idx += cur;
        if (cur_idx + B < size) {
            cur = B;
        } else {
            cur = (int)(size - cur_idx);
            if (!test) break;
        }
    }
    // full batches: W at a time in lockstep, rank r takes the r-th of each group
    size_t i = 0;
    const int saved_world = ctx->world;
    auto is_full = [&](size_t k) { return k < batches.size() && batches[k].second == B; };
    while (W > 1) {
        bool group = true;
        for (int r = 0; r < W; ++r) group = group && is_full(i + r);
        if (!group) break;
        // loss returned is the mean over the W batches, hits their sum
        eval_batch(ctx, m, data, fwd, setX, setY, batches[i + ctx->rank].first, B, (long)B * W, z, probs,
                   errors, tot);
        i += W;
    }
    // the rest: every rank evaluates the same batches on its own (no exchange)
    ctx->world = 1;
    try {
        for (; i < batches.size(); ++i) {
            const long first = batches[i].first;
            const int n = batches[i].second;
            if (n <= 0) continue;
            if (n == B) {
                eval_batch(ctx, m, data, fwd, setX, setY, first, n, n, z, probs, errors, tot);
            } else {
                // partial last batch: the same net laid out for n images; the running statistics move
                // into its layout and back (every other part of z is scratch for an evaluation)
                CNN_MODEL tail = *m;
                tail.batchSize = n;
                FITRE_RC(fitre_model_finalize(&tail));
                move_running_stats(ctx, m, z, packed, true);
                move_running_stats(ctx, &tail, z, packed, false);
                eval_batch(ctx, &tail, data, fwd, setX, setY, first, n, n, z, probs, errors, tot);
                move_running_stats(ctx, m, z, packed, false);
            }
        }
    } catch (...) {
        ctx->world = saved_world;
        data->currentBatch = saved_batch;
        throw;
    }
    ctx->world = saved_world;
    data->currentBatch = saved_batch;
    *accuracy = tot.hits * 100. / (double)size;
    *likelihood = tot.likelihood / (double)size;
    FITRE_ENTRY_END
}

// ---------------------------------------------------------------------------------------------
// .params text files (utilities/print_utils.c:136-186)
extern "C" int fitre_write_vector(const char *path, const real *host, long n, int referenceFormat) {
    if (!path || !host || n < 0) return FITRE_ERR_BAD_ARG;
    FILE *f = fopen(path, "w");
    if (!f) return FITRE_ERR_BAD_ARG;
    for (long i = 0; i < n; ++i) fprintf(f, referenceFormat ? "%6.10f\n" : "%.17g\n", host[i]);
    return fclose(f) == 0 ? FITRE_OK : FITRE_ERR_BAD_ARG;
}

extern "C" int fitre_read_vector(const char *path, real *host, long n, long *read_out) {
    if (!path || !host || n < 0) return FITRE_ERR_BAD_ARG;
    FILE *f = fopen(path, "r");
    if (!f) return FITRE_ERR_BAD_ARG;
    char line[1024];
    long k = 0;
    while (k < n && fgets(line, sizeof line, f)) {
        if (line[0] == 0 || line[0] == '\n') break;
        host[k++] = atof(line);
    }
    fclose(f);
    if (read_out) *read_out = k;
    return FITRE_OK;
}

// ---------------------------------------------------------------------------------------------
// The FITRE outer loop (solvers/kfac_trust_region.cu:94-661), inverseFreq == 1.
namespace fitre {
namespace {

// splitmix64 (public-domain counter-based generator): every rank draws the same stream
struct Rng {
    unsigned long long s;
    unsigned long long next() {
        unsigned long long z = (s += 0x9E3779B97F4A7C15ull);
        z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
        z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
        return z ^ (z >> 31);
    }
    double uniform() { return (double)(next() >> 11) * (1.0 / 9007199254740992.0); }  // [0,1)
};

struct TrLayout {
    long indices, uniforms, A, Ainv, G, Ginv, gradient, distGradient, prevWeights, nGradient, z, dx,
        distDX, probs, errors, dist1, dist2, distTarget, dInput, dZ, dLambda, scratch, factorScratch, total;
};
TrLayout tr_layout(const CNN_MODEL *m, const DEVICE_DATASET *data, const FITRE_KFAC_INFO &info) {
    TrLayout L{};
    long o = 0;
    auto take = [&](long n) {
        long at = o;
        o += align32(n);
        return at;
    };
    const long B = m->batchSize, P = m->pSize, Z = m->zSize, md = max_delta_elems(m) + 32;
    L.indices = take((data->trainSizeX + 1) / 2);
    L.uniforms = take(4 * B);
    L.A = take(info.OmegaZSize);
    L.Ainv = take(info.OmegaZSize);
    L.G = take(info.LambdaGSize);
    L.Ginv = take(info.LambdaGSize);
    L.gradient = take(P);
    L.distGradient = take(P);
    L.prevWeights = take(P);
    L.nGradient = take(P);
    L.z = take(Z);
    L.dx = take(Z);
    L.distDX = take(Z);
    L.probs = take(B * data->numClasses);
    L.errors = take(md);
    L.dist1 = take(md);
    L.dist2 = take(md);
    L.distTarget = take(B);
    if (info.inverseFreq > 1) {  // running averages of the "speed-up" variant
        L.dInput = take(B * data->features);
        L.dZ = take(m->zztSize);
        L.dLambda = take(m->zztSize);
    }
    long need = std::max(fitre_cnn_gradient_mem_required(m), fitre_quadratic_model_mem_required(m));
    need = std::max(need, fitre_kfac_mem_required(m));
    need = std::max(need, fitre_kfac_factors_and_inverses_mem_required(m));
    need = std::max(need, fitre_kfac_natural_gradient_mem_required(m));
    need = std::max(need, fitre_generalization_mem_required(m));
    L.scratch = take(need);
    // the A side of the factor step runs underneath the backward passes: scratch of its own
    L.factorScratch = take(fitre_kfac_factors_and_inverses_mem_required(m));
    L.total = o;
    return L;
}

}  // namespace
}  // namespace fitre

extern "C" long fitre_trust_region_kfac_mem_required(const CNN_MODEL *m, const DEVICE_DATASET *data,
                                                     const FITRE_KFAC_INFO *kfacInfo) {
    if (!m || !data) return -1;
    FITRE_KFAC_INFO info{};
    if (kfacInfo) info = *kfacInfo;
    if (fitre_kfac_storage_indices(m, &info) != FITRE_OK) return -1;
    return tr_layout(m, data, info).total;
}

extern "C" int fitre_subsampled_trust_region_kfac(fitre_context *ctx, CNN_MODEL *m, DEVICE_DATASET *data,
                                                  FITRE_KFAC_INFO *kfacInfo, TRUST_REGION_PARAMS *trParams,
                                                  SCRATCH_AREA *scratch, unsigned long long seed,
                                                  int enableDA, int maxMiniBatches, FITRE_TR_STEP *steps,
                                                  int stepsCap, FITRE_TR_EPOCH *epochs) {
    FITRE_ENTRY_BEGIN
    FITRE_REQUIRE(m && data && kfacInfo && trParams && scratch && scratch->nextDevPtr, FITRE_ERR_BAD_ARG,
                  "NULL pointer argument");
    FITRE_REQUIRE(data->trainSetX && data->trainSetY && data->weights && data->sampledTrainX &&
                      data->sampledTrainY,
                  FITRE_ERR_BAD_ARG, "data set pointers missing");
    FITRE_RC(fitre_model_validate(m));
    FITRE_RC(fitre_kfac_storage_indices(m, kfacInfo));
    // the factor and inverse buffers are the loop's own: with ranks each layer's factors stay on an
    // owner rank and only the natural gradient is exchanged
    struct OwnedFactors {
        fitre_context *c;
        int prev;
        explicit OwnedFactors(fitre_context *ctx_) : c(ctx_), prev(ctx_->kfac_owned) { c->kfac_owned = 1; }
        ~OwnedFactors() { c->kfac_owned = prev; }
    } owned_factors(ctx);
    const TrLayout L = tr_layout(m, data, *kfacInfo);
    double *base = scratch->nextDevPtr;
    int *shuffle = (int *)(base + L.indices);
    double *uniforms = base + L.uniforms, *A = base + L.A, *Ainv = base + L.Ainv, *G = base + L.G,
           *Ginv = base + L.Ginv, *gradient = base + L.gradient, *distGradient = base + L.distGradient,
           *prevWeights = base + L.prevWeights, *nGradient = base + L.nGradient, *z = base + L.z,
           *dx = base + L.dx, *distDX = base + L.distDX, *probs = base + L.probs,
           *errors = base + L.errors, *dist1 = base + L.dist1, *dist2 = base + L.dist2,
           *distTarget = base + L.distTarget, *work = base + L.scratch, *fwork = base + L.factorScratch;
    const int invFreq = kfacInfo->inverseFreq > 1 ? kfacInfo->inverseFreq : 1;
    double *dInput = invFreq > 1 ? base + L.dInput : nullptr, *dZ = invFreq > 1 ? base + L.dZ : nullptr,
           *dLambda = invFreq > 1 ? base + L.dLambda : nullptr;
    int total_mb = 0;
    SCRATCH_AREA inner = *scratch;
    inner.nextDevPtr = work;

    const int B = m->batchSize, W = ctx->world, P = m->pSize, classes = data->numClasses;
    const long trainN = data->trainSizeX;
    const long GB = (long)B * W;  // images per global minibatch
    const double damp_l = kfacInfo->regLambda;
    Rng rng{seed};
    std::vector<int> host_idx(trainN);
    std::vector<double> host_u(4 * GB);

    vec_fill(ctx, P, 0.0, prevWeights);
    init_batch_norm_data(ctx, m, z);
    int step_no = 0;
    for (int iter = 0; iter < trParams->maxIters; ++iter) {
        const auto t0 = std::chrono::steady_clock::now();
        // shuffled order of the training set (device/gen_random.c:76-98 with m == n: a permutation)
        for (long i = 0; i < trainN; ++i) host_idx[i] = (int)i;
        for (long i = trainN - 1; i > 0; --i) std::swap(host_idx[i], host_idx[rng.next() % (unsigned long long)(i + 1)]);
        FITRE_CUDA(cudaMemcpyAsync(shuffle, host_idx.data(), sizeof(int) * trainN, cudaMemcpyHostToDevice, ctx->stream));
        stream_wait(ctx, ctx->stream);
        long offset = 0;
        int mb = 0;
        // the reference stops before the last batch that would reach the end of the set (:303-308)
        while (offset + GB < trainN && (maxMiniBatches <= 0 || mb < maxMiniBatches)) {
            // random draws of this minibatch: [rows | cols | flips | labels] x GB, rank r uses its slice
            for (long i = 0; i < 4 * GB; ++i) host_u[i] = rng.uniform();
            for (int part = 0; part < 4; ++part)
                FITRE_CUDA(cudaMemcpyAsync(uniforms + (long)part * B, host_u.data() + part * GB + (long)ctx->rank * B,
                                           sizeof(double) * B, cudaMemcpyHostToDevice, ctx->stream));
            stream_wait(ctx, ctx->stream);
            prepare_minibatch(ctx, m, data, data->trainSetX, data->trainSetY, shuffle,
                              offset + (long)ctx->rank * B, B, enableDA ? uniforms : nullptr);

            // gradient of the regularised loss (:343-362)
            const double trainLik = cnn_forward(ctx, m, data, work, z, probs, errors, B, true, false);
            // Live-state factors: the A side needs the forward state only, so its factor products and
            // the factorisation chains start here, on the library's own streams, and run underneath the
            // two backward passes; the G side joins them after the sampled-label pass.
            const bool two_call = invFreq <= 1;
            if (two_call)
                FITRE_RC(fitre_kfac_omega_z_begin(ctx, m, data->currentBatch, z, 0, B, A, Ainv, kfacInfo, fwork));
            vec_copy(ctx, (long)B * classes, errors, dist1);
            cnn_backward(ctx, m, data, work, z, gradient, dx, dist1, dist2, B);
            comm_allreduce_sum(ctx, gradient, P);
            vec_axpy(ctx, P, damp_l, data->weights, gradient);

            // backward pass with labels sampled from the model's own predictions (:371-389)
            distribution_errors(ctx, probs, uniforms + 3L * B, B, classes, distTarget, dist1,
                                1.0 / ((double)B * W));
            cnn_backward(ctx, m, data, work, z, distGradient, distDX, dist1, dist2, B);

            // factors and their damped inverses (:404-411, solvers/kfac_inverses.cu:450-630,759-857)
            // with inverseFreq > 1: running averages every minibatch, factors on the very first minibatch from
            // the live state and then every inverseFreq minibatches from the averages (:392-411)
            bool refresh = true, from_avg = false;
            if (invFreq > 1) {
                FITRE_RC(fitre_kfac_speedup_omega_z(ctx, kfacInfo, m, data, B, z, dInput, dZ, iter + (int)offset));
                FITRE_RC(fitre_kfac_speedup_lambda_delta(ctx, kfacInfo, m, B, distDX, dLambda, iter + (int)offset));
                if (iter == 0 && total_mb == 0) from_avg = false;
                else if (total_mb % invFreq == 0) from_avg = true;
                else refresh = false;
            }
            // one call forms the factors and inverts them, the factorisations under the factor products
            if (two_call)
                FITRE_RC(fitre_kfac_lambda_delta_finish(ctx, m, distDX, 0, B, G, Ginv, kfacInfo, fwork));
            else if (refresh && from_avg)
                FITRE_RC(fitre_kfac_factors_and_inverses(ctx, m, dInput, dZ, dLambda, 1, B, A, Ainv, G, Ginv,
                                                         kfacInfo, work));
            else if (refresh)
                FITRE_RC(fitre_kfac_factors_and_inverses(ctx, m, data->currentBatch, z, distDX, 0, B, A, Ainv, G,
                                                         Ginv, kfacInfo, work));
            FITRE_RC(fitre_compute_natural_gradient(ctx, m, kfacInfo, Ainv, Ginv, gradient, nGradient, work));

            // quadratic models of the two candidate steps (:452-470); each call scales its direction
            double mKfac = 0, mGrad = 0;
            FITRE_RC(fitre_compute_quadratic_model(ctx, m, data, z, probs, errors, dx, gradient, nGradient,
                                                   trParams->delta, 0, B, damp_l, work, nullptr, nullptr, &mKfac));
            if (kfacInfo->checkGrad)
                FITRE_RC(fitre_compute_quadratic_model(ctx, m, data, z, probs, errors, dx, gradient, gradient,
                                                       trParams->delta, 0, B, damp_l, work, nullptr, nullptr, &mGrad));
            const bool use_kfac = !kfacInfo->checkGrad || mKfac < mGrad;
            double *dir = use_kfac ? nGradient : gradient;
            // momentum, step, remember the step (:476-492 / :520-534)
            vec_axpy(ctx, P, kfacInfo->momentum, prevWeights, dir);
            vec_axpy(ctx, P, -1.0, dir, data->weights);
            vec_copy(ctx, P, dir, prevWeights);

            const double newLik = cnn_forward(ctx, m, data, work, z, probs, errors, B, true, false);
            const double hits = compute_hits(ctx, probs, data->sampledTrainY, B, classes);
            const double newAcc = hits * 100. / ((double)B * W);
            check_device_error(ctx);
            const double rho = (newLik - trainLik) / ((use_kfac ? mKfac : mGrad) - 1e-16);
            if (rho > 0.75) trParams->delta = std::min(trParams->maxDelta, 2. * trParams->delta);
            if (rho < 0.25) trParams->delta = std::max(trParams->minDelta, 0.5 * trParams->delta);
            bool reverted = false;
            if (rho < 1e-4 || newLik > 10. * trainLik) {
                vec_axpy(ctx, P, 1.0, prevWeights, data->weights);  // :575-583
                reverted = true;
            }
            if (steps && step_no < stepsCap)
                steps[step_no] = FITRE_TR_STEP{trainLik, newLik, newAcc, mKfac, mGrad, rho, trParams->delta,
                                               use_kfac ? 1 : 0, reverted ? 1 : 0};
            ++step_no;
            offset += GB;
            ++mb;
            ++total_mb;
        }
        stream_wait(ctx, ctx->stream);
        const double secs = std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
        // end of epoch: generalisation errors with the running statistics (:621-640)
        FITRE_TR_EPOCH ep{};
        ep.seconds = secs;
        ep.miniBatches = mb;
        if (data->testSetX && data->testSetY && data->testSizeX > 0)
            FITRE_RC(fitre_compute_generalization_errors(ctx, m, data, &inner, z, probs, errors,
                                                         FITRE_MODEL_TEST_ACCURACY, &ep.testLikelihood, &ep.testAccuracy));
        FITRE_RC(fitre_compute_generalization_errors(ctx, m, data, &inner, z, probs, errors,
                                                     FITRE_MODEL_TRAIN_ACCURACY, &ep.trainLikelihood, &ep.trainAccuracy));
        if (epochs) epochs[iter] = ep;
    }
    trParams->curIteration = step_no;
    FITRE_ENTRY_END
}
