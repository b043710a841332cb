// Link-level drop-in for the reference's drivers: the C++ functions the reference's solver and
// test drivers call on this path, under the reference's own (mangled) names and parameter lists,
// forwarding to the C ABI of libfitre_b200.  A reference object file compiled against the
// reference's headers links against this library instead of the reference's functions/*.cu and
// solvers/kfac_*.cu objects.
//
// The struct types appear here only as opaque tags spelled as the reference spells them (struct
// cnn, dev_dataset, scratch_space, host_dataset, kfac_curvature), which is what C++ name mangling
// records; the layouts are those of include/fitre_b200.h (same fields in the same order).
//
// Conventions kept from the reference (device/cuda_utils.h:28-92, core/errors.h): calls are
// synchronous and a failure prints a message and exits the process.  The library context the
// reference keeps as global handles (device/handles.h:15-20) is one lazily created
// fitre_context on the calling thread's current CUDA device.
#include <cuda_runtime.h>

#include <cstdio>
#include <cstdlib>
#include <vector>

#include "fitre_b200.h"

struct cnn;
struct dev_dataset;
struct scratch_space;
struct host_dataset;
struct cublasContext;
struct cusolverDnContext;
struct CUstream_st;
enum eval_type { MODEL_TRAIN = 10, MODEL_TRAIN_ACCURACY = 20, MODEL_TEST_ACCURACY = 30 };  // nn/nn_decl.h:28-32
enum dataset_type { CIFAR10 = 10, CIFAR100 = 20, IMAGENET = 30 };                          // core/structdefs.h:17-21

// solvers/kfac_structs.h:12-48, field for field (the reference's MAX_LAYERS is FITRE_MAX_LAYERS)
struct kfac_curvature {
    real *OmegaZZT, *LambdaGGT, *OmegaZInv, *LambdaGInv;
    real *vec, *nGradient, *gradient;
    int OmegaZOffsets[FITRE_MAX_LAYERS], LambdaGOffsets[FITRE_MAX_LAYERS];
    real stats_decay, momentum, regLambda, dampGamma;
    int checkGrad;
    int dampedInputSize;
    real *dampedInput, *dampedZ, *dampedLambda;
    int inverseFreq;
};

namespace {

fitre_context *g_ctx = nullptr;
unsigned long long g_rng = 0x9E3779B97F4A7C15ull;  // uniforms for the draws the reference takes from cuRAND

fitre_context *ctx() {
    if (!g_ctx) {
        int dev = 0;
        cudaGetDevice(&dev);
        if (fitre_context_create(&g_ctx, dev, nullptr) != FITRE_OK) {
            fprintf(stderr, "fitre shim: cannot create a context on device %d\n", dev);
            exit(-1);
        }
    }
    return g_ctx;
}
void die(int rc, const char *what) {
    // a NaN loss is not a failure in the reference: it returns the value and carries on
    if (rc == FITRE_OK || rc == FITRE_ERR_NOT_FINITE) return;
    fprintf(stderr, "fitre shim: %s failed (%d): %s\n", what, rc, fitre_last_error(g_ctx));
    exit(rc);
}
double next_uniform() {
    unsigned long long z = (g_rng += 0x9E3779B97F4A7C15ull);
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    z ^= z >> 31;
    return (double)(z >> 11) * (1.0 / 9007199254740992.0);
}
void upload_uniforms(real *dev, long n) {
    std::vector<double> u(n);
    for (long i = 0; i < n; ++i) u[i] = next_uniform();
    if (cudaMemcpy(dev, u.data(), sizeof(double) * n, cudaMemcpyHostToDevice) != cudaSuccess) {
        fprintf(stderr, "fitre shim: uniform upload failed\n");
        exit(-1);
    }
}
CNN_MODEL *M(cnn *m) { return reinterpret_cast<CNN_MODEL *>(m); }
DEVICE_DATASET *D(dev_dataset *d) { return reinterpret_cast<DEVICE_DATASET *>(d); }
SCRATCH_AREA *S(scratch_space *s) { return reinterpret_cast<SCRATCH_AREA *>(s); }
void block_sizes(const CNN_MODEL *m, int l, int *a, int *g) {
    if (l < m->cLayers) {
        const CONV_LAYER &c = m->convLayer[l];
        *a = c.inChannels * c.kSize * c.kSize + (m->bias ? 1 : 0);
        *g = c.outChannels;
    } else {
        const FC_LAYER &f = m->fcLayer[l - m->cLayers];
        *a = f.in + (m->bias ? 1 : 0);
        *g = f.out;
    }
}
void fill_info(const CNN_MODEL *m, const kfac_curvature *k, FITRE_KFAC_INFO *info) {
    die(fitre_kfac_storage_indices(m, info), "computeKFACStorageIndices");
    info->regLambda = k->regLambda;
    info->dampGamma = k->dampGamma;
    info->stats_decay = k->stats_decay;
    info->momentum = k->momentum;
    info->checkGrad = k->checkGrad;
    info->inverseFreq = k->inverseFreq;
}

}  // namespace

// Seeds the generator behind augmentData / computeDistributionErrors (the reference seeds cuRAND
// from the clock, device/gen_random.c).  Not part of the reference's interface.
void fitreShimSeed(unsigned long long seed) { g_rng = seed; }
// The context behind the shim, e.g. to attach a communicator (fitre_comm_init) or set a mode.
fitre_context *fitreShimContext() { return ctx(); }

// functions/cnn_gradient.h:9-12
real computeCNNGradient(cnn *model, dev_dataset *data, scratch_space *scratch, real *z, real *dx, real *probs,
                        real *lossFuncErrors, real *gradient, int offset, int curBatchSize, real weightDecay) {
    real loss = 0;
    die(fitre_compute_cnn_gradient(ctx(), M(model), D(data), S(scratch), z, dx, probs, lossFuncErrors, gradient,
                                   offset, curBatchSize, weightDecay, &loss),
        "computeCNNGradient");
    return loss;
}
// functions/cnn_forward.h:9-13
long cnnForwardMemRequired(cnn *model) { return fitre_cnn_forward_mem_required(M(model)); }
real cnnForward(cnn *model, dev_dataset *data, scratch_space *scratch, real *z, real *probs, real *errors, int s,
                int curBatchSize, eval_type forTesting) {
    real loss = 0;
    die(fitre_cnn_forward(ctx(), M(model), D(data), S(scratch), z, probs, errors, s, curBatchSize, (int)forTesting,
                          &loss),
        "cnnForward");
    return loss;
}
// functions/cnn_backward.h:11-16
long cnnBackwardMemRequired(cnn *model) { return fitre_cnn_backward_mem_required(M(model)); }
void cnnBackward(cnn *model, dev_dataset *data, real *devPtr, real *z, real *gradient, real *dx, real *delta,
                 real *delta_new, int offset, int batchSize, real *hostPtr) {
    die(fitre_cnn_backward(ctx(), M(model), D(data), devPtr, z, gradient, dx, delta, delta_new, offset, batchSize,
                           hostPtr),
        "cnnBackward");
    cudaDeviceSynchronize();
}
// functions/cnn_hessian_vec.h:9-13
void cnnHv(cnn *model, dev_dataset *data, real *z, real *probs, real *lossFuncErrors, real *dx, real *vector,
           real *hv, int s, int curBatchSize, real *devPtr, real *hostPtr, real weightDecay) {
    die(fitre_cnn_hv(ctx(), M(model), D(data), z, probs, lossFuncErrors, dx, vector, hv, s, curBatchSize, devPtr,
                     hostPtr, weightDecay),
        "cnnHv");
    cudaDeviceSynchronize();
}
// functions/cnn_hv_forward.h:8-13, functions/cnn_hv_backward.h:10-15
long cnnROpForwardMemRequired(cnn *model) { return fitre_cnn_rop_forward_mem_required(M(model)); }
void cnnROpForward(cnn *model, dev_dataset *data, scratch_space *scratch, real *z, real *vector, real *rz, int s,
                   int curBatchSize, real *devPtr, real *hostPtr) {
    die(fitre_cnn_rop_forward(ctx(), M(model), D(data), S(scratch), z, vector, rz, s, curBatchSize, devPtr, hostPtr),
        "cnnROpForward");
    cudaDeviceSynchronize();
}
long cnnROpBackwardMemRequired(cnn *model) { return fitre_cnn_rop_backward_mem_required(M(model)); }
void cnnROpBackward(cnn *model, dev_dataset *data, scratch_space *scratch, real *z, real *dx, real *lossFuncErrors,
                    real *rError, real *rz, real *vector, real *hv, int s, int curBatchSize, real *devPtr,
                    real *hostPtr) {
    die(fitre_cnn_rop_backward(ctx(), M(model), D(data), S(scratch), z, dx, lossFuncErrors, rError, rz, vector, hv,
                               s, curBatchSize, devPtr, hostPtr),
        "cnnROpBackward");
    cudaDeviceSynchronize();
}
// functions/model_reduction.h
real computeQuadraticModel(cnn *model, dev_dataset *data, real *z, real *probs, real *lossFuncErrors, real *dx,
                           real *gradient, real *vector, real delta, int offset, int curBatchSize,
                           real weightDecay, real *devPtr, real *hostPtr, real *pageLckPtr) {
    real val = 0;
    die(fitre_compute_quadratic_model(ctx(), M(model), D(data), z, probs, lossFuncErrors, dx, gradient, vector,
                                      delta, offset, curBatchSize, weightDecay, devPtr, hostPtr, pageLckPtr, &val),
        "computeQuadraticModel");
    return val;
}
// functions/cnn_eval_model.h, functions/cnn_accuracy.h
real evaluateCNNModel(cnn *model, dev_dataset *data, scratch_space *scratch, real *z, real *probs,
                      real *lossFuncErrors, int offset, int curBatchSize) {
    real loss = 0;
    die(fitre_evaluate_cnn_model(ctx(), M(model), D(data), S(scratch), z, probs, lossFuncErrors, offset,
                                 curBatchSize, &loss),
        "evaluateCNNModel");
    return loss;
}
real computeAccuracy(real *probs, real *target, int rows, int numClasses, real *devPtr, real *pageLckPtr) {
    (void)devPtr;
    real hits = 0, acc = 0;
    die(fitre_compute_accuracy(ctx(), probs, target, rows, numClasses, &hits, &acc), "computeAccuracy");
    if (pageLckPtr) *pageLckPtr = hits;  // callers read the hit count here (functions/cnn_accuracy.cu:55-58,99)
    return acc;
}
void computeTestGeneralizationErrors(cnn *model, dev_dataset *data, scratch_space *scratch, real *z, real *probs,
                                     real *errors, real *likelihood, real *accuracy) {
    die(fitre_compute_generalization_errors(ctx(), M(model), D(data), S(scratch), z, probs, errors,
                                            FITRE_MODEL_TEST_ACCURACY, likelihood, accuracy),
        "computeTestGeneralizationErrors");
}
void computeTrainGeneralizationErrors(cnn *model, dev_dataset *data, host_dataset *host, scratch_space *scratch,
                                      real *z, real *probs, real *errors, real *likelihood, real *accuracy) {
    (void)host;  // host-resident (IMAGENET) training sets are outside this path
    die(fitre_compute_generalization_errors(ctx(), M(model), D(data), S(scratch), z, probs, errors,
                                            FITRE_MODEL_TRAIN_ACCURACY, likelihood, accuracy),
        "computeTrainGeneralizationErrors");
}
// solvers/kfac_trust_region.cu:66-77
void initBatchNormData(cnn *model, real *z, int *zOffsets) {
    (void)zOffsets;
    die(fitre_init_batch_norm_data(ctx(), M(model), z), "initBatchNormData");
    cudaDeviceSynchronize();
}
// utilities/sample_matrix.h, solvers/kfac_da.h
void selectColumnMatrix(dev_dataset *data, int sampleSize, int *indices, int offset) {
    die(fitre_select_column_matrix(ctx(), D(data), sampleSize, indices, offset), "selectColumnMatrix");
    cudaDeviceSynchronize();
}
void augmentData(cnn *model, dev_dataset *data, int offset, int currentBatchSize, real *devPtr, real *hostPtr,
                 int enableDA, dataset_type datasetType) {
    (void)offset;
    (void)hostPtr;
    DEVICE_DATASET *d = D(data);
    d->datasetType = (int)datasetType;
    const real *u = nullptr;
    if (enableDA >= 1) {
        upload_uniforms(devPtr, 3L * currentBatchSize);
        u = devPtr;
    }
    // the gathered images sit in the first half of sampledTrainX; the assembled batch goes to the second
    die(fitre_prepare_minibatch(ctx(), M(model), d, d->sampledTrainX, d->sampledTrainY, nullptr, 0, currentBatchSize, u),
        "augmentData");
    cudaDeviceSynchronize();
}
// functions/softmax_loss.h:6-7
void computeDistributionErrors(real *probs, real *distTarget, real *distError, int rows, int num_classes,
                               real *devPtr, real *hostPtr) {
    (void)hostPtr;
    upload_uniforms(devPtr, rows);
    die(fitre_compute_distribution_errors(ctx(), probs, devPtr, distTarget, distError, rows, num_classes),
        "computeDistributionErrors");
    cudaDeviceSynchronize();
}
// solvers/kfac_utils.h, solvers/kfac_inverses.h:28-36, solvers/kfac_natural_gradient.h
void computeKFACStorageIndices(cnn *model, kfac_curvature *kfacInfo) {
    FITRE_KFAC_INFO info{};
    die(fitre_kfac_storage_indices(M(model), &info), "computeKFACStorageIndices");
    for (int i = 0; i < FITRE_MAX_LAYERS; ++i) {
        kfacInfo->OmegaZOffsets[i] = info.OmegaZOffsets[i];
        kfacInfo->LambdaGOffsets[i] = info.LambdaGOffsets[i];
    }
}
void computeOmegaZ(kfac_curvature *kfac_info, cnn *model, dev_dataset *data, int samples, real *dampedInput,
                   real *dampedZ, real *omegaZInv, int *zOffsets, int *zztOffsets, real *devPtr, real *pageLckPtr,
                   cublasContext *blasHandle, CUstream_st *curStream, cusolverDnContext *curHandle) {
    (void)zOffsets; (void)zztOffsets; (void)pageLckPtr; (void)blasHandle; (void)curStream; (void)curHandle;
    if (!dampedZ || (!data && !dampedInput)) {
        fprintf(stderr, "fitre shim: computeOmegaZ needs the batch and z, or dampedInput and dampedZ\n");
        exit(-1);
    }
    const CNN_MODEL *m = M(model);
    FITRE_KFAC_INFO info{};
    fill_info(m, kfac_info, &info);
    // factors into the head of the scratch, inverses block by block behind them
    real *A = devPtr, *work = devPtr + ((info.OmegaZSize + 31) / 32) * 32;
    if (dampedInput)  // running averages (solvers/kfac_inverses.cu:479-489)
        die(fitre_kfac_omega_z_damped(ctx(), m, dampedInput, dampedZ, samples, A, &info, work), "computeOmegaZ");
    else
        die(fitre_kfac_omega_z(ctx(), m, D(data), dampedZ, samples, A, &info, work), "computeOmegaZ");
    for (int l = 0; l < m->cLayers + m->lLayers; ++l) {
        int a, g;
        block_sizes(m, l, &a, &g);
        // the A slots hold what computeNaturalGradient expects under the context's solver setting
        if (fitre_get_kfac_solver(ctx()) == FITRE_KFAC_SOLVER_CHOLESKY)
            die(fitre_kfac_matrix_factor(ctx(), A + info.OmegaZOffsets[l], omegaZInv + info.OmegaZOffsets[l], a,
                                         info.regLambda, info.dampGamma),
                "computeOmegaZ (factor)");
        else
            die(fitre_kfac_matrix_inverse(ctx(), A + info.OmegaZOffsets[l], omegaZInv + info.OmegaZOffsets[l], a,
                                          work, info.regLambda, info.dampGamma),
                "computeOmegaZ (inverse)");
    }
    cudaDeviceSynchronize();
}
void computeLambdaDelta(kfac_curvature *kfac_info, cnn *model, int samples, real *dx, real *dampedLambda,
                        real *lambdaGInv, int *zOffsets, int *zztOffsets, real *devPtr, real *pageLckPtr,
                        cublasContext *blasHandle, CUstream_st *curStream, cusolverDnContext *curHandle) {
    (void)zOffsets; (void)zztOffsets; (void)pageLckPtr; (void)blasHandle; (void)curStream; (void)curHandle;
    if (!dx && !dampedLambda) {
        fprintf(stderr, "fitre shim: computeLambdaDelta needs dx or dampedLambda\n");
        exit(-1);
    }
    const CNN_MODEL *m = M(model);
    FITRE_KFAC_INFO info{};
    fill_info(m, kfac_info, &info);
    real *G = devPtr, *work = devPtr + ((info.LambdaGSize + 31) / 32) * 32;
    if (dampedLambda)
        die(fitre_kfac_lambda_delta_damped(ctx(), m, dampedLambda, samples, G, &info, work), "computeLambdaDelta");
    else
        die(fitre_kfac_lambda_delta(ctx(), m, dx, samples, G, &info, work), "computeLambdaDelta");
    for (int l = 0; l < m->cLayers + m->lLayers; ++l) {
        int a, g;
        block_sizes(m, l, &a, &g);
        die(fitre_kfac_matrix_inverse(ctx(), G + info.LambdaGOffsets[l], lambdaGInv + info.LambdaGOffsets[l], g, work,
                                      info.regLambda, info.dampGamma),
            "computeLambdaDelta (inverse)");
    }
    cudaDeviceSynchronize();
}
// solvers/kfac_inverses.h: the running-average variant
void updateRunningStats(real *src, real *update, int numElements, real momentum) {
    die(fitre_update_running_stats(ctx(), src, update, numElements, momentum), "updateRunningStats");
    cudaDeviceSynchronize();
}
void computeSpeedUpOmegaZ(kfac_curvature *kfac_info, cnn *model, dev_dataset *data, int samples, real *z,
                          int *zOffsets, real *dampedInput, real *dampedZ, int *zztOffsets, int iterCount) {
    (void)zOffsets; (void)zztOffsets;
    const CNN_MODEL *m = M(model);
    FITRE_KFAC_INFO info{};
    fill_info(m, kfac_info, &info);
    die(fitre_kfac_speedup_omega_z(ctx(), &info, m, D(data), samples, z, dampedInput, dampedZ, iterCount),
        "computeSpeedUpOmegaZ");
    cudaDeviceSynchronize();
}
void computeSpeedUpLambdaDelta(kfac_curvature *kfac_info, cnn *model, int samples, real *dx, real *dampedLambda,
                               int *zOffsets, int *zztOffsets, int iterCount) {
    (void)zOffsets; (void)zztOffsets;
    const CNN_MODEL *m = M(model);
    FITRE_KFAC_INFO info{};
    fill_info(m, kfac_info, &info);
    die(fitre_kfac_speedup_lambda_delta(ctx(), &info, m, samples, dx, dampedLambda, iterCount),
        "computeSpeedUpLambdaDelta");
    cudaDeviceSynchronize();
}
void computeNaturalGradient(cnn *model, kfac_curvature *kfacInfo, real *devPtr, real *hostPtr) {
    (void)hostPtr;
    const CNN_MODEL *m = M(model);
    FITRE_KFAC_INFO info{};
    fill_info(m, kfacInfo, &info);
    die(fitre_compute_natural_gradient(ctx(), m, &info, kfacInfo->OmegaZInv, kfacInfo->LambdaGInv,
                                       kfacInfo->gradient, kfacInfo->nGradient, devPtr),
        "computeNaturalGradient");
    cudaDeviceSynchronize();
}
