/*
 * fitre_b200.h -- C ABI of the B200-native FITRE hot path.
 *
 * The library accelerates one path of kylasa/FITRE: the CNN gradient
 * (forward + backward), the exact Hessian-vector product by Pearlmutter's
 * R-operator, the one-direction quadratic model, Steihaug-CG driven by that
 * Hessian-vector product, and KFAC factor accumulation.  Every entry point is
 * `extern "C"`, takes plain pointers and sizes, and returns an `int` status
 * (FITRE_OK == 0).  `real` is `double` (reference: core/datadefs.h:5).
 *
 * All `real *` arguments are DEVICE pointers unless the name ends in `_host`
 * or the comment says otherwise.  The caller owns every buffer; the library
 * never frees or keeps them.  Calls are stream-ordered on the context's
 * stream; entry points that return a scalar synchronise that stream.
 *
 * The model / dataset / scratch structs below are field-for-field compatible
 * with the reference's (nn/nn_decl.h:64-155, core/structdefs.h:25-83) so a
 * reference driver can hand its own structs to this library.
 */
#ifndef FITRE_B200_H
#define FITRE_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef double real;

#define FITRE_MAX_LAYERS 20 /* reference: nn/nn_decl.h:4 */

/* ---- enum values (binary compatible with nn/nn_decl.h:13-101) ---------- */
enum { FITRE_NET_LENET = 0, FITRE_NET_ALEXNET = 1, FITRE_NET_VGG11 = 2 };
enum { FITRE_NO_BATCH_NORM = 0, FITRE_BATCH_NORM = 10, FITRE_BATCH_NORM_TRAINABLE = 20 };
enum { FITRE_MODEL_TRAIN = 10, FITRE_MODEL_TRAIN_ACCURACY = 20, FITRE_MODEL_TEST_ACCURACY = 30 };
enum { FITRE_ACT_LOGISTIC = 1, FITRE_ACT_TANH = 2, FITRE_ACT_LINEAR = 3 }; /* FC layers */
enum {
    FITRE_CNN_ACT_NONE = 10,
    FITRE_CNN_ACT_SOFTPLUS = 11,
    FITRE_CNN_ACT_ELU = 12,
    FITRE_CNN_ACT_RELU = 13,
    FITRE_CNN_ACT_SWISH = 14
};
enum { FITRE_MAX_POOL = 0, FITRE_AVG_POOL = 1, FITRE_NO_POOL = 2 };
enum { FITRE_TRUE_HESSIAN = 0, FITRE_GAUSS_NEWTON = 1 }; /* solvers/params.h:6-9 */

/* ---- status codes ------------------------------------------------------ */
enum {
    FITRE_OK = 0,
    FITRE_ERR_BAD_ARG = 1,       /* NULL pointer, negative size, batch mismatch */
    FITRE_ERR_UNSUPPORTED = 2,   /* layer / activation / pool geometry outside the path */
    FITRE_ERR_WORKSPACE = 3,     /* scratch smaller than the *_mem_required figure */
    FITRE_ERR_CUDA = 4,          /* a CUDA runtime call or launch failed */
    FITRE_ERR_COMM = 5,          /* NCCL error or time-out */
    FITRE_ERR_NOT_CONVERGED = 6, /* solver hit its iteration limit (informational) */
    FITRE_ERR_TOO_LARGE = 7,     /* size beyond a fixed built-in limit */
    FITRE_ERR_NOT_FINITE = 8     /* the loss came out NaN or Inf (non-finite inputs or weights); the
                                  * outputs are written as computed, the reference would carry on */
};

/* ---- boundary structs (reference layouts) ------------------------------ */
typedef struct fitre_conv_layer { /* nn/nn_decl.h:64-95 */
    int inChannels, outChannels;
    int width, height, outWidth, outHeight;
    int kSize, stride, padding;
    int activationOffset, poolOffset, batchNormOffset, outputOffset;
    int batchNorm; /* FITRE_NO_BATCH_NORM | FITRE_BATCH_NORM */
    int meansOffset, variancesOffset;
    int runningMeansOffset, runningVariancesOffset;
    int convVolumn, activationVolumn, poolVolumn, batchNormVolumn;
} CONV_LAYER;

typedef struct fitre_pool_layer { /* nn/nn_decl.h:103-113 */
    int height, width, outHeight, outWidth;
    int type; /* FITRE_MAX_POOL | FITRE_AVG_POOL | FITRE_NO_POOL */
    int pSize, padding, stride;
} POOL_LAYER;

typedef struct fitre_fc_layer { /* nn/nn_decl.h:115-121 */
    int in, out, actFun, batchNorm;
    int offset; /* out * batchSize: where the pre-activation copy lives */
} FC_LAYER;

typedef struct fitre_cnn_model { /* nn/nn_decl.h:123-155 */
    CONV_LAYER convLayer[FITRE_MAX_LAYERS];
    int actFuns[FITRE_MAX_LAYERS];
    POOL_LAYER poolLayer[FITRE_MAX_LAYERS];
    int cLayers;
    int lLayers;
    FC_LAYER fcLayer[FITRE_MAX_LAYERS];
    int bias, pSize, zSize, batchSize, maxDeltaSize, name, enableBatchNorm;
    int wOffsets[FITRE_MAX_LAYERS];
    int bOffsets[FITRE_MAX_LAYERS];
    int zOffsets[FITRE_MAX_LAYERS];
    int zztSize;
    int zztOffsets[FITRE_MAX_LAYERS];
    int rZOffsets[FITRE_MAX_LAYERS];
} CNN_MODEL;

typedef struct fitre_scratch_area { /* core/structdefs.h:25-33 */
    real *hostWorkspace, *devWorkspace, *pageLckWorkspace;
    real *nextDevPtr, *nextHostPtr, *nextPageLckPtr;
} SCRATCH_AREA;

typedef struct fitre_sparse_dataset { /* core/sparsedefs.h:17-29, opaque to this path */
    int *rowPtr, *colPtr, *rowCsrPtr;
    real *valPtr;
    int nnz;
    real *sortedVals;
    int *P;
    void *descr;
} FITRE_SPARSE_DATASET;

typedef struct fitre_device_dataset { /* core/structdefs.h:55-83 */
    real *trainSetX, *trainSetY, *testSetX, *testSetY;
    real *weights; /* flat parameter vector, pSize doubles */
    int numClasses;
    int datasetType;
    int features, height, width;
    int testSizeX, testSizeY, trainSizeX, trainSizeY;
    int sampleSize;
    real *sampledTrainX;
    real *sampledTrainY; /* labels of the current batch: doubles in 1..numClasses */
    real *currentBatch;  /* [Cin][N][W][H], h fastest */
    FITRE_SPARSE_DATASET spSamplingMatrix;
} DEVICE_DATASET;

/* KFAC block offsets (reference: solvers/kfac_structs.h:12-48, the fields this path uses). */
typedef struct fitre_kfac_info {
    int OmegaZOffsets[FITRE_MAX_LAYERS];     /* A-factor block start per layer (doubles) */
    int LambdaGOffsets[FITRE_MAX_LAYERS];    /* G-factor block start per layer (doubles) */
    int OmegaZSize, LambdaGSize;
    real regLambda, dampGamma;
    /* knobs of the training loop (same names as the reference's struct) */
    real stats_decay, momentum;
    int checkGrad;   /* 1: also evaluate the quadratic model along the gradient and take the better */
    int inverseFreq; /* factors are refreshed and inverted every inverseFreq minibatches (<= 1: every one) */
} FITRE_KFAC_INFO;

/* solvers/params.h:11-33, field for field. */
typedef struct fitre_trust_region_params {
    real delta, minDelta, maxDelta;
    real eta1, eta2, gamma1, gamma2;
    unsigned long int maxProps;
    int maxMatVecs, maxEpochs, maxIters;
    int hessianType;
    real alpha;
    int curIteration;
    real hs;
    real lambda;
} TRUST_REGION_PARAMS;

/* What fitre_subsampled_trust_region_kfac records per minibatch / per epoch (caller-owned
 * arrays; the reference prints these values to stderr). */
typedef struct fitre_tr_step {
    real trainLikelihood;    /* loss of the minibatch before the step */
    real newTrainLikelihood; /* loss after the step (batch statistics) */
    real newTrainAccuracy;   /* percent, after the step */
    real modelKfac, modelGradient; /* quadratic-model values of the two directions */
    real rho, delta;         /* reduction ratio; radius after the update */
    int usedKfac, reverted;
} FITRE_TR_STEP;
typedef struct fitre_tr_epoch {
    real testLikelihood, testAccuracy, trainLikelihood, trainAccuracy;
    real seconds; /* wall time of the minibatch sweep (without the two evaluation sweeps) */
    int miniBatches;
} FITRE_TR_EPOCH;

/* Steihaug-CG parameters and results (reference: solvers/cg_steihaug.h:10-35). */
enum {
    FITRE_CG_CONVERGED = 0,     /* residual below tolerance */
    FITRE_CG_NEG_CURVATURE = 1, /* d'Hd <= 0, stepped to the boundary */
    FITRE_CG_HIT_BOUNDARY = 2,  /* iterate left the trust region */
    FITRE_CG_MAX_ITERS = 3
};
typedef struct fitre_cg_params {
    real delta;     /* trust-region radius */
    real tolerance; /* stop when ||r||^2 < tolerance */
    int maxIterations;
    real weightDecay; /* H + weightDecay * I */
    /* results */
    int iterations;
    int flag;
    real modelValue; /* 0.5 p'Hp + p'g (+ 0.5 weightDecay p'p) */
    int hvCalls;
} FITRE_CG_PARAMS;

typedef struct fitre_context fitre_context; /* one per GPU / host thread */

/* ---- context ------------------------------------------------------------ */
/* Create a context on CUDA device `device`.  `stream` is a cudaStream_t (NULL = the
 * legacy default stream).  Replaces the reference's global handles and BLOCK_SIZE
 * globals (device/handles.h:15-20, drivers/main_driver.c:52-60).  Does not reset the
 * device and grabs no workspace (contrast device/cuda_environment.c:33,48-66). */
int fitre_context_create(fitre_context **ctx, int device, void *stream);
int fitre_context_destroy(fitre_context *ctx);
/* Last error text of this context (host string, valid until the next call). */
const char *fitre_last_error(const fitre_context *ctx);
/* Number of kernels of this library launched through `ctx` since creation. */
long long fitre_launch_count(const fitre_context *ctx);
/* 1 = replicate the reference's softmax quirks (max-shift starts at 0 and
 * probs += 1e-10: functions/softmax_loss.cu:24-27,55); 0 = textbook softmax. Default 1. */
int fitre_set_reference_softmax(fitre_context *ctx, int on);
/* Term that fitre_compute_quadratic_model adds to the Hessian-vector product when weightDecay
 * is non-zero: 1 (default) = weightDecay * data->weights, as the C reference does
 * (functions/model_reduction.cu:50-52); 0 = weightDecay * vector, the curvature of the L2 term,
 * as the reference's PyTorch twin does (pytorch/peng/utils.py:77).  The trust-region loop
 * (fitre_subsampled_trust_region_kfac) follows the setting. */
int fitre_set_reference_quadratic_damping(fitre_context *ctx, int on);
/* Declares how many doubles are available behind the scratch pointer handed to the calls that
 * follow (SCRATCH_AREA.nextDevPtr, devPtr): a call that needs more, by the matching
 * *_mem_required figure, returns FITRE_ERR_WORKSPACE before launching anything.  0 (default) =
 * unknown, no check, as in the reference, whose callers carve the workspace by pointer arithmetic
 * without passing sizes (drivers/cnn_driver.cu:193-209). */
int fitre_set_scratch_limit(fitre_context *ctx, long doubles);
/* Number of launches the host has issued through `ctx` of the kernel called `name` (the
 * __global__ function's name without template arguments, e.g. "conv_tma_kernel"); launches
 * replayed from a captured CUDA graph are counted once, at capture.  -1 on a NULL argument.
 * Lets a caller or a test see which kernel variant a shape was routed to.  No counterpart in
 * the reference. */
long long fitre_kernel_launches(const fitre_context *ctx, const char *name);

/* Arithmetic of the convolution products: forward, data gradient, weight gradient and their
 * R-operator forms.  FITRE_PRECISION_FP64 (default) is the reference's arithmetic.  The two other
 * values are opt-in reduced-precision modes on the tcgen05 tensor cores with fp32 accumulation in
 * tensor memory; batch norm, activations, pooling, FC layers and all stored tensors stay fp64.
 *   FITRE_PRECISION_TF32X3: every operand is split into a TF32 head and tail and each product is
 *     three tensor-core products (lo*hi + hi*lo + hi*hi), about 22 mantissa bits.  Stated
 *     tolerance of loss, gradient and Hessian-vector product against the fp64 result, relative
 *     and norm-wise: 1e-3 wherever the routing of max pooling is the fp64 run's (nets without max
 *     pooling; small batches; backward and R passes run in this mode on a forward state computed
 *     in fp64) -- measured 2e-5 / 6e-5 on VGG-11-BN at 512 images; 1e-2 when this mode's own
 *     forward pass decides the routing of a max-pooling net at batch sizes in the hundreds:
 *     at 512 images 25 of 16 million pooling windows are near enough to a tie to flip, each flip
 *     re-routes an error path, and gradient / Hessian-vector product move by 3e-3 / 5e-3.
 *   FITRE_PRECISION_TF32: one product on TF32-rounded operands.  Each convolution is within 5e-4
 *     relative of fp64 and the loss within 1e-3, but batch normalisation and the backward sweep
 *     amplify the rounding: gradients and Hessian-vector products of deep nets are only within
 *     1e-1 relative (measured 3e-2 / 5e-2 on VGG-11-BN), so this mode does not meet 1e-3.
 *   FITRE_PRECISION_FP64_I8: fp64-class results from the integer tensor cores: operands in fixed
 *     point (power-of-two scale per channel), six signed base-128 digits each, the digit
 *     products summed exactly in int32 (tcgen05.mma.kind::i8) and recombined in fp64; terms below
 *     128^-7 of full scale are dropped.  Stated tolerance against the fp64 result: 1e-10
 *     relative, the same as the default mode's against the reference.
 * Shapes the tensor-core kernels do not cover (the 3-channel first layer, odd input heights, ...)
 * use the fp64 kernels in every mode.  No counterpart in the reference (fp64 only). */
enum { FITRE_PRECISION_FP64 = 0, FITRE_PRECISION_TF32 = 1, FITRE_PRECISION_TF32X3 = 2, FITRE_PRECISION_FP64_I8 = 3 };
int fitre_set_precision(fitre_context *ctx, int precision);

/* How the KFAC A-factor blocks are applied (the G blocks, at most a few hundred rows, are always
 * inverted):
 *   FITRE_KFAC_SOLVER_INVERSE (default): fitre_kfac_invert_factors writes the explicit inverses
 *     (F + (lambda+gamma) I)^-1, as computeMatrixInverseCusolver does
 *     (solvers/kfac_inverses.cu:133-186), and fitre_compute_natural_gradient multiplies by them.
 *   FITRE_KFAC_SOLVER_CHOLESKY: fitre_kfac_invert_factors writes into the same slots the Cholesky
 *     factor L of each damped A block (lower triangle; the upper triangles of the 64 x 64
 *     diagonal blocks hold those blocks' inverses) and fitre_compute_natural_gradient applies
 *     A^-1 = L^-T L^-1 to G^-1 [W|b] by two triangular solves.  One third of the factorisation
 *     work and no triangular inversion or L^-T L^-1 product; the natural gradient agrees with the
 *     explicit-inverse form to rounding (about cond(A) * 1e-16 relative).  The slots are then
 *     only meaningful to these two calls.  fitre_subsampled_trust_region_kfac follows the
 *     setting.  No counterpart in the reference. */
enum { FITRE_KFAC_SOLVER_INVERSE = 0, FITRE_KFAC_SOLVER_CHOLESKY = 1 };
int fitre_set_kfac_solver(fitre_context *ctx, int solver);
int fitre_get_kfac_solver(const fitre_context *ctx); /* the current setting; -1 without a context */

/* Where the KFAC factors live when the context has a communicator (no effect on one GPU):
 *   FITRE_KFAC_REPLICATED (default): every rank ends up with all global factors and all inverses
 *     (factor blocks all-reduced, the factorisations divided among the ranks and exchanged).
 *   FITRE_KFAC_LAYER_OWNED: every layer has an owner rank (most expensive layer first onto the
 *     least loaded rank).  fitre_kfac_factors_and_inverses reduces each factor block onto its
 *     owner only, which factorises it; nothing is sent back, so omegaZ / lambdaG and the inverse
 *     slots of a layer are valid on its owner alone.  fitre_compute_natural_gradient forms each
 *     layer's slice on the owner and one all-reduce of nGradient (pSize doubles) completes the
 *     vector on every rank: the 2 x OmegaZSize doubles of factor traffic per step become about
 *     half of one, and the natural-gradient work is divided as well.  Set it before both calls;
 *     fitre_subsampled_trust_region_kfac uses it by itself.  The reference is single-GPU; its
 *     dormant second-GPU thread (solvers/kfac_thread.cu:77-204) is the nearest counterpart. */
enum { FITRE_KFAC_REPLICATED = 0, FITRE_KFAC_LAYER_OWNED = 1 };
int fitre_set_kfac_distribution(fitre_context *ctx, int mode);

/* 1 (default) = calls whose launch sequence is fixed by the model and the buffers capture it
 * into a CUDA graph on first use and replay it while the model description, pointers, sizes,
 * damping and solver stay the same; 0 = launch kernel by kernel.  Covered: the KFAC factor,
 * factorisation and natural-gradient calls (a thousand small dependent kernels), and on one GPU
 * fitre_compute_cnn_gradient and fitre_cnn_hv (the last two gradient and the last four Hv
 * argument sets are kept, so a CG loop alternating between two direction buffers replays).
 * With a communicator the gradient and Hv passes launch directly, because their slices are
 * all-reduced from a second stream under the sweep.  Same kernels and results either way.  No
 * counterpart in the reference. */
int fitre_set_graphs(fitre_context *ctx, int on);

/* 1 (default) = use the TMA-fed convolution kernels wherever shape and alignment allow;
 * 0 = always use the gather kernels (same results; kept for comparison and as the path
 * for odd shapes).  No counterpart in the reference. */
int fitre_set_tma(fitre_context *ctx, int on);

/* Optional per-kernel timing.  While enabled, every launch of the two convolution kernel
 * classes (0 = implicit-GEMM forward / data-gradient kernel, 1 = weight-gradient kernel) is
 * bracketed by CUDA events on the context's stream.  fitre_profile_read synchronises the
 * stream, returns the summed device time (ms), algorithmic flops (2*M*K*Cout per product)
 * and launch count of one class since the last read, and clears them.  No counterpart in
 * the reference (its timers are gettimeofday around whole phases, utilities/utils.c:16-33). */
int fitre_profile_enable(fitre_context *ctx, int on);
int fitre_profile_read(fitre_context *ctx, int kind, double *ms, double *flops, long *launches);

/* Data-parallel set-up: `unique_id` is the 128-byte ncclUniqueId obtained on rank 0
 * (fitre_comm_unique_id) and broadcast by the caller.  After this call every batch
 * statistic (loss, batch-norm sums, gradient, Hv, KFAC factors, dot products) is
 * all-reduced over `world` ranks and 1/N uses the global batch world*curBatchSize.
 * No counterpart in the reference (single GPU). */
int fitre_comm_unique_id(void *unique_id_128_host);
int fitre_comm_init(fitre_context *ctx, const void *unique_id_128_host, int rank, int world);
int fitre_comm_world(const fitre_context *ctx);
/* Failure handling of the data-parallel mode, all on the host.  `seconds` (default 300) bounds
 * (1) fitre_comm_init: the communicator is created on a helper thread and a peer that never
 * joins yields FITRE_ERR_COMM after that time instead of a hang; (2) every host wait on the
 * context's stream while a communicator exists: the wait polls the stream together with
 * ncclCommGetAsyncError, and on a reported error or when the time runs out the communicator is
 * aborted (ncclCommAbort stops NCCL's device work; the CUDA context and the fitre context stay
 * usable) and the call returns FITRE_ERR_COMM.  After that every collective fails fast with
 * FITRE_ERR_COMM until fitre_comm_init is called again (world 1 returns to single-GPU mode).
 * The environment variable FITRE_NCCL_LIBRARY names the NCCL library to load instead of
 * libnccl.so.2.  The reference has no counterpart: every failure there is print + exit
 * (device/cuda_utils.h:28-92). */
int fitre_set_comm_timeout(fitre_context *ctx, double seconds);
/* Short vectors that the data-parallel passes exchange on their critical path (batch-norm
 * statistics, about forty per step, and the loss) do not go through NCCL when the ranks share a
 * node: every rank maps every other rank's mailbox (CUDA IPC, set up by fitre_comm_init) and one
 * kernel -- the same launch that finishes the per-channel sums -- stores this rank's vector into all
 * mailboxes, waits for the peers' flags in its own and adds the rows in rank order, so all ranks
 * hold the same bits.  fitre_peer_reduce_enabled tells whether that path is up (it is all-or-nothing
 * over the ranks; FITRE_PEER_REDUCE=0 in the environment, more than 8 ranks or a failed IPC mapping
 * leave these vectors to NCCL).  The kernel's wait is bounded (the smaller of the communicator
 * time-out and 30 s); when it runs out the call returns FITRE_ERR_COMM through the device error
 * word.  fitre_peer_wait_selftest runs that kernel on ONE GPU against a two-rank mailbox whose
 * second flag nothing raises and returns FITRE_ERR_COMM after about wait_ms: the host-visible
 * proof that a lost peer ends in a status.  No counterpart in the reference. */
int fitre_peer_reduce_enabled(const fitre_context *ctx);
int fitre_peer_wait_selftest(fitre_context *ctx, double wait_ms);

/* ---- model builders (nn/read_nn.c:500-725, nn/read_alexnet.c:14-243,
 *      nn/read_vgg.c:25-120,122-212,216-299, nn/utils.c:19-172) ---------- */
/* `actFun` overrides the builders' Swish (pass FITRE_CNN_ACT_SWISH to keep it);
 * `poolType` overrides LeNet's average pooling (FITRE_AVG_POOL to keep it). */
int fitre_read_lenet_cnn(CNN_MODEL *m, int channels, int width, int height, int batchSize,
                         int enableBias, int enableBatchNorm, int actFun, int poolType);
int fitre_read_alexnet_cnn(CNN_MODEL *m, int batchSize, int height, int width, int numClasses,
                           int enableBias, int enableBatchNorm, int actFun);
int fitre_read_vgg11(CNN_MODEL *m, int batchSize, int height, int width, int numClasses,
                     int inChannels, int enableBias, int enableBatchNorm, int actFun);
int fitre_read_test_vgg(CNN_MODEL *m, int batchSize, int height, int width, int numClasses,
                        int inChannels, int enableBias, int batchNorm, int actFun);
/* Generic: the caller fills cLayers/lLayers, per conv layer {inChannels,outChannels,height,
 * width,kSize,stride,padding,batchNorm}, actFuns[], per pool layer {type,pSize,stride,padding},
 * per FC layer {in,out,actFun}, bias and batchSize; this fills every derived field
 * (output sizes, offsets, volumes, pSize, zSize, maxDeltaSize) with the layout of
 * nn/read_vgg.c:63-101 and nn/utils.c:44-172. */
int fitre_model_finalize(CNN_MODEL *m);
/* Checks that the model is inside the supported path (stride-1 square convs, pooling with
 * ksize - stride == padding, square planes at the conv->FC boundary, known activations). */
int fitre_model_validate(const CNN_MODEL *m);

/* ---- scratch sizing: element counts of `real` (functions/cnn_forward.cu:16,
 *      cnn_backward.cu:51, cnn_hv_forward.cu:15, cnn_hv_backward.cu:24) --- */
long fitre_cnn_forward_mem_required(const CNN_MODEL *m);
long fitre_cnn_backward_mem_required(const CNN_MODEL *m);
long fitre_cnn_rop_forward_mem_required(const CNN_MODEL *m);
long fitre_cnn_rop_backward_mem_required(const CNN_MODEL *m);
/* Scratch needed behind scratch->nextDevPtr by fitre_compute_cnn_gradient (two delta
 * buffers + forward/backward scratch) and behind devPtr by fitre_cnn_hv (rz + rError + scratch). */
long fitre_cnn_gradient_mem_required(const CNN_MODEL *m);
long fitre_cnn_hv_mem_required(const CNN_MODEL *m);

/* ---- the hot path --------------------------------------------------------- */
/* functions/cnn_forward.h:11-13.  Writes every intermediate to `z`, the class
 * probabilities to `probs`, (p - onehot)/N to `errors`, and the mean loss to *loss_host. */
int fitre_cnn_forward(fitre_context *ctx, const CNN_MODEL *m, const DEVICE_DATASET *data,
                      SCRATCH_AREA *scratch, real *z, real *probs, real *errors, int s,
                      int curBatchSize, int evalType, real *loss_host);
/* functions/cnn_backward.h:13-16.  `delta` holds the loss errors on entry and is destroyed. */
int fitre_cnn_backward(fitre_context *ctx, const CNN_MODEL *m, const DEVICE_DATASET *data,
                       real *devPtr, real *z, real *gradient, real *dx, real *delta,
                       real *delta_new, int offset, int batchSize, real *hostPtr);
/* functions/cnn_gradient.h:9-12.  loss -> *loss_host, gradient (+ weightDecay*w) -> gradient. */
int fitre_compute_cnn_gradient(fitre_context *ctx, const CNN_MODEL *m, const DEVICE_DATASET *data,
                               SCRATCH_AREA *scratch, real *z, real *dx, real *probs,
                               real *lossFuncErrors, real *gradient, int offset, int curBatchSize,
                               real weightDecay, real *loss_host);
/* functions/cnn_hv_forward.h:10-13 */
int fitre_cnn_rop_forward(fitre_context *ctx, const CNN_MODEL *m, const DEVICE_DATASET *data,
                          SCRATCH_AREA *scratch, real *z, real *vector, real *rz, int s,
                          int curBatchSize, real *devPtr, real *hostPtr);
/* functions/cnn_hv_backward.h:12-15 */
int fitre_cnn_rop_backward(fitre_context *ctx, const CNN_MODEL *m, const DEVICE_DATASET *data,
                           SCRATCH_AREA *scratch, real *z, real *dx, real *lossFuncErrors,
                           real *rError, real *rz, real *vector, real *hv, int s,
                           int curBatchSize, real *devPtr, real *hostPtr);
/* functions/cnn_hessian_vec.h:9-13.  Uses z/probs/lossFuncErrors/dx left by the gradient on
 * the same batch.  weightDecay is accepted and unused, as in the reference. */
int fitre_cnn_hv(fitre_context *ctx, const CNN_MODEL *m, const DEVICE_DATASET *data, real *z,
                 real *probs, real *lossFuncErrors, real *dx, real *vector, real *hv, int s,
                 int curBatchSize, real *devPtr, real *hostPtr, real weightDecay);
/* functions/model_reduction.cu:20-93.  Scales `vector` in place; model value -> *m_host.
 * devPtr needs fitre_quadratic_model_mem_required doubles (one pSize vector for the Hessian-vector
 * product in front of fitre_cnn_hv_mem_required). */
long fitre_quadratic_model_mem_required(const CNN_MODEL *m);
int fitre_compute_quadratic_model(fitre_context *ctx, const CNN_MODEL *m,
                                  const DEVICE_DATASET *data, real *z, real *probs,
                                  real *lossFuncErrors, real *dx, real *gradient, real *vector,
                                  real delta, int offset, int curBatchSize, real weightDecay,
                                  real *devPtr, real *hostPtr, real *pageLckPtr, real *m_host);
/* Steihaug-CG on the trust-region subproblem min g'p + 0.5 p'Hp, ||p|| <= delta, with
 * H applied by fitre_cnn_hv (algorithm: solvers/cg_steihaug.c:28-260 and its CNN twin
 * pytorch/peng/utils.py:104-165).  `p` (pSize) receives the step.  devPtr needs
 * 4*pSize + fitre_cnn_hv_mem_required doubles. */
int fitre_cg_steihaug(fitre_context *ctx, const CNN_MODEL *m, const DEVICE_DATASET *data,
                      real *z, real *probs, real *lossFuncErrors, real *dx, real *gradient,
                      real *p, int curBatchSize, real *devPtr, FITRE_CG_PARAMS *params);

/* ---- KFAC factors (solvers/kfac_utils.cu:7-55, kfac_inverses.cu:450-630,759-857) */
int fitre_kfac_storage_indices(const CNN_MODEL *m, FITRE_KFAC_INFO *info);
/* functions/softmax_loss.cu:104-136 (computeDistributionErrors): sample one label per image from
 * `probs` by inverse CDF (functions/dev_dist_errors.cu:12-29) and form (p - onehot(label))/N for
 * the second backward pass of the KFAC step.  `uniforms` (rows doubles in [0,1), device) replaces
 * the reference's time-seeded cuRAND draw so that results are reproducible. */
int fitre_compute_distribution_errors(fitre_context *ctx, const real *probs, const real *uniforms,
                                      real *distTarget, real *distError, int rows, int numClasses);
/* Scratch (doubles) the two factor routines below need behind devPtr. */
long fitre_kfac_mem_required(const CNN_MODEL *m);
/* A factors: conv (1/N) P~'P~ with P~ = [im2col(X)/(Ho*Wo), 1]; FC (1/N) z~ z~'.  Raw
 * (undamped, uninverted) factors are written to omegaZ + OmegaZOffsets[l]. */
int fitre_kfac_omega_z(fitre_context *ctx, const CNN_MODEL *m, const DEVICE_DATASET *data,
                       const real *z, int samples, real *omegaZ, const FITRE_KFAC_INFO *info,
                       real *devPtr);
/* G factors: conv (N*Ho*Wo) d'd, FC N d d' from the stored backward errors `dx`. */
int fitre_kfac_lambda_delta(fitre_context *ctx, const CNN_MODEL *m, const real *dx, int samples,
                            real *lambdaG, const FITRE_KFAC_INFO *info, real *devPtr);

/* solvers/kfac_inverses.cu:133-186 (computeMatrixInverseCusolver): inverse = (matrix +
 * (lambda + dampGamma) I)^-1 for a symmetric positive definite n x n factor, by blocked Cholesky
 * and triangular inversion on the device.  devPtr needs fitre_kfac_inverse_mem_required(n)
 * doubles.  A non-positive pivot returns FITRE_ERR_NOT_CONVERGED (the reference exits). */
long fitre_kfac_inverse_mem_required(int n);
int fitre_kfac_matrix_inverse(fitre_context *ctx, const real *matrix, real *inverse, int n,
                              real *devPtr, real lambda, real dampGamma);
/* The Cholesky form of one block: factor <- the packed Cholesky factor of matrix + (lambda +
 * dampGamma) I (lower triangle L; the upper triangles of the 64 x 64 diagonal blocks hold those
 * blocks' inverses), what fitre_kfac_invert_factors writes into an A slot under
 * FITRE_KFAC_SOLVER_CHOLESKY.  No scratch.  For callers that invert block by block as
 * computeOmegaZ does (solvers/kfac_inverses.cu:542-544). */
int fitre_kfac_matrix_factor(fitre_context *ctx, const real *matrix, real *factor, int n, real lambda,
                             real dampGamma);
/* The running-average ("speed-up") variant, solvers/kfac_inverses.cu:106-126 (updateRunningStats:
 * theta <- m*theta + (1-m)*update in the reference's operation order, m == 0 copies), :386-447
 * (computeSpeedUpOmegaZ: averages of the batch into dampedInput and of every layer's output into
 * dampedZ at the model's zzt offsets; iterCount == 0 copies), :699-755
 * (computeSpeedUpLambdaDelta: the same for the layer errors), and the dampedInput / dampedZ /
 * dampedLambda branches of computeOmegaZ / computeLambdaDelta (factors from those averages).
 * dampedInput: features*samples doubles; dampedZ, dampedLambda: model->zztSize doubles. */
int fitre_update_running_stats(fitre_context *ctx, real *src, const real *update, long numElements,
                               real momentum);
int fitre_kfac_speedup_omega_z(fitre_context *ctx, const FITRE_KFAC_INFO *info, const CNN_MODEL *m,
                               const DEVICE_DATASET *data, int samples, const real *z,
                               real *dampedInput, real *dampedZ, int iterCount);
int fitre_kfac_speedup_lambda_delta(fitre_context *ctx, const FITRE_KFAC_INFO *info, const CNN_MODEL *m,
                                    int samples, const real *dx, real *dampedLambda, int iterCount);
int fitre_kfac_omega_z_damped(fitre_context *ctx, const CNN_MODEL *m, const real *dampedInput,
                              const real *dampedZ, int samples, real *omegaZ,
                              const FITRE_KFAC_INFO *info, real *devPtr);
int fitre_kfac_lambda_delta_damped(fitre_context *ctx, const CNN_MODEL *m, const real *dampedLambda,
                                   int samples, real *lambdaG, const FITRE_KFAC_INFO *info,
                                   real *devPtr);
/* Every damped inverse of one KFAC step in one call: omegaZInv / lambdaGInv <- the inverses of
 * all A blocks (K' x K', K' = K + bias) and G blocks of omegaZ / lambdaG at the offsets of `info`,
 * damping info->regLambda + info->dampGamma (what the reference does block by block inside
 * computeOmegaZ / computeLambdaDelta, solvers/kfac_inverses.cu:542-544,624-627,822-824,852-855).
 * The independent matrices run on several streams of the GPU and, with a communicator, are
 * divided among the ranks (largest first onto the least loaded rank) and exchanged by one sum
 * all-reduce, which replaces the reference's dormant second-GPU inverse thread
 * (solvers/kfac_thread.cu:77-204).  With FITRE_KFAC_SOLVER_CHOLESKY the A slots receive Cholesky
 * factors instead (see fitre_set_kfac_solver).  The launch sequence is replayed from a CUDA graph
 * while the arguments stay the same (fitre_set_graphs).  devPtr:
 * fitre_kfac_invert_factors_mem_required doubles. */
long fitre_kfac_invert_factors_mem_required(const CNN_MODEL *m);
int fitre_kfac_invert_factors(fitre_context *ctx, const CNN_MODEL *m, const FITRE_KFAC_INFO *info,
                              const real *omegaZ, real *omegaZInv, const real *lambdaG,
                              real *lambdaGInv, real *devPtr);
/* Factors and damped inverses of one KFAC step in one call -- what computeOmegaZ and
 * computeLambdaDelta do together in the reference, where each factor is inverted right after it
 * is formed (solvers/kfac_inverses.cu:450-630,759-857).  x0 / zbase / dbase: the batch
 * (data->currentBatch), z and the dx of the sampled-label backward pass (packed == 0), or the
 * running averages dampedInput / dampedZ / dampedLambda of the inverseFreq > 1 variant
 * (packed == 1, as fitre_kfac_omega_z_damped / fitre_kfac_lambda_delta_damped take them).  Same
 * results as fitre_kfac_omega_z + fitre_kfac_lambda_delta + fitre_kfac_invert_factors, bit for
 * bit; on one GPU the factor products run on the context's stream, largest first, and every
 * factorisation starts on a side stream as soon as its factor is ready, so the chains of small
 * kernels hide under the remaining products (one CUDA graph on a single GPU).  With a
 * communicator each factor is all-reduced before its factorisation starts on the rank that owns
 * it.  devPtr: fitre_kfac_factors_and_inverses_mem_required doubles. */
long fitre_kfac_factors_and_inverses_mem_required(const CNN_MODEL *m);
int fitre_kfac_factors_and_inverses(fitre_context *ctx, const CNN_MODEL *m, const real *x0,
                                    const real *zbase, const real *dbase, int packed, int samples,
                                    real *omegaZ, real *omegaZInv, real *lambdaG, real *lambdaGInv,
                                    const FITRE_KFAC_INFO *info, real *devPtr);
/* fitre_kfac_factors_and_inverses as two calls, so that the A side -- whose factorisations are
 * chains of about a thousand small dependent kernels that leave most of the GPU idle -- runs
 * underneath whatever the caller queues between the two (in a KFAC step: the second backward pass on
 * the sampled labels, which only the G factors depend on).
 *   fitre_kfac_omega_z_begin: the A factors (they need the forward state z only) and the damped
 *     factorisation of each as soon as it is ready, on streams of the library's own, ordered after
 *     everything queued on the context's stream so far.  Returns without waiting, and the context's
 *     stream does not wait either: omegaZ / omegaZInv and devPtr belong to the library until the
 *     finish call returns.
 *   fitre_kfac_lambda_delta_finish: the G factors and their inverses (after the A side, with which
 *     they share devPtr), then the context's stream and the host wait for everything both calls
 *     started; FITRE_ERR_NOT_CONVERGED as in the one-call form.
 * devPtr: fitre_kfac_factors_and_inverses_mem_required(m) doubles, the same buffer in both calls
 * and not the scratch of the work queued in between.  Same bits as the one-call form; follows
 * fitre_set_kfac_solver / fitre_set_kfac_distribution.  Reference: the two halves are
 * computeOmegaZ and computeLambdaDelta (solvers/kfac_inverses.cu:450-630,759-857), which it
 * runs one after the other. */
int fitre_kfac_omega_z_begin(fitre_context *ctx, const CNN_MODEL *m, const real *x0, const real *zbase,
                             int packed, int samples, real *omegaZ, real *omegaZInv,
                             const FITRE_KFAC_INFO *info, real *devPtr);
int fitre_kfac_lambda_delta_finish(fitre_context *ctx, const CNN_MODEL *m, const real *dbase, int packed,
                                   int samples, real *lambdaG, real *lambdaGInv,
                                   const FITRE_KFAC_INFO *info, real *devPtr);

/* solvers/kfac_natural_gradient.cu:36-241 (computeNaturalGradient): nGradient = G^-1 [W|b] A^-1
 * per layer, in the flat layout of `gradient`.  omegaZInv / lambdaGInv hold what
 * fitre_kfac_invert_factors left there under the same solver setting: the inverted factors at
 * the offsets of `info` (A blocks K' x K' with K' = K + bias), or, with
 * FITRE_KFAC_SOLVER_CHOLESKY, Cholesky factors in the A slots, applied by triangular solves.  The
 * layers run on side streams; devPtr: fitre_kfac_natural_gradient_mem_required doubles. */
long fitre_kfac_natural_gradient_mem_required(const CNN_MODEL *m);
int fitre_compute_natural_gradient(fitre_context *ctx, const CNN_MODEL *m,
                                   const FITRE_KFAC_INFO *info, const real *omegaZInv,
                                   const real *lambdaGInv, const real *gradient, real *nGradient,
                                   real *devPtr);

/* C (n x n, both triangles) = alpha * A'A with A rows x n column-major (lda), the product behind
 * every G-factor block above, for callers that cannot allocate device memory (a driver whose
 * workspace already owns all of it, code between stream-capture calls, threads barred from the
 * allocator): it needs no context and no scratch argument because its split-sum slabs live in
 * an 8 MiB array built into the library (held on every GPU that loads it).  Limit n <= 1024
 * (FITRE_ERR_TOO_LARGE beyond).  The first call on a device resolves the array's address and
 * should precede any stream capture; calls that overlap on the GPU race on the shared array.
 * `stream` is a cudaStream_t.  This entry point has no counterpart in the reference. */
int fitre_syrk_tn_static_scratch(const real *A, long rows, int n, long lda, real alpha, real *C,
                                 void *stream);

/* ---- training loop pieces either side of the path ------------------------------------- */
/* solvers/kfac_trust_region.cu:66-77 (initBatchNormData): running mean 0 / variance 1 in the
 * running-statistics slots of `z` for every batch-normalised layer. */
int fitre_init_batch_norm_data(fitre_context *ctx, const CNN_MODEL *m, real *z);
/* functions/cnn_eval_model.cu:7-13 (evaluateCNNModel): a MODEL_TRAIN forward, loss -> *loss_host. */
int fitre_evaluate_cnn_model(fitre_context *ctx, const CNN_MODEL *m, const DEVICE_DATASET *data,
                             SCRATCH_AREA *scratch, real *z, real *probs, real *lossFuncErrors,
                             int offset, int curBatchSize, real *loss_host);
/* functions/cnn_accuracy.cu:16-59 (computeAccuracy): predicted class = first class whose
 * probability strictly exceeds the running maximum (starting at 0); *hits_host = number of hits
 * and *accuracy_host = percentage, both over the global batch when a communicator is set. */
int fitre_compute_accuracy(fitre_context *ctx, const real *probs, const real *target, int rows,
                           int numClasses, real *hits_host, real *accuracy_host);
/* Minibatch assembly in one kernel: utilities/sample_matrix.cu:70-92 (selectColumnMatrix: gather
 * images `indices[offset..offset+n)` -- or offset..offset+n when indices is NULL -- and their
 * labels from the features x samples matrix setX / setY), solvers/kfac_da.cu:22-89 (augmentData:
 * per-image [C][W][H] -> batch [C][N][W][H]; when `uniforms` is given, random crop with padding 4
 * then random horizontal flip, augmentation/dev_crop.cu, dev_flip.cu) and
 * augmentation/dev_normalize.cu (v/255, minus channel mean, over channel deviation, chosen by
 * data->datasetType).  `uniforms` = 3n device doubles in [0,1): row shifts, column shifts, flips
 * (replaces the reference's cuRAND draws).  Writes data->sampledTrainY and the second half of
 * data->sampledTrainX (2n*features doubles, as allocSampledDataset sizes it) and points
 * data->currentBatch there. */
/* utilities/sample_matrix.cu:70-92 (selectColumnMatrix) on its own: images and labels
 * indices[offset .. offset+sampleSize) of the training set -> data->sampledTrainX / sampledTrainY,
 * no layout change.  fitre_prepare_minibatch does this and the rest of the pipeline in one
 * kernel; this entry point exists for callers that keep the reference's two-step sequence. */
int fitre_select_column_matrix(fitre_context *ctx, DEVICE_DATASET *data, int sampleSize,
                               const int *indices, int offset);
int fitre_prepare_minibatch(fitre_context *ctx, const CNN_MODEL *m, DEVICE_DATASET *data,
                            const real *setX, const real *setY, const int *indices, long offset,
                            int n, const real *uniforms);
/* functions/cnn_accuracy.cu:61-174 (computeTestGeneralizationErrors for evalType =
 * FITRE_MODEL_TEST_ACCURACY, computeTrainGeneralizationErrors for FITRE_MODEL_TRAIN_ACCURACY):
 * mean loss and accuracy (percent) over the whole set in minibatches of model->batchSize,
 * batch norm with the running statistics of `z`, no augmentation.  Loop bounds follow the
 * reference: the test sweep includes the partial last batch, the train sweep stops before the
 * last batch; both divide by the set size.  With a communicator each global batch is split
 * over the ranks and what does not fill a global batch is evaluated redundantly by every rank.
 * Scratch behind scratch->nextDevPtr: fitre_generalization_mem_required doubles. */
long fitre_generalization_mem_required(const CNN_MODEL *m);
int fitre_compute_generalization_errors(fitre_context *ctx, const CNN_MODEL *m, DEVICE_DATASET *data,
                                        SCRATCH_AREA *scratch, real *z, real *probs, real *errors,
                                        int evalType, real *likelihood, real *accuracy);
/* solvers/kfac_trust_region.cu:94-661 (subsampledTrustRegionKFAC): per epoch a
 * shuffled sweep over the training set; per minibatch gradient, sampled-label backward, A and G
 * factors with damped inverses, natural gradient, quadratic model of the KFAC direction (and of
 * the gradient when checkGrad), momentum, weight update, re-evaluation, reduction ratio, radius
 * update and the reference's revert rule; after each epoch the two generalisation sweeps.
 * kfacInfo->inverseFreq > 1 selects the running-average variant: factors and inverses on the
 * very first minibatch, then every inverseFreq minibatches from running averages of the layer
 * inputs and errors (decay sqrt(stats_decay)); the natural gradient uses the latest inverses.
 * trParams->maxIters epochs; `maxMiniBatches` > 0 stops each epoch early (tests).  Random draws
 * (shuffle, augmentation, sampled labels) come from a counter-based generator seeded with `seed`,
 * identical on every rank.  `steps` (capacity stepsCap) and `epochs` (capacity maxIters) may be
 * NULL.  All device memory comes from scratch->nextDevPtr: fitre_trust_region_kfac_mem_required
 * doubles (kfacInfo may be NULL there for inverseFreq <= 1).  data->weights is updated in place; data->sampledTrainX/Y must hold 2*batch*features
 * and batch doubles. */
long fitre_trust_region_kfac_mem_required(const CNN_MODEL *m, const DEVICE_DATASET *data,
                                          const FITRE_KFAC_INFO *kfacInfo);
int fitre_subsampled_trust_region_kfac(fitre_context *ctx, CNN_MODEL *m, DEVICE_DATASET *data,
                                       FITRE_KFAC_INFO *kfacInfo, TRUST_REGION_PARAMS *trParams,
                                       SCRATCH_AREA *scratch, unsigned long long seed, int enableDA,
                                       int maxMiniBatches, FITRE_TR_STEP *steps, int stepsCap,
                                       FITRE_TR_EPOCH *epochs);
/* utilities/print_utils.c:136-186 (writeVector / readVector): the `.params` text format, one
 * value per line.  referenceFormat = 1 writes the reference's "%6.10f" (byte-identical files,
 * 10 decimals); 0 writes "%.17g" (round-trips every double).  The reader takes either (atof per
 * line, stops at `n` values or end of file) and returns the count in *read_out.  Host pointers. */
int fitre_write_vector(const char *path, const real *host, long n, int referenceFormat);
int fitre_read_vector(const char *path, real *host, long n, long *read_out);

/* ---- host-buffer entry point (what a reference driver calls per minibatch) ---- */
/* One gradient + one Hessian-vector product with HOST inputs and outputs: copies the
 * batch, labels, weights and `vector` to the device, runs fitre_compute_cnn_gradient and
 * fitre_cnn_hv, all-reduces when a communicator is set, and copies gradient and hv back.
 * Device state lives in a workspace the context allocates on first use for this model
 * and batch size (stream-ordered allocation; reused by later calls). */
int fitre_gradient_hv_host(fitre_context *ctx, const CNN_MODEL *m, const real *batch_host,
                           const real *labels_host, const real *weights_host,
                           const real *vector_host, int curBatchSize, int numClasses,
                           real weightDecay, real *loss_host, real *gradient_host,
                           real *hv_host);
/* With ranks, gradient and hv are the same vectors on every rank, and on one node the ranks' host
 * memory is one memory.  on = 1 tells fitre_gradient_hv_host that gradient_host and hv_host
 * address the SAME physical buffers on every rank of the communicator (one shared-memory segment
 * mapped, and page-locked, by every process): each rank then copies only its 1/world share of
 * every finished slice, and the call returns once all ranks' shares have landed (a one-element
 * all-reduce queued behind the copies is the barrier), so the node moves each result across
 * PCIe once instead of `world` times.  loss_host stays private.  Default 0: every rank fills its
 * own buffers.  No counterpart in the reference (one GPU, device-resident results). */
int fitre_set_host_results_shared(fitre_context *ctx, int on);
/* The inputs' counterpart: on = 1 tells fitre_gradient_hv_host that weights_host and vector_host
 * hold the same values on every rank (what data parallelism means: replicated parameters, one
 * direction).  Each rank then uploads one of `world` equal chunks of either vector and the chunks
 * are exchanged by an all-gather over NVLink, so the node reads each from host memory once.  All
 * ranks must set it alike (the all-gather is a collective).  Batch and labels are per rank and
 * travel as before.  Default 0.  Falls back to full uploads when the NCCL library has no
 * ncclAllGather. */
int fitre_set_host_inputs_replicated(fitre_context *ctx, int on);

#ifdef __cplusplus
}
#endif
#endif /* FITRE_B200_H */
