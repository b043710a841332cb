/*
 * fitre_oracle.h -- CPU restatement of FITRE's CNN gradient / Hessian-vector /
 * KFAC-factor path.  TEST INFRASTRUCTURE ONLY: it is the checker the CUDA library is
 * compared against (tests, the smoke check and the benchmark's CPU baseline leg); the
 * product never links or calls it.
 *
 * Every function follows the operation order of the reference's CUDA host code, with
 * the GPU kernels and cuBLAS calls replaced by plain loops (OpenMP over independent
 * outputs).  All buffers are HOST memory in the reference's layouts.
 */
#ifndef FITRE_ORACLE_H
#define FITRE_ORACLE_H

#include "../include/fitre_b200.h"

#ifdef __cplusplus
extern "C" {
#endif

/* Sum-all-reduce hook used to emulate data-parallel ranks (NULL = single rank). */
typedef void (*ora_allreduce_fn)(double *buf, long n, void *user);

typedef struct ora_env {
    int ref_softmax;        /* 1: max-shift starts at 0 and probs += 1e-10 (softmax_loss.cu:24-27,55) */
    int world;              /* data-parallel ranks; N_global = world * curBatchSize */
    ora_allreduce_fn allreduce;
    void *user;
    int eval_type;          /* FITRE_MODEL_TRAIN (default): batch statistics, running statistics
                             * updated; the two *_ACCURACY values: normalise with the running
                             * statistics (functions/dev_batch_norm.cu:331-393) */
    int rank;               /* this rank's index among `world` (outer loop: which slice of each
                             * global minibatch it assembles) */
    int ref_quadratic;      /* 1: the quadratic model adds weightDecay * weights to Hv
                             * (functions/model_reduction.cu:50-52); 0: weightDecay * vector
                             * (pytorch/peng/utils.py:77) */
} ORA_ENV;

void ora_env_default(ORA_ENV *env);
void ora_set_num_threads(int n);

/* model set-up: nn/utils.c:12-172, nn/read_vgg.c:25-120 */
int ora_model_finalize(CNN_MODEL *m);
long ora_model_zsize64(const CNN_MODEL *m);

/* unit operators (each cites its reference source in the .c file) */
void ora_im2col(const double *x, int N, int C, int H, int W, int k, int pad, int stride,
                double *cols);
void ora_im2col_index(int N, int C, int H, int W, int k, int pad, int stride, long *src_index);
void ora_gemm(int transA, int transB, long m, long n, long k, double alpha, const double *A,
              long lda, const double *B, long ldb, double beta, double *C, long ldc);
void ora_pool_forward(const double *in, int N, int C, int H, int W, int ks, int stride, int pad,
                      int type, double *out);
void ora_max_pool_argmax(const double *act, int N, int C, int H, int W, int ks, int stride,
                         int pad, int *argmax);
void ora_max_pool_backward(const double *delta, const double *act, int C, int H, int W, int ks,
                           int stride, int pad, int Hp, int Wp, int N, double *out);
void ora_avg_pool_backward(const double *delta, int Hp, int C, int ks, int N, double *out);
void ora_rop_max_pool(const double *rz, const double *zact, int N, int C, int H, int W, int ks,
                      int stride, int pad, double *out);
void ora_batch_norm_forward(const ORA_ENV *env, const double *in, int H, int W, int C, int N,
                            double *out, double *mean, double *var, double eps);
void ora_init_batch_norm_data(const CNN_MODEL *m, double *z);
double ora_compute_accuracy(const ORA_ENV *env, const double *probs, const double *target, int rows,
                            int classes, double *hits_out);
void ora_prepare_minibatch(const double *setX, const double *setY, const int *indices, long offset,
                           int n, int C, int H, int W, int datasetType, const double *uniforms,
                           double *batch, double *labels);
void ora_batch_norm_backward(const ORA_ENV *env, const double *delta, int H, int W, int C,
                             int N, const double *var, const double *zhat, double eps,
                             double *out);
void ora_rop_batch_norm_forward(const ORA_ENV *env, const double *z, const double *mean,
                                const double *var, const double *rz_in, double eps, int H,
                                int W, int C, int N, double *rz_out);
void ora_rop_batch_norm_backward(const ORA_ENV *env, const double *z_in, const double *z_out,
                                 const double *rz_in, const double *rz_out, const double *delta,
                                 double *rdelta, double eps, const double *mean,
                                 const double *var, int H, int W, int C, int N);
void ora_conv_dgrad(const double *delta, int dH, int dW, int dC, const double *filter, int k,
                    int H, int W, int pad, int C, int N, double *out);
void ora_activation(int act, double *x, long n);
double ora_softmax_loss(const ORA_ENV *env, const double *logits, const double *target, int N,
                        int classes, double *probs);

void ora_distribution_errors(const ORA_ENV *env, const double *probs, const double *uniforms,
                             int N, int classes, double *distTarget, double *distError);

/* whole-network passes */
double ora_cnn_forward(const ORA_ENV *env, const CNN_MODEL *m, const double *batch,
                       const double *labels, const double *weights, int numClasses, double *z,
                       double *probs, double *errors, int n);
void ora_cnn_backward(const ORA_ENV *env, const CNN_MODEL *m, const double *batch,
                      const double *weights, const double *z, double *gradient, double *dx,
                      const double *errors, int n);
double ora_cnn_gradient(const ORA_ENV *env, const CNN_MODEL *m, const double *batch,
                        const double *labels, const double *weights, int numClasses, double *z,
                        double *dx, double *probs, double *errors, double *gradient, int n,
                        double weightDecay);
void ora_cnn_rop_forward(const ORA_ENV *env, const CNN_MODEL *m, const double *batch,
                         const double *weights, const double *z, const double *vector,
                         double *rz, int n);
void ora_cnn_rop_backward(const ORA_ENV *env, const CNN_MODEL *m, const double *batch,
                          const double *weights, const double *z, const double *dx,
                          const double *errors, double *rError, const double *rz,
                          const double *vector, double *hv, int n);
void ora_cnn_hv(const ORA_ENV *env, const CNN_MODEL *m, const double *batch,
                const double *weights, int numClasses, const double *z, const double *probs,
                const double *errors, const double *dx, const double *vector, double *hv,
                double *rz, int n);
double ora_quadratic_model(const ORA_ENV *env, const CNN_MODEL *m, const double *batch,
                           const double *weights, int numClasses, const double *z,
                           const double *probs, const double *errors, const double *dx,
                           const double *gradient, double *vector, double delta, int n,
                           double weightDecay);
void ora_cg_steihaug(const ORA_ENV *env, const CNN_MODEL *m, const double *batch,
                     const double *weights, int numClasses, const double *z,
                     const double *probs, const double *errors, const double *dx,
                     const double *gradient, double *p, int n, FITRE_CG_PARAMS *params);

/* KFAC factors */
int ora_kfac_storage_indices(const CNN_MODEL *m, FITRE_KFAC_INFO *info);
void ora_kfac_omega_z(const ORA_ENV *env, const CNN_MODEL *m, const double *batch,
                      const double *z, int n, double *omegaZ, const FITRE_KFAC_INFO *info);
void ora_kfac_lambda_delta(const ORA_ENV *env, const CNN_MODEL *m, const double *dx, int n,
                           double *lambdaG, const FITRE_KFAC_INFO *info);

/* the running-average ("speed-up") variant: solvers/kfac_inverses.cu:106-126,386-447,699-755 */
void ora_update_running_stats(double *src, const double *update, long n, double momentum);
void ora_kfac_speedup_omega_z(const FITRE_KFAC_INFO *info, const CNN_MODEL *m, const double *batch, long features,
                              int n, const double *z, double *dampedInput, double *dampedZ, int iterCount);
void ora_kfac_speedup_lambda_delta(const FITRE_KFAC_INFO *info, const CNN_MODEL *m, int n, const double *dx,
                                   double *dampedLambda, int iterCount);
void ora_kfac_omega_z_damped(const ORA_ENV *env, const CNN_MODEL *m, const double *dampedInput,
                             const double *dampedZ, int n, double *omegaZ, const FITRE_KFAC_INFO *info);
void ora_kfac_lambda_delta_damped(const ORA_ENV *env, const CNN_MODEL *m, const double *dampedLambda, int n,
                                  double *lambdaG, const FITRE_KFAC_INFO *info);

int ora_kfac_matrix_inverse(const double *matrix, double *inverse, int n, double lambda,
                            double gamma);
void ora_natural_gradient(const CNN_MODEL *m, const FITRE_KFAC_INFO *info, const double *omegaZInv,
                          const double *lambdaGInv, const double *gradient, double *nGradient);

/* evaluation sweeps and the FITRE outer loop (single rank over the global batch) */
void ora_generalization_errors(const ORA_ENV *env, const CNN_MODEL *m, const double *setX,
                               const double *setY, long size, int datasetType,
                               const double *weights, int numClasses, double *z, int test,
                               double *likelihood, double *accuracy);
int ora_subsampled_trust_region_kfac(const ORA_ENV *env, const CNN_MODEL *m, const double *trainX,
                                     const double *trainY, long trainN, const double *testX,
                                     const double *testY, long testN, int datasetType,
                                     double *weights, int numClasses, FITRE_KFAC_INFO *info,
                                     TRUST_REGION_PARAMS *tr, unsigned long long seed, int enableDA,
                                     int maxMiniBatches, FITRE_TR_STEP *steps, int stepsCap,
                                     FITRE_TR_EPOCH *epochs);

#ifdef __cplusplus
}
#endif
#endif
