/*
 * fitre_oracle.c -- CPU restatement of FITRE's CNN gradient / Hessian-vector / KFAC-factor
 * path.  TEST INFRASTRUCTURE ONLY (the checker for the CUDA library; never linked into it).
 *
 * Each function names the reference source (path within kylasa/FITRE, file:line) whose
 * operation order it follows.  GPU kernels and cuBLAS calls become plain loops; results
 * therefore agree with the reference up to floating-point summation order.
 *
 * Pinned against: the reference's batch-norm known-answer vectors
 * (pytorch/testing/batchnorm_derivative.py + my.out, batchnorm_rop.py), the LeNet offset
 * table of pytorch/kfac/cifar_kfac_trust_iteration.txt:12-13, and gradient / Hessian-vector
 * fixtures produced by PyTorch double-backward through the reference's own weight-layout
 * reader pytorch/testing/readWeights.py (see tests/golden/).
 *
 * Deviations from the reference, on purpose:
 *  - ReLU is differentiated (h' = 1[z>0], h'' = 0); the reference leaves ReLU out of the
 *    backward and R-op passes (functions/cnn_backward.cu:561-562, cnn_hv_backward.cu:676).
 *  - the R-op batch-norm backward uses the per-channel scale the reference intends; its
 *    ker_rI_scale launch indexes past the per-channel buffer (dev_batch_norm.cu:174-183,910).
 *  - cnnROpForward passes actFuns[0] for every layer (cnn_hv_forward.cu:86,125); here layer
 *    l uses actFuns[l] (identical for every builder of the reference).
 *  - the R-op pooling uses the backward pass's arg-max scan order (dev_pool.cu:374-391) for
 *    both directions; the reference's two scans differ only on exact ties.
 */
#include "fitre_oracle.h"

#include <float.h>
#ifdef _OPENMP
#include <omp.h>
#endif
#include <limits.h>
#include <math.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#define BN_EPS 1e-5 /* functions/dev_batch_norm.h:10 */

static double *xmalloc(long n) {
    if (n < 1) n = 1;
    double *p = (double *)malloc(sizeof(double) * (size_t)n);
    if (!p) {
        fprintf(stderr, "fitre_oracle: out of memory (%ld doubles)\n", n);
        abort();
    }
    return p;
}

void ora_env_default(ORA_ENV *env) {
    env->ref_softmax = 1;
    env->world = 1;
    env->allreduce = NULL;
    env->user = NULL;
    env->eval_type = FITRE_MODEL_TRAIN;
    env->rank = 0;
    env->ref_quadratic = 1;
}

/* number of OpenMP threads of the following calls (a launcher may have exported OMP_NUM_THREADS=1) */
void ora_set_num_threads(int n) {
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}

static void env_allreduce(const ORA_ENV *env, double *buf, long n) {
    if (env && env->allreduce) env->allreduce(buf, n, env->user);
}
static int env_world(const ORA_ENV *env) { return (env && env->world > 0) ? env->world : 1; }

/* ------------------------------------------------------------------------------------ */
/* Model set-up                                                                          */
/* ------------------------------------------------------------------------------------ */

/* nn/utils.c:12-17 */
static void out_dims(int h, int w, int pad, int stride, int k, int *oh, int *ow) {
    *oh = (h + 2 * pad - k) / stride + 1;
    *ow = (w + 2 * pad - k) / stride + 1;
}

/* Per-layer offsets: nn/read_vgg.c:25-120 (makeLayer).  Parameter offsets:
 * nn/utils.c:19-105.  z offsets: nn/utils.c:107-172. */
int ora_model_finalize(CNN_MODEL *m) {
    int B = m->batchSize;
    if (m->cLayers < 1 || m->cLayers + m->lLayers + 1 >= FITRE_MAX_LAYERS || B < 1) return 1;
    for (int l = 0; l < m->cLayers; l++) {
        CONV_LAYER *c = &m->convLayer[l];
        POOL_LAYER *p = &m->poolLayer[l];
        out_dims(c->height, c->width, c->padding, c->stride, c->kSize, &c->outHeight,
                 &c->outWidth);
        p->height = c->outHeight;
        p->width = c->outWidth;
        if (p->type == FITRE_NO_POOL) {
            p->outHeight = p->height;
            p->outWidth = p->width;
        } else {
            /* functions/dev_pool.cu:226-227 */
            p->outHeight = (int)floor((double)(p->height - p->pSize + 2 * p->padding) / p->stride + 1.);
            p->outWidth = (int)floor((double)(p->width - p->pSize + 2 * p->padding) / p->stride + 1.);
        }
        long V = (long)c->outHeight * c->outWidth * c->outChannels * B;
        long P = (long)p->outHeight * p->outWidth * c->outChannels * B;
        if (3 * V + 4 * c->outChannels + P > INT_MAX) return 2;
        if (c->batchNorm == FITRE_NO_BATCH_NORM) {
            c->activationOffset = (int)V;
            c->batchNormOffset = INT_MAX;
            c->meansOffset = c->variancesOffset = INT_MAX;
            c->runningMeansOffset = c->runningVariancesOffset = INT_MAX;
            if (p->type == FITRE_NO_POOL) {
                c->poolOffset = INT_MAX;
                c->outputOffset = c->activationOffset;
            } else {
                c->poolOffset = (int)(2 * V);
                c->outputOffset = c->poolOffset;
            }
        } else {
            c->batchNormOffset = (int)V;
            c->meansOffset = (int)V; /* relative to the batch-norm output */
            c->variancesOffset = c->meansOffset + c->outChannels;
            c->runningMeansOffset = c->variancesOffset + c->outChannels;
            c->runningVariancesOffset = c->runningMeansOffset + c->outChannels;
            c->activationOffset = (int)(2 * V + 4 * c->outChannels);
            if (p->type == FITRE_NO_POOL) {
                c->poolOffset = INT_MAX;
                c->outputOffset = c->activationOffset;
            } else {
                c->poolOffset = c->activationOffset + (int)V;
                c->outputOffset = c->poolOffset;
            }
        }
        c->convVolumn = c->outHeight * c->outWidth * c->outChannels;
        c->activationVolumn = c->convVolumn;
        c->batchNormVolumn = (c->batchNorm != FITRE_NO_BATCH_NORM) ? INT_MAX : c->convVolumn;
        c->poolVolumn = (p->type == FITRE_NO_POOL)
                            ? INT_MAX
                            : p->outHeight * p->outWidth * c->outChannels;
    }
    for (int l = 0; l < m->lLayers; l++) m->fcLayer[l].offset = m->fcLayer[l].out * B;

    /* nn/utils.c:19-42 */
    long ps = 0;
    for (int i = 0; i < m->cLayers; i++) {
        CONV_LAYER *t = &m->convLayer[i];
        ps += (long)t->outChannels * t->kSize * t->kSize * t->inChannels;
        if (m->bias >= 1) ps += t->outChannels;
    }
    for (int i = 0; i < m->lLayers; i++) {
        ps += (long)m->fcLayer[i].out * m->fcLayer[i].in;
        if (m->bias >= 1) ps += m->fcLayer[i].out;
    }
    if (ps > INT_MAX) return 2;
    m->pSize = (int)ps;

    for (int i = 0; i < FITRE_MAX_LAYERS; i++) m->wOffsets[i] = m->bOffsets[i] = m->zOffsets[i] = 0;
    int L = m->cLayers + m->lLayers;
    int off = 0;
    for (int i = 0; i < L; i++) { /* weights then (optionally) bias, layer by layer */
        int wsz, bsz;
        if (i < m->cLayers) {
            CONV_LAYER *t = &m->convLayer[i];
            wsz = t->outChannels * t->kSize * t->kSize * t->inChannels;
            bsz = t->outChannels;
        } else {
            wsz = m->fcLayer[i - m->cLayers].out * m->fcLayer[i - m->cLayers].in;
            bsz = m->fcLayer[i - m->cLayers].out;
        }
        m->wOffsets[i] = off;
        off += wsz;
        if (m->bias != 0) {
            m->bOffsets[i] = off;
            off += bsz;
        } else {
            m->bOffsets[i] = INT_MAX; /* nn/utils.c:49 */
        }
    }
    if (m->bias == 0) m->wOffsets[L] = off; /* nn/utils.c:60,70 */

    /* nn/utils.c:107-172 */
    for (int i = 0; i < FITRE_MAX_LAYERS; i++) m->zztOffsets[i] = 0;
    m->maxDeltaSize = 0;
    m->zztSize = 0;
    long zo = 0;
    m->zOffsets[0] = 0;
    m->zOffsets[1] = 0;
    for (int i = 1; i <= m->cLayers; i++) {
        CONV_LAYER *t = &m->convLayer[i - 1];
        POOL_LAYER *p = &m->poolLayer[i - 1];
        long V = (long)B * t->outHeight * t->outWidth * t->outChannels;
        long sz = 2 * V;
        if (t->batchNorm != FITRE_NO_BATCH_NORM) sz += V + 4 * t->outChannels;
        if (p->type != FITRE_NO_POOL) sz += (long)B * p->outHeight * p->outWidth * t->outChannels;
        zo += sz;
        if (zo > INT_MAX) return 2;
        m->zOffsets[i + 1] = (int)zo;
        m->zztOffsets[i + 1] = m->zztOffsets[i] + (int)V;
        m->zztSize += (int)V;
        if (sz > m->maxDeltaSize) m->maxDeltaSize = (int)sz;
    }
    for (int i = 1; i <= m->lLayers; i++) {
        FC_LAYER *t = &m->fcLayer[i - 1];
        long sz = (long)t->out * B * 2;
        zo += sz;
        if (zo > INT_MAX) return 2;
        m->zOffsets[i + m->cLayers + 1] = (int)zo;
        m->zztOffsets[i + 1 + m->cLayers] = m->zztOffsets[i + m->cLayers] + t->out * B;
        m->zztSize += t->out * B;
        if (sz > m->maxDeltaSize) m->maxDeltaSize = (int)sz;
    }
    m->zSize = m->zOffsets[m->cLayers + m->lLayers + 1];
    return 0;
}

long ora_model_zsize64(const CNN_MODEL *m) { return m->zSize; }

/* ------------------------------------------------------------------------------------ */
/* Dense helpers                                                                         */
/* ------------------------------------------------------------------------------------ */

/* Column-major C = alpha * op(A) * op(B) + beta * C  (cublasDgemm semantics). */
/* C = alpha op(A) op(B) + beta C, column-major (the cublasDgemm calls of the reference).  Plain
 * loops, blocked so that operands are reused from cache and registers: every C element is still
 * the sum over p in ascending order. */
#define GEMM_MB 256
#define GEMM_NB 8
void ora_gemm(int tA, int tB, long m, long n, long k, double alpha, const double *A, long lda,
              const double *B, long ldb, double beta, double *C, long ldc) {
    if (!tA) {
        const long mblocks = (m + GEMM_MB - 1) / GEMM_MB, nblocks = (n + GEMM_NB - 1) / GEMM_NB;
#pragma omp parallel for collapse(2) schedule(static)
        for (long jb = 0; jb < nblocks; jb++)
            for (long ib = 0; ib < mblocks; ib++) {
                const long i0 = ib * GEMM_MB, j0 = jb * GEMM_NB;
                const long mb = (m - i0 < GEMM_MB) ? m - i0 : GEMM_MB;
                const long nb = (n - j0 < GEMM_NB) ? n - j0 : GEMM_NB;
                double acc[GEMM_NB][GEMM_MB];
                for (long j = 0; j < nb; j++)
                    for (long i = 0; i < mb; i++) acc[j][i] = 0.0;
                for (long p = 0; p < k; p++) {
                    const double *a = A + p * lda + i0;
                    for (long j = 0; j < nb; j++) {
                        const double bv = alpha * (tB ? B[(j0 + j) + p * ldb] : B[p + (j0 + j) * ldb]);
                        double *c = acc[j];
                        for (long i = 0; i < mb; i++) c[i] += a[i] * bv;
                    }
                }
                for (long j = 0; j < nb; j++) {
                    double *c = C + (j0 + j) * ldc + i0;
                    if (beta == 0.0)
                        for (long i = 0; i < mb; i++) c[i] = acc[j][i];
                    else
                        for (long i = 0; i < mb; i++) c[i] = beta * c[i] + acc[j][i];
                }
            }
        return;
    }
    /* op(A) = A': rows of op(A) are contiguous columns of A; 4 x 4 register blocks of dot products */
    const long iblocks = (m + 3) / 4, jblocks = (n + 3) / 4;
#pragma omp parallel for collapse(2) schedule(static)
    for (long jb = 0; jb < jblocks; jb++)
        for (long ib = 0; ib < iblocks; ib++) {
            const long i0 = ib * 4, j0 = jb * 4;
            const long mb = (m - i0 < 4) ? m - i0 : 4, nb = (n - j0 < 4) ? n - j0 : 4;
            double s[4][4] = {{0}};
            if (mb == 4 && nb == 4 && !tB) {
                const double *a0 = A + i0 * lda, *a1 = a0 + lda, *a2 = a1 + lda, *a3 = a2 + lda;
                const double *b0 = B + j0 * ldb, *b1 = b0 + ldb, *b2 = b1 + ldb, *b3 = b2 + ldb;
                for (long p = 0; p < k; p++) {
                    const double x0 = a0[p], x1 = a1[p], x2 = a2[p], x3 = a3[p];
                    const double y0 = b0[p], y1 = b1[p], y2 = b2[p], y3 = b3[p];
                    s[0][0] += x0 * y0; s[0][1] += x0 * y1; s[0][2] += x0 * y2; s[0][3] += x0 * y3;
                    s[1][0] += x1 * y0; s[1][1] += x1 * y1; s[1][2] += x1 * y2; s[1][3] += x1 * y3;
                    s[2][0] += x2 * y0; s[2][1] += x2 * y1; s[2][2] += x2 * y2; s[2][3] += x2 * y3;
                    s[3][0] += x3 * y0; s[3][1] += x3 * y1; s[3][2] += x3 * y2; s[3][3] += x3 * y3;
                }
            } else {
                for (long i = 0; i < mb; i++)
                    for (long j = 0; j < nb; j++) {
                        const double *a = A + (i0 + i) * lda;
                        double t = 0.0;
                        if (!tB) {
                            const double *bb = B + (j0 + j) * ldb;
                            for (long p = 0; p < k; p++) t += a[p] * bb[p];
                        } else {
                            for (long p = 0; p < k; p++) t += a[p] * B[(j0 + j) + p * ldb];
                        }
                        s[i][j] = t;
                    }
            }
            for (long i = 0; i < mb; i++)
                for (long j = 0; j < nb; j++) {
                    double *c = C + (j0 + j) * ldc + (i0 + i);
                    *c = (beta == 0.0 ? 0.0 : beta * *c) + alpha * s[i][j];
                }
        }
}

static void axpy(long n, double a, const double *x, double *y) {
#pragma omp parallel for schedule(static)
    for (long i = 0; i < n; i++) y[i] += a * x[i];
}
static double dot(long n, const double *x, const double *y) {
    double s = 0.0;
#pragma omp parallel for reduction(+ : s) schedule(static)
    for (long i = 0; i < n; i++) s += x[i] * y[i];
    return s;
}

/* ------------------------------------------------------------------------------------ */
/* im2col: functions/dev_image.cu:12-51                                                  */
/* ------------------------------------------------------------------------------------ */

/* Source flat index of every im2col element (-1 = zero padding).  Row r = n*Ho*Wo + wo*Ho + ho,
 * column q = cin*k*k + j*k + i, stored column-major with leading dimension M. */
void ora_im2col_index(int N, int C, int H, int W, int k, int pad, int stride, long *idx) {
    int Ho, Wo;
    out_dims(H, W, pad, stride, k, &Ho, &Wo);
    long M = (long)N * Ho * Wo;
#pragma omp parallel for collapse(2) schedule(static)
    for (int cin = 0; cin < C; cin++)
        for (int n = 0; n < N; n++)
            for (int wo = 0; wo < Wo; wo++)
                for (int ho = 0; ho < Ho; ho++) {
                    int h_in = ho * stride - pad, w_in = wo * stride - pad;
                    long row = (long)n * Ho * Wo + (long)wo * Ho + ho;
                    for (int j = 0; j < k; j++)
                        for (int i = 0; i < k; i++) {
                            int h = h_in + i, w = w_in + j;
                            long q = (long)cin * k * k + j * k + i;
                            long src = -1;
                            if (h >= 0 && w >= 0 && h < H && w < W)
                                src = (((long)cin * N + n) * W + w) * H + h;
                            idx[q * M + row] = src;
                        }
                }
}

void ora_im2col(const double *x, int N, int C, int H, int W, int k, int pad, int stride,
                double *cols) {
    int Ho, Wo;
    out_dims(H, W, pad, stride, k, &Ho, &Wo);
    long M = (long)N * Ho * Wo;
#pragma omp parallel for collapse(2) schedule(static)
    for (int cin = 0; cin < C; cin++)
        for (int n = 0; n < N; n++)
            for (int wo = 0; wo < Wo; wo++)
                for (int ho = 0; ho < Ho; ho++) {
                    int h_in = ho * stride - pad, w_in = wo * stride - pad;
                    long row = (long)n * Ho * Wo + (long)wo * Ho + ho;
                    const double *src = x + ((long)cin * N + n) * W * H;
                    for (int j = 0; j < k; j++)
                        for (int i = 0; i < k; i++) {
                            int h = h_in + i, w = w_in + j;
                            long q = (long)cin * k * k + j * k + i;
                            cols[q * M + row] =
                                (h >= 0 && w >= 0 && h < H && w < W) ? src[(long)w * H + h] : 0.0;
                        }
                }
}

/* [right][left][chunk] -> [left][right][chunk]: functions/dev_backprop_convolution.cu:140-156 */
static void reshape_matrix(const double *in, int right, int left, int chunk, double *out) {
    long n = (long)right * left * chunk;
#pragma omp parallel for schedule(static)
    for (long idx = 0; idx < n; idx++) {
        long nId = idx / ((long)chunk * left);
        long nIdx = idx % ((long)chunk * left);
        long cId = nIdx / chunk;
        long chunkId = nIdx % chunk;
        out[cId * ((long)chunk * right) + nId * chunk + chunkId] = in[idx];
    }
}

/* Per-plane column-major -> row-major: functions/dev_transpose.cu:8-30 (square planes). */
static void transpose_planes(const double *in, long count, int height, int width, double *out) {
    long plane = (long)height * width;
#pragma omp parallel for schedule(static)
    for (long idx = 0; idx < count; idx++) {
        long base = (idx / plane) * plane;
        long r = idx % plane;
        long col = r / height, row = r % height;
        out[base + row * height + col] = in[idx];
    }
}

/* conv-layout [C][N][P] -> FC layout (feature c*P + h*Wp + w, sample-major columns):
 * functions/cnn_forward.cu:237-261 */
static void conv_to_fc(double *buf, int C, int N, int Hp, int Wp) {
    long cnt = (long)C * N * Hp * Wp;
    double *tmp = xmalloc(cnt);
    reshape_matrix(buf, C, N, Hp * Wp, tmp);
    transpose_planes(tmp, cnt, Hp, Wp, buf);
    free(tmp);
}
/* inverse direction for the errors: functions/cnn_backward.cu:310-326 */
static void fc_to_conv(double *buf, int C, int N, int Hp, int Wp) {
    long cnt = (long)C * N * Hp * Wp;
    double *tmp = xmalloc(cnt);
    reshape_matrix(buf, N, C, Hp * Wp, tmp);
    transpose_planes(tmp, cnt, Hp, Wp, buf);
    free(tmp);
}

/* ------------------------------------------------------------------------------------ */
/* Activations: functions/dev_activations.cu:8-77, swish.cu:14-84,                       */
/* dev_layer_error.cu:13-47, dev_layer_r_error.cu:24-38.  Logistic and tanh (FC layers,  */
/* functions/eval_gradient.cu:142-157, cnn_backward.cu:121-136) are differentiated from  */
/* their output as the reference does: y(1-y) and (1+y)(1-y); their second derivatives   */
/* y(1-y)(1-2y) and -2y(1+y)(1-y) complete the R-operator, which the reference lacks.    */
/* ------------------------------------------------------------------------------------ */
static int act_known(int a) {
    return a == FITRE_CNN_ACT_NONE || a == FITRE_ACT_LINEAR || a == FITRE_CNN_ACT_SOFTPLUS ||
           a == FITRE_CNN_ACT_RELU || a == FITRE_CNN_ACT_SWISH || a == FITRE_ACT_LOGISTIC ||
           a == FITRE_ACT_TANH;
}

void ora_activation(int act, double *x, long n) {
    if (!act_known(act)) {
        fprintf(stderr, "fitre_oracle: unknown activation %d\n", act);
        abort();
    }
#pragma omp parallel for schedule(static)
    for (long i = 0; i < n; i++) {
        double t = x[i];
        switch (act) {
            case FITRE_CNN_ACT_RELU: x[i] = t < 0 ? 0 : t; break;
            case FITRE_CNN_ACT_SOFTPLUS: x[i] = (t < 20) ? log(1 + exp(t)) : t; break;
            case FITRE_CNN_ACT_SWISH: x[i] = t / (1 + exp(-t)); break;
            case FITRE_ACT_LOGISTIC: x[i] = 1. / (1. + exp(-t)); break;
            case FITRE_ACT_TANH: x[i] = tanh(t); break;
            default: break;
        }
    }
}

/* h'(zin) given pre-activation zin and output zout */
static inline double act_d1(int act, double zin, double zout) {
    switch (act) {
        case FITRE_CNN_ACT_RELU: return zin > 0 ? 1.0 : 0.0;
        case FITRE_CNN_ACT_SOFTPLUS: return 1. / (1. + exp(-zin));
        case FITRE_CNN_ACT_SWISH: {
            double t = 1. / (1. + exp(-zin));
            return zout + t * (1. - zout);
        }
        case FITRE_ACT_LOGISTIC: return zout * (1.0 - zout);
        case FITRE_ACT_TANH: return (1.0 + zout) * (1.0 - zout);
        default: return 1.0;
    }
}
/* h''(zin) */
static inline double act_d2(int act, double zin, double zout) {
    switch (act) {
        case FITRE_CNN_ACT_SOFTPLUS: {
            double tm = exp(-zin);
            return (1. / (1. + tm)) * (tm / (1. + tm));
        }
        case FITRE_CNN_ACT_SWISH: {
            double t = 1. / (1. + exp(-zin));
            return (1. - t) * (zout + 2. * t * (1. - zout));
        }
        case FITRE_ACT_LOGISTIC: return zout * (1.0 - zout) * (1.0 - 2.0 * zout);
        case FITRE_ACT_TANH: return -2.0 * zout * (1.0 + zout) * (1.0 - zout);
        default: return 0.0;
    }
}

/* delta *= h'(zin) */
static void act_backward(int act, double *delta, const double *zin, const double *zout, long n) {
    if (act == FITRE_CNN_ACT_NONE || act == FITRE_ACT_LINEAR) return;
#pragma omp parallel for schedule(static)
    for (long i = 0; i < n; i++) delta[i] *= act_d1(act, zin[i], zout[i]);
}
/* rdelta = h'(zin) * rdelta + h''(zin) * rzin * delta_in */
static void act_rop_backward(int act, double *rdelta, const double *delta_in, const double *rzin,
                             const double *zin, const double *zout, long n) {
    if (act == FITRE_CNN_ACT_NONE || act == FITRE_ACT_LINEAR) return;
#pragma omp parallel for schedule(static)
    for (long i = 0; i < n; i++)
        rdelta[i] = act_d1(act, zin[i], zout[i]) * rdelta[i] +
                    act_d2(act, zin[i], zout[i]) * rzin[i] * delta_in[i];
}

/* ------------------------------------------------------------------------------------ */
/* Pooling: functions/dev_pool.cu                                                        */
/* ------------------------------------------------------------------------------------ */

/* :41-121 (window start (k-1)*stride + ksize - 2*pad, :55,94) */
void ora_pool_forward(const double *in, int N, int C, int H, int W, int ks, int stride, int pad,
                      int type, double *out) {
    int Hp = (int)floor((double)(H - ks + 2 * pad) / stride + 1.);
    int Wp = (int)floor((double)(W - ks + 2 * pad) / stride + 1.);
#pragma omp parallel for collapse(2) schedule(static)
    for (int c = 0; c < C; c++)
        for (int n = 0; n < N; n++)
            for (int l = 0; l < Wp; l++)
                for (int k = 0; k < Hp; k++) {
                    int i = (k - 1) * stride + ks - 2 * pad;
                    int j = (l - 1) * stride + ks - 2 * pad;
                    const double *src = in + ((long)c * N + n) * H * W;
                    double val = (type == FITRE_MAX_POOL) ? -DBL_MAX : 0.0;
                    for (int r = 0; r < ks; r++)
                        for (int cc = 0; cc < ks; cc++) {
                            int fr = i + r, fc = j + cc;
                            if (fr < 0 || fc < 0 || fr >= H || fc >= W) continue;
                            double t = src[(long)fc * H + fr];
                            if (type == FITRE_MAX_POOL) {
                                if (t > val) val = t;
                            } else
                                val += t;
                        }
                    if (type != FITRE_MAX_POOL) val = val / (ks * ks);
                    out[((long)c * N + n) * Hp * Wp + (long)l * Hp + k] = val;
                }
}

/* arg-max flat index into the activation tensor per pooled cell, scan order of the
 * backward kernel (:374-391: column outer, row inner, strict >). */
void ora_max_pool_argmax(const double *act, int N, int C, int H, int W, int ks, int stride,
                         int pad, int *argmax) {
    int Hp = (int)floor((double)(H - ks + 2 * pad) / stride + 1.);
    int Wp = (int)floor((double)(W - ks + 2 * pad) / stride + 1.);
#pragma omp parallel for collapse(2) schedule(static)
    for (int c = 0; c < C; c++)
        for (int n = 0; n < N; n++)
            for (int l = 0; l < Wp; l++)
                for (int k = 0; k < Hp; k++) {
                    int i = (k - 1) * stride + ks - 2 * pad;
                    int j = (l - 1) * stride + ks - 2 * pad;
                    long base = ((long)c * N + n) * H * W;
                    double mv = -DBL_MAX;
                    long mi = -1;
                    for (int cc = 0; cc < ks; cc++)
                        for (int r = 0; r < ks; r++) {
                            int fc = j + cc, fr = i + r;
                            if (fc < 0 || fc >= W || fr < 0 || fr >= H) continue;
                            long tid = base + (long)fc * H + fr;
                            if (act[tid] > mv) {
                                mv = act[tid];
                                mi = tid;
                            }
                        }
                    argmax[((long)c * N + n) * Hp * Wp + (long)l * Hp + k] = (int)mi;
                }
}

/* :346-398, :474-497 -- scatter delta to the arg-max (sequential adds, so deterministic) */
void ora_max_pool_backward(const double *delta, const double *act, int C, int H, int W, int ks,
                           int stride, int pad, int Hp, int Wp, int N, double *out) {
    long V = (long)C * N * H * W, P = (long)C * N * Hp * Wp;
    int *am = (int *)malloc(sizeof(int) * (size_t)(P > 0 ? P : 1));
    ora_max_pool_argmax(act, N, C, H, W, ks, stride, pad, am);
    memset(out, 0, sizeof(double) * (size_t)V);
    for (long i = 0; i < P; i++)
        if (am[i] >= 0) out[am[i]] += delta[i];
    free(am);
}

/* :269-298 with the 1/k^2 scale of functions/cnn_backward.cu:471-473 folded in.
 * stride == kernel, no padding, square planes (the reference's only form). */
void ora_avg_pool_backward(const double *delta, int Hp, int C, int ks, int N, double *out) {
    int inSize = Hp;
    long n = (long)inSize * inSize * C * N;
    double sc = 1. / (ks * ks);
#pragma omp parallel for schedule(static)
    for (long idx = 0; idx < n; idx++) {
        long plane = (long)inSize * inSize;
        long cn = idx / plane; /* c*N + n */
        long r = idx % plane;
        long sCol = r / inSize, sRow = r % inSize;
        double v = delta[idx] * sc;
        long H = (long)inSize * ks;
        double *dst = out + cn * H * H;
        for (int i = 0; i < ks; i++)
            for (int j = 0; j < ks; j++) dst[(sCol * ks + j) * H + sRow * ks + i] = v;
    }
}

/* :123-174 -- R{pool}: pick rz at the arg-max of z */
void ora_rop_max_pool(const double *rz, const double *zact, int N, int C, int H, int W, int ks,
                      int stride, int pad, double *out) {
    int Hp = (int)floor((double)(H - ks + 2 * pad) / stride + 1.);
    int Wp = (int)floor((double)(W - ks + 2 * pad) / stride + 1.);
    long P = (long)C * N * Hp * Wp;
    int *am = (int *)malloc(sizeof(int) * (size_t)(P > 0 ? P : 1));
    ora_max_pool_argmax(zact, N, C, H, W, ks, stride, pad, am);
#pragma omp parallel for schedule(static)
    for (long i = 0; i < P; i++) out[i] = am[i] >= 0 ? rz[am[i]] : 0.0;
    free(am);
}

/* ------------------------------------------------------------------------------------ */
/* Batch norm: functions/dev_batch_norm.cu                                               */
/* ------------------------------------------------------------------------------------ */

/* per-channel sum of f(idx) over the (N,H,W) block of channel c; all-reduced over ranks */
static void channel_sums(const ORA_ENV *env, int C, long rows, const double *a, const double *b,
                         int mode, const double *p0, const double *p1, double *out) {
    /* mode 0: sum a ; 1: sum a*b ; 2: sum (a-p0[c])^2 ; 3: sum (a-p0[c])*(b-p1[c]) */
#pragma omp parallel for schedule(static)
    for (int c = 0; c < C; c++) {
        const double *ac = a + (long)c * rows;
        const double *bc = b ? b + (long)c * rows : NULL;
        double s = 0.0;
        for (long i = 0; i < rows; i++) {
            switch (mode) {
                case 0: s += ac[i]; break;
                case 1: s += ac[i] * bc[i]; break;
                case 2: s += (ac[i] - p0[c]) * (ac[i] - p0[c]); break;
                default: s += (ac[i] - p0[c]) * (bc[i] - p1[c]); break;
            }
        }
        out[c] = s;
    }
    env_allreduce(env, out, C);
}

/* :263-315, :331-393 -- batch mean, biased variance (two passes), zhat */
void ora_batch_norm_forward(const ORA_ENV *env, const double *in, int H, int W, int C, int N,
                            double *out, double *mean, double *var, double eps) {
    long rows = (long)H * W * N;
    double m = (double)rows * env_world(env);
    channel_sums(env, C, rows, in, NULL, 0, NULL, NULL, mean);
    for (int c = 0; c < C; c++) mean[c] *= 1. / m;
    channel_sums(env, C, rows, in, NULL, 2, mean, NULL, var);
    for (int c = 0; c < C; c++) var[c] *= 1. / m;
#pragma omp parallel for schedule(static)
    for (int c = 0; c < C; c++)
        for (long i = 0; i < rows; i++)
            out[(long)c * rows + i] = (in[(long)c * rows + i] - mean[c]) / sqrt(var[c] + eps);
}

/* :398-466, :550-621, kernel :132-150 */
void ora_batch_norm_backward(const ORA_ENV *env, const double *delta, int H, int W, int C,
                             int N, const double *var, const double *zhat, double eps,
                             double *out) {
    long rows = (long)H * W * N;
    double m = (double)rows * env_world(env);
    double *s1 = xmalloc(C), *s2 = xmalloc(C);
    channel_sums(env, C, rows, delta, NULL, 0, NULL, NULL, s1);
    channel_sums(env, C, rows, delta, zhat, 1, NULL, NULL, s2);
#pragma omp parallel for schedule(static)
    for (int c = 0; c < C; c++)
        for (long i = 0; i < rows; i++) {
            long id = (long)c * rows + i;
            double t = delta[id] * m - s1[c] - s2[c] * zhat[id];
            out[id] = t / (m * sqrt(eps + var[c]));
        }
    free(s1);
    free(s2);
}

/* :637-770 */
void ora_rop_batch_norm_forward(const ORA_ENV *env, const double *z, const double *mean,
                                const double *var, const double *rz_in, double eps, int H,
                                int W, int C, int N, double *rz_out) {
    long rows = (long)H * W * N;
    double m = (double)rows * env_world(env);
    double *rmean = xmalloc(C), *s = xmalloc(C);
    channel_sums(env, C, rows, rz_in, NULL, 0, NULL, NULL, rmean);
    for (int c = 0; c < C; c++) rmean[c] *= 1. / m;
    channel_sums(env, C, rows, z, rz_in, 3, mean, rmean, s);
#pragma omp parallel for schedule(static)
    for (int c = 0; c < C; c++)
        for (long i = 0; i < rows; i++) {
            long id = (long)c * rows + i;
            double first = (rz_in[id] - rmean[c]) / sqrt(eps + var[c]);
            double second = s[c] * (z[id] - mean[c]) / (m * pow(eps + var[c], 1.5));
            rz_out[id] = first - second;
        }
    free(rmean);
    free(s);
}

/* :787-960 (helpers :468-529; kernels :92-128,153-183,207-218) */
void ora_rop_batch_norm_backward(const ORA_ENV *env, const double *z_in, const double *z_out,
                                 const double *rz_in, const double *rz_out, const double *delta,
                                 double *rdelta, double eps, const double *mean,
                                 const double *var, int H, int W, int C, int N) {
    long rows = (long)H * W * N;
    double m = (double)rows * env_world(env);
    double *s1 = xmalloc(C), *s2 = xmalloc(C), *s3 = xmalloc(C), *rmean = xmalloc(C);
    double *rI = xmalloc(C), *d1 = xmalloc(C);
    /* R(II): sum Rdelta, sum delta*zhat, sum (delta*Rzhat + zhat*Rdelta) */
    channel_sums(env, C, rows, rdelta, NULL, 0, NULL, NULL, s1);
    channel_sums(env, C, rows, delta, z_out, 1, NULL, NULL, s2);
    {
        double *t = xmalloc(C);
        channel_sums(env, C, rows, delta, rz_out, 1, NULL, NULL, s3);
        channel_sums(env, C, rows, z_out, rdelta, 1, NULL, NULL, t);
        for (int c = 0; c < C; c++) s3[c] += t[c];
        free(t);
    }
    /* R(I) = -sum[(z-mu)(Rz - mean Rz)] / (m^2 (var+eps)^1.5) */
    channel_sums(env, C, rows, rz_in, NULL, 0, NULL, NULL, rmean);
    for (int c = 0; c < C; c++) rmean[c] *= 1. / m;
    channel_sums(env, C, rows, z_in, rz_in, 3, mean, rmean, rI);
    for (int c = 0; c < C; c++) rI[c] *= -1. / (m * m * pow(eps + var[c], 1.5));
    /* II = m*delta - sum delta - zhat * sum(delta*zhat) */
    channel_sums(env, C, rows, delta, NULL, 0, NULL, NULL, d1);
#pragma omp parallel for schedule(static)
    for (int c = 0; c < C; c++)
        for (long i = 0; i < rows; i++) {
            long id = (long)c * rows + i;
            double rII = rdelta[id] * m - s1[c] - s2[c] * rz_out[id] - s3[c] * z_out[id];
            rII /= m * sqrt(eps + var[c]);
            double II = delta[id] * m - d1[c] - s2[c] * z_out[id];
            rdelta[id] = rII + II * rI[c];
        }
    free(s1); free(s2); free(s3); free(rmean); free(rI); free(d1);
}

/* ------------------------------------------------------------------------------------ */
/* Convolution data gradient: functions/dev_backprop_convolution.cu:60-97,173-247        */
/* ------------------------------------------------------------------------------------ */
void ora_conv_dgrad(const double *delta, int dH, int dW, int dC, const double *filter, int k,
                    int H, int W, int pad, int C, int N, double *out) {
    long R = (long)N * H * W, K2 = (long)dC * k * k;
    double *cols = xmalloc(R * K2);
    double *wperm = xmalloc(K2 * C);
    /* transposed im2col of delta, taps enumerated downwards (:86-95) */
#pragma omp parallel for collapse(2) schedule(static)
    for (int ch = 0; ch < dC; ch++)
        for (int n = 0; n < N; n++)
            for (int col = 0; col < W; col++)
                for (int row = 0; row < H; row++) {
                    long r = (long)n * H * W + (long)col * H + row;
                    const double *src = delta + ((long)ch * N + n) * dH * dW;
                    long q = (long)ch * k * k;
                    for (int c = col + pad; c > col + pad - k; c--)
                        for (int rr = row + pad; rr > row + pad - k; rr--) {
                            int ok = (c < dW) && (c >= 0) && (rr >= 0) && (rr < dH);
                            cols[q * R + r] = ok ? src[(long)c * dH + rr] : 0.0;
                            q++;
                        }
                }
    /* weights [(k*k*C) x dC] -> [(k*k*dC) x C] (:215-217) */
    reshape_matrix(filter, dC, C, k * k, wperm);
    ora_gemm(0, 0, R, C, K2, 1.0, cols, R, wperm, K2, 0.0, out, R);
    free(cols);
    free(wperm);
}

/* ------------------------------------------------------------------------------------ */
/* Softmax cross-entropy: functions/softmax_loss.cu:17-79,141-245,251-299                */
/* ------------------------------------------------------------------------------------ */
double ora_softmax_loss(const ORA_ENV *env, const double *logits, const double *target, int N,
                        int classes, double *probs) {
    int ref = env ? env->ref_softmax : 1;
    double total = 0.0;
    for (int r = 0; r < N; r++) {
        const double *x = logits + (long)r * classes;
        double *p = probs + (long)r * classes;
        double mx = ref ? 0.0 : -DBL_MAX;
        for (int i = 0; i < classes; i++)
            if (mx < x[i]) mx = x[i];
        double s = 0.0;
        for (int i = 0; i < classes; i++) {
            p[i] = exp(x[i] - mx);
            s += p[i];
        }
        for (int i = 0; i < classes; i++) p[i] = p[i] / s + (ref ? 1e-10 : 0.0);
        for (int i = 0; i < classes; i++)
            if ((int)target[r] == i + 1) total += -log(p[i]);
    }
    double buf = total;
    env_allreduce(env, &buf, 1);
    return buf / ((double)N * env_world(env));
}

/* (p - onehot) / N_global : :215-245 */
static void ce_error(const ORA_ENV *env, const double *probs, int N, int classes,
                     const double *target, double *errors) {
    double sc = 1. / ((double)N * env_world(env));
    for (int r = 0; r < N; r++)
        for (int c = 0; c < classes; c++) {
            double v = probs[(long)r * classes + c];
            if ((double)(c + 1) == target[r]) v -= 1.;
            errors[(long)r * classes + c] = v * sc;
        }
}
/* Labels sampled from the model's own distribution (KFAC), then (p - onehot(label)) / N_global.
 * functions/dev_dist_errors.cu:12-50 (inverse CDF: first class whose running sum reaches the
 * uniform; classes+1 if none does), functions/softmax_loss.cu:104-136.  The reference draws the
 * uniforms from a time-seeded cuRAND stream; here they are an input. */
void ora_distribution_errors(const ORA_ENV *env, const double *probs, const double *uniforms,
                             int N, int classes, double *distTarget, double *distError) {
    for (int r = 0; r < N; r++) {
        double c = 0.0;
        distTarget[r] = -1;
        for (int i = 0; i < classes; i++) {
            c += probs[(long)r * classes + i];
            if (c >= uniforms[r]) {
                distTarget[r] = i + 1;
                break;
            }
        }
        if (distTarget[r] == -1) distTarget[r] = classes + 1;
    }
    double sc = 1. / ((double)N * env_world(env));
    for (int r = 0; r < N; r++)
        for (int c = 0; c < classes; c++) {
            double v = probs[(long)r * classes + c];
            if ((double)(c + 1) == distTarget[r]) v -= 1.;
            distError[(long)r * classes + c] = v * sc;
        }
}

/* R{p - y} = p .* (Rz - sum_j p_j Rz_j) / N_global : :251-299 */
static void ce_rop_error(const ORA_ENV *env, const double *rz, const double *probs, int N,
                         int classes, double *rError) {
    double sc = 1. / ((double)N * env_world(env));
    for (int r = 0; r < N; r++) {
        double s = 0.0;
        for (int j = 0; j < classes; j++) s += probs[(long)r * classes + j] * rz[(long)r * classes + j];
        for (int i = 0; i < classes; i++)
            rError[(long)r * classes + i] =
                probs[(long)r * classes + i] * (rz[(long)r * classes + i] - s) * sc;
    }
}

/* ------------------------------------------------------------------------------------ */
/* Forward: functions/cnn_forward.cu:48-382, eval_convolution.cu:52-267,                 */
/* eval_gradient.cu:29-228                                                               */
/* ------------------------------------------------------------------------------------ */
static void add_channel_bias(double *x, const double *b, long rows, int C) {
#pragma omp parallel for schedule(static)
    for (int c = 0; c < C; c++)
        for (long i = 0; i < rows; i++) x[(long)c * rows + i] += b[c];
}
static void add_column_bias(double *x, const double *b, int rows, int cols) {
    for (int j = 0; j < cols; j++)
        for (int i = 0; i < rows; i++) x[(long)j * rows + i] += b[i];
}

static const double *layer_input(const CNN_MODEL *m, const double *batch, const double *z, int l) {
    if (l == 0) return batch;
    return z + m->zOffsets[l] + m->convLayer[l - 1].outputOffset;
}

double ora_cnn_forward(const ORA_ENV *env, const CNN_MODEL *m, const double *batch,
                       const double *labels, const double *weights, int numClasses, double *z,
                       double *probs, double *errors, int n) {
    const int *wO = m->wOffsets, *bO = m->bOffsets, *zO = m->zOffsets;
    for (int l = 0; l < m->cLayers; l++) {
        const CONV_LAYER *c = &m->convLayer[l];
        const POOL_LAYER *p = &m->poolLayer[l];
        const double *in = layer_input(m, batch, z, l);
        double *out = z + zO[l + 1];
        long M = (long)n * c->outHeight * c->outWidth;
        long K = (long)c->kSize * c->kSize * c->inChannels;
        long V = M * c->outChannels;
        double *cols = xmalloc(M * K);
        ora_im2col(in, n, c->inChannels, c->height, c->width, c->kSize, c->padding, c->stride, cols);
        ora_gemm(0, 0, M, c->outChannels, K, 1.0, cols, M, weights + wO[l], K, 0.0, out, M);
        free(cols);
        if (m->bias != 0) add_channel_bias(out, weights + bO[l], M, c->outChannels);
        double *actOut = out + c->activationOffset;
        if (c->batchNorm != FITRE_NO_BATCH_NORM) {
            double *bn = out + c->batchNormOffset;
            double *run_mean = bn + c->runningMeansOffset, *run_var = bn + c->runningVariancesOffset;
            if (env && env->eval_type != FITRE_MODEL_TRAIN && env->eval_type != 0) {
                /* accuracy modes: dataset statistics, nothing updated (dev_batch_norm.cu:386-392) */
                long rows = (long)c->outHeight * c->outWidth * n;
#pragma omp parallel for schedule(static)
                for (int ch = 0; ch < c->outChannels; ch++)
                    for (long i = 0; i < rows; i++)
                        bn[(long)ch * rows + i] =
                            (out[(long)ch * rows + i] - run_mean[ch]) / sqrt(run_var[ch] + BN_EPS);
            } else {
                double *mean = bn + c->meansOffset, *var = bn + c->variancesOffset;
                ora_batch_norm_forward(env, out, c->outHeight, c->outWidth, c->outChannels, n, bn,
                                       mean, var, BN_EPS);
                /* running statistics, momentum 0.9 (dev_batch_norm.cu:307-314): Dscal then Daxpy */
                for (int ch = 0; ch < c->outChannels; ch++) {
                    run_mean[ch] = 0.9 * run_mean[ch];
                    run_var[ch] = 0.9 * run_var[ch];
                    run_mean[ch] += (1. - 0.9) * mean[ch];
                    run_var[ch] += (1. - 0.9) * var[ch];
                }
            }
            memcpy(actOut, bn, sizeof(double) * (size_t)V);
        } else {
            memcpy(actOut, out, sizeof(double) * (size_t)V);
        }
        ora_activation(m->actFuns[l], actOut, V);
        if (p->type != FITRE_NO_POOL)
            ora_pool_forward(actOut, n, c->outChannels, c->outHeight, c->outWidth, p->pSize,
                             p->stride, p->padding, p->type, out + c->poolOffset);
    }
    const CONV_LAYER *lc = &m->convLayer[m->cLayers - 1];
    const POOL_LAYER *lp = &m->poolLayer[m->cLayers - 1];
    conv_to_fc(z + zO[m->cLayers] + lc->outputOffset, lc->outChannels, n, lp->outHeight,
               lp->outWidth);
    int outputOffset = lc->outputOffset;
    for (int l = 0; l < m->lLayers; l++) {
        if (l != 0) outputOffset = 0;
        const FC_LAYER *f = &m->fcLayer[l];
        const double *zin = z + zO[l + m->cLayers] + outputOffset;
        double *out = z + zO[l + 1 + m->cLayers];
        ora_gemm(0, 0, f->out, n, f->in, 1.0, weights + wO[l + m->cLayers], f->out, zin, f->in,
                 0.0, out, f->out);
        if (m->bias != 0) add_column_bias(out, weights + bO[l + m->cLayers], f->out, n);
        memcpy(out + (long)f->out * n, out, sizeof(double) * (size_t)f->out * n);
        ora_activation(f->actFun, out, (long)f->out * n);
    }
    const double *logits = (m->lLayers == 0) ? z + zO[m->cLayers] + lc->outputOffset
                                             : z + zO[m->lLayers + m->cLayers];
    double loss = ora_softmax_loss(env, logits, labels, n, numClasses, probs);
    ce_error(env, probs, n, numClasses, labels, errors);
    return loss;
}

/* ------------------------------------------------------------------------------------ */
/* Backward: functions/cnn_backward.cu:76-857                                            */
/* ------------------------------------------------------------------------------------ */
void ora_cnn_backward(const ORA_ENV *env, const CNN_MODEL *m, const double *batch,
                      const double *weights, const double *z, double *gradient, double *dx,
                      const double *errors, int n) {
    const int *wO = m->wOffsets, *bO = m->bOffsets, *zO = m->zOffsets;
    int cL = m->cLayers, lL = m->lLayers;
    long md = m->maxDeltaSize;
    { /* the first conv layer's errors can be larger than any z block when its input is wide */
        for (int l = 0; l < cL; l++) {
            long v = (long)n * m->convLayer[l].height * m->convLayer[l].width * m->convLayer[l].inChannels;
            if (v > md) md = v;
        }
    }
    double *delta = xmalloc(md), *delta_new = xmalloc(md), *tmp;
    const CONV_LAYER *lc = &m->convLayer[cL - 1];
    const POOL_LAYER *lp = &m->poolLayer[cL - 1];
    int last_out = (lL > 0) ? m->fcLayer[lL - 1].out : 0;
    memcpy(delta, errors, sizeof(double) * (size_t)(lL > 0 ? (long)last_out * n
                              : (long)lc->outChannels * lp->outHeight * lp->outWidth * n));

    for (int f = lL - 1; f >= 0; f--) { /* :111-280 */
        const FC_LAYER *l = &m->fcLayer[f];
        const double *zl = z + zO[f + cL + 1];
        act_backward(l->actFun, delta, zl + (long)l->out * n, zl, (long)l->out * n);
        const double *zin = z + zO[f + cL] + ((f == 0) ? lc->outputOffset : 0);
        ora_gemm(0, 1, l->out, l->in, n, 1.0, delta, l->out, zin, l->in, 0.0,
                 gradient + wO[f + cL], l->out);
        if (m->bias != 0) {
            double *db = gradient + bO[f + cL];
            for (int i = 0; i < l->out; i++) {
                double s = 0.0;
                for (int j = 0; j < n; j++) s += delta[(long)j * l->out + i];
                db[i] = s;
            }
        }
        memcpy(dx + zO[f + cL + 1], delta, sizeof(double) * (size_t)l->out * n);
        ora_gemm(1, 0, l->in, n, l->out, 1.0, weights + wO[f + cL], l->out, delta, l->out, 0.0,
                 delta_new, l->in);
        tmp = delta_new; delta_new = delta; delta = tmp;
    }
    if (lL > 0) fc_to_conv(delta, lc->outChannels, n, lp->outHeight, lp->outWidth); /* :310-326 */

    for (int c = cL - 1; c >= 0; c--) { /* :355-852 */
        const CONV_LAYER *l = &m->convLayer[c];
        const POOL_LAYER *p = &m->poolLayer[c];
        const double *zl = z + zO[c + 1];
        double *dxl = dx + zO[c + 1];
        long V = (long)n * l->activationVolumn;
        long M = (long)p->height * p->width * n;
        switch (p->type) { /* :434-493 */
            case FITRE_MAX_POOL:
                ora_max_pool_backward(delta, zl + l->activationOffset, l->outChannels, p->height,
                                      p->width, p->pSize, p->stride, p->padding, p->outHeight,
                                      p->outWidth, n, delta_new);
                break;
            case FITRE_AVG_POOL:
                ora_avg_pool_backward(delta, p->outHeight, l->outChannels, p->pSize, n, delta_new);
                break;
            default: memcpy(delta_new, delta, sizeof(double) * (size_t)V); break;
        }
        memcpy(dxl, delta_new, sizeof(double) * (size_t)V); /* :513 */
        const double *zin = (l->batchNorm != FITRE_NO_BATCH_NORM) ? zl + l->batchNormOffset : zl;
        act_backward(m->actFuns[c], delta_new, zin, zl + l->activationOffset, V); /* :523-592 */
        memcpy(dxl + l->activationOffset, delta_new, sizeof(double) * (size_t)V); /* :605 */
        if (l->batchNorm != FITRE_NO_BATCH_NORM) { /* :643-659 */
            const double *bn = zl + l->batchNormOffset;
            ora_batch_norm_backward(env, delta_new, l->outHeight, l->outWidth, l->outChannels, n,
                                    bn + l->variancesOffset, bn, BN_EPS, delta);
            memcpy(dxl + l->batchNormOffset, delta, sizeof(double) * (size_t)V);
            memcpy(delta_new, delta, sizeof(double) * (size_t)V);
        }
        if (m->bias != 0) { /* :662-689 */
            double *db = gradient + bO[c];
#pragma omp parallel for schedule(static)
            for (int ch = 0; ch < l->outChannels; ch++) {
                double s = 0.0;
                for (long i = 0; i < M; i++) s += delta_new[(long)ch * M + i];
                db[ch] = s;
            }
        }
        const double *in = layer_input(m, batch, z, c);
        long K = (long)l->kSize * l->kSize * l->inChannels;
        double *cols = xmalloc(M * K);
        ora_im2col(in, n, l->inChannels, l->height, l->width, l->kSize, l->padding, l->stride, cols);
        ora_gemm(1, 0, K, l->outChannels, M, 1.0, cols, M, delta_new, M, 0.0, gradient + wO[c], K);
        free(cols);
        if (c != 0) /* :803-819 */
            ora_conv_dgrad(delta_new, p->height, p->width, l->outChannels, weights + wO[c],
                           l->kSize, l->height, l->width, l->padding, l->inChannels, n, delta);
    }
    free(delta);
    free(delta_new);
}

/* functions/cnn_gradient.cu:12-63 */
double ora_cnn_gradient(const ORA_ENV *env, const CNN_MODEL *m, const double *batch,
                        const double *labels, const double *weights, int numClasses, double *z,
                        double *dx, double *probs, double *errors, double *gradient, int n,
                        double weightDecay) {
    double loss = ora_cnn_forward(env, m, batch, labels, weights, numClasses, z, probs, errors, n);
    ora_cnn_backward(env, m, batch, weights, z, gradient, dx, errors, n);
    env_allreduce(env, gradient, m->pSize);
    axpy(m->pSize, weightDecay, weights, gradient);
    return loss;
}

/* ------------------------------------------------------------------------------------ */
/* R-forward: functions/cnn_hv_forward.cu:53-222, eval_convolution.cu:285-539,           */
/* rop_fc_layer.cu:34-133                                                                */
/* ------------------------------------------------------------------------------------ */
void ora_cnn_rop_forward(const ORA_ENV *env, const CNN_MODEL *m, const double *batch,
                         const double *weights, const double *z, const double *vector,
                         double *rz, int n) {
    const int *wO = m->wOffsets, *bO = m->bOffsets, *zO = m->zOffsets;
    for (int l = 0; l < m->cLayers; l++) {
        const CONV_LAYER *c = &m->convLayer[l];
        const POOL_LAYER *p = &m->poolLayer[l];
        const double *zl = z + zO[l + 1];
        double *rzl = rz + zO[l + 1];
        long M = (long)n * c->outHeight * c->outWidth;
        long K = (long)c->kSize * c->kSize * c->inChannels;
        long V = M * c->outChannels;
        const double *in = layer_input(m, batch, z, l);
        double *cols = xmalloc(M * K);
        ora_im2col(in, n, c->inChannels, c->height, c->width, c->kSize, c->padding, c->stride, cols);
        ora_gemm(0, 0, M, c->outChannels, K, 1.0, cols, M, vector + wO[l], K, 0.0, rzl, M);
        if (l > 0) {
            const double *rin = rz + zO[l] + m->convLayer[l - 1].outputOffset;
            ora_im2col(rin, n, c->inChannels, c->height, c->width, c->kSize, c->padding, c->stride, cols);
            ora_gemm(0, 0, M, c->outChannels, K, 1.0, cols, M, weights + wO[l], K, 1.0, rzl, M);
        }
        free(cols);
        if (m->bias != 0) add_channel_bias(rzl, vector + bO[l], M, c->outChannels);
        double *actOut = rzl + c->activationOffset;
        const double *zin = zl;
        if (c->batchNorm != FITRE_NO_BATCH_NORM) {
            const double *bn = zl + c->batchNormOffset;
            ora_rop_batch_norm_forward(env, zl, bn + c->meansOffset, bn + c->variancesOffset, rzl,
                                       BN_EPS, c->outHeight, c->outWidth, c->outChannels, n,
                                       rzl + c->batchNormOffset);
            memcpy(actOut, rzl + c->batchNormOffset, sizeof(double) * (size_t)V);
            zin = bn;
        } else {
            memcpy(actOut, rzl, sizeof(double) * (size_t)V);
        }
        act_backward(m->actFuns[l], actOut, zin, zl + c->activationOffset, V);
        if (p->type == FITRE_MAX_POOL)
            ora_rop_max_pool(actOut, zl + c->activationOffset, n, c->outChannels, c->outHeight,
                             c->outWidth, p->pSize, p->stride, p->padding, rzl + c->poolOffset);
        else if (p->type == FITRE_AVG_POOL)
            ora_pool_forward(actOut, n, c->outChannels, c->outHeight, c->outWidth, p->pSize,
                             p->stride, p->padding, FITRE_AVG_POOL, rzl + c->poolOffset);
    }
    const CONV_LAYER *lc = &m->convLayer[m->cLayers - 1];
    const POOL_LAYER *lp = &m->poolLayer[m->cLayers - 1];
    conv_to_fc(rz + zO[m->cLayers] + lc->outputOffset, lc->outChannels, n, lp->outHeight,
               lp->outWidth);
    int outputOffset = lc->outputOffset;
    for (int l = 0; l < m->lLayers; l++) {
        if (l > 0) outputOffset = 0;
        const FC_LAYER *f = &m->fcLayer[l];
        const double *zin = z + zO[l + m->cLayers] + outputOffset;
        const double *rzin = rz + zO[l + m->cLayers] + outputOffset;
        const double *z1 = z + zO[l + 1 + m->cLayers];
        double *out = rz + zO[l + 1 + m->cLayers];
        ora_gemm(0, 0, f->out, n, f->in, 1.0, vector + wO[l + m->cLayers], f->out, zin, f->in, 0.0,
                 out, f->out);
        ora_gemm(0, 0, f->out, n, f->in, 1.0, weights + wO[l + m->cLayers], f->out, rzin, f->in,
                 1.0, out, f->out);
        if (m->bias != 0) add_column_bias(out, vector + bO[l + m->cLayers], f->out, n);
        memcpy(out + (long)f->out * n, out, sizeof(double) * (size_t)f->out * n);
        act_backward(f->actFun, out, z1 + (long)f->out * n, z1, (long)f->out * n);
    }
}

/* ------------------------------------------------------------------------------------ */
/* R-backward: functions/cnn_hv_backward.cu:70-912                                       */
/* ------------------------------------------------------------------------------------ */
void ora_cnn_rop_backward(const ORA_ENV *env, const CNN_MODEL *m, const double *batch,
                          const double *weights, const double *z, const double *dx,
                          const double *errors, double *rError, const double *rz,
                          const double *vector, double *hv, int n) {
    const int *wO = m->wOffsets, *bO = m->bOffsets, *zO = m->zOffsets;
    int cL = m->cLayers, lL = m->lLayers;
    const CONV_LAYER *lc = &m->convLayer[cL - 1];
    const POOL_LAYER *lp = &m->poolLayer[cL - 1];
    long md = m->maxDeltaSize;
    for (int l = 0; l < cL; l++) {
        long v = (long)n * m->convLayer[l].height * m->convLayer[l].width * m->convLayer[l].inChannels;
        if (v > md) md = v;
    }
    double *t1 = xmalloc(md), *t2 = xmalloc(md);

    for (int f = lL - 1; f >= 0; f--) { /* :153-395 */
        const FC_LAYER *l = &m->fcLayer[f];
        int outputOffset = (f == 0) ? lc->outputOffset : 0;
        const double *zl = z + zO[cL + f + 1];
        const double *rzl = rz + zO[cL + f + 1];
        long cnt = (long)l->out * n;
        if (l->actFun != FITRE_CNN_ACT_NONE && l->actFun != FITRE_ACT_LINEAR) {
            /* errors entering this activation: loss errors (last layer) or W_{f+1}' dx_{f+1} */
            const double *din = errors;
            if (f != lL - 1) {
                const FC_LAYER *ll = &m->fcLayer[f + 1];
                ora_gemm(1, 0, ll->in, n, ll->out, 1.0, weights + wO[cL + f + 1], ll->out,
                         dx + zO[cL + f + 2], ll->out, 0.0, t1, ll->in);
                din = t1;
            }
            act_rop_backward(l->actFun, rError, din, rzl + cnt, zl + cnt, zl, cnt);
        }
        /* R dW = Rdelta z' + delta Rz' */
        ora_gemm(0, 1, l->out, l->in, n, 1.0, rError, l->out, z + zO[cL + f] + outputOffset,
                 l->in, 0.0, hv + wO[cL + f], l->out);
        ora_gemm(0, 1, l->out, l->in, n, 1.0, dx + zO[cL + f + 1], l->out,
                 rz + zO[cL + f] + outputOffset, l->in, 1.0, hv + wO[cL + f], l->out);
        if (m->bias != 0) {
            double *db = hv + bO[cL + f];
            for (int i = 0; i < l->out; i++) {
                double s = 0.0;
                for (int j = 0; j < n; j++) s += rError[(long)j * l->out + i];
                db[i] = s;
            }
        }
        /* Rdelta <- W' Rdelta + V' delta */
        ora_gemm(1, 0, l->in, n, l->out, 1.0, weights + wO[cL + f], l->out, rError, l->out, 0.0,
                 t2, l->in);
        ora_gemm(1, 0, l->in, n, l->out, 1.0, vector + wO[cL + f], l->out, dx + zO[cL + f + 1],
                 l->out, 1.0, t2, l->in);
        memcpy(rError, t2, sizeof(double) * (size_t)l->in * n);
    }
    if (lL > 0) fc_to_conv(rError, lc->outChannels, n, lp->outHeight, lp->outWidth); /* :414-427 */

    for (int c = cL - 1; c >= 0; c--) { /* :436-907 */
        const CONV_LAYER *l = &m->convLayer[c];
        const POOL_LAYER *p = &m->poolLayer[c];
        const double *zl = z + zO[c + 1], *rzl = rz + zO[c + 1], *dxl = dx + zO[c + 1];
        long V = (long)n * l->activationVolumn;
        long M = (long)p->height * p->width * n;
        long K = (long)l->kSize * l->kSize * l->inChannels;
        if (p->type == FITRE_MAX_POOL) { /* :498-553 */
            ora_max_pool_backward(rError, zl + l->activationOffset, l->outChannels, p->height,
                                  p->width, p->pSize, p->stride, p->padding, p->outHeight,
                                  p->outWidth, n, t1);
            memcpy(rError, t1, sizeof(double) * (size_t)V);
        } else if (p->type == FITRE_AVG_POOL) {
            ora_avg_pool_backward(rError, p->outHeight, l->outChannels, p->pSize, n, t1);
            memcpy(rError, t1, sizeof(double) * (size_t)V);
        }
        int bn = l->batchNorm != FITRE_NO_BATCH_NORM;
        const double *zin = bn ? zl + l->batchNormOffset : zl;
        const double *rzin = bn ? rzl + l->batchNormOffset : rzl;
        act_rop_backward(m->actFuns[c], rError, dxl, rzin, zin, zl + l->activationOffset, V); /* :566-679 */
        if (bn) { /* :693-713 */
            const double *b = zl + l->batchNormOffset;
            ora_rop_batch_norm_backward(env, zl, b, rzl, rzl + l->batchNormOffset,
                                        dxl + l->activationOffset, rError, BN_EPS,
                                        b + l->meansOffset, b + l->variancesOffset, l->outHeight,
                                        l->outWidth, l->outChannels, n);
        }
        const double *dprev = bn ? dxl + l->batchNormOffset : dxl + l->activationOffset;
        double *cols = xmalloc(M * K);
        if (c != 0) { /* :727-761 */
            ora_im2col(rz + zO[c] + m->convLayer[c - 1].outputOffset, n, l->inChannels, l->height,
                       l->width, l->kSize, l->padding, l->stride, cols);
            ora_gemm(1, 0, K, l->outChannels, M, 1.0, cols, M, dprev, M, 0.0, hv + wO[c], K);
        } else {
            memset(hv + wO[c], 0, sizeof(double) * (size_t)(K * l->outChannels));
        }
        ora_im2col(layer_input(m, batch, z, c), n, l->inChannels, l->height, l->width, l->kSize,
                   l->padding, l->stride, cols);
        ora_gemm(1, 0, K, l->outChannels, M, 1.0, cols, M, rError, M, 1.0, hv + wO[c], K); /* :776-803 */
        free(cols);
        if (m->bias != 0) { /* :821-834 */
            double *db = hv + bO[c];
#pragma omp parallel for schedule(static)
            for (int ch = 0; ch < l->outChannels; ch++) {
                double s = 0.0;
                for (long i = 0; i < M; i++) s += rError[(long)ch * M + i];
                db[ch] = s;
            }
        }
        if (c != 0) { /* :854-898 */
            long R = (long)l->height * l->width * l->inChannels * n;
            ora_conv_dgrad(rError, p->height, p->width, l->outChannels, weights + wO[c], l->kSize,
                           l->height, l->width, l->padding, l->inChannels, n, t1);
            ora_conv_dgrad(dprev, p->height, p->width, l->outChannels, vector + wO[c], l->kSize,
                           l->height, l->width, l->padding, l->inChannels, n, rError);
            axpy(R, 1.0, t1, rError);
        }
    }
    free(t1);
    free(t2);
}

/* functions/cnn_hessian_vec.cu:18-122.  `rz` (zSize) is caller scratch. */
void ora_cnn_hv(const ORA_ENV *env, const CNN_MODEL *m, const double *batch,
                const double *weights, int numClasses, const double *z, const double *probs,
                const double *errors, const double *dx, const double *vector, double *hv,
                double *rz, int n) {
    long md = m->maxDeltaSize;
    for (int l = 0; l < m->cLayers; l++) {
        long v = (long)n * m->convLayer[l].height * m->convLayer[l].width * m->convLayer[l].inChannels;
        if (v > md) md = v;
    }
    double *rError = xmalloc(md);
    ora_cnn_rop_forward(env, m, batch, weights, z, vector, rz, n);
    const double *logitsR;
    if (m->lLayers == 0)
        logitsR = rz + m->zOffsets[m->cLayers] + m->convLayer[m->cLayers - 1].outputOffset;
    else
        logitsR = rz + m->zOffsets[m->cLayers + m->lLayers];
    ce_rop_error(env, logitsR, probs, n, numClasses, rError);
    ora_cnn_rop_backward(env, m, batch, weights, z, dx, errors, rError, rz, vector, hv, n);
    env_allreduce(env, hv, m->pSize);
    free(rError);
}

/* functions/model_reduction.cu:20-93.  The term added to Hv is weightDecay * weights as the C
 * reference has it (:50-52) when env->ref_quadratic is set (NULL env: set), else
 * weightDecay * vector (the PyTorch twin, pytorch/peng/utils.py:77). */
double ora_quadratic_model(const ORA_ENV *env, const CNN_MODEL *m, const double *batch,
                           const double *weights, int numClasses, const double *z,
                           const double *probs, const double *errors, const double *dx,
                           const double *gradient, double *vector, double delta, int n,
                           double weightDecay) {
    long P = m->pSize;
    double *hv = xmalloc(P), *rz = xmalloc(m->zSize);
    ora_cnn_hv(env, m, batch, weights, numClasses, z, probs, errors, dx, vector, hv, rz, n);
    axpy(P, weightDecay, (!env || env->ref_quadratic) ? weights : vector, hv);
    double vHv = dot(P, hv, vector);
    double nrm = sqrt(dot(P, vector, vector));
    double gv = dot(P, gradient, vector);
    double alpha, val;
    if (vHv < 0) {
        alpha = delta / nrm;
        val = 0.5 * vHv * alpha * alpha - gv * alpha;
    } else {
        double step = gv / (vHv + 1e-6);
        double lim = delta / (nrm + 1e-16);
        alpha = step < lim ? step : lim;
        val = vHv * 0.5 * alpha * alpha - gv * alpha;
    }
    for (long i = 0; i < P; i++) vector[i] *= alpha;
    free(hv);
    free(rz);
    return val;
}

/* Steihaug-CG for min g'p + 0.5 p'Hp, ||p|| <= delta.  Algorithm: solvers/cg_steihaug.c:28-260;
 * constants (the 1e-6 guards, ||r||^2 < tol test) follow its CNN twin
 * pytorch/peng/utils.py:104-165, which is what the reference runs on CNNs. */
void ora_cg_steihaug(const ORA_ENV *env, const CNN_MODEL *m, const double *batch,
                     const double *weights, int numClasses, const double *z,
                     const double *probs, const double *errors, const double *dx,
                     const double *gradient, double *p, int n, FITRE_CG_PARAMS *prm) {
    long P = m->pSize;
    double *zs = xmalloc(P), *rs = xmalloc(P), *ds = xmalloc(P), *Hd = xmalloc(P);
    double *rz = xmalloc(m->zSize), *zn = xmalloc(P);
    double delta = prm->delta, wd = prm->weightDecay;
    for (long i = 0; i < P; i++) {
        zs[i] = 0.0;
        rs[i] = gradient[i];
        ds[i] = -gradient[i];
    }
    int flag = FITRE_CG_MAX_ITERS, it = 0, hvc = 0, done = 0;
    for (it = 0; it < prm->maxIterations; it++) {
        ora_cnn_hv(env, m, batch, weights, numClasses, z, probs, errors, dx, ds, Hd, rz, n);
        hvc++;
        axpy(P, wd, ds, Hd);
        double dHd = dot(P, Hd, ds);
        if (dHd <= 0.0) {
            double ac = dot(P, ds, ds), bc = 2 * dot(P, zs, ds), cc = dot(P, zs, zs) - delta * delta;
            double tau = (-bc + sqrt(bc * bc - 4 * ac * cc)) / (2 * ac + 1e-6);
            for (long i = 0; i < P; i++) p[i] = zs[i] + tau * ds[i];
            flag = FITRE_CG_NEG_CURVATURE;
            done = 1;
            break;
        }
        double rr = dot(P, rs, rs);
        double alpha = rr / (dHd + 1e-6);
        for (long i = 0; i < P; i++) zn[i] = zs[i] + alpha * ds[i];
        if (sqrt(dot(P, zn, zn)) >= delta) {
            double ac = dot(P, ds, ds), bc = 2 * dot(P, zs, ds), cc = dot(P, zs, zs) - delta * delta;
            double tau = (-bc + sqrt(bc * bc - 4 * ac * cc)) / (2 * ac + 1e-6);
            for (long i = 0; i < P; i++) p[i] = zs[i] + tau * ds[i];
            flag = FITRE_CG_HIT_BOUNDARY;
            done = 1;
            break;
        }
        memcpy(zs, zn, sizeof(double) * (size_t)P);
        axpy(P, alpha, Hd, rs);
        double rn = dot(P, rs, rs);
        if (rn < prm->tolerance) {
            memcpy(p, zs, sizeof(double) * (size_t)P);
            flag = FITRE_CG_CONVERGED;
            done = 1;
            break;
        }
        double beta = rn / (rr + 1e-6);
        for (long i = 0; i < P; i++) ds[i] = -rs[i] + beta * ds[i];
    }
    /* pytorch/peng/utils.py:156-158: an exit taken on the very last iteration is also
     * reported as "Maximum Iterations" and returns the last accepted iterate. */
    if (!done) it = prm->maxIterations - 1;
    if (it == prm->maxIterations - 1) {
        memcpy(p, zs, sizeof(double) * (size_t)P);
        flag = FITRE_CG_MAX_ITERS;
    }
    ora_cnn_hv(env, m, batch, weights, numClasses, z, probs, errors, dx, p, Hd, rz, n);
    hvc++;
    prm->modelValue = 0.5 * dot(P, Hd, p) + dot(P, p, gradient) + 0.5 * wd * dot(P, p, p);
    prm->iterations = it + 1;
    prm->flag = flag;
    prm->hvCalls = hvc;
    free(zs); free(rs); free(ds); free(Hd); free(rz); free(zn);
}

/* ------------------------------------------------------------------------------------ */
/* KFAC factors: solvers/kfac_utils.cu:7-55, kfac_inverses.cu:450-630,759-857            */
/* ------------------------------------------------------------------------------------ */
int ora_kfac_storage_indices(const CNN_MODEL *m, FITRE_KFAC_INFO *info) {
    for (int i = 0; i < FITRE_MAX_LAYERS; i++) info->OmegaZOffsets[i] = info->LambdaGOffsets[i] = 0;
    long o = 0, g = 0;
    for (int i = 0; i < m->cLayers; i++) {
        long K = (long)m->convLayer[i].inChannels * m->convLayer[i].kSize * m->convLayer[i].kSize;
        o += (K + 1) * (K + 1);
        g += (long)m->convLayer[i].outChannels * m->convLayer[i].outChannels;
        if (o > INT_MAX || g > INT_MAX) return 2;
        info->OmegaZOffsets[i + 1] = (int)o;
        info->LambdaGOffsets[i + 1] = (int)g;
    }
    for (int i = 0; i < m->lLayers; i++) {
        long in = m->fcLayer[i].in, out = m->fcLayer[i].out;
        o += (in + 1) * (in + 1);
        g += out * out;
        if (o > INT_MAX || g > INT_MAX) return 2;
        info->OmegaZOffsets[m->cLayers + i + 1] = (int)o;
        info->LambdaGOffsets[m->cLayers + i + 1] = (int)g;
    }
    info->OmegaZSize = (int)o;
    info->LambdaGSize = (int)g;
    return 0;
}

/* A factors, undamped: conv (1/N) P~'P~ with P~ = [im2col(X)/(Ho*Wo), 1] (:515-540);
 * FC (1/N) z~ z~' with z~ = [z; 1] (:592-622).  N is the global batch. */
static void omega_z_impl(const ORA_ENV *env, const CNN_MODEL *m, const double *batch, const double *z,
                         int packed, int n, double *omegaZ, const FITRE_KFAC_INFO *info);
void ora_kfac_omega_z(const ORA_ENV *env, const CNN_MODEL *m, const double *batch,
                      const double *z, int n, double *omegaZ, const FITRE_KFAC_INFO *info) {
    omega_z_impl(env, m, batch, z, 0, n, omegaZ, info);
}
/* packed != 0: inputs are the running averages of the speed-up variant, layer l reading
 * dampedZ + zztOffsets[l] (solvers/kfac_inverses.cu:479-489,553-575) */
void ora_kfac_omega_z_damped(const ORA_ENV *env, const CNN_MODEL *m, const double *dampedInput,
                             const double *dampedZ, int n, double *omegaZ, const FITRE_KFAC_INFO *info) {
    omega_z_impl(env, m, dampedInput, dampedZ, 1, n, omegaZ, info);
}
static void omega_z_impl(const ORA_ENV *env, const CNN_MODEL *m, const double *batch, const double *z,
                         int packed, int n, double *omegaZ, const FITRE_KFAC_INFO *info) {
    double Ng = (double)n * env_world(env);
    for (int l = 0; l < m->cLayers; l++) {
        const CONV_LAYER *c = &m->convLayer[l];
        long M = (long)n * c->outHeight * c->outWidth;
        long K = (long)c->inChannels * c->kSize * c->kSize;
        long Kb = K + (m->bias != 0 ? 1 : 0);
        double *cols = xmalloc(M * Kb);
        const double *xin = (packed && l > 0) ? z + m->zztOffsets[l] : layer_input(m, batch, z, l);
        ora_im2col(xin, n, c->inChannels, c->height, c->width, c->kSize, c->padding, c->stride, cols);
        double sc = 1. / (double)(c->outHeight * c->outWidth);
        for (long i = 0; i < M * K; i++) cols[i] *= sc;
        if (m->bias != 0)
            for (long i = 0; i < M; i++) cols[K * M + i] = 1.0;
        double *A = omegaZ + info->OmegaZOffsets[l];
        ora_gemm(1, 0, Kb, Kb, M, 1.0, cols, M, cols, M, 0.0, A, Kb);
        env_allreduce(env, A, Kb * Kb);
        for (long i = 0; i < Kb * Kb; i++) A[i] *= 1. / Ng;
        free(cols);
    }
    const CONV_LAYER *lc = &m->convLayer[m->cLayers - 1];
    for (int l = 0; l < m->lLayers; l++) {
        const FC_LAYER *f = &m->fcLayer[l];
        const double *zin = packed ? z + m->zztOffsets[m->cLayers + l]
                                   : z + m->zOffsets[m->cLayers + l] + (l == 0 ? lc->outputOffset : 0);
        long R = f->in + (m->bias != 0 ? 1 : 0);
        double *zm = xmalloc(R * n);
        for (int j = 0; j < n; j++) {
            memcpy(zm + (long)j * R, zin + (long)j * f->in, sizeof(double) * (size_t)f->in);
            if (m->bias != 0) zm[(long)j * R + f->in] = 1.0;
        }
        double *A = omegaZ + info->OmegaZOffsets[m->cLayers + l];
        ora_gemm(0, 1, R, R, n, 1.0, zm, R, zm, R, 0.0, A, R);
        env_allreduce(env, A, R * R);
        for (long i = 0; i < R * R; i++) A[i] *= 1. / Ng;
        free(zm);
    }
}

/* G factors, undamped: conv (N*Ho*Wo) d'd (:808-816), FC N d d' (:839-849). */
static void lambda_delta_impl(const ORA_ENV *env, const CNN_MODEL *m, const double *dx, int packed, int n,
                              double *lambdaG, const FITRE_KFAC_INFO *info);
void ora_kfac_lambda_delta(const ORA_ENV *env, const CNN_MODEL *m, const double *dx, int n,
                           double *lambdaG, const FITRE_KFAC_INFO *info) {
    lambda_delta_impl(env, m, dx, 0, n, lambdaG, info);
}
void ora_kfac_lambda_delta_damped(const ORA_ENV *env, const CNN_MODEL *m, const double *dampedLambda, int n,
                                  double *lambdaG, const FITRE_KFAC_INFO *info) {
    lambda_delta_impl(env, m, dampedLambda, 1, n, lambdaG, info);
}
static void lambda_delta_impl(const ORA_ENV *env, const CNN_MODEL *m, const double *dx, int packed, int n,
                              double *lambdaG, const FITRE_KFAC_INFO *info) {
    double Ng = (double)n * env_world(env);
    for (int l = 0; l < m->cLayers; l++) {
        const CONV_LAYER *c = &m->convLayer[l];
        const double *d = packed ? dx + m->zztOffsets[l + 1]
                                 : dx + m->zOffsets[l + 1] + (c->batchNorm == FITRE_NO_BATCH_NORM
                                                                  ? c->activationOffset : c->batchNormOffset);
        long M = (long)n * c->outHeight * c->outWidth;
        double *G = lambdaG + info->LambdaGOffsets[l];
        ora_gemm(1, 0, c->outChannels, c->outChannels, M, 1.0, d, M, d, M, 0.0, G, c->outChannels);
        env_allreduce(env, G, (long)c->outChannels * c->outChannels);
        double sc = (double)c->outHeight * c->outWidth * Ng;
        for (long i = 0; i < (long)c->outChannels * c->outChannels; i++) G[i] *= sc;
    }
    for (int l = 0; l < m->lLayers; l++) {
        const FC_LAYER *f = &m->fcLayer[l];
        const double *d = packed ? dx + m->zztOffsets[m->cLayers + l + 1] : dx + m->zOffsets[m->cLayers + l + 1];
        double *G = lambdaG + info->LambdaGOffsets[m->cLayers + l];
        ora_gemm(0, 1, f->out, f->out, n, 1.0, d, f->out, d, f->out, 0.0, G, f->out);
        env_allreduce(env, G, (long)f->out * f->out);
        for (long i = 0; i < (long)f->out * f->out; i++) G[i] *= Ng;
    }
}

/* solvers/kfac_inverses.cu:106-126 (updateRunningStats): theta *= m/(1-m); theta += update;
 * theta *= 1-m; momentum 0 copies. */
void ora_update_running_stats(double *src, const double *update, long n, double momentum) {
    if (momentum != 0) {
        double a = momentum / (1. - momentum), b = 1. - momentum;
        for (long i = 0; i < n; i++) src[i] = (src[i] * a + update[i]) * b;
    } else {
        memcpy(src, update, sizeof(double) * (size_t)n);
    }
}
static void running_or_copy(double *dst, const double *src, long n, double mom, int first) {
    if (first) memcpy(dst, src, sizeof(double) * (size_t)n);
    else ora_update_running_stats(dst, src, n, mom);
}
/* :386-447 (computeSpeedUpOmegaZ): running averages of the batch and of every layer's output */
void ora_kfac_speedup_omega_z(const FITRE_KFAC_INFO *info, const CNN_MODEL *m, const double *batch, long features,
                              int n, const double *z, double *dampedInput, double *dampedZ, int iterCount) {
    double mom = sqrt(info->stats_decay);
    int first = iterCount == 0;
    running_or_copy(dampedInput, batch, features * n, mom, first);
    for (int l = 0; l < m->cLayers; l++) {
        const CONV_LAYER *c = &m->convLayer[l];
        const POOL_LAYER *p = &m->poolLayer[l];
        long vol = (p->type == FITRE_NO_POOL ? (long)c->outHeight * c->outWidth : (long)p->outHeight * p->outWidth) *
                   c->outChannels * n;
        running_or_copy(dampedZ + m->zztOffsets[l + 1], z + m->zOffsets[l + 1] + c->outputOffset, vol, mom, first);
    }
    for (int l = 0; l < m->lLayers; l++)
        running_or_copy(dampedZ + m->zztOffsets[l + 1 + m->cLayers], z + m->zOffsets[l + 1 + m->cLayers],
                        (long)m->fcLayer[l].out * n, mom, first);
}
/* :699-755 (computeSpeedUpLambdaDelta): running averages of every layer's errors */
void ora_kfac_speedup_lambda_delta(const FITRE_KFAC_INFO *info, const CNN_MODEL *m, int n, const double *dx,
                                   double *dampedLambda, int iterCount) {
    double mom = sqrt(info->stats_decay);
    int first = iterCount == 0;
    for (int l = 0; l < m->cLayers; l++) {
        const CONV_LAYER *c = &m->convLayer[l];
        const double *delta = dx + m->zOffsets[l + 1] +
                              (c->batchNorm == FITRE_NO_BATCH_NORM ? c->activationOffset : c->batchNormOffset);
        running_or_copy(dampedLambda + m->zztOffsets[l + 1], delta,
                        (long)c->outChannels * c->outHeight * c->outWidth * n, mom, first);
    }
    for (int l = 0; l < m->lLayers; l++)
        running_or_copy(dampedLambda + m->zztOffsets[l + 1 + m->cLayers], dx + m->zOffsets[l + 1 + m->cLayers],
                        (long)m->fcLayer[l].out * n, mom, first);
}

/* inverse = (matrix + (lambda + gamma) I)^-1 by Cholesky factorisation and two triangular solves
 * against the identity: solvers/kfac_inverses.cu:133-186 (cusolverDnDpotrf + cusolverDnDpotrs).
 * Returns 0, or 1 + the column of a non-positive pivot. */
int ora_kfac_matrix_inverse(const double *matrix, double *inverse, int n, double lambda,
                            double gamma) {
    long nn = (long)n * n;
    double *L = xmalloc(nn);
    memcpy(L, matrix, sizeof(double) * (size_t)nn);
    for (int i = 0; i < n; i++) L[(long)i * n + i] += lambda + gamma;
    for (int j = 0; j < n; j++) { /* column-major lower Cholesky, left-looking */
        double d = L[(long)j * n + j];
        for (int k = 0; k < j; k++) d -= L[(long)k * n + j] * L[(long)k * n + j];
        if (!(d > 0)) {
            free(L);
            return j + 1;
        }
        d = sqrt(d);
        L[(long)j * n + j] = d;
#pragma omp parallel for schedule(static)
        for (int i = j + 1; i < n; i++) {
            double s = L[(long)j * n + i];
            for (int k = 0; k < j; k++) s -= L[(long)k * n + i] * L[(long)k * n + j];
            L[(long)j * n + i] = s / d;
        }
    }
#pragma omp parallel for schedule(dynamic)
    for (int c = 0; c < n; c++) { /* solve L L' x = e_c */
        double *x = inverse + (long)c * n;
        for (int i = 0; i < n; i++) x[i] = (i == c) ? 1.0 : 0.0;
        for (int i = c; i < n; i++) {
            double s = x[i];
            for (int k = c; k < i; k++) s -= L[(long)k * n + i] * x[k];
            x[i] = s / L[(long)i * n + i];
        }
        for (int i = n - 1; i >= 0; i--) {
            double s = x[i];
            for (int k = i + 1; k < n; k++) s -= L[(long)i * n + k] * x[k];
            x[i] = s / L[(long)i * n + i];
        }
    }
    free(L);
    return 0;
}

/* nGradient = G^-1 [W|b] A^-1 per layer in the flat gradient layout:
 * solvers/kfac_natural_gradient.cu:36-241. */
void ora_natural_gradient(const CNN_MODEL *m, const FITRE_KFAC_INFO *info, const double *omegaZInv,
                          const double *lambdaGInv, const double *gradient, double *nGradient) {
    int hasb = m->bias != 0;
    for (int c = 0; c < m->cLayers; c++) {
        const CONV_LAYER *L = &m->convLayer[c];
        long K = (long)L->inChannels * L->kSize * L->kSize, Kb = K + hasb, Co = L->outChannels;
        const double *Ai = omegaZInv + info->OmegaZOffsets[c], *Gi = lambdaGInv + info->LambdaGOffsets[c];
        double *wb = xmalloc(Kb * Co), *t1 = xmalloc(Kb * Co), *t2 = xmalloc(Kb * Co);
        for (long o = 0; o < Co; o++) {
            memcpy(wb + o * Kb, gradient + m->wOffsets[c] + o * K, sizeof(double) * (size_t)K);
            if (hasb) wb[o * Kb + K] = gradient[m->bOffsets[c] + o];
        }
        ora_gemm(0, 1, Co, Kb, Co, 1.0, Gi, Co, wb, Kb, 0.0, t1, Co);
        ora_gemm(0, 0, Co, Kb, Kb, 1.0, t1, Co, Ai, Kb, 0.0, t2, Co);
        for (long o = 0; o < Co; o++) {
            for (long r = 0; r < K; r++) nGradient[m->wOffsets[c] + o * K + r] = t2[o + r * Co];
            if (hasb) nGradient[m->bOffsets[c] + o] = t2[o + K * Co];
        }
        free(wb); free(t1); free(t2);
    }
    for (int l = 0; l < m->lLayers; l++) {
        const FC_LAYER *F = &m->fcLayer[l];
        int li = m->cLayers + l;
        long in = F->in + hasb;
        const double *Ai = omegaZInv + info->OmegaZOffsets[li], *Gi = lambdaGInv + info->LambdaGOffsets[li];
        double *t = xmalloc((long)F->out * in);
        ora_gemm(0, 0, F->out, in, F->out, 1.0, Gi, F->out, gradient + m->wOffsets[li], F->out, 0.0, t, F->out);
        ora_gemm(0, 0, F->out, in, in, 1.0, t, F->out, Ai, in, 0.0, nGradient + m->wOffsets[li], F->out);
        free(t);
    }
}

/* ------------------------------------------------------------------------------------ */
/* Evaluation pass and input pipeline                                                     */
/* ------------------------------------------------------------------------------------ */

/* solvers/kfac_trust_region.cu:66-77 with functions/dev_batch_norm.cu:235-255: running mean 0,
 * running variance 1 for every batch-normalised layer. */
void ora_init_batch_norm_data(const CNN_MODEL *m, double *z) {
    for (int l = 0; l < m->cLayers; l++) {
        const CONV_LAYER *c = &m->convLayer[l];
        if (c->batchNorm == FITRE_NO_BATCH_NORM) continue;
        double *bn = z + m->zOffsets[l + 1] + c->batchNormOffset;
        for (int ch = 0; ch < c->outChannels; ch++) {
            bn[c->runningMeansOffset + ch] = 0.;
            bn[c->runningVariancesOffset + ch] = 1.;
        }
    }
}

/* functions/cnn_accuracy.cu:16-59: predicted class = first class whose probability strictly
 * exceeds the running maximum (which starts at 0); a hit when class + 1 equals the label.
 * Returns the percentage over the (global) batch, *hits_out the hit count. */
double ora_compute_accuracy(const ORA_ENV *env, const double *probs, const double *target, int rows,
                            int classes, double *hits_out) {
    double hits = 0;
    for (int i = 0; i < rows; i++) {
        double best = 0;
        int cls = 0;
        for (int c = 0; c < classes; c++)
            if (best < probs[(long)i * classes + c]) {
                best = probs[(long)i * classes + c];
                cls = c;
            }
        if ((double)(cls + 1) == target[i]) hits += 1;
    }
    env_allreduce(env, &hits, 1);
    if (hits_out) *hits_out = hits;
    return hits * 100. / ((double)rows * env_world(env));
}

/* Minibatch assembly: utilities/sample_matrix.cu:70-92 (column gather of images and labels),
 * solvers/kfac_da.cu:22-89 (per-image [C][W][H] -> batch [C][N][W][H]; with augmentation: random
 * crop with padding 4 then random horizontal flip), augmentation/dev_crop.cu:14-62 (shift =
 * trunc(u*100) % 9 - 4 per axis, zero outside), augmentation/dev_flip.cu:61-92 (mirror the
 * columns when u < 0.5), augmentation/dev_normalize.cu:12-100 (v/255, minus mean, over std).
 * `indices` NULL = images offset .. offset+n-1; `uniforms` NULL = no augmentation, else
 * [row shifts n][column shifts n][flip n] in [0,1). */
static const double k_norm_mean[3][3] = {{0.4914, 0.4822, 0.4465}, {0.5071, 0.4865, 0.4409},
                                         {0.4799, 0.4478, 0.3972}};
static const double k_norm_std[3][3] = {{0.2470, 0.2435, 0.2616}, {0.2673, 0.2564, 0.2762},
                                        {0.2769, 0.2690, 0.2820}};

void ora_prepare_minibatch(const double *setX, const double *setY, const int *indices, long offset,
                           int n, int C, int H, int W, int datasetType, const double *uniforms,
                           double *batch, double *labels) {
    const long plane = (long)H * W, feat = plane * C;
    /* DATASET_TYPE: CIFAR10 = 10, CIFAR100 = 20, IMAGENET = 30 (core/structdefs.h:17-21) */
    const int di = datasetType == 20 ? 1 : datasetType == 30 ? 2 : 0;
    const double *mean = k_norm_mean[di], *sd = k_norm_std[di];
    for (int im = 0; im < n; im++) {
        const long src = indices ? indices[offset + im] : offset + im;
        labels[im] = setY[src];
        int dr = 0, dc = 0, flip = 0;
        if (uniforms) {
            dr = (int)(uniforms[im] * 100.) % 9 - 4;
            dc = (int)(uniforms[n + im] * 100.) % 9 - 4;
            flip = uniforms[2 * n + im] < 0.5;
        }
        for (int c = 0; c < C; c++)
            for (int col = 0; col < W; col++)
                for (int row = 0; row < H; row++) {
                    /* flipped output column col holds cropped column W-1-col */
                    const int ccol = flip ? W - 1 - col : col;
                    const int sr = row + dr, sc = ccol + dc;
                    double v = 0.;
                    if (sr >= 0 && sc >= 0 && sr < H && sc < W)
                        v = setX[src * feat + c * plane + (long)sc * H + sr];
                    v /= 255.;
                    v = (v - mean[c % 3]) / sd[c % 3];
                    batch[((long)c * n + im) * plane + (long)col * H + row] = v;
                }
    }
}

/* functions/cnn_accuracy.cu:61-174: mean loss / accuracy over a whole set in minibatches of
 * model->batchSize with the running batch-norm statistics of `z`.  test != 0: the partial last
 * batch is included; test == 0: the loop leaves before the last batch; both divide by the set
 * size.  A partial batch is run on the same net laid out for that many images, the running
 * statistics carried over (every other part of z is scratch during an evaluation). */
static long move_running_stats(const CNN_MODEL *m, double *z, double *packed, int to_packed) {
    long o = 0;
    for (int l = 0; l < m->cLayers; l++) {
        const CONV_LAYER *c = &m->convLayer[l];
        if (c->batchNorm == FITRE_NO_BATCH_NORM) continue;
        double *bn = z + m->zOffsets[l + 1] + c->batchNormOffset;
        for (int ch = 0; ch < c->outChannels; ch++) {
            if (to_packed) {
                packed[o + ch] = bn[c->runningMeansOffset + ch];
                packed[o + c->outChannels + ch] = bn[c->runningVariancesOffset + ch];
            } else {
                bn[c->runningMeansOffset + ch] = packed[o + ch];
                bn[c->runningVariancesOffset + ch] = packed[o + c->outChannels + ch];
            }
        }
        o += 2L * c->outChannels;
    }
    return o;
}

void ora_generalization_errors(const ORA_ENV *env_in, const CNN_MODEL *m, const double *setX,
                               const double *setY, long size, int datasetType,
                               const double *weights, int numClasses, double *z, int test,
                               double *likelihood, double *accuracy) {
    ORA_ENV env = *env_in;
    env.eval_type = test ? FITRE_MODEL_TEST_ACCURACY : FITRE_MODEL_TRAIN_ACCURACY;
    env.world = 1;
    env.allreduce = NULL;
    const CONV_LAYER *c0 = &m->convLayer[0];
    const int C = c0->inChannels, H = c0->height, W = c0->width, B = m->batchSize;
    const long feat = (long)C * H * W;
    double *batch = xmalloc(feat * B), *labels = xmalloc(B), *probs = xmalloc((long)B * numClasses);
    double *errors = xmalloc((long)B * numClasses), *packed = xmalloc(2L * FITRE_MAX_LAYERS * 4096);
    double lik = 0, hits = 0;
    long cur_idx = 0;
    int cur = B;
    while (cur_idx < size) {
        const CNN_MODEL *mm = m;
        CNN_MODEL tail;
        if (cur != B) {
            tail = *m;
            tail.batchSize = cur;
            ora_model_finalize(&tail);
            move_running_stats(m, z, packed, 1);
            move_running_stats(&tail, z, packed, 0);
            mm = &tail;
        }
        ora_prepare_minibatch(setX, setY, NULL, cur_idx, cur, C, H, W, datasetType, NULL, batch, labels);
        double l = ora_cnn_forward(&env, mm, batch, labels, weights, numClasses, z, probs, errors, cur);
        double h = 0;
        ora_compute_accuracy(&env, probs, labels, cur, numClasses, &h);
        if (cur != B) move_running_stats(m, z, packed, 0);
        lik += l * cur;
        hits += h;
        cur_idx += cur;
        if (cur_idx + B < size) {
            cur = B;
        } else {
            cur = (int)(size - cur_idx);
            if (!test) break;
        }
    }
    *accuracy = hits * 100. / (double)size;
    *likelihood = lik / (double)size;
    free(batch); free(labels); free(probs); free(errors); free(packed);
}

/* solvers/kfac_trust_region.cu:94-661 with inverseFreq == 1.  Random draws: splitmix64 seeded
 * with `seed`, the same stream on every rank; per epoch a Fisher-Yates shuffle of the training
 * indices, per global minibatch of GB = world * B images 4*GB uniforms [row shifts | column
 * shifts | flips | sampled labels], of which rank r uses entries r*B .. r*B+B-1 of each part. */
static unsigned long long sm64_next(unsigned long long *s) {
    unsigned long long z = (*s += 0x9E3779B97F4A7C15ull);
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}

static void layer_block_sizes(const CNN_MODEL *m, int l, int *a, int *g) {
    if (l < m->cLayers) {
        const CONV_LAYER *c = &m->convLayer[l];
        *a = c->inChannels * c->kSize * c->kSize + (m->bias ? 1 : 0);
        *g = c->outChannels;
    } else {
        const FC_LAYER *f = &m->fcLayer[l - m->cLayers];
        *a = f->in + (m->bias ? 1 : 0);
        *g = f->out;
    }
}

int ora_subsampled_trust_region_kfac(const ORA_ENV *env, const CNN_MODEL *m, const double *trainX,
                                     const double *trainY, long trainN, const double *testX,
                                     const double *testY, long testN, int datasetType,
                                     double *weights, int numClasses, FITRE_KFAC_INFO *info,
                                     TRUST_REGION_PARAMS *tr, unsigned long long seed, int enableDA,
                                     int maxMiniBatches, FITRE_TR_STEP *steps, int stepsCap,
                                     FITRE_TR_EPOCH *epochs) {
    ora_kfac_storage_indices(m, info);
    const CONV_LAYER *c0 = &m->convLayer[0];
    const int C = c0->inChannels, H = c0->height, W = c0->width, B = m->batchSize;
    const long feat = (long)C * H * W, P = m->pSize, Z = m->zSize;
    const long md = (m->maxDeltaSize > (long)B * numClasses ? m->maxDeltaSize : (long)B * numClasses) + 32;
    const int layers = m->cLayers + m->lLayers;
    const int Wn = env_world(env), rank = env ? env->rank : 0;
    const long GB = (long)B * Wn;
    double *batch = xmalloc(feat * B), *labels = xmalloc(B), *u = xmalloc(4L * B), *ug = xmalloc(4L * GB);
    double *z = xmalloc(Z), *dx = xmalloc(Z), *distDX = xmalloc(Z);
    double *probs = xmalloc((long)B * numClasses), *errors = xmalloc(md), *dist1 = xmalloc(md);
    double *distTarget = xmalloc(B);
    double *gradient = xmalloc(P), *distGradient = xmalloc(P), *prev = xmalloc(P), *ngrad = xmalloc(P);
    double *A = xmalloc(info->OmegaZSize), *Ai = xmalloc(info->OmegaZSize);
    double *G = xmalloc(info->LambdaGSize), *Gi = xmalloc(info->LambdaGSize);
    int *idx = (int *)malloc(sizeof(int) * (size_t)trainN);
    memset(z, 0, sizeof(double) * (size_t)Z);
    memset(prev, 0, sizeof(double) * (size_t)P);
    ora_init_batch_norm_data(m, z);
    unsigned long long s = seed;
    int step_no = 0, rc = 0, total_mb = 0;
    double *dInput = NULL, *dZ = NULL, *dLambda = NULL;
    if (info->inverseFreq > 1) {
        dInput = xmalloc(feat * B);
        dZ = xmalloc(m->zztSize);
        dLambda = xmalloc(m->zztSize);
    }
    for (int iter = 0; iter < tr->maxIters && rc == 0; iter++) {
        for (long i = 0; i < trainN; i++) idx[i] = (int)i;
        for (long i = trainN - 1; i > 0; i--) {
            long j = (long)(sm64_next(&s) % (unsigned long long)(i + 1));
            int t = idx[i]; idx[i] = idx[j]; idx[j] = t;
        }
        long offset = 0;
        int mb = 0;
        while (offset + GB < trainN && (maxMiniBatches <= 0 || mb < maxMiniBatches)) {
            for (long i = 0; i < 4L * GB; i++) ug[i] = (double)(sm64_next(&s) >> 11) * (1.0 / 9007199254740992.0);
            for (int part = 0; part < 4; part++)
                memcpy(u + (long)part * B, ug + part * GB + (long)rank * B, sizeof(double) * (size_t)B);
            ora_prepare_minibatch(trainX, trainY, idx, offset + (long)rank * B, B, C, H, W, datasetType,
                                  enableDA ? u : NULL, batch, labels);
            double lik = ora_cnn_forward(env, m, batch, labels, weights, numClasses, z, probs, errors, B);
            memcpy(dist1, errors, sizeof(double) * (size_t)B * numClasses);
            ora_cnn_backward(env, m, batch, weights, z, gradient, dx, dist1, B);
            env_allreduce(env, gradient, P);
            axpy(P, info->regLambda, weights, gradient);
            ora_distribution_errors(env, probs, u + 3L * B, B, numClasses, distTarget, dist1);
            ora_cnn_backward(env, m, batch, weights, z, distGradient, distDX, dist1, B);
            /* :392-411: running averages every minibatch; factors and inverses on the very first
             * minibatch from the live state, afterwards every inverseFreq minibatches from the averages */
            int refresh = 1, from_avg = 0;
            if (info->inverseFreq > 1) {
                ora_kfac_speedup_omega_z(info, m, batch, feat, B, z, dInput, dZ, iter + (int)offset);
                ora_kfac_speedup_lambda_delta(info, m, B, distDX, dLambda, iter + (int)offset);
                if (iter == 0 && total_mb == 0) from_avg = 0;
                else if (total_mb % info->inverseFreq == 0) from_avg = 1;
                else refresh = 0;
            }
            if (refresh && from_avg) {
                ora_kfac_omega_z_damped(env, m, dInput, dZ, B, A, info);
                ora_kfac_lambda_delta_damped(env, m, dLambda, B, G, info);
            } else if (refresh) {
                ora_kfac_omega_z(env, m, batch, z, B, A, info);
                ora_kfac_lambda_delta(env, m, distDX, B, G, info);
            }
            for (int l = 0; refresh && l < layers && rc == 0; l++) {
                int a, g;
                layer_block_sizes(m, l, &a, &g);
                rc |= ora_kfac_matrix_inverse(A + info->OmegaZOffsets[l], Ai + info->OmegaZOffsets[l], a,
                                              info->regLambda, info->dampGamma);
                rc |= ora_kfac_matrix_inverse(G + info->LambdaGOffsets[l], Gi + info->LambdaGOffsets[l], g,
                                              info->regLambda, info->dampGamma);
            }
            if (rc) break;
            ora_natural_gradient(m, info, Ai, Gi, gradient, ngrad);
            double mK = ora_quadratic_model(env, m, batch, weights, numClasses, z, probs, errors, dx,
                                            gradient, ngrad, tr->delta, B, info->regLambda);
            double mG = 0;
            if (info->checkGrad)
                mG = ora_quadratic_model(env, m, batch, weights, numClasses, z, probs, errors, dx,
                                         gradient, gradient, tr->delta, B, info->regLambda);
            int use_kfac = !info->checkGrad || mK < mG;
            double *dir = use_kfac ? ngrad : gradient;
            axpy(P, info->momentum, prev, dir);
            axpy(P, -1.0, dir, weights);
            memcpy(prev, dir, sizeof(double) * (size_t)P);
            double nlik = ora_cnn_forward(env, m, batch, labels, weights, numClasses, z, probs, errors, B);
            double hits = 0;
            double acc = ora_compute_accuracy(env, probs, labels, B, numClasses, &hits);
            double rho = (nlik - lik) / ((use_kfac ? mK : mG) - 1e-16);
            if (rho > 0.75) tr->delta = tr->maxDelta < 2. * tr->delta ? tr->maxDelta : 2. * tr->delta;
            if (rho < 0.25) tr->delta = tr->minDelta > 0.5 * tr->delta ? tr->minDelta : 0.5 * tr->delta;
            int reverted = 0;
            if (rho < 1e-4 || nlik > 10. * lik) {
                axpy(P, 1.0, prev, weights);
                reverted = 1;
            }
            if (steps && step_no < stepsCap) {
                FITRE_TR_STEP st = {lik, nlik, acc, mK, mG, rho, tr->delta, use_kfac, reverted};
                steps[step_no] = st;
            }
            step_no++;
            offset += GB;
            mb++;
            total_mb++;
        }
        if (rc) break;
        FITRE_TR_EPOCH ep;
        memset(&ep, 0, sizeof ep);
        ep.miniBatches = mb;
        if (testX && testN > 0)
            ora_generalization_errors(env, m, testX, testY, testN, datasetType, weights, numClasses, z, 1,
                                      &ep.testLikelihood, &ep.testAccuracy);
        ora_generalization_errors(env, m, trainX, trainY, trainN, datasetType, weights, numClasses, z, 0,
                                  &ep.trainLikelihood, &ep.trainAccuracy);
        if (epochs) epochs[iter] = ep;
    }
    tr->curIteration = step_no;
    free(batch); free(labels); free(u); free(ug); free(z); free(dx); free(distDX); free(probs); free(errors);
    free(dist1); free(distTarget); free(gradient); free(distGradient); free(prev); free(ngrad);
    free(A); free(Ai); free(G); free(Gi); free(idx);
    free(dInput); free(dZ); free(dLambda);
    return rc;
}
