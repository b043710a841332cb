// KFAC factor accumulation: A = activation covariance, G = error covariance, per layer.
// Reference: solvers/kfac_utils.cu:7-55 (block offsets), solvers/kfac_inverses.cu:450-630
// (computeOmegaZ) and :759-857 (computeLambdaDelta).  The reference materialises the im2col
// matrix and calls cublasDgemm for the full square; here the convolution A factor is a
// tensor-core SYRK over implicit patches (lower tiles only) and every factor is summed over
// the data-parallel ranks before the 1/N (A) or N (G) scaling with the global batch.
#include <algorithm>
#include <climits>
#include <cmath>
#include <cstring>
#include <string>
#include <vector>

#include <cstdlib>

#include "common.h"
#include "graphs.h"

using namespace fitre;

namespace {
long align32(long n) { return (n + 31) / 32 * 32; }

__global__ void fc_augment_kernel(const double *z, double *out, int in, int n) {
    // out ((in+1) x n) = [z; 1]   (solvers/kfac_inverses.cu:592-606)
    const long total = (long)(in + 1) * n;
    for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < total;
         i += (long)gridDim.x * blockDim.x) {
        const long col = i / (in + 1);
        const int row = (int)(i - col * (in + 1));
        out[i] = row < in ? z[col * in + row] : 1.0;
    }
}
}  // namespace

extern "C" int fitre_kfac_storage_indices(const CNN_MODEL *m, FITRE_KFAC_INFO *info) {
    if (!m || !info) return FITRE_ERR_BAD_ARG;
    for (int i = 0; i < FITRE_MAX_LAYERS; ++i) info->OmegaZOffsets[i] = info->LambdaGOffsets[i] = 0;
    long o = 0, g = 0;
    const int L = m->cLayers + m->lLayers;
    for (int i = 0; i < L; ++i) {
        long a, c;
        if (i < m->cLayers) {
            a = (long)m->convLayer[i].inChannels * m->convLayer[i].kSize * m->convLayer[i].kSize + 1;
            c = m->convLayer[i].outChannels;
        } else {
            a = (long)m->fcLayer[i - m->cLayers].in + 1;
            c = m->fcLayer[i - m->cLayers].out;
        }
        o += a * a;  // the bias row/column is always reserved (solvers/kfac_utils.cu:25-40)
        g += c * c;
        if (o > INT_MAX || g > INT_MAX) return FITRE_ERR_TOO_LARGE;
        info->OmegaZOffsets[i + 1] = (int)o;
        info->LambdaGOffsets[i + 1] = (int)g;
    }
    info->OmegaZSize = (int)o;
    info->LambdaGSize = (int)g;
    return FITRE_OK;
}

extern "C" long fitre_kfac_mem_required(const CNN_MODEL *m) {
    if (!m) return -1;
    long need = 0;
    const int n = m->batchSize;
    for (int l = 0; l < m->cLayers; ++l) {
        const CONV_LAYER &c = m->convLayer[l];
        need = std::max(need, conv_patch_syrk_scratch(n, c.inChannels, c.height, c.width, c.kSize,
                                                      c.padding, m->bias != 0));
        need = std::max(need, syrk_scratch((long)n * c.outHeight * c.outWidth, c.outChannels));
    }
    for (int l = 0; l < m->lLayers; ++l)
        need = std::max(need, (long)(m->fcLayer[l].in + 1) * n);
    return align32(need);
}

extern "C" int fitre_compute_distribution_errors(fitre_context *ctx, const real *probs,
                                                 const real *uniforms, real *distTarget,
                                                 real *distError, int rows, int numClasses) {
    if (!ctx) return FITRE_ERR_BAD_ARG;
    try {
        FITRE_CUDA(cudaSetDevice(ctx->device));
        FITRE_REQUIRE(probs && uniforms && distTarget && distError && rows > 0 && numClasses > 0,
                      FITRE_ERR_BAD_ARG, "bad argument");
        distribution_errors(ctx, probs, uniforms, rows, numClasses, distTarget, distError,
                            1.0 / ((double)rows * ctx->world));
        return FITRE_OK;
    } catch (const Error &e) {
        ctx->err = e.what();
        return e.code;
    }
}

namespace {
// Layer inputs come either from the live state (x0 = the batch, zbase = z with the model's z
// offsets) or, packed == true, from the running averages of the "speed-up" variant (x0 =
// dampedInput, zbase = dampedZ with the model's zzt offsets: solvers/kfac_inverses.cu:479-489,553-575).
// A factor of layer li (convolutions first, then the FC layers), all-reduced when there are ranks
// sum of a factor block over the ranks: on every rank (root < 0) or on `root` only, then the scale
void reduce_block(fitre_context *ctx, double *F, long n, double scale, int root) {
    if (ctx->world <= 1) return;
    if (root < 0) comm_allreduce_sum(ctx, F, (size_t)n);
    else comm_reduce_sum(ctx, F, (size_t)n, root);
    if (root < 0 || root == ctx->rank) vec_scale(ctx, n, scale, F);
}

void omega_z_layer(fitre_context *ctx, const CNN_MODEL *m, const double *x0, const double *zbase, bool packed,
                   int samples, double *omegaZ, const FITRE_KFAC_INFO *info, double *devPtr, int li,
                   int root = -1) {
    const double Ng = (double)samples * ctx->world;
    if (li < m->cLayers) {
        const int l = li;
        const ConvGeom g = conv_geom(m, l);
        const double *x = (l == 0) ? x0
                          : packed ? zbase + m->zztOffsets[l]
                                   : zbase + m->zOffsets[l] + m->convLayer[l - 1].outputOffset;
        double *A = omegaZ + info->OmegaZOffsets[l];
        const int Kb = g.Cin * g.k * g.k + (m->bias ? 1 : 0);
        // sum over ranks first, then 1/N: with world == 1 the scale is applied directly
        const double alpha = ctx->world > 1 ? 1.0 : 1.0 / Ng;
        conv_patch_syrk(ctx, x, A, samples, g.Cin, g.H, g.W, g.k, g.pad, m->bias != 0, alpha,
                        1.0 / (double)(g.Ho * g.Wo), devPtr);
        reduce_block(ctx, A, (long)Kb * Kb, 1.0 / Ng, root);
        return;
    }
    const int l = li - m->cLayers;
    const ConvGeom lg = conv_geom(m, m->cLayers - 1);
    const FC_LAYER &f = m->fcLayer[l];
    const double *zin = packed ? zbase + m->zztOffsets[m->cLayers + l]
                        : (l == 0) ? zbase + lg.zoff + lg.outOff
                                   : zbase + m->zOffsets[m->cLayers + l];
    double *A = omegaZ + info->OmegaZOffsets[m->cLayers + l];
    int R = f.in;
    const double *zm = zin;
    if (m->bias) {
        R = f.in + 1;
        const long total = (long)R * samples;
        int blocks = (int)std::min<long>((total + 255) / 256, 1184);
        fc_augment_kernel<<<blocks, 256, 0, ctx->stream>>>(zin, devPtr, f.in, samples);
        check_launch(ctx, "fc_augment_kernel");
        zm = devPtr;
    }
    dgemm(ctx, false, true, R, R, samples, ctx->world > 1 ? 1.0 : 1.0 / Ng, zm, R, zm, R, 0.0, A, R);
    reduce_block(ctx, A, (long)R * R, 1.0 / Ng, root);
}

void omega_z_impl(fitre_context *ctx, const CNN_MODEL *m, const double *x0, const double *zbase, bool packed,
                  int samples, double *omegaZ, const FITRE_KFAC_INFO *info, double *devPtr) {
    for (int li = 0; li < m->cLayers + m->lLayers; ++li)
        omega_z_layer(ctx, m, x0, zbase, packed, samples, omegaZ, info, devPtr, li);
}

// G factor of layer li (convolutions first, then the FC layers)
void lambda_delta_layer(fitre_context *ctx, const CNN_MODEL *m, const double *dbase, bool packed, int samples,
                        double *lambdaG, const FITRE_KFAC_INFO *info, double *devPtr, int li, int root = -1) {
    const double Ng = (double)samples * ctx->world;
    if (li < m->cLayers) {
        const int l = li;
        const ConvGeom g = conv_geom(m, l);
        const double *d = packed ? dbase + m->zztOffsets[l + 1] : dbase + g.zoff + (g.bn ? g.bnOff : g.actOff);
        const long M = (long)samples * g.Ho * g.Wo;
        double *G = lambdaG + info->LambdaGOffsets[l];
        const double sc = (double)g.Ho * g.Wo * Ng;  // solvers/kfac_inverses.cu:815-816
        syrk_tn(ctx, M, g.Cout, ctx->world > 1 ? 1.0 : sc, d, M, G, devPtr);
        reduce_block(ctx, G, (long)g.Cout * g.Cout, sc, root);
        return;
    }
    const int l = li - m->cLayers;
    const FC_LAYER &f = m->fcLayer[l];
    const double *d = packed ? dbase + m->zztOffsets[m->cLayers + l + 1] : dbase + m->zOffsets[m->cLayers + l + 1];
    double *G = lambdaG + info->LambdaGOffsets[m->cLayers + l];
    dgemm(ctx, false, true, f.out, f.out, samples, ctx->world > 1 ? 1.0 : Ng, d, f.out, d, f.out, 0.0, G, f.out);
    reduce_block(ctx, G, (long)f.out * f.out, Ng, root);
}

void lambda_delta_impl(fitre_context *ctx, const CNN_MODEL *m, const double *dbase, bool packed, int samples,
                       double *lambdaG, const FITRE_KFAC_INFO *info, double *devPtr) {
    for (int li = 0; li < m->cLayers + m->lLayers; ++li)
        lambda_delta_layer(ctx, m, dbase, packed, samples, lambdaG, info, devPtr, li);
}

// theta <- m * theta + (1 - m) * update, in the reference's operation order
// (solvers/kfac_inverses.cu:106-126: scale by m/(1-m), add, scale by 1-m); m == 0 copies.
__global__ void running_stats_kernel(double *theta, const double *update, long n, double mom) {
    const double a = mom / (1. - mom), b = 1. - mom;
    for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < n; i += (long)gridDim.x * blockDim.x)
        theta[i] = (theta[i] * a + update[i]) * b;
}
void update_running(fitre_context *ctx, double *theta, const double *update, long n, double mom, bool first) {
    if (first || mom == 0.0) {
        vec_copy(ctx, n, update, theta);
        return;
    }
    running_stats_kernel<<<(int)std::min<long>((n + 255) / 256, 2368), 256, 0, ctx->stream>>>(theta, update, n, mom);
    check_launch(ctx, "running_stats_kernel");
}
}  // namespace

#define KFAC_ENTRY_BEGIN               \
    if (!ctx) return FITRE_ERR_BAD_ARG; \
    try {                               \
        FITRE_CUDA(cudaSetDevice(ctx->device));
#define KFAC_ENTRY_END       \
    return FITRE_OK;         \
    }                        \
    catch (const Error &e) { \
        ctx->err = e.what(); \
        return e.code;       \
    }

extern "C" int fitre_kfac_omega_z(fitre_context *ctx, const CNN_MODEL *m, const DEVICE_DATASET *data,
                                  const real *z, int samples, real *omegaZ, const FITRE_KFAC_INFO *info,
                                  real *devPtr) {
    KFAC_ENTRY_BEGIN
    FITRE_REQUIRE(m && data && z && omegaZ && info && devPtr, FITRE_ERR_BAD_ARG, "NULL pointer argument");
    require_scratch(ctx, fitre_kfac_mem_required(m), "fitre_kfac_omega_z");
    model_check_batch(m, samples);
    omega_z_impl(ctx, m, data->currentBatch, z, false, samples, omegaZ, info, devPtr);
    check_device_error(ctx);  // the TMA-fed A-factor kernel has bounded waits
    KFAC_ENTRY_END
}

extern "C" int fitre_kfac_lambda_delta(fitre_context *ctx, const CNN_MODEL *m, const real *dx, int samples,
                                       real *lambdaG, const FITRE_KFAC_INFO *info, real *devPtr) {
    KFAC_ENTRY_BEGIN
    FITRE_REQUIRE(m && dx && lambdaG && info && devPtr, FITRE_ERR_BAD_ARG, "NULL pointer argument");
    require_scratch(ctx, fitre_kfac_mem_required(m), "fitre_kfac_lambda_delta");
    model_check_batch(m, samples);
    lambda_delta_impl(ctx, m, dx, false, samples, lambdaG, info, devPtr);
    KFAC_ENTRY_END
}

// The "speed-up" variant (factors refreshed every inverseFreq minibatches from running averages of
// the layer inputs and errors): solvers/kfac_inverses.cu:106-126 (updateRunningStats), :386-447
// (computeSpeedUpOmegaZ), :699-755 (computeSpeedUpLambdaDelta), and the dampedInput / dampedZ /
// dampedLambda branches of computeOmegaZ / computeLambdaDelta.
extern "C" int fitre_update_running_stats(fitre_context *ctx, real *src, const real *update, long numElements,
                                          real momentum) {
    KFAC_ENTRY_BEGIN
    FITRE_REQUIRE(src && update && numElements >= 0 && momentum >= 0 && momentum < 1, FITRE_ERR_BAD_ARG,
                  "bad argument");
    update_running(ctx, src, update, numElements, momentum, false);
    KFAC_ENTRY_END
}

extern "C" int fitre_kfac_speedup_omega_z(fitre_context *ctx, const FITRE_KFAC_INFO *info, const CNN_MODEL *m,
                                          const DEVICE_DATASET *data, int samples, const real *z,
                                          real *dampedInput, real *dampedZ, int iterCount) {
    KFAC_ENTRY_BEGIN
    FITRE_REQUIRE(info && m && data && data->currentBatch && z && dampedInput && dampedZ, FITRE_ERR_BAD_ARG,
                  "NULL pointer argument");
    model_check_batch(m, samples);
    const bool first = iterCount == 0;
    const double mom = std::sqrt(info->stats_decay);
    update_running(ctx, dampedInput, data->currentBatch, (long)data->features * samples, mom, first);
    for (int l = 0; l < m->cLayers; ++l) {
        const CONV_LAYER &c = m->convLayer[l];
        const POOL_LAYER &p = m->poolLayer[l];
        const long vol = (p.type == FITRE_NO_POOL ? (long)c.outHeight * c.outWidth : (long)p.outHeight * p.outWidth) *
                         c.outChannels * samples;
        update_running(ctx, dampedZ + m->zztOffsets[l + 1], z + m->zOffsets[l + 1] + c.outputOffset, vol, mom, first);
    }
    for (int l = 0; l < m->lLayers; ++l)
        update_running(ctx, dampedZ + m->zztOffsets[l + 1 + m->cLayers], z + m->zOffsets[l + 1 + m->cLayers],
                       (long)m->fcLayer[l].out * samples, mom, first);
    KFAC_ENTRY_END
}

extern "C" int fitre_kfac_speedup_lambda_delta(fitre_context *ctx, const FITRE_KFAC_INFO *info, const CNN_MODEL *m,
                                               int samples, const real *dx, real *dampedLambda, int iterCount) {
    KFAC_ENTRY_BEGIN
    FITRE_REQUIRE(info && m && dx && dampedLambda, FITRE_ERR_BAD_ARG, "NULL pointer argument");
    model_check_batch(m, samples);
    const bool first = iterCount == 0;
    const double mom = std::sqrt(info->stats_decay);
    for (int l = 0; l < m->cLayers; ++l) {
        const CONV_LAYER &c = m->convLayer[l];
        const real *delta = dx + m->zOffsets[l + 1] +
                            (c.batchNorm == FITRE_NO_BATCH_NORM ? c.activationOffset : c.batchNormOffset);
        update_running(ctx, dampedLambda + m->zztOffsets[l + 1], delta,
                       (long)c.outChannels * c.outHeight * c.outWidth * samples, mom, first);
    }
    for (int l = 0; l < m->lLayers; ++l)
        update_running(ctx, dampedLambda + m->zztOffsets[l + 1 + m->cLayers], dx + m->zOffsets[l + 1 + m->cLayers],
                       (long)m->fcLayer[l].out * samples, mom, first);
    KFAC_ENTRY_END
}

extern "C" int fitre_kfac_omega_z_damped(fitre_context *ctx, const CNN_MODEL *m, const real *dampedInput,
                                         const real *dampedZ, int samples, real *omegaZ,
                                         const FITRE_KFAC_INFO *info, real *devPtr) {
    KFAC_ENTRY_BEGIN
    FITRE_REQUIRE(m && dampedInput && dampedZ && omegaZ && info && devPtr, FITRE_ERR_BAD_ARG, "NULL pointer argument");
    require_scratch(ctx, fitre_kfac_mem_required(m), "fitre_kfac_omega_z_damped");
    model_check_batch(m, samples);
    omega_z_impl(ctx, m, dampedInput, dampedZ, true, samples, omegaZ, info, devPtr);
    KFAC_ENTRY_END
}

extern "C" int fitre_kfac_lambda_delta_damped(fitre_context *ctx, const CNN_MODEL *m, const real *dampedLambda,
                                              int samples, real *lambdaG, const FITRE_KFAC_INFO *info,
                                              real *devPtr) {
    KFAC_ENTRY_BEGIN
    FITRE_REQUIRE(m && dampedLambda && lambdaG && info && devPtr, FITRE_ERR_BAD_ARG, "NULL pointer argument");
    require_scratch(ctx, fitre_kfac_mem_required(m), "fitre_kfac_lambda_delta_damped");
    model_check_batch(m, samples);
    lambda_delta_impl(ctx, m, dampedLambda, true, samples, lambdaG, info, devPtr);
    KFAC_ENTRY_END
}

// ---------------------------------------------------------------------------------------------
// Damped factor inverses and the natural gradient.
// Reference: computeMatrixInverseCusolver (solvers/kfac_inverses.cu:133-186: add (lambda+gamma)
// to the diagonal, cusolverDnDpotrf, cusolverDnDpotrs against the identity) and
// computeNaturalGradient (solvers/kfac_natural_gradient.cu:36-241: G^-1 [W|b] A^-1 per layer).
// Here: explicit inverses by one recursion that factors and inverts with GEMMs (factor_invert),
// or, with FITRE_KFAC_SOLVER_CHOLESKY, a recursive blocked Cholesky factorisation in place
// (chol_factor) whose factors the natural gradient applies by triangular solves (trsm_right).
// Only the 64x64 diagonal blocks and triangles up to 256 run in small dedicated kernels; every
// other product is a DMMA GEMM.  No cuSOLVER / cuBLAS.
// ---------------------------------------------------------------------------------------------
namespace {
constexpr int NB = 64;

// Right-looking elimination of a 64 x 64 block held in registers by 256 threads: thread (ty, tx)
// owns the cyclic 4 x 4 sub-tile rows ty + 16 i, columns tx + 16 jj of the block (a) and of W, which
// starts as the identity and receives the same row operations, so that a ends as L (lower part) and
// W as L^-1.  One block barrier per column: the owners publish column j of a, row j of W and the
// pivot unscaled, every thread forms 1/sqrt(pivot) for itself.  bad <- 1 + first column whose
// pivot is not positive.
__device__ __forceinline__ void chol64_eliminate(double (&a)[4][4], double (&w)[4][4], double (*lcol)[64],
                                                 double (*wrow)[64], double *piv, int &bad, int ty, int tx) {
    constexpr int NB = 64;
    // jq (which of a thread's four rows / columns holds index j) is unrolled so that the register
    // tiles are indexed statically; the sixteen columns of each group run as a loop, which keeps the
    // code small enough to stay in the instruction cache
#pragma unroll
    for (int jq = 0; jq < 4; ++jq)
#pragma unroll 1
    for (int jr = 0; jr < 16; ++jr) {
        const int j = jq * 16 + jr, b = j & 1;
        if (tx == jr) {
#pragma unroll
            for (int i = 0; i < 4; ++i) lcol[b][ty + 16 * i] = a[i][jq];
            if (ty == jr) piv[b] = a[jq][jq];
        }
        if (ty == jr) {
#pragma unroll
            for (int jj = 0; jj < 4; ++jj) wrow[b][tx + 16 * jj] = w[jq][jj];
        }
        __syncthreads();
        const double p = piv[b];
        double rinv = 1.0;
        if (p > 0.0) rinv = rsqrt(p);
        else if (!bad) bad = j + 1;
        double lr[4], lc[4], wr[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) lr[i] = lcol[b][ty + 16 * i] * rinv;
#pragma unroll
        for (int jj = 0; jj < 4; ++jj) {
            lc[jj] = lcol[b][tx + 16 * jj] * rinv;
            wr[jj] = wrow[b][tx + 16 * jj] * rinv;
        }
        if (tx == jr) {  // column j of L is final
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i][jq] = (ty + 16 * i == j) ? p * rinv : lr[i];
        }
        if (ty == jr) {  // row j of L^-1 is final
#pragma unroll
            for (int jj = 0; jj < 4; ++jj) w[jq][jj] = wr[jj];
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) {
#pragma unroll
            for (int jj = 0; jj < 4; ++jj) {
                if (tx + 16 * jj > j) a[i][jj] -= lr[i] * lc[jj];
                if (ty + 16 * i > j) w[i][jj] -= lr[i] * wr[jj];
            }
        }
    }
}

// In place: A (nb x nb, lower, leading dim lda) <- its Cholesky factor L;
// Linv (nb x nb, leading dim ldi, upper part zero) <- L^-1.  *fail is set to 1 + column on a pivot <= 0.
// With Linv == nullptr the inverse is packed into the block itself: the strictly upper triangle
// of A receives (L^-1)' (element (a, b), a < b, holds L^-1[b][a]; the diagonal of L^-1 is the
// reciprocal of the diagonal of L), which is what trsm_small_kernel reads.
__global__ void __launch_bounds__(256) chol_block_kernel(double *A, long lda, int nb, double *Linv,
                                                         long ldi, int *fail, int col0) {
    // staging for the coalesced write-out: lower triangle L; strictly upper triangle (L^-1)'
    // off-diagonal; xd: diagonal of L^-1
    __shared__ double L[NB][NB + 1];
    __shared__ double xd[NB];
    __shared__ double lcol[2][NB], wrow[2][NB], piv[2];
    const int tid = threadIdx.x, ty = tid & 15, tx = tid >> 4;
    double a[4][4], w[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
#pragma unroll
        for (int jj = 0; jj < 4; ++jj) {
            const int r = ty + 16 * i, c = tx + 16 * jj;
            a[i][jj] = (r < nb && c < nb) ? (r >= c ? A[(long)c * lda + r] : 0.0) : (r == c ? 1.0 : 0.0);
            w[i][jj] = r == c ? 1.0 : 0.0;
        }
    }
    int bad = 0;
    chol64_eliminate(a, w, lcol, wrow, piv, bad, ty, tx);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
#pragma unroll
        for (int jj = 0; jj < 4; ++jj) {
            const int r = ty + 16 * i, c = tx + 16 * jj;
            if (r > c) {
                L[r][c] = a[i][jj];
                L[c][r] = w[i][jj];
            } else if (r == c) {
                L[r][r] = a[i][jj];
                xd[r] = w[i][jj];
            }
        }
    }
    __syncthreads();
    for (int e = tid; e < NB * NB; e += 256) {
        const int r = e % NB, c = e / NB;
        if (r < nb && c < nb && (r >= c || !Linv)) A[(long)c * lda + r] = L[r][c];
        if (Linv && r < nb && c < nb) Linv[(long)c * ldi + r] = (r == c) ? xd[c] : (r > c ? L[c][r] : 0.0);
    }
    if (tid == 0 && bad) atomicCAS(fail, 0, col0 + bad);
}

// Two 64 x 64 leaves, the solve and the update between them in one launch (packed form only):
// A (n x n, 64 < n <= 128, lower, leading dim lda) <- L, the upper triangles of its two diagonal
// blocks <- their packed inverses.  The block lives in shared memory (S, row stride 129); the two
// eliminations run in registers as in chol_block_kernel, L21 = A21 L11^-T and A22 -= L21 L21' as
// 64 x 64 x 64 products with 16 results per thread.  Replaces four dependent launches.
// D (8 x 8, two entries per lane) += A (8 x 4) B (4 x 8) on the fp64 tensor cores
__device__ __forceinline__ void dmma_f64(double &c0, double &c1, double a, double b) {
    asm volatile("mma.sync.aligned.m8n8k4.row.col.f64.f64.f64.f64 {%0,%1}, {%2}, {%3}, {%0,%1};\n"
                 : "+d"(c0), "+d"(c1)
                 : "d"(a), "d"(b));
}
constexpr int CH2 = 2 * NB, CH2_LD = CH2 + 4, CHW_LD = NB + 4;  // strides = 4 mod 16: DMMA fragments conflict-free
constexpr int CH2_SMEM = (CH2 * CH2_LD + NB * CHW_LD + 4 * NB + 2) * (int)sizeof(double);

__global__ void __launch_bounds__(256) chol128_kernel(double *A, long lda, int n, int *fail, int col0) {
    extern __shared__ __align__(16) double ch_sm[];
    double (*S)[CH2_LD] = reinterpret_cast<double (*)[CH2_LD]>(ch_sm);
    double (*Wb)[CHW_LD] = reinterpret_cast<double (*)[CHW_LD]>(ch_sm + CH2 * CH2_LD);  // Wb[k][c] = L11^-1[c][k]
    double *aux = ch_sm + CH2 * CH2_LD + NB * CHW_LD;
    double (*lcol)[NB] = reinterpret_cast<double (*)[NB]>(aux);           // [2][64]
    double (*wrow)[NB] = reinterpret_cast<double (*)[NB]>(aux + 2 * NB);  // [2][64]
    double *piv = aux + 4 * NB;                                           // [2]
    const int tid = threadIdx.x, ty = tid & 15, tx = tid >> 4;
    const int lane = tid & 31, warp = tid >> 5, lr = lane >> 2, lc = lane & 3;
    const int warp_m = warp & 1, warp_n = warp >> 1;  // 64 x 64 products: warp tile 32 x 16
    // lower triangle in, identity outside a ragged block
    for (int e = tid; e < CH2 * CH2; e += 256) {
        const int r = e % CH2, c = e / CH2;
        S[r][c] = (r < n && c < n) ? (r >= c ? A[(long)c * lda + r] : 0.0) : (r == c ? 1.0 : 0.0);
    }
    __syncthreads();
    int bad_all = 0;
    double a[4][4], w[4][4];
    for (int blk = 0; blk < 2; ++blk) {
        const int o = blk * NB;
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int jj = 0; jj < 4; ++jj) {
                const int r = ty + 16 * i, c = tx + 16 * jj;
                a[i][jj] = r >= c ? S[o + r][o + c] : 0.0;
                w[i][jj] = r == c ? 1.0 : 0.0;
            }
        int bad = 0;
        chol64_eliminate(a, w, lcol, wrow, piv, bad, ty, tx);
        if (bad && !bad_all) bad_all = o + bad;
        __syncthreads();
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int jj = 0; jj < 4; ++jj) {
                const int r = ty + 16 * i, c = tx + 16 * jj;
                if (r > c) {
                    S[o + r][o + c] = a[i][jj];
                    S[o + c][o + r] = w[i][jj];  // packed inverse: (row c, col r) holds L^-1[r][c]
                } else if (r == c) {
                    S[o + r][o + r] = a[i][jj];
                }
                if (blk == 0) Wb[c][r] = w[i][jj];  // all of L11^-1 (zero above its diagonal), transposed
            }
        __syncthreads();
        if (blk == 1) break;
        // L21 = A21 L11^-T and then A22 -= L21 L21', each a 64 x 64 x 64 product on the fp64 tensor cores
        for (int pass = 0; pass < 2; ++pass) {
            double acc[4][2][2];
#pragma unroll
            for (int mi = 0; mi < 4; ++mi)
#pragma unroll
                for (int ni = 0; ni < 2; ++ni) acc[mi][ni][0] = acc[mi][ni][1] = 0.0;
#pragma unroll 4
            for (int k4 = 0; k4 < NB / 4; ++k4) {
                const int k = k4 * 4 + lc;
                double fa[4], fb[2];
#pragma unroll
                for (int mi = 0; mi < 4; ++mi) fa[mi] = S[NB + warp_m * 32 + mi * 8 + lr][k];
#pragma unroll
                for (int ni = 0; ni < 2; ++ni) {
                    const int c = warp_n * 16 + ni * 8 + lr;
                    fb[ni] = pass == 0 ? Wb[k][c] : S[NB + c][k];
                }
#pragma unroll
                for (int mi = 0; mi < 4; ++mi)
#pragma unroll
                    for (int ni = 0; ni < 2; ++ni) dmma_f64(acc[mi][ni][0], acc[mi][ni][1], fa[mi], fb[ni]);
            }
            __syncthreads();  // every read of A21 / L21 is done
#pragma unroll
            for (int mi = 0; mi < 4; ++mi)
#pragma unroll
                for (int ni = 0; ni < 2; ++ni)
#pragma unroll
                    for (int e = 0; e < 2; ++e) {
                        const int r = warp_m * 32 + mi * 8 + lr, c = warp_n * 16 + ni * 8 + 2 * lc + e;
                        if (pass == 0) S[NB + r][c] = acc[mi][ni][e];
                        else if (r >= c) S[NB + r][NB + c] -= acc[mi][ni][e];
                    }
            __syncthreads();
        }
    }
    // out: everything at or below the diagonal, and the upper triangles of the two diagonal blocks
    for (int e = tid; e < CH2 * CH2; e += 256) {
        const int r = e % CH2, c = e / CH2;
        if (r < n && c < n && (r >= c || r / NB == c / NB)) A[(long)c * lda + r] = S[r][c];
    }
    if (tid == 0 && bad_all) atomicCAS(fail, 0, col0 + bad_all);
}

__global__ void add_diagonal_kernel(double *A, int n, double v) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) A[(long)i * n + i] += v;
}
__global__ void zero_upper_kernel(double *A, int n) {  // strictly upper triangle <- 0
    const long nn = (long)n * n;
    for (long e = blockIdx.x * (long)blockDim.x + threadIdx.x; e < nn; e += (long)gridDim.x * blockDim.x) {
        const int c = (int)(e / n), r = (int)(e - (long)c * n);
        if (r < c) A[e] = 0.0;
    }
}
// conv weights (K x Cout) + bias -> wb (K' x Cout): solvers/kfac_natural_gradient.cu:79-94
__global__ void pack_wb_kernel(const double *w, const double *b, double *wb, int K, int Kb, int Cout) {
    const long total = (long)Kb * Cout;
    for (long e = blockIdx.x * (long)blockDim.x + threadIdx.x; e < total; e += (long)gridDim.x * blockDim.x) {
        const int o = (int)(e / Kb), r = (int)(e - (long)o * Kb);
        wb[e] = r < K ? w[(long)o * K + r] : b[o];
    }
}
// ng (Cout x K', col-major) -> weights (K x Cout col-major) and bias (Cout): :166-173
__global__ void unpack_ng_kernel(const double *t, double *w, double *b, int K, int Kb, int Cout) {
    const long total = (long)Kb * Cout;
    for (long e = blockIdx.x * (long)blockDim.x + threadIdx.x; e < total; e += (long)gridDim.x * blockDim.x) {
        const int r = (int)(e / Cout), o = (int)(e - (long)r * Cout);  // t[o + r*Cout]
        if (r < K) w[(long)o * K + r] = t[e];
        else b[o] = t[e];
    }
}
int blocks_for(long n) { return (int)std::max<long>(1, std::min<long>((n + 255) / 256, 1184)); }

// Factor and invert in one recursion.  A (n x n, leading dim ld, lower triangle read, destroyed)
// is symmetric positive definite; on exit Y (same shape, zero on entry) holds L^-1 with
// A = L L'.  For A = [A11 .; A21 A22]:  L11, Y11 from A11;  L21 = A21 Y11';  A22 -= L21 L21';
// L22, Y22 from the updated A22;  Y21 = -Y22 L21 Y11.  Every product is a plain GEMM with large
// inner dimensions; only the NB x NB leaves run in the small shared-memory kernel.  `tmp` is a
// bump region of at most n*n/2 doubles.
void factor_invert(fitre_context *ctx, double *A, double *Y, long ld, int n, int col0, int *fail,
                   double *tmp) {
    if (n <= NB) {
        chol_block_kernel<<<1, 256, 0, ctx->stream>>>(A, ld, n, Y, ld, fail, col0);
        check_launch(ctx, "chol_block_kernel");
        return;
    }
    const int n1 = ((n / 2 + NB - 1) / NB) * NB, n2 = n - n1;
    double *A21 = A + n1, *A22 = A + (long)n1 * ld + n1;
    double *Y21 = Y + n1, *Y22 = Y + (long)n1 * ld + n1;
    double *L21 = tmp, *next = tmp + (long)n2 * n1;
    factor_invert(ctx, A, Y, ld, n1, col0, fail, next);
    // Y11 and Y22 are lower triangular and only the lower triangle of A22 is ever read again, so
    // each product skips the blocks that are zero or unused
    dgemm_structured(ctx, false, true, n2, n1, n1, 1.0, A21, (int)ld, Y, (int)ld, 0.0, L21, n2, GEMM_K_LE_COL);
    dgemm_structured(ctx, false, true, n2, n2, n1, -1.0, L21, n2, L21, n2, 1.0, A22, (int)ld, GEMM_LOWER_C);
    factor_invert(ctx, A22, Y22, ld, n2, col0 + n1, fail, next);
    double *T = next;  // free again after the recursion: L21 * Y11
    dgemm_structured(ctx, false, false, n2, n1, n1, 1.0, L21, n2, Y, (int)ld, 0.0, T, n2, GEMM_K_GE_COL);
    dgemm_structured(ctx, false, false, n2, n1, n2, -1.0, Y22, (int)ld, T, n2, 0.0, Y21, (int)ld, GEMM_K_LE_ROW);
}


// ---- Cholesky without the explicit inverse --------------------------------------------------
// Triangular solves from the right for a chunk of TR_ROWS rows of B (rows are independent):
//   trans != 0:  X L' = B   (block columns ascending:  X_j = (B_j - sum_{k<j} X_k L_jk') L_jj^-T)
//   trans == 0:  X L  = B   (block columns descending: X_j = (B_j - sum_{k>j} X_k L_kj ) L_jj^-1)
// L is t x t (t <= TR_MAX), lower, with the inverse of every NB x NB diagonal block packed in that
// block's upper triangle by chol_block_kernel.  B is overwritten by X.
constexpr int TR_ROWS = 16, TR_MAX = 256;
constexpr int TR_SMEM = (TR_MAX * TR_ROWS + 2 * NB * (NB + 1)) * (int)sizeof(double);

// The NB x NB tile of step (s, s2) of the sweep, 16 elements per thread, still in registers: s2 < s
// is the coupling tile of block column j with an already solved block k, s2 == s the diagonal
// block (lower = L_jj, strictly upper = packed inverse; identity outside a ragged block).
__device__ __forceinline__ void trsm_tile_load(double (&reg)[16], const double *L, long ldl, int t, int nblk,
                                               int trans, int s, int s2, int tid) {
    const int j = trans ? s : nblk - 1 - s;
    const int jb = min(NB, t - j * NB);
    if (s2 == s) {
#pragma unroll
        for (int u = 0; u < 16; ++u) {
            const int e = tid + u * 256, rr = e % NB, cc = e / NB;
            reg[u] = (rr < jb && cc < jb) ? L[(long)(j * NB + cc) * ldl + j * NB + rr] : (rr == cc ? 1.0 : 0.0);
        }
        return;
    }
    const int k = trans ? s2 : nblk - 1 - s2;
    const int kb = min(NB, t - k * NB);
#pragma unroll
    for (int u = 0; u < 16; ++u) {
        const int e = tid + u * 256, lo = e % NB, hi = e / NB;  // global reads run along a column
        if (trans) reg[u] = (lo < jb && hi < kb) ? L[(long)(k * NB + hi) * ldl + j * NB + lo] : 0.0;
        else reg[u] = (lo < kb && hi < jb) ? L[(long)(j * NB + hi) * ldl + k * NB + lo] : 0.0;
    }
}

__global__ void __launch_bounds__(256) trsm_small_kernel(double *B, long ldb, int r, const double *L, long ldl,
                                                         int t, int trans) {
    extern __shared__ __align__(16) double tr_sm[];
    double (*xs)[TR_ROWS] = reinterpret_cast<double (*)[TR_ROWS]>(tr_sm);
    typedef double Tile[NB][NB + 1];
    Tile *tiles = reinterpret_cast<Tile *>(tr_sm + TR_MAX * TR_ROWS);
    const int tid = threadIdx.x;
    const long row0 = (long)blockIdx.x * TR_ROWS;
    const int nrows = (int)min((long)TR_ROWS, r - row0);
    const int nblk = (t + NB - 1) / NB;
    double reg[16];
    trsm_tile_load(reg, L, ldl, t, nblk, trans, 0, 0, tid);
    for (int e = tid; e < TR_MAX * TR_ROWS; e += 256) {
        const int i = e % TR_ROWS, c = e / TR_ROWS;
        xs[c][i] = (i < nrows && c < t) ? B[(long)c * ldb + row0 + i] : 0.0;
    }
    __syncthreads();
    const int c = tid % NB, r4 = (tid / NB) * 4;
    int buf = 0;
    for (int s = 0; s < nblk; ++s) {
        const int j = trans ? s : nblk - 1 - s;
        const int jb = min(NB, t - j * NB);
        double acc[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[i] = xs[j * NB + c][r4 + i];
        for (int s2 = 0; s2 <= s; ++s2) {
            Tile &tl = tiles[buf];
            // tl[q][cc]: coupling tiles hold L[j*NB+cc][k*NB+q] (trans) or L[k*NB+q][j*NB+cc];
            // the diagonal tile is stored as it lies, tl[row][col]
            const bool flip = trans && s2 < s;
#pragma unroll
            for (int u = 0; u < 16; ++u) {
                const int e = tid + u * 256, lo = e % NB, hi = e / NB;
                if (flip) tl[hi][lo] = reg[u];
                else tl[lo][hi] = reg[u];
            }
            __syncthreads();
            // the next tile travels while this one is used
            if (s2 < s) trsm_tile_load(reg, L, ldl, t, nblk, trans, s, s2 + 1, tid);
            else if (s + 1 < nblk) trsm_tile_load(reg, L, ldl, t, nblk, trans, s + 1, 0, tid);
            if (s2 < s) {
                const int k = trans ? s2 : nblk - 1 - s2;
#pragma unroll 8
                for (int q = 0; q < NB; ++q) {
                    const double l = tl[q][c];
                    const double2 x01 = *reinterpret_cast<const double2 *>(&xs[k * NB + q][r4]);
                    const double2 x23 = *reinterpret_cast<const double2 *>(&xs[k * NB + q][r4 + 2]);
                    acc[0] -= x01.x * l;
                    acc[1] -= x01.y * l;
                    acc[2] -= x23.x * l;
                    acc[3] -= x23.y * l;
                }
            } else {
#pragma unroll
                for (int i = 0; i < 4; ++i) xs[j * NB + c][r4 + i] = acc[i];
                __syncthreads();
                double out[4];
                const double dinv = 1.0 / tl[c][c];
#pragma unroll
                for (int i = 0; i < 4; ++i) out[i] = acc[i] * dinv;
                if (trans) {
                    for (int k = 0; k < c; ++k) {
                        const double w = tl[k][c];  // L^-1[c][k]
#pragma unroll
                        for (int i = 0; i < 4; ++i) out[i] += xs[j * NB + k][r4 + i] * w;
                    }
                } else {
                    for (int k = c + 1; k < jb; ++k) {
                        const double w = tl[c][k];  // L^-1[k][c]
#pragma unroll
                        for (int i = 0; i < 4; ++i) out[i] += xs[j * NB + k][r4 + i] * w;
                    }
                }
                __syncthreads();
#pragma unroll
                for (int i = 0; i < 4; ++i) xs[j * NB + c][r4 + i] = out[i];
            }
            buf ^= 1;
        }
    }
    __syncthreads();
    for (int e = tid; e < t * TR_ROWS; e += 256) {
        const int i = e % TR_ROWS, cc = e / TR_ROWS;
        if (i < nrows) B[(long)cc * ldb + row0 + i] = xs[cc][i];
    }
}

// B (r x t, leading dim ldb) <- B L^-T (trans) or B L^-1, L as left by chol_factor.  Above TR_MAX
// the triangle is halved and the coupling term is one GEMM; splits fall on multiples of NB so
// that the packed diagonal blocks line up.
void trsm_right(fitre_context *ctx, double *B, long ldb, int r, const double *L, long ldl, int t, bool trans) {
    if (t <= TR_MAX) {
        trsm_small_kernel<<<(r + TR_ROWS - 1) / TR_ROWS, 256, TR_SMEM, ctx->stream>>>(B, ldb, r, L, ldl, t,
                                                                                      trans ? 1 : 0);
        check_launch(ctx, "trsm_small_kernel");
        return;
    }
    const int t1 = ((t / 2 + NB - 1) / NB) * NB, t2 = t - t1;
    const double *L21 = L + t1, *L22 = L + (long)t1 * ldl + t1;
    double *B2 = B + (long)t1 * ldb;
    if (trans) {
        trsm_right(ctx, B, ldb, r, L, ldl, t1, true);
        dgemm(ctx, false, true, r, t2, t1, -1.0, B, (int)ldb, L21, (int)ldl, 1.0, B2, (int)ldb);
        trsm_right(ctx, B2, ldb, r, L22, ldl, t2, true);
    } else {
        trsm_right(ctx, B2, ldb, r, L22, ldl, t2, false);
        dgemm(ctx, false, false, r, t1, t2, -1.0, B2, (int)ldb, L21, (int)ldl, 1.0, B, (int)ldb);
        trsm_right(ctx, B, ldb, r, L, ldl, t1, false);
    }
}

// In place: the lower triangle of A (n x n, leading dim ld, symmetric positive definite) <- L with
// A = L L'; the upper triangles of the NB x NB diagonal blocks <- their packed inverses.  The rest
// of the upper triangle keeps whatever it held.  No scratch: the panel solve and the trailing
// update work inside A.
void chol_factor(fitre_context *ctx, double *A, long ld, int n, int col0, int *fail) {
    if (n <= NB) {
        chol_block_kernel<<<1, 256, 0, ctx->stream>>>(A, ld, n, nullptr, 0, fail, col0);
        check_launch(ctx, "chol_block_kernel");
        return;
    }
    if (n <= CH2) {
        chol128_kernel<<<1, 256, CH2_SMEM, ctx->stream>>>(A, ld, n, fail, col0);
        check_launch(ctx, "chol128_kernel");
        return;
    }
    const int n1 = ((n / 2 + NB - 1) / NB) * NB, n2 = n - n1;
    double *A21 = A + n1, *A22 = A + (long)n1 * ld + n1;
    chol_factor(ctx, A, ld, n1, col0, fail);
    trsm_right(ctx, A21, ld, n2, A, ld, n1, true);  // L21 = A21 L11^-T
    dgemm_structured(ctx, false, true, n2, n2, n1, -1.0, A21, (int)ld, A21, (int)ld, 1.0, A22, (int)ld,
                     GEMM_LOWER_C);
    chol_factor(ctx, A22, ld, n2, col0 + n1, fail);
}

// factor <- Cholesky factor of (matrix + damp I), packed as chol_factor leaves it
void factor_spd(fitre_context *ctx, const double *matrix, double *factor, int n, double damp, int *fail) {
    vec_copy(ctx, (long)n * n, matrix, factor);
    add_diagonal_kernel<<<(n + 255) / 256, 256, 0, ctx->stream>>>(factor, n, damp);
    check_launch(ctx, "add_diagonal_kernel");
    chol_factor(ctx, factor, n, n, 0, fail);
}

// inverse <- (matrix + damp I)^-1 on ctx->stream, no host synchronisation; a pivot <= 0 is
// recorded in *fail.  scratch: fitre_kfac_inverse_mem_required(n) doubles.
void invert_spd(fitre_context *ctx, const double *matrix, double *inverse, int n, double damp,
                double *scratch, int *fail) {
    const long nn = (long)n * n;
    double *Am = scratch;                    // damped copy, destroyed by the factorisation
    double *Y = Am + align32(nn);            // L^-1
    double *tmp = Y + align32(nn);           // recursion scratch
    double *slabs = tmp + align32(nn / 2 + (long)n * NB);
    vec_copy(ctx, nn, matrix, Am);
    add_diagonal_kernel<<<(n + 255) / 256, 256, 0, ctx->stream>>>(Am, n, damp);
    check_launch(ctx, "add_diagonal_kernel");
    vec_fill(ctx, nn, 0.0, Y);
    factor_invert(ctx, Am, Y, n, n, 0, fail, tmp);
    syrk_tn(ctx, n, n, 1.0, Y, n, inverse, slabs);  // (L^-1)' L^-1
}

void check_fail_word(fitre_context *ctx, int *fail) {
    FITRE_CUDA(cudaMemcpyAsync(ctx->pinned + 202, fail, sizeof(double), cudaMemcpyDeviceToHost, ctx->stream));
    check_device_error(ctx);  // synchronises the stream; also reports a TMA wait that ran out
    int f;
    std::memcpy(&f, ctx->pinned + 202, sizeof(int));
    FITRE_REQUIRE(f == 0, FITRE_ERR_NOT_CONVERGED,
                  "Cholesky pivot <= 0 at column " + std::to_string(f - 1) + " (matrix not positive definite)");
}
}  // namespace

namespace fitre {
void kfac_init_attributes() {
    FITRE_CUDA(cudaFuncSetAttribute(chol128_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, CH2_SMEM));
    FITRE_CUDA(cudaFuncSetAttribute(trsm_small_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, TR_SMEM));
}
}  // namespace fitre

extern "C" long fitre_kfac_inverse_mem_required(int n) {
    if (n < 1) return -1;
    const long nn = (long)n * n;
    return 2 * align32(nn) + align32(nn / 2 + (long)n * NB) + align32(syrk_scratch(n, n)) + 64;
}

// inverse = (matrix + (lambda + dampGamma) I)^-1, both n x n column-major.
extern "C" int fitre_kfac_matrix_inverse(fitre_context *ctx, const real *matrix, real *inverse, int n,
                                         real *devPtr, real lambda, real dampGamma) {
    if (!ctx) return FITRE_ERR_BAD_ARG;
    try {
        FITRE_CUDA(cudaSetDevice(ctx->device));
        FITRE_REQUIRE(matrix && inverse && devPtr && n > 0, FITRE_ERR_BAD_ARG, "bad argument");
        require_scratch(ctx, fitre_kfac_inverse_mem_required(n), "fitre_kfac_matrix_inverse");
        int *fail = (int *)(ctx->dscal + 4002);
        FITRE_CUDA(cudaMemsetAsync(fail, 0, sizeof(double), ctx->stream));
        invert_spd(ctx, matrix, inverse, n, lambda + dampGamma, devPtr, fail);
        check_fail_word(ctx, fail);
        return FITRE_OK;
    } catch (const Error &e) {
        ctx->err = e.what();
        return e.code;
    }
}

// factor = packed Cholesky factor of matrix + (lambda + dampGamma) I, both n x n column-major.
extern "C" int fitre_kfac_matrix_factor(fitre_context *ctx, const real *matrix, real *factor, int n,
                                        real lambda, real dampGamma) {
    if (!ctx) return FITRE_ERR_BAD_ARG;
    try {
        FITRE_CUDA(cudaSetDevice(ctx->device));
        FITRE_REQUIRE(matrix && factor && n > 0, FITRE_ERR_BAD_ARG, "bad argument");
        int *fail = (int *)(ctx->dscal + 4002);
        FITRE_CUDA(cudaMemsetAsync(fail, 0, sizeof(double), ctx->stream));
        factor_spd(ctx, matrix, factor, n, lambda + dampGamma, fail);
        check_fail_word(ctx, fail);
        return FITRE_OK;
    } catch (const Error &e) {
        ctx->err = e.what();
        return e.code;
    }
}

// ---------------------------------------------------------------------------------------------
// All 2L factor inverses of one KFAC step.  The matrices are independent: they are spread over a
// few streams of this GPU (the leaves of the factorisation occupy one SM, so concurrent matrices
// fill the rest), and over the ranks of the communicator when there is one (largest first onto
// the least loaded rank; every rank then receives the others' inverses by one sum all-reduce over
// buffers that hold zeros where a rank did no work).
namespace {
constexpr int kInvStreams = 4;   // explicit inverses: each stream owns a scratch region of 2.5 n^2
constexpr int kSideStreams = 8;  // streams that exist; the scratch-free sequences use all of them
struct InvJob {
    const double *src;
    double *dst;
    int n;
    double cost;
    bool factor_only;  // Cholesky factor instead of the inverse
    int layer;
};
std::vector<InvJob> inverse_jobs(const CNN_MODEL *m, const FITRE_KFAC_INFO *info, const double *A,
                                 double *Ainv, const double *G, double *Ginv, bool chol) {
    std::vector<InvJob> jobs;
    for (int l = 0; l < m->cLayers + m->lLayers; ++l) {
        int a, g;
        if (l < m->cLayers) {
            const CONV_LAYER &c = m->convLayer[l];
            a = c.inChannels * c.kSize * c.kSize + (m->bias ? 1 : 0);
            g = c.outChannels;
        } else {
            a = m->fcLayer[l - m->cLayers].in + (m->bias ? 1 : 0);
            g = m->fcLayer[l - m->cLayers].out;
        }
        jobs.push_back({A + info->OmegaZOffsets[l], Ainv + info->OmegaZOffsets[l], a,
                        (double)a * a * a / (chol ? 3.0 : 1.0), chol, l});
        jobs.push_back({G + info->LambdaGOffsets[l], Ginv + info->LambdaGOffsets[l], g, (double)g * g * g, false, l});
    }
    std::stable_sort(jobs.begin(), jobs.end(), [](const InvJob &x, const InvJob &y) { return x.cost > y.cost; });
    return jobs;
}
// FITRE_KFAC_LAYER_OWNED: which rank holds the factors of each layer and forms its slice of the
// natural gradient (most expensive layer first onto the least loaded rank)
std::vector<int> layer_owners(const CNN_MODEL *m, int world, bool chol) {
    const int nl = m->cLayers + m->lLayers;
    std::vector<double> cost(nl);
    std::vector<int> order(nl), owner(nl, 0);
    for (int l = 0; l < nl; ++l) {
        const double a = l < m->cLayers ? (double)m->convLayer[l].inChannels * m->convLayer[l].kSize *
                                              m->convLayer[l].kSize
                                        : (double)m->fcLayer[l - m->cLayers].in;
        const double g = l < m->cLayers ? m->convLayer[l].outChannels : m->fcLayer[l - m->cLayers].out;
        cost[l] = a * a * a / (chol ? 3.0 : 1.0) + g * g * g + 2.0 * g * a * (a + g);
        order[l] = l;
    }
    std::stable_sort(order.begin(), order.end(), [&](int x, int y) { return cost[x] > cost[y]; });
    std::vector<double> load(world, 0.0);
    for (int l : order) {
        const int r = (int)(std::min_element(load.begin(), load.end()) - load.begin());
        load[r] += cost[l];
        owner[l] = r;
    }
    return owner;
}
void ensure_side_streams(fitre_context *ctx) {
    if (ctx->inv_streams[0]) return;
    // The chains on these streams are short kernels on the critical path of the factorisations;
    // the highest stream priority lets their blocks go first whenever a slot frees up beside the
    // large kernels of the other streams.  (FITRE_SIDE_PRIORITY=0: default priority.)
    int lo = 0, hi = 0;
    FITRE_CUDA(cudaDeviceGetStreamPriorityRange(&lo, &hi));
    const char *sw = std::getenv("FITRE_SIDE_PRIORITY");
    const int prio = (sw && sw[0] == '0') ? lo : hi;
    for (int s = 0; s < kSideStreams; ++s)
        FITRE_CUDA(cudaStreamCreateWithPriority(&ctx->inv_streams[s], cudaStreamNonBlocking, prio));
    FITRE_CUDA(cudaEventCreateWithFlags(&ctx->inv_fork, cudaEventDisableTiming));
    for (int s = 0; s < kSideStreams; ++s)
        FITRE_CUDA(cudaEventCreateWithFlags(&ctx->inv_join[s], cudaEventDisableTiming));
}
int max_block(const CNN_MODEL *m) {
    int mx = 1;
    for (int l = 0; l < m->cLayers; ++l)
        mx = std::max(mx, std::max(m->convLayer[l].inChannels * m->convLayer[l].kSize * m->convLayer[l].kSize + 1,
                                   m->convLayer[l].outChannels));
    for (int l = 0; l < m->lLayers; ++l) mx = std::max(mx, std::max(m->fcLayer[l].in + 1, m->fcLayer[l].out));
    return mx;
}
}  // namespace

extern "C" long fitre_kfac_invert_factors_mem_required(const CNN_MODEL *m) {
    if (!m) return -1;
    return kInvStreams * align32(fitre_kfac_inverse_mem_required(max_block(m)));
}

extern "C" int fitre_kfac_invert_factors(fitre_context *ctx, const CNN_MODEL *m, const FITRE_KFAC_INFO *info,
                                         const real *omegaZ, real *omegaZInv, const real *lambdaG,
                                         real *lambdaGInv, real *devPtr) {
    if (!ctx) return FITRE_ERR_BAD_ARG;
    try {
        FITRE_CUDA(cudaSetDevice(ctx->device));
        FITRE_REQUIRE(m && info && omegaZ && omegaZInv && lambdaG && lambdaGInv && devPtr, FITRE_ERR_BAD_ARG,
                      "NULL pointer argument");
        require_scratch(ctx, fitre_kfac_invert_factors_mem_required(m), "fitre_kfac_invert_factors");
        const double damp = info->regLambda + info->dampGamma;
        std::vector<InvJob> jobs = inverse_jobs(m, info, omegaZ, omegaZInv, lambdaG, lambdaGInv,
                                                ctx->kfac_solver == FITRE_KFAC_SOLVER_CHOLESKY);
        const int W = ctx->world;
        std::vector<double> load(W, 0.0);
        std::vector<InvJob> mine;
        for (const InvJob &j : jobs) {
            const int r = (int)(std::min_element(load.begin(), load.end()) - load.begin());
            load[r] += j.cost;
            if (r == ctx->rank) mine.push_back(j);
        }
        int *fail = (int *)(ctx->dscal + 4002);
        ensure_side_streams(ctx);
        std::vector<long long> key = {ptr_key(omegaZ), ptr_key(omegaZInv), ptr_key(lambdaG), ptr_key(lambdaGInv),
                                      ptr_key(devPtr), bits_key(damp), ctx->kfac_solver, ctx->rank, W,
                                      info->OmegaZSize, info->LambdaGSize};
        for (const InvJob &j : jobs) {
            key.push_back(j.n);
            key.push_back(ptr_key(j.dst));
        }
        run_graphed(ctx, ctx->graph_invert, key, [&] {
        FITRE_CUDA(cudaMemsetAsync(fail, 0, sizeof(double), ctx->stream));
        if (W > 1) {
            vec_fill(ctx, info->OmegaZSize, 0.0, omegaZInv);
            vec_fill(ctx, info->LambdaGSize, 0.0, lambdaGInv);
        }
        // fork: the side streams start after everything queued on the context's stream
        cudaStream_t main_stream = ctx->stream;
        FITRE_CUDA(cudaEventRecord(ctx->inv_fork, main_stream));
        const long per = align32(fitre_kfac_inverse_mem_required(max_block(m)));
        std::vector<double> sload(kSideStreams, 0.0);
        try {
            for (int s = 0; s < kSideStreams; ++s) FITRE_CUDA(cudaStreamWaitEvent(ctx->inv_streams[s], ctx->inv_fork, 0));
            for (const InvJob &j : mine) {
                // an explicit inverse needs one of the kInvStreams scratch regions; a factorisation needs none
                const int ns = j.factor_only ? kSideStreams : kInvStreams;
                const int s = (int)(std::min_element(sload.begin(), sload.begin() + ns) - sload.begin());
                sload[s] += j.cost;
                ctx->stream = ctx->inv_streams[s];
                if (j.factor_only) factor_spd(ctx, j.src, j.dst, j.n, damp, fail);
                else invert_spd(ctx, j.src, j.dst, j.n, damp, devPtr + (long)s * per, fail);
            }
        } catch (...) {
            ctx->stream = main_stream;
            throw;
        }
        ctx->stream = main_stream;
        for (int s = 0; s < kSideStreams; ++s) {
            FITRE_CUDA(cudaEventRecord(ctx->inv_join[s], ctx->inv_streams[s]));
            FITRE_CUDA(cudaStreamWaitEvent(main_stream, ctx->inv_join[s], 0));
        }
        });
        if (W > 1) {
            comm_allreduce_sum(ctx, omegaZInv, info->OmegaZSize);
            comm_allreduce_sum(ctx, lambdaGInv, info->LambdaGSize);
            comm_allreduce_sum(ctx, ctx->dscal + 4002, 1);  // a failure on any rank is seen by all
        }
        check_fail_word(ctx, fail);
        return FITRE_OK;
    } catch (const Error &e) {
        ctx->err = e.what();
        return e.code;
    }
}

// ---------------------------------------------------------------------------------------------
// Factors and their damped inverses in one call, as computeOmegaZ / computeLambdaDelta do layer
// by layer (solvers/kfac_inverses.cu:450-630,759-857: each factor is inverted right after it is
// formed).  On one GPU the two kinds of work are overlapped: the factor products (tensor-bound,
// fill the GPU) run on the context's stream, largest A blocks first, and every factorisation
// (a chain of small dependent kernels) starts on a side stream as soon as its factor is ready,
// so the chains hide under the remaining products.  On one GPU the whole sequence is one CUDA
// graph; with ranks each factor is all-reduced on the context's stream before its factorisation
// starts on the rank that owns it, and the results are exchanged as fitre_kfac_invert_factors does.
// ---------------------------------------------------------------------------------------------
extern "C" long fitre_kfac_factors_and_inverses_mem_required(const CNN_MODEL *m) {
    if (!m) return -1;
    return align32(fitre_kfac_mem_required(m)) + fitre_kfac_invert_factors_mem_required(m);
}

extern "C" int fitre_kfac_factors_and_inverses(fitre_context *ctx, const CNN_MODEL *m, const real *x0,
                                               const real *zbase, const real *dbase, int packed, int samples,
                                               real *omegaZ, real *omegaZInv, real *lambdaG, real *lambdaGInv,
                                               const FITRE_KFAC_INFO *info, real *devPtr) {
    KFAC_ENTRY_BEGIN
    FITRE_REQUIRE(m && x0 && zbase && dbase && omegaZ && omegaZInv && lambdaG && lambdaGInv && info && devPtr,
                  FITRE_ERR_BAD_ARG, "NULL pointer argument");
    model_check_batch(m, samples);
    require_scratch(ctx, fitre_kfac_factors_and_inverses_mem_required(m), "fitre_kfac_factors_and_inverses");
    double *inv_scratch = devPtr + align32(fitre_kfac_mem_required(m));
    const int W = ctx->world;
    const bool chol = ctx->kfac_solver == FITRE_KFAC_SOLVER_CHOLESKY;
    const double damp = info->regLambda + info->dampGamma;
    const int nl = m->cLayers + m->lLayers;
    std::vector<InvJob> jobs = inverse_jobs(m, info, omegaZ, omegaZInv, lambdaG, lambdaGInv, chol);
    // with ranks: the same division of the factorisations as fitre_kfac_invert_factors
    std::vector<char> mine(jobs.size(), 1);
    const bool owned = W > 1 && ctx->kfac_owned;
    std::vector<int> owner(nl, -1);  // -1: factors summed onto every rank
    if (owned) {
        owner = layer_owners(m, W, chol);
        for (size_t i = 0; i < jobs.size(); ++i) mine[i] = owner[jobs[i].layer] == ctx->rank;
    } else if (W > 1) {
        std::vector<double> load(W, 0.0);
        for (size_t i = 0; i < jobs.size(); ++i) {
            const int r = (int)(std::min_element(load.begin(), load.end()) - load.begin());
            load[r] += jobs[i].cost;
            mine[i] = r == ctx->rank;
        }
    }
    int *fail = (int *)(ctx->dscal + 4002);
    ensure_side_streams(ctx);
    while ((int)ctx->layer_ev.size() < nl) {
        cudaEvent_t e;
        FITRE_CUDA(cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
        ctx->layer_ev.push_back(e);
    }
    std::vector<long long> key = {ptr_key(x0), ptr_key(zbase), ptr_key(dbase), packed, samples, ptr_key(omegaZ),
                                  ptr_key(omegaZInv), ptr_key(lambdaG), ptr_key(lambdaGInv), ptr_key(devPtr),
                                  bits_key(damp), ctx->kfac_solver, m->bias, info->OmegaZSize, info->LambdaGSize};
    for (const InvJob &j : jobs) {
        key.push_back(j.n);
        key.push_back(ptr_key(j.dst));
    }
    for (int l = 0; l < m->cLayers; ++l) {
        key.push_back(m->convLayer[l].height);
        key.push_back(m->convLayer[l].width);
        key.push_back(m->convLayer[l].outputOffset);
        key.push_back(m->convLayer[l].batchNormOffset);
        key.push_back(m->convLayer[l].activationOffset);
    }
    for (int l = 0; l <= nl; ++l) {
        key.push_back(m->zOffsets[l]);
        key.push_back(m->zztOffsets[l]);
    }
    auto body = [&] {
        cudaStream_t main_stream = ctx->stream;
        FITRE_CUDA(cudaMemsetAsync(fail, 0, sizeof(double), main_stream));
        if (W > 1 && !owned) {
            vec_fill(ctx, info->OmegaZSize, 0.0, omegaZInv);
            vec_fill(ctx, info->LambdaGSize, 0.0, lambdaGInv);
        }
        const long per = align32(fitre_kfac_inverse_mem_required(max_block(m)));
        std::vector<double> sload(kSideStreams, 0.0);
        // one job on the least loaded side stream, after `ready` (recorded on the main stream)
        auto start_job = [&](const InvJob &j, cudaEvent_t ready) {
            const int ns = j.factor_only ? kSideStreams : kInvStreams;
            const int s = (int)(std::min_element(sload.begin(), sload.begin() + ns) - sload.begin());
            sload[s] += j.cost;
            FITRE_CUDA(cudaStreamWaitEvent(ctx->inv_streams[s], ready, 0));
            ctx->stream = ctx->inv_streams[s];
            if (j.factor_only) factor_spd(ctx, j.src, j.dst, j.n, damp, fail);
            else invert_spd(ctx, j.src, j.dst, j.n, damp, inv_scratch + (long)s * per, fail);
            ctx->stream = main_stream;
        };
        try {
            // every side stream joins the sequence, whether or not a job lands on it
            FITRE_CUDA(cudaEventRecord(ctx->inv_fork, main_stream));
            for (int s = 0; s < kSideStreams; ++s)
                FITRE_CUDA(cudaStreamWaitEvent(ctx->inv_streams[s], ctx->inv_fork, 0));
            // G factors: a fraction of a millisecond in all; their inverses start at once
            for (int l = 0; l < nl; ++l)
                lambda_delta_layer(ctx, m, dbase, packed != 0, samples, lambdaG, info, devPtr, l, owner[l]);
            FITRE_CUDA(cudaEventRecord(ctx->inv_fork, main_stream));
            for (size_t i = 0; i < jobs.size(); ++i)
                if (mine[i] && jobs[i].src >= lambdaG && jobs[i].src < lambdaG + info->LambdaGSize)
                    start_job(jobs[i], ctx->inv_fork);
            // A factors, most expensive factorisation first
            std::vector<int> order(nl);
            for (int l = 0; l < nl; ++l) order[l] = l;
            auto block = [&](int l) {
                return l < m->cLayers ? m->convLayer[l].inChannels * m->convLayer[l].kSize * m->convLayer[l].kSize
                                      : m->fcLayer[l - m->cLayers].in;
            };
            std::stable_sort(order.begin(), order.end(), [&](int x, int y) { return block(x) > block(y); });
            for (int l : order) {
                omega_z_layer(ctx, m, x0, zbase, packed != 0, samples, omegaZ, info, devPtr, l, owner[l]);
                FITRE_CUDA(cudaEventRecord(ctx->layer_ev[l], main_stream));
                for (size_t i = 0; i < jobs.size(); ++i)
                    if (mine[i] && jobs[i].src == omegaZ + info->OmegaZOffsets[l]) start_job(jobs[i], ctx->layer_ev[l]);
            }
        } catch (...) {
            ctx->stream = main_stream;
            throw;
        }
        for (int s = 0; s < kSideStreams; ++s) {
            FITRE_CUDA(cudaEventRecord(ctx->inv_join[s], ctx->inv_streams[s]));
            FITRE_CUDA(cudaStreamWaitEvent(main_stream, ctx->inv_join[s], 0));
        }
    };
    if (W > 1) {
        // the per-layer all-reduces of the factors sit between the kernels: launched directly
        body();
        if (!owned) {
            comm_allreduce_sum(ctx, omegaZInv, info->OmegaZSize);
            comm_allreduce_sum(ctx, lambdaGInv, info->LambdaGSize);
        }
        comm_allreduce_sum(ctx, ctx->dscal + 4002, 1);  // a failure on any rank is seen by all
    } else {
        run_graphed(ctx, ctx->graph_factors, key, body);
    }
    check_fail_word(ctx, fail);
    KFAC_ENTRY_END
}

// ---------------------------------------------------------------------------------------------
// The same work in two calls, so that the A side -- whose factorisations are chains of a thousand
// small dependent kernels that leave most of the GPU idle -- runs underneath whatever the caller
// queues between them (in the KFAC step: the second backward pass on the sampled labels, which
// only the G factors depend on).
//   fitre_kfac_omega_z_begin: A factors (they need the forward state only) and the factorisation
//     of each as soon as it is ready, all on streams of the library's own, ordered after the work
//     queued on the context's stream so far.  Returns without waiting; the context's stream does
//     not wait either.
//   fitre_kfac_lambda_delta_finish: G factors and their inverses, then the context's stream (and
//     the host, for the "not positive definite" status) waits for everything both calls started.
// Same bits as fitre_kfac_factors_and_inverses.
// ---------------------------------------------------------------------------------------------
namespace {
struct PhasePlan {
    std::vector<InvJob> jobs;
    std::vector<char> mine;
    std::vector<int> owner;
    bool owned = false, chol = false;
    double damp = 0.0;
    int nl = 0;
};
PhasePlan make_phase_plan(fitre_context *ctx, const CNN_MODEL *m, const FITRE_KFAC_INFO *info, const double *omegaZ,
                          double *omegaZInv, const double *lambdaG, double *lambdaGInv) {
    PhasePlan p;
    const int W = ctx->world;
    p.chol = ctx->kfac_solver == FITRE_KFAC_SOLVER_CHOLESKY;
    p.damp = info->regLambda + info->dampGamma;
    p.nl = m->cLayers + m->lLayers;
    p.jobs = inverse_jobs(m, info, omegaZ, omegaZInv, lambdaG, lambdaGInv, p.chol);
    p.mine.assign(p.jobs.size(), 1);
    p.owned = W > 1 && ctx->kfac_owned;
    p.owner.assign(p.nl, -1);
    if (p.owned) {
        p.owner = layer_owners(m, W, p.chol);
        for (size_t i = 0; i < p.jobs.size(); ++i) p.mine[i] = p.owner[p.jobs[i].layer] == ctx->rank;
    } else if (W > 1) {
        std::vector<double> load(W, 0.0);
        for (size_t i = 0; i < p.jobs.size(); ++i) {
            const int r = (int)(std::min_element(load.begin(), load.end()) - load.begin());
            load[r] += p.jobs[i].cost;
            p.mine[i] = r == ctx->rank;
        }
    }
    return p;
}
std::vector<long long> phase_key(fitre_context *ctx, const CNN_MODEL *m, const FITRE_KFAC_INFO *info,
                                 const PhasePlan &p, const void *a, const void *b, const void *c, const void *d,
                                 const void *e, int packed, int samples) {
    std::vector<long long> key = {ptr_key(a), ptr_key(b), ptr_key(c), ptr_key(d), ptr_key(e), packed, samples,
                                  bits_key(p.damp), ctx->kfac_solver, m->bias, info->OmegaZSize, info->LambdaGSize};
    for (const InvJob &j : p.jobs) {
        key.push_back(j.n);
        key.push_back(ptr_key(j.dst));
    }
    for (int l = 0; l < m->cLayers; ++l) {
        key.push_back(m->convLayer[l].height);
        key.push_back(m->convLayer[l].width);
        key.push_back(m->convLayer[l].outputOffset);
        key.push_back(m->convLayer[l].batchNormOffset);
        key.push_back(m->convLayer[l].activationOffset);
    }
    for (int l = 0; l <= p.nl; ++l) {
        key.push_back(m->zOffsets[l]);
        key.push_back(m->zztOffsets[l]);
    }
    return key;
}
// One side of the factors (A: doA, G: !doA) on ctx->stream with its factorisations forked onto the
// side streams and joined back at the end.
void run_factor_phase(fitre_context *ctx, const CNN_MODEL *m, const FITRE_KFAC_INFO *info, const PhasePlan &p,
                      bool doA, const double *x0, const double *base, bool packed, int samples, double *factors,
                      double *devPtr, int *fail) {
    cudaStream_t main_stream = ctx->stream;
    double *inv_scratch = devPtr + align32(fitre_kfac_mem_required(m));
    const long per = align32(fitre_kfac_inverse_mem_required(max_block(m)));
    std::vector<double> sload(kSideStreams, 0.0);
    auto start_job = [&](const InvJob &j, cudaEvent_t ready) {
        const int ns = j.factor_only ? kSideStreams : kInvStreams;
        const int s = (int)(std::min_element(sload.begin(), sload.begin() + ns) - sload.begin());
        sload[s] += j.cost;
        FITRE_CUDA(cudaStreamWaitEvent(ctx->inv_streams[s], ready, 0));
        ctx->stream = ctx->inv_streams[s];
        if (j.factor_only) factor_spd(ctx, j.src, j.dst, j.n, p.damp, fail);
        else invert_spd(ctx, j.src, j.dst, j.n, p.damp, inv_scratch + (long)s * per, fail);
        ctx->stream = main_stream;
    };
    try {
        FITRE_CUDA(cudaEventRecord(ctx->inv_fork, main_stream));
        for (int s = 0; s < kSideStreams; ++s) FITRE_CUDA(cudaStreamWaitEvent(ctx->inv_streams[s], ctx->inv_fork, 0));
        if (!doA) {
            for (int l = 0; l < p.nl; ++l)
                lambda_delta_layer(ctx, m, base, packed, samples, factors, info, devPtr, l, p.owner[l]);
            FITRE_CUDA(cudaEventRecord(ctx->inv_fork, main_stream));
            for (size_t i = 0; i < p.jobs.size(); ++i)
                if (p.mine[i] && p.jobs[i].src >= factors && p.jobs[i].src < factors + info->LambdaGSize)
                    start_job(p.jobs[i], ctx->inv_fork);
        } else {
            std::vector<int> order(p.nl);
            for (int l = 0; l < p.nl; ++l) order[l] = l;
            auto block = [&](int l) {
                return l < m->cLayers ? m->convLayer[l].inChannels * m->convLayer[l].kSize * m->convLayer[l].kSize
                                      : m->fcLayer[l - m->cLayers].in;
            };
            std::stable_sort(order.begin(), order.end(), [&](int x, int y) { return block(x) > block(y); });
            for (int l : order) {
                omega_z_layer(ctx, m, x0, base, packed, samples, factors, info, devPtr, l, p.owner[l]);
                FITRE_CUDA(cudaEventRecord(ctx->layer_ev[l], main_stream));
                for (size_t i = 0; i < p.jobs.size(); ++i)
                    if (p.mine[i] && p.jobs[i].src == factors + info->OmegaZOffsets[l])
                        start_job(p.jobs[i], ctx->layer_ev[l]);
            }
        }
    } catch (...) {
        ctx->stream = main_stream;
        throw;
    }
    for (int s = 0; s < kSideStreams; ++s) {
        FITRE_CUDA(cudaEventRecord(ctx->inv_join[s], ctx->inv_streams[s]));
        FITRE_CUDA(cudaStreamWaitEvent(main_stream, ctx->inv_join[s], 0));
    }
}
void ensure_phase_objects(fitre_context *ctx, int nl) {
    ensure_side_streams(ctx);
    while ((int)ctx->layer_ev.size() < nl) {
        cudaEvent_t e;
        FITRE_CUDA(cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
        ctx->layer_ev.push_back(e);
    }
    if (!ctx->phase_stream) {
        FITRE_CUDA(cudaStreamCreateWithFlags(&ctx->phase_stream, cudaStreamNonBlocking));
        FITRE_CUDA(cudaEventCreateWithFlags(&ctx->phase_fork, cudaEventDisableTiming));
        FITRE_CUDA(cudaEventCreateWithFlags(&ctx->phase_done, cudaEventDisableTiming));
    }
}
}  // namespace

extern "C" int fitre_kfac_omega_z_begin(fitre_context *ctx, const CNN_MODEL *m, const real *x0, const real *zbase,
                                        int packed, int samples, real *omegaZ, real *omegaZInv,
                                        const FITRE_KFAC_INFO *info, real *devPtr) {
    KFAC_ENTRY_BEGIN
    FITRE_REQUIRE(m && x0 && zbase && omegaZ && omegaZInv && info && devPtr, FITRE_ERR_BAD_ARG, "NULL pointer argument");
    FITRE_REQUIRE(!ctx->phase_open, FITRE_ERR_BAD_ARG, "fitre_kfac_omega_z_begin called twice without the finish call");
    model_check_batch(m, samples);
    require_scratch(ctx, fitre_kfac_factors_and_inverses_mem_required(m), "fitre_kfac_omega_z_begin");
    // the G side's blocks are not touched here: placeholders that match no A block
    double *none = reinterpret_cast<double *>((uintptr_t)64);
    const PhasePlan p = make_phase_plan(ctx, m, info, omegaZ, omegaZInv, none, none);
    int *fail = (int *)(ctx->dscal + 4002);
    ensure_phase_objects(ctx, p.nl);
    // everything of this call runs on the phase stream (and the side streams forked from it)
    cudaStream_t user = ctx->stream;
    FITRE_CUDA(cudaEventRecord(ctx->phase_fork, user));
    FITRE_CUDA(cudaStreamWaitEvent(ctx->phase_stream, ctx->phase_fork, 0));
    ctx->stream = ctx->phase_stream;
    try {
        std::vector<long long> key = phase_key(ctx, m, info, p, x0, zbase, omegaZ, omegaZInv, devPtr, packed, samples);
        key.push_back(1);
        auto body = [&] {
            FITRE_CUDA(cudaMemsetAsync(fail, 0, sizeof(double), ctx->stream));
            if (ctx->world > 1 && !p.owned) vec_fill(ctx, info->OmegaZSize, 0.0, omegaZInv);
            run_factor_phase(ctx, m, info, p, true, x0, zbase, packed != 0, samples, omegaZ, devPtr, fail);
        };
        if (ctx->world > 1) {
            body();
            if (!p.owned) comm_allreduce_sum(ctx, omegaZInv, info->OmegaZSize);
        } else {
            run_graphed(ctx, ctx->graph_factors_a, key, body);
        }
        FITRE_CUDA(cudaEventRecord(ctx->phase_done, ctx->phase_stream));
    } catch (...) {
        ctx->stream = user;
        throw;
    }
    ctx->stream = user;
    ctx->phase_open = true;
    KFAC_ENTRY_END
}

extern "C" int fitre_kfac_lambda_delta_finish(fitre_context *ctx, const CNN_MODEL *m, const real *dbase, int packed,
                                              int samples, real *lambdaG, real *lambdaGInv,
                                              const FITRE_KFAC_INFO *info, real *devPtr) {
    KFAC_ENTRY_BEGIN
    FITRE_REQUIRE(m && dbase && lambdaG && lambdaGInv && info && devPtr, FITRE_ERR_BAD_ARG, "NULL pointer argument");
    FITRE_REQUIRE(ctx->phase_open, FITRE_ERR_BAD_ARG, "fitre_kfac_lambda_delta_finish without fitre_kfac_omega_z_begin");
    model_check_batch(m, samples);
    require_scratch(ctx, fitre_kfac_factors_and_inverses_mem_required(m), "fitre_kfac_lambda_delta_finish");
    ctx->phase_open = false;
    double *none = reinterpret_cast<double *>((uintptr_t)64);
    const PhasePlan p = make_phase_plan(ctx, m, info, none, none, lambdaG, lambdaGInv);
    int *fail = (int *)(ctx->dscal + 4002);
    ensure_phase_objects(ctx, p.nl);
    // the A side owns the scratch and the side streams until it is done: G comes after it
    FITRE_CUDA(cudaStreamWaitEvent(ctx->stream, ctx->phase_done, 0));
    std::vector<long long> key = phase_key(ctx, m, info, p, dbase, lambdaG, lambdaGInv, devPtr, nullptr, packed, samples);
    key.push_back(2);
    auto body = [&] {
        if (ctx->world > 1 && !p.owned) vec_fill(ctx, info->LambdaGSize, 0.0, lambdaGInv);
        run_factor_phase(ctx, m, info, p, false, nullptr, dbase, packed != 0, samples, lambdaG, devPtr, fail);
    };
    if (ctx->world > 1) {
        body();
        if (!p.owned) comm_allreduce_sum(ctx, lambdaGInv, info->LambdaGSize);
        comm_allreduce_sum(ctx, ctx->dscal + 4002, 1);  // a failure on any rank is seen by all
    } else {
        run_graphed(ctx, ctx->graph_factors_g, key, body);
    }
    check_fail_word(ctx, fail);
    KFAC_ENTRY_END
}

namespace {
long natural_gradient_layer_scratch(const CNN_MODEL *m) {
    long need = 0;
    for (int l = 0; l < m->cLayers; ++l) {
        const CONV_LAYER &c = m->convLayer[l];
        const long Kb = (long)c.inChannels * c.kSize * c.kSize + 1;
        need = std::max(need, 3 * align32(Kb * c.outChannels));
    }
    for (int l = 0; l < m->lLayers; ++l)
        need = std::max(need, align32((long)m->fcLayer[l].out * (m->fcLayer[l].in + 1)));
    return need;
}
}  // namespace

extern "C" long fitre_kfac_natural_gradient_mem_required(const CNN_MODEL *m) {
    if (!m) return -1;
    return kSideStreams * natural_gradient_layer_scratch(m);
}

// nGradient = G^-1 [W|b] A^-1 per layer, in the flat gradient layout.  The layers are independent
// and their products are small next to the GPU, so they are spread over the side streams.
extern "C" int fitre_compute_natural_gradient(fitre_context *ctx, const CNN_MODEL *m,
                                              const FITRE_KFAC_INFO *info, const real *omegaZInv,
                                              const real *lambdaGInv, const real *gradient,
                                              real *nGradient, real *devPtr) {
    if (!ctx) return FITRE_ERR_BAD_ARG;
    try {
        FITRE_CUDA(cudaSetDevice(ctx->device));
        FITRE_REQUIRE(m && info && omegaZInv && lambdaGInv && gradient && nGradient && devPtr,
                      FITRE_ERR_BAD_ARG, "NULL pointer argument");
        require_scratch(ctx, fitre_kfac_natural_gradient_mem_required(m), "fitre_compute_natural_gradient");
        const int hasb = m->bias ? 1 : 0;
        const bool chol = ctx->kfac_solver == FITRE_KFAC_SOLVER_CHOLESKY;
        const long per = natural_gradient_layer_scratch(m);
        ensure_side_streams(ctx);
        const bool owned = ctx->world > 1 && ctx->kfac_owned;
        std::vector<int> owner;
        if (owned) owner = layer_owners(m, ctx->world, chol);
        std::vector<long long> key = {ptr_key(omegaZInv), ptr_key(lambdaGInv), ptr_key(gradient), ptr_key(nGradient),
                                      ptr_key(devPtr), ctx->kfac_solver, hasb, m->cLayers, m->lLayers,
                                      owned ? ctx->rank : -1, owned ? ctx->world : 1, m->pSize};
        for (int l = 0; l < m->cLayers + m->lLayers; ++l) {
            key.push_back(info->OmegaZOffsets[l]);
            key.push_back(info->LambdaGOffsets[l]);
            key.push_back(m->wOffsets[l]);
            key.push_back(m->bOffsets[l]);
            key.push_back(l < m->cLayers ? m->convLayer[l].outChannels : m->fcLayer[l - m->cLayers].out);
            key.push_back(l < m->cLayers ? m->convLayer[l].inChannels * m->convLayer[l].kSize * m->convLayer[l].kSize
                                         : m->fcLayer[l - m->cLayers].in);
        }
        run_graphed(ctx, ctx->graph_natgrad, key, [&] {
        cudaStream_t main_stream = ctx->stream;
        if (owned) vec_fill(ctx, m->pSize, 0.0, nGradient);  // the other ranks' slices arrive by the all-reduce
        FITRE_CUDA(cudaEventRecord(ctx->inv_fork, main_stream));
        for (int s = 0; s < kSideStreams; ++s) FITRE_CUDA(cudaStreamWaitEvent(ctx->inv_streams[s], ctx->inv_fork, 0));
        std::vector<double> sload(kSideStreams, 0.0);
        auto pick_stream = [&](double cost) {
            const int s = (int)(std::min_element(sload.begin(), sload.end()) - sload.begin());
            sload[s] += cost;
            ctx->stream = ctx->inv_streams[s];
            return devPtr + (long)s * per;
        };
        try {
            // largest layers first, so that the long chains start early
            std::vector<int> order(m->cLayers + m->lLayers);
            std::vector<double> cost(order.size());
            for (int l = 0; l < (int)order.size(); ++l) {
                order[l] = l;
                const double kb = l < m->cLayers ? (double)m->convLayer[l].inChannels * m->convLayer[l].kSize *
                                                       m->convLayer[l].kSize
                                                 : (double)m->fcLayer[l - m->cLayers].in;
                const double co = l < m->cLayers ? m->convLayer[l].outChannels : m->fcLayer[l - m->cLayers].out;
                cost[l] = co * kb * (kb + co);
            }
            std::stable_sort(order.begin(), order.end(), [&](int x, int y) { return cost[x] > cost[y]; });
            for (int li : order) {
                if (owned && owner[li] != ctx->rank) continue;
                double *work = pick_stream(cost[li]);
                const double *Ai = omegaZInv + info->OmegaZOffsets[li];
                const double *Gi = lambdaGInv + info->LambdaGOffsets[li];
                if (li < m->cLayers) {
                    const CONV_LAYER &L = m->convLayer[li];
                    const int K = L.inChannels * L.kSize * L.kSize, Kb = K + hasb, Co = L.outChannels;
                    const long sz = align32((long)Kb * Co);
                    double *wb = work, *t1 = wb + sz, *t2 = t1 + sz;
                    pack_wb_kernel<<<blocks_for((long)Kb * Co), 256, 0, ctx->stream>>>(
                        gradient + m->wOffsets[li], hasb ? gradient + m->bOffsets[li] : nullptr, wb, K, Kb, Co);
                    check_launch(ctx, "pack_wb_kernel");
                    dgemm(ctx, false, true, Co, Kb, Co, 1.0, Gi, Co, wb, Kb, 0.0, t1, Co);  // G^-1 wb'
                    if (chol) {  // ... A^-1 = L^-T L^-1 by two solves in place
                        trsm_right(ctx, t1, Co, Co, Ai, Kb, Kb, true);
                        trsm_right(ctx, t1, Co, Co, Ai, Kb, Kb, false);
                        t2 = t1;
                    } else {
                        dgemm(ctx, false, false, Co, Kb, Kb, 1.0, t1, Co, Ai, Kb, 0.0, t2, Co);  // ... A^-1
                    }
                    unpack_ng_kernel<<<blocks_for((long)Kb * Co), 256, 0, ctx->stream>>>(
                        t2, nGradient + m->wOffsets[li], hasb ? nGradient + m->bOffsets[li] : nullptr, K, Kb, Co);
                    check_launch(ctx, "unpack_ng_kernel");
                } else {
                    const FC_LAYER &F = m->fcLayer[li - m->cLayers];
                    const int in = F.in + hasb;
                    // [W | b] is contiguous in the flat layout: out x (in + bias), column-major
                    double *ng = nGradient + m->wOffsets[li];
                    if (chol) {
                        dgemm(ctx, false, false, F.out, in, F.out, 1.0, Gi, F.out, gradient + m->wOffsets[li],
                              F.out, 0.0, ng, F.out);
                        trsm_right(ctx, ng, F.out, F.out, Ai, in, in, true);
                        trsm_right(ctx, ng, F.out, F.out, Ai, in, in, false);
                    } else {
                        dgemm(ctx, false, false, F.out, in, F.out, 1.0, Gi, F.out, gradient + m->wOffsets[li],
                              F.out, 0.0, work, F.out);
                        dgemm(ctx, false, false, F.out, in, in, 1.0, work, F.out, Ai, in, 0.0, ng, F.out);
                    }
                }
            }
        } catch (...) {
            ctx->stream = main_stream;
            throw;
        }
        ctx->stream = main_stream;
        for (int s = 0; s < kSideStreams; ++s) {
            FITRE_CUDA(cudaEventRecord(ctx->inv_join[s], ctx->inv_streams[s]));
            FITRE_CUDA(cudaStreamWaitEvent(main_stream, ctx->inv_join[s], 0));
        }
        });
        if (owned) comm_allreduce_sum(ctx, nGradient, (size_t)m->pSize);
        return FITRE_OK;
    } catch (const Error &e) {
        ctx->err = e.what();
        return e.code;
    }
}
