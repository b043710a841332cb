// KFAC factor accumulation: A = activation covariance, G = error covariance, per layer.
// Reference: solvers/kfac_utils.cu:7-55 (block offsets), solvers/kfac_inverses.cu:450-630
// (computeOmegaZ) and :759-857 (computeLambdaDelta).  The reference materialises the im2col
// matrix and calls cublasDgemm for the full square; here the convolution A factor is a
// tensor-core SYRK over implicit patches (lower tiles only) and every factor is summed over
// the data-parallel ranks before the 1/N (A) or N (G) scaling with the global batch.
#include <algorithm>
#include <climits>

#include "common.h"

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

extern "C" int fitre_kfac_omega_z(fitre_context *ctx, const CNN_MODEL *m,
                                  const DEVICE_DATASET *data, const real *z, int samples,
                                  real *omegaZ, const FITRE_KFAC_INFO *info, real *devPtr) {
    if (!ctx) return FITRE_ERR_BAD_ARG;
    try {
        FITRE_CUDA(cudaSetDevice(ctx->device));
        FITRE_REQUIRE(m && data && z && omegaZ && info && devPtr, FITRE_ERR_BAD_ARG, "NULL pointer argument");
        model_check_batch(m, samples);
        const double Ng = (double)samples * ctx->world;
        for (int l = 0; l < m->cLayers; ++l) {
            const ConvGeom g = conv_geom(m, l);
            const double *x = (l == 0) ? data->currentBatch
                                       : z + m->zOffsets[l] + m->convLayer[l - 1].outputOffset;
            double *A = omegaZ + info->OmegaZOffsets[l];
            const int Kb = g.Cin * g.k * g.k + (m->bias ? 1 : 0);
            // sum over ranks first, then 1/N: with world == 1 the scale is applied directly
            const double alpha = ctx->world > 1 ? 1.0 : 1.0 / Ng;
            conv_patch_syrk(ctx, x, A, samples, g.Cin, g.H, g.W, g.k, g.pad, m->bias != 0, alpha,
                            1.0 / (double)(g.Ho * g.Wo), devPtr);
            if (ctx->world > 1) {
                comm_allreduce_sum(ctx, A, (size_t)Kb * Kb);
                vec_scale(ctx, (long)Kb * Kb, 1.0 / Ng, A);
            }
        }
        const ConvGeom lg = conv_geom(m, m->cLayers - 1);
        for (int l = 0; l < m->lLayers; ++l) {
            const FC_LAYER &f = m->fcLayer[l];
            const double *zin = (l == 0) ? z + lg.zoff + lg.outOff : z + m->zOffsets[m->cLayers + l];
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
            if (ctx->world > 1) {
                comm_allreduce_sum(ctx, A, (size_t)R * R);
                vec_scale(ctx, (long)R * R, 1.0 / Ng, A);
            }
        }
        return FITRE_OK;
    } catch (const Error &e) {
        ctx->err = e.what();
        return e.code;
    }
}

extern "C" int fitre_kfac_lambda_delta(fitre_context *ctx, const CNN_MODEL *m, const real *dx,
                                       int samples, real *lambdaG, const FITRE_KFAC_INFO *info,
                                       real *devPtr) {
    if (!ctx) return FITRE_ERR_BAD_ARG;
    try {
        FITRE_CUDA(cudaSetDevice(ctx->device));
        FITRE_REQUIRE(m && dx && lambdaG && info && devPtr, FITRE_ERR_BAD_ARG, "NULL pointer argument");
        model_check_batch(m, samples);
        const double Ng = (double)samples * ctx->world;
        for (int l = 0; l < m->cLayers; ++l) {
            const ConvGeom g = conv_geom(m, l);
            const double *d = dx + g.zoff + (g.bn ? g.bnOff : g.actOff);
            const long M = (long)samples * g.Ho * g.Wo;
            double *G = lambdaG + info->LambdaGOffsets[l];
            const double sc = (double)g.Ho * g.Wo * Ng;  // solvers/kfac_inverses.cu:815-816
            syrk_tn(ctx, M, g.Cout, ctx->world > 1 ? 1.0 : sc, d, M, G, devPtr);
            if (ctx->world > 1) {
                comm_allreduce_sum(ctx, G, (size_t)g.Cout * g.Cout);
                vec_scale(ctx, (long)g.Cout * g.Cout, sc, G);
            }
        }
        for (int l = 0; l < m->lLayers; ++l) {
            const FC_LAYER &f = m->fcLayer[l];
            const double *d = dx + m->zOffsets[m->cLayers + l + 1];
            double *G = lambdaG + info->LambdaGOffsets[m->cLayers + l];
            dgemm(ctx, false, true, f.out, f.out, samples, ctx->world > 1 ? 1.0 : Ng, d, f.out, d,
                  f.out, 0.0, G, f.out);
            if (ctx->world > 1) {
                comm_allreduce_sum(ctx, G, (size_t)f.out * f.out);
                vec_scale(ctx, (long)f.out * f.out, Ng, G);
            }
        }
        return FITRE_OK;
    } catch (const Error &e) {
        ctx->err = e.what();
        return e.code;
    }
}
