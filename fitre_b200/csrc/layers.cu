// HBM-bound layer kernels: batch norm (forward, backward and both R-op directions),
// activations and their first/second derivatives, pooling (forward, gather-form backward,
// R-forward), softmax cross-entropy, layout changes at the conv<->FC boundary and
// parameter-vector helpers.
//
// One skeleton serves every per-channel pass: block (c, s) walks slice s of channel c's
// N*H*W block, applies an element functor (which may write outputs) and reduces up to NS
// per-channel sums with warp shuffles + shared memory.  Slice partials are summed in a
// fixed order by a second kernel, so results are bit-reproducible; the finished C*NS vector
// is what gets all-reduced across data-parallel ranks (sync batch norm).
//
// Reference maths: functions/dev_batch_norm.cu:263-960, dev_pool.cu:41-497, swish.cu:14-84,
// dev_activations.cu:8-39, dev_layer_error.cu:34-47, dev_layer_r_error.cu:24-38,
// softmax_loss.cu:17-299, dev_transpose.cu:8-30, dev_backprop_convolution.cu:140-156.
#include <algorithm>
#include <cfloat>

#include "common.h"

namespace fitre {
namespace {

constexpr int kThreads = 256;
constexpr long kScratchDoubles = 32768;

// ---- activation maths ------------------------------------------------------------------
__device__ __forceinline__ double act_fwd(int act, double x) {
    switch (act) {
        case FITRE_CNN_ACT_RELU: return x < 0 ? 0.0 : x;
        case FITRE_CNN_ACT_SOFTPLUS: return x < 20 ? log(1 + exp(x)) : x;
        case FITRE_CNN_ACT_SWISH: return x / (1 + exp(-x));
        default: return x;
    }
}
__device__ __forceinline__ double act_d1(int act, double zin, double zout) {
    switch (act) {
        case FITRE_CNN_ACT_RELU: return zin > 0 ? 1.0 : 0.0;
        case FITRE_CNN_ACT_SOFTPLUS: return 1. / (1. + exp(-zin));
        case FITRE_CNN_ACT_SWISH: {
            const double t = 1. / (1. + exp(-zin));
            return zout + t * (1. - zout);
        }
        default: return 1.0;
    }
}
__device__ __forceinline__ double act_d2(int act, double zin, double zout) {
    switch (act) {
        case FITRE_CNN_ACT_SOFTPLUS: {
            const double tm = exp(-zin);
            return (1. / (1. + tm)) * (tm / (1. + tm));
        }
        case FITRE_CNN_ACT_SWISH: {
            const double t = 1. / (1. + exp(-zin));
            return (1. - t) * (zout + 2. * t * (1. - zout));
        }
        default: return 0.0;
    }
}

// ---- per-channel map + reduce skeleton ---------------------------------------------------
template <int NS>
__device__ __forceinline__ void block_reduce_store(double (&acc)[NS], double *dst) {
    __shared__ double red[NS][kThreads / 32];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int k = 0; k < NS; ++k) {
        double v = acc[k];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
        if (lane == 0) red[k][warp] = v;
    }
    __syncthreads();
    if (threadIdx.x < NS) {
        double s = 0.0;
#pragma unroll
        for (int w = 0; w < kThreads / 32; ++w) s += red[threadIdx.x][w];
        dst[threadIdx.x] = s;
    }
}

template <int NS, class Op>
__global__ void __launch_bounds__(kThreads) channel_pass_kernel(Op op, long rows, int S,
                                                                double *partials) {
    const int c = blockIdx.x, s = blockIdx.y;
    const long per = (rows + S - 1) / S;
    const long beg = (long)s * per;
    const long end = min(rows, beg + per);
    double acc[NS > 0 ? NS : 1];
#pragma unroll
    for (int k = 0; k < (NS > 0 ? NS : 1); ++k) acc[k] = 0.0;
    for (long r = beg + threadIdx.x; r < end; r += kThreads) op(c, r, acc);
    if (NS > 0) block_reduce_store<(NS > 0 ? NS : 1)>(acc, partials + ((long)c * S + s) * NS);
}

__global__ void finalize_partials_kernel(const double *partials, int C, int S, int NS,
                                         double *out) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= C * NS) return;
    const int c = i / NS, k = i - c * NS;
    double s = 0.0;
    for (int j = 0; j < S; ++j) s += partials[((long)c * S + j) * NS + k];
    out[i] = s;
}

int slices_for(int C, long rows) {
    long want = (148L * 8 + C - 1) / C;
    long cap = std::max(1L, rows / 2048);
    long S = std::max(1L, std::min(want, cap));
    // scratch holds C*S*NS partials + C*NS sums, NS <= 7
    while (S > 1 && (long)C * (S + 1) * 7 > kScratchDoubles) --S;
    return (int)S;
}

// Runs op over a [C][rows] tensor; if NS > 0 leaves the per-channel sums (C x NS, row-major by
// channel) at `sums` (= scratch) and, when `sync`, all-reduces them over the ranks.
template <int NS, class Op>
double *channel_pass(fitre_context *ctx, const Op &op, int C, long rows, double *scratch,
                     bool sync, const char *name) {
    FITRE_REQUIRE((long)C * 2 * 7 <= kScratchDoubles, FITRE_ERR_TOO_LARGE, "too many channels");
    const int S = slices_for(C, rows);
    double *sums = scratch;
    double *partials = scratch + (long)C * (NS > 0 ? NS : 1);
    dim3 grid(C, S);
    channel_pass_kernel<NS, Op><<<grid, kThreads, 0, ctx->stream>>>(op, rows, S, partials);
    check_launch(ctx, name);
    if (NS > 0) {
        const int n = C * NS;
        finalize_partials_kernel<<<(n + 127) / 128, 128, 0, ctx->stream>>>(partials, C, S, NS, sums);
        check_launch(ctx, "finalize_partials_kernel");
        if (sync) comm_allreduce_sum(ctx, sums, n);
    }
    return sums;
}

// ---- functors ------------------------------------------------------------------------------
struct SumOp {  // sum x
    const double *x;
    long rows;
    __device__ void operator()(int c, long r, double (&a)[1]) const { a[0] += x[(long)c * rows + r]; }
};
struct VarOp {  // sum (x - mean)^2, mean = sums[c] * inv_m
    const double *x, *sum;
    long rows;
    double inv_m;
    __device__ void operator()(int c, long r, double (&a)[1]) const {
        const double d = x[(long)c * rows + r] - sum[c] * inv_m;
        a[0] += d * d;
    }
};
__global__ void bn_stats_store_kernel(const double *sum, const double *ssq, double inv_m, int C,
                                      double *mean, double *var, double *run_mean,
                                      double *run_var) {
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= C) return;
    const double mu = sum[c] * inv_m, v = ssq[c] * inv_m;
    mean[c] = mu;
    var[c] = v;
    // running statistics, momentum 0.9 (functions/dev_batch_norm.cu:307-314)
    run_mean[c] = 0.9 * run_mean[c] + 0.1 * mu;
    run_var[c] = 0.9 * run_var[c] + 0.1 * v;
}
struct NormActOp {  // bn out (optional) and activation out
    const double *x, *mean, *var;
    double *bn, *actout;
    long rows;
    int act, has_bn;
    __device__ void operator()(int c, long r, double (&)[1]) const {
        const long i = (long)c * rows + r;
        double v = x[i];
        if (has_bn) {
            v = (v - mean[c]) / sqrt(var[c] + kBnEps);
            bn[i] = v;
        }
        actout[i] = act_fwd(act, v);
    }
};

struct PoolGeom {
    int type, pk, ps, pp, H, W, Hp, Wp;  // H,W: pool input (= conv output) plane
};

// arg-max of one pooling window, scan order of the backward kernel: column outer, row inner,
// strict '>' (functions/dev_pool.cu:374-391).  Returns w*H + h of the winner.
__device__ __forceinline__ int window_argmax(const double *plane, const PoolGeom &g, int k, int l) {
    const int i0 = k * g.ps - g.pp, j0 = l * g.ps - g.pp;  // == (k-1)*ps + pk - 2*pp when pk-ps == pp
    double best = -DBL_MAX;
    int arg = -1;
    for (int cc = 0; cc < g.pk; ++cc) {
        const int w = j0 + cc;
        if (w < 0 || w >= g.W) continue;
        for (int rr = 0; rr < g.pk; ++rr) {
            const int h = i0 + rr;
            if (h < 0 || h >= g.H) continue;
            const double t = plane[w * g.H + h];
            if (t > best) {
                best = t;
                arg = w * g.H + h;
            }
        }
    }
    return arg;
}

// errors arriving at element (h, w) of one plane through the pooling layer (gather form of
// functions/dev_pool.cu:269-298,346-398 and the 1/k^2 scale of functions/cnn_backward.cu:471-473)
__device__ __forceinline__ double pool_gather(const double *dpool_plane, const double *act_plane,
                                              const PoolGeom &g, int h, int w) {
    if (g.type == FITRE_NO_POOL) return dpool_plane[w * g.H + h];
    if (g.type == FITRE_AVG_POOL) {
        const int k = h / g.pk, l = w / g.pk;
        return (k < g.Hp && l < g.Wp) ? dpool_plane[l * g.Hp + k] / (double)(g.pk * g.pk) : 0.0;
    }
    // windows k with k*ps - pp <= h < k*ps - pp + pk
    int kmin = (h + g.pp - g.pk + g.ps) / g.ps;  // ceil((h + pp - pk + 1) / ps) for non-negative args
    if (h + g.pp - g.pk + 1 <= 0) kmin = 0;
    const int kmax = min((h + g.pp) / g.ps, g.Hp - 1);
    int lmin = (w + g.pp - g.pk + g.ps) / g.ps;
    if (w + g.pp - g.pk + 1 <= 0) lmin = 0;
    const int lmax = min((w + g.pp) / g.ps, g.Wp - 1);
    const int me = w * g.H + h;
    double s = 0.0;
    for (int l = lmin; l <= lmax; ++l)
        for (int k = kmin; k <= kmax; ++k)
            if (window_argmax(act_plane, g, k, l) == me) s += dpool_plane[l * g.Hp + k];
    return s;
}

template <int NS>
struct PoolActBwdOp {  // dxP, dxA (+ sums: dA [, dA*zhat])
    const double *dpool, *actv, *zin;
    double *dxP, *dxA;
    long rows;
    PoolGeom g;
    int act;
    __device__ void operator()(int c, long r, double (&a)[NS > 0 ? NS : 1]) const {
        const int hw = g.H * g.W;
        const long n = r / hw;
        const int rem = (int)(r - n * hw);
        const int w = rem / g.H, h = rem - w * g.H;
        const long i = (long)c * rows + r;
        const long plane = (long)c * rows + n * hw;
        const long pplane = g.type == FITRE_NO_POOL
                                ? plane
                                : ((long)c * (rows / hw) + n) * (g.Hp * g.Wp);
        const double dP = pool_gather(dpool + pplane, actv + plane, g, h, w);
        dxP[i] = dP;
        const double zi = zin[i];
        const double dA = dP * act_d1(act, zi, actv[i]);
        dxA[i] = dA;
        if (NS >= 1) a[0] += dA;
        if (NS >= 2) a[1] += dA * zi;
    }
};

template <int NS>
struct BnBwdApplyOp {  // dBN = (m dA - s1 - zhat s2) / (m sigma)   (+ sum dBN)
    const double *dA, *zhat, *var, *sums;  // sums: [C][2] = (sum dA, sum dA*zhat)
    double *out;
    long rows;
    double m;
    __device__ void operator()(int c, long r, double (&a)[NS > 0 ? NS : 1]) const {
        const long i = (long)c * rows + r;
        const double v = (dA[i] * m - sums[2 * c] - sums[2 * c + 1] * zhat[i]) /
                         (m * sqrt(kBnEps + var[c]));
        out[i] = v;
        if (NS >= 1) a[0] += v;
    }
};

struct RbnSumsOp {  // sum Rz, sum (z-mu) Rz, sum (z-mu)
    const double *z, *rz, *mean;
    long rows;
    __device__ void operator()(int c, long r, double (&a)[3]) const {
        const long i = (long)c * rows + r;
        const double d = z[i] - mean[c], t = rz[i];
        a[0] += t;
        a[1] += d * t;
        a[2] += d;
    }
};
struct RNormActOp {  // R bn-out, R act-out
    const double *z, *rz, *mean, *var, *sums, *zin, *actv;
    double *rbn, *ract;
    long rows;
    double m;
    int act, has_bn;
    __device__ void operator()(int c, long r, double (&)[1]) const {
        const long i = (long)c * rows + r;
        double v = rz[i];
        if (has_bn) {
            const double rmean = sums[3 * c] / m;
            // sum (z-mu)(Rz - mean Rz) = sum (z-mu) Rz - mean Rz * sum (z-mu)
            const double s = sums[3 * c + 1] - rmean * sums[3 * c + 2];
            const double ve = var[c] + kBnEps, sd = sqrt(ve);
            v = (v - rmean) / sd - s * (z[i] - mean[c]) / (m * ve * sd);
            rbn[i] = v;
        }
        ract[i] = v * act_d1(act, zin[i], actv[i]);
    }
};

template <int NS>
struct RPoolActBwdOp {  // RdA = h' RdP + h'' Rzin dxP   (+ sums, see conv_post_rop_backward)
    const double *rdpool, *actv, *zin, *rzin, *dxP, *dxA, *zconv, *rzconv, *mean;
    double *rout;
    long rows;
    PoolGeom g;
    int act;
    __device__ void operator()(int c, long r, double (&a)[NS > 0 ? NS : 1]) const {
        const int hw = g.H * g.W;
        const long n = r / hw;
        const int rem = (int)(r - n * hw);
        const int w = rem / g.H, h = rem - w * g.H;
        const long i = (long)c * rows + r;
        const long plane = (long)c * rows + n * hw;
        const long pplane = g.type == FITRE_NO_POOL
                                ? plane
                                : ((long)c * (rows / hw) + n) * (g.Hp * g.Wp);
        const double RdP = pool_gather(rdpool + pplane, actv + plane, g, h, w);
        const double zi = zin[i], zo = actv[i];
        const double RdA = act_d1(act, zi, zo) * RdP + act_d2(act, zi, zo) * rzin[i] * dxP[i];
        rout[i] = RdA;
        if (NS == 1) a[0] += RdA;
        if (NS == 7) {
            const double dA = dxA[i], rzh = rzin[i];
            const double d = zconv[i] - mean[c], rzc = rzconv[i];
            a[0] += RdA;
            a[1] += dA * zi;
            a[2] += dA * rzh + zi * RdA;
            a[3] += dA;
            a[4] += rzc;
            a[5] += d * rzc;
            a[6] += d;
        }
    }
};

template <int NS>
struct RBnBwdApplyOp {
    const double *dA, *zhat, *rzhat, *var, *sums;  // sums [C][7]
    double *rout;
    long rows;
    double m;
    __device__ void operator()(int c, long r, double (&a)[NS > 0 ? NS : 1]) const {
        const long i = (long)c * rows + r;
        const double *s = sums + 7 * c;
        const double ve = var[c] + kBnEps, sd = sqrt(ve);
        const double zh = zhat[i];
        const double rII = (rout[i] * m - s[0] - s[1] * rzhat[i] - s[2] * zh) / (m * sd);
        const double II = dA[i] * m - s[3] - s[1] * zh;
        const double rmean = s[4] / m;
        const double rI = -(s[5] - rmean * s[6]) / (m * m * ve * sd);
        const double v = rII + II * rI;
        rout[i] = v;
        if (NS >= 1) a[0] += v;
    }
};

// ---- stand-alone kernels ---------------------------------------------------------------------
__global__ void pool_forward_kernel(const double *in, double *out, long planes, PoolGeom g) {
    const long total = planes * g.Hp * g.Wp;
    for (long idx = blockIdx.x * (long)blockDim.x + threadIdx.x; idx < total;
         idx += (long)gridDim.x * blockDim.x) {
        const long pl = idx / (g.Hp * g.Wp);
        const int rem = (int)(idx - pl * (g.Hp * g.Wp));
        const int l = rem / g.Hp, k = rem - l * g.Hp;
        const double *src = in + pl * (long)(g.H * g.W);
        const int i0 = k * g.ps - g.pp, j0 = l * g.ps - g.pp;
        double val = g.type == FITRE_MAX_POOL ? -DBL_MAX : 0.0;
        for (int rr = 0; rr < g.pk; ++rr)
            for (int cc = 0; cc < g.pk; ++cc) {
                const int h = i0 + rr, w = j0 + cc;
                if (h < 0 || w < 0 || h >= g.H || w >= g.W) continue;
                const double t = src[w * g.H + h];
                if (g.type == FITRE_MAX_POOL) {
                    if (t > val) val = t;
                } else {
                    val += t;
                }
            }
        if (g.type != FITRE_MAX_POOL) val /= (double)(g.pk * g.pk);
        out[idx] = val;
    }
}

// R{max pool}: value of rz at the arg-max of the activation (functions/dev_pool.cu:123-174)
__global__ void rop_max_pool_kernel(const double *rz, const double *actv, double *out, long planes,
                                    PoolGeom g) {
    const long total = planes * g.Hp * g.Wp;
    for (long idx = blockIdx.x * (long)blockDim.x + threadIdx.x; idx < total;
         idx += (long)gridDim.x * blockDim.x) {
        const long pl = idx / (g.Hp * g.Wp);
        const int rem = (int)(idx - pl * (g.Hp * g.Wp));
        const int l = rem / g.Hp, k = rem - l * g.Hp;
        const long base = pl * (long)(g.H * g.W);
        const int arg = window_argmax(actv + base, g, k, l);
        out[idx] = arg >= 0 ? rz[base + arg] : 0.0;
    }
}

__global__ void channel_bias_kernel(double *x, const double *bias, long rows, long total) {
    for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < total;
         i += (long)gridDim.x * blockDim.x)
        x[i] += bias[i / rows];
}
__global__ void column_bias_kernel(double *x, const double *bias, int rows, long total) {
    for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < total;
         i += (long)gridDim.x * blockDim.x)
        x[i] += bias[i % rows];
}
__global__ void activation_kernel(int act, const double *in, double *out, long n) {
    for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < n;
         i += (long)gridDim.x * blockDim.x)
        out[i] = act_fwd(act, in[i]);
}
__global__ void act_backward_kernel(int act, double *delta, const double *zin, const double *zout,
                                    long n) {
    for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < n;
         i += (long)gridDim.x * blockDim.x)
        delta[i] *= act_d1(act, zin[i], zout[i]);
}
__global__ void act_rop_backward_kernel(int act, double *rdelta, const double *din,
                                        const double *rzin, const double *zin, const double *zout,
                                        long n) {
    for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < n;
         i += (long)gridDim.x * blockDim.x)
        rdelta[i] = act_d1(act, zin[i], zout[i]) * rdelta[i] +
                    act_d2(act, zin[i], zout[i]) * rzin[i] * din[i];
}

// [C][N][Wp][Hp] (h fastest) -> [N][C*P] with feature c*P + h*Wp + w  (square planes)
__global__ void conv_to_fc_kernel(const double *in, double *out, int C, int N, int Hp, int Wp) {
    const long P = (long)Hp * Wp, total = P * C * N;
    for (long idx = blockIdx.x * (long)blockDim.x + threadIdx.x; idx < total;
         idx += (long)gridDim.x * blockDim.x) {
        const long c = idx / (N * P);
        const long r = idx - c * N * P;
        const long n = r / P;
        const int q = (int)(r - n * P);
        const int w = q / Hp, h = q - w * Hp;
        out[n * (C * P) + c * P + (long)h * Wp + w] = in[idx];
    }
}
__global__ void fc_to_conv_kernel(const double *in, double *out, int C, int N, int Hp, int Wp) {
    const long P = (long)Hp * Wp, total = P * C * N;
    for (long idx = blockIdx.x * (long)blockDim.x + threadIdx.x; idx < total;
         idx += (long)gridDim.x * blockDim.x) {
        const long c = idx / (N * P);
        const long r = idx - c * N * P;
        const long n = r / P;
        const int q = (int)(r - n * P);
        const int w = q / Hp, h = q - w * Hp;
        out[idx] = in[n * (C * P) + c * P + (long)h * Wp + w];
    }
}

// out[i] = sum_j x[i + j*rows]   (FC bias gradient, functions/cnn_backward.cu:221)
__global__ void row_sums_kernel(const double *x, int rows, int cols, double *out) {
    const int i = blockIdx.x;
    double s = 0.0;
    for (int j = threadIdx.x; j < cols; j += blockDim.x) s += x[(long)j * rows + i];
    double acc[1] = {s};
    __shared__ double red[32];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    double v = acc[0];
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    if (lane == 0) red[warp] = v;
    __syncthreads();
    if (threadIdx.x == 0) {
        double t = 0.0;
        for (int w = 0; w < (blockDim.x + 31) / 32; ++w) t += red[w];
        out[i] = t;
    }
}

// softmax + probabilities + errors + loss (one thread per sample; one block, fixed order)
__global__ void softmax_loss_kernel(const double *logits, const double *labels, int N,
                                    int classes, double *probs, double *errors, double inv_ng,
                                    int ref_quirks, double *loss_out) {
    double local = 0.0;
    for (int r = threadIdx.x; r < N; r += blockDim.x) {
        const double *x = logits + (long)r * classes;
        double *p = probs + (long)r * classes;
        double mx = ref_quirks ? 0.0 : -DBL_MAX;  // functions/softmax_loss.cu:24-27
        for (int i = 0; i < classes; ++i)
            if (mx < x[i]) mx = x[i];
        double s = 0.0;
        for (int i = 0; i < classes; ++i) {
            const double e = exp(x[i] - mx);
            p[i] = e;
            s += e;
        }
        const int y = (int)labels[r];
        for (int i = 0; i < classes; ++i) {
            const double pi = p[i] / s + (ref_quirks ? 1e-10 : 0.0);  // :55
            p[i] = pi;
            if (y == i + 1) local += -log(pi);
            errors[(long)r * classes + i] = (pi - ((double)(i + 1) == labels[r] ? 1.0 : 0.0)) * inv_ng;
        }
    }
    __shared__ double red[kThreads];
    red[threadIdx.x] = local;
    __syncthreads();
    if (threadIdx.x == 0) {
        double t = 0.0;
        for (int i = 0; i < blockDim.x; ++i) t += red[i];
        loss_out[0] = t;
    }
}
__global__ void softmax_rop_error_kernel(const double *rz, const double *probs, int N, int classes,
                                         double *rerr, double inv_ng) {
    const int r = blockIdx.x * blockDim.x + threadIdx.x;
    if (r >= N) return;
    double s = 0.0;
    for (int j = 0; j < classes; ++j) s += probs[(long)r * classes + j] * rz[(long)r * classes + j];
    for (int i = 0; i < classes; ++i)
        rerr[(long)r * classes + i] =
            probs[(long)r * classes + i] * (rz[(long)r * classes + i] - s) * inv_ng;
}

__global__ void axpby_kernel(long n, double a, const double *x, double b, double *y) {
    for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < n;
         i += (long)gridDim.x * blockDim.x)
        y[i] = a * x[i] + (b == 0.0 ? 0.0 : b * y[i]);
}
__global__ void fill_kernel(long n, double v, double *x) {
    for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < n;
         i += (long)gridDim.x * blockDim.x)
        x[i] = v;
}
constexpr int kDotBlocks = 296;
__global__ void dots_partial_kernel(long n, const double *a0, const double *b0, const double *a1,
                                    const double *b1, const double *a2, const double *b2,
                                    double *partials) {
    double acc[3] = {0.0, 0.0, 0.0};
    for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < n;
         i += (long)gridDim.x * blockDim.x) {
        if (a0) acc[0] += a0[i] * b0[i];
        if (a1) acc[1] += a1[i] * b1[i];
        if (a2) acc[2] += a2[i] * b2[i];
    }
    block_reduce_store<3>(acc, partials + 3 * blockIdx.x);
}
__global__ void dots_final_kernel(const double *partials, int blocks, double *out) {
    if (threadIdx.x < 3) {
        double s = 0.0;
        for (int b = 0; b < blocks; ++b) s += partials[3 * b + threadIdx.x];
        out[threadIdx.x] = s;
    }
}

int grid_for(long n) { return (int)std::max<long>(1, std::min<long>((n + kThreads - 1) / kThreads, 148 * 8)); }

PoolGeom pool_geom(const ConvGeom &g) {
    PoolGeom p;
    p.type = g.poolType;
    p.pk = g.pk; p.ps = g.ps; p.pp = g.pp;
    p.H = g.Ho; p.W = g.Wo;
    p.Hp = g.Hp; p.Wp = g.Wp;
    return p;
}

}  // namespace

long bn_scratch(int) { return kScratchDoubles; }

void add_channel_bias(fitre_context *ctx, double *x, const double *bias, long rows, int C) {
    const long total = rows * C;
    channel_bias_kernel<<<grid_for(total), kThreads, 0, ctx->stream>>>(x, bias, rows, total);
    check_launch(ctx, "channel_bias_kernel");
}
void add_column_bias(fitre_context *ctx, double *x, const double *bias, int rows, int cols) {
    const long total = (long)rows * cols;
    column_bias_kernel<<<grid_for(total), kThreads, 0, ctx->stream>>>(x, bias, rows, total);
    check_launch(ctx, "column_bias_kernel");
}
void apply_activation(fitre_context *ctx, int act, const double *in, double *out, long n) {
    activation_kernel<<<grid_for(n), kThreads, 0, ctx->stream>>>(act, in, out, n);
    check_launch(ctx, "activation_kernel");
}
void act_backward(fitre_context *ctx, int act, double *delta, const double *zin,
                  const double *zout, long n) {
    if (act == FITRE_CNN_ACT_NONE || act == FITRE_ACT_LINEAR) return;
    act_backward_kernel<<<grid_for(n), kThreads, 0, ctx->stream>>>(act, delta, zin, zout, n);
    check_launch(ctx, "act_backward_kernel");
}
void act_rop_backward(fitre_context *ctx, int act, double *rdelta, const double *delta_in,
                      const double *rzin, const double *zin, const double *zout, long n) {
    if (act == FITRE_CNN_ACT_NONE || act == FITRE_ACT_LINEAR) return;
    act_rop_backward_kernel<<<grid_for(n), kThreads, 0, ctx->stream>>>(act, rdelta, delta_in, rzin,
                                                                       zin, zout, n);
    check_launch(ctx, "act_rop_backward_kernel");
}

void conv_post_forward(fitre_context *ctx, const ConvGeom &g, int N, double *zl, double *scratch) {
    const long rows = (long)N * g.Ho * g.Wo;
    const double m = (double)rows * ctx->world;
    double *bn = g.bn ? zl + g.bnOff : nullptr;
    double *mean = g.bn ? bn + g.meanOff : nullptr;
    double *var = g.bn ? bn + g.varOff : nullptr;
    if (g.bn) {
        // two-pass batch statistics (functions/dev_batch_norm.cu:263-315)
        double *sum = channel_pass<1>(ctx, SumOp{zl, rows}, g.Cout, rows, scratch, true, "bn_sum");
        double *sum_keep = scratch + kScratchDoubles - g.Cout;  // parked above the partials
        FITRE_CUDA(cudaMemcpyAsync(sum_keep, sum, sizeof(double) * g.Cout, cudaMemcpyDeviceToDevice,
                                   ctx->stream));
        double *ssq = channel_pass<1>(ctx, VarOp{zl, sum_keep, rows, 1.0 / m}, g.Cout, rows, scratch,
                                      true, "bn_var");
        bn_stats_store_kernel<<<(g.Cout + 127) / 128, 128, 0, ctx->stream>>>(
            sum_keep, ssq, 1.0 / m, g.Cout, mean, var, var + g.Cout, var + 2 * g.Cout);
        check_launch(ctx, "bn_stats_store_kernel");
    }
    NormActOp op{zl, mean, var, bn, zl + g.actOff, rows, g.act, g.bn};
    channel_pass<0>(ctx, op, g.Cout, rows, scratch, false, "bn_norm_act");
    if (g.poolType != FITRE_NO_POOL) {
        const long planes = (long)g.Cout * N;
        pool_forward_kernel<<<grid_for(planes * g.Hp * g.Wp), kThreads, 0, ctx->stream>>>(
            zl + g.actOff, zl + g.poolOff, planes, pool_geom(g));
        check_launch(ctx, "pool_forward_kernel");
    }
}

void conv_post_rop_forward(fitre_context *ctx, const ConvGeom &g, int N, const double *zl,
                           double *rzl, double *scratch) {
    const long rows = (long)N * g.Ho * g.Wo;
    const double m = (double)rows * ctx->world;
    const double *bn = g.bn ? zl + g.bnOff : nullptr;
    const double *mean = g.bn ? bn + g.meanOff : nullptr;
    const double *var = g.bn ? bn + g.varOff : nullptr;
    double *sums = nullptr;
    if (g.bn)
        sums = channel_pass<3>(ctx, RbnSumsOp{zl, rzl, mean, rows}, g.Cout, rows, scratch, true,
                               "rbn_sums");
    double *sums_keep = nullptr;
    if (g.bn) {
        sums_keep = scratch + kScratchDoubles - 3 * g.Cout;
        FITRE_CUDA(cudaMemcpyAsync(sums_keep, sums, sizeof(double) * 3 * g.Cout,
                                   cudaMemcpyDeviceToDevice, ctx->stream));
    }
    RNormActOp op{zl, rzl, mean, var, sums_keep, g.bn ? bn : zl, zl + g.actOff,
                  g.bn ? rzl + g.bnOff : nullptr, rzl + g.actOff, rows, m, g.act, g.bn};
    channel_pass<0>(ctx, op, g.Cout, rows, scratch, false, "rbn_norm_act");
    const long planes = (long)g.Cout * N;
    if (g.poolType == FITRE_MAX_POOL) {
        rop_max_pool_kernel<<<grid_for(planes * g.Hp * g.Wp), kThreads, 0, ctx->stream>>>(
            rzl + g.actOff, zl + g.actOff, rzl + g.poolOff, planes, pool_geom(g));
        check_launch(ctx, "rop_max_pool_kernel");
    } else if (g.poolType == FITRE_AVG_POOL) {
        pool_forward_kernel<<<grid_for(planes * g.Hp * g.Wp), kThreads, 0, ctx->stream>>>(
            rzl + g.actOff, rzl + g.poolOff, planes, pool_geom(g));
        check_launch(ctx, "pool_forward_kernel");
    }
}

const double *conv_post_backward(fitre_context *ctx, const ConvGeom &g, int N, const double *zl,
                                 double *dxl, const double *delta_pool, double *db,
                                 double *scratch) {
    const long rows = (long)N * g.Ho * g.Wo;
    const double m = (double)rows * ctx->world;
    const double *zin = g.bn ? zl + g.bnOff : zl;
    const PoolGeom pg = pool_geom(g);
    if (g.bn) {
        PoolActBwdOp<2> op{delta_pool, zl + g.actOff, zin, dxl, dxl + g.actOff, rows, pg, g.act};
        double *sums = channel_pass<2>(ctx, op, g.Cout, rows, scratch, true, "pool_act_bwd");
        double *keep = scratch + kScratchDoubles - 2 * g.Cout;
        FITRE_CUDA(cudaMemcpyAsync(keep, sums, sizeof(double) * 2 * g.Cout, cudaMemcpyDeviceToDevice,
                                   ctx->stream));
        const double *var = zl + g.bnOff + g.varOff;
        if (db) {
            BnBwdApplyOp<1> ap{dxl + g.actOff, zin, var, keep, dxl + g.bnOff, rows, m};
            double *s = channel_pass<1>(ctx, ap, g.Cout, rows, scratch, false, "bn_bwd_apply");
            FITRE_CUDA(cudaMemcpyAsync(db, s, sizeof(double) * g.Cout, cudaMemcpyDeviceToDevice,
                                       ctx->stream));
        } else {
            BnBwdApplyOp<0> ap{dxl + g.actOff, zin, var, keep, dxl + g.bnOff, rows, m};
            channel_pass<0>(ctx, ap, g.Cout, rows, scratch, false, "bn_bwd_apply");
        }
        return dxl + g.bnOff;
    }
    if (db) {
        PoolActBwdOp<1> op{delta_pool, zl + g.actOff, zin, dxl, dxl + g.actOff, rows, pg, g.act};
        double *s = channel_pass<1>(ctx, op, g.Cout, rows, scratch, false, "pool_act_bwd");
        FITRE_CUDA(cudaMemcpyAsync(db, s, sizeof(double) * g.Cout, cudaMemcpyDeviceToDevice,
                                   ctx->stream));
    } else {
        PoolActBwdOp<0> op{delta_pool, zl + g.actOff, zin, dxl, dxl + g.actOff, rows, pg, g.act};
        channel_pass<0>(ctx, op, g.Cout, rows, scratch, false, "pool_act_bwd");
    }
    return dxl + g.actOff;
}

void conv_post_rop_backward(fitre_context *ctx, const ConvGeom &g, int N, const double *zl,
                            const double *rzl, const double *dxl, const double *rdelta_pool,
                            double *rout, double *rdb, double *scratch) {
    const long rows = (long)N * g.Ho * g.Wo;
    const double m = (double)rows * ctx->world;
    const PoolGeom pg = pool_geom(g);
    const double *zin = g.bn ? zl + g.bnOff : zl;
    const double *rzin = g.bn ? rzl + g.bnOff : rzl;
    const double *mean = g.bn ? zl + g.bnOff + g.meanOff : nullptr;
    if (g.bn) {
        RPoolActBwdOp<7> op{rdelta_pool, zl + g.actOff, zin, rzin, dxl, dxl + g.actOff, zl, rzl,
                            mean, rout, rows, pg, g.act};
        double *sums = channel_pass<7>(ctx, op, g.Cout, rows, scratch, true, "rop_pool_act_bwd");
        double *keep = scratch + kScratchDoubles - 7 * g.Cout;
        FITRE_CUDA(cudaMemcpyAsync(keep, sums, sizeof(double) * 7 * g.Cout, cudaMemcpyDeviceToDevice,
                                   ctx->stream));
        const double *var = zl + g.bnOff + g.varOff;
        if (rdb) {
            RBnBwdApplyOp<1> ap{dxl + g.actOff, zin, rzin, var, keep, rout, rows, m};
            double *s = channel_pass<1>(ctx, ap, g.Cout, rows, scratch, false, "rbn_bwd_apply");
            FITRE_CUDA(cudaMemcpyAsync(rdb, s, sizeof(double) * g.Cout, cudaMemcpyDeviceToDevice,
                                       ctx->stream));
        } else {
            RBnBwdApplyOp<0> ap{dxl + g.actOff, zin, rzin, var, keep, rout, rows, m};
            channel_pass<0>(ctx, ap, g.Cout, rows, scratch, false, "rbn_bwd_apply");
        }
        return;
    }
    if (rdb) {
        RPoolActBwdOp<1> op{rdelta_pool, zl + g.actOff, zin, rzin, dxl, dxl + g.actOff, zl, rzl,
                            mean, rout, rows, pg, g.act};
        double *s = channel_pass<1>(ctx, op, g.Cout, rows, scratch, false, "rop_pool_act_bwd");
        FITRE_CUDA(cudaMemcpyAsync(rdb, s, sizeof(double) * g.Cout, cudaMemcpyDeviceToDevice,
                                   ctx->stream));
    } else {
        RPoolActBwdOp<0> op{rdelta_pool, zl + g.actOff, zin, rzin, dxl, dxl + g.actOff, zl, rzl,
                            mean, rout, rows, pg, g.act};
        channel_pass<0>(ctx, op, g.Cout, rows, scratch, false, "rop_pool_act_bwd");
    }
}

void conv_to_fc(fitre_context *ctx, double *buf, int C, int N, int Hp, int Wp, double *tmp) {
    const long total = (long)C * N * Hp * Wp;
    conv_to_fc_kernel<<<grid_for(total), kThreads, 0, ctx->stream>>>(buf, tmp, C, N, Hp, Wp);
    check_launch(ctx, "conv_to_fc_kernel");
    FITRE_CUDA(cudaMemcpyAsync(buf, tmp, sizeof(double) * total, cudaMemcpyDeviceToDevice, ctx->stream));
}
void fc_to_conv(fitre_context *ctx, double *buf, int C, int N, int Hp, int Wp, double *tmp) {
    const long total = (long)C * N * Hp * Wp;
    fc_to_conv_kernel<<<grid_for(total), kThreads, 0, ctx->stream>>>(buf, tmp, C, N, Hp, Wp);
    check_launch(ctx, "fc_to_conv_kernel");
    FITRE_CUDA(cudaMemcpyAsync(buf, tmp, sizeof(double) * total, cudaMemcpyDeviceToDevice, ctx->stream));
}

void row_sums(fitre_context *ctx, const double *x, int rows, int cols, double *out) {
    row_sums_kernel<<<rows, 128, 0, ctx->stream>>>(x, rows, cols, out);
    check_launch(ctx, "row_sums_kernel");
}

void softmax_loss(fitre_context *ctx, const double *logits, const double *labels, int N,
                  int classes, double *probs, double *errors, double inv_n_global) {
    softmax_loss_kernel<<<1, kThreads, 0, ctx->stream>>>(logits, labels, N, classes, probs, errors,
                                                         inv_n_global, ctx->ref_softmax, ctx->dscal);
    check_launch(ctx, "softmax_loss_kernel");
}
void softmax_rop_error(fitre_context *ctx, const double *rz, const double *probs, int N,
                       int classes, double *rerr, double inv_n_global) {
    softmax_rop_error_kernel<<<(N + 127) / 128, 128, 0, ctx->stream>>>(rz, probs, N, classes, rerr,
                                                                       inv_n_global);
    check_launch(ctx, "softmax_rop_error_kernel");
}

void vec_axpby(fitre_context *ctx, long n, double a, const double *x, double b, double *y) {
    axpby_kernel<<<grid_for(n), kThreads, 0, ctx->stream>>>(n, a, x, b, y);
    check_launch(ctx, "axpby_kernel");
}
void vec_axpy(fitre_context *ctx, long n, double a, const double *x, double *y) {
    if (a == 0.0) return;
    vec_axpby(ctx, n, a, x, 1.0, y);
}
void vec_scale(fitre_context *ctx, long n, double a, double *x) { vec_axpby(ctx, n, a, x, 0.0, x); }
void vec_copy(fitre_context *ctx, long n, const double *x, double *y) {
    FITRE_CUDA(cudaMemcpyAsync(y, x, sizeof(double) * n, cudaMemcpyDeviceToDevice, ctx->stream));
}
void vec_fill(fitre_context *ctx, long n, double v, double *x) {
    fill_kernel<<<grid_for(n), kThreads, 0, ctx->stream>>>(n, v, x);
    check_launch(ctx, "fill_kernel");
}
void vec_dots(fitre_context *ctx, long n, const double *a0, const double *b0, const double *a1,
              const double *b1, const double *a2, const double *b2, double *host_out) {
    double *partials = ctx->dscal + 16;
    dots_partial_kernel<<<kDotBlocks, kThreads, 0, ctx->stream>>>(n, a0, b0, a1, b1, a2, b2, partials);
    check_launch(ctx, "dots_partial_kernel");
    dots_final_kernel<<<1, 32, 0, ctx->stream>>>(partials, kDotBlocks, ctx->dscal + 8);
    check_launch(ctx, "dots_final_kernel");
    FITRE_CUDA(cudaMemcpyAsync(ctx->pinned + 8, ctx->dscal + 8, 3 * sizeof(double),
                               cudaMemcpyDeviceToHost, ctx->stream));
    FITRE_CUDA(cudaStreamSynchronize(ctx->stream));
    for (int i = 0; i < 3; ++i) host_out[i] = ctx->pinned[8 + i];
}

}  // namespace fitre
