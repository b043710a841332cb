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
        case FITRE_ACT_LOGISTIC: return 1. / (1. + exp(-x));
        case FITRE_ACT_TANH: return tanh(x);
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
        // logistic and tanh from the output, as functions/dev_layer_error.cu:13-29
        case FITRE_ACT_LOGISTIC: return zout * (1.0 - zout);
        case FITRE_ACT_TANH: return (1.0 + zout) * (1.0 - zout);
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
        case FITRE_ACT_LOGISTIC: return zout * (1.0 - zout) * (1.0 - 2.0 * zout);
        case FITRE_ACT_TANH: return -2.0 * zout * (1.0 + zout) * (1.0 - zout);
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

// V consecutive doubles moved with one instruction (V = 2: 16-byte accesses)
template <int V>
struct Pk {
    double v[V];
};
template <int V>
__device__ __forceinline__ Pk<V> ldp(const double *p) {
    Pk<V> r;
    if (V == 2) {
        const double2 t = *reinterpret_cast<const double2 *>(p);
        r.v[0] = t.x;
        r.v[V - 1] = t.y;
    } else {
        r.v[0] = *p;
    }
    return r;
}
template <int V>
__device__ __forceinline__ void stp(double *p, const Pk<V> &a) {
    if (V == 2)
        *reinterpret_cast<double2 *>(p) = make_double2(a.v[0], a.v[V - 1]);
    else
        *p = a.v[0];
}

// Block (c, s) walks slice s of channel c.  Op::chan(c) hoists everything that depends only
// on the channel (base pointers, 1/sigma, the finished sums); Op::run<V> handles V
// consecutive rows.  Row indices are 32-bit (one channel of one shard is far below 2^31
// elements), which keeps the index arithmetic off the 64-bit divider.
template <int NS, int V, class Op>
__global__ void __launch_bounds__(kThreads) channel_pass_kernel(Op op, unsigned rows, int S,
                                                                double *partials) {
    const int c = blockIdx.x, s = blockIdx.y;
    unsigned per = (rows + S - 1) / S;
    per = (per + V - 1) / V * V;
    const unsigned beg = min(rows, (unsigned)s * per);
    const unsigned end = min(rows, beg + per);
    const typename Op::Chan ch = op.chan(c);
    double acc[NS > 0 ? NS : 1];
#pragma unroll
    for (int k = 0; k < (NS > 0 ? NS : 1); ++k) acc[k] = 0.0;
    for (unsigned r = beg + V * threadIdx.x; r < end; r += V * kThreads) op.template run<V>(ch, r, acc);
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
    // scratch holds C*S*NS partials + C*NS sums + a parked copy of C*NS sums, NS <= 7
    while (S > 1 && (long)C * (S + 2) * 7 > kScratchDoubles) --S;
    return (int)S;
}

// Runs op over a [C][rows] tensor; if NS > 0 leaves the per-channel sums (C x NS, row-major by
// channel) at `sums` (= scratch) and, when `sync`, all-reduces them over the ranks.
template <int NS, class Op>
double *channel_pass(fitre_context *ctx, const Op &op, int C, long rows, double *scratch,
                     bool sync, const char *name, bool vec2) {
    FITRE_REQUIRE((long)C * 3 * 7 <= kScratchDoubles, FITRE_ERR_TOO_LARGE, "too many channels");
    FITRE_REQUIRE(rows < (1L << 31), FITRE_ERR_TOO_LARGE, "channel block beyond 2^31 elements");
    const int S = slices_for(C, rows);
    double *sums = scratch;
    double *partials = scratch + (long)C * (NS > 0 ? NS : 1);
    dim3 grid(C, S);
    if (vec2 && (rows & 1) == 0)
        channel_pass_kernel<NS, 2, Op><<<grid, kThreads, 0, ctx->stream>>>(op, (unsigned)rows, S, partials);
    else
        channel_pass_kernel<NS, 1, Op><<<grid, kThreads, 0, ctx->stream>>>(op, (unsigned)rows, S, partials);
    check_launch(ctx, name);
    if (NS > 0) {
        const int n = C * NS;
        if (sync && peer_allreduce_ready(ctx, n)) {
            // slice sums and the exchange with the other ranks in one launch over peer memory
            peer_allreduce(ctx, partials, S, NS, sums, n);
        } else {
            finalize_partials_kernel<<<(n + 127) / 128, 128, 0, ctx->stream>>>(partials, C, S, NS, sums);
            check_launch(ctx, "finalize_partials_kernel");
            if (sync) comm_allreduce_sum(ctx, sums, n);
        }
    }
    return sums;
}

// ---- functors ------------------------------------------------------------------------------
struct SumOp {  // sum x
    const double *x;
    long rows;
    struct Chan { const double *x; };
    __device__ Chan chan(int c) const { return Chan{x + (long)c * rows}; }
    template <int V>
    __device__ void run(const Chan &ch, unsigned r, double (&a)[1]) const {
        const Pk<V> p = ldp<V>(ch.x + r);
#pragma unroll
        for (int e = 0; e < V; ++e) a[0] += p.v[e];
    }
};
struct VarOp {  // sum (x - mean)^2, mean = sums[c] * inv_m
    const double *x, *sum;
    long rows;
    double inv_m;
    struct Chan { const double *x; double mean; };
    __device__ Chan chan(int c) const { return Chan{x + (long)c * rows, sum[c] * inv_m}; }
    template <int V>
    __device__ void run(const Chan &ch, unsigned r, double (&a)[1]) const {
        const Pk<V> p = ldp<V>(ch.x + r);
#pragma unroll
        for (int e = 0; e < V; ++e) {
            const double d = p.v[e] - ch.mean;
            a[0] += d * d;
        }
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
    run_mean[c] = 0.9 * run_mean[c] + (1. - 0.9) * mu;
    run_var[c] = 0.9 * run_var[c] + (1. - 0.9) * v;
}
struct NormActOp {  // bn out (optional) and activation out
    const double *x, *mean, *var;
    double *bn, *actout;
    long rows;
    int act, has_bn;
    struct Chan { const double *x; double *bn, *actout; double mean, sd; };
    __device__ Chan chan(int c) const {
        const long b = (long)c * rows;
        return Chan{x + b, has_bn ? bn + b : nullptr, actout + b, has_bn ? mean[c] : 0.0,
                    has_bn ? 1.0 / sqrt(var[c] + kBnEps) : 1.0};
    }
    template <int V>
    __device__ void run(const Chan &ch, unsigned r, double (&)[1]) const {
        Pk<V> p = ldp<V>(ch.x + r), o;
#pragma unroll
        for (int e = 0; e < V; ++e) {
            if (has_bn) p.v[e] = (p.v[e] - ch.mean) * ch.sd;  // sd holds 1/sigma
            o.v[e] = act_fwd(act, p.v[e]);
        }
        if (has_bn) stp<V>(ch.bn + r, p);
        stp<V>(ch.actout + r, o);
    }
};

struct PoolGeom {
    int type, pk, ps, pp, H, W, Hp, Wp;  // H,W: pool input (= conv output) plane
    // optional: for every pooling window the position of its arg-max inside the window
    // (column * pk + row, 255 = empty window), laid out like the pooled tensor; filled by
    // pool_argmax_map_kernel so that the gather below compares one byte per covering window
    // instead of re-scanning the window's pk * pk activations
    const unsigned char *map;
    // optional, instead of `map`, for pools with at most two windows over an element in either
    // direction (ceil(pk / ps) <= 2): one byte per ELEMENT of the pool input, bit 2*dl + dk set
    // when the window (kmin(h) + dk, lmin(w) + dl) has its arg-max at this element; filled by
    // pool_winner_mask_kernel.  Three elements in four are zero and skip the gather altogether.
    const unsigned char *emask;
};
// first window that covers coordinate x: ceil((x + pp - pk + 1) / ps), 0 when the numerator is <= 0
__device__ __forceinline__ int first_window(int x, const PoolGeom &g) {
    const int t = x + g.pp - g.pk + 1;
    if (t <= 0) return 0;
    return g.ps == 2 ? (t + 1) >> 1 : (t + g.ps - 1) / g.ps;
}

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
__device__ __forceinline__ double pool_gather_masked(const double *dpool_plane, const PoolGeom &g, int h,
                                                     int w, unsigned mask) {
    if (!mask) return 0.0;
    const int kmin = first_window(h, g), lmin = first_window(w, g);
    double s = 0.0;  // same order as the scan below: l outer, k inner
    if (mask & 1u) s += dpool_plane[lmin * g.Hp + kmin];
    if (mask & 2u) s += dpool_plane[lmin * g.Hp + kmin + 1];
    if (mask & 4u) s += dpool_plane[(lmin + 1) * g.Hp + kmin];
    if (mask & 8u) s += dpool_plane[(lmin + 1) * g.Hp + kmin + 1];
    return s;
}

__device__ __forceinline__ double pool_gather(const double *dpool_plane, const double *act_plane,
                                              const PoolGeom &g, int h, int w,
                                              const unsigned char *map_plane = nullptr) {
    if (g.type == FITRE_NO_POOL) return dpool_plane[w * g.H + h];
    if (g.type == FITRE_AVG_POOL) {
        const int k = h / g.pk, l = w / g.pk;
        return (k < g.Hp && l < g.Wp) ? dpool_plane[l * g.Hp + k] / (double)(g.pk * g.pk) : 0.0;
    }
    // windows k with k*ps - pp <= h < k*ps - pp + pk: kmin = ceil((h + pp - pk + 1) / ps) (0 when the
    // numerator is not positive), kmax = floor((h + pp) / ps); stride 2, the usual case, by shifts
    const int th = h + g.pp - g.pk + 1, tw = w + g.pp - g.pk + 1;
    int kmin, kmax, lmin, lmax;
    if (g.ps == 2) {
        kmin = th <= 0 ? 0 : (th + 1) >> 1;
        lmin = tw <= 0 ? 0 : (tw + 1) >> 1;
        kmax = (h + g.pp) >> 1;
        lmax = (w + g.pp) >> 1;
    } else {
        kmin = th <= 0 ? 0 : (th + g.ps - 1) / g.ps;
        lmin = tw <= 0 ? 0 : (tw + g.ps - 1) / g.ps;
        kmax = (h + g.pp) / g.ps;
        lmax = (w + g.pp) / g.ps;
    }
    kmax = min(kmax, g.Hp - 1);
    lmax = min(lmax, g.Wp - 1);
    const int me = w * g.H + h;
    double s = 0.0;
    if (map_plane) {
        for (int l = lmin; l <= lmax; ++l)
            for (int k = kmin; k <= kmax; ++k) {
                const int code = (w - (l * g.ps - g.pp)) * g.pk + (h - (k * g.ps - g.pp));
                if (map_plane[l * g.Hp + k] == code) s += dpool_plane[l * g.Hp + k];
            }
        return s;
    }
    for (int l = lmin; l <= lmax; ++l)
        for (int k = kmin; k <= kmax; ++k)
            if (window_argmax(act_plane, g, k, l) == me) s += dpool_plane[l * g.Hp + k];
    return s;
}

// Pooled errors for V consecutive rows (h, h+1, same column w) of one plane.  `a` holds the
// activations of those rows.  The 2x2/stride-2 max pool with V == 2 (both rows in one window)
// is resolved from the two window columns directly; everything else takes the general gather.
template <int V>
__device__ __forceinline__ Pk<V> pool_gather_v(const double *dpool_plane, const double *act_plane,
                                               const PoolGeom &g, int h, int w, const Pk<V> &a,
                                               const unsigned char *map_plane = nullptr,
                                               const unsigned char *elem_mask = nullptr) {
    Pk<V> out;
    if (elem_mask) {  // elem_mask points at the byte of element (h, w); V == 2 reads both rows at once
        unsigned m;
        if (V == 2) m = *reinterpret_cast<const unsigned short *>(elem_mask);
        else m = elem_mask[0];
#pragma unroll
        for (int e = 0; e < V; ++e) out.v[e] = pool_gather_masked(dpool_plane, g, h + e, w, (m >> (8 * e)) & 0xffu);
        return out;
    }
    if (V == 2 && g.type == FITRE_MAX_POOL && g.pk == 2 && g.ps == 2 && g.pp == 0 &&
        !(g.H & 1) && !(g.W & 1)) {
        const Pk<V> b = ldp<V>(act_plane + (w ^ 1) * g.H + h);  // the window's other column
        const bool first = !(w & 1);                             // is our column scanned first?
        const double c0 = first ? a.v[0] : b.v[0], c1 = first ? a.v[V - 1] : b.v[V - 1];
        const double c2 = first ? b.v[0] : a.v[0], c3 = first ? b.v[V - 1] : a.v[V - 1];
        int win = 0;
        double best = c0;
        if (c1 > best) { best = c1; win = 1; }
        if (c2 > best) { best = c2; win = 2; }
        if (c3 > best) { best = c3; win = 3; }
        const double d = dpool_plane[(w >> 1) * g.Hp + (h >> 1)];
        const int mine = first ? 0 : 2;
        out.v[0] = (win == mine) ? d : 0.0;
        out.v[V - 1] = (win == mine + 1) ? d : 0.0;
        return out;
    }
    if (g.type == FITRE_NO_POOL) return ldp<V>(dpool_plane + w * g.H + h);
#pragma unroll
    for (int e = 0; e < V; ++e) out.v[e] = pool_gather(dpool_plane, act_plane, g, h + e, w, map_plane);
    return out;
}

struct PlaneChan {   // per-channel bases shared by the pool/activation functors
    long cbase;      // c * rows
    long pbase;      // start of channel c in the pooled tensor
    unsigned hw, H, pw;
    int sh_hw, sh_H;  // log2 of hw / H when they are powers of two (the usual planes), else -1
};
// (image, column, row) of element r of a channel block; shifts when the plane sizes allow
__device__ __forceinline__ void plane_coords(const PlaneChan &p, unsigned r, unsigned &n, unsigned &w,
                                             unsigned &h) {
    n = p.sh_hw >= 0 ? r >> p.sh_hw : r / p.hw;
    const unsigned rem = r - n * p.hw;
    w = p.sh_H >= 0 ? rem >> p.sh_H : rem / p.H;
    h = rem - w * p.H;
}
__device__ __forceinline__ PlaneChan plane_chan(int c, long rows, const PoolGeom &g) {
    PlaneChan p;
    p.hw = (unsigned)(g.H * g.W);
    p.H = (unsigned)g.H;
    p.sh_hw = (p.hw & (p.hw - 1)) == 0 ? 31 - __clz(p.hw) : -1;
    p.sh_H = (p.H & (p.H - 1)) == 0 ? 31 - __clz(p.H) : -1;
    p.pw = (unsigned)(g.Hp * g.Wp);
    p.cbase = (long)c * rows;
    p.pbase = g.type == FITRE_NO_POOL ? p.cbase : (long)c * (rows / p.hw) * p.pw;
    return p;
}

template <int NS>
struct PoolActBwdOp {  // dxP, dxA (+ sums: dA [, dA*zhat])
    const double *dpool, *actv, *zin;
    double *dxP, *dxA;
    long rows;
    PoolGeom g;
    int act;
    typedef PlaneChan Chan;
    __device__ Chan chan(int c) const { return plane_chan(c, rows, g); }
    template <int V>
    __device__ void run(const Chan &ch, unsigned r, double (&a)[NS > 0 ? NS : 1]) const {
        unsigned n, w, h;
        plane_coords(ch, r, n, w, h);
        const long i = ch.cbase + r;
        const double *aplane = actv + ch.cbase + (long)n * ch.hw;
        const double *pplane = dpool + ch.pbase + (long)n * (g.type == FITRE_NO_POOL ? ch.hw : ch.pw);
        const Pk<V> av = ldp<V>(actv + i), zi = ldp<V>(zin + i);
        const unsigned char *mplane = g.map ? g.map + ch.pbase + (long)n * ch.pw : nullptr;
        const Pk<V> dP = pool_gather_v<V>(pplane, aplane, g, (int)h, (int)w, av, mplane,
                                          g.emask ? g.emask + i : nullptr);
        Pk<V> dA;
#pragma unroll
        for (int e = 0; e < V; ++e) {
            dA.v[e] = dP.v[e] * act_d1(act, zi.v[e], av.v[e]);
            if (NS >= 1) a[0] += dA.v[e];
            if (NS >= 2) a[1] += dA.v[e] * zi.v[e];
        }
        stp<V>(dxP + i, dP);
        stp<V>(dxA + i, dA);
    }
};

template <int NS>
struct BnBwdApplyOp {  // dBN = (m dA - s1 - zhat s2) / (m sigma)   (+ sum dBN)
    const double *dA, *zhat, *var, *sums;  // sums: [C][2] = (sum dA, sum dA*zhat)
    double *out;
    long rows;
    double m;
    struct Chan { long b; double s1, s2, den; };
    __device__ Chan chan(int c) const {
        return Chan{(long)c * rows, sums[2 * c], sums[2 * c + 1], 1.0 / (m * sqrt(kBnEps + var[c]))};
    }
    template <int V>
    __device__ void run(const Chan &ch, unsigned r, double (&a)[NS > 0 ? NS : 1]) const {
        const long i = ch.b + r;
        const Pk<V> d = ldp<V>(dA + i), zh = ldp<V>(zhat + i);
        Pk<V> o;
#pragma unroll
        for (int e = 0; e < V; ++e) {
            o.v[e] = (d.v[e] * m - ch.s1 - ch.s2 * zh.v[e]) * ch.den;  // den holds 1/(m sigma)
            if (NS >= 1) a[0] += o.v[e];
        }
        stp<V>(out + i, o);
    }
};

struct RbnSumsOp {  // sum Rz, sum (z-mu) Rz, sum (z-mu)
    const double *z, *rz, *mean;
    long rows;
    struct Chan { long b; double mean; };
    __device__ Chan chan(int c) const { return Chan{(long)c * rows, mean[c]}; }
    template <int V>
    __device__ void run(const Chan &ch, unsigned r, double (&a)[3]) const {
        const long i = ch.b + r;
        const Pk<V> zz = ldp<V>(z + i), t = ldp<V>(rz + i);
#pragma unroll
        for (int e = 0; e < V; ++e) {
            const double d = zz.v[e] - ch.mean;
            a[0] += t.v[e];
            a[1] += d * t.v[e];
            a[2] += d;
        }
    }
};
struct RNormActOp {  // R bn-out, R act-out
    const double *z, *rz, *mean, *var, *sums, *zin, *actv;
    double *rbn, *ract;
    long rows;
    double m;
    int act, has_bn;
    struct Chan { long b; double mean, rmean, sd, coef; };
    __device__ Chan chan(int c) const {
        Chan ch{(long)c * rows, 0.0, 0.0, 1.0, 0.0};
        if (has_bn) {
            ch.mean = mean[c];
            ch.rmean = sums[3 * c] / m;
            // sum (z-mu)(Rz - mean Rz) = sum (z-mu) Rz - mean Rz * sum (z-mu)
            const double s = sums[3 * c + 1] - ch.rmean * sums[3 * c + 2];
            const double ve = var[c] + kBnEps;
            const double sd = sqrt(ve);
            ch.sd = 1.0 / sd;  // 1/sigma
            ch.coef = s / (m * ve * sd);
        }
        return ch;
    }
    template <int V>
    __device__ void run(const Chan &ch, unsigned r, double (&)[1]) const {
        const long i = ch.b + r;
        Pk<V> v = ldp<V>(rz + i), o;
        const Pk<V> zi = ldp<V>(zin + i), av = ldp<V>(actv + i);
        if (has_bn) {
            const Pk<V> zz = ldp<V>(z + i);
#pragma unroll
            for (int e = 0; e < V; ++e)
                v.v[e] = (v.v[e] - ch.rmean) * ch.sd - ch.coef * (zz.v[e] - ch.mean);
            stp<V>(rbn + i, v);
        }
#pragma unroll
        for (int e = 0; e < V; ++e) o.v[e] = v.v[e] * act_d1(act, zi.v[e], av.v[e]);
        stp<V>(ract + i, o);
    }
};

template <int NS>
struct RPoolActBwdOp {  // RdA = h' RdP + h'' Rzin dxP   (+ sums, see conv_post_rop_backward)
    const double *rdpool, *actv, *zin, *rzin, *dxP, *dxA, *zconv, *rzconv, *mean;
    double *rout;
    long rows;
    PoolGeom g;
    int act;
    struct Chan { PlaneChan p; double mean; };
    __device__ Chan chan(int c) const { return Chan{plane_chan(c, rows, g), NS == 7 ? mean[c] : 0.0}; }
    template <int V>
    __device__ void run(const Chan &ch, unsigned r, double (&a)[NS > 0 ? NS : 1]) const {
        const PlaneChan &pc = ch.p;
        unsigned n, w, h;
        plane_coords(pc, r, n, w, h);
        const long i = pc.cbase + r;
        const double *aplane = actv + pc.cbase + (long)n * pc.hw;
        const double *pplane = rdpool + pc.pbase + (long)n * (g.type == FITRE_NO_POOL ? pc.hw : pc.pw);
        const Pk<V> av = ldp<V>(actv + i), zi = ldp<V>(zin + i), rzh = ldp<V>(rzin + i);
        const Pk<V> dp = ldp<V>(dxP + i);
        const unsigned char *mplane = g.map ? g.map + pc.pbase + (long)n * pc.pw : nullptr;
        const Pk<V> RdP = pool_gather_v<V>(pplane, aplane, g, (int)h, (int)w, av, mplane,
                                           g.emask ? g.emask + i : nullptr);
        Pk<V> RdA;
#pragma unroll
        for (int e = 0; e < V; ++e)
            RdA.v[e] = act_d1(act, zi.v[e], av.v[e]) * RdP.v[e] +
                       act_d2(act, zi.v[e], av.v[e]) * rzh.v[e] * dp.v[e];
        stp<V>(rout + i, RdA);
        if (NS == 1) {
#pragma unroll
            for (int e = 0; e < V; ++e) a[0] += RdA.v[e];
        }
        if (NS == 7) {
            const Pk<V> dA = ldp<V>(dxA + i), zc = ldp<V>(zconv + i), rzc = ldp<V>(rzconv + i);
#pragma unroll
            for (int e = 0; e < V; ++e) {
                const double d = zc.v[e] - ch.mean;
                a[0] += RdA.v[e];
                a[1] += dA.v[e] * zi.v[e];
                a[2] += dA.v[e] * rzh.v[e] + zi.v[e] * RdA.v[e];
                a[3] += dA.v[e];
                a[4] += rzc.v[e];
                a[5] += d * rzc.v[e];
                a[6] += d;
            }
        }
    }
};

template <int NS>
struct RBnBwdApplyOp {
    const double *dA, *zhat, *rzhat, *var, *sums;  // sums [C][7]
    double *rout;
    long rows;
    double m;
    struct Chan { long b; double s0, s1, s2, s3, den, rI; };
    __device__ Chan chan(int c) const {
        const double *s = sums + 7 * c;
        const double ve = var[c] + kBnEps, sd = sqrt(ve);
        const double rmean = s[4] / m;
        return Chan{(long)c * rows, s[0], s[1], s[2], s[3], 1.0 / (m * sd),
                    -(s[5] - rmean * s[6]) / (m * m * ve * sd)};
    }
    template <int V>
    __device__ void run(const Chan &ch, unsigned r, double (&a)[NS > 0 ? NS : 1]) const {
        const long i = ch.b + r;
        const Pk<V> rd = ldp<V>(rout + i), d = ldp<V>(dA + i), zh = ldp<V>(zhat + i),
                    rzh = ldp<V>(rzhat + i);
        Pk<V> o;
#pragma unroll
        for (int e = 0; e < V; ++e) {
            const double rII = (rd.v[e] * m - ch.s0 - ch.s1 * rzh.v[e] - ch.s2 * zh.v[e]) * ch.den;
            const double II = d.v[e] * m - ch.s3 - ch.s1 * zh.v[e];
            o.v[e] = rII + II * ch.rI;
            if (NS >= 1) a[0] += o.v[e];
        }
        stp<V>(rout + i, o);
    }
};

// ---- stand-alone kernels ---------------------------------------------------------------------
// One thread per pooling window: where inside the window its arg-max lies (see PoolGeom::map).
__global__ void pool_argmax_map_kernel(const double *act, unsigned char *map, long planes, PoolGeom g) {
    const long total = planes * g.Hp * g.Wp;
    for (long t = blockIdx.x * (long)blockDim.x + threadIdx.x; t < total; t += (long)gridDim.x * blockDim.x) {
        const long plane = t / (g.Hp * g.Wp);
        const int rem = (int)(t - plane * (g.Hp * g.Wp));
        const int l = rem / g.Hp, k = rem - l * g.Hp;
        const int arg = window_argmax(act + plane * (long)(g.H * g.W), g, k, l);
        int code = 255;
        if (arg >= 0) {
            const int w = arg / g.H, h = arg - w * g.H;
            code = (w - (l * g.ps - g.pp)) * g.pk + (h - (k * g.ps - g.pp));
        }
        map[t] = (unsigned char)code;
    }
}

// One thread per pooling window: sets, in the byte of the element that is the window's arg-max,
// the bit that names this window among the (at most 2 x 2) windows over that element (see
// PoolGeom::emask).  OR is order-independent, so the map is the same whatever the schedule.
__global__ void pool_winner_mask_kernel(const double *act, unsigned char *emask, long planes, PoolGeom g) {
    const long total = planes * g.Hp * g.Wp;
    for (long t = blockIdx.x * (long)blockDim.x + threadIdx.x; t < total; t += (long)gridDim.x * blockDim.x) {
        const long plane = t / (g.Hp * g.Wp);
        const int rem = (int)(t - plane * (g.Hp * g.Wp));
        const int l = rem / g.Hp, k = rem - l * g.Hp;
        const int arg = window_argmax(act + plane * (long)(g.H * g.W), g, k, l);
        if (arg < 0) continue;
        const int w = arg / g.H, h = arg - w * g.H;
        const int bit = 2 * (l - first_window(w, g)) + (k - first_window(h, g));
        const long idx = plane * (long)(g.H * g.W) + arg;
        atomicOr(reinterpret_cast<unsigned *>(emask + (idx & ~3L)), 1u << (8 * (int)(idx & 3) + bit));
    }
}

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

// inverse-CDF label sampling + (p - onehot(label)) / N  (functions/dev_dist_errors.cu:12-29,
// functions/softmax_loss.cu:104-136,215-245)
__global__ void distribution_errors_kernel(const double *probs, const double *uniforms, int N,
                                           int classes, double *target, double *errors,
                                           double inv_ng) {
    const int r = blockIdx.x * blockDim.x + threadIdx.x;
    if (r >= N) return;
    double c = 0.0;
    int label = -1;
    for (int i = 0; i < classes; ++i) {
        c += probs[(long)r * classes + i];
        if (c >= uniforms[r]) {
            label = i + 1;
            break;
        }
    }
    if (label == -1) label = classes + 1;
    target[r] = (double)label;
    for (int i = 0; i < classes; ++i)
        errors[(long)r * classes + i] = (probs[(long)r * classes + i] - (i + 1 == label ? 1.0 : 0.0)) * inv_ng;
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
// One warp per dot product: lane l adds the partials of blocks l, l + 32, ... in ascending order,
// then the 32 lane sums are folded by a fixed shuffle tree.
__global__ void dots_final_kernel(const double *partials, int blocks, double *out) {
    const int which = threadIdx.x >> 5, lane = threadIdx.x & 31;
    double s = 0.0;
    for (int b = lane; b < blocks; b += 32) s += partials[3 * b + which];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    if (lane == 0) out[which] = s;
}

int grid_for(long n) { return (int)std::max<long>(1, std::min<long>((n + kThreads - 1) / kThreads, 148 * 8)); }

// 16-byte accesses need every tensor of the pass on a 16-byte boundary and an even plane height
// (so that a pair of rows never straddles a column or a plane).
bool vec2_ok(const ConvGeom &g, int N, std::initializer_list<const void *> ptrs) {
    if ((g.Ho & 1) || (((long)N * g.Ho * g.Wo) & 1)) return false;
    if ((g.actOff | (g.bn ? g.bnOff : 0)) & 1) return false;
    for (const void *p : ptrs)
        if (p && ((uintptr_t)p & 15)) return false;
    return true;
}

PoolGeom pool_geom(const ConvGeom &g) {
    PoolGeom p;
    p.map = nullptr;
    p.emask = nullptr;
    p.type = g.poolType;
    p.pk = g.pk; p.ps = g.ps; p.pp = g.pp;
    p.H = g.Ho; p.W = g.Wo;
    p.Hp = g.Hp; p.Wp = g.Wp;
    return p;
}

}  // namespace

long bn_scratch(int) { return kScratchDoubles; }

namespace {
bool pool_wants_map(const ConvGeom &g) {
    if (g.poolType != FITRE_MAX_POOL || g.pk > 15) return false;
    const bool fast = g.pk == 2 && g.ps == 2 && g.pp == 0 && !(g.Ho & 1) && !(g.Wo & 1);
    return !fast;  // the 2/2/0 pool resolves its window from two loads
}
// at most two windows over an element in either direction: the per-element winner mask serves
bool pool_mask_per_element(const ConvGeom &g) { return pool_wants_map(g) && (g.pk + g.ps - 1) / g.ps <= 2; }
// fills the arg-max map of this layer's pooling windows and hands it to the gather
void prepare_pool_map(fitre_context *ctx, const ConvGeom &g, int N, const double *act, unsigned char *map,
                      PoolGeom &pg) {
    if (!map || !pool_wants_map(g)) return;
    const long planes = (long)g.Cout * N;
    if (pool_mask_per_element(g)) {
        FITRE_CUDA(cudaMemsetAsync(map, 0, (size_t)pool_map_doubles(g, N) * sizeof(double), ctx->stream));
        pool_winner_mask_kernel<<<grid_for(planes * g.Hp * g.Wp), kThreads, 0, ctx->stream>>>(act, map, planes, pg);
        check_launch(ctx, "pool_winner_mask_kernel");
        pg.emask = map;
        return;
    }
    pool_argmax_map_kernel<<<grid_for(planes * g.Hp * g.Wp), kThreads, 0, ctx->stream>>>(act, map, planes, pg);
    check_launch(ctx, "pool_argmax_map_kernel");
    pg.map = map;
}
}  // namespace

// doubles of scratch the backward passes need for the arg-max map of layer g's pooling: one byte
// per element of the pool input (winner mask) or one per window (arg-max code)
long pool_map_doubles(const ConvGeom &g, int N) {
    if (!pool_wants_map(g)) return 0;
    const long bytes = pool_mask_per_element(g) ? (long)g.Cout * N * g.Ho * g.Wo : (long)g.Cout * N * g.Hp * g.Wp;
    return (bytes + 7) / 8;
}

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

void conv_post_forward(fitre_context *ctx, const ConvGeom &g, int N, double *zl, double *scratch,
                       bool running_stats) {
    const long rows = (long)N * g.Ho * g.Wo;
    const double m = (double)rows * ctx->world;
    double *bn = g.bn ? zl + g.bnOff : nullptr;
    double *mean = g.bn ? bn + g.meanOff : nullptr;
    double *var = g.bn ? bn + g.varOff : nullptr;
    const bool v2 = vec2_ok(g, N, {zl});
    if (g.bn && running_stats) {
        // accuracy evaluation: normalise with the running statistics, leave every statistic as it
        // is (functions/dev_batch_norm.cu:386-392)
        mean = var + g.Cout;
        var = var + 2 * g.Cout;
    } else if (g.bn) {
        // two-pass batch statistics (functions/dev_batch_norm.cu:263-315)
        double *sum = channel_pass<1>(ctx, SumOp{zl, rows}, g.Cout, rows, scratch, true, "bn_sum", v2);
        double *sum_keep = scratch + kScratchDoubles - g.Cout;  // parked above the partials
        FITRE_CUDA(cudaMemcpyAsync(sum_keep, sum, sizeof(double) * g.Cout, cudaMemcpyDeviceToDevice,
                                   ctx->stream));
        double *ssq = channel_pass<1>(ctx, VarOp{zl, sum_keep, rows, 1.0 / m}, g.Cout, rows, scratch,
                                      true, "bn_var", v2);
        bn_stats_store_kernel<<<(g.Cout + 127) / 128, 128, 0, ctx->stream>>>(
            sum_keep, ssq, 1.0 / m, g.Cout, mean, var, var + g.Cout, var + 2 * g.Cout);
        check_launch(ctx, "bn_stats_store_kernel");
    }
    NormActOp op{zl, mean, var, bn, zl + g.actOff, rows, g.act, g.bn};
    channel_pass<0>(ctx, op, g.Cout, rows, scratch, false, "bn_norm_act", v2);
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
    const bool v2 = vec2_ok(g, N, {zl, rzl});
    if (g.bn)
        sums = channel_pass<3>(ctx, RbnSumsOp{zl, rzl, mean, rows}, g.Cout, rows, scratch, true,
                               "rbn_sums", v2);
    double *sums_keep = nullptr;
    if (g.bn) {
        sums_keep = scratch + kScratchDoubles - 3 * g.Cout;
        FITRE_CUDA(cudaMemcpyAsync(sums_keep, sums, sizeof(double) * 3 * g.Cout,
                                   cudaMemcpyDeviceToDevice, ctx->stream));
    }
    RNormActOp op{zl, rzl, mean, var, sums_keep, g.bn ? bn : zl, zl + g.actOff,
                  g.bn ? rzl + g.bnOff : nullptr, rzl + g.actOff, rows, m, g.act, g.bn};
    channel_pass<0>(ctx, op, g.Cout, rows, scratch, false, "rbn_norm_act", v2);
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
                                 double *scratch, unsigned char *pool_map) {
    const long rows = (long)N * g.Ho * g.Wo;
    const double m = (double)rows * ctx->world;
    const double *zin = g.bn ? zl + g.bnOff : zl;
    PoolGeom pg = pool_geom(g);
    prepare_pool_map(ctx, g, N, zl + g.actOff, pool_map, pg);
    const bool v2 = vec2_ok(g, N, {zl, dxl, g.poolType == FITRE_NO_POOL ? delta_pool : nullptr});
    if (g.bn) {
        PoolActBwdOp<2> op{delta_pool, zl + g.actOff, zin, dxl, dxl + g.actOff, rows, pg, g.act};
        double *sums = channel_pass<2>(ctx, op, g.Cout, rows, scratch, true, "pool_act_bwd", v2);
        double *keep = scratch + kScratchDoubles - 2 * g.Cout;
        FITRE_CUDA(cudaMemcpyAsync(keep, sums, sizeof(double) * 2 * g.Cout, cudaMemcpyDeviceToDevice,
                                   ctx->stream));
        const double *var = zl + g.bnOff + g.varOff;
        if (db) {
            BnBwdApplyOp<1> ap{dxl + g.actOff, zin, var, keep, dxl + g.bnOff, rows, m};
            double *s = channel_pass<1>(ctx, ap, g.Cout, rows, scratch, false, "bn_bwd_apply", v2);
            FITRE_CUDA(cudaMemcpyAsync(db, s, sizeof(double) * g.Cout, cudaMemcpyDeviceToDevice,
                                       ctx->stream));
        } else {
            BnBwdApplyOp<0> ap{dxl + g.actOff, zin, var, keep, dxl + g.bnOff, rows, m};
            channel_pass<0>(ctx, ap, g.Cout, rows, scratch, false, "bn_bwd_apply", v2);
        }
        return dxl + g.bnOff;
    }
    if (db) {
        PoolActBwdOp<1> op{delta_pool, zl + g.actOff, zin, dxl, dxl + g.actOff, rows, pg, g.act};
        double *s = channel_pass<1>(ctx, op, g.Cout, rows, scratch, false, "pool_act_bwd", v2);
        FITRE_CUDA(cudaMemcpyAsync(db, s, sizeof(double) * g.Cout, cudaMemcpyDeviceToDevice,
                                   ctx->stream));
    } else {
        PoolActBwdOp<0> op{delta_pool, zl + g.actOff, zin, dxl, dxl + g.actOff, rows, pg, g.act};
        channel_pass<0>(ctx, op, g.Cout, rows, scratch, false, "pool_act_bwd", v2);
    }
    return dxl + g.actOff;
}

void conv_post_rop_backward(fitre_context *ctx, const ConvGeom &g, int N, const double *zl,
                            const double *rzl, const double *dxl, const double *rdelta_pool,
                            double *rout, double *rdb, double *scratch, unsigned char *pool_map) {
    const long rows = (long)N * g.Ho * g.Wo;
    const double m = (double)rows * ctx->world;
    PoolGeom pg = pool_geom(g);
    prepare_pool_map(ctx, g, N, zl + g.actOff, pool_map, pg);
    const double *zin = g.bn ? zl + g.bnOff : zl;
    const double *rzin = g.bn ? rzl + g.bnOff : rzl;
    const double *mean = g.bn ? zl + g.bnOff + g.meanOff : nullptr;
    const bool v2 = vec2_ok(g, N, {zl, rzl, dxl, rout, g.poolType == FITRE_NO_POOL ? rdelta_pool : nullptr});
    if (g.bn) {
        RPoolActBwdOp<7> op{rdelta_pool, zl + g.actOff, zin, rzin, dxl, dxl + g.actOff, zl, rzl,
                            mean, rout, rows, pg, g.act};
        double *sums = channel_pass<7>(ctx, op, g.Cout, rows, scratch, true, "rop_pool_act_bwd", v2);
        double *keep = scratch + kScratchDoubles - 7 * g.Cout;
        FITRE_CUDA(cudaMemcpyAsync(keep, sums, sizeof(double) * 7 * g.Cout, cudaMemcpyDeviceToDevice,
                                   ctx->stream));
        const double *var = zl + g.bnOff + g.varOff;
        if (rdb) {
            RBnBwdApplyOp<1> ap{dxl + g.actOff, zin, rzin, var, keep, rout, rows, m};
            double *s = channel_pass<1>(ctx, ap, g.Cout, rows, scratch, false, "rbn_bwd_apply", v2);
            FITRE_CUDA(cudaMemcpyAsync(rdb, s, sizeof(double) * g.Cout, cudaMemcpyDeviceToDevice,
                                       ctx->stream));
        } else {
            RBnBwdApplyOp<0> ap{dxl + g.actOff, zin, rzin, var, keep, rout, rows, m};
            channel_pass<0>(ctx, ap, g.Cout, rows, scratch, false, "rbn_bwd_apply", v2);
        }
        return;
    }
    if (rdb) {
        RPoolActBwdOp<1> op{rdelta_pool, zl + g.actOff, zin, rzin, dxl, dxl + g.actOff, zl, rzl,
                            mean, rout, rows, pg, g.act};
        double *s = channel_pass<1>(ctx, op, g.Cout, rows, scratch, false, "rop_pool_act_bwd", v2);
        FITRE_CUDA(cudaMemcpyAsync(rdb, s, sizeof(double) * g.Cout, cudaMemcpyDeviceToDevice,
                                   ctx->stream));
    } else {
        RPoolActBwdOp<0> op{rdelta_pool, zl + g.actOff, zin, rzin, dxl, dxl + g.actOff, zl, rzl,
                            mean, rout, rows, pg, g.act};
        channel_pass<0>(ctx, op, g.Cout, rows, scratch, false, "rop_pool_act_bwd", v2);
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

void distribution_errors(fitre_context *ctx, const double *probs, const double *uniforms, int N,
                         int classes, double *target, double *errors, double inv_n_global) {
    distribution_errors_kernel<<<(N + 127) / 128, 128, 0, ctx->stream>>>(probs, uniforms, N, classes,
                                                                         target, errors, inv_n_global);
    check_launch(ctx, "distribution_errors_kernel");
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
    dots_final_kernel<<<1, 96, 0, ctx->stream>>>(partials, kDotBlocks, ctx->dscal + 8);
    check_launch(ctx, "dots_final_kernel");
    FITRE_CUDA(cudaMemcpyAsync(ctx->pinned + 8, ctx->dscal + 8, 3 * sizeof(double),
                               cudaMemcpyDeviceToHost, ctx->stream));
    stream_wait(ctx, ctx->stream);
    for (int i = 0; i < 3; ++i) host_out[i] = ctx->pinned[8 + i];
}

}  // namespace fitre
