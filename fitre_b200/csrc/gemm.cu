// fp64 tensor-core (DMMA) GEMM-shaped kernels for sm_100a:
//   * implicit-GEMM convolution forward / data gradient, with up to two K-concatenated
//     (input, weight) segments so that an R-op product X*V + RX*W is one launch;
//   * implicit-GEMM weight gradient with up to two M-concatenated segments and a
//     deterministic split over the N*Ho*Wo reduction;
//   * a dense column-major DGEMM for the fully connected layers;
//   * A'A (SYRK-shaped) for the KFAC G factors.
// The im2col matrix of the reference (functions/dev_image.cu:12-51) is never materialised:
// tiles are gathered straight from the [C][N][W][H] tensor with the same index map
// (row r = n*Ho*Wo + wo*Ho + ho, column q = cin*k*k + j*k + i, zero outside the image).
// tcgen05 has no fp64 kind, so the fp64 path uses mma.sync m8n8k4 (DMMA).
#include <algorithm>
#include <mutex>

#include "common.h"

namespace fitre {
namespace {

__device__ __forceinline__ void dmma884(double &c0, double &c1, double a, double b) {
    asm volatile("mma.sync.aligned.m8n8k4.row.col.f64.f64.f64.f64 {%0,%1}, {%2}, {%3}, {%0,%1};\n"
                 : "+d"(c0), "+d"(c1)
                 : "d"(a), "d"(b));
}

// ----------------------------------------------------------------------------------------
// Implicit-GEMM convolution:  Y[M x Cout] = sum_seg im2col(X_seg)[M x K] * W_seg[K x Cout]
// ----------------------------------------------------------------------------------------
struct ConvArgs {
    const double *x[2];
    const double *w[2];
    int nseg;
    const double *bias;
    double *y;
    int N, Cin, H, W, k, pad, Cout, Ho, Wo, K;
    long M;
};

constexpr int FP_BM = 128, FP_BN = 64, FP_BK = 16, FP_THREADS = 256;
constexpr int FP_LDA = FP_BM + 4;  // As[k][m]: (lane%4)*LDA + lane/4 hits 16 distinct 8-byte banks
constexpr int FP_LDB = FP_BK + 4;  // Bs[n][k]
constexpr int FP_SMEM = 2 * (FP_BK * FP_LDA + FP_BN * FP_LDB) * (int)sizeof(double);

// KS = compile-time kernel size (0 = runtime); NT = 8-column MMA tiles per warp: 4 gives the
// 128 x 64 block tile, 1 a 128 x 16 tile for layers with at most 16 output channels (LeNet, the
// data gradient into a 3- or 6-channel input), which would otherwise spend 3/4 or more of their
// tensor work on columns that do not exist.
template <int KS, int NT>
__global__ void __launch_bounds__(FP_THREADS, NT == 1 ? 3 : 2) conv_fprop_kernel(ConvArgs p) {
    constexpr int BN = 16 * NT;
    extern __shared__ double smem[];
    double *As = smem;                           // [2][BK][LDA]
    double *Bs = smem + 2 * FP_BK * FP_LDA;      // [2][BN][LDB]

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int warp_m = warp & 3, warp_n = warp >> 2;
    const long m0 = (long)blockIdx.x * FP_BM;
    const int c0 = blockIdx.y * BN;
    const int k = KS ? KS : p.k, kk2 = k * k;

    // this thread gathers rows mm of the A tile for k-slots a_k0, a_k0 + 2, ...
    const int a_mm = tid & (FP_BM - 1), a_k0 = tid >> 7;
    const long am = m0 + a_mm;
    const bool a_mvalid = am < p.M;
    int a_ho = 0, a_wo = 0;
    long a_base = 0;
    if (a_mvalid) {
        const int howo = p.Ho * p.Wo;
        const int n = (int)(am / howo);
        const int r = (int)(am - (long)n * howo);
        a_wo = r / p.Ho;
        a_ho = r - a_wo * p.Ho;
        a_base = ((long)n * p.W + (a_wo - p.pad)) * p.H + (a_ho - p.pad);
    }
    const long chan_stride = (long)p.N * p.W * p.H;
    // B tile: thread loads 4 consecutive k of column b_nn
    const int b_nn = tid >> 2, b_k0 = (tid & 3) * 4;
    const bool b_loader = b_nn < BN;
    const bool b_cvalid = b_loader && (c0 + b_nn) < p.Cout;

    const int nk = (p.K + FP_BK - 1) / FP_BK;
    const int iters = nk * p.nseg;

    double ra[8], rb[4];
    auto gload = [&](int it) {
        const int seg = it / nk, kt = it - seg * nk;
        const double *x = p.x[seg];
        const double *w = p.w[seg];
#pragma unroll
        for (int r = 0; r < 8; ++r) {
            const int q = kt * FP_BK + a_k0 + 2 * r;
            double v = 0.0;
            if (a_mvalid && q < p.K) {
                const int cin = q / kk2;
                const int rem = q - cin * kk2;
                const int j = rem / k, i = rem - j * k;
                const int h = a_ho - p.pad + i, wv = a_wo - p.pad + j;
                if (h >= 0 && h < p.H && wv >= 0 && wv < p.W)
                    v = __ldg(x + a_base + cin * chan_stride + (long)j * p.H + i);
            }
            ra[r] = v;
        }
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int q = kt * FP_BK + b_k0 + e;
            rb[e] = (b_cvalid && q < p.K) ? __ldg(w + (long)(c0 + b_nn) * p.K + q) : 0.0;
        }
    };
    auto sstore = [&](int buf) {
        double *a = As + buf * FP_BK * FP_LDA;
        double *b = Bs + buf * BN * FP_LDB;
#pragma unroll
        for (int r = 0; r < 8; ++r) a[(a_k0 + 2 * r) * FP_LDA + a_mm] = ra[r];
        if (b_loader) {
#pragma unroll
            for (int e = 0; e < 4; ++e) b[b_nn * FP_LDB + b_k0 + e] = rb[e];
        }
    };

    double acc[4][NT][2];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < NT; ++j) acc[i][j][0] = acc[i][j][1] = 0.0;

    gload(0);
    sstore(0);
    __syncthreads();
    const int lr = lane >> 2, lc = lane & 3;
    for (int it = 0; it < iters; ++it) {
        const int buf = it & 1;
        if (it + 1 < iters) gload(it + 1);
        const double *a = As + buf * FP_BK * FP_LDA + warp_m * 32 + lr;
        const double *b = Bs + buf * BN * FP_LDB + (warp_n * 8 * NT + lr) * FP_LDB;
#pragma unroll
        for (int k4 = 0; k4 < FP_BK / 4; ++k4) {
            double fa[4], fb[NT];
#pragma unroll
            for (int mi = 0; mi < 4; ++mi) fa[mi] = a[(k4 * 4 + lc) * FP_LDA + mi * 8];
#pragma unroll
            for (int ni = 0; ni < NT; ++ni) fb[ni] = b[ni * 8 * FP_LDB + k4 * 4 + lc];
#pragma unroll
            for (int mi = 0; mi < 4; ++mi)
#pragma unroll
                for (int ni = 0; ni < NT; ++ni) dmma884(acc[mi][ni][0], acc[mi][ni][1], fa[mi], fb[ni]);
        }
        if (it + 1 < iters) {
            sstore(buf ^ 1);
            __syncthreads();
        }
    }

#pragma unroll
    for (int ni = 0; ni < NT; ++ni)
#pragma unroll
        for (int e = 0; e < 2; ++e) {
            const int col = c0 + warp_n * 8 * NT + ni * 8 + 2 * lc + e;
            if (col >= p.Cout) continue;
            const double bv = p.bias ? p.bias[col] : 0.0;
#pragma unroll
            for (int mi = 0; mi < 4; ++mi) {
                const long row = m0 + warp_m * 32 + mi * 8 + lr;
                if (row < p.M) p.y[(long)col * p.M + row] = acc[mi][ni][e] + bv;
            }
        }
}

// Weights for the data gradient: Wd[(cout*k*k + j'*k + i') + cin*(Cout*k*k)] =
// W[cout][cin][k-1-j'][k-1-i'] (functions/dev_backprop_convolution.cu:86-95,140-156,215-217).
__global__ void dgrad_weight_perm_kernel(const double *w, double *wd, int Cin, int Cout, int k) {
    const long n = (long)Cin * Cout * k * k;
    const int kk2 = k * k;
    for (long idx = blockIdx.x * (long)blockDim.x + threadIdx.x; idx < n;
         idx += (long)gridDim.x * blockDim.x) {
        const int cin = (int)(idx / ((long)Cout * kk2));
        const long r = idx - (long)cin * Cout * kk2;
        const int cout = (int)(r / kk2);
        const int t = (int)(r - (long)cout * kk2);
        const int jp = t / k, ip = t - jp * k;
        wd[idx] = w[(long)cout * Cin * kk2 + (long)cin * kk2 + (k - 1 - jp) * k + (k - 1 - ip)];
    }
}

// ----------------------------------------------------------------------------------------
// Implicit-GEMM weight gradient: dW[K x Cout] = sum_seg im2col(X_seg)' [K x M] * D_seg[M x Cout]
// ----------------------------------------------------------------------------------------
struct WgradArgs {
    const double *x[2];
    const double *d[2];
    int nseg;
    double *out;      // dW when splits == 1, else partial slabs [split][K*Cout]
    int N, Cin, H, W, k, pad, Cout, Ho, Wo, K;
    long M;
    long chunk;       // rows of M per split (multiple of WG_BK)
};

constexpr int WG_BQ = 64, WG_BN = 64, WG_BK = 16, WG_THREADS = 256;
constexpr int WG_LD = WG_BK + 4;  // Sa[q][m], Sb[c][m]: (lane/4)*LD + lane%4 is conflict-free
constexpr int WG_SMEM = 2 * (WG_BQ + WG_BN) * WG_LD * (int)sizeof(double);

// NARROW (layers with at most 16 output channels): the block tile is 64 (q) x 16 (c), warps 4 x 2
// with 16 x 8 tiles, instead of 64 x 64 with warps 2 x 4 and 32 x 16 tiles; the gather is the same
// (columns past Cout are zeros that nobody multiplies any more).
template <int KS, bool NARROW>
__global__ void __launch_bounds__(WG_THREADS, 2) conv_wgrad_kernel(WgradArgs p) {
    constexpr int MI = NARROW ? 2 : 4, NI = NARROW ? 1 : 2;
    extern __shared__ double smem[];
    double *Sa = smem;                          // [2][BQ][LD]
    double *Sb = smem + 2 * WG_BQ * WG_LD;      // [2][BN][LD]
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int warp_q = NARROW ? (warp & 3) : (warp & 1), warp_n = NARROW ? (warp >> 2) : (warp >> 1);
    const int q0 = blockIdx.x * WG_BQ, c0 = blockIdx.y * (NARROW ? 16 : WG_BN);
    const long mbeg = (long)blockIdx.z * p.chunk;
    const long mend = min(p.M, mbeg + p.chunk);
    const int k = KS ? KS : p.k, kk2 = k * k;
    const long chan_stride = (long)p.N * p.W * p.H;
    const int howo = p.Ho * p.Wo;

    // gather roles: element (qq = t_q + 16 r, mm = t_m)
    const int t_m = tid & 15, t_q = tid >> 4;
    long q_off[4];
    int q_i[4], q_j[4];
    bool q_ok[4];
#pragma unroll
    for (int r = 0; r < 4; ++r) {
        const int q = q0 + t_q + 16 * r;
        q_ok[r] = q < p.K;
        const int cin = q_ok[r] ? q / kk2 : 0;
        const int rem = q_ok[r] ? q - cin * kk2 : 0;
        q_j[r] = rem / k;
        q_i[r] = rem - q_j[r] * k;
        q_off[r] = cin * chan_stride + (long)q_j[r] * p.H + q_i[r];
    }
    bool c_ok[4];
#pragma unroll
    for (int r = 0; r < 4; ++r) c_ok[r] = (c0 + t_q + 16 * r) < p.Cout;

    const long span = mend > mbeg ? mend - mbeg : 0;
    const int nk = (int)((span + WG_BK - 1) / WG_BK);
    const int iters = nk * p.nseg;

    double ra[4], rb[4];
    auto gload = [&](int it) {
        const int seg = it / nk, kt = it - seg * nk;
        const double *x = p.x[seg];
        const double *d = p.d[seg];
        const long m = mbeg + (long)kt * WG_BK + t_m;
        const bool mv = m < mend;
        int ho = 0, wo = 0;
        long base = 0;
        if (mv) {
            const int n = (int)(m / howo);
            const int r = (int)(m - (long)n * howo);
            wo = r / p.Ho;
            ho = r - wo * p.Ho;
            base = ((long)n * p.W + (wo - p.pad)) * p.H + (ho - p.pad);
        }
#pragma unroll
        for (int r = 0; r < 4; ++r) {
            double v = 0.0;
            if (mv && q_ok[r]) {
                const int h = ho - p.pad + q_i[r], wv = wo - p.pad + q_j[r];
                if (h >= 0 && h < p.H && wv >= 0 && wv < p.W) v = __ldg(x + base + q_off[r]);
            }
            ra[r] = v;
            rb[r] = (mv && c_ok[r]) ? __ldg(d + (long)(c0 + t_q + 16 * r) * p.M + m) : 0.0;
        }
    };
    auto sstore = [&](int buf) {
        double *a = Sa + buf * WG_BQ * WG_LD;
        double *b = Sb + buf * WG_BN * WG_LD;
#pragma unroll
        for (int r = 0; r < 4; ++r) {
            a[(t_q + 16 * r) * WG_LD + t_m] = ra[r];
            b[(t_q + 16 * r) * WG_LD + t_m] = rb[r];
        }
    };

    double acc[MI][NI][2];
#pragma unroll
    for (int i = 0; i < MI; ++i)
#pragma unroll
        for (int j = 0; j < NI; ++j) acc[i][j][0] = acc[i][j][1] = 0.0;

    const int lr = lane >> 2, lc = lane & 3;
    if (iters > 0) {
        gload(0);
        sstore(0);
    }
    __syncthreads();
    for (int it = 0; it < iters; ++it) {
        const int buf = it & 1;
        if (it + 1 < iters) gload(it + 1);
        const double *a = Sa + buf * WG_BQ * WG_LD + (warp_q * 8 * MI + lr) * WG_LD + lc;
        const double *b = Sb + buf * WG_BN * WG_LD + (warp_n * 8 * NI + lr) * WG_LD + lc;
#pragma unroll
        for (int k4 = 0; k4 < WG_BK / 4; ++k4) {
            double fa[MI], fb[NI];
#pragma unroll
            for (int mi = 0; mi < MI; ++mi) fa[mi] = a[mi * 8 * WG_LD + k4 * 4];
#pragma unroll
            for (int ni = 0; ni < NI; ++ni) fb[ni] = b[ni * 8 * WG_LD + k4 * 4];
#pragma unroll
            for (int mi = 0; mi < MI; ++mi)
#pragma unroll
                for (int ni = 0; ni < NI; ++ni) dmma884(acc[mi][ni][0], acc[mi][ni][1], fa[mi], fb[ni]);
        }
        if (it + 1 < iters) {
            sstore(buf ^ 1);
            __syncthreads();
        }
    }
    double *out = p.out + (long)blockIdx.z * p.K * p.Cout;
#pragma unroll
    for (int ni = 0; ni < NI; ++ni)
#pragma unroll
        for (int e = 0; e < 2; ++e) {
            const int col = c0 + warp_n * 8 * NI + ni * 8 + 2 * lc + e;
            if (col >= p.Cout) continue;
#pragma unroll
            for (int mi = 0; mi < MI; ++mi) {
                const int row = q0 + warp_q * 8 * MI + mi * 8 + lr;
                if (row < p.K) out[(long)col * p.K + row] = acc[mi][ni][e];
            }
        }
}

// out[i] = alpha * sum_s partial[s][i], s ascending (deterministic)
__global__ void reduce_slabs_kernel(const double *partial, double *out, long n, int slabs,
                                    double alpha) {
    for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < n;
         i += (long)gridDim.x * blockDim.x) {
        double s = 0.0;
        for (int k = 0; k < slabs; ++k) s += partial[(long)k * n + i];
        out[i] = alpha * s;
    }
}

// The same sum for many slabs of a small output (LeNet's first layer: 296 slabs of 450 values):
// eight warps share the slabs of 32 outputs, each adds its contiguous range in ascending order,
// and the eight part sums are added in ascending order -- a fixed order, like the kernel above.
__global__ void reduce_slabs_tall_kernel(const double *partial, double *out, long n, int slabs,
                                         double alpha) {
    __shared__ double part[8][33];
    const int li = threadIdx.x & 31, g = threadIdx.x >> 5;
    const long i = blockIdx.x * 32L + li;
    const int per = (slabs + 7) / 8;
    const int k0 = g * per, k1 = min(slabs, k0 + per);
    double s = 0.0;
    if (i < n)
        for (int k = k0; k < k1; ++k) s += partial[(long)k * n + i];
    part[g][li] = s;
    __syncthreads();
    if (g == 0 && i < n) {
        double t = 0.0;
#pragma unroll
        for (int j = 0; j < 8; ++j) t += part[j][li];
        out[i] = alpha * t;
    }
}

// ----------------------------------------------------------------------------------------
// Dense DGEMM (fully connected layers): C = alpha op(A) op(B) + beta C, column-major
// ----------------------------------------------------------------------------------------
constexpr int DG_BM = 64, DG_BN = 64, DG_BK = 16, DG_THREADS = 256;
// Structure hints for products with a triangular operand (the factor inversion): which k blocks of
// a C tile can be non-zero, or that only tiles touching the lower triangle of C are wanted.
//   GEMM_K_LE_COL: terms with k <= column only  (B' lower triangular:  C = A * L')
//   GEMM_K_GE_COL: terms with k >= column only  (B lower triangular:   C = A * L)
//   GEMM_K_LE_ROW: terms with k <= row only     (A lower triangular:   C = L * B)
//   GEMM_LOWER_C:  tiles strictly above the diagonal of C are skipped (C symmetric, lower wanted)
// The skipped terms are exact zeros, so results equal the plain product.
__device__ __forceinline__ bool gemm_k_range(int kmode, int m0, int n0, int bm, int bn, int k, int &kt0, int &nk,
                                             int bk = DG_BK) {
    kt0 = 0;
    nk = (k + bk - 1) / bk;
    if (kmode == GEMM_K_LE_COL) nk = min(nk, (min(n0 + bn, k) + bk - 1) / bk);
    else if (kmode == GEMM_K_GE_COL) kt0 = n0 / bk;
    else if (kmode == GEMM_K_LE_ROW) nk = min(nk, (min(m0 + bm, k) + bk - 1) / bk);
    else if (kmode == GEMM_LOWER_C && n0 >= m0 + bm) return false;
    return true;
}
constexpr int DG_LDA = DG_BM + 4, DG_LDB = DG_BN + 4;  // As[k][m], Bs[k][n]
constexpr int DG_SMEM = 2 * 16 * (DG_LDA + DG_LDB) * (int)sizeof(double);
constexpr int DG_SMEM_DEEP = 2 * 64 * (DG_LDA + DG_LDB) * (int)sizeof(double);

// BK = depth of one k step.  16 for grids that fill the GPU (several resident blocks per SM hide
// the operand fetch); 64 for grids of at most one block per SM with a long k loop (FC layers at
// small batch, the couplings of the factorisation recursion), where a block is alone on its SM
// and every step costs one round trip to L2 or HBM: four times fewer, four times longer steps,
// each fetch hidden behind a full step of tensor work.  Terms are added in the same order
// (groups of four k, ascending), so both depths return the same bits.
template <bool TA, bool TB, int BK>
__global__ void __launch_bounds__(DG_THREADS) dgemm_kernel(int m, int n, int k, double alpha,
                                                          const double *A, int lda,
                                                          const double *B, int ldb, double beta,
                                                          double *C, int ldc, int kmode) {
    extern __shared__ double dg_smem[];
    double *As = dg_smem;                        // [2][BK * DG_LDA], As[k][m]
    double *Bs = dg_smem + 2 * BK * DG_LDA;      // [2][BK * DG_LDB], Bs[k][n]
    constexpr int PER = BK / 4;                  // elements of each operand tile per thread
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int warp_m = warp & 1, warp_n = warp >> 1;  // warp tile 32 x 16
    const int m0 = blockIdx.x * DG_BM, n0 = blockIdx.y * DG_BN;
    int kt0, nk;
    if (!gemm_k_range(kmode, m0, n0, DG_BM, DG_BN, k, kt0, nk, BK)) return;
    // loader roles: 64 * BK elements per operand tile, BK / 4 per thread.  The fast thread index
    // follows the contiguous direction of the operand in memory.
    double ra[PER], rb[PER];
    auto role = [&](bool along_k, int r, int &fast64, int &kk) {
        if (!along_k) { fast64 = tid & 63; kk = (tid >> 6) + 4 * r; }
        else          { kk = tid % BK; fast64 = tid / BK + (DG_THREADS / BK) * r; }
    };
    auto gload = [&](int kt) {
#pragma unroll
        for (int r = 0; r < PER; ++r) {
            int mm, kk;
            role(TA, r, mm, kk);
            const int gi = m0 + mm, gp = kt * BK + kk;
            double v = 0.0;
            if (gi < m && gp < k) v = TA ? A[gp + (long)gi * lda] : A[gi + (long)gp * lda];
            ra[r] = v;
            int nn, kb;
            role(!TB, r, nn, kb);
            const int gj = n0 + nn, gq = kt * BK + kb;
            double u = 0.0;
            if (gj < n && gq < k) u = TB ? B[gj + (long)gq * ldb] : B[gq + (long)gj * ldb];
            rb[r] = u;
        }
    };
    auto sstore = [&](int buf) {
#pragma unroll
        for (int r = 0; r < PER; ++r) {
            int mm, kk;
            role(TA, r, mm, kk);
            As[buf * BK * DG_LDA + kk * DG_LDA + mm] = ra[r];
            int nn, kb;
            role(!TB, r, nn, kb);
            Bs[buf * BK * DG_LDB + kb * DG_LDB + nn] = rb[r];
        }
    };
    double acc[4][2][2];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 2; ++j) acc[i][j][0] = acc[i][j][1] = 0.0;
    const int lr = lane >> 2, lc = lane & 3;
    if (nk > kt0) {
        gload(kt0);
        sstore(kt0 & 1);
    }
    __syncthreads();
    for (int kt = kt0; kt < nk; ++kt) {
        const int buf = kt & 1;
        if (kt + 1 < nk) gload(kt + 1);
        const double *a = As + buf * BK * DG_LDA + warp_m * 32 + lr;
        const double *b = Bs + buf * BK * DG_LDB + warp_n * 16 + lr;
#pragma unroll
        for (int k4 = 0; k4 < BK / 4; ++k4) {
            double fa[4], fb[2];
#pragma unroll
            for (int mi = 0; mi < 4; ++mi) fa[mi] = a[(k4 * 4 + lc) * DG_LDA + mi * 8];
#pragma unroll
            for (int ni = 0; ni < 2; ++ni) fb[ni] = b[(k4 * 4 + lc) * DG_LDB + ni * 8];
#pragma unroll
            for (int mi = 0; mi < 4; ++mi)
#pragma unroll
                for (int ni = 0; ni < 2; ++ni) dmma884(acc[mi][ni][0], acc[mi][ni][1], fa[mi], fb[ni]);
        }
        if (kt + 1 < nk) {
            sstore(buf ^ 1);
            __syncthreads();
        }
    }
#pragma unroll
    for (int ni = 0; ni < 2; ++ni)
#pragma unroll
        for (int e = 0; e < 2; ++e) {
            const int col = n0 + warp_n * 16 + ni * 8 + 2 * lc + e;
            if (col >= n) continue;
#pragma unroll
            for (int mi = 0; mi < 4; ++mi) {
                const int row = m0 + warp_m * 32 + mi * 8 + lr;
                if (row >= m) continue;
                double *c = C + (long)col * ldc + row;
                const double v = alpha * acc[mi][ni][e];
                *c = (beta == 0.0) ? v : v + beta * (*c);
            }
        }
}

// ----------------------------------------------------------------------------------------
// The same product on 128 x 128 tiles for large shapes (the GEMMs of the factor inversion and
// the natural gradient): 8 warps as 2 x 4, each 64 x 32, so 12 shared-memory fragment loads feed
// 32 DMMAs per 4-deep k step (the 64 x 64 kernel above: 6 loads for 8).  Double-buffered
// register-staged loads as above; shared memory is dynamic (two 16 x 132 tiles per operand).
// ----------------------------------------------------------------------------------------
constexpr int DL_BM = 128, DL_BN = 128, DL_LD = 128 + 4;
constexpr int DL_SMEM = 2 * 2 * DG_BK * DL_LD * (int)sizeof(double);

template <bool TA, bool TB>
__global__ void __launch_bounds__(DG_THREADS) dgemm_large_kernel(int m, int n, int k, double alpha,
                                                                const double *A, int lda,
                                                                const double *B, int ldb, double beta,
                                                                double *C, int ldc, int kmode) {
    extern __shared__ double dl_smem[];
    double *As = dl_smem;                          // [2][DG_BK * DL_LD], As[k][m]
    double *Bs = dl_smem + 2 * DG_BK * DL_LD;      // [2][DG_BK * DL_LD], Bs[k][n]
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int warp_m = warp & 1, warp_n = warp >> 1;  // warp tile 64 x 32
    const int m0 = blockIdx.x * DL_BM, n0 = blockIdx.y * DL_BN;
    int kt0, nk;
    if (!gemm_k_range(kmode, m0, n0, DL_BM, DL_BN, k, kt0, nk)) return;
    double ra[8], rb[8];
    auto gload = [&](int kt) {
#pragma unroll
        for (int r = 0; r < 8; ++r) {
            int mm, kk;
            if (!TA) { mm = tid & 127; kk = (tid >> 7) + 2 * r; }
            else     { kk = tid & 15; mm = (tid >> 4) + 16 * r; }
            const int gi = m0 + mm, gp = kt * DG_BK + kk;
            ra[r] = (gi < m && gp < k) ? (TA ? A[gp + (long)gi * lda] : A[gi + (long)gp * lda]) : 0.0;
            int nn, kb;
            if (!TB) { kb = tid & 15; nn = (tid >> 4) + 16 * r; }
            else     { nn = tid & 127; kb = (tid >> 7) + 2 * r; }
            const int gj = n0 + nn, gq = kt * DG_BK + kb;
            rb[r] = (gj < n && gq < k) ? (TB ? B[gj + (long)gq * ldb] : B[gq + (long)gj * ldb]) : 0.0;
        }
    };
    auto sstore = [&](int buf) {
#pragma unroll
        for (int r = 0; r < 8; ++r) {
            int mm, kk;
            if (!TA) { mm = tid & 127; kk = (tid >> 7) + 2 * r; }
            else     { kk = tid & 15; mm = (tid >> 4) + 16 * r; }
            As[buf * DG_BK * DL_LD + kk * DL_LD + mm] = ra[r];
            int nn, kb;
            if (!TB) { kb = tid & 15; nn = (tid >> 4) + 16 * r; }
            else     { nn = tid & 127; kb = (tid >> 7) + 2 * r; }
            Bs[buf * DG_BK * DL_LD + kb * DL_LD + nn] = rb[r];
        }
    };
    double acc[8][4][2];
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j][0] = acc[i][j][1] = 0.0;
    const int lr = lane >> 2, lc = lane & 3;
    if (nk > kt0) {
        gload(kt0);
        sstore(kt0 & 1);
    }
    __syncthreads();
    for (int kt = kt0; kt < nk; ++kt) {
        const int buf = kt & 1;
        if (kt + 1 < nk) gload(kt + 1);
        const double *a = As + buf * DG_BK * DL_LD + warp_m * 64 + lr;
        const double *b = Bs + buf * DG_BK * DL_LD + warp_n * 32 + lr;
#pragma unroll
        for (int k4 = 0; k4 < DG_BK / 4; ++k4) {
            double fa[8], fb[4];
#pragma unroll
            for (int mi = 0; mi < 8; ++mi) fa[mi] = a[(k4 * 4 + lc) * DL_LD + mi * 8];
#pragma unroll
            for (int ni = 0; ni < 4; ++ni) fb[ni] = b[(k4 * 4 + lc) * DL_LD + ni * 8];
#pragma unroll
            for (int mi = 0; mi < 8; ++mi)
#pragma unroll
                for (int ni = 0; ni < 4; ++ni) dmma884(acc[mi][ni][0], acc[mi][ni][1], fa[mi], fb[ni]);
        }
        if (kt + 1 < nk) {
            sstore(buf ^ 1);
            __syncthreads();
        }
    }
#pragma unroll
    for (int ni = 0; ni < 4; ++ni)
#pragma unroll
        for (int e = 0; e < 2; ++e) {
            const int col = n0 + warp_n * 32 + ni * 8 + 2 * lc + e;
            if (col >= n) continue;
#pragma unroll
            for (int mi = 0; mi < 8; ++mi) {
                const int row = m0 + warp_m * 64 + mi * 8 + lr;
                if (row >= m) continue;
                double *c = C + (long)col * ldc + row;
                const double v = alpha * acc[mi][ni][e];
                *c = (beta == 0.0) ? v : v + beta * (*c);
            }
        }
}

// ----------------------------------------------------------------------------------------
// C[n x n] = alpha * A' A with A rows x n column-major; split over rows, both triangles.
// ----------------------------------------------------------------------------------------
struct SyrkArgs {
    const double *A;
    long lda, rows, chunk;
    int n;
    double *out;
};

__global__ void __launch_bounds__(WG_THREADS, 2) syrk_tn_kernel(SyrkArgs p) {
    extern __shared__ double smem[];
    double *Sa = smem;
    double *Sb = smem + 2 * WG_BQ * WG_LD;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int warp_q = warp & 1, warp_n = warp >> 1;
    const int q0 = blockIdx.x * WG_BQ, c0 = blockIdx.y * WG_BN;
    if (c0 > q0 + WG_BQ - 1) return;  // lower-triangular tiles only; mirrored by the reducer
    const long mbeg = (long)blockIdx.z * p.chunk;
    const long mend = min(p.rows, mbeg + p.chunk);
    const int t_m = tid & 15, t_q = tid >> 4;
    const long span = mend > mbeg ? mend - mbeg : 0;
    const int nk = (int)((span + WG_BK - 1) / WG_BK);
    double ra[4], rb[4];
    auto gload = [&](int kt) {
        const long m = mbeg + (long)kt * WG_BK + t_m;
        const bool mv = m < mend;
#pragma unroll
        for (int r = 0; r < 4; ++r) {
            const int qa = q0 + t_q + 16 * r, qb = c0 + t_q + 16 * r;
            ra[r] = (mv && qa < p.n) ? __ldg(p.A + (long)qa * p.lda + m) : 0.0;
            rb[r] = (mv && qb < p.n) ? __ldg(p.A + (long)qb * p.lda + m) : 0.0;
        }
    };
    auto sstore = [&](int buf) {
        double *a = Sa + buf * WG_BQ * WG_LD;
        double *b = Sb + buf * WG_BN * WG_LD;
#pragma unroll
        for (int r = 0; r < 4; ++r) {
            a[(t_q + 16 * r) * WG_LD + t_m] = ra[r];
            b[(t_q + 16 * r) * WG_LD + t_m] = rb[r];
        }
    };
    double acc[4][2][2];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 2; ++j) acc[i][j][0] = acc[i][j][1] = 0.0;
    const int lr = lane >> 2, lc = lane & 3;
    if (nk > 0) {
        gload(0);
        sstore(0);
    }
    __syncthreads();
    for (int kt = 0; kt < nk; ++kt) {
        const int buf = kt & 1;
        if (kt + 1 < nk) gload(kt + 1);
        const double *a = Sa + buf * WG_BQ * WG_LD + (warp_q * 32 + lr) * WG_LD + lc;
        const double *b = Sb + buf * WG_BN * WG_LD + (warp_n * 16 + lr) * WG_LD + lc;
#pragma unroll
        for (int k4 = 0; k4 < WG_BK / 4; ++k4) {
            double fa[4], fb[2];
#pragma unroll
            for (int mi = 0; mi < 4; ++mi) fa[mi] = a[mi * 8 * WG_LD + k4 * 4];
#pragma unroll
            for (int ni = 0; ni < 2; ++ni) fb[ni] = b[ni * 8 * WG_LD + k4 * 4];
#pragma unroll
            for (int mi = 0; mi < 4; ++mi)
#pragma unroll
                for (int ni = 0; ni < 2; ++ni) dmma884(acc[mi][ni][0], acc[mi][ni][1], fa[mi], fb[ni]);
        }
        if (kt + 1 < nk) {
            sstore(buf ^ 1);
            __syncthreads();
        }
    }
    double *out = p.out + (long)blockIdx.z * p.n * p.n;
#pragma unroll
    for (int ni = 0; ni < 2; ++ni)
#pragma unroll
        for (int e = 0; e < 2; ++e) {
            const int col = c0 + warp_n * 16 + ni * 8 + 2 * lc + e;
            if (col >= p.n) continue;
#pragma unroll
            for (int mi = 0; mi < 4; ++mi) {
                const int row = q0 + warp_q * 32 + mi * 8 + lr;
                if (row < p.n) out[(long)col * p.n + row] = acc[mi][ni][e];
            }
        }
}

// out = alpha * sum of slabs; entries above the diagonal are taken from their mirror image
// (tiles strictly above the diagonal are not computed).
__global__ void syrk_reduce_kernel(const double *partial, double *out, int n, int slabs,
                                   double alpha) {
    const long nn = (long)n * n;
    for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < nn;
         i += (long)gridDim.x * blockDim.x) {
        int col = (int)(i / n), row = (int)(i - (long)col * n);
        // tile (row/64, col/64) is computed iff col_tile <= row_tile
        long src = (col / WG_BN <= row / WG_BQ) ? i : (long)row * n + col;
        double s = 0.0;
        for (int k = 0; k < slabs; ++k) s += partial[(long)k * nn + src];
        out[i] = alpha * s;
    }
}


// ----------------------------------------------------------------------------------------
// KFAC A factor of a convolution: A = (1/N) P~' P~ with P~ = [im2col(X) / (Ho*Wo), 1]
// (solvers/kfac_inverses.cu:515-540), as a tensor-core SYRK over implicit patches: both
// operands are gathered from X, only lower-triangular tiles are computed, the scaling and
// the mirror image are applied by the slab reducer.
// ----------------------------------------------------------------------------------------
struct PatchSyrkArgs {
    const double *x;
    double *out;
    int N, Cin, H, W, k, pad, Ho, Wo, K, Kb;  // Kb = K + (bias column ? 1 : 0)
    long M, chunk;
};

template <int KS>
__global__ void __launch_bounds__(WG_THREADS, 2) patch_syrk_kernel(PatchSyrkArgs p) {
    extern __shared__ double smem[];
    double *Sa = smem;
    double *Sb = smem + 2 * WG_BQ * WG_LD;
    const int q0 = blockIdx.x * WG_BQ, c0 = blockIdx.y * WG_BN;
    if (c0 > q0 + WG_BQ - 1) return;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int warp_q = warp & 1, warp_n = warp >> 1;
    const long mbeg = (long)blockIdx.z * p.chunk;
    const long mend = min(p.M, mbeg + p.chunk);
    const int k = KS ? KS : p.k, kk2 = k * k;
    const long chan_stride = (long)p.N * p.W * p.H;
    const int howo = p.Ho * p.Wo;
    const int t_m = tid & 15, t_q = tid >> 4;
    // per-thread column descriptors for both operands: kind 0 = outside, 1 = patch, 2 = ones
    long off[2][4];
    int qi[2][4], qj[2][4], kind[2][4];
#pragma unroll
    for (int o = 0; o < 2; ++o)
#pragma unroll
        for (int r = 0; r < 4; ++r) {
            const int q = (o == 0 ? q0 : c0) + t_q + 16 * r;
            kind[o][r] = q < p.K ? 1 : (q < p.Kb ? 2 : 0);
            const int cin = kind[o][r] == 1 ? q / kk2 : 0;
            const int rem = kind[o][r] == 1 ? q - cin * kk2 : 0;
            qj[o][r] = rem / k;
            qi[o][r] = rem - qj[o][r] * k;
            off[o][r] = cin * chan_stride + (long)qj[o][r] * p.H + qi[o][r];
        }
    const long span = mend > mbeg ? mend - mbeg : 0;
    const int nk = (int)((span + WG_BK - 1) / WG_BK);
    double rr[2][4];
    auto gload = [&](int kt) {
        const long m = mbeg + (long)kt * WG_BK + t_m;
        const bool mv = m < mend;
        int ho = 0, wo = 0;
        long base = 0;
        if (mv) {
            const int n = (int)(m / howo);
            const int r = (int)(m - (long)n * howo);
            wo = r / p.Ho;
            ho = r - wo * p.Ho;
            base = ((long)n * p.W + (wo - p.pad)) * p.H + (ho - p.pad);
        }
#pragma unroll
        for (int o = 0; o < 2; ++o)
#pragma unroll
            for (int r = 0; r < 4; ++r) {
                double v = 0.0;
                if (mv && kind[o][r] == 1) {
                    const int h = ho - p.pad + qi[o][r], wv = wo - p.pad + qj[o][r];
                    if (h >= 0 && h < p.H && wv >= 0 && wv < p.W) v = __ldg(p.x + base + off[o][r]);
                } else if (mv && kind[o][r] == 2) {
                    v = 1.0;
                }
                rr[o][r] = v;
            }
    };
    auto sstore = [&](int buf) {
        double *a = Sa + buf * WG_BQ * WG_LD;
        double *b = Sb + buf * WG_BN * WG_LD;
#pragma unroll
        for (int r = 0; r < 4; ++r) {
            a[(t_q + 16 * r) * WG_LD + t_m] = rr[0][r];
            b[(t_q + 16 * r) * WG_LD + t_m] = rr[1][r];
        }
    };
    double acc[4][2][2];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 2; ++j) acc[i][j][0] = acc[i][j][1] = 0.0;
    const int lr = lane >> 2, lc = lane & 3;
    if (nk > 0) {
        gload(0);
        sstore(0);
    }
    __syncthreads();
    for (int kt = 0; kt < nk; ++kt) {
        const int buf = kt & 1;
        if (kt + 1 < nk) gload(kt + 1);
        const double *a = Sa + buf * WG_BQ * WG_LD + (warp_q * 32 + lr) * WG_LD + lc;
        const double *b = Sb + buf * WG_BN * WG_LD + (warp_n * 16 + lr) * WG_LD + lc;
#pragma unroll
        for (int k4 = 0; k4 < WG_BK / 4; ++k4) {
            double fa[4], fb[2];
#pragma unroll
            for (int mi = 0; mi < 4; ++mi) fa[mi] = a[mi * 8 * WG_LD + k4 * 4];
#pragma unroll
            for (int ni = 0; ni < 2; ++ni) fb[ni] = b[ni * 8 * WG_LD + k4 * 4];
#pragma unroll
            for (int mi = 0; mi < 4; ++mi)
#pragma unroll
                for (int ni = 0; ni < 2; ++ni) dmma884(acc[mi][ni][0], acc[mi][ni][1], fa[mi], fb[ni]);
        }
        if (kt + 1 < nk) {
            sstore(buf ^ 1);
            __syncthreads();
        }
    }
    double *out = p.out + (long)blockIdx.z * p.Kb * p.Kb;
#pragma unroll
    for (int ni = 0; ni < 2; ++ni)
#pragma unroll
        for (int e = 0; e < 2; ++e) {
            const int col = c0 + warp_n * 16 + ni * 8 + 2 * lc + e;
            if (col >= p.Kb) continue;
#pragma unroll
            for (int mi = 0; mi < 4; ++mi) {
                const int row = q0 + warp_q * 32 + mi * 8 + lr;
                if (row < p.Kb) out[(long)col * p.Kb + row] = acc[mi][ni][e];
            }
        }
}

// A[i][j] = alpha * s_i * s_j * sum of slabs, s = patch_scale for patch columns (< K) and 1 for
// the ones column; upper triangle mirrored from the computed lower tiles.
__global__ void patch_syrk_reduce_kernel(const double *partial, double *out, int Kb, int K,
                                         int slabs, double alpha, double patch_scale) {
    const long nn = (long)Kb * Kb;
    for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < nn;
         i += (long)gridDim.x * blockDim.x) {
        const int col = (int)(i / Kb), row = (int)(i - (long)col * Kb);
        // every producer computes at least the tiles that hold the lower triangle
        const long src = (row >= col) ? i : (long)row * Kb + col;
        double s = 0.0;
        for (int k = 0; k < slabs; ++k) s += partial[(long)k * nn + src];
        const double sc = (row < K ? patch_scale : 1.0) * (col < K ? patch_scale : 1.0);
        out[i] = alpha * sc * s;
    }
}

int split_count(long tiles, long reduce_len, long min_len) {
    long want = (2L * 148 * 2 + tiles - 1) / tiles;  // about two waves of 2 CTAs per SM
    long cap = std::max(1L, reduce_len / min_len);
    return (int)std::max(1L, std::min(want, cap));
}

}  // namespace

long conv_fprop_scratch(int N, int Cin, int H, int W, int k, int pad, int Cout) {
    return std::max(conv_fprop_tma_scratch(N, Cin, H, W, k, pad, Cout),
                    conv_fprop_tf32_scratch(N, Cin, H, W, k, pad, Cout));
}
long conv_dgrad_scratch(int N, int Cin, int H, int W, int k, int pad, int Cout) {
    // the data gradient is a convolution of the errors: Cout input channels, Cin outputs
    const int Ho = H + 2 * pad - k + 1, Wo = W + 2 * pad - k + 1;
    return conv_fprop_scratch(N, Cout, Ho, Wo, k, k - 1 - pad, Cin);
}

void conv_fprop(fitre_context *ctx, int nseg, const ConvSeg *segs, const double *bias, double *y,
                int N, int Cin, int H, int W, int k, int pad, int Cout, double *split) {
    if (ctx->precision == FITRE_PRECISION_FP64_I8) {
        if (conv_fprop_i8(ctx, nseg, segs, bias, y, N, Cin, H, W, k, pad, Cout)) return;
    } else if (ctx->precision != FITRE_PRECISION_FP64 &&
               conv_fprop_tf32(ctx, nseg, segs, bias, y, N, Cin, H, W, k, pad, Cout, split)) {
        return;
    }
    if (ctx->use_tma && conv_fprop_tma(ctx, nseg, segs, bias, y, N, Cin, H, W, k, pad, Cout, split)) return;
    ConvArgs a{};
    for (int s = 0; s < nseg; ++s) {
        a.x[s] = segs[s].x;
        a.w[s] = segs[s].w;
    }
    a.nseg = nseg;
    a.bias = bias;
    a.y = y;
    a.N = N; a.Cin = Cin; a.H = H; a.W = W; a.k = k; a.pad = pad; a.Cout = Cout;
    a.Ho = H + 2 * pad - k + 1;
    a.Wo = W + 2 * pad - k + 1;
    a.K = Cin * k * k;
    a.M = (long)N * a.Ho * a.Wo;
    const bool narrow = Cout <= 16;  // 128 x 16 block tile: gather-bound, so three blocks per SM
    const int bn = narrow ? 16 : FP_BN;
    constexpr int FP_SMEM_NARROW = 2 * (FP_BK * FP_LDA + 16 * FP_LDB) * (int)sizeof(double);
    dim3 grid((unsigned)((a.M + FP_BM - 1) / FP_BM), (unsigned)((Cout + bn - 1) / bn));
    ProfScope prof(ctx, PROF_CONV_IGEMM, 2.0 * (double)a.M * a.K * Cout * nseg);
    if (k == 3) {
        if (narrow) conv_fprop_kernel<3, 1><<<grid, FP_THREADS, FP_SMEM_NARROW, ctx->stream>>>(a);
        else conv_fprop_kernel<3, 4><<<grid, FP_THREADS, FP_SMEM, ctx->stream>>>(a);
    } else if (k == 5) {
        if (narrow) conv_fprop_kernel<5, 1><<<grid, FP_THREADS, FP_SMEM_NARROW, ctx->stream>>>(a);
        else conv_fprop_kernel<5, 4><<<grid, FP_THREADS, FP_SMEM, ctx->stream>>>(a);
    } else {
        if (narrow) conv_fprop_kernel<0, 1><<<grid, FP_THREADS, FP_SMEM_NARROW, ctx->stream>>>(a);
        else conv_fprop_kernel<0, 4><<<grid, FP_THREADS, FP_SMEM, ctx->stream>>>(a);
    }
    check_launch(ctx, "conv_fprop_kernel");
}

void conv_dgrad(fitre_context *ctx, int nseg, const ConvSeg *segs, double *dx, int N, int Cin,
                int H, int W, int k, int pad, int Cout, double *wscratch, double *split) {
    const int Ho = H + 2 * pad - k + 1, Wo = W + 2 * pad - k + 1;
    const long wsz = (long)Cin * Cout * k * k;
    ConvSeg t[2];
    for (int s = 0; s < nseg; ++s) {
        double *wd = wscratch + s * wsz;
        int blocks = (int)std::min<long>((wsz + 255) / 256, 1184);
        dgrad_weight_perm_kernel<<<blocks, 256, 0, ctx->stream>>>(segs[s].w, wd, Cin, Cout, k);
        check_launch(ctx, "dgrad_weight_perm_kernel");
        t[s].x = segs[s].x;
        t[s].w = wd;
    }
    // a convolution of the errors ([Cout][N][Wo][Ho]) with flipped taps and pad k-1-pad
    conv_fprop(ctx, nseg, t, nullptr, dx, N, Cout, Ho, Wo, k, k - 1 - pad, Cin, split);
}

long conv_wgrad_scratch(int N, int Cin, int H, int W, int k, int pad, int Cout) {
    const int Ho = H + 2 * pad - k + 1, Wo = W + 2 * pad - k + 1;
    const long M = (long)N * Ho * Wo;
    const int K = Cin * k * k;
    const long tiles = (long)((K + WG_BQ - 1) / WG_BQ) * ((Cout + WG_BN - 1) / WG_BN);
    const int S = split_count(tiles, M, 512);
    const long gather = S > 1 ? (long)S * K * Cout : 0;
    return std::max(std::max(gather, conv_wgrad_tma_scratch(N, Cin, H, W, k, pad, Cout)),
                    conv_wgrad_tf32_scratch(N, Cin, H, W, k, pad, Cout));
}

void conv_wgrad(fitre_context *ctx, int nseg, const ConvSeg *segs, double *dw, int N, int Cin,
                int H, int W, int k, int pad, int Cout, double *partials) {
    if ((ctx->precision == FITRE_PRECISION_TF32 || ctx->precision == FITRE_PRECISION_TF32X3) &&
        conv_wgrad_tf32(ctx, nseg, segs, dw, N, Cin, H, W, k, pad, Cout, partials))
        return;
    if (ctx->precision == FITRE_PRECISION_FP64_I8 &&
        conv_wgrad_i8(ctx, nseg, segs, dw, N, Cin, H, W, k, pad, Cout))
        return;
    if (ctx->use_tma && conv_wgrad_tma(ctx, nseg, segs, dw, N, Cin, H, W, k, pad, Cout, partials)) return;
    WgradArgs a{};
    for (int s = 0; s < nseg; ++s) {
        a.x[s] = segs[s].x;
        a.d[s] = segs[s].w;
    }
    a.nseg = nseg;
    a.N = N; a.Cin = Cin; a.H = H; a.W = W; a.k = k; a.pad = pad; a.Cout = Cout;
    a.Ho = H + 2 * pad - k + 1;
    a.Wo = W + 2 * pad - k + 1;
    a.K = Cin * k * k;
    a.M = (long)N * a.Ho * a.Wo;
    const int tq = (a.K + WG_BQ - 1) / WG_BQ, tn = (Cout + WG_BN - 1) / WG_BN;
    const int S = split_count((long)tq * tn, a.M, 512);
    a.chunk = ((a.M + S - 1) / S + WG_BK - 1) / WG_BK * WG_BK;
    a.out = S > 1 ? partials : dw;
    dim3 grid(tq, tn, S);
    ProfScope prof(ctx, PROF_CONV_WGRAD, 2.0 * (double)a.M * a.K * Cout * nseg);
    const bool narrow = Cout <= 16;  // one 16-column tile (tn is 1 either way)
    if (k == 3) {
        if (narrow) conv_wgrad_kernel<3, true><<<grid, WG_THREADS, WG_SMEM, ctx->stream>>>(a);
        else conv_wgrad_kernel<3, false><<<grid, WG_THREADS, WG_SMEM, ctx->stream>>>(a);
    } else if (k == 5) {
        if (narrow) conv_wgrad_kernel<5, true><<<grid, WG_THREADS, WG_SMEM, ctx->stream>>>(a);
        else conv_wgrad_kernel<5, false><<<grid, WG_THREADS, WG_SMEM, ctx->stream>>>(a);
    } else {
        if (narrow) conv_wgrad_kernel<0, true><<<grid, WG_THREADS, WG_SMEM, ctx->stream>>>(a);
        else conv_wgrad_kernel<0, false><<<grid, WG_THREADS, WG_SMEM, ctx->stream>>>(a);
    }
    check_launch(ctx, "conv_wgrad_kernel");
    if (S > 1) {
        const long n = (long)a.K * Cout;
        int blocks = (int)std::min<long>((n + 255) / 256, 1184);
        if (S >= 32 && n <= 32 * 1184)
            reduce_slabs_tall_kernel<<<(unsigned)((n + 31) / 32), 256, 0, ctx->stream>>>(partials, dw, n, S, 1.0);
        else
            reduce_slabs_kernel<<<blocks, 256, 0, ctx->stream>>>(partials, dw, n, S, 1.0);
        check_launch(ctx, "reduce_slabs_kernel");
    }
}

void dgemm(fitre_context *ctx, bool tA, bool tB, int m, int n, int k, double alpha,
           const double *A, int lda, const double *B, int ldb, double beta, double *C, int ldc) {
    dgemm_structured(ctx, tA, tB, m, n, k, alpha, A, lda, B, ldb, beta, C, ldc, GEMM_FULL);
}

void dgemm_structured(fitre_context *ctx, bool tA, bool tB, int m, int n, int k, double alpha,
                      const double *A, int lda, const double *B, int ldb, double beta, double *C, int ldc,
                      int kmode) {
    if (m <= 0 || n <= 0) return;
    // large shapes: 128 x 128 tiles once they still fill the GPU
    if ((long)((m + DL_BM - 1) / DL_BM) * ((n + DL_BN - 1) / DL_BN) >= 96 && k >= 64) {
        dim3 gl((m + DL_BM - 1) / DL_BM, (n + DL_BN - 1) / DL_BN);
        if (!tA && !tB)
            dgemm_large_kernel<false, false><<<gl, DG_THREADS, DL_SMEM, ctx->stream>>>(m, n, k, alpha, A, lda, B, ldb, beta, C, ldc, kmode);
        else if (!tA && tB)
            dgemm_large_kernel<false, true><<<gl, DG_THREADS, DL_SMEM, ctx->stream>>>(m, n, k, alpha, A, lda, B, ldb, beta, C, ldc, kmode);
        else if (tA && !tB)
            dgemm_large_kernel<true, false><<<gl, DG_THREADS, DL_SMEM, ctx->stream>>>(m, n, k, alpha, A, lda, B, ldb, beta, C, ldc, kmode);
        else
            dgemm_large_kernel<true, true><<<gl, DG_THREADS, DL_SMEM, ctx->stream>>>(m, n, k, alpha, A, lda, B, ldb, beta, C, ldc, kmode);
        check_launch(ctx, "dgemm_large_kernel");
        return;
    }
    dim3 grid((m + DG_BM - 1) / DG_BM, (n + DG_BN - 1) / DG_BN);
    // at most one block per SM and a long k loop: the deep-step form (see dgemm_kernel)
    // -- but not on the side streams, where several factorisations share the SMs and a block that
    // takes 139 KB of shared memory keeps the others' blocks out
    bool side = false;
    for (cudaStream_t st : ctx->inv_streams) side = side || (st && st == ctx->stream);
    const bool deep = !side && (long)grid.x * grid.y <= 148 && k >= 128;
#define FITRE_DGEMM_LAUNCH(TA_, TB_)                                                                              \
    do {                                                                                                          \
        if (deep)                                                                                                 \
            dgemm_kernel<TA_, TB_, 64><<<grid, DG_THREADS, DG_SMEM_DEEP, ctx->stream>>>(m, n, k, alpha, A, lda, B, \
                                                                                        ldb, beta, C, ldc, kmode); \
        else                                                                                                      \
            dgemm_kernel<TA_, TB_, 16><<<grid, DG_THREADS, DG_SMEM, ctx->stream>>>(m, n, k, alpha, A, lda, B, ldb, \
                                                                                   beta, C, ldc, kmode);          \
    } while (0)
    if (!tA && !tB) FITRE_DGEMM_LAUNCH(false, false);
    else if (!tA && tB) FITRE_DGEMM_LAUNCH(false, true);
    else if (tA && !tB) FITRE_DGEMM_LAUNCH(true, false);
    else FITRE_DGEMM_LAUNCH(true, true);
#undef FITRE_DGEMM_LAUNCH
    check_launch(ctx, "dgemm_kernel");
}

static int syrk_splits(long rows, int n) {
    const long t = (n + WG_BQ - 1) / WG_BQ;
    return split_count(t * (t + 1) / 2, rows, 512);
}

long syrk_scratch(long rows, int n) { return (long)syrk_splits(rows, n) * n * n; }

void syrk_tn(fitre_context *ctx, long rows, int n, double alpha, const double *A, long lda,
             double *C, double *partials) {
    SyrkArgs a{};
    a.A = A; a.lda = lda; a.rows = rows; a.n = n;
    const int S = syrk_splits(rows, n);
    a.chunk = ((rows + S - 1) / S + WG_BK - 1) / WG_BK * WG_BK;
    a.out = partials;
    const int t = (n + WG_BQ - 1) / WG_BQ;
    dim3 grid(t, t, S);
    syrk_tn_kernel<<<grid, WG_THREADS, WG_SMEM, ctx->stream>>>(a);
    check_launch(ctx, "syrk_tn_kernel");
    const long nn = (long)n * n;
    int blocks = (int)std::min<long>((nn + 255) / 256, 1184);
    syrk_reduce_kernel<<<blocks, 256, 0, ctx->stream>>>(partials, C, n, S, alpha);
    check_launch(ctx, "syrk_reduce_kernel");
}

static int patch_syrk_splits(long M, int Kb) {
    const long t = (Kb + WG_BQ - 1) / WG_BQ;
    return split_count(t * (t + 1) / 2, M, 512);
}

long conv_patch_syrk_scratch(int N, int Cin, int H, int W, int k, int pad, bool bias) {
    const long M = (long)N * (H + 2 * pad - k + 1) * (W + 2 * pad - k + 1);
    const int Kb = Cin * k * k + (bias ? 1 : 0);
    long need = (long)patch_syrk_splits(M, Kb) * Kb * Kb;
    if (!bias) need = std::max(need, conv_patch_syrk_tma_scratch(N, Cin, H, W, k, pad));
    return need;
}

void conv_patch_syrk(fitre_context *ctx, const double *x, double *A, int N, int Cin, int H, int W,
                     int k, int pad, bool bias, double alpha, double patch_scale,
                     double *partials) {
    PatchSyrkArgs a{};
    a.x = x;
    a.out = partials;
    a.N = N; a.Cin = Cin; a.H = H; a.W = W; a.k = k; a.pad = pad;
    a.Ho = H + 2 * pad - k + 1;
    a.Wo = W + 2 * pad - k + 1;
    a.K = Cin * k * k;
    a.Kb = a.K + (bias ? 1 : 0);
    a.M = (long)N * a.Ho * a.Wo;
    const long nn = (long)a.Kb * a.Kb;
    const int blocks = (int)std::min<long>((nn + 255) / 256, 1184);
    if (!bias && ctx->use_tma) {  // the TMA kernel has no ones column
        const int St = conv_patch_syrk_tma(ctx, x, partials, N, Cin, H, W, k, pad);
        if (St > 0) {
            patch_syrk_reduce_kernel<<<blocks, 256, 0, ctx->stream>>>(partials, A, a.Kb, a.K, St, alpha,
                                                                      patch_scale);
            check_launch(ctx, "patch_syrk_reduce_kernel");
            return;
        }
    }
    const int S = patch_syrk_splits(a.M, a.Kb);
    a.chunk = ((a.M + S - 1) / S + WG_BK - 1) / WG_BK * WG_BK;
    const int t = (a.Kb + WG_BQ - 1) / WG_BQ;
    dim3 grid(t, t, S);
    if (k == 3)
        patch_syrk_kernel<3><<<grid, WG_THREADS, WG_SMEM, ctx->stream>>>(a);
    else if (k == 5)
        patch_syrk_kernel<5><<<grid, WG_THREADS, WG_SMEM, ctx->stream>>>(a);
    else
        patch_syrk_kernel<0><<<grid, WG_THREADS, WG_SMEM, ctx->stream>>>(a);
    check_launch(ctx, "patch_syrk_kernel");
    patch_syrk_reduce_kernel<<<blocks, 256, 0, ctx->stream>>>(partials, A, a.Kb, a.K, S, alpha,
                                                              patch_scale);
    check_launch(ctx, "patch_syrk_reduce_kernel");
}

void gemm_init_attributes() {
    conv_tma_init_attributes();
    conv_tf32_init_attributes();
    conv_i8_init_attributes();
    kfac_init_attributes();
    FITRE_CUDA(cudaFuncSetAttribute(conv_fprop_kernel<0, 4>, cudaFuncAttributeMaxDynamicSharedMemorySize, FP_SMEM));
    FITRE_CUDA(cudaFuncSetAttribute(conv_fprop_kernel<0, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, FP_SMEM));
    FITRE_CUDA(cudaFuncSetAttribute(conv_fprop_kernel<3, 4>, cudaFuncAttributeMaxDynamicSharedMemorySize, FP_SMEM));
    FITRE_CUDA(cudaFuncSetAttribute(conv_fprop_kernel<3, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, FP_SMEM));
    FITRE_CUDA(cudaFuncSetAttribute(conv_fprop_kernel<5, 4>, cudaFuncAttributeMaxDynamicSharedMemorySize, FP_SMEM));
    FITRE_CUDA(cudaFuncSetAttribute(conv_fprop_kernel<5, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, FP_SMEM));
    FITRE_CUDA(cudaFuncSetAttribute(conv_wgrad_kernel<0, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, WG_SMEM));
    FITRE_CUDA(cudaFuncSetAttribute(conv_wgrad_kernel<0, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, WG_SMEM));
    FITRE_CUDA(cudaFuncSetAttribute(conv_wgrad_kernel<3, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, WG_SMEM));
    FITRE_CUDA(cudaFuncSetAttribute(conv_wgrad_kernel<3, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, WG_SMEM));
    FITRE_CUDA(cudaFuncSetAttribute(conv_wgrad_kernel<5, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, WG_SMEM));
    FITRE_CUDA(cudaFuncSetAttribute(conv_wgrad_kernel<5, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, WG_SMEM));
    FITRE_CUDA(cudaFuncSetAttribute(patch_syrk_kernel<0>, cudaFuncAttributeMaxDynamicSharedMemorySize, WG_SMEM));
    FITRE_CUDA(cudaFuncSetAttribute(patch_syrk_kernel<3>, cudaFuncAttributeMaxDynamicSharedMemorySize, WG_SMEM));
    FITRE_CUDA(cudaFuncSetAttribute(patch_syrk_kernel<5>, cudaFuncAttributeMaxDynamicSharedMemorySize, WG_SMEM));
    FITRE_CUDA(cudaFuncSetAttribute(syrk_tn_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, WG_SMEM));
    FITRE_CUDA(cudaFuncSetAttribute(dgemm_kernel<false, false, 64>, cudaFuncAttributeMaxDynamicSharedMemorySize, DG_SMEM_DEEP));
    FITRE_CUDA(cudaFuncSetAttribute(dgemm_kernel<false, true, 64>, cudaFuncAttributeMaxDynamicSharedMemorySize, DG_SMEM_DEEP));
    FITRE_CUDA(cudaFuncSetAttribute(dgemm_kernel<true, false, 64>, cudaFuncAttributeMaxDynamicSharedMemorySize, DG_SMEM_DEEP));
    FITRE_CUDA(cudaFuncSetAttribute(dgemm_kernel<true, true, 64>, cudaFuncAttributeMaxDynamicSharedMemorySize, DG_SMEM_DEEP));
    FITRE_CUDA(cudaFuncSetAttribute(dgemm_large_kernel<false, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, DL_SMEM));
    FITRE_CUDA(cudaFuncSetAttribute(dgemm_large_kernel<false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, DL_SMEM));
    FITRE_CUDA(cudaFuncSetAttribute(dgemm_large_kernel<true, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, DL_SMEM));
    FITRE_CUDA(cudaFuncSetAttribute(dgemm_large_kernel<true, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, DL_SMEM));
}

}  // namespace fitre

// ---------------------------------------------------------------------------------------------
// Allocation-free variant of the A'A product (the KFAC G-factor kernel).
//
// Some callers cannot allocate device memory at all: a driver that has already handed every
// free byte to its own bump-pointer workspace (the reference does exactly that,
// device/cuda_environment.c:48-66), code running between the capture calls of a stream, or a
// host thread that is not allowed to take the allocator's lock.  For them the split-sum slabs
// of the product live in the fixed device array below instead of caller-provided scratch.
// Every GPU that loads this library holds the array (8 MiB) until the process exits.
// ---------------------------------------------------------------------------------------------
namespace fitre {
namespace {
constexpr long kStaticSlabDoubles = 1L << 20;  // 8 MiB: the stated maximum of the entry point
static __device__ __align__(256) double g_static_slabs[kStaticSlabDoubles];
constexpr int kMaxDevices = 64;
double *g_static_slabs_addr[kMaxDevices];  // device address per device, resolved on first use
std::mutex g_static_slabs_mutex;
}  // namespace
}  // namespace fitre

// C (n x n, column-major, both triangles) = alpha * A' A, A rows x n column-major with leading
// dimension lda.  Same kernels and the same arithmetic as the G-factor blocks of
// fitre_kfac_lambda_delta; the only difference is where the split-sum slabs live.
//   * allocates nothing: no cudaMalloc / cudaFree, no allocating library call, no context;
//   * the first call on a device looks the array's device address up (cudaGetSymbolAddress on
//     the current device); make that first call before starting any stream capture;
//   * limit: splits * n * n <= 2^20 doubles, so n <= 1024; larger n returns
//     FITRE_ERR_TOO_LARGE and prints the limit;
//   * every call on a device shares the one array and leaves its slabs behind; the kernels
//     overwrite every slab entry they later read, so nothing needs clearing, but two calls
//     whose kernels overlap on the GPU (different streams) race on it: serialise them.
extern "C" int fitre_syrk_tn_static_scratch(const real *A, long rows, int n, long lda, real alpha,
                                            real *C, void *stream) {
    using namespace fitre;
    if (!A || !C || rows < 1 || n < 1 || lda < rows) return FITRE_ERR_BAD_ARG;
    const long nn = (long)n * n;
    if (nn > kStaticSlabDoubles) {
        std::fprintf(stderr,
                     "fitre_syrk_tn_static_scratch: n = %d needs %ld doubles of slab space, the "
                     "built-in array holds %ld (n <= 1024)\n", n, nn, kStaticSlabDoubles);
        return FITRE_ERR_TOO_LARGE;
    }
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return FITRE_ERR_CUDA;
    double *slabs = nullptr;
    {
        std::lock_guard<std::mutex> lock(g_static_slabs_mutex);
        if (!g_static_slabs_addr[dev]) {
            // In host code the array's name is only a handle; the kernels need this address.
            void *p = nullptr;
            if (cudaGetSymbolAddress(&p, g_static_slabs) != cudaSuccess || !p) {
                cudaGetLastError();
                return FITRE_ERR_CUDA;
            }
            g_static_slabs_addr[dev] = (double *)p;
        }
        slabs = g_static_slabs_addr[dev];
    }
    const long t = (n + WG_BQ - 1) / WG_BQ;
    long S = split_count(t * (t + 1) / 2, rows, 512);
    S = std::max(1L, std::min(S, kStaticSlabDoubles / nn));  // fewer splits rather than more space
    SyrkArgs a{};
    a.A = A;
    a.lda = lda;
    a.rows = rows;
    a.n = n;
    a.chunk = ((rows + S - 1) / S + WG_BK - 1) / WG_BK * WG_BK;
    a.out = slabs;
    cudaStream_t st = (cudaStream_t)stream;
    dim3 grid((unsigned)t, (unsigned)t, (unsigned)S);
    syrk_tn_kernel<<<grid, WG_THREADS, WG_SMEM, st>>>(a);
    if (cudaGetLastError() != cudaSuccess) return FITRE_ERR_CUDA;
    const int blocks = (int)std::min<long>((nn + 255) / 256, 1184);
    syrk_reduce_kernel<<<blocks, 256, 0, st>>>(slabs, C, n, (int)S, alpha);
    if (cudaGetLastError() != cudaSuccess) return FITRE_ERR_CUDA;
    return FITRE_OK;
}
