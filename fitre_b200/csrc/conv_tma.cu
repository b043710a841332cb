// TMA-fed implicit-GEMM convolution (forward / data-gradient shape) for sm_100a, fp64 DMMA.
//
// Y[M x Cout] = sum_seg im2col(X_seg) * W_seg, computed without ever forming im2col:
//  * a CTA owns 128 output positions chosen as a box (all Ho rows) x (TW columns) x (TN images)
//    and 64 output channels;
//  * per K-chunk of 4 input channels one `cp.async.bulk.tensor.4d` brings the raw input patch
//    of that box -- halo included, zero-filled outside the image, which is exactly the padding
//    rule of the reference's im2col (functions/dev_image.cu:45-47) -- and one
//    `cp.async.bulk.tensor.2d` brings the matching (4*k*k) x 64 slab of the weight matrix;
//  * the DMMA A fragments are read straight out of the patch: im2col element (m, q) with
//    m = (n, wo, ho), q = (cin, j, i) lives at patch[cin][n][wo + j][ho + i], so the gather is
//    one shared-memory load with address rowbase(m) + colofs(q);
//  * stages form a ring guarded by mbarriers (complete_tx); every wait is bounded and reports
//    through an error word instead of spinning forever.
// No cluster multicast is used anywhere (each CTA fetches its own tiles).
#include <cstdlib>
#include <cuda.h>

#include <algorithm>
#include <cstdint>
#include <mutex>

#include "common.h"
#include "tma_util.cuh"

namespace fitre {
namespace {

constexpr int T_BM = 128, T_BN = 64, T_THREADS = 256;
constexpr int kSmemBudget = 110 * 1024;  // two CTAs per SM
// Input channels per K-chunk of the forward / data-gradient kernel.  3x3 taps: 4 channels = 36
// rows of the weight matrix.  5x5 taps: 2 channels = 50 rows, carried as 52 (the DMMA step is 4
// rows; the two extra rows belong to the next chunk and meet zeros on the A side), so that a
// ring of three stages fits the shared memory of two resident blocks.  36 and 52 are both
// 4 mod 16: the B fragments of 8 channels x 4 rows then fall into distinct banks.
__host__ __device__ constexpr int chunk_channels(int ks) { return ks == 5 ? 2 : 4; }

struct alignas(64) TmaConvArgs {
    CUtensorMap xmap[2];
    CUtensorMap wmap[2];
    const double *bias;
    double *y;
    int *err;
    long M;
    int nseg, N, Cout, Ho, Wo, pad, TW, TN, HB, WB, xoff, x0, nchunks, stages, tilesW;
    int patchBytes;
    int iters_per_split;  // K-chunk iterations per blockIdx.z slice (split-K: slabs in y)
};

template <int KS>
__global__ void __launch_bounds__(T_THREADS, 2)
conv_tma_kernel(const __grid_constant__ TmaConvArgs p) {
    constexpr int T_CB = chunk_channels(KS);
    constexpr int KROWS = T_CB * KS * KS;   // rows of the weight matrix one chunk consumes: 36 / 50
    constexpr int KCH = (KROWS + 3) & ~3;   // rows one stage holds: 36 / 52
    // Aligned by declaration, not by rounding the address: a pointer that went through an integer is a
    // generic pointer to the compiler, and generic loads of shared memory cost the DMMA loop 5 %
    // (35.2 against 37.0 TFLOP/s in a fragment-load + DMMA loop over a resident tile).
    extern __shared__ __align__(1024) unsigned char smraw[];
    unsigned char *sm = smraw;
    const int stageBytes = p.patchBytes + KCH * T_BN * 8;
    int *colofs = (int *)(sm + (size_t)p.stages * stageBytes);
    unsigned long long *bars = (unsigned long long *)(colofs + ((KCH + 3) & ~3) + 4);
    __shared__ int abort_flag;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int warp_m = warp & 3, warp_n = warp >> 2;
    const int lr = lane >> 2, lc = lane & 3;
    const int wt = blockIdx.x % p.tilesW, nt = blockIdx.x / p.tilesW;
    const int w0 = wt * p.TW, n0 = nt * p.TN;
    const int c0 = blockIdx.y * T_BN;

    // bars[s]: "full" (TMA bytes landed); bars[4 + s]: "empty" (all 8 warps done reading)
    if (tid == 0) {
        abort_flag = 0;
        for (int s = 0; s < p.stages; ++s) {
            mbar_init(smem_u32(bars + s), 1);
            mbar_init(smem_u32(bars + 4 + s), T_THREADS / 32);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    for (int q = tid; q < KCH; q += T_THREADS) {
        const int cl = q / (KS * KS), rem = q - cl * (KS * KS);
        const int j = rem / KS, i = rem - j * KS;
        colofs[q] = q < KROWS ? (cl * p.TN * p.WB + j) * p.HB + i : 0;
    }
    __syncthreads();

    // rows of this thread's A fragments and of its output elements
    int rowbase[4];
    long grow[4];
#pragma unroll
    for (int mi = 0; mi < 4; ++mi) {
        const int ml = warp_m * 32 + mi * 8 + lr;
        const int ho = ml % p.Ho, r = ml / p.Ho;
        const int wl = r % p.TW, nl = r / p.TW;
        rowbase[mi] = (nl * p.WB + wl) * p.HB + ho + p.xoff;
        const bool ok = (n0 + nl) < p.N && (w0 + wl) < p.Wo && nl < p.TN;
        grow[mi] = ok ? ((long)(n0 + nl) * p.Wo + (w0 + wl)) * p.Ho + ho : -1;
    }

    // split-K: slice blockIdx.z owns iterations [it0, it0 + iters) of the flattened
    // (segment, K-chunk) sequence and writes its own output slab
    const int it0 = blockIdx.z * p.iters_per_split;
    const int iters = max(0, min(p.nseg * p.nchunks - it0, p.iters_per_split));
    const uint32_t txBytes = (uint32_t)(p.HB * p.WB * p.TN * T_CB * 8 + KCH * T_BN * 8);
    auto issue = [&](int it) {
        const int seg = (it0 + it) / p.nchunks, ch = (it0 + it) - seg * p.nchunks;
        const int s = it % p.stages;
        const uint32_t bar = smem_u32(bars + s);
        unsigned char *dst = sm + (size_t)s * stageBytes;
        mbar_expect_tx(bar, txBytes);
        tma_load_4d(smem_u32(dst), &p.xmap[seg], bar, p.x0, w0 - p.pad, n0, ch * T_CB);
        tma_load_2d(smem_u32(dst + p.patchBytes), &p.wmap[seg], bar, ch * KROWS, c0);
    };
    if (tid == 0)
        for (int it = 0; it < p.stages - 1 && it < iters; ++it) issue(it);

    double acc[4][4][2];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j][0] = acc[i][j][1] = 0.0;

    // Warps run decoupled: a stage is refilled once every warp has arrived on its "empty"
    // barrier; only the issuing thread waits for that, the others go on to the next stage.
    volatile int *vabort = &abort_flag;
    for (int it = 0; it < iters; ++it) {
        const int s = it % p.stages;
        if (tid == 0 && it + p.stages - 1 < iters) {
            const int nit = it + p.stages - 1, use = nit / p.stages;
            if (use > 0 && !mbar_wait(smem_u32(bars + 4 + nit % p.stages), (uint32_t)((use - 1) & 1)))
                *vabort = 1;
            else
                issue(nit);
        }
        if (*vabort || !mbar_wait(smem_u32(bars + s), (uint32_t)((it / p.stages) & 1))) {
            *vabort = 1;
            break;
        }
        {
            const double *patch = (const double *)(sm + (size_t)s * stageBytes);
            const double *Bs = (const double *)(sm + (size_t)s * stageBytes + p.patchBytes) +
                               (warp_n * 32 + lr) * KCH + lc;
#pragma unroll
            for (int k4 = 0; k4 < KCH / 4; ++k4) {
                const int co = colofs[k4 * 4 + lc];
                double fa[4], fb[4];
#pragma unroll
                for (int mi = 0; mi < 4; ++mi) fa[mi] = patch[co + rowbase[mi]];
                if (KROWS != KCH && k4 == KCH / 4 - 1 && k4 * 4 + lc >= KROWS) {
                    // rows past the chunk hold the next chunk's weights: they meet zeros
#pragma unroll
                    for (int mi = 0; mi < 4; ++mi) fa[mi] = 0.0;
                }
#pragma unroll
                for (int ni = 0; ni < 4; ++ni) fb[ni] = Bs[ni * 8 * KCH + k4 * 4];
#pragma unroll
                for (int mi = 0; mi < 4; ++mi)
#pragma unroll
                    for (int ni = 0; ni < 4; ++ni)
                        dmma884(acc[mi][ni][0], acc[mi][ni][1], fa[mi], fb[ni]);
            }
        }
        release_stage_reads();
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(bars + 4 + s));
    }
    __syncthreads();
    if (abort_flag) {
        if (tid == 0) atomicExch(p.err, 1);
        return;
    }

    double *y = p.y + (long)blockIdx.z * p.M * p.Cout;
#pragma unroll
    for (int ni = 0; ni < 4; ++ni)
#pragma unroll
        for (int e = 0; e < 2; ++e) {
            const int col = c0 + warp_n * 32 + ni * 8 + 2 * lc + e;
            if (col >= p.Cout) continue;
            const double bv = p.bias ? p.bias[col] : 0.0;
#pragma unroll
            for (int mi = 0; mi < 4; ++mi)
                if (grow[mi] >= 0) y[(long)col * p.M + grow[mi]] = acc[mi][ni][e] + bv;
        }
}

// y[c][m] = sum over split-K slabs (fixed order) + bias[c]
__global__ void reduce_out_slabs_kernel(const double *slabs, double *y, long M, int Cout, int SK,
                                        const double *bias) {
    const long n = M * Cout;
    for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < n;
         i += (long)gridDim.x * blockDim.x) {
        double s = 0.0;
        for (int k = 0; k < SK; ++k) s += slabs[(long)k * n + i];
        if (bias) s += bias[i / M];
        y[i] = s;
    }
}


// ---------------------------------------------------------------------------------------------
// TMA-fed weight gradient: dW[K x Cout] = sum_seg im2col(X_seg)' * D_seg, reduction over
// M = N*Ho*Wo split across blockIdx.z (slabs summed afterwards in fixed order).
// CTA tile: 128 rows of q = (cin, j, i) x 64 output channels.  Per step of BMT output positions
// (a box: all Ho rows x TW columns x TN images, contiguous in M) TMA brings
//   * the raw input patch of that box for the <= CBW input channels the 128 q-rows touch, and
//   * the BMT x 64 slab of the errors as BMT/16 boxes with the 128-byte swizzle, so that the
//     DMMA B fragments (4 consecutive m x 8 channels) are read without bank conflicts.
// A fragments come straight from the patch: element (q, m) = patch[rowbase(m) + qofs(q)].
// ---------------------------------------------------------------------------------------------
constexpr int W_BQ = 128, W_BN = 64;

struct alignas(64) TmaWgradArgs {
    CUtensorMap xmap[2];
    CUtensorMap dmap[2];
    double *out;   // dW (splits == 1) or slabs [split][K*Cout]
    int *err;
    long M;
    int nseg, N, K, Cout, Ho, Wo, pad, TW, TN, HB, WB, xoff, x0, CBW, stages, tilesW;
    int tiles_total, tiles_per_split, patchBytes;
};

template <int KS, int BMT>
__global__ void __launch_bounds__(T_THREADS, 2)
wgrad_tma_kernel(const __grid_constant__ TmaWgradArgs p) {
    extern __shared__ __align__(1024) unsigned char smraw[];
    unsigned char *sm = smraw;
    constexpr int dBytes = BMT * W_BN * 8;           // BMT/16 swizzled boxes of 16 x 64 doubles
    const int stageBytes = dBytes + p.patchBytes;    // [errors | patch], both 1024-aligned
    int *rowbase_s = (int *)(sm + (size_t)p.stages * stageBytes);
    unsigned long long *bars = (unsigned long long *)(rowbase_s + BMT);
    __shared__ int abort_flag;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int warp_q = warp & 3, warp_n = warp >> 2;
    const int lr = lane >> 2, lc = lane & 3;
    const int q0 = blockIdx.x * W_BQ, c0 = blockIdx.y * W_BN;
    const int c_lo = q0 / (KS * KS);

    if (tid == 0) {
        abort_flag = 0;
        for (int s = 0; s < p.stages; ++s) {
            mbar_init(smem_u32(bars + s), 1);                  // full
            mbar_init(smem_u32(bars + 4 + s), T_THREADS / 32);  // empty
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    for (int ml = tid; ml < BMT; ml += T_THREADS) {
        const int ho = ml % p.Ho, r = ml / p.Ho;
        const int wl = r % p.TW, nl = r / p.TW;
        rowbase_s[ml] = (nl * p.WB + wl) * p.HB + ho + p.xoff;
    }
    __syncthreads();

    // Rows q >= K of the last tile fall on channels >= Cin, which TMA zero-fills; a 128-row tile
    // never spans more than CBW channels, so every offset stays inside the patch.
    int qofs[4];
#pragma unroll
    for (int mi = 0; mi < 4; ++mi) {
        const int q = q0 + warp_q * 32 + mi * 8 + lr;
        const int c = q / (KS * KS), rem = q - c * (KS * KS);
        const int j = rem / KS, i = rem - j * KS;
        qofs[mi] = ((c - c_lo) * p.TN * p.WB + j) * p.HB + i;
    }
    // swizzled B addressing: channel row r = warp_n*32 + (ni>>1)*16 + 2*lr + (ni&1); within a
    // 16-double box row the 16-byte chunk index is XORed with (r & 7) = (2*lr + (ni&1)) & 7
    const int boff0 = (warp_n * 32 + 2 * lr) * 16 + (lc & 1);
    const int bx0 = (2 * lr) & 7, bx1 = (2 * lr + 1) & 7;

    const int t_beg = blockIdx.z * p.tiles_per_split;
    const int t_end = min(p.tiles_total, t_beg + p.tiles_per_split);
    const int ntile = max(0, t_end - t_beg);
    const int iters = ntile * p.nseg;
    const uint32_t txBytes = (uint32_t)(p.HB * p.WB * p.TN * p.CBW * 8 + dBytes);
    auto issue = [&](int it) {
        const int seg = it / ntile, t = t_beg + (it - seg * ntile);
        const int wt = t % p.tilesW, nt = t / p.tilesW;
        const int s = it % p.stages;
        const uint32_t bar = smem_u32(bars + s);
        unsigned char *dst = sm + (size_t)s * stageBytes;
        mbar_expect_tx(bar, txBytes);
        const int mstart = t * BMT;
#pragma unroll
        for (int b = 0; b < BMT / 16; ++b)
            tma_load_2d(smem_u32(dst + b * (16 * W_BN * 8)), &p.dmap[seg], bar, mstart + 16 * b, c0);
        tma_load_4d(smem_u32(dst + dBytes), &p.xmap[seg], bar, p.x0, wt * p.TW - p.pad, nt * p.TN, c_lo);
    };
    if (tid == 0)
        for (int it = 0; it < p.stages - 1 && it < iters; ++it) issue(it);

    double acc[4][4][2];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j][0] = acc[i][j][1] = 0.0;

    volatile int *vabort = &abort_flag;
    for (int it = 0; it < iters; ++it) {
        const int s = it % p.stages;
        if (tid == 0 && it + p.stages - 1 < iters) {
            const int nit = it + p.stages - 1, use = nit / p.stages;
            if (use > 0 && !mbar_wait(smem_u32(bars + 4 + nit % p.stages), (uint32_t)((use - 1) & 1)))
                *vabort = 1;
            else
                issue(nit);
        }
        if (*vabort || !mbar_wait(smem_u32(bars + s), (uint32_t)((it / p.stages) & 1))) {
            *vabort = 1;
            break;
        }
        {
            const double *dS = (const double *)(sm + (size_t)s * stageBytes);
            const double *patch = (const double *)(sm + (size_t)s * stageBytes + dBytes);
#pragma unroll
            for (int k4 = 0; k4 < BMT / 4; ++k4) {
                const int rb = rowbase_s[k4 * 4 + lc];
                const double *box = dS + (k4 >> 2) * (16 * W_BN);
                const int chunk = (k4 & 3) * 2 + (lc >> 1);
                double fa[4], fb[4];
#pragma unroll
                for (int mi = 0; mi < 4; ++mi) fa[mi] = patch[rb + qofs[mi]];
#pragma unroll
                for (int ni = 0; ni < 4; ++ni)
                    fb[ni] = box[boff0 + ((ni >> 1) * 16 + (ni & 1)) * 16 +
                                 ((chunk ^ ((ni & 1) ? bx1 : bx0)) << 1)];
#pragma unroll
                for (int mi = 0; mi < 4; ++mi)
#pragma unroll
                    for (int ni = 0; ni < 4; ++ni)
                        dmma884(acc[mi][ni][0], acc[mi][ni][1], fa[mi], fb[ni]);
            }
        }
        release_stage_reads();
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(bars + 4 + s));
    }
    __syncthreads();
    if (abort_flag) {
        if (tid == 0) atomicExch(p.err, 1);
        return;
    }

    double *out = p.out + (long)blockIdx.z * p.K * p.Cout;
#pragma unroll
    for (int ni = 0; ni < 4; ++ni)
#pragma unroll
        for (int e = 0; e < 2; ++e) {
            // mma column 2*lc+e of tile ni is channel row warp_n*32 + (ni>>1)*16 + 2*(2*lc+e) + (ni&1)
            const int col = c0 + warp_n * 32 + (ni >> 1) * 16 + 2 * (2 * lc + e) + (ni & 1);
            if (col >= p.Cout) continue;
#pragma unroll
            for (int mi = 0; mi < 4; ++mi) {
                const int row = q0 + warp_q * 32 + mi * 8 + lr;
                if (row < p.K) out[(long)col * p.K + row] = acc[mi][ni][e];
            }
        }
}

// ---------------------------------------------------------------------------------------------
// TMA-fed KFAC A factor of a convolution without bias column: slab = im2col(X)' im2col(X)
// (solvers/kfac_inverses.cu:515-540 forms the patch matrix and multiplies it by itself), the same
// data flow as the weight gradient above with the errors replaced by a second raw patch: CTA tile
// 128 rows q x 64 columns q', both operands read straight from the raw input boxes in shared
// memory (element (q, m) = patch[rowbase(m) + qofs(q)]).  Only tiles that touch the lower
// triangle are computed; scaling and the mirror image are applied by the caller's reducer.
// ---------------------------------------------------------------------------------------------
struct alignas(64) TmaSyrkArgs {
    CUtensorMap amap, bmap;  // same tensor, boxes of CBW / CBB channels
    double *out;             // slabs [split][K*K]
    int *err;
    long M;
    int N, K, Ho, Wo, pad, TW, TN, HB, WB, xoff, x0, CBW, CBB, stages, tilesW;
    int tiles_total, tiles_per_split, patchBytesA, patchBytesB;
};

template <int KS, int BMT>
__global__ void __launch_bounds__(T_THREADS, 2)
patch_syrk_tma_kernel(const __grid_constant__ TmaSyrkArgs p) {
    const int q0 = blockIdx.x * W_BQ, c0 = blockIdx.y * W_BN;
    if (c0 > q0 + W_BQ - 1) return;  // strictly above the diagonal: mirrored by the reducer
    extern __shared__ __align__(1024) unsigned char smraw[];
    unsigned char *sm = smraw;
    const int stageBytes = p.patchBytesA + p.patchBytesB;  // [patch of the rows | patch of the columns]
    int *rowbase_s = (int *)(sm + (size_t)p.stages * stageBytes);
    unsigned long long *bars = (unsigned long long *)(rowbase_s + BMT);
    __shared__ int abort_flag;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int warp_q = warp & 3, warp_n = warp >> 2;
    const int lr = lane >> 2, lc = lane & 3;
    const int ca_lo = q0 / (KS * KS), cb_lo = c0 / (KS * KS);

    if (tid == 0) {
        abort_flag = 0;
        for (int s = 0; s < p.stages; ++s) {
            mbar_init(smem_u32(bars + s), 1);                  // full
            mbar_init(smem_u32(bars + 4 + s), T_THREADS / 32);  // empty
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    for (int ml = tid; ml < BMT; ml += T_THREADS) {
        const int ho = ml % p.Ho, r = ml / p.Ho;
        const int wl = r % p.TW, nl = r / p.TW;
        rowbase_s[ml] = (nl * p.WB + wl) * p.HB + ho + p.xoff;
    }
    __syncthreads();

    // q >= K falls on channels >= Cin, which TMA zero-fills; 128 rows span at most CBW channels and
    // 64 columns at most CBB, so every offset stays inside its patch
    int qa[4], qb[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int q = q0 + warp_q * 32 + i * 8 + lr;
        const int c = q / (KS * KS), rem = q - c * (KS * KS);
        const int j = rem / KS, ii = rem - j * KS;
        qa[i] = ((c - ca_lo) * p.TN * p.WB + j) * p.HB + ii;
        const int q2 = c0 + warp_n * 32 + i * 8 + lr;
        const int c2 = q2 / (KS * KS), rem2 = q2 - c2 * (KS * KS);
        const int j2 = rem2 / KS, i2 = rem2 - j2 * KS;
        qb[i] = ((c2 - cb_lo) * p.TN * p.WB + j2) * p.HB + i2;
    }

    const int t_beg = blockIdx.z * p.tiles_per_split;
    const int t_end = min(p.tiles_total, t_beg + p.tiles_per_split);
    const int iters = max(0, t_end - t_beg);
    const uint32_t txBytes = (uint32_t)(p.HB * p.WB * p.TN * (p.CBW + p.CBB) * 8);
    auto issue = [&](int it) {
        const int t = t_beg + it;
        const int wt = t % p.tilesW, nt = t / p.tilesW;
        const int s = it % p.stages;
        const uint32_t bar = smem_u32(bars + s);
        unsigned char *dst = sm + (size_t)s * stageBytes;
        mbar_expect_tx(bar, txBytes);
        tma_load_4d(smem_u32(dst), &p.amap, bar, p.x0, wt * p.TW - p.pad, nt * p.TN, ca_lo);
        tma_load_4d(smem_u32(dst + p.patchBytesA), &p.bmap, bar, p.x0, wt * p.TW - p.pad, nt * p.TN, cb_lo);
    };
    if (tid == 0)
        for (int it = 0; it < p.stages - 1 && it < iters; ++it) issue(it);

    double acc[4][4][2];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j][0] = acc[i][j][1] = 0.0;

    volatile int *vabort = &abort_flag;
    for (int it = 0; it < iters; ++it) {
        const int s = it % p.stages;
        if (tid == 0 && it + p.stages - 1 < iters) {
            const int nit = it + p.stages - 1, use = nit / p.stages;
            if (use > 0 && !mbar_wait(smem_u32(bars + 4 + nit % p.stages), (uint32_t)((use - 1) & 1)))
                *vabort = 1;
            else
                issue(nit);
        }
        if (*vabort || !mbar_wait(smem_u32(bars + s), (uint32_t)((it / p.stages) & 1))) {
            *vabort = 1;
            break;
        }
        {
            const double *pa = (const double *)(sm + (size_t)s * stageBytes);
            const double *pb = (const double *)(sm + (size_t)s * stageBytes + p.patchBytesA);
#pragma unroll
            for (int k4 = 0; k4 < BMT / 4; ++k4) {
                const int rb = rowbase_s[k4 * 4 + lc];
                double fa[4], fb[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    fa[i] = pa[rb + qa[i]];
                    fb[i] = pb[rb + qb[i]];
                }
#pragma unroll
                for (int mi = 0; mi < 4; ++mi)
#pragma unroll
                    for (int ni = 0; ni < 4; ++ni)
                        dmma884(acc[mi][ni][0], acc[mi][ni][1], fa[mi], fb[ni]);
            }
        }
        release_stage_reads();
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(bars + 4 + s));
    }
    __syncthreads();
    if (abort_flag) {
        if (tid == 0) atomicExch(p.err, 1);
        return;
    }

    double *out = p.out + (long)blockIdx.z * p.K * p.K;
#pragma unroll
    for (int ni = 0; ni < 4; ++ni)
#pragma unroll
        for (int e = 0; e < 2; ++e) {
            const int col = c0 + warp_n * 32 + ni * 8 + 2 * lc + e;
            if (col >= p.K) continue;
#pragma unroll
            for (int mi = 0; mi < 4; ++mi) {
                const int row = q0 + warp_q * 32 + mi * 8 + lr;
                if (row < p.K) out[(long)col * p.K + row] = acc[mi][ni][e];
            }
        }
}

__global__ void reduce_slabs_tma_kernel(const double *partial, double *out, long n, int slabs) {
    for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < n;
         i += (long)gridDim.x * blockDim.x) {
        double s = 0.0;
        for (int k = 0; k < slabs; ++k) s += partial[(long)k * n + i];
        out[i] = s;
    }
}

// Picks the split count that minimises a simple time model: waves of 296 CTAs (2 per SM) times
// the steps each CTA runs, plus the slab write/read traffic a split adds.
int best_split(long tiles, int steps, int max_split, int min_steps, double step_us, double slab_bytes) {
    int best = 1;
    double best_t = 1e300;
    for (int s = 1; s <= max_split; ++s) {
        const int per = (steps + s - 1) / s;
        if (s > 1 && per < min_steps) break;
        const long ctas = tiles * s;
        const long waves = (ctas + 295) / 296;
        // a last wave that fills less than half of the slots runs with one CTA per SM, i.e. faster
        const double tail = (ctas - (waves - 1) * 296 <= 148) ? 0.55 : 1.0;
        double t = ((waves - 1) + tail) * per * step_us;
        if (s > 1) t += (s + 2) * slab_bytes / 5.0e6;  // bytes / (5 TB/s) in microseconds
        if (t < best_t * 0.98) {
            best_t = t;
            best = s;
        }
    }
    return best;
}

// Tiling plan of the TMA weight-gradient kernel; ok == false when shape/alignment rule it out.
struct WgradPlan {
    bool ok = false;
    int BMT = 0, TW = 0, TN = 0, HB = 0, WB = 0, x0 = 0, xoff = 0, CBW = 0, patchBytes = 0;
    int stages = 0, tiles_total = 0, splits = 1, tiles_per_split = 0, tq = 0, tn = 0, smem = 0;
};

WgradPlan wgrad_plan(int N, int Cin, int H, int W, int k, int pad, int Cout) {
    WgradPlan pl;
    if (!encode_fn() || (k != 3 && k != 5)) return pl;
    if (Cin * k * k <= 64) return pl;  // a 128-row q tile would be mostly empty: gather kernel
    const int Ho = H + 2 * pad - k + 1, Wo = W + 2 * pad - k + 1;
    const long M = (long)N * Ho * Wo;
    if (Ho < 1 || Wo < 1 || (H & 1) || (M & 1)) return pl;
    const int padE = pad + (pad & 1);
    pl.x0 = -padE;
    pl.xoff = padE - pad;
    pl.HB = (H + pad + padE + 1) & ~1;
    pl.CBW = (k == 3) ? 16 : 8;  // input channels a 128-row q tile can touch
    for (int bmt : {64, 32}) {
        int TW, TN;
        if (Ho * Wo >= bmt) {
            if (bmt % Ho) continue;
            TW = bmt / Ho;
            TN = 1;
            if (Wo % TW) continue;
        } else {
            if (bmt % (Ho * Wo)) continue;
            TW = Wo;
            TN = bmt / (Ho * Wo);
        }
        const int WB = TW + k - 1;
        if (pl.HB > 256 || WB > 256 || TN > 256) continue;
        const int patchBytes = (pl.HB * WB * TN * pl.CBW * 8 + 1023) & ~1023;
        const int stageBytes = bmt * W_BN * 8 + patchBytes;
        const int fixed = 1024 + bmt * 4 + 8 * 8;
        int stages = (kSmemBudget - fixed) / stageBytes;
        if (stages < 2) continue;
        pl.BMT = bmt; pl.TW = TW; pl.TN = TN; pl.WB = WB; pl.patchBytes = patchBytes;
        pl.stages = std::min(stages, 4);
        pl.smem = pl.stages * stageBytes + fixed;
        pl.ok = true;
        break;
    }
    if (!pl.ok) return pl;
    const int K = Cin * k * k;
    pl.tq = (K + W_BQ - 1) / W_BQ;
    pl.tn = (Cout + W_BN - 1) / W_BN;
    pl.tiles_total = (int)((M + pl.BMT - 1) / pl.BMT);
    const long tiles = (long)pl.tq * pl.tn;
    const double step_us = 8.3 * pl.BMT / 64.0;  // one BMT x 128 x 64 step with two CTAs per SM
    pl.splits = best_split(tiles, pl.tiles_total, 256, 8, step_us, (double)K * Cout * 8);
    // One wave of equal blocks does not end together: a block whose neighbour on the SM has
    // retired runs at twice the rate, and the slots it leaves stay empty.  Four times finer units
    // (down to 8 steps each) let the block scheduler even that out; measured on VGG-11-BN at 512
    // images 31.5 -> 32.6 TFLOP/s, 2x and 8x finer gave less.
    {
        int finer = pl.splits * 4;
        while (finer > pl.splits && pl.tiles_total / finer < 8) --finer;
        pl.splits = std::max(pl.splits, finer);
    }
    pl.tiles_per_split = (pl.tiles_total + pl.splits - 1) / pl.splits;
    pl.splits = (pl.tiles_total + pl.tiles_per_split - 1) / pl.tiles_per_split;
    return pl;
}

// Tiling plan of the TMA A-factor kernel; ok == false when shape/alignment rule it out.
struct SyrkPlan {
    bool ok = false;
    int BMT = 0, TW = 0, TN = 0, HB = 0, WB = 0, x0 = 0, xoff = 0, CBW = 0, CBB = 0;
    int patchBytesA = 0, patchBytesB = 0, stages = 0, tiles_total = 0, splits = 1, tiles_per_split = 0;
    int tq = 0, tn = 0, smem = 0;
};

SyrkPlan syrk_plan(int N, int Cin, int H, int W, int k, int pad) {
    SyrkPlan pl;
    if (!encode_fn() || (k != 3 && k != 5)) return pl;
    const int K = Cin * k * k;
    if (K <= 128) return pl;  // one mostly empty tile: gather kernel
    const int Ho = H + 2 * pad - k + 1, Wo = W + 2 * pad - k + 1;
    const long M = (long)N * Ho * Wo;
    if (Ho < 1 || Wo < 1 || (H & 1) || (M & 1)) return pl;
    const int padE = pad + (pad & 1);
    pl.x0 = -padE;
    pl.xoff = padE - pad;
    pl.HB = (H + pad + padE + 1) & ~1;
    pl.CBW = (k == 3) ? 16 : 8;                  // input channels 128 rows of q can touch
    pl.CBB = (W_BN + k * k - 1) / (k * k) + 1;   // ... and 64 columns
    for (int bmt : {64, 32}) {
        int TW, TN;
        if (Ho * Wo >= bmt) {
            if (bmt % Ho) continue;
            TW = bmt / Ho;
            TN = 1;
            if (Wo % TW) continue;
        } else {
            if (bmt % (Ho * Wo)) continue;
            TW = Wo;
            TN = bmt / (Ho * Wo);
        }
        const int WB = TW + k - 1;
        if (pl.HB > 256 || WB > 256 || TN > 256) continue;
        const int pa = (pl.HB * WB * TN * pl.CBW * 8 + 1023) & ~1023;
        const int pb = (pl.HB * WB * TN * pl.CBB * 8 + 1023) & ~1023;
        const int fixed = 1024 + bmt * 4 + 8 * 8;
        const int stages = (kSmemBudget - fixed) / (pa + pb);
        if (stages < 2) continue;
        pl.BMT = bmt; pl.TW = TW; pl.TN = TN; pl.WB = WB; pl.patchBytesA = pa; pl.patchBytesB = pb;
        pl.stages = std::min(stages, 4);
        pl.smem = pl.stages * (pa + pb) + fixed;
        pl.ok = true;
        break;
    }
    if (!pl.ok) return pl;
    pl.tq = (K + W_BQ - 1) / W_BQ;
    pl.tn = (K + W_BN - 1) / W_BN;
    pl.tiles_total = (int)((M + pl.BMT - 1) / pl.BMT);
    long tiles = 0;  // tiles that touch the lower triangle
    for (int qt = 0; qt < pl.tq; ++qt) tiles += std::min(pl.tn, 2 * qt + 2);
    const double step_us = 8.3 * pl.BMT / 64.0;
    pl.splits = best_split(tiles, pl.tiles_total, 256, 8, step_us, (double)K * K * 8);
    pl.tiles_per_split = (pl.tiles_total + pl.splits - 1) / pl.splits;
    pl.splits = (pl.tiles_total + pl.tiles_per_split - 1) / pl.tiles_per_split;
    return pl;
}

}  // namespace

void conv_tma_init_attributes() {
    FITRE_CUDA(cudaFuncSetAttribute(patch_syrk_tma_kernel<3, 64>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBudget));
    FITRE_CUDA(cudaFuncSetAttribute(patch_syrk_tma_kernel<3, 32>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBudget));
    FITRE_CUDA(cudaFuncSetAttribute(patch_syrk_tma_kernel<5, 64>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBudget));
    FITRE_CUDA(cudaFuncSetAttribute(patch_syrk_tma_kernel<5, 32>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBudget));
    FITRE_CUDA(cudaFuncSetAttribute(wgrad_tma_kernel<3, 64>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBudget));
    FITRE_CUDA(cudaFuncSetAttribute(wgrad_tma_kernel<3, 32>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBudget));
    FITRE_CUDA(cudaFuncSetAttribute(wgrad_tma_kernel<5, 64>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBudget));
    FITRE_CUDA(cudaFuncSetAttribute(wgrad_tma_kernel<5, 32>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBudget));
    FITRE_CUDA(cudaFuncSetAttribute(conv_tma_kernel<3>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                    kSmemBudget));
    FITRE_CUDA(cudaFuncSetAttribute(conv_tma_kernel<5>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                    kSmemBudget));
}

namespace {
// Split-K factor: small grids (late layers with few output positions) are cut along K so that
// about 3.5 waves of CTAs exist; each slice keeps at least 8 K-chunks.
int fprop_split(int N, int Cin, int H, int W, int k, int pad, int Cout, int nseg) {
    const int Ho = H + 2 * pad - k + 1, Wo = W + 2 * pad - k + 1;
    const long M = (long)N * Ho * Wo;
    const long tiles = ((M + T_BM - 1) / T_BM) * ((Cout + T_BN - 1) / T_BN);
    const int cb = chunk_channels(k);
    const int iters = nseg * ((Cin + cb - 1) / cb);
    const double step_us = 4.7 * (cb * k * k) / 36.0;  // one 128 x 64 x (cb k^2) chunk with two CTAs per SM
    return best_split(tiles, iters, 16, 8, step_us, (double)M * Cout * 8);
}
}  // namespace

long conv_fprop_tma_scratch(int N, int Cin, int H, int W, int k, int pad, int Cout) {
    const int Ho = H + 2 * pad - k + 1, Wo = W + 2 * pad - k + 1;
    const int sk = std::max(fprop_split(N, Cin, H, W, k, pad, Cout, 1),
                            fprop_split(N, Cin, H, W, k, pad, Cout, 2));
    return sk > 1 ? (long)sk * N * Ho * Wo * Cout : 0;
}

// Returns false when the shape or the alignment is outside what the TMA kernel handles; the
// caller then uses the gather kernel.  `split_scratch` (conv_fprop_tma_scratch doubles, may be
// NULL) enables split-K.
bool conv_fprop_tma(fitre_context *ctx, int nseg, const ConvSeg *segs, const double *bias,
                    double *y, int N, int Cin, int H, int W, int k, int pad, int Cout,
                    double *split_scratch) {
    if (!encode_fn()) return false;
    if (k != 3 && k != 5) return false;
    const int Ho = H + 2 * pad - k + 1, Wo = W + 2 * pad - k + 1;
    const int K = Cin * k * k;
    if (Ho < 1 || Wo < 1 || (H & 1) || (K & 1)) return false;  // 16-byte global strides
    for (int s = 0; s < nseg; ++s)
        if (((uintptr_t)segs[s].x & 15) || ((uintptr_t)segs[s].w & 15)) return false;
    int TW, TN;
    if (Ho * Wo >= T_BM) {
        if (T_BM % Ho) return false;
        TW = T_BM / Ho;
        TN = 1;
    } else {
        if (T_BM % (Ho * Wo)) return false;
        TW = Wo;
        TN = T_BM / (Ho * Wo);
    }
    TmaConvArgs a{};
    const int padE = pad + (pad & 1);  // start the box on an even x: 16-byte rule of TMA
    a.x0 = -padE;
    a.xoff = padE - pad;
    a.HB = (H + pad + padE + 1) & ~1;
    a.WB = TW + k - 1;
    if (a.HB > 256 || a.WB > 256 || TN > 256) return false;
    const int T_CB = chunk_channels(k);
    const int KCH = (T_CB * k * k + 3) & ~3;
    a.patchBytes = (a.HB * a.WB * TN * T_CB * 8 + 127) & ~127;
    const int stageBytes = a.patchBytes + KCH * T_BN * 8;
    const int fixed = 128 + (((KCH + 3) & ~3) + 4) * 4 + 8 * 8;
    int stages = (kSmemBudget - fixed) / stageBytes;
    if (stages < 2) return false;
    a.stages = std::min(stages, 4);
    a.nchunks = (Cin + T_CB - 1) / T_CB;
    a.nseg = nseg;
    a.N = N; a.Cout = Cout; a.Ho = Ho; a.Wo = Wo; a.pad = pad; a.TW = TW; a.TN = TN;
    a.tilesW = (Wo + TW - 1) / TW;
    a.M = (long)N * Ho * Wo;
    a.bias = bias;
    a.y = y;
    a.err = (int *)(ctx->dscal + 4000);
    for (int s = 0; s < nseg; ++s) {
        cuuint64_t xd[4] = {(cuuint64_t)H, (cuuint64_t)W, (cuuint64_t)N, (cuuint64_t)Cin};
        cuuint64_t xs[3] = {(cuuint64_t)H * 8, (cuuint64_t)H * W * 8, (cuuint64_t)H * W * N * 8};
        cuuint32_t xb[4] = {(cuuint32_t)a.HB, (cuuint32_t)a.WB, (cuuint32_t)TN, (cuuint32_t)T_CB};
        if (!encode(&a.xmap[s], segs[s].x, 4, xd, xs, xb)) return false;
        cuuint64_t wd[2] = {(cuuint64_t)K, (cuuint64_t)Cout};
        cuuint64_t wsb[1] = {(cuuint64_t)K * 8};
        cuuint32_t wb[2] = {(cuuint32_t)KCH, (cuuint32_t)T_BN};
        if (!encode(&a.wmap[s], segs[s].w, 2, wd, wsb, wb)) return false;
    }
    const int tilesN = (N + TN - 1) / TN;
    int SK = split_scratch ? fprop_split(N, Cin, H, W, k, pad, Cout, nseg) : 1;
    const int iters = nseg * a.nchunks;
    a.iters_per_split = (iters + SK - 1) / SK;
    SK = (iters + a.iters_per_split - 1) / a.iters_per_split;
    if (SK > 1) {
        a.y = split_scratch;
        a.bias = nullptr;
    }
    dim3 grid((unsigned)(a.tilesW * tilesN), (unsigned)((Cout + T_BN - 1) / T_BN), (unsigned)SK);
    const int smem = a.stages * stageBytes + fixed;
    {   // the event pair brackets the product kernel alone, not the slab reducer behind it
        ProfScope prof(ctx, PROF_CONV_IGEMM, 2.0 * (double)a.M * K * Cout * nseg);
        if (k == 3)
            conv_tma_kernel<3><<<grid, T_THREADS, smem, ctx->stream>>>(a);
        else
            conv_tma_kernel<5><<<grid, T_THREADS, smem, ctx->stream>>>(a);
        check_launch(ctx, "conv_tma_kernel");
    }
    if (SK > 1) {
        const long n = a.M * Cout;
        const int blocks = (int)std::min<long>((n + 255) / 256, 148 * 8);
        reduce_out_slabs_kernel<<<blocks, 256, 0, ctx->stream>>>(split_scratch, y, a.M, Cout, SK, bias);
        check_launch(ctx, "reduce_out_slabs_kernel");
    }
    return true;
}

long conv_wgrad_tma_scratch(int N, int Cin, int H, int W, int k, int pad, int Cout) {
    const WgradPlan pl = wgrad_plan(N, Cin, H, W, k, pad, Cout);
    if (!pl.ok || pl.splits <= 1) return 0;
    return (long)pl.splits * Cin * k * k * Cout;
}

// dW = sum_seg im2col(x_seg)' * d_seg (segs[i].w is the errors tensor, M x Cout).  Returns
// false when the TMA kernel cannot take the shape; the caller then uses the gather kernel.
bool conv_wgrad_tma(fitre_context *ctx, int nseg, const ConvSeg *segs, double *dw, int N, int Cin,
                    int H, int W, int k, int pad, int Cout, double *partials) {
    const WgradPlan pl = wgrad_plan(N, Cin, H, W, k, pad, Cout);
    if (!pl.ok) return false;
    for (int s = 0; s < nseg; ++s)
        if (((uintptr_t)segs[s].x & 15) || ((uintptr_t)segs[s].w & 15)) return false;
    const int Ho = H + 2 * pad - k + 1, Wo = W + 2 * pad - k + 1;
    TmaWgradArgs a{};
    a.M = (long)N * Ho * Wo;
    a.nseg = nseg; a.N = N; a.K = Cin * k * k; a.Cout = Cout; a.Ho = Ho; a.Wo = Wo; a.pad = pad;
    a.TW = pl.TW; a.TN = pl.TN; a.HB = pl.HB; a.WB = pl.WB; a.xoff = pl.xoff; a.x0 = pl.x0;
    a.CBW = pl.CBW; a.stages = pl.stages; a.tilesW = Wo / pl.TW;
    a.tiles_total = pl.tiles_total; a.tiles_per_split = pl.tiles_per_split;
    a.patchBytes = pl.patchBytes;
    a.out = pl.splits > 1 ? partials : dw;
    a.err = (int *)(ctx->dscal + 4000);
    for (int s = 0; s < nseg; ++s) {
        cuuint64_t xd[4] = {(cuuint64_t)H, (cuuint64_t)W, (cuuint64_t)N, (cuuint64_t)Cin};
        cuuint64_t xs[3] = {(cuuint64_t)H * 8, (cuuint64_t)H * W * 8, (cuuint64_t)H * W * N * 8};
        cuuint32_t xb[4] = {(cuuint32_t)pl.HB, (cuuint32_t)pl.WB, (cuuint32_t)pl.TN, (cuuint32_t)pl.CBW};
        if (!encode(&a.xmap[s], segs[s].x, 4, xd, xs, xb)) return false;
        cuuint64_t dd[2] = {(cuuint64_t)a.M, (cuuint64_t)Cout};
        cuuint64_t ds[1] = {(cuuint64_t)a.M * 8};
        cuuint32_t db[2] = {16u, (cuuint32_t)W_BN};
        if (!encode(&a.dmap[s], segs[s].w, 2, dd, ds, db, CU_TENSOR_MAP_SWIZZLE_128B)) return false;
    }
    dim3 grid(pl.tq, pl.tn, pl.splits);
    {
        ProfScope prof(ctx, PROF_CONV_WGRAD, 2.0 * (double)a.M * a.K * Cout * nseg);
        if (k == 3 && pl.BMT == 64) wgrad_tma_kernel<3, 64><<<grid, T_THREADS, pl.smem, ctx->stream>>>(a);
        else if (k == 3) wgrad_tma_kernel<3, 32><<<grid, T_THREADS, pl.smem, ctx->stream>>>(a);
        else if (pl.BMT == 64) wgrad_tma_kernel<5, 64><<<grid, T_THREADS, pl.smem, ctx->stream>>>(a);
        else wgrad_tma_kernel<5, 32><<<grid, T_THREADS, pl.smem, ctx->stream>>>(a);
        check_launch(ctx, "wgrad_tma_kernel");
    }
    if (pl.splits > 1) {
        const long n = (long)a.K * Cout;
        const int blocks = (int)std::min<long>((n + 255) / 256, 1184);
        reduce_slabs_tma_kernel<<<blocks, 256, 0, ctx->stream>>>(partials, dw, n, pl.splits);
        check_launch(ctx, "reduce_slabs_tma_kernel");
    }
    return true;
}

long conv_patch_syrk_tma_scratch(int N, int Cin, int H, int W, int k, int pad) {
    const SyrkPlan pl = syrk_plan(N, Cin, H, W, k, pad);
    if (!pl.ok) return 0;
    return (long)pl.splits * Cin * k * k * Cin * k * k;
}

// slabs[s] (K x K each, lower triangle valid) = partial sums of im2col(x)' im2col(x); returns the
// number of slabs, or 0 when the TMA kernel cannot take the shape (the caller then gathers).
int conv_patch_syrk_tma(fitre_context *ctx, const double *x, double *slabs, int N, int Cin, int H, int W,
                        int k, int pad) {
    const SyrkPlan pl = syrk_plan(N, Cin, H, W, k, pad);
    if (!pl.ok || ((uintptr_t)x & 15)) return 0;
    const int Ho = H + 2 * pad - k + 1, Wo = W + 2 * pad - k + 1;
    TmaSyrkArgs a{};
    a.M = (long)N * Ho * Wo;
    a.N = N; a.K = Cin * k * k; a.Ho = Ho; a.Wo = Wo; a.pad = pad;
    a.TW = pl.TW; a.TN = pl.TN; a.HB = pl.HB; a.WB = pl.WB; a.xoff = pl.xoff; a.x0 = pl.x0;
    a.CBW = pl.CBW; a.CBB = pl.CBB; a.stages = pl.stages; a.tilesW = Wo / pl.TW;
    a.tiles_total = pl.tiles_total; a.tiles_per_split = pl.tiles_per_split;
    a.patchBytesA = pl.patchBytesA; a.patchBytesB = pl.patchBytesB;
    a.out = slabs;
    a.err = (int *)(ctx->dscal + 4000);
    cuuint64_t xd[4] = {(cuuint64_t)H, (cuuint64_t)W, (cuuint64_t)N, (cuuint64_t)Cin};
    cuuint64_t xs[3] = {(cuuint64_t)H * 8, (cuuint64_t)H * W * 8, (cuuint64_t)H * W * N * 8};
    cuuint32_t xa[4] = {(cuuint32_t)pl.HB, (cuuint32_t)pl.WB, (cuuint32_t)pl.TN, (cuuint32_t)pl.CBW};
    cuuint32_t xb[4] = {(cuuint32_t)pl.HB, (cuuint32_t)pl.WB, (cuuint32_t)pl.TN, (cuuint32_t)pl.CBB};
    if (!encode(&a.amap, x, 4, xd, xs, xa) || !encode(&a.bmap, x, 4, xd, xs, xb)) return 0;
    dim3 grid(pl.tq, pl.tn, pl.splits);
    if (k == 3 && pl.BMT == 64) patch_syrk_tma_kernel<3, 64><<<grid, T_THREADS, pl.smem, ctx->stream>>>(a);
    else if (k == 3) patch_syrk_tma_kernel<3, 32><<<grid, T_THREADS, pl.smem, ctx->stream>>>(a);
    else if (pl.BMT == 64) patch_syrk_tma_kernel<5, 64><<<grid, T_THREADS, pl.smem, ctx->stream>>>(a);
    else patch_syrk_tma_kernel<5, 32><<<grid, T_THREADS, pl.smem, ctx->stream>>>(a);
    check_launch(ctx, "patch_syrk_tma_kernel");
    return pl.splits;
}

}  // namespace fitre
