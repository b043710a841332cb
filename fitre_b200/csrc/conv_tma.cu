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
#include <cuda.h>

#include <algorithm>
#include <cstdint>
#include <mutex>

#include "common.h"

namespace fitre {
namespace {

constexpr int T_BM = 128, T_BN = 64, T_CB = 4, T_THREADS = 256;
constexpr int kSmemBudget = 110 * 1024;  // two CTAs per SM

struct alignas(64) TmaConvArgs {
    CUtensorMap xmap[2];
    CUtensorMap wmap[2];
    const double *bias;
    double *y;
    int *err;
    long M;
    int nseg, N, Cout, Ho, Wo, pad, TW, TN, HB, WB, xoff, x0, nchunks, stages, tilesW;
    int patchBytes;
};

__device__ __forceinline__ void dmma884(double &c0, double &c1, double a, double b) {
    asm volatile("mma.sync.aligned.m8n8k4.row.col.f64.f64.f64.f64 {%0,%1}, {%2}, {%3}, {%0,%1};\n"
                 : "+d"(c0), "+d"(c1)
                 : "d"(a), "d"(b));
}
__device__ __forceinline__ uint32_t smem_u32(const void *p) {
    return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
                 : "memory");
}
// Bounded wait: gives up after ~2^31 clock ticks and returns false.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
    const long long t0 = clock64();
    for (;;) {
        uint32_t ok;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(ok)
            : "r"(bar), "r"(parity)
            : "memory");
        if (ok) return true;
        if (clock64() - t0 > (1LL << 31)) return false;
    }
}
__device__ __forceinline__ void tma_load_4d(uint32_t dst, const CUtensorMap *map, uint32_t bar,
                                            int x, int y, int z, int w) {
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes "
        "[%0], [%1, {%3, %4, %5, %6}], [%2];"
        ::"r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y), "r"(z), "r"(w)
        : "memory");
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap *map, uint32_t bar,
                                            int x, int y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes "
        "[%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y)
        : "memory");
}

template <int KS>
__global__ void __launch_bounds__(T_THREADS, 2)
conv_tma_kernel(const __grid_constant__ TmaConvArgs p) {
    constexpr int KCH = T_CB * KS * KS;  // K rows per chunk: 36 (3x3) or 100 (5x5); both = 4 mod 16
    extern __shared__ unsigned char smraw[];
    unsigned char *sm = (unsigned char *)(((uintptr_t)smraw + 127) & ~(uintptr_t)127);
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

    if (tid == 0) {
        abort_flag = 0;
        for (int s = 0; s < p.stages; ++s) mbar_init(smem_u32(bars + s), 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    for (int q = tid; q < KCH; q += T_THREADS) {
        const int cl = q / (KS * KS), rem = q - cl * (KS * KS);
        const int j = rem / KS, i = rem - j * KS;
        colofs[q] = (cl * p.TN * p.WB + j) * p.HB + i;
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

    const int iters = p.nseg * p.nchunks;
    const uint32_t txBytes = (uint32_t)(p.HB * p.WB * p.TN * T_CB * 8 + KCH * T_BN * 8);
    auto issue = [&](int it) {
        const int seg = it / p.nchunks, ch = it - seg * p.nchunks;
        const int s = it % p.stages;
        const uint32_t bar = smem_u32(bars + s);
        unsigned char *dst = sm + (size_t)s * stageBytes;
        mbar_expect_tx(bar, txBytes);
        tma_load_4d(smem_u32(dst), &p.xmap[seg], bar, p.x0, w0 - p.pad, n0, ch * T_CB);
        tma_load_2d(smem_u32(dst + p.patchBytes), &p.wmap[seg], bar, ch * KCH, c0);
    };
    if (tid == 0)
        for (int it = 0; it < p.stages - 1 && it < iters; ++it) issue(it);

    double acc[4][4][2];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j][0] = acc[i][j][1] = 0.0;

    for (int it = 0; it < iters; ++it) {
        const int s = it % p.stages;
        // stage (it-1) % stages was released by the barrier that ended the previous iteration
        if (tid == 0 && it + p.stages - 1 < iters) issue(it + p.stages - 1);
        const bool ready = mbar_wait(smem_u32(bars + s), (uint32_t)((it / p.stages) & 1));
        if (!ready) {
            abort_flag = 1;
        } else {
            const double *patch = (const double *)(sm + (size_t)s * stageBytes);
            const double *Bs = (const double *)(sm + (size_t)s * stageBytes + p.patchBytes) +
                               (warp_n * 32 + lr) * KCH + lc;
#pragma unroll
            for (int k4 = 0; k4 < KCH / 4; ++k4) {
                const int co = colofs[k4 * 4 + lc];
                double fa[4], fb[4];
#pragma unroll
                for (int mi = 0; mi < 4; ++mi) fa[mi] = patch[co + rowbase[mi]];
#pragma unroll
                for (int ni = 0; ni < 4; ++ni) fb[ni] = Bs[ni * 8 * KCH + k4 * 4];
#pragma unroll
                for (int mi = 0; mi < 4; ++mi)
#pragma unroll
                    for (int ni = 0; ni < 4; ++ni)
                        dmma884(acc[mi][ni][0], acc[mi][ni][1], fa[mi], fb[ni]);
            }
        }
        __syncthreads();
        if (abort_flag) {
            if (tid == 0) atomicExch(p.err, 1);
            return;
        }
    }

#pragma unroll
    for (int ni = 0; ni < 4; ++ni)
#pragma unroll
        for (int e = 0; e < 2; ++e) {
            const int col = c0 + warp_n * 32 + ni * 8 + 2 * lc + e;
            if (col >= p.Cout) continue;
            const double bv = p.bias ? p.bias[col] : 0.0;
#pragma unroll
            for (int mi = 0; mi < 4; ++mi)
                if (grow[mi] >= 0) p.y[(long)col * p.M + grow[mi]] = acc[mi][ni][e] + bv;
        }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *,
                                  const cuuint64_t *, const cuuint64_t *, const cuuint32_t *,
                                  const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void *f = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &f, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = (EncodeTiledFn)f;
        cudaGetLastError();
    });
    return fn;
}

bool encode(CUtensorMap *map, const void *base, int rank, const cuuint64_t *dims,
            const cuuint64_t *strides_bytes, const cuuint32_t *box) {
    cuuint32_t estr[4] = {1, 1, 1, 1};
    CUresult r = encode_fn()(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT64, (cuuint32_t)rank, (void *)base, dims,
                             strides_bytes, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                             CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS;
}

}  // namespace

void conv_tma_init_attributes() {
    FITRE_CUDA(cudaFuncSetAttribute(conv_tma_kernel<3>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                    kSmemBudget));
    FITRE_CUDA(cudaFuncSetAttribute(conv_tma_kernel<5>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                    kSmemBudget));
}

// Returns false when the shape or the alignment is outside what the TMA kernel handles; the
// caller then uses the gather kernel.
bool conv_fprop_tma(fitre_context *ctx, int nseg, const ConvSeg *segs, const double *bias,
                    double *y, int N, int Cin, int H, int W, int k, int pad, int Cout) {
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
    const int KCH = T_CB * k * k;
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
    dim3 grid((unsigned)(a.tilesW * tilesN), (unsigned)((Cout + T_BN - 1) / T_BN));
    const int smem = a.stages * stageBytes + fixed;
    ProfScope prof(ctx, PROF_CONV_IGEMM, 2.0 * (double)a.M * K * Cout * nseg);
    if (k == 3)
        conv_tma_kernel<3><<<grid, T_THREADS, smem, ctx->stream>>>(a);
    else
        conv_tma_kernel<5><<<grid, T_THREADS, smem, ctx->stream>>>(a);
    check_launch(ctx, "conv_tma_kernel");
    return true;
}

}  // namespace fitre
