// Opt-in "fp64 from int8 tensor cores" convolution (FITRE_PRECISION_FP64_I8): the forward /
// data-gradient product computed to fp64-class accuracy on the integer tensor cores.
//
// Every operand is brought to fixed point with a power-of-two scale that is constant along the
// reduction index (inputs: one scale per channel, folded into the weights; weights: one scale per
// output channel), and written as six signed base-128 digits:  v = sum_i d_i 128^-i + r,
// |d_i| <= 64, |r| <= 0.5 * 128^-6.  A product of two such numbers is a sum of digit products
// weighted by 128^-(i+j); the integer tensor cores (tcgen05.mma.kind::i8, int32 accumulators in
// TMEM) form sum_k d_i^a d_j^b EXACTLY, one accumulator per weight i+j (pairs with i+j <= 8: 26
// products, 7 accumulators x 64 columns), and the epilogue adds the accumulators in fp64 and
// applies the scales.  Dropped terms are below 128^-8 of full scale and the operands are cut at
// 128^-6 of their channel maximum: about 1e-12 relative to the result for operands whose channel
// maxima are within a few orders of magnitude of their typical size (with 21 products the
// dropped terms alone gave 1e-11 per convolution on VGG-11-BN).  Data flow as in the expander-free TF32 kernel: a pre-pass writes the digit planes
// channels-last ([plane][N][W][H][C] int8) so that one 4-D tiled TMA load per plane, filter tap and
// 64 channels lands a 128-row operand tile in the 64-byte-swizzled K-major layout the MMA reads;
// warp 0 issues TMA, warp 1 the MMAs, warps 2-5 the epilogue.  All waits bounded, TMEM freed on
// every path, plain one-CTA launches.
#include <algorithm>
#include <cmath>

#include "common.h"
#include "tma_util.cuh"

namespace fitre {
namespace {

constexpr int I_BM = 128, I_BN = 64, I_KC = 64, I_S = 6, I_THREADS = 192;
constexpr int I_ABYTES = I_BM * I_KC, I_BBYTES = I_BN * I_KC;
constexpr int I_STAGE = I_S * (I_ABYTES + I_BBYTES);      // 73,728 bytes
constexpr int I_ACC = 7;                                   // accumulators: digit-pair weights 128^-(s+2), s = 0..6
constexpr int I_TMEM_COLS = 512;                           // seven 64-column accumulators (448) -> next power of two
constexpr int kSmemI8 = 222 * 1024;

struct alignas(64) I8ConvArgs {
    CUtensorMap amap[2][I_S];   // [segment][digit plane]: (C, H, W, N) int8
    CUtensorMap wmap[2];        // [segment]: (K, I_S * CoutPad) int8, plane p at row p * CoutPad
    const double *colscale;     // per output channel
    const double *bias;
    double *y;
    int *err;
    long M;
    int nseg, N, Cout, CoutPad, Ho, Wo, pad, k, TH, TW, TN, tilesW, cchunks, nchunks, stages;
    int iters_per_split;
};

// shared-memory matrix descriptor: K-major, 64-byte swizzle, 8-row groups 512 bytes apart
__device__ __forceinline__ uint64_t umma_desc_sw64(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr & 0x3FFFF) >> 4);
    d |= (uint64_t)1 << 16;
    d |= (uint64_t)(512 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)4 << 61;   // SWIZZLE_64B
    return d;
}
// instruction descriptor: D int32, A/B signed int8, both K-major, N = 64, M = 128
constexpr uint32_t kIdescI8 = (2u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(I_BN >> 3) << 17) |
                              ((uint32_t)(I_BM >> 4) << 24);

__device__ __forceinline__ void umma_i8(uint32_t d_tmem, uint64_t a, uint64_t b, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a), "l"(b), "r"(kIdescI8), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void umma_commit_i8(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar)
                 : "memory");
}
__device__ __forceinline__ void tmem_ld32_i8(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]),
          "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]),
          "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]),
          "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

__global__ void __launch_bounds__(I_THREADS, 1) conv_i8_kernel(const __grid_constant__ I8ConvArgs p) {
    extern __shared__ unsigned char smraw[];
    unsigned char *sm = (unsigned char *)(((uintptr_t)smraw + 1023) & ~(uintptr_t)1023);
    unsigned long long *bars = (unsigned long long *)(sm + (size_t)p.stages * I_STAGE);
    // bars: [0,8) stage full, [8,16) stage consumed, [16] accumulators complete
    uint32_t *tmem_slot = (uint32_t *)(bars + 17);
    __shared__ int abort_flag;
    volatile int *vabort = &abort_flag;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int wt = blockIdx.x % p.tilesW, nt = blockIdx.x / p.tilesW;
    const int w0 = wt * p.TW, n0 = nt * p.TN;
    const int c0 = blockIdx.y * I_BN;
    const int it0 = blockIdx.z * p.iters_per_split;
    const int iters = max(0, min(p.nseg * p.nchunks - it0, p.iters_per_split));

    if (tid == 0) {
        abort_flag = 0;
        for (int s = 0; s < p.stages; ++s) {
            mbar_init(smem_u32(bars + s), 1);
            mbar_init(smem_u32(bars + 8 + s), 1);
        }
        mbar_init(smem_u32(bars + 16), 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                         smem_u32(tmem_slot)), "r"(I_TMEM_COLS)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        if (lane == 0) {
            for (int it = 0; it < iters; ++it) {
                const int s = it % p.stages, fill = it / p.stages;
                if (fill > 0 && !mbar_wait(smem_u32(bars + 8 + s), (uint32_t)((fill - 1) & 1))) {
                    *vabort = 1;
                    break;
                }
                if (*vabort) break;
                const int g = it0 + it, seg = g / p.nchunks, ch = g - seg * p.nchunks;
                const int tap = ch / p.cchunks, cc = ch - tap * p.cchunks;
                const int tj = tap / p.k, ti = tap - tj * p.k;
                unsigned char *st = sm + (size_t)s * I_STAGE;
                const uint32_t bar = smem_u32(bars + s);
                mbar_expect_tx(bar, I_STAGE);
                for (int pl = 0; pl < I_S; ++pl) {
                    tma_load_4d(smem_u32(st + pl * I_ABYTES), &p.amap[seg][pl], bar, cc * I_KC, ti - p.pad,
                                w0 + tj - p.pad, n0);
                    tma_load_2d(smem_u32(st + I_S * I_ABYTES + pl * I_BBYTES), &p.wmap[seg], bar, ch * I_KC,
                                c0 + pl * p.CoutPad);
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            for (int it = 0; it < iters; ++it) {
                const int s = it % p.stages;
                if (*vabort || !mbar_wait(smem_u32(bars + s), (uint32_t)((it / p.stages) & 1))) {
                    *vabort = 1;
                    break;
                }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                unsigned char *st = sm + (size_t)s * I_STAGE;
                const uint64_t da = umma_desc_sw64(smem_u32(st));
                const uint64_t db = umma_desc_sw64(smem_u32(st + I_S * I_ABYTES));
#pragma unroll
                for (int ks = 0; ks < I_KC / 32; ++ks) {       // 32 int8 = 32 bytes = 2 descriptor units
#pragma unroll
                    for (int i = 0; i < I_S; ++i)
#pragma unroll
                        for (int j = 0; j < I_S && j + i < I_ACC; ++j)   // digit weights 128^-(i+j+2), i + j <= 6
                            umma_i8(tmem_base + (uint32_t)((i + j) * I_BN),
                                    da + (uint64_t)(i * (I_ABYTES >> 4)) + 2 * ks,
                                    db + (uint64_t)(j * (I_BBYTES >> 4)) + 2 * ks,
                                    (it > 0 || ks > 0 || i > (i + j > I_S - 1 ? i + j - (I_S - 1) : 0)) ? 1u : 0u);
                }
                umma_commit_i8(smem_u32(bars + 8 + s));
            }
            if (!*vabort) umma_commit_i8(smem_u32(bars + 16));
        }
    } else {
        const int q = warp & 3;
        const int ml = q * 32 + lane;
        const int hl = ml % p.TH, r = ml / p.TH;
        const int wl = r % p.TW, nl = r / p.TW;
        if (iters > 0 && mbar_wait(smem_u32(bars + 16), 0) && !*vabort) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const bool ok = (n0 + nl) < p.N && (w0 + wl) < p.Wo && hl < p.Ho;
            const long grow = ok ? ((long)(n0 + nl) * p.Wo + (w0 + wl)) * p.Ho + hl : -1;
            double *y = p.y + (long)blockIdx.z * p.M * p.Cout;
#pragma unroll 1
            for (int cb = 0; cb < I_BN / 32; ++cb) {
                double val[32];
#pragma unroll
                for (int c = 0; c < 32; ++c) val[c] = 0.0;
                double wgt = 1.0 / 16384.0;                     // 128^-2
#pragma unroll 1
                for (int s = 0; s < I_ACC; ++s) {
                    uint32_t rr[32];
                    tmem_ld32_i8(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(s * I_BN + cb * 32), rr);
#pragma unroll
                    for (int c = 0; c < 32; ++c) val[c] += (double)(int)rr[c] * wgt;
                    wgt *= 1.0 / 128.0;
                }
                if (grow >= 0) {
#pragma unroll
                    for (int c = 0; c < 32; ++c) {
                        const int col = c0 + cb * 32 + c;
                        if (col < p.Cout)
                            y[(long)col * p.M + grow] = val[c] * p.colscale[col] + (p.bias ? p.bias[col] : 0.0);
                    }
                }
            }
        } else if (iters > 0) {
            *vabort = 1;
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                     "r"(I_TMEM_COLS)
                     : "memory");
    }
    if (tid == 0 && abort_flag) atomicExch(p.err, 3);
}

// ---- pre-passes ------------------------------------------------------------------------------
// smallest power of two s with |v| / s < 0.5 for all |v| <= mx (1 when mx == 0)
__device__ __forceinline__ double pow2_scale(double mx) {
    if (!(mx > 0.0)) return 1.0;
    int e;
    frexp(mx, &e);                 // mx = f * 2^e, 0.5 <= f < 1
    return ldexp(1.0, e + 1);
}
// six signed base-128 digits of v (|v| < 0.5): v = sum_i d_i 128^-(i+1) + r, |r| <= 0.5 * 128^-6
__device__ __forceinline__ void digits128(double v, signed char (&d)[I_S]) {
    double r = v * 128.0;
#pragma unroll
    for (int i = 0; i < I_S; ++i) {
        const double di = rint(r);
        d[i] = (signed char)(int)di;
        r = (r - di) * 128.0;      // exact: |r - di| <= 0.5 and it only drops leading bits
    }
}

// per-channel maximum magnitude of x [C][P]; out must be zero on entry (bit patterns of non-negative
// doubles order like unsigned integers, so the maximum is an atomicMax and order-independent)
__global__ void channel_absmax_kernel(const double *__restrict__ x, long P, unsigned long long *out) {
    const int c = blockIdx.y;
    const double *xc = x + (long)c * P;
    double m = 0.0;
    for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < P; i += (long)gridDim.x * blockDim.x)
        m = fmax(m, fabs(xc[i]));
    for (int o = 16; o > 0; o >>= 1) m = fmax(m, __shfl_xor_sync(0xffffffffu, m, o));
    if ((threadIdx.x & 31) == 0 && m > 0.0) atomicMax(out + c, (unsigned long long)__double_as_longlong(m));
}

// x [C][P] fp64 -> digit planes [plane][P][C] int8 of x[c][p] / scale(c); 64 channels x 32 positions
// per tile through shared memory, each thread writes two adjacent channels (a warp: 64 bytes)
__global__ void slice_channels_last_kernel(const double *__restrict__ x, const double *__restrict__ chmax,
                                           signed char *__restrict__ planes, int C, long P) {
    __shared__ double tile[64][33];
    const long ptiles = (P + 31) / 32;
    const long ntiles = ptiles * (C / 64);
    for (long t = blockIdx.x; t < ntiles; t += gridDim.x) {
        const long pt = t % ptiles;
        const int cbase = (int)(t / ptiles) * 64;
        const long p0 = pt * 32;
        for (int r = threadIdx.y; r < 64; r += blockDim.y) {
            const long pp = p0 + threadIdx.x;
            tile[r][threadIdx.x] = pp < P ? x[(long)(cbase + r) * P + pp] : 0.0;
        }
        __syncthreads();
        const int ca = 2 * threadIdx.x, cb = ca + 1;
        const double ia = 1.0 / pow2_scale(chmax[cbase + ca]), ib = 1.0 / pow2_scale(chmax[cbase + cb]);
        for (int r = threadIdx.y; r < 32; r += blockDim.y) {
            const long pp = p0 + r;
            if (pp < P) {
                signed char da[I_S], db[I_S];
                digits128(tile[ca][r] * ia, da);
                digits128(tile[cb][r] * ib, db);
#pragma unroll
                for (int pl = 0; pl < I_S; ++pl) {
                    char2 v;
                    v.x = da[pl];
                    v.y = db[pl];
                    *reinterpret_cast<char2 *>(planes + (long)pl * P * C + pp * C + cbase + ca) = v;
                }
            }
        }
        __syncthreads();
    }
}

// One block per output channel n: weights W_seg[n][c*kk + tap] times the input channel scale, brought
// to a common per-n power-of-two scale over all segments, written as digit planes in tap-major K
// order: out_seg[plane][n][tap*Cin + c].  colscale[n] = that scale.  Rows n >= Cout are zero.
struct I8WeightArgs {
    const double *w[2];
    const double *chmax[2];
    signed char *out[2];
    int nseg, Cin, kk, Cout, CoutPad;
};
__global__ void slice_weights_kernel(I8WeightArgs a, double *colscale) {
    const int n = blockIdx.x;
    const long K = (long)a.Cin * a.kk;
    __shared__ double red[256];
    double m = 0.0;
    if (n < a.Cout)
        for (int s = 0; s < a.nseg; ++s)
            for (long q = threadIdx.x; q < K; q += blockDim.x) {
                const int c = (int)(q / a.kk);
                m = fmax(m, fabs(a.w[s][(long)n * K + q]) * pow2_scale(a.chmax[s][c]));
            }
    red[threadIdx.x] = m;
    __syncthreads();
    for (int o = 128; o > 0; o >>= 1) {
        if (threadIdx.x < o) red[threadIdx.x] = fmax(red[threadIdx.x], red[threadIdx.x + o]);
        __syncthreads();
    }
    const double sc = pow2_scale(red[0]);
    if (threadIdx.x == 0 && n < a.Cout) colscale[n] = sc;
    const double inv = 1.0 / sc;
    for (int s = 0; s < a.nseg; ++s)
        for (long q = threadIdx.x; q < K; q += blockDim.x) {   // q = tap * Cin + c in the output
            const int tap = (int)(q / a.Cin), c = (int)(q - (long)tap * a.Cin);
            signed char d[I_S];
            const double v = n < a.Cout ? a.w[s][(long)n * K + (long)c * a.kk + tap] * pow2_scale(a.chmax[s][c]) * inv : 0.0;
            digits128(v, d);
#pragma unroll
            for (int pl = 0; pl < I_S; ++pl) a.out[s][((long)pl * a.CoutPad + n) * K + q] = d[pl];
        }
}

__global__ void reduce_out_slabs_i8_kernel(const double *slabs, double *y, long M, int Cout, int SK,
                                           const double *bias) {
    const long n = M * Cout;
    for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < n; i += (long)gridDim.x * blockDim.x) {
        double s = 0.0;
        for (int k = 0; k < SK; ++k) s += slabs[(long)k * n + i];
        if (bias) s += bias[i / M];
        y[i] = s;
    }
}

// ---- weight gradient ---------------------------------------------------------------------------
// dW[q, cout] = sum_m patch[m, q] * err[m, cout] by the same digit scheme: the errors [Cout][M] with
// one scale per output channel, the patches staged as [K][M] with the scale of their input channel
// (row q = (channel, tap)); both K-major with the positions m contiguous, 64 per chunk.  Positions
// are split over blockIdx.z so that every int32 accumulator stays below 2^31, and the slabs are
// summed in fixed order by the reducer.
struct alignas(64) I8WgradArgs {
    CUtensorMap dmap[2];      // errors  [segment]: (M, I_S * CoutPad), plane p at row p * CoutPad
    CUtensorMap pmap[2];      // patches [segment]: (M, I_S * K), plane p at row p * K
    const double *escale[2];  // per output channel
    const double *chmax[2];   // per input channel
    double *out;
    int *err;
    int nseg, Cout, CoutPad, K, kk, chunks, chunks_per_split, stages;
};

__global__ void __launch_bounds__(I_THREADS, 1) wgrad_i8_kernel(const __grid_constant__ I8WgradArgs p) {
    extern __shared__ unsigned char smraw[];
    unsigned char *sm = (unsigned char *)(((uintptr_t)smraw + 1023) & ~(uintptr_t)1023);
    unsigned long long *bars = (unsigned long long *)(sm + (size_t)p.stages * I_STAGE);
    uint32_t *tmem_slot = (uint32_t *)(bars + 17);
    __shared__ int abort_flag;
    volatile int *vabort = &abort_flag;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int q0 = blockIdx.x * I_BN, co0 = blockIdx.y * I_BM;
    const int g0 = blockIdx.z * p.chunks_per_split;
    const int per_seg = max(0, min(p.chunks - g0, p.chunks_per_split));

    if (tid == 0) {
        abort_flag = 0;
        for (int s = 0; s < p.stages; ++s) {
            mbar_init(smem_u32(bars + s), 1);
            mbar_init(smem_u32(bars + 8 + s), 1);
        }
        mbar_init(smem_u32(bars + 16), 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                         smem_u32(tmem_slot)), "r"(I_TMEM_COLS)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = *tmem_slot;
    double *out = p.out + (long)blockIdx.z * p.nseg * p.K * p.Cout;

    // the segments have different scales, so each is accumulated and written out on its own
    for (int seg = 0; seg < p.nseg; ++seg) {
        const int base_it = seg * per_seg;   // running count of stage uses, for the barrier phases
        if (warp == 0) {
            if (lane == 0) {
                for (int it = 0; it < per_seg; ++it) {
                    const int u = base_it + it, s = u % p.stages, fill = u / p.stages;
                    if (fill > 0 && !mbar_wait(smem_u32(bars + 8 + s), (uint32_t)((fill - 1) & 1))) {
                        *vabort = 1;
                        break;
                    }
                    if (*vabort) break;
                    const int g = g0 + it;
                    unsigned char *st = sm + (size_t)s * I_STAGE;
                    const uint32_t bar = smem_u32(bars + s);
                    mbar_expect_tx(bar, I_STAGE);
                    for (int pl = 0; pl < I_S; ++pl) {
                        tma_load_2d(smem_u32(st + pl * I_ABYTES), &p.dmap[seg], bar, g * I_KC, co0 + pl * p.CoutPad);
                        tma_load_2d(smem_u32(st + I_S * I_ABYTES + pl * I_BBYTES), &p.pmap[seg], bar, g * I_KC,
                                    q0 + pl * p.K);
                    }
                }
            }
        } else if (warp == 1) {
            if (lane == 0) {
                for (int it = 0; it < per_seg; ++it) {
                    const int u = base_it + it, s = u % p.stages;
                    if (*vabort || !mbar_wait(smem_u32(bars + s), (uint32_t)((u / p.stages) & 1))) {
                        *vabort = 1;
                        break;
                    }
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    unsigned char *st = sm + (size_t)s * I_STAGE;
                    const uint64_t da = umma_desc_sw64(smem_u32(st));
                    const uint64_t db = umma_desc_sw64(smem_u32(st + I_S * I_ABYTES));
#pragma unroll
                    for (int ks = 0; ks < I_KC / 32; ++ks) {
#pragma unroll
                        for (int i = 0; i < I_S; ++i)
#pragma unroll
                            for (int j = 0; j < I_S && j + i < I_ACC; ++j)
                                umma_i8(tmem_base + (uint32_t)((i + j) * I_BN),
                                        da + (uint64_t)(i * (I_ABYTES >> 4)) + 2 * ks,
                                        db + (uint64_t)(j * (I_BBYTES >> 4)) + 2 * ks,
                                        (it > 0 || ks > 0 || i > (i + j > I_S - 1 ? i + j - (I_S - 1) : 0)) ? 1u : 0u);
                    }
                    umma_commit_i8(smem_u32(bars + 8 + s));
                }
                if (!*vabort) umma_commit_i8(smem_u32(bars + 16));
            }
        } else {
            const int q = warp & 3;
            const int co = co0 + q * 32 + lane;
            if (per_seg > 0 && mbar_wait(smem_u32(bars + 16), (uint32_t)(seg & 1)) && !*vabort) {
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const double es = co < p.Cout ? p.escale[seg][co] : 0.0;
#pragma unroll 1
                for (int cb = 0; cb < I_BN / 32; ++cb) {
                    double val[32];
#pragma unroll
                    for (int c = 0; c < 32; ++c) val[c] = 0.0;
                    double wgt = 1.0 / 16384.0;
#pragma unroll 1
                    for (int s = 0; s < I_ACC; ++s) {
                        uint32_t rr[32];
                        tmem_ld32_i8(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(s * I_BN + cb * 32), rr);
#pragma unroll
                        for (int c = 0; c < 32; ++c) val[c] += (double)(int)rr[c] * wgt;
                        wgt *= 1.0 / 128.0;
                    }
                    if (co < p.Cout) {
#pragma unroll
                        for (int c = 0; c < 32; ++c) {
                            const int col = q0 + cb * 32 + c;
                            if (col < p.K)
                                out[((long)seg * p.Cout + co) * p.K + col] =
                                    val[c] * es * pow2_scale(p.chmax[seg][col / p.kk]);
                        }
                    }
                }
            } else if (per_seg > 0) {
                *vabort = 1;
            }
        }
        // the accumulators are reused by the next segment only after every epilogue warp has read them
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        __syncthreads();
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                     "r"(I_TMEM_COLS)
                     : "memory");
    }
    if (tid == 0 && abort_flag) atomicExch(p.err, 3);
}

// per-row maximum magnitude of e [rows][M] (one block row per matrix row)
__global__ void row_absmax_kernel(const double *__restrict__ e, long M, unsigned long long *out) {
    const int r = blockIdx.y;
    const double *er = e + (long)r * M;
    double m = 0.0;
    for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < M; i += (long)gridDim.x * blockDim.x)
        m = fmax(m, fabs(er[i]));
    for (int o = 16; o > 0; o >>= 1) m = fmax(m, __shfl_xor_sync(0xffffffffu, m, o));
    if ((threadIdx.x & 31) == 0 && m > 0.0) atomicMax(out + r, (unsigned long long)__double_as_longlong(m));
}
// rowmax -> power-of-two scale in place
__global__ void to_pow2_scale_kernel(double *v, int n) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) v[i] = pow2_scale(v[i]);
}
// e [rows][M] fp64 -> digit planes [plane][rowsPad][M] int8 of e / scale(row); four positions per thread
__global__ void slice_rows_kernel(const double *__restrict__ e, const double *__restrict__ scale,
                                  signed char *__restrict__ planes, int rowsPad, long M) {
    const int r = blockIdx.y;
    const double inv = 1.0 / scale[r];
    const double *er = e + (long)r * M;
    for (long m4 = (blockIdx.x * (long)blockDim.x + threadIdx.x) * 4; m4 < M; m4 += (long)gridDim.x * blockDim.x * 4) {
        signed char d[4][I_S];
#pragma unroll
        for (int t = 0; t < 4; ++t) digits128(er[m4 + t] * inv, d[t]);
#pragma unroll
        for (int pl = 0; pl < I_S; ++pl) {
            char4 v;
            v.x = d[0][pl]; v.y = d[1][pl]; v.z = d[2][pl]; v.w = d[3][pl];
            *reinterpret_cast<char4 *>(planes + ((long)pl * rowsPad + r) * M + m4) = v;
        }
    }
}
// x [C][P] fp64 -> digit planes [plane][C][P] int8 of x / scale(channel), same element order; four
// elements per thread
__global__ void slice_same_layout_kernel(const double *__restrict__ x, const double *__restrict__ chmax,
                                         signed char *__restrict__ planes, int C, long P) {
    const int c = blockIdx.y;
    const double inv = 1.0 / pow2_scale(chmax[c]);
    const double *xc = x + (long)c * P;
    for (long p4 = (blockIdx.x * (long)blockDim.x + threadIdx.x) * 4; p4 < P; p4 += (long)gridDim.x * blockDim.x * 4) {
        signed char d[4][I_S];
#pragma unroll
        for (int t = 0; t < 4; ++t) digits128(p4 + t < P ? xc[p4 + t] * inv : 0.0, d[t]);
#pragma unroll
        for (int pl = 0; pl < I_S; ++pl) {
            char4 v;
            v.x = d[0][pl]; v.y = d[1][pl]; v.z = d[2][pl]; v.w = d[3][pl];
            *reinterpret_cast<char4 *>(planes + ((long)pl * C + c) * P + p4) = v;
        }
    }
}
// digit planes of the input [plane][C][N][W][H] -> patch digit planes [plane][K][M] (row q = c*kk +
// j*k + i, column m = (n, wo, ho), zero outside the image): a byte gather, the digits of an input
// element being the same in all k*k patches it appears in.  blockIdx.y = q; a thread resolves the
// source offsets of sixteen consecutive positions once (walking (ho, wo, n) incrementally) and
// reuses them for all six planes, one 16-byte store per plane.
__global__ void im2col_bytes_kernel(const signed char *__restrict__ xin, signed char *__restrict__ planes,
                                    int C, int N, int H, int W, int k, int pad, int Ho, int Wo, int M, int K) {
    const int q = blockIdx.y, kk = k * k;
    const int c = q / kk, tap = q - c * kk;
    const int j = tap / k, i = tap - j * k;
    const long plane_in = (long)C * N * W * H, plane_out = (long)K * M;
    const signed char *xc = xin + (long)c * N * W * H;
    signed char *out = planes + (long)q * M;
    for (int m16 = (blockIdx.x * blockDim.x + threadIdx.x) * 16; m16 < M; m16 += gridDim.x * blockDim.x * 16) {
        int off[16];
        int ho = m16 % Ho, u = m16 / Ho;
        int wo = u % Wo, n = u / Wo;
#pragma unroll
        for (int t = 0; t < 16; ++t) {
            const int h = ho + i - pad, w = wo + j - pad;
            off[t] = (m16 + t < M && h >= 0 && h < H && w >= 0 && w < W) ? (n * W + w) * H + h : -1;
            if (++ho == Ho) {
                ho = 0;
                if (++wo == Wo) {
                    wo = 0;
                    ++n;
                }
            }
        }
#pragma unroll 1
        for (int pl = 0; pl < I_S; ++pl) {
            const signed char *xp = xc + pl * plane_in;
            alignas(16) signed char v[16];
#pragma unroll
            for (int t = 0; t < 16; ++t) v[t] = off[t] >= 0 ? xp[off[t]] : (signed char)0;
            *reinterpret_cast<int4 *>(out + pl * plane_out + m16) = *reinterpret_cast<const int4 *>(v);
        }
    }
}
// dW = sum over splits and segments of the slabs, fixed order
__global__ void sum_slabs_i8_kernel(const double *slabs, double *out, long n, int S) {
    for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < n; i += (long)gridDim.x * blockDim.x) {
        double s = 0.0;
        for (int k = 0; k < S; ++k) s += slabs[(long)k * n + i];
        out[i] = s;
    }
}

inline long up32(long n) { return (n + 31) / 32 * 32; }
int i8_split(long M, int Cout, int iters) {
    const long tiles = ((M + I_BM - 1) / I_BM) * ((Cout + I_BN - 1) / I_BN);
    if (tiles >= 296) return 1;
    return (int)std::max<long>(1, std::min<long>(std::min<long>((592 + tiles - 1) / tiles, 8), iters / 8));
}

}  // namespace

void conv_i8_init_attributes() {
    FITRE_CUDA(cudaFuncSetAttribute(conv_i8_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemI8));
    FITRE_CUDA(cudaFuncSetAttribute(wgrad_i8_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemI8));
}

double *staging_workspace(fitre_context *ctx, long doubles);   // the context-owned staging buffer (conv_tf32.cu)

// Y = sum_seg im2col(x_seg) * w_seg (+ bias) through int8 digit planes; false when the shape does
// not fit (channel count not a multiple of 64, tile shape), the caller then uses the fp64 kernels.
bool conv_fprop_i8(fitre_context *ctx, int nseg, const ConvSeg *segs, const double *bias, double *y, int N,
                   int Cin, int H, int W, int k, int pad, int Cout) {
    if (!encode_fn() || Cin % I_KC != 0 || k < 1 || k > 7) return false;
    const int Ho = H + 2 * pad - k + 1, Wo = W + 2 * pad - k + 1;
    if (Ho < 1 || Wo < 1 || Ho > I_BM || I_BM % Ho) return false;
    const int TH = Ho;
    const int TW = std::min(Wo, I_BM / TH);
    if (Wo % TW || I_BM % (TH * TW)) return false;
    const int TN = I_BM / (TH * TW);
    if (TH > 256 || TW > 256 || TN > 256) return false;
    const long K = (long)Cin * k * k, M = (long)N * Ho * Wo, P = (long)N * W * H;
    // int32 accumulators: at most 6 digit pairs per accumulator, |digit| <= 64
    if ((double)nseg * K * 6.0 * 4096.0 >= 2147483648.0) return false;
    I8ConvArgs a{};
    a.nseg = nseg; a.N = N; a.Cout = Cout; a.Ho = Ho; a.Wo = Wo; a.pad = pad; a.k = k;
    a.TH = TH; a.TW = TW; a.TN = TN;
    a.CoutPad = (Cout + I_BN - 1) / I_BN * I_BN;
    a.tilesW = Wo / TW;
    a.cchunks = Cin / I_KC;
    a.nchunks = k * k * a.cchunks;
    a.M = M;
    a.err = (int *)(ctx->dscal + 4000);
    const int fixed = 1024 + 17 * 8 + 16;
    a.stages = std::min((kSmemI8 - fixed) / I_STAGE, 6);
    if (a.stages < 2) return false;
    const int iters = nseg * a.nchunks;
    int SK = i8_split(M, Cout, iters);
    a.iters_per_split = (iters + SK - 1) / SK;
    SK = (iters + a.iters_per_split - 1) / a.iters_per_split;
    // workspace (doubles): slabs | column scales | per segment: channel maxima, input planes, weight planes
    const long o_scale = up32(SK > 1 ? (long)SK * M * Cout : 0);
    const long o_seg = o_scale + up32(Cout);
    const long seg_doubles = up32(Cin) + up32((I_S * P * Cin + 7) / 8) + up32((I_S * K * a.CoutPad + 7) / 8);
    double *ws = staging_workspace(ctx, o_seg + 2 * seg_doubles + 64);
    double *slabs = ws, *colscale = ws + o_scale;
    a.colscale = colscale;
    a.y = SK > 1 ? slabs : y;
    a.bias = SK > 1 ? nullptr : bias;
    I8WeightArgs wa{};
    wa.nseg = nseg; wa.Cin = Cin; wa.kk = k * k; wa.Cout = Cout; wa.CoutPad = a.CoutPad;
    for (int s = 0; s < nseg; ++s) {
        if ((uintptr_t)segs[s].x & 15) return false;
        double *chmax = ws + o_seg + (long)s * seg_doubles;
        signed char *xp = (signed char *)(chmax + up32(Cin));
        signed char *wp = xp + up32((I_S * P * Cin + 7) / 8) * 8;
        FITRE_CUDA(cudaMemsetAsync(chmax, 0, sizeof(double) * Cin, ctx->stream));
        channel_absmax_kernel<<<dim3((unsigned)std::min<long>((P + 1023) / 1024, 64), (unsigned)Cin), 256, 0,
                                ctx->stream>>>(segs[s].x, P, (unsigned long long *)chmax);
        check_launch(ctx, "channel_absmax_kernel");
        const long ntiles = ((P + 31) / 32) * (Cin / 64);
        slice_channels_last_kernel<<<(int)std::min<long>(ntiles, 148 * 16), dim3(32, 8), 0, ctx->stream>>>(
            segs[s].x, chmax, xp, Cin, P);
        check_launch(ctx, "slice_channels_last_kernel");
        wa.w[s] = segs[s].w;
        wa.chmax[s] = chmax;
        wa.out[s] = wp;
        cuuint64_t xd[4] = {(cuuint64_t)Cin, (cuuint64_t)H, (cuuint64_t)W, (cuuint64_t)N};
        cuuint64_t xs[3] = {(cuuint64_t)Cin, (cuuint64_t)H * Cin, (cuuint64_t)W * H * Cin};
        cuuint32_t xb[4] = {(cuuint32_t)I_KC, (cuuint32_t)TH, (cuuint32_t)TW, (cuuint32_t)TN};
        for (int pl = 0; pl < I_S; ++pl)
            if (!encode(&a.amap[s][pl], xp + (long)pl * P * Cin, 4, xd, xs, xb, CU_TENSOR_MAP_SWIZZLE_64B,
                        CU_TENSOR_MAP_DATA_TYPE_UINT8))
                return false;
        cuuint64_t wd[2] = {(cuuint64_t)K, (cuuint64_t)I_S * a.CoutPad};
        cuuint64_t wsb[1] = {(cuuint64_t)K};
        cuuint32_t wb[2] = {(cuuint32_t)I_KC, (cuuint32_t)I_BN};
        if (!encode(&a.wmap[s], wp, 2, wd, wsb, wb, CU_TENSOR_MAP_SWIZZLE_64B, CU_TENSOR_MAP_DATA_TYPE_UINT8))
            return false;
    }
    slice_weights_kernel<<<a.CoutPad, 256, 0, ctx->stream>>>(wa, colscale);
    check_launch(ctx, "slice_weights_kernel");
    const int tilesN = (N + TN - 1) / TN;
    dim3 grid((unsigned)(a.tilesW * tilesN), (unsigned)((Cout + I_BN - 1) / I_BN), (unsigned)SK);
    const int smem = a.stages * I_STAGE + fixed;
    {
        ProfScope prof(ctx, PROF_CONV_IGEMM, 2.0 * (double)M * K * Cout * nseg);
        conv_i8_kernel<<<grid, I_THREADS, smem, ctx->stream>>>(a);
        check_launch(ctx, "conv_i8_kernel");
        if (SK > 1) {
            const long n = M * Cout;
            reduce_out_slabs_i8_kernel<<<(int)std::min<long>((n + 255) / 256, 1184), 256, 0, ctx->stream>>>(
                slabs, y, M, Cout, SK, bias);
            check_launch(ctx, "reduce_out_slabs_i8_kernel");
        }
    }
    return true;
}

// dW = sum_seg im2col(x_seg)' * err_seg through int8 digit planes; false when the shape does not fit.
bool conv_wgrad_i8(fitre_context *ctx, int nseg, const ConvSeg *segs, double *dw, int N, int Cin, int H, int W,
                   int k, int pad, int Cout) {
    if (!encode_fn() || k < 1 || k > 7) return false;
    const int Ho = H + 2 * pad - k + 1, Wo = W + 2 * pad - k + 1;
    const long K = (long)Cin * k * k, M = (long)N * Ho * Wo;
    // row strides of both int8 matrices are M bytes and must be multiples of 16
    if (Ho < 1 || Wo < 1 || K % I_BN != 0 || K > 65535 || (M & 15) || M < 256 || M > (1L << 30) ||
        (((long)N * W * H) & 3))
        return false;
    I8WgradArgs a{};
    a.nseg = nseg; a.Cout = Cout; a.K = (int)K; a.kk = k * k;
    a.CoutPad = (Cout + I_BM - 1) / I_BM * I_BM;
    a.chunks = (int)((M + I_KC - 1) / I_KC);
    const long tiles = (K / I_BN) * ((Cout + I_BM - 1) / I_BM);
    // enough splits to fill the GPU, and never more than 2^31 / (6 * 64 * 64) positions per accumulator
    int S = (int)std::max<long>(1, std::min<long>(std::min<long>((2 * 148 + tiles - 1) / tiles, 64), a.chunks / 8));
    S = (int)std::max<long>(S, (M + 65535) / 65536);
    a.chunks_per_split = (a.chunks + S - 1) / S;
    S = (a.chunks + a.chunks_per_split - 1) / a.chunks_per_split;
    a.err = (int *)(ctx->dscal + 4000);
    const int fixed = 1024 + 17 * 8 + 16;
    a.stages = std::min((kSmemI8 - fixed) / I_STAGE, 6);
    if (a.stages < 2) return false;
    // workspace (doubles): slabs (S x nseg) | per segment: error scales, channel maxima, error planes, patch planes
    const long o_seg = up32((long)S * nseg * K * Cout);
    const long e_bytes = (long)I_S * a.CoutPad * M, p_bytes = (long)I_S * K * M;
    const long x_bytes = (long)I_S * Cin * N * W * H;
    const long seg_doubles = up32(a.CoutPad) + up32(Cin) + up32((e_bytes + 7) / 8) + up32((p_bytes + 7) / 8) +
                             up32((x_bytes + 7) / 8);
    double *ws = staging_workspace(ctx, o_seg + 2 * seg_doubles + 64);
    a.out = ws;
    for (int s = 0; s < nseg; ++s) {
        if (((uintptr_t)segs[s].x & 15) || ((uintptr_t)segs[s].w & 15)) return false;
        double *escale = ws + o_seg + (long)s * seg_doubles;
        double *chmax = escale + up32(a.CoutPad);
        signed char *ep = (signed char *)(chmax + up32(Cin));
        signed char *pp = ep + up32((e_bytes + 7) / 8) * 8;
        signed char *xq = pp + up32((p_bytes + 7) / 8) * 8;
        FITRE_CUDA(cudaMemsetAsync(escale, 0, sizeof(double) * (up32(a.CoutPad) + up32(Cin)), ctx->stream));
        const unsigned gx = (unsigned)std::min<long>((M + 1023) / 1024, 64);
        row_absmax_kernel<<<dim3(gx, (unsigned)Cout), 256, 0, ctx->stream>>>(segs[s].w, M, (unsigned long long *)escale);
        check_launch(ctx, "row_absmax_kernel");
        to_pow2_scale_kernel<<<(a.CoutPad + 127) / 128, 128, 0, ctx->stream>>>(escale, a.CoutPad);
        check_launch(ctx, "to_pow2_scale_kernel");
        const long P = (long)N * W * H;
        channel_absmax_kernel<<<dim3((unsigned)std::min<long>((P + 1023) / 1024, 64), (unsigned)Cin), 256, 0,
                                ctx->stream>>>(segs[s].x, P, (unsigned long long *)chmax);
        check_launch(ctx, "channel_absmax_kernel");
        // rows Cout .. CoutPad of the error planes are never written: clear them once
        if (a.CoutPad != Cout) FITRE_CUDA(cudaMemsetAsync(ep, 0, (size_t)e_bytes, ctx->stream));
        slice_rows_kernel<<<dim3((unsigned)std::min<long>((M / 4 + 255) / 256, 64), (unsigned)Cout), 256, 0,
                            ctx->stream>>>(segs[s].w, escale, ep, a.CoutPad, M);
        check_launch(ctx, "slice_rows_kernel");
        slice_same_layout_kernel<<<dim3((unsigned)std::min<long>((P / 4 + 255) / 256, 64), (unsigned)Cin), 256, 0,
                                   ctx->stream>>>(segs[s].x, chmax, xq, Cin, P);
        check_launch(ctx, "slice_same_layout_kernel");
        im2col_bytes_kernel<<<dim3((unsigned)std::min<long>((M / 16 + 127) / 128, 64), (unsigned)K), 128, 0,
                              ctx->stream>>>(xq, pp, Cin, N, H, W, k, pad, Ho, Wo, (int)M, (int)K);
        check_launch(ctx, "im2col_bytes_kernel");
        a.escale[s] = escale;
        a.chmax[s] = chmax;
        cuuint64_t dd[2] = {(cuuint64_t)M, (cuuint64_t)I_S * a.CoutPad};
        cuuint64_t pd[2] = {(cuuint64_t)M, (cuuint64_t)I_S * K};
        cuuint64_t st[1] = {(cuuint64_t)M};
        cuuint32_t db[2] = {(cuuint32_t)I_KC, (cuuint32_t)I_BM};
        cuuint32_t pb[2] = {(cuuint32_t)I_KC, (cuuint32_t)I_BN};
        if (!encode(&a.dmap[s], ep, 2, dd, st, db, CU_TENSOR_MAP_SWIZZLE_64B, CU_TENSOR_MAP_DATA_TYPE_UINT8)) return false;
        if (!encode(&a.pmap[s], pp, 2, pd, st, pb, CU_TENSOR_MAP_SWIZZLE_64B, CU_TENSOR_MAP_DATA_TYPE_UINT8)) return false;
    }
    dim3 grid((unsigned)(K / I_BN), (unsigned)((Cout + I_BM - 1) / I_BM), (unsigned)S);
    const int smem = a.stages * I_STAGE + fixed;
    ProfScope prof(ctx, PROF_CONV_WGRAD, 2.0 * (double)M * K * Cout * nseg);
    wgrad_i8_kernel<<<grid, I_THREADS, smem, ctx->stream>>>(a);
    check_launch(ctx, "wgrad_i8_kernel");
    const long n = K * Cout;
    sum_slabs_i8_kernel<<<(int)std::min<long>((n + 255) / 256, 1184), 256, 0, ctx->stream>>>(ws, dw, n, S * nseg);
    check_launch(ctx, "sum_slabs_i8_kernel");
    return true;
}

}  // namespace fitre
