// Opt-in reduced-precision convolution (forward / data-gradient shape): TF32 operands, FP32
// accumulation on the 5th-generation tensor cores (tcgen05.mma, accumulator in TMEM).
//
// The tensors stay fp64 in HBM (the reference's `real`); precision is reduced only inside the
// product:
//   * warp 0 (one lane) is the TMA producer: per K-chunk of 32 im2col columns it fetches the raw
//     fp64 input patch of the CTA's 128 output positions (same box as the fp64 kernel) and the
//     32 x 64 slab of the weight matrix, which a small pre-pass has rounded to TF32 and which
//     lands in shared memory in the 128-byte-swizzled K-major layout tcgen05 reads;
//   * warps 2-9 expand the patch into the A operand: each thread owns half an output position's row,
//     gathers its 16 im2col values from the patch (rowbase(m) + offset(q)), rounds them to TF32
//     and writes them into the same swizzled K-major layout (fence.proxy.async, then arrive);
//   * warp 1 (one lane) issues tcgen05.mma (M 128, N 64, K 8; four per chunk) and commits each
//     stage back to the producer; the last commit releases the epilogue;
//   * warps 2-9 read the 128 x 64 fp32 accumulator with tcgen05.ld, widen to fp64, add the bias
//     and store (or write a split-K slab).
// X3 = true is the error-compensated variant: every operand is split into a TF32 head and a TF32
// tail (x = hi + lo, about 22 mantissa bits together) and the product is accumulated as
// lo*hi + hi*lo + hi*hi, three tensor-core products per K step.  A single TF32 product carries a
// relative error near 3e-4 per convolution, which batch normalisation and the backward sweep of a
// deep net amplify a hundredfold; the compensated form stays near 1e-6 per convolution.
// Every mbarrier wait is bounded; on a time-out the CTA sets the error word, still frees its
// TMEM columns and returns.  Plain one-CTA launches; every CTA fetches its own tiles.
#include <algorithm>

#include "common.h"
#include "tma_util.cuh"

namespace fitre {
namespace {

constexpr int F_BM = 128, F_BN = 64, F_KC = 32, F_THREADS = 320, F_STAGES_MAX = 4;
constexpr int F_ABYTES = F_BM * F_KC * 4, F_BBYTES = F_BN * F_KC * 4;
constexpr int F_TMEM_COLS = 64;
constexpr int kSmemHalf = 100 * 1024;   // two CTAs per SM
constexpr int kSmemFull = 200 * 1024;   // one CTA per SM

struct alignas(64) Tf32ConvArgs {
    CUtensorMap xmap[2];
    CUtensorMap wmap[2];
    const double *bias;
    double *y;
    int *err;
    long M;
    int nseg, N, Cout, CoutPad, K, Ho, Wo, pad, TW, TN, HB, WB, xoff, x0, CBP, nchunks, stages, tilesW;
    int patchBytes, iters_per_split;
};

__device__ __forceinline__ uint32_t f32_to_tf32(float f) {
    uint32_t r;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(f));
    return r;
}
// shared-memory matrix descriptor: K-major, 128-byte swizzle, 8-row groups 1024 bytes apart
__device__ __forceinline__ uint64_t umma_desc_sw128(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr & 0x3FFFF) >> 4);          // start address
    d |= (uint64_t)1 << 16;                               // leading byte offset (unused here)
    d |= (uint64_t)(1024 >> 4) << 32;                     // stride byte offset
    d |= (uint64_t)1 << 46;                               // descriptor version (sm_100)
    d |= (uint64_t)2 << 61;                               // SWIZZLE_128B
    return d;
}
// instruction descriptor: D fp32, A/B tf32, both K-major, N = 64, M = 128
constexpr uint32_t kIdescTf32 = (1u << 4) | (2u << 7) | (2u << 10) | ((F_BN >> 3) << 17) | ((F_BM >> 4) << 24);

__device__ __forceinline__ void umma_tf32(uint32_t d_tmem, uint64_t a, uint64_t b, uint32_t idesc,
                                          uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a), "l"(b), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar)
                 : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
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

template <int KS, bool X3>
__global__ void __launch_bounds__(F_THREADS, X3 ? 1 : 2)
conv_tf32_kernel(const __grid_constant__ Tf32ConvArgs p) {
    constexpr int KK = KS * KS;
    constexpr int NP = X3 ? 2 : 1;                       // operand parts: head (and tail)
    constexpr int OPBYTES = NP * (F_ABYTES + F_BBYTES);  // A head [A tail] B head [B tail]
    extern __shared__ unsigned char smraw[];
    unsigned char *sm = (unsigned char *)(((uintptr_t)smraw + 1023) & ~(uintptr_t)1023);
    const int stageBytes = OPBYTES + p.patchBytes;   // all multiples of 1024
    unsigned long long *bars = (unsigned long long *)(sm + (size_t)p.stages * stageBytes);
    // bars: [0,4) patch full, [4,8) weights full, [8,12) A ready, [12,16) stage consumed, [16] accumulator
    uint32_t *tmem_slot = (uint32_t *)(bars + 17);
    __shared__ int abort_flag;
    volatile int *vabort = &abort_flag;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int wt = blockIdx.x % p.tilesW, nt = blockIdx.x / p.tilesW;
    const int w0 = wt * p.TW, n0 = nt * p.TN;
    const int c0 = blockIdx.y * F_BN;
    const int it0 = blockIdx.z * p.iters_per_split;
    const int iters = max(0, min(p.nseg * p.nchunks - it0, p.iters_per_split));

    if (tid == 0) {
        abort_flag = 0;
        for (int s = 0; s < p.stages; ++s) {
            mbar_init(smem_u32(bars + s), 1);
            mbar_init(smem_u32(bars + 4 + s), 1);
            mbar_init(smem_u32(bars + 8 + s), 256);
            mbar_init(smem_u32(bars + 12 + s), 1);
        }
        mbar_init(smem_u32(bars + 16), 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                         smem_u32(tmem_slot)), "r"(F_TMEM_COLS)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ---------------- TMA producer ----------------
        if (lane == 0) {
            const uint32_t patchTx = (uint32_t)(p.HB * p.WB * p.TN * p.CBP * 8);
            for (int it = 0; it < iters; ++it) {
                const int s = it % p.stages, fill = it / p.stages;
                if (fill > 0 && !mbar_wait(smem_u32(bars + 12 + s), (uint32_t)((fill - 1) & 1))) {
                    *vabort = 1;
                    break;
                }
                if (*vabort) break;
                const int g = it0 + it, seg = g / p.nchunks, ch = g - seg * p.nchunks;
                unsigned char *st = sm + (size_t)s * stageBytes;
                const uint32_t bp = smem_u32(bars + s), bw = smem_u32(bars + 4 + s);
                mbar_expect_tx(bp, patchTx);
                tma_load_4d(smem_u32(st + OPBYTES), &p.xmap[seg], bp, p.x0, w0 - p.pad, n0,
                            (ch * F_KC) / KK);
                mbar_expect_tx(bw, NP * F_BBYTES);
                // head and tail of the weights are stacked along the channel axis of one map
                for (int part = 0; part < NP; ++part)
                    tma_load_2d(smem_u32(st + NP * F_ABYTES + part * F_BBYTES), &p.wmap[seg], bw, ch * F_KC,
                                c0 + part * p.CoutPad);
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            for (int it = 0; it < iters; ++it) {
                const int s = it % p.stages;
                const uint32_t par = (uint32_t)((it / p.stages) & 1);
                if (*vabort || !mbar_wait(smem_u32(bars + 4 + s), par) ||
                    !mbar_wait(smem_u32(bars + 8 + s), par)) {
                    *vabort = 1;
                    break;
                }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                unsigned char *st = sm + (size_t)s * stageBytes;
                const uint64_t da = umma_desc_sw128(smem_u32(st));
                const uint64_t db = umma_desc_sw128(smem_u32(st + NP * F_ABYTES));
                constexpr uint64_t kATail = F_ABYTES >> 4, kBTail = F_BBYTES >> 4;
#pragma unroll
                for (int k = 0; k < F_KC / 8; ++k) {  // 8 tf32 = 32 bytes = 2 descriptor units per step
                    const uint32_t acc = (it > 0 || k > 0) ? 1u : 0u;
                    if (X3) {
                        umma_tf32(tmem_base, da + kATail + 2 * k, db + 2 * k, kIdescTf32, acc);   // lo * hi
                        umma_tf32(tmem_base, da + 2 * k, db + kBTail + 2 * k, kIdescTf32, 1u);    // hi * lo
                        umma_tf32(tmem_base, da + 2 * k, db + 2 * k, kIdescTf32, 1u);             // hi * hi
                    } else {
                        umma_tf32(tmem_base, da + 2 * k, db + 2 * k, kIdescTf32, acc);
                    }
                }
                umma_commit(smem_u32(bars + 12 + s));
            }
            if (!*vabort) umma_commit(smem_u32(bars + 16));
        }
    } else {
        // ---------------- expanders (A operand) and epilogue: 256 threads, half a row each ----------------
        const int q = warp & 3;                 // TMEM lane quarter this warp may read
        const int hf = (warp - 2) >> 2;         // which half of the chunk's columns / of the 64 channels
        const int ml = q * 32 + lane;           // row of the tile = output position
        const int ho = ml % p.Ho, r = ml / p.Ho;
        const int wl = r % p.TW, nl = r / p.TW;
        const int rowbase = (nl * p.WB + wl) * p.HB + ho + p.xoff;
        const int chanStride = p.TN * p.WB * p.HB;
        const uint32_t a_row = (uint32_t)((ml >> 3) * 1024 + (ml & 7) * 128);
        for (int it = 0; it < iters; ++it) {
            const int s = it % p.stages;
            if (*vabort || !mbar_wait(smem_u32(bars + s), (uint32_t)((it / p.stages) & 1))) {
                *vabort = 1;
                break;
            }
            unsigned char *st = sm + (size_t)s * stageBytes;
            const double *patch = (const double *)(st + OPBYTES) + rowbase;
            const int g = it0 + it, ch = g % p.nchunks;
            const int qq = ch * F_KC;
            const int cbase = qq / KK;           // first channel of the chunk = channel 0 of the patch
            const int q0 = qq + hf * (F_KC / 2); // this thread's first im2col column
            int cc = q0 / KK, rem = q0 - cc * KK;
            cc -= cbase;
            int j = rem / KS, i = rem - j * KS;
#pragma unroll
            for (int grp = 0; grp < F_KC / 8; ++grp) {
                uint32_t v[4], t[4];
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const double x = patch[cc * chanStride + j * p.HB + i];
                    v[e] = f32_to_tf32(__double2float_rn(x));
                    if (X3) t[e] = f32_to_tf32(__double2float_rn(x - (double)__uint_as_float(v[e])));
                    if (++i == KS) {
                        i = 0;
                        if (++j == KS) {
                            j = 0;
                            ++cc;
                        }
                    }
                }
                const uint32_t off = a_row + (uint32_t)(((hf * 4 + grp) ^ (ml & 7)) << 4);
                *reinterpret_cast<uint4 *>(st + off) = make_uint4(v[0], v[1], v[2], v[3]);
                if (X3) *reinterpret_cast<uint4 *>(st + F_ABYTES + off) = make_uint4(t[0], t[1], t[2], t[3]);
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            mbar_arrive(smem_u32(bars + 8 + s));
        }
        // ---------------- epilogue ----------------
        if (!*vabort && iters > 0 && mbar_wait(smem_u32(bars + 16), 0)) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const bool ok = (n0 + nl) < p.N && (w0 + wl) < p.Wo && nl < p.TN;
            const long grow = ok ? ((long)(n0 + nl) * p.Wo + (w0 + wl)) * p.Ho + ho : -1;
            double *y = p.y + (long)blockIdx.z * p.M * p.Cout;
            uint32_t rr[32];
            tmem_ld32(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(hf * 32), rr);
            if (grow >= 0) {
#pragma unroll
                for (int c = 0; c < 32; ++c) {
                    const int col = c0 + hf * 32 + c;
                    if (col < p.Cout)
                        y[(long)col * p.M + grow] =
                            (double)__uint_as_float(rr[c]) + (p.bias ? p.bias[col] : 0.0);
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
                     "r"(F_TMEM_COLS)
                     : "memory");
    }
    if (tid == 0 && abort_flag) atomicExch(p.err, 2);
}

// fp64 weights (K x Cout column-major = K contiguous per channel) -> TF32-rounded fp32 in the same
// element order; with parts == 2 the TF32 tails follow at channel offset CoutPad, and the padding
// channels of both halves are zero.
__global__ void split_weights_tf32_kernel(const double *in, float *out, int K, int Cout, int CoutPad,
                                          int parts) {
    const long n = (long)K * (parts == 2 ? CoutPad : Cout);
    for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < n; i += (long)gridDim.x * blockDim.x) {
        const bool live = i < (long)K * Cout;
        const double w = live ? in[i] : 0.0;
        const float hi = __uint_as_float(f32_to_tf32(__double2float_rn(w)));
        out[i] = hi;
        if (parts == 2)
            out[(long)K * CoutPad + i] = __uint_as_float(f32_to_tf32(__double2float_rn(w - (double)hi)));
    }
}

__global__ void reduce_out_slabs_tf32_kernel(const double *slabs, double *y, long M, int Cout, int SK,
                                             const double *bias) {
    const long n = M * Cout;
    for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < n; i += (long)gridDim.x * blockDim.x) {
        double s = 0.0;
        for (int k = 0; k < SK; ++k) s += slabs[(long)k * n + i];
        if (bias) s += bias[i / M];
        y[i] = s;
    }
}


// =============================================================================================
// Second form, used whenever the input channel count is a multiple of 32: no thread ever touches
// an operand.  A pre-pass rewrites the fp64 input [C][N][W][H] as fp32 planes with the channel
// innermost ([N][W][H][C]; TF32 head and, when compensated, tail), so that for one filter tap and
// 32 consecutive channels the 128 rows of the im2col tile are 128-byte runs of memory: one 4-D
// tiled TMA load (box 32 channels x TH x TW x TN positions, shifted by the tap, halo zero-filled)
// lands them in shared memory already in the 128-byte-swizzled K-major layout tcgen05.mma reads.
// The weight matrix is reordered to the same K order (tap-major) by its own pre-pass.  Warp 0
// issues the TMA loads, warp 1 the MMAs (accumulator 128 x BN fp32 in TMEM), warps 2-5 only run
// the epilogue.
// =============================================================================================
struct alignas(64) Tf32DirectArgs {
    CUtensorMap amap[2][2];   // [segment][head / tail]
    CUtensorMap wmap[2];      // [segment]; the tail rows follow at row CoutPad
    const double *bias;
    double *y;
    int *err;
    long M;
    int nseg, N, Cout, CoutPad, Ho, Wo, pad, k, TH, TW, TN, tilesW, cchunks, nchunks, stages;
    int iters_per_split;
};

constexpr int D_THREADS = 192;

template <int BN, bool X3>
__global__ void __launch_bounds__(D_THREADS, 1)
conv_tf32_direct_kernel(const __grid_constant__ Tf32DirectArgs p) {
    constexpr int NP = X3 ? 2 : 1;
    constexpr int ABYTES = F_BM * F_KC * 4, BBYTES = BN * F_KC * 4;
    constexpr int STAGE = NP * (ABYTES + BBYTES);
    extern __shared__ unsigned char smraw[];
    unsigned char *sm = (unsigned char *)(((uintptr_t)smraw + 1023) & ~(uintptr_t)1023);
    unsigned long long *bars = (unsigned long long *)(sm + (size_t)p.stages * STAGE);
    // bars: [0,8) stage full, [8,16) stage consumed, [16] accumulator complete
    uint32_t *tmem_slot = (uint32_t *)(bars + 17);
    __shared__ int abort_flag;
    volatile int *vabort = &abort_flag;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int wt = blockIdx.x % p.tilesW, nt = blockIdx.x / p.tilesW;
    const int w0 = wt * p.TW, n0 = nt * p.TN;
    const int c0 = blockIdx.y * BN;
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
                         smem_u32(tmem_slot)), "r"(BN)
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
                const int tj = tap / p.k, ti = tap - tj * p.k;   // kernel column, kernel row
                unsigned char *st = sm + (size_t)s * STAGE;
                const uint32_t bar = smem_u32(bars + s);
                mbar_expect_tx(bar, STAGE);
                for (int part = 0; part < NP; ++part) {
                    tma_load_4d(smem_u32(st + part * ABYTES), &p.amap[seg][part], bar, cc * F_KC, ti - p.pad,
                                w0 + tj - p.pad, n0);
                    tma_load_2d(smem_u32(st + NP * ABYTES + part * BBYTES), &p.wmap[seg], bar, ch * F_KC,
                                c0 + part * p.CoutPad);
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t idesc = (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(BN >> 3) << 17) |
                                       ((uint32_t)(F_BM >> 4) << 24);
            constexpr uint64_t kATail = ABYTES >> 4, kBTail = BBYTES >> 4;
            for (int it = 0; it < iters; ++it) {
                const int s = it % p.stages;
                if (*vabort || !mbar_wait(smem_u32(bars + s), (uint32_t)((it / p.stages) & 1))) {
                    *vabort = 1;
                    break;
                }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                unsigned char *st = sm + (size_t)s * STAGE;
                const uint64_t da = umma_desc_sw128(smem_u32(st));
                const uint64_t db = umma_desc_sw128(smem_u32(st + NP * ABYTES));
#pragma unroll
                for (int k = 0; k < F_KC / 8; ++k) {
                    const uint32_t acc = (it > 0 || k > 0) ? 1u : 0u;
                    if (X3) {
                        umma_tf32(tmem_base, da + kATail + 2 * k, db + 2 * k, idesc, acc);
                        umma_tf32(tmem_base, da + 2 * k, db + kBTail + 2 * k, idesc, 1u);
                        umma_tf32(tmem_base, da + 2 * k, db + 2 * k, idesc, 1u);
                    } else {
                        umma_tf32(tmem_base, da + 2 * k, db + 2 * k, idesc, acc);
                    }
                }
                umma_commit(smem_u32(bars + 8 + s));
            }
            if (!*vabort) umma_commit(smem_u32(bars + 16));
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
            for (int cb = 0; cb < BN / 32; ++cb) {
                uint32_t rr[32];
                tmem_ld32(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(cb * 32), rr);
                if (grow >= 0) {
#pragma unroll
                    for (int c = 0; c < 32; ++c) {
                        const int col = c0 + cb * 32 + c;
                        if (col < p.Cout)
                            y[(long)col * p.M + grow] =
                                (double)__uint_as_float(rr[c]) + (p.bias ? p.bias[col] : 0.0);
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
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(BN)
                     : "memory");
    }
    if (tid == 0 && abort_flag) atomicExch(p.err, 2);
}

// in[c][p] fp64 (p = position within the channel plane, contiguous) -> hi[p][c] (and lo[p][c]) fp32,
// TF32-rounded; 32 x 32 tiles through shared memory so that reads and writes both coalesce.
template <bool X3>
__global__ void split_channels_last_kernel(const double *__restrict__ in, float *__restrict__ hi,
                                           float *__restrict__ lo, int C, long P) {
    __shared__ double tile[32][33];
    const long ptiles = (P + 31) / 32;
    const long ntiles = ptiles * (C / 32);
    for (long t = blockIdx.x; t < ntiles; t += gridDim.x) {
        const long pt = t % ptiles;
        const int ct = (int)(t / ptiles);
        const long p0 = pt * 32;
        const int cbase = ct * 32;
        for (int r = threadIdx.y; r < 32; r += blockDim.y) {
            const long pp = p0 + threadIdx.x;
            tile[r][threadIdx.x] = pp < P ? in[(long)(cbase + r) * P + pp] : 0.0;
        }
        __syncthreads();
        for (int r = threadIdx.y; r < 32; r += blockDim.y) {
            const long pp = p0 + r;
            if (pp < P) {
                const double x = tile[threadIdx.x][r];
                const float h = __uint_as_float(f32_to_tf32(__double2float_rn(x)));
                hi[pp * C + cbase + threadIdx.x] = h;
                if (X3) lo[pp * C + cbase + threadIdx.x] = __uint_as_float(f32_to_tf32(__double2float_rn(x - (double)h)));
            }
        }
        __syncthreads();
    }
}

// weights W[cout][c*kk + tap] fp64 -> out[cout][tap*Cin + c] fp32 (TF32 head; tail rows at
// cout + CoutPad when parts == 2; padding rows zero)
__global__ void split_weights_tap_major_kernel(const double *__restrict__ in, float *__restrict__ out, int Cin,
                                               int kk, int Cout, int CoutPad, int parts) {
    const long K = (long)Cin * kk;
    const long n = K * (parts == 2 ? CoutPad : Cout);
    for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < n; i += (long)gridDim.x * blockDim.x) {
        const long co = i / K, q = i - co * K;          // q = tap * Cin + c in the output
        const int tap = (int)(q / Cin), c = (int)(q - (long)tap * Cin);
        const double w = co < Cout ? in[co * K + (long)c * kk + tap] : 0.0;
        const float h = __uint_as_float(f32_to_tf32(__double2float_rn(w)));
        out[i] = h;
        if (parts == 2) out[K * CoutPad + i] = __uint_as_float(f32_to_tf32(__double2float_rn(w - (double)h)));
    }
}


// =============================================================================================
// Weight gradient on the same tensor cores: dW[q, cout] = sum_m patch[m, q] * err[m, cout], a plain
// GEMM whose reduction runs over the output positions m.  Both operands are wanted K-major with m
// contiguous.  The errors [Cout][M] already are (A tile: 2-D box 32 x 128).  The patches are written
// once per call by a pre-pass as an fp32 matrix [K][M] (row q = (channel, tap), TF32 head and, when
// compensated, tail), so the B tile is a 2-D box 32 x BNQ as well and every TMA load is a full
// 128-byte-wide box starting on a 128-byte boundary.  (Reading the taps straight from the image
// would need loads that start at h - 1, which a TMA load cannot: its innermost coordinate must sit
// on a 16-byte boundary.)  The positions are split over blockIdx.z into slabs that a reducer sums in
// fixed order.  Warp roles as in the forward kernel.
// =============================================================================================
struct alignas(64) Tf32WgradArgs {
    CUtensorMap dmap[2][2];   // errors  [segment][head / tail]: (M, Cout)
    CUtensorMap pmap[2][2];   // patches [segment][head / tail]: (M, K)
    double *out;              // slabs (or dW itself when there is one split)
    int *err;
    int nseg, Cout, K, chunks, chunks_per_split, stages;
};

template <int BNQ, bool X3>
__global__ void __launch_bounds__(D_THREADS, 1)
wgrad_tf32_kernel(const __grid_constant__ Tf32WgradArgs p) {
    constexpr int NP = X3 ? 2 : 1;
    constexpr int ABYTES = F_BM * F_KC * 4, BBYTES = BNQ * F_KC * 4;
    constexpr int STAGE = NP * (ABYTES + BBYTES);
    extern __shared__ unsigned char smraw[];
    unsigned char *sm = (unsigned char *)(((uintptr_t)smraw + 1023) & ~(uintptr_t)1023);
    unsigned long long *bars = (unsigned long long *)(sm + (size_t)p.stages * STAGE);
    uint32_t *tmem_slot = (uint32_t *)(bars + 17);
    __shared__ int abort_flag;
    volatile int *vabort = &abort_flag;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int q0 = blockIdx.x * BNQ, co0 = blockIdx.y * F_BM;
    const int g0 = blockIdx.z * p.chunks_per_split;
    const int per_seg = max(0, min(p.chunks - g0, p.chunks_per_split));
    const int iters = per_seg * p.nseg;

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
                         smem_u32(tmem_slot)), "r"(BNQ)
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
                const int seg = it / per_seg, g = g0 + (it - seg * per_seg);
                unsigned char *st = sm + (size_t)s * STAGE;
                const uint32_t bar = smem_u32(bars + s);
                mbar_expect_tx(bar, STAGE);
                for (int part = 0; part < NP; ++part) {
                    tma_load_2d(smem_u32(st + part * ABYTES), &p.dmap[seg][part], bar, g * F_KC, co0);
                    tma_load_2d(smem_u32(st + NP * ABYTES + part * BBYTES), &p.pmap[seg][part], bar, g * F_KC, q0);
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t idesc = (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(BNQ >> 3) << 17) |
                                       ((uint32_t)(F_BM >> 4) << 24);
            constexpr uint64_t kATail = ABYTES >> 4, kBTail = BBYTES >> 4;
            for (int it = 0; it < iters; ++it) {
                const int s = it % p.stages;
                if (*vabort || !mbar_wait(smem_u32(bars + s), (uint32_t)((it / p.stages) & 1))) {
                    *vabort = 1;
                    break;
                }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                unsigned char *st = sm + (size_t)s * STAGE;
                const uint64_t da = umma_desc_sw128(smem_u32(st));
                const uint64_t db = umma_desc_sw128(smem_u32(st + NP * ABYTES));
#pragma unroll
                for (int k = 0; k < F_KC / 8; ++k) {
                    const uint32_t acc = (it > 0 || k > 0) ? 1u : 0u;
                    if (X3) {
                        umma_tf32(tmem_base, da + kATail + 2 * k, db + 2 * k, idesc, acc);
                        umma_tf32(tmem_base, da + 2 * k, db + kBTail + 2 * k, idesc, 1u);
                        umma_tf32(tmem_base, da + 2 * k, db + 2 * k, idesc, 1u);
                    } else {
                        umma_tf32(tmem_base, da + 2 * k, db + 2 * k, idesc, acc);
                    }
                }
                umma_commit(smem_u32(bars + 8 + s));
            }
            if (!*vabort) umma_commit(smem_u32(bars + 16));
        }
    } else {
        const int q = warp & 3;
        const int co = co0 + q * 32 + lane;           // this thread's output channel (tile row)
        if (iters > 0 && mbar_wait(smem_u32(bars + 16), 0) && !*vabort) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            double *out = p.out + (long)blockIdx.z * p.K * p.Cout;
#pragma unroll 1
            for (int cb = 0; cb < BNQ / 32; ++cb) {
                uint32_t rr[32];
                tmem_ld32(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(cb * 32), rr);
                if (co < p.Cout) {
#pragma unroll
                    for (int c = 0; c < 32; ++c) {
                        const int col = q0 + cb * 32 + c;
                        if (col < p.K) out[(long)co * p.K + col] = (double)__uint_as_float(rr[c]);
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
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(BNQ)
                     : "memory");
    }
    if (tid == 0 && abort_flag) atomicExch(p.err, 2);
}

// x fp64 [C][N][W][H] -> patches [K][M] fp32 (row q = c*k*k + j*k + i, column m = (n, wo, ho), the
// reference's im2col indexing, functions/dev_image.cu:20-49), TF32 head (and tail).  blockIdx.y is
// the row q; each thread converts four consecutive positions and stores them as one float4.
template <bool X3>
__global__ void im2col_split_kernel(const double *__restrict__ x, float *__restrict__ hi, float *__restrict__ lo,
                                    int N, int H, int W, int k, int pad, int Ho, int Wo, int M) {
    const int q = blockIdx.y, kk = k * k;
    const int c = q / kk, tap = q - c * kk;
    const int j = tap / k, i = tap - j * k;
    const double *xc = x + (long)c * N * W * H;
    float *hq = hi + (long)q * M, *lq = lo + (long)q * M;
    for (int m4 = (blockIdx.x * blockDim.x + threadIdx.x) * 4; m4 < M; m4 += gridDim.x * blockDim.x * 4) {
        float vh[4], vl[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int m = m4 + e;
            const int ho = m % Ho, t = m / Ho;
            const int wo = t % Wo, n = t / Wo;
            const int h = ho + i - pad, w = wo + j - pad;
            const double v = (m < M && h >= 0 && h < H && w >= 0 && w < W) ? xc[((long)n * W + w) * H + h] : 0.0;
            vh[e] = __uint_as_float(f32_to_tf32(__double2float_rn(v)));
            if (X3) vl[e] = __uint_as_float(f32_to_tf32(__double2float_rn(v - (double)vh[e])));
        }
        // M is a multiple of 4 (checked by the planner), so the four stay inside the row
        *reinterpret_cast<float4 *>(hq + m4) = make_float4(vh[0], vh[1], vh[2], vh[3]);
        if (X3) *reinterpret_cast<float4 *>(lq + m4) = make_float4(vl[0], vl[1], vl[2], vl[3]);
    }
}
// fp64 -> fp32 TF32 head (and tail), same element order
template <bool X3>
__global__ void split_same_layout_kernel(const double *__restrict__ in, float *__restrict__ hi,
                                         float *__restrict__ lo, long n) {
    for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < n; i += (long)gridDim.x * blockDim.x) {
        const double x = in[i];
        const float h = __uint_as_float(f32_to_tf32(__double2float_rn(x)));
        hi[i] = h;
        if (X3) lo[i] = __uint_as_float(f32_to_tf32(__double2float_rn(x - (double)h)));
    }
}
__global__ void sum_slabs_tf32_kernel(const double *slabs, double *out, long n, int S) {
    for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < n; i += (long)gridDim.x * blockDim.x) {
        double s = 0.0;
        for (int k = 0; k < S; ++k) s += slabs[(long)k * n + i];
        out[i] = s;
    }
}

}  // namespace

void conv_tf32_init_attributes() {
    FITRE_CUDA(cudaFuncSetAttribute(conv_tf32_kernel<3, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemFull));
    FITRE_CUDA(cudaFuncSetAttribute(conv_tf32_kernel<5, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemFull));
    FITRE_CUDA(cudaFuncSetAttribute(conv_tf32_kernel<3, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemFull));
    FITRE_CUDA(cudaFuncSetAttribute(conv_tf32_kernel<5, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemFull));
    FITRE_CUDA(cudaFuncSetAttribute(conv_tf32_direct_kernel<64, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemFull));
    FITRE_CUDA(cudaFuncSetAttribute(conv_tf32_direct_kernel<64, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemFull));
    FITRE_CUDA(cudaFuncSetAttribute(conv_tf32_direct_kernel<128, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemFull));
    FITRE_CUDA(cudaFuncSetAttribute(conv_tf32_direct_kernel<128, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemFull));
    FITRE_CUDA(cudaFuncSetAttribute(wgrad_tf32_kernel<64, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemFull));
    FITRE_CUDA(cudaFuncSetAttribute(wgrad_tf32_kernel<64, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemFull));
    FITRE_CUDA(cudaFuncSetAttribute(wgrad_tf32_kernel<128, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemFull));
    FITRE_CUDA(cudaFuncSetAttribute(wgrad_tf32_kernel<128, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemFull));
}

namespace {
int tf32_split_bn(long M, int Cout, int iters, int bn) {
    const long tiles = ((M + F_BM - 1) / F_BM) * ((Cout + bn - 1) / bn);
    if (tiles >= 296) return 1;
    return (int)std::max<long>(1, std::min<long>(std::min<long>((592 + tiles - 1) / tiles, 8), iters / 8));
}
int tf32_split(long M, int Cout, int iters) { return tf32_split_bn(M, Cout, iters, F_BN); }
inline long cout_pad(int Cout) { return ((long)Cout + 127) / 128 * 128; }
inline long up32(long n) { return (n + 31) / 32 * 32; }

struct Tf32Scratch {
    long slabs, weights, inputs, total;   // offsets in doubles
    int sk_max;
};
// split-K slabs (small grids only) | TF32 heads and tails of two weight matrices | fp32
// channels-last heads and tails of two inputs (direct kernel only)
Tf32Scratch tf32_scratch_layout(int N, int Cin, int H, int W, int k, int pad, int Cout) {
    const int Ho = H + 2 * pad - k + 1, Wo = W + 2 * pad - k + 1;
    const long K = (long)Cin * k * k, M = (long)N * Ho * Wo;
    Tf32Scratch L{};
    const int iters = 2 * (int)((K + F_KC - 1) / F_KC);
    L.sk_max = std::max(tf32_split_bn(M, Cout, iters, 64), tf32_split_bn(M, Cout, iters, 128));
    L.slabs = 0;
    L.weights = up32(L.sk_max > 1 ? (long)L.sk_max * M * Cout : 0);
    L.inputs = L.weights + up32(2 * K * cout_pad(Cout));
    L.total = L.inputs + ((Cin % 32 == 0) ? up32(2L * Cin * N * H * W) : 0) + 64;
    return L;
}
}  // namespace

// The reduced-precision modes have no counterpart in the reference, so their staging does not
// come out of the caller's scratch (whose size is the fp64 path's): the context owns one buffer,
// allocated and grown in stream order on first need.
double *staging_workspace(fitre_context *ctx, long doubles) {
    if (doubles > ctx->staging_cap) {
        if (ctx->staging_buf) FITRE_CUDA(cudaFreeAsync(ctx->staging_buf, ctx->stream));
        ctx->staging_buf = nullptr;
        ctx->staging_cap = 0;
        const long cap = doubles + doubles / 8;
        FITRE_CUDA(cudaMallocAsync((void **)&ctx->staging_buf, sizeof(double) * (size_t)cap, ctx->stream));
        ctx->staging_cap = cap;
    }
    return ctx->staging_buf;
}

long conv_fprop_tf32_scratch(int, int, int, int, int, int, int) { return 0; }

namespace {
// The expander-free form; false when the shape does not fit it (the caller then tries the other).
bool conv_fprop_tf32_direct(fitre_context *ctx, int nseg, const ConvSeg *segs, const double *bias, double *y,
                            int N, int Cin, int H, int W, int k, int pad, int Cout) {
    if (Cin % 32 != 0 || k < 1 || k > 7) return false;
    const bool x3 = ctx->precision == FITRE_PRECISION_TF32X3;
    const int parts = x3 ? 2 : 1;
    const int Ho = H + 2 * pad - k + 1, Wo = W + 2 * pad - k + 1;
    if (Ho < 1 || Wo < 1 || Ho > F_BM || F_BM % Ho) return false;
    const int TH = Ho;
    const int TW = std::min(Wo, F_BM / TH);
    if (Wo % TW || F_BM % (TH * TW)) return false;
    const int TN = F_BM / (TH * TW);
    if (TH > 256 || TW > 256 || TN > 256) return false;
    const Tf32Scratch L = tf32_scratch_layout(N, Cin, H, W, k, pad, Cout);
    double *scratch = staging_workspace(ctx, L.total);
    const int BN = (Cout % 128 == 0) ? 128 : 64;
    const int K = Cin * k * k;
    Tf32DirectArgs a{};
    a.nseg = nseg; a.N = N; a.Cout = Cout; a.Ho = Ho; a.Wo = Wo; a.pad = pad; a.k = k;
    a.TH = TH; a.TW = TW; a.TN = TN;
    a.CoutPad = (int)cout_pad(Cout);
    a.tilesW = Wo / TW;
    a.cchunks = Cin / F_KC;
    a.nchunks = k * k * a.cchunks;
    a.M = (long)N * Ho * Wo;
    a.err = (int *)(ctx->dscal + 4000);
    const int stageBytes = parts * (F_BM * F_KC * 4 + BN * F_KC * 4);
    const int fixed = 1024 + 17 * 8 + 16;
    a.stages = std::min((kSmemFull - fixed) / stageBytes, 6);
    if (a.stages < 2) return false;
    const int iters = nseg * a.nchunks;
    int SK = std::min(L.sk_max, tf32_split_bn(a.M, Cout, iters, BN));
    a.iters_per_split = (iters + SK - 1) / SK;
    SK = (iters + a.iters_per_split - 1) / a.iters_per_split;
    double *slabs = scratch + L.slabs;
    a.y = SK > 1 ? slabs : y;
    a.bias = SK > 1 ? nullptr : bias;
    const long P = (long)N * W * H;
    for (int s = 0; s < nseg; ++s) {
        float *ws = (float *)(scratch + L.weights) + (long)s * 2 * K * a.CoutPad;
        const long nw = (long)K * a.CoutPad;
        split_weights_tap_major_kernel<<<(int)std::min<long>((nw + 255) / 256, 1184), 256, 0, ctx->stream>>>(
            segs[s].w, ws, Cin, k * k, Cout, a.CoutPad, parts);
        check_launch(ctx, "split_weights_tap_major_kernel");
        float *xh = (float *)(scratch + L.inputs) + (long)s * 2 * Cin * P, *xl = xh + (long)Cin * P;
        const long ntiles = ((P + 31) / 32) * (Cin / 32);
        const int blocks = (int)std::min<long>(ntiles, 148 * 16);
        if (x3)
            split_channels_last_kernel<true><<<blocks, dim3(32, 8), 0, ctx->stream>>>(segs[s].x, xh, xl, Cin, P);
        else
            split_channels_last_kernel<false><<<blocks, dim3(32, 8), 0, ctx->stream>>>(segs[s].x, xh, xl, Cin, P);
        check_launch(ctx, "split_channels_last_kernel");
        cuuint64_t xd[4] = {(cuuint64_t)Cin, (cuuint64_t)H, (cuuint64_t)W, (cuuint64_t)N};
        cuuint64_t xs[3] = {(cuuint64_t)Cin * 4, (cuuint64_t)H * Cin * 4, (cuuint64_t)W * H * Cin * 4};
        cuuint32_t xb[4] = {(cuuint32_t)F_KC, (cuuint32_t)TH, (cuuint32_t)TW, (cuuint32_t)TN};
        for (int part = 0; part < parts; ++part)
            if (!encode(&a.amap[s][part], part ? xl : xh, 4, xd, xs, xb, CU_TENSOR_MAP_SWIZZLE_128B,
                        CU_TENSOR_MAP_DATA_TYPE_FLOAT32))
                return false;
        cuuint64_t wd[2] = {(cuuint64_t)K, (cuuint64_t)(x3 ? 2 * a.CoutPad : Cout)};
        cuuint64_t wsb[1] = {(cuuint64_t)K * 4};
        cuuint32_t wb[2] = {(cuuint32_t)F_KC, (cuuint32_t)BN};
        if (!encode(&a.wmap[s], ws, 2, wd, wsb, wb, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_DATA_TYPE_FLOAT32))
            return false;
    }
    const int tilesN = (N + TN - 1) / TN;
    dim3 grid((unsigned)(a.tilesW * tilesN), (unsigned)((Cout + BN - 1) / BN), (unsigned)SK);
    const int smem = a.stages * stageBytes + fixed;
    {
        ProfScope prof(ctx, PROF_CONV_IGEMM, 2.0 * (double)a.M * K * Cout * nseg);
        if (BN == 128 && x3)
            conv_tf32_direct_kernel<128, true><<<grid, D_THREADS, smem, ctx->stream>>>(a);
        else if (BN == 128)
            conv_tf32_direct_kernel<128, false><<<grid, D_THREADS, smem, ctx->stream>>>(a);
        else if (x3)
            conv_tf32_direct_kernel<64, true><<<grid, D_THREADS, smem, ctx->stream>>>(a);
        else
            conv_tf32_direct_kernel<64, false><<<grid, D_THREADS, smem, ctx->stream>>>(a);
        check_launch(ctx, "conv_tf32_direct_kernel");
        if (SK > 1) {
            const long n = a.M * Cout;
            reduce_out_slabs_tf32_kernel<<<(int)std::min<long>((n + 255) / 256, 1184), 256, 0, ctx->stream>>>(
                slabs, y, a.M, Cout, SK, bias);
            check_launch(ctx, "reduce_out_slabs_tf32_kernel");
        }
    }
    return true;
}
}  // namespace

bool conv_fprop_tf32(fitre_context *ctx, int nseg, const ConvSeg *segs, const double *bias, double *y,
                     int N, int Cin, int H, int W, int k, int pad, int Cout, double *caller_scratch) {
    (void)caller_scratch;
    if (!encode_fn()) return false;
    for (int s = 0; s < nseg; ++s)
        if ((uintptr_t)segs[s].x & 15) return false;
    if (conv_fprop_tf32_direct(ctx, nseg, segs, bias, y, N, Cin, H, W, k, pad, Cout)) return true;
    if (k != 3 && k != 5) return false;
    const Tf32Scratch L = tf32_scratch_layout(N, Cin, H, W, k, pad, Cout);
    const bool x3 = ctx->precision == FITRE_PRECISION_TF32X3;
    const int parts = x3 ? 2 : 1;
    const int Ho = H + 2 * pad - k + 1, Wo = W + 2 * pad - k + 1;
    const int K = Cin * k * k;
    if (Ho < 1 || Wo < 1 || (H & 1) || (K & 3) || K < F_KC) return false;
    for (int s = 0; s < nseg; ++s)
        if ((uintptr_t)segs[s].x & 15) return false;
    int TW, TN;
    if (Ho * Wo >= F_BM) {
        if (F_BM % Ho) return false;
        TW = F_BM / Ho;
        TN = 1;
    } else {
        if (F_BM % (Ho * Wo)) return false;
        TW = Wo;
        TN = F_BM / (Ho * Wo);
    }
    Tf32ConvArgs a{};
    const int padE = pad + (pad & 1);
    a.x0 = -padE;
    a.xoff = padE - pad;
    a.HB = (H + pad + padE + 1) & ~1;
    a.WB = TW + k - 1;
    a.CBP = (k == 3) ? 5 : 3;  // channels a run of 32 im2col columns can touch
    if (a.HB > 256 || a.WB > 256 || TN > 256) return false;
    a.patchBytes = (a.HB * a.WB * TN * a.CBP * 8 + 1023) & ~1023;
    const int stageBytes = parts * (F_ABYTES + F_BBYTES) + a.patchBytes;
    const int fixed = 1024 + 17 * 8 + 16;
    int stages = x3 ? 0 : (kSmemHalf - fixed) / stageBytes;     // two CTAs per SM when they fit
    if (stages < 2) stages = (kSmemFull - fixed) / stageBytes;  // else one
    if (stages < 2) return false;
    a.stages = std::min(stages, F_STAGES_MAX);
    a.nchunks = (K + F_KC - 1) / F_KC;
    a.nseg = nseg;
    a.N = N; a.Cout = Cout; a.K = K; a.Ho = Ho; a.Wo = Wo; a.pad = pad; a.TW = TW; a.TN = TN;
    a.CoutPad = (int)cout_pad(Cout);
    a.tilesW = (Wo + TW - 1) / TW;
    a.M = (long)N * Ho * Wo;
    a.err = (int *)(ctx->dscal + 4000);
    // split-K for small grids (same rule of thumb as the fp64 kernel, fewer CTAs needed)
    const int iters = nseg * a.nchunks;
    int SK = std::min(L.sk_max, tf32_split(a.M, Cout, iters));   // L.sk_max: what the scratch was sized for
    a.iters_per_split = (iters + SK - 1) / SK;
    SK = (iters + a.iters_per_split - 1) / a.iters_per_split;
    double *scratch = staging_workspace(ctx, L.total);
    double *slabs = scratch + L.slabs;
    float *w32 = (float *)(scratch + L.weights);
    a.y = SK > 1 ? slabs : y;
    a.bias = SK > 1 ? nullptr : bias;
    for (int s = 0; s < nseg; ++s) {
        float *ws = w32 + (long)s * 2 * K * a.CoutPad;
        const long n = (long)K * a.CoutPad;
        split_weights_tf32_kernel<<<(int)std::min<long>((n + 255) / 256, 1184), 256, 0, ctx->stream>>>(
            segs[s].w, ws, K, Cout, a.CoutPad, parts);
        check_launch(ctx, "split_weights_tf32_kernel");
        cuuint64_t xd[4] = {(cuuint64_t)H, (cuuint64_t)W, (cuuint64_t)N, (cuuint64_t)Cin};
        cuuint64_t xs[3] = {(cuuint64_t)H * 8, (cuuint64_t)H * W * 8, (cuuint64_t)H * W * N * 8};
        cuuint32_t xb[4] = {(cuuint32_t)a.HB, (cuuint32_t)a.WB, (cuuint32_t)TN, (cuuint32_t)a.CBP};
        if (!encode(&a.xmap[s], segs[s].x, 4, xd, xs, xb)) return false;
        cuuint64_t wd[2] = {(cuuint64_t)K, (cuuint64_t)(x3 ? 2 * a.CoutPad : Cout)};
        cuuint64_t wsb[1] = {(cuuint64_t)K * 4};
        cuuint32_t wb[2] = {(cuuint32_t)F_KC, (cuuint32_t)F_BN};
        if (!encode(&a.wmap[s], ws, 2, wd, wsb, wb, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_DATA_TYPE_FLOAT32))
            return false;
    }
    const int tilesN = (N + TN - 1) / TN;
    dim3 grid((unsigned)(a.tilesW * tilesN), (unsigned)((Cout + F_BN - 1) / F_BN), (unsigned)SK);
    const int smem = a.stages * stageBytes + fixed;
    {
        ProfScope prof(ctx, PROF_CONV_IGEMM, 2.0 * (double)a.M * K * Cout * nseg);
        if (k == 3 && x3)
            conv_tf32_kernel<3, true><<<grid, F_THREADS, smem, ctx->stream>>>(a);
        else if (k == 3)
            conv_tf32_kernel<3, false><<<grid, F_THREADS, smem, ctx->stream>>>(a);
        else if (x3)
            conv_tf32_kernel<5, true><<<grid, F_THREADS, smem, ctx->stream>>>(a);
        else
            conv_tf32_kernel<5, false><<<grid, F_THREADS, smem, ctx->stream>>>(a);
        check_launch(ctx, "conv_tf32_kernel");
        if (SK > 1) {
            const long n = a.M * Cout;
            reduce_out_slabs_tf32_kernel<<<(int)std::min<long>((n + 255) / 256, 1184), 256, 0, ctx->stream>>>(
                slabs, y, a.M, Cout, SK, bias);
            check_launch(ctx, "reduce_out_slabs_tf32_kernel");
        }
    }
    return true;
}


namespace {
struct WgradTf32Plan {
    bool ok;
    int Ho, Wo, BNQ, S, chunks;
    long M, K, slabs, errs, patches, total;   // scratch offsets in doubles
};
WgradTf32Plan wgrad_tf32_plan(int N, int Cin, int H, int W, int k, int pad, int Cout) {
    WgradTf32Plan P{};
    P.Ho = H + 2 * pad - k + 1;
    P.Wo = W + 2 * pad - k + 1;
    P.K = (long)Cin * k * k;
    P.M = (long)N * P.Ho * P.Wo;
    // row strides of both fp32 matrices are M * 4 bytes and must be multiples of 16
    if (P.Ho < 1 || P.Wo < 1 || P.K % 64 != 0 || P.K > 65535 || (P.M & 3) || P.M < 256 || P.M > (1L << 30)) return P;
    P.BNQ = (P.K % 128 == 0) ? 128 : 64;
    P.chunks = (int)((P.M + F_KC - 1) / F_KC);
    const long tiles = (P.K / P.BNQ) * ((Cout + F_BM - 1) / F_BM);
    P.S = (int)std::max<long>(1, std::min<long>(std::min<long>((2 * 148 + tiles - 1) / tiles, 64), P.chunks / 8));
    P.slabs = 0;
    P.errs = up32(P.S > 1 ? (long)P.S * P.K * Cout : 0);
    P.patches = P.errs + up32(2 * P.M * Cout);        // two segments x head/tail, fp32
    P.total = P.patches + up32(2 * P.K * P.M) + 64;
    P.ok = true;
    return P;
}
}  // namespace

long conv_wgrad_tf32_scratch(int, int, int, int, int, int, int) { return 0; }  // staged in the context's buffer

// dW = sum_seg im2col(x_seg)' * err_seg on the tensor cores; false when the shape does not fit.
bool conv_wgrad_tf32(fitre_context *ctx, int nseg, const ConvSeg *segs, double *dw, int N, int Cin, int H,
                     int W, int k, int pad, int Cout, double *caller_scratch) {
    (void)caller_scratch;
    if (!encode_fn()) return false;
    const WgradTf32Plan P = wgrad_tf32_plan(N, Cin, H, W, k, pad, Cout);
    if (!P.ok) return false;
    double *scratch = staging_workspace(ctx, P.total);
    const bool x3 = ctx->precision == FITRE_PRECISION_TF32X3;
    const int parts = x3 ? 2 : 1;
    Tf32WgradArgs a{};
    a.nseg = nseg; a.Cout = Cout; a.K = (int)P.K;
    a.chunks = P.chunks;
    a.chunks_per_split = (P.chunks + P.S - 1) / P.S;
    const int S = (P.chunks + a.chunks_per_split - 1) / a.chunks_per_split;
    a.err = (int *)(ctx->dscal + 4000);
    a.out = S > 1 ? scratch + P.slabs : dw;
    const int stageBytes = parts * (F_BM * F_KC * 4 + P.BNQ * F_KC * 4);
    const int fixed = 1024 + 17 * 8 + 16;
    a.stages = std::min((kSmemFull - fixed) / stageBytes, 6);
    if (a.stages < 2) return false;
    const long EP = P.M * Cout, PP = P.K * P.M;
    for (int s = 0; s < nseg; ++s) {
        float *eh = (float *)(scratch + P.errs) + (long)s * 2 * EP, *el = eh + EP;
        float *ph = (float *)(scratch + P.patches) + (long)s * 2 * PP, *pl = ph + PP;
        const int be = (int)std::min<long>((EP + 255) / 256, 2368);
        const dim3 gp((unsigned)std::min<long>((P.M / 4 + 255) / 256, 64), (unsigned)P.K);
        if (x3) {
            split_same_layout_kernel<true><<<be, 256, 0, ctx->stream>>>(segs[s].w, eh, el, EP);
            im2col_split_kernel<true><<<gp, 256, 0, ctx->stream>>>(segs[s].x, ph, pl, N, H, W, k, pad, P.Ho, P.Wo, (int)P.M);
        } else {
            split_same_layout_kernel<false><<<be, 256, 0, ctx->stream>>>(segs[s].w, eh, el, EP);
            im2col_split_kernel<false><<<gp, 256, 0, ctx->stream>>>(segs[s].x, ph, pl, N, H, W, k, pad, P.Ho, P.Wo, (int)P.M);
        }
        check_launch(ctx, "im2col_split_kernel");
        cuuint64_t dd[2] = {(cuuint64_t)P.M, (cuuint64_t)Cout};
        cuuint64_t pd[2] = {(cuuint64_t)P.M, (cuuint64_t)P.K};
        cuuint64_t st[1] = {(cuuint64_t)P.M * 4};
        cuuint32_t db[2] = {(cuuint32_t)F_KC, (cuuint32_t)F_BM};
        cuuint32_t pb[2] = {(cuuint32_t)F_KC, (cuuint32_t)P.BNQ};
        for (int part = 0; part < parts; ++part) {
            if (!encode(&a.dmap[s][part], part ? el : eh, 2, dd, st, db, CU_TENSOR_MAP_SWIZZLE_128B,
                        CU_TENSOR_MAP_DATA_TYPE_FLOAT32))
                return false;
            if (!encode(&a.pmap[s][part], part ? pl : ph, 2, pd, st, pb, CU_TENSOR_MAP_SWIZZLE_128B,
                        CU_TENSOR_MAP_DATA_TYPE_FLOAT32))
                return false;
        }
    }
    dim3 grid((unsigned)(P.K / P.BNQ), (unsigned)((Cout + F_BM - 1) / F_BM), (unsigned)S);
    const int smem = a.stages * stageBytes + fixed;
    ProfScope prof(ctx, PROF_CONV_WGRAD, 2.0 * (double)P.M * P.K * Cout * nseg);
    if (P.BNQ == 128 && x3)
        wgrad_tf32_kernel<128, true><<<grid, D_THREADS, smem, ctx->stream>>>(a);
    else if (P.BNQ == 128)
        wgrad_tf32_kernel<128, false><<<grid, D_THREADS, smem, ctx->stream>>>(a);
    else if (x3)
        wgrad_tf32_kernel<64, true><<<grid, D_THREADS, smem, ctx->stream>>>(a);
    else
        wgrad_tf32_kernel<64, false><<<grid, D_THREADS, smem, ctx->stream>>>(a);
    check_launch(ctx, "wgrad_tf32_kernel");
    if (S > 1) {
        const long n = P.K * Cout;
        sum_slabs_tf32_kernel<<<(int)std::min<long>((n + 255) / 256, 1184), 256, 0, ctx->stream>>>(a.out, dw, n, S);
        check_launch(ctx, "sum_slabs_tf32_kernel");
    }
    return true;
}

}  // namespace fitre
