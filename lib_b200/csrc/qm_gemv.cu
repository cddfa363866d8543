// qm_gemv.cu — decode GEMV (1..8 activation rows) over block-quantized weights
// for sm_100a, dequantization fused into the product.
//
// Replaces the reference's one-warp-per-row matvec kernels, which read one
// byte per lane and run a five-step shuffle reduction for every 32-element
// block (nvidia/x/egraph/codegen.go:443-482 q8_0_matvec, :674-735 q2_k_matvec).
//
// Design. At the HBM rate of a B200 a 4.5-bit format delivers about 11.6e12
// weights per second, more than the FP32 pipes can convert and multiply one at
// a time, so the inner product runs on the tensor cores even at one
// activation row:
//   * each lane pulls 16-byte pieces of its rows straight from HBM
//     (ld.global.nc, L1 no-allocate) — 4 lanes per row, 16 rows per warp;
//   * nibbles/bytes become exact small integers in fp16 with one LOP3/PRMT and
//     one half2 FMA per pair (magic-number trick: 0x6400|q == 1024+q);
//     for Q4_K the 6-bit sub-block scale is folded in exactly (sc*q <= 945);
//   * activations are staged once per CTA in shared memory as fp16 hi+lo
//     pairs (x = hi + lo to ~22 bits) in mma-fragment order;
//   * mma.sync.m16n8k16 (A = weights, B = activations) accumulates in fp32;
//     block/super-block scales are applied in fp32 on the accumulators;
//   * the Q4_K minimum term sum_j m_j * sum(x in sub-block j) is one extra mma
//     per super-block against pre-reduced activation sums.
// 8 warps of a CTA split a K range between them; results meet in shared
// memory. Long K with many activation rows is split over CTAs as well, with
// per-split partial sums in global scratch, summed in a fixed order by the
// last CTA to arrive (deterministic, no floating-point atomics).
#include <cuda_fp16.h>
#include <stdint.h>

#include "qm_kernel_args.h"

#define QM_FMT_Q4_0 2
#define QM_FMT_Q8_0 8
#define QM_FMT_Q4_K 12

namespace {

__device__ __forceinline__ uint32_t lop_and_or(uint32_t a, uint32_t mask, uint32_t orv) {
    uint32_t d;
    asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(d) : "r"(a), "r"(mask), "r"(orv));
    return d;
}
__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
    uint32_t d;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(sel));
    return d;
}
__device__ __forceinline__ uint32_t hfma2(uint32_t a, uint32_t b, uint32_t c) {
    uint32_t d;
    asm("fma.rn.f16x2 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}
__device__ __forceinline__ uint32_t hsub2(uint32_t a, uint32_t b) {
    uint32_t d;
    asm("sub.rn.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
    return d;
}
__device__ __forceinline__ uint32_t hmul2(uint32_t a, uint32_t b) {
    uint32_t d;
    asm("mul.rn.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
    return d;
}
__device__ __forceinline__ float h2f_lo(uint32_t h2) {
    return __half2float(__ushort_as_half((unsigned short)(h2 & 0xFFFFu)));
}
__device__ __forceinline__ float h2f_hi(uint32_t h2) {
    return __half2float(__ushort_as_half((unsigned short)(h2 >> 16)));
}
__device__ __forceinline__ uint4 ldg_stream(const void *p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}
// D = A(16x16, row) * B(16x8, col) + C, fp16 inputs, fp32 accumulate.
__device__ __forceinline__ void mma16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                         uint32_t a3, uint32_t b0, uint32_t b1, const float (&c)[4]) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%10,%11,%12,%13};"
        : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(c[0]), "f"(c[1]), "f"(c[2]),
          "f"(c[3]));
}

constexpr uint32_t kMagic = 0x64006400u;   // half2(1024, 1024)
constexpr uint32_t kH1032 = 0x64086408u;   // half2(1032)
constexpr uint32_t kH1152 = 0x64806480u;   // half2(1152)
constexpr uint32_t kHInv16 = 0x2C002C00u;  // half2(1/16)
constexpr uint32_t kHNeg72 = 0xD480D480u;  // half2(-72)
constexpr uint32_t kHNeg1024 = 0xE400E400u;
constexpr uint32_t kHNeg64 = 0xD400D400u;

// ---- per-format raw data of one K unit (256 columns) for a lane's two rows ----
template <int FMT> struct UnitData;
template <> struct UnitData<QM_FMT_Q4_K> {
    uint4 hdr[2];   // d | dmin | 12 scale bytes
    uint4 q[2][2];  // bytes 32t..32t+31 of the 128 quant bytes
};
template <> struct UnitData<QM_FMT_Q4_0> {
    uint4 d[2];     // 8 fp16 block scales
    uint4 q[2][2];  // two 4-block groups, word i = word t of block 4G+i
};
template <> struct UnitData<QM_FMT_Q8_0> {
    uint4 d[2];
    uint4 q[2][4];  // four 2-block groups, word 2*bi+hf = word 4*hf+t of block 2G+bi
};

template <int FMT>
__device__ __forceinline__ void load_unit(UnitData<FMT> &ud, const QmGemvArgs &a, int64_t rowA,
                                          int64_t rowB, int u, int t) {
    const int64_t rows2[2] = {rowA, rowB};
#pragma unroll
    for (int rh = 0; rh < 2; rh++) {
        if constexpr (FMT == QM_FMT_Q4_K) {
            const uint8_t *p = a.wq + (rows2[rh] * a.units + u) * 144;
            ud.hdr[rh] = ldg_stream(p);
            ud.q[rh][0] = ldg_stream(p + 16 + 32 * t);
            ud.q[rh][1] = ldg_stream(p + 32 + 32 * t);
        } else if constexpr (FMT == QM_FMT_Q4_0) {
            const int64_t blk0 = (rows2[rh] * a.units + u) * 8;
            ud.d[rh] = ldg_stream(a.wd + blk0);
            const uint8_t *p = a.wq + blk0 * 16;
            ud.q[rh][0] = ldg_stream(p + 16 * t);
            ud.q[rh][1] = ldg_stream(p + 64 + 16 * t);
        } else {
            const int64_t blk0 = (rows2[rh] * a.units + u) * 8;
            ud.d[rh] = ldg_stream(a.wd + blk0);
            const uint8_t *p = a.wq + blk0 * 32;
#pragma unroll
            for (int G = 0; G < 4; G++) ud.q[rh][G] = ldg_stream(p + 64 * G + 16 * t);
        }
    }
}

__device__ __forceinline__ uint32_t u4w(const uint4 &v, int i) {
    return i == 0 ? v.x : i == 1 ? v.y : i == 2 ? v.z : v.w;
}

// MODE 0: m <= 4, B column n = 2*j + {0: hi, 1: lo} of activation row j.
// MODE 1: m <= 8, two B sets: hi (planes 0..7) and lo (planes 8..15), n = j.
template <int FMT, int MODE>
__device__ __forceinline__ void compute_unit(const UnitData<FMT> &ud, float (&acc)[4],
                                             const uint8_t *xs_plane, const uint8_t *xs_plane_lo,
                                             const uint32_t *xsum_hi, const uint32_t *xsum_lo,
                                             int ul, int t, bool bact) {
    const float zero4[4] = {0.f, 0.f, 0.f, 0.f};
    // B fragments of fragment pair jp: 16 bytes = {b0,b1} of mma 2jp, {b0,b1} of mma 2jp+1
    auto load_b = [&](const uint8_t *plane, int jp) -> uint4 {
        uint4 b = make_uint4(0, 0, 0, 0);
        if (bact) b = *reinterpret_cast<const uint4 *>(plane + ((ul * 8 + jp) * 4 + t) * 16);
        return b;
    };
    if constexpr (FMT == QM_FMT_Q4_K) {
        uint32_t mulLo[2], addLo[2], mulHi[2], addHi[2], mAB[2];
        float d[2], dmin[2];
#pragma unroll
        for (int rh = 0; rh < 2; rh++) {
            d[rh] = h2f_lo(ud.hdr[rh].x);
            dmin[rh] = h2f_hi(ud.hdr[rh].x);
            const uint32_t S0 = ud.hdr[rh].y, S1 = ud.hdr[rh].z, S2 = ud.hdr[rh].w;
            const uint32_t scv = (t < 2) ? (S0 & 0x3F3F3F3Fu)
                                         : ((S2 & 0x0F0F0F0Fu) | ((S0 >> 2) & 0x30303030u));
            const uint32_t mv = (t < 2) ? (S1 & 0x3F3F3F3Fu)
                                        : (((S2 >> 4) & 0x0F0F0F0Fu) | ((S1 >> 2) & 0x30303030u));
            const uint32_t scp = scv >> ((t & 1) * 16), mp = mv >> ((t & 1) * 16);
            const uint32_t scA = hsub2(prmt(scp, 0x64646464u, 0x4040u), kMagic);  // (sc_2t, sc_2t)
            const uint32_t scB = hsub2(prmt(scp, 0x64646464u, 0x4141u), kMagic);  // (sc_2t+1, ..)
            mulLo[rh] = scA;
            addLo[rh] = hmul2(scA, kHNeg1024);
            mulHi[rh] = hmul2(scB, kHInv16);
            addHi[rh] = hmul2(scB, kHNeg64);
            mAB[rh] = hsub2(prmt(mp, 0x64646464u, 0x4140u), kMagic);  // (m_2t, m_2t+1)
        }
        float accQ[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int h = 0; h < 2; h++) {
#pragma unroll
            for (int k = 0; k < 4; k++) {
                const uint32_t wA = u4w(ud.q[0][h], k), wB = u4w(ud.q[1][h], k);
                const uint32_t wA8 = wA >> 8, wB8 = wB >> 8;
                const int jp = h * 4 + k;
                const uint4 b = load_b(xs_plane, jp);
                uint32_t a0 = hfma2(lop_and_or(wA, 0x000F000Fu, kMagic), mulLo[0], addLo[0]);
                uint32_t a1 = hfma2(lop_and_or(wB, 0x000F000Fu, kMagic), mulLo[1], addLo[1]);
                uint32_t a2 = hfma2(lop_and_or(wA8, 0x000F000Fu, kMagic), mulLo[0], addLo[0]);
                uint32_t a3 = hfma2(lop_and_or(wB8, 0x000F000Fu, kMagic), mulLo[1], addLo[1]);
                mma16816(accQ, a0, a1, a2, a3, b.x, b.y, accQ);
                uint32_t c0 = hfma2(lop_and_or(wA, 0x00F000F0u, kMagic), mulHi[0], addHi[0]);
                uint32_t c1 = hfma2(lop_and_or(wB, 0x00F000F0u, kMagic), mulHi[1], addHi[1]);
                uint32_t c2 = hfma2(lop_and_or(wA8, 0x00F000F0u, kMagic), mulHi[0], addHi[0]);
                uint32_t c3 = hfma2(lop_and_or(wB8, 0x00F000F0u, kMagic), mulHi[1], addHi[1]);
                mma16816(accQ, c0, c1, c2, c3, b.z, b.w, accQ);
                if constexpr (MODE == 1) {
                    const uint4 bl = load_b(xs_plane_lo, jp);
                    mma16816(accQ, a0, a1, a2, a3, bl.x, bl.y, accQ);
                    mma16816(accQ, c0, c1, c2, c3, bl.z, bl.w, accQ);
                }
            }
        }
        float accM[4];
        {
            const uint32_t bm = bact ? xsum_hi[t] : 0u;
            mma16816(accM, mAB[0], mAB[1], 0u, 0u, bm, 0u, zero4);
            if constexpr (MODE == 1) {
                const uint32_t bml = bact ? xsum_lo[t] : 0u;
                mma16816(accM, mAB[0], mAB[1], 0u, 0u, bml, 0u, accM);
            }
        }
        acc[0] = fmaf(d[0], accQ[0], acc[0]);
        acc[1] = fmaf(d[0], accQ[1], acc[1]);
        acc[2] = fmaf(d[1], accQ[2], acc[2]);
        acc[3] = fmaf(d[1], accQ[3], acc[3]);
        acc[0] = fmaf(-dmin[0], accM[0], acc[0]);
        acc[1] = fmaf(-dmin[0], accM[1], acc[1]);
        acc[2] = fmaf(-dmin[1], accM[2], acc[2]);
        acc[3] = fmaf(-dmin[1], accM[3], acc[3]);
    } else {
        // Q4_0 / Q8_0: every pair of mmas covers one 32-element block of each
        // row, so the block scale is applied in fp32 on the pair's result.
#pragma unroll
        for (int blk = 0; blk < 8; blk++) {
            uint32_t a0, a1, a2, a3, c0, c1, c2, c3;
            if constexpr (FMT == QM_FMT_Q4_0) {
                const uint32_t wA = u4w(ud.q[0][blk >> 2], blk & 3), wB = u4w(ud.q[1][blk >> 2], blk & 3);
                const uint32_t wA8 = wA >> 8, wB8 = wB >> 8;
                a0 = hsub2(lop_and_or(wA, 0x000F000Fu, kMagic), kH1032);
                a1 = hsub2(lop_and_or(wB, 0x000F000Fu, kMagic), kH1032);
                a2 = hsub2(lop_and_or(wA8, 0x000F000Fu, kMagic), kH1032);
                a3 = hsub2(lop_and_or(wB8, 0x000F000Fu, kMagic), kH1032);
                c0 = hfma2(lop_and_or(wA, 0x00F000F0u, kMagic), kHInv16, kHNeg72);
                c1 = hfma2(lop_and_or(wB, 0x00F000F0u, kMagic), kHInv16, kHNeg72);
                c2 = hfma2(lop_and_or(wA8, 0x00F000F0u, kMagic), kHInv16, kHNeg72);
                c3 = hfma2(lop_and_or(wB8, 0x00F000F0u, kMagic), kHInv16, kHNeg72);
            } else {
                const int G = blk >> 1, bi = blk & 1;
                const uint32_t wA0 = u4w(ud.q[0][G], 2 * bi) ^ 0x80808080u;
                const uint32_t wB0 = u4w(ud.q[1][G], 2 * bi) ^ 0x80808080u;
                const uint32_t wA1 = u4w(ud.q[0][G], 2 * bi + 1) ^ 0x80808080u;
                const uint32_t wB1 = u4w(ud.q[1][G], 2 * bi + 1) ^ 0x80808080u;
                a0 = hsub2(prmt(wA0, 0x64646464u, 0x4240u), kH1152);
                a1 = hsub2(prmt(wB0, 0x64646464u, 0x4240u), kH1152);
                a2 = hsub2(prmt(wA0, 0x64646464u, 0x4341u), kH1152);
                a3 = hsub2(prmt(wB0, 0x64646464u, 0x4341u), kH1152);
                c0 = hsub2(prmt(wA1, 0x64646464u, 0x4240u), kH1152);
                c1 = hsub2(prmt(wB1, 0x64646464u, 0x4240u), kH1152);
                c2 = hsub2(prmt(wA1, 0x64646464u, 0x4341u), kH1152);
                c3 = hsub2(prmt(wB1, 0x64646464u, 0x4341u), kH1152);
            }
            const uint4 b = load_b(xs_plane, blk);
            float tmp[4];
            mma16816(tmp, a0, a1, a2, a3, b.x, b.y, zero4);
            mma16816(tmp, c0, c1, c2, c3, b.z, b.w, tmp);
            if constexpr (MODE == 1) {
                const uint4 bl = load_b(xs_plane_lo, blk);
                mma16816(tmp, a0, a1, a2, a3, bl.x, bl.y, tmp);
                mma16816(tmp, c0, c1, c2, c3, bl.z, bl.w, tmp);
            }
            const uint32_t dwA = u4w(ud.d[0], blk >> 1), dwB = u4w(ud.d[1], blk >> 1);
            const float dA = (blk & 1) ? h2f_hi(dwA) : h2f_lo(dwA);
            const float dB = (blk & 1) ? h2f_hi(dwB) : h2f_lo(dwB);
            acc[0] = fmaf(dA, tmp[0], acc[0]);
            acc[1] = fmaf(dA, tmp[1], acc[1]);
            acc[2] = fmaf(dB, tmp[2], acc[2]);
            acc[3] = fmaf(dB, tmp[3], acc[3]);
        }
    }
}

__device__ __forceinline__ uint32_t pack_h2(float lo, float hi) {
    __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t *>(&h);
}

template <int FMT, int MODE>
__device__ __forceinline__ void gemv_body(const QmGemvArgs &a) {
    extern __shared__ __align__(16) uint8_t smem[];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, t = lane & 3;
    const int T = a.tiles_per_cta;
    const int tile = warp % T, kp = warp / T, nkp = (QM_GEMV_THREADS / 32) / T;
    const int us0 = blockIdx.y * a.units_per_split;
    const int us1 = min(us0 + a.units_per_split, a.units);
    const int nun = us1 - us0;
    // contiguous share of the CTA's K range for this warp
    const int wu0 = us0 + (int)(((int64_t)nun * kp) / nkp);
    const int wu1 = us0 + (int)(((int64_t)nun * (kp + 1)) / nkp);
    const int row0 = (blockIdx.x * T + tile) * QM_GEMV_TILE_ROWS;
    const int64_t rowA = min(row0 + g, a.rows - 1);
    const int64_t rowB = min(row0 + g + 8, a.rows - 1);

    // Activation planes: MODE 0 plane 2j / 2j+1 = hi / lo of activation row j (mma column n);
    // MODE 1 plane j = hi, plane m+j = lo.
    const int NPL = 2 * a.m;
    const int plane_stride = nun * 512 + 64;
    uint8_t *xs = smem;                                                                // [NPL][plane_stride]
    uint32_t *xsum = reinterpret_cast<uint32_t *>(smem + (size_t)NPL * plane_stride);  // [nun][NPL][4]
    float *red = reinterpret_cast<float *>(xsum + (size_t)nun * NPL * 4);              // [8][16][8]
    float *s_scale = red + 8 * 16 * 8;                                                 // [8]
    __shared__ unsigned int s_last;

    // Weights do not depend on the producer of x: start the first loads before
    // waiting for it, and let the next kernel in the stream do the same.
    asm volatile("griddepcontrol.launch_dependents;");
    UnitData<FMT> cur;
    if (wu0 < wu1) load_unit<FMT>(cur, a, rowA, rowB, wu0, t);
    asm volatile("griddepcontrol.wait;" ::: "memory");

    // ---- stage the activations -------------------------------------------------
    const bool norm = (a.xop == 1 || a.xop == 2);
    if (norm) {
        for (int j = 0; j < a.m; j++) {
            float s = 0.f;
            const float *xr = a.x + (int64_t)j * a.ldx;
            const float *x2r = a.x2 ? a.x2 + (int64_t)j * a.ldx : nullptr;
            for (int c = tid * 4; c < a.cols; c += QM_GEMV_THREADS * 4) {
                float4 v = *reinterpret_cast<const float4 *>(xr + c);
                if (a.xop == 2) {
                    const float4 w = *reinterpret_cast<const float4 *>(x2r + c);
                    v.x += w.x; v.y += w.y; v.z += w.z; v.w += w.w;
                }
                s = fmaf(v.x, v.x, s); s = fmaf(v.y, v.y, s);
                s = fmaf(v.z, v.z, s); s = fmaf(v.w, v.w, s);
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
            if (lane == 0) red[warp * 8 + j] = s;
        }
        __syncthreads();
        if (tid < a.m) {
            float s = 0.f;
            for (int w = 0; w < 8; w++) s += red[w * 8 + tid];
            s_scale[tid] = rsqrtf(s / (float)a.cols + a.eps);
        }
        __syncthreads();
    }
    {
        const int groups = nun * 64;
        const int total = groups * a.m;
        for (int idx = tid; idx < total; idx += QM_GEMV_THREADS) {
            const int j = idx / groups;
            const int gi = idx - j * groups;
            const int ul = gi >> 6, cg = gi & 63;
            const int col = (us0 + ul) * QM_K_UNIT + cg * 4;
            float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
            if (col < a.cols) {
                v = *reinterpret_cast<const float4 *>(a.x + (int64_t)j * a.ldx + col);
                if (a.xop == 2) {
                    const float4 w = *reinterpret_cast<const float4 *>(a.x2 + (int64_t)j * a.ldx + col);
                    v.x += w.x; v.y += w.y; v.z += w.z; v.w += w.w;
                } else if (a.xop == 3) {
                    const float4 w = *reinterpret_cast<const float4 *>(a.x2 + (int64_t)j * a.ldx + col);
                    v.x = v.x / (1.f + __expf(-v.x)) * w.x;
                    v.y = v.y / (1.f + __expf(-v.y)) * w.y;
                    v.z = v.z / (1.f + __expf(-v.z)) * w.z;
                    v.w = v.w / (1.f + __expf(-v.w)) * w.w;
                }
                if (norm) {
                    const float sc = s_scale[j];
                    v.x *= sc; v.y *= sc; v.z *= sc; v.w *= sc;
                }
            }
            // fragment order inside a group of four columns: (c0, c2 | c1, c3)
            const uint32_t hA = pack_h2(v.x, v.z), hB = pack_h2(v.y, v.w);
            const uint32_t lA = pack_h2(v.x - h2f_lo(hA), v.z - h2f_hi(hA));
            const uint32_t lB = pack_h2(v.y - h2f_lo(hB), v.w - h2f_hi(hB));
            int jp, tt, hs;
            if constexpr (FMT == QM_FMT_Q4_K) {
                // column bits inside the unit: t(2) | nibble(1) | h(1) | k(2) | e(2)
                tt = cg >> 4; hs = (cg >> 3) & 1; jp = (cg & 7);
            } else {
                // column bits: block(3) | half(1) | t(2) | e(2)
                tt = cg & 3; hs = (cg >> 2) & 1; jp = cg >> 3;
            }
            const int off = ((ul * 8 + jp) * 4 + tt) * 16 + hs * 8;
            const int phi = MODE == 0 ? 2 * j : j, plo = MODE == 0 ? 2 * j + 1 : a.m + j;
            *reinterpret_cast<uint2 *>(xs + (size_t)phi * plane_stride + off) = make_uint2(hA, hB);
            *reinterpret_cast<uint2 *>(xs + (size_t)plo * plane_stride + off) = make_uint2(lA, lB);
            if constexpr (FMT == QM_FMT_Q4_K) {
                // sum of the 32 activations under each sub-block scale
                float s = (v.x + v.y) + (v.z + v.w);
                s += __shfl_xor_sync(0xffffffffu, s, 1);
                s += __shfl_xor_sync(0xffffffffu, s, 2);
                s += __shfl_xor_sync(0xffffffffu, s, 4);
                if ((cg & 7) == 0) {
                    const __half sh = __float2half_rn(s);
                    const __half sl = __float2half_rn(s - __half2float(sh));
                    __half *xh = reinterpret_cast<__half *>(xsum);
                    xh[((size_t)ul * NPL + phi) * 8 + (cg >> 3)] = sh;
                    xh[((size_t)ul * NPL + plo) * 8 + (cg >> 3)] = sl;
                }
            }
        }
    }
    __syncthreads();

    // ---- main loop over this warp's K units ---------------------------------------
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    const bool bact = MODE == 0 ? (g < 2 * a.m) : (g < a.m);
    const uint8_t *plane_hi = xs + (size_t)g * plane_stride;
    const uint8_t *plane_lo = xs + (size_t)(g + a.m) * plane_stride;
    auto run = [&](const UnitData<FMT> &ud, int u) {
        const int ul = u - us0;
        compute_unit<FMT, MODE>(ud, acc, plane_hi, plane_lo, xsum + ((size_t)ul * NPL + g) * 4,
                                xsum + ((size_t)ul * NPL + g + a.m) * 4, ul, t, bact);
    };
    // two register buffers, ping-pong: the next unit's loads are in flight while
    // the current one is multiplied
    for (int u = wu0; u < wu1; u += 2) {
        UnitData<FMT> nxt;
        const bool has1 = u + 1 < wu1;
        if (has1) load_unit<FMT>(nxt, a, rowA, rowB, u + 1, t);
        run(cur, u);
        if (has1) {
            if (u + 2 < wu1) load_unit<FMT>(cur, a, rowA, rowB, u + 2, t);
            run(nxt, u + 1);
        }
    }

    // ---- meet the other warps -------------------------------------------------------
    {
        float *r = red + (size_t)warp * 128;
        *reinterpret_cast<float2 *>(r + g * 8 + 2 * t) = make_float2(acc[0], acc[1]);
        *reinterpret_cast<float2 *>(r + (g + 8) * 8 + 2 * t) = make_float2(acc[2], acc[3]);
    }
    __syncthreads();
    const int nout = T * 16 * a.m;
    const int rbase = blockIdx.x * T * 16;
    for (int o = tid; o < nout; o += QM_GEMV_THREADS) {
        const int r = o & 15, tl = (o >> 4) % T, j = (o >> 4) / T;
        float s = 0.f;
        for (int p = 0; p < nkp; p++) {
            const float *rr = red + (size_t)(p * T + tl) * 128 + r * 8;
            s += MODE == 0 ? (rr[2 * j] + rr[2 * j + 1]) : rr[j];
        }
        const int row = rbase + tl * 16 + r;
        if (a.ksplit == 1) {
            if (row < a.rows) a.y[(int64_t)j * a.ldy + row] = s;
        } else {
            a.partials[((size_t)blockIdx.y * 8 + j) * a.rows_pad + row] = s;
        }
    }
    if (a.ksplit > 1) {
        __threadfence();
        __syncthreads();
        if (tid == 0) {
            const unsigned int old = atomicAdd(a.tickets + blockIdx.x, 1u);
            s_last = (old == (unsigned int)(a.ksplit - 1));
        }
        __syncthreads();
        if (s_last) {
            __threadfence();
            for (int o = tid; o < nout; o += QM_GEMV_THREADS) {
                const int r = o & 15, tl = (o >> 4) % T, j = (o >> 4) / T;
                const int row = rbase + tl * 16 + r;
                float s = 0.f;
                for (int p = 0; p < a.ksplit; p++)
                    s += __ldcg(a.partials + ((size_t)p * 8 + j) * a.rows_pad + row);
                if (row < a.rows) a.y[(int64_t)j * a.ldy + row] = s;
            }
            if (tid == 0) a.tickets[blockIdx.x] = 0u;  // ready for the next launch
        }
    }
}

}  // namespace

#define QM_GEMV_KERNEL(name, FMT, MODE)                                                         \
    extern "C" __global__ void __launch_bounds__(QM_GEMV_THREADS, 2)                            \
        name(const __grid_constant__ QmGemvArgs a) {                                            \
        gemv_body<FMT, MODE>(a);                                                                \
    }

QM_GEMV_KERNEL(qm_gemv_q4k_m4, QM_FMT_Q4_K, 0)
QM_GEMV_KERNEL(qm_gemv_q4k_m8, QM_FMT_Q4_K, 1)
QM_GEMV_KERNEL(qm_gemv_q40_m4, QM_FMT_Q4_0, 0)
QM_GEMV_KERNEL(qm_gemv_q40_m8, QM_FMT_Q4_0, 1)
QM_GEMV_KERNEL(qm_gemv_q80_m4, QM_FMT_Q8_0, 0)
QM_GEMV_KERNEL(qm_gemv_q80_m8, QM_FMT_Q8_0, 1)
