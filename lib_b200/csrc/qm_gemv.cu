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
//   * every warp streams its own (16-row tile, K range) pieces from HBM into a
//     private shared-memory ring with cp.async.bulk copies that complete on an
//     mbarrier, so the bytes in flight do not depend on registers or occupancy;
//     lanes then read 16-byte pieces of their rows (4 lanes per row);
//   * nibbles/bytes become exact small integers in fp16 with one LOP3/PRMT and
//     one half2 FMA per pair (magic-number trick: 0x6400|q == 1024+q);
//   * activations are staged once per CTA in shared memory as fp16 hi+lo
//     pairs (x = hi + lo to ~22 bits) in mma-fragment order;
//   * mma.sync.m16n8k16 (A = weights, B = activations) accumulates in fp32;
//     block scales are applied in fp32 on the accumulators.
// The grid is one persistent CTA per SM. The (tile, K unit) item space is cut
// into equal contiguous shares, one per warp of the whole grid, so there is no
// tail wave and the activations are staged once per CTA. A tile whose K range
// is shared by several warps (or by several K slices, when the activations of
// the whole K do not fit in shared memory) is finished through per-segment
// partial sums in global scratch, added in a fixed order by the last segment
// to arrive (deterministic, no floating-point atomics).
#include <cuda_fp16.h>
#include <stdint.h>

#include "qm_kernel_args.h"
#include "qm_pipe.cuh"

#define QM_FMT_Q4_0 2
#define QM_FMT_Q8_0 8

using namespace qm;

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
__device__ __forceinline__ float h2f_lo(uint32_t h2) {
    return __half2float(__ushort_as_half((unsigned short)(h2 & 0xFFFFu)));
}
__device__ __forceinline__ float h2f_hi(uint32_t h2) {
    return __half2float(__ushort_as_half((unsigned short)(h2 >> 16)));
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

// ---- per-format raw data of one K unit (256 columns) for a lane's two rows ----
template <int FMT> struct UnitData;
template <> struct UnitData<QM_FMT_Q4_0> {
    uint4 d[2];     // 8 fp16 block scales
    uint4 q[2][2];  // two 4-block groups, word i = word t of block 4G+i
};
template <> struct UnitData<QM_FMT_Q8_0> {
    uint4 d[2];
    uint4 q[2][4];  // four 2-block groups, word 2*bi+hf = word 4*hf+t of block 2G+bi
};

// bytes of one row of one K unit in a stage, and the row strides of a stage
template <int FMT> struct StageGeom;
template <> struct StageGeom<QM_FMT_Q4_0> {
    static constexpr int kQ = 128, kD = 16;
};
template <> struct StageGeom<QM_FMT_Q8_0> {
    static constexpr int kQ = 256, kD = 16;
};

// One K unit of a lane's two rows, read from a landed stage.
template <int FMT>
__device__ __forceinline__ void read_unit(UnitData<FMT> &ud, const uint8_t *stage, int rsq, int rsd, int un,
                                          int g, int t) {
#pragma unroll
    for (int rh = 0; rh < 2; rh++) {
        const uint8_t *row = stage + (g + 8 * rh) * rsq + un * StageGeom<FMT>::kQ;
        ud.d[rh] = *reinterpret_cast<const uint4 *>(stage + 16 * rsq + (g + 8 * rh) * rsd + un * 16);
        if constexpr (FMT == QM_FMT_Q4_0) {
            ud.q[rh][0] = *reinterpret_cast<const uint4 *>(row + 16 * t);
            ud.q[rh][1] = *reinterpret_cast<const uint4 *>(row + 64 + 16 * t);
        } else {
#pragma unroll
            for (int G = 0; G < 4; G++) ud.q[rh][G] = *reinterpret_cast<const uint4 *>(row + 64 * G + 16 * t);
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

__device__ __forceinline__ uint32_t pack_h2(float lo, float hi) {
    __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t *>(&h);
}

template <int FMT, int MODE>
__device__ __forceinline__ void gemv_body(const QmGemvArgs &a) {
    extern __shared__ __align__(128) uint8_t smem[];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, t = lane & 3;
    const int C = a.consumers, D = a.depth, KC = a.kc;
    const int nthreads = C * 32;

    // K slice and share of the (tile, unit) item space of this warp
    const int slice = blockIdx.x / a.ctas_per_slice;
    const int cta_in_slice = blockIdx.x - slice * a.ctas_per_slice;
    const int us0 = slice * a.units_per_slice;
    const int nun = min(a.units_per_slice, a.units - us0);
    // Warps are numbered warp-major over the CTAs of the slice, so that when there are fewer
    // items than warps the busy warps spread over all SMs; surplus warps stay idle. Every busy
    // warp owns at least one item, so a tile's segments are exactly the warps vf..vl below.
    const int64_t I = (int64_t)a.tiles * nun;
    const int64_t Wt = min((int64_t)a.ctas_per_slice * C, I);
    const int64_t v = (int64_t)warp * a.ctas_per_slice + cta_in_slice;
    const int64_t lo = v < Wt ? v * I / Wt : 0, hi = v < Wt ? (v + 1) * I / Wt : 0;

    // shared memory carve-up (the host computes the same sizes)
    const int NPL = 2 * a.m;
    const int plane_stride = a.units_per_slice * 512 + 64;
    uint8_t *xs = smem;                                                                  // [NPL][plane_stride]
    uint32_t *xsum = reinterpret_cast<uint32_t *>(smem + (size_t)NPL * plane_stride);    // [ups][NPL][4]
    float *red = reinterpret_cast<float *>(xsum + (size_t)a.units_per_slice * NPL * 4);  // [32][8]
    float *s_scale = red + 32 * 8;                                                       // [8]
    uint64_t *bars = reinterpret_cast<uint64_t *>(s_scale + 8);                          // [C][D]
    const int rsq = KC * StageGeom<FMT>::kQ + 16;   // odd multiple of 16 bytes: conflict-free row reads
    const int rsd = KC * StageGeom<FMT>::kD + 16;
    const int stage_bytes = (16 * rsq + (StageGeom<FMT>::kD ? 16 * rsd : 0) + 127) & ~127;
    uint8_t *stages = reinterpret_cast<uint8_t *>(
        ((uintptr_t)(bars + (size_t)C * D) + 127) & ~(uintptr_t)127);                    // [C][D][stage_bytes]
    uint8_t *my_stages = stages + (size_t)warp * D * stage_bytes;
    const uint32_t my_bars = smem_u32(bars + (size_t)warp * D);

    asm volatile("griddepcontrol.launch_dependents;");
    if (lane == 0)
        for (int d = 0; d < D; d++) mbar_init(my_bars + 8 * d, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    __syncwarp();

    // chunk cursors: a chunk is up to KC consecutive K units of one tile
    int64_t ii = lo;
    int itile = (int)(lo / nun), iu = (int)(lo - (int64_t)itile * nun), islot = 0;
    auto issue = [&]() {
        const int n = (int)min((int64_t)min(KC, nun - iu), hi - ii);
        const uint32_t bar = my_bars + 8 * islot;
        const uint32_t dst = smem_u32(my_stages + (size_t)islot * stage_bytes);
        if (lane == 0) mbar_expect_tx(bar, (uint32_t)(16 * n * (StageGeom<FMT>::kQ + StageGeom<FMT>::kD)));
        __syncwarp();
        const int r = lane & 15;
        const int64_t row = min(itile * 16 + r, a.rows - 1);
        const int64_t unit = row * a.units + us0 + iu;
        if (lane < 16) {
            bulk_g2s(dst + r * rsq, a.wq + unit * StageGeom<FMT>::kQ, (uint32_t)(n * StageGeom<FMT>::kQ), bar);
        } else if (StageGeom<FMT>::kD) {
            bulk_g2s(dst + 16 * rsq + r * rsd, a.wd + unit * 8, (uint32_t)(n * StageGeom<FMT>::kD), bar);
        }
        ii += n;
        iu += n;
        if (iu == nun) { iu = 0; itile++; }
        islot = islot + 1 == D ? 0 : islot + 1;
    };
    // Weights do not depend on the producer of x: fill the ring before waiting for it.
    for (int d = 0; d < D && ii < hi; d++) issue();
    asm volatile("griddepcontrol.wait;" ::: "memory");

    // ---- stage the activations of this K slice, once per CTA ---------------------------
    const bool norm = (a.xop == 1 || a.xop == 2);
    if (norm) {
        for (int j = 0; j < a.m; j++) {
            float s = 0.f;
            const float *xr = a.x + (int64_t)j * a.ldx;
            const float *x2r = a.x2 ? a.x2 + (int64_t)j * a.ldx : nullptr;
            for (int c = tid * 4; c < a.cols; c += nthreads * 4) {
                float4 v4 = *reinterpret_cast<const float4 *>(xr + c);
                if (a.xop == 2) {
                    const float4 w = *reinterpret_cast<const float4 *>(x2r + c);
                    v4.x += w.x; v4.y += w.y; v4.z += w.z; v4.w += w.w;
                }
                s = fmaf(v4.x, v4.x, s); s = fmaf(v4.y, v4.y, s);
                s = fmaf(v4.z, v4.z, s); s = fmaf(v4.w, v4.w, s);
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
            if (lane == 0) red[warp * 8 + j] = s;
        }
        __syncthreads();
        if (tid < a.m) {
            float s = 0.f;
            for (int w = 0; w < C; w++) s += red[w * 8 + tid];
            s_scale[tid] = rsqrtf(s / (float)a.cols + a.eps);
        }
        __syncthreads();
    }
    {
        const int groups = nun * 64;
        const int total = groups * a.m;
        for (int idx = tid; idx < total; idx += nthreads) {
            const int j = idx / groups;
            const int gi = idx - j * groups;
            const int ul = gi >> 6, cg = gi & 63;
            const int col = (us0 + ul) * QM_K_UNIT + cg * 4;
            float4 v4 = make_float4(0.f, 0.f, 0.f, 0.f);
            if (col < a.cols) {
                v4 = *reinterpret_cast<const float4 *>(a.x + (int64_t)j * a.ldx + col);
                if (a.xop == 2) {
                    const float4 w = *reinterpret_cast<const float4 *>(a.x2 + (int64_t)j * a.ldx + col);
                    v4.x += w.x; v4.y += w.y; v4.z += w.z; v4.w += w.w;
                } else if (a.xop == 3) {
                    const float4 w = *reinterpret_cast<const float4 *>(a.x2 + (int64_t)j * a.ldx + col);
                    v4.x = v4.x / (1.f + __expf(-v4.x)) * w.x;
                    v4.y = v4.y / (1.f + __expf(-v4.y)) * w.y;
                    v4.z = v4.z / (1.f + __expf(-v4.z)) * w.z;
                    v4.w = v4.w / (1.f + __expf(-v4.w)) * w.w;
                }
                if (norm) {
                    const float sc = s_scale[j];
                    v4.x *= sc; v4.y *= sc; v4.z *= sc; v4.w *= sc;
                }
            }
            // fragment order inside a group of four columns: (c0, c2 | c1, c3)
            const uint32_t hA = pack_h2(v4.x, v4.z), hB = pack_h2(v4.y, v4.w);
            const uint32_t lA = pack_h2(v4.x - h2f_lo(hA), v4.z - h2f_hi(hA));
            const uint32_t lB = pack_h2(v4.y - h2f_lo(hB), v4.w - h2f_hi(hB));
            // column bits: block(3) | half(1) | t(2) | e(2)
            const int tt = cg & 3, hs = (cg >> 2) & 1, jp = cg >> 3;
            const int off = ((ul * 8 + jp) * 4 + tt) * 16 + hs * 8;
            const int phi = MODE == 0 ? 2 * j : j, plo = MODE == 0 ? 2 * j + 1 : a.m + j;
            *reinterpret_cast<uint2 *>(xs + (size_t)phi * plane_stride + off) = make_uint2(hA, hB);
            *reinterpret_cast<uint2 *>(xs + (size_t)plo * plane_stride + off) = make_uint2(lA, lB);
        }
    }
    __syncthreads();

    // ---- stream this warp's chunks ----------------------------------------------------------
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    const bool bact = MODE == 0 ? (g < 2 * a.m) : (g < a.m);
    const uint8_t *plane_hi = xs + (size_t)g * plane_stride;
    const uint8_t *plane_lo = xs + (size_t)(g + a.m) * plane_stride;

    // Writes the finished sums of one tile. A tile whose K range is shared with other warps
    // (or other K slices) goes through per-segment partial sums; the last segment to arrive
    // adds them in a fixed order.
    auto flush = [&](int tile) {
        float v0, v1, v2, v3;  // MODE 0: (row g, row g+8) of activation row t; MODE 1: rows x (2t, 2t+1)
        if (MODE == 0) { v0 = acc[0] + acc[1]; v1 = acc[2] + acc[3]; v2 = v3 = 0.f; }
        else { v0 = acc[0]; v1 = acc[1]; v2 = acc[2]; v3 = acc[3]; }
        const int64_t i0 = (int64_t)tile * nun, i1 = i0 + nun - 1;
        const int64_t vf = ((i0 + 1) * Wt - 1) / I, vl = ((i1 + 1) * Wt - 1) / I;
        if (a.ksplit == 1 && vf == vl) {
            const int rA = tile * 16 + g, rB = rA + 8;
            if (MODE == 0) {
                if (t < a.m) {
                    if (rA < a.rows) a.y[(int64_t)t * a.ldy + rA] = v0;
                    if (rB < a.rows) a.y[(int64_t)t * a.ldy + rB] = v1;
                }
            } else {
                if (2 * t < a.m) {
                    if (rA < a.rows) a.y[(int64_t)(2 * t) * a.ldy + rA] = v0;
                    if (rB < a.rows) a.y[(int64_t)(2 * t) * a.ldy + rB] = v2;
                }
                if (2 * t + 1 < a.m) {
                    if (rA < a.rows) a.y[(int64_t)(2 * t + 1) * a.ldy + rA] = v1;
                    if (rB < a.rows) a.y[(int64_t)(2 * t + 1) * a.ldy + rB] = v3;
                }
            }
            return;
        }
        float *p = a.partials + (((size_t)slice * a.tiles + tile) * a.maxseg + (size_t)(v - vf)) * 128;
        if (MODE == 0) {
            if (t < a.m) { p[t * 16 + g] = v0; p[t * 16 + g + 8] = v1; }
        } else {
            if (2 * t < a.m) { p[2 * t * 16 + g] = v0; p[2 * t * 16 + g + 8] = v2; }
            if (2 * t + 1 < a.m) { p[(2 * t + 1) * 16 + g] = v1; p[(2 * t + 1) * 16 + g + 8] = v3; }
        }
        // segments of this tile over all K slices
        unsigned int expected = 0;
        for (int s = 0; s < a.ksplit; s++) {
            const int n_s = min(a.units_per_slice, a.units - s * a.units_per_slice);
            const int64_t I_s = (int64_t)a.tiles * n_s, j0 = (int64_t)tile * n_s, j1 = j0 + n_s - 1;
            const int64_t W_s = min((int64_t)a.ctas_per_slice * C, I_s);
            expected += (unsigned int)(((j1 + 1) * W_s - 1) / I_s - ((j0 + 1) * W_s - 1) / I_s + 1);
        }
        __threadfence();
        __syncwarp();
        unsigned int old = 0;
        if (lane == 0) old = atomicAdd(a.tickets + tile, 1u);
        old = __shfl_sync(0xffffffffu, old, 0);
        if (old != expected - 1) return;
        __threadfence();
        for (int o = lane; o < 16 * a.m; o += 32) {
            const int j = o >> 4, r = o & 15;
            float s = 0.f;
            for (int sl = 0; sl < a.ksplit; sl++) {
                const int n_s = min(a.units_per_slice, a.units - sl * a.units_per_slice);
                const int64_t I_s = (int64_t)a.tiles * n_s, j0 = (int64_t)tile * n_s, j1 = j0 + n_s - 1;
                const int64_t W_s = min((int64_t)a.ctas_per_slice * C, I_s);
                const int nseg = (int)(((j1 + 1) * W_s - 1) / I_s - ((j0 + 1) * W_s - 1) / I_s + 1);
                const float *q = a.partials + ((size_t)sl * a.tiles + tile) * a.maxseg * 128 + o;
                for (int sg = 0; sg < nseg; sg++) s += __ldcg(q + (size_t)sg * 128);
            }
            if (tile * 16 + r < a.rows) a.y[(int64_t)j * a.ldy + tile * 16 + r] = s;
        }
        if (lane == 0) a.tickets[tile] = 0u;  // ready for the next launch
    };

    int64_t ci = lo;
    int ctile = (int)(lo / nun), cu = (int)(lo - (int64_t)ctile * nun), cslot = 0;
    uint32_t phases = 0;  // bit d = parity to wait for on slot d
    int cur_tile = ctile;
    bool alive = true;
    while (ci < hi) {
        const int n = (int)min((int64_t)min(KC, nun - cu), hi - ci);
        if (ctile != cur_tile) {
            flush(cur_tile);
            acc[0] = acc[1] = acc[2] = acc[3] = 0.f;
            cur_tile = ctile;
        }
        if (!mbar_wait_bounded(my_bars + 8 * cslot, (phases >> cslot) & 1u)) {
            if (lane == 0) atomicOr(a.status, QM_STATUS_TIMEOUT);
            alive = false;
            break;
        }
        phases ^= 1u << cslot;
        const uint8_t *stage = my_stages + (size_t)cslot * stage_bytes;
        for (int un = 0; un < n; un++) {
            UnitData<FMT> ud;
            read_unit<FMT>(ud, stage, rsq, rsd, un, g, t);
            const int ul = cu + un;
            compute_unit<FMT, MODE>(ud, acc, plane_hi, plane_lo, xsum + ((size_t)ul * NPL + g) * 4,
                                    xsum + ((size_t)ul * NPL + g + a.m) * 4, ul, t, bact);
        }
        ci += n;
        cu += n;
        if (cu == nun) { cu = 0; ctile++; }
        cslot = cslot + 1 == D ? 0 : cslot + 1;
        // the slot just read is free again: every lane's reads of it have returned (their values
        // were consumed above), so after the warp converges the next bulk copy may overwrite it
        __syncwarp();
        if (ii < hi) issue();
    }
    if (alive && lo < hi) flush(cur_tile);
}

}  // namespace

#define QM_GEMV_KERNEL(name, FMT, MODE)                                                         \
    extern "C" __global__ void __launch_bounds__(QM_GEMV_MAX_THREADS, 1)                        \
        name(const __grid_constant__ QmGemvArgs a) {                                            \
        gemv_body<FMT, MODE>(a);                                                                \
    }

QM_GEMV_KERNEL(qm_gemv_q40_m4, QM_FMT_Q4_0, 0)
QM_GEMV_KERNEL(qm_gemv_q40_m8, QM_FMT_Q4_0, 1)
QM_GEMV_KERNEL(qm_gemv_q80_m4, QM_FMT_Q8_0, 0)
QM_GEMV_KERNEL(qm_gemv_q80_m8, QM_FMT_Q8_0, 1)
