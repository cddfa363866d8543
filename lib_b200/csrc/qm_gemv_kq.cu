// qm_gemv_kq.cu — decode GEMV (1..8 activation rows) over the two low-bit super-block formats
// the reference decodes on the CPU with golden vectors, Q2_K and IQ2_XXS, for sm_100a.
//
// Supersedes the reference's one-warp-per-row device kernels q2_k_matvec
// (nvidia/x/egraph/codegen.go:674-735) and iq2_xxs_matvec (:737-809). The weights stay in the
// GGUF byte layout (84- and 66-byte super-blocks of 256 elements, rows contiguous): a warp
// owns a row at a time and walks its super-blocks, the 32 lanes covering the 256 elements of
// one super-block — 8 elements per lane, so every lane decodes whole bytes and the per-group
// scales are read once per lane. Rows are dealt to the warps of a grid that fills the SMs.
// HBM-bound: algorithmic bytes per 256 weights = 84 (Q2_K) or 66 (IQ2_XXS) plus 4 bytes per
// activation.
//
// Arithmetic: dequantized values are formed exactly as the CPU decoders do
// (lm/quant/kquant.go:66-73 and :103-118) and multiplied into float32 accumulators, one per
// activation row and lane, reduced over the warp by shuffles at the end of the row.
//
// Two variations the reference also has as kernels of their own:
//   * _q8_1: the activations arrive as Q8_1 blocks (36 bytes: fp16 d, fp16 sum, 32 quants) and
//     element i is widened d times quant, as q8_1_at does (codegen.go:125-128) — the product
//     d*q is exact in float32, so this equals the float kernel run on the decoded vector;
//   * selected (a.ids set): blockIdx.y is a slot, ids[slot] an expert, the weights are
//     [expert][row][block] and y is [slot][row] (q2_k_selected_matvec_q8_1, codegen.go:554-583;
//     iq2_xxs_selected_matvec_q8_1, :585-616). An id outside [0, experts) fills the slot's
//     outputs with the NaN 0x7fffffff.
#include <cuda_fp16.h>
#include <stdint.h>

#define QM_GRID_QUALIFIER __device__ __constant__
#include "qm_iq2xxs_grid.h"
#include "qm_kernel_args.h"

namespace {

__device__ __forceinline__ float h2f(uint32_t bits) { return __half2float(__ushort_as_half((unsigned short)bits)); }

// Elements e, e+1 (e even) of activation row `row` (x: floats, or Q8_1 blocks when XQ; ldx in floats or blocks).
template <bool XQ>
__device__ __forceinline__ float2 load_x2(const void *x, int64_t row, int64_t ldx, int e) {
    if (!XQ) return __ldg(reinterpret_cast<const float2 *>(static_cast<const float *>(x) + row * ldx + e));
    const uint8_t *b = static_cast<const uint8_t *>(x) + (row * ldx + (e >> 5)) * 36;
    const float d = h2f(__ldg(reinterpret_cast<const uint16_t *>(b)));
    const uint32_t q = __ldg(reinterpret_cast<const uint16_t *>(b + 4 + (e & 31)));
    return make_float2(d * (float)(int8_t)(q & 0xFFu), d * (float)(int8_t)(q >> 8));
}
// Elements e..e+7 (e a multiple of 8).
template <bool XQ>
__device__ __forceinline__ void load_x8(const void *x, int64_t row, int64_t ldx, int e, float (&v)[8]) {
    if (!XQ) {
        const float *xr = static_cast<const float *>(x) + row * ldx + e;
        const float4 a = __ldg(reinterpret_cast<const float4 *>(xr));
        const float4 b = __ldg(reinterpret_cast<const float4 *>(xr + 4));
        v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
        return;
    }
    const uint8_t *b = static_cast<const uint8_t *>(x) + (row * ldx + (e >> 5)) * 36;
    const float d = h2f(__ldg(reinterpret_cast<const uint16_t *>(b)));
    const uint32_t q0 = __ldg(reinterpret_cast<const uint32_t *>(b + 4 + (e & 31)));
    const uint32_t q1 = __ldg(reinterpret_cast<const uint32_t *>(b + 8 + (e & 31)));
#pragma unroll
    for (int i = 0; i < 4; i++) {
        v[i] = d * (float)(int8_t)((q0 >> (8 * i)) & 0xFFu);
        v[4 + i] = d * (float)(int8_t)((q1 >> (8 * i)) & 0xFFu);
    }
}

// One lane's share of a Q2_K super-block: the two quant bytes 2*lane and 2*lane+1 carry, at bit
// shifts 0/2/4/6, two neighbouring elements of four 16-element groups (kquant.go:60-70).
template <int M, bool XQ>
__device__ __forceinline__ void q2k_block(const uint8_t *blk, const void *x, int64_t ldx, int m, int col0, int lane,
                                          float (&acc)[M]) {
    const uint32_t dd = *reinterpret_cast<const uint32_t *>(blk + 80);
    const float d = h2f(dd & 0xFFFFu), dmin = h2f(dd >> 16);
    const int k = 2 * lane, h = k >> 5, b1 = (k >> 4) & 1, l = k & 15;
    const uint32_t q = *reinterpret_cast<const uint16_t *>(blk + 16 + k);
    const uint32_t s_lo = *reinterpret_cast<const uint32_t *>(blk + 8 * h);       // scales of groups 8h..8h+3
    const uint32_t s_hi = *reinterpret_cast<const uint32_t *>(blk + 8 * h + 4);   // groups 8h+4..8h+7
#pragma unroll
    for (int s = 0; s < 4; s++) {
        const int group = 8 * h + 2 * s + b1;
        const uint32_t scb = ((s < 2 ? s_lo : s_hi) >> (8 * ((2 * s + b1) & 3))) & 0xFFu;
        const float t1 = d * (float)(scb & 0x0Fu), t3 = dmin * (float)(scb >> 4);
        const float w0 = t1 * (float)((q >> (2 * s)) & 3u) - t3;
        const float w1 = t1 * (float)((q >> (8 + 2 * s)) & 3u) - t3;
        const int e = col0 + 16 * group + l;
#pragma unroll
        for (int j = 0; j < M; j++) {
            const float2 xv = load_x2<XQ>(x, j < m ? j : 0, ldx, e);
            acc[j] = fmaf(w0, xv.x, acc[j]);
            acc[j] = fmaf(w1, xv.y, acc[j]);
        }
    }
}

// One lane's share of an IQ2_XXS super-block: lane = 4*group + l decodes the eight elements of
// codebook entry l of its group (kquant.go:103-118). Blocks are only 2-byte aligned.
template <int M, bool XQ>
__device__ __forceinline__ void iq2xxs_block(const uint8_t *blk, const void *x, int64_t ldx, int m, int col0, int lane,
                                             const unsigned long long *grid, float (&acc)[M]) {
    const float d = h2f(*reinterpret_cast<const uint16_t *>(blk));
    const int group = lane >> 2, l = lane & 3;
    const uint16_t *g16 = reinterpret_cast<const uint16_t *>(blk + 2 + 8 * group);
    const uint32_t indices = (uint32_t)g16[0] | ((uint32_t)g16[1] << 16);
    const uint32_t aux = (uint32_t)g16[2] | ((uint32_t)g16[3] << 16);
    const float scale = (0.125f * d) * (float)(2u * (aux >> 28) + 1u);
    const unsigned long long code = grid[(indices >> (8 * l)) & 0xFFu];
    const uint32_t si = (aux >> (7 * l)) & 127u;
    const uint32_t signs = si | ((uint32_t)(__popc(si) & 1) << 7);
    float w[8];
#pragma unroll
    for (int j = 0; j < 8; j++) {
        const float v = (float)(uint32_t)((code >> (8 * j)) & 0xFFull);
        w[j] = scale * ((signs >> j) & 1u ? -v : v);
    }
    const int e = col0 + 32 * group + 8 * l;
#pragma unroll
    for (int j = 0; j < M; j++) {
        float xv[8];
        load_x8<XQ>(x, j < m ? j : 0, ldx, e, xv);
        float s = acc[j];
#pragma unroll
        for (int i = 0; i < 8; i++) s = fmaf(w[i], xv[i], s);
        acc[j] = s;
    }
}

template <int FMT, int M, bool XQ>
__device__ __forceinline__ void gemv_kq_body(const QmKqArgs &a) {
    __shared__ unsigned long long grid[FMT == 16 ? 256 : 1];
    if (FMT == 16) {
        for (int i = threadIdx.x; i < 256; i += blockDim.x) grid[i] = QM_IQ2XXS_GRID_INIT[i];
        __syncthreads();
    }
    constexpr int kBlockBytes = FMT == 10 ? 84 : 66;
    const int lane = threadIdx.x & 31;
    const int warps = (gridDim.x * blockDim.x) >> 5;
    const int wid = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int m = a.m < M ? a.m : M;   // the kernel's activation rows beyond a.m re-read row 0 and are not stored
    // selected form: this CTA row of the grid works for one slot, on the rows of the slot's expert
    const int slot = blockIdx.y;
    const uint8_t *wq = a.wq;
    float *y = a.y + (int64_t)slot * a.y_slot_stride;
    const void *x = XQ ? static_cast<const void *>(static_cast<const uint8_t *>(a.x) + (int64_t)slot * a.x_slot_stride * 36)
                       : static_cast<const void *>(static_cast<const float *>(a.x) + (int64_t)slot * a.x_slot_stride);
    if (a.ids) {
        const int e = a.ids[slot];
        if (e < 0 || e >= a.experts) {
            for (int64_t row = wid * 32 + lane; row < a.rows; row += (int64_t)warps * 32)
                for (int j = 0; j < m; j++) y[(int64_t)j * a.ldy + row] = __int_as_float(0x7fffffff);
            return;
        }
        wq += (int64_t)e * a.rows * a.units * kBlockBytes;
    }
    for (int64_t row = wid; row < a.rows; row += warps) {
        const uint8_t *wr = wq + row * (int64_t)a.units * kBlockBytes;
        float acc[M];
#pragma unroll
        for (int j = 0; j < M; j++) acc[j] = 0.f;
        const int64_t ldx = a.ldx;
        for (int u = 0; u < a.units; u++) {
            if (FMT == 10) q2k_block<M, XQ>(wr + (int64_t)u * kBlockBytes, x, ldx, m, u * 256, lane, acc);
            else iq2xxs_block<M, XQ>(wr + (int64_t)u * kBlockBytes, x, ldx, m, u * 256, lane, grid, acc);
        }
#pragma unroll
        for (int j = 0; j < M; j++) {
            float s = acc[j];
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
            if (lane == 0 && j < m) y[(int64_t)j * a.ldy + row] = s;
        }
    }
}

}  // namespace

// Instantiated for 1, 2, 4 and 8 activation rows (the host picks the smallest that holds m), each for float32
// and for Q8_1 activations.
#define QM_KQ_KERNEL(name, fmt, mm, xq)                                                                        \
    extern "C" __global__ void __launch_bounds__(256) name(const __grid_constant__ QmKqArgs a) {               \
        gemv_kq_body<fmt, mm, xq>(a);                                                                          \
    }
QM_KQ_KERNEL(qm_gemv_q2k_m1, 10, 1, false)
QM_KQ_KERNEL(qm_gemv_q2k_m2, 10, 2, false)
QM_KQ_KERNEL(qm_gemv_q2k_m4, 10, 4, false)
QM_KQ_KERNEL(qm_gemv_q2k_m8, 10, 8, false)
QM_KQ_KERNEL(qm_gemv_iq2xxs_m1, 16, 1, false)
QM_KQ_KERNEL(qm_gemv_iq2xxs_m2, 16, 2, false)
QM_KQ_KERNEL(qm_gemv_iq2xxs_m4, 16, 4, false)
QM_KQ_KERNEL(qm_gemv_iq2xxs_m8, 16, 8, false)
QM_KQ_KERNEL(qm_gemv_q2k_q81_m1, 10, 1, true)
QM_KQ_KERNEL(qm_gemv_q2k_q81_m2, 10, 2, true)
QM_KQ_KERNEL(qm_gemv_q2k_q81_m4, 10, 4, true)
QM_KQ_KERNEL(qm_gemv_q2k_q81_m8, 10, 8, true)
QM_KQ_KERNEL(qm_gemv_iq2xxs_q81_m1, 16, 1, true)
QM_KQ_KERNEL(qm_gemv_iq2xxs_q81_m2, 16, 2, true)
QM_KQ_KERNEL(qm_gemv_iq2xxs_q81_m4, 16, 4, true)
QM_KQ_KERNEL(qm_gemv_iq2xxs_q81_m8, 16, 8, true)
