// qm_gemv_kq.cu — decode GEMV (1..8 activation rows) over the two low-bit super-block formats
// the reference decodes on the CPU with golden vectors, Q2_K and IQ2_XXS, for sm_100a.
//
// Supersedes the reference's one-warp-per-row device kernels q2_k_matvec
// (nvidia/x/egraph/codegen.go:674-735) and iq2_xxs_matvec (:737-809). The weights stay in the
// GGUF byte layout (84- and 66-byte super-blocks of 256 elements, rows contiguous): a warp
// owns a row at a time and walks its super-blocks, the 32 lanes covering the 256 elements of
// one super-block — 8 elements per lane, so every lane decodes whole bytes and the per-group
// scales are read once per lane. Rows are dealt to the warps of a grid that fills the SMs; a
// warp streams its rows through a private shared-memory ring (cp.async, 2..4 rows in flight).
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
// Exact float of an integer of magnitude below 2^22 with two full-rate instructions (the conversion
// instruction runs at a quarter of that rate and was the busiest pipe of the Q8_1 kernels).
__device__ __forceinline__ float small_int_to_float(int v) { return __int_as_float(v + 0x4B400000) - 12582912.f; }
// Bytes 0..3 of `a`, each replaced by eight copies of its top bit (PRMT selector nibbles with bit 3 set).
__device__ __forceinline__ uint32_t top_bits_to_bytes(uint32_t a) {
    uint32_t d;
    asm("prmt.b32 %0, %1, %1, 0xBA98;" : "=r"(d) : "r"(a));
    return d;
}

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

// ---- Q8_1 activations: integer dot products ---------------------------------------------------
// With the activations already in 8-bit quants the products run on dp4a: four 2-bit codes (or four
// codebook magnitudes) times four quants per instruction, the block scales applied once per group
// in float32 — a sixth of the instructions of the float form, which is bound by int-to-float
// conversions.

// Q2_K x Q8_1. Eight lanes cover a super-block, one Q8_1 block each (32 elements = two scale groups: 32 bytes
// of qs at one bit position, eight words times eight words on dp4a, each group's scale and minimum applied
// once to its integer sums), so a warp takes four super-blocks per step; `blk` is this lane's super-block (or
// null past the row's end), i = lane & 7 = the Q8_1 block within it, xb0 the index of its first Q8_1 block.
template <int M>
__device__ __forceinline__ void q2k_q81_block(const uint8_t *blk, const uint8_t *xq, int ldx, int m, int xb0, int i,
                                              float (&acc)[M]) {
    if (!blk) return;
    // elements 32i .. 32i+31: the 32 bytes of half i>>2, bit pair i&3; scale groups 2i and 2i+1
    const int sh = 2 * (i & 3);
    const uint32_t *qw = reinterpret_cast<const uint32_t *>(blk + 16 + 32 * (i >> 2));
    const uint32_t sc2 = *reinterpret_cast<const uint16_t *>(blk + 2 * i);
    const uint32_t dd = *reinterpret_cast<const uint32_t *>(blk + 80);
    const float d = h2f(dd & 0xFFFFu), dmin = h2f(dd >> 16);
    // (an fp16 times an integer below 16 is exact in float32)
    const float dsc0 = d * (float)(sc2 & 0x0Fu), dmn0 = dmin * (float)((sc2 >> 4) & 0x0Fu);
    const float dsc1 = d * (float)((sc2 >> 8) & 0x0Fu), dmn1 = dmin * (float)(sc2 >> 12);
    int v[8];
#pragma unroll
    for (int w = 0; w < 8; w++) v[w] = (int)((qw[w] >> sh) & 0x03030303u);
#pragma unroll
    for (int j = 0; j < M; j++) {
        const uint8_t *xb = xq + ((j < m ? j : 0) * ldx + xb0 + i) * 36;
        const uint32_t *xw = reinterpret_cast<const uint32_t *>(xb + 4);
        int dot0 = 0, sum0 = 0, dot1 = 0, sum1 = 0;
#pragma unroll
        for (int w = 0; w < 4; w++) {
            const int x0 = (int)xw[w], x1 = (int)xw[4 + w];
            dot0 = __dp4a(v[w], x0, dot0);
            sum0 = __dp4a(0x01010101, x0, sum0);
            dot1 = __dp4a(v[4 + w], x1, dot1);
            sum1 = __dp4a(0x01010101, x1, sum1);
        }
        const float dx = h2f(*reinterpret_cast<const uint16_t *>(xb));
        const float g0 = dsc0 * small_int_to_float(dot0) - dmn0 * small_int_to_float(sum0);   // |.| <= 16*3*127
        const float g1 = dsc1 * small_int_to_float(dot1) - dmn1 * small_int_to_float(sum1);
        acc[j] = fmaf(dx, g0 + g1, acc[j]);
    }
}

// IQ2_XXS x Q8_1: eight lanes cover a super-block, one group of 32 elements (four codebook entries, one Q8_1
// block) each, so a warp takes four super-blocks per step; `blk` is this lane's super-block (or null past the
// row's end). The signs go into the sum as dot(all) - 2*dot(negated ones), which needs no per-byte negation;
// the group's scale is applied once to the integer sum.
template <int M>
__device__ __forceinline__ void iq2xxs_q81_block(const uint8_t *blk, const uint8_t *xq, int ldx, int m, int xb0, int group,
                                                 const unsigned long long *grid, float (&acc)[M]) {
    if (!blk) return;
    const float d = h2f(*reinterpret_cast<const uint16_t *>(blk));
    const uint16_t *g16 = reinterpret_cast<const uint16_t *>(blk + 2 + 8 * group);
    const uint32_t indices = (uint32_t)g16[0] | ((uint32_t)g16[1] << 16);
    const uint32_t aux = (uint32_t)g16[2] | ((uint32_t)g16[3] << 16);
    const float scale = (0.125f * d) * (float)(2u * (aux >> 28) + 1u);
    int gw[8], nw[8];
#pragma unroll
    for (int l = 0; l < 4; l++) {
        const unsigned long long code = grid[(indices >> (8 * l)) & 0xFFu];
        const uint32_t si = (aux >> (7 * l)) & 127u;
        const uint32_t signs = si | ((uint32_t)(__popc(si) & 1) << 7);
        // byte k of a mask word = 0xFF where sign bit k is set: the bit goes to the byte's top, PRMT replicates it
        const uint32_t t0 = ((signs & 0xFu) * 0x10204080u) & 0x80808080u, t1 = ((signs >> 4) * 0x10204080u) & 0x80808080u;
        gw[2 * l] = (int)(uint32_t)code;
        gw[2 * l + 1] = (int)(uint32_t)(code >> 32);
        nw[2 * l] = gw[2 * l] & (int)top_bits_to_bytes(t0);
        nw[2 * l + 1] = gw[2 * l + 1] & (int)top_bits_to_bytes(t1);
    }
#pragma unroll
    for (int j = 0; j < M; j++) {
        const uint8_t *xb = xq + ((j < m ? j : 0) * ldx + xb0 + group) * 36;
        const uint32_t *xw = reinterpret_cast<const uint32_t *>(xb + 4);
        int all = 0, neg = 0;
#pragma unroll
        for (int k = 0; k < 8; k++) {
            const int xv = (int)xw[k];
            all = __dp4a(gw[k], xv, all);
            neg = __dp4a(nw[k], xv, neg);
        }
        const float dx = h2f(*reinterpret_cast<const uint16_t *>(xb));
        acc[j] = fmaf(scale * dx, small_int_to_float(all - 2 * neg), acc[j]);   // |.| <= 32*43*127
    }
}

// SM: the rows go through the shared-memory rings and (Q8_1 kernels) the activations are staged in shared
// memory — a compile-time property, so that those reads are shared-memory loads with 32-bit addresses.
template <int FMT, int M, bool XQ, bool SM>
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
    const int64_t row_bytes = (int64_t)a.units * kBlockBytes;
    extern __shared__ __align__(16) uint8_t dyn_smem[];
    int xld = (int)a.ldx;
    if (XQ && SM) {
        // the CTA's Q8_1 activations go to shared memory once: rows packed units*8 blocks apart
        const int words = a.units * 8 * 9;
        for (int idx = threadIdx.x; idx < m * words; idx += blockDim.x) {
            const int j = idx / words, wd = idx - j * words;
            reinterpret_cast<uint32_t *>(dyn_smem)[idx] =
                __ldg(reinterpret_cast<const uint32_t *>(static_cast<const uint8_t *>(x) + (int64_t)j * a.ldx * 36) + wd);
        }
        __syncthreads();
        xld = a.units * 8;
    }
    auto finish_row = [&](int64_t row, float (&acc)[M]) {
#pragma unroll
        for (int j = 0; j < M; j++) {
            float s = acc[j];
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
            if (lane == 0 && j < m) y[(int64_t)j * a.ldy + row] = s;
        }
    };
    // one row's products: wr = the row's super-blocks (shared or global memory)
    auto row_dot = [&](const uint8_t *wr, float (&acc)[M]) {
        if (XQ && FMT == 10) {
            const uint8_t *xq = SM ? dyn_smem : static_cast<const uint8_t *>(x);
            for (int u = lane >> 3; u < a.units + (lane >> 3); u += 4)   // every lane makes the same number of steps
                q2k_q81_block<M>(u < a.units ? wr + (int64_t)u * kBlockBytes : nullptr, xq, xld, m, u * 8, lane & 7, acc);
        } else if (XQ) {
            const uint8_t *xq = SM ? dyn_smem : static_cast<const uint8_t *>(x);
            for (int u = lane >> 3; u < a.units + (lane >> 3); u += 4)   // every lane makes the same number of steps
                iq2xxs_q81_block<M>(u < a.units ? wr + (int64_t)u * kBlockBytes : nullptr, xq, xld, m, u * 8, lane & 7, grid, acc);
        } else {
            for (int u = 0; u < a.units; u++) {
                if (FMT == 10) q2k_block<M, false>(wr + (int64_t)u * kBlockBytes, x, a.ldx, m, u * 256, lane, acc);
                else iq2xxs_block<M, false>(wr + (int64_t)u * kBlockBytes, x, a.ldx, m, u * 256, lane, grid, acc);
            }
        }
    };
    if (SM) {
        // Staged form (rows are whole 16-byte pieces): every warp keeps `depth` rows in flight in a ring of its
        // own in shared memory, filled by 16-byte cp.async copies, and decodes from there — the bytes in
        // flight no longer depend on how many scattered loads a lane can have outstanding.
        const int D = a.depth;
        const uint32_t stage_bytes = (uint32_t)row_bytes;
        uint8_t *ring = dyn_smem + (XQ ? a.xs_bytes : 0) + (threadIdx.x >> 5) * D * stage_bytes;
        const uint32_t ring_s = (uint32_t)__cvta_generic_to_shared(ring);
        const int pieces = (int)(row_bytes >> 4);
        int64_t p_row = wid;
        int p_slot = 0;
        auto issue = [&]() {
            if (p_row < a.rows) {
                const uint8_t *src = wq + p_row * row_bytes;
                const uint32_t dst = ring_s + (uint32_t)p_slot * stage_bytes;
                for (int i = lane; i < pieces; i += 32)
                    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst + 16u * i), "l"(src + 16 * i) : "memory");
                p_row += warps;
            }
            asm volatile("cp.async.commit_group;" ::: "memory");
            p_slot = p_slot + 1 == D ? 0 : p_slot + 1;
        };
        for (int d = 0; d < D; d++) issue();
        int c_slot = 0;
        for (int64_t row = wid; row < a.rows; row += warps) {
            // the oldest of the D groups in flight is this row
            if (D == 2) asm volatile("cp.async.wait_group 1;" ::: "memory");
            else if (D == 3) asm volatile("cp.async.wait_group 2;" ::: "memory");
            else asm volatile("cp.async.wait_group 3;" ::: "memory");
            __syncwarp();
            const uint8_t *wr = ring + (size_t)c_slot * stage_bytes;
            float acc[M];
#pragma unroll
            for (int j = 0; j < M; j++) acc[j] = 0.f;
            row_dot(wr, acc);
            finish_row(row, acc);
            __syncwarp();   // every lane has read the slot before the next copy overwrites it
            issue();
            c_slot = c_slot + 1 == D ? 0 : c_slot + 1;
        }
        asm volatile("cp.async.wait_group 0;" ::: "memory");
    }
    for (int64_t row = wid; !SM && row < a.rows; row += warps) {
        const uint8_t *wr = wq + row * row_bytes;
        float acc[M];
#pragma unroll
        for (int j = 0; j < M; j++) acc[j] = 0.f;
        row_dot(wr, acc);
        finish_row(row, acc);
    }
}

}  // namespace

// Instantiated for 1, 2, 4 and 8 activation rows (the host picks the smallest that holds m), each for float32
// and for Q8_1 activations.
#define QM_KQ_KERNEL(name, fmt, mm, xq)                                                                        \
    extern "C" __global__ void __launch_bounds__(256) name(const __grid_constant__ QmKqArgs a) {               \
        if (a.depth >= 2) gemv_kq_body<fmt, mm, xq, true>(a);                                                  \
        else gemv_kq_body<fmt, mm, xq, false>(a);                                                              \
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
