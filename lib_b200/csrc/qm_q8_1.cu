// qm_q8_1.cu — the Q8_1 activation ABI for sm_100a: producers that write activation vectors as
// 36-byte blocks (fp16 d, fp16 sum field, 32 signed quants) and the expansion back to float32
// for the matvecs whose staging quantizes on its own.
//
// Replaces the reference's "bounded correctness" producers, which run ONE thread per row
// (rms_quant_q8_1, nvidia/x/cudaquant/quant.go:129-155) or one thread per block after a
// 32-thread barrier (fused_swiglu_q8_1, nvidia/x/egraph/codegen.go:513-552):
//   * qm_rmsnorm_q8_1: one CTA of 1024 threads per row, four neighbouring elements per thread;
//     the sum of squares is accumulated in float64 by all threads and reduced in a fixed order,
//     then every group of eight lanes turns its 32-element block into Q8_1 (maxima and quant
//     sums by shuffles), from registers when the row has at most 4096 columns. Bytes follow
//     cudaquant.RMSNormQ8_1 (quant.go:46-118): inv = float32(1/sqrt(ss/cols + eps)),
//     v = x*inv (*weight), qscale = max|v|/127, d = fp16(qscale), q = round-half-away(v/qscale)
//     clamped to +-127, s = fp16(float32(sum q) * qscale). The float64 sum is added in a
//     different order than the reference's serial loop; inv is its float32 rounding, so a
//     differing byte needs the two orders to straddle a float32 rounding boundary.
//   * qm_swiglu_q8_1: a warp per block; silu(min(gate,10)) * clamp(up,+-10) * weight[slot],
//     d = fp16(max/127), sum field = fp16(sum of the values), q = round(v / widened d).
//   * qm_q8_1_expand: element i -> widened d * q (q8_1_at, codegen.go:125-128), exact in
//     float32.
// All three are bound by launch latency at decode sizes (a few KB per row); they are written to
// be one short wave, not to stream.
#include <cuda_fp16.h>
#include <stdint.h>

#include "qm_kernel_args.h"

namespace {

__device__ __forceinline__ float h2f(uint32_t bits) { return __half2float(__ushort_as_half((unsigned short)bits)); }
__device__ __forceinline__ uint32_t f2h(float f) { return (uint32_t)__half_as_ushort(__float2half_rn(f)); }

// Writes one block from a warp: lane l holds quant q (already clamped), `head` = d | s << 16.
__device__ __forceinline__ void store_block(uint8_t *dst, uint32_t head, int q, int lane) {
    uint32_t w = (uint32_t)q & 0xFFu;
    w |= __shfl_down_sync(0xffffffffu, w, 1) << 8;    // lanes 0, 2, 4, ...: two quants
    w |= __shfl_down_sync(0xffffffffu, w, 2) << 16;   // lanes 0, 4, 8, ...: four quants
    const uint32_t word = __shfl_sync(0xffffffffu, w, lane >= 1 && lane <= 8 ? 4 * (lane - 1) : 0);
    if (lane == 0) reinterpret_cast<uint32_t *>(dst)[0] = head;
    else if (lane <= 8) reinterpret_cast<uint32_t *>(dst)[lane] = word;
}

}  // namespace

// One CTA of 1024 threads per row: thread t owns elements 4t..4t+3 of every 4096-column chunk, so a block of 32
// elements lies in eight neighbouring lanes and a row of up to 4096 columns is read from memory once.
extern "C" __global__ void __launch_bounds__(1024) qm_rmsnorm_q8_1(const __grid_constant__ QmNormQ81Args a) {
    __shared__ double part[32];
    __shared__ int bad;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int64_t r = blockIdx.x;
    const float *in = a.x + r * a.ldx;
    const bool vec = ((reinterpret_cast<uintptr_t>(in) | (a.weight ? reinterpret_cast<uintptr_t>(a.weight) : 0)) & 15) == 0;
    auto load4 = [&](const float *p, int c) {
        if (vec) return *reinterpret_cast<const float4 *>(p + c);
        return make_float4(p[c], p[c + 1], p[c + 2], p[c + 3]);
    };
    if (tid == 0) bad = 0;
    double ss = 0.0;
    bool nonfinite = false;
    float4 keep = make_float4(0.f, 0.f, 0.f, 0.f);   // the row's first chunk stays in registers
    for (int c = 4 * tid; c < a.cols; c += 4096) {
        const float4 v = load4(in, c);
        if (c < 4096) keep = v;
        nonfinite |= !(isfinite(v.x) && isfinite(v.y) && isfinite(v.z) && isfinite(v.w));
        if (a.weight && r == 0) {
            const float4 w = load4(a.weight, c);
            nonfinite |= !(isfinite(w.x) && isfinite(w.y) && isfinite(w.z) && isfinite(w.w));
        }
        // every square is exact in float64, so each fma rounds once, as a separate add would
        ss = fma((double)v.x, (double)v.x, ss);
        ss = fma((double)v.y, (double)v.y, ss);
        ss = fma((double)v.z, (double)v.z, ss);
        ss = fma((double)v.w, (double)v.w, ss);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    __syncthreads();
    if (lane == 0) part[warp] = ss;
    if (nonfinite) bad = 1;
    __syncthreads();
    double tot = part[lane];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) tot += __shfl_xor_sync(0xffffffffu, tot, o);
    const double denom = tot / (double)a.cols + (double)a.eps;
    bool domain = bad != 0 || denom == 0.0;
    const float inv = (float)(1.0 / sqrt(denom));
    uint8_t *out = a.out + r * (int64_t)(a.cols / 32) * 36;
    for (int c = 4 * tid; c < a.cols; c += 4096) {
        const float4 x = c < 4096 ? keep : load4(in, c);
        float v[4] = {x.x * inv, x.y * inv, x.z * inv, x.w * inv};
        if (a.weight) {
            const float4 w = load4(a.weight, c);
            v[0] *= w.x; v[1] *= w.y; v[2] *= w.z; v[3] *= w.w;
        }
        domain |= !(isfinite(v[0]) && isfinite(v[1]) && isfinite(v[2]) && isfinite(v[3]));
        // the block's eight lanes are all here or all absent (cols is a multiple of 32); other lanes of the warp may be absent
        const uint32_t grp = 0xFFu << (lane & 24);
        float mx = fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3])));
#pragma unroll
        for (int o = 4; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(grp, mx, o));
        const float qscale = mx / 127.f;
        uint32_t word = 0;
        int sum = 0;
        if (qscale != 0.f) {
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const float t = roundf(v[i] / qscale);
                const int q = t > 127.f ? 127 : t < -127.f ? -127 : (int)t;   // also maps a NaN to a definite value
                sum += q;
                word |= ((uint32_t)q & 0xFFu) << (8 * i);
            }
        }
#pragma unroll
        for (int o = 4; o > 0; o >>= 1) sum += __shfl_xor_sync(grp, sum, o);
        uint32_t *dst = reinterpret_cast<uint32_t *>(out + (int64_t)(c >> 5) * 36);
        if ((lane & 7) == 0) dst[0] = f2h(qscale) | (qscale != 0.f ? f2h((float)sum * qscale) << 16 : 0u);
        dst[1 + (lane & 7)] = word;
    }
    if (domain) atomicOr(a.status, QM_STATUS_DOMAIN);
}

extern "C" __global__ void __launch_bounds__(256) qm_swiglu_q8_1(const __grid_constant__ QmSwigluQ81Args a) {
    const int lane = threadIdx.x & 31;
    const int64_t total = (int64_t)a.width * a.slots, blocks = (total + 31) / 32;
    const int64_t warps = ((int64_t)gridDim.x * blockDim.x) >> 5;
    for (int64_t b = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5; b < blocks; b += warps) {
        const int64_t i = b * 32 + lane;
        float v = 0.f;
        if (i < total) {
            const float g = fminf(a.gate[i], 10.0f);
            const float u = fminf(fmaxf(a.up[i], -10.0f), 10.0f);
            v = (g / (1.0f + expf(-g))) * u * a.weights[i / a.width];
        }
        float mx = fabsf(v), s = v;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
        // the sum field: the reference adds the block's values one after the other in float32; the same order here
        // (lane 0 walks the 32 values) keeps the field's bytes equal
        s = 0.f;
        for (int j = 0; j < 32; j++) {
            const float vj = __shfl_sync(0xffffffffu, v, j);
            if (b * 32 + j < total) s += vj;
        }
        const uint32_t dh = f2h(mx / 127.0f);
        const float d = h2f(dh);
        float t = d == 0.0f ? 0.0f : roundf(v / d);
        t = t > 127.f ? 127.f : t < -127.f ? -127.f : t;
        uint8_t *dst = a.out + b * 36;
        if (b * 32 + 32 <= total) {
            store_block(dst, dh | (f2h(s) << 16), (int)t, lane);
        } else {   // the last, partial block: the quants past the end are not written
            if (lane == 0) reinterpret_cast<uint32_t *>(dst)[0] = dh | (f2h(s) << 16);
            if (i < total) dst[4 + lane] = (uint8_t)(int8_t)(int)t;
        }
    }
}

// out[j][i] = widened d * q of row j's Q8_1 vector (rows ldx blocks apart; out rows ld_out floats apart).
extern "C" __global__ void __launch_bounds__(256) qm_q8_1_expand(const __grid_constant__ QmQ81ExpandArgs a) {
    const int64_t per_row = a.cols / 4;
    const int64_t total = per_row * a.m;
    for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (int64_t)gridDim.x * blockDim.x) {
        const int64_t j = idx / per_row;
        const int e = (int)(idx - j * per_row) * 4;
        const uint8_t *b = a.xq + (j * a.ldx + (e >> 5)) * 36;
        const float d = h2f(*reinterpret_cast<const uint16_t *>(b));
        const uint32_t q = *reinterpret_cast<const uint32_t *>(b + 4 + (e & 31));
        float4 v;
        v.x = d * (float)(int8_t)(q & 0xFFu);
        v.y = d * (float)(int8_t)((q >> 8) & 0xFFu);
        v.z = d * (float)(int8_t)((q >> 16) & 0xFFu);
        v.w = d * (float)(int8_t)(q >> 24);
        *reinterpret_cast<float4 *>(a.out + j * a.ld_out + e) = v;
    }
}
