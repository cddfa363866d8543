// qm_dequant.cu — bit-exact dequantization of stored weights to float32, and the
// upload-time repack of Q4_0/Q8_0 GGUF blocks into the store's layout (sm_100a).
//
// The arithmetic is that of the reference's CPU decoders, one float32
// operation at a time with no fused multiply-add:
//   Q4_0  (nibble-8)*scale            lm/quant/quant.go:60-64
//   Q8_0  int8*scale                  lm/quant/quant.go:87
//   Q2_K  d*(sc&15)*q - dmin*(sc>>4)  lm/quant/kquant.go:66-73
//   Q4_K  d*sc*q - dmin*m             same form; layout of GGUF type 12
//   IQ2_XXS (0.125*d*(2s+1))*(+-code) lm/quant/kquant.go:103-118
// fp16 scales go through an integer restatement of Float16ToFloat32
// (lm/quant/quant.go:94-116) so that NaN payloads survive unchanged.
#include <stdint.h>

#define QM_GRID_QUALIFIER __device__ __constant__
#include "qm_iq2xxs_grid.h"
#include "qm_kernel_args.h"

namespace {

__device__ __forceinline__ float f16_bits_to_f32(uint32_t h) {
    const uint32_t sign = (h & 0x8000u) << 16;
    uint32_t exp = (h & 0x7C00u) >> 10;
    uint32_t mant = h & 0x03FFu;
    if (exp == 0) {
        if (mant == 0) return __uint_as_float(sign);
        const int shift = __clz(mant) - 21;  // bring the leading one to bit 10
        mant = (mant << shift) & 0x03FFu;
        exp = (uint32_t)(1 - shift);
    } else if (exp == 0x1F) {
        return __uint_as_float(sign | 0x7F800000u | (mant << 13));
    }
    return __uint_as_float(sign | ((exp + 112u) << 23) | (mant << 13));
}

__device__ __forceinline__ float4 scale4(uint32_t bytes4, float t1, float t3) {
    float4 o;
    o.x = __fsub_rn(__fmul_rn(t1, (float)(bytes4 & 0xFF)), t3);
    o.y = __fsub_rn(__fmul_rn(t1, (float)((bytes4 >> 8) & 0xFF)), t3);
    o.z = __fsub_rn(__fmul_rn(t1, (float)((bytes4 >> 16) & 0xFF)), t3);
    o.w = __fsub_rn(__fmul_rn(t1, (float)(bytes4 >> 24)), t3);
    return o;
}

}  // namespace

// Q4_K store layout: item (tile, unit) = 16 headers of 16 bytes, then for each 32-byte quant
// group p the 16 rows side by side. One thread per four consecutive output columns.
extern "C" __global__ void __launch_bounds__(256) qm_dequant_q4k(const __grid_constant__ QmDequantArgs a) {
    const int64_t ngroups = a.rows * (int64_t)(a.cols / 4);
    for (int64_t idx = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; idx < ngroups;
         idx += (int64_t)gridDim.x * blockDim.x) {
        const int64_t row = idx / (a.cols / 4);
        const int col = (int)(idx - row * (a.cols / 4)) * 4;
        const int u = col >> 8, e = col & 255, j = e >> 5, i = e & 31;
        const int r = (int)(row & 15);
        const uint8_t *item = a.wq + ((row >> 4) * a.units + u) * QM_Q4K_ITEM_BYTES;
        const uint8_t *blk = item + 16 * r;
        const uint32_t dd = *reinterpret_cast<const uint32_t *>(blk);
        const float d = f16_bits_to_f32(dd & 0xFFFFu), dmin = f16_bits_to_f32(dd >> 16);
        const uint8_t *S = blk + 4;
        int sc, m;
        if (j < 4) {
            sc = S[j] & 63;
            m = S[j + 4] & 63;
        } else {
            sc = (S[j + 4] & 0x0F) | ((S[j - 4] >> 6) << 4);
            m = (S[j + 4] >> 4) | ((S[j] >> 6) << 4);
        }
        uint32_t q4 = *reinterpret_cast<const uint32_t *>(item + 256 + 512 * (j >> 1) + 32 * r + i);
        q4 = (j & 1) ? ((q4 >> 4) & 0x0F0F0F0Fu) : (q4 & 0x0F0F0F0Fu);
        const float t1 = __fmul_rn(d, (float)sc), t3 = __fmul_rn(dmin, (float)m);
        *reinterpret_cast<float4 *>(a.out + row * a.cols + col) = scale4(q4, t1, t3);
    }
}

// GGUF Q4_K rows (144-byte super-blocks) -> store layout. One thread per super-block.
extern "C" __global__ void __launch_bounds__(256) qm_repack_q4k(const __grid_constant__ QmRepackArgs a) {
    const int nblk = a.cols / 256;
    const int64_t total = a.nrows * nblk;
    for (int64_t idx = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; idx < total;
         idx += (int64_t)gridDim.x * blockDim.x) {
        const int64_t rr = idx / nblk;
        const int u = (int)(idx - rr * nblk);
        const int64_t row = a.row_offset + rr;
        const uint4 *s = reinterpret_cast<const uint4 *>(a.src + idx * 144);
        uint8_t *item = a.wq + ((row >> 4) * a.units + u) * QM_Q4K_ITEM_BYTES;
        const int r = (int)(row & 15);
        *reinterpret_cast<uint4 *>(item + 16 * r) = s[0];
#pragma unroll
        for (int p = 0; p < 4; p++) {
            *reinterpret_cast<uint4 *>(item + 256 + 512 * p + 32 * r) = s[1 + 2 * p];
            *reinterpret_cast<uint4 *>(item + 256 + 512 * p + 32 * r + 16) = s[2 + 2 * p];
        }
    }
}

extern "C" __global__ void __launch_bounds__(256) qm_dequant_q2k(const __grid_constant__ QmDequantArgs a) {
    const int64_t ngroups = a.rows * (int64_t)(a.cols / 4);
    for (int64_t idx = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; idx < ngroups;
         idx += (int64_t)gridDim.x * blockDim.x) {
        const int64_t row = idx / (a.cols / 4);
        const int col = (int)(idx - row * (a.cols / 4)) * 4;
        const int u = col >> 8, e = col & 255, group = e >> 4, l = e & 15;
        const uint8_t *blk = a.wq + (row * a.units + u) * 84;
        const uint32_t dd = *reinterpret_cast<const uint32_t *>(blk + 80);
        const float d = f16_bits_to_f32(dd & 0xFFFFu), dmin = f16_bits_to_f32(dd >> 16);
        const int base = 32 * (group >> 3) + 16 * (group & 1);
        const int shift = ((group >> 1) & 3) * 2;
        const uint32_t q4 = (*reinterpret_cast<const uint32_t *>(blk + 16 + base + l) >> shift) & 0x03030303u;
        const uint32_t sc = blk[group];
        const float t1 = __fmul_rn(d, (float)(sc & 0x0F)), t3 = __fmul_rn(dmin, (float)(sc >> 4));
        *reinterpret_cast<float4 *>(a.out + row * a.cols + col) = scale4(q4, t1, t3);
    }
}

// IQ2_XXS: GGUF bytes unchanged, 66-byte super-blocks (2-byte aligned): d, then eight groups of
// two little-endian words (four codebook indices | four 7-bit sign indices and the 4-bit scale).
// Sign index i stands for the byte i | parity(i) << 7; bit j set negates element j.
extern "C" __global__ void __launch_bounds__(256) qm_dequant_iq2xxs(const __grid_constant__ QmDequantArgs a) {
    const int64_t ngroups = a.rows * (int64_t)(a.cols / 4);
    for (int64_t idx = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; idx < ngroups;
         idx += (int64_t)gridDim.x * blockDim.x) {
        const int64_t row = idx / (a.cols / 4);
        const int col = (int)(idx - row * (a.cols / 4)) * 4;
        const int u = col >> 8, e = col & 255, group = e >> 5, l = (e >> 3) & 3, j0 = e & 7;
        const uint8_t *blk = a.wq + (row * a.units + u) * 66;
        const float d = f16_bits_to_f32(*reinterpret_cast<const uint16_t *>(blk));
        const uint16_t *g16 = reinterpret_cast<const uint16_t *>(blk + 2 + 8 * group);
        const uint32_t indices = (uint32_t)g16[0] | ((uint32_t)g16[1] << 16);
        const uint32_t aux = (uint32_t)g16[2] | ((uint32_t)g16[3] << 16);
        const float scale = __fmul_rn(__fmul_rn(0.125f, d), (float)(2u * (aux >> 28) + 1u));
        const unsigned long long code = QM_IQ2XXS_GRID_INIT[(indices >> (8 * l)) & 0xFFu];
        const uint32_t si = (aux >> (7 * l)) & 127u;
        const uint32_t signs = si | ((uint32_t)(__popc(si) & 1) << 7);
        float o[4];
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const float v = (float)(uint32_t)((code >> (8 * (j0 + j))) & 0xFFull);
            o[j] = __fmul_rn(scale, ((signs >> (j0 + j)) & 1u) ? -v : v);
        }
        *reinterpret_cast<float4 *>(a.out + row * a.cols + col) = make_float4(o[0], o[1], o[2], o[3]);
    }
}

// Store layout of Q4_0: 4-block groups of 64 bytes, word t*4+i = word t of block 4G+i.
extern "C" __global__ void __launch_bounds__(256) qm_dequant_q40(const __grid_constant__ QmDequantArgs a) {
    const int64_t ngroups = a.rows * (int64_t)(a.cols / 4);
    for (int64_t idx = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; idx < ngroups;
         idx += (int64_t)gridDim.x * blockDim.x) {
        const int64_t row = idx / (a.cols / 4);
        const int col = (int)(idx - row * (a.cols / 4)) * 4;
        const int blk = col >> 5, i = col & 31, half = i >> 4, t = (i & 15) >> 2;
        const int64_t b0 = row * a.units * 8;
        const float d = f16_bits_to_f32(a.wd[b0 + blk]);
        const uint32_t *words = reinterpret_cast<const uint32_t *>(a.wq + b0 * 16);
        uint32_t q4 = words[(blk >> 2) * 16 + t * 4 + (blk & 3)];
        q4 = half ? ((q4 >> 4) & 0x0F0F0F0Fu) : (q4 & 0x0F0F0F0Fu);
        float4 o;
        o.x = __fmul_rn((float)((int)(q4 & 0xFF) - 8), d);
        o.y = __fmul_rn((float)((int)((q4 >> 8) & 0xFF) - 8), d);
        o.z = __fmul_rn((float)((int)((q4 >> 16) & 0xFF) - 8), d);
        o.w = __fmul_rn((float)((int)(q4 >> 24) - 8), d);
        *reinterpret_cast<float4 *>(a.out + row * a.cols + col) = o;
    }
}

// Store layout of Q8_0: 2-block groups of 64 bytes, word t*4+2*bi+hf = word 4*hf+t of block 2G+bi.
extern "C" __global__ void __launch_bounds__(256) qm_dequant_q80(const __grid_constant__ QmDequantArgs a) {
    const int64_t ngroups = a.rows * (int64_t)(a.cols / 4);
    for (int64_t idx = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; idx < ngroups;
         idx += (int64_t)gridDim.x * blockDim.x) {
        const int64_t row = idx / (a.cols / 4);
        const int col = (int)(idx - row * (a.cols / 4)) * 4;
        const int blk = col >> 5, w = (col & 31) >> 2, hf = w >> 2, t = w & 3;
        const int64_t b0 = row * a.units * 8;
        const float d = f16_bits_to_f32(a.wd[b0 + blk]);
        const uint32_t *words = reinterpret_cast<const uint32_t *>(a.wq + b0 * 32);
        const uint32_t q4 = words[(blk >> 1) * 16 + t * 4 + 2 * (blk & 1) + hf];
        float4 o;
        o.x = __fmul_rn((float)(int8_t)(q4 & 0xFF), d);
        o.y = __fmul_rn((float)(int8_t)((q4 >> 8) & 0xFF), d);
        o.z = __fmul_rn((float)(int8_t)((q4 >> 16) & 0xFF), d);
        o.w = __fmul_rn((float)(int8_t)(q4 >> 24), d);
        *reinterpret_cast<float4 *>(a.out + row * a.cols + col) = o;
    }
}

// GGUF Q4_0 rows (18-byte blocks, 2-byte aligned) -> store layout. One thread per block.
extern "C" __global__ void __launch_bounds__(256) qm_repack_q40(const __grid_constant__ QmRepackArgs a) {
    const int nblk = a.cols / 32;
    const int64_t total = a.nrows * nblk;
    for (int64_t idx = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; idx < total;
         idx += (int64_t)gridDim.x * blockDim.x) {
        const int64_t r = idx / nblk;
        const int blk = (int)(idx - r * nblk);
        const uint16_t *s = reinterpret_cast<const uint16_t *>(a.src + idx * 18);
        const int64_t b0 = (a.row_offset + r) * a.units * 8;
        a.wd[b0 + blk] = s[0];
        uint32_t *words = reinterpret_cast<uint32_t *>(a.wq + b0 * 16);
#pragma unroll
        for (int t = 0; t < 4; t++)
            words[(blk >> 2) * 16 + t * 4 + (blk & 3)] = (uint32_t)s[1 + 2 * t] | ((uint32_t)s[2 + 2 * t] << 16);
    }
}

extern "C" __global__ void __launch_bounds__(256) qm_repack_q80(const __grid_constant__ QmRepackArgs a) {
    const int nblk = a.cols / 32;
    const int64_t total = a.nrows * nblk;
    for (int64_t idx = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; idx < total;
         idx += (int64_t)gridDim.x * blockDim.x) {
        const int64_t r = idx / nblk;
        const int blk = (int)(idx - r * nblk);
        const uint16_t *s = reinterpret_cast<const uint16_t *>(a.src + idx * 34);
        const int64_t b0 = (a.row_offset + r) * a.units * 8;
        a.wd[b0 + blk] = s[0];
        uint32_t *words = reinterpret_cast<uint32_t *>(a.wq + b0 * 32);
#pragma unroll
        for (int w = 0; w < 8; w++)
            words[(blk >> 1) * 16 + (w & 3) * 4 + 2 * (blk & 1) + (w >> 2)] =
                (uint32_t)s[1 + 2 * w] | ((uint32_t)s[2 + 2 * w] << 16);
    }
}

// Part-major copy of a tiled Q4_K store: item (tile, unit) of the [tiles][units] store goes to
// [unit / ups][tile][unit % ups], so that the items of one K part of every tile are contiguous.
// Sixteen bytes per thread.
extern "C" __global__ void __launch_bounds__(256) qm_repack_parts(const __grid_constant__ QmPartsArgs a) {
    const int64_t per_item = QM_Q4K_ITEM_BYTES / 16;
    const int64_t total = (int64_t)a.tiles * a.units * per_item;
    for (int64_t idx = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; idx < total;
         idx += (int64_t)gridDim.x * blockDim.x) {
        const int64_t item = idx / per_item, piece = idx - item * per_item;
        const int64_t tile = item / a.units;
        const int u = (int)(item - tile * a.units), part = u / a.ups, ul = u - part * a.ups;
        const int64_t dst = (((int64_t)part * a.tiles + tile) * a.ups + ul) * per_item + piece;
        reinterpret_cast<uint4 *>(a.dst)[dst] = reinterpret_cast<const uint4 *>(a.src)[idx];
    }
}
