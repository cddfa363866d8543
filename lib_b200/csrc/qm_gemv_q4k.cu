// qm_gemv_q4k.cu — decode GEMV (1..8 activation rows) over Q4_K weights for
// sm_100a on the integer tensor-core path, one matvec or a fused sequence of
// dependent matvecs (a whole decode step) in a single persistent launch.
//
// Supersedes the reference's one-warp-per-row k-quant matvec
// (nvidia/x/egraph/codegen.go:674-735) and its persistent task kernel idea
// (nvidia/x/cudamega/mega.go:36-71).
//
// Arithmetic. Q4_K stores value = d*sc_j*q - dmin*m_j with 4-bit q and 6-bit
// integers sc_j, m_j per 32-element sub-block. At HBM rate a B200 delivers
// ~11.6e12 such weights per second, so every instruction per weight counts:
//   * activations are quantized once per CTA into signed 8-bit limbs per
//     256-column unit: x = sx * (h + l1/128 [+ l2/16384]), sx = max|x|/127
//     (three limbs = 21 bits for up to 2 activation rows, two limbs beyond);
//   * four 4-bit codes become four u8 mma operands with ONE and-mask (low
//     nibbles) or one and-mask that leaves them multiplied by 16 (high
//     nibbles); mma.sync.m16n8k32.s32.u8.s8 (A = weights, B = limbs, one limb
//     per column) gives exact integer sub-block sums;
//   * the 6-bit sub-block scale multiplies the exact sums in integer
//     (one IMAD per accumulator); d, sx and the limb weight are applied once
//     per 256-column unit in fp32;
//   * the minimum term sum_j m_j * sum(x in sub-block j) is one fp16 mma per
//     unit against pre-reduced activation sums (fp16 hi+lo).
// Everything up to the per-unit fp32 scaling is exact integer arithmetic.
//
// Work split. One persistent CTA per SM; an op's 16-row tiles are dealt to the CTAs in
// contiguous runs, and inside a CTA the (tile, K unit) items of its run are dealt evenly to
// the warps. A tile whose K range is shared by several warps is finished through
// shared-memory partial sums added in warp order after one CTA barrier: no global scratch,
// no atomics, bit-reproducible.
//
// Data movement. One persistent CTA per SM; every warp streams its share of the
// (16-row tile, K unit) items of an op through a private ring of shared-memory
// stages filled by 16-byte cp.async copies (one commit group per stage), so the
// bytes in flight are bounded by shared memory, not by registers.
// Weights never depend on activations, so the rings run ahead across op
// boundaries: while the CTAs meet at the grid barrier that separates two
// dependent matvecs, the next matrix is already streaming in.
#include <cuda_fp16.h>
#include <stdint.h>

#include "qm_kernel_args.h"
#include "qm_pipe.cuh"

using namespace qm;

namespace {

__device__ __forceinline__ void mma_u8s8(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%10,%10,%10,%10};"
        : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(0));
}
__device__ __forceinline__ void mma_f16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t b0) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%6}, {%7,%6}, "
        "{%8,%8,%8,%8};"
        : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
        : "r"(a0), "r"(a1), "r"(0u), "r"(b0), "f"(0.f));
}
__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
    uint32_t d;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(sel));
    return d;
}
__device__ __forceinline__ uint32_t hsub2(uint32_t a, uint32_t b) {
    uint32_t d;
    asm("sub.rn.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
    return d;
}

__device__ __forceinline__ void cp_async16(uint32_t dst, const void *src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
// Waits until at most n of this thread's most recent commit groups are still in flight.
__device__ __forceinline__ void cp_async_wait(int n) {
    switch (n) {
    case 0: asm volatile("cp.async.wait_group 0;" ::: "memory"); break;
    case 1: asm volatile("cp.async.wait_group 1;" ::: "memory"); break;
    case 2: asm volatile("cp.async.wait_group 2;" ::: "memory"); break;
    case 3: asm volatile("cp.async.wait_group 3;" ::: "memory"); break;
    case 4: asm volatile("cp.async.wait_group 4;" ::: "memory"); break;
    case 5: asm volatile("cp.async.wait_group 5;" ::: "memory"); break;
    case 6: asm volatile("cp.async.wait_group 6;" ::: "memory"); break;
    default: asm volatile("cp.async.wait_group 7;" ::: "memory"); break;
    }
}

#ifdef QM_DEBUG
__device__ __forceinline__ unsigned long long gtime() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
#endif
// Debug builds only (-DQM_DEBUG, a.debug == 9): phase timestamps of op a.debug_slot for the
// first and last CTA.
#ifdef QM_DEBUG
#define QM_MARK(k)                                                                          \
    do {                                                                                    \
        if (a.debug == 9 && lane == 0 && mark_op == a.debug_slot &&                        \
            (blockIdx.x == 0 || blockIdx.x == gridDim.x - 1))                               \
            reinterpret_cast<unsigned long long *>(a.status + 16)[((blockIdx.x != 0) * 16 + warp) * 8 + (k)] = gtime(); \
    } while (0)
#define QM_DEBUG_IS(v) (a.debug == (v))
#else
#define QM_MARK(k) do { } while (0)
#define QM_DEBUG_IS(v) false
#endif

constexpr int kRowTab = 64;     // bytes of one row of the per-warp scale table
constexpr int kTabBytes = 16 * kRowTab;

// A stage holds one item of the store: 16 headers of 16 bytes, then for each of the four
// 32-byte quant groups p the 16 rows side by side — so the 8-byte reads of four rows at a
// time cover 128 contiguous bytes and the copy from HBM is one contiguous 2304-byte run.
constexpr int kStageBytes = QM_Q4K_ITEM_BYTES;
constexpr int kCopiesPerLane = (kStageBytes / 16 + 31) / 32;   // 16-byte pieces of a stage per lane

struct Cursor {   // walks the items of this warp, op after op
    int op;
    int i, hi;            // current item and end of the warp's range in op
    int tile, u, units;   // position and K units of the op's slice
    const uint8_t *src;   // store address of the current item
    int64_t tile_skip;    // bytes from the end of a tile's slice to the start of the next tile's
};

// Quantizes the 256 activations of row j, unit ul (eight per lane, v) into limbs and writes
// them, their sub-block sums and the column weights in the layout the main loop reads; the
// destination is shared memory or an activation image. Returns this lane's sum of squares.
// NAT: the weights keep the order of the GGUF block (mma k index i <-> element i of the sub-block), as
// the Q4_0 / Q8_0 stores do; otherwise k index 4t+i <-> element 8t+i, 16+4t+i <-> element 8t+4+i, the
// order of the tiled Q4_K store.
template <int NT, bool NAT = false>
__device__ __forceinline__ float quantize_pair(const float (&v)[8], int j, int ul, int lane, int NL, int CPM,
                                               uint8_t *xs_b, int pstride, uint32_t *xsum_b, float *sxw_b,
                                               float wmul = 1.f) {
    float amax = 0.f, sum = 0.f, sq = 0.f;
#pragma unroll
    for (int e = 0; e < 8; e++) { amax = fmaxf(amax, fabsf(v[e])); sum += v[e]; sq = fmaf(v[e], v[e], sq); }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    sum += __shfl_xor_sync(0xffffffffu, sum, 1);
    sum += __shfl_xor_sync(0xffffffffu, sum, 2);
    const float sx = amax > 0.f ? amax * (1.f / 127.f) : 1.f;
    const float inv = amax > 0.f ? 127.f / amax : 0.f;
    // Limbs by magic-number rounding: adding 1.5*2^23 rounds to the nearest integer and
    // leaves it (two's complement) in the low mantissa bits — no conversion instructions.
    uint32_t hb[8], l1b[8], l2b[8];
    constexpr float kMagicF = 12582912.f;
#pragma unroll
    for (int e = 0; e < 8; e++) {
        const float r = v[e] * inv;
        const float t0 = r + kMagicF;
        const float r1 = (r - (t0 - kMagicF)) * 128.f;
        const float t1 = r1 + kMagicF;
        const float r2 = (r1 - (t1 - kMagicF)) * 128.f;
        const float t2 = r2 + kMagicF;
        hb[e] = __float_as_uint(t0);
        l1b[e] = __float_as_uint(t1);
        l2b[e] = __float_as_uint(t2);
    }
    auto pack4 = [](uint32_t b0, uint32_t b1, uint32_t b2, uint32_t b3) -> uint32_t {
        return prmt(prmt(b0, b1, 0x0040u), prmt(b2, b3, 0x0040u), 0x5410u);  // low bytes of the four
    };
    const uint32_t w0[3] = {pack4(hb[0], hb[1], hb[2], hb[3]), pack4(l1b[0], l1b[1], l1b[2], l1b[3]),
                            pack4(l2b[0], l2b[1], l2b[2], l2b[3])};
    const uint32_t w1[3] = {pack4(hb[4], hb[5], hb[6], hb[7]), pack4(l1b[4], l1b[5], l1b[6], l1b[7]),
                            pack4(l2b[4], l2b[5], l2b[6], l2b[7])};
    // lane = 4*sub-block + t': this lane's 8 columns are the B fragment of lane t' for
    // sub-block sb; the fragments of sub-blocks 2p and 2p+1 sit side by side
    const int sb = lane >> 2, tq = lane & 3;
    if (NAT) {
        // elements 8tq..8tq+3 are register b[tq >> 1] of lane t' = 2*(tq & 1), the next four that of lane t' + 1
        const int off = ((ul * 4 + (sb >> 1)) * 4 + 2 * (tq & 1)) * 16 + (sb & 1) * 8 + (tq >> 1) * 4;
        for (int l = 0; l < NL; l++) {
            uint8_t *pl = xs_b + (size_t)(j * NL + l) * pstride + off;
            *reinterpret_cast<uint32_t *>(pl) = w0[l];
            *reinterpret_cast<uint32_t *>(pl + 16) = w1[l];
        }
    } else {
        const int off = ((ul * 4 + (sb >> 1)) * 4 + tq) * 16 + (sb & 1) * 8;
        for (int l = 0; l < NL; l++)
            *reinterpret_cast<uint2 *>(xs_b + (size_t)(j * NL + l) * pstride + off) = make_uint2(w0[l], w1[l]);
    }
    const int n0 = j * CPM;   // first mma column of this activation row
    if (tq == 0) {
        // sub-block sums in units of the unit's maximum (|.| <= 32): safe in fp16 whatever
        // the magnitude of the activations; the factor comes back with the column weight
        const float sn = sum * inv * (1.f / 127.f);
        const __half sh = __float2half_rn(sn);
        const __half sl = __float2half_rn(sn - __half2float(sh));
        __half *xh = reinterpret_cast<__half *>(xsum_b);
        xh[((size_t)ul * 8 * NT + n0) * 8 + sb] = sh;
        xh[((size_t)ul * 8 * NT + n0 + 1) * 8 + sb] = sl;
    }
    if (lane < CPM) {
        const float lw = lane == 0 ? 1.f : lane == 1 ? (1.f / 128.f) : lane == 2 && NL == 3 ? (1.f / 16384.f) : 0.f;
        sxw_b[(size_t)ul * 8 * NT + n0 + lane] = sx * lw * wmul;   // wmul: a constant the consumer folds into the column weight
    }
    return sq;
}

// One warp writes activation row j of unit u of the next op's activation image:
// x = y[u] (+ y[half + u] when the next op adds two halves of y). Called outside the streaming
// loop only, so that it does not cost the loop its registers.
template <int NT>
__device__ __noinline__ void quantize_row(const float *y, int64_t ldy, int u, int j, int NL, int CPM, int halves,
                                          int half_tiles, uint8_t *img, int img_plane_stride, size_t off_xsum,
                                          size_t off_sxw, size_t off_ssq) {
    const int lane = threadIdx.x & 31;
    const float *xp = y + (int64_t)j * ldy + u * QM_K_UNIT + lane * 8;
    const float4 r0 = __ldcg(reinterpret_cast<const float4 *>(xp));
    const float4 r1 = __ldcg(reinterpret_cast<const float4 *>(xp + 4));
    float v[8] = {r0.x, r0.y, r0.z, r0.w, r1.x, r1.y, r1.z, r1.w};
    if (halves == 2) {
        const float *x2p = xp + (int64_t)half_tiles * 16;
        const float4 s0 = __ldcg(reinterpret_cast<const float4 *>(x2p));
        const float4 s1 = __ldcg(reinterpret_cast<const float4 *>(x2p + 4));
        v[0] += s0.x; v[1] += s0.y; v[2] += s0.z; v[3] += s0.w;
        v[4] += s1.x; v[5] += s1.y; v[6] += s1.z; v[7] += s1.w;
    }
    float sq = quantize_pair<NT>(v, j, u, lane, NL, CPM, img, img_plane_stride,
                                 reinterpret_cast<uint32_t *>(img + off_xsum), reinterpret_cast<float *>(img + off_sxw));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
    if (lane == 0) reinterpret_cast<float *>(img + off_ssq)[u * 8 + j] = sq;
}

template <int NT, bool IMG, bool TP>
__device__ __forceinline__ void fused_body(const QmFusedArgs &a) {
    extern __shared__ __align__(128) uint8_t smem[];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, t = lane & 3;
    const int C = a.consumers, D = a.depth, M = a.m, CPM = a.cpm;
    const int nthreads = C * 32;
    const int NL = CPM == 4 ? 3 : 2;            // limbs per activation row
    const int P = M * NL;                        // stored activation planes
    const QmOp *ops = a.ops ? a.ops : a.inl;

    // ---- shared memory carve-up (qm_plan_fused on the host computes the same sizes) -------
    const int plane_stride = a.max_units * 256 + 64;
    uint8_t *xs = smem;                                                             // [P][plane_stride]
    uint32_t *xsum = reinterpret_cast<uint32_t *>(xs + (size_t)P * plane_stride);    // [units][8NT][4]
    float *sxw = reinterpret_cast<float *>(xsum + (size_t)a.max_units * 8 * NT * 4); // [units][8NT]
    uint8_t *tabs = reinterpret_cast<uint8_t *>(sxw + (size_t)a.max_units * 8 * NT); // [C][kTabBytes]
    float *red = reinterpret_cast<float *>(tabs + (size_t)C * kTabBytes);            // [32][8]
    float *s_scale = red + 32 * 8;                                                   // [8]
    constexpr int stage_bytes = kStageBytes;
    float *ssq = s_scale + 8;                                                        // [8][16]
    float *slots = ssq + 8 * 16;                                    // [C][2][M*16]
    uint8_t *stages = reinterpret_cast<uint8_t *>(((uintptr_t)(slots + (size_t)C * 2 * M * 16) + 127) & ~(uintptr_t)127);  // [C][D]
    uint8_t *my_stages = stages + (size_t)warp * D * stage_bytes;
    uint8_t *my_tab = tabs + (size_t)warp * kTabBytes;

#ifdef QM_DEBUG
    int mark_op = -1;
#endif
    asm volatile("griddepcontrol.launch_dependents;");
    // columns of absent activation rows and pad columns must read as zero
    for (int i = tid; i < a.max_units * 8 * NT * 5; i += nthreads) xsum[i] = 0u;   // xsum and sxw are adjacent
    __syncthreads();

    // This warp's share of an op: warps are numbered warp-major over the CTAs so that a short
    // op still spreads over all SMs; every busy warp owns at least one item.
    // CTA-local item range [lo, hi) of this warp and first tile of the CTA's run
    // This CTA's run of an op in global item coordinates: first item and item count.
    auto cta_run = [&](const QmOp &op, unsigned int &cbase, unsigned int &Ic) {
        const int c = (int)blockIdx.x;
        const unsigned int first = (unsigned int)(c * op.q + min(c, op.rem));
        const unsigned int count = (unsigned int)(op.q + (c < op.rem ? 1 : 0));
        if (op.balanced) { cbase = first; Ic = count; }
        else { cbase = first * (unsigned int)op.units; Ic = count * (unsigned int)op.units; }
    };
    // Item range [lo, hi) of this warp in coordinates that start at the first item of tile0 (the
    // tile holding the CTA's first item): the CTA's own run is [off0, off0 + Ic).
    auto op_range = [&](const QmOp &op, int &lo, int &hi, int &tile0, int &wq, int &wrem, int &off0, int &Ic_) {
        unsigned int cbase, Ic;
        cta_run(op, cbase, Ic);
        tile0 = (int)(cbase / (unsigned int)op.units);
        off0 = (int)(cbase - (unsigned int)tile0 * (unsigned int)op.units);
        Ic_ = (int)Ic;
        wq = (int)(Ic / (unsigned int)C);
        wrem = (int)(Ic - (unsigned int)wq * (unsigned int)C);
        lo = off0 + warp * wq + min(warp, wrem);
        hi = lo + wq + (warp < wrem ? 1 : 0);
    };
    auto cursor_at = [&](Cursor &c, int op) {
        c.op = op;
        c.i = c.hi = 0;
        c.tile = c.u = 0;
        c.units = 1;
        c.src = nullptr;
        c.tile_skip = 0;
        if (op < a.nops) {
            const QmOp o = ops[op];   // by value: the fields live in registers from here on
            int lo, hi, tile0, wq, wrem, off0, Ic;
            op_range(o, lo, hi, tile0, wq, wrem, off0, Ic);
            c.i = lo;
            c.hi = hi;
            c.units = o.units;
            c.tile = (int)((unsigned)lo / (unsigned)o.units);   // CTA-local tile
            c.u = lo - c.tile * o.units;
            c.src = o.wq + ((int64_t)(tile0 + c.tile) * o.units_total + o.unit0 + c.u) * QM_Q4K_ITEM_BYTES;
            c.tile_skip = (int64_t)(o.units_total - o.units) * QM_Q4K_ITEM_BYTES;
        }
    };
    auto cursor_skip_empty = [&](Cursor &c) {
        while (c.op < a.nops && c.i >= c.hi) cursor_at(c, c.op + 1);
    };

    // ---- producer side of the ring ----------------------------------------------------------
    Cursor ic;
    cursor_at(ic, 0);
    cursor_skip_empty(ic);
    int islot = 0;
    // Starts the copy of the next item into ring slot `islot` and commits one group; commits an
    // empty group when the warp has nothing left, so that group counting stays uniform.
    auto issue = [&]() {
        if (ic.op < a.nops) {
            const uint32_t dst = smem_u32(my_stages + (size_t)islot * stage_bytes) + lane * 16;
            const uint8_t *src = ic.src + lane * 16;
            if (!QM_DEBUG_IS(3)) {
#pragma unroll
                for (int k = 0; k < kCopiesPerLane; k++)
                    if (lane + 32 * k < kStageBytes / 16) cp_async16(dst + 512 * k, src + 512 * k);
            }
            ic.i += 1;
            ic.u += 1;
            ic.src += QM_Q4K_ITEM_BYTES;
            if (ic.u == ic.units) { ic.u = 0; ic.tile++; ic.src += ic.tile_skip; }
            cursor_skip_empty(ic);
        }
        cp_async_commit();
        islot = islot + 1 == D ? 0 : islot + 1;
    };
    for (int d = 0; d < D; d++) issue();
    asm volatile("griddepcontrol.wait;" ::: "memory");

    // ---- lane roles on the activation side ---------------------------------------------------
    // mma column n = 8*nt + g holds limb (n % CPM) of activation row (n / CPM).
    bool bact[NT], mact[NT];
    const uint8_t *bplane[NT];
#pragma unroll
    for (int nt = 0; nt < NT; nt++) {
        const int n = 8 * nt + g, j = n / CPM, l = n - j * CPM;
        bact[nt] = j < M && l < NL;
        mact[nt] = j < M && l < 2;
        bplane[nt] = xs + (size_t)(bact[nt] ? j * NL + l : 0) * plane_stride + t * 16;
    }

    int cslot = 0;
    Cursor cc;
    cursor_at(cc, 0);

    // Layout of an activation image in global memory: the limb planes with room for
    // a.img_units units each, then the sub-block sums, the column weights and the sums of squares
    // per (unit, activation row).
    const int img_plane_stride = a.img_units * 256 + 64;
    const size_t img_off_xsum = (size_t)P * img_plane_stride;
    const size_t img_off_sxw = img_off_xsum + (size_t)a.img_units * 8 * NT * 16;
    const size_t img_off_ssq = img_off_sxw + (size_t)a.img_units * 8 * NT * 4;

    auto quant_pair = [&](const float (&v)[8], int j, int ul, uint8_t *xs_b, int pstride, uint32_t *xsum_b,
                          float *sxw_b) -> float {
        return quantize_pair<NT>(v, j, ul, lane, NL, CPM, xs_b, pstride, xsum_b, sxw_b);
    };
    // Producer side of the activation image: called by a warp after its final stores (or adds)
    // to tile `gtile` of y. `add` is 2 when the warp completed the whole tile and 1 when it is
    // one of the two CTAs that share it. The warp that brings a unit's counter to its full count
    // quantizes the unit for every activation row.
    // The image fields of an op are read where they are needed (once per finished tile), not
    // kept in registers through the streaming loop.
    auto arrive = [&](int opi, int gtile, unsigned int add) -> int {
        if (!IMG) return -1;
        const QmOp *po = ops + opi;
        unsigned int *cnt = po->q_cnt;
        if (!cnt) return -1;
        const int half_tiles = po->q_half_tiles, halves = po->q_halves;
        if (gtile >= half_tiles * halves) return -1;    // rows that the next op does not read
        const int half = gtile >= half_tiles ? 1 : 0;
        const int u = (gtile - half * half_tiles) >> 4;
        const int tiles_in_unit = min(16, half_tiles - 16 * u);
        const unsigned int full = 2u * (unsigned int)(tiles_in_unit * halves);
        __threadfence();
        __syncwarp();
        unsigned int old = 0;
        if (lane == 0) old = atomicAdd(cnt + u, add);
        old = __shfl_sync(0xffffffffu, old, 0);
        return old + add == full ? u : -1;
    };
    // Units completed by this CTA's warps wait in a short shared list (the reduction scratch is
    // free between staging and the next op); after the CTA's last stores all warps share the
    // (unit, activation row) pairs, so the tail is one row per warp, not a unit per warp.
    int *done = reinterpret_cast<int *>(red);
    constexpr int kDoneCap = 31;
    auto quantize_rows = [&](int opi, int u, int j0, int j1) {
        const QmOp *po = ops + opi;
        const float *y = po->y;
        const int64_t ldy = po->ldy;
        const int halves = po->q_halves, half_tiles = po->q_half_tiles;
        uint8_t *img = po->q_img;
        for (int j = j0; j < j1; j++)
            quantize_row<NT>(y, ldy, u, j, NL, CPM, halves, half_tiles, img, img_plane_stride, img_off_xsum,
                             img_off_sxw, img_off_ssq);
    };
    auto note_done = [&](int opi, int du) {
        if (du < 0) return;
        int slot = 0;
        if (lane == 0) slot = atomicAdd(&done[0], 1);
        slot = __shfl_sync(0xffffffffu, slot, 0);
        if (slot < kDoneCap) {
            if (lane == 0) done[1 + slot] = du;
        } else {
            quantize_rows(opi, du, 0, M);   // list full: this warp does the unit alone
        }
    };

    // Barrier over all CTAs (and, tensor-parallel, over all GPUs). Every wait is bounded: after
    // about two seconds the CTA records QM_STATUS_TIMEOUT, stops waiting at this and all later
    // barriers, and runs to the end.
    bool dead = false;   // meaningful in thread 0
    unsigned int nloc = 0, ncross = 0;   // barriers so far on the local counter / over all GPUs
    auto grid_sync = [&](bool cross) {
        if (TP && cross && a.tp_counter) {
            // Counter form: every CTA adds its arrival to the counter word of every GPU's arena
            // (its own included) and waits until its own counter has seen all CTAs of all GPUs.
            // The count grows from launch to launch; the comparison is wrap-safe.
            if (tid == 0) {
                __threadfence_system();
                unsigned int *cnt = a.tp_flags + 32;
                for (int p = 0; p < a.tp_world; p++)
                    red_add_release_sys(reinterpret_cast<unsigned int *>(reinterpret_cast<char *>(cnt) + a.peer_delta[p]), 1u);
                const unsigned int target = a.tp_epoch0 + (ncross + 1) * gridDim.x * (unsigned int)a.tp_world;
                const long long t0 = clock64();
                while (!dead && (int)(ld_acquire_sys(cnt) - target) < 0) {
                    if (clock64() - t0 > a.wait_cycles) {
                        atomicOr(a.status, QM_STATUS_TIMEOUT);
                        dead = true;
                    }
                }
            }
            ncross++;
            __syncthreads();
            return;
        }
        if (tid == 0) {
            if (TP && cross) __threadfence_system(); else __threadfence();
            const unsigned int target = (nloc + 1) * gridDim.x;
            const unsigned int old = atomicAdd(a.grid_bar, 1u);
            const unsigned int epoch = a.tp_epoch0 + ncross + 1;
            if (TP && cross && old + 1 == target) {   // this GPU's slice is complete: tell the peers
                __threadfence_system();
                for (int p = 0; p < a.tp_world; p++)
                    if (p != a.tp_rank)
                        st_release_sys(reinterpret_cast<unsigned int *>(
                                           reinterpret_cast<char *>(a.tp_flags + a.tp_rank) + a.peer_delta[p]), epoch);
            }
            const long long t0 = clock64();
            while (!dead && ld_acquire(a.grid_bar) < target) {
                if (clock64() - t0 > a.wait_cycles) {
                    atomicOr(a.status, QM_STATUS_TIMEOUT);
                    dead = true;
                }
            }
            if (TP && cross) {
                for (int p = 0; p < a.tp_world; p++) {
                    if (p == a.tp_rank) continue;
                    while (!dead && (int)(ld_acquire_sys(a.tp_flags + p) - epoch) < 0) {
                        if (clock64() - t0 > a.wait_cycles) {
                            atomicOr(a.status, QM_STATUS_TIMEOUT);
                            dead = true;
                        }
                    }
                }
            }
        }
        nloc++;
        if (TP && cross) ncross++;
        __syncthreads();
    };
    // Stores a finished output; for an op that is shared between the GPUs also into every peer's arena.
    bool share_cur = false;
    auto store_y = [&](float *yp, float val) {
        *yp = val;
        if (TP && share_cur) {
            for (int p = 0; p < a.tp_world; p++)
                if (p != a.tp_rank) *reinterpret_cast<float *>(reinterpret_cast<char *>(yp) + a.peer_delta[p]) = val;
        }
    };

    for (int opi = 0; opi < a.nops; opi++) {
        const QmOp op = ops[opi];   // by value: no reloads through the generic pointer
#ifdef QM_DEBUG
        mark_op = opi;
#endif
        QM_MARK(0);
        const int nun = op.units;
        // ---- wait for the producers of x, and for this CTA's readers of the old planes --------
        if (opi > 0) {
            __syncthreads();
            // the barrier spans the GPUs when the op before this one was shared between them
            if (op.barrier) grid_sync(TP && (ops + opi - 1)->tp_shared != 0);
        }
        share_cur = TP && op.tp_shared != 0;
        QM_MARK(1);
        // ---- quantize the activations of this op into limbs, once per CTA ---------------------
        // Tiles of the NEXT op that this CTA will share with a neighbour are added to with
        // red.global.add: zero them now, a whole grid barrier before anybody adds.
        if (opi + 1 < a.nops) {
            const QmOp nx = ops[opi + 1];
            if (nx.balanced && tid < 2 * 16 * M) {
                unsigned int cb, ic;
                cta_run(nx, cb, ic);
                const unsigned int un = (unsigned int)nx.units;
                const unsigned int edge = (tid >= 16 * M) ? cb + ic : cb;   // tail, head
                if (ic > 0 && edge % un != 0) {
                    const int tl = (int)((tid >= 16 * M ? edge - 1 : edge) / un);
                    const int o = tid % (16 * M), r = tl * 16 + (o & 15);
                    if (r < nx.rows) nx.y[(int64_t)(o >> 4) * nx.ldy + r] = 0.f;
                }
            }
        }
        // RMS normalisation is a scalar per activation row, so it commutes with the product:
        // the raw activations are quantized and the scale is applied to the finished sums.
        // The sum of squares is collected per K unit while staging (one pass over x); only an
        // op that covers a slice of K needs a pass of its own over the whole row.
        const bool norm = (op.xop == 1 || op.xop == 2);
        const bool sliced = op.units != op.units_total;
        const uint8_t *op_img = IMG ? (ops + opi)->img : nullptr;
        const bool pre = op_img != nullptr;
        if (norm && sliced && !pre) {
            for (int j = 0; j < M; j++) {
                float s = 0.f;
                const float *xr = op.x + (int64_t)j * op.ldx;
                const float *x2r = op.x2 ? op.x2 + (int64_t)j * op.ldx : nullptr;
                for (int c = tid * 4; c < op.cols; c += nthreads * 4) {
                    float4 v4 = __ldcg(reinterpret_cast<const float4 *>(xr + c));
                    if (op.xop == 2) {
                        const float4 w = __ldcg(reinterpret_cast<const float4 *>(x2r + c));
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
            if (tid < M) {
                float s = 0.f;
                for (int w = 0; w < C; w++) s += red[w * 8 + tid];
                s_scale[tid] = rsqrtf(s / (float)op.cols + op.eps);
            }
            __syncthreads();
        }
        // the loads of the next (row, unit) pair are in flight while this one is quantized
        auto load_raw = [&](int idx, float4 (&r)[4]) {
            const int j = idx / nun, ul = idx - j * nun;
            const int col = (op.unit0 + ul) * QM_K_UNIT + lane * 8;
            const float *xp = op.x + (int64_t)j * op.ldx + col;
            r[0] = __ldcg(reinterpret_cast<const float4 *>(xp));
            r[1] = __ldcg(reinterpret_cast<const float4 *>(xp + 4));
            if (op.xop >= 2) {
                const float *x2p = op.x2 + (int64_t)j * op.ldx + col;
                r[2] = __ldcg(reinterpret_cast<const float4 *>(x2p));
                r[3] = __ldcg(reinterpret_cast<const float4 *>(x2p + 4));
            }
        };
        if (!pre) {
            float4 raw[4], raw_next[4];
            float sq_run = 0.f;
            int sq_j = -1;
            if (norm && !sliced && lane < 8) ssq[lane * 16 + warp] = 0.f;
            __syncwarp();
            if (warp < M * nun) load_raw(warp, raw);
            for (int idx = warp; idx < M * nun; idx += C) {
                const int j = idx / nun, ul = idx - j * nun;
                if (idx + C < M * nun) load_raw(idx + C, raw_next);
                float v[8] = {raw[0].x, raw[0].y, raw[0].z, raw[0].w, raw[1].x, raw[1].y, raw[1].z, raw[1].w};
                if (op.xop >= 2) {
                    const float w[8] = {raw[2].x, raw[2].y, raw[2].z, raw[2].w, raw[3].x, raw[3].y, raw[3].z, raw[3].w};
#pragma unroll
                    for (int e = 0; e < 8; e++)
                        v[e] = op.xop == 2 ? v[e] + w[e] : v[e] / (1.f + __expf(-v[e])) * w[e];
                }
#pragma unroll
                for (int e = 0; e < 4; e++) raw[e] = raw_next[e];
                const float sq = quant_pair(v, j, ul, xs, plane_stride, xsum, sxw);
                if (norm && !sliced) {   // per-warp running sum of squares of activation row j
                    if (j != sq_j) {
                        if (sq_j >= 0) {
#pragma unroll
                            for (int o = 16; o > 0; o >>= 1) sq_run += __shfl_xor_sync(0xffffffffu, sq_run, o);
                            if (lane == 0) ssq[sq_j * 16 + warp] = sq_run;
                        }
                        sq_j = j;
                        sq_run = 0.f;
                    }
                    sq_run += sq;
                }
            }
            if (sq_j >= 0) {
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) sq_run += __shfl_xor_sync(0xffffffffu, sq_run, o);
                if (lane == 0) ssq[sq_j * 16 + warp] = sq_run;
            }
        } else {
            // ---- the previous op left the quantized x in global memory: copy this slice in -------
            const uint8_t *img = op_img;
            const int nplanes = M * NL;
            const int per_plane = nun * 16;                       // 16-byte pieces of a plane's slice
            const int n_xs = nplanes * per_plane, n_sum = nun * 8 * NT, n_w = nun * 2 * NT;
            const uint4 *g_xsum = reinterpret_cast<const uint4 *>(img + img_off_xsum) + (size_t)op.unit0 * 8 * NT;
            const uint4 *g_sxw = reinterpret_cast<const uint4 *>(img + img_off_sxw) + (size_t)op.unit0 * 2 * NT;
            // sixteen-byte asynchronous copies: nothing is staged in registers. They form a commit
            // group of their own behind the ring's groups; waiting for all groups costs nothing here,
            // the ring's copies were started before the grid barrier.
            const uint8_t *img_xs = img + (size_t)op.unit0 * 256;
            for (int i = tid; i < n_xs; i += nthreads) {
                const int pl = i / per_plane, kk = i - pl * per_plane;
                cp_async16(smem_u32(xs + (size_t)pl * plane_stride + (size_t)kk * 16),
                           img_xs + (size_t)pl * img_plane_stride + (size_t)kk * 16);
            }
            for (int i = tid; i < n_sum + n_w; i += nthreads) {
                if (i < n_sum) cp_async16(smem_u32(reinterpret_cast<uint4 *>(xsum) + i), g_xsum + i);
                else cp_async16(smem_u32(reinterpret_cast<uint4 *>(sxw) + (i - n_sum)), g_sxw + (i - n_sum));
            }
            cp_async_commit();
            asm volatile("cp.async.wait_group 0;" ::: "memory");
            if (norm && tid < M) {   // sum of squares of row tid: the units' parts in unit order
                const float *g_ssq = reinterpret_cast<const float *>(img + img_off_ssq);
                float sq = 0.f;
                for (int u = 0; u < op.units_total; u++) sq += __ldcg(g_ssq + u * 8 + tid);
                s_scale[tid] = rsqrtf(sq / (float)op.cols + op.eps);
            }
        }
        if (IMG && tid == 0) done[0] = 0;
        __syncthreads();

        float myscale[NT];
#pragma unroll
        for (int nt = 0; nt < NT; nt++) myscale[nt] = 1.f;
        if (norm) {
            for (int j = 0; j < M; j++) {
                float sc;
                if (sliced || pre) {
                    sc = s_scale[j];
                } else {
                    // the warps' parts, added as a fixed tree over sixteen lanes
                    float sq = (lane & 15) < C ? ssq[j * 16 + (lane & 15)] : 0.f;
#pragma unroll
                    for (int o = 8; o > 0; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
                    sc = rsqrtf(sq / (float)op.cols + op.eps);
                }
#pragma unroll
                for (int nt = 0; nt < NT; nt++)
                    if ((CPM == 4 ? 2 * nt + (t >> 1) : 4 * nt + t) == j) myscale[nt] = sc;
            }
        }
        QM_MARK(2);
        // ---- stream this warp's chunks of the op ---------------------------------------------------
        int lo, hi, tile0, wq, wrem, off0, Ic;
        op_range(op, lo, hi, tile0, wq, wrem, off0, Ic);
        if (cc.op != opi) cursor_at(cc, opi);
        int fin_tile = -1;   // CTA-local tile this warp finishes after the barrier
        float accF[NT][4];
#pragma unroll
        for (int nt = 0; nt < NT; nt++) accF[nt][0] = accF[nt][1] = accF[nt][2] = accF[nt][3] = 0.f;
        int cur_tile = cc.tile;

        auto flush = [&](int tile) {
            // per activation row: sum of its CPM columns; lanes t hold columns 2t, 2t+1
            float vA[NT], vB[NT];
            int jrow[NT];
            bool valid[NT];
#pragma unroll
            for (int nt = 0; nt < NT; nt++) {
                vA[nt] = accF[nt][0] + accF[nt][1];
                vB[nt] = accF[nt][2] + accF[nt][3];
                if (CPM == 4) {
                    vA[nt] += __shfl_xor_sync(0xffffffffu, vA[nt], 1);
                    vB[nt] += __shfl_xor_sync(0xffffffffu, vB[nt], 1);
                    jrow[nt] = 2 * nt + (t >> 1);
                    valid[nt] = (t & 1) == 0 && jrow[nt] < M;
                } else {
                    jrow[nt] = 4 * nt + t;
                    valid[nt] = jrow[nt] < M;
                }
                vA[nt] *= myscale[nt];
                vB[nt] *= myscale[nt];
            }
            // the part of the tile inside this CTA's run; `whole` when that is all of it
            const int ts = max(tile * nun, off0), te = min(tile * nun + nun, off0 + Ic);
            const bool whole = te - ts == nun;
            const bool from_start = lo <= ts, to_end = hi >= te;
            if (from_start && to_end) {   // this warp had all of the CTA's part of the tile
                const int rA = (tile0 + tile) * 16 + g, rB = rA + 8;
#pragma unroll
                for (int nt = 0; nt < NT; nt++)
                    if (valid[nt]) {
                        float *yA = op.y + (int64_t)jrow[nt] * op.ldy + rA, *yB = yA + 8;
                        if (whole) {
                            if (rA < op.rows) store_y(yA, vA[nt] + (op.accumulate ? __ldcg(yA) : 0.f));
                            if (rB < op.rows) store_y(yB, vB[nt] + (op.accumulate ? __ldcg(yB) : 0.f));
                        } else {   // the tile is shared with a neighbouring CTA
                            if (rA < op.rows) atomicAdd(yA, vA[nt]);
                            if (rB < op.rows) atomicAdd(yB, vB[nt]);
                        }
                    }
                // a unit that this store completed is quantized by the CTA after its last stores
                const int du = arrive(opi, tile0 + tile, whole ? 2u : 1u);
                note_done(opi, du);
                return;
            }
            // slot 1: this warp's range ends inside the tile; slot 0: it joined the tile late and
            // reaches its end, so it adds up the tile after the barrier
            float *p = slots + ((size_t)warp * 2 + (to_end ? 0 : 1)) * M * 16;
#pragma unroll
            for (int nt = 0; nt < NT; nt++)
                if (valid[nt]) { p[jrow[nt] * 16 + g] = vA[nt]; p[jrow[nt] * 16 + g + 8] = vB[nt]; }
            if (to_end) fin_tile = tile;
        };

        // per-warp scale table of unit `un` of the landed stage, built by all 32 lanes:
        // lane = 2*row + half handles sub-blocks 4*half .. 4*half+3 of its row
        auto build_table = [&](const uint8_t *stage, uint8_t *tab) {
            const int row = lane >> 1, half = lane & 1;
            const uint4 hdr = *reinterpret_cast<const uint4 *>(stage + row * 16);
            const uint32_t S0 = hdr.y, S1 = hdr.z, S2 = hdr.w;
            const uint32_t scv = half == 0 ? (S0 & 0x3F3F3F3Fu) : ((S2 & 0x0F0F0F0Fu) | ((S0 >> 2) & 0x30303030u));
            const uint32_t mv = half == 0 ? (S1 & 0x3F3F3F3Fu) : (((S2 >> 4) & 0x0F0F0F0Fu) | ((S1 >> 2) & 0x30303030u));
            uint8_t *r = tab + row * kRowTab;
            // even sub-blocks (low nibbles) carry a factor 16 so that they add up with the odd ones,
            // whose nibbles stay in place and are sixteen times too large
            *reinterpret_cast<uint4 *>(r + half * 16) =
                make_uint4((scv & 0xFF) << 4, (scv >> 8) & 0xFF, ((scv >> 16) & 0xFF) << 4, scv >> 24);
            const uint32_t m01 = hsub2(prmt(mv, 0x64646464u, 0x4140u), 0x64006400u);
            const uint32_t m23 = hsub2(prmt(mv, 0x64646464u, 0x4342u), 0x64006400u);
            *reinterpret_cast<uint2 *>(r + 32 + half * 8) = make_uint2(m01, m23);
            if (half == 0) {
                const float d = __half2float(__ushort_as_half((unsigned short)(hdr.x & 0xFFFFu)));
                const float dmin = __half2float(__ushort_as_half((unsigned short)(hdr.x >> 16)));
                *reinterpret_cast<float2 *>(r + 48) = make_float2(d, dmin);
            }
        };

        while (cc.op == opi && cc.i < cc.hi) {
            if (cc.tile != cur_tile) {
                flush(cur_tile);
#pragma unroll
                for (int nt = 0; nt < NT; nt++) accF[nt][0] = accF[nt][1] = accF[nt][2] = accF[nt][3] = 0.f;
                cur_tile = cc.tile;
            }
            // the oldest of the D groups in flight is this unit; the copies of every lane are
            // visible to the whole warp once all lanes have waited
            cp_async_wait(D - 1);
            __syncwarp();
            const uint8_t *stage = my_stages + (size_t)cslot * stage_bytes;
            if (!QM_DEBUG_IS(1)) {   // debug builds: 1 = copies only, no arithmetic
                const uint8_t *tab = my_tab;
                build_table(stage, my_tab);
                __syncwarp();
                const int ul = cc.u;
                // scales of this lane's two rows
                const uint4 sA0 = *reinterpret_cast<const uint4 *>(tab + g * kRowTab);
                const uint4 sA1 = *reinterpret_cast<const uint4 *>(tab + g * kRowTab + 16);
                const uint4 sB0 = *reinterpret_cast<const uint4 *>(tab + (g + 8) * kRowTab);
                const uint4 sB1 = *reinterpret_cast<const uint4 *>(tab + (g + 8) * kRowTab + 16);
                const int scA[8] = {(int)sA0.x, (int)sA0.y, (int)sA0.z, (int)sA0.w, (int)sA1.x, (int)sA1.y, (int)sA1.z, (int)sA1.w};
                const int scB[8] = {(int)sB0.x, (int)sB0.y, (int)sB0.z, (int)sB0.w, (int)sB1.x, (int)sB1.y, (int)sB1.z, (int)sB1.w};
                int accI[NT][4];   // sixteen times the scaled integer sums: < 2^30
#pragma unroll
                for (int nt = 0; nt < NT; nt++)
#pragma unroll
                    for (int c = 0; c < 4; c++) accI[nt][c] = 0;
                const uint8_t *rowA = stage + 256 + 32 * g + 8 * t;
                const uint8_t *rowB = rowA + 256;
#pragma unroll
                for (int p = 0; p < 4; p++) {
                    const uint2 wA = *reinterpret_cast<const uint2 *>(rowA + 512 * p);
                    const uint2 wB = *reinterpret_cast<const uint2 *>(rowB + 512 * p);
                    const uint32_t a0 = wA.x & 0x0F0F0F0Fu, a1 = wB.x & 0x0F0F0F0Fu;
                    const uint32_t a2 = wA.y & 0x0F0F0F0Fu, a3 = wB.y & 0x0F0F0F0Fu;
                    const uint32_t h0 = wA.x & 0xF0F0F0F0u, h1 = wB.x & 0xF0F0F0F0u;
                    const uint32_t h2 = wA.y & 0xF0F0F0F0u, h3 = wB.y & 0xF0F0F0F0u;
#pragma unroll
                    for (int nt = 0; nt < NT; nt++) {
                        uint4 b = make_uint4(0, 0, 0, 0);
                        if (bact[nt]) b = *reinterpret_cast<const uint4 *>(bplane[nt] + (ul * 4 + p) * 64);
                        int S[4];
                        mma_u8s8(S, a0, a1, a2, a3, b.x, b.y);
                        accI[nt][0] += scA[2 * p] * S[0];
                        accI[nt][1] += scA[2 * p] * S[1];
                        accI[nt][2] += scB[2 * p] * S[2];
                        accI[nt][3] += scB[2 * p] * S[3];
                        mma_u8s8(S, h0, h1, h2, h3, b.z, b.w);   // sixteen times the sub-block sums
                        accI[nt][0] += scA[2 * p + 1] * S[0];
                        accI[nt][1] += scA[2 * p + 1] * S[1];
                        accI[nt][2] += scB[2 * p + 1] * S[2];
                        accI[nt][3] += scB[2 * p + 1] * S[3];
                    }
                }
                const uint32_t mpA = *reinterpret_cast<const uint32_t *>(tab + g * kRowTab + 32 + 4 * t);
                const uint32_t mpB = *reinterpret_cast<const uint32_t *>(tab + (g + 8) * kRowTab + 32 + 4 * t);
                const float2 ddA = *reinterpret_cast<const float2 *>(tab + g * kRowTab + 48);
                const float2 ddB = *reinterpret_cast<const float2 *>(tab + (g + 8) * kRowTab + 48);
#pragma unroll
                for (int nt = 0; nt < NT; nt++) {
                    const float2 cw = *reinterpret_cast<const float2 *>(sxw + (size_t)ul * 8 * NT + 8 * nt + 2 * t);
                    float accM[4];
                    const uint32_t bm = mact[nt] ? xsum[((size_t)ul * 8 * NT + 8 * nt + g) * 4 + t] : 0u;
                    mma_f16(accM, mpA, mpB, bm);
                    const float f0 = (float)accI[nt][0] * 0.0625f, f1 = (float)accI[nt][1] * 0.0625f;
                    const float f2 = (float)accI[nt][2] * 0.0625f, f3 = (float)accI[nt][3] * 0.0625f;
                    // even column: first limb / high half of the sums, weight sx; odd column:
                    // second limb / low half, weight sx/128; the sums are in units of 127*sx
                    const float mx = 127.f * cw.x, my = 16256.f * cw.y;
                    accF[nt][0] = fmaf(ddA.x * cw.x, f0, fmaf(-ddA.y * mx, accM[0], accF[nt][0]));
                    accF[nt][1] = fmaf(ddA.x * cw.y, f1, fmaf(-ddA.y * my, accM[1], accF[nt][1]));
                    accF[nt][2] = fmaf(ddB.x * cw.x, f2, fmaf(-ddB.y * mx, accM[2], accF[nt][2]));
                    accF[nt][3] = fmaf(ddB.x * cw.y, f3, fmaf(-ddB.y * my, accM[3], accF[nt][3]));
                }
                __syncwarp();   // all lanes are done with the table before it is rebuilt
            }
            cc.i += 1;
            cc.u += 1;
            if (cc.u == nun) { cc.u = 0; cc.tile++; }
            cslot = cslot + 1 == D ? 0 : cslot + 1;
            // every lane's reads of the slot have returned (their values were consumed above):
            // after the warp converges the next copy may overwrite it
            __syncwarp();
            issue();
        }
        if (lo < hi) flush(cur_tile);
        QM_MARK(3);
        __syncthreads();
        QM_MARK(4);
        if (fin_tile >= 0) {
            // partial sums of the warps that worked on the tile before this one, in warp order
            const int tsf = max(fin_tile * nun, off0);
            const bool whole = min(fin_tile * nun + nun, off0 + Ic) - tsf == nun;
            const unsigned int ts = (unsigned int)(tsf - off0), big = (unsigned int)wrem * (unsigned int)(wq + 1);
            const int wf = wq == 0 ? (int)ts : ts < big ? (int)(ts / (unsigned int)(wq + 1))
                                                         : wrem + (int)((ts - big) / (unsigned int)wq);
            for (int o = lane; o < 16 * M; o += 32) {
                float sum = 0.f;
                for (int x = wf; x < warp; x++) sum += slots[((size_t)x * 2 + 1) * M * 16 + o];
                sum += slots[(size_t)warp * 2 * M * 16 + o];
                const int j = o >> 4, r = (tile0 + fin_tile) * 16 + (o & 15);
                float *yp = op.y + (int64_t)j * op.ldy + r;
                if (r < op.rows) {
                    if (whole) store_y(yp, sum + (op.accumulate ? __ldcg(yp) : 0.f));
                    else atomicAdd(yp, sum);
                }
            }
            const int du = arrive(opi, tile0 + fin_tile, whole ? 2u : 1u);
            note_done(opi, du);
        }
        if (IMG && (ops + opi)->q_cnt) {
            __syncthreads();
            const int n = min(done[0], kDoneCap);
            for (int idx = warp; idx < n * M; idx += C) {
                const int k = idx / M, j = idx - k * M;
                quantize_rows(opi, done[1 + k], j, j + 1);
            }
        }
        QM_MARK(5);
    }
    // Tensor-parallel: the launch ends only when every GPU's last slice has arrived everywhere,
    // so that the host may read the outputs and the next launch may overwrite the inputs.
    if (TP) {
        __syncthreads();
        grid_sync(true);
    }
}


// ---------------------------------------------------------------------------------------------
// Data-driven decode step for up to four activation rows (kernels qm_fused_q4k_dd*).
//
// Dependent matvecs are not separated by a grid barrier. Every output buffer of the launch
// holds the "not yet written" pattern when the launch starts (the host fills them), a consumer
// staging x polls the very words it needs until none of them holds the pattern, and a producer
// simply stores its results: a value that has arrived is its own flag. The chain
// store -> fence -> counter -> poll -> load of a barrier becomes store -> load. It needs whole
// tiles per CTA (no adds from two CTAs into one output), no K slices, and an output buffer of
// its own for every op.
//
// The body is specialised at compile time (sixteen warps, D ring stages, CPM mma columns per
// activation row) and keeps the per-item instruction count low, because at batch 1 the
// streaming loop is bound by instruction issue, not by HBM: the scales of a lane's two rows are
// unpacked in registers (no shared table, no extra warp barriers), sub-blocks in the high
// nibbles accumulate separately and are divided by 16 once per unit, every lane reads a valid
// activation plane (columns without an activation row carry a zero column weight instead of a
// predicate), and the producer side is a pointer and a count.
// ---------------------------------------------------------------------------------------------
// Accesses of the hand-over: strong (gpu scope) relaxed loads and stores that go to L2, where
// every SM sees them.
__device__ __forceinline__ float4 ld_relaxed_v4(const float *p) {
    float4 v;
    asm volatile("ld.relaxed.gpu.global.v4.f32 {%0,%1,%2,%3}, [%4];"
                 : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
                 : "l"(p)
                 : "memory");
    return v;
}
__device__ __forceinline__ void st_relaxed_f32(float *p, float v) {
    asm volatile("st.relaxed.gpu.global.f32 [%0], %1;" ::"l"(p), "f"(v) : "memory");
}
// System scope: the other party is another GPU (tensor-parallel launches).
__device__ __forceinline__ float4 ld_relaxed_sys_v4(const float *p) {
    float4 v;
    asm volatile("ld.relaxed.sys.global.v4.f32 {%0,%1,%2,%3}, [%4];"
                 : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
                 : "l"(p)
                 : "memory");
    return v;
}
__device__ __forceinline__ void st_relaxed_sys_f32(float *p, float v) {
    asm volatile("st.relaxed.sys.global.f32 [%0], %1;" ::"l"(p), "f"(v) : "memory");
}
// "Not yet written": a NaN that no arithmetic here produces (sums of products give the canonical
// quiet NaN; fp16 scales widen to NaNs whose low 13 bits are zero).
constexpr uint32_t kUnwritten = 0xFFFFFFFFu;
__device__ __forceinline__ bool written4(const float4 &v) {
    return (__float_as_uint(v.x) != kUnwritten) & (__float_as_uint(v.y) != kUnwritten) &
           (__float_as_uint(v.z) != kUnwritten) & (__float_as_uint(v.w) != kUnwritten);
}
template <typename T>
__device__ __forceinline__ T *ldg_ptr(T *const *p) {   // read-only load of a pointer field
    return reinterpret_cast<T *>(__ldg(reinterpret_cast<const unsigned long long *>(p)));
}
template <int N>
__device__ __forceinline__ void cp_async_wait_n() {
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

// Stages the x of one op for this CTA: polls the words until the producers have written them,
// adds the partial vectors of a producer that ran in K parts, applies the input transform and
// quantizes into limb planes, sub-block sums and column weights; leaves each warp's part of the
// sums of squares in ssq. Returns the thread's "gave up waiting" flag.
template <int CPM, bool TP, int NT = 1>
__device__ __forceinline__ bool dd_stage(const QmFusedArgs *ap, const QmOp *po, uint8_t *xs, int plane_stride,
                                      uint32_t *xsum, float *sxw, float *ssq, bool dead) {
    const QmFusedArgs &a = *ap;
    constexpr int C = 16, NL = CPM == 4 ? 3 : 2;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int M = a.m;
    const int nun = po->units, xop = po->xop;
    const float *opx = po->x, *opx2 = po->x2;
    const int64_t ldx = po->ldx;
    const bool norm = xop == 1 || xop == 2;
    const int x_parts = po->x_parts;
    const int col0 = po->unit0 * QM_K_UNIT;   // first column of this op's K range
    const int64_t xps = po->x_part_stride;
    {
            const int total = M * nun;
            const bool poll = po->barrier != 0;   // x is an earlier op's output
            float sq_run = 0.f;
            int sq_j = -1;
            if (norm && lane < 8) ssq[lane * 16 + warp] = 0.f;
            __syncwarp();
            auto load_x = [&](int idx, float4 (&r)[4]) {
                const int j = idx / nun, ul = idx - j * nun;
                const float *xp = opx + (int64_t)j * ldx + col0 + ul * QM_K_UNIT + lane * 8;
                r[0] = TP ? ld_relaxed_sys_v4(xp) : ld_relaxed_v4(xp);
                r[1] = TP ? ld_relaxed_sys_v4(xp + 4) : ld_relaxed_v4(xp + 4);
                if (xop >= 2) {
                    const float *x2p = opx2 + (int64_t)j * ldx + col0 + ul * QM_K_UNIT + lane * 8;
                    r[2] = TP ? ld_relaxed_sys_v4(x2p) : ld_relaxed_v4(x2p);
                    r[3] = TP ? ld_relaxed_sys_v4(x2p + 4) : ld_relaxed_v4(x2p + 4);
                }
            };
            // x given as several partial vectors (the producer was cut into K parts): all of them are
            // in flight at once, one (row, unit) pair per warp and round
            if (x_parts > 1) {
                for (int idx = warp; idx < total; idx += C) {
                    const int j = idx / nun, ul = idx - j * nun;
                    const float *xp = opx + (int64_t)j * ldx + col0 + ul * QM_K_UNIT + lane * 8;
                    float4 r[8];
                    long long t0 = 0;
                    for (;;) {
                        bool ok = true;
#pragma unroll
                        for (int k = 0; k < 4; k++)
                            if (k < x_parts) {
                                r[2 * k] = TP ? ld_relaxed_sys_v4(xp + k * xps) : ld_relaxed_v4(xp + k * xps);
                                r[2 * k + 1] = TP ? ld_relaxed_sys_v4(xp + k * xps + 4) : ld_relaxed_v4(xp + k * xps + 4);
                            }
#pragma unroll
                        for (int k = 0; k < 4; k++)
                            if (k < x_parts) ok = ok & written4(r[2 * k]) & written4(r[2 * k + 1]);
                        if (__all_sync(0xffffffffu, ok || dead)) break;
                        if (t0 == 0) t0 = clock64();
                        else if (clock64() - t0 > a.wait_cycles) {
                            if (lane == 0) atomicOr(a.status, QM_STATUS_TIMEOUT);
                            dead = true;
                        }
                    }
                    float v[8] = {r[0].x, r[0].y, r[0].z, r[0].w, r[1].x, r[1].y, r[1].z, r[1].w};
#pragma unroll
                    for (int k = 1; k < 4; k++)
                        if (k < x_parts) {   // the parts in order: the same sum on every CTA and GPU
                            v[0] += r[2 * k].x; v[1] += r[2 * k].y; v[2] += r[2 * k].z; v[3] += r[2 * k].w;
                            v[4] += r[2 * k + 1].x; v[5] += r[2 * k + 1].y; v[6] += r[2 * k + 1].z; v[7] += r[2 * k + 1].w;
                        }
                    if (TP && x_parts > 4) {
                        // tensor-parallel lists have up to eight partial vectors (one per GPU): the second four
                        for (;;) {
                            bool ok = true;
#pragma unroll
                            for (int k = 0; k < 4; k++)
                                if (4 + k < x_parts) {
                                    r[2 * k] = ld_relaxed_sys_v4(xp + (4 + k) * xps);
                                    r[2 * k + 1] = ld_relaxed_sys_v4(xp + (4 + k) * xps + 4);
                                }
#pragma unroll
                            for (int k = 0; k < 4; k++)
                                if (4 + k < x_parts) ok = ok & written4(r[2 * k]) & written4(r[2 * k + 1]);
                            if (__all_sync(0xffffffffu, ok || dead)) break;
                            if (t0 == 0) t0 = clock64();
                            else if (clock64() - t0 > a.wait_cycles) {
                                if (lane == 0) atomicOr(a.status, QM_STATUS_TIMEOUT);
                                dead = true;
                            }
                        }
#pragma unroll
                        for (int k = 0; k < 4; k++)
                            if (4 + k < x_parts) {
                                v[0] += r[2 * k].x; v[1] += r[2 * k].y; v[2] += r[2 * k].z; v[3] += r[2 * k].w;
                                v[4] += r[2 * k + 1].x; v[5] += r[2 * k + 1].y; v[6] += r[2 * k + 1].z; v[7] += r[2 * k + 1].w;
                            }
                    }
                    const float sq = quantize_pair<NT>(v, j, ul, lane, NL, CPM, xs, plane_stride, xsum, sxw, 0.0625f);
                    if (norm) {
                        if (j != sq_j) {
                            if (sq_j >= 0) {
#pragma unroll
                                for (int o = 16; o > 0; o >>= 1) sq_run += __shfl_xor_sync(0xffffffffu, sq_run, o);
                                if (lane == 0) ssq[sq_j * 16 + warp] = sq_run;
                            }
                            sq_j = j;
                            sq_run = 0.f;
                        }
                        sq_run += sq;
                    }
                }
            } else {
            // Two register sets alternate: while one (row, unit) pair is quantized the loads of the
            // next pair but one are in flight, so only the first wait of an op is fully exposed.
            auto consume = [&](int idx, float4 (&r)[4]) {
                if (poll) {
                    long long t0 = 0;
                    for (;;) {
                        bool ok = written4(r[0]) & written4(r[1]);
                        if (xop >= 2) ok = ok & written4(r[2]) & written4(r[3]);
                        if (__all_sync(0xffffffffu, ok || dead)) break;
                        if (t0 == 0) t0 = clock64();
                        else if (clock64() - t0 > a.wait_cycles) {
                            if (lane == 0) atomicOr(a.status, QM_STATUS_TIMEOUT);
                            dead = true;   // this and every later wait of the thread give up at once
                        }
                        load_x(idx, r);
                    }
                }
                const int j = idx / nun, ul = idx - j * nun;
                float v[8] = {r[0].x, r[0].y, r[0].z, r[0].w, r[1].x, r[1].y, r[1].z, r[1].w};
                if (xop >= 2) {
                    const float w[8] = {r[2].x, r[2].y, r[2].z, r[2].w, r[3].x, r[3].y, r[3].z, r[3].w};
#pragma unroll
                    for (int e = 0; e < 8; e++)
                        v[e] = xop == 2 ? v[e] + w[e] : v[e] / (1.f + __expf(-v[e])) * w[e];
                }
                const float sq = quantize_pair<NT>(v, j, ul, lane, NL, CPM, xs, plane_stride, xsum, sxw, 0.0625f);
                if (norm) {   // per-warp running sum of squares of activation row j
                    if (j != sq_j) {
                        if (sq_j >= 0) {
#pragma unroll
                            for (int o = 16; o > 0; o >>= 1) sq_run += __shfl_xor_sync(0xffffffffu, sq_run, o);
                            if (lane == 0) ssq[sq_j * 16 + warp] = sq_run;
                        }
                        sq_j = j;
                        sq_run = 0.f;
                    }
                    sq_run += sq;
                }
            };
            {
                float4 rawA[4], rawB[4];
                if (warp < total) load_x(warp, rawA);
                if (warp + C < total) load_x(warp + C, rawB);
                for (int idx = warp; idx < total; idx += 2 * C) {
                    consume(idx, rawA);
                    if (idx + 2 * C < total) load_x(idx + 2 * C, rawA);
                    if (idx + C < total) {
                        consume(idx + C, rawB);
                        if (idx + 3 * C < total) load_x(idx + 3 * C, rawB);
                    }
                }
            }
            }
            if (sq_j >= 0) {
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) sq_run += __shfl_xor_sync(0xffffffffu, sq_run, o);
                if (lane == 0) ssq[sq_j * 16 + warp] = sq_run;
            }
    }
    return dead;
}

// TP (tensor parallel): this GPU computes a row slice of every op and stores each result into
// the same place of every GPU's activation arena (plain peer stores over NVLink); consumers
// poll their own arena only, so no barrier crosses the GPUs inside a step. One barrier over the
// GPUs ends the launch: when it returns, every slice of the step has arrived everywhere, which
// is what lets the host refill the other arena half with the "not yet written" pattern.
// NT = column tiles of eight mma columns: 1, or 2 with CPM = 2 for five to eight activation rows (each weight
// fragment then feeds two mma, one per tile; the low- and high-nibble sums share one accumulator).
template <int CPM, int D, bool TP, bool SEL = false, int NT = 1>
__device__ __forceinline__ void dd_body(const QmFusedArgs &a) {
    constexpr int C = 16;                       // warps per CTA
    constexpr int NL = CPM == 4 ? 3 : 2;        // limbs per activation row
    extern __shared__ __align__(128) uint8_t smem[];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, t = lane & 3;
    const int M = a.m, P = M * NL;
    const bool inl = a.ops == nullptr;   // a single matvec: its few ops travel in the launch parameters

    // ---- shared memory (qm_plan_fused computes an upper bound of this) -------------------------
    const int plane_stride = a.max_units * 256 + 64;
    uint8_t *xs = smem;                                                            // [P][plane_stride]
    uint32_t *xsum = reinterpret_cast<uint32_t *>(xs + (size_t)P * plane_stride);   // [units][8*NT][4] f16 pairs
    float *sxw = reinterpret_cast<float *>(xsum + (size_t)a.max_units * 8 * NT * 4);   // [units][8*NT] column weights
    float *ssq = sxw + (size_t)a.max_units * 8 * NT;                                // [8][16]
    float *slots = ssq + 8 * 16;                                                    // [C][2][M*16]
    QmOp *sop = reinterpret_cast<QmOp *>(((uintptr_t)(slots + (size_t)C * 2 * M * 16) + 15) & ~(uintptr_t)15);   // [2], or [nops] inline
    uint8_t *stages = reinterpret_cast<uint8_t *>(((uintptr_t)(sop + (inl ? QM_MAX_INLINE_OPS : 2)) + 127) & ~(uintptr_t)127);
    uint8_t *my_stages = stages + (size_t)warp * D * kStageBytes;

    asm volatile("griddepcontrol.launch_dependents;");
    // columns of absent activation rows and pad columns must read as zero weights and sums
    for (int i = tid; i < a.max_units * 8 * NT * 5; i += C * 32) xsum[i] = 0u;   // xsum and sxw are adjacent
    // inline ops: all of them into shared memory, where the producer side reads ahead too
    if (inl)
        for (int i = tid; i < a.nops * (int)(sizeof(QmOp) / 16); i += C * 32)
            reinterpret_cast<uint4 *>(sop)[i] = reinterpret_cast<const uint4 *>(a.inl)[i];
    __syncthreads();
    // K parts: the CTAs form a.ngroups groups and each group runs its own copy of the op list (the
    // copies differ only in the ops that are cut into parts)
    const int ngroups = a.ngroups > 1 && !inl ? a.ngroups : 1;
    const QmOp *ops = inl ? sop : a.ops + (size_t)((int)blockIdx.x / ((int)gridDim.x / ngroups)) * a.nops;

    // This warp's items of op `o`: the CTA owns a run of whole tiles, its items are dealt evenly to
    // the warps in order. Returns the first item and the count in CTA-local coordinates.
    // An op cut into K parts splits the CTAs into as many groups; `c` is then the CTA's index within
    // its group (q and rem are computed for the group's size).
    auto warp_range = [&](int q, int rem, int units, int c, int nctas, int &tile0, int &lo, int &n, int &wq, int &wrem) {
        tile0 = c * q + min(c, rem);
        const int Ic = (c >= 0 && c < nctas) ? (q + (c < rem ? 1 : 0)) * units : 0;
        wq = Ic / C;
        wrem = Ic - wq * C;
        lo = warp * wq + min(warp, wrem);
        n = wq + (warp < wrem ? 1 : 0);
    };

    // ---- producer side of the ring: a pointer and a count per op -------------------------------
    // (a warp's items of an op are one contiguous run of the store)
    int p_op = -1, p_n = 0;
    const uint8_t *p_src = nullptr;
    auto p_next_op = [&]() {
        p_n = 0;
        for (p_op++; p_op < a.nops; p_op++) {
            const QmOp *po = ops + p_op;
            int tile0, lo, n, wq, wrem;
            const int units = po->units;
            warp_range(po->q, po->rem, units, (int)blockIdx.x - po->cta0, po->nctas, tile0, lo, n, wq, wrem);
            if (n > 0) {
                p_n = n;
                const uint8_t *wq = po->wq;
                if (SEL && po->sel_table) {   // the slot's expert, known on the device only
                    const int id = po->sel_ids[po->sel_index];
                    wq = po->sel_table[min(max(id, 0), po->sel_count - 1)];
                }
                p_src = wq + ((int64_t)tile0 * units + lo) * QM_Q4K_ITEM_BYTES + lane * 16;
                break;
            }
        }
    };
    const uint32_t ring0 = smem_u32(my_stages) + lane * 16;
    uint32_t p_dst = ring0;
    auto issue = [&]() {
        if (p_n > 0) {
            cp_async16(p_dst, p_src);
            cp_async16(p_dst + 512, p_src + 512);
            cp_async16(p_dst + 1024, p_src + 1024);
            cp_async16(p_dst + 1536, p_src + 1536);
            if (lane < 16) cp_async16(p_dst + 2048, p_src + 2048);
            p_src += QM_Q4K_ITEM_BYTES;
            if (--p_n == 0) p_next_op();
        }
        cp_async_commit();
        p_dst = p_dst + kStageBytes == ring0 + D * kStageBytes ? ring0 : p_dst + kStageBytes;
    };
    p_next_op();
#pragma unroll
    for (int d = 0; d < D; d++) issue();

    // mma column n = g holds limb (n % CPM) of activation row (n / CPM); lanes whose column has no
    // row read plane 0 (their column weight is zero)
    const int col_row = g / CPM, col_limb = g - col_row * CPM;
    const bool col_on = col_row < M && col_limb < NL;
    const uint8_t *bplane = xs + (size_t)(col_on ? col_row * NL + col_limb : 0) * plane_stride + t * 16;
    // second column tile (NT == 2): mma column 8 + g = limb (g % 2) of activation row 4 + g / 2
    const bool col2_on = NT == 2 && 4 + g / 2 < M;
    const uint8_t *bplane2 = xs + (size_t)(col2_on ? (4 + g / 2) * NL + (g & 1) : 0) * plane_stride + t * 16;
    // byte selector that brings the minima of sub-blocks 2t and 2t+1 (of the eight in two words)
    // to the low half of a word
    const uint32_t min_sel = (uint32_t)(2 * t) | ((uint32_t)(2 * t + 1) << 4) | 0x4400u;

    const uint8_t *c_stage = my_stages;   // consumer slot
    bool dead = false;
#ifdef QM_DEBUG
    // debug builds, a.debug == 9: time stamps of every op's phases as seen by thread 0 of the first and last CTA
#define QM_DD_MARK(k)                                                                                             \
    do {                                                                                                          \
        if (a.debug == 9 && tid == 0 && (blockIdx.x == 0 || blockIdx.x == gridDim.x - 1) && opi < 480)            \
            reinterpret_cast<unsigned long long *>(a.status + 16)[(opi * 2 + (blockIdx.x != 0)) * 4 + (k)] = gtime(); \
        /* a.debug == 10: every CTA's stamps of the four ops of layer a.debug_slot */                             \
        if (a.debug == 10 && tid == 0 && (opi >> 2) == a.debug_slot && gridDim.x <= 200)                          \
            reinterpret_cast<unsigned long long *>(a.status + 16)[(((opi & 3) * gridDim.x) + blockIdx.x) * 4 + (k)] = gtime(); \
    } while (0)
#else
#define QM_DD_MARK(k) do { } while (0)
#endif

    // The descriptor of the current op is read from shared memory; a warp copies the next op's
    // there while the current one streams.
    static_assert(sizeof(QmOp) % 16 == 0, "QmOp is copied in 16-byte pieces");
    if (!inl && warp == 0 && lane < (int)(sizeof(QmOp) / 16))
        reinterpret_cast<uint4 *>(&sop[0])[lane] = __ldg(reinterpret_cast<const uint4 *>(ops) + lane);
    // the activations of a launch's first op may come from the launch before it in the stream
    asm volatile("griddepcontrol.wait;" ::: "memory");

    for (int opi = 0; opi < a.nops; opi++) {
        const QmOp *po = inl ? &sop[opi] : &sop[opi & 1];
        QM_DD_MARK(0);
        // every warp has finished with the activation planes and the partial sums of the op before
        __syncthreads();
        const int nun = po->units;
        const int xop = po->xop;
        const bool norm = xop == 1 || xop == 2;
        const int parts = po->parts, x_parts = po->x_parts;
        const int cta_in_grp = (int)blockIdx.x - po->cta0;

        const float *ssq_in = po->ssq_in;
        // The words of a producer that ran in K parts (its sums of squares per part and row): every lane reads
        // ONE word — part lane / 8 (and that plus four, with more than four parts), row lane % 8 — so that all of
        // them cost one trip to L2, not one each; the loads are issued here and their values looked at after x has
        // been staged (the producer published them when it started, long before its outputs).
        float ssq_w0 = 0.f, ssq_w1 = 0.f;
        const bool want_w0 = norm && ssq_in && parts == 1 && (lane >> 3) < x_parts && (lane & 7) < M;
        const bool want_w1 = TP && norm && ssq_in && parts == 1 && (lane >> 3) + 4 < x_parts && (lane & 7) < M;
        auto load_word = [&](int k) -> float {
            float part;
            if (TP) asm volatile("ld.relaxed.sys.global.f32 %0, [%1];" : "=f"(part) : "l"(ssq_in + k * 8 + (lane & 7)) : "memory");
            else asm volatile("ld.relaxed.gpu.global.f32 %0, [%1];" : "=f"(part) : "l"(ssq_in + k * 8 + (lane & 7)) : "memory");
            return part;
        };
        if (want_w0) ssq_w0 = load_word(lane >> 3);
        if (want_w1) ssq_w1 = load_word((lane >> 3) + 4);
        // ---- stage x: poll until written, quantize into limbs --------------------------------------
        dead = dd_stage<CPM, TP, NT>(&a, po, xs, plane_stride, xsum, sxw, ssq, dead);
        {   // a word that had not been written yet: wait for it (bounded)
            auto settle = [&](float &w, int k) {
                long long t0 = 0;
                while (__float_as_uint(w) == kUnwritten && !dead) {
                    if (t0 == 0) t0 = clock64();
                    else if (clock64() - t0 > a.wait_cycles) {
                        atomicOr(a.status, QM_STATUS_TIMEOUT);
                        dead = true;
                    }
                    w = load_word(k);
                }
            };
            if (want_w0) settle(ssq_w0, lane >> 3);
            if (want_w1) settle(ssq_w1, (lane >> 3) + 4);
        }
        __syncthreads();
        QM_DD_MARK(1);
        if (!inl && warp == C - 1 && opi + 1 < a.nops && lane < (int)(sizeof(QmOp) / 16))
            reinterpret_cast<uint4 *>(&sop[(opi + 1) & 1])[lane] = __ldg(reinterpret_cast<const uint4 *>(ops + opi + 1) + lane);

        // RMS normalisation is a scalar per activation row: it multiplies the finished sums
        float myscale = 1.f, myscale2 = 1.f;   // myscale2: the row of the second column tile
        if (norm) {
            const float inv_cols = 1.f / (float)po->cols;
            float *ssq_out = po->ssq_out;
            for (int j = 0; j < M; j++) {
                float sq = ssq[j * 16 + (lane & 15)];   // the warps' parts, added as a fixed tree
#pragma unroll
                for (int o = 8; o > 0; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
                if (parts > 1) {
                    // a K part leaves its products unscaled; the consumer scales the sum. One CTA of the
                    // group publishes the part's sum of squares.
                    if (cta_in_grp == 0 && tid == 0) {
                        float *word = ssq_out + po->part * 8 + j;
                        if (TP && (po->tp_shared & 1)) {   // a GPU's K part: every GPU's consumers read the word
                            for (int p = 0; p < a.tp_world; p++)
                                st_relaxed_sys_f32(reinterpret_cast<float *>(reinterpret_cast<char *>(word) + a.peer_delta[p]), sq);
                        } else {
                            st_relaxed_f32(word, sq);
                        }
                    }
                    continue;
                }
                float eps = po->eps;
                if (ssq_in) {
                    // x is c times the sum that was staged, c = rsqrt(ms + eps') of the producer's input:
                    // normalising c*v with eps equals normalising v with eps / c^2
                    float ms = 0.f;   // the parts in order: the same sum on every CTA and GPU
                    for (int k = 0; k < x_parts && k < 4; k++) ms += __shfl_sync(0xffffffffu, ssq_w0, k * 8 + j);
                    if (TP)
                        for (int k = 4; k < x_parts; k++) ms += __shfl_sync(0xffffffffu, ssq_w1, (k - 4) * 8 + j);
                    eps *= ms * po->ssq_in_inv_cols + po->ssq_in_eps;
                }
                const float sc = rsqrtf(sq * inv_cols + eps);
                if ((CPM == 4 ? (t >> 1) : t) == j) myscale = sc;
                if (NT == 2 && 4 + t == j) myscale2 = sc;
            }
        }

        // ---- stream this warp's items of the op ---------------------------------------------------
        int tile0, lo, n;
        {
            int wq_, wrem_;
            warp_range(po->q, po->rem, nun, cta_in_grp, po->nctas, tile0, lo, n, wq_, wrem_);
        }
        float *opy = po->y;
        const int64_t ldy = po->ldy;
        const int rows = po->rows;
        const int hi = lo + n;
        int fin_tile = -1;   // CTA-local tile this warp adds up after the CTA barrier

        // Tensor-parallel lists: rows from split_row on go to a second output (q|k|v and gate|up slices that are
        // two row ranges of the full vector); tp_shared bit 0 / bit 1 = the first / second output goes to every
        // GPU's arena, otherwise to this GPU's only.
        // (read from the descriptor in shared memory where they are used: the streaming loop has no register to spare)
        auto store_y = [&](float *yp, float val, bool share) {   // a result must never look like "not yet written"
            if (__float_as_uint(val) == kUnwritten) val = __uint_as_float(0x7FC00000u);
            if (TP && share) {
                for (int p = 0; p < a.tp_world; p++)   // the same place of every GPU's arena, this one included
                    st_relaxed_sys_f32(reinterpret_cast<float *>(reinterpret_cast<char *>(yp) + a.peer_delta[p]), val);
            } else if (TP) {
                st_relaxed_sys_f32(yp, val);
            } else {
                st_relaxed_f32(yp, val);
            }
        };
        // Ends a tile's segment [s0, s1) of this warp: stores the outputs if the warp had the whole
        // tile, else leaves its partial sums for the warp that reaches the tile's end.
        auto flush = [&](int tile, int s0, int s1, const float (&accF)[4], const float (&accF2)[4]) {
            float vA = accF[0] + accF[1], vB = accF[2] + accF[3];
            int jrow;
            bool valid;
            if (CPM == 4) {
                vA += __shfl_xor_sync(0xffffffffu, vA, 1);
                vB += __shfl_xor_sync(0xffffffffu, vB, 1);
                jrow = t >> 1;
                valid = (t & 1) == 0 && jrow < M;
            } else {
                jrow = t;
                valid = jrow < M;
            }
            vA *= myscale;
            vB *= myscale;
            // second column tile: activation row 4 + t
            float vA2 = 0.f, vB2 = 0.f;
            const bool valid2 = NT == 2 && 4 + t < M;
            if (NT == 2) {
                vA2 = (accF2[0] + accF2[1]) * myscale2;
                vB2 = (accF2[2] + accF2[3]) * myscale2;
            }
            const bool from_start = s0 == tile * nun, to_end = s1 == tile * nun + nun;
            if (from_start && to_end) {
                const int rA = (tile0 + tile) * 16 + g, rB = rA + 8;
                if (valid || valid2) {
                    const int split = TP ? po->split_row : 0;
                    const bool second = TP && split > 0 && (tile0 + tile) * 16 >= split;   // whole tiles on either side
                    float *y0 = (second ? po->y2 - split : opy) + rA;
                    const bool share = TP && (po->tp_shared & (second ? 2 : 1)) != 0;
                    if (valid) {
                        float *yA = y0 + (int64_t)jrow * ldy;
                        if (rA < rows) store_y(yA, vA, share);
                        if (rB < rows) store_y(yA + 8, vB, share);
                    }
                    if (valid2) {
                        float *yA = y0 + (int64_t)(4 + t) * ldy;
                        if (rA < rows) store_y(yA, vA2, share);
                        if (rB < rows) store_y(yA + 8, vB2, share);
                    }
                }
                return;
            }
            // slot 1: the segment ends inside the tile; slot 0: it joined the tile late and reaches
            // its end, so this warp adds the tile up after the barrier
            float *p = slots + ((size_t)warp * 2 + (to_end ? 0 : 1)) * M * 16;
            if (valid) { p[jrow * 16 + g] = vA; p[jrow * 16 + g + 8] = vB; }
            if (valid2) { p[(4 + t) * 16 + g] = vA2; p[(4 + t) * 16 + g + 8] = vB2; }
            if (to_end) fin_tile = tile;
        };

        const uint8_t *bp = bplane;                 // activation limbs of the current unit
        const float *cwp = sxw + 2 * t;             // column weights of the current unit
        const uint32_t *bmp = xsum + g * 4 + t;     // sub-block sums of the current unit
        for (int i = lo; i < hi;) {
            const int tile = i / nun, u0 = i - tile * nun;
            const int seg_end = min(hi, (tile + 1) * nun);
            float accF[4] = {0.f, 0.f, 0.f, 0.f}, accF2[4] = {0.f, 0.f, 0.f, 0.f};
            bp = bplane + (size_t)u0 * 256;
            cwp = sxw + (size_t)u0 * 8 * NT + 2 * t;
            bmp = xsum + (size_t)u0 * 32 * NT + g * 4 + t;
            for (int k = i; k < seg_end; k++) {
                cp_async_wait_n<D - 1>();   // the oldest of the D groups in flight is this item
                __syncwarp();               // ... and every lane's copies of it have landed
                const uint8_t *stage = c_stage;
                // ---- scales of this lane's rows g and g+8 -------------------------------------------
                const uint4 hA = *reinterpret_cast<const uint4 *>(stage + 16 * g);
                const uint4 hB = *reinterpret_cast<const uint4 *>(stage + 16 * g + 128);
                const uint32_t scA0 = hA.y & 0x3F3F3F3Fu, scA1 = (hA.w & 0x0F0F0F0Fu) | ((hA.y >> 2) & 0x30303030u);
                const uint32_t scB0 = hB.y & 0x3F3F3F3Fu, scB1 = (hB.w & 0x0F0F0F0Fu) | ((hB.y >> 2) & 0x30303030u);
                const uint32_t mnA0 = hA.z & 0x3F3F3F3Fu, mnA1 = ((hA.w >> 4) & 0x0F0F0F0Fu) | ((hA.z >> 2) & 0x30303030u);
                const uint32_t mnB0 = hB.z & 0x3F3F3F3Fu, mnB1 = ((hB.w >> 4) & 0x0F0F0F0Fu) | ((hB.z >> 2) & 0x30303030u);
                if constexpr (NT == 1) {
                    int accL[4] = {0, 0, 0, 0}, accH[4] = {0, 0, 0, 0};   // low-nibble / high-nibble sub-blocks
                    const uint8_t *rowA = stage + 256 + 32 * g + 8 * t;
    #pragma unroll
                    for (int p = 0; p < 4; p++) {
                        const uint2 wA = *reinterpret_cast<const uint2 *>(rowA + 512 * p);
                        const uint2 wB = *reinterpret_cast<const uint2 *>(rowA + 512 * p + 256);
                        const uint4 b = *reinterpret_cast<const uint4 *>(bp + 64 * p);
                        // sub-block 2p in the low nibbles, 2p+1 in the high ones (left in place: x16)
                        const int sAl = (int)__byte_perm(p < 2 ? scA0 : scA1, 0, 0x4440 + ((2 * p) & 3));
                        const int sAh = (int)__byte_perm(p < 2 ? scA0 : scA1, 0, 0x4440 + ((2 * p + 1) & 3));
                        const int sBl = (int)__byte_perm(p < 2 ? scB0 : scB1, 0, 0x4440 + ((2 * p) & 3));
                        const int sBh = (int)__byte_perm(p < 2 ? scB0 : scB1, 0, 0x4440 + ((2 * p + 1) & 3));
                        int S[4];
                        mma_u8s8(S, wA.x & 0x0F0F0F0Fu, wB.x & 0x0F0F0F0Fu, wA.y & 0x0F0F0F0Fu, wB.y & 0x0F0F0F0Fu, b.x, b.y);
                        accL[0] += sAl * S[0];
                        accL[1] += sAl * S[1];
                        accL[2] += sBl * S[2];
                        accL[3] += sBl * S[3];
                        mma_u8s8(S, wA.x & 0xF0F0F0F0u, wB.x & 0xF0F0F0F0u, wA.y & 0xF0F0F0F0u, wB.y & 0xF0F0F0F0u, b.z, b.w);
                        accH[0] += sAh * S[0];
                        accH[1] += sAh * S[1];
                        accH[2] += sBh * S[2];
                        accH[3] += sBh * S[3];
                    }
                    // ---- minima: one f16 mma against the sub-block sums of the activations -----------------
                    const uint32_t mpA = hsub2(__byte_perm(__byte_perm(mnA0, mnA1, min_sel), 0x64646464u, 0x4140), 0x64006400u);
                    const uint32_t mpB = hsub2(__byte_perm(__byte_perm(mnB0, mnB1, min_sel), 0x64646464u, 0x4140), 0x64006400u);
                    float accM[4];
                    mma_f16(accM, mpA, mpB, *bmp);
                    // ---- per-unit float32 scaling -------------------------------------------------------
                    const float2 ddA = __half22float2(*reinterpret_cast<const __half2 *>(&hA.x));   // d, dmin of row g
                    const float2 ddB = __half22float2(*reinterpret_cast<const __half2 *>(&hB.x));
                    const float2 cw = *reinterpret_cast<const float2 *>(cwp);
                    // even column: first limb / high half of the sums, weight sx; odd column: second limb /
                    // low half, weight sx/128; the sums are in units of 127*sx. The column weights come
                    // divided by 16: the integer sums are taken as 16*low + high (below 2^29).
                    const float mx = 2032.f * cw.x, my = 260096.f * cw.y;
                    const float f0 = (float)(accL[0] * 16 + accH[0]), f1 = (float)(accL[1] * 16 + accH[1]);
                    const float f2 = (float)(accL[2] * 16 + accH[2]), f3 = (float)(accL[3] * 16 + accH[3]);
                    accF[0] = fmaf(ddA.x * cw.x, f0, fmaf(-ddA.y * mx, accM[0], accF[0]));
                    accF[1] = fmaf(ddA.x * cw.y, f1, fmaf(-ddA.y * my, accM[1], accF[1]));
                    accF[2] = fmaf(ddB.x * cw.x, f2, fmaf(-ddB.y * mx, accM[2], accF[2]));
                    accF[3] = fmaf(ddB.x * cw.y, f3, fmaf(-ddB.y * my, accM[3], accF[3]));
                } else {
                    // Two column tiles: every weight fragment feeds two mma. One integer accumulator per output:
                    // the low-nibble sums enter with their scale times 16 (the high nibbles stay in place, x16).
                    int acc[2][4] = {{0, 0, 0, 0}, {0, 0, 0, 0}};
                    const uint8_t *rowA = stage + 256 + 32 * g + 8 * t;
                    const uint8_t *bp2 = bplane2 + (bp - bplane);
#pragma unroll
                    for (int p = 0; p < 4; p++) {
                        const uint2 wA = *reinterpret_cast<const uint2 *>(rowA + 512 * p);
                        const uint2 wB = *reinterpret_cast<const uint2 *>(rowA + 512 * p + 256);
                        const int sAl = (int)__byte_perm(p < 2 ? scA0 : scA1, 0, 0x4440 + ((2 * p) & 3)) << 4;
                        const int sAh = (int)__byte_perm(p < 2 ? scA0 : scA1, 0, 0x4440 + ((2 * p + 1) & 3));
                        const int sBl = (int)__byte_perm(p < 2 ? scB0 : scB1, 0, 0x4440 + ((2 * p) & 3)) << 4;
                        const int sBh = (int)__byte_perm(p < 2 ? scB0 : scB1, 0, 0x4440 + ((2 * p + 1) & 3));
                        const uint32_t a0l = wA.x & 0x0F0F0F0Fu, a1l = wB.x & 0x0F0F0F0Fu, a2l = wA.y & 0x0F0F0F0Fu, a3l = wB.y & 0x0F0F0F0Fu;
                        const uint32_t a0h = wA.x & 0xF0F0F0F0u, a1h = wB.x & 0xF0F0F0F0u, a2h = wA.y & 0xF0F0F0F0u, a3h = wB.y & 0xF0F0F0F0u;
#pragma unroll
                        for (int ct = 0; ct < 2; ct++) {
                            const uint4 b = *reinterpret_cast<const uint4 *>((ct ? bp2 : bp) + 64 * p);
                            int S[4];
                            mma_u8s8(S, a0l, a1l, a2l, a3l, b.x, b.y);
                            acc[ct][0] += sAl * S[0];
                            acc[ct][1] += sAl * S[1];
                            acc[ct][2] += sBl * S[2];
                            acc[ct][3] += sBl * S[3];
                            mma_u8s8(S, a0h, a1h, a2h, a3h, b.z, b.w);
                            acc[ct][0] += sAh * S[0];
                            acc[ct][1] += sAh * S[1];
                            acc[ct][2] += sBh * S[2];
                            acc[ct][3] += sBh * S[3];
                        }
                    }
                    const uint32_t mpA = hsub2(__byte_perm(__byte_perm(mnA0, mnA1, min_sel), 0x64646464u, 0x4140), 0x64006400u);
                    const uint32_t mpB = hsub2(__byte_perm(__byte_perm(mnB0, mnB1, min_sel), 0x64646464u, 0x4140), 0x64006400u);
                    const float2 ddA = __half22float2(*reinterpret_cast<const __half2 *>(&hA.x));   // d, dmin of row g
                    const float2 ddB = __half22float2(*reinterpret_cast<const __half2 *>(&hB.x));
#pragma unroll
                    for (int ct = 0; ct < 2; ct++) {
                        float accM[4];
                        mma_f16(accM, mpA, mpB, bmp[32 * ct]);
                        const float2 cw = *reinterpret_cast<const float2 *>(cwp + 8 * ct);
                        const float mx = 2032.f * cw.x, my = 260096.f * cw.y;
                        float (&out)[4] = ct ? accF2 : accF;
                        out[0] = fmaf(ddA.x * cw.x, (float)acc[ct][0], fmaf(-ddA.y * mx, accM[0], out[0]));
                        out[1] = fmaf(ddA.x * cw.y, (float)acc[ct][1], fmaf(-ddA.y * my, accM[1], out[1]));
                        out[2] = fmaf(ddB.x * cw.x, (float)acc[ct][2], fmaf(-ddB.y * mx, accM[2], out[2]));
                        out[3] = fmaf(ddB.x * cw.y, (float)acc[ct][3], fmaf(-ddB.y * my, accM[3], out[3]));
                    }
                }
                bp += 256;
                cwp += 8 * NT;
                bmp += 32 * NT;
                c_stage = c_stage + kStageBytes == my_stages + D * kStageBytes ? my_stages : c_stage + kStageBytes;
                // every lane's reads of the slot have returned (their values were consumed above):
                // after the warp converges the next copy may overwrite it
                __syncwarp();
                issue();
            }
            flush(tile, i, seg_end, accF, accF2);
            i = seg_end;
        }
        QM_DD_MARK(2);
        __syncthreads();
        if (fin_tile >= 0) {
            // partial sums of the warps that worked on the tile before this one, in warp order
            int t0_, lo_, n_, wq, wrem;
            warp_range(po->q, po->rem, nun, (int)blockIdx.x - po->cta0, po->nctas, t0_, lo_, n_, wq, wrem);
            const unsigned int ts = (unsigned int)(fin_tile * nun), big = (unsigned int)wrem * (unsigned int)(wq + 1);
            const int wf = wq == 0 ? (int)ts : ts < big ? (int)(ts / (unsigned int)(wq + 1))
                                                         : wrem + (int)((ts - big) / (unsigned int)wq);
            for (int o = lane; o < 16 * M; o += 32) {
                float sum = 0.f;
                for (int x = wf; x < warp; x++) sum += slots[((size_t)x * 2 + 1) * M * 16 + o];
                sum += slots[(size_t)warp * 2 * M * 16 + o];
                const int j = o >> 4, r = (tile0 + fin_tile) * 16 + (o & 15);
                const int split = TP ? po->split_row : 0;
                const bool second = TP && split > 0 && (tile0 + fin_tile) * 16 >= split;
                if (r < rows)
                    store_y((second ? po->y2 - split : opy) + (int64_t)j * ldy + r, sum, TP && (po->tp_shared & (second ? 2 : 1)) != 0);
            }
        }
        QM_DD_MARK(3);
    }
    if (TP) {
        // The launch ends only when every GPU's stores of this step have been performed everywhere:
        // each CTA fences at system scope and arrives at the local counter; the last one tells the
        // peers (its GPU's flag in their arenas takes the launch's epoch) and waits, bounded, for theirs.
        __syncthreads();
        if (tid == 0) {
            __threadfence_system();
            const unsigned int old = atomicAdd(a.grid_bar, 1u);
            if (old + 1 == gridDim.x) {
                __threadfence_system();
                const unsigned int epoch = a.tp_epoch0 + 1;
                for (int p = 0; p < a.tp_world; p++)
                    if (p != a.tp_rank)
                        st_release_sys(reinterpret_cast<unsigned int *>(
                                           reinterpret_cast<char *>(a.tp_flags + a.tp_rank) + a.peer_delta[p]), epoch);
                const long long t0 = clock64();
                for (int p = 0; p < a.tp_world; p++) {
                    if (p == a.tp_rank) continue;
                    while (!dead && (int)(ld_acquire_sys(a.tp_flags + p) - epoch) < 0) {
                        if (clock64() - t0 > a.wait_cycles) {
                            atomicOr(a.status, QM_STATUS_TIMEOUT);
                            dead = true;
                        }
                    }
                }
            }
        }
    }
}


// ---------------------------------------------------------------------------------------------
// Q4_0 / Q8_0 on the same integer path (kernels qm_gemv_q40_lean_*, qm_gemv_q80_lean_*): one matvec of up
// to four activation rows. The stores of these formats are row-major planes (quants and fp16 scales), laid
// out so that one 16-byte piece holds a lane's mma operands of four (Q4_0) or two (Q8_0) blocks; an item
// (16 rows x 256 columns) is gathered into a stage by 16-byte cp.async copies, row by row (every row of an
// item is a whole 128- or 256-byte line), with the pieces of odd rows swapped between the two halves of
// each 128 bytes so that the 16-byte reads of a quarter warp touch all banks.
// Arithmetic: Q8_0 value = d_b*q (s8 x s8 mma), Q4_0 value = d_b*(q - 8): u8 x s8 mma on the codes, the
// -8*d_b*sum(x) term as one f16 mma per unit of the block scales (fp16 as stored) against the sub-block
// sums of the activations. The block scale multiplies the exact integer sum of its sub-block in fp32.
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void mma_s8s8(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%10,%10,%10,%10};"
        : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(0));
}

// FMT: 2 = Q4_0, 8 = Q8_0. CPM mma columns per activation row (4: up to two rows, three limbs; 2: two
// limbs), NT column tiles of eight (NT = 2 with CPM = 2: up to eight rows), D ring stages per warp.
// K parts (a.parts > 1): the CTAs form a.parts groups, group p multiplies K units [p*units, (p+1)*units) of
// every tile — it stages only that range of x — and leaves its products, without the RMS scale, in partial
// vector p (a.y + p*a.part_stride) and its sums of squares in a.ssq[p*8 + row]; qm_lean_sum adds them up.
template <int FMT, int CPM, int D, int NT>
__device__ __forceinline__ void lean_body(const QmLeanArgs &a) {
    constexpr int C = 16;
    constexpr int NL = CPM == 4 ? 3 : 2;
    constexpr int ROWB = FMT == 2 ? 128 : 256;            // quant bytes of one row of an item
    constexpr int QB = 16 * ROWB;                         // quant bytes of an item
    constexpr int STAGE = QB + 256;                       // + 16 rows of 8 fp16 scales
    extern __shared__ __align__(128) uint8_t smem[];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, t = lane & 3;
    const int M = a.m, P = M * NL, nun = a.units;

    const int plane_stride = nun * 256 + 64;
    uint8_t *xs = smem;                                                             // [P][plane_stride]
    uint32_t *xsum = reinterpret_cast<uint32_t *>(xs + (size_t)P * plane_stride);    // [units][8*NT][4] f16 pairs
    float *sxw = reinterpret_cast<float *>(xsum + (size_t)nun * 8 * NT * 4);         // [units][8*NT] column weights
    float *ssq = sxw + (size_t)nun * 8 * NT;                                         // [8][16]
    float *slots = ssq + 8 * 16;                                                     // [C][2][M*16]
    uint8_t *stages = reinterpret_cast<uint8_t *>(((uintptr_t)(slots + (size_t)C * 2 * M * 16) + 127) & ~(uintptr_t)127);
    uint8_t *my_stages = stages + (size_t)warp * D * STAGE;

    asm volatile("griddepcontrol.launch_dependents;");
    for (int i = tid; i < nun * 8 * NT * 5; i += C * 32) xsum[i] = 0u;   // xsum and sxw are adjacent: absent columns read zero

    // ---- this warp's items: the CTA owns a run of whole tiles of its K part, its items go evenly to the warps
    const int G = (int)gridDim.x / a.parts;               // CTAs per K part
    const int part = (int)blockIdx.x / G, c = (int)blockIdx.x - part * G;
    const int unit0 = part * nun;
    const int tile0 = c * a.q + min(c, a.rem);
    const int Ic = (a.q + (c < a.rem ? 1 : 0)) * nun;
    const int wq_ = Ic / C, wrem = Ic - wq_ * C;
    const int lo = warp * wq_ + min(warp, wrem), n = wq_ + (warp < wrem ? 1 : 0), hi = lo + n;
    float *const yout = a.y + (int64_t)part * a.part_stride;

    // ---- producer: gathers one item per call into the next stage ------------------------------------
    const int64_t rs = (int64_t)a.units_total * ROWB, srs = (int64_t)a.units_total * 16;   // bytes between rows: quants, scales
    constexpr int RPP = 32 / (ROWB / 16);                 // rows covered by one pass of the warp's 32 pieces
    constexpr int PASSES = 16 / RPP;
    const int prow = lane / (ROWB / 16), pcol = lane % (ROWB / 16);   // this lane's row within a pass and piece
    const uint32_t ring0 = smem_u32(my_stages);
    const uint32_t dst_q = prow * ROWB + ((pcol ^ (4 * (prow & 1))) * 16), dst_s = QB + lane * 16;
    int p_left = n, p_tile = lo / nun, p_u = lo - p_tile * nun;
    uint32_t p_dst = ring0;
    auto issue = [&]() {
        if (p_left > 0) {
            const int row0 = (tile0 + p_tile) * 16;
            const uint8_t *qsrc = a.wq + (int64_t)(unit0 + p_u) * ROWB + pcol * 16;
#pragma unroll
            for (int j = 0; j < PASSES; j++) {
                const int r = min(row0 + prow + j * RPP, a.rows - 1);   // rows past the last one repeat it; never stored
                cp_async16(p_dst + dst_q + j * RPP * ROWB, qsrc + r * rs);
            }
            if (lane < 16)
                cp_async16(p_dst + dst_s, reinterpret_cast<const uint8_t *>(a.wd) + min(row0 + lane, a.rows - 1) * srs + (unit0 + p_u) * 16);
            p_left--;
            if (++p_u == nun) { p_u = 0; p_tile++; }
        }
        cp_async_commit();
        p_dst = p_dst + STAGE == ring0 + D * STAGE ? ring0 : p_dst + STAGE;
    };
#pragma unroll
    for (int d = 0; d < D; d++) issue();

    // ---- stage x (the launch's input: no polling), quantize into limb planes --------------------------
    asm volatile("griddepcontrol.wait;" ::: "memory");
    __syncthreads();
    const int xop = a.xop;
    const bool norm = xop == 1 || xop == 2;
    {
        float sq_run = 0.f;
        int sq_j = -1;
        if (norm && lane < 8) ssq[lane * 16 + warp] = 0.f;
        __syncwarp();
        for (int idx = warp; idx < M * nun; idx += C) {
            const int j = idx / nun, ul = idx - j * nun;
            const int col = (unit0 + ul) * QM_K_UNIT + lane * 8;
            float v[8];
#pragma unroll
            for (int e = 0; e < 8; e++) v[e] = 0.f;
            if (col < a.cols) {   // cols is a multiple of 32: a lane's eight columns are all inside or all outside
                const float *xp = a.x + (int64_t)j * a.ldx + col;
                const float4 r0 = *reinterpret_cast<const float4 *>(xp), r1 = *reinterpret_cast<const float4 *>(xp + 4);
                v[0] = r0.x; v[1] = r0.y; v[2] = r0.z; v[3] = r0.w; v[4] = r1.x; v[5] = r1.y; v[6] = r1.z; v[7] = r1.w;
                if (xop >= 2) {
                    const float *x2p = a.x2 + (int64_t)j * a.ldx + col;
                    const float4 s0 = *reinterpret_cast<const float4 *>(x2p), s1 = *reinterpret_cast<const float4 *>(x2p + 4);
                    const float w[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
#pragma unroll
                    for (int e = 0; e < 8; e++) v[e] = xop == 2 ? v[e] + w[e] : v[e] / (1.f + __expf(-v[e])) * w[e];
                }
            }
            const float sq = quantize_pair<NT, true>(v, j, ul, lane, NL, CPM, xs, plane_stride, xsum, sxw, 1.f);
            if (norm) {
                if (j != sq_j) {
                    if (sq_j >= 0) {
#pragma unroll
                        for (int o = 16; o > 0; o >>= 1) sq_run += __shfl_xor_sync(0xffffffffu, sq_run, o);
                        if (lane == 0) ssq[sq_j * 16 + warp] = sq_run;
                    }
                    sq_j = j;
                    sq_run = 0.f;
                }
                sq_run += sq;
            }
        }
        if (sq_j >= 0) {
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) sq_run += __shfl_xor_sync(0xffffffffu, sq_run, o);
            if (lane == 0) ssq[sq_j * 16 + warp] = sq_run;
        }
    }
    __syncthreads();
    float myscale[NT];
#pragma unroll
    for (int ct = 0; ct < NT; ct++) myscale[ct] = 1.f;
    if (norm) {
        const float inv_cols = 1.f / (float)a.cols;
        for (int j = 0; j < M; j++) {
            float sq = ssq[j * 16 + (lane & 15)];
#pragma unroll
            for (int o = 8; o > 0; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
            if (a.parts > 1) {   // a part leaves its products unscaled and publishes its share of the sum of squares
                if (c == 0 && tid == 0) a.ssq[part * 8 + j] = sq;
                continue;
            }
            const float sc = rsqrtf(sq * inv_cols + a.eps);
#pragma unroll
            for (int ct = 0; ct < NT; ct++)
                if ((CPM == 4 ? (t >> 1) : ct * 4 + t) == j) myscale[ct] = sc;
        }
    }

    // ---- stream --------------------------------------------------------------------------------------
    const uint8_t *bplane[NT];
#pragma unroll
    for (int ct = 0; ct < NT; ct++) {
        const int ncol = ct * 8 + g, col_row = ncol / CPM, col_limb = ncol - col_row * CPM;
        const bool col_on = col_row < M && col_limb < NL;
        bplane[ct] = xs + (size_t)(col_on ? col_row * NL + col_limb : 0) * plane_stride + t * 16;
    }
    const uint32_t swz = 4u * (g & 1);
    const uint8_t *c_stage = my_stages;
    int fin_tile = -1;
    auto flush = [&](int tile, int s0, int s1, const float (&accF)[NT][4]) {
        const bool from_start = s0 == tile * nun, to_end = s1 == tile * nun + nun;
        if (!(from_start && to_end) && to_end) fin_tile = tile;
#pragma unroll
        for (int ct = 0; ct < NT; ct++) {
            float vA = accF[ct][0] + accF[ct][1], vB = accF[ct][2] + accF[ct][3];
            int jrow;
            bool valid;
            if (CPM == 4) {
                vA += __shfl_xor_sync(0xffffffffu, vA, 1);
                vB += __shfl_xor_sync(0xffffffffu, vB, 1);
                jrow = t >> 1;
                valid = (t & 1) == 0 && jrow < M;
            } else {
                jrow = ct * 4 + t;
                valid = jrow < M;
            }
            vA *= myscale[ct];
            vB *= myscale[ct];
            if (from_start && to_end) {
                const int rA = (tile0 + tile) * 16 + g, rB = rA + 8;
                if (valid) {
                    float *yA = yout + (int64_t)jrow * a.ldy + rA;
                    if (rA < a.rows) yA[0] = vA;
                    if (rB < a.rows) yA[8] = vB;
                }
            } else {
                // slot 1: the segment ends inside the tile; slot 0: it joined the tile late and reaches its end
                float *p = slots + ((size_t)warp * 2 + (to_end ? 0 : 1)) * M * 16;
                if (valid) { p[jrow * 16 + g] = vA; p[jrow * 16 + g + 8] = vB; }
            }
        }
    };
    for (int i = lo; i < hi;) {
        const int tile = i / nun, u0 = i - tile * nun;
        const int seg_end = min(hi, (tile + 1) * nun);
        float accF[NT][4];
#pragma unroll
        for (int ct = 0; ct < NT; ct++) accF[ct][0] = accF[ct][1] = accF[ct][2] = accF[ct][3] = 0.f;
        int boff = u0 * 256;                                            // byte offset of the unit in a plane
        const float *cwp = sxw + (size_t)u0 * 8 * NT + 2 * t;
        const uint32_t *bmp = xsum + (size_t)u0 * 32 * NT + g * 4 + t;
        for (int k = i; k < seg_end; k++) {
            cp_async_wait_n<D - 1>();
            __syncwarp();
            const uint8_t *stage = c_stage;
            const uint4 hA = *reinterpret_cast<const uint4 *>(stage + QB + 16 * g);        // eight fp16 block scales of row g
            const uint4 hB = *reinterpret_cast<const uint4 *>(stage + QB + 16 * g + 128);   // ... of row g + 8
            const uint32_t hAw[4] = {hA.x, hA.y, hA.z, hA.w}, hBw[4] = {hB.x, hB.y, hB.z, hB.w};
            float accU[NT][4];
#pragma unroll
            for (int ct = 0; ct < NT; ct++) accU[ct][0] = accU[ct][1] = accU[ct][2] = accU[ct][3] = 0.f;
            const uint8_t *rowA = stage + g * ROWB, *rowB = rowA + 8 * ROWB;
            constexpr int GROUPS = ROWB / 64;   // 64-byte groups per row: four blocks (Q4_0) or two (Q8_0) each
#pragma unroll
            for (int q = 0; q < GROUPS; q++) {
                const uint32_t piece = (((uint32_t)(q * 4 + t)) ^ swz) * 16;
                const uint4 wA = *reinterpret_cast<const uint4 *>(rowA + piece);
                const uint4 wB = *reinterpret_cast<const uint4 *>(rowB + piece);
                const uint32_t wAw[4] = {wA.x, wA.y, wA.z, wA.w}, wBw[4] = {wB.x, wB.y, wB.z, wB.w};
                constexpr int BPG = FMT == 2 ? 4 : 2;   // blocks per group
#pragma unroll
                for (int s = 0; s < BPG; s++) {
                    const int sb = q * BPG + s;   // sub-block of the unit
                    uint32_t a0, a1, a2, a3;
                    if (FMT == 2) {
                        a0 = wAw[s] & 0x0F0F0F0Fu; a1 = wBw[s] & 0x0F0F0F0Fu;
                        a2 = (wAw[s] >> 4) & 0x0F0F0F0Fu; a3 = (wBw[s] >> 4) & 0x0F0F0F0Fu;
                    } else {
                        a0 = wAw[2 * s]; a1 = wBw[2 * s]; a2 = wAw[2 * s + 1]; a3 = wBw[2 * s + 1];
                    }
                    const uint32_t pa = hAw[sb >> 1], pb = hBw[sb >> 1];
                    const float dA = __half2float(__ushort_as_half((unsigned short)((sb & 1) ? pa >> 16 : pa & 0xFFFFu)));
                    const float dB = __half2float(__ushort_as_half((unsigned short)((sb & 1) ? pb >> 16 : pb & 0xFFFFu)));
#pragma unroll
                    for (int ct = 0; ct < NT; ct++) {
                        const uint2 b = *reinterpret_cast<const uint2 *>(bplane[ct] + boff + 64 * (sb >> 1) + 8 * (sb & 1));
                        int S[4];
                        if (FMT == 2) mma_u8s8(S, a0, a1, a2, a3, b.x, b.y);
                        else mma_s8s8(S, a0, a1, a2, a3, b.x, b.y);
                        accU[ct][0] = fmaf(dA, (float)S[0], accU[ct][0]);
                        accU[ct][1] = fmaf(dA, (float)S[1], accU[ct][1]);
                        accU[ct][2] = fmaf(dB, (float)S[2], accU[ct][2]);
                        accU[ct][3] = fmaf(dB, (float)S[3], accU[ct][3]);
                    }
                }
            }
#pragma unroll
            for (int ct = 0; ct < NT; ct++) {
                const float2 cw = *reinterpret_cast<const float2 *>(cwp + 8 * ct);
                if (FMT == 2) {
                    // - 8 * sum_b d_b * sum(x in block b): the scales as they are stored (fp16 pairs 2t, 2t+1) times the sums
                    float accM[4];
                    mma_f16(accM, *reinterpret_cast<const uint32_t *>(stage + QB + 16 * g + 4 * t),
                            *reinterpret_cast<const uint32_t *>(stage + QB + 16 * g + 128 + 4 * t), bmp[32 * ct]);
                    const float mx = -8.f * 127.f * cw.x, my = -8.f * 16256.f * cw.y;
                    accF[ct][0] = fmaf(cw.x, accU[ct][0], fmaf(mx, accM[0], accF[ct][0]));
                    accF[ct][1] = fmaf(cw.y, accU[ct][1], fmaf(my, accM[1], accF[ct][1]));
                    accF[ct][2] = fmaf(cw.x, accU[ct][2], fmaf(mx, accM[2], accF[ct][2]));
                    accF[ct][3] = fmaf(cw.y, accU[ct][3], fmaf(my, accM[3], accF[ct][3]));
                } else {
                    accF[ct][0] = fmaf(cw.x, accU[ct][0], accF[ct][0]);
                    accF[ct][1] = fmaf(cw.y, accU[ct][1], accF[ct][1]);
                    accF[ct][2] = fmaf(cw.x, accU[ct][2], accF[ct][2]);
                    accF[ct][3] = fmaf(cw.y, accU[ct][3], accF[ct][3]);
                }
            }
            boff += 256;
            cwp += 8 * NT;
            bmp += 32 * NT;
            c_stage = c_stage + STAGE == my_stages + D * STAGE ? my_stages : c_stage + STAGE;
            __syncwarp();
            issue();
        }
        flush(tile, i, seg_end, accF);
        i = seg_end;
    }
    __syncthreads();
    if (fin_tile >= 0) {
        // partial sums of the warps that worked on the tile before this one, in warp order
        const unsigned int ts = (unsigned int)(fin_tile * nun), big = (unsigned int)wrem * (unsigned int)(wq_ + 1);
        const int wf = wq_ == 0 ? (int)ts : ts < big ? (int)(ts / (unsigned int)(wq_ + 1))
                                                      : wrem + (int)((ts - big) / (unsigned int)wq_);
        for (int o = lane; o < 16 * M; o += 32) {
            float sum = 0.f;
            for (int x = wf; x < warp; x++) sum += slots[((size_t)x * 2 + 1) * M * 16 + o];
            sum += slots[(size_t)warp * 2 * M * 16 + o];
            const int j = o >> 4, r = (tile0 + fin_tile) * 16 + (o & 15);
            if (r < a.rows) yout[(int64_t)j * a.ldy + r] = sum;
        }
    }
}

}  // namespace

extern "C" __global__ void __launch_bounds__(QM_GEMV_MAX_THREADS, 1)
    qm_fused_q4k_nt1(const __grid_constant__ QmFusedArgs a) {
    fused_body<1, false, false>(a);
}
extern "C" __global__ void __launch_bounds__(QM_GEMV_MAX_THREADS, 1)
    qm_fused_q4k_nt2(const __grid_constant__ QmFusedArgs a) {
    fused_body<2, false, false>(a);
}
// The same with activation images between dependent ops (used from two activation rows on).
extern "C" __global__ void __launch_bounds__(QM_GEMV_MAX_THREADS, 1)
    qm_fused_q4k_nt1_img(const __grid_constant__ QmFusedArgs a) {
    fused_body<1, true, false>(a);
}
extern "C" __global__ void __launch_bounds__(QM_GEMV_MAX_THREADS, 1)
    qm_fused_q4k_nt2_img(const __grid_constant__ QmFusedArgs a) {
    fused_body<2, true, false>(a);
}
// Data-driven variants (no grid barrier between dependent ops): CPM = 4 mma columns per
// activation row (up to two rows, three limbs) or 2 (up to four rows, two limbs), D ring stages
// per warp as shared memory allows; _tp: tensor parallel, results stored into every GPU's arena
// and one barrier over the GPUs at the end of the launch.
#define QM_DD_KERNEL(name, cpm, d, tp)                                                       \
    extern "C" __global__ void __launch_bounds__(QM_GEMV_MAX_THREADS, 1)                     \
        name(const __grid_constant__ QmFusedArgs a) {                                        \
        dd_body<cpm, d, tp>(a);                                                              \
    }
QM_DD_KERNEL(qm_fused_q4k_dd_c4d2, 4, 2, false)
QM_DD_KERNEL(qm_fused_q4k_dd_c4d3, 4, 3, false)
QM_DD_KERNEL(qm_fused_q4k_dd_c4d4, 4, 4, false)
QM_DD_KERNEL(qm_fused_q4k_dd_c2d2, 2, 2, false)
QM_DD_KERNEL(qm_fused_q4k_dd_c2d3, 2, 3, false)
QM_DD_KERNEL(qm_fused_q4k_dd_c2d4, 2, 4, false)
QM_DD_KERNEL(qm_fused_q4k_dd_c4d2_tp, 4, 2, true)
QM_DD_KERNEL(qm_fused_q4k_dd_c4d3_tp, 4, 3, true)
QM_DD_KERNEL(qm_fused_q4k_dd_c4d4_tp, 4, 4, true)
QM_DD_KERNEL(qm_fused_q4k_dd_c2d2_tp, 2, 2, true)
QM_DD_KERNEL(qm_fused_q4k_dd_c2d3_tp, 2, 3, true)
QM_DD_KERNEL(qm_fused_q4k_dd_c2d4_tp, 2, 4, true)

// Five to eight activation rows: two column tiles (D = 2 or 3 stages: sixteen limb planes take the room of the fourth).
#define QM_DD8_KERNEL(name, d)                                                               \
    extern "C" __global__ void __launch_bounds__(QM_GEMV_MAX_THREADS, 1)                     \
        name(const __grid_constant__ QmFusedArgs a) {                                        \
        dd_body<2, d, false, false, 2>(a);                                                   \
    }
QM_DD8_KERNEL(qm_fused_q4k_dd_n2d2, 2)
QM_DD8_KERNEL(qm_fused_q4k_dd_n2d3, 3)

// One activation row per op and ops whose matrix is chosen on the device from a table of experts
// (QmOp::sel_table): decode-time MoE as a list of (token, slot) matvecs.
#define QM_DD_SEL_KERNEL(name, d)                                                            \
    extern "C" __global__ void __launch_bounds__(QM_GEMV_MAX_THREADS, 1)                     \
        name(const __grid_constant__ QmFusedArgs a) {                                        \
        dd_body<4, d, false, true>(a);                                                       \
    }
QM_DD_SEL_KERNEL(qm_fused_q4k_dd_c4d2_sel, 2)
QM_DD_SEL_KERNEL(qm_fused_q4k_dd_c4d3_sel, 3)
QM_DD_SEL_KERNEL(qm_fused_q4k_dd_c4d4_sel, 4)

// h = c * (sum of the K parts of the step's last matvec), see QmSumPartsArgs.
extern "C" __global__ void __launch_bounds__(256) qm_sum_parts(const __grid_constant__ QmSumPartsArgs a) {
    const int total = a.m * a.n;
    for (int idx = blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += gridDim.x * blockDim.x) {
        const int j = idx / a.n, r = idx - j * a.n;
        float sum = 0.f, sq = 0.f;
        for (int k = 0; k < a.nparts; k++) {
            sum += a.parts[k * a.part_stride + (int64_t)j * a.ld_in + r];
            sq += a.ssq[k * 8 + j];
        }
        a.out[(int64_t)j * a.ld_out + r] = sum * rsqrtf(sq * a.inv_cols + a.eps);
    }
}

// Tensor-parallel variants with barriers: outputs go to every peer's arena, barriers span the GPUs.
extern "C" __global__ void __launch_bounds__(QM_GEMV_MAX_THREADS, 1)
    qm_fused_q4k_nt1_tp(const __grid_constant__ QmFusedArgs a) {
    fused_body<1, false, true>(a);
}
extern "C" __global__ void __launch_bounds__(QM_GEMV_MAX_THREADS, 1)
    qm_fused_q4k_nt2_tp(const __grid_constant__ QmFusedArgs a) {
    fused_body<2, false, true>(a);
}

// Q4_0 / Q8_0 matvec on the integer path (see lean_body): c4 = up to two activation rows (three limbs), c2 = up
// to four, c2n2 = up to eight (two column tiles); d = ring stages per warp.
#define QM_LEAN_KERNEL(name, fmt, cpm, d, nt)                                                \
    extern "C" __global__ void __launch_bounds__(QM_GEMV_MAX_THREADS, 1)                     \
        name(const __grid_constant__ QmLeanArgs a) {                                         \
        lean_body<fmt, cpm, d, nt>(a);                                                       \
    }
QM_LEAN_KERNEL(qm_gemv_q40_lean_c4d4, 2, 4, 4, 1)
QM_LEAN_KERNEL(qm_gemv_q40_lean_c4d2, 2, 4, 2, 1)
QM_LEAN_KERNEL(qm_gemv_q40_lean_c2d4, 2, 2, 4, 1)
QM_LEAN_KERNEL(qm_gemv_q40_lean_c2d2, 2, 2, 2, 1)
QM_LEAN_KERNEL(qm_gemv_q40_lean_c2n2d4, 2, 2, 4, 2)
QM_LEAN_KERNEL(qm_gemv_q40_lean_c2n2d2, 2, 2, 2, 2)
QM_LEAN_KERNEL(qm_gemv_q80_lean_c4d3, 8, 4, 3, 1)
QM_LEAN_KERNEL(qm_gemv_q80_lean_c4d2, 8, 4, 2, 1)
QM_LEAN_KERNEL(qm_gemv_q80_lean_c2d3, 8, 2, 3, 1)
QM_LEAN_KERNEL(qm_gemv_q80_lean_c2d2, 8, 2, 2, 1)
QM_LEAN_KERNEL(qm_gemv_q80_lean_c2n2d3, 8, 2, 3, 2)
QM_LEAN_KERNEL(qm_gemv_q80_lean_c2n2d2, 8, 2, 2, 2)

// out[j][r] = c_j * sum over the K parts of a lean matvec, c_j = rsqrt(mean square + eps) from the parts' sums of
// squares when the matvec normalises its input, else 1.
extern "C" __global__ void __launch_bounds__(256) qm_lean_sum(const __grid_constant__ QmSumPartsArgs a) {
    asm volatile("griddepcontrol.launch_dependents;");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const int total = a.m * a.n;
    for (int idx = blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += gridDim.x * blockDim.x) {
        const int j = idx / a.n, r = idx - j * a.n;
        float sum = 0.f, sq = 0.f;
        for (int k = 0; k < a.nparts; k++) {
            sum += a.parts[k * a.part_stride + (int64_t)j * a.ld_in + r];
            if (a.ssq) sq += a.ssq[k * 8 + j];
        }
        a.out[(int64_t)j * a.ld_out + r] = a.ssq ? sum * rsqrtf(sq * a.inv_cols + a.eps) : sum;
    }
}
