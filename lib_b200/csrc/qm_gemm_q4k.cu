// qm_gemm_q4k.cu — prefill / batched matmul over Q4_K weights on the sm_100a tensor cores:
// C[m][n] = sum_k A[m][k] * W[n][k], A bf16 activations, W dequantized on the fly, fp32 out.
//
// Supersedes the reference's fp16 wmma 256-row "prefill" GEMM
// (nvidia/x/cudamoe/prefill.go:97-121), which is neither quantized nor tcgen05.
//
// One CTA computes a 128 (weight rows) x BN (tokens, 64..512) tile of C^T:
//   * warps 2..17 form four groups of 128 threads; group g handles the K chunks g, g+4, ...: one
//     thread per weight row reads the row's 32 quant bytes of a 64-column K chunk from the tiled
//     weight store, turns the nibbles into exact bf16 integers with the magic-number trick (byte
//     0x43 beside the code = 128+q), applies the sub-block scale and minimum with one bf16x2 FMA
//     per pair, and writes the row into shared memory in the canonical K-major 128-byte-swizzled
//     layout of tcgen05 (A operand); four chunks in flight hide the latency of that chain
//     (each stage has two release barriers, so four groups may run ahead of two or three stages);
//   * warp 0 streams the matching 64 x BN activation chunk with 2-D TMA tile copies
//     (SWIZZLE_128B, no multicast; only the boxes that hold rows of the tile) that complete on an
//     mbarrier (B operand) — or, for a grouped launch given the dispatch list instead of gathered
//     rows, with tile::gather4 copies of four token rows each;
//   * one elected thread of warp 1 issues four tcgen05.mma.kind::f16 (K = 16 each) per chunk
//     and per 256 tokens into a TMEM accumulator of BN fp32 columns (BN = 512 uses the whole
//     tensor memory: the dequantized tile then feeds two MMAs; N = the tile's tokens rounded up to
//     16), tcgen05.commit frees the stage;
//   * after the last chunk warps 2..17 read the accumulator back with tcgen05.ld (16 columns at a
//     time, dealt evenly to the four warps of a lane quarter) and store C.
// A ring of 2..8 shared-memory stages decouples the three roles. Every mbarrier wait is
// bounded (qm_pipe.cuh); on expiry the status word gets QM_STATUS_TIMEOUT, the roles leave
// their loops, TMEM is freed and the kernel returns.
#include <cuda.h>
#include <cuda_bf16.h>
#include <stdint.h>

#include "qm_kernel_args.h"
#include "qm_pipe.cuh"

// Debug builds (-DQM_DEBUG) can switch pipeline roles off for timing experiments; the results are
// then wrong. The shipped build compiles the switches out.
#ifdef QM_DEBUG
#define QM_GEMM_DEBUG_BIT(b) ((a.debug & (b)) != 0)
#else
#define QM_GEMM_DEBUG_BIT(b) false
#endif

using namespace qm;

namespace {

constexpr int kMaxStages = 8;
constexpr int kBM = 128;          // weight rows per CTA (tcgen05 M)
constexpr int kBK = 64;           // K columns per stage: one 32-byte quant group, 128 bytes of bf16
constexpr int kATile = kBM * kBK * 2;

__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
    uint32_t d;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(sel));
    return d;
}
__device__ __forceinline__ uint32_t bsub2(uint32_t a, uint32_t b) {
    uint32_t d;
    asm("sub.rn.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
    return d;
}
__device__ __forceinline__ uint32_t bfma2(uint32_t a, uint32_t b, uint32_t c) {
    uint32_t d;
    asm("fma.rn.bf16x2 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}
__device__ __forceinline__ uint32_t bf2(float v) {   // (v, v) as bf16x2
    __nv_bfloat162 h = __float2bfloat162_rn(v);
    return *reinterpret_cast<uint32_t *>(&h);
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const void *tmap, int x, int y, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(dst),
        "l"(tmap), "r"(x), "r"(y), "r"(bar)
        : "memory");
}
// K-major, 128-byte swizzle, 8-row groups 1024 bytes apart (sm_100 descriptor version 1)
// Four rows (y0..y3) of a 2-D tensor, box columns starting at x, into four consecutive rows at dst.
__device__ __forceinline__ void tma_gather4(uint32_t dst, const void *tmap, int x, int y0, int y1, int y2, int y3,
                                            uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile::gather4.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6, %7}], [%2];" ::"r"(dst),
        "l"(tmap), "r"(bar), "r"(x), "r"(y0), "r"(y1), "r"(y2), "r"(y3)
        : "memory");
}
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr) {
    return (uint64_t)((addr >> 4) & 0x3FFFu) | (1ull << 16) | (64ull << 32) | (1ull << 46) | (2ull << 61);
}
__device__ __forceinline__ void umma_f16(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t acc) {
    asm volatile(
        "{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}" ::"r"(d_tmem),
        "l"(adesc), "l"(bdesc), "r"(idesc), "r"(acc)
        : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

}  // namespace

// NSUB = 128-row sub-tiles of weight rows per CTA: 1 (128 x BN tile, BN up to 512) or 2
// (256 x BN tile, BN up to 256: half the activation traffic per flop and room for a third stage).
// KS = 64-column K chunks per pipeline stage: 1, or 2 for small token tiles, where the barrier
// handshake of a stage (about 0.3 us, whatever the stage count) is longer than the MMAs of one
// chunk: two chunks per handshake halve it.
#ifdef QM_DEBUG
__device__ __forceinline__ unsigned long long gtime() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}
#define QM_GEMM_STAMP(i)                                                                                       \
    do {                                                                                                       \
        if ((a.debug & 64) && a.swiglu) {                                                                      \
            const int L_ = blockIdx.y * gridDim.x + blockIdx.x;                                                \
            if (L_ < 990) reinterpret_cast<unsigned long long *>(a.status + 256)[L_ * 4 + (i)] = gtime();      \
        }                                                                                                      \
    } while (0)
#else
#define QM_GEMM_STAMP(i)
#endif

template <int NSUB, int KS>
__device__ __forceinline__ void gemm_body(const QmGemmArgs &a) {
    extern __shared__ uint8_t smem_raw[];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    if (tid == 0) QM_GEMM_STAMP(0);
    const int BN = a.bn, kStages = a.stages;
    const int b_tile = BN * kBK * 2;          // one 64-column chunk of the activations
    constexpr int a_tile = NSUB * kATile;     // one 64-column chunk of the weights
    const int a_bytes = KS * a_tile;
    const int stage_bytes = a_bytes + KS * b_tile;
    uint8_t *smem = reinterpret_cast<uint8_t *>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem + (size_t)kStages * stage_bytes);
    const uint32_t full_a = smem_u32(bars), full_b = full_a + 8 * kMaxStages, empty = full_b + 8 * kMaxStages;
    // Two "empty" barriers per stage, taken in turn by the stage's phases: a parity wait cannot tell a
    // barrier's completions two apart, and with one barrier per stage that allowed no more chunks in
    // production than stages. With two, the chunks whose release could be mistaken lie four phases apart,
    // so four groups of dequantizing warps may work ahead of two or three stages.
    const uint32_t tmem_full = empty + 8 * 2 * kMaxStages;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 4 * kMaxStages + 1);
    // chunk kc may be written into its stage when the MMAs of chunk kc - kStages have read it
    auto wait_empty = [&](int kc) -> bool {
        const int ph = kc / kStages;
        if (ph == 0) return true;
        return mbar_wait_bounded(empty + 8 * (2 * (kc % kStages) + ((ph - 1) & 1)), (uint32_t)((ph - 1) >> 1) & 1u);
    };
    const uint32_t smem_base = smem_u32(smem);

    const bool fuse_swiglu = NSUB == 2 && a.swiglu != 0;
    // grouped launches put the expert in blockIdx.y and the token tile in blockIdx.z: CTAs are
    // handed out x-fastest, then y, then z, so every expert's first token tiles (the ones with
    // work) start before the mostly empty later tiles
    // (grouped launches with split K: blockIdx.z = token tile * splitk + K share)
    const int n0 = blockIdx.x * kBM * (fuse_swiglu ? 1 : NSUB), m0 = (a.grouped ? (int)blockIdx.z / a.splitk : (int)blockIdx.y) * BN;
    // grouped launch: this CTA's expert, its rows of the gathered activations and its weights
    int row_off = 0, m_cnt = a.m;
    const uint8_t *wq = a.wq;
    if (a.grouped) {
        const int e = blockIdx.y;
        row_off = a.offsets[e];
        m_cnt = a.offsets[e + 1] - row_off;
        if (m0 >= m_cnt) return;   // nothing routed here (uniform over the CTA, before any barrier)
        wq = a.wq_list[e];
    }
    // 64-column chunks along K; with split K (splitk > 1) this CTA takes a contiguous share
    // and stores its partial tile to its own plane of the scratch (added up in a fixed order at the end)
    const int nk_all = a.units * 4 / KS;      // stage chunks of KS x 64 columns
    const int zk = a.grouped ? (int)blockIdx.z % a.splitk : (int)blockIdx.z;
    const int kc_lo = (int)((int64_t)nk_all * zk / a.splitk);
    const int nk = (int)((int64_t)nk_all * (zk + 1) / a.splitk) - kc_lo;

    if (tid == 0) {
        for (int s = 0; s < kStages; s++) {
            mbar_init(full_a + 8 * s, a.groups == 4 ? 4 : 8);   // warps of one producer group
            mbar_init(full_b + 8 * s, 1);
            mbar_init(empty + 8 * (2 * s), 1);
            mbar_init(empty + 8 * (2 * s + 1), 1);
        }
        mbar_init(tmem_full, 1);
        fence_barrier_init();
    }
    // TMEM columns come in powers of two
    uint32_t tmem_cols = 32;
    while (tmem_cols < (uint32_t)(NSUB * BN)) tmem_cols <<= 1;
    if (warp == 1) {   // TMEM accumulators: NSUB x BN fp32 columns x 128 lanes
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                     "r"(tmem_cols)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0 && a.gather_list) {
        // ---- activation chunks gathered by the rows' token numbers ----------------------------
        // One tile::gather4 copy brings the 64-column chunk of four rows named by their row numbers
        // in the tokens' own matrix (a tensor map with a one-row box) into four consecutive
        // 128-byte rows of the swizzled tile; lane l issues the copies of row groups l, l+32, ...
        int *tok = reinterpret_cast<int *>(tmem_slot + 6);   // 16-byte aligned
        for (int r = lane; r < BN; r += 32)   // rows past the list read its last row; the epilogue drops them
            tok[r] = a.gather_list[row_off + min(m0 + r, m_cnt - 1)] / a.gather_topk;
        __syncwarp();
        for (int kc = 0; kc < nk; kc++) {
            const int s = kc % kStages;
            if (!wait_empty(kc)) {
                if (lane == 0) atomicOr(a.status, QM_STATUS_TIMEOUT);
                break;
            }
            if (lane == 0) mbar_expect_tx(full_b + 8 * s, (uint32_t)(KS * b_tile));
            __syncwarp();
#pragma unroll
            for (int j = 0; j < KS; j++)
                for (int g4 = lane; g4 < BN / 4; g4 += 32) {
                    const int4 t = *reinterpret_cast<const int4 *>(tok + 4 * g4);
                    tma_gather4(smem_base + s * stage_bytes + a_bytes + j * b_tile + g4 * 512, &a.tmap_gather,
                                ((kc_lo + kc) * KS + j) * kBK, t.x, t.y, t.z, t.w, full_b + 8 * s);
                }
        }
    } else if (warp == 0) {
        // ---- activation chunks by TMA ---------------------------------------------------------
        if (lane == 0) {
            const int box = a.box_rows, nbox = (min(BN, m_cnt - m0) + box - 1) / box;
            for (int kc = 0; kc < nk; kc++) {
                const int s = kc % kStages;
                if (!wait_empty(kc)) { atomicOr(a.status, QM_STATUS_TIMEOUT); break; }
                if (QM_GEMM_DEBUG_BIT(2)) { mbar_arrive(full_b + 8 * s); continue; }
                // only the boxes that hold rows of this tile (an MMA reads no further than its N)
                mbar_expect_tx(full_b + 8 * s, (uint32_t)(KS * nbox * box * 128));
#pragma unroll
                for (int j = 0; j < KS; j++)
                    for (int nb = 0; nb < nbox * box; nb += box)   // a TMA box has at most 256 rows
                        tma_load_2d(smem_base + s * stage_bytes + a_bytes + j * b_tile + nb * 128, &a.tmap_act,
                                    ((kc_lo + kc) * KS + j) * kBK, row_off + m0 + nb, full_b + 8 * s);
            }
        }
    } else if (warp == 1) {
        // ---- MMA issue ----------------------------------------------------------------------------
        if (lane == 0) {
            // kind::f16, fp32 accumulate, A and B bf16, both K-major, N = BN, M = 128
            // (N = the tile's tokens that exist, rounded up to 16: a short expert list does not pay for the
            // whole token tile)
            const uint32_t idesc0 = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(kBM >> 4) << 24);
            const int mv = min(BN, m_cnt - m0);
            bool ok = true;
            for (int kc = 0; kc < nk && ok; kc++) {
                const int s = kc % kStages;
                const uint32_t ph = (uint32_t)(kc / kStages) & 1u;
                ok = mbar_wait_bounded(full_a + 8 * s, ph) && mbar_wait_bounded(full_b + 8 * s, ph);
                if (!ok) { atomicOr(a.status, QM_STATUS_TIMEOUT); break; }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
                for (int j = 0; j < KS; j++) {
                    const uint64_t adesc = smem_desc(smem_base + s * stage_bytes + j * a_tile);
                    const uint64_t bdesc = smem_desc(smem_base + s * stage_bytes + a_bytes + j * b_tile);
#pragma unroll
                    for (int sub = 0; sub < NSUB; sub++)
                        for (int nb = 0; nb < mv && !QM_GEMM_DEBUG_BIT(4); nb += 256) {
                            const uint32_t idesc = idesc0 | ((uint32_t)(min(256, (mv - nb + 15) & ~15) >> 3) << 17);
#pragma unroll
                            for (int k16 = 0; k16 < kBK / 16; k16++)   // 16 bf16 = 32 bytes = 2 descriptor units
                                umma_f16(tmem_base + (uint32_t)(sub * BN + nb), adesc + sub * (kATile >> 4) + 2 * k16,
                                         bdesc + (nb * 128 >> 4) + 2 * k16, idesc, (kc | j | k16) != 0);
                        }
                }
                if (QM_GEMM_DEBUG_BIT(16)) mbar_arrive(empty + 8 * (2 * s + ((kc / kStages) & 1)));
                else
                umma_commit(empty + 8 * (2 * s + ((kc / kStages) & 1)));   // frees the stage when these MMAs have read it
            }
            umma_commit(tmem_full);           // accumulator complete (or abandoned)
            QM_GEMM_STAMP(2);
        }
    } else {
        // ---- dequantize weight rows into the A tile, then the epilogue --------------------------
        // Sixteen producer warps in four groups of 128 threads. Group g converts the chunks
        // kc = g, g+4, g+8, ...: one thread per weight row turns the row's 32 quant bytes of the
        // chunk into its 64 bf16 columns. A thread's iteration is a chain of dependent steps (wait
        // for the stage, convert, store, fence, arrive); four chunks in flight hide that latency.
        // With fewer stages than groups a group's loads are in flight while it waits for a stage.
        // (Two groups — two threads per row, one per nibble half — is the other form the host can ask for.)
        const int kGroups = a.groups == 4 ? 4 : 2;
        const int pt = tid - 64;
        const int r = pt & 127;              // row of a 128-row sub-tile
        const int grp = kGroups == 4 ? pt >> 7 : pt >> 8;   // warp-uniform
        const int my_hs = kGroups == 4 ? -1 : (pt >> 7) & 1;   // the nibble half of this thread, or both
        const int rr = (n0 + r) & 15;
        const uint8_t *row_items[NSUB];
#pragma unroll
        for (int sub = 0; sub < NSUB; sub++) {
            const int sub_row = fuse_swiglu ? sub * a.up_offset : sub * kBM;   // up rows sit up_offset below the gate rows
            const int64_t tile16 = min((n0 + sub_row + r) >> 4, a.tiles16 - 1);
            row_items[sub] = wq + tile16 * a.units * QM_Q4K_ITEM_BYTES;
        }
        bool ok = true;
        // The quant bytes and headers of the group's next stage chunk are loaded right after the
        // current one has been handed over, into the same registers: the other groups' turns lie
        // between the loads and their use.
        uint4 qa[KS][NSUB], qb[KS][NSUB], hd[KS][NSUB];
#ifdef QM_DEBUG
#pragma unroll
        for (int j = 0; j < KS; j++)
#pragma unroll
            for (int sub = 0; sub < NSUB; sub++) qa[j][sub] = qb[j][sub] = hd[j][sub] = make_uint4(0x11111111u, 0x3c003c00u, 0x01010101u, 0x02020202u);
#endif
        auto load_stage = [&](int kcl) {
            if (QM_GEMM_DEBUG_BIT(8)) return;
#pragma unroll
            for (int j = 0; j < KS; j++) {
                const int c64 = (kc_lo + kcl) * KS + j;   // 64-column chunk along K
#pragma unroll
                for (int sub = 0; sub < NSUB; sub++) {
                    const uint8_t *item = row_items[sub] + (size_t)(c64 >> 2) * QM_Q4K_ITEM_BYTES;
                    hd[j][sub] = __ldg(reinterpret_cast<const uint4 *>(item + 16 * rr));
                    qa[j][sub] = __ldg(reinterpret_cast<const uint4 *>(item + 256 + 512 * (c64 & 3) + 32 * rr));
                    qb[j][sub] = __ldg(reinterpret_cast<const uint4 *>(item + 256 + 512 * (c64 & 3) + 32 * rr + 16));
                }
            }
        };
        if (grp < nk) load_stage(grp);
        for (int kc = grp; kc < nk; kc += kGroups) {
            const int s = kc % kStages;
            if (!wait_empty(kc)) { atomicOr(a.status, QM_STATUS_TIMEOUT); ok = false; break; }
#pragma unroll
            for (int j = 0; j < KS; j++) {
                const int p = ((kc_lo + kc) * KS + j) & 3;
#pragma unroll
                for (int sub = 0; sub < NSUB; sub++) {
                    if (QM_GEMM_DEBUG_BIT(1)) break;
                    // scales and minima of sub-blocks 2p (low nibbles, columns 0..31) and 2p+1 (high, 32..63)
                    const uint4 h4 = hd[j][sub];
                    uint32_t av[2], bv[2];
                    const float d = __half2float(__ushort_as_half((unsigned short)(h4.x & 0xFFFFu)));
                    const float dmin = __half2float(__ushort_as_half((unsigned short)(h4.x >> 16)));
#pragma unroll
                    for (int hs = 0; hs < 2; hs++) {
                        const int jj4 = 2 * p + hs;
                        int sc, mn;
                        if (jj4 < 4) {
                            sc = (h4.y >> (8 * jj4)) & 63;
                            mn = (h4.z >> (8 * jj4)) & 63;
                        } else {
                            const int jj = jj4 - 4;
                            sc = ((h4.w >> (8 * jj)) & 0xF) | (((h4.y >> (8 * jj + 6)) & 3) << 4);
                            mn = ((h4.w >> (8 * jj + 4)) & 0xF) | (((h4.z >> (8 * jj + 6)) & 3) << 4);
                        }
                        av[hs] = bf2(d * (float)sc);
                        bv[hs] = bf2(-dmin * (float)mn);
                    }
                    const uint32_t w[8] = {qa[j][sub].x, qa[j][sub].y, qa[j][sub].z, qa[j][sub].w,
                                           qb[j][sub].x, qb[j][sub].y, qb[j][sub].z, qb[j][sub].w};
                    uint8_t *arow = smem + (size_t)s * stage_bytes + j * a_tile + sub * kATile + r * 128;
#pragma unroll
                    for (int hs = 0; hs < 2; hs++) {
                        if (my_hs >= 0 && hs != my_hs) continue;
#pragma unroll
                        for (int c = 0; c < 4; c++) {   // 16-byte pieces (eight columns), XOR-swizzled by the row inside its 8-row group
                            uint32_t o[4];
#pragma unroll
                            for (int i = 0; i < 2; i++) {
                                // four codes of this nibble half, then each next to the byte 0x43: bf16 128+q
                                const uint32_t wv = w[2 * c + i];
                                const uint32_t nib = hs ? (wv >> 4) & 0x0F0F0F0Fu : wv & 0x0F0F0F0Fu;
                                const uint32_t p01 = prmt(nib, 0x43434343u, 0x4140u), p23 = prmt(nib, 0x43434343u, 0x4342u);
                                o[2 * i] = bfma2(bsub2(p01, 0x43004300u), av[hs], bv[hs]);
                                o[2 * i + 1] = bfma2(bsub2(p23, 0x43004300u), av[hs], bv[hs]);
                            }
                            *reinterpret_cast<uint4 *>(arow + (((c + 4 * hs) ^ (r & 7)) << 4)) = make_uint4(o[0], o[1], o[2], o[3]);
                        }
                    }
                }
            }
            if (!QM_GEMM_DEBUG_BIT(32))
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // generic writes -> tensor-core reads
            __syncwarp();
            if (lane == 0) mbar_arrive(full_a + 8 * s);   // one arrival per warp: 128 arrivals on one barrier serialize
            if (kc + kGroups < nk) load_stage(kc + kGroups);
        }
        // ---- epilogue: accumulator row r holds C[m0..m0+BN)[n0+r] -------------------------------------
        if (ok && mbar_wait_bounded(tmem_full, 0u)) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            if (tid == 64) QM_GEMM_STAMP(1);
            // the four warps of a TMEM lane quarter split the token columns that hold tokens (the rest of
            // the accumulator was never written) in blocks of 16, as evenly as the count allows
            const int blocks = (min(BN, m_cnt - m0) + 15) >> 4, q = (warp - 2) >> 2;
            const int cbeg = 16 * (q * (blocks >> 2) + min(q, blocks & 3)), cend = cbeg + 16 * ((blocks >> 2) + (q < (blocks & 3) ? 1 : 0));
            auto tmem_ld16 = [](uint32_t addr, uint32_t (&v)[16]) {
                asm volatile(
                    "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
                    : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
                      "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
                    : "r"(addr)
                    : "memory");
            };
            const uint32_t quarter_base = tmem_base + ((uint32_t)((warp & 3) * 32) << 16);   // TMEM lane quarter of this warp
            if (fuse_swiglu) {
                // gate in accumulator 0, the matching up rows in accumulator 1: h = silu(gate) * up
                const int n = n0 + (warp & 3) * 32 + lane;
                for (int c0 = cbeg; c0 < cend; c0 += 16) {
                    uint32_t g[16], u[16];
                    tmem_ld16(quarter_base + (uint32_t)c0, g);
                    tmem_ld16(quarter_base + (uint32_t)(BN + c0), u);
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                    if (n < a.n) {
                        uint16_t *hp = a.h + (int64_t)(row_off + m0 + c0) * a.ldh + n;
#pragma unroll
                        for (int j = 0; j < 16; j++) {
                            if (m0 + c0 + j < m_cnt) {
                                const float gv = __uint_as_float(g[j]), uv = __uint_as_float(u[j]);
                                // (fast division: the quotient is rounded to bf16 next; the IEEE form cost 10 us per CTA here)
                                const __nv_bfloat16 hv = __float2bfloat16_rn(__fdividef(gv, 1.f + __expf(-gv)) * uv);
                                hp[(int64_t)j * a.ldh] = *reinterpret_cast<const uint16_t *>(&hv);
                            }
                        }
                    }
                }
            } else {
#pragma unroll 1
                for (int sub = 0; sub < NSUB; sub++) {
                    const int n = n0 + sub * kBM + (warp & 3) * 32 + lane;
                    // split K: this CTA's share of the tile goes to its own plane of the scratch
                    float *base = a.splitk == 1 ? a.c : a.partials + (int64_t)zk * a.plane_rows * a.n;
                    const int64_t ld = a.splitk == 1 ? a.ldc : a.n;
                    for (int c0 = cbeg; c0 < cend; c0 += 32) {   // two blocks per wait where there are two
                        uint32_t v[16], w[16];
                        const bool two = c0 + 16 < cend;
                        tmem_ld16(quarter_base + (uint32_t)(sub * BN + c0), v);
                        if (two) tmem_ld16(quarter_base + (uint32_t)(sub * BN + c0 + 16), w);
                        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                        if (n < a.n) {
                            float *cp = base + (int64_t)(row_off + m0 + c0) * ld + n;
#pragma unroll
                            for (int j = 0; j < 16; j++)
                                if (m0 + c0 + j < m_cnt) cp[(int64_t)j * ld] = __uint_as_float(v[j]);
                            if (two) {
#pragma unroll
                                for (int j = 0; j < 16; j++)
                                    if (m0 + c0 + 16 + j < m_cnt) cp[(int64_t)(16 + j) * ld] = __uint_as_float(w[j]);
                            }
                        }
                    }
                }
            }
        } else if (ok) {
            atomicOr(a.status, QM_STATUS_TIMEOUT);
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (tid == 0) QM_GEMM_STAMP(3);
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(tmem_cols) : "memory");
    }
    if (a.splitk > 1) {
        // Every CTA of the tile adds one band of it, in order of z, once all splitk shares are in the scratch:
        // the launch is cooperative (all CTAs resident), the wait for the others is bounded. (The barrier
        // above ordered every thread's stores before thread 0's fence and arrival.)
        volatile uint32_t *s_ok = tmem_slot + 1;   // a free word of the dynamic shared memory's tail
        const unsigned int tile_id = a.grouped ? ((blockIdx.z / a.splitk) * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x
                                               : blockIdx.y * gridDim.x + blockIdx.x;
        unsigned int *ticket = a.tickets + 2 * tile_id;
        if (tid == 0) {
            __threadfence();
            atomicAdd(ticket, 1u);
            const long long t0 = clock64();
            bool ok = true;
            while (ld_acquire(ticket) < (unsigned int)a.splitk) {
                if (clock64() - t0 > a.wait_cycles) { atomicOr(a.status, QM_STATUS_TIMEOUT); ok = false; break; }
            }
            *s_ok = ok ? 1u : 0u;
        }
        __syncthreads();
        if (*s_ok) {
            const int rows = min(NSUB * kBM, a.n - n0), toks = min(BN, m_cnt - m0);
            const int t_lo = (int)((int64_t)toks * zk / a.splitk) + row_off, t_hi = (int)((int64_t)toks * (zk + 1) / a.splitk) + row_off;
            const int64_t plane = (int64_t)a.plane_rows * a.n;
            if ((rows & 3) == 0 && (a.n & 3) == 0 && (a.ldc & 3) == 0 && (reinterpret_cast<uintptr_t>(a.c) & 15) == 0) {
                // 16 bytes per thread and four of them in flight: the loop is bound by the latency of its loads
                const int r4 = rows >> 2, total = r4 * (t_hi - t_lo), step = (int)blockDim.x;
                for (int i0 = tid; i0 < total; i0 += 4 * step) {
                    float4 acc[4];
#pragma unroll
                    for (int u = 0; u < 4; u++) {
                        const int i = i0 + u * step;
                        acc[u] = make_float4(0.f, 0.f, 0.f, 0.f);
                        if (i < total) {
                            const int mm = t_lo + i / r4, nn = (i % r4) << 2;
                            const float *src = a.partials + (int64_t)(m0 + mm) * a.n + n0 + nn;
                            for (int z = 0; z < a.splitk; z++) {
                                const float4 v = __ldcg(reinterpret_cast<const float4 *>(src + z * plane));
                                acc[u].x += v.x; acc[u].y += v.y; acc[u].z += v.z; acc[u].w += v.w;
                            }
                        }
                    }
#pragma unroll
                    for (int u = 0; u < 4; u++) {
                        const int i = i0 + u * step;
                        if (i < total) {
                            const int mm = t_lo + i / r4, nn = (i % r4) << 2;
                            *reinterpret_cast<float4 *>(a.c + (int64_t)(m0 + mm) * a.ldc + n0 + nn) = acc[u];
                        }
                    }
                }
            } else {
                for (int i = tid; i < rows * (t_hi - t_lo); i += blockDim.x) {
                    const int mm = t_lo + i / rows, nn = i % rows;
                    const int64_t at = (int64_t)(m0 + mm) * a.n + n0 + nn;
                    float sum = 0.f;
                    for (int z = 0; z < a.splitk; z++) sum += __ldcg(a.partials + z * plane + at);
                    a.c[(int64_t)(m0 + mm) * a.ldc + n0 + nn] = sum;
                }
            }
        }
        // the last CTA to finish its band zeroes the tile's two words for the next launch
        __syncthreads();
        if (tid == 0 && atomicAdd(ticket + 1, 1u) + 1u == (unsigned int)a.splitk) {
            ticket[0] = 0u;
            ticket[1] = 0u;
        }
    }
}

extern "C" __global__ void __launch_bounds__(576, 1) qm_gemm_q4k_bf16(const __grid_constant__ QmGemmArgs a) {
    gemm_body<1, 1>(a);
}
extern "C" __global__ void __launch_bounds__(576, 1) qm_gemm_q4k_bf16_r256(const __grid_constant__ QmGemmArgs a) {
    gemm_body<2, 1>(a);
}
// Two 64-column chunks per stage (small token tiles).
extern "C" __global__ void __launch_bounds__(576, 1) qm_gemm_q4k_bf16_k128(const __grid_constant__ QmGemmArgs a) {
    gemm_body<1, 2>(a);
}
extern "C" __global__ void __launch_bounds__(576, 1) qm_gemm_q4k_bf16_r256_k128(const __grid_constant__ QmGemmArgs a) {
    gemm_body<2, 2>(a);
}
