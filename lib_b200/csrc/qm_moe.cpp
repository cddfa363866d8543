// qm_moe.cpp — host side of the mixture-of-experts path: routing and the grouped expert
// matmul that reuses the quantized prefill GEMM over per-expert token lists.
// The Go-facing surface it stands behind is lm/moe: GroupedTopKRouter.Route
// (lm/moe/moe.go:73-141) for the routing; the grouped matmul is new API of this path.
#include <string.h>

#include <algorithm>
#include <vector>

#include "qm_internal.h"

static unsigned grid_for(int64_t work, int block, int cap) {
    return (unsigned)std::max<int64_t>(1, std::min<int64_t>((work + block - 1) / block, cap));
}

extern "C" int32_t qm_moe_route(qm_ctx *c, uint64_t logits_dev, int32_t tokens, int64_t ld, int32_t experts,
                                int32_t topk, uint64_t bias_dev, uint64_t ids_dev, uint64_t weights_dev) {
    CHECK_CTX(c);
    if (!logits_dev || !ids_dev || !weights_dev) return QM_ERR_ARG;
    if (tokens < 0 || experts < 1 || experts > QM_MAX_EXPERTS || topk < 0 || topk > experts || ld < experts) return QM_ERR_SHAPE;
    if (tokens == 0 || topk == 0) return QM_OK;
    CtxGuard g(c);
    DRV(g.rc);
    QmRouteArgs a;
    memset(&a, 0, sizeof a);
    a.logits = (const float *)(uintptr_t)logits_dev;
    a.bias = (const float *)(uintptr_t)bias_dev;
    a.ids = (int32_t *)(uintptr_t)ids_dev;
    a.weights = (float *)(uintptr_t)weights_dev;
    a.ld = ld;
    a.tokens = tokens;
    a.experts = experts;
    a.topk = topk;
    return qm_launch(c, QM_K_MOE_ROUTE, (unsigned)((tokens + 127) / 128), 1, 128, 0, &a, false);
}

// Three growing scratch areas, one per stage, so that the stages can call one another:
// the dispatch lists, the expert intermediates, and the grouped call's rows and outputs.
static int32_t grow(qm_ctx *c, CUdeviceptr *p, int64_t *have, int64_t bytes) {
    if (bytes <= *have) return QM_OK;
    DRV(c->drv->cuStreamSynchronize(c->stream));
    if (*p) DRV(c->drv->cuMemFree_v2(*p));
    *p = 0;
    *have = 0;
    DRV(c->drv->cuMemAlloc_v2(p, (size_t)bytes));
    *have = bytes;
    return QM_OK;
}
static int32_t ensure_ws(qm_ctx *c, int64_t bytes) { return grow(c, &c->moe_ws, &c->moe_ws_bytes, bytes); }
static int32_t ensure_ws2(qm_ctx *c, int64_t bytes) { return grow(c, &c->moe_ws2, &c->moe_ws2_bytes, bytes); }
static int32_t ensure_ws3(qm_ctx *c, int64_t bytes) { return grow(c, &c->moe_ws3, &c->moe_ws3_bytes, bytes); }

static int32_t check_experts(const qm_weight *gate_up, const qm_weight *down, int32_t experts,
                             std::vector<QmWeight *> &wg, std::vector<QmWeight *> &wd, int64_t *hidden, int64_t *ffn) {
    if (!gate_up || !down) return QM_ERR_ARG;
    if (experts < 1 || experts > QM_MAX_EXPERTS) return QM_ERR_SHAPE;
    wg.resize(experts);
    wd.resize(experts);
    for (int e = 0; e < experts; e++) {
        wg[e] = qm_weight_from_handle(gate_up[e]);
        wd[e] = qm_weight_from_handle(down[e]);
        if (!wg[e] || !wd[e]) return QM_ERR_ARG;
        if (wg[e]->fmt != QM_FMT_Q4_K || wd[e]->fmt != QM_FMT_Q4_K) return QM_ERR_FORMAT;
    }
    *hidden = wg[0]->cols;
    *ffn = wd[0]->cols;
    for (int e = 0; e < experts; e++)
        if (wg[e]->cols != *hidden || wg[e]->rows != 2 * *ffn || wd[e]->rows != *hidden || wd[e]->cols != *ffn)
            return QM_ERR_SHAPE;
    if ((*hidden & 7) || (*ffn & 7)) return QM_ERR_SHAPE;
    return QM_OK;
}

static inline int64_t up256(int64_t v) { return (v + 255) & ~(int64_t)255; }

// Groups the (token, slot) pairs by expert and copies the bf16 rows of their tokens into that
// order. Blocks until the list lengths are on the host: the caller sizes its launches (and, in
// expert-parallel runs, its exchange) with them.
// counts_host == nullptr: nothing is read back (no synchronization); the gather then covers all
// pairs and *offsets_dev_out names the device array [experts + 1] of list starts.
static int32_t dispatch_impl(qm_ctx *c, uint64_t ids_dev, int32_t tokens, int32_t topk, int32_t experts,
                             uint64_t x_bf16_dev, int64_t ldx, int32_t hidden, uint64_t rows_dev, uint64_t pos_dev,
                             int32_t *counts_host, CUdeviceptr *offsets_dev_out, CUdeviceptr *list_dev_out = nullptr) {
    CHECK_CTX(c);
    // list_dev_out: the caller's matmul fetches the rows by the list itself; nothing is copied here
    if (!ids_dev || !x_bf16_dev || (!rows_dev && !list_dev_out) || !pos_dev) return QM_ERR_ARG;
    if (experts < 1 || experts > QM_MAX_EXPERTS || tokens < 0 || topk < 1 || hidden < 8 || (hidden & 7) || ldx < hidden ||
        (x_bf16_dev & 15) || (rows_dev & 15) || ((ldx * 2) & 15))
        return QM_ERR_SHAPE;
    for (int e = 0; e < experts && counts_host; e++) counts_host[e] = 0;
    if (tokens == 0) return QM_OK;
    CtxGuard g(c);
    DRV(g.rc);
    const int64_t pairs = (int64_t)tokens * topk;
    const int64_t o_rank = 0, o_counts = up256(pairs * 4), o_offsets = o_counts + up256(QM_MAX_EXPERTS * 4),
                  o_list = o_offsets + up256((QM_MAX_EXPERTS + 1) * 4), total = o_list + up256(pairs * 4);
    int32_t rc = ensure_ws(c, total);
    if (rc) return rc;
    const CUdeviceptr ws = c->moe_ws;
    QmListArgs la;
    memset(&la, 0, sizeof la);
    la.ids = (const int32_t *)(uintptr_t)ids_dev;
    la.rank = (int32_t *)(uintptr_t)(ws + o_rank);
    la.counts = (int32_t *)(uintptr_t)(ws + o_counts);
    la.offsets = (int32_t *)(uintptr_t)(ws + o_offsets);
    la.list = (int32_t *)(uintptr_t)(ws + o_list);
    la.pos = (int32_t *)(uintptr_t)pos_dev;
    la.tokens = tokens;
    la.experts = experts;
    la.topk = topk;
    rc = qm_launch(c, QM_K_MOE_LISTS, 1, 1, 1024, 0, &la, false);
    if (rc) return rc;
    if (offsets_dev_out) *offsets_dev_out = ws + o_offsets;
    if (list_dev_out) *list_dev_out = ws + o_list;
    int rows = (int)pairs;   // every pair names an expert, so the lists hold all pairs
    if (counts_host) {
        int32_t offsets[QM_MAX_EXPERTS + 1];
        DRV(c->drv->cuMemcpyDtoHAsync_v2(offsets, ws + o_offsets, (size_t)(experts + 1) * 4, c->stream));
        DRV(c->drv->cuStreamSynchronize(c->stream));
        rows = offsets[experts];
        if (rows < 0 || rows > pairs) return QM_ERR_STATE;
        for (int e = 0; e < experts; e++) counts_host[e] = offsets[e + 1] - offsets[e];
        if (rows == 0) return QM_OK;
    }
    if (list_dev_out) return QM_OK;
    QmGatherArgs ga;
    memset(&ga, 0, sizeof ga);
    ga.x = (const uint16_t *)(uintptr_t)x_bf16_dev;
    ga.list = (const int32_t *)(uintptr_t)(ws + o_list);
    ga.out = (uint16_t *)(uintptr_t)rows_dev;
    ga.ldx = ldx;
    ga.rows = rows;
    ga.hidden = hidden;
    ga.topk = topk;
    return qm_launch(c, QM_K_MOE_GATHER, grid_for((int64_t)rows * hidden / 8, 256, c->sm_count * 8), 1, 256, 0, &ga, false);
}

extern "C" int32_t qm_moe_dispatch(qm_ctx *c, uint64_t ids_dev, int32_t tokens, int32_t topk, int32_t experts,
                                   uint64_t x_bf16_dev, int64_t ldx, int32_t hidden, uint64_t rows_dev,
                                   uint64_t pos_dev, int32_t *counts_host) {
    if (!counts_host) return QM_ERR_ARG;
    return dispatch_impl(c, ids_dev, tokens, topk, experts, x_bf16_dev, ldx, hidden, rows_dev, pos_dev, counts_host,
                         nullptr);
}

// The two grouped launches over rows grouped by expert (list starts in offsets_dev): gate|up with
// the SwiGLU in the epilogue (bf16 h in the stage's workspace), then down into y. `longest`
// bounds the list lengths (sizes the grid), `typical` chooses the token tile.
static int32_t experts_launch(qm_ctx *c, const std::vector<QmWeight *> &wg, const std::vector<QmWeight *> &wd,
                              int32_t experts, uint64_t rows_bf16_dev, int64_t rows, int32_t longest, int32_t typical,
                              CUdeviceptr offsets_dev, uint64_t y_dev, int64_t hidden, int64_t ffn,
                              CUdeviceptr gather_list_dev = 0, int gather_topk = 0, int64_t x_rows = 0, int64_t ldx = 0) {
    const int64_t o_h = 0, o_gl = up256(rows * ffn * 2) + up256((QM_MAX_EXPERTS + 1) * 4), o_dl = o_gl + QM_MAX_EXPERTS * 8,
                  total = o_dl + QM_MAX_EXPERTS * 8;
    int32_t rc = ensure_ws2(c, total);
    if (rc) return rc;
    const CUdeviceptr ws = c->moe_ws2;
    uint64_t lists[2][QM_MAX_EXPERTS];
    for (int e = 0; e < experts; e++) {
        lists[0][e] = (uint64_t)wg[e]->wq;
        lists[1][e] = (uint64_t)wd[e]->wq;
    }
    DRV(c->drv->cuMemcpyHtoDAsync_v2(ws + o_gl, lists[0], (size_t)experts * 8, c->stream));
    DRV(c->drv->cuMemcpyHtoDAsync_v2(ws + o_dl, lists[1], (size_t)experts * 8, c->stream));
    QmGemmGroup grp;
    memset(&grp, 0, sizeof grp);
    grp.experts = experts;
    grp.m_typical = typical;
    grp.offsets_dev = offsets_dev;
    grp.wq_list_dev = ws + o_gl;
    grp.swiglu = true;
    grp.h_dev = ws + o_h;
    grp.ldh = ffn;
    if (gather_list_dev) {   // rows_bf16_dev holds the tokens' rows as the caller has them; the matmul gathers
        grp.gather_list_dev = gather_list_dev;
        grp.gather_topk = gather_topk;
        rc = qm_gemm_launch(c, wg[0], rows_bf16_dev, longest, x_rows, ldx, 0, 0, grp);
        grp.gather_list_dev = 0;
    } else {
        rc = qm_gemm_launch(c, wg[0], rows_bf16_dev, longest, rows, hidden, 0, 0, grp);
    }
    if (rc) return rc;
    grp.wq_list_dev = ws + o_dl;
    grp.swiglu = false;
    grp.h_dev = 0;
    return qm_gemm_launch(c, wd[0], ws + o_h, longest, rows, ffn, y_dev, hidden, grp);
}

// y[p][:] = down_e( silu(gate_e r_p) * (up_e r_p) ) for rows r grouped by expert: the first
// counts[0] rows belong to expert 0, the next counts[1] to expert 1, and so on. Two launches
// for all experts together: gate|up with the SwiGLU in the epilogue (bf16 h), then down.
extern "C" int32_t qm_moe_experts(qm_ctx *c, const qm_weight *gate_up, const qm_weight *down, int32_t experts,
                                  uint64_t rows_bf16_dev, const int32_t *counts_host, uint64_t y_dev) {
    CHECK_CTX(c);
    if (!rows_bf16_dev || !counts_host || !y_dev) return QM_ERR_ARG;
    std::vector<QmWeight *> wg, wd;
    int64_t hidden = 0, ffn = 0;
    int32_t rc = check_experts(gate_up, down, experts, wg, wd, &hidden, &ffn);
    if (rc) return rc;
    if ((rows_bf16_dev & 15) || (ffn & 127)) return QM_ERR_SHAPE;   // SwiGLU epilogue: whole 128-row tiles of gate rows
    int64_t rows = 0;
    int32_t longest = 0;
    int32_t offsets[QM_MAX_EXPERTS + 1];
    for (int e = 0; e < experts; e++) {
        if (counts_host[e] < 0) return QM_ERR_COUNT;
        offsets[e] = (int32_t)rows;
        rows += counts_host[e];
        longest = std::max(longest, counts_host[e]);
    }
    offsets[experts] = (int32_t)rows;
    if (rows == 0) return QM_OK;
    if (rows >= (1 << 24)) return QM_ERR_SHAPE;
    CtxGuard g(c);
    DRV(g.rc);
    // workspace: the bf16 hidden activations, the offsets, then the two lists of weight stores
    const int64_t o_off = up256(rows * ffn * 2), total = o_off + up256((QM_MAX_EXPERTS + 1) * 4) + 2 * QM_MAX_EXPERTS * 8;
    rc = ensure_ws2(c, total);
    if (rc) return rc;
    const CUdeviceptr ws = c->moe_ws2;
    // the offsets travel in stream order; the host copy is read before the call returns
    DRV(c->drv->cuMemcpyHtoDAsync_v2(ws + o_off, offsets, (size_t)(experts + 1) * 4, c->stream));
    return experts_launch(c, wg, wd, experts, rows_bf16_dev, rows, longest, longest, ws + o_off, y_dev, hidden, ffn);
}

// out[t][:] = sum_s weights[t][s] * y[pos[t*topk+s]][:], slots in order (deterministic).
extern "C" int32_t qm_moe_combine(qm_ctx *c, uint64_t y_dev, uint64_t pos_dev, uint64_t weights_dev, int32_t tokens,
                                  int32_t topk, int32_t hidden, uint64_t out_dev, int64_t ldo) {
    CHECK_CTX(c);
    if (!y_dev || !pos_dev || !weights_dev || !out_dev) return QM_ERR_ARG;
    if (tokens < 0 || topk < 1 || hidden < 1 || ldo < hidden) return QM_ERR_SHAPE;
    if (tokens == 0) return QM_OK;
    CtxGuard g(c);
    DRV(g.rc);
    QmCombineArgs a;
    memset(&a, 0, sizeof a);
    a.y = (const float *)(uintptr_t)y_dev;
    a.pos = (const int32_t *)(uintptr_t)pos_dev;
    a.weights = (const float *)(uintptr_t)weights_dev;
    a.out = (float *)(uintptr_t)out_dev;
    a.ldo = ldo;
    a.tokens = tokens;
    a.hidden = hidden;
    a.topk = topk;
    return qm_launch(c, QM_K_MOE_COMBINE, grid_for((int64_t)tokens * hidden, 256, c->sm_count * 8), 1, 256, 0, &a, false);
}

// out[t][:] = sum_s weights[t][s] * down_e( silu(gate_e x_t) * (up_e x_t) ), e = ids[t][s].
// gate_up[e]: stored Q4_K [2*ffn][hidden] (gate rows then up rows); down[e]: [hidden][ffn].
extern "C" int32_t qm_moe_grouped(qm_ctx *c, const qm_weight *gate_up, const qm_weight *down, int32_t experts,
                                  uint64_t x_bf16_dev, int32_t tokens, int64_t ldx, uint64_t ids_dev,
                                  uint64_t weights_dev, int32_t topk, uint64_t out_dev, int64_t ldo) {
    CHECK_CTX(c);
    if (!x_bf16_dev || !ids_dev || !weights_dev || !out_dev) return QM_ERR_ARG;
    if (tokens < 1 || topk < 1 || topk > experts) return QM_ERR_SHAPE;
    std::vector<QmWeight *> wg, wd;
    int64_t hidden = 0, ffn = 0;
    int32_t rc = check_experts(gate_up, down, experts, wg, wd, &hidden, &ffn);
    if (rc) return rc;
    if (ldx < hidden || ldo < hidden) return QM_ERR_SHAPE;
    const int64_t pairs = (int64_t)tokens * topk;
    const int64_t o_rows = 0, o_pos = up256(pairs * hidden * 2), o_y = o_pos + up256(pairs * 4),
                  total = o_y + up256(pairs * hidden * 4);
    {
        CtxGuard g(c);
        DRV(g.rc);
        rc = ensure_ws3(c, total);
        if (rc) return rc;
    }
    const CUdeviceptr ws = c->moe_ws3;
    if (ffn & 127) return QM_ERR_SHAPE;
    // Default: the list lengths are read back once, so that the grouped launches have exactly the
    // token tiles that hold rows (measured 0.75 ms per Mixtral-shaped layer). QM_MOE_NOSYNC=1
    // keeps everything on the device instead: the launches then cover the longest possible list
    // (all pairs) and the CTAs beyond an expert's rows leave at once — no synchronization, but
    // those thousands of empty CTAs each hold an SM's shared memory for a moment (0.95 ms).
    // QM_MOE_FOLD=1: the gate|up matmul fetches each grouped row from the token's own row of x (its
    // loader warp follows the dispatch list with tile::gather4 copies), so no gathered copy is written.
    // Same bits as the separate gather pass (the matmul sees the same rows in the same order), but
    // slower at the Mixtral shape: a gather4 copy moves 512 bytes and one SM completes one every ~26 ns,
    // which is 20 GB/s per SM where the 256-token tiles want 51 GB/s (1.62 ms per layer against
    // 0.82 ms; the same loader with 16-byte cp.async from one warp: 1.32 ms), while the pass it
    // saves costs about 5 us. So the separate pass stays the default.
    const bool fold = qm_env_int("QM_MOE_FOLD", 0) != 0 && (x_bf16_dev & 15) == 0 && (ldx & 7) == 0;
    const bool nosync = qm_env_int("QM_MOE_NOSYNC", 0) != 0;
    if (fold) {
        int32_t counts[QM_MAX_EXPERTS];
        CUdeviceptr offsets_dev = 0, list_dev = 0;
        rc = dispatch_impl(c, ids_dev, tokens, topk, experts, x_bf16_dev, ldx, (int32_t)hidden, 0, ws + o_pos,
                           nosync ? nullptr : counts, &offsets_dev, &list_dev);
        if (rc) return rc;
        int32_t longest = (int32_t)pairs, typical = (int32_t)std::max<int64_t>(1, (pairs + experts - 1) / experts);
        if (!nosync) {
            longest = 0;
            for (int e = 0; e < experts; e++) longest = std::max(longest, counts[e]);
            typical = longest;
        }
        if (longest > 0) {
            CtxGuard g(c);
            DRV(g.rc);
            rc = experts_launch(c, wg, wd, experts, x_bf16_dev, pairs, longest, typical, offsets_dev, ws + o_y, hidden, ffn,
                                list_dev, topk, tokens, ldx);
            if (rc) return rc;
        }
        return qm_moe_combine(c, ws + o_y, ws + o_pos, weights_dev, tokens, topk, (int32_t)hidden, out_dev, ldo);
    }
    if (!nosync) {
        int32_t counts[QM_MAX_EXPERTS];
        rc = qm_moe_dispatch(c, ids_dev, tokens, topk, experts, x_bf16_dev, ldx, (int32_t)hidden, ws + o_rows, ws + o_pos,
                             counts);
        if (rc) return rc;
        rc = qm_moe_experts(c, gate_up, down, experts, ws + o_rows, counts, ws + o_y);
        if (rc) return rc;
        return qm_moe_combine(c, ws + o_y, ws + o_pos, weights_dev, tokens, topk, (int32_t)hidden, out_dev, ldo);
    }
    CUdeviceptr offsets_dev = 0;
    rc = dispatch_impl(c, ids_dev, tokens, topk, experts, x_bf16_dev, ldx, (int32_t)hidden, ws + o_rows, ws + o_pos,
                       nullptr, &offsets_dev);
    if (rc) return rc;
    {
        CtxGuard g(c);
        DRV(g.rc);
        const int32_t typical = (int32_t)std::max<int64_t>(1, (pairs + experts - 1) / experts);
        rc = experts_launch(c, wg, wd, experts, ws + o_rows, pairs, (int32_t)pairs, typical, offsets_dev, ws + o_y, hidden,
                            ffn);
        if (rc) return rc;
    }
    return qm_moe_combine(c, ws + o_y, ws + o_pos, weights_dev, tokens, topk, (int32_t)hidden, out_dev, ldo);
}

// ---- decode-time MoE over selected experts ----------------------------------------------------
// One persistent launch of the data-driven decode kernel runs every (token, slot) pair of a small
// batch as two dependent matvecs of one activation row: gate|up of the slot's expert on the token's
// x, then down on silu(gate) * up. Which expert a pair uses is read on the device (QmOp::sel_*),
// so the host never sees the router's output. The reference's counterpart is the pair of
// *_selected_matvec_q8_1 kernels (nvidia/x/egraph/codegen.go:554-616), one launch per projection,
// one warp per row.
struct qm_moe_decode {
    uint32_t magic;
    int experts, topk, max_tokens;
    int64_t hidden, ffn;
    std::vector<const QmWeight *> gu, dn;
    CUdeviceptr tables;      // [2][experts] device pointers: gate|up stores, then down stores
    CUdeviceptr bufs;        // per pair: gate|up output [2*ffn], then per pair: down output [hidden]
    CUdeviceptr ops_dev;
    CUdeviceptr sync;
    QmFusedPlan plan;
    int kernel;
    // what the device op list was built for
    int built_tokens;
    uint64_t built_x, built_ids;
    int64_t built_ldx;
};
#define QM_MOE_DECODE_MAGIC 0x514D4D44u   // "QMMD"
#define QM_MOE_DECODE_MAX_PAIRS 32

extern "C" int32_t qm_moe_decode_destroy(qm_ctx *c, qm_moe_decode *d) {
    CHECK_CTX(c);
    if (!d || d->magic != QM_MOE_DECODE_MAGIC) return QM_ERR_ARG;
    CtxGuard g(c);
    DRV(g.rc);
    c->drv->cuStreamSynchronize(c->stream);
    if (d->tables) c->drv->cuMemFree_v2(d->tables);
    if (d->bufs) c->drv->cuMemFree_v2(d->bufs);
    if (d->ops_dev) c->drv->cuMemFree_v2(d->ops_dev);
    if (d->sync) c->drv->cuMemFree_v2(d->sync);
    d->magic = 0;
    delete d;
    return QM_OK;
}

extern "C" int32_t qm_moe_decode_create(qm_ctx *c, const qm_weight *gate_up, const qm_weight *down, int32_t experts,
                                        int32_t topk, int32_t max_tokens, qm_moe_decode **out) {
    CHECK_CTX(c);
    if (!gate_up || !down || !out) return QM_ERR_ARG;
    *out = nullptr;
    if (experts < 1 || experts > 4096 || topk < 1 || topk > experts || max_tokens < 1 ||
        (int64_t)max_tokens * topk > QM_MOE_DECODE_MAX_PAIRS)
        return QM_ERR_SHAPE;
    qm_moe_decode *d = new (std::nothrow) qm_moe_decode();
    if (!d) return QM_ERR_NOMEM;
    d->magic = QM_MOE_DECODE_MAGIC;
    d->experts = experts;
    d->topk = topk;
    d->max_tokens = max_tokens;
    d->built_tokens = 0;
    for (int e = 0; e < experts; e++) {
        const QmWeight *g = qm_weight_from_handle(gate_up[e]), *dn = qm_weight_from_handle(down[e]);
        int32_t bad = QM_OK;
        if (!g || !dn) bad = QM_ERR_ARG;
        else if (g->fmt != QM_FMT_Q4_K || dn->fmt != QM_FMT_Q4_K) bad = QM_ERR_FORMAT;
        else if (g->device != c->device || dn->device != c->device) bad = QM_ERR_ARG;
        else if (e == 0) {
            d->hidden = g->cols;
            d->ffn = dn->cols;
        }
        if (!bad && (g->cols != d->hidden || g->rows != 2 * d->ffn || dn->cols != d->ffn || dn->rows != d->hidden))
            bad = QM_ERR_SHAPE;
        if (bad) {
            delete d;
            return bad;
        }
        d->gu.push_back(g);
        d->dn.push_back(dn);
    }
    const int max_units = (int)std::max(d->gu[0]->units, d->dn[0]->units);
    if (qm_plan_fused(c, 1, max_units, false, &d->plan) != QM_OK || d->plan.consumers != 16 || d->plan.depth < 2 ||
        d->plan.depth > 4) {
        delete d;
        return QM_ERR_SHAPE;
    }
    d->kernel = QM_K_FUSED_Q4K_DD_C4D2_SEL + (d->plan.depth - 2);
    CtxGuard g(c);
    if (g.rc != CUDA_SUCCESS) {
        delete d;
        return (int32_t)g.rc;
    }
    std::vector<uint64_t> tab((size_t)2 * experts);
    for (int e = 0; e < experts; e++) {
        tab[e] = (uint64_t)d->gu[e]->wq;
        tab[experts + e] = (uint64_t)d->dn[e]->wq;
    }
    const int64_t pairs = (int64_t)max_tokens * topk;
    CUresult r = c->drv->cuMemAlloc_v2(&d->tables, tab.size() * 8);
    if (r == CUDA_SUCCESS) r = c->drv->cuMemcpyHtoD_v2(d->tables, tab.data(), tab.size() * 8);
    if (r == CUDA_SUCCESS) r = c->drv->cuMemAlloc_v2(&d->bufs, (size_t)(pairs * (2 * d->ffn + d->hidden) * 4));
    if (r == CUDA_SUCCESS) r = c->drv->cuMemAlloc_v2(&d->ops_dev, (size_t)(2 * pairs) * sizeof(QmOp));
    if (r == CUDA_SUCCESS) r = c->drv->cuMemAlloc_v2(&d->sync, 256);
    if (r != CUDA_SUCCESS) {
        qm_moe_decode_destroy(c, d);
        return (int32_t)r;
    }
    *out = d;
    return QM_OK;
}

extern "C" int32_t qm_moe_decode_run(qm_ctx *c, qm_moe_decode *d, uint64_t x_dev, int32_t tokens, int64_t ldx,
                                     uint64_t ids_dev, uint64_t weights_dev, uint64_t out_dev, int64_t ldo) {
    CHECK_CTX(c);
    if (!d || d->magic != QM_MOE_DECODE_MAGIC) return QM_ERR_ARG;
    if (tokens < 0 || tokens > d->max_tokens || ldx < d->hidden || ldo < d->hidden || (ldx & 3)) return QM_ERR_SHAPE;
    if (!x_dev || !ids_dev || !weights_dev || !out_dev || (x_dev & 15) || (ids_dev & 3) || (weights_dev & 3))
        return QM_ERR_ARG;
    if (tokens == 0) return QM_OK;
    CtxGuard g(c);
    DRV(g.rc);
    const int pairs = tokens * d->topk;
    const int64_t gu_floats = 2 * d->ffn;
    const CUdeviceptr gu0 = d->bufs, dn0 = d->bufs + (size_t)((int64_t)d->max_tokens * d->topk * gu_floats * 4);
    if (tokens != d->built_tokens || x_dev != d->built_x || ids_dev != d->built_ids || ldx != d->built_ldx) {
        // all gate|up ops first: by the time a pair's down op stages its x, that x has long been written
        std::vector<QmOp> ops((size_t)2 * pairs);
        for (int pr = 0; pr < pairs; pr++) {
            const int t = pr / d->topk;
            QmOp &a = ops[pr], &b = ops[pairs + pr];
            const CUdeviceptr gu = gu0 + (size_t)pr * gu_floats * 4, dn = dn0 + (size_t)pr * d->hidden * 4;
            qm_fill_op(c, d->plan, d->gu[0], x_dev + (size_t)t * ldx * 4, 0, ldx, gu, gu_floats, QM_XOP_NONE, 0, 0,
                       d->gu[0]->units, 0, &a);
            qm_fill_op(c, d->plan, d->dn[0], gu, gu + (size_t)d->ffn * 4, gu_floats, dn, d->hidden, QM_XOP_SWIGLU, 1, 0,
                       d->dn[0]->units, 0, &b);
            a.sel_table = (const uint8_t *const *)(uintptr_t)d->tables;
            b.sel_table = (const uint8_t *const *)(uintptr_t)(d->tables + (size_t)d->experts * 8);
            a.sel_ids = b.sel_ids = (const int32_t *)(uintptr_t)ids_dev;
            a.sel_index = b.sel_index = pr;
            a.sel_count = b.sel_count = d->experts;
        }
        DRV(c->drv->cuStreamSynchronize(c->stream));   // the list in use may still be read
        DRV(c->drv->cuMemcpyHtoD_v2(d->ops_dev, ops.data(), ops.size() * sizeof(QmOp)));
        d->built_tokens = tokens;
        d->built_x = x_dev;
        d->built_ids = ids_dev;
        d->built_ldx = ldx;
    }
    // every output word starts as "not yet written" (all ones)
    DRV(c->drv->cuMemsetD32Async(gu0, 0xFFFFFFFFu, (size_t)pairs * gu_floats, c->stream));
    DRV(c->drv->cuMemsetD32Async(dn0, 0xFFFFFFFFu, (size_t)pairs * d->hidden, c->stream));
    DRV(c->drv->cuMemsetD32Async(d->sync, 0, 64, c->stream));
    QmFusedArgs a;
    memset(&a, 0, sizeof a);
    a.ops = (const QmOp *)(uintptr_t)d->ops_dev;
    a.status = (unsigned int *)(uintptr_t)c->status_dev;
    a.grid_bar = (unsigned int *)(uintptr_t)d->sync;
    a.nops = 2 * pairs;
    a.ngroups = 1;
    a.m = 1;
    a.consumers = d->plan.consumers;
    a.depth = d->plan.depth;
    a.max_units = d->plan.max_units;
    a.cpm = d->plan.cpm;
    a.wait_cycles = qm_wait_cycles();
    // no programmatic launch: the ids must be complete before the first copy is issued; cooperative: the CTAs
    // poll one another's outputs and must all be resident
    int32_t rc = qm_launch_ex(c, d->kernel, (unsigned)qm_fused_grid(c), (unsigned)d->plan.consumers * 32,
                              (unsigned)d->plan.smem, &a, false, true);
    if (rc) return rc;
    QmDecodeCombineArgs ca;
    memset(&ca, 0, sizeof ca);
    ca.y = (const float *)(uintptr_t)dn0;
    ca.ids = (const int32_t *)(uintptr_t)ids_dev;
    ca.weights = (const float *)(uintptr_t)weights_dev;
    ca.out = (float *)(uintptr_t)out_dev;
    ca.ldo = ldo;
    ca.tokens = tokens;
    ca.topk = d->topk;
    ca.experts = d->experts;
    ca.hidden = (int32_t)d->hidden;
    return qm_launch(c, QM_K_MOE_DECODE_COMBINE, grid_for((int64_t)tokens * d->hidden, 256, c->sm_count * 4), 1, 256, 0,
                     &ca, false);
}

// ---- expert parallelism behind the C ABI ------------------------------------------------------------
// Rank r of `world` owns experts [r*eloc, (r+1)*eloc). A step moves the routed rows to their owners and the
// results back through peer memory (the kernels of qm_moe.cu, qm_ep_*), so a caller needs no collective
// library for it: the ranks exchange one 64-byte IPC handle each at set-up (or, in one process, plain
// pointers), as for the tensor-parallel decode stack. Every rank must run the same number of steps.
struct qm_ep {
    uint32_t magic;
    int eloc, experts, topk, max_tokens, cap, rank, world;
    int64_t hidden, ffn;
    std::vector<QmWeight *> wg, wd;
    CUdeviceptr arena;          // flags | counts_in | rows_in | ret_in (the part the peers write)
    int64_t arena_bytes, o_flags, o_counts, o_rows, o_ret;
    CUdeviceptr local;          // lists | compact | back | loff | y | done
    int64_t o_rankbuf, o_lcounts, o_offsets, o_list, o_pos, o_compact, o_back, o_loff, o_y, o_done;
    CUdeviceptr peer_base[QM_MAX_PEERS];
    bool peers_open, peers_ipc;
    unsigned int epoch;
    // the step in flight between begin and end
    QmEpArgs step;
    int phase;                  // 0: idle, 1: after begin, 2: after run
};
#define QM_EP_MAGIC 0x514D4550u   // "QMEP"

static bool ep_check(qm_ep *e) { return e && e->magic == QM_EP_MAGIC; }

extern "C" int32_t qm_ep_destroy(qm_ctx *c, qm_ep *e) {
    CHECK_CTX(c);
    if (!ep_check(e)) return QM_ERR_ARG;
    CtxGuard g(c);
    DRV(g.rc);
    c->drv->cuStreamSynchronize(c->stream);
    if (e->peers_open && e->peers_ipc)
        for (int p = 0; p < e->world; p++)
            if (p != e->rank && e->peer_base[p]) c->drv->cuIpcCloseMemHandle(e->peer_base[p]);
    if (e->arena) c->drv->cuMemFree_v2(e->arena);
    if (e->local) c->drv->cuMemFree_v2(e->local);
    e->magic = 0;
    delete e;
    return QM_OK;
}

extern "C" int32_t qm_ep_create(qm_ctx *c, const qm_weight *gate_up, const qm_weight *down, int32_t experts_local,
                                int32_t experts_total, int32_t topk, int32_t max_tokens, int32_t rank, int32_t world,
                                qm_ep **out) {
    CHECK_CTX(c);
    if (!out) return QM_ERR_ARG;
    *out = nullptr;
    if (world < 1 || world > QM_MAX_PEERS || rank < 0 || rank >= world || experts_local < 1 || experts_local > 64 ||
        experts_total != experts_local * world || experts_total > QM_MAX_EXPERTS || topk < 1 || topk > experts_total ||
        max_tokens < 1 || (int64_t)max_tokens * topk >= (1 << 20))
        return QM_ERR_SHAPE;
    qm_ep *e = new (std::nothrow) qm_ep();
    if (!e) return QM_ERR_NOMEM;
    int32_t rc = check_experts(gate_up, down, experts_local, e->wg, e->wd, &e->hidden, &e->ffn);
    if (!rc && (e->ffn & 127)) rc = QM_ERR_SHAPE;   // the SwiGLU epilogue of the grouped matmul: whole 128-row tiles
    if (rc) {
        delete e;
        return rc;
    }
    e->magic = QM_EP_MAGIC;
    e->eloc = experts_local;
    e->experts = experts_total;
    e->topk = topk;
    e->max_tokens = max_tokens;
    e->cap = max_tokens * topk;
    e->rank = rank;
    e->world = world;
    e->epoch = 0;
    e->phase = 0;
    e->peers_open = world == 1;
    e->peers_ipc = false;
    memset(e->peer_base, 0, sizeof e->peer_base);
    const int64_t cap = e->cap, H = e->hidden, W = world;
    e->o_flags = 0;
    e->o_counts = 256;
    e->o_rows = up256(e->o_counts + W * experts_local * 4);
    e->o_ret = up256(e->o_rows + W * cap * H * 2);
    e->arena_bytes = up256(e->o_ret + W * cap * H * 4);
    int64_t o = 0;
    auto take = [&](int64_t bytes) { const int64_t at = o; o = up256(o + bytes); return at; };
    e->o_rankbuf = take(cap * 4);
    e->o_lcounts = take(QM_MAX_EXPERTS * 4);
    e->o_offsets = take((QM_MAX_EXPERTS + 1) * 4);
    e->o_list = take(cap * 4);
    e->o_pos = take(cap * 4);
    e->o_compact = take(W * cap * H * 2);
    e->o_back = take(W * cap * 4);
    e->o_loff = take(65 * 4);
    e->o_y = take(W * cap * H * 4);
    e->o_done = take(256);
    CtxGuard g(c);
    CUresult r = g.rc;
    if (r == CUDA_SUCCESS) r = c->drv->cuMemAlloc_v2(&e->arena, (size_t)e->arena_bytes);
    if (r == CUDA_SUCCESS) r = c->drv->cuMemsetD8Async(e->arena, 0, (size_t)e->o_rows, c->stream);   // flags and counts
    if (r == CUDA_SUCCESS) r = c->drv->cuMemAlloc_v2(&e->local, (size_t)o);
    if (r == CUDA_SUCCESS) r = c->drv->cuStreamSynchronize(c->stream);
    if (r != CUDA_SUCCESS) {
        if (e->arena) c->drv->cuMemFree_v2(e->arena);
        if (e->local) c->drv->cuMemFree_v2(e->local);
        delete e;
        return (int32_t)r;
    }
    e->peer_base[rank] = e->arena;
    *out = e;
    return QM_OK;
}

extern "C" int32_t qm_ep_arena(qm_ctx *c, qm_ep *e, uint64_t *base, int64_t *bytes) {
    CHECK_CTX(c);
    if (!ep_check(e) || !base || !bytes) return QM_ERR_ARG;
    *base = (uint64_t)e->arena;
    *bytes = e->arena_bytes;
    return QM_OK;
}

extern "C" int32_t qm_ep_ipc_handle(qm_ctx *c, qm_ep *e, void *handle64) {
    CHECK_CTX(c);
    if (!ep_check(e) || !handle64) return QM_ERR_ARG;
    CtxGuard g(c);
    DRV(g.rc);
    CUipcMemHandle h;
    DRV(c->drv->cuIpcGetMemHandle(&h, e->arena));
    memcpy(handle64, &h, 64);
    return QM_OK;
}

extern "C" int32_t qm_ep_set_peers(qm_ctx *c, qm_ep *e, const void *handles) {
    CHECK_CTX(c);
    if (!ep_check(e) || !handles || e->world < 2 || e->peers_open) return QM_ERR_ARG;
    CtxGuard g(c);
    DRV(g.rc);
    for (int p = 0; p < e->world; p++) {
        if (p == e->rank) continue;
        CUipcMemHandle h;
        memcpy(&h, (const char *)handles + (size_t)p * 64, 64);
        CUresult r = c->drv->cuIpcOpenMemHandle_v2(&e->peer_base[p], h, CU_IPC_MEM_LAZY_ENABLE_PEER_ACCESS);
        if (r != CUDA_SUCCESS) {
            for (int q = 0; q < p; q++)
                if (q != e->rank && e->peer_base[q]) {
                    c->drv->cuIpcCloseMemHandle(e->peer_base[q]);
                    e->peer_base[q] = 0;
                }
            return (int32_t)r;
        }
    }
    e->peers_open = true;
    e->peers_ipc = true;
    return QM_OK;
}

extern "C" int32_t qm_ep_set_peer_pointers(qm_ctx *c, qm_ep *e, const uint64_t *bases) {
    CHECK_CTX(c);
    if (!ep_check(e) || !bases || e->world < 2 || e->peers_open) return QM_ERR_ARG;
    for (int p = 0; p < e->world; p++) {
        if (p != e->rank && !bases[p]) return QM_ERR_ARG;
        if (p != e->rank) e->peer_base[p] = (CUdeviceptr)bases[p];
    }
    e->peers_open = true;
    e->peers_ipc = false;
    return QM_OK;
}

static unsigned ep_grid(qm_ctx *c, int64_t rows) {
    return (unsigned)std::max<int64_t>(1, std::min<int64_t>((rows + 7) / 8, (int64_t)c->sm_count * 4));
}

// begin: lists of this rank's pairs by global expert, rows pushed to their owners.
extern "C" int32_t qm_ep_begin(qm_ctx *c, qm_ep *e, uint64_t x_bf16_dev, int32_t tokens, int64_t ldx, uint64_t ids_dev,
                               uint64_t weights_dev, uint64_t out_dev, int64_t ldo) {
    CHECK_CTX(c);
    if (!ep_check(e)) return QM_ERR_ARG;
    if (!e->peers_open || e->phase != 0) return QM_ERR_STATE;
    if (tokens < 0 || tokens > e->max_tokens || ldx < e->hidden || ldo < e->hidden || ((ldx * 2) & 15)) return QM_ERR_SHAPE;
    if (tokens > 0 && (!x_bf16_dev || !ids_dev || !weights_dev || !out_dev || (x_bf16_dev & 15) || (ids_dev & 3)))
        return QM_ERR_ARG;
    CtxGuard g(c);
    DRV(g.rc);
    e->epoch += 1;
    QmEpArgs &a = e->step;
    memset(&a, 0, sizeof a);
    const CUdeviceptr L = e->local, A = e->arena;
    a.x = (const uint16_t *)(uintptr_t)x_bf16_dev;
    a.ids = (const int32_t *)(uintptr_t)ids_dev;
    a.list = (const int32_t *)(uintptr_t)(L + e->o_list);
    a.offsets = (const int32_t *)(uintptr_t)(L + e->o_offsets);
    a.pos = (const int32_t *)(uintptr_t)(L + e->o_pos);
    a.weights = (const float *)(uintptr_t)weights_dev;
    a.out = (float *)(uintptr_t)out_dev;
    a.ldx = ldx;
    a.ldo = ldo;
    a.compact = (uint16_t *)(uintptr_t)(L + e->o_compact);
    a.back = (int32_t *)(uintptr_t)(L + e->o_back);
    a.loff = (int32_t *)(uintptr_t)(L + e->o_loff);
    a.y = (const float *)(uintptr_t)(L + e->o_y);
    a.done = (unsigned int *)(uintptr_t)(L + e->o_done);
    a.status = (unsigned int *)(uintptr_t)c->status_dev;
    a.flags = (unsigned int *)(uintptr_t)(A + e->o_flags);
    a.counts_in = (int32_t *)(uintptr_t)(A + e->o_counts);
    a.rows_in = (uint16_t *)(uintptr_t)(A + e->o_rows);
    a.ret_in = (float *)(uintptr_t)(A + e->o_ret);
    for (int p = 0; p < e->world; p++) a.peer_delta[p] = (int64_t)e->peer_base[p] - (int64_t)A;
    a.tokens = tokens;
    a.topk = e->topk;
    a.hidden = (int32_t)e->hidden;
    a.experts = e->experts;
    a.eloc = e->eloc;
    a.world = e->world;
    a.rank = e->rank;
    a.cap = e->cap;
    a.epoch = e->epoch;
    a.wait_cycles = qm_wait_cycles();
    DRV(c->drv->cuMemsetD32Async(L + e->o_done, 0, 2, c->stream));
    QmListArgs la;
    memset(&la, 0, sizeof la);
    la.ids = a.ids;
    la.rank = (int32_t *)(uintptr_t)(L + e->o_rankbuf);
    la.counts = (int32_t *)(uintptr_t)(L + e->o_lcounts);
    la.offsets = (int32_t *)(uintptr_t)(L + e->o_offsets);
    la.list = (int32_t *)(uintptr_t)(L + e->o_list);
    la.pos = (int32_t *)(uintptr_t)(L + e->o_pos);
    la.tokens = tokens;
    la.experts = e->experts;
    la.topk = e->topk;
    int32_t rc = qm_launch(c, QM_K_MOE_LISTS, 1, 1, 1024, 0, &la, false);
    if (!rc) rc = qm_launch(c, QM_K_EP_PUSH, ep_grid(c, (int64_t)tokens * e->topk), 1, 256, 0, &a, false);
    if (!rc) e->phase = 1;
    return rc;
}

// run: what the other ranks pushed is regrouped by local expert, multiplied, and sent back.
extern "C" int32_t qm_ep_run(qm_ctx *c, qm_ep *e) {
    CHECK_CTX(c);
    if (!ep_check(e)) return QM_ERR_ARG;
    if (e->phase != 1) return QM_ERR_STATE;
    CtxGuard g(c);
    DRV(g.rc);
    QmEpArgs &a = e->step;
    const int64_t bound = (int64_t)e->world * e->cap;   // rows this rank can receive
    int32_t rc = qm_launch(c, QM_K_EP_COLLECT, ep_grid(c, bound), 1, 256, 0, &a, false);
    if (rc) return rc;
    // As in qm_moe_grouped, the list lengths are read back once so that the grouped launches have exactly the
    // token tiles that hold rows; QM_MOE_NOSYNC=1 sizes them for the longest possible list instead (no
    // synchronization; the empty CTAs cost more than the read-back on the shapes measured).
    int32_t longest = (int32_t)bound, typical = (int32_t)std::max<int64_t>(1, bound / e->experts);
    if (!qm_env_int("QM_MOE_NOSYNC", 0)) {
        int32_t loff[65];
        DRV(c->drv->cuMemcpyDtoHAsync_v2(loff, e->local + e->o_loff, (size_t)(e->eloc + 1) * 4, c->stream));
        DRV(c->drv->cuStreamSynchronize(c->stream));
        longest = 0;
        for (int k = 0; k < e->eloc; k++) longest = std::max(longest, loff[k + 1] - loff[k]);
        if (longest < 0 || longest > bound) return QM_ERR_STATE;
        typical = longest;
    }
    if (longest > 0) {
        rc = experts_launch(c, e->wg, e->wd, e->eloc, e->local + e->o_compact, bound, longest, typical,
                            e->local + e->o_loff, e->local + e->o_y, e->hidden, e->ffn);
        if (rc) return rc;
    }
    rc = qm_launch(c, QM_K_EP_RETURN, ep_grid(c, bound), 1, 256, 0, &a, false);
    if (!rc) e->phase = 2;
    return rc;
}

// end: the results that came back are combined with the routing weights.
extern "C" int32_t qm_ep_end(qm_ctx *c, qm_ep *e) {
    CHECK_CTX(c);
    if (!ep_check(e)) return QM_ERR_ARG;
    if (e->phase != 2) return QM_ERR_STATE;
    CtxGuard g(c);
    DRV(g.rc);
    e->phase = 0;
    return qm_launch(c, QM_K_EP_COMBINE, grid_for((int64_t)std::max(1, e->step.tokens) * e->hidden, 256, c->sm_count * 8),
                     1, 256, 0, &e->step, false);
}

extern "C" int32_t qm_ep_moe(qm_ctx *c, qm_ep *e, uint64_t x_bf16_dev, int32_t tokens, int64_t ldx, uint64_t ids_dev,
                             uint64_t weights_dev, uint64_t out_dev, int64_t ldo) {
    int32_t rc = qm_ep_begin(c, e, x_bf16_dev, tokens, ldx, ids_dev, weights_dev, out_dev, ldo);
    if (!rc) rc = qm_ep_run(c, e);
    if (!rc) rc = qm_ep_end(c, e);
    return rc;
}
