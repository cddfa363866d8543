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
    if (tokens < 0 || experts < 1 || experts > 64 || topk < 0 || topk > experts || ld < experts) return QM_ERR_SHAPE;
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

static int32_t ensure_ws(qm_ctx *c, int64_t bytes) {
    if (bytes <= c->moe_ws_bytes) return QM_OK;
    DRV(c->drv->cuStreamSynchronize(c->stream));
    if (c->moe_ws) DRV(c->drv->cuMemFree_v2(c->moe_ws));
    c->moe_ws = 0;
    c->moe_ws_bytes = 0;
    DRV(c->drv->cuMemAlloc_v2(&c->moe_ws, (size_t)bytes));
    c->moe_ws_bytes = bytes;
    return QM_OK;
}

// out[t][:] = sum_s weights[t][s] * down_e( silu(gate_e x_t) * (up_e x_t) ), e = ids[t][s].
// gate_up[e]: stored Q4_K [2*ffn][hidden] (gate rows then up rows); down[e]: [hidden][ffn].
extern "C" int32_t qm_moe_grouped(qm_ctx *c, const qm_weight *gate_up, const qm_weight *down, int32_t experts,
                                  uint64_t x_bf16_dev, int32_t tokens, int64_t ldx, uint64_t ids_dev,
                                  uint64_t weights_dev, int32_t topk, uint64_t out_dev, int64_t ldo) {
    CHECK_CTX(c);
    if (!gate_up || !down || !x_bf16_dev || !ids_dev || !weights_dev || !out_dev) return QM_ERR_ARG;
    if (experts < 1 || experts > 64 || tokens < 1 || topk < 1 || topk > experts) return QM_ERR_SHAPE;
    std::vector<QmWeight *> wg(experts), wd(experts);
    for (int e = 0; e < experts; e++) {
        wg[e] = qm_weight_from_handle(gate_up[e]);
        wd[e] = qm_weight_from_handle(down[e]);
        if (!wg[e] || !wd[e]) return QM_ERR_ARG;
        if (wg[e]->fmt != QM_FMT_Q4_K || wd[e]->fmt != QM_FMT_Q4_K) return QM_ERR_FORMAT;
    }
    const int64_t hidden = wg[0]->cols, ffn = wd[0]->cols;
    for (int e = 0; e < experts; e++)
        if (wg[e]->cols != hidden || wg[e]->rows != 2 * ffn || wd[e]->rows != hidden || wd[e]->cols != ffn) return QM_ERR_SHAPE;
    if (ldx < hidden || ldo < hidden || (hidden & 7) || (ffn & 7) || (x_bf16_dev & 15) || ((ldx * 2) & 15)) return QM_ERR_SHAPE;
    CtxGuard g(c);
    DRV(g.rc);
    const int64_t pairs = (int64_t)tokens * topk;
    // workspace: int arrays, then gathered bf16, gate|up fp32, h bf16, expert outputs fp32
    auto up256 = [](int64_t v) { return (v + 255) & ~(int64_t)255; };
    const int64_t o_rank = 0, o_counts = up256(pairs * 4), o_offsets = o_counts + 256, o_list = o_offsets + 512,
                  o_pos = o_list + up256(pairs * 4), o_gath = o_pos + up256(pairs * 4),
                  o_gu = o_gath + up256(pairs * hidden * 2), o_h = o_gu + up256(pairs * 2 * ffn * 4),
                  o_y = o_h + up256(pairs * ffn * 2), total = o_y + up256(pairs * hidden * 4);
    int32_t rc = ensure_ws(c, total);
    if (rc) return rc;
    const CUdeviceptr ws = c->moe_ws;
    {
        QmListArgs a;
        memset(&a, 0, sizeof a);
        a.ids = (const int32_t *)(uintptr_t)ids_dev;
        a.rank = (int32_t *)(uintptr_t)(ws + o_rank);
        a.counts = (int32_t *)(uintptr_t)(ws + o_counts);
        a.offsets = (int32_t *)(uintptr_t)(ws + o_offsets);
        a.list = (int32_t *)(uintptr_t)(ws + o_list);
        a.pos = (int32_t *)(uintptr_t)(ws + o_pos);
        a.tokens = tokens;
        a.experts = experts;
        a.topk = topk;
        rc = qm_launch(c, QM_K_MOE_LISTS, 1, 1, 1024, 0, &a, false);
        if (rc) return rc;
    }
    // the per-expert launches need the list lengths on the host
    int32_t offsets[65];
    DRV(c->drv->cuMemcpyDtoHAsync_v2(offsets, ws + o_offsets, (size_t)(experts + 1) * 4, c->stream));
    DRV(c->drv->cuStreamSynchronize(c->stream));
    const int rows = offsets[experts];
    if (rows < 0 || rows > pairs) return QM_ERR_STATE;
    {
        QmGatherArgs a;
        memset(&a, 0, sizeof a);
        a.x = (const uint16_t *)(uintptr_t)x_bf16_dev;
        a.list = (const int32_t *)(uintptr_t)(ws + o_list);
        a.out = (uint16_t *)(uintptr_t)(ws + o_gath);
        a.ldx = ldx;
        a.rows = rows;
        a.hidden = (int32_t)hidden;
        a.topk = topk;
        rc = qm_launch(c, QM_K_MOE_GATHER, grid_for((int64_t)rows * hidden / 8, 256, c->sm_count * 8), 1, 256, 0, &a, false);
        if (rc) return rc;
    }
    for (int e = 0; e < experts; e++) {
        const int n_e = offsets[e + 1] - offsets[e];
        if (n_e <= 0) continue;
        rc = qm_matmul_bf16(c, gate_up[e], ws + o_gath + (int64_t)offsets[e] * hidden * 2, n_e, hidden,
                            ws + o_gu + (int64_t)offsets[e] * 2 * ffn * 4, 2 * ffn);
        if (rc) return rc;
    }
    {
        QmSwigluArgs a;
        a.gu = (const float *)(uintptr_t)(ws + o_gu);
        a.h = (uint16_t *)(uintptr_t)(ws + o_h);
        a.rows = rows;
        a.ffn = (int32_t)ffn;
        rc = qm_launch(c, QM_K_MOE_SWIGLU, grid_for((int64_t)rows * ffn / 2, 256, c->sm_count * 8), 1, 256, 0, &a, false);
        if (rc) return rc;
    }
    for (int e = 0; e < experts; e++) {
        const int n_e = offsets[e + 1] - offsets[e];
        if (n_e <= 0) continue;
        rc = qm_matmul_bf16(c, down[e], ws + o_h + (int64_t)offsets[e] * ffn * 2, n_e, ffn,
                            ws + o_y + (int64_t)offsets[e] * hidden * 4, hidden);
        if (rc) return rc;
    }
    {
        QmCombineArgs a;
        memset(&a, 0, sizeof a);
        a.y = (const float *)(uintptr_t)(ws + o_y);
        a.pos = (const int32_t *)(uintptr_t)(ws + o_pos);
        a.weights = (const float *)(uintptr_t)weights_dev;
        a.out = (float *)(uintptr_t)out_dev;
        a.ldo = ldo;
        a.tokens = tokens;
        a.hidden = (int32_t)hidden;
        a.topk = topk;
        rc = qm_launch(c, QM_K_MOE_COMBINE, grid_for((int64_t)tokens * hidden, 256, c->sm_count * 8), 1, 256, 0, &a, false);
    }
    return rc;
}
