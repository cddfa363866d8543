// qm_q8_1.cpp — host side of the Q8_1 activation ABI (include/qmatmul.h): the producers
// RMSNorm -> Q8_1 and SwiGLU -> Q8_1, matvecs that take Q8_1 activations, and the matvec over
// selected experts. The reference's counterparts are cudaquant.RMSNormQ8_1 with its kernel
// (nvidia/x/cudaquant/quant.go:46-156) and the *_q8_1 kernels of nvidia/x/egraph/codegen.go.
#include <math.h>
#include <string.h>

#include <algorithm>

#include "qm_internal.h"

static int32_t norm_launch(qm_ctx *c, uint64_t x_dev, int64_t ldx, uint64_t weight_dev, int64_t rows, int64_t cols,
                           float eps, uint64_t out_dev) {
    QmNormQ81Args a;
    memset(&a, 0, sizeof a);
    a.x = (const float *)(uintptr_t)x_dev;
    a.weight = (const float *)(uintptr_t)weight_dev;
    a.out = (uint8_t *)(uintptr_t)out_dev;
    a.status = (unsigned int *)(uintptr_t)c->status_dev;
    a.ldx = ldx;
    a.cols = (int32_t)cols;
    a.eps = eps;
    return qm_launch(c, QM_K_RMSNORM_Q81, (unsigned)rows, 1, 1024, 0, &a, false);
}

// The argument checks of cudaquant.RMSNormQ8_1 (quant.go:47-49) that need no data.
static bool norm_dims_ok(int64_t rows, int64_t cols, float eps) {
    return rows > 0 && cols > 0 && rows <= INT64_MAX / cols && cols % 32 == 0 && !(eps < 0) && !isnan(eps) && !isinf(eps);
}

extern "C" int32_t qm_rmsnorm_q8_1(qm_ctx *c, uint64_t x_dev, int64_t ldx, uint64_t weight_dev, int64_t rows,
                                   int64_t cols, float eps, uint64_t out_dev) {
    CHECK_CTX(c);
    if (!norm_dims_ok(rows, cols, eps) || rows > (1 << 30) || cols > (1 << 24) || ldx < cols) return QM_ERR_SHAPE;
    if (!x_dev || !out_dev || (out_dev & 3) || (x_dev & 3) || (weight_dev & 3)) return QM_ERR_ARG;
    CtxGuard g(c);
    DRV(g.rc);
    return norm_launch(c, x_dev, ldx, weight_dev, rows, cols, eps, out_dev);
}

// Grows the context's scratch to `bytes` (outside any steady-state loop: sizes repeat).
static int32_t q81_scratch(qm_ctx *c, int64_t bytes) {
    if (bytes <= c->q81_ws_bytes) return QM_OK;
    DRV(c->drv->cuStreamSynchronize(c->stream));
    if (c->q81_ws) DRV(c->drv->cuMemFree_v2(c->q81_ws));
    c->q81_ws = 0;
    c->q81_ws_bytes = 0;
    DRV(c->drv->cuMemAlloc_v2(&c->q81_ws, (size_t)bytes));
    c->q81_ws_bytes = bytes;
    return QM_OK;
}

extern "C" int32_t qm_rmsnorm_q8_1_host(qm_ctx *c, const float *input, int64_t n_input, const float *weight,
                                        int64_t n_weight, int64_t rows, int64_t cols, float eps, int32_t weighted,
                                        void *out_blocks) {
    CHECK_CTX(c);
    // the order of cudaquant.RMSNormQ8_1's refusals (quant.go:47-55)
    if (!norm_dims_ok(rows, cols, eps)) return QM_ERR_SHAPE;
    if (n_input != rows * cols) return QM_ERR_BUFFER;
    if (weighted && n_weight != cols) return QM_ERR_BUFFER;
    if (!input || !out_blocks || (weighted && !weight)) return QM_ERR_ARG;
    if (rows > (1 << 30) || cols > (1 << 24)) return QM_ERR_SHAPE;
    CtxGuard g(c);
    DRV(g.rc);
    const int64_t xb = rows * cols * 4, wb = weighted ? cols * 4 : 0, ob = rows * cols / 32 * 36;
    const int64_t xo = 0, wo = (xb + 255) & ~(int64_t)255, oo = (wo + wb + 255) & ~(int64_t)255;
    int32_t rc = q81_scratch(c, oo + ob);
    if (rc) return rc;
    // nonfinite inputs or weights, a zero denominator and nonfinite normalised values are found by the
    // kernel and come back through the status word (quant.go:56-68,76-78,88-90)
    DRV(c->drv->cuMemsetD8Async(c->status_dev, 0, 4, c->stream));
    DRV(c->drv->cuMemcpyHtoDAsync_v2(c->q81_ws + xo, input, (size_t)xb, c->stream));
    if (weighted) DRV(c->drv->cuMemcpyHtoDAsync_v2(c->q81_ws + wo, weight, (size_t)wb, c->stream));
    rc = norm_launch(c, c->q81_ws + xo, cols, weighted ? c->q81_ws + wo : 0, rows, cols, eps, c->q81_ws + oo);
    if (rc) return rc;
    uint32_t status = 0;
    DRV(c->drv->cuMemcpyDtoHAsync_v2(&status, c->status_dev, 4, c->stream));
    DRV(c->drv->cuStreamSynchronize(c->stream));
    if (status & QM_STATUS_DOMAIN) {
        DRV(c->drv->cuMemsetD8Async(c->status_dev, 0, 4, c->stream));
        return QM_ERR_DOMAIN;   // like the reference, no blocks are handed out
    }
    DRV(c->drv->cuMemcpyDtoHAsync_v2(out_blocks, c->q81_ws + oo, (size_t)ob, c->stream));
    DRV(c->drv->cuStreamSynchronize(c->stream));
    return QM_OK;
}

extern "C" int32_t qm_swiglu_q8_1(qm_ctx *c, uint64_t gate_dev, uint64_t up_dev, uint64_t weights_dev, int32_t width,
                                  int32_t slots, uint64_t out_dev) {
    CHECK_CTX(c);
    if (width <= 0 || slots <= 0 || (int64_t)width * slots > (1ll << 31) - 64) return QM_ERR_SHAPE;
    if (!gate_dev || !up_dev || !weights_dev || !out_dev || (out_dev & 3) || ((gate_dev | up_dev | weights_dev) & 3))
        return QM_ERR_ARG;
    CtxGuard g(c);
    DRV(g.rc);
    QmSwigluQ81Args a;
    memset(&a, 0, sizeof a);
    a.gate = (const float *)(uintptr_t)gate_dev;
    a.up = (const float *)(uintptr_t)up_dev;
    a.weights = (const float *)(uintptr_t)weights_dev;
    a.out = (uint8_t *)(uintptr_t)out_dev;
    a.width = width;
    a.slots = slots;
    const int64_t blocks = ((int64_t)width * slots + 31) / 32;
    const unsigned grid = (unsigned)std::max<int64_t>(1, std::min<int64_t>((blocks + 7) / 8, (int64_t)c->sm_count * 8));
    return qm_launch(c, QM_K_SWIGLU_Q81, grid, 1, 256, 0, &a, false);
}

static int32_t expand_launch(qm_ctx *c, uint64_t xq_dev, int32_t m, int64_t ldx_blocks, int64_t cols, uint64_t out_dev,
                             int64_t ld_out, bool pdl) {
    QmQ81ExpandArgs a;
    memset(&a, 0, sizeof a);
    a.xq = (const uint8_t *)(uintptr_t)xq_dev;
    a.out = (float *)(uintptr_t)out_dev;
    a.ldx = ldx_blocks;
    a.ld_out = ld_out;
    a.cols = (int32_t)cols;
    a.m = m;
    const int64_t work = (int64_t)m * cols / 4;
    const unsigned grid = (unsigned)std::max<int64_t>(1, std::min<int64_t>((work + 255) / 256, (int64_t)c->sm_count * 4));
    return qm_launch(c, QM_K_Q81_EXPAND, grid, 1, 256, 0, &a, pdl);
}

extern "C" int32_t qm_q8_1_dequantize(qm_ctx *c, uint64_t xq_dev, int32_t m, int64_t ldx_blocks, int64_t cols,
                                      uint64_t out_dev, int64_t ld_out) {
    CHECK_CTX(c);
    if (m < 1 || cols <= 0 || cols % 32 != 0 || cols > (1 << 24) || ldx_blocks < cols / 32 || ld_out < cols || (ld_out & 3))
        return QM_ERR_SHAPE;
    if (!xq_dev || !out_dev || (xq_dev & 3) || (out_dev & 15)) return QM_ERR_ARG;
    CtxGuard g(c);
    DRV(g.rc);
    return expand_launch(c, xq_dev, m, ldx_blocks, cols, out_dev, ld_out, false);
}

extern "C" int32_t qm_matvec_q8_1(qm_ctx *c, qm_weight h, uint64_t xq_dev, int32_t m, int64_t ldx_blocks, uint64_t y_dev,
                                  int64_t ldy, uint32_t flags) {
    CHECK_CTX(c);
    QmWeight *w = qm_weight_from_handle(h);
    if (!w) return QM_ERR_ARG;
    if (m < 1 || m > 8 || w->cols % 32 != 0 || ldx_blocks < w->cols / 32 || ldx_blocks > (1 << 22) || ldy < w->rows)
        return QM_ERR_SHAPE;
    if (!xq_dev || !y_dev || (xq_dev & 3) || (flags & 0xFu) != QM_XOP_NONE) return QM_ERR_ARG;
    CtxGuard g(c);
    DRV(g.rc);
    const bool pdl = (flags & QM_FLAG_PDL) != 0;
    if (w->fmt == QM_FMT_Q2_K || w->fmt == QM_FMT_IQ2_XXS)   // the blocks are read where they are multiplied
        return qm_kq_launch(c, w, xq_dev, true, m, ldx_blocks, y_dev, ldy, 0, 0, 1, 0, pdl);
    // Q4_0 / Q8_0 / Q4_K stage and quantize their activations themselves: they get the exact float32 values
    const int64_t cols4 = (w->cols + 3) & ~(int64_t)3;
    int32_t rc = q81_scratch(c, (int64_t)m * cols4 * 4);
    if (rc) return rc;
    rc = expand_launch(c, xq_dev, m, ldx_blocks, w->cols, c->q81_ws, cols4, pdl);
    if (rc) return rc;
    return qm_matvec_launch(c, w, c->q81_ws, 0, m, cols4, y_dev, ldy, flags, c->partials_dev, c->tickets_dev);
}

extern "C" int32_t qm_matvec_selected(qm_ctx *c, qm_weight h, int32_t experts, uint64_t ids_dev, int32_t slots,
                                      uint64_t x_dev, int64_t x_slot_stride, uint64_t y_dev, uint32_t flags) {
    CHECK_CTX(c);
    QmWeight *w = qm_weight_from_handle(h);
    if (!w) return QM_ERR_ARG;
    if (w->fmt != QM_FMT_Q2_K && w->fmt != QM_FMT_IQ2_XXS) return QM_ERR_FORMAT;
    if (experts < 1 || w->rows % experts != 0 || slots < 1 || slots > 65535 || x_slot_stride < 0) return QM_ERR_SHAPE;
    const bool xq = (flags & QM_FLAG_X_Q8_1) != 0;
    if (x_slot_stride != 0 && x_slot_stride < (xq ? w->cols / 32 : w->cols)) return QM_ERR_SHAPE;
    if (x_slot_stride > (1ll << 40)) return QM_ERR_SHAPE;
    if (!ids_dev || !x_dev || !y_dev || (ids_dev & 3) || (x_dev & (xq ? 3 : 15)) || (!xq && (x_slot_stride & 3)))
        return QM_ERR_ARG;
    if ((flags & 0xFu) != QM_XOP_NONE) return QM_ERR_ARG;
    CtxGuard g(c);
    DRV(g.rc);
    const int64_t rows_e = w->rows / experts;
    return qm_kq_launch(c, w, x_dev, xq, 1, xq ? w->cols / 32 : w->cols, y_dev, rows_e, ids_dev, experts, slots,
                        x_slot_stride, (flags & QM_FLAG_PDL) != 0);
}
