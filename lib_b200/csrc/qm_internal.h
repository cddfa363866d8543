// Internal types of libqmatmul.so shared between its translation units.
#pragma once
#include <stdint.h>

#include "../../include/qmatmul.h"
#include "qm_driver.h"
#include "qm_kernel_args.h"

#define QM_CTX_MAGIC 0x514D4358u     // "QMCX"
#define QM_WEIGHT_MAGIC 0x514D5754u  // "QMWT"

enum { QM_MOD_GEMV = 0, QM_MOD_DEQUANT, QM_MOD_Q4K, QM_MOD_GEMM, QM_MOD_MOE, QM_MOD_KQ, QM_MOD_Q81, QM_MOD_COUNT };
enum {
    QM_K_GEMV_Q40_M4 = 0, QM_K_GEMV_Q40_M8, QM_K_GEMV_Q80_M4,
    QM_K_GEMV_Q80_M8, QM_K_DEQUANT_Q4K, QM_K_DEQUANT_Q2K, QM_K_DEQUANT_Q40, QM_K_DEQUANT_Q80,
    QM_K_REPACK_Q40, QM_K_REPACK_Q80, QM_K_REPACK_Q4K, QM_K_FUSED_Q4K_NT1, QM_K_FUSED_Q4K_NT2, QM_K_FUSED_Q4K_NT1_IMG, QM_K_FUSED_Q4K_NT2_IMG, QM_K_FUSED_Q4K_NT1_TP, QM_K_FUSED_Q4K_NT2_TP, QM_K_FUSED_Q4K_DD_C4D2, QM_K_FUSED_Q4K_DD_C4D3, QM_K_FUSED_Q4K_DD_C4D4,
    QM_K_FUSED_Q4K_DD_C2D2, QM_K_FUSED_Q4K_DD_C2D3, QM_K_FUSED_Q4K_DD_C2D4,
    QM_K_FUSED_Q4K_DD_C4D2_TP, QM_K_FUSED_Q4K_DD_C4D3_TP, QM_K_FUSED_Q4K_DD_C4D4_TP,
    QM_K_FUSED_Q4K_DD_C2D2_TP, QM_K_FUSED_Q4K_DD_C2D3_TP, QM_K_FUSED_Q4K_DD_C2D4_TP,
    QM_K_SUM_PARTS, QM_K_REPACK_PARTS,
    QM_K_GEMM_Q4K, QM_K_GEMM_Q4K_R256, QM_K_GEMM_Q4K_K128, QM_K_GEMM_Q4K_R256_K128, QM_K_MOE_ROUTE, QM_K_MOE_LISTS, QM_K_MOE_GATHER, QM_K_MOE_COMBINE,
    QM_K_DEQUANT_IQ2XXS, QM_K_GEMV_Q2K_M1, QM_K_GEMV_Q2K_M2, QM_K_GEMV_Q2K_M4, QM_K_GEMV_Q2K_M8,
    QM_K_GEMV_IQ2XXS_M1, QM_K_GEMV_IQ2XXS_M2, QM_K_GEMV_IQ2XXS_M4, QM_K_GEMV_IQ2XXS_M8,
    QM_K_GEMV_Q2K_Q81_M1, QM_K_GEMV_Q2K_Q81_M2, QM_K_GEMV_Q2K_Q81_M4, QM_K_GEMV_Q2K_Q81_M8,
    QM_K_GEMV_IQ2XXS_Q81_M1, QM_K_GEMV_IQ2XXS_Q81_M2, QM_K_GEMV_IQ2XXS_Q81_M4, QM_K_GEMV_IQ2XXS_Q81_M8,
    QM_K_RMSNORM_Q81, QM_K_SWIGLU_Q81, QM_K_Q81_EXPAND,
    QM_K_FUSED_Q4K_DD_C4D2_SEL, QM_K_FUSED_Q4K_DD_C4D3_SEL, QM_K_FUSED_Q4K_DD_C4D4_SEL, QM_K_MOE_DECODE_COMBINE,
    QM_K_EP_PUSH, QM_K_EP_COLLECT, QM_K_EP_RETURN, QM_K_EP_COMBINE,
    QM_K_Q40_LEAN_C4D4, QM_K_Q40_LEAN_C4D2, QM_K_Q40_LEAN_C2D4, QM_K_Q40_LEAN_C2D2, QM_K_Q40_LEAN_C2N2D4, QM_K_Q40_LEAN_C2N2D2,
    QM_K_Q80_LEAN_C4D3, QM_K_Q80_LEAN_C4D2, QM_K_Q80_LEAN_C2D3, QM_K_Q80_LEAN_C2D2, QM_K_Q80_LEAN_C2N2D3, QM_K_Q80_LEAN_C2N2D2,
    QM_K_LEAN_SUM, QM_K_FUSED_Q4K_DD_N2D2, QM_K_FUSED_Q4K_DD_N2D3, QM_K_COUNT
};

#define QM_GEMV_SMEM_MAX (227 * 1024)
#define QM_KQ_SMEM_MAX (96 * 1024)   // ring bytes per CTA of the Q2_K / IQ2_XXS GEMV
#define QM_TICKETS 65536
#define QM_PARTIALS_BYTES (64ll << 20)
#define QM_UPLOAD_CHUNK (64ll << 20)

struct qm_ctx {
    uint32_t magic;
    QmDriver *drv;
    int device;
    CUdevice cudev;
    CUcontext cuctx;
    bool have_ctx;
    int sm_count, l2_bytes;
    CUmodule modules[QM_MOD_COUNT];
    CUfunction fn[QM_K_COUNT];
    CUstream own_stream, stream;
    CUdeviceptr status_dev, tickets_dev, partials_dev, gridbar_dev;
    CUdeviceptr xstage_dev;
    int64_t xstage_bytes;
    CUdeviceptr upload_dev;
    CUdeviceptr moe_ws, moe_ws2, moe_ws3;   // scratch of the MoE stages (grown on demand)
    int64_t moe_ws_bytes, moe_ws2_bytes, moe_ws3_bytes;
    CUdeviceptr q81_ws;                     // float32 copy of Q8_1 activations for the matvecs that quantize on their own
    int64_t q81_ws_bytes;
    int64_t launches;
};

struct QmWeight {
    uint32_t magic;
    int32_t fmt;
    int32_t device;   // ordinal of the GPU that holds the bytes
    int64_t rows, cols;
    int32_t units;
    int64_t gguf_row_bytes;
    int64_t qbytes, dbytes;
    CUdeviceptr wq, wd;
};

struct QmGemvPlan {
    int consumers, depth, kc, ksplit, units_per_slice, ctas_per_slice, tiles, maxseg, smem;
};

struct QmFusedPlan {
    int consumers, depth, max_units, cpm, nt, smem;
    int slices, units_per_slice;   // K slices of one matvec when its activations do not fit whole
};

struct CtxGuard {
    qm_ctx *ctx;
    CUresult rc;
    explicit CtxGuard(qm_ctx *c);
    ~CtxGuard();
};

#define DRV(expr)                                       \
    do {                                                \
        CUresult _r = (expr);                           \
        if (_r != CUDA_SUCCESS) return (int32_t)_r;     \
    } while (0)
#define CHECK_CTX(c)                                            \
    do {                                                        \
        if (!(c) || (c)->magic != QM_CTX_MAGIC) return QM_ERR_ARG; \
    } while (0)

struct qm_stack;
QmWeight *qm_weight_from_handle(qm_weight h);
int32_t qm_launch(qm_ctx *c, int kernel, unsigned gx, unsigned gy, unsigned block, unsigned smem, void *args,
                  bool pdl);
int32_t qm_launch_ex(qm_ctx *c, int kernel, unsigned gx, unsigned block, unsigned smem, void *args, bool pdl,
                     bool cooperative);
// Integer tensor-core path for Q4_K: plan for activation rows m and the largest K (in units)
// of the ops; QM_ERR_SHAPE when the activation planes do not fit in shared memory.
int qm_fused_grid(qm_ctx *c);
int64_t qm_wait_cycles();
void qm_balance_op(qm_ctx *c, QmOp *op);
struct QmGemmGroup {
    int experts;               // 0: a single matmul
    int m_typical;             // 0, or the list length to choose the token tile for (the grid still covers m)
    CUdeviceptr wq_list_dev;   // device array of the experts' weight stores
    CUdeviceptr offsets_dev;   // device array [experts + 1]: first activation row of each expert
    bool swiglu;               // gate|up weights, output bf16 silu(gate)*up to h_dev
    CUdeviceptr h_dev;
    int64_t ldh;
    // gather folded into the activation load: grouped row p is row list[p] / topk of a_dev
    // [rows_total][lda] (the tokens as the caller holds them); 0: a_dev is already grouped
    CUdeviceptr gather_list_dev;
    int gather_topk;
};
int32_t qm_gemm_launch(qm_ctx *c, const QmWeight *w, uint64_t a_dev, int32_t m, int64_t rows_total, int64_t lda,
                       uint64_t c_dev, int64_t ldc, const QmGemmGroup &g);
int qm_env_int(const char *name, int dflt);
int32_t qm_plan_fused(qm_ctx *c, int32_t m, int32_t units, bool allow_slices, QmFusedPlan *p);
void qm_fill_op(qm_ctx *c, const QmFusedPlan &p, const QmWeight *w, uint64_t x, uint64_t x2, int64_t ldx, uint64_t y,
                int64_t ldy, uint32_t xop, int barrier, int unit0, int units, int accumulate, QmOp *op);
int32_t qm_plan_gemv(qm_ctx *c, const QmWeight *w, int32_t m, QmGemvPlan *p);
// The same plan for a device with `sm_count` SMs (no context needed).
int32_t qm_plan_gemv_sms(int sm_count, const QmWeight *w, int32_t m, QmGemvPlan *p);
int32_t qm_matvec_launch(qm_ctx *c, const QmWeight *w, uint64_t x_dev, uint64_t x2_dev, int32_t m, int64_t ldx,
                         uint64_t y_dev, int64_t ldy, uint32_t flags, CUdeviceptr partials, CUdeviceptr tickets);
int32_t qm_kq_launch(qm_ctx *c, const QmWeight *w, uint64_t x_dev, bool xq, int32_t m, int64_t ldx, uint64_t y_dev,
                     int64_t ldy, uint64_t ids_dev, int32_t experts, int32_t slots, int64_t x_slot_stride, bool pdl);
