// qm_host.cpp — host side of libqmatmul.so: context, weight store, launch
// planning and the C ABI of include/qmatmul.h, over the CUDA driver API.
//
// There is no CPU implementation of any operation in this library: if libcuda
// or a kernel image cannot be loaded, qm_init fails and nothing else works.
#include <dlfcn.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <algorithm>
#include <mutex>
#include <new>

#include "../../include/qmatmul.h"
#include "qm_driver.h"
#include "qm_internal.h"

// ---- driver binding --------------------------------------------------------------
static QmDriver g_drv;
static std::once_flag g_drv_once;
static int g_drv_rc = QM_ERR_NO_DRIVER;

int qm_driver_load(QmDriver **out) {
    std::call_once(g_drv_once, [] {
        const char *path = getenv("CUDA_LIB_PATH");  // same override as nvidia/driver/init.gen.go:190
        void *h = nullptr;
        if (path && *path) h = dlopen(path, RTLD_LAZY | RTLD_GLOBAL);
        if (!h) h = dlopen("libcuda.so.1", RTLD_LAZY | RTLD_GLOBAL);
        if (!h) h = dlopen("libcuda.so", RTLD_LAZY | RTLD_GLOBAL);
        if (!h) return;
        bool ok = true;
#define X(name, ...)                                                          \
    g_drv.name = reinterpret_cast<qm_fnptr<__VA_ARGS__>>(dlsym(h, #name));   \
    if (!g_drv.name) ok = false;
        QM_DRV_FUNCS(X)
#undef X
        g_drv.loaded = ok;
        g_drv_rc = ok ? QM_OK : QM_ERR_NO_DRIVER;
    });
    *out = &g_drv;
    return g_drv_rc;
}

// ---- embedded kernel images --------------------------------------------------------
#define QM_STR2(x) #x
#define QM_STR(x) QM_STR2(x)
#define QM_INCBIN(sym, file)                                                               \
    __asm__(".section .rodata\n.balign 16\n.global " #sym "\n" #sym ":\n.incbin \"" file   \
            "\"\n.global " #sym "_end\n" #sym "_end:\n.byte 0\n.previous\n");              \
    extern "C" const unsigned char sym[];                                                  \
    extern "C" const unsigned char sym##_end[];

QM_INCBIN(qm_cubin_gemv, QM_STR(QM_CUBIN_DIR) "/qm_gemv.sm_100a.cubin")
QM_INCBIN(qm_cubin_dequant, QM_STR(QM_CUBIN_DIR) "/qm_dequant.sm_100a.cubin")
QM_INCBIN(qm_cubin_q4k, QM_STR(QM_CUBIN_DIR) "/qm_gemv_q4k.sm_100a.cubin")
QM_INCBIN(qm_cubin_gemm, QM_STR(QM_CUBIN_DIR) "/qm_gemm_q4k.sm_100a.cubin")
QM_INCBIN(qm_cubin_moe, QM_STR(QM_CUBIN_DIR) "/qm_moe.sm_100a.cubin")
QM_INCBIN(qm_cubin_kq, QM_STR(QM_CUBIN_DIR) "/qm_gemv_kq.sm_100a.cubin")
QM_INCBIN(qm_cubin_q81, QM_STR(QM_CUBIN_DIR) "/qm_q8_1.sm_100a.cubin")

struct KernelImage {
    const unsigned char *begin;
    const unsigned char *end;
};
static const KernelImage kImages[QM_MOD_COUNT] = {
    {qm_cubin_gemv, qm_cubin_gemv_end},
    {qm_cubin_dequant, qm_cubin_dequant_end},
    {qm_cubin_q4k, qm_cubin_q4k_end},
    {qm_cubin_gemm, qm_cubin_gemm_end},
    {qm_cubin_moe, qm_cubin_moe_end},
    {qm_cubin_kq, qm_cubin_kq_end},
    {qm_cubin_q81, qm_cubin_q81_end},
};
struct KernelName {
    int module;
    const char *name;
};
static const KernelName kKernels[QM_K_COUNT] = {
    {QM_MOD_GEMV, "qm_gemv_q40_m4"},
    {QM_MOD_GEMV, "qm_gemv_q40_m8"},   {QM_MOD_GEMV, "qm_gemv_q80_m4"},    {QM_MOD_GEMV, "qm_gemv_q80_m8"},
    {QM_MOD_DEQUANT, "qm_dequant_q4k"}, {QM_MOD_DEQUANT, "qm_dequant_q2k"}, {QM_MOD_DEQUANT, "qm_dequant_q40"},
    {QM_MOD_DEQUANT, "qm_dequant_q80"}, {QM_MOD_DEQUANT, "qm_repack_q40"},  {QM_MOD_DEQUANT, "qm_repack_q80"},
    {QM_MOD_DEQUANT, "qm_repack_q4k"},
    {QM_MOD_Q4K, "qm_fused_q4k_nt1"},  {QM_MOD_Q4K, "qm_fused_q4k_nt2"},
    {QM_MOD_Q4K, "qm_fused_q4k_nt1_img"},  {QM_MOD_Q4K, "qm_fused_q4k_nt2_img"},
    {QM_MOD_Q4K, "qm_fused_q4k_nt1_tp"},  {QM_MOD_Q4K, "qm_fused_q4k_nt2_tp"},
    {QM_MOD_Q4K, "qm_fused_q4k_dd_c4d2"}, {QM_MOD_Q4K, "qm_fused_q4k_dd_c4d3"}, {QM_MOD_Q4K, "qm_fused_q4k_dd_c4d4"},
    {QM_MOD_Q4K, "qm_fused_q4k_dd_c2d2"}, {QM_MOD_Q4K, "qm_fused_q4k_dd_c2d3"}, {QM_MOD_Q4K, "qm_fused_q4k_dd_c2d4"},
    {QM_MOD_Q4K, "qm_fused_q4k_dd_c4d2_tp"}, {QM_MOD_Q4K, "qm_fused_q4k_dd_c4d3_tp"}, {QM_MOD_Q4K, "qm_fused_q4k_dd_c4d4_tp"},
    {QM_MOD_Q4K, "qm_fused_q4k_dd_c2d2_tp"}, {QM_MOD_Q4K, "qm_fused_q4k_dd_c2d3_tp"}, {QM_MOD_Q4K, "qm_fused_q4k_dd_c2d4_tp"},
    {QM_MOD_Q4K, "qm_sum_parts"}, {QM_MOD_DEQUANT, "qm_repack_parts"},
    {QM_MOD_GEMM, "qm_gemm_q4k_bf16"}, {QM_MOD_GEMM, "qm_gemm_q4k_bf16_r256"},
    {QM_MOD_GEMM, "qm_gemm_q4k_bf16_k128"}, {QM_MOD_GEMM, "qm_gemm_q4k_bf16_r256_k128"},
    {QM_MOD_MOE, "qm_moe_route"},      {QM_MOD_MOE, "qm_moe_lists"},      {QM_MOD_MOE, "qm_moe_gather"},
    {QM_MOD_MOE, "qm_moe_combine"},
    {QM_MOD_DEQUANT, "qm_dequant_iq2xxs"},
    {QM_MOD_KQ, "qm_gemv_q2k_m1"},     {QM_MOD_KQ, "qm_gemv_q2k_m2"},     {QM_MOD_KQ, "qm_gemv_q2k_m4"},
    {QM_MOD_KQ, "qm_gemv_q2k_m8"},     {QM_MOD_KQ, "qm_gemv_iq2xxs_m1"},  {QM_MOD_KQ, "qm_gemv_iq2xxs_m2"},
    {QM_MOD_KQ, "qm_gemv_iq2xxs_m4"},  {QM_MOD_KQ, "qm_gemv_iq2xxs_m8"},
    {QM_MOD_KQ, "qm_gemv_q2k_q81_m1"}, {QM_MOD_KQ, "qm_gemv_q2k_q81_m2"}, {QM_MOD_KQ, "qm_gemv_q2k_q81_m4"},
    {QM_MOD_KQ, "qm_gemv_q2k_q81_m8"}, {QM_MOD_KQ, "qm_gemv_iq2xxs_q81_m1"}, {QM_MOD_KQ, "qm_gemv_iq2xxs_q81_m2"},
    {QM_MOD_KQ, "qm_gemv_iq2xxs_q81_m4"}, {QM_MOD_KQ, "qm_gemv_iq2xxs_q81_m8"},
    {QM_MOD_Q81, "qm_rmsnorm_q8_1"},   {QM_MOD_Q81, "qm_swiglu_q8_1"},    {QM_MOD_Q81, "qm_q8_1_expand"},
    {QM_MOD_Q4K, "qm_fused_q4k_dd_c4d2_sel"}, {QM_MOD_Q4K, "qm_fused_q4k_dd_c4d3_sel"}, {QM_MOD_Q4K, "qm_fused_q4k_dd_c4d4_sel"},
    {QM_MOD_MOE, "qm_moe_decode_combine"},
    {QM_MOD_MOE, "qm_ep_push"},        {QM_MOD_MOE, "qm_ep_collect"},     {QM_MOD_MOE, "qm_ep_return"},
    {QM_MOD_MOE, "qm_ep_combine"},
    {QM_MOD_Q4K, "qm_gemv_q40_lean_c4d4"}, {QM_MOD_Q4K, "qm_gemv_q40_lean_c4d2"}, {QM_MOD_Q4K, "qm_gemv_q40_lean_c2d4"},
    {QM_MOD_Q4K, "qm_gemv_q40_lean_c2d2"}, {QM_MOD_Q4K, "qm_gemv_q40_lean_c2n2d4"}, {QM_MOD_Q4K, "qm_gemv_q40_lean_c2n2d2"},
    {QM_MOD_Q4K, "qm_gemv_q80_lean_c4d3"}, {QM_MOD_Q4K, "qm_gemv_q80_lean_c4d2"}, {QM_MOD_Q4K, "qm_gemv_q80_lean_c2d3"},
    {QM_MOD_Q4K, "qm_gemv_q80_lean_c2d2"}, {QM_MOD_Q4K, "qm_gemv_q80_lean_c2n2d3"}, {QM_MOD_Q4K, "qm_gemv_q80_lean_c2n2d2"},
    {QM_MOD_Q4K, "qm_lean_sum"},
    {QM_MOD_Q4K, "qm_fused_q4k_dd_n2d2"}, {QM_MOD_Q4K, "qm_fused_q4k_dd_n2d3"},
};

// ---- errors --------------------------------------------------------------------------
extern "C" int32_t qm_version(void) { return QM_VERSION; }

extern "C" const char *qm_error_string(int32_t code) {
    switch (code) {
    case QM_OK: return "success";
    case QM_ERR_COUNT: return "quant: element count is not a non-negative multiple of the block";
    case QM_ERR_BUFFER: return "quant: buffer length insufficient for the blocks";
    case QM_ERR_FORMAT: return "quant: unknown or unsupported weight format";
    case QM_ERR_SHAPE: return "quant: shape out of range for the operation";
    case QM_ERR_ARG: return "quant: null pointer or invalid handle";
    case QM_ERR_NO_DRIVER: return "quant: CUDA driver library not available";
    case QM_ERR_NO_KERNEL: return "quant: kernel image failed to load";
    case QM_ERR_TIMEOUT: return "quant: bounded device wait expired";
    case QM_ERR_NOMEM: return "quant: host allocation failed";
    case QM_ERR_STATE: return "quant: call not valid in this state";
    case QM_ERR_LIMIT: return "quant: size beyond the fixed maximum of this entry point";
    case QM_ERR_DOMAIN: return "cudaquant: nonfinite value or zero normalization denominator";
    }
    if (code > 0 && g_drv.loaded) {
        const char *s = nullptr;
        if (g_drv.cuGetErrorString((CUresult)code, &s) == CUDA_SUCCESS && s) return s;
    }
    return "quant: unknown status";
}

// ---- context -----------------------------------------------------------------------------
CtxGuard::CtxGuard(qm_ctx *c) : ctx(c) { rc = c->drv->cuCtxPushCurrent_v2(c->cuctx); }
CtxGuard::~CtxGuard() {
    if (rc == CUDA_SUCCESS) {
        CUcontext old;
        ctx->drv->cuCtxPopCurrent_v2(&old);
    }
}

extern "C" int32_t qm_init(int32_t device, qm_ctx **out) {
    if (!out) return QM_ERR_ARG;
    *out = nullptr;
    QmDriver *d;
    int rc = qm_driver_load(&d);
    if (rc) return rc;
    DRV(d->cuInit(0));
    qm_ctx *c = new (std::nothrow) qm_ctx();
    if (!c) return QM_ERR_NOMEM;
    c->magic = QM_CTX_MAGIC;
    c->drv = d;
    c->device = device;
    CUresult r = d->cuDeviceGet(&c->cudev, device);
    if (r == CUDA_SUCCESS) r = d->cuDevicePrimaryCtxRetain(&c->cuctx, c->cudev);
    if (r != CUDA_SUCCESS) {
        delete c;
        return (int32_t)r;
    }
    c->have_ctx = true;
    int32_t err = QM_OK;
    {
        CtxGuard g(c);
        if (g.rc != CUDA_SUCCESS) err = (int32_t)g.rc;
        int major = 0, minor = 0;
        if (!err) {
            d->cuDeviceGetAttribute(&major, CU_DEVICE_ATTRIBUTE_COMPUTE_CAPABILITY_MAJOR, c->cudev);
            d->cuDeviceGetAttribute(&minor, CU_DEVICE_ATTRIBUTE_COMPUTE_CAPABILITY_MINOR, c->cudev);
            d->cuDeviceGetAttribute(&c->sm_count, CU_DEVICE_ATTRIBUTE_MULTIPROCESSOR_COUNT, c->cudev);
            d->cuDeviceGetAttribute(&c->l2_bytes, CU_DEVICE_ATTRIBUTE_L2_CACHE_SIZE, c->cudev);
        }
        for (int m = 0; m < QM_MOD_COUNT && !err; m++) {
            // the images are sm_100a cubins: loading fails on any other device
            r = d->cuModuleLoadData(&c->modules[m], kImages[m].begin);
            if (r != CUDA_SUCCESS) {
                fprintf(stderr, "qmatmul: kernel image %d failed to load on sm_%d%d: %s\n", m, major, minor,
                        qm_error_string((int32_t)r));
                err = QM_ERR_NO_KERNEL;
            }
        }
        for (int k = 0; k < QM_K_COUNT && !err; k++) {
            r = d->cuModuleGetFunction(&c->fn[k], c->modules[kKernels[k].module], kKernels[k].name);
            if (r != CUDA_SUCCESS) err = QM_ERR_NO_KERNEL;
        }
        for (int k = QM_K_FUSED_Q4K_NT1; k <= QM_K_FUSED_Q4K_DD_C2D4_TP && !err; k++) {
            r = d->cuFuncSetAttribute(c->fn[k], CU_FUNC_ATTRIBUTE_MAX_DYNAMIC_SHARED_SIZE_BYTES, QM_GEMV_SMEM_MAX);
            if (r != CUDA_SUCCESS) err = (int32_t)r;
        }
        if (!err) {
            r = d->cuFuncSetAttribute(c->fn[QM_K_GEMM_Q4K], CU_FUNC_ATTRIBUTE_MAX_DYNAMIC_SHARED_SIZE_BYTES, QM_GEMV_SMEM_MAX);
            for (int k = QM_K_GEMM_Q4K_R256; k <= QM_K_GEMM_Q4K_R256_K128 && r == CUDA_SUCCESS; k++)
                r = d->cuFuncSetAttribute(c->fn[k], CU_FUNC_ATTRIBUTE_MAX_DYNAMIC_SHARED_SIZE_BYTES, QM_GEMV_SMEM_MAX);

            if (r != CUDA_SUCCESS) err = (int32_t)r;
        }
        for (int k = QM_K_FUSED_Q4K_DD_N2D2; k <= QM_K_FUSED_Q4K_DD_N2D3 && !err; k++) {
            r = d->cuFuncSetAttribute(c->fn[k], CU_FUNC_ATTRIBUTE_MAX_DYNAMIC_SHARED_SIZE_BYTES, QM_GEMV_SMEM_MAX);
            if (r != CUDA_SUCCESS) err = (int32_t)r;
        }
        for (int k = QM_K_Q40_LEAN_C4D4; k <= QM_K_Q80_LEAN_C2N2D2 && !err; k++) {
            r = d->cuFuncSetAttribute(c->fn[k], CU_FUNC_ATTRIBUTE_MAX_DYNAMIC_SHARED_SIZE_BYTES, QM_GEMV_SMEM_MAX);
            if (r != CUDA_SUCCESS) err = (int32_t)r;
        }
        for (int k = QM_K_FUSED_Q4K_DD_C4D2_SEL; k <= QM_K_FUSED_Q4K_DD_C4D4_SEL && !err; k++) {
            r = d->cuFuncSetAttribute(c->fn[k], CU_FUNC_ATTRIBUTE_MAX_DYNAMIC_SHARED_SIZE_BYTES, QM_GEMV_SMEM_MAX);
            if (r != CUDA_SUCCESS) err = (int32_t)r;
        }
        for (int k = QM_K_GEMV_Q2K_M1; k <= QM_K_GEMV_IQ2XXS_Q81_M8 && !err; k++) {
            r = d->cuFuncSetAttribute(c->fn[k], CU_FUNC_ATTRIBUTE_MAX_DYNAMIC_SHARED_SIZE_BYTES, QM_KQ_SMEM_MAX);
            if (r != CUDA_SUCCESS) err = (int32_t)r;
        }
        for (int k = QM_K_GEMV_Q40_M4; k <= QM_K_GEMV_Q80_M8 && !err; k++) {
            r = d->cuFuncSetAttribute(c->fn[k], CU_FUNC_ATTRIBUTE_MAX_DYNAMIC_SHARED_SIZE_BYTES, QM_GEMV_SMEM_MAX);
            if (r != CUDA_SUCCESS) err = (int32_t)r;
        }
        if (!err) {
            r = d->cuStreamCreate(&c->own_stream, CU_STREAM_NON_BLOCKING);
            if (r != CUDA_SUCCESS) err = (int32_t)r;
            c->stream = c->own_stream;
        }
        if (!err) {
            r = d->cuMemAlloc_v2(&c->status_dev, 32768);
            if (r == CUDA_SUCCESS) r = d->cuMemsetD8Async(c->status_dev, 0, 32768, c->stream);
            if (r == CUDA_SUCCESS) r = d->cuMemAlloc_v2(&c->tickets_dev, QM_TICKETS * sizeof(unsigned));
            if (r == CUDA_SUCCESS) r = d->cuMemsetD8Async(c->tickets_dev, 0, QM_TICKETS * sizeof(unsigned), c->stream);
            if (r == CUDA_SUCCESS) r = d->cuMemAlloc_v2(&c->partials_dev, QM_PARTIALS_BYTES);
            if (r == CUDA_SUCCESS) r = d->cuMemAlloc_v2(&c->gridbar_dev, 256);
            if (r == CUDA_SUCCESS) r = d->cuMemsetD8Async(c->gridbar_dev, 0, 256, c->stream);
            if (r == CUDA_SUCCESS) r = d->cuStreamSynchronize(c->stream);
            if (r != CUDA_SUCCESS) err = (int32_t)r;
        }
    }
    if (err) {
        qm_destroy(c);
        return err;
    }
    *out = c;
    return QM_OK;
}

extern "C" int32_t qm_destroy(qm_ctx *c) {
    if (!c || c->magic != QM_CTX_MAGIC) return QM_ERR_ARG;
    QmDriver *d = c->drv;
    if (c->have_ctx) {
        CtxGuard g(c);
        if (g.rc == CUDA_SUCCESS) {
            if (c->own_stream) d->cuStreamSynchronize(c->own_stream);
            if (c->status_dev) d->cuMemFree_v2(c->status_dev);
            if (c->tickets_dev) d->cuMemFree_v2(c->tickets_dev);
            if (c->partials_dev) d->cuMemFree_v2(c->partials_dev);
            if (c->gridbar_dev) d->cuMemFree_v2(c->gridbar_dev);
            if (c->xstage_dev) d->cuMemFree_v2(c->xstage_dev);
            if (c->upload_dev) d->cuMemFree_v2(c->upload_dev);
            if (c->moe_ws) d->cuMemFree_v2(c->moe_ws);
            if (c->moe_ws2) d->cuMemFree_v2(c->moe_ws2);
            if (c->moe_ws3) d->cuMemFree_v2(c->moe_ws3);
            if (c->q81_ws) d->cuMemFree_v2(c->q81_ws);
            if (c->own_stream) d->cuStreamDestroy_v2(c->own_stream);
            for (int m = 0; m < QM_MOD_COUNT; m++)
                if (c->modules[m]) d->cuModuleUnload(c->modules[m]);
        }
    }
    if (c->have_ctx) d->cuDevicePrimaryCtxRelease_v2(c->cudev);
    c->magic = 0;
    delete c;
    return QM_OK;
}

extern "C" int32_t qm_set_stream(qm_ctx *c, uint64_t s) {
    CHECK_CTX(c);
    c->stream = s ? (CUstream)(uintptr_t)s : c->own_stream;
    return QM_OK;
}

extern "C" int32_t qm_sync(qm_ctx *c) {
    CHECK_CTX(c);
    CtxGuard g(c);
    DRV(g.rc);
    DRV(c->drv->cuStreamSynchronize(c->stream));
    return QM_OK;
}

extern "C" int32_t qm_last_status(qm_ctx *c, uint32_t *status) {
    CHECK_CTX(c);
    if (!status) return QM_ERR_ARG;
    CtxGuard g(c);
    DRV(g.rc);
    DRV(c->drv->cuStreamSynchronize(c->stream));
    DRV(c->drv->cuMemcpyDtoH_v2(status, c->status_dev, 4));
    if (*status) DRV(c->drv->cuMemsetD8Async(c->status_dev, 0, 4, c->stream));
    return (*status & QM_STATUS_TIMEOUT) ? QM_ERR_TIMEOUT : (*status & QM_STATUS_DOMAIN) ? QM_ERR_DOMAIN : QM_OK;
}

#ifdef QM_DEBUG
// Debug builds only: raw copy of the device status block (status word + phase timestamps).
extern "C" __attribute__((visibility("default"))) int32_t qm_debug_status(qm_ctx *c, void *out, int64_t bytes) {
    CHECK_CTX(c);
    CtxGuard g(c);
    DRV(g.rc);
    DRV(c->drv->cuStreamSynchronize(c->stream));
    DRV(c->drv->cuMemcpyDtoH_v2(out, c->status_dev, (size_t)std::min<int64_t>(bytes, 32768)));
    return QM_OK;
}
#endif

extern "C" int64_t qm_launch_count(qm_ctx *c) {
    if (!c || c->magic != QM_CTX_MAGIC) return -1;
    return c->launches;
}

extern "C" int32_t qm_malloc(qm_ctx *c, int64_t bytes, uint64_t *dptr) {
    CHECK_CTX(c);
    if (!dptr || bytes < 0) return QM_ERR_ARG;
    CtxGuard g(c);
    DRV(g.rc);
    CUdeviceptr p = 0;
    DRV(c->drv->cuMemAlloc_v2(&p, bytes ? (size_t)bytes : 1));
    *dptr = (uint64_t)p;
    return QM_OK;
}
extern "C" int32_t qm_free(qm_ctx *c, uint64_t dptr) {
    CHECK_CTX(c);
    CtxGuard g(c);
    DRV(g.rc);
    if (dptr) DRV(c->drv->cuMemFree_v2((CUdeviceptr)dptr));
    return QM_OK;
}
extern "C" int32_t qm_memcpy_h2d(qm_ctx *c, uint64_t dst, const void *src, int64_t bytes) {
    CHECK_CTX(c);
    if (bytes < 0 || (bytes && (!dst || !src))) return QM_ERR_ARG;
    CtxGuard g(c);
    DRV(g.rc);
    if (bytes) {
        DRV(c->drv->cuMemcpyHtoDAsync_v2((CUdeviceptr)dst, src, (size_t)bytes, c->stream));
        DRV(c->drv->cuStreamSynchronize(c->stream));
    }
    return QM_OK;
}
extern "C" int32_t qm_memcpy_d2h(qm_ctx *c, void *dst, uint64_t src, int64_t bytes) {
    CHECK_CTX(c);
    if (bytes < 0 || (bytes && (!dst || !src))) return QM_ERR_ARG;
    CtxGuard g(c);
    DRV(g.rc);
    if (bytes) {
        DRV(c->drv->cuMemcpyDtoHAsync_v2(dst, (CUdeviceptr)src, (size_t)bytes, c->stream));
        DRV(c->drv->cuStreamSynchronize(c->stream));
    }
    return QM_OK;
}

// ---- launch helper ----------------------------------------------------------------------
static int32_t launch_grid(qm_ctx *c, int kernel, unsigned gx, unsigned gy, unsigned block, unsigned smem, void *args,
                           bool pdl, bool cooperative) {
    void *params[1] = {args};
    CUlaunchConfig cfg;
    memset(&cfg, 0, sizeof cfg);
    cfg.gridDimX = gx;
    cfg.gridDimY = gy;
    cfg.gridDimZ = 1;
    cfg.blockDimX = block;
    cfg.blockDimY = 1;
    cfg.blockDimZ = 1;
    cfg.sharedMemBytes = smem;
    cfg.hStream = c->stream;
    CUlaunchAttribute attr[2];
    unsigned n = 0;
    if (pdl) {
        attr[n].id = CU_LAUNCH_ATTRIBUTE_PROGRAMMATIC_STREAM_SERIALIZATION;
        attr[n].value.programmaticStreamSerializationAllowed = 1;
        n++;
    }
    if (cooperative) {  // all CTAs co-resident: required by the grid barrier between fused ops
        attr[n].id = CU_LAUNCH_ATTRIBUTE_COOPERATIVE;
        attr[n].value.cooperative = 1;
        n++;
    }
    cfg.attrs = n ? attr : nullptr;
    cfg.numAttrs = n;
    DRV(c->drv->cuLaunchKernelEx(&cfg, c->fn[kernel], params, nullptr));
    c->launches++;
    return QM_OK;
}

int32_t qm_launch_ex(qm_ctx *c, int kernel, unsigned gx, unsigned block, unsigned smem, void *args, bool pdl,
                     bool cooperative) {
    return launch_grid(c, kernel, gx, 1, block, smem, args, pdl, cooperative);
}

int32_t qm_launch(qm_ctx *c, int kernel, unsigned gx, unsigned gy, unsigned block, unsigned smem, void *args,
                  bool pdl) {
    return launch_grid(c, kernel, gx, gy ? gy : 1, block, smem, args, pdl, false);
}

// ---- weight store -----------------------------------------------------------------------
static bool fmt_geometry(int32_t fmt, int64_t *block, int64_t *bytes) {
    switch (fmt) {
    case QM_FMT_Q4_0: *block = 32; *bytes = 18; return true;
    case QM_FMT_Q8_0: *block = 32; *bytes = 34; return true;
    case QM_FMT_Q2_K: *block = 256; *bytes = 84; return true;
    case QM_FMT_Q4_K: *block = 256; *bytes = 144; return true;
    case QM_FMT_IQ2_XXS: *block = 256; *bytes = 66; return true;
    }
    return false;
}

QmWeight *qm_weight_from_handle(qm_weight h) {
    QmWeight *w = reinterpret_cast<QmWeight *>((uintptr_t)h);
    if (!w || w->magic != QM_WEIGHT_MAGIC) return nullptr;
    return w;
}

extern "C" int32_t qm_store_create(qm_ctx *c, int32_t fmt, int64_t rows, int64_t cols, qm_weight *out) {
    CHECK_CTX(c);
    if (!out) return QM_ERR_ARG;
    *out = 0;
    int64_t block, bbytes;
    if (!fmt_geometry(fmt, &block, &bbytes)) return QM_ERR_FORMAT;
    if (cols < 0 || cols % block != 0) return QM_ERR_COUNT;  // gguf/gguf.go:290-292
    if (rows <= 0 || cols <= 0 || rows > (1 << 30) || cols > (1 << 24)) return QM_ERR_SHAPE;
    QmWeight *w = new (std::nothrow) QmWeight();
    if (!w) return QM_ERR_NOMEM;
    w->magic = QM_WEIGHT_MAGIC;
    w->fmt = fmt;
    w->device = c->device;
    w->rows = rows;
    w->cols = cols;
    w->units = (int32_t)((cols + QM_K_UNIT - 1) / QM_K_UNIT);
    w->gguf_row_bytes = cols / block * bbytes;
    int64_t qbytes = 0, dbytes = 0;
    if (fmt == QM_FMT_Q2_K || fmt == QM_FMT_IQ2_XXS) qbytes = rows * w->units * bbytes;
    if (fmt == QM_FMT_Q4_K) qbytes = (rows + 15) / 16 * w->units * QM_Q4K_ITEM_BYTES;  // whole 16-row tiles
    if (fmt == QM_FMT_Q4_0) { qbytes = rows * w->units * 8 * 16; dbytes = rows * w->units * 8 * 2; }
    if (fmt == QM_FMT_Q8_0) { qbytes = rows * w->units * 8 * 32; dbytes = rows * w->units * 8 * 2; }
    w->qbytes = qbytes;
    w->dbytes = dbytes;
    CtxGuard g(c);
    CUresult r = g.rc;
    // 64 bytes of slack: rows past the last one are clamped, never read beyond
    if (r == CUDA_SUCCESS) r = c->drv->cuMemAlloc_v2(&w->wq, (size_t)qbytes + 64);
    if (r == CUDA_SUCCESS && dbytes) r = c->drv->cuMemAlloc_v2(&w->wd, (size_t)dbytes + 64);
    // padding must read as zero: Q4_0/Q8_0 rows that end inside a K unit, Q4_K rows past the last
    if (r == CUDA_SUCCESS && (dbytes || fmt == QM_FMT_Q4_K))
        r = c->drv->cuMemsetD8Async(w->wq, 0, (size_t)qbytes + 64, c->stream);
    if (r == CUDA_SUCCESS && dbytes) r = c->drv->cuMemsetD8Async(w->wd, 0, (size_t)dbytes + 64, c->stream);
    if (r != CUDA_SUCCESS) {
        if (w->wq) c->drv->cuMemFree_v2(w->wq);
        if (w->wd) c->drv->cuMemFree_v2(w->wd);
        delete w;
        return (int32_t)r;
    }
    *out = (qm_weight)(uintptr_t)w;
    return QM_OK;
}

static int32_t store_write_dev(qm_ctx *c, QmWeight *w, int64_t row_offset, int64_t nrows, CUdeviceptr src) {
    if (w->fmt == QM_FMT_Q2_K || w->fmt == QM_FMT_IQ2_XXS) {
        DRV(c->drv->cuMemcpyDtoDAsync_v2(w->wq + row_offset * w->gguf_row_bytes, src,
                                         (size_t)(nrows * w->gguf_row_bytes), c->stream));
        return QM_OK;
    }
    QmRepackArgs a;
    a.src = (const uint8_t *)(uintptr_t)src;
    a.wq = (uint8_t *)(uintptr_t)w->wq;
    a.wd = (uint16_t *)(uintptr_t)w->wd;
    a.row_offset = row_offset;
    a.nrows = nrows;
    a.cols = (int32_t)w->cols;
    a.units = w->units;
    const int64_t nblk = nrows * (w->cols / (w->fmt == QM_FMT_Q4_K ? 256 : 32));
    const unsigned grid = (unsigned)std::min<int64_t>((nblk + 255) / 256, 148 * 16);
    const int k = w->fmt == QM_FMT_Q4_0 ? QM_K_REPACK_Q40 : w->fmt == QM_FMT_Q8_0 ? QM_K_REPACK_Q80 : QM_K_REPACK_Q4K;
    return qm_launch(c, k, grid, 1, 256, 0, &a, false);
}

extern "C" int32_t qm_store_write_rows_device(qm_ctx *c, qm_weight h, int64_t row_offset, int64_t nrows,
                                              uint64_t dev_bytes, int64_t len) {
    CHECK_CTX(c);
    QmWeight *w = qm_weight_from_handle(h);
    if (!w || !dev_bytes) return QM_ERR_ARG;
    if (row_offset < 0 || nrows < 0 || row_offset + nrows > w->rows) return QM_ERR_SHAPE;
    if (len < nrows * w->gguf_row_bytes) return QM_ERR_BUFFER;
    if ((dev_bytes & (w->fmt == QM_FMT_Q4_K ? 15 : 1)) != 0) return QM_ERR_ARG;
    if (nrows == 0) return QM_OK;
    CtxGuard g(c);
    DRV(g.rc);
    return store_write_dev(c, w, row_offset, nrows, (CUdeviceptr)dev_bytes);
}

extern "C" int32_t qm_store_write_rows(qm_ctx *c, qm_weight h, int64_t row_offset, int64_t nrows,
                                       const void *host_bytes, int64_t len) {
    CHECK_CTX(c);
    QmWeight *w = qm_weight_from_handle(h);
    if (!w || !host_bytes) return QM_ERR_ARG;
    if (row_offset < 0 || nrows < 0 || row_offset + nrows > w->rows) return QM_ERR_SHAPE;
    if (len < nrows * w->gguf_row_bytes) return QM_ERR_BUFFER;
    if (nrows == 0) return QM_OK;
    CtxGuard g(c);
    DRV(g.rc);
    const int64_t bytes = nrows * w->gguf_row_bytes;
    if (w->fmt == QM_FMT_Q2_K || w->fmt == QM_FMT_IQ2_XXS) {
        // GGUF bytes are the device layout: copy straight into place
        DRV(c->drv->cuMemcpyHtoDAsync_v2(w->wq + row_offset * w->gguf_row_bytes, host_bytes, (size_t)bytes,
                                         c->stream));
        DRV(c->drv->cuStreamSynchronize(c->stream));
        return QM_OK;
    }
    // stage the GGUF bytes on the device, then permute them into the store layout
    const int64_t chunk_rows = std::max<int64_t>(1, QM_UPLOAD_CHUNK / w->gguf_row_bytes);
    if (!c->upload_dev) DRV(c->drv->cuMemAlloc_v2(&c->upload_dev, QM_UPLOAD_CHUNK + w->gguf_row_bytes));
    if (w->gguf_row_bytes > QM_UPLOAD_CHUNK) return QM_ERR_SHAPE;
    for (int64_t r0 = 0; r0 < nrows; r0 += chunk_rows) {
        const int64_t nr = std::min(chunk_rows, nrows - r0);
        DRV(c->drv->cuMemcpyHtoDAsync_v2(c->upload_dev, (const uint8_t *)host_bytes + r0 * w->gguf_row_bytes,
                                         (size_t)(nr * w->gguf_row_bytes), c->stream));
        int32_t rc = store_write_dev(c, w, row_offset + r0, nr, c->upload_dev);
        if (rc) return rc;
        DRV(c->drv->cuStreamSynchronize(c->stream));  // the staging buffer is reused
    }
    return QM_OK;
}

extern "C" int32_t qm_store_upload(qm_ctx *c, int32_t fmt, int64_t rows, int64_t cols, const void *host_bytes,
                                   int64_t len, int64_t row_lo, int64_t row_hi, qm_weight *out) {
    CHECK_CTX(c);
    if (!out) return QM_ERR_ARG;
    *out = 0;
    int64_t block, bbytes;
    if (!fmt_geometry(fmt, &block, &bbytes)) return QM_ERR_FORMAT;
    if (rows < 0 || cols < 0 || cols % block != 0) return QM_ERR_COUNT;
    if (!host_bytes) return QM_ERR_ARG;
    if (row_lo < 0 || row_hi > rows || row_lo >= row_hi) return QM_ERR_SHAPE;
    const int64_t row_bytes = cols / block * bbytes;
    if (len < rows * row_bytes) return QM_ERR_BUFFER;  // trailing bytes are accepted (lm/quant/quant.go:49)
    qm_weight h = 0;
    int32_t rc = qm_store_create(c, fmt, row_hi - row_lo, cols, &h);
    if (rc) return rc;
    rc = qm_store_write_rows(c, h, 0, row_hi - row_lo, (const uint8_t *)host_bytes + row_lo * row_bytes,
                             (row_hi - row_lo) * row_bytes);
    if (rc) {
        qm_store_free(c, h);
        return rc;
    }
    *out = h;
    return QM_OK;
}

extern "C" int32_t qm_store_free(qm_ctx *c, qm_weight h) {
    CHECK_CTX(c);
    QmWeight *w = qm_weight_from_handle(h);
    if (!w) return QM_ERR_ARG;
    CtxGuard g(c);
    DRV(g.rc);
    c->drv->cuStreamSynchronize(c->stream);
    if (w->wq) c->drv->cuMemFree_v2(w->wq);
    if (w->wd) c->drv->cuMemFree_v2(w->wd);
    w->magic = 0;
    delete w;
    return QM_OK;
}

extern "C" int32_t qm_store_info(qm_ctx *c, qm_weight h, int64_t *info5) {
    CHECK_CTX(c);
    QmWeight *w = qm_weight_from_handle(h);
    if (!w || !info5) return QM_ERR_ARG;
    info5[0] = w->fmt;
    info5[1] = w->rows;
    info5[2] = w->cols;
    info5[3] = w->qbytes + w->dbytes;
    info5[4] = w->rows * w->gguf_row_bytes;
    return QM_OK;
}

// ---- dequantize ---------------------------------------------------------------------------
extern "C" int32_t qm_dequantize(qm_ctx *c, qm_weight h, uint64_t out_dev) {
    CHECK_CTX(c);
    QmWeight *w = qm_weight_from_handle(h);
    if (!w || !out_dev || (out_dev & 15)) return QM_ERR_ARG;
    CtxGuard g(c);
    DRV(g.rc);
    QmDequantArgs a;
    a.wq = (const uint8_t *)(uintptr_t)w->wq;
    a.wd = (const uint16_t *)(uintptr_t)w->wd;
    a.out = (float *)(uintptr_t)out_dev;
    a.rows = w->rows;
    a.cols = (int32_t)w->cols;
    a.units = w->units;
    int k = w->fmt == QM_FMT_Q4_K ? QM_K_DEQUANT_Q4K : w->fmt == QM_FMT_Q2_K ? QM_K_DEQUANT_Q2K
          : w->fmt == QM_FMT_IQ2_XXS ? QM_K_DEQUANT_IQ2XXS
          : w->fmt == QM_FMT_Q4_0 ? QM_K_DEQUANT_Q40 : QM_K_DEQUANT_Q80;
    const int64_t groups = w->rows * (w->cols / 4);
    const unsigned grid = (unsigned)std::min<int64_t>((groups + 255) / 256, (int64_t)c->sm_count * 32);
    return qm_launch(c, k, grid, 1, 256, 0, &a, false);
}

extern "C" int32_t qm_dequantize_host(qm_ctx *c, int32_t fmt, const void *data, int64_t len, int64_t n,
                                      float *out_host) {
    CHECK_CTX(c);
    int64_t block, bbytes;
    if (!fmt_geometry(fmt, &block, &bbytes)) return QM_ERR_FORMAT;
    // validation order of lm/quant/quant.go:45-51
    if (n < 0 || n % block != 0) return QM_ERR_COUNT;
    if (len < 0 || len < n / block * bbytes) return QM_ERR_BUFFER;
    if (n == 0) return QM_OK;
    if (!data || !out_host) return QM_ERR_ARG;
    // one logical row of n elements, cut into rows of at most 2^20 elements for the store
    const int64_t row_elems = (n % (1 << 20) == 0) ? (1 << 20) : (n <= (1 << 24) ? n : block);
    const int64_t rows = n / row_elems;
    qm_weight h = 0;
    int32_t rc = qm_store_upload(c, fmt, rows, row_elems, data, len, 0, rows, &h);
    if (rc) return rc;
    uint64_t out_dev = 0;
    rc = qm_malloc(c, n * 4, &out_dev);
    if (!rc) rc = qm_dequantize(c, h, out_dev);
    if (!rc) rc = qm_memcpy_d2h(c, out_host, out_dev, n * 4);
    if (out_dev) qm_free(c, out_dev);
    qm_store_free(c, h);
    return rc;
}

// ---- matvec ---------------------------------------------------------------------------------
int qm_env_int(const char *name, int dflt);
static int env_int(const char *name, int dflt) { return qm_env_int(name, dflt); }
int qm_env_int(const char *name, int dflt) {
    const char *s = getenv(name);
    return (s && *s) ? atoi(s) : dflt;
}

int32_t qm_plan_gemv(qm_ctx *c, const QmWeight *w, int32_t m, QmGemvPlan *p) {
    return qm_plan_gemv_sms(c->sm_count, w, m, p);
}

int32_t qm_plan_gemv_sms(int sm_count, const QmWeight *w, int32_t m, QmGemvPlan *p) {
    // One persistent CTA per SM: `consumers` warps, each streaming its own share of the
    // (16-row tile, K unit) items through a private ring of `depth` bulk-copy stages of `kc`
    // units. The activations of the CTA's K slice live in shared memory next to the rings; when
    // they do not fit, K is cut into slices and groups of CTAs take one slice each.
    const int q = w->fmt == QM_FMT_Q4_0 ? 128 : 256;
    const int dq = 16;
    p->consumers = env_int("QM_GEMV_C", 16);
    p->depth = env_int("QM_GEMV_D", 2);
    p->kc = env_int("QM_GEMV_KC", w->fmt == QM_FMT_Q8_0 ? 1 : 2);
    if (p->consumers < 1 || p->consumers > QM_GEMV_MAX_THREADS / 32 || p->depth < 1 || p->depth > 8 ||
        p->kc < 1 || p->kc > 8)
        return QM_ERR_ARG;
    const int rsq = p->kc * q + 16, rsd = p->kc * dq + 16;
    const int stage = (16 * rsq + (dq ? 16 * rsd : 0) + 127) & ~127;
    const int rings = p->consumers * p->depth * stage;
    const int fixed = 32 * 8 * 4 + 32 + p->consumers * p->depth * 8 + 128 + rings;
    const int planes = 2 * m;
    const int room = QM_GEMV_SMEM_MAX - fixed - planes * 64;
    int max_units = room / (planes * 528);
    if (max_units < 1) return QM_ERR_SHAPE;
    int ksplit = (w->units + max_units - 1) / max_units;
    ksplit = std::max(ksplit, env_int("QM_GEMV_KSPLIT", 1));
    ksplit = std::min(ksplit, (int)w->units);
    if (ksplit > sm_count) return QM_ERR_SHAPE;
    p->units_per_slice = (w->units + ksplit - 1) / ksplit;
    p->ksplit = (w->units + p->units_per_slice - 1) / p->units_per_slice;
    p->ctas_per_slice = std::max(1, env_int("QM_GEMV_CTAS", sm_count) / p->ksplit);
    p->tiles = (int)((w->rows + 15) / 16);
    const int n = p->units_per_slice;
    const int64_t Wt = std::min<int64_t>((int64_t)p->ctas_per_slice * p->consumers, (int64_t)p->tiles * n);
    p->maxseg = (int)std::min<int64_t>(n, (int64_t)(n - 1) * Wt / ((int64_t)p->tiles * n) + 2);
    p->smem = planes * (p->units_per_slice * 528 + 64) + fixed;
    if (p->tiles > QM_TICKETS) return QM_ERR_SHAPE;
    if ((int64_t)p->ksplit * p->tiles * p->maxseg * 512 > QM_PARTIALS_BYTES) return QM_ERR_SHAPE;
    return QM_OK;
}

// Bound of every device-side wait in SM clock cycles: about two seconds by default,
// QM_WAIT_LIMIT (cycles) overrides it (tests use a short bound to see a wait run out).
int64_t qm_wait_cycles() {
    const char *s = getenv("QM_WAIT_LIMIT");
    const long long v = (s && *s) ? atoll(s) : 0;
    return v > 0 ? (int64_t)v : 4000000000ll;
}

int qm_fused_grid(qm_ctx *c) { return std::max(1, env_int("QM_GEMV_CTAS", c->sm_count)); }

int32_t qm_plan_fused(qm_ctx *c, int32_t m, int32_t units, bool allow_slices, QmFusedPlan *p) {
    (void)c;
    p->nt = m <= 4 ? 1 : 2;
    p->cpm = m <= 2 ? 4 : 2;
    const int planes = m * (p->cpm == 4 ? 3 : 2);
    // ring shapes in order of preference: (warps, stages per warp)
    // (five stages fit at batch 1 once the down projection runs in parts, and measured slower: 1.13 against 1.11 ms per step)
    static const int cand[][2] = {{16, 4}, {16, 3}, {16, 2}};
    const int forced = env_int("QM_GEMV_C", 0);
    for (int slices = 1; slices <= (allow_slices ? QM_MAX_INLINE_OPS : 1); slices++) {
        const int ups = (units + slices - 1) / slices;
        for (const auto &cd : cand) {
            int C = cd[0], D = cd[1];
            if (D > env_int("QM_GEMV_DMAX", 8)) continue;
            if (forced) { C = forced; D = env_int("QM_GEMV_D", 3); }
            if (C < 1 || C > QM_GEMV_MAX_THREADS / 32 || D < 1 || D > 8) return QM_ERR_ARG;
            const int smem = planes * (ups * 256 + 64) + ups * 160 * p->nt + C * 1024 + 32 * 8 * 4 + 32 + 512 +
                             C * 2 * m * 64 + 128 + C * D * QM_Q4K_ITEM_BYTES;
            if (smem <= QM_GEMV_SMEM_MAX) {
                p->consumers = C;
                p->depth = D;
                p->smem = smem;
                p->max_units = ups;
                p->units_per_slice = ups;
                p->slices = (units + ups - 1) / ups;
                return QM_OK;
            }
            if (forced) break;
        }
    }
    return QM_ERR_SHAPE;
}

// Deals the op's items, not its tiles, to the CTAs. Only valid inside a fused list, for an op
// that is not the first, whose y is not touched by the op before it, and whose K units per
// tile do not exceed a CTA's share (so that at most two CTAs meet in a tile).
void qm_balance_op(qm_ctx *c, QmOp *op) {
    const int grid = qm_fused_grid(c);
    const int64_t I = (int64_t)op->tiles * op->units;
    if (op->accumulate || I / grid < op->units || qm_env_int("QM_NO_BALANCE", 0)) return;
    op->q = (int32_t)(I / grid);
    op->rem = (int32_t)(I % grid);
    op->balanced = 1;
}

void qm_fill_op(qm_ctx *c, const QmFusedPlan &p, const QmWeight *w, uint64_t x, uint64_t x2, int64_t ldx, uint64_t y,
                int64_t ldy, uint32_t xop, int barrier, int unit0, int units, int accumulate, QmOp *op) {
    memset(op, 0, sizeof *op);
    op->wq = (const uint8_t *)(uintptr_t)w->wq;
    op->x = (const float *)(uintptr_t)x;
    op->x2 = (const float *)(uintptr_t)x2;
    op->y = (float *)(uintptr_t)y;
    op->ldx = ldx;
    op->ldy = ldy;
    op->rows = (int32_t)w->rows;
    op->cols = (int32_t)w->cols;
    op->units = units;
    op->units_total = w->units;
    op->unit0 = unit0;
    op->accumulate = accumulate;
    op->tiles = (int32_t)((w->rows + 15) / 16);
    op->xop = (int32_t)xop;
    op->barrier = barrier;
    const int grid = qm_fused_grid(c);
    op->q = op->tiles / grid;
    op->rem = op->tiles % grid;
    op->balanced = 0;
    op->parts = op->x_parts = 1;
    op->part = 0;
    op->cta0 = 0;
    op->nctas = grid;
    (void)p;
    op->eps = 1e-6f;
}

static int32_t fused_matvec_launch(qm_ctx *c, const QmWeight *w, uint64_t x_dev, uint64_t x2_dev, int32_t m,
                                   int64_t ldx, uint64_t y_dev, int64_t ldy, uint32_t flags, const QmFusedPlan &p) {
    QmFusedArgs a;
    memset(&a, 0, sizeof a);
    for (int s = 0; s < p.slices; s++) {
        const int u0 = s * p.units_per_slice, n = std::min(p.units_per_slice, w->units - u0);
        qm_fill_op(c, p, w, x_dev, x2_dev, ldx, y_dev, ldy, flags & 0xFu, s > 0, u0, n, s > 0, &a.inl[s]);
        if ((int64_t)a.inl[s].tiles * a.inl[s].units >= (1ll << 31))
            return QM_ERR_SHAPE;
    }
    a.ops = nullptr;
    a.status = (unsigned int *)(uintptr_t)c->status_dev;
    a.grid_bar = (unsigned int *)(uintptr_t)c->gridbar_dev;
    a.nops = p.slices;
    a.m = m;
    a.consumers = p.consumers;
    a.depth = p.depth;
    a.max_units = p.max_units;
    a.cpm = p.cpm;
#ifdef QM_DEBUG
    a.debug = env_int("QM_DEBUG_SKIP", 0);
    a.debug_slot = env_int("QM_DEBUG_OP", 0);
#endif
    a.wait_cycles = qm_wait_cycles();
    // One op of up to four activation rows whose K fits whole: the lean body of the data-driven
    // kernels (an op that reads the launch's input polls nothing).
    if (p.slices == 1 && p.nt == 1 && p.consumers == 16 && p.depth >= 2 && p.depth <= 4 && env_int("QM_DD", 1) != 0) {
        const int k = (p.cpm == 4 ? QM_K_FUSED_Q4K_DD_C4D2 : QM_K_FUSED_Q4K_DD_C2D2) + (p.depth - 2);
        return qm_launch_ex(c, k, (unsigned)qm_fused_grid(c), (unsigned)p.consumers * 32, (unsigned)p.smem, &a,
                            (flags & QM_FLAG_PDL) != 0, false);
    }
    const bool coop = p.slices > 1;  // K slices meet at a grid barrier: all CTAs must be co-resident
    if (coop) DRV(c->drv->cuMemsetD32Async(c->gridbar_dev, 0, 1, c->stream));
    return qm_launch_ex(c, p.nt == 1 ? QM_K_FUSED_Q4K_NT1 : QM_K_FUSED_Q4K_NT2,
                        (unsigned)qm_fused_grid(c), (unsigned)p.consumers * 32, (unsigned)p.smem, &a,
                        (flags & QM_FLAG_PDL) != 0 && !coop, coop);
}

// Q2_K / IQ2_XXS: warp-per-row kernels over the GGUF bytes. x: float32 or (xq) Q8_1 blocks; ids_dev != 0: the
// selected form over `experts` matrices stacked by rows in w, one grid row per slot, y = [slot][rows of one expert].
int32_t qm_kq_launch(qm_ctx *c, const QmWeight *w, uint64_t x_dev, bool xq, int32_t m, int64_t ldx, uint64_t y_dev,
                     int64_t ldy, uint64_t ids_dev, int32_t experts, int32_t slots, int64_t x_slot_stride, bool pdl) {
    QmKqArgs ka;
    memset(&ka, 0, sizeof ka);
    ka.wq = (const uint8_t *)(uintptr_t)w->wq;
    ka.x = (const void *)(uintptr_t)x_dev;
    ka.y = (float *)(uintptr_t)y_dev;
    ka.ldx = ldx;
    ka.ldy = ldy;
    ka.rows = ids_dev ? w->rows / experts : w->rows;
    ka.units = w->units;
    ka.m = m;
    ka.ids = (const int32_t *)(uintptr_t)ids_dev;
    ka.experts = experts;
    ka.x_slot_stride = x_slot_stride;
    ka.y_slot_stride = ids_dev ? ka.rows : 0;
    const int mi = m <= 1 ? 0 : m <= 2 ? 1 : m <= 4 ? 2 : 3;
    const int k = (w->fmt == QM_FMT_Q2_K ? (xq ? QM_K_GEMV_Q2K_Q81_M1 : QM_K_GEMV_Q2K_M1)
                                         : (xq ? QM_K_GEMV_IQ2XXS_Q81_M1 : QM_K_GEMV_IQ2XXS_M1)) + mi;
    // eight warps per CTA, one row per warp at a time. Rows that are whole 16-byte pieces are streamed through
    // per-warp rings in shared memory (2..4 rows in flight per warp, at most 96 KB per CTA); other shapes are
    // read with direct loads.
    const int64_t row_bytes = (int64_t)w->units * (w->fmt == QM_FMT_Q2_K ? 84 : 66);
    unsigned smem = 0;
    if (row_bytes % 16 == 0 && (w->wq & 15) == 0 && qm_env_int("QM_KQ_DIRECT", 0) == 0) {
        // Q8_1 kernels also keep the activations of the CTA's slot in shared memory
        const int64_t xs = xq ? ((int64_t)m * w->units * 8 * 36 + 15) & ~(int64_t)15 : 0;
        const int64_t d = std::min<int64_t>(4, (QM_KQ_SMEM_MAX - xs) / (8 * row_bytes));
        if (d >= 2) {
            ka.depth = (int32_t)d;
            ka.xs_bytes = (int32_t)xs;
            smem = (unsigned)(xs + 8 * d * row_bytes);
        }
    }
    const int per_sm = smem ? (int)std::max<int64_t>(1, std::min<int64_t>(8, (200 * 1024) / (smem + 3072))) : 8;
    const int64_t want = (ka.rows + 7) / 8;
    const int64_t cap = std::max<int64_t>(1, (int64_t)c->sm_count * per_sm / std::max(1, slots));
    const unsigned grid = (unsigned)std::max<int64_t>(1, std::min<int64_t>(want, cap));
    return qm_launch(c, k, grid, (unsigned)std::max(1, slots), 256, smem, &ka, pdl);
}

int32_t qm_matvec_launch(qm_ctx *c, const QmWeight *w, uint64_t x_dev, uint64_t x2_dev, int32_t m, int64_t ldx,
                         uint64_t y_dev, int64_t ldy, uint32_t flags, CUdeviceptr partials, CUdeviceptr tickets) {
    if (w->fmt != QM_FMT_Q4_K && w->fmt != QM_FMT_Q4_0 && w->fmt != QM_FMT_Q8_0 && w->fmt != QM_FMT_Q2_K &&
        w->fmt != QM_FMT_IQ2_XXS)
        return QM_ERR_FORMAT;
    if (m < 1 || m > 8 || ldx < w->cols || ldy < w->rows) return QM_ERR_SHAPE;
    const uint32_t xop = flags & 0xFu;
    if (xop > QM_XOP_SWIGLU) return QM_ERR_ARG;
    if (!x_dev || !y_dev || (x_dev & 15) || (ldx & 3)) return QM_ERR_ARG;
    if ((xop == QM_XOP_ADD_RMSNORM || xop == QM_XOP_SWIGLU) && (!x2_dev || (x2_dev & 15))) return QM_ERR_ARG;
    if (w->fmt == QM_FMT_Q2_K || w->fmt == QM_FMT_IQ2_XXS) {
        // warp-per-row kernels over the GGUF bytes; plain products only (no fused input transform)
        if (xop != QM_XOP_NONE) return QM_ERR_ARG;
        return qm_kq_launch(c, w, x_dev, false, m, ldx, y_dev, ldy, 0, 0, 1, 0, (flags & QM_FLAG_PDL) != 0);
    }
    if (w->fmt == QM_FMT_Q4_K) {
        // integer tensor-core path; K is cut into slices when the activation planes of the
        // whole K do not fit in shared memory (many rows times a long K)
        QmFusedPlan fp;
        int32_t frc = qm_plan_fused(c, m, w->units, true, &fp);
        if (frc) return frc;
        return fused_matvec_launch(c, w, x_dev, x2_dev, m, ldx, y_dev, ldy, flags, fp);
    }
    if (env_int("QM_LEAN", 1) != 0) {
        // The integer tensor-core body: one persistent CTA of 16 warps per SM, whole tiles per CTA, per-warp
        // cp.async rings. A long K is cut into parts (CTA groups that each stage only their range of x and
        // leave partial vectors which a small second launch adds up); the deepest ring that fits is taken.
        // The older kernel takes what fits in no form.
        const bool q40 = w->fmt == QM_FMT_Q4_0;
        const int cpm = m <= 2 ? 4 : 2, nt = m <= 4 ? 1 : 2, planes = m * (cpm == 4 ? 3 : 2);
        const int stage = (q40 ? 2048 : 4096) + 256;
        const int grid = qm_fused_grid(c), tiles = (int)((w->rows + 15) / 16);
        const int64_t ldp = (w->rows + 3) & ~(int64_t)3;
        const int want = env_int("QM_LEAN_PARTS", w->units >= 32 ? 4 : 1);
        const int order[3] = {want, want == 4 ? 2 : want == 2 ? 4 : 2, want == 1 ? 4 : 1};
        const int depths[2] = {q40 ? 4 : 3, 2};
        for (int oi = 0; oi < 3; oi++) {
            const int S = order[oi];
            if (S < 1 || w->units % S != 0 || grid % S != 0) continue;
            if (S > 1 && (!partials || 256 + (int64_t)S * m * ldp * 4 > QM_PARTIALS_BYTES)) continue;
            const int ups = w->units / S;
            const int64_t fixed = (int64_t)planes * (ups * 256 + 64) + (int64_t)ups * nt * 160 + 512 + 16 * 2 * m * 64 + 128;
            for (int di = 0; di < 2; di++) {
                const int64_t smem = fixed + (int64_t)16 * depths[di] * stage;
                if (smem > QM_GEMV_SMEM_MAX) continue;
                QmLeanArgs la;
                memset(&la, 0, sizeof la);
                la.wq = (const uint8_t *)(uintptr_t)w->wq;
                la.wd = (const uint16_t *)(uintptr_t)w->wd;
                la.x = (const float *)(uintptr_t)x_dev;
                la.x2 = (const float *)(uintptr_t)x2_dev;
                la.ldx = ldx;
                la.rows = (int32_t)w->rows;
                la.cols = (int32_t)w->cols;
                la.units = ups;
                la.units_total = w->units;
                la.m = m;
                la.xop = (int32_t)xop;
                la.eps = 1e-6f;
                la.parts = S;
                const int G = grid / S;
                la.q = tiles / G;
                la.rem = tiles % G;
                const bool norm = xop == QM_XOP_RMSNORM || xop == QM_XOP_ADD_RMSNORM;
                if (S == 1) {
                    la.y = (float *)(uintptr_t)y_dev;
                    la.ldy = ldy;
                } else {
                    la.ssq = (float *)(uintptr_t)partials;
                    la.y = (float *)(uintptr_t)(partials + 256);
                    la.ldy = ldp;
                    la.part_stride = (int64_t)m * ldp;
                }
                const int k = (q40 ? QM_K_Q40_LEAN_C4D4 : QM_K_Q80_LEAN_C4D3) + (cpm == 4 ? 0 : nt == 1 ? 2 : 4) + di;
                const bool pdl = (flags & QM_FLAG_PDL) != 0;
                int32_t lrc = qm_launch_ex(c, k, (unsigned)grid, 512, (unsigned)smem, &la, pdl, false);
                if (lrc || S == 1) return lrc;
                QmSumPartsArgs sa;
                memset(&sa, 0, sizeof sa);
                sa.parts = la.y;
                sa.ssq = norm ? la.ssq : nullptr;
                sa.out = (float *)(uintptr_t)y_dev;
                sa.part_stride = la.part_stride;
                sa.ld_in = ldp;
                sa.ld_out = ldy;
                sa.nparts = S;
                sa.m = m;
                sa.n = (int32_t)w->rows;
                sa.inv_cols = 1.f / (float)w->cols;
                sa.eps = 1e-6f;
                const unsigned sgrid = (unsigned)std::max<int64_t>(1, std::min<int64_t>(((int64_t)m * w->rows + 255) / 256, c->sm_count));
                return qm_launch(c, QM_K_LEAN_SUM, sgrid, 1, 256, 0, &sa, true);
            }
        }
    }
    QmGemvPlan p;
    int32_t rc = qm_plan_gemv(c, w, m, &p);
    if (rc) return rc;
    QmGemvArgs a;
    memset(&a, 0, sizeof a);
    a.wq = (const uint8_t *)(uintptr_t)w->wq;
    a.wd = (const uint16_t *)(uintptr_t)w->wd;
    a.x = (const float *)(uintptr_t)x_dev;
    a.x2 = (const float *)(uintptr_t)x2_dev;
    a.y = (float *)(uintptr_t)y_dev;
    a.partials = (float *)(uintptr_t)partials;
    a.tickets = (unsigned int *)(uintptr_t)tickets;
    a.status = (unsigned int *)(uintptr_t)c->status_dev;
    a.ldx = ldx;
    a.ldy = ldy;
    a.rows = (int32_t)w->rows;
    a.cols = (int32_t)w->cols;
    a.units = w->units;
    a.m = m;
    a.tiles = p.tiles;
    a.ksplit = p.ksplit;
    a.units_per_slice = p.units_per_slice;
    a.ctas_per_slice = p.ctas_per_slice;
    a.consumers = p.consumers;
    a.depth = p.depth;
    a.kc = p.kc;
    a.maxseg = p.maxseg;
    a.xop = (int32_t)xop;
    a.eps = 1e-6f;
    const int mode = m <= 4 ? 0 : 1;
    const int k = (w->fmt == QM_FMT_Q4_0 ? QM_K_GEMV_Q40_M4 : QM_K_GEMV_Q80_M4) + mode;
    return qm_launch(c, k, (unsigned)(p.ksplit * p.ctas_per_slice), 1, (unsigned)p.consumers * 32, (unsigned)p.smem,
                     &a, (flags & QM_FLAG_PDL) != 0);
}

extern "C" int32_t qm_matvec(qm_ctx *c, qm_weight h, uint64_t x_dev, uint64_t x2_dev, int32_t m, int64_t ldx,
                             uint64_t y_dev, int64_t ldy, uint32_t flags) {
    CHECK_CTX(c);
    QmWeight *w = qm_weight_from_handle(h);
    if (!w) return QM_ERR_ARG;
    CtxGuard g(c);
    DRV(g.rc);
    return qm_matvec_launch(c, w, x_dev, x2_dev, m, ldx, y_dev, ldy, flags, c->partials_dev, c->tickets_dev);
}

extern "C" int32_t qm_matvec_host(qm_ctx *c, qm_weight h, const float *x_host, int32_t m, int64_t ldx,
                                  float *y_host, int64_t ldy, uint32_t flags) {
    CHECK_CTX(c);
    QmWeight *w = qm_weight_from_handle(h);
    if (!w || !x_host || !y_host) return QM_ERR_ARG;
    if (m < 1 || m > 8 || ldx < w->cols || ldy < w->rows) return QM_ERR_SHAPE;
    if ((flags & 0xFu) > QM_XOP_RMSNORM) return QM_ERR_ARG;  // two-operand transforms need device buffers
    CtxGuard g(c);
    DRV(g.rc);
    // device staging: x as [m][cols4] and y as [m][rows], reused across calls
    const int64_t cols4 = (w->cols + 3) & ~(int64_t)3;
    const int64_t need = (m * cols4 + m * w->rows) * 4 + 256;
    if (need > c->xstage_bytes) {
        DRV(c->drv->cuStreamSynchronize(c->stream));
        if (c->xstage_dev) DRV(c->drv->cuMemFree_v2(c->xstage_dev));
        c->xstage_dev = 0;
        c->xstage_bytes = 0;
        DRV(c->drv->cuMemAlloc_v2(&c->xstage_dev, (size_t)need * 2));
        c->xstage_bytes = need * 2;
    }
    const CUdeviceptr xd = c->xstage_dev;
    const CUdeviceptr yd = c->xstage_dev + (((m * cols4 * 4) + 255) & ~(int64_t)255);
    for (int j = 0; j < m; j++)
        DRV(c->drv->cuMemcpyHtoDAsync_v2(xd + j * cols4 * 4, x_host + j * ldx, (size_t)w->cols * 4, c->stream));
    int32_t rc = qm_matvec_launch(c, w, xd, 0, m, cols4, yd, w->rows, flags, c->partials_dev, c->tickets_dev);
    if (rc) return rc;
    for (int j = 0; j < m; j++)
        DRV(c->drv->cuMemcpyDtoHAsync_v2(y_host + j * ldy, yd + j * w->rows * 4, (size_t)w->rows * 4, c->stream));
    DRV(c->drv->cuStreamSynchronize(c->stream));
    return QM_OK;
}

// ---- prefill matmul (tcgen05) ----------------------------------------------------------------
// One launch of the tcgen05 matmul. Single matrix: g.experts == 0, weights w, activations
// a_dev [m][lda]. Grouped over experts (g.experts > 0): blockIdx.z = expert, its activation rows
// are [offsets[e], offsets[e+1]) of a_dev [rows_total][lda], its weights wq_list[e] (all experts
// shaped like w); m = the longest expert list (sizes the grid). With g.swiglu the weights are
// gate|up matrices [2*ffn][k] and the launch stores bf16 silu(gate)*up to g.h instead of C.
int32_t qm_gemm_launch(qm_ctx *c, const QmWeight *w, uint64_t a_dev, int32_t m, int64_t rows_total, int64_t lda,
                       uint64_t c_dev, int64_t ldc, const QmGemmGroup &g) {
    QmGemmArgs a;
    memset(&a, 0, sizeof a);
    const bool grouped = g.experts > 0;
    // Tile shapes: 128 weight rows x 64..512 tokens per CTA (four stages, two at 512 tokens). A
    // 256-row variant (two accumulators, three or four stages) serves the fused SwiGLU epilogue
    // (gate rows in one accumulator, the matching up rows in the other); for plain matmuls it is
    // kept behind QM_GEMM_R256=1: measured equal within noise (76.6 us against 74.0 us at
    // 4096 x 4096 x 2048), so neither the stage count nor the activation traffic is the limit.
    const int mt = g.m_typical > 0 ? g.m_typical : m;
    // ... and the grouped down launch where 128-row tiles would not fit one wave of the SMs (eight experts
    // of 4096 rows: 256 tiles are 1.73 waves, 128 tiles of 256 rows are one; MoE layer 0.647 -> 0.612 ms)
    const bool r256_wave = grouped && !g.swiglu && mt <= 256 && w->rows >= 256 &&
                           ((w->rows + 127) / 128) * (int64_t)g.experts > c->sm_count;
    const bool r256 = g.swiglu || (env_int("QM_GEMM_R256", r256_wave ? 1 : 0) != 0 && w->rows >= 256);
    const int nsub = r256 ? 2 : 1;
    // (192: a grouped launch whose longest list fits gets a smaller activation tile and with it a fourth stage)
    const int bn_auto = mt <= 64 ? 64 : mt <= 128 ? 128 : (grouped && mt <= 192) ? 192 : (mt <= 256 || r256) ? 256 : 512;
    const int bn = std::min(bn_auto, std::max(64, env_int("QM_GEMM_BN", 512)));
    // Two 64-column chunks per stage where at least two such stages fit and the token tile is
    // small: the handshake of a stage costs ~0.3 us, more than the MMAs of one small chunk.
    const int chunk_bytes = nsub * 128 * 64 * 2 + bn * 64 * 2;
    const int ks = env_int("QM_GEMM_KS", (bn <= 256 && (QM_GEMV_SMEM_MAX - 2048) / (2 * chunk_bytes) >= 2) ? 2 : 1) == 2 ? 2 : 1;
    const int stage_bytes = ks * chunk_bytes;
    const int stages = std::max(2, std::min(8, (QM_GEMV_SMEM_MAX - 2048) / stage_bytes));
    if (stages * stage_bytes + 2048 > QM_GEMV_SMEM_MAX) return QM_ERR_SHAPE;
    const cuuint64_t dims[2] = {(cuuint64_t)w->cols, (cuuint64_t)rows_total};
    const cuuint64_t strides[1] = {(cuuint64_t)lda * 2};
    // grouped launches fetch the token tile in boxes of 64 rows, as many as the expert's list fills
    const int box_rows = grouped ? 64 : std::min(bn, 256);
    const cuuint32_t box[2] = {64, (cuuint32_t)box_rows};
    const cuuint32_t estr[2] = {1, 1};
    DRV(c->drv->cuTensorMapEncodeTiled(&a.tmap_act, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (void *)(uintptr_t)a_dev, dims,
                                       strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                       CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE));
    const int64_t out_cols = g.swiglu ? w->rows / 2 : w->rows;   // columns of the output matrix
    a.wq = (const uint8_t *)(uintptr_t)w->wq;
    a.c = (float *)(uintptr_t)c_dev;
    a.status = (unsigned int *)(uintptr_t)c->status_dev;
    a.ldc = ldc;
    a.m = m;
    a.n = (int32_t)out_cols;
    a.units = w->units;
    a.tiles16 = (int32_t)((w->rows + 15) / 16);
    a.bn = bn;
    a.stages = stages;
    a.box_rows = box_rows;
    a.groups = env_int("QM_GEMM_GROUPS", 4) == 2 ? 2 : 4;
    a.grouped = grouped ? 1 : 0;
    a.wq_list = (const uint8_t *const *)(uintptr_t)g.wq_list_dev;
    a.offsets = (const int32_t *)(uintptr_t)g.offsets_dev;
    a.swiglu = g.swiglu ? 1 : 0;
    a.up_offset = (int32_t)(w->rows / 2);
    a.h = (uint16_t *)(uintptr_t)g.h_dev;
    a.ldh = g.ldh;
#ifdef QM_DEBUG
    a.debug = env_int("QM_GEMM_DEBUG", 0);
#endif
    unsigned smem = 1024 + stages * stage_bytes + 512;   // alignment slack, stages, barriers
    if (g.gather_list_dev) {   // the loader warp's table of token numbers sits behind the barriers
        if (!grouped || bn > 256 || g.gather_topk < 1) return QM_ERR_SHAPE;
        a.gather_list = (const int32_t *)(uintptr_t)g.gather_list_dev;
        a.gather_topk = g.gather_topk;
        const cuuint32_t row_box[2] = {64, 1};   // tile::gather4 names the four rows itself
        DRV(c->drv->cuTensorMapEncodeTiled(&a.tmap_gather, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (void *)(uintptr_t)a_dev,
                                           dims, strides, row_box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                                           CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                                           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE));
        smem += 1024;
        if (smem > QM_GEMV_SMEM_MAX) return QM_ERR_SHAPE;
    }
    void *params[1] = {&a};
    CUlaunchConfig cfg;
    memset(&cfg, 0, sizeof cfg);
    const int rows_per_cta = g.swiglu ? 128 : 128 * nsub;
    cfg.gridDimX = (unsigned)((out_cols + rows_per_cta - 1) / rows_per_cta);
    cfg.gridDimY = (unsigned)((m + bn - 1) / bn);
    // few tokens: split K over CTAs until the SMs are covered; the last CTA of a tile adds the shares in a
    // fixed order (no atomics on C: the same bits every run)
    int splitk = 1;
    // (grouped launches too, where the experts' tiles leave SMs idle — few experts per GPU in expert-parallel
    // runs; not with the SwiGLU epilogue, whose launches have row tiles enough)
    const int64_t tiles = (int64_t)cfg.gridDimX * cfg.gridDimY * (grouped ? g.experts : 1);
    const int64_t plane_rows = grouped ? rows_total : m;
    if (!g.swiglu) {
        while (splitk < 8 && tiles * splitk * 2 <= c->sm_count && w->units * 4 / (splitk * 2) >= 8) splitk *= 2;
        if (!grouped) splitk = env_int("QM_GEMM_SPLITK", splitk);
        else if (env_int("QM_GEMM_GROUPED_SPLITK", 1) == 0) splitk = 1;
    }
    // the shares go through the context's scratch (one plane of rows x n floats per share) and a ticket per tile
    while (splitk > 1 && ((int64_t)splitk * plane_rows * out_cols * 4 > QM_PARTIALS_BYTES || tiles * 2 > QM_TICKETS))
        splitk /= 2;
    a.splitk = splitk;
    a.plane_rows = (int32_t)plane_rows;
    a.partials = (float *)(uintptr_t)c->partials_dev;
    a.tickets = (unsigned int *)(uintptr_t)c->tickets_dev;
    a.wait_cycles = qm_wait_cycles();
    cfg.gridDimZ = (unsigned)splitk;
    if (grouped) {   // expert in y, token tile and K share in z (see the kernel)
        cfg.gridDimZ = cfg.gridDimY * (unsigned)splitk;
        cfg.gridDimY = (unsigned)g.experts;
    }
    cfg.blockDimX = 576;   // TMA warp, MMA warp, sixteen dequantizing warps
    cfg.blockDimY = cfg.blockDimZ = 1;
    cfg.sharedMemBytes = smem;
    cfg.hStream = c->stream;
    const int kern = ks == 2 ? (r256 ? QM_K_GEMM_Q4K_R256_K128 : QM_K_GEMM_Q4K_K128) : (r256 ? QM_K_GEMM_Q4K_R256 : QM_K_GEMM_Q4K);
    CUlaunchAttribute coop;
    if (splitk > 1) {   // the CTAs of a tile wait for one another before they add the shares: all must be resident
        coop.id = CU_LAUNCH_ATTRIBUTE_COOPERATIVE;
        coop.value.cooperative = 1;
        cfg.attrs = &coop;
        cfg.numAttrs = 1;
    }
    DRV(c->drv->cuLaunchKernelEx(&cfg, c->fn[kern], params, nullptr));
    c->launches++;
    return QM_OK;
}

extern "C" int32_t qm_matmul_bf16(qm_ctx *c, qm_weight h, uint64_t a_dev, int32_t m, int64_t lda, uint64_t c_dev,
                                  int64_t ldc) {
    CHECK_CTX(c);
    QmWeight *w = qm_weight_from_handle(h);
    if (!w || !a_dev || !c_dev) return QM_ERR_ARG;
    if (w->fmt != QM_FMT_Q4_K) return QM_ERR_FORMAT;
    if (m < 1 || m > (1 << 20) || lda < w->cols || ldc < w->rows) return QM_ERR_SHAPE;
    // TMA: base 16-byte aligned, row pitch a multiple of 16 bytes
    if ((a_dev & 15) || ((lda * 2) & 15)) return QM_ERR_ARG;
    CtxGuard g(c);
    DRV(g.rc);
    QmGemmGroup none;
    memset(&none, 0, sizeof none);
    return qm_gemm_launch(c, w, a_dev, m, m, lda, c_dev, ldc, none);
}
