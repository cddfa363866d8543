// qm_noalloc.cu — qm_matvec_noalloc: the Q4_0 / Q8_0 matvec for callers that must not
// allocate device memory.
//
// Who needs it: code that runs where cudaMalloc is off limits — inside a region whose memory
// budget was fixed up front (an inference server that handed every spare byte to its KV
// cache), inside a latency-critical loop where an allocation would synchronize the device,
// or under a host framework that owns the allocator and forbids side allocations by
// libraries it calls. qm_matvec keeps its split-K scratch (per-slice partial sums and arrival
// tickets) in buffers that qm_init allocates; this entry point keeps the same scratch in a
// fixed array that is part of the library image instead, so no call here ever allocates.
//
// Cost and limits: every GPU that loads the library holds QM_NOALLOC_SCRATCH_BYTES
// (4 MiB) of device memory for that array until the process exits. A matvec whose partial
// sums and tickets would not fit is refused with QM_ERR_LIMIT; nothing falls back to an
// allocation. All calls on one device share the one array and it keeps whatever the last call
// left, so each call clears the tickets and the status word it starts from, and two calls
// whose kernels overlap on the GPU (different streams, no ordering) race on it — order them.
//
// Set-up: the first call on a device resolves the array's device address
// (cudaGetSymbolAddress) and raises the kernels' shared-memory limit. Make that first call
// outside any stream capture.
#include <cuda_runtime.h>

#include <algorithm>
#include <mutex>

#include "qm_internal.h"

// the kernels themselves: the same source as the cubin the driver-API path loads
#include "qm_gemv.cu"

#define QM_NOALLOC_SCRATCH_BYTES (4 << 20)
#define QM_NOALLOC_MAX_DEVICES 64

// In host code this name is only a stand-in for the device array: its device address comes
// from cudaGetSymbolAddress, never from taking the address of the name.
static __device__ __align__(256) unsigned char qm_noalloc_scratch[QM_NOALLOC_SCRATCH_BYTES];

namespace {

struct DeviceSetup {
    unsigned char *scratch;  // device address of qm_noalloc_scratch on this device
    int sm_count;
};
DeviceSetup g_setup[QM_NOALLOC_MAX_DEVICES];
std::mutex g_setup_mutex;

// Once per device, with that device current.
int32_t setup_device(int dev, DeviceSetup **out) {
    if (dev < 0 || dev >= QM_NOALLOC_MAX_DEVICES) return QM_ERR_ARG;
    std::lock_guard<std::mutex> lock(g_setup_mutex);
    DeviceSetup &s = g_setup[dev];
    if (!s.scratch) {
        void *ptr = nullptr;
        cudaError_t e = cudaGetSymbolAddress(&ptr, qm_noalloc_scratch);
        if (e != cudaSuccess || !ptr) return e != cudaSuccess ? (int32_t)e : QM_ERR_STATE;
        int sms = 0;
        e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        if (e != cudaSuccess) return (int32_t)e;
        const void *kernels[4] = {(const void *)qm_gemv_q40_m4, (const void *)qm_gemv_q40_m8,
                                  (const void *)qm_gemv_q80_m4, (const void *)qm_gemv_q80_m8};
        for (const void *k : kernels) {
            e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, QM_GEMV_SMEM_MAX);
            if (e != cudaSuccess) return (int32_t)e;
        }
        s.sm_count = sms;
        s.scratch = static_cast<unsigned char *>(ptr);
    }
    *out = &s;
    return QM_OK;
}

}  // namespace

// y[j][r] = sum_c x[j][c] * W[r][c], j < m <= 8, for a stored Q4_0 or Q8_0 matrix; x and y are
// float32 device pointers in the current device's primary context, the launch goes to
// `cu_stream` (0 = the default stream) and the call returns without waiting for it. The current
// device must be the one that holds the weights (QM_ERR_ARG otherwise).
extern "C" __attribute__((visibility("default"))) int32_t qm_matvec_noalloc(qm_weight h, uint64_t x_dev, int32_t m,
                                                                              int64_t ldx, uint64_t y_dev,
                                                                              int64_t ldy, uint64_t cu_stream) {
    const QmWeight *w = qm_weight_from_handle(h);
    if (!w || !x_dev || !y_dev || (x_dev & 15) || (ldx & 3)) return QM_ERR_ARG;
    if (w->fmt != QM_FMT_Q4_0 && w->fmt != QM_FMT_Q8_0) return QM_ERR_FORMAT;
    if (m < 1 || m > 8 || ldx < w->cols || ldy < w->rows) return QM_ERR_SHAPE;
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int32_t)e;
    if (dev != w->device) return QM_ERR_ARG;   // the weights live on another GPU than the current one
    DeviceSetup *ds = nullptr;
    int32_t rc = setup_device(dev, &ds);
    if (rc) return rc;

    // the launch shape is the one qm_matvec uses (same planner)
    QmGemvPlan p;
    rc = qm_plan_gemv_sms(ds->sm_count, w, m, &p);
    if (rc) return rc == QM_ERR_SHAPE ? QM_ERR_LIMIT : rc;
    const int tiles = p.tiles, ksplit = p.ksplit, maxseg = p.maxseg, smem = p.smem;

    // scratch layout: [status 256 B][tickets: tiles x 4 B, rounded to 256][partial sums]
    const size_t tickets_bytes = ((size_t)tiles * 4 + 255) & ~(size_t)255;
    const size_t partial_bytes = (size_t)ksplit * tiles * maxseg * 512;
    if (256 + tickets_bytes + partial_bytes > QM_NOALLOC_SCRATCH_BYTES)
        return QM_ERR_LIMIT;  // this matrix needs more scratch than the fixed array holds
    cudaStream_t stream = (cudaStream_t)(uintptr_t)cu_stream;
    // the array keeps the previous call's contents: the status word and the tickets start at zero
    e = cudaMemsetAsync(ds->scratch, 0, 256 + tickets_bytes, stream);
    if (e != cudaSuccess) return (int32_t)e;

    QmGemvArgs a;
    memset(&a, 0, sizeof a);
    a.wq = (const uint8_t *)(uintptr_t)w->wq;
    a.wd = (const uint16_t *)(uintptr_t)w->wd;
    a.x = (const float *)(uintptr_t)x_dev;
    a.y = (float *)(uintptr_t)y_dev;
    a.status = reinterpret_cast<unsigned int *>(ds->scratch);
    a.tickets = reinterpret_cast<unsigned int *>(ds->scratch + 256);
    a.partials = reinterpret_cast<float *>(ds->scratch + 256 + tickets_bytes);
    a.ldx = ldx;
    a.ldy = ldy;
    a.rows = (int32_t)w->rows;
    a.cols = (int32_t)w->cols;
    a.units = w->units;
    a.m = m;
    a.tiles = tiles;
    a.ksplit = ksplit;
    a.units_per_slice = p.units_per_slice;
    a.ctas_per_slice = p.ctas_per_slice;
    a.consumers = p.consumers;
    a.depth = p.depth;
    a.kc = p.kc;
    a.maxseg = maxseg;
    a.xop = 0;
    a.eps = 1e-6f;
    const dim3 grid((unsigned)(ksplit * p.ctas_per_slice)), block((unsigned)p.consumers * 32);
    if (w->fmt == QM_FMT_Q4_0) {
        if (m <= 4) qm_gemv_q40_m4<<<grid, block, smem, stream>>>(a);
        else qm_gemv_q40_m8<<<grid, block, smem, stream>>>(a);
    } else {
        if (m <= 4) qm_gemv_q80_m4<<<grid, block, smem, stream>>>(a);
        else qm_gemv_q80_m8<<<grid, block, smem, stream>>>(a);
    }
    e = cudaGetLastError();
    return e == cudaSuccess ? QM_OK : (int32_t)e;
}

// The status word of the most recent qm_matvec_noalloc on the current device (0 = clean,
// QM_STATUS_TIMEOUT = a bounded wait inside the kernel ran out and y is incomplete). The word
// lives in the fixed array, so reading it allocates nothing: a 4-byte copy that waits for the
// device. Call it after the stream of the matvec has been synchronized, and before the next
// qm_matvec_noalloc on this device, which clears the word. Returns QM_ERR_TIMEOUT when the
// timeout bit is set.
extern "C" __attribute__((visibility("default"))) int32_t qm_noalloc_status(uint32_t *status) {
    if (!status) return QM_ERR_ARG;
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int32_t)e;
    DeviceSetup *ds = nullptr;
    int32_t rc = setup_device(dev, &ds);
    if (rc) return rc;
    e = cudaMemcpy(status, ds->scratch, 4, cudaMemcpyDeviceToHost);
    if (e != cudaSuccess) return (int32_t)e;
    return (*status & QM_STATUS_TIMEOUT) ? QM_ERR_TIMEOUT : QM_OK;
}
