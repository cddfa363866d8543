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
// `cu_stream` (0 = the default stream) and the call returns without waiting for it.
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
    DeviceSetup *ds = nullptr;
    int32_t rc = setup_device(dev, &ds);
    if (rc) return rc;

    // launch shape: 16 warps per CTA, one CTA per SM, K cut into slices until the activation
    // planes of a slice fit in shared memory next to the copy rings
    const int C = 16, D = 2, KC = w->fmt == QM_FMT_Q8_0 ? 1 : 2;
    const int q = w->fmt == QM_FMT_Q4_0 ? 128 : 256;
    const int stage = (16 * (KC * q + 16) + 16 * (KC * 16 + 16) + 127) & ~127;
    const int fixed = 32 * 8 * 4 + 32 + C * D * 8 + 128 + C * D * stage;
    const int planes = 2 * m;
    const int max_units = (QM_GEMV_SMEM_MAX - fixed - planes * 64) / (planes * 528);
    if (max_units < 1) return QM_ERR_LIMIT;
    int ksplit = std::min((int)w->units, (w->units + max_units - 1) / max_units);
    if (ksplit > ds->sm_count) return QM_ERR_LIMIT;
    const int ups = (w->units + ksplit - 1) / ksplit;
    ksplit = (w->units + ups - 1) / ups;
    const int ctas = std::max(1, ds->sm_count / ksplit);
    const int tiles = (int)((w->rows + 15) / 16);
    const int64_t Wt = std::min<int64_t>((int64_t)ctas * C, (int64_t)tiles * ups);
    const int maxseg = (int)std::min<int64_t>(ups, (int64_t)(ups - 1) * Wt / ((int64_t)tiles * ups) + 2);
    const int smem = planes * (ups * 528 + 64) + fixed;

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
    a.units_per_slice = ups;
    a.ctas_per_slice = ctas;
    a.consumers = C;
    a.depth = D;
    a.kc = KC;
    a.maxseg = maxseg;
    a.xop = 0;
    a.eps = 1e-6f;
    const dim3 grid((unsigned)(ksplit * ctas)), block((unsigned)C * 32);
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
