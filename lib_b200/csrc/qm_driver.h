// Lazy binding of the CUDA driver API: dlopen("libcuda.so.1") + dlsym per
// symbol on first use, the way the reference binds it without cgo
// (nvidia/driver/loader_unix.gen.go:8-14, init.gen.go:185-199). Nothing here
// needs a GPU until qm_init runs, so the library loads on a machine without one.
#pragma once
#include <cuda.h>

#define QM_DRV_FUNCS(X)                                                                           \
    X(cuInit, CUresult (*)(unsigned int))                                                         \
    X(cuDeviceGet, CUresult (*)(CUdevice *, int))                                                 \
    X(cuDeviceGetAttribute, CUresult (*)(int *, CUdevice_attribute, CUdevice))                    \
    X(cuDevicePrimaryCtxRetain, CUresult (*)(CUcontext *, CUdevice))                              \
    X(cuDevicePrimaryCtxRelease_v2, CUresult (*)(CUdevice))                                       \
    X(cuCtxPushCurrent_v2, CUresult (*)(CUcontext))                                               \
    X(cuCtxPopCurrent_v2, CUresult (*)(CUcontext *))                                              \
    X(cuModuleLoadData, CUresult (*)(CUmodule *, const void *))                                   \
    X(cuModuleUnload, CUresult (*)(CUmodule))                                                     \
    X(cuModuleGetFunction, CUresult (*)(CUfunction *, CUmodule, const char *))                    \
    X(cuFuncSetAttribute, CUresult (*)(CUfunction, CUfunction_attribute, int))                    \
    X(cuLaunchKernel, CUresult (*)(CUfunction, unsigned, unsigned, unsigned, unsigned, unsigned,  \
                                   unsigned, unsigned, CUstream, void **, void **))               \
    X(cuLaunchKernelEx, CUresult (*)(const CUlaunchConfig *, CUfunction, void **, void **))       \
    X(cuMemAlloc_v2, CUresult (*)(CUdeviceptr *, size_t))                                         \
    X(cuMemFree_v2, CUresult (*)(CUdeviceptr))                                                    \
    X(cuMemHostAlloc, CUresult (*)(void **, size_t, unsigned int))                                \
    X(cuMemFreeHost, CUresult (*)(void *))                                                        \
    X(cuMemcpyHtoD_v2, CUresult (*)(CUdeviceptr, const void *, size_t))                           \
    X(cuMemcpyDtoH_v2, CUresult (*)(void *, CUdeviceptr, size_t))                                 \
    X(cuMemcpyHtoDAsync_v2, CUresult (*)(CUdeviceptr, const void *, size_t, CUstream))            \
    X(cuMemcpyDtoHAsync_v2, CUresult (*)(void *, CUdeviceptr, size_t, CUstream))                  \
    X(cuMemcpy2DAsync_v2, CUresult (*)(const CUDA_MEMCPY2D *, CUstream))                          \
    X(cuMemcpyDtoDAsync_v2, CUresult (*)(CUdeviceptr, CUdeviceptr, size_t, CUstream))             \
    X(cuMemsetD8Async, CUresult (*)(CUdeviceptr, unsigned char, size_t, CUstream))                \
    X(cuMemsetD32Async, CUresult (*)(CUdeviceptr, unsigned int, size_t, CUstream))                \
    X(cuMemsetD2D32Async, CUresult (*)(CUdeviceptr, size_t, unsigned int, size_t, size_t, CUstream)) \
    X(cuStreamCreate, CUresult (*)(CUstream *, unsigned int))                                     \
    X(cuStreamDestroy_v2, CUresult (*)(CUstream))                                                 \
    X(cuStreamSynchronize, CUresult (*)(CUstream))                                                \
    X(cuStreamBeginCapture_v2, CUresult (*)(CUstream, CUstreamCaptureMode))                       \
    X(cuStreamEndCapture, CUresult (*)(CUstream, CUgraph *))                                      \
    X(cuGraphInstantiateWithFlags, CUresult (*)(CUgraphExec *, CUgraph, unsigned long long))      \
    X(cuGraphLaunch, CUresult (*)(CUgraphExec, CUstream))                                         \
    X(cuGraphExecDestroy, CUresult (*)(CUgraphExec))                                              \
    X(cuGraphDestroy, CUresult (*)(CUgraph))                                                      \
    X(cuEventCreate, CUresult (*)(CUevent *, unsigned int))                                       \
    X(cuEventRecord, CUresult (*)(CUevent, CUstream))                                             \
    X(cuEventSynchronize, CUresult (*)(CUevent))                                                  \
    X(cuEventElapsedTime, CUresult (*)(float *, CUevent, CUevent))                                \
    X(cuEventDestroy_v2, CUresult (*)(CUevent))                                                   \
    X(cuGetErrorString, CUresult (*)(CUresult, const char **))                                    \
    X(cuIpcGetMemHandle, CUresult (*)(CUipcMemHandle *, CUdeviceptr))                             \
    X(cuIpcOpenMemHandle_v2, CUresult (*)(CUdeviceptr *, CUipcMemHandle, unsigned int))           \
    X(cuIpcCloseMemHandle, CUresult (*)(CUdeviceptr))                                             \
    X(cuPointerGetAttribute, CUresult (*)(void *, CUpointer_attribute, CUdeviceptr))              \
    X(cuDeviceGetP2PAttribute, CUresult (*)(int *, CUdevice_P2PAttribute, CUdevice, CUdevice))    \
    X(cuTensorMapEncodeTiled,                                                                     \
      CUresult (*)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,    \
                   const cuuint64_t *, const cuuint32_t *, const cuuint32_t *,                    \
                   CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,             \
                   CUtensorMapFloatOOBfill))

template <class T> using qm_fnptr = T;

struct QmDriver {
#define X(name, ...) qm_fnptr<__VA_ARGS__> name;
    QM_DRV_FUNCS(X)
#undef X
    bool loaded;
};

// Returns 0 or QM_ERR_NO_DRIVER. Thread-safe, idempotent.
int qm_driver_load(QmDriver **out);
