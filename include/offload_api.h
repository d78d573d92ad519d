/* Offload C-ABI of the HC GPU runtime, as exported by this build's
 * libhc-cuda-runtime.so (the CUDA driver-API backend) and by
 * libhc-gpu-runtime-loader.so (the backend-agnostic shim).
 *
 * The thirteen ol* entry points keep the reference ABI bit for bit
 * (reference: gpu-runtime/common/include/offload_api.h:9-63).  Every function
 * returns nullptr or a nonzero int on failure and reports the reason through
 * the OlErrorCallback given to olCreateDevice (reference:
 * gpu-runtime/common/include/offload_api.h:30-32).
 *
 * The olx* entry points at the end are additions of this build.  The loader
 * forwards them when the backend exports them; a backend without them still
 * loads.
 */
#pragma once

#include <stddef.h>

#ifdef __cplusplus
#define HC_NOEXCEPT noexcept
#else
#define HC_NOEXCEPT
#endif

#ifndef OFFLOAD_API_EXPORT
#define OFFLOAD_API_EXPORT __attribute__((visibility("default")))
#endif

typedef void *OlDevice; /* reference: offload_api.h:9  */
typedef void *OlModule; /* reference: offload_api.h:10 */
typedef void *OlKernel; /* reference: offload_api.h:11 */
typedef void *OlQueue;  /* reference: offload_api.h:12 */

/* reference: offload_api.h:14-18 (an `enum class : int` there; same values). */
#ifdef __cplusplus
enum class OlSeverity : int { Error = 0, Warning = 1, Message = 2 };
#else
typedef int OlSeverity;
enum { OlSeverityError = 0, OlSeverityWarning = 1, OlSeverityMessage = 2 };
#endif

/* reference: offload_api.h:20 */
typedef void (*OlErrorCallback)(void *ctx, OlSeverity sev, const char *desc);

#ifdef __cplusplus
extern "C" {
#endif

/* Backend and device id are encoded in `desc` ("cuda:<ordinal>").
 * reference: offload_api.h:33-35, gpu-runtime/cuda-runtime/src/Runtime.cpp:122-148 */
OFFLOAD_API_EXPORT OlDevice olCreateDevice(const char *desc,
                                           OlErrorCallback errCallback,
                                           void *ctx) HC_NOEXCEPT;
/* reference: offload_api.h:36, Runtime.cpp:149-151 */
OFFLOAD_API_EXPORT void olReleaseDevice(OlDevice dev) HC_NOEXCEPT;

/* Creates a GPU module from a binary blob; here the blob is a precompiled
 * sm_100a cubin (or fatbin / PTX text, anything cuModuleLoadData accepts).
 * reference: offload_api.h:39-40, Runtime.cpp:153-167 */
OFFLOAD_API_EXPORT OlModule olCreateModule(OlDevice dev, const void *data,
                                           size_t len) HC_NOEXCEPT;
/* reference: offload_api.h:41, Runtime.cpp:168-170 */
OFFLOAD_API_EXPORT void olReleaseModule(OlModule mod) HC_NOEXCEPT;

/* reference: offload_api.h:43-44, Runtime.cpp:172-180 */
OFFLOAD_API_EXPORT OlKernel olGetKernel(OlModule mod,
                                        const char *name) HC_NOEXCEPT;
/* reference: offload_api.h:45, Runtime.cpp:182-184 */
OFFLOAD_API_EXPORT void olReleaseKernel(OlKernel k) HC_NOEXCEPT;

/* Greedy per-dimension block shape with at most 1024 threads in total.
 * reference: offload_api.h:47-50, Runtime.cpp:186-216 */
OFFLOAD_API_EXPORT int olSuggestBlockSize(OlKernel k,
                                          const size_t *globalsSizes,
                                          size_t *blockSizesRet,
                                          size_t nDims) HC_NOEXCEPT;

/* reference: offload_api.h:52-54, Runtime.cpp:218-240 */
OFFLOAD_API_EXPORT OlQueue olCreateQueue(OlDevice dev) HC_NOEXCEPT;
OFFLOAD_API_EXPORT void olReleaseQueue(OlQueue q) HC_NOEXCEPT;
OFFLOAD_API_EXPORT int olSyncQueue(OlQueue q) HC_NOEXCEPT;

/* reference: offload_api.h:56-58, Runtime.cpp:242-262 */
OFFLOAD_API_EXPORT void *olAllocDevice(OlQueue q, size_t size,
                                       size_t align) HC_NOEXCEPT;
OFFLOAD_API_EXPORT void olDeallocDevice(OlQueue q, void *data) HC_NOEXCEPT;

/* nDims must be 3; args[i] points at the i-th kernel parameter.
 * reference: offload_api.h:60-64, Runtime.cpp:264-281 */
OFFLOAD_API_EXPORT int olLaunchKernel(OlQueue q, OlKernel k,
                                      const size_t *gridSizes,
                                      const size_t *blockSizes, size_t nDims,
                                      void **args, size_t nArgs,
                                      size_t sharedMemSize) HC_NOEXCEPT;

/* ---- additions of this build (no counterpart in the reference) ---------- */

/* The CUstream behind a queue, so that a caller can record its own events on
 * it or hand it to another library (e.g. wrap it as a torch ExternalStream). */
OFFLOAD_API_EXPORT void *olxQueueNativeHandle(OlQueue q) HC_NOEXCEPT;

/* Asynchronous copies on the queue's stream.  The reference ABI has no copy
 * call because its callers always pass device-resident torch tensors. */
OFFLOAD_API_EXPORT int olxMemcpyHtoD(OlQueue q, void *dst, const void *src,
                                     size_t size) HC_NOEXCEPT;
OFFLOAD_API_EXPORT int olxMemcpyDtoH(OlQueue q, void *dst, const void *src,
                                     size_t size) HC_NOEXCEPT;
OFFLOAD_API_EXPORT int olxMemsetD8(OlQueue q, void *dst, int value,
                                   size_t size) HC_NOEXCEPT;

/* Integer attribute of the device behind `dev`; `what` is one of the
 * OLX_DEVICE_* constants.  Returns 0 on success. */
#define OLX_DEVICE_SM_COUNT 1
#define OLX_DEVICE_CC_MAJOR 2
#define OLX_DEVICE_CC_MINOR 3
#define OLX_DEVICE_L2_BYTES 4
#define OLX_DEVICE_MAX_SMEM_OPTIN 5
#define OLX_DEVICE_ORDINAL 6 /* the N of the "cuda:N" the device was created from */
OFFLOAD_API_EXPORT int olxDeviceAttribute(OlDevice dev, int what,
                                          long long *valueRet) HC_NOEXCEPT;

/* Encodes a rank-2 tiled TMA descriptor (128 bytes, 64-byte aligned `mapOut`)
 * for a row-major matrix whose rows are `rowPitchBytes` apart.  `elemKind` is
 * 0 = bf16, 1 = f32, 2 = u8.  `swizzle` is 0 (none) or 128. */
OFFLOAD_API_EXPORT int olxEncodeTensorMap2D(OlDevice dev, void *mapOut,
                                            int elemKind, const void *base,
                                            size_t rows, size_t cols,
                                            size_t rowPitchBytes,
                                            unsigned boxRows, unsigned boxCols,
                                            int swizzle) HC_NOEXCEPT;

/* The same for a tensor of rank 2..5: `dims[rank]` and `box[rank]` innermost
 * first, `stridesBytes[rank - 1]` the pitch of every dimension but the
 * innermost (which is contiguous).  Coordinates outside the tensor read zeros. */
OFFLOAD_API_EXPORT int olxEncodeTensorMapTiled(OlDevice dev, void *mapOut,
                                               int elemKind, const void *base,
                                               int rank, const size_t *dims,
                                               const size_t *stridesBytes,
                                               const unsigned *box,
                                               int swizzle) HC_NOEXCEPT;

/* How many clusters of `clusterSize` CTAs (each `blockThreads` threads and
 * `sharedMemSize` bytes of dynamic shared memory) of kernel `k` the device can
 * hold at once.  A persistent kernel launched with more CTAs than that runs
 * the excess as a second wave.  Returns 0 on success. */
OFFLOAD_API_EXPORT int olxMaxActiveClusters(OlQueue q, OlKernel k,
                                            unsigned blockThreads,
                                            size_t sharedMemSize,
                                            unsigned clusterSize,
                                            int *clustersRet) HC_NOEXCEPT;

/* Makes the device's primary context current on the calling thread until the
 * matching olxDeviceContextLeave (a push and a pop of the driver's context
 * stack; the thread's previous context, if any, is current again afterwards).
 * For code that must call another CUDA library on this device without
 * changing the thread's device.  Returns 0 on success. */
OFFLOAD_API_EXPORT int olxDeviceContextEnter(OlDevice dev) HC_NOEXCEPT;
OFFLOAD_API_EXPORT int olxDeviceContextLeave(OlDevice dev) HC_NOEXCEPT;

/* Which GPU owns the memory `ptr` points into: *ordinalRet is its ordinal, or
 * -1 when `ptr` is not device memory (host memory, unknown to the driver).
 * Returns 0 on success. */
OFFLOAD_API_EXPORT int olxPointerDevice(OlDevice dev, const void *ptr,
                                        int *ordinalRet) HC_NOEXCEPT;

/* Events order work between queues of one device without blocking the host:
 * olxRecordEvent marks a point in a queue, olxQueueWaitEvent makes everything
 * submitted to a queue afterwards wait for that point.  The reference needs
 * none because it synchronises the host after every launch
 * (python/cpp/py-runtime/src/GpuRuntime.cpp:67). */
typedef void *OlxEvent;
/* `timing` 0 makes an event that only orders work (cheaper); nonzero one that
 * olxEventElapsedMs can read. */
OFFLOAD_API_EXPORT OlxEvent olxCreateEvent(OlDevice dev, int timing) HC_NOEXCEPT;
OFFLOAD_API_EXPORT void olxReleaseEvent(OlDevice dev, OlxEvent ev) HC_NOEXCEPT;
OFFLOAD_API_EXPORT int olxRecordEvent(OlQueue q, OlxEvent ev) HC_NOEXCEPT;
OFFLOAD_API_EXPORT int olxQueueWaitEvent(OlQueue q, OlxEvent ev) HC_NOEXCEPT;
/* Milliseconds between two recorded events that have both completed. */
OFFLOAD_API_EXPORT int olxEventElapsedMs(OlDevice dev, OlxEvent from, OlxEvent to,
                                         float *msRet) HC_NOEXCEPT;

/* Page-locks (pins) an existing host range so that copies to and from it run
 * asynchronously at full link speed, and undoes it.  Returns 0 on success. */
OFFLOAD_API_EXPORT int olxHostRegister(OlDevice dev, void *ptr,
                                       size_t size) HC_NOEXCEPT;
OFFLOAD_API_EXPORT int olxHostUnregister(OlDevice dev, void *ptr) HC_NOEXCEPT;

#ifdef __cplusplus
}
#endif
