/* A stand-in for libcuda.so.1 that knows no devices.
 *
 * TEST INFRASTRUCTURE ONLY.  The reference's CUDA backend
 * (gpu-runtime/cuda-runtime/src/Runtime.cpp) links against the driver library,
 * so it cannot even be loaded on a machine without one.  This file defines the
 * driver entry points that backend imports; every call fails with
 * CUDA_ERROR_NO_DEVICE (100).  With it the reference's runtime libraries,
 * compiled from their own sources by oracle/build_ref.py, load on any host, so
 * their pure-host behaviour (exported symbols, olSuggestBlockSize, device
 * description parsing, error texts) can be compared with this repository's
 * libraries.  It is never loaded in a process that uses a real GPU.
 */
#include <stddef.h>

#define FAKE(name) int name() { return 100; }

FAKE(cuInit)
FAKE(cuDeviceGet)
FAKE(cuDevicePrimaryCtxRetain)
FAKE(cuCtxPushCurrent_v2)
FAKE(cuCtxPopCurrent_v2)
FAKE(cuModuleLoadData)
FAKE(cuModuleUnload)
FAKE(cuModuleGetFunction)
FAKE(cuStreamCreate)
FAKE(cuStreamDestroy_v2)
FAKE(cuStreamSynchronize)
FAKE(cuMemAlloc_v2)
FAKE(cuMemFree_v2)
FAKE(cuLaunchKernel)

int cuGetErrorName(int error, const char **name) {
  *name = error == 100 ? "CUDA_ERROR_NO_DEVICE" : "CUDA_ERROR_UNKNOWN";
  return 0;
}
