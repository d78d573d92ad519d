/* C-ABI of libhc-python-runtime.so: the glue between Python objects and the
 * ol* offload ABI that host code of a compiled kernel calls.
 *
 * Same seven exports as the reference
 * (python/cpp/py-runtime/src/PyRuntime.cpp:36-94).  Functions that take a
 * `void *obj` expect a borrowed `PyObject *` and must be called with the GIL
 * held.
 */
#pragma once

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
#include <string>
namespace hc {
/* reference: python/cpp/shared/include/PyRuntimeShared.hpp:9-13 */
struct ExceptionDesc {
  std::string message;
};
} // namespace hc
typedef hc::ExceptionDesc HcExceptionDesc;
extern "C" {
#else
typedef struct HcExceptionDescOpaque HcExceptionDesc;
#endif

#define HC_PYRT_API __attribute__((visibility("default")))

/* What hcgpuConvertPyArray fills: an MLIR ranked memref descriptor with
 * `rank` sizes followed by `rank` strides, strides counted in elements.
 * reference: python/cpp/py-runtime/src/PyABI.cpp:15-37 */
typedef struct HcMemrefDescriptor {
  void *allocated;
  void *aligned;
  intptr_t offset;
  intptr_t sizesAndStrides[1]; /* really 2 * rank entries */
} HcMemrefDescriptor;

/* reference: PyRuntime.cpp:36-39 */
HC_PYRT_API void hcgpuEnableTraceFunctions(int val);

/* `obj` is a Python list of `bytes` paths handed to the loader.
 * reference: PyRuntime.cpp:41-45, PyABI.cpp:45-54 */
HC_PYRT_API void hcgpuSetRuntimeSearchPaths(void *obj);

/* Array-like Python object (torch tensor, or anything with
 * __cuda_array_interface__ / __array_interface__) -> memref descriptor.
 * Returns 0, or 1 with `errorDesc->message` set ("Invalid rank", ...).
 * reference: PyRuntime.cpp:47-58, PyABI.cpp:23-37 */
HC_PYRT_API int hcgpuConvertPyArray(HcExceptionDesc *errorDesc, void *obj,
                                    int rank, void *ret);

/* Python int -> int64.  reference: PyRuntime.cpp:60-71, PyABI.cpp:39-41 */
HC_PYRT_API int hcgpuConvertPyInt64(HcExceptionDesc *errorDesc, void *obj,
                                    int64_t *ret);

/* Creates (once per `*handle`) device, queue, module and kernel; later calls
 * with the same handle slot return the cached kernel.  Aborts the process on
 * failure, as the reference does.
 * reference: PyRuntime.cpp:73-78, GpuRuntime.cpp:26-51 */
HC_PYRT_API void *hcgpuGetKernel(void **handle, const char *deviceDesc,
                                 const void *data, size_t dataSize,
                                 const char *kernelName);

/* reference: PyRuntime.cpp:80-85, GpuRuntime.cpp:53-58 */
HC_PYRT_API void hcgpuSuggestBlockSize(void *kernel, const size_t *globalSizes,
                                       size_t *blockSizesRet, size_t nDim);

/* Launches and waits for the kernel to finish, as the reference does.
 * reference: PyRuntime.cpp:87-94, GpuRuntime.cpp:60-69 */
HC_PYRT_API void hcgpuLaunchKernel(void *kernel, const size_t *gridSizes,
                                   const size_t *blockSizes, size_t nDim,
                                   void **args, size_t nArgs,
                                   size_t sharedMemSize);

#ifdef __cplusplus
}
#endif
