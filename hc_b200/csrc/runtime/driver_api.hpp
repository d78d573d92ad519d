// Lazily bound CUDA driver API.
//
// The backend library must load (and report a clean error through the
// OlErrorCallback) on a host without an NVIDIA driver, so libcuda is not a
// link-time dependency: it is opened with dlopen on the first olCreateDevice
// and the entry points used here are resolved by name.
#pragma once

#include <cuda.h>
#include <dlfcn.h>

#include <mutex>
#include <string>

namespace hc {

struct DriverApi {
  // Signatures follow cuda.h; the `_v2` names are the ones libcuda exports
  // for the 64-bit-pointer variants.
  CUresult (*Init)(unsigned) = nullptr;
  CUresult (*GetErrorName)(CUresult, const char **) = nullptr;
  CUresult (*DeviceGet)(CUdevice *, int) = nullptr;
  CUresult (*DeviceGetCount)(int *) = nullptr;
  CUresult (*DeviceGetAttribute)(int *, CUdevice_attribute, CUdevice) = nullptr;
  CUresult (*DevicePrimaryCtxRetain)(CUcontext *, CUdevice) = nullptr;
  CUresult (*DevicePrimaryCtxRelease)(CUdevice) = nullptr;
  CUresult (*CtxPushCurrent)(CUcontext) = nullptr;
  CUresult (*CtxPopCurrent)(CUcontext *) = nullptr;
  CUresult (*ModuleLoadData)(CUmodule *, const void *) = nullptr;
  CUresult (*ModuleUnload)(CUmodule) = nullptr;
  CUresult (*ModuleGetFunction)(CUfunction *, CUmodule, const char *) = nullptr;
  CUresult (*FuncSetAttribute)(CUfunction, CUfunction_attribute, int) = nullptr;
  CUresult (*FuncGetAttribute)(int *, CUfunction_attribute, CUfunction) = nullptr;
  CUresult (*StreamCreate)(CUstream *, unsigned) = nullptr;
  CUresult (*StreamDestroy)(CUstream) = nullptr;
  CUresult (*StreamSynchronize)(CUstream) = nullptr;
  CUresult (*MemAlloc)(CUdeviceptr *, size_t) = nullptr;
  CUresult (*MemFree)(CUdeviceptr) = nullptr;
  CUresult (*MemcpyHtoDAsync)(CUdeviceptr, const void *, size_t, CUstream) = nullptr;
  CUresult (*MemcpyDtoHAsync)(void *, CUdeviceptr, size_t, CUstream) = nullptr;
  CUresult (*MemsetD8Async)(CUdeviceptr, unsigned char, size_t, CUstream) = nullptr;
  CUresult (*LaunchKernel)(CUfunction, unsigned, unsigned, unsigned, unsigned,
                           unsigned, unsigned, unsigned, CUstream, void **,
                           void **) = nullptr;
  CUresult (*TensorMapEncodeTiled)(
      CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *,
      const cuuint64_t *, const cuuint64_t *, const cuuint32_t *,
      const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
      CUtensorMapL2promotion, CUtensorMapFloatOOBfill) = nullptr;

  CUresult (*OccupancyMaxActiveClusters)(int *, CUfunction,
                                         const CUlaunchConfig *) = nullptr;
  CUresult (*PointerGetAttribute)(void *, CUpointer_attribute, CUdeviceptr) = nullptr;
  CUresult (*EventCreate)(CUevent *, unsigned) = nullptr;
  CUresult (*EventDestroy)(CUevent) = nullptr;
  CUresult (*EventRecord)(CUevent, CUstream) = nullptr;
  CUresult (*EventElapsedTime)(float *, CUevent, CUevent) = nullptr;
  CUresult (*StreamWaitEvent)(CUstream, CUevent, unsigned) = nullptr;
  CUresult (*MemHostRegister)(void *, size_t, unsigned) = nullptr;
  CUresult (*MemHostUnregister)(void *) = nullptr;

  bool ok = false;
  std::string error;

  // Returns the process-wide table; `ok` is false (and `error` says why) when
  // the driver library or one of its symbols is missing.
  static const DriverApi &get() {
    static DriverApi api;
    static std::once_flag once;
    std::call_once(once, [] { api.load(); });
    return api;
  }

private:
  void *lib = nullptr;

  template <typename F> bool bind(F &slot, const char *name) {
    slot = reinterpret_cast<F>(dlsym(lib, name));
    if (!slot) {
      error = std::string("CUDA driver symbol not found: ") + name;
      return false;
    }
    return true;
  }

  void load() {
    const char *names[] = {"libcuda.so.1", "libcuda.so"};
    for (const char *n : names) {
      lib = dlopen(n, RTLD_NOW | RTLD_GLOBAL);
      if (lib)
        break;
    }
    if (!lib) {
      const char *e = dlerror();
      error = std::string("CUDA driver library not found: ") + (e ? e : "?");
      return;
    }
    ok = bind(Init, "cuInit") && bind(GetErrorName, "cuGetErrorName") &&
         bind(DeviceGet, "cuDeviceGet") &&
         bind(DeviceGetCount, "cuDeviceGetCount") &&
         bind(DeviceGetAttribute, "cuDeviceGetAttribute") &&
         bind(DevicePrimaryCtxRetain, "cuDevicePrimaryCtxRetain") &&
         bind(DevicePrimaryCtxRelease, "cuDevicePrimaryCtxRelease_v2") &&
         bind(CtxPushCurrent, "cuCtxPushCurrent_v2") &&
         bind(CtxPopCurrent, "cuCtxPopCurrent_v2") &&
         bind(ModuleLoadData, "cuModuleLoadData") &&
         bind(ModuleUnload, "cuModuleUnload") &&
         bind(ModuleGetFunction, "cuModuleGetFunction") &&
         bind(FuncSetAttribute, "cuFuncSetAttribute") &&
         bind(FuncGetAttribute, "cuFuncGetAttribute") &&
         bind(StreamCreate, "cuStreamCreate") &&
         bind(StreamDestroy, "cuStreamDestroy_v2") &&
         bind(StreamSynchronize, "cuStreamSynchronize") &&
         bind(MemAlloc, "cuMemAlloc_v2") && bind(MemFree, "cuMemFree_v2") &&
         bind(MemcpyHtoDAsync, "cuMemcpyHtoDAsync_v2") &&
         bind(MemcpyDtoHAsync, "cuMemcpyDtoHAsync_v2") &&
         bind(MemsetD8Async, "cuMemsetD8Async") &&
         bind(LaunchKernel, "cuLaunchKernel") &&
         bind(TensorMapEncodeTiled, "cuTensorMapEncodeTiled") &&
         bind(OccupancyMaxActiveClusters, "cuOccupancyMaxActiveClusters") &&
         bind(PointerGetAttribute, "cuPointerGetAttribute") &&
         bind(EventCreate, "cuEventCreate") &&
         bind(EventDestroy, "cuEventDestroy_v2") &&
         bind(EventRecord, "cuEventRecord") &&
         bind(EventElapsedTime, "cuEventElapsedTime") &&
         bind(StreamWaitEvent, "cuStreamWaitEvent") &&
         bind(MemHostRegister, "cuMemHostRegister_v2") &&
         bind(MemHostUnregister, "cuMemHostUnregister");
  }
};

} // namespace hc
