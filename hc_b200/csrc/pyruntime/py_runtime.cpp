// libhc-python-runtime.so: the hcgpu* entry points that host code of a
// compiled kernel calls - convert Python arguments, fetch a kernel from a
// binary blob, launch it (reference: python/cpp/py-runtime/src/PyRuntime.cpp:
// 36-94, GpuRuntime.cpp:23-69, PyABI.cpp:15-54).
//
// Differences from the reference, all behind the same seven signatures:
//   * Python objects are read with pybind11 (array_arg.hpp) instead of
//     nanobind's ndarray caster;
//   * device and queue are kept per device description instead of in one
//     process-wide pair (GpuRuntime.cpp:23-24), so "cuda:0" and "cuda:1" can be
//     used from one process;
//   * a module is created once per (device, blob) and shared by its kernels;
//     the reference creates a new module for every call site
//     (GpuRuntime.cpp:41-43).
// Failure of hcgpuGetKernel / hcgpuSuggestBlockSize / hcgpuLaunchKernel still
// prints "Offload error: ..." and aborts, as in GpuRuntime.cpp:11-21: their
// signatures have no way to report an error.
#include "hc_python_runtime.h"

#include "array_arg.hpp"
#include "offload_api.h"

#include <cstdio>
#include <cstdlib>
#include <map>
#include <string>
#include <utility>

extern "C" void setGPULoaderSearchPaths(const char *paths[], size_t count);

namespace {

namespace py = pybind11;

bool traceCalls = false;

struct Trace {
  explicit Trace(const char *fn) : name(fn), on(traceCalls) {
    if (on) {
      std::fprintf(stdout, "%s enter\n", name);
      std::fflush(stdout);
    }
  }
  ~Trace() {
    if (on) {
      std::fprintf(stdout, "%s exit\n", name);
      std::fflush(stdout);
    }
  }
  const char *name;
  bool on;
};

void report(void *, OlSeverity sev, const char *desc) {
  static const char *kinds[] = {"error", "warning", "message"};
  int i = static_cast<int>(sev);
  std::fprintf(stderr, "Offload %s: %s\n", kinds[i < 0 || i > 2 ? 0 : i], desc);
  std::fflush(stderr);
}

[[noreturn]] void fatal(const char *what) {
  report(nullptr, OlSeverity::Error, what);
  std::abort();
}

struct DeviceSlot {
  OlDevice device = nullptr;
  OlQueue queue = nullptr;
  std::map<std::pair<const void *, size_t>, OlModule> modules;
};

std::map<std::string, DeviceSlot> devices;  // by device description
std::map<void *, OlQueue> queueOfKernel;    // kernel handle -> its queue

} // namespace

extern "C" {

void hcgpuEnableTraceFunctions(int val) { traceCalls = val != 0; }

void hcgpuSetRuntimeSearchPaths(void *obj) {
  Trace t(__func__);
  py::gil_scoped_acquire gil;
  std::vector<std::string> keep;
  for (auto item : py::reinterpret_borrow<py::list>(static_cast<PyObject *>(obj)))
    keep.push_back(item.cast<py::bytes>());
  std::vector<const char *> ptrs;
  for (auto &s : keep)
    ptrs.push_back(s.c_str());
  setGPULoaderSearchPaths(ptrs.data(), ptrs.size());
}

int hcgpuConvertPyArray(HcExceptionDesc *errorDesc, void *obj, int rank,
                        void *ret) {
  Trace t(__func__);
  try {
    py::gil_scoped_acquire gil;
    hc::ArrayArg a = hc::arrayFromPython(py::handle(static_cast<PyObject *>(obj)));
    if (a.rank() != rank)
      throw std::runtime_error("Invalid rank");
    auto *desc = static_cast<HcMemrefDescriptor *>(ret);
    desc->allocated = a.data;
    desc->aligned = a.data;
    desc->offset = 0;
    for (int i = 0; i < rank; ++i) {
      desc->sizesAndStrides[i] = a.shape[i];
      desc->sizesAndStrides[i + rank] = a.strides[i];
    }
    return 0;
  } catch (const std::exception &e) {
    if (errorDesc)
      errorDesc->message = e.what();
    return 1;
  }
}

int hcgpuConvertPyInt64(HcExceptionDesc *errorDesc, void *obj, int64_t *ret) {
  Trace t(__func__);
  try {
    py::gil_scoped_acquire gil;
    *ret = py::handle(static_cast<PyObject *>(obj)).cast<int64_t>();
    return 0;
  } catch (const std::exception &e) {
    if (errorDesc)
      errorDesc->message = e.what();
    return 1;
  }
}

void *hcgpuGetKernel(void **handle, const char *deviceDesc, const void *data,
                     size_t dataSize, const char *kernelName) {
  Trace t(__func__);
  if (handle && *handle)
    return *handle;
  DeviceSlot &slot = devices[deviceDesc ? deviceDesc : ""];
  if (!slot.device) {
    slot.device = olCreateDevice(deviceDesc, &report, nullptr);
    if (!slot.device)
      fatal("olCreateDevice failed");
    slot.queue = olCreateQueue(slot.device);
    if (!slot.queue)
      fatal("olCreateSyncQueue failed");
  }
  OlModule &module = slot.modules[{data, dataSize}];
  if (!module) {
    module = olCreateModule(slot.device, data, dataSize);
    if (!module)
      fatal("olCreateModule failed");
  }
  OlKernel kernel = olGetKernel(module, kernelName);
  if (!kernel)
    fatal("olGetKernel failed");
  queueOfKernel[kernel] = slot.queue;
  if (handle)
    *handle = kernel;
  return kernel;
}

void hcgpuSuggestBlockSize(void *kernel, const size_t *globalSizes,
                           size_t *blockSizesRet, size_t nDim) {
  Trace t(__func__);
  if (olSuggestBlockSize(kernel, globalSizes, blockSizesRet, nDim))
    fatal("olSuggestBlockSize failed");
}

void hcgpuLaunchKernel(void *kernel, const size_t *gridSizes,
                       const size_t *blockSizes, size_t nDim, void **args,
                       size_t nArgs, size_t sharedMemSize) {
  Trace t(__func__);
  auto it = queueOfKernel.find(kernel);
  if (it == queueOfKernel.end())
    fatal("hcgpuLaunchKernel: unknown kernel handle");
  if (olLaunchKernel(it->second, kernel, gridSizes, blockSizes, nDim, args,
                     nArgs, sharedMemSize))
    fatal("olLaunchKernel failed");
  if (olSyncQueue(it->second))
    fatal("olSyncQueue failed");
}

} // extern "C"
