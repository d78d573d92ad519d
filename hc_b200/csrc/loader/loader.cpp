// libhc-gpu-runtime-loader.so: backend-agnostic front of the ol* offload ABI.
//
// `olCreateDevice("<backend>:<id>")` picks `libhc-<backend>-runtime.so`, binds
// its thirteen ol* entry points and forwards every later call to it; handles
// returned to the caller are loader-side wrappers that remember which backend
// owns them.  Same exports and error texts as the reference shim
// (gpu-runtime/loader/src/Loader.cpp:20-45,326-444 and SharedLib.cpp:17-79).
//
// Two deliberate differences:
//   * the reference opens a backend with RTLD_NOLOAD (SharedLib.cpp:22), which
//     only works when something else already loaded it; here that is tried
//     first and a real dlopen follows, so the loader works stand-alone;
//   * a backend library is opened once per process and shared by all devices
//     (the reference re-opens it per device, Loader.cpp:237-262).
#include "offload_api.h"

#include <dlfcn.h>

#include <cstdio>
#include <cstring>
#include <map>
#include <memory>
#include <mutex>
#include <string>
#include <vector>

namespace {

// ---- configuration set through the two extra exports ----------------------
std::mutex configLock;
std::vector<std::string> searchPaths;
bool traceCalls = false;

// Prints "<name> enter" / "<name> exit" around a call when tracing is on; an
// optional detail string is appended to the first line.
class Trace {
public:
  explicit Trace(const char *fn, const std::string &detail = {})
      : name(fn), on(traceCalls) {
    if (!on)
      return;
    if (detail.empty())
      std::fprintf(stdout, "%s enter\n", name);
    else
      std::fprintf(stdout, "%s %s\n", name, detail.c_str());
    std::fflush(stdout);
  }
  ~Trace() {
    if (!on)
      return;
    std::fprintf(stdout, "%s exit\n", name);
    std::fflush(stdout);
  }

private:
  const char *name;
  bool on;
};

std::string listOf(const size_t *v, size_t n) {
  std::string s = "[";
  for (size_t i = 0; v && i < n; ++i) {
    if (i)
      s += ", ";
    s += std::to_string(v[i]);
  }
  return s + "]";
}

// ---- one opened backend library -------------------------------------------
struct Backend {
  void *lib = nullptr;

  decltype(&olCreateDevice) CreateDevice = nullptr;
  decltype(&olReleaseDevice) ReleaseDevice = nullptr;
  decltype(&olCreateModule) CreateModule = nullptr;
  decltype(&olReleaseModule) ReleaseModule = nullptr;
  decltype(&olGetKernel) GetKernel = nullptr;
  decltype(&olReleaseKernel) ReleaseKernel = nullptr;
  decltype(&olSuggestBlockSize) SuggestBlockSize = nullptr;
  decltype(&olCreateQueue) CreateQueue = nullptr;
  decltype(&olReleaseQueue) ReleaseQueue = nullptr;
  decltype(&olSyncQueue) SyncQueue = nullptr;
  decltype(&olAllocDevice) AllocDevice = nullptr;
  decltype(&olDeallocDevice) DeallocDevice = nullptr;
  decltype(&olLaunchKernel) LaunchKernel = nullptr;
  // Optional additions; null when the backend does not have them.
  decltype(&olxQueueNativeHandle) QueueNativeHandle = nullptr;
  decltype(&olxMemcpyHtoD) MemcpyHtoD = nullptr;
  decltype(&olxMemcpyDtoH) MemcpyDtoH = nullptr;
  decltype(&olxMemsetD8) MemsetD8 = nullptr;
  decltype(&olxDeviceAttribute) DeviceAttribute = nullptr;
  decltype(&olxEncodeTensorMap2D) EncodeTensorMap2D = nullptr;
  decltype(&olxEncodeTensorMapTiled) EncodeTensorMapTiled = nullptr;
  decltype(&olxMaxActiveClusters) MaxActiveClusters = nullptr;
  decltype(&olxDeviceContextEnter) DeviceContextEnter = nullptr;
  decltype(&olxDeviceContextLeave) DeviceContextLeave = nullptr;
  decltype(&olxPointerDevice) PointerDevice = nullptr;
  decltype(&olxCreateEvent) CreateEvent = nullptr;
  decltype(&olxReleaseEvent) ReleaseEvent = nullptr;
  decltype(&olxRecordEvent) RecordEvent = nullptr;
  decltype(&olxQueueWaitEvent) QueueWaitEvent = nullptr;
  decltype(&olxEventElapsedMs) EventElapsedMs = nullptr;
  decltype(&olxHostRegister) HostRegister = nullptr;
  decltype(&olxHostUnregister) HostUnregister = nullptr;
};

struct Reporter {
  OlErrorCallback callback;
  void *ctx;
  void operator()(OlSeverity sev, const std::string &text) const {
    if (callback)
      callback(ctx, sev, text.c_str());
  }
};

template <typename F>
bool bindSymbol(void *lib, F &slot, const char *name, const Reporter *report) {
  dlerror();
  slot = reinterpret_cast<F>(dlsym(lib, name));
  if (slot)
    return true;
  if (report) {
    const char *e = dlerror();
    (*report)(OlSeverity::Error, std::string("Could not retrieve symbol ") +
                                     name + ". Error encountered: " +
                                     (e ? e : "<null>"));
  }
  return false;
}

// Opens `path` and binds the ABI.  A library missing any of the thirteen
// required symbols is rejected as a whole.
std::unique_ptr<Backend> openBackend(const std::string &path,
                                     const Reporter &report) {
  void *lib = dlopen(path.c_str(), RTLD_NOLOAD | RTLD_NOW | RTLD_LOCAL);
  if (!lib)
    lib = dlopen(path.c_str(), RTLD_NOW | RTLD_LOCAL);
  if (!lib) {
    const char *e = dlerror();
    report(OlSeverity::Message, "Could not load library " + path +
                                    ". Error encountered: " +
                                    (e ? e : "<null>"));
    return nullptr;
  }
  auto b = std::make_unique<Backend>();
  b->lib = lib;
  bool ok = true;
#define HC_BIND(fn) ok = bindSymbol(lib, b->fn, "ol" #fn, &report) && ok
  HC_BIND(CreateDevice);
  HC_BIND(ReleaseDevice);
  HC_BIND(CreateModule);
  HC_BIND(ReleaseModule);
  HC_BIND(GetKernel);
  HC_BIND(ReleaseKernel);
  HC_BIND(SuggestBlockSize);
  HC_BIND(CreateQueue);
  HC_BIND(ReleaseQueue);
  HC_BIND(SyncQueue);
  HC_BIND(AllocDevice);
  HC_BIND(DeallocDevice);
  HC_BIND(LaunchKernel);
#undef HC_BIND
  if (!ok) {
    dlclose(lib);
    return nullptr;
  }
#define HC_BIND_OPT(fn) bindSymbol(lib, b->fn, "olx" #fn, nullptr)
  HC_BIND_OPT(QueueNativeHandle);
  HC_BIND_OPT(MemcpyHtoD);
  HC_BIND_OPT(MemcpyDtoH);
  HC_BIND_OPT(MemsetD8);
  HC_BIND_OPT(DeviceAttribute);
  HC_BIND_OPT(EncodeTensorMap2D);
  HC_BIND_OPT(EncodeTensorMapTiled);
  HC_BIND_OPT(MaxActiveClusters);
  HC_BIND_OPT(DeviceContextEnter);
  HC_BIND_OPT(DeviceContextLeave);
  HC_BIND_OPT(PointerDevice);
  HC_BIND_OPT(CreateEvent);
  HC_BIND_OPT(ReleaseEvent);
  HC_BIND_OPT(RecordEvent);
  HC_BIND_OPT(QueueWaitEvent);
  HC_BIND_OPT(EventElapsedMs);
  HC_BIND_OPT(HostRegister);
  HC_BIND_OPT(HostUnregister);
#undef HC_BIND_OPT
  return b;
}

// Backends stay open for the life of the process, keyed by the path that
// opened them.
std::mutex backendLock;
std::map<std::string, std::unique_ptr<Backend>> backends;

const Backend *findBackend(const std::string &path, const Reporter &report) {
  std::lock_guard<std::mutex> lock(backendLock);
  auto it = backends.find(path);
  if (it != backends.end())
    return it->second.get();
  auto opened = openBackend(path, report);
  if (!opened)
    return nullptr;
  return (backends[path] = std::move(opened)).get();
}

// ---- caller-visible handles -------------------------------------------------
struct DeviceHandle {
  const Backend *api;
  OlDevice inner;
  Reporter report;
};
struct ModuleHandle {
  DeviceHandle *device;
  OlModule inner;
};
struct KernelHandle {
  ModuleHandle *module;
  OlKernel inner;
};
struct QueueHandle {
  DeviceHandle *device;
  OlQueue inner;
};

} // namespace

extern "C" {

// reference: gpu-runtime/loader/src/Loader.cpp:20-39
OFFLOAD_API_EXPORT void setGPULoaderSearchPaths(const char *paths[],
                                                size_t count) {
  std::lock_guard<std::mutex> lock(configLock);
  searchPaths.clear();
  for (size_t i = 0; paths && i < count; ++i)
    if (paths[i])
      searchPaths.emplace_back(paths[i]);
}

// reference: gpu-runtime/loader/src/Loader.cpp:41-45
OFFLOAD_API_EXPORT void enableFuncTracing(int val) { traceCalls = val != 0; }

OlDevice olCreateDevice(const char *desc, OlErrorCallback errCallback,
                        void *ctx) noexcept {
  Trace t(__func__);
  Reporter report{errCallback, ctx};
  std::string text(desc ? desc : "");
  auto colon = text.find(':');
  if (colon == std::string::npos) {
    report(OlSeverity::Error, "Invalid device desc: " + text);
    return nullptr;
  }
  std::string backendName = text.substr(0, colon);
  std::string libName = "libhc-" + backendName + "-runtime.so";

  std::vector<std::string> candidates;
  {
    std::lock_guard<std::mutex> lock(configLock);
    for (const auto &dir : searchPaths)
      candidates.push_back(dir + "/" + libName);
  }
  candidates.push_back(libName);

  for (const auto &path : candidates) {
    const Backend *api = findBackend(path, report);
    if (!api)
      continue;
    OlDevice inner = api->CreateDevice(desc, errCallback, ctx);
    if (!inner)
      return nullptr; // the backend has already said why
    return new DeviceHandle{api, inner, report};
  }
  report(OlSeverity::Error, "Runtime not found: " + backendName);
  return nullptr;
}

void olReleaseDevice(OlDevice d) noexcept {
  Trace t(__func__);
  auto *dev = static_cast<DeviceHandle *>(d);
  if (!dev)
    return;
  dev->api->ReleaseDevice(dev->inner);
  delete dev;
}

OlModule olCreateModule(OlDevice d, const void *data, size_t len) noexcept {
  Trace t(__func__);
  auto *dev = static_cast<DeviceHandle *>(d);
  if (!dev)
    return nullptr;
  OlModule inner = dev->api->CreateModule(dev->inner, data, len);
  return inner ? new ModuleHandle{dev, inner} : nullptr;
}

void olReleaseModule(OlModule m) noexcept {
  Trace t(__func__);
  auto *mod = static_cast<ModuleHandle *>(m);
  if (!mod)
    return;
  mod->device->api->ReleaseModule(mod->inner);
  delete mod;
}

OlKernel olGetKernel(OlModule m, const char *name) noexcept {
  Trace t(__func__);
  auto *mod = static_cast<ModuleHandle *>(m);
  if (!mod)
    return nullptr;
  OlKernel inner = mod->device->api->GetKernel(mod->inner, name);
  return inner ? new KernelHandle{mod, inner} : nullptr;
}

void olReleaseKernel(OlKernel k) noexcept {
  Trace t(__func__);
  auto *kernel = static_cast<KernelHandle *>(k);
  if (!kernel)
    return;
  kernel->module->device->api->ReleaseKernel(kernel->inner);
  delete kernel;
}

int olSuggestBlockSize(OlKernel k, const size_t *globalsSizes,
                       size_t *blockSizesRet, size_t nDims) noexcept {
  Trace t(__func__);
  auto *kernel = static_cast<KernelHandle *>(k);
  if (!kernel)
    return 1;
  return kernel->module->device->api->SuggestBlockSize(
      kernel->inner, globalsSizes, blockSizesRet, nDims);
}

OlQueue olCreateQueue(OlDevice d) noexcept {
  Trace t(__func__);
  auto *dev = static_cast<DeviceHandle *>(d);
  if (!dev)
    return nullptr;
  OlQueue inner = dev->api->CreateQueue(dev->inner);
  return inner ? new QueueHandle{dev, inner} : nullptr;
}

void olReleaseQueue(OlQueue q) noexcept {
  Trace t(__func__);
  auto *queue = static_cast<QueueHandle *>(q);
  if (!queue)
    return;
  queue->device->api->ReleaseQueue(queue->inner);
  delete queue;
}

int olSyncQueue(OlQueue q) noexcept {
  Trace t(__func__);
  auto *queue = static_cast<QueueHandle *>(q);
  return queue ? queue->device->api->SyncQueue(queue->inner) : 1;
}

void *olAllocDevice(OlQueue q, size_t size, size_t align) noexcept {
  Trace t(__func__);
  auto *queue = static_cast<QueueHandle *>(q);
  return queue ? queue->device->api->AllocDevice(queue->inner, size, align)
               : nullptr;
}

void olDeallocDevice(OlQueue q, void *data) noexcept {
  Trace t(__func__);
  auto *queue = static_cast<QueueHandle *>(q);
  if (queue)
    queue->device->api->DeallocDevice(queue->inner, data);
}

int olLaunchKernel(OlQueue q, OlKernel k, const size_t *gridSizes,
                   const size_t *blockSizes, size_t nDims, void **args,
                   size_t nArgs, size_t sharedMemSize) noexcept {
  Trace t(__func__,
          traceCalls ? "grid: " + listOf(gridSizes, nDims) + ", blocks " +
                           listOf(blockSizes, nDims) + ", nargs " +
                           std::to_string(nArgs) + ", shMem " +
                           std::to_string(sharedMemSize)
                     : std::string());
  auto *queue = static_cast<QueueHandle *>(q);
  auto *kernel = static_cast<KernelHandle *>(k);
  if (!queue)
    return 1;
  if (!kernel) {
    queue->device->report(OlSeverity::Error, "Invalid kernel handle");
    return 1;
  }
  return queue->device->api->LaunchKernel(queue->inner, kernel->inner,
                                          gridSizes, blockSizes, nDims, args,
                                          nArgs, sharedMemSize);
}

// ---- optional additions, forwarded when the backend has them ---------------

static int missing(const DeviceHandle *dev, const char *what) {
  dev->report(OlSeverity::Error,
              std::string("Backend does not export ") + what);
  return 1;
}

void *olxQueueNativeHandle(OlQueue q) noexcept {
  auto *queue = static_cast<QueueHandle *>(q);
  if (!queue || !queue->device->api->QueueNativeHandle)
    return nullptr;
  return queue->device->api->QueueNativeHandle(queue->inner);
}

int olxMemcpyHtoD(OlQueue q, void *dst, const void *src, size_t size) noexcept {
  Trace t(__func__);
  auto *queue = static_cast<QueueHandle *>(q);
  if (!queue)
    return 1;
  auto fn = queue->device->api->MemcpyHtoD;
  return fn ? fn(queue->inner, dst, src, size)
            : missing(queue->device, "olxMemcpyHtoD");
}

int olxMemcpyDtoH(OlQueue q, void *dst, const void *src, size_t size) noexcept {
  Trace t(__func__);
  auto *queue = static_cast<QueueHandle *>(q);
  if (!queue)
    return 1;
  auto fn = queue->device->api->MemcpyDtoH;
  return fn ? fn(queue->inner, dst, src, size)
            : missing(queue->device, "olxMemcpyDtoH");
}

int olxMemsetD8(OlQueue q, void *dst, int value, size_t size) noexcept {
  Trace t(__func__);
  auto *queue = static_cast<QueueHandle *>(q);
  if (!queue)
    return 1;
  auto fn = queue->device->api->MemsetD8;
  return fn ? fn(queue->inner, dst, value, size)
            : missing(queue->device, "olxMemsetD8");
}

int olxDeviceAttribute(OlDevice d, int what, long long *valueRet) noexcept {
  auto *dev = static_cast<DeviceHandle *>(d);
  if (!dev)
    return 1;
  auto fn = dev->api->DeviceAttribute;
  return fn ? fn(dev->inner, what, valueRet)
            : missing(dev, "olxDeviceAttribute");
}

int olxEncodeTensorMap2D(OlDevice d, void *mapOut, int elemKind,
                         const void *base, size_t rows, size_t cols,
                         size_t rowPitchBytes, unsigned boxRows,
                         unsigned boxCols, int swizzle) noexcept {
  auto *dev = static_cast<DeviceHandle *>(d);
  if (!dev)
    return 1;
  auto fn = dev->api->EncodeTensorMap2D;
  return fn ? fn(dev->inner, mapOut, elemKind, base, rows, cols, rowPitchBytes,
                 boxRows, boxCols, swizzle)
            : missing(dev, "olxEncodeTensorMap2D");
}

int olxEncodeTensorMapTiled(OlDevice d, void *mapOut, int elemKind, const void *base,
                            int rank, const size_t *dims, const size_t *stridesBytes,
                            const unsigned *box, int swizzle) noexcept {
  auto *dev = static_cast<DeviceHandle *>(d);
  if (!dev)
    return 1;
  auto fn = dev->api->EncodeTensorMapTiled;
  return fn ? fn(dev->inner, mapOut, elemKind, base, rank, dims, stridesBytes, box, swizzle)
            : missing(dev, "olxEncodeTensorMapTiled");
}

int olxMaxActiveClusters(OlQueue q, OlKernel k, unsigned blockThreads,
                         size_t sharedMemSize, unsigned clusterSize,
                         int *clustersRet) noexcept {
  auto *queue = static_cast<QueueHandle *>(q);
  auto *kernel = static_cast<KernelHandle *>(k);
  if (!queue || !kernel)
    return 1;
  auto fn = queue->device->api->MaxActiveClusters;
  return fn ? fn(queue->inner, kernel->inner, blockThreads, sharedMemSize,
                 clusterSize, clustersRet)
            : missing(queue->device, "olxMaxActiveClusters");
}

int olxDeviceContextEnter(OlDevice d) noexcept {
  auto *dev = static_cast<DeviceHandle *>(d);
  if (!dev)
    return 1;
  auto fn = dev->api->DeviceContextEnter;
  return fn ? fn(dev->inner) : missing(dev, "olxDeviceContextEnter");
}

int olxDeviceContextLeave(OlDevice d) noexcept {
  auto *dev = static_cast<DeviceHandle *>(d);
  if (!dev)
    return 1;
  auto fn = dev->api->DeviceContextLeave;
  return fn ? fn(dev->inner) : missing(dev, "olxDeviceContextLeave");
}

int olxPointerDevice(OlDevice d, const void *ptr, int *ordinalRet) noexcept {
  auto *dev = static_cast<DeviceHandle *>(d);
  if (!dev)
    return 1;
  auto fn = dev->api->PointerDevice;
  return fn ? fn(dev->inner, ptr, ordinalRet) : missing(dev, "olxPointerDevice");
}

OlxEvent olxCreateEvent(OlDevice d, int timing) noexcept {
  auto *dev = static_cast<DeviceHandle *>(d);
  if (!dev)
    return nullptr;
  auto fn = dev->api->CreateEvent;
  if (!fn) {
    missing(dev, "olxCreateEvent");
    return nullptr;
  }
  return fn(dev->inner, timing);
}

void olxReleaseEvent(OlDevice d, OlxEvent ev) noexcept {
  auto *dev = static_cast<DeviceHandle *>(d);
  if (dev && dev->api->ReleaseEvent)
    dev->api->ReleaseEvent(dev->inner, ev);
}

int olxRecordEvent(OlQueue q, OlxEvent ev) noexcept {
  auto *queue = static_cast<QueueHandle *>(q);
  if (!queue)
    return 1;
  auto fn = queue->device->api->RecordEvent;
  return fn ? fn(queue->inner, ev) : missing(queue->device, "olxRecordEvent");
}

int olxQueueWaitEvent(OlQueue q, OlxEvent ev) noexcept {
  auto *queue = static_cast<QueueHandle *>(q);
  if (!queue)
    return 1;
  auto fn = queue->device->api->QueueWaitEvent;
  return fn ? fn(queue->inner, ev) : missing(queue->device, "olxQueueWaitEvent");
}

int olxEventElapsedMs(OlDevice d, OlxEvent from, OlxEvent to, float *msRet) noexcept {
  auto *dev = static_cast<DeviceHandle *>(d);
  if (!dev)
    return 1;
  auto fn = dev->api->EventElapsedMs;
  return fn ? fn(dev->inner, from, to, msRet) : missing(dev, "olxEventElapsedMs");
}

int olxHostRegister(OlDevice d, void *ptr, size_t size) noexcept {
  auto *dev = static_cast<DeviceHandle *>(d);
  if (!dev)
    return 1;
  auto fn = dev->api->HostRegister;
  return fn ? fn(dev->inner, ptr, size) : missing(dev, "olxHostRegister");
}

int olxHostUnregister(OlDevice d, void *ptr) noexcept {
  auto *dev = static_cast<DeviceHandle *>(d);
  if (!dev)
    return 1;
  auto fn = dev->api->HostUnregister;
  return fn ? fn(dev->inner, ptr) : missing(dev, "olxHostUnregister");
}

} // extern "C"
