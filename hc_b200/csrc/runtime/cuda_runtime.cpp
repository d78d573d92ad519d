// libhc-cuda-runtime.so: the ol* offload ABI over the CUDA driver API, for
// precompiled sm_100a images.
//
// Same exports, argument meaning and error convention as the reference backend
// (gpu-runtime/cuda-runtime/src/Runtime.cpp:122-281).  What differs, and why:
//   * libcuda is bound at run time (driver_api.hpp), so the library loads and
//     fails cleanly on a host without a driver;
//   * olCreateModule checks the blob before the driver parses it, because the
//     blobs are now files shipped with the package rather than JIT output;
//   * olLaunchKernel raises the per-function dynamic shared memory limit when
//     a launch asks for more than 48 KiB (the TMA/tcgen05 kernels need ~200
//     KiB) - the reference never sets that attribute
//     (Runtime.cpp:264-281), so such launches could not work there;
//   * an OlKernel is a small heap object (function + its raised limit) instead
//     of a bare CUfunction (Runtime.cpp:172-184), and olReleaseKernel frees it;
//   * olAllocDevice honours `align` (ignored at Runtime.cpp:242) and
//     olReleaseDevice gives the primary context back.
#include "driver_api.hpp"

#include "offload_api.h"

#include <bit>
#include <charconv>
#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <memory>
#include <mutex>
#include <string_view>
#include <unordered_map>

namespace {

using hc::DriverApi;

struct DeviceState {
  OlErrorCallback callback = nullptr;
  void *callbackCtx = nullptr;
  int ordinal = 0;
  CUdevice handle = 0;
  CUcontext context = nullptr;
  // Over-aligned allocations: user pointer -> pointer cuMemAlloc returned.
  std::mutex allocLock;
  std::unordered_map<void *, CUdeviceptr> overAligned;

  void report(OlSeverity sev, const char *fmt, ...) const
      __attribute__((format(printf, 3, 4))) {
    if (!callback)
      return;
    char text[320];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(text, sizeof(text), fmt, ap);
    va_end(ap);
    callback(callbackCtx, sev, text);
  }

  // Returns 0 when `rc` is CUDA_SUCCESS; otherwise reports
  // "'<call>' failed with '<CUDA_ERROR_...>'" and returns 1.
  int check(const char *call, CUresult rc) const {
    if (rc == CUDA_SUCCESS)
      return 0;
    const char *name = nullptr;
    DriverApi::get().GetErrorName(rc, &name);
    report(OlSeverity::Error, "'%s' failed with '%s'", call,
           name ? name : "<unknown>");
    return 1;
  }
};

// Makes the device's primary context current for the lifetime of the object.
class ContextScope {
public:
  explicit ContextScope(const DeviceState *d) : dev(d) {
    failed = dev->check("cuCtxPushCurrent",
                        DriverApi::get().CtxPushCurrent(dev->context));
  }
  ~ContextScope() {
    if (!failed)
      dev->check("cuCtxPopCurrent", DriverApi::get().CtxPopCurrent(nullptr));
  }
  explicit operator bool() const { return !failed; }

private:
  const DeviceState *dev;
  int failed;
};

struct ModuleState {
  DeviceState *device = nullptr;
  CUmodule module = nullptr;
};

struct KernelState {
  DeviceState *device = nullptr;
  CUfunction function = nullptr;
  int dynSmemLimit = 48 * 1024; // what the driver allows without opt-in
};

struct QueueState {
  DeviceState *device = nullptr;
  CUstream stream = nullptr;
};

// A blob is accepted when it is a complete ELF image (cubin), a fatbin
// container, or NUL-terminated text (PTX).  Anything else would make the
// driver read past `len`.
const char *validateImage(const void *data, size_t len) {
  if (!data || len == 0)
    return "Invalid module image: empty";
  auto *bytes = static_cast<const unsigned char *>(data);
  if (len >= 4 && bytes[0] == 0x7f && bytes[1] == 'E' && bytes[2] == 'L' &&
      bytes[3] == 'F') {
    if (len < 64)
      return "Invalid module image: truncated ELF header";
    uint64_t shoff;
    uint16_t shentsize, shnum;
    std::memcpy(&shoff, bytes + 0x28, 8);
    std::memcpy(&shentsize, bytes + 0x3a, 2);
    std::memcpy(&shnum, bytes + 0x3c, 2);
    if (shoff > len || uint64_t(shentsize) * shnum > len - shoff)
      return "Invalid module image: truncated ELF sections";
    return nullptr;
  }
  uint32_t magic = 0;
  if (len >= 4)
    std::memcpy(&magic, bytes, 4);
  if (magic == 0xBA55ED50u || magic == 0x466243B1u) // fatbin containers
    return nullptr;
  if (bytes[len - 1] == '\0' || std::memchr(bytes, '\0', len))
    return nullptr; // text image
  return "Invalid module image: neither ELF, fatbin nor terminated text";
}

} // namespace

extern "C" {

OlDevice olCreateDevice(const char *desc, OlErrorCallback errCallback,
                        void *ctx) noexcept {
  auto fail = [&](const char *why) -> OlDevice {
    if (errCallback)
      errCallback(ctx, OlSeverity::Error, why);
    return nullptr;
  };
  constexpr std::string_view prefix = "cuda:";
  std::string_view text(desc ? desc : "");
  if (text.substr(0, prefix.size()) != prefix)
    return fail("Invalid device desc");
  text.remove_prefix(prefix.size());
  int ordinal = 0;
  auto parsed = std::from_chars(text.data(), text.data() + text.size(), ordinal);
  if (parsed.ec != std::errc{} || ordinal < 0)
    return fail("Invalid device id");

  const DriverApi &cu = DriverApi::get();
  if (!cu.ok)
    return fail(cu.error.c_str());

  auto dev = std::make_unique<DeviceState>();
  dev->callback = errCallback;
  dev->callbackCtx = ctx;
  dev->ordinal = ordinal;
  static std::once_flag initOnce;
  static CUresult initResult = CUDA_SUCCESS;
  std::call_once(initOnce, [&] { initResult = cu.Init(0); });
  if (dev->check("cuInit", initResult) ||
      dev->check("cuDeviceGet", cu.DeviceGet(&dev->handle, ordinal)) ||
      dev->check("cuDevicePrimaryCtxRetain",
                 cu.DevicePrimaryCtxRetain(&dev->context, dev->handle)))
    return nullptr;
  return dev.release();
}

void olReleaseDevice(OlDevice d) noexcept {
  auto *dev = static_cast<DeviceState *>(d);
  if (!dev)
    return;
  if (dev->context)
    dev->check("cuDevicePrimaryCtxRelease",
               DriverApi::get().DevicePrimaryCtxRelease(dev->handle));
  delete dev;
}

OlModule olCreateModule(OlDevice d, const void *data, size_t len) noexcept {
  auto *dev = static_cast<DeviceState *>(d);
  if (!dev)
    return nullptr;
  if (const char *why = validateImage(data, len)) {
    dev->report(OlSeverity::Error, "%s", why);
    return nullptr;
  }
  ContextScope scope(dev);
  if (!scope)
    return nullptr;
  auto mod = std::make_unique<ModuleState>();
  mod->device = dev;
  if (dev->check("cuModuleLoadData",
                 DriverApi::get().ModuleLoadData(&mod->module, data)))
    return nullptr;
  return mod.release();
}

void olReleaseModule(OlModule m) noexcept {
  auto *mod = static_cast<ModuleState *>(m);
  if (!mod)
    return;
  if (mod->module) {
    ContextScope scope(mod->device);
    if (scope)
      mod->device->check("cuModuleUnload",
                         DriverApi::get().ModuleUnload(mod->module));
  }
  delete mod;
}

OlKernel olGetKernel(OlModule m, const char *name) noexcept {
  auto *mod = static_cast<ModuleState *>(m);
  if (!mod)
    return nullptr;
  if (!name) {
    mod->device->report(OlSeverity::Error, "Invalid kernel name");
    return nullptr;
  }
  auto k = std::make_unique<KernelState>();
  k->device = mod->device;
  if (mod->device->check(
          "cuModuleGetFunction",
          DriverApi::get().ModuleGetFunction(&k->function, mod->module, name)))
    return nullptr;
  return k.release();
}

void olReleaseKernel(OlKernel k) noexcept {
  delete static_cast<KernelState *>(k);
}

int olSuggestBlockSize(OlKernel /*k*/, const size_t *globalsSizes,
                       size_t *blockSizesRet, size_t nDims) noexcept {
  if (nDims < 1 || nDims > 3 || !globalsSizes || !blockSizesRet)
    return 1;
  // Dimensions are served in order; each takes what is left of a 1024-thread
  // budget, and the budget shrinks by the power of two that covers the take.
  size_t budget = 1024;
  for (size_t i = 0; i < nDims; ++i) {
    size_t want = globalsSizes[i];
    if (want <= 1) {
      blockSizesRet[i] = 1;
      continue;
    }
    size_t take = want < budget ? want : budget;
    blockSizesRet[i] = take;
    budget /= std::bit_ceil(take);
  }
  return 0;
}

OlQueue olCreateQueue(OlDevice d) noexcept {
  auto *dev = static_cast<DeviceState *>(d);
  if (!dev)
    return nullptr;
  ContextScope scope(dev);
  if (!scope)
    return nullptr;
  auto q = std::make_unique<QueueState>();
  q->device = dev;
  if (dev->check("cuStreamCreate", DriverApi::get().StreamCreate(
                                       &q->stream, CU_STREAM_NON_BLOCKING)))
    return nullptr;
  return q.release();
}

void olReleaseQueue(OlQueue queue) noexcept {
  auto *q = static_cast<QueueState *>(queue);
  if (!q)
    return;
  if (q->stream) {
    ContextScope scope(q->device);
    if (scope)
      q->device->check("cuStreamDestroy",
                       DriverApi::get().StreamDestroy(q->stream));
  }
  delete q;
}

int olSyncQueue(OlQueue queue) noexcept {
  auto *q = static_cast<QueueState *>(queue);
  if (!q)
    return 1;
  ContextScope scope(q->device);
  if (!scope)
    return 1;
  return q->device->check("cuStreamSynchronize",
                          DriverApi::get().StreamSynchronize(q->stream));
}

void *olAllocDevice(OlQueue queue, size_t size, size_t align) noexcept {
  auto *q = static_cast<QueueState *>(queue);
  if (!q)
    return nullptr;
  DeviceState *dev = q->device;
  if (align & (align - 1)) {
    dev->report(OlSeverity::Error, "Invalid alignment: %zu", align);
    return nullptr;
  }
  ContextScope scope(dev);
  if (!scope)
    return nullptr;
  constexpr size_t driverAlign = 256; // what cuMemAlloc guarantees
  size_t pad = align > driverAlign ? align : 0;
  CUdeviceptr raw = 0;
  if (dev->check("cuMemAlloc",
                 DriverApi::get().MemAlloc(&raw, (size ? size : 1) + pad)))
    return nullptr;
  if (!pad)
    return reinterpret_cast<void *>(raw);
  CUdeviceptr user = (raw + align - 1) & ~CUdeviceptr(align - 1);
  std::lock_guard<std::mutex> lock(dev->allocLock);
  dev->overAligned[reinterpret_cast<void *>(user)] = raw;
  return reinterpret_cast<void *>(user);
}

void olDeallocDevice(OlQueue queue, void *data) noexcept {
  auto *q = static_cast<QueueState *>(queue);
  if (!q || !data)
    return;
  DeviceState *dev = q->device;
  CUdeviceptr raw = reinterpret_cast<CUdeviceptr>(data);
  {
    std::lock_guard<std::mutex> lock(dev->allocLock);
    auto it = dev->overAligned.find(data);
    if (it != dev->overAligned.end()) {
      raw = it->second;
      dev->overAligned.erase(it);
    }
  }
  ContextScope scope(dev);
  if (scope)
    dev->check("cuMemFree", DriverApi::get().MemFree(raw));
}

int olLaunchKernel(OlQueue queue, OlKernel kernel, const size_t *gridSizes,
                   const size_t *blockSizes, size_t nDims, void **args,
                   size_t /*nArgs*/, size_t sharedMemSize) noexcept {
  auto *q = static_cast<QueueState *>(queue);
  auto *k = static_cast<KernelState *>(kernel);
  if (!q)
    return 1;
  DeviceState *dev = q->device;
  if (nDims != 3) {
    dev->report(OlSeverity::Error, "Invalid launch dims: %d",
                static_cast<int>(nDims));
    return 1;
  }
  if (!k || !gridSizes || !blockSizes) {
    dev->report(OlSeverity::Error, "Invalid launch arguments");
    return 1;
  }
  const DriverApi &cu = DriverApi::get();
  ContextScope scope(dev);
  if (!scope)
    return 1;
  if (sharedMemSize > size_t(k->dynSmemLimit)) {
    if (dev->check("cuFuncSetAttribute",
                   cu.FuncSetAttribute(
                       k->function,
                       CU_FUNC_ATTRIBUTE_MAX_DYNAMIC_SHARED_SIZE_BYTES,
                       static_cast<int>(sharedMemSize))))
      return 1;
    k->dynSmemLimit = static_cast<int>(sharedMemSize);
  }
  return dev->check(
      "cuLaunchKernel",
      cu.LaunchKernel(k->function, unsigned(gridSizes[0]),
                      unsigned(gridSizes[1]), unsigned(gridSizes[2]),
                      unsigned(blockSizes[0]), unsigned(blockSizes[1]),
                      unsigned(blockSizes[2]), unsigned(sharedMemSize),
                      q->stream, args, nullptr));
}

// ---- additions -----------------------------------------------------------

void *olxQueueNativeHandle(OlQueue queue) noexcept {
  auto *q = static_cast<QueueState *>(queue);
  return q ? q->stream : nullptr;
}

int olxMemcpyHtoD(OlQueue queue, void *dst, const void *src,
                  size_t size) noexcept {
  auto *q = static_cast<QueueState *>(queue);
  if (!q)
    return 1;
  ContextScope scope(q->device);
  if (!scope)
    return 1;
  return q->device->check(
      "cuMemcpyHtoDAsync",
      DriverApi::get().MemcpyHtoDAsync(reinterpret_cast<CUdeviceptr>(dst), src,
                                       size, q->stream));
}

int olxMemcpyDtoH(OlQueue queue, void *dst, const void *src,
                  size_t size) noexcept {
  auto *q = static_cast<QueueState *>(queue);
  if (!q)
    return 1;
  ContextScope scope(q->device);
  if (!scope)
    return 1;
  return q->device->check(
      "cuMemcpyDtoHAsync",
      DriverApi::get().MemcpyDtoHAsync(
          dst, reinterpret_cast<CUdeviceptr>(src), size, q->stream));
}

int olxMemsetD8(OlQueue queue, void *dst, int value, size_t size) noexcept {
  auto *q = static_cast<QueueState *>(queue);
  if (!q)
    return 1;
  ContextScope scope(q->device);
  if (!scope)
    return 1;
  return q->device->check(
      "cuMemsetD8Async",
      DriverApi::get().MemsetD8Async(reinterpret_cast<CUdeviceptr>(dst),
                                     static_cast<unsigned char>(value), size,
                                     q->stream));
}

int olxDeviceAttribute(OlDevice d, int what, long long *valueRet) noexcept {
  auto *dev = static_cast<DeviceState *>(d);
  if (!dev || !valueRet)
    return 1;
  CUdevice_attribute attr;
  switch (what) {
  case OLX_DEVICE_SM_COUNT:
    attr = CU_DEVICE_ATTRIBUTE_MULTIPROCESSOR_COUNT;
    break;
  case OLX_DEVICE_CC_MAJOR:
    attr = CU_DEVICE_ATTRIBUTE_COMPUTE_CAPABILITY_MAJOR;
    break;
  case OLX_DEVICE_CC_MINOR:
    attr = CU_DEVICE_ATTRIBUTE_COMPUTE_CAPABILITY_MINOR;
    break;
  case OLX_DEVICE_L2_BYTES:
    attr = CU_DEVICE_ATTRIBUTE_L2_CACHE_SIZE;
    break;
  case OLX_DEVICE_MAX_SMEM_OPTIN:
    attr = CU_DEVICE_ATTRIBUTE_MAX_SHARED_MEMORY_PER_BLOCK_OPTIN;
    break;
  case OLX_DEVICE_ORDINAL:
    *valueRet = dev->ordinal;
    return 0;
  default:
    dev->report(OlSeverity::Error, "Invalid device attribute: %d", what);
    return 1;
  }
  int value = 0;
  if (dev->check("cuDeviceGetAttribute", DriverApi::get().DeviceGetAttribute(
                                             &value, attr, dev->handle)))
    return 1;
  *valueRet = value;
  return 0;
}

int olxMaxActiveClusters(OlQueue queue, OlKernel kernel, unsigned blockThreads,
                         size_t sharedMemSize, unsigned clusterSize,
                         int *clustersRet) noexcept {
  auto *q = static_cast<QueueState *>(queue);
  auto *k = static_cast<KernelState *>(kernel);
  if (!q || !k || !clustersRet || clusterSize == 0)
    return 1;
  DeviceState *dev = q->device;
  const DriverApi &cu = DriverApi::get();
  ContextScope scope(dev);
  if (!scope)
    return 1;
  if (sharedMemSize > size_t(k->dynSmemLimit)) {
    if (dev->check("cuFuncSetAttribute",
                   cu.FuncSetAttribute(
                       k->function,
                       CU_FUNC_ATTRIBUTE_MAX_DYNAMIC_SHARED_SIZE_BYTES,
                       static_cast<int>(sharedMemSize))))
      return 1;
    k->dynSmemLimit = static_cast<int>(sharedMemSize);
  }
  CUlaunchAttribute attr{};
  attr.id = CU_LAUNCH_ATTRIBUTE_CLUSTER_DIMENSION;
  attr.value.clusterDim.x = clusterSize;
  attr.value.clusterDim.y = 1;
  attr.value.clusterDim.z = 1;
  CUlaunchConfig config{};
  config.gridDimX = clusterSize;
  config.gridDimY = 1;
  config.gridDimZ = 1;
  config.blockDimX = blockThreads;
  config.blockDimY = 1;
  config.blockDimZ = 1;
  config.sharedMemBytes = static_cast<unsigned>(sharedMemSize);
  config.hStream = q->stream;
  config.attrs = &attr;
  config.numAttrs = 1;
  return dev->check("cuOccupancyMaxActiveClusters",
                    cu.OccupancyMaxActiveClusters(clustersRet, k->function,
                                                  &config));
}

int olxEncodeTensorMapTiled(OlDevice d, void *mapOut, int elemKind, const void *base,
                            int rank, const size_t *dims, const size_t *stridesBytes,
                            const unsigned *box, int swizzle) noexcept {
  auto *dev = static_cast<DeviceState *>(d);
  if (!dev || !mapOut || !dims || !stridesBytes || !box)
    return 1;
  CUtensorMapDataType type;
  size_t elemBytes;
  switch (elemKind) {
  case 0:
    type = CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
    elemBytes = 2;
    break;
  case 1:
    type = CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
    elemBytes = 4;
    break;
  case 2:
    type = CU_TENSOR_MAP_DATA_TYPE_UINT8;
    elemBytes = 1;
    break;
  default:
    dev->report(OlSeverity::Error, "Invalid tensor map element kind: %d", elemKind);
    return 1;
  }
  bool ok = rank >= 2 && rank <= 5 && reinterpret_cast<uintptr_t>(base) % 16 == 0 &&
            reinterpret_cast<uintptr_t>(mapOut) % 64 == 0 && (swizzle == 0 || swizzle == 128);
  cuuint64_t d64[5] = {1, 1, 1, 1, 1}, s64[4] = {0, 0, 0, 0};
  cuuint32_t b32[5] = {1, 1, 1, 1, 1}, e32[5] = {1, 1, 1, 1, 1};
  for (int i = 0; ok && i < rank; ++i) {
    d64[i] = dims[i];
    b32[i] = box[i];
    ok = dims[i] > 0 && box[i] > 0 && box[i] <= 256;
    if (ok && i > 0) {
      s64[i - 1] = stridesBytes[i - 1];
      ok = stridesBytes[i - 1] % 16 == 0;
    }
  }
  ok = ok && (box[0] * elemBytes) % 16 == 0 && (swizzle != 128 || box[0] * elemBytes <= 128);
  if (!ok) {
    dev->report(OlSeverity::Error, "Invalid tensor map geometry: rank %d base %p swizzle %d",
                rank, base, swizzle);
    return 1;
  }
  ContextScope scope(dev);
  if (!scope)
    return 1;
  return dev->check(
      "cuTensorMapEncodeTiled",
      DriverApi::get().TensorMapEncodeTiled(
          static_cast<CUtensorMap *>(mapOut), type, cuuint32_t(rank), const_cast<void *>(base),
          d64, s64, b32, e32, CU_TENSOR_MAP_INTERLEAVE_NONE,
          swizzle == 128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
          CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE));
}

int olxEncodeTensorMap2D(OlDevice d, void *mapOut, int elemKind,
                         const void *base, size_t rows, size_t cols,
                         size_t rowPitchBytes, unsigned boxRows,
                         unsigned boxCols, int swizzle) noexcept {
  auto *dev = static_cast<DeviceState *>(d);
  if (!dev || !mapOut)
    return 1;
  CUtensorMapDataType type;
  size_t elemBytes;
  switch (elemKind) {
  case 0:
    type = CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
    elemBytes = 2;
    break;
  case 1:
    type = CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
    elemBytes = 4;
    break;
  case 2:
    type = CU_TENSOR_MAP_DATA_TYPE_UINT8;
    elemBytes = 1;
    break;
  default:
    dev->report(OlSeverity::Error, "Invalid tensor map element kind: %d",
                elemKind);
    return 1;
  }
  // The hardware wants a 16-byte aligned base, row pitches that are multiples
  // of 16 bytes and an inner box extent that is a multiple of 16 bytes.
  if (reinterpret_cast<uintptr_t>(base) % 16 || rowPitchBytes % 16 ||
      (boxCols * elemBytes) % 16 || boxRows == 0 || boxRows > 256 ||
      boxCols == 0 || boxCols > 256 ||
      (swizzle == 128 && boxCols * elemBytes > 128) ||
      (swizzle != 0 && swizzle != 128) ||
      reinterpret_cast<uintptr_t>(mapOut) % 64) {
    dev->report(OlSeverity::Error,
                "Invalid tensor map geometry: base %p pitch %zu box %ux%u "
                "swizzle %d",
                base, rowPitchBytes, boxRows, boxCols, swizzle);
    return 1;
  }
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {rowPitchBytes};
  cuuint32_t box[2] = {boxCols, boxRows};
  cuuint32_t elemStrides[2] = {1, 1};
  ContextScope scope(dev);
  if (!scope)
    return 1;
  return dev->check(
      "cuTensorMapEncodeTiled",
      DriverApi::get().TensorMapEncodeTiled(
          static_cast<CUtensorMap *>(mapOut), type, 2,
          const_cast<void *>(base), dims, strides, box, elemStrides,
          CU_TENSOR_MAP_INTERLEAVE_NONE,
          swizzle == 128 ? CU_TENSOR_MAP_SWIZZLE_128B
                         : CU_TENSOR_MAP_SWIZZLE_NONE,
          CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE));
}

int olxDeviceContextEnter(OlDevice d) noexcept {
  auto *dev = static_cast<DeviceState *>(d);
  if (!dev)
    return 1;
  return dev->check("cuCtxPushCurrent",
                    DriverApi::get().CtxPushCurrent(dev->context));
}

int olxDeviceContextLeave(OlDevice d) noexcept {
  auto *dev = static_cast<DeviceState *>(d);
  if (!dev)
    return 1;
  return dev->check("cuCtxPopCurrent", DriverApi::get().CtxPopCurrent(nullptr));
}

int olxPointerDevice(OlDevice d, const void *ptr, int *ordinalRet) noexcept {
  auto *dev = static_cast<DeviceState *>(d);
  if (!dev || !ordinalRet)
    return 1;
  *ordinalRet = -1;
  if (!ptr)
    return 0;
  ContextScope scope(dev);
  if (!scope)
    return 1;
  const DriverApi &cu = DriverApi::get();
  const auto address = reinterpret_cast<CUdeviceptr>(ptr);
  unsigned memoryType = 0;
  // A pointer the driver has never seen is not an error here: it is host memory.
  if (cu.PointerGetAttribute(&memoryType, CU_POINTER_ATTRIBUTE_MEMORY_TYPE,
                             address) != CUDA_SUCCESS ||
      memoryType != CU_MEMORYTYPE_DEVICE)
    return 0;
  int ordinal = -1;
  if (dev->check("cuPointerGetAttribute",
                 cu.PointerGetAttribute(&ordinal, CU_POINTER_ATTRIBUTE_DEVICE_ORDINAL,
                                        address)))
    return 1;
  *ordinalRet = ordinal;
  return 0;
}

OlxEvent olxCreateEvent(OlDevice d, int timing) noexcept {
  auto *dev = static_cast<DeviceState *>(d);
  if (!dev)
    return nullptr;
  ContextScope scope(dev);
  if (!scope)
    return nullptr;
  CUevent ev = nullptr;
  if (dev->check("cuEventCreate", DriverApi::get().EventCreate(
                                      &ev, timing ? CU_EVENT_DEFAULT : CU_EVENT_DISABLE_TIMING)))
    return nullptr;
  return ev;
}

void olxReleaseEvent(OlDevice d, OlxEvent ev) noexcept {
  auto *dev = static_cast<DeviceState *>(d);
  if (!dev || !ev)
    return;
  ContextScope scope(dev);
  if (scope)
    dev->check("cuEventDestroy", DriverApi::get().EventDestroy(static_cast<CUevent>(ev)));
}

int olxRecordEvent(OlQueue queue, OlxEvent ev) noexcept {
  auto *q = static_cast<QueueState *>(queue);
  if (!q || !ev)
    return 1;
  ContextScope scope(q->device);
  if (!scope)
    return 1;
  return q->device->check(
      "cuEventRecord", DriverApi::get().EventRecord(static_cast<CUevent>(ev), q->stream));
}

int olxQueueWaitEvent(OlQueue queue, OlxEvent ev) noexcept {
  auto *q = static_cast<QueueState *>(queue);
  if (!q || !ev)
    return 1;
  ContextScope scope(q->device);
  if (!scope)
    return 1;
  return q->device->check(
      "cuStreamWaitEvent",
      DriverApi::get().StreamWaitEvent(q->stream, static_cast<CUevent>(ev), 0));
}

int olxEventElapsedMs(OlDevice d, OlxEvent from, OlxEvent to, float *msRet) noexcept {
  auto *dev = static_cast<DeviceState *>(d);
  if (!dev || !from || !to || !msRet)
    return 1;
  ContextScope scope(dev);
  if (!scope)
    return 1;
  return dev->check("cuEventElapsedTime",
                    DriverApi::get().EventElapsedTime(msRet, static_cast<CUevent>(from),
                                                      static_cast<CUevent>(to)));
}

int olxHostRegister(OlDevice d, void *ptr, size_t size) noexcept {
  auto *dev = static_cast<DeviceState *>(d);
  if (!dev || !ptr || size == 0)
    return 1;
  ContextScope scope(dev);
  if (!scope)
    return 1;
  return dev->check("cuMemHostRegister",
                    DriverApi::get().MemHostRegister(ptr, size, CU_MEMHOSTREGISTER_PORTABLE));
}

int olxHostUnregister(OlDevice d, void *ptr) noexcept {
  auto *dev = static_cast<DeviceState *>(d);
  if (!dev || !ptr)
    return 1;
  ContextScope scope(dev);
  if (!scope)
    return 1;
  return dev->check("cuMemHostUnregister", DriverApi::get().MemHostUnregister(ptr));
}

} // extern "C"
