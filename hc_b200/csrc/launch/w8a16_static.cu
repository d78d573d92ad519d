// hcGemmW8A16Static: the int8 weight-only dequant GEMM for callers that must
// not allocate device memory.
//
// hcGemmW8A16 needs a scratch matrix (the weights converted to bf16) and asks
// its caller to provide it.  Some callers cannot: a serving loop whose device
// memory is carved up once at start-up and never grown, or a host application
// that lends this library a stream but owns every allocation itself.  For them
// cudaMalloc on the launch path is not an option - it synchronises the whole
// device, it can fail when memory is tight, and they simply may not be allowed
// to call it.  This entry point therefore brings its own scratch: a fixed
// array in the library's device image.  The price is a size limit (the
// converted weights must fit in kScratchBytes) and that every GPU which loads
// the library carries the array until the process exits.
//
// The scratch is one array shared by all calls on a device.  It is fully
// rewritten by the conversion step of each call before the GEMM reads it, so
// nothing in it has to start at zero and nothing needs clearing between
// calls; but two calls whose GPU work overlaps (different streams, no
// ordering between them) would convert into the same bytes and race.  Calls
// issued on one context are ordered by its queue and are safe.
//
// The first call on a device does set-up work - with the context's own CUDA
// context made current it asks the CUDA runtime for the device address of the
// array, and it makes sure the kernel images are loaded
// - and should therefore be made before any stream capture is started on the
// context's stream.  After that the entry point calls no cudaMalloc, cudaFree
// or any other allocating routine: it looks up a cached pointer and launches.
#include "hc_b200_kernels.h"

#include <cuda_runtime.h>

#include <cstdio>
#include <mutex>

namespace {

// 32 MiB: room for K x N = 4096 x 4096 bf16 weights (N rounded up to 16).
constexpr size_t kScratchBytes = 32u << 20;
constexpr int kMaxDevices = 64;

// Lives in the device image of this library; on the host this name is only a
// handle for cudaGetSymbolAddress, never a usable address.
static __device__ __align__(256) unsigned char hcW8A16Scratch[kScratchBytes];

std::mutex setupLock;
void *scratchOnDevice[kMaxDevices]; // device address of the array, per ordinal

// Device address of the scratch array on the context's GPU, resolved once per
// GPU.  The context's own primary context is made current for the look-up (a
// push and a pop through the backend), so the calling thread's device is never
// changed and no other GPU is touched.  Returns nullptr and fills `why` on
// failure.
void *scratchAddress(HcContext c, int ordinal, char *why, size_t whyLen) {
  std::lock_guard<std::mutex> lock(setupLock);
  if (scratchOnDevice[ordinal])
    return scratchOnDevice[ordinal];
  OlDevice dev = hcContextDevice(c);
  if (olxDeviceContextEnter(dev)) {
    snprintf(why, whyLen, "hcGemmW8A16Static: could not make the context's device current");
    return nullptr;
  }
  void *ptr = nullptr;
  const cudaError_t rc = cudaGetSymbolAddress(&ptr, hcW8A16Scratch);
  olxDeviceContextLeave(dev);
  if (rc != cudaSuccess || !ptr) {
    snprintf(why, whyLen, "cudaGetSymbolAddress for the static scratch failed: %s",
             cudaGetErrorString(rc));
    return nullptr;
  }
  scratchOnDevice[ordinal] = ptr;
  return ptr;
}

} // namespace

extern "C" {

size_t hcGemmW8A16StaticMaxBytes(void) { return kScratchBytes; }

int hcGemmW8A16Static(HcContext c, const void *a, const void *w,
                      const float *scale, void *out, long long M, long long N,
                      long long K, long long lda, long long ldw,
                      long long ldc) {
  if (!c)
    return 1;
  char why[256];
  const size_t need = hcGemmW8A16WorkspaceBytes(N, K);
  if (need > kScratchBytes) {
    snprintf(why, sizeof(why),
             "hcGemmW8A16Static: weights of %lld x %lld need %zu bytes of scratch, the "
             "built-in scratch holds %zu; use hcGemmW8A16 with a caller-provided workspace",
             K, N, need, kScratchBytes);
    return hcReportError(c, why);
  }
  if (M <= 0 || N <= 0 || K <= 0) // nothing to convert; let the common path validate
    return hcGemmW8A16(c, a, w, scale, out, nullptr, 0, M, N, K, lda, ldw, ldc);
  // The scratch is the array of the context's GPU, and `out` must live there
  // too: a context never launches against another GPU's copy of the array.
  OlDevice dev = hcContextDevice(c);
  long long ordinal = -1;
  if (olxDeviceAttribute(dev, OLX_DEVICE_ORDINAL, &ordinal) || ordinal < 0 ||
      ordinal >= kMaxDevices)
    return hcReportError(c, "hcGemmW8A16Static: the context's device has no usable ordinal");
  int owner = -1;
  if (olxPointerDevice(dev, out, &owner))
    return 1;
  if (owner < 0)
    return hcReportError(c, "hcGemmW8A16Static: `out` is not a device pointer");
  if (owner != int(ordinal)) {
    snprintf(why, sizeof(why),
             "hcGemmW8A16Static: `out` lives on cuda:%d but the context drives cuda:%lld",
             owner, ordinal);
    return hcReportError(c, why);
  }
  void *scratch = scratchAddress(c, int(ordinal), why, sizeof(why));
  if (!scratch)
    return hcReportError(c, why);
  return hcGemmW8A16(c, a, w, scale, out, scratch, kScratchBytes, M, N, K, lda, ldw, ldc);
}

} // extern "C"
