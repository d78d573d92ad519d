// libhc-b200-kernels.so: owns the precompiled sm_100a images and launches the
// workload kernels through the ol* ABI of the loader.
//
// This is the host side that the reference generates with its JIT: create the
// module from a blob, look the kernel up, pack `void *args[]`, launch
// (mlir/lib/Transforms/GpuToGpuRuntime.cpp:163-309 emits that sequence;
// python/cpp/py-runtime/src/GpuRuntime.cpp:26-69 executes it).  Here the blobs
// are fixed, so the sequence is ordinary C++ and each workload gets a typed
// entry point that validates its arguments and chooses a kernel variant.
#include "context.hpp"

#include "../kernels/fused_programs.h"
#include "../kernels/conv_params.h"
#include "../kernels/gemm_band_params.h"
#include "../kernels/items_params.h"
#include "../kernels/map_params.h"
#include "../kernels/mapped_params.h"
#include "../kernels/peer_params.h"

#include <cuda.h> // CUtensorMap (type only; no driver call is made here)
#include <dlfcn.h>

#include <algorithm>
#include <cstdarg>
#include <cstddef>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <map>
#include <memory>
#include <string>
#include <vector>

// Loader-only export (gpu-runtime/loader/src/Loader.cpp:20-39 in the
// reference); declared here because offload_api.h covers the shared ABI only.
extern "C" void setGPULoaderSearchPaths(const char *paths[], size_t count);

// ---- embedded images (images_gen.S) -------------------------------------------
struct HcImage {
  const char *name;
  const unsigned char *begin;
  const unsigned char *end;
};
extern "C" const HcImage hc_b200_images[];
extern "C" const int hc_b200_image_count;

namespace {

struct KernelEntry {
  const char *kernel;
  const char *image;
};

// Which image defines which kernel.
const KernelEntry kKernelTable[] = {
    {"hc_copy2d", "copy2d"},
    // hc_map_elements_{f32_v4,f32_v1,f64_v2,f64_v1}_n{1..4}[i]: element type, packet
    // width, number of input arrays, and whether element indices are operands.
    {"hc_map_elements_", "map_elements"},
    // hc_row_program_{f32_v4,f32_v1,f64_v2,f64_v1}_n{1,2} (a warp walks the row) and
    // hc_row_program_held_{f32_v4,f64_v2}_p{8_t64,8_t96,8_t128,4_t256}_n{1,2} (a CTA
    // holds the row: packets per thread, threads).
    {"hc_row_program_", "row_program"},
    // hc_row_fused_<body>_{f32_held_t64,f32_held_t128,f32_v4,f32_v1,f64_v2,f64_v1} and
    // hc_map_fused_<body>_{f32_v4,f32_v1,f64_v2,f64_v1}: the bodies of
    // fused_programs.h compiled ahead of time.
    {"hc_conv_f32_taps", "conv_f32_taps"},
    {"hc_conv_f32_rows", "conv_f32_taps"},
    {"hc_split_tf32_nhwc", "conv_f32_taps"},
    {"hc_work_items_f32", "work_items"},
    {"hc_work_items_f64", "work_items"},
    {"hc_row_fused_", "row_fused"},
    {"hc_map_fused_", "map_fused"},
    {"hc_softmax_rows_f32_w1", "softmax_rows"},
    {"hc_softmax_rows_f32_w2", "softmax_rows"},
    {"hc_softmax_rows_f32_w4", "softmax_rows"},
    {"hc_softmax_rows_f32_w8", "softmax_rows"},
    {"hc_softmax_rows_f32_w16", "softmax_rows"},
    {"hc_softmax_rows_f32_w32", "softmax_rows"},
    {"hc_softmax_rows_f32_w1_peers", "softmax_rows"},
    {"hc_softmax_rows_f32_w2_peers", "softmax_rows"},
    {"hc_softmax_rows_f32_w4_peers", "softmax_rows"},
    {"hc_softmax_rows_f32_w8_peers", "softmax_rows"},
    {"hc_softmax_rows_f32_w16_peers", "softmax_rows"},
    {"hc_softmax_rows_f32_w32_peers", "softmax_rows"},
    {"hc_reduce_rows_warp_f32_peers", "reduce_rows"},
    {"hc_softmax_rows_f32_tma_v16", "softmax_rows"},
    {"hc_softmax_rows_f32_tma_v32", "softmax_rows"},
    {"hc_softmax_rows_generic_f32", "softmax_rows"},
    {"hc_softmax_rows_generic_f64", "softmax_rows"},
    {"hc_reduce_rows_warp_f32", "reduce_rows"},
    {"hc_reduce_rows_warp_f64", "reduce_rows"},
    {"hc_reduce_rows_block_f32", "reduce_rows"},
    {"hc_reduce_rows_block_f64", "reduce_rows"},
    {"hc_reduce_all_f32_f32", "reduce_all"},
    {"hc_reduce_all_f32_f64", "reduce_all"},
    {"hc_reduce_all_f64_f64", "reduce_all"},
    {"hc_reduce_all_f64_f32", "reduce_all"},
    {"hc_reduce_all_i32_f32", "reduce_all"},
    {"hc_reduce_all_i32_f64", "reduce_all"},
    {"hc_reduce_all_i64_f32", "reduce_all"},
    {"hc_reduce_all_i64_f64", "reduce_all"},
    {"hc_selftest_wait_timeout", "selftest"},
    {"hc_pairwise_distance_f32", "pairwise_distance"},
    {"hc_pairwise_distance_f64", "pairwise_distance"},
    // hc_mapped_gemm_{f32,f64}_{8,16,32,64}x{8,16,32,64}: one per piece shape.
    {"hc_mapped_gemm_", "mapped_gemm"},
    {"hc_gemm_tiled_f32", "gemm_tiled"},
    {"hc_gemm_tiled_f32_async", "gemm_tiled"},
    {"hc_gemm_tiled_f32_splitk", "gemm_tiled"},
    {"hc_gemm_tiled_f64", "gemm_tiled"},
    {"hc_gemm_tiled_bf16", "gemm_tiled"},
    {"hc_gemm_tiled_w8a16", "gemm_tiled"},
    {"hc_gemm_bf16_umma", "gemm_bf16_umma"},
    {"hc_gemm_bf16_umma_scaled", "gemm_bf16_umma"},
    {"hc_gemm_bf16_umma_pair", "gemm_bf16_umma"},
    {"hc_gemm_bf16_umma_pair_scaled", "gemm_bf16_umma"},
    {"hc_gemm_bf16_umma_peers", "gemm_bf16_umma"},
    {"hc_gemm_bf16_umma_scaled_peers", "gemm_bf16_umma"},
    {"hc_gemm_bf16_umma_pair_peers", "gemm_bf16_umma"},
    {"hc_gemm_bf16_umma_pair_scaled_peers", "gemm_bf16_umma"},
    {"hc_dequant_w8_bf16", "dequant_w8"},
    {"hc_split_tf32", "gemm_f32_umma"},
    {"hc_split_tf32_t", "gemm_f32_umma"},
    {"hc_gemm_f32_umma", "gemm_f32_umma"},
    {"hc_gemm_f32_umma_pair", "gemm_f32_umma"},
    {"hc_gemm_w8a16_umma_pair", "gemm_w8a16_umma"},
    {"hc_gemm_w8a16_umma_banded", "gemm_bf16_umma"},
    {"hc_conv_f32_umma", "conv_f32_umma"},
    {"hc_conv_f32_umma_ta", "conv_f32_umma"},
    {"hc_split_tf32_pairs", "conv_f32_umma"},
};

// Image that defines `kernel`; a table entry ending in '_' stands for every
// kernel whose name starts with it.
const char *imageOfKernel(const char *kernel) {
  for (const auto &e : kKernelTable) {
    const size_t n = std::strlen(e.kernel);
    if (n && e.kernel[n - 1] == '_' ? std::strncmp(e.kernel, kernel, n) == 0
                                    : std::strcmp(e.kernel, kernel) == 0)
      return e.image;
  }
  return nullptr;
}

int findImage(const char *name) {
  for (int i = 0; i < hc_b200_image_count; ++i)
    if (std::strcmp(hc_b200_images[i].name, name) == 0)
      return i;
  return -1;
}

long long ceilDiv(long long a, long long b) { return (a + b - 1) / b; }
long long roundUp(long long a, long long b) { return ceilDiv(a, b) * b; }
bool aligned(const void *p, size_t a) {
  return reinterpret_cast<uintptr_t>(p) % a == 0;
}

// Geometry of the tensor-core GEMM kernels (gemm_bf16_umma.cu).
constexpr int kUmmaBM = 128, kUmmaBN = 256, kUmmaBK = 64;
constexpr int kUmmaThreads = 192;
// The banded dequantising GEMM: converted columns per band, bands in its ring.
constexpr int kBandCols = 1024, kBandSlots = 3;
constexpr size_t kUmmaSmemBytes = 4 * 48 * 1024 /*stages*/ + 1024 /*align*/ +
                                  512 /*barriers*/;

// Programs that exist as precompiled straight-line kernels (fused_programs.h).
struct FusedProgram {
  const char *name;
  int nin, n;
  const uint32_t *code;
};
#define HC_FUSED_ENTRY(body)                                                             \
  {#body, hcfused::row_##body::nin, hcfused::row_##body::n, hcfused::row_##body::code},
const FusedProgram kFusedRows[] = {HC_FUSED_ROW_LIST(HC_FUSED_ENTRY)};
#undef HC_FUSED_ENTRY
#define HC_FUSED_ENTRY(body)                                                             \
  {#body, hcfused::map_##body::nin, hcfused::map_##body::n, hcfused::map_##body::code},
const FusedProgram kFusedMaps[] = {HC_FUSED_MAP_LIST(HC_FUSED_ENTRY)};
#undef HC_FUSED_ENTRY

// Name of the precompiled body whose instruction words are exactly those of
// `p` (constants are operands and not compared), or nullptr.
template <size_t N>
const char *matchFused(const FusedProgram (&table)[N], const HcMapProgramDev &p) {
  for (const FusedProgram &f : table)
    if (f.nin == p.nInputs && f.n == p.nInstr &&
        std::equal(f.code, f.code + f.n, p.code))
      return f.name;
  return nullptr;
}

// hcRowProgram holds a row in a CTA's registers when the row fills at least
// this share of the CTA's packet slots.
constexpr int kRowHeldFillPercent = 90;

} // namespace

OlKernel HcContextImpl::kernel(const char *name) {
  auto it = kernels.find(name);
  if (it != kernels.end())
    return it->second;
  const char *imageName = imageOfKernel(name);
  int idx = imageName ? findImage(imageName) : -1;
  if (idx < 0) {
    fail("Unknown kernel: %s", name);
    return nullptr;
  }
  if (!modules[idx]) {
    const HcImage &img = hc_b200_images[idx];
    modules[idx] = olCreateModule(device, img.begin, size_t(img.end - img.begin));
    if (!modules[idx]) {
      fail("olCreateModule failed for image %s: %s", img.name,
           lastError.c_str());
      return nullptr;
    }
  }
  OlKernel k = olGetKernel(modules[idx], name);
  if (!k) {
    fail("olGetKernel failed for %s: %s", name, lastError.c_str());
    return nullptr;
  }
  kernels[name] = k;
  return k;
}

int HcContextImpl::launch(const char *name, size_t gx, size_t gy, size_t gz, size_t threads,
                        void **args, size_t nArgs, size_t smem) {
  OlKernel k = kernel(name);
  if (!k)
    return 1;
  const size_t grid[3] = {gx, gy, gz};
  const size_t block[3] = {threads, 1, 1};
  if (olLaunchKernel(queue, k, grid, block, 3, args, nArgs, smem))
    return fail("olLaunchKernel failed for %s: %s", name, lastError.c_str());
  ++launches;
  return 0;
}

namespace {

// Directory this shared library was loaded from; the backend library lives
// next to it.
std::string ownDirectory() {
  Dl_info info;
  if (!dladdr(reinterpret_cast<const void *>(&hcImageCount), &info) ||
      !info.dli_fname)
    return ".";
  std::string path(info.dli_fname);
  auto slash = path.rfind('/');
  return slash == std::string::npos ? "." : path.substr(0, slash);
}

} // namespace

extern "C" {

int hcImageCount(void) { return hc_b200_image_count; }

const char *hcImageName(int index) {
  return index >= 0 && index < hc_b200_image_count ? hc_b200_images[index].name
                                                   : nullptr;
}

const void *hcImageData(int index, size_t *lenRet) {
  if (index < 0 || index >= hc_b200_image_count)
    return nullptr;
  if (lenRet)
    *lenRet = size_t(hc_b200_images[index].end - hc_b200_images[index].begin);
  return hc_b200_images[index].begin;
}

int hcImageOfKernel(const char *kernelName) {
  if (!kernelName)
    return -1;
  const char *image = imageOfKernel(kernelName);
  return image ? findImage(image) : -1;
}

HcContext hcCreateContext(const char *deviceDesc, OlErrorCallback errCallback,
                          void *ctx) {
  auto c = std::make_unique<HcContextImpl>();
  c->callback = errCallback;
  c->callbackCtx = ctx;
  c->modules.assign(size_t(hc_b200_image_count), nullptr);

  static const std::string dir = ownDirectory();
  const char *paths[1] = {dir.c_str()};
  setGPULoaderSearchPaths(paths, 1);

  c->device = olCreateDevice(deviceDesc, &HcContextImpl::onBackendMessage, c.get());
  if (!c->device)
    return nullptr;
  c->queue = olCreateQueue(c->device);
  if (!c->queue) {
    olReleaseDevice(c->device);
    return nullptr;
  }
  olxDeviceAttribute(c->device, OLX_DEVICE_SM_COUNT, &c->smCount);
  olxDeviceAttribute(c->device, OLX_DEVICE_CC_MAJOR, &c->ccMajor);
  olxDeviceAttribute(c->device, OLX_DEVICE_CC_MINOR, &c->ccMinor);
  if (c->smCount <= 0)
    c->smCount = 1;
  c->statusWord = static_cast<int *>(olAllocDevice(c->queue, 256, 256));
  if (!c->statusWord || olxMemsetD8(c->queue, c->statusWord, 0, 256) ||
      olSyncQueue(c->queue)) {
    hcReleaseContext(c.release());
    return nullptr;
  }
  return c.release();
}

void hcReleaseContext(HcContext c) {
  if (!c)
    return;
  if (c->queue)
    olSyncQueue(c->queue);
  for (auto &kv : c->kernels)
    olReleaseKernel(kv.second);
  for (OlModule m : c->modules)
    if (m)
      olReleaseModule(m);
  hcReleaseHostPipeline(c);
  hcReleaseSpecialiser(c);
  if (c->statusWord)
    olDeallocDevice(c->queue, c->statusWord);
  if (c->queue)
    olReleaseQueue(c->queue);
  if (c->device)
    olReleaseDevice(c->device);
  delete c;
}

OlDevice hcContextDevice(HcContext c) { return c ? c->device : nullptr; }
OlQueue hcContextQueue(HcContext c) { return c ? c->queue : nullptr; }
void *hcContextStream(HcContext c) {
  return c ? olxQueueNativeHandle(c->queue) : nullptr;
}
int hcSynchronize(HcContext c) { return c ? olSyncQueue(c->queue) : 1; }
const char *hcLastError(HcContext c) { return c ? c->lastError.c_str() : ""; }
long long hcLaunchCount(HcContext c) { return c ? c->launches : 0; }

long long hcSpecialisedPrograms(HcContext c, int fromDisk) {
  return c ? hcSpecialiserCount(c, fromDisk ? 1 : 0) : 0;
}

const char *hcSpecialiseNote(HcContext c) { return c ? hcSpecialiserNote(c) : ""; }

int hcKernelStatus(HcContext c, int *statusRet) {
  if (!c || !statusRet)
    return 1;
  int value = 0;
  if (olxMemcpyDtoH(c->queue, &value, c->statusWord, sizeof(int)) ||
      olSyncQueue(c->queue))
    return c->fail("reading the kernel status word failed: %s",
                   c->lastError.c_str());
  if (value != 0 && (olxMemsetD8(c->queue, c->statusWord, 0, sizeof(int)) ||
                     olSyncQueue(c->queue)))
    return 1;
  *statusRet = value;
  return 0;
}

int hcSelfTestWaitTimeout(HcContext c, unsigned long long limitNs, int *statusRet,
                          unsigned long long *elapsedNsRet, int observedRet[2]) {
  if (!c || !statusRet || !elapsedNsRet || !observedRet)
    return 1;
  if (limitNs == 0 || limitNs > 1000000000ull)
    return c->fail("hcSelfTestWaitTimeout: limit must be between 1 ns and 1 s");
  // Scratch: [0] elapsed ns (8 bytes), [8..16) the two observed flags.
  auto *scratch = static_cast<unsigned char *>(olAllocDevice(c->queue, 256, 256));
  if (!scratch)
    return c->fail("hcSelfTestWaitTimeout: allocation failed: %s", c->lastError.c_str());
  int rc = olxMemsetD8(c->queue, scratch, 0xff, 256);
  auto *elapsed = reinterpret_cast<unsigned long long *>(scratch);
  auto *observed = reinterpret_cast<int *>(scratch + 8);
  void *args[] = {&limitNs, &c->statusWord, &elapsed, &observed};
  rc = rc || c->launch("hc_selftest_wait_timeout", 1, 1, 1, 64, args, 4, 0);
  unsigned char host[16] = {0};
  rc = rc || olxMemcpyDtoH(c->queue, host, scratch, sizeof(host)) || olSyncQueue(c->queue);
  olDeallocDevice(c->queue, scratch);
  if (rc)
    return c->fail("hcSelfTestWaitTimeout failed: %s", c->lastError.c_str());
  std::memcpy(elapsedNsRet, host, 8);
  std::memcpy(observedRet, host + 8, 8);
  return hcKernelStatus(c, statusRet);
}

int hcReportError(HcContext c, const char *text) {
  return c ? c->fail("%s", text ? text : "") : 1;
}

int hcSetOption(HcContext c, const char *name, long long value) {
  if (!c || !name)
    return 1;
  if (std::strcmp(name, "gemm_variant") == 0 && value >= 0 && value <= 3) {
    c->gemmVariant = value;
    return 0;
  }
  if (std::strcmp(name, "softmax_variant") == 0 && value >= 0 && value <= 2) {
    c->softmaxVariant = value;
    return 0;
  }
  if (std::strcmp(name, "reduce_variant") == 0 && value >= 0 && value <= 1) {
    c->reduceVariant = value; // 1: persistent grid for the warp-per-row kernel
    return 0;
  }
  if (std::strcmp(name, "tiled_variant") == 0 && value >= 0 && value <= 2) {
    // 1: never use the cp.async pipelined fp32 kernel; 2: use it, but never
    // split K over a cluster.
    c->tiledVariant = value;
    return 0;
  }
  if (std::strcmp(name, "mapped_stack") == 0 && value >= 0 && value <= 2) {
    // 1: one work-group per CTA even where groups share a tile; 2: stacks of at
    // most 64 rows.
    c->mappedStack = value;
    return 0;
  }
  if (std::strcmp(name, "fused") == 0 && value >= 0 && value <= 1) {
    c->fusedVariant = value; // 1: interpret every program, precompiled or not
    return 0;
  }
  if (std::strcmp(name, "gemm_band") == 0 && value >= 0 && value <= 64) {
    // Row tiles per band of the tcgen05 GEMMs' tile order (0: the default).
    c->gemmBand = value;
    return 0;
  }
  if (std::strcmp(name, "conv_variant") == 0 && value >= 0 && value <= 4) {
    // hcConvF32Tensor: 1 = the image operand through shared memory, 2 = through
    // tensor memory (at most 128 filters), 0 = tensor memory where it fits.
    c->convVariant = value;
    return 0;
  }
  if (std::strcmp(name, "w8a16_variant") == 0 && value >= 0 && value <= 3) {
    // hcGemmW8A16: 0 and 1 = the weights are converted in a pass of their own (needs
    // the workspace; the faster form at the benchmark size), 2 = inside the GEMM's
    // pipeline (no workspace; fails where the layout does not allow it), 3 = inside
    // the GEMM kernel band by band, by warps of their own (the first
    // hcGemmW8A16BandedBytes of the workspace; fails where the layout does not allow it).
    c->w8Variant = value;
    return 0;
  }
  if (std::strcmp(name, "conv_stacked") == 0 && value >= 0 && value <= 1) {
    c->convStacked = value; // 1: hcConvF32Tensor never stacks b_hi and b_lo into one MMA
    return 0;
  }
  if (std::strcmp(name, "conv_stages") == 0 && (value == 0 || (value >= 2 && value <= 6))) {
    c->convStages = value; // hcConvF32Tensor: fewer stages leave more of the SM's L1
    return 0;
  }
  if (std::strcmp(name, "specialise") == 0 && value >= 0 && value <= 2) {
    // 0: programs without a precompiled body are interpreted; 1: they are compiled
    // at their first launch, and interpreted where that is not possible; 2: as 1,
    // but the launch fails where it is not possible.
    c->specialiseMode = value;
    return 0;
  }
  if (std::strcmp(name, "row_variant") == 0 && value >= 0 && value <= 3) {
    c->rowVariant = value; // see hcRowProgram
    return 0;
  }
  return c->fail("Invalid option: %s = %lld", name, value);
}

// ---- copy -----------------------------------------------------------------------
int hcCopy2D(HcContext c, const void *src, void *dst, long long rows,
             long long cols, long long srcPitch, long long dstPitch,
             int elemBytes) {
  if (!c)
    return 1;
  if (elemBytes != 1 && elemBytes != 2 && elemBytes != 4 && elemBytes != 8)
    return c->fail("hcCopy2D: unsupported element size %d", elemBytes);
  if (rows < 0 || cols < 0 || srcPitch < cols || dstPitch < cols)
    return c->fail("hcCopy2D: invalid shape %lld x %lld (pitch %lld -> %lld)",
                   rows, cols, srcPitch, dstPitch);
  if (rows == 0 || cols == 0)
    return 0;
  if (!src || !dst)
    return c->fail("hcCopy2D: null buffer");
  long long rowBytes = cols * elemBytes;
  long long sp = srcPitch * elemBytes, dp = dstPitch * elemBytes;
  // A fully contiguous matrix is one long row.
  if (sp == rowBytes && dp == rowBytes) {
    rowBytes *= rows;
    sp = dp = rowBytes;
    rows = 1;
  }
  int packet = 16;
  while (packet > elemBytes &&
         (rowBytes % packet || sp % packet || dp % packet ||
          !aligned(src, packet) || !aligned(dst, packet)))
    packet >>= 1;
  long long perRow = rowBytes / packet;
  long long gx = std::min<long long>(ceilDiv(perRow, 256 * 4), c->smCount * 8);
  gx = std::max<long long>(gx, 1);
  long long gy = std::min<long long>(rows, std::max<long long>(1, c->smCount * 8 / gx));
  void *args[] = {&src, &dst, &rows, &rowBytes, &sp, &dp, &packet};
  return c->launch("hc_copy2d", size_t(gx), size_t(gy), 1, 256, args, 7, 0);
}

// ---- element-wise expressions -------------------------------------------------------
static_assert(sizeof(HcMapProgram) == sizeof(HcMapProgramDev) &&
                  offsetof(HcMapProgram, out) == offsetof(HcMapProgramDev, out) &&
                  offsetof(HcMapProgram, rows) == offsetof(HcMapProgramDev, rows) &&
                  offsetof(HcMapProgram, nInputs) == offsetof(HcMapProgramDev, nInputs) &&
                  offsetof(HcMapProgram, code) == offsetof(HcMapProgramDev, code) &&
                  offsetof(HcMapProgram, consts) == offsetof(HcMapProgramDev, consts),
              "public program description and kernel parameter block differ");

// Checks a program before it reaches the GPU: known operations, operands that
// exist, temporaries and row scalars written before they are read, an
// accumulator that is loaded before it is used.  `rowProgram`: reductions and
// row scalars are allowed (and a last pass that stores is required); element
// indices are not.
static int checkMapProgram(HcContext c, const char *who, const HcMapProgramDev &p,
                           bool rowProgram, bool *usesIndices, bool integer = false) {
  bool saved[3] = {false, false, false};
  bool reduced[HC_MAP_MAX_SCALARS] = {false, false, false, false};
  bool passStart = true;
  bool uniformLoaded = false; // inside a uniform prologue: its accumulator holds a value
  for (int pc = 0; pc < p.nInstr; ++pc) {
    const uint32_t src = p.code[pc] >> 8;
    uint32_t op = p.code[pc] & 0xffu;
    if (op & HC_MAP_UNIFORM) {
      // One value per row, computed before the pass walks the row.
      op &= 0x7fu;
      if (!rowProgram)
        return c->fail("%s: uniform instructions belong to hcRowProgram (instruction %d)", who,
                       pc);
      if (!passStart)
        return c->fail("%s: uniform instruction %d is not at the start of a pass", who, pc);
      if (pc == p.nInstr - 1)
        return c->fail("%s: the program ends in a uniform instruction; a last pass must compute "
                       "what is stored",
                       who);
      const bool arithmetic = op <= HC_MAP_SQRT || op == HC_MAP_LOG;
      if (!arithmetic && op != HC_MAP_SET)
        return c->fail("%s: operation %u cannot be uniform (instruction %d)", who, op, pc);
      if (op != HC_MAP_LOAD && !uniformLoaded)
        return c->fail("%s: uniform instruction %d uses an accumulator that holds nothing", who,
                       pc);
      if (op <= HC_MAP_MIN) {
        const bool constant =
            src >= HC_MAP_SRC_CONST && src < HC_MAP_SRC_CONST + uint32_t(HC_MAP_MAX_CONSTS);
        const bool scalar = src >= HC_MAP_SRC_SCALAR &&
                            src < HC_MAP_SRC_SCALAR + uint32_t(HC_MAP_MAX_SCALARS) &&
                            reduced[src - HC_MAP_SRC_SCALAR];
        if (!constant && !scalar)
          return c->fail("%s: uniform instruction %d reads operand %u; only constants and row "
                         "scalars that are already set can be read there",
                         who, pc, src);
      }
      uniformLoaded = true;
      if (op == HC_MAP_SET) {
        if (src >= uint32_t(HC_MAP_MAX_SCALARS))
          return c->fail("%s: instruction %d sets row scalar %u of %d", who, pc, src,
                         HC_MAP_MAX_SCALARS);
        reduced[src] = true;
        uniformLoaded = false;
      }
      continue;
    }
    if (op >= HC_MAP_OP_COUNT || op == HC_MAP_SET)
      return c->fail("%s: unknown operation %u at instruction %d", who, op, pc);
    if (rowProgram && op >= HC_MAP_FLOORDIV)
      return c->fail("%s: operation %u (instruction %d) belongs to hcMapElements", who, op, pc);
    if (integer && (op == HC_MAP_DIV || op == HC_MAP_RDIV || op == HC_MAP_EXP ||
                    op == HC_MAP_SQRT || op == HC_MAP_LOG || op == HC_MAP_RPOW))
      return c->fail("%s: operation %u (instruction %d) is not defined on integer arrays", who,
                     op, pc);
    if (!integer && op >= HC_MAP_SHL && op <= HC_MAP_RSHR)
      return c->fail("%s: shifts (instruction %d) are defined on integer arrays only", who, pc);
    if (passStart && op != HC_MAP_LOAD)
      return c->fail(pc == 0 ? "%s: the first instruction must load the accumulator"
                             : "%s: the instruction after a reduction must load the accumulator",
                     who);
    passStart = false;
    if (hcMapIsBinary(op)) {
      const bool input = src < uint32_t(p.nInputs);
      const bool temp = src >= HC_MAP_SRC_TEMP && src < HC_MAP_SRC_TEMP + 3 &&
                        saved[src - HC_MAP_SRC_TEMP];
      const bool constant =
          src >= HC_MAP_SRC_CONST && src < HC_MAP_SRC_CONST + uint32_t(HC_MAP_MAX_CONSTS);
      const bool index = !rowProgram && (src == HC_MAP_SRC_ROW || src == HC_MAP_SRC_COL);
      const bool scalar = rowProgram && src >= HC_MAP_SRC_SCALAR &&
                          src < HC_MAP_SRC_SCALAR + uint32_t(HC_MAP_MAX_SCALARS) &&
                          reduced[src - HC_MAP_SRC_SCALAR];
      *usesIndices = *usesIndices || index;
      if (!input && !temp && !constant && !index && !scalar)
        return c->fail("%s: instruction %d reads operand %u, which does not exist "
                       "or is not written yet",
                       who, pc, src);
      if (integer && constant) {
        const double value = p.consts[src - HC_MAP_SRC_CONST];
        if (value != double((long long)value) || value < -9.2e18 || value > 9.2e18)
          return c->fail("%s: constant %g (instruction %d) is not an integer", who, value, pc);
        if (op == HC_MAP_POW && value < 0)
          return c->fail("%s: integers to negative integer powers are not allowed "
                         "(instruction %d)",
                         who, pc);
      }
      if (integer && op == HC_MAP_POW && !constant)
        return c->fail("%s: integer arrays take constant exponents only (instruction %d)", who,
                       pc);
    }
    if (op >= HC_MAP_SAVE0 && op <= HC_MAP_SAVE2)
      saved[op - HC_MAP_SAVE0] = true;
    if (op == HC_MAP_RSUM || op == HC_MAP_RMAX) {
      if (!rowProgram)
        return c->fail("%s: row reductions belong to hcRowProgram (instruction %d)", who, pc);
      if (src >= uint32_t(HC_MAP_MAX_SCALARS))
        return c->fail("%s: instruction %d reduces into row scalar %u of %d", who, pc, src,
                       HC_MAP_MAX_SCALARS);
      if (pc == p.nInstr - 1)
        return c->fail("%s: the program ends in a reduction; a last pass must compute what is "
                       "stored",
                       who);
      reduced[src] = true;
      passStart = true;
      // Temporaries do not outlive a pass (every pass walks the row again).
      saved[0] = saved[1] = saved[2] = false;
    }
  }
  return 0;
}

int hcMapElements(HcContext c, const HcMapProgram *program, int dtype) {
  if (!c)
    return 1;
  if (dtype != HC_F32 && dtype != HC_F64 && dtype != HC_I32 && dtype != HC_I64)
    return c->fail("hcMapElements: unsupported dtype %d", dtype);
  const bool integer = dtype == HC_I32 || dtype == HC_I64;
  if (!program)
    return c->fail("hcMapElements: null program");
  HcMapProgramDev p;
  std::memcpy(&p, program, sizeof p);
  if (p.nInputs < 0 || p.nInputs > HC_MAP_MAX_INPUTS || p.nInstr < 1 ||
      p.nInstr > HC_MAP_MAX_INSTR)
    return c->fail("hcMapElements: %d inputs, %d instructions (at most %d and 1..%d)", p.nInputs,
                   p.nInstr, HC_MAP_MAX_INPUTS, HC_MAP_MAX_INSTR);
  bool usesIndices = false;
  if (checkMapProgram(c, "hcMapElements", p, false, &usesIndices, integer))
    return 1;
  if (p.rows < 0 || p.cols < 0 || p.outPitch < p.cols)
    return c->fail("hcMapElements: invalid shape %lld x %lld", (long long)p.rows,
                   (long long)p.cols);
  for (int k = 0; k < p.nInputs; ++k)
    if (p.inPitch[k] < p.cols)
      return c->fail("hcMapElements: pitch of input %d is shorter than a row", k);
  if (p.rows == 0 || p.cols == 0)
    return 0;
  if (!p.out)
    return c->fail("hcMapElements: null output");
  for (int k = 0; k < p.nInputs; ++k)
    if (!p.in[k])
      return c->fail("hcMapElements: null input %d", k);
  const int elem = dtype == HC_F32 || dtype == HC_I32 ? 4 : 8;
  const char *tname = dtype == HC_F32   ? "f32"
                      : dtype == HC_F64 ? "f64"
                      : dtype == HC_I32 ? "i32"
                                        : "i64";
  // Contiguous matrices are one long row (unless the program asks where an
  // element is).
  bool flat = p.outPitch == p.cols && !usesIndices;
  for (int k = 0; k < p.nInputs; ++k)
    flat = flat && p.inPitch[k] == p.cols;
  if (flat) {
    p.cols *= p.rows;
    p.rows = 1;
    p.outPitch = p.cols;
    for (int k = 0; k < p.nInputs; ++k)
      p.inPitch[k] = p.cols;
  }
  // 16-byte packets when every base, pitch and the row length allow it.
  const int perPacket = 16 / elem;
  bool wide = p.cols % perPacket == 0 && aligned(p.out, 16) &&
              (p.rows == 1 || p.outPitch % perPacket == 0);
  for (int k = 0; k < p.nInputs; ++k)
    wide = wide && aligned(p.in[k], 16) && (p.rows == 1 || p.inPitch[k] % perPacket == 0);
  const int v = wide ? perPacket : 1;
  char name[64];
  // A body that was compiled ahead of time runs as straight-line code; any
  // other program is interpreted.
  const char *fused =
      c->fusedVariant == 1 || integer ? nullptr : matchFused(kFusedMaps, p);
  if (!fused && c->fusedVariant != 1 && c->specialiseMode != 0 &&
      hcSpecialisable(p, false, dtype)) {
    fused = hcSpecialise(c, false, dtype, p);
    if (!fused && c->specialiseMode == 2)
      return c->fail("hcMapElements: the program could not be compiled: %s",
                     hcSpecialiserNote(c));
  }
  if (fused)
    std::snprintf(name, sizeof name, "hc_map_fused_%s_%s_v%d", fused, tname, v);
  else {
    // Programs that divide, compare, use the later operators or work on integers
    // take the extended kernel, which tracks the validity of every element.
    bool extended = integer;
    for (int pc = 0; pc < p.nInstr; ++pc) {
      const uint32_t op = p.code[pc] & 0xffu;
      extended = extended || op == HC_MAP_DIV || op == HC_MAP_RDIV || op >= HC_MAP_FLOORDIV;
    }
    std::snprintf(name, sizeof name, "hc_map_elements_%s_v%d_n%d%s%s", tname, v,
                  std::max(1, p.nInputs), usesIndices ? "i" : "", extended ? "x" : "");
  }
  const long long perRow = p.cols / v;
  // One CTA per 1024 packets of a row (four per thread; 512 and two with three
  // or four inputs - map_elements.cu); rows beyond 65535 and very long rows are
  // walked by the kernel's strides.
  const long long perCta = p.nInputs <= 2 ? 1024 : 512;
  long long gx = std::min<long long>(ceilDiv(perRow, perCta), 1 << 20);
  long long gy = std::min<long long>(p.rows, 65535);
  void *args[] = {&p};
  return c->launch(name, size_t(gx), size_t(gy), 1, 256, args, 1, 0);
}

int hcRowProgram(HcContext c, const HcMapProgram *program, int dtype) {
  if (!c)
    return 1;
  if (dtype != HC_F32 && dtype != HC_F64)
    return c->fail("hcRowProgram: unsupported dtype %d", dtype);
  if (!program)
    return c->fail("hcRowProgram: null program");
  HcMapProgramDev p;
  std::memcpy(&p, program, sizeof p);
  if (p.nInputs < 1 || p.nInputs > 2 || p.nInstr < 1 || p.nInstr > HC_MAP_MAX_INSTR)
    return c->fail("hcRowProgram: %d inputs, %d instructions (1..2 and 1..%d)", p.nInputs,
                   p.nInstr, HC_MAP_MAX_INSTR);
  bool usesIndices = false;
  if (checkMapProgram(c, "hcRowProgram", p, true, &usesIndices))
    return 1;
  if (p.rows < 0 || p.cols < 0 || p.outPitch < p.cols)
    return c->fail("hcRowProgram: invalid shape %lld x %lld", (long long)p.rows,
                   (long long)p.cols);
  for (int k = 0; k < p.nInputs; ++k)
    if (p.inPitch[k] < p.cols)
      return c->fail("hcRowProgram: pitch of input %d is shorter than a row", k);
  if (p.rows == 0 || p.cols == 0)
    return 0;
  if (!p.out)
    return c->fail("hcRowProgram: null output");
  for (int k = 0; k < p.nInputs; ++k)
    if (!p.in[k])
      return c->fail("hcRowProgram: null input %d", k);
  if (ceilDiv(p.rows, 8) > 0x7fffffffLL)
    return c->fail("hcRowProgram: %lld rows exceed one launch", (long long)p.rows);
  if (p.cols > 0x7fffff00LL) // the kernel counts the packets of a row in an int
    return c->fail("hcRowProgram: rows of %lld elements are too long", (long long)p.cols);
  const int perPacket = 16 / (dtype == HC_F32 ? 4 : 8);
  bool wide = p.cols % perPacket == 0 && aligned(p.out, 16) && p.outPitch % perPacket == 0;
  for (int k = 0; k < p.nInputs; ++k)
    wide = wide && aligned(p.in[k], 16) && p.inPitch[k] % perPacket == 0;
  char name[64];
  void *args[] = {&p};
  const char *fused =
      c->fusedVariant == 1 || c->rowVariant >= 2 ? nullptr : matchFused(kFusedRows, p);
  if (!fused && c->fusedVariant != 1 && c->rowVariant < 2 && c->specialiseMode != 0 &&
      hcSpecialisable(p, true, dtype)) {
    fused = hcSpecialise(c, true, dtype, p);
    if (!fused && c->specialiseMode == 2)
      return c->fail("hcRowProgram: the program could not be compiled: %s",
                     hcSpecialiserNote(c));
  }
  // Rows of 257..1024 packets can be held in the registers of one CTA per row:
  // eight packets per thread on 64, 96 or 128 threads.  That pays when the row
  // fills most of the CTA's slots; otherwise a warp that walks the row is
  // faster.  row_variant 1 never holds, 2 holds rows beyond 512 packets on 256
  // threads with four packets each, 3 holds whatever the fill.
  const long long packets = p.cols / perPacket;
  if (wide && packets > 256 && packets <= 1024 && c->rowVariant != 1 &&
      p.rows <= 0x7fffffffLL /* one CTA per row */) {
    int held = 8;
    size_t threads = packets > 768 ? 128 : packets > 512 ? 96 : 64;
    if (c->rowVariant == 2 && packets > 512) {
      held = 4;
      threads = 256;
    }
    // Measured with a log-softmax program on 512 MB: float rows that fill a CTA
    // of 64 or 128 threads run at 3.8-4.0 TB/s held against 3.65-3.8 TB/s walked
    // and fall behind below about 90 % fill; on 96 threads (3.6 against 3.7 TB/s)
    // and for doubles (2.2 against 2.4 TB/s) walking is faster throughout.
    const bool filled = dtype == HC_F32 && threads != 96 &&
                        packets * 100 >= (long long)(held * threads) * kRowHeldFillPercent;
    if (filled && fused) {
      std::snprintf(name, sizeof name, "hc_row_fused_%s_f32_held_t%d", fused, int(threads));
      return c->launch(name, size_t(p.rows), 1, 1, threads, args, 1, 0);
    }
    if (filled || c->rowVariant >= 2) {
      int temps = 0; // the temporaries the program saves to, t0 first
      for (int pc = 0; pc < p.nInstr; ++pc) {
        const uint32_t op = p.code[pc] & 0xffu;
        if (op >= HC_MAP_SAVE0 && op <= HC_MAP_SAVE2)
          temps = std::max(temps, int(op - HC_MAP_SAVE0) + 1);
      }
      std::snprintf(name, sizeof name, "hc_row_program_held_%s_v%d_p%d_t%d_n%d",
                    dtype == HC_F32 ? "f32" : "f64", perPacket, held, int(threads), p.nInputs);
      const size_t smem = 256 + size_t(temps) * held * 16 * threads;
      return c->launch(name, size_t(p.rows), 1, 1, threads, args, 1, smem);
    }
  }
  if (fused)
    std::snprintf(name, sizeof name, "hc_row_fused_%s_%s_v%d", fused,
                  dtype == HC_F32 ? "f32" : "f64", wide ? perPacket : 1);
  else
    std::snprintf(name, sizeof name, "hc_row_program_%s_v%d_n%d",
                  dtype == HC_F32 ? "f32" : "f64", wide ? perPacket : 1, p.nInputs);
  // One warp per row, eight rows per CTA.
  return c->launch(name, size_t(ceilDiv(p.rows, 8)), 1, 1, 256, args, 1, 0);
}

// ---- work-item programs ---------------------------------------------------------------
static_assert(sizeof(HcItemProgram) == offsetof(HcItemProgramDev, groupsY) &&
                  offsetof(HcItemProgram, out) == offsetof(HcItemProgramDev, out) &&
                  offsetof(HcItemProgram, groupRows) == offsetof(HcItemProgramDev, groupRows) &&
                  offsetof(HcItemProgram, code) == offsetof(HcItemProgramDev, code) &&
                  offsetof(HcItemProgram, guardLo) == offsetof(HcItemProgramDev, guardLo) &&
                  offsetof(HcItemProgram, tileScale) == offsetof(HcItemProgramDev, tileScale) &&
                  offsetof(HcItemProgram, tileFill) == offsetof(HcItemProgramDev, tileFill),
              "public work-item program and kernel parameter block differ");

int hcWorkItems(HcContext c, const HcItemProgram *program, int dtype) {
  if (!c)
    return 1;
  const char *who = "hcWorkItems";
  if (dtype != HC_F32 && dtype != HC_F64)
    return c->fail("%s: unsupported dtype %d", who, dtype);
  if (!program)
    return c->fail("%s: null program", who);
  HcItemProgramDev p = {};
  std::memcpy(&p, program, sizeof *program);
  if (p.nInputs < 0 || p.nInputs > HC_MAP_MAX_INPUTS || p.nInstr < 1 ||
      p.nInstr > HC_ITEM_MAX_INSTR)
    return c->fail("%s: %d inputs, %d instructions (at most %d and 1..%d)", who, p.nInputs,
                   p.nInstr, HC_MAP_MAX_INPUTS, HC_ITEM_MAX_INSTR);
  if (p.rows < 0 || p.cols < 0 || p.outPitch < p.cols)
    return c->fail("%s: invalid shape %lld x %lld", who, (long long)p.rows, (long long)p.cols);
  if (p.groupRows < 1 || p.groupCols < 1 || (long long)p.groupRows * p.groupCols > 1024)
    return c->fail("%s: a work-group of %d x %d work-items (1..1024 in all)", who, p.groupRows,
                   p.groupCols);
  // Guards never reach beyond the arrays.
  for (int ph = 0; ph < HC_ITEM_MAX_PHASES; ++ph) {
    p.guardLo[ph][0] = std::max<long long>(p.guardLo[ph][0], 0);
    p.guardLo[ph][1] = std::max<long long>(p.guardLo[ph][1], 0);
    p.guardHi[ph][0] = std::min<long long>(p.guardHi[ph][0], p.rows);
    p.guardHi[ph][1] = std::min<long long>(p.guardHi[ph][1], p.cols);
  }
  int phase = 0;
  bool loaded = false, stores = false;
  bool saved[3] = {false, false, false};
  for (int pc = 0; pc < p.nInstr; ++pc) {
    const uint32_t op = p.code[pc] & 0xffu, src = (p.code[pc] >> 8) & 0xffu;
    if (op == HC_ITEM_BARRIER) {
      if (++phase >= HC_ITEM_MAX_PHASES)
        return c->fail("%s: more than one barrier (instruction %d)", who, pc);
      loaded = false;
      continue;
    }
    if (op == HC_ITEM_STORE_TILE || op == HC_ITEM_STORE_OUT) {
      if (!loaded)
        return c->fail("%s: instruction %d stores an accumulator that holds nothing", who, pc);
      stores = stores || op == HC_ITEM_STORE_OUT;
      continue;
    }
    if (op >= HC_MAP_OP_COUNT || op == HC_MAP_RSUM || op == HC_MAP_RMAX || op == HC_MAP_SET ||
        (op >= HC_MAP_SHL && op <= HC_MAP_RSHR))
      return c->fail("%s: unknown operation %u at instruction %d", who, op, pc);
    if (op != HC_MAP_LOAD && !loaded)
      return c->fail("%s: instruction %d uses an accumulator that holds nothing", who, pc);
    if (hcMapIsBinary(op)) {
      const bool input = src < uint32_t(p.nInputs);
      const bool temp =
          src >= HC_MAP_SRC_TEMP && src < HC_MAP_SRC_TEMP + 3 && saved[src - HC_MAP_SRC_TEMP];
      const bool constant =
          src >= HC_MAP_SRC_CONST && src < HC_MAP_SRC_CONST + uint32_t(HC_MAP_MAX_CONSTS);
      const bool index = src >= HC_MAP_SRC_ROW && src <= HC_ITEM_SRC_LOCAL_COL;
      const bool tile =
          src >= HC_ITEM_SRC_TILE && src < HC_ITEM_SRC_TILE + uint32_t(HC_ITEM_MAX_TILE_READS);
      if (!input && !temp && !constant && !index && !tile)
        return c->fail("%s: instruction %d reads operand %u, which does not exist or is not "
                       "written yet",
                       who, pc, src);
      if (input) {
        // Every work-item that passes the phase's guard must find its element.
        if (!p.in[src])
          return c->fail("%s: null input %u", who, src);
        if (p.inPitch[src] < p.cols)
          return c->fail("%s: pitch of input %u is shorter than a row", who, src);
        const bool empty = p.guardLo[phase][0] >= p.guardHi[phase][0] ||
                           p.guardLo[phase][1] >= p.guardHi[phase][1];
        if (!empty && (p.guardLo[phase][0] + p.inRow[src] < 0 ||
                       p.guardHi[phase][0] + p.inRow[src] > p.rows ||
                       p.guardLo[phase][1] + p.inCol[src] < 0 ||
                       p.guardHi[phase][1] + p.inCol[src] > p.cols))
          return c->fail("%s: input %u read at offset (%d, %d) leaves the array for work-items "
                         "that pass the guard of phase %d",
                         who, src, p.inRow[src], p.inCol[src], phase);
      }
      if (tile) {
        const int k = int(src - HC_ITEM_SRC_TILE);
        const int extent[2] = {p.groupRows, p.groupCols};
        for (int a = 0; a < 2; ++a) {
          if (p.tileMod[k][a] < 0 || p.tileMod[k][a] > extent[a])
            return c->fail("%s: tile read %d wraps at %d, beyond the group", who, k,
                           p.tileMod[k][a]);
          if (p.tileMod[k][a] == 0) {
            const long long first = p.tileOffset[k][a];
            const long long last = (long long)p.tileScale[k][a] * (extent[a] - 1) + first;
            if (std::min(first, last) < 0 || std::max(first, last) >= extent[a])
              return c->fail("%s: tile read %d leaves the group's tile", who, k);
          }
        }
      }
    }
    if (op >= HC_MAP_SAVE0 && op <= HC_MAP_SAVE2)
      saved[op - HC_MAP_SAVE0] = true;
    loaded = true;
  }
  if (!stores)
    return c->fail("%s: the program stores nothing", who);
  if (p.rows == 0 || p.cols == 0)
    return 0;
  if (!p.out)
    return c->fail("%s: null output", who);
  const long long groups = ceilDiv(p.rows, p.groupRows) * ceilDiv(p.cols, p.groupCols);
  if (groups > 0x7fffffffLL)
    return c->fail("%s: %lld work-groups exceed one launch", who, groups);
  const size_t threads = size_t(p.groupRows) * size_t(p.groupCols);
  // The groups that lie inside the guards of every phase the program has: the
  // kernel runs them without evaluating a guard.
  p.groupsY = uint32_t(ceilDiv(p.rows, p.groupRows));
  p.groupsX = uint32_t(ceilDiv(p.cols, p.groupCols));
  {
    const long long extent[2] = {p.groupRows, p.groupCols};
    long long lo[2] = {0, 0}, hi[2] = {(long long)p.groupsY, (long long)p.groupsX};
    for (int ph = 0; ph <= phase; ++ph)
      for (int a = 0; a < 2; ++a) {
        lo[a] = std::max(lo[a], ceilDiv(p.guardLo[ph][a], extent[a]));
        hi[a] = std::min(hi[a], std::max<long long>(p.guardHi[ph][a], 0) / extent[a]);
      }
    for (int a = 0; a < 2; ++a) {
      p.insideLo[a] = uint32_t(lo[a]);
      p.insideHi[a] = uint32_t(std::max(hi[a], lo[a]));
    }
  }
  void *args[] = {&p};
  // The program compiled at its first launch, as for element-wise and row programs.
  const int elemSize = dtype == HC_F32 ? 4 : 8;
  const bool wide = threads <= size_t(HC_ITEM_WIDE_THREADS);
  int perPass = HC_ITEM_NARROW_GROUPS;
  char name[64];
  std::snprintf(name, sizeof name, "%s", dtype == HC_F32 ? "hc_work_items_f32" : "hc_work_items_f64");
  if (c->fusedVariant != 1 && c->specialiseMode != 0) {
    const char *tag = hcSpecialiseItems(c, dtype, p.code, p.nInstr, wide);
    if (tag) {
      std::snprintf(name, sizeof name, "hc_work_items_fused_%s_%s", tag,
                    dtype == HC_F32 ? "f32" : "f64");
      if (wide)
        perPass = HC_ITEM_WIDE_BYTES / elemSize;
    } else if (c->specialiseMode == 2) {
      return c->fail("%s: the program could not be compiled: %s", who, hcSpecialiserNote(c));
    }
  }
  // A CTA takes `perPass` work-groups at a time and several such passes in turn:
  // a few CTAs per SM's worth of threads.
  const long long passes = ceilDiv(groups, (long long)perPass);
  const long long resident = std::max<long long>(1, 2048 / (long long)threads);
  const long long grid = std::min<long long>(passes, c->smCount * resident * 4);
  return c->launch(name, size_t(grid), 1, 1, threads, args, 1,
                   threads * size_t(perPass) * size_t(elemSize));
}

// ---- softmax --------------------------------------------------------------------
int hcSoftmaxRows(HcContext c, const void *x, void *y, long long rows,
                  long long cols, long long xPitch, long long yPitch,
                  int dtype) {
  if (!c)
    return 1;
  if (dtype != HC_F32 && dtype != HC_F64)
    return c->fail("hcSoftmaxRows: unsupported dtype %d", dtype);
  if (rows < 0 || cols < 0 || xPitch < cols || yPitch < cols)
    return c->fail("hcSoftmaxRows: invalid shape %lld x %lld", rows, cols);
  if (rows == 0 || cols == 0)
    return 0;
  if (!x || !y)
    return c->fail("hcSoftmaxRows: null buffer");
  const bool vecOk = dtype == HC_F32 && cols % 4 == 0 && cols <= 4096 &&
                     xPitch % 4 == 0 && yPitch % 4 == 0 && aligned(x, 16) &&
                     aligned(y, 16);
  // The bulk-copy pipelined kernel (one persistent CTA per SM, a ring of row
  // slots in shared memory) is opt-in: at 32768 x 4096 it measured 5.88 TB/s
  // against 6.76 TB/s for the register kernel below.
  if (vecOk && cols > 1024 && c->ccMajor >= 9 && c->softmaxVariant == 2) {
    // Long rows: 32 float4 per lane and 6 consumer warps; else 16 and 8.
    const int v = cols > 2048 ? 32 : 16;
    const int consumers = v == 32 ? 6 : 8;
    int slotBytes = int(roundUp(cols * 4, 128));
    // Slots per consumer warp: what fits in 200 KiB, at most 16 slots in all.
    int depth = int(std::min<long long>(16 / consumers,
                                        (200 * 1024) / ((long long)slotBytes * consumers)));
    const size_t smem = size_t(consumers) * depth * slotBytes + 128 /*align*/ + 384 /*barriers*/;
    long long grid = std::min<long long>(rows, c->smCount);
    int icols = int(cols);
    void *args[] = {&x, &y, &rows, &icols, &xPitch, &yPitch, &depth, &slotBytes,
                    &c->statusWord};
    return c->launch(v == 32 ? "hc_softmax_rows_f32_tma_v32" : "hc_softmax_rows_f32_tma_v16",
                     size_t(grid), 1, 1, size_t(32 * (consumers + 1)), args, 9, smem);
  }
  if (vecOk) {
    int v = 1;
    while (128 * v < cols)
      v <<= 1;
    char name[48];
    snprintf(name, sizeof(name), "hc_softmax_rows_f32_w%d", v);
    // One row per warp, four rows per CTA, as many CTAs as that takes.  A
    // persistent grid (SMs x resident CTAs walking the rows) measured 6.03 TB/s
    // at 32768 x 4096 against 6.76 TB/s for this: CTAs that start and retire
    // independently keep loads and stores of different rows interleaved,
    // while resident warps drift into doing the same phase at the same time.
    long long grid = std::min<long long>(ceilDiv(rows, 4), 0x7fffffffLL);
    int icols = int(cols);
    void *args[] = {&x, &y, &rows, &icols, &xPitch, &yPitch};
    return c->launch(name, size_t(grid), 1, 1, 128, args, 6, 0);
  }
  const size_t elem = dtype == HC_F32 ? 4 : 8;
  long long cacheElems = cols;
  size_t smem = size_t(roundUp(cols * (long long)elem, 16));
  if (smem > 160 * 1024) { // does not fit: the kernel re-reads the row instead
    smem = 0;
    cacheElems = 0;
  }
  long long grid = std::min<long long>(rows, c->smCount * 8);
  void *args[] = {&x, &y, &rows, &cols, &xPitch, &yPitch, &cacheElems};
  return c->launch(dtype == HC_F32 ? "hc_softmax_rows_generic_f32"
                                   : "hc_softmax_rows_generic_f64",
                   size_t(grid), 1, 1, 256, args, 7, smem);
}

// ---- compute and all-gather in one kernel ------------------------------------------
static_assert(sizeof(HcPeerOutputs) == sizeof(HcPeerDsts) &&
                  offsetof(HcPeerOutputs, count) == offsetof(HcPeerDsts, count),
              "public destination list and kernel parameter block differ");

static int checkPeers(HcContext c, const char *who, const HcPeerOutputs *dsts) {
  if (!dsts || dsts->count < 1 || dsts->count > HC_MAX_PEERS)
    return c->fail("%s: 1..%d destinations expected", who, HC_MAX_PEERS);
  for (int d = 0; d < dsts->count; ++d)
    if (!dsts->base[d] || !aligned(dsts->base[d], 16))
      return c->fail("%s: destination %d is null or not 16-byte aligned", who, d);
  return 0;
}

int hcSoftmaxRowsPeers(HcContext c, const void *x, const HcPeerOutputs *dsts, long long rows,
                       long long cols, long long xPitch, long long yPitch, int dtype) {
  if (!c)
    return 1;
  if (dtype != HC_F32)
    return c->fail("hcSoftmaxRowsPeers: float32 only");
  if (rows < 0 || cols < 0 || xPitch < cols || yPitch < cols)
    return c->fail("hcSoftmaxRowsPeers: invalid shape %lld x %lld", rows, cols);
  if (checkPeers(c, "hcSoftmaxRowsPeers", dsts))
    return 1;
  if (rows == 0 || cols == 0)
    return 0;
  if (!x)
    return c->fail("hcSoftmaxRowsPeers: null buffer");
  if (cols % 4 || cols > 4096 || xPitch % 4 || yPitch % 4 || !aligned(x, 16))
    return c->fail("hcSoftmaxRowsPeers: rows of at most 4096 columns, a multiple of 4, and "
                   "16-byte aligned bases and pitches (use hcSoftmaxRows and a collective "
                   "otherwise)");
  int v = 1;
  while (128 * v < cols)
    v <<= 1;
  char name[48];
  snprintf(name, sizeof(name), "hc_softmax_rows_f32_w%d_peers", v);
  long long grid = std::min<long long>(ceilDiv(rows, 4), 0x7fffffffLL);
  int icols = int(cols);
  HcPeerDsts peers;
  std::memcpy(&peers, dsts, sizeof peers);
  void *args[] = {&x, &rows, &icols, &xPitch, &yPitch, &peers};
  return c->launch(name, size_t(grid), 1, 1, 128, args, 6, 0);
}

int hcReduceRowsPeers(HcContext c, const void *x, const HcPeerOutputs *dsts,
                      long long maxOffset, long long rows, long long cols, long long pitch,
                      int dtype) {
  if (!c)
    return 1;
  if (dtype != HC_F32)
    return c->fail("hcReduceRowsPeers: float32 only");
  if (rows < 0 || cols < 0 || pitch < cols || maxOffset < rows)
    return c->fail("hcReduceRowsPeers: invalid shape %lld x %lld (maxima %lld elements after "
                   "the sums)",
                   rows, cols, maxOffset);
  if (checkPeers(c, "hcReduceRowsPeers", dsts))
    return 1;
  if (rows == 0)
    return 0;
  if (!x && cols > 0)
    return c->fail("hcReduceRowsPeers: null buffer");
  int vec = cols % 4 == 0 && pitch % 4 == 0 && aligned(x, 16);
  long long grid = std::min<long long>(ceilDiv(rows, 8), 0x7fffffffLL);
  HcPeerDsts peers;
  std::memcpy(&peers, dsts, sizeof peers);
  void *args[] = {&x, &rows, &cols, &pitch, &vec, &maxOffset, &peers};
  return c->launch("hc_reduce_rows_warp_f32_peers", size_t(grid), 1, 1, 256, args, 7, 0);
}

// ---- reductions -----------------------------------------------------------------
int hcReduceRows(HcContext c, const void *x, void *sumOut, void *maxOut,
                 long long rows, long long cols, long long pitch, int dtype) {
  if (!c)
    return 1;
  if (dtype != HC_F32 && dtype != HC_F64)
    return c->fail("hcReduceRows: unsupported dtype %d", dtype);
  if (rows < 0 || cols < 0 || pitch < cols)
    return c->fail("hcReduceRows: invalid shape %lld x %lld", rows, cols);
  if (rows == 0 || (!sumOut && !maxOut))
    return 0;
  if (!x && cols > 0)
    return c->fail("hcReduceRows: null buffer");
  int vec = dtype == HC_F32 && cols % 4 == 0 && pitch % 4 == 0 && aligned(x, 16);
  const bool f32 = dtype == HC_F32;
  void *args[] = {&x, &sumOut, &maxOut, &rows, &cols, &pitch, &vec};
  if (rows >= c->smCount * 8) {
    long long grid = ceilDiv(rows, 8);
    if (c->reduceVariant == 1) // persistent: SMs x 8 CTAs walking the rows
      grid = std::min<long long>(grid, c->smCount * 8);
    return c->launch(f32 ? "hc_reduce_rows_warp_f32" : "hc_reduce_rows_warp_f64",
                     size_t(grid), 1, 1, 256, args, 7, 0);
  }
  long long grid = std::min<long long>(rows, c->smCount * 8);
  return c->launch(f32 ? "hc_reduce_rows_block_f32" : "hc_reduce_rows_block_f64",
                   size_t(grid), 1, 1, 256, args, 7, 0);
}

int hcReduceAll(HcContext c, const void *a, long long n, void *result,
                int inDtype, int resultDtype) {
  if (!c)
    return 1;
  const char *in = inDtype == HC_F32   ? "f32"
                   : inDtype == HC_F64 ? "f64"
                   : inDtype == HC_I32 ? "i32"
                   : inDtype == HC_I64 ? "i64"
                                       : nullptr;
  const char *out = resultDtype == HC_F32 ? "f32" : resultDtype == HC_F64 ? "f64" : nullptr;
  if (!in || !out)
    return c->fail("hcReduceAll: unsupported dtypes %d -> %d", inDtype, resultDtype);
  if (n < 0)
    return c->fail("hcReduceAll: invalid length %lld", n);
  if (n == 0)
    return 0;
  if (!a || !result)
    return c->fail("hcReduceAll: null buffer");
  char name[48];
  snprintf(name, sizeof(name), "hc_reduce_all_%s_%s", in, out);
  // Enough CTAs to fill the GPU, each with at least a few elements per thread.
  long long grid = std::max<long long>(
      1, std::min<long long>(ceilDiv(n, 256 * 8), c->smCount * 8));
  void *args[] = {&a, &n, &result};
  return c->launch(name, size_t(grid), 1, 1, 256, args, 3, 0);
}

int hcPairwiseDistance(HcContext c, const void *a, const void *b, void *out,
                       long long M, long long N, long long D, long long lda,
                       long long ldb, long long ldo, int dtype) {
  if (!c)
    return 1;
  if (dtype != HC_F32 && dtype != HC_F64)
    return c->fail("hcPairwiseDistance: unsupported dtype %d", dtype);
  if (M < 0 || N < 0 || D < 0 || lda < D || ldb < D || ldo < N)
    return c->fail("hcPairwiseDistance: invalid shape M=%lld N=%lld D=%lld", M, N, D);
  if (M == 0 || N == 0)
    return 0;
  if (!out || (D > 0 && (!a || !b)))
    return c->fail("hcPairwiseDistance: null buffer");
  void *args[] = {&a, &b, &out, &M, &N, &D, &lda, &ldb, &ldo};
  return c->launch(dtype == HC_F32 ? "hc_pairwise_distance_f32" : "hc_pairwise_distance_f64",
                   size_t(ceilDiv(N, 64)), size_t(ceilDiv(M, 64)), 1, 256, args, 9, 0);
}

// ---- gathered tile product --------------------------------------------------------
static_assert(sizeof(HcMappedOperand) == sizeof(HcMappedOperandDev) &&
                  offsetof(HcMappedOperand, shape) == offsetof(HcMappedOperandDev, shape) &&
                  offsetof(HcMappedOperand, stride) == offsetof(HcMappedOperandDev, stride) &&
                  offsetof(HcMappedOperand, lo) == offsetof(HcMappedOperandDev, lo) &&
                  offsetof(HcMappedOperand, hi) == offsetof(HcMappedOperandDev, hi) &&
                  offsetof(HcMappedOperand, transposed) ==
                      offsetof(HcMappedOperandDev, transposed),
              "public operand description and kernel parameter block differ");

int hcMappedGemm(HcContext c, const HcMappedOperand *x, const HcMappedOperand *f,
                 const HcMappedOperand *out, long long groups, int TM, int TN, int K,
                 int dtype) {
  if (!c)
    return 1;
  if (dtype != HC_F32 && dtype != HC_F64)
    return c->fail("hcMappedGemm: unsupported dtype %d", dtype);
  if (!x || !f || !out)
    return c->fail("hcMappedGemm: null operand description");
  if (groups < 0 || TM < 0 || TN < 0 || K < 0)
    return c->fail("hcMappedGemm: invalid sizes groups=%lld TM=%d TN=%d K=%d", groups, TM, TN,
                   K);
  if (groups > 0x7fffffffLL)
    return c->fail("hcMappedGemm: %lld work-groups exceed one launch", groups);
  // Tile element indices are ints inside the kernel.
  if ((long long)TM * K > 0x7fffffffLL || (long long)K * TN > 0x7fffffffLL ||
      (long long)TM * TN > 0x7fffffffLL)
    return c->fail("hcMappedGemm: tile of %d x %d x %d is too large", TM, TN, K);
  if (groups == 0 || TM == 0 || TN == 0)
    return 0;
  const HcMappedOperand *ops[3] = {x, f, out};
  const char *names[3] = {"x", "f", "out"};
  for (int i = 0; i < 3; ++i) {
    // The tile origins are read for every operand; with K == 0 the elements and
    // the element tables of x and f are not (their tiles are empty).
    const bool elementsUsed = i == 2 || K > 0;
    if (!ops[i]->origins)
      return c->fail("hcMappedGemm: null origins table in %s", names[i]);
    if (elementsUsed && (!ops[i]->base || !ops[i]->map || !ops[i]->lin))
      return c->fail("hcMappedGemm: null buffer or table in %s", names[i]);
    if (!aligned(ops[i]->map, 16) || !aligned(ops[i]->origins, 16))
      return c->fail("hcMappedGemm: tables of %s are not 16-byte aligned", names[i]);
    for (int d = 0; d < 4; ++d)
      if (ops[i]->shape[d] < 0 || ops[i]->stride[d] < 0)
        return c->fail("hcMappedGemm: negative extent or stride in %s", names[i]);
  }
  HcMappedGemmParams p;
  std::memcpy(&p.x, x, sizeof(HcMappedOperand));
  std::memcpy(&p.f, f, sizeof(HcMappedOperand));
  std::memcpy(&p.out, out, sizeof(HcMappedOperand));
  p.TM = TM;
  p.TN = TN;
  p.K = K;
  if (out->transposed)
    return c->fail("hcMappedGemm: the tables of out must be in row-major order");
  // Smallest piece (8, 16, 32 or 64 each way) that holds the tile; larger tiles
  // are walked in 64-wide pieces by the kernel.  A side of 32 or more is worked
  // on by 16 threads, a shorter one by 8 (mapped_gemm.cu: Side).
  auto side = [](int extent) { return extent <= 8 ? 8 : extent <= 16 ? 16 : extent <= 32 ? 32 : 64; };
  // Work-groups that share their f tile are stacked along the rows of one CTA:
  // the largest power of two that the caller vouches for (f->sharedRun), that
  // the kernel holds (8) and that keeps the stacked rows within one piece: 128
  // rows for float tiles of more than 16 columns (mapped_stack 2: 64), else 64.
  const int sx = side(TN);
  const int tallest = dtype == HC_F32 && sx >= 32 && c->mappedStack != 2 ? 128 : 64;
  int stack = 1;
  while (stack * 2 <= 8 && stack * 2 <= f->sharedRun && f->sharedRun % (stack * 2) == 0 &&
         (long long)stack * 2 * TM <= tallest && c->mappedStack != 1)
    stack *= 2;
  p.stack = stack;
  p.groups = groups;
  const int sy = stack * TM > 64 && tallest == 128 ? 128 : side(stack * TM);
  const int threads = (sy >= 32 ? 16 : 8) * (sx >= 32 ? 16 : 8);
  char name[48];
  std::snprintf(name, sizeof name, "hc_mapped_gemm_%s_%dx%d", dtype == HC_F32 ? "f32" : "f64", sy,
                sx);
  void *args[] = {&p};
  return c->launch(name, size_t(ceilDiv(groups, stack)), 1, 1, size_t(threads), args, 1, 0);
}

// ---- GEMMs ----------------------------------------------------------------------
static int checkGemmShape(HcContext c, const char *who, const void *a,
                          const void *b, const void *out, long long M,
                          long long N, long long K, long long lda,
                          long long ldb, long long ldc) {
  if (M < 0 || N < 0 || K < 0 || lda < K || ldb < N || ldc < N)
    return c->fail("%s: invalid shape M=%lld N=%lld K=%lld (lda %lld ldb %lld "
                   "ldc %lld)",
                   who, M, N, K, lda, ldb, ldc);
  if (M > 0 && N > 0 && (!out || (K > 0 && (!a || !b))))
    return c->fail("%s: null buffer", who);
  return 0;
}

int hcGemmTiled(HcContext c, const void *a, const void *b, void *out,
                long long M, long long N, long long K, long long lda,
                long long ldb, long long ldc, int dtype) {
  if (!c)
    return 1;
  const char *name = dtype == HC_F32    ? "hc_gemm_tiled_f32"
                     : dtype == HC_F64  ? "hc_gemm_tiled_f64"
                     : dtype == HC_BF16 ? "hc_gemm_tiled_bf16"
                                        : nullptr;
  if (!name)
    return c->fail("hcGemmTiled: unsupported dtype %d", dtype);
  if (checkGemmShape(c, "hcGemmTiled", a, b, out, M, N, K, lda, ldb, ldc))
    return 1;
  if (M == 0 || N == 0)
    return 0;
  void *args[] = {&a, &b, &out, &M, &N, &K, &lda, &ldb, &ldc};
  // fp32 operands that 16-byte cp.async can fetch take the pipelined variant
  // (3 stages of a 64x36 A block and a 32x68 B block of floats).
  if (dtype == HC_F32 && K > 0 && c->tiledVariant != 1 && lda % 4 == 0 &&
      ldb % 4 == 0 && aligned(a, 16) && aligned(b, 16)) {
    const size_t smem = 3 * (64 * 36 + 32 * 68) * sizeof(float);
    const long long tiles = ceilDiv(N, 64) * ceilDiv(M, 64);
    // Few tiles and a K loop worth splitting: a cluster of four CTAs per tile,
    // each summing a quarter of K (gemm_tiled.cu), as long as the clusters of
    // all tiles can be resident at once.
    if (c->tiledVariant != 2 && c->ccMajor >= 9 && K >= 4 * 32 && tiles * 4 <= c->smCount)
      return c->launch("hc_gemm_tiled_f32_splitk", size_t(ceilDiv(N, 64)),
                       size_t(ceilDiv(M, 64)), 4, 256, args, 9, smem);
    return c->launch("hc_gemm_tiled_f32_async", size_t(ceilDiv(N, 64)),
                     size_t(ceilDiv(M, 64)), 1, 256, args, 9, smem);
  }
  return c->launch(name, size_t(ceilDiv(N, 64)), size_t(ceilDiv(M, 64)), 1, 256,
                   args, 9, 0);
}

// Launches one of the tcgen05 kernels; `b` is bf16 [K, N].
static int launchUmma(HcContext c, const void *a, const void *b,
                      const float *scale, void *out, long long M, long long N,
                      long long K, long long lda, long long ldb, long long ldc,
                      bool pair, const HcPeerOutputs *dsts = nullptr) {
  alignas(64) CUtensorMap mapA, mapB;
  if (olxEncodeTensorMap2D(c->device, &mapA, /*bf16*/ 0, a, size_t(M), size_t(K),
                           size_t(lda) * 2, kUmmaBM, kUmmaBK, 128) ||
      olxEncodeTensorMap2D(c->device, &mapB, /*bf16*/ 0, b, size_t(K), size_t(N),
                           size_t(ldb) * 2, kUmmaBK, 64, 128))
    return c->fail("tensor map encoding failed: %s", c->lastError.c_str());
  const int tileM = pair ? 2 * kUmmaBM : kUmmaBM;
  int tilesM = int(ceilDiv(M, tileM)), tilesN = int(ceilDiv(N, kUmmaBN));
  // Tiles that run concurrently should form a compact block of the output so
  // that the A and B panels they share stay in L2.
  int bandM = c->gemmBand ? int(c->gemmBand) : 16;
  int vecStore = aligned(out, 16) && ldc % 8 == 0;
  HcPeerDsts peers{};
  if (dsts) {
    // Every destination takes the same tiles: all must allow 16-byte stores.
    std::memcpy(&peers, dsts, sizeof peers);
    vecStore = ldc % 8 == 0;
    for (int d = 0; d < peers.count; ++d)
      vecStore = vecStore && aligned(peers.base[d], 16);
  }
  long long tiles = (long long)tilesM * tilesN;
  char name[56];
  std::snprintf(name, sizeof name, "hc_gemm_bf16_umma%s%s%s", pair ? "_pair" : "",
                scale ? "_scaled" : "", dsts ? "_peers" : "");
  long long grid = std::min<long long>(tiles, c->smCount);
  if (pair) {
    // The kernel is persistent: CTA pairs beyond what the GPU can hold at once
    // would only start when the first wave has finished all its tiles.
    if (c->pairSlots == 0) {
      OlKernel k = c->kernel(name);
      int slots = 0;
      if (!k || olxMaxActiveClusters(c->queue, k, kUmmaThreads, kUmmaSmemBytes, 2,
                                     &slots) || slots <= 0)
        return c->fail("cluster occupancy query failed: %s", c->lastError.c_str());
      c->pairSlots = slots;
    }
    grid = 2 * std::min<long long>(tiles, c->pairSlots);
  }
  void *args[] = {&mapA,   &mapB,   &out,   &scale,    &M,           &N,    &K,
                  &ldc,    &tilesM, &tilesN, &bandM,   &vecStore, &c->statusWord, &peers};
  return c->launch(name, size_t(grid), 1, 1, kUmmaThreads, args, dsts ? 14 : 13,
                   kUmmaSmemBytes);
}

static bool ummaEligible(HcContext c, const void *a, const void *b,
                         long long K, long long lda, long long ldb) {
  return c->ccMajor == 10 && K > 0 && lda % 8 == 0 && ldb % 8 == 0 &&
         aligned(a, 16) && aligned(b, 16);
}

int hcGemmBf16(HcContext c, const void *a, const void *b, void *out,
               long long M, long long N, long long K, long long lda,
               long long ldb, long long ldc) {
  if (!c)
    return 1;
  if (checkGemmShape(c, "hcGemmBf16", a, b, out, M, N, K, lda, ldb, ldc))
    return 1;
  if (M == 0 || N == 0)
    return 0;
  if (c->gemmVariant == 3 || !ummaEligible(c, a, b, K, lda, ldb))
    return hcGemmTiled(c, a, b, out, M, N, K, lda, ldb, ldc, HC_BF16);
  // A CTA pair per 256 x 256 tile moves a third less data per CTA than one CTA
  // per 128 x 256 tile; it needs at least two row blocks to be worth a cluster.
  const bool pair = c->gemmVariant == 2 || (c->gemmVariant == 0 && M > kUmmaBM);
  return launchUmma(c, a, b, nullptr, out, M, N, K, lda, ldb, ldc, pair);
}

// ---- fp32 GEMM on the tensor cores (three tf32 products per fp32 product) ----------
static long long f32Pitch(long long K) { return roundUp(K, 4); }

size_t hcGemmF32TensorWorkspaceBytes(long long M, long long N, long long K) {
  if (M <= 0 || N <= 0 || K <= 0)
    return 0;
  // hi and lo parts of A [M, Kp] and of B transposed [N, Kp], each 1 KiB aligned.
  const size_t a = size_t(roundUp(M * f32Pitch(K) * 4, 1024));
  const size_t b = size_t(roundUp(N * f32Pitch(K) * 4, 1024));
  return 2 * a + 2 * b;
}

int hcGemmF32Tensor(HcContext c, const void *a, const void *b, void *out, void *workspace,
                    size_t workspaceBytes, long long M, long long N, long long K,
                    long long lda, long long ldb, long long ldc) {
  if (!c)
    return 1;
  if (checkGemmShape(c, "hcGemmF32Tensor", a, b, out, M, N, K, lda, ldb, ldc))
    return 1;
  if (M == 0 || N == 0)
    return 0;
  // Without tcgen05, or with nothing to sum, the CUDA-core kernel does it.
  if (c->ccMajor != 10 || K == 0 || c->gemmVariant == 3)
    return hcGemmTiled(c, a, b, out, M, N, K, lda, ldb, ldc, HC_F32);
  const size_t need = hcGemmF32TensorWorkspaceBytes(M, N, K);
  if (!workspace || workspaceBytes < need || !aligned(workspace, 1024))
    return c->fail("hcGemmF32Tensor: workspace of %zu bytes (1 KiB aligned) needed, got %zu",
                   need, workspaceBytes);
  const long long kp = f32Pitch(K);
  const size_t aBytes = size_t(roundUp(M * kp * 4, 1024)), bBytes = size_t(roundUp(N * kp * 4, 1024));
  auto *base = static_cast<unsigned char *>(workspace);
  float *aHi = reinterpret_cast<float *>(base), *aLo = reinterpret_cast<float *>(base + aBytes);
  float *bHi = reinterpret_cast<float *>(base + 2 * aBytes);
  float *bLo = reinterpret_cast<float *>(base + 2 * aBytes + bBytes);
  {
    // (Packets of four columns and two rows per thread where the layout allows.)
    long long gx = std::max<long long>(1, std::min<long long>(ceilDiv(kp, 1024), 64));
    long long gy = std::max<long long>(1, std::min<long long>(ceilDiv(M, 2), 65535));
    void *args[] = {&a, &aHi, &aLo, &M, &K, &lda, (void *)&kp};
    if (c->launch("hc_split_tf32", size_t(gx), size_t(gy), 1, 256, args, 7, 0))
      return 1;
  }
  {
    const long long tiles = ceilDiv(N, 32) * ceilDiv(kp, 64);
    long long grid = std::max<long long>(1, std::min<long long>(tiles, c->smCount * 16));
    void *args[] = {&b, &bHi, &bLo, &K, &N, &ldb, (void *)&kp};
    if (c->launch("hc_split_tf32_t", size_t(grid), 1, 1, 256, args, 7, 0))
      return 1;
  }
  // A CTA pair per 256 x 256 tile stages 64 KiB per K-block and CTA instead of 96
  // (three stages fit instead of two); it needs two row blocks to be worth a cluster.
  const bool pair = c->gemmVariant == 2 || (c->gemmVariant == 0 && M > 128);
  alignas(64) CUtensorMap maps[4];
  const void *parts[4] = {aHi, aLo, bHi, bLo};
  for (int i = 0; i < 4; ++i) {
    const bool isA = i < 2;
    if (olxEncodeTensorMap2D(c->device, &maps[i], /*f32*/ 1, parts[i], size_t(isA ? M : N),
                             size_t(kp), size_t(kp) * 4, (isA || pair) ? 128 : 256, 32, 128))
      return c->fail("tensor map encoding failed: %s", c->lastError.c_str());
  }
  int tilesM = int(ceilDiv(M, pair ? 256 : 128)), tilesN = int(ceilDiv(N, 256));
  int bandM = pair ? 8 : 16;
  int vecStore = aligned(out, 16) && ldc % 4 == 0;
  const long long tiles = (long long)tilesM * tilesN;
  long long grid = std::min<long long>(tiles, c->smCount);
  const size_t smem = (pair ? 3 * 64 : 2 * 96) * 1024 /*stages*/ + 1024 /*align*/ + 256 /*barriers*/;
  const char *name = pair ? "hc_gemm_f32_umma_pair" : "hc_gemm_f32_umma";
  if (pair) {
    // Persistent kernel: no more CTA pairs than the GPU holds at once.
    if (c->pairSlotsF32 == 0) {
      OlKernel k = c->kernel(name);
      int slots = 0;
      if (!k || olxMaxActiveClusters(c->queue, k, 192, smem, 2, &slots) || slots <= 0)
        return c->fail("cluster occupancy query failed: %s", c->lastError.c_str());
      c->pairSlotsF32 = slots;
    }
    grid = 2 * std::min<long long>(tiles, c->pairSlotsF32);
  }
  void *args[] = {&maps[0], &maps[1], &maps[2], &maps[3], &out,    &M,        &N,
                  &K,       &ldc,     &tilesM,  &tilesN,  &bandM, &vecStore, &c->statusWord};
  return c->launch(name, size_t(grid), 1, 1, 192, args, 14, smem);
}

// ---- float32 convolution on the tensor cores (conv_f32_umma.cu) ---------------------
static size_t convFilterBytes(long long NF, long long C, long long HF, long long WF) {
  // hi and lo parts of f as a matrix [NF, Kp], each 1 KiB aligned.
  return 2 * size_t(roundUp(NF * f32Pitch(C * HF * WF) * 4, 1024));
}

size_t hcConvF32TensorWorkspaceBytes(long long N, long long C, long long H, long long W,
                                     long long NF, long long HF, long long WF) {
  if (N <= 0 || C <= 0 || H <= 0 || W <= 0 || NF <= 0 || HF <= 0 || WF <= 0)
    return 0;
  // The split filters, then the image as (hi, lo) pairs; or, for the form whose image
  // tiles come by TMA, filters and image with the channels padded to 32.
  const long long cp = roundUp(C, 32);
  const size_t gathered = convFilterBytes(NF, C, HF, WF) + size_t(roundUp(N * C * H * W * 8, 1024));
  const size_t taps = 2 * size_t(roundUp(NF * HF * WF * cp * 4, 1024)) +
                      2 * size_t(roundUp(N * H * W * cp * 4, 1024));
  return std::max(gathered, taps);
}

// The rectangle of 128 output pixels (a power of two wide, inside the image) that
// wastes least of the tiles; false when the image is smaller than every rectangle.
static bool pickConvBox(long long H, long long W, long long HO, long long WO, long long &boxW,
                        long long &boxH) {
  double best = -1.0;
  boxW = boxH = 0;
  for (long long bw = 128; bw >= 8; bw /= 2) {
    const long long bh = 128 / bw;
    if (bw > W || bh > H)
      continue;
    const double use = double(WO) / double(roundUp(WO, bw)) * double(HO) / double(roundUp(HO, bh));
    if (use > best + 1e-9)
      best = use, boxW = bw, boxH = bh;
  }
  return boxW != 0;
}

// The convolution with both operands by TMA (conv_f32_taps.cu): stride 1.
static long long convRowsStages(long long NF, long long WF) {
  // hc_conv_f32_rows: a stage holds the image patch (hi, lo) and WF filter tiles (hi, lo).
  const long long nPad = roundUp(NF, 16), patchRows = roundUp(128 + WF - 1, 8);
  const long long stageBytes = 2 * patchRows * 128 + WF * 2 * nPad * 32 * 4;
  return std::min<long long>(6, (227 * 1024 - 1024 - 256) / stageBytes);
}

static int convF32Taps(HcContext c, const void *x, const void *f, void *out, long long N,
                       long long C, long long H, long long W, long long NF, long long HF,
                       long long WF, void *workspace, bool stacked, bool rows) {
  const char *who = "hcConvF32Tensor";
  const long long HO = H - HF + 1, WO = W - WF + 1, nPad = roundUp(NF, 16);
  const long long cp = roundUp(C, 32), cBlocks = cp / 32, taps = HF * WF;
  const long long kBlocks = taps * cBlocks, kp = taps * cp;
  long long boxW = 0, boxH = 0;
  if (!rows && !pickConvBox(H, W, HO, WO, boxW, boxH))
    return c->fail("%s: an image of %lld x %lld is too small for the TMA form", who, H, W);
  const long long tilesW = rows ? 0 : ceilDiv(WO, boxW), tilesH = rows ? 0 : ceilDiv(HO, boxH);
  const long long patchRows = roundUp(128 + WF - 1, 8);
  const long long tilesFlat = ceilDiv((HO - 1) * W + WO, 128);
  const long long stageBytes = rows ? 2 * patchRows * 128 + WF * 2 * nPad * 32 * 4
                                    : 2 * 128 * 32 * 4 + 2 * nPad * 32 * 4;
  const long long fixed = 1024 /*align*/ + 256 /*barriers*/;
  long long stages = std::min<long long>(6, (227 * 1024 - fixed) / stageBytes);
  if (c->convStages)
    stages = std::min(stages, c->convStages);
  if (stages < 2)
    return c->fail("%s: %lld filters do not fit in shared memory", who, NF);
  auto *base = static_cast<unsigned char *>(workspace);
  const size_t filterBytes = size_t(roundUp(NF * kp * 4, 1024));
  const size_t imageBytes = size_t(roundUp(N * H * W * cp * 4, 1024));
  float *fHi = reinterpret_cast<float *>(base), *fLo = reinterpret_cast<float *>(base + filterBytes);
  float *xHi = reinterpret_cast<float *>(base + 2 * filterBytes);
  float *xLo = reinterpret_cast<float *>(base + 2 * filterBytes + imageBytes);
  {
    // Image and filters rewritten by one launch (the last row of the grid takes the filters).
    int ci = int(C), hw = int(H * W), cpi = int(cp), images = int(N), nf = int(NF), ti = int(taps);
    const long long work = ceilDiv(H * W, 32) * ceilDiv(cp, 64);
    const long long gx = std::max<long long>(1, std::min<long long>(work, c->smCount * 8));
    void *args[] = {&x, &xHi, &xLo, &ci, &hw, &cpi, &images, &f, &fHi, &fLo, &nf, &ti};
    if (c->launch("hc_split_tf32_nhwc", size_t(gx), size_t(N + 1), 1, 256, args, 12, 0))
      return 1;
  }
  alignas(64) CUtensorMap maps[4];
  // The image as [N, H, W, Cp] for boxes of pixels, as [N, H * W, Cp] for runs of
  // positions.
  const size_t dims4[4] = {size_t(cp), size_t(W), size_t(H), size_t(N)};
  const size_t pitches4[3] = {size_t(cp) * 4, size_t(W * cp) * 4, size_t(H * W * cp) * 4};
  const unsigned box4[4] = {32, unsigned(boxW), unsigned(boxH), 1};
  const size_t dims3[3] = {size_t(cp), size_t(H * W), size_t(N)};
  const size_t pitches3[2] = {size_t(cp) * 4, size_t(H * W * cp) * 4};
  const unsigned box3[3] = {32, unsigned(patchRows), 1};
  const void *images[2] = {xHi, xLo}, *filters[2] = {fHi, fLo};
  for (int i = 0; i < 2; ++i)
    if ((rows ? olxEncodeTensorMapTiled(c->device, &maps[i], /*f32*/ 1, images[i], 3, dims3,
                                        pitches3, box3, 128)
              : olxEncodeTensorMapTiled(c->device, &maps[i], /*f32*/ 1, images[i], 4, dims4,
                                        pitches4, box4, 128)) ||
        olxEncodeTensorMap2D(c->device, &maps[2 + i], /*f32*/ 1, filters[i], size_t(NF),
                             size_t(kp), size_t(kp) * 4, size_t(nPad), 32, 128))
      return c->fail("tensor map encoding failed: %s", c->lastError.c_str());
  HcConvTapParams p{};
  p.out = static_cast<float *>(out);
  p.N = int(N), p.C = int(C), p.H = int(H), p.W = int(W);
  p.NF = int(NF), p.HF = int(HF), p.WF = int(WF);
  p.HO = int(HO), p.WO = int(WO);
  p.cBlocks = int(cBlocks), p.kBlocks = int(kBlocks), p.nPad = int(nPad);
  p.boxW = int(boxW), p.boxH = int(boxH), p.tilesW = int(tilesW), p.tilesH = int(tilesH);
  p.stages = int(stages);
  p.stacked = stacked ? 1 : 0;
  p.status = c->statusWord;
  p.tilesFlat = int(tilesFlat), p.patchRows = int(patchRows);
  const long long tiles = rows ? N * tilesFlat : N * tilesW * tilesH;
  const long long grid = std::min<long long>(tiles, c->smCount);
  const size_t smem = size_t(stages * stageBytes + fixed);
  void *args[] = {&maps[0], &maps[1], &maps[2], &maps[3], &p};
  return c->launch(rows ? "hc_conv_f32_rows" : "hc_conv_f32_taps", size_t(grid), 1, 1, 192, args,
                   5, smem);
}

int hcConvF32Tensor(HcContext c, const void *x, const void *f, void *out, long long N,
                    long long C, long long H, long long W, long long NF, long long HF,
                    long long WF, long long stride, void *workspace, size_t workspaceBytes) {
  if (!c)
    return 1;
  const char *who = "hcConvF32Tensor";
  if (N < 0 || C <= 0 || H <= 0 || W <= 0 || NF <= 0 || HF <= 0 || WF <= 0 || stride <= 0 ||
      HF > H || WF > W)
    return c->fail("%s: invalid shape x [%lld, %lld, %lld, %lld], f [%lld, %lld, %lld, %lld], "
                   "stride %lld", who, N, C, H, W, NF, C, HF, WF, stride);
  if (N == 0)
    return 0;
  if (!x || !f || !out)
    return c->fail("%s: null array", who);
  if (c->ccMajor != 10)
    return c->fail("%s: needs the tcgen05 tensor cores (compute capability 10.x, this device "
                   "has %lld.%lld); hcMappedGemm runs the same convolution anywhere", who,
                   c->ccMajor, c->ccMinor);
  const long long HO = (H - HF) / stride + 1, WO = (W - WF) / stride + 1;
  const long long K = C * HF * WF, kp = f32Pitch(K), kBlocks = ceilDiv(K, 32);
  const long long nPad = roundUp(NF, 16), pixels = HO * WO;
  const long long tilesPerImage = ceilDiv(pixels, 128);
  if (NF > 256)
    return c->fail("%s: at most 256 filters per call, got %lld", who, NF);
  if (C * H * W >= (1ll << 31) || N * tilesPerImage >= (1ll << 31) || NF * pixels >= (1ll << 31))
    return c->fail("%s: an image of %lld x %lld x %lld exceeds 32-bit element offsets", who, C, H,
                   W);
  // The two products that share a_hi run as one MMA of twice the width when the
  // accumulator has room for both halves (at most 128 filters; at most 64 when the
  // tensor-memory form is demanded, which needs room there too).
  const bool stacked = nPad <= 128 && c->convStacked != 1 &&
                       !(c->convVariant == 2 && nPad > 64);
  // The image operand of a K block goes through tensor memory when there is room
  // beside the accumulators, else through shared memory.
  const long long accColumns = stacked ? 2 * nPad : nPad;
  const bool tmemA = c->convVariant == 2 || (c->convVariant == 0 && accColumns <= 128);
  if (tmemA && accColumns > 128)
    return c->fail("%s: the tensor-memory form takes at most %d filters, got %lld", who,
                   stacked ? 64 : 128, NF);
  // Shared memory: the stages, the offset of every k, the barriers.
  const long long stageBytes = (tmemA ? 0 : 2 * 128 * 32 * 4) + 2 * nPad * 32 * 4;
  const long long fixed = kBlocks * 32 * 4 + 1024 /*align*/ + 256 /*barriers*/;
  const long long room = 227 * 1024 - fixed;
  // (In tensor memory: six stages beside accumulators of 64 columns, else four.)
  long long stages = std::min<long long>(tmemA && accColumns <= 64 ? 6 : 4, room / stageBytes);
  if (c->convStages)
    stages = std::min(stages, c->convStages);
  if (stages < 2)
    return c->fail("%s: a reduction over %lld elements with %lld filters does not fit in "
                   "shared memory", who, K, NF);
  const size_t need = hcConvF32TensorWorkspaceBytes(N, C, H, W, NF, HF, WF);
  if (!workspace || workspaceBytes < need || !aligned(workspace, 1024))
    return c->fail("%s: workspace of %zu bytes (1 KiB aligned) needed, got %zu", who, need,
                   workspaceBytes);
  if (!aligned(x, 4) || !aligned(out, 4) || !aligned(f, 4))
    return c->fail("%s: arrays must be 4-byte aligned", who);
  // Stride 1: both operands by TMA, no gathering threads (conv_f32_taps.cu).
  long long boxW = 0, boxH = 0;
  const bool tapsFit = stride == 1 && pickConvBox(H, W, HO, WO, boxW, boxH) &&
                       N * H * W < (1ll << 31) && N * HO * ceilDiv(WO, 8) < (1ll << 31);
  if (c->convVariant == 3 && !tapsFit)
    return c->fail("%s: the TMA form takes stride 1 and images that hold a rectangle of 128 "
                   "pixels (8 x 16 ... 128 x 1)", who);
  // Runs of 128 positions of the flattened image, the patch of a filter row shared
  // by its taps: the patch has to fit a TMA box and two stages shared memory.
  const bool rowsFit = stride == 1 && 128 + WF - 1 <= 256 && H * W >= roundUp(128 + WF - 1, 8) &&
                       convRowsStages(NF, WF) >= 2 && N * H * W < (1ll << 31);
  if (c->convVariant == 4 && !rowsFit)
    return c->fail("%s: the form that shares an image patch among the taps of a filter row "
                   "takes stride 1, images of at least %lld positions and filters of which "
                   "two stages fit in shared memory", who, roundUp(128 + WF - 1, 8));
  const bool tapsStacked = nPad <= 128 && c->convStacked != 1;
  if (rowsFit && (c->convVariant == 4 || c->convVariant == 0))
    return convF32Taps(c, x, f, out, N, C, H, W, NF, HF, WF, workspace, tapsStacked, true);
  if (tapsFit && (c->convVariant == 3 || c->convVariant == 0))
    return convF32Taps(c, x, f, out, N, C, H, W, NF, HF, WF, workspace, tapsStacked, false);
  auto *base = static_cast<unsigned char *>(workspace);
  const size_t filterBytes = convFilterBytes(NF, C, HF, WF);
  float *fHi = reinterpret_cast<float *>(base);
  float *fLo = reinterpret_cast<float *>(base + filterBytes / 2);
  void *xPairs = base + filterBytes;
  {
    // x once as (hi, lo) pairs: every element is read once per filter tap.
    long long count = N * C * H * W;
    long long grid = std::max<long long>(1, std::min<long long>(ceilDiv(count, 256),
                                                                c->smCount * 8));
    void *args[] = {&x, &xPairs, &count};
    if (c->launch("hc_split_tf32_pairs", size_t(grid), 1, 1, 256, args, 3, 0))
      return 1;
  }
  {
    // f is the K-major [NF, K] operand as it lies in memory.
    long long gx = std::max<long long>(1, std::min<long long>(ceilDiv(kp, 256), 64));
    long long gy = std::max<long long>(1, std::min<long long>(NF, 65535));
    void *args[] = {&f, &fHi, &fLo, &NF, (void *)&K, (void *)&K, (void *)&kp};
    if (c->launch("hc_split_tf32", size_t(gx), size_t(gy), 1, 256, args, 7, 0))
      return 1;
  }
  alignas(64) CUtensorMap maps[2];
  const void *parts[2] = {fHi, fLo};
  for (int i = 0; i < 2; ++i)
    if (olxEncodeTensorMap2D(c->device, &maps[i], /*f32*/ 1, parts[i], size_t(NF), size_t(kp),
                             size_t(kp) * 4, size_t(nPad), 32, 128))
      return c->fail("tensor map encoding failed: %s", c->lastError.c_str());
  HcConvParams p{};
  p.x = xPairs;
  p.out = static_cast<float *>(out);
  p.N = int(N), p.C = int(C), p.H = int(H), p.W = int(W);
  p.NF = int(NF), p.HF = int(HF), p.WF = int(WF), p.stride = int(stride);
  p.HO = int(HO), p.WO = int(WO);
  p.K = int(K), p.kBlocks = int(kBlocks), p.nPad = int(nPad);
  p.tilesPerImage = int(tilesPerImage);
  p.stages = int(stages);
  p.stacked = stacked ? 1 : 0;
  p.status = c->statusWord;
  const long long tiles = N * tilesPerImage;
  const long long grid = std::min<long long>(tiles, c->smCount);
  const size_t smem = size_t(stages * stageBytes + fixed);
  void *args[] = {&maps[0], &maps[1], &p};
  return c->launch(tmemA ? "hc_conv_f32_umma_ta" : "hc_conv_f32_umma", size_t(grid), 1, 1, 448,
                   args, 3, smem);
}

int hcGemmBf16Peers(HcContext c, const void *a, const void *b, const HcPeerOutputs *dsts,
                    long long M, long long N, long long K, long long lda, long long ldb,
                    long long ldc) {
  if (!c)
    return 1;
  if (checkPeers(c, "hcGemmBf16Peers", dsts))
    return 1;
  if (checkGemmShape(c, "hcGemmBf16Peers", a, b, dsts->base[0], M, N, K, lda, ldb, ldc))
    return 1;
  if (M == 0 || N == 0)
    return 0;
  if (!ummaEligible(c, a, b, K, lda, ldb))
    return c->fail("hcGemmBf16Peers: operands the tensor-core kernel cannot take (pitches that "
                   "are multiples of 8 elements and 16-byte aligned bases; use hcGemmBf16 and a "
                   "collective otherwise)");
  const bool pair = c->gemmVariant == 2 || (c->gemmVariant != 1 && M > kUmmaBM);
  return launchUmma(c, a, b, nullptr, dsts->base[0], M, N, K, lda, ldb, ldc, pair, dsts);
}

int hcGemmW8A16Peers(HcContext c, const void *a, const void *w, const float *scale,
                     const HcPeerOutputs *dsts, void *workspace, size_t workspaceBytes,
                     long long M, long long N, long long K, long long lda, long long ldw,
                     long long ldc) {
  if (!c)
    return 1;
  if (checkPeers(c, "hcGemmW8A16Peers", dsts))
    return 1;
  if (checkGemmShape(c, "hcGemmW8A16Peers", a, w, dsts->base[0], M, N, K, lda, ldw, ldc))
    return 1;
  if (M == 0 || N == 0)
    return 0;
  if (!scale)
    return c->fail("hcGemmW8A16Peers: null scale");
  const long long wsPitch = roundUp(N, 16);
  if (!ummaEligible(c, a, workspace, K, lda, wsPitch))
    return c->fail("hcGemmW8A16Peers: operands the tensor-core kernel cannot take (use "
                   "hcGemmW8A16 and a collective)");
  if (!workspace || workspaceBytes < hcGemmW8A16WorkspaceBytes(N, K))
    return c->fail("hcGemmW8A16Peers: workspace of %zu bytes is too small, need %zu",
                   workspaceBytes, hcGemmW8A16WorkspaceBytes(N, K));
  if (hcDequantW8(c, w, workspace, K, N, ldw, wsPitch))
    return 1;
  const bool pair = c->gemmVariant == 2 || (c->gemmVariant != 1 && M > kUmmaBM);
  return launchUmma(c, a, workspace, scale, dsts->base[0], M, N, K, lda, wsPitch, ldc, pair,
                    dsts);
}

// The banded form's part of the workspace: a ring of kBandSlots bands of
// kBandCols converted columns, and two counters per band.
size_t hcGemmW8A16BandedBytes(long long N, long long K) {
  if (N <= 0 || K <= 0)
    return 0;
  const size_t bands = size_t(ceilDiv(N, (long long)kBandCols));
  return size_t(kBandSlots) * size_t(K) * kBandCols * 2 + roundUp(bands * 8, 256);
}

size_t hcGemmW8A16WorkspaceBytes(long long N, long long K) {
  if (N <= 0 || K <= 0)
    return 0;
  return size_t(roundUp(N, 16)) * size_t(K) * 2;
}

int hcDequantW8(HcContext c, const void *w, void *out, long long rows,
                long long cols, long long wPitch, long long outPitch) {
  if (!c)
    return 1;
  if (rows < 0 || cols < 0 || wPitch < cols || outPitch < cols)
    return c->fail("hcDequantW8: invalid shape %lld x %lld", rows, cols);
  if (rows == 0 || cols == 0)
    return 0;
  if (!w || !out)
    return c->fail("hcDequantW8: null buffer");
  int vec = cols % 16 == 0 && wPitch % 16 == 0 && outPitch % 16 == 0 &&
            aligned(w, 16) && aligned(out, 16);
  long long perRow = vec ? cols / 16 : cols;
  long long gx = std::max<long long>(
      1, std::min<long long>(ceilDiv(perRow, 256), c->smCount * 8));
  // Each thread converts four rows (one batch of four loads in flight); one
  // CTA row per batch rather than a persistent grid, as for the softmax.
  long long gy = std::max<long long>(1, std::min<long long>(ceilDiv(rows, 4), 65535));
  void *args[] = {&w, &out, &rows, &cols, &wPitch, &outPitch, &vec};
  return c->launch("hc_dequant_w8_bf16", size_t(gx), size_t(gy), 1, 256, args, 7,
                   0);
}

int hcGemmW8A16(HcContext c, const void *a, const void *w, const float *scale,
                void *out, void *workspace, size_t workspaceBytes, long long M,
                long long N, long long K, long long lda, long long ldw,
                long long ldc) {
  if (!c)
    return 1;
  if (checkGemmShape(c, "hcGemmW8A16", a, w, out, M, N, K, lda, ldw, ldc))
    return 1;
  if (M == 0 || N == 0)
    return 0;
  if (!scale)
    return c->fail("hcGemmW8A16: null scale");
  // Conversion inside the pipeline (gemm_w8a16_umma.cu): a CTA pair per 256 x 256
  // tile, TMA boxes of A (bf16) and of w (bytes).
  const bool fusedFits = c->ccMajor == 10 && K > 0 && M > kUmmaBM && lda % 8 == 0 &&
                         ldw % 16 == 0 && N % 16 == 0 && aligned(a, 16) && aligned(w, 16) &&
                         (c->gemmVariant == 0 || c->gemmVariant == 2);
  if (c->w8Variant == 2 && !fusedFits)
    return c->fail("hcGemmW8A16: the layout does not allow converting in the pipeline "
                   "(tcgen05 device, M > 128, lda %% 8 == 0, N and ldw multiples of 16, 16-byte "
                   "aligned a and w)");
  if (fusedFits && c->w8Variant == 2) {
    alignas(64) CUtensorMap mapA, mapW;
    if (olxEncodeTensorMap2D(c->device, &mapA, /*bf16*/ 0, a, size_t(M), size_t(K),
                             size_t(lda) * 2, kUmmaBM, kUmmaBK, 128) ||
        olxEncodeTensorMap2D(c->device, &mapW, /*bytes*/ 2, w, size_t(K), size_t(N), size_t(ldw),
                             kUmmaBK, 128, 0))
      return c->fail("tensor map encoding failed: %s", c->lastError.c_str());
    int tilesM = int(ceilDiv(M, 2 * kUmmaBM)), tilesN = int(ceilDiv(N, kUmmaBN));
    int bandM = c->gemmBand ? int(c->gemmBand) : 16;
    int vecStore = aligned(out, 16) && ldc % 8 == 0;
    const long long tiles = (long long)tilesM * tilesN;
    const size_t smem = 5 * 32 * 1024 /*stages*/ + 8 * 8 * 1024 /*int8 tiles*/ + 1024 /*align*/ +
                        512 /*barriers*/;
    const char *name = "hc_gemm_w8a16_umma_pair";
    if (c->pairSlotsW8 == 0) {
      OlKernel k = c->kernel(name);
      int slots = 0;
      if (!k || olxMaxActiveClusters(c->queue, k, 480, smem, 2, &slots) || slots <= 0)
        return c->fail("cluster occupancy query failed: %s", c->lastError.c_str());
      c->pairSlotsW8 = slots;
    }
    const long long grid = 2 * std::min<long long>(tiles, c->pairSlotsW8);
    void *args[] = {&mapA, &mapW, &out, &scale, &M, &N, &K, &ldc, &tilesM, &tilesN, &bandM,
                    &vecStore, &c->statusWord};
    return c->launch(name, size_t(grid), 1, 1, 480, args, 13, smem);
  }
  // Conversion inside the GEMM kernel, band by band (hc_gemm_w8a16_umma_banded):
  // the converted weights live in a ring of three bands of 1024 columns.
  const size_t bandedBytes = hcGemmW8A16BandedBytes(N, K);
  const bool bandedFits = fusedFits && K % kUmmaBK == 0 && N >= 4 * kBandCols && workspace &&
                          aligned(workspace, 256) && workspaceBytes >= bandedBytes &&
                          (long long)kBandSlots * K < (1ll << 31);
  if (c->w8Variant == 3 && !bandedFits)
    return c->fail("hcGemmW8A16: the banded form needs a tcgen05 device, M > 128, K %% 64 == 0, "
                   "N >= %d and a multiple of 16, lda %% 8 == 0, ldw %% 16 == 0, 16-byte aligned "
                   "a and w, and a 256-byte aligned workspace of %zu bytes",
                   4 * kBandCols, bandedBytes);
  if (bandedFits && c->w8Variant == 3) {
    int tilesM = int(ceilDiv(M, 2 * kUmmaBM)), tilesN = int(ceilDiv(N, kUmmaBN));
    HcBandPlan plan{};
    plan.w = static_cast<const int8_t *>(w);
    plan.ldw = ldw;
    plan.ring = workspace;
    plan.bandTiles = kBandCols / kUmmaBN;
    plan.numBands = int(ceilDiv(tilesN, plan.bandTiles));
    plan.slots = kBandSlots;
    const size_t ringBytes = size_t(kBandSlots) * size_t(K) * kBandCols * 2;
    plan.converted = reinterpret_cast<unsigned *>(static_cast<char *>(workspace) + ringBytes);
    plan.consumed = plan.converted + plan.numBands;
    if (olxMemsetD8(c->queue, plan.converted, 0, size_t(plan.numBands) * 2 * sizeof(unsigned)))
      return c->fail("hcGemmW8A16: clearing the band counters failed: %s", c->lastError.c_str());
    alignas(64) CUtensorMap mapA, mapB;
    if (olxEncodeTensorMap2D(c->device, &mapA, /*bf16*/ 0, a, size_t(M), size_t(K),
                             size_t(lda) * 2, kUmmaBM, kUmmaBK, 128) ||
        olxEncodeTensorMap2D(c->device, &mapB, /*bf16*/ 0, workspace, size_t(kBandSlots) * K,
                             size_t(kBandCols), size_t(kBandCols) * 2, kUmmaBK, 64, 128))
      return c->fail("tensor map encoding failed: %s", c->lastError.c_str());
    int bandM = 16; // unused by the band-by-band tile order
    int vecStore = aligned(out, 16) && ldc % 8 == 0;
    const char *name = "hc_gemm_w8a16_umma_banded";
    if (c->pairSlotsBanded == 0) {
      OlKernel k = c->kernel(name);
      int slots = 0;
      if (!k || olxMaxActiveClusters(c->queue, k, kUmmaThreads + 128, kUmmaSmemBytes, 2, &slots) ||
          slots <= 0)
        return c->fail("cluster occupancy query failed: %s", c->lastError.c_str());
      c->pairSlotsBanded = slots;
    }
    // Every CTA converts a share of every band, so all of the grid has to be
    // resident at once: never more clusters than the device holds.
    const long long tiles = (long long)tilesM * tilesN;
    const long long grid = 2 * std::min<long long>(tiles, c->pairSlotsBanded);
    void *args[] = {&mapA, &mapB, &out, &scale, &M, &N, &K, &ldc, &tilesM, &tilesN, &bandM,
                    &vecStore, &c->statusWord, &plan};
    return c->launch(name, size_t(grid), 1, 1, kUmmaThreads + 128, args, 14, kUmmaSmemBytes);
  }
  const long long wsPitch = roundUp(N, 16);
  if (c->gemmVariant == 3 || !ummaEligible(c, a, workspace, K, lda, wsPitch)) {
    void *args[] = {&a, &w, &scale, &out, &M, &N, &K, &lda, &ldw, &ldc};
    return c->launch("hc_gemm_tiled_w8a16", size_t(ceilDiv(N, 64)),
                     size_t(ceilDiv(M, 64)), 1, 256, args, 10, 0);
  }
  if (!workspace || workspaceBytes < hcGemmW8A16WorkspaceBytes(N, K))
    return c->fail("hcGemmW8A16: workspace of %zu bytes is too small, need %zu",
                   workspaceBytes, hcGemmW8A16WorkspaceBytes(N, K));
  if (hcDequantW8(c, w, workspace, K, N, ldw, wsPitch))
    return 1;
  // A CTA pair per 256 x 256 tile moves a third less data per CTA than one CTA
  // per 128 x 256 tile; it needs at least two row blocks to be worth a cluster.
  const bool pair = c->gemmVariant == 2 || (c->gemmVariant == 0 && M > kUmmaBM);
  return launchUmma(c, a, workspace, scale, out, M, N, K, lda, wsPitch, ldc, pair);
}

} // extern "C"
