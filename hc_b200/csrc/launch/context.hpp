// The context behind an HcContext handle, shared by the translation units of
// libhc-b200-kernels.so.
#pragma once

#include "hc_b200_kernels.h"

#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <map>
#include <string>
#include <vector>

struct HcContextImpl {
  OlErrorCallback callback = nullptr;
  void *callbackCtx = nullptr;
  OlDevice device = nullptr;
  OlQueue queue = nullptr;
  std::vector<OlModule> modules; // one slot per image, loaded on first use
  std::map<std::string, OlKernel> kernels;
  int *statusWord = nullptr; // device
  std::string lastError;
  long long launches = 0;
  long long smCount = 0;
  long long ccMajor = 0;
  long long ccMinor = 0;
  long long gemmVariant = 0;
  long long softmaxVariant = 0; // 0 auto, 1 register kernel, 2 bulk-copy pipeline
  long long tiledVariant = 0;
  long long reduceVariant = 0;
  long long mappedStack = 0;
  long long rowVariant = 0;
  long long fusedVariant = 0; // 1: never use the precompiled bodies
  long long gemmBand = 0;     // row tiles per band of the tcgen05 GEMMs' tile order (0: default)
  long long convVariant = 0;  // 1: image operand in shared memory, 2: in tensor memory
  long long convStacked = 0;  // 1: never run a_hi * [b_hi; b_lo] as one MMA of double width
  long long convStages = 0;   // 2..6: pipeline stages of the convolution (0: as many as fit)
  long long pairSlots = 0; // CTA pairs of the tcgen05 kernels resident at once
  int pairSlotsF32 = 0; // the same for the float32 tensor-core kernel
  int pairSlotsBanded = 0; // the same for the dequant GEMM that converts band by band
  int pairSlotsW8 = 0;  // the same for the dequant GEMM that converts in its pipeline
  long long w8Variant = 0; // 1: convert the weights in a pass of its own, 2: never
  // Programs without a precompiled body: 0 interpret them, 1 compile them at their
  // first launch and interpret where that is not possible, 2 fail where it is not.
  long long specialiseMode = 1;
  struct HcSpecialiser *specialiser = nullptr; // specialise.cpp

  int fail(const char *fmt, ...) __attribute__((format(printf, 2, 3))) {
    char text[320];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(text, sizeof(text), fmt, ap);
    va_end(ap);
    lastError = text;
    if (callback)
      callback(callbackCtx, OlSeverity::Error, text);
    return 1;
  }

  // ol* failures arrive here through the loader/backend callback.
  static void onBackendMessage(void *self, OlSeverity sev, const char *desc) {
    auto *c = static_cast<HcContextImpl *>(self);
    if (sev == OlSeverity::Error)
      c->lastError = desc ? desc : "";
    if (c->callback)
      c->callback(c->callbackCtx, sev, desc);
  }

  // The kernel `name` from the embedded images (loaded on first use), or null.
  OlKernel kernel(const char *name);
  // Launches `name` with a one-dimensional block on the context's queue.
  int launch(const char *name, size_t gx, size_t gy, size_t gz, size_t threads, void **args,
             size_t nArgs, size_t smem);
  // Scratch of the host-buffer entry points (host_api.cpp), released with the context.
  struct HostPipeline *hostPipeline = nullptr;
};

// Frees what the host-buffer entry points keep in a context (host_api.cpp).
void hcReleaseHostPipeline(HcContextImpl *c);

// Run-time specialisation (specialise.cpp).
struct HcMapProgramDev;
bool hcSpecialisable(const HcMapProgramDev &p, bool row, int dtype);
const char *hcSpecialise(HcContextImpl *c, bool row, int dtype, const HcMapProgramDev &p);
const char *hcSpecialiseItems(HcContextImpl *c, int dtype, const uint32_t *code, int nInstr,
                              bool wide);
const char *hcSpecialiserNote(HcContextImpl *c);
long long hcSpecialiserCount(HcContextImpl *c, int which);
void hcReleaseSpecialiser(HcContextImpl *c);
