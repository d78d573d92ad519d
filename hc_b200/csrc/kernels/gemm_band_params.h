// Parameter block of the dequantising GEMM that converts its weights inside the
// kernel, band by band (hc_gemm_w8a16_umma_banded in gemm_bf16_umma.cu), shared
// by the kernel and the host code that fills it.
#pragma once

#include <stdint.h>

// The int8 weights w [K, N] are converted to bf16 one band of `bandTiles` tile
// columns (256 columns each) at a time into a ring of `slots` band-sized buffers
// ([K, bandTiles * 256] each, one after the other), by extra warps of every CTA
// that run ahead of the tiles; the tiles go band by band and read B from the
// ring.  Two counters per band, zero at launch, order the two sides: `converted`
// (warps that have written their share of the band) and `consumed` (tiles of the
// band whose MMAs are complete, so that its slot may be overwritten).
struct HcBandPlan {
  const int8_t *w;
  long long ldw;
  void *ring; // bf16
  unsigned *converted;
  unsigned *consumed;
  int32_t bandTiles, numBands, slots;
};
