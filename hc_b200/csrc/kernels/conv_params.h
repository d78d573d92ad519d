// Kernel parameter block of the tensor-core convolution (conv_f32_umma.cu),
// shared by the kernel and the host code that fills it.
#pragma once

#include <stdint.h>

// out[n, q, oh, ow] = sum over (c, kh, kw) of
//   x[n, c, oh * stride + kh, ow * stride + kw] * f[q, c, kh, kw]
// x [N, C, H, W], f [NF, C, HF, WF], out [N, NF, HO, WO], all float32 and
// contiguous; no padding: HO = (H - HF) / stride + 1, WO likewise.
struct HcConvParams {
  const void *x;   // the image as (hi, lo) float pairs (hc_split_tf32_pairs), layout of x
  float *out;
  int32_t N, C, H, W;
  int32_t NF, HF, WF, stride;
  int32_t HO, WO;
  int32_t K;             // C * HF * WF, the reduction length
  int32_t kBlocks;       // ceil(K / 32)
  int32_t nPad;          // NF rounded up to 16: the N of the MMA
  int32_t tilesPerImage; // ceil(HO * WO / 128)
  int32_t stages;        // shared-memory stages the launch has room for
  int32_t stacked;       // 1: a_hi * [b_hi; b_lo] as one MMA of width 2 nPad (nPad <= 128)
  int *status;           // the context's status word
};

// Parameter block of the convolution whose image tiles come by TMA
// (conv_f32_taps.cu): stride 1, the image rewritten as [N, H, W, Cp] (hi and lo),
// the filters as [NF, taps * Cp]; the tensor maps are kernel arguments of their own.
struct HcConvTapParams {
  float *out;
  int32_t N, C, H, W;
  int32_t NF, HF, WF;
  int32_t HO, WO;
  int32_t cBlocks;        // Cp / 32
  int32_t kBlocks;        // HF * WF * cBlocks
  int32_t nPad;           // NF rounded up to 16: the N of the MMA
  int32_t boxW, boxH;     // the tile's rectangle of output pixels, boxW * boxH = 128
  int32_t tilesW, tilesH; // tiles per image along W and H
  int32_t stages;         // shared-memory stages the launch has room for
  int32_t stacked;        // 1: a_hi * [b_hi; b_lo] as one MMA of width 2 nPad (nPad <= 128)
  int *status;            // the context's status word
  // hc_conv_f32_rows only: tiles of 128 consecutive positions of the flattened
  // image (oh * W + ow) and the rows of a stage's image patch, 128 + WF - 1
  // rounded up to 8.
  int32_t tilesFlat, patchRows;
};
