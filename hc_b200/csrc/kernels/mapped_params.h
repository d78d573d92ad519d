// Kernel parameter block of the gathered tile product (mapped_gemm.cu), shared
// by the kernel and by the host code that fills it, so both see one layout.
#pragma once

#include <stdint.h>

// One array as a work-group sees it through an index mapping.  Ranks below 4
// are padded: shape 1, stride 0, origin 0, relative index 0.
struct HcMappedOperandDev {
  void *base;             // element [0, 0, 0, 0] of the array
  const int32_t *map;     // [tile elements][4]: index relative to the tile origin
  const int32_t *lin;     // [tile elements]: sum(map[d] * stride[d]), in elements
  const int32_t *origins; // [groups][4]: tile origin of every work-group
  int32_t shape[4];
  int64_t stride[4]; // in elements
  int32_t lo[4];     // smallest relative index per dimension over the tile
  int32_t hi[4];     // largest relative index per dimension over the tile
  // Order of the tile elements in `map` and `lin`: 0 = row-major of the tile as
  // the kernel body declares it, 1 = transposed.  The kernel walks an operand
  // in table order, so the host picks the order in which neighbouring elements
  // are neighbours in memory.
  int32_t transposed;
  // Work-groups g with equal g / sharedRun have the same tile origin in this
  // array (0 or 1: nothing known).  Read for f only: such groups multiply
  // against one and the same B tile, so one CTA can take several of them.
  int32_t sharedRun;
};

struct HcMappedGemmParams {
  HcMappedOperandDev x, f, out; // tiles [TM, K], [K, TN], [TM, TN]
  int32_t TM, TN, K;
  int32_t stack;  // consecutive work-groups one CTA computes, stacked along the rows
  int64_t groups; // work-groups in all
};
