// Parameter block of the work-item kernel (work_items.cu), shared by the kernel
// and by the host code that fills it.
#pragma once

#include "map_params.h"

// A work-item program runs once per work-item, one thread each, one CTA per
// work-group.  It uses the operations of the element-wise machine
// (map_params.h: one accumulator, three temporaries) on single values, plus:
enum HcItemOp : uint32_t {
  HC_ITEM_STORE_TILE = 64, // tile[local id] = acc        (the group's tile in shared memory)
  HC_ITEM_BARRIER = 65,    // group.barrier(): every work-item of the group waits here
  HC_ITEM_STORE_OUT = 66,  // out[global id] = acc, if the work-item passes the phase's guard
};
// Operand names beyond those of map_params.h: the local row / column index as a
// value, and reads of the group's tile at a mapped local index (table entry
// src - HC_ITEM_SRC_TILE).
constexpr uint32_t HC_ITEM_SRC_LOCAL_ROW = 18, HC_ITEM_SRC_LOCAL_COL = 19;
constexpr uint32_t HC_ITEM_SRC_TILE = 24;
constexpr int HC_ITEM_MAX_INSTR = 48, HC_ITEM_MAX_TILE_READS = 4, HC_ITEM_MAX_PHASES = 2;
// A CTA works on several consecutive work-groups at a time (one pass): a kernel
// compiled for work-groups of up to HC_ITEM_WIDE_THREADS work-items takes
// HC_ITEM_WIDE_BYTES / element size of them, every other kernel
// HC_ITEM_NARROW_GROUPS.  The launch gives the kernel one tile per group of a
// pass in shared memory.
constexpr int HC_ITEM_WIDE_THREADS = 256, HC_ITEM_WIDE_BYTES = 32, HC_ITEM_NARROW_GROUPS = 2;

struct HcItemProgramDev {
  const void *in[HC_MAP_MAX_INPUTS]; // read at (row + inRow[k], col + inCol[k])
  int64_t inPitch[HC_MAP_MAX_INPUTS];
  int32_t inRow[HC_MAP_MAX_INPUTS], inCol[HC_MAP_MAX_INPUTS];
  void *out;
  int64_t outPitch;
  int64_t rows, cols;           // the work shape (rows = 1 for one-dimensional work)
  int32_t groupRows, groupCols; // work-group shape; groupRows * groupCols threads per CTA
  int32_t nInputs, nInstr;
  uint32_t code[HC_ITEM_MAX_INSTR];
  double consts[HC_MAP_MAX_CONSTS];
  // A work-item takes part in the reads and stores of phase p (the instructions
  // before / after the barrier) only if guardLo[p][a] <= global id[a] < guardHi[p][a].
  int64_t guardLo[HC_ITEM_MAX_PHASES][2], guardHi[HC_ITEM_MAX_PHASES][2];
  // Tile read k: element (tileScale * local id + tileOffset) mod tileMod per axis
  // (tileMod 0: no wrap); [k][0] rows, [k][1] columns.
  int32_t tileScale[HC_ITEM_MAX_TILE_READS][2], tileOffset[HC_ITEM_MAX_TILE_READS][2],
      tileMod[HC_ITEM_MAX_TILE_READS][2];
  double tileFill; // what the group's tile holds before anything is stored to it
  // Filled by the launch, not by the caller.  The grid of work-groups, and the
  // groups all of whose work-items pass the guards of every phase of the program:
  // insideLo[a] <= group coordinate[a] < insideHi[a] ([0] rows, [1] columns).
  uint32_t groupsY, groupsX;
  uint32_t insideLo[2], insideHi[2];
};
