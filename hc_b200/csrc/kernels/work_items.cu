// Work-item kernels: bodies written at work-item level that need more than an
// element-wise pass - the work-item's local id as a value, reads of a
// neighbour's element, and two phases separated by group.barrier() that
// exchange values through a tile of the work-group (the reference's
// CurrentGroup.workitems / barrier, python/hckernel/kernel_api.py:395-431; its
// lowering puts group tiles in work-group memory,
// mlir/lib/Transforms/LowerScope.cpp:246-309).
//
// One thread per work-item, a CTA per work-group at a time (a CTA takes the
// groups blockIdx.x, blockIdx.x + gridDim.x, ... in turn: a group of 256
// work-items is too little work to pay for a CTA of its own), the reference's
// execution model; the group's tile lives in shared memory and the barrier is
// the CTA barrier.  The body arrives as a program for the accumulator machine
// of map_params.h, interpreted on single values (items_params.h).  A work-item
// outside a phase's guard (the `if gid < n` of the body) computes nothing in
// that phase but still takes part in the barrier, as in the reference, where
// every work-item of a group runs to the barrier.
//
// FIXED: the program is a compile-time constant (a type with `n` and `code[n]`,
// as in fused_programs.h) and the instruction loop is unrolled, so that every
// decision the interpreter takes per instruction and work-item is taken by the
// compiler - the form that a run-time specialisation compiles
// (launch/specialise.cpp).  Same operations in the same order: same results.
#include "items_params.h"
#include "map_machine.cuh"
#ifdef HC_ITEM_FIXED_PROGRAM
#include "fused_programs.h"
#endif

namespace {

using namespace hcmap;

struct Interpreted {}; // the program is read from the parameter block

template <typename T, typename P>
__device__ __forceinline__ void workGroup(const HcItemProgramDev &p, T *tile, int localRow,
                                          int localCol, long long row, long long col) {
  using N = Num<T>;
  constexpr bool fixed = !std::is_same<P, Interpreted>::value;
  int phase = 0;
  auto inside = [&]() {
    return row >= p.guardLo[phase][0] && row < p.guardHi[phase][0] &&
           col >= p.guardLo[phase][1] && col < p.guardHi[phase][1];
  };
  bool active = inside();
  T acc = T(0), temps[3] = {T(0), T(0), T(0)};
  int count;
  if constexpr (fixed)
    count = P::n;
  else
    count = p.nInstr;
#pragma unroll
  for (int pc = 0; pc < count; ++pc) {
    uint32_t ins;
    if constexpr (fixed)
      ins = P::code[pc];
    else
      ins = p.code[pc];
    const uint32_t op = ins & 0xffu, src = (ins >> 8) & 0xffu;
    if (op == HC_ITEM_BARRIER) {
      __syncthreads(); // uniform: every thread of the CTA runs the same instructions
      phase = 1;
      active = inside();
      continue;
    }
    if (!active)
      continue;
    if (op == HC_ITEM_STORE_TILE) {
      tile[threadIdx.x] = acc;
      continue;
    }
    if (op == HC_ITEM_STORE_OUT) {
      static_cast<T *>(p.out)[row * p.outPitch + col] = acc;
      continue;
    }
    if (hcMapIsBinary(op)) {
      T v;
      if (src < HC_MAP_SRC_TEMP) {
        v = static_cast<const T *>(p.in[src])[(row + p.inRow[src]) * p.inPitch[src] + col +
                                              p.inCol[src]];
      } else if (src < HC_MAP_SRC_CONST) {
        v = temps[src - HC_MAP_SRC_TEMP];
      } else if (src < HC_MAP_SRC_ROW) {
        v = T(p.consts[src - HC_MAP_SRC_CONST]);
      } else if (src == HC_MAP_SRC_ROW) {
        v = T(row);
      } else if (src == HC_MAP_SRC_COL) {
        v = T(col);
      } else if (src == HC_ITEM_SRC_LOCAL_ROW) {
        v = T(localRow);
      } else if (src == HC_ITEM_SRC_LOCAL_COL) {
        v = T(localCol);
      } else {
        const int k = int(src - HC_ITEM_SRC_TILE);
        int r = p.tileScale[k][0] * localRow + p.tileOffset[k][0];
        int c = p.tileScale[k][1] * localCol + p.tileOffset[k][1];
        if (p.tileMod[k][0])
          r = ((r % p.tileMod[k][0]) + p.tileMod[k][0]) % p.tileMod[k][0];
        if (p.tileMod[k][1])
          c = ((c % p.tileMod[k][1]) + p.tileMod[k][1]) % p.tileMod[k][1];
        v = tile[r * p.groupCols + c]; // the host has checked that (r, c) lies inside
      }
      switch (op) {
      case HC_MAP_LOAD: acc = v; break;
      case HC_MAP_ADD: acc = addOf(acc, v); break;
      case HC_MAP_SUB: acc = subOf(acc, v); break;
      case HC_MAP_RSUB: acc = subOf(v, acc); break;
      case HC_MAP_MUL: acc = mulOf(acc, v); break;
      case HC_MAP_DIV: acc = N::div(acc, v); break;
      case HC_MAP_RDIV: acc = N::div(v, acc); break;
      case HC_MAP_MAX: acc = maxOf(acc, v); break;
      case HC_MAP_MIN: acc = minOf(acc, v); break;
      case HC_MAP_FLOORDIV: acc = N::floordiv(acc, v); break;
      case HC_MAP_RFLOORDIV: acc = N::floordiv(v, acc); break;
      case HC_MAP_MOD: acc = N::mod(acc, v); break;
      case HC_MAP_RMOD: acc = N::mod(v, acc); break;
      case HC_MAP_POW: acc = N::pow(acc, v); break;
      case HC_MAP_RPOW: acc = N::pow(v, acc); break;
      case HC_MAP_LT: acc = T(acc < v); break;
      case HC_MAP_LE: acc = T(acc <= v); break;
      case HC_MAP_EQ: acc = T(acc == v); break;
      case HC_MAP_NE: acc = T(acc != v); break;
      case HC_MAP_GE: acc = T(acc >= v); break;
      case HC_MAP_GT: acc = T(acc > v); break;
      case HC_MAP_AND: acc = N::bitAnd(acc, v); break;
      case HC_MAP_OR: acc = N::bitOr(acc, v); break;
      default: acc = N::bitXor(acc, v); break;
      }
      continue;
    }
    switch (op) {
    case HC_MAP_NEG: acc = negOf(acc); break;
    case HC_MAP_ABS: acc = N::absOf(acc); break;
    case HC_MAP_EXP: acc = N::exp(acc); break;
    case HC_MAP_SQRT: acc = N::sqrtOf(acc); break;
    case HC_MAP_LOG: acc = N::log(acc); break;
    case HC_MAP_INV: acc = N::inv(acc); break;
    case HC_MAP_SAVE0: temps[0] = acc; break;
    case HC_MAP_SAVE1: temps[1] = acc; break;
    case HC_MAP_SAVE2: temps[2] = acc; break;
    default: break;
    }
  }
}

template <typename T, typename P>
__device__ __forceinline__ void workItems(const HcItemProgramDev &p) {
  extern __shared__ __align__(16) unsigned char raw[];
  T *const tile = reinterpret_cast<T *>(raw);
  const int localCol = threadIdx.x % p.groupCols, localRow = threadIdx.x / p.groupCols;
  const long long groupsX = (p.cols + p.groupCols - 1) / p.groupCols;
  const long long groups = groupsX * ((p.rows + p.groupRows - 1) / p.groupRows);
  for (long long g = blockIdx.x; g < groups; g += gridDim.x) {
    const long long row = (g / groupsX) * p.groupRows + localRow;
    const long long col = (g % groupsX) * p.groupCols + localCol;
    tile[threadIdx.x] = T(p.tileFill);
    __syncthreads();
    workGroup<T, P>(p, tile, localRow, localCol, row, col);
    __syncthreads(); // the tile belongs to the next group from here on
  }
}

} // namespace

#ifndef HC_ITEM_FIXED_PROGRAM
extern "C" __global__ void __launch_bounds__(1024)
    hc_work_items_f32(const __grid_constant__ HcItemProgramDev p) {
  workItems<float, Interpreted>(p);
}
extern "C" __global__ void __launch_bounds__(1024)
    hc_work_items_f64(const __grid_constant__ HcItemProgramDev p) {
  workItems<double, Interpreted>(p);
}
#else
// One program, one element type (HC_FUSED_ONLY: 0 float32, 1 float64), named by
// the list macro of the generated header.
#if HC_FUSED_ONLY == 0
#define HC_ITEM_FIXED(body)                                                              \
  extern "C" __global__ void __launch_bounds__(1024)                                     \
      hc_work_items_fused_##body##_f32(const __grid_constant__ HcItemProgramDev p) {     \
    workItems<float, hcfused::item_##body>(p);                                           \
  }
#else
#define HC_ITEM_FIXED(body)                                                              \
  extern "C" __global__ void __launch_bounds__(1024)                                     \
      hc_work_items_fused_##body##_f64(const __grid_constant__ HcItemProgramDev p) {     \
    workItems<double, hcfused::item_##body>(p);                                          \
  }
#endif
HC_FUSED_ITEM_LIST(HC_ITEM_FIXED)
#endif
