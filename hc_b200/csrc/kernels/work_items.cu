// Work-item kernels: bodies written at work-item level that need more than an
// element-wise pass - the work-item's local id as a value, reads of a
// neighbour's element, and two phases separated by group.barrier() that
// exchange values through a tile of the work-group (the reference's
// CurrentGroup.workitems / barrier, python/hckernel/kernel_api.py:395-431; its
// lowering puts group tiles in work-group memory,
// mlir/lib/Transforms/LowerScope.cpp:246-309).
//
// One thread per work-item, one CTA per work-group, exactly the reference's
// execution model; the group's tile lives in shared memory and the barrier is
// the CTA barrier.  The body arrives as a program for the accumulator machine
// of map_params.h, interpreted on single values (items_params.h).  A work-item
// outside a phase's guard (the `if gid < n` of the body) computes nothing in
// that phase but still takes part in the barrier, as in the reference, where
// every work-item of a group runs to the barrier.
#include "items_params.h"
#include "map_machine.cuh"

namespace {

using namespace hcmap;

template <typename T>
__device__ __forceinline__ void workItems(const HcItemProgramDev &p) {
  extern __shared__ __align__(16) unsigned char raw[];
  T *const tile = reinterpret_cast<T *>(raw);
  using N = Num<T>;
  const int localCol = threadIdx.x % p.groupCols, localRow = threadIdx.x / p.groupCols;
  const int groupsX = int((p.cols + p.groupCols - 1) / p.groupCols);
  const long long row = (long long)(blockIdx.x / groupsX) * p.groupRows + localRow;
  const long long col = (long long)(blockIdx.x % groupsX) * p.groupCols + localCol;
  tile[threadIdx.x] = T(p.tileFill);
  __syncthreads();

  int phase = 0;
  auto inside = [&]() {
    return row >= p.guardLo[phase][0] && row < p.guardHi[phase][0] &&
           col >= p.guardLo[phase][1] && col < p.guardHi[phase][1];
  };
  bool active = inside();
  T acc = T(0), temps[3] = {T(0), T(0), T(0)};
  for (int pc = 0; pc < p.nInstr; ++pc) {
    const uint32_t ins = p.code[pc], op = ins & 0xffu, src = (ins >> 8) & 0xffu;
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

} // namespace

extern "C" __global__ void __launch_bounds__(1024)
    hc_work_items_f32(const __grid_constant__ HcItemProgramDev p) {
  workItems<float>(p);
}
extern "C" __global__ void __launch_bounds__(1024)
    hc_work_items_f64(const __grid_constant__ HcItemProgramDev p) {
  workItems<double>(p);
}
