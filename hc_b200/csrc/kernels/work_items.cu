// Work-item kernels: bodies written at work-item level that need more than an
// element-wise pass - the work-item's local id as a value, reads of a
// neighbour's element, and two phases separated by group.barrier() that
// exchange values through a tile of the work-group (the reference's
// CurrentGroup.workitems / barrier, python/hckernel/kernel_api.py:395-431; its
// lowering puts group tiles in work-group memory,
// mlir/lib/Transforms/LowerScope.cpp:246-309).
//
// One thread per work-item and a CTA of the work-group's size, the reference's
// execution model; the group's tile lives in shared memory and the barrier is
// the CTA barrier.  A CTA works on U consecutive work-groups at a time - thread t
// is work-item t of each of them, with U tiles side by side in shared memory -
// and takes such sets of groups in turn (blockIdx.x, blockIdx.x + gridDim.x, ...).
// A work-item reads one element per input, so a single group per CTA leaves
// four bytes in flight per thread and three CTA barriers per 256 elements; with
// U groups the U loads of a thread are independent and the barriers are shared.
// Nothing in the model orders work-groups against one another, so this is the
// same computation.
//
// The body arrives as a program for the accumulator machine of map_params.h,
// interpreted on single values (items_params.h).  A work-item outside a phase's
// guard (the `if gid < n` of the body) loads and stores nothing in that phase
// (its arithmetic runs on zeros and is dropped) but still takes part in the
// barrier, as in the reference, where every work-item of a group runs to the
// barrier.
//
// FIXED: the program is a compile-time constant (a type with `n` and `code[n]`,
// as in fused_programs.h) and the instruction loop is unrolled, so that every
// decision the interpreter takes per instruction and work-item is taken by the
// compiler - the form that a run-time specialisation compiles
// (launch/specialise.cpp), for work-groups of up to HC_ITEM_WIDE_THREADS
// work-items with more groups per pass (HC_ITEM_WIDE).  Same operations in the
// same order on every element: same results.
#include "items_params.h"
#include "map_machine.cuh"
#ifdef HC_ITEM_FIXED_PROGRAM
#include "fused_programs.h"
#endif

namespace {

using namespace hcmap;

struct Interpreted {}; // the program is read from the parameter block

// acc[u] = EXPR(a = acc[u], b = v[u]) for the U groups of the pass.
#define HC_ITEM_EACH(EXPR)                                                               \
  {                                                                                      \
    _Pragma("unroll") for (int u = 0; u < U; ++u) {                                      \
      const T a = acc[u], b = v[u];                                                      \
      acc[u] = (EXPR);                                                                   \
    }                                                                                    \
  }                                                                                      \
  break

// The element of the group's tile that tile read k of this work-item names.
__device__ __forceinline__ int tileElement(const HcItemProgramDev &p, int k, int localRow,
                                           int localCol) {
  int r = p.tileScale[k][0] * localRow + p.tileOffset[k][0];
  int c = p.tileScale[k][1] * localCol + p.tileOffset[k][1];
  if (p.tileMod[k][0])
    r = ((r % p.tileMod[k][0]) + p.tileMod[k][0]) % p.tileMod[k][0];
  if (p.tileMod[k][1])
    c = ((c % p.tileMod[k][1]) + p.tileMod[k][1]) % p.tileMod[k][1];
  return r * p.groupCols + c; // the host has checked that (r, c) lies inside
}

// One pass: work-item (localRow, localCol) of U work-groups side by side in one
// row of groups, whose global ids are (row[u], col[u]): row[u] = row[0] and
// col[u] = col[0] + u * groupCols, so an array is addressed from the element of
// group 0 in steps of groupCols.  FAST: the caller has seen that every work-item
// of the U groups passes the guards of every phase, so none is evaluated.
template <typename T, typename P, int U, bool FAST>
__device__ __forceinline__ void workGroups(const HcItemProgramDev &p, T *tile, int localRow,
                                           int localCol, const long long (&row)[U],
                                           const long long (&col)[U],
                                           const int (&tileAt)[HC_ITEM_MAX_TILE_READS]) {
  using N = Num<T>;
  constexpr bool fixed = !std::is_same<P, Interpreted>::value;
  const int threads = blockDim.x;
  auto inside = [&](int phase) {
    if constexpr (FAST)
      return (1u << U) - 1u;
    unsigned mask = 0;
#pragma unroll
    for (int u = 0; u < U; ++u)
      if (col[u] >= p.guardLo[phase][1] && col[u] < p.guardHi[phase][1])
        mask |= 1u << u;
    return row[0] >= p.guardLo[phase][0] && row[0] < p.guardHi[phase][0] ? mask : 0u;
  };
  unsigned active = inside(0);
  T acc[U], temps[3][U];
#pragma unroll
  for (int u = 0; u < U; ++u)
    acc[u] = temps[0][u] = temps[1][u] = temps[2][u] = T(0);
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
      active = inside(1);
      continue;
    }
    if (op == HC_ITEM_STORE_TILE) {
#pragma unroll
      for (int u = 0; u < U; ++u)
        if (FAST || (active >> u & 1u))
          tile[u * threads + threadIdx.x] = acc[u];
      continue;
    }
    if (op == HC_ITEM_STORE_OUT) {
      T *first = static_cast<T *>(p.out) + (row[0] * p.outPitch + col[0]);
#pragma unroll
      for (int u = 0; u < U; ++u)
        if (FAST || (active >> u & 1u))
          first[u * p.groupCols] = acc[u];
      continue;
    }
    if (hcMapIsBinary(op)) {
      T v[U];
      if (src < HC_MAP_SRC_TEMP) {
        const T *in = static_cast<const T *>(p.in[src]);
        const T *first = in + ((row[0] + p.inRow[src]) * p.inPitch[src] + col[0] + p.inCol[src]);
#pragma unroll
        for (int u = 0; u < U; ++u)
          v[u] = FAST || (active >> u & 1u) ? first[u * p.groupCols] : T(0);
      } else if (src < HC_MAP_SRC_CONST) {
        const int t = int(src - HC_MAP_SRC_TEMP);
#pragma unroll
        for (int u = 0; u < U; ++u)
          v[u] = t == 0 ? temps[0][u] : t == 1 ? temps[1][u] : temps[2][u];
      } else if (src < HC_MAP_SRC_ROW) {
#pragma unroll
        for (int u = 0; u < U; ++u)
          v[u] = T(p.consts[src - HC_MAP_SRC_CONST]);
      } else if (src == HC_MAP_SRC_ROW) {
#pragma unroll
        for (int u = 0; u < U; ++u)
          v[u] = T(row[0]);
      } else if (src == HC_MAP_SRC_COL) {
#pragma unroll
        for (int u = 0; u < U; ++u)
          v[u] = T(col[u]);
      } else if (src == HC_ITEM_SRC_LOCAL_ROW) {
#pragma unroll
        for (int u = 0; u < U; ++u)
          v[u] = T(localRow);
      } else if (src == HC_ITEM_SRC_LOCAL_COL) {
#pragma unroll
        for (int u = 0; u < U; ++u)
          v[u] = T(localCol);
      } else {
        const int k = int(src - HC_ITEM_SRC_TILE);
        int at;
        if constexpr (fixed)
          at = tileAt[k]; // k is a constant here: a register
        else
          at = tileElement(p, k, localRow, localCol);
#pragma unroll
        for (int u = 0; u < U; ++u)
          v[u] = tile[u * threads + at];
      }
      switch (op) {
      case HC_MAP_LOAD: HC_ITEM_EACH(((void)a, b));
      case HC_MAP_ADD: HC_ITEM_EACH(addOf(a, b));
      case HC_MAP_SUB: HC_ITEM_EACH(subOf(a, b));
      case HC_MAP_RSUB: HC_ITEM_EACH(subOf(b, a));
      case HC_MAP_MUL: HC_ITEM_EACH(mulOf(a, b));
      case HC_MAP_DIV: HC_ITEM_EACH(N::div(a, b));
      case HC_MAP_RDIV: HC_ITEM_EACH(N::div(b, a));
      case HC_MAP_MAX: HC_ITEM_EACH(maxOf(a, b));
      case HC_MAP_MIN: HC_ITEM_EACH(minOf(a, b));
      case HC_MAP_FLOORDIV: HC_ITEM_EACH(N::floordiv(a, b));
      case HC_MAP_RFLOORDIV: HC_ITEM_EACH(N::floordiv(b, a));
      case HC_MAP_MOD: HC_ITEM_EACH(N::mod(a, b));
      case HC_MAP_RMOD: HC_ITEM_EACH(N::mod(b, a));
      case HC_MAP_POW: HC_ITEM_EACH(N::pow(a, b));
      case HC_MAP_RPOW: HC_ITEM_EACH(N::pow(b, a));
      case HC_MAP_LT: HC_ITEM_EACH(T(a < b));
      case HC_MAP_LE: HC_ITEM_EACH(T(a <= b));
      case HC_MAP_EQ: HC_ITEM_EACH(T(a == b));
      case HC_MAP_NE: HC_ITEM_EACH(T(a != b));
      case HC_MAP_GE: HC_ITEM_EACH(T(a >= b));
      case HC_MAP_GT: HC_ITEM_EACH(T(a > b));
      case HC_MAP_AND: HC_ITEM_EACH(N::bitAnd(a, b));
      case HC_MAP_OR: HC_ITEM_EACH(N::bitOr(a, b));
      default: HC_ITEM_EACH(N::bitXor(a, b));
      }
      continue;
    }
    T v[U]; // unused by the unary operations
#pragma unroll
    for (int u = 0; u < U; ++u)
      v[u] = T(0);
    switch (op) {
    case HC_MAP_NEG: HC_ITEM_EACH(((void)b, negOf(a)));
    case HC_MAP_ABS: HC_ITEM_EACH(((void)b, N::absOf(a)));
    case HC_MAP_EXP: HC_ITEM_EACH(((void)b, N::exp(a)));
    case HC_MAP_SQRT: HC_ITEM_EACH(((void)b, N::sqrtOf(a)));
    case HC_MAP_LOG: HC_ITEM_EACH(((void)b, N::log(a)));
    case HC_MAP_INV: HC_ITEM_EACH(((void)b, N::inv(a)));
    case HC_MAP_SAVE0:
#pragma unroll
      for (int u = 0; u < U; ++u)
        temps[0][u] = acc[u];
      break;
    case HC_MAP_SAVE1:
#pragma unroll
      for (int u = 0; u < U; ++u)
        temps[1][u] = acc[u];
      break;
    case HC_MAP_SAVE2:
#pragma unroll
      for (int u = 0; u < U; ++u)
        temps[2][u] = acc[u];
      break;
    default: break;
    }
  }
}

// What the launch needs to know of the program: whether it touches the group's
// tile at all (else the tile is neither filled nor fenced by barriers of its
// own), whether every work-item stores to the tile before the barrier (then a
// pass whose work-items all pass the guards needs no fill), and its phases.
struct ProgramTraits {
  bool tiled, storesFirst;
  int phases;
};
template <typename P>
__device__ __forceinline__ ProgramTraits traitsOf(const HcItemProgramDev &p) {
  constexpr bool fixed = !std::is_same<P, Interpreted>::value;
  int count;
  if constexpr (fixed)
    count = P::n;
  else
    count = p.nInstr;
  ProgramTraits t = {false, false, 1};
#pragma unroll
  for (int pc = 0; pc < count; ++pc) {
    uint32_t ins;
    if constexpr (fixed)
      ins = P::code[pc];
    else
      ins = p.code[pc];
    const uint32_t op = ins & 0xffu, src = (ins >> 8) & 0xffu;
    t.tiled |= op == HC_ITEM_STORE_TILE || (hcMapIsBinary(op) && src >= HC_ITEM_SRC_TILE);
    t.storesFirst |= op == HC_ITEM_STORE_TILE && t.phases == 1;
    if (op == HC_ITEM_BARRIER)
      t.phases = 2;
  }
  return t;
}

template <typename T, typename P, int U>
__device__ __forceinline__ void workItems(const HcItemProgramDev &p) {
  extern __shared__ __align__(16) unsigned char raw[];
  T *const tile = reinterpret_cast<T *>(raw);
  const int threads = blockDim.x;
  const int localCol = threadIdx.x % p.groupCols, localRow = threadIdx.x / p.groupCols;
  // The launch keeps the number of work-groups below 2^31.
  const unsigned groupsX = p.groupsX, groups = p.groupsX * p.groupsY;
  const ProgramTraits traits = traitsOf<P>(p);
  int tileAt[HC_ITEM_MAX_TILE_READS];
#pragma unroll
  for (int k = 0; k < HC_ITEM_MAX_TILE_READS; ++k)
    tileAt[k] = tileElement(p, k, localRow, localCol);
  // Group coordinates advance by a fixed step from pass to pass.
  const unsigned long long step = (unsigned long long)gridDim.x * U;
  const unsigned stepY = unsigned(step) / groupsX, stepX = unsigned(step) % groupsX;
  const unsigned first = blockIdx.x * U;
  unsigned gy = first / groupsX, gx = first % groupsX;
  for (unsigned long long base = first; base < groups; base += step) {
    // The common pass: U groups side by side in one row of groups; all of their
    // work-items pass every guard (decided once for the CTA), or the pass touches
    // the edge of a guard and every work-item evaluates its own.
    const bool inRow = gx + U <= groupsX;
    const bool fast = inRow && gy >= p.insideLo[0] && gy < p.insideHi[0] &&
                      gx >= p.insideLo[1] && gx + U <= p.insideHi[1];
    const long long boxRow = (long long)gy * p.groupRows, boxCol = (long long)gx * p.groupCols;
    const unsigned passY = gy, passX = gx;
    gx += stepX, gy += stepY; // for the next pass
    if (gx >= groupsX)
      gx -= groupsX, ++gy;
    if (inRow) {
      long long row[U], col[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        row[u] = boxRow + localRow;
        col[u] = boxCol + u * p.groupCols + localCol;
      }
      if (traits.tiled && !(fast && traits.storesFirst)) {
#pragma unroll
        for (int u = 0; u < U; ++u)
          tile[u * threads + threadIdx.x] = T(p.tileFill);
        __syncthreads();
      }
      if (fast)
        workGroups<T, P, U, true>(p, tile, localRow, localCol, row, col, tileAt);
      else
        workGroups<T, P, U, false>(p, tile, localRow, localCol, row, col, tileAt);
    } else {
      // A pass that wraps to the next row of groups (or runs past the last
      // group): one group after the other.
      unsigned y = passY, x = passX;
#pragma unroll 1
      for (int u = 0; u < U && base + u < groups; ++u) {
        const long long row[1] = {(long long)y * p.groupRows + localRow};
        const long long col[1] = {(long long)x * p.groupCols + localCol};
        if (++x == groupsX) {
          x = 0;
          ++y;
        }
        if (traits.tiled) {
          if (u)
            __syncthreads(); // the tile belonged to the group before
          tile[threadIdx.x] = T(p.tileFill);
          __syncthreads();
        }
        workGroups<T, P, 1, false>(p, tile, localRow, localCol, row, col, tileAt);
      }
    }
    if (traits.tiled)
      __syncthreads(); // the tiles belong to the next groups from here on
  }
}

} // namespace

#ifndef HC_ITEM_FIXED_PROGRAM
extern "C" __global__ void __launch_bounds__(1024)
    hc_work_items_f32(const __grid_constant__ HcItemProgramDev p) {
  workItems<float, Interpreted, HC_ITEM_NARROW_GROUPS>(p);
}
extern "C" __global__ void __launch_bounds__(1024)
    hc_work_items_f64(const __grid_constant__ HcItemProgramDev p) {
  workItems<double, Interpreted, HC_ITEM_NARROW_GROUPS>(p);
}
#else
// One program, one element type (HC_FUSED_ONLY: 0 float32, 1 float64), named by
// the list macro of the generated header, for one class of work-group sizes
// (HC_ITEM_WIDE: up to HC_ITEM_WIDE_THREADS work-items, HC_ITEM_WIDE_BYTES of
// loads in flight per thread).
#ifdef HC_ITEM_WIDE
#define HC_ITEM_BOUNDS __launch_bounds__(HC_ITEM_WIDE_THREADS, 6)
#define HC_ITEM_GROUPS(T) (HC_ITEM_WIDE_BYTES / int(sizeof(T)))
#else
#define HC_ITEM_BOUNDS __launch_bounds__(1024)
#define HC_ITEM_GROUPS(T) HC_ITEM_NARROW_GROUPS
#endif
#if HC_FUSED_ONLY == 0
#define HC_ITEM_FIXED(body)                                                              \
  extern "C" __global__ void HC_ITEM_BOUNDS hc_work_items_fused_##body##_f32(            \
      const __grid_constant__ HcItemProgramDev p) {                                      \
    workItems<float, hcfused::item_##body, HC_ITEM_GROUPS(float)>(p);                    \
  }
#else
#define HC_ITEM_FIXED(body)                                                              \
  extern "C" __global__ void HC_ITEM_BOUNDS hc_work_items_fused_##body##_f64(            \
      const __grid_constant__ HcItemProgramDev p) {                                      \
    workItems<double, hcfused::item_##body, HC_ITEM_GROUPS(double)>(p);                  \
  }
#endif
HC_FUSED_ITEM_LIST(HC_ITEM_FIXED)
#endif
