// The expression machine shared by the element-wise kernel (map_elements.cu)
// and the row-program kernel (row_program.cu): one accumulator, three
// temporaries, up to four input arrays, eight constants (map_params.h).  A
// thread interprets the program on the W elements it holds in registers: one
// decode and one (uniform) branch per instruction, then W independent
// operations.  Operations are never contracted into FMAs, so + - * / and sqrt
// are the correctly rounded results NumPy gives.
#pragma once

#include "map_params.h"

#include <math.h>
#include <stdint.h>

namespace hcmap {

constexpr int THREADS = 256;

template <typename T> __device__ __forceinline__ T expOf(T v);
template <> __device__ __forceinline__ float expOf<float>(float v) { return expf(v); }
template <> __device__ __forceinline__ double expOf<double>(double v) { return exp(v); }
template <typename T> __device__ __forceinline__ T logOf(T v);
template <> __device__ __forceinline__ float logOf<float>(float v) { return logf(v); }
template <> __device__ __forceinline__ double logOf<double>(double v) { return log(v); }

// NumPy's maximum/minimum: NaN if either operand is NaN, the first operand on
// a tie (which matters for +0 against -0 only).
template <typename T> __device__ __forceinline__ T maxOf(T a, T b) {
  return (a >= b || a != a) ? a : b;
}
template <typename T> __device__ __forceinline__ T minOf(T a, T b) {
  return (a <= b || a != a) ? a : b;
}

template <typename T, int V> struct Packet { T v[V]; };

template <typename T, int V>
__device__ __forceinline__ Packet<T, V> loadPacket(const T *p) {
  Packet<T, V> out;
  if constexpr (V * sizeof(T) == 16) {
    const float4 raw = __ldcs(reinterpret_cast<const float4 *>(p));
    *reinterpret_cast<float4 *>(out.v) = raw;
  } else {
    out.v[0] = __ldcs(p);
  }
  return out;
}

template <typename T, int V>
__device__ __forceinline__ void storePacket(T *p, const Packet<T, V> &value) {
  if constexpr (V * sizeof(T) == 16)
    __stcs(reinterpret_cast<float4 *>(p), *reinterpret_cast<const float4 *>(value.v));
  else
    __stcs(p, value.v[0]);
}

// A load that leaves the line in the caches (a later pass of a row program
// reads the row again), where loadPacket streams.
template <typename T, int V>
__device__ __forceinline__ Packet<T, V> loadPacketKept(const T *p) {
  Packet<T, V> out;
  if constexpr (V * sizeof(T) == 16)
    *reinterpret_cast<float4 *>(out.v) = *reinterpret_cast<const float4 *>(p);
  else
    out.v[0] = *p;
  return out;
}

template <typename T> __device__ __forceinline__ T lowest();
template <> __device__ __forceinline__ float lowest<float>() { return -INFINITY; }
template <> __device__ __forceinline__ double lowest<double>() { return -INFINITY; }

// The larger of two values, NaN if either is NaN (what NumPy's max along an
// axis gives); one instruction for float.
__device__ __forceinline__ float maxNan(float a, float b) {
  float out;
  asm("max.NaN.f32 %0, %1, %2;" : "=f"(out) : "f"(a), "f"(b));
  return out;
}
__device__ __forceinline__ double maxNan(double a, double b) { return maxOf(a, b); }

// The binary operations of the machine on W accumulators; `operand(i)` names
// the second operand of element i (a register, a uniform value or an
// expression of the element's position), so that no operand is copied before
// it is used.
template <typename T, int W, typename F>
__device__ __forceinline__ void binary(uint32_t op, T (&acc)[W], F operand) {
#define HC_MAP_EACH(expr)                                                               \
  _Pragma("unroll") for (int i = 0; i < W; ++i) {                                       \
    const T a = acc[i], b = operand(i);                                                 \
    (void)a;                                                                            \
    acc[i] = (expr);                                                                    \
  }                                                                                     \
  break
  switch (op) {
  case HC_MAP_LOAD: HC_MAP_EACH(b);
  case HC_MAP_ADD: HC_MAP_EACH(a + b);
  case HC_MAP_SUB: HC_MAP_EACH(a - b);
  case HC_MAP_RSUB: HC_MAP_EACH(b - a);
  case HC_MAP_MUL: HC_MAP_EACH(a * b);
  case HC_MAP_DIV: HC_MAP_EACH(a / b);
  case HC_MAP_RDIV: HC_MAP_EACH(b / a);
  case HC_MAP_MAX: HC_MAP_EACH(maxOf(a, b));
  default: HC_MAP_EACH(minOf(a, b));
  }
#undef HC_MAP_EACH
}

// Runs instructions [pcBegin, pcEnd) of the program on W elements.  The
// inputs and the accumulator live in registers; the temporaries, which few
// expressions need, in this thread's column of a shared-memory array, so that
// registers stay free for loads in flight.  The first instruction of a range
// is always a load of the accumulator (the host refuses other programs), so
// `acc` needs no initial value.
//
// INDEXED: `row` and `packet` say where the elements sit (element i is in
// packet `packet + (i / V) * STRIDE`, at position i % V of it) - programs
// written at work-item level use the indices themselves as operands.
// ROWS: `scalars` are the values earlier passes of a row program reduced.
template <typename T, int W, int V, int NIN, bool INDEXED, bool ROWS, int STRIDE,
          int COLUMNS = THREADS>
__device__ __forceinline__ void evaluate(const HcMapProgramDev &p, int pcBegin, int pcEnd,
                                         const T (&x)[NIN][W], T (&acc)[W],
                                         T (&temps)[3][W][COLUMNS], long long row,
                                         long long packet, const T (&scalars)[4]) {
  const int lane = threadIdx.x;
#define HC_MAP_EACH(expr)                                                               \
  _Pragma("unroll") for (int i = 0; i < W; ++i) {                                       \
    const T a = acc[i];                                                                 \
    acc[i] = (expr);                                                                    \
  }                                                                                     \
  break
  for (int pc = pcBegin; pc < pcEnd; ++pc) {
    const uint32_t ins = p.code[pc], op = ins & 0xffu, src = ins >> 8;
    if (op <= HC_MAP_MIN) {
      if (src >= HC_MAP_SRC_CONST) {
        // One value for all elements: a constant, a row scalar, the row index.
        if (INDEXED && src == HC_MAP_SRC_COL) {
          binary<T, W>(op, acc, [&](int i) {
            return T((packet + (long long)(i / V) * STRIDE) * V + i % V);
          });
          continue;
        }
        T one;
        if (ROWS && src >= HC_MAP_SRC_SCALAR) {
          const uint32_t k = src - HC_MAP_SRC_SCALAR;
          one = k == 0 ? scalars[0] : k == 1 ? scalars[1] : k == 2 ? scalars[2] : scalars[3];
        } else if (INDEXED && src == HC_MAP_SRC_ROW) {
          one = T(row);
        } else {
          one = T(p.consts[src - HC_MAP_SRC_CONST]);
        }
        binary<T, W>(op, acc, [&](int) { return one; });
      } else if (src >= HC_MAP_SRC_TEMP) {
        T v[W]; // shared memory may be indexed by the operand number, registers not
#pragma unroll
        for (int i = 0; i < W; ++i)
          v[i] = temps[src - HC_MAP_SRC_TEMP][i][lane];
        binary<T, W>(op, acc, [&](int i) { return v[i]; });
      } else {
        // Named registers only: an indexed access would go to local memory.
        switch (src) {
        case 0: binary<T, W>(op, acc, [&](int i) { return x[0][i]; }); break;
        case 1: if constexpr (NIN > 1) binary<T, W>(op, acc, [&](int i) { return x[1][i]; }); break;
        case 2: if constexpr (NIN > 2) binary<T, W>(op, acc, [&](int i) { return x[2][i]; }); break;
        default: if constexpr (NIN > 3) binary<T, W>(op, acc, [&](int i) { return x[3][i]; }); break;
        }
      }
      continue;
    }
    switch (op) {
    case HC_MAP_NEG: HC_MAP_EACH(-a);
    case HC_MAP_ABS: HC_MAP_EACH(a < T(0) ? -a : (a == T(0) ? T(0) : a));
    case HC_MAP_EXP: HC_MAP_EACH(expOf(a));
    case HC_MAP_SQRT: HC_MAP_EACH(sqrt(a));
    case HC_MAP_LOG: HC_MAP_EACH(logOf(a));
    case HC_MAP_SAVE0:
    case HC_MAP_SAVE1:
    case HC_MAP_SAVE2: // park the accumulator
#pragma unroll
      for (int i = 0; i < W; ++i)
        temps[op - HC_MAP_SAVE0][i][lane] = acc[i];
      break;
    default: // the row reductions end a pass and are handled by the caller
      break;
    }
  }
#undef HC_MAP_EACH
}

} // namespace hcmap
