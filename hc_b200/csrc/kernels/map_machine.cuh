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

// NumPy's maximum/minimum: NaN if either operand is NaN.
template <typename T> __device__ __forceinline__ T maxOf(T a, T b) {
  return (a > b || a != a) ? a : b;
}
template <typename T> __device__ __forceinline__ T minOf(T a, T b) {
  return (a < b || a != a) ? a : b;
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

// Runs instructions [pcBegin, pcEnd) of the program on W elements.  The
// inputs and the accumulator live in registers; the temporaries, which few
// expressions need, in this thread's column of a shared-memory array, so that
// registers stay free for loads in flight.
//
// INDEXED: `row` and `packet` say where the elements sit (element i is in
// packet `packet + (i / V) * STRIDE`, at position i % V of it) - programs
// written at work-item level use the indices themselves as operands.
// ROWS: `scalars` are the values earlier passes of a row program reduced.
template <typename T, int W, int V, int NIN, bool INDEXED, bool ROWS, int STRIDE>
__device__ __forceinline__ void evaluate(const HcMapProgramDev &p, int pcBegin, int pcEnd,
                                         const T (&x)[NIN][W], T (&acc)[W],
                                         T (&temps)[3][W][THREADS], long long row,
                                         long long packet, const T (&scalars)[4]) {
  const int lane = threadIdx.x;
#pragma unroll
  for (int i = 0; i < W; ++i)
    acc[i] = T(0);
#define HC_MAP_EACH(expr)                                                               \
  _Pragma("unroll") for (int i = 0; i < W; ++i) {                                       \
    const T a = acc[i], b = v[i];                                                       \
    (void)b;                                                                            \
    acc[i] = (expr);                                                                    \
  }                                                                                     \
  break
#define HC_MAP_TAKE(from)                                                               \
  _Pragma("unroll") for (int i = 0; i < W; ++i) v[i] = from;                            \
  break
  for (int pc = pcBegin; pc < pcEnd; ++pc) {
    const uint32_t ins = p.code[pc], op = ins & 0xffu, src = ins >> 8;
    T v[W]; // operand of the binary operations (the unary ones never read it)
    if (op <= HC_MAP_MIN) {
      if (ROWS && src >= HC_MAP_SRC_SCALAR) {
        switch (src - HC_MAP_SRC_SCALAR) {
        case 0: HC_MAP_TAKE(scalars[0]);
        case 1: HC_MAP_TAKE(scalars[1]);
        case 2: HC_MAP_TAKE(scalars[2]);
        default: HC_MAP_TAKE(scalars[3]);
        }
      } else if (INDEXED && src >= HC_MAP_SRC_ROW) {
#pragma unroll
        for (int i = 0; i < W; ++i)
          v[i] = src == HC_MAP_SRC_ROW
                     ? T(row)
                     : T((packet + (long long)(i / V) * STRIDE) * V + i % V);
      } else if (src >= HC_MAP_SRC_CONST) {
        const T c = T(p.consts[src - HC_MAP_SRC_CONST]);
#pragma unroll
        for (int i = 0; i < W; ++i)
          v[i] = c;
      } else {
        // Named registers only: an indexed access would go to local memory.
        switch (src) {
        case 0: HC_MAP_TAKE(x[0][i]);
        case 1: if constexpr (NIN > 1) { HC_MAP_TAKE(x[1][i]); } break;
        case 2: if constexpr (NIN > 2) { HC_MAP_TAKE(x[2][i]); } break;
        case 3: if constexpr (NIN > 3) { HC_MAP_TAKE(x[3][i]); } break;
        case 4: HC_MAP_TAKE(temps[0][i][lane]);
        case 5: HC_MAP_TAKE(temps[1][i][lane]);
        default: HC_MAP_TAKE(temps[2][i][lane]);
        }
      }
    }
    switch (op) {
    case HC_MAP_LOAD: HC_MAP_EACH(b);
    case HC_MAP_ADD: HC_MAP_EACH(a + b);
    case HC_MAP_SUB: HC_MAP_EACH(a - b);
    case HC_MAP_RSUB: HC_MAP_EACH(b - a);
    case HC_MAP_MUL: HC_MAP_EACH(a * b);
    case HC_MAP_DIV: HC_MAP_EACH(a / b);
    case HC_MAP_RDIV: HC_MAP_EACH(b / a);
    case HC_MAP_MAX: HC_MAP_EACH(maxOf(a, b));
    case HC_MAP_MIN: HC_MAP_EACH(minOf(a, b));
    case HC_MAP_NEG: HC_MAP_EACH(-a);
    case HC_MAP_ABS: HC_MAP_EACH(a < T(0) ? -a : (a == T(0) ? T(0) : a));
    case HC_MAP_EXP: HC_MAP_EACH(expOf(a));
    case HC_MAP_SQRT: HC_MAP_EACH(sqrt(a));
    case HC_MAP_LOG: HC_MAP_EACH(logOf(a));
    case HC_MAP_SAVE0:
    case HC_MAP_SAVE1:
    case HC_MAP_SAVE2: { // park the accumulator
      const int t = int(op) - int(HC_MAP_SAVE0);
#pragma unroll
      for (int i = 0; i < W; ++i)
        temps[t][i][lane] = acc[i];
      break;
    }
    default: // the row reductions end a pass and are handled by the caller
      break;
    }
  }
#undef HC_MAP_EACH
#undef HC_MAP_TAKE
}

} // namespace hcmap
