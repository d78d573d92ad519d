// Element-wise expression kernel: out[r, c] = f(in0[r, c], ..., in3[r, c]) for
// rows x cols matrices (row-major, own pitches), f a composition of + - * /,
// max, min, neg, abs, exp, sqrt and constants.
//
// This is the GPU form of work-groups that load tiles at one origin, combine
// them element by element and store the result at the same origin - the shape
// of the reference's copy kernels (python/hckernel/tests/test_e2e.py:57-136)
// with arithmetic in between (tile arithmetic: python/hckernel/kernel_api.py:
// 136-211).  The reference compiles each such body; here there is no compiler,
// so f arrives as data: a short program for a machine with one accumulator and
// three temporaries (map_params.h), which every thread interprets on the
// elements it holds in registers.  The interpretation costs a few uniform
// branches per operation and element packet; the kernel stays bound by HBM,
// which is what an element-wise pass over large arrays is bound by anyway.
//
// A thread handles packets of 16 bytes (4 floats / 2 doubles) when every base
// and pitch allows it, single elements otherwise.  Operations are not fused
// across instructions (no contraction into FMAs), so + - * / and sqrt give the
// correctly rounded results NumPy gives; exp differs in the last bits.
#include "map_params.h"

#include <math.h>
#include <stdint.h>

namespace {

constexpr int THREADS = 256, UNROLL = 2;

template <typename T> __device__ __forceinline__ T expOf(T v);
template <> __device__ __forceinline__ float expOf<float>(float v) { return expf(v); }
template <> __device__ __forceinline__ double expOf<double>(double v) { return exp(v); }

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

template <typename T, int V>
__device__ __forceinline__ Packet<T, V> evaluate(const HcMapProgramDev &p,
                                                 const Packet<T, V> (&x)[HC_MAP_MAX_INPUTS]) {
  Packet<T, V> acc, t0, t1, t2;
#pragma unroll
  for (int i = 0; i < V; ++i)
    acc.v[i] = t0.v[i] = t1.v[i] = t2.v[i] = T(0);
  for (int pc = 0; pc < p.nInstr; ++pc) {
    const uint32_t ins = p.code[pc], op = ins & 0xffu, src = ins >> 8;
    Packet<T, V> v = acc; // operand of the binary operations
    if (op <= HC_MAP_MIN) {
      if (src >= HC_MAP_SRC_CONST) {
        const T c = T(p.consts[src - HC_MAP_SRC_CONST]);
#pragma unroll
        for (int i = 0; i < V; ++i)
          v.v[i] = c;
      } else {
        switch (src) { // named registers only: no indexed (local-memory) access
        case 0: v = x[0]; break;
        case 1: v = x[1]; break;
        case 2: v = x[2]; break;
        case 3: v = x[3]; break;
        case 4: v = t0; break;
        case 5: v = t1; break;
        default: v = t2; break;
        }
      }
    }
#pragma unroll
    for (int i = 0; i < V; ++i) {
      const T a = acc.v[i], b = v.v[i];
      T r = a;
      switch (op) {
      case HC_MAP_LOAD: r = b; break;
      case HC_MAP_ADD: r = a + b; break;
      case HC_MAP_SUB: r = a - b; break;
      case HC_MAP_RSUB: r = b - a; break;
      case HC_MAP_MUL: r = a * b; break;
      case HC_MAP_DIV: r = a / b; break;
      case HC_MAP_RDIV: r = b / a; break;
      case HC_MAP_MAX: r = maxOf(a, b); break;
      case HC_MAP_MIN: r = minOf(a, b); break;
      case HC_MAP_NEG: r = -a; break;
      case HC_MAP_ABS: r = a < T(0) ? -a : (a == T(0) ? T(0) : a); break;
      case HC_MAP_EXP: r = expOf(a); break;
      case HC_MAP_SQRT: r = sqrt(a); break;
      default: break; // the SAVE operations leave the accumulator alone
      }
      acc.v[i] = r;
    }
    if (op == HC_MAP_SAVE0)
      t0 = acc;
    else if (op == HC_MAP_SAVE1)
      t1 = acc;
    else if (op == HC_MAP_SAVE2)
      t2 = acc;
  }
  return acc;
}

template <typename T, int V>
__device__ __forceinline__ void mapRows(const HcMapProgramDev &p) {
  const long long perRow = p.cols / V;
  for (long long r = blockIdx.y; r < p.rows; r += gridDim.y) {
    const long long first = ((long long)blockIdx.x * UNROLL) * THREADS + threadIdx.x;
    for (long long base = first; base < perRow;
         base += (long long)gridDim.x * UNROLL * THREADS) {
      // All loads of the UNROLL packets are issued before any arithmetic.
      Packet<T, V> x[UNROLL][HC_MAP_MAX_INPUTS];
#pragma unroll
      for (int u = 0; u < UNROLL; ++u) {
        const long long i = base + (long long)u * THREADS;
#pragma unroll
        for (int k = 0; k < HC_MAP_MAX_INPUTS; ++k)
          if (k < p.nInputs && i < perRow)
            x[u][k] = loadPacket<T, V>(static_cast<const T *>(p.in[k]) + r * p.inPitch[k] + i * V);
      }
#pragma unroll
      for (int u = 0; u < UNROLL; ++u) {
        const long long i = base + (long long)u * THREADS;
        if (i < perRow)
          storePacket<T, V>(static_cast<T *>(p.out) + r * p.outPitch + i * V,
                            evaluate<T, V>(p, x[u]));
      }
    }
  }
}

} // namespace

#define HC_MAP_KERNEL(name, T, V)                                                       \
  extern "C" __global__ void __launch_bounds__(THREADS)                                 \
      name(const __grid_constant__ HcMapProgramDev p) {                                 \
    mapRows<T, V>(p);                                                                   \
  }

HC_MAP_KERNEL(hc_map_elements_f32_v4, float, 4)
HC_MAP_KERNEL(hc_map_elements_f32_v1, float, 1)
HC_MAP_KERNEL(hc_map_elements_f64_v2, double, 2)
HC_MAP_KERNEL(hc_map_elements_f64_v1, double, 1)
