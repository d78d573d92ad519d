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

// Runs the program on all W elements this thread holds at once: one decode
// and one (uniform) branch per instruction, then W independent operations.
// The inputs and the accumulator live in registers; the temporaries, which few
// expressions need, in this thread's column of a shared-memory array, so that
// registers stay free for loads in flight (occupancy is what a streaming
// kernel lives on).
//
// `row` and `packet` say where the elements sit (element i is in packet
// `packet + (i / V) * THREADS`, at position i % V of it): programs written at
// work-item level use the indices themselves as operands.
template <typename T, int W, int V, int NIN, bool INDEXED>
__device__ __forceinline__ void evaluate(const HcMapProgramDev &p, const T (&x)[NIN][W],
                                         T (&acc)[W], T (&temps)[3][W][THREADS], long long row,
                                         long long packet) {
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
  for (int pc = 0; pc < p.nInstr; ++pc) {
    const uint32_t ins = p.code[pc], op = ins & 0xffu, src = ins >> 8;
    T v[W]; // operand of the binary operations (the unary ones never read it)
    if (op <= HC_MAP_MIN) {
      if (INDEXED && src >= HC_MAP_SRC_ROW) {
#pragma unroll
        for (int i = 0; i < W; ++i)
          v[i] = src == HC_MAP_SRC_ROW
                     ? T(row)
                     : T((packet + (long long)(i / V) * THREADS) * V + i % V);
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
    default: { // HC_MAP_SAVE0..2: park the accumulator
      const int t = int(op) - int(HC_MAP_SAVE0);
#pragma unroll
      for (int i = 0; i < W; ++i)
        temps[t][i][lane] = acc[i];
      break;
    }
    }
  }
#undef HC_MAP_EACH
#undef HC_MAP_TAKE
}

template <typename T, int V, int NIN, bool INDEXED>
__device__ __forceinline__ void mapRows(const HcMapProgramDev &p) {
  constexpr int W = V * UNROLL;
  __shared__ T temps[3][W][THREADS];
  const long long perRow = p.cols / V;
  for (long long r = blockIdx.y; r < p.rows; r += gridDim.y) {
    const long long first = ((long long)blockIdx.x * UNROLL) * THREADS + threadIdx.x;
    for (long long base = first; base < perRow;
         base += (long long)gridDim.x * UNROLL * THREADS) {
      // All loads of the UNROLL packets are issued before any arithmetic.
      T x[NIN][W];
#pragma unroll
      for (int k = 0; k < NIN; ++k)
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
          const long long i = base + (long long)u * THREADS;
          Packet<T, V> packet;
#pragma unroll
          for (int e = 0; e < V; ++e)
            packet.v[e] = T(0);
          if (k < p.nInputs && i < perRow)
            packet = loadPacket<T, V>(static_cast<const T *>(p.in[k]) + r * p.inPitch[k] + i * V);
#pragma unroll
          for (int e = 0; e < V; ++e)
            x[k][u * V + e] = packet.v[e];
        }
      T result[W];
      evaluate<T, W, V, NIN, INDEXED>(p, x, result, temps, r, base);
#pragma unroll
      for (int u = 0; u < UNROLL; ++u) {
        const long long i = base + (long long)u * THREADS;
        if (i < perRow) {
          Packet<T, V> packet;
#pragma unroll
          for (int e = 0; e < V; ++e)
            packet.v[e] = result[u * V + e];
          storePacket<T, V>(static_cast<T *>(p.out) + r * p.outPitch + i * V, packet);
        }
      }
    }
  }
}

} // namespace

// One kernel per element type, packet width and number of input arrays (a
// program without inputs runs on the one-input kernel and loads nothing), and
// a twin of each (suffix `i`) for programs that use the element indices, so
// that the streaming kernels do not carry the index bookkeeping.
#define HC_MAP_KERNEL(tname, T, V, NIN)                                                 \
  extern "C" __global__ void __launch_bounds__(THREADS, 4)                              \
      hc_map_elements_##tname##_v##V##_n##NIN(const __grid_constant__ HcMapProgramDev p) { \
    mapRows<T, V, NIN, false>(p);                                                       \
  }                                                                                     \
  extern "C" __global__ void __launch_bounds__(THREADS, 4)                              \
      hc_map_elements_##tname##_v##V##_n##NIN##i(const __grid_constant__ HcMapProgramDev p) { \
    mapRows<T, V, NIN, true>(p);                                                        \
  }
#define HC_MAP_KERNELS(tname, T, V)                                                     \
  HC_MAP_KERNEL(tname, T, V, 1)                                                         \
  HC_MAP_KERNEL(tname, T, V, 2)                                                         \
  HC_MAP_KERNEL(tname, T, V, 3)                                                         \
  HC_MAP_KERNEL(tname, T, V, 4)

HC_MAP_KERNELS(f32, float, 4)
HC_MAP_KERNELS(f32, float, 1)
HC_MAP_KERNELS(f64, double, 2)
HC_MAP_KERNELS(f64, double, 1)
