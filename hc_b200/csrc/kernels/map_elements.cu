// Element-wise expression kernel: out[r, c] = f(in0[r, c], ..., in3[r, c]) for
// rows x cols matrices (row-major, own pitches) of float32, float64, int32 or
// int64, f a composition of the reference's tile operators (+ - * / // % **,
// comparisons, & | ^ << >> ~, neg, abs: python/hckernel/kernel_api.py:157-176),
// max, min, exp, log, sqrt and constants.  Elements that the arithmetic masks -
// a zero divisor, a power that is not finite - are not stored, like the
// reference's masked store (kernel_api.py:338-340).
//
// This is the GPU form of work-groups that load tiles at one origin, combine
// them element by element and store the result at the same origin - the shape
// of the reference's copy kernels (python/hckernel/tests/test_e2e.py:57-136)
// with arithmetic in between (tile arithmetic: python/hckernel/kernel_api.py:
// 136-211).  The reference compiles each such body; here there is no compiler,
// so f arrives as data: a short program for a machine with one accumulator and
// three temporaries (map_params.h, map_machine.cuh), which every thread
// interprets on the elements it holds in registers.  The interpretation costs
// a few uniform branches per operation and element packet; the kernel stays
// bound by HBM, which is what an element-wise pass over large arrays is bound
// by anyway.
//
// A thread handles packets of 16 bytes (4 floats / 2 doubles) when every base
// and pitch allows it, single elements otherwise.
#include "map_machine.cuh"

namespace {

using namespace hcmap;

// EXTENDED: the kernel for programs that divide (/ // %), raise to a power,
// compare, use bitwise operators or work on integers - it tracks which elements
// stay valid and stores only those.  The basic kernel carries none of that.
template <typename T, int V, int NIN, bool INDEXED, bool EXTENDED>
__device__ __forceinline__ void mapRows(const HcMapProgramDev &p) {
  // Packets per thread and decode: four with one or two inputs (three CTAs per
  // SM), two beyond (the inputs of four packets would not fit the registers).
  constexpr int UNROLL = NIN <= 2 ? 4 : 2;
  constexpr int W = V * UNROLL;
  __shared__ T temps[3][W][THREADS];
  const T noScalars[4] = {T(0), T(0), T(0), T(0)};
  const long long perRow = p.cols / V;
  for (long long r = blockIdx.y; r < p.rows; r += gridDim.y) {
    const T *rowIn[NIN];
#pragma unroll
    for (int k = 0; k < NIN; ++k) {
      const int kk = k < p.nInputs ? k : 0; // a program without inputs loads input 0's slot
      rowIn[k] = static_cast<const T *>(p.in[kk]) + r * p.inPitch[kk];
    }
    T *const rowOut = static_cast<T *>(p.out) + r * p.outPitch;
    const long long first = ((long long)blockIdx.x * UNROLL) * THREADS + threadIdx.x;
    for (long long base = first; base < perRow;
         base += (long long)gridDim.x * UNROLL * THREADS) {
      // Every packet of this step lies inside the row (the same for the whole CTA)?
      const bool whole = base - threadIdx.x + (long long)UNROLL * THREADS <= perRow;
      // All loads of the UNROLL packets are issued before any arithmetic.
      T x[NIN][W];
#pragma unroll
      for (int k = 0; k < NIN; ++k)
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
          const long long i = base + (long long)u * THREADS;
          Packet<T, V> packet;
          if (k < p.nInputs && (whole || i < perRow)) {
            packet = loadPacket<T, V>(rowIn[k] + i * V);
          } else {
#pragma unroll
            for (int e = 0; e < V; ++e)
              packet.v[e] = T(0);
          }
#pragma unroll
          for (int e = 0; e < V; ++e)
            x[k][u * V + e] = packet.v[e];
        }
      T result[W];
      uint32_t ok = ~0u;
      uint64_t parkedOk = ~0ull;
      evaluate<T, W, V, NIN, INDEXED, false, THREADS, THREADS, EXTENDED>(
          p, 0, p.nInstr, x, result, temps, r, base, noScalars, ok, parkedOk);
      if constexpr (EXTENDED) {
        storeValid<T, V, UNROLL, THREADS>(rowOut, result, ok, base, perRow, whole);
      } else {
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
          const long long i = base + (long long)u * THREADS;
          if (whole || i < perRow) {
            Packet<T, V> packet;
#pragma unroll
            for (int e = 0; e < V; ++e)
              packet.v[e] = result[u * V + e];
            storePacket<T, V>(rowOut + i * V, packet);
          }
        }
      }
    }
  }
}

} // namespace

// One kernel per element type, packet width and number of input arrays (a
// program without inputs runs on the one-input kernel and loads nothing), a
// twin of each (suffix `i`) for programs that use the element indices, so that
// the streaming kernels do not carry the index bookkeeping, and of each of
// those the extended form (suffix `x`).  Integer arrays have extended kernels
// only.
// (The extended kernels get the registers of two CTAs per SM: the out-of-line
// operations would otherwise spill around their calls.)
#define HC_MAP_KERNEL_FORM(tname, T, V, NIN, suffix, INDEXED, EXTENDED)                 \
  extern "C" __global__ void __launch_bounds__(THREADS, EXTENDED ? 2 : NIN <= 2 ? 3 : 4) \
      hc_map_elements_##tname##_v##V##_n##NIN##suffix(                                  \
          const __grid_constant__ HcMapProgramDev p) {                                  \
    mapRows<T, V, NIN, INDEXED, EXTENDED>(p);                                           \
  }
#define HC_MAP_BASIC(tname, T, V, NIN)                                                  \
  HC_MAP_KERNEL_FORM(tname, T, V, NIN, , false, false)                                  \
  HC_MAP_KERNEL_FORM(tname, T, V, NIN, i, true, false)
#define HC_MAP_EXTENDED(tname, T, V, NIN)                                               \
  HC_MAP_KERNEL_FORM(tname, T, V, NIN, x, false, true)                                  \
  HC_MAP_KERNEL_FORM(tname, T, V, NIN, ix, true, true)
#define HC_MAP_EACH_NIN(FORM, tname, T, V)                                              \
  FORM(tname, T, V, 1) FORM(tname, T, V, 2) FORM(tname, T, V, 3) FORM(tname, T, V, 4)

HC_MAP_EACH_NIN(HC_MAP_BASIC, f32, float, 4)
HC_MAP_EACH_NIN(HC_MAP_BASIC, f32, float, 1)
HC_MAP_EACH_NIN(HC_MAP_BASIC, f64, double, 2)
HC_MAP_EACH_NIN(HC_MAP_BASIC, f64, double, 1)
HC_MAP_EACH_NIN(HC_MAP_EXTENDED, f32, float, 4)
HC_MAP_EACH_NIN(HC_MAP_EXTENDED, f32, float, 1)
HC_MAP_EACH_NIN(HC_MAP_EXTENDED, f64, double, 2)
HC_MAP_EACH_NIN(HC_MAP_EXTENDED, f64, double, 1)
HC_MAP_EACH_NIN(HC_MAP_EXTENDED, i32, int32_t, 4)
HC_MAP_EACH_NIN(HC_MAP_EXTENDED, i32, int32_t, 1)
HC_MAP_EACH_NIN(HC_MAP_EXTENDED, i64, int64_t, 2)
HC_MAP_EACH_NIN(HC_MAP_EXTENDED, i64, int64_t, 1)
