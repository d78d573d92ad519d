// Element-wise expression kernel: out[r, c] = f(in0[r, c], ..., in3[r, c]) for
// rows x cols matrices (row-major, own pitches), f a composition of + - * /,
// max, min, neg, abs, exp, log, sqrt and constants.
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

template <typename T, int V, int NIN, bool INDEXED>
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
      evaluate<T, W, V, NIN, INDEXED, false, THREADS>(p, 0, p.nInstr, x, result, temps, r, base,
                                                      noScalars);
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

} // namespace

// One kernel per element type, packet width and number of input arrays (a
// program without inputs runs on the one-input kernel and loads nothing), and
// a twin of each (suffix `i`) for programs that use the element indices, so
// that the streaming kernels do not carry the index bookkeeping.
#define HC_MAP_KERNEL(tname, T, V, NIN)                                                 \
  extern "C" __global__ void __launch_bounds__(THREADS, NIN <= 2 ? 3 : 4)                              \
      hc_map_elements_##tname##_v##V##_n##NIN(const __grid_constant__ HcMapProgramDev p) { \
    mapRows<T, V, NIN, false>(p);                                                       \
  }                                                                                     \
  extern "C" __global__ void __launch_bounds__(THREADS, NIN <= 2 ? 3 : 4)                              \
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
