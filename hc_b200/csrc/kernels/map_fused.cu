// Element-wise bodies compiled ahead of time: the bodies listed in
// fused_programs.h (scale-and-shift, rectifiers, differences, a Horner
// polynomial ... - tile arithmetic between a load and a store at one origin,
// python/hckernel/kernel_api.py:136-211) as straight-line kernels.
//
// Same launch shape and element order as the interpreting kernel of
// map_elements.cu; every instruction of the program is a template constant
// (fused_machine.cuh), so a thread loads its packets, runs the arithmetic and
// stores, with nothing in between.  Results are bit for bit the interpreter's.
#include "fused_machine.cuh"
#include "fused_programs.h"

namespace {

using namespace hcmap;
using namespace hcfused;

template <typename T, int V, typename P>
__device__ __forceinline__ void mapFused(const HcMapProgramDev &p) {
  constexpr int NIN = P::nin;
  // Packets per thread and step, as in map_elements.cu.
  constexpr int UNROLL = NIN <= 2 ? 4 : 2;
  constexpr int W = V * UNROLL;
  const long long perRow = p.cols / V;
  for (long long r = blockIdx.y; r < p.rows; r += gridDim.y) {
    const T *rowIn[NIN > 0 ? NIN : 1];
#pragma unroll
    for (int k = 0; k < NIN; ++k)
      rowIn[k] = static_cast<const T *>(p.in[k]) + r * p.inPitch[k];
    T *const rowOut = static_cast<T *>(p.out) + r * p.outPitch;
    const long long first = ((long long)blockIdx.x * UNROLL) * THREADS + threadIdx.x;
    for (long long base = first; base < perRow;
         base += (long long)gridDim.x * UNROLL * THREADS) {
      // Every packet of this step lies inside the row (the same for the whole CTA)?
      const bool whole = base - threadIdx.x + (long long)UNROLL * THREADS <= perRow;
      Frame<T, W, NIN> f;
#pragma unroll
      for (int k = 0; k < NIN; ++k)
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
          const long long i = base + (long long)u * THREADS;
          Packet<T, V> packet;
          if (whole || i < perRow) {
            packet = loadPacket<T, V>(rowIn[k] + i * V);
          } else {
#pragma unroll
            for (int e = 0; e < V; ++e)
              packet.v[e] = T(0);
          }
#pragma unroll
          for (int e = 0; e < V; ++e)
            f.x[k][u * V + e] = packet.v[e];
        }
      T result[W];
      run<T, W, V, NIN, P, 0, P::n, THREADS, true>(p, f, result, r, base);
      // Elements whose divisor was zero are left unwritten (a program without
      // divisions keeps all bits set and the test folds away).
      storeValid<T, V, UNROLL, THREADS>(rowOut, result, f.ok, base, perRow, whole);
    }
  }
}

} // namespace

#define HC_MAP_FUSED_F32(body)                                                                      \
  extern "C" __global__ void __launch_bounds__(THREADS, 3) hc_map_fused_##body##_f32_v4(            \
      const __grid_constant__ HcMapProgramDev p) {                                               \
    mapFused<float, 4, hcfused::map_##body>(p);                                                  \
  }                                                                                              \
  extern "C" __global__ void __launch_bounds__(THREADS) hc_map_fused_##body##_f32_v1(            \
      const __grid_constant__ HcMapProgramDev p) {                                               \
    mapFused<float, 1, hcfused::map_##body>(p);                                                  \
  }
#define HC_MAP_FUSED_F64(body)                                                                   \
  extern "C" __global__ void __launch_bounds__(THREADS) hc_map_fused_##body##_f64_v2(            \
      const __grid_constant__ HcMapProgramDev p) {                                               \
    mapFused<double, 2, hcfused::map_##body>(p);                                                 \
  }                                                                                              \
  extern "C" __global__ void __launch_bounds__(THREADS) hc_map_fused_##body##_f64_v1(            \
      const __grid_constant__ HcMapProgramDev p) {                                               \
    mapFused<double, 1, hcfused::map_##body>(p);                                                 \
  }

#define HC_MAP_FUSED_I32(body)                                                                   \
  extern "C" __global__ void __launch_bounds__(THREADS, 3) hc_map_fused_##body##_i32_v4(         \
      const __grid_constant__ HcMapProgramDev p) {                                               \
    mapFused<int32_t, 4, hcfused::map_##body>(p);                                                \
  }                                                                                              \
  extern "C" __global__ void __launch_bounds__(THREADS) hc_map_fused_##body##_i32_v1(            \
      const __grid_constant__ HcMapProgramDev p) {                                               \
    mapFused<int32_t, 1, hcfused::map_##body>(p);                                                \
  }
#define HC_MAP_FUSED_I64(body)                                                                   \
  extern "C" __global__ void __launch_bounds__(THREADS) hc_map_fused_##body##_i64_v2(            \
      const __grid_constant__ HcMapProgramDev p) {                                               \
    mapFused<int64_t, 2, hcfused::map_##body>(p);                                                \
  }                                                                                              \
  extern "C" __global__ void __launch_bounds__(THREADS) hc_map_fused_##body##_i64_v1(            \
      const __grid_constant__ HcMapProgramDev p) {                                               \
    mapFused<int64_t, 1, hcfused::map_##body>(p);                                                \
  }

// The bodies compiled ahead of time are float bodies, in both float types.  A
// run-time specialisation (launch/specialise.cpp) compiles this file for one
// program and one element type, named by HC_FUSED_ONLY (0 float32, 1 float64,
// 2 int32, 3 int64).
#ifndef HC_FUSED_ONLY
HC_FUSED_MAP_LIST(HC_MAP_FUSED_F32)
HC_FUSED_MAP_LIST(HC_MAP_FUSED_F64)
#elif HC_FUSED_ONLY == 0
HC_FUSED_MAP_LIST(HC_MAP_FUSED_F32)
#elif HC_FUSED_ONLY == 1
HC_FUSED_MAP_LIST(HC_MAP_FUSED_F64)
#elif HC_FUSED_ONLY == 2
HC_FUSED_MAP_LIST(HC_MAP_FUSED_I32)
#else
HC_FUSED_MAP_LIST(HC_MAP_FUSED_I64)
#endif
