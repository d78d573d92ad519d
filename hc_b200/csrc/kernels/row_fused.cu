// Row programs compiled ahead of time: the row bodies listed in
// fused_programs.h (centring, normalising, log-softmax and their relatives -
// the family of the reference's row softmax,
// python/hckernel/tests/test_examples.py:312-321) as straight-line kernels.
//
// Same launch shapes, same passes and the same reduction order as the
// interpreting kernels of row_program.cu, so the results are bit for bit the
// interpreter's; what changes is that every instruction of the program is a
// template constant (fused_machine.cuh).  The interpreter issues about 45
// instructions per element for a log-softmax whose arithmetic needs about 17;
// here the compiler sees the arithmetic alone.
//
//   hc_row_fused_<body>_<type>_held_t<64|128>   one CTA per row, eight 16-byte
//       packets per thread, the row read once and kept in registers over all
//       passes (float rows of 257..1024 packets that fill the CTA);
//   hc_row_fused_<body>_<type>_v<V>              one warp per row, eight rows per
//       CTA, every pass walks the row (any length, pitch and alignment).
#include "fused_machine.cuh"
#include "fused_programs.h"

namespace {

using namespace hcmap;
using namespace hcfused;

constexpr int UNROLL = 4; // packets per lane and step of the walking kernel

template <typename T, bool TAKE_MAX> __device__ __forceinline__ T combine(T a, T b) {
  if constexpr (TAKE_MAX)
    return maxNan(a, b);
  else
    return Arith<T>::add(a, b);
}

template <typename T, bool TAKE_MAX> __device__ __forceinline__ T warpReduce(T v) {
#pragma unroll
  for (int offset = 16; offset > 0; offset >>= 1)
    v = combine<T, TAKE_MAX>(v, __shfl_xor_sync(0xffffffffu, v, offset));
  return v;
}

// ---- a warp walks the row ----------------------------------------------------------
template <typename T, int V, typename P, int PC>
__device__ __forceinline__ void walkPasses(const HcMapProgramDev &p, const T *(&rowIn)[P::nin],
                                           T *rowOut, int perRow, long long r, T (&scalars)[4]) {
  constexpr int NIN = P::nin, W = V * UNROLL;
  if constexpr (PC < P::n) {
    runUniform<T, P, PC>(p, scalars, T(0));
    constexpr int begin = afterUniform<P>(PC), end = passEnd<P>(begin);
    constexpr bool last = end >= P::n;
    constexpr uint32_t terminator = P::code[last ? 0 : end]; // the reduction that ends the pass
    constexpr bool takeMax = !last && (terminator & 0xffu) == HC_MAP_RMAX;
    constexpr uint32_t target = terminator >> 8;
    const int lane = threadIdx.x & 31;
    T running = takeMax ? lowest<T>() : T(0);
    for (int base = lane; base < perRow; base += 32 * UNROLL) {
      // Every packet of this step lies inside the row (the same for all lanes)?
      const bool whole = base - lane + 32 * UNROLL <= perRow;
      Frame<T, W, NIN> f;
#pragma unroll
      for (int k = 0; k < 4; ++k)
        f.s[k] = scalars[k];
#pragma unroll
      for (int k = 0; k < NIN; ++k)
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
          const int i = base + u * 32;
          Packet<T, V> packet;
          if (whole || i < perRow) {
            const T *src = rowIn[k] + (long long)i * V;
            packet = last ? loadPacket<T, V>(src) : loadPacketKept<T, V>(src);
          } else {
#pragma unroll
            for (int e = 0; e < V; ++e)
              packet.v[e] = T(0);
          }
#pragma unroll
          for (int e = 0; e < V; ++e)
            f.x[k][u * V + e] = packet.v[e];
        }
      T value[W];
      run<T, W, V, NIN, P, begin, end, 32>(p, f, value, r, base);
      if constexpr (last) {
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
          const int i = base + u * 32;
          if (whole || i < perRow) {
            Packet<T, V> packet;
#pragma unroll
            for (int e = 0; e < V; ++e)
              packet.v[e] = value[u * V + e];
            storePacket<T, V>(rowOut + (long long)i * V, packet);
          }
        }
      } else {
#pragma unroll
        for (int u = 0; u < UNROLL; ++u)
          if (whole || base + u * 32 < perRow) {
#pragma unroll
            for (int e = 0; e < V; ++e)
              running = combine<T, takeMax>(running, value[u * V + e]);
          }
      }
    }
    if constexpr (!last) {
      scalars[target] = warpReduce<T, takeMax>(running);
      walkPasses<T, V, P, end + 1>(p, rowIn, rowOut, perRow, r, scalars);
    }
  }
}

template <typename T, int V, typename P>
__device__ __forceinline__ void rowFusedWalk(const HcMapProgramDev &p) {
  const long long r = (long long)blockIdx.x * (THREADS / 32) + (threadIdx.x >> 5);
  if (r >= p.rows)
    return; // whole warps leave; nothing below synchronises the CTA
  const T *rowIn[P::nin];
#pragma unroll
  for (int k = 0; k < P::nin; ++k)
    rowIn[k] = static_cast<const T *>(p.in[k]) + r * p.inPitch[k];
  T scalars[4] = {T(0), T(0), T(0), T(0)};
  walkPasses<T, V, P, 0>(p, rowIn, static_cast<T *>(p.out) + r * p.outPitch, int(p.cols / V), r,
                         scalars);
}

// ---- a CTA holds the row ---------------------------------------------------------------
template <typename T, int V, int HELD, int NT, typename P, int PC, int REDUCTION>
__device__ __forceinline__ void heldPasses(const HcMapProgramDev &p, Frame<T, V * HELD, P::nin> &f,
                                           T (*partial)[NT / 32], int perRow, long long r) {
  constexpr int NIN = P::nin, W = V * HELD;
  if constexpr (PC < P::n) {
    runUniform<T, P, PC>(p, f.s, T(0));
    constexpr int begin = afterUniform<P>(PC), end = passEnd<P>(begin);
    constexpr bool last = end >= P::n;
    constexpr uint32_t terminator = P::code[last ? 0 : end]; // the reduction that ends the pass
    constexpr bool takeMax = !last && (terminator & 0xffu) == HC_MAP_RMAX;
    constexpr uint32_t target = terminator >> 8;
    T value[W];
    run<T, W, V, NIN, P, begin, end, NT>(p, f, value, r, threadIdx.x);
    if constexpr (last) {
      T *const rowOut = static_cast<T *>(p.out) + r * p.outPitch;
#pragma unroll
      for (int u = 0; u < HELD; ++u) {
        const int i = threadIdx.x + u * NT;
        if (i < perRow) {
          Packet<T, V> packet;
#pragma unroll
          for (int e = 0; e < V; ++e)
            packet.v[e] = value[u * V + e];
          storePacket<T, V>(rowOut + (long long)i * V, packet);
        }
      }
    } else {
      T running = takeMax ? lowest<T>() : T(0);
#pragma unroll
      for (int u = 0; u < HELD; ++u)
        if (threadIdx.x + u * NT < perRow) {
#pragma unroll
          for (int e = 0; e < V; ++e)
            running = combine<T, takeMax>(running, value[u * V + e]);
        }
      running = warpReduce<T, takeMax>(running);
      // Slot n is written again only after three more barriers, long after its
      // last reader has passed the next one.
      T *const slot = partial[REDUCTION & 3];
      if ((threadIdx.x & 31) == 0)
        slot[threadIdx.x >> 5] = running;
      __syncthreads();
      T whole = slot[0];
#pragma unroll
      for (int w = 1; w < NT / 32; ++w)
        whole = combine<T, takeMax>(whole, slot[w]);
      f.s[target] = whole;
      heldPasses<T, V, HELD, NT, P, end + 1, REDUCTION + 1>(p, f, partial, perRow, r);
    }
  }
}

template <typename T, int V, int HELD, int NT, typename P>
__device__ __forceinline__ void rowFusedHeld(const HcMapProgramDev &p) {
  constexpr int NIN = P::nin, W = V * HELD;
  __shared__ T partial[4][NT / 32];
  const long long r = blockIdx.x;
  const int perRow = int(p.cols / V);
  Frame<T, W, NIN> f;
#pragma unroll
  for (int k = 0; k < 4; ++k)
    f.s[k] = T(0);
#pragma unroll
  for (int k = 0; k < NIN; ++k)
#pragma unroll
    for (int u = 0; u < HELD; ++u) {
      const int i = threadIdx.x + u * NT;
      Packet<T, V> packet;
      if (i < perRow) {
        packet = loadPacket<T, V>(static_cast<const T *>(p.in[k]) + r * p.inPitch[k] +
                                  (long long)i * V);
      } else {
#pragma unroll
        for (int e = 0; e < V; ++e)
          packet.v[e] = T(0);
      }
#pragma unroll
      for (int e = 0; e < V; ++e)
        f.x[k][u * V + e] = packet.v[e];
    }
  heldPasses<T, V, HELD, NT, P, 0, 0>(p, f, partial, perRow, r);
}

} // namespace

// Per body: float rows held by a CTA of 64 or 128 threads, and walked rows for
// float (16-byte packets or single elements) and double.
#define HC_ROW_FUSED_F32(body)                                                                      \
  extern "C" __global__ void __launch_bounds__(64) hc_row_fused_##body##_f32_held_t64(           \
      const __grid_constant__ HcMapProgramDev p) {                                               \
    rowFusedHeld<float, 4, 8, 64, hcfused::row_##body>(p);                                       \
  }                                                                                              \
  extern "C" __global__ void __launch_bounds__(128) hc_row_fused_##body##_f32_held_t128(         \
      const __grid_constant__ HcMapProgramDev p) {                                               \
    rowFusedHeld<float, 4, 8, 128, hcfused::row_##body>(p);                                      \
  }                                                                                              \
  extern "C" __global__ void __launch_bounds__(THREADS) hc_row_fused_##body##_f32_v4(            \
      const __grid_constant__ HcMapProgramDev p) {                                               \
    rowFusedWalk<float, 4, hcfused::row_##body>(p);                                              \
  }                                                                                              \
  extern "C" __global__ void __launch_bounds__(THREADS) hc_row_fused_##body##_f32_v1(            \
      const __grid_constant__ HcMapProgramDev p) {                                               \
    rowFusedWalk<float, 1, hcfused::row_##body>(p);                                              \
  }
#define HC_ROW_FUSED_F64(body)                                                                   \
  extern "C" __global__ void __launch_bounds__(THREADS) hc_row_fused_##body##_f64_v2(            \
      const __grid_constant__ HcMapProgramDev p) {                                               \
    rowFusedWalk<double, 2, hcfused::row_##body>(p);                                             \
  }                                                                                              \
  extern "C" __global__ void __launch_bounds__(THREADS) hc_row_fused_##body##_f64_v1(            \
      const __grid_constant__ HcMapProgramDev p) {                                               \
    rowFusedWalk<double, 1, hcfused::row_##body>(p);                                             \
  }

// A run-time specialisation (launch/specialise.cpp) compiles this file for one
// program and one element type, named by HC_FUSED_ONLY (0 float32, 1 float64).
#ifndef HC_FUSED_ONLY
HC_FUSED_ROW_LIST(HC_ROW_FUSED_F32)
HC_FUSED_ROW_LIST(HC_ROW_FUSED_F64)
#elif HC_FUSED_ONLY == 0
HC_FUSED_ROW_LIST(HC_ROW_FUSED_F32)
#else
HC_FUSED_ROW_LIST(HC_ROW_FUSED_F64)
#endif
