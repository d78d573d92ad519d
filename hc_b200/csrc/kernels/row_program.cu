// Row programs: out[r, :] = f(in0[r, :], in1[r, :], ...) where f may reduce
// along the row (sum, max) and use the reduced values again - the shape of the
// reference's row softmax (python/hckernel/tests/test_examples.py:312-321)
// generalised: centring, normalising, scaling rows by their own statistics.
//
// The expression arrives as a program for the machine of map_machine.cuh,
// cut into passes.  A pass computes an element-wise expression along the row;
// it ends either in a reduction instruction (HC_MAP_RSUM / HC_MAP_RMAX, whose
// result becomes row scalar s[k], an operand of later passes) or, for the last
// pass, in the store of the accumulator to the output row.
//
// One warp per row, eight rows per CTA, one CTA per eight rows.  Every pass
// walks the row again; only the first walk comes from HBM, the row (a few tens
// of KB) is still in L1/L2 for the others, which therefore use ordinary loads
// while the last pass streams.  Reductions are a running value per lane (in
// row order for that lane) and a shuffle tree at the end of the pass, so the
// sum order differs from NumPy's pairwise one in the last bits; max is exact.
#include "map_machine.cuh"

namespace {

using namespace hcmap;

constexpr int UNROLL = 2;

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

template <typename T, int V, int NIN>
__device__ __forceinline__ void rowProgram(const HcMapProgramDev &p) {
  constexpr int W = V * UNROLL;
  __shared__ T temps[3][W][THREADS];
  const int lane = threadIdx.x & 31;
  const long long r = (long long)blockIdx.x * (THREADS / 32) + (threadIdx.x >> 5);
  if (r >= p.rows)
    return; // whole warps leave; nothing below synchronises the CTA
  const int perRow = int(p.cols / V); // the host refuses rows of 2^31 packets and more
  const T *rowIn[NIN];
#pragma unroll
  for (int k = 0; k < NIN; ++k)
    rowIn[k] = static_cast<const T *>(p.in[k < p.nInputs ? k : 0]) + r * p.inPitch[k < p.nInputs ? k : 0];
  T *const rowOut = static_cast<T *>(p.out) + r * p.outPitch;
  T scalars[4] = {T(0), T(0), T(0), T(0)};

  int pc = 0;
  while (pc < p.nInstr) {
    // Uniform prologue: expressions of row scalars and constants only (the
    // log of a sum, a mean from a sum ...) are computed once per row here,
    // not once per element in the walk below.
    T one = T(0);
    for (; pc < p.nInstr && (p.code[pc] & HC_MAP_UNIFORM); ++pc) {
      const uint32_t op = p.code[pc] & 0x7fu, src = p.code[pc] >> 8;
      T b = T(0);
      if (op <= HC_MAP_MIN) {
        if (src >= HC_MAP_SRC_SCALAR) {
          const uint32_t k = src - HC_MAP_SRC_SCALAR;
          b = k == 0 ? scalars[0] : k == 1 ? scalars[1] : k == 2 ? scalars[2] : scalars[3];
        } else {
          b = T(p.consts[src - HC_MAP_SRC_CONST]);
        }
      }
      switch (op) {
      case HC_MAP_LOAD: one = b; break;
      case HC_MAP_ADD: one = one + b; break;
      case HC_MAP_SUB: one = one - b; break;
      case HC_MAP_RSUB: one = b - one; break;
      case HC_MAP_MUL: one = one * b; break;
      case HC_MAP_DIV: one = one / b; break;
      case HC_MAP_RDIV: one = b / one; break;
      case HC_MAP_MAX: one = maxOf(one, b); break;
      case HC_MAP_MIN: one = minOf(one, b); break;
      case HC_MAP_NEG: one = -one; break;
      case HC_MAP_ABS: one = one < T(0) ? -one : (one == T(0) ? T(0) : one); break;
      case HC_MAP_EXP: one = expOf(one); break;
      case HC_MAP_SQRT: one = sqrt(one); break;
      case HC_MAP_LOG: one = logOf(one); break;
      case HC_MAP_SET:
        switch (src) {
        case 0: scalars[0] = one; break;
        case 1: scalars[1] = one; break;
        case 2: scalars[2] = one; break;
        default: scalars[3] = one; break;
        }
        break;
      default: break;
      }
    }
    // The pass runs to the next reduction instruction or to the end.
    int end = pc;
    uint32_t reduction = 0, target = 0;
    for (; end < p.nInstr; ++end) {
      const uint32_t op = p.code[end] & 0xffu;
      if (op == HC_MAP_RSUM || op == HC_MAP_RMAX) {
        reduction = op;
        target = p.code[end] >> 8;
        break;
      }
    }
    const bool last = end >= p.nInstr;
    const bool takeMax = reduction == HC_MAP_RMAX;
    T running = takeMax ? lowest<T>() : T(0);

    for (int base = lane; base < perRow; base += 32 * UNROLL) {
      // Every packet of this step lies inside the row (the same for all lanes)?
      const bool whole = base - lane + 32 * UNROLL <= perRow;
      T x[NIN][W];
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
            x[k][u * V + e] = packet.v[e];
        }
      T value[W];
      evaluate<T, W, V, NIN, false, true, 32>(p, pc, end, x, value, temps, r, base, scalars);
      if (last) {
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
      } else if (takeMax) {
#pragma unroll
        for (int u = 0; u < UNROLL; ++u)
          if (whole || base + u * 32 < perRow) {
#pragma unroll
            for (int e = 0; e < V; ++e)
              running = maxNan(running, value[u * V + e]);
          }
      } else {
#pragma unroll
        for (int u = 0; u < UNROLL; ++u)
          if (whole || base + u * 32 < perRow) {
#pragma unroll
            for (int e = 0; e < V; ++e)
              running = running + value[u * V + e];
          }
      }
    }
    if (last)
      break;
#pragma unroll
    for (int offset = 16; offset > 0; offset >>= 1) {
      const T other = __shfl_xor_sync(0xffffffffu, running, offset);
      running = takeMax ? maxNan(running, other) : running + other;
    }
    switch (target) { // named registers, no indexed access
    case 0: scalars[0] = running; break;
    case 1: scalars[1] = running; break;
    case 2: scalars[2] = running; break;
    default: scalars[3] = running; break;
    }
    pc = end + 1;
  }
}

} // namespace

#define HC_ROW_KERNEL(tname, T, V, NIN)                                                 \
  extern "C" __global__ void __launch_bounds__(THREADS, sizeof(T) == 8 ? 3 : 4)         \
      hc_row_program_##tname##_v##V##_n##NIN(const __grid_constant__ HcMapProgramDev p) { \
    rowProgram<T, V, NIN>(p);                                                           \
  }
#define HC_ROW_KERNELS(tname, T, V)                                                     \
  HC_ROW_KERNEL(tname, T, V, 1)                                                         \
  HC_ROW_KERNEL(tname, T, V, 2)

HC_ROW_KERNELS(f32, float, 4)
HC_ROW_KERNELS(f32, float, 1)
HC_ROW_KERNELS(f64, double, 2)
HC_ROW_KERNELS(f64, double, 1)
