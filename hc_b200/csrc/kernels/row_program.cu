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

// Packets per lane and decode of the walking kernel.  Four (three CTAs per SM
// for float) measured 3.8 TB/s on a log-softmax of 4096-column rows where two
// (four CTAs per SM) gave 3.1: the decode is shared by twice the elements.
constexpr int UNROLL = 4;

// Uniform prologue of a pass: expressions of row scalars and constants only
// (the log of a sum, a mean from a sum ...) are computed once per row here, not
// once per element in the walk that follows.  Returns the first instruction
// of the walk.
template <typename T>
__device__ __forceinline__ int uniformPrologue(const HcMapProgramDev &p, int pc, T (&scalars)[4]) {
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
  return pc;
}

// Where the pass that starts at `pc` ends: at the next reduction instruction
// (returned through `reduction` and `target`) or at the end of the program.
__device__ __forceinline__ int passEnd(const HcMapProgramDev &p, int pc, uint32_t &reduction,
                                       uint32_t &target) {
  reduction = 0;
  target = 0;
  int end = pc;
  for (; end < p.nInstr; ++end) {
    const uint32_t op = p.code[end] & 0xffu;
    if (op == HC_MAP_RSUM || op == HC_MAP_RMAX) {
      reduction = op;
      target = p.code[end] >> 8;
      break;
    }
  }
  return end;
}

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
    pc = uniformPrologue<T>(p, pc, scalars);
    uint32_t reduction, target;
    const int end = passEnd(p, pc, reduction, target);
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
      uint32_t ok = ~0u; // row programs do not track validity
      uint64_t parkedOk = ~0ull;
      evaluate<T, W, V, NIN, false, true, 32>(p, pc, end, x, value, temps, r, base, scalars, ok,
                                              parkedOk);
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

// Rows of up to P * 256 packets, held in registers: one CTA per row, thread t
// owns packets t, t + 256, ... of the row.  The row is read from HBM once, with
// streaming loads; every pass works on the registers, so the later passes issue
// no loads and no address arithmetic, and an instruction is decoded once for
// P packets.  A reduction is a running value per thread, a shuffle tree per
// warp and the eight warp results added (or compared) in warp order by every
// thread, so all threads hold the same row scalar.
//
// Dynamic shared memory: 256 bytes for the warp results (four slots of eight
// values, so that one barrier per reduction is enough), then as many of the
// three temporaries as the program saves to.
template <typename T, int V, int P, int NIN, int NT>
__device__ __forceinline__ void rowProgramHeld(const HcMapProgramDev &p) {
  constexpr int W = V * P;
  extern __shared__ __align__(16) unsigned char raw[];
  T(*const partial)[NT / 32] = reinterpret_cast<T(*)[NT / 32]>(raw);
  T(&temps)[3][W][NT] = *reinterpret_cast<T(*)[3][W][NT]>(raw + 256);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const long long r = blockIdx.x;
  const int perRow = int(p.cols / V);

  T x[NIN][W];
#pragma unroll
  for (int k = 0; k < NIN; ++k)
#pragma unroll
    for (int u = 0; u < P; ++u) {
      const int i = threadIdx.x + u * NT;
      Packet<T, V> packet;
      if (k < p.nInputs && i < perRow) {
        packet = loadPacket<T, V>(static_cast<const T *>(p.in[k]) + r * p.inPitch[k] +
                                  (long long)i * V);
      } else {
#pragma unroll
        for (int e = 0; e < V; ++e)
          packet.v[e] = T(0);
      }
#pragma unroll
      for (int e = 0; e < V; ++e)
        x[k][u * V + e] = packet.v[e];
    }

  T scalars[4] = {T(0), T(0), T(0), T(0)};
  int pc = 0, reductions = 0;
  while (pc < p.nInstr) { // the same trip count for every thread of the CTA
    pc = uniformPrologue<T>(p, pc, scalars);
    uint32_t reduction, target;
    const int end = passEnd(p, pc, reduction, target);
    T value[W];
    uint32_t ok = ~0u; // row programs do not track validity
    uint64_t parkedOk = ~0ull;
    evaluate<T, W, V, NIN, false, true, NT, NT>(p, pc, end, x, value, temps, r, threadIdx.x,
                                                 scalars, ok, parkedOk);
    if (end >= p.nInstr) {
      T *const rowOut = static_cast<T *>(p.out) + r * p.outPitch;
#pragma unroll
      for (int u = 0; u < P; ++u) {
        const int i = threadIdx.x + u * NT;
        if (i < perRow) {
          Packet<T, V> packet;
#pragma unroll
          for (int e = 0; e < V; ++e)
            packet.v[e] = value[u * V + e];
          storePacket<T, V>(rowOut + (long long)i * V, packet);
        }
      }
      break;
    }
    const bool takeMax = reduction == HC_MAP_RMAX;
    T running = takeMax ? lowest<T>() : T(0);
    if (takeMax) {
#pragma unroll
      for (int u = 0; u < P; ++u)
        if (threadIdx.x + u * NT < perRow) {
#pragma unroll
          for (int e = 0; e < V; ++e)
            running = maxNan(running, value[u * V + e]);
        }
    } else {
#pragma unroll
      for (int u = 0; u < P; ++u)
        if (threadIdx.x + u * NT < perRow) {
#pragma unroll
          for (int e = 0; e < V; ++e)
            running = running + value[u * V + e];
        }
    }
    if (takeMax) {
#pragma unroll
      for (int offset = 16; offset > 0; offset >>= 1)
        running = maxNan(running, __shfl_xor_sync(0xffffffffu, running, offset));
    } else {
#pragma unroll
      for (int offset = 16; offset > 0; offset >>= 1)
        running = running + __shfl_xor_sync(0xffffffffu, running, offset);
    }
    // Slot n is written again only after three more barriers, long after its
    // last reader has passed the next one.
    T *const slot = partial[reductions & 3];
    ++reductions;
    if (lane == 0)
      slot[warp] = running;
    __syncthreads();
    T whole = slot[0];
    if (takeMax) {
#pragma unroll
      for (int w = 1; w < NT / 32; ++w)
        whole = maxNan(whole, slot[w]);
    } else {
#pragma unroll
      for (int w = 1; w < NT / 32; ++w)
        whole = whole + slot[w];
    }
    switch (target) {
    case 0: scalars[0] = whole; break;
    case 1: scalars[1] = whole; break;
    case 2: scalars[2] = whole; break;
    default: scalars[3] = whole; break;
    }
    pc = end + 1;
  }
}

} // namespace

#define HC_ROW_KERNEL(tname, T, V, NIN)                                                 \
  extern "C" __global__ void __launch_bounds__(THREADS, sizeof(T) == 8 ? 2 : 3)         \
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

// Held-row kernels.  Eight packets per thread on 64, 96 or 128 threads (rows
// of up to 512, 768, 1024 packets): the fewer threads share a row, the fewer
// decode each instruction, and the more elements each decode serves.  Four
// packets per thread on 256 threads is the alternative for rows of 513..1024
// packets with twice the resident warps.  The last argument is the number of
// CTAs per SM the register budget is set for.
#define HC_ROW_HELD_KERNEL(tname, T, V, P, NT, NIN, CTAS)                               \
  extern "C" __global__ void __launch_bounds__(NT, CTAS)                                \
      hc_row_program_held_##tname##_v##V##_p##P##_t##NT##_n##NIN(                       \
          const __grid_constant__ HcMapProgramDev p) {                                  \
    rowProgramHeld<T, V, P, NIN, NT>(p);                                                \
  }

HC_ROW_HELD_KERNEL(f32, float, 4, 8, 128, 1, 4)
HC_ROW_HELD_KERNEL(f32, float, 4, 8, 96, 1, 5)
HC_ROW_HELD_KERNEL(f32, float, 4, 8, 64, 1, 8)
HC_ROW_HELD_KERNEL(f32, float, 4, 8, 128, 2, 3)
HC_ROW_HELD_KERNEL(f32, float, 4, 8, 96, 2, 4)
HC_ROW_HELD_KERNEL(f32, float, 4, 8, 64, 2, 6)
HC_ROW_HELD_KERNEL(f32, float, 4, 4, 256, 1, 4)
HC_ROW_HELD_KERNEL(f32, float, 4, 4, 256, 2, 3)
HC_ROW_HELD_KERNEL(f64, double, 2, 8, 128, 1, 3)
HC_ROW_HELD_KERNEL(f64, double, 2, 8, 96, 1, 4)
HC_ROW_HELD_KERNEL(f64, double, 2, 8, 64, 1, 6)
HC_ROW_HELD_KERNEL(f64, double, 2, 8, 128, 2, 2)
HC_ROW_HELD_KERNEL(f64, double, 2, 8, 96, 2, 3)
HC_ROW_HELD_KERNEL(f64, double, 2, 8, 64, 2, 4)
HC_ROW_HELD_KERNEL(f64, double, 2, 4, 256, 1, 3)
HC_ROW_HELD_KERNEL(f64, double, 2, 4, 256, 2, 2)
