// Gathered tile product - the GPU form of work-groups that load their operand
// tiles through index mappings, multiply them and scatter the result:
//
//   A_g[a, k]                 = x[xOrigin(g) + xMap(a, k)]      (0 if outside x)
//   B_g[k, b]                 = f[fOrigin(g) + fMap(k, b)]      (0 if outside f)
//   out[oOrigin(g) + oMap(a, b)] = sum_k A_g[a, k] * B_g[k, b]  (dropped if outside out)
//
// for every work-group g.  This is what group.load(view, shape, mapping=m),
// np.dot over K blocks and group.store(view, tile, mapping=m) compute in the
// reference (python/hckernel/kernel_api.py:297-336); its example is the
// convolution written as an implicit GEMM
// (python/hckernel/tests/test_examples.py:203-252), where xMap walks the
// receptive field of an output position and fMap reads the filter bank
// transposed.
//
// The mappings are arbitrary Python functions, so they reach the kernel as
// tables evaluated once on the host: per tile element the mapped index
// (relative to the tile origin, one int per dimension) and the same index as a
// linear element offset; per work-group the tile origins.  One CTA computes
// one work-group.  A group whose whole tile lies inside the array ("interior",
// decided from the per-dimension extremes of the table) only reads the 4-byte
// linear offsets; an edge group also reads the 16-byte index and compares it
// with what is left of the array from its origin.
//
// Gathers are only as fast as they are coalesced, and which neighbours in a
// tile are neighbours in memory depends on the mapping (the filter tile of the
// convolution is contiguous along K, not along its columns).  So each operand
// table comes in the order the host found best (row-major or transposed) and
// consecutive threads take consecutive table entries.
//
// A gather is two dependent loads (offset, then element), both usually served
// by L2.  To keep that latency off the multiply loop the operands travel as
// 4- or 8-byte cp.async copies straight into a three-stage ring of K chunks
// in shared memory (a copy with source size 0 writes the zero of an element
// outside its array), and the offsets a chunk needs are loaded into registers
// one chunk before its copies are issued.
//
// TY x TX threads (8 or 16 each way), each owning MY adjacent rows and MX
// adjacent columns of the result (1, 2, 4, or 8 rows in the 128-row pieces), so
// that one or two 8- or 16-byte shared-memory loads bring all of a thread's
// rows (columns) for one k.  A
// chunk is [k][row] and [k][column] with 4-element groups XOR-swizzled with k,
// so that the copies of a warp spread over the banks.  Tiles larger than
// TY*MY x TX*MX are walked in pieces.
//
// Work-groups whose f tile is the same (consecutive output positions of the
// convolution) are stacked: one CTA takes up to eight of them, as long as the
// stacked rows fit one piece (128 rows for float, 64 for double), gathers the f tile once and multiplies it
// with the rows of all of them.  The result of every group is what it would be
// alone (same sum order); the stack only shares the B side.
//
// What bounds it: with tiles of a few thousand elements a thread owns few
// results, so the shared-memory side of the L1 pipe (one or two wavefronts per
// 8- or 16-byte load of a quarter warp), not the FMA pipe, sets the pace;
// larger tiles and stacks move the balance towards the FMA pipe.
#include "mapped_params.h"

#include <stdint.h>

namespace {

constexpr int KC = 16;
constexpr int kMaxStack = 8; // work-groups one CTA may stack (the launcher asks for <= 8)

struct GroupView {
  long long base; // linear offset of the tile origin
  int lim[4];     // what is left of the array from the origin, per dimension
  int interior;   // every element of the tile is inside the array
};

__device__ __forceinline__ void openView(const HcMappedOperandDev &op, long long g,
                                         GroupView &v) {
  const int4 org = reinterpret_cast<const int4 *>(op.origins)[g];
  const int o[4] = {org.x, org.y, org.z, org.w};
  long long base = 0;
  int interior = 1;
#pragma unroll
  for (int d = 0; d < 4; ++d) {
    base += (long long)o[d] * op.stride[d];
    const int lim = op.shape[d] - o[d];
    v.lim[d] = lim;
    interior &= (op.lo[d] >= 0 && op.hi[d] < lim) ? 1 : 0;
  }
  v.base = base;
  v.interior = interior;
}

__device__ __forceinline__ bool inside(const HcMappedOperandDev &op, const GroupView &v,
                                       int idx) {
  if (v.interior)
    return true;
  const int4 r = reinterpret_cast<const int4 *>(op.map)[idx];
  return r.x >= 0 && r.x < v.lim[0] && r.y >= 0 && r.y < v.lim[1] && r.z >= 0 &&
         r.z < v.lim[2] && r.w >= 0 && r.w < v.lim[3];
}

// Which element of a [rows x KC] chunk thread-slot `e` carries: in table
// order, so a warp takes all 16 k of two adjacent rows where the table has k
// as its fastest index, and 32 adjacent rows of one k otherwise.
__device__ __forceinline__ void chunkElement(int e, int span, bool kFastest, int &r, int &kk) {
  if (kFastest) {
    kk = e % KC;
    r = e / KC;
  } else {
    r = e % span;
    kk = e / span;
  }
}

// Position of element `c` in row `kk` of a staged chunk.  The group of four
// that `c` is in is XOR-ed with k (8 phases), and the two pairs inside a group
// change places for k >= 8, so that the 32 copies of a warp (16 k of two
// adjacent elements) land in 32 different banks.  Aligned runs of one or two
// elements stay whole; a run of four comes back with its halves exchanged for
// k >= 8 (loadRun puts them right).
template <int SPAN>
__device__ __forceinline__ int swizzled(int kk, int c) {
  constexpr int groups = SPAN / 4; // 2, 4, 8 or 16 groups per row
  return c ^ (((kk & (groups < 8 ? groups - 1 : 7)) << 2) | (((kk >> 3) & 1) << 1));
}

// The N adjacent elements that start at (unswizzled) position `c` of row `kk`.
template <typename T, int N, int SPAN>
__device__ __forceinline__ void loadRun(const T (&row)[SPAN], int kk, int c, T (&dst)[N]) {
  constexpr int bytes = N * int(sizeof(T));
  if constexpr (N == 8) { // two runs of four
    T low[4], high[4];
    loadRun<T, 4, SPAN>(row, kk, c, low);
    loadRun<T, 4, SPAN>(row, kk, c + 4, high);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      dst[i] = low[i];
      dst[4 + i] = high[i];
    }
  } else if constexpr (N == 4) {
    const T *src = &row[swizzled<SPAN>(kk, c) & ~3];
    alignas(16) T raw[4];
#pragma unroll
    for (int i = 0; i < bytes / 16; ++i)
      reinterpret_cast<uint4 *>(raw)[i] = reinterpret_cast<const uint4 *>(src)[i];
    const bool exchanged = (kk & 8) != 0;
    dst[0] = exchanged ? raw[2] : raw[0];
    dst[1] = exchanged ? raw[3] : raw[1];
    dst[2] = exchanged ? raw[0] : raw[2];
    dst[3] = exchanged ? raw[1] : raw[3];
  } else if constexpr (bytes == 16) {
    *reinterpret_cast<uint4 *>(dst) = *reinterpret_cast<const uint4 *>(&row[swizzled<SPAN>(kk, c)]);
  } else if constexpr (bytes == 8) {
    *reinterpret_cast<uint2 *>(dst) = *reinterpret_cast<const uint2 *>(&row[swizzled<SPAN>(kk, c)]);
  } else {
    dst[0] = row[swizzled<SPAN>(kk, c)];
  }
}

// One element, global -> shared, asynchronously; `valid` false writes zero and
// reads nothing.
template <typename T>
__device__ __forceinline__ void copyAsync(T *dstShared, const T *src, bool valid) {
  const unsigned dst = static_cast<unsigned>(__cvta_generic_to_shared(dstShared));
  const int bytes = valid ? int(sizeof(T)) : 0;
  if constexpr (sizeof(T) == 4)
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;" ::"r"(dst), "l"(src), "r"(bytes)
                 : "memory");
  else
    asm volatile("cp.async.ca.shared.global [%0], [%1], 8, %2;" ::"r"(dst), "l"(src), "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ void commitCopies() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void waitCopies() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

// How one side of the CTA's piece of the tile is split: `SPAN` rows (columns)
// as `threads` threads with `each` adjacent rows (columns) apiece.
template <int SPAN>
struct Side {
  static constexpr int threads = SPAN >= 32 ? 16 : 8;
  static constexpr int each = SPAN / threads; // 1, 2, 2, 4, 8 for 8, 16, 32, 64, 128
};

template <int SY, int SX>
__host__ __device__ constexpr int threadsOf() {
  return Side<SY>::threads * Side<SX>::threads;
}

// CTAs per SM the register allocation should leave room for (occupancy is what
// hides the gathers): 40 registers of addressing, the copy offsets and one and
// a half times the accumulators per thread.
template <typename T, int SY, int SX>
__host__ __device__ constexpr int residentCtas() {
  constexpr int MY = Side<SY>::each, MX = Side<SX>::each, NT = threadsOf<SY, SX>();
  constexpr int regs =
      40 + MY * MX * int(sizeof(T) / 4) * 3 / 2 + (SY + SX) * KC / NT + 2 * SY * KC / NT;
  constexpr int fit = 65536 / (NT * regs);
  return fit < 1 ? 1 : fit > 8 ? 8 : fit;
}

template <typename T, int SY, int SX>
__device__ __forceinline__ void mappedGemm(const HcMappedGemmParams &p) {
  constexpr int MY = Side<SY>::each, MX = Side<SX>::each;
  constexpr int TX = Side<SX>::threads, THREADS = threadsOf<SY, SX>();
  constexpr int NA = SY * KC / THREADS, NB = SX * KC / THREADS; // copies per thread and chunk
  // Three stages, two where three would pass the 48 KB of static shared memory.
  constexpr int STAGES = 3 * KC * (SY + SX) * int(sizeof(T)) > 47 * 1024 ? 2 : 3;
  __shared__ __align__(16) T sA[STAGES][KC][SY]; // [stage][k][row], swizzled
  __shared__ __align__(16) T sB[STAGES][KC][SX]; // [stage][k][column], swizzled
  // A CTA takes `stack` consecutive work-groups that share their f tile and
  // computes them as one product with stack * TM rows.
  __shared__ GroupView xViews[kMaxStack], outViews[kMaxStack], fView;

  const int tid = threadIdx.x;
  const int TM = p.TM, TN = p.TN, K = p.K, stack = p.stack;
  const long long g0 = (long long)blockIdx.x * stack;
  if (tid < 2 * stack + 1) {
    const int which = tid % 2, j = tid / 2; // (x, out) of stacked group j; the last one: f
    const long long g = g0 + j;
    if (tid == 2 * stack) {
      openView(p.f, g0, fView);
    } else if (g < p.groups) {
      openView(which == 0 ? p.x : p.out, g, which == 0 ? xViews[j] : outViews[j]);
    } else { // past the last work-group: nothing is inside
      GroupView &v = which == 0 ? xViews[j] : outViews[j];
      v.base = 0;
      v.interior = 0;
      v.lim[0] = v.lim[1] = v.lim[2] = v.lim[3] = 0;
    }
  }
  __syncthreads();
  const int ty = tid / TX, tx = tid % TX;
  const int rows = stack * TM;
  // x natural order is [a][k] (k fastest); f natural order is [k][b].
  const bool xKFast = !p.x.transposed, fKFast = p.f.transposed != 0;
  const T *xArray = static_cast<const T *>(p.x.base);
  const T *fArray = static_cast<const T *>(p.f.base), *fBase = fArray + fView.base;
  const int chunks = (K + KC - 1) / KC;

  for (int m0 = 0; m0 < rows; m0 += SY)
    for (int n0 = 0; n0 < TN; n0 += SX) {
      T acc[MY][MX];
#pragma unroll
      for (int i = 0; i < MY; ++i)
#pragma unroll
        for (int j = 0; j < MX; ++j)
          acc[i][j] = T(0);

      // What stays the same from chunk to chunk for each of this thread's
      // elements: where it lands in a stage, its table index in chunk 0 (the
      // index advances by a fixed step per chunk) and, for A, the stacked
      // group its row belongs to (-1: a row or column past the tile).
      int landA[NA], landB[NB], tableA[NA], tableB[NB], groupOfA[NA];
#pragma unroll
      for (int i = 0; i < NA; ++i) {
        int aa, kk;
        chunkElement(tid + i * THREADS, SY, xKFast, aa, kk);
        const int row = m0 + aa, a = row % TM;
        landA[i] = kk * SY + swizzled<SY>(kk, aa);
        tableA[i] = xKFast ? a * K + kk : kk * TM + a;
        groupOfA[i] = row < rows ? row / TM : -1;
      }
#pragma unroll
      for (int j = 0; j < NB; ++j) {
        int bb, kk;
        chunkElement(tid + j * THREADS, SX, fKFast, bb, kk);
        const int b = n0 + bb;
        landB[j] = kk * SX + swizzled<SX>(kk, bb);
        tableB[j] = b < TN ? (fKFast ? b * K + kk : kk * TN + b) : -1;
      }
      const int stepA = xKFast ? KC : KC * TM, stepB = fKFast ? KC : KC * TN;
      // Offsets of this thread's elements of one chunk; negative = reads as zero.
      int offA[NA], offB[NB];
      auto loadOffsets = [&](int chunk) {
        const int k0 = chunk * KC;
#pragma unroll
        for (int i = 0; i < NA; ++i) {
          const int k = k0 + landA[i] / SY, idx = tableA[i] + chunk * stepA;
          offA[i] = (groupOfA[i] >= 0 && k < K && inside(p.x, xViews[groupOfA[i]], idx))
                        ? __ldg(p.x.lin + idx)
                        : -1;
        }
#pragma unroll
        for (int j = 0; j < NB; ++j) {
          const int k = k0 + landB[j] / SX, idx = tableB[j] + chunk * stepB;
          offB[j] = (tableB[j] >= 0 && k < K && inside(p.f, fView, idx)) ? __ldg(p.f.lin + idx)
                                                                          : -1;
        }
      };
      // Mapped offsets are never negative for an element inside its array
      // (origins and in-range relative indices are >= 0, strides are >= 0).
      auto issueCopies = [&](int stage) {
        T *stageA = &sA[stage][0][0], *stageB = &sB[stage][0][0];
#pragma unroll
        for (int i = 0; i < NA; ++i) {
          const bool valid = offA[i] >= 0;
          copyAsync(stageA + landA[i],
                    valid ? xArray + xViews[groupOfA[i]].base + offA[i] : xArray, valid);
        }
#pragma unroll
        for (int j = 0; j < NB; ++j) {
          const bool valid = offB[j] >= 0;
          copyAsync(stageB + landB[j], valid ? fBase + offB[j] : fArray, valid);
        }
        commitCopies();
      };

      __syncthreads(); // the previous piece is done with the ring
      // Fill the first STAGES-1 stages; keep the offsets of the next chunk ready.
      loadOffsets(0);
#pragma unroll
      for (int s = 0; s < STAGES - 1; ++s) {
        issueCopies(s); // chunks past the end copy zeros
        loadOffsets(s + 1);
      }
      for (int c = 0; c < chunks; ++c) {
        waitCopies<STAGES - 2>(); // chunk c has landed (this thread's part)
        __syncthreads();          // ... everyone's part; and chunk c-1 is no longer read
        issueCopies((c + STAGES - 1) % STAGES);
        loadOffsets(c + STAGES);
        const int stage = c % STAGES;
#pragma unroll
        for (int kk = 0; kk < KC; ++kk) {
          alignas(16) T av[MY];
          alignas(16) T bv[MX];
          loadRun<T, MY, SY>(sA[stage][kk], kk, ty * MY, av);
          loadRun<T, MX, SX>(sB[stage][kk], kk, tx * MX, bv);
#pragma unroll
          for (int i = 0; i < MY; ++i)
#pragma unroll
            for (int j = 0; j < MX; ++j)
              acc[i][j] += av[i] * bv[j];
        }
      }
      waitCopies<0>();

#pragma unroll
      for (int i = 0; i < MY; ++i) {
        const int row = m0 + ty * MY + i;
        if (row >= rows)
          continue;
        const GroupView &view = outViews[row / TM];
        const int a = row % TM;
#pragma unroll
        for (int j = 0; j < MX; ++j) {
          const int b = n0 + tx * MX + j;
          if (b >= TN)
            continue;
          const int idx = a * TN + b;
          if (inside(p.out, view, idx))
            static_cast<T *>(p.out.base)[view.base + p.out.lin[idx]] = acc[i][j];
        }
      }
    }
}

} // namespace

// One kernel per piece shape SY x SX (8, 16, 32 or 64 each way, and 128 rows
// for float); the launcher picks the smallest piece that holds the tile.
#define HC_MAPPED_KERNEL(T, tname, SY, SX)                                              \
  extern "C" __global__ void                                                            \
      __launch_bounds__(threadsOf<SY, SX>(), residentCtas<T, SY, SX>())                 \
          hc_mapped_gemm_##tname##_##SY##x##SX(const __grid_constant__ HcMappedGemmParams p) { \
    mappedGemm<T, SY, SX>(p);                                                           \
  }
#define HC_MAPPED_ROW(T, tname, SY)                                                     \
  HC_MAPPED_KERNEL(T, tname, SY, 8)                                                     \
  HC_MAPPED_KERNEL(T, tname, SY, 16)                                                    \
  HC_MAPPED_KERNEL(T, tname, SY, 32)                                                    \
  HC_MAPPED_KERNEL(T, tname, SY, 64)
#define HC_MAPPED_KERNELS(T, tname)                                                     \
  HC_MAPPED_ROW(T, tname, 8)                                                            \
  HC_MAPPED_ROW(T, tname, 16)                                                           \
  HC_MAPPED_ROW(T, tname, 32)                                                           \
  HC_MAPPED_ROW(T, tname, 64)

HC_MAPPED_KERNELS(float, f32)
HC_MAPPED_KERNELS(double, f64)
// Tall pieces for stacks of work-groups (float only: three stages of a
// 128-row piece of doubles would not fit the static shared memory): a thread
// owns 8 rows, so a k costs three 16-byte shared loads for 32 products where
// the 64-row piece needs two for 16.  Only with 16 threads across: on 8 the
// copies per thread would double.
HC_MAPPED_KERNEL(float, f32, 128, 32)
HC_MAPPED_KERNEL(float, f32, 128, 64)
