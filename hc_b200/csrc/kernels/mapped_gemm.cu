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
// 256 threads as 16 x 16, each owning MY adjacent rows and MX adjacent columns
// of the result, so that one 8- or 16-byte shared-memory load brings all of a
// thread's rows (columns) for one k.  The operands pass through shared memory
// in K chunks of 16 ([k][row] and [k][column], 4-element groups XOR-swizzled
// with k so that a warp that stages 16 consecutive k of two rows spreads over
// the banks); the next chunk is fetched into registers while the current one
// is multiplied.  Tiles larger than 16*MY x 16*MX are walked in pieces.
#include "mapped_params.h"

#include <stdint.h>

namespace {

constexpr int KC = 16, THREADS = 256;

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

template <typename T>
__device__ __forceinline__ T fetch(const HcMappedOperandDev &op, const GroupView &v, int idx) {
  if (!inside(op, v, idx))
    return T(0);
  return __ldg(static_cast<const T *>(op.base) + v.base + __ldg(op.lin + idx));
}

// Element `e` of a [rows x KC] chunk in table order: k fastest when the table
// has k as its fastest index, the row (or column) of the tile otherwise.
__device__ __forceinline__ void chunkElement(int e, int span, bool kFastest, int &r, int &kk) {
  if (kFastest) {
    kk = e % KC;
    r = e / KC;
  } else {
    r = e % span;
    kk = e / span;
  }
}

// Position of element `c` in row `kk` of a staged chunk: groups of four
// elements are XOR-ed with k.  Aligned runs of 1, 2 or 4 elements stay whole.
template <int SPAN>
__device__ __forceinline__ int swizzled(int kk, int c) {
  constexpr int groups = SPAN / 4; // 4, 8 or 16 groups per row
  return c ^ ((kk & (groups < 8 ? groups - 1 : 7)) << 2);
}

// N adjacent elements from shared memory with the widest loads that fit.
template <typename T, int N>
__device__ __forceinline__ void loadRun(const T *src, T (&dst)[N]) {
  constexpr int bytes = N * int(sizeof(T));
  if constexpr (bytes % 16 == 0) {
#pragma unroll
    for (int i = 0; i < bytes / 16; ++i)
      reinterpret_cast<uint4 *>(dst)[i] = reinterpret_cast<const uint4 *>(src)[i];
  } else if constexpr (bytes == 8) {
    *reinterpret_cast<uint2 *>(dst) = *reinterpret_cast<const uint2 *>(src);
  } else {
    dst[0] = src[0];
  }
}

template <typename T, int MY, int MX>
__device__ __forceinline__ void mappedGemm(const HcMappedGemmParams &p) {
  constexpr int SY = 16 * MY, SX = 16 * MX;
  __shared__ __align__(16) T sA[KC][SY]; // [k][row], swizzled
  __shared__ __align__(16) T sB[KC][SX]; // [k][column], swizzled
  __shared__ GroupView views[3];

  const int tid = threadIdx.x;
  const long long g = blockIdx.x;
  if (tid < 3)
    openView(tid == 0 ? p.x : tid == 1 ? p.f : p.out, g, views[tid]);
  __syncthreads();
  const int ty = tid >> 4, tx = tid & 15;
  const int TM = p.TM, TN = p.TN, K = p.K;
  // x natural order is [a][k] (k fastest); f natural order is [k][b].
  const bool xKFast = !p.x.transposed, fKFast = p.f.transposed != 0;

  for (int m0 = 0; m0 < TM; m0 += SY)
    for (int n0 = 0; n0 < TN; n0 += SX) {
      T acc[MY][MX];
#pragma unroll
      for (int i = 0; i < MY; ++i)
#pragma unroll
        for (int j = 0; j < MX; ++j)
          acc[i][j] = T(0);

      T ra[MY], rb[MX]; // this thread's share of the chunk in flight
      auto fetchChunk = [&](int k0) {
#pragma unroll
        for (int i = 0; i < MY; ++i) {
          int aa, kk;
          chunkElement(tid + i * THREADS, SY, xKFast, aa, kk);
          const int a = m0 + aa, k = k0 + kk;
          ra[i] = (a < TM && k < K)
                      ? fetch<T>(p.x, views[0], xKFast ? a * K + k : k * TM + a)
                      : T(0);
        }
#pragma unroll
        for (int j = 0; j < MX; ++j) {
          int bb, kk;
          chunkElement(tid + j * THREADS, SX, fKFast, bb, kk);
          const int b = n0 + bb, k = k0 + kk;
          rb[j] = (b < TN && k < K)
                      ? fetch<T>(p.f, views[1], fKFast ? b * K + k : k * TN + b)
                      : T(0);
        }
      };
      auto stageChunk = [&]() {
#pragma unroll
        for (int i = 0; i < MY; ++i) {
          int aa, kk;
          chunkElement(tid + i * THREADS, SY, xKFast, aa, kk);
          sA[kk][swizzled<SY>(kk, aa)] = ra[i];
        }
#pragma unroll
        for (int j = 0; j < MX; ++j) {
          int bb, kk;
          chunkElement(tid + j * THREADS, SX, fKFast, bb, kk);
          sB[kk][swizzled<SX>(kk, bb)] = rb[j];
        }
      };

      if (K > 0)
        fetchChunk(0);
      for (int k0 = 0; k0 < K; k0 += KC) {
        stageChunk();
        __syncthreads();
        if (k0 + KC < K)
          fetchChunk(k0 + KC);
#pragma unroll
        for (int kk = 0; kk < KC; ++kk) {
          alignas(16) T av[MY];
          alignas(16) T bv[MX];
          loadRun<T, MY>(&sA[kk][swizzled<SY>(kk, ty * MY)], av);
          loadRun<T, MX>(&sB[kk][swizzled<SX>(kk, tx * MX)], bv);
#pragma unroll
          for (int i = 0; i < MY; ++i)
#pragma unroll
            for (int j = 0; j < MX; ++j)
              acc[i][j] += av[i] * bv[j];
        }
        __syncthreads();
      }

#pragma unroll
      for (int i = 0; i < MY; ++i) {
        const int a = m0 + ty * MY + i;
        if (a >= TM)
          continue;
#pragma unroll
        for (int j = 0; j < MX; ++j) {
          const int b = n0 + tx * MX + j;
          if (b >= TN)
            continue;
          const int idx = a * TN + b;
          if (inside(p.out, views[2], idx))
            static_cast<T *>(p.out.base)[views[2].base + p.out.lin[idx]] = acc[i][j];
        }
      }
    }
}

} // namespace

// Gathers hide their latency behind other CTAs: cap the registers so that four
// CTAs fit on an SM (three or two where the accumulators alone take 64 or 128
// bytes per thread).
#define HC_MAPPED_KERNEL(T, tname, MY, MX)                                              \
  extern "C" __global__ void __launch_bounds__(                                         \
      THREADS, MY * MX * sizeof(T) >= 128 ? 2 : MY * MX * sizeof(T) >= 64 ? 3 : 4)      \
      hc_mapped_gemm_##tname##_m##MY##n##MX(const __grid_constant__ HcMappedGemmParams p) { \
    mappedGemm<T, MY, MX>(p);                                                           \
  }
#define HC_MAPPED_KERNELS(T, tname)                                                     \
  HC_MAPPED_KERNEL(T, tname, 1, 1)                                                      \
  HC_MAPPED_KERNEL(T, tname, 1, 2)                                                      \
  HC_MAPPED_KERNEL(T, tname, 1, 4)                                                      \
  HC_MAPPED_KERNEL(T, tname, 2, 1)                                                      \
  HC_MAPPED_KERNEL(T, tname, 2, 2)                                                      \
  HC_MAPPED_KERNEL(T, tname, 2, 4)                                                      \
  HC_MAPPED_KERNEL(T, tname, 4, 1)                                                      \
  HC_MAPPED_KERNEL(T, tname, 4, 2)                                                      \
  HC_MAPPED_KERNEL(T, tname, 4, 4)

HC_MAPPED_KERNELS(float, f32)
HC_MAPPED_KERNELS(double, f64)
