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
// 256 threads as 16 x 16, each owning an MY x MX block of the result with a
// stride of 16 between its rows and columns; the operands pass through shared
// memory in K chunks of 16, the next chunk being fetched into registers while
// the current one is multiplied.  Tiles larger than 16*MY x 16*MX are walked
// in pieces.
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

template <typename T, int MY, int MX>
__device__ __forceinline__ void mappedGemm(const HcMappedGemmParams &p) {
  constexpr int SY = 16 * MY, SX = 16 * MX;
  __shared__ T sA[KC][SY + 1]; // [k][row]
  __shared__ T sB[KC][SX + 1]; // [k][column]
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
          sA[kk][aa] = ra[i];
        }
#pragma unroll
        for (int j = 0; j < MX; ++j) {
          int bb, kk;
          chunkElement(tid + j * THREADS, SX, fKFast, bb, kk);
          sB[kk][bb] = rb[j];
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
          T av[MY], bv[MX];
#pragma unroll
          for (int i = 0; i < MY; ++i)
            av[i] = sA[kk][ty + 16 * i];
#pragma unroll
          for (int j = 0; j < MX; ++j)
            bv[j] = sB[kk][tx + 16 * j];
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
        const int a = m0 + ty + 16 * i;
        if (a >= TM)
          continue;
#pragma unroll
        for (int j = 0; j < MX; ++j) {
          const int b = n0 + tx + 16 * j;
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

#define HC_MAPPED_KERNEL(T, tname, MY, MX)                                              \
  extern "C" __global__ void __launch_bounds__(THREADS)                                 \
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
