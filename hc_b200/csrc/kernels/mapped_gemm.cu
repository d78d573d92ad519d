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
// 256 threads as 16 x 16, each owning an MT x MT block of the result with a
// stride of 16 between its rows and columns; the operands pass through shared
// memory in K chunks of 16.  Tiles larger than 16*MT are walked in pieces.
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
  return static_cast<const T *>(op.base)[v.base + op.lin[idx]];
}

template <typename T, int MT>
__device__ __forceinline__ void mappedGemm(const HcMappedGemmParams &p) {
  constexpr int S = 16 * MT;
  __shared__ T sA[KC][S + 1]; // [k][row]
  __shared__ T sB[KC][S + 1]; // [k][column]
  __shared__ GroupView views[3];

  const int tid = threadIdx.x;
  const long long g = blockIdx.x;
  if (tid < 3)
    openView(tid == 0 ? p.x : tid == 1 ? p.f : p.out, g, views[tid]);
  __syncthreads();
  const int ty = tid >> 4, tx = tid & 15;
  const int TM = p.TM, TN = p.TN, K = p.K;

  for (int m0 = 0; m0 < TM; m0 += S)
    for (int n0 = 0; n0 < TN; n0 += S) {
      T acc[MT][MT];
#pragma unroll
      for (int i = 0; i < MT; ++i)
#pragma unroll
        for (int j = 0; j < MT; ++j)
          acc[i][j] = T(0);

      for (int k0 = 0; k0 < K; k0 += KC) {
        // A: consecutive threads take consecutive k of one row (the table and,
        // for patch gathers, the data are contiguous that way).
        for (int e = tid; e < S * KC; e += THREADS) {
          const int kk = e % KC, aa = e / KC;
          const int a = m0 + aa, k = k0 + kk;
          sA[kk][aa] = (a < TM && k < K) ? fetch<T>(p.x, views[0], a * K + k) : T(0);
        }
        // B: consecutive threads take consecutive columns of one k.
        for (int e = tid; e < S * KC; e += THREADS) {
          const int bb = e % S, kk = e / S;
          const int b = n0 + bb, k = k0 + kk;
          sB[kk][bb] = (b < TN && k < K) ? fetch<T>(p.f, views[1], k * TN + b) : T(0);
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < KC; ++kk) {
          T av[MT], bv[MT];
#pragma unroll
          for (int i = 0; i < MT; ++i) {
            av[i] = sA[kk][ty + 16 * i];
            bv[i] = sB[kk][tx + 16 * i];
          }
#pragma unroll
          for (int i = 0; i < MT; ++i)
#pragma unroll
            for (int j = 0; j < MT; ++j)
              acc[i][j] += av[i] * bv[j];
        }
        __syncthreads();
      }

#pragma unroll
      for (int i = 0; i < MT; ++i) {
        const int a = m0 + ty + 16 * i;
        if (a >= TM)
          continue;
#pragma unroll
        for (int j = 0; j < MT; ++j) {
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

#define HC_MAPPED_KERNEL(name, T, MT)                                                   \
  extern "C" __global__ void __launch_bounds__(THREADS)                                 \
      name(const __grid_constant__ HcMappedGemmParams p) {                              \
    mappedGemm<T, MT>(p);                                                               \
  }

HC_MAPPED_KERNEL(hc_mapped_gemm_f32_t1, float, 1)
HC_MAPPED_KERNEL(hc_mapped_gemm_f32_t2, float, 2)
HC_MAPPED_KERNEL(hc_mapped_gemm_f32_t4, float, 4)
HC_MAPPED_KERNEL(hc_mapped_gemm_f64_t1, double, 1)
HC_MAPPED_KERNEL(hc_mapped_gemm_f64_t2, double, 2)
HC_MAPPED_KERNEL(hc_mapped_gemm_f64_t4, double, 4)
