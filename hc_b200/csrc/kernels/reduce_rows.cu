// Last-axis reductions: sum[r] = sum_c x[r, c] and max[r] = max_c x[r, c], in
// one pass over x (either output may be absent).
//
// The reference expresses reductions as `tile.sum()` / `tile.max()` on a
// loaded tile (python/hckernel/tests/test_examples.py:36-40,55-64 for the sum;
// the masked-array reductions come from python/hckernel/kernel_api.py:150-151).
// The last-axis form loads whole rows per work-group and stores one value per
// row, so rows are independent and the group shape does not affect results.
//
// max is exact (and propagates NaN like numpy's max); the sum is accumulated
// in the element type, in 128 (warp kernel) or 1024 (block kernel) interleaved
// partial sums per row that are then combined as a tree.
//
// x is read exactly once with 16-byte streaming loads when the layout allows
// it (`vec` != 0: base 16-byte aligned, cols and pitch multiples of 4 floats);
// the outputs are 4 or 8 bytes per row, so the kernel moves
// rows*cols*sizeof(T) bytes and is HBM-bound.
#include "hc_ptx.cuh"
#include "peer_params.h"

#include <math.h>

namespace {

template <typename T> struct Acc {
  T sum;
  T max;
};

template <typename T> __device__ __forceinline__ T lowest();
template <> __device__ __forceinline__ float lowest<float>() {
  return -INFINITY;
}
template <> __device__ __forceinline__ double lowest<double>() {
  return -(double)INFINITY;
}

template <typename T>
__device__ __forceinline__ Acc<T> warpCombine(Acc<T> a) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    a.sum += __shfl_xor_sync(0xffffffffu, a.sum, o);
    a.max = hc::maxNan(a.max, __shfl_xor_sync(0xffffffffu, a.max, o));
  }
  return a;
}

// Partial reduction of one row by `nThreads` cooperating threads, of which
// this thread is number `tid`.
template <int UNROLL>
__device__ __forceinline__ Acc<float> rowPartialVec(const float *row,
                                                    long long cols, int tid,
                                                    int nThreads) {
  const float4 *src = reinterpret_cast<const float4 *>(row);
  const long long packets = cols >> 2;
  float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
  float m0 = -INFINITY, m1 = -INFINITY;
  long long p = tid;
  const long long step = (long long)nThreads * UNROLL;
  // Full batches: UNROLL independent 16-byte loads in flight per thread.
  for (; p + (long long)nThreads * (UNROLL - 1) < packets; p += step) {
    float4 v[UNROLL];
#pragma unroll
    for (int u = 0; u < UNROLL; ++u)
      v[u] = hc::loadStream(src + p + (long long)u * nThreads);
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      s0 += v[u].x;
      s1 += v[u].y;
      s2 += v[u].z;
      s3 += v[u].w;
      m0 = hc::maxNan(m0, hc::maxNan(v[u].x, v[u].y));
      m1 = hc::maxNan(m1, hc::maxNan(v[u].z, v[u].w));
    }
  }
  for (; p < packets; p += nThreads) {
    float4 v = hc::loadStream(src + p);
    s0 += v.x;
    s1 += v.y;
    s2 += v.z;
    s3 += v.w;
    m0 = hc::maxNan(m0, hc::maxNan(v.x, v.y));
    m1 = hc::maxNan(m1, hc::maxNan(v.z, v.w));
  }
  return {(s0 + s2) + (s1 + s3), hc::maxNan(m0, m1)};
}

template <typename T>
__device__ __forceinline__ Acc<T> rowPartialScalar(const T *row, long long cols,
                                                   int tid, int nThreads) {
  T s = T(0), m = lowest<T>();
  for (long long c = tid; c < cols; c += nThreads) {
    T v = row[c];
    s += v;
    m = hc::maxNan(m, v);
  }
  return {s, m};
}

template <typename T>
__device__ __forceinline__ Acc<T> rowPartial(const T *row, long long cols,
                                             int tid, int nThreads, int vec) {
  if constexpr (sizeof(T) == 4) {
    if (vec)
      return rowPartialVec<8>(row, cols, tid, nThreads);
  }
  return rowPartialScalar<T>(row, cols, tid, nThreads);
}

// One warp per row.
template <typename T>
__device__ __forceinline__ void
reduceWarpRows(const T *__restrict__ x, T *__restrict__ sumOut,
               T *__restrict__ maxOut, long long rows, long long cols,
               long long pitch, int vec) {
  const int lane = threadIdx.x & 31;
  const long long warpsPerGrid = (long long)gridDim.x * (blockDim.x >> 5);
  for (long long r = (long long)blockIdx.x * (blockDim.x >> 5) +
                     (threadIdx.x >> 5);
       r < rows; r += warpsPerGrid) {
    Acc<T> a = warpCombine(rowPartial<T>(x + r * pitch, cols, lane, 32, vec));
    if (lane == 0) {
      if (sumOut)
        sumOut[r] = a.sum;
      if (maxOut)
        maxOut[r] = a.max;
    }
  }
}

// One CTA per row, for matrices with few, long rows.
template <typename T>
__device__ __forceinline__ void
reduceBlockRows(const T *__restrict__ x, T *__restrict__ sumOut,
                T *__restrict__ maxOut, long long rows, long long cols,
                long long pitch, int vec, Acc<T> *scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nWarps = blockDim.x >> 5;
  for (long long r = blockIdx.x; r < rows; r += gridDim.x) {
    Acc<T> a = warpCombine(
        rowPartial<T>(x + r * pitch, cols, threadIdx.x, blockDim.x, vec));
    if (lane == 0)
      scratch[warp] = a;
    __syncthreads();
    if (warp == 0) {
      Acc<T> b = lane < nWarps ? scratch[lane] : Acc<T>{T(0), lowest<T>()};
      b = warpCombine(b);
      if (lane == 0) {
        if (sumOut)
          sumOut[r] = b.sum;
        if (maxOut)
          maxOut[r] = b.max;
      }
    }
    __syncthreads();
  }
}

// One warp per row, the two results of a row written to every destination of
// `peers`: base[d] holds the sums of this kernel's rows, followed `maxOffset`
// elements later by their maxima (the output all-gather of a multi-GPU run done
// by the kernel itself).
template <typename T>
__device__ __forceinline__ void reduceWarpRowsPeers(const T *__restrict__ x, long long rows,
                                                    long long cols, long long pitch, int vec,
                                                    long long maxOffset,
                                                    const HcPeerDsts &peers) {
  const int lane = threadIdx.x & 31;
  const long long warpsPerGrid = (long long)gridDim.x * (blockDim.x >> 5);
  for (long long r = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); r < rows;
       r += warpsPerGrid) {
    Acc<T> a = warpCombine(rowPartial<T>(x + r * pitch, cols, lane, 32, vec));
    // Lane d writes destination d.
    if (lane < peers.count) {
      T *out = static_cast<T *>(peers.base[lane]);
      out[r] = a.sum;
      out[maxOffset + r] = a.max;
    }
  }
}

} // namespace

extern "C" __global__ void __launch_bounds__(256)
    hc_reduce_rows_warp_f32_peers(const float *x, long long rows, long long cols,
                                  long long pitch, int vec, long long maxOffset,
                                  const __grid_constant__ HcPeerDsts peers) {
  reduceWarpRowsPeers<float>(x, rows, cols, pitch, vec, maxOffset, peers);
}

extern "C" __global__ void __launch_bounds__(256)
    hc_reduce_rows_warp_f32(const float *x, float *sumOut, float *maxOut,
                            long long rows, long long cols, long long pitch,
                            int vec) {
  reduceWarpRows<float>(x, sumOut, maxOut, rows, cols, pitch, vec);
}

extern "C" __global__ void __launch_bounds__(256)
    hc_reduce_rows_warp_f64(const double *x, double *sumOut, double *maxOut,
                            long long rows, long long cols, long long pitch,
                            int vec) {
  reduceWarpRows<double>(x, sumOut, maxOut, rows, cols, pitch, vec);
}

extern "C" __global__ void __launch_bounds__(256)
    hc_reduce_rows_block_f32(const float *x, float *sumOut, float *maxOut,
                             long long rows, long long cols, long long pitch,
                             int vec) {
  __shared__ Acc<float> scratch[32];
  reduceBlockRows<float>(x, sumOut, maxOut, rows, cols, pitch, vec, scratch);
}

extern "C" __global__ void __launch_bounds__(256)
    hc_reduce_rows_block_f64(const double *x, double *sumOut, double *maxOut,
                             long long rows, long long cols, long long pitch,
                             int vec) {
  __shared__ Acc<double> scratch[32];
  reduceBlockRows<double>(x, sumOut, maxOut, rows, cols, pitch, vec, scratch);
}
