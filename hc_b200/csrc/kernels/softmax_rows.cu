// Row softmax over the last axis: y[r, :] = exp(x[r, :] - max(x[r, :])) /
// sum(exp(x[r, :] - max(x[r, :]))).
//
// Follows the reference kernel body (python/hckernel/tests/test_examples.py:
// 312-321): each work-group loads whole rows, subtracts the row maximum,
// exponentiates, and divides by the row sum.  Rows are independent, so the
// group shape of the reference (how many rows a group takes) has no effect on
// the result and is not a parameter here.
//
// Two kernels:
//   hc_softmax_rows_f32_w<V>  one warp per row, the row lives in registers
//       (V float4 per lane, so up to 128*V columns); x is read once with
//       16-byte streaming loads and y written once with 16-byte stores.  This
//       is the HBM-bound path: 8 bytes of traffic per element and nothing else.
//   hc_softmax_rows_generic_{f32,f64}  one CTA per row, any column count,
//       pitch or alignment; the row is cached in shared memory when it fits
//       and re-read otherwise.
#include "hc_ptx.cuh"

#include <float.h>
#include <math.h>

namespace {

constexpr float kLog2e = 1.4426950408889634f;

__device__ __forceinline__ float warpMax(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1)
    v = hc::maxNan(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

template <typename T> __device__ __forceinline__ T warpSum(T v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1)
    v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

__device__ __forceinline__ float fastExp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// One warp per row.  `cols` is a multiple of 4 and at most 128 * V; both row
// pitches are multiples of 4 elements and both bases 16-byte aligned (the
// host dispatcher guarantees all of it).
template <int V>
__device__ __forceinline__ void
softmaxWarpRows(const float *__restrict__ x, float *__restrict__ y,
                long long rows, int cols, long long xPitch, long long yPitch) {
  const int lane = threadIdx.x & 31;
  const long long warpsPerGrid = (long long)gridDim.x * (blockDim.x >> 5);
  const long long firstRow =
      (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int packets = cols >> 2; // float4 per row

  for (long long r = firstRow; r < rows; r += warpsPerGrid) {
    const float4 *src = reinterpret_cast<const float4 *>(x + r * xPitch);
    float4 *dst = reinterpret_cast<float4 *>(y + r * yPitch);
    float4 v[V];
    // Lanes past the end of the row hold -inf: neutral for max, and
    // exp(-inf - m) = 0 is neutral for the sum.
#pragma unroll
    for (int i = 0; i < V; ++i) {
      int p = lane + 32 * i;
      if (p < packets)
        v[i] = hc::loadStream(src + p);
      else
        v[i] = make_float4(-INFINITY, -INFINITY, -INFINITY, -INFINITY);
    }
    float m = -INFINITY;
#pragma unroll
    for (int i = 0; i < V; ++i)
      m = hc::maxNan(hc::maxNan(hc::maxNan(v[i].x, v[i].y),
                                hc::maxNan(v[i].z, v[i].w)),
                     m);
    m = warpMax(m);
    // A row of -inf only (or an empty tail) must not produce inf - inf.
    const float shift = (m == -INFINITY) ? 0.f : m * kLog2e;
    float s0 = 0.f, s1 = 0.f;
#pragma unroll
    for (int i = 0; i < V; ++i) {
      v[i].x = fastExp2(fmaf(v[i].x, kLog2e, -shift));
      v[i].y = fastExp2(fmaf(v[i].y, kLog2e, -shift));
      v[i].z = fastExp2(fmaf(v[i].z, kLog2e, -shift));
      v[i].w = fastExp2(fmaf(v[i].w, kLog2e, -shift));
      s0 += v[i].x + v[i].z;
      s1 += v[i].y + v[i].w;
    }
    const float inv = 1.0f / warpSum(s0 + s1);
#pragma unroll
    for (int i = 0; i < V; ++i) {
      int p = lane + 32 * i;
      if (p < packets)
        hc::storeStream(dst + p, make_float4(v[i].x * inv, v[i].y * inv,
                                             v[i].z * inv, v[i].w * inv));
    }
  }
}

template <typename T> struct Limits;
template <> struct Limits<float> {
  static __device__ float lowest() { return -INFINITY; }
};
template <> struct Limits<double> {
  static __device__ double lowest() { return -(double)INFINITY; }
};

__device__ __forceinline__ float expOf(float v) { return expf(v); }
__device__ __forceinline__ double expOf(double v) { return exp(v); }

// Block-wide reduction through shared memory; every thread gets the result.
template <typename T, typename Op>
__device__ __forceinline__ T blockReduce(T v, T *scratch, Op op) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1)
    v = op(v, __shfl_xor_sync(0xffffffffu, v, o));
  __syncthreads(); // scratch may still be read from the previous reduction
  if (lane == 0)
    scratch[warp] = v;
  __syncthreads();
  T total = scratch[0];
  for (int w = 1; w < (blockDim.x >> 5); ++w)
    total = op(total, scratch[w]);
  return total;
}

template <typename T>
__device__ __forceinline__ void
softmaxBlockRows(const T *__restrict__ x, T *__restrict__ y, long long rows,
                 long long cols, long long xPitch, long long yPitch,
                 long long cacheElems, T *cache, T *scratch) {
  const bool cached = cols <= cacheElems;
  for (long long r = blockIdx.x; r < rows; r += gridDim.x) {
    const T *src = x + r * xPitch;
    T *dst = y + r * yPitch;
    T m = Limits<T>::lowest();
    for (long long c = threadIdx.x; c < cols; c += blockDim.x) {
      T v = src[c];
      if (cached)
        cache[c] = v;
      m = hc::maxNan(m, v);
    }
    m = blockReduce(m, scratch, [](T a, T b) { return hc::maxNan(a, b); });
    if (m == Limits<T>::lowest())
      m = T(0);
    T s = T(0);
    for (long long c = threadIdx.x; c < cols; c += blockDim.x) {
      T e = expOf((cached ? cache[c] : src[c]) - m);
      if (cached)
        cache[c] = e;
      s += e;
    }
    s = blockReduce(s, scratch, [](T a, T b) { return a + b; });
    for (long long c = threadIdx.x; c < cols; c += blockDim.x) {
      T e = cached ? cache[c] : expOf(src[c] - m);
      dst[c] = e / s;
    }
    __syncthreads(); // the cache is reused by the next row
  }
}

} // namespace

#define HC_SOFTMAX_WARP(V, MINB)                                               \
  extern "C" __global__ void __launch_bounds__(128, MINB)                      \
      hc_softmax_rows_f32_w##V(const float *x, float *y, long long rows,       \
                               int cols, long long xPitch, long long yPitch) { \
    softmaxWarpRows<V>(x, y, rows, cols, xPitch, yPitch);                      \
  }

HC_SOFTMAX_WARP(1, 8)
HC_SOFTMAX_WARP(2, 8)
HC_SOFTMAX_WARP(4, 8)
HC_SOFTMAX_WARP(8, 8)
HC_SOFTMAX_WARP(16, 5)
HC_SOFTMAX_WARP(32, 3)

extern "C" __global__ void __launch_bounds__(256)
    hc_softmax_rows_generic_f32(const float *x, float *y, long long rows,
                                long long cols, long long xPitch,
                                long long yPitch, long long cacheElems) {
  extern __shared__ __align__(16) unsigned char dynSmem[];
  __shared__ float scratch[32];
  softmaxBlockRows<float>(x, y, rows, cols, xPitch, yPitch, cacheElems,
                          reinterpret_cast<float *>(dynSmem), scratch);
}

extern "C" __global__ void __launch_bounds__(256)
    hc_softmax_rows_generic_f64(const double *x, double *y, long long rows,
                                long long cols, long long xPitch,
                                long long yPitch, long long cacheElems) {
  extern __shared__ __align__(16) unsigned char dynSmem[];
  __shared__ double scratch[32];
  softmaxBlockRows<double>(x, y, rows, cols, xPitch, yPitch, cacheElems,
                           reinterpret_cast<double *>(dynSmem), scratch);
}
