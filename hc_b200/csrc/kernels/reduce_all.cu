// Whole-array sum into one element: result[0] += sum(a[0:n]).
//
// The reference's scalar reduction kernels (python/hckernel/tests/
// test_examples.py:31-71): every work-group loads its slice of `a`, zero-
// padded past the end (python/hckernel/kernel_api.py:297-316), sums it and
// adds the partial sum to `result[0]` through `atomic_ref`, which is the
// identity on the simulator (kernel_api.py:450-451) and a real atomic here.
// `result` is NOT cleared: like the reference, the kernel adds to whatever
// the caller put there.
//
// Each thread accumulates a strided share of the array, a CTA combines its
// threads with shuffles and shared memory, and one thread per CTA issues a
// single atomicAdd, so the number of atomics is the grid size (a few hundred),
// not the element count.  The partial sums are kept in the wider of the input
// and the result type - double for float64 and integer inputs whatever the
// result, as the reference sums a group's slice in the input dtype and only
// the per-group partial sum meets the (possibly float32) result - and are
// converted to the result type for the atomicAdd alone.  Floating-point
// partial sums are combined in an order that depends on CTA scheduling;
// integer inputs summed in float64 are exact as long as the total is below
// 2^53.
#include <stdint.h>

namespace {

template <typename TIn, typename TOut> struct Wide { using type = double; };
template <> struct Wide<float, float> { using type = float; };

template <typename TIn, typename TOut>
__device__ __forceinline__ void reduceAll(const TIn *__restrict__ a, long long n,
                                          TOut *result) {
  using TAcc = typename Wide<TIn, TOut>::type;
  TAcc acc = TAcc(0);
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += stride)
    acc += TAcc(a[i]);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1)
    acc += __shfl_xor_sync(0xffffffffu, acc, o);
  __shared__ TAcc partial[32];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0)
    partial[warp] = acc;
  __syncthreads();
  if (warp == 0) {
    acc = lane < (blockDim.x >> 5) ? partial[lane] : TAcc(0);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1)
      acc += __shfl_xor_sync(0xffffffffu, acc, o);
    if (lane == 0)
      atomicAdd(result, TOut(acc));
  }
}

} // namespace

#define HC_REDUCE_ALL(NAME, TIN, TACC)                                         \
  extern "C" __global__ void __launch_bounds__(256)                            \
      hc_reduce_all_##NAME(const TIN *a, long long n, TACC *result) {          \
    reduceAll<TIN, TACC>(a, n, result);                                        \
  }

HC_REDUCE_ALL(f32_f32, float, float)
HC_REDUCE_ALL(f32_f64, float, double)
HC_REDUCE_ALL(f64_f64, double, double)
HC_REDUCE_ALL(f64_f32, double, float)
HC_REDUCE_ALL(i32_f32, int32_t, float)
HC_REDUCE_ALL(i32_f64, int32_t, double)
HC_REDUCE_ALL(i64_f32, long long, float)
HC_REDUCE_ALL(i64_f64, long long, double)
