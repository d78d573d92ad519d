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
#include "peer_params.h"

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
//
// PEERS: the result row is written to every destination of `peers` (row r at
// base[d] + r * yPitch) instead of `y` - the output all-gather of a multi-GPU run
// done by the kernel itself: every GPU writes its rows straight into the full
// output of every GPU, over NVLink for the others.
template <int V, bool PEERS = false>
__device__ __forceinline__ void
softmaxWarpRows(const float *__restrict__ x, float *__restrict__ y,
                long long rows, int cols, long long xPitch, long long yPitch,
                const HcPeerDsts *peers = nullptr) {
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
    if constexpr (PEERS) {
#pragma unroll
      for (int i = 0; i < V; ++i)
        v[i] = make_float4(v[i].x * inv, v[i].y * inv, v[i].z * inv, v[i].w * inv);
      for (int d = 0; d < peers->count; ++d) {
        float4 *out = reinterpret_cast<float4 *>(static_cast<float *>(peers->base[d]) +
                                                 r * yPitch);
#pragma unroll
        for (int i = 0; i < V; ++i) {
          int p = lane + 32 * i;
          if (p < packets)
            out[p] = v[i];
        }
      }
    } else {
#pragma unroll
      for (int i = 0; i < V; ++i) {
        int p = lane + 32 * i;
        if (p < packets)
          hc::storeStream(dst + p, make_float4(v[i].x * inv, v[i].y * inv,
                                               v[i].z * inv, v[i].w * inv));
      }
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

// The same kernels writing every row to all destinations of `peers`.
#define HC_SOFTMAX_WARP_PEERS(V, MINB)                                         \
  extern "C" __global__ void __launch_bounds__(128, MINB)                      \
      hc_softmax_rows_f32_w##V##_peers(const float *x, long long rows, int cols, \
                                       long long xPitch, long long yPitch,     \
                                       const __grid_constant__ HcPeerDsts peers) { \
    softmaxWarpRows<V, true>(x, nullptr, rows, cols, xPitch, yPitch, &peers);  \
  }

HC_SOFTMAX_WARP_PEERS(1, 8)
HC_SOFTMAX_WARP_PEERS(2, 8)
HC_SOFTMAX_WARP_PEERS(4, 8)
HC_SOFTMAX_WARP_PEERS(8, 8)
HC_SOFTMAX_WARP_PEERS(16, 5)
HC_SOFTMAX_WARP_PEERS(32, 3)

// ---- bulk-copy pipelined variant --------------------------------------------------
// One persistent CTA per SM: a producer thread streams whole rows into a ring
// of shared-memory slots with cp.async.bulk (completion counted on an mbarrier
// per slot), eight consumer warps each take a landed row into registers, free
// the slot at once, and then compute and store from registers.  Loads for the
// next dozen rows stay in flight while the current rows are exponentiated and
// written, which the register-only kernel above cannot do (a warp there has
// nothing in flight between its load burst and its store burst).
namespace {

constexpr int kTmaMaxSlots = 16;

struct TmaBarriers {
  uint64_t full[kTmaMaxSlots];
  uint64_t empty[kTmaMaxSlots];
  int abortFlag;
};

__device__ __forceinline__ void bulkLoad(uint32_t dst, const void *src,
                                         uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::"
               "bytes [%0], [%1], %2, [%3];" ::"r"(dst),
               "l"(src), "r"(bytes), "r"(bar)
               : "memory");
}

// Which slot, and which use of that slot, iteration i of a CTA maps to.  Rows
// are dealt to the C consumer warps round-robin and every warp owns `depth`
// slots of its own, so all uses of a slot are waited for by ONE warp, in
// order.  (With slots shared between warps a fast warp could wait for the
// second use of a slot before the first had landed; a parity wait cannot tell
// "not yet" from "already over", and the ring would come apart.)
template <int C>
__device__ __forceinline__ void slotOf(long long i, int depth, int &slot,
                                       uint32_t &phase) {
  const long long turn = i / C; // how many rows this warp has taken before
  slot = int(i % C) + C * int(turn % depth);
  phase = uint32_t(turn / depth) & 1u;
}

// `cols` is a multiple of 4 and at most 128 * V; pitches are multiples of 4
// elements and the bases 16-byte aligned, so every row is a legal bulk copy.
// C * depth rows of `slotBytes` each fit in the dynamic shared memory.
template <int V, int C>
__device__ __forceinline__ void
softmaxTmaRows(const float *__restrict__ x, float *__restrict__ y,
               long long rows, int cols, long long xPitch, long long yPitch,
               int depth, int slotBytes, int *status, unsigned char *smemRaw) {
  const uint32_t ring = (hc::smemAddr(smemRaw) + 127u) & ~127u;
  unsigned char *ringPtr = smemRaw + (ring - hc::smemAddr(smemRaw));
  const int slots = C * depth;
  TmaBarriers *bars =
      reinterpret_cast<TmaBarriers *>(ringPtr + (size_t)slots * slotBytes);
  volatile int *abortFlag = &bars->abortFlag;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < slots; ++s) {
      hc::mbarInit(hc::smemAddr(&bars->full[s]), 1);
      hc::mbarInit(hc::smemAddr(&bars->empty[s]), 1);
    }
    bars->abortFlag = 0;
    hc::fenceBarrierInit();
  }
  __syncthreads();

  // Row of iteration i for this CTA: blockIdx.x + i * gridDim.x.
  const long long myRows =
      rows > blockIdx.x ? (rows - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;
  const uint32_t rowBytes = uint32_t(cols) * 4u;

  if (warp == 0) {
    if (lane == 0) {
      for (long long i = 0; i < myRows; ++i) {
        int s;
        uint32_t phase;
        slotOf<C>(i, depth, s, phase);
        if (!hc::mbarWait(hc::smemAddr(&bars->empty[s]), phase ^ 1u, abortFlag,
                          status, hc::kStatusProducerWait))
          break;
        const long long r = blockIdx.x + i * (long long)gridDim.x;
        const uint32_t bar = hc::smemAddr(&bars->full[s]);
        hc::mbarExpectTx(bar, rowBytes);
        bulkLoad(ring + uint32_t(s) * uint32_t(slotBytes), x + r * xPitch,
                 rowBytes, bar);
      }
      if (*abortFlag) { // copies may still be landing: give them time
        const unsigned long long t0 = hc::globalTimerNs();
        while (hc::globalTimerNs() - t0 < 1000000ull) {
        }
      }
    }
  } else {
    const int cw = warp - 1;
    const int packets = cols >> 2;
    for (long long i = cw; i < myRows; i += C) {
      int s;
      uint32_t phase;
      slotOf<C>(i, depth, s, phase);
      bool ok = true;
      if (lane == 0)
        ok = hc::mbarWait(hc::smemAddr(&bars->full[s]), phase, abortFlag, status,
                          hc::kStatusEpilogueWait);
      ok = __shfl_sync(0xffffffffu, ok, 0);
      if (!ok)
        break;
      const float4 *src =
          reinterpret_cast<const float4 *>(ringPtr + (size_t)s * slotBytes);
      float4 v[V];
#pragma unroll
      for (int j = 0; j < V; ++j) {
        const int p = lane + 32 * j;
        v[j] = p < packets
                   ? src[p]
                   : make_float4(-INFINITY, -INFINITY, -INFINITY, -INFINITY);
      }
      // The row is in registers: hand the slot back before computing.
      __syncwarp();
      if (lane == 0)
        hc::mbarArrive(hc::smemAddr(&bars->empty[s]));

      float m = -INFINITY;
#pragma unroll
      for (int j = 0; j < V; ++j)
        m = hc::maxNan(hc::maxNan(hc::maxNan(v[j].x, v[j].y),
                                  hc::maxNan(v[j].z, v[j].w)),
                       m);
      m = warpMax(m);
      const float shift = (m == -INFINITY) ? 0.f : m * kLog2e;
      float s0 = 0.f, s1 = 0.f;
#pragma unroll
      for (int j = 0; j < V; ++j) {
        v[j].x = fastExp2(fmaf(v[j].x, kLog2e, -shift));
        v[j].y = fastExp2(fmaf(v[j].y, kLog2e, -shift));
        v[j].z = fastExp2(fmaf(v[j].z, kLog2e, -shift));
        v[j].w = fastExp2(fmaf(v[j].w, kLog2e, -shift));
        s0 += v[j].x + v[j].z;
        s1 += v[j].y + v[j].w;
      }
      const float inv = 1.0f / warpSum(s0 + s1);
      const long long r = blockIdx.x + i * (long long)gridDim.x;
      float4 *dst = reinterpret_cast<float4 *>(y + r * yPitch);
#pragma unroll
      for (int j = 0; j < V; ++j) {
        const int p = lane + 32 * j;
        if (p < packets)
          hc::storeStream(dst + p, make_float4(v[j].x * inv, v[j].y * inv,
                                               v[j].z * inv, v[j].w * inv));
      }
    }
  }
  // Nobody leaves while a bulk copy could still target this CTA's memory: the
  // consumers have waited for every copy they used, and after an abort the
  // producer has waited above.
  __syncthreads();
}

} // namespace

// V float4 per lane, C consumer warps (+ 1 producer warp).
#define HC_SOFTMAX_TMA(V, C)                                                   \
  extern "C" __global__ void __launch_bounds__(32 * (C + 1), 1)                \
      hc_softmax_rows_f32_tma_v##V(const float *x, float *y, long long rows,   \
                                   int cols, long long xPitch,                 \
                                   long long yPitch, int depth, int slotBytes, \
                                   int *status) {                              \
    extern __shared__ __align__(128) unsigned char tmaSmem[];                  \
    softmaxTmaRows<V, C>(x, y, rows, cols, xPitch, yPitch, depth, slotBytes,   \
                         status, tmaSmem);                                     \
  }

HC_SOFTMAX_TMA(16, 8)
HC_SOFTMAX_TMA(32, 6)

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
