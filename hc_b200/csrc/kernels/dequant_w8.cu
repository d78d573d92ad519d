// int8 -> bf16 conversion of a weight matrix: out[k, n] = bf16(w[k, n]).
//
// First half of the weight-only dequant GEMM out = bf16(s[n] * sum_k a[m, k] *
// float(w[k, n])).  Every int8 value is exactly representable in bf16 and the
// per-output-channel scale factors out of the K-sum, so the weights are
// converted once, unscaled, into a bf16 scratch matrix and the scale is
// applied to the fp32 accumulator in the GEMM epilogue.  Converting once costs
// K*N conversions; converting inside the GEMM main loop would repeat them for
// every 128- or 256-row block of activations.
//
// The kernel is a pure stream: 1 byte read and 2 bytes written per element.
#include <cuda_bf16.h>
#include <stdint.h>

namespace {

__device__ __forceinline__ uint32_t pairToBf16(int lo, int hi) {
  __nv_bfloat162 h = __floats2bfloat162_rn(float(lo), float(hi));
  return *reinterpret_cast<uint32_t *>(&h);
}

} // namespace

// `vec` != 0 promises: w and out 16-byte aligned, cols and both pitches
// multiples of 16 elements.  Pitches are in elements.
extern "C" __global__ void __launch_bounds__(256)
    hc_dequant_w8_bf16(const int8_t *__restrict__ w,
                       __nv_bfloat16 *__restrict__ out, long long rows,
                       long long cols, long long wPitch, long long outPitch,
                       int vec) {
  if (vec) {
    const long long packets = cols >> 4; // 16 weights per packet
    for (long long r = blockIdx.y; r < rows; r += gridDim.y) {
      const int4 *src = reinterpret_cast<const int4 *>(w + r * wPitch);
      uint4 *dst = reinterpret_cast<uint4 *>(out + r * outPitch);
      for (long long p = blockIdx.x * (long long)blockDim.x + threadIdx.x;
           p < packets; p += (long long)gridDim.x * blockDim.x) {
        const int4 q = __ldg(src + p);
        const int words[4] = {q.x, q.y, q.z, q.w};
        uint32_t o[8];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int x = words[i];
          o[2 * i] = pairToBf16(int(int8_t(x)), int(int8_t(x >> 8)));
          o[2 * i + 1] = pairToBf16(int(int8_t(x >> 16)), int(int8_t(x >> 24)));
        }
        dst[2 * p] = make_uint4(o[0], o[1], o[2], o[3]);
        dst[2 * p + 1] = make_uint4(o[4], o[5], o[6], o[7]);
      }
    }
  } else {
    for (long long r = blockIdx.y; r < rows; r += gridDim.y)
      for (long long c = blockIdx.x * (long long)blockDim.x + threadIdx.x;
           c < cols; c += (long long)gridDim.x * blockDim.x)
        out[r * outPitch + c] = __float2bfloat16_rn(float(w[r * wPitch + c]));
  }
}
