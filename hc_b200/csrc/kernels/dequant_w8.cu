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
// Each thread owns one 16-weight packet column and walks the rows four at a
// time, so four independent 16-byte loads are in flight before the eight
// 16-byte stores they turn into.
#include <cuda_bf16.h>
#include <stdint.h>

namespace {

__device__ __forceinline__ int4 loadStream16(const int4 *p) {
  int4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.s32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}

// Two int8 (bytes `sel` picks out of `word`) -> two bf16, without the
// int-to-float conversion unit.  Writing a byte x under the exponent byte 0x43
// gives the bf16 pattern 0x43xx; with bit 7 masked off that is the number
// 128 + (x & 0x7f), exactly.  In two's complement x = (x & 0x7f) - 128 * sign,
// so the value is (128 + (x & 0x7f)) - 128 for x >= 0 and - 256 for x < 0; and
// 128.0 = 0x4300, 256.0 = 0x4380 differ in exactly the bit where the sign of x
// sits in 0x43xx.  One byte permute, two masks and one packed subtract per pair;
// every intermediate fits bf16's 8 significant bits, so the result is exact.
__device__ __forceinline__ uint32_t int8PairToBf16(uint32_t word, uint32_t sel) {
  const uint32_t t = __byte_perm(word, 0x43434343u, sel);
  const uint32_t biased = t & 0xFF7FFF7Fu;
  const uint32_t bias = t & 0xFF80FF80u;
  const __nv_bfloat162 d = __hsub2(*reinterpret_cast<const __nv_bfloat162 *>(&biased),
                                   *reinterpret_cast<const __nv_bfloat162 *>(&bias));
  return *reinterpret_cast<const uint32_t *>(&d);
}

__device__ __forceinline__ void convertAndStore(int4 q, uint4 *dst) {
  const int words[4] = {q.x, q.y, q.z, q.w};
  uint32_t o[8];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const uint32_t x = uint32_t(words[i]);
    o[2 * i] = int8PairToBf16(x, 0x5140u);     // bytes 0 and 1
    o[2 * i + 1] = int8PairToBf16(x, 0x7362u); // bytes 2 and 3
  }
  dst[0] = make_uint4(o[0], o[1], o[2], o[3]);
  dst[1] = make_uint4(o[4], o[5], o[6], o[7]);
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
    constexpr int R = 4;                 // rows in flight per thread
    const long long packets = cols >> 4; // 16 weights per packet
    // blockIdx.y picks a band of R adjacent rows; bands stride by gridDim.y.
    for (long long p = blockIdx.x * (long long)blockDim.x + threadIdx.x;
         p < packets; p += (long long)gridDim.x * blockDim.x) {
      for (long long r = (long long)blockIdx.y * R; r < rows;
           r += (long long)gridDim.y * R) {
        if (r + R <= rows) {
          int4 q[R];
#pragma unroll
          for (int i = 0; i < R; ++i)
            q[i] = loadStream16(
                reinterpret_cast<const int4 *>(w + (r + i) * wPitch) + p);
#pragma unroll
          for (int i = 0; i < R; ++i)
            convertAndStore(q[i], reinterpret_cast<uint4 *>(
                                      out + (r + i) * outPitch) +
                                      2 * p);
        } else {
          for (long long t = r; t < rows; ++t)
            convertAndStore(
                loadStream16(reinterpret_cast<const int4 *>(w + t * wPitch) + p),
                reinterpret_cast<uint4 *>(out + t * outPitch) + 2 * p);
        }
      }
    }
  } else {
    for (long long r = blockIdx.y; r < rows; r += gridDim.y)
      for (long long c = blockIdx.x * (long long)blockDim.x + threadIdx.x;
           c < cols; c += (long long)gridDim.x * blockDim.x)
        out[r * outPitch + c] = __float2bfloat16_rn(float(w[r * wPitch + c]));
  }
}
