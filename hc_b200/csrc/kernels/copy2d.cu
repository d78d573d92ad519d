// 2-D copy: dst[r, c] = src[r, c] for a rows x cols matrix of 1-, 2-, 4- or
// 8-byte elements, both sides row-major with their own row pitch.
//
// This is the one workload the reference's compiled GPU path can run itself:
// every work-group loads a (group_shape) tile and stores it back, clipped at
// the matrix edge (python/hckernel/tests/test_e2e.py:57-136; tile semantics in
// python/hckernel/kernel_api.py:297-342).  A tile-by-tile copy of a whole
// matrix is a plain strided copy, so the kernel works on bytes: rows are cut
// into 16-byte packets when both pitches and both bases allow it, otherwise
// into single elements.
#include <stdint.h>

namespace {

template <typename T>
__device__ __forceinline__ void copyRows(const char *src, char *dst,
                                         long long rows, long long perRow,
                                         long long srcPitch,
                                         long long dstPitch) {
  // One CTA walks rows; its threads walk the packets of a row.  blockIdx.y
  // strides over rows so that tall, narrow matrices still fill the GPU.
  for (long long r = blockIdx.y; r < rows; r += gridDim.y) {
    const T *s = reinterpret_cast<const T *>(src + r * srcPitch);
    T *d = reinterpret_cast<T *>(dst + r * dstPitch);
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x;
         i < perRow; i += (long long)gridDim.x * blockDim.x)
      d[i] = s[i];
  }
}

} // namespace

// rowBytes = cols * element size; pitches are in bytes.  `packet` is the
// widest power-of-two access (1..16 bytes) the host found legal for both sides.
extern "C" __global__ void __launch_bounds__(256)
    hc_copy2d(const char *src, char *dst, long long rows, long long rowBytes,
              long long srcPitch, long long dstPitch, int packet) {
  switch (packet) {
  case 16:
    copyRows<uint4>(src, dst, rows, rowBytes / 16, srcPitch, dstPitch);
    break;
  case 8:
    copyRows<uint2>(src, dst, rows, rowBytes / 8, srcPitch, dstPitch);
    break;
  case 4:
    copyRows<uint32_t>(src, dst, rows, rowBytes / 4, srcPitch, dstPitch);
    break;
  case 2:
    copyRows<uint16_t>(src, dst, rows, rowBytes / 2, srcPitch, dstPitch);
    break;
  default:
    copyRows<uint8_t>(src, dst, rows, rowBytes, srcPitch, dstPitch);
    break;
  }
}
