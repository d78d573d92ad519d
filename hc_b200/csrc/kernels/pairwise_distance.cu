// Pairwise Euclidean distance: out[i, j] = sqrt(sum_d (a[i, d] - b[j, d])^2),
// a [M, D], b [N, D], out [M, N], all row-major with explicit pitches.
//
// The reference's example kernel (python/hckernel/tests/test_examples.py:
// 261-301): a work-group loads an (m_block, D) tile of `a` and an (n_block, D)
// tile of `b`, forms the broadcast difference a[:, None, :] - b[None, :, :] and
// stores np.linalg.norm(diff, axis=2) into its (m_block, n_block) tile of the
// output.  Rows loaded past the end of either array are zero padding and the
// clipped store drops them (python/hckernel/kernel_api.py:297-342).
//
// The differences are formed explicitly, as the reference does (no
// |a|^2 + |b|^2 - 2ab rewriting, which would lose accuracy for close points).
// A CTA of 256 threads owns a 64 x 64 output tile and walks D in chunks of 16
// staged through shared memory; each thread accumulates a 4 x 4 block of
// squared distances.
#include <math.h>
#include <stdint.h>

namespace {

constexpr int PT = 64, PD = 16, PTHREADS = 256;

template <typename T>
__device__ __forceinline__ void
pairwiseTile(const T *__restrict__ a, const T *__restrict__ b,
             T *__restrict__ out, long long M, long long N, long long D,
             long long lda, long long ldb, long long ldo) {
  __shared__ T sA[PD][PT + 4]; // [d][row], transposed on the way in
  __shared__ T sB[PD][PT + 4];
  const int tid = threadIdx.x;
  const long long m0 = (long long)blockIdx.y * PT;
  const long long n0 = (long long)blockIdx.x * PT;
  const int row = tid >> 2, d4 = (tid & 3) << 2; // each thread stages 4 values of a and of b
  const int ty = tid >> 4, tx = tid & 15;

  T acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j)
      acc[i][j] = T(0);

  for (long long d0 = 0; d0 < D; d0 += PD) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const long long d = d0 + d4 + i;
      const long long gm = m0 + row, gn = n0 + row;
      sA[d4 + i][row] = (gm < M && d < D) ? a[gm * lda + d] : T(0);
      sB[d4 + i][row] = (gn < N && d < D) ? b[gn * ldb + d] : T(0);
    }
    __syncthreads();
#pragma unroll
    for (int d = 0; d < PD; ++d) {
      T av[4], bv[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        av[i] = sA[d][ty * 4 + i];
        bv[i] = sB[d][tx * 4 + i];
      }
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const T diff = av[i] - bv[j];
          acc[i][j] += diff * diff;
        }
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const long long gm = m0 + ty * 4 + i;
    if (gm >= M)
      continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const long long gn = n0 + tx * 4 + j;
      if (gn < N)
        out[gm * ldo + gn] = sqrt(acc[i][j]);
    }
  }
}

} // namespace

extern "C" __global__ void __launch_bounds__(PTHREADS)
    hc_pairwise_distance_f32(const float *a, const float *b, float *out,
                             long long M, long long N, long long D,
                             long long lda, long long ldb, long long ldo) {
  pairwiseTile<float>(a, b, out, M, N, D, lda, ldb, ldo);
}

extern "C" __global__ void __launch_bounds__(PTHREADS)
    hc_pairwise_distance_f64(const double *a, const double *b, double *out,
                             long long M, long long N, long long D,
                             long long lda, long long ldb, long long ldo) {
  pairwiseTile<double>(a, b, out, M, N, D, lda, ldb, ldo);
}
