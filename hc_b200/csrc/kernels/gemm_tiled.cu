// Tiled GEMM on the CUDA cores: C[M, N] = A[M, K] @ B[K, N] (* scale[N]), all
// row-major with explicit row pitches, any M, N, K.
//
// This is the reference's K-blocked dot kernel (python/hckernel/tests/
// test_examples.py:88-111): a 2-D grid of work-groups, each owning an
// (m_block x n_block) tile of the output, walks K in blocks of KB, loads the
// A and B tiles (zero-filled past the matrix edge, python/hckernel/
// kernel_api.py:297-316), accumulates their product and finally stores the
// tile clipped to the matrix (kernel_api.py:318-342).  Here a work-group is a
// CTA of 256 threads that owns a 64 x 64 tile and walks K in blocks of 16 -
// the group shape and KB of the reference's fp32 benchmark case - with a 4 x 4
// register tile per thread, fp32 (or fp64) FMA accumulation, and the next
// K-block prefetched into registers while the current one is multiplied.
//
// The same template also serves as the any-shape fallback of the tensor-core
// kernels: bf16 inputs with fp32 accumulation and bf16 output, and bf16 x int8
// with a per-output-column fp32 scale applied to the accumulator before
// rounding (the weight-only dequant GEMM).
#include <cooperative_groups.h>
#include <cuda_bf16.h>
#include <stdint.h>

namespace cg = cooperative_groups;

namespace {

constexpr int TM = 64, TN = 64, TK = 16, THREADS = 256;

template <typename T> struct Conv;
template <> struct Conv<float> {
  static __device__ __forceinline__ float load(float v) { return v; }
  static __device__ __forceinline__ float store(float v) { return v; }
};
template <> struct Conv<double> {
  static __device__ __forceinline__ double load(double v) { return v; }
  static __device__ __forceinline__ double store(double v) { return v; }
};
template <> struct Conv<__nv_bfloat16> {
  static __device__ __forceinline__ float load(__nv_bfloat16 v) {
    return __bfloat162float(v);
  }
  static __device__ __forceinline__ __nv_bfloat16 store(float v) {
    return __float2bfloat16_rn(v);
  }
};
template <> struct Conv<int8_t> {
  static __device__ __forceinline__ float load(int8_t v) { return float(v); }
};

template <typename TA, typename TB, typename TC, typename TAcc>
__device__ __forceinline__ void
gemmTile(const TA *__restrict__ a, const TB *__restrict__ b,
         TC *__restrict__ c, const float *__restrict__ scale, long long M,
         long long N, long long K, long long lda, long long ldb,
         long long ldc) {
  // +4 padding keeps the transposed A stores and the row reads conflict-free.
  __shared__ TAcc sA[2][TK][TM + 4];
  __shared__ TAcc sB[2][TK][TN + 4];

  const int tid = threadIdx.x;
  const long long m0 = (long long)blockIdx.y * TM;
  const long long n0 = (long long)blockIdx.x * TN;

  // Global -> register staging: each thread moves 4 elements of A and of B.
  const int aRow = tid >> 2, aCol = (tid & 3) << 2; // A tile is 64 x 16
  const int bRow = tid >> 4, bCol = (tid & 15) << 2; // B tile is 16 x 64
  TAcc ra[4], rb[4];

  auto fetch = [&](long long k0) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      long long gm = m0 + aRow, gk = k0 + aCol + i;
      ra[i] = (gm < M && gk < K) ? TAcc(Conv<TA>::load(a[gm * lda + gk]))
                                 : TAcc(0);
      long long gkb = k0 + bRow, gn = n0 + bCol + i;
      rb[i] = (gkb < K && gn < N) ? TAcc(Conv<TB>::load(b[gkb * ldb + gn]))
                                  : TAcc(0);
    }
  };
  auto stash = [&](int buf) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      sA[buf][aCol + i][aRow] = ra[i];
      sB[buf][bRow][bCol + i] = rb[i];
    }
  };

  const int ty = tid >> 4, tx = tid & 15; // 16 x 16 threads, 4 x 4 outputs each
  TAcc acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j)
      acc[i][j] = TAcc(0);

  const long long kBlocks = (K + TK - 1) / TK;
  if (kBlocks > 0) {
    fetch(0);
    stash(0);
  }
  __syncthreads();
  for (long long kb = 0; kb < kBlocks; ++kb) {
    const int cur = kb & 1;
    if (kb + 1 < kBlocks)
      fetch((kb + 1) * TK);
#pragma unroll
    for (int k = 0; k < TK; ++k) {
      TAcc av[4], bv[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        av[i] = sA[cur][k][ty * 4 + i];
        bv[i] = sB[cur][k][tx * 4 + i];
      }
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j)
          acc[i][j] += av[i] * bv[j];
    }
    if (kb + 1 < kBlocks)
      stash(cur ^ 1);
    __syncthreads();
  }

#pragma unroll
  for (int i = 0; i < 4; ++i) {
    long long gm = m0 + ty * 4 + i;
    if (gm >= M)
      continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      long long gn = n0 + tx * 4 + j;
      if (gn >= N)
        continue;
      TAcc v = acc[i][j];
      if (scale)
        v *= TAcc(scale[gn]);
      c[gm * ldc + gn] = Conv<TC>::store(v);
    }
  }
}

// ---- fp32 variant with an asynchronous-copy pipeline ------------------------------
// Same tiling (64 x 64 per CTA, 4 x 4 per thread) but K blocks of 32 travel
// global -> shared with 16-byte cp.async copies, three blocks ahead of the
// FMAs, so a small problem (the 256^3 case runs on 16 CTAs) is no longer paced
// by one global-memory round trip per K block.  Needs 16-byte aligned A and B
// and row pitches that are multiples of 4 floats; edges are zero-filled by
// giving cp.async a short (or zero) source size.
constexpr int AK = 32, ASTAGES = 3;
constexpr int A_PITCH = AK + 4;  // floats; keeps 16-byte alignment, spreads banks
constexpr int B_PITCH = TN + 4;

struct AsyncStage {
  float a[TM][A_PITCH];
  float b[AK][B_PITCH];
};

__device__ __forceinline__ void cpAsync16(void *smemDst, const void *gmemSrc,
                                          int srcBytes) {
  const unsigned dst = static_cast<unsigned>(__cvta_generic_to_shared(smemDst));
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst),
               "l"(gmemSrc), "r"(srcBytes)
               : "memory");
}

// acc += A[m0.., kBegin:K] @ B[kBegin:K, n0..] for this thread's 4 x 4 block
// (kBegin a multiple of 4, K the end of the range this CTA sums over).
__device__ __forceinline__ void gemmTileAsyncRange(const float *__restrict__ a,
                                                   const float *__restrict__ b, long long M,
                                                   long long N, long long kBegin, long long K,
                                                   long long lda, long long ldb,
                                                   AsyncStage *stages, float (&acc)[4][4]) {
  const int tid = threadIdx.x;
  const long long m0 = (long long)blockIdx.y * TM;
  const long long n0 = (long long)blockIdx.x * TN;

  // Copy assignment: A tile 64 x 32 = 512 packets of 4 floats, B tile 32 x 64
  // = 512 packets; each thread moves two of each.
  auto issue = [&](int stage, long long k0) {
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int ar = (tid >> 3) + 32 * h, ac = (tid & 7) << 2;
      const long long gm = m0 + ar, gk = k0 + ac;
      int bytes = 0;
      if (gm < M && gk < K)
        bytes = int(min((long long)4, K - gk)) * 4;
      // A clamped in-range address keeps the copy legal when nothing is read.
      const float *src = a + (gm < M ? gm : 0) * lda + (gk < K ? gk : 0);
      cpAsync16(&stages[stage].a[ar][ac], src, bytes);

      const int br = (tid >> 4) + 16 * h, bc = (tid & 15) << 2;
      const long long gkb = k0 + br, gn = n0 + bc;
      bytes = 0;
      if (gkb < K && gn < N)
        bytes = int(min((long long)4, N - gn)) * 4;
      const float *srcB = b + (gkb < K ? gkb : 0) * ldb + (gn < N ? gn : 0);
      cpAsync16(&stages[stage].b[br][bc], srcB, bytes);
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };

  const int ty = tid >> 4, tx = tid & 15;
  const long long kBlocks = K > kBegin ? (K - kBegin + AK - 1) / AK : 0;
  // Prologue: fill the pipeline (empty commits keep the group count uniform).
  for (int s = 0; s < ASTAGES - 1; ++s) {
    if (s < kBlocks)
      issue(s, kBegin + (long long)s * AK);
    else
      asm volatile("cp.async.commit_group;" ::: "memory");
  }
  for (long long kb = 0; kb < kBlocks; ++kb) {
    asm volatile("cp.async.wait_group %0;" ::"n"(ASTAGES - 2) : "memory");
    __syncthreads(); // block kb has landed; block kb-1's buffer is free
    const long long next = kb + ASTAGES - 1;
    if (next < kBlocks)
      issue(int(next % ASTAGES), kBegin + next * AK);
    else
      asm volatile("cp.async.commit_group;" ::: "memory");
    const AsyncStage &st = stages[kb % ASTAGES];
#pragma unroll
    for (int k = 0; k < AK; ++k) {
      float av[4];
#pragma unroll
      for (int i = 0; i < 4; ++i)
        av[i] = st.a[ty * 4 + i][k];
      const float4 bv = *reinterpret_cast<const float4 *>(&st.b[k][tx * 4]);
      const float bb[4] = {bv.x, bv.y, bv.z, bv.w};
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j)
          acc[i][j] = fmaf(av[i], bb[j], acc[i][j]);
    }
  }
}

__device__ __forceinline__ void gemmTileAsync(const float *__restrict__ a,
                                              const float *__restrict__ b,
                                              float *__restrict__ c, long long M,
                                              long long N, long long K,
                                              long long lda, long long ldb,
                                              long long ldc, AsyncStage *stages) {
  float acc[4][4] = {};
  gemmTileAsyncRange(a, b, M, N, 0, K, lda, ldb, stages, acc);
  const int ty = threadIdx.x >> 4, tx = threadIdx.x & 15;
  const long long m0 = (long long)blockIdx.y * TM, n0 = (long long)blockIdx.x * TN;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const long long gm = m0 + ty * 4 + i;
    if (gm >= M)
      continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const long long gn = n0 + tx * 4 + j;
      if (gn < N)
        c[gm * ldc + gn] = acc[i][j];
    }
  }
}

// ---- split-K over a thread-block cluster --------------------------------------------
// A problem with few output tiles (the 256^3 case has 16) leaves most SMs
// idle and is paced by the K loop of one CTA.  Here a cluster of four CTAs
// shares one tile: each sums a quarter of K (rounded to whole K blocks), parks
// its 64 x 64 partial result in its own shared memory, and after a cluster
// barrier each CTA adds up a quarter of the rows - reading the three other
// partials through distributed shared memory, always in rank order, so the
// result does not depend on timing - and stores them.
constexpr int SPLIT = 4;
constexpr int P_PITCH = TN + 4; // floats per row of a parked partial tile

__device__ __forceinline__ void gemmTileSplitK(const float *__restrict__ a,
                                               const float *__restrict__ b,
                                               float *__restrict__ c, long long M,
                                               long long N, long long K, long long lda,
                                               long long ldb, long long ldc,
                                               AsyncStage *stages) {
  cg::cluster_group cluster = cg::this_cluster();
  const int rank = int(cluster.block_rank());
  const long long perRank = ((K + SPLIT - 1) / SPLIT + AK - 1) / AK * AK;
  const long long kBegin = rank * perRank;
  const long long kEnd = kBegin + perRank < K ? kBegin + perRank : K;
  float acc[4][4] = {};
  gemmTileAsyncRange(a, b, M, N, kBegin, kEnd, lda, ldb, stages, acc);

  const int tid = threadIdx.x, ty = tid >> 4, tx = tid & 15;
  asm volatile("cp.async.wait_group 0;" ::: "memory");
  __syncthreads(); // every thread is done with the stages: reuse them for the partial
  float *partial = reinterpret_cast<float *>(stages);
#pragma unroll
  for (int i = 0; i < 4; ++i)
    *reinterpret_cast<float4 *>(&partial[(ty * 4 + i) * P_PITCH + tx * 4]) =
        make_float4(acc[i][0], acc[i][1], acc[i][2], acc[i][3]);
  cluster.sync();

  // This CTA's quarter of the rows: 16 rows x 64 columns, one float4 per thread.
  const int row = rank * (TM / SPLIT) + (tid >> 4), col = (tid & 15) << 2;
  float4 sum = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
  for (int r = 0; r < SPLIT; ++r) {
    const float *peer = cluster.map_shared_rank(partial, r);
    const float4 v = *reinterpret_cast<const float4 *>(&peer[row * P_PITCH + col]);
    sum.x += v.x;
    sum.y += v.y;
    sum.z += v.z;
    sum.w += v.w;
  }
  const long long gm = (long long)blockIdx.y * TM + row;
  const long long gn = (long long)blockIdx.x * TN + col;
  if (gm < M) {
    const float out[4] = {sum.x, sum.y, sum.z, sum.w};
#pragma unroll
    for (int j = 0; j < 4; ++j)
      if (gn + j < N)
        c[gm * ldc + gn + j] = out[j];
  }
  cluster.sync(); // nobody leaves while a peer may still read its partial
}

} // namespace

extern "C" __global__ void __launch_bounds__(THREADS)
    hc_gemm_tiled_f32_async(const float *a, const float *b, float *c,
                            long long M, long long N, long long K,
                            long long lda, long long ldb, long long ldc) {
  extern __shared__ __align__(16) unsigned char asyncSmem[];
  gemmTileAsync(a, b, c, M, N, K, lda, ldb, ldc,
                reinterpret_cast<AsyncStage *>(asyncSmem));
}

extern "C" __global__ void __cluster_dims__(1, 1, SPLIT) __launch_bounds__(THREADS)
    hc_gemm_tiled_f32_splitk(const float *a, const float *b, float *c,
                             long long M, long long N, long long K,
                             long long lda, long long ldb, long long ldc) {
  extern __shared__ __align__(16) unsigned char splitSmem[];
  gemmTileSplitK(a, b, c, M, N, K, lda, ldb, ldc,
                 reinterpret_cast<AsyncStage *>(splitSmem));
}

extern "C" __global__ void __launch_bounds__(THREADS)
    hc_gemm_tiled_f32(const float *a, const float *b, float *c, long long M,
                      long long N, long long K, long long lda, long long ldb,
                      long long ldc) {
  gemmTile<float, float, float, float>(a, b, c, nullptr, M, N, K, lda, ldb,
                                       ldc);
}

extern "C" __global__ void __launch_bounds__(THREADS)
    hc_gemm_tiled_f64(const double *a, const double *b, double *c, long long M,
                      long long N, long long K, long long lda, long long ldb,
                      long long ldc) {
  gemmTile<double, double, double, double>(a, b, c, nullptr, M, N, K, lda, ldb,
                                           ldc);
}

extern "C" __global__ void __launch_bounds__(THREADS)
    hc_gemm_tiled_bf16(const __nv_bfloat16 *a, const __nv_bfloat16 *b,
                       __nv_bfloat16 *c, long long M, long long N, long long K,
                       long long lda, long long ldb, long long ldc) {
  gemmTile<__nv_bfloat16, __nv_bfloat16, __nv_bfloat16, float>(
      a, b, c, nullptr, M, N, K, lda, ldb, ldc);
}

extern "C" __global__ void __launch_bounds__(THREADS)
    hc_gemm_tiled_w8a16(const __nv_bfloat16 *a, const int8_t *w,
                        const float *scale, __nv_bfloat16 *c, long long M,
                        long long N, long long K, long long lda, long long ldw,
                        long long ldc) {
  gemmTile<__nv_bfloat16, int8_t, __nv_bfloat16, float>(a, w, c, scale, M, N, K,
                                                        lda, ldw, ldc);
}
