// fp32 GEMM on the 5th-generation tensor cores: C[M, N] = A[M, K] @ B[K, N] with
// float32 inputs and outputs, accurate to float32 level.
//
// It computes what the reference's dot kernels compute on float32 arrays
// (python/hckernel/tests/test_examples.py:88-111 K-blocked, :136-155 full-K):
// every work-group owns an output tile, accumulates A-tile x B-tile products
// over K in a zero-initialised accumulator and stores the tile clipped to the
// matrix.  The CUDA-core kernel (gemm_tiled.cu) does that with one FMA per
// product; here the products run on tcgen05.mma.kind::tf32.
//
// tf32 keeps 10 of float32's 23 fraction bits, so a single tf32 product is
// three decimal digits short of float32.  Every operand is therefore split in
// two tf32 numbers, a = hi + lo with hi = tf32(a) and lo = tf32(a - hi), and
// three products are accumulated in the fp32 accumulator in TMEM:
//     a * b ~= lo_a * hi_b + hi_a * lo_b + hi_a * hi_b
// The term left out, lo_a * lo_b, is 2^-22 of the product, and the split parts
// are rounded to nearest, so the result stays within about 3e-7 * sum|a||b| of
// the exact one - the accuracy class of a float32 FMA loop (the parity tests
// ask for 1e-5 * sum|a||b|).  Three tf32 products on the tensor cores still run
// several times faster than one FMA per product on the CUDA cores.
//
// Two kernels:
//   hc_split_tf32        A[M, K] -> hi, lo [M, Kp] (Kp = K rounded up to 4, the
//                        pad zero-filled);
//   hc_split_tf32_t      B[K, N] -> hi, lo of B transposed, [N, Kp]: both MMA
//                        operands are then K-major, the layout of A in the bf16
//                        kernel (gemm_bf16_umma.cu);
//   hc_gemm_f32_umma[_pair]  the product: one persistent CTA per SM (or a CTA pair
//                        on a 256 x 256 tile, cta_group::2), 192 threads -
//                        warp 0 TMA producer (four boxes per 32-deep K-block:
//                        A hi, A lo, B hi, B lo; 128-byte swizzle, zero fill at
//                        the edges, no multicast), warp 1 MMA issuer (M128 N256
//                        K8, twelve per K-block), warps 2-5 epilogue
//                        (tcgen05.ld -> 16-byte float stores), two 256-column
//                        accumulators in TMEM so that the epilogue of a tile
//                        overlaps the main loop of the next.
//
// Every mbarrier wait is bounded (hc_ptx.cuh), as in the bf16 kernel.
#include "hc_ptx.cuh"

namespace {

using namespace hc;

constexpr int BM = 128;    // accumulator rows per CTA (TMEM lanes)
constexpr int BN = 256;    // accumulator columns per tile
constexpr int BK = 32;     // K depth of one stage: 32 floats = one 128-byte row
constexpr int UMMA_K = 8;  // K depth of one tcgen05.mma with tf32 inputs
constexpr int NUM_THREADS = 192;
constexpr int TMEM_COLS = 512;
constexpr int kABytes = BM * BK * 4;  // one of hi / lo: 128 rows of A per CTA

// PAIR: two CTAs (a cluster of 2) work on one 256 x 256 tile with
// tcgen05.mma.cta_group::2; each stages its own 128 rows of A and its own 128
// columns of B (128 rows of B transposed), 64 KiB per K-block instead of 96.
template <bool PAIR> struct Config {
  static constexpr int kCtas = PAIR ? 2 : 1;
  static constexpr int kTileM = BM * kCtas;
  static constexpr int kBRows = BN / kCtas; // rows of B transposed a CTA stages
  static constexpr int kBBytes = kBRows * BK * 4;
  static constexpr int kStageBytes = 2 * kABytes + 2 * kBBytes; // 96 / 64 KiB
  static constexpr int kStages = PAIR ? 3 : 2;
  // Instruction descriptor for kind::tf32 with f32 accumulation: bits 4-5 D format
  // (1 = f32), 7-9 A format (2 = tf32), 10-12 B format, 15 / 16 A / B major
  // (0 = K), 17-22 N >> 3, 24-28 M >> 4.
  static constexpr uint32_t kInstrDesc = (1u << 4) | (2u << 7) | (2u << 10) |
                                         (uint32_t(BN >> 3) << 17) |
                                         (uint32_t(kTileM >> 4) << 24);
};

struct alignas(8) Barriers {
  uint64_t full[4];
  uint64_t empty[4];
  uint64_t tmemFull[2];
  uint64_t tmemEmpty[2];
  uint32_t tmemBase;
  int abortFlag;
};

} // namespace

// hi / lo parts of a row-major matrix, rows padded to `outPitch` with zeros.
// Packets of four columns where the layout allows 16-byte accesses (all pitches
// and `cols` multiples of 4, 16-byte aligned bases), two rows in flight per thread.
extern "C" __global__ void __launch_bounds__(256)
    hc_split_tf32(const float *__restrict__ in, float *__restrict__ hi, float *__restrict__ lo,
                  long long rows, long long cols, long long inPitch, long long outPitch) {
  const bool packets = ((inPitch | outPitch | cols) & 3) == 0 &&
                       ((reinterpret_cast<uintptr_t>(in) | reinterpret_cast<uintptr_t>(hi) |
                         reinterpret_cast<uintptr_t>(lo)) & 15) == 0;
  if (packets) {
    const long long perRow = outPitch >> 2, live = cols >> 2;
    auto one = [&](float4 v, long long r, long long c) {
      float4 h, l;
      splitTf32(v.x, h.x, l.x);
      splitTf32(v.y, h.y, l.y);
      splitTf32(v.z, h.z, l.z);
      splitTf32(v.w, h.w, l.w);
      reinterpret_cast<float4 *>(hi + r * outPitch)[c] = h;
      reinterpret_cast<float4 *>(lo + r * outPitch)[c] = l;
    };
    const float4 zero = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    for (long long r = 2ll * blockIdx.y; r < rows; r += 2ll * gridDim.y)
      for (long long c = (long long)blockIdx.x * blockDim.x + threadIdx.x; c < perRow;
           c += (long long)gridDim.x * blockDim.x) {
        const bool second = r + 1 < rows;
        const float4 v0 = c < live ? reinterpret_cast<const float4 *>(in + r * inPitch)[c] : zero;
        const float4 v1 = second && c < live
                              ? reinterpret_cast<const float4 *>(in + (r + 1) * inPitch)[c]
                              : zero;
        one(v0, r, c);
        if (second)
          one(v1, r + 1, c);
      }
    return;
  }
  const long long perRow = outPitch;
  for (long long r = blockIdx.y; r < rows; r += gridDim.y)
    for (long long c = (long long)blockIdx.x * blockDim.x + threadIdx.x; c < perRow;
         c += (long long)gridDim.x * blockDim.x) {
      float h = 0.0f, l = 0.0f;
      if (c < cols)
        splitTf32(in[r * inPitch + c], h, l);
      hi[r * outPitch + c] = h;
      lo[r * outPitch + c] = l;
    }
}

// hi / lo parts of the transpose: in [rows, cols] -> out [cols, outPitch >= rows].
// Tiles of 64 rows x 32 columns: eight loads in flight per thread, and an output
// row gets 256 contiguous bytes per tile.
extern "C" __global__ void __launch_bounds__(256)
    hc_split_tf32_t(const float *__restrict__ in, float *__restrict__ hi,
                    float *__restrict__ lo, long long rows, long long cols, long long inPitch,
                    long long outPitch) {
  __shared__ float tile[64][33];
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5; // 32 x 8 threads
  const long long tilesX = (cols + 31) / 32, tilesY = (outPitch + 63) / 64;
  for (long long t = blockIdx.x; t < tilesX * tilesY; t += gridDim.x) {
    const long long c0 = (t % tilesX) * 32, r0 = (t / tilesX) * 64;
    float v[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const long long r = r0 + ty + 8 * j, c = c0 + tx;
      v[j] = (r < rows && c < cols) ? in[r * inPitch + c] : 0.0f;
    }
    __syncthreads(); // the tile of the round before has been read
#pragma unroll
    for (int j = 0; j < 8; ++j)
      tile[ty + 8 * j][tx] = v[j];
    __syncthreads();
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const long long c = c0 + ty + 8 * j; // out[c][r]
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        const long long r = r0 + 32 * half + tx;
        if (c < cols && r < outPitch) {
          float h, l;
          splitTf32(tile[32 * half + tx][ty + 8 * j], h, l);
          hi[c * outPitch + r] = h;
          lo[c * outPitch + r] = l;
        }
      }
    }
  }
}

namespace {

template <bool PAIR>
__device__ __forceinline__ void
gemmF32(const CUtensorMap &mapAHi, const CUtensorMap &mapALo, const CUtensorMap &mapBHi,
        const CUtensorMap &mapBLo, float *__restrict__ c, long long M, long long N, long long K,
        long long ldc, int tilesM, int tilesN, int bandM, int vecStore, int *status,
        unsigned char *smemRaw) {
  using Cfg = Config<PAIR>;
  constexpr int kStages = Cfg::kStages, kStageBytes = Cfg::kStageBytes, kBBytes = Cfg::kBBytes;
  const uint32_t smemBase = (smemAddr(smemRaw) + 1023u) & ~1023u;
  Barriers *bars = reinterpret_cast<Barriers *>(smemRaw + (smemBase - smemAddr(smemRaw)) +
                                                kStages * kStageBytes);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t ctaRank = PAIR ? clusterCtaRank() : 0u;
  const bool leader = ctaRank == 0;
  volatile int *abortFlag = &bars->abortFlag;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbarInit(smemAddr(&bars->full[s]), 1);
      mbarInit(smemAddr(&bars->empty[s]), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbarInit(smemAddr(&bars->tmemFull[a]), 1);
      mbarInit(smemAddr(&bars->tmemEmpty[a]), 4 * Cfg::kCtas);
    }
    bars->abortFlag = 0;
    fenceBarrierInit();
    prefetchTensorMap(&mapAHi);
    prefetchTensorMap(&mapALo);
    prefetchTensorMap(&mapBHi);
    prefetchTensorMap(&mapBLo);
  }
  if (warp == 1) {
    tmemAlloc<Cfg::kCtas>(smemAddr(&bars->tmemBase), TMEM_COLS);
    tmemRelinquish<Cfg::kCtas>();
  }
  tcgen05FenceBefore();
  if constexpr (PAIR)
    clusterSync();
  else
    __syncthreads();
  tcgen05FenceAfter();
  const uint32_t tmemBase = bars->tmemBase;

  const int kBlocks = int((K + BK - 1) / BK);
  const int numTiles = tilesM * tilesN;
  const int firstTile = PAIR ? (blockIdx.x >> 1) : blockIdx.x;
  const int tileStep = PAIR ? (gridDim.x >> 1) : gridDim.x;
  auto tileCoords = [&](int t, int &tm, int &tn) {
    const int perBand = bandM * tilesN;
    const int band = t / perBand, rem = t - band * perBand;
    const int rowsInBand = min(bandM, tilesM - band * bandM);
    tm = band * bandM + rem % rowsInBand;
    tn = rem / rowsInBand;
  };

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    if (lane == 0) {
      uint32_t it = 0;
      for (int t = firstTile; t < numTiles && !*abortFlag; t += tileStep) {
        int tm, tn;
        tileCoords(t, tm, tn);
        const int row0 = tm * Cfg::kTileM + int(ctaRank) * BM;
        const int col0 = tn * BN + int(ctaRank) * Cfg::kBRows;
        for (int kb = 0; kb < kBlocks; ++kb, ++it) {
          const uint32_t s = it % kStages, phase = (it / kStages) & 1u;
          if (!mbarWait(smemAddr(&bars->empty[s]), phase ^ 1u, abortFlag, status,
                        kStatusProducerWait))
            break;
          uint32_t fullBar = smemAddr(&bars->full[s]);
          const uint32_t stage = smemBase + s * kStageBytes;
          if constexpr (PAIR) {
            // Completion bytes of both CTAs are counted on the leader's barrier,
            // and only the leader arrives, expecting the bytes of both.
            fullBar = mapSharedToCta(fullBar, 0);
            if (leader)
              mbarExpectTx(smemAddr(&bars->full[s]), 2 * kStageBytes);
            tmaLoad2DPair(stage, &mapAHi, fullBar, kb * BK, row0);
            tmaLoad2DPair(stage + kABytes, &mapALo, fullBar, kb * BK, row0);
            tmaLoad2DPair(stage + 2 * kABytes, &mapBHi, fullBar, kb * BK, col0);
            tmaLoad2DPair(stage + 2 * kABytes + kBBytes, &mapBLo, fullBar, kb * BK, col0);
          } else {
            mbarExpectTx(fullBar, kStageBytes);
            tmaLoad2D(stage, &mapAHi, fullBar, kb * BK, row0);
            tmaLoad2D(stage + kABytes, &mapALo, fullBar, kb * BK, row0);
            tmaLoad2D(stage + 2 * kABytes, &mapBHi, fullBar, kb * BK, col0);
            tmaLoad2D(stage + 2 * kABytes + kBBytes, &mapBLo, fullBar, kb * BK, col0);
          }
        }
      }
      // Tail: the commits that free the last stages must have landed before the
      // CTA's shared memory goes away.
      for (int i = 0; i < kStages && !*abortFlag; ++i, ++it) {
        const uint32_t s = it % kStages, phase = (it / kStages) & 1u;
        if (!mbarWait(smemAddr(&bars->empty[s]), phase ^ 1u, abortFlag, status,
                      kStatusDrainWait))
          break;
      }
      if (*abortFlag) {
        // Copies may still be landing in this CTA's stages: give them time.
        const unsigned long long t0 = globalTimerNs();
        while (globalTimerNs() - t0 < 1000000ull) {
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------- MMA issuer -------------------------------
    if (lane == 0 && leader) {
      uint32_t it = 0;
      int tileIter = 0;
      for (int t = firstTile; t < numTiles && !*abortFlag; t += tileStep, ++tileIter) {
        const int acc = tileIter & 1;
        const uint32_t accPhase = (tileIter >> 1) & 1u;
        if (!mbarWait(smemAddr(&bars->tmemEmpty[acc]), accPhase ^ 1u, abortFlag, status,
                      kStatusMmaWaitTmem))
          break;
        tcgen05FenceAfter();
        const uint32_t dTmem = tmemBase + uint32_t(acc * BN);
        bool ok = true;
        for (int kb = 0; kb < kBlocks; ++kb, ++it) {
          const uint32_t s = it % kStages, phase = (it / kStages) & 1u;
          if (!mbarWait(smemAddr(&bars->full[s]), phase, abortFlag, status,
                        kStatusMmaWaitData)) {
            ok = false;
            break;
          }
          tcgen05FenceAfter();
          const uint32_t stage = smemBase + s * kStageBytes;
          // All four operands are K-major: rows of 128 bytes, 8-row groups 1024
          // bytes apart.
          const uint64_t aHi = makeSmemDesc(stage, 16, 1024);
          const uint64_t aLo = makeSmemDesc(stage + kABytes, 16, 1024);
          const uint64_t bHi = makeSmemDesc(stage + 2 * kABytes, 16, 1024);
          const uint64_t bLo = makeSmemDesc(stage + 2 * kABytes + kBBytes, 16, 1024);
#pragma unroll
          for (int kk = 0; kk < BK / UMMA_K; ++kk) {
            // 8 K-elements further: 32 bytes along a row.  The small terms first.
            const uint64_t step = uint64_t(kk * 2);
            ummaTf32<Cfg::kCtas>(dTmem, aLo + step, bHi + step, Cfg::kInstrDesc, (kb | kk) != 0);
            ummaTf32<Cfg::kCtas>(dTmem, aHi + step, bLo + step, Cfg::kInstrDesc, 1);
            ummaTf32<Cfg::kCtas>(dTmem, aHi + step, bHi + step, Cfg::kInstrDesc, 1);
          }
          // Frees the stage (in both CTAs of a pair) once these MMAs are done.
          if constexpr (PAIR)
            ummaCommitPair(smemAddr(&bars->empty[s]), 0x3);
          else
            ummaCommit(smemAddr(&bars->empty[s]));
        }
        if (!ok)
          break;
        if constexpr (PAIR)
          ummaCommitPair(smemAddr(&bars->tmemFull[acc]), 0x3);
        else
          ummaCommit(smemAddr(&bars->tmemFull[acc]));
      }
    }
  } else {
    // -------------------------------- epilogue --------------------------------
    const int quad = warp & 3; // TMEM lanes [32*quad, 32*quad+32) for this warp
    uint32_t tmemEmptyBar[2];
    for (int a = 0; a < 2; ++a) {
      tmemEmptyBar[a] = smemAddr(&bars->tmemEmpty[a]);
      if constexpr (PAIR)
        tmemEmptyBar[a] = mapSharedToCta(tmemEmptyBar[a], 0);
    }
    int tileIter = 0;
    for (int t = firstTile; t < numTiles; t += tileStep, ++tileIter) {
      int tm, tn;
      tileCoords(t, tm, tn);
      const int acc = tileIter & 1;
      const uint32_t accPhase = (tileIter >> 1) & 1u;
      bool ok = true;
      if (lane == 0)
        ok = mbarWait(smemAddr(&bars->tmemFull[acc]), accPhase, abortFlag, status,
                      kStatusEpilogueWait);
      ok = __shfl_sync(0xffffffffu, ok, 0);
      if (!ok)
        break;
      tcgen05FenceAfter();
      const long long row = (long long)tm * Cfg::kTileM + int(ctaRank) * BM + quad * 32 + lane;
      const long long colBase = (long long)tn * BN;
      const uint32_t taddr = tmemBase + (uint32_t(quad * 32) << 16) + uint32_t(acc * BN);
      float *crow = c + row * ldc;
#pragma unroll 1
      for (int ch = 0; ch < BN / 32; ++ch) {
        uint32_t v[32];
        __syncwarp(); // tcgen05.ld needs the whole warp, converged
        tmemLoad32x32(taddr + uint32_t(ch * 32), v);
        tmemLoadWait();
        const long long col = colBase + ch * 32;
        if (col >= N) // uniform over the warp
          break;
        if (row < M) {
          if (vecStore && col + 32 <= N) {
            float4 *dst = reinterpret_cast<float4 *>(crow + col);
#pragma unroll
            for (int q = 0; q < 8; ++q)
              dst[q] = make_float4(__uint_as_float(v[4 * q]), __uint_as_float(v[4 * q + 1]),
                                   __uint_as_float(v[4 * q + 2]), __uint_as_float(v[4 * q + 3]));
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (col + j < N)
                crow[col + j] = __uint_as_float(v[j]);
          }
        }
      }
      // This warp has read its quarter of the accumulator.
      tcgen05FenceBefore();
      __syncwarp();
      if (lane == 0) {
        if constexpr (PAIR)
          mbarArriveCluster(tmemEmptyBar[acc]);
        else
          mbarArrive(tmemEmptyBar[acc]);
      }
    }
  }

  // -------------------------------- teardown ----------------------------------
  __syncwarp();
  tcgen05FenceBefore();
  if constexpr (PAIR)
    clusterSync();
  else
    __syncthreads();
  if (warp == 1) {
    tcgen05FenceAfter();
    tmemFree<Cfg::kCtas>(tmemBase, TMEM_COLS);
  }
}

} // namespace

#define HC_GEMM_F32_ARGS                                                                 \
  const __grid_constant__ CUtensorMap mapAHi, const __grid_constant__ CUtensorMap mapALo, \
      const __grid_constant__ CUtensorMap mapBHi, const __grid_constant__ CUtensorMap mapBLo, \
      float *c, long long M, long long N, long long K, long long ldc, int tilesM, int tilesN, \
      int bandM, int vecStore, int *status

extern "C" __global__ void __launch_bounds__(NUM_THREADS, 1) hc_gemm_f32_umma(HC_GEMM_F32_ARGS) {
  extern __shared__ __align__(1024) unsigned char smemRaw[];
  gemmF32<false>(mapAHi, mapALo, mapBHi, mapBLo, c, M, N, K, ldc, tilesM, tilesN, bandM,
                 vecStore, status, smemRaw);
}

extern "C" __global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(NUM_THREADS, 1)
    hc_gemm_f32_umma_pair(HC_GEMM_F32_ARGS) {
  extern __shared__ __align__(1024) unsigned char smemRaw[];
  gemmF32<true>(mapAHi, mapALo, mapBHi, mapBLo, c, M, N, K, ldc, tilesM, tilesN, bandM,
                vecStore, status, smemRaw);
}
