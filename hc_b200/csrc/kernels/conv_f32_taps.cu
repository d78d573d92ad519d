// float32 convolution (stride 1) on the 5th-generation tensor cores with both
// operands delivered by TMA: no thread touches the image.
//
//   out[n, q, oh, ow] = sum over (kh, kw, c) of
//       x[n, c, oh + kh, ow + kw] * f[q, c, kh, kw]
//
// The same sums as conv_f32_umma.cu (the reference's implicit-GEMM convolution,
// python/hckernel/tests/test_examples.py:203-252), tiled for the copy engine
// instead of for gathering threads.  The image is rewritten once with the
// channels innermost (hc_split_tf32_nhwc: x [N, C, H, W] -> hi and lo parts as
// [N, H, W, Cp], Cp = C rounded up to 32, zeros beyond C).  The GEMM's M is a
// rectangle of boxH x boxW = 128 output pixels of one image, N the filters, K
// runs over the filter taps (kh, kw) and inside a tap over blocks of 32
// channels.  For one K block the A tile is then a box of the rewritten image:
// [boxH rows, boxW pixels, 32 channels] at (oh0 + kh, ow0 + kw, 32 cb) - 128 rows
// of 128 bytes, which a rank-4 TMA load with the 128-byte swizzle puts into
// shared memory exactly as the K-major MMA descriptor reads it.  A tap shifts
// the box along W and H, which are not the innermost dimension, so no alignment
// rule is in the way; pixels beyond the image read zeros and are not stored.
// The filters are rewritten to the same K order by the same launch
// (f [NF, C, HF, WF] -> hi, lo as [NF, taps * Cp]).
//
// Arithmetic as in gemm_f32_umma.cu: three tf32 products lo*hi + hi*lo + hi*hi
// per float32 product, accumulated in fp32 in TMEM; with at most 128 filters the
// two products that share a_hi run as one MMA of double width (B = [b_hi; b_lo]).
//
// hc_conv_f32_rows goes one step further and fetches every image element once
// per filter row instead of once per tap.  Its M is 128 consecutive positions of
// the flattened image, p = oh * W + ow (the positions with ow >= WO are computed
// and not stored: 2 of 56 at the benchmark size), so that a tap (kh, kw) is a
// shift by kh * W + kw positions whatever the tile.  A stage holds, for one
// filter row kh and one block of 32 channels, the 128 + WF - 1 positions from
// p0 + kh * W on (one rank-3 TMA box, hi and lo) and the WF filter tiles; the
// A operand of tap kw is the same patch read kw rows further down - its
// descriptor starts kw * 128 bytes later (the 128-byte swizzle is a function of
// the address, so nothing else changes).
// Per tile that is a fifth of the bytes the boxes of hc_conv_f32_taps pull from
// L2 (which set its pace: 2.6 MB per tile).
//
// hc_conv_f32_taps: one persistent CTA per SM, 192 threads: warp 0 the TMA
// producer (four boxes per K block), warp 1 the MMA issuer, warps 2-5 the
// epilogue (tcgen05.ld, then for every filter a store that is contiguous along
// the pixels of a row).  Two accumulators in TMEM let the epilogue of a tile
// overlap the next tile's main loop.  Every mbarrier wait is bounded (hc_ptx.cuh).
#include "conv_params.h"
#include "hc_ptx.cuh"

namespace {

using namespace hc;

constexpr int BM = 128; // output pixels per tile (TMEM lanes)
constexpr int BK = 32;  // channels per K block: one 128-byte row
constexpr int UMMA_K = 8;
constexpr int NUM_THREADS = 192;
constexpr int TMEM_COLS = 512;
constexpr int ACC_STRIDE = 256; // TMEM columns between the two accumulators
constexpr int kABytes = BM * BK * 4;
constexpr int MAX_STAGES = 6;

struct alignas(8) Barriers {
  uint64_t full[MAX_STAGES];
  uint64_t empty[MAX_STAGES];
  uint64_t tmemFull[2];
  uint64_t tmemEmpty[2];
  uint32_t tmemBase;
  int abortFlag;
};

__device__ __forceinline__ void tmaLoad4D(uint32_t dst, const CUtensorMap *map, uint32_t bar,
                                          int c0, int c1, int c2, int c3) {
  asm volatile("cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::"
               "bytes [%0], [%1, {%3, %4, %5, %6}], [%2];" ::"r"(dst),
               "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
               : "memory");
}

} // namespace

// Both operands rewritten in one launch.  blockIdx.y < images: image blockIdx.y,
// x [C, HW] -> hi, lo [HW, Cp] - the tf32 parts of every element, channels
// innermost, zeros in the channels beyond C.  blockIdx.y == images: the filters,
// f [NF, C, taps] -> hi, lo [NF, taps * Cp] in the K order of the kernels below.
extern "C" __global__ void __launch_bounds__(256)
    hc_split_tf32_nhwc(const float *__restrict__ x, float *__restrict__ hi, float *__restrict__ lo,
                       int C, int HW, int Cp, int images, const float *__restrict__ f,
                       float *__restrict__ fHi, float *__restrict__ fLo, int NF, int taps) {
  if (int(blockIdx.y) == images) {
    const long long total = (long long)NF * taps * Cp;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * blockDim.x) {
      const int c = int(i % Cp), tap = int((i / Cp) % taps), q = int(i / ((long long)Cp * taps));
      float h = 0.0f, l = 0.0f;
      if (c < C)
        splitTf32(f[((long long)q * C + c) * taps + tap], h, l);
      fHi[i] = h;
      fLo[i] = l;
    }
    return;
  }
  // Tiles of 32 positions x 64 channels: eight loads in flight per thread, and a
  // position's 64 channels leave as 256 contiguous bytes.
  __shared__ float tile[64][33];
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5; // 32 x 8 threads
  const float *in = x + (long long)blockIdx.y * C * HW;
  float *outHi = hi + (long long)blockIdx.y * HW * Cp, *outLo = lo + (long long)blockIdx.y * HW * Cp;
  const int tilesP = (HW + 31) / 32, tilesC = (Cp + 63) / 64;
  for (int t = blockIdx.x; t < tilesP * tilesC; t += gridDim.x) {
    const int p0 = (t % tilesP) * 32, c0 = (t / tilesP) * 64;
    const int p = p0 + tx;
    float v[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int c = c0 + ty + 8 * j;
      v[j] = (c < C && p < HW) ? in[c * HW + p] : 0.0f;
    }
    __syncthreads(); // the tile of the round before has been read
#pragma unroll
    for (int j = 0; j < 8; ++j)
      tile[ty + 8 * j][tx] = v[j];
    __syncthreads();
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int q = p0 + ty + 8 * j; // position
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        const int c = c0 + 32 * half + tx;
        if (q < HW && c < Cp) {
          float h, l;
          splitTf32(tile[32 * half + tx][ty + 8 * j], h, l);
          outHi[(long long)q * Cp + c] = h;
          outLo[(long long)q * Cp + c] = l;
        }
      }
    }
  }
}

extern "C" __global__ void __launch_bounds__(NUM_THREADS, 1)
    hc_conv_f32_taps(const __grid_constant__ CUtensorMap mapXHi,
                     const __grid_constant__ CUtensorMap mapXLo,
                     const __grid_constant__ CUtensorMap mapFHi,
                     const __grid_constant__ CUtensorMap mapFLo,
                     const __grid_constant__ HcConvTapParams p) {
  extern __shared__ __align__(1024) unsigned char smemRaw[];
  const bool stacked = p.stacked != 0;
  const int bBytes = p.nPad * BK * 4; // one of f hi / f lo
  const int stageBytes = 2 * kABytes + 2 * bBytes;
  const int stages = p.stages;
  const uint32_t smemBase = (smemAddr(smemRaw) + 1023u) & ~1023u;
  unsigned char *aligned = smemRaw + (smemBase - smemAddr(smemRaw));
  Barriers *bars = reinterpret_cast<Barriers *>(aligned + stages * stageBytes);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  volatile int *abortFlag = &bars->abortFlag;

  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) {
      mbarInit(smemAddr(&bars->full[s]), 1); // the producer's expect_tx
      mbarInit(smemAddr(&bars->empty[s]), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbarInit(smemAddr(&bars->tmemFull[a]), 1);
      mbarInit(smemAddr(&bars->tmemEmpty[a]), 4);
    }
    bars->abortFlag = 0;
    fenceBarrierInit();
    prefetchTensorMap(&mapXHi);
    prefetchTensorMap(&mapXLo);
    prefetchTensorMap(&mapFHi);
    prefetchTensorMap(&mapFLo);
  }
  if (warp == 1) {
    tmemAlloc<1>(smemAddr(&bars->tmemBase), TMEM_COLS);
    tmemRelinquish<1>();
  }
  tcgen05FenceBefore();
  __syncthreads();
  tcgen05FenceAfter();
  const uint32_t tmemBase = bars->tmemBase;

  const int kBlocks = p.kBlocks;
  const int tilesPerImage = p.tilesW * p.tilesH;
  const int numTiles = p.N * tilesPerImage;

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    if (lane == 0) {
      uint32_t it = 0;
      for (int t = blockIdx.x; t < numTiles && !*abortFlag; t += gridDim.x) {
        const int n = t / tilesPerImage, r = t - n * tilesPerImage;
        const int oh0 = (r / p.tilesW) * p.boxH, ow0 = (r % p.tilesW) * p.boxW;
        int kh = 0, kw = 0, cb = 0;
        for (int kb = 0; kb < kBlocks; ++kb, ++it) {
          const uint32_t s = it % stages, phase = (it / stages) & 1u;
          if (!mbarWait(smemAddr(&bars->empty[s]), phase ^ 1u, abortFlag, p.status,
                        kStatusProducerWait))
            break;
          const uint32_t fullBar = smemAddr(&bars->full[s]);
          const uint32_t stage = smemBase + s * stageBytes;
          mbarExpectTx(fullBar, uint32_t(stageBytes));
          tmaLoad4D(stage, &mapXHi, fullBar, cb * BK, ow0 + kw, oh0 + kh, n);
          tmaLoad4D(stage + kABytes, &mapXLo, fullBar, cb * BK, ow0 + kw, oh0 + kh, n);
          tmaLoad2D(stage + 2 * kABytes, &mapFHi, fullBar, kb * BK, 0);
          tmaLoad2D(stage + 2 * kABytes + bBytes, &mapFLo, fullBar, kb * BK, 0);
          if (++cb == p.cBlocks) {
            cb = 0;
            if (++kw == p.WF) {
              kw = 0;
              ++kh;
            }
          }
        }
      }
      // Tail: the commits that free the last stages must have landed before the
      // CTA's shared memory goes away.
      for (int i = 0; i < stages && !*abortFlag; ++i, ++it) {
        const uint32_t s = it % stages, phase = (it / stages) & 1u;
        if (!mbarWait(smemAddr(&bars->empty[s]), phase ^ 1u, abortFlag, p.status,
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
    // The whole warp walks the loop, converged, and one elected lane issues.
    const bool issuer = electOne();
    // kind::tf32, f32 accumulation: bits 4-5 D format, 7-9 / 10-12 A / B format
    // (2 = tf32), 15 / 16 A / B major (0 = K), 17-22 N >> 3, 24-28 M >> 4.
    const uint32_t iDesc = (1u << 4) | (2u << 7) | (2u << 10) | (uint32_t(p.nPad >> 3) << 17) |
                           (uint32_t(BM >> 4) << 24);
    const uint32_t iDescWide = (1u << 4) | (2u << 7) | (2u << 10) |
                               (uint32_t(2 * p.nPad >> 3) << 17) | (uint32_t(BM >> 4) << 24);
    uint32_t it = 0;
    int tileIter = 0;
    for (int t = blockIdx.x; t < numTiles && !*abortFlag; t += gridDim.x, ++tileIter) {
      const int acc = tileIter & 1;
      const uint32_t accPhase = (tileIter >> 1) & 1u;
      bool ok = mbarWait(smemAddr(&bars->tmemEmpty[acc]), accPhase ^ 1u, abortFlag, p.status,
                         kStatusMmaWaitTmem);
      if (!__all_sync(0xffffffffu, ok))
        break;
      tcgen05FenceAfter();
      const uint32_t dTmem = tmemBase + uint32_t(acc * ACC_STRIDE);
      for (int kb = 0; kb < kBlocks; ++kb, ++it) {
        const uint32_t s = it % stages, phase = (it / stages) & 1u;
        ok = mbarWait(smemAddr(&bars->full[s]), phase, abortFlag, p.status, kStatusMmaWaitData);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok)
          break;
        tcgen05FenceAfter();
        const uint32_t stage = smemBase + s * stageBytes;
        // All four tiles are K-major: rows of 128 bytes, 8-row groups 1024 bytes apart.
        const uint64_t aHi = makeSmemDesc(stage, 16, 1024);
        const uint64_t aLo = makeSmemDesc(stage + kABytes, 16, 1024);
        const uint64_t bHi = makeSmemDesc(stage + 2 * kABytes, 16, 1024);
        const uint64_t bLo = makeSmemDesc(stage + 2 * kABytes + bBytes, 16, 1024);
        if (issuer && stacked) {
#pragma unroll
          for (int kk = 0; kk < BK / UMMA_K; ++kk) {
            // 8 K-elements further: 32 bytes along a row.
            const uint64_t step = uint64_t(kk * 2);
            ummaTf32<1>(dTmem, aHi + step, bHi + step, iDescWide, (kb | kk) != 0);
            ummaTf32<1>(dTmem, aLo + step, bHi + step, iDesc, 1);
          }
        } else if (issuer) {
#pragma unroll
          for (int kk = 0; kk < BK / UMMA_K; ++kk) {
            const uint64_t step = uint64_t(kk * 2);
            ummaTf32<1>(dTmem, aLo + step, bHi + step, iDesc, (kb | kk) != 0); // small terms first
            ummaTf32<1>(dTmem, aHi + step, bLo + step, iDesc, 1);
            ummaTf32<1>(dTmem, aHi + step, bHi + step, iDesc, 1);
          }
        }
        if (issuer)
          ummaCommit(smemAddr(&bars->empty[s])); // frees the stage when these are done
        __syncwarp();
      }
      if (!ok)
        break;
      if (issuer)
        ummaCommit(smemAddr(&bars->tmemFull[acc]));
      __syncwarp();
    }
  } else {
    // -------------------------------- epilogue --------------------------------
    const int quad = warp & 3; // TMEM lanes [32*quad, 32*quad+32) for this warp
    const int m = quad * 32 + lane;
    const int hl = m / p.boxW, wl = m - hl * p.boxW; // this lane's pixel inside the tile
    const long long plane = (long long)p.HO * p.WO;
    int tileIter = 0;
    for (int t = blockIdx.x; t < numTiles; t += gridDim.x, ++tileIter) {
      const int n = t / tilesPerImage, r = t - n * tilesPerImage;
      const int oh = (r / p.tilesW) * p.boxH + hl, ow = (r % p.tilesW) * p.boxW + wl;
      const int acc = tileIter & 1;
      const uint32_t accPhase = (tileIter >> 1) & 1u;
      bool ok = true;
      if (lane == 0)
        ok = mbarWait(smemAddr(&bars->tmemFull[acc]), accPhase, abortFlag, p.status,
                      kStatusEpilogueWait);
      ok = __shfl_sync(0xffffffffu, ok, 0);
      if (!ok)
        break;
      tcgen05FenceAfter();
      const bool inside = oh < p.HO && ow < p.WO;
      // Pixel (oh, ow) of filter q: lanes along a row write consecutive floats.
      float *dst = p.out + (long long)n * p.NF * plane + (long long)oh * p.WO + ow;
      const uint32_t taddr = tmemBase + (uint32_t(quad * 32) << 16) + uint32_t(acc * ACC_STRIDE);
#pragma unroll 1
      for (int ch = 0; ch * 32 < p.NF; ++ch) { // uniform over the warp
        uint32_t v[32];
        __syncwarp(); // tcgen05.ld needs the whole warp, converged
        tmemLoad32x32(taddr + uint32_t(ch * 32), v);
        if (stacked) { // the second half of the accumulator: the a_hi * b_lo sums
          uint32_t w[32];
          tmemLoad32x32(taddr + uint32_t(p.nPad + ch * 32), w);
          tmemLoadWait();
#pragma unroll
          for (int j = 0; j < 32; ++j)
            v[j] = __float_as_uint(__uint_as_float(v[j]) + __uint_as_float(w[j]));
        }
        tmemLoadWait();
        if (inside) {
#pragma unroll
          for (int j = 0; j < 32; ++j)
            if (ch * 32 + j < p.NF)
              dst[(long long)(ch * 32 + j) * plane] = __uint_as_float(v[j]);
        }
      }
      // This warp has read its quarter of the accumulator.
      tcgen05FenceBefore();
      __syncwarp();
      if (lane == 0)
        mbarArrive(smemAddr(&bars->tmemEmpty[acc]));
    }
  }

  // -------------------------------- teardown ----------------------------------
  __syncwarp();
  tcgen05FenceBefore();
  __syncthreads();
  if (warp == 1) {
    tcgen05FenceAfter();
    tmemFree<1>(tmemBase, TMEM_COLS);
  }
}

namespace {

__device__ __forceinline__ void tmaLoad3D(uint32_t dst, const CUtensorMap *map, uint32_t bar,
                                          int c0, int c1, int c2) {
  asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::"
               "bytes [%0], [%1, {%3, %4, %5}], [%2];" ::"r"(dst),
               "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(c0), "r"(c1), "r"(c2)
               : "memory");
}

// K-major, 128-byte swizzle, rows 128 bytes apart; `addr` may start at any row
// of the 8-row pattern: the swizzle is a function of the shared-memory address,
// the same one the TMA write applied, so a start further down reads the rows
// that lie there.
__device__ __forceinline__ uint64_t makeRowDesc(uint32_t addr) {
  return makeSmemDesc(addr, 16, 1024);
}

} // namespace

extern "C" __global__ void __launch_bounds__(NUM_THREADS, 1)
    hc_conv_f32_rows(const __grid_constant__ CUtensorMap mapXHi,
                     const __grid_constant__ CUtensorMap mapXLo,
                     const __grid_constant__ CUtensorMap mapFHi,
                     const __grid_constant__ CUtensorMap mapFLo,
                     const __grid_constant__ HcConvTapParams p) {
  extern __shared__ __align__(1024) unsigned char smemRaw[];
  const bool stacked = p.stacked != 0;
  const int bBytes = p.nPad * BK * 4;      // one of f hi / f lo of one tap
  const int patchBytes = p.patchRows * 128; // one of x hi / x lo
  const int stageBytes = 2 * patchBytes + p.WF * 2 * bBytes;
  const int stages = p.stages;
  const uint32_t smemBase = (smemAddr(smemRaw) + 1023u) & ~1023u;
  unsigned char *aligned = smemRaw + (smemBase - smemAddr(smemRaw));
  Barriers *bars = reinterpret_cast<Barriers *>(aligned + stages * stageBytes);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  volatile int *abortFlag = &bars->abortFlag;

  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) {
      mbarInit(smemAddr(&bars->full[s]), 1); // the producer's expect_tx
      mbarInit(smemAddr(&bars->empty[s]), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbarInit(smemAddr(&bars->tmemFull[a]), 1);
      mbarInit(smemAddr(&bars->tmemEmpty[a]), 4);
    }
    bars->abortFlag = 0;
    fenceBarrierInit();
    prefetchTensorMap(&mapXHi);
    prefetchTensorMap(&mapXLo);
    prefetchTensorMap(&mapFHi);
    prefetchTensorMap(&mapFLo);
  }
  if (warp == 1) {
    tmemAlloc<1>(smemAddr(&bars->tmemBase), TMEM_COLS);
    tmemRelinquish<1>();
  }
  tcgen05FenceBefore();
  __syncthreads();
  tcgen05FenceAfter();
  const uint32_t tmemBase = bars->tmemBase;

  const int rowBlocks = p.HF * p.cBlocks; // stages per tile
  const int numTiles = p.N * p.tilesFlat;

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    if (lane == 0) {
      uint32_t it = 0;
      for (int t = blockIdx.x; t < numTiles && !*abortFlag; t += gridDim.x) {
        const int n = t / p.tilesFlat, p0 = (t - n * p.tilesFlat) * BM;
        int kh = 0, cb = 0;
        for (int rb = 0; rb < rowBlocks; ++rb, ++it) {
          const uint32_t s = it % stages, phase = (it / stages) & 1u;
          if (!mbarWait(smemAddr(&bars->empty[s]), phase ^ 1u, abortFlag, p.status,
                        kStatusProducerWait))
            break;
          const uint32_t fullBar = smemAddr(&bars->full[s]);
          const uint32_t stage = smemBase + s * stageBytes;
          mbarExpectTx(fullBar, uint32_t(stageBytes));
          tmaLoad3D(stage, &mapXHi, fullBar, cb * BK, p0 + kh * p.W, n);
          tmaLoad3D(stage + patchBytes, &mapXLo, fullBar, cb * BK, p0 + kh * p.W, n);
          for (int kw = 0; kw < p.WF; ++kw) {
            const int col = ((kh * p.WF + kw) * p.cBlocks + cb) * BK;
            const uint32_t at = stage + 2 * patchBytes + kw * 2 * bBytes;
            tmaLoad2D(at, &mapFHi, fullBar, col, 0);
            tmaLoad2D(at + bBytes, &mapFLo, fullBar, col, 0);
          }
          if (++cb == p.cBlocks) {
            cb = 0;
            ++kh;
          }
        }
      }
      for (int i = 0; i < stages && !*abortFlag; ++i, ++it) {
        const uint32_t s = it % stages, phase = (it / stages) & 1u;
        if (!mbarWait(smemAddr(&bars->empty[s]), phase ^ 1u, abortFlag, p.status,
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
    const bool issuer = electOne();
    const uint32_t iDesc = (1u << 4) | (2u << 7) | (2u << 10) | (uint32_t(p.nPad >> 3) << 17) |
                           (uint32_t(BM >> 4) << 24);
    const uint32_t iDescWide = (1u << 4) | (2u << 7) | (2u << 10) |
                               (uint32_t(2 * p.nPad >> 3) << 17) | (uint32_t(BM >> 4) << 24);
    uint32_t it = 0;
    int tileIter = 0;
    for (int t = blockIdx.x; t < numTiles && !*abortFlag; t += gridDim.x, ++tileIter) {
      const int acc = tileIter & 1;
      const uint32_t accPhase = (tileIter >> 1) & 1u;
      bool ok = mbarWait(smemAddr(&bars->tmemEmpty[acc]), accPhase ^ 1u, abortFlag, p.status,
                         kStatusMmaWaitTmem);
      if (!__all_sync(0xffffffffu, ok))
        break;
      tcgen05FenceAfter();
      const uint32_t dTmem = tmemBase + uint32_t(acc * ACC_STRIDE);
      for (int rb = 0; rb < rowBlocks; ++rb, ++it) {
        const uint32_t s = it % stages, phase = (it / stages) & 1u;
        ok = mbarWait(smemAddr(&bars->full[s]), phase, abortFlag, p.status, kStatusMmaWaitData);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok)
          break;
        tcgen05FenceAfter();
        const uint32_t stage = smemBase + s * stageBytes;
        for (int kw = 0; kw < p.WF; ++kw) {
          // The patch kw positions further on: kw rows of 128 bytes.
          const uint64_t aHi = makeRowDesc(stage + kw * 128);
          const uint64_t aLo = makeRowDesc(stage + patchBytes + kw * 128);
          const uint32_t bAt = stage + 2 * patchBytes + kw * 2 * bBytes;
          const uint64_t bHi = makeSmemDesc(bAt, 16, 1024);
          const uint64_t bLo = makeSmemDesc(bAt + bBytes, 16, 1024);
          if (issuer && stacked) {
#pragma unroll
            for (int kk = 0; kk < BK / UMMA_K; ++kk) {
              const uint64_t step = uint64_t(kk * 2);
              ummaTf32<1>(dTmem, aHi + step, bHi + step, iDescWide, (rb | kw | kk) != 0);
              ummaTf32<1>(dTmem, aLo + step, bHi + step, iDesc, 1);
            }
          } else if (issuer) {
#pragma unroll
            for (int kk = 0; kk < BK / UMMA_K; ++kk) {
              const uint64_t step = uint64_t(kk * 2);
              ummaTf32<1>(dTmem, aLo + step, bHi + step, iDesc, (rb | kw | kk) != 0);
              ummaTf32<1>(dTmem, aHi + step, bLo + step, iDesc, 1);
              ummaTf32<1>(dTmem, aHi + step, bHi + step, iDesc, 1);
            }
          }
        }
        if (issuer)
          ummaCommit(smemAddr(&bars->empty[s])); // frees the stage when these are done
        __syncwarp();
      }
      if (!ok)
        break;
      if (issuer)
        ummaCommit(smemAddr(&bars->tmemFull[acc]));
      __syncwarp();
    }
  } else {
    // -------------------------------- epilogue --------------------------------
    const int quad = warp & 3; // TMEM lanes [32*quad, 32*quad+32) for this warp
    const long long plane = (long long)p.HO * p.WO;
    int tileIter = 0;
    for (int t = blockIdx.x; t < numTiles; t += gridDim.x, ++tileIter) {
      const int n = t / p.tilesFlat;
      const int pos = (t - n * p.tilesFlat) * BM + quad * 32 + lane; // oh * W + ow
      const int oh = pos / p.W, ow = pos - oh * p.W;
      const int acc = tileIter & 1;
      const uint32_t accPhase = (tileIter >> 1) & 1u;
      bool ok = true;
      if (lane == 0)
        ok = mbarWait(smemAddr(&bars->tmemFull[acc]), accPhase, abortFlag, p.status,
                      kStatusEpilogueWait);
      ok = __shfl_sync(0xffffffffu, ok, 0);
      if (!ok)
        break;
      tcgen05FenceAfter();
      const bool inside = oh < p.HO && ow < p.WO;
      float *dst = p.out + (long long)n * p.NF * plane + (long long)oh * p.WO + ow;
      const uint32_t taddr = tmemBase + (uint32_t(quad * 32) << 16) + uint32_t(acc * ACC_STRIDE);
#pragma unroll 1
      for (int ch = 0; ch * 32 < p.NF; ++ch) { // uniform over the warp
        uint32_t v[32];
        __syncwarp(); // tcgen05.ld needs the whole warp, converged
        tmemLoad32x32(taddr + uint32_t(ch * 32), v);
        if (stacked) { // the second half of the accumulator: the a_hi * b_lo sums
          uint32_t w[32];
          tmemLoad32x32(taddr + uint32_t(p.nPad + ch * 32), w);
          tmemLoadWait();
#pragma unroll
          for (int j = 0; j < 32; ++j)
            v[j] = __float_as_uint(__uint_as_float(v[j]) + __uint_as_float(w[j]));
        }
        tmemLoadWait();
        if (inside) {
#pragma unroll
          for (int j = 0; j < 32; ++j)
            if (ch * 32 + j < p.NF)
              dst[(long long)(ch * 32 + j) * plane] = __uint_as_float(v[j]);
        }
      }
      tcgen05FenceBefore();
      __syncwarp();
      if (lane == 0)
        mbarArrive(smemAddr(&bars->tmemEmpty[acc]));
    }
  }

  // -------------------------------- teardown ----------------------------------
  __syncwarp();
  tcgen05FenceBefore();
  __syncthreads();
  if (warp == 1) {
    tcgen05FenceAfter();
    tmemFree<1>(tmemBase, TMEM_COLS);
  }
}
