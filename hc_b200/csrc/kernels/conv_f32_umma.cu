// float32 convolution as an implicit GEMM on the 5th-generation tensor cores.
//
//   out[n, q, oh, ow] = sum over (c, kh, kw) of
//       x[n, c, oh * s + kh, ow * s + kw] * f[q, c, kh, kw]
//
// This is what the reference's implicit-GEMM convolution computes
// (python/hckernel/tests/test_examples.py:203-252: tiles of image patches and of
// filters gathered through index mappings, multiplied in K blocks, the result
// scattered to the output positions) whenever the output is square, where its
// enumeration of the positions (`i = w % W_OUT` on the H axis, `j = w // W_OUT`
// on the W axis, :237-240) visits every output element exactly once.  The body
// tiles the problem as (images x filters) per output position, which makes
// every operand element a lone 4-byte gather; here the same sums are tiled the
// way the memory lies: the GEMM's M runs over 128 consecutive output pixels of
// one image (so that for a fixed (c, kh, kw) neighbouring rows read
// neighbouring addresses), N over the filters, K over (c, kh, kw) in the order
// f is stored, so that f is the K-major B operand as it stands.
//
// Arithmetic as in gemm_f32_umma.cu: every operand is split in two tf32
// numbers (hi = tf32(v), lo = tf32(v - hi)) and three products lo*hi + hi*lo +
// hi*hi accumulate in fp32 in TMEM - float32-class results (the parity bound
// of the float32 kernels is 1e-5 * sum|x||f|).
//
// Two kernels.  hc_split_tf32_pairs writes x once as (hi, lo) pairs - the nine
// taps of a 3 x 3 filter read every element nine times, and splitting it in the
// main loop cost three times the instructions of loading it.  hc_conv_f32_umma:
// one persistent CTA per SM, 448 threads:
//   warp 0      TMA producer of the filter tiles: per 32-deep K block two boxes
//               (f hi, f lo; [NF rows, 32 k], 128-byte swizzle, rows beyond NF
//               and k beyond K zero-filled; no multicast);
//   warp 1      MMA issuer (one elected lane of the converged warp):
//               tcgen05.mma.kind::tf32, M128 N=NF(padded to 16) K8, twelve per K
//               block, small terms first;
//   warps 2-5   epilogue: tcgen05.ld, then for every filter a store that is
//               contiguous across the warp's 32 pixels;
//   warps 6-13  the image operand: thread (row m, half h) loads its 16
//               (hi, lo) pairs of the K block with 8-byte loads (read-only
//               path, L1 keeps the lines that the taps share), one block
//               ahead of their use, and writes hi and lo into the stage in the
//               128-byte-swizzled K-major layout the MMA descriptors expect,
//               then fence.proxy.async.  The 256 threads meet once per K block
//               at a named barrier (bar.sync 1); only their leader touches the
//               mbarriers - it waits for the next free stage before the meeting
//               and reports the stage filled after it.
// Two accumulators in TMEM let the epilogue of a tile overlap the next tile's
// main loop.  Every mbarrier wait is bounded (hc_ptx.cuh).
#include "conv_params.h"
#include "hc_ptx.cuh"

namespace {

using namespace hc;

constexpr int BM = 128;   // output pixels per tile (TMEM lanes)
constexpr int BK = 32;    // K depth of a stage: one 128-byte row
constexpr int UMMA_K = 8;
constexpr int GATHER_WARPS = 8;
constexpr int PER_THREAD = BM * BK / (32 * GATHER_WARPS); // k of a block per thread: 16
constexpr int NUM_THREADS = 32 * (6 + GATHER_WARPS);
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
  int gatherGo[2]; // what the gatherers' leader found: go on (1) or leave (0), per parity
};

enum : int { kStatusGatherWait = 6 }; // the image gatherers waiting for a free stage

} // namespace

// (hi, lo) of every element, interleaved: out[i] = {tf32(in[i]), tf32(in[i] - hi)}.
extern "C" __global__ void __launch_bounds__(256)
    hc_split_tf32_pairs(const float *__restrict__ in, float2 *__restrict__ out, long long n) {
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    float hi, lo;
    splitTf32(in[i], hi, lo);
    out[i] = make_float2(hi, lo);
  }
}

namespace {

// TMEM_A: the image operand of a K block goes to tensor memory (tcgen05.st: lane =
// row, 32 columns hi then 32 columns lo per stage) and the MMA reads it from
// there, so that shared memory carries the filter tiles alone.  With the image
// operand in shared memory every MMA of N = 64 reads 4 KiB of A for 2 KiB of B,
// and the shared-memory port, not the tensor pipe, sets the pace.  Needs room in
// TMEM: two accumulators of at most 128 columns and four to six stages of 64.
template <bool TMEM_A>
__device__ __forceinline__ void convF32(const CUtensorMap &mapFHi, const CUtensorMap &mapFLo,
                                        const HcConvParams &p, unsigned char *smemRaw) {
  constexpr int kAStage = TMEM_A ? 0 : 2 * kABytes; // bytes of A in a shared-memory stage
  // Stacked (p.stacked): the two products that share a_hi run as ONE MMA of twice
  // the width - B = [b_hi; b_lo], which lie behind one another in the stage, N =
  // 2 NF - into an accumulator of two halves that the epilogue adds: a_hi * b_hi
  // (+ a_lo * b_hi, a second MMA of width NF) in the first, a_hi * b_lo in the
  // second.  An M128 K8 MMA has to fetch its 4 KiB of A whatever its width, which
  // takes longer than the arithmetic of 64 columns: two instructions per K step
  // instead of three are a third less of that.
  // TMEM columns: the two accumulators, then (TMEM_A) the A stages of 64 columns
  // each - six stages beside accumulators of 64 columns, four beside 128.
  const bool stacked = p.stacked != 0;
  const int kAccStride =
      TMEM_A ? ((stacked ? 2 * p.nPad : p.nPad) <= 64 ? 64 : 128) : ACC_STRIDE;
  const uint32_t kATmemBase = uint32_t(2 * kAccStride);
  const int bBytes = p.nPad * BK * 4; // one of f hi / f lo
  const int stageBytes = kAStage + 2 * bBytes;
  const int stages = p.stages;
  const uint32_t smemBase = (smemAddr(smemRaw) + 1023u) & ~1023u;
  unsigned char *aligned = smemRaw + (smemBase - smemAddr(smemRaw));
  // Offset of (c, kh, kw) from a pixel's first element, for every k; then the barriers.
  int *koff = reinterpret_cast<int *>(aligned + stages * stageBytes);
  Barriers *bars = reinterpret_cast<Barriers *>(koff + p.kBlocks * BK);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  volatile int *abortFlag = &bars->abortFlag;

  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) {
      mbarInit(smemAddr(&bars->full[s]), 2); // the filter tile's expect_tx, the gatherers' leader
      mbarInit(smemAddr(&bars->empty[s]), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbarInit(smemAddr(&bars->tmemFull[a]), 1);
      mbarInit(smemAddr(&bars->tmemEmpty[a]), 4);
    }
    bars->abortFlag = 0;
    fenceBarrierInit();
    prefetchTensorMap(&mapFHi);
    prefetchTensorMap(&mapFLo);
  }
  {
    const int taps = p.HF * p.WF;
    const long long xsC = (long long)p.H * p.W;
    for (int k = threadIdx.x; k < p.kBlocks * BK; k += NUM_THREADS) {
      int off = 0;
      if (k < p.K) {
        const int c = k / taps, r = k - c * taps;
        const int kh = r / p.WF, kw = r - kh * p.WF;
        off = int(c * xsC + (long long)kh * p.W + kw);
      }
      koff[k] = off;
    }
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
  const int numTiles = p.N * p.tilesPerImage;
  const int pixels = p.HO * p.WO;

  if (warp == 0) {
    // --------------------------- filter tiles by TMA ---------------------------
    if (lane == 0) {
      uint32_t it = 0;
      for (int t = blockIdx.x; t < numTiles && !*abortFlag; t += gridDim.x) {
        for (int kb = 0; kb < kBlocks; ++kb, ++it) {
          const uint32_t s = it % stages, phase = (it / stages) & 1u;
          if (!mbarWait(smemAddr(&bars->empty[s]), phase ^ 1u, abortFlag, p.status,
                        kStatusProducerWait))
            break;
          const uint32_t fullBar = smemAddr(&bars->full[s]);
          const uint32_t stage = smemBase + s * stageBytes;
          mbarExpectTx(fullBar, 2 * bBytes);
          tmaLoad2D(stage + kAStage, &mapFHi, fullBar, kb * BK, 0);
          tmaLoad2D(stage + kAStage + bBytes, &mapFLo, fullBar, kb * BK, 0);
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
  } else if (warp >= 6) {
    // ------------------------ image operand by the threads ----------------------
    const int g = warp - 6;
    // A warp reaches the TMEM lanes of its quarter (warp index mod 4) only.
    const int m = (warp & 3) * 32 + lane; // row of the tile
    const int part = g >> 2;              // which 16 of the 32 k of a block
    const long long xsN = (long long)p.C * p.H * p.W;
    const float2 *pairs = static_cast<const float2 *>(p.x);
    // Where row m keeps chunk c (16 bytes, four k) of its 128-byte row.
    const uint32_t rowOffset = uint32_t(m >> 3) * 1024u + uint32_t(m & 7) * 128u;
    // Where the elements of tile `t` start for this row.
    auto rowSource = [&](int t) {
      const int n = t / p.tilesPerImage, tp = t - n * p.tilesPerImage;
      int pix = tp * BM + m;
      if (pix >= pixels)
        pix = 0; // a row past the image computes something that is never stored
      const int oh = pix / p.WO, ow = pix - oh * p.WO;
      return pairs + n * xsN + (long long)oh * p.stride * p.W + ow * p.stride;
    };
    auto loadBlock = [&](const float2 *src, int kb, float2 (&v)[PER_THREAD]) {
      const int k0 = kb * BK + part * PER_THREAD;
#pragma unroll
      for (int q = 0; q < PER_THREAD / 4; ++q) {
        const int4 o = *reinterpret_cast<const int4 *>(koff + k0 + 4 * q);
        v[4 * q + 0] = __ldg(src + o.x);
        v[4 * q + 1] = __ldg(src + o.y);
        v[4 * q + 2] = __ldg(src + o.z);
        v[4 * q + 3] = __ldg(src + o.w);
      }
    };
    // The loads of a K block are issued one block ahead of its stores, into one of
    // two register buffers that the unrolled loop names at compile time, so that
    // their latency is covered by the storing of the block before (nothing is
    // copied between buffers, which would wait for the loads).  Eight warps with
    // 16 pairs per thread measured 10 % faster than sixteen with 8 (the work a
    // warp does per K block besides its elements is the same) and four with 32
    // spill.
    struct Cursor {
      int t, kb;
      const float2 *src;
      bool have;
    };
    auto advance = [&](Cursor &c) {
      if (c.have && ++c.kb == kBlocks) {
        c.kb = 0;
        c.t += gridDim.x;
        c.have = c.t < numTiles;
        if (c.have)
          c.src = rowSource(c.t);
      }
    };
    constexpr int AHEAD = 1, BUFFERS = AHEAD + 1;
    Cursor fetch{int(blockIdx.x), 0, pairs, int(blockIdx.x) < numTiles};
    if (fetch.have)
      fetch.src = rowSource(fetch.t);
    Cursor use = fetch;
    float2 buf[BUFFERS][PER_THREAD];
#pragma unroll
    for (int r = 0; r < AHEAD; ++r) {
      if (fetch.have)
        loadBlock(fetch.src, fetch.kb, buf[r]);
      advance(fetch);
    }
    const bool leader = threadIdx.x == 6 * 32;
    auto meet = [] { asm volatile("bar.sync 1, %0;" ::"r"(32 * GATHER_WARPS) : "memory"); };
    // The leader waits for the stage of block `index` and notes the outcome where
    // the others read it after the next meeting.
    auto awaitStage = [&](uint32_t index) {
      const uint32_t s = index % stages, phase = (index / stages) & 1u;
      const bool ok = mbarWait(smemAddr(&bars->empty[s]), phase ^ 1u, abortFlag, p.status,
                               kStatusGatherWait);
      *(volatile int *)&bars->gatherGo[index & 1u] = ok ? 1 : 0;
    };
    uint32_t it = 0;
    if (leader && use.have)
      awaitStage(0);
    bool go = use.have;
    bool pending = false; // block it - 1 is stored but not yet reported
    while (go) {
#pragma unroll
      for (int r = 0; r < BUFFERS; ++r) {
        if (!go)
          break;
        if (fetch.have)
          loadBlock(fetch.src, fetch.kb, buf[(r + AHEAD) % BUFFERS]);
        advance(fetch);
        // Everybody's stores of the block before are done and fenced, and the
        // leader knows whether the stage of this block is free.
        meet();
        if (leader && pending)
          mbarArrive(smemAddr(&bars->full[(it - 1) % stages]));
        pending = false;
        if (*(volatile int *)&bars->gatherGo[it & 1u] == 0) {
          go = false; // a wait gave up: everybody leaves here, together
          break;
        }
        const uint32_t s = it % stages;
        const int k0 = use.kb * BK + part * PER_THREAD;
        // Beyond K the filter tile is zero; the image side must then be finite
        // (only the last block can reach beyond K).
        const bool ragged = k0 + PER_THREAD > p.K;
        if constexpr (TMEM_A) {
          uint32_t hi[PER_THREAD], lo[PER_THREAD];
#pragma unroll
          for (int e = 0; e < PER_THREAD; ++e) {
            const bool beyond = ragged && k0 + e >= p.K;
            hi[e] = beyond ? 0u : __float_as_uint(buf[r][e].x);
            lo[e] = beyond ? 0u : __float_as_uint(buf[r][e].y);
          }
          const uint32_t at = tmemBase + (uint32_t((warp & 3) * 32) << 16) + kATmemBase +
                              s * 64u + uint32_t(part * PER_THREAD);
#pragma unroll
          for (int h8 = 0; h8 < PER_THREAD / 8; ++h8) {
            uint32_t a8[8], b8[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) {
              a8[e] = hi[8 * h8 + e];
              b8[e] = lo[8 * h8 + e];
            }
            tmemStore32x8(at + uint32_t(8 * h8), a8);
            tmemStore32x8(at + 32u + uint32_t(8 * h8), b8);
          }
          tmemStoreWait();
          tcgen05FenceBefore();
        } else {
          unsigned char *stage = aligned + s * stageBytes;
#pragma unroll
          for (int q = 0; q < PER_THREAD / 4; ++q) {
            float hi[4], lo[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const bool beyond = ragged && k0 + 4 * q + e >= p.K;
              hi[e] = beyond ? 0.0f : buf[r][4 * q + e].x;
              lo[e] = beyond ? 0.0f : buf[r][4 * q + e].y;
            }
            const uint32_t chunk = uint32_t(part * (PER_THREAD / 4) + q);
            const uint32_t at = rowOffset + ((chunk ^ uint32_t(m & 7)) << 4);
            *reinterpret_cast<float4 *>(stage + at) = make_float4(hi[0], hi[1], hi[2], hi[3]);
            *reinterpret_cast<float4 *>(stage + kABytes + at) =
                make_float4(lo[0], lo[1], lo[2], lo[3]);
          }
          // The MMA reads shared memory through the async proxy.
          fenceProxyAsync();
        }
        pending = true;
        advance(use);
        ++it;
        if (!use.have)
          go = false; // the last block: the meeting below closes it
        else if (leader)
          awaitStage(it);
      }
    }
    // The stores of the last block (none are left if a wait gave up).
    meet();
    if (leader && pending)
      mbarArrive(smemAddr(&bars->full[(it - 1) % stages]));
  } else if (warp == 1) {
    // ------------------------------- MMA issuer -------------------------------
    // The whole warp walks the loop, converged, and one elected lane issues: what
    // the instructions take (descriptors, addresses) is then uniform over the warp
    // as far as the compiler can see (4 % faster than one lane alone in a
    // divergent branch).
    {
      const bool issuer = electOne();
      const uint32_t iDesc = (1u << 4) | (2u << 7) | (2u << 10) |
                             (uint32_t(p.nPad >> 3) << 17) | (uint32_t(BM >> 4) << 24);
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
        const uint32_t dTmem = tmemBase + uint32_t(acc * kAccStride);
        for (int kb = 0; kb < kBlocks; ++kb, ++it) {
          const uint32_t s = it % stages, phase = (it / stages) & 1u;
          ok = mbarWait(smemAddr(&bars->full[s]), phase, abortFlag, p.status,
                        kStatusMmaWaitData);
          ok = __all_sync(0xffffffffu, ok);
          if (!ok)
            break;
          tcgen05FenceAfter();
          const uint32_t stage = smemBase + s * stageBytes;
          // The filter tiles are K-major: rows of 128 bytes, 8-row groups 1024
          // bytes apart; so are the image tiles when they are in shared memory.
          const uint64_t bHi = makeSmemDesc(stage + kAStage, 16, 1024);
          const uint64_t bLo = makeSmemDesc(stage + kAStage + bBytes, 16, 1024);
          if constexpr (TMEM_A) {
            const uint32_t aHi = tmemBase + kATmemBase + s * 64u, aLo = aHi + 32u;
            if (issuer && stacked) {
#pragma unroll
              for (int kk = 0; kk < BK / UMMA_K; ++kk) {
                const uint32_t col = uint32_t(kk * UMMA_K);
                const uint64_t step = uint64_t(kk * 2);
                ummaTf32TmemA(dTmem, aHi + col, bHi + step, iDescWide, (kb | kk) != 0);
                ummaTf32TmemA(dTmem, aLo + col, bHi + step, iDesc, 1);
              }
            } else if (issuer) {
#pragma unroll
              for (int kk = 0; kk < BK / UMMA_K; ++kk) {
                // 8 K-elements further: 8 columns of A, 32 bytes along a row of B.
                const uint32_t col = uint32_t(kk * UMMA_K);
                const uint64_t step = uint64_t(kk * 2);
                ummaTf32TmemA(dTmem, aLo + col, bHi + step, iDesc, (kb | kk) != 0);
                ummaTf32TmemA(dTmem, aHi + col, bLo + step, iDesc, 1);
                ummaTf32TmemA(dTmem, aHi + col, bHi + step, iDesc, 1);
              }
            }
          } else {
            const uint64_t aHi = makeSmemDesc(stage, 16, 1024);
            const uint64_t aLo = makeSmemDesc(stage + kABytes, 16, 1024);
            if (issuer && stacked) {
#pragma unroll
              for (int kk = 0; kk < BK / UMMA_K; ++kk) {
                const uint64_t step = uint64_t(kk * 2);
                ummaTf32<1>(dTmem, aHi + step, bHi + step, iDescWide, (kb | kk) != 0);
                ummaTf32<1>(dTmem, aLo + step, bHi + step, iDesc, 1);
              }
            } else if (issuer) {
#pragma unroll
              for (int kk = 0; kk < BK / UMMA_K; ++kk) {
                // 8 K-elements further: 32 bytes along a row.  The small terms first.
                const uint64_t step = uint64_t(kk * 2);
                ummaTf32<1>(dTmem, aLo + step, bHi + step, iDesc, (kb | kk) != 0);
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
    }
  } else {
    // -------------------------------- epilogue --------------------------------
    const int quad = warp & 3; // TMEM lanes [32*quad, 32*quad+32) for this warp
    const long long osN = (long long)p.NF * pixels;
    int tileIter = 0;
    for (int t = blockIdx.x; t < numTiles; t += gridDim.x, ++tileIter) {
      const int n = t / p.tilesPerImage, tp = t - n * p.tilesPerImage;
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
      const int pix = tp * BM + quad * 32 + lane;
      // Pixel `pix` of filter q: consecutive lanes write consecutive floats.
      float *dst = p.out + n * osN + pix;
      const uint32_t taddr = tmemBase + (uint32_t(quad * 32) << 16) + uint32_t(acc * kAccStride);
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
        if (pix < pixels) {
#pragma unroll
          for (int j = 0; j < 32; ++j)
            if (ch * 32 + j < p.NF)
              dst[(long long)(ch * 32 + j) * pixels] = __uint_as_float(v[j]);
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

} // namespace

extern "C" __global__ void __launch_bounds__(NUM_THREADS, 1)
    hc_conv_f32_umma(const __grid_constant__ CUtensorMap mapFHi,
                     const __grid_constant__ CUtensorMap mapFLo,
                     const __grid_constant__ HcConvParams p) {
  extern __shared__ __align__(1024) unsigned char smemRaw[];
  convF32<false>(mapFHi, mapFLo, p, smemRaw);
}

// The image operand in tensor memory: up to 128 filters.
extern "C" __global__ void __launch_bounds__(NUM_THREADS, 1)
    hc_conv_f32_umma_ta(const __grid_constant__ CUtensorMap mapFHi,
                        const __grid_constant__ CUtensorMap mapFLo,
                        const __grid_constant__ HcConvParams p) {
  extern __shared__ __align__(1024) unsigned char smemRaw[];
  convF32<true>(mapFHi, mapFLo, p, smemRaw);
}
