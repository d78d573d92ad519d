// Dense bf16 GEMM on the 5th-generation tensor cores:
//   C[M, N] = bf16( (A[M, K] @ B[K, N]) (* scale[N]) ),  fp32 accumulation,
// A, B, C row-major with explicit row pitches.
//
// It computes what the reference's dot kernels compute (python/hckernel/tests/
// test_examples.py:88-111 K-blocked, :136-155 full-K): every work-group owns
// one output tile, accumulates A-tile x B-tile products over K in a zero-
// initialised accumulator and stores the tile clipped to the matrix; tiles
// loaded past the matrix edge read as zero (python/hckernel/kernel_api.py:
// 297-342).  B is [K, N] row-major as in the reference's `b: Buffer[K, N]`.
//
// Mapping to the hardware (one persistent CTA per SM, 192 threads):
//   warp 0     TMA producer: cp.async.bulk.tensor boxes of 64 bf16 per row,
//              128-byte swizzle, into a ring of shared-memory stages; out-of-
//              range parts of a box are zero-filled by the TMA unit, which is
//              exactly the reference's zero-padded edge tile.  No cluster
//              multicast is used anywhere.
//   warp 1     allocates TMEM and issues tcgen05.mma (one thread): A is
//              K-major, B is N-major (row-major [K, N] needs no transpose),
//              the fp32 accumulator (128 lanes x 256 columns) lives in TMEM
//              and is double-buffered so the epilogue of tile i overlaps the
//              main loop of tile i+1.
//   warps 2-5  epilogue: tcgen05.ld the accumulator, optional per-column
//              scale, round to bf16 (nearest even), store clipped to M x N.
//
// PAIR = true runs two CTAs (a cluster of 2 neighbouring SMs) on one 256 x 256
// tile with tcgen05.mma.cta_group::2: each CTA stages its own 128 rows of A
// and its own 128 columns of B, so a CTA moves 32 KiB per 64-deep K-block
// instead of 48 KiB for the same flops, and the leader CTA issues the MMAs for
// both.
//
// Every mbarrier wait is bounded (hc_ptx.cuh); a wait that runs out records a
// code in `status`, raises a CTA-wide abort flag that makes all roles leave
// their loops, and the kernel exits through the normal teardown.
//
// PEERS: the epilogue writes every output tile to all destinations of `peers`
// (this GPU's copy of C and the copies of the other GPUs of a multi-GPU job,
// peer memory reached with plain stores over NVLink) - the output all-gather of
// an M- or N-sharded product done by the kernel itself.
#include "gemm_band_params.h"
#include "hc_ptx.cuh"
#include "peer_params.h"

namespace {

using namespace hc;

constexpr int BM = 128;      // accumulator rows per CTA (TMEM lanes)
constexpr int BN = 256;      // accumulator columns per tile
constexpr int BK = 64;       // K depth of one stage: 64 bf16 = one 128-byte row
constexpr int UMMA_K = 16;   // K depth of one tcgen05.mma with 16-bit inputs
constexpr int NUM_THREADS = 192;
constexpr int TMEM_COLS = 512; // two 256-column accumulators

template <bool PAIR> struct Config {
  static constexpr int kCtas = PAIR ? 2 : 1;
  static constexpr int kTileM = BM * kCtas;
  static constexpr int kBColsPerCta = BN / kCtas; // B columns a CTA stages
  static constexpr int kBChunks = kBColsPerCta / 64;
  static constexpr int kABytes = BM * BK * 2;
  static constexpr int kBChunkBytes = BK * 64 * 2;
  static constexpr int kStageBytes = kABytes + kBChunks * kBChunkBytes;
  static constexpr int kStages = PAIR ? 6 : 4;
  static constexpr uint32_t kInstrDesc =
      makeInstrDescBf16(kTileM, BN, /*aMnMajor=*/false, /*bMnMajor=*/true);
};

struct alignas(8) Barriers {
  uint64_t full[8];
  uint64_t empty[8];
  uint64_t tmemFull[2];
  uint64_t tmemEmpty[2];
  uint32_t tmemBase;
  int abortFlag;
};

struct Params {
  long long M, N, K;
  long long ldc;     // elements
  int tilesM, tilesN;
  int bandM;         // M-tiles per rasterisation band
  int vecStore;      // C base 16-byte aligned and ldc % 8 == 0
};

// The dequantising form that converts inside the GEMM kernel (BANDED):
// gemm_band_params.h describes the ring of converted bands and its counters.
using BandPlan = HcBandPlan;
constexpr int kConverterWarps = 4;
constexpr int kBandedThreads = NUM_THREADS + 32 * kConverterWarps;
constexpr int kStatusBandWait = 6;  // TMA producer waiting for a converted band
constexpr int kStatusSlotWait = 7;  // converters waiting for a consumed band

// Waits (bounded like mbarWait) until *counter >= want.
__device__ __forceinline__ bool counterWait(const unsigned *counter, unsigned want,
                                            volatile int *abortFlag, int *status, int code) {
  const unsigned long long start = globalTimerNs();
  for (uint32_t spin = 1;; ++spin) {
    unsigned v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(counter) : "memory");
    if (v >= want)
      return true;
    __nanosleep(100);
    if ((spin & 15u) == 0) {
      if (*abortFlag)
        return false;
      if (globalTimerNs() - start > kWaitLimitNs) {
        *abortFlag = 1;
        atomicCAS(status, kStatusOk, code);
        return false;
      }
    }
  }
}

// Generic-proxy writes to global memory before, async-proxy (TMA) reads after.
__device__ __forceinline__ void fenceProxyAsyncAll() {
  asm volatile("fence.proxy.async;" ::: "memory");
}

// int8 -> bf16, exact, two at a time: the bytes of `word` picked by `sel` become
// the low bytes of 0x43xx.  With bit 7 of the byte cleared that is 128 + (b & 127);
// subtracting 0x4300 (128) or, for a negative byte, 0x4380 (256) gives b.
__device__ __forceinline__ uint32_t bytesToBf16(uint32_t word, uint32_t sel) {
  const uint32_t t = __byte_perm(word, 0x43434343u, sel);
  const uint32_t biased = t & 0xFF7FFF7Fu;
  const uint32_t bias = t & 0xFF80FF80u;
  const __nv_bfloat162 d = __hsub2(*reinterpret_cast<const __nv_bfloat162 *>(&biased),
                                   *reinterpret_cast<const __nv_bfloat162 *>(&bias));
  return *reinterpret_cast<const uint32_t *>(&d);
}

// The first bands are needed before any tile can start, when the epilogue warps
// have nothing to do yet: they convert a share of those bands too.
constexpr int kHelpedBands = 2;

// Warp `me` of `total` converts rows me, me + total, ... of the band, eight rows
// at a time (the weights come from HBM: what is in flight per warp sets the
// pace); a lane takes 16 weights (16 bytes in, 32 out) per row.  Then it reports
// its share as written.
__device__ __forceinline__ void convertShare(const Params &p, const BandPlan &bp, int band,
                                             unsigned me, unsigned total, int lane) {
  const long long bandCols = (long long)bp.bandTiles * BN;
  const long long col0 = (long long)band * bandCols;
  const int packets = int(min(bandCols, p.N - col0) >> 4);
  const int8_t *src = bp.w + col0;
  __nv_bfloat16 *dst =
      static_cast<__nv_bfloat16 *>(bp.ring) + (long long)(band % bp.slots) * p.K * bandCols;
  constexpr int R = 8;
  for (long long r = me; r < p.K; r += (long long)total * R) {
    for (int pk = lane; pk < packets; pk += 32) {
      int4 q[R];
#pragma unroll
      for (int i = 0; i < R; ++i) {
        const long long row = r + (long long)i * total;
        q[i] = make_int4(0, 0, 0, 0);
        if (row < p.K)
          asm volatile("ld.global.nc.L1::no_allocate.v4.s32 {%0, %1, %2, %3}, [%4];"
                       : "=r"(q[i].x), "=r"(q[i].y), "=r"(q[i].z), "=r"(q[i].w)
                       : "l"(reinterpret_cast<const int4 *>(src + row * bp.ldw) + pk));
      }
#pragma unroll
      for (int i = 0; i < R; ++i) {
        const long long row = r + (long long)i * total;
        if (row < p.K) {
          const uint32_t words[4] = {uint32_t(q[i].x), uint32_t(q[i].y), uint32_t(q[i].z),
                                     uint32_t(q[i].w)};
          uint32_t o[8];
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            o[2 * j] = bytesToBf16(words[j], 0x5140u);     // bytes 0 and 1
            o[2 * j + 1] = bytesToBf16(words[j], 0x7362u); // bytes 2 and 3
          }
          uint4 *out = reinterpret_cast<uint4 *>(dst + row * bandCols) + 2 * pk;
          out[0] = make_uint4(o[0], o[1], o[2], o[3]);
          out[1] = make_uint4(o[4], o[5], o[6], o[7]);
        }
      }
    }
  }
  // This warp's share is written: visible to the TMA reads of every CTA.
  fenceProxyAsyncAll();
  __threadfence();
  __syncwarp();
  if (lane == 0)
    atomicAdd(bp.converted + band, 1u);
}

// Tile t of the band-by-band order: bands of `bandTiles` tile columns, inside a
// band the tile columns run fastest (the tiles in flight share rows of A).
__device__ __forceinline__ void bandTileCoords(int t, const Params &p, const BandPlan &bp,
                                               int &tm, int &tn, int &band) {
  const int full = p.tilesM * bp.bandTiles;
  band = t / full;
  const int rem = t - band * full;
  const int cols = min(bp.bandTiles, p.tilesN - band * bp.bandTiles);
  tm = rem / cols;
  tn = band * bp.bandTiles + rem % cols;
}

__device__ __forceinline__ void tileCoords(int t, const Params &p, int &tm,
                                           int &tn) {
  const int perBand = p.bandM * p.tilesN;
  const int band = t / perBand;
  const int rem = t - band * perBand;
  const int rowsInBand = min(p.bandM, p.tilesM - band * p.bandM);
  tm = band * p.bandM + rem % rowsInBand;
  tn = rem / rowsInBand;
}

template <bool PAIR, bool SCALED, bool PEERS = false, bool BANDED = false>
__device__ __forceinline__ void
gemmUmma(const CUtensorMap *mapA, const CUtensorMap *mapB,
         __nv_bfloat16 *__restrict__ c, const float *__restrict__ scale,
         const Params &p, int *status, unsigned char *smemRaw,
         const HcPeerDsts *peers = nullptr, const BandPlan *bp = nullptr) {
  using Cfg = Config<PAIR>;
  // The swizzled stages need 1024-byte alignment.
  const uint32_t smemBase = (smemAddr(smemRaw) + 1023u) & ~1023u;
  Barriers *bars = reinterpret_cast<Barriers *>(
      smemRaw + (smemBase - smemAddr(smemRaw)) + Cfg::kStages * Cfg::kStageBytes);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t ctaRank = PAIR ? clusterCtaRank() : 0u;
  const bool leader = ctaRank == 0;
  volatile int *abortFlag = &bars->abortFlag;

  if (threadIdx.x == 0) {
    for (int s = 0; s < Cfg::kStages; ++s) {
      mbarInit(smemAddr(&bars->full[s]), 1);          // the (leader's) expect_tx
      mbarInit(smemAddr(&bars->empty[s]), 1);         // one MMA commit
    }
    for (int a = 0; a < 2; ++a) {
      mbarInit(smemAddr(&bars->tmemFull[a]), 1);
      mbarInit(smemAddr(&bars->tmemEmpty[a]), 4 * Cfg::kCtas); // epilogue warps
    }
    bars->abortFlag = 0;
    fenceBarrierInit();
    prefetchTensorMap(mapA);
    prefetchTensorMap(mapB);
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

  const int kBlocks = int((p.K + BK - 1) / BK);
  const int numTiles = p.tilesM * p.tilesN;
  const int firstTile = PAIR ? (blockIdx.x >> 1) : blockIdx.x;
  const int tileStep = PAIR ? (gridDim.x >> 1) : gridDim.x;

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    if (lane == 0) {
      uint32_t it = 0;
      int readyBand = -1;
      for (int t = firstTile; t < numTiles && !*abortFlag; t += tileStep) {
        int tm, tn;
        int bRow0 = 0; // row of B's map at K block 0
        if constexpr (BANDED) {
          int band;
          bandTileCoords(t, p, *bp, tm, tn, band);
          if (band != readyBand) {
            // Every converter warp of the grid has written its share of the band.
            const unsigned writers =
                gridDim.x * (band < kHelpedBands ? kConverterWarps + 4 : kConverterWarps);
            if (!counterWait(bp->converted + band, writers, abortFlag, status, kStatusBandWait))
              break;
            fenceProxyAsyncAll();
            readyBand = band;
          }
          bRow0 = (band % bp->slots) * int(p.K);
          tn -= band * bp->bandTiles; // the column inside the band's buffer
        } else {
          tileCoords(t, p, tm, tn);
        }
        const int row0 = tm * Cfg::kTileM + int(ctaRank) * BM;
        const int col0 = tn * BN + int(ctaRank) * Cfg::kBColsPerCta;
        for (int kb = 0; kb < kBlocks; ++kb, ++it) {
          const uint32_t s = it % Cfg::kStages;
          const uint32_t phase = (it / Cfg::kStages) & 1u;
          if (!mbarWait(smemAddr(&bars->empty[s]), phase ^ 1u, abortFlag,
                        status, kStatusProducerWait))
            break;
          // Completion bytes of both CTAs are counted on the leader's barrier.
          uint32_t fullBar = smemAddr(&bars->full[s]);
          if constexpr (PAIR)
            fullBar = mapSharedToCta(fullBar, 0);
          const uint32_t stage = smemBase + s * Cfg::kStageBytes;
          if constexpr (PAIR) {
            // Only the leader arrives, expecting the bytes of both CTAs.  The
            // peer's copies may land before this arrival; they only drive the
            // barrier's byte count negative for a moment, and the phase cannot
            // complete before the leader has arrived.  (A remote
            // arrive.expect_tx from the peer instead serialised the stages and
            // halved the throughput.)
            if (leader)
              mbarExpectTx(smemAddr(&bars->full[s]), 2 * Cfg::kStageBytes);
            tmaLoad2DPair(stage, mapA, fullBar, kb * BK, row0);
            for (int ch = 0; ch < Cfg::kBChunks; ++ch)
              tmaLoad2DPair(stage + Cfg::kABytes + ch * Cfg::kBChunkBytes, mapB,
                            fullBar, col0 + ch * 64, bRow0 + kb * BK);
          } else {
            mbarExpectTx(fullBar, Cfg::kStageBytes);
            tmaLoad2D(stage, mapA, fullBar, kb * BK, row0);
            for (int ch = 0; ch < Cfg::kBChunks; ++ch)
              tmaLoad2D(stage + Cfg::kABytes + ch * Cfg::kBChunkBytes, mapB,
                        fullBar, col0 + ch * 64, kb * BK);
          }
        }
      }
      // Tail: the commits that free the last stages must have landed in this
      // CTA's barriers before its shared memory goes away.
      for (int i = 0; i < Cfg::kStages && !*abortFlag; ++i, ++it) {
        const uint32_t s = it % Cfg::kStages;
        const uint32_t phase = (it / Cfg::kStages) & 1u;
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
      for (int t = firstTile; t < numTiles && !*abortFlag;
           t += tileStep, ++tileIter) {
        const int acc = tileIter & 1;
        const uint32_t accPhase = (tileIter >> 1) & 1u;
        if (!mbarWait(smemAddr(&bars->tmemEmpty[acc]), accPhase ^ 1u, abortFlag,
                      status, kStatusMmaWaitTmem))
          break;
        tcgen05FenceAfter();
        const uint32_t dTmem = tmemBase + uint32_t(acc * BN);
        bool ok = true;
        for (int kb = 0; kb < kBlocks; ++kb, ++it) {
          const uint32_t s = it % Cfg::kStages;
          const uint32_t phase = (it / Cfg::kStages) & 1u;
          if (!mbarWait(smemAddr(&bars->full[s]), phase, abortFlag, status,
                        kStatusMmaWaitData)) {
            ok = false;
            break;
          }
          tcgen05FenceAfter();
          const uint32_t stage = smemBase + s * Cfg::kStageBytes;
          // A: K-major, rows 128 bytes apart, 8-row groups 1024 bytes apart.
          const uint64_t aDesc = makeSmemDesc(stage, 16, 1024);
          // B: N-major, 64-column chunks BK*128 bytes apart (leading), 8-deep
          // K groups 1024 bytes apart (stride).
          const uint64_t bDesc =
              makeSmemDesc(stage + Cfg::kABytes, Cfg::kBChunkBytes, 1024);
#pragma unroll
          for (int kk = 0; kk < BK / UMMA_K; ++kk) {
            // 16 K-elements further: 32 bytes along an A row, 16 rows of
            // 128 bytes down a B chunk.
            umma<Cfg::kCtas>(dTmem, aDesc + uint64_t(kk * 2),
                             bDesc + uint64_t(kk * 128), Cfg::kInstrDesc,
                             (kb | kk) != 0);
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
  } else if (warp < NUM_THREADS / 32) {
    // -------------------------------- epilogue --------------------------------
    const int quad = warp & 3; // TMEM lanes [32*quad, 32*quad+32) for this warp
    uint32_t tmemEmptyBar[2];
    for (int a = 0; a < 2; ++a) {
      tmemEmptyBar[a] = smemAddr(&bars->tmemEmpty[a]);
      if constexpr (PAIR)
        tmemEmptyBar[a] = mapSharedToCta(tmemEmptyBar[a], 0);
    }
    if constexpr (BANDED) {
      // Nothing to drain yet: convert a share of the first bands (warps 2..5 take
      // the places after the converter warps).
      for (int band = 0; band < min(kHelpedBands, bp->numBands); ++band)
        convertShare(p, *bp, band,
                     blockIdx.x * (kConverterWarps + 4) + unsigned(kConverterWarps + warp - 2),
                     gridDim.x * (kConverterWarps + 4), lane);
    }
    int tileIter = 0;
    for (int t = firstTile; t < numTiles; t += tileStep, ++tileIter) {
      int tm, tn, band = 0;
      if constexpr (BANDED)
        bandTileCoords(t, p, *bp, tm, tn, band);
      else
        tileCoords(t, p, tm, tn);
      const int acc = tileIter & 1;
      const uint32_t accPhase = (tileIter >> 1) & 1u;
      bool ok = true;
      if (lane == 0)
        ok = mbarWait(smemAddr(&bars->tmemFull[acc]), accPhase, abortFlag,
                      status, kStatusEpilogueWait);
      ok = __shfl_sync(0xffffffffu, ok, 0);
      if (!ok)
        break;
      tcgen05FenceAfter();
      if constexpr (BANDED) {
        // The tile's MMAs are complete: nothing reads its part of the band any more.
        if (leader && quad == 0 && lane == 0)
          atomicAdd(bp->consumed + band, 1u);
      }
      const long long row =
          (long long)tm * Cfg::kTileM + int(ctaRank) * BM + quad * 32 + lane;
      const long long colBase = (long long)tn * BN;
      const uint32_t taddr =
          tmemBase + (uint32_t(quad * 32) << 16) + uint32_t(acc * BN);
      const int destinations = PEERS ? peers->count : 1;
#pragma unroll 1
      for (int ch = 0; ch < BN / 32; ++ch) {
        uint32_t v[32];
        __syncwarp(); // tcgen05.ld needs the whole warp, converged
        tmemLoad32x32(taddr + uint32_t(ch * 32), v);
        tmemLoadWait();
        const long long col = colBase + ch * 32;
        if (col >= p.N) // the same for the whole warp
          break;
        if (row < p.M) { // per lane: only loads and stores are predicated
          float f[32];
#pragma unroll
          for (int j = 0; j < 32; ++j)
            f[j] = __uint_as_float(v[j]);
          if constexpr (SCALED) {
            if (col + 32 <= p.N) {
#pragma unroll
              for (int j = 0; j < 32; j += 4) {
                const float4 s =
                    __ldg(reinterpret_cast<const float4 *>(scale + col + j));
                f[j] *= s.x;
                f[j + 1] *= s.y;
                f[j + 2] *= s.z;
                f[j + 3] *= s.w;
              }
            } else {
#pragma unroll
              for (int j = 0; j < 32; ++j)
                if (col + j < p.N)
                  f[j] *= __ldg(scale + col + j);
            }
          }
          uint32_t w[16]; // the 32 values rounded to bf16, two per word
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            __nv_bfloat162 h = __floats2bfloat162_rn(f[2 * j], f[2 * j + 1]);
            w[j] = *reinterpret_cast<uint32_t *>(&h);
          }
          for (int d = 0; d < destinations; ++d) {
            __nv_bfloat16 *crow =
                (PEERS ? static_cast<__nv_bfloat16 *>(peers->base[d]) : c) + row * p.ldc;
            if (p.vecStore && col + 32 <= p.N) {
              uint4 *dst = reinterpret_cast<uint4 *>(crow + col);
#pragma unroll
              for (int q = 0; q < 4; ++q)
                dst[q] = make_uint4(w[4 * q], w[4 * q + 1], w[4 * q + 2], w[4 * q + 3]);
            } else {
#pragma unroll
              for (int j = 0; j < 32; ++j)
                if (col + j < p.N)
                  crow[col + j] = __ushort_as_bfloat16(
                      static_cast<unsigned short>(j & 1 ? w[j >> 1] >> 16 : w[j >> 1] & 0xffffu));
            }
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

  else if constexpr (BANDED) {
    // ------------------------------- converters -------------------------------
    // Every band in turn, as soon as its slot of the ring is free.
    for (int band = 0; band < bp->numBands && !*abortFlag; ++band) {
      if (band >= bp->slots) {
        // The slot still belongs to the band `slots` before until its tiles are done.
        const int old = band - bp->slots;
        const unsigned tiles =
            unsigned(p.tilesM * min(bp->bandTiles, p.tilesN - old * bp->bandTiles));
        bool ok = true;
        if (lane == 0)
          ok = counterWait(bp->consumed + old, tiles, abortFlag, status, kStatusSlotWait);
        if (!__shfl_sync(0xffffffffu, ok, 0))
          break;
      }
      const unsigned width = band < kHelpedBands ? kConverterWarps + 4 : kConverterWarps;
      convertShare(p, *bp, band, blockIdx.x * width + unsigned(warp - NUM_THREADS / 32),
                   gridDim.x * width, lane);
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

// Dynamic shared memory: stages + barriers + 1 KiB alignment slack; the host
// computes the same numbers (kernels_api.cpp).
#define HC_GEMM_ARGS                                                           \
  const __grid_constant__ CUtensorMap mapA,                                    \
      const __grid_constant__ CUtensorMap mapB, __nv_bfloat16 *c,              \
      const float *scale, long long M, long long N, long long K,               \
      long long ldc, int tilesM, int tilesN, int bandM, int vecStore,          \
      int *status

#define HC_GEMM_BODY(PAIR, SCALED)                                             \
  extern __shared__ __align__(1024) unsigned char smemRaw[];                   \
  Params p{M, N, K, ldc, tilesM, tilesN, bandM, vecStore};                     \
  gemmUmma<PAIR, SCALED>(&mapA, &mapB, c, scale, p, status, smemRaw);

extern "C" __global__ void __launch_bounds__(NUM_THREADS, 1)
    hc_gemm_bf16_umma(HC_GEMM_ARGS) {
  HC_GEMM_BODY(false, false)
}

extern "C" __global__ void __launch_bounds__(NUM_THREADS, 1)
    hc_gemm_bf16_umma_scaled(HC_GEMM_ARGS) {
  HC_GEMM_BODY(false, true)
}

extern "C" __global__ void __cluster_dims__(2, 1, 1)
    __launch_bounds__(NUM_THREADS, 1) hc_gemm_bf16_umma_pair(HC_GEMM_ARGS) {
  HC_GEMM_BODY(true, false)
}

extern "C" __global__ void __cluster_dims__(2, 1, 1)
    __launch_bounds__(NUM_THREADS, 1)
        hc_gemm_bf16_umma_pair_scaled(HC_GEMM_ARGS) {
  HC_GEMM_BODY(true, true)
}

// The dequantising GEMM that converts its weights inside the kernel, band by
// band (BandPlan): mapB covers the ring of converted bands, [slots * K, bandCols].
extern "C" __global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kBandedThreads, 1)
    hc_gemm_w8a16_umma_banded(HC_GEMM_ARGS, const __grid_constant__ BandPlan plan) {
  extern __shared__ __align__(1024) unsigned char smemRaw[];
  Params p{M, N, K, ldc, tilesM, tilesN, bandM, vecStore};
  gemmUmma<true, true, false, true>(&mapA, &mapB, c, scale, p, status, smemRaw, nullptr, &plan);
}

// The same four kernels writing every tile to all destinations of `peers`.
#define HC_GEMM_PEERS_BODY(PAIR, SCALED)                                       \
  extern __shared__ __align__(1024) unsigned char smemRaw[];                   \
  Params p{M, N, K, ldc, tilesM, tilesN, bandM, vecStore};                     \
  gemmUmma<PAIR, SCALED, true>(&mapA, &mapB, c, scale, p, status, smemRaw,     \
                               &peers);

extern "C" __global__ void __launch_bounds__(NUM_THREADS, 1)
    hc_gemm_bf16_umma_peers(HC_GEMM_ARGS, const __grid_constant__ HcPeerDsts peers) {
  HC_GEMM_PEERS_BODY(false, false)
}

extern "C" __global__ void __launch_bounds__(NUM_THREADS, 1)
    hc_gemm_bf16_umma_scaled_peers(HC_GEMM_ARGS,
                                   const __grid_constant__ HcPeerDsts peers) {
  HC_GEMM_PEERS_BODY(false, true)
}

extern "C" __global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(NUM_THREADS, 1)
    hc_gemm_bf16_umma_pair_peers(HC_GEMM_ARGS, const __grid_constant__ HcPeerDsts peers) {
  HC_GEMM_PEERS_BODY(true, false)
}

extern "C" __global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(NUM_THREADS, 1)
    hc_gemm_bf16_umma_pair_scaled_peers(HC_GEMM_ARGS,
                                        const __grid_constant__ HcPeerDsts peers) {
  HC_GEMM_PEERS_BODY(true, true)
}
