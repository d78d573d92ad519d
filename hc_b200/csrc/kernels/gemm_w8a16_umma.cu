// int8 weight-only dequant GEMM with the conversion inside the pipeline:
//   out[m, n] = bf16( scale[n] * sum_k a[m, k] * float(w[k, n]) )
// a bf16 [M, K], w int8 [K, N] row-major (the reference's `b: Buffer[K, N]`
// convention, python/hckernel/tests/test_examples.py:91), scale fp32 [N], out
// bf16 [M, N]; fp32 accumulation.  The same sums, in the same order, as
// converting w to bf16 first (dequant_w8.cu) and multiplying with the scaled
// CTA-pair kernel of gemm_bf16_umma.cu - results are bit for bit the same -
// but the converted weights never exist in global memory: no scratch matrix,
// no pass that reads 1 and writes 2 bytes per weight, and the weight tiles
// cross HBM, L2 and the SM boundary as one byte per element instead of two.
//
// A cluster of two CTAs works on one 256 x 256 output tile with
// tcgen05.mma.cta_group::2 (as hc_gemm_bf16_umma_pair).  Per CTA, 480 threads:
//   warp 0     TMA producer of A: per 64-deep K block its 128 rows (bf16, 128-byte
//              swizzle, completion counted on the leader CTA's barrier; no
//              multicast);
//   warp 14    TMA producer of w: its 64 x 128 tile as raw bytes (no swizzle,
//              completion on this CTA's own `raw` barrier) into a ring of eight
//              slots of its own - deeper than the stages, because the way of a
//              weight into an MMA is the longest; no multicast anywhere;
//   warps 6-13 converters, four groups of two warps that take the K blocks in
//              turn: 16 weights per 16-byte shared-memory load -> two
//              16-byte stores of bf16 into the stage, in the N-major 128-byte-
//              swizzled layout a TMA box of bf16 would have produced
//              (int8 -> bf16 by byte permute and one packed subtract, exact);
//              fence.proxy.async, then one arrival per warp on the leader CTA's
//              `full` barrier (release at CTA scope: the data is read by this
//              SM's own tensor core; a cluster-scope release cost 1000 cycles
//              per arrival); the warps run ahead of the MMAs by up to the ring
//              of stages;
//   warp 1     (leader CTA) MMA issuer, M256 N256 K16, four per K block;
//   warps 2-5  epilogue: tcgen05.ld, per-column scale, bf16, 16-byte stores.
// Every weight tile is converted once per 256-row block of activations - work
// the CUDA cores do while the tensor cores run the block before.
//
// Measured at 4096 x 8192 x 8192: 0.51-0.52 ms, against 0.42-0.45 ms for the
// conversion pass plus the bf16 kernel: per K block the shared-memory port now
// carries 80 KiB (A and the bytes of w in, the bytes out again, bf16 in, A and
// bf16 out to the tensor core) where the bf16 kernel carries 64.  It is therefore not the default (option
// "w8a16_variant" = 2 selects it): it is the form for callers that cannot spare
// the 2 bytes per weight of scratch memory.
//
// Every mbarrier wait is bounded (hc_ptx.cuh); the roles synchronise through
// mbarriers alone, so a wait that gives up raises the abort flag and every
// role leaves its loop at its next wait.
#include "hc_ptx.cuh"

namespace {

using namespace hc;

constexpr int BM = 128;    // accumulator rows per CTA (TMEM lanes)
constexpr int BN = 256;    // accumulator columns per tile
constexpr int BK = 64;     // K depth of one stage
constexpr int UMMA_K = 16;
constexpr int CONVERTER_WARPS = 8;
constexpr int RAW_PRODUCER_WARP = 6 + CONVERTER_WARPS;
constexpr int NUM_THREADS = 32 * (7 + CONVERTER_WARPS);
constexpr int TMEM_COLS = 512;
constexpr int kTileM = 2 * BM;
constexpr int kBCols = BN / 2;             // columns of w a CTA stages
// The converter warps work in groups that take the K blocks in turn, so that a
// group has GROUPS block times for one block.
constexpr int GROUPS = 4;
constexpr int GROUP_WARPS = CONVERTER_WARPS / GROUPS;
constexpr int PACKETS = BK * kBCols / 16 / (32 * GROUP_WARPS); // 16-weight packets per thread: 8
constexpr int kABytes = BM * BK * 2;       // 16 KiB
constexpr int kBChunkBytes = BK * 64 * 2;  // 64 columns of bf16, 64 deep: 8 KiB
constexpr int kBBytes = 2 * kBChunkBytes;  // 16 KiB
constexpr int kStageBytes = kABytes + kBBytes; // 32 KiB: A and the converted B
constexpr int kStages = 5;
// The int8 tiles wait in a ring of their own, deeper than the stages: what must be
// in flight to cover the latency of L2 under this kernel's traffic is more than
// registers can hold, so TMA brings the bytes and the converters read them from
// shared memory.
constexpr int kRawBytes = BK * kBCols; // 8 KiB
constexpr int kRawSlots = 8;

constexpr uint32_t kInstrDesc = makeInstrDescBf16(kTileM, BN, /*aMnMajor=*/false,
                                                  /*bMnMajor=*/true);

struct alignas(8) Barriers {
  uint64_t full[kStages];  // leader CTA: A of both CTAs landed, both CTAs' B converted
  uint64_t empty[kStages]; // the MMAs that read the stage are done (both CTAs)
  uint64_t raw[kRawSlots];      // this CTA: the int8 tile landed
  uint64_t rawEmpty[kRawSlots]; // this CTA: the group that converts the tile has read it
  uint64_t tmemFull[2];
  uint64_t tmemEmpty[2];
  uint32_t tmemBase;
  int abortFlag;
};

enum : int { kStatusConverterWait = 7 }; // the converters waiting for an int8 tile

struct Params {
  long long M, N, K;
  long long ldc;
  int tilesM, tilesN;
  int bandM;
  int vecStore;
};

__device__ __forceinline__ void tileCoords(int t, const Params &p, int &tm, int &tn) {
  const int perBand = p.bandM * p.tilesN;
  const int band = t / perBand;
  const int rem = t - band * perBand;
  const int rowsInBand = min(p.bandM, p.tilesM - band * p.bandM);
  tm = band * p.bandM + rem % rowsInBand;
  tn = rem / rowsInBand;
}

// Which 16-weight packet of a 64 x 128 tile has number `id` (0..511): row k and
// packet column 0..7.  32 consecutive numbers cover four rows, as a warp's load
// wants it (whole 128-byte rows); within them, 8 consecutive numbers are the four
// packets of one 64-column chunk in two neighbouring rows, whose 16-byte slots in
// the swizzled stage fall into eight different bank groups - a 16-byte store is
// served eight lanes at a time.
__device__ __forceinline__ int rowOfPacket(int id) {
  return 4 * (id >> 5) + 2 * ((id >> 4) & 1) + ((id >> 2) & 1);
}
__device__ __forceinline__ int columnOfPacket(int id) { return 4 * ((id >> 3) & 1) + (id & 3); }

// Two int8 (the bytes `sel` picks out of `word`) -> two bf16, exactly (see
// dequant_w8.cu: the byte under exponent 0x43, minus 128 or 256).
__device__ __forceinline__ uint32_t int8PairToBf16(uint32_t word, uint32_t sel) {
  const uint32_t t = __byte_perm(word, 0x43434343u, sel);
  const uint32_t biased = t & 0xFF7FFF7Fu;
  const uint32_t bias = t & 0xFF80FF80u;
  const __nv_bfloat162 d = __hsub2(*reinterpret_cast<const __nv_bfloat162 *>(&biased),
                                   *reinterpret_cast<const __nv_bfloat162 *>(&bias));
  return *reinterpret_cast<const uint32_t *>(&d);
}

} // namespace

extern "C" __global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(NUM_THREADS, 1)
    hc_gemm_w8a16_umma_pair(const __grid_constant__ CUtensorMap mapA,
                            const __grid_constant__ CUtensorMap mapW,
                            __nv_bfloat16 *__restrict__ c, const float *__restrict__ scale,
                            long long M, long long N, long long K, long long ldc, int tilesM,
                            int tilesN, int bandM, int vecStore, int *status) {
  extern __shared__ __align__(1024) unsigned char smemRaw[];
  const Params p{M, N, K, ldc, tilesM, tilesN, bandM, vecStore};
  const uint32_t smemBase = (smemAddr(smemRaw) + 1023u) & ~1023u;
  unsigned char *aligned = smemRaw + (smemBase - smemAddr(smemRaw));
  unsigned char *rawRing = aligned + kStages * kStageBytes;
  Barriers *bars = reinterpret_cast<Barriers *>(rawRing + kRawSlots * kRawBytes);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t ctaRank = clusterCtaRank();
  const bool leaderCta = ctaRank == 0;
  volatile int *abortFlag = &bars->abortFlag;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      // The leader's expect_tx for both CTAs' A, and one report per converter warp of
      // both CTAs.
      mbarInit(smemAddr(&bars->full[s]), 1 + 2 * GROUP_WARPS);
      mbarInit(smemAddr(&bars->empty[s]), 1);
    }
    for (int q = 0; q < kRawSlots; ++q) {
      mbarInit(smemAddr(&bars->raw[q]), 1);
      mbarInit(smemAddr(&bars->rawEmpty[q]), GROUP_WARPS);
    }
    for (int a = 0; a < 2; ++a) {
      mbarInit(smemAddr(&bars->tmemFull[a]), 1);
      mbarInit(smemAddr(&bars->tmemEmpty[a]), 8); // epilogue warps of both CTAs
    }
    bars->abortFlag = 0;
    fenceBarrierInit();
    prefetchTensorMap(&mapA);
    prefetchTensorMap(&mapW);
  }
  if (warp == 1) {
    tmemAlloc<2>(smemAddr(&bars->tmemBase), TMEM_COLS);
    tmemRelinquish<2>();
  }
  tcgen05FenceBefore();
  clusterSync();
  tcgen05FenceAfter();
  const uint32_t tmemBase = bars->tmemBase;

  const int kBlocks = int((p.K + BK - 1) / BK);
  const int numTiles = p.tilesM * p.tilesN;
  const int firstTile = blockIdx.x >> 1, tileStep = gridDim.x >> 1;

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    if (lane == 0) {
      uint32_t it = 0;
      for (int t = firstTile; t < numTiles && !*abortFlag; t += tileStep) {
        int tm, tn;
        tileCoords(t, p, tm, tn);
        const int row0 = tm * kTileM + int(ctaRank) * BM;
        for (int kb = 0; kb < kBlocks; ++kb, ++it) {
          const uint32_t s = it % kStages, phase = (it / kStages) & 1u;
          if (!mbarWait(smemAddr(&bars->empty[s]), phase ^ 1u, abortFlag, status,
                        kStatusProducerWait))
            break;
          const uint32_t stage = smemBase + s * kStageBytes;
          // A: completion bytes of both CTAs are counted on the leader's barrier,
          // and only the leader arrives, expecting the bytes of both.
          const uint32_t fullBar = mapSharedToCta(smemAddr(&bars->full[s]), 0);
          if (leaderCta)
            mbarExpectTx(smemAddr(&bars->full[s]), 2 * kABytes);
          tmaLoad2DPair(stage, &mapA, fullBar, kb * BK, row0);
        }
      }
      // Tail: the commits that free the last stages must have landed in this
      // CTA's barriers before its shared memory goes away.
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
  } else if (warp == RAW_PRODUCER_WARP) {
    // ------------------------- TMA producer of the int8 tiles -------------------------
    if (lane == 0) {
      uint32_t it = 0;
      for (int t = firstTile; t < numTiles && !*abortFlag; t += tileStep) {
        int tm, tn;
        tileCoords(t, p, tm, tn);
        const int col0 = tn * BN + int(ctaRank) * kBCols;
        for (int kb = 0; kb < kBlocks; ++kb, ++it) {
          const uint32_t q = it % kRawSlots, phase = (it / kRawSlots) & 1u;
          if (!mbarWait(smemAddr(&bars->rawEmpty[q]), phase ^ 1u, abortFlag, status,
                        kStatusProducerWait))
            break;
          // The weights as bytes: rows of 128 bytes, no swizzle, this CTA's own barrier;
          // past K or N the box is zero-filled.
          const uint32_t rawBar = smemAddr(&bars->raw[q]);
          mbarExpectTx(rawBar, kRawBytes);
          tmaLoad2D(smemBase + kStages * kStageBytes + q * kRawBytes, &mapW, rawBar, col0,
                    kb * BK);
        }
      }
      // Nothing may still be landing when this CTA's shared memory goes away: the
      // converters read every tile before they finish (the teardown's cluster
      // barrier waits for them); after a wait that gave up, give the copies time.
      if (*abortFlag) {
        const unsigned long long t0 = globalTimerNs();
        while (globalTimerNs() - t0 < 1000000ull) {
        }
      }
    }
  } else if (warp >= 6) {
    // -------------------------------- converters --------------------------------
    // The eight warps form four groups that take the K blocks in turn; a thread owns
    // eight 16-weight packets of its group's tile.  When the tile has landed and the
    // stage is free it reads them from the ring of int8 tiles, converts them and
    // stores the bf16 where a TMA box of bf16 would have put them.  What a warp does
    // per block besides its packets (waiting, fencing, reporting) is done a quarter
    // as often per warp, and four blocks are in the making at once.
    const int group = (warp - 6) / GROUP_WARPS;              // takes blocks group, group + GROUPS ...
    const int tid = threadIdx.x - (6 + group * GROUP_WARPS) * 32; // 0 .. 32 * GROUP_WARPS - 1
    // What does not change from block to block, per packet of this thread: where it
    // lies in the tile of w (row k, byte column) and in the stage (two 16-byte slots
    // of row k in the chunk of 64 columns pkt / 4, swizzled with the row).
    uint32_t rawOf[PACKETS], slotA[PACKETS], slotB[PACKETS];
#pragma unroll
    for (int i = 0; i < PACKETS; ++i) {
      const int id = tid + 32 * GROUP_WARPS * i;
      const int k = rowOfPacket(id), pkt = columnOfPacket(id);
      rawOf[i] = uint32_t(k * kBCols + pkt * 16);
      const uint32_t base = uint32_t(kABytes + (pkt >> 2) * kBChunkBytes + k * 128);
      const uint32_t slot = uint32_t(pkt & 3) * 2u, x = uint32_t(k & 7);
      slotA[i] = base + ((slot ^ x) << 4);
      slotB[i] = base + (((slot + 1u) ^ x) << 4);
    }
    int myTiles = 0;
    for (int t = firstTile; t < numTiles; t += tileStep)
      ++myTiles;
    const uint32_t blocks = uint32_t(myTiles) * uint32_t(kBlocks);
    for (uint32_t it = uint32_t(group); it < blocks; it += GROUPS) {
      const uint32_t s = it % kStages, phase = (it / kStages) & 1u;
      const uint32_t q = it % kRawSlots, rawPhase = (it / kRawSlots) & 1u;
      bool ok = true;
      if (lane == 0)
        // The tile has landed, and the MMAs that read the stage before are done.
        ok = mbarWait(smemAddr(&bars->raw[q]), rawPhase, abortFlag, status,
                      kStatusConverterWait) &&
             mbarWait(smemAddr(&bars->empty[s]), phase ^ 1u, abortFlag, status,
                      kStatusConverterWait);
      ok = __shfl_sync(0xffffffffu, ok, 0);
      if (!ok)
        break;
      const unsigned char *raw = rawRing + q * kRawBytes;
      unsigned char *stage = aligned + s * kStageBytes;
      int4 loaded[PACKETS];
#pragma unroll
      for (int i = 0; i < PACKETS; ++i)
        loaded[i] = *reinterpret_cast<const int4 *>(raw + rawOf[i]);
#pragma unroll
      for (int i = 0; i < PACKETS; ++i) {
        const int4 v = loaded[i];
        const uint32_t words[4] = {uint32_t(v.x), uint32_t(v.y), uint32_t(v.z), uint32_t(v.w)};
        uint32_t o[8];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          o[2 * j] = int8PairToBf16(words[j], 0x5140u);     // bytes 0 and 1
          o[2 * j + 1] = int8PairToBf16(words[j], 0x7362u); // bytes 2 and 3
        }
        *reinterpret_cast<uint4 *>(stage + slotA[i]) = make_uint4(o[0], o[1], o[2], o[3]);
        *reinterpret_cast<uint4 *>(stage + slotB[i]) = make_uint4(o[4], o[5], o[6], o[7]);
      }
      // The MMA reads shared memory through the async proxy.
      fenceProxyAsync();
      __syncwarp();
      if (lane == 0) {
        // Straight to the leader CTA's barrier (release at CTA scope); the slot of
        // the int8 tile is free again.
        mbarArriveRemote(mapSharedToCta(smemAddr(&bars->full[s]), 0));
        mbarArrive(smemAddr(&bars->rawEmpty[q]));
      }
    }
  } else if (warp == 1) {
    // ------------------------------- MMA issuer -------------------------------
    if (lane == 0 && leaderCta) {
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
          // A: K-major, rows 128 bytes apart, 8-row groups 1024 bytes apart.
          const uint64_t aDesc = makeSmemDesc(stage, 16, 1024);
          // B: N-major, 64-column chunks BK*128 bytes apart (leading), 8-deep
          // K groups 1024 bytes apart (stride).
          const uint64_t bDesc = makeSmemDesc(stage + kABytes, kBChunkBytes, 1024);
#pragma unroll
          for (int kk = 0; kk < BK / UMMA_K; ++kk)
            umma<2>(dTmem, aDesc + uint64_t(kk * 2), bDesc + uint64_t(kk * 128), kInstrDesc,
                    (kb | kk) != 0);
          // Frees the stage in both CTAs once these MMAs are done.
          ummaCommitPair(smemAddr(&bars->empty[s]), 0x3);
        }
        if (!ok)
          break;
        ummaCommitPair(smemAddr(&bars->tmemFull[acc]), 0x3);
      }
    }
  } else {
    // -------------------------------- epilogue --------------------------------
    const int quad = warp & 3; // TMEM lanes [32*quad, 32*quad+32) for this warp
    uint32_t tmemEmptyBar[2];
    for (int a = 0; a < 2; ++a)
      tmemEmptyBar[a] = mapSharedToCta(smemAddr(&bars->tmemEmpty[a]), 0);
    int tileIter = 0;
    for (int t = firstTile; t < numTiles; t += tileStep, ++tileIter) {
      int tm, tn;
      tileCoords(t, p, tm, tn);
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
      const long long row = (long long)tm * kTileM + int(ctaRank) * BM + quad * 32 + lane;
      const long long colBase = (long long)tn * BN;
      const uint32_t taddr = tmemBase + (uint32_t(quad * 32) << 16) + uint32_t(acc * BN);
      __nv_bfloat16 *crow = c + row * p.ldc;
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
          if (col + 32 <= p.N) {
#pragma unroll
            for (int j = 0; j < 32; j += 4) {
              const float4 s4 = __ldg(reinterpret_cast<const float4 *>(scale + col + j));
              f[j] *= s4.x;
              f[j + 1] *= s4.y;
              f[j + 2] *= s4.z;
              f[j + 3] *= s4.w;
            }
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (col + j < p.N)
                f[j] *= __ldg(scale + col + j);
          }
          uint32_t w[16]; // the 32 values rounded to bf16, two per word
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            __nv_bfloat162 h = __floats2bfloat162_rn(f[2 * j], f[2 * j + 1]);
            w[j] = *reinterpret_cast<uint32_t *>(&h);
          }
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
      // This warp has read its quarter of the accumulator.
      tcgen05FenceBefore();
      __syncwarp();
      if (lane == 0)
        mbarArriveCluster(tmemEmptyBar[acc]);
    }
  }

  // -------------------------------- teardown ----------------------------------
  __syncwarp();
  tcgen05FenceBefore();
  clusterSync();
  if (warp == 1) {
    tcgen05FenceAfter();
    tmemFree<2>(tmemBase, TMEM_COLS);
  }
}
