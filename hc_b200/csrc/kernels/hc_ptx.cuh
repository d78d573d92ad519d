// Thin inline-PTX wrappers for the sm_100a features the kernels use:
// mbarrier, TMA (cp.async.bulk.tensor, never with cluster multicast), tcgen05
// MMA / TMEM, and a few cache-hinted global accesses.
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <stdint.h>

namespace hc {

// ---- bounded waits ----------------------------------------------------------
// Every spin in these kernels gives up after kWaitLimitNs; the kernel then
// records where it gave up in a status word the host reads and leaves through
// its normal teardown (TMEM freed, copies drained), so a protocol bug cannot
// hang the GPU.
constexpr unsigned long long kWaitLimitNs = 2000000000ull; // 2 s

enum StatusCode : int {
  kStatusOk = 0,
  kStatusProducerWait = 1, // TMA producer waiting for a free stage
  kStatusMmaWaitData = 2,  // MMA issuer waiting for a filled stage
  kStatusMmaWaitTmem = 3,  // MMA issuer waiting for a drained accumulator
  kStatusEpilogueWait = 4, // epilogue waiting for a finished accumulator
  kStatusDrainWait = 5,    // teardown waiting for copies in flight
};

__device__ __forceinline__ unsigned long long globalTimerNs() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

__device__ __forceinline__ uint32_t smemAddr(const void *p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ bool electOne() {
  uint32_t pred;
  asm volatile("{\n"
               ".reg .pred p;\n"
               "elect.sync _|p, 0xffffffff;\n"
               "selp.u32 %0, 1, 0, p;\n"
               "}\n"
               : "=r"(pred));
  return pred != 0;
}

// ---- mbarrier ---------------------------------------------------------------
__device__ __forceinline__ void mbarInit(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar),
               "r"(count));
}

__device__ __forceinline__ void fenceBarrierInit() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

__device__ __forceinline__ void fenceProxyAsync() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

__device__ __forceinline__ void mbarArrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar)
               : "memory");
}

// Arrive on a barrier that lives in another CTA of the cluster (`bar` is a
// shared::cluster address obtained with mapSharedToCta).
__device__ __forceinline__ void mbarArriveCluster(uint32_t bar) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::
                   "r"(bar)
               : "memory");
}

// The same with the default semantics (release at CTA scope): for a report about
// this CTA's own shared memory, which only this SM's tensor core reads (under an
// MMA of the pair that the other CTA issues).  The cluster-scope release above
// was measured at about 1000 cycles per arrival after 16 KiB of stores.
__device__ __forceinline__ void mbarArriveRemote(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(bar) : "memory");
}

__device__ __forceinline__ void mbarExpectTx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(
                   bar),
               "r"(bytes)
               : "memory");
}

__device__ __forceinline__ bool mbarTryWait(uint32_t bar, uint32_t parity) {
  uint32_t done;
  asm volatile("{\n"
               ".reg .pred p;\n"
               "mbarrier.try_wait.parity.shared::cta.b64 p, [%0], %1;\n"
               "selp.u32 %2, 1, 0, p;\n"
               "}\n"
               : "+r"(bar), "+r"(parity), "=r"(done)::"memory");
  return done != 0;
}

// The same, letting the hardware keep the thread suspended for up to `hintNs`
// while the phase is incomplete (it wakes when the phase completes): a waiting
// thread then leaves the issue slots to the warps that have work.
__device__ __forceinline__ bool mbarTryWaitFor(uint32_t bar, uint32_t parity, uint32_t hintNs) {
  uint32_t done;
  asm volatile("{\n"
               ".reg .pred p;\n"
               "mbarrier.try_wait.parity.shared::cta.b64 p, [%0], %1, %3;\n"
               "selp.u32 %2, 1, 0, p;\n"
               "}\n"
               : "+r"(bar), "+r"(parity), "=r"(done)
               : "r"(hintNs)
               : "memory");
  return done != 0;
}

// Waits for the phase with the given parity.  Returns false when the wait was
// abandoned: either it ran out of time (then `*abortFlag` is raised and `code`
// is published in `*status`), or another thread of the CTA had already raised
// the flag.
__device__ __forceinline__ bool mbarWait(uint32_t bar, uint32_t parity,
                                         volatile int *abortFlag, int *status,
                                         int code,
                                         unsigned long long limitNs = kWaitLimitNs) {
  if (mbarTryWait(bar, parity))
    return true;
  unsigned long long start = globalTimerNs();
  for (uint32_t spin = 1;; ++spin) {
    if (mbarTryWaitFor(bar, parity, 20000u))
      return true;
    if ((spin & 1u) == 0) { // (a failed poll may have slept for its whole hint)
      if (*abortFlag)
        return false;
      if (globalTimerNs() - start > limitNs) {
        *abortFlag = 1;
        atomicCAS(status, kStatusOk, code);
        return false;
      }
    }
  }
}

// ---- cluster ----------------------------------------------------------------
__device__ __forceinline__ uint32_t clusterCtaRank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}

__device__ __forceinline__ void clusterSync() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n"
               "barrier.cluster.wait.acquire.aligned;" ::
                   : "memory");
}

// shared::cta address in this CTA -> shared::cluster address of the same
// offset in CTA `rank` of the cluster.
__device__ __forceinline__ uint32_t mapSharedToCta(uint32_t addr,
                                                   uint32_t rank) {
  uint32_t out;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;"
               : "=r"(out)
               : "r"(addr), "r"(rank));
  return out;
}

// ---- TMA --------------------------------------------------------------------
__device__ __forceinline__ void prefetchTensorMap(const CUtensorMap *map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(
                   reinterpret_cast<uint64_t>(map))
               : "memory");
}

// 2-D tile load into this CTA's shared memory; completion bytes are counted
// on this CTA's mbarrier.  x is the innermost (contiguous) coordinate and must
// be a multiple of 16 bytes worth of elements.
__device__ __forceinline__ void tmaLoad2D(uint32_t dst, const CUtensorMap *map,
                                          uint32_t bar, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::"
      "bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(dst),
      "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(x), "r"(y)
      : "memory");
}

// Same, for a CTA pair driving one cta_group::2 MMA: the data lands in this
// CTA's shared memory while the completion bytes are counted on the barrier of
// the pair's leader (`bar` is a shared::cluster address).
__device__ __forceinline__ void tmaLoad2DPair(uint32_t dst,
                                              const CUtensorMap *map,
                                              uint32_t bar, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::"
      "complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(dst),
      "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(x), "r"(y)
      : "memory");
}

// ---- tcgen05 / TMEM ---------------------------------------------------------
template <int CtaGroup>
__device__ __forceinline__ void tmemAlloc(uint32_t resultSmem, uint32_t cols) {
  if constexpr (CtaGroup == 1)
    asm volatile(
        "tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::
            "r"(resultSmem),
        "r"(cols)
        : "memory");
  else
    asm volatile(
        "tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::
            "r"(resultSmem),
        "r"(cols)
        : "memory");
}

template <int CtaGroup> __device__ __forceinline__ void tmemRelinquish() {
  if constexpr (CtaGroup == 1)
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;");
  else
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;");
}

template <int CtaGroup>
__device__ __forceinline__ void tmemFree(uint32_t taddr, uint32_t cols) {
  if constexpr (CtaGroup == 1)
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(
                     taddr),
                 "r"(cols)
                 : "memory");
  else
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(
                     taddr),
                 "r"(cols)
                 : "memory");
}

__device__ __forceinline__ void tcgen05FenceBefore() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tcgen05FenceAfter() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

// Shared-memory matrix descriptor for tcgen05.mma operands staged with the
// 128-byte swizzle (the layout a TMA box of 64 bf16 per row produces):
//   bits  0-13  start address  >> 4
//   bits 16-29  leading-dimension byte offset >> 4
//   bits 32-45  stride-dimension byte offset  >> 4
//   bits 46-47  descriptor version (1 on sm_100)
//   bits 61-63  swizzle mode (2 = 128 B)
__device__ __forceinline__ uint64_t makeSmemDesc(uint32_t addr,
                                                 uint32_t leadingBytes,
                                                 uint32_t strideBytes) {
  uint64_t d = 0;
  d |= uint64_t((addr & 0x3FFFFu) >> 4);
  d |= uint64_t((leadingBytes >> 4) & 0x3FFFu) << 16;
  d |= uint64_t((strideBytes >> 4) & 0x3FFFu) << 32;
  d |= uint64_t(1) << 46;
  d |= uint64_t(2) << 61;
  return d;
}

// Instruction descriptor for kind::f16 with bf16 inputs and f32 accumulation:
//   bits 4-5 D format (1 = f32), 7-9 A format (1 = bf16), 10-12 B format,
//   bit 15 A major (0 = K), bit 16 B major (1 = MN), 17-22 N >> 3, 24-28 M >> 4.
__host__ __device__ constexpr uint32_t makeInstrDescBf16(int m, int n,
                                                         bool aMnMajor,
                                                         bool bMnMajor) {
  return (1u << 4) | (1u << 7) | (1u << 10) | (uint32_t(aMnMajor) << 15) |
         (uint32_t(bMnMajor) << 16) | (uint32_t(n >> 3) << 17) |
         (uint32_t(m >> 4) << 24);
}

// D[tmem] (+)= A[smem] * B[smem]; issued by ONE thread.
template <int CtaGroup>
__device__ __forceinline__ void umma(uint32_t dTmem, uint64_t aDesc,
                                     uint64_t bDesc, uint32_t iDesc,
                                     uint32_t accumulate) {
  if constexpr (CtaGroup == 1)
    asm volatile("{\n"
                 ".reg .pred p;\n"
                 "setp.ne.b32 p, %4, 0;\n"
                 "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n"
                 "}\n" ::"r"(dTmem),
                 "l"(aDesc), "l"(bDesc), "r"(iDesc), "r"(accumulate)
                 : "memory");
  else
    asm volatile("{\n"
                 ".reg .pred p;\n"
                 "setp.ne.b32 p, %4, 0;\n"
                 "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n"
                 "}\n" ::"r"(dTmem),
                 "l"(aDesc), "l"(bDesc), "r"(iDesc), "r"(accumulate)
                 : "memory");
}

// The same with tf32 inputs (kind::tf32, K = 8 per instruction).
template <int CtaGroup>
__device__ __forceinline__ void ummaTf32(uint32_t dTmem, uint64_t aDesc, uint64_t bDesc,
                                         uint32_t iDesc, uint32_t accumulate) {
  if constexpr (CtaGroup == 1)
    asm volatile("{\n"
                 ".reg .pred p;\n"
                 "setp.ne.b32 p, %4, 0;\n"
                 "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n"
                 "}\n" ::"r"(dTmem),
                 "l"(aDesc), "l"(bDesc), "r"(iDesc), "r"(accumulate)
                 : "memory");
  else
    asm volatile("{\n"
                 ".reg .pred p;\n"
                 "setp.ne.b32 p, %4, 0;\n"
                 "tcgen05.mma.cta_group::2.kind::tf32 [%0], %1, %2, %3, p;\n"
                 "}\n" ::"r"(dTmem),
                 "l"(aDesc), "l"(bDesc), "r"(iDesc), "r"(accumulate)
                 : "memory");
}

// The same with the A operand in tensor memory: 128 lanes (the rows) by 8 columns
// (the K elements, 32 bits each) starting at `aTmem`.
__device__ __forceinline__ void ummaTf32TmemA(uint32_t dTmem, uint32_t aTmem, uint64_t bDesc,
                                              uint32_t iDesc, uint32_t accumulate) {
  asm volatile("{\n"
               ".reg .pred p;\n"
               "setp.ne.b32 p, %4, 0;\n"
               "tcgen05.mma.cta_group::1.kind::tf32 [%0], [%1], %2, %3, p;\n"
               "}\n" ::"r"(dTmem),
               "r"(aTmem), "l"(bDesc), "r"(iDesc), "r"(accumulate)
               : "memory");
}

// Makes `bar` (this CTA) complete one arrival once every MMA issued so far by
// this thread has finished.
__device__ __forceinline__ void ummaCommit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::"
               "cluster.b64 [%0];" ::"r"(bar)
               : "memory");
}

// Pair form: the arrival is delivered to the barrier at the same offset in
// every CTA named by `ctaMask`.
__device__ __forceinline__ void ummaCommitPair(uint32_t bar, uint16_t ctaMask) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::"
               "cluster.multicast::cluster.b64 [%0], %1;" ::"r"(bar),
               "h"(ctaMask)
               : "memory");
}

// 32 lanes x 32 consecutive 32-bit columns: thread i of the warp receives
// columns [col, col+32) of TMEM lane (laneBase + i).
__device__ __forceinline__ void tmemLoad32x32(uint32_t taddr, uint32_t (&v)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, "
      "%30, %31}, [%32];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]),
        "=r"(v[6]), "=r"(v[7]), "=r"(v[8]), "=r"(v[9]), "=r"(v[10]),
        "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]),
        "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]),
        "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]), "=r"(v[25]),
        "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]),
        "=r"(v[31])
      : "r"(taddr)
      : "memory");
}

// 32 lanes x 8 consecutive 32-bit columns: thread i of the warp writes columns
// [col, col+8) of TMEM lane (laneBase + i).
__device__ __forceinline__ void tmemStore32x8(uint32_t taddr, const uint32_t (&v)[8]) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::
                   "r"(taddr),
               "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]),
               "r"(v[7])
               : "memory");
}

__device__ __forceinline__ void tmemStoreWait() {
  asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void tmemLoadWait() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// ---- float32 as two tf32 numbers ----------------------------------------------
// The nearest tf32 number, as a float whose low 13 fraction bits are zero.
__device__ __forceinline__ float toTf32(float v) {
  uint32_t bits;
  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(bits) : "f"(v));
  return __uint_as_float(bits);
}

// v = hi + lo with hi = tf32(v) and lo = tf32(v - hi).
__device__ __forceinline__ void splitTf32(float v, float &hi, float &lo) {
  hi = toTf32(v);
  // Infinities and NaNs stay in the high part alone (inf - inf would poison lo).
  lo = (hi - hi == 0.0f) ? toTf32(v - hi) : 0.0f;
}

// ---- global memory with cache hints ------------------------------------------
// Streaming 16-byte load: data is read once, so it should not displace what
// other kernels keep in L1.
__device__ __forceinline__ float4 loadStream(const float4 *p) {
  float4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
               : "l"(p));
  return v;
}

__device__ __forceinline__ void storeStream(float4 *p, float4 v) {
  asm volatile("st.global.cs.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(p),
               "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w)
               : "memory");
}

// max that returns NaN when either input is NaN (what numpy's max does).
__device__ __forceinline__ float maxNan(float a, float b) {
  float r;
  asm("max.NaN.f32 %0, %1, %2;" : "=f"(r) : "f"(a), "f"(b));
  return r;
}
__device__ __forceinline__ double maxNan(double a, double b) {
  return (a != a) ? a : ((b != b) ? b : (a > b ? a : b));
}

} // namespace hc
