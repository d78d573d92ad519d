// Self-test of the bounded-wait machinery the TMA/tcgen05 kernels rely on.
//
// One CTA, two waiting threads, one barrier that nothing ever arrives on:
//   * thread 0 waits with a short limit; the wait must run out, publish
//     `kStatusProducerWait` in the status word and raise the CTA's abort flag;
//   * thread 32 waits on a second idle barrier with the normal (long) limit;
//     it must notice the abort flag and give up at once instead of waiting
//     out its own limit.
// The kernel then leaves through an ordinary __syncthreads and reports how
// long it was inside, so the host can check that giving up was prompt and
// that the context is still usable afterwards.  Nothing here faults, traps or
// spins without a bound.
#include "hc_ptx.cuh"

extern "C" __global__ void __launch_bounds__(64)
    hc_selftest_wait_timeout(unsigned long long limitNs, int *status,
                             unsigned long long *elapsedNs, int *observed) {
  __shared__ uint64_t idle[2];
  __shared__ int abortFlag;
  const unsigned long long t0 = hc::globalTimerNs();
  if (threadIdx.x == 0) {
    hc::mbarInit(hc::smemAddr(&idle[0]), 1);
    hc::mbarInit(hc::smemAddr(&idle[1]), 1);
    abortFlag = 0;
    hc::fenceBarrierInit();
  }
  __syncthreads();
  volatile int *flag = &abortFlag;
  if (threadIdx.x == 0) {
    const bool ok = hc::mbarWait(hc::smemAddr(&idle[0]), 0, flag, status,
                                 hc::kStatusProducerWait, limitNs);
    observed[0] = ok ? 1 : 0; // expected 0: the wait ran out
  } else if (threadIdx.x == 32) {
    const bool ok = hc::mbarWait(hc::smemAddr(&idle[1]), 0, flag, status,
                                 hc::kStatusMmaWaitData);
    observed[1] = ok ? 1 : 0; // expected 0: left because of the abort flag
  }
  __syncthreads();
  if (threadIdx.x == 0)
    *elapsedNs = hc::globalTimerNs() - t0;
}
