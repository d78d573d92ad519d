// Host-buffer entry points of libhc-b200-kernels.so: the row-wise workloads and
// the bf16 GEMM on data that lives in host memory.
//
// The reference's runtime only ever sees device pointers: its callers hand
// torch CUDA tensors to a kernel and every launch is followed by a host
// synchronisation (python/cpp/py-runtime/src/GpuRuntime.cpp:60-69).  A caller
// whose data starts and ends on the host would have to copy, launch, wait and
// copy back, one after the other.  Rows are independent in all of these
// workloads, so the matrix is cut into row chunks here and three queues of the
// context's device are chained with events:
//
//     upload queue     H2D chunk i+1 ----\
//     context's queue      kernel chunk i ----\
//     download queue           D2H chunk i-1
//
// PCIe is full duplex and the copy engines run beside the SMs, so upload,
// kernel and download overlap; two device slots per direction keep all three
// busy.  Only whole rows are handed to the kernels, so the result is that of
// one launch on the whole matrix - bit for bit for the softmax, the row maxima
// and the GEMM; a row sum may differ in its last bits when a chunk has so few
// rows that hcReduceRows takes its other kernel (a CTA per row instead of a warp
// per row).  The calls return when the result is in host memory.  Copies are asynchronous (and overlap) only for page-locked
// host memory: hcHostPin / hcHostUnpin lock an existing range.
#include "context.hpp"

#include <algorithm>
#include <cstdint>

namespace {

// Chunks of about this many bytes per matrix: small enough that the first
// upload and the last download, which nothing overlaps, are a few percent of
// the whole; large enough that every copy runs at full link speed.
constexpr size_t kChunkBytes = 16u << 20;

struct Slot {
  void *data = nullptr;
  size_t bytes = 0;
};

} // namespace

struct HostPipeline {
  OlQueue up = nullptr, down = nullptr;
  OlxEvent uploaded[2] = {nullptr, nullptr};
  OlxEvent kernelDone[2] = {nullptr, nullptr};
  OlxEvent downloaded[2] = {nullptr, nullptr};
  OlxEvent start = nullptr;
  Slot in[2][2], out[2][2]; // [slot][operand]
  Slot resident;            // a whole operand kept on the device (B of the GEMM)
};

void hcReleaseHostPipeline(HcContextImpl *c) {
  HostPipeline *p = c->hostPipeline;
  if (!p)
    return;
  if (p->up)
    olSyncQueue(p->up);
  if (p->down)
    olSyncQueue(p->down);
  for (int s = 0; s < 2; ++s) {
    for (int k = 0; k < 2; ++k) {
      if (p->in[s][k].data)
        olDeallocDevice(c->queue, p->in[s][k].data);
      if (p->out[s][k].data)
        olDeallocDevice(c->queue, p->out[s][k].data);
    }
    olxReleaseEvent(c->device, p->uploaded[s]);
    olxReleaseEvent(c->device, p->kernelDone[s]);
    olxReleaseEvent(c->device, p->downloaded[s]);
  }
  olxReleaseEvent(c->device, p->start);
  if (p->resident.data)
    olDeallocDevice(c->queue, p->resident.data);
  if (p->up)
    olReleaseQueue(p->up);
  if (p->down)
    olReleaseQueue(p->down);
  delete p;
  c->hostPipeline = nullptr;
}

namespace {

HostPipeline *pipelineOf(HcContextImpl *c) {
  if (c->hostPipeline)
    return c->hostPipeline;
  auto *p = new HostPipeline;
  c->hostPipeline = p;
  p->up = olCreateQueue(c->device);
  p->down = olCreateQueue(c->device);
  p->start = olxCreateEvent(c->device, 0);
  bool ok = p->up && p->down && p->start;
  for (int s = 0; s < 2 && ok; ++s) {
    p->uploaded[s] = olxCreateEvent(c->device, 0);
    p->kernelDone[s] = olxCreateEvent(c->device, 0);
    p->downloaded[s] = olxCreateEvent(c->device, 0);
    ok = p->uploaded[s] && p->kernelDone[s] && p->downloaded[s];
  }
  if (!ok) {
    hcReleaseHostPipeline(c);
    c->fail("host pipeline: could not create queues and events: %s", c->lastError.c_str());
    return nullptr;
  }
  return p;
}

// Grows a device buffer to at least `bytes` (buffers are kept between calls).
int reserve(HcContextImpl *c, Slot &slot, size_t bytes) {
  if (slot.bytes >= bytes)
    return 0;
  if (slot.data) {
    // Nothing may still use the old buffer.
    if (olSyncQueue(c->queue))
      return 1;
    olDeallocDevice(c->queue, slot.data);
    slot = Slot{};
  }
  slot.data = olAllocDevice(c->queue, bytes, 256);
  if (!slot.data)
    return c->fail("host pipeline: device allocation of %zu bytes failed: %s", bytes,
                   c->lastError.c_str());
  slot.bytes = bytes;
  return 0;
}

// Rows [r0, r0 + n) of a host matrix into a packed device buffer, or back.
int copyRows(HcContextImpl *c, OlQueue q, bool toDevice, void *device, void *host,
             long long r0, long long n, long long rowBytes, long long pitchBytes) {
  auto *h = static_cast<unsigned char *>(host) + r0 * pitchBytes;
  if (pitchBytes == rowBytes || n == 1) {
    const size_t bytes = size_t(n) * size_t(rowBytes);
    return toDevice ? olxMemcpyHtoD(q, device, h, bytes) : olxMemcpyDtoH(q, h, device, bytes);
  }
  auto *d = static_cast<unsigned char *>(device);
  for (long long r = 0; r < n; ++r) {
    const int rc = toDevice ? olxMemcpyHtoD(q, d + r * rowBytes, h + r * pitchBytes, size_t(rowBytes))
                            : olxMemcpyDtoH(q, h + r * pitchBytes, d + r * rowBytes, size_t(rowBytes));
    if (rc)
      return rc;
  }
  return 0;
}

// One streamed operand: a host matrix (or vector, rowBytes = element size) whose
// first dimension is the row dimension.
struct Streamed {
  void *host;
  long long rowBytes, pitchBytes;
};

// Runs `launch(slotInputs, slotOutputs, r0, n)` over row chunks with upload,
// kernel and download overlapped.  `launch` queues kernels on the context's
// queue only.
template <typename Launch>
int streamRows(HcContextImpl *c, long long rows, long long chunkRows, const Streamed *ins,
               int nIn, const Streamed *outs, int nOut, Launch launch) {
  HostPipeline *p = pipelineOf(c);
  if (!p)
    return 1;
  chunkRows = std::max<long long>(1, std::min(chunkRows, rows));
  // Equal chunks rather than full ones and a short tail.
  const long long chunks = (rows + chunkRows - 1) / chunkRows;
  chunkRows = (rows + chunks - 1) / chunks;
  for (int s = 0; s < 2; ++s) {
    for (int k = 0; k < nIn; ++k)
      if (reserve(c, p->in[s][k], size_t(chunkRows) * size_t(ins[k].rowBytes)))
        return 1;
    for (int k = 0; k < nOut; ++k)
      if (reserve(c, p->out[s][k], size_t(chunkRows) * size_t(outs[k].rowBytes)))
        return 1;
  }
  // Whatever is already queued on the context's queue comes first.
  int rc = olxRecordEvent(c->queue, p->start) || olxQueueWaitEvent(p->up, p->start) ||
           olxQueueWaitEvent(p->down, p->start);
  bool used[2] = {false, false};
  long long index = 0;
  for (long long r0 = 0; r0 < rows && !rc; r0 += chunkRows, ++index) {
    const long long n = std::min(chunkRows, rows - r0);
    const int s = int(index & 1);
    if (used[s]) // the kernel that read this slot's inputs two chunks ago
      rc = rc || olxQueueWaitEvent(p->up, p->kernelDone[s]);
    for (int k = 0; k < nIn && !rc; ++k)
      rc = copyRows(c, p->up, true, p->in[s][k].data, ins[k].host, r0, n, ins[k].rowBytes,
                    ins[k].pitchBytes);
    rc = rc || olxRecordEvent(p->up, p->uploaded[s]) ||
         olxQueueWaitEvent(c->queue, p->uploaded[s]);
    if (used[s]) // the download that read this slot's outputs two chunks ago
      rc = rc || olxQueueWaitEvent(c->queue, p->downloaded[s]);
    if (!rc) {
      void *inPtr[2] = {p->in[s][0].data, p->in[s][1].data};
      void *outPtr[2] = {p->out[s][0].data, p->out[s][1].data};
      rc = launch(inPtr, outPtr, r0, n);
    }
    rc = rc || olxRecordEvent(c->queue, p->kernelDone[s]) ||
         olxQueueWaitEvent(p->down, p->kernelDone[s]);
    for (int k = 0; k < nOut && !rc; ++k)
      rc = copyRows(c, p->down, false, p->out[s][k].data, outs[k].host, r0, n,
                    outs[k].rowBytes, outs[k].pitchBytes);
    rc = rc || olxRecordEvent(p->down, p->downloaded[s]);
    used[s] = true;
  }
  // The result is in host memory when the call returns - also after an error,
  // so that nothing is in flight on buffers the caller may free.
  const int s1 = olSyncQueue(p->up), s2 = olSyncQueue(c->queue), s3 = olSyncQueue(p->down);
  if (rc || s1 || s2 || s3)
    return c->fail("host pipeline failed: %s", c->lastError.c_str());
  return 0;
}

long long chunkRowsFor(long long rowBytes) {
  return std::max<long long>(1, (long long)kChunkBytes / std::max<long long>(1, rowBytes));
}

int elemBytesOf(int dtype) { return dtype == HC_F32 ? 4 : dtype == HC_F64 ? 8 : 0; }

} // namespace

extern "C" {

int hcHostPin(HcContext c, void *ptr, size_t bytes) {
  if (!c)
    return 1;
  if (!ptr || bytes == 0)
    return c->fail("hcHostPin: empty range");
  if (olxHostRegister(c->device, ptr, bytes))
    return c->fail("hcHostPin failed: %s", c->lastError.c_str());
  return 0;
}

int hcHostUnpin(HcContext c, void *ptr) {
  if (!c)
    return 1;
  if (!ptr || olxHostUnregister(c->device, ptr))
    return c->fail("hcHostUnpin failed: %s", c->lastError.c_str());
  return 0;
}

int hcSoftmaxRowsHost(HcContext c, const void *xHost, void *yHost, long long rows,
                      long long cols, long long xPitch, long long yPitch, int dtype) {
  if (!c)
    return 1;
  const int elem = elemBytesOf(dtype);
  if (!elem)
    return c->fail("hcSoftmaxRowsHost: unsupported dtype %d", dtype);
  if (rows < 0 || cols < 0 || xPitch < cols || yPitch < cols)
    return c->fail("hcSoftmaxRowsHost: invalid shape %lld x %lld", rows, cols);
  if (rows == 0 || cols == 0)
    return 0;
  if (!xHost || !yHost)
    return c->fail("hcSoftmaxRowsHost: null buffer");
  const Streamed in = {const_cast<void *>(xHost), cols * elem, xPitch * elem};
  const Streamed out = {yHost, cols * elem, yPitch * elem};
  return streamRows(c, rows, chunkRowsFor(cols * elem), &in, 1, &out, 1,
                    [&](void **i, void **o, long long, long long n) {
                      return hcSoftmaxRows(c, i[0], o[0], n, cols, cols, cols, dtype);
                    });
}

int hcReduceRowsHost(HcContext c, const void *xHost, void *sumHost, void *maxHost,
                     long long rows, long long cols, long long pitch, int dtype) {
  if (!c)
    return 1;
  const int elem = elemBytesOf(dtype);
  if (!elem)
    return c->fail("hcReduceRowsHost: unsupported dtype %d", dtype);
  if (rows < 0 || cols < 0 || pitch < cols)
    return c->fail("hcReduceRowsHost: invalid shape %lld x %lld", rows, cols);
  if (rows == 0 || (!sumHost && !maxHost))
    return 0;
  if (!xHost && cols > 0)
    return c->fail("hcReduceRowsHost: null buffer");
  const Streamed in = {const_cast<void *>(xHost), cols * elem, pitch * elem};
  Streamed outs[2];
  int nOut = 0;
  const int sumAt = sumHost ? nOut++ : -1;
  if (sumHost)
    outs[sumAt] = {sumHost, elem, elem};
  const int maxAt = maxHost ? nOut++ : -1;
  if (maxHost)
    outs[maxAt] = {maxHost, elem, elem};
  return streamRows(c, rows, chunkRowsFor(std::max<long long>(1, cols) * elem), &in, 1, outs,
                    nOut, [&](void **i, void **o, long long, long long n) {
                      return hcReduceRows(c, i[0], sumAt < 0 ? nullptr : o[sumAt],
                                          maxAt < 0 ? nullptr : o[maxAt], n, cols, cols, dtype);
                    });
}

int hcGemmBf16Host(HcContext c, const void *aHost, const void *bHost, void *cHost,
                   long long M, long long N, long long K, long long lda, long long ldb,
                   long long ldc) {
  if (!c)
    return 1;
  if (M < 0 || N < 0 || K < 0 || lda < K || ldb < N || ldc < N)
    return c->fail("hcGemmBf16Host: invalid shape M=%lld N=%lld K=%lld", M, N, K);
  if (M == 0 || N == 0)
    return 0;
  if (!cHost || (K > 0 && (!aHost || !bHost)))
    return c->fail("hcGemmBf16Host: null buffer");
  HostPipeline *p = pipelineOf(c);
  if (!p)
    return 1;
  // B goes up whole, on the upload queue, ahead of the row blocks of A: every
  // product waits for its block of A, which follows B on that queue.  Device
  // rows are padded to 8 elements so that TMA can describe them.
  const long long kPad = (K + 7) / 8 * 8, nPad = (N + 7) / 8 * 8;
  if (reserve(c, p->resident, size_t(std::max<long long>(1, K)) * size_t(nPad) * 2))
    return 1;
  if (olxRecordEvent(c->queue, p->start) || olxQueueWaitEvent(p->up, p->start))
    return c->fail("hcGemmBf16Host: %s", c->lastError.c_str());
  if (K > 0 && copyRows(c, p->up, true, p->resident.data, const_cast<void *>(bHost), 0, K,
                        ldb == N && nPad == N ? N * 2 : N * 2, ldb * 2))
    return c->fail("hcGemmBf16Host: upload of B failed: %s", c->lastError.c_str());
  // (B is packed with pitch N on the device; when N is not a multiple of 8 the
  // GEMM entry point falls back to its CUDA-core kernel by itself.)
  (void)kPad;
  const Streamed in = {const_cast<void *>(aHost), K * 2, lda * 2};
  const Streamed out = {cHost, N * 2, ldc * 2};
  const long long rowBytes = std::max<long long>(1, std::max(K, N)) * 2;
  // Row blocks that are multiples of the 256-row tile of the tensor-core kernel.
  long long chunk = chunkRowsFor(rowBytes);
  if (chunk >= 256)
    chunk = chunk / 256 * 256;
  void *const bDev = p->resident.data;
  return streamRows(c, M, chunk, &in, 1, &out, 1,
                    [&](void **i, void **o, long long, long long n) {
                      return hcGemmBf16(c, i[0], bDev, o[0], n, N, K, K, N, N);
                    });
}

} // extern "C"
