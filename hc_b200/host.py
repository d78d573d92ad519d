r"""Host-buffer entry points: run a row-wise workload on data that lives in
(pinned) host memory, streaming it through the GPU in row chunks so that the
upload of chunk i+1, the kernel on chunk i and the download of chunk i-1
overlap.

The reference's callers hand device tensors to a kernel and fetch results
themselves, one blocking launch at a time (python/cpp/py-runtime/src/
GpuRuntime.cpp:60-69).  For data that starts and ends on the host that
serialises three transfers that the hardware can do at once: PCIe is full
duplex and the copy engines run beside the SMs.  Rows are independent in the
softmax and in the last-axis reductions, so the matrix is cut into row chunks
and three streams are chained with events:

    upload stream    H2D chunk i+1 ----\
    kernel stream        kernel chunk i ----\      (the native context's own stream)
    download stream          D2H chunk i-1

Two device slots per stream pair are enough to keep all three busy.  The
kernels are the same precompiled ones, reached through the same ``@kernel``
objects; only whole rows are ever passed, so results are bit-identical to a
single launch on the whole matrix.
"""

from __future__ import annotations

import torch

from .hckernel.kernel import get_context
from .workloads import make_kernels

_kernel_sets = {}


def _kernels(device: str):
    ks = _kernel_sets.get(device)
    if ks is None:
        ks = _kernel_sets[device] = make_kernels(device)
    return ks


class _RowPipeline:
    """Chunked upload -> kernel -> download over the rows of host tensors."""

    def __init__(self, device: str, chunk_rows: int):
        self.device = device
        self.ctx = get_context(device)
        self.dev = torch.device("cuda", self.ctx.ordinal)
        self.chunk_rows = int(chunk_rows)
        self.s_up = torch.cuda.Stream(self.dev)
        self.s_down = torch.cuda.Stream(self.dev)
        self.s_kernel = torch.cuda.ExternalStream(self.ctx.stream, device=self.dev)
        self._slots = {}

    def _slot_buffers(self, key, shapes_dtypes):
        bufs = self._slots.get(key)
        if bufs is None:
            bufs = self._slots[key] = [
                [torch.empty(shape, dtype=dtype, device=self.dev) for shape, dtype in shapes_dtypes]
                for _ in range(2)
            ]
        return bufs

    def run(self, launch, host_ins, host_outs):
        """``launch(dev_ins, dev_outs)`` is called once per chunk with device
        views of ``rows`` rows; ``host_ins``/``host_outs`` are host tensors whose
        first dimension is the row dimension (pinned memory makes the copies
        asynchronous; pageable memory works but serialises them)."""
        rows = host_ins[0].shape[0]
        step = max(1, min(self.chunk_rows, rows))
        d_ins = self._slot_buffers(
            ("in", step) + tuple((tuple(t.shape[1:]), t.dtype) for t in host_ins),
            [((step,) + tuple(t.shape[1:]), t.dtype) for t in host_ins])
        d_outs = self._slot_buffers(
            ("out", step) + tuple((tuple(t.shape[1:]), t.dtype) for t in host_outs),
            [((step,) + tuple(t.shape[1:]), t.dtype) for t in host_outs])
        kernel_done = [None, None]    # kernel finished reading/writing slot s
        download_done = [None, None]  # download finished reading slot s
        caller = torch.cuda.current_stream(self.dev)
        start = torch.cuda.Event()
        start.record(caller)
        for s in (self.s_up, self.s_kernel, self.s_down):
            s.wait_event(start)
        for i, r0 in enumerate(range(0, rows, step)):
            n = min(step, rows - r0)
            slot = i & 1
            if kernel_done[slot] is not None:
                self.s_up.wait_event(kernel_done[slot])
            with torch.cuda.stream(self.s_up):
                for d, h in zip(d_ins[slot], host_ins):
                    d[:n].copy_(h[r0:r0 + n], non_blocking=True)
                uploaded = torch.cuda.Event()
                uploaded.record(self.s_up)
            self.s_kernel.wait_event(uploaded)
            if download_done[slot] is not None:
                self.s_kernel.wait_event(download_done[slot])
            with torch.cuda.stream(self.s_kernel):
                launch([d[:n] for d in d_ins[slot]], [d[:n] for d in d_outs[slot]])
                kernel_done[slot] = torch.cuda.Event()
                kernel_done[slot].record(self.s_kernel)
            self.s_down.wait_event(kernel_done[slot])
            with torch.cuda.stream(self.s_down):
                for h, d in zip(host_outs, d_outs[slot]):
                    h[r0:r0 + n].copy_(d[:n], non_blocking=True)
                download_done[slot] = torch.cuda.Event()
                download_done[slot].record(self.s_down)
        # The caller's stream continues only after the last download.
        caller.wait_stream(self.s_down)
        caller.wait_stream(self.s_kernel)


_pipelines = {}


# Chunks of about this many bytes per matrix: small enough that the first
# upload and the last download (which nothing overlaps) are a few percent of the
# whole, large enough that each copy runs at full PCIe speed.
_CHUNK_BYTES = 16 << 20


def _default_chunk_rows(t):
    row_bytes = max(1, t[0].numel() * t.element_size()) if t.shape[0] else 1
    return max(1, _CHUNK_BYTES // row_bytes)


def _pipeline(device, chunk_rows):
    key = (device, int(chunk_rows))
    p = _pipelines.get(key)
    if p is None:
        p = _pipelines[key] = _RowPipeline(device, chunk_rows)
    return p


def softmax_rows_host(x_host, out_host, device="cuda:0", chunk_rows=None, group_rows=256):
    """Row softmax of a host matrix into a host matrix (both [M, N], same dtype)."""
    if x_host.shape != out_host.shape or x_host.dtype != out_host.dtype or x_host.dim() != 2:
        raise ValueError("softmax_rows_host: x and out must be matrices of one shape and dtype")
    k = _kernels(device)
    _pipeline(device, chunk_rows or _default_chunk_rows(x_host)).run(
        lambda ins, outs: k.softmax(ins[0], outs[0], group_rows), [x_host], [out_host])


def reduce_rows_host(x_host, sum_host, max_host, device="cuda:0", chunk_rows=None,
                     group_rows=256):
    """Last-axis sum and max of a host matrix [M, N] into host vectors [M]."""
    if x_host.dim() != 2 or sum_host.shape != (x_host.shape[0],) or max_host.shape != sum_host.shape:
        raise ValueError("reduce_rows_host: expected x [M, N], sum [M], max [M]")
    k = _kernels(device)
    _pipeline(device, chunk_rows or _default_chunk_rows(x_host)).run(
        lambda ins, outs: k.reduce_rows(ins[0], outs[0], outs[1], group_rows),
        [x_host], [sum_host, max_host])


def rows_body_host(body, in_hosts, out_host, device="cuda:0", chunk_rows=None, group_rows=256):
    """An element-wise or row body on host matrices: ``body`` is a kernel from
    :func:`hc_b200.workloads.make_rowwise` (called as ``body(*ins, out,
    group_rows)``) or :func:`hc_b200.workloads.make_elementwise`
    (``group_rows=None``: ``body(*ins, out)``) made for ``device``; the inputs
    and ``out`` are [M, N] of one dtype.  Rows are independent in both, so row
    chunks stream through the GPU as in :func:`softmax_rows_host`."""
    in_hosts = list(in_hosts)
    if not in_hosts or any(t.shape != out_host.shape or t.dtype != out_host.dtype
                           for t in in_hosts) or out_host.dim() != 2:
        raise ValueError("rows_body_host: inputs and out must be matrices of one shape and dtype")

    def launch(ins, outs):
        if group_rows is None:
            body(*ins, outs[0])
        else:
            body(*ins, outs[0], group_rows)

    _pipeline(device, chunk_rows or _default_chunk_rows(out_host)).run(launch, in_hosts, [out_host])


_resident = {}


def gemm_host(a_host, b_host, out_host, device="cuda:0", chunk_rows=None, group_shape=(256, 256)):
    """``out = a @ b`` for host matrices a [M, K], b [K, N], out [M, N] (one
    dtype: bfloat16, float32 or float64).  ``b`` is uploaded whole, then row
    blocks of ``a`` stream through: upload of block i+1, product of block i and
    download of block i-1 overlap.  Row blocks of a product are independent; in
    bfloat16 the result is bit for bit that of one launch on the whole
    matrices, in float32 the CUDA-core kernel may split K differently for a row
    block than for the whole matrix, so low-order bits can differ."""
    if (a_host.dim() != 2 or b_host.dim() != 2 or a_host.shape[1] != b_host.shape[0]
            or tuple(out_host.shape) != (a_host.shape[0], b_host.shape[1])):
        raise ValueError("gemm_host: expected a [M, K], b [K, N], out [M, N]")
    if not a_host.dtype == b_host.dtype == out_host.dtype:
        raise ValueError("gemm_host: a, b and out must have one dtype")
    k = _kernels(device)
    pipe = _pipeline(device, chunk_rows or _default_chunk_rows(a_host))
    # One device copy of b per (device, shape, dtype), refilled on every call.
    key = (device, tuple(b_host.shape), b_host.dtype)
    b_dev = _resident.get(key)
    if b_dev is None:
        b_dev = _resident[key] = torch.empty(b_host.shape, dtype=b_host.dtype, device=pipe.dev)
    caller = torch.cuda.current_stream(pipe.dev)
    # The kernels of an earlier call may still read b on the kernel stream.
    pipe.s_up.wait_stream(caller)
    pipe.s_up.wait_stream(pipe.s_kernel)
    with torch.cuda.stream(pipe.s_up):
        b_dev.copy_(b_host, non_blocking=True)
    # The row uploads follow b on the upload stream, and every kernel waits for
    # its row upload, so b is in place before the first product starts.
    pipe.run(lambda ins, outs: k.dot_fullk(ins[0], b_dev, outs[0], group_shape),
             [a_host], [out_host])


def synchronize(device="cuda:0"):
    """Block until everything queued by the host entry points has finished."""
    torch.cuda.synchronize(torch.device("cuda", get_context(device).ordinal))
