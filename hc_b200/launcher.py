"""Single-box multi-GPU launcher: one process per GPU, each runs the workload
kernels on its shard; the only communication is the all-gather of the output.

The reference has no multi-GPU support at all (its py-runtime holds one
process-wide device and queue, python/cpp/py-runtime/src/GpuRuntime.cpp:23-24),
so this module has no counterpart there.  Every workload shards without any
exchange during the computation:

* row softmax and row reductions - rows are independent: rank r owns rows
  ``partition(M, world, r)``;
* bf16 GEMM - sharded over M: rank r owns a row block of A and of C, B is
  replicated on every GPU beforehand;
* int8 dequant GEMM - sharded over N: rank r owns a column block of W, of the
  scales and of the output, A is replicated.

Processes are started by ``torchrun`` (``RANK``/``LOCAL_RANK``/``WORLD_SIZE``
in the environment) and talk through ``torch.distributed``: NCCL over
NVLink/NVSwitch for device tensors, gloo when the tensors live on the host
(which is how the sharding and gathering logic is tested without GPUs).  No
kernel ever reads another GPU's memory.

Two ways to the gathered output:

* the collective: every rank computes into its block of the full output and
  ``gather_band`` / ``gather_cols_even`` run NCCL's all-gather (in row bands, so
  that the gather of one band overlaps the kernel of the next);
* the kernel itself: with a :class:`PeerOutput` (the full output of every rank in
  symmetric memory) the ``*_peers`` kernels write a rank's rows straight into
  every rank's buffer over NVLink - compute and all-gather in one launch, no
  second pass over the output and no separate collective; a 4-byte all-reduce
  orders the ranks afterwards.  Kernels only ever *write* peer memory.
"""

from __future__ import annotations

import os
from dataclasses import dataclass

import torch
import torch.distributed as dist


@dataclass(frozen=True)
class Span:
    begin: int
    end: int

    @property
    def size(self):
        return self.end - self.begin


def partition(n: int, world: int, rank: int, align: int = 1) -> Span:
    """Rank ``rank``'s share of ``n`` units split over ``world`` ranks.

    Shares are contiguous, ordered by rank, multiples of ``align`` (except
    possibly the last non-empty one) and differ by at most one ``align`` block;
    ragged totals leave trailing ranks with less (possibly nothing)."""
    if world <= 0 or not 0 <= rank < world:
        raise ValueError(f"invalid rank {rank} of {world}")
    if n < 0 or align <= 0:
        raise ValueError("n must be >= 0 and align > 0")
    blocks = -(-n // align)
    base, extra = divmod(blocks, world)
    begin_block = rank * base + min(rank, extra)
    end_block = begin_block + base + (1 if rank < extra else 0)
    return Span(min(n, begin_block * align), min(n, end_block * align))


class BandPlan:
    """Block-cyclic partition of ``m`` rows: the rows are cut into ``bands``
    consecutive bands and every band is split over the ranks, so a rank owns
    one block of rows per band.

    With one band this is the plain contiguous partition.  With several, the
    all-gather of band ``b`` (whose blocks, in rank order, are exactly the rows
    of the band, so it lands in place in the full output) can run on the
    communication stream while the kernel computes band ``b + 1``: the output
    all-gather, which moves far more bytes than a shard's kernel takes time for,
    hides behind the computation instead of following it."""

    def __init__(self, m: int, world: int, bands: int = 1, align: int = 1):
        if bands <= 0:
            raise ValueError("bands must be positive")
        self.m, self.world, self.bands = m, world, bands
        self.band_spans = [partition(m, bands, b, align) for b in range(bands)]
        self.blocks = []  # [band][rank] -> Span of absolute rows
        for band in self.band_spans:
            inner = [partition(band.size, world, r, align) for r in range(world)]
            self.blocks.append([Span(band.begin + s.begin, band.begin + s.end) for s in inner])

    def block(self, band: int, rank: int) -> Span:
        """Absolute rows of ``rank``'s block in ``band``."""
        return self.blocks[band][rank]

    def local(self, band: int, rank: int) -> Span:
        """The same block as rows of the rank's compact shard (its blocks of all
        bands, in band order)."""
        begin = sum(self.blocks[b][rank].size for b in range(band))
        return Span(begin, begin + self.blocks[band][rank].size)

    def shard_rows(self, rank: int) -> int:
        return sum(self.blocks[b][rank].size for b in range(self.bands))

    def even(self, band: int) -> bool:
        return len({s.size for s in self.blocks[band]}) == 1

    def take_shard(self, full, rank: int):
        """Rank ``rank``'s compact shard of a tensor whose first dimension is the
        row dimension (a copy unless there is one band)."""
        parts = [full[self.blocks[b][rank].begin:self.blocks[b][rank].end]
                 for b in range(self.bands)]
        return parts[0] if len(parts) == 1 else torch.cat(parts, dim=0)


class PeerOutput:
    """A full output array that every rank holds and every rank can write: one
    buffer per GPU in symmetric memory (torch.distributed._symmetric_memory),
    each mapped into every process of the job.

    It is what lets a kernel do the output all-gather itself: the ``*_peers``
    entry points (include/hc_b200_kernels.h: hcSoftmaxRowsPeers,
    hcReduceRowsPeers, hcGemmBf16Peers, hcGemmW8A16Peers) take the addresses
    ``bases(offset)`` and write a rank's rows into all of them with plain stores
    over NVLink.  No kernel waits for another; ``fence()`` orders the ranks
    afterwards on the stream (a 4-byte all-reduce), after which every rank may
    read its ``tensor``."""

    def __init__(self, shape, dtype, device, group=None):
        import torch.distributed._symmetric_memory as symm_mem

        self.group = group if group is not None else dist.group.WORLD
        self.tensor = symm_mem.empty(*shape, dtype=dtype, device=device)
        self.handle = symm_mem.rendezvous(self.tensor, self.group)
        self.addresses = [int(p) for p in self.handle.buffer_ptrs]
        self._token = torch.zeros(1, dtype=torch.int32, device=device)

    def bases(self, element_offset: int = 0):
        """Address of element ``element_offset`` (row-major) in every rank's buffer."""
        step = element_offset * self.tensor.element_size()
        return [a + step for a in self.addresses]

    def fence(self):
        """Every rank's stores issued so far (on the current stream) are complete
        and visible before any rank's later work on its stream starts."""
        dist.all_reduce(self._token, group=self.group)


def init_process_group(backend: str | None = None):
    """Join the job described by the torchrun environment; returns
    ``(rank, world, local_rank)``.  With no ``WORLD_SIZE`` in the environment
    this is a single-process job and nothing is initialised."""
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", str(rank)))
    if world > 1 and not dist.is_initialized():
        if backend is None:
            backend = "nccl" if torch.cuda.is_available() else "gloo"
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        kwargs = {}
        if backend == "nccl":
            torch.cuda.set_device(local)
            kwargs["device_id"] = torch.device("cuda", local)
        dist.init_process_group(backend=backend, rank=rank, world_size=world, **kwargs)
    return rank, world, local


class ShardedLauncher:
    """Runs this rank's shard of a workload and gathers outputs.

    ``kernels`` is a namespace like the one :func:`hc_b200.workloads.make_kernels`
    returns.  Tests pass a stand-in with the same attribute names, which lets
    the partitioning and gathering run on CPU ranks.
    """

    def __init__(self, kernels, rank: int = 0, world: int = 1, group=None):
        self.kernels = kernels
        self.rank = rank
        self.world = world
        self.group = group

    # -- shards ---------------------------------------------------------------------
    def rows(self, m: int) -> Span:
        return partition(m, self.world, self.rank)

    def cols(self, n: int) -> Span:
        # Column shards start on multiples of 16 elements so that every shard
        # of a bf16 or int8 matrix keeps the 16-byte alignment TMA needs.
        return partition(n, self.world, self.rank, align=16)

    # -- compute on the local shard -----------------------------------------------------
    def softmax(self, x_shard, out_shard, group_rows: int = 256):
        if x_shard.shape[0]:
            self.kernels.softmax(x_shard, out_shard, group_rows)

    def reduce_rows(self, x_shard, sum_shard, max_shard, group_rows: int = 256):
        if x_shard.shape[0]:
            self.kernels.reduce_rows(x_shard, sum_shard, max_shard, group_rows)

    def gemm_rows(self, a_shard, b_full, c_shard, group=(256, 256)):
        """M-sharded GEMM: this rank's rows of A times the replicated B."""
        if a_shard.shape[0]:
            self.kernels.dot_fullk(a_shard, b_full, c_shard, group)

    def dequant_gemm_cols(self, a_full, w_shard, scale_shard, out_shard, group=(256, 256)):
        """N-sharded dequant GEMM: replicated A times this rank's columns of W."""
        if w_shard.shape[1]:
            self.kernels.dequant_dot(a_full, w_shard, scale_shard, out_shard, group)

    def conv_images(self, conv, x_shard, f_full, out_shard):
        """Batch-sharded convolution: this rank's images against the replicated
        filters; ``conv`` is a kernel from :func:`hc_b200.workloads.make_conv`.
        Output images are independent, so ``gather_rows`` assembles the result."""
        if x_shard.shape[0]:
            conv(x_shard, f_full, out_shard)

    def rows_body(self, body, in_shards, out_shard, group_rows: int = 256):
        """Row-sharded element-wise or row body: ``body`` is a kernel from
        :func:`hc_b200.workloads.make_rowwise` (called with the rows per group) or
        :func:`hc_b200.workloads.make_elementwise` (``group_rows=None``); rows are
        independent, so ``gather_rows`` assembles the result."""
        if out_shard.shape[0]:
            if group_rows is None:
                body(*in_shards, out_shard)
            else:
                body(*in_shards, out_shard, group_rows)

    # -- the one collective: gather the output ------------------------------------------
    def gather_rows(self, shard, full):
        """All-gather row shards (``partition`` order) into ``full`` on every rank."""
        if self.world == 1:
            if full.data_ptr() != shard.data_ptr():
                full.copy_(shard)
            return full
        m = full.shape[0]
        spans = [partition(m, self.world, r) for r in range(self.world)]
        if len({s.size for s in spans}) == 1 and full.is_contiguous() and shard.is_contiguous():
            dist.all_gather_into_tensor(full, shard, group=self.group)
            return full
        # Ragged: every rank contributes a buffer padded to the largest share.
        widest = max(s.size for s in spans)
        padded = shard.new_zeros((widest,) + tuple(shard.shape[1:]))
        padded[: shard.shape[0]] = shard
        parts = [torch.empty_like(padded) for _ in range(self.world)]
        dist.all_gather(parts, padded, group=self.group)
        for s, part in zip(spans, parts):
            full[s.begin : s.end] = part[: s.size]
        return full

    def gather_band(self, full, plan: BandPlan, band: int, async_op: bool = False):
        """All-gather one band of ``full`` in place: this rank's block of the band
        is already written at its rows of ``full``; afterwards every rank holds
        the whole band.  Even blocks take one ``all_gather_into_tensor`` whose
        input is the rank's own slice of the output (NCCL's in-place form, no
        staging copy) and, with ``async_op``, return the work handle to wait on;
        ragged bands are gathered padded, synchronously."""
        if self.world == 1:
            return None
        span = plan.band_spans[band]
        mine = plan.block(band, self.rank)
        if plan.even(band) and full.is_contiguous():
            return dist.all_gather_into_tensor(full[span.begin:span.end],
                                               full[mine.begin:mine.end], group=self.group,
                                               async_op=async_op)
        widest = max(s.size for s in plan.blocks[band])
        padded = full.new_zeros((widest,) + tuple(full.shape[1:]))
        padded[: mine.size] = full[mine.begin:mine.end]
        parts = [torch.empty_like(padded) for _ in range(self.world)]
        dist.all_gather(parts, padded, group=self.group)
        for s, part in zip(plan.blocks[band], parts):
            full[s.begin:s.end] = part[: s.size]
        return None

    def run_rows_pipelined(self, compute, full, plan: BandPlan, gather: bool = True):
        """The sharded step of a row-partitioned workload: for every band,
        ``compute(band, local_span, out_block)`` runs this rank's kernel on its
        block (``local_span``: rows of the compact input shard; ``out_block``: the
        block's rows of ``full``, written in place) and the band's all-gather is
        queued behind it without waiting, so it overlaps the next band's
        kernel.  Returns when everything is queued and the current stream has
        been made to wait for the gathers."""
        pending = []
        for band in range(plan.bands):
            mine = plan.block(band, self.rank)
            if mine.size:
                compute(band, plan.local(band, self.rank), full[mine.begin:mine.end])
            if gather:
                work = self.gather_band(full, plan, band, async_op=True)
                if work is not None:
                    pending.append(work)
        for work in pending:
            work.wait()
        return full

    def gather_cols_even(self, shard, staging, full, place=None):
        """All-gather equal column shards without allocating: ``shard`` [M, n]
        is gathered into ``staging`` [world, M, n] (one ``all_gather_into_tensor``)
        and block r is then placed into columns ``[r*n, (r+1)*n)`` of ``full``
        by ``place(src_block, dst_view)`` (default: a strided tensor copy)."""
        if self.world == 1:
            if full.data_ptr() != shard.data_ptr():
                full.copy_(shard)
            return full
        n = shard.shape[1]
        if tuple(staging.shape) != (self.world,) + tuple(shard.shape) or \
                full.shape[1] != n * self.world:
            raise ValueError("gather_cols_even: staging must be [world, M, n] and full [M, world*n]")
        dist.all_gather_into_tensor(staging.view(-1, n), shard, group=self.group)
        for r in range(self.world):
            dst = full[:, r * n:(r + 1) * n]
            if place is None:
                dst.copy_(staging[r])
            else:
                place(staging[r], dst)
        return full

    def gather_cols(self, shard, full):
        """All-gather column shards: gathered as ``[world, M, n_r]`` blocks, then
        placed into the column ranges of ``full``."""
        if self.world == 1:
            if full.data_ptr() != shard.data_ptr():
                full.copy_(shard)
            return full
        n = full.shape[1]
        spans = [partition(n, self.world, r, align=16) for r in range(self.world)]
        widest = max(s.size for s in spans)
        padded = shard.new_zeros((shard.shape[0], widest))
        padded[:, : shard.shape[1]] = shard
        parts = [torch.empty_like(padded) for _ in range(self.world)]
        dist.all_gather(parts, padded.contiguous(), group=self.group)
        for s, part in zip(spans, parts):
            full[:, s.begin : s.end] = part[:, : s.size]
        return full
