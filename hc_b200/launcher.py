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
