"""The multi-GPU launcher's host logic on CPU: partitioning, and a two-rank
gloo run of every sharded workload with the CPU oracle standing in for the
kernels (the launcher only decides who computes what and gathers the output;
the kernels themselves are covered by the GPU tests)."""

import os
import socket
import types

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from hc_b200.launcher import BandPlan, ShardedLauncher, Span, partition
from oracle import workloads as oracle


def test_partition_properties():
    for n in (0, 1, 7, 16, 100, 8192, 32768, 65537):
        for world in (1, 2, 3, 4, 8):
            for align in (1, 16):
                spans = [partition(n, world, r, align) for r in range(world)]
                assert spans[0].begin == 0 and spans[-1].end == n
                for a, b in zip(spans, spans[1:]):
                    assert a.end == b.begin  # contiguous, ordered, no overlap
                sizes = [s.size for s in spans]
                # One whole block of difference at most, plus the ragged tail block.
                assert max(sizes) - min(sizes) < 2 * align or n < align * world
                for s in spans:
                    assert s.size == 0 or s.begin % align == 0
    assert partition(10, 4, 0) == Span(0, 3) and partition(10, 4, 3) == Span(8, 10)
    assert partition(8192, 8, 3, 16) == Span(3072, 4096)
    with pytest.raises(ValueError):
        partition(10, 0, 0)
    with pytest.raises(ValueError):
        partition(10, 2, 2)


def test_band_plan_covers_every_row_once():
    for m in (0, 5, 64, 37, 32768):
        for world in (1, 2, 8):
            for bands in (1, 2, 8):
                plan = BandPlan(m, world, bands)
                seen = np.zeros(m, int)
                for r in range(world):
                    at = 0
                    for b in range(bands):
                        blk, loc = plan.block(b, r), plan.local(b, r)
                        seen[blk.begin:blk.end] += 1
                        assert (loc.begin, loc.size) == (at, blk.size)
                        at += blk.size
                    assert plan.shard_rows(r) == at
                assert np.all(seen == 1)
                # Blocks of a band are consecutive in rank order: gathered in that
                # order they are the band itself.
                for b in range(bands):
                    assert plan.blocks[b][0].begin == plan.band_spans[b].begin
                    assert plan.blocks[b][-1].end == plan.band_spans[b].end
    assert BandPlan(32768, 8, 8).block(3, 5) == Span(3 * 4096 + 5 * 512, 3 * 4096 + 6 * 512)


def _oracle_kernels():
    """Stand-ins with the call signatures of hc_b200.workloads.make_kernels."""

    def softmax(x, out, gm):
        o = np.zeros(tuple(x.shape), np.float32)
        oracle.softmax_rows(x.numpy(), o, gm)
        out.copy_(torch.from_numpy(o))

    def reduce_rows(x, s, mx, gm):
        so, mo = np.zeros(x.shape[0], np.float32), np.zeros(x.shape[0], np.float32)
        oracle.reduce_rows(x.numpy(), so, mo, gm)
        s.copy_(torch.from_numpy(so))
        mx.copy_(torch.from_numpy(mo))

    def dot_fullk(a, b, c, group):
        o = np.zeros(tuple(c.shape), np.float32)
        oracle.gemm_bf16(a.numpy(), b.numpy(), o, group)
        c.copy_(torch.from_numpy(o))

    def dequant_dot(a, w, s, out, group):
        o = np.zeros(tuple(out.shape), np.float32)
        oracle.gemm_w8a16(a.numpy(), np.ascontiguousarray(w.numpy()), s.numpy(), o, group)
        out.copy_(torch.from_numpy(o))

    return types.SimpleNamespace(softmax=softmax, reduce_rows=reduce_rows, dot_fullk=dot_fullk,
                                 dequant_dot=dequant_dot)


def _worker(rank, world, port, rows, results):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        L = ShardedLauncher(_oracle_kernels(), rank, world)
        ok = {}

        (x,) = oracle.make_inputs("softmax", shape=(rows, 96))
        span = L.rows(rows)
        xs = torch.from_numpy(x[span.begin:span.end].copy())
        ys = torch.empty_like(xs)
        L.softmax(xs, ys, 8)
        full = torch.empty(rows, 96)
        L.gather_rows(ys, full)
        expect = np.zeros_like(x)
        oracle.softmax_rows(x, expect, 8)
        ok["softmax"] = np.array_equal(full.numpy(), expect)

        (x,) = oracle.make_inputs("reduce", shape=(rows, 64))
        xs = torch.from_numpy(x[span.begin:span.end].copy())
        ss, ms = torch.empty(span.size), torch.empty(span.size)
        L.reduce_rows(xs, ss, ms, 16)
        fs, fm = torch.empty(rows), torch.empty(rows)
        L.gather_rows(ss, fs)
        L.gather_rows(ms, fm)
        ok["reduce"] = (np.array_equal(fm.numpy(), x.max(axis=1))
                        and np.array_equal(fs.numpy(), x.sum(axis=1)))

        a, b = oracle.make_inputs("gemm_bf16", shape=(rows, 48, 32))
        a_s = torch.from_numpy(a[span.begin:span.end].copy())
        c_s = torch.empty(span.size, 48)
        L.gemm_rows(a_s, torch.from_numpy(b), c_s, (16, 16))
        c_full = torch.empty(rows, 48)
        L.gather_rows(c_s, c_full)
        expect = np.zeros((rows, 48), np.float32)
        oracle.gemm_bf16(a, b, expect, (16, 16))
        ok["gemm_rows"] = np.array_equal(c_full.numpy(), expect)

        n = 80  # column shards of 48 and 32 (aligned to 16)
        a, w, s = oracle.make_inputs("gemm_w8a16", shape=(24, n, 32))
        cs = L.cols(n)
        w_s = torch.from_numpy(w)[:, cs.begin:cs.end]
        o_s = torch.empty(24, cs.size)
        L.dequant_gemm_cols(torch.from_numpy(a), w_s, torch.from_numpy(s[cs.begin:cs.end].copy()),
                            o_s, (8, 16))
        o_full = torch.empty(24, n)
        L.gather_cols(o_s, o_full)
        expect = np.zeros((24, n), np.float32)
        oracle.gemm_w8a16(a, w, s, expect, (8, 16))
        ok["dequant_cols"] = np.array_equal(o_full.numpy(), expect)

        # A row body (rows centred on their mean) and an element-wise body, sharded
        # by rows; the stand-ins run the oracle's tile arithmetic.
        def centre(t):
            return t - t.mean(axis=1, keepdims=True)

        def centre_body(x_t, out_t, gm):
            o = np.zeros(tuple(out_t.shape), np.float32)
            oracle.rowwise(centre, [x_t.numpy()], o, gm)
            out_t.copy_(torch.from_numpy(o))

        def double_body(x_t, out_t):
            o = np.zeros(tuple(out_t.shape), np.float32)
            oracle.elementwise(lambda t: t * 2.0, [x_t.numpy()], o, (4, 16))
            out_t.copy_(torch.from_numpy(o))

        (x,) = oracle.make_elementwise_inputs(1, (rows, 40), "float32", seed=3)
        span = L.rows(rows)
        xs = torch.from_numpy(x[span.begin:span.end].copy())
        ys = torch.empty_like(xs)
        L.rows_body(centre_body, [xs], ys, 8)
        full = torch.empty(rows, 40)
        L.gather_rows(ys, full)
        expect = np.zeros_like(x)
        oracle.rowwise(centre, [x], expect, 8)
        ok["rows_body"] = np.array_equal(full.numpy(), expect)
        L.rows_body(double_body, [xs], ys, None)
        L.gather_rows(ys, full)
        ok["map_body"] = np.array_equal(full.numpy(), x * 2)

        # Row bands: every band is computed in place in the full output and
        # gathered behind its kernel; ragged bands take the padded path.
        for bands in (1, 2, 4):
            plan = BandPlan(rows, world, bands)
            (x,) = oracle.make_inputs("softmax", shape=(rows, 96))
            shard = plan.take_shard(torch.from_numpy(x), rank).contiguous()
            assert shard.shape[0] == plan.shard_rows(rank)
            full = torch.full((rows, 96), float("nan"))

            def compute(band, loc, out_block, shard=shard):
                L.softmax(shard[loc.begin:loc.end], out_block, 8)

            L.run_rows_pipelined(compute, full, plan)
            expect = np.zeros_like(x)
            oracle.softmax_rows(x, expect, 8)
            ok[f"bands{bands}"] = np.array_equal(full.numpy(), expect)

        if True:
            n = 64  # equal column shards of 32
            a, w, s = oracle.make_inputs("gemm_w8a16", shape=(24, n, 32))
            cs = L.cols(n)
            o_s = torch.empty(24, cs.size)
            L.dequant_gemm_cols(torch.from_numpy(a), torch.from_numpy(w)[:, cs.begin:cs.end],
                                torch.from_numpy(s[cs.begin:cs.end].copy()), o_s, (8, 16))
            staging = torch.empty(world, 24, cs.size)
            o_full = torch.empty(24, n)
            L.gather_cols_even(o_s, staging, o_full)
            expect = np.zeros((24, n), np.float32)
            oracle.gemm_w8a16(a, w, s, expect, (8, 16))
            ok["cols_even"] = np.array_equal(o_full.numpy(), expect)
        results[rank] = ok
    finally:
        dist.destroy_process_group()


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


@pytest.mark.parametrize("rows", [64, 37])  # even shards and ragged shards
def test_two_rank_sharded_workloads_match_single_rank(rows):
    world = 2
    with mp.Manager() as manager:
        results = manager.dict()
        mp.spawn(_worker, args=(world, _free_port(), rows, results), nprocs=world, join=True)
        assert len(results) == world
        for rank in range(world):
            assert all(results[rank].values()), (rank, dict(results[rank]))


def test_single_rank_gather_is_a_copy():
    L = ShardedLauncher(_oracle_kernels(), 0, 1)
    shard = torch.arange(12.0).reshape(3, 4)
    full = torch.zeros(3, 4)
    L.gather_rows(shard, full)
    assert torch.equal(full, shard)
    assert L.rows(10) == Span(0, 10) and L.cols(100) == Span(0, 100)
