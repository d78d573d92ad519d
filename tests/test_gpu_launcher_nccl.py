"""Two-GPU run of the sharded launcher with the real kernels and NCCL: every
rank computes its shard on its own GPU, the outputs are all-gathered - by NCCL,
and by the kernels that write into both ranks' buffers themselves - and each
rank checks the gathered result against the CPU oracle of the whole problem.
Skipped on a box with fewer than two GPUs (the single-GPU suite covers the
kernels; tests/test_launcher_gloo.py covers the sharding logic on CPU)."""

import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import workloads as oracle

pytestmark = pytest.mark.gpu


def _worker(rank, world, port, results):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        from hc_b200.hckernel.kernel import get_context
        from hc_b200.launcher import ShardedLauncher
        from hc_b200.workloads import make_kernels

        L = ShardedLauncher(make_kernels(f"cuda:{rank}"), rank, world)
        ok = {}

        rows = 600
        (x,) = oracle.make_inputs("softmax", shape=(rows, 2048))
        span = L.rows(rows)
        xs = torch.from_numpy(x[span.begin:span.end]).to(dev)
        ys = torch.empty_like(xs)
        L.softmax(xs, ys)
        full = torch.empty(rows, 2048, device=dev)
        L.gather_rows(ys, full)
        expect = np.zeros_like(x)
        oracle.softmax_rows(x, expect, 256)
        got = full.cpu().numpy()
        ok["softmax"] = bool(np.all(np.abs(got - expect) <= 1e-6 + 1e-5 * np.abs(expect)))

        (x,) = oracle.make_inputs("reduce", shape=(rows + 1, 1024))  # ragged: 301 + 300 rows
        span = L.rows(rows + 1)
        xs = torch.from_numpy(x[span.begin:span.end]).to(dev)
        ss, ms = torch.empty(span.size, device=dev), torch.empty(span.size, device=dev)
        L.reduce_rows(xs, ss, ms)
        fs, fm = torch.empty(rows + 1, device=dev), torch.empty(rows + 1, device=dev)
        L.gather_rows(ss, fs)
        L.gather_rows(ms, fm)
        bound = 1e-5 * np.abs(x).astype(np.float64).sum(axis=1)
        ok["reduce"] = bool(np.array_equal(fm.cpu().numpy(), x.max(axis=1)) and np.all(
            np.abs(fs.cpu().numpy() - x.astype(np.float64).sum(axis=1)) <= bound))

        m, n, k = 512, 768, 256
        a, b = oracle.make_inputs("gemm_bf16", shape=(m, n, k))
        span = L.rows(m)
        a_s = torch.from_numpy(a[span.begin:span.end]).to(dev).bfloat16()
        b_d = torch.from_numpy(b).to(dev).bfloat16()  # replicated
        c_s = torch.empty(span.size, n, device=dev, dtype=torch.bfloat16)
        L.gemm_rows(a_s, b_d, c_s)
        c_full = torch.empty(m, n, device=dev, dtype=torch.bfloat16)
        L.gather_rows(c_s, c_full)
        expect = np.zeros((m, n), np.float32)
        oracle.gemm_bf16(a, b, expect, (256, 256))
        got = c_full.float().cpu().numpy()
        ok["gemm_rows"] = bool(np.all(np.abs(got - expect) <= 1e-2 * np.abs(expect)
                                      + 1e-4 * (np.abs(a) @ np.abs(b))))

        m, n, k = 256, 544, 512  # column shards of 272 each
        a, w, s = oracle.make_inputs("gemm_w8a16", shape=(m, n, k))
        cs = L.cols(n)
        a_d = torch.from_numpy(a).to(dev).bfloat16()  # replicated
        w_d = torch.from_numpy(w).to(dev)
        s_d = torch.from_numpy(s).to(dev)
        o_s = torch.empty(m, cs.size, device=dev, dtype=torch.bfloat16)
        L.dequant_gemm_cols(a_d, w_d[:, cs.begin:cs.end], s_d[cs.begin:cs.end], o_s)
        o_full = torch.empty(m, n, device=dev, dtype=torch.bfloat16)
        L.gather_cols(o_s, o_full)
        expect = np.zeros((m, n), np.float32)
        oracle.gemm_w8a16(a, w, s, expect, (256, 256))
        got = o_full.float().cpu().numpy()
        mag = np.abs(a) @ (np.abs(w.astype(np.float32)) * s)
        ok["dequant_cols"] = bool(np.all(np.abs(got - expect) <= 1e-2 * np.abs(expect) + 1e-4 * mag))

        from hc_b200.workloads import make_conv

        x_shape, f_shape = (11, 4, 9, 9), (12, 4, 3, 3)  # 6 + 5 images
        x, f = oracle.make_conv_inputs(x_shape, f_shape, "float32")
        out_shape = oracle.conv_out_shape(x_shape, f_shape, 1)
        span = L.rows(x_shape[0])
        x_s = torch.from_numpy(x[span.begin:span.end]).to(dev)
        f_d = torch.from_numpy(f).to(dev)  # replicated
        o_s = torch.zeros((span.size,) + out_shape[1:], device=dev)
        L.conv_images(make_conv(1, f"cuda:{rank}"), x_s, f_d, o_s)
        o_full = torch.empty(out_shape, device=dev)
        L.gather_rows(o_s, o_full)
        expect = np.zeros(out_shape, np.float32)
        oracle.conv_implicit_gemm(x, f, expect, 1)
        ok["conv_images"] = bool(np.allclose(o_full.cpu().numpy(), expect, rtol=1e-5, atol=1e-5))

        # Row bodies and element-wise bodies shard by rows like the softmax.
        from hc_b200.workloads import make_elementwise, make_rowwise

        rows = 301  # 151 + 150 rows of 4096: held in registers by the row-program kernel
        (x,) = oracle.make_elementwise_inputs(1, (rows, 4096), "float32", seed=5)
        span = L.rows(rows)
        xs = torch.from_numpy(x[span.begin:span.end]).to(dev)
        ys = torch.full_like(xs, float("nan"))
        centre = make_rowwise(lambda t: t - t.mean(axis=1, keepdims=True), 1, f"cuda:{rank}")
        L.rows_body(centre, [xs], ys, 64)
        full = torch.empty(rows, 4096, device=dev)
        L.gather_rows(ys, full)
        x64 = x.astype(np.float64)
        ok["rows_body"] = bool(np.allclose(full.cpu().numpy(), x64 - x64.mean(axis=1, keepdims=True),
                                           rtol=2e-6, atol=1e-6))
        relu = make_elementwise(lambda t: np.maximum(t * 2.0 - 1.0, 0.0), 1, 2, (4, 256),
                                f"cuda:{rank}")
        L.rows_body(relu, [xs], ys, None)
        L.gather_rows(ys, full)
        ok["map_body"] = bool(np.array_equal(full.cpu().numpy(),
                                             np.maximum(x * np.float32(2) - np.float32(1), 0)))

        # Compute and all-gather in one kernel: every rank writes its shard into the
        # full output of both ranks (symmetric memory, stores over NVLink); a small
        # all-reduce orders the ranks; then every rank holds the whole result.
        from hc_b200._native import _dispatcher as native
        from hc_b200.launcher import PeerOutput

        ctx = get_context(f"cuda:{rank}")
        stream = torch.cuda.ExternalStream(ctx.stream, device=dev)
        rows, cols = 600, 2048
        (x,) = oracle.make_inputs("softmax", shape=(rows, cols))
        span = L.rows(rows)
        xs = torch.from_numpy(x[span.begin:span.end]).to(dev)
        peer = PeerOutput((rows, cols), torch.float32, dev)
        peer.tensor.fill_(float("nan"))
        torch.cuda.synchronize(dev)
        dist.barrier()
        with torch.cuda.stream(stream):
            native.softmax_rows_peers(ctx, xs, peer.bases(span.begin * cols), cols)
            peer.fence()
            stream.synchronize()
        expect = np.zeros_like(x)
        oracle.softmax_rows(x, expect, 256)
        got = peer.tensor.cpu().numpy()
        ok["softmax_peers"] = bool(np.all(np.abs(got - expect) <= 1e-6 + 1e-5 * np.abs(expect)))

        (x,) = oracle.make_inputs("reduce", shape=(rows, 1024))
        xs = torch.from_numpy(x[span.begin:span.end]).to(dev)
        both = PeerOutput((2, rows), torch.float32, dev)
        both.tensor.fill_(float("nan"))
        torch.cuda.synchronize(dev)
        dist.barrier()
        with torch.cuda.stream(stream):
            native.reduce_rows_peers(ctx, xs, both.bases(span.begin), rows)
            both.fence()
            stream.synchronize()
        got = both.tensor.cpu().numpy()
        bound = 1e-5 * np.abs(x).astype(np.float64).sum(axis=1)
        ok["reduce_peers"] = bool(np.array_equal(got[1], x.max(axis=1)) and np.all(
            np.abs(got[0] - x.astype(np.float64).sum(axis=1)) <= bound))

        m, n, k = 512, 768, 256
        a, b = oracle.make_inputs("gemm_bf16", shape=(m, n, k))
        span = L.rows(m)
        a_s = torch.from_numpy(a[span.begin:span.end]).to(dev).bfloat16()
        b_d = torch.from_numpy(b).to(dev).bfloat16()
        c_all = PeerOutput((m, n), torch.bfloat16, dev)
        torch.cuda.synchronize(dev)
        dist.barrier()
        with torch.cuda.stream(stream):
            native.gemm_bf16_peers(ctx, a_s, b_d, c_all.bases(span.begin * n), n)
            c_all.fence()
            stream.synchronize()
        expect = np.zeros((m, n), np.float32)
        oracle.gemm_bf16(a, b, expect, (256, 256))
        got = c_all.tensor.float().cpu().numpy()
        ok["gemm_peers"] = bool(np.all(np.abs(got - expect) <= 1e-2 * np.abs(expect)
                                       + 1e-4 * (np.abs(a) @ np.abs(b))))

        m, n, k = 256, 512, 512  # column shards of 256 each
        a, w, s = oracle.make_inputs("gemm_w8a16", shape=(m, n, k))
        cs = L.cols(n)
        a_d = torch.from_numpy(a).to(dev).bfloat16()
        w_d, s_d = torch.from_numpy(w).to(dev), torch.from_numpy(s).to(dev)
        o_all = PeerOutput((m, n), torch.bfloat16, dev)
        ws = torch.empty(native.w8a16_workspace_bytes(cs.size, k), dtype=torch.uint8, device=dev)
        torch.cuda.synchronize(dev)
        dist.barrier()
        with torch.cuda.stream(stream):
            native.gemm_w8a16_peers(ctx, a_d, w_d[:, cs.begin:cs.end],
                                    s_d[cs.begin:cs.end].contiguous(), o_all.bases(cs.begin), n, ws)
            o_all.fence()
            stream.synchronize()
        expect = np.zeros((m, n), np.float32)
        oracle.gemm_w8a16(a, w, s, expect, (256, 256))
        mag = np.abs(a) @ (np.abs(w.astype(np.float32)) * s)
        got = o_all.tensor.float().cpu().numpy()
        ok["dequant_peers"] = bool(np.all(np.abs(got - expect)
                                          <= 1e-2 * np.abs(expect) + 1e-4 * mag))

        ok["status"] = get_context(f"cuda:{rank}").kernel_status() == 0
        results[rank] = ok
    finally:
        dist.destroy_process_group()


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def test_two_gpu_sharded_workloads_with_nccl_gather():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    world = 2
    with mp.Manager() as manager:
        results = manager.dict()
        mp.spawn(_worker, args=(world, _free_port(), results), nprocs=world, join=True)
        assert len(results) == world
        for rank in range(world):
            assert all(results[rank].values()), (rank, dict(results[rank]))
