#!/usr/bin/env python
"""Benchmark of the hot path: the workload kernels, measured against the B200
roofline, next to the CPU restatement of the reference timed on the host cores.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME]
    torchrun --nproc-per-node N bench.py --gpus N ...      (N > 1)
    python bench.py --impl reference ...                   (CPU arm)

One JSON line is printed by rank 0.  The headline workload is the row softmax
over X[32768, 4096] fp32 (HBM-bound); ``metric`` is its algorithmic throughput
in GB/s: bytes that must move (read X once, write Y once) divided by the time
of the timed region.  ``--workload`` selects another headline
(``reduce``, ``gemm_f32``, ``gemm_bf16``, ``gemm_w8a16``); with the default
headline the other four are measured too and reported under ``workloads``.

Scaling is weak: every rank runs the full single-GPU workload on its own rows
(the shards are independent, so there is no collective in the timed path);
``value`` is the sum over ranks divided by the slowest rank's time.
"""

import argparse
import json
import os
import statistics
import sys
import threading
import time

REPO = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, REPO)

# Algorithmic work of each workload at its full size.
SHAPES = {
    "softmax": (32768, 4096),
    "reduce": (65536, 8192),
    "gemm_f32": (256, 256, 256),
    "gemm_bf16": (8192, 8192, 8192),
    "gemm_w8a16": (4096, 8192, 8192),
}


# Reduced shapes for profiler captures (--small): the streaming kernels still
# move more than the 126 MB L2 holds, but a launch lasts tens of microseconds.
SMALL_SHAPES = {
    "softmax": (8192, 4096),
    "reduce": (16384, 8192),
    "gemm_f32": (256, 256, 256),
    "gemm_bf16": (2048, 2048, 2048),
    "gemm_w8a16": (1024, 2048, 2048),
}


def algorithmic(name):
    """(bytes, flops, bound) one launch of the workload must move / compute."""
    s = SHAPES[name]
    if name == "softmax":
        m, n = s
        return 2 * m * n * 4, 0, "hbm"
    if name == "reduce":
        m, n = s
        return m * n * 4 + 2 * m * 4, 0, "hbm"
    m, n, k = s
    if name == "gemm_f32":
        return 3 * m * n * 4, 2 * m * n * k, "latency"
    if name == "gemm_bf16":
        return (m * k + k * n + m * n) * 2, 2 * m * n * k, "tensor"
    return m * k * 2 + k * n + n * 4 + m * n * 2, 2 * m * n * k, "tensor"


# dram bytes per launch of the headline kernels from the ncu captures summarised
# under profiles/ (None until a capture exists for that kernel).
NCU_TRAFFIC = {
    # profiles/softmax_rows_f32_w32_8192x4096.md: (134.26 + 79.48) MB for a quarter of
    # the rows, scaled by 4 (the part of Y still in L2 at kernel end is not counted).
    "softmax": 854.9e6,
    # profiles/reduce_rows_warp_f32_16384x8192.md: (536.92 + 3.38) MB for a quarter of the rows.
    "reduce": 2161.2e6,
    "gemm_bf16": None,
    "gemm_w8a16": None,
    "gemm_f32": None,
}


def load_peaks():
    path = os.path.join(REPO, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            p = json.load(f)
        return {"hbm_gbs": float(p["hbm_gbs"]), "bf16_tflops": float(p["bf16_tflops"]),
                "bf16_tflops_sustained": float(p.get("bf16_tflops_sustained", p["bf16_tflops"])),
                "source": "measured"}
    except (OSError, KeyError, ValueError):
        return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0,
                "source": "fallback"}


class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU while the timed regions
    run (read-only NVML queries)."""

    REASONS = {
        0x2: "applications_clocks_setting", 0x4: "sw_power_cap", 0x8: "hw_slowdown",
        0x10: "sync_boost", 0x20: "sw_thermal_slowdown", 0x40: "hw_thermal_slowdown",
        0x80: "hw_power_brake_slowdown", 0x100: "display_clock_setting",
    }

    def __init__(self, index):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml

            pynvml.nvmlInit()
            self.nvml = pynvml
            self.handle = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.handle, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nvml = None

    def _run(self):
        n = self.nvml
        while not self._stop.is_set():
            try:
                self.samples.append(n.nvmlDeviceGetClockInfo(self.handle, n.NVML_CLOCK_SM))
                mask = n.nvmlDeviceGetCurrentClocksThrottleReasons(self.handle)
                for bit, name in self.REASONS.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            self._stop.wait(0.02)

    def __enter__(self):
        if self.nvml is not None:
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        if self._thread is not None:
            self._thread.join()

    def summary(self):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": ["unavailable"]}
        # "Under load": ignore samples taken while the GPU idled between regions.
        busy = [s for s in self.samples if s >= 0.5 * max(self.samples)] or self.samples
        return {"sm_mhz": statistics.median(busy), "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(self.samples)}


# ---- CPU arm ----------------------------------------------------------------------------
def cpu_softmax_sample(rows, threads, repeats):
    """Times the oracle's softmax (oracle/workloads.py) on `rows` rows of the
    headline workload; returns (GB/s, seconds per pass)."""
    import numpy as np

    from oracle import workloads as oracle

    (x,) = oracle.make_inputs("softmax", shape=(rows, SHAPES["softmax"][1]))
    out = np.empty_like(x)

    def one_pass():
        oracle.run_row_groups_parallel(
            lambda r0, r1: oracle.softmax_rows(x[r0:r1], out[r0:r1], 256), rows, 256, threads)

    one_pass()
    t0 = time.perf_counter()
    for _ in range(repeats):
        one_pass()
    dt = (time.perf_counter() - t0) / repeats
    return 2 * x.nbytes / dt / 1e9, dt


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    threads = len(os.sched_getaffinity(0))
    rows = 8192  # one step = a quarter of the 32768-row workload
    t0 = time.perf_counter()
    gbs, dt = cpu_softmax_sample(rows, threads, max(1, args.warmup))  # warm-up passes
    gbs, dt = cpu_softmax_sample(rows, threads, max(1, args.steps))
    sample = f"{rows} of 32768 rows per step, NumPy oracle, {threads} threads"
    line = {
        "impl": "reference", "metric": "softmax_rows_f32_algorithmic_bandwidth", "value": gbs,
        "unit": "GB/s", "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": dt * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "row softmax fp32 X[32768,4096] (bounded sample per step)",
                   "rows_per_step": rows, "cols": 4096},
        "cpu_baseline": {"value": gbs, "unit": "GB/s", "cores": threads, "kind": "port",
                         "sample": sample},
        "e2e": {"value": gbs, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "wall_s": time.perf_counter() - t0,
    }
    print(json.dumps(line), flush=True)


# ---- GPU arm ----------------------------------------------------------------------------
def run_gpu(args):
    import torch
    import torch.distributed as dist

    from hc_b200.hckernel.kernel import get_context
    from hc_b200.launcher import init_process_group
    from hc_b200.workloads import make_kernels
    from hc_b200._native import _dispatcher as native

    rank, world, local = init_process_group()
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE is {world}: launch with torchrun")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    desc = f"cuda:{local}"
    kernels = make_kernels(desc)
    ctx = get_context(desc)
    stream = torch.cuda.ExternalStream(ctx.stream, device=dev)
    peaks = load_peaks()

    def barrier():
        ctx.synchronize()
        torch.cuda.synchronize(dev)
        if world > 1:
            dist.barrier()

    def max_over_ranks(ms):
        if world == 1:
            return ms
        t = torch.tensor([ms], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def timed(fn, steps, warmup):
        """ms for `steps` calls of fn on the context's stream (max over ranks)
        and the number of kernel launches they issued."""
        for _ in range(warmup):
            fn()
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        before = ctx.launch_count
        e0.record(stream)
        for _ in range(steps):
            fn()
        e1.record(stream)
        barrier()
        return max_over_ranks(e0.elapsed_time(e1)), ctx.launch_count - before

    def measure(name, steps, warmup):
        """Device-resident throughput of one workload; returns a result dict."""
        nbytes, flops, bound = algorithmic(name)
        g = torch.Generator(device=dev).manual_seed(1000 + rank)
        if name == "softmax":
            m, n = SHAPES[name]
            x = torch.randn(m, n, device=dev, generator=g)
            y = torch.empty_like(x)
            fn = lambda: native.softmax_rows(ctx, x, y)  # noqa: E731
        elif name == "reduce":
            m, n = SHAPES[name]
            x = torch.rand(m, n, device=dev, generator=g) * 20 - 10
            s, mx = torch.empty(m, device=dev), torch.empty(m, device=dev)
            fn = lambda: native.reduce_rows(ctx, x, s, mx)  # noqa: E731
        elif name == "gemm_f32":
            m, n, k = SHAPES[name]
            a = torch.rand(m, k, device=dev, generator=g) * 2 - 1
            b = torch.rand(k, n, device=dev, generator=g) * 2 - 1
            c = torch.empty(m, n, device=dev)
            fn = lambda: native.gemm(ctx, a, b, c)  # noqa: E731
        elif name == "gemm_bf16":
            m, n, k = SHAPES[name]
            a = (torch.randn(m, k, device=dev, generator=g) * 0.02).bfloat16()
            b = (torch.randn(k, n, device=dev, generator=g) * 0.02).bfloat16()
            c = torch.empty(m, n, device=dev, dtype=torch.bfloat16)
            fn = lambda: native.gemm(ctx, a, b, c)  # noqa: E731
        else:
            m, n, k = SHAPES[name]
            a = torch.randn(m, k, device=dev, generator=g).bfloat16()
            w = torch.randint(-127, 128, (k, n), device=dev, generator=g, dtype=torch.int8)
            sc = torch.rand(n, device=dev, generator=g) * 0.019 + 0.001
            c = torch.empty(m, n, device=dev, dtype=torch.bfloat16)
            ws = torch.empty(native.w8a16_workspace_bytes(n, k), dtype=torch.uint8, device=dev)
            fn = lambda: native.gemm_w8a16(ctx, a, w, sc, c, ws)  # noqa: E731
        torch.cuda.synchronize(dev)
        ms, launches = timed(fn, steps, warmup)
        status = ctx.kernel_status()
        per_step = ms / steps
        out = {"ms_per_step": per_step, "steps": steps, "launches": launches, "status": status}
        if bound == "hbm":
            ach = nbytes / per_step / 1e6
            out.update(value=ach * world, unit="GB/s",
                       roofline={"bound": "hbm", "achieved": ach, "peak": peaks["hbm_gbs"],
                                 "unit": "GB/s", "frac": ach / peaks["hbm_gbs"],
                                 "traffic": NCU_TRAFFIC[name], "peak_source": peaks["source"]})
        else:
            ach = flops / per_step / 1e9
            out.update(value=ach * world, unit="TFLOP/s",
                       roofline={"bound": "tensor" if bound == "tensor" else "latency",
                                 "achieved": ach, "peak": peaks["bf16_tflops"],
                                 "unit": "TFLOP/s", "frac": ach / peaks["bf16_tflops"],
                                 "frac_of_sustained": ach / peaks["bf16_tflops_sustained"],
                                 "traffic": NCU_TRAFFIC[name], "peak_source": peaks["source"]})
        return out

    def measure_e2e(name, steps, warmup):
        """Same workload through the public call surface with HOST buffers: per
        step, pinned host -> device copy of the inputs, the @kernel call, and a
        device -> host copy of the result."""
        if name != "softmax":
            return None
        m, n = SHAPES[name]
        hx = torch.randn(m, n).pin_memory()
        hy = torch.empty(m, n).pin_memory()
        dx, dy = torch.empty(m, n, device=dev), torch.empty(m, n, device=dev)

        def step():
            with torch.cuda.stream(stream):
                dx.copy_(hx, non_blocking=True)
                kernels.softmax(dx, dy, 256)
                hy.copy_(dy, non_blocking=True)

        ms, launches = timed(step, steps, warmup)
        nbytes, _, _ = algorithmic(name)
        row_sums = hy[:64].sum(dim=1)
        assert torch.allclose(row_sums, torch.ones_like(row_sums), atol=1e-4), "softmax rows != 1"
        return {"value": nbytes * world / (ms / steps) / 1e6, "unit": "GB/s",
                "h2d_bytes_per_step": hx.numel() * 4, "d2h_bytes_per_step": hy.numel() * 4,
                "ms_per_step": ms / steps, "steps": steps}

    sampler = ClockSampler(local)
    with sampler:
        head = measure(args.workload, args.steps, args.warmup)
        e2e = measure_e2e(args.workload, max(3, min(args.steps, 20)), 3)
        extras = {}
        if args.workload == "softmax" and not args.no_extras:
            for name, steps in (("reduce", 200), ("gemm_bf16", 50), ("gemm_w8a16", 50),
                                ("gemm_f32", 500)):
                extras[name] = measure(name, steps, 5)

    if rank == 0:
        nbytes, flops, bound = algorithmic(args.workload)
        metric = {
            "softmax": "softmax_rows_f32_algorithmic_bandwidth",
            "reduce": "reduce_rows_f32_algorithmic_bandwidth",
            "gemm_f32": "gemm_f32_tiled_throughput",
            "gemm_bf16": "gemm_bf16_throughput",
            "gemm_w8a16": "gemm_w8a16_throughput",
        }[args.workload]
        line = {
            "metric": metric, "value": head["value"], "unit": head["unit"], "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": head["ms_per_step"],
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": {"softmax": "f32", "reduce": "f32", "gemm_f32": "f32",
                      "gemm_bf16": "bf16", "gemm_w8a16": "bf16"}[args.workload],
            "data": "synthetic",
            "config": {"workload": f"{args.workload} {list(SHAPES[args.workload])} per GPU",
                       "rows_or_tiles_sharded": "independent shards, no collective in the timed path",
                       "l2": "inputs and outputs larger than L2 (no flush needed)"
                       if args.workload != "gemm_f32" else "operands fit in L2 (latency-bound case)"},
            "roofline": head["roofline"], "gpu_launches": head["launches"],
            "kernel_status": head["status"], "clocks": sampler.summary(),
        }
        if args.small:
            line["config"]["small"] = "reduced shape for profiling; not a benchmark result"
        if e2e is not None:
            line["e2e"] = e2e
        if extras:
            line["workloads"] = extras
        if world == 1 and not args.no_cpu_baseline:
            threads = 1
            gbs, dt = cpu_softmax_sample(4096, threads, 5)
            line["cpu_baseline"] = {"value": gbs, "unit": "GB/s", "cores": threads,
                                    "kind": "port",
                                    "sample": "4096 of 32768 rows of the softmax workload, "
                                              "5 passes, NumPy oracle, single thread"}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=1000)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="hc_b200", choices=["hc_b200", "reference"])
    ap.add_argument("--workload", default="softmax", choices=sorted(SHAPES))
    ap.add_argument("--no-extras", action="store_true")
    ap.add_argument("--small", action="store_true",
                    help="reduced shapes, for profiler captures; not a benchmark result")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    args = ap.parse_args()
    if args.small:
        SHAPES.update(SMALL_SHAPES)
    if args.impl == "reference":
        run_reference(args)
    else:
        run_gpu(args)


if __name__ == "__main__":
    main()
