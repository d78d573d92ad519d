#!/usr/bin/env python
"""Benchmark of the hot path: the workload kernels, measured against the B200
roofline, next to the CPU restatement of the reference timed on the host cores.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME]
    torchrun --nproc-per-node N bench.py --gpus N ...      (N > 1)
    python bench.py --impl reference ...                   (CPU arm)

One JSON line is printed by rank 0.  The headline workload is the row softmax
over X[32768, 4096] fp32 (HBM-bound); ``metric`` is its algorithmic throughput
in GB/s: bytes that must move (read X once, write Y once) divided by the time
of the timed region.  ``--workload`` selects another headline (``reduce``,
``gemm_f32``, ``gemm_bf16``, ``gemm_w8a16``; GEMMs report TFLOP/s); with the
default headline the other four are measured too and reported under
``workloads``.

* ``value``  device-resident inputs, the C++ dispatcher called directly,
             CUDA events on the stream the kernels run on.
* ``e2e``    the same workload with HOST buffers, every step uploading the
             inputs from pinned memory and downloading the result: the
             row-wise workloads through the host-buffer entry points
             (``hc_b200.host``: row chunks with upload, ``@kernel`` call and
             download overlapped), the GEMMs as copy, ``@kernel`` call, copy.
* with several GPUs the scaling is strong: the fixed full-size problem is
  sharded (rows of the softmax, of the reductions and of the row bodies, M of
  the bf16 GEMM, N of the dequant GEMM), every rank runs the kernels on its
  share and the timed step ends with the NCCL all-gather that leaves the whole
  output on every GPU; ``phases`` times the kernels and the collective apart,
  and the gathered output is compared with the single-GPU output and with the
  CPU oracle inside the run.  ``--replicas`` runs independent replicas instead
  (weak scaling, no collective).
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

# Full-size shapes of the five configurations.
SHAPES = {
    "softmax": (32768, 4096),
    "reduce": (65536, 8192),
    "gemm_f32": (256, 256, 256),
    "gemm_bf16": (8192, 8192, 8192),
    "gemm_w8a16": (4096, 8192, 8192),
    # Implicit-GEMM convolution through index mappings, fp32: images [N, C, H, W],
    # filters [NF, C, HF, WF], stride (a ResNet-style 3x3 layer; not one of the
    # five benchmark configurations, measured as the next kernel family).
    "conv": (32, 64, 56, 56, 64, 3, 3, 1),
    # Element-wise body out = max(2a - b, 0) on fp32 matrices (three 512 MiB
    # arrays; likewise measured as a further kernel family).
    "map": (32768, 4096),
    # Row body with reductions used again (log-softmax), interpreted as a
    # three-pass row program; same shape as the softmax configuration.
    "rows": (32768, 4096),
    # float32 GEMM large enough for the tensor cores (three tf32 products per
    # product); not one of the five configurations.
    "gemm_f32_tensor": (4096, 4096, 4096),
}
# Tile sizes (TN images x TNF filters per work-group, K block) the conv is run with.
CONV_TILES = (32, 64, 16)

# Reduced shapes for profiler captures (--small): the streaming kernels still
# move more than the 126 MB L2 holds, but a launch lasts tens of microseconds.
SMALL_SHAPES = {
    "softmax": (8192, 4096),
    "reduce": (16384, 8192),
    "gemm_f32": (256, 256, 256),
    "gemm_bf16": (2048, 2048, 2048),
    "gemm_w8a16": (1024, 2048, 2048),
    "conv": (32, 64, 30, 30, 64, 3, 3, 1),
    "map": (8192, 4096),
    "rows": (8192, 4096),
    "gemm_f32_tensor": (2048, 2048, 2048),
}

# Dense tf32 rate of the tensor cores, nominal (no measured figure exists); a
# float32 product costs three tf32 products.
TF32_NOMINAL_TFLOPS = 1125.0

# fp32 FMA rate of the CUDA cores, nominal (no measured figure exists for it):
# 148 SMs x 128 lanes x 2 flop x 1.965 GHz.
FP32_NOMINAL_TFLOPS = 148 * 128 * 2 * 1.965e9 / 1e12

METRIC = {
    "conv": "conv_implicit_gemm_f32_throughput",
    "map": "elementwise_relu_axpby_f32_algorithmic_bandwidth",
    "rows": "row_program_log_softmax_f32_algorithmic_bandwidth",
    "softmax": "softmax_rows_f32_algorithmic_bandwidth",
    "reduce": "reduce_rows_f32_algorithmic_bandwidth",
    "gemm_f32": "gemm_f32_tiled_throughput",
    "gemm_bf16": "gemm_bf16_throughput",
    "gemm_w8a16": "gemm_w8a16_throughput",
    "gemm_f32_tensor": "gemm_f32_3xtf32_throughput",
}
DTYPE = {"softmax": "f32", "reduce": "f32", "gemm_f32": "f32", "gemm_bf16": "bf16",
         "gemm_w8a16": "bf16", "conv": "f32", "map": "f32", "rows": "f32",
         "gemm_f32_tensor": "f32 (3 x tf32)"}


def relu_axpby(a, b):
    """The element-wise body of the ``map`` workload."""
    import numpy as np

    return np.maximum(a * 2.0 - b, 0.0)


def scaled_log_softmax(t):
    """A row body that is NOT compiled ahead of time (the log-softmax of half the
    input): the library compiles it at its first launch."""
    import numpy as np

    shifted = (t - t.max(axis=1, keepdims=True)) * 0.5
    return shifted - np.log(np.exp(shifted).sum(axis=1, keepdims=True))


def leaky_axpby(a, b):
    """An element-wise body that is NOT compiled ahead of time."""
    import numpy as np

    d = a * 2.0 - b
    return np.maximum(d, d * 0.125)


def log_softmax(t):
    """The row body of the ``rows`` workload."""
    import numpy as np

    shifted = t - t.max(axis=1, keepdims=True)
    return shifted - np.log(np.exp(shifted).sum(axis=1, keepdims=True))


def conv_shapes(s):
    """x, f and out shapes of the conv workload tuple."""
    n, c, h, w, nf, hf, wf, stride = s
    return ((n, c, h, w), (nf, c, hf, wf),
            (n, nf, (h - hf) // stride + 1, (w - wf) // stride + 1))


def algorithmic(name):
    """(bytes, flops, bound) one launch of the workload must move / compute."""
    s = SHAPES[name]
    if name == "conv":
        xs, fs, os_ = conv_shapes(s)
        size = lambda shape: shape[0] * shape[1] * shape[2] * shape[3]  # noqa: E731
        return ((size(xs) + size(fs) + size(os_)) * 4,
                2 * size(os_) * fs[1] * fs[2] * fs[3], "tf32x3")
    if name in ("softmax", "rows"):
        m, n = s
        return 2 * m * n * 4, 0, "hbm"
    if name == "map":
        m, n = s
        return 3 * m * n * 4, 0, "hbm"
    if name == "reduce":
        m, n = s
        return m * n * 4 + 2 * m * 4, 0, "hbm"
    m, n, k = s
    if name == "gemm_f32":
        return 3 * m * n * 4, 2 * m * n * k, "latency"
    if name == "gemm_bf16":
        return (m * k + k * n + m * n) * 2, 2 * m * n * k, "tensor"
    if name == "gemm_f32_tensor":
        return (m * k + k * n + m * n) * 4, 2 * m * n * k, "tf32x3"
    return m * k * 2 + k * n + n * 4 + m * n * 2, 2 * m * n * k, "tensor"


def bind_to_gpu_numa_node(local_rank):
    """Restricts this process to the CPUs of the NUMA node that GPU `local_rank` is
    attached to (read from sysfs), so that memory it pins afterwards is local to
    the GPU's PCIe root.  Returns what was done, for the record; never raises."""
    try:
        import torch

        props = torch.cuda.get_device_properties(local_rank)
        bdf = "%04x:%02x:%02x.0" % (props.pci_domain_id, props.pci_bus_id, props.pci_device_id)
        with open(f"/sys/bus/pci/devices/{bdf}/numa_node") as fh:
            node = int(fh.read().strip())
        if node < 0:
            return {"gpu": bdf, "node": node, "bound": False, "why": "no NUMA information"}
        with open(f"/sys/devices/system/node/node{node}/cpulist") as fh:
            cpus = set()
            for part in fh.read().strip().split(","):
                lo, _, hi = part.partition("-")
                cpus.update(range(int(lo), int(hi or lo) + 1))
        allowed = cpus & os.sched_getaffinity(0)
        if not allowed:
            return {"gpu": bdf, "node": node, "bound": False,
                    "why": "none of the node's CPUs is available to this process"}
        os.sched_setaffinity(0, allowed)
        return {"gpu": bdf, "node": node, "bound": True, "cpus": len(allowed)}
    except Exception as err:  # no sysfs, no such attribute: carry on unbound
        return {"bound": False, "why": f"{type(err).__name__}: {err}"}


def unit_of(name):
    return "GB/s" if algorithmic(name)[2] == "hbm" else "TFLOP/s"


def throughput(name, seconds, scale=1.0):
    """Algorithmic throughput in the workload's unit for `scale` x full size."""
    nbytes, flops, bound = algorithmic(name)
    return (nbytes * scale / seconds / 1e9) if bound == "hbm" else (flops * scale / seconds / 1e12)


def describe(name):
    return f"{name} {list(SHAPES[name])} per GPU"


# dram bytes per launch from the ncu captures summarised under profiles/ (None
# where there is no capture of the full-size launch).  The streaming bodies were
# captured at full size, one launch each (profiles/dram_traffic_full_size_streaming_bodies.md);
# the part of the output still in L2 when the kernel ends is not in the figure.
NCU_TRAFFIC = {
    "softmax": 536906496 + 481441280,
    # profiles/reduce_rows_warp_f32_16384x8192.md: (536.89 + 3.88) MB for a quarter of the
    # rows; the read traffic grows with the rows, so four times that.
    "reduce": 2163.1e6,
    # profiles/gemm_umma_full_size_tensor_pipe.md (one full-size launch each; the GEMM kernel
    # alone, without the operand conversion passes of w8a16 and float32).
    "gemm_bf16": 1259.3e6 + 128.1e6,
    "gemm_w8a16": 593.8e6 + 59.8e6,
    "gemm_f32": None,
    "gemm_f32_tensor": 628.8e6 + 61.5e6,
    # profiles/conv_f32_rows_32x64x56x56.md (the convolution kernel alone, one full-size
    # launch: x as hi and lo parts read once; the output was still in L2 at kernel end).
    "conv": 51.7e6 + 1.5e6,
    "map": 1073761280 + 495959040,
    "rows": 536891392 + 481583104,
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


# ---- CPU arm: the oracle (NumPy port of the reference simulator) --------------------------
def cpu_sample(name, threads, repeats):
    """Time the oracle on a bounded sample of workload `name`.

    Returns (throughput in the workload's unit, seconds per pass, description).
    The sample is a block of rows of the full-size problem, so that a pass takes
    a fraction of a second to a few seconds on one host.
    """
    import numpy as np

    from oracle import workloads as oracle

    try:
        from threadpoolctl import threadpool_limits
    except ImportError:  # BLAS then uses its own default thread count
        from contextlib import nullcontext as threadpool_limits

    s = SHAPES[name]
    if name == "softmax":
        rows = min(s[0], 8192 if threads > 1 else 4096)
        (x,) = oracle.make_inputs("softmax", shape=(rows, s[1]))
        out = np.empty_like(x)
        scale = rows / s[0]
        what = f"{rows} of {s[0]} rows"

        def one_pass():
            oracle.run_row_groups_parallel(
                lambda r0, r1: oracle.softmax_rows(x[r0:r1], out[r0:r1], 256), rows, 256, threads)
    elif name == "reduce":
        rows = min(s[0], 8192 if threads > 1 else 4096)
        (x,) = oracle.make_inputs("reduce", shape=(rows, s[1]))
        so, mo = np.empty(rows, np.float32), np.empty(rows, np.float32)
        scale = rows / s[0]
        what = f"{rows} of {s[0]} rows"

        def one_pass():
            oracle.run_row_groups_parallel(
                lambda r0, r1: oracle.reduce_rows(x[r0:r1], so[r0:r1], mo[r0:r1], 256),
                rows, 256, threads)
    elif name == "gemm_f32":
        a, b = oracle.make_inputs("gemm_f32", shape=s)
        out = np.zeros((s[0], s[1]), np.float32)
        scale = 1.0
        what = "the full 256^3 problem, 64x64 groups, KB=16"

        def one_pass():
            oracle.gemm_kblocked(a, b, out, (64, 64), kb=16)
    elif name == "gemm_f32_tensor":
        rows = min(s[0], 512)
        a, b = oracle.make_inputs("gemm_f32", shape=(rows, s[1], s[2]))
        out = np.zeros((rows, s[1]), np.float32)
        scale = rows / s[0]
        what = f"{rows} of {s[0]} rows of A against the full B, 256x256 groups, full K"

        def one_pass():
            oracle.gemm_fullk(a, b, out, (256, 256))
    elif name == "gemm_bf16":
        rows = min(s[0], 512)
        a, b = oracle.make_inputs("gemm_bf16", shape=(rows, s[1], s[2]))
        out = np.zeros((rows, s[1]), np.float32)
        scale = rows / s[0]
        what = f"{rows} of {s[0]} rows of A against the full B, 256x256 groups"

        def one_pass():
            oracle.gemm_bf16(a, b, out, (256, 256))
    elif name == "rows":
        rows = min(s[0], 8192 if threads > 1 else 2048)
        (x,) = oracle.make_inputs("softmax", shape=(rows, s[1]))
        out = np.empty_like(x)
        scale = rows / s[0]
        what = f"{rows} of {s[0]} rows, groups of 256 rows"

        def one_pass():
            oracle.run_row_groups_parallel(
                lambda r0, r1: oracle.rowwise(log_softmax, [x[r0:r1]], out[r0:r1], 256),
                rows, 256, threads)
    elif name == "map":
        rows = min(s[0], 8192 if threads > 1 else 2048)
        a, b = oracle.make_elementwise_inputs(2, (rows, s[1]), "float32")
        out = np.empty_like(a)
        scale = rows / s[0]
        what = f"{rows} of {s[0]} rows, groups of 256 rows"

        def one_pass():
            oracle.run_row_groups_parallel(
                lambda r0, r1: oracle.elementwise(relu_axpby, [a[r0:r1], b[r0:r1]], out[r0:r1],
                                                  (256, s[1])), rows, 256, threads)
    elif name == "conv":
        xs, fs, os_ = conv_shapes(s)
        images = min(xs[0], 4)
        x, f = oracle.make_conv_inputs((images,) + xs[1:], fs, "float32")
        out = np.zeros((images,) + os_[1:], np.float32)
        scale = images / xs[0]
        tn, tnf, kb = min(CONV_TILES[0], images), CONV_TILES[1], CONV_TILES[2]
        what = f"{images} of {xs[0]} images, groups of {tn} images x {tnf} filters, KB={kb}"

        def one_pass():
            oracle.conv_implicit_gemm(x, f, out, s[7], tn, tnf, kb)
    else:
        rows = min(s[0], 256)
        a, w, sc = oracle.make_inputs("gemm_w8a16", shape=(rows, s[1], s[2]))
        out = np.zeros((rows, s[1]), np.float32)
        scale = rows / s[0]
        what = f"{rows} of {s[0]} rows of A against the full W, 256x256 groups"

        def one_pass():
            oracle.gemm_w8a16(a, w, sc, out, (256, 256))

    with threadpool_limits(limits=threads):
        one_pass()
        t0 = time.perf_counter()
        for _ in range(repeats):
            one_pass()
        dt = (time.perf_counter() - t0) / repeats
    return throughput(name, dt, scale), dt, what


def run_reference(args):
    if int(os.environ.get("RANK", "0")) != 0:
        return
    name = args.workload
    threads = len(os.sched_getaffinity(0))
    t0 = time.perf_counter()
    # Heavy samples get fewer passes so that any --steps stays within minutes.
    passes = max(1, min(args.steps, 20 if name in ("softmax", "reduce", "gemm_f32") else 5))
    value, dt, what = cpu_sample(name, threads, passes)
    sample = f"{what}; NumPy oracle on {threads} threads; {passes} timed passes"
    line = {
        "impl": "reference", "metric": METRIC[name], "value": value, "unit": unit_of(name),
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": dt * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": DTYPE[name], "data": "synthetic",
        "config": {"workload": describe(name), "sample_per_step": what},
        "cpu_baseline": {"value": value, "unit": unit_of(name), "cores": threads, "kind": "port",
                         "sample": sample},
        "e2e": {"value": value, "unit": unit_of(name), "h2d_bytes_per_step": 0,
                "d2h_bytes_per_step": 0},
        "wall_s": time.perf_counter() - t0,
    }
    print(json.dumps(line), flush=True)


# ---- GPU arm ----------------------------------------------------------------------------
# Sharding of each workload across ranks (strong scaling: the problem is the
# fixed full-size one, a rank works on its share, every rank ends with the whole
# output).  "rows": the rows of the output (softmax, reductions, row and
# element-wise bodies; M of the bf16 GEMM with B replicated); "cols": N of the
# dequant GEMM with A replicated; "replicas": too small to shard.
SHARDING = {"gemm_f32_tensor": "replicas", "softmax": "rows", "rows": "rows", "map": "rows", "reduce": "rows",
            "gemm_bf16": "rows", "gemm_w8a16": "cols", "gemm_f32": "replicas",
            "conv": "replicas"}

# Row bands per workload at N > 1 (launcher.BandPlan): the all-gather of band b
# overlaps the kernel of band b + 1.
# The HBM-bound bodies take 8 / N bands: their shard's kernel is short against the
# gather, so more bands only add launches.
DEFAULT_BANDS = {"softmax": 0, "rows": 0, "map": 0, "reduce": 1, "gemm_bf16": 2}
# Workloads whose kernel does the output all-gather itself by default (the *_peers
# entry points: stores into every rank's buffer over NVLink); the others gather with
# NCCL.  The GEMMs have such kernels too (`--gather fused-all` uses them), but their
# epilogue writes 64-byte pieces per lane, which NVLink moves at a sixth of the rate
# of the softmax's 512-byte rows, and the stalled epilogue holds the tensor cores
# back: on 2 GPUs 0.61 ms against 0.55 ms with NCCL's gather behind the kernel.
FUSED_GATHER = ("softmax", "reduce")
# ... up to this many GPUs: with 8, every rank of the softmax stores 7 x 64 MiB and the
# step measured 1.07 ms against 0.93 ms for the same bytes through NCCL's all-gather
# behind the kernels (at 4: 0.71 against 0.82).
FUSED_GATHER_MAX_WORLD = {"softmax": 4}
FUSED_GATHER_ALL = ("softmax", "reduce", "gemm_bf16", "gemm_w8a16")
# Which inputs of a row-sharded workload are split by rows (the others are replicated).
ROW_INPUTS = {"softmax": (0,), "rows": (0,), "map": (0, 1), "reduce": (0,), "gemm_bf16": (0,)}


def run_gpu(args):
    import numpy as np
    import torch
    import torch.distributed as dist

    from hc_b200._native import _dispatcher as native
    from hc_b200.hckernel.kernel import get_context
    from hc_b200.launcher import (BandPlan, PeerOutput, ShardedLauncher, init_process_group,
                                  partition)
    from hc_b200.workloads import make_kernels

    rank, world, local = init_process_group()
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE is {world}: launch with torchrun")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    desc = f"cuda:{local}"
    kernels = make_kernels(desc)
    ctx = get_context(desc)
    if args.w8a16_fused:
        ctx.set_option("w8a16_variant", 2)  # convert the weights inside the GEMM's pipeline
    if args.w8a16_variant:
        ctx.set_option("w8a16_variant", args.w8a16_variant)
    stream = torch.cuda.ExternalStream(ctx.stream, device=dev)
    peaks = load_peaks()
    launcher = ShardedLauncher(kernels, rank, world)
    sharded = world > 1 and not args.replicas

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
        """ms for `steps` calls of fn queued from the context's stream (max over
        ranks) and the number of kernel launches they issued."""
        with torch.cuda.stream(stream):
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

    def timed_regions(fn, steps, warmup, min_seconds=0.2, max_regions=64):
        """Regions of exactly `steps` steps, repeated until they cover
        `min_seconds`; returns per-step ms of every region and the launches of one."""
        per_step, launches, total = [], 0, 0.0
        while not per_step or (total < min_seconds * 1e3 and len(per_step) < max_regions):
            ms, launches = timed(fn, steps, warmup if not per_step else 0)
            per_step.append(ms / steps)
            total += ms
        return per_step, launches

    # ---- inputs: the seeded arrays of the benchmark configurations ---------------
    def to_device(array, bf16=False):
        t = torch.from_numpy(np.ascontiguousarray(array)).to(dev)
        return t.bfloat16() if bf16 else t

    inputs_cache = {}

    def baseline_inputs(name):
        if name not in inputs_cache:
            inputs_cache.clear()  # one workload's arrays at a time
            inputs_cache[name] = draw_inputs(name)
        return inputs_cache[name]

    def draw_inputs(name):
        """(host arrays on rank 0 or None, device tensors on every rank, what they
        are).  Rank 0 draws them with the configuration's own generator and seed
        and the other ranks receive them over NCCL, so every GPU works on the
        arrays the parity tests use; workloads outside the five configurations
        draw on the device."""
        s = SHAPES[name]
        config = {"softmax": "softmax", "rows": "softmax", "reduce": "reduce",
                  "gemm_f32": "gemm_f32", "gemm_bf16": "gemm_bf16",
                  "gemm_w8a16": "gemm_w8a16"}.get(name)
        if config is None:
            g = torch.Generator(device=dev).manual_seed(1000)
            if name == "map":
                return None, [torch.randn(*s, device=dev, generator=g) for _ in range(2)], \
                    "torch.randn on the device, seed 1000"
            if name == "gemm_f32_tensor":
                return None, [torch.rand(s[0], s[2], device=dev, generator=g) * 2 - 1,
                              torch.rand(s[2], s[1], device=dev, generator=g) * 2 - 1], \
                    "torch.rand on the device, seed 1000"
            xs, fs, _ = conv_shapes(s)
            return None, [torch.randn(*xs, device=dev, generator=g),
                          torch.randn(*fs, device=dev, generator=g)], \
                "torch.randn on the device, seed 1000"
        kinds = {"gemm_bf16": (True, True), "gemm_w8a16": (True, False, False)}.get(
            name, (False,) * 3)
        host, tensors = None, []
        if rank == 0:
            from oracle import workloads as oracle

            host = oracle.make_inputs(config, shape=s)
            tensors = [to_device(a, bf) for a, bf in zip(host, kinds)]
        if world > 1:
            if len(s) == 2:
                shapes = [s]
            elif name == "gemm_w8a16":
                shapes = [(s[0], s[2]), (s[2], s[1]), (s[1],)]
            else:
                shapes = [(s[0], s[2]), (s[2], s[1])]
            dtypes = {"gemm_bf16": [torch.bfloat16] * 2,
                      "gemm_w8a16": [torch.bfloat16, torch.int8, torch.float32]}.get(
                          name, [torch.float32] * 2)
            if rank != 0:
                tensors = [torch.empty(sh, dtype=dt, device=dev) for sh, dt in zip(shapes, dtypes)]
            for t in tensors:
                dist.broadcast(t, src=0)
        seed = {"gemm_f32": 0, "softmax": 1, "rows": 1, "reduce": 2, "gemm_bf16": 3,
                "gemm_w8a16": 4}[name]
        return host, tensors, f"numpy default_rng({seed}) arrays of the configuration, uploaded"

    conv_cache, rows_cache, map_cache = [], [], []

    def conv_kernel():
        if not conv_cache:
            from hc_b200.hckernel.kernel import sym
            from hc_b200.workloads import make_conv

            tn, tnf, kb = CONV_TILES
            conv_cache.append(make_conv(SHAPES["conv"][7], desc).parametrize(
                {sym.TN: tn, sym.TNF: tnf, sym.KB: kb}))
        return conv_cache[0]

    def rows_kernel():
        if not rows_cache:
            from hc_b200.workloads import make_rowwise

            rows_cache.append(make_rowwise(log_softmax, 1, desc))
        return rows_cache[0]

    def map_kernel():
        if not map_cache:
            from hc_b200.workloads import make_elementwise

            map_cache.append(make_elementwise(relu_axpby, 2, 2, (4, 256), desc))
        return map_cache[0]

    def output_like(name, ins):
        s = SHAPES[name]
        if name in ("softmax", "rows", "map"):
            return [torch.empty(s, device=dev)]
        if name == "reduce":
            return [torch.empty(s[0], device=dev), torch.empty(s[0], device=dev)]
        if name == "conv":
            return [torch.zeros(*conv_shapes(s)[2], device=dev)]
        dtype = torch.float32 if name in ("gemm_f32", "gemm_f32_tensor") else torch.bfloat16
        return [torch.empty(s[0], s[1], device=dev, dtype=dtype)]

    def row_call(name, ins, outs):
        """The C++ dispatcher entry of a workload on row views (no Python front
        door): returns fn(in_views, out_views)."""
        if name == "softmax":
            return lambda i, o: native.softmax_rows(ctx, i[0], o[0])
        if name == "reduce":
            return lambda i, o: native.reduce_rows(ctx, i[0], o[0], o[1])
        if name in ("gemm_f32", "gemm_bf16"):
            return lambda i, o: native.gemm(ctx, i[0], i[1], o[0])
        if name == "gemm_f32_tensor":
            s3 = SHAPES[name]
            need = native.gemm_f32_workspace_bytes(s3[0], s3[1], s3[2])
            raw = torch.empty(need + 1024, dtype=torch.uint8, device=dev)
            ws = raw[(-raw.data_ptr()) % 1024:][:need]
            return lambda i, o: native.gemm(ctx, i[0], i[1], o[0], ws)
        if name == "map":
            roles = map_kernel().plan_for((ins[0], ins[1], outs[0])).roles
            order = roles["inputs"]
            return lambda i, o: native.map_elements(ctx, [i[k] for k in order], o[0],
                                                    roles["code"], roles["consts"])
        if name == "rows":
            roles = rows_kernel().plan_for((ins[0], outs[0], 256)).roles
            return lambda i, o: native.row_program(ctx, [i[0]], o[0], roles["code"],
                                                   roles["consts"])
        if name == "conv":
            # What the @kernel call does with this body: its work-groups form a plain
            # convolution (decided on their index tables), which runs on the tensor cores.
            spec = conv_kernel().plan_for((ins[0], ins[1], outs[0])).roles["spec"]
            stride = spec.as_convolution(tuple(ins[0].shape), tuple(ins[1].shape),
                                         tuple(outs[0].shape))
            if stride is None:
                raise SystemExit("the conv body was not recognised as a convolution")
            need = native.conv_f32_workspace_bytes(*ins[0].shape, ins[1].shape[0],
                                                   *ins[1].shape[2:])
            raw = torch.empty(need + 1024, dtype=torch.uint8, device=dev)
            ws = raw[(-raw.data_ptr()) % 1024:][:need]
            return lambda i, o: native.conv_f32_tensor(ctx, i[0], i[1], o[0], stride, ws)
        spaces = {}

        def w8a16(i, o):
            n, k = i[1].shape[1], i[1].shape[0]
            ws = spaces.get((n, k))
            if ws is None:
                ws = spaces[(n, k)] = torch.empty(native.w8a16_workspace_bytes(n, k),
                                                  dtype=torch.uint8, device=dev)
            native.gemm_w8a16(ctx, i[0], i[1], i[2], o[0], ws)
        return w8a16

    def public_call(name, ins, outs):
        """The same workload through the @kernel call surface."""
        if name == "softmax":
            return lambda: kernels.softmax(ins[0], outs[0], 256)
        if name == "reduce":
            return lambda: kernels.reduce_rows(ins[0], outs[0], outs[1], 256)
        if name == "gemm_f32":
            return lambda: kernels.dot(ins[0], ins[1], outs[0], (64, 64))
        if name in ("gemm_bf16", "gemm_f32_tensor"):
            return lambda: kernels.dot_fullk(ins[0], ins[1], outs[0], (256, 256))
        if name == "conv":
            return lambda: conv_kernel()(ins[0], ins[1], outs[0])
        if name == "map":
            return lambda: map_kernel()(ins[0], ins[1], outs[0])
        if name == "rows":
            return lambda: rows_kernel()(ins[0], outs[0], 256)
        return lambda: kernels.dequant_dot(ins[0], ins[1], ins[2], outs[0], (256, 256))

    def roofline(name, per_step_ms, share=1.0):
        """Throughput of `share` x the full problem done in `per_step_ms`, and the
        roofline record that goes with it."""
        nbytes, flops, bound = algorithmic(name)
        nbytes, flops = nbytes * share, flops * share
        if bound == "hbm":
            ach = nbytes / per_step_ms / 1e6
            return ach, {"bound": "hbm", "achieved": ach, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                         "frac": ach / peaks["hbm_gbs"], "traffic": NCU_TRAFFIC[name],
                         "peak_source": peaks["source"]}
        ach = flops / per_step_ms / 1e9
        if bound == "tf32x3":
            peak = TF32_NOMINAL_TFLOPS / 3
            return ach, {"bound": "tensor (three tf32 products per float32 product)",
                         "achieved": ach, "peak": peak, "unit": "TFLOP/s", "frac": ach / peak,
                         "traffic": NCU_TRAFFIC[name], "peak_source": "nominal tf32 / 3",
                         "cuda_core_peak": FP32_NOMINAL_TFLOPS}
        if bound == "fp32":
            return ach, {"bound": "fp32 CUDA cores", "achieved": ach, "peak": FP32_NOMINAL_TFLOPS,
                         "unit": "TFLOP/s", "frac": ach / FP32_NOMINAL_TFLOPS,
                         "traffic": NCU_TRAFFIC[name], "peak_source": "nominal"}
        return ach, {"bound": "tensor" if bound == "tensor" else "latency", "achieved": ach,
                     "peak": peaks["bf16_tflops"], "unit": "TFLOP/s",
                     "frac": ach / peaks["bf16_tflops"],
                     "frac_of_sustained": ach / peaks["bf16_tflops_sustained"],
                     "traffic": NCU_TRAFFIC[name], "peak_source": peaks["source"]}

    # ---- in-run parity: sampled rows of the output against the CPU oracle -----------
    def oracle_rows(name, host, rows):
        """Expected output rows `rows` (float64 where the bound needs it) and the
        per-element error bound, computed on rank 0 from the host arrays."""
        from oracle import workloads as oracle

        if name == "softmax":
            expect = np.zeros((len(rows), host[0].shape[1]), np.float32)
            oracle.softmax_rows(host[0][rows], expect, 32)
            return [expect], [1e-6 + 1e-5 * np.abs(expect)]
        if name == "rows":
            expect = np.zeros((len(rows), host[0].shape[1]), np.float32)
            oracle.rowwise(log_softmax, [host[0][rows]], expect, 32)
            return [expect], [1e-5 + 1e-5 * np.abs(expect)]
        if name == "reduce":
            x = host[0][rows]
            exact = x.astype(np.float64).sum(axis=1)
            return [exact, x.max(axis=1).astype(np.float64)], \
                [1e-5 * np.abs(x).astype(np.float64).sum(axis=1), np.zeros(len(rows))]
        if name == "gemm_bf16":
            a, b = host
            expect = np.zeros((len(rows), b.shape[1]), np.float32)
            oracle.gemm_bf16(a[rows], b, expect, (256, 256))
            return [expect], [1e-2 * np.abs(expect) + 1e-4 * (np.abs(a[rows]) @ np.abs(b))]
        if name == "gemm_w8a16":
            a, w, sc = host
            expect = np.zeros((len(rows), w.shape[1]), np.float32)
            oracle.gemm_w8a16(a[rows], w, sc, expect, (256, 256))
            mag = np.abs(a[rows]) @ (np.abs(w.astype(np.float32)) * sc)
            return [expect], [1e-2 * np.abs(expect) + 1e-4 * mag]
        if name == "gemm_f32":
            a, b = host
            expect = a[rows].astype(np.float64) @ b.astype(np.float64)
            return [expect], [1e-5 * (np.abs(a[rows]).astype(np.float64)
                                      @ np.abs(b).astype(np.float64))]
        raise ValueError(name)

    def verify(name, host, outs, samples=96):
        """Every rank compares sampled rows of its own copy of the output with the
        oracle's rows (computed once, on rank 0, and sent round)."""
        if name in ("map", "conv", "gemm_f32_tensor"):
            return None  # no host arrays: these are covered by the GPU test-suite only
        m = outs[0].shape[0]
        rows = np.unique(np.r_[0:8, m - 8:m,
                               np.random.default_rng(11).integers(0, m, samples)]).astype(np.int64)
        expect = bound = None
        if rank == 0:
            expect, bound = oracle_rows(name, host, rows)
        if world > 1:
            box = [expect, bound]
            dist.broadcast_object_list(box, src=0)
            expect, bound = box
        index = torch.from_numpy(rows).to(dev)
        worst = 0.0
        for out, e, b in zip(outs, expect, bound):
            got = out[index].double().cpu().numpy()
            err = np.abs(got - e.astype(np.float64))
            if not np.all(err <= b):
                raise AssertionError(f"{name}: rank {rank}: output differs from the oracle on "
                                     f"{int((err > b).sum())} sampled elements")
            scale = np.maximum(b, 1e-300)
            worst = max(worst, float((err / scale).max())) if b.any() else worst
        return {"rows_checked": int(len(rows)), "worst_error_over_bound": worst, "ok": True}

    def other_forms(name, ins, outs, precompiled_call, steps):
        """The same arrays through the two other ways a body can run: interpreted
        (the precompiled body switched off) and compiled at its first launch (a
        body of the same traffic that is not in the ahead-of-time list)."""
        from hc_b200.workloads import make_elementwise, make_rowwise

        nbytes = algorithmic(name)[0]
        figures = {}
        ctx.set_option("fused", 1)
        try:
            ms, _ = timed(precompiled_call, steps, 3)
        finally:
            ctx.set_option("fused", 0)
        figures["interpreted"] = {"ms_per_step": ms / steps, "gbs": nbytes / (ms / steps) / 1e6}
        before = ctx.specialised_programs() + ctx.specialised_programs(True)
        if name == "rows":
            roles = make_rowwise(scaled_log_softmax, 1, desc).plan_for(
                (ins[0], outs[0], 256)).roles
            call = lambda: native.row_program(ctx, [ins[0]], outs[0], roles["code"],  # noqa: E731
                                              roles["consts"])
            body = "log-softmax of (x - max) / 2"
        else:
            roles = make_elementwise(leaky_axpby, 2, 2, (4, 256), desc).plan_for(
                (ins[0], ins[1], outs[0])).roles
            order = roles["inputs"]
            call = lambda: native.map_elements(ctx, [ins[k] for k in order], outs[0],  # noqa: E731
                                               roles["code"], roles["consts"])
            body = "max(d, d / 8) with d = 2a - b"
        t0 = time.perf_counter()
        call()
        torch.cuda.synchronize(dev)
        first_call_s = time.perf_counter() - t0
        ms, _ = timed(call, steps, 3)
        compiled = ctx.specialised_programs() + ctx.specialised_programs(True) - before
        figures["compiled_at_first_launch"] = {
            "body": body, "ms_per_step": ms / steps, "gbs": nbytes / (ms / steps) / 1e6,
            "first_call_s": first_call_s, "programs_compiled": int(compiled),
            "note": ctx.specialise_note or None}
        return figures

    def work_item_bodies(a, out, steps):
        """Two bodies written at work-item level on the first input of the
        element-wise workload, through the @kernel call: one array read, one
        written, each checked against the same arithmetic in torch (the
        operations round once each, so equal means bit for bit)."""
        from hc_b200.workloads import make_work_item_bodies

        bodies = make_work_item_bodies(desc)
        nbytes = 2 * a.numel() * 4
        figures = {}
        for label, call in (("rotate_through_the_group_tile", bodies.rotate),
                            ("stencil_with_the_right_neighbour", bodies.stencil)):
            out.fill_(-77.0)
            t0 = time.perf_counter()
            call(a, out)
            torch.cuda.synchronize(dev)
            first_call_s = time.perf_counter() - t0
            rows = slice(0, 64)  # sixteen rows of groups
            if label.startswith("rotate"):
                tile = (a[rows] + 1.0).view(64, -1, 64)
                want = (torch.roll(tile, -5, dims=2) * 0.5).reshape(64, -1)
            else:
                want = torch.full_like(a[rows], -77.0)
                want[:, :-1] = a[rows, :-1] + a[rows, 1:] * 0.5
            equal = bool(torch.equal(out[rows], want))
            ms, _ = timed(lambda: call(a, out), steps, 3)
            figures[label] = {"ms_per_step": ms / steps, "gbs": nbytes / (ms / steps) / 1e6,
                              "first_call_s": first_call_s, "equals_torch_on_64_rows": equal}
        return figures

    # ---- one workload -----------------------------------------------------------------
    def measure(name, steps, warmup, regions=True):
        """Device-resident throughput of one workload; returns a result dict."""
        host, ins, data = baseline_inputs(name)
        full_outs = output_like(name, ins)
        call = row_call(name, ins, full_outs)
        mode = SHARDING[name] if sharded else "single"
        phases = parity_note = None

        single = lambda: call(ins, full_outs)  # noqa: E731  the whole problem on this GPU
        if mode in ("single", "replicas"):
            step = single
            units = float(world)  # replicas: every rank does the whole problem
        elif mode == "rows":
            m = full_outs[0].shape[0]
            want = args.bands or DEFAULT_BANDS[name] or max(1, 8 // world)
            bands = max(1, want)
            while bands > 1 and m % (bands * world):
                bands //= 2
            plan = BandPlan(m, world, bands)
            # Inputs whose first dimension is the row dimension are sharded; the
            # others (B of the GEMM) are replicated.
            shard_in = [plan.take_shard(t, rank).contiguous() if k in ROW_INPUTS[name] else t
                        for k, t in enumerate(ins)]
            sharded_outs = [torch.empty_like(t) for t in full_outs]
            fused = ((args.gather == "fused" and name in FUSED_GATHER
                      and world <= FUSED_GATHER_MAX_WORLD.get(name, world))
                     or (args.gather == "fused-all" and name in FUSED_GATHER_ALL))
            if fused:
                # Compute and all-gather in one kernel: the contiguous row shard of
                # this rank is written into the full output of every rank.
                plan = BandPlan(m, world, 1)
                span = plan.block(0, rank)
                shard_in = [t[span.begin:span.end].contiguous() if k in ROW_INPUTS[name] else t
                            for k, t in enumerate(ins)]
                if name == "reduce":
                    peer = PeerOutput((2, m), torch.float32, dev)  # sums, then maxima
                    sharded_outs = [peer.tensor[0], peer.tensor[1]]

                    def kernel_only():
                        native.reduce_rows_peers(ctx, shard_in[0], peer.bases(span.begin), m)

                    def compute_only():  # the same kernel writing this rank's copy alone
                        native.reduce_rows_peers(ctx, shard_in[0],
                                                 peer.bases(span.begin)[rank:rank + 1], m)
                else:
                    n_cols = full_outs[0].shape[1]
                    peer = PeerOutput(tuple(full_outs[0].shape), full_outs[0].dtype, dev)
                    sharded_outs = [peer.tensor]
                    if name == "softmax":
                        def kernel_only():
                            native.softmax_rows_peers(ctx, shard_in[0],
                                                      peer.bases(span.begin * n_cols), n_cols)

                        def compute_only():  # the same kernel writing this rank's copy alone
                            native.softmax_rows_peers(
                                ctx, shard_in[0],
                                peer.bases(span.begin * n_cols)[rank:rank + 1], n_cols)
                    else:
                        def kernel_only():
                            native.gemm_bf16_peers(ctx, shard_in[0], shard_in[1],
                                                   peer.bases(span.begin * n_cols), n_cols)

                        def compute_only():
                            native.gemm_bf16_peers(
                                ctx, shard_in[0], shard_in[1],
                                peer.bases(span.begin * n_cols)[rank:rank + 1], n_cols)

                def step(do_compute=True, do_gather=True):
                    if do_compute:
                        kernel_only()
                    if do_gather:
                        peer.fence()
                out = sharded_outs[0]
                gathered = (sum(t.numel() * t.element_size() for t in sharded_outs)
                            * (world - 1) // world)
            elif name == "reduce":
                # One in-place all-gather for both vectors: rank r writes its sums and
                # maxima into pair[r, 0] and pair[r, 1]; two small copies lay them out.
                share = m // world
                pair = torch.empty(world, 2, share, device=dev)

                def compute(band, loc, out_block):
                    call([shard_in[0][loc.begin:loc.end]], [pair[rank, 0], pair[rank, 1]])

                def gather():
                    dist.all_gather_into_tensor(pair.view(world * 2, share), pair[rank])
                    native.copy2d(ctx, pair[:, 0], sharded_outs[0].view(world, share))
                    native.copy2d(ctx, pair[:, 1], sharded_outs[1].view(world, share))

                def step(do_compute=True, do_gather=True):
                    if do_compute:
                        compute(0, plan.local(0, rank), None)
                    if do_gather:
                        gather()
                gathered = 2 * 4 * m * (world - 1) // world
            else:
                def compute(band, loc, out_block):
                    views = [t[loc.begin:loc.end] if k in ROW_INPUTS[name] else t
                             for k, t in enumerate(shard_in)]
                    call(views, [out_block])

                def step(do_compute=True, do_gather=True):
                    if do_compute:
                        launcher.run_rows_pipelined(compute, sharded_outs[0], plan, do_gather)
                    else:
                        pending = [launcher.gather_band(sharded_outs[0], plan, b, async_op=True)
                                   for b in range(plan.bands)]
                        for work in pending:
                            work.wait()
                out = sharded_outs[0]
                gathered = out.numel() * out.element_size() * (world - 1) // world
            units = 1.0
            collective = (
                "none: the kernel writes its rows into every rank's output over NVLink (peer "
                "stores into symmetric memory); a 4-byte ncclAllReduce orders the ranks"
                if fused else
                f"ncclAllGather (torch all_gather_into_tensor, in place), {plan.bands} row "
                f"band(s), each queued behind its kernel")
        else:  # "cols": N of the dequant GEMM
            a, w, sc = ins
            n = w.shape[1]
            span = partition(n, world, rank, align=16)
            if n % (16 * world):
                raise SystemExit("column shards must be equal multiples of 16")
            w_s = w[:, span.begin:span.end]
            sc_s = sc[span.begin:span.end].contiguous()
            out_s = torch.empty(a.shape[0], span.size, device=dev, dtype=torch.bfloat16)
            staging = torch.empty(world, a.shape[0], span.size, device=dev, dtype=torch.bfloat16)
            sharded_outs = [torch.empty_like(full_outs[0])]
            fused = args.gather == "fused-all" and name in FUSED_GATHER_ALL
            if fused:
                # The epilogue writes this rank's column block into every rank's [M, N].
                peer = PeerOutput(tuple(full_outs[0].shape), torch.bfloat16, dev)
                sharded_outs = [peer.tensor]
                ws = torch.empty(native.w8a16_workspace_bytes(span.size, w.shape[0]),
                                 dtype=torch.uint8, device=dev)

                def step(do_compute=True, do_gather=True):
                    if do_compute:
                        native.gemm_w8a16_peers(ctx, a, w_s, sc_s, peer.bases(span.begin), n, ws)
                    if do_gather:
                        peer.fence()
            else:
                def step(do_compute=True, do_gather=True):
                    if do_compute:
                        call([a, w_s, sc_s], [out_s])
                    if do_gather:
                        launcher.gather_cols_even(out_s, staging, sharded_outs[0],
                                                  lambda src, dst: native.copy2d(ctx, src, dst))
            units = 1.0
            gathered = out_s.numel() * 2 * (world - 1)
            collective = (
                "none: the epilogue writes its column block into every rank's output over NVLink "
                "(peer stores into symmetric memory); a 4-byte ncclAllReduce orders the ranks"
                if fused else
                "ncclAllGather of [M, N/g] column blocks into [g, M, N/g], then g strided copies "
                "(hc_copy2d) into [M, N]")

        torch.cuda.synchronize(dev)
        if regions:
            per_step, launches = timed_regions(step, steps, warmup)
        else:
            ms, launches = timed(step, steps, warmup)
            per_step = [ms / steps]
        ms_per_step = statistics.median(per_step)
        value, roof = roofline(name, ms_per_step, units)
        if mode == "replicas":
            roof = roofline(name, ms_per_step)[1]  # the kernel on one GPU
        result = {"ms_per_step": ms_per_step, "steps": steps, "launches": launches,
                  "regions": {"count": len(per_step), "min_ms_per_step": min(per_step),
                              "median_ms_per_step": ms_per_step},
                  "data": data}
        if mode in ("rows", "cols"):
            # Phases, each timed alone: the kernels of the shard, the collective, and
            # (above) the step that overlaps them; and the whole problem on one GPU.
            k_ms, _ = timed(lambda: step(True, False), steps, 2)
            g_ms, _ = timed(lambda: step(False, True), steps, 2)
            one_ms, _ = timed(single, max(3, steps // 2), 2)
            k_ms, g_ms, one_ms = k_ms / steps, g_ms / steps, one_ms / max(3, steps // 2)
            phases = {"kernel_ms": k_ms, "gather_ms": g_ms, "total_ms": ms_per_step,
                      "single_gpu_ms": one_ms, "kernel_speedup": one_ms / k_ms,
                      "total_speedup": one_ms / ms_per_step,
                      "gather_bytes_in_per_rank": gathered,
                      # Bytes every rank receives (and sends) over NVLink per step, over
                      # the phase that moves them: the collective, or - when the kernel
                      # does the gather itself - the kernel.
                      "gather_gbs_in_per_rank": gathered / (k_ms if fused else g_ms) / 1e6,
                      "nvlink_gbs_per_direction": {"nominal": 900, "measured_peer_copy": 770},
                      "fused": bool(fused), "collective": collective}
            if fused and mode == "rows":
                # The kernel phase above includes the stores into the other GPUs; the
                # same kernel writing only this GPU's copy shows how the compute scales.
                c_ms, _ = timed(compute_only, steps, 2)
                phases["compute_only_ms"] = c_ms / steps
                phases["compute_speedup"] = one_ms / (c_ms / steps)
            # The roofline is the kernel's: this GPU's share of the problem in the
            # time its kernels take when nothing else runs.
            roof = roofline(name, k_ms, 1.0 / world)[1]
            roof["of"] = "the kernel phase of one GPU (its 1/%d share of the problem)" % world
            if fused:
                roof["of"] += ("; the kernel also writes its share into the other %d GPUs over "
                               "NVLink, which is what bounds it when the output is large"
                               % (world - 1))
                roof["nvlink_frac_of_measured_peer_copy"] = gathered / k_ms / 1e6 / 770.0
            # Sharded == single GPU, bit for bit, on every rank.
            step()
            single()
            barrier()
            for a_t, b_t in zip(sharded_outs, full_outs):
                if not torch.equal(a_t, b_t):
                    raise AssertionError(f"{name}: rank {rank}: gathered output differs from the "
                                         f"single-GPU output")
            parity_note = "gathered == single-GPU output bit for bit on every rank"
            outs_to_check = sharded_outs
        else:
            single()
            barrier()
            outs_to_check = full_outs
        parity = verify(name, host, outs_to_check)
        if parity and parity_note:
            parity["sharded"] = parity_note
        # Spread of single steps, each between its own pair of events (after the
        # timed regions, so the figures above are untouched).
        events = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
                  for _ in range(min(steps, 50))]
        with torch.cuda.stream(stream):
            for e0, e1 in events:
                e0.record(stream)
                step()
                e1.record(stream)
            stream.synchronize()
        each = sorted(e0.elapsed_time(e1) for e0, e1 in events)
        roof["step_ms"] = {"min": each[0], "median": statistics.median(each), "steps": len(each)}
        result.update({"status": ctx.kernel_status(), "value": value, "unit": roof["unit"],
                       "roofline": roof, "sharding": mode})
        if name in ("rows", "map") and mode == "single" and not args.no_extras:
            result["other_forms"] = other_forms(name, ins, full_outs, single, steps)
            if name == "map":
                result["other_forms"]["work_item_bodies"] = work_item_bodies(
                    ins[0], full_outs[0], steps)
        if name == "conv" and not args.no_extras:
            # The same body as it tiles the problem itself: (images x filters) per output
            # position, every operand element gathered through the index tables.
            spec = conv_kernel().plan_for((ins[0], ins[1], full_outs[0])).roles["spec"]
            tx, tf, to = spec.device_tables((ins[0], ins[1], full_outs[0]))
            tiled = torch.empty_like(full_outs[0])
            g_ms, _ = timed(lambda: native.mapped_gemm(ctx, ins[0], tx, ins[1], tf, tiled, to,
                                                       spec.groups, spec.tm, spec.tn, spec.k),
                            steps, 3)
            flops = algorithmic(name)[1]
            bound = 1e-5 * float(ins[0].abs().max() * ins[1].abs().max()) * spec.k
            worst = float((tiled - full_outs[0]).abs().max())
            result["other_forms"] = {"gathered_as_the_body_tiles_it": {
                "ms_per_step": g_ms / steps, "tflops": flops / (g_ms / steps) / 1e9,
                "max_abs_difference_from_the_tensor_core_result": worst,
                "within_float32_bound": bool(worst <= bound)}}
        if phases:
            result["phases"] = phases
        if parity:
            result["parity"] = parity
        return result

    def measure_e2e(name, steps, warmup):
        """Host buffers in, host buffers out, through the public call surface; with
        several ranks every rank streams its own rows of the problem."""
        _, ins, _ = baseline_inputs(name)
        outs = output_like(name, ins)
        share = 1.0
        if sharded and SHARDING[name] == "rows":
            m = outs[0].shape[0]
            span = partition(m, world, rank)
            ins = [t[span.begin:span.end] if k in ROW_INPUTS[name] else t
                   for k, t in enumerate(ins)]
            outs = [t[span.begin:span.end] for t in outs]
        else:
            share = float(world) if world > 1 else 1.0
        # With several ranks, each one's staging buffers should live on the NUMA node
        # its GPU hangs off: bind the process there before the buffers are made.
        numa = bind_to_gpu_numa_node(local) if world > 1 else None
        h_ins = [t.cpu().pin_memory() for t in ins]
        h_outs = [torch.empty(t.shape, dtype=t.dtype).pin_memory() for t in outs]
        # What the host side alone gives: a pinned-to-pinned copy of the step's output
        # bytes by this rank's cores (every rank at the same time).
        host_gbs = None
        if world > 1 and h_outs:
            twin = torch.empty_like(h_outs[0]).pin_memory()
            barrier()
            t0 = time.perf_counter()
            for _ in range(3):
                twin.copy_(h_outs[0])
            host_gbs = 3 * 2 * twin.numel() * twin.element_size() / (time.perf_counter() - t0) / 1e9
            del twin

        if name in ("softmax", "reduce", "gemm_bf16"):
            # The host-buffer entry points of the C-ABI (hcSoftmaxRowsHost,
            # hcReduceRowsHost, hcGemmBf16Host): row chunks stream through the GPU,
            # upload, kernel and download overlapped, all in the C++ library.
            dev_copies = (ins, outs)  # kept for the link-only measurement below

            def step():
                if name == "softmax":
                    native.softmax_rows_host(ctx, h_ins[0], h_outs[0])
                elif name == "reduce":
                    native.reduce_rows_host(ctx, h_ins[0], h_outs[0], h_outs[1])
                else:
                    native.gemm_bf16_host(ctx, h_ins[0], h_ins[1], h_outs[0])
            via = "C-ABI host-buffer entry point (libhc-b200-kernels.so)"
        elif name in ("map", "rows"):
            # Recorded bodies stream the same way through hc_b200.host (the chunk
            # pipeline around the @kernel call).
            from hc_b200 import host as hc_host

            dev_copies = (ins, outs)

            def step():
                if name == "map":
                    hc_host.rows_body_host(map_kernel(), h_ins, h_outs[0], desc, group_rows=None)
                else:
                    hc_host.rows_body_host(rows_kernel(), h_ins, h_outs[0], desc)
            via = "hc_b200.host chunk pipeline around the @kernel call"
        else:
            call = public_call(name, ins, outs)
            dev_copies = (ins, outs)

            def step():
                for d, h in zip(ins, h_ins):
                    d.copy_(h, non_blocking=True)
                call()
                for h, d in zip(h_outs, outs):
                    h.copy_(d, non_blocking=True)
            via = "copy, @kernel call, copy"

        ms, _ = timed(step, steps, warmup)
        if name == "softmax":  # the result really came back
            sums = h_outs[0][:64].sum(dim=1)
            assert torch.allclose(sums, torch.ones_like(sums), atol=1e-4), "softmax rows != 1"
        ach, roof = roofline(name, ms / steps, share)
        up = sum(t.numel() * t.element_size() for t in h_ins)
        down = sum(t.numel() * t.element_size() for t in h_outs)
        if world > 1:
            t = torch.tensor([up, down], dtype=torch.float64, device=dev)
            dist.all_reduce(t)
            up, down = int(t[0].item()), int(t[1].item())
        # What the link alone allows: the same bytes up and down at once on two
        # streams, nothing computed (every rank at the same time).
        side = torch.cuda.Stream(dev)

        def link_only():
            side.wait_stream(torch.cuda.current_stream(dev))
            for d, h in zip(dev_copies[0], h_ins):
                d.copy_(h, non_blocking=True)
            with torch.cuda.stream(side):
                for h, d in zip(h_outs, dev_copies[1]):
                    h.copy_(d, non_blocking=True)
            torch.cuda.current_stream(dev).wait_stream(side)

        link_ms, _ = timed(link_only, max(3, steps // 2), 1)
        link_ms /= max(3, steps // 2)
        return {"value": ach, "unit": roof["unit"], "h2d_bytes_per_step": up,
                "d2h_bytes_per_step": down, "ms_per_step": ms / steps, "steps": steps,
                "via": via, "link_only_ms_per_step": link_ms,
                "numa": numa, "host_memcpy_gbs_rank0": host_gbs,
                "what": "every rank streams its rows from pinned host memory and back"
                if world > 1 else "pinned host memory in, pinned host memory out"}

    name = args.workload
    sampler = ClockSampler(local)
    with sampler:
        head = measure(name, args.steps, args.warmup)
        e2e = measure_e2e(name, max(3, min(args.steps, 20)), 3)
        extras = {}
        if name == "softmax" and not args.no_extras:
            others = [("reduce", 100), ("gemm_bf16", 50), ("gemm_w8a16", 50), ("gemm_f32", 500),
                      ("gemm_f32_tensor", 20)]
            if not sharded:
                others += [("conv", 50)]
            others += [("map", 100), ("rows", 100)]
            for other, steps in others:
                # Each kernel is timed alone: let the board's power state settle
                # after the previous one (a dense GEMM runs into the 1 kW cap and
                # would hand lower clocks to whatever is measured right after it).
                time.sleep(1.5)
                extras[other] = measure(other, steps, 5)

    if rank == 0:
        mode = SHARDING[name] if sharded else ("replicas" if world > 1 else "single GPU")
        line = {
            "metric": METRIC[name], "value": head["value"], "unit": head["unit"], "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": head["ms_per_step"],
            "higher_is_better": True, "scaling": "strong" if sharded else "weak",
            "vs_baseline": None, "dtype": DTYPE[name], "data": "synthetic: " + head["data"],
            "config": {"workload": describe(name),
                       "sharding": {"rows": "rows of the fixed full-size problem split over the "
                                            "ranks; every rank ends the timed step with the whole "
                                            "output (phases.collective says how)",
                                    "cols": "output columns split over the ranks; every rank ends "
                                            "the timed step with the whole output",
                                    "replicas": "independent replicas, no collective",
                                    "single GPU": "one GPU"}[mode],
                       "l2": {"gemm_f32": "operands fit in L2 (latency-bound case)",
                              "conv": "operands (50 MB) fit in L2; the kernel is bound by "
                                      "compute, not by memory"}.get(
                                  name, "inputs and outputs larger than L2 (no flush needed)")},
            "roofline": head["roofline"], "gpu_launches": head["launches"],
            "kernel_status": head["status"], "regions": head["regions"],
            "clocks": sampler.summary(), "e2e": e2e,
        }
        for key in ("phases", "parity", "other_forms"):
            if key in head:
                line[key] = head[key]
        if args.small:
            line["config"]["small"] = "reduced shape for profiling; not a benchmark result"
        if extras:
            # Short figures first (they survive a truncated record), details after.
            line["summary"] = {k: {"value": round(v["value"], 1), "unit": v["unit"],
                                   "frac": round(v["roofline"]["frac"], 3),
                                   "ms": round(v["ms_per_step"], 4),
                                   **({"kernel_speedup": round(v["phases"]["kernel_speedup"], 2),
                                       "total_speedup": round(v["phases"]["total_speedup"], 2)}
                                      if "phases" in v else {})}
                               for k, v in extras.items()}
            items = extras.get("map", {}).get("other_forms", {}).get("work_item_bodies")
            if items:
                line["summary"]["work_items"] = {
                    k: {"value": round(v["gbs"], 1), "unit": "GB/s",
                        "frac": round(v["gbs"] / load_peaks()["hbm_gbs"], 3)} for k, v in items.items()}
        if world == 1 and not args.no_cpu_baseline:
            value, dt, what = cpu_sample(name, 1, 3)
            line["cpu_baseline"] = {"value": value, "unit": unit_of(name), "cores": 1,
                                    "kind": "port",
                                    "sample": f"{what}; NumPy oracle, single thread, 3 passes"}
        if extras:
            line["workloads"] = extras
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
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--replicas", action="store_true",
                    help="with several GPUs: every rank runs the whole problem on its own "
                         "(weak scaling, no collective) instead of sharding the fixed problem")
    ap.add_argument("--gather", default="fused", choices=["fused", "fused-all", "nccl"],
                    help="how the sharded run assembles the full output on every rank: the "
                         "kernels write into every rank's buffer themselves (peer stores over "
                         "NVLink), or NCCL's all-gather runs behind them")
    ap.add_argument("--bands", type=int, default=0,
                    help="row bands of the sharded run (0: the workload's default)")
    ap.add_argument("--w8a16-fused", action="store_true",
                    help="gemm_w8a16: convert the int8 weights inside the GEMM's pipeline "
                         "(no scratch matrix) instead of in a pass of their own")
    ap.add_argument("--w8a16-variant", type=int, default=0, choices=[0, 1, 2, 3],
                    help="gemm_w8a16: 1 = conversion pass then GEMM (the default), 2 = as "
                         "--w8a16-fused, 3 = converted inside the GEMM kernel band by band "
                         "into a ring of three bands")
    ap.add_argument("--small", action="store_true",
                    help="reduced shapes, for profiler captures; not a benchmark result")
    args = ap.parse_args()
    if args.small:
        SHAPES.update(SMALL_SHAPES)
    if args.impl == "reference":
        run_reference(args)
    else:
        run_gpu(args)


if __name__ == "__main__":
    main()
