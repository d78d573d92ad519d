"""``autotune``: pick kernel hyper-parameters by measuring on the device.

The reference describes this API in its language RFC (docs/langref.md:471-586:
``TunableParam``, ``tunables=`` on the decorator, ``autotune(kernel, *args)``
returning parameters to hand to ``kernel.parametrize``, ``save``/``load``) but
does not implement ``autotune`` itself.  Here it is implemented for what can
actually differ on this backend:

* the symbolic tunables of the decorator (work-group size, items per group,
  K-block ...) select how the *reference* would tile the computation.  The
  precompiled kernels bring their own tiling, so every combination that the
  front door still recognises runs the same device code; ``autotune`` keeps the
  defaults when they are valid and otherwise the first valid combination;
* the native variants of the recognised kernel family - one CTA or a CTA pair
  per GEMM tile, register or bulk-copy softmax, plain or cp.async fp32 GEMM -
  do differ, and are timed with CUDA events on the stream the kernels run on;
* tile products gathered through index mappings (the implicit-GEMM
  convolution) are the exception to the first point: they run one CTA per
  work-group exactly as the body tiles the problem, so for them the symbolic
  tunables are searched and timed, which is what the RFC meant them for.

The result is a :class:`TunedParams`: a ``{symbol: value}`` mapping accepted by
``kernel.parametrize`` that also carries the chosen native options.
"""

import itertools
import json

from .indexing import index_symbol
from .kernel_api import TunableParam, UnsupportedKernel

# Native options worth trying, per recognised family.
_VARIANTS = {
    "gemm": [{"gemm_variant": 1}, {"gemm_variant": 2}, {"tiled_variant": 1}, {"tiled_variant": 2},
             {}],
    "gemm_w8a16": [{"gemm_variant": 1}, {"gemm_variant": 2}],
    "softmax_rows": [{"softmax_variant": 1}, {"softmax_variant": 2}],
    # a warp walks the row / a CTA holds it (on 256 threads; on as few as fit)
    "row_program": [{"row_variant": 1}, {"row_variant": 2}, {"row_variant": 3}],
}


class TunedParams(dict):
    """Tuned symbol values (the mapping itself) plus native launch options."""

    def __init__(self, symbols=(), options=None, timings=None):
        super().__init__(symbols)
        self.options = dict(options or {})
        self.timings = dict(timings or {})  # description -> milliseconds, for inspection

    def save(self, path):
        with open(path, "w") as f:
            json.dump({"symbols": {str(k): int(v) for k, v in self.items()},
                       "options": self.options, "timings_ms": self.timings}, f, indent=1)

    @staticmethod
    def load(path):
        with open(path) as f:
            data = json.load(f)
        return TunedParams({index_symbol(k): int(v) for k, v in data["symbols"].items()},
                           data.get("options"), data.get("timings_ms"))


def _tunable_list(tunables):
    if isinstance(tunables, TunableParam):
        return [tunables]
    return list(tunables)


def _candidate_symbol_sets(kernel, limit):
    tunables = _tunable_list(kernel.tunables)
    yield {t.sym: t.default for t in tunables}
    if not tunables:
        return
    count = 0
    for combo in itertools.product(*(list(t.vals) for t in tunables)):
        if count >= limit:
            return
        count += 1
        yield dict(zip((t.sym for t in tunables), combo))


def _time_call(kernel, args, options, repeats):
    import torch

    from .kernel import get_context

    ctx = get_context(kernel.device)
    stream = torch.cuda.ExternalStream(ctx.stream, device=torch.device("cuda", ctx.ordinal))
    tuned = kernel.parametrize(TunedParams({}, options))
    for _ in range(2):
        tuned(*args)
    ctx.synchronize()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record(stream)
    for _ in range(repeats):
        tuned(*args)
    stop.record(stream)
    ctx.synchronize()
    return start.elapsed_time(stop) / repeats


def _spread_of(tunable):
    """The default, the largest value and the powers of two among a tunable's
    values - a coarse grid that still spans its range."""
    values = set(tunable.vals)
    picks = {tunable.default, max(values)}
    power = 1
    while power <= max(values):
        if power in values:
            picks.add(power)
        power *= 2
    return sorted(picks)


def _tune_mapped_tiles(kernel, args, defaults, repeats, limit):
    """Tile products gathered through mappings run one CTA per work-group, so
    here the symbolic tunables (the tile sizes of the body) are what decides the
    speed: every combination of a coarse grid of their values is recorded, and
    each distinct launch (tile sizes and group counts; tunables that only
    restructure the body's K loop give the same launch) is timed once."""
    tunables = _tunable_list(kernel.tunables)
    timings, timed, best = {}, {}, (dict(defaults), None)
    combos = itertools.islice(itertools.product(*(_spread_of(t) for t in tunables)), limit)
    for combo in itertools.chain([tuple(defaults[t.sym] for t in tunables)], combos):
        symbols = dict(zip((t.sym for t in tunables), combo))
        try:
            spec = kernel.parametrize(symbols).plan_for(args).roles.get("spec")
            if spec is None:
                continue
            launch = (spec.tm, spec.tn, spec.k, spec.counts)
            if launch not in timed:
                timed[launch] = _time_call(kernel.parametrize(symbols), args, {}, repeats)
                timings[json.dumps({str(k): int(v) for k, v in symbols.items()},
                                   sort_keys=True)] = timed[launch]
        except (UnsupportedKernel, ValueError, RuntimeError):
            continue  # a combination the front door or the launcher refuses
        if best[1] is None or timed[launch] < best[1]:
            best = (symbols, timed[launch])
    return TunedParams(best[0], {}, timings)


def autotune(kernel, *args, repeats=5, max_symbol_sets=256):
    """Tuned parameters of ``kernel`` for arguments shaped like ``args``.

    ``args`` are real device tensors (they are overwritten by the timed runs).
    """
    chosen = None
    for symbols in _candidate_symbol_sets(kernel, max_symbol_sets):
        try:
            plan = kernel.parametrize(symbols).plan_for(args)
        except (UnsupportedKernel, ValueError):
            continue
        chosen = (symbols, plan)
        break
    if chosen is None:
        raise UnsupportedKernel(
            f"{kernel.func.__name__}: no combination of tunables gives a supported kernel")
    symbols, plan = chosen
    if plan.family == "mapped_gemm":
        return _tune_mapped_tiles(kernel, args, symbols, repeats, max_symbol_sets)
    timings, best = {}, ({}, None)
    for options in _VARIANTS.get(plan.family, [{}]):
        try:
            ms = _time_call(kernel.parametrize(symbols), args, options, repeats)
        except RuntimeError:  # a variant that cannot run these shapes
            continue
        timings[json.dumps(options, sort_keys=True)] = ms
        if best[1] is None or ms < best[1]:
            best = (options, ms)
    return TunedParams(symbols, best[0], timings)


autotune.load = TunedParams.load
