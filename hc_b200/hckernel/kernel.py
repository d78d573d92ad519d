"""The ``@kernel`` decorator of the GPU path (reference: ``hckernel/kernel.py``).

Same call surface as the reference::

    @kernel(work_shape=(W, H), backend="nvvm", device="cuda:0")
    def copy_kernel(group: CurrentGroup, src: Buffer[W, H, DT], dst: Buffer[W, H, DT]):
        x, y = group.work_offset
        group.store(dst[x:, y:], group.load(src[x:, y:], shape=group.shape))

    copy_kernel(a, b)          # torch CUDA tensors

(signature and defaults: reference kernel.py:134-142; call: tests/test_e2e.py:
57-75).  Where the reference's dispatcher imports the body's AST and JIT
compiles it (python/cpp/compiler/src/DispatcherBase.cpp:228-280), this one

1. binds the symbols of the ``Buffer[...]`` / tuple / scalar annotations to the
   argument shapes and values and substitutes tunables, as the simulator does
   (reference kernel_sim.py:42-127,144-155);
2. runs the body once with recording objects (:mod:`.kernel_api`);
3. recognises the recorded graph as one of the precompiled kernel families and
   checks that the work-groups together cover the whole arrays, so that one
   whole-array launch computes what all groups would;
4. launches through ``_dispatcher`` (C++), which validates the tensors and
   calls the C-ABI of ``libhc-b200-kernels.so``.

A body that matches no family raises :class:`UnsupportedKernel`; there is no
CPU fallback.  Steps 1-3 are cached per (shapes, dtypes, scalar arguments).
"""

import functools
import inspect
import types
import typing
from collections.abc import Iterable

import sympy

from . import settings
from .kernel_api import *  # noqa: F401,F403  (the reference re-exports kernel_api)
from .elementwise import match_items, match_map, match_rows
from .mapped import match_mapped
from .kernel_api import (
    Affine,
    Buffer,
    BufferRef,
    CurrentGroup,
    CurrentGroup1,
    CurrentGroup2,
    CurrentGroup3,
    CurrentSubGroup,
    CurrentWorkitem,
    Mapping,
    Tile,
    TunableParam,
    UnsupportedKernel,
    _verify_kernel_params,
    dtype_name,
)

__all__ = [
    "kernel", "sym", "typename", "Buffer", "CurrentGroup", "CurrentGroup1", "CurrentGroup2",
    "CurrentGroup3", "CurrentSubGroup", "CurrentWorkitem", "TunableParam", "create_mapping",
    "atomic_ref", "UnsupportedKernel", "Typename", "autotune", "TunedParams",
]

_BACKENDS = {"nvvm": "cuda", "cuda": "cuda"}

# One native context (device + queue + loaded images) per device description.
_contexts = {}

# What a context's options go back to after a call that overrode them.
_DEFAULT_OPTIONS = {"gemm_variant": settings.GEMM_VARIANT}


def get_context(device):
    """The shared native context of ``device`` ("cuda:<ordinal>")."""
    ctx = _contexts.get(device)
    if ctx is None:
        from .._native import _dispatcher

        ctx = _dispatcher.Context(device)
        if settings.GEMM_VARIANT:
            ctx.set_option("gemm_variant", settings.GEMM_VARIANT)
        _contexts[device] = ctx
    return ctx


# ---- symbol binding (reference kernel_sim.py:42-127) ------------------------------
def _bind_symbols(func, args):
    """Symbol -> value from the annotations of ``func`` and the call arguments."""
    subs = {}

    def bind(symbol, value, where):
        if not isinstance(symbol, sympy.Symbol):
            return
        value = int(value)
        if symbol in subs and subs[symbol] != value:
            raise ValueError(
                f"Symbol value conflict for {symbol}: {subs[symbol]} and {value} ({where})"
            )
        subs[symbol] = value

    annotations = inspect.get_annotations(func)
    params = list(inspect.signature(func).parameters)
    for pos, name in enumerate(params[1:]):  # params[0] is the group
        ann = annotations.get(name)
        if ann is None:
            continue
        if pos >= len(args):
            raise TypeError(f"{func.__name__}() missing argument '{name}'")
        value = args[pos]
        if isinstance(ann, sympy.Symbol):
            bind(ann, value, name)
        elif isinstance(ann, type) and issubclass(ann, Buffer):
            shape = tuple(value.shape)
            if len(shape) != len(ann.shape):
                raise ValueError(
                    f"{name}: expected rank {len(ann.shape)} (Buffer{list(ann.shape)}), got "
                    f"shape {list(shape)}"
                )
            for s, v in zip(ann.shape, shape):
                if isinstance(s, sympy.Symbol):
                    bind(s, v, name)
                elif isinstance(s, (int, sympy.Integer)) and int(s) != int(v):
                    raise ValueError(f"{name}: dimension {v} does not match annotation {s}")
        elif isinstance(ann, (tuple, list)) or typing.get_origin(ann) is tuple:
            symbols = typing.get_args(ann) if typing.get_origin(ann) is tuple else ann
            if not isinstance(value, Iterable) or len(tuple(value)) != len(symbols):
                raise ValueError(f"{name}: expected {len(symbols)} values")
            for s, v in zip(symbols, value):
                bind(s, v, name)
        elif ann in (CurrentGroup, CurrentSubGroup, CurrentWorkitem):
            continue
        else:
            raise TypeError(f"Unsupported annotation: {type(ann)} {ann}")
    return subs


def _to_int(value, subs, what):
    if isinstance(value, Iterable):
        return tuple(_to_int(v, subs, what) for v in value)
    if isinstance(value, sympy.Expr):
        value = value.subs(subs)
        if value.free_symbols:
            raise ValueError(f"{what} does not resolve to a number: {value}")
    # A fraction is truncated, as the reference's int() does
    # (kernel_sim.py:121-127); its convolution example relies on it.
    return int(value)


def _resolve_symbols(func, subs, extra, _open=()):
    """``func`` with every global and closure value that is a symbol or symbolic
    expression replaced by its integer value, and ``extra`` objects swapped
    (reference kernel_api.py:43-90 does the same for the simulator).  The
    functions of index mappings are resolved the same way (kernel_api.py:53-54);
    ``_open`` holds the mappings being resolved, so that one that is visible
    from its own function's globals does not recurse for ever."""

    def resolve(value):
        if isinstance(value, sympy.Expr) and value.free_symbols:
            out = value.subs(subs)
            return int(out) if out.is_Integer else out
        if isinstance(value, Mapping):
            if any(value is m for m in _open):
                return value
            return Mapping(_resolve_symbols(value.func, subs, extra, _open + (value,)))
        try:
            return extra.get(value, value)
        except TypeError:  # unhashable
            return value

    closure = func.__closure__
    if closure is not None:
        closure = tuple(types.CellType(resolve(c.cell_contents)) for c in closure)
    new_globals = {k: resolve(v) for k, v in func.__globals__.items()}
    out = types.FunctionType(func.__code__, new_globals, func.__name__, func.__defaults__, closure)
    out.__kwdefaults__ = func.__kwdefaults__
    return functools.update_wrapper(out, func)


def suggest_block_size(global_sizes):
    """The launch-geometry heuristic the reference applies when no group shape
    is given (gpu-runtime/cuda-runtime/src/Runtime.cpp:198-216): dimensions in
    order take what is left of 1024 threads."""
    budget, out = 1024, []
    for g in global_sizes:
        if g <= 1:
            out.append(1)
            continue
        take = min(g, budget)
        out.append(take)
        budget //= 1 << (take - 1).bit_length()
    return tuple(out)


# ---- recognising the recorded graph -------------------------------------------------
class _Plan:
    """What to launch: a family name plus which call arguments play which role."""

    def __init__(self, family, **roles):
        self.family = family
        self.roles = roles

    def __repr__(self):
        return f"<plan {self.family} {self.roles}>"


def _covers(origin, tile_shape, extents, group_counts, what):
    """Check that tiles at ``origin`` (affine in the group ids) of ``tile_shape``
    jointly cover an array of ``extents``: no gaps, full reach, and every
    dimension driven by its own group axis (or by none)."""
    used = set()
    for d, (o, t, e) in enumerate(zip(origin, tile_shape, extents)):
        if o.const != 0 or len(o.coefs) > 1:
            raise UnsupportedKernel(f"{what}: tile origin {o!r} in dimension {d} is not gid*step")
        if not o.coefs:
            if t < e:
                raise UnsupportedKernel(f"{what}: dimension {d} is only covered up to {t} of {e}")
            continue
        ((axis, step),) = o.coefs.items()
        if not isinstance(axis, int):
            raise UnsupportedKernel(f"{what}: tile origin {o!r} depends on the sub-group id alone")
        if axis in used:
            raise UnsupportedKernel(f"{what}: group axis {axis} drives two dimensions")
        used.add(axis)
        if step <= 0 or step > t:
            raise UnsupportedKernel(f"{what}: tiles of {t} placed every {step} leave gaps")
        if step * (group_counts[axis] - 1) + t < e:
            raise UnsupportedKernel(f"{what}: work shape does not reach the end of dimension {d}")


def _is_load(node, ndim=None):
    return isinstance(node, Tile) and node.op == "load" and (ndim is None or node.ndim == ndim)


def _view(node):
    return node.args[0]


def _flatten_sum(node):
    if node.op == "add":
        return _flatten_sum(node.args[0]) + _flatten_sum(node.args[1])
    return [node]


def _match_copy(stores, counts):
    if len(stores) != 1:
        return None
    dst, src = stores[0]
    if not _is_load(src):
        return None
    sv = _view(src)
    if sv.buffer.ndim != 2 or dst.buffer.ndim != 2:
        raise UnsupportedKernel("copy kernels are supported for rank-2 buffers")
    if tuple(sv.origin) != tuple(dst.origin):
        raise UnsupportedKernel("copy with different source and destination origins")
    if sv.buffer.shape != dst.buffer.shape:
        raise UnsupportedKernel("copy between buffers of different shape")
    _covers(dst.origin, src.shape, dst.buffer.shape, counts, "copy")
    return _Plan("copy2d", src=sv.buffer.index, dst=dst.buffer.index)


def _match_softmax(stores, counts):
    if len(stores) != 1:
        return None
    dst, expr = stores[0]
    if expr.op != "div":
        return None
    e, denom = expr.args
    if not (denom.op == "sum" and denom.attrs == {"axis": 1, "keepdims": True}
            and denom.args[0].key() == e.key() and e.op == "exp"):
        return None
    shifted = e.args[0]
    if shifted.op != "sub":
        return None
    x, mx = shifted.args
    if not (_is_load(x, 2) and mx.op == "max" and mx.attrs == {"axis": 1, "keepdims": True}
            and mx.args[0].key() == x.key()):
        return None
    xv = _view(x)
    if x.shape[1] != xv.buffer.shape[1]:
        raise UnsupportedKernel("softmax tiles must hold whole rows")
    if tuple(xv.origin) != tuple(dst.origin) or xv.buffer.shape != dst.buffer.shape:
        raise UnsupportedKernel("softmax input and output tiles differ")
    _covers(dst.origin, x.shape, dst.buffer.shape, counts, "softmax")
    return _Plan("softmax_rows", x=xv.buffer.index, out=dst.buffer.index)


def _match_reduce(stores, counts):
    roles = {}
    source = None
    for dst, expr in stores:
        if expr.op not in ("sum", "max") or expr.attrs != {"axis": 1, "keepdims": False}:
            return None
        x = expr.args[0]
        if not _is_load(x, 2):
            return None
        xv = _view(x)
        if source is None:
            source = x
        elif source.key() != x.key():
            raise UnsupportedKernel("row reductions of different tiles in one kernel")
        if x.shape[1] != xv.buffer.shape[1]:
            raise UnsupportedKernel("row reductions need tiles that hold whole rows")
        if dst.buffer.ndim != 1 or dst.buffer.shape[0] != xv.buffer.shape[0]:
            raise UnsupportedKernel("row reduction output must have one element per row")
        if dst.origin[0] != xv.origin[0]:
            raise UnsupportedKernel("row reduction output offset differs from the row offset")
        role = expr.op + "_out"
        if role in roles:
            raise UnsupportedKernel(f"two {expr.op} outputs")
        roles[role] = dst.buffer.index
    if source is None:
        return None
    xv = _view(source)
    _covers(xv.origin, source.shape, xv.buffer.shape, counts, "row reduction")
    return _Plan("reduce_rows", x=xv.buffer.index, **roles)


def _match_gemm(stores, counts):
    if len(stores) != 1:
        return None
    dst, expr = stores[0]
    scale = None
    if expr.op == "mul":  # dequant form: dot(...) * scale_tile
        lhs, rhs = expr.args
        if _is_load(rhs, 1):
            expr, scale = lhs, rhs
        elif _is_load(lhs, 1):
            expr, scale = rhs, lhs
        else:
            return None
    terms = _flatten_sum(expr)
    dots = [t for t in terms if t.op == "dot"]
    rest = [t for t in terms if t.op != "dot"]
    if not dots:
        return None
    for t in rest:  # only a zero accumulator may be added to the products
        if not (t.op == "alloc" and t.args[0] == 0.0):
            return None
    a_buf = b_buf = None
    spans = []
    widened = False
    for d in dots:
        a, b = d.args
        if b.op == "astype":  # w_tile.astype(float32)
            widened = True
            b = b.args[0]
        if not (_is_load(a, 2) and _is_load(b, 2)):
            return None
        av, bv = _view(a), _view(b)
        if a_buf is None:
            a_buf, b_buf, first_a, first_b = av.buffer, bv.buffer, a, b
        if av.buffer is not a_buf or bv.buffer is not b_buf:
            raise UnsupportedKernel("GEMM terms read different buffers")
        if av.origin[0] != _view(first_a).origin[0] or bv.origin[1] != _view(first_b).origin[1]:
            raise UnsupportedKernel("GEMM terms use different output tiles")
        if a.shape[0] != first_a.shape[0] or b.shape[1] != first_b.shape[1]:
            raise UnsupportedKernel("GEMM terms use different tile sizes")
        ka, kb = av.origin[1], bv.origin[0]
        if not (ka.is_const() and kb.is_const() and ka == kb):
            raise UnsupportedKernel("GEMM K offsets of A and B tiles differ")
        spans.append((ka.const, a.shape[1]))
    m, k = a_buf.shape
    k2, n = b_buf.shape
    if k != k2 or dst.buffer.shape != (m, n):
        raise UnsupportedKernel("GEMM buffer shapes do not form [M,K] @ [K,N] -> [M,N]")
    # The K blocks must partition [0, K): in order, no overlap, no gap.
    reach = 0
    for start, width in sorted(spans):
        if start != reach:
            raise UnsupportedKernel("GEMM K blocks overlap or leave gaps")
        reach += width
    if reach < k:
        raise UnsupportedKernel(f"GEMM K blocks stop at {reach} of {k}")
    mo, no = _view(first_a).origin[0], _view(first_b).origin[1]
    if (mo, no) != tuple(dst.origin):
        raise UnsupportedKernel("GEMM output tile origin differs from its operands")
    _covers(dst.origin, (first_a.shape[0], first_b.shape[1]), (m, n), counts, "GEMM")
    if scale is not None:
        sv = _view(scale)
        if sv.buffer.shape != (n,) or sv.origin[0] != no or scale.shape[0] != first_b.shape[1]:
            raise UnsupportedKernel("dequant scale tile does not line up with the output columns")
        return _Plan("gemm_w8a16", a=a_buf.index, w=b_buf.index, scale=sv.buffer.index,
                     out=dst.buffer.index)
    if widened:
        raise UnsupportedKernel("GEMM with a widened operand but no per-column scale")
    return _Plan("gemm", a=a_buf.index, b=b_buf.index, out=dst.buffer.index)


def _match_reduce_all(atomics, counts):
    """``atomic_ref(result)[0] += tile.sum()`` where the tiles of all groups
    partition a 1-D buffer: no gaps (every element is summed) and no overlap
    (none is summed twice)."""
    if len(atomics) != 1:
        return None
    update = atomics[0]
    expr = update.value
    if expr.op != "sum" or expr.attrs.get("axis") is not None:
        return None
    loads = []
    for term in _flatten_sum(expr.args[0]):
        if term.op == "alloc" and term.args[0] == 0.0:
            continue  # the zero accumulator of the reference's second form
        if not _is_load(term, 1):
            return None
        loads.append(term)
    if not loads:
        return None
    source = _view(loads[0]).buffer
    if source.ndim != 1 or any(_view(t).buffer is not source for t in loads):
        raise UnsupportedKernel("whole-array sum over more than one 1-D buffer")
    if update.buffer is source or tuple(update.index) != (0,) * update.buffer.ndim:
        raise UnsupportedKernel("whole-array sum must accumulate into element 0 of another buffer")
    # Within a group: pieces in order, touching, starting at the group's offset.
    pieces = sorted((_view(t).origin[0].const, t.shape[0], _view(t).origin[0].coefs) for t in loads)
    coefs = pieces[0][2]
    if pieces[0][0] != 0 or len(coefs) > 1 or any(p[2] != coefs for p in pieces):
        raise UnsupportedKernel("whole-array sum: tile offsets are not gid*step + piece")
    reach = 0
    for start, length, _ in pieces:
        if start != reach:
            raise UnsupportedKernel("whole-array sum: tiles overlap or leave gaps inside a group")
        reach += length
    n = source.shape[0]
    if coefs:
        ((axis, step),) = coefs.items()
        if step != reach:
            raise UnsupportedKernel("whole-array sum: groups overlap or leave gaps")
        if step * (counts[axis] - 1) + reach < n:
            raise UnsupportedKernel("whole-array sum: work shape does not reach the end")
    elif reach < n or any(c != 1 for c in counts):
        raise UnsupportedKernel("whole-array sum: a single tile must cover the array once")
    return _Plan("reduce_all", a=source.index, result=update.buffer.index)


def _match_pairwise(stores, counts):
    """``store(out[m0:, n0:], np.linalg.norm(a_t[:, None, :] - b_t[None, :, :], axis=2))``
    with a_t, b_t row blocks of [M, D] and [N, D] that hold whole rows."""
    if len(stores) != 1:
        return None
    dst, expr = stores[0]
    if expr.op != "norm" or expr.attrs != {"axis": 2, "keepdims": False}:
        return None
    diff = expr.args[0]
    if diff.op != "sub":
        return None
    ea, eb = diff.args
    if not (ea.op == "expand" and eb.op == "expand" and ea.attrs["axes"] == (1,)
            and eb.attrs["axes"] == (0,)):
        return None
    a, b = ea.args[0], eb.args[0]
    if not (_is_load(a, 2) and _is_load(b, 2)):
        return None
    av, bv = _view(a), _view(b)
    (m, d), (n, d2) = av.buffer.shape, bv.buffer.shape
    if d != d2 or dst.buffer.shape != (m, n):
        raise UnsupportedKernel("pairwise distance: shapes do not form [M,D], [N,D] -> [M,N]")
    if a.shape[1] != d or b.shape[1] != d or av.origin[1] != 0 or bv.origin[1] != 0:
        raise UnsupportedKernel("pairwise distance tiles must hold whole rows")
    if (av.origin[0], bv.origin[0]) != tuple(dst.origin):
        raise UnsupportedKernel("pairwise distance: output tile origin differs from its operands")
    _covers(dst.origin, (a.shape[0], b.shape[0]), (m, n), counts, "pairwise distance")
    return _Plan("pairwise_distance", a=av.buffer.index, b=bv.buffer.index, out=dst.buffer.index)


_MATCHERS = (_match_copy, _match_softmax, _match_reduce, _match_gemm, _match_pairwise)


# ---- the callable the decorator returns ----------------------------------------------
class KernelDispatcher:
    """Callable returned by :func:`kernel`; plays the role of the reference's
    ``Dispatcher`` (python/cpp/compiler/src/Dispatcher.cpp:20-42)."""

    def __init__(self, func, work_shape, group_shape, subgroup_size, literals, tunables,
                 backend, device, tuned=None, options=None):
        self.options = dict(options or {})  # native launch options chosen by autotune
        self.func = func
        self.work_shape = work_shape
        self.group_shape = group_shape
        self.subgroup_size = subgroup_size
        self.literals = literals
        self.tunables = tunables
        self.backend = backend
        self.device = device
        self.tuned = dict(tuned or {})
        self._plans = {}
        functools.update_wrapper(self, func)

    def parametrize(self, tuned):
        """A copy with tunable symbols fixed (reference kernel_sim.py:165-174).
        ``tuned`` may be the result of :func:`hckernel.autotune.autotune`, which
        also carries native launch options."""
        options = {**self.options, **getattr(tuned, "options", {})}
        return KernelDispatcher(self.func, self.work_shape, self.group_shape, self.subgroup_size,
                                self.literals, self.tunables, self.backend, self.device,
                                {**self.tuned, **tuned}, options)

    # -- steps 1-3 -------------------------------------------------------------------
    def _default_tunables(self):
        t = self.tunables
        if isinstance(t, TunableParam):
            t = (t,)
        return {p.sym: p.default for p in t}

    def plan_for(self, args):
        """The launch plan for these arguments (recording the body on a miss)."""
        key = []
        for a in args:
            if hasattr(a, "shape") and hasattr(a, "dtype"):
                key.append((tuple(a.shape), dtype_name(a.dtype)))
            elif isinstance(a, Iterable):
                key.append(tuple(a))
            else:
                key.append(a)
        key = tuple(key)
        plan = self._plans.get(key)
        if plan is None:
            plan = self._plans[key] = self._record(args)
        return plan

    def _record(self, args):
        subs = {**_bind_symbols(self.func, args), **self._default_tunables(), **self.tuned}
        work = _to_int(self.work_shape if isinstance(self.work_shape, Iterable)
                       else (self.work_shape,), subs, "work_shape")
        if len(work) > 3:
            raise ValueError("work_shape has more than 3 dimensions")
        if self.group_shape is None:
            # Last work dimension is the fastest (x) launch dimension
            # (mlir/lib/Transforms/LowerHKernel.cpp:296,343-344).
            group = tuple(reversed(suggest_block_size(tuple(reversed(work)))))
        else:
            group = _to_int(self.group_shape if isinstance(self.group_shape, Iterable)
                            else (self.group_shape,), subs, "group_shape")
        if len(group) != len(work):
            raise ValueError("work_shape and group_shape differ in rank")
        if any(g <= 0 for g in group):
            raise ValueError(f"group_shape must be positive, got {group}")
        counts = tuple(-(-w // g) for w, g in zip(work, group))

        group_cls = (CurrentGroup1, CurrentGroup2, CurrentGroup3)[len(work) - 1]
        body = _resolve_symbols(self.func, subs, {CurrentGroup: group_cls})
        subgroup = self.subgroup_size
        if subgroup is None:
            subgroup = 16  # the reference simulator's default (kernel_sim.py:10)
        elif not isinstance(subgroup, int):
            subgroup = _to_int(subgroup, subs, "subgroup_size")
        recorder = group_cls(group, subgroup)
        params = list(inspect.signature(self.func).parameters)[1:]
        stand_ins = []
        for i, a in enumerate(args):
            if hasattr(a, "shape") and hasattr(a, "dtype"):
                name = params[i] if i < len(params) else f"arg{i}"
                stand_ins.append(BufferRef(i, name, a.shape, a.dtype, recorder))
            else:
                stand_ins.append(a)
        from . import kernel_api as _api

        _api._RECORDING.append(recorder)
        try:
            body(recorder, *stand_ins)
        finally:
            _api._RECORDING.pop()
        if recorder.refined is not None:
            # A sub-group function ran: its tiles belong to the grid of sub-groups.
            if recorder.item_events or recorder.scatters or recorder.stores_outside_subgroups:
                raise UnsupportedKernel("kernels that mix sub-group functions with stores or "
                                        "updates at group or work-item level")
            counts = tuple(c * (g // t) for c, g, t in zip(counts, group, recorder.refined))
        if recorder.item_events:
            if recorder.stores or recorder.atomics or recorder.scatters:
                raise UnsupportedKernel("kernels that mix work-item stores with tile stores")
            from . import workitems

            found = workitems.match_item_pairwise(recorder)
            if found is not None:
                a, b, out = found
                return _Plan("pairwise_distance", a=a.index, b=b.index, out=out.index)
            if workitems.needs_work_items(recorder):
                program, dst, group2, guards, fill = workitems.match_work_items(recorder, work,
                                                                                group)
                return _Plan("work_items", out=dst.index,
                             inputs=[buffer.index for buffer, _ in program.slots],
                             offsets=[offsets for _, offsets in program.slots],
                             group=group2, code=list(program.code), consts=list(program.consts),
                             guards=guards, tiles=list(program.tile_reads), tile_fill=fill)
            program, dst = match_items(recorder.item_stores, recorder.guards, work)
            return _Plan("map_elements", out=dst.index,
                         inputs=[tile.args[0].index for tile in program.inputs],
                         code=list(program.code), consts=list(program.consts))
        if not recorder.stores and not recorder.atomics and not recorder.scatters:
            raise UnsupportedKernel(f"{self.func.__name__}: the kernel stores nothing")
        if recorder.scatters:
            if recorder.atomics:
                raise UnsupportedKernel("kernels that mix mapped stores and atomic updates")
            spec = match_mapped(recorder.scatters, recorder.stores, counts)
            return _Plan("mapped_gemm", x=spec.x.arg, f=spec.f.arg, out=spec.out.arg, spec=spec)
        if recorder.atomics:
            if recorder.stores:
                raise UnsupportedKernel("kernels that mix stores and atomic updates")
            plan = _match_reduce_all(recorder.atomics, counts)
            if plan is not None:
                return plan
        else:
            for matcher in _MATCHERS:
                plan = matcher(recorder.stores, counts)
                if plan is not None:
                    return plan
            found = match_rows(recorder.stores, counts, _covers)
            if found is not None:
                program, dst = found
                return _Plan("row_program", out=dst.buffer.index,
                             inputs=[tile.args[0].buffer.index for tile in program.inputs],
                             code=list(program.code), consts=list(program.consts))
            found = match_map(recorder.stores, counts, _covers)
            if found is not None:
                program, dst = found
                return _Plan("map_elements", out=dst.buffer.index,
                             inputs=[tile.args[0].buffer.index for tile in program.inputs],
                             code=list(program.code), consts=list(program.consts))
        raise UnsupportedKernel(
            f"{self.func.__name__}: the body matches none of the precompiled kernel families "
            f"(copy, row softmax, last-axis sum/max, whole-array sum, pairwise distance, GEMM, "
            f"tile products gathered through mappings, element-wise tile arithmetic, "
            f"int8 dequant GEMM)"
        )

    # -- step 4 -----------------------------------------------------------------------
    def __call__(self, *args, workspace=None):
        if self.backend not in _BACKENDS:
            raise ValueError(
                f"backend {self.backend!r} is not available: this build drives NVIDIA GPUs "
                f"only (backend='nvvm', device='cuda:<id>')"
            )
        plan = self.plan_for(args)
        from .._native import _dispatcher as native

        ctx = get_context(self.device)
        r = plan.roles
        if plan.family == "mapped_gemm":
            # Upload the index tables (first call only) on torch's stream, before
            # the fence orders the launch after that stream.
            operands = (args[r["x"]], args[r["f"]], args[r["out"]])
            if _tensor_convolution(r["spec"], *operands) is None:
                r["spec"].device_tables(operands)
            else:
                _conv_workspace_for(self.device, operands[0], operands[1])
        fence = _StreamFence(ctx, args)
        fence.before()
        for name, value in self.options.items():
            ctx.set_option(name, value)
        try:
            self._launch(native, ctx, plan, r, args, workspace)
        finally:
            for name in self.options:
                ctx.set_option(name, _DEFAULT_OPTIONS.get(name, 0))
            fence.after()

    def _launch(self, native, ctx, plan, r, args, workspace):
        if plan.family == "copy2d":
            native.copy2d(ctx, args[r["src"]], args[r["dst"]])
        elif plan.family == "softmax_rows":
            native.softmax_rows(ctx, args[r["x"]], args[r["out"]])
        elif plan.family == "reduce_rows":
            native.reduce_rows(ctx, args[r["x"]],
                               args[r["sum_out"]] if "sum_out" in r else None,
                               args[r["max_out"]] if "max_out" in r else None)
        elif plan.family == "reduce_all":
            native.reduce_all(ctx, args[r["a"]], args[r["result"]])
        elif plan.family == "pairwise_distance":
            native.pairwise_distance(ctx, args[r["a"]], args[r["b"]], args[r["out"]])
        elif plan.family == "map_elements":
            native.map_elements(ctx, [args[i] for i in r["inputs"]], args[r["out"]], r["code"],
                                r["consts"])
        elif plan.family == "work_items":
            native.work_items(ctx, [args[i] for i in r["inputs"]], r["offsets"], args[r["out"]],
                              r["group"], r["code"], r["consts"], r["guards"], r["tiles"],
                              r["tile_fill"])
        elif plan.family == "row_program":
            native.row_program(ctx, [args[i] for i in r["inputs"]], args[r["out"]], r["code"],
                               r["consts"])
        elif plan.family == "mapped_gemm":
            spec = r["spec"]
            x, f, out = args[r["x"]], args[r["f"]], args[r["out"]]
            stride = _tensor_convolution(spec, x, f, out)
            if stride is not None:
                # The groups together are a plain float32 convolution: the same sums,
                # tiled by output pixels, on the tensor cores.
                native.conv_f32_tensor(ctx, x, f, out, stride,
                                       _conv_workspace_for(self.device, x, f))
                return
            tx, tf, to = spec.device_tables((x, f, out))
            native.mapped_gemm(ctx, x, tx, f, tf, out, to, spec.groups, spec.tm, spec.tn, spec.k)
        elif plan.family == "gemm":
            a, b = args[r["a"]], args[r["b"]]
            m, k, n = a.shape[0], a.shape[1], b.shape[1]
            # float32 products of at least 1024 each way go to the tensor cores
            # (three tf32 products per product); smaller ones stay on the CUDA
            # cores, where the launch is what they cost.
            if (dtype_name(a.dtype) == "float32" and min(m, n, k) >= _F32_TENSOR_MIN
                    and settings.GEMM_VARIANT != 3):
                if workspace is None:
                    workspace = _f32_workspace_for(self.device, a, m, n, k)
                native.gemm(ctx, a, b, args[r["out"]], workspace)
            else:
                native.gemm(ctx, a, b, args[r["out"]])
        elif plan.family == "gemm_w8a16":
            a, w = args[r["a"]], args[r["w"]]
            if workspace is None:
                workspace = _workspace_for(self.device, w)
            native.gemm_w8a16(ctx, a, w, args[r["scale"]], args[r["out"]], workspace)
        else:  # pragma: no cover
            raise AssertionError(plan.family)


class _StreamFence:
    """Orders a launch on the context's own stream after the work already
    queued on torch's current stream, and torch's later work after the launch -
    on the device, without blocking the host.

    The reference launches on a private non-blocking stream and then blocks
    the host until the kernel is done (python/cpp/py-runtime/src/
    GpuRuntime.cpp:60-69).  Blocking after every launch is what its callers
    get; it is not what a B200 pipeline wants, so the ordering is expressed
    with events instead.  ``HC_SYNC=1`` restores the blocking behaviour.
    """

    _streams = {}

    def __init__(self, ctx, args):
        self.ctx = ctx
        self.torch = None
        if any(getattr(a, "is_cuda", False) for a in args):
            import torch

            self.torch = torch
            key = ctx.stream
            self.ours = _StreamFence._streams.get(key)
            if self.ours is None:
                self.ours = _StreamFence._streams[key] = torch.cuda.ExternalStream(
                    ctx.stream, device=torch.device("cuda", ctx.ordinal))

    def before(self):
        if self.torch is not None:
            self.ours.wait_stream(self.torch.cuda.current_stream(self.ours.device))

    def after(self):
        if self.torch is not None:
            self.torch.cuda.current_stream(self.ours.device).wait_stream(self.ours)
        if settings.SYNC:
            self.ctx.synchronize()


_workspaces = {}
_F32_TENSOR_MIN = 1024


# Convolutions of at least this many multiply-adds go to the tensor-core kernel
# (below, the launch and the filter split cost more than the gathered kernel).
_CONV_TENSOR_MIN = 1 << 24


def _tensor_convolution(spec, x, f, out):
    """The stride, when these mapped work-groups are a float32 convolution that
    hcConvF32Tensor takes (contiguous arrays, at most 256 filters, a tcgen05
    device, large enough, not switched off with HC_CONV_VARIANT=1); else None."""
    import torch

    if settings.CONV_VARIANT == 1 or not all(
            dtype_name(t.dtype) == "float32" and t.dim() == 4 and t.is_contiguous()
            for t in (x, f, out)):
        return None
    if f.shape[0] > 256 or torch.cuda.get_device_capability(x.device)[0] != 10:
        return None
    if out.numel() * f.shape[1] * f.shape[2] * f.shape[3] < _CONV_TENSOR_MIN:
        return None
    return spec.as_convolution(tuple(x.shape), tuple(f.shape), tuple(out.shape))


def _conv_workspace_for(device, x, f):
    """Scratch for the split operands of hcConvF32Tensor, kept per (device, shapes)."""
    import torch
    from .._native import _dispatcher as native

    n, c, h, w = x.shape
    nf, _, hf, wf = f.shape
    need = native.conv_f32_workspace_bytes(n, c, h, w, nf, hf, wf)
    key = (device, "conv", n, c, h, w, nf, hf, wf)
    buf = _workspaces.get(key)
    if buf is None or buf.numel() < need:
        buf = _workspaces[key] = torch.empty(need + 1024, dtype=torch.uint8, device=f.device)
    offset = (-buf.data_ptr()) % 1024  # the entry point wants 1 KiB alignment
    return buf[offset:offset + need]


def _f32_workspace_for(device, a, m, n, k):
    """Scratch for the split operands of a float32 product on the tensor cores,
    kept per (device, M, N, K)."""
    import torch
    from .._native import _dispatcher as native

    need = native.gemm_f32_workspace_bytes(m, n, k)
    key = (device, "f32", m, n, k)
    buf = _workspaces.get(key)
    if buf is None or buf.numel() < need:
        buf = _workspaces[key] = torch.empty(need + 1024, dtype=torch.uint8, device=a.device)
    offset = (-buf.data_ptr()) % 1024  # the entry point wants 1 KiB alignment
    return buf[offset:offset + need]


def _workspace_for(device, w):
    """Scratch for the bf16 copy of the weights, kept per (device, K, N)."""
    import torch
    from .._native import _dispatcher as native

    k, n = w.shape
    need = native.w8a16_workspace_bytes(n, k)
    buf = _workspaces.get((device, k, n))
    if buf is None or buf.numel() < need:
        buf = _workspaces[(device, k, n)] = torch.empty(max(need, 16), dtype=torch.uint8,
                                                        device=w.device)
    return buf


def kernel(
    work_shape,
    group_shape=None,
    subgroup_size=None,
    literals=(),
    tunables=(),
    backend="rocm",
    device="hip:0",
):
    """Decorator with the reference's signature and defaults (kernel.py:134-142).

    The defaults name the reference's HIP backend, which this build does not
    have; pass ``backend="nvvm", device="cuda:<id>"`` as the reference's CUDA
    tests do (tests/test_e2e.py:23-43).
    """
    _verify_kernel_params(work_shape, group_shape, subgroup_size, literals, tunables)

    def decorate(func):
        return KernelDispatcher(func, work_shape, group_shape, subgroup_size, literals, tunables,
                                backend, device)

    return decorate


from .autotune import TunedParams, autotune  # noqa: E402  (needs the names above)
