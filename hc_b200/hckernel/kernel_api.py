"""Objects a kernel body is written against: ``CurrentGroup``, ``Buffer``,
``TunableParam``, ``sym``, ``typename`` ... - the names the reference exports
from ``hckernel/kernel_api.py`` (:21-23, :35-40, :214-220, :255-463).

In the reference these objects have two lives: the simulator executes them on
NumPy, the compiler reads them from the Python AST.  Here they have one: the
body is *run once with recording objects*.  ``group.load`` returns a
:class:`Tile` that remembers where it was loaded from, arithmetic and NumPy
calls on tiles build an expression graph, ``group.store`` appends to the
group's list of stores.  ``hckernel.kernel`` then recognises the recorded
graph as one of the precompiled kernel families (copy, row softmax, last-axis
reductions, GEMM, weight-only dequant GEMM) and launches that kernel on the
whole arrays - or, for tile products gathered through index mappings, one CTA
per work-group.  Nothing is computed on the host.

Semantics the recording keeps from the reference:

* ``group.work_offset[d] == group.id[d] * group.shape[d]``
  (kernel_api.py:293-295) - here an :class:`Affine` expression in the group id,
  so one recording stands for every work-group;
* ``group.load(view, shape)`` reads a tile whose origin is where ``view``
  starts, zero-padded past the array edge (kernel_api.py:297-316);
* ``group.store(view, tile)`` writes the tile clipped to the array
  (kernel_api.py:318-342);
* ``zeros/ones/full/empty`` and their ``v*`` twins allocate tiles
  (kernel_api.py:347-369);
* ``group.load(view, shape, mapping=m)`` gathers: tile element ``index`` is
  ``view[m.func(*index)]`` or zero when that falls outside ``view``
  (kernel_api.py:303-310); ``group.store(view, tile, mapping=m)`` scatters the
  same way and drops what falls outside (kernel_api.py:319-336).  The recording
  keeps the mapping object; the launch plan evaluates it into index tables;
* ``@group.workitems`` (kernel_api.py:395-414): the function is recorded once
  with a :class:`WorkIndex` per axis in place of ``global_id()``; reads and one
  guarded write of the work-item's own element become an element-wise program,
  local ids, neighbour reads and two phases around ``group.barrier()`` a
  work-item program (``hckernel/workitems.py``);
* ``@group.subgroups`` (kernel_api.py:378-393): the function is recorded once with
  the sub-group id as a symbol; the tiles it loads and stores at
  ``work_offset + subgroup_id * (1, ..., size)`` are tiles of the finer grid of
  sub-groups, on which the launch is planned.
"""

import fractions
from collections.abc import Iterable
from math import prod

import numpy as np
import sympy

from .indexing import sym  # noqa: F401  (re-exported, as the reference does)
from .typename import Typename, typename  # noqa: F401


class UnsupportedKernel(NotImplementedError):
    """The body uses a construct no precompiled kernel family provides."""


def _verify_kernel_params(work_shape, group_shape, subgroup_size, literals, tunables):
    # Same two checks as the reference (kernel_api.py:26-32), as exceptions.
    if not (subgroup_size is None or isinstance(subgroup_size, int) or subgroup_size in literals):
        raise AssertionError("Subgroup size must be const or literal")
    if not isinstance(literals, Iterable):
        raise AssertionError(f"literals must iterable, got {literals}")


def _divup(a, b):
    return (a + b - 1) // b


class TunableParam:
    """A symbol the kernel may be tuned over, with its default
    (reference: kernel_api.py:35-40)."""

    def __init__(self, sym, default, vals, strategy=None):
        self.sym = sym
        self.default = default
        self.vals = vals
        self.strategy = strategy


class Buffer(type):
    """``Buffer[M, K, DT]``: an array argument whose shape binds the symbols
    (reference: kernel_api.py:437-447)."""

    def __class_getitem__(cls, shape_and_dtype):
        if not isinstance(shape_and_dtype, tuple) or len(shape_and_dtype) == 0:
            raise AssertionError("Invalid shape and dtype")

        class _Annotated(cls):
            shape = tuple(shape_and_dtype[:-1])
            dtype = shape_and_dtype[-1]

        return _Annotated


class Mapping:
    def __init__(self, func):
        self.func = func


def create_mapping(func):
    """Index mapping for gathering loads and scattering stores (reference:
    kernel_api.py:214-220): ``func(*tile_index)`` gives the index, relative to
    the sliced array, that the tile element is read from or written to."""
    return Mapping(func)


def atomic_ref(a):
    return a


# ---- recording values -----------------------------------------------------------
class Affine:
    """``const + sum(coef[d] * group_id[d])`` with integer coefficients."""

    __slots__ = ("const", "coefs")

    def __init__(self, const=0, coefs=None):
        self.const = int(const)
        self.coefs = {d: int(c) for d, c in (coefs or {}).items() if c}

    @staticmethod
    def of(value):
        if isinstance(value, Affine):
            return value
        if isinstance(value, (int, np.integer)):
            return Affine(int(value))
        if isinstance(value, sympy.Integer):
            return Affine(int(value))
        raise UnsupportedKernel(f"index expression {value!r} is not an integer or group offset")

    def is_const(self):
        return not self.coefs

    def __add__(self, other):
        if isinstance(other, IndexExpr):
            return NotImplemented
        o = Affine.of(other)
        coefs = dict(self.coefs)
        for d, c in o.coefs.items():
            coefs[d] = coefs.get(d, 0) + c
        return Affine(self.const + o.const, coefs)

    __radd__ = __add__

    def __neg__(self):
        return Affine(-self.const, {d: -c for d, c in self.coefs.items()})

    def __sub__(self, other):
        return self + (-Affine.of(other))

    def __rsub__(self, other):
        return Affine.of(other) - self

    def __mul__(self, other):
        if isinstance(other, IndexExpr):
            return NotImplemented
        o = Affine.of(other)
        if o.is_const():
            return Affine(self.const * o.const, {d: c * o.const for d, c in self.coefs.items()})
        if self.is_const():
            return o * self
        return IndexExpr("mul", self, o)

    __rmul__ = __mul__

    def _as_int(self, what):
        if not self.is_const():
            raise UnsupportedKernel(f"{what} of a group offset")
        return self.const

    # `w // W_OUT` and `w % W_OUT` (reference tests/test_examples.py:237-238):
    # the divisor is a constant, possibly a fraction; a group offset on the
    # left makes the result a non-affine IndexExpr.
    def __floordiv__(self, other):
        p, q = _ratio(other, "division")
        if self.is_const():
            return Affine((self.const * q) // p)
        return IndexExpr("floordiv", self, p, q)

    def __mod__(self, other):
        p, q = _ratio(other, "modulo")
        if self.is_const():
            rest = (self.const * q) % p
            if rest % q:
                raise UnsupportedKernel(f"{self.const} % {p}/{q} is not an integer")
            return Affine(rest // q)
        return IndexExpr("mod", self, p, q)

    def evaluate(self, gids):
        """Value for group ids given as one integer array per group axis."""
        out = np.full(np.shape(gids[0]) if len(gids) else (), self.const, dtype=np.int64)
        for d, c in self.coefs.items():
            out = out + c * gids[d]
        return out

    def __index__(self):
        return self._as_int("integer value")

    __int__ = __index__

    def __eq__(self, other):
        try:
            o = Affine.of(other)
        except UnsupportedKernel:
            return NotImplemented
        return self.const == o.const and self.coefs == o.coefs

    def __hash__(self):
        return hash((self.const, tuple(sorted(self.coefs.items()))))

    def key(self):
        return (self.const, tuple(sorted(self.coefs.items())))

    def __repr__(self):
        terms = [str(self.const)] if self.const or not self.coefs else []
        terms += [f"{c}*gid{d}" for d, c in sorted(self.coefs.items(), key=repr)]
        return " + ".join(terms)


def _ratio(value, what):
    """A positive constant divisor as (numerator, denominator)."""
    if isinstance(value, Affine) and value.is_const():
        value = value.const
    if isinstance(value, (int, np.integer, sympy.Integer)):
        p, q = int(value), 1
    elif isinstance(value, sympy.Rational):
        p, q = int(value.p), int(value.q)
    elif isinstance(value, fractions.Fraction):
        p, q = value.numerator, value.denominator
    else:
        raise UnsupportedKernel(f"{what} by {value!r}: the divisor must be a constant")
    if p <= 0:
        raise UnsupportedKernel(f"{what} by the non-positive constant {value}")
    return p, q


class IndexExpr:
    """An integer that depends on the group id in a non-affine way: quotients
    and remainders of group offsets by constants, and sums and products built
    from them.  Evaluated for all work-groups at once when a launch plan is
    made; never needed as a single number while the body is recorded."""

    __slots__ = ("op", "args")

    def __init__(self, op, *args):
        self.op = op
        self.args = args

    @staticmethod
    def of(value):
        return value if isinstance(value, (Affine, IndexExpr)) else Affine.of(value)

    def is_const(self):
        return False

    # The affine view the family matchers read: a non-affine origin fits none.
    @property
    def const(self):
        raise UnsupportedKernel(f"tile origin {self!r} is not affine in the group id")

    coefs = const

    def __add__(self, other):
        return IndexExpr("add", self, IndexExpr.of(other))

    __radd__ = __add__

    def __sub__(self, other):
        return IndexExpr("add", self, IndexExpr.of(other) * -1)

    def __rsub__(self, other):
        return IndexExpr("add", IndexExpr.of(other), self * -1)

    def __neg__(self):
        return self * -1

    def __mul__(self, other):
        return IndexExpr("mul", self, IndexExpr.of(other))

    __rmul__ = __mul__

    def __floordiv__(self, other):
        return IndexExpr("floordiv", self, *_ratio(other, "division"))

    def __mod__(self, other):
        return IndexExpr("mod", self, *_ratio(other, "modulo"))

    def __index__(self):
        raise UnsupportedKernel(f"{self!r} has no single value: it depends on the group id")

    __int__ = __index__

    def key(self):
        return (self.op,) + tuple(a.key() if hasattr(a, "key") else a for a in self.args)

    def __eq__(self, other):
        return isinstance(other, IndexExpr) and self.key() == other.key()

    def __hash__(self):
        return hash(self.key())

    def evaluate(self, gids):
        a = self.args[0].evaluate(gids)
        if self.op == "add":
            return a + self.args[1].evaluate(gids)
        if self.op == "mul":
            return a * self.args[1].evaluate(gids)
        p, q = self.args[1], self.args[2]
        if self.op == "floordiv":
            return (a * q) // p
        rest = (a * q) % p  # self.op == "mod"
        if q != 1:
            if np.any(rest % q):
                raise UnsupportedKernel(f"{self!r} is not an integer for every work-group")
            rest = rest // q
        return rest

    def __repr__(self):
        if self.op in ("add", "mul"):
            sign = " + " if self.op == "add" else " * "
            return f"({self.args[0]!r}{sign}{self.args[1]!r})"
        sign = " // " if self.op == "floordiv" else " % "
        divisor = str(self.args[1]) if self.args[2] == 1 else f"({self.args[1]}/{self.args[2]})"
        return f"({self.args[0]!r}{sign}{divisor})"


def dtype_name(dtype):
    """Canonical element-type name of a torch/NumPy dtype or dtype-like."""
    if isinstance(dtype, str):
        return dtype
    text = str(dtype)
    if text.startswith("torch."):
        return text[len("torch."):]
    try:
        return np.dtype(dtype).name
    except TypeError:
        return text


class BufferRef:
    """Stands for an array argument while the body is recorded."""

    def __init__(self, index, name, shape, dtype, recorder=None):
        self.index = index
        self.name = name
        self.shape = tuple(int(s) for s in shape)
        self.dtype = dtype_name(dtype)
        self.recorder = recorder  # the CurrentGroup that collects element updates

    @property
    def ndim(self):
        return len(self.shape)

    def __len__(self):
        return self.shape[0]

    def _origin(self, key):
        if not isinstance(key, tuple):
            key = (key,)
        if len(key) > self.ndim:
            raise IndexError(f"too many indices for {self.name}")
        origin = []
        for k in key:
            if not isinstance(k, slice):
                raise UnsupportedKernel(
                    f"{self.name}[...]: only `start:` slices select a tile origin; element "
                    f"indexing (e.g. the scalar atomic-reduction form) is not supported"
                )
            if k.stop is not None or k.step is not None:
                raise UnsupportedKernel(f"{self.name}[...]: slices with stop/step are not supported")
            origin.append(IndexExpr.of(0 if k.start is None else k.start))
        origin += [Affine(0)] * (self.ndim - len(origin))
        return tuple(origin)

    @staticmethod
    def _is_element(key):
        keys = key if isinstance(key, tuple) else (key,)
        return len(keys) > 0 and all(isinstance(k, (int, np.integer)) for k in keys)

    def __getitem__(self, key):
        if self._is_element(key):
            # `atomic_ref(result)[0]`: one element, to be updated in place.
            index = tuple(int(k) for k in (key if isinstance(key, tuple) else (key,)))
            if len(index) != self.ndim or any(not 0 <= i < s for i, s in zip(index, self.shape)):
                raise IndexError(f"{self.name}{list(index)} is out of range")
            return ElementRef(self, index)
        item = self._item_axes(key)
        if item is not None:  # `buf[gid]`, `buf[i, j + 1]`, `buf[i]` (a row) at work-item level
            axes, offsets = item
            if len(axes) > self.ndim:
                raise IndexError(f"too many indices for {self.name}")
            attrs = {"axes": axes}
            if any(offsets):
                attrs["offsets"] = offsets
            return Tile("item_load", (self,), self.shape[len(axes):], self.dtype, **attrs)
        return BufferView(self, self._origin(key))

    @staticmethod
    def _item_axes(key):
        """``(work axes, offsets)`` of ``buf[gid]`` / ``buf[i, j]`` / ``buf[i, j + 1]``
        written at work-item level - every index the work-item's global id along
        some axis plus a constant - or None when ``key`` is anything else."""
        keys = key if isinstance(key, tuple) else (key,)
        axes, offsets = [], []
        for k in keys:
            form = index_form(k)
            if form is None or form[0] != "global" or form[2] != 1 or form[4]:
                return None
            axes.append(form[1])
            offsets.append(form[3])
        return (tuple(axes), tuple(offsets)) if keys else None

    def __setitem__(self, key, value):
        # `buf[i] += tile` arrives here after ElementRef.__iadd__.
        if isinstance(value, AtomicUpdate) and self._is_element(key):
            if self.recorder is None:
                raise UnsupportedKernel("element update outside a kernel body")
            if not self.recorder.in_subgroups:
                self.recorder.stores_outside_subgroups += 1
            self.recorder.atomics.append(value)
            return
        item = self._item_axes(key)
        if item is not None:  # `buf[gid] = value` inside a work-item function
            if self.recorder is None:
                raise UnsupportedKernel("element store outside a kernel body")
            axes, offsets = item
            if any(offsets):
                raise UnsupportedKernel(
                    f"{self.name}[...] = value: a work-item may write its own element only")
            self.recorder.item_stores.append((self, axes, Tile._wrap(value)))
            self.recorder.item_events.append(("out", self, axes, Tile._wrap(value)))
            return
        raise UnsupportedKernel(f"direct assignment into {self.name}; use group.store")

    def __repr__(self):
        return f"<buffer {self.name}{list(self.shape)} {self.dtype}>"


class AtomicUpdate:
    """``buffer[index] += value`` recorded as an atomic add."""

    def __init__(self, buffer, index, value):
        self.buffer, self.index, self.value = buffer, index, value


class ElementRef:
    """One element of a buffer; only ``+=`` with a tile expression is recorded
    (the ``atomic_ref(result)[0] += tile.sum()`` idiom of the reference,
    python/hckernel/tests/test_examples.py:40,64)."""

    def __init__(self, buffer, index):
        self.buffer, self.index = buffer, index

    def __iadd__(self, value):
        return AtomicUpdate(self.buffer, self.index, Tile._wrap(value))


class BufferView:
    """``buffer[m0:, k0:]`` - a buffer seen from a tile origin onwards."""

    def __init__(self, buffer, origin):
        self.buffer = buffer
        self.origin = origin

    @property
    def dtype(self):
        return self.buffer.dtype

    @property
    def shape(self):
        raise UnsupportedKernel("shape of a sliced buffer depends on the work-group")

    def key(self):
        return ("view", self.buffer.index, tuple(o.key() for o in self.origin))


def _shape_tuple(shape):
    if isinstance(shape, Iterable):
        return tuple(int(Affine.of(s)) for s in shape)
    return (int(Affine.of(shape)),)


def _broadcast(a, b):
    out = []
    for x, y in zip(((1,) * (len(b) - len(a)) + tuple(a)), ((1,) * (len(a) - len(b)) + tuple(b))):
        if x != y and 1 not in (x, y):
            raise ValueError(f"tile shapes {a} and {b} do not broadcast")
        out.append(max(x, y))
    return tuple(out)


_COMPARISONS = ("lt", "le", "eq", "ne", "ge", "gt")

# The work-group whose body is being recorded (conditions on work-item indices
# are noted there when an `if` asks for their truth).
_RECORDING = []


def index_form(value):
    """``(kind, axis, scale, offset, wrap)`` when ``value`` is a work-item index
    (``kind`` "global" or "local") times a constant plus a constant, optionally
    modulo a constant - ``lid``, ``gid + 1``, ``n - 1 - lid``, ``(lid + 3) % 8`` -
    else None."""
    if isinstance(value, WorkIndex):
        return (value.kind, value.axis, 1, 0, 0)
    if not isinstance(value, Tile):
        return None
    if value.op == "index":
        return (value.attrs.get("kind", "global"), value.attrs["axis"], 1, 0, 0)

    def number(node):
        if isinstance(node, Tile) and node.op == "const" and float(node.args[0]) == int(node.args[0]):
            return int(node.args[0])
        return None

    if value.op == "neg":
        inner = index_form(value.args[0])
        return inner and not inner[4] and (inner[0], inner[1], -inner[2], -inner[3], 0)
    if value.op in ("add", "sub", "mul", "mod") and len(value.args) == 2:
        left, right = value.args
        a, b = index_form(left), index_form(right)
        ca, cb = number(left), number(right)
        if value.op == "add" and a and cb is not None and not a[4]:
            return (a[0], a[1], a[2], a[3] + cb, 0)
        if value.op == "add" and b and ca is not None and not b[4]:
            return (b[0], b[1], b[2], b[3] + ca, 0)
        if value.op == "sub" and a and cb is not None and not a[4]:
            return (a[0], a[1], a[2], a[3] - cb, 0)
        if value.op == "sub" and b and ca is not None and not b[4]:
            return (b[0], b[1], -b[2], ca - b[3], 0)
        if value.op == "mul" and a and cb is not None and not a[4]:
            return (a[0], a[1], a[2] * cb, a[3] * cb, 0)
        if value.op == "mul" and b and ca is not None and not b[4]:
            return (b[0], b[1], b[2] * ca, b[3] * ca, 0)
        if value.op == "mod" and a and cb is not None and cb > 0 and not a[4]:
            return (a[0], a[1], a[2], a[3], cb)
    return None


class Tile:
    """A node of the recorded expression graph.

    ``op`` is one of ``load``, ``alloc``, ``const``, ``add``/``sub``/``mul``/
    ``div``, ``exp``, ``dot``, ``astype``, ``sum``/``max`` (with ``axis`` and
    ``keepdims``), ``gather`` (a load through a mapping), ``slice`` (a tile
    seen from ``offsets`` onwards) and ``window`` (a slice cut or zero-padded
    to a shape by ``vload``).
    """

    __array_priority__ = 1000

    def __init__(self, op, args=(), shape=(), dtype="float32", **attrs):
        self.op = op
        self.args = tuple(args)
        self.shape = tuple(shape)
        self.dtype = dtype
        self.attrs = attrs

    # -- structure ---------------------------------------------------------------
    def key(self):
        parts = []
        for a in self.args:
            parts.append(a.key() if hasattr(a, "key") else ("lit", a))
        return (self.op, tuple(parts), self.shape, tuple(sorted(self.attrs.items())))

    def __repr__(self):
        return f"<tile {self.op}{list(self.shape)} {self.dtype}>"

    @property
    def ndim(self):
        return len(self.shape)

    @property
    def size(self):
        return prod(self.shape)

    # -- arithmetic --------------------------------------------------------------
    @staticmethod
    def _wrap(value):
        if isinstance(value, Tile):
            return value
        if isinstance(value, WorkIndex):
            return value.tile()
        if isinstance(value, (int, float, np.integer, np.floating)):
            return Tile("const", (float(value),), (), "scalar")
        raise UnsupportedKernel(f"operand {value!r} is not a tile or a number")

    def _binary(self, op, other, swapped=False):
        o = Tile._wrap(other)
        lhs, rhs = (o, self) if swapped else (self, o)
        kinds = [d for d in (lhs.dtype, rhs.dtype) if d != "scalar"]
        if kinds == ["bool", "bool"]:
            # Truth values among themselves, as NumPy treats bool arrays.
            if op in ("add", "or", "maximum"):
                op = "or"
            elif op in ("mul", "and", "minimum"):
                op = "and"
            elif op not in _COMPARISONS and op != "xor":
                raise TypeError(f"numpy boolean {op} is not supported; use & | ^ on truth values")
            dtype = "bool"
        else:
            # A truth value (0 / 1) takes the type of what it is combined with.
            others = [d for d in kinds if d != "bool"]
            dtype = others[0] if others else (kinds[0] if kinds else "scalar")
        if op in _COMPARISONS:
            dtype = "bool"
        return Tile(op, (lhs, rhs), _broadcast(lhs.shape, rhs.shape), dtype)

    def __add__(self, o): return self._binary("add", o)
    def __radd__(self, o): return self._binary("add", o, True)
    def __sub__(self, o): return self._binary("sub", o)
    def __rsub__(self, o): return self._binary("sub", o, True)
    def __mul__(self, o): return self._binary("mul", o)
    def __rmul__(self, o): return self._binary("mul", o, True)
    def __truediv__(self, o): return self._binary("div", o)
    def __rtruediv__(self, o): return self._binary("div", o, True)
    def __matmul__(self, o): return _dot(self, o)
    def __neg__(self): return self._unary("neg")
    def __abs__(self): return self._unary("abs")

    def _unary(self, op):
        return Tile(op, (self,), self.shape, self.dtype)

    def __pow__(self, exponent):
        # NumPy computes squares as products and ** 0.5 as a square root.
        if isinstance(exponent, (int, float)) and exponent == 2:
            return self * self
        if isinstance(exponent, (int, float)) and exponent == 0.5:
            return self._unary("sqrt")
        return self._binary("pow", exponent)

    def __rpow__(self, base): return self._binary("pow", base, True)

    # The rest of the reference's operator table (kernel_api.py:157-176).
    # Comparisons give truth values (0 / 1 in the element type once they meet
    # arithmetic); & | ^ are bitwise on integer tiles and logical on truth values.
    def __floordiv__(self, o): return self._binary("floordiv", o)
    def __rfloordiv__(self, o): return self._binary("floordiv", o, True)
    def __mod__(self, o): return self._binary("mod", o)
    def __rmod__(self, o): return self._binary("mod", o, True)
    def __lt__(self, o): return self._binary("lt", o)
    def __le__(self, o): return self._binary("le", o)
    def __eq__(self, o): return self._binary("eq", o)
    def __ne__(self, o): return self._binary("ne", o)
    def __ge__(self, o): return self._binary("ge", o)
    def __gt__(self, o): return self._binary("gt", o)
    def __and__(self, o): return self._binary("and", o)
    def __rand__(self, o): return self._binary("and", o, True)
    def __or__(self, o): return self._binary("or", o)
    def __ror__(self, o): return self._binary("or", o, True)
    def __xor__(self, o): return self._binary("xor", o)
    def __rxor__(self, o): return self._binary("xor", o, True)
    def __lshift__(self, o): return self._binary("lshift", o)
    def __rlshift__(self, o): return self._binary("lshift", o, True)
    def __rshift__(self, o): return self._binary("rshift", o)
    def __rrshift__(self, o): return self._binary("rshift", o, True)
    def __invert__(self): return self._unary("invert")
    __hash__ = object.__hash__  # (nodes are compared through key(), never with ==)

    def __bool__(self):
        # A condition on a work-item index (`if gid + 1 < n:`): the recording
        # takes the branch and notes the range of indices that pass.
        if self.op in _COMPARISONS and _RECORDING:
            left, right = self.args
            for index, other, op in ((index_form(left), right, self.op),
                                     (index_form(right), left,
                                      {"lt": "gt", "le": "ge", "gt": "lt", "ge": "le"}.get(self.op))):
                if (index and op and isinstance(other, Tile) and other.op == "const"
                        and index[0] == "global" and index[2] in (1, -1) and not index[4]):
                    _RECORDING[-1].note_guard(index[1], index[2], index[3], op,
                                              float(other.args[0]))
                    return True
            raise UnsupportedKernel(
                "a condition inside a work-item function must compare the work-item's global "
                "index (plus a constant) with a number")
        # `not tile`, `if tile:` - NumPy's answer for arrays (the reference's
        # operator.not_ entry fails the same way on a tile of several elements).
        raise ValueError("The truth value of a tile with more than one element is ambiguous")

    def __ifloordiv__(self, o): return self._binary("floordiv", o)
    def __imod__(self, o): return self._binary("mod", o)
    def __itruediv__(self, o): return self._binary("div", o)
    # `acc += x` rebinds the name to the new node, like any immutable value.
    def __iadd__(self, o): return self._binary("add", o)
    def __isub__(self, o): return self._binary("sub", o)
    def __imul__(self, o): return self._binary("mul", o)

    def _reduce(self, op, axis, keepdims):
        if axis is None:
            shape = (1,) * self.ndim if keepdims else ()
        else:
            axis = axis % self.ndim
            shape = tuple(
                (1 if i == axis else s) for i, s in enumerate(self.shape) if keepdims or i != axis
            )
        return Tile(op, (self,), shape, self.dtype, axis=axis, keepdims=bool(keepdims))

    def sum(self, axis=None, keepdims=False, **_):
        return self._reduce("sum", axis, keepdims)

    def max(self, axis=None, keepdims=False, **_):
        return self._reduce("max", axis, keepdims)

    def mean(self, axis=None, keepdims=False, **_):
        count = self.size if axis is None else self.shape[axis % self.ndim]
        return self._reduce("sum", axis, keepdims) / float(count)

    def astype(self, dtype, **_):
        return Tile("astype", (self,), self.shape, dtype_name(dtype))

    def copy(self):
        return self

    def _window(self, key):
        """``tile[:, k0:]`` - the tile seen from an offset onwards (to be cut to
        size by ``group.vload(..., shape)``)."""
        if len(key) > self.ndim:
            raise IndexError("too many indices for a tile")
        offsets = []
        for k in key:
            if k.stop is not None or k.step is not None:
                raise UnsupportedKernel("tile slices with stop or step are not supported")
            start = 0 if k.start is None else int(Affine.of(k.start))
            if start < 0:
                raise UnsupportedKernel("tile slices from a negative offset are not supported")
            offsets.append(start)
        offsets += [0] * (self.ndim - len(offsets))
        shape = tuple(max(0, s - o) for s, o in zip(self.shape, offsets))
        return Tile("slice", (self,), shape, self.dtype, offsets=tuple(offsets))

    def __getitem__(self, key):
        # `tile[:, None, :]` (full slices and new axes) or `tile[:, k0:]`.
        if not isinstance(key, tuple):
            key = (key,)
        if all(isinstance(k, slice) for k in key) and any(k != slice(None) for k in key):
            return self._window(key)
        shape, dims = [], iter(self.shape)
        for k in key:
            if k is None:
                shape.append(1)
            elif isinstance(k, slice) and k == slice(None):
                shape.append(next(dims))
            else:
                raise UnsupportedKernel(
                    "slicing a loaded tile is not supported by the precompiled kernels")
        shape.extend(dims)
        if tuple(shape) == self.shape:
            return self
        axes = tuple(i for i, k in enumerate(key) if k is None)
        return Tile("expand", (self,), shape, self.dtype, axes=axes)

    # -- NumPy protocols: np.exp(tile), np.dot(a, b), np.add(a, b) ... -------------
    def __array_ufunc__(self, ufunc, method, *inputs, **kwargs):
        if method != "__call__" or kwargs.get("out") is not None:
            raise UnsupportedKernel(f"np.{ufunc.__name__}.{method} on a tile")
        names = {"add": "add", "subtract": "sub", "multiply": "mul", "true_divide": "div",
                 "divide": "div", "maximum": "maximum", "minimum": "minimum",
                 "floor_divide": "floordiv", "remainder": "mod", "mod": "mod", "power": "pow",
                 "less": "lt", "less_equal": "le", "equal": "eq", "not_equal": "ne",
                 "greater_equal": "ge", "greater": "gt", "bitwise_and": "and",
                 "bitwise_or": "or", "bitwise_xor": "xor", "logical_and": "and",
                 "logical_or": "or", "logical_xor": "xor", "left_shift": "lshift",
                 "right_shift": "rshift"}
        unary = {"exp": "exp", "sqrt": "sqrt", "absolute": "abs", "fabs": "abs",
                 "negative": "neg", "log": "log", "invert": "invert", "bitwise_not": "invert",
                 "logical_not": "invert"}
        if ufunc.__name__ in unary:
            (x,) = inputs
            return x._unary(unary[ufunc.__name__])
        if ufunc.__name__ in names:
            a, b = (Tile._wrap(v) for v in inputs)
            return a._binary(names[ufunc.__name__], b)
        raise UnsupportedKernel(f"np.{ufunc.__name__} on a tile")

    def __array_function__(self, func, types, args, kwargs):
        if func in (np.dot, np.matmul):
            return _dot(*args)
        if func is np.sum:
            return args[0].sum(*args[1:], **kwargs)
        if func in (np.max, np.amax):
            return args[0].max(*args[1:], **kwargs)
        if func is np.mean:
            return args[0].mean(*args[1:], **kwargs)
        if func is np.linalg.norm:
            extra = {k: v for k, v in kwargs.items() if k != "axis" and v is not None and v is not False}
            if len(args) != 1 or extra or not isinstance(kwargs.get("axis"), int):
                raise UnsupportedKernel("np.linalg.norm on a tile: only norm(x, axis=<int>)")
            return args[0]._reduce("norm", kwargs["axis"], False)
        raise UnsupportedKernel(f"np.{func.__name__} on a tile")


class GroupTile(Tile):
    """A tile allocated by the group (``group.zeros`` and friends).  At group
    level it is a constant tile like any other; inside a work-item function it is
    the group's shared storage: ``tile[lid] = value`` before a barrier,
    ``tile.data[n - 1 - lid]`` (or ``tile[...]``) after it."""

    def __init__(self, fill, shape, dtype, recorder):
        super().__init__("alloc", (fill,), shape, dtype)
        self.recorder = recorder

    @property
    def data(self):
        return self

    @staticmethod
    def _local_forms(key):
        keys = key if isinstance(key, tuple) else (key,)
        forms = [index_form(k) for k in keys]
        if keys and all(f is not None and f[0] == "local" for f in forms):
            return tuple(forms)
        return None

    def __setitem__(self, key, value):
        forms = self._local_forms(key)
        if forms is None or not self.recorder.in_workitems:
            raise UnsupportedKernel("a group tile is written as tile[local_id] inside a "
                                    "work-item function")
        if len(forms) != self.ndim or any(f != ("local", d, 1, 0, 0) for d, f in enumerate(forms)):
            raise UnsupportedKernel("a work-item writes the group tile at its own local id only")
        self.recorder.item_events.append(("tile", self, forms, Tile._wrap(value)))

    def __getitem__(self, key):
        forms = self._local_forms(key)
        if forms is not None:
            if len(forms) != self.ndim:
                raise IndexError("a group tile is read with one index per dimension")
            return Tile("tile_read", (self,), (), self.dtype,
                        index=tuple((f[1], f[2], f[3], f[4]) for f in forms))
        return super().__getitem__(key)


def _dot(a, b):
    a, b = Tile._wrap(a), Tile._wrap(b)
    if a.ndim != 2 or b.ndim != 2 or a.shape[1] != b.shape[0]:
        raise ValueError(f"np.dot of tiles shaped {a.shape} and {b.shape}")
    # NumPy's result type: float wins over int, wider wins over narrower.
    order = ["int8", "bfloat16", "float16", "float32", "float64"]
    dtype = max((a.dtype, b.dtype), key=lambda d: order.index(d) if d in order else -1)
    return Tile("dot", (a, b), (a.shape[0], b.shape[1]), dtype)


class CurrentSubGroup:
    """The sub-group a ``group.subgroups`` function sees (reference:
    kernel_api.py:231-240): its size and its id inside the work-group."""

    def __init__(self, size, subgroup_id):
        self._size, self._subgroup_id = size, subgroup_id

    def size(self):
        return self._size

    def subgroup_id(self):
        return self._subgroup_id


class Guard:
    """``gid < bound`` inside a work-item function.  ``if`` asks for its truth:
    the recording takes the branch (the function is recorded for the work-items
    that pass) and notes the bound, which must turn out to be an array bound -
    the only kind of condition a launch over whole arrays can honour."""

    def __init__(self, axis, bound, recorder):
        self.axis, self.bound, self.recorder = axis, bound, recorder

    def __bool__(self):
        self.recorder.guards.append((self.axis, self.bound))
        self.recorder.note_guard(self.axis, 1, 0, "lt", float(self.bound))
        return True


class WorkIndex:
    """One component of ``global_id()`` while a work-item function is recorded:
    it stands for every work-item along that axis at once.  It indexes buffers
    (``buf[gid]``), takes part in arithmetic as the index value, and compares
    against a bound in a guarding ``if``."""

    def __init__(self, axis, recorder, kind="global"):
        self.axis, self.recorder, self.kind = axis, recorder, kind

    def tile(self):
        if self.kind == "local":
            return Tile("index", (), (), "scalar", axis=self.axis, kind="local")
        return Tile("index", (), (), "scalar", axis=self.axis)

    def __lt__(self, bound):
        if self.kind != "global":
            return self.tile() < bound
        return Guard(self.axis, int(Affine.of(bound)), self.recorder)

    def __le__(self, bound):
        if self.kind != "global":
            return self.tile() <= bound
        return Guard(self.axis, int(Affine.of(bound)) + 1, self.recorder)

    def __gt__(self, bound): return self.tile() > bound
    def __ge__(self, bound): return self.tile() >= bound
    def __eq__(self, other): return self.tile() == other
    def __ne__(self, other): return self.tile() != other
    __hash__ = object.__hash__
    def __mod__(self, o): return self.tile() % o
    def __floordiv__(self, o): return self.tile() // o

    def __index__(self):
        raise UnsupportedKernel("a work-item index has no single value while the kernel is recorded")

    __int__ = __index__

    def __add__(self, o): return self.tile() + o
    def __radd__(self, o): return o + self.tile()
    def __sub__(self, o): return self.tile() - o
    def __rsub__(self, o): return o - self.tile()
    def __mul__(self, o): return self.tile() * o
    def __rmul__(self, o): return o * self.tile()
    def __truediv__(self, o): return self.tile() / o
    def __rtruediv__(self, o): return o / self.tile()
    def __neg__(self): return -self.tile()


class CurrentWorkitem:
    """The work-item a ``@group.workitems`` function sees (reference:
    kernel_api.py:243-252), recording instead of iterating."""

    def __init__(self, lid, gid):
        self._local_id, self._global_id = lid, gid

    def local_id(self):
        return self._local_id

    def global_id(self):
        return self._global_id


class CurrentGroup:
    """The work-group a kernel body sees (reference: kernel_api.py:255-434),
    recording instead of computing."""

    def __init__(self, group_shape, subgroup_size):
        self._group_shape = tuple(int(g) for g in group_shape)
        self._subgroup_size = subgroup_size
        self._group_id = tuple(Affine(0, {d: 1}) for d in range(len(self._group_shape)))
        self.stores = []
        self.scatters = []  # stores through a mapping: (view, tile, mapping)
        self.atomics = []
        self.item_stores = []  # `buf[gid] = value` at work-item level: (buffer, axes, tile)
        self.guards = []       # `gid < bound` conditions taken at work-item level: (axis, bound)
        # Everything a work-item function does, in order: ("out", buffer, axes, value),
        # ("tile", group tile, local index forms, value), ("barrier",); and per phase
        # (the stretch before / after a barrier) the index ranges its conditions allow:
        # phase -> axis -> [lo, hi).
        self.item_events = []
        self.item_ranges = [{}]
        self.in_workitems = False
        # Sub-group scope: while a sub-group function is recorded, the group axes
        # stand for the grid of sub-groups (`refined` holds that grid's tile per
        # axis once a sub-group function has run).
        self.in_subgroups = False
        self.refined = None
        self.stores_outside_subgroups = 0

    def note_guard(self, axis, scale, offset, op, bound):
        """``scale * gid[axis] + offset  OP  bound`` was taken as true."""
        lo, hi = self.item_ranges[-1].get(axis, (-(1 << 62), 1 << 62))
        if scale < 0:  # -gid + offset OP bound  <=>  gid  OP'  offset - bound
            op = {"lt": "gt", "le": "ge", "gt": "lt", "ge": "le"}.get(op, op)
            bound = offset - bound
        else:
            bound = bound - offset
        import math

        if op == "lt":
            hi = min(hi, math.ceil(bound))
        elif op == "le":
            hi = min(hi, math.floor(bound) + 1)
        elif op == "gt":
            lo = max(lo, math.floor(bound) + 1)
        elif op == "ge":
            lo = max(lo, math.ceil(bound))
        else:
            raise UnsupportedKernel("work-item indices can be compared with < <= > >= only")
        self.item_ranges[-1][axis] = (lo, hi)

    @property
    def id(self):
        if self.in_subgroups and any(t != g for t, g in zip(self.refined, self._group_shape)):
            raise UnsupportedKernel("group.id inside a sub-group function (use group.work_offset "
                                    "and the sub-group's id)")
        return self._group_id

    @property
    def shape(self):
        return self._group_shape

    @property
    def size(self):
        return prod(self._group_shape)

    @property
    def work_offset(self):
        if self.in_subgroups:
            # Axis d of the recording counts sub-groups: v = id * (shape / tile) + s with
            # s the sub-group's id, so id * shape = (v - s) * tile.  The s terms
            # cancel in `work_offset + s * tile`, the origin of the sub-group's part.
            return tuple(Affine(0, {d: t, ("sg", d): -t}) for d, t in enumerate(self.refined))
        return tuple(g * s for g, s in zip(self._group_id, self._group_shape))

    # -- memory ------------------------------------------------------------------
    def load(self, array, shape, mapping=None):
        if mapping is not None and not isinstance(mapping, Mapping):
            raise TypeError("mapping must come from create_mapping")
        if isinstance(array, Tile):
            # A tile (or a slice of one) loaded again: cut or zero-padded to
            # `shape`, as the reference's load does with any array-like source.
            if mapping is not None:
                raise UnsupportedKernel("a mapping on a load from a tile is not supported")
            base, offsets = array, (0,) * array.ndim
            if array.op == "slice":
                base, offsets = array.args[0], array.attrs["offsets"]
            shape = _shape_tuple(shape)
            if len(shape) != base.ndim:
                raise UnsupportedKernel("load from a tile with a different rank")
            return Tile("window", (base,), shape, base.dtype, offsets=offsets)
        if isinstance(array, BufferRef):
            array = array[()]
        if not isinstance(array, BufferView):
            raise UnsupportedKernel(f"group.load source {array!r} is not a kernel buffer")
        if mapping is not None:
            return Tile("gather", (array,), _shape_tuple(shape), array.dtype, mapping=mapping)
        return Tile("load", (array,), _shape_tuple(shape), array.dtype)

    def vload(self, array, shape, mapping=None):
        return self.load(array, shape, mapping)

    def store(self, dst, src, mapping=None):
        if isinstance(dst, BufferRef):
            dst = dst[()]
        if not isinstance(dst, BufferView):
            raise UnsupportedKernel(f"group.store destination {dst!r} is not a kernel buffer")
        if mapping is not None:
            if not isinstance(mapping, Mapping):
                raise TypeError("mapping must come from create_mapping")
            self.scatters.append((dst, Tile._wrap(src), mapping))
            return
        if not self.in_subgroups:
            self.stores_outside_subgroups += 1
        self.stores.append((dst, Tile._wrap(src)))

    # -- allocators ---------------------------------------------------------------
    def _alloc(self, shape, dtype, fill):
        return GroupTile(float(fill), _shape_tuple(shape), dtype_name(dtype), self)

    def empty(self, shape, dtype): return self._alloc(shape, dtype, 0)
    def zeros(self, shape, dtype): return self._alloc(shape, dtype, 0)
    def ones(self, shape, dtype): return self._alloc(shape, dtype, 1)
    def full(self, shape, dtype, fill_value): return self._alloc(shape, dtype, fill_value)
    def vempty(self, shape, dtype): return self._alloc(shape, dtype, 0)
    def vzeros(self, shape, dtype): return self._alloc(shape, dtype, 0)
    def vones(self, shape, dtype): return self._alloc(shape, dtype, 1)
    def vfull(self, shape, dtype, fill_value): return self._alloc(shape, dtype, fill_value)

    def vec(self, src, shape=None):
        if shape is not None and _shape_tuple(shape) != src.shape:
            raise UnsupportedKernel("group.vec with a different shape")
        return src

    # -- scopes ---------------------------------------------------------------------
    def subgroups(self, func):
        """Sub-group scope (reference kernel_api.py:378-393, which runs ``func``
        once per sub-group: every index of the leading group axes, and
        ``ceil(shape[-1] / subgroup_size)`` pieces of the last one).  ``func`` is
        recorded once; the tiles it loads and stores at
        ``work_offset + subgroup_id * (1, ..., 1, size)`` are the tiles of a finer
        grid of work-groups, one per sub-group, and the launch is planned on that
        grid.  The sub-group size has to divide the last group axis."""
        size = self._subgroup_size
        last = self._group_shape[-1]
        if not isinstance(size, int) or size <= 0:
            raise UnsupportedKernel(f"group.subgroups needs a numeric subgroup_size, got {size!r}")
        if last % size:
            raise UnsupportedKernel(f"a sub-group size of {size} does not divide the group's "
                                    f"last axis ({last})")

        def run():
            if self.in_workitems or self.in_subgroups:
                raise UnsupportedKernel("group.subgroups inside another scope")
            dims = len(self._group_shape)
            self.refined = (1,) * (dims - 1) + (size,)
            self.in_subgroups = True
            try:
                func(CurrentSubGroup(size, tuple(Affine(0, {("sg", d): 1}) for d in range(dims))))
            finally:
                self.in_subgroups = False

        return run

    def workitems(self, func):
        """Work-item scope (reference kernel_api.py:395-414, which runs ``func``
        once per work-item).  Here ``func`` is recorded once, with a
        :class:`WorkIndex` per axis standing for all work-items: what it may do
        is what every work-item can do independently - read ``buf[gid]``,
        compute, write ``buf[gid]`` under a bounds guard."""

        def run():
            dims = range(len(self._group_shape))
            gids = tuple(WorkIndex(d, self) for d in dims)
            lids = tuple(WorkIndex(d, self, "local") for d in dims)
            self.in_workitems = True
            try:
                func(CurrentWorkitem(lids, gids))
            finally:
                self.in_workitems = False

        return run

    def barrier(self):
        """``group.barrier()`` inside a work-item function (reference
        kernel_api.py:416-431): every work-item of the group arrives before any
        goes on.  Splits the function into two phases; values cross it through a
        tile of the group (``group.zeros(...)`` written at ``tile[lid]``)."""
        if not self.in_workitems:
            # At group level nothing runs concurrently, and the sub-groups of a group
            # share nothing that a recorded body can express: nothing to wait for.
            return
        if any(e[0] == "barrier" for e in self.item_events):
            raise UnsupportedKernel("more than one group.barrier() in a work-item function")
        self.item_events.append(("barrier",))
        self.item_ranges.append({})


class CurrentGroup1(CurrentGroup):
    pass


class CurrentGroup2(CurrentGroup):
    pass


class CurrentGroup3(CurrentGroup):
    pass
