"""CPU oracle: a NumPy restatement of the reference's kernel simulator.

TEST INFRASTRUCTURE ONLY.  Nothing in the ``hc_b200`` package imports this
module; it exists so that tests, ``__graft_entry__.smoke()`` and the CPU-baseline
leg of ``bench.py`` can check (and time) what the reference computes.  The
product path has no CPU fallback.

What is restated, and from where (paths are relative to the reference tree):

* work-group enumeration - ``ceil(work/group)`` groups per dimension, visited in
  row-major order, each seeing ``work_offset = group_id * group_shape``
  (python/hckernel/kernel_sim.py:13-14, 159-163;
  python/hckernel/kernel_api.py:293-295);
* ``group.load`` - a zero-filled tile of the requested shape, the in-bounds part
  copied from the array view, a mask marking which elements are real
  (python/hckernel/kernel_api.py:297-316);
* ``group.store`` - the tile clipped to the destination view; with a masked
  source only the valid elements are written
  (python/hckernel/kernel_api.py:318-342);
* ``group.load`` / ``group.store`` through an index mapping - element-wise
  gather and scatter with out-of-range indices masked or dropped
  (python/hckernel/kernel_api.py:303-310, 319-336);
* tile allocators ``zeros``/``full`` (python/hckernel/kernel_api.py:347-369,
  433-434);
* masked reductions that ignore padding (numpy.ma behaviour reached through
  python/hckernel/kernel_api.py:150-151).

Parity pin: ``tests/golden/make_golden.py`` runs the reference simulator itself
(imported from the reference tree) and this restatement on the same inputs and
stores the reference's outputs; ``tests/test_oracle_golden.py`` then checks this
module against those stored outputs bit for bit, including the reference's own
test vectors for dot, softmax and reduction
(python/hckernel/tests/test_examples.py:31-165, 304-335).  The row-max, bf16
and int8-dequant workloads have no test in the reference; their golden outputs
come from the same workload written in the reference's DSL and run on the
reference simulator, so they pin this restatement to the reference's tile
semantics, not to an independent known answer.
"""

from __future__ import annotations

from dataclasses import dataclass
from itertools import product

import operator

import numpy as np


def ceil_div(a: int, b: int) -> int:
    return -(-a // b)


def iter_groups(work_shape, group_shape):
    """Yield ``(group_id, work_offset)`` in the simulator's order.

    python/hckernel/kernel_sim.py:13-14 (group count) and :159-163 (row-major
    ``product`` over the group ranges); offsets as in
    python/hckernel/kernel_api.py:293-295.
    """
    work_shape = tuple(np.atleast_1d(work_shape).tolist())
    group_shape = tuple(np.atleast_1d(group_shape).tolist())
    if len(work_shape) != len(group_shape):
        raise ValueError("work_shape and group_shape differ in rank")
    counts = [ceil_div(w, g) for w, g in zip(work_shape, group_shape)]
    for gid in product(*(range(c) for c in counts)):
        yield gid, tuple(i * g for i, g in zip(gid, group_shape))


@dataclass
class Tile:
    """A work-group tile: values plus a validity mask (True = real element)."""

    data: np.ndarray
    valid: np.ndarray

    @property
    def shape(self):
        return self.data.shape


def load_tile(view: np.ndarray, shape) -> Tile:
    """``group.load(view, shape)``: python/hckernel/kernel_api.py:297-316.

    ``view`` is the array sliced so that it starts at the tile origin; the tile
    is zero-filled (``_get_uninit_value`` returns 0, kernel_api.py:222-223) and
    only the part that exists in ``view`` is copied and marked valid.
    """
    shape = tuple(np.atleast_1d(shape).tolist())
    data = np.zeros(shape, dtype=view.dtype)
    valid = np.zeros(shape, dtype=bool)
    inside = tuple(slice(0, min(have, want)) for have, want in zip(view.shape, shape))
    data[inside] = view[inside]
    valid[inside] = True
    return Tile(data, valid)


class ArithmeticTile:
    """A tile as the reference's arithmetic sees it: a thin wrapper around a
    ``numpy.ma`` array (python/hckernel/kernel_api.py:106-211).

    Operators go to ``numpy.ma`` and give a wrapped tile again (:136-148,
    :157-211; there are no reflected operators, so ``1.0 + tile`` is an error
    there and here).  NumPy functions reach the masked array through
    ``__array__`` (:150-151) and return a bare masked array, which ``store``
    then treats as a plain array (:338-342).  Consequences kept on purpose:
    a Python float operand becomes a float64 array inside ``numpy.ma``, so
    ``tile_f32 * 2.0`` continues in float64 until it is stored.
    """

    def __init__(self, masked):
        self.ma = masked

    def __array__(self, dtype=None, copy=None):
        return self.ma if dtype is None else self.ma.astype(dtype)

    def _binary(self, other, op):
        return ArithmeticTile(op(self.ma, other.ma if isinstance(other, ArithmeticTile) else other))

    def __add__(self, other): return self._binary(other, np.ma.add)
    def __sub__(self, other): return self._binary(other, np.ma.subtract)
    def __mul__(self, other): return self._binary(other, np.ma.multiply)
    def __truediv__(self, other): return self._binary(other, np.ma.true_divide)
    def __neg__(self): return ArithmeticTile(-self.ma)
    def __abs__(self): return ArithmeticTile(abs(self.ma))

    # The rest of the reference's operator table (kernel_api.py:157-176): the
    # Python operator applied to the masked arrays.  Division-like operators
    # mask the elements whose divisor is zero, ``**`` those whose result is not
    # finite (numpy.ma's domains); the masked store then leaves them unwritten.
    def __floordiv__(self, other): return self._binary(other, operator.floordiv)
    def __mod__(self, other): return self._binary(other, operator.mod)
    def __pow__(self, other): return self._binary(other, operator.pow)
    def __lt__(self, other): return self._binary(other, operator.lt)
    def __le__(self, other): return self._binary(other, operator.le)
    def __eq__(self, other): return self._binary(other, operator.eq)
    def __ne__(self, other): return self._binary(other, operator.ne)
    def __ge__(self, other): return self._binary(other, operator.ge)
    def __gt__(self, other): return self._binary(other, operator.gt)
    def __and__(self, other): return self._binary(other, operator.and_)
    def __or__(self, other): return self._binary(other, operator.or_)
    def __xor__(self, other): return self._binary(other, operator.xor)
    def __lshift__(self, other): return self._binary(other, operator.lshift)
    def __rshift__(self, other): return self._binary(other, operator.rshift)
    def __invert__(self): return ArithmeticTile(~self.ma)
    __hash__ = None

    def __getattr__(self, name):
        return getattr(self.ma, name)


def arithmetic_tile(tile: Tile) -> ArithmeticTile:
    return ArithmeticTile(np.ma.masked_array(tile.data, mask=~tile.valid))


def store_result(dst_view: np.ndarray, result) -> None:
    """``group.store`` of whatever tile arithmetic produced: a wrapped tile
    writes its unmasked elements only, anything else is assigned as it is
    (python/hckernel/kernel_api.py:338-342)."""
    if isinstance(result, ArithmeticTile):
        mask = np.ma.getmaskarray(result.ma)
        store_tile(dst_view, Tile(np.asarray(result.ma.data), ~mask))
    else:
        store_tile(dst_view, np.asarray(np.ma.getdata(result)))


def alloc_tile(shape, dtype, fill=0) -> Tile:
    """``group.zeros/ones/full``: every element valid
    (python/hckernel/kernel_api.py:347-369, 433-434)."""
    shape = tuple(np.atleast_1d(shape).tolist())
    return Tile(np.full(shape, fill, dtype=dtype), np.ones(shape, dtype=bool))


def store_tile(dst_view: np.ndarray, src) -> None:
    """``group.store(dst_view, src)``: python/hckernel/kernel_api.py:318-342.

    The source is clipped to the destination view.  A :class:`Tile` writes only
    its valid elements (the ``np.where(src.mask, ...)`` branch, :339-340); a
    plain array is assigned as is (:341-342), which is what reaches ``store``
    after ``np.dot`` / ``np.exp`` / a reduction turned the tile into an
    ordinary (masked) NumPy array.
    """
    if isinstance(src, Tile):
        region = tuple(slice(0, min(a, b)) for a, b in zip(src.shape, dst_view.shape))
        dst_view[region] = np.where(src.valid[region], src.data[region], dst_view[region])
    else:
        src = np.asarray(src)
        region = tuple(slice(0, min(a, b)) for a, b in zip(src.shape, dst_view.shape))
        dst_view[region] = src[region]


def _mapped_indices(func, shape, extents):
    """Index arrays ``func(*index)`` for every ``index`` of a tile of ``shape``
    plus the mask of those that fall inside ``extents``; ``func`` is applied to
    whole index grids (the mapping lambdas only use ``+ * // %``, which NumPy
    evaluates element-wise with the same floor semantics as Python ints)."""
    grids = np.indices(shape, dtype=np.int64)
    mapped = func(*grids)
    if len(mapped) != len(extents):
        raise ValueError("mapping returns a different rank than the array has")
    mapped = [np.broadcast_to(np.asarray(m, dtype=np.int64), shape) for m in mapped]
    inside = np.ones(shape, dtype=bool)
    for m, extent in zip(mapped, extents):
        inside &= (m >= 0) & (m < extent)
    return mapped, inside


def load_tile_mapped(view: np.ndarray, shape, func) -> Tile:
    """``group.load(view, shape, mapping=m)``: python/hckernel/kernel_api.py:303-310.

    Element ``index`` of the tile is ``view[func(*index)]`` when every component
    of the mapped index lies inside ``view`` (which already starts at the tile
    origin); otherwise it stays zero and is marked invalid.
    """
    shape = tuple(np.atleast_1d(shape).tolist())
    data = np.zeros(shape, dtype=view.dtype)
    mapped, inside = _mapped_indices(func, shape, view.shape)
    data[inside] = view[tuple(m[inside] for m in mapped)]
    return Tile(data, inside)


def store_tile_mapped(dst_view: np.ndarray, src: Tile, func) -> None:
    """``group.store(dst_view, src, mapping=m)``: python/hckernel/kernel_api.py:319-336.

    Valid element ``index`` of the tile goes to ``dst_view[func(*index)]`` when
    the mapped index lies inside ``dst_view``; everything else is dropped.  The
    reference visits the elements in row-major order, so of two elements mapped
    to one place the later one wins; NumPy's fancy assignment does the same.
    """
    mapped, inside = _mapped_indices(func, src.shape, dst_view.shape)
    keep = inside & src.valid
    dst_view[tuple(m[keep] for m in mapped)] = src.data[keep]


def valid_rows(tile: Tile) -> int:
    """Number of leading rows of a row-block tile that exist in the array.

    For tiles loaded as whole rows (no column padding) the mask is a prefix of
    rows; masked reductions over the last axis (numpy.ma ``max``/``sum`` reached
    through kernel_api.py:150-151) then equal plain reductions over these rows,
    and rows past the end are dropped again when the result is stored.
    """
    if tile.valid.ndim == 1:
        return int(tile.valid.sum())
    rows = tile.valid.all(axis=tuple(range(1, tile.valid.ndim)))
    return int(rows.sum())
