"""Work-item functions that an element-wise pass cannot express::

    tmp = group.zeros(shape=group.shape[0], dtype=a.dtype)

    @group.workitems
    def inner(wi):
        lid, gid = wi.local_id()[0], wi.global_id()[0]
        if gid < a.shape[0]:
            tmp[lid] = a[gid] * 2.0
        group.barrier()
        if gid < a.shape[0]:
            out[gid] = tmp.data[group.shape[0] - 1 - lid] + lid

The reference runs such a function once per work-item, as greenlets that hand
over to one another at ``group.barrier()`` (python/hckernel/kernel_api.py:
395-431); its compiler puts the group's tiles into work-group memory
(mlir/lib/Transforms/LowerScope.cpp:246-309).  Here the function is recorded
once and becomes a program for ``csrc/kernels/work_items.cu``: one thread per
work-item, one CTA per work-group, the group's tile in shared memory, the
barrier the CTA's.  What a work-item may do: read arrays at its own global id
plus a constant offset (a neighbour's element), use its local and global id as
values, write the group's tile at its local id before the barrier and read it at
``scale * lid + offset`` (optionally modulo a constant) after it, and write
output arrays at its own global id - all under conditions that compare its
global id with numbers.

The work-item form of the pairwise distance (docs/langref.md:47-63),
``D[i, j] = np.sqrt(((X1[i] - X2[j]) ** 2).sum())``, is recognised as a whole
and runs on the pairwise-distance kernel.
"""

from .elementwise import (EQ, LOAD, SAVE0, SRC_CONST, SRC_TEMP, TEMPS, MapProgram, _BINARY,
                          _UNARY, check_types, refuse_inexact_indices)
from .kernel_api import Tile, UnsupportedKernel

STORE_TILE, BARRIER, STORE_OUT = 64, 65, 66
SRC_ROW, SRC_COL, SRC_LOCAL_ROW, SRC_LOCAL_COL, SRC_TILE = 16, 17, 18, 19, 24
MAX_INSTR, MAX_TILE_READS = 48, 4


def needs_work_items(recorder):
    """Does the recorded work-item function go beyond one element-wise store?"""
    if len([e for e in recorder.item_events if e[0] == "out"]) != 1:
        return True
    if any(e[0] != "out" for e in recorder.item_events):
        return True
    out = recorder.item_events[0][1]
    for axis, (lo, hi) in recorder.item_ranges[0].items():
        if axis < out.ndim and (lo > 0 or hi < out.shape[axis]):
            return True  # a condition that excludes work-items inside the array

    def special(node, seen):
        if not isinstance(node, Tile) or id(node) in seen:
            return False
        seen.add(id(node))
        if node.op == "tile_read" or node.attrs.get("kind") == "local" or node.attrs.get("offsets"):
            return True
        if node.op == "item_load" and node.shape:
            return True  # a row of a matrix, not an element
        return any(special(a, seen) for a in node.args)

    return special(recorder.item_events[0][3], set())


def match_item_pairwise(recorder):
    """Buffers ``(a, b, out)`` when the function is the work-item form of the
    pairwise distance: ``out[i, j] = sqrt(sum((a[i] - b[j]) ** 2))``."""
    events = recorder.item_events
    if len(events) != 1 or events[0][0] != "out":
        return None
    _, out, axes, expr = events[0]
    if axes != (0, 1) or out.ndim != 2 or expr.op != "sqrt":
        return None
    total = expr.args[0]
    if total.op != "sum" or total.attrs.get("axis") is not None:
        return None
    square = total.args[0]
    if square.op != "mul" or square.args[0].key() != square.args[1].key():
        return None
    diff = square.args[0]
    if diff.op != "sub":
        return None
    left, right = diff.args
    for t, axis in ((left, 0), (right, 1)):
        if not (isinstance(t, Tile) and t.op == "item_load" and t.attrs["axes"] == (axis,)
                and not t.attrs.get("offsets") and t.args[0].ndim == 2):
            return None
    a, b = left.args[0], right.args[0]
    if a.shape[1] != b.shape[1] or out.shape != (a.shape[0], b.shape[0]):
        raise UnsupportedKernel("work-item pairwise distance: shapes do not form [M,D], [N,D] -> "
                                "[M,N]")
    if not a.dtype == b.dtype == out.dtype or out.dtype not in ("float32", "float64"):
        raise UnsupportedKernel("work-item pairwise distance: one float type for all arrays")
    ranges = recorder.item_ranges[0]
    for axis, extent in ((0, out.shape[0]), (1, out.shape[1])):
        lo, hi = ranges.get(axis, (0, extent))
        if lo > 0 or hi < extent:
            raise UnsupportedKernel("work-item pairwise distance: conditions that exclude part of "
                                    "the output are not supported")
    return a, b, out


class ItemProgram(MapProgram):
    """The accumulator-machine program of a work-item function: scalar values,
    operands that include neighbour reads, local ids and the group's tile."""

    def __init__(self, rank):
        super().__init__(())
        self.rank = rank
        self.slots = []       # (buffer, (row offset, column offset))
        self.tile_reads = []  # (row scale, row offset, row wrap, col scale, col offset, col wrap)
        self.tile = None      # the one group tile
        self.phase_of_slot = {}
        self.phase = 0

    def _emit(self, op, src=0):
        if len(self.code) == MAX_INSTR:
            raise UnsupportedKernel(f"work-item kernel: more than {MAX_INSTR} operations")
        self.code.append(op | (src << 8))

    def _axes2(self, per_axis, fill):
        """Values per work axis laid out as (row, column): one-dimensional work
        runs along the columns."""
        if self.rank == 1:
            return (fill, per_axis[0])
        return (per_axis[0], per_axis[1])

    def _leaf(self, node):
        if node.op == "item_load":
            buffer = node.args[0]
            if node.shape or node.attrs["axes"] != tuple(range(buffer.ndim)):
                raise UnsupportedKernel(
                    f"work-item kernel: {buffer.name} must be read with one index per dimension, "
                    f"the work-item's global id plus a constant, in order")
            offsets = node.attrs.get("offsets", (0,) * buffer.ndim)
            key = (buffer, self._axes2(offsets, 0))
            if key not in self.slots:
                if len(self.slots) == 4:
                    raise UnsupportedKernel("work-item kernel: more than 4 different array reads")
                self.slots.append(key)
            return self.slots.index(key)
        if node.op == "index":
            self.uses_index = True
            local = node.attrs.get("kind") == "local"
            row, col = (SRC_LOCAL_ROW, SRC_LOCAL_COL) if local else (SRC_ROW, SRC_COL)
            if self.rank == 1:  # one-dimensional work runs along the columns
                return col
            return (row, col)[node.attrs["axis"]]
        if node.op == "tile_read":
            tile = node.args[0]
            if self.tile is None:
                self.tile = tile
            if tile is not self.tile:
                raise UnsupportedKernel("work-item kernel: one group tile at most")
            if self.phase == 0:
                raise UnsupportedKernel(
                    "work-item kernel: the group tile is read after group.barrier() only (before "
                    "it, other work-items may not have written their element yet)")
            per_axis = {axis: (scale, offset, wrap) for axis, scale, offset, wrap in
                        node.attrs["index"]}
            if sorted(per_axis) != list(range(self.rank)):
                raise UnsupportedKernel("work-item kernel: the group tile is indexed by the local "
                                        "id of each axis, in order")
            entry = sum(self._axes2([per_axis[d] for d in range(self.rank)], (0, 0, 0)), ())
            if entry not in self.tile_reads:
                if len(self.tile_reads) == MAX_TILE_READS:
                    raise UnsupportedKernel(
                        f"work-item kernel: more than {MAX_TILE_READS} different tile reads")
                self.tile_reads.append(entry)
            return SRC_TILE + self.tile_reads.index(entry)
        if node.op == "load":
            raise UnsupportedKernel("work-item kernel: tile loads inside a work-item function")
        return super()._leaf(node)


def match_work_items(recorder, work, group):
    """The launch description of a recorded work-item function:
    ``(program, output buffer, group shape as (rows, columns))``."""
    what = "work-item kernel"
    rank = len(work)
    if rank not in (1, 2):
        raise UnsupportedKernel(f"{what}: one- or two-dimensional work shapes")
    outs = [e for e in recorder.item_events if e[0] == "out"]
    if not outs:
        raise UnsupportedKernel(f"{what}: the function stores nothing")
    out = outs[0][1]
    if any(e[1] is not out for e in outs):
        raise UnsupportedKernel(f"{what}: one output array")
    if out.ndim != rank or tuple(out.shape) != tuple(work):
        raise UnsupportedKernel(
            f"{what}: the work shape {list(work)} must be the shape of {out.name} "
            f"{list(out.shape)}")
    if out.dtype not in ("float32", "float64"):
        raise UnsupportedKernel(f"{what}: float32 or float64 arrays, not {out.dtype}")
    program = ItemProgram(rank)
    for event in recorder.item_events:
        if event[0] == "barrier":
            program._emit(BARRIER)
            program.phase = 1
            program._free = list(range(TEMPS))
            continue
        value = event[3]
        check_types(value, out.dtype, what)
        if event[0] == "tile":
            tile = event[1]
            if program.tile is None:
                program.tile = tile
            if tile is not program.tile:
                raise UnsupportedKernel(f"{what}: one group tile at most")
            if tuple(tile.shape) != tuple(group) or tile.dtype != out.dtype:
                raise UnsupportedKernel(
                    f"{what}: the group tile must have the group's shape {list(group)} and the "
                    f"arrays' element type")
            if program.phase != 0:
                raise UnsupportedKernel(f"{what}: the group tile is written before the barrier")
            program.evaluate(value)
            program._emit(STORE_TILE)
        else:
            if event[2] != tuple(range(rank)):
                raise UnsupportedKernel(
                    f"{what}: {out.name} must be written at the work-item's own global id")
            program.evaluate(value)
            program._emit(STORE_OUT)
    for buffer, _ in program.slots:
        if tuple(buffer.shape) != tuple(out.shape) or buffer.dtype != out.dtype:
            raise UnsupportedKernel(
                f"{what}: {buffer.name} and {out.name} differ in shape or element type")
    # Per phase the range of global ids that take part, as (lo row, hi row, lo col, hi col).
    guards = []
    phases = recorder.item_ranges + [recorder.item_ranges[-1]] * (2 - len(recorder.item_ranges))
    for ranges in phases[:2]:
        per_axis = [ranges.get(d, (0, out.shape[d])) for d in range(rank)]
        per_axis = [(max(lo, 0), min(hi, out.shape[d])) for d, (lo, hi) in enumerate(per_axis)]
        (lo_r, hi_r), (lo_c, hi_c) = program._axes2(per_axis, (0, 1))
        guards.append((lo_r, hi_r, lo_c, hi_c))
    group2 = program._axes2(tuple(group), 1)
    if group2[0] * group2[1] > 1024:
        raise UnsupportedKernel(f"{what}: work-groups of at most 1024 work-items")
    fill = float(program.tile.args[0]) if program.tile is not None else 0.0
    refuse_inexact_indices(program, out, what)
    return program, out, group2, guards, fill
