"""Element-wise kernel bodies: tiles loaded at one origin, combined element by
element, stored at the same origin::

    x, y = gr.work_offset
    a_t = gr.load(a[x:, y:], shape=gr.shape)
    b_t = gr.load(b[x:, y:], shape=gr.shape)
    gr.store(out[x:, y:], np.maximum(a_t * 2.0 - b_t, 0.0))

The reference compiles such a body to GPU code (its copy kernels are the
degenerate case, python/hckernel/tests/test_e2e.py:57-136; tile arithmetic is
python/hckernel/kernel_api.py:136-211).  There is no compiler here, so the
recorded expression is translated into a short program for the one-accumulator
machine that ``csrc/kernels/map_elements.cu`` interprets - three temporaries,
up to four input arrays, eight constants, 32 instructions - and one launch on
the whole arrays computes what all work-groups would.

Translation: the right operand of a binary operation is taken straight from an
input, a constant or a temporary whenever it is a leaf; when only the left one
is a leaf the operation is emitted in its reversed form (``v - acc``,
``v / acc``); when neither is, the right subtree is evaluated first and parked
in a temporary.  An expression that needs more than three temporaries at once
or more than 32 instructions is refused.
"""

from .kernel_api import Tile, UnsupportedKernel

LOAD, ADD, SUB, RSUB, MUL, DIV, RDIV, MAX, MIN, NEG, ABS, EXP, SQRT, SAVE0 = range(14)
LOG, RSUM, RMAX, SET = 16, 17, 18, 19
# The rest of the reference's tile operator table (element-wise bodies only).
(FLOORDIV, RFLOORDIV, MOD, RMOD, POW, RPOW, LT, LE, EQ, NE, GE, GT, AND, OR, XOR, SHL, SHR, RSHL,
 RSHR, INV) = range(20, 40)
UNIFORM = 0x80  # flag in the operation byte: one value per row, computed before the walk
SRC_TEMP, SRC_CONST, SRC_SCALAR = 4, 8, 20
MAX_INPUTS, MAX_CONSTS, MAX_INSTR, TEMPS, MAX_SCALARS = 4, 8, 32, 3, 4

# operation -> (acc OP v, v OP acc)
_BINARY = {"add": (ADD, ADD), "sub": (SUB, RSUB), "mul": (MUL, MUL), "div": (DIV, RDIV),
           "maximum": (MAX, MAX), "minimum": (MIN, MIN),
           "floordiv": (FLOORDIV, RFLOORDIV), "mod": (MOD, RMOD), "pow": (POW, RPOW),
           "lt": (LT, GT), "le": (LE, GE), "eq": (EQ, EQ), "ne": (NE, NE), "ge": (GE, LE),
           "gt": (GT, LT), "and": (AND, AND), "or": (OR, OR), "xor": (XOR, XOR),
           "lshift": (SHL, RSHL), "rshift": (SHR, RSHR)}
_UNARY = {"neg": NEG, "abs": ABS, "exp": EXP, "sqrt": SQRT, "log": LOG, "invert": INV}
_FLOAT_ONLY = ("div", "exp", "sqrt", "log")
_INTEGER_ONLY = ("lshift", "rshift")
_LOGICAL = ("and", "or", "xor", "invert")


def check_types(expr, dtype, what):
    """Refuses what the element type of the arrays has no operation for, with
    NumPy's reasons: integers have no true division (its result is a float
    array), exp, sqrt or log here, floats no shifts and no bitwise operators
    except on truth values (the results of comparisons)."""
    integer = dtype.startswith("int")
    seen = set()

    def walk(node):
        if not isinstance(node, Tile) or id(node) in seen:
            return
        seen.add(id(node))
        for arg in node.args:
            walk(arg)
        if integer and node.op in _FLOAT_ONLY:
            raise UnsupportedKernel(
                f"{what}: '{node.op}' on {dtype} tiles gives floating-point values; compute in a "
                f"float array")
        if integer and node.op == "const" and float(node.args[0]) != int(node.args[0]):
            raise UnsupportedKernel(
                f"{what}: the constant {node.args[0]!r} turns {dtype} tiles into floating-point "
                f"values; compute in a float array")
        if integer and node.op == "pow":
            exponent = node.args[1]
            if not (isinstance(exponent, Tile) and exponent.op == "const"):
                raise UnsupportedKernel(f"{what}: {dtype} tiles take constant exponents only")
            if float(exponent.args[0]) < 0:
                raise ValueError("Integers to negative integer powers are not allowed.")
        if not integer and node.op in _INTEGER_ONLY:
            raise TypeError(f"{what}: shifts are not supported for {dtype} tiles")
        if not integer and node.op in _LOGICAL:
            operands = [a for a in node.args if isinstance(a, Tile) and a.op != "const"]
            if any(a.dtype != "bool" for a in operands):
                raise TypeError(
                    f"{what}: '{node.op}' is not supported for {dtype} tiles (only for truth "
                    f"values, the results of comparisons)")

    walk(expr)
_ROW_REDUCTIONS = {"sum": RSUM, "max": RMAX}


class MapProgram:
    """The translated expression: which loads feed it (``inputs``, Tile nodes),
    the instructions and the constants."""

    def __init__(self, shape, index_sources=None):
        self.shape = tuple(shape)
        self.inputs, self.code, self.consts = [], [], []
        self._free = list(range(TEMPS))
        self.index_sources = index_sources  # work axis -> operand name (work-item level only)
        self.uses_index = False  # a work-item index is an operand of the expression
        self.scalars = []  # row programs: the reductions already computed, in scalar order
        # Row programs: expressions of row scalars and constants only are computed
        # once per row, in a uniform prologue of the pass that first needs them,
        # and kept in a row scalar of their own.
        self.row_mode = False
        self.reserved_scalars = 0   # scalars 0..n-1 belong to the reductions
        self.hoisted = []           # uniform nodes that got a scalar, in order
        self._prologue = []         # uniform instructions of the pass being written
        self._pass_start = 0

    # -- row programs: passes and uniform prologues ---------------------------------------
    def begin_pass(self):
        self._pass_start, self._prologue = len(self.code), []
        self._free = list(range(TEMPS))  # temporaries do not outlive a pass

    def end_pass(self):
        if len(self.code) + len(self._prologue) > MAX_INSTR:
            raise UnsupportedKernel(f"element-wise kernel: more than {MAX_INSTR} operations")
        self.code[self._pass_start:self._pass_start] = self._prologue
        self._prologue = []

    def _scalar_of(self, node):
        for i, seen in enumerate(self.scalars):
            if seen.key() == node.key():
                return SRC_SCALAR + i
        for i, seen in enumerate(self.hoisted):
            if seen.key() == node.key():
                return SRC_SCALAR + self.reserved_scalars + i
        return None

    def _is_uniform(self, node):
        if not isinstance(node, Tile):
            return False
        if node.op in ("const", "alloc") or self._scalar_of(node) is not None:
            return True
        if node.op in _UNARY or node.op in _BINARY:
            return all(self._is_uniform(a) for a in node.args)
        return False

    def _uniform_chain(self, node):
        """Instructions that compute a uniform expression in the one-value
        accumulator of the prologue (which has no temporaries), or None."""
        src = self._scalar_of(node)
        if src is None and node.op in ("const", "alloc"):
            src = self._leaf(node)
        if src is not None:
            return [LOAD | (src << 8)]
        if node.op in _UNARY:
            inner = self._uniform_chain(node.args[0])
            return None if inner is None else inner + [_UNARY[node.op]]
        forward, reverse = _BINARY[node.op]
        left, right = node.args
        for operand, other, op in ((right, left, forward), (left, right, reverse)):
            src = self._scalar_of(operand)
            if src is None and operand.op in ("const", "alloc"):
                src = self._leaf(operand)
            if src is not None:
                inner = self._uniform_chain(other)
                return None if inner is None else inner + [op | (src << 8)]
        return None

    def _hoist(self, node):
        """Row scalar that holds the uniform expression ``node``, computing it in
        the prologue of the current pass on first use; None if it cannot be."""
        known = self._scalar_of(node)
        if known is not None:
            return known
        index = self.reserved_scalars + len(self.hoisted)
        if index >= MAX_SCALARS:
            return None
        chain = self._uniform_chain(node)
        if chain is None:
            return None
        self._prologue += [ins | UNIFORM for ins in chain] + [SET | UNIFORM | (index << 8)]
        self.hoisted.append(node)
        return SRC_SCALAR + index

    def _leaf(self, node):
        """Operand name of a leaf, or None for an inner node."""
        if self.row_mode and (node.op in _UNARY or node.op in _BINARY) and self._is_uniform(node):
            hoisted = self._hoist(node)
            if hoisted is not None:
                return hoisted
        if node.op in _ROW_REDUCTIONS:  # a value an earlier pass of a row program reduced
            for i, seen in enumerate(self.scalars):
                if seen.key() == node.key():
                    return SRC_SCALAR + i
            raise UnsupportedKernel(
                f"element-wise kernel: operation '{node.op}' has no element-wise form")
        if node.op == "load":
            if node.shape != self.shape:
                raise UnsupportedKernel(
                    f"element-wise kernel: a tile of shape {node.shape} in an expression of shape "
                    f"{self.shape} (broadcasting between tiles is not supported)")
            for i, seen in enumerate(self.inputs):
                if seen.key() == node.key():
                    return i
            if len(self.inputs) == MAX_INPUTS:
                raise UnsupportedKernel(f"element-wise kernel: more than {MAX_INPUTS} input tiles")
            self.inputs.append(node)
            return len(self.inputs) - 1
        if node.op == "item_load":  # `buf[gid]` at work-item level
            for i, seen in enumerate(self.inputs):
                if seen.op == "item_load" and seen.args[0] is node.args[0] \
                        and seen.attrs["axes"] == node.attrs["axes"]:
                    return i
            if len(self.inputs) == MAX_INPUTS:
                raise UnsupportedKernel(f"element-wise kernel: more than {MAX_INPUTS} input arrays")
            self.inputs.append(node)
            return len(self.inputs) - 1
        if node.op == "index":  # the work-item's own index as a value
            if self.index_sources is None:
                raise UnsupportedKernel("a work-item index outside a work-item function")
            self.uses_index = True
            return self.index_sources[node.attrs["axis"]]
        if node.op in ("const", "alloc"):
            value = float(node.args[0])
            for i, seen in enumerate(self.consts):
                # Bit-for-bit the same constant (so that 0.0 and -0.0 stay apart).
                if seen == value and str(seen) == str(value):
                    return SRC_CONST + i
            if len(self.consts) == MAX_CONSTS:
                raise UnsupportedKernel(f"element-wise kernel: more than {MAX_CONSTS} constants")
            self.consts.append(value)
            return SRC_CONST + len(self.consts) - 1
        return None

    def _emit(self, op, src=0):
        if len(self.code) == MAX_INSTR:
            raise UnsupportedKernel(f"element-wise kernel: more than {MAX_INSTR} operations")
        self.code.append(op | (src << 8))

    def evaluate(self, node):
        """Append the instructions that leave the value of ``node`` in the accumulator."""
        if not isinstance(node, Tile):
            raise UnsupportedKernel(f"element-wise kernel: operand {node!r}")
        src = self._leaf(node)
        if src is not None:
            self._emit(LOAD, src)
        elif node.op == "invert" and node.args[0].dtype == "bool":
            # NumPy's ~ on truth values is "not": 1 where the value is 0 (the
            # machine's own `inv` is the bitwise one on integer arrays).
            self.evaluate(node.args[0])
            self._emit(EQ, self._leaf(Tile("const", (0.0,), (), "scalar")))
        elif node.op in _UNARY:
            self.evaluate(node.args[0])
            self._emit(_UNARY[node.op])
        elif node.op == "astype" and node.dtype == node.args[0].dtype:
            self.evaluate(node.args[0])
        elif node.op in _BINARY:
            forward, reverse = _BINARY[node.op]
            left, right = node.args
            right_src = self._leaf(right)
            if right_src is not None:
                self.evaluate(left)
                self._emit(forward, right_src)
                return
            left_src = self._leaf(left)
            if left_src is not None:
                self.evaluate(right)
                self._emit(reverse, left_src)
                return
            self.evaluate(right)
            if not self._free:
                raise UnsupportedKernel("element-wise kernel: the expression needs more than "
                                        f"{TEMPS} intermediate values at once")
            temp = self._free.pop(0)
            self._emit(SAVE0 + temp)
            self.evaluate(left)
            self._emit(forward, SRC_TEMP + temp)
            self._free.insert(0, temp)
        else:
            raise UnsupportedKernel(
                f"element-wise kernel: operation '{node.op}' has no element-wise form")


def match_map(stores, counts, covers):
    """``(program, destination view)`` when the single store of a body is an
    element-wise expression of tiles loaded where it is stored, else None.
    ``covers`` is the coverage check shared with the other families."""
    if len(stores) != 1:
        return None
    dst, expr = stores[0]
    if expr.op not in _BINARY and expr.op not in _UNARY and expr.op not in ("alloc", "astype"):
        return None
    if dst.buffer.ndim not in (1, 2) or len(expr.shape) != dst.buffer.ndim:
        raise UnsupportedKernel("element-wise kernels are supported for vectors and matrices")
    if dst.buffer.dtype not in ("float32", "float64", "int32", "int64"):
        raise UnsupportedKernel(
            f"element-wise kernels compute in float32, float64, int32 or int64, not "
            f"{dst.buffer.dtype}")
    check_types(expr, dst.buffer.dtype, "element-wise kernel")
    program = MapProgram(expr.shape)
    program.evaluate(expr)
    for tile in program.inputs:
        if tile.op != "load":
            raise UnsupportedKernel("element-wise kernel: work-item reads inside a tile expression")
        view = tile.args[0]
        if view.buffer.shape != dst.buffer.shape or view.buffer.dtype != dst.buffer.dtype:
            raise UnsupportedKernel(
                f"element-wise kernel: {view.buffer.name} and {dst.buffer.name} differ in shape or "
                f"element type")
        if tuple(view.origin) != tuple(dst.origin):
            raise UnsupportedKernel(
                f"element-wise kernel: {view.buffer.name} is loaded at another origin than "
                f"{dst.buffer.name} is stored")
    covers(dst.origin, expr.shape, dst.buffer.shape, counts, "element-wise kernel")
    return program, dst


def refuse_inexact_indices(program, dst, what):
    """The machine computes in the arrays' element type, indices included, with
    a rounding per operation; the reference computes index arithmetic in Python
    integers and rounds once, on the store.  float32 holds every integer up to
    2**24 exactly, so as long as the array has no more elements than that, an
    expression such as ``gid[0] * shape[1] + gid[1]`` gives the same float32
    either way; beyond it the two can differ by an ulp, so the kernel is refused."""
    elements = 1
    for extent in dst.shape:
        elements *= int(extent)
    if program.uses_index and dst.dtype == "float32" and elements > 1 << 24:
        raise UnsupportedKernel(
            f"{what}: {dst.name} has {elements} float32 elements and the body computes with the "
            f"work-item's index; index arithmetic is exact in float32 only up to 2**24 elements - "
            f"use a float64 array")


def match_rows(stores, counts, covers):
    """``(program, destination view)`` when the single store of a body is an
    expression of whole-row tiles that reduces along the rows (``sum`` / ``max``
    / ``mean`` with ``axis=1, keepdims=True``) and uses the reduced values
    again - the reference's softmax body (python/hckernel/tests/
    test_examples.py:312-321) and its relatives; None when nothing is reduced.

    The program is cut into passes: one per distinct reduction, in dependency
    order (the argument of a reduction may use earlier reductions), each ending
    in the instruction that reduces the accumulator into a row scalar; a last
    pass computes the stored value with the scalars as operands."""
    if len(stores) != 1:
        return None
    dst, expr = stores[0]
    reductions = []

    def collect(node):  # post-order: what a reduction depends on comes first
        for arg in node.args:
            if isinstance(arg, Tile):
                collect(arg)
        if node.op in _ROW_REDUCTIONS and not any(r.key() == node.key() for r in reductions):
            reductions.append(node)

    collect(expr)
    if not reductions or expr.op in _ROW_REDUCTIONS:
        return None
    what = "row kernel"
    if dst.buffer.ndim != 2 or len(expr.shape) != 2:
        raise UnsupportedKernel(f"{what}: matrices expected")
    if dst.buffer.dtype not in ("float32", "float64"):
        raise UnsupportedKernel(f"{what}: float32 or float64, not {dst.buffer.dtype}")
    if len(reductions) > MAX_SCALARS:
        raise UnsupportedKernel(f"{what}: more than {MAX_SCALARS} different row reductions")
    if expr.shape[1] != dst.buffer.shape[1]:
        raise UnsupportedKernel(f"{what}: tiles must hold whole rows")
    program = MapProgram(expr.shape)
    program.row_mode, program.reserved_scalars = True, len(reductions)
    for i, node in enumerate(reductions):
        if node.attrs != {"axis": 1, "keepdims": True} or node.args[0].shape != expr.shape:
            raise UnsupportedKernel(
                f"{what}: reductions must be over whole rows with axis=1, keepdims=True")
        program.begin_pass()
        program.evaluate(node.args[0])
        program._emit(_ROW_REDUCTIONS[node.op], i)
        program.end_pass()
        program.scalars.append(node)
    program.begin_pass()
    program.evaluate(expr)
    program.end_pass()
    if any((ins & 0x7F) >= FLOORDIV for ins in program.code):
        raise UnsupportedKernel(
            f"{what}: // % ** comparisons and bitwise operators are supported in element-wise "
            f"bodies only, not together with row reductions")
    if len(program.inputs) > 2 or not program.inputs:
        raise UnsupportedKernel(f"{what}: one or two input matrices")
    for tile in program.inputs:
        if tile.op != "load":
            raise UnsupportedKernel(f"{what}: work-item reads inside a tile expression")
        view = tile.args[0]
        if view.buffer.shape != dst.buffer.shape or view.buffer.dtype != dst.buffer.dtype:
            raise UnsupportedKernel(
                f"{what}: {view.buffer.name} and {dst.buffer.name} differ in shape or element type")
        if tuple(view.origin) != tuple(dst.origin):
            raise UnsupportedKernel(
                f"{what}: {view.buffer.name} is loaded at another origin than {dst.buffer.name} "
                f"is stored")
    covers(dst.origin, expr.shape, dst.buffer.shape, counts, what)
    return program, dst


SRC_ROW, SRC_COL = 16, 17


def match_items(item_stores, guards, work_shape):
    """``(program, destination buffer)`` for a body written at work-item level
    (``@group.workitems``; reference python/hckernel/kernel_api.py:395-414, its
    tests python/hckernel/tests/test_kernel_sim.py:381-412)::

        gid = wi.global_id()[:2]
        if gid[0] < arr.shape[0] and gid[1] < arr.shape[1]:
            arr[gid] = gid[0] * arr.shape[1] + gid[1]

    Every work-item writes the element of one array that its own global id
    names, computed from its index and from the same element of other arrays -
    an element-wise program whose operands include the row and column index.
    The launch covers whole arrays, so the conditions taken must be implied by
    the array bounds and the work shape must reach every element."""
    what = "work-item kernel"
    if len(item_stores) != 1:
        raise UnsupportedKernel(f"{what}: exactly one element store per work-item is supported")
    dst, axes, expr = item_stores[0]
    rank = dst.ndim
    if rank not in (1, 2) or axes != tuple(range(rank)):
        raise UnsupportedKernel(
            f"{what}: the store must be {dst.name}[global_id] with one index per dimension, in "
            f"order, of a vector or matrix")
    if dst.dtype not in ("float32", "float64", "int32", "int64"):
        raise UnsupportedKernel(
            f"{what}: float32, float64, int32 or int64 arrays, not {dst.dtype}")
    check_types(expr, dst.dtype, what)
    for axis, bound in guards:
        if axis >= rank or bound < dst.shape[axis]:
            raise UnsupportedKernel(
                f"{what}: the condition index{axis} < {bound} is not implied by the shape "
                f"{list(dst.shape)} of {dst.name}; only bounds guards can be honoured")
    for d in range(rank):
        if work_shape[d] < dst.shape[d]:
            raise UnsupportedKernel(
                f"{what}: the work shape stops at {work_shape[d]} of {dst.shape[d]} in dimension {d}")
    # Rows and columns of the kernel: a vector is one row.
    sources = {0: SRC_COL} if rank == 1 else {0: SRC_ROW, 1: SRC_COL}
    program = MapProgram((), sources)
    program.evaluate(expr)
    for tile in program.inputs:
        src = tile.args[0]
        if tile.op != "item_load":
            raise UnsupportedKernel(f"{what}: tile loads cannot be mixed into a work-item function")
        if tile.attrs["axes"] != axes or src.shape != dst.shape or src.dtype != dst.dtype:
            raise UnsupportedKernel(
                f"{what}: {src.name} must be read at the work-item's own index and match "
                f"{dst.name} in shape and element type")
    refuse_inexact_indices(program, dst, what)
    return program, dst
