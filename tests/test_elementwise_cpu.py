"""Element-wise bodies on CPU: the oracle against the reference simulator's
outputs (bit for bit), and the front door - the recorded expression must be
translated into a program for the accumulator machine of
csrc/kernels/map_elements.cu that, run here in NumPy, gives exactly what NumPy
gives for the same expression.  No kernel is launched."""

import numpy as np
import pytest

from hc_b200.hckernel import elementwise as ew
from hc_b200.hckernel.kernel import *  # noqa: F401,F403
from hc_b200.hckernel.kernel import UnsupportedKernel
from hc_b200.workloads import make_elementwise
from oracle import workloads as oracle

CASES = oracle.elementwise_cases()


class FakeTensor:
    def __init__(self, shape, dtype="float32"):
        self.shape, self.dtype = tuple(shape), dtype


F = FakeTensor


def _divides(a, b):
    """Where numpy.ma does not mask a / b, a // b, a % b (its _DomainSafeDivide)."""
    a, b = np.broadcast_arrays(np.asarray(a), np.asarray(b))
    if a.dtype.kind == "f":
        return ~(np.abs(a.astype(np.float64)) * np.finfo(np.float64).tiny
                 >= np.abs(b.astype(np.float64)))
    return b != 0


def run_program(code, consts, inputs, dtype, shape=None, valid_out=None):
    """The machine of map_elements.cu, one NumPy operation per instruction.
    ``valid_out`` (a list) receives the validity of the result's elements: what
    the kernel stores and what it leaves untouched."""
    dtype = np.dtype(dtype).type
    shape = inputs[0].shape if shape is None else shape
    acc, temps, scalars, one = None, [None, None, None], [None] * 4, None
    ok, temps_ok = np.ones(shape, bool), [None, None, None]
    truth = lambda cond: cond.astype(dtype)  # noqa: E731
    if np.dtype(dtype).kind == "f":
        bits = {ew.AND: lambda a, b: truth((a != 0) & (b != 0)),
                ew.OR: lambda a, b: truth((a != 0) | (b != 0)),
                ew.XOR: lambda a, b: truth((a != 0) ^ (b != 0))}
    else:
        bits = {ew.AND: np.bitwise_and, ew.OR: np.bitwise_or, ew.XOR: np.bitwise_xor}
    extended = {
        ew.FLOORDIV: lambda a, b: (np.floor_divide(a, b), _divides(a, b)),
        ew.RFLOORDIV: lambda a, b: (np.floor_divide(b, a), _divides(b, a)),
        ew.MOD: lambda a, b: (np.remainder(a, b), _divides(a, b)),
        ew.RMOD: lambda a, b: (np.remainder(b, a), _divides(b, a)),
        ew.POW: lambda a, b: (np.power(a, b), None),
        ew.RPOW: lambda a, b: (np.power(b, a), None),
        ew.LT: lambda a, b: (truth(a < b), True), ew.LE: lambda a, b: (truth(a <= b), True),
        ew.EQ: lambda a, b: (truth(a == b), True), ew.NE: lambda a, b: (truth(a != b), True),
        ew.GE: lambda a, b: (truth(a >= b), True), ew.GT: lambda a, b: (truth(a > b), True),
        ew.AND: lambda a, b: (bits[ew.AND](a, b), True),
        ew.OR: lambda a, b: (bits[ew.OR](a, b), True),
        ew.XOR: lambda a, b: (bits[ew.XOR](a, b), True),
        ew.SHL: lambda a, b: (np.left_shift(a, b), True),
        ew.SHR: lambda a, b: (np.right_shift(a, b), True),
        ew.RSHL: lambda a, b: (np.left_shift(b, a), True),
        ew.RSHR: lambda a, b: (np.right_shift(b, a), True),
    }
    with np.errstate(all="ignore"):
        for ins in code:
            op, src = ins & 0xFF, ins >> 8
            if op & ew.UNIFORM:  # row programs: one value per row, before the pass walks it
                op &= 0x7F
                if op <= ew.MIN:
                    b = scalars[src - ew.SRC_SCALAR] if src >= ew.SRC_SCALAR \
                        else dtype(consts[src - ew.SRC_CONST])
                if op == ew.SET:
                    scalars[src] = np.broadcast_to(one, (shape[0], 1)).astype(dtype)
                else:
                    one = {ew.LOAD: lambda: b, ew.ADD: lambda: one + b, ew.SUB: lambda: one - b,
                           ew.RSUB: lambda: b - one, ew.MUL: lambda: one * b,
                           ew.DIV: lambda: one / b, ew.RDIV: lambda: b / one,
                           ew.MAX: lambda: np.maximum(one, b), ew.MIN: lambda: np.minimum(one, b),
                           ew.NEG: lambda: -one, ew.ABS: lambda: np.abs(one),
                           ew.EXP: lambda: np.exp(one), ew.SQRT: lambda: np.sqrt(one),
                           ew.LOG: lambda: np.log(one)}[op]()
                continue
            if op in (ew.RSUM, ew.RMAX):  # row programs: reduce along the rows, end the pass
                reduce = np.sum if op == ew.RSUM else np.max
                scalars[src] = reduce(acc, axis=1, keepdims=True).astype(dtype)
                acc, temps = None, [None, None, None]
                continue
            v_ok = True
            if op <= ew.MIN or ew.FLOORDIV <= op <= ew.RSHR:
                if 4 <= src < 8:
                    v_ok = temps_ok[src - 4]
                if src >= ew.SRC_SCALAR:
                    v = np.broadcast_to(scalars[src - ew.SRC_SCALAR], shape)
                elif src >= ew.SRC_ROW:  # the element's own row / column index
                    rows, cols = np.indices(np.atleast_2d(np.empty(shape)).shape)
                    v = (rows if src == ew.SRC_ROW else cols).reshape(shape).astype(dtype)
                else:
                    v = (inputs[src] if src < 4 else temps[src - 4] if src < 8
                         else dtype(consts[src - 8]))
            if op == ew.LOAD:
                acc = v if isinstance(v, np.ndarray) else np.full(shape, v, dtype)
                ok = np.ones(shape, bool) & v_ok
            elif op in extended:
                ok = ok & v_ok
                acc, fine = extended[op](acc, v)
                acc = acc.astype(dtype)
                ok = ok & (np.isfinite(acc) if fine is None else fine)
            elif op == ew.INV:
                acc = truth(acc == 0) if np.dtype(dtype).kind == "f" else ~acc
            elif op == ew.ADD: acc, ok = acc + v, ok & v_ok
            elif op == ew.SUB: acc, ok = acc - v, ok & v_ok
            elif op == ew.RSUB: acc, ok = v - acc, ok & v_ok
            elif op == ew.MUL: acc, ok = acc * v, ok & v_ok
            elif op == ew.DIV: acc, ok = (acc / v).astype(dtype), ok & v_ok & _divides(acc, v)
            elif op == ew.RDIV: acc, ok = (v / acc).astype(dtype), ok & v_ok & _divides(v, acc)
            elif op == ew.MAX: acc, ok = np.maximum(acc, v), ok & v_ok
            elif op == ew.MIN: acc, ok = np.minimum(acc, v), ok & v_ok
            elif op == ew.NEG: acc = -acc
            elif op == ew.ABS: acc = np.abs(acc)
            elif op == ew.EXP: acc = np.exp(acc)
            elif op == ew.SQRT: acc = np.sqrt(acc)
            elif op == ew.LOG: acc = np.log(acc)
            else:
                temps[op - ew.SAVE0], temps_ok[op - ew.SAVE0] = acc, ok
            assert acc.dtype == dtype
    if valid_out is not None:
        valid_out.append(ok)
    return acc


@pytest.mark.parametrize("case", CASES, ids=lambda c: c[0])
def test_oracle_matches_the_reference_simulator(golden, case):
    name, fn, count, shape, dtype, group = case
    inputs = oracle.make_elementwise_inputs(count, shape, dtype)
    out = np.zeros(shape, dtype)
    oracle.elementwise(fn, inputs, out, group)
    assert np.array_equal(out, golden[name])


@pytest.mark.parametrize("case", CASES, ids=lambda c: c[0])
def test_recorded_expression_becomes_an_equivalent_program(golden, case):
    name, fn, count, shape, dtype, group = case
    k = make_elementwise(fn, count, len(shape), group)
    plan = k.plan_for(tuple(F(shape, dtype) for _ in range(count + 1)))
    assert plan.family == "map_elements"
    # Program input k is call argument inputs[k] (numbered in order of first use).
    assert sorted(plan.roles["inputs"]) == list(range(count)) and plan.roles["out"] == count
    inputs = oracle.make_elementwise_inputs(count, shape, dtype)
    got = run_program(plan.roles["code"], plan.roles["consts"],
                      [inputs[i] for i in plan.roles["inputs"]], dtype)
    with np.errstate(all="ignore"):
        assert np.array_equal(got, fn(*inputs))  # the same IEEE operations, one by one
    # ... and the reference's result up to its float64 detours (see oracle.elementwise).
    np.testing.assert_allclose(got, golden[name], rtol=3e-7 if dtype == "float32" else 0)


def test_random_expressions_translate_exactly():
    """200 random expression trees: the program, run one NumPy operation per
    instruction, must give bit for bit what NumPy gives for the expression
    (float64, where NumPy's scalar promotion rules cannot interfere)."""
    rng = np.random.default_rng(2024)
    translated = 0
    for _ in range(200):
        count = int(rng.integers(1, 4))
        fn, text = oracle.random_expression(rng, count, int(rng.integers(1, 5)))
        k = make_elementwise(fn, count, 2, (4, 16))
        try:
            plan = k.plan_for(tuple(F((8, 32), "float64") for _ in range(count + 1)))
        except UnsupportedKernel as e:  # too many values parked at once, too long
            assert "more than" in str(e), text
            continue
        if plan.family == "copy2d":  # the expression was a bare input
            continue
        translated += 1
        inputs = oracle.make_elementwise_inputs(count, (8, 32), "float64", seed=translated)
        got = run_program(plan.roles["code"], plan.roles["consts"],
                          [inputs[i] for i in plan.roles["inputs"]], "float64", (8, 32))
        with np.errstate(all="ignore"):
            want = np.broadcast_to(fn(*inputs), (8, 32))
        assert np.array_equal(got, want, equal_nan=True), text
    assert translated > 120


def test_translation_details():
    a = make_elementwise(lambda t: (t + 1.0) * (t - 1.0) / ((t * t + 2.0) * (t + 3.0)), 1, 2, (4, 16))
    plan = a.plan_for((F((8, 32)), F((8, 32))))
    code, consts = plan.roles["code"], plan.roles["consts"]
    assert consts == [3.0, 2.0, 1.0]  # in order of first use: right operands are evaluated first
    ops = [c & 0xFF for c in code]
    # Three products/quotients of two inner nodes each park one value; at most
    # two are parked at once, so t2 is never needed.
    assert (ops.count(ew.SAVE0), ops.count(ew.SAVE0 + 1), ops.count(ew.SAVE0 + 2)) == (2, 1, 0)
    x = np.linspace(-2, 2, 256, dtype=np.float32).reshape(8, 32)
    want = (x + np.float32(1)) * (x - np.float32(1)) / ((x * x + np.float32(2)) * (x + np.float32(3)))
    assert np.array_equal(run_program(code, consts, [x], "float32"), want)
    # Reversed forms: constant on the left of a non-commutative operation.
    b = make_elementwise(lambda t: 1.0 / (2.0 - t * t), 1, 2, (4, 16))
    code = b.plan_for((F((8, 32)), F((8, 32)))).roles["code"]
    assert [c & 0xFF for c in code] == [ew.LOAD, ew.MUL, ew.RSUB, ew.RDIV]
    # The same tile used twice is one input; squares and roots through **.
    c = make_elementwise(lambda s, t: (s * s + t * t) ** 0.5, 2, 2, (4, 16))
    plan = c.plan_for((F((8, 32)), F((8, 32)), F((8, 32))))
    assert sorted(plan.roles["inputs"]) == [0, 1] and (plan.roles["code"][-1] & 0xFF) == ew.SQRT
    # A constant tile: no inputs at all.
    fill = make_elementwise(lambda t: t * 0.0 + 7.0, 1, 2, (4, 16))
    assert fill.plan_for((F((8, 32)), F((8, 32)))).roles["inputs"] == [0]


def test_bodies_outside_the_element_wise_family():
    W, H, DT = sym.W, sym.H, typename.DT
    target = dict(backend="nvvm", device="cuda:0")
    with pytest.raises(UnsupportedKernel, match="np.tanh"):
        make_elementwise(np.tanh, 1, 2, (4, 16)).plan_for((F((8, 32)), F((8, 32))))
    with pytest.raises(UnsupportedKernel, match="int32 or int64, not int16"):
        make_elementwise(lambda t: t + 1, 1, 2, (4, 16)).plan_for(
            (F((8, 32), "int16"), F((8, 32), "int16")))

    @kernel(work_shape=(W, H), group_shape=(4, 16), **target)
    def shifted(gr: CurrentGroup, a: Buffer[W, H, DT], out: Buffer[W, H, DT]):
        x, y = gr.work_offset
        gr.store(out[x:, y:], gr.load(a[x:, y + 1:], shape=gr.shape) * 2.0)

    with pytest.raises(UnsupportedKernel, match="another origin"):
        shifted.plan_for((F((8, 32)), F((8, 32))))

    @kernel(work_shape=(W, H), group_shape=(4, 16), **target)
    def row_broadcast(gr: CurrentGroup, a: Buffer[W, H, DT], out: Buffer[W, H, DT]):
        x, y = gr.work_offset
        t = gr.load(a[x:, y:], shape=gr.shape)
        gr.store(out[x:, y:], t - gr.load(a[x:, y:], shape=(gr.shape[0], 1)))

    with pytest.raises(UnsupportedKernel, match="broadcasting between tiles"):
        row_broadcast.plan_for((F((8, 32)), F((8, 32))))

    def deep(t):  # needs four values parked at once
        p = lambda u, v: (u + v) * (u - v)  # noqa: E731
        return p(p(p(p(t, t * 2.0), p(t, t * 3.0)), p(p(t, t * 4.0), p(t, t * 5.0))), t)

    with pytest.raises(UnsupportedKernel, match="more than|intermediate"):
        make_elementwise(deep, 1, 2, (4, 16)).plan_for((F((8, 32)), F((8, 32))))


def test_work_item_bodies_of_the_reference_tests():
    """python/hckernel/tests/test_kernel_sim.py:381-412, bodies unchanged: every
    work-item writes its own (linearised) global id under a bounds guard."""
    G, G1, G2, DT = sym.G, sym.G1, sym.G2, typename.DT
    target = dict(backend="nvvm", device="cuda:0")

    @kernel(work_shape=G, **target)
    def dims1(gr: CurrentGroup, arr: Buffer[G, DT]):
        @gr.workitems
        def inner(wi: CurrentWorkitem):
            gid = wi.global_id()[0]
            if gid < arr.shape[0]:
                arr[gid] = gid

        inner()

    plan = dims1.plan_for((F((12,), "float64"),))
    assert (plan.family, plan.roles["inputs"], plan.roles["out"]) == ("map_elements", [], 0)
    got = run_program(plan.roles["code"], plan.roles["consts"], [], "float64", (12,))
    assert np.array_equal(got, np.arange(12))

    @kernel(work_shape=(G1, G2), **target)
    def dims2(gr: CurrentGroup, arr: Buffer[G1, G2, DT]):
        @gr.workitems
        def inner(wi: CurrentWorkitem):
            gid = wi.global_id()[:2]
            if gid[0] < arr.shape[0] and gid[1] < arr.shape[1]:
                arr[gid] = gid[0] * arr.shape[1] + gid[1]

        inner()

    plan = dims2.plan_for((F((12, 5), "float64"),))
    got = run_program(plan.roles["code"], plan.roles["consts"], [], "float64", (12, 5))
    assert np.array_equal(got, np.arange(60).reshape(12, 5))

    # The machine computes indices in the element type.  float32 holds integers up
    # to 2**24 exactly: at that many elements the program still gives what integer
    # arithmetic rounded once gives (checked on the last rows, where the values are
    # largest); one row more is refused, float64 is not.
    rows, cols = 4096, 4096
    plan = dims2.plan_for((F((rows, cols), "float32"),))
    last = np.arange(rows - 8, rows, dtype=np.float32)[:, None]
    col = np.arange(cols, dtype=np.float32)[None, :]
    with np.errstate(all="ignore"):  # the machine's own order: one rounding per operation
        got = last * np.float32(cols) + col
    exact = (np.arange(rows - 8, rows, dtype=np.int64)[:, None] * cols
             + np.arange(cols, dtype=np.int64)[None, :])
    assert got.dtype == np.float32 and np.array_equal(got, exact.astype(np.float32))
    with pytest.raises(UnsupportedKernel, match="exact in float32 only up to"):
        dims2.plan_for((F((rows + 1, cols), "float32"),))
    assert dims2.plan_for((F((rows + 1, cols), "float64"),)).family == "map_elements"


def test_work_item_bodies_with_reads_and_their_limits():
    W, H, DT = sym.W, sym.H, typename.DT
    target = dict(backend="nvvm", device="cuda:0")

    def item_kernel(body, work=(W, H)):
        @kernel(work_shape=work, **target)
        def k(gr: CurrentGroup, a: Buffer[W, H, DT], out: Buffer[W, H, DT]):
            @gr.workitems
            def inner(wi: CurrentWorkitem):
                body(wi.global_id(), a, out)

            inner()

        return k

    def scaled(gid, a, out):
        i, j = gid
        if i < out.shape[0] and j < out.shape[1]:
            out[i, j] = a[i, j] * 2.0 + j

    plan = item_kernel(scaled).plan_for((F((6, 9)), F((6, 9))))
    assert (plan.roles["inputs"], plan.roles["out"]) == ([0], 1)
    a = np.arange(54, dtype=np.float32).reshape(6, 9)
    got = run_program(plan.roles["code"], plan.roles["consts"], [a], "float32")
    assert np.array_equal(got, a * 2 + np.arange(9, dtype=np.float32))

    def half(gid, a, out):  # a condition that is not a bounds guard: the work-item kernel
        if gid[0] < 3:
            out[gid] = a[gid]

    plan = item_kernel(half).plan_for((F((6, 9)), F((6, 9))))
    assert plan.family == "work_items" and plan.roles["guards"][0] == (0, 3, 0, 9)

    def transposed(gid, a, out):
        out[gid[1], gid[0]] = a[gid]

    with pytest.raises(UnsupportedKernel, match="one index per dimension, in order"):
        item_kernel(transposed).plan_for((F((6, 6)), F((6, 6))))

    def shifted_read(gid, a, out):
        out[gid] = a[gid[1], gid[0]]

    with pytest.raises(UnsupportedKernel, match="own index"):
        item_kernel(shifted_read).plan_for((F((6, 6)), F((6, 6))))

    def plain(gid, a, out):
        out[gid] = a[gid] + 1.0

    with pytest.raises(UnsupportedKernel, match="work shape stops"):
        item_kernel(plain, work=(W, 4)).plan_for((F((6, 9)), F((6, 9))))

    def local(gid, a, out):
        out[gid] = a[gid]

    @kernel(work_shape=(W, H), **target)
    def uses_local_id(gr: CurrentGroup, a: Buffer[W, H, DT], out: Buffer[W, H, DT]):
        @gr.workitems
        def inner(wi: CurrentWorkitem):
            out[wi.local_id()] = a[wi.local_id()]

        inner()

    with pytest.raises(UnsupportedKernel):  # arrays are indexed by global ids
        uses_local_id.plan_for((F((6, 9)), F((6, 9))))


OPERATOR_CASES = oracle.operator_cases()


@pytest.mark.parametrize("case", OPERATOR_CASES, ids=lambda c: c[0])
def test_operator_table_oracle_matches_the_reference_simulator(golden, case):
    """// % / with zero divisors, ** with results that are not finite, comparisons
    as 0/1 factors, integer tiles: the oracle against the outputs of the
    reference simulator, bit for bit, unwritten elements (-77) included."""
    name, fn, inputs, group = case
    out = np.full(inputs[0].shape, -77, inputs[0].dtype)
    oracle.elementwise(fn, list(inputs), out, group)
    assert np.array_equal(out, golden[name])


@pytest.mark.parametrize("case", OPERATOR_CASES, ids=lambda c: c[0])
def test_operator_table_translates_to_an_equivalent_program(golden, case):
    """The recorded body as a program, run one NumPy operation per instruction:
    the elements it marks valid are the ones the reference wrote, with the
    reference's values (bit for bit for everything but **, whose float32 power
    the reference computes through float64)."""
    name, fn, inputs, group = case
    dtype = inputs[0].dtype.name
    k = make_elementwise(fn, len(inputs), 2, group)
    plan = k.plan_for(tuple(F(a.shape, dtype) for a in inputs) + (F(inputs[0].shape, dtype),))
    assert plan.family == "map_elements"
    valid = []
    with np.errstate(all="ignore"):
        got = run_program(plan.roles["code"], plan.roles["consts"],
                          [inputs[i] for i in plan.roles["inputs"]], dtype, valid_out=valid)
    out = np.where(valid[0], got, np.asarray(-77, got.dtype))
    want = golden[name]
    if "pow" in name:
        assert np.array_equal(out == -77, want == -77)
        np.testing.assert_allclose(out, want, rtol=1e-6)
    else:
        assert np.array_equal(out, want)


def test_operator_table_refusals_follow_numpy():
    shape = (8, 32)
    ints = (F(shape, "int32"), F(shape, "int32"), F(shape, "int32"))
    floats = (F(shape), F(shape), F(shape))
    two = lambda fn: make_elementwise(fn, 2, 2, (4, 16))  # noqa: E731
    with pytest.raises(UnsupportedKernel, match="floating-point values"):
        two(lambda a, b: a / b).plan_for(ints)
    with pytest.raises(UnsupportedKernel, match="floating-point values"):
        two(lambda a, b: a * 2.5 + b).plan_for(ints)
    with pytest.raises(UnsupportedKernel, match="constant exponents"):
        two(lambda a, b: a ** b).plan_for(ints)
    with pytest.raises(ValueError, match="negative integer powers"):
        two(lambda a, b: a ** -1 + b).plan_for(ints)
    with pytest.raises(TypeError, match="shifts are not supported"):
        two(lambda a, b: a << b).plan_for(floats)
    with pytest.raises(TypeError, match="only for truth values"):
        two(lambda a, b: a & b).plan_for(floats)
    with pytest.raises(ValueError, match="truth value of a tile"):
        two(lambda a, b: (not a) + b).plan_for(floats)
    # What NumPy allows: logical operators on the results of comparisons, stored
    # as 0 / 1; shifts and bitwise operators on integer tiles.
    plan = two(lambda a, b: ((a < b) & (b > 0.0)) | ~(a >= 1.0)).plan_for(floats)
    rng = np.random.default_rng(4)
    a, b = rng.standard_normal(shape).astype("float32"), rng.standard_normal(shape).astype("float32")
    got = run_program(plan.roles["code"], plan.roles["consts"],
                      [(a, b)[i] for i in plan.roles["inputs"]], "float32")
    assert np.array_equal(got, (((a < b) & (b > 0)) | ~(a >= 1)).astype("float32"))
    plan = two(lambda a, b: ((a << 3) ^ (b >> 1)) & ~a | (a % 7 == 3)).plan_for(ints)
    a, b = rng.integers(-99, 99, shape, dtype="int32"), rng.integers(-99, 99, shape, dtype="int32")
    got = run_program(plan.roles["code"], plan.roles["consts"],
                      [(a, b)[i] for i in plan.roles["inputs"]], "int32")
    assert np.array_equal(got, ((a << 3) ^ (b >> 1)) & ~a | (a % 7 == 3))
