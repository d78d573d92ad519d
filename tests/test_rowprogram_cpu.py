"""Row bodies (reductions along the rows used again in the same expression) on
CPU: the oracle against the reference simulator's outputs, bit for bit, and the
front door - the recorded expression must become a multi-pass program for the
machine of csrc/kernels/row_program.cu that, run here in NumPy, agrees with
NumPy on the same arrays.  No kernel is launched."""

import numpy as np
import pytest

from hc_b200.hckernel import elementwise as ew
from hc_b200.hckernel.kernel import *  # noqa: F401,F403
from hc_b200.hckernel.kernel import UnsupportedKernel
from hc_b200.workloads import make_kernels, make_rowwise
from oracle import workloads as oracle
from tests.test_elementwise_cpu import F, run_program

CASES = oracle.rowwise_cases()


@pytest.mark.parametrize("case", CASES, ids=lambda c: c[0])
def test_oracle_matches_the_reference_simulator(golden, case):
    name, fn, count, shape, dtype, group_rows = case
    inputs = oracle.make_elementwise_inputs(count, shape, dtype, seed=8)
    out = np.zeros(shape, dtype)
    oracle.rowwise(fn, inputs, out, group_rows)
    assert np.array_equal(out, golden[name])


@pytest.mark.parametrize("case", CASES, ids=lambda c: c[0])
def test_recorded_row_body_becomes_a_multi_pass_program(golden, case):
    name, fn, count, shape, dtype, group_rows = case
    k = make_rowwise(fn, count)
    plan = k.plan_for(tuple(F(shape, dtype) for _ in range(count + 1)) + (group_rows,))
    assert plan.family == "row_program"
    assert sorted(plan.roles["inputs"]) == list(range(count)) and plan.roles["out"] == count
    code = plan.roles["code"]
    ops = [c & 0xFF for c in code]
    passes = sum(op in (ew.RSUM, ew.RMAX) for op in ops)
    assert passes >= 1 and ops[-1] not in (ew.RSUM, ew.RMAX)
    inputs = oracle.make_elementwise_inputs(count, shape, dtype, seed=8)
    got = run_program(code, plan.roles["consts"], [inputs[i] for i in plan.roles["inputs"]], dtype)
    with np.errstate(all="ignore"):
        want = fn(*inputs)
    # Same operations on the same values; only NumPy's pairwise summation order
    # and its float64 detours for Python-float operands differ.
    tol = dict(rtol=2e-6, atol=1e-6) if dtype == "float32" else dict(rtol=1e-14, atol=0)
    np.testing.assert_allclose(got, want, **tol)
    np.testing.assert_allclose(got, golden[name], **tol)


def test_pass_structure_of_log_softmax():
    name, fn, count, shape, dtype, group_rows = CASES[2]
    plan = make_rowwise(fn).plan_for((F(shape, dtype), F(shape, dtype), group_rows))
    ops = [(c & 0xFF, c >> 8) for c in plan.roles["code"]]
    # max(t) -> s0 ; sum(exp(t - s0)) -> s1 ; (t - s0) - log(s1)
    assert ops[:2] == [(ew.LOAD, 0), (ew.RMAX, 0)]
    second = ops[2:ops.index((ew.RSUM, 1)) + 1]
    assert second == [(ew.LOAD, 0), (ew.SUB, ew.SRC_SCALAR + 0), (ew.EXP, 0), (ew.RSUM, 1)]
    # The last pass opens with a uniform prologue - log(s1) once per row, kept in
    # s2 - and then walks the row with three cheap instructions.
    last = ops[ops.index((ew.RSUM, 1)) + 1:]
    u = ew.UNIFORM
    assert last == [(ew.LOAD | u, ew.SRC_SCALAR + 1), (ew.LOG | u, 0), (ew.SET | u, 2),
                    (ew.LOAD, 0), (ew.SUB, ew.SRC_SCALAR + 0), (ew.SUB, ew.SRC_SCALAR + 2)]
    # The same reduction written twice is computed once.
    twice = make_rowwise(lambda t: (t - t.max(axis=1, keepdims=True))
                         / (t.max(axis=1, keepdims=True) + 2.0))
    ops = [c & 0xFF for c in twice.plan_for((F((8, 16)), F((8, 16)), 4)).roles["code"]]
    assert ops.count(ew.RMAX) == 1


def test_softmax_itself_keeps_its_own_kernel():
    k = make_kernels("cuda:0")
    assert k.softmax.plan_for((F((30, 25)), F((30, 25)), 8)).family == "softmax_rows"


def test_row_bodies_outside_the_family():
    with pytest.raises(UnsupportedKernel, match="axis=1, keepdims=True"):
        make_rowwise(lambda t: t - t.sum(axis=0, keepdims=True)).plan_for(
            (F((8, 16)), F((8, 16)), 8))
    with pytest.raises(UnsupportedKernel, match="more than 4 different row reductions"):
        make_rowwise(lambda t: t.sum(axis=1, keepdims=True) + (t * 2.0).sum(axis=1, keepdims=True)
                     + (t * 3.0).sum(axis=1, keepdims=True) + (t * 4.0).sum(axis=1, keepdims=True)
                     + (t * 5.0).sum(axis=1, keepdims=True) + t).plan_for(
            (F((8, 16)), F((8, 16)), 8))
    M, N, GM, DT = sym.M, sym.N, sym.GM, typename.DT

    @kernel(work_shape=M, group_shape=GM, backend="nvvm", device="cuda:0")
    def half_rows(gr: CurrentGroup, a: Buffer[M, N, DT], out: Buffer[M, N, DT], gshape: GM):
        m0 = gr.work_offset[0]
        t = gr.load(a[m0:, :], shape=(gr.shape[0], N // 2))
        gr.store(out[m0:, :], t - t.mean(axis=1, keepdims=True))

    with pytest.raises(UnsupportedKernel, match="whole rows"):
        half_rows.plan_for((F((8, 16)), F((8, 16)), 8))
    with pytest.raises(UnsupportedKernel, match="float32 or float64"):
        make_rowwise(lambda t: t - t.max(axis=1, keepdims=True)).plan_for(
            (F((8, 16), "int32"), F((8, 16), "int32"), 8))


def test_random_row_bodies_translate():
    """150 random row bodies (one or two reductions, the second possibly of an
    expression of the first): the multi-pass program, run one NumPy operation
    per instruction in float64, must agree with NumPy on the expression."""
    rng = np.random.default_rng(77)
    translated = 0
    for _ in range(150):
        count = int(rng.integers(1, 3))
        fn, text = oracle.random_row_expression(rng, count)
        k = make_rowwise(fn, count)
        try:
            plan = k.plan_for(tuple(F((8, 32), "float64") for _ in range(count + 1)) + (4,))
        except UnsupportedKernel as e:  # too many values parked at once, too long
            assert "more than" in str(e), text
            continue
        assert plan.family == "row_program", text
        translated += 1
        inputs = oracle.make_elementwise_inputs(count, (8, 32), "float64", seed=translated)
        got = run_program(plan.roles["code"], plan.roles["consts"],
                          [inputs[i] for i in plan.roles["inputs"]], "float64", (8, 32))
        with np.errstate(all="ignore"):
            want = fn(*inputs)
        np.testing.assert_allclose(got, want, rtol=1e-12, atol=1e-13, err_msg=text)
    assert translated > 100
