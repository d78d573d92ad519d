"""The ahead-of-time half of the element-wise and row bodies, on CPU: the
header of constant programs must be what the listed bodies translate to today,
and every listed program, run one NumPy operation per instruction, must agree
with NumPy on the body it came from."""

import numpy as np
import pytest

from hc_b200.hckernel import precompiled
from tests.test_elementwise_cpu import run_program


def test_header_of_constant_programs_is_current():
    assert precompiled.HEADER.read_text() == precompiled.render(), (
        "run `python -m hc_b200.hckernel.precompiled` and rebuild")


def test_listed_programs_are_distinct_and_small():
    rows, maps = precompiled.translate()
    assert len(rows) == len(precompiled.ROW_BODIES) and len(maps) == len(precompiled.MAP_BODIES)
    for _, count, code in rows + maps:
        assert 1 <= len(code) <= 32 and 1 <= count <= 4


@pytest.mark.parametrize("body", precompiled.ROW_BODIES + precompiled.MAP_BODIES,
                         ids=lambda b: b[0])
def test_program_words_compute_the_body(body):
    name, fn, count = body
    rows, maps = precompiled.translate()
    code = {n: c for n, _, c in rows + maps}[name]
    rng = np.random.default_rng(5)
    inputs = [rng.standard_normal((6, 40)) + 0.25 for _ in range(count)]
    # The constants are operands, not part of the program: take them from a
    # fresh translation of the same body.
    from hc_b200.workloads import make_elementwise, make_rowwise

    arrays = tuple(precompiled._Array((6, 40), "float64") for _ in range(count + 1))
    is_row = any(n == name for n, _, _ in rows)
    plan = (make_rowwise(fn, count).plan_for(arrays + (2,)) if is_row
            else make_elementwise(fn, count, 2, (2, 8)).plan_for(arrays))
    assert tuple(plan.roles["code"]) == code
    got = run_program(code, plan.roles["consts"], [inputs[i] for i in plan.roles["inputs"]],
                      "float64")
    with np.errstate(all="ignore"):
        np.testing.assert_allclose(got, fn(*inputs), rtol=1e-13, atol=1e-14)
