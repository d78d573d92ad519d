"""Sub-group scope (reference python/hckernel/kernel_api.py:229-240, 378-393)
without a GPU: the oracle's restatement against the outputs of the reference
simulator, the recorded sub-group function as a launch on the grid of
sub-groups, and what such a function may not do."""

import types

import numpy as np
import pytest

from hc_b200.hckernel.kernel import *  # noqa: F401,F403
from hc_b200.hckernel.kernel import UnsupportedKernel
from oracle import workitems as oracle_items
from tests.test_elementwise_cpu import run_program

CASES = oracle_items.subgroup_cases()
NS = types.SimpleNamespace(kernel=kernel, sym=sym, CurrentGroup=CurrentGroup, Buffer=Buffer,
                           DT=typename.DT, atomic_ref=atomic_ref,
                           target=dict(backend="nvvm", device="cuda:0"))


class F:
    def __init__(self, shape, dtype):
        self.shape, self.dtype = tuple(shape), np.dtype(dtype)


@pytest.mark.parametrize("case", CASES, ids=lambda c: c["name"])
def test_oracle_matches_the_reference_simulator(golden, case):
    shape, dtype = case["out"]
    out = np.full(shape, -77, dtype)
    case["oracle"](case["inputs"], out)
    if "sums" in case["name"]:  # the reference adds in the same order: equal, not just close
        assert np.array_equal(out, golden[case["name"]])
        np.testing.assert_allclose(out[0], -77 + case["inputs"][0].sum(), rtol=1e-13)
        return
    assert np.array_equal(out, golden[case["name"]])
    assert not (out == -77).any()  # the sub-groups cover the arrays


@pytest.mark.parametrize("case", CASES, ids=lambda c: c["name"])
def test_recorded_subgroup_function_becomes_an_equivalent_launch(golden, case):
    shape, dtype = case["out"]
    k = case["make"](NS)
    plan = k.plan_for(tuple(F(a.shape, a.dtype) for a in case["inputs"]) + (F(shape, dtype),))
    if "sums" in case["name"]:
        # One partial sum per sub-group into element 0: the whole-array sum.
        assert plan.family == "reduce_all" and (plan.roles["a"], plan.roles["result"]) == (0, 1)
        return
    assert plan.family == "map_elements" and plan.roles["out"] == len(case["inputs"])
    got = run_program(plan.roles["code"], plan.roles["consts"],
                      [case["inputs"][i] for i in plan.roles["inputs"]], dtype)
    want = golden[case["name"]]
    # The reference carries Python-float factors on in float64 (`a * 2.0`).
    np.testing.assert_allclose(got, want, rtol=3e-7 if dtype == np.float32 else 0)


def _one_dimensional(body, group=64, subgroup=16):
    G, DT = sym.G, typename.DT

    @kernel(work_shape=G, group_shape=group, subgroup_size=subgroup, backend="nvvm",
            device="cuda:0")
    def k(gr: CurrentGroup, a: Buffer[G, DT], out: Buffer[G, DT]):
        @gr.subgroups
        def inner(sg):
            body(gr, sg, a, out)

        inner()

    return lambda n=1000: k.plan_for((F((n,), np.float32), F((n,), np.float32)))


def test_what_a_subgroup_function_may_not_do():
    def own_part(gr, sg, a, out):
        x = gr.work_offset[0] + sg.subgroup_id()[0] * sg.size()
        gr.store(out[x:], gr.load(a[x:], shape=sg.size()) + 1.0)

    assert _one_dimensional(own_part)().family == "map_elements"
    # a size given by a literal symbol is resolved at the call, as the group shape is
    assert _one_dimensional(own_part, subgroup=32)().family == "map_elements"

    def by_id_alone(gr, sg, a, out):  # every group would write the same elements
        x = sg.subgroup_id()[0] * sg.size()
        gr.store(out[x:], gr.load(a[x:], shape=sg.size()) + 1.0)

    with pytest.raises(UnsupportedKernel, match="sub-group id alone"):
        _one_dimensional(by_id_alone)()

    def wrong_step(gr, sg, a, out):  # parts of 16 placed every 32: gaps
        x = gr.work_offset[0] + sg.subgroup_id()[0] * 2 * sg.size()
        gr.store(out[x:], gr.load(a[x:], shape=sg.size()) + 1.0)

    with pytest.raises(UnsupportedKernel):
        _one_dimensional(wrong_step)()

    def group_id(gr, sg, a, out):
        gr.store(out[gr.id[0] * 64:], gr.load(a[gr.id[0] * 64:], shape=64))

    with pytest.raises(UnsupportedKernel, match="group.id inside a sub-group"):
        _one_dimensional(group_id)()

    with pytest.raises(UnsupportedKernel, match="does not divide"):
        _one_dimensional(own_part, group=40, subgroup=16)()


def test_subgroup_and_group_level_stores_do_not_mix():
    G, DT = sym.G, typename.DT

    @kernel(work_shape=G, group_shape=64, subgroup_size=16, backend="nvvm", device="cuda:0")
    def k(gr: CurrentGroup, a: Buffer[G, DT], out: Buffer[G, DT], other: Buffer[G, DT]):
        x0 = gr.work_offset[0]
        gr.store(other[x0:], gr.load(a[x0:], shape=gr.shape[0]))

        @gr.subgroups
        def inner(sg):
            x = gr.work_offset[0] + sg.subgroup_id()[0] * sg.size()
            gr.store(out[x:], gr.load(a[x:], shape=sg.size()) + 1.0)

        inner()

    with pytest.raises(UnsupportedKernel, match="mix sub-group functions"):
        k.plan_for(tuple(F((256,), np.float32) for _ in range(3)))


def test_subgroup_size_as_a_literal_symbol():
    """subgroup_size may be a symbol listed in `literals`, bound by a call argument
    (reference kernel_api.py:26-31, tests/test_kernel_sim.py:254-283)."""
    G, DT, SG = sym.G, typename.DT, sym.SG

    @kernel(work_shape=G, group_shape=64, subgroup_size=SG, literals={SG}, backend="nvvm",
            device="cuda:0")
    def k(gr: CurrentGroup, a: Buffer[G, DT], out: Buffer[G, DT], size: SG):
        @gr.subgroups
        def inner(sg):
            x = gr.work_offset[0] + sg.subgroup_id()[0] * sg.size()
            gr.store(out[x:], gr.load(a[x:], shape=sg.size()) * 2.0 + 1.0)

        inner()

    arrays = (F((1000,), np.float32), F((1000,), np.float32))
    assert k.plan_for(arrays + (16,)).family == "map_elements"
    with pytest.raises(UnsupportedKernel, match="does not divide"):
        k.plan_for(arrays + (24,))
