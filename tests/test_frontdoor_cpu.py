"""The recording front door on CPU: which kernel family a decorated body is
recognised as, symbol binding, tunables, launch-geometry defaults and the
errors for bodies outside the precompiled families.  No kernel is launched:
`plan_for` stops before the native dispatcher."""

import numpy as np
import pytest
import sympy

from hc_b200.hckernel.kernel import *  # noqa: F401,F403
from hc_b200.hckernel.kernel import UnsupportedKernel, suggest_block_size
from hc_b200.hckernel.kernel_api import Affine
from hc_b200.workloads import make_kernels

DT = typename.DT
TARGET = dict(backend="nvvm", device="cuda:0")


class FakeTensor:
    def __init__(self, shape, dtype="float32"):
        self.shape, self.dtype = tuple(shape), dtype


F = FakeTensor


@pytest.fixture(scope="module")
def k():
    return make_kernels("cuda:0")


def test_workload_kernels_are_recognised(k):
    assert k.copy.plan_for((F((111, 813), "int32"), F((111, 813), "int32"))).family == "copy2d"
    p = k.softmax.plan_for((F((30, 25)), F((30, 25)), 8))
    assert (p.family, p.roles) == ("softmax_rows", {"x": 0, "out": 1})
    p = k.reduce_rows.plan_for((F((300, 64)), F((300,)), F((300,)), 256))
    assert (p.family, p.roles) == ("reduce_rows", {"x": 0, "sum_out": 1, "max_out": 2})
    p = k.dot.plan_for((F((256, 256)), F((256, 256)), F((256, 256)), (64, 64)))
    assert (p.family, p.roles) == ("gemm", {"a": 0, "b": 1, "out": 2})
    p = k.dot.plan_for((F((70, 33)), F((33, 45)), F((70, 45)), (64, 64)))  # ragged K and edges
    assert p.family == "gemm"
    p = k.dot_fullk.plan_for((F((128, 512), "bfloat16"), F((512, 256), "bfloat16"),
                              F((128, 256), "bfloat16"), (128, 128)))
    assert p.family == "gemm"
    p = k.dequant_dot.plan_for((F((128, 512), "bfloat16"), F((512, 256), "int8"), F((256,)),
                                F((128, 256), "bfloat16"), (128, 128)))
    assert (p.family, p.roles) == ("gemm_w8a16", {"a": 0, "w": 1, "scale": 2, "out": 3})


def test_plans_are_cached_per_shape_and_dtype(k):
    args = (F((64, 32)), F((64, 32)), 8)
    assert k.softmax.plan_for(args) is k.softmax.plan_for((F((64, 32)), F((64, 32)), 8))
    assert k.softmax.plan_for(args) is not k.softmax.plan_for((F((64, 48)), F((64, 48)), 8))


def test_tunables_and_parametrize(k):
    MI, KB = sym.MI, sym.KB
    tuned = k.dot.parametrize({KB: 32, MI: 2})
    assert tuned.tuned == {KB: 32, MI: 2} and k.dot.tuned == {}
    assert tuned.plan_for((F((70, 33)), F((33, 45)), F((70, 45)), (8, 8))).family == "gemm"
    # KB larger than K: a single zero-padded block still covers K.
    assert k.dot.parametrize({KB: 64}).plan_for(
        (F((16, 33)), F((33, 8)), F((16, 8)), (8, 8))).family == "gemm"


def test_unrolled_copy_from_the_reference_tests():
    W, H, V = sym.W, sym.H, sym.V
    H1 = sympy.ceiling(H / V)

    @kernel(work_shape=(W, H1), literals=[V], **TARGET)
    def copy_kernel(group: CurrentGroup, src: Buffer[W, H, DT], dst: Buffer[W, H, DT], v: V):
        x, y = group.work_offset
        val = group.vload(src[x:, y * V :], shape=(group.shape[0], group.shape[1] * V))
        group.store(dst[x:, y * V :], val)

    for shape in [(1, 27), (111, 813), (256, 1024)]:
        for unroll in (1, 2, 4):
            assert copy_kernel.plan_for((F(shape, "int32"), F(shape, "int32"), unroll)).family == "copy2d"


def test_scalar_reductions_from_the_reference_tests():
    # python/hckernel/tests/test_examples.py:31-71, both forms.
    WS, GS, N = sym.WS, sym.GS, sym.N
    TN = TunableParam(N, 2, range(1, 64))

    def ceil_div(a, b):
        return (a + b - 1) // b

    @kernel(work_shape=ceil_div(WS, N), group_shape=GS, tunables=TN, **TARGET)
    def reduction_1(gr: CurrentGroup, a: Buffer[WS, DT], result: Buffer[1, DT], gshape: GS):
        a_view = gr.load(a[gr.work_offset[0] * N :], shape=gr.size * N)
        atomic_ref(result)[0] += a_view.sum()

    @kernel(work_shape=ceil_div(WS, N), group_shape=GS, tunables=TN, **TARGET)
    def reduction_2(group: CurrentGroup, a: Buffer[WS, DT], result: Buffer[1, DT], gshape: GS):
        temp_result = group.zeros(group.size, dtype=a.dtype)
        for i in range(N):
            work_offset = group.work_offset[0] * N + i * group.size
            a_view = group.load(a[work_offset:], shape=group.size)
            temp_result += a_view
        atomic_ref(result)[0] += temp_result.sum()

    for kern in (reduction_1, reduction_2, reduction_2.parametrize({N: 5})):
        plan = kern.plan_for((F((20,), "int64"), F((1,), "float64"), 8))
        assert (plan.family, plan.roles) == ("reduce_all", {"a": 0, "result": 1})


def test_pairwise_distance_from_the_reference_tests():
    # python/hckernel/tests/test_examples.py:261-289
    M, N, D, GM, GN, MI, NI = sym.M, sym.N, sym.D, sym.GM, sym.GN, sym.MI, sym.NI

    def ceil_div(a, b):
        return (a + b - 1) // b

    tun = (TunableParam(MI, 1, range(1, 8)), TunableParam(NI, 1, range(1, 8)))

    @kernel(work_shape=(ceil_div(M, MI), ceil_div(N, NI)), group_shape=(GM, GN), tunables=tun,
            **TARGET)
    def pw_distance(gr: CurrentGroup, a: Buffer[M, D, DT], b: Buffer[N, D, DT],
                    out: Buffer[M, N, DT], gshape: (GM, GN)):
        m_start = gr.work_offset[0] * MI
        n_start = gr.work_offset[1] * NI
        m_block = gr.shape[0] * MI
        n_block = gr.shape[1] * NI
        a_view = gr.load(a[m_start:, :], shape=(m_block, D))
        b_view = gr.load(b[n_start:, :], shape=(n_block, D))
        diff = a_view[:, None, :] - b_view[None, :, :]
        gr.store(out[m_start:, n_start:], np.linalg.norm(diff, axis=2))

    plan = pw_distance.plan_for((F((16, 8), "float64"), F((32, 8), "float64"),
                                 F((16, 32), "float64"), (8, 8)))
    assert (plan.family, plan.roles) == ("pairwise_distance", {"a": 0, "b": 1, "out": 2})
    assert pw_distance.parametrize({MI: 3}).plan_for(
        (F((70, 19)), F((45, 19)), F((70, 45)), (8, 8))).family == "pairwise_distance"


def test_tuned_params_round_trip_and_parametrize(tmp_path, k):
    from hc_b200.hckernel.kernel import TunedParams, autotune

    KB, MI = sym.KB, sym.MI
    tp = TunedParams({KB: 32, MI: 2}, {"gemm_variant": 2}, {"{}": 0.5})
    path = tmp_path / "tuned.json"
    tp.save(path)
    back = autotune.load(path)
    assert dict(back) == {KB: 32, MI: 2} and back.options == {"gemm_variant": 2}
    tuned = k.dot.parametrize(back)
    assert tuned.tuned == {KB: 32, MI: 2} and tuned.options == {"gemm_variant": 2}
    assert k.dot.options == {}
    # Options survive a further parametrize with plain symbols.
    assert tuned.parametrize({KB: 64}).options == {"gemm_variant": 2}


def test_symbol_conflicts_and_rank_errors(k):
    with pytest.raises(ValueError, match="Symbol value conflict for M"):
        k.softmax.plan_for((F((30, 25)), F((31, 25)), 8))
    with pytest.raises(ValueError, match="expected rank 2"):
        k.softmax.plan_for((F((30,)), F((30, 25)), 8))
    with pytest.raises(TypeError, match="missing argument"):
        k.softmax.plan_for((F((30, 25)), F((30, 25))))


def test_bodies_outside_the_families_are_refused():
    M, N, GM = sym.M, sym.N, sym.GM

    @kernel(work_shape=M, group_shape=GM, **TARGET)
    def half_rows(gr: CurrentGroup, a: Buffer[M, N, DT], out: Buffer[M, N, DT], gshape: GM):
        m0 = gr.work_offset[0]
        t = gr.load(a[m0:, :], shape=(gr.shape[0], N // 2))  # not whole rows
        e = np.exp(t - t.max(axis=1, keepdims=True))
        gr.store(out[m0:, :], e / e.sum(axis=1, keepdims=True))

    with pytest.raises(UnsupportedKernel, match="whole rows"):
        half_rows.plan_for((F((32, 64)), F((32, 64)), 8))

    @kernel(work_shape=M, group_shape=GM, **TARGET)
    def gappy(gr: CurrentGroup, a: Buffer[M, N, DT], out: Buffer[M, N, DT], gshape: GM):
        m0 = gr.work_offset[0] * 2  # every other block of rows is skipped
        t = gr.load(a[m0:, :], shape=(gr.shape[0], N))
        gr.store(out[m0:, :], t)

    with pytest.raises(UnsupportedKernel, match="leave gaps"):
        gappy.plan_for((F((32, 64)), F((32, 64)), 8))

    WS, GS = sym.WS, sym.GS

    @kernel(work_shape=WS, group_shape=GS, **TARGET)
    def overlapping_reduce(gr: CurrentGroup, a: Buffer[WS, DT], result: Buffer[1, DT], gshape: GS):
        v = gr.load(a[gr.work_offset[0] :], shape=gr.size * 2)  # tiles twice as long as the step
        atomic_ref(result)[0] += v.sum()

    with pytest.raises(UnsupportedKernel, match="overlap"):
        overlapping_reduce.plan_for((F((20,)), F((1,)), 8))

    @kernel(work_shape=M, group_shape=GM, **TARGET)
    def squares(gr: CurrentGroup, a: Buffer[M, N, DT], out: Buffer[M, N, DT], gshape: GM):
        m0 = gr.work_offset[0]
        t = gr.load(a[m0:, :], shape=(gr.shape[0], N))
        gr.store(out[m0:, :], t * t)

    # Element-wise arithmetic is a family of its own (tests/test_elementwise_cpu.py).
    assert squares.plan_for((F((32, 64)), F((32, 64)), 8)).family == "map_elements"

    @kernel(work_shape=M, group_shape=GM, **TARGET)
    def column_sums(gr: CurrentGroup, a: Buffer[M, N, DT], out: Buffer[N, DT], gshape: GM):
        m0 = gr.work_offset[0]
        t = gr.load(a[m0:, :], shape=(gr.shape[0], N))
        gr.store(out, t.sum(axis=0))

    with pytest.raises(UnsupportedKernel, match="matches none"):
        column_sums.plan_for((F((32, 64)), F((64,)), 8))

    @kernel(work_shape=M, group_shape=GM, **TARGET)
    def with_subgroups(gr: CurrentGroup, a: Buffer[M, N, DT], out: Buffer[M, N, DT], gshape: GM):
        gr.subgroups(lambda sg: None)

    # Sub-group functions are a scope of their own (tests/test_subgroups_cpu.py); the
    # default sub-group size of 16 does not divide a group of 8.
    with pytest.raises(UnsupportedKernel, match="does not divide the group's last axis"):
        with_subgroups.plan_for((F((32, 64)), F((32, 64)), 8))

    @kernel(work_shape=M, group_shape=GM, **TARGET)
    def with_barrier(gr: CurrentGroup, a: Buffer[M, N, DT], out: Buffer[M, N, DT], gshape: GM):
        gr.barrier()

    # At group level a barrier has nothing to wait for (the reference's returns at
    # once, kernel_api.py:416-420); what is refused is the body that stores nothing.
    with pytest.raises(UnsupportedKernel, match="stores nothing"):
        with_barrier.plan_for((F((32, 64)), F((32, 64)), 8))


def test_default_group_shape_follows_the_launch_heuristic():
    # x is the last work dimension (mlir/lib/Transforms/LowerHKernel.cpp:296,343-344).
    assert suggest_block_size((813, 111)) == (813, 1)
    assert suggest_block_size((20, 10)) == (20, 10)
    assert suggest_block_size((1, 27)) == (1, 27)
    assert suggest_block_size((4096, 4096)) == (1024, 1)


def test_affine_offsets():
    g0, g1 = Affine(0, {0: 1}), Affine(0, {1: 1})
    assert (g0 * 8 + 3).key() == (3, ((0, 8),))
    assert (g0 * 4) * 2 == g0 * 8
    assert (g0 + g1 - g0) == g1
    assert int(Affine(7) // 2) == 3 and int(Affine(7) % 4) == 3
    # Products, quotients and remainders of group offsets leave the affine
    # family: no whole-array kernel takes such a tile origin (tests/
    # test_mapped_cpu.py covers where they are accepted).
    with pytest.raises(UnsupportedKernel, match="not affine"):
        _ = (g0 * g1).const
    with pytest.raises(UnsupportedKernel, match="not affine"):
        _ = (g0 % 3).coefs
    with pytest.raises(UnsupportedKernel):
        int(g0)


def test_decorator_signature_matches_the_reference():
    import inspect

    params = inspect.signature(kernel).parameters
    assert list(params) == ["work_shape", "group_shape", "subgroup_size", "literals", "tunables",
                            "backend", "device"]
    assert params["backend"].default == "rocm" and params["device"].default == "hip:0"
    with pytest.raises(AssertionError, match="Subgroup size must be const or literal"):
        kernel(work_shape=4, subgroup_size=sym.S)
