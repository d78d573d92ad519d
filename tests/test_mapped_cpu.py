"""Host side of the mapped (gather/scatter) kernels on CPU: the reference's
implicit-GEMM convolution body (python/hckernel/tests/test_examples.py:203-252)
is recorded, its mappings and tile origins are evaluated into the index tables
the GPU kernel reads, and those tables - applied with the kernel's formula in
NumPy - must reproduce the outputs of the reference simulator stored under
tests/golden.  No kernel is launched."""

import numpy as np
import pytest
import sympy

from hc_b200.hckernel.kernel import *  # noqa: F401,F403
from hc_b200.hckernel.kernel import UnsupportedKernel
from hc_b200.hckernel.kernel_api import Affine, IndexExpr
from hc_b200.workloads import make_conv
from oracle import workloads as oracle

DT = typename.DT
TARGET = dict(backend="nvvm", device="cuda:0")


class FakeTensor:
    def __init__(self, shape, dtype="float64"):
        self.shape, self.dtype = tuple(shape), dtype


F = FakeTensor


def apply_tables(spec, x, f, out):
    """What csrc/kernels/mapped_gemm.cu computes, from the same tables."""
    tables = spec.host_tables()

    def locate(arr, role, g):
        mp, org = tables[role]
        rel = mp[:, :arr.ndim]
        index = org[g][None, :arr.ndim] + rel
        inside = np.all((rel >= 0) & (index < np.array(arr.shape)), axis=1)
        return index, inside

    def gather(arr, role, g, shape):
        index, inside = locate(arr, role, g)
        values = np.zeros(index.shape[0], arr.dtype)
        values[inside] = arr[tuple(index[inside].T)]
        return values.reshape(shape)

    for g in range(spec.groups):
        product = gather(x, "x", g, (spec.tm, spec.k)) @ gather(f, "f", g, (spec.k, spec.tn))
        index, inside = locate(out, "out", g)
        out[tuple(index[inside].T)] = product.reshape(-1)[inside]


@pytest.mark.parametrize("case", oracle.conv_golden_cases(), ids=lambda c: c[0])
def test_conv_tables_reproduce_the_reference(golden, case):
    name, x_shape, f_shape, stride, dtype, (tn, tnf, kb) = case
    x, f = oracle.make_conv_inputs(x_shape, f_shape, dtype)
    out_shape = oracle.conv_out_shape(x_shape, f_shape, stride)
    conv = make_conv(stride).parametrize({sym.TN: tn, sym.TNF: tnf, sym.KB: kb})
    plan = conv.plan_for((F(x_shape, dtype), F(f_shape, dtype), F(out_shape, dtype)))
    assert plan.family == "mapped_gemm"
    assert (plan.roles["x"], plan.roles["f"], plan.roles["out"]) == (0, 1, 2)
    spec = plan.roles["spec"]
    assert (spec.tm, spec.tn, spec.k) == (tn, tnf, x_shape[1] * f_shape[2] * f_shape[3])
    out = np.zeros(out_shape, dtype)
    apply_tables(spec, x, f, out)
    # One dot over all of K instead of the reference's K blocks: equal up to
    # summation order.
    tol = dict(rtol=1e-5, atol=1e-5) if dtype == "float32" else dict(rtol=1e-12, atol=1e-12)
    np.testing.assert_allclose(out, golden[name], **tol)


def test_fractional_output_extent_truncates_like_the_reference():
    # stride 3 on a 4x4 image with a 2x2 filter: H_OUT = W_OUT = 5/3, the work
    # shape int(25/9) = 2 (kernel_sim.py:121-127); position 1 maps to (i, j) =
    # (1, 0), whose store falls outside the 1x1 output.
    conv = make_conv(3)
    spec = conv.plan_for((F((2, 1, 4, 4)), F((1, 1, 2, 2)), F((2, 1, 1, 1)))).roles["spec"]
    assert spec.counts == (1, 1, 2)
    _, x_origins = spec.host_tables()["x"]
    assert x_origins.tolist() == [[0, 0, 0, 0], [0, 0, 3, 0]]
    _, out_origins = spec.host_tables()["out"]
    assert out_origins.tolist() == [[0, 0, 0, 0], [0, 0, 1, 0]]


def test_table_order_follows_memory_order():
    """Consecutive threads take consecutive table entries, so an operand tile is
    stored transposed when its columns are what lies together in memory: the
    filter tile [K, TNF] of the convolution is contiguous along K."""
    import torch

    x, f, out = torch.zeros(4, 3, 8, 8), torch.zeros(16, 3, 3, 3), torch.zeros(4, 16, 6, 6)
    spec = make_conv(1).plan_for((x, f, out)).roles["spec"]
    tx, tf, to = spec.device_tables((x, f, out))
    assert (tx[5], tf[5], to[5]) == (False, True, False)
    # 1 x 2 x 36 work-groups: the 36 positions of one filter block share their f
    # tile; aligned runs of 8 would straddle the two blocks, runs of 4 do not.
    assert spec.counts == (1, 2, 36) and (tx[6], tf[6], to[6]) == (1, 4, 1)
    natural_map, _ = spec.host_tables()["f"]
    k, tnf = spec.k, spec.tn
    assert np.array_equal(tf[0].numpy().reshape(tnf, k, 4),
                          natural_map.reshape(k, tnf, 4).transpose(1, 0, 2))
    # lin = map . strides, in the same order as map.
    stride = np.array(f.stride())
    assert np.array_equal(tf[1].numpy(), tf[0].numpy() @ stride)
    assert tf[3] == [0, 0, 0, 0] and tf[4] == [tnf - 1, 2, 2, 2]
    assert spec.device_tables((x, f, out)) is spec.device_tables((x, f, out))  # cached


def test_shared_runs_of_tile_origins():
    from hc_b200.hckernel.mapped import _shared_run

    same = np.zeros((20, 4), np.int64)
    assert _shared_run(same) == 8            # 20 = 2 runs of 8 + a tail of 4, all equal
    blocks = np.repeat(np.arange(5), 4)[:, None] * np.ones((1, 4), np.int64)
    assert _shared_run(blocks) == 4          # origins change every 4 groups
    assert _shared_run(blocks[:18]) == 4     # a short last run is fine
    assert _shared_run(blocks[2:]) == 2      # shifted by 2: aligned runs of 4 would mix blocks
    assert _shared_run(np.arange(12)[:, None] * np.ones((1, 4), np.int64)) == 1
    assert _shared_run(same[:1]) == 1


def test_autotune_grid_of_a_tunable():
    from hc_b200.hckernel.autotune import _spread_of

    assert _spread_of(TunableParam(sym.TN, 8, range(1, 64))) == [1, 2, 4, 8, 16, 32, 63]
    assert _spread_of(TunableParam(sym.KB, 16, range(8, 128))) == [8, 16, 32, 64, 127]
    assert _spread_of(TunableParam(sym.V, 3, [3, 5, 6])) == [3, 6]


def test_index_expressions():
    g = tuple(Affine(0, {d: 1}) for d in range(3))
    gids = np.indices((2, 3, 4)).reshape(3, -1)
    w = g[2] * 5 + g[1]
    assert isinstance(w, Affine)
    e = (w % 3) * 2 + w // 3 - g[0]
    assert isinstance(e, IndexExpr)
    want = ((gids[2] * 5 + gids[1]) % 3) * 2 + (gids[2] * 5 + gids[1]) // 3 - gids[0]
    assert np.array_equal(e.evaluate(gids), want)
    assert np.array_equal((g[0] * g[1]).evaluate(gids), gids[0] * gids[1])
    # Constants fold at once, fractions included: 7 % (5/3) = 1/3 is refused,
    # 5 % (5/3) = 0 and 5 // (5/3) = 3 are integers.
    five_thirds = sympy.Rational(5, 3)
    assert Affine(5) % five_thirds == 0 and Affine(5) // five_thirds == 3
    with pytest.raises(UnsupportedKernel, match="not an integer"):
        Affine(7) % five_thirds
    frac = g[2] % five_thirds
    assert np.array_equal(frac.evaluate((None, None, np.array([0, 1]))), [0, 1])
    with pytest.raises(UnsupportedKernel, match="not an integer for every work-group"):
        frac.evaluate((None, None, np.array([0, 1, 2])))
    with pytest.raises(UnsupportedKernel, match="no single value"):
        int(e)
    with pytest.raises(UnsupportedKernel, match="must be a constant"):
        g[0] % g[1]
    with pytest.raises(UnsupportedKernel, match="non-positive"):
        g[0] // 0


def _gather_kernel(x_map, out_map, origin=lambda m0: m0):
    M, K, N, GM = sym.M, sym.K, sym.N, sym.GM

    @kernel(work_shape=M, group_shape=GM, **TARGET)
    def k(gr: CurrentGroup, a: Buffer[M, K, DT], b: Buffer[K, N, DT], out: Buffer[M, N, DT],
          gshape: GM):
        m0 = gr.work_offset[0]
        a_t = gr.load(a[origin(m0):, :], shape=(gr.shape[0], K), mapping=x_map)
        b_t = gr.load(b, shape=(K, N))  # a plain load is a gather with the identity mapping
        gr.store(out[m0:, :], np.dot(a_t, b_t), mapping=out_map)

    return k


def test_plain_loads_mix_with_mapped_ones():
    rows = create_mapping(lambda i, j: (i, j))
    k = _gather_kernel(rows, rows)
    spec = k.plan_for((F((10, 6)), F((6, 5)), F((10, 5)), 4)).roles["spec"]
    assert (spec.tm, spec.tn, spec.k, spec.counts) == (4, 5, 6, (3,))
    rng = np.random.default_rng(0)
    a, b = rng.standard_normal((10, 6)), rng.standard_normal((6, 5))
    out = np.zeros((10, 5))
    apply_tables(spec, a, b, out)
    np.testing.assert_allclose(out, a @ b, rtol=1e-12)


def test_writes_that_collide_are_refused():
    rows = create_mapping(lambda i, j: (i, j))
    one_row = create_mapping(lambda i, j: (0, j))  # every tile row lands on row 0
    k = _gather_kernel(rows, one_row)
    with pytest.raises(UnsupportedKernel, match="write the same output"):
        k.plan_for((F((8, 6)), F((6, 5)), F((8, 5)), 4)).roles["spec"].host_tables()
    # Overlapping groups: tiles of 4 rows placed every 4 rows but shifted maps.
    shifted = create_mapping(lambda i, j: (i + 2, j))
    k = _gather_kernel(rows, shifted)
    spec = k.plan_for((F((8, 6)), F((6, 5)), F((8, 5)), 4)).roles["spec"]
    spec.host_tables()  # rows 2..5 and 6..7(+2 dropped): disjoint, accepted
    wide = create_mapping(lambda i, j: (i * 2, j))  # rows 0,2,4,6 and 4,6,8,10: collide
    k = _gather_kernel(rows, wide)
    with pytest.raises(UnsupportedKernel, match="write the same output"):
        k.plan_for((F((8, 6)), F((6, 5)), F((8, 5)), 4)).roles["spec"].host_tables()


def test_negative_origins_and_wrong_rank_are_refused():
    rows = create_mapping(lambda i, j: (i, j))
    k = _gather_kernel(rows, rows, origin=lambda m0: m0 - 1)
    with pytest.raises(UnsupportedKernel, match="negative"):
        k.plan_for((F((8, 6)), F((6, 5)), F((8, 5)), 4)).roles["spec"].host_tables()
    k = _gather_kernel(create_mapping(lambda i, j: (i, j, 0)), rows)
    with pytest.raises(UnsupportedKernel, match="returns 3 indices for an array of rank 2"):
        k.plan_for((F((8, 6)), F((6, 5)), F((8, 5)), 4)).roles["spec"].host_tables()


def test_mapping_that_branches_falls_back_to_per_element_calls():
    clamp = create_mapping(lambda i, j: (i if i < 2 else 1, j))  # `if` on an index grid fails
    rows = create_mapping(lambda i, j: (i, j))
    k = _gather_kernel(clamp, rows)
    spec = k.plan_for((F((4, 3)), F((3, 2)), F((4, 2)), 4)).roles["spec"]
    table, _ = spec.host_tables()["x"]
    assert table[:, 0].reshape(4, 3)[:, 0].tolist() == [0, 1, 1, 1]


def test_bodies_the_mapped_family_does_not_cover():
    M, K, N = sym.M, sym.K, sym.N
    rows = create_mapping(lambda i, j: (i, j))

    @kernel(work_shape=M, group_shape=4, **TARGET)
    def not_a_product(gr: CurrentGroup, a: Buffer[M, K, DT], out: Buffer[M, K, DT]):
        m0 = gr.work_offset[0]
        gr.store(out[m0:, :], gr.load(a[m0:, :], shape=(4, K), mapping=rows) * 2.0, mapping=rows)

    with pytest.raises(UnsupportedKernel, match="not a sum of np.dot products"):
        not_a_product.plan_for((F((8, 6)), F((8, 6))))

    @kernel(work_shape=M, group_shape=4, **TARGET)
    def gap_in_k(gr: CurrentGroup, a: Buffer[M, K, DT], b: Buffer[K, N, DT],
                 out: Buffer[M, N, DT]):
        m0 = gr.work_offset[0]
        a_t = gr.load(a[m0:, :], shape=(4, K), mapping=rows)
        b_t = gr.load(b, shape=(K, N), mapping=rows)
        acc = np.dot(gr.vload(a_t[:, 2:], shape=(4, 2)), gr.vload(b_t[2:, :], shape=(2, N)))
        gr.store(out[m0:, :], acc, mapping=rows)

    with pytest.raises(UnsupportedKernel, match="overlap or leave gaps"):
        gap_in_k.plan_for((F((8, 6)), F((6, 5)), F((8, 5))))
