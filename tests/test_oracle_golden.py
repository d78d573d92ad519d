"""The NumPy oracle against the outputs of the reference simulator
(tests/golden/reference_outputs.npz, written by tests/golden/make_golden.py).

Every comparison is bit-exact: the oracle restates the reference's tiling and
calls the same NumPy routines, so any difference means the restatement is
wrong.  These are the reference's own known-answer cases
(python/hckernel/tests/test_examples.py:31-165, 304-335) plus reduced-size
instances of the benchmark configurations.
"""

import numpy as np
import pytest

from oracle import hcsim
from oracle import workloads as oracle


def test_reference_dot_vectors(golden):
    m, n, k = 16, 32, 64
    a = 2 * np.arange(m * k).reshape(m, k) / (m * k)
    b = np.arange(n * k).reshape(k, n) / (n * k)
    out = np.zeros((m, n))
    oracle.gemm_kblocked(a, b, out, (8, 8), kb=16)
    assert np.array_equal(out, golden["kat_dot_kblocked_f64"])
    assert np.array_equal(out, np.dot(a, b))  # the assertion of the reference test
    out = np.zeros((m, n))
    oracle.gemm_fullk(a, b, out, (8, 8))
    assert np.array_equal(out, golden["kat_dot_fullk_f64"])


def test_reference_softmax_vector(golden):
    m, n = 30, 25
    a = 2 * np.arange(m * n).reshape(m, n) / (m * n)
    out = np.zeros((m, n))
    oracle.softmax_rows(a, out, 8)
    assert np.array_equal(out, golden["kat_softmax_f64"])


def test_reference_reduction_vector(golden):
    a = np.arange(0, 20)
    out = np.zeros(1)
    oracle.reduce_sum_all(a, out, 8, 2)
    assert np.array_equal(out, golden["kat_reduce_all"])
    assert out[0] == a.sum()


@pytest.mark.parametrize("shape", [(1, 27), (10, 20), (111, 813)])
def test_copy_vectors(golden, shape):
    src = np.arange(shape[0] * shape[1], dtype=np.int32).reshape(shape)
    out = np.zeros_like(src)
    oracle.copy2d(src, out, (4, 16))
    assert np.array_equal(out, golden[f"copy_{shape[0]}x{shape[1]}"])
    out = np.zeros_like(src)
    oracle.copy2d(src, out, (4, 16), unroll=4)
    assert np.array_equal(out, src)


def test_benchmark_configs_reduced(golden):
    a, b = oracle.make_inputs("gemm_f32")
    out = np.zeros((256, 256), np.float32)
    oracle.gemm_kblocked(a, b, out, (64, 64), kb=16)
    assert np.array_equal(out, golden["cfg1_gemm_f32_256"])

    a, b = oracle.make_inputs("gemm_f32", shape=(70, 45, 33))
    out = np.zeros((70, 45), np.float32)
    oracle.gemm_kblocked(a, b, out, (64, 64), kb=16)
    assert np.array_equal(out, golden["cfg1_gemm_f32_70x45x33"])

    for shape, rows in (((48, 4096), 32), ((30, 25), 8)):
        (x,) = oracle.make_inputs("softmax", shape=shape)
        out = np.zeros_like(x)
        oracle.softmax_rows(x, out, rows)
        assert np.array_equal(out, golden[f"cfg2_softmax_{shape[0]}x{shape[1]}"])

    for shape, rows in (((300, 8192), 256), ((37, 101), 16)):
        (x,) = oracle.make_inputs("reduce", shape=shape)
        s, m = np.zeros(shape[0], np.float32), np.zeros(shape[0], np.float32)
        oracle.reduce_rows(x, s, m, rows)
        assert np.array_equal(s, golden[f"cfg3_sum_{shape[0]}x{shape[1]}"])
        assert np.array_equal(m, golden[f"cfg3_max_{shape[0]}x{shape[1]}"])

    a, b = oracle.make_inputs("gemm_bf16", shape=(256, 512, 384))
    out = np.zeros((256, 512), np.float32)
    oracle.gemm_bf16(a, b, out, (256, 256))
    assert np.array_equal(oracle.bf16_bits(out), golden["cfg4_gemm_bf16_256x512x384_bits"])

    a, w, s = oracle.make_inputs("gemm_w8a16", shape=(128, 256, 512))
    out = np.zeros((128, 256), np.float32)
    oracle.gemm_w8a16(a, w, s, out, (128, 128))
    assert np.array_equal(oracle.bf16_bits(out), golden["cfg5_gemm_w8a16_128x256x512_bits"])


def test_pairwise_distance_vectors(golden):
    # python/hckernel/tests/test_examples.py:291-301
    m, n, d = 16, 32, 8
    a = 2 * np.arange(m * d).reshape(m, d) / (m * d)
    b = np.arange(n * d).reshape(n, d) / (n * d)
    out = np.zeros((m, n))
    oracle.pairwise_distance(a, b, out, (8, 8))
    assert np.array_equal(out, golden["kat_pairwise_f64"])
    assert np.array_equal(out, np.linalg.norm(a[:, None, :] - b[None, :, :], axis=2))
    rng = np.random.default_rng(5)
    a = rng.standard_normal((70, 19)).astype(np.float32)
    b = rng.standard_normal((45, 19)).astype(np.float32)
    out = np.zeros((70, 45), np.float32)
    oracle.pairwise_distance(a, b, out, (16, 8))
    assert np.array_equal(out, golden["pairwise_f32_70x45x19"])


@pytest.mark.parametrize("case", oracle.conv_golden_cases(), ids=lambda c: c[0])
def test_conv_implicit_gemm_vectors(golden, case):
    """Gathers and scatters through index mappings
    (python/hckernel/tests/test_examples.py:168-258), bit for bit."""
    name, x_shape, f_shape, stride, dtype, (tn, tnf, kb) = case
    x, f = oracle.make_conv_inputs(x_shape, f_shape, dtype)
    out = np.zeros(oracle.conv_out_shape(x_shape, f_shape, stride), dtype)
    oracle.conv_implicit_gemm(x, f, out, stride, tn, tnf, kb)
    assert np.array_equal(out, golden[name])
    square = x_shape[2] == x_shape[3] and f_shape[2] == f_shape[3]
    if square and (x_shape[2] - f_shape[2]) % stride == 0:
        # What the reference test asserts: the plain correlation.
        tol = dict(rtol=1e-4, atol=1e-5) if dtype == "float32" else dict(rtol=1e-10, atol=1e-12)
        np.testing.assert_allclose(out, oracle.conv_direct(x, f, stride), **tol)


def test_mapped_tiles_mask_and_scatter():
    """kernel_api.py:303-310, 319-336: out-of-range mapped indices leave zeros
    (load) or are dropped (store); invalid tile elements are not stored."""
    a = np.arange(12.0).reshape(3, 4)
    t = hcsim.load_tile_mapped(a[1:, 2:], (3, 3), lambda i, j: (j, i))  # transposed gather
    assert np.array_equal(t.data, [[6, 10, 0], [7, 11, 0], [0, 0, 0]])
    assert np.array_equal(t.valid, [[1, 1, 0], [1, 1, 0], [0, 0, 0]])
    dst = np.full((3, 4), -1.0)
    hcsim.store_tile_mapped(dst[1:, :], t, lambda i, j: (i, j + 1))
    assert np.array_equal(dst, [[-1, -1, -1, -1], [-1, 6, 10, -1], [-1, 7, 11, -1]])


def test_group_order_and_offsets():
    # python/hckernel/tests/test_kernel_sim.py:26-54 checks the same facts on
    # the simulator: row-major group order, offsets = id * group shape.
    got = list(hcsim.iter_groups((5, 7), (2, 4)))
    assert [g for g, _ in got] == [(0, 0), (0, 1), (1, 0), (1, 1), (2, 0), (2, 1)]
    assert [o for _, o in got] == [(0, 0), (0, 4), (2, 0), (2, 4), (4, 0), (4, 4)]
    assert list(hcsim.iter_groups(10, 4)) == [((0,), (0,)), ((1,), (4,)), ((2,), (8,))]


def test_edge_tiles_load_and_store():
    # Masked edge tiles, as in python/hckernel/tests/test_kernel_sim.py:57-104.
    a = np.arange(12).reshape(3, 4)
    t = hcsim.load_tile(a[2:, 2:], (2, 3))
    assert np.array_equal(t.data, [[10, 11, 0], [0, 0, 0]])
    assert np.array_equal(t.valid, [[True, True, False], [False, False, False]])
    dst = np.full((3, 4), -1)
    hcsim.store_tile(dst[2:, 2:], t)
    assert np.array_equal(dst, [[-1, -1, -1, -1], [-1, -1, -1, -1], [-1, -1, 10, 11]])
    dst = np.full((3, 4), -1)
    hcsim.store_tile(dst[1:, 3:], np.array([[5, 6], [7, 8], [9, 9]]))  # plain source, clipped
    assert np.array_equal(dst[:, 3], [-1, 5, 7])
    z = hcsim.alloc_tile((2, 2), np.float32, 3)
    assert z.valid.all() and (z.data == 3).all()


def test_bf16_rounding_helper():
    x = np.array([1.0, 1.00390625, 1.005859375, -2.5, 3.0e38, 1e-40, np.inf], np.float32)
    r = oracle.round_to_bf16(x)
    assert r[0] == 1.0
    assert r[1] == 1.0            # exactly half way between 1.0 and 1.0078125: ties to even
    assert r[2] == 1.0078125
    assert r[3] == -2.5
    assert np.isinf(r[6])
    assert np.array_equal(oracle.bf16_from_bits(oracle.bf16_bits(r)), r)
    assert np.isnan(oracle.round_to_bf16(np.array([np.nan], np.float32))[0])


def test_inputs_are_reproducible():
    a1, b1 = oracle.make_inputs("gemm_bf16", shape=(8, 16, 24))
    a2, b2 = oracle.make_inputs("gemm_bf16", shape=(8, 16, 24))
    assert np.array_equal(a1, a2) and np.array_equal(b1, b2)
    assert np.array_equal(oracle.round_to_bf16(a1), a1)  # already bf16-exact
    _, w, s = oracle.make_inputs("gemm_w8a16", shape=(4, 32, 16))
    assert w.dtype == np.int8 and w.min() >= -127 and s.min() >= 0.001 and s.max() <= 0.02


def test_parallel_row_driver_matches_serial():
    (x,) = oracle.make_inputs("softmax", shape=(100, 64))
    a, b = np.zeros_like(x), np.zeros_like(x)
    oracle.softmax_rows(x, a, 8)
    oracle.run_row_groups_parallel(lambda r0, r1: oracle.softmax_rows(x[r0:r1], b[r0:r1], 8),
                                   100, 8, 4)
    assert np.array_equal(a, b)
