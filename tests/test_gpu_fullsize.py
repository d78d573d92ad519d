"""Full-size parity: the five benchmark configurations at their real shapes
(and the convolution at the shape bench.py measures it on).

The CPU oracle cannot redo 10^12 flops in a test, so each configuration is
checked (a) against the oracle on a sample of rows, computed from the same
seeded inputs, and (b) through properties that do not depend on size:

* softmax: rows sum to one, order of elements preserved, values in [0, 1];
* reductions: max is bit-exact against the oracle on every row; the sum of
  2x is exactly twice the sum of x (scaling by a power of two is exact, so
  the reduction order must be the same in both runs);
* GEMMs: scaling B by two scales the bf16 result by exactly two; computing a
  row block (M-shard) or a column block (N-shard) alone gives bit-identical
  values to the same block of the full result - which is what makes the
  multi-GPU launcher's sharded output equal to the single-GPU output.
"""

import os

import numpy as np
import pytest
import torch

from oracle import workloads as oracle
from tests.gpu_util import dev, dev_bf16, empty_like_dev, finish, host_bf16

pytestmark = pytest.mark.gpu


def test_config1_fp32_gemm_256(hc, golden):
    a, b = oracle.make_inputs("gemm_f32")
    d_a, d_b, d_c = dev(a), dev(b), empty_like_dev((256, 256), torch.float32)
    hc.gemm_tiled(d_a.data_ptr(), d_b.data_ptr(), d_c.data_ptr(), 256, 256, 256, 256, 256, 256)
    finish(hc)
    got = d_c.cpu().numpy().astype(np.float64)
    bound = 1e-5 * (np.abs(a).astype(np.float64) @ np.abs(b).astype(np.float64))
    assert np.all(np.abs(got - golden["cfg1_gemm_f32_256"]) <= bound)
    # Relative form of the same statement: well inside 1e-5 of the result scale.
    assert np.abs(got - golden["cfg1_gemm_f32_256"]).max() <= 1e-5 * np.abs(got).max()


def test_config2_softmax_32768x4096(hc):
    m, n = 32768, 4096
    (x,) = oracle.make_inputs("softmax")
    d_x, d_y = dev(x), empty_like_dev((m, n), torch.float32)
    hc.softmax_rows(d_x.data_ptr(), d_y.data_ptr(), m, n, n, n)
    finish(hc)
    sums = d_y.sum(dim=1, dtype=torch.float64)
    assert torch.all((sums - 1).abs() < 1e-5)
    assert float(d_y.min()) >= 0.0 and float(d_y.max()) <= 1.0
    assert torch.equal(d_y.argmax(dim=1), d_x.argmax(dim=1))
    # Every one of the 32768 rows against the oracle (groups of 256 rows spread
    # over the host threads; the tiling is the oracle's own).
    expect = np.empty((m, n), np.float32)
    oracle.run_row_groups_parallel(
        lambda r0, r1: oracle.softmax_rows(x[r0:r1], expect[r0:r1], 256), m, 256,
        len(os.sched_getaffinity(0)))
    got = d_y.cpu().numpy()
    for r0 in range(0, m, 4096):  # in blocks, to keep the temporaries small
        e, g = expect[r0:r0 + 4096], got[r0:r0 + 4096]
        assert np.all(np.abs(g - e) <= 1e-6 + 1e-5 * np.abs(e))


def test_config3_row_sum_and_max_65536x8192(hc):
    m, n = 65536, 8192
    (x,) = oracle.make_inputs("reduce")
    d_x = dev(x)
    d_s, d_m = empty_like_dev((m,), torch.float32), empty_like_dev((m,), torch.float32)
    hc.reduce_rows(d_x.data_ptr(), d_s.data_ptr(), d_m.data_ptr(), m, n, n)
    finish(hc)
    got_s, got_m = d_s.cpu().numpy(), d_m.cpu().numpy()
    assert np.array_equal(got_m, x.max(axis=1))  # bit-exact on every row
    # Every one of the 65536 row sums against the float64 sum of the row.
    for r0 in range(0, m, 4096):
        block = x[r0:r0 + 4096].astype(np.float64)
        exact, bound = block.sum(axis=1), 1e-5 * np.abs(block).sum(axis=1)
        assert np.all(np.abs(got_s[r0:r0 + 4096] - exact) <= bound)
    # And the oracle's own sums (float32, NumPy's pairwise order) within the same bound.
    rows = np.r_[0:1024, 40000:41024, m - 1024:m]
    so, mo = np.zeros(len(rows), np.float32), np.zeros(len(rows), np.float32)
    oracle.reduce_rows(x[rows], so, mo, 256)
    bound = 1e-5 * np.abs(x[rows]).astype(np.float64).sum(axis=1)
    assert np.all(np.abs(got_s[rows].astype(np.float64) - so) <= 2 * bound)
    assert np.array_equal(got_m[rows], mo)
    d_x.mul_(2.0)
    d_s2 = empty_like_dev((m,), torch.float32)
    hc.reduce_rows(d_x.data_ptr(), d_s2.data_ptr(), 0, m, n, n)
    finish(hc)
    assert np.array_equal(d_s2.cpu().numpy(), 2.0 * got_s)


def _bf16_close(got, expect, mag):
    return np.all(np.abs(got - expect) <= 1e-2 * np.abs(expect) + 1e-4 * mag)


def test_config4_bf16_gemm_8192(hc):
    m = n = k = 8192
    a, b = oracle.make_inputs("gemm_bf16")
    d_a, d_b = dev_bf16(a), dev_bf16(b)
    d_c = empty_like_dev((m, n), torch.bfloat16)
    hc.gemm_bf16(d_a.data_ptr(), d_b.data_ptr(), d_c.data_ptr(), m, n, k, k, n, n)
    finish(hc)
    # 1280 rows (five whole 256-row groups spread over the matrix, so every row
    # position inside a tile is covered) against the oracle's full-K GEMM.
    rows = np.r_[0:256, 1792:2048, 4000:4256, 6100:6356, m - 256:m]
    expect = np.zeros((len(rows), n), np.float32)
    oracle.gemm_bf16(a[rows], b, expect, (256, 256))
    got = host_bf16(d_c[torch.from_numpy(rows).cuda()])
    assert _bf16_close(got, expect, np.abs(a[rows]) @ np.abs(b))

    # M-shard: rows [2048, 4096) computed alone equal the same rows of the full result.
    d_part = empty_like_dev((2048, n), torch.bfloat16)
    hc.gemm_bf16(d_a[2048:].data_ptr(), d_b.data_ptr(), d_part.data_ptr(), 2048, n, k, k, n, n)
    finish(hc)
    assert torch.equal(d_part.view(torch.int16), d_c[2048:4096].view(torch.int16))

    # Scaling B by two scales the result by exactly two.
    d_b.mul_(2.0)
    d_c2 = empty_like_dev((m, n), torch.bfloat16)
    hc.gemm_bf16(d_a.data_ptr(), d_b.data_ptr(), d_c2.data_ptr(), m, n, k, k, n, n)
    finish(hc)
    assert torch.equal(d_c2.float(), 2.0 * d_c.float())


def test_config5_w8a16_4096x8192x8192(hc):
    m, n, k = 4096, 8192, 8192
    a, w, s = oracle.make_inputs("gemm_w8a16")
    d_a, d_w, d_s = dev_bf16(a), dev(w), dev(s)
    d_c = empty_like_dev((m, n), torch.bfloat16)
    ws_bytes = hc.gemm_w8a16_workspace_bytes(n, k)
    ws = torch.empty(ws_bytes, dtype=torch.uint8, device="cuda")
    torch.cuda.synchronize()
    hc.gemm_w8a16(d_a.data_ptr(), d_w.data_ptr(), d_s.data_ptr(), d_c.data_ptr(), ws.data_ptr(),
                  ws_bytes, m, n, k, k, n, n)
    finish(hc)
    # 768 rows (three whole 256-row groups) against the oracle.
    rows = np.r_[0:256, 2000:2256, m - 256:m]
    expect = np.zeros((len(rows), n), np.float32)
    oracle.gemm_w8a16(a[rows], w, s, expect, (256, 256))
    got = host_bf16(d_c[torch.from_numpy(rows).cuda()])
    assert _bf16_close(got, expect, np.abs(a[rows]) @ (np.abs(w.astype(np.float32)) * s))

    # N-shard: columns [1024, 2048) computed alone (as one rank of eight would).
    d_part = empty_like_dev((m, n), torch.bfloat16)
    hc.gemm_w8a16(d_a.data_ptr(), d_w[:, 1024:].data_ptr(), d_s[1024:].data_ptr(),
                  d_part[:, 1024:].data_ptr(), ws.data_ptr(), ws_bytes, m, 1024, k, k, n, n)
    finish(hc)
    assert torch.equal(d_part[:, 1024:2048].contiguous().view(torch.int16),
                       d_c[:, 1024:2048].contiguous().view(torch.int16))


def test_conv_benchmark_shape_properties():
    """The implicit-GEMM convolution at the shape bench.py measures (a 3x3 layer,
    32 x 64 x 56 x 56 images, 64 filters): against the oracle on a sample of
    output positions, against float64 sums of the same products, and through
    properties that hold at any size - the result scales exactly with a power
    of two, and an image alone gives bit for bit what it gives inside the batch
    (tiles of other images never leak into it)."""
    from hc_b200.hckernel.kernel import sym
    from hc_b200.workloads import make_conv

    x_shape, f_shape, stride = (32, 64, 56, 56), (64, 64, 3, 3), 1
    x, f = oracle.make_conv_inputs(x_shape, f_shape, "float32", seed=21)
    conv = make_conv(stride).parametrize({sym.TN: 32, sym.TNF: 64, sym.KB: 16})
    d_x, d_f = torch.from_numpy(x).cuda(), torch.from_numpy(f).cuda()
    out_shape = oracle.conv_out_shape(x_shape, f_shape, stride)
    d_out = torch.full(out_shape, float("nan"), device="cuda")
    conv(d_x, d_f, d_out)
    torch.cuda.synchronize()
    assert not torch.isnan(d_out).any()  # every output element was written

    # Sampled positions against exact float64 sums of the same products.
    got = d_out.cpu().numpy()
    rng = np.random.default_rng(0)
    for _ in range(64):
        n, q = rng.integers(0, 32), rng.integers(0, 64)
        i, j = rng.integers(0, out_shape[2]), rng.integers(0, out_shape[3])
        patch = x[n, :, i:i + 3, j:j + 3].astype(np.float64)
        terms = patch * f[q].astype(np.float64)
        assert abs(got[n, q, i, j] - terms.sum()) <= 1e-5 * np.abs(terms).sum()

    # The oracle on a corner of the problem small enough for it: 2 images, 8
    # filters, a 6x6 window of the image (4x4 output positions).
    sub_x, sub_f = np.ascontiguousarray(x[:2, :, :6, :6]), np.ascontiguousarray(f[:8])
    expect = np.zeros((2, 8, 4, 4), np.float32)
    oracle.conv_implicit_gemm(sub_x, sub_f, expect, stride, 2, 8, 16)
    np.testing.assert_allclose(got[:2, :8, :4, :4], expect, rtol=1e-4, atol=1e-4)

    # Scaling the filters by two scales every output by exactly two.
    d_twice = torch.empty_like(d_out)
    conv(d_x, d_f * 2, d_twice)
    torch.cuda.synchronize()
    assert torch.equal(d_twice, d_out * 2)

    # One image alone (ragged tile: 1 of 32 rows real) equals its slice of the batch.
    d_one = torch.empty((1,) + out_shape[1:], device="cuda")
    conv(d_x[5:6].contiguous(), d_f, d_one)
    torch.cuda.synchronize()
    assert torch.equal(d_one[0], d_out[5])
