"""The host-buffer entry points of the C-ABI (hcSoftmaxRowsHost,
hcReduceRowsHost, hcGemmBf16Host, hcHostPin): called through ctypes with plain
NumPy arrays, as a foreign-language host would call them.  Row chunks streamed
through the GPU must give bit for bit what the device entry point gives on the
whole matrix - for page-locked and pageable memory, pitched host matrices,
matrices several chunks long, and repeated calls that reuse the device slots -
and agree with the CPU oracle within the tolerances of the device tests."""

import numpy as np
import pytest
import torch

from hc_b200 import capi
from oracle import workloads as oracle
from tests.gpu_util import dev, dev_bf16, empty_like_dev, finish, host_bf16

pytestmark = pytest.mark.gpu


def _addr(a):
    return a.ctypes.data


@pytest.mark.parametrize("pinned", [True, False], ids=["pinned", "pageable"])
@pytest.mark.parametrize("rows,cols,pitch", [(3000, 2048, 2048), (64, 4096, 4100), (257, 100, 100),
                                             (1, 7, 7)])
def test_softmax_rows_host(hc, pinned, rows, cols, pitch):
    (x,) = oracle.make_inputs("softmax", shape=(rows, cols))
    hx = np.zeros((rows, pitch), np.float32)
    hx[:, :cols] = x
    hy = np.full((rows, pitch), np.nan, np.float32)
    if pinned:
        hc.host_pin(_addr(hx), hx.nbytes)
        hc.host_pin(_addr(hy), hy.nbytes)
    try:
        d_x, d_y = dev(x), empty_like_dev((rows, cols), torch.float32)
        hc.softmax_rows(d_x.data_ptr(), d_y.data_ptr(), rows, cols, cols, cols)
        finish(hc)
        for _ in range(2):  # the second call reuses the device slots
            hy[:] = np.nan
            hc.softmax_rows_host(_addr(hx), _addr(hy), rows, cols, pitch, pitch)
            assert np.array_equal(hy[:, :cols], d_y.cpu().numpy())  # no sync needed: the call waited
            assert np.isnan(hy[:, cols:]).all()  # the padding of a pitched matrix stays untouched
    finally:
        if pinned:
            hc.host_unpin(_addr(hx))
            hc.host_unpin(_addr(hy))
    expect = np.zeros_like(x)
    oracle.softmax_rows(x, expect, 32)
    assert np.all(np.abs(hy[:, :cols] - expect) <= 1e-6 + 1e-5 * np.abs(expect))


def test_softmax_rows_host_many_chunks(hc):
    """40 MiB in, 40 MiB out: three chunks per direction, both slots reused."""
    rows, cols = 2560, 4096
    (x,) = oracle.make_inputs("softmax", shape=(rows, cols))
    hy = np.empty_like(x)
    hc.host_pin(_addr(x), x.nbytes)
    hc.host_pin(_addr(hy), hy.nbytes)
    try:
        hc.softmax_rows_host(_addr(x), _addr(hy), rows, cols, cols, cols)
    finally:
        hc.host_unpin(_addr(x))
        hc.host_unpin(_addr(hy))
    d_y = empty_like_dev((rows, cols), torch.float32)
    d_x = dev(x)  # kept alive until the kernel has run
    hc.softmax_rows(d_x.data_ptr(), d_y.data_ptr(), rows, cols, cols, cols)
    finish(hc)
    assert np.array_equal(hy, d_y.cpu().numpy())


def test_reduce_rows_host(hc):
    rows, cols = 5000, 2048  # 39 MiB: three chunks
    (x,) = oracle.make_inputs("reduce", shape=(rows, cols))
    hs, hm = np.full(rows, np.nan, np.float32), np.full(rows, np.nan, np.float32)
    hc.host_pin(_addr(x), x.nbytes)
    try:
        hc.reduce_rows_host(_addr(x), _addr(hs), _addr(hm), rows, cols, cols)
        assert np.array_equal(hm, x.max(axis=1))
        exact = x.astype(np.float64).sum(axis=1)
        assert np.all(np.abs(hs - exact) <= 1e-5 * np.abs(x).astype(np.float64).sum(axis=1))
        only_max = np.full(rows, np.nan, np.float32)
        hc.reduce_rows_host(_addr(x), 0, _addr(only_max), rows, cols, cols)
        assert np.array_equal(only_max, hm)
    finally:
        hc.host_unpin(_addr(x))
    d_s, d_m = empty_like_dev((rows,), torch.float32), empty_like_dev((rows,), torch.float32)
    d_x = dev(x)  # kept alive until the kernel has run
    hc.reduce_rows(d_x.data_ptr(), d_s.data_ptr(), d_m.data_ptr(), rows, cols, cols)
    finish(hc)
    # (A chunk may take the other reduction kernel than the whole matrix does: same
    # sums up to the order of the additions.)
    assert np.all(np.abs(hs - d_s.cpu().numpy())
                  <= 1e-6 * np.abs(x).astype(np.float64).sum(axis=1))
    assert np.array_equal(hm, d_m.cpu().numpy())


@pytest.mark.parametrize("m,n,k", [(600, 384, 256), (2500, 512, 4096), (100, 72, 40)])
def test_gemm_bf16_host(hc, m, n, k):
    a, b = oracle.make_inputs("gemm_bf16", shape=(m, n, k))  # float32 holding bf16 values
    ha = oracle.bf16_bits(a).copy()
    hb = oracle.bf16_bits(b).copy()
    hc_out = np.zeros((m, n), np.uint16)
    hc.host_pin(_addr(ha), ha.nbytes)
    try:
        for _ in range(2):
            hc_out[:] = 0
            hc.gemm_bf16_host(_addr(ha), _addr(hb), _addr(hc_out), m, n, k, k, n, n)
    finally:
        hc.host_unpin(_addr(ha))
    d_c = empty_like_dev((m, n), torch.bfloat16)
    d_a, d_b = dev_bf16(a), dev_bf16(b)  # kept alive until the kernel has run
    hc.gemm_bf16(d_a.data_ptr(), d_b.data_ptr(), d_c.data_ptr(), m, n, k, k, n, n)
    finish(hc)
    got = oracle.bf16_from_bits(hc_out)
    assert np.array_equal(got, host_bf16(d_c))  # row blocks of a product are independent
    expect = np.zeros((m, n), np.float32)
    oracle.gemm_bf16(a, b, expect, (256, 256))
    assert np.all(np.abs(got - expect) <= 1e-2 * np.abs(expect) + 1e-4 * (np.abs(a) @ np.abs(b)))


def test_host_entry_points_refuse_bad_arguments(hc):
    x = np.zeros((4, 8), np.float32)
    with pytest.raises(capi.HcError, match="invalid shape"):
        hc.softmax_rows_host(_addr(x), _addr(x), 4, 8, 4, 8)
    with pytest.raises(capi.HcError, match="null buffer"):
        hc.softmax_rows_host(0, _addr(x), 4, 8, 8, 8)
    with pytest.raises(capi.HcError, match="unsupported dtype"):
        hc.softmax_rows_host(_addr(x), _addr(x), 4, 8, 8, 8, capi.HC_BF16)
    with pytest.raises(capi.HcError, match="invalid shape"):
        hc.gemm_bf16_host(_addr(x), _addr(x), _addr(x), 4, 8, 8, 4, 8, 8)
    with pytest.raises(capi.HcError, match="hcHostPin"):
        hc.host_pin(0, 0)
    hc.softmax_rows_host(_addr(x), _addr(x), 0, 8, 8, 8)  # nothing to do
