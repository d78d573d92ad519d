"""Host-buffer entry points (hc_b200/host.py): row chunks streamed through the
GPU with upload, kernel and download overlapped must give exactly what one
launch on the whole matrix gives, for ragged chunking, pinned and pageable
host memory, and repeated calls that reuse the device slots."""

import numpy as np
import pytest
import torch

from hc_b200 import host as hc_host
from hc_b200.workloads import make_kernels
from oracle import workloads as oracle

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("pinned", [True, False])
@pytest.mark.parametrize("rows,cols,chunk", [(1000, 2048, 300), (64, 4096, 4096), (257, 100, 64)])
def test_softmax_rows_host_equals_single_launch(pinned, rows, cols, chunk):
    (x,) = oracle.make_inputs("softmax", shape=(rows, cols))
    hx = torch.from_numpy(x)
    hy = torch.full((rows, cols), float("nan"))
    if pinned:
        hx, hy = hx.pin_memory(), hy.pin_memory()
    for _ in range(2):  # the second call reuses the device slots
        hy.fill_(float("nan"))
        hc_host.softmax_rows_host(hx, hy, "cuda:0", chunk_rows=chunk, group_rows=32)
        hc_host.synchronize("cuda:0")
        k = make_kernels("cuda:0")
        d_x = hx.cuda()
        d_y = torch.empty_like(d_x)
        k.softmax(d_x, d_y, 32)
        assert torch.equal(hy, d_y.cpu())  # bit-identical to one launch
    expect = np.zeros_like(x)
    oracle.softmax_rows(x, expect, 32)
    assert np.all(np.abs(hy.numpy() - expect) <= 1e-6 + 1e-5 * np.abs(expect))


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_gemm_host_equals_single_launch(dtype):
    m, k, n = 600, 256, 384
    a, b = oracle.make_inputs("gemm_bf16", shape=(m, n, k))  # bf16-exact float32 values
    ha, hb = torch.from_numpy(a).to(dtype).pin_memory(), torch.from_numpy(b).to(dtype).pin_memory()
    hc_out = torch.zeros((m, n), dtype=dtype).pin_memory()
    kernels = make_kernels("cuda:0")
    d_out = torch.zeros((m, n), dtype=dtype, device="cuda")
    kernels.dot_fullk(ha.cuda(), hb.cuda(), d_out, (256, 256))
    for _ in range(2):  # the second call reuses the resident copy of b and the slots
        hc_out.zero_()
        hc_host.gemm_host(ha, hb, hc_out, "cuda:0", chunk_rows=250)
        hc_host.synchronize("cuda:0")
        if dtype == torch.bfloat16:
            assert torch.equal(hc_out, d_out.cpu())  # same tcgen05 kernel, same sum order
        else:
            # A row block has few tiles, so its K loop may be split over a cluster
            # where the whole matrix is not: equal up to summation order.
            assert torch.allclose(hc_out, d_out.cpu(), rtol=1e-5, atol=1e-6)
    expect = a.astype(np.float64) @ b.astype(np.float64)
    tol = 1e-2 if dtype == torch.bfloat16 else 1e-5
    assert np.all(np.abs(hc_out.double().numpy() - expect)
                  <= tol * (np.abs(a).astype(np.float64) @ np.abs(b).astype(np.float64)) + 1e-30)
    with pytest.raises(ValueError, match="expected a"):
        hc_host.gemm_host(ha, hb[:10], hc_out, "cuda:0")


def test_reduce_rows_host_matches_oracle():
    rows, cols = 3000, 1024
    (x,) = oracle.make_inputs("reduce", shape=(rows, cols))
    hx = torch.from_numpy(x).pin_memory()
    hs, hm = torch.empty(rows).pin_memory(), torch.empty(rows).pin_memory()
    hc_host.reduce_rows_host(hx, hs, hm, "cuda:0", chunk_rows=700)
    hc_host.synchronize("cuda:0")
    assert np.array_equal(hm.numpy(), x.max(axis=1))
    exact = x.astype(np.float64).sum(axis=1)
    assert np.all(np.abs(hs.numpy() - exact) <= 1e-5 * np.abs(x).astype(np.float64).sum(axis=1))
    with pytest.raises(ValueError, match="expected x"):
        hc_host.reduce_rows_host(hx, hs[:10], hm, "cuda:0")


def test_rows_body_host_equals_single_launch():
    """A row body (rows centred and scaled by their own statistics) and an
    element-wise body on host matrices, in ragged row chunks: bit for bit what one
    launch on the whole matrix gives."""
    from hc_b200.workloads import make_elementwise, make_rowwise

    rows, cols = 777, 2048
    a, b = oracle.make_elementwise_inputs(2, (rows, cols), "float32", seed=21)
    ha, hb = torch.from_numpy(a).pin_memory(), torch.from_numpy(b).pin_memory()
    hy = torch.full((rows, cols), float("nan")).pin_memory()
    body = make_rowwise(lambda t: (t - t.mean(axis=1, keepdims=True))
                        / np.sqrt((t * t).sum(axis=1, keepdims=True) + 1.0))
    hc_host.rows_body_host(body, [ha], hy, "cuda:0", chunk_rows=200, group_rows=64)
    hc_host.synchronize("cuda:0")
    d_y = torch.empty(rows, cols, device="cuda")
    body(ha.cuda(), d_y, 64)
    torch.cuda.synchronize()
    assert torch.equal(hy, d_y.cpu())
    a64 = a.astype(np.float64)
    want = (a64 - a64.mean(axis=1, keepdims=True)) / np.sqrt((a64 * a64).sum(axis=1, keepdims=True) + 1)
    np.testing.assert_allclose(hy.numpy(), want, rtol=1e-5, atol=1e-6)

    relu = make_elementwise(lambda s, t: np.maximum(s * 2.0 - t, 0.0), 2, 2, (4, 256))
    hy.fill_(float("nan"))
    hc_host.rows_body_host(relu, [ha, hb], hy, "cuda:0", chunk_rows=333, group_rows=None)
    hc_host.synchronize("cuda:0")
    assert np.array_equal(hy.numpy(), np.maximum(a * np.float32(2) - b, 0))
    with pytest.raises(ValueError, match="one shape and dtype"):
        hc_host.rows_body_host(relu, [ha, hb[:10]], hy, "cuda:0", group_rows=None)
