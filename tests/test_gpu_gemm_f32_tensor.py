"""The float32 GEMM on the tensor cores (hcGemmF32Tensor: three tf32 products
per float32 product, fp32 accumulation in TMEM) through the C-ABI and through
the front door.

Tolerance: the parity bound of the float32 dot kernels, |got - exact| <=
1e-5 * sum|a||b| against the float64 product; and, up to K = 1024, the tighter
2e-6 * sum|a||b| that a single tf32 product (about 5e-4 * sum|a||b|) could not
meet - to show that the operand split does its job.  (Beyond that the float32
accumulation itself, whose error grows with the square root of K, takes over.)"""

import numpy as np
import pytest
import torch

from hc_b200 import capi
from oracle import workloads as oracle
from tests.gpu_util import dev, empty_like_dev, finish

pytestmark = pytest.mark.gpu


def _workspace(hc, m, n, k):
    need = hc.lib.hcGemmF32TensorWorkspaceBytes(m, n, k)
    buf = torch.empty(need + 1024, dtype=torch.uint8, device="cuda")
    offset = (-buf.data_ptr()) % 1024
    return buf, buf.data_ptr() + offset, need


# gemm_variant: 1 = one CTA per 128 x 256 tile, 2 = a CTA pair per 256 x 256 tile
# (tcgen05 cta_group::2), 0 = the library's choice (the pair from two row blocks on).
@pytest.mark.parametrize("variant", [0, 1, 2])
@pytest.mark.parametrize("m,n,k", [(128, 256, 32), (256, 512, 64), (300, 500, 100), (1, 1, 1),
                                   (129, 257, 33), (1024, 1024, 1024), (70, 45, 333),
                                   (2048 + 256, 4096 + 8, 520)])
def test_matches_float64_product(hc, m, n, k, variant):
    hc.set_option("gemm_variant", variant)
    try:
        _matches_float64_product(hc, m, n, k)
    finally:
        hc.set_option("gemm_variant", 0)


def _matches_float64_product(hc, m, n, k):
    rng = np.random.default_rng(m * 7 + n * 3 + k)
    a = rng.uniform(-1, 1, (m, k)).astype(np.float32)
    b = rng.uniform(-1, 1, (k, n)).astype(np.float32)
    keep, ws, need = _workspace(hc, m, n, k)
    d_a, d_b, d_c = dev(a), dev(b), empty_like_dev((m, n), torch.float32)
    hc.gemm_f32_tensor(d_a.data_ptr(), d_b.data_ptr(), d_c.data_ptr(), ws, need, m, n, k, k, n, n)
    finish(hc)
    got = d_c.cpu().numpy().astype(np.float64)
    exact = a.astype(np.float64) @ b.astype(np.float64)
    scale = np.abs(a).astype(np.float64) @ np.abs(b).astype(np.float64)
    assert not np.isnan(got).any()
    assert np.all(np.abs(got - exact) <= 1e-5 * scale + 1e-30)
    assert np.all(np.abs(got - exact) <= 2e-6 * scale + 1e-30)
    del keep


def test_pitched_operands_and_untouched_padding(hc):
    m, n, k = 200, 300, 150
    rng = np.random.default_rng(9)
    a_store = rng.standard_normal((m, k + 5)).astype(np.float32)
    b_store = rng.standard_normal((k, n + 3)).astype(np.float32)
    keep, ws, need = _workspace(hc, m, n, k)
    d_a, d_b = dev(a_store), dev(b_store)
    d_c = empty_like_dev((m, n + 7), torch.float32)
    hc.gemm_f32_tensor(d_a.data_ptr(), d_b.data_ptr(), d_c.data_ptr(), ws, need, m, n, k, k + 5,
                       n + 3, n + 7)
    finish(hc)
    got = d_c.cpu().numpy()
    assert np.isnan(got[:, n:]).all()  # the padding of C stays untouched
    a, b = a_store[:, :k].astype(np.float64), b_store[:, :n].astype(np.float64)
    assert np.all(np.abs(got[:, :n] - a @ b) <= 2e-6 * (np.abs(a) @ np.abs(b)))
    del keep


def test_agrees_with_the_cuda_core_kernel_and_the_oracle(hc):
    """Both float32 kernels against the oracle's K-blocked dot on the same inputs."""
    m, n, k = 384, 512, 256
    a, b = oracle.make_inputs("gemm_f32", shape=(m, n, k))
    keep, ws, need = _workspace(hc, m, n, k)
    d_a, d_b = dev(a), dev(b)
    d_t, d_s = empty_like_dev((m, n), torch.float32), empty_like_dev((m, n), torch.float32)
    hc.gemm_f32_tensor(d_a.data_ptr(), d_b.data_ptr(), d_t.data_ptr(), ws, need, m, n, k, k, n, n)
    hc.gemm_tiled(d_a.data_ptr(), d_b.data_ptr(), d_s.data_ptr(), m, n, k, k, n, n)
    finish(hc)
    expect = np.zeros((m, n), np.float32)
    oracle.gemm_kblocked(a, b, expect, (64, 64), kb=16)
    bound = 1e-5 * (np.abs(a).astype(np.float64) @ np.abs(b).astype(np.float64))
    for got in (d_t.cpu().numpy(), d_s.cpu().numpy()):
        assert np.all(np.abs(got.astype(np.float64) - expect) <= 2 * bound)
    del keep


def test_refusals(hc):
    m = n = k = 256
    keep, ws, need = _workspace(hc, m, n, k)
    x = torch.zeros(m * k, device="cuda")
    with pytest.raises(capi.HcError, match="workspace of"):
        hc.gemm_f32_tensor(x.data_ptr(), x.data_ptr(), x.data_ptr(), ws, need - 1, m, n, k, k, n, n)
    with pytest.raises(capi.HcError, match="workspace of"):
        hc.gemm_f32_tensor(x.data_ptr(), x.data_ptr(), x.data_ptr(), ws + 4, need, m, n, k, k, n, n)
    with pytest.raises(capi.HcError, match="invalid shape"):
        hc.gemm_f32_tensor(x.data_ptr(), x.data_ptr(), x.data_ptr(), ws, need, m, n, k, k - 1, n, n)
    assert hc.lib.hcGemmF32TensorWorkspaceBytes(0, 5, 5) == 0
    del keep


def test_front_door_sends_large_float32_products_to_the_tensor_cores():
    from hc_b200.hckernel.kernel import get_context
    from hc_b200.workloads import make_kernels

    m = n = k = 2048
    a, b = oracle.make_inputs("gemm_f32", shape=(m, n, k))
    d_a, d_b = torch.from_numpy(a).cuda(), torch.from_numpy(b).cuda()
    d_c = torch.full((m, n), float("nan"), device="cuda")
    kernels = make_kernels("cuda:0")
    ctx = get_context("cuda:0")
    before = ctx.launch_count
    kernels.dot_fullk(d_a, d_b, d_c, (256, 256))
    torch.cuda.synchronize()
    assert ctx.launch_count - before == 3  # two operand splits and the product
    assert ctx.kernel_status() == 0
    rows = np.r_[0:64, 1000:1064, m - 64:m]
    got = d_c[torch.from_numpy(rows).cuda()].cpu().numpy().astype(np.float64)
    exact = a[rows].astype(np.float64) @ b.astype(np.float64)
    scale = np.abs(a[rows]).astype(np.float64) @ np.abs(b).astype(np.float64)
    # The accumulator in TMEM rounds like a float32 sum, so the error grows with
    # the square root of K; at K = 2048 it is still well inside the parity bound.
    assert np.all(np.abs(got - exact) <= 1e-5 * scale)
    assert np.abs(got - exact).max() <= 5e-6 * scale.max()
    assert not torch.isnan(d_c).any()
