"""The dequant GEMM that converts the int8 weights inside its pipeline
(hc_gemm_w8a16_umma_pair, option ``w8a16_variant`` 2) against the one that
converts them in a pass of its own (``w8a16_variant`` 1): the same products in
the same order, so the outputs must be equal bit for bit; and both against the
oracle's restatement of the DSL body within the bf16 tolerance (relative 1e-2
plus 1e-4 * sum|a||w|s)."""

import numpy as np
import pytest
import torch

from oracle import workloads as oracle
from tests.gpu_util import dev, dev_bf16, empty_like_dev, finish, host_bf16

pytestmark = pytest.mark.gpu


def _run(hc, d_a, d_w, d_s, m, n, k, lda, ldw, variant, workspace=True):
    d_c = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device="cuda")
    ws_bytes = hc.gemm_w8a16_workspace_bytes(n, k) if workspace else 0
    ws = torch.empty(max(1, ws_bytes), dtype=torch.uint8, device="cuda")
    torch.cuda.synchronize()
    hc.set_option("w8a16_variant", variant)
    try:
        for _ in range(2):
            hc.gemm_w8a16(d_a.data_ptr(), d_w.data_ptr(), d_s.data_ptr(), d_c.data_ptr(),
                          ws.data_ptr() if workspace else 0, ws_bytes, m, n, k, lda, ldw, n)
    finally:
        hc.set_option("w8a16_variant", 0)
    finish(hc)
    return host_bf16(d_c)


@pytest.mark.parametrize("shape", [(256, 256, 64), (256, 512, 512), (384, 256, 192),
                                   (1000, 784, 520), (129, 48, 72), (2048, 2048, 1024),
                                   (4096, 8192, 256)])
def test_fused_equals_the_two_pass_form_bit_for_bit(hc, shape):
    m, n, k = shape
    a, w, s = oracle.make_inputs("gemm_w8a16", shape=shape)
    d_a, d_w, d_s = dev_bf16(a), dev(w), dev(s)
    fused = _run(hc, d_a, d_w, d_s, m, n, k, k, n, 2, workspace=False)  # needs no scratch
    two_pass = _run(hc, d_a, d_w, d_s, m, n, k, k, n, 1)
    assert not np.isnan(fused).any()
    assert np.array_equal(fused, two_pass)
    if m * n * k <= 1 << 28:
        expect = np.zeros((m, n), np.float32)
        oracle.gemm_w8a16(a, w, s, expect, (256, 256))
        mag = np.abs(a) @ (np.abs(w.astype(np.float32)) * s)
        assert np.all(np.abs(fused - expect) <= 1e-2 * np.abs(expect) + 1e-4 * mag)


def test_pitched_operands(hc):
    m, n, k = 300, 400, 200
    a, w, s = oracle.make_inputs("gemm_w8a16", shape=(m, n, k))
    a_store = np.zeros((m, k + 8), np.float32)
    a_store[:, :k] = a
    w_store = np.full((k, n + 16), 77, np.int8)
    w_store[:, :n] = w
    d_a, d_w, d_s = dev_bf16(a_store), dev(w_store), dev(s)
    fused = _run(hc, d_a, d_w, d_s, m, n, k, k + 8, n + 16, 2, workspace=False)
    two_pass = _run(hc, d_a, d_w, d_s, m, n, k, k + 8, n + 16, 1)
    assert np.array_equal(fused, two_pass)


def test_layouts_it_does_not_take(hc):
    """A weight pitch that TMA cannot describe runs the two-pass form by default and
    is refused when the fused form is demanded; so is a single row block."""
    m, n, k = 256, 264, 128  # ldw = 264 is not a multiple of 16
    a, w, s = oracle.make_inputs("gemm_w8a16", shape=(m, n, k))
    d_a, d_w, d_s = dev_bf16(a), dev(w), dev(s)
    auto = _run(hc, d_a, d_w, d_s, m, n, k, k, n, 0)
    expect = np.zeros((m, n), np.float32)
    oracle.gemm_w8a16(a, w, s, expect, (256, 256))
    mag = np.abs(a) @ (np.abs(w.astype(np.float32)) * s)
    assert np.all(np.abs(auto - expect) <= 1e-2 * np.abs(expect) + 1e-4 * mag)
    with pytest.raises(RuntimeError, match="does not allow converting in the pipeline"):
        _run(hc, d_a, d_w, d_s, m, n, k, k, n, 2)
    a1, w1, s1 = oracle.make_inputs("gemm_w8a16", shape=(128, 256, 128))
    with pytest.raises(RuntimeError, match="does not allow converting in the pipeline"):
        _run(hc, dev_bf16(a1), dev(w1), dev(s1), 128, 256, 128, 128, 256, 2)
