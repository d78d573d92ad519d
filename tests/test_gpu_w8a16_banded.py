"""The dequant GEMM that converts the int8 weights inside the GEMM kernel, band
by band (hc_gemm_w8a16_umma_banded, option ``w8a16_variant`` 3: four warps per
CTA convert a band of 1024 columns into a ring of three bands while the tiles of
earlier bands run), against the form that converts them in a pass of its own
(``w8a16_variant`` 1): the same products in the same order, so the outputs must
be equal bit for bit; and the kernel status word stays 0 (no wait ran out)."""

import numpy as np
import pytest
import torch

from oracle import workloads as oracle
from tests.gpu_util import dev, dev_bf16, finish, host_bf16

pytestmark = pytest.mark.gpu


def _run(hc, d_a, d_w, d_s, m, n, k, lda, ldw, variant, ws_bytes=None):
    d_c = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device="cuda")
    if ws_bytes is None:
        ws_bytes = hc.gemm_w8a16_workspace_bytes(n, k)
    raw = torch.empty(ws_bytes + 1024, dtype=torch.uint8, device="cuda")
    ws = raw[(-raw.data_ptr()) % 1024:][:ws_bytes]
    # A NaN pattern in the scratch: a band read before it is converted would show.
    ws.fill_(0xff)
    torch.cuda.synchronize()
    hc.set_option("w8a16_variant", variant)
    try:
        for _ in range(2):
            hc.gemm_w8a16(d_a.data_ptr(), d_w.data_ptr(), d_s.data_ptr(), d_c.data_ptr(),
                          ws.data_ptr(), ws_bytes, m, n, k, lda, ldw, n)
    finally:
        hc.set_option("w8a16_variant", 0)
    finish(hc)
    assert hc.kernel_status() == 0
    return host_bf16(d_c)


# Four bands exactly; a last band of one tile column and a ragged last tile; more
# bands than ring slots with few row tiles; many row tiles.
@pytest.mark.parametrize("shape", [(256, 4096, 64), (512, 4368, 128), (300, 8192, 192),
                                   (2048, 6144, 512), (4096, 8192, 256)])
def test_banded_equals_the_two_pass_form_bit_for_bit(hc, shape):
    m, n, k = shape
    a, w, s = oracle.make_inputs("gemm_w8a16", shape=shape)
    d_a, d_w, d_s = dev_bf16(a), dev(w), dev(s)
    banded = _run(hc, d_a, d_w, d_s, m, n, k, k, n, 3, hc.gemm_w8a16_banded_bytes(n, k))
    two_pass = _run(hc, d_a, d_w, d_s, m, n, k, k, n, 1)
    assert not np.isnan(banded).any()
    assert np.array_equal(banded, two_pass)
    if m * n * k <= 1 << 28:
        expect = np.zeros((m, n), np.float32)
        oracle.gemm_w8a16(a, w, s, expect, (256, 256))
        mag = np.abs(a) @ (np.abs(w.astype(np.float32)) * s)
        assert np.all(np.abs(banded - expect) <= 1e-2 * np.abs(expect) + 1e-4 * mag)


def test_the_ring_is_smaller_than_the_converted_matrix(hc):
    assert hc.gemm_w8a16_banded_bytes(8192, 8192) == 3 * 8192 * 1024 * 2 + 256
    assert hc.gemm_w8a16_banded_bytes(8192, 8192) * 2 < hc.gemm_w8a16_workspace_bytes(8192, 8192)


def test_layouts_it_does_not_take(hc):
    """Fewer than four bands, a K that is not a multiple of 64, or a workspace
    that is too small are refused when the banded form is demanded."""
    for shape in [(256, 2048, 128), (256, 4096, 96)]:
        m, n, k = shape
        a, w, s = oracle.make_inputs("gemm_w8a16", shape=shape)
        with pytest.raises(RuntimeError, match="the banded form needs"):
            _run(hc, dev_bf16(a), dev(w), dev(s), m, n, k, k, n, 3)
    m, n, k = 256, 4096, 128
    a, w, s = oracle.make_inputs("gemm_w8a16", shape=(m, n, k))
    with pytest.raises(RuntimeError, match="the banded form needs"):
        _run(hc, dev_bf16(a), dev(w), dev(s), m, n, k, k, n, 3,
             hc.gemm_w8a16_banded_bytes(n, k) - 256)
