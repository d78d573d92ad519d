"""The float32 convolution on the tensor cores (hcConvF32Tensor: an implicit GEMM
over output pixels, image operand gathered by the kernel, three tf32 products
per product) through the C-ABI, against the textbook correlation the reference's
own test compares with (python/hckernel/tests/test_examples.py:179-199) computed
in float64.

Tolerance: the parity bound of the float32 kernels, |got - exact| <= 1e-5 *
sum|x||f| per element, and the tighter 2e-6 * sum|x||f| that a single tf32
product (about 5e-4) could not meet."""

import numpy as np
import pytest
import torch

from oracle import workloads as oracle
from tests.gpu_util import dev, empty_like_dev, finish

pytestmark = pytest.mark.gpu


def _workspace(hc, n, c, h, w, nf, hf, wf):
    need = hc.lib.hcConvF32TensorWorkspaceBytes(n, c, h, w, nf, hf, wf)
    buf = torch.empty(need + 1024, dtype=torch.uint8, device="cuda")
    return buf, buf.data_ptr() + (-buf.data_ptr()) % 1024, need


def _conv(hc, x, f, stride):
    n, c, h, w = x.shape
    nf, _, hf, wf = f.shape
    ho, wo = (h - hf) // stride + 1, (w - wf) // stride + 1
    keep, ws, need = _workspace(hc, n, c, h, w, nf, hf, wf)
    d_x, d_f = dev(x), dev(f)
    d_o = torch.full((n, nf, ho, wo), float("nan"), dtype=torch.float32, device="cuda")
    torch.cuda.synchronize()
    for _ in range(2):  # twice: the second call reuses the loaded kernel and the workspace
        hc.conv_f32_tensor(d_x.data_ptr(), d_f.data_ptr(), d_o.data_ptr(), n, c, h, w, nf, hf,
                           wf, stride, ws, need)
    finish(hc)
    del keep
    return d_o.cpu().numpy()


CASES = [
    # x shape, f shape, stride
    ((2, 8, 30, 30), (128, 8, 3, 3), 1),    # 128 filters: the most the tensor-memory form takes
    ((2, 3, 8, 8), (4, 3, 3, 3), 1),        # K = 27: one partial K block, 36 pixels
    ((1, 1, 5, 5), (1, 1, 1, 1), 1),        # a 1 x 1 filter, one filter
    ((3, 8, 20, 20), (5, 8, 3, 3), 1),      # 324 pixels: three tiles, the last ragged; NF = 5
    ((2, 4, 17, 23), (16, 4, 3, 5), 2),     # rectangular image and filter, stride 2
    ((2, 16, 12, 12), (33, 16, 2, 2), 1),   # NF = 33 -> N of 48, two column chunks
    ((1, 64, 14, 14), (64, 64, 3, 3), 1),   # K = 576 as at the benchmark size
    ((5, 7, 9, 40), (200, 7, 3, 3), 3),     # many filters (two stages of shared memory)
    ((1, 2, 3, 3), (2, 2, 3, 3), 1),        # one output pixel
    ((2, 40, 16, 70), (24, 40, 3, 3), 1),   # 40 channels: a partial channel block; wide rows
    ((1, 32, 130, 9), (16, 32, 5, 2), 1),   # tall and narrow: rectangles of 8 x 16
    ((3, 96, 28, 28), (192, 96, 1, 1), 1),  # a 1 x 1 filter over three channel blocks, 192 filters
    ((2, 16, 40, 40), (16, 16, 7, 7), 1),   # seven taps per filter row share a patch of 136 rows
    ((1, 8, 64, 64), (32, 8, 5, 3), 1),     # 64-wide rows: tiles of two whole rows
    ((2, 8, 20, 40), (8, 8, 1, 9), 1),      # nine taps in a row: shifts of more than 1 KiB
]


# conv_variant: 1 = the image operand of a K block is gathered by threads into shared
# memory, 2 = into tensor memory (at most 128 filters), 3 = both operands come by TMA
# (stride 1, images that hold a rectangle of 128 pixels), 4 = both by TMA with the image
# patch of a filter row shared by its taps, 0 = the library's choice.
# conv_stacked: 0 = with at most 128 filters the two products that share a_hi run as
# one MMA of twice the width, 1 = three MMAs per K step throughout.
@pytest.mark.parametrize("unstacked", [0, 1])
@pytest.mark.parametrize("variant", [0, 1, 2, 3, 4])
@pytest.mark.parametrize("xs,fs,stride", CASES)
def test_matches_the_float64_correlation(hc, xs, fs, stride, variant, unstacked):
    if variant == 2 and fs[0] > 128:
        pytest.skip("more filters than the tensor-memory form takes")
    if variant == 3 and (stride != 1 or not any(bw <= xs[3] and 128 // bw <= xs[2]
                                                for bw in (8, 16, 32, 64, 128))):
        pytest.skip("the TMA form takes stride 1 and images that hold 128 pixels")
    patch = -(-(128 + fs[3] - 1) // 8) * 8
    stage = 2 * patch * 128 + fs[3] * 2 * (-(-fs[0] // 16) * 16) * 128
    if variant == 4 and (stride != 1 or xs[2] * xs[3] < patch or 2 * stage > 227 * 1024 - 1280):
        pytest.skip("the shared-patch form takes stride 1, images of 128 + WF - 1 positions "
                    "and filters of which two stages fit in shared memory")
    hc.set_option("conv_variant", variant)
    hc.set_option("conv_stacked", unstacked)
    try:
        _matches_the_float64_correlation(hc, xs, fs, stride)
    finally:
        hc.set_option("conv_variant", 0)
        hc.set_option("conv_stacked", 0)


def _matches_the_float64_correlation(hc, xs, fs, stride):
    rng = np.random.default_rng(sum(xs) * 31 + sum(fs))
    x = rng.uniform(-1, 1, xs).astype(np.float32)
    f = rng.uniform(-1, 1, fs).astype(np.float32)
    got = _conv(hc, x, f, stride).astype(np.float64)
    exact = _direct(x, f, stride)
    scale = _direct(np.abs(x), np.abs(f), stride)
    assert got.shape == exact.shape and not np.isnan(got).any()
    assert np.all(np.abs(got - exact) <= 1e-5 * scale + 1e-30)
    assert np.all(np.abs(got - exact) <= 2e-6 * scale + 1e-30)


def _direct(x, f, stride):
    """The correlation for any rectangle, in float64."""
    x, f = x.astype(np.float64), f.astype(np.float64)
    n, c, h, w = x.shape
    nf, _, hf, wf = f.shape
    ho, wo = (h - hf) // stride + 1, (w - wf) // stride + 1
    out = np.zeros((n, nf, ho, wo))
    for kh in range(hf):
        for kw in range(wf):
            patch = x[:, :, kh: kh + (ho - 1) * stride + 1: stride,
                      kw: kw + (wo - 1) * stride + 1: stride]
            out += np.einsum("nchw,qc->nqhw", patch, f[:, :, kh, kw])
    return out


def test_agrees_with_the_gathered_kernel_and_the_oracle(hc):
    """The reference's own tiling of the same convolution (oracle) on a square case."""
    x, f = oracle.make_conv_inputs((4, 6, 12, 12), (8, 6, 3, 3), "float32")
    expect = np.zeros((4, 8, 10, 10), np.float32)
    oracle.conv_implicit_gemm(x, f, expect, 1, 4, 8, 16)
    got = _conv(hc, x, f, 1)
    bound = 1e-5 * _direct(np.abs(x), np.abs(f), 1)
    assert np.all(np.abs(got.astype(np.float64) - expect) <= 2 * bound)


def test_refusals(hc):
    keep, ws, need = _workspace(hc, 2, 3, 8, 8, 4, 3, 3)
    with pytest.raises(RuntimeError, match="invalid shape"):
        hc.conv_f32_tensor(1, 1, 1, 2, 3, 2, 8, 4, 3, 3, 1, ws, need)  # filter taller than image
    with pytest.raises(RuntimeError, match="at most 256 filters"):
        hc.conv_f32_tensor(1, 1, 1, 2, 3, 8, 8, 300, 3, 3, 1, ws, need)
    with pytest.raises(RuntimeError, match="workspace"):
        hc.conv_f32_tensor(1, 1, 1, 2, 3, 8, 8, 4, 3, 3, 1, ws, need - 1)
    with pytest.raises(RuntimeError, match="null array"):
        hc.conv_f32_tensor(0, 1, 1, 2, 3, 8, 8, 4, 3, 3, 1, ws, need)
    hc.conv_f32_tensor(0, 0, 0, 0, 3, 8, 8, 4, 3, 3, 1, 0, 0)  # no images: nothing to do
    del keep


def test_the_front_door_sends_convolution_bodies_to_the_tensor_cores():
    """The reference's implicit-GEMM body (python/hckernel/tests/test_examples.py:203-252):
    its work-groups are recognised from their evaluated index tables as a plain
    convolution and run on hcConvF32Tensor (two launches: the rewriting of both operands and
    the convolution);
    with ``settings.CONV_VARIANT = 1`` they run as the body tiles them (one launch of
    the gathered kernel).  Both within the float32 parity bound of the exact sums."""
    from hc_b200.hckernel import settings
    from hc_b200.hckernel.kernel import get_context, sym
    from hc_b200.workloads import make_conv

    x, f = oracle.make_conv_inputs((8, 16, 34, 34), (32, 16, 3, 3), "float32")
    d_x, d_f = torch.from_numpy(x).cuda(), torch.from_numpy(f).cuda()
    conv = make_conv(1).parametrize({sym.TN: 8, sym.TNF: 32, sym.KB: 16})
    ctx = get_context("cuda:0")
    exact = _direct(x, f, 1)
    bound = 1e-5 * _direct(np.abs(x), np.abs(f), 1)
    launches = {}
    for variant in (0, 1):
        settings.CONV_VARIANT = variant
        try:
            out = torch.full((8, 32, 32, 32), float("nan"), device="cuda")
            conv(d_x, d_f, out)  # plans, uploads tables or makes the workspace
            before = ctx.launch_count
            conv(d_x, d_f, out)
            torch.cuda.synchronize()
            launches[variant] = ctx.launch_count - before
        finally:
            settings.CONV_VARIANT = 0
        assert np.all(np.abs(out.cpu().numpy().astype(np.float64) - exact) <= bound)
    assert launches == {0: 2, 1: 1}
    # A rectangular image is not the plain convolution (the body walks the output
    # positions transposed): it stays with the gathered kernel.
    xr, fr = oracle.make_conv_inputs((8, 16, 34, 66), (32, 16, 3, 3), "float32")
    out_r = torch.zeros((8, 32, 32, 64), device="cuda")
    before = ctx.launch_count
    conv(torch.from_numpy(xr).cuda(), torch.from_numpy(fr).cuda(), out_r)
    torch.cuda.synchronize()
    assert ctx.launch_count - before == 1
    expect = np.zeros((8, 32, 32, 64), np.float32)
    oracle.conv_implicit_gemm(xr, fr, expect, 1, 8, 32, 16)
    assert np.allclose(out_r.cpu().numpy(), expect, rtol=1e-4, atol=1e-3)
