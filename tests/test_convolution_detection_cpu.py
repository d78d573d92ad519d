"""Which mapped work-groups are recognised as a plain convolution (no GPU needed).

The reference's implicit-GEMM body (python/hckernel/tests/test_examples.py:203-252)
walks the output positions and the filter taps transposed (``i = w % W_OUT`` on the H
axis, :237-240; tap ``r % WF`` on the H axis, :220-226).  For square outputs and
filters that is the plain convolution in another order, which is what the
tensor-core kernel computes; for rectangles it is not, and the body keeps running as
it tiles the problem itself.  The decision is taken on the evaluated index tables
(`MappedSpec.as_convolution`), so it is checked here against the oracle's run of the
same body and the textbook correlation."""

import numpy as np
import pytest

from hc_b200.hckernel.kernel import sym
from hc_b200.workloads import make_conv
from oracle import workloads as oracle
from tests.test_frontdoor_cpu import F


def _spec(xs, fs, stride, tiles):
    conv = make_conv(stride).parametrize({sym.TN: tiles[0], sym.TNF: tiles[1], sym.KB: tiles[2]})
    os_ = oracle.conv_out_shape(xs, fs, stride)
    plan = conv.plan_for((F(xs), F(fs), F(os_)))
    assert plan.family == "mapped_gemm"
    return plan.roles["spec"], os_


@pytest.mark.parametrize("xs,fs,stride,tiles", [
    ((4, 6, 12, 12), (8, 6, 3, 3), 1, (4, 8, 16)),
    ((3, 3, 9, 9), (5, 3, 3, 3), 2, (2, 4, 8)),      # ragged image and filter blocks, stride 2
    ((2, 2, 7, 7), (3, 2, 1, 1), 3, (1, 1, 8)),      # 1 x 1 filter, one image and filter per group
    ((32, 64, 30, 30), (64, 64, 3, 3), 1, (32, 64, 16)),
])
def test_square_cases_are_the_plain_convolution(xs, fs, stride, tiles):
    spec, os_ = _spec(xs, fs, stride, tiles)
    assert spec.as_convolution(xs, fs, os_) == stride
    if np.prod(xs) < 10000:  # and the body's result is the textbook correlation there
        x, f = oracle.make_conv_inputs(xs, fs, "float64")
        out = np.zeros(os_)
        oracle.conv_implicit_gemm(x, f, out, stride, *tiles)
        assert np.allclose(out, oracle.conv_direct(x, f, stride), rtol=1e-12, atol=1e-12)


@pytest.mark.parametrize("xs,fs,stride,tiles", [
    ((2, 3, 9, 13), (5, 3, 3, 3), 2, (2, 4, 8)),     # rectangular image
    ((2, 3, 9, 9), (5, 3, 3, 2), 1, (2, 4, 8)),      # rectangular filter
])
def test_rectangles_are_not(xs, fs, stride, tiles):
    spec, os_ = _spec(xs, fs, stride, tiles)
    assert spec.as_convolution(xs, fs, os_) is None


def test_other_arrays_than_the_plan_was_made_for_are_not():
    spec, os_ = _spec((4, 6, 12, 12), (8, 6, 3, 3), 1, (4, 8, 16))
    assert spec.as_convolution((4, 6, 12, 12), (8, 6, 3, 3), (4, 8, 10, 9)) is None
    assert spec.as_convolution((4, 6, 12), (8, 6, 3, 3), os_) is None
    assert spec.as_convolution((4, 5, 12, 12), (8, 5, 3, 3), os_) is None
