"""GPU parity of the bodies that are compiled ahead of time (fused_programs.h):
every listed body, float32 and float64, on shapes that reach each kernel form
(16-byte packets and single elements, rows held by a CTA and rows walked by a
warp, ragged and pitched rows), must give bit for bit what the interpreter
gives for the same program (option ``fused`` = 1 turns the precompiled kernels
off), and agree with NumPy within the tolerances of the interpreter's own tests
(2e-6 relative in float32 - a row sum is a running value per lane plus a
shuffle tree where NumPy's is pairwise - 1e-13 in float64)."""

import numpy as np
import pytest
import torch

from hc_b200.hckernel import precompiled
from hc_b200.hckernel.kernel import get_context
from hc_b200.workloads import make_elementwise, make_rowwise

pytestmark = pytest.mark.gpu

TOL = {"float32": dict(rtol=4e-6, atol=2e-6), "float64": dict(rtol=1e-13, atol=1e-14)}


def _inputs(count, shape, dtype, seed, positive=False):
    rng = np.random.default_rng(seed)
    if positive:  # row statistics (a sum in a denominator) stay well conditioned
        return [(rng.random(shape) + 0.25).astype(dtype) for _ in range(count)]
    return [(rng.standard_normal(shape) + 0.25).astype(dtype) for _ in range(count)]


def _run_both(kernel, d_in, shape, pitch, tail):
    """The kernel with and without the precompiled bodies; returns both outputs."""
    ctx = get_context("cuda:0")
    outs = []
    for off in (0, 1):
        store = torch.full((shape[0], pitch), float("nan"), dtype=d_in[0].dtype, device="cuda")
        d_out = store[:, : shape[1]]
        ctx.set_option("fused", off)
        try:
            kernel(*d_in, d_out, *tail)
        finally:
            ctx.set_option("fused", 0)
        torch.cuda.synchronize()
        if pitch > shape[1]:
            assert torch.isnan(store[:, shape[1]:]).all()  # the padding stays untouched
        outs.append(d_out.cpu().numpy())
    return outs


ROW_SHAPES = [((19, 4096), 4096), ((5, 2048), 2048), ((7, 3840), 3840), ((9, 1028), 1032),
              ((33, 1001), 1001), ((300, 36), 40), ((3, 8192), 8192), ((1, 1), 1)]


@pytest.mark.parametrize("dtype", ["float32", "float64"])
@pytest.mark.parametrize("body", precompiled.ROW_BODIES, ids=lambda b: b[0])
def test_precompiled_row_bodies_equal_the_interpreter(body, dtype):
    name, fn, count = body
    for shape, pitch in ROW_SHAPES:
        for positive in (True, False):
            inputs = _inputs(count, shape, dtype, shape[1], positive)
            d_in = []
            for a in inputs:
                store = torch.zeros((shape[0], pitch), dtype=torch.from_numpy(a).dtype,
                                    device="cuda")
                store[:, : shape[1]] = torch.from_numpy(a).cuda()
                d_in.append(store[:, : shape[1]])
            fused, interpreted = _run_both(make_rowwise(fn, count), d_in, shape, pitch, (8,))
            assert np.array_equal(fused, interpreted, equal_nan=True), (name, shape)
            if positive:  # (signed inputs make sums cancel: no fixed tolerance against NumPy)
                with np.errstate(all="ignore"):
                    want = fn(*[a.astype(np.float64) for a in inputs])
                np.testing.assert_allclose(fused, want, **TOL[dtype])


MAP_SHAPES = [((64, 1024), 1024), ((33, 1001), 1001), ((17, 100), 104), ((1, 7), 7),
              ((2048, 2048), 2048)]


@pytest.mark.parametrize("dtype", ["float32", "float64"])
@pytest.mark.parametrize("body", precompiled.MAP_BODIES, ids=lambda b: b[0])
def test_precompiled_elementwise_bodies_equal_the_interpreter(body, dtype):
    name, fn, count = body
    for shape, pitch in MAP_SHAPES:
        inputs = _inputs(count, shape, dtype, shape[1] + 1)
        d_in = []
        for a in inputs:
            store = torch.zeros((shape[0], pitch), dtype=torch.from_numpy(a).dtype, device="cuda")
            store[:, : shape[1]] = torch.from_numpy(a).cuda()
            d_in.append(store[:, : shape[1]])
        fused, interpreted = _run_both(make_elementwise(fn, count, 2, (4, 64)), d_in, shape, pitch,
                                       ())
        assert np.array_equal(fused, interpreted, equal_nan=True), (name, shape)
        with np.errstate(all="ignore"):
            want = fn(*inputs)  # NumPy in the arrays' own type: the same IEEE operations
        assert np.array_equal(fused, want, equal_nan=True) or np.allclose(
            fused, want, **TOL[dtype], equal_nan=True), (name, shape)


def test_the_precompiled_kernel_is_what_runs():
    """The launch really goes to the straight-line kernel: the same body is
    faster per launch than interpreted on a case large enough to tell, and a
    body that is not in the list still runs (interpreted)."""
    ctx = get_context("cuda:0")
    name, fn, count = precompiled.ROW_BODIES[2]
    assert name == "log_softmax"
    x = torch.randn(4096, 4096, device="cuda")
    out = torch.empty_like(x)
    k = make_rowwise(fn, count)

    def timed(off):
        ctx.set_option("fused", off)
        try:
            k(x, out, 8)
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(20):
                k(x, out, 8)
            e1.record()
            torch.cuda.synchronize()
            return e0.elapsed_time(e1)
        finally:
            ctx.set_option("fused", 0)

    assert timed(0) < timed(1)
    other = make_rowwise(lambda t: t * 3.0 - t.max(axis=1, keepdims=True) * t.sum(axis=1, keepdims=True))
    other(x, out, 8)
    torch.cuda.synchronize()
    xs = x.double()
    want = xs * 3 - xs.max(dim=1, keepdim=True).values * xs.sum(dim=1, keepdim=True)
    assert torch.allclose(out.double(), want, rtol=1e-4, atol=1e-3)
