"""Run-time specialisation on the GPU: a body that was not compiled ahead of
time is compiled by NVRTC at its first launch and from then on runs as a
straight-line kernel.  It must give bit for bit what the interpreter gives
(option ``fused`` = 1 sends every program to the interpreter), be compiled once
per context and program whatever the constants and shapes.  Element-wise programs
are compiled whatever their operators and element type; row programs on floats."""

import numpy as np
import pytest
import torch

from hc_b200.hckernel.kernel import get_context
from hc_b200.workloads import make_elementwise, make_rowwise

pytestmark = pytest.mark.gpu


def _place(arrays, shape, pitch):
    d_in = []
    for a in arrays:
        store = torch.zeros((shape[0], pitch), dtype=torch.from_numpy(a).dtype, device="cuda")
        store[:, : shape[1]] = torch.from_numpy(a).cuda()
        d_in.append(store[:, : shape[1]])
    return d_in


def _run(kernel, d_in, shape, pitch, tail, interpret):
    ctx = get_context("cuda:0")
    store = torch.full((shape[0], pitch), -77.0, dtype=d_in[0].dtype, device="cuda")
    d_out = store[:, : shape[1]]
    ctx.set_option("fused", int(interpret))
    try:
        kernel(*d_in, d_out, *tail)
    finally:
        ctx.set_option("fused", 0)
    torch.cuda.synchronize()
    assert (store[:, shape[1]:] == -77.0).all()  # the padding stays untouched
    return d_out.cpu().numpy()


MAP_BODIES = [
    ("exp_of_max", lambda a, b: np.exp(np.maximum(a * 1.5, b) + 0.25), 2),
    ("quotient", lambda a, b: (a - b) / (b * b + a), 2),           # divisions: masked stores
    ("three_inputs", lambda a, b, c: np.sqrt(np.abs(a * b - c * 0.5)) + a, 3),
    ("one_input", lambda a: np.minimum(a * a * 0.5 - a, a * 0.125), 1),
    ("select", lambda a, b: (a < b) * a + (a >= b) * b, 2),          # comparisons
    ("divmod", lambda a, b: (a // b) * b + a % b, 2),                # out-of-line routines, masks
]
MAP_SHAPES = [((64, 1024), 1024), ((33, 1001), 1001), ((17, 100), 104), ((1, 7), 7),
              ((1024, 2048), 2048)]


@pytest.mark.parametrize("dtype", ["float32", "float64"])
@pytest.mark.parametrize("body", MAP_BODIES, ids=lambda b: b[0])
def test_specialised_elementwise_bodies_equal_the_interpreter(body, dtype):
    name, fn, count = body
    ctx = get_context("cuda:0")
    kernel = make_elementwise(fn, count, 2, (4, 64))
    before = ctx.specialised_programs() + ctx.specialised_programs(from_disk=True)
    for shape, pitch in MAP_SHAPES:
        rng = np.random.default_rng(shape[1])
        arrays = [(rng.standard_normal(shape) + 0.25).astype(dtype) for _ in range(count)]
        if name in ("quotient", "divmod"):
            arrays[1][::3, ::5] = 0  # some divisors are zero: b*b + a == a ... and
            arrays[0][::3, ::5] = 0  # ... a too: 0 / 0, which numpy.ma masks
        d_in = _place(arrays, shape, pitch)
        compiled = _run(kernel, d_in, shape, pitch, (), interpret=False)
        interpreted = _run(kernel, d_in, shape, pitch, (), interpret=True)
        assert np.array_equal(compiled, interpreted, equal_nan=True), (name, shape)
        if name in ("quotient", "divmod"):
            assert (compiled[::3, ::5] == -77.0).all()  # masked elements are not stored
        else:
            with np.errstate(all="ignore"):
                want = fn(*arrays)  # NumPy in the arrays' own type
            np.testing.assert_allclose(compiled, want, rtol=4e-6 if dtype == "float32" else 1e-13,
                                       atol=2e-6, equal_nan=True)
    after = ctx.specialised_programs() + ctx.specialised_programs(from_disk=True)
    # One program, compiled once for all shapes (not at all when an earlier test of the
    # session, which shares the context, launched the same program).
    assert after - before in (0, 1), ctx.specialise_note


ROW_BODIES = [
    ("centred_exp", lambda t: np.exp(t - t.max(axis=1, keepdims=True)) * 0.5
     + t.sum(axis=1, keepdims=True) * 0.001, 1),
    ("two_inputs", lambda a, b: (a * b) / np.sqrt((a * a).sum(axis=1, keepdims=True))
     - b.max(axis=1, keepdims=True), 2),
]
ROW_SHAPES = [((19, 4096), 4096), ((5, 2048), 2048), ((9, 1028), 1032), ((33, 1001), 1001),
              ((300, 36), 40), ((3, 8192), 8192)]


@pytest.mark.parametrize("dtype", ["float32", "float64"])
@pytest.mark.parametrize("body", ROW_BODIES, ids=lambda b: b[0])
def test_specialised_row_bodies_equal_the_interpreter(body, dtype):
    name, fn, count = body
    ctx = get_context("cuda:0")
    kernel = make_rowwise(fn, count)
    before = ctx.specialised_programs() + ctx.specialised_programs(from_disk=True)
    for shape, pitch in ROW_SHAPES:
        rng = np.random.default_rng(shape[1])
        arrays = [(rng.random(shape) + 0.25).astype(dtype) for _ in range(count)]
        d_in = _place(arrays, shape, pitch)
        compiled = _run(kernel, d_in, shape, pitch, (8,), interpret=False)
        interpreted = _run(kernel, d_in, shape, pitch, (8,), interpret=True)
        assert np.array_equal(compiled, interpreted, equal_nan=True), (name, shape)
        assert np.isfinite(compiled).all()
    after = ctx.specialised_programs() + ctx.specialised_programs(from_disk=True)
    assert after - before in (0, 1), ctx.specialise_note


@pytest.mark.parametrize("dtype", ["int32", "int64"])
def test_specialised_integer_bodies_equal_the_interpreter(dtype):
    ctx = get_context("cuda:0")
    fn = lambda a, b: ((a << 2) ^ b) // 7 + (a % 5) * (b & 12) - abs(a)  # noqa: E731
    kernel = make_elementwise(fn, 2, 2, (4, 64))
    before = ctx.specialised_programs() + ctx.specialised_programs(from_disk=True)
    for shape, pitch in MAP_SHAPES:
        rng = np.random.default_rng(shape[1] + 5)
        arrays = [rng.integers(-1000, 1000, shape).astype(dtype) for _ in range(2)]
        d_in = _place(arrays, shape, pitch)
        compiled = _run(kernel, d_in, shape, pitch, (), interpret=False)
        interpreted = _run(kernel, d_in, shape, pitch, (), interpret=True)
        assert np.array_equal(compiled, interpreted), shape
        assert np.array_equal(compiled, fn(*arrays)), shape  # NumPy's integer arithmetic
    after = ctx.specialised_programs() + ctx.specialised_programs(from_disk=True)
    assert after - before in (0, 1), ctx.specialise_note


def test_switch_and_scope():
    ctx = get_context("cuda:0")
    x = torch.randn(256, 512, device="cuda")
    out = torch.empty_like(x)
    count = lambda: ctx.specialised_programs() + ctx.specialised_programs(from_disk=True)  # noqa: E731
    body = lambda a: a * 0.75 + np.exp(a) * 0.375  # noqa: E731
    # Off: interpreted, nothing compiled.
    before = count()
    ctx.set_option("specialise", 0)
    try:
        make_elementwise(body, 1, 2, (4, 64))(x, out)
    finally:
        ctx.set_option("specialise", 1)
    torch.cuda.synchronize()
    assert count() == before
    assert torch.allclose(out, x * 0.75 + x.exp() * 0.375, rtol=1e-5, atol=1e-6)
    # Demanded: compiled (NVRTC is there), and the launch succeeds.
    ctx.set_option("specialise", 2)
    try:
        make_elementwise(body, 1, 2, (4, 64))(x, out)
        torch.cuda.synchronize()
        assert count() == before + 1, ctx.specialise_note
    finally:
        ctx.set_option("specialise", 1)
    assert torch.allclose(out, x * 0.75 + x.exp() * 0.375, rtol=1e-5, atol=1e-6)
    # Another constant is the same program: nothing new is compiled.
    make_elementwise(lambda a: a * 0.5 + np.exp(a) * 2.0, 1, 2, (4, 64))(x, out)
    torch.cuda.synchronize()
    assert count() == before + 1
    assert torch.allclose(out, x * 0.5 + x.exp() * 2.0, rtol=1e-5, atol=1e-6)


def test_a_specialised_body_runs_at_the_speed_of_a_precompiled_one():
    """A body outside the ahead-of-time list against itself interpreted, on a case
    large enough to tell (512 MB in, 512 MB out)."""
    ctx = get_context("cuda:0")
    x = torch.randn(32768, 4096, device="cuda")
    out = torch.empty_like(x)
    k = make_rowwise(lambda t: (t - t.max(axis=1, keepdims=True)) * 0.5
                     - np.log(np.exp(t * 0.25).sum(axis=1, keepdims=True)))

    def timed(interpret):
        ctx.set_option("fused", int(interpret))
        try:
            k(x, out, 8)
            ctx.synchronize()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(10):
                k(x, out, 8)
            e1.record()
            torch.cuda.synchronize()
            return e0.elapsed_time(e1) / 10
        finally:
            ctx.set_option("fused", 0)

    fast, slow = timed(False), timed(True)
    assert fast < slow
    assert 2 * x.numel() * 4 / (fast * 1e-3) / 1e9 > 4500  # GB/s; the copy peak is about 6500
