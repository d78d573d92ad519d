"""GPU parity of element-wise bodies: through the ``@kernel`` front door against
the outputs of the reference simulator (tests/golden) and against NumPy, and
hcMapElements called directly through the C-ABI.

Tolerances: + - * / sqrt, max, min, abs and negation are single correctly
rounded IEEE operations in the array's type, never contracted, so against
NumPy on the same arrays the result is bit-exact; ``exp`` is within 4 ulp
(expf is accurate to 2 ulp, NumPy's own exp to about 1).
Against the reference simulator float32 results may differ in the last bits
where the reference carries a Python-float operand on in float64
(oracle.elementwise explains): 3e-7 relative."""

import numpy as np
import pytest
import torch

from hc_b200 import capi
from hc_b200.hckernel import elementwise as ew
from hc_b200.workloads import make_elementwise
from oracle import workloads as oracle
from tests.gpu_util import finish

pytestmark = pytest.mark.gpu

CASES = oracle.elementwise_cases()


@pytest.mark.parametrize("case", CASES, ids=lambda c: c[0])
def test_element_wise_bodies_match_reference_and_numpy(golden, case):
    name, fn, count, shape, dtype, group = case
    inputs = oracle.make_elementwise_inputs(count, shape, dtype)
    k = make_elementwise(fn, count, len(shape), group)
    d_in = [torch.from_numpy(a).cuda() for a in inputs]
    d_out = torch.full(shape, float("nan"), dtype=d_in[0].dtype, device="cuda")
    k(*d_in, d_out)
    torch.cuda.synchronize()
    got = d_out.cpu().numpy()
    with np.errstate(all="ignore"):
        want = fn(*inputs)
    if "gauss" in name:
        np.testing.assert_array_max_ulp(got, want, maxulp=4)
    else:
        assert np.array_equal(got, want)
    np.testing.assert_allclose(got, golden[name], rtol=3e-7 if dtype == "float32" else 2e-16)


@pytest.mark.parametrize("shape,pitch", [((37, 101), 101), ((64, 256), 260), ((5, 8), 12),
                                         ((1, 1), 1), ((300, 4), 4)])
def test_unaligned_and_pitched_matrices(shape, pitch):
    """Rows that are not multiples of 16 bytes, views with a pitch, tiny arrays."""
    rng = np.random.default_rng(shape[0] * 1000 + shape[1])
    a = rng.standard_normal(shape).astype(np.float32)
    b = rng.standard_normal(shape).astype(np.float32)
    k = make_elementwise(lambda s, t: np.minimum(s, t) / (np.abs(t) + 0.5), 2, 2, (8, 32))
    store = torch.zeros((3, shape[0], pitch), device="cuda")
    d_a, d_b, d_out = (store[i, :, : shape[1]] for i in range(3))
    d_a.copy_(torch.from_numpy(a))
    d_b.copy_(torch.from_numpy(b))
    k(d_a, d_b, d_out)
    torch.cuda.synchronize()
    assert np.array_equal(d_out.cpu().numpy(), np.minimum(a, b) / (np.abs(b) + np.float32(0.5)))
    if pitch > shape[1]:  # the gap between rows is not touched
        assert float(store[2, :, shape[1]:].abs().max()) == 0.0


def test_random_expressions_on_the_gpu():
    """40 random expression trees, float64, ragged shape: bit for bit what NumPy
    gives on the same arrays (no operation in the generator's set is inexact on
    the GPU: + - * / sqrt abs neg max min are correctly rounded)."""
    from hc_b200.hckernel.kernel import UnsupportedKernel

    rng = np.random.default_rng(77)
    shape, ran = (37, 53), 0
    for _ in range(40):
        count = int(rng.integers(1, 4))
        fn, text = oracle.random_expression(rng, count, int(rng.integers(1, 5)))
        inputs = oracle.make_elementwise_inputs(count, shape, "float64", seed=ran + 100)
        d_in = [torch.from_numpy(a).cuda() for a in inputs]
        d_out = torch.full(shape, float("nan"), dtype=torch.float64, device="cuda")
        try:
            make_elementwise(fn, count, 2, (8, 16))(*d_in, d_out)
        except UnsupportedKernel:
            continue
        torch.cuda.synchronize()
        with np.errstate(all="ignore"):
            want = np.broadcast_to(fn(*inputs), shape)
        assert np.array_equal(d_out.cpu().numpy(), want, equal_nan=True), text
        ran += 1
    assert ran > 25


def test_nan_and_signed_zero_semantics():
    """NumPy's maximum/minimum propagate NaN; abs and negation handle -0.0."""
    a = np.array([[np.nan, 1.0, -0.0, 0.0, -2.0, np.inf, 3.0, np.nan]], np.float32)
    b = np.array([[1.0, np.nan, 0.0, -0.0, 5.0, -np.inf, 3.0, np.nan]], np.float32)
    for fn in (lambda s, t: np.maximum(s, t), lambda s, t: np.minimum(s, t),
               lambda s, t: np.abs(s) - (-t)):
        k = make_elementwise(fn, 2, 2, (1, 8))
        d_out = torch.zeros((1, 8), device="cuda")
        k(torch.from_numpy(a).cuda(), torch.from_numpy(b).cuda(), d_out)
        torch.cuda.synchronize()
        with np.errstate(all="ignore"):
            want = fn(a, b)
        got = d_out.cpu().numpy()
        assert np.array_equal(np.isnan(got), np.isnan(want))
        ok = ~np.isnan(want)
        assert np.array_equal(got[ok], want[ok])
        assert np.array_equal(np.signbit(got[ok]), np.signbit(want[ok]))


def test_map_elements_through_the_c_abi(hc):
    rng = np.random.default_rng(5)
    rows, cols = 19, 40
    a, b = rng.standard_normal((rows, cols)), rng.standard_normal((rows, cols))
    d_a, d_b = torch.from_numpy(a).cuda(), torch.from_numpy(b).cuda()
    d_out = torch.zeros((rows, cols), dtype=torch.float64, device="cuda")
    p = capi.HcMapProgram()
    p.inputs[0], p.inputs[1] = d_a.data_ptr(), d_b.data_ptr()
    p.inPitch[0] = p.inPitch[1] = p.outPitch = cols
    p.out, p.rows, p.cols, p.nInputs = d_out.data_ptr(), rows, cols, 2
    # sqrt(a*a + b*b) * 0.5: load a; mul a; save t0; load b; mul b; add t0; sqrt; mul c0
    program = [ew.LOAD | 0 << 8, ew.MUL | 0 << 8, ew.SAVE0, ew.LOAD | 1 << 8, ew.MUL | 1 << 8,
               ew.ADD | (ew.SRC_TEMP + 0) << 8, ew.SQRT, ew.MUL | (ew.SRC_CONST + 0) << 8]
    p.nInstr = len(program)
    for i, ins in enumerate(program):
        p.code[i] = ins
    p.consts[0] = 0.5
    hc.map_elements(p, capi.HC_F64)
    finish(hc)
    assert np.array_equal(d_out.cpu().numpy(), np.sqrt(b * b + a * a) * 0.5)

    # Malformed programs are refused with a message before anything is launched.
    p.code[5] = ew.ADD | (ew.SRC_TEMP + 1) << 8       # t1 was never written
    with pytest.raises(RuntimeError, match="not written yet"):
        hc.map_elements(p, capi.HC_F64)
    p.code[5] = 99                                    # unknown operation
    with pytest.raises(RuntimeError, match="unknown operation"):
        hc.map_elements(p, capi.HC_F64)
    p.code[5] = ew.ADD | 3 << 8                       # input 3 of 2
    with pytest.raises(RuntimeError, match="does not exist"):
        hc.map_elements(p, capi.HC_F64)
    p.code[5] = ew.ADD | (ew.SRC_TEMP + 0) << 8
    p.code[0] = ew.ADD | 0 << 8                       # accumulator read before it is set
    with pytest.raises(RuntimeError, match="first instruction"):
        hc.map_elements(p, capi.HC_F64)
    p.code[0] = ew.LOAD | 0 << 8
    p.nInstr = 0
    with pytest.raises(RuntimeError, match="instructions"):
        hc.map_elements(p, capi.HC_F64)
    p.nInstr = len(program)
    with pytest.raises(RuntimeError, match="unsupported dtype"):
        hc.map_elements(p, capi.HC_BF16)
    p.rows = 0
    hc.map_elements(p, capi.HC_F64)                   # empty: nothing to do


def test_work_item_kernels_of_the_reference_tests():
    """python/hckernel/tests/test_kernel_sim.py:381-412 (test_buffer_dims1/2) with
    the bodies unchanged: each work-item writes its own linearised global id."""
    from hc_b200.hckernel.kernel import (Buffer, CurrentGroup, CurrentWorkitem, kernel, sym,
                                         typename)

    G, G1, G2, DT = sym.G, sym.G1, sym.G2, typename.DT
    target = dict(backend="nvvm", device="cuda:0")

    @kernel(work_shape=G, **target)
    def dims1(gr: CurrentGroup, arr: Buffer[G, DT]):
        @gr.workitems
        def inner(wi: CurrentWorkitem):
            gid = wi.global_id()[0]
            if gid < arr.shape[0]:
                arr[gid] = gid

        inner()

    src = torch.zeros(12, dtype=torch.float64, device="cuda")
    dims1(src)
    torch.cuda.synchronize()
    assert np.array_equal(src.cpu().numpy(), np.arange(12))

    @kernel(work_shape=(G1, G2), **target)
    def dims2(gr: CurrentGroup, arr: Buffer[G1, G2, DT]):
        @gr.workitems
        def inner(wi: CurrentWorkitem):
            gid = wi.global_id()[:2]
            if gid[0] < arr.shape[0] and gid[1] < arr.shape[1]:
                arr[gid] = gid[0] * arr.shape[1] + gid[1]

        inner()

    for shape, dtype in (((12, 5), torch.float64), ((300, 1000), torch.float32)):
        src = torch.zeros(shape, dtype=dtype, device="cuda")
        dims2(src)
        torch.cuda.synchronize()
        assert np.array_equal(src.cpu().numpy(), np.arange(shape[0] * shape[1]).reshape(shape))


def test_work_item_kernel_with_reads():
    from hc_b200.hckernel.kernel import (Buffer, CurrentGroup, CurrentWorkitem, kernel, sym,
                                         typename)

    W, H, DT = sym.W, sym.H, typename.DT

    @kernel(work_shape=(W, H), backend="nvvm", device="cuda:0")
    def k(gr: CurrentGroup, a: Buffer[W, H, DT], b: Buffer[W, H, DT], out: Buffer[W, H, DT]):
        @gr.workitems
        def inner(wi: CurrentWorkitem):
            i, j = wi.global_id()
            if i < out.shape[0] and j < out.shape[1]:
                out[i, j] = (a[i, j] - b[i, j]) * (i + 1.0) + j

        inner()

    rng = np.random.default_rng(9)
    a, b = (rng.standard_normal((37, 130)).astype(np.float32) for _ in range(2))
    d_out = torch.full((37, 130), float("nan"), device="cuda")
    k(torch.from_numpy(a).cuda(), torch.from_numpy(b).cuda(), d_out)
    torch.cuda.synchronize()
    rows = np.arange(37, dtype=np.float32)[:, None]
    cols = np.arange(130, dtype=np.float32)[None, :]
    assert np.array_equal(d_out.cpu().numpy(), (a - b) * (rows + np.float32(1)) + cols)


OPERATOR_CASES = oracle.operator_cases()


@pytest.mark.parametrize("fused", [0, 1], ids=["precompiled-or-interpreted", "interpreted"])
@pytest.mark.parametrize("case", OPERATOR_CASES, ids=lambda c: c[0])
def test_operator_table_and_masked_store_match_the_reference(golden, case, fused):
    """The rest of the reference's tile operator table (// % ** comparisons,
    integer tiles) and its masked store: elements whose divisor is zero, or whose
    power is not finite, keep what the output held (-77 here), everything else is
    bit for bit the reference simulator's output - except ``**``, where the
    reference computes a float32 power through float64 and powf is within a few
    ulp (1e-6 relative)."""
    from hc_b200.hckernel.kernel import get_context

    name, fn, inputs, group = case
    k = make_elementwise(fn, len(inputs), 2, group)
    d_in = [torch.from_numpy(a).cuda() for a in inputs]
    d_out = torch.full(inputs[0].shape, -77, dtype=d_in[0].dtype, device="cuda")
    ctx = get_context("cuda:0")
    ctx.set_option("fused", fused)
    try:
        k(*d_in, d_out)
    finally:
        ctx.set_option("fused", 0)
    torch.cuda.synchronize()
    got, want = d_out.cpu().numpy(), golden[name]
    if "pow" in name:
        assert np.array_equal(got == -77, want == -77)
        np.testing.assert_allclose(got, want, rtol=1e-6)
    else:
        assert np.array_equal(got, want)


@pytest.mark.parametrize("dtype", ["int32", "int64", "float32", "float64"])
def test_every_operator_against_numpy(dtype):
    """Each operator of the table on its own, on ragged and pitched arrays (both
    the 16-byte packet kernels and the single-element ones), against NumPy on the
    same arrays; zero divisors keep the output's old value."""
    rng = np.random.default_rng(31)
    integer = dtype.startswith("int")
    for shape, pitch in (((33, 64), 64), ((17, 101), 104), ((5, 7), 7)):
        if integer:
            a = rng.integers(-40, 40, shape).astype(dtype)
            b = rng.integers(-5, 6, shape).astype(dtype)
        else:
            a = (rng.standard_normal(shape) * 3).astype(dtype)
            b = np.round(rng.standard_normal(shape) * 2).astype(dtype)
        bodies = {
            "floordiv": (lambda s, t: s // t, True), "mod": (lambda s, t: s % t, True),
            "lt": (lambda s, t: (s < t) * 1, False), "le": (lambda s, t: (s <= t) * 1, False),
            "eq": (lambda s, t: (s == t) * 1, False), "ne": (lambda s, t: (s != t) * 1, False),
            "ge": (lambda s, t: (s >= t) * 1, False), "gt": (lambda s, t: (s > t) * 1, False),
            "logic": (lambda s, t: ((s < t) & (t > 0)) | ((s > 1) ^ (t < 1)), False),
            "not": (lambda s, t: ~(s < t) * s, False),
            "neg_abs": (lambda s, t: abs(-s) - t, False),
            "max_min": (lambda s, t: np.maximum(s, t) - np.minimum(s, t), False),
        }
        if integer:
            bodies.update({
                "bits": (lambda s, t: (s & t) | (s ^ 21), False),
                "shifts": (lambda s, t: (s << 3) + (s >> 2) + (t << 1), False),
                "inv": (lambda s, t: ~s - t, False),
                "pow3": (lambda s, t: s ** 3 + t, False),
                "rfloordiv": (lambda s, t: 1000 // t, True),
                "rmod": (lambda s, t: 1000 % t, True),
            })
        else:
            bodies.update({
                "div": (lambda s, t: s / t, True),
                "pow": (lambda s, t: np.abs(s) ** 1.5 + t, False),
                "rdiv": (lambda s, t: 2.0 / t, True),
            })
        for name, (fn, divides) in bodies.items():
            k = make_elementwise(fn, 2, 2, (4, 16))
            store = torch.full((3, shape[0], pitch), -77, dtype=torch.from_numpy(a).dtype,
                               device="cuda")
            d_a, d_b, d_out = (store[i, :, : shape[1]] for i in range(3))
            d_a.copy_(torch.from_numpy(a))
            d_b.copy_(torch.from_numpy(b))
            k(d_a, d_b, d_out)
            torch.cuda.synchronize()
            got = d_out.cpu().numpy()
            with np.errstate(all="ignore"):
                want = np.asarray(fn(a, b)).astype(dtype)
            if divides:
                want = np.where(b == 0, np.asarray(-77, dtype), want)
            if name == "pow":
                # (powf is within a few ulp; the added tile may cancel most of the power)
                tol = dict(rtol=2e-6, atol=2e-6) if dtype == "float32" else dict(rtol=1e-14,
                                                                                 atol=1e-14)
                np.testing.assert_allclose(got, want, **tol)
            else:
                assert np.array_equal(got, want), (name, shape, dtype)
            if pitch > shape[1]:
                assert (store[2, :, shape[1]:] == -77).all()
