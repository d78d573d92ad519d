"""GPU parity of row bodies (reductions along the rows used again in the same
expression): through the ``@kernel`` front door against the outputs of the
reference simulator (tests/golden) and against NumPy, and hcRowProgram called
directly through the C-ABI.

Tolerances: a row sum is a running value per lane plus a shuffle tree, NumPy's
is pairwise, and exp/log are within a few ulp, so float32 results agree to
2e-6 relative (1e-6 absolute near zero), float64 to 1e-13; row max is exact."""

import numpy as np
import pytest
import torch

from hc_b200 import capi
from hc_b200.hckernel import elementwise as ew
from hc_b200.workloads import make_rowwise
from oracle import workloads as oracle
from tests.gpu_util import finish

pytestmark = pytest.mark.gpu

CASES = oracle.rowwise_cases()
TOL = {"float32": dict(rtol=2e-6, atol=1e-6), "float64": dict(rtol=1e-13, atol=1e-15)}


@pytest.mark.parametrize("case", CASES, ids=lambda c: c[0])
def test_row_bodies_match_reference_and_numpy(golden, case):
    name, fn, count, shape, dtype, group_rows = case
    inputs = oracle.make_elementwise_inputs(count, shape, dtype, seed=8)
    k = make_rowwise(fn, count)
    d_in = [torch.from_numpy(a).cuda() for a in inputs]
    d_out = torch.full(shape, float("nan"), dtype=d_in[0].dtype, device="cuda")
    k(*d_in, d_out, group_rows)
    torch.cuda.synchronize()
    got = d_out.cpu().numpy()
    with np.errstate(all="ignore"):
        np.testing.assert_allclose(got, fn(*inputs), **TOL[dtype])
    np.testing.assert_allclose(got, golden[name], **TOL[dtype])


@pytest.mark.parametrize("shape,pitch", [((33, 4096), 4096), ((7, 1001), 1001), ((300, 36), 40),
                                         ((1, 1), 1), ((9, 8), 8)])
def test_rows_of_many_lengths_and_pitches(shape, pitch):
    """Long rows, rows that are not multiples of 16 bytes, pitched views, fewer
    rows than a CTA holds."""
    rng = np.random.default_rng(shape[0] * 7 + shape[1])
    a = rng.standard_normal(shape).astype(np.float32)
    k = make_rowwise(lambda t: (t - t.mean(axis=1, keepdims=True))
                     / np.sqrt((t * t).sum(axis=1, keepdims=True) + 1.0))
    store = torch.zeros((2, shape[0], pitch), device="cuda")
    d_a, d_out = store[0, :, : shape[1]], store[1, :, : shape[1]]
    d_a.copy_(torch.from_numpy(a))
    k(d_a, d_out, 16)
    torch.cuda.synchronize()
    a64 = a.astype(np.float64)
    want = (a64 - a64.mean(axis=1, keepdims=True)) / np.sqrt((a64 * a64).sum(axis=1, keepdims=True) + 1)
    np.testing.assert_allclose(d_out.cpu().numpy(), want, rtol=1e-5, atol=1e-6)
    if pitch > shape[1]:
        assert float(store[1, :, shape[1]:].abs().max()) == 0.0


def test_row_max_propagates_nan_like_numpy():
    a = np.array([[1.0, np.nan, 3.0, 0.0], [1.0, 2.0, 3.0, 4.0]], np.float32)
    k = make_rowwise(lambda t: t - t.max(axis=1, keepdims=True))
    d_out = torch.zeros((2, 4), device="cuda")
    k(torch.from_numpy(a).cuda(), d_out, 2)
    torch.cuda.synchronize()
    got = d_out.cpu().numpy()
    assert np.all(np.isnan(got[0])) and np.array_equal(got[1], [-3.0, -2.0, -1.0, 0.0])


def _program(code, consts, d_in, d_out, pitch_in=None, pitch_out=None):
    p = capi.HcMapProgram()
    rows, cols = d_out.shape
    p.inputs[0], p.inPitch[0] = d_in.data_ptr(), pitch_in or cols
    p.out, p.outPitch, p.rows, p.cols, p.nInputs = d_out.data_ptr(), pitch_out or cols, rows, cols, 1
    p.nInstr = len(code)
    for i, ins in enumerate(code):
        p.code[i] = ins
    for i, value in enumerate(consts):
        p.consts[i] = value
    return p


@pytest.mark.parametrize("variant", [0, 3, 2, 1], ids=["auto", "held", "held256", "walked"])
@pytest.mark.parametrize("dtype,cols", [("float32", 4096), ("float32", 4092), ("float32", 2048),
                                        ("float32", 1028), ("float32", 1024), ("float64", 2048),
                                        ("float64", 1030), ("float64", 514), ("float64", 512)])
def test_rows_held_in_registers_and_rows_walked_agree(hc, variant, dtype, cols):
    """Rows of 257..1024 16-byte packets that fill most of a CTA's slots take the
    kernel that holds the row in registers (eight packets per thread on 64, 96 or
    128 threads; row_variant 3 holds whatever the fill, 2 uses 256 threads with
    four packets each beyond 512 packets), others (and all rows under row_variant
    1) the warp that walks the row once per pass.  Two programs: log-softmax (max,
    sum, a uniform prologue), and a variance normalisation that parks values in
    all three temporaries (more than 48 KB of dynamic shared memory for rows
    beyond 768 packets)."""
    rows = 19
    rng = np.random.default_rng(cols)
    x = rng.standard_normal((rows, cols)).astype(dtype)
    x[3, 5] = 9.0
    d_x = torch.from_numpy(x).cuda()
    d_out = torch.full((rows, cols), float("nan"), dtype=d_x.dtype, device="cuda")
    kind = capi.HC_F32 if dtype == "float32" else capi.HC_F64
    u, c0, s0, t0 = ew.UNIFORM, ew.SRC_CONST, ew.SRC_SCALAR, ew.SRC_TEMP
    tol = dict(rtol=3e-6, atol=2e-6) if dtype == "float32" else dict(rtol=1e-13, atol=1e-14)
    x64 = x.astype(np.float64)
    hc.set_option("row_variant", variant)
    try:
        log_softmax = [
            ew.LOAD | 0 << 8, ew.RMAX | 0 << 8,
            ew.LOAD | 0 << 8, ew.SUB | s0 << 8, ew.EXP, ew.RSUM | 1 << 8,
            ew.LOAD | u | (s0 + 1) << 8, ew.LOG | u, ew.SET | u | 2 << 8,
            ew.LOAD | 0 << 8, ew.SUB | s0 << 8, ew.SUB | (s0 + 2) << 8,
        ]
        hc.row_program(_program(log_softmax, [], d_x, d_out), kind)
        finish(hc)
        shifted = x64 - x64.max(axis=1, keepdims=True)
        want = shifted - np.log(np.exp(shifted).sum(axis=1, keepdims=True))
        np.testing.assert_allclose(d_out.cpu().numpy(), want, **tol)

        # d = x - mean; t0 = d; t1 = d*d; t2 = |d|; out = t0 / sqrt(sum(t1)/N) + t2 * 0
        normalise = [
            ew.LOAD | 0 << 8, ew.RSUM | 0 << 8,
            ew.LOAD | u | s0 << 8, ew.MUL | u | c0 << 8, ew.SET | u | 1 << 8,
            ew.LOAD | 0 << 8, ew.SUB | (s0 + 1) << 8, ew.SAVE0, ew.MUL | t0 << 8, ew.RSUM | 2 << 8,
            ew.LOAD | u | (s0 + 2) << 8, ew.MUL | u | c0 << 8, ew.SQRT | u, ew.SET | u | 3 << 8,
            ew.LOAD | 0 << 8, ew.SUB | (s0 + 1) << 8, ew.SAVE0, ew.MUL | t0 << 8, ew.SAVE0 + 1,
            ew.LOAD | t0 << 8, ew.ABS, ew.SAVE0 + 2,
            ew.MUL | (c0 + 1) << 8, ew.SAVE0 + 2,
            ew.LOAD | t0 << 8, ew.DIV | (s0 + 3) << 8, ew.ADD | (t0 + 2) << 8,
        ]
        d_out.fill_(float("nan"))
        hc.row_program(_program(normalise, [1.0 / cols, 0.0], d_x, d_out), kind)
        finish(hc)
        d = x64 - x64.mean(axis=1, keepdims=True)
        want = d / np.sqrt((d * d).sum(axis=1, keepdims=True) / cols)
        np.testing.assert_allclose(d_out.cpu().numpy(), want, **tol)
    finally:
        hc.set_option("row_variant", 0)


@pytest.mark.parametrize("dtype,cols", [("float32", 4096), ("float32", 1540), ("float64", 1030)])
def test_more_rows_than_resident_ctas(hc, dtype, cols):
    """Several waves of CTAs of the held-row kernel: every row must come out as
    its own centred self."""
    rows = 1900
    rng = np.random.default_rng(rows + cols)
    x = rng.standard_normal((rows, cols)).astype(dtype) + np.arange(rows, dtype=dtype)[:, None]
    d_x = torch.from_numpy(x).cuda()
    d_out = torch.full((rows, cols), float("nan"), dtype=d_x.dtype, device="cuda")
    centre = [ew.LOAD | 0 << 8, ew.RSUM | 0 << 8,
              ew.LOAD | ew.UNIFORM | ew.SRC_SCALAR << 8, ew.MUL | ew.UNIFORM | ew.SRC_CONST << 8,
              ew.SET | ew.UNIFORM | 1 << 8,
              ew.LOAD | 0 << 8, ew.SUB | (ew.SRC_SCALAR + 1) << 8]
    hc.row_program(_program(centre, [1.0 / cols], d_x, d_out),
                   capi.HC_F32 if dtype == "float32" else capi.HC_F64)
    finish(hc)
    x64 = x.astype(np.float64)
    # Row r lies around the value r, so a row taken from the wrong buffer is off
    # by at least 1; the float32 mean of 4096 values near 1900 is good to ~5e-4.
    tol = dict(rtol=0, atol=2e-3) if dtype == "float32" else dict(rtol=0, atol=1e-10)
    np.testing.assert_allclose(d_out.cpu().numpy(), x64 - x64.mean(axis=1, keepdims=True), **tol)


def test_held_rows_respect_pitches(hc):
    """Pitched input and output (multiples of 16 bytes) with the held-row kernel:
    nothing outside the rows is written."""
    rows, cols, pitch = 11, 2044, 2052
    rng = np.random.default_rng(2)
    store = torch.zeros((2, rows, pitch), device="cuda")
    x = rng.standard_normal((rows, cols)).astype(np.float32)
    store[0, :, :cols].copy_(torch.from_numpy(x))
    d_out = store[1, :, :cols]
    centre = [ew.LOAD | 0 << 8, ew.RSUM | 0 << 8,
              ew.LOAD | ew.UNIFORM | ew.SRC_SCALAR << 8, ew.MUL | ew.UNIFORM | ew.SRC_CONST << 8,
              ew.SET | ew.UNIFORM | 1 << 8,
              ew.LOAD | 0 << 8, ew.SUB | (ew.SRC_SCALAR + 1) << 8]
    hc.row_program(_program(centre, [1.0 / cols], store[0], d_out, pitch, pitch), capi.HC_F32)
    finish(hc)
    want = x.astype(np.float64) - x.astype(np.float64).mean(axis=1, keepdims=True)
    np.testing.assert_allclose(d_out.cpu().numpy(), want, rtol=3e-6, atol=2e-6)
    assert float(store[1, :, cols:].abs().max()) == 0.0


def test_row_program_through_the_c_abi(hc):
    """Variance-normalise rows in float64: s0 = sum(x); s1 = sum((x - s0/N)^2);
    out = (x - s0/N) / sqrt(s1/N)."""
    rng = np.random.default_rng(4)
    rows, cols = 21, 50
    x = rng.standard_normal((rows, cols))
    d_x = torch.from_numpy(x).cuda()
    d_out = torch.zeros((rows, cols), dtype=torch.float64, device="cuda")
    p = capi.HcMapProgram()
    p.inputs[0], p.inPitch[0], p.outPitch = d_x.data_ptr(), cols, cols
    p.out, p.rows, p.cols, p.nInputs = d_out.data_ptr(), rows, cols, 1
    c0, s0, s1, t0 = ew.SRC_CONST, ew.SRC_SCALAR, ew.SRC_SCALAR + 1, ew.SRC_TEMP
    program = [
        ew.LOAD | 0 << 8, ew.RSUM | 0 << 8,                                   # s0 = sum(x)
        ew.LOAD | s0 << 8, ew.MUL | c0 << 8, ew.RSUB | 0 << 8,                # x - s0/N
        ew.SAVE0, ew.MUL | t0 << 8, ew.RSUM | 1 << 8,                         # s1 = sum(d*d)
        ew.LOAD | s1 << 8, ew.MUL | c0 << 8, ew.SQRT, ew.SAVE0,               # t0 = sqrt(s1/N)
        ew.LOAD | s0 << 8, ew.MUL | c0 << 8, ew.RSUB | 0 << 8, ew.DIV | t0 << 8,
    ]
    p.nInstr = len(program)
    for i, ins in enumerate(program):
        p.code[i] = ins
    p.consts[0] = 1.0 / cols
    hc.row_program(p, capi.HC_F64)
    finish(hc)
    mean = x.sum(axis=1, keepdims=True) * (1.0 / cols)
    want = (x - mean) / np.sqrt(((x - mean) ** 2).sum(axis=1, keepdims=True) * (1.0 / cols))
    np.testing.assert_allclose(d_out.cpu().numpy(), want, rtol=1e-13)

    # The same with the per-row values computed once per row, in uniform prologues:
    # s2 = s0/N before the second pass, s3 = sqrt(s1/N) before the third.
    u = ew.UNIFORM
    uniform = [
        ew.LOAD | 0 << 8, ew.RSUM | 0 << 8,
        ew.LOAD | u | s0 << 8, ew.MUL | u | c0 << 8, ew.SET | u | 2 << 8,
        ew.LOAD | 0 << 8, ew.SUB | (ew.SRC_SCALAR + 2) << 8, ew.SAVE0, ew.MUL | t0 << 8,
        ew.RSUM | 1 << 8,
        ew.LOAD | u | s1 << 8, ew.MUL | u | c0 << 8, ew.SQRT | u, ew.SET | u | 3 << 8,
        ew.LOAD | 0 << 8, ew.SUB | (ew.SRC_SCALAR + 2) << 8, ew.DIV | (ew.SRC_SCALAR + 3) << 8,
    ]
    q = capi.HcMapProgram()
    q.inputs[0], q.inPitch[0], q.outPitch = d_x.data_ptr(), cols, cols
    d_out2 = torch.zeros_like(d_out)
    q.out, q.rows, q.cols, q.nInputs, q.nInstr = d_out2.data_ptr(), rows, cols, 1, len(uniform)
    for i, ins in enumerate(uniform):
        q.code[i] = ins
    q.consts[0] = 1.0 / cols
    hc.row_program(q, capi.HC_F64)
    finish(hc)
    assert torch.equal(d_out2, d_out)  # the same operations on the same values
    q.code[5] = ew.LOAD | u | s0 << 8  # a uniform instruction in the middle of a pass
    q.code[4] = ew.LOAD | 0 << 8
    with pytest.raises(RuntimeError, match="not at the start of a pass"):
        hc.row_program(q, capi.HC_F64)
    q.code[4], q.code[5] = ew.SET | u | 2 << 8, ew.LOAD | 0 << 8
    q.code[2] = ew.LOAD | u | 0 << 8  # an array as a uniform operand
    with pytest.raises(RuntimeError, match="only constants and row scalars"):
        hc.row_program(q, capi.HC_F64)
    q.code[2] = ew.LOAD | u | s0 << 8
    q.code[0] = ew.LOAD | u | c0 << 8  # hcMapElements knows no uniform instructions
    with pytest.raises(RuntimeError, match="uniform instructions belong to hcRowProgram"):
        hc.map_elements(q, capi.HC_F64)

    # Malformed programs are refused before anything is launched.
    p.code[len(program) - 1] = ew.RSUM | 2 << 8
    with pytest.raises(RuntimeError, match="ends in a reduction"):
        hc.row_program(p, capi.HC_F64)
    p.code[len(program) - 1] = ew.DIV | t0 << 8
    p.code[2] = ew.ADD | s0 << 8
    with pytest.raises(RuntimeError, match="after a reduction must load"):
        hc.row_program(p, capi.HC_F64)
    p.code[2] = ew.LOAD | (ew.SRC_SCALAR + 3) << 8
    with pytest.raises(RuntimeError, match="not written yet"):
        hc.row_program(p, capi.HC_F64)
    p.code[2] = ew.LOAD | s0 << 8
    p.code[6] = ew.MUL | (t0 + 1) << 8
    with pytest.raises(RuntimeError, match="not written yet"):
        hc.row_program(p, capi.HC_F64)
    p.code[6] = ew.MUL | t0 << 8
    p.code[1] = ew.RSUM | 7 << 8
    with pytest.raises(RuntimeError, match="row scalar 7"):
        hc.row_program(p, capi.HC_F64)
    p.code[1] = ew.RSUM | 0 << 8
    with pytest.raises(RuntimeError, match="row reductions belong to hcRowProgram"):
        hc.map_elements(p, capi.HC_F64)
    p.nInputs = 3
    with pytest.raises(RuntimeError, match="inputs"):
        hc.row_program(p, capi.HC_F64)


@pytest.mark.parametrize("cols", [4096, 3072, 2048, 1000, 777])
def test_random_row_bodies_against_numpy(cols):
    """Random row bodies through the front door on rows that are held by 128, 96
    and 64 threads, on walked rows and on rows that are no multiple of 16 bytes.
    The float32 kernel must be as close to the float64 value of the expression
    as NumPy's own float32 evaluation is, up to a small factor (sum orders and
    a few ulp in exp differ; anything structural is off by far more)."""
    rng = np.random.default_rng(cols)
    rows, done = 21, 0
    while done < 12:
        count = int(rng.integers(1, 3))
        fn, text = oracle.random_row_expression(rng, count)
        k = make_rowwise(fn, count)
        inputs = oracle.make_elementwise_inputs(count, (rows, cols), "float32", seed=done + cols)
        d_in = [torch.from_numpy(a).cuda() for a in inputs]
        d_out = torch.full((rows, cols), float("nan"), device="cuda")
        try:
            k(*d_in, d_out, 8)
        except Exception as e:  # noqa: BLE001 - too long for the machine: not this test's subject
            assert "more than" in str(e), text
            continue
        torch.cuda.synchronize()
        done += 1
        got = d_out.cpu().numpy().astype(np.float64)
        with np.errstate(all="ignore"):
            single = fn(*inputs).astype(np.float64)
            truth = fn(*[a.astype(np.float64) for a in inputs])
        scale = np.abs(truth).max(axis=1, keepdims=True) + 1e-30
        ours = (np.abs(got - truth) / scale).max()
        numpys = (np.abs(single - truth) / scale).max()
        assert ours <= 8 * numpys + 2e-6, (text, ours, numpys)
