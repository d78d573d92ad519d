"""GPU parity of the mapped (gather/scatter) kernels: the reference's
implicit-GEMM convolution (python/hckernel/tests/test_examples.py:168-258) run
through the ``@kernel`` front door against the outputs of the reference
simulator (tests/golden), larger cases against the oracle, and hcMappedGemm
called directly through the C-ABI.

Tolerances: the kernel sums each dot product over all of K in one pass, in the
element type, while the reference adds np.dot results of K blocks; float64
agrees to 1e-12, float32 to 1e-5 relative (plus 1e-5 absolute near zero)."""

import ctypes

import numpy as np
import pytest
import torch

from hc_b200 import capi
from hc_b200.hckernel.kernel import *  # noqa: F401,F403
from hc_b200.workloads import make_conv
from oracle import workloads as oracle
from tests.gpu_util import finish

pytestmark = pytest.mark.gpu

TOL = {"float32": dict(rtol=1e-5, atol=1e-5), "float64": dict(rtol=1e-12, atol=1e-12)}


def run_conv(x, f, out_shape, stride, tiles, canary=0.0):
    tn, tnf, kb = tiles
    conv = make_conv(stride).parametrize({sym.TN: tn, sym.TNF: tnf, sym.KB: kb})
    d_x, d_f = torch.from_numpy(x).cuda(), torch.from_numpy(f).cuda()
    d_out = torch.full(out_shape, canary, dtype=d_x.dtype, device="cuda")
    conv(d_x, d_f, d_out)
    torch.cuda.synchronize()
    return d_out.cpu().numpy()


@pytest.mark.parametrize("case", oracle.conv_golden_cases(), ids=lambda c: c[0])
def test_conv_matches_the_reference_simulator(golden, case):
    name, x_shape, f_shape, stride, dtype, tiles = case
    x, f = oracle.make_conv_inputs(x_shape, f_shape, dtype)
    out = run_conv(x, f, oracle.conv_out_shape(x_shape, f_shape, stride), stride, tiles)
    np.testing.assert_allclose(out, golden[name], **TOL[dtype])


@pytest.mark.parametrize("dtype", ["float32", "float64"])
@pytest.mark.parametrize("tiles", [(8, 8, 16), (16, 24, 32), (33, 64, 16), (5, 80, 24)])
def test_conv_larger_cases_match_the_oracle(dtype, tiles):
    # Ragged in every tile dimension; (5, 80, ..) walks a tile wider than the
    # 64 columns one pass of the kernel covers.
    x_shape, f_shape, stride = (37, 6, 13, 13), (70, 6, 3, 3), 2
    x, f = oracle.make_conv_inputs(x_shape, f_shape, dtype, seed=11)
    out_shape = oracle.conv_out_shape(x_shape, f_shape, stride)
    out = run_conv(x, f, out_shape, stride, tiles)
    expect = np.zeros(out_shape, dtype)
    oracle.conv_implicit_gemm(x, f, expect, stride, *tiles)
    np.testing.assert_allclose(out, expect, **TOL[dtype])
    np.testing.assert_allclose(out, oracle.conv_direct(x, f, stride), rtol=1e-4, atol=1e-4)


@pytest.mark.parametrize("tiles", [(8, 8, 16), (5, 24, 16), (16, 64, 16), (32, 64, 16)])
def test_stacked_groups_give_what_single_groups_give(tiles):
    """Consecutive output positions share their filter tile, so one CTA computes
    up to eight of them (fewer for taller tiles); bit for bit the result must be
    what one CTA per work-group produces."""
    from hc_b200.hckernel.autotune import TunedParams

    x_shape, f_shape = (19, 5, 11, 11), (40, 5, 3, 3)
    x, f = oracle.make_conv_inputs(x_shape, f_shape, "float32", seed=12)
    out_shape = oracle.conv_out_shape(x_shape, f_shape, 1)
    tn, tnf, kb = tiles
    conv = make_conv(1).parametrize({sym.TN: tn, sym.TNF: tnf, sym.KB: kb})
    d_x, d_f = torch.from_numpy(x).cuda(), torch.from_numpy(f).cuda()
    stacked = torch.full(out_shape, -3.0, device="cuda")
    single = torch.full(out_shape, -3.0, device="cuda")
    conv(d_x, d_f, stacked)
    conv.parametrize(TunedParams({}, {"mapped_stack": 1}))(d_x, d_f, single)
    torch.cuda.synchronize()
    assert torch.equal(stacked, single)
    # Stacks kept within 64 rows (the float default goes up to 128-row pieces).
    short = torch.full(out_shape, -3.0, device="cuda")
    conv.parametrize(TunedParams({}, {"mapped_stack": 2}))(d_x, d_f, short)
    torch.cuda.synchronize()
    assert torch.equal(short, single)
    np.testing.assert_allclose(stacked.cpu().numpy(), oracle.conv_direct(x, f, 1),
                               rtol=1e-4, atol=1e-4)


def test_elements_no_group_writes_stay_untouched():
    # A 5x8 image: positions run over W_OUT on the H axis (test_examples.py:
    # 237-240), so output columns 4..6 are never written - by the reference or here.
    x_shape, f_shape = (2, 2, 5, 8), (3, 2, 2, 2)
    x, f = oracle.make_conv_inputs(x_shape, f_shape, "float64")
    out_shape = oracle.conv_out_shape(x_shape, f_shape, 1)
    out = run_conv(x, f, out_shape, 1, (8, 8, 16), canary=-7.0)
    expect = np.full(out_shape, -7.0)
    oracle.conv_implicit_gemm(x, f, expect, 1)
    assert np.all(expect[..., 4:] == -7.0) and np.all(out[..., 4:] == -7.0)
    np.testing.assert_allclose(out, expect, **TOL["float64"])


def test_non_contiguous_arguments():
    x_shape, f_shape = (6, 3, 9, 9), (10, 3, 3, 3)
    x, f = oracle.make_conv_inputs(x_shape, f_shape, "float32")
    out_shape = oracle.conv_out_shape(x_shape, f_shape, 1)
    conv = make_conv(1)
    big = torch.zeros((6, 3, 9, 12), device="cuda")
    d_x = big[..., :9]  # row pitch 12
    d_x.copy_(torch.from_numpy(x))
    d_f = torch.from_numpy(f).cuda()
    d_out = torch.zeros(out_shape[:2] + out_shape[:1:-1], device="cuda").permute(0, 1, 3, 2)
    conv(d_x, d_f, d_out)
    conv(d_x.contiguous(), d_f, d_out2 := torch.zeros(out_shape, device="cuda"))
    torch.cuda.synchronize()
    expect = np.zeros(out_shape, np.float32)
    oracle.conv_implicit_gemm(x, f, expect, 1)
    np.testing.assert_allclose(d_out.cpu().numpy(), expect, **TOL["float32"])
    assert torch.equal(d_out.contiguous(), d_out2)  # one plan, tables per stride set


def test_autotune_searches_the_tile_sizes():
    """For this family the symbolic tunables decide the launch, so autotune
    times a grid of them (docs/langref.md:471-586 of the reference describes the
    API; the reference does not implement it)."""
    from hc_b200.hckernel.autotune import autotune

    x_shape, f_shape = (16, 8, 20, 20), (32, 8, 3, 3)
    x, f = oracle.make_conv_inputs(x_shape, f_shape, "float32")
    out_shape = oracle.conv_out_shape(x_shape, f_shape, 1)
    d_x, d_f = torch.from_numpy(x).cuda(), torch.from_numpy(f).cuda()
    d_out = torch.zeros(out_shape, device="cuda")
    conv = make_conv(1)
    tuned = autotune(conv, d_x, d_f, d_out, repeats=3)
    assert set(tuned) == {sym.TN, sym.TNF, sym.KB}
    # Tile sizes were really compared (KB only restructures the body's K loop
    # and is not timed separately), and the fastest launch was taken.
    assert len(tuned.timings) >= 9
    import json
    best = json.dumps({str(k): int(v) for k, v in tuned.items()}, sort_keys=True)
    assert tuned.timings[best] == min(tuned.timings.values())
    d_out.zero_()
    conv.parametrize(tuned)(d_x, d_f, d_out)
    torch.cuda.synchronize()
    np.testing.assert_allclose(d_out.cpu().numpy(), oracle.conv_direct(x, f, 1),
                               rtol=1e-4, atol=1e-4)


def _operand(array, table, lin, origins):
    op = capi.HcMappedOperand()
    op.base = array.data_ptr()
    op.map, op.lin, op.origins = table.data_ptr(), lin.data_ptr(), origins.data_ptr()
    rank = array.dim()
    for d in range(4):
        op.shape[d] = array.shape[d] if d < rank else 1
        op.stride[d] = array.stride(d) if d < rank else 0
        column = table[:, d]
        op.lo[d] = int(column.min()) if column.numel() else 0
        op.hi[d] = int(column.max()) if column.numel() else 0
    return op


def test_mapped_gemm_through_the_c_abi(hc):
    """Transposed gather, shifted scatter, edge groups: out[g*4 + a + 1, b] =
    sum_k x[k, g*4 + a] * f[k, b] with tiles hanging over every edge."""
    rng = np.random.default_rng(3)
    m, k, n, tm = 10, 7, 5, 4
    x = rng.standard_normal((k, m))
    f = rng.standard_normal((k, n))
    groups = 3
    aa, kk = np.indices((tm, k))
    x_map = np.stack([kk, aa, 0 * aa, 0 * aa], axis=-1).reshape(-1, 4)         # x[k, a]
    kk, bb = np.indices((k, n + 2))                                            # tile wider than f
    f_map = np.stack([kk, bb, 0 * kk, 0 * kk], axis=-1).reshape(-1, 4)
    aa, bb = np.indices((tm, n + 2))
    o_map = np.stack([aa + 1, bb, 0 * aa, 0 * aa], axis=-1).reshape(-1, 4)
    x_org = np.array([[0, g * tm, 0, 0] for g in range(groups)])
    f_org = np.zeros((groups, 4), np.int64)
    o_org = np.array([[g * tm, 0, 0, 0] for g in range(groups)])

    def i32(a):
        return torch.from_numpy(np.ascontiguousarray(a.astype(np.int32))).cuda()

    d_x, d_f = torch.from_numpy(x).cuda(), torch.from_numpy(f).cuda()
    d_out = torch.full((m, n), -1.0, dtype=torch.float64, device="cuda")
    tables = []
    for arr, mp, org in ((d_x, x_map, x_org), (d_f, f_map, f_org), (d_out, o_map, o_org)):
        stride = np.array([arr.stride(d) if d < arr.dim() else 0 for d in range(4)])
        tables.append((i32(mp), i32(mp @ stride), i32(org)))
    ops = [_operand(arr, *t) for arr, t in zip((d_x, d_f, d_out), tables)]
    hc.mapped_gemm(ops[0], ops[1], ops[2], groups, tm, n + 2, k, capi.HC_F64)
    finish(hc)
    expect = np.full((m, n), -1.0)
    expect[1:] = (x.T @ f)[: m - 1]
    np.testing.assert_allclose(d_out.cpu().numpy(), expect, rtol=1e-12, atol=1e-12)

    # The same product with the operand tables in transposed tile order.
    d_out.fill_(-1.0)
    flipped = []
    for arr, (mp, org), (rows, cols) in ((d_x, (x_map, x_org), (tm, k)),
                                        (d_f, (f_map, f_org), (k, n + 2))):
        stride = np.array([arr.stride(d) if d < arr.dim() else 0 for d in range(4)])
        mp_t = mp.reshape(rows, cols, 4).transpose(1, 0, 2).reshape(-1, 4)
        flipped.append((i32(mp_t), i32(mp_t @ stride), i32(org)))
    ops_t = [_operand(arr, *t) for arr, t in zip((d_x, d_f), flipped)]
    for op in ops_t:
        op.transposed = 1
    hc.mapped_gemm(ops_t[0], ops_t[1], ops[2], groups, tm, n + 2, k, capi.HC_F64)
    finish(hc)
    np.testing.assert_allclose(d_out.cpu().numpy(), expect, rtol=1e-12, atol=1e-12)
    # All three groups read the same f tile: tell the kernel, which then computes
    # two groups per CTA (and the odd last one alone) - same result.
    for run in (2, 8):
        d_out.fill_(-1.0)
        ops[1].sharedRun = run
        hc.mapped_gemm(ops[0], ops[1], ops[2], groups, tm, n + 2, k, capi.HC_F64)
        finish(hc)
        np.testing.assert_allclose(d_out.cpu().numpy(), expect, rtol=1e-12, atol=1e-12)
    ops[1].sharedRun = 0
    ops[2].transposed = 1
    with pytest.raises(RuntimeError, match="row-major"):
        hc.mapped_gemm(ops[0], ops[1], ops[2], groups, tm, n + 2, k, capi.HC_F64)
    ops[2].transposed = 0

    # Argument errors come back as error codes with a message, not as faults.
    with pytest.raises(RuntimeError, match="unsupported dtype"):
        hc.mapped_gemm(ops[0], ops[1], ops[2], groups, tm, n + 2, k, capi.HC_BF16)
    bad = _operand(d_out, *tables[2])
    bad.map = tables[2][0].data_ptr() + 4
    with pytest.raises(RuntimeError, match="not 16-byte aligned"):
        hc.mapped_gemm(ops[0], ops[1], bad, groups, tm, n + 2, k, capi.HC_F64)
    hc.mapped_gemm(ops[0], ops[1], ops[2], 0, tm, n + 2, k, capi.HC_F64)  # no groups: no-op
    # K == 0: empty operand tiles (their element tables may be absent), the
    # products are empty sums, so every mapped output element becomes zero.
    d_out.fill_(-1.0)
    empty_x, empty_f = _operand(d_x, *tables[0]), _operand(d_f, *tables[1])
    for op in (empty_x, empty_f):
        op.map, op.lin = None, None
    hc.mapped_gemm(empty_x, empty_f, ops[2], groups, tm, n + 2, 0, capi.HC_F64)
    finish(hc)
    zeros = np.full((m, n), -1.0)
    zeros[1:] = 0.0
    assert np.array_equal(d_out.cpu().numpy(), zeros)
    empty_x.origins = None
    with pytest.raises(RuntimeError, match="null origins"):
        hc.mapped_gemm(empty_x, empty_f, ops[2], groups, tm, n + 2, 0, capi.HC_F64)
    assert ctypes.sizeof(capi.HcMappedOperand) == 120
