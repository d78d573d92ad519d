"""GPU parity tests: every CUDA kernel, called through the C-ABI
(``include/hc_b200_kernels.h`` via ctypes), against the CPU oracle and the
committed golden vectors.

Tolerances (the reference's own tests use exact equality on float64 toy
inputs, which no GPU reduction order can reproduce, so the bounds are stated
here):

* copies and row max: bit-exact;
* float32 tiled GEMM: |got - oracle| <= 1e-5 * sum_k |a||b| per element;
* softmax: |got - oracle| <= 1e-6 + 1e-5 * |oracle|;
* row sum: |got - float64 sum| <= 1e-5 * sum |x| per row;
* bf16 GEMMs (fp32 accumulation, bf16 output): relative 1e-2 against the
  oracle plus an absolute term of 1e-2 of the per-element sum_k |a||b| bound
  scaled to bf16 resolution;
* float64 variants: 1e-12 relative.
"""

import numpy as np
import pytest
import torch

from hc_b200 import capi
from oracle import workloads as oracle
from tests.gpu_util import dev, dev_bf16, empty_like_dev, finish, host_bf16

pytestmark = pytest.mark.gpu


# ---- copy ----------------------------------------------------------------------
COPY_SHAPES = [(1, 27), (1, 72), (1, 128), (10, 20), (111, 813), (256, 64), (256, 1024)]


@pytest.mark.parametrize("shape", COPY_SHAPES)
def test_copy2d_int32(hc, shape, golden):
    src = np.arange(shape[0] * shape[1], dtype=np.int32).reshape(shape)
    d_src, d_dst = dev(src), empty_like_dev(shape, torch.int32)
    hc.copy2d(d_src.data_ptr(), d_dst.data_ptr(), shape[0], shape[1], shape[1], shape[1], 4)
    finish(hc)
    got = d_dst.cpu().numpy()
    expect = np.zeros_like(src)
    oracle.copy2d(src, expect, (4, 16))
    assert np.array_equal(got, expect)
    key = f"copy_{shape[0]}x{shape[1]}"
    if key in golden:
        assert np.array_equal(got, golden[key])


@pytest.mark.parametrize("elem", [1, 2, 8])
def test_copy2d_strided_views(hc, elem):
    # A (37 x 53) window of a larger matrix into a window of another one:
    # pitches differ from the width and the bases are not 16-byte aligned.
    dtype = {1: torch.uint8, 2: torch.int16, 8: torch.int64}[elem]
    big = torch.randint(0, 100, (64, 80), device="cuda").to(dtype)
    out = torch.zeros((50, 70), dtype=dtype, device="cuda")
    torch.cuda.synchronize()
    src = big[3:40, 5:58]
    dst = out[7:44, 9:62]
    hc.copy2d(src.data_ptr(), dst.data_ptr(), 37, 53, 80, 70, elem)
    finish(hc)
    expect = torch.zeros_like(out)
    expect[7:44, 9:62] = src
    assert torch.equal(out, expect)


def test_copy2d_empty_and_errors(hc):
    hc.copy2d(0, 0, 0, 16, 16, 16, 4)  # nothing to do
    with pytest.raises(capi.HcError, match="unsupported element size"):
        hc.copy2d(0, 0, 4, 4, 4, 4, 3)
    with pytest.raises(capi.HcError, match="invalid shape"):
        hc.copy2d(0, 0, 4, 8, 4, 8, 4)  # pitch smaller than the row


# ---- softmax ---------------------------------------------------------------------
def _softmax_check(got, expect):
    assert np.all(np.abs(got - expect) <= 1e-6 + 1e-5 * np.abs(expect))


def test_softmax_golden_rows_of_4096(hc, golden):
    (x,) = oracle.make_inputs("softmax", shape=(48, 4096))
    d_x, d_y = dev(x), empty_like_dev(x.shape, torch.float32)
    hc.softmax_rows(d_x.data_ptr(), d_y.data_ptr(), 48, 4096, 4096, 4096)
    finish(hc)
    _softmax_check(d_y.cpu().numpy(), golden["cfg2_softmax_48x4096"])


def test_softmax_golden_ragged(hc, golden):
    (x,) = oracle.make_inputs("softmax", shape=(30, 25))
    d_x, d_y = dev(x), empty_like_dev(x.shape, torch.float32)
    hc.softmax_rows(d_x.data_ptr(), d_y.data_ptr(), 30, 25, 25, 25)
    finish(hc)
    _softmax_check(d_y.cpu().numpy(), golden["cfg2_softmax_30x25"])


def test_softmax_reference_vector_f64(hc, golden):
    m, n = 30, 25
    a = 2 * np.arange(m * n).reshape(m, n) / (m * n)
    d_x, d_y = dev(a), empty_like_dev(a.shape, torch.float64)
    hc.softmax_rows(d_x.data_ptr(), d_y.data_ptr(), m, n, n, n, capi.HC_F64)
    finish(hc)
    np.testing.assert_allclose(d_y.cpu().numpy(), golden["kat_softmax_f64"], rtol=1e-12, atol=0)


@pytest.mark.parametrize(
    "rows,cols",
    [(5, 4), (33, 128), (17, 132), (64, 256), (9, 1000), (130, 1024), (40, 2048), (7, 3000),
     (600, 4096), (3, 4100), (2, 50000), (1, 70001)],
)
def test_softmax_shapes(hc, rows, cols):
    rng = np.random.default_rng(rows * 100003 + cols)
    x = (rng.standard_normal((rows, cols)) * 3).astype(np.float32)
    d_x, d_y = dev(x), empty_like_dev(x.shape, torch.float32)
    hc.softmax_rows(d_x.data_ptr(), d_y.data_ptr(), rows, cols, cols, cols)
    finish(hc)
    expect = np.zeros_like(x)
    oracle.softmax_rows(x, expect, 8)
    _softmax_check(d_y.cpu().numpy(), expect)


def test_softmax_strided_and_untouched_padding(hc):
    rng = np.random.default_rng(11)
    x = rng.standard_normal((20, 512)).astype(np.float32)
    d_x = dev(x)
    d_y = torch.full((20, 640), -5.0, device="cuda")
    torch.cuda.synchronize()
    hc.softmax_rows(d_x[:, :384].data_ptr(), d_y.data_ptr(), 20, 384, 512, 640)
    finish(hc)
    got = d_y.cpu().numpy()
    expect = np.zeros((20, 384), np.float32)
    oracle.softmax_rows(np.ascontiguousarray(x[:, :384]), expect, 8)
    _softmax_check(got[:, :384], expect)
    assert np.all(got[:, 384:] == -5.0)


def test_softmax_extreme_values(hc):
    x = np.zeros((4, 256), np.float32)
    x[0, :] = 1e4          # all equal, huge: must not overflow
    x[1, 5] = 88.0         # one dominant entry
    x[2, :] = -1e4
    x[3, ::2] = -np.inf    # -inf entries contribute zero
    d_x, d_y = dev(x), empty_like_dev(x.shape, torch.float32)
    hc.softmax_rows(d_x.data_ptr(), d_y.data_ptr(), 4, 256, 256, 256)
    finish(hc)
    expect = np.zeros_like(x)
    oracle.softmax_rows(x, expect, 8)
    _softmax_check(d_y.cpu().numpy(), expect)


# ---- reductions --------------------------------------------------------------------
def _reduce_check(x, got_sum, got_max, golden_sum=None, golden_max=None):
    expect_max = x.max(axis=1)
    assert np.array_equal(got_max, expect_max)  # bit-exact
    if golden_max is not None:
        assert np.array_equal(got_max, golden_max)
    exact = x.astype(np.float64).sum(axis=1)
    bound = 1e-5 * np.abs(x).astype(np.float64).sum(axis=1)
    assert np.all(np.abs(got_sum.astype(np.float64) - exact) <= bound)
    if golden_sum is not None:
        assert np.all(np.abs(got_sum.astype(np.float64) - golden_sum.astype(np.float64)) <= 2 * bound)


@pytest.mark.parametrize("shape", [(300, 8192), (37, 101)])
def test_reduce_rows_golden(hc, golden, shape):
    (x,) = oracle.make_inputs("reduce", shape=shape)
    d_x = dev(x)
    d_s, d_m = empty_like_dev((shape[0],), torch.float32), empty_like_dev((shape[0],), torch.float32)
    hc.reduce_rows(d_x.data_ptr(), d_s.data_ptr(), d_m.data_ptr(), shape[0], shape[1], shape[1])
    finish(hc)
    tag = f"{shape[0]}x{shape[1]}"
    _reduce_check(x, d_s.cpu().numpy(), d_m.cpu().numpy(), golden[f"cfg3_sum_{tag}"],
                  golden[f"cfg3_max_{tag}"])


@pytest.mark.parametrize(
    "rows,cols", [(1, 1), (3, 7), (2000, 8192), (5000, 100), (1500, 36), (2, 1 << 20), (1300, 4099)]
)
def test_reduce_rows_shapes(hc, rows, cols):
    rng = np.random.default_rng(rows * 7 + cols)
    x = rng.uniform(-10, 10, (rows, cols)).astype(np.float32)
    d_x = dev(x)
    d_s, d_m = empty_like_dev((rows,), torch.float32), empty_like_dev((rows,), torch.float32)
    hc.reduce_rows(d_x.data_ptr(), d_s.data_ptr(), d_m.data_ptr(), rows, cols, cols)
    finish(hc)
    expect_s, expect_m = np.zeros(rows, np.float32), np.zeros(rows, np.float32)
    oracle.reduce_rows(x, expect_s, expect_m, 256)
    _reduce_check(x, d_s.cpu().numpy(), d_m.cpu().numpy(), expect_s, expect_m)


def test_reduce_rows_single_outputs_nan_and_f64(hc):
    rng = np.random.default_rng(5)
    x = rng.uniform(-10, 10, (40, 333)).astype(np.float32)
    x[3, 17] = np.nan
    d_x = dev(x)
    d_m = empty_like_dev((40,), torch.float32)
    hc.reduce_rows(d_x.data_ptr(), 0, d_m.data_ptr(), 40, 333, 333)  # max only
    finish(hc)
    got = d_m.cpu().numpy()
    assert np.isnan(got[3])  # NaN propagates, as in numpy
    assert np.array_equal(np.delete(got, 3), np.delete(x.max(axis=1), 3))
    d_s = empty_like_dev((40,), torch.float32)
    hc.reduce_rows(d_x.data_ptr(), d_s.data_ptr(), 0, 40, 333, 333)  # sum only
    finish(hc)
    assert np.isnan(d_s.cpu().numpy()[3])

    x64 = rng.uniform(-10, 10, (50, 777))
    d_x = dev(x64)
    d_s, d_m = empty_like_dev((50,), torch.float64), empty_like_dev((50,), torch.float64)
    hc.reduce_rows(d_x.data_ptr(), d_s.data_ptr(), d_m.data_ptr(), 50, 777, 777, capi.HC_F64)
    finish(hc)
    assert np.array_equal(d_m.cpu().numpy(), x64.max(axis=1))
    np.testing.assert_allclose(d_s.cpu().numpy(), x64.sum(axis=1), rtol=1e-12, atol=1e-10)


# ---- tiled GEMM ----------------------------------------------------------------------
def _gemm_f32_check(a, b, got, expect):
    bound = 1e-5 * (np.abs(a).astype(np.float64) @ np.abs(b).astype(np.float64))
    assert np.all(np.abs(got.astype(np.float64) - expect.astype(np.float64)) <= bound)


@pytest.mark.parametrize("shape,key", [((256, 256, 256), "cfg1_gemm_f32_256"),
                                       ((70, 45, 33), "cfg1_gemm_f32_70x45x33")])
def test_gemm_tiled_f32_golden(hc, golden, shape, key):
    m, n, k = shape
    a, b = oracle.make_inputs("gemm_f32", shape=shape)
    d_a, d_b, d_c = dev(a), dev(b), empty_like_dev((m, n), torch.float32)
    hc.gemm_tiled(d_a.data_ptr(), d_b.data_ptr(), d_c.data_ptr(), m, n, k, k, n, n)
    finish(hc)
    _gemm_f32_check(a, b, d_c.cpu().numpy(), golden[key])


def test_gemm_tiled_reference_vector_f64(hc, golden):
    m, n, k = 16, 32, 64
    a = 2 * np.arange(m * k).reshape(m, k) / (m * k)
    b = np.arange(n * k).reshape(k, n) / (n * k)
    d_a, d_b, d_c = dev(a), dev(b), empty_like_dev((m, n), torch.float64)
    hc.gemm_tiled(d_a.data_ptr(), d_b.data_ptr(), d_c.data_ptr(), m, n, k, k, n, n, capi.HC_F64)
    finish(hc)
    np.testing.assert_allclose(d_c.cpu().numpy(), golden["kat_dot_kblocked_f64"], rtol=1e-12)
    np.testing.assert_allclose(d_c.cpu().numpy(), golden["kat_dot_fullk_f64"], rtol=1e-12)


@pytest.mark.parametrize("shape", [(1, 1, 1), (65, 63, 17), (128, 192, 300), (300, 100, 1)])
def test_gemm_tiled_f32_shapes(hc, shape):
    m, n, k = shape
    rng = np.random.default_rng(m + 10 * n + 100 * k)
    a = rng.uniform(-1, 1, (m, k)).astype(np.float32)
    b = rng.uniform(-1, 1, (k, n)).astype(np.float32)
    d_a, d_b, d_c = dev(a), dev(b), empty_like_dev((m, n), torch.float32)
    hc.gemm_tiled(d_a.data_ptr(), d_b.data_ptr(), d_c.data_ptr(), m, n, k, k, n, n)
    finish(hc)
    expect = np.zeros((m, n), np.float32)
    oracle.gemm_kblocked(a, b, expect, (64, 64), kb=16)
    _gemm_f32_check(a, b, d_c.cpu().numpy(), expect)


# 0: cp.async pipeline when legal, K split over a four-CTA cluster when there are
# few tiles and K >= 128; 1: neither; 2: the pipeline without the split.
@pytest.mark.parametrize("variant", [0, 1, 2])
@pytest.mark.parametrize("shape", [(256, 256, 256), (70, 44, 36), (130, 68, 100), (64, 64, 4),
                                   (1, 4, 8), (200, 260, 1028), (64, 64, 128), (65, 124, 132),
                                   (300, 380, 516), (37, 8, 4100), (64, 64, 160)])
def test_gemm_tiled_f32_pipelined_and_plain_agree(hc, variant, shape):
    m, n, k = shape
    rng = np.random.default_rng(m + n + k)
    a = rng.uniform(-1, 1, (m, k)).astype(np.float32)
    b = rng.uniform(-1, 1, (k, n)).astype(np.float32)
    d_a, d_b, d_c = dev(a), dev(b), empty_like_dev((m, n), torch.float32)
    hc.set_option("tiled_variant", variant)
    try:
        hc.gemm_tiled(d_a.data_ptr(), d_b.data_ptr(), d_c.data_ptr(), m, n, k, k, n, n)
        finish(hc)
    finally:
        hc.set_option("tiled_variant", 0)
    expect = np.zeros((m, n), np.float32)
    oracle.gemm_kblocked(a, b, expect, (64, 64), kb=16)
    _gemm_f32_check(a, b, d_c.cpu().numpy(), expect)


# ---- bf16 GEMM (tensor cores) -------------------------------------------------------
VARIANTS = {"single": 1, "pair": 2, "tiled": 3, "auto": 0}


def _bf16_check(a, b, got, expect):
    # bf16 keeps 8 significant bits: half an ulp is 2^-9 relative.  The fp32
    # accumulation error is bounded by sum|a||b| * K * 2^-24, far below that.
    mag = np.abs(a).astype(np.float64) @ np.abs(b).astype(np.float64)
    bound = 1e-2 * np.abs(expect).astype(np.float64) + 1e-4 * mag + 1e-30
    bad = np.abs(got.astype(np.float64) - expect.astype(np.float64)) > bound
    assert not bad.any(), (
        f"{bad.sum()} of {bad.size} elements out of tolerance; first at "
        f"{np.argwhere(bad)[0].tolist()}: got {got[bad][0]} expect {expect[bad][0]}"
    )


def _run_gemm_bf16(hc, a, b, variant):
    m, k = a.shape
    n = b.shape[1]
    d_a, d_b = dev_bf16(a), dev_bf16(b)
    d_c = empty_like_dev((m, n), torch.bfloat16)
    hc.set_option("gemm_variant", VARIANTS[variant])
    try:
        hc.gemm_bf16(d_a.data_ptr(), d_b.data_ptr(), d_c.data_ptr(), m, n, k, k, n, n)
        finish(hc)
    finally:
        hc.set_option("gemm_variant", 0)
    return host_bf16(d_c)


@pytest.mark.parametrize("variant", ["tiled", "single", "pair"])
def test_gemm_bf16_golden(hc, golden, variant):
    shape = (256, 512, 384)
    a, b = oracle.make_inputs("gemm_bf16", shape=shape)
    got = _run_gemm_bf16(hc, a, b, variant)
    expect = oracle.bf16_from_bits(golden["cfg4_gemm_bf16_256x512x384_bits"])
    _bf16_check(a, b, got, expect)


@pytest.mark.parametrize("variant", ["single", "pair"])
@pytest.mark.parametrize(
    "shape",
    [(128, 256, 64), (128, 256, 128), (256, 256, 512), (512, 768, 1024), (200, 264, 136),
     (1, 8, 8), (129, 520, 72), (1000, 1000, 1000), (2048, 2304, 1536)],
)
def test_gemm_bf16_shapes(hc, variant, shape):
    m, n, k = shape
    rng = np.random.default_rng(m * 31 + n * 17 + k)
    a = oracle.round_to_bf16(rng.standard_normal((m, k)).astype(np.float32))
    b = oracle.round_to_bf16(rng.standard_normal((k, n)).astype(np.float32))
    got = _run_gemm_bf16(hc, a, b, variant)
    expect = np.zeros((m, n), np.float32)
    oracle.gemm_bf16(a, b, expect, (256, 256))
    _bf16_check(a, b, got, expect)


def test_gemm_bf16_unaligned_falls_back_to_tiled(hc):
    # K = 100 gives an A pitch of 200 bytes: TMA cannot describe it.
    m, n, k = 70, 90, 100
    rng = np.random.default_rng(9)
    a = oracle.round_to_bf16(rng.standard_normal((m, k)).astype(np.float32))
    b = oracle.round_to_bf16(rng.standard_normal((k, n)).astype(np.float32))
    got = _run_gemm_bf16(hc, a, b, "auto")
    expect = np.zeros((m, n), np.float32)
    oracle.gemm_bf16(a, b, expect, (256, 256))
    _bf16_check(a, b, got, expect)


def test_gemm_bf16_row_shard_view(hc):
    # The multi-GPU launcher hands each rank a row block of A and C: pitches
    # equal the full width, the base is offset.
    m, n, k = 384, 512, 256
    rng = np.random.default_rng(21)
    a = oracle.round_to_bf16(rng.standard_normal((m, k)).astype(np.float32))
    b = oracle.round_to_bf16(rng.standard_normal((k, n)).astype(np.float32))
    d_a, d_b = dev_bf16(a), dev_bf16(b)
    d_c = empty_like_dev((m, n), torch.bfloat16)
    hc.gemm_bf16(d_a[128:].data_ptr(), d_b.data_ptr(), d_c[128:].data_ptr(), 256, n, k, k, n, n)
    finish(hc)
    expect = np.zeros((m, n), np.float32)
    oracle.gemm_bf16(a, b, expect, (256, 256))
    got = host_bf16(d_c)
    _bf16_check(a[128:], b, got[128:], expect[128:])
    assert np.isnan(got[:128]).all()  # rows of other ranks untouched


# ---- int8 weight-only dequant GEMM -----------------------------------------------------
def _run_w8a16(hc, a, w, s, variant="auto", col_shard=None):
    m, k = a.shape
    n = w.shape[1]
    d_a, d_w, d_s = dev_bf16(a), dev(w), dev(s)
    d_c = empty_like_dev((m, n), torch.bfloat16)
    n0, n1 = col_shard or (0, n)
    nn = n1 - n0
    ws_bytes = hc.gemm_w8a16_workspace_bytes(nn, k)
    ws = torch.empty(max(ws_bytes, 16), dtype=torch.uint8, device="cuda")
    torch.cuda.synchronize()
    hc.set_option("gemm_variant", VARIANTS[variant])
    try:
        hc.gemm_w8a16(d_a.data_ptr(), d_w[:, n0:].data_ptr(), d_s[n0:].data_ptr(),
                      d_c[:, n0:].data_ptr(), ws.data_ptr(), ws_bytes, m, nn, k, k, n, n)
        finish(hc)
    finally:
        hc.set_option("gemm_variant", 0)
    return host_bf16(d_c)


@pytest.mark.parametrize("variant", ["tiled", "single", "pair"])
def test_gemm_w8a16_golden(hc, golden, variant):
    a, w, s = oracle.make_inputs("gemm_w8a16", shape=(128, 256, 512))
    got = _run_w8a16(hc, a, w, s, variant)
    expect = oracle.bf16_from_bits(golden["cfg5_gemm_w8a16_128x256x512_bits"])
    _bf16_check(a, w.astype(np.float32) * s, got, expect)


@pytest.mark.parametrize("shape", [(512, 1024, 1024), (100, 48, 200), (300, 272, 520), (64, 7, 33)])
def test_gemm_w8a16_shapes(hc, shape):
    a, w, s = oracle.make_inputs("gemm_w8a16", shape=shape)
    w[0, 0] = -128  # the one int8 value outside the benchmark's range
    got = _run_w8a16(hc, a, w, s)
    expect = np.zeros((shape[0], shape[1]), np.float32)
    oracle.gemm_w8a16(a, w, s, expect, (256, 256))
    _bf16_check(a, w.astype(np.float32) * s, got, expect)


def test_gemm_w8a16_column_shard(hc):
    # N-sharding: a rank owns columns [256, 512) of W, scale and out.
    a, w, s = oracle.make_inputs("gemm_w8a16", shape=(256, 768, 512))
    got = _run_w8a16(hc, a, w, s, col_shard=(256, 512))
    expect = np.zeros((256, 768), np.float32)
    oracle.gemm_w8a16(a, w, s, expect, (256, 256))
    _bf16_check(a, (w.astype(np.float32) * s)[:, 256:512], got[:, 256:512], expect[:, 256:512])
    assert np.isnan(got[:, :256]).all() and np.isnan(got[:, 512:]).all()


def test_dequant_w8_is_exact(hc):
    w = np.arange(-128, 128, dtype=np.int8).reshape(4, 64)
    w = np.tile(w, (3, 5))  # 12 x 320
    d_w = dev(w)
    d_o = empty_like_dev(w.shape, torch.bfloat16)
    hc.dequant_w8(d_w.data_ptr(), d_o.data_ptr(), 12, 320, 320, 320)
    finish(hc)
    assert np.array_equal(host_bf16(d_o), w.astype(np.float32))
    d_o2 = empty_like_dev((12, 37), torch.bfloat16)  # ragged, scalar path
    hc.dequant_w8(d_w.data_ptr(), d_o2.data_ptr(), 12, 37, 320, 37)
    finish(hc)
    assert np.array_equal(host_bf16(d_o2), w[:, :37].astype(np.float32))


def test_gemm_w8a16_needs_workspace(hc):
    a, w, s = oracle.make_inputs("gemm_w8a16", shape=(128, 256, 512))
    d_a, d_w, d_s = dev_bf16(a), dev(w), dev(s)
    d_c = empty_like_dev((128, 256), torch.bfloat16)
    with pytest.raises(capi.HcError, match="workspace"):
        hc.gemm_w8a16(d_a.data_ptr(), d_w.data_ptr(), d_s.data_ptr(), d_c.data_ptr(), 0, 0,
                      128, 256, 512, 512, 256, 256)


# ---- softmax kernel variants ------------------------------------------------------------
@pytest.mark.parametrize("variant", [1, 2])  # 1: row in registers, 2: bulk-copy pipeline
@pytest.mark.parametrize("rows,cols", [(40, 2048), (7, 3000), (600, 4096), (3000, 1028),
                                       (149, 1280), (5000, 4096)])
def test_softmax_variants_agree_with_oracle(hc, variant, rows, cols):
    rng = np.random.default_rng(rows + cols)
    x = (rng.standard_normal((rows, cols)) * 2).astype(np.float32)
    d_x, d_y = dev(x), empty_like_dev(x.shape, torch.float32)
    hc.set_option("softmax_variant", variant)
    try:
        hc.softmax_rows(d_x.data_ptr(), d_y.data_ptr(), rows, cols, cols, cols)
        finish(hc)
    finally:
        hc.set_option("softmax_variant", 0)
    expect = np.zeros_like(x)
    oracle.softmax_rows(x, expect, 8)
    _softmax_check(d_y.cpu().numpy(), expect)


# ---- whole-array sum ------------------------------------------------------------------
@pytest.mark.parametrize("n", [1, 20, 1000, 1 << 20, 5_000_003])
@pytest.mark.parametrize("in_dtype", ["f32", "f64", "i32", "i64"])
def test_reduce_all_matches_oracle(hc, n, in_dtype):
    np_t = {"f32": np.float32, "f64": np.float64, "i32": np.int32, "i64": np.int64}[in_dtype]
    code = {"f32": capi.HC_F32, "f64": capi.HC_F64, "i32": capi.HC_I32, "i64": capi.HC_I64}[in_dtype]
    rng = np.random.default_rng(n)
    a = (rng.integers(-1000, 1000, n) if in_dtype.startswith("i")
         else rng.uniform(-10, 10, n)).astype(np_t)
    d_a = dev(a)
    d_r = torch.full((1,), 5.0, dtype=torch.float64, device="cuda")  # pre-existing content is kept
    torch.cuda.synchronize()
    hc.reduce_all(d_a.data_ptr(), n, d_r.data_ptr(), code, capi.HC_F64)
    finish(hc)
    expect = np.zeros(1)
    oracle.reduce_sum_all(a, expect, 8, 2)
    got = d_r.cpu().numpy()[0] - 5.0
    if in_dtype.startswith("i"):
        assert got == expect[0] == a.sum()  # integers are exact in float64
    else:
        assert abs(got - a.astype(np.float64).sum()) <= 1e-12 * np.abs(a).astype(np.float64).sum() + 1e-9
    d_r32 = torch.zeros(1, dtype=torch.float32, device="cuda")
    torch.cuda.synchronize()
    hc.reduce_all(d_a.data_ptr(), n, d_r32.data_ptr(), code, capi.HC_F32)
    finish(hc)
    # float64 and integer inputs are summed in double and meet float32 only in the
    # one atomicAdd per CTA; float32 inputs are summed in float32 throughout.
    rel = 1e-5 if in_dtype == "f32" else 1e-6
    bound = rel * np.abs(a).astype(np.float64).sum() + 1e-6
    assert abs(float(d_r32.cpu().numpy()[0]) - a.astype(np.float64).sum()) <= bound


@pytest.mark.parametrize("dtype", ["f32", "f64"])
@pytest.mark.parametrize("shape", [(16, 32, 8), (70, 45, 19), (1, 1, 1), (200, 130, 300), (64, 64, 0)])
def test_pairwise_distance_matches_oracle(hc, golden, dtype, shape):
    m, n, d = shape
    np_t, t_t, code = ((np.float32, torch.float32, capi.HC_F32) if dtype == "f32"
                       else (np.float64, torch.float64, capi.HC_F64))
    if shape == (16, 32, 8):  # the reference's own test vector
        a = (2 * np.arange(m * d).reshape(m, d) / (m * d)).astype(np_t)
        b = (np.arange(n * d).reshape(n, d) / (n * d)).astype(np_t)
    else:
        rng = np.random.default_rng(5)
        a = rng.standard_normal((m, d)).astype(np_t)
        b = rng.standard_normal((n, d)).astype(np_t)
    d_a, d_b = dev(a), dev(b)
    d_o = empty_like_dev((m, n), t_t)
    hc.pairwise_distance(d_a.data_ptr() if d else 0, d_b.data_ptr() if d else 0, d_o.data_ptr(),
                         m, n, d, max(d, 1), max(d, 1), n, code)
    finish(hc)
    expect = np.zeros((m, n), np_t)
    oracle.pairwise_distance(a, b, expect, (8, 8))
    rtol = 1e-5 if dtype == "f32" else 1e-13
    np.testing.assert_allclose(d_o.cpu().numpy(), expect, rtol=rtol, atol=rtol)
    if shape == (16, 32, 8) and dtype == "f64":
        np.testing.assert_allclose(d_o.cpu().numpy(), golden["kat_pairwise_f64"], rtol=1e-13)
    if shape == (70, 45, 19) and dtype == "f32":
        np.testing.assert_allclose(d_o.cpu().numpy(), golden["pairwise_f32_70x45x19"], rtol=1e-5,
                                   atol=1e-6)


def test_empty_and_degenerate_shapes(hc):
    # Nothing to do: no launch, no error.
    before = hc.launch_count
    hc.softmax_rows(0, 0, 0, 128, 128, 128)
    hc.softmax_rows(0, 0, 16, 0, 0, 0)
    hc.reduce_rows(0, 0, 0, 0, 64, 64)
    hc.gemm_tiled(0, 0, 0, 0, 64, 64, 64, 64, 64)
    hc.gemm_bf16(0, 0, 0, 64, 0, 64, 64, 0, 0)
    hc.dequant_w8(0, 0, 0, 64, 64, 64)
    assert hc.launch_count == before
    # K = 0: an empty sum, so the product is all zeros (and must be written).
    for dtype, t, fn in ((capi.HC_F32, torch.float32, "tiled"), (None, torch.bfloat16, "bf16")):
        d_c = empty_like_dev((70, 40), t)
        if fn == "tiled":
            hc.gemm_tiled(0, 0, d_c.data_ptr(), 70, 40, 0, 0, 40, 40, dtype)
        else:
            hc.gemm_bf16(0, 0, d_c.data_ptr(), 70, 40, 0, 0, 40, 40)
        finish(hc)
        assert torch.count_nonzero(d_c.float()) == 0 and not torch.isnan(d_c.float()).any()
    # One row, one column.
    x = np.array([[3.5]], np.float32)
    d_x, d_y = dev(x), empty_like_dev((1, 1), torch.float32)
    hc.softmax_rows(d_x.data_ptr(), d_y.data_ptr(), 1, 1, 1, 1)
    d_s, d_m = empty_like_dev((1,), torch.float32), empty_like_dev((1,), torch.float32)
    hc.reduce_rows(d_x.data_ptr(), d_s.data_ptr(), d_m.data_ptr(), 1, 1, 1)
    finish(hc)
    assert d_y.item() == 1.0 and d_s.item() == 3.5 and d_m.item() == 3.5
    with pytest.raises(capi.HcError, match="invalid shape"):
        hc.gemm_bf16(0, 0, 0, 8, 8, 8, 4, 8, 8)  # lda smaller than K
    with pytest.raises(capi.HcError, match="null buffer"):
        hc.gemm_bf16(0, 0, 0, 8, 8, 8, 8, 8, 8)


def test_reduce_all_errors(hc):
    hc.reduce_all(0, 0, 0)  # nothing to do
    with pytest.raises(capi.HcError, match="unsupported dtypes"):
        hc.reduce_all(0, 4, 0, capi.HC_BF16, capi.HC_F32)
    with pytest.raises(capi.HcError, match="null buffer"):
        hc.reduce_all(0, 4, 0, capi.HC_F32, capi.HC_F32)
