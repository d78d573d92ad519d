"""GPU tests of the ``@kernel`` call surface: the reference's own end-to-end
tests (python/hckernel/tests/test_e2e.py:57-136, same kernels, same shapes,
same assertions) and the benchmark workloads written in the DSL, each checked
against the CPU oracle.
"""

import numpy as np
import pytest
import sympy
import torch
from torch.testing import assert_close

from hc_b200.hckernel.kernel import *  # noqa: F401,F403  (as the reference's tests import)
from hc_b200.hckernel.kernel import UnsupportedKernel, get_context
from hc_b200.workloads import make_kernels
from oracle import workloads as oracle

pytestmark = pytest.mark.gpu

BACKEND, DEVICE = "nvvm", "cuda:0"

_copy_shapes = [(1, 27), (1, 72), (1, 128), (10, 20), (111, 813), (256, 64), (256, 1024)]


def to_device(array):
    return array.to("cuda")


@pytest.mark.parametrize("shape", _copy_shapes)
def test_copy(shape):
    W, H, DT = sym.W, sym.H, typename.DT

    @kernel(work_shape=(W, H), backend=BACKEND, device=DEVICE)
    def copy_kernel(group: CurrentGroup, src: Buffer[W, H, DT], dst: Buffer[W, H, DT]):
        x, y = group.work_offset
        val = group.load(src[x:, y:], shape=group.shape)
        group.store(dst[x:, y:], val)

    a = to_device(torch.arange(shape[0] * shape[1], dtype=torch.int32).reshape(shape))
    b = torch.zeros_like(a)
    copy_kernel(a, b)
    assert_close(b, a)


@pytest.mark.parametrize("shape", _copy_shapes)
@pytest.mark.parametrize("unroll", [1, 2, 4])
def test_copy_unroll(shape, unroll):
    W, H, DT, V = sym.W, sym.H, typename.DT, sym.V
    H1 = sympy.ceiling(H / V)

    @kernel(work_shape=(W, H1), backend=BACKEND, device=DEVICE)
    def copy_kernel(group: CurrentGroup, src: Buffer[W, H, DT], dst: Buffer[W, H, DT], v: V):
        x, y = group.work_offset
        val = group.load(src[x:, y * V :], shape=(group.shape[0], group.shape[1] * V))
        group.store(dst[x:, y * V :], val)

    a = to_device(torch.arange(shape[0] * shape[1], dtype=torch.int32).reshape(shape))
    b = torch.zeros_like(a)
    copy_kernel(a, b, unroll)
    assert_close(b, a)


@pytest.mark.parametrize("shape", _copy_shapes)
@pytest.mark.parametrize("unroll", [1, 2, 4])
def test_copy_vec(shape, unroll):
    W, H, DT, V = sym.W, sym.H, typename.DT, sym.V
    H1 = sympy.ceiling(H / V)

    @kernel(work_shape=(W, H1), backend=BACKEND, device=DEVICE, literals=[V])
    def copy_kernel(group: CurrentGroup, src: Buffer[W, H, DT], dst: Buffer[W, H, DT], v: V):
        x, y = group.work_offset
        val = group.vload(src[x:, y * V :], shape=(group.shape[0], group.shape[1] * V))
        group.store(dst[x:, y * V :], val)

    a = to_device(torch.arange(shape[0] * shape[1], dtype=torch.int32).reshape(shape))
    b = torch.zeros_like(a)
    copy_kernel(a, b, unroll)
    assert_close(b, a)


@pytest.fixture(scope="module")
def k():
    return make_kernels(DEVICE)


def test_softmax_kernel_matches_oracle(k):
    (x,) = oracle.make_inputs("softmax", shape=(100, 4096))
    d_x = to_device(torch.from_numpy(x))
    d_y = torch.empty_like(d_x)
    k.softmax(d_x, d_y, 8)
    expect = np.zeros_like(x)
    oracle.softmax_rows(x, expect, 8)
    got = d_y.cpu().numpy()
    assert np.all(np.abs(got - expect) <= 1e-6 + 1e-5 * np.abs(expect))


def test_softmax_reference_vector_f64(k, golden):
    m, n = 30, 25
    a = 2 * np.arange(m * n).reshape(m, n) / (m * n)
    d_x = to_device(torch.from_numpy(a))
    d_y = torch.zeros_like(d_x)
    k.softmax(d_x, d_y, 8)
    np.testing.assert_allclose(d_y.cpu().numpy(), golden["kat_softmax_f64"], rtol=1e-12)


def test_reduce_rows_kernel_matches_oracle(k):
    (x,) = oracle.make_inputs("reduce", shape=(1500, 2048))
    d_x = to_device(torch.from_numpy(x))
    d_s = torch.empty(1500, device="cuda")
    d_m = torch.empty(1500, device="cuda")
    k.reduce_rows(d_x, d_s, d_m, 256)
    assert np.array_equal(d_m.cpu().numpy(), x.max(axis=1))
    exact = x.astype(np.float64).sum(axis=1)
    assert np.all(np.abs(d_s.cpu().numpy() - exact) <= 1e-5 * np.abs(x).sum(axis=1))


def test_dot_kernels_f32_f64_bf16(k, golden):
    a, b = oracle.make_inputs("gemm_f32")
    d_a, d_b = to_device(torch.from_numpy(a)), to_device(torch.from_numpy(b))
    d_c = torch.zeros(256, 256, device="cuda")
    k.dot(d_a, d_b, d_c, (64, 64))
    bound = 1e-5 * (np.abs(a).astype(np.float64) @ np.abs(b).astype(np.float64))
    assert np.all(np.abs(d_c.cpu().numpy().astype(np.float64) - golden["cfg1_gemm_f32_256"]) <= bound)
    # Tunables change the tiling of the reference, not the result.
    d_c2 = torch.zeros_like(d_c)
    k.dot.parametrize({sym.KB: 32, sym.MI: 2})(d_a, d_b, d_c2, (32, 64))
    assert np.all(np.abs(d_c2.cpu().numpy().astype(np.float64) - golden["cfg1_gemm_f32_256"]) <= bound)

    m, n, kk = 16, 32, 64
    a64 = 2 * np.arange(m * kk).reshape(m, kk) / (m * kk)
    b64 = np.arange(n * kk).reshape(kk, n) / (n * kk)
    d_c = torch.zeros(m, n, dtype=torch.float64, device="cuda")
    k.dot(to_device(torch.from_numpy(a64)), to_device(torch.from_numpy(b64)), d_c, (8, 8))
    np.testing.assert_allclose(d_c.cpu().numpy(), golden["kat_dot_kblocked_f64"], rtol=1e-12)

    a, b = oracle.make_inputs("gemm_bf16", shape=(256, 512, 384))
    d_a = to_device(torch.from_numpy(a)).bfloat16()
    d_b = to_device(torch.from_numpy(b)).bfloat16()
    d_c = torch.zeros(256, 512, dtype=torch.bfloat16, device="cuda")
    k.dot_fullk(d_a, d_b, d_c, (128, 256))
    expect = oracle.bf16_from_bits(golden["cfg4_gemm_bf16_256x512x384_bits"])
    got = d_c.float().cpu().numpy()
    assert np.all(np.abs(got - expect) <= 1e-2 * np.abs(expect) + 1e-4 * (np.abs(a) @ np.abs(b)))


def test_dequant_dot_kernel(k, golden):
    a, w, s = oracle.make_inputs("gemm_w8a16", shape=(128, 256, 512))
    d_a = to_device(torch.from_numpy(a)).bfloat16()
    d_w, d_s = to_device(torch.from_numpy(w)), to_device(torch.from_numpy(s))
    d_c = torch.zeros(128, 256, dtype=torch.bfloat16, device="cuda")
    k.dequant_dot(d_a, d_w, d_s, d_c, (128, 128))
    expect = oracle.bf16_from_bits(golden["cfg5_gemm_w8a16_128x256x512_bits"])
    got = d_c.float().cpu().numpy()
    mag = np.abs(a) @ (np.abs(w.astype(np.float32)) * s)
    assert np.all(np.abs(got - expect) <= 1e-2 * np.abs(expect) + 1e-4 * mag)


def test_launch_is_ordered_with_torch_streams(k):
    # The kernel runs on the context's own stream; results must still be
    # ordered after torch work that produced the inputs and before torch work
    # that consumes the outputs, without any host synchronisation here.
    x = torch.randn(4096, 4096, device="cuda")
    for _ in range(3):
        x = x * 1.0001 + 0.5  # queued on torch's stream
    y = torch.empty_like(x)
    k.softmax(x, y, 256)
    total = y.sum(dim=1)  # queued on torch's stream right after
    assert torch.allclose(total, torch.ones_like(total), atol=1e-4)


def test_argument_errors(k):
    x = torch.randn(8, 16, device="cuda")
    with pytest.raises(ValueError, match="host memory"):
        k.softmax(torch.randn(8, 16), torch.randn(8, 16), 8)
    with pytest.raises(ValueError, match="Symbol value conflict"):
        k.softmax(x, torch.empty(9, 16, device="cuda"), 8)
    with pytest.raises(TypeError, match="float32 but out is float64"):
        k.softmax(x, torch.empty(8, 16, device="cuda", dtype=torch.float64), 8)
    with pytest.raises(ValueError, match="rows must be contiguous"):
        k.softmax(x.t().contiguous().t(), torch.empty(8, 16, device="cuda"), 8)
    with pytest.raises(TypeError, match="float32 or float64"):
        k.softmax(x.half(), torch.empty(8, 16, device="cuda", dtype=torch.half), 8)

    W, H, DT = sym.W, sym.H, typename.DT

    @kernel(work_shape=(W, H), backend="rocm", device="hip:0")
    def on_hip(group: CurrentGroup, src: Buffer[W, H, DT], dst: Buffer[W, H, DT]):
        x0, y0 = group.work_offset
        group.store(dst[x0:, y0:], group.load(src[x0:, y0:], shape=group.shape))

    with pytest.raises(ValueError, match="backend 'rocm' is not available"):
        on_hip(x, torch.empty_like(x))

    @kernel(work_shape=(W, H), backend=BACKEND, device=DEVICE)
    def shifted(group: CurrentGroup, src: Buffer[W, H, DT], dst: Buffer[W, H, DT]):
        x0, y0 = group.work_offset
        group.store(dst[x0:, y0:], group.load(src[x0:, y0 + 1 :], shape=group.shape))

    with pytest.raises(UnsupportedKernel):
        shifted(x, torch.empty_like(x))
    assert get_context(DEVICE).kernel_status() == 0


def ceil_div(a, b):
    return (a + b - 1) // b


def test_autotune_picks_a_variant_and_keeps_results_right(k, tmp_path):
    # The API of the reference's RFC (docs/langref.md:526-560):
    # tparams = autotune(kernel, *args); tuned = kernel.parametrize(tparams).
    a, b = oracle.make_inputs("gemm_bf16", shape=(512, 512, 256))
    d_a = to_device(torch.from_numpy(a)).bfloat16()
    d_b = to_device(torch.from_numpy(b)).bfloat16()
    d_c = torch.zeros(512, 512, dtype=torch.bfloat16, device="cuda")
    tparams = autotune(k.dot_fullk, d_a, d_b, d_c, (128, 128), repeats=3)
    assert isinstance(tparams, TunedParams) and len(tparams.timings) >= 2
    assert set(tparams.options) <= {"gemm_variant", "tiled_variant"}
    tparams.save(tmp_path / "gemm.json")
    tuned = k.dot_fullk.parametrize(autotune.load(tmp_path / "gemm.json"))
    d_c.zero_()
    tuned(d_a, d_b, d_c, (128, 128))
    expect = np.zeros((512, 512), np.float32)
    oracle.gemm_bf16(a, b, expect, (256, 256))
    got = d_c.float().cpu().numpy()
    assert np.all(np.abs(got - expect) <= 1e-2 * np.abs(expect) + 1e-4 * (np.abs(a) @ np.abs(b)))

    (x,) = oracle.make_inputs("softmax", shape=(3000, 2048))
    d_x = to_device(torch.from_numpy(x))
    d_y = torch.empty_like(d_x)
    tparams = autotune(k.softmax, d_x, d_y, 64, repeats=3)
    assert tparams.options.get("softmax_variant") in (1, 2)
    k.softmax.parametrize(tparams)(d_x, d_y, 64)
    expect = np.zeros_like(x)
    oracle.softmax_rows(x, expect, 64)
    assert np.all(np.abs(d_y.cpu().numpy() - expect) <= 1e-6 + 1e-5 * np.abs(expect))

    # A row body: a warp that walks the row against a CTA that holds it.
    from hc_b200.workloads import make_rowwise

    centre = make_rowwise(lambda t: t - t.mean(axis=1, keepdims=True))
    d_y.fill_(float("nan"))
    tparams = autotune(centre, d_x, d_y, 64, repeats=3)
    assert tparams.options.get("row_variant") in (1, 2, 3) and len(tparams.timings) == 3
    centre.parametrize(tparams)(d_x, d_y, 64)
    torch.cuda.synchronize()
    x64 = x.astype(np.float64)
    np.testing.assert_allclose(d_y.cpu().numpy(), x64 - x64.mean(axis=1, keepdims=True),
                               rtol=2e-6, atol=1e-6)
    assert get_context(DEVICE).kernel_status() == 0


def test_pairwise_distance():
    # python/hckernel/tests/test_examples.py:261-301, on the GPU.
    M, N, D = sym.M, sym.N, sym.D
    GM, GN, MI, NI = sym.GM, sym.GN, sym.MI, sym.NI
    TMI = TunableParam(MI, 1, range(1, 8))
    TNI = TunableParam(NI, 1, range(1, 8))

    @kernel(work_shape=(ceil_div(M, MI), ceil_div(N, NI)), group_shape=(GM, GN),
            tunables=(TMI, TNI), backend=BACKEND, device=DEVICE)
    def pw_distance(gr: CurrentGroup, a: Buffer[M, D, typename.DT], b: Buffer[N, D, typename.DT],
                    out: Buffer[M, N, typename.DT], gshape: (GM, GN)):
        m_start = gr.work_offset[0] * MI
        n_start = gr.work_offset[1] * NI
        m_block = gr.shape[0] * MI
        n_block = gr.shape[1] * NI
        a_view = gr.load(a[m_start:, :], shape=(m_block, D))
        b_view = gr.load(b[n_start:, :], shape=(n_block, D))
        diff = a_view[:, None, :] - b_view[None, :, :]
        gr.store(out[m_start:, n_start:], np.linalg.norm(diff, axis=2))

    m, n, d = 16, 32, 8
    a = 2 * np.arange(m * d).reshape(m, d) / (m * d)
    b = np.arange(n * d).reshape(n, d) / (n * d)
    result = torch.zeros(m, n, dtype=torch.float64, device="cuda")
    pw_distance(to_device(torch.from_numpy(a)), to_device(torch.from_numpy(b)), result, (8, 8))
    np.testing.assert_allclose(result.cpu().numpy(),
                               np.linalg.norm(a[:, None, :] - b[None, :, :], axis=2), rtol=1e-13)


def test_reduction_1():
    # python/hckernel/tests/test_examples.py:31-47, on the GPU.
    WS, GS, N = sym.WS, sym.GS, sym.N
    TN = TunableParam(N, 2, range(1, 64))

    @kernel(work_shape=ceil_div(WS, N), group_shape=GS, tunables=TN, backend=BACKEND, device=DEVICE)
    def reduction(gr: CurrentGroup, a: Buffer[WS, typename.DT], result: Buffer[1, typename.DT],
                  gshape: GS):
        a_view = gr.load(a[gr.work_offset[0] * N :], shape=gr.size * N)
        atomic_ref(result)[0] += a_view.sum()

    a = np.arange(0, 20)
    d_a = to_device(torch.from_numpy(a))
    d_result = torch.zeros(1, dtype=torch.float64, device="cuda")
    reduction(d_a, d_result, 8)
    assert d_result.cpu().numpy()[0] == a.sum()


def test_reduction_2():
    # python/hckernel/tests/test_examples.py:50-71, on the GPU.
    WS, GS, N = sym.WS, sym.GS, sym.N
    TN = TunableParam(N, 2, range(1, 64))

    @kernel(work_shape=ceil_div(WS, N), group_shape=GS, tunables=TN, backend=BACKEND, device=DEVICE)
    def reduction(group: CurrentGroup, a: Buffer[WS, typename.DT], result: Buffer[1, typename.DT],
                  gshape: GS):
        temp_result = group.zeros(group.size, dtype=a.dtype)
        for i in range(N):
            work_offset = group.work_offset[0] * N + i * group.size
            a_view = group.load(a[work_offset:], shape=group.size)
            temp_result += a_view
        atomic_ref(result)[0] += temp_result.sum()

    a = np.arange(0, 20)
    d_a = to_device(torch.from_numpy(a))
    d_result = torch.zeros(1, dtype=torch.float64, device="cuda")
    reduction(d_a, d_result, 8)
    assert d_result.cpu().numpy()[0] == a.sum()
    # The kernel adds to what is already there, like `+=` on the simulator.
    reduction(d_a, d_result, 8)
    assert d_result.cpu().numpy()[0] == 2 * a.sum()
