"""Generate the golden vectors under ``tests/golden/`` from the reference itself.

Run on a machine that has the reference tree (its location is taken from
``HC_REFERENCE_ROOT``)::

    python tests/golden/make_golden.py

The script imports the reference's simulator (``hckernel.kernel_sim``) straight
from the reference tree, runs the workload kernels written in the reference's
DSL on seeded inputs, and stores the *reference's* outputs (plus the inputs
when they are not reproducible from a seed) as ``.npz`` files.  It also runs the
NumPy oracle (``oracle/``) on the same inputs and refuses to write anything if
the two disagree, so a committed fixture always means "reference == oracle on
this case".  The tests never import the reference; they only read the files.

``greenlet`` is imported unconditionally by the reference's ``kernel_api`` and
drives its work-item scopes; when the package is absent ``greenlet_shim.py``
(one thread per task, one baton) stands in for it.
"""


import os
import sys
import types
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
REPO = HERE.parent.parent
REFERENCE = Path(os.environ.get("HC_REFERENCE_ROOT", "/root/reference"))

sys.path.insert(0, str(REPO))
sys.path.insert(0, str(REFERENCE / "python"))

try:
    import greenlet  # noqa: F401
except ImportError:
    # Work-item scopes and group.barrier() need real task switching
    # (greenlet_shim.py explains).
    sys.path.insert(0, str(HERE))
    import greenlet_shim

    sys.modules["greenlet"] = greenlet_shim

from hckernel.kernel_sim import (  # noqa: E402  (the reference)
    Buffer,
    CurrentGroup,
    TunableParam,
    atomic_ref,
    create_mapping,
    kernel,
    sym,
    typename,
)

from oracle import workloads as oracle  # noqa: E402

DT = typename.DT


def cdiv(a, b):
    return (a + b - 1) // b


# ---- the workload kernels, in the reference's DSL -------------------------------
def ref_dot_kblocked():
    M, N, K, GM, GN = sym.M, sym.N, sym.K, sym.GM, sym.GN
    MI, NI, KB = sym.MI, sym.NI, sym.KB
    steps = cdiv(K, KB)
    tun = (
        TunableParam(MI, 1, range(1, 8)),
        TunableParam(NI, 1, range(1, 8)),
        TunableParam(KB, 16, range(8, 128)),
    )

    @kernel(work_shape=(cdiv(M, MI), cdiv(N, NI)), group_shape=(GM, GN), tunables=tun)
    def dot(gr: CurrentGroup, a: Buffer[M, K, DT], b: Buffer[K, N, DT], out: Buffer[M, N, DT],
            gshape: (GM, GN)):
        m0, n0 = gr.work_offset[0] * MI, gr.work_offset[1] * NI
        mb, nb = gr.shape[0] * MI, gr.shape[1] * NI
        acc = gr.zeros(shape=(mb, nb), dtype=out.dtype)
        for step in range(steps):
            k0 = step * KB
            acc += np.dot(gr.load(a[m0:, k0:], shape=(mb, KB)), gr.load(b[k0:, n0:], shape=(KB, nb)))
        gr.store(out[m0:, n0:], acc)

    return dot


def ref_dot_fullk():
    M, N, K, GM, GN = sym.M, sym.N, sym.K, sym.GM, sym.GN

    @kernel(work_shape=(M, N), group_shape=(GM, GN))
    def dot(gr: CurrentGroup, a: Buffer[M, K, DT], b: Buffer[K, N, DT], out: Buffer[M, N, DT],
            gshape: (GM, GN)):
        m0, n0 = gr.work_offset
        mb, nb = gr.shape
        acc = gr.zeros(shape=(mb, nb), dtype=out.dtype)
        acc += np.dot(gr.load(a[m0:, :], shape=(mb, K)), gr.load(b[:, n0:], shape=(K, nb)))
        gr.store(out[m0:, n0:], acc)

    return dot


def ref_w8a16():
    M, N, K, GM, GN = sym.M, sym.N, sym.K, sym.GM, sym.GN

    @kernel(work_shape=(M, N), group_shape=(GM, GN))
    def dq(gr: CurrentGroup, a: Buffer[M, K, DT], w: Buffer[K, N, DT], s: Buffer[N, DT],
           out: Buffer[M, N, DT], gshape: (GM, GN)):
        m0, n0 = gr.work_offset
        mb, nb = gr.shape
        a_t = gr.load(a[m0:, :], shape=(mb, K))
        w_t = gr.load(w[:, n0:], shape=(K, nb))
        s_t = gr.load(s[n0:], shape=nb)
        gr.store(out[m0:, n0:], np.dot(a_t, w_t.astype(np.float32)) * s_t)

    return dq


def ref_softmax():
    M, N, GM = sym.M, sym.N, sym.GM

    @kernel(work_shape=M, group_shape=GM)
    def softmax(gr: CurrentGroup, a: Buffer[M, N, DT], out: Buffer[M, N, DT], gshape: GM):
        m0 = gr.work_offset[0]
        t = gr.load(a[m0:, :], shape=(gr.shape[0], N))
        e = np.exp(t - t.max(axis=1, keepdims=True))
        gr.store(out[m0:, :], e / e.sum(axis=1, keepdims=True))

    return softmax


def ref_reduce_rows():
    M, N, GM = sym.M, sym.N, sym.GM

    @kernel(work_shape=M, group_shape=GM)
    def red(gr: CurrentGroup, x: Buffer[M, N, DT], s: Buffer[M, DT], mx: Buffer[M, DT], gshape: GM):
        m0 = gr.work_offset[0]
        t = gr.load(x[m0:, :], shape=(gr.shape[0], N))
        gr.store(s[m0:], t.sum(axis=1))
        gr.store(mx[m0:], t.max(axis=1))

    return red


def ref_reduce_all():
    WS, GS, N = sym.WS, sym.GS, sym.N

    @kernel(work_shape=cdiv(WS, N), group_shape=GS, tunables=TunableParam(N, 2, range(1, 64)))
    def red(gr: CurrentGroup, a: Buffer[WS, DT], result: Buffer[1, DT], gshape: GS):
        v = gr.load(a[gr.work_offset[0] * N :], shape=gr.size * N)
        atomic_ref(result)[0] += v.sum()

    return red


def ref_pairwise():
    M, N, D, GM, GN = sym.M, sym.N, sym.D, sym.GM, sym.GN

    @kernel(work_shape=(M, N), group_shape=(GM, GN))
    def pw(gr: CurrentGroup, a: Buffer[M, D, DT], b: Buffer[N, D, DT], out: Buffer[M, N, DT],
           gshape: (GM, GN)):
        m0, n0 = gr.work_offset
        a_t = gr.load(a[m0:, :], shape=(gr.shape[0], D))
        b_t = gr.load(b[n0:, :], shape=(gr.shape[1], D))
        gr.store(out[m0:, n0:], np.linalg.norm(a_t[:, None, :] - b_t[None, :, :], axis=2))

    return pw


def ref_conv(stride):
    """The reference's implicit-GEMM convolution (test_examples.py:203-252)."""
    N, C, H, W, NF, HF, WF = sym.N, sym.C, sym.H, sym.W, sym.NF, sym.HF, sym.WF
    KB, TN, TNF = sym.KB, sym.TN, sym.TNF
    H_OUT = (H - HF) / stride + 1
    W_OUT = (W - WF) / stride + 1
    SZ = HF * WF * C
    steps = cdiv(SZ, KB)
    tun = (
        TunableParam(TN, 8, range(1, 64)),
        TunableParam(TNF, 8, range(1, 64)),
        TunableParam(KB, 16, range(8, 128)),
    )
    x_map = create_mapping(
        lambda i, j: (i, j // (HF * WF), (j % (HF * WF)) % WF, (j % (HF * WF)) // WF))
    f_map = create_mapping(lambda i, j: (j, i // (HF * WF), i % WF, (i % (HF * WF)) // WF))
    out_map = create_mapping(lambda i, j: (i, j, 0, 0))

    @kernel(work_shape=(N, NF, H_OUT * W_OUT), group_shape=(TN, TNF, 1), tunables=tun)
    def conv(gr: CurrentGroup, x: Buffer[N, C, H, W, DT], f: Buffer[NF, C, HF, WF, DT],
             out: Buffer[N, NF, H_OUT, W_OUT, DT]):
        n0, q0, pos = gr.work_offset
        i, j = pos % W_OUT, pos // W_OUT
        x_view = gr.load(x[n0:, :, i * stride:, j * stride:], shape=(TN, SZ), mapping=x_map)
        f_view = gr.load(f[q0:, :, :, :], shape=(SZ, TNF), mapping=f_map)
        acc = gr.zeros(shape=(x_view.shape[0], f_view.shape[1]), dtype=out.dtype)
        for step in range(steps):
            k0 = step * KB
            acc += np.dot(gr.vload(x_view[:, k0:], shape=(TN, KB)),
                          gr.vload(f_view[k0:, :], shape=(KB, TNF)))
        gr.store(out[n0:, q0:, i:, j:], acc, mapping=out_map)

    return conv


def ref_map(fn, count, rank, group):
    """An element-wise body in the reference's DSL: one tile per input loaded at
    the group's offset, ``fn`` of them stored at the same offset."""
    W, H = sym.W, sym.H
    if rank == 1:
        @kernel(work_shape=W, group_shape=group[0])
        def k1(gr: CurrentGroup, a: Buffer[W, DT], out: Buffer[W, DT]):
            x = gr.work_offset[0]
            gr.store(out[x:], fn(gr.load(a[x:], shape=gr.shape[0])))

        return k1
    if count == 1:
        @kernel(work_shape=(W, H), group_shape=group)
        def k2(gr: CurrentGroup, a: Buffer[W, H, DT], out: Buffer[W, H, DT]):
            x, y = gr.work_offset
            gr.store(out[x:, y:], fn(gr.load(a[x:, y:], shape=gr.shape)))

        return k2
    if count == 2:
        @kernel(work_shape=(W, H), group_shape=group)
        def k3(gr: CurrentGroup, a: Buffer[W, H, DT], b: Buffer[W, H, DT], out: Buffer[W, H, DT]):
            x, y = gr.work_offset
            gr.store(out[x:, y:], fn(gr.load(a[x:, y:], shape=gr.shape),
                                     gr.load(b[x:, y:], shape=gr.shape)))

        return k3

    @kernel(work_shape=(W, H), group_shape=group)
    def k4(gr: CurrentGroup, a: Buffer[W, H, DT], b: Buffer[W, H, DT], c: Buffer[W, H, DT],
           out: Buffer[W, H, DT]):
        x, y = gr.work_offset
        gr.store(out[x:, y:], fn(gr.load(a[x:, y:], shape=gr.shape),
                                 gr.load(b[x:, y:], shape=gr.shape),
                                 gr.load(c[x:, y:], shape=gr.shape)))

    return k4


def ref_rows(fn, count):
    """A row body in the reference's DSL: whole rows loaded, ``fn`` stored."""
    M, N, GM = sym.M, sym.N, sym.GM
    if count == 1:
        @kernel(work_shape=M, group_shape=GM)
        def r1(gr: CurrentGroup, a: Buffer[M, N, DT], out: Buffer[M, N, DT], gshape: GM):
            m0 = gr.work_offset[0]
            gr.store(out[m0:, :], fn(gr.load(a[m0:, :], shape=(gr.shape[0], N))))

        return r1

    @kernel(work_shape=M, group_shape=GM)
    def r2(gr: CurrentGroup, a: Buffer[M, N, DT], b: Buffer[M, N, DT], out: Buffer[M, N, DT],
           gshape: GM):
        m0 = gr.work_offset[0]
        gr.store(out[m0:, :], fn(gr.load(a[m0:, :], shape=(gr.shape[0], N)),
                                 gr.load(b[m0:, :], shape=(gr.shape[0], N))))

    return r2


def ref_copy():
    W, H = sym.W, sym.H

    @kernel(work_shape=(W, H), group_shape=(4, 16))
    def cp(gr: CurrentGroup, src: Buffer[W, H, DT], dst: Buffer[W, H, DT]):
        x, y = gr.work_offset
        gr.store(dst[x:, y:], gr.load(src[x:, y:], shape=gr.shape))

    return cp


def same(name, ref, got):
    if ref.shape != got.shape or not np.array_equal(ref, got, equal_nan=True):
        raise SystemExit(f"oracle differs from the reference on {name}")


def main():
    out = {}

    # 1. The reference's own test vectors (test_examples.py:113-121, 157-165,
    #    323-335, 42-47): same inputs, outputs taken from the reference run.
    m, n, k = 16, 32, 64
    a = 2 * np.arange(m * k).reshape(m, k) / (m * k)
    b = np.arange(n * k).reshape(k, n) / (n * k)
    r = np.zeros((m, n))
    ref_dot_kblocked()(a, b, r, (8, 8))
    assert np.array_equal(r, np.dot(a, b))  # what the reference test asserts
    o = np.zeros((m, n))
    oracle.gemm_kblocked(a, b, o, (8, 8), kb=16)
    same("dot_kblocked_f64", r, o)
    out["kat_dot_kblocked_f64"] = r
    r2 = np.zeros((m, n))
    ref_dot_fullk()(a, b, r2, (8, 8))
    o = np.zeros((m, n))
    oracle.gemm_fullk(a, b, o, (8, 8))
    same("dot_fullk_f64", r2, o)
    out["kat_dot_fullk_f64"] = r2

    m, n = 30, 25
    a = 2 * np.arange(m * n).reshape(m, n) / (m * n)
    r = np.zeros((m, n))
    ref_softmax()(a, r, 8)
    o = np.zeros((m, n))
    oracle.softmax_rows(a, o, 8)
    same("softmax_f64", r, o)
    out["kat_softmax_f64"] = r

    a = np.arange(0, 20)
    r = np.zeros(1)
    ref_reduce_all()(a, r, 8)
    assert r[0] == a.sum()
    o = np.zeros(1)
    oracle.reduce_sum_all(a, o, 8, 2)
    same("reduce_all", r, o)
    out["kat_reduce_all"] = r

    # 2. Ragged copy (shapes of test_e2e.py:46-54 that exercise clipping).
    for shape in [(1, 27), (10, 20), (111, 813)]:
        src = np.arange(shape[0] * shape[1], dtype=np.int32).reshape(shape)
        r = np.zeros_like(src)
        ref_copy()(src, r)
        o = np.zeros_like(src)
        oracle.copy2d(src, o, (4, 16))
        same(f"copy{shape}", r, o)
        out[f"copy_{shape[0]}x{shape[1]}"] = r

    # 3. Reduced-size instances of the five benchmark configurations, inputs
    #    from oracle.make_inputs (seeded), outputs from the reference simulator.
    a, b = oracle.make_inputs("gemm_f32")  # config 1 at full size
    r = np.zeros((256, 256), np.float32)
    ref_dot_kblocked()(a, b, r, (64, 64))
    o = np.zeros_like(r)
    oracle.gemm_kblocked(a, b, o, (64, 64), kb=16)
    same("cfg1", r, o)
    out["cfg1_gemm_f32_256"] = r

    a, b = oracle.make_inputs("gemm_f32", shape=(70, 45, 33))  # ragged edges
    r = np.zeros((70, 45), np.float32)
    ref_dot_kblocked()(a, b, r, (64, 64))
    o = np.zeros_like(r)
    oracle.gemm_kblocked(a, b, o, (64, 64), kb=16)
    same("cfg1_ragged", r, o)
    out["cfg1_gemm_f32_70x45x33"] = r

    (x,) = oracle.make_inputs("softmax", shape=(48, 4096))
    r = np.zeros_like(x)
    ref_softmax()(x, r, 32)
    o = np.zeros_like(x)
    oracle.softmax_rows(x, o, 32)
    same("cfg2", r, o)
    out["cfg2_softmax_48x4096"] = r
    (x,) = oracle.make_inputs("softmax", shape=(30, 25))
    r = np.zeros_like(x)
    ref_softmax()(x, r, 8)
    o = np.zeros_like(x)
    oracle.softmax_rows(x, o, 8)
    same("cfg2_ragged", r, o)
    out["cfg2_softmax_30x25"] = r

    (x,) = oracle.make_inputs("reduce", shape=(300, 8192))
    rs, rm = np.zeros(300, np.float32), np.zeros(300, np.float32)
    ref_reduce_rows()(x, rs, rm, 256)
    os_, om = np.zeros_like(rs), np.zeros_like(rm)
    oracle.reduce_rows(x, os_, om, 256)
    same("cfg3_sum", rs, os_)
    same("cfg3_max", rm, om)
    out["cfg3_sum_300x8192"] = rs
    out["cfg3_max_300x8192"] = rm
    (x,) = oracle.make_inputs("reduce", shape=(37, 101))
    rs, rm = np.zeros(37, np.float32), np.zeros(37, np.float32)
    ref_reduce_rows()(x, rs, rm, 16)
    os_, om = np.zeros_like(rs), np.zeros_like(rm)
    oracle.reduce_rows(x, os_, om, 16)
    same("cfg3r_sum", rs, os_)
    same("cfg3r_max", rm, om)
    out["cfg3_sum_37x101"] = rs
    out["cfg3_max_37x101"] = rm

    a, b = oracle.make_inputs("gemm_bf16", shape=(256, 512, 384))
    r = np.zeros((256, 512), np.float32)
    ref_dot_fullk()(a, b, r, (256, 256))
    r = oracle.round_to_bf16(r)
    o = np.zeros_like(r)
    oracle.gemm_bf16(a, b, o, (256, 256))
    same("cfg4", r, o)
    out["cfg4_gemm_bf16_256x512x384_bits"] = oracle.bf16_bits(r)

    a, w, s = oracle.make_inputs("gemm_w8a16", shape=(128, 256, 512))
    r = np.zeros((128, 256), np.float32)
    ref_w8a16()(a, w, s, r, (128, 128))
    r = oracle.round_to_bf16(r)
    o = np.zeros_like(r)
    oracle.gemm_w8a16(a, w, s, o, (128, 128))
    same("cfg5", r, o)
    out["cfg5_gemm_w8a16_128x256x512_bits"] = oracle.bf16_bits(r)

    # 4. Pairwise distance: the reference's own vector (test_examples.py:291-301)
    #    and a ragged float32 case.
    m, n, d = 16, 32, 8
    a = 2 * np.arange(m * d).reshape(m, d) / (m * d)
    b = np.arange(n * d).reshape(n, d) / (n * d)
    r = np.zeros((m, n))
    ref_pairwise()(a, b, r, (8, 8))
    assert np.array_equal(r, np.linalg.norm(a[:, None, :] - b[None, :, :], axis=2))
    o = np.zeros((m, n))
    oracle.pairwise_distance(a, b, o, (8, 8))
    same("pairwise_f64", r, o)
    out["kat_pairwise_f64"] = r
    rng = np.random.default_rng(5)
    a = rng.standard_normal((70, 19)).astype(np.float32)
    b = rng.standard_normal((45, 19)).astype(np.float32)
    r = np.zeros((70, 45), np.float32)
    ref_pairwise()(a, b, r, (16, 8))
    o = np.zeros_like(r)
    oracle.pairwise_distance(a, b, o, (16, 8))
    same("pairwise_f32", r, o)
    out["pairwise_f32_70x45x19"] = r

    # 5. Implicit-GEMM convolution through index mappings: the grid of the
    #    reference's own test (test_examples.py:168-176; for square images and
    #    filters the result also equals the plain correlation that test compares
    #    with) and cases beyond it.
    TN, TNF, KB = sym.TN, sym.TNF, sym.KB
    for name, x_shape, f_shape, stride, dtype, (tn, tnf, kb) in oracle.conv_golden_cases():
        x, f = oracle.make_conv_inputs(x_shape, f_shape, dtype)
        shape = oracle.conv_out_shape(x_shape, f_shape, stride)
        r = np.zeros(shape, dtype)
        ref_conv(stride).parametrize({TN: tn, TNF: tnf, KB: kb})(x, f, r)
        o = np.zeros(shape, dtype)
        oracle.conv_implicit_gemm(x, f, o, stride, tn, tnf, kb)
        same(name, r, o)
        square = x_shape[2] == x_shape[3] and f_shape[2] == f_shape[3]
        if square and (x_shape[2] - f_shape[2]) % stride == 0:
            np.testing.assert_allclose(r, oracle.conv_direct(x, f, stride),
                                       rtol=1e-4 if dtype == "float32" else 1e-10, atol=1e-5)
        out[name] = r

    # 6. Element-wise bodies (tile arithmetic between a load and a store).
    for name, fn, count, shape, dtype, group in oracle.elementwise_cases():
        inputs = oracle.make_elementwise_inputs(count, shape, dtype)
        r = np.zeros(shape, dtype)
        with np.errstate(all="ignore"):
            ref_map(fn, count, len(shape), group)(*inputs, r)
        o = np.zeros(shape, dtype)
        oracle.elementwise(fn, inputs, o, group)
        same(name, r, o)
        # Plain NumPy on whole arrays agrees up to the last bit or two: the
        # reference's tiles carry Python-float operands on in float64 where
        # NumPy arrays stay in float32.
        np.testing.assert_allclose(r, fn(*inputs), rtol=3e-7 if dtype == "float32" else 0)
        out[name] = r

    # 6b. The rest of the tile operator table and the masked store: elements the
    #     arithmetic masks (zero divisors, results that are not finite) stay -77.
    for name, fn, inputs, group in oracle.operator_cases():
        shape, dtype = inputs[0].shape, inputs[0].dtype
        r = np.full(shape, -77, dtype)
        with np.errstate(all="ignore"):
            ref_map(fn, len(inputs), 2, group)(*inputs, r)
        o = np.full(shape, -77, dtype)
        oracle.elementwise(fn, list(inputs), o, group)
        same(name, r, o)
        assert (r == -77).any() or "compare" in name or "equal" in name or "i64" in name, name
        out[name] = r

    # 6c. Work-item bodies: the work-item form of the pairwise distance
    #     (docs/langref.md:47-63), neighbour reads, local ids, and two phases
    #     separated by group.barrier() that exchange values through a group tile.
    import hckernel.kernel_sim as ref_sim

    ns = types.SimpleNamespace(kernel=ref_sim.kernel, sym=sym, CurrentGroup=CurrentGroup,
                               Buffer=Buffer, DT=DT, target={}, atomic_ref=atomic_ref)
    from oracle import workitems as oracle_items

    for case in oracle_items.work_item_cases():
        shape, dtype = case["out"]
        r = np.full(shape, -77, dtype)
        case["make"](ns)(*case["inputs"], r)
        o = np.full(shape, -77, dtype)
        case["oracle"](case["inputs"], o)
        same(case["name"], r, o)
        out[case["name"]] = r

    # 6d. Sub-group bodies: every sub-group works on its part of the group's tile.
    for case in oracle_items.subgroup_cases():
        shape, dtype = case["out"]
        r = np.full(shape, -77, dtype)
        case["make"](ns)(*case["inputs"], r)
        o = np.full(shape, -77, dtype)
        case["oracle"](case["inputs"], o)
        same(case["name"], r, o)
        out[case["name"]] = r

    # 7. Row bodies: reductions along the rows used again in the same expression.
    for name, fn, count, shape, dtype, group_rows in oracle.rowwise_cases():
        inputs = oracle.make_elementwise_inputs(count, shape, dtype, seed=8)
        r = np.zeros(shape, dtype)
        with np.errstate(all="ignore"):
            ref_rows(fn, count)(*inputs, r, group_rows)
        o = np.zeros(shape, dtype)
        oracle.rowwise(fn, inputs, o, group_rows)
        same(name, r, o)
        np.testing.assert_allclose(r, fn(*inputs), rtol=2e-6 if dtype == "float32" else 1e-14,
                                   atol=1e-6 if dtype == "float32" else 0)
        out[name] = r

    np.savez_compressed(HERE / "reference_outputs.npz", **out)
    (HERE / "VERSIONS.txt").write_text(
        f"numpy {np.__version__}\n"
        f"blas {np.show_config(mode='dicts')['Build Dependencies']['blas'].get('name', '?')} "
        f"{np.show_config(mode='dicts')['Build Dependencies']['blas'].get('version', '?')}\n"
        f"python {sys.version.split()[0]}\n"
        "generated by tests/golden/make_golden.py from the reference simulator\n"
    )
    print("wrote", HERE / "reference_outputs.npz", {k: v.shape for k, v in out.items()})


if __name__ == "__main__":
    main()
