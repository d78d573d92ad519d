"""The benchmark workloads written in the kernel DSL, bound to a device.

Each body is what a user of the reference would write (and what its tests
write: python/hckernel/tests/test_examples.py:88-111, 136-155, 312-321;
tests/test_e2e.py:66-70); :func:`make_kernels` decorates them for one GPU.
Calling one of the returned kernels goes through the whole product path:
symbol binding, recording, family recognition, the C++ dispatcher, the C-ABI
and a precompiled sm_100a kernel.
"""

import types

import numpy as np

from .hckernel.kernel import Buffer, CurrentGroup, TunableParam, kernel, sym, typename

DT = typename.DT


def _cdiv(a, b):
    return (a + b - 1) // b


def make_kernels(device="cuda:0"):
    """Namespace with ``copy``, ``softmax``, ``reduce_rows``, ``dot``,
    ``dot_fullk`` and ``dequant_dot`` kernels that run on ``device``."""
    target = dict(backend="nvvm", device=device)
    M, N, K, W, H = sym.M, sym.N, sym.K, sym.W, sym.H
    GM, GN, MI, NI, KB = sym.GM, sym.GN, sym.MI, sym.NI, sym.KB

    @kernel(work_shape=(W, H), **target)
    def copy(group: CurrentGroup, src: Buffer[W, H, DT], dst: Buffer[W, H, DT]):
        x, y = group.work_offset
        group.store(dst[x:, y:], group.load(src[x:, y:], shape=group.shape))

    @kernel(work_shape=M, group_shape=GM, **target)
    def softmax(gr: CurrentGroup, a: Buffer[M, N, DT], out: Buffer[M, N, DT], gshape: GM):
        m0 = gr.work_offset[0]
        rows = gr.load(a[m0:, :], shape=(gr.shape[0], N))
        e = np.exp(rows - rows.max(axis=1, keepdims=True))
        gr.store(out[m0:, :], e / e.sum(axis=1, keepdims=True))

    @kernel(work_shape=M, group_shape=GM, **target)
    def reduce_rows(gr: CurrentGroup, x: Buffer[M, N, DT], s: Buffer[M, DT], mx: Buffer[M, DT],
                    gshape: GM):
        m0 = gr.work_offset[0]
        rows = gr.load(x[m0:, :], shape=(gr.shape[0], N))
        gr.store(s[m0:], rows.sum(axis=1))
        gr.store(mx[m0:], rows.max(axis=1))

    steps = _cdiv(K, KB)
    tunables = (
        TunableParam(MI, 1, range(1, 8)),
        TunableParam(NI, 1, range(1, 8)),
        TunableParam(KB, 16, range(8, 128)),
    )

    @kernel(work_shape=(_cdiv(M, MI), _cdiv(N, NI)), group_shape=(GM, GN), tunables=tunables,
            **target)
    def dot(gr: CurrentGroup, a: Buffer[M, K, DT], b: Buffer[K, N, DT], out: Buffer[M, N, DT],
            gshape: (GM, GN)):
        m0, n0 = gr.work_offset[0] * MI, gr.work_offset[1] * NI
        mb, nb = gr.shape[0] * MI, gr.shape[1] * NI
        acc = gr.zeros(shape=(mb, nb), dtype=out.dtype)
        for step in range(steps):
            k0 = step * KB
            acc += np.dot(gr.load(a[m0:, k0:], shape=(mb, KB)),
                          gr.load(b[k0:, n0:], shape=(KB, nb)))
        gr.store(out[m0:, n0:], acc)

    @kernel(work_shape=(M, N), group_shape=(GM, GN), **target)
    def dot_fullk(gr: CurrentGroup, a: Buffer[M, K, DT], b: Buffer[K, N, DT],
                  out: Buffer[M, N, DT], gshape: (GM, GN)):
        m0, n0 = gr.work_offset
        mb, nb = gr.shape
        acc = gr.zeros(shape=(mb, nb), dtype=out.dtype)
        acc += np.dot(gr.load(a[m0:, :], shape=(mb, K)), gr.load(b[:, n0:], shape=(K, nb)))
        gr.store(out[m0:, n0:], acc)

    @kernel(work_shape=(M, N), group_shape=(GM, GN), **target)
    def dequant_dot(gr: CurrentGroup, a: Buffer[M, K, DT], w: Buffer[K, N, DT], s: Buffer[N, DT],
                    out: Buffer[M, N, DT], gshape: (GM, GN)):
        m0, n0 = gr.work_offset
        mb, nb = gr.shape
        a_t = gr.load(a[m0:, :], shape=(mb, K))
        w_t = gr.load(w[:, n0:], shape=(K, nb))
        s_t = gr.load(s[n0:], shape=nb)
        gr.store(out[m0:, n0:], np.dot(a_t, w_t.astype(np.float32)) * s_t)

    return types.SimpleNamespace(copy=copy, softmax=softmax, reduce_rows=reduce_rows, dot=dot,
                                 dot_fullk=dot_fullk, dequant_dot=dequant_dot, device=device)


def make_elementwise(fn, inputs=1, rank=2, group_shape=None, device="cuda:0"):
    """An element-wise kernel ``k(a[, b[, c]], out)``: every work-group loads one
    tile per input at its offset, stores ``fn`` of them at the same offset.
    ``fn`` is written with operators and NumPy calls (``np.maximum``, ``np.exp``,
    ``np.sqrt``, ``np.abs`` ...) on tiles, as in the reference's tile arithmetic
    (python/hckernel/kernel_api.py:136-211)."""
    target = dict(backend="nvvm", device=device)
    W, H = sym.W, sym.H
    if rank == 1:
        if inputs != 1:
            raise ValueError("vector kernels take one input here")

        @kernel(work_shape=W, group_shape=group_shape and group_shape[0], **target)
        def map1(gr: CurrentGroup, a: Buffer[W, DT], out: Buffer[W, DT]):
            x = gr.work_offset[0]
            gr.store(out[x:], fn(gr.load(a[x:], shape=gr.shape[0])))

        return map1
    if inputs == 1:
        @kernel(work_shape=(W, H), group_shape=group_shape, **target)
        def map2(gr: CurrentGroup, a: Buffer[W, H, DT], out: Buffer[W, H, DT]):
            x, y = gr.work_offset
            gr.store(out[x:, y:], fn(gr.load(a[x:, y:], shape=gr.shape)))

        return map2
    if inputs == 2:
        @kernel(work_shape=(W, H), group_shape=group_shape, **target)
        def map3(gr: CurrentGroup, a: Buffer[W, H, DT], b: Buffer[W, H, DT], out: Buffer[W, H, DT]):
            x, y = gr.work_offset
            gr.store(out[x:, y:], fn(gr.load(a[x:, y:], shape=gr.shape),
                                     gr.load(b[x:, y:], shape=gr.shape)))

        return map3
    if inputs == 3:
        @kernel(work_shape=(W, H), group_shape=group_shape, **target)
        def map4(gr: CurrentGroup, a: Buffer[W, H, DT], b: Buffer[W, H, DT], c: Buffer[W, H, DT],
                 out: Buffer[W, H, DT]):
            x, y = gr.work_offset
            gr.store(out[x:, y:], fn(gr.load(a[x:, y:], shape=gr.shape),
                                     gr.load(b[x:, y:], shape=gr.shape),
                                     gr.load(c[x:, y:], shape=gr.shape)))

        return map4
    raise ValueError("one to three inputs")


def make_rowwise(fn, inputs=1, device="cuda:0"):
    """A row kernel ``k(a[, b], out, group_rows)``: every work-group loads whole
    rows of each input, stores ``fn`` of them.  ``fn`` may reduce along the rows
    (``.sum/.max/.mean(axis=1, keepdims=True)``) and use the reduced values
    again, like the reference's softmax body
    (python/hckernel/tests/test_examples.py:312-321)."""
    target = dict(backend="nvvm", device=device)
    M, N, GM = sym.M, sym.N, sym.GM
    if inputs == 1:
        @kernel(work_shape=M, group_shape=GM, **target)
        def rows1(gr: CurrentGroup, a: Buffer[M, N, DT], out: Buffer[M, N, DT], gshape: GM):
            m0 = gr.work_offset[0]
            gr.store(out[m0:, :], fn(gr.load(a[m0:, :], shape=(gr.shape[0], N))))

        return rows1
    if inputs == 2:
        @kernel(work_shape=M, group_shape=GM, **target)
        def rows2(gr: CurrentGroup, a: Buffer[M, N, DT], b: Buffer[M, N, DT], out: Buffer[M, N, DT],
                  gshape: GM):
            m0 = gr.work_offset[0]
            gr.store(out[m0:, :], fn(gr.load(a[m0:, :], shape=(gr.shape[0], N)),
                                     gr.load(b[m0:, :], shape=(gr.shape[0], N))))

        return rows2
    raise ValueError("one or two inputs")


def make_work_item_bodies(device="cuda:0"):
    """Two bodies written at work-item level (python/hckernel/kernel_api.py:395-431),
    on matrices [W, H] with work-groups of 4 x 64 work-items:

    ``rotate(a, out)``: every work-item puts ``a + 1`` into the group's tile,
    the group meets at a barrier, and each takes half of the element five
    columns on (wrapping inside its row of the tile);
    ``stencil(a, out)``: ``out[i, j] = a[i, j] + a[i, j + 1] / 2`` wherever the
    neighbour exists."""
    target = dict(backend="nvvm", device=device)
    W, H = sym.W, sym.H

    @kernel(work_shape=(W, H), group_shape=(4, 64), **target)
    def rotate(group: CurrentGroup, a: Buffer[W, H, DT], out: Buffer[W, H, DT]):
        tmp = group.zeros(shape=group.shape, dtype=a.dtype)

        @group.workitems
        def inner(w):
            (li, lj), (i, j) = w.local_id()[:2], w.global_id()[:2]
            if i < a.shape[0] and j < a.shape[1]:
                tmp[li, lj] = a[i, j] + 1.0
            group.barrier()
            if i < a.shape[0] and j < a.shape[1]:
                out[i, j] = tmp.data[li, (lj + 5) % 64] * 0.5

        inner()

    @kernel(work_shape=(W, H), group_shape=(4, 64), **target)
    def stencil(group: CurrentGroup, a: Buffer[W, H, DT], out: Buffer[W, H, DT]):
        @group.workitems
        def inner(w):
            i, j = w.global_id()[:2]
            if i < a.shape[0] and j + 1 < a.shape[1]:
                out[i, j] = a[i, j] + a[i, j + 1] * 0.5

        inner()

    return types.SimpleNamespace(rotate=rotate, stencil=stencil)


def make_conv(stride=1, device="cuda:0"):
    """The convolution written as an implicit GEMM, as in the reference's
    example (python/hckernel/tests/test_examples.py:203-252): ``conv(x, f, out)``
    with x [N, C, H, W], f [NF, C, HF, WF], out [N, NF, H_OUT, W_OUT], no
    padding.  A work-group of (TN, TNF, 1) gathers TN receptive fields and TNF
    filters through index mappings, multiplies them in K blocks of KB and
    scatters the (TN, TNF) products to one output position.  TN, TNF and KB are
    tunables (defaults 8, 8, 16): ``conv.parametrize({sym.TN: 32, ...})``."""
    from .hckernel.kernel import create_mapping

    N, C, H, W, NF, HF, WF = sym.N, sym.C, sym.H, sym.W, sym.NF, sym.HF, sym.WF
    KB, TN, TNF = sym.KB, sym.TN, sym.TNF
    H_OUT = (H - HF) / stride + 1
    W_OUT = (W - WF) / stride + 1
    SZ = HF * WF * C
    steps = _cdiv(SZ, KB)
    tunables = (
        TunableParam(TN, 8, range(1, 64)),
        TunableParam(TNF, 8, range(1, 64)),
        TunableParam(KB, 16, range(8, 128)),
    )
    x_map = create_mapping(
        lambda i, j: (i, j // (HF * WF), (j % (HF * WF)) % WF, (j % (HF * WF)) // WF))
    f_map = create_mapping(lambda i, j: (j, i // (HF * WF), i % WF, (i % (HF * WF)) // WF))
    out_map = create_mapping(lambda i, j: (i, j, 0, 0))

    @kernel(work_shape=(N, NF, H_OUT * W_OUT), group_shape=(TN, TNF, 1), tunables=tunables,
            backend="nvvm", device=device)
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
