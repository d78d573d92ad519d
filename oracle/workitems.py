"""Work-item bodies: the CPU restatement and the cases pinned under
``tests/golden``.  Test infrastructure: imported by ``tests/`` and by the golden
generator only.

Kept apart from ``workloads.py`` because the kernels below are written in the
DSL with real annotation objects (``Buffer[W, H, DT]``), which the reference's
decorator inspects (python/hckernel/kernel_sim.py:42-127); a module with
postponed annotations would hand it strings.
"""

import numpy as np

from .hcsim import iter_groups


def run_work_items(phases, work_shape, group_shape, tile_dtype=None) -> None:
    """Work-item scope with barriers (python/hckernel/kernel_api.py:395-431): per
    work-group, every work-item runs up to the barrier before any goes on - the
    reference's greenlets hand over to the next work-item at ``group.barrier()``
    and wrap round, which for a function that is straight-line between barriers
    is exactly "phase by phase, work-items in row-major order".  ``phases`` is
    the work-item function cut at its barriers: callables
    ``(local id, global id, group shape, tile)``; ``tile`` is the group's zeroed
    tile (``group.zeros(group.shape)``), fresh for every work-group."""
    for _, offset in iter_groups(work_shape, group_shape):
        group_shape_t = tuple(np.atleast_1d(group_shape).tolist())
        tile = np.zeros(group_shape_t, tile_dtype) if tile_dtype is not None else None
        for phase in phases:
            for lid in np.ndindex(*group_shape_t):
                gid = tuple(o + l for o, l in zip(offset, lid))
                phase(lid, gid, group_shape_t, tile)


def work_item_cases():
    """The work-item bodies stored under ``tests/golden``: ``name``, ``make``
    (the kernel in the DSL, given a namespace with ``kernel``, ``sym``,
    ``CurrentGroup``, ``Buffer``, ``DT`` and the decorator's extra keywords, so
    that the same source runs on the reference simulator and on the front door),
    ``inputs``, ``out`` (shape, dtype), ``args`` after the arrays, ``oracle``
    (the restatement: a function of inputs and out)."""
    rng = np.random.default_rng(17)

    def pairwise(ns):
        W1, W2, H = ns.sym.W1, ns.sym.W2, ns.sym.H

        @ns.kernel(work_shape=(W1, W2), group_shape=(4, 4), **ns.target)
        def k(group: ns.CurrentGroup, X1: ns.Buffer[W1, H, ns.DT], X2: ns.Buffer[W2, H, ns.DT],
              D: ns.Buffer[W1, W2, ns.DT]):
            # docs/langref.md:47-63
            @group.workitems
            def inner(ind):
                i, j = ind.global_id()
                if i < X1.shape[0] and j < X2.shape[0]:
                    d = ((X1[i] - X2[j]) ** 2).sum()
                    D[i, j] = np.sqrt(d)

            inner()

        return k

    def pairwise_oracle(ins, out):
        x1, x2 = ins

        def phase(lid, gid, group, tile):
            i, j = gid
            if i < x1.shape[0] and j < x2.shape[0]:
                out[i, j] = np.sqrt(((x1[i] - x2[j]) ** 2).sum())

        run_work_items([phase], out.shape, (4, 4))

    def reverse(ns):
        G = ns.sym.G

        @ns.kernel(work_shape=G, group_shape=8, **ns.target)
        def k(group: ns.CurrentGroup, a: ns.Buffer[G, ns.DT], out: ns.Buffer[G, ns.DT]):
            tmp = group.zeros(shape=group.shape[0], dtype=a.dtype)

            @group.workitems
            def inner(wi):
                lid, gid = wi.local_id()[0], wi.global_id()[0]
                if gid < a.shape[0]:
                    tmp[lid] = a[gid] * 2.0
                group.barrier()
                if gid < a.shape[0]:
                    out[gid] = tmp.data[group.shape[0] - 1 - lid] + lid

            inner()

        return k

    def reverse_oracle(ins, out):
        (a,) = ins

        def first(lid, gid, group, tile):
            if gid[0] < a.shape[0]:
                tile[lid[0]] = a[gid[0]] * 2.0

        def second(lid, gid, group, tile):
            if gid[0] < a.shape[0]:
                out[gid[0]] = tile[group[0] - 1 - lid[0]] + lid[0]

        run_work_items([first, second], out.shape, 8, a.dtype)

    def stencil(ns):
        W, H = ns.sym.W, ns.sym.H

        @ns.kernel(work_shape=(W, H), group_shape=(4, 8), **ns.target)
        def k(group: ns.CurrentGroup, a: ns.Buffer[W, H, ns.DT], out: ns.Buffer[W, H, ns.DT]):
            @group.workitems
            def inner(wi):
                i, j = wi.global_id()
                if i < a.shape[0] and j + 1 < a.shape[1] and i >= 1:
                    out[i, j] = a[i, j + 1] - a[i - 1, j] + a[i, j] * 0.5

            inner()

        return k

    def stencil_oracle(ins, out):
        (a,) = ins

        def phase(lid, gid, group, tile):
            i, j = gid
            if i < a.shape[0] and j + 1 < a.shape[1] and i >= 1:
                out[i, j] = a[i, j + 1] - a[i - 1, j] + a[i, j] * 0.5

        run_work_items([phase], out.shape, (4, 8))

    def local_ids(ns):
        W, H = ns.sym.W, ns.sym.H

        @ns.kernel(work_shape=(W, H), group_shape=(2, 4), **ns.target)
        def k(group: ns.CurrentGroup, a: ns.Buffer[W, H, ns.DT], out: ns.Buffer[W, H, ns.DT]):
            @group.workitems
            def inner(wi):
                li, lj = wi.local_id()
                i, j = wi.global_id()
                if i < a.shape[0] and j < a.shape[1]:
                    out[i, j] = a[i, j] * li + lj * 10.0 + i

            inner()

        return k

    def local_ids_oracle(ins, out):
        (a,) = ins

        def phase(lid, gid, group, tile):
            if gid[0] < a.shape[0] and gid[1] < a.shape[1]:
                out[gid] = a[gid] * lid[0] + lid[1] * 10.0 + gid[0]

        run_work_items([phase], out.shape, (2, 4))

    def mirror(ns):
        W, H = ns.sym.W, ns.sym.H

        @ns.kernel(work_shape=(W, H), group_shape=(4, 8), **ns.target)
        def k(group: ns.CurrentGroup, a: ns.Buffer[W, H, ns.DT], b: ns.Buffer[W, H, ns.DT],
              out: ns.Buffer[W, H, ns.DT]):
            tmp = group.zeros(shape=group.shape, dtype=a.dtype)

            @group.workitems
            def inner(wi):
                li, lj = wi.local_id()
                i, j = wi.global_id()
                if i < a.shape[0] and j < a.shape[1]:
                    tmp[li, lj] = a[i, j] - b[i, j]
                group.barrier()
                if i < a.shape[0] and j < a.shape[1]:
                    out[i, j] = tmp.data[li, group.shape[1] - 1 - lj] * 2.0 \
                        + tmp.data[(li + 1) % 4, lj] - a[i, j]

            inner()

        return k

    def mirror_oracle(ins, out):
        a, b = ins

        def first(lid, gid, group, tile):
            if gid[0] < a.shape[0] and gid[1] < a.shape[1]:
                tile[lid] = a[gid] - b[gid]

        def second(lid, gid, group, tile):
            if gid[0] < a.shape[0] and gid[1] < a.shape[1]:
                out[gid] = tile[lid[0], group[1] - 1 - lid[1]] * 2.0 \
                    + tile[(lid[0] + 1) % 4, lid[1]] - a[gid]

        run_work_items([first, second], out.shape, (4, 8), a.dtype)

    f32, f64 = np.float32, np.float64
    return [
        dict(name="wi_pairwise_f64", make=pairwise, oracle=pairwise_oracle,
             inputs=[rng.standard_normal((10, 5)), rng.standard_normal((7, 5))],
             out=((10, 7), f64)),
        dict(name="wi_pairwise_f32", make=pairwise, oracle=pairwise_oracle,
             inputs=[rng.standard_normal((33, 19)).astype(f32),
                     rng.standard_normal((18, 19)).astype(f32)], out=((33, 18), f32)),
        dict(name="wi_reverse_in_group_f32", make=reverse, oracle=reverse_oracle,
             inputs=[rng.standard_normal(20).astype(f32)], out=((20,), f32)),
        dict(name="wi_reverse_in_group_f64", make=reverse, oracle=reverse_oracle,
             inputs=[rng.standard_normal(64)], out=((64,), f64)),
        dict(name="wi_stencil_f32", make=stencil, oracle=stencil_oracle,
             inputs=[rng.standard_normal((11, 21)).astype(f32)], out=((11, 21), f32)),
        dict(name="wi_local_ids_f64", make=local_ids, oracle=local_ids_oracle,
             inputs=[rng.standard_normal((7, 10))], out=((7, 10), f64)),
        dict(name="wi_mirror_exchange_f32", make=mirror, oracle=mirror_oracle,
             inputs=[rng.standard_normal((10, 19)).astype(f32),
                     rng.standard_normal((10, 19)).astype(f32)], out=((10, 19), f32)),
    ]


def run_subgroups(body, work_shape, group_shape, subgroup_size) -> None:
    """Sub-group scope (python/hckernel/kernel_api.py:266-272, 378-393): per
    work-group, ``body(work offset, sub-group id, size)`` once for every index
    of the leading group axes and every ``size``-wide piece of the last one, in
    row-major order."""
    group_shape_t = tuple(np.atleast_1d(group_shape).tolist())
    pieces = -(-group_shape_t[-1] // subgroup_size)
    for _, offset in iter_groups(work_shape, group_shape):
        for sgid in np.ndindex(*group_shape_t[:-1], pieces):
            body(offset, sgid, subgroup_size)


def subgroup_cases():
    """Bodies written at sub-group level, pinned under ``tests/golden`` like the
    work-item cases: every sub-group loads its part of the group's tile at
    ``work_offset + subgroup_id * (1, ..., size)``, computes, and stores it at
    the same place.  Elements beyond the arrays are masked by the load and
    skipped by the store (python/hckernel/kernel_api.py:297-340)."""
    rng = np.random.default_rng(23)

    def scale_shift(ns):
        G = ns.sym.G

        @ns.kernel(work_shape=G, group_shape=64, subgroup_size=16, **ns.target)
        def k(gr: ns.CurrentGroup, a: ns.Buffer[G, ns.DT], out: ns.Buffer[G, ns.DT]):
            @gr.subgroups
            def inner(sg):
                n = sg.size()
                x = gr.work_offset[0] + sg.subgroup_id()[0] * n
                gr.store(out[x:], gr.load(a[x:], shape=n) * 2.0 + 1.0)

            inner()

        return k

    def scale_shift_oracle(ins, out):
        (a,) = ins

        def body(offset, sgid, n):
            x = offset[0] + sgid[0] * n
            out[x:x + n] = a[x:x + n] * 2.0 + 1.0

        run_subgroups(body, out.shape, 64, 16)

    def rows_of_pieces(ns):
        W, H = ns.sym.W, ns.sym.H

        @ns.kernel(work_shape=(W, H), group_shape=(2, 64), subgroup_size=32, **ns.target)
        def k(gr: ns.CurrentGroup, a: ns.Buffer[W, H, ns.DT], b: ns.Buffer[W, H, ns.DT],
              out: ns.Buffer[W, H, ns.DT]):
            @gr.subgroups
            def inner(sg):
                n, sid = sg.size(), sg.subgroup_id()
                i = gr.work_offset[0] + sid[0]
                j = gr.work_offset[1] + sid[1] * n
                x = gr.load(a[i:, j:], shape=(1, n))
                y = gr.load(b[i:, j:], shape=(1, n))
                gr.store(out[i:, j:], np.maximum(x * y - 0.5, y))

            inner()

        return k

    def rows_of_pieces_oracle(ins, out):
        a, b = ins

        def body(offset, sgid, n):
            i, j = offset[0] + sgid[0], offset[1] + sgid[1] * n
            if i < out.shape[0]:
                x, y = a[i, j:j + n], b[i, j:j + n]
                out[i, j:j + n] = np.maximum(x * y - 0.5, y)

        run_subgroups(body, out.shape, (2, 64), 32)

    def partial_sums(ns):
        G = ns.sym.G

        @ns.kernel(work_shape=G, group_shape=64, subgroup_size=16, **ns.target)
        def k(gr: ns.CurrentGroup, a: ns.Buffer[G, ns.DT], result: ns.Buffer[1, ns.DT]):
            # The whole-array sum of python/hckernel/tests/test_examples.py:31-49, one
            # partial sum per sub-group.
            @gr.subgroups
            def inner(sg):
                n = sg.size()
                x = gr.work_offset[0] + sg.subgroup_id()[0] * n
                ns.atomic_ref(result)[0] += gr.load(a[x:], shape=n).sum()

            inner()

        return k

    def partial_sums_oracle(ins, out):
        (a,) = ins

        def body(offset, sgid, n):
            x = offset[0] + sgid[0] * n
            # The sum of a wholly masked tile is masked, and adding it to the element
            # makes that NaN in the reference (NumPy converts the masked value with
            # a warning): the pinned case has no such piece.
            out[0] += a[x:x + n].sum() if x < a.shape[0] else np.nan

        run_subgroups(body, a.shape, 64, 16)

    f32, f64 = np.float32, np.float64
    return [
        dict(name="sg_partial_sums_f64", make=partial_sums, oracle=partial_sums_oracle,
             inputs=[rng.standard_normal(1010)], out=((1,), f64)),
        dict(name="sg_scale_shift_f32", make=scale_shift, oracle=scale_shift_oracle,
             inputs=[rng.standard_normal(1000).astype(f32)], out=((1000,), f32)),
        dict(name="sg_scale_shift_f64", make=scale_shift, oracle=scale_shift_oracle,
             inputs=[rng.standard_normal(130)], out=((130,), f64)),
        dict(name="sg_rows_of_pieces_f64", make=rows_of_pieces, oracle=rows_of_pieces_oracle,
             inputs=[rng.standard_normal((9, 200)), rng.standard_normal((9, 200))],
             out=((9, 200), f64)),
        dict(name="sg_rows_of_pieces_f32", make=rows_of_pieces, oracle=rows_of_pieces_oracle,
             inputs=[rng.standard_normal((4, 64)).astype(f32),
                     rng.standard_normal((4, 64)).astype(f32)], out=((4, 64), f32)),
    ]
