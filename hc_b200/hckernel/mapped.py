"""Kernels that gather their operand tiles through index mappings, multiply
them and scatter the result - the reference's implicit-GEMM convolution
(python/hckernel/tests/test_examples.py:203-252) and anything of that shape::

    x_t = gr.load(x[...origin...], shape=(TM, K), mapping=x_map)
    f_t = gr.load(f[...origin...], shape=(K, TN), mapping=f_map)
    acc = gr.zeros((TM, TN), dtype)
    for k0 in range(0, K, KB):
        acc += np.dot(gr.vload(x_t[:, k0:], (TM, KB)), gr.vload(f_t[k0:, :], (KB, TN)))
    gr.store(out[...origin...], acc, mapping=out_map)

The mappings are Python functions and the tile origins may be any integer
expression in the group id (``w % W_OUT``, ``w // W_OUT`` ...), so nothing here
pattern-matches them.  They are *evaluated*: once per launch plan the mapping
functions are called on whole index grids and the origin expressions on all
group ids, giving the index tables the kernel reads
(csrc/kernels/mapped_gemm.cu).  Every work-group runs exactly as written - one
CTA each - so, as in the reference, what no group writes stays untouched.

What is checked on the host because a parallel launch could not honour it:
two tile elements, or two work-groups, that write the same output element (the
reference runs groups one after another and the last write wins); negative
tile origins (NumPy slicing would wrap them around).
"""

import numpy as np

from .kernel_api import Tile, UnsupportedKernel

_INT32_MAX = 2**31 - 1


class MappedOperand:
    """One array of the product: which call argument, where its tiles start
    (one index expression per dimension) and the mapping function."""

    def __init__(self, view, tile_shape, func):
        self.arg = view.buffer.index
        self.name = view.buffer.name
        self.rank = view.buffer.ndim
        self.shape = view.buffer.shape
        self.origin = tuple(view.origin)
        self.tile_shape = tuple(tile_shape)
        self.func = func

    def key(self):
        return (self.arg, tuple(o.key() for o in self.origin), self.tile_shape)


def _identity(*index):
    return index


def _shared_run(origins):
    """Largest n in (8, 4, 2) such that work-groups g with equal ``g // n`` all
    have the same tile origin, else 1.  Groups of such a run read one and the
    same tile, so the kernel lets one CTA compute several of them against it."""
    groups = origins.shape[0]
    for n in (8, 4, 2):
        if groups < n:
            continue
        whole = groups // n * n
        runs = origins[:whole].reshape(-1, n, origins.shape[1])
        tail = origins[whole:]
        if (runs == runs[:, :1]).all() and (tail == tail[:1]).all():
            return n
    return 1


def _neighbour_distance(offsets, axis, sector):
    """Mean distance in memory, capped at one 32-byte sector, between tile
    elements adjacent along ``axis`` - how well a warp that walks the tile along
    that axis coalesces."""
    if offsets.shape[axis] < 2:
        return float(sector)
    return float(np.minimum(np.abs(np.diff(offsets, axis=axis)), sector).mean())


def _source(tile, what):
    """(base tile, offsets) of a dot operand: a gathered or loaded tile, whole
    or seen through ``vload(tile[a:, b:], shape)``."""
    offsets = (0, 0)
    if tile.op == "window":
        offsets = tile.attrs["offsets"]
        base = tile.args[0]
    elif tile.op in ("gather", "load"):
        base = tile
    else:
        raise UnsupportedKernel(f"{what}: operand of np.dot is {tile!r}, not a loaded tile")
    if base.op not in ("gather", "load") or base.ndim != 2:
        raise UnsupportedKernel(f"{what}: operand of np.dot is not a rank-2 loaded tile")
    return base, offsets


def match_mapped(scatters, stores, counts):
    """The launch description for a body whose single store goes through a
    mapping; raises UnsupportedKernel when the body is anything else."""
    what = "mapped tile product"
    if len(scatters) != 1 or stores:
        raise UnsupportedKernel(f"{what}: exactly one store, through a mapping, is supported")
    dst, expr, out_map = scatters[0]
    terms = []

    def flatten(node):
        if node.op == "add":
            flatten(node.args[0])
            flatten(node.args[1])
        else:
            terms.append(node)

    flatten(expr)
    dots = [t for t in terms if t.op == "dot"]
    if not dots:
        raise UnsupportedKernel(f"{what}: the stored tile is not a sum of np.dot products")
    for t in terms:
        if t.op != "dot" and not (t.op == "alloc" and t.args[0] == 0.0):
            raise UnsupportedKernel(f"{what}: only a zero accumulator may be added to the products")

    a_base = b_base = None
    spans = []
    for d in dots:
        a, b = d.args
        if not isinstance(a, Tile) or not isinstance(b, Tile):
            raise UnsupportedKernel(f"{what}: np.dot of non-tiles")
        ab, a_off = _source(a, what)
        bb, b_off = _source(b, what)
        if a_base is None:
            a_base, b_base = ab, bb
        if ab is not a_base or bb is not b_base:
            raise UnsupportedKernel(f"{what}: the products read different tiles")
        if a_off[0] != 0 or b_off[1] != 0 or a_off[1] != b_off[0]:
            raise UnsupportedKernel(f"{what}: K offsets of the two operands differ")
        if a.shape[0] != ab.shape[0] or b.shape[1] != bb.shape[1] or a.shape[1] != b.shape[0]:
            raise UnsupportedKernel(f"{what}: operand windows do not span the tiles")
        spans.append((a_off[1], a.shape[1]))
    tm, k = a_base.shape
    k2, tn = b_base.shape
    if k != k2:
        raise UnsupportedKernel(f"{what}: tiles of {a_base.shape} and {b_base.shape} do not multiply")
    reach = 0
    for start, width in sorted(spans):
        if start != reach:
            raise UnsupportedKernel(f"{what}: K blocks overlap or leave gaps")
        reach += width
    if reach < k:
        raise UnsupportedKernel(f"{what}: K blocks stop at {reach} of {k}")
    if tuple(expr.shape) != (tm, tn):
        raise UnsupportedKernel(f"{what}: stored tile is {expr.shape}, product is {(tm, tn)}")

    def operand(base):
        func = base.attrs["mapping"].func if base.op == "gather" else _identity
        return MappedOperand(base.args[0], base.shape, func)

    x, f = operand(a_base), operand(b_base)
    out = MappedOperand(dst, (tm, tn), out_map.func)
    dtypes = {a_base.dtype, b_base.dtype, dst.dtype}
    if len(dtypes) != 1 or dtypes & {"float32", "float64"} != dtypes:
        raise UnsupportedKernel(f"{what}: operands and result must all be float32 or all float64")
    if out.arg in (x.arg, f.arg):
        raise UnsupportedKernel(f"{what}: the result is stored into an operand")
    return MappedSpec(x, f, out, tm, tn, k, counts)


class MappedSpec:
    def __init__(self, x, f, out, tm, tn, k, counts):
        self.x, self.f, self.out = x, f, out
        self.tm, self.tn, self.k = tm, tn, k
        self.counts = tuple(counts)
        self.groups = int(np.prod(self.counts, dtype=np.int64))
        self._host = None   # tables as NumPy arrays, independent of strides
        self._device = {}   # (device, strides) -> tables as device tensors
        self._conv = {}     # array shapes -> stride of the convolution, or None

    # -- evaluation ---------------------------------------------------------------
    @staticmethod
    def _map_table(op):
        """[tile elements, 4] mapped index of every tile element."""
        shape = op.tile_shape
        elems = int(np.prod(shape, dtype=np.int64))
        table = np.zeros((elems, 4), dtype=np.int64)
        if elems == 0:
            return table
        try:
            mapped = op.func(*np.indices(shape, dtype=np.int64))
            mapped = [np.broadcast_to(np.asarray(m, dtype=np.int64), shape) for m in mapped]
        except UnsupportedKernel:
            raise
        except Exception:
            # A mapping that cannot take whole index grids (it branches on its
            # arguments, say): call it per element, as the reference does.
            rows = [op.func(*index) for index in np.ndindex(*shape)]
            mapped = [np.asarray([int(r[d]) for r in rows], dtype=np.int64).reshape(shape)
                      for d in range(len(rows[0]))]
        if len(mapped) != op.rank:
            raise UnsupportedKernel(
                f"mapping of {op.name} returns {len(mapped)} indices for an array of rank {op.rank}")
        for d, m in enumerate(mapped):
            table[:, d] = m.reshape(-1)
        if np.abs(table).max() > _INT32_MAX:
            raise UnsupportedKernel(f"mapping of {op.name} leaves the 32-bit index range")
        return table

    def _origin_table(self, op):
        """[groups, 4] tile origin of every work-group, groups in row-major order."""
        gids = np.indices(self.counts, dtype=np.int64).reshape(len(self.counts), -1)
        table = np.zeros((self.groups, 4), dtype=np.int64)
        for d, expr in enumerate(op.origin):
            table[:, d] = expr.evaluate(gids)
        if self.groups and table.min() < 0:
            raise UnsupportedKernel(f"{op.name}: a tile origin is negative for some work-group")
        if self.groups and table.max() > _INT32_MAX:
            raise UnsupportedKernel(f"{op.name}: a tile origin leaves the 32-bit index range")
        return table

    def _check_single_writer(self, omap, origins):
        """No output element may be written twice (by two tile elements or by
        two work-groups): the reference's sequential last-write-wins order has
        no parallel equivalent."""
        shape = np.array(self.out.shape + (1,) * (4 - self.out.rank), dtype=np.int64)
        weight = np.array([np.prod(shape[d + 1:], dtype=np.int64) for d in range(4)])
        total = int(np.prod(shape, dtype=np.int64))
        elems = omap.shape[0]
        if elems == 0 or self.groups == 0 or total == 0:
            return
        seen = np.zeros(total, dtype=bool)
        step = max(1, (1 << 20) // elems)
        for g0 in range(0, self.groups, step):
            org = origins[g0:g0 + step]                      # [g, 4]
            index = org[:, None, :] + omap[None, :, :]      # [g, e, 4]
            valid = np.all((omap[None, :, :] >= 0) & (index < shape), axis=2)
            flat = (index * weight).sum(axis=2)[valid]
            if flat.size != np.unique(flat).size or seen[flat].any():
                raise UnsupportedKernel(
                    "mapped store: two tile elements or two work-groups write the same output "
                    "element; the reference resolves that by running groups in order, which a "
                    "parallel launch cannot reproduce")
            seen[flat] = True

    def as_convolution(self, x_shape, f_shape, out_shape):
        """The stride, when the work-groups together compute the plain convolution
        without padding

            out[n, q, oh, ow] = sum over (c, kh, kw) of
                x[n, c, oh*s + kh, ow*s + kw] * f[q, c, kh, kw]

        of arrays with these shapes - whatever the tiling, and in whatever order the
        body enumerates the output positions and the filter taps (the reference's
        example walks both transposed, python/hckernel/tests/test_examples.py:220-240,
        which comes to the same sums for square outputs and filters).  None
        otherwise.  Decided on the evaluated tables, not on the body's text."""
        key = (tuple(x_shape), tuple(f_shape), tuple(out_shape))
        if key not in self._conv:
            try:
                self._conv[key] = self._find_convolution(*key)
            except UnsupportedKernel:
                self._conv[key] = None
        return self._conv[key]

    def _find_convolution(self, x_shape, f_shape, out_shape):
        if not (len(x_shape) == len(f_shape) == len(out_shape) == 4) or self.groups == 0:
            return None
        n, c, h, w = x_shape
        nf, cf, hf, wf = f_shape
        if cf != c or out_shape[:2] != (n, nf) or self.k != c * hf * wf:
            return None
        host = self.host_tables()
        (xm, xo), (fm, fo), (om, oo) = host["x"], host["f"], host["out"]
        tm, tn, k = self.tm, self.tn, self.k
        xm, fm, om = xm.reshape(tm, k, 4), fm.reshape(k, tn, 4), om.reshape(tm, tn, 4)
        rows, cols = np.arange(tm)[:, None], np.arange(tn)[None, :]
        # Tile rows are images, tile columns filters; the output tile is one position.
        if not (np.array_equal(om[:, :, 0], np.broadcast_to(rows, (tm, tn)))
                and np.array_equal(om[:, :, 1], np.broadcast_to(cols, (tm, tn)))
                and not om[:, :, 2:].any()):
            return None
        if not (np.array_equal(xm[:, :, 0], np.broadcast_to(rows, (tm, k)))
                and np.array_equal(fm[:, :, 0], np.broadcast_to(cols, (k, tn)))):
            return None
        # (c, kh, kw) of every k: the same for every row of x and column of f, the
        # same in x and f, and every tap of every channel exactly once.
        taps = xm[0, :, 1:]
        if not (np.array_equal(xm[:, :, 1:], np.broadcast_to(taps, (tm, k, 3)))
                and np.array_equal(fm[:, :, 1:], np.broadcast_to(taps[:, None, :], (k, tn, 3)))):
            return None
        if taps.min() < 0 or (taps >= np.array([c, hf, wf])).any():
            return None
        flat = (taps[:, 0] * hf + taps[:, 1]) * wf + taps[:, 2]
        if np.unique(flat).size != k:
            return None
        # Origins: image block, filter block and one output position per group; every
        # (block, block, position) exactly once.
        if fo[:, 1:].any() or xo[:, 1].any():
            return None
        if not (np.array_equal(xo[:, 0], oo[:, 0]) and np.array_equal(fo[:, 0], oo[:, 1])):
            return None
        if (oo[:, 0] % tm).any() or (oo[:, 1] % tn).any():
            return None
        ho, wo = out_shape[2:]
        inside = (oo[:, 2] < ho) & (oo[:, 3] < wo)
        if not inside.all():
            return None
        blocks_n, blocks_q = -(-n // tm), -(-nf // tn)
        code = ((oo[:, 0] // tm) * blocks_q + oo[:, 1] // tn) * (ho * wo) + oo[:, 2] * wo + oo[:, 3]
        if self.groups != blocks_n * blocks_q * ho * wo or np.unique(code).size != self.groups:
            return None
        if code.max() >= self.groups:
            return None
        # x origin = stride x output position.
        moved = oo[:, 2:].max(axis=0)
        stride = None
        for axis in (0, 1):
            if moved[axis] > 0:
                at = np.argmax(oo[:, 2 + axis])
                s_axis, rest = divmod(int(xo[at, 2 + axis]), int(oo[at, 2 + axis]))
                if rest or s_axis < 1 or (stride is not None and stride != s_axis):
                    return None
                stride = s_axis
        if stride is None:
            stride = 1
        if not np.array_equal(xo[:, 2:], oo[:, 2:] * stride):
            return None
        if (h - hf) // stride + 1 != ho or (w - wf) // stride + 1 != wo:
            return None
        return stride

    def host_tables(self):
        if self._host is None:
            if self.groups > _INT32_MAX:
                raise UnsupportedKernel("more than 2^31 work-groups")
            host = {}
            for role, op in (("x", self.x), ("f", self.f), ("out", self.out)):
                host[role] = (self._map_table(op), self._origin_table(op))
            self._check_single_writer(*host["out"])
            self._host = host
        return self._host

    def device_tables(self, tensors):
        """(map, lin, origins, lo, hi, transposed, shared_run) per operand, on the
        device of ``tensors`` (the x, f, out call arguments) and for their strides."""
        import torch

        key = (str(tensors[0].device),) + tuple(tuple(t.stride()) for t in tensors)
        tables = self._device.get(key)
        if tables is None:
            tables = []
            for (role, op), t in zip((("x", self.x), ("f", self.f), ("out", self.out)), tensors):
                mp, org = self.host_tables()[role]
                stride = np.array(tuple(t.stride()) + (0,) * (4 - t.dim()), dtype=np.int64)
                lin = mp @ stride
                if lin.size and np.abs(lin).max() > _INT32_MAX:
                    raise UnsupportedKernel(f"{op.name}: tile offsets leave the 32-bit range")
                lo = mp.min(axis=0) if mp.size else np.zeros(4, np.int64)
                hi = mp.max(axis=0) if mp.size else np.zeros(4, np.int64)
                # The kernel gives consecutive table entries to consecutive
                # threads: store an operand tile transposed when its columns,
                # not its rows, are what lies together in memory.
                rows, cols = op.tile_shape
                transposed = False
                if role != "out" and mp.size:
                    sector = max(1, 32 // t.element_size())
                    grid = lin.reshape(rows, cols)
                    transposed = (_neighbour_distance(grid, 0, sector)
                                  < _neighbour_distance(grid, 1, sector))
                if transposed:
                    mp = mp.reshape(rows, cols, 4).transpose(1, 0, 2).reshape(-1, 4)
                    lin = lin.reshape(rows, cols).T.reshape(-1)

                def dev(a):
                    return torch.from_numpy(np.ascontiguousarray(a.astype(np.int32))).to(t.device)

                tables.append((dev(mp), dev(lin), dev(org), [int(v) for v in lo],
                               [int(v) for v in hi], bool(transposed), _shared_run(org)))
            self._device[key] = tables
        return tables
