"""CPU oracle: the workload kernels, restated on top of :mod:`oracle.hcsim`.

TEST INFRASTRUCTURE ONLY - see the header of ``oracle/hcsim.py``.

Each function follows one kernel body of the reference (or, where the
reference has none, the same computation written with the reference's
primitives) group by group, so tiling and edge handling are the reference's.
bf16 is represented the way the reference would have to represent it (NumPy
has no bf16): float32 arrays whose values are bf16-representable, fp32
arithmetic, and a final round-to-nearest-even to bf16.
"""

from __future__ import annotations

import re
from concurrent.futures import ThreadPoolExecutor

import numpy as np

from .hcsim import (
    alloc_tile,
    arithmetic_tile,
    store_result,
    ceil_div,
    iter_groups,
    load_tile,
    load_tile_mapped,
    store_tile,
    store_tile_mapped,
    valid_rows,
)


# ---- bf16 helpers ------------------------------------------------------------
def round_to_bf16(x: np.ndarray) -> np.ndarray:
    """float32 -> nearest-even bf16, returned as float32 holding bf16 values."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    bits = x.view(np.uint32).astype(np.uint64)
    rounded = ((bits + 0x7FFF + ((bits >> 16) & 1)) >> 16) << 16
    out = rounded.astype(np.uint32).view(np.float32)
    nan = np.isnan(x)
    if nan.any():
        out = out.copy()
        out[nan] = np.nan
    return out.reshape(x.shape)


def bf16_bits(x: np.ndarray) -> np.ndarray:
    """uint16 bit patterns of float32 values that are already bf16-exact."""
    return (np.ascontiguousarray(x, dtype=np.float32).view(np.uint32) >> 16).astype(np.uint16)


def bf16_from_bits(bits: np.ndarray) -> np.ndarray:
    return (bits.astype(np.uint32) << 16).view(np.float32)


# ---- copy --------------------------------------------------------------------
def copy2d(src: np.ndarray, dst: np.ndarray, group_shape=(1, 64), unroll: int = 1) -> None:
    """The compiled path's copy kernels, run tile by tile.

    python/hckernel/tests/test_e2e.py:66-70 (unroll 1) and :95-100 (each group
    covers ``group_shape[1] * V`` columns); work shape (W, ceil(H / V)).
    """
    w, h = src.shape
    for _, (x, y) in iter_groups((w, ceil_div(h, unroll)), group_shape):
        tile = load_tile(src[x:, y * unroll :], (group_shape[0], group_shape[1] * unroll))
        store_tile(dst[x:, y * unroll :], tile)


# ---- GEMM --------------------------------------------------------------------
def gemm_kblocked(a, b, out, group_shape=(64, 64), kb: int = 16, mi: int = 1, ni: int = 1) -> None:
    """K-blocked tiled GEMM: python/hckernel/tests/test_examples.py:88-111.

    Work shape (ceil(M/MI), ceil(N/NI)); a group owns an (gm*MI, gn*NI) output
    tile, accumulates ``np.dot`` of (m_block, KB) x (KB, n_block) tiles over
    ceil(K/KB) steps into a zero tile of the output dtype, then stores it.
    """
    m, k = a.shape
    n = b.shape[1]
    gm, gn = group_shape
    m_block, n_block = gm * mi, gn * ni
    steps = ceil_div(k, kb)
    for _, (wm, wn) in iter_groups((ceil_div(m, mi), ceil_div(n, ni)), group_shape):
        m0, n0 = wm * mi, wn * ni
        acc = alloc_tile((m_block, n_block), out.dtype)
        for step in range(steps):
            k0 = step * kb
            a_tile = load_tile(a[m0:, k0:], (m_block, kb))
            b_tile = load_tile(b[k0:, n0:], (kb, n_block))
            # `r += np.dot(...)` (kernel_api.py:142-145): the product is a plain
            # array, so every element of the accumulator is updated.
            acc.data[...] = acc.data + np.dot(a_tile.data, b_tile.data)
        store_tile(out[m0:, n0:], acc)


def gemm_fullk(a, b, out, group_shape=(64, 64), mi: int = 1, ni: int = 1, acc_dtype=None) -> None:
    """Full-K tiled GEMM: python/hckernel/tests/test_examples.py:136-155."""
    m, k = a.shape
    n = b.shape[1]
    gm, gn = group_shape
    m_block, n_block = gm * mi, gn * ni
    acc_dtype = acc_dtype or out.dtype
    for _, (wm, wn) in iter_groups((ceil_div(m, mi), ceil_div(n, ni)), group_shape):
        m0, n0 = wm * mi, wn * ni
        acc = alloc_tile((m_block, n_block), acc_dtype)
        a_tile = load_tile(a[m0:, :], (m_block, k))
        b_tile = load_tile(b[:, n0:], (k, n_block))
        acc.data[...] = acc.data + np.dot(a_tile.data, b_tile.data)
        store_tile(out[m0:, n0:], acc)


def gemm_bf16(a, b, out, group_shape=(256, 256)) -> None:
    """bf16 GEMM, fp32 accumulation, bf16-rounded output.

    The full-K kernel above with float32 arrays holding bf16 values; the
    rounding happens where the reference would cast on store.  ``out`` is
    float32 and receives bf16-representable values.
    """
    tmp = np.zeros(out.shape, dtype=np.float32)
    gemm_fullk(a, b, tmp, group_shape, acc_dtype=np.float32)
    out[...] = round_to_bf16(tmp)


def gemm_w8a16(a, w, scale, out, group_shape=(256, 256)) -> None:
    """int8 weight-only dequant GEMM with the reference's primitives.

    Per group: ``r = np.dot(a_tile, w_tile.astype(float32)) * scale_tile``,
    stored with a cast to bf16.  ``a`` is float32 holding bf16 values, ``w``
    int8 [K, N] (the reference's ``b: Buffer[K, N]`` convention,
    python/hckernel/tests/test_examples.py:91), ``scale`` float32 [N].
    """
    m, k = a.shape
    n = w.shape[1]
    gm, gn = group_shape
    tmp = np.zeros(out.shape, dtype=np.float32)
    for _, (m0, n0) in iter_groups((m, n), group_shape):
        a_tile = load_tile(a[m0:, :], (gm, k))
        w_tile = load_tile(w[:, n0:], (k, gn))
        s_tile = load_tile(scale[n0:], (gn,))
        r = np.dot(a_tile.data, w_tile.data.astype(np.float32)) * s_tile.data
        store_tile(tmp[m0:, n0:], r)
    out[...] = round_to_bf16(tmp)


# ---- softmax -----------------------------------------------------------------
def softmax_rows(a, out, group_rows: int = 8, mi: int = 1) -> None:
    """Row softmax: python/hckernel/tests/test_examples.py:312-321.

    A group loads ``group_rows * MI`` whole rows, subtracts the row maximum,
    exponentiates and divides by the row sum; rows past the end of the array
    are padding and are dropped by the clipped store.
    """
    m, n = a.shape
    m_block = group_rows * mi
    for _, (wm,) in iter_groups((ceil_div(m, mi),), (group_rows,)):
        m0 = wm * mi
        tile = load_tile(a[m0:, :], (m_block, n))
        rows = valid_rows(tile)
        x = tile.data[:rows]
        e = np.exp(x - x.max(axis=1, keepdims=True))
        store_tile(out[m0:, :], e / e.sum(axis=1, keepdims=True))


# ---- reductions ----------------------------------------------------------------
def reduce_sum_all(a, result, group_size: int = 8, n_per_item: int = 2) -> None:
    """Whole-array sum: python/hckernel/tests/test_examples.py:36-40.

    Each group loads ``group_size * N`` elements (zero padded) and adds the
    tile's sum to ``result[0]`` (``atomic_ref`` is the identity on the
    simulator, python/hckernel/kernel_api.py:450-451).
    """
    ws = a.shape[0]
    for _, (off,) in iter_groups((ceil_div(ws, n_per_item),), (group_size,)):
        tile = load_tile(a[off * n_per_item :], (group_size * n_per_item,))
        result[0] += tile.data[tile.valid].sum()


def reduce_rows(x, sum_out=None, max_out=None, group_rows: int = 256) -> None:
    """Last-axis sum and max, written with the reference's primitives:

    ``v = group.load(x[m0:, :], (gm, N)); group.store(s[m0:], v.sum(axis=1));
    group.store(mx[m0:], v.max(axis=1))`` - masked reductions ignore padding
    rows, and the clipped store drops them.
    """
    m, n = x.shape
    for _, (m0,) in iter_groups((m,), (group_rows,)):
        tile = load_tile(x[m0:, :], (group_rows, n))
        rows = valid_rows(tile)
        v = tile.data[:rows]
        if sum_out is not None:
            store_tile(sum_out[m0:], v.sum(axis=1))
        if max_out is not None:
            store_tile(max_out[m0:], v.max(axis=1))


# ---- pairwise distance ---------------------------------------------------------------
def pairwise_distance(a, b, out, group_shape=(8, 8), mi: int = 1, ni: int = 1) -> None:
    """Pairwise Euclidean distance: python/hckernel/tests/test_examples.py:274-301.

    A group loads (m_block, D) rows of ``a`` and (n_block, D) rows of ``b`` (zero
    padded past the ends), forms the broadcast difference and stores its norm
    over the last axis; the clipped store drops the rows that were padding.
    """
    m, d = a.shape
    n = b.shape[0]
    gm, gn = group_shape
    m_block, n_block = gm * mi, gn * ni
    for _, (wm, wn) in iter_groups((ceil_div(m, mi), ceil_div(n, ni)), group_shape):
        m0, n0 = wm * mi, wn * ni
        a_tile = load_tile(a[m0:, :], (m_block, d))
        b_tile = load_tile(b[n0:, :], (n_block, d))
        diff = a_tile.data[:, None, :] - b_tile.data[None, :, :]
        store_tile(out[m0:, n0:], np.linalg.norm(diff, axis=2))


# ---- element-wise bodies ------------------------------------------------------------
def elementwise(fn, inputs, out, group_shape) -> None:
    """A body that loads one tile per input at the group's offset, combines
    them element by element with ``fn`` and stores the result at the same offset
    (the reference's copy kernels with arithmetic in between:
    python/hckernel/tests/test_e2e.py:57-136, tile arithmetic
    python/hckernel/kernel_api.py:136-211).

    The reference's tiles are ``numpy.ma`` arrays (kernel_api.py:106-155), and
    that is kept here because it is visible in the results: ``numpy.ma``
    turns a Python float operand into a float64 array, so ``tile_f32 + 1.0`` is
    computed and carried on in float64 and only rounded to float32 when it is
    stored (plain NumPy would stay in float32), and its division masks the
    elements whose divisor is zero, which the masked store then leaves
    unwritten.  The padding of edge tiles is masked from the start and dropped
    by the store."""
    group_shape = tuple(np.atleast_1d(group_shape).tolist())
    for _, offset in iter_groups(out.shape, group_shape):
        window = tuple(slice(o, None) for o in offset)
        tiles = [arithmetic_tile(load_tile(a[window], group_shape)) for a in inputs]
        with np.errstate(all="ignore"):
            store_result(out[window], fn(*tiles))


def elementwise_cases():
    """``(name, fn, number of inputs, shape, dtype, group shape)`` of the
    element-wise vectors stored under ``tests/golden``.  Every ``fn`` is written
    with NumPy calls and operators only, so the same function object runs on
    the reference simulator's tiles, on NumPy arrays and on recorded tiles."""
    return [
        ("map_relu_axpby_f32", lambda a, b: np.maximum(a * 2.0 - b, 0.0), 2, (111, 813), "float32",
         (4, 16)),
        ("map_mixed_f64",
         lambda a, b: (a + b) / (np.sqrt(np.abs(a)) + 1.5) - np.minimum(a, b) * (-b),
         2, (70, 45), "float64", (8, 8)),
        ("map_gauss_f32", lambda a: np.exp(-(a * a)), 1, (33, 130), "float32", (16, 32)),
        ("map_vector_f32", lambda a: a * a + 1.0, 1, (1000,), "float32", (64,)),
        # (the reference's tiles have no reflected operators: `c * c + 1.0`, not `1.0 + c * c`)
        ("map_three_inputs_f32", lambda a, b, c: (a - b) * (b - c) / (c * c + 1.0), 3, (64, 256),
         "float32", (8, 64)),
    ]


def operator_cases():
    """``(name, fn, input arrays, group shape)`` of the vectors under
    ``tests/golden`` that pin the rest of the reference's tile operator table
    (python/hckernel/kernel_api.py:157-176) and its masked store (:338-340):
    floor division, remainder and division with zero divisors (those elements
    stay unwritten), ``**`` with results that are not finite (likewise),
    comparisons used as 0/1 factors, and integer tiles.  Every case runs on the
    reference simulator; outputs start as -77 so that unwritten elements show.

    Not in the list because the reference simulator itself fails on them
    (``AssertionError`` from its mask helper when numpy.ma returns ``nomask``,
    ``TypeError`` for ``~``): a comparison or ``& | ^ << >>`` stored directly,
    ``tile ** tile`` and integer ``**``."""
    rng = np.random.default_rng(12)

    def floats(shape, dtype):
        a = rng.standard_normal(shape).astype(dtype) * 4
        b = np.round(rng.standard_normal(shape) * 1.5).astype(dtype)  # whole numbers, many zeros
        a[0, :3] = [0.0, -0.0, 5.0]
        b[0, :3] = [0.0, 0.0, -0.0]
        return a, b

    def ints(shape, dtype):
        a = rng.integers(-50, 50, shape).astype(dtype)
        b = rng.integers(-4, 5, shape).astype(dtype)  # one in nine is zero
        return a, b

    af, bf = floats((37, 53), "float32")
    ad, bd = floats((20, 33), "float64")
    ai, bi = ints((41, 29), "int32")
    al, bl = ints((18, 70), "int64")
    return [
        ("ops_floordiv_f32", lambda a, b: a // b, (af, bf), (8, 16)),
        ("ops_mod_f32", lambda a, b: a % b, (af, bf), (8, 16)),
        ("ops_div_zero_f32", lambda a, b: a / b, (af, bf), (8, 16)),
        ("ops_floordiv_mod_f64", lambda a, b: (a // b) * b + a % b, (ad, bd), (4, 8)),
        ("ops_pow_f32", lambda a, b: a ** 2.5 + b, (af, bf), (8, 16)),
        ("ops_compare_f32", lambda a, b: (a < b) * a + (a >= b) * b, (af, bf), (8, 16)),
        ("ops_equal_f64", lambda a, b: (a == b) * 3.0 + (a != b) * a - (a > b) * (a <= 0.5),
         (np.round(ad), bd), (4, 8)),
        ("ops_arith_i32", lambda a, b: a * 3 - b + a // b, (ai, bi), (8, 8)),
        ("ops_mod_abs_i32", lambda a, b: a % b - abs(-a), (ai, bi), (8, 8)),
        ("ops_compare_i32", lambda a, b: (a <= b) * a + (a > b) * b, (ai, bi), (8, 8)),
        ("ops_arith_i64", lambda a, b: a * a - b // 7 + a % 5, (al, bl), (4, 32)),
    ]


def rowwise(fn, inputs, out, group_rows: int = 8) -> None:
    """A body that loads ``group_rows`` whole rows per input, computes ``fn`` of
    them - which may reduce along the rows and use the reduced values again, as
    the reference's softmax does (python/hckernel/tests/test_examples.py:
    312-321) - and stores the rows.  Same tile arithmetic as
    :func:`elementwise`; reductions reach ``numpy.ma`` through the tile wrapper
    (python/hckernel/kernel_api.py:150-151) and ignore the padding rows."""
    cols = out.shape[1]
    for _, (m0,) in iter_groups(out.shape[0], group_rows):
        tiles = [arithmetic_tile(load_tile(a[m0:, :], (group_rows, cols))) for a in inputs]
        with np.errstate(all="ignore"):
            store_result(out[m0:, :], fn(*tiles))


def rowwise_cases():
    """``(name, fn, number of inputs, shape, dtype, rows per group)`` of the row
    bodies stored under ``tests/golden``; every ``fn`` runs unchanged on the
    reference simulator's tiles, on NumPy arrays and on recorded tiles."""
    def centre(t):
        return t - t.mean(axis=1, keepdims=True)

    def l2_normalise(t):
        return t / np.sqrt((t * t).sum(axis=1, keepdims=True))

    def log_softmax(t):
        shifted = t - t.max(axis=1, keepdims=True)
        return shifted - np.log(np.exp(shifted).sum(axis=1, keepdims=True))

    def softmax_temperature(t):
        e = np.exp((t - t.max(axis=1, keepdims=True)) * 0.5)
        return e / e.sum(axis=1, keepdims=True)

    def scaled_difference(a, b):
        return (a - b) / np.maximum(np.abs(a).max(axis=1, keepdims=True), 1.0)

    return [
        ("rows_centre_f32", centre, 1, (37, 300), "float32", 8),
        ("rows_l2_normalise_f64", l2_normalise, 1, (30, 25), "float64", 8),
        ("rows_log_softmax_f32", log_softmax, 1, (48, 1024), "float32", 16),
        ("rows_softmax_temperature_f32", softmax_temperature, 1, (19, 130), "float32", 4),
        ("rows_scaled_difference_f32", scaled_difference, 2, (64, 512), "float32", 32),
    ]


def random_expression(rng, inputs: int, depth: int):
    """A random element-wise function of ``inputs`` arrays as ``(fn, text)``:
    a tree of + - * /, maximum, minimum, abs, negation and sqrt(abs(.)) over the
    inputs and a few constants, at most ``depth`` levels deep.  Divisors are
    kept away from zero (``abs(.) + 0.5``).  Used to test the translation of
    recorded expressions against NumPy on the same arrays."""
    names = "abcd"[:inputs]

    def build(level):
        if level == 0 or rng.random() < 0.2:
            if rng.random() < 0.75:
                return str(rng.choice(list(names)))
            return repr(float(rng.choice([0.5, 1.0, 2.0, -1.5, 3.0])))
        kind = rng.integers(0, 9)
        x = build(level - 1)
        if kind == 6:
            return f"np.abs({x})"
        if kind == 7:
            return f"(-({x}))"
        if kind == 8:
            return f"np.sqrt(np.abs({x}))"
        y = build(level - 1)
        if kind == 3:
            return f"(({x}) / (np.abs({y}) + 0.5))"
        if kind == 4:
            return f"np.maximum({x}, {y})"
        if kind == 5:
            return f"np.minimum({x}, {y})"
        return f"(({x}) {'+-*'[kind]} ({y}))"

    while True:
        text = build(depth)
        if re.search(rf"\b[{names}]\b", text):  # at least one array takes part
            break
    fn = eval(f"lambda {', '.join(names)}: {text}", {"np": np})  # noqa: S307 (own text)
    return fn, text


def random_row_expression(rng, inputs: int):
    """A random row body of ``inputs`` matrices as ``(fn, text)``: one or two
    reductions along the rows (sum, max, mean of a random element-wise
    expression; the second may use the first) and a final element-wise
    expression of the matrices and the reduced values.  Magnitudes stay tame:
    divisors are ``abs(.) + 0.5``, exponentials are of ``-abs(.)``.  Used to test
    the translation of recorded row bodies against NumPy on the same arrays."""
    names = list("ab"[:inputs])

    def build(level, leaves):
        if level == 0 or rng.random() < 0.25:
            if rng.random() < 0.8:
                return str(rng.choice(leaves))
            return repr(float(rng.choice([0.5, 1.0, 2.0, -1.5, 0.25])))
        kind = rng.integers(0, 9)
        x = build(level - 1, leaves)
        if kind == 5:
            return f"np.abs({x})"
        if kind == 6:
            return f"np.exp(-np.abs({x}))"
        if kind == 7:
            return f"np.sqrt(np.abs({x}) + 1.0)"
        y = build(level - 1, leaves)
        if kind == 3:
            return f"(({x}) / (np.abs({y}) + 0.5))"
        if kind == 4:
            return f"np.maximum({x}, {y})"
        if kind == 8:
            return f"np.minimum({x}, {y})"
        return f"(({x}) {'+-*'[kind]} ({y}))"

    def with_array(level, leaves):
        while True:
            text = build(level, leaves)
            if re.search(rf"\b[{''.join(names)}]\b", text):  # a matrix takes part
                return text

    def reduced(text):
        how = str(rng.choice(["sum", "max", "mean"]))
        return f"(({text}).{how}(axis=1, keepdims=True))"

    # Reduced values travel as the placeholders R0, R1 until the end, so that
    # "a matrix takes part" is asked of each expression's own leaves.
    scalars = {"R0": reduced(with_array(int(rng.integers(0, 3)), names))}
    if rng.random() < 0.5:
        scalars["R1"] = reduced(with_array(int(rng.integers(1, 3)), names + ["R0"]))
    text = with_array(int(rng.integers(1, 3)), names + list(scalars))
    if not any(s in text for s in scalars):  # the body must use a reduction
        text = f"(({text}) - {list(scalars)[-1]})"
    for name in ("R1", "R0"):
        if name in scalars:
            text = text.replace(name, scalars[name])
    fn = eval(f"lambda {', '.join(names)}: {text}", {"np": np})  # noqa: S307 (own text)
    return fn, text


def make_elementwise_inputs(count, shape, dtype, seed: int = 7):
    rng = np.random.default_rng(seed)
    return [rng.standard_normal(shape).astype(dtype) for _ in range(count)]


# ---- implicit-GEMM convolution (gathers through index mappings) ---------------------
def conv_mappings(hf: int, wf: int):
    """The three index mappings of the reference's convolution example
    (python/hckernel/tests/test_examples.py:220-226): tile element -> index in
    the sliced image / filter / output array."""
    win = hf * wf

    def x_map(i, j):
        return (i, j // win, (j % win) % wf, (j % win) // wf)

    def f_map(i, j):
        return (j, i // win, i % wf, (i % win) // wf)

    def out_map(i, j):
        return (i, j, 0, 0)

    return x_map, f_map, out_map


def conv_implicit_gemm(x, f, out, stride: int = 1, tn: int = 8, tnf: int = 8, kb: int = 16) -> None:
    """Convolution as an implicit GEMM: python/hckernel/tests/test_examples.py:203-252.

    ``x`` [N, C, H, W], ``f`` [NF, C, HF, WF], ``out`` [N, NF, H_OUT, W_OUT], no
    padding.  Work shape (N, NF, H_OUT*W_OUT) in groups of (TN, TNF, 1): a group
    gathers a (TN, C*HF*WF) tile of image patches and a (C*HF*WF, TNF) tile of
    filters through the index mappings, multiplies them in K blocks of ``kb``
    and scatters the (TN, TNF) result to one output position.

    Kept as the reference has them: ``H_OUT = (H - HF)/stride + 1`` is an exact
    fraction, the work shape is truncated to an integer
    (python/hckernel/kernel_sim.py:121-127), and the linear position ``w`` is
    split as ``i = w % W_OUT`` (used on the H axis) and ``j = w // W_OUT`` (used
    on the W axis), test_examples.py:237-240, 252.
    """
    from fractions import Fraction

    n_img, c, h, w = x.shape
    n_flt, cf, hf, wf = f.shape
    if cf != c:
        raise ValueError("image and filter channel counts differ")
    h_out = Fraction(h - hf, stride) + 1
    w_out = Fraction(w - wf, stride) + 1
    sz = hf * wf * c
    steps = ceil_div(sz, kb)
    x_map, f_map, out_map = conv_mappings(hf, wf)

    def as_index(value):
        if Fraction(value).denominator != 1:
            raise TypeError(f"tile origin {value} is not an integer")
        return int(value)

    work = (n_img, n_flt, int(h_out * w_out))
    for _, (n0, q0, pos) in iter_groups(work, (tn, tnf, 1)):
        i = as_index(pos % w_out)
        j = as_index(pos // w_out)
        x_view = load_tile_mapped(x[n0:, :, i * stride:, j * stride:], (tn, sz), x_map)
        f_view = load_tile_mapped(f[q0:, :, :, :], (sz, tnf), f_map)
        acc = alloc_tile((tn, tnf), out.dtype)
        for step in range(steps):
            k0 = step * kb
            # vload of a slice of a loaded tile: zero-padded to (TN, KB); the
            # elements the gather left invalid already hold zero.
            x_slice = load_tile(x_view.data[:, k0:], (tn, kb))
            f_slice = load_tile(f_view.data[k0:, :], (kb, tnf))
            acc.data[...] = acc.data + np.dot(x_slice.data, f_slice.data)
        store_tile_mapped(out[n0:, q0:, i:, j:], acc, out_map)


def conv_direct(x, f, stride: int = 1) -> np.ndarray:
    """Plain correlation, the textbook form the reference's test compares with
    (python/hckernel/tests/test_examples.py:179-199) for square images and
    filters: out[n, q, oh, ow] = sum x[n, :, oh*s : oh*s+HF, ow*s : ow*s+WF] * f[q]."""
    n_img, c, h, w = x.shape
    n_flt, _, hf, wf = f.shape
    h_out = (h - hf) // stride + 1
    w_out = (w - wf) // stride + 1
    out = np.zeros((n_img, n_flt, h_out, w_out), dtype=np.result_type(x, f))
    for oh in range(h_out):
        for ow in range(w_out):
            patch = x[:, :, oh * stride: oh * stride + hf, ow * stride: ow * stride + wf]
            out[:, :, oh, ow] = np.einsum("nchw,qchw->nq", patch, f)
    return out


def conv_golden_cases():
    """``(name, x shape, f shape, stride, dtype, tiles)`` of the convolution
    vectors stored under ``tests/golden``: the grid of the reference's own test
    (python/hckernel/tests/test_examples.py:168-176, float64) and cases it does
    not reach - ragged tiles, rectangular images and filters, other tile sizes,
    float32.  ``tiles`` is (TN, TNF, KB)."""
    cases = []
    for n in (1, 2, 4):
        for c in (1, 3):
            for nf in (1, 2, 8):
                for stride in (1, 2, 3):
                    cases.append((f"conv_n{n}_c{c}_nf{nf}_s{stride}", (n, c, 4, 4), (nf, c, 2, 2),
                                  stride, "float64", (8, 8, 16)))
    cases.append(("conv_ragged_tiles", (11, 3, 7, 7), (10, 3, 3, 3), 1, "float64", (8, 8, 16)))
    cases.append(("conv_stride2_f32", (3, 2, 9, 9), (5, 2, 3, 3), 2, "float32", (8, 8, 16)))
    cases.append(("conv_wide_image", (2, 2, 5, 8), (3, 2, 2, 2), 1, "float64", (8, 8, 16)))
    cases.append(("conv_tall_image", (2, 2, 8, 5), (3, 2, 2, 2), 1, "float64", (8, 8, 16)))
    cases.append(("conv_wide_filter", (2, 2, 6, 6), (3, 2, 2, 3), 1, "float64", (8, 8, 16)))
    cases.append(("conv_tall_filter", (2, 2, 6, 6), (3, 2, 3, 2), 1, "float64", (8, 8, 16)))
    cases.append(("conv_tiles_4x16_kb8_f32", (9, 3, 6, 6), (20, 3, 3, 3), 1, "float32", (4, 16, 8)))
    return cases


def make_conv_inputs(x_shape, f_shape, dtype="float32", seed: int = 6):
    """Seeded standard-normal image and filter arrays."""
    rng = np.random.default_rng(seed)
    x = rng.standard_normal(x_shape).astype(dtype)
    f = rng.standard_normal(f_shape).astype(dtype)
    return x, f


def conv_out_shape(x_shape, f_shape, stride):
    """Output shape as the reference's test computes it (test_examples.py:182-185):
    ``int((extent - filter) / stride) + 1`` per spatial axis."""
    return (x_shape[0], f_shape[0], int((x_shape[2] - f_shape[2]) / stride) + 1,
            int((x_shape[3] - f_shape[3]) / stride) + 1)


# ---- seeded inputs of the benchmark configurations -----------------------------
def make_inputs(config: str, scale_rows: int | None = None, shape=None):
    """Seeded synthetic inputs of the five benchmark configurations.

    ``config`` is one of ``gemm_f32``, ``softmax``, ``reduce``, ``gemm_bf16``,
    ``gemm_w8a16``; seeds, distributions and draw order are fixed (NumPy PCG64
    ``default_rng(seed)``), so every process regenerates the same arrays.
    ``shape`` overrides the full-size shape for reduced-size parity cases.
    """
    if config == "gemm_f32":
        m, n, k = shape or (256, 256, 256)
        rng = np.random.default_rng(0)
        a = rng.uniform(-1, 1, (m, k)).astype(np.float32)
        b = rng.uniform(-1, 1, (k, n)).astype(np.float32)
        return a, b
    if config == "softmax":
        m, n = shape or (32768, 4096)
        return (np.random.default_rng(1).standard_normal((m, n), dtype=np.float32),)
    if config == "reduce":
        m, n = shape or (65536, 8192)
        rng = np.random.default_rng(2)
        # Drawn in float32 directly: the full-size float64 draw would need 4 GiB.
        return ((rng.random((m, n), dtype=np.float32) * np.float32(20.0) - np.float32(10.0)),)
    if config == "gemm_bf16":
        m, n, k = shape or (8192, 8192, 8192)
        rng = np.random.default_rng(3)
        a = round_to_bf16((rng.standard_normal((m, k), dtype=np.float32) * np.float32(0.02)))
        b = round_to_bf16((rng.standard_normal((k, n), dtype=np.float32) * np.float32(0.02)))
        return a, b
    if config == "gemm_w8a16":
        m, n, k = shape or (4096, 8192, 8192)
        rng = np.random.default_rng(4)
        a = round_to_bf16(rng.standard_normal((m, k), dtype=np.float32))
        w = rng.integers(-127, 128, (k, n), dtype=np.int8)
        s = rng.uniform(0.001, 0.02, n).astype(np.float32)
        return a, w, s
    raise ValueError(f"unknown config {config!r}")


# ---- multi-threaded drivers for the timed CPU baseline ---------------------------
def run_row_groups_parallel(fn, m: int, group_rows: int, threads: int) -> None:
    """Run ``fn(row_begin, row_end)`` over row blocks on a thread pool.

    The simulator visits groups one after another; groups of these workloads
    are independent, so the timed CPU baseline may spread them over the host
    cores (NumPy releases the GIL inside its loops).  ``row_begin`` is always a
    multiple of ``group_rows`` so the tiling is unchanged.
    """
    groups = ceil_div(m, group_rows)
    per = ceil_div(groups, max(1, threads)) * group_rows
    spans = [(r0, min(m, r0 + per)) for r0 in range(0, m, per)]
    if threads <= 1 or len(spans) == 1:
        for r0, r1 in spans:
            fn(r0, r1)
        return
    with ThreadPoolExecutor(max_workers=threads) as pool:
        list(pool.map(lambda s: fn(*s), spans))
