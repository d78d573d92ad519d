"""Work-item bodies on CPU: the oracle against the outputs of the reference
simulator (bit for bit), and the front door - the recorded function must become
the pairwise-distance launch or a program for csrc/kernels/work_items.cu that,
run here one work-item at a time with the phases of a work-group in order,
gives the reference's output.  No kernel is launched."""

import types

import numpy as np
import pytest

from hc_b200.hckernel import elementwise as ew
from hc_b200.hckernel import workitems as wi
from hc_b200.hckernel.kernel import *  # noqa: F401,F403
from hc_b200.hckernel.kernel import UnsupportedKernel
from oracle import workitems as oracle_items

CASES = oracle_items.work_item_cases()
NS = types.SimpleNamespace(kernel=kernel, sym=sym, CurrentGroup=CurrentGroup, Buffer=Buffer,
                           DT=typename.DT, target=dict(backend="nvvm", device="cuda:0"))


class F:
    def __init__(self, shape, dtype):
        self.shape, self.dtype = tuple(shape), np.dtype(dtype).name


def run_item_program(roles, inputs, out):
    """csrc/kernels/work_items.cu in Python: per work-group, phase by phase,
    one work-item at a time."""
    dtype = out.dtype.type
    rows, cols = (1, out.shape[0]) if out.ndim == 1 else out.shape
    out2 = out.reshape(rows, cols)
    ins = [a.reshape(rows, cols) for a in inputs]
    gr, gc = roles["group"]
    phases, current = [[]], 0
    for ins_word in roles["code"]:
        if ins_word & 0xFF == wi.BARRIER:
            phases.append([])
        else:
            phases[-1].append(ins_word)
    for g0 in range(0, rows, gr):
        for g1 in range(0, cols, gc):
            tile = np.full((gr, gc), roles["tile_fill"], dtype)
            for ph, code in enumerate(phases):
                lo_r, hi_r, lo_c, hi_c = roles["guards"][min(ph, len(roles["guards"]) - 1)]
                for lr in range(gr):
                    for lc in range(gc):
                        r, c = g0 + lr, g1 + lc
                        if not (max(lo_r, 0) <= r < min(hi_r, rows)
                                and max(lo_c, 0) <= c < min(hi_c, cols)):
                            continue
                        acc, temps = None, [None] * 3
                        for word in code:
                            op, src = word & 0xFF, (word >> 8) & 0xFF
                            if op == wi.STORE_TILE:
                                tile[lr, lc] = acc
                                continue
                            if op == wi.STORE_OUT:
                                out2[r, c] = acc
                                continue
                            if op <= ew.MIN or ew.FLOORDIV <= op <= ew.XOR:
                                if src < 4:
                                    dr, dc = roles["offsets"][src]
                                    v = ins[src][r + dr, c + dc]
                                elif src < 8:
                                    v = temps[src - 4]
                                elif src < 16:
                                    v = dtype(roles["consts"][src - 8])
                                elif src < 20:
                                    v = dtype((r, c, lr, lc)[src - 16])
                                else:
                                    sr, orow, mr, sc, ocol, mc = roles["tiles"][src - 24]
                                    tr, tc = sr * lr + orow, sc * lc + ocol
                                    tr, tc = (tr % mr if mr else tr), (tc % mc if mc else tc)
                                    assert 0 <= tr < gr and 0 <= tc < gc
                                    v = tile[tr, tc]
                                acc = {ew.LOAD: lambda: v, ew.ADD: lambda: acc + v,
                                       ew.SUB: lambda: acc - v, ew.RSUB: lambda: v - acc,
                                       ew.MUL: lambda: acc * v, ew.DIV: lambda: acc / v,
                                       ew.RDIV: lambda: v / acc,
                                       ew.MAX: lambda: np.maximum(acc, v),
                                       ew.MIN: lambda: np.minimum(acc, v)}[op]()
                            elif op in (ew.SAVE0, ew.SAVE0 + 1, ew.SAVE0 + 2):
                                temps[op - ew.SAVE0] = acc
                            else:
                                acc = {ew.NEG: lambda: -acc, ew.ABS: lambda: abs(acc),
                                       ew.EXP: lambda: np.exp(acc), ew.SQRT: lambda: np.sqrt(acc),
                                       ew.LOG: lambda: np.log(acc)}[op]()
                            acc = dtype(acc)


@pytest.mark.parametrize("case", CASES, ids=lambda c: c["name"])
def test_oracle_matches_the_reference_simulator(golden, case):
    shape, dtype = case["out"]
    out = np.full(shape, -77, dtype)
    case["oracle"](case["inputs"], out)
    assert np.array_equal(out, golden[case["name"]])


@pytest.mark.parametrize("case", CASES, ids=lambda c: c["name"])
def test_recorded_work_item_function_becomes_an_equivalent_launch(golden, case):
    shape, dtype = case["out"]
    k = case["make"](NS)
    plan = k.plan_for(tuple(F(a.shape, a.dtype) for a in case["inputs"]) + (F(shape, dtype),))
    if "pairwise" in case["name"]:
        assert plan.family == "pairwise_distance"
        assert (plan.roles["a"], plan.roles["b"], plan.roles["out"]) == (0, 1, 2)
        return
    assert plan.family == "work_items"
    out = np.full(shape, -77, dtype)
    run_item_program(plan.roles, [case["inputs"][i] for i in plan.roles["inputs"]], out)
    want = golden[case["name"]]
    if dtype == np.float32:
        # The reference carries Python-float factors on in float64 (`a * 2.0`).
        assert np.array_equal(out == -77, want == -77)
        np.testing.assert_allclose(out, want, rtol=3e-7)
    else:
        assert np.array_equal(out, want)


def test_what_a_work_item_function_may_not_do():
    G, DT = sym.G, typename.DT
    target = dict(backend="nvvm", device="cuda:0")

    def build(body):
        @kernel(work_shape=G, group_shape=8, **target)
        def k(group: CurrentGroup, a: Buffer[G, DT], out: Buffer[G, DT]):
            tmp = group.zeros(shape=group.shape[0], dtype=a.dtype)

            @group.workitems
            def inner(w):
                body(group, tmp, w.local_id()[0], w.global_id()[0], a, out)

            inner()

        return k

    arrays = (F((20,), "float32"), F((20,), "float32"))

    def read_before_barrier(group, tmp, lid, gid, a, out):
        tmp[lid] = a[gid]
        out[gid] = tmp.data[7 - lid]

    with pytest.raises(UnsupportedKernel, match="after group.barrier"):
        build(read_before_barrier).plan_for(arrays)

    def two_barriers(group, tmp, lid, gid, a, out):
        tmp[lid] = a[gid]
        group.barrier()
        group.barrier()
        out[gid] = tmp.data[lid]

    with pytest.raises(UnsupportedKernel, match="more than one group.barrier"):
        build(two_barriers).plan_for(arrays)

    def foreign_write(group, tmp, lid, gid, a, out):
        out[gid + 1] = a[gid]

    with pytest.raises(UnsupportedKernel, match="its own element only"):
        build(foreign_write).plan_for(arrays)

    def tile_elsewhere(group, tmp, lid, gid, a, out):
        tmp[7 - lid] = a[gid]
        group.barrier()
        out[gid] = tmp.data[lid]

    with pytest.raises(UnsupportedKernel, match="own local id"):
        build(tile_elsewhere).plan_for(arrays)

    def data_dependent(group, tmp, lid, gid, a, out):
        if a[gid] > 0.0:
            out[gid] = a[gid]

    with pytest.raises(UnsupportedKernel, match="global index"):
        build(data_dependent).plan_for(arrays)

    # What is fine: a rotation inside the group, with a guard on both phases.
    def rotate(group, tmp, lid, gid, a, out):
        if gid < a.shape[0]:
            tmp[lid] = a[gid]
        group.barrier()
        if gid < a.shape[0]:
            out[gid] = tmp.data[(lid + 3) % 8]

    plan = build(rotate).plan_for(arrays)
    assert plan.family == "work_items" and plan.roles["tiles"] == [(0, 0, 0, 1, 3, 8)]
    assert plan.roles["group"] == (1, 8) and plan.roles["guards"] == [(0, 1, 0, 20), (0, 1, 0, 20)]


@pytest.mark.parametrize("case", [c for c in CASES if "pairwise" not in c["name"]],
                         ids=lambda c: c["name"])
def test_work_item_programs_compile_to_device_images(case):
    """hcWorkItems' program as straight-line code: NVRTC makes an sm_100a image of
    the recorded program without a GPU, one element type per image."""
    from hc_b200 import capi

    shape, dtype = case["out"]
    k = case["make"](NS)
    plan = k.plan_for(tuple(F(a.shape, a.dtype) for a in case["inputs"]) + (F(shape, dtype),))
    code = [int(w) for w in plan.roles["code"]]
    hc_dtype = capi.HC_F32 if dtype == np.float32 else capi.HC_F64
    image, tag = capi.specialise_compile_items(code, dtype=hc_dtype)
    assert image[:4] == b"\x7fELF"
    name = "f32" if dtype == np.float32 else "f64"
    other = "f64" if dtype == np.float32 else "f32"
    assert f"hc_work_items_fused_{tag}_{name}".encode() in image
    assert f"hc_work_items_fused_{tag}_{other}".encode() not in image
    assert capi.specialise_compile_items(code, dtype=hc_dtype)[1] == tag
    with pytest.raises(RuntimeError, match="valid size"):
        capi.specialise_compile_items([0] * 49, dtype=hc_dtype)
