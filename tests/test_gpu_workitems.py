"""GPU parity of work-item bodies (local ids, neighbour reads, two phases around
group.barrier() exchanging through a group tile, the work-item form of the
pairwise distance): through the ``@kernel`` front door against the outputs of
the reference simulator, and hcWorkItems called directly through the C-ABI.

Tolerances: the float64 cases are bit-exact; float32 results agree to 3e-7
relative because the reference carries Python-float factors on in float64
(``a * 2.0``); the pairwise distance sums squares in another order than NumPy
(1e-6 / 1e-13 relative).  Elements no work-item writes keep the -77 the output
was filled with."""

import types

import numpy as np
import pytest
import torch

from hc_b200 import capi
from hc_b200.hckernel import elementwise as ew
from hc_b200.hckernel import workitems as wi
from hc_b200.hckernel.kernel import *  # noqa: F401,F403
from hc_b200.hckernel.kernel import get_context
from oracle import workitems as oracle_items
from tests.gpu_util import finish

pytestmark = pytest.mark.gpu

CASES = oracle_items.work_item_cases()
NS = types.SimpleNamespace(kernel=kernel, sym=sym, CurrentGroup=CurrentGroup, Buffer=Buffer,
                           DT=typename.DT, atomic_ref=atomic_ref,
                           target=dict(backend="nvvm", device="cuda:0"))


@pytest.mark.parametrize("case", CASES, ids=lambda c: c["name"])
def test_work_item_bodies_match_the_reference(golden, case):
    shape, dtype = case["out"]
    k = case["make"](NS)
    d_in = [torch.from_numpy(np.ascontiguousarray(a)).cuda() for a in case["inputs"]]
    d_out = torch.full(shape, -77, dtype=d_in[0].dtype, device="cuda")
    k(*d_in, d_out)
    torch.cuda.synchronize()
    got, want = d_out.cpu().numpy(), golden[case["name"]]
    assert np.array_equal(got == -77, want == -77)
    if "pairwise" in case["name"]:
        np.testing.assert_allclose(got, want, rtol=1e-6 if dtype == np.float32 else 1e-13)
    elif dtype == np.float32:
        np.testing.assert_allclose(got, want, rtol=3e-7)
    else:
        assert np.array_equal(got, want)


def test_many_groups_and_a_large_group():
    """A rotation inside work-groups of 1024 work-items over 100 000 elements."""
    G, DT = sym.G, typename.DT

    @kernel(work_shape=G, group_shape=1024, backend="nvvm", device="cuda:0")
    def rotate(group: CurrentGroup, a: Buffer[G, DT], out: Buffer[G, DT]):
        tmp = group.zeros(shape=group.shape[0], dtype=a.dtype)

        @group.workitems
        def inner(w):
            lid, gid = w.local_id()[0], w.global_id()[0]
            if gid < a.shape[0]:
                tmp[lid] = a[gid] + 1.0
            group.barrier()
            if gid < a.shape[0]:
                out[gid] = tmp.data[(lid + 5) % 1024] - gid

        inner()

    n = 100_000
    a = np.random.default_rng(3).standard_normal(n)
    d_out = torch.full((n,), -77.0, dtype=torch.float64, device="cuda")
    rotate(torch.from_numpy(a).cuda(), d_out)
    torch.cuda.synchronize()
    tile = np.zeros(-(-n // 1024) * 1024)
    tile[:n] = a + 1.0
    tile = tile.reshape(-1, 1024)
    want = np.roll(tile, -5, axis=1).reshape(-1)[:n] - np.arange(n)
    assert np.array_equal(d_out.cpu().numpy(), want)


def test_work_items_entry_point_refuses_bad_programs(hc):
    a = torch.zeros(4, 8, device="cuda")
    out = torch.zeros(4, 8, device="cuda")

    def program(code, group=(2, 4), offsets=(0, 0), guard_hi=(4, 8), tile=(1, 0, 0, 1, 0, 0)):
        p = capi.HcItemProgram()
        p.inputs[0], p.inPitch[0] = a.data_ptr(), 8
        p.inRow[0], p.inCol[0] = offsets
        p.out, p.outPitch, p.rows, p.cols = out.data_ptr(), 8, 4, 8
        p.groupRows, p.groupCols, p.nInputs, p.nInstr = group[0], group[1], 1, len(code)
        for i, word in enumerate(code):
            p.code[i] = word
        for ph in range(2):
            p.guardLo[ph][0] = p.guardLo[ph][1] = 0
            p.guardHi[ph][0], p.guardHi[ph][1] = guard_hi
        (p.tileScale[0][0], p.tileOffset[0][0], p.tileMod[0][0], p.tileScale[0][1],
         p.tileOffset[0][1], p.tileMod[0][1]) = tile
        return p

    copy = [ew.LOAD | (0 << 8), wi.STORE_OUT]
    hc.work_items(program(copy))
    finish(hc)
    with pytest.raises(capi.HcError, match="1..1024"):
        hc.work_items(program(copy, group=(64, 32)))
    with pytest.raises(capi.HcError, match="stores nothing"):
        hc.work_items(program([ew.LOAD]))
    with pytest.raises(capi.HcError, match="holds nothing"):
        hc.work_items(program([wi.STORE_OUT]))
    with pytest.raises(capi.HcError, match="more than one barrier"):
        hc.work_items(program([wi.BARRIER, wi.BARRIER] + copy))
    with pytest.raises(capi.HcError, match="leaves the array"):
        hc.work_items(program(copy, offsets=(0, 1)))
    hc.work_items(program(copy, offsets=(0, 1), guard_hi=(4, 7)))  # guarded: fine
    with pytest.raises(capi.HcError, match="leaves the group's tile"):
        hc.work_items(program([ew.LOAD | (24 << 8), wi.STORE_OUT], tile=(1, 0, 0, 1, 1, 0)))
    with pytest.raises(capi.HcError, match="unknown operation"):
        hc.work_items(program([ew.LOAD, 200, wi.STORE_OUT]))
    with pytest.raises(capi.HcError, match="unsupported dtype"):
        hc.work_items(program(copy), capi.HC_I32)
    finish(hc)


@pytest.mark.parametrize("case", [c for c in CASES if "pairwise" not in c["name"]],
                         ids=lambda c: c["name"])
def test_compiled_work_item_programs_equal_the_interpreter(case):
    """hcWorkItems compiles its program with NVRTC at the first launch (option
    `specialise`; 2 = refuse instead of interpreting); the straight-line kernel
    writes bit for bit what the interpreting kernel writes (option `fused` = 1)."""
    ctx = get_context("cuda:0")
    shape, _ = case["out"]
    k = case["make"](NS)
    d_in = [torch.from_numpy(np.ascontiguousarray(a)).cuda() for a in case["inputs"]]
    outs = []
    for interpret in (True, False):
        d_out = torch.full(shape, -77, dtype=d_in[0].dtype, device="cuda")
        ctx.set_option("fused", int(interpret))
        ctx.set_option("specialise", 2)
        before = ctx.specialised_programs() + ctx.specialised_programs(from_disk=True)
        try:
            k(*d_in, d_out)
        finally:
            ctx.set_option("fused", 0)
            ctx.set_option("specialise", 1)
        torch.cuda.synchronize()
        after = ctx.specialised_programs() + ctx.specialised_programs(from_disk=True)
        assert after - before == 0 if interpret else after - before in (0, 1), ctx.specialise_note
        outs.append(d_out.cpu().numpy())
    assert np.array_equal(outs[0], outs[1], equal_nan=True)


@pytest.mark.parametrize("case", oracle_items.subgroup_cases(), ids=lambda c: c["name"])
def test_subgroup_bodies_match_the_reference(golden, case):
    """group.subgroups: every sub-group works on its part of the group's tile; the
    launch runs on the grid of sub-groups (element-wise kernels)."""
    shape, dtype = case["out"]
    k = case["make"](NS)
    d_in = [torch.from_numpy(np.ascontiguousarray(a)).cuda() for a in case["inputs"]]
    d_out = torch.full(shape, -77, dtype=d_in[0].dtype, device="cuda")
    k(*d_in, d_out)
    torch.cuda.synchronize()
    got, want = d_out.cpu().numpy(), golden[case["name"]]
    if "sums" in case["name"]:
        # Partial sums are added in another order than the simulator's: 1e-13 of sum|a|.
        assert abs(got[0] - want[0]) <= 1e-13 * np.abs(case["inputs"][0]).sum()
    elif dtype == np.float32:
        np.testing.assert_allclose(got, want, rtol=3e-7)
    else:
        assert np.array_equal(got, want)
