"""The allocation-free dequant GEMM entry point (``hcGemmW8A16Static``).

Some callers of this library are not allowed to allocate device memory on the
launch path - a serving loop whose memory was handed out once at start-up, or
a host application that lends the library a stream but owns every allocation.
``hcGemmW8A16`` asks such a caller for a workspace it cannot provide;
``hcGemmW8A16Static`` uses a fixed scratch array built into the library
instead.  The test calls it through the C-ABI twice in a row with different
inputs (the second call reuses the scratch the first one left behind) and
checks each result against the workspace-taking entry point on the same
inputs, with the bf16 tolerance the other GEMM tests use.  It also checks that
a problem too large for the built-in scratch is refused with a clear message.

This file is collected last on purpose: if it fails under ``-x`` every other
test has already run.
"""

import numpy as np
import pytest
import torch

from hc_b200 import capi
from oracle import workloads as oracle
from tests.gpu_util import dev, dev_bf16, empty_like_dev, finish, host_bf16

pytestmark = pytest.mark.gpu


def _both_ways(hc, shape, seed_shift):
    m, n, k = shape
    a, w, s = oracle.make_inputs("gemm_w8a16", shape=shape)
    w = np.roll(w, seed_shift, axis=0)  # different weights on the second call
    d_a, d_w, d_s = dev_bf16(a), dev(w), dev(s)

    d_static = empty_like_dev((m, n), torch.bfloat16)
    hc.gemm_w8a16_static(d_a.data_ptr(), d_w.data_ptr(), d_s.data_ptr(), d_static.data_ptr(),
                         m, n, k, k, n, n)
    finish(hc)

    ws_bytes = hc.gemm_w8a16_workspace_bytes(n, k)
    ws = torch.empty(ws_bytes, dtype=torch.uint8, device="cuda")
    d_ref = empty_like_dev((m, n), torch.bfloat16)
    torch.cuda.synchronize()
    hc.gemm_w8a16(d_a.data_ptr(), d_w.data_ptr(), d_s.data_ptr(), d_ref.data_ptr(),
                  ws.data_ptr(), ws_bytes, m, n, k, k, n, n)
    finish(hc)

    got, ref = host_bf16(d_static), host_bf16(d_ref)
    assert not np.isnan(got).any()
    mag = np.abs(a) @ (np.abs(w.astype(np.float32)) * s)
    assert np.all(np.abs(got - ref) <= 1e-2 * np.abs(ref) + 1e-4 * mag)
    # And against the CPU oracle, so that both being wrong alike cannot pass.
    expect = np.zeros((m, n), np.float32)
    oracle.gemm_w8a16(a, w, s, expect, (256, 256))
    assert np.all(np.abs(got - expect) <= 1e-2 * np.abs(expect) + 1e-4 * mag)


def test_static_scratch_matches_workspace_entry_point_twice():
    hc = capi.Context("cuda:0")
    try:
        _both_ways(hc, (256, 512, 1024), 0)
        _both_ways(hc, (192, 272, 520), 7)  # smaller, ragged N: reuses the same scratch
        _both_ways(hc, (160, 264, 520), 3)  # N not a multiple of 16: padded scratch pitch
    finally:
        hc.close()


def test_static_scratch_takes_the_largest_admitted_weights():
    """4096 x 4096 weights need exactly the 32 MiB the scratch holds."""
    hc = capi.Context("cuda:0")
    try:
        assert hc.gemm_w8a16_workspace_bytes(4096, 4096) == hc.lib.hcGemmW8A16StaticMaxBytes()
        _both_ways(hc, (64, 4096, 4096), 1)
    finally:
        hc.close()


def test_static_scratch_calls_after_the_first_allocate_nothing():
    """What the entry point is for: once the first call on a device has done its
    set-up, a call changes neither the free device memory nor torch's pool."""
    hc = capi.Context("cuda:0")
    try:
        m, n, k = 128, 512, 512
        a, w, s = oracle.make_inputs("gemm_w8a16", shape=(m, n, k))
        d_a, d_w, d_s = dev_bf16(a), dev(w), dev(s)
        out = empty_like_dev((m, n), torch.bfloat16)

        def call():
            hc.gemm_w8a16_static(d_a.data_ptr(), d_w.data_ptr(), d_s.data_ptr(), out.data_ptr(),
                                 m, n, k, k, n, n)
            finish(hc)

        call()  # set-up: symbol address, kernel images
        torch.cuda.synchronize()
        free_before, _ = torch.cuda.mem_get_info()
        reserved_before = torch.cuda.memory_reserved()
        for _ in range(3):
            call()
        torch.cuda.synchronize()
        assert torch.cuda.mem_get_info()[0] == free_before
        assert torch.cuda.memory_reserved() == reserved_before
    finally:
        hc.close()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_static_scratch_refuses_an_output_on_another_gpu():
    hc = capi.Context("cuda:0")
    try:
        here = torch.empty(256 * 512, dtype=torch.bfloat16, device="cuda:0")
        there = torch.empty(128 * 256, dtype=torch.bfloat16, device="cuda:1")
        with pytest.raises(capi.HcError, match="lives on cuda:1 but the context drives cuda:0"):
            hc.gemm_w8a16_static(here.data_ptr(), here.data_ptr(), here.data_ptr(),
                                 there.data_ptr(), 128, 256, 512, 512, 256, 256)
    finally:
        hc.close()


def test_static_scratch_rejects_oversized_weights():
    hc = capi.Context("cuda:0")
    try:
        limit = hc.lib.hcGemmW8A16StaticMaxBytes()
        assert limit == 32 << 20
        n, k = 8192, 8192  # 128 MiB of bf16 weights
        assert hc.gemm_w8a16_workspace_bytes(n, k) > limit
        out = torch.empty(16, dtype=torch.bfloat16, device="cuda")
        with pytest.raises(capi.HcError, match="built-in scratch holds"):
            hc.gemm_w8a16_static(out.data_ptr(), out.data_ptr(), out.data_ptr(), out.data_ptr(),
                                 128, n, k, k, n, n)
        with pytest.raises(capi.HcError, match="not a device pointer"):
            hc.gemm_w8a16_static(out.data_ptr(), out.data_ptr(), out.data_ptr(), 0,
                                 128, 256, 512, 512, 256, 256)
    finally:
        hc.close()
