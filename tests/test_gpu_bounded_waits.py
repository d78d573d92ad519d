"""The bounded-wait mechanism of the TMA/tcgen05 kernels, exercised on the GPU
without any fault: a self-test kernel waits on a barrier that nothing sets,
with a short limit; the wait must run out, publish a status code the host can
read, make the other waiting thread of the CTA leave too, and return through
the normal teardown - after which the context is still usable.
"""

import ctypes as C

import numpy as np
import pytest
import torch

from oracle import workloads as oracle
from tests.gpu_util import dev, empty_like_dev, finish

pytestmark = pytest.mark.gpu


def _selftest(hc, limit_ns):
    status, elapsed, observed = C.c_int(-1), C.c_ulonglong(0), (C.c_int * 2)(-1, -1)
    rc = hc.lib.hcSelfTestWaitTimeout(hc.handle, limit_ns, C.byref(status), C.byref(elapsed),
                                      observed)
    assert rc == 0, hc.lib.hcLastError(hc.handle)
    return status.value, elapsed.value, list(observed)


def test_wait_that_cannot_succeed_gives_up_and_reports(hc):
    assert hc.kernel_status() == 0
    status, elapsed_ns, observed = _selftest(hc, 2_000_000)  # 2 ms
    assert status == 1            # kStatusProducerWait, written by the thread that ran out
    assert observed == [0, 0]     # neither wait "succeeded"; the second left on the abort flag
    assert 2_000_000 <= elapsed_ns < 200_000_000  # gave up after the limit, and promptly
    assert hc.kernel_status() == 0  # reading the status cleared it

    # The context survived: a real kernel still runs and is right.
    (x,) = oracle.make_inputs("softmax", shape=(64, 512))
    d_x, d_y = dev(x), empty_like_dev(x.shape, torch.float32)
    hc.softmax_rows(d_x.data_ptr(), d_y.data_ptr(), 64, 512, 512, 512)
    finish(hc)
    expect = np.zeros_like(x)
    oracle.softmax_rows(x, expect, 8)
    assert np.all(np.abs(d_y.cpu().numpy() - expect) <= 1e-6 + 1e-5 * np.abs(expect))


def test_limit_is_honoured_and_checked(hc):
    _, short, _ = _selftest(hc, 500_000)
    _, longer, _ = _selftest(hc, 20_000_000)
    assert short < longer and longer >= 20_000_000
    status = C.c_int(0)
    elapsed = C.c_ulonglong(0)
    observed = (C.c_int * 2)()
    assert hc.lib.hcSelfTestWaitTimeout(hc.handle, 0, C.byref(status), C.byref(elapsed),
                                        observed) == 1
    assert b"limit must be" in hc.lib.hcLastError(hc.handle)
