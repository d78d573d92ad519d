"""The kernels that do the output all-gather themselves (hcSoftmaxRowsPeers,
hcReduceRowsPeers, hcGemmBf16Peers, hcGemmW8A16Peers), through the C-ABI.

On one GPU the "ranks" are separate buffers of the same device: the kernel must
write every row of its shard into every destination, bit for bit what the plain
entry point writes, and touch nothing else.  With two GPUs the destinations are
real peer memory: two processes, symmetric memory, every rank ends with the
whole result (``tests/test_gpu_launcher_nccl.py`` launches that part)."""

import numpy as np
import pytest
import torch

from hc_b200 import capi
from oracle import workloads as oracle
from tests.gpu_util import dev, dev_bf16, empty_like_dev, finish

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("rows,cols,count", [(64, 4096, 3), (37, 1000, 8), (5, 128, 1)])
def test_softmax_rows_peers_writes_every_destination(hc, rows, cols, count):
    total = 100  # the destinations are full outputs of 100 rows; the shard starts at row 20
    (x,) = oracle.make_inputs("softmax", shape=(rows, cols))
    d_x = dev(x)
    ref = empty_like_dev((rows, cols), torch.float32)
    hc.softmax_rows(d_x.data_ptr(), ref.data_ptr(), rows, cols, cols, cols)
    outs = [empty_like_dev((total, cols), torch.float32) for _ in range(count)]
    hc.softmax_rows_peers(d_x.data_ptr(), [o[20].data_ptr() for o in outs], rows, cols, cols, cols)
    finish(hc)
    for o in outs:
        assert torch.equal(o[20:20 + rows], ref)
        assert torch.isnan(o[:20]).all() and torch.isnan(o[20 + rows:]).all()
    with pytest.raises(capi.HcError, match="multiple of 4"):
        hc.softmax_rows_peers(d_x.data_ptr(), [outs[0].data_ptr()], rows, cols - 1, cols, cols)
    with pytest.raises(capi.HcError, match="destinations expected"):
        hc.softmax_rows_peers(d_x.data_ptr(), [], rows, cols, cols, cols)


def test_reduce_rows_peers_writes_sums_and_maxima(hc):
    rows, cols, total, count = 300, 2048, 1000, 4
    (x,) = oracle.make_inputs("reduce", shape=(rows, cols))
    d_x = dev(x)
    outs = [empty_like_dev((2, total), torch.float32) for _ in range(count)]
    hc.reduce_rows_peers(d_x.data_ptr(), [o[0, 400:].data_ptr() for o in outs], total, rows, cols,
                         cols)
    finish(hc)
    exact = x.astype(np.float64).sum(axis=1)
    for o in outs:
        got = o.cpu().numpy()
        assert np.array_equal(got[1, 400:700], x.max(axis=1))
        assert np.all(np.abs(got[0, 400:700] - exact)
                      <= 1e-5 * np.abs(x).astype(np.float64).sum(axis=1))
        assert np.isnan(got[:, :400]).all() and np.isnan(got[:, 700:]).all()


@pytest.mark.parametrize("m", [512, 100])  # the CTA-pair kernel and the single-CTA kernel
def test_gemm_bf16_peers_writes_row_blocks(hc, m):
    n, k, total, count = 512, 256, 1024, 3
    a, b = oracle.make_inputs("gemm_bf16", shape=(m, n, k))
    d_a, d_b = dev_bf16(a), dev_bf16(b)
    ref = empty_like_dev((m, n), torch.bfloat16)
    hc.gemm_bf16(d_a.data_ptr(), d_b.data_ptr(), ref.data_ptr(), m, n, k, k, n, n)
    outs = [empty_like_dev((total, n), torch.bfloat16) for _ in range(count)]
    hc.gemm_bf16_peers(d_a.data_ptr(), d_b.data_ptr(), [o[256].data_ptr() for o in outs], m, n, k,
                       k, n, n)
    finish(hc)
    for o in outs:
        assert torch.equal(o[256:256 + m].view(torch.int16), ref.view(torch.int16))
        assert torch.isnan(o[:256].float()).all() and torch.isnan(o[256 + m:].float()).all()


def test_gemm_w8a16_peers_writes_column_blocks(hc):
    m, n, k, total_n, count = 384, 256, 512, 1024, 2
    a, w, s = oracle.make_inputs("gemm_w8a16", shape=(m, n, k))
    d_a, d_w, d_s = dev_bf16(a), dev(w), dev(s)
    ws_bytes = hc.gemm_w8a16_workspace_bytes(n, k)
    ws = torch.empty(ws_bytes, dtype=torch.uint8, device="cuda")
    ref = empty_like_dev((m, n), torch.bfloat16)
    hc.gemm_w8a16(d_a.data_ptr(), d_w.data_ptr(), d_s.data_ptr(), ref.data_ptr(), ws.data_ptr(),
                  ws_bytes, m, n, k, k, n, n)
    outs = [empty_like_dev((m, total_n), torch.bfloat16) for _ in range(count)]
    hc.gemm_w8a16_peers(d_a.data_ptr(), d_w.data_ptr(), d_s.data_ptr(),
                        [o[:, 512:].data_ptr() for o in outs], ws.data_ptr(), ws_bytes, m, n, k,
                        k, n, total_n)
    finish(hc)
    for o in outs:
        assert torch.equal(o[:, 512:768].contiguous().view(torch.int16), ref.view(torch.int16))
        assert torch.isnan(o[:, :512].float()).all() and torch.isnan(o[:, 768:].float()).all()
