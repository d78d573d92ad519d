"""Helpers for the GPU parity tests: device buffers via torch, calls via ctypes."""

import numpy as np
import torch

from oracle import workloads as oracle


def dev(array: np.ndarray) -> torch.Tensor:
    """Upload a NumPy array; bf16 travels as its uint16 bit pattern."""
    t = torch.from_numpy(np.ascontiguousarray(array)).cuda()
    torch.cuda.synchronize()
    return t


def dev_bf16(values_f32: np.ndarray) -> torch.Tensor:
    """float32 array holding bf16-exact values -> bf16 device tensor."""
    bits = oracle.bf16_bits(values_f32).view(np.int16)
    t = torch.from_numpy(bits).cuda().view(torch.bfloat16)
    torch.cuda.synchronize()
    return t


def host_bf16(t: torch.Tensor) -> np.ndarray:
    """bf16 device tensor -> float32 NumPy array."""
    return t.float().cpu().numpy()


def empty_like_dev(shape, dtype) -> torch.Tensor:
    # Filled with a canary so that elements a kernel fails to write are visible.
    t = torch.empty(shape, dtype=dtype, device="cuda")
    if dtype.is_floating_point:
        t.fill_(float("nan"))
    else:
        t.fill_(-77)
    torch.cuda.synchronize()
    return t


def finish(hc):
    hc.synchronize()
    assert hc.kernel_status() == 0, "a bounded wait inside a kernel gave up"
