"""Shared pytest configuration.

``-m "not gpu"`` runs everything that needs no GPU (oracle vs golden vectors,
host logic, C-ABI export checks, two-rank gloo runs); ``-m gpu`` runs the
parity tests proper, which call the CUDA kernels through the C-ABI.
"""

import sys
from pathlib import Path

import pytest

REPO = Path(__file__).resolve().parent.parent
if str(REPO) not in sys.path:
    sys.path.insert(0, str(REPO))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200)")


@pytest.fixture(scope="session")
def golden():
    import numpy as np

    with np.load(REPO / "tests" / "golden" / "reference_outputs.npz") as z:
        return {k: z[k] for k in z.files}


@pytest.fixture(scope="session")
def hc():
    """One C-ABI context on cuda:0 for the whole session.

    Fails (does not skip) when the native libraries are missing or the device
    cannot be opened: a GPU run must exercise the CUDA path.
    """
    from hc_b200 import capi

    ctx = capi.Context("cuda:0")
    yield ctx
    ctx.close()
