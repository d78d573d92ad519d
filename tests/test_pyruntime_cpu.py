"""libhc-python-runtime.so on CPU: argument conversion into memref descriptors
(reference: python/cpp/py-runtime/src/PyABI.cpp:15-41), search paths, tracing,
and that a failing hcgpuGetKernel aborts the process as the reference does
(python/cpp/py-runtime/src/GpuRuntime.cpp:18-21) - checked in a child process."""

import ctypes as C
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

from hc_b200 import capi

REPO = Path(__file__).resolve().parent.parent


class _Desc2(C.Structure):
    _fields_ = [("allocated", C.c_void_p), ("aligned", C.c_void_p), ("offset", C.c_ssize_t),
                ("sizes", C.c_ssize_t * 2), ("strides", C.c_ssize_t * 2)]


@pytest.fixture(scope="module")
def rt():
    return capi.load_python_runtime()




def test_convert_numpy_and_torch_arrays(rt):
    a = np.arange(12, dtype=np.float32).reshape(3, 4)
    d = _Desc2()
    assert rt.hcgpuConvertPyArray(None, a, 2, C.byref(d)) == 0
    assert d.allocated == a.ctypes.data and d.aligned == a.ctypes.data and d.offset == 0
    assert list(d.sizes) == [3, 4] and list(d.strides) == [4, 1]  # strides in elements

    view = a[:, 1:3]
    assert rt.hcgpuConvertPyArray(None, view, 2, C.byref(d)) == 0
    assert d.allocated == view.ctypes.data and list(d.sizes) == [3, 2] and list(d.strides) == [4, 1]

    t = torch.arange(24, dtype=torch.bfloat16).reshape(4, 6)
    assert rt.hcgpuConvertPyArray(None, t, 2, C.byref(d)) == 0
    assert d.allocated == t.data_ptr() and list(d.sizes) == [4, 6] and list(d.strides) == [6, 1]
    tt = t.t()
    assert rt.hcgpuConvertPyArray(None, tt, 2, C.byref(d)) == 0
    assert list(d.sizes) == [6, 4] and list(d.strides) == [1, 6]


def test_convert_int64(rt):
    out = C.c_int64(0)
    assert rt.hcgpuConvertPyInt64(None, 1234567890123, C.byref(out)) == 0
    assert out.value == 1234567890123
    assert rt.hcgpuConvertPyInt64(None, "not a number", C.byref(out)) == 1


def test_convert_errors_return_one(rt):
    d = _Desc2()
    assert rt.hcgpuConvertPyArray(None, np.zeros(5), 2, C.byref(d)) == 1  # "Invalid rank"
    assert rt.hcgpuConvertPyArray(None, object(), 2, C.byref(d)) == 1


def test_search_paths_and_tracing(rt, capfd):
    rt.hcgpuSetRuntimeSearchPaths([str(REPO / "hc_b200" / "_native").encode()])
    rt.hcgpuEnableTraceFunctions(1)
    try:
        out = C.c_int64(0)
        rt.hcgpuConvertPyInt64(None, 5, C.byref(out))
    finally:
        rt.hcgpuEnableTraceFunctions(0)
    text = capfd.readouterr().out
    assert "hcgpuConvertPyInt64 enter" in text and "hcgpuConvertPyInt64 exit" in text


def test_hckernel_py_runtime_module_loads_and_toggles_tracing(capfd):
    from hc_b200.hckernel import py_runtime

    py_runtime.enable_func_tracing(1)
    py_runtime.enable_func_tracing(0)
    assert py_runtime.runtime_lib is not None


def test_get_kernel_failure_aborts_like_the_reference():
    if torch.cuda.is_available():
        pytest.skip("needs a host without a CUDA driver")
    code = (
        "import ctypes as C, sys; sys.path.insert(0, %r)\n"
        "from hc_b200 import capi\n"
        "rt = capi.load_python_runtime()\n"
        "h = C.c_void_p(0)\n"
        "rt.hcgpuGetKernel(C.byref(h), b'cuda:0', b'x', 1, b'k')\n"
        "print('survived')\n" % str(REPO)
    )
    proc = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True)
    assert proc.returncode == -6  # SIGABRT
    assert "Offload error: olCreateDevice failed" in proc.stderr
    assert "survived" not in proc.stdout
