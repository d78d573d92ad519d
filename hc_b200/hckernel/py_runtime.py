"""ctypes access to ``libhc-python-runtime.so`` (reference:
``hckernel/py_runtime.py:9-28``): loads the library, hands it the runtime
search paths and exposes the trace switch."""

import ctypes

from .utils import get_runtime_search_paths, load_lib

runtime_lib = load_lib("hc-python-runtime")

_enable_tracing = runtime_lib.hcgpuEnableTraceFunctions
_enable_tracing.argtypes = [ctypes.c_int]
_enable_tracing.restype = None

_set_runtime_search_paths = runtime_lib.hcgpuSetRuntimeSearchPaths
_set_runtime_search_paths.argtypes = [ctypes.py_object]
_set_runtime_search_paths.restype = None

_search_paths = [p.encode() for p in get_runtime_search_paths()]
_set_runtime_search_paths(ctypes.py_object(_search_paths))

_loader = load_lib("hc-gpu-runtime-loader")
_loader.enableFuncTracing.argtypes = [ctypes.c_int]
_loader.enableFuncTracing.restype = None


def enable_func_tracing(val):
    """Trace both the hcgpu* layer and the ol* loader underneath it."""
    _enable_tracing(ctypes.c_int(int(val)))
    _loader.enableFuncTracing(ctypes.c_int(int(val)))
