"""Small helpers shared by the package (reference: ``hckernel/utils.py``)."""

import ctypes
import os
import sys
import warnings


def readenv(name, ctor, default):
    """Value of environment variable ``name`` converted with ``ctor``; the
    default when it is unset, and the default plus a warning when it does not
    parse (reference: utils.py:12-24)."""
    raw = os.environ.get(name)
    if raw is None:
        return default() if callable(default) else default
    try:
        return ctor(raw)
    except Exception:
        warnings.warn(f"environ {name} defined but failed to parse '{raw}'", RuntimeWarning)
        return default


def get_runtime_search_paths():
    """Where the runtime libraries are looked for: the package's ``_native``
    directory first, then every ``PYTHONPATH`` entry (reference: utils.py:26-35)."""
    here = os.path.dirname(os.path.abspath(__file__))
    paths = [os.path.join(os.path.dirname(here), "_native")]
    paths += [p for p in os.environ.get("PYTHONPATH", "").split(os.pathsep) if p]
    return paths


def load_lib(name):
    """``ctypes.CDLL`` of ``lib<name>.so`` from the first search path that has
    it; ``ValueError`` listing every attempt otherwise (reference:
    utils.py:38-61)."""
    if not sys.platform.startswith("linux"):
        raise ValueError(f"Unsupported platform: {sys.platform}")
    lib_name = f"lib{name}.so"
    errors = []
    for path in get_runtime_search_paths():
        full = os.path.join(path, lib_name) if path else lib_name
        try:
            return ctypes.PyDLL(full) if name == "hc-python-runtime" else ctypes.CDLL(full)
        except OSError as exc:
            errors.append(f'CDLL("{full}"): {exc}')
    raise ValueError(f'load_lib("{name}") failed:\n' + "\n".join(errors))
