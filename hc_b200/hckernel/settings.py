"""Run-time switches read from ``HC_*`` environment variables at import
(reference: ``hckernel/settings.py:24-30`` reads its dump flags the same way).

``HC_TRACE``     1: print enter/exit of every runtime-library call
``HC_DEVICE``    default device description when a kernel names none
                 reachable here ("cuda:0")
``HC_SYNC``      1: block the host after every launch, as the reference does
``HC_GEMM_VARIANT`` 0 automatic, 1 one CTA per tile, 2 CTA pair, 3 CUDA cores
``HC_CONV_VARIANT`` 0 mapped work-groups that form a float32 convolution run on the
                 tensor cores, 1 they run as the body tiles them (gathered kernel);
                 read at every launch, so a program may also set
                 ``settings.CONV_VARIANT``
"""

from .utils import readenv as _readenv_raw

settings = {}


def _readenv(name, ctor, default):
    value = _readenv_raw(name, ctor, default)
    settings[name[len("HC_"):]] = value
    return value


TRACE = _readenv("HC_TRACE", int, 0)
DEVICE = _readenv("HC_DEVICE", str, "cuda:0")
GEMM_VARIANT = _readenv("HC_GEMM_VARIANT", int, 0)
SYNC = _readenv("HC_SYNC", int, 0)
CONV_VARIANT = _readenv("HC_CONV_VARIANT", int, 0)
