"""`hckernel`: the kernel-decorator call surface of the reference, backed by
precompiled sm_100a kernels.

Import from :mod:`hc_b200.hckernel.kernel` exactly what a program written for
the reference imports from ``hckernel.kernel``.  Adding ``hc_b200`` to
``sys.path`` makes this package importable under its original top-level name
``hckernel``.
"""
