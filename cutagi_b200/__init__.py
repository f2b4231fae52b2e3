"""cutagi_b200 - B200 (sm_100a) kernels for cuTAGI's Linear / Conv2d hot path behind a C ABI.

The package is a thin ctypes layer over ``libtagi_b200.so`` (declared in ``include/tagi_b200.h``).
There is no CPU or PyTorch fallback: if the library has not been built, importing ``capi`` raises.
Build it with ``python -m cutagi_b200.build`` (nvcc, sm_100a).
"""
from .capi import TagiError, ConvGeom, lib, load  # noqa: F401

__version__ = "0.1.0"
