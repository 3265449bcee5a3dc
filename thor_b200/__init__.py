"""thor_b200 — B200 (sm_100a) kernels for the hot path of Thor's expression engine.

The product is ``lib/libthor_b200.so`` (C ABI in ``include/thor_b200.h``) plus the C++ host layer
``lib/libthor_b200_host.so`` that mirrors the reference's Expression / FusedEquation /
CubReduction / TypeConverter interface.  This Python package is a thin ctypes binding over both,
in the role of the reference's ``bindings/python`` module; torch is used only for device memory,
streams and ``torch.distributed``.  There is no CPU fallback: a missing library raises.
"""
from . import _native  # noqa: F401  (loads the library or raises)
from ._native import ThorB200Error, ThorB200InvalidArgument, launch_count
from .dtypes import DataType
from .type_converter import TypeConverter

__all__ = ["DataType", "TypeConverter", "ThorB200Error", "ThorB200InvalidArgument", "launch_count"]
