"""paella_b200: B200-native serving hot path behind Paella's job-plugin boundary.

The product is the native library ``libpaella_b200.so`` (CUDA kernels, notification ring,
scheduler, server, load generator) and the job plugins ``jobs/libjob_*.so``.  This package
only locates and binds them (ctypes) for tests and the benchmark, and holds the model packer.
There is no CPU fallback: if the native library is missing, loading raises.
"""
from . import packer  # noqa: F401
from .capi import lib, load, plugin_path, PbError, check  # noqa: F401
