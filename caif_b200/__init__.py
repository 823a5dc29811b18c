"""caif_b200: B200-native (sm_100a) quantized frozen-linear path of cppaif/caif.

The product is the shared library `libcaifq.so` (C ABI in include/caifq.h) and
the C++ layer classes under caif_b200/host/ that mirror the reference's
CAIF_DeviceFrozenLinear / CAIF_DeviceLoRAAdapter / CAIF_DeviceMoEFrozenExpert.
This Python package is the ctypes binding used by the tests, the benchmark and
the multi-GPU harness; it holds no compute of its own and has no fallback.
"""
from . import native  # noqa: F401

__all__ = ["native"]
