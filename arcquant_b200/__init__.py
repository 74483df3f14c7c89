"""arcquant_b200: the ARC-NVFP4 quantized-linear hot path for NVIDIA B200 (sm_100a).

Native code lives in ``libarcq.so`` (C ABI, ``include/arcq.h``); ``agemm`` is the
reference-compatible operator module on top of it; ``ops`` offers the same
operators through ctypes.  Nothing here computes on the CPU.
"""
from . import _lib  # noqa: F401

__all__ = ["_lib", "ops", "synth"]
