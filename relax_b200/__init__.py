"""relax_b200: B200-native q4f16 dequantize+matmul kernels behind Relax's plugin surface.

Only the path is here: the CUDA kernel library (``csrc/`` -> ``libb200_q4f16.so``, C ABI in
``include/b200_q4f16.h``), its ctypes/torch host binding, and the host-side mirror of the
reference's plugin interface for this path (pattern table, codegen entry, packed-function
registry).  No CPU or library fallback exists: without the built extension calls raise.
"""
from ._lib import B200Error, LIB_PATH, get_option, last_error, set_option  # noqa: F401

__all__ = ["B200Error", "LIB_PATH", "set_option", "get_option", "last_error"]
