"""CPU oracle for the q4f16 dequantize+matmul path.  TEST INFRASTRUCTURE ONLY.

Two forms of the same restatement of the reference's semantics:

* ``numpy`` functions in :mod:`oracle.q4f16` (small cases, readable), and
* a C library (``oracle/q4f16_oracle.c``) reached through ``ctypes`` for sizes the
  numpy form would take minutes on; it is also what the benchmark times as the CPU
  baseline.

Only ``tests/``, ``__graft_entry__.smoke()`` and the ``cpu_baseline`` / reference arm of
``bench.py`` may import this package.  Parity with the reference itself is unpinned (it
ships no vectors for this path and cannot be built here); see the header of
``q4f16_oracle.c`` for what the oracle is pinned against.
"""
from .q4f16 import (  # noqa: F401
    pack_nibbles,
    unpack_nibbles,
    repack_paired,
    unpack_paired,
    dequantize,
    matmul,
    matmul_acc32,
    c_dequantize,
    c_matmul,
    c_max_threads,
    build_c_oracle,
)
