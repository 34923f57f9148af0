"""numpy restatement of the q4f16 path + ctypes access to the C restatement.

Reference semantics followed (paths inside the reference tree):

* decode: ``q = (Wq[n, k//8] >> (4*(k%8))) & 0xF`` (low nibble = lowest k), then
  ``w = fp16(q - 7) * S[n, k//32]`` as ONE round-to-nearest-even fp16 multiply
  (generic TIR ops ``src/tir/op/op.cc:564,606,282``).
* matmul: operands cast to fp32 before the multiply, sum over ascending k in fp32 from 0
  (``python/tvm/relax/transform/legalize_ops.py:203-264``; pinned by
  ``tests/python/relax/test_transform_legalize_ops_index_linear_algebra.py:283-315``).
* astype: fp32 -> fp16 round-to-nearest-even (``legalize_ops.py:157-162``).
"""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libq4f16_oracle.so")
_lib = None


# ----------------------------------------------------------------------------- numpy form
def pack_nibbles(q: np.ndarray) -> np.ndarray:
    """q uint8 [N,K] with values 0..15 -> uint32 [N,K/8], element k in bits 4*(k%8).."""
    q = np.asarray(q)
    n, k = q.shape
    assert k % 8 == 0
    q = q.astype(np.uint32).reshape(n, k // 8, 8)
    shifts = (4 * np.arange(8, dtype=np.uint32))[None, None, :]
    return np.bitwise_or.reduce(q << shifts, axis=2).astype(np.uint32)


def unpack_nibbles(wq: np.ndarray) -> np.ndarray:
    """uint32 [N,K/8] -> uint8 [N,K]."""
    wq = np.asarray(wq, dtype=np.uint32)
    shifts = (4 * np.arange(8, dtype=np.uint32))[None, None, :]
    q = (wq[:, :, None] >> shifts) & np.uint32(0xF)
    return q.reshape(wq.shape[0], -1).astype(np.uint8)


# Nibble position p of a word of the "paired" layout holds element k = PAIRED_ORDER[p] of the word's eight
# (the library's offline repack, include/b200_q4f16.h B200_LAYOUT_PAIRED).  Stated here from the definition,
# nibble by nibble, to check the device permutation against.
PAIRED_ORDER = (0, 2, 4, 6, 1, 3, 5, 7)


def repack_paired(wq: np.ndarray) -> np.ndarray:
    """Reference nibble order -> paired layout, same shape."""
    q = unpack_nibbles(wq).reshape(wq.shape[0], -1, 8)
    return pack_nibbles(q[:, :, list(PAIRED_ORDER)].reshape(wq.shape[0], -1))


def unpack_paired(packed: np.ndarray) -> np.ndarray:
    """Paired layout -> reference nibble order."""
    q = unpack_nibbles(packed).reshape(packed.shape[0], -1, 8)
    inv = np.argsort(np.array(PAIRED_ORDER))
    return pack_nibbles(q[:, :, inv].reshape(packed.shape[0], -1))


def dequantize(wq: np.ndarray, scales: np.ndarray, group: int = 32) -> np.ndarray:
    """fp16 [N,K] = (q - 7) * scale, one fp16 rounding."""
    q = unpack_nibbles(wq).astype(np.int32) - 7
    s = np.asarray(scales, dtype=np.float16)
    assert q.shape[1] == s.shape[1] * group, (q.shape, s.shape)
    qh = q.astype(np.float16)  # exact, |q-7| <= 8
    sh = np.repeat(s, group, axis=1)
    # numpy's float16 multiply computes in fp32 and rounds once: the product of a 4-bit
    # integer and an 11-bit significand is exact in fp32, so this is one RN-even rounding.
    return (qh * sh).astype(np.float16)


def matmul_acc32(x: np.ndarray, w: np.ndarray) -> np.ndarray:
    """fp32 [M,N]: acc += f32(x[:,k]) * f32(w[:,k]) for k ascending (strict order)."""
    xf = np.asarray(x, dtype=np.float16).astype(np.float32)
    wf = np.asarray(w, dtype=np.float16).astype(np.float32)
    m, k = xf.shape
    n = wf.shape[0]
    acc = np.zeros((m, n), dtype=np.float32)
    for kk in range(k):
        acc += xf[:, kk, None] * wf[None, :, kk]
    return acc


def matmul(x: np.ndarray, wq: np.ndarray, scales: np.ndarray) -> np.ndarray:
    """fp16 [M,N] = astype(matmul(x, decode(wq, scales)^T, fp32), fp16)."""
    return matmul_acc32(x, dequantize(wq, scales)).astype(np.float16)


# ----------------------------------------------------------------------------- C form
def build_c_oracle(force: bool = False) -> str:
    """Compile oracle/q4f16_oracle.c with the committed Makefile; returns the .so path."""
    src = os.path.join(_HERE, "q4f16_oracle.c")
    if force or not os.path.exists(_LIB_PATH) or os.path.getmtime(_LIB_PATH) < os.path.getmtime(src):
        subprocess.run(["make", "-C", _HERE, "-B", "libq4f16_oracle.so"], check=True, capture_output=True)
    return _LIB_PATH


def _load():
    global _lib
    if _lib is None:
        if not os.path.exists(_LIB_PATH):
            build_c_oracle()
        lib = ctypes.CDLL(_LIB_PATH)
        i64, vp, ci = ctypes.c_int64, ctypes.c_void_p, ctypes.c_int
        lib.q4f16_oracle_dequantize.argtypes = [vp, vp, vp, i64, i64, ci]
        lib.q4f16_oracle_dequantize.restype = ci
        lib.q4f16_oracle_matmul.argtypes = [vp, vp, vp, vp, vp, i64, i64, i64, ci]
        lib.q4f16_oracle_matmul.restype = ci
        lib.q4f16_oracle_matmul_unfused.argtypes = [vp, vp, vp, vp, vp, i64, i64, i64, ci]
        lib.q4f16_oracle_matmul_unfused.restype = ci
        lib.q4f16_oracle_max_threads.restype = ci
        _lib = lib
    return _lib


def _ptr(a: np.ndarray):
    return a.ctypes.data_as(ctypes.c_void_p)


def c_max_threads() -> int:
    return int(_load().q4f16_oracle_max_threads())


def c_dequantize(wq: np.ndarray, scales: np.ndarray, nthreads: int = 0) -> np.ndarray:
    wq = np.ascontiguousarray(wq, dtype=np.uint32)
    s = np.ascontiguousarray(scales, dtype=np.float16)
    n, k = wq.shape[0], wq.shape[1] * 8
    assert s.shape == (n, k // 32)
    w = np.empty((n, k), dtype=np.float16)
    rc = _load().q4f16_oracle_dequantize(_ptr(wq), _ptr(s), _ptr(w), n, k, nthreads)
    if rc:
        raise ValueError(f"oracle dequantize failed rc={rc}")
    return w


def c_matmul(x, wq, scales, nthreads: int = 0, return_acc32: bool = False, unfused: bool = False):
    x = np.ascontiguousarray(x, dtype=np.float16)
    wq = np.ascontiguousarray(wq, dtype=np.uint32)
    s = np.ascontiguousarray(scales, dtype=np.float16)
    m, k = x.shape
    n = wq.shape[0]
    assert wq.shape == (n, k // 8) and s.shape == (n, k // 32), (x.shape, wq.shape, s.shape)
    y = np.empty((m, n), dtype=np.float16)
    if unfused:
        wtmp = np.empty((n, k), dtype=np.float16)
        rc = _load().q4f16_oracle_matmul_unfused(_ptr(x), _ptr(wq), _ptr(s), _ptr(wtmp), _ptr(y), m, n, k, nthreads)
        acc = None
    else:
        acc = np.empty((m, n), dtype=np.float32) if return_acc32 else None
        rc = _load().q4f16_oracle_matmul(
            _ptr(x), _ptr(wq), _ptr(s), _ptr(y), _ptr(acc) if acc is not None else None, m, n, k, nthreads
        )
    if rc:
        raise ValueError(f"oracle matmul failed rc={rc}")
    return (y, acc) if return_acc32 else y
