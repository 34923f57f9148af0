"""Host-side operators on torch tensors: thin, allocation-explicit wrappers over the C ABI.

These mirror how the reference reaches an external kernel: destination-passing packed
functions on DLPack tensors (``R.call_tir("b200.q4f16_matmul", (x, wq, scales), out_sinfo)``;
reference: python/tvm/relax/op/base.py:47-91, src/relax/transform/call_tir_rewrite.cc:55-116).
torch is used only for device memory and streams.
"""
from __future__ import annotations

import ctypes

import torch

from . import _lib
from ._lib import B200Error, DLDataType, DLDevice, DLTensor  # noqa: F401


import contextlib


def _stream_ptr(device) -> int:
    if torch.device(device).type != "cuda":
        return 0
    return torch.cuda.current_stream(device).cuda_stream


def _on(device):
    """Makes `device` current for the call; a CPU tensor is passed through so that the library's
    own validation rejects it (there is no host implementation to fall back to)."""
    return torch.cuda.device(device) if torch.device(device).type == "cuda" else contextlib.nullcontext()


_DTYPES = {
    torch.float16: (2, 16),
    torch.float32: (2, 32),
    torch.uint32: (1, 32),
    torch.int32: (0, 32),
    torch.uint8: (1, 8),
}


class _DLView:
    """Keeps the ctypes arrays of a DLTensor view alive."""

    def __init__(self, t: torch.Tensor):
        code, bits = _DTYPES[t.dtype]
        self.shape = (ctypes.c_int64 * t.dim())(*t.shape)
        self.strides = (ctypes.c_int64 * t.dim())(*t.stride())
        if t.is_cuda:
            dev = DLDevice(2, t.device.index if t.device.index is not None else torch.cuda.current_device())
        else:
            dev = DLDevice(1, 0)
        self.tensor = DLTensor(
            ctypes.c_void_p(t.data_ptr()), dev, t.dim(), DLDataType(code, bits, 1),
            ctypes.cast(self.shape, ctypes.POINTER(ctypes.c_int64)),
            ctypes.cast(self.strides, ctypes.POINTER(ctypes.c_int64)), 0,
        )
        self.keep = t

    def ptr(self):
        return ctypes.byref(self.tensor)


def to_dltensor(t: torch.Tensor) -> _DLView:
    return _DLView(t)


def q4f16_matmul(x: torch.Tensor, wq: torch.Tensor, scales: torch.Tensor, out: torch.Tensor | None = None,
                 family: str = "auto") -> torch.Tensor:
    """y[M,N] fp16 = x[M,K] . decode(wq[N,K/8], scales[N,K/32])^T, through the DLPack entry point
    (all validation happens in the library).  ``family`` = "auto" | "gemv" | "gemm" picks the raw
    entry point of one kernel family instead."""
    if out is None:
        out = torch.empty((x.shape[0], wq.shape[0]), dtype=torch.float16, device=x.device)
    L = _lib.lib()
    if family == "auto":
        with _on(x.device):
            L.b200_set_stream(_stream_ptr(x.device))
            vx, vw, vs, vy = (_DLView(t) for t in (x, wq, scales, out))
            _lib.check(L.b200_q4f16_matmul_dl(vx.ptr(), vw.ptr(), vs.ptr(), vy.ptr()))
        return out
    fn = {"gemv": L.b200_q4f16_gemv, "gemm": L.b200_q4f16_gemm, "gemm_ws": L.b200_q4f16_gemm_ws,
          "matmul": L.b200_q4f16_matmul}[family]
    M, K = x.shape
    N = wq.shape[0]
    with _on(x.device):
        _lib.check(fn(x.data_ptr(), wq.data_ptr(), scales.data_ptr(), out.data_ptr(), M, N, K, _stream_ptr(x.device)))
    return out


def q4f16_dequantize(wq: torch.Tensor, scales: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    """w[N,K] fp16 = decode(wq, scales); bit-exact with the reference's decode stage."""
    if out is None:
        out = torch.empty((wq.shape[0], wq.shape[1] * 8), dtype=torch.float16, device=wq.device)
    L = _lib.lib()
    with _on(wq.device):
        L.b200_set_stream(_stream_ptr(wq.device))
        vw, vs, vo = (_DLView(t) for t in (wq, scales, out))
        _lib.check(L.b200_q4f16_dequantize_dl(vw.ptr(), vs.ptr(), vo.ptr()))
    return out


def launch_count() -> int:
    return int(_lib.lib().b200_launch_count())


def reset_launch_count() -> None:
    _lib.lib().b200_reset_launch_count()
