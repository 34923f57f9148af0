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


LAYOUTS = {"reference": _lib.LAYOUT_REFERENCE, "paired": _lib.LAYOUT_PAIRED}


def _layout_code(layout) -> int:
    if isinstance(layout, str):
        if layout not in LAYOUTS:
            raise ValueError(f"unknown weight layout {layout!r}; one of {sorted(LAYOUTS)}")
        return LAYOUTS[layout]
    return int(layout)


class _option_scope:
    """Sets a process-wide option of the library for the duration of a block."""

    def __init__(self, name: str, value: int):
        self.name, self.value = name, value

    def __enter__(self):
        L = _lib.lib()
        self.saved = L.b200_get_option(self.name.encode())
        _lib.check(L.b200_set_option(self.name.encode(), self.value))

    def __exit__(self, *exc):
        _lib.check(_lib.lib().b200_set_option(self.name.encode(), self.saved))


def q4f16_matmul(x: torch.Tensor, wq: torch.Tensor, scales: torch.Tensor, out: torch.Tensor | None = None,
                 family: str = "auto", layout=None) -> torch.Tensor:
    """y[M,N] fp16 = x[M,K] . decode(wq[N,K/8], scales[N,K/32])^T, through the DLPack entry point
    (all validation happens in the library).  ``family`` = "auto" | "gemv" | "gemm" picks the raw
    entry point of one kernel family instead.  ``layout`` ("reference" | "paired") names the nibble order
    of ``wq`` for this call; None takes the library's option "weights.layout"."""
    if out is None:
        out = torch.empty((x.shape[0], wq.shape[0]), dtype=torch.float16, device=x.device)
    L = _lib.lib()
    if family == "auto":
        with _on(x.device):
            L.b200_set_stream(_stream_ptr(x.device))
            vx, vw, vs, vy = (_DLView(t) for t in (x, wq, scales, out))
            if layout is None:
                _lib.check(L.b200_q4f16_matmul_dl(vx.ptr(), vw.ptr(), vs.ptr(), vy.ptr()))
            else:
                code = _lib.family_with_layout(_lib.FAMILY_AUTO, _layout_code(layout))
                _lib.check(L.b200_q4f16_matmul_dl_family(vx.ptr(), vw.ptr(), vs.ptr(), vy.ptr(), code))
        return out
    fn = {"gemv": L.b200_q4f16_gemv, "gemm": L.b200_q4f16_gemm, "gemm_ws": L.b200_q4f16_gemm_ws,
          "matmul": L.b200_q4f16_matmul}[family]
    M, K = x.shape
    N = wq.shape[0]
    with _on(x.device):
        if layout is None:
            _lib.check(fn(x.data_ptr(), wq.data_ptr(), scales.data_ptr(), out.data_ptr(), M, N, K, _stream_ptr(x.device)))
        else:
            with _option_scope("weights.layout", _layout_code(layout)):
                _lib.check(fn(x.data_ptr(), wq.data_ptr(), scales.data_ptr(), out.data_ptr(), M, N, K, _stream_ptr(x.device)))
    return out


def q4f16_repack(wq: torch.Tensor, layout="paired", out: torch.Tensor | None = None) -> torch.Tensor:
    """The packed words of ``wq`` (reference nibble order) in ``layout``; ``out`` may be ``wq`` itself."""
    return _repack(wq, layout, out, to_layout=True)


def q4f16_unpack(packed: torch.Tensor, layout="paired", out: torch.Tensor | None = None) -> torch.Tensor:
    """Back to the reference's nibble order: the exact inverse of :func:`q4f16_repack`."""
    return _repack(packed, layout, out, to_layout=False)


def _repack(src: torch.Tensor, layout, out, to_layout: bool) -> torch.Tensor:
    if src.dtype not in (torch.int32, torch.uint32) or src.dim() != 2 or not src.is_contiguous():
        raise ValueError("packed weights are a contiguous 2-D 32-bit integer tensor [N, K/8]")
    if out is None:
        out = torch.empty_like(src)
    if out.shape != src.shape or out.dtype != src.dtype or out.device != src.device or not out.is_contiguous():
        raise ValueError("out must match the packed tensor")
    L = _lib.lib()
    fn = L.b200_q4f16_repack if to_layout else L.b200_q4f16_unpack
    N, K = src.shape[0], src.shape[1] * 8
    with _on(src.device):
        _lib.check(fn(src.data_ptr(), out.data_ptr(), N, K, _layout_code(layout), _stream_ptr(src.device)))
    return out


def q4f16_dequantize(wq: torch.Tensor, scales: torch.Tensor, out: torch.Tensor | None = None, layout=None) -> torch.Tensor:
    """w[N,K] fp16 = decode(wq, scales); bit-exact with the reference's decode stage."""
    if out is None:
        out = torch.empty((wq.shape[0], wq.shape[1] * 8), dtype=torch.float16, device=wq.device)
    L = _lib.lib()
    if layout is not None:
        N, K = wq.shape[0], wq.shape[1] * 8
        with _on(wq.device):
            _lib.check(L.b200_q4f16_dequantize_layout(wq.data_ptr(), scales.data_ptr(), out.data_ptr(), N, K,
                                                      _layout_code(layout), _stream_ptr(wq.device)))
        return out
    with _on(wq.device):
        L.b200_set_stream(_stream_ptr(wq.device))
        vw, vs, vo = (_DLView(t) for t in (wq, scales, out))
        _lib.check(L.b200_q4f16_dequantize_dl(vw.ptr(), vs.ptr(), vo.ptr()))
    return out


def launch_count() -> int:
    return int(_lib.lib().b200_launch_count())


def reset_launch_count() -> None:
    _lib.lib().b200_reset_launch_count()
