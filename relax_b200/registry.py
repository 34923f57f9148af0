"""Name -> packed function registry for the kernels, mirroring the reference's global function
table (include/tvm/runtime/registry.h:339-340; Python: tvm.register_func / tvm.get_global_func).

The built-in entries are destination-passing functions on torch tensors or on anything that
exports DLPack (``__dlpack__``), exactly what ``R.call_tir("b200.q4f16_matmul", (x, wq, scales),
out_sinfo)`` hands to a packed function: inputs first, pre-allocated output last, no return value.
"""
from __future__ import annotations

from typing import Callable, Dict

import torch

from . import ops

_REGISTRY: Dict[str, Callable] = {}


def register_func(name: str, f: Callable | None = None, override: bool = False):
    def deco(fn):
        if name in _REGISTRY and not override:
            raise ValueError(f"global function {name} is already registered")
        _REGISTRY[name] = fn
        return fn

    return deco(f) if f is not None else deco


def get_global_func(name: str, allow_missing: bool = False):
    if name not in _REGISTRY:
        if allow_missing:
            return None
        raise ValueError(f"Cannot find global function {name}")
    return _REGISTRY[name]


def list_global_func_names():
    return sorted(_REGISTRY)


def as_torch(t) -> torch.Tensor:
    """Zero-copy view of a DLPack-capable tensor (TVM NDArray/Tensor, torch, cupy ...)."""
    if isinstance(t, torch.Tensor):
        return t
    v = torch.from_dlpack(t)
    return v


def _as_u32(t: torch.Tensor) -> torch.Tensor:
    # DLPack producers that have no unsigned 32-bit type hand the packed words over as int32
    return t.view(torch.uint32) if t.dtype == torch.int32 else t


@register_func("b200.q4f16_matmul")
def _q4f16_matmul(x, wq, scales, y):
    ops.q4f16_matmul(as_torch(x), _as_u32(as_torch(wq)), as_torch(scales), out=as_torch(y))


@register_func("b200.q4f16_dequantize")
def _q4f16_dequantize(wq, scales, w):
    ops.q4f16_dequantize(_as_u32(as_torch(wq)), as_torch(scales), out=as_torch(w))
