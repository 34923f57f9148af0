"""ctypes binding of the C ABI declared in include/b200_q4f16.h.

The library is the product; there is no fallback.  If the shared object is missing the
import of :mod:`relax_b200` still works (so the build step can run) but every call raises.
"""
from __future__ import annotations

import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.environ.get("B200_Q4F16_LIB") or os.path.join(_HERE, "libb200_q4f16.so")

OK, EINVAL, ENODEVICE, ELAUNCH, EDEVICE, ENOTREADY = 0, -1, -2, -3, -4, -5
ATTN_EARLY_KV_LOADS = 1   # B200_ATTN_EARLY_KV_LOADS
FAMILY_AUTO, FAMILY_GEMV, FAMILY_GEMM = 0, 1, 2
LAYOUT_REFERENCE, LAYOUT_PAIRED = 0, 1


def family_with_layout(family, layout):
    """The `family` argument of b200_q4f16_matmul_dl_family that also names the weight layout of the call."""
    return family | ((layout + 1) << 8)


class B200Error(RuntimeError):
    """Raised when an entry point returns a non-zero status; carries the code."""

    def __init__(self, code: int, msg: str):
        super().__init__(f"[b200 {code}] {msg}")
        self.code = code
        self.message = msg


class DLDevice(ctypes.Structure):
    _fields_ = [("device_type", ctypes.c_int32), ("device_id", ctypes.c_int32)]


class DLDataType(ctypes.Structure):
    _fields_ = [("code", ctypes.c_uint8), ("bits", ctypes.c_uint8), ("lanes", ctypes.c_uint16)]


class DLTensor(ctypes.Structure):
    _fields_ = [
        ("data", ctypes.c_void_p),
        ("device", DLDevice),
        ("ndim", ctypes.c_int32),
        ("dtype", DLDataType),
        ("shape", ctypes.POINTER(ctypes.c_int64)),
        ("strides", ctypes.POINTER(ctypes.c_int64)),
        ("byte_offset", ctypes.c_uint64),
    ]


class PeerReduce(ctypes.Structure):
    """B200PeerReduce of include/b200_q4f16.h."""

    _fields_ = [
        ("world", ctypes.c_int32), ("rank", ctypes.c_int32),
        ("peer_y", ctypes.c_void_p * 8), ("peer_flags", ctypes.c_void_p * 8),
        ("flag_base", ctypes.c_int32), ("epoch", ctypes.c_void_p), ("done_counter", ctypes.c_void_p),
        ("out", ctypes.c_void_p),
    ]


class DecodeLayer(ctypes.Structure):
    """B200DecodeLayer of include/b200_q4f16.h."""

    _fields_ = [
        ("world", ctypes.c_int32), ("rank", ctypes.c_int32),
        ("hidden", ctypes.c_int64), ("inter_local", ctypes.c_int64), ("max_ctx", ctypes.c_int64),
        ("heads", ctypes.c_int32), ("eps", ctypes.c_float),
        ("x_in", ctypes.c_void_p), ("delta_in", ctypes.c_void_p),
        ("x_mid", ctypes.c_void_p), ("qkv", ctypes.c_void_p), ("attn", ctypes.c_void_p), ("o", ctypes.c_void_p),
        ("x_out", ctypes.c_void_p), ("act", ctypes.c_void_p), ("down", ctypes.c_void_p),
        ("norm1", ctypes.c_void_p), ("norm2", ctypes.c_void_p),
        ("cos_t", ctypes.c_void_p), ("sin_t", ctypes.c_void_p), ("pos", ctypes.c_void_p),
        ("k_cache", ctypes.c_void_p), ("v_cache", ctypes.c_void_p),
        ("scratch", ctypes.c_void_p), ("step", ctypes.c_void_p),
        ("wq_qkv", ctypes.c_void_p), ("s_qkv", ctypes.c_void_p), ("wq_o", ctypes.c_void_p), ("s_o", ctypes.c_void_p),
        ("wq_gu", ctypes.c_void_p), ("s_gu", ctypes.c_void_p), ("wq_down", ctypes.c_void_p), ("s_down", ctypes.c_void_p),
        ("reduce_o", PeerReduce), ("reduce_down", PeerReduce),
    ]


# name -> (restype, argtypes); one entry per prototype in include/b200_q4f16.h
_vp, _i64, _ci = ctypes.c_void_p, ctypes.c_int64, ctypes.c_int
_dlp = ctypes.POINTER(DLTensor)
_ip = ctypes.POINTER(ctypes.c_int)
PROTOTYPES = {
    "b200_last_error": (ctypes.c_char_p, []),
    "b200_abi_version": (_ci, []),
    "b200_set_stream": (_ci, [_vp]),
    "b200_get_stream": (_vp, []),
    "b200_q4f16_dequantize": (_ci, [_vp, _vp, _vp, _i64, _i64, _vp]),
    "b200_q4f16_matmul": (_ci, [_vp, _vp, _vp, _vp, _i64, _i64, _i64, _vp]),
    "b200_q4f16_gemv": (_ci, [_vp, _vp, _vp, _vp, _i64, _i64, _i64, _vp]),
    "b200_q4f16_gemm": (_ci, [_vp, _vp, _vp, _vp, _i64, _i64, _i64, _vp]),
    "b200_q4f16_gemm_ws": (_ci, [_vp, _vp, _vp, _vp, _i64, _i64, _i64, _vp]),
    "b200_q4f16_matmul_host": (_ci, [_vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _vp]),
    "b200_q4f16_matmul_dl": (_ci, [_dlp, _dlp, _dlp, _dlp]),
    "b200_q4f16_dequantize_dl": (_ci, [_dlp, _dlp, _dlp]),
    "b200_q4f16_matmul_dl_family": (_ci, [_dlp, _dlp, _dlp, _dlp, ctypes.c_int32]),
    "b200_allreduce_peer": (_ci, [_i64, ctypes.POINTER(PeerReduce), _vp]),
    "b200_lm_head_scratch_bytes": (_i64, []),
    "b200_lm_head": (_ci, [_vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _vp]),
    "b200_q4f16_repack": (_ci, [_vp, _vp, _i64, _i64, ctypes.c_int32, _vp]),
    "b200_q4f16_unpack": (_ci, [_vp, _vp, _i64, _i64, ctypes.c_int32, _vp]),
    "b200_q4f16_matmul_layout": (_ci, [_vp, _vp, _vp, _vp, _i64, _i64, _i64, ctypes.c_int32, _vp]),
    "b200_q4f16_dequantize_layout": (_ci, [_vp, _vp, _vp, _i64, _i64, ctypes.c_int32, _vp]),
    "b200_q4f16_matmul_packed": (ctypes.c_int32, [_vp, _ip, _ci, _vp, _ip, _vp]),
    "b200_q4f16_dequantize_packed": (ctypes.c_int32, [_vp, _ip, _ci, _vp, _ip, _vp]),
    "b200_q4f16_gemv_rmsnorm": (_ci, [_vp, _vp, _vp, _vp, ctypes.c_float, _vp, _vp, _vp, _i64, _i64, _i64, _vp]),
    "b200_q4f16_gemv_rmsnorm_rope": (_ci, [_vp, _vp, _vp, _vp, ctypes.c_float, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _vp]),
    "b200_q4f16_gemv_swiglu": (_ci, [_vp, _vp, _vp, _vp, _i64, _i64, _i64, _vp]),
    "b200_q4f16_gemv_allreduce": (_ci, [_vp, _vp, _vp, _vp, _i64, _i64, _i64, ctypes.c_int32, ctypes.POINTER(PeerReduce), _vp]),
    "b200_decode_layer_scratch_bytes": (_i64, [_i64, _i64]),
    "b200_decode_layer": (_ci, [ctypes.POINTER(DecodeLayer), _vp]),
    "b200_rmsnorm": (_ci, [_vp, _vp, _vp, _vp, _i64, _i64, ctypes.c_float, _vp]),
    "b200_rope_kv_append": (_ci, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _vp]),
    "b200_attn_decode_scratch_bytes": (_i64, [_i64, _i64, _i64]),
    "b200_attn_decode": (_ci, [_vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, ctypes.c_uint32, _vp]),
    "b200_attn_decode_fused_scratch_bytes": (_i64, [_i64, _i64, _i64]),
    "b200_attn_decode_fused": (_ci, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _vp]),
    "b200_attn_decode_rope": (_ci, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _vp]),
    "b200_attn_decode_static": (_ci, [_vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, ctypes.c_uint32, _vp]),
    "b200_silu_mul": (_ci, [_vp, _vp, _i64, _i64, _vp]),
    "b200_embed_rows": (_ci, [_vp, _vp, _vp, _i64, _i64, _i64, _vp]),
    "b200_advance_pos": (_ci, [_vp, _i64, _vp]),
    "b200_launch_count": (_i64, []),
    "b200_reset_launch_count": (None, []),
    "b200_device_error_flags": (_ci, []),
    "b200_set_option": (_ci, [ctypes.c_char_p, _i64]),
    "b200_get_option": (_i64, [ctypes.c_char_p]),
}

_lib = None


def lib() -> ctypes.CDLL:
    """The loaded library; raises if it has not been built (python -m relax_b200.build)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise B200Error(ENODEVICE, f"{LIB_PATH} is missing: build it with `python -m relax_b200.build`; "
                            "there is no fallback implementation")
        handle = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in PROTOTYPES.items():
            fn = getattr(handle, name)  # AttributeError if the .so lacks a declared symbol
            fn.restype = res
            fn.argtypes = args
        _lib = handle
    return _lib


def last_error() -> str:
    return lib().b200_last_error().decode("utf-8", "replace")


def check(rc: int) -> None:
    if rc != 0:
        raise B200Error(rc, last_error())


def set_option(name: str, value: int) -> None:
    check(lib().b200_set_option(name.encode(), int(value)))


def get_option(name: str) -> int:
    return int(lib().b200_get_option(name.encode()))
