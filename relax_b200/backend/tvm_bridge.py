"""Finds an importable TVM with Relax and registers the kernels' packed functions with its FFI."""
from __future__ import annotations

_tvm = None
_registered = False


def import_tvm():
    """Returns the tvm module (the tilelang wheel bundles TVM 0.23 and puts it on sys.path)."""
    global _tvm
    if _tvm is None:
        try:
            import tvm  # noqa: F401
        except ImportError:
            import tilelang  # noqa: F401
            import tvm  # noqa: F401
        from tvm import relax  # noqa: F401

        _tvm = tvm
    return _tvm


def have_tvm() -> bool:
    try:
        import_tvm()
        return True
    except Exception:
        return False


def register_packed_funcs(override: bool = True):
    """Registers b200.q4f16_matmul / b200.q4f16_dequantize as global functions of the TVM FFI, so
    that ``R.call_dps_packed("b200.q4f16_matmul", (x, wq, scales), out_sinfo)`` (the descendant's
    spelling of the reference's ``R.call_tir("<symbol>", ...)``) reaches the kernel library."""
    global _registered
    import_tvm()
    import tvm_ffi

    from .. import registry

    for name in ("b200.q4f16_matmul", "b200.q4f16_dequantize"):
        tvm_ffi.register_global_func(name, registry.get_global_func(name), override=override)
    _registered = True
