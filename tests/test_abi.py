"""CPU tests of the drop-in boundary: the library loads, exports every declared symbol,
and its entry points validate arguments and fail loudly without a GPU (no fallback)."""
import ctypes
import os
import re

import numpy as np
import pytest
import torch

import relax_b200
from relax_b200 import _lib, ops, synth

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "b200_q4f16.h")).read()
    return sorted(set(re.findall(r"B200_API[^;(]*?\b(b200_\w+)\s*\(", text)))


def test_header_symbols_all_exported_and_bound():
    syms = declared_symbols()
    assert len(syms) >= 15
    handle = ctypes.CDLL(_lib.LIB_PATH)
    for s in syms:
        assert hasattr(handle, s), f"{s} declared in include/b200_q4f16.h but not exported"
    assert sorted(_lib.PROTOTYPES) == syms, "ctypes prototypes out of sync with the header"
    assert _lib.lib().b200_abi_version() == 102


def _cpu_case(m=2, n=16, k=64):
    x, wq, s = synth.make_case(m, n, k)
    return torch.from_numpy(x), torch.from_numpy(wq), torch.from_numpy(s)


def test_cpu_tensors_are_rejected_not_computed():
    x, wq, s = _cpu_case()
    with pytest.raises(relax_b200.B200Error) as e:
        ops.q4f16_matmul(x, wq, s)
    assert e.value.code == _lib.EINVAL and "not on a CUDA device" in e.value.message
    with pytest.raises(relax_b200.B200Error):
        ops.q4f16_dequantize(wq, s)


@pytest.mark.skipif(torch.cuda.is_available(), reason="checks the no-GPU behaviour")
def test_raw_entry_points_fail_loudly_without_a_gpu():
    x, wq, s = _cpu_case()
    y = torch.empty((2, 16), dtype=torch.float16)
    rc = _lib.lib().b200_q4f16_matmul(x.data_ptr(), wq.data_ptr(), s.data_ptr(), y.data_ptr(), 2, 16, 64, None)
    assert rc == _lib.ENODEVICE and "CUDA" in _lib.last_error()


def _dl(t, **over):
    v = ops.to_dltensor(t)
    for k_, val in over.items():
        if k_ == "device_type":
            v.tensor.device.device_type = val
        elif k_ == "code":
            v.tensor.dtype.code = val
        elif k_ == "bits":
            v.tensor.dtype.bits = val
        elif k_ == "ndim":
            v.tensor.ndim = val
    return v


def test_dlpack_validation_messages():
    L = _lib.lib()
    x, wq, s = _cpu_case()
    y = torch.empty((2, 16), dtype=torch.float16)

    def call(vx, vw, vs, vy):
        rc = L.b200_q4f16_matmul_dl(vx.ptr(), vw.ptr(), vs.ptr(), vy.ptr())
        return rc, _lib.last_error()

    cuda = dict(device_type=2)
    # wrong dtype of the packed weights
    rc, msg = call(_dl(x, **cuda), _dl(wq.view(torch.int32), **cuda), _dl(s, **cuda), _dl(y, **cuda))
    assert rc == _lib.EINVAL and "wq must be uint32" in msg
    # K not a multiple of 32
    x40 = torch.zeros((2, 40), dtype=torch.float16)
    rc, msg = call(_dl(x40, **cuda), _dl(wq, **cuda), _dl(s, **cuda), _dl(y, **cuda))
    assert rc == _lib.EINVAL and "multiple of the group size" in msg
    # shape disagreement between wq and x
    rc, msg = call(_dl(x, **cuda), _dl(wq[:, :4].contiguous(), **cuda), _dl(s, **cuda), _dl(y, **cuda))
    assert rc == _lib.EINVAL and "wq is" in msg
    # scales with the wrong group count
    rc, msg = call(_dl(x, **cuda), _dl(wq, **cuda), _dl(s[:, :1].contiguous(), **cuda), _dl(y, **cuda))
    assert rc == _lib.EINVAL and "scales is" in msg
    # output of the wrong shape
    rc, msg = call(_dl(x, **cuda), _dl(wq, **cuda), _dl(s, **cuda), _dl(y[:, :8].contiguous(), **cuda))
    assert rc == _lib.EINVAL and "y is" in msg
    # non-contiguous activation
    xt = torch.zeros((64, 2), dtype=torch.float16).t()
    rc, msg = call(_dl(xt, **cuda), _dl(wq, **cuda), _dl(s, **cuda), _dl(y, **cuda))
    assert rc == _lib.EINVAL and "not contiguous" in msg
    # rank
    rc, msg = call(_dl(x.reshape(2, 8, 8), **cuda), _dl(wq, **cuda), _dl(s, **cuda), _dl(y, **cuda))
    assert rc == _lib.EINVAL and "2 dimensions" in msg


def test_packed_entry_point_argument_checks():
    L = _lib.lib()
    x, wq, s = _cpu_case()
    y = torch.empty((2, 16), dtype=torch.float16)
    views = [ops.to_dltensor(t) for t in (x, wq, s, y)]
    vals = (ctypes.c_void_p * 4)(*[ctypes.addressof(v.tensor) for v in views])
    codes = (ctypes.c_int * 4)(7, 7, 7, 7)
    out_code = ctypes.c_int(0)
    # wrong arity
    assert L.b200_q4f16_matmul_packed(vals, codes, 3, None, ctypes.byref(out_code), None) == -1
    assert "expected 4 arguments" in _lib.last_error()
    # a non-tensor type code
    bad = (ctypes.c_int * 4)(7, 0, 7, 7)
    assert L.b200_q4f16_matmul_packed(vals, bad, 4, None, ctypes.byref(out_code), None) == -1
    assert "type code" in _lib.last_error()
    # tensors on the CPU are refused with the reference's -1 convention
    assert L.b200_q4f16_matmul_packed(vals, codes, 4, None, ctypes.byref(out_code), None) == -1
    assert "not on a CUDA device" in _lib.last_error()


def test_raw_pointer_validation():
    L = _lib.lib()
    x, wq, s = _cpu_case()
    y = torch.empty((2, 16), dtype=torch.float16)
    assert L.b200_q4f16_matmul(x.data_ptr(), wq.data_ptr(), s.data_ptr(), y.data_ptr(), 2, 16, 40, None) == _lib.EINVAL
    assert L.b200_q4f16_matmul(x.data_ptr() + 2, wq.data_ptr(), s.data_ptr(), y.data_ptr(), 2, 16, 64, None) == _lib.EINVAL
    assert "aligned" in _lib.last_error()
    assert L.b200_q4f16_gemv(x.data_ptr(), wq.data_ptr(), s.data_ptr(), y.data_ptr(), 17, 16, 64, None) == _lib.EINVAL
    assert L.b200_q4f16_matmul(None, wq.data_ptr(), s.data_ptr(), y.data_ptr(), 2, 16, 64, None) == _lib.EINVAL
    assert L.b200_q4f16_dequantize(wq.data_ptr(), s.data_ptr(), None, 16, 64, None) == _lib.EINVAL


def test_options_roundtrip():
    relax_b200.set_option("gemv.warps", 4)
    assert relax_b200.get_option("gemv.warps") == 4
    relax_b200.set_option("gemv.warps", 0)
    with pytest.raises(relax_b200.B200Error):
        relax_b200.set_option("no.such.option", 1)


def test_weight_file_format_cpu(tmp_path):
    """The on-disk container of packed weights: round trip, alignment of the payload, and the errors of a
    damaged file (host logic only)."""
    import numpy as np

    from relax_b200 import synth, weights_io

    _, wq, s = synth.make_case(1, 24, 320, seed=3)
    p = str(tmp_path / "w.b2q4")
    weights_io.save(p, {"m": (wq, s), "empty": (np.zeros((0, 4), np.uint32), np.zeros((0, 1), np.float16))}, "paired")
    layout, t = weights_io.load(p)
    assert layout == "paired" and (t["m"][0] == wq).all() and (t["m"][1].view(np.uint16) == s.view(np.uint16)).all()
    assert t["empty"][0].shape == (0, 4)
    raw = open(p, "rb").read()
    hlen = int.from_bytes(raw[12:16], "little")
    assert (16 + hlen) % 64 == 0
    import pytest

    with pytest.raises(ValueError):
        weights_io.save(p, {"m": (wq, s[:, :5])})
    with pytest.raises(ValueError):
        weights_io.save(p, {"m": (wq, s)}, "swizzled")
    bad = str(tmp_path / "bad.b2q4")
    open(bad, "wb").write(b"NOTAFILE" + raw[8:])
    with pytest.raises(weights_io.FormatError):
        weights_io.load(bad)
    open(bad, "wb").write(raw[:8] + (9).to_bytes(4, "little") + raw[12:])
    with pytest.raises(weights_io.FormatError):
        weights_io.load(bad)
    open(bad, "wb").write(raw[:-100])
    with pytest.raises(weights_io.FormatError):
        weights_io.load(bad)


def test_argument_checks_of_the_newer_entry_points_need_no_gpu():
    """Validation comes before any device call: bad arguments give B200_EINVAL with a message on a box without a
    GPU; well-formed calls then fail with B200_ENODEVICE there (never a silent success)."""
    import ctypes

    import torch

    L = _lib.lib()
    buf = torch.zeros(4096, dtype=torch.int32)
    p = buf.data_ptr()
    no_gpu = not torch.cuda.is_available()
    # offline repack
    assert L.b200_q4f16_repack(p, p, 2, 256, 7, None) == _lib.EINVAL and "layout" in _lib.last_error()
    assert L.b200_q4f16_repack(p, p, 2, 40, 1, None) == _lib.EINVAL
    assert L.b200_q4f16_unpack(p, p + 16, 2, 256, 1, None) == _lib.EINVAL and "overlap" in _lib.last_error()
    assert L.b200_q4f16_matmul_layout(p, p, p, p, 1, 2, 256, 9, None) == _lib.EINVAL
    assert L.b200_set_option(b"weights.layout", 2) == _lib.EINVAL
    assert L.b200_set_option(b"gemv.exact", 3) == _lib.EINVAL
    if no_gpu:
        assert L.b200_q4f16_repack(p, p, 2, 256, 1, None) == _lib.ENODEVICE
    # output projection
    assert L.b200_lm_head(p, p, p, None, None, 17, 4, 32, 0, None) == _lib.EINVAL and "16 rows" in _lib.last_error()
    assert L.b200_lm_head(p, p, p, None, None, 1, 4, 48, 0, None) == _lib.EINVAL
    assert L.b200_lm_head(p, p, None, p, None, 1, 4, 32, 0, None) == _lib.EINVAL and "scratch" in _lib.last_error()
    if no_gpu:
        assert L.b200_lm_head(p, p, p, None, None, 1, 4, 32, 0, None) == _lib.ENODEVICE
        assert L.b200_lm_head_scratch_bytes() == -1
    # sum over ranks as its own kernel
    d = _lib.PeerReduce()
    assert L.b200_allreduce_peer(12, ctypes.byref(d), None) == _lib.EINVAL and "multiple of 8" in _lib.last_error()
    assert L.b200_allreduce_peer(16, None, None) == _lib.EINVAL
    d.world, d.rank = 1, 0
    assert L.b200_allreduce_peer(16, ctypes.byref(d), None) == _lib.EINVAL and "world" in _lib.last_error()
    d.world, d.rank = 2, 0
    assert L.b200_allreduce_peer(16, ctypes.byref(d), None) == _lib.EINVAL      # no epoch / out / peers
    d.epoch, d.out = p, p
    d.peer_y[0], d.peer_flags[0] = p, p
    assert L.b200_allreduce_peer(16, ctypes.byref(d), None) == _lib.EINVAL and "peer 1" in _lib.last_error()
    # qkv matmul with the rotary epilogue
    args = [p, None, p, None, 1e-5, p, p, p, p, p, p, p, p]
    assert L.b200_q4f16_gemv_rmsnorm_rope(*args, 0, 256, None) == _lib.EINVAL and "heads" in _lib.last_error()
    assert L.b200_q4f16_gemv_rmsnorm_rope(*args, 2, 200, None) == _lib.EINVAL
    assert L.b200_q4f16_gemv_rmsnorm_rope(*(args[:7] + [None] + args[8:]), 2, 256, None) == _lib.EINVAL
    if no_gpu:
        assert L.b200_q4f16_gemv_rmsnorm_rope(*args, 2, 256, None) == _lib.ENODEVICE
