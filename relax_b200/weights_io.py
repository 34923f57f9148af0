"""On-disk container for q4f16 weights (one file per model shard) and the offline repack.

The reference keeps an executable's weights as constants bound at build time and serialises them with the
module (python/tvm/relax/vm.py:620-629 in its tree passes ``const_name_to_constant`` to the external
modules; python/tvm/runtime/ndarray.py's ``save_param_dict`` is its stand-alone parameter file).  This is
the counterpart for this path: a flat file holding, per matrix, the packed words and the scales together
with the nibble layout they are stored in, so that a deployment can repack ONCE offline
(:func:`repack_file`) and every later load hands the kernels the order they prefer.

File layout (little endian):

    bytes 0..7    magic  b"B2Q4F16\\0"
    bytes 8..11   uint32 format version (1)
    bytes 12..15  uint32 length L of the JSON header
    bytes 16..    JSON header (UTF-8), padded with spaces to a multiple of 64 bytes:
                  {"layout": "reference" | "paired", "group": 32, "zero_point": 7,
                   "tensors": [{"name", "N", "K", "wq_offset", "wq_bytes", "scales_offset", "scales_bytes"}, ...]}
    then          the arrays, each at its 64-byte aligned offset counted from the end of the header:
                  wq uint32 [N, K/8] row-major, scales fp16 [N, K/32] row-major.

Reading and writing are plain numpy on the host; the repack of a loaded file runs on the GPU through the
library (:func:`relax_b200.ops.q4f16_repack`), there is no CPU fallback for it.
"""
from __future__ import annotations

import json
import struct

import numpy as np

MAGIC = b"B2Q4F16\0"
VERSION = 1
LAYOUT_NAMES = ("reference", "paired")


class FormatError(ValueError):
    """The file is not a q4f16 weight container, or its header and payload disagree."""


def _align(n: int, a: int = 64) -> int:
    return (n + a - 1) // a * a


def save(path: str, tensors: dict, layout: str = "reference") -> None:
    """``tensors``: name -> (wq uint32 [N,K/8], scales fp16 [N,K/32]) as numpy arrays, all in ``layout``."""
    if layout not in LAYOUT_NAMES:
        raise ValueError(f"unknown layout {layout!r}")
    entries, blobs, off = [], [], 0
    for name, (wq, scales) in tensors.items():
        wq = np.ascontiguousarray(wq)
        scales = np.ascontiguousarray(scales)
        if wq.dtype not in (np.uint32, np.int32) or wq.ndim != 2:
            raise ValueError(f"{name}: packed weights must be 32-bit integers [N, K/8]")
        if scales.dtype != np.float16 or scales.ndim != 2:
            raise ValueError(f"{name}: scales must be fp16 [N, K/32]")
        N, K = wq.shape[0], wq.shape[1] * 8
        if K % 32 or scales.shape != (N, K // 32):
            raise ValueError(f"{name}: shapes {wq.shape} / {scales.shape} are not [N,K/8] / [N,K/32] with K % 32 == 0")
        e = {"name": name, "N": N, "K": K}
        for key, arr in (("wq", wq.view(np.uint32)), ("scales", scales)):
            e[key + "_offset"], e[key + "_bytes"] = off, arr.nbytes
            blobs.append((off, arr))
            off = _align(off + arr.nbytes)
        entries.append(e)
    header = json.dumps({"layout": layout, "group": 32, "zero_point": 7, "tensors": entries}).encode()
    header += b" " * (_align(16 + len(header)) - 16 - len(header))
    with open(path, "wb") as f:
        f.write(MAGIC + struct.pack("<II", VERSION, len(header)) + header)
        base = f.tell()
        for o, arr in blobs:
            f.seek(base + o)
            f.write(arr.tobytes())
        f.truncate(base + off)


def load(path: str):
    """Returns (layout, {name: (wq uint32 [N,K/8], scales fp16 [N,K/32])}); raises FormatError on a bad file."""
    with open(path, "rb") as f:
        head = f.read(16)
        if len(head) < 16 or head[:8] != MAGIC:
            raise FormatError(f"{path}: not a q4f16 weight file")
        version, hlen = struct.unpack("<II", head[8:])
        if version != VERSION:
            raise FormatError(f"{path}: format version {version}, this reader knows {VERSION}")
        try:
            meta = json.loads(f.read(hlen).decode())
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise FormatError(f"{path}: unreadable header: {e}") from None
        if meta.get("layout") not in LAYOUT_NAMES or meta.get("group") != 32 or meta.get("zero_point") != 7:
            raise FormatError(f"{path}: unsupported layout/group/zero point in header")
        payload = f.read()
    out = {}
    for e in meta["tensors"]:
        N, K = int(e["N"]), int(e["K"])
        if K % 32 or e["wq_bytes"] != N * K // 2 or e["scales_bytes"] != N * (K // 32) * 2:
            raise FormatError(f"{path}: tensor {e['name']!r}: sizes do not match N={N} K={K}")
        if e["wq_offset"] + e["wq_bytes"] > len(payload) or e["scales_offset"] + e["scales_bytes"] > len(payload):
            raise FormatError(f"{path}: tensor {e['name']!r} runs past the end of the file")
        wq = np.frombuffer(payload, np.uint32, N * K // 8, e["wq_offset"]).reshape(N, K // 8)
        sc = np.frombuffer(payload, np.float16, N * (K // 32), e["scales_offset"]).reshape(N, K // 32)
        out[e["name"]] = (wq, sc)
    return meta["layout"], out


def repack_file(src: str, dst: str, layout: str = "paired", device="cuda") -> None:
    """Offline repack: reads ``src`` (any layout), writes ``dst`` in ``layout``.  The permutation runs on the GPU."""
    import torch

    from . import ops

    have, tensors = load(src)
    out = {}
    for name, (wq, sc) in tensors.items():
        t = torch.from_numpy(wq.view(np.int32).copy()).to(device)
        if have != "reference":
            ops.q4f16_unpack(t, have, out=t)
        if layout != "reference":
            ops.q4f16_repack(t, layout, out=t)
        out[name] = (t.cpu().numpy().view(np.uint32), sc)
    save(dst, out, layout)
