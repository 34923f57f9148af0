"""Generates tests/golden/q4f16_relax_vm.npz.

The reference (tlc-pack/relax, early 2023) cannot be built or imported in this
environment (no LLVM, empty submodules), and it ships no vectors for int4 decode.  The
closest executable relative is the TVM 0.23 Relax VM that the ``tilelang`` wheel bundles:
the same lineage with renamed entry points (``relax.build`` for ``relax.vm.build``,
``R.call_dps_packed`` for ``R.call_tir("symbol")``).  This script builds the module a user
of the reference would write for a q4f16 linear layer -- a TE ``decode`` stage feeding a
fp32-accumulating ``matmul`` and a cast to fp16, emitted with ``BlockBuilder.emit_te`` --
compiles it for the CPU with target "c" (the wheel has no LLVM either) and records
inputs and outputs.  The vectors pin the oracle's nibble order, zero point, single fp16
rounding of the decode, accumulation order and final rounding against code that is NOT
ours.  They do not pin it against the reference proper, which stays "parity unpinned".

Run from the repository root:  python tests/golden/make_golden.py
"""
from __future__ import annotations

import os
import sys
import tempfile

import numpy as np


def _import_tvm():
    import tilelang  # noqa: F401  (puts its bundled TVM 0.23 on sys.path)
    import tvm

    return tvm


def build_vm(M: int, N: int, K: int):
    tvm = _import_tvm()
    from tvm import relax, te

    def q4f16_linear(x, wq, s):
        w = te.compute(
            (N, K),
            lambda n, k: (
                (((wq[n, k // 8] >> (k % 8 * 4).astype("uint32")) & tvm.tir.const(0xF, "uint32")).astype("int32") - 7)
            ).astype("float16")
            * s[n, k // 32],
            name="decode",
        )
        kk = te.reduce_axis((0, K), name="k")
        acc = te.compute(
            (M, N),
            lambda m, n: te.sum(x[m, kk].astype("float32") * w[n, kk].astype("float32"), axis=kk),
            name="matmul",
        )
        return te.compute((M, N), lambda m, n: acc[m, n].astype("float16"), name="cast")

    bb = relax.BlockBuilder()
    x = relax.Var("x", relax.TensorStructInfo((M, K), "float16"))
    wq = relax.Var("wq", relax.TensorStructInfo((N, K // 8), "uint32"))
    s = relax.Var("s", relax.TensorStructInfo((N, K // 32), "float16"))
    with bb.function("main", [x, wq, s]):
        with bb.dataflow():
            y = bb.emit_te(q4f16_linear, x, wq, s)
            out = bb.emit_output(y)
        bb.emit_func_output(out)
    mod = bb.get()
    ex = relax.build(mod, target="c")
    tmp = tempfile.mkdtemp()
    path = os.path.join(tmp, "q4.so")
    ex.export_library(path, options=["-Dhalf=_Float16", "-O2", "-ffp-contract=off"])
    lib = tvm.runtime.load_module(path)
    return relax.VirtualMachine(lib, tvm.cpu())


def build_decode_vm(N: int, K: int):
    """The decode stage alone, so its fp16 output is recorded bit for bit."""
    tvm = _import_tvm()
    from tvm import relax, te

    def decode(wq, s):
        return te.compute(
            (N, K),
            lambda n, k: (
                (((wq[n, k // 8] >> (k % 8 * 4).astype("uint32")) & tvm.tir.const(0xF, "uint32")).astype("int32") - 7)
            ).astype("float16")
            * s[n, k // 32],
            name="decode",
        )

    bb = relax.BlockBuilder()
    wq = relax.Var("wq", relax.TensorStructInfo((N, K // 8), "uint32"))
    s = relax.Var("s", relax.TensorStructInfo((N, K // 32), "float16"))
    with bb.function("main", [wq, s]):
        with bb.dataflow():
            out = bb.emit_output(bb.emit_te(decode, wq, s))
        bb.emit_func_output(out)
    ex = relax.build(bb.get(), target="c")
    path = os.path.join(tempfile.mkdtemp(), "dec.so")
    ex.export_library(path, options=["-Dhalf=_Float16", "-O2", "-ffp-contract=off"])
    return relax.VirtualMachine(tvm.runtime.load_module(path), tvm.cpu())


def pack(q):
    n, k = q.shape
    q = q.astype(np.uint32).reshape(n, k // 8, 8)
    out = np.zeros((n, k // 8), dtype=np.uint32)
    for j in range(8):
        out |= q[:, :, j] << np.uint32(4 * j)
    return out


def cases():
    rng = np.random.default_rng(20230301)
    out = []
    for name, (M, N, K) in {
        "rand_m1": (1, 64, 128),
        "rand_m3": (3, 48, 256),
        "rand_m16": (16, 32, 64),
        "rand_k32": (2, 16, 32),
    }.items():
        q = rng.integers(0, 16, (N, K), dtype=np.uint8)
        s = rng.uniform(0.005, 0.02, (N, K // 32)).astype(np.float16)
        x = rng.standard_normal((M, K)).astype(np.float16)
        out.append((name, x, pack(q), s))
    # known-answer style edge cases
    M, N, K = 2, 16, 64
    x = rng.standard_normal((M, K)).astype(np.float16)
    s = rng.uniform(0.005, 0.02, (N, K // 32)).astype(np.float16)
    out.append(("all_zero_nibbles", x, np.zeros((N, K // 8), np.uint32), s))
    out.append(("all_f_nibbles", x, np.full((N, K // 8), 0xFFFFFFFF, np.uint32), s))
    ramp = np.tile(np.arange(16, dtype=np.uint8), (N, K // 16))
    out.append(("nibble_ramp", x, pack(ramp), s))
    onehot = np.zeros((M, K), np.float16)
    onehot[0, 5] = 1.0
    onehot[1, K - 1] = -2.0
    out.append(("one_hot_x", onehot, pack(rng.integers(0, 16, (N, K), dtype=np.uint8)), s))
    # scales at the edges of fp16: smallest subnormal, largest subnormal, smallest normal, large, odd significands
    edge = np.array([0x0001, 0x03FF, 0x0400, 0x7BFF // 16, 0x3C01, 0x2E67, 0x1234, 0x0201], dtype=np.uint16).view(np.float16)
    s_edge = np.resize(edge, (N, K // 32)).astype(np.float16)
    out.append(("edge_scales", x, pack(rng.integers(0, 16, (N, K), dtype=np.uint8)), s_edge))
    return out


def main():
    tvm = _import_tvm()

    vms = {}
    dvms = {}
    blob = {}
    for name, x, wq, s in cases():
        M, K = x.shape
        N = wq.shape[0]
        key = (M, N, K)
        if key not in vms:
            vms[key] = build_vm(M, N, K)
        y = vms[key]["main"](tvm.runtime.tensor(x), tvm.runtime.tensor(wq), tvm.runtime.tensor(s)).numpy()
        if (N, K) not in dvms:
            dvms[(N, K)] = build_decode_vm(N, K)
        w = dvms[(N, K)]["main"](tvm.runtime.tensor(wq), tvm.runtime.tensor(s)).numpy()
        blob[name + ".w"] = w.view(np.uint16)
        blob[name + ".x"] = x.view(np.uint16)
        blob[name + ".wq"] = wq
        blob[name + ".s"] = s.view(np.uint16)
        blob[name + ".y"] = y.view(np.uint16)
        print(name, (M, N, K), "y[0,:4] =", y[0, :4])
    here = os.path.dirname(os.path.abspath(__file__))
    np.savez_compressed(os.path.join(here, "q4f16_relax_vm.npz"), **blob)
    print("wrote", os.path.join(here, "q4f16_relax_vm.npz"))


if __name__ == "__main__":
    sys.exit(main())
