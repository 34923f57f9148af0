"""Pattern table of the b200 backend: (name, DFPattern) pairs for FuseOpsByPattern.

The q4f16 linear layer a user of the reference writes is
    w   = call_tir(decode, (wq, scales))                       # TE/TIR decode stage, kInjective
    acc = relax.matmul(x, permute_dims(w) | w, out_dtype="float32")
    y   = relax.astype(acc, "float16")
Plain FuseOps keeps decode and matmul apart (the injective rule needs an injective sink,
src/relay/analysis/graph_partitioner.cc:317-325), so the group is formed by pattern.  Patterns can
only name the decode PrimFunc exactly (GlobalVarPattern, src/relax/ir/dataflow_matcher.cc:490-495):
the table takes the names to look for.
"""
from __future__ import annotations

from .tvm_bridge import import_tvm

COMPOSITE_NAME = "b200.q4f16_matmul"


def q4f16_matmul_patterns(decode_names=("decode",)):
    import_tvm()
    from tvm.relax.dpl import is_op, wildcard
    from tvm.relax.dpl.pattern import is_call_tir

    pats = []
    for dn in decode_names:
        for transposed in (True, False):
            w = is_call_tir(dn, [wildcard(), wildcard()])
            if transposed:
                w = is_op("relax.permute_dims")(w)
            mm = is_op("relax.matmul")(wildcard(), w)
            pats.append((COMPOSITE_NAME, is_op("relax.astype")(mm)))
    return pats


def decode_func_names(mod):
    """Names of PrimFuncs in `mod` whose name starts with "decode" (what emit_te calls them)."""
    import_tvm()
    from tvm import tir

    return tuple(sorted(gv.name_hint for gv, f in mod.functions.items()
                        if isinstance(f, tir.PrimFunc) and gv.name_hint.startswith("decode")))
