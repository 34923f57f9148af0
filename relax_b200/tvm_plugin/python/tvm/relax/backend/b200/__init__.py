"""Pattern table and partition helper of the B200 q4f16 backend, for the reference tree
(python/tvm/relax/backend/b200/__init__.py; mirrors python/tvm/contrib/cutlass/build.py and the
pattern helpers of python/tvm/relax/dpl/pattern.py:804-860,1049-1095).

    mod = partition_for_b200(mod)            # FuseOpsByPattern(annotate_codegen=True) + RunCodegen
    ex = relax.vm.build(mod, "cuda")         # the offloaded calls become call_tir(ExternFunc(symbol))
"""
from tvm import relax
from tvm.relax.dpl.pattern import is_call_tir, is_op, wildcard


def q4f16_matmul_patterns(decode_names=("decode", "decode1", "decode2", "decode3")):
    """(name, pattern) pairs: astype(matmul(x, [permute_dims](call_tir(<decode>, (wq, scales)))))."""
    pats = []
    for dn in decode_names:
        for transposed in (True, False):
            w = is_call_tir(dn, [wildcard(), wildcard()])
            if transposed:
                w = is_op("relax.permute_dims")(w)
            mm = is_op("relax.matmul")(wildcard(), w)
            pats.append(("b200.q4f16_matmul", is_op("relax.astype")(mm)))
    return pats


def partition_for_b200(mod, options=None, decode_names=None):
    """Offloads every q4f16 decode->matmul->astype group of `main` to relax.ext.b200."""
    pats = q4f16_matmul_patterns(decode_names) if decode_names else q4f16_matmul_patterns()
    mod = relax.transform.FuseOpsByPattern(pats, annotate_codegen=True)(mod)
    return relax.transform.RunCodegen({"b200": options or {}})(mod)
