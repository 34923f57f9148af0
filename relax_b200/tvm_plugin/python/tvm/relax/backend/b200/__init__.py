"""Pattern table and partition helper of the B200 q4f16 backend, for the reference tree
(python/tvm/relax/backend/b200/__init__.py; mirrors python/tvm/contrib/cutlass/build.py and the
pattern helpers of python/tvm/relax/dpl/pattern.py:804-860,1049-1095).

    mod = partition_for_b200(mod)            # FuseOpsByPattern(annotate_codegen=True) + RunCodegen
    ex = relax.vm.build(mod, "cuda")         # the offloaded calls become call_tir(ExternFunc(symbol))

Patterns can only name a decode PrimFunc, and FuseOpsByPattern has no check callback in this tree, so
what the PrimFunc computes is established here, before its name enters the table: it must be
structurally equal to the canonical TE decode (zero point 7, low nibble first, one fp16 scale per 32
elements of K).  The result travels to the C++ codegen in the option map ("decode_layouts").
"""
import tvm
from tvm import relax, te, tir
from tvm.relax.dpl.pattern import is_call_tir, is_op, wildcard

COMPOSITE_NAME = "b200.q4f16_matmul"


def canonical_decode_te(N, K, layout="nk", spelling=0):
    """f(wq, scales) -> te.Tensor: w[n,k] = fp16(((wq[n,k//8] >> 4*(k%8)) & 15) - 7) * scales[n,k//32],
    emitted as [N,K] ("nk") or [K,N] ("kn").  spelling 1 subtracts in fp16 instead of int32 (same values)."""

    def value(wq, s, n, k):
        q = (wq[n, k // 8] >> (k % 8 * 4).astype("uint32")) & tir.const(0xF, "uint32")
        centred = (q.astype("int32") - 7).astype("float16") if spelling == 0 else q.astype("float16") - tir.const(7, "float16")
        return centred * s[n, k // 32]

    def decode(wq, s):
        if layout == "nk":
            return te.compute((N, K), lambda n, k: value(wq, s, n, k), name="decode")
        return te.compute((K, N), lambda k, n: value(wq, s, n, k), name="decode")

    return decode


def _canonical_primfunc(N, K, layout, spelling):
    bb = relax.BlockBuilder()
    wq = relax.Var("wq", relax.TensorStructInfo((N, K // 8), "uint32"))
    s = relax.Var("s", relax.TensorStructInfo((N, K // 32), "float16"))
    with bb.function("f", [wq, s]):
        bb.emit_func_output(bb.emit_te(canonical_decode_te(N, K, layout, spelling), wq, s, primfunc_name_hint="decode"))
    for _, f in bb.get().functions.items():
        if isinstance(f, tir.PrimFunc):
            return f.without_attr("global_symbol")
    raise RuntimeError("emit_te produced no PrimFunc")


def classify_decode(func):
    """"nk" / "kn" when the PrimFunc is this scheme's decode, else None."""
    if not isinstance(func, tir.PrimFunc) or len(func.params) != 3:
        return None
    bufs = [func.buffer_map.get(p) for p in func.params]
    if any(b is None for b in bufs) or any(len(b.shape) != 2 for b in bufs):
        return None
    if [str(b.dtype) for b in bufs] != ["uint32", "float16", "float16"]:
        return None
    if not all(isinstance(d, tir.IntImm) for b in bufs for d in b.shape):
        return None
    wq, s, w = ([int(d) for d in b.shape] for b in bufs)
    N, K = wq[0], wq[1] * 8
    if K % 32 or s != [N, K // 32]:
        return None
    plain = func.without_attr("global_symbol")
    for layout, shape in (("nk", [N, K]), ("kn", [K, N])):
        if w != shape:
            continue
        for spelling in (0, 1):
            if tvm.ir.structural_equal(plain, _canonical_primfunc(N, K, layout, spelling)):
                return layout
    return None


def decode_layouts(mod):
    out = {}
    for gv, f in mod.functions.items():
        layout = classify_decode(f)
        if layout is not None:
            out[gv.name_hint] = layout
    return out


def q4f16_matmul_patterns(decodes):
    """(name, pattern) pairs, one per validated decode {name: layout}:
    astype(matmul(x, permute_dims(call_tir(<decode [N,K]>))))  or  astype(matmul(x, call_tir(<decode [K,N]>)))."""
    pats = []
    for name in sorted(decodes):
        w = is_call_tir(name, [wildcard(), wildcard()])
        if decodes[name] == "nk":
            w = is_op("relax.permute_dims")(w)
        pats.append((COMPOSITE_NAME, is_op("relax.astype")(is_op("relax.matmul")(wildcard(), w))))
    return pats


def partition_for_b200(mod, options=None, merge=False):
    """Offloads every q4f16 decode->matmul->astype group to relax.ext.b200.  options: {"family":
    "auto"|"gemv"|"gemm", "weight_layout": "reference"|"paired"}.  merge=True runs MergeCompositeFunctions so that chained matmuls share one
    offloaded function."""
    found = decode_layouts(mod)
    if not found:
        return mod
    pats = q4f16_matmul_patterns(found)
    if merge:
        mod = relax.transform.FuseOpsByPattern(pats, annotate_codegen=False)(mod)
        mod = relax.transform.MergeCompositeFunctions()(mod)
    else:
        mod = relax.transform.FuseOpsByPattern(pats, annotate_codegen=True)(mod)
    opts = dict(options or {})
    opts["decode_layouts"] = found
    return relax.transform.RunCodegen({"b200": opts})(mod)
