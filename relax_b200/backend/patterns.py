"""Pattern table of the b200 backend: (name, DFPattern) pairs for FuseOpsByPattern.

The q4f16 linear layer a user of the reference writes is
    w   = call_tir(decode, (wq, scales))                       # TE/TIR decode stage, kInjective
    acc = relax.matmul(x, permute_dims(w), out_dtype="float32")   # decode emits [N, K]
    y   = relax.astype(acc, "float16")
or, with a decode stage that emits the transposed layout [K, N] directly, the same without the
``permute_dims``.  Plain FuseOps keeps decode and matmul apart (the injective rule needs an
injective sink, src/relay/analysis/graph_partitioner.cc:317-325), so the group is formed by pattern.

Patterns can only name the decode PrimFunc (GlobalVarPattern matches by exact name,
src/relax/ir/dataflow_matcher.cc:490-495) and FuseOpsByPattern takes no check callback in the
reference snapshot, so WHAT the PrimFunc computes has to be established before its name goes into
the table: :func:`decode_layouts` compares every candidate PrimFunc structurally with the canonical
TE decode of this quantisation scheme (zero point 7, low nibble first, one fp16 scale per 32
elements of K).  A decode with another zero point, nibble order, scale layout or dtype keeps the
same tensor signature but is not equal, is left out of the table and stays on the reference's own
lowering.
"""
from __future__ import annotations

from .tvm_bridge import import_tvm

COMPOSITE_NAME = "b200.q4f16_matmul"

LAYOUT_NK = "nk"   # decode emits w[N, K]; the matmul takes permute_dims(w)
LAYOUT_KN = "kn"   # decode emits w[K, N]; the matmul takes it as it is


def canonical_decode_te(N: int, K: int, layout: str = LAYOUT_NK, spelling: int = 0):
    """The TE compute a user of the reference writes for this scheme; returns ``f(wq, scales)``.

    ``spelling`` selects between equivalent ways of writing the same arithmetic that have different
    expression trees (both exact: q and q-7 are representable in int32 and in fp16):
      0:  fp16(int32(q) - 7) * s          1:  (fp16(q) - fp16(7)) * s
    """
    tvm = import_tvm()
    from tvm import te

    def value(wq, s, n, k):
        q = (wq[n, k // 8] >> (k % 8 * 4).astype("uint32")) & tvm.tir.const(0xF, "uint32")
        if spelling == 0:
            centred = (q.astype("int32") - 7).astype("float16")
        else:
            centred = q.astype("float16") - tvm.tir.const(7, "float16")
        return centred * s[n, k // 32]

    def decode(wq, s):
        if layout == LAYOUT_NK:
            return te.compute((N, K), lambda n, k: value(wq, s, n, k), name="decode")
        return te.compute((K, N), lambda k, n: value(wq, s, n, k), name="decode")

    return decode


def _canonical_primfunc(N, K, layout, spelling):
    """PrimFunc of the canonical decode, produced the way BlockBuilder.emit_te produces a user's
    (python/tvm/relax/block_builder.py:385-464 -> te.create_prim_func)."""
    tvm = import_tvm()
    from tvm import relax

    bb = relax.BlockBuilder()
    wq = relax.Var("wq", relax.TensorStructInfo((N, K // 8), "uint32"))
    s = relax.Var("s", relax.TensorStructInfo((N, K // 32), "float16"))
    with bb.function("f", [wq, s]):
        out = bb.emit_te(canonical_decode_te(N, K, layout, spelling), wq, s, primfunc_name_hint="decode")
        bb.emit_func_output(out)
    mod = bb.get()
    for gv, f in mod.functions.items():
        if isinstance(f, tvm.tir.PrimFunc):
            return f
    raise RuntimeError("emit_te produced no PrimFunc")


def _buffer_dims(buf):
    tvm = import_tvm()
    dims = []
    for d in buf.shape:
        if not isinstance(d, tvm.tir.IntImm):
            return None
        dims.append(int(d))
    return dims


def classify_decode(func):
    """``LAYOUT_NK`` / ``LAYOUT_KN`` when `func` (a PrimFunc) IS this scheme's decode, else None."""
    tvm = import_tvm()
    if not isinstance(func, tvm.tir.PrimFunc) or len(func.params) != 3:
        return None
    bufs = [func.buffer_map.get(p) for p in func.params]
    if any(b is None for b in bufs):
        return None
    wq, s, w = (_buffer_dims(b) for b in bufs)
    if wq is None or s is None or w is None or len(wq) != 2 or len(s) != 2 or len(w) != 2:
        return None
    if (str(bufs[0].dtype), str(bufs[1].dtype), str(bufs[2].dtype)) != ("uint32", "float16", "float16"):
        return None
    N, K = wq[0], wq[1] * 8
    if K % 32 or s != [N, K // 32]:
        return None
    layouts = [l for l, shape in ((LAYOUT_NK, [N, K]), (LAYOUT_KN, [K, N])) if w == shape]
    plain = func.without_attr("global_symbol") if func.attrs and "global_symbol" in func.attrs else func
    for layout in layouts:
        for spelling in (0, 1):
            ref = _canonical_primfunc(N, K, layout, spelling)
            ref = ref.without_attr("global_symbol") if ref.attrs and "global_symbol" in ref.attrs else ref
            if tvm.ir.structural_equal(plain, ref):
                return layout
    return None


def decode_layouts(mod):
    """{name: layout} of the PrimFuncs in `mod` that are structurally this scheme's decode."""
    import_tvm()
    out = {}
    for gv, f in mod.functions.items():
        layout = classify_decode(f)
        if layout is not None:
            out[gv.name_hint] = layout
    return out


def q4f16_matmul_patterns(decodes=None):
    """Pattern table for decode PrimFuncs given as ``{name: layout}`` (from :func:`decode_layouts`)
    or as a sequence of names whose layout is [N, K].  One pattern per name: a [N, K] decode is
    matched only under ``permute_dims``, a [K, N] decode only without it -- the other combinations
    are a different product (x . w instead of x . w^T) and are never offloaded."""
    import_tvm()
    from tvm.relax.dpl import is_op, wildcard
    from tvm.relax.dpl.pattern import is_call_tir

    if decodes is None:
        decodes = {"decode": LAYOUT_NK}
    elif not isinstance(decodes, dict):
        decodes = {n: LAYOUT_NK for n in decodes}
    pats = []
    for name in sorted(decodes):
        w = is_call_tir(name, [wildcard(), wildcard()])
        if decodes[name] == LAYOUT_NK:
            w = is_op("relax.permute_dims")(w)
        mm = is_op("relax.matmul")(wildcard(), w)
        pats.append((COMPOSITE_NAME, is_op("relax.astype")(mm)))
    return pats
