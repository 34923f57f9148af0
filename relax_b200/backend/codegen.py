"""The ``relax.ext.b200`` codegen and the partition helper.

Calling convention (src/relax/transform/run_codegen.cc:158-163 in the reference):
    codegen(functions: Array<Function>, options: Map, constant_names: Map) -> Array<runtime.Module>
Every function has attrs Codegen="b200" and global_symbol=<symbol>; its body calls one local
function with Composite="b200.q4f16_matmul".  RunCodegen rewrites each call site to a
destination-passing extern call of <symbol> with the function's OWN parameter order, which is
first-use order inside the group, e.g. (wq, scales, x) -- so the roles are recovered by walking the
composite body, never by position.

Instead of emitting C source (the reference-tree codegen in relax_b200/tvm_plugin does that), this
Python codegen binds <symbol> in the FFI's global registry to a closure that reorders the arguments
and calls the kernel library; the VM resolves extern symbols through that registry after the
executable's own imports (src/runtime/relax_vm/vm.cc:700-725).  It returns no modules.
"""
from __future__ import annotations

from dataclasses import dataclass

from .patterns import COMPOSITE_NAME, decode_func_names, q4f16_matmul_patterns
from .tvm_bridge import import_tvm


class B200CodegenError(ValueError):
    """The matched group is not something the kernels compute; nothing is offloaded silently."""


@dataclass
class Q4Roles:
    symbol: str
    x: int          # positions in the offloaded function's parameter list
    wq: int
    scales: int
    M: int
    N: int
    K: int
    transposed: bool


def _static_shape(sinfo, what):
    tvm = import_tvm()
    if not isinstance(sinfo, tvm.relax.TensorStructInfo) or sinfo.shape is None:
        raise B200CodegenError(f"b200: {what} must be a tensor with a static shape")
    dims = []
    for d in sinfo.shape.values:
        if not isinstance(d, tvm.tir.IntImm):
            raise B200CodegenError(f"b200: {what} has a symbolic dimension {d}")
        dims.append(int(d))
    return dims, str(sinfo.dtype)


def analyze_composite(func) -> Q4Roles:
    """Maps the parameters of an offloaded function to (x, wq, scales) and validates the group."""
    tvm = import_tvm()
    relax = tvm.relax
    symbol = str(func.attrs["global_symbol"])
    # the outer body: one binding  gv = local_func(args...)  where local_func is a nested Function
    inner, call_args = None, None
    bindings = {}
    for blk in func.body.blocks:
        for b in blk.bindings:
            bindings[b.var] = b.value
    for var, val in bindings.items():
        if isinstance(val, relax.Function):
            if str(val.attrs.get("Composite", "")) != COMPOSITE_NAME:
                raise B200CodegenError(f"b200: unsupported composite {val.attrs.get('Composite')}")
            inner = (var, val)
    if inner is None:
        raise B200CodegenError(f"b200: {symbol} holds no composite function")
    for var, val in bindings.items():
        if isinstance(val, relax.Call) and val.op.same_as(inner[0]):
            call_args = list(val.args)
    if call_args is None:
        raise B200CodegenError(f"b200: the composite function of {symbol} is never called")
    comp = inner[1]
    outer_pos = {p: i for i, p in enumerate(func.params)}
    inner_to_outer = {}
    for p, a in zip(comp.params, call_args):
        if a not in outer_pos:
            raise B200CodegenError("b200: composite arguments must be parameters of the offloaded function")
        inner_to_outer[p] = outer_pos[a]

    cb = {}
    for blk in comp.body.blocks:
        for b in blk.bindings:
            cb[b.var] = b.value

    def resolve(e):
        return cb.get(e, e) if isinstance(e, relax.Var) else e

    def is_op(e, name):
        return isinstance(e, relax.Call) and isinstance(e.op, tvm.ir.Op) and e.op.name == name

    matmuls = [v for v in cb.values() if is_op(v, "relax.matmul")]
    casts = [v for v in cb.values() if is_op(v, "relax.astype")]
    if len(matmuls) != 1 or len(casts) != 1:
        raise B200CodegenError("b200: the group must hold exactly one matmul and one astype")
    mm, cast = matmuls[0], casts[0]
    if str(mm.attrs.out_dtype) != "float32":
        raise B200CodegenError('b200: the matmul must accumulate in float32 (out_dtype="float32")')
    if str(cast.attrs.dtype) != "float16":
        raise B200CodegenError("b200: the result must be cast to float16")
    x_param = mm.args[0]
    if x_param not in inner_to_outer:
        raise B200CodegenError("b200: the activation must be a parameter of the group")
    w = resolve(mm.args[1])
    transposed = False
    if is_op(w, "relax.permute_dims"):
        transposed = True
        w = resolve(w.args[0])
    if not is_op(w, "relax.call_tir"):
        raise B200CodegenError("b200: the weight operand must come from call_tir(decode, (wq, scales))")
    targs = list(w.args[1].fields)
    if len(targs) != 2 or any(a not in inner_to_outer for a in targs):
        raise B200CodegenError("b200: decode takes the two parameters (wq, scales)")
    (xs, xd) = _static_shape(x_param.struct_info, "x")
    (ws, wd) = _static_shape(targs[0].struct_info, "wq")
    (ss, sd) = _static_shape(targs[1].struct_info, "scales")
    (dw, dd) = _static_shape(w.struct_info, "decoded weight")
    if (xd, wd, sd, dd) != ("float16", "uint32", "float16", "float16"):
        raise B200CodegenError(f"b200: dtypes must be x f16, wq u32, scales f16, w f16; got {xd},{wd},{sd},{dd}")
    if len(xs) != 2 or len(ws) != 2 or len(ss) != 2:
        raise B200CodegenError("b200: x, wq and scales must be 2-D")
    M, K = xs
    N = ws[0]
    if K % 32 != 0 or ws[1] * 8 != K or ss != [N, K // 32]:
        raise B200CodegenError(f"b200: need wq [N,K/8] and scales [N,K/32] with K % 32 == 0; got x{xs} wq{ws} s{ss}")
    want_w = [N, K]
    if dw != want_w:
        raise B200CodegenError(f"b200: decode must produce [N,K]={want_w}, got {dw}")
    if not transposed and N != K:
        raise B200CodegenError("b200: matmul(x, w) without a transpose needs w as [K,N]; decode emits [N,K]")
    return Q4Roles(symbol, inner_to_outer[x_param], inner_to_outer[targs[0]], inner_to_outer[targs[1]], M, N, K,
                   transposed)


COMPILED: dict = {}   # symbol -> Q4Roles of everything this process has offloaded


def b200_codegen(functions, options, constant_names):
    """relax.ext.b200: validates each offloaded function and binds its symbol to the kernel."""
    import tvm_ffi

    from .. import registry

    matmul = registry.get_global_func("b200.q4f16_matmul")
    for func in functions:
        roles = analyze_composite(func)
        COMPILED[roles.symbol] = roles

        def packed(*args, _r=roles):
            if len(args) != 4:
                raise TypeError(f"{_r.symbol}: expected 3 inputs and 1 output, got {len(args)} arguments")
            matmul(args[_r.x], args[_r.wq], args[_r.scales], args[3])

        tvm_ffi.register_global_func(roles.symbol, packed, override=True)
    return []


def register_codegen():
    import_tvm()
    import tvm_ffi

    tvm_ffi.register_global_func("relax.ext.b200", b200_codegen, override=True)


def partition_for_b200(mod, options=None, decode_names=None):
    """FuseOpsByPattern(patterns, annotate_codegen=True) followed by RunCodegen({"b200": options}).
    Mirrors the offload recipe of the reference's tests
    (tests/python/relax/test_codegen_cutlass.py:223-240)."""
    tvm = import_tvm()
    register_codegen()
    names = tuple(decode_names) if decode_names else decode_func_names(mod)
    pats = q4f16_matmul_patterns(names or ("decode",))
    mod = tvm.relax.transform.FuseOpsByPattern(pats, annotate_codegen=True)(mod)
    return tvm.relax.transform.RunCodegen({"b200": options or {}})(mod)
