"""The ``relax.ext.b200`` codegen and the partition helper.

Calling convention (src/relax/transform/run_codegen.cc:158-163 in the reference):
    codegen(functions: Array<Function>, options: Map, constant_names: Map) -> Array<runtime.Module>
Every function has attrs Codegen="b200" and global_symbol=<symbol>; its body binds local functions
with Composite="b200.q4f16_matmul" and calls them: one when the group comes from
FuseOpsByPattern(annotate_codegen=True), possibly a chain of several after MergeCompositeFunctions
(src/relax/transform/merge_composite_functions.cc:30-60).  RunCodegen rewrites each call site to a
destination-passing extern call of <symbol> with the function's OWN parameter order, which is
first-use order inside the group, e.g. (wq, scales, x) -- so the roles are recovered by walking the
composite bodies, never by position -- and stores the returned modules in the IRModule's
"external_mods" attribute (run_codegen.cc:53-55), from where the VM build links them
(python/tvm/relax/vm.py:620-629).

What is returned: one C-source module per offloaded function (``runtime.CSourceModuleCreate``,
src/target/source/source_module.cc:146, as the reference's CUTLASS codegen does through
src/relay/backend/contrib/codegen_c/codegen_c.h:163-235).  The generated wrapper contains no kernel:
it unpacks the tensors, maps them to (x, wq, scales, y) and forwards to the prebuilt kernel library's
``b200_q4f16_matmul_dl_family``; intermediates of a merged chain come from the runtime's workspace
pool (TVMBackendAllocWorkspace, include/tvm/runtime/c_backend_api.h:60-84).  The source is compiled
when the executable is exported (``export_library``), linked against ``libb200_q4f16.so``
(:func:`link_options`), and the result can be loaded back in another process
(:func:`finalize_modules` does export + load, the counterpart of ``finalize_modules_relax``,
python/tvm/contrib/cutlass/build.py:856-879).

The wrapper is written for the packed-function ABI of the importable runtime (tvm_ffi "safe call":
``int __tvm_ffi_<symbol>(void*, const TVMFFIAny*, int32_t, TVMFFIAny*)``); the codegen for the
reference tree itself, which emits the same forwarding for its ``TVMBackendPackedCFunc`` ABI, is
relax_b200/tvm_plugin/src/relax/backend/contrib/b200/codegen.cc.

Options (the map given to ``RunCodegen({"b200": {...}})``, run_codegen.cc:42,155):
    "family": "auto" (default) | "gemv" | "gemm"    kernel family the wrapper asks for
    "weight_layout": "reference" | "paired"          nibble order of the bound weights (the offline repack of
                                                     b200_q4f16_repack); absent = the library's option "weights.layout"
"""
from __future__ import annotations

import os
import tempfile
from dataclasses import dataclass, field

from . import patterns
from .patterns import COMPOSITE_NAME, LAYOUT_KN, LAYOUT_NK, decode_layouts, q4f16_matmul_patterns
from .tvm_bridge import import_tvm


class B200CodegenError(ValueError):
    """The matched group is not something the kernels compute; nothing is offloaded silently."""


FAMILIES = {"auto": 0, "gemv": 1, "gemm": 2}
# code added to the family argument of b200_q4f16_matmul_dl_family (bits 8-15 = layout + 1, B200_FAMILY_WITH_LAYOUT)
WEIGHT_LAYOUTS = {"reference": (0 + 1) << 8, "paired": (1 + 1) << 8}

# decode PrimFuncs whose body has been compared with the canonical decode: name -> layout.
# Filled by partition_for_b200 / validate_decodes; the codegen refuses call_tir to any other name.
VALIDATED_DECODES: dict = {}


@dataclass
class Q4Step:
    """One q4f16 matmul of an offloaded function.  Tensor sources are ("param", i) -- the i-th
    parameter of the offloaded function -- or ("tmp", j), the result of step j."""
    x: tuple
    wq: int
    scales: int
    M: object          # int, or None when the batch dimension is symbolic (read from x at run time)
    N: int
    K: int
    layout: str


@dataclass
class Q4Plan:
    symbol: str
    num_params: int
    steps: list = field(default_factory=list)
    family: int = 0

    # single-matmul view kept for callers that only handle the unmerged case
    @property
    def x(self):
        return self.steps[0].x[1]

    @property
    def wq(self):
        return self.steps[0].wq

    @property
    def scales(self):
        return self.steps[0].scales

    @property
    def M(self):
        return self.steps[0].M

    @property
    def N(self):
        return self.steps[0].N

    @property
    def K(self):
        return self.steps[0].K

    @property
    def transposed(self):
        return self.steps[0].layout == LAYOUT_NK


def _shape(sinfo, what, allow_symbolic_first=False):
    tvm = import_tvm()
    if not isinstance(sinfo, tvm.relax.TensorStructInfo) or sinfo.shape is None:
        raise B200CodegenError(f"b200: {what} must be a tensor with a known shape")
    dims = []
    for i, d in enumerate(sinfo.shape.values):
        if isinstance(d, tvm.tir.IntImm):
            dims.append(int(d))
        elif allow_symbolic_first and i == 0:
            dims.append(None)
        else:
            raise B200CodegenError(f"b200: {what} has a symbolic dimension {d}")
    return dims, str(sinfo.dtype)


def _bindings(seq):
    out = []
    for blk in seq.blocks:
        for b in blk.bindings:
            out.append((b.var, b.value))
    return out


def _analyze_group(comp):
    """(x, wq, scales) as indices into comp.params, plus (M, N, K, layout), for one composite."""
    tvm = import_tvm()
    relax = tvm.relax
    pidx = {p: i for i, p in enumerate(comp.params)}
    cb = dict(_bindings(comp.body))

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
    if resolve(cast.args[0]) is not mm and not mm.same_as(resolve(cast.args[0])):
        raise B200CodegenError("b200: the astype must consume the matmul")
    x_param = mm.args[0]
    if x_param not in pidx:
        raise B200CodegenError("b200: the activation must be a parameter of the group")
    w = resolve(mm.args[1])
    transposed = False
    if is_op(w, "relax.permute_dims"):
        axes = w.attrs.axes
        if axes is not None and [int(a) for a in axes] not in ([1, 0], [-1, -2], [1, -2], [-1, 0]):
            raise B200CodegenError(f"b200: permute_dims must swap the two weight axes, got axes={list(axes)}")
        transposed = True
        w = resolve(w.args[0])
    if not is_op(w, "relax.call_tir"):
        raise B200CodegenError("b200: the weight operand must come from call_tir(decode, (wq, scales))")
    dname = w.args[0].name_hint if isinstance(w.args[0], tvm.ir.GlobalVar) else None
    layout = VALIDATED_DECODES.get(dname)
    if layout is None:
        raise B200CodegenError(
            f"b200: the body of decode PrimFunc {dname!r} has not been checked against this backend's quantisation scheme; "
            "partition with partition_for_b200 (or call validate_decodes(mod) before FuseOpsByPattern)")
    if transposed != (layout == LAYOUT_NK):
        raise B200CodegenError(
            "b200: a decode that emits [N, K] must be consumed through permute_dims and one that emits [K, N] "
            "directly; the other combination is x . w, not x . w^T")
    targs = list(w.args[1].fields)
    if len(targs) != 2 or any(a not in pidx for a in targs):
        raise B200CodegenError("b200: decode takes the two parameters (wq, scales)")
    (xs, xd) = _shape(x_param.struct_info, "x", allow_symbolic_first=True)
    (ws, wd) = _shape(targs[0].struct_info, "wq")
    (ss, sd) = _shape(targs[1].struct_info, "scales")
    (dw, dd) = _shape(w.struct_info, "decoded weight")
    if (xd, wd, sd, dd) != ("float16", "uint32", "float16", "float16"):
        raise B200CodegenError(f"b200: dtypes must be x f16, wq u32, scales f16, w f16; got {xd},{wd},{sd},{dd}")
    if len(xs) != 2 or len(ws) != 2 or len(ss) != 2:
        raise B200CodegenError("b200: x, wq and scales must be 2-D")
    M, K = xs
    N = ws[0]
    if K % 32 != 0 or ws[1] * 8 != K or ss != [N, K // 32]:
        raise B200CodegenError(f"b200: need wq [N,K/8] and scales [N,K/32] with K % 32 == 0; got x{xs} wq{ws} s{ss}")
    want_w = [N, K] if layout == LAYOUT_NK else [K, N]
    if dw != want_w:
        raise B200CodegenError(f"b200: decode must produce {want_w}, got {dw}")
    return pidx[x_param], pidx[targs[0]], pidx[targs[1]], M, N, K, layout


def analyze_function(func, options=None) -> Q4Plan:
    """Turns an offloaded function (attrs Codegen="b200", global_symbol) into a plan of kernel calls."""
    tvm = import_tvm()
    relax = tvm.relax
    options = dict(options or {})
    family = str(options.pop("family", "auto"))
    if family not in FAMILIES:
        raise B200CodegenError(f"b200: option family={family!r}; expected one of {sorted(FAMILIES)}")
    layout_code = 0
    if "weight_layout" in options:
        layout = str(options.pop("weight_layout"))
        if layout not in WEIGHT_LAYOUTS:
            raise B200CodegenError(f"b200: option weight_layout={layout!r}; expected one of {sorted(WEIGHT_LAYOUTS)}")
        layout_code = WEIGHT_LAYOUTS[layout]
    if options:
        raise B200CodegenError(f"b200: unknown codegen option(s) {sorted(options)}; known: ['family', 'weight_layout']")
    symbol = str(func.attrs["global_symbol"])
    plan = Q4Plan(symbol, len(func.params), [], FAMILIES[family] | layout_code)
    source = {p: ("param", i) for i, p in enumerate(func.params)}
    local = {}
    last_var = None
    for var, val in _bindings(func.body):
        if isinstance(val, relax.Function):
            if str(val.attrs.get("Composite", "")) != COMPOSITE_NAME:
                raise B200CodegenError(f"b200: unsupported composite {val.attrs.get('Composite')}")
            local[var] = val
        elif isinstance(val, relax.Call) and isinstance(val.op, relax.Var) and val.op in local:
            comp = local[val.op]
            xi, wi, si, M, N, K, layout = _analyze_group(comp)
            args = list(val.args)
            for a in args:
                if a not in source:
                    raise B200CodegenError("b200: composite arguments must be parameters of the offloaded function "
                                           "or results of earlier composites of the same group")
            if source[args[wi]][0] != "param" or source[args[si]][0] != "param":
                raise B200CodegenError("b200: packed weights and scales must be parameters of the offloaded function")
            plan.steps.append(Q4Step(source[args[xi]], source[args[wi]][1], source[args[si]][1], M, N, K, layout))
            source[var] = ("tmp", len(plan.steps) - 1)
            last_var = var
        elif isinstance(val, relax.Var) and val in source:
            source[var] = source[val]          # gv = lv
            if val is last_var or val.same_as(last_var):
                last_var = var
        else:
            raise B200CodegenError(f"b200: unexpected binding in {symbol}: {val}")
    if not plan.steps:
        raise B200CodegenError(f"b200: {symbol} holds no composite call")
    ret = func.body.body
    if not isinstance(ret, relax.Var) or source.get(ret) != ("tmp", len(plan.steps) - 1):
        raise B200CodegenError(f"b200: {symbol} must return the result of its last matmul (single tensor output)")
    # every intermediate must feed a later step as its activation (no other consumer can exist in the group)
    used = {s.x[1] for s in plan.steps if s.x[0] == "tmp"}
    if used != set(range(len(plan.steps) - 1)):
        raise B200CodegenError(f"b200: {symbol} is not a chain of matmuls")
    return plan


def analyze_composite(func) -> Q4Plan:
    """Plan of an offloaded function that holds exactly one matmul (the unmerged case)."""
    plan = analyze_function(func)
    if len(plan.steps) != 1:
        raise B200CodegenError(f"b200: {plan.symbol} holds {len(plan.steps)} matmuls")
    return plan


_PRELUDE = r'''/* Generated by the relax.ext.b200 codegen: forwards to the prebuilt kernel library. */
#include <stdint.h>
#include <tvm/ffi/c_api.h>
#include <tvm/ffi/extra/c_env_api.h>
#include <dlpack/dlpack.h>
#ifdef __cplusplus
extern "C" {
#endif
int b200_q4f16_matmul_dl_family(const void* x, const void* wq, const void* scales, void* y, int32_t family);
int b200_set_stream(void* cuda_stream);
const char* b200_last_error(void);
void* TVMBackendAllocWorkspace(int device_type, int device_id, uint64_t nbytes, int dtype_code_hint, int dtype_bits_hint);
int TVMBackendFreeWorkspace(int device_type, int device_id, void* ptr);
static DLTensor* b200_arg_tensor(const TVMFFIAny* a) {
  if (a->type_index == kTVMFFIDLTensorPtr) return (DLTensor*)a->v_ptr;
  if (a->type_index == kTVMFFITensor) return (DLTensor*)((char*)a->v_obj + sizeof(TVMFFIObject));
  return 0;
}
'''

_EPILOGUE = r'''#ifdef __cplusplus
}
#endif
'''


def emit_wrapper(plan: Q4Plan) -> str:
    """C source of the packed function <symbol>(params..., out) for the tvm_ffi ABI."""
    np_, sym = plan.num_params, plan.symbol
    ntmp = len(plan.steps) - 1
    o = [_PRELUDE]
    o.append(f"TVM_FFI_DLL_EXPORT int __tvm_ffi_{sym}(void* self, const TVMFFIAny* args, int32_t num_args, TVMFFIAny* result) {{")
    o.append(f"  DLTensor* t[{np_ + 1}];")
    if ntmp:
        o.append(f"  DLTensor tmp[{ntmp}];")
        o.append(f"  int64_t tmp_shape[{ntmp}][2];")
        o.append(f"  void* tmp_data[{ntmp}] = {{0}};")
    o.append("  int i, rc = 0, dev_type, dev_id;")
    o.append("  (void)self; (void)result;")
    o.append(f'  if (num_args != {np_ + 1}) {{ TVMFFIErrorSetRaisedFromCStr("TypeError", "{sym}: expected {np_} inputs and 1 output"); return -1; }}')
    o.append(f"  for (i = 0; i < {np_ + 1}; ++i) {{")
    o.append("    t[i] = b200_arg_tensor(&args[i]);")
    o.append(f'    if (!t[i]) {{ TVMFFIErrorSetRaisedFromCStr("TypeError", "{sym}: every argument must be a tensor"); return -1; }}')
    o.append("  }")
    o.append(f"  dev_type = t[{np_}]->device.device_type; dev_id = t[{np_}]->device.device_id;")
    o.append("  /* launch on the runtime's current stream for this device */")
    o.append("  b200_set_stream(TVMFFIEnvGetStream(dev_type, dev_id));")
    for j, st in enumerate(plan.steps):
        xs = f"t[{st.x[1]}]" if st.x[0] == "param" else f"&tmp[{st.x[1]}]"
        if j < ntmp:
            o.append(f"  if (rc == 0) {{   /* intermediate {j}: fp16 [M, {st.N}] from the runtime's workspace pool */")
            o.append(f"    tmp_shape[{j}][0] = {xs}->shape[0]; tmp_shape[{j}][1] = {st.N};")
            o.append(f"    tmp_data[{j}] = TVMBackendAllocWorkspace(dev_type, dev_id, (uint64_t)tmp_shape[{j}][0] * {st.N} * 2, 2, 16);")
            o.append(f'    if (!tmp_data[{j}] && tmp_shape[{j}][0] > 0) {{ TVMFFIErrorSetRaisedFromCStr("RuntimeError", "{sym}: workspace allocation failed"); rc = -1; }}')
            o.append(f"    tmp[{j}].data = tmp_data[{j}]; tmp[{j}].device = t[{np_}]->device; tmp[{j}].ndim = 2;")
            o.append(f"    tmp[{j}].dtype.code = 2; tmp[{j}].dtype.bits = 16; tmp[{j}].dtype.lanes = 1;")
            o.append(f"    tmp[{j}].shape = tmp_shape[{j}]; tmp[{j}].strides = 0; tmp[{j}].byte_offset = 0;")
            o.append("  }")
            ys = f"&tmp[{j}]"
        else:
            ys = f"t[{np_}]"
        o.append(f"  if (rc == 0 && b200_q4f16_matmul_dl_family({xs}, t[{st.wq}], t[{st.scales}], {ys}, {plan.family}) != 0) {{")
        o.append('    TVMFFIErrorSetRaisedFromCStr("RuntimeError", b200_last_error());')
        o.append("    rc = -1;")
        o.append("  }")
    for j in reversed(range(ntmp)):
        o.append(f"  if (tmp_data[{j}]) TVMBackendFreeWorkspace(dev_type, dev_id, tmp_data[{j}]);")
    o.append("  return rc;")
    o.append("}")
    o.append(_EPILOGUE)
    return "\n".join(o)


COMPILED: dict = {}   # symbol -> Q4Plan of everything this process has offloaded


def b200_codegen(functions, options, constant_names):
    """relax.ext.b200: validates each offloaded function and returns one C-source module per function."""
    tvm = import_tvm()
    create = tvm.get_global_func("runtime.CSourceModuleCreate")
    opts = {str(k): (str(v) if not isinstance(v, (int, float)) else v) for k, v in dict(options or {}).items()}
    mods = []
    for func in functions:
        plan = analyze_function(func, opts)
        COMPILED[plan.symbol] = plan
        mods.append(create(emit_wrapper(plan), "c", [plan.symbol], []))
    return mods


def register_codegen():
    import_tvm()
    import tvm_ffi

    tvm_ffi.register_global_func("relax.ext.b200", b200_codegen, override=True)


def validate_decodes(mod) -> dict:
    """Checks the body of every PrimFunc of `mod` against the canonical decode; records and returns
    {name: layout} of those that match."""
    found = decode_layouts(mod)
    VALIDATED_DECODES.update(found)
    return found


def partition_for_b200(mod, options=None, merge=False):
    """FuseOpsByPattern + RunCodegen({"b200": options}), the offload recipe of the reference's tests
    (tests/python/relax/test_codegen_cutlass.py:223-240).  merge=False annotates each matched group for
    the codegen directly (annotate_codegen=True); merge=True runs MergeCompositeFunctions in between, so
    that chained matmuls share one offloaded function."""
    tvm = import_tvm()
    register_codegen()
    found = validate_decodes(mod)
    if not found:
        return mod
    pats = q4f16_matmul_patterns(found)
    if merge:
        mod = tvm.relax.transform.FuseOpsByPattern(pats, annotate_codegen=False)(mod)
        mod = tvm.relax.transform.MergeCompositeFunctions()(mod)
    else:
        mod = tvm.relax.transform.FuseOpsByPattern(pats, annotate_codegen=True)(mod)
    return tvm.relax.transform.RunCodegen({"b200": dict(options or {})})(mod)


def link_options():
    """Compiler options with which ``export_library`` links the generated wrappers against the kernel
    library (placed before the object files on the command line, hence --no-as-needed)."""
    from .. import _lib

    libdir = os.path.dirname(os.path.abspath(_lib.LIB_PATH))
    name = os.path.basename(_lib.LIB_PATH)
    stem = name[3:-3] if name.startswith("lib") and name.endswith(".so") else None
    if stem is None:
        return ["-Wl,--no-as-needed", os.path.abspath(_lib.LIB_PATH), f"-Wl,-rpath,{libdir}"]
    return ["-Wl,--no-as-needed", f"-L{libdir}", f"-l{stem}", f"-Wl,-rpath,{libdir}"]


def finalize_modules(executable, lib_path=None):
    """Exports `executable` (the result of ``relax.build``) as a shared library, compiling the
    generated wrappers and linking them against the kernel library, and loads it back.  Returns the
    loaded runtime module, ready for ``relax.VirtualMachine(module, device)``.  Counterpart of
    finalize_modules_relax (python/tvm/contrib/cutlass/build.py:856-879)."""
    tvm = import_tvm()
    if lib_path is None:
        lib_path = os.path.join(tempfile.mkdtemp(prefix="b200_relax_"), "offloaded.so")
    executable.export_library(lib_path, options=link_options())
    return tvm.runtime.load_module(lib_path)
