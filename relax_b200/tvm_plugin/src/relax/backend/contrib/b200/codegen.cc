/*
 * BYOC codegen "relax.ext.b200" for the reference tree (place at src/relax/backend/contrib/b200/).
 *
 * Calling convention fixed by RunCodegen (src/relax/transform/run_codegen.cc:158-163):
 *     Array<runtime::Module>(Array<Function> functions, Map<String,ObjectRef> options,
 *                            Map<Constant,String> constant_names)
 * registered like the CUTLASS backend (src/relax/backend/contrib/cutlass/codegen.cc:270).
 *
 * Each incoming function carries Codegen="b200" and global_symbol=<name>; its body binds local
 * functions with Composite="b200.q4f16_matmul" and calls them -- one after
 * FuseOpsByPattern(annotate_codegen=true), a chain of several after MergeCompositeFunctions
 * (src/relax/transform/merge_composite_functions.cc:30-60).  A composite holds
 *     w = call_tir(decode, (wq, scales));  acc = relax.matmul(x, permute_dims(w) | w, "float32");
 *     y = relax.astype(acc, "float16")
 * Parameters arrive in first-use order of the group (FunctionCreator::CheckDefAndUpdateParam,
 * src/relax/transform/fuse_ops.cc:495-517), so roles are recovered by walking the composite body,
 * never by position.  There is no check-callback in this snapshot's FuseOpsByPattern, so every
 * dtype / shape / layout assumption is validated here and a mismatch is a hard error.
 *
 * What the decode PrimFunc computes cannot be seen from here (the codegen receives functions, not the
 * module).  The Python half (python/tvm/relax/backend/b200) compares each decode PrimFunc with the
 * canonical one before its name enters the pattern table and passes the result in the option map:
 *     options["decode_layouts"] = {"<primfunc name>": "nk" | "kn"}   ([N,K] needs permute_dims, [K,N] must not have it)
 *     options["family"]         = "auto" | "gemv" | "gemm"            (kernel family the wrapper asks for)
 *     options["weight_layout"]  = "reference" | "paired"              (nibble order of the bound weights after the
 *                                                                      offline repack; absent = the library's option)
 * A call_tir to a name that is not in the map is refused.
 *
 * The returned module is a CSourceModule ("cc") per function whose code unpacks the DLTensor
 * arguments in the function's own parameter order and forwards them, reordered to (x, wq, scales,
 * y), to b200_q4f16_matmul_dl_family of the prebuilt kernel library; intermediates of a chain come
 * from TVMBackendAllocWorkspace (include/tvm/runtime/c_backend_api.h:60-84).  Nothing is generated
 * but glue.
 */
#include <tvm/relax/analysis.h>
#include <tvm/relax/attrs/datatype.h>
#include <tvm/relax/attrs/linear_algebra.h>
#include <tvm/relax/attrs/manipulate.h>
#include <tvm/relax/expr_functor.h>
#include <tvm/runtime/registry.h>

#include <sstream>
#include <string>
#include <unordered_map>
#include <vector>

#include "../../../transform/utils.h"
#include "../utils.h"

namespace tvm {
namespace relax {
namespace contrib {

namespace {

struct Q4Group {
  int x = -1, wq = -1, scales = -1;  // parameter positions inside the composite function
  int64_t N = -1, K = -1;            // M is read from x at run time (it may be symbolic)
};

// One kernel call of the emitted wrapper.  x_arg >= 0: packed-call argument index; x_tmp >= 0: result of an
// earlier step.
struct Q4Step {
  int x_arg = -1, x_tmp = -1, wq_arg = -1, scales_arg = -1;
  int64_t N = -1, K = -1;
};

int ParamIndex(const Function& f, const Expr& e) {
  const auto* v = e.as<VarNode>();
  if (!v) return -1;
  for (size_t i = 0; i < f->params.size(); ++i)
    if (f->params[i].get() == v) return static_cast<int>(i);
  return -1;
}

// Walks a composite function: finds matmul, its activation operand and the decode call_tir that
// produces the weight operand (through permute_dims for an [N,K] decode), and maps them to parameters.
Q4Group AnalyzeComposite(const Function& composite, const Map<String, ObjectRef>& decode_layouts) {
  Q4Group r;
  Map<Var, Expr> bind = AnalyzeVar2Value(composite);
  const CallNode* matmul = backend::GetOpInFunction(composite, "relax.matmul");
  const auto* mm_attrs = matmul->attrs.as<MatmulAttrs>();
  ICHECK(mm_attrs && mm_attrs->out_dtype == DataType::Float(32))
      << "b200: the matmul must accumulate in float32 (out_dtype=\"float32\")";
  r.x = ParamIndex(composite, matmul->args[0]);
  ICHECK_GE(r.x, 0) << "b200: the activation must be a parameter of the composite function";

  auto resolve = [&](Expr e) -> const CallNode* {
    if (const auto* v = e.as<VarNode>()) {
      auto it = bind.find(GetRef<Var>(v));
      if (it != bind.end()) return (*it).second.as<CallNode>();
    }
    return e.as<CallNode>();
  };
  const CallNode* wc = resolve(matmul->args[1]);
  ICHECK(wc) << "b200: the weight operand is not produced inside the composite function";
  bool transposed = false;
  if (backend::IsOp(wc, "relax.permute_dims")) {
    const auto* pa = wc->attrs.as<PermuteDimsAttrs>();
    if (pa && pa->axes.defined()) {
      Array<Integer> axes = pa->axes.value();
      ICHECK(axes.size() == 2 && (axes[0]->value == 1 || axes[0]->value == -1) &&
             (axes[1]->value == 0 || axes[1]->value == -2))
          << "b200: permute_dims must swap the two weight axes";
    }
    transposed = true;
    wc = resolve(wc->args[0]);
  }
  ICHECK(wc && backend::IsOp(wc, "relax.call_tir")) << "b200: expected call_tir(decode, (wq, scales))";
  const auto* gv = wc->args[0].as<GlobalVarNode>();
  ICHECK(gv) << "b200: call_tir callee must be a PrimFunc of the module";
  auto lit = decode_layouts.find(gv->name_hint);
  ICHECK(lit != decode_layouts.end())
      << "b200: the body of decode PrimFunc '" << gv->name_hint
      << "' has not been checked against this backend's quantisation scheme (options[\"decode_layouts\"])";
  const auto* layout = (*lit).second.as<StringObj>();
  ICHECK(layout) << "b200: decode_layouts values must be strings";
  const bool nk = std::string(layout->data, layout->size) == "nk";
  ICHECK(nk == transposed) << "b200: a decode that emits [N,K] must be consumed through permute_dims and one that "
                              "emits [K,N] directly; the other combination is x.w, not x.w^T";
  const auto* targs = wc->args[1].as<TupleNode>();
  ICHECK(targs && targs->fields.size() == 2) << "b200: decode takes (wq, scales)";
  r.wq = ParamIndex(composite, targs->fields[0]);
  r.scales = ParamIndex(composite, targs->fields[1]);
  ICHECK(r.wq >= 0 && r.scales >= 0) << "b200: packed weights and scales must be parameters";

  auto tensor_of = [&](int idx, DataType want, const char* what) {
    const auto* sinfo = GetStructInfoAs<TensorStructInfoNode>(composite->params[idx]);
    ICHECK(sinfo && sinfo->dtype == want) << "b200: " << what << " must be " << want;
    const auto* sh = sinfo->shape.as<ShapeExprNode>();
    ICHECK(sh && sh->values.size() == 2) << "b200: " << what << " must be a 2-D tensor with a known shape";
    return sh;
  };
  auto static_dim = [&](const PrimExpr& e, const char* what) {
    const auto* imm = e.as<IntImmNode>();
    ICHECK(imm) << "b200: " << what << " must be a static dimension";
    return imm->value;
  };
  const auto* xs = tensor_of(r.x, DataType::Float(16), "x");
  const auto* ws = tensor_of(r.wq, DataType::UInt(32), "wq");
  const auto* ss = tensor_of(r.scales, DataType::Float(16), "scales");
  r.K = static_dim(xs->values[1], "K");          // xs->values[0] (the batch) may be symbolic
  r.N = static_dim(ws->values[0], "N");
  ICHECK(r.K > 0 && r.K % 32 == 0) << "b200: K must be a positive multiple of the group size 32";
  ICHECK(static_dim(ws->values[1], "wq columns") == r.K / 8 && static_dim(ss->values[0], "scale rows") == r.N &&
         static_dim(ss->values[1], "scale columns") == r.K / 32)
      << "b200: wq must be [N, K/8] and scales [N, K/32] (group size 32, 8 nibbles per word)";
  const CallNode* cast = backend::GetOpInFunction(composite, "relax.astype");
  ICHECK(cast->attrs.as<AstypeAttrs>()->dtype == DataType::Float(16)) << "b200: result must be float16";
  return r;
}

std::string EmitWrapper(const std::string& symbol, const std::vector<Q4Step>& steps, int num_params, int family) {
  // argument i of the packed call = parameter i of the offloaded function; the last one is the output
  const int ntmp = static_cast<int>(steps.size()) - 1;
  std::ostringstream os;
  os << "#include <tvm/runtime/c_runtime_api.h>\n#include <tvm/runtime/c_backend_api.h>\n"
     << "#include <dlpack/dlpack.h>\n#include \"b200_q4f16.h\"\n"
     << "#ifdef __cplusplus\nextern \"C\"\n#endif\n"
     << "TVM_DLL int32_t " << symbol
     << "(TVMValue* args, int* type_code, int num_args, TVMValue* out_value, int* out_type_code) {\n"
     << "  if (num_args != " << num_params + 1 << ") { TVMAPISetLastError(\"" << symbol
     << ": wrong number of arguments\"); return -1; }\n"
     << "  for (int i = 0; i < num_args; ++i)\n"
     << "    if (type_code[i] != kTVMDLTensorHandle && type_code[i] != kTVMNDArrayHandle) { TVMAPISetLastError(\"" << symbol
     << ": every argument must be a tensor\"); return -1; }\n"
     << "  B200DLTensor* y = (B200DLTensor*)args[" << num_params << "].v_handle;\n"
     << "  int rc = 0;\n";
  if (ntmp > 0)
    os << "  B200DLTensor tmp[" << ntmp << "]; int64_t tmp_shape[" << ntmp << "][2]; void* tmp_data[" << ntmp
       << "] = {0};\n";
  for (size_t j = 0; j < steps.size(); ++j) {
    const Q4Step& st = steps[j];
    std::ostringstream xs;
    if (st.x_arg >= 0) xs << "((const B200DLTensor*)args[" << st.x_arg << "].v_handle)";
    else xs << "(&tmp[" << st.x_tmp << "])";
    std::string out = "y";
    if (static_cast<int>(j) < ntmp) {
      os << "  if (rc == 0) {\n"
         << "    tmp_shape[" << j << "][0] = " << xs.str() << "->shape[0]; tmp_shape[" << j << "][1] = " << st.N << ";\n"
         << "    tmp_data[" << j << "] = TVMBackendAllocWorkspace(y->device.device_type, y->device.device_id, (uint64_t)tmp_shape["
         << j << "][0] * " << st.N << " * 2, kDLFloat, 16);\n"
         << "    if (!tmp_data[" << j << "] && tmp_shape[" << j << "][0] > 0) { TVMAPISetLastError(\"" << symbol
         << ": workspace allocation failed\"); rc = -1; }\n"
         << "    tmp[" << j << "].data = tmp_data[" << j << "]; tmp[" << j << "].device = y->device; tmp[" << j << "].ndim = 2;\n"
         << "    tmp[" << j << "].dtype.code = 2; tmp[" << j << "].dtype.bits = 16; tmp[" << j << "].dtype.lanes = 1;\n"
         << "    tmp[" << j << "].shape = tmp_shape[" << j << "]; tmp[" << j << "].strides = 0; tmp[" << j << "].byte_offset = 0;\n"
         << "  }\n";
      std::ostringstream o2;
      o2 << "&tmp[" << j << "]";
      out = o2.str();
    }
    os << "  if (rc == 0 && b200_q4f16_matmul_dl_family(" << xs.str() << ", (const B200DLTensor*)args[" << st.wq_arg
       << "].v_handle, (const B200DLTensor*)args[" << st.scales_arg << "].v_handle, " << out << ", " << family
       << ") != 0) { TVMAPISetLastError(b200_last_error()); rc = -1; }\n";
  }
  for (int j = ntmp - 1; j >= 0; --j)
    os << "  if (tmp_data[" << j << "]) TVMBackendFreeWorkspace(y->device.device_type, y->device.device_id, tmp_data[" << j
       << "]);\n";
  os << "  (void)out_value; (void)out_type_code;\n  return rc;\n}\n";
  return os.str();
}

int FamilyOf(const Map<String, ObjectRef>& options) {
  auto it = options.find("family");
  if (it == options.end()) return 0;
  const auto* s = (*it).second.as<StringObj>();
  ICHECK(s) << "relax.ext.b200: option \"family\" must be a string";
  std::string v(s->data, s->size);
  if (v == "auto") return 0;
  if (v == "gemv") return 1;
  if (v == "gemm") return 2;
  LOG(FATAL) << "relax.ext.b200: option family=\"" << v << "\"; expected auto, gemv or gemm";
  return 0;
}

// Bits 8-15 of the family argument: weight layout + 1 (B200_FAMILY_WITH_LAYOUT in b200_q4f16.h), 0 = the library's option.
int LayoutBitsOf(const Map<String, ObjectRef>& options) {
  auto it = options.find("weight_layout");
  if (it == options.end()) return 0;
  const auto* s = (*it).second.as<StringObj>();
  ICHECK(s) << "relax.ext.b200: option \"weight_layout\" must be a string";
  std::string v(s->data, s->size);
  if (v == "reference") return (0 + 1) << 8;
  if (v == "paired") return (1 + 1) << 8;
  LOG(FATAL) << "relax.ext.b200: option weight_layout=\"" << v << "\"; expected reference or paired";
  return 0;
}

}  // namespace

Array<runtime::Module> B200Compiler(Array<Function> functions, Map<String, ObjectRef> options,
                                    Map<Constant, String> /*constant_names*/) {
  const auto* create = runtime::Registry::Get("runtime.CSourceModuleCreate");
  ICHECK(create) << "runtime.CSourceModuleCreate is not registered";
  for (const auto& kv : options)
    ICHECK(kv.first == "family" || kv.first == "decode_layouts" || kv.first == "weight_layout")
        << "relax.ext.b200: unknown option " << kv.first;
  const int family = FamilyOf(options) | LayoutBitsOf(options);
  Map<String, ObjectRef> decode_layouts;
  if (options.count("decode_layouts")) decode_layouts = Downcast<Map<String, ObjectRef>>(options["decode_layouts"]);

  Array<runtime::Module> out;
  for (const Function& func : functions) {
    const std::string symbol = GetExtSymbol(func);
    const auto* seq = func->body.as<SeqExprNode>();
    ICHECK(seq) << "relax.ext.b200: " << symbol << " has no binding block";
    std::unordered_map<const VarNode*, Function> local;       // var -> composite function
    std::unordered_map<const VarNode*, int> produced_by;      // var -> step that produced it
    std::vector<Q4Step> steps;
    for (const BindingBlock& blk : seq->blocks) {
      for (const Binding& b : blk->bindings) {
        const auto* vb = b.as<VarBindingNode>();
        ICHECK(vb) << "relax.ext.b200: unexpected binding kind in " << symbol;
        if (const auto* fn = vb->value.as<FunctionNode>()) {
          auto name = fn->GetAttr<String>(attr::kComposite);
          ICHECK(name.defined() && name.value() == "b200.q4f16_matmul") << "relax.ext.b200: unsupported composite " << name;
          local[vb->var.get()] = GetRef<Function>(fn);
        } else if (const auto* call = vb->value.as<CallNode>()) {
          const auto* callee = call->op.as<VarNode>();
          ICHECK(callee && local.count(callee)) << "relax.ext.b200: " << symbol << " may only call its composite functions";
          const Function& composite = local[callee];
          Q4Group g = AnalyzeComposite(composite, decode_layouts);
          Q4Step st;
          st.N = g.N;
          st.K = g.K;
          st.wq_arg = ParamIndex(func, call->args[g.wq]);
          st.scales_arg = ParamIndex(func, call->args[g.scales]);
          ICHECK(st.wq_arg >= 0 && st.scales_arg >= 0) << "relax.ext.b200: packed weights and scales must be function parameters";
          st.x_arg = ParamIndex(func, call->args[g.x]);
          if (st.x_arg < 0) {
            const auto* xv = call->args[g.x].as<VarNode>();
            ICHECK(xv && produced_by.count(xv)) << "relax.ext.b200: the activation must be a parameter or an earlier result";
            st.x_tmp = produced_by[xv];
          }
          produced_by[vb->var.get()] = static_cast<int>(steps.size());
          steps.push_back(st);
        } else if (const auto* alias = vb->value.as<VarNode>()) {
          ICHECK(produced_by.count(alias)) << "relax.ext.b200: unexpected alias in " << symbol;
          produced_by[vb->var.get()] = produced_by[alias];
        } else {
          LOG(FATAL) << "relax.ext.b200: unexpected binding in " << symbol;
        }
      }
    }
    ICHECK(!steps.empty()) << "relax.ext.b200: no composite call in " << symbol;
    const auto* ret = seq->body.as<VarNode>();
    ICHECK(ret && produced_by.count(ret) && produced_by[ret] == static_cast<int>(steps.size()) - 1)
        << "relax.ext.b200: " << symbol << " must return the result of its last matmul";
    for (size_t j = 1; j < steps.size(); ++j)
      ICHECK(steps[j].x_tmp == static_cast<int>(j) - 1) << "relax.ext.b200: " << symbol << " is not a chain of matmuls";
    std::string code = EmitWrapper(symbol, steps, static_cast<int>(func->params.size()), family);
    out.push_back((*create)(code, "cc", Array<String>{symbol}, Array<String>{}));
  }
  return out;
}

TVM_REGISTER_GLOBAL("relax.ext.b200").set_body_typed(B200Compiler);

}  // namespace contrib
}  // namespace relax
}  // namespace tvm
