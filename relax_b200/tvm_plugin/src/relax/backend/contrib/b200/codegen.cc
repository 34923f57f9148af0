/*
 * BYOC codegen "relax.ext.b200" for the reference tree (place at src/relax/backend/contrib/b200/).
 *
 * Calling convention fixed by RunCodegen (src/relax/transform/run_codegen.cc:158-163):
 *     Array<runtime::Module>(Array<Function> functions, Map<String,ObjectRef> options,
 *                            Map<Constant,String> constant_names)
 * registered like the CUTLASS backend (src/relax/backend/contrib/cutlass/codegen.cc:270).
 *
 * Each incoming function carries Codegen="b200" and global_symbol=<name>; its body calls one local
 * function with Composite="b200.q4f16_matmul" holding
 *     w = call_tir(decode, (wq, scales));  acc = relax.matmul(x, permute_dims(w)|w, "float32");
 *     y = relax.astype(acc, "float16")
 * Parameters arrive in first-use order of the group (FunctionCreator::CheckDefAndUpdateParam,
 * src/relax/transform/fuse_ops.cc:495-517), so roles are recovered by walking the composite body,
 * never by position.  There is no check-callback in this snapshot's FuseOpsByPattern, so every
 * dtype / shape / group-size assumption is validated here and a mismatch is a hard error.
 *
 * The returned module is a CSourceModule ("cc") whose single function unpacks the DLTensor
 * arguments in the function's own parameter order and forwards them, reordered to (x, wq, scales,
 * y), to b200_q4f16_matmul_dl of the prebuilt kernel library: nothing is generated but glue.
 */
#include <tvm/relax/analysis.h>
#include <tvm/relax/attrs/datatype.h>
#include <tvm/relax/attrs/linear_algebra.h>
#include <tvm/relax/expr_functor.h>
#include <tvm/runtime/registry.h>

#include <sstream>
#include <string>

#include "../../../transform/utils.h"
#include "../utils.h"

namespace tvm {
namespace relax {
namespace contrib {

namespace {

struct Q4Roles {
  int x = -1, wq = -1, scales = -1;  // parameter positions of the outer function
  int64_t M = -1, N = -1, K = -1;
};

int ParamIndex(const Function& f, const Expr& e) {
  const auto* v = e.as<VarNode>();
  if (!v) return -1;
  for (size_t i = 0; i < f->params.size(); ++i)
    if (f->params[i].get() == v) return static_cast<int>(i);
  return -1;
}

// Walks the composite function: finds matmul, its activation operand and the decode call_tir that
// produces the weight operand (through an optional permute_dims), and maps them to parameters.
Q4Roles AnalyzeComposite(const Function& composite) {
  Q4Roles r;
  Map<Var, Expr> bind = AnalyzeVar2Value(composite);
  const CallNode* matmul = backend::GetOpInFunction(composite, "relax.matmul");
  const auto* mm_attrs = matmul->attrs.as<MatmulAttrs>();
  ICHECK(mm_attrs && mm_attrs->out_dtype == DataType::Float(32))
      << "b200: the matmul must accumulate in float32 (out_dtype=\"float32\")";
  r.x = ParamIndex(composite, matmul->args[0]);
  ICHECK_GE(r.x, 0) << "b200: the activation must be a parameter of the composite function";

  Expr w = matmul->args[1];
  auto resolve = [&](Expr e) -> const CallNode* {
    if (const auto* v = e.as<VarNode>()) {
      auto it = bind.find(GetRef<Var>(v));
      if (it != bind.end()) return (*it).second.as<CallNode>();
    }
    return e.as<CallNode>();
  };
  const CallNode* wc = resolve(w);
  ICHECK(wc) << "b200: the weight operand is not produced inside the composite function";
  if (backend::IsOp(wc, "relax.permute_dims")) wc = resolve(wc->args[0]);
  ICHECK(wc && backend::IsOp(wc, "relax.call_tir")) << "b200: expected call_tir(decode, (wq, scales))";
  const auto* targs = wc->args[1].as<TupleNode>();
  ICHECK(targs && targs->fields.size() == 2) << "b200: decode takes (wq, scales)";
  r.wq = ParamIndex(composite, targs->fields[0]);
  r.scales = ParamIndex(composite, targs->fields[1]);
  ICHECK(r.wq >= 0 && r.scales >= 0) << "b200: packed weights and scales must be parameters";

  auto shape_of = [&](int idx, DataType want, const char* what) {
    const auto* sinfo = GetStructInfoAs<TensorStructInfoNode>(composite->params[idx]);
    ICHECK(sinfo && sinfo->dtype == want) << "b200: " << what << " must be " << want;
    const auto* sh = sinfo->shape.as<ShapeExprNode>();
    ICHECK(sh && sh->values.size() == 2) << "b200: " << what << " must be a static 2-D tensor";
    return backend::GetIntShape(sh->values);
  };
  auto xs = shape_of(r.x, DataType::Float(16), "x");
  auto ws = shape_of(r.wq, DataType::UInt(32), "wq");
  auto ss = shape_of(r.scales, DataType::Float(16), "scales");
  r.M = xs[0];
  r.K = xs[1];
  r.N = ws[0];
  ICHECK(r.K > 0 && r.K % 32 == 0) << "b200: K must be a positive multiple of the group size 32";
  ICHECK(ws[1] == r.K / 8 && ss[0] == r.N && ss[1] == r.K / 32)
      << "b200: wq must be [N, K/8] and scales [N, K/32] (group size 32, 8 nibbles per word)";
  const CallNode* cast = backend::GetOpInFunction(composite, "relax.astype");
  ICHECK(cast->attrs.as<AstypeAttrs>()->dtype == DataType::Float(16)) << "b200: result must be float16";
  return r;
}

std::string EmitWrapper(const std::string& symbol, const Q4Roles& inner, const std::vector<int>& outer_of_inner,
                        int num_params) {
  // argument i of the packed call = parameter i of the outer function; the last one is the output
  std::ostringstream os;
  os << "#include <tvm/runtime/c_runtime_api.h>\n#include <tvm/runtime/c_backend_api.h>\n"
     << "#include <dlpack/dlpack.h>\n#include \"b200_q4f16.h\"\n"
     << "#ifdef __cplusplus\nextern \"C\"\n#endif\n"
     << "TVM_DLL int32_t " << symbol
     << "(TVMValue* args, int* type_code, int num_args, TVMValue* out_value, int* out_type_code) {\n"
     << "  if (num_args != " << num_params + 1 << ") { TVMAPISetLastError(\"" << symbol
     << ": wrong number of arguments\"); return -1; }\n"
     << "  const B200DLTensor* x = (const B200DLTensor*)args[" << outer_of_inner[inner.x] << "].v_handle;\n"
     << "  const B200DLTensor* wq = (const B200DLTensor*)args[" << outer_of_inner[inner.wq] << "].v_handle;\n"
     << "  const B200DLTensor* sc = (const B200DLTensor*)args[" << outer_of_inner[inner.scales] << "].v_handle;\n"
     << "  B200DLTensor* y = (B200DLTensor*)args[" << num_params << "].v_handle;\n"
     << "  if (b200_q4f16_matmul_dl(x, wq, sc, y) != 0) { TVMAPISetLastError(b200_last_error()); return -1; }\n"
     << "  return 0;\n}\n";
  return os.str();
}

}  // namespace

Array<runtime::Module> B200Compiler(Array<Function> functions, Map<String, ObjectRef> options,
                                    Map<Constant, String> /*constant_names*/) {
  const auto* create = runtime::Registry::Get("runtime.CSourceModuleCreate");
  ICHECK(create) << "runtime.CSourceModuleCreate is not registered";
  Array<runtime::Module> out;
  for (const Function& func : functions) {
    // the outer function's body is a single call to the local composite function
    Map<Var, Expr> bind = AnalyzeVar2Value(func);
    Function composite;
    const CallNode* call = nullptr;
    for (const auto& kv : bind) {
      if (const auto* fn = kv.second.as<FunctionNode>()) {
        auto name = fn->GetAttr<String>(attr::kComposite);
        ICHECK(name.defined() && name.value() == "b200.q4f16_matmul")
            << "relax.ext.b200: unsupported composite " << name;
        composite = GetRef<Function>(fn);
      }
    }
    ICHECK(composite.defined()) << "relax.ext.b200: no composite function in " << GetExtSymbol(func);
    for (const auto& kv : bind)
      if (const auto* c = kv.second.as<CallNode>())
        if (const auto* v = c->op.as<VarNode>())
          if (bind.count(GetRef<Var>(v)) && bind[GetRef<Var>(v)].same_as(composite)) call = c;
    ICHECK(call) << "relax.ext.b200: the composite function is never called";
    Q4Roles roles = AnalyzeComposite(composite);
    std::vector<int> outer_of_inner(composite->params.size(), -1);
    for (size_t i = 0; i < call->args.size(); ++i) outer_of_inner[i] = ParamIndex(func, call->args[i]);
    for (int idx : {roles.x, roles.wq, roles.scales})
      ICHECK_GE(outer_of_inner[idx], 0) << "relax.ext.b200: composite arguments must be function parameters";
    std::string symbol = GetExtSymbol(func);
    std::string code = EmitWrapper(symbol, roles, outer_of_inner, static_cast<int>(func->params.size()));
    out.push_back((*create)(code, "cc", Array<String>{symbol}, Array<String>{}));
  }
  return out;
}

TVM_REGISTER_GLOBAL("relax.ext.b200").set_body_typed(B200Compiler);

}  // namespace contrib
}  // namespace relax
}  // namespace tvm
