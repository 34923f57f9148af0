/*
 * Packed-function registration of the B200 q4f16 kernel library inside a TVM runtime build.
 *
 * Drop this file into the reference tree at src/runtime/contrib/b200/ (it is picked up by
 * cmake/modules/contrib/B200.cmake, next to this file's siblings in this directory tree) and link
 * libb200_q4f16.so.  It is the counterpart of src/runtime/contrib/cublas/cublas.cc:347-368 in the
 * reference: one TVM_REGISTER_GLOBAL per kernel, arguments are DLTensor handles in
 * destination-passing order, the launch goes to the calling thread's current CUDA stream
 * (CUDAThreadEntry, src/runtime/cuda/cuda_common.h:55-66) and errors surface as TVM errors.
 *
 * After this, a Relax module reaches the kernels with
 *     R.call_tir("b200.q4f16_matmul", (x, wq, scales), out_sinfo=R.Tensor((M, N), "float16"))
 * (python/tvm/relax/op/base.py:47-91 turns the string callee into an ExternFunc; the VM resolves it
 * through the global registry, src/runtime/relax_vm/vm.cc:700-725).
 */
#include <tvm/runtime/logging.h>
#include <tvm/runtime/packed_func.h>
#include <tvm/runtime/registry.h>

#include "../../cuda/cuda_common.h"
#include "b200_q4f16.h"  // include/b200_q4f16.h of the kernel library

namespace tvm {
namespace contrib {

using runtime::TVMArgs;
using runtime::TVMRetValue;

namespace {
// B200DLTensor is layout-compatible with DLTensor (see the header); the cast is the whole binding.
inline const B200DLTensor* AsB200(DLTensor* t) { return reinterpret_cast<const B200DLTensor*>(t); }

inline void BindStream() {
  b200_set_stream(static_cast<void*>(runtime::CUDAThreadEntry::ThreadLocal()->stream));
}
}  // namespace

// (x fp16 [M,K], wq uint32 [N,K/8], scales fp16 [N,K/32], y fp16 [M,N])
TVM_REGISTER_GLOBAL("b200.q4f16_matmul").set_body([](TVMArgs args, TVMRetValue* ret) {
  ICHECK_EQ(args.size(), 4) << "b200.q4f16_matmul expects (x, wq, scales, y)";
  DLTensor* x = args[0];
  DLTensor* wq = args[1];
  DLTensor* scales = args[2];
  DLTensor* y = args[3];
  BindStream();
  int rc = b200_q4f16_matmul_dl(AsB200(x), AsB200(wq), AsB200(scales), const_cast<B200DLTensor*>(AsB200(y)));
  ICHECK_EQ(rc, 0) << b200_last_error();
});

// (wq uint32 [N,K/8], scales fp16 [N,K/32], w fp16 [N,K])
TVM_REGISTER_GLOBAL("b200.q4f16_dequantize").set_body([](TVMArgs args, TVMRetValue* ret) {
  ICHECK_EQ(args.size(), 3) << "b200.q4f16_dequantize expects (wq, scales, w)";
  DLTensor* wq = args[0];
  DLTensor* scales = args[1];
  DLTensor* w = args[2];
  BindStream();
  int rc = b200_q4f16_dequantize_dl(AsB200(wq), AsB200(scales), const_cast<B200DLTensor*>(AsB200(w)));
  ICHECK_EQ(rc, 0) << b200_last_error();
});

}  // namespace contrib
}  // namespace tvm
