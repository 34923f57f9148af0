"""The BYOC surface (pattern table, partitioning, relax.ext.b200) against a real Relax
implementation: the TVM 0.23 bundled with the tilelang wheel, the importable descendant of the
reference.  Structural checks run on CPU; the end-to-end VM run needs the GPU."""
import numpy as np
import pytest

from relax_b200 import backend

pytestmark = pytest.mark.skipif(not backend.have_tvm(), reason="no TVM with Relax importable")


def q4_module(M, N, K, transposed=True, acc="float32", wq_dtype="uint32"):
    tvm = backend.import_tvm()
    from tvm import relax, te

    def decode(wq, s):
        return te.compute(
            (N, K),
            lambda n, k: ((((wq[n, k // 8] >> (k % 8 * 4).astype(wq_dtype)) & tvm.tir.const(0xF, wq_dtype))
                           .astype("int32") - 7)).astype("float16") * s[n, k // 32],
            name="decode")

    bb = relax.BlockBuilder()
    x = relax.Var("x", relax.TensorStructInfo((M, K), "float16"))
    wq = relax.Var("wq", relax.TensorStructInfo((N, K // 8), wq_dtype))
    s = relax.Var("s", relax.TensorStructInfo((N, K // 32), "float16"))
    with bb.function("main", [x, wq, s]):
        with bb.dataflow():
            w = bb.emit_te(decode, wq, s, primfunc_name_hint="decode")
            if transposed:
                w = bb.emit(relax.op.permute_dims(w))
            acc_v = bb.emit(relax.op.matmul(x, w, out_dtype=acc))
            y = bb.emit(relax.op.astype(acc_v, "float16"))
            out = bb.emit_output(y)
        bb.emit_func_output(out)
    return bb.get()


def test_partition_rewrites_main_to_one_extern_call():
    mod = backend.partition_for_b200(q4_module(2, 64, 128))
    text = mod.script()
    # RunCodegen leaves a destination-passing extern call with the group's own parameter order
    assert 'R.call_dps_packed("fused_decode_relax_permute_dims_relax_matmul_relax_astype_b200", (wq, s, x)' in text
    assert "decode" not in [gv.name_hint for gv in mod.functions]      # the unused PrimFunc is dropped
    roles = backend.codegen.COMPILED["fused_decode_relax_permute_dims_relax_matmul_relax_astype_b200"]
    assert (roles.wq, roles.scales, roles.x) == (0, 1, 2)             # first-use order, not main's order
    assert (roles.M, roles.N, roles.K, roles.transposed) == (2, 64, 128, True)


def test_codegen_rejects_what_the_kernels_do_not_compute():
    tvm = backend.import_tvm()
    # fp16 accumulation is a different computation
    with pytest.raises(Exception, match="float32"):
        backend.partition_for_b200(q4_module(2, 64, 128, acc="float16"))
    # int32-packed weights: the dtype check of the codegen, not a silent reinterpretation
    with pytest.raises(Exception, match="dtypes must be"):
        backend.partition_for_b200(q4_module(2, 64, 128, wq_dtype="int32"))


def test_pattern_table_leaves_other_matmuls_alone():
    tvm = backend.import_tvm()
    from tvm import relax

    bb = relax.BlockBuilder()
    a = relax.Var("a", relax.TensorStructInfo((4, 8), "float16"))
    b = relax.Var("b", relax.TensorStructInfo((8, 4), "float16"))
    with bb.function("main", [a, b]):
        with bb.dataflow():
            y = bb.emit(relax.op.astype(relax.op.matmul(a, b, out_dtype="float32"), "float16"))
            out = bb.emit_output(y)
        bb.emit_func_output(out)
    mod = backend.partition_for_b200(bb.get())
    assert "call_dps_packed" not in mod.script()


@pytest.mark.gpu
@pytest.mark.parametrize("M,N,K", [(1, 512, 1024), (160, 512, 256)])
def test_relax_vm_runs_the_offloaded_module_on_the_gpu(M, N, K):
    import torch

    import oracle
    from relax_b200 import synth
    from relax_b200.backend import tvm_bridge
    from util import assert_matmul_close

    tvm = backend.import_tvm()
    from tvm import relax

    tvm_bridge.register_packed_funcs()
    mod = backend.partition_for_b200(q4_module(M, N, K))
    ex = relax.build(mod, target="cuda")
    vm = relax.VirtualMachine(ex, tvm.cuda(0))
    x, wq, s = synth.make_case(M, N, K, seed=5)
    dev = tvm.cuda(0)
    y = vm["main"](tvm.runtime.tensor(x, dev), tvm.runtime.tensor(wq, dev), tvm.runtime.tensor(s, dev))
    torch.cuda.synchronize()
    assert_matmul_close(y.numpy(), x, wq, s, f"relax vm M={M}")


@pytest.mark.gpu
def test_relax_vm_calls_the_registered_packed_function_directly():
    import torch

    from relax_b200 import synth
    from relax_b200.backend import tvm_bridge
    from util import assert_matmul_close

    tvm = backend.import_tvm()
    from tvm import relax
    from tvm.script import relax as R  # noqa: F401

    tvm_bridge.register_packed_funcs()
    M, N, K = 3, 256, 512
    bb = relax.BlockBuilder()
    x = relax.Var("x", relax.TensorStructInfo((M, K), "float16"))
    wq = relax.Var("wq", relax.TensorStructInfo((N, K // 8), "uint32"))
    s = relax.Var("s", relax.TensorStructInfo((N, K // 32), "float16"))
    with bb.function("main", [x, wq, s]):
        with bb.dataflow():
            y = bb.emit(relax.op.call_dps_packed("b200.q4f16_matmul", (x, wq, s),
                                                 relax.TensorStructInfo((M, N), "float16")))
            out = bb.emit_output(y)
        bb.emit_func_output(out)
    ex = relax.build(bb.get(), target="cuda")
    vm = relax.VirtualMachine(ex, tvm.cuda(0))
    xa, wqa, sa = synth.make_case(M, N, K, seed=6)
    dev = tvm.cuda(0)
    yv = vm["main"](tvm.runtime.tensor(xa, dev), tvm.runtime.tensor(wqa, dev), tvm.runtime.tensor(sa, dev))
    torch.cuda.synchronize()
    assert_matmul_close(yv.numpy(), xa, wqa, sa, "call_dps_packed")
