"""The BYOC surface (pattern table, decode check, partitioning, relax.ext.b200, export round trip)
against a real Relax implementation: the TVM 0.23 bundled with the tilelang wheel, the importable
descendant of the reference.  Structural checks and the export -> load -> call chain run on CPU (the
call ends in the kernel library's own "not a CUDA device" error, which proves the wrapper reached
it); the numeric runs need the GPU.

Reference tests these mirror: tests/python/relax/test_transform_codegen_pass.py:57-65 (export
round trip), :184-256 (RunCodegen's rewritten IR), tests/python/relax/test_transform_fuse_ops_by_pattern.py
:41-82 (annotated groups), tests/python/relax/test_transform_merge_composite_functions.py (merged groups).
"""
import numpy as np
import pytest

from relax_b200 import backend

pytestmark = pytest.mark.skipif(not backend.have_tvm(), reason="no TVM with Relax importable")

SYMBOL = "fused_decode_relax_permute_dims_relax_matmul_relax_astype_b200"


def make_decode(N, K, layout="nk", zero_point=7, wq_dtype="uint32", high_nibble_first=False):
    """TE decode stage as a model author writes it; the defaults are this backend's scheme."""
    tvm = backend.import_tvm()
    from tvm import te

    def value(wq, s, n, k):
        sel = (7 - k % 8) if high_nibble_first else k % 8
        q = (wq[n, k // 8] >> (sel * 4).astype(wq_dtype)) & tvm.tir.const(0xF, wq_dtype)
        return (q.astype("int32") - zero_point).astype("float16") * s[n, k // 32]

    def decode(wq, s):
        if layout == "nk":
            return te.compute((N, K), lambda n, k: value(wq, s, n, k), name="decode")
        return te.compute((K, N), lambda k, n: value(wq, s, n, k), name="decode")

    return decode


def q4_module(M, N, K, transposed=True, acc="float32", wq_dtype="uint32", layout="nk", zero_point=7,
              high_nibble_first=False, symbolic_m=False):
    tvm = backend.import_tvm()
    from tvm import relax

    bb = relax.BlockBuilder()
    m = tvm.tir.Var("m", "int64") if symbolic_m else M
    x = relax.Var("x", relax.TensorStructInfo((m, K), "float16"))
    wq = relax.Var("wq", relax.TensorStructInfo((N, K // 8), wq_dtype))
    s = relax.Var("s", relax.TensorStructInfo((N, K // 32), "float16"))
    with bb.function("main", [x, wq, s]):
        with bb.dataflow():
            w = bb.emit_te(make_decode(N, K, layout, zero_point, wq_dtype, high_nibble_first), wq, s,
                           primfunc_name_hint="decode")
            if transposed:
                w = bb.emit(relax.op.permute_dims(w))
            acc_v = bb.emit(relax.op.matmul(x, w, out_dtype=acc))
            y = bb.emit(relax.op.astype(acc_v, "float16"))
            out = bb.emit_output(y)
        bb.emit_func_output(out)
    return bb.get()


def chain_module(M, K, N1, N2):
    """Two q4f16 linear layers back to back: y = q4(q4(x, w1), w2)."""
    tvm = backend.import_tvm()
    from tvm import relax

    bb = relax.BlockBuilder()
    x = relax.Var("x", relax.TensorStructInfo((M, K), "float16"))
    wq1 = relax.Var("wq1", relax.TensorStructInfo((N1, K // 8), "uint32"))
    s1 = relax.Var("s1", relax.TensorStructInfo((N1, K // 32), "float16"))
    wq2 = relax.Var("wq2", relax.TensorStructInfo((N2, N1 // 8), "uint32"))
    s2 = relax.Var("s2", relax.TensorStructInfo((N2, N1 // 32), "float16"))
    with bb.function("main", [x, wq1, s1, wq2, s2]):
        with bb.dataflow():
            h = x
            for (n, k, wq, s) in ((N1, K, wq1, s1), (N2, N1, wq2, s2)):
                w = bb.emit_te(make_decode(n, k), wq, s, primfunc_name_hint="decode")
                w = bb.emit(relax.op.permute_dims(w))
                h = bb.emit(relax.op.astype(bb.emit(relax.op.matmul(h, w, out_dtype="float32")), "float16"))
            out = bb.emit_output(h)
        bb.emit_func_output(out)
    return bb.get()


def offloaded(mod):
    return "call_dps_packed" in mod.script()


# ------------------------------------------------------------------------------------ structure (CPU)
def test_partition_rewrites_main_to_one_extern_call_and_returns_a_module():
    mod = backend.partition_for_b200(q4_module(2, 64, 128))
    text = mod.script()
    # RunCodegen leaves a destination-passing extern call with the group's own parameter order
    assert f'R.call_dps_packed("{SYMBOL}", (wq, s, x)' in text
    assert "decode" not in [gv.name_hint for gv in mod.functions]      # the unused PrimFunc is dropped
    # ... and stores what the codegen returned where the VM build picks it up (run_codegen.cc:53-55)
    ext = mod.attrs["external_mods"]
    assert len(ext) == 1
    plan = backend.codegen.COMPILED[SYMBOL]
    assert (plan.wq, plan.scales, plan.x) == (0, 1, 2)                 # first-use order, not main's order
    assert (plan.M, plan.N, plan.K, plan.transposed) == (2, 64, 128, True)
    src = backend.emit_wrapper(plan)
    assert f"__tvm_ffi_{SYMBOL}" in src and "b200_q4f16_matmul_dl_family(t[2], t[0], t[1], t[3], 0)" in src


def test_codegen_rejects_what_the_kernels_do_not_compute():
    # fp16 accumulation is a different computation: the pattern matches, the codegen refuses
    with pytest.raises(Exception, match="float32"):
        backend.partition_for_b200(q4_module(2, 64, 128, acc="float16"))


@pytest.mark.parametrize("kwargs", [
    dict(wq_dtype="int32"),                 # arithmetic shift on a signed word is another function
    dict(zero_point=8),                     # same tensor signature, different arithmetic
    dict(high_nibble_first=True),           # other nibble order
])
def test_a_decode_with_other_arithmetic_is_left_alone(kwargs):
    mod = q4_module(2, 64, 128, **kwargs)
    assert backend.decode_layouts(mod) == {}
    assert not offloaded(backend.partition_for_b200(mod))


def test_untransposed_matmul_on_a_square_weight_is_not_offloaded():
    # decode emits [N, K] with N == K, and the matmul takes it WITHOUT permute_dims: that is x . w, which the
    # kernels (x . w^T) do not compute.  It must stay on the reference's own lowering.
    mod = q4_module(2, 128, 128, transposed=False)
    assert backend.decode_layouts(mod) == {"decode": "nk"}
    assert not offloaded(backend.partition_for_b200(mod))


def test_decode_that_emits_the_transposed_layout_is_offloaded_without_permute_dims():
    mod = q4_module(2, 64, 128, transposed=False, layout="kn")
    assert backend.decode_layouts(mod) == {"decode": "kn"}
    out = backend.partition_for_b200(mod)
    assert offloaded(out)
    plan = backend.codegen.COMPILED["fused_decode_relax_matmul_relax_astype_b200"]
    assert (plan.M, plan.N, plan.K, plan.transposed) == (2, 64, 128, False)
    # ... but not when it is transposed once more
    assert not offloaded(backend.partition_for_b200(q4_module(2, 128, 128, transposed=True, layout="kn")))


def test_second_spelling_of_the_same_arithmetic_is_recognised():
    tvm = backend.import_tvm()
    from tvm import relax

    N, K = 32, 64
    bb = relax.BlockBuilder()
    wq = relax.Var("wq", relax.TensorStructInfo((N, K // 8), "uint32"))
    s = relax.Var("s", relax.TensorStructInfo((N, K // 32), "float16"))
    with bb.function("f", [wq, s]):
        bb.emit_func_output(bb.emit_te(backend.canonical_decode_te(N, K, "nk", spelling=1), wq, s, primfunc_name_hint="decode"))
    assert backend.decode_layouts(bb.get()) == {"decode": "nk"}


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
    assert not offloaded(mod)


def test_codegen_options():
    mod = backend.partition_for_b200(q4_module(2, 64, 128), options={"family": "gemv"})
    assert offloaded(mod)
    assert backend.codegen.COMPILED[SYMBOL].family == 1
    assert ", 1) != 0" in backend.emit_wrapper(backend.codegen.COMPILED[SYMBOL])
    with pytest.raises(Exception, match="family"):
        backend.partition_for_b200(q4_module(2, 64, 128), options={"family": "warp-speed"})
    with pytest.raises(Exception, match="unknown codegen option"):
        backend.partition_for_b200(q4_module(2, 64, 128), options={"tile": "128"})
    # the layout of weights repacked offline travels in bits 8-15 of the family argument (layout + 1)
    backend.partition_for_b200(q4_module(2, 64, 128), options={"family": "gemv", "weight_layout": "paired"})
    assert backend.codegen.COMPILED[SYMBOL].family == (1 | (2 << 8))
    assert ", 513) != 0" in backend.emit_wrapper(backend.codegen.COMPILED[SYMBOL])
    backend.partition_for_b200(q4_module(2, 64, 128), options={"weight_layout": "reference"})
    assert backend.codegen.COMPILED[SYMBOL].family == (1 << 8)
    with pytest.raises(Exception, match="weight_layout"):
        backend.partition_for_b200(q4_module(2, 64, 128), options={"weight_layout": "zigzag"})


def test_unvalidated_decode_name_is_refused_by_the_codegen():
    """FuseOpsByPattern run by hand with a decode whose body nobody checked: the codegen refuses."""
    tvm = backend.import_tvm()
    from tvm import relax

    backend.register_codegen()
    backend.codegen.VALIDATED_DECODES.pop("decode", None)
    mod = q4_module(2, 64, 128, zero_point=8)
    pats = backend.q4f16_matmul_patterns({"decode": "nk"})
    mod = relax.transform.FuseOpsByPattern(pats, annotate_codegen=True)(mod)
    with pytest.raises(Exception, match="has not been checked"):
        relax.transform.RunCodegen({"b200": {}})(mod)


def _cpu_args(*shapes_dtypes):
    tvm = backend.import_tvm()
    return [tvm.runtime.tensor(np.zeros(sh, dt)) for sh, dt in shapes_dtypes]


def test_export_load_call_reaches_the_kernel_library():
    """relax.build -> export_library (wrapper compiled, kernel library linked) -> load_module -> VM call.
    Mirrors check_roundtrip of the reference (tests/python/relax/test_transform_codegen_pass.py:57-65).
    On a CPU tensor the call must come back with the kernel library's own validation message."""
    tvm = backend.import_tvm()
    from tvm import relax

    mod = backend.partition_for_b200(q4_module(2, 64, 128))
    ex = relax.build(mod, target="c")
    lib = backend.finalize_modules(ex)
    vm = relax.VirtualMachine(lib, tvm.cpu())
    with pytest.raises(Exception, match="b200.q4f16_matmul: x is not on a CUDA device"):
        vm["main"](*_cpu_args(((2, 128), "float16"), ((64, 16), "uint32"), ((64, 4), "float16")))


def test_merge_composite_functions_gives_one_offloaded_chain():
    tvm = backend.import_tvm()
    from tvm import relax

    mod = backend.partition_for_b200(chain_module(3, 128, 64, 32), merge=True)
    text = mod.script()
    assert text.count("call_dps_packed") == 1, text
    plans = [p for p in backend.codegen.COMPILED.values() if len(p.steps) == 2]
    assert plans, "the merged group must hold both matmuls"
    plan = plans[-1]
    assert plan.steps[0].x[0] == "param" and plan.steps[1].x == ("tmp", 0)
    assert (plan.steps[0].N, plan.steps[0].K, plan.steps[1].N, plan.steps[1].K) == (64, 128, 32, 64)
    src = backend.emit_wrapper(plan)
    assert "TVMBackendAllocWorkspace" in src and src.count("b200_q4f16_matmul_dl_family(") == 3   # declaration + 2 calls
    # the chain compiles, links and loads; on CPU tensors the first step reports the device error
    ex = relax.build(mod, target="c")
    vm = relax.VirtualMachine(backend.finalize_modules(ex), tvm.cpu())
    with pytest.raises(Exception, match="not on a CUDA device"):
        vm["main"](*_cpu_args(((3, 128), "float16"), ((64, 16), "uint32"), ((64, 4), "float16"),
                              ((32, 8), "uint32"), ((32, 2), "float16")))
    # without the merge pass the same module gives two offloaded functions
    assert backend.partition_for_b200(chain_module(3, 128, 64, 32)).script().count("call_dps_packed") == 2


def test_symbolic_batch_is_offloaded():
    tvm = backend.import_tvm()
    from tvm import relax

    mod = backend.partition_for_b200(q4_module(None, 64, 128, symbolic_m=True))
    assert offloaded(mod)
    assert backend.codegen.COMPILED[SYMBOL].M is None
    ex = relax.build(mod, target="c")
    vm = relax.VirtualMachine(backend.finalize_modules(ex), tvm.cpu())
    for m in (1, 5):
        with pytest.raises(Exception, match="not on a CUDA device"):
            vm["main"](*_cpu_args(((m, 128), "float16"), ((64, 16), "uint32"), ((64, 4), "float16")))


# ------------------------------------------------------------------------------------ numbers (GPU)
def _gpu_vm(mod):
    tvm = backend.import_tvm()
    from tvm import relax

    ex = relax.build(mod, target="cuda")
    return relax.VirtualMachine(backend.finalize_modules(ex), tvm.cuda(0))


def _on_gpu(*arrays):
    tvm = backend.import_tvm()
    return [tvm.runtime.tensor(a, tvm.cuda(0)) for a in arrays]


@pytest.mark.gpu
@pytest.mark.parametrize("M,N,K,options", [(1, 512, 1024, None), (160, 512, 256, None), (4, 256, 512, {"family": "gemm"})])
def test_relax_vm_runs_the_offloaded_module_on_the_gpu(M, N, K, options):
    import torch

    from relax_b200 import synth
    from util import assert_matmul_close

    vm = _gpu_vm(backend.partition_for_b200(q4_module(M, N, K), options=options))
    x, wq, s = synth.make_case(M, N, K, seed=5)
    y = vm["main"](*_on_gpu(x, wq, s))
    torch.cuda.synchronize()
    assert_matmul_close(y.numpy(), x, wq, s, f"relax vm M={M}")


@pytest.mark.gpu
@pytest.mark.parametrize("M", [1, 40])
def test_relax_vm_on_weights_repacked_offline(M):
    """Weights bound in the paired layout (b200_q4f16_repack): the codegen option names the layout, the VM's
    result is the one of the reference's words."""
    import torch

    from relax_b200 import ops, synth
    from util import assert_matmul_close

    N, K = 512, 1024
    vm = _gpu_vm(backend.partition_for_b200(q4_module(M, N, K), options={"weight_layout": "paired"}))
    x, wq, s = synth.make_case(M, N, K, seed=6)
    packed = ops.q4f16_repack(torch.from_numpy(wq).cuda(), "paired").cpu().numpy()
    y = vm["main"](*_on_gpu(x, packed, s))
    torch.cuda.synchronize()
    assert_matmul_close(y.numpy(), x, wq, s, f"relax vm, paired weights, M={M}")


@pytest.mark.gpu
def test_transposed_layout_decode_on_a_non_symmetric_square_weight():
    """N == K: the shapes cannot tell x . w from x . w^T, only the numbers can."""
    import torch

    from relax_b200 import synth
    from util import assert_matmul_close

    M, N, K = 3, 256, 256
    x, wq, s = synth.make_case(M, N, K, seed=9)
    for kwargs in (dict(transposed=True, layout="nk"), dict(transposed=False, layout="kn")):
        vm = _gpu_vm(backend.partition_for_b200(q4_module(M, N, K, **kwargs)))
        y = vm["main"](*_on_gpu(x, wq, s))
        torch.cuda.synchronize()
        assert_matmul_close(y.numpy(), x, wq, s, f"layout {kwargs}")


@pytest.mark.gpu
def test_merged_chain_and_symbolic_batch_on_the_gpu():
    import torch

    import oracle
    from relax_b200 import synth
    from util import assert_matmul_close, skinny_form_is_unrounded, unrounded_slack

    M, K, N1, N2 = 5, 512, 256, 128
    x, wq1, s1 = synth.make_case(M, N1, K, seed=21)
    _, wq2, s2 = synth.make_case(1, N2, N1, seed=22)
    vm = _gpu_vm(backend.partition_for_b200(chain_module(M, K, N1, N2), merge=True))
    y = vm["main"](*_on_gpu(x, wq1, s1, wq2, s2))
    torch.cuda.synchronize()
    h = oracle.c_matmul(x, wq1, s1)
    # the first layer's output may differ from the oracle's by an fp16 ulp; feed the kernel's own chain
    # through the oracle's second layer with a tolerance for that
    ref = oracle.c_matmul(h, wq2, s2).astype(np.float32)
    w2 = oracle.c_dequantize(wq2, s2).astype(np.float32)
    slack = 2.0 ** -10 * (np.abs(h.astype(np.float32)) @ np.abs(w2).T)
    if skinny_form_is_unrounded(M):
        slack = slack + 20 * unrounded_slack(h, w2)
    err = np.abs(y.numpy().astype(np.float32) - ref)
    assert (err <= 2.0 ** -9 * np.abs(ref) + 0.05 * slack + 1e-4).all(), err.max()
    # one executable, two batch sizes
    vm = _gpu_vm(backend.partition_for_b200(q4_module(None, 256, 512, symbolic_m=True)))
    for m in (1, 40):
        xa, wqa, sa = synth.make_case(m, 256, 512, seed=30 + m)
        ya = vm["main"](*_on_gpu(xa, wqa, sa))
        torch.cuda.synchronize()
        assert ya.numpy().shape == (m, 256)
        assert_matmul_close(ya.numpy(), xa, wqa, sa, f"symbolic batch m={m}")


@pytest.mark.gpu
def test_vm_profiler_names_the_offloaded_function():
    """The VM's profiler reports calls by the callee's name (src/runtime/relax_vm/vm.cc:885-918): the
    offloaded function must show up under its global symbol."""
    from relax_b200 import synth

    tvm = backend.import_tvm()
    from tvm import relax

    mod = backend.partition_for_b200(q4_module(2, 256, 512))
    ex = relax.build(mod, target="cuda")
    vm = relax.VirtualMachine(backend.finalize_modules(ex), tvm.cuda(0), profile=True)
    x, wq, s = synth.make_case(2, 256, 512, seed=3)
    report = vm.profile("main", *_on_gpu(x, wq, s))
    assert SYMBOL in str(report)


@pytest.mark.gpu
def test_relax_vm_calls_the_registered_packed_function_directly():
    import torch

    from relax_b200 import synth
    from relax_b200.backend import tvm_bridge
    from util import assert_matmul_close

    tvm = backend.import_tvm()
    from tvm import relax

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
    yv = vm["main"](*_on_gpu(xa, wqa, sa))
    torch.cuda.synchronize()
    assert_matmul_close(yv.numpy(), xa, wqa, sa, "call_dps_packed")
