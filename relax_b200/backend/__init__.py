"""Host-side mirror of the reference's BYOC plugin surface for the q4f16 path.

``patterns``   the pattern table and the structural check of the decode PrimFunc  (reference:
               python/tvm/relax/dpl/pattern.py:1049-1095 builders, python/tvm/contrib/cutlass/build.py
               for a backend's Python half)
``codegen``    the ``relax.ext.b200`` callee, which returns C-source modules (reference:
               src/relax/backend/contrib/cutlass/codegen.cc:248-270; calling convention
               src/relax/transform/run_codegen.cc:158-163)
``partition_for_b200``  FuseOpsByPattern (+ MergeCompositeFunctions) + RunCodegen
``finalize_modules``    export_library with the kernel library linked in, then load_module

These run against a TVM that has Relax (here: the TVM 0.23 bundled with the tilelang wheel, the
only importable member of the reference's lineage); the C++ equivalents for the reference tree
itself live in relax_b200/tvm_plugin/.
"""
from .tvm_bridge import have_tvm, import_tvm  # noqa: F401
from .patterns import canonical_decode_te, classify_decode, decode_layouts, q4f16_matmul_patterns  # noqa: F401
from .codegen import (  # noqa: F401
    B200CodegenError,
    analyze_composite,
    analyze_function,
    b200_codegen,
    emit_wrapper,
    finalize_modules,
    link_options,
    partition_for_b200,
    register_codegen,
    validate_decodes,
)
