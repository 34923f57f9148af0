"""Compile check of the C++ sources meant for the reference tree (relax_b200/tvm_plugin/src/...): each file
is placed at its intended path inside a shadow of the tree (real directories along that path, everything
else symlinked to the tree), so that its relative includes resolve exactly as they would after the drop-in,
and run through ``g++ -std=c++17 -fsyntax-only`` against the tree's own headers.  The submodule headers the
tree does not carry (dlpack, dmlc-core) come from the installed tvm_ffi and tilelang wheels.

The tree is looked for in $B200_RELAX_TREE, then in a directory named ``reference`` beside the repository;
without one the test is skipped.
"""
import os
import shutil
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PLUGIN = os.path.join(ROOT, "relax_b200", "tvm_plugin")
SOURCES = [
    "src/relax/backend/contrib/b200/codegen.cc",
    "src/runtime/contrib/b200/b200_packed.cc",
]


def _tree():
    for cand in (os.environ.get("B200_RELAX_TREE"), os.path.join(os.path.dirname(ROOT), "reference")):
        if cand and os.path.isdir(os.path.join(cand, "include", "tvm", "relax")) and os.path.isdir(os.path.join(cand, "src", "relax")):
            return cand
    return None


def _wheel_includes():
    out = []
    try:
        import tvm_ffi

        out.append(os.path.join(os.path.dirname(tvm_ffi.__file__), "include"))          # dlpack/dlpack.h
    except ImportError:
        pass
    try:
        import importlib.util

        spec = importlib.util.find_spec("tilelang")
        if spec and spec.submodule_search_locations:
            out.append(os.path.join(list(spec.submodule_search_locations)[0], "3rdparty", "tvm", "3rdparty", "dmlc-core", "include"))
    except ImportError:
        pass
    return [p for p in out if os.path.isdir(p)]


def _shadow(tree, rel_dir, dst):
    """dst/rel_dir as real directories; every other entry met on the way is a symlink into `tree`."""
    cur_tree, cur_dst = tree, dst
    os.makedirs(cur_dst, exist_ok=True)
    for part in rel_dir.split("/"):
        if cur_tree is not None:
            for name in os.listdir(cur_tree):
                link = os.path.join(cur_dst, name)
                if name != part and not os.path.lexists(link):
                    os.symlink(os.path.join(cur_tree, name), link)
            nxt = os.path.join(cur_tree, part)
            cur_tree = nxt if os.path.isdir(nxt) else None
        cur_dst = os.path.join(cur_dst, part)
        os.makedirs(cur_dst, exist_ok=True)
    if cur_tree is not None:
        for name in os.listdir(cur_tree):
            link = os.path.join(cur_dst, name)
            if not os.path.lexists(link):
                os.symlink(os.path.join(cur_tree, name), link)
    return cur_dst


@pytest.mark.parametrize("rel", SOURCES)
def test_plugin_source_compiles_against_the_reference_headers(rel, tmp_path):
    tree = _tree()
    if tree is None:
        pytest.skip("no Relax source tree available (set B200_RELAX_TREE)")
    wheels = _wheel_includes()
    if len(wheels) < 2 or shutil.which("g++") is None:
        pytest.skip("dlpack / dmlc headers or g++ not available")
    dst_dir = _shadow(tree, os.path.dirname(rel), str(tmp_path / "tree"))
    dst = os.path.join(dst_dir, os.path.basename(rel))
    shutil.copy(os.path.join(PLUGIN, rel), dst)
    cmd = ["g++", "-std=c++17", "-fsyntax-only", "-DDMLC_USE_LOGGING_LIBRARY=<tvm/runtime/logging.h>", "-DTVM_USE_LIBBACKTRACE=0",
           "-I" + os.path.join(tree, "include"), *("-I" + w for w in wheels), "-I" + os.path.join(ROOT, "include")]
    cuda_inc = "/usr/local/cuda/include"
    if os.path.isdir(cuda_inc):
        cmd.append("-I" + cuda_inc)          # cuda_common.h of the tree includes cuda_runtime.h
    r = subprocess.run(cmd + [dst], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-4000:]


def test_plugin_cmake_lists_both_source_directories():
    text = open(os.path.join(PLUGIN, "cmake", "modules", "contrib", "B200.cmake")).read()
    for rel in SOURCES:
        assert os.path.dirname(rel) + "/*.cc" in text
