import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (run with -m gpu on the GPU box)")


@pytest.fixture(scope="session")
def golden():
    import numpy as np

    return np.load(os.path.join(ROOT, "tests", "golden", "q4f16_relax_vm.npz"))


@pytest.fixture(scope="session")
def cuda_lib():
    """The C-ABI library on a GPU box; fails (never skips) when it is missing or unusable there."""
    import torch

    from relax_b200 import _lib

    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    return _lib.lib()


@pytest.fixture(params=["fast", "exact"])
def gemv_form(request, cuda_lib):
    """Runs a test under both arithmetic forms of the skinny kernel: the default one (group scale applied to
    fp32 group sums) and the exact one (every weight rounded to fp16 first, option gemv.exact)."""
    from relax_b200 import _lib

    # 2 forces the fast form for every K (the default, 0, picks the exact form where K fills its stages poorly)
    _lib.set_option("gemv.exact", 1 if request.param == "exact" else 2)
    yield request.param
    _lib.set_option("gemv.exact", 0)
