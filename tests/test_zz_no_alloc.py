"""The attention entry point that brings its own scratch memory (for callers that may not
allocate on the device) must give exactly what the caller-scratch entry point gives, call after
call.  Collected last on purpose: a failure here cannot hide the other tests' results."""
import numpy as np
import pytest
import torch

from relax_b200 import _lib

pytestmark = pytest.mark.gpu


def _run(L, fn_static, B, nh, ctx, max_ctx, seed):
    g = torch.Generator(device="cuda")
    g.manual_seed(seed)
    q = torch.randn((B, nh, 128), device="cuda", generator=g).to(torch.float16)
    kc = torch.randn((B, max_ctx, nh, 128), device="cuda", generator=g).to(torch.float16)
    vc = torch.randn((B, max_ctx, nh, 128), device="cuda", generator=g).to(torch.float16)
    pos = torch.tensor([ctx - 1], dtype=torch.int32, device="cuda")
    out = torch.full((B, nh * 128), float("nan"), dtype=torch.float16, device="cuda")
    if fn_static:
        rc = L.b200_attn_decode_static(q.data_ptr(), kc.data_ptr(), vc.data_ptr(), pos.data_ptr(), out.data_ptr(), B, nh, max_ctx, 0, 0)
    else:
        scratch = torch.empty(L.b200_attn_decode_scratch_bytes(B, nh, max_ctx) // 4, dtype=torch.float32, device="cuda")
        rc = L.b200_attn_decode(q.data_ptr(), kc.data_ptr(), vc.data_ptr(), pos.data_ptr(), out.data_ptr(), scratch.data_ptr(),
                                B, nh, max_ctx, 0, 0)
    assert rc == 0, _lib.last_error()
    torch.cuda.synchronize()
    return out.cpu().numpy()


def test_static_scratch_attention_matches_caller_scratch(cuda_lib):
    L = cuda_lib
    # two different problems back to back through the shared built-in scratch: the second call must
    # not see anything of the first (a longer context first, then a shorter one)
    for (B, nh, ctx, max_ctx, seed) in ((2, 8, 1000, 1024, 1), (3, 4, 130, 512, 2)):
        want = _run(L, False, B, nh, ctx, max_ctx, seed)
        got = _run(L, True, B, nh, ctx, max_ctx, seed)
        assert np.isfinite(got.astype(np.float32)).all()
        # same kernels, same inputs, only the scratch buffer differs: bit-identical
        assert (got.view(np.uint16) == want.view(np.uint16)).all()


def test_static_scratch_attention_rejects_oversize(cuda_lib):
    t = torch.zeros(8, dtype=torch.float16, device="cuda")
    # 64 sequences x 32 heads x 16 chunks = 32768 partial results > 8192: refused before any launch
    rc = cuda_lib.b200_attn_decode_static(t.data_ptr(), t.data_ptr(), t.data_ptr(), t.data_ptr(), t.data_ptr(), 64, 32, 2048, 0, 0)
    assert rc == _lib.EINVAL
    assert "8192" in _lib.last_error()
