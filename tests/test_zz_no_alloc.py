"""The attention entry point that brings its own scratch memory (for callers that may not
allocate on the device) must give exactly what the caller-scratch entry point gives, call after
call.  Collected last on purpose: a failure here cannot hide the other tests' results."""
import numpy as np
import pytest
import torch

from relax_b200 import _lib

pytestmark = pytest.mark.gpu


def _inputs(B, nh, max_ctx, seed):
    g = torch.Generator(device="cuda")
    g.manual_seed(seed)
    q = torch.randn((B, nh, 128), device="cuda", generator=g).to(torch.float16)
    kc = torch.randn((B, max_ctx, nh, 128), device="cuda", generator=g).to(torch.float16)
    vc = torch.randn((B, max_ctx, nh, 128), device="cuda", generator=g).to(torch.float16)
    return q, kc, vc


def _run(L, fn_static, B, nh, ctx, max_ctx, seed):
    q, kc, vc = _inputs(B, nh, max_ctx, seed)
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


def _close_to_oracle(got, q, kc, vc, ctx, what):
    from oracle import decoder as odec

    ref = odec.attention_decode(q.cpu().numpy(), kc.cpu().numpy(), vc.cpu().numpy(), ctx).astype(np.float64)
    err = np.abs(got.astype(np.float64) - ref)
    bound = 2e-3 + 4e-3 * np.abs(ref)                 # the tolerance of the other attention tests
    assert (err <= bound).all(), f"{what}: max err {err.max():.3e}"


def test_static_scratch_attention_matches_the_oracle(cuda_lib):
    """Against the CPU oracle itself (not only against the sibling entry point), two calls in a row."""
    for (B, nh, ctx, max_ctx, seed) in ((2, 8, 700, 1024, 3), (1, 4, 129, 256, 4)):
        q, kc, vc = _inputs(B, nh, max_ctx, seed)
        got = _run(cuda_lib, True, B, nh, ctx, max_ctx, seed)
        _close_to_oracle(got, q, kc, vc, ctx, f"B={B} nh={nh} ctx={ctx}")


def test_static_scratch_attention_at_its_documented_maximum(cuda_lib):
    """16 sequences x 32 heads x 2048 tokens = exactly the 8192 partial results the built-in array holds:
    accepted, and right up to the last slot (sampled sequences against the oracle, all of them against the
    caller-scratch entry point)."""
    B, nh, max_ctx, ctx, seed = 16, 32, 2048, 2048, 8
    want = _run(cuda_lib, False, B, nh, ctx, max_ctx, seed)
    got = _run(cuda_lib, True, B, nh, ctx, max_ctx, seed)
    assert (got.view(np.uint16) == want.view(np.uint16)).all()
    q, kc, vc = _inputs(B, nh, max_ctx, seed)
    for b in (0, B - 1):                                # the first and the last sequence (the last slots of the array)
        _close_to_oracle(got[b:b + 1], q[b:b + 1], kc[b:b + 1], vc[b:b + 1], ctx, f"sequence {b} at the maximum size")
    # one more chunk does not fit
    t = torch.zeros(8, dtype=torch.float16, device="cuda")
    assert cuda_lib.b200_attn_decode_static(t.data_ptr(), t.data_ptr(), t.data_ptr(), t.data_ptr(), t.data_ptr(), B, nh,
                                            max_ctx + 1, 0, 0) == _lib.EINVAL


def test_static_scratch_attention_rejects_oversize(cuda_lib):
    t = torch.zeros(8, dtype=torch.float16, device="cuda")
    # 64 sequences x 32 heads x 16 chunks = 32768 partial results > 8192: refused before any launch
    rc = cuda_lib.b200_attn_decode_static(t.data_ptr(), t.data_ptr(), t.data_ptr(), t.data_ptr(), t.data_ptr(), 64, 32, 2048, 0, 0)
    assert rc == _lib.EINVAL
    assert "8192" in _lib.last_error()
