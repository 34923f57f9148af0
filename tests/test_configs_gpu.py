"""GPU parity at the sizes the benchmark configurations name: the full-size decoder layer (config 3), the
shapes the 7B decode step really runs through the fused-prologue kernels (also the tensor-parallel K
slices), the 70B-shaped sweep (config 5), the batch-64 engine, and two ordering / failure contracts of the
C ABI.  Everything goes through the C ABI and is checked against the CPU oracle."""
import ctypes

import numpy as np
import pytest
import torch

import oracle
from oracle import decoder as odec
from relax_b200 import _lib, decoder, ops, synth, tp
from util import assert_matmul_close, skinny_form_is_unrounded, unrounded_slack

pytestmark = pytest.mark.gpu

F16 = np.float16


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def close(a, b, rtol, atol, what):
    a = np.asarray(a, dtype=np.float64)
    b = np.asarray(b, dtype=np.float64)
    err = np.abs(a - b)
    bound = atol + rtol * np.abs(b)
    i = np.argmax(err - bound)
    assert (err <= bound).all(), f"{what}: |a-b|={err.ravel()[i]:.3e} > {bound.ravel()[i]:.3e} (a={a.ravel()[i]}, b={b.ravel()[i]})"


def prologue_bound(a, wq, s, ref):
    """|y - ref| allowed when the activation `a` fed to the matmul may differ from the oracle's by one fp16 ulp
    per element (rsqrt against 1/sqrt, __expf against exp)."""
    wd = oracle.c_dequantize(wq, s).astype(np.float32)
    slack = 2.0 ** -10 * (np.abs(a.astype(np.float32)) @ np.abs(wd).T)
    if skinny_form_is_unrounded(a.shape[0]):
        slack = slack + 20 * unrounded_slack(a, wd)       # (0.05 * 20 = one times the fast form's own slack)
    return 2.0 ** -9 * np.abs(ref) + 0.05 * slack + 1e-4


# ------------------------------------------------------------------------------ config 3: one full-size layer
@pytest.mark.parametrize("fused", [True, False, "layer"])
def test_full_size_decoder_layer_matches_oracle(cuda_lib, fused):
    """hidden 4096, 32 heads x 128, SwiGLU 11008, eps 1e-5, theta 10000, fp16 KV cache of length 1024 ~N(0,1),
    batch 1: the residual stream after attention, the MLP output and the appended cache rows against
    oracle.decoder.layer_decode."""
    cfg = decoder.DecoderConfig(hidden=4096, heads=32, inter=11008, layers=1, vocab=64)
    ctx = 1024
    pos = ctx - 1
    w = decoder.synth_layer_numpy(cfg, 31)
    rng = np.random.default_rng(32)
    x = rng.standard_normal((1, cfg.hidden)).astype(F16)
    kc = np.zeros((1, ctx, cfg.heads, 128), F16)
    vc = np.zeros((1, ctx, cfg.heads, 128), F16)
    kc[:, :pos] = rng.standard_normal((1, pos, cfg.heads, 128)).astype(F16)
    vc[:, :pos] = rng.standard_normal((1, pos, cfg.heads, 128)).astype(F16)
    cos, sin = odec.rope_tables(ctx, 128, cfg.theta)
    kc_ref, vc_ref = kc.copy(), vc.copy()
    x_ref, down_ref = odec.layer_decode(x, None, w, kc_ref, vc_ref, pos, cos, sin, cfg.heads, cfg.eps)

    shard = decoder.to_device(tp.shard_layer(w, 0, 1, cfg.hidden, cfg.inter), "cuda")
    embed = torch.zeros((cfg.vocab, cfg.hidden), dtype=torch.float16, device="cuda")
    layer_kernel = fused == "layer"          # the layer as one persistent kernel
    eng = decoder.DecodeEngine(cfg, [shard], embed, torch.ones(cfg.hidden, dtype=torch.float16, device="cuda"), None, 1, ctx,
                               "cuda", fused=bool(fused), layer_kernel=layer_kernel)
    assert eng.fused == bool(fused) and eng.layer_kernel == layer_kernel
    eng.kc[0].copy_(dev(kc))
    eng.vc[0].copy_(dev(vc))
    eng.x.copy_(dev(x))
    eng.set_position(pos)
    sp = torch.cuda.current_stream().cuda_stream
    if layer_kernel:
        assert cuda_lib.b200_decode_layer(ctypes.byref(eng.layer_desc[0]), sp) == 0, _lib.last_error()
        down = eng.down
        eng.x = eng.x_last
    else:
        down = eng.layer_step(0, None, sp)
    torch.cuda.synchronize()
    assert cuda_lib.b200_device_error_flags() == 0
    xs = np.abs(x_ref.astype(np.float32)).max()
    ds = np.abs(down_ref.astype(np.float32)).max()
    close(eng.x.cpu().numpy(), x_ref, 1e-2, 1e-2 * xs, "residual stream after attention")
    close(down.cpu().numpy(), down_ref, 1e-2, 1e-2 * ds, "MLP output")
    close(eng.kc[0].cpu().numpy()[:, pos], kc_ref[:, pos], 1e-2, 1e-2 * np.abs(kc_ref[:, pos].astype(np.float32)).max(), "appended keys")
    close(eng.vc[0].cpu().numpy()[:, pos], vc_ref[:, pos], 1e-2, 1e-2 * np.abs(vc_ref[:, pos].astype(np.float32)).max(), "appended values")
    assert (eng.kc[0].cpu().numpy()[:, :pos].view(np.uint16) == kc[:, :pos].view(np.uint16)).all(), "older cache entries untouched"


# ------------------------------------------------------------------------------ the shapes the 7B step runs
# RMSNorm prologue: q|k|v (N = 12288) and gate|up (N = 22016) at K = 4096, batch 1 and 16
@pytest.mark.parametrize("M,N,K", [(1, 12288, 4096), (16, 12288, 4096), (1, 22016, 4096), (16, 22016, 4096),
                                   (1, 1536, 4096), (1, 3072, 4096), (1, 2560, 4096)])   # ... and their 8-way tensor-parallel shards
def test_rmsnorm_prologue_at_decoder_shapes(cuda_lib, M, N, K, gemv_form):
    rng = np.random.default_rng(M * 7 + N)
    _, wq, s = synth.make_case(1, N, K, seed=N + M)
    twq, ts = dev(wq), dev(s)
    x = rng.standard_normal((M, K)).astype(F16)
    d = rng.standard_normal((M, K)).astype(F16)
    w = (1 + 0.02 * rng.standard_normal(K)).astype(F16)
    tx, td, tw = dev(x), dev(d), dev(w)
    x_out = torch.full((M, K), float("nan"), dtype=torch.float16, device="cuda")
    y = torch.empty((M, N), dtype=torch.float16, device="cuda")
    assert cuda_lib.b200_q4f16_gemv_rmsnorm(tx.data_ptr(), td.data_ptr(), tw.data_ptr(), x_out.data_ptr(), 1e-5, twq.data_ptr(),
                                            ts.data_ptr(), y.data_ptr(), M, N, K, 0) == 0, _lib.last_error()
    torch.cuda.synchronize()
    r = odec.add_f16(x, d)
    assert (x_out.cpu().numpy().view(np.uint16) == r.view(np.uint16)).all(), "updated residual stream"
    a = odec.rmsnorm(r, w, 1e-5)
    ref = oracle.c_matmul(a, wq, s).astype(np.float32)
    err = np.abs(y.cpu().numpy().astype(np.float32) - ref)
    assert (err <= prologue_bound(a, wq, s, ref)).all(), f"max err {err.max()}"
    assert cuda_lib.b200_device_error_flags() == 0


# SwiGLU prologue: the down projection (N = 4096) at the full K and at every K slice a rank gets under 2-, 4- and
# 8-way tensor parallelism (11008 = 43 blocks of 256, cut into whole blocks: 5632 / 5376, 2816 / 2560, 1536 / 1280)
@pytest.mark.parametrize("K", [11008, 5632, 5376, 2816, 2560, 1536, 1280])
@pytest.mark.parametrize("M", [1, 16])
def test_swiglu_prologue_at_decoder_shapes(cuda_lib, M, K, gemv_form):
    N = 4096
    rng = np.random.default_rng(M + K)
    _, wq, s = synth.make_case(1, N, K, seed=K + M)
    gu = (1.5 * rng.standard_normal((M, 2 * K))).astype(F16)
    y = torch.empty((M, N), dtype=torch.float16, device="cuda")
    twq, ts, tg = dev(wq), dev(s), dev(gu)
    assert cuda_lib.b200_q4f16_gemv_swiglu(tg.data_ptr(), twq.data_ptr(), ts.data_ptr(), y.data_ptr(), M, N, K, 0) == 0, _lib.last_error()
    torch.cuda.synchronize()
    a = odec.silu_mul(gu)
    ref = oracle.c_matmul(a, wq, s).astype(np.float32)
    err = np.abs(y.cpu().numpy().astype(np.float32) - ref)
    assert (err <= prologue_bound(a, wq, s, ref)).all(), f"max err {err.max()}"
    assert cuda_lib.b200_device_error_flags() == 0


# ------------------------------------------------------------------------------ config 5: 70B-shaped sweep
@pytest.mark.parametrize("N", [1280, 3584, 1024])           # 10240, 28672, 8192 sharded 8 ways
@pytest.mark.parametrize("M", [1, 16, 128, 2048])
def test_70b_shaped_sweep(cuda_lib, M, N):
    K = 8192
    x, wq, s = synth.make_case(M, N, K, seed=M + N)
    y = ops.q4f16_matmul(dev(x), dev(wq), dev(s))
    torch.cuda.synchronize()
    assert cuda_lib.b200_device_error_flags() == 0
    yh = y.cpu().numpy()
    assert yh.shape == (M, N)
    if M <= 128:
        assert_matmul_close(yh, x, wq, s, f"70B shard M={M} N={N}")
    else:
        # every output depends on one row of x and one row of W only: a sample of both is an exact check
        rng = np.random.default_rng(N)
        toks = np.sort(rng.choice(M, 96, replace=False))
        rows = np.sort(rng.choice(N, 256, replace=False))
        assert_matmul_close(yh[np.ix_(toks, rows)], x[toks], wq[rows], s[rows], f"70B shard M={M} N={N} (sample)")
        assert np.isfinite(yh.astype(np.float32)).all()


# ------------------------------------------------------------------------------ batch 64: the unfused engine
def test_batch_64_engine_matches_oracle(cuda_lib):
    """Batch 64 is outside the skinny kernel's range: RMSNorm / SwiGLU as their own kernels and the
    mid-batch tensor-core matmul.  Two steps at a small configuration against the oracle."""
    from test_decoder_gpu import oracle_steps

    cfg = decoder.DecoderConfig(hidden=512, heads=4, inter=768, layers=2, vocab=1000)
    B, max_ctx, steps = 64, 16, 2
    rng = np.random.default_rng(64)
    layers = [decoder.synth_layer_numpy(cfg, 300 + i) for i in range(cfg.layers)]
    embed = (0.5 * rng.standard_normal((cfg.vocab, cfg.hidden))).astype(F16)
    final_norm = np.ones(cfg.hidden, F16)
    lm_head = (0.05 * rng.standard_normal((cfg.vocab, cfg.hidden))).astype(F16)
    tokens = list(rng.integers(0, cfg.vocab, B))
    ref = oracle_steps(cfg, layers, embed, final_norm, lm_head, tokens, steps, max_ctx)
    shards = [decoder.to_device(tp.shard_layer(l, 0, 1, cfg.hidden, cfg.inter), "cuda") for l in layers]
    eng = decoder.DecodeEngine(cfg, shards, dev(embed), dev(final_norm), dev(lm_head), B, max_ctx, "cuda")
    assert not eng.fused, "batch 64 must take the unfused path"
    eng.tokens.copy_(torch.tensor(tokens, dtype=torch.int32))
    for st in range(steps):
        if st > 0:
            eng.tokens.copy_(torch.from_numpy(np.argmax(ref[st - 1][1].astype(np.float32), axis=1).astype(np.int32)))
        eng.step()
        torch.cuda.synchronize()
        scale = np.abs(ref[st][0].astype(np.float32)).max()
        close(eng.h.cpu().numpy(), ref[st][0], 1e-2, 1e-2 * scale, f"hidden state at step {st}")
        lscale = np.abs(ref[st][1].astype(np.float32)).max()
        close(eng.logits.cpu().numpy(), ref[st][1], 1e-2, 1e-2 * lscale, f"logits at step {st}")
    assert cuda_lib.b200_device_error_flags() == 0


# ------------------------------------------------------------------------------ ordering contract of the attention
def test_attention_after_a_matmul_after_a_position_writer(cuda_lib):
    """advance_pos -> skinny matmul (produces q) -> attention, back to back 200 times with no host
    synchronisation.  The matmul releases its dependents before it has waited for the position writer, so an
    attention that read *pos before its own wait could see the old position.  With flags = 0 it must not:
    every iteration has to equal, bit for bit, the same sequence run with a synchronisation after every launch."""
    L = cuda_lib
    nh, max_ctx, K = 8, 512, 1024
    iters, pos0 = 200, 100
    g = torch.Generator(device="cuda")
    g.manual_seed(5)
    kc = torch.randn((1, max_ctx, nh, 128), device="cuda", generator=g).to(torch.float16)
    vc = torch.randn((1, max_ctx, nh, 128), device="cuda", generator=g).to(torch.float16)
    x = torch.randn((1, K), device="cuda", generator=g).to(torch.float16)
    wq, s = synth.make_weights_torch(nh * 128, K, 77, "cuda")
    scratch = torch.empty(L.b200_attn_decode_scratch_bytes(1, nh, max_ctx) // 4, dtype=torch.float32, device="cuda")

    def run(serialised):
        pos = torch.tensor([pos0], dtype=torch.int32, device="cuda")
        q = torch.zeros((1, nh * 128), dtype=torch.float16, device="cuda")
        outs = torch.zeros((iters, nh * 128), dtype=torch.float16, device="cuda")
        torch.cuda.synchronize()
        sp = torch.cuda.current_stream().cuda_stream
        for i in range(iters):
            assert L.b200_advance_pos(pos.data_ptr(), 1, sp) == 0
            if serialised:
                torch.cuda.synchronize()
            assert L.b200_q4f16_gemv(x.data_ptr(), wq.data_ptr(), s.data_ptr(), q.data_ptr(), 1, nh * 128, K, sp) == 0, _lib.last_error()
            if serialised:
                torch.cuda.synchronize()
            assert L.b200_attn_decode(q.data_ptr(), kc.data_ptr(), vc.data_ptr(), pos.data_ptr(), outs[i].data_ptr(),
                                      scratch.data_ptr(), 1, nh, max_ctx, 0, sp) == 0, _lib.last_error()
            if serialised:
                torch.cuda.synchronize()
        torch.cuda.synchronize()
        assert int(pos.item()) == pos0 + iters
        return outs.cpu().numpy()

    want = run(True)
    got = run(False)
    # positions differ from iteration to iteration, so a stale position changes the result
    assert not (want[0].view(np.uint16) == want[1].view(np.uint16)).all()
    bad = np.flatnonzero((got.view(np.uint16) != want.view(np.uint16)).any(axis=1))
    assert bad.size == 0, f"iterations {bad[:8]} differ from the serialised run"
    # and the first iteration is the oracle's attention at position pos0 + 1
    qh = oracle.c_matmul(x.cpu().numpy(), wq.cpu().numpy().view(np.uint32), s.cpu().numpy())
    ref = odec.attention_decode(qh.reshape(1, nh, 128), kc.cpu().numpy(), vc.cpu().numpy(), pos0 + 2)
    close(want[0:1], ref, 4e-3, 2e-3, "attention at the first iteration")
    assert L.b200_attn_decode(None, kc.data_ptr(), vc.data_ptr(), kc.data_ptr(), kc.data_ptr(), scratch.data_ptr(), 1, nh, max_ctx, 6, 0) == _lib.EINVAL


# ------------------------------------------------------------------------------ bounded wait of the fused sum over ranks
def test_peer_wait_runs_out_without_hanging(cuda_lib):
    """The row-parallel matmul with the fused sum over ranks, told that there are two ranks whose buffers both
    live on this GPU, with rank 1 never publishing its flag: the bounded wait (set to 20 ms for the test) must
    run out, the kernel must finish and still write `out`, the error word must read 16 once, and the next
    ordinary call must work."""
    L = cuda_lib
    M, N, K = 1, 512, 1024
    x, wq, s = synth.make_case(M, N, K, seed=16)
    tx, twq, ts = dev(x), dev(wq), dev(s)
    y0 = torch.zeros((M, N), dtype=torch.float16, device="cuda")          # this rank's partial result
    y1 = torch.zeros((M, N), dtype=torch.float16, device="cuda")          # "rank 1": stays zero, never published
    flags = torch.zeros(16, dtype=torch.int32, device="cuda")
    epoch = torch.zeros(1, dtype=torch.int32, device="cuda")
    done = torch.zeros(1, dtype=torch.int32, device="cuda")
    out = torch.full((M, N), float("nan"), dtype=torch.float16, device="cuda")
    d = _lib.PeerReduce()
    d.world, d.rank = 2, 0
    d.peer_y[0], d.peer_y[1] = y0.data_ptr(), y1.data_ptr()
    d.peer_flags[0], d.peer_flags[1] = flags.data_ptr(), flags.data_ptr() + 32     # rank 1's own flag array: never read here
    d.flag_base, d.epoch, d.done_counter, d.out = 0, epoch.data_ptr(), done.data_ptr(), out.data_ptr()
    assert L.b200_device_error_flags() == 0
    try:
        _lib.set_option("gemv.peer_wait_ms", 20)
        rc = L.b200_q4f16_gemv_allreduce(tx.data_ptr(), twq.data_ptr(), ts.data_ptr(), y0.data_ptr(), M, N, K, 0, ctypes.byref(d), 0)
        assert rc == 0, _lib.last_error()
        torch.cuda.synchronize()                                             # returns: nothing hangs
    finally:
        _lib.set_option("gemv.peer_wait_ms", 2000)
    assert L.b200_device_error_flags() == 16, "the wait that ran out must be reported"
    assert L.b200_device_error_flags() == 0, "reading the error word clears it"
    assert int(done.item()) == 0
    # out = y0 + 0 was still written
    assert_matmul_close(out.cpu().numpy(), x, wq, s, "out after the wait ran out")
    # a normal call afterwards
    y = ops.q4f16_matmul(tx, twq, ts)
    torch.cuda.synchronize()
    assert_matmul_close(y.cpu().numpy(), x, wq, s, "call after the failure")
    assert L.b200_device_error_flags() == 0


# ------------------------------------------------------------------------------ the layer kernel's own contracts
def _small_layer_engine(layers=2, max_ctx=16):
    cfg = decoder.DecoderConfig(hidden=512, heads=4, inter=768, layers=layers, vocab=100)
    rng = np.random.default_rng(77)
    shards = [decoder.to_device(tp.shard_layer(decoder.synth_layer_numpy(cfg, 400 + i), 0, 1, cfg.hidden, cfg.inter), "cuda")
              for i in range(cfg.layers)]
    embed = dev((0.5 * rng.standard_normal((cfg.vocab, cfg.hidden))).astype(F16))
    fn = dev(np.ones(cfg.hidden, F16))
    return cfg, shards, embed, fn


@pytest.mark.parametrize("ctas", [1, 3, 40])
def test_layer_kernel_on_small_grids_matches_the_seven_launch_engine(cuda_lib, ctas):
    """Few CTAs: every CTA takes many tiles of every matmul and many attention units, the weight ring wraps
    many times and runs across the stage boundaries.  Results must equal the seven-launch engine's bit for bit
    (same arithmetic, same summation order inside a tile) for four steps."""
    cfg, shards, embed, fn = _small_layer_engine()
    outs = []
    for layer_kernel in (False, True):
        eng = decoder.DecodeEngine(cfg, shards, embed, fn, embed, 1, 16, "cuda", layer_kernel=layer_kernel)
        eng.tokens.copy_(torch.tensor([7], dtype=torch.int32))
        hs = []
        try:
            if layer_kernel:
                _lib.set_option("layer.max_ctas", ctas)
            for _ in range(4):
                eng.step()
                torch.cuda.synchronize()
                hs.append(eng.h.cpu().numpy().copy())
        finally:
            _lib.set_option("layer.max_ctas", 0)
        outs.append(hs)
        assert cuda_lib.b200_device_error_flags() == 0
    for a, b in zip(*outs):
        err = np.abs(a.astype(np.float32) - b.astype(np.float32)).max() / np.abs(a.astype(np.float32)).max()
        assert err < 2e-3, err


def test_layer_kernel_wait_runs_out_without_hanging(cuda_lib):
    """A stage counter that can never reach its target (the step scalar says 5 decode steps have passed, the
    counters say none): with the wait limit set to 5 ms every CTA's first wait must run out, the kernel must
    run through and end, the error word must report it (bit 5 of the layer kernel's byte), and after the
    scratch is brought back in step an ordinary run must work."""
    cfg, shards, embed, fn = _small_layer_engine(layers=1)
    eng = decoder.DecodeEngine(cfg, shards, embed, fn, embed, 1, 16, "cuda", layer_kernel=True)
    eng.tokens.copy_(torch.tensor([3], dtype=torch.int32))
    sp = torch.cuda.current_stream().cuda_stream
    assert cuda_lib.b200_device_error_flags() == 0
    try:
        _lib.set_option("layer.wait_ms", 5)
        _lib.set_option("layer.max_ctas", 4)
        eng.epoch.fill_(5)
        assert cuda_lib.b200_decode_layer(ctypes.byref(eng.layer_desc[0]), sp) == 0, _lib.last_error()
        torch.cuda.synchronize()                                  # returns: nothing hangs
    finally:
        _lib.set_option("layer.wait_ms", 2000)
        _lib.set_option("layer.max_ctas", 0)
    flags = cuda_lib.b200_device_error_flags()
    assert (flags >> 24) & 32, hex(flags)
    assert cuda_lib.b200_device_error_flags() == 0
    # back in step: zero counters, step 0
    eng.epoch.zero_()
    eng.layer_scratch[0].zero_()
    eng.set_position(0)
    ref = decoder.DecodeEngine(cfg, shards, embed, fn, embed, 1, 16, "cuda", layer_kernel=False)
    for e in (eng, ref):
        e.tokens.copy_(torch.tensor([3], dtype=torch.int32))
        e.step()
    torch.cuda.synchronize()
    assert cuda_lib.b200_device_error_flags() == 0
    a, b = eng.h.float().cpu().numpy(), ref.h.float().cpu().numpy()
    assert np.abs(a - b).max() / np.abs(b).max() < 2e-3
