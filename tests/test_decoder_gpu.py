"""GPU parity of the decode-step glue kernels and of whole decoder layers against the numpy oracle."""
import numpy as np
import pytest
import torch

import oracle
from oracle import decoder as odec
from relax_b200 import _lib, decoder, synth, tp

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


@pytest.mark.parametrize("B,H", [(1, 4096), (3, 512), (16, 4096), (5, 11008)])
def test_rmsnorm(cuda_lib, B, H):
    rng = np.random.default_rng(B + H)
    x = rng.standard_normal((B, H)).astype(F16)
    d = rng.standard_normal((B, H)).astype(F16)
    w = (1 + 0.1 * rng.standard_normal(H)).astype(F16)
    tx, td, tw = dev(x), dev(d), dev(w)
    ty = torch.empty_like(tx)
    # without and with the fused residual add
    assert cuda_lib.b200_rmsnorm(tx.data_ptr(), None, tw.data_ptr(), ty.data_ptr(), B, H, 1e-5, 0) == 0, _lib.last_error()
    torch.cuda.synchronize()
    close(ty.cpu().numpy(), odec.rmsnorm(x, w, 1e-5), 2e-3, 1e-4, "rmsnorm")
    assert cuda_lib.b200_rmsnorm(tx.data_ptr(), td.data_ptr(), tw.data_ptr(), ty.data_ptr(), B, H, 1e-5, 0) == 0, _lib.last_error()
    torch.cuda.synchronize()
    xs = odec.add_f16(x, d)
    assert (tx.cpu().numpy().view(np.uint16) == xs.view(np.uint16)).all(), "residual stream must be fp16(x + delta) exactly"
    close(ty.cpu().numpy(), odec.rmsnorm(xs, w, 1e-5), 2e-3, 1e-4, "add+rmsnorm")


def test_rmsnorm_rejects_bad_sizes(cuda_lib):
    t = torch.zeros(64, dtype=torch.float16, device="cuda")
    assert cuda_lib.b200_rmsnorm(t.data_ptr(), None, t.data_ptr(), t.data_ptr(), 1, 12, 1e-5, 0) == _lib.EINVAL
    assert cuda_lib.b200_rmsnorm(None, None, t.data_ptr(), t.data_ptr(), 1, 64, 1e-5, 0) == _lib.EINVAL


@pytest.mark.parametrize("B,I", [(1, 11008), (4, 256), (16, 1376)])
def test_silu_mul(cuda_lib, B, I):
    rng = np.random.default_rng(I)
    gu = (2 * rng.standard_normal((B, 2 * I))).astype(F16)
    tg = dev(gu)
    out = torch.empty((B, I), dtype=torch.float16, device="cuda")
    assert cuda_lib.b200_silu_mul(tg.data_ptr(), out.data_ptr(), B, I, 0) == 0, _lib.last_error()
    torch.cuda.synchronize()
    close(out.cpu().numpy(), odec.silu_mul(gu), 2e-3, 1e-4, "silu_mul")


@pytest.mark.parametrize("B,nh,ctx,max_ctx", [(1, 32, 1024, 1024), (2, 4, 1, 64), (3, 8, 129, 300), (1, 2, 2048, 2048)])
def test_rope_append_attention(cuda_lib, B, nh, ctx, max_ctx):
    rng = np.random.default_rng(ctx)
    D = 128
    pos = ctx - 1
    kc = np.zeros((B, max_ctx, nh, D), F16)
    vc = np.zeros((B, max_ctx, nh, D), F16)
    kc[:, :pos] = rng.standard_normal((B, pos, nh, D)).astype(F16)
    vc[:, :pos] = rng.standard_normal((B, pos, nh, D)).astype(F16)
    qkv = rng.standard_normal((B, 3 * nh * D)).astype(F16)
    cos, sin = odec.rope_tables(max_ctx, D)
    tq, tk, tv = dev(qkv), dev(kc), dev(vc)
    tcos, tsin = dev(cos), dev(sin)
    tpos = torch.tensor([pos], dtype=torch.int32, device="cuda")
    q_out = torch.empty((B, nh, D), dtype=torch.float16, device="cuda")
    assert cuda_lib.b200_rope_kv_append(tq.data_ptr(), tcos.data_ptr(), tsin.data_ptr(), tpos.data_ptr(), q_out.data_ptr(),
                                        tk.data_ptr(), tv.data_ptr(), B, nh, max_ctx, 0) == 0, _lib.last_error()
    # oracle
    q = odec.rope(qkv[:, :nh * D].reshape(B, nh, D), cos[pos], sin[pos])
    k = odec.rope(qkv[:, nh * D:2 * nh * D].reshape(B, nh, D), cos[pos], sin[pos])
    kc[:, pos] = k
    vc[:, pos] = qkv[:, 2 * nh * D:].reshape(B, nh, D)
    torch.cuda.synchronize()
    close(q_out.cpu().numpy(), q, 2e-3, 2e-3, "rope q")
    close(tk.cpu().numpy()[:, pos], k, 2e-3, 2e-3, "rope k in cache")
    assert (tv.cpu().numpy()[:, pos].view(np.uint16) == vc[:, pos].view(np.uint16)).all(), "v is copied verbatim"
    assert (tk.cpu().numpy()[:, :pos].view(np.uint16) == kc[:, :pos].view(np.uint16)).all(), "older cache entries untouched"
    # attention over the cache as the kernel left it
    nbytes = cuda_lib.b200_attn_decode_scratch_bytes(B, nh, max_ctx)
    scratch = torch.empty(nbytes // 4, dtype=torch.float32, device="cuda")
    out = torch.empty((B, nh * D), dtype=torch.float16, device="cuda")
    assert cuda_lib.b200_attn_decode(q_out.data_ptr(), tk.data_ptr(), tv.data_ptr(), tpos.data_ptr(), out.data_ptr(),
                                     scratch.data_ptr(), B, nh, max_ctx, 0, 0) == 0, _lib.last_error()
    torch.cuda.synchronize()
    ref = odec.attention_decode(q_out.cpu().numpy(), tk.cpu().numpy(), tv.cpu().numpy(), ctx)
    close(out.cpu().numpy(), ref, 4e-3, 2e-3, "attention")
    # the one-launch form (rotary + append + attention + merge) on fresh copies of the caches, twice in a
    # row through the same scratch (the arrival counters must come back to zero)
    kc0 = kc.copy(); kc0[:, pos] = 0
    vc0 = vc.copy(); vc0[:, pos] = 0
    fbytes = cuda_lib.b200_attn_decode_fused_scratch_bytes(B, nh, max_ctx)
    fscratch = torch.zeros(fbytes // 4, dtype=torch.float32, device="cuda")
    for _ in range(2):
        tk2, tv2 = dev(kc0), dev(vc0)
        out2 = torch.empty((B, nh * D), dtype=torch.float16, device="cuda")
        assert cuda_lib.b200_attn_decode_fused(tq.data_ptr(), tcos.data_ptr(), tsin.data_ptr(), tpos.data_ptr(), tk2.data_ptr(),
                                               tv2.data_ptr(), out2.data_ptr(), fscratch.data_ptr(), B, nh, max_ctx, 0) == 0, _lib.last_error()
        torch.cuda.synchronize()
        close(tk2.cpu().numpy()[:, pos], k, 2e-3, 2e-3, "rotated k appended by the fused kernel")
        assert (tk2.cpu().numpy()[:, :pos].view(np.uint16) == kc[:, :pos].view(np.uint16)).all(), "older cache entries untouched"
        assert (tv2.cpu().numpy().view(np.uint16) == tv.cpu().numpy().view(np.uint16)).all()
        close(out2.cpu().numpy(), ref, 4e-3, 2e-3, "fused attention")
    assert int(fscratch[-B * nh:].view(torch.int32).abs().sum().item()) == 0, "arrival counters are left at zero"
    # the two-launch form: rotary + append + per-chunk attention, then the merge (no counters, scratch not initialised)
    tk3, tv3 = dev(kc0), dev(vc0)
    out3 = torch.empty((B, nh * D), dtype=torch.float16, device="cuda")
    rscratch = torch.full((nbytes // 4,), float("nan"), dtype=torch.float32, device="cuda")
    assert cuda_lib.b200_attn_decode_rope(tq.data_ptr(), tcos.data_ptr(), tsin.data_ptr(), tpos.data_ptr(), tk3.data_ptr(),
                                          tv3.data_ptr(), out3.data_ptr(), rscratch.data_ptr(), B, nh, max_ctx, 0) == 0, _lib.last_error()
    torch.cuda.synchronize()
    close(tk3.cpu().numpy()[:, pos], k, 2e-3, 2e-3, "rotated k appended by the two-launch form")
    assert (tv3.cpu().numpy().view(np.uint16) == tv.cpu().numpy().view(np.uint16)).all()
    close(out3.cpu().numpy(), ref, 4e-3, 2e-3, "two-launch attention")


def test_embed_and_advance(cuda_lib):
    rng = np.random.default_rng(0)
    table = rng.standard_normal((50, 256)).astype(F16)
    ids = np.array([3, 49, 0, 7, 999, -4], dtype=np.int32)       # out-of-range ids are clamped
    tt, ti = dev(table), dev(ids)
    out = torch.empty((6, 256), dtype=torch.float16, device="cuda")
    assert cuda_lib.b200_embed_rows(tt.data_ptr(), ti.data_ptr(), out.data_ptr(), 6, 256, 50, 0) == 0, _lib.last_error()
    pos = torch.tensor([41], dtype=torch.int32, device="cuda")
    assert cuda_lib.b200_advance_pos(pos.data_ptr(), 1, 0) == 0
    torch.cuda.synchronize()
    assert (out.cpu().numpy().view(np.uint16) == table[np.clip(ids, 0, 49)].view(np.uint16)).all()
    assert int(pos.item()) == 42


SMALL = decoder.DecoderConfig(hidden=512, heads=4, inter=768, layers=2, vocab=1000)


def oracle_steps(cfg, layers, embed, final_norm, lm_head, tokens, steps, max_ctx, start_pos=0):
    """Greedy decode with the numpy oracle; returns per-step (hidden after final norm, logits)."""
    B = len(tokens)
    D = cfg.head_dim
    cos, sin = odec.rope_tables(max_ctx, D, cfg.theta)
    kc = [np.zeros((B, max_ctx, cfg.heads, D), F16) for _ in layers]
    vc = [np.zeros((B, max_ctx, cfg.heads, D), F16) for _ in layers]
    out = []
    tok = np.array(tokens)
    for s in range(steps):
        x = embed[tok]
        delta = None
        for i, w in enumerate(layers):
            x, delta = odec.layer_decode(x, delta, w, kc[i], vc[i], start_pos + s, cos, sin, cfg.heads, cfg.eps)
        x = odec.add_f16(x, delta)
        h = odec.rmsnorm(x, final_norm, cfg.eps)
        logits = (h.astype(np.float32) @ lm_head.astype(np.float32).T).astype(F16)
        out.append((h, logits))
        tok = np.argmax(logits.astype(np.float32), axis=1)
    return out


# M = 1 with K <= 4096 takes the one-pass form of the RMSNorm prologue (row kept in registers)
@pytest.mark.parametrize("M,N,K", [(1, 512, 1024), (1, 4096, 4096), (1, 272, 2304), (1, 128, 8192), (3, 300, 4096), (16, 64, 256),
                                   (8, 4096, 2816)])
def test_gemv_with_fused_neighbours(cuda_lib, M, N, K, gemv_form):
    from relax_b200 import synth
    from util import assert_matmul_close, skinny_form_is_unrounded, unrounded_slack

    rng = np.random.default_rng(M * N + K)
    _, wq, s = synth.make_case(1, N, K, seed=K + M)
    twq, ts = dev(wq), dev(s)
    # RMSNorm (+ residual add) prologue
    x = rng.standard_normal((M, K)).astype(F16)
    d = rng.standard_normal((M, K)).astype(F16)
    w = (1 + 0.1 * rng.standard_normal(K)).astype(F16)
    tx, td, tw = dev(x), dev(d), dev(w)
    x_out = torch.full((M, K), float("nan"), dtype=torch.float16, device="cuda")
    y = torch.empty((M, N), dtype=torch.float16, device="cuda")
    for delta in (None, td):
        assert cuda_lib.b200_q4f16_gemv_rmsnorm(tx.data_ptr(), delta.data_ptr() if delta is not None else None, tw.data_ptr(),
                                                x_out.data_ptr(), 1e-5, twq.data_ptr(), ts.data_ptr(), y.data_ptr(), M, N, K, 0) == 0, _lib.last_error()
        torch.cuda.synchronize()
        r = odec.add_f16(x, d) if delta is not None else x
        assert (x_out.cpu().numpy().view(np.uint16) == r.view(np.uint16)).all(), "updated residual stream"
        a = odec.rmsnorm(r, w, 1e-5)
        # the activation may differ from the oracle's by one fp16 ulp (rsqrt vs 1/sqrt): compare against
        # the matmul of the oracle's activation with a tolerance that covers one ulp per element
        ref = oracle.c_matmul(a, wq, s).astype(np.float32)
        wd = oracle.c_dequantize(wq, s).astype(np.float32)
        slack = 2.0 ** -10 * (np.abs(a.astype(np.float32)) @ np.abs(wd).T)
        if skinny_form_is_unrounded(M):
            slack = slack + 20 * unrounded_slack(a, wd)
        err = np.abs(y.cpu().numpy().astype(np.float32) - ref)
        assert (err <= 2.0 ** -9 * np.abs(ref) + 0.05 * slack + 1e-4).all(), f"gemv_rmsnorm: max err {err.max()}"
    # aliasing x_out with x is refused
    assert cuda_lib.b200_q4f16_gemv_rmsnorm(tx.data_ptr(), None, tw.data_ptr(), tx.data_ptr(), 1e-5, twq.data_ptr(), ts.data_ptr(),
                                            y.data_ptr(), M, N, K, 0) == _lib.EINVAL
    # SwiGLU prologue
    gu = (1.5 * rng.standard_normal((M, 2 * K))).astype(F16)
    tg = dev(gu)
    assert cuda_lib.b200_q4f16_gemv_swiglu(tg.data_ptr(), twq.data_ptr(), ts.data_ptr(), y.data_ptr(), M, N, K, 0) == 0, _lib.last_error()
    torch.cuda.synchronize()
    a = odec.silu_mul(gu)
    ref = oracle.c_matmul(a, wq, s).astype(np.float32)
    wd = oracle.c_dequantize(wq, s).astype(np.float32)
    slack = 2.0 ** -10 * (np.abs(a.astype(np.float32)) @ np.abs(wd).T)
    if skinny_form_is_unrounded(M):
        slack = slack + 20 * unrounded_slack(a, wd)
    err = np.abs(y.cpu().numpy().astype(np.float32) - ref)
    assert (err <= 2.0 ** -9 * np.abs(ref) + 0.05 * slack + 1e-4).all(), f"gemv_swiglu: max err {err.max()}"
    assert cuda_lib.b200_device_error_flags() == 0


@pytest.mark.parametrize("fused", [False, True, "layer"])
@pytest.mark.parametrize("B", [1, 3])
def test_decoder_steps_match_oracle(cuda_lib, B, fused):
    # "layer": the one-persistent-kernel-per-layer path (batch 1)
    layer_kernel = fused == "layer"
    if layer_kernel and B != 1:
        pytest.skip("the layer kernel is the batch-1 path")
    fused = bool(fused)
    cfg = SMALL
    rng = np.random.default_rng(11)
    layers = [decoder.synth_layer_numpy(cfg, 100 + i) for i in range(cfg.layers)]
    embed = (0.5 * rng.standard_normal((cfg.vocab, cfg.hidden))).astype(F16)
    final_norm = np.ones(cfg.hidden, F16)
    lm_head = (0.05 * rng.standard_normal((cfg.vocab, cfg.hidden))).astype(F16)
    tokens = list(rng.integers(0, cfg.vocab, B))
    max_ctx, steps = 32, 3
    ref = oracle_steps(cfg, layers, embed, final_norm, lm_head, tokens, steps, max_ctx)

    shards = [decoder.to_device(tp.shard_layer(l, 0, 1, cfg.hidden, cfg.inter), "cuda") for l in layers]
    eng = decoder.DecodeEngine(cfg, shards, dev(embed), dev(final_norm), dev(lm_head), B, max_ctx, "cuda", fused=fused,
                               layer_kernel=layer_kernel)
    assert eng.fused == fused and eng.layer_kernel == layer_kernel
    eng.tokens.copy_(torch.tensor(tokens, dtype=torch.int32))
    for s in range(steps):
        # feed the oracle's token choice so that a near-tie in the logits cannot fork the two runs
        if s > 0:
            eng.tokens.copy_(torch.from_numpy(np.argmax(ref[s - 1][1].astype(np.float32), axis=1).astype(np.int32)))
        eng.step()
        torch.cuda.synchronize()
        h = eng.h.cpu().numpy()
        scale = np.abs(ref[s][0].astype(np.float32)).max()
        close(h, ref[s][0], 1e-2, 1e-2 * scale, f"hidden state at step {s}")
        lscale = np.abs(ref[s][1].astype(np.float32)).max()
        close(eng.logits.cpu().numpy(), ref[s][1], 1e-2, 1e-2 * lscale, f"logits at step {s}")
    assert int(eng.pos.item()) == steps
    assert cuda_lib.b200_device_error_flags() == 0


def test_decoder_graph_replay_matches_eager(cuda_lib):
    cfg = SMALL
    rng = np.random.default_rng(5)
    layers = [decoder.to_device(tp.shard_layer(decoder.synth_layer_numpy(cfg, 7 + i), 0, 1, cfg.hidden, cfg.inter), "cuda")
              for i in range(cfg.layers)]
    embed = dev((0.5 * rng.standard_normal((cfg.vocab, cfg.hidden))).astype(F16))
    lm_head = dev((0.05 * rng.standard_normal((cfg.vocab, cfg.hidden))).astype(F16))
    fn = dev(np.ones(cfg.hidden, F16))
    runs = []
    for use_graph in (False, True):
        eng = decoder.DecodeEngine(cfg, layers, embed, fn, lm_head, 2, 16, "cuda")
        eng.tokens.copy_(torch.tensor([5, 900], dtype=torch.int32))
        stream = torch.cuda.Stream()
        if use_graph:
            eng.capture(stream)
        toks = []
        with torch.cuda.stream(stream):
            for _ in range(4):
                eng.graph.replay() if use_graph else eng.step()
                stream.synchronize()
                toks.append(eng.tokens.cpu().numpy().copy())
        runs.append((toks, eng.logits.cpu().numpy().copy(), int(eng.pos.item())))
    assert runs[0][2] == runs[1][2] == 4
    for a, b in zip(runs[0][0], runs[1][0]):
        assert (a == b).all()
    assert (runs[0][1].view(np.uint16) == runs[1][1].view(np.uint16)).all(), "graph replay must reproduce the eager step bit for bit"


@pytest.mark.parametrize("B,V,H", [(1, 32000, 4096), (3, 1000, 512), (8, 4099, 1024), (9, 2048, 4096), (16, 32000, 4096), (2, 17, 32)])
def test_lm_head_matches_oracle(cuda_lib, B, V, H):
    """Output projection over an fp16 table: fp32 accumulation of exact products, one rounding to fp16 (the
    reference's matmul + astype), and the greedy token = first maximum of the fp16 logits."""
    rng = np.random.default_rng(B * 7 + V + H)
    h = (0.5 * rng.standard_normal((B, H))).astype(np.float16)
    w = (0.05 * rng.standard_normal((V, H))).astype(np.float16)
    if V > 40:
        w[V - 1] = w[7]                      # an exact tie between two rows: the lower index must win
    th, tw = torch.from_numpy(h).cuda(), torch.from_numpy(w).cuda()
    nbytes = cuda_lib.b200_lm_head_scratch_bytes()
    assert nbytes > 0
    scr = torch.zeros(nbytes // 4, dtype=torch.float32, device="cuda")
    canary = 64
    buf = torch.full((B * V + canary,), float("nan"), dtype=torch.float16, device="cuda")
    toks = torch.full((B + 2,), -5, dtype=torch.int32, device="cuda")
    for rep in range(2):                     # twice: the scratch counter must come back to zero by itself
        assert cuda_lib.b200_lm_head(th.data_ptr(), tw.data_ptr(), buf.data_ptr(), toks.data_ptr(), scr.data_ptr(), B, V, H,
                                     1000, 0) == 0, _lib.last_error()
        torch.cuda.synchronize()
        logits = buf[:B * V].view(B, V).cpu().numpy()
        assert torch.isnan(buf[B * V:]).all() and (toks[B:] == -5).all()
        ref32 = h.astype(np.float32) @ w.astype(np.float32).T
        absdot = np.abs(h.astype(np.float32)) @ np.abs(w.astype(np.float32)).T
        err = np.abs(logits.astype(np.float64) - ref32.astype(np.float64))
        assert (err <= 2.0 ** -10 * np.abs(ref32) + 8e-6 * absdot + 2.0 ** -24).all(), err.max()
        want = np.argmax(logits.astype(np.float32), axis=1) + 1000      # numpy: first occurrence of the maximum
        assert (toks[:B].cpu().numpy() == want).all(), (toks[:B].cpu().numpy(), want)
    # logits only, tokens only
    buf.fill_(float("nan"))
    assert cuda_lib.b200_lm_head(th.data_ptr(), tw.data_ptr(), buf.data_ptr(), None, None, B, V, H, 0, 0) == 0
    toks.fill_(-5)
    assert cuda_lib.b200_lm_head(th.data_ptr(), tw.data_ptr(), None, toks.data_ptr(), scr.data_ptr(), B, V, H, 0, 0) == 0
    torch.cuda.synchronize()
    assert (buf[:B * V].view(B, V).cpu().numpy().view(np.uint16) == logits.view(np.uint16)).all()
    assert (toks[:B].cpu().numpy() == want - 1000).all()


def test_lm_head_argument_checks(cuda_lib):
    t = torch.zeros(64 * 32, dtype=torch.float16, device="cuda")
    p = t.data_ptr()
    L = cuda_lib
    assert L.b200_lm_head(p, p, p, None, None, 17, 4, 32, 0, 0) == _lib.EINVAL and "16 rows" in _lib.last_error()
    assert L.b200_lm_head(p, p, p, None, None, 1, 4, 48, 0, 0) == _lib.EINVAL
    assert L.b200_lm_head(p, p, None, None, None, 1, 4, 32, 0, 0) == _lib.EINVAL
    assert L.b200_lm_head(p, p, None, p, None, 1, 4, 32, 0, 0) == _lib.EINVAL and "scratch" in _lib.last_error()
    assert L.b200_lm_head(p + 2, p, p, None, None, 1, 4, 32, 0, 0) == _lib.EINVAL
    assert L.b200_lm_head(p, p, p, None, None, 16, 4, 65536, 0, 0) == _lib.EINVAL and "shared memory" in _lib.last_error()


@pytest.mark.parametrize("nh,K,with_delta", [(32, 4096, True), (4, 4096, False), (2, 8192, True), (12, 3584, True)])
def test_qkv_matmul_with_rotary_epilogue_equals_the_two_kernels(cuda_lib, nh, K, with_delta):
    """b200_q4f16_gemv_rmsnorm_rope against b200_q4f16_gemv_rmsnorm followed by b200_rope_kv_append: the same
    arithmetic, so the rotated query, the cache slot of the new token and the updated residual stream agree bit
    for bit; nothing else in the caches is touched."""
    N, max_ctx, pos = 3 * nh * 128, 24, 17
    rng = np.random.default_rng(nh + K)
    x, wq, s = synth.make_case(1, N, K, seed=nh * 3 + 1)
    delta = (0.1 * rng.standard_normal((1, K))).astype(np.float16)
    norm = (1.0 + 0.1 * rng.standard_normal(K)).astype(np.float16)
    tx, twq, ts, td, tn = (dev(a) for a in (x, wq, s, delta, norm))
    dptr = td.data_ptr() if with_delta else None
    cos, sin = decoder.rope_tables(max_ctx, 128, 10000.0, "cuda")
    tpos = torch.tensor([pos], dtype=torch.int32, device="cuda")
    fill = torch.from_numpy(rng.standard_normal((max_ctx, nh, 128)).astype(np.float16)).cuda()
    out = {}
    for name in ("two", "one"):
        kc, vc = fill.clone(), (fill * 0.5).clone()
        q = torch.zeros(nh * 128, dtype=torch.float16, device="cuda")
        xo = torch.zeros(1, K, dtype=torch.float16, device="cuda")
        if name == "two":
            qkv = torch.zeros(1, N, dtype=torch.float16, device="cuda")
            assert cuda_lib.b200_q4f16_gemv_rmsnorm(tx.data_ptr(), dptr, tn.data_ptr(), xo.data_ptr(), 1e-5, twq.data_ptr(),
                                                    ts.data_ptr(), qkv.data_ptr(), 1, N, K, 0) == 0, _lib.last_error()
            assert cuda_lib.b200_rope_kv_append(qkv.data_ptr(), cos.data_ptr(), sin.data_ptr(), tpos.data_ptr(), q.data_ptr(),
                                                kc.data_ptr(), vc.data_ptr(), 1, nh, max_ctx, 0) == 0, _lib.last_error()
        else:
            rc = cuda_lib.b200_q4f16_gemv_rmsnorm_rope(tx.data_ptr(), dptr, tn.data_ptr(), xo.data_ptr(), 1e-5, twq.data_ptr(),
                                                       ts.data_ptr(), cos.data_ptr(), sin.data_ptr(), tpos.data_ptr(),
                                                       q.data_ptr(), kc.data_ptr(), vc.data_ptr(), nh, K, 0)
            assert rc == 0, (rc, _lib.last_error())
        torch.cuda.synchronize()
        out[name] = [t.cpu().numpy().view(np.uint16) for t in (q, kc, vc, xo)]
    for a, b, what in zip(out["one"], out["two"], ("q", "k cache", "v cache", "x_out")):
        assert np.array_equal(a, b), what
    assert cuda_lib.b200_device_error_flags() == 0
    # the exact form has another epilogue layout: the entry point says so and launches nothing
    _lib.set_option("gemv.exact", 1)
    try:
        q = torch.zeros(nh * 128, dtype=torch.float16, device="cuda")
        rc = cuda_lib.b200_q4f16_gemv_rmsnorm_rope(tx.data_ptr(), dptr, tn.data_ptr(), None, 1e-5, twq.data_ptr(), ts.data_ptr(),
                                                   cos.data_ptr(), sin.data_ptr(), tpos.data_ptr(), q.data_ptr(),
                                                   fill.data_ptr(), fill.data_ptr(), nh, K, 0)
        assert rc == _lib.ENOTREADY
    finally:
        _lib.set_option("gemv.exact", 0)
