"""Offline weight repack (b200_q4f16_repack / _unpack) and the kernels that consume the repacked order.

The permutation is checked bit for bit against the oracle's nibble-by-nibble statement of it, the round trip
restores the reference's words exactly, and every kernel family fed the repacked words gives what it gives
on the reference's words: the decode bit for bit, the matmuls against the CPU oracle with the bounds of the
other parity tests (and bit for bit where the kernel's arithmetic does not depend on the order inside a word)."""
import os

import numpy as np
import pytest
import torch

import oracle
from relax_b200 import _lib, ops, synth, weights_io
from util import assert_bits_equal, assert_matmul_close

pytestmark = pytest.mark.gpu


def dev(*arrs):
    return [torch.from_numpy(np.ascontiguousarray(a)).cuda() for a in arrs]


@pytest.mark.parametrize("n,k", [(1, 32), (3, 96), (257, 1056), (4096, 4096), (1000, 11008)])
def test_repack_matches_oracle_and_round_trips(cuda_lib, n, k):
    _, wq, _ = synth.make_case(1, n, k, seed=7 * n + k)
    (twq,) = dev(wq.view(np.int32))
    packed = ops.q4f16_repack(twq, "paired")
    assert (packed.cpu().numpy().view(np.uint32) == oracle.repack_paired(wq)).all()
    back = ops.q4f16_unpack(packed, "paired")
    assert (back.cpu().numpy().view(np.uint32) == wq).all()
    # in place, and the identity layout
    ops.q4f16_repack(twq, "paired", out=twq)
    assert (twq.cpu().numpy().view(np.uint32) == oracle.repack_paired(wq)).all()
    ops.q4f16_unpack(twq, "paired", out=twq)
    assert (twq.cpu().numpy().view(np.uint32) == wq).all()
    assert (ops.q4f16_repack(twq, "reference").cpu().numpy().view(np.uint32) == wq).all()


def test_repack_unaligned_views_and_every_word_pattern(cuda_lib):
    # words that exercise every nibble position with every value, through buffers that are only 4-byte aligned
    q = np.zeros((16 * 8, 8), np.uint8)
    for pos in range(8):
        for v in range(16):
            q[pos * 16 + v, pos] = v
            q[pos * 16 + v, (pos + 3) % 8] = 15 - v
    wq = oracle.pack_nibbles(q.reshape(1, -1))          # [1, 128] words
    buf_in = torch.zeros(wq.size + 3, dtype=torch.int32, device="cuda")
    buf_out = torch.zeros(wq.size + 3, dtype=torch.int32, device="cuda")
    buf_in[1:1 + wq.size] = torch.from_numpy(wq.view(np.int32).ravel()).cuda()
    src = buf_in[1:1 + wq.size].view(1, -1)
    dst = buf_out[1:1 + wq.size].view(1, -1)
    ops.q4f16_repack(src, "paired", out=dst)
    assert (dst.cpu().numpy().view(np.uint32) == oracle.repack_paired(wq)).all()
    assert int(buf_out[0]) == 0 and int(buf_out[-2]) == 0 and int(buf_out[-1]) == 0
    ops.q4f16_unpack(dst, "paired", out=dst)
    assert (dst.cpu().numpy().view(np.uint32) == wq).all()


def test_repack_argument_checks(cuda_lib):
    L = cuda_lib
    t = torch.zeros(64, dtype=torch.int32, device="cuda")
    p = t.data_ptr()
    assert L.b200_q4f16_repack(p, p, 2, 256, 7, None) == _lib.EINVAL and "layout" in _lib.last_error()
    assert L.b200_q4f16_repack(p, p, 2, 40, 1, None) == _lib.EINVAL
    assert L.b200_q4f16_repack(None, p, 2, 256, 1, None) == _lib.EINVAL
    assert L.b200_q4f16_repack(p, p + 16, 2, 256, 1, None) == _lib.EINVAL and "overlap" in _lib.last_error()
    assert L.b200_q4f16_unpack(p, p, 0, 256, 1, None) == 0
    assert L.b200_set_option(b"weights.layout", 2) == _lib.EINVAL
    x = torch.zeros(1, 256, dtype=torch.float16, device="cuda")
    assert L.b200_q4f16_matmul_layout(x.data_ptr(), p, p, p, 1, 2, 256, 9, None) == _lib.EINVAL


@pytest.mark.parametrize("n,k", [(3, 96), (4096, 4096), (1000, 11008)])
def test_dequantize_of_repacked_weights_bit_exact(cuda_lib, n, k):
    _, wq, s = synth.make_case(1, n, k, seed=n + 3 * k)
    twq, ts = dev(wq, s)
    packed = ops.q4f16_repack(twq, "paired")
    out = ops.q4f16_dequantize(packed, ts, layout="paired").cpu().numpy()
    assert_bits_equal(out, oracle.c_dequantize(wq, s), f"decode of repacked {n}x{k}")


# every kernel family, through the per-call layout of the DLPack entry point and through the process-wide option
CASES = [(1, 4096, 4096), (1, 22016, 4096), (1, 4096, 11008), (4, 1024, 1536), (16, 4096, 4096), (16, 1000, 2080),
         (64, 4096, 4096), (128, 1280, 8192), (300, 1024, 512), (2048, 1280, 1024)]


@pytest.mark.parametrize("m,n,k", CASES)
def test_matmul_on_repacked_weights(cuda_lib, gemv_form, m, n, k):
    if m > 16 and gemv_form == "exact":
        pytest.skip("the exact form only concerns the skinny kernel")
    x, wq, s = synth.make_case(m, n, k, seed=m + n + k)
    tx, twq, ts = dev(x, wq, s)
    packed = ops.q4f16_repack(twq, "paired")
    y_ref_layout = ops.q4f16_matmul(tx, twq, ts)
    y = ops.q4f16_matmul(tx, packed, ts, layout="paired")
    assert_matmul_close(y.cpu().numpy(), x, wq, s, f"paired {m}x{n}x{k}")
    if m > 16:
        # the tensor-core kernels write the same dequantised tile whatever the order inside the packed word
        assert_bits_equal(y.cpu().numpy(), y_ref_layout.cpu().numpy(), f"paired vs reference {m}x{n}x{k}")
    # the process-wide option reaches the raw-pointer entry points
    y2 = torch.empty_like(y)
    _lib.set_option("weights.layout", _lib.LAYOUT_PAIRED)
    try:
        assert _lib.get_option("weights.layout") == _lib.LAYOUT_PAIRED
        rc = cuda_lib.b200_q4f16_matmul(tx.data_ptr(), packed.data_ptr(), ts.data_ptr(), y2.data_ptr(), m, n, k, None)
        assert rc == 0, _lib.last_error()
        torch.cuda.synchronize()
    finally:
        _lib.set_option("weights.layout", _lib.LAYOUT_REFERENCE)
    assert_bits_equal(y2.cpu().numpy(), y.cpu().numpy(), "option vs per-call layout")
    assert cuda_lib.b200_device_error_flags() == 0


def test_one_hot_rows_bit_exact_on_repacked_weights(cuda_lib, gemv_form):
    # x = e_j picks column j of the dequantised matrix: the result must be that fp16 value exactly, for every
    # position inside a word (a misplaced nibble shows at once)
    n, k = 64, 512
    _, wq, s = synth.make_case(1, n, k, seed=11)
    w = oracle.c_dequantize(wq, s)
    js = [0, 1, 2, 3, 4, 5, 6, 7, 8, 37, 250, 511]
    x = np.zeros((len(js), k), np.float16)
    for r, j in enumerate(js):
        x[r, j] = 1.0
    tx, twq, ts = dev(x, wq, s)
    packed = ops.q4f16_repack(twq, "paired")
    y = ops.q4f16_matmul(tx, packed, ts, layout="paired").cpu().numpy()
    for r, j in enumerate(js):
        assert_bits_equal(y[r], w[:, j], f"column {j}")
    for fam in ("gemm", "gemm_ws"):
        yf = ops.q4f16_matmul(tx, packed, ts, family=fam, layout="paired").cpu().numpy()
        for r, j in enumerate(js):
            assert_bits_equal(yf[r], w[:, j], f"{fam} column {j}")


def test_fused_decoder_kernels_on_repacked_weights(cuda_lib):
    """The fused skinny entry points and the layer kernel read the process-wide layout: a two-layer decoder on
    repacked weights reproduces the one on the reference's words."""
    from relax_b200 import decoder, tp

    cfg = decoder.DecoderConfig(hidden=512, heads=4, inter=768, layers=2, vocab=256)
    rng = np.random.default_rng(5)
    full = [decoder.synth_layer_numpy(cfg, 20 + i) for i in range(cfg.layers)]
    embed = torch.from_numpy((0.5 * rng.standard_normal((cfg.vocab, cfg.hidden))).astype(np.float16)).cuda()
    fnorm = torch.ones(cfg.hidden, dtype=torch.float16, device="cuda")
    outs = {}
    for name, layout, layer_kernel in (("ref", "reference", False), ("paired", "paired", False), ("paired-layer", "paired", True)):
        layers = [decoder.to_device(tp.shard_layer(l, 0, 1, cfg.hidden, cfg.inter), "cuda") for l in full]
        if layout == "paired":
            for l in layers:
                for key in ("qkv", "o", "gu", "down"):
                    ops.q4f16_repack(l[key][0], "paired", out=l[key][0])
        _lib.set_option("weights.layout", ops.LAYOUTS[layout])
        try:
            eng = decoder.DecodeEngine(cfg, layers, embed, fnorm, embed, 1, 16, torch.device("cuda"), layer_kernel=layer_kernel)
            eng.tokens.copy_(torch.tensor([5], dtype=torch.int32))
            hs = []
            for _ in range(3):
                eng.step()
                torch.cuda.synchronize()
                hs.append(eng.h.float().cpu().numpy().copy())
                eng.tokens.copy_(torch.tensor([9], dtype=torch.int32))
        finally:
            _lib.set_option("weights.layout", _lib.LAYOUT_REFERENCE)
        outs[name] = hs
        assert cuda_lib.b200_device_error_flags() == 0
    for name in ("paired", "paired-layer"):
        for a, b in zip(outs[name], outs["ref"]):
            assert np.abs(a - b).max() <= 1e-2 * np.abs(b).max(), name


def test_weight_file_repack_round_trip(cuda_lib, tmp_path):
    _, wq1, s1 = synth.make_case(1, 48, 256, seed=1)
    _, wq2, s2 = synth.make_case(1, 16, 1056, seed=2)
    src, dst, back = (str(tmp_path / f) for f in ("a.b2q4", "b.b2q4", "c.b2q4"))
    weights_io.save(src, {"qkv": (wq1, s1), "down": (wq2, s2)})
    weights_io.repack_file(src, dst, "paired")
    layout, tensors = weights_io.load(dst)
    assert layout == "paired" and list(tensors) == ["qkv", "down"]
    assert (tensors["qkv"][0] == oracle.repack_paired(wq1)).all() and (tensors["down"][0] == oracle.repack_paired(wq2)).all()
    assert_bits_equal(tensors["down"][1], s2)
    weights_io.repack_file(dst, back, "reference")
    with open(src, "rb") as f1, open(back, "rb") as f2:
        assert f1.read() == f2.read()
    assert os.path.getsize(dst) == os.path.getsize(src)
