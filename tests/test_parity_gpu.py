"""GPU parity tests: the CUDA kernels, called through the C ABI, against the CPU oracle."""
import ctypes

import numpy as np
import pytest
import torch

import oracle
import relax_b200
from relax_b200 import _lib, ops, synth
from util import assert_bits_equal, assert_matmul_close, golden_cases

pytestmark = pytest.mark.gpu


def dev(*arrs):
    return [torch.from_numpy(np.ascontiguousarray(a)).cuda() for a in arrs]


# ------------------------------------------------------------------------------ decode
def test_dequantize_golden_bit_exact(cuda_lib, golden):
    for name, x, wq, s, w, y in golden_cases(golden):
        twq, ts = dev(wq, s)
        out = ops.q4f16_dequantize(twq, ts)
        assert_bits_equal(out.cpu().numpy(), w, name)


@pytest.mark.parametrize("n,k", [(1, 32), (3, 96), (257, 1056), (4096, 4096), (1000, 11008)])
def test_dequantize_bit_exact_random(cuda_lib, n, k):
    _, wq, s = synth.make_case(1, n, k, seed=n + k)
    twq, ts = dev(wq, s)
    out = ops.q4f16_dequantize(twq, ts).cpu().numpy()
    assert_bits_equal(out, oracle.c_dequantize(wq, s), f"decode {n}x{k}")


def test_dequantize_all_scale_bit_patterns(cuda_lib):
    # every finite fp16 scale (both signs, subnormals included) times every nibble value
    bits = np.arange(0x10000, dtype=np.uint32)
    bits = bits[(bits & 0x7C00) != 0x7C00].astype(np.uint16)      # drop inf/nan
    n = bits.size
    s = bits.view(np.float16).reshape(n, 1)
    q = np.tile(np.arange(16, dtype=np.uint8), 2)[None, :].repeat(n, axis=0)
    wq = oracle.pack_nibbles(q)
    twq, ts = dev(wq, s)
    out = ops.q4f16_dequantize(twq, ts).cpu().numpy()
    assert_bits_equal(out, oracle.c_dequantize(wq, s), "all scales x all nibbles")


def test_dequantize_empty(cuda_lib):
    twq = torch.zeros((0, 16), dtype=torch.uint32, device="cuda")
    ts = torch.zeros((0, 4), dtype=torch.float16, device="cuda")
    assert ops.q4f16_dequantize(twq, ts).shape == (0, 128)


# ------------------------------------------------------------------------------ skinny matmul
def run_matmul(x, wq, s, family="auto"):
    tx, twq, ts = dev(x, wq, s)
    # canary-padded output: the kernel must write exactly M*N values
    m, n = x.shape[0], wq.shape[0]
    buf = torch.full((m * n + 64,), float("nan"), dtype=torch.float16, device="cuda")
    out = buf[: m * n].view(m, n)
    ops.q4f16_matmul(tx, twq, ts, out=out, family=family)
    torch.cuda.synchronize()
    assert torch.isnan(buf[m * n:]).all(), "kernel wrote past the end of y"
    return out.cpu().numpy()


def test_gemv_golden(cuda_lib, golden, gemv_form):
    for name, x, wq, s, w, y in golden_cases(golden):
        out = run_matmul(x, wq, s)
        assert_matmul_close(out, x, wq, s, name, y_ref=y)


@pytest.mark.parametrize("m", list(range(1, 17)))
def test_gemv_every_m(cuda_lib, m, gemv_form):
    x, wq, s = synth.make_case(m, 300, 1024, seed=m)
    assert_matmul_close(run_matmul(x, wq, s), x, wq, s, f"M={m}")


@pytest.mark.parametrize("n,k", [(1, 32), (15, 32), (16, 64), (17, 96), (33, 224), (100, 256), (129, 288),
                                 (4096, 4096), (11008, 4096), (4096, 11008), (1280, 8192), (1024, 1376)])
@pytest.mark.parametrize("m", [1, 3, 8, 16])
def test_gemv_shapes(cuda_lib, m, n, k, gemv_form):
    x, wq, s = synth.make_case(m, n, k, seed=7 * n + k + m)
    assert_matmul_close(run_matmul(x, wq, s), x, wq, s, f"M={m} N={n} K={k}")


def test_gemv_known_answers(cuda_lib, gemv_form):
    k, n = 256, 48
    rng = np.random.default_rng(5)
    s = rng.uniform(0.005, 0.02, (n, k // 32)).astype(np.float16)
    x = rng.standard_normal((2, k)).astype(np.float16)
    for fill in (0x00000000, 0xFFFFFFFF, 0x77777777):   # all -7*s, all 8*s, all zero weights
        wq = np.full((n, k // 8), fill, dtype=np.uint32)
        out = run_matmul(x, wq, s)
        assert_matmul_close(out, x, wq, s, f"fill {fill:#x}")
    # one-hot x picks out single dequantised weights exactly (no summation involved)
    q = rng.integers(0, 16, (n, k), dtype=np.uint8)
    wq = oracle.pack_nibbles(q)
    for pos in (0, 5, 31, 32, 100, k - 1):
        xo = np.zeros((1, k), np.float16)
        xo[0, pos] = 1.0
        out = run_matmul(xo, wq, s)
        assert_bits_equal(out[0], oracle.c_dequantize(wq, s)[:, pos], f"one-hot at {pos}")


@pytest.mark.parametrize("variant", [1, 2])
@pytest.mark.parametrize("m,n,k", [(1, 4096, 4096), (1, 100, 256), (2, 37, 1280), (4, 4096, 11008), (7, 333, 2304),
                                   (8, 2000, 11008), (13, 500, 4096), (16, 4096, 4096), (16, 1280, 8192),
                                   (16, 700, 11008), (16, 20000, 2048)])
def test_gemv_both_kernels(cuda_lib, variant, m, n, k, gemv_form):
    x, wq, s = synth.make_case(m, n, k, seed=n + k + m)
    try:
        relax_b200.set_option("gemv.variant", variant)
        out = run_matmul(x, wq, s, family="gemv")
    finally:
        relax_b200.set_option("gemv.variant", 0)
    assert_matmul_close(out, x, wq, s, f"variant={variant} M={m} N={n} K={k}")
    assert cuda_lib.b200_device_error_flags() == 0


@pytest.mark.parametrize("stages", [2, 3, 8, 16])
def test_gemv_pipeline_depths(cuda_lib, stages, gemv_form):
    x, wq, s = synth.make_case(3, 5000, 4096, seed=stages)
    try:
        relax_b200.set_option("gemv.stages", stages)
        out = run_matmul(x, wq, s, family="gemv")
    finally:
        relax_b200.set_option("gemv.stages", 0)
    assert_matmul_close(out, x, wq, s, f"stages={stages}")
    assert cuda_lib.b200_device_error_flags() == 0


def test_gemv_back_to_back_dependent_launches(cuda_lib, gemv_form):
    # a chain y1 = W1 x, y2 = W2 y1, ... launched back to back: each launch may start (and
    # prefetch its weights) before the previous one has finished, but must not read x early
    n = k = 1024
    rng = np.random.default_rng(3)
    ws = [synth.make_weights(n, k, rng) for _ in range(6)]
    x0 = (rng.standard_normal((1, k)) * 0.5).astype(np.float16)
    dws = [dev(wq, s) for wq, s in ws]
    bufs = [torch.from_numpy(x0).cuda()] + [torch.empty((1, n), dtype=torch.float16, device="cuda") for _ in ws]
    for i, (twq, ts) in enumerate(dws):
        ops.q4f16_matmul(bufs[i], twq, ts, out=bufs[i + 1], family="gemv")
    torch.cuda.synchronize()
    ref = x0
    for i, (wq, s) in enumerate(ws):
        got = bufs[i + 1].cpu().numpy()
        assert_matmul_close(got, ref, wq, s, f"chain step {i}")
        ref = got          # feed the kernel's own output forward so each step is checked in isolation
    assert cuda_lib.b200_device_error_flags() == 0


def test_gemv_warp_counts_agree(cuda_lib):
    x, wq, s = synth.make_case(4, 500, 2048, seed=11)
    try:
        for w in (1, 2, 4, 8, 16):
            relax_b200.set_option("gemv.warps", w)
            relax_b200.set_option("gemv.variant", 1)
            assert_matmul_close(run_matmul(x, wq, s, family="gemv"), x, wq, s, f"warps={w}")
    finally:
        relax_b200.set_option("gemv.warps", 0)
        relax_b200.set_option("gemv.variant", 0)


def test_matmul_k_zero_and_empty(cuda_lib):
    x = torch.zeros((3, 0), dtype=torch.float16, device="cuda")  # K == 0: the empty sum
    wq = torch.zeros((5, 0), dtype=torch.uint32, device="cuda")
    s = torch.zeros((5, 0), dtype=torch.float16, device="cuda")
    y = torch.full((3, 5), 7.0, dtype=torch.float16, device="cuda")
    ops.q4f16_matmul(x, wq, s, out=y)
    assert (y == 0).all()
    x = torch.zeros((0, 64), dtype=torch.float16, device="cuda")
    wq = torch.zeros((5, 8), dtype=torch.uint32, device="cuda")
    s = torch.zeros((5, 2), dtype=torch.float16, device="cuda")
    assert ops.q4f16_matmul(x, wq, s).shape == (0, 5)


def test_packed_entry_point_runs_on_device(cuda_lib):
    x, wq, s = synth.make_case(2, 64, 128, seed=2)
    tx, twq, ts = dev(x, wq, s)
    ty = torch.empty((2, 64), dtype=torch.float16, device="cuda")
    views = [ops.to_dltensor(t) for t in (tx, twq, ts, ty)]
    vals = (ctypes.c_void_p * 4)(*[ctypes.addressof(v.tensor) for v in views])
    codes = (ctypes.c_int * 4)(7, 13, 7, 7)
    out_code = ctypes.c_int(-1)
    cuda_lib.b200_set_stream(torch.cuda.current_stream().cuda_stream)
    rc = cuda_lib.b200_q4f16_matmul_packed(vals, codes, 4, None, ctypes.byref(out_code), None)
    assert rc == 0, _lib.last_error()
    assert out_code.value == 4
    torch.cuda.synchronize()
    assert_matmul_close(ty.cpu().numpy(), x, wq, s, "packed")


@pytest.mark.parametrize("m,n,k,pinned", [
    (4, 256, 512, True),        # pinned host buffers: the transfers run as kernels over the mapped buffers
    (4, 256, 512, False),       # pageable host buffers: copy-engine transfers
    (1, 4096, 4096, True),      # the benchmark shape
    (3, 1001, 256, True),       # result size that is not a multiple of 16 bytes
    (300, 512, 512, True),      # activations above the kernel-transfer limit, result below it
    (64, 4096, 512, True),      # result above the limit
])
def test_host_buffer_entry_point(cuda_lib, m, n, k, pinned):
    x, wq, s = synth.make_case(m, n, k, seed=9)
    _, twq, ts = dev(x, wq, s)
    xh = torch.from_numpy(x)
    yh = torch.zeros((m, n), dtype=torch.float16)
    if pinned:
        xh, yh = xh.pin_memory(), yh.pin_memory()
    xd = torch.empty((m, k), dtype=torch.float16, device="cuda")
    yd = torch.empty((m, n), dtype=torch.float16, device="cuda")
    st = torch.cuda.current_stream().cuda_stream
    for _ in range(2):          # twice: the second call's input transfer follows the first call's result transfer
        rc = cuda_lib.b200_q4f16_matmul_host(xh.data_ptr(), xd.data_ptr(), twq.data_ptr(), ts.data_ptr(), yd.data_ptr(),
                                             yh.data_ptr(), m, n, k, st)
        assert rc == 0, _lib.last_error()
    torch.cuda.synchronize()
    assert_matmul_close(yh.numpy(), x, wq, s, "host buffers")
    assert np.array_equal(yh.numpy().view(np.uint16), yd.cpu().numpy().view(np.uint16))
    assert np.array_equal(xd.cpu().numpy().view(np.uint16), x.view(np.uint16))


def test_launch_counter(cuda_lib):
    x, wq, s = synth.make_case(1, 64, 128)
    tx, twq, ts = dev(x, wq, s)
    ops.reset_launch_count()
    ops.q4f16_matmul(tx, twq, ts)
    ops.q4f16_dequantize(twq, ts)
    assert ops.launch_count() == 2


# ------------------------------------------------------------------------------ tensor-core matmul
def test_gemm_one_hot_rows_select_weights_exactly(cuda_lib):
    # x row m is one-hot at k_m: y[m, n] = w[n, k_m] with no summation, so the result must equal the
    # reference's dequantised weight bit for bit.  Exercises every position of the swizzled operand
    # tiles (k_m sweeps 0..K-1) and both halves of every scale group.
    n, k = 256, 256
    m = k
    rng = np.random.default_rng(17)
    wq, s = synth.make_weights(n, k, rng)
    x = np.zeros((m, k), np.float16)
    x[np.arange(m), np.arange(k)] = 1.0
    out = run_matmul(x, wq, s, family="gemm")
    assert_bits_equal(out, oracle.c_dequantize(wq, s).T.copy(), "one-hot rows")
    assert cuda_lib.b200_device_error_flags() == 0


def test_gemm_one_hot_weights_select_activations(cuda_lib):
    # every weight row has a single non-zero weight (q=8 -> +1 * scale=1 at k_n, q=7 -> 0 elsewhere):
    # y[m, n] = x[m, k_n] exactly.  Checks the x-side tile layout and the accumulator/epilogue mapping.
    m, n, k = 128, 256, 128
    rng = np.random.default_rng(18)
    q = np.full((n, k), 7, np.uint8)
    kn = rng.integers(0, k, n)
    q[np.arange(n), kn] = 8
    wq = oracle.pack_nibbles(q)
    s = np.ones((n, k // 32), np.float16)
    x = rng.standard_normal((m, k)).astype(np.float16)
    out = run_matmul(x, wq, s, family="gemm")
    assert_bits_equal(out, x[:, kn].copy(), "one-hot weights")


@pytest.mark.parametrize("m,n,k", [(128, 256, 64), (128, 256, 256), (256, 512, 512), (17, 256, 128), (129, 300, 96),
                                   (200, 264, 1376), (384, 1000, 2048), (1024, 1280, 8192), (130, 11008, 4096),
                                   (2048, 520, 4096)])
def test_gemm_shapes(cuda_lib, m, n, k):
    x, wq, s = synth.make_case(m, n, k, seed=m + n + k)
    out = run_matmul(x, wq, s, family="gemm")
    assert_matmul_close(out, x, wq, s, f"gemm M={m} N={n} K={k}")
    assert cuda_lib.b200_device_error_flags() == 0


def test_gemm_matches_gemv_family(cuda_lib):
    # the two kernel families on the same problem (M=16 is in both domains)
    x, wq, s = synth.make_case(16, 512, 1024, seed=3)
    a = run_matmul(x, wq, s, family="gemm")
    b = run_matmul(x, wq, s, family="gemv")
    assert_matmul_close(a, x, wq, s, "gemm@16")
    assert_matmul_close(b, x, wq, s, "gemv@16")


def test_prefill_config_full_size(cuda_lib):
    # second benchmark config at full size: sampled rows against the oracle, then properties that
    # need no oracle: linearity in x and agreement with matmul over the library's own decode.
    m, n, k = 2048, 11008, 4096
    x, wq, s = synth.make_case(m, n, k, seed=2)
    tx, twq, ts = dev(x, wq, s)
    y = ops.q4f16_matmul(tx, twq, ts)
    torch.cuda.synchronize()
    assert cuda_lib.b200_device_error_flags() == 0
    yh = y.cpu().numpy()
    rng = np.random.default_rng(0)
    rows = np.sort(rng.choice(n, 96, replace=False))
    toks = np.sort(rng.choice(m, 64, replace=False))
    assert_matmul_close(yh[np.ix_(toks, rows)], x[toks], wq[rows], s[rows], "cfg2 sample")
    # (2x) . W == 2 (x . W): scaling by two commutes with every rounding in the path except where the
    # fp16 result is subnormal (|y| < 2^-14), where it may differ by one subnormal step
    y2 = ops.q4f16_matmul(tx * 2, twq, ts)
    normal = y.abs() >= 2.0 ** -13
    assert torch.equal(y2[normal], (y * 2)[normal])
    assert ((y2.float() - 2 * y.float()).abs()[~normal] <= 2.0 ** -23).all()
    # against a dense fp32 matmul over the bit-exact decode, on a slab
    w = ops.q4f16_dequantize(twq[:512].contiguous(), ts[:512].contiguous()).float()
    ref = (tx.float() @ w.t())
    err = (y[:, :512].float() - ref).abs().max().item()
    assert err < 0.05, err


@pytest.mark.parametrize("k,tiles,ctas", [(256, 16, 4), (512, 16, 4), (1024, 12, 3), (4096, 8, 1)])
def test_gemm_many_tiles_per_cta_bit_exact(cuda_lib, k, tiles, ctas):
    # Few CTAs, many tiles each: the shared-memory rings wrap many times and tiles follow each other
    # inside one CTA (accumulator double buffering, stage reuse across tile boundaries).  One-hot
    # activations make every output a single dequantised weight, so any stage that is refilled or
    # read at the wrong moment shows up as a bit difference.  Repeated, because such races are
    # timing dependent.
    m, n = 128, 256 * tiles
    rng = np.random.default_rng(k + tiles)
    wq, s = synth.make_weights(n, k, rng)
    w = oracle.c_dequantize(wq, s)
    twq, ts = dev(wq, s)
    try:
        relax_b200.set_option("gemm.max_ctas", ctas)
        for kbase in range(0, k, 128):
            x = np.zeros((m, k), np.float16)
            x[np.arange(128), kbase + np.arange(128)] = 1.0
            tx = torch.from_numpy(x).cuda()
            want = np.ascontiguousarray(w[:, kbase:kbase + 128].T)
            for _ in range(3 if k <= 1024 else 1):
                out = ops.q4f16_matmul(tx, twq, ts, family="gemm").cpu().numpy()
                assert_bits_equal(out, want, f"K={k} kbase={kbase}")
    finally:
        relax_b200.set_option("gemm.max_ctas", 0)
    assert cuda_lib.b200_device_error_flags() == 0


# ------------------------------------------------------------------------------ weight-stationary GEMM (mid-sized batches)
@pytest.mark.parametrize("ksplit", [0, 1, 2, 4, 8])
@pytest.mark.parametrize("m,n,k", [(1, 128, 256), (9, 300, 1024), (16, 4096, 4096), (17, 129, 2048), (33, 1000, 4096),
                                   (64, 4096, 4096), (100, 512, 11008), (128, 2000, 2048), (128, 4096, 11008)])
def test_gemm_ws_shapes(cuda_lib, m, n, k, ksplit):
    x, wq, s = synth.make_case(m, n, k, seed=m + n + k)
    try:
        relax_b200.set_option("gemm.ws_ksplit", ksplit)
        out = run_matmul(x, wq, s, family="gemm_ws")
    finally:
        relax_b200.set_option("gemm.ws_ksplit", 0)
    assert_matmul_close(out, x, wq, s, f"gemm_ws M={m} N={n} K={k} ksplit={ksplit}")
    assert cuda_lib.b200_device_error_flags() == 0


def test_gemm_ws_one_hot_selects_weights_exactly(cuda_lib):
    # x row m is one-hot at k_m: y[m, n] = w[n, k_m] with no summation (the other K slices add exact
    # zeros), so the result must equal the reference's dequantised weight bit for bit
    n, k = 256, 1024
    rng = np.random.default_rng(23)
    wq, s = synth.make_weights(n, k, rng)
    w = oracle.c_dequantize(wq, s)
    for base in range(0, k, 128):
        x = np.zeros((128, k), np.float16)
        x[np.arange(128), base + np.arange(128)] = 1.0
        out = run_matmul(x, wq, s, family="gemm_ws")
        assert_bits_equal(out, w[:, base:base + 128].T.copy(), f"one-hot rows at {base}")
    assert cuda_lib.b200_device_error_flags() == 0


def test_gemm_ws_rejects_what_it_cannot_take(cuda_lib):
    x, wq, s = synth.make_case(129, 64, 256, seed=1)
    tx, twq, ts = dev(x, wq, s)
    y = torch.empty((129, 64), dtype=torch.float16, device="cuda")
    assert cuda_lib.b200_q4f16_gemm_ws(tx.data_ptr(), twq.data_ptr(), ts.data_ptr(), y.data_ptr(), 129, 64, 256, 0) == _lib.EINVAL
    x, wq, s = synth.make_case(32, 64, 96, seed=1)       # K not a multiple of 256
    tx, twq, ts = dev(x, wq, s)
    assert cuda_lib.b200_q4f16_gemm_ws(tx.data_ptr(), twq.data_ptr(), ts.data_ptr(), y.data_ptr(), 32, 64, 96, 0) == _lib.EINVAL


@pytest.mark.parametrize("m", [17, 48, 128, 129, 200])
def test_auto_dispatch_mid_batches(cuda_lib, m):
    # 16 < M <= 128 goes to the weight-stationary kernel, above that to the prefill kernel; both must agree with the oracle
    x, wq, s = synth.make_case(m, 768, 1024, seed=m)
    assert_matmul_close(run_matmul(x, wq, s), x, wq, s, f"auto M={m}")
    assert cuda_lib.b200_device_error_flags() == 0


@pytest.mark.parametrize("m,n,k", [(9, 512, 11008), (16, 1280, 8192), (12, 300, 16384)])
def test_auto_dispatch_small_batch_long_k(cuda_lib, m, n, k):
    # 9..16 rows whose x block does not fit beside the skinny kernel's ring go to the weight-stationary kernel
    x, wq, s = synth.make_case(m, n, k, seed=m + k)
    assert_matmul_close(run_matmul(x, wq, s), x, wq, s, f"auto M={m} K={k}")
    assert cuda_lib.b200_device_error_flags() == 0
