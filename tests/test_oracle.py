"""CPU tests: the oracle against the committed golden vectors and against itself."""
import numpy as np
import pytest

import oracle
from relax_b200 import synth
from util import assert_bits_equal, golden_cases


def test_golden_vectors_numpy_and_c(golden):
    n = 0
    for name, x, wq, s, w, y in golden_cases(golden):
        assert_bits_equal(oracle.dequantize(wq, s), w, name + " numpy decode")
        assert_bits_equal(oracle.c_dequantize(wq, s), w, name + " C decode")
        assert_bits_equal(oracle.matmul(x, wq, s), y, name + " numpy matmul")
        assert_bits_equal(oracle.c_matmul(x, wq, s), y, name + " C matmul")
        assert_bits_equal(oracle.c_matmul(x, wq, s, unfused=True), y, name + " C unfused")
        n += 1
    assert n >= 9


def test_nibble_order_and_zero_point():
    # word 0x76543210 holds q = 0,1,...,7 for k = 0..7 (low nibble first); zero point 7
    wq = np.full((1, 4), 0x76543210, dtype=np.uint32)
    s = np.array([[0.5]], dtype=np.float16)
    w = oracle.dequantize(wq, s)
    assert w.shape == (1, 32)
    np.testing.assert_array_equal(w[0, :8].astype(np.float32), (np.arange(8) - 7) * 0.5)
    wq = np.full((1, 4), 0xFEDCBA98, dtype=np.uint32)
    np.testing.assert_array_equal(oracle.c_dequantize(wq, s)[0, :8].astype(np.float32), (np.arange(8, 16) - 7) * 0.5)


def test_pack_unpack_roundtrip():
    rng = np.random.default_rng(1)
    q = rng.integers(0, 16, (7, 96), dtype=np.uint8)
    assert (oracle.unpack_nibbles(oracle.pack_nibbles(q)) == q).all()
    assert (synth.pack_nibbles(q) == oracle.pack_nibbles(q)).all()


def test_single_rounding_of_decode():
    # a scale whose product with (q-7) needs rounding: every result must equal the fp16 rounding
    # of the exact product, never a doubly rounded or fused value
    s = np.array([[0x2E67]], dtype=np.uint16).view(np.float16)  # ~0.1000 with odd significand
    q = np.tile(np.arange(16, dtype=np.uint8), 2)[None, :]
    wq = oracle.pack_nibbles(q)
    w = oracle.dequantize(wq, s)[0, :16]
    exact = (np.arange(16) - 7).astype(np.float64) * float(s[0, 0])
    np.testing.assert_array_equal(w, exact.astype(np.float16))


@pytest.mark.parametrize("m,n,k", [(1, 4096, 4096), (16, 200, 1024), (5, 33, 11008)])
def test_c_matches_numpy_on_bench_shapes(m, n, k):
    x, wq, s = synth.make_case(m, n, k, seed=3)
    rows = slice(0, min(n, 64))
    assert_bits_equal(oracle.c_dequantize(wq, s)[rows], oracle.dequantize(wq[rows], s[rows]), "decode")
    assert_bits_equal(oracle.c_matmul(x, wq, s)[:, rows], oracle.matmul(x, wq[rows], s[rows]), "matmul")


def test_sequential_accumulation_order_matters_and_is_kept():
    # fp32 addition is not associative: 2^24 + 1 + 1 summed left to right stays 2^24, pairing the
    # ones first gives 2^24 + 2.  x carries the 2^24 (as 4096*4096), w = 1 via q=8, scale=1.
    k = 32
    x = np.zeros((1, k), dtype=np.float16)
    x[0, 0] = 4096.0
    x[0, 1:3] = 2.0 ** -12
    wq = np.full((1, k // 8), 0x88888888, dtype=np.uint32)  # q = 8 -> (q-7) = 1
    s = np.array([[4096.0]], dtype=np.float16)
    y, acc = oracle.c_matmul(x, wq, s, return_acc32=True)
    assert acc[0, 0] == np.float32(2.0 ** 24)  # the two 1.0 terms are each absorbed
    assert oracle.matmul_acc32(x, oracle.dequantize(wq, s))[0, 0] == np.float32(2.0 ** 24)


def test_empty_shapes():
    s = np.zeros((0, 4), np.float16)
    assert oracle.c_dequantize(np.zeros((0, 16), np.uint32), s).shape == (0, 128)
    x = np.zeros((0, 128), np.float16)
    assert oracle.c_matmul(x, np.zeros((3, 16), np.uint32), np.zeros((3, 4), np.float16)).shape == (0, 3)
