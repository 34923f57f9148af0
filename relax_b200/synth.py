"""Seeded synthetic inputs with the shapes and value distributions of the benchmark configs.

x ~ N(0,1) fp16; nibbles uniform in 0..15 packed 8 per uint32 word, low nibble first; scales
fp16 ~ U(0.005, 0.02).  Draw order for a given seed is always x, nibbles, scales.
"""
from __future__ import annotations

import numpy as np

# (M, N, K) of the named single-matmul configurations
CONFIGS = {
    "decode_gemv_4096": (1, 4096, 4096),
    "prefill_gemm_2048x11008x4096": (2048, 11008, 4096),
}
# per-GPU shapes of the 70B-shaped sweep (K=8192, N sharded 8 ways)
SWEEP_70B = [(m, n // 8, 8192) for n in (10240, 28672, 8192) for m in (1, 16, 128, 2048)]


def pack_nibbles(q: np.ndarray) -> np.ndarray:
    """uint8 [N,K] in 0..15 -> uint32 [N,K/8]; element k lands in bits 4*(k%8) of word k//8."""
    n, k = q.shape
    q = q.astype(np.uint32).reshape(n, k // 8, 8)
    out = np.zeros((n, k // 8), dtype=np.uint32)
    for j in range(8):
        out |= q[:, :, j] << np.uint32(4 * j)
    return out


def make_weights(n: int, k: int, rng: np.random.Generator):
    q = rng.integers(0, 16, size=(n, k), dtype=np.uint8)
    scales = rng.uniform(0.005, 0.02, size=(n, k // 32)).astype(np.float16)
    return pack_nibbles(q), scales


def make_case(m: int, n: int, k: int, seed: int = 0):
    """Returns (x fp16 [m,k], wq uint32 [n,k/8], scales fp16 [n,k/32]) as numpy arrays."""
    rng = np.random.default_rng(seed)
    x = rng.standard_normal((m, k)).astype(np.float16)
    wq, scales = make_weights(n, k, rng)
    return x, wq, scales


def make_weights_torch(n: int, k: int, seed: int, device):
    """Same distributions generated on the device (for model-sized tensors where a host
    round trip would dominate set-up time).  Returns (wq int32-viewed-as-uint32, scales)."""
    import torch

    gen = torch.Generator(device=device)
    gen.manual_seed(seed)
    wq = torch.randint(-(2**31), 2**31 - 1, (n, k // 8), dtype=torch.int32, device=device, generator=gen)
    scales = torch.empty((n, k // 32), dtype=torch.float32, device=device).uniform_(0.005, 0.02, generator=gen)
    return wq.view(torch.uint32), scales.to(torch.float16)
