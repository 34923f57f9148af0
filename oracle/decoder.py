"""numpy restatement of one Llama-style decoder layer in decode mode.  TEST INFRASTRUCTURE ONLY.

The reference has no RMSNorm, RoPE or attention operator.  A Relax module for this layer is
written with its elementwise and reduction ops, and these functions follow their legalizations
(paths inside the reference tree, ``python/tvm/relax/transform/legalize_ops.py``):

* ``mean`` (:378-381), ``sqrt``/``divide``/``multiply`` (elementwise table) -> RMSNorm
* ``strided_slice`` (:176), ``negative``, ``concat`` (:280), ``multiply``, ``add`` -> rotary
  embedding with the "rotate half" pairing (i, i + head_dim/2) and cos/sin tables as inputs
* ``matmul`` (:203-264), ``softmax`` = topi.nn.softmax (:513-514) -> attention
* ``silu`` = x * sigmoid(x) (:506-510) -> SwiGLU
* the seven projections are the q4f16 dequantize+matmul of :mod:`oracle.q4f16`

The reference does not pin the precision of this composition; the choice made here (and in the
CUDA kernels) is: statistics and accumulations in fp32, one round-to-nearest fp16 rounding at
every operator output, the residual stream stored in fp16.
"""
from __future__ import annotations

import numpy as np

from . import q4f16

F16, F32 = np.float16, np.float32


def rope_tables(max_pos: int, head_dim: int = 128, theta: float = 10000.0):
    """cos, sin fp32 [max_pos, head_dim/2]; angle = pos * theta^(-2i/head_dim), computed in fp64."""
    half = head_dim // 2
    inv = theta ** (-np.arange(half, dtype=np.float64) * 2.0 / head_dim)
    ang = np.arange(max_pos, dtype=np.float64)[:, None] * inv[None, :]
    return np.cos(ang).astype(F32), np.sin(ang).astype(F32)


def rmsnorm(x, w, eps):
    """fp16 [B,H] = fp16( f32(x) * rsqrt(mean(f32(x)^2) + eps) * f32(w) )."""
    xf = x.astype(F32)
    ss = np.mean(xf * xf, axis=-1, keepdims=True, dtype=F32)
    inv = (1.0 / np.sqrt(ss + F32(eps))).astype(F32)
    return (xf * inv * w.astype(F32)[None, :]).astype(F16)


def add_f16(a, b):
    """fp16(a + b) with the sum formed in fp32 (one rounding)."""
    return (a.astype(F32) + b.astype(F32)).astype(F16)


def rope(v, cos, sin):
    """v fp16 [..., D]; pairs (i, i + D/2); cos/sin fp32 [D/2]."""
    vf = v.astype(F32)
    half = v.shape[-1] // 2
    a, b = vf[..., :half], vf[..., half:]
    return np.concatenate([a * cos - b * sin, b * cos + a * sin], axis=-1).astype(F16)


def attention_decode(q, k_cache, v_cache, ctx):
    """q fp16 [B,nh,D]; caches fp16 [B,max_ctx,nh,D]; attends to positions < ctx.
    Returns fp16 [B, nh*D]."""
    B, nh, D = q.shape
    qf = q.astype(F32)
    kf = k_cache[:, :ctx].astype(F32)           # [B,ctx,nh,D]
    vf = v_cache[:, :ctx].astype(F32)
    s = np.einsum("bhd,bthd->bht", qf, kf).astype(F32) / F32(np.sqrt(D))
    s = s - s.max(axis=-1, keepdims=True)
    p = np.exp(s).astype(F32)
    p = p / p.sum(axis=-1, keepdims=True, dtype=F32)
    o = np.einsum("bht,bthd->bhd", p, vf).astype(F32)
    return o.astype(F16).reshape(B, nh * D)


def silu_mul(gu):
    """gu fp16 [B, 2I] = [gate | up] -> fp16 [B, I] = silu(gate) * up (fp32 inside)."""
    I = gu.shape[1] // 2
    g, u = gu[:, :I].astype(F32), gu[:, I:].astype(F32)
    return (g / (1.0 + np.exp(-g)) * u).astype(F16)


def q4_linear(x, wq_s, matmul=None):
    """x fp16 [B,K] times one quantised projection (wq, scales)."""
    f = matmul or q4f16.c_matmul
    return f(x, wq_s[0], wq_s[1])


def layer_decode(x, delta, weights, k_cache, v_cache, pos, cos_t, sin_t, nh, eps=1e-5, matmul=None):
    """One decoder layer for the token at position `pos` (caches are updated in place).

    x fp16 [B,H] is the residual stream, `delta` (or None) the previous layer's MLP output that
    has not been added yet.  weights: dict with 'qkv', 'o', 'gu', 'down' = (wq, scales) and
    'norm1', 'norm2' fp16 [H].  Returns (x_after_attention_residual, mlp_output): the caller (the
    next layer's first norm, or the final norm) adds mlp_output.
    """
    B, H = x.shape
    D = H // nh
    if delta is not None:
        x = add_f16(x, delta)
    h = rmsnorm(x, weights["norm1"], eps)
    qkv = q4_linear(h, weights["qkv"], matmul)                    # [B, 3H] = [q | k | v]
    q = qkv[:, :H].reshape(B, nh, D)
    k = qkv[:, H:2 * H].reshape(B, nh, D)
    v = qkv[:, 2 * H:].reshape(B, nh, D)
    q = rope(q, cos_t[pos], sin_t[pos])
    k = rope(k, cos_t[pos], sin_t[pos])
    k_cache[:, pos] = k
    v_cache[:, pos] = v
    a = attention_decode(q, k_cache, v_cache, pos + 1)
    o = q4_linear(a, weights["o"], matmul)
    x = add_f16(x, o)
    h2 = rmsnorm(x, weights["norm2"], eps)
    gu = q4_linear(h2, weights["gu"], matmul)
    act = silu_mul(gu)
    down = q4_linear(act, weights["down"], matmul)
    return x, down
