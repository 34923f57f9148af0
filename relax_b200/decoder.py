"""Decode-step harness for a Llama-style q4f16 decoder: the callers either side of the quantised
matmul (RMSNorm, RoPE + KV cache, attention, SwiGLU) wired to the C-ABI kernels, optionally
tensor-parallel with one NCCL all-reduce after each row-parallel matmul.

torch is used for device memory, streams, CUDA graphs and the NCCL process group; every kernel of a step is
this library's for batches of up to 16 (above that the fp16 output projection is a plain library GEMM, and under
tensor parallelism the sampling over the gathered vocabulary slices is torch's argmax).

Layout per rank (world size t, hidden H, heads nh, head dim 128, intermediate I):

    qkv   q4  [3*H/t, H]      rows = q heads | k heads | v heads of this rank
    o     q4  [H, H/t]        row-parallel   -> all-reduce
    gu    q4  [2*I_r, H]      rows = gate | up rows of this rank's slice of I
    down  q4  [H, I_r]        row-parallel   -> all-reduce
    KV    fp16 [B, max_ctx, nh/t, 128] per layer, K and V
"""
from __future__ import annotations

import ctypes
import dataclasses

import numpy as np
import torch

from . import _lib, tp


@dataclasses.dataclass
class DecoderConfig:
    hidden: int = 4096
    heads: int = 32
    inter: int = 11008
    layers: int = 32
    vocab: int = 32000
    eps: float = 1e-5
    theta: float = 10000.0
    head_dim: int = 128

    def __post_init__(self):
        if self.hidden != self.heads * self.head_dim or self.head_dim != 128:
            raise ValueError("the attention kernels take head_dim 128 and hidden = heads * 128")


def rope_tables(max_pos: int, head_dim: int, theta: float, device):
    half = head_dim // 2
    inv = theta ** (-np.arange(half, dtype=np.float64) * 2.0 / head_dim)
    ang = np.arange(max_pos, dtype=np.float64)[:, None] * inv[None, :]
    cos = torch.from_numpy(np.cos(ang).astype(np.float32)).to(device)
    sin = torch.from_numpy(np.sin(ang).astype(np.float32)).to(device)
    return cos.contiguous(), sin.contiguous()


def synth_layer_numpy(cfg: DecoderConfig, seed: int):
    """Full (unsharded) random layer on the host: nibbles uniform 0..15, scales U(0.005, 0.02),
    norm weights ~ N(1, 0.02).  Small configurations only (tests)."""
    from . import synth

    rng = np.random.default_rng(seed)
    H, I = cfg.hidden, cfg.inter
    w = {}
    for name, (n, k) in (("qkv", (3 * H, H)), ("o", (H, H)), ("gu", (2 * I, H)), ("down", (H, I))):
        w[name] = synth.make_weights(n, k, rng)
    w["norm1"] = (1.0 + 0.02 * rng.standard_normal(H)).astype(np.float16)
    w["norm2"] = (1.0 + 0.02 * rng.standard_normal(H)).astype(np.float16)
    return w


def synth_layer_torch(cfg: DecoderConfig, seed: int, device):
    """Same distributions generated on the device (model-sized tensors)."""
    from . import synth

    H, I = cfg.hidden, cfg.inter
    w = {}
    for j, (name, (n, k)) in enumerate((("qkv", (3 * H, H)), ("o", (H, H)), ("gu", (2 * I, H)), ("down", (H, I)))):
        w[name] = synth.make_weights_torch(n, k, seed * 16 + j, device)
    gen = torch.Generator(device=device)
    gen.manual_seed(seed * 16 + 9)
    w["norm1"] = (1.0 + 0.02 * torch.randn(H, device=device, generator=gen)).to(torch.float16)
    w["norm2"] = (1.0 + 0.02 * torch.randn(H, device=device, generator=gen)).to(torch.float16)
    return w


def to_device(layer: dict, device):
    out = {}
    for k, v in layer.items():
        if isinstance(v, tuple):
            out[k] = tuple(torch.from_numpy(np.ascontiguousarray(a)).to(device) if isinstance(a, np.ndarray) else a.to(device)
                           for a in v)
        elif isinstance(v, np.ndarray):
            out[k] = torch.from_numpy(v).to(device)
        else:
            out[k] = v
    return out


class DecodeEngine:
    """Buffers and kernel sequence of one decode step for `batch` sequences.

    `layers` is a list of per-rank layer shards (see tp.shard_layer) on `device`; `embed` the fp16
    embedding table [vocab, H]; `lm_head` fp16 [vocab_local, H] (rows of this rank's vocabulary
    slice) or None to stop at the final norm; `final_norm` fp16 [H].
    """

    def __init__(self, cfg: DecoderConfig, layers, embed, final_norm, lm_head, batch: int, max_ctx: int,
                 device, rank: int = 0, world: int = 1, group=None, fused=None, peer_reduce: bool = True,
                 fused_attention=False, guard=None, verify: bool = True, layer_kernel=None, rope_epilogue: bool = True):
        self.cfg, self.batch, self.max_ctx, self.device = cfg, batch, max_ctx, torch.device(device)
        self.rank, self.world, self.group = rank, world, group
        self.layers, self.embed, self.final_norm, self.lm_head = layers, embed, final_norm, lm_head
        self.L = _lib.lib()
        H, B = cfg.hidden, batch
        self.nh_local = cfg.heads // world
        if cfg.heads % world:
            raise ValueError("heads must divide by the tensor-parallel size")
        # host-side checks of the tensor-parallel set-up: shard shapes agree across ranks before anything is
        # launched; `guard` (tp.StepGuard on a CPU-capable group) is consulted before every eager step
        self.guard = guard
        if world > 1 and verify and layers:
            tp.verify_sharding(layers, rank, world, cfg.hidden, cfg.inter, group=group)
        f16 = dict(dtype=torch.float16, device=self.device)
        hl = H // world
        il_max = max(l["inter_local"] for l in layers) if layers else cfg.inter
        # fused: RMSNorm (+ residual add) and SwiGLU run inside the staging of the next skinny matmul
        # (7 kernels per layer instead of 11); needs batch <= 16, the skinny kernel's range.  By default only at
        # batch 1: every CTA of a fused kernel recomputes the statistics of all the batch's rows, and from two rows on
        # the separate kernels are faster (measured per layer at context 2000: 80 against 88 us at batch 2, 124 against
        # 176 at batch 8, 174 against 291 at batch 16).
        self.fused = (B == 1) if fused is None else (bool(fused) and B <= 16)
        # False: rotary/append, attention, merge as three launches; True: one launch; "rope": rotary/append
        # inside the attention launch, merge as a second launch
        self.fused_attention = "rope" if fused_attention == "rope" else bool(fused_attention)
        self.x = torch.zeros((B, H), **f16)            # residual stream
        self.x2 = torch.zeros((B, H), **f16)           # its second buffer (fused path ping-pongs)
        self.h = torch.zeros((B, H), **f16)            # normalised activations
        self.qkv = torch.zeros((B, 3 * hl), **f16)
        self.q = torch.zeros((B, self.nh_local, 128), **f16)
        self.attn = torch.zeros((B, hl), **f16)
        self.o = torch.zeros((B, H), **f16)
        self.gu = torch.zeros((B, 2 * il_max), **f16)
        self.act = torch.zeros((B, il_max), **f16)
        self.down = torch.zeros((B, H), **f16)
        self.kc = [torch.zeros((B, max_ctx, self.nh_local, 128), **f16) for _ in layers]
        self.vc = [torch.zeros((B, max_ctx, self.nh_local, 128), **f16) for _ in layers]
        nbytes = int(self.L.b200_attn_decode_fused_scratch_bytes(B, self.nh_local, max_ctx))
        self.scratch = torch.zeros((max(nbytes, 4) // 4,), dtype=torch.float32, device=self.device)   # counters start at 0
        self.pos = torch.zeros((1,), dtype=torch.int32, device=self.device)
        self.tokens = torch.zeros((B,), dtype=torch.int32, device=self.device)
        self.cos, self.sin = rope_tables(max_ctx, 128, cfg.theta, self.device)
        vl = lm_head.shape[0] if lm_head is not None else 0
        self.logits_local = torch.zeros((B, vl), **f16) if vl else None
        self.logits = torch.zeros((B, vl * world), **f16) if vl and world > 1 else self.logits_local
        self.gathered = torch.zeros((world, B, vl), **f16) if vl and world > 1 else None
        self.lm_scratch = torch.zeros((max(int(self.L.b200_lm_head_scratch_bytes()), 16) // 4,), dtype=torch.float32, device=self.device)
        self.graph = None
        self.launches_per_step = 0
        # batch 1: one persistent kernel per layer (b200_decode_layer) instead of seven launches.  Off by default:
        # measured on B200 at the 7B shape it is as fast as the seven launches on one GPU (1.94 against 1.90 ms per
        # token) and slower on two (2.07 against 1.89), because every stage boundary inside it costs what a
        # dependent launch costs, and its attention stage has only eight warps per SM with loads in flight
        self.layer_kernel = False if layer_kernel is None else bool(layer_kernel)
        # batch 1, fused prologues, three-launch attention: rotary embedding + KV append run in the epilogue of the
        # qkv matmul (b200_q4f16_gemv_rmsnorm_rope), one launch less per layer
        self.rope_epilogue = bool(rope_epilogue) and self.fused and B == 1 and not self.fused_attention and not self.layer_kernel
        if self.layer_kernel and B != 1:
            raise ValueError("the one-kernel-per-layer path is the batch-1 path")
        # tensor parallel: the sum over ranks after o and down runs over NVLink peer memory, inside those matmul
        # kernels (b200_q4f16_gemv_allreduce) for up to 8 rows, as a kernel of this library behind the mid-batch
        # matmul above that (b200_allreduce_peer); with peer_reduce=False it is an NCCL all-reduce
        self.peer = None
        self.epoch = torch.zeros((1,), dtype=torch.int32, device=self.device)
        if world > 1 and (peer_reduce or self.layer_kernel):
            self._setup_peer_reduce()
        if self.layer_kernel:
            self._setup_layer_kernel()

    def _setup_peer_reduce(self):
        import torch.distributed._symmetric_memory as symm_mem

        B, H, nl, world = self.batch, self.cfg.hidden, len(self.layers), self.world
        ybytes = B * H * 2
        ybytes = (ybytes + 255) // 256 * 256
        fbytes = 2 * nl * world * 4
        total = 2 * ybytes + fbytes
        buf = symm_mem.empty(total, dtype=torch.uint8, device=self.device)
        buf.zero_()
        torch.cuda.synchronize(self.device)
        hdl = symm_mem.rendezvous(buf, group=self.group if self.group is not None else torch.distributed.group.WORLD)
        torch.distributed.barrier(group=self.group)
        ptrs = [int(p) for p in hdl.buffer_ptrs]
        self.peer = {
            "buf": buf, "hdl": hdl,
            "y": [[p + k * ybytes for p in ptrs] for k in range(2)],          # [kind][rank]
            "flags": [p + 2 * ybytes for p in ptrs],
            "done": torch.zeros((1,), dtype=torch.int32, device=self.device),
        }

    def _setup_layer_kernel(self):
        """Buffers and one B200DecodeLayer descriptor per layer.  The residual stream rotates through three
        buffers (a layer reads x_in, writes x_mid = x_in + delta and x_out = x_mid + o; the next layer's x_in is this
        layer's x_out and it may overwrite the two others)."""
        cfg, L = self.cfg, self.L
        H, dev = cfg.hidden, self.device
        f16 = dict(dtype=torch.float16, device=dev)
        self.xr = [self.x, self.x2, torch.zeros((1, H), **f16)]
        nbytes = int(L.b200_decode_layer_scratch_bytes(self.nh_local, self.max_ctx))
        self.layer_scratch = [torch.zeros(((nbytes + 3) // 4,), dtype=torch.int32, device=dev) for _ in self.layers]
        self.layer_desc = []
        for i, w in enumerate(self.layers):
            d = _lib.DecodeLayer()
            d.world, d.rank = self.world, self.rank
            d.hidden, d.inter_local, d.max_ctx = H, w["inter_local"], self.max_ctx
            d.heads, d.eps = cfg.heads, cfg.eps
            xin, xmid, xout = self.xr[(2 * i) % 3], self.xr[(2 * i + 1) % 3], self.xr[(2 * i + 2) % 3]
            d.x_in, d.x_mid, d.x_out = xin.data_ptr(), xmid.data_ptr(), xout.data_ptr()
            d.delta_in = self.down.data_ptr() if i > 0 else None
            d.qkv, d.attn, d.o, d.act, d.down = (self.qkv.data_ptr(), self.attn.data_ptr(), self.o.data_ptr(), self.act.data_ptr(),
                                                 self.down.data_ptr())
            d.norm1, d.norm2 = w["norm1"].data_ptr(), w["norm2"].data_ptr()
            d.cos_t, d.sin_t, d.pos = self.cos.data_ptr(), self.sin.data_ptr(), self.pos.data_ptr()
            d.k_cache, d.v_cache = self.kc[i].data_ptr(), self.vc[i].data_ptr()
            d.scratch, d.step = self.layer_scratch[i].data_ptr(), self.epoch.data_ptr()
            d.wq_qkv, d.s_qkv = w["qkv"][0].data_ptr(), w["qkv"][1].data_ptr()
            d.wq_o, d.s_o = w["o"][0].data_ptr(), w["o"][1].data_ptr()
            d.wq_gu, d.s_gu = w["gu"][0].data_ptr(), w["gu"][1].data_ptr()
            d.wq_down, d.s_down = w["down"][0].data_ptr(), w["down"][1].data_ptr()
            if self.world > 1:
                d.reduce_o = self._reduce_desc(0, i, self.o)
                d.reduce_down = self._reduce_desc(1, i, self.down)
            self.layer_desc.append(d)
        self.x_last = self.xr[(2 * len(self.layers)) % 3]     # the residual stream after the last layer

    def _reduce_desc(self, kind: int, layer: int, out):
        d = _lib.PeerReduce()
        d.world, d.rank = self.world, self.rank
        for r in range(self.world):
            d.peer_y[r] = self.peer["y"][kind][r]
            d.peer_flags[r] = self.peer["flags"][r]
        d.flag_base = (kind * len(self.layers) + layer) * self.world
        d.epoch = self.epoch.data_ptr()
        d.done_counter = self.peer["done"].data_ptr()
        d.out = out.data_ptr()
        return d

    # ------------------------------------------------------------------ kernel calls
    def _check(self, rc):
        if rc:
            raise _lib.B200Error(rc, _lib.last_error())

    def _matmul(self, x, w, y, n, k, sp):
        self._check(self.L.b200_q4f16_matmul(x.data_ptr(), w[0].data_ptr(), w[1].data_ptr(), y.data_ptr(), self.batch, n, k, sp))

    # up to this many rows the sum over ranks runs inside the skinny matmul kernel; above, the matmul (mid-batch
    # or prefill kernel) writes its partial result into the peer-mapped buffer and b200_allreduce_peer adds up
    PEER_FUSED_MAX_ROWS = 8

    def _matmul_then_peer_sum(self, kind: int, layer: int, x, w, out, n, k, sp):
        d = self._reduce_desc(kind, layer, out)
        self._check(self.L.b200_q4f16_matmul(x.data_ptr(), w[0].data_ptr(), w[1].data_ptr(), self.peer["y"][kind][self.rank],
                                             self.batch, n, k, sp))
        self._check(self.L.b200_allreduce_peer(self.batch * n, ctypes.byref(d), sp))

    def _allreduce(self, t):
        if self.world > 1:
            torch.distributed.all_reduce(t, group=self.group)

    def layer_step(self, i: int, delta, sp: int):
        """One layer; `delta` is the tensor still to be added to the residual stream (or None).
        Returns the layer's MLP output (to be added by whoever consumes the stream next)."""
        cfg, L, B, w = self.cfg, self.L, self.batch, self.layers[i]
        H, hl, il = cfg.hidden, cfg.hidden // self.world, w["inter_local"]
        dptr = delta.data_ptr() if delta is not None else None
        roped = False
        if self.fused and self.rope_epilogue:
            # residual stream: x --(+delta)--> x2 --(+o)--> x; rotary embedding and KV append in the matmul's epilogue
            rc = L.b200_q4f16_gemv_rmsnorm_rope(self.x.data_ptr(), dptr, w["norm1"].data_ptr(), self.x2.data_ptr(), cfg.eps,
                                                w["qkv"][0].data_ptr(), w["qkv"][1].data_ptr(), self.cos.data_ptr(),
                                                self.sin.data_ptr(), self.pos.data_ptr(), self.q.data_ptr(),
                                                self.kc[i].data_ptr(), self.vc[i].data_ptr(), self.nh_local, H, sp)
            if rc == _lib.ENOTREADY:
                self.rope_epilogue = False      # (the exact form is selected: two kernels from now on)
            else:
                self._check(rc)
                roped = True
        if roped:
            pass
        elif self.fused:
            # residual stream: x --(+delta)--> x2 --(+o)--> x
            self._check(L.b200_q4f16_gemv_rmsnorm(self.x.data_ptr(), dptr, w["norm1"].data_ptr(), self.x2.data_ptr(), cfg.eps,
                                                  w["qkv"][0].data_ptr(), w["qkv"][1].data_ptr(), self.qkv.data_ptr(),
                                                  B, 3 * hl, H, sp))
        else:
            self._check(L.b200_rmsnorm(self.x.data_ptr(), dptr, w["norm1"].data_ptr(), self.h.data_ptr(), B, H, cfg.eps, sp))
            self._matmul(self.h, w["qkv"], self.qkv, 3 * hl, H, sp)
        if roped:
            # The position and the older cache entries were final before the matmul in front began (the position was
            # advanced two launches before this step's first kernel, each of which waits before it lets the next
            # one start; the matmul's epilogue writes only the new token's slot, which the attention reads after
            # its own wait)
            self._check(L.b200_attn_decode(self.q.data_ptr(), self.kc[i].data_ptr(), self.vc[i].data_ptr(), self.pos.data_ptr(),
                                           self.attn.data_ptr(), self.scratch.data_ptr(), B, self.nh_local, self.max_ctx,
                                           _lib.ATTN_EARLY_KV_LOADS, sp))
        elif self.fused_attention == "rope":
            # rotary embedding + KV append + per-chunk attention in one launch, the merge in a second
            self._check(L.b200_attn_decode_rope(self.qkv.data_ptr(), self.cos.data_ptr(), self.sin.data_ptr(), self.pos.data_ptr(),
                                                self.kc[i].data_ptr(), self.vc[i].data_ptr(), self.attn.data_ptr(),
                                                self.scratch.data_ptr(), B, self.nh_local, self.max_ctx, sp))
        elif self.fused_attention:
            # rotary embedding + KV append + attention + merge in one launch
            self._check(L.b200_attn_decode_fused(self.qkv.data_ptr(), self.cos.data_ptr(), self.sin.data_ptr(), self.pos.data_ptr(),
                                                 self.kc[i].data_ptr(), self.vc[i].data_ptr(), self.attn.data_ptr(),
                                                 self.scratch.data_ptr(), B, self.nh_local, self.max_ctx, sp))
        else:
            self._check(L.b200_rope_kv_append(self.qkv.data_ptr(), self.cos.data_ptr(), self.sin.data_ptr(), self.pos.data_ptr(),
                                              self.q.data_ptr(), self.kc[i].data_ptr(), self.vc[i].data_ptr(), B, self.nh_local,
                                              self.max_ctx, sp))
            self._check(L.b200_attn_decode(self.q.data_ptr(), self.kc[i].data_ptr(), self.vc[i].data_ptr(), self.pos.data_ptr(),
                                           self.attn.data_ptr(), self.scratch.data_ptr(), B, self.nh_local, self.max_ctx,
                                           _lib.ATTN_EARLY_KV_LOADS,   # rope_kv_append sits directly in front and waits first
                                           sp))
        if self.peer is not None and B <= self.PEER_FUSED_MAX_ROWS:
            d = self._reduce_desc(0, i, self.o)
            self._check(L.b200_q4f16_gemv_allreduce(self.attn.data_ptr(), w["o"][0].data_ptr(), w["o"][1].data_ptr(),
                                                    self.peer["y"][0][self.rank], B, H, hl, 0, ctypes.byref(d), sp))
        elif self.peer is not None:
            self._matmul_then_peer_sum(0, i, self.attn, w["o"], self.o, H, hl, sp)
        else:
            self._matmul(self.attn, w["o"], self.o, H, hl, sp)
            self._allreduce(self.o)
        if self.fused:
            self._check(L.b200_q4f16_gemv_rmsnorm(self.x2.data_ptr(), self.o.data_ptr(), w["norm2"].data_ptr(), self.x.data_ptr(),
                                                  cfg.eps, w["gu"][0].data_ptr(), w["gu"][1].data_ptr(), self.gu.data_ptr(),
                                                  B, 2 * il, H, sp))
            if self.peer is not None:
                d = self._reduce_desc(1, i, self.down)
                self._check(L.b200_q4f16_gemv_allreduce(self.gu.data_ptr(), w["down"][0].data_ptr(), w["down"][1].data_ptr(),
                                                        self.peer["y"][1][self.rank], B, H, il, 1, ctypes.byref(d), sp))
                return self.down
            self._check(L.b200_q4f16_gemv_swiglu(self.gu.data_ptr(), w["down"][0].data_ptr(), w["down"][1].data_ptr(),
                                                 self.down.data_ptr(), B, H, il, sp))
        else:
            self._check(L.b200_rmsnorm(self.x.data_ptr(), self.o.data_ptr(), w["norm2"].data_ptr(), self.h.data_ptr(), B, H,
                                       cfg.eps, sp))
            self._matmul(self.h, w["gu"], self.gu, 2 * il, H, sp)
            self._check(L.b200_silu_mul(self.gu.data_ptr(), self.act.data_ptr(), B, il, sp))
            if self.peer is not None and B <= self.PEER_FUSED_MAX_ROWS:
                d = self._reduce_desc(1, i, self.down)
                self._check(L.b200_q4f16_gemv_allreduce(self.act.data_ptr(), w["down"][0].data_ptr(), w["down"][1].data_ptr(),
                                                        self.peer["y"][1][self.rank], B, H, il, 0, ctypes.byref(d), sp))
                return self.down
            if self.peer is not None:
                self._matmul_then_peer_sum(1, i, self.act, w["down"], self.down, H, il, sp)
                return self.down
            self._matmul(self.act, w["down"], self.down, H, il, sp)
        self._allreduce(self.down)
        return self.down

    def step(self):
        """One decode step on the current stream: embeds self.tokens, runs every layer at position
        self.pos, writes logits (when there is an lm_head), samples greedily into self.tokens and
        advances self.pos.  All inputs live on the device, so the step can be captured and replayed."""
        cfg, L, B = self.cfg, self.L, self.batch
        if self.guard is not None and not torch.cuda.is_current_stream_capturing():
            self.guard.check()
        sp = torch.cuda.current_stream(self.device).cuda_stream
        self._check(L.b200_embed_rows(self.embed.data_ptr(), self.tokens.data_ptr(), self.x.data_ptr(), B, cfg.hidden,
                                      self.embed.shape[0], sp))
        delta = None
        xlast = self.x
        if self.layer_kernel:
            for i in range(len(self.layers)):
                self._check(L.b200_decode_layer(ctypes.byref(self.layer_desc[i]), sp))
            if self.layers:
                delta, xlast = self.down, self.x_last
        else:
            for i in range(len(self.layers)):
                delta = self.layer_step(i, delta, sp)
        self._check(L.b200_rmsnorm(xlast.data_ptr(), delta.data_ptr() if delta is not None else None,
                                   self.final_norm.data_ptr(), self.h.data_ptr(), B, cfg.hidden, cfg.eps, sp))
        if self.lm_head is not None:
            own = B <= 16                       # the library's output projection takes up to 16 rows; above that a library GEMM
            if own:
                toks = self.tokens.data_ptr() if self.world == 1 else None
                self._check(L.b200_lm_head(self.h.data_ptr(), self.lm_head.data_ptr(), self.logits_local.data_ptr(), toks,
                                           self.lm_scratch.data_ptr(), B, self.lm_head.shape[0], cfg.hidden, 0, sp))
            else:
                torch.matmul(self.h, self.lm_head.t(), out=self.logits_local)
            if self.world > 1:
                # gather the vocabulary slices: [world, B, V_l] -> [B, world * V_l]
                torch.distributed.all_gather_into_tensor(self.gathered, self.logits_local, group=self.group)
                self.logits.view(B, self.world, -1).copy_(self.gathered.permute(1, 0, 2))
            if not own or self.world > 1:
                self.tokens.copy_(torch.argmax(self.logits, dim=1).to(torch.int32))
        self._check(L.b200_advance_pos(self.pos.data_ptr(), 1, sp))
        self._check(L.b200_advance_pos(self.epoch.data_ptr(), 1, sp))

    def kernels_per_step(self) -> int:
        """Kernels of this library launched by one step (embed + 5 or 11 per layer + final norm + output projection
        for up to 16 rows + advance)."""
        head = 1 if self.lm_head is not None and self.batch <= 16 else 0
        if self.layer_kernel:
            return 1 + len(self.layers) + 1 + head + 2
        per_layer = (5 if self.fused else 9) + (1 if self.fused_attention == "rope" else (0 if self.fused_attention else 2))
        if self.rope_epilogue:
            per_layer -= 1
        return 1 + len(self.layers) * per_layer + 1 + head + 2

    def capture(self, stream):
        """Captures one step into a CUDA graph on `stream` (after one eager warm-up step, which
        also lets NCCL set up its channels outside the capture)."""
        stream.wait_stream(torch.cuda.current_stream(self.device))   # buffers were filled on the caller's stream
        with torch.cuda.stream(stream):
            pos0 = int(self.pos.item())
            tok0 = self.tokens.clone()
            self.step()
            stream.synchronize()
            self.pos.fill_(pos0)
            self.tokens.copy_(tok0)
            self.graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(self.graph, stream=stream):
                self.step()
            self.pos.fill_(pos0)
            self.tokens.copy_(tok0)
            stream.synchronize()
        return self.graph

    def set_position(self, pos: int):
        self.pos.fill_(int(pos))
