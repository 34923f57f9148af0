"""Tensor-parallel sharding checked on the CPU: two gloo ranks, each computing its shard with the
oracle, must reproduce the unsharded oracle after the one all-reduce per row-parallel matmul."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import oracle
from oracle import decoder as odec
from relax_b200 import decoder, tp


def test_split_blocks():
    assert tp.split_blocks(11008, 8) == [(0, 1536), (1536, 3072), (3072, 4608), (4608, 5888), (5888, 7168), (7168, 8448),
                                         (8448, 9728), (9728, 11008)]
    assert tp.split_blocks(11008, 1) == [(0, 11008)]
    assert tp.split_blocks(4096, 4) == [(0, 1024), (1024, 2048), (2048, 3072), (3072, 4096)]
    for parts in (1, 2, 4, 8):
        r = tp.split_blocks(11008, parts)
        assert r[0][0] == 0 and r[-1][1] == 11008 and all(a[1] == b[0] for a, b in zip(r, r[1:]))
        assert all((b - a) % 256 == 0 and b > a for a, b in r)
    with pytest.raises(ValueError):
        tp.split_blocks(1000, 2)
    with pytest.raises(ValueError):
        tp.split_blocks(512, 4)


def test_shard_shapes():
    cfg = decoder.DecoderConfig(hidden=1024, heads=8, inter=1280, layers=1, vocab=10)
    full = decoder.synth_layer_numpy(cfg, 1)
    tot_i = 0
    for r in range(4):
        s = tp.shard_layer(full, r, 4, cfg.hidden, cfg.inter)
        il = s["inter_local"]
        tot_i += il
        assert s["qkv"][0].shape == (3 * 256, 1024 // 8) and s["qkv"][1].shape == (3 * 256, 1024 // 32)
        assert s["o"][0].shape == (1024, 256 // 8) and s["o"][1].shape == (1024, 256 // 32)
        assert s["gu"][0].shape == (2 * il, 1024 // 8)
        assert s["down"][0].shape == (1024, il // 8) and s["down"][1].shape == (1024, il // 32)
        assert all(a.flags["C_CONTIGUOUS"] for k in ("qkv", "o", "gu", "down") for a in s[k])
    assert tot_i == cfg.inter


def _rank_main(rank, world, port, ret):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        cfg = decoder.DecoderConfig(hidden=512, heads=4, inter=768, layers=1, vocab=10)
        full = decoder.synth_layer_numpy(cfg, 3)
        sh = tp.shard_layer(full, rank, world, cfg.hidden, cfg.inter)
        rng = np.random.default_rng(0)
        B, max_ctx, pos, D = 2, 8, 3, 128
        x = rng.standard_normal((B, cfg.hidden)).astype(np.float16)
        nhl = cfg.heads // world
        cos, sin = odec.rope_tables(max_ctx, D)
        kc_full = rng.standard_normal((B, max_ctx, cfg.heads, D)).astype(np.float16)
        vc_full = rng.standard_normal((B, max_ctx, cfg.heads, D)).astype(np.float16)
        kc = np.ascontiguousarray(kc_full[:, :, rank * nhl:(rank + 1) * nhl])
        vc = np.ascontiguousarray(vc_full[:, :, rank * nhl:(rank + 1) * nhl])

        def allreduce(y):           # fp32 partial sums are exchanged, rounded once afterwards
            t = torch.from_numpy(y.copy())
            dist.all_reduce(t)
            return t.numpy()

        # sharded layer: local matmuls on slices, one sum after each row-parallel matmul
        h = odec.rmsnorm(x, sh["norm1"], cfg.eps)
        qkv = oracle.c_matmul(h, *sh["qkv"])
        hl = cfg.hidden // world
        q = odec.rope(qkv[:, :hl].reshape(B, nhl, D), cos[pos], sin[pos])
        k = odec.rope(qkv[:, hl:2 * hl].reshape(B, nhl, D), cos[pos], sin[pos])
        kc[:, pos] = k
        vc[:, pos] = qkv[:, 2 * hl:].reshape(B, nhl, D)
        a = odec.attention_decode(q, kc, vc, pos + 1)
        _, acc = oracle.c_matmul(a, *sh["o"], return_acc32=True)
        o = allreduce(acc).astype(np.float16)
        x1 = odec.add_f16(x, o)
        h2 = odec.rmsnorm(x1, sh["norm2"], cfg.eps)
        act = odec.silu_mul(oracle.c_matmul(h2, *sh["gu"]))
        _, acc = oracle.c_matmul(act, *sh["down"], return_acc32=True)
        down = allreduce(acc).astype(np.float16)
        if rank == 0:
            # unsharded reference
            x_ref, down_ref = odec.layer_decode(x, None, full, kc_full.copy(), vc_full.copy(), pos, cos, sin, cfg.heads, cfg.eps)
            e1 = np.abs(x1.astype(np.float32) - x_ref.astype(np.float32)).max() / np.abs(x_ref.astype(np.float32)).max()
            e2 = np.abs(down.astype(np.float32) - down_ref.astype(np.float32)).max() / np.abs(down_ref.astype(np.float32)).max()
            ret["err"] = (float(e1), float(e2))
    finally:
        dist.destroy_process_group()


def test_sharded_layer_matches_unsharded_gloo():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_rank_main, args=(2, port, ret), nprocs=2, join=True)
    e1, e2 = ret["err"]
    # only the fp32 summation order and fp16 roundings at op boundaries differ
    assert e1 < 2e-3 and e2 < 4e-3, (e1, e2)
