"""Tensor-parallel sharding checked on the CPU: gloo ranks (2, 4 and 8, the last two with an uneven
K split like 11008's), each computing its shard with the oracle, must reproduce the unsharded oracle
after the one all-reduce per row-parallel matmul.  Plus the host-side failure handling: shard shapes
that disagree across ranks, and a rank that leaves between steps, end in an error on every remaining
rank instead of a hang."""
import datetime
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


def _rank_main(rank, world, port, ret, hidden, heads, inter):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["OMP_NUM_THREADS"] = "1"          # one oracle thread per rank: the ranks share the host's cores
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        cfg = decoder.DecoderConfig(hidden=hidden, heads=heads, inter=inter, layers=1, vocab=10)
        full = decoder.synth_layer_numpy(cfg, 3)
        sh = tp.shard_layer(full, rank, world, cfg.hidden, cfg.inter)
        tp.verify_sharding([sh], rank, world, cfg.hidden, cfg.inter)
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


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


# inter 2816 = 11 blocks of 256: 3,3,3,2 over 4 ranks and 2,2,2,1,1,1,1,1 over 8 (the same kind of uneven split
# that 11008 = 43 blocks gets)
@pytest.mark.parametrize("world,hidden,heads,inter", [(2, 512, 4, 768), (4, 2048, 16, 2816), (8, 2048, 16, 2816)])
def test_sharded_layer_matches_unsharded_gloo(world, hidden, heads, inter):
    sizes = [b - a for a, b in tp.split_blocks(inter, world)]
    if world == 4:
        assert sizes == [768, 768, 768, 512]
    if world == 8:
        assert sizes == [512, 512, 512, 256, 256, 256, 256, 256]
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_rank_main, args=(world, _free_port(), ret, hidden, heads, inter), nprocs=world, join=True)
    e1, e2 = ret["err"]
    # only the fp32 summation order and fp16 roundings at op boundaries differ
    assert e1 < 2e-3 and e2 < 4e-3, (e1, e2)


def _mismatch_main(rank, world, port, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), OMP_NUM_THREADS="1")
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        cfg = decoder.DecoderConfig(hidden=512, heads=4, inter=768, layers=1, vocab=10)
        full = decoder.synth_layer_numpy(cfg, 3)
        # rank 1 was sharded from a model with another intermediate size: the K slices of the down projection
        # (512 + 512) no longer add up to 768
        if rank == 1:
            other = decoder.DecoderConfig(hidden=512, heads=4, inter=1024, layers=1, vocab=10)
            sh = tp.shard_layer(decoder.synth_layer_numpy(other, 3), rank, world, other.hidden, other.inter)
        else:
            sh = tp.shard_layer(full, rank, world, cfg.hidden, cfg.inter)
        try:
            tp.verify_sharding([sh], rank, world, cfg.hidden, cfg.inter)
            ret[rank] = "no error"
        except tp.ShardingMismatch as e:
            ret[rank] = "mismatch: " + str(e)
    finally:
        dist.destroy_process_group()


def test_disagreeing_shard_shapes_raise_on_every_rank():
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_mismatch_main, args=(2, _free_port(), ret), nprocs=2, join=True)
    assert all(str(ret[r]).startswith("mismatch") for r in range(2)), dict(ret)
    assert "add up to" in ret[0]


def _leaver_main(rank, world, port, ret, announce):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), OMP_NUM_THREADS="1")
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=20))
    guard = tp.StepGuard()
    steps_done = 0
    try:
        for step in range(4):
            if rank == world - 1 and step == 2:
                # this rank leaves between steps, with nothing of its own in flight
                if announce:
                    guard.leave()
                ret[rank] = ("left", steps_done)
                return
            guard.check()                      # raises RankLeft instead of launching the step
            t = torch.ones(4)
            dist.all_reduce(t)                 # the step's own collective
            assert float(t[0]) == world
            steps_done += 1
        ret[rank] = ("finished", steps_done)
    except tp.RankLeft as e:
        ret[rank] = ("rank_left", steps_done)
    finally:
        if not (rank == world - 1 and not announce):
            try:
                dist.destroy_process_group()
            except Exception:
                pass


@pytest.mark.parametrize("announce", [True, False])
def test_rank_leaving_between_steps_is_an_error_not_a_hang(announce):
    world = 3
    mgr = mp.Manager()
    ret = mgr.dict()
    ctx = mp.spawn(_leaver_main, args=(world, _free_port(), ret, announce), nprocs=world, join=False)
    import time

    t0 = time.time()
    while not ctx.join(timeout=5):
        assert time.time() - t0 < 120, "ranks still running: the remaining ranks hang"
    assert ret[world - 1] == ("left", 2)
    for r in range(world - 1):
        assert ret[r] == ("rank_left", 2), dict(ret)
