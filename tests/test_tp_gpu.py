"""Tensor-parallel decode on two GPUs: NCCL all-reduce and the all-reduce fused into the matmul kernel
must both reproduce the single-GPU engine (and hence the oracle it is tested against).  Needs two
GPUs; on a one-GPU box the test reports itself as skipped."""
import os
import socket

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _worker(rank, world, port, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    import torch.distributed as dist

    from relax_b200 import _lib, decoder, tp

    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        cfg = decoder.DecoderConfig(hidden=1024, heads=8, inter=1280, layers=3, vocab=512)
        rng = np.random.default_rng(3)
        full = [decoder.synth_layer_numpy(cfg, 50 + i) for i in range(cfg.layers)]
        embed = torch.from_numpy((0.5 * rng.standard_normal((cfg.vocab, cfg.hidden))).astype(np.float16)).to(dev)
        fnorm = torch.ones(cfg.hidden, dtype=torch.float16, device=dev)
        B, max_ctx, steps = 2, 16, 4
        results = {}
        for name, w, peer in (("single", 1, False), ("nccl", world, False), ("peer", world, True)):
            r = 0 if w == 1 else rank
            layers = [decoder.to_device(tp.shard_layer(l, r, w, cfg.hidden, cfg.inter), dev) for l in full]
            vl = cfg.vocab // w
            eng = decoder.DecodeEngine(cfg, layers, embed, fnorm, embed[r * vl:(r + 1) * vl].contiguous(), B, max_ctx, dev,
                                       rank=r, world=w, peer_reduce=peer)
            assert (eng.peer is not None) == peer
            eng.tokens.copy_(torch.tensor([3, 200], dtype=torch.int32))
            hs = []
            for _ in range(steps):
                eng.step()
                torch.cuda.synchronize()
                hs.append(eng.h.float().cpu().numpy().copy())
            results[name] = (hs, eng.logits.float().cpu().numpy().copy())
            assert _lib.lib().b200_device_error_flags() == 0
            dist.barrier()
        if rank == 0:
            errs = {}
            for name in ("nccl", "peer"):
                e = 0.0
                for a, b in zip(results[name][0], results["single"][0]):
                    e = max(e, float(np.abs(a - b).max() / np.abs(b).max()))
                errs[name] = e
            ret["errs"] = errs
    finally:
        dist.destroy_process_group()


def test_tensor_parallel_decode_two_gpus():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp

    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_worker, args=(2, port, ret), nprocs=2, join=True)
    errs = dict(ret["errs"])
    # K slices change the fp32 summation order and add one fp16 rounding per rank's partial result
    assert errs["nccl"] < 1e-2 and errs["peer"] < 1e-2, errs
