"""Tensor-parallel decode on 2, 4 and 8 GPUs: the NCCL all-reduce form and the sum over ranks fused into
the row-parallel matmul kernels must both reproduce the CPU ORACLE (unsharded, oracle.decoder) within the
decoder tolerance, and the one-GPU engine.  The 4- and 8-rank cases use an intermediate size that splits
unevenly (2816 = 11 blocks of 256: 3,3,3,2 and 2,2,2,1,1,1,1,1), as 11008 does.  A case that needs more
GPUs than the box has reports itself as skipped."""
import os
import socket
import sys

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

TESTS_DIR = os.path.dirname(os.path.abspath(__file__))


def _worker(rank, world, port, ret, hidden, heads, inter):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    for p in (TESTS_DIR, os.path.dirname(TESTS_DIR)):
        if p not in sys.path:
            sys.path.insert(0, p)
    import torch.distributed as dist

    from relax_b200 import _lib, decoder, tp

    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        cfg = decoder.DecoderConfig(hidden=hidden, heads=heads, inter=inter, layers=2, vocab=512)
        rng = np.random.default_rng(3)
        full = [decoder.synth_layer_numpy(cfg, 50 + i) for i in range(cfg.layers)]
        embed_h = (0.5 * rng.standard_normal((cfg.vocab, cfg.hidden))).astype(np.float16)
        embed = torch.from_numpy(embed_h).to(dev)
        fnorm = torch.ones(cfg.hidden, dtype=torch.float16, device=dev)
        B, max_ctx, steps = 2, 16, 3
        tokens = [3, 200]
        ref = None
        if rank == 0:
            from test_decoder_gpu import oracle_steps

            ref = oracle_steps(cfg, full, embed_h, np.ones(cfg.hidden, np.float16), embed_h, tokens, steps, max_ctx)
        # every rank feeds the oracle's token choice, so that a near-tie in the logits cannot fork the runs
        feed = [None]
        if rank == 0:
            feed = [[np.argmax(r[1].astype(np.float32), axis=1).astype(np.int32) for r in ref]]
        dist.broadcast_object_list(feed, src=0)
        feed = feed[0]
        results = {}
        # "layer": batch 1 (the first sequence) through the one-kernel-per-layer path, whose sums over ranks run
        # inside the layer kernel
        # "peer-wide": 12 rows (the first two sequences repeated), above the range of the matmul kernel with the sum
        # inside it: mid-batch matmul into the peer-mapped buffer + b200_allreduce_peer
        wide = 12
        # "peer-one": batch 1 through the separate kernels (fused prologues, rotary embedding in the qkv matmul's epilogue,
        # sums over ranks inside the o / down matmuls)
        for name, w, peer in (("single", 1, False), ("nccl", world, False), ("peer", world, True), ("layer", world, True),
                              ("peer-wide", world, True), ("peer-one", world, True)):
            r = 0 if w == 1 else rank
            nb = 1 if name in ("layer", "peer-one") else wide if name == "peer-wide" else B
            layers = [decoder.to_device(tp.shard_layer(l, r, w, cfg.hidden, cfg.inter), dev) for l in full]
            vl = cfg.vocab // w
            eng = decoder.DecodeEngine(cfg, layers, embed, fnorm, embed[r * vl:(r + 1) * vl].contiguous(), nb, max_ctx, dev,
                                       rank=r, world=w, peer_reduce=peer, layer_kernel=(name == "layer"))
            assert (eng.peer is not None) == peer and eng.layer_kernel == (name == "layer")
            assert (nb > eng.PEER_FUSED_MAX_ROWS) == (name == "peer-wide")
            assert eng.rope_epilogue == (name == "peer-one")
            rows = [j % B for j in range(nb)]           # which of the oracle's sequences each row repeats
            eng.tokens.copy_(torch.tensor([tokens[j] for j in rows], dtype=torch.int32))
            hs, ls = [], []
            for st in range(steps):
                if st > 0:
                    eng.tokens.copy_(torch.from_numpy(feed[st - 1][rows]))
                eng.step()
                torch.cuda.synchronize()
                hs.append(eng.h.float().cpu().numpy().copy())
                ls.append(eng.logits.float().cpu().numpy().copy())
            results[name] = (hs, ls)
            assert _lib.lib().b200_device_error_flags() == 0
            dist.barrier()
        if rank == 0:
            errs = {}
            for name in ("single", "nccl", "peer", "layer", "peer-wide", "peer-one"):
                e_or, e_l = 0.0, 0.0
                nb = results[name][0][0].shape[0]
                rows = [j % B for j in range(nb)]
                for st in range(steps):
                    h_ref = ref[st][0].astype(np.float32)[rows]
                    l_ref = ref[st][1].astype(np.float32)[rows]
                    e_or = max(e_or, float(np.abs(results[name][0][st] - h_ref).max() / np.abs(h_ref).max()))
                    e_l = max(e_l, float(np.abs(results[name][1][st] - l_ref).max() / np.abs(l_ref).max()))
                e_single = max(float(np.abs(a - b[rows]).max() / np.abs(b[rows]).max()) for a, b in zip(results[name][0], results["single"][0]))
                errs[name] = (e_or, e_l, e_single)
            ret["errs"] = errs
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,hidden,heads,inter", [(2, 1024, 8, 1280), (4, 2048, 16, 2816), (8, 2048, 16, 2816)])
def test_tensor_parallel_decode_matches_oracle(world, hidden, heads, inter):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    import torch.multiprocessing as mp

    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_worker, args=(world, port, ret, hidden, heads, inter), nprocs=world, join=True)
    errs = dict(ret["errs"])
    # the decoder tolerance of the one-GPU tests: 1e-2 of the tensor's scale, after 3 steps x 2 layers.  K slices
    # change the fp32 summation order and add one fp16 rounding per rank's partial result.
    for name, (e_oracle, e_logits, e_single) in errs.items():
        assert e_oracle < 1e-2 and e_logits < 1e-2, (name, errs)
        assert e_single < 1e-2, (name, errs)
