#!/usr/bin/env python
"""Benchmark of the q4f16 hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload gemv|prefill] [--impl reference]

One JSON line on stdout (rank 0).  A "step" is one pass of the hot path over one batch of
synthetic input:

* ``gemv`` (default): the decode matmul of the first benchmark config (x fp16 [1,4096], W int4
  [4096,4096] group 32), launched over ``copies`` DISTINCT weight sets back to back so that the
  working set (copies x 9.45 MB) is several times the 126 MB L2 and every launch streams its
  weights from HBM; the pass over the copies is repeated ``--reps`` times per step so that a step
  lasts several milliseconds.  value = algorithmic bytes moved per second.
* ``prefill``: the tensor-core dequant-GEMM of the second config (M=2048, N=11008, K=4096);
  value = TFLOP/s.

The default line also carries a ``prefill`` object (the second config measured the same way) and a
``decode`` list: tokens/s of the 7B-shaped decoder at batch 1, 16 and 64, each with the parity of one
step against an independent one-GPU engine.

With --gpus N > 1 (launched under torchrun) every rank runs the same independent stream of
matmuls on its own GPU (the matmul path shards by rows of W with no exchange): weak scaling,
value = sum over ranks of bytes / max over ranks of time.

``--impl reference`` times the CPU restatement of the reference's path (oracle/, OpenMP over all
host cores) on the same config and metric; rank 0 only.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

import numpy as np  # noqa: E402


def algorithmic_bytes(m, n, k):
    """Packed weights + scales + activation + output: what a launch must move at least."""
    return n * k // 2 + n * (k // 32) * 2 + m * k * 2 + m * n * 2


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        d = json.load(open(path))
        return {"hbm_gbs": d["hbm_gbs"], "tflops": d["bf16_tflops"], "tflops_sustained": d["bf16_tflops_sustained"],
                "source": "measured"}
    return {"hbm_gbs": 6650.0, "tflops": 1590.0, "tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clocks and throttle reasons while the timed region runs: through NVML every
    5 ms when the bindings are importable, else with an `nvidia-smi -lms` child process."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.proc = None
        self.lines = []

    def _nvml_sample(self):
        nv, h = self.nv, self.nv_handle
        self.nv_sm.append(nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM))
        r = nv.nvmlDeviceGetCurrentClocksThrottleReasons(h)
        for name, bit in self.nv_bad.items():
            if r & bit:
                self.nv_reasons.add(name)

    def _nvml_loop(self):
        while not self.stop_flag:
            self._nvml_sample()
            time.sleep(0.005)

    def start(self):
        self.stop_flag, self.nv_sm, self.nv_reasons, self.nv_max, self.nv_thread = False, [], set(), None, None
        try:
            import pynvml as nv

            nv.nvmlInit()
            # NVML orders devices by PCI bus id; honour CUDA_VISIBLE_DEVICES remapping when it is a plain list
            vis = os.environ.get("CUDA_VISIBLE_DEVICES")
            if vis and all(v.strip().isdigit() for v in vis.split(",")):
                self.index = int(vis.split(",")[self.index])
            # handle and limits are fetched here, before the timed region, so that the thread's first
            # sample falls inside it even when the region lasts only tens of milliseconds
            self.nv = nv
            self.nv_handle = nv.nvmlDeviceGetHandleByIndex(self.index)
            self.nv_bad = {"hw_slowdown": nv.nvmlClocksThrottleReasonHwSlowdown,
                           "hw_thermal_slowdown": nv.nvmlClocksThrottleReasonHwThermalSlowdown,
                           "sw_thermal_slowdown": nv.nvmlClocksThrottleReasonSwThermalSlowdown,
                           "sw_power_cap": nv.nvmlClocksThrottleReasonSwPowerCap}
            self.nv_max = nv.nvmlDeviceGetMaxClockInfo(self.nv_handle, nv.NVML_CLOCK_SM)
            self.nv_thread = threading.Thread(target=self._nvml_loop, daemon=True)
            self.nv_thread.start()
            return
        except Exception:
            self.nv_thread = None
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._pump, daemon=True).start()
        except OSError:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.nv_thread is not None:
            self.stop_flag = True
            self.nv_thread.join(timeout=1.0)
            return {"sm_mhz": float(np.median(self.nv_sm)) if self.nv_sm else None, "sm_max_mhz": self.nv_max,
                    "reasons": sorted(self.nv_reasons), "samples": len(self.nv_sm), "via": "nvml"}
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        sm, mx, reasons = [], [], set()
        for ln in self.lines:
            parts = [p.strip() for p in ln.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), parts[3:7]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


# ------------------------------------------------------------------------------------------ CPU arm
def host_cores():
    """Cores this process may run on (the launcher's OMP_NUM_THREADS=1 is not a property of the host)."""
    try:
        return max(1, len(os.sched_getaffinity(0)))
    except AttributeError:
        return max(1, os.cpu_count() or 1)


def cpu_time_matmul(m, n, k, seed, budget_s=12.0, max_reps=50, threads=None):
    """Times the oracle (C restatement, OpenMP over rows of W) on one matmul with `threads` threads (default:
    every core of the host); returns (s/matmul, threads, reps)."""
    import oracle
    from relax_b200 import synth

    x, wq, s = synth.make_case(m, n, k, seed=seed)
    threads = int(threads or host_cores())
    oracle.c_matmul(x, wq, s, nthreads=threads)  # warm-up (page faults, thread pool)
    reps, t0 = 0, time.perf_counter()
    while reps < max_reps and (time.perf_counter() - t0) < budget_s:
        oracle.c_matmul(x, wq, s, nthreads=threads)
        reps += 1
    return (time.perf_counter() - t0) / reps, threads, reps


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return 0
    if args.workload == "gemv":
        m, n, k = 1, 4096, 4096
        times = []
        for _ in range(args.warmup):
            cpu_time_matmul(m, n, k, seed=0, budget_s=0.2, max_reps=2)
        for _ in range(args.steps):
            t, threads, reps = cpu_time_matmul(m, n, k, seed=0, budget_s=max(0.5, 20.0 / args.steps), max_reps=200)
            times.append(t)
        per = float(np.mean(times))
        value = algorithmic_bytes(m, n, k) / per / 1e9
        unit, metric = "GB/s", "q4f16 dequant-GEMV HBM GB/s"
        sample = f"{args.steps} steps x up to 200 repeats of the full 1x4096x4096 matmul"
        config = {"workload": "q4f16 decode GEMV M=1 N=4096 K=4096 group32"}
    else:
        m, n, k = 2048, 11008, 4096
        ms = 64  # bounded sample: 64 of the 2048 rows of x; cost is linear in M
        t, threads, reps = cpu_time_matmul(ms, n, k, seed=1, budget_s=20.0, max_reps=max(1, args.steps))
        per = t * (m / ms)
        value = 2.0 * m * n * k / per / 1e12
        unit, metric = "TFLOP/s", "q4f16 prefill dequant-GEMM TFLOP/s"
        sample = f"{ms} of {m} activation rows, time scaled linearly to M={m}"
        config = {"workload": "q4f16 prefill dequant-GEMM M=2048 N=11008 K=4096 group32"}
    line = {
        "impl": "reference", "metric": metric, "value": value, "unit": unit, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": per * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f16 (fp32 accumulate)", "data": "synthetic", "config": config,
        "cpu_baseline": {"value": value, "unit": unit, "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "note": "CPU restatement of the reference's LLVM path (oracle/q4f16_oracle.c), OpenMP over rows of W; "
                "the reference itself cannot be built here (no LLVM, empty submodules)",
    }
    print(json.dumps(line), flush=True)
    return 0


# ------------------------------------------------------------------------------------------ decode (7B shape)
def _n1_store():
    """Where rank 0 of a one-GPU run leaves its decode figures for later runs on more GPUs of the same box (the
    denominators of decode[].scaling_efficiency)."""
    import tempfile

    return os.path.join(tempfile.gettempdir(), "b200_q4f16_bench_decode_n1.json")


def run_decode(args, world, rank, dev, batches):
    """Tokens/s of a 32-layer 7B-shaped random-init q4f16 decoder at context 2048, tensor-parallel over
    `world` GPUs (column-/row-parallel matmuls, the sum over ranks after o and down), for every batch in
    `batches`.  One CUDA graph per token.  After the timed region one more step runs eagerly at a fixed position
    and its logits are compared with an independent one-GPU engine on rank 0 (separate RMSNorm / SwiGLU
    kernels, no fused sum, full weights from the same seeds) on the first sequences of the batch.
    Returns a list of dicts (meaningful on rank 0)."""
    import torch
    import torch.distributed as dist

    from relax_b200 import decoder, tp

    cfg = decoder.DecoderConfig()
    steps, warmup = args.decode_steps, 3
    ctx = 2048
    max_ctx = ctx
    start = ctx - steps - warmup - 2 * (steps + warmup) - 2   # room for the graph, eager and e2e passes
    parity_pos = start - 1                                     # every cache entry below it is still the synthetic one
    layers, full_layers = [], []
    for i in range(cfg.layers):
        full = decoder.synth_layer_torch(cfg, 1000 + i, dev)
        layers.append(tp.shard_layer(full, rank, world, cfg.hidden, cfg.inter))
        if rank == 0 and world > 1 and not args.no_decode_parity:
            full_layers.append(tp.shard_layer(full, 0, 1, cfg.hidden, cfg.inter))
        del full
    if world == 1:
        full_layers = layers
    gen = torch.Generator(device=dev)
    gen.manual_seed(7)
    embed = (0.02 * torch.randn((cfg.vocab, cfg.hidden), device=dev, generator=gen)).to(torch.float16)
    vl = cfg.vocab // world
    lm_head = embed[rank * vl:(rank + 1) * vl].contiguous()      # tied fp16 head, vocabulary-sharded
    final_norm = torch.ones(cfg.hidden, dtype=torch.float16, device=dev)
    n1 = {}
    if world > 1 and os.path.exists(_n1_store()):
        try:
            n1 = json.load(open(_n1_store()))
        except (OSError, ValueError):
            n1 = {}
    results = []

    def barrier():
        torch.cuda.synchronize(dev)
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(dev)

    for batch in batches:
        eng = decoder.DecodeEngine(cfg, layers, embed, final_norm, lm_head, batch, max_ctx, dev, rank, world,
                                   peer_reduce=not args.decode_nccl,
                                   fused_attention="rope" if args.decode_attn2 else args.decode_attn1,
                                   layer_kernel=(None if args.decode_layer_kernel < 0 else bool(args.decode_layer_kernel)))
        bp = min(batch, 4)                                            # sequences checked by the parity step
        ref = None
        if rank == 0 and not args.no_decode_parity:
            ref = decoder.DecodeEngine(cfg, full_layers, embed, final_norm, embed, bp, max_ctx, dev, 0, 1, fused=False,
                                       peer_reduce=False)
        # a full context of N(0,1) keys and values, the same whatever the number of ranks: every layer's cache is
        # drawn for all heads and each rank keeps its heads
        nhl = eng.nh_local
        for i in range(cfg.layers):
            g = torch.Generator(device=dev)
            g.manual_seed(50000 + i)
            for cache, rcache in ((eng.kc[i], ref.kc[i] if ref else None), (eng.vc[i], ref.vc[i] if ref else None)):
                for b0 in range(0, batch, 8):                         # 8 sequences at a time bounds the transient
                    b1 = min(batch, b0 + 8)
                    t = torch.randn((b1 - b0, max_ctx, cfg.heads, 128), device=dev, generator=g).to(torch.float16)
                    cache[b0:b1].copy_(t[:, :, rank * nhl:(rank + 1) * nhl])
                    if rcache is not None and b0 < bp:
                        rcache[b0:min(bp, b1)].copy_(t[:min(bp, b1) - b0])
                    del t
        tok0 = (torch.arange(batch, dtype=torch.int32, device=dev) * 37 + 11) % cfg.vocab
        eng.tokens.copy_(tok0)
        eng.set_position(start)
        torch.cuda.synchronize(dev)
        stream = torch.cuda.Stream(device=dev)
        eng.capture(stream)

        def timed(fn, n):
            barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            with torch.cuda.stream(stream):
                e0.record(stream)
                for _ in range(n):
                    fn()
                e1.record(stream)
            barrier()
            ms = e0.elapsed_time(e1)
            if world > 1:
                t = torch.tensor([ms], device=dev)
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
                ms = float(t.item())
            return ms

        with torch.cuda.stream(stream):
            for _ in range(warmup):
                eng.graph.replay()
        ms = timed(eng.graph.replay, steps)
        # end to end: the host feeds the token ids of every step and reads the sampled ids back
        tok_host = torch.zeros((batch,), dtype=torch.int32).pin_memory()

        def e2e_step():
            eng.tokens.copy_(tok_host, non_blocking=True)
            eng.graph.replay()
            tok_host.copy_(eng.tokens, non_blocking=True)
            stream.synchronize()

        with torch.cuda.stream(stream):
            for _ in range(warmup):
                e2e_step()
        ms_e2e = timed(e2e_step, steps)
        end_pos = int(eng.pos.item())
        err = eng.L.b200_device_error_flags()
        if err:
            raise RuntimeError(f"device error flags {err:#x} after the decode run")

        # ---- parity of one step (outside every timed region)
        parity, parity_rows, parity_overflow = None, 0, 0
        if not args.no_decode_parity:
            barrier()
            with torch.cuda.stream(stream):
                eng.set_position(parity_pos)
                eng.tokens.copy_(tok0)
                eng.step()
                stream.synchronize()
            got = eng.logits[:bp].float()
            if rank == 0:
                with torch.cuda.stream(stream):
                    ref.set_position(parity_pos)
                    ref.tokens.copy_(tok0[:bp])
                    ref.step()
                    stream.synchronize()
                want = ref.logits.float()
                # A random-init model with these weight statistics overflows fp16 in the residual stream for some
                # token sequences (the CPU oracle does the same: fp16 semantics, not a kernel property).  Such a
                # sequence must be non-finite in BOTH engines; the others are compared.
                ok_g, ok_w = torch.isfinite(got).all(dim=1), torch.isfinite(want).all(dim=1)
                parity_overflow = int((~ok_g & ~ok_w).sum())
                if bool((ok_g != ok_w).any()):
                    parity = 1.0                                      # one engine overflowed where the other did not
                elif bool(ok_w.any()):
                    parity_rows = int(ok_w.sum())
                    parity = float(((got[ok_w] - want[ok_w]).abs().amax(dim=1) / want[ok_w].abs().amax(dim=1)).max())
            barrier()

        # weights + KV + lm_head actually read per token by one rank
        wbytes = sum(a.numel() * a.element_size() for l in layers for k in ("qkv", "o", "gu", "down") for a in l[k])
        kvbytes = 2 * cfg.layers * batch * end_pos * eng.nh_local * 128 * 2
        per_rank = wbytes + kvbytes + lm_head.numel() * 2
        value = batch * steps / (ms * 1e-3)
        out = {
            "metric": "7B-shape decode tokens/s", "batch": batch, "context": end_pos, "tp": world,
            "value": value, "unit": "tokens/s", "ms_per_token_step": ms / steps,
            "e2e": {"value": batch * steps / (ms_e2e * 1e-3), "unit": "tokens/s", "h2d_bytes_per_step": 4 * batch,
                    "d2h_bytes_per_step": 4 * batch},
            "bytes_per_step_per_gpu": per_rank,
            "hbm_frac_of_measured": per_rank / (ms / steps * 1e-3) / 1e9 / measured_peaks()["hbm_gbs"],
            "kernels_per_step": eng.kernels_per_step(), "engine": "one persistent kernel per layer" if eng.layer_kernel else
            "fused prologues, skinny kernels" if eng.fused else
            "separate RMSNorm/SwiGLU kernels, mid-batch tensor-core matmul",
            "lm_head": ("fp16, tied to the embedding, vocabulary-sharded; this library's kernel (b200_lm_head)"
                        + (", greedy token inside it" if world == 1 else ", torch argmax over the gathered slices")
                        if batch <= 16 else "fp16, tied to the embedding, vocabulary-sharded (library GEMM + torch argmax above 16 rows)"),
            "allreduce": (None if world == 1 else "NCCL fp16, 2 per layer" if eng.peer is None else
                          "fused into the o/down matmul kernels over NVLink peer memory (fp16 partials, rank-order sum)"
                          if batch <= eng.PEER_FUSED_MAX_ROWS else
                          "this library's peer-memory sum (b200_allreduce_peer) behind the o/down matmuls (fp16 partials, rank-order sum)"),
            "steps": steps,
            "parity_max_rel": parity,
            "parity_against": None if args.no_decode_parity else
            f"one-GPU engine on rank 0 (unfused kernels, same seeds), logits of the first {bp} sequence(s) at position {parity_pos}: "
            f"{parity_rows} compared, {parity_overflow} overflow fp16 in both engines alike",
            "scaling_efficiency": (value / (world * n1[str(batch)]) if world > 1 and str(batch) in n1 else None),
        }
        results.append(out)
        del eng, ref
        torch.cuda.empty_cache()
    if world == 1 and rank == 0:
        try:
            json.dump({str(r["batch"]): r["value"] for r in results}, open(_n1_store(), "w"))
        except OSError:
            pass
    del layers, full_layers
    torch.cuda.empty_cache()
    return results


# dram__bytes_read.sum + dram__bytes_write.sum per launch of the dominant kernel, from the ncu captures
# summarised under profiles/ (one capture per kernel change; not re-measured by this script).
NCU_TRAFFIC_BYTES = {
    ("gemv", 1, 4096, 4096): (9476352, "profiles/gemv_pipe_kernel__decode_gemv_M1_N4096_K4096.md (ncu capture, not re-measured by this run)"),
    ("gemv", 64, 4096, 4096): (10006272, "profiles/gemm_ws_tcgen05_kernel__mid_batch_M64_N4096_K4096.md (ncu capture, not re-measured by this run)"),
    ("prefill", 2048, 11008, 4096): (42236416 + 2993664, "profiles/gemm_tcgen05_kernel__prefill_M2048_N11008_K4096.md (ncu capture, not re-measured by this run)"),
}


# ------------------------------------------------------------------------------------------ GPU arm
def measure_matmul(args, workload, world, rank, dev, steps, warmup, reps, with_cpu):
    """One workload ("gemv" or "prefill") on this rank's GPU: device-resident figure from a CUDA graph of `copies`
    launches replayed `reps` times per step, end-to-end figure through b200_q4f16_matmul_host with pinned host
    activations and results.  Returns the fields of a bench line (rank 0: complete)."""
    import torch
    import torch.distributed as dist

    from relax_b200 import _lib, ops, synth

    L = _lib.lib()
    peaks = measured_peaks()
    if workload == "gemv":
        m, n, k = 1, 4096, 4096
        copies = args.copies
        metric, unit = "q4f16 dequant-GEMV HBM GB/s", "GB/s"
    else:
        m, n, k = 2048, 11008, 4096
        copies = 2
        metric, unit = "q4f16 prefill dequant-GEMM TFLOP/s", "TFLOP/s"
    if args.shape and workload == args.workload:
        m, n, k = (int(v) for v in args.shape.split(","))
    per_launch_bytes = algorithmic_bytes(m, n, k)
    weights = [synth.make_weights_torch(n, k, 1000 * rank + i, dev) for i in range(copies)]
    x_host = torch.from_numpy(synth.make_case(m, 8, k, seed=rank)[0]).pin_memory()
    y_host = torch.empty((m, n), dtype=torch.float16).pin_memory()
    x = x_host.to(dev)
    ys = [torch.empty((m, n), dtype=torch.float16, device=dev) for _ in range(copies)]
    stream = torch.cuda.Stream(device=dev)
    sp = stream.cuda_stream

    def pass_device():
        for (wq, s), y in zip(weights, ys):
            rc = L.b200_q4f16_matmul(x.data_ptr(), wq.data_ptr(), s.data_ptr(), y.data_ptr(), m, n, k, sp)
            if rc:
                raise RuntimeError(_lib.last_error())

    def step_e2e():
        # the call a user of the plugin makes, with HOST activation and result buffers
        for _ in range(reps):
            for (wq, s), y in zip(weights, ys):
                rc = L.b200_q4f16_matmul_host(x_host.data_ptr(), x.data_ptr(), wq.data_ptr(), s.data_ptr(), y.data_ptr(),
                                              y_host.data_ptr(), m, n, k, sp)
                if rc:
                    raise RuntimeError(_lib.last_error())

    # One CUDA graph per pass for the device-resident measurement (a 1.5 us kernel is shorter than
    # a launch; a decoder replays exactly such a graph).
    with torch.cuda.stream(stream):
        pass_device()
        stream.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            pass_device()

    def step_device():
        for _ in range(reps):
            if args.no_graph:
                pass_device()
            else:
                graph.replay()

    def barrier():
        torch.cuda.synchronize(dev)
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(dev)

    def timed(fn, nsteps, nwarm):
        with torch.cuda.stream(stream):
            for _ in range(nwarm):
                fn()
        barrier()
        e0 = torch.cuda.Event(enable_timing=True)
        e1 = torch.cuda.Event(enable_timing=True)
        with torch.cuda.stream(stream):
            e0.record(stream)
            for _ in range(nsteps):
                fn()
            e1.record(stream)
        barrier()
        ms = e0.elapsed_time(e1)
        if world > 1:
            t = torch.tensor([ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms

    sampler = ClockSampler(dev.index or 0)
    if rank == 0:
        sampler.start()
    ops.reset_launch_count()
    ms_total = timed(step_device, steps, warmup)
    clocks = sampler.stop() if rank == 0 else None
    launches = steps * reps * copies  # graph replays do not pass through the library's launch counter
    ms_e2e = timed(step_e2e, steps, max(1, warmup))
    err = L.b200_device_error_flags()
    if err:
        raise RuntimeError(f"device error flags {err:#x}")
    del weights, ys
    torch.cuda.empty_cache()

    ms_per_step = ms_total / steps
    us_per_launch = ms_per_step * 1e3 / (copies * reps)
    traffic, traffic_source = NCU_TRAFFIC_BYTES.get((workload, m, n, k), (None, None))
    sm_mhz = (clocks or {}).get("sm_mhz")
    if workload == "gemv":
        value = world * copies * reps * per_launch_bytes / (ms_per_step * 1e-3) / 1e9
        e2e_value = world * copies * reps * per_launch_bytes / (ms_e2e / steps * 1e-3) / 1e9
        achieved = per_launch_bytes / (us_per_launch * 1e-6) / 1e9
        roofline = {"bound": "hbm", "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                    "frac": achieved / peaks["hbm_gbs"], "traffic": traffic, "traffic_source": traffic_source,
                    "peak_source": peaks["source"], "kernel": "q4f16_gemv_pipe_kernel", "us_per_launch": us_per_launch,
                    "us_x_sm_mhz": us_per_launch * sm_mhz if sm_mhz else None,
                    "algorithmic_bytes_per_launch": per_launch_bytes}
    else:
        flops = 2.0 * m * n * k
        value = world * copies * reps * flops / (ms_per_step * 1e-3) / 1e12
        e2e_value = world * copies * reps * flops / (ms_e2e / steps * 1e-3) / 1e12
        achieved = flops / (us_per_launch * 1e-6) / 1e12
        roofline = {"bound": "tensor", "achieved": achieved, "peak": peaks["tflops"], "unit": "TFLOP/s",
                    "frac": achieved / peaks["tflops"], "frac_of_sustained": achieved / peaks["tflops_sustained"],
                    "frac_of_nominal_2250": achieved / 2250.0, "traffic": traffic, "traffic_source": traffic_source,
                    "peak_source": peaks["source"], "kernel": "q4f16_gemm_tcgen05_kernel", "us_per_launch": us_per_launch,
                    "us_x_sm_mhz": us_per_launch * sm_mhz if sm_mhz else None,
                    "algorithmic_flops_per_launch": flops}
    cpu = None
    if rank == 0 and with_cpu:
        # CPU baseline on a bounded sample, rank 0, N=1 only: every core of the host, and one thread beside it
        if workload == "gemv":
            t, threads, nrep = cpu_time_matmul(m, n, k, seed=0, budget_s=8.0, max_reps=300)
            t1, _, _ = cpu_time_matmul(m, n, k, seed=0, budget_s=3.0, max_reps=50, threads=1)
            cpu = {"value": per_launch_bytes / t / 1e9, "unit": "GB/s", "cores": threads, "kind": "port",
                   "sample": f"{nrep} repeats of the full {m}x{n}x{k} matmul", "value_1_thread": per_launch_bytes / t1 / 1e9}
        else:
            ms_ = 32
            t, threads, nrep = cpu_time_matmul(ms_, n, k, seed=1, budget_s=10.0, max_reps=3)
            cpu = {"value": 2.0 * m * n * k / (t * m / ms_) / 1e12, "unit": "TFLOP/s", "cores": threads,
                   "kind": "port", "sample": f"{ms_} of {m} activation rows, scaled linearly"}
    return {
        "metric": metric, "value": value, "unit": unit, "n_gpus": world, "steps": steps, "warmup": warmup,
        "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f16 (int4 weights, fp32 accumulate)", "data": "synthetic",
        "config": {"workload": f"q4f16 {'decode GEMV' if workload == 'gemv' else 'prefill dequant-GEMM'} "
                               f"M={m} N={n} K={k} group32",
                   "launches_per_step": copies * reps,
                   "l2": f"{copies} distinct weight sets ({copies * per_launch_bytes / 1e6:.0f} MB) rotate through "
                         f"each pass ({reps} passes per step), larger than the 126 MB L2"},
        "roofline": roofline, "cpu_baseline": cpu,
        "e2e": {"value": e2e_value, "unit": unit, "h2d_bytes_per_step": copies * reps * m * k * 2,
                "d2h_bytes_per_step": copies * reps * m * n * 2},
        "gpu_launches": launches, "clocks": clocks,
    }


def run_gpu(args):
    import torch
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    if args.decode_only:
        decode = run_decode(args, world, rank, dev, args.decode_batches)
        if rank == 0:
            d0 = decode[0]
            print(json.dumps({"metric": d0["metric"], "value": d0["value"], "unit": d0["unit"], "n_gpus": world,
                              "steps": d0["steps"], "warmup": 3, "ms_per_step": d0["ms_per_token_step"],
                              "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
                              "dtype": "f16 (int4 weights, fp32 accumulate)", "data": "synthetic",
                              "config": {"workload": f"7B-shaped decode, batch {d0['batch']}, context {d0['context']}, tp {world}"},
                              "e2e": d0["e2e"], "gpu_launches": d0["kernels_per_step"] * d0["steps"], "decode": decode}),
                  flush=True)
        if world > 1:
            dist.destroy_process_group()
        return 0

    reps = args.reps if args.reps else (50 if args.workload == "gemv" else 10)
    line = measure_matmul(args, args.workload, world, rank, dev, args.steps, args.warmup, reps,
                          with_cpu=(world == 1 and not args.no_cpu))
    if args.workload == "gemv" and not args.no_prefill:
        # the second benchmark config beside the headline: 20 steps of 20 GEMMs (about 70 ms of tensor-core work)
        pre = measure_matmul(args, "prefill", world, rank, dev, 20, 3, 10, with_cpu=False)
        line["prefill"] = {k: pre[k] for k in ("metric", "value", "unit", "ms_per_step", "config", "roofline", "e2e", "clocks",
                                                 "gpu_launches", "steps", "warmup", "scaling")}
    if args.workload == "gemv" and not args.no_decode:
        decode = run_decode(args, world, rank, dev, args.decode_batches)
        line["decode"] = decode
    if rank == 0:
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=None)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--workload", choices=["gemv", "prefill"], default="gemv")
    ap.add_argument("--copies", type=int, default=40, help="distinct weight sets per pass (gemv)")
    ap.add_argument("--reps", type=int, default=0, help="passes over the weight sets per step (0 = 50 for gemv, 10 for prefill)")
    ap.add_argument("--impl", choices=["b200", "reference"], default="b200")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--shape", default=None, help="M,N,K override (profiling of other shapes of the same kernels)")
    ap.add_argument("--no-graph", action="store_true", help="launch directly instead of replaying a CUDA graph")
    ap.add_argument("--no-decode", action="store_true", help="skip the 7B-shaped decode measurement")
    ap.add_argument("--no-prefill", action="store_true", help="skip the prefill object of the default line")
    ap.add_argument("--no-decode-parity", action="store_true", help="skip the parity step of the decode measurement")
    ap.add_argument("--decode-only", action="store_true",
                    help="only the 7B-shaped decode measurement, as the line's own metric (for profiling the decode step)")
    ap.add_argument("--decode-attn1", action="store_true", help="rotary + attention + merge as one launch (measured slightly slower in a graph)")
    ap.add_argument("--decode-attn2", action="store_true", help="rotary + KV append inside the attention launch, merge as a second launch")
    ap.add_argument("--decode-layer-kernel", type=int, default=-1,
                    help="batch 1: 1 = one persistent kernel per layer, 0 = seven launches per layer, -1 = the engine's default")
    ap.add_argument("--decode-nccl", action="store_true", help="tensor-parallel sums through NCCL instead of the fused kernel")
    ap.add_argument("--decode-steps", type=int, default=32, help="timed tokens per sequence of the decode measurement")
    ap.add_argument("--decode-batches", type=lambda v: [int(x) for x in v.split(",")], default=[1, 16, 64],
                    help="batch sizes of the decode measurement, e.g. 1,16,64")
    args = ap.parse_args()
    if args.steps is None:
        # gemv: 20 steps x 2000 launches; prefill: 10 steps x 20 GEMMs = 36 ms of back-to-back GEMMs, the regime the
        # burst peak is measured in (at 115 ms the same kernel is 6 % slower, at 0.4 s 10 % with sw_power_cap active)
        args.steps = {"gemv": 20, "prefill": 10}[args.workload] if args.impl == "b200" else 10
    if args.warmup < 3:
        args.warmup = 3
    if args.impl == "reference":
        return run_reference(args)
    return run_gpu(args)


if __name__ == "__main__":
    sys.exit(main())
