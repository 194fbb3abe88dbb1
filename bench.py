#!/usr/bin/env python3
"""Benchmark of the attention + KV-cache hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--config C2]

One "step" is one pass of the path over one prompt of the workload: for C2 (the default, the
configuration the metric is quoted on) KV append + causal GQA attention for the 4096-token prompt
in 512-token chunks, then one decode step at context 4096.  `value` is prefill tokens per second
with inputs resident in HBM; `decode` reports the KV bytes per second of the decode step; `e2e` is
the same prefill through hc_layer_step_host with pinned HOST buffers (copies inside the timed
region).  With N > 1 (launched by torch.distributed.run, one rank per GPU) the 8 KV heads are
sharded N ways with no exchange inside attention; the time is the maximum over ranks.

`--impl reference` times the reference's CPU algorithm (the oracle restating HydraReference, the
Swift original cannot be built here) on the host cores, on a bounded sample of the same workload.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return {"hbm_gbs": p["hbm_gbs"], "bf16_tflops": p["bf16_tflops"],
                "bf16_tflops_sustained": p["bf16_tflops_sustained"], "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, sm_max, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 9:
                continue
            try:
                sm.append(float(parts[1]))
                sm_max.append(float(parts[2]))
            except ValueError:
                continue
            for name, flag in zip(names, parts[5:9]):
                if flag.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None,
                "sm_max_mhz": max(sm_max) if sm_max else None,
                "samples": len(sm), "reasons": sorted(reasons)}


def dist_setup(n_gpus: int):
    import torch
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1:
        import torch.distributed as dist
        torch.cuda.set_device(local)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    else:
        torch.cuda.set_device(0)
        local = 0
    if world != max(n_gpus, 1) and rank == 0:
        print(f"warning: --gpus {n_gpus} but WORLD_SIZE {world}", file=sys.stderr)
    return rank, world, local


def barrier(world):
    import torch
    torch.cuda.synchronize()
    if world > 1:
        import torch.distributed as dist
        dist.barrier()
    torch.cuda.synchronize()


def max_over_ranks(value: float, world: int) -> float:
    if world == 1:
        return value
    import torch
    import torch.distributed as dist
    t = torch.tensor([value], device="cuda", dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


# ---- the reference arm: the oracle on the host cores ---------------------------------------------

def cpu_sample(cfg_name: str, rows_per_step: int, steps: int, threads: int):
    """Times the oracle on `rows_per_step` query tokens of the workload per step.  The tokens sit at
    the midpoints of equal slices of the prompt, so their mean context equals the prompt's."""
    from hydra_b200 import workloads as wl
    from oracle import hydra_oracle as ho
    cfg = wl.config(cfg_name)
    inputs = wl.Inputs(cfg, device="cpu")
    entry, spec = inputs.layers[0], cfg.layers[0]
    prompt = cfg.prompt
    stride = prompt / rows_per_step
    rows = np.array([int(stride * (i + 0.5)) for i in range(rows_per_step)])
    inv = ho.inverse_frequencies(cfg.head_dim, spec.theta)
    allpos = np.arange(prompt)
    cos, sin = ho.rope_tables(inv, allpos, as_float32=True)
    k = ho.prepare_heads(entry["k"][:prompt], None, False, 1e-6, cos, sin, threads=threads)
    times = []
    for _ in range(steps):
        t0 = time.perf_counter()
        q = ho.prepare_heads(entry["q"][rows], None, False, 1e-6, cos[rows], sin[rows], threads=threads)
        ho.attention_rows(q, rows, k, entry["v"][:prompt], cfg.scale, spec.window, sinks=entry["sinks"],
                          threads=threads)
        times.append(time.perf_counter() - t0)
    return rows_per_step, times


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return 0
    from oracle import hydra_oracle as ho
    threads = ho.hardware_threads()
    rows = 128
    for _ in range(max(args.warmup, 0)):
        cpu_sample(args.config, 16, 1, threads)
    n, times = cpu_sample(args.config, rows, max(args.steps, 1), threads)
    total = sum(times)
    value = n * len(times) / total
    line = {
        "impl": "reference", "metric": "attn_prefill_tok_s", "value": value, "unit": "tok/s",
        "n_gpus": args.gpus, "steps": len(times), "warmup": args.warmup,
        "ms_per_step": 1e3 * total / len(times), "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "f64", "data": "synthetic",
        "config": {"workload": f"{args.config}: attention of {rows} sampled query tokens per step over the "
                               "4096-token bf16 K/V history (mean context = the prompt's), 64q/8kv d64, sinks"},
        "cpu_baseline": {"value": value, "unit": "tok/s", "cores": threads, "kind": "port",
                         "sample": f"{rows} query tokens at slice midpoints of the 4096-token prompt, all 64 heads, "
                                   "double precision, two-pass softmax"},
        "e2e": {"value": value, "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))
    return 0


# ---- the CUDA arm -----------------------------------------------------------------------------------

def run_cuda(args):
    import torch
    import hydra_b200 as hb
    from hydra_b200 import workloads as wl

    rank, world, local = dist_setup(args.gpus)
    peaks = measured_peaks()
    full = wl.config(args.config)
    if full.kv_heads % world != 0:
        raise SystemExit(f"{full.kv_heads} KV heads cannot be sharded over {world} GPUs")
    per = full.kv_heads // world
    cfg = wl.config(args.config, kv_heads=per)
    ctx = hb.Context(local)
    inputs = wl.Inputs(cfg, full_heads=full, head_offset=rank * per)

    # Rotate over several copies of the prompt's buffers so that a step's inputs are not in L2 from
    # the step before: the copies together exceed twice the 126 MB L2.
    d = cfg.head_dim
    set_bytes = cfg.prompt * (2 * cfg.q_heads * d + 2 * cfg.kv_heads * d) * 2 + 2 * cfg.context * cfg.kv_heads * d * 2
    n_sets = max(2, int(np.ceil(2 * 126e6 / max(set_bytes, 1))))
    n_sets = min(n_sets, 64)
    cfg.batch = n_sets
    run = wl.PathRunner(ctx, cfg, inputs)
    dev, params, backend, cache = run.dev[0], run.params[0], run.backend, run.cache
    q_sets = [dev["q"].clone() for _ in range(n_sets)]
    k_sets = [dev["k"].clone() for _ in range(n_sets)]
    v_sets = [dev["v"].clone() for _ in range(n_sets)]
    o_sets = [torch.zeros_like(dev["out"]) for _ in range(n_sets)]
    stream = torch.cuda.current_stream()
    chunks = [(s, min(cfg.chunk, cfg.prompt - s)) for s in range(0, cfg.prompt, cfg.chunk)]
    events = []

    def one_step(index: int):
        """The headline step: the prompt chunk by chunk through hc_layer_step (one prologue launch
        for k, v and q + the attention kernel per chunk), then one decode step."""
        s = index % n_sets
        for start, n in chunks:
            backend.layer_step(cache, 0, q_sets[s][start:], k_sets[s][start:], v_sets[s][start:], o_sets[s][start:],
                               n, start, params, seq=s, stream=stream)
        pos = cfg.prompt
        backend.layer_step(cache, 0, q_sets[s][pos:], k_sets[s][pos:], v_sets[s][pos:], o_sets[s][pos:], 1, pos,
                           params, seq=s, stream=stream)

    # For the roofline of the dominant kernel alone: queries rotated beforehand (the same kernel code
    # as the fused prologue, so the same bits), so that the timed call is one launch, the attention
    # kernel.  Only when the query prologue is nothing but the rotation (no QK norm, no gate).
    import dataclasses
    kernel_only = not cfg.qk_norm and not cfg.gate
    if kernel_only:
        q_rot = [q.clone() for q in q_sets]
        for q in q_rot:
            backend.apply_rope(q, run.tables[0], cfg.prompt + 1, cfg.q_heads, d, 0, io_dtype=wl.capi.HC_BF16, stream=stream)
        params_rot = dataclasses.replace(params, rope=None)
        torch.cuda.synchronize()

    def roofline_step(index: int):
        """The same prompt with the append and the attention as separate calls and CUDA events
        around each attention call: the dominant kernel's time."""
        s = index % n_sets
        for start, n in chunks:
            backend.write_key_value(cache, 0, k_sets[s][start:], v_sets[s][start:], n, start, params, seq=s, stream=stream)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            if kernel_only:
                backend.attention_prefill(cache, 0, q_rot[s][start:], o_sets[s][start:], n, start, params_rot, seq=s, stream=stream)
            else:
                backend.attention_prefill(cache, 0, q_sets[s][start:], o_sets[s][start:], n, start, params, seq=s, stream=stream)
            e1.record(stream)
            events.append((start, n, e0, e1))

    for i in range(max(args.warmup, 3)):
        one_step(i)
    ctx.check()

    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    launches_before = ctx.launch_count
    barrier(world)
    start_ev, end_ev = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start_ev.record(stream)
    for i in range(args.steps):
        one_step(i)
    end_ev.record(stream)
    barrier(world)
    elapsed_ms = max_over_ranks(start_ev.elapsed_time(end_ev), world)
    launches = ctx.launch_count - launches_before
    ctx.check()
    for i in range(args.steps):
        roofline_step(args.steps + i)
    torch.cuda.synchronize()
    ctx.check()
    ms_per_step = elapsed_ms / args.steps
    value = cfg.prompt / (ms_per_step * 1e-3)

    # The dominant kernel: prefill attention.  Per call: its algorithmic flops / its CUDA-event time.
    group = cfg.q_heads // cfg.kv_heads
    flops_total, ms_total = 0.0, 0.0
    for start, n, e0, e1 in events:
        p = np.arange(start, start + n, dtype=np.float64)
        window = cfg.layers[0].window
        visible = p + 1 if window == 0 else np.minimum(p + 1, window)
        flops_total += float(visible.sum()) * cfg.q_heads * 4 * d
        ms_total += e0.elapsed_time(e1)
    achieved_tflops = flops_total / (ms_total * 1e-3) / 1e12 if ms_total > 0 else 0.0
    achieved_tflops = achieved_tflops  # this rank's; ranks are symmetric
    roofline = {"bound": "tensor", "achieved": achieved_tflops, "peak": peaks["bf16_tflops"], "unit": "TFLOP/s",
                "frac": achieved_tflops / peaks["bf16_tflops"],
                # dram__bytes_read + write of one launch, from the committed ncu capture of the last
                # chunk (context 4096); earlier chunks read proportionally fewer keys.
                "traffic": 12.72e6 if args.config == "C2" and world == 1 else None,
                "kernel": ("attention_tc_kernel, one launch per 512-token chunk (queries rotated beforehand)" if kernel_only
                           else "prefill attention call (q prologue + attention kernel), per 512-token chunk")
                          + "; timed in a pass of its own right after the headline steps, same buffers and rotation",
                "peak_source": f"{peaks['source']} cuBLAS bf16 burst",
                "avg_launch_ms": ms_total / max(len(events), 1)}

    # Decode at context 4096: L2 flushed before every timed launch (the 8 MB of K/V would sit in L2).
    flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device="cuda")
    pos = cfg.prompt
    dec_ms = []
    for i in range(20):
        s = i % n_sets
        flush.fill_(i & 0xFF)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        backend.attention(cache, 0, q_sets[s][pos:], o_sets[s][pos:], [pos], params, seq_ids=[s], stream=stream)
        e1.record(stream)
        torch.cuda.synchronize()
        if i >= 4:
            dec_ms.append(e0.elapsed_time(e1))
    dec_us = max_over_ranks(statistics.median(dec_ms) * 1e3, world)
    dec_bytes_rank = wl.decode_bytes(cfg, pos, cfg.layers[0])
    dec_gbs = dec_bytes_rank * world / (dec_us * 1e-6) / 1e9
    decode = {"context": pos + 1, "us_per_step": dec_us, "kv_bytes_per_step": dec_bytes_rank * world,
              "kv_gbs": dec_gbs, "frac_of_8tbs": dec_gbs / (8000.0 * world),
              "frac_of_measured": dec_gbs / (peaks["hbm_gbs"] * world),
              "note": "call = q prologue + split kernel + merge; L2 flushed before each timed call"}

    # The HBM-bound decode case: one batched decode step over 64 ragged sequences (lengths U[1024,
    # 16384], seed 7; the full-attention layer of configuration C5), KV heads sharded like C2's.
    # 1.2 GB of K/V per step at one GPU, far beyond L2, so no flush is needed.
    lens = np.random.default_rng(7).integers(1024, 16385, size=64)
    big = hb.KVCache(ctx, [dict(q_heads=cfg.q_heads, kv_heads=per, head_dim=d, window=0)], 16384, max_seqs=64)
    gen = torch.Generator(device="cuda").manual_seed(7 + rank)
    plain = hb.AttnParams(q_heads=cfg.q_heads, kv_heads=per, head_dim=d, window=0, sm_scale=cfg.scale,
                          io_dtype=hb.capi.HC_BF16, sinks=params.sinks)
    for seq, n in enumerate(lens):
        block = torch.randn(int(n), per, d, device="cuda", generator=gen).to(torch.bfloat16)
        backend.write_key_value(big, 0, block, block, int(n), 0, plain, seq=seq, stream=stream)
    torch.cuda.synchronize()
    bq = torch.randn(64, cfg.q_heads, d, device="cuda", generator=gen).to(torch.bfloat16)
    bo = torch.empty_like(bq)
    bpos = [int(n) - 1 for n in lens]
    big_ms = []
    for i in range(12):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        backend.attention(big, 0, bq, bo, bpos, plain, seq_ids=list(range(64)), stream=stream)
        e1.record(stream)
        torch.cuda.synchronize()
        if i >= 3:
            big_ms.append(e0.elapsed_time(e1))
    ctx.check()
    big_us = max_over_ranks(statistics.median(big_ms) * 1e3, world)
    big_bytes = int(lens.sum()) * per * d * 2 * 2
    big_gbs = big_bytes * world / (big_us * 1e-6) / 1e9
    decode_large = {"workload": "C5 full-attention layer: 64 ragged sequences (sum of lengths 591950), one decode step",
                    "us_per_step": big_us, "kv_bytes_per_step": big_bytes * world, "kv_gbs": big_gbs,
                    "frac_of_8tbs": big_gbs / (8000.0 * world), "frac_of_measured": big_gbs / (peaks["hbm_gbs"] * world),
                    "note": "call = split kernel + merge, CUDA events; per-GPU peak x n_gpus in the fractions"}
    big.close()

    # End to end: the same prefill through hc_layer_step_host with pinned host buffers.
    host = {name: dev[name].cpu().pin_memory() for name in ("q", "k", "v")}
    host_out = torch.zeros_like(dev["out"], device="cpu").pin_memory()
    eb = 2

    def e2e_step():
        for start, n in chunks:
            backend.layer_step_host(cache, 0, host["q"][start:], host["k"][start:], host["v"][start:],
                                    host_out[start:], n, start, params, seq=0, stream=stream)

    for _ in range(2):
        e2e_step()
    barrier(world)
    t0 = time.perf_counter()
    e2e_steps = max(2, min(args.steps, 5))
    for _ in range(e2e_steps):
        e2e_step()
    barrier(world)
    e2e_ms = max_over_ranks((time.perf_counter() - t0) * 1e3 / e2e_steps, world)
    e2e = {"value": cfg.prompt / (e2e_ms * 1e-3), "unit": "tok/s",
           "h2d_bytes_per_step": cfg.prompt * (cfg.q_heads + 2 * cfg.kv_heads) * d * eb,
           "d2h_bytes_per_step": cfg.prompt * cfg.q_heads * d * eb, "ms_per_step": e2e_ms,
           "note": "per rank bytes; hc_layer_step_host per 512-token chunk, pinned host buffers"}

    clocks = sampler.stop() if rank == 0 else None

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        from oracle import hydra_oracle as ho
        threads = ho.hardware_threads()
        n, times = cpu_sample(args.config, 64, 1, threads)
        cpu = {"value": n / sum(times), "unit": "tok/s", "cores": threads, "kind": "port",
               "sample": "64 query tokens at slice midpoints of the 4096-token prompt, all 64 heads"}

    if rank == 0:
        line = {
            "metric": "attn_prefill_tok_s", "value": value, "unit": "tok/s", "n_gpus": world,
            "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic",
            "config": {"workload": f"{args.config}: 64q/8kv d64 full causal, 4096-token prompt in 512-token chunks "
                                   "(hc_layer_step: KV append + attention), then one decode step at context 4096",
                       "kv_heads_per_gpu": per, "parallelism": f"kv-head shard x{world}",
                       "l2": f"{n_sets} rotating copies of the prompt's buffers (> 2x L2); decode flushes L2"},
            "roofline": roofline, "decode": decode, "decode_large": decode_large, "e2e": e2e, "cpu_baseline": cpu, "clocks": clocks,
            "gpu_launches": launches,
            "prefill_tflops_whole_step": wl.prefill_flops(cfg) * world / (ms_per_step * 1e-3) / 1e12,
        }
        print(json.dumps(line))
    run.close()
    ctx.close()
    if world > 1:
        import torch.distributed as dist
        dist.destroy_process_group()
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="cuda", choices=["cuda", "reference"])
    ap.add_argument("--config", default="C2", choices=["C2"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    args = ap.parse_args()
    if args.impl == "reference":
        return run_reference(args)
    return run_cuda(args)


if __name__ == "__main__":
    sys.exit(main())
