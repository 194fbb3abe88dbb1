#!/usr/bin/env python3
"""Benchmark of the attention + KV-cache hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--no-configs]
    python bench.py --case prefill|decode|prefill256|decode256|c4 [--repeat R]

Headline (configuration C2, the one the metric is quoted on): one "step" is KV append + causal GQA
attention for the 4096-token prompt in 512-token chunks (hc_prefill_chunks: one hc_layer_step per
chunk), then one decode step at context 4096.  `value` is prefill tokens per second with the inputs
resident in HBM; `e2e` is the same prompt through hc_prefill_host from pinned HOST buffers (copies
inside the timed region); `roofline` is the prefill attention kernel against the measured bf16
tensor peak.  `configs` carries the other configurations (C1, C3, C4 and both layers of C5) at the
run's GPU count: time, prefill tok/s or KV bytes per second, and the fraction of the peak that bounds
each.  With N > 1 (torch.distributed.run, one rank per GPU) C2, C3 and C5 shard their 8 KV heads N
ways with no exchange inside attention; C4 (2 KV heads) splits the KV sequence and the library
all-gathers the ranks' partials over NCCL (hc_attention_decode_sharded).  Times are CUDA events on
the launching stream, maximum over ranks.

`--case` runs one small, self-ending case of a hot kernel (what the profiler captures under
profiles/ use).  `--impl reference` times the reference's CPU algorithm (the oracle restating
HydraReference; the Swift original cannot be built here) on the host cores, on a bounded sample.
"""
from __future__ import annotations

import argparse
import dataclasses
import json
import os
import re
import statistics
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

NOMINAL_HBM_GBS = 8000.0          # the peak BASELINE.json quotes decode against


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return {"hbm_gbs": p["hbm_gbs"], "bf16_tflops": p["bf16_tflops"],
                "bf16_tflops_sustained": p["bf16_tflops_sustained"], "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


def profiled_traffic(kernel: str, workload: str):
    """DRAM bytes (read + write) of one launch from the committed profiler summaries
    (profiles/dram_traffic.md: one table row per kernel and workload), or None."""
    path = os.path.join(ROOT, "profiles", "dram_traffic.md")
    if not os.path.exists(path):
        return None
    for line in open(path):
        cells = [c.strip().strip("`") for c in line.strip().strip("|").split("|")]
        if len(cells) >= 4 and cells[0] == kernel and cells[1] == workload:
            try:
                return (float(cells[2]) + float(cells[3])) * 1e6
            except ValueError:
                return None
    return None


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
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "50",
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


# ---- torch.distributed plumbing ------------------------------------------------------------------

class Ranks:
    def __init__(self, n_gpus: int):
        import torch
        self.rank = int(os.environ.get("RANK", "0"))
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.local = int(os.environ.get("LOCAL_RANK", "0"))
        if self.world > 1:
            import torch.distributed as dist
            torch.cuda.set_device(self.local)
            dist.init_process_group("nccl", device_id=torch.device("cuda", self.local))
        else:
            torch.cuda.set_device(0)
            self.local = 0
        if self.world != max(n_gpus, 1) and self.rank == 0:
            print(f"warning: --gpus {n_gpus} but WORLD_SIZE {self.world}", file=sys.stderr)

    def barrier(self):
        import torch
        torch.cuda.synchronize()
        if self.world > 1:
            import torch.distributed as dist
            dist.barrier()
        torch.cuda.synchronize()

    def max(self, value: float) -> float:
        if self.world == 1:
            return value
        import torch
        import torch.distributed as dist
        t = torch.tensor([value], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def bits_equal(self, tensor) -> bool:
        """True when every rank holds the same bits in `tensor`."""
        if self.world == 1:
            return True
        import torch
        import torch.distributed as dist
        bits = tensor.contiguous().view(torch.int16).to(torch.int32)
        lo, hi = bits.clone(), bits.clone()
        dist.all_reduce(lo, op=dist.ReduceOp.MIN)
        dist.all_reduce(hi, op=dist.ReduceOp.MAX)
        return bool(torch.equal(lo, hi))

    def close(self):
        if self.world > 1:
            import torch.distributed as dist
            dist.destroy_process_group()


class Timer:
    """CUDA-event timing of repeated calls on one stream, L2 flushed before each when asked."""

    def __init__(self, stream, flush_bytes: int = 0):
        import torch
        self.torch, self.stream = torch, stream
        self.flush = torch.empty(flush_bytes, dtype=torch.uint8, device="cuda") if flush_bytes else None

    def run(self, call, repeat: int, warm: int = 3):
        torch = self.torch
        times = []
        for i in range(warm + repeat):
            if self.flush is not None:
                self.flush.fill_(i & 0xFF)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(self.stream)
            call(i)
            e1.record(self.stream)
            torch.cuda.synchronize()
            if i >= warm:
                times.append(e0.elapsed_time(e1))
        return times


def typical(times):
    """Interquartile mean: as robust as the median, and finer than the event timer's tick (about 2 us
    on this part) when the samples straddle one."""
    ordered = sorted(times)
    quarter = len(ordered) // 4
    middle = ordered[quarter:len(ordered) - quarter] or ordered
    return sum(middle) / len(middle)


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
        cpu_sample("C2", 16, 1, threads)
    n, times = cpu_sample("C2", rows, max(args.steps, 1), threads)
    total = sum(times)
    value = n * len(times) / total
    line = {
        "impl": "reference", "metric": "attn_prefill_tok_s", "value": value, "unit": "tok/s",
        "n_gpus": args.gpus, "steps": len(times), "warmup": args.warmup,
        "ms_per_step": 1e3 * total / len(times), "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "f64", "data": "synthetic",
        "config": {"workload": f"C2: attention of {rows} sampled query tokens per step over the "
                               "4096-token bf16 K/V history (mean context = the prompt's), 64q/8kv d64, sinks"},
        "cpu_baseline": {"value": value, "unit": "tok/s", "cores": threads, "kind": "port",
                         "sample": f"{rows} query tokens at slice midpoints of the 4096-token prompt, all 64 heads, "
                                   "double precision, two-pass softmax"},
        "e2e": {"value": value, "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))
    return 0


# ---- the other configurations ----------------------------------------------------------------------

def visible_pairs(prompt: int, window: int) -> float:
    p = np.arange(prompt, dtype=np.float64)
    return float((p + 1 if window == 0 else np.minimum(p + 1, window)).sum())


def bench_prefill_config(name, ctx, ranks, peaks, repeat):
    """C1 / C3: every layer's prompt through hc_prefill_chunks, then the decode steps through
    hc_layer_step; KV heads sharded over the ranks."""
    import torch
    import hydra_b200 as hb
    from hydra_b200 import workloads as wl
    full = wl.config(name)
    per = full.kv_heads // ranks.world
    cfg = wl.config(name, kv_heads=per)
    inputs = wl.Inputs(cfg, full_heads=full, head_offset=ranks.rank * per)
    run = wl.PathRunner(ctx, cfg, inputs)
    stream = torch.cuda.current_stream()
    layers = range(len(cfg.layers))

    def prefill(_):
        for layer in layers:
            t = run.dev[layer]
            run.backend.prefill_chunks(run.cache, layer, t["q"], t["k"], t["v"], t["out"], cfg.prompt, 0, cfg.chunk,
                                       run.params[layer], stream=stream)

    def decode(i):
        step = i % cfg.decode_steps
        pos = cfg.prompt + step
        for layer in layers:
            t = run.dev[layer]
            run.backend.layer_step(run.cache, layer, t["q"][pos:], t["k"][pos:], t["v"][pos:], t["out"][pos:], 1, pos,
                                   run.params[layer], stream=stream)

    # The prompt's buffers of one layer stack exceed L2 for C3 (6 layers x 75 MB of q, k, v, out);
    # C1's do not, so its passes flush L2 first.
    small = name == "C1"
    pre_ms = ranks.max(typical(Timer(stream, 256 << 20 if small else 0).run(prefill, repeat)))
    ctx.check()
    # every decode step of the configuration, in order, appending as it goes (after the prefill pass above)
    dec_ms = Timer(stream, 256 << 20).run(decode, cfg.decode_steps, warm=0)
    dec_us = ranks.max(typical(dec_ms) * 1e3)
    ctx.check()
    flops = sum(visible_pairs(cfg.prompt, l.window) for l in cfg.layers) * full.q_heads * 4 * cfg.head_dim
    tflops = flops / (pre_ms * 1e-3) / 1e12
    # a decode step reads, per layer, each visible K and V element once
    mid = cfg.prompt + cfg.decode_steps // 2
    dec_bytes = sum(wl.decode_bytes(full, mid, l) for l in cfg.layers)
    dec_gbs = dec_bytes / (dec_us * 1e-6) / 1e9
    run.close()
    return {
        "workload": f"{name}: {len(cfg.layers)} layer(s), {full.q_heads}q/{full.kv_heads}kv d{cfg.head_dim}, "
                    f"{cfg.prompt}-token prompt in {cfg.chunk}-token chunks, {cfg.decode_steps} decode steps",
        "parallelism": f"kv-head shard x{ranks.world}",
        "prefill_ms": pre_ms, "prefill_tok_s": cfg.prompt / (pre_ms * 1e-3), "prefill_tflops": tflops,
        "frac_of_tensor_peak": tflops / (peaks["bf16_tflops"] * ranks.world),
        "decode_us_per_step": dec_us, "decode_kv_gbs": dec_gbs,
        "decode_frac_of_8tbs": dec_gbs / (NOMINAL_HBM_GBS * ranks.world),
        "decode_frac_of_measured": dec_gbs / (peaks["hbm_gbs"] * ranks.world),
        "l2": "flushed before each timed pass" if small else "prefill buffers exceed L2; decode flushes L2",
    }


def bench_c4(ctx, ranks, peaks, repeat):
    """C4: one decode step at context 32768 over 2 KV heads.  One GPU: hc_layer_step.  More: the KV
    sequence is split over the ranks and hc_attention_decode_sharded does partial -> ncclAllGather ->
    combine; every rank must end with the same bits."""
    import torch
    import torch.distributed as dist
    import hydra_b200 as hb
    from hydra_b200 import workloads as wl
    cfg = wl.config("C4")
    inputs = wl.Inputs(cfg)
    shard_desc = (hb.capi.HC_SHARD_SEQUENCE, ranks.rank, ranks.world) if ranks.world > 1 else None
    run = wl.PathRunner(ctx, cfg, inputs, shard=shard_desc)
    run.fill_history([cfg.prefilled])
    stream = torch.cuda.current_stream()
    t, params, pos = run.dev[0], run.params[0], cfg.prefilled
    run.backend.write_key_value(run.cache, 0, t["k"], t["v"], 1, pos, params, stream=stream)
    comm = shard = None
    if ranks.world > 1:
        def exchange(raw):
            box = [raw]
            dist.broadcast_object_list(box, src=0)
            return box[0]
        comm = hb.NcclCommunicator(ranks.rank, ranks.world, exchange)
        shard = hb.Shard(ctx, hb.capi.HC_SHARD_SEQUENCE, ranks.rank, ranks.world, comm,
                         run.backend.partial_bytes(params, 1))

        def step(_):
            run.backend.attention_sharded(shard, run.cache, 0, t["q"], t["out"], [pos], params, stream=stream)
    else:
        def step(_):
            run.backend.attention(run.cache, 0, t["q"], t["out"], [pos], params, stream=stream)
    ranks.barrier()
    us = ranks.max(typical(Timer(stream, 256 << 20).run(step, repeat)) * 1e3)
    ctx.check()
    equal = ranks.bits_equal(t["out"])
    nbytes = wl.decode_bytes(cfg, pos, cfg.layers[0])
    gbs = nbytes / (us * 1e-6) / 1e9
    if shard is not None:
        shard.close()
        comm.close()
    run.close()
    return {
        "workload": "C4: 16q/2kv d256 gated, partial rotary, q/k norm; one decode step at context 32768",
        "parallelism": "single GPU" if ranks.world == 1 else f"kv-sequence split x{ranks.world}, partials all-gathered by the "
                                                             "library over NCCL (hc_attention_decode_sharded)",
        "us_per_step": us, "kv_bytes_per_step": nbytes, "kv_gbs": gbs,
        "frac_of_8tbs": gbs / (NOMINAL_HBM_GBS * ranks.world), "frac_of_measured": gbs / (peaks["hbm_gbs"] * ranks.world),
        "ranks_bit_equal": equal, "l2": "flushed before each timed call (67 MB of K/V would sit in L2)",
    }


def bench_projections(ctx, ranks, peaks, repeat):
    """The Q, K, V and O projections of one C2 layer for the whole 4096-token prompt through hc_linear
    (tcgen05 GEMM), the rows of §8(f) that bracket the attention path.  With N > 1 the weights are
    split like the heads: Q/K/V by output rows, O by input columns (its partial sums would be reduced
    by the next op)."""
    import torch
    import hydra_b200 as hb
    from hydra_b200 import workloads as wl
    full = wl.config("C2")
    backend = hb.AttentionBackend(ctx)
    hidden, tokens = 2880, full.prompt
    q_out = full.q_heads * full.head_dim // ranks.world
    kv_out = full.kv_heads * full.head_dim // ranks.world
    gen = torch.Generator(device="cuda").manual_seed(11)
    bf = torch.bfloat16
    x = torch.randn(tokens, hidden, device="cuda", generator=gen).to(bf)
    attn = torch.randn(tokens, q_out, device="cuda", generator=gen).to(bf)
    weights = [(torch.randn(n, hidden, device="cuda", generator=gen) * 0.02).to(bf) for n in (q_out, kv_out, kv_out)]
    biases = [torch.randn(n, device="cuda", generator=gen).to(bf) for n in (q_out, kv_out, kv_out)]
    outs = [torch.empty(tokens, n, device="cuda", dtype=bf) for n in (q_out, kv_out, kv_out)]
    w_o = (torch.randn(hidden, q_out, device="cuda", generator=gen) * 0.02).to(bf)
    b_o = torch.randn(hidden, device="cuda", generator=gen).to(bf)
    y_o = torch.empty(tokens, hidden, device="cuda", dtype=torch.float32)
    stream = torch.cuda.current_stream()

    def step(_):
        backend.linear_group(x, weights, biases, outs, tokens, hidden, y_dtype=hb.capi.HC_BF16, stream=stream)
        backend.linear(attn, w_o, b_o, y_o, tokens, q_out, hidden, y_dtype=hb.capi.HC_F32, stream=stream)

    ms = ranks.max(typical(Timer(stream, 256 << 20).run(step, repeat)))

    def decode_step(_):
        backend.linear_group(x, weights, biases, outs, 1, hidden, y_dtype=hb.capi.HC_BF16, stream=stream)
        backend.linear(attn, w_o, b_o, y_o, 1, q_out, hidden, y_dtype=hb.capi.HC_F32, stream=stream)

    decode_us = ranks.max(typical(Timer(stream, 256 << 20).run(decode_step, 16)) * 1e3)
    weight_bytes = 2.0 * (hidden * (q_out + 2 * kv_out) + q_out * hidden)
    flops = 2.0 * tokens * hidden * (q_out + 2 * kv_out) + 2.0 * tokens * q_out * hidden
    tflops = flops * ranks.world / (ms * 1e-3) / 1e12
    return {"workload": f"C2 layer projections for {tokens} tokens: hidden {hidden} -> q {q_out}, k {kv_out}, v {kv_out} "
                        f"(bf16 out) in one hc_linear_group launch, attention {q_out} -> hidden (fp32 out) in one hc_linear, bias on all four",
            "ms": ms, "tflops": tflops, "frac_of_tensor_peak": tflops / (peaks["bf16_tflops"] * ranks.world),
            "decode_us": decode_us, "decode_weight_gbs": weight_bytes * ranks.world / (decode_us * 1e-6) / 1e9,
            "decode_note": "the same four projections for one token: bound by reading the weights once",
            "l2": "flushed before each timed pass"}


def bench_c5(ctx, ranks, peaks, repeat):
    """C5: one batched decode step over 64 ragged sequences, the window-128 layer and the full layer."""
    import torch
    import hydra_b200 as hb
    from hydra_b200 import workloads as wl
    full = wl.config("C5")
    per = full.kv_heads // ranks.world
    cfg = wl.config("C5", kv_heads=per)
    inputs = wl.Inputs(cfg, full_heads=full, head_offset=ranks.rank * per)
    lengths = inputs.lengths
    run = wl.PathRunner(ctx, cfg, inputs)
    stream = torch.cuda.current_stream()
    # device-side fill of the histories (N(0, 1) bf16): the values do not matter to the timing
    gen = torch.Generator(device="cuda").manual_seed(7 + ranks.rank)
    for seq, n in enumerate(lengths):
        history = int(n) - 1
        block = torch.randn(history, per, cfg.head_dim, device="cuda", generator=gen).to(torch.bfloat16)
        for layer, spec in enumerate(cfg.layers):
            plain = hb.AttnParams(q_heads=cfg.q_heads, kv_heads=per, head_dim=cfg.head_dim, window=spec.window,
                                  sm_scale=cfg.scale, io_dtype=hb.capi.HC_BF16)
            ring = run.cache.layer(layer).ring_size
            # a ring keeps its last rows only, and takes at most (ring - window) tokens per append
            first = 0 if ring == 0 else max(0, history - (ring - spec.window))
            step_tokens = history - first if ring == 0 else ring - spec.window
            for start in range(first, history, max(step_tokens, 1)):
                count = min(step_tokens, history - start)
                run.backend.write_key_value(run.cache, layer, block[start:], block[start:], count, start, plain, seq=seq,
                                            stream=stream)
    torch.cuda.synchronize()
    positions = [int(n) - 1 for n in lengths]
    seqs = list(range(len(positions)))
    out = {}
    for layer, spec in enumerate(cfg.layers):
        t, params = run.dev[layer], run.params[layer]
        run.backend.write_key_value_batch(run.cache, layer, t["k"], t["v"], seqs, positions, params, stream=stream)

        def step(_):
            run.backend.attention(run.cache, layer, t["q"], t["out"], positions, params, seq_ids=seqs, stream=stream)
        visible = int(sum(min(n, spec.window) if spec.window else n for n in lengths))
        nbytes = visible * full.kv_heads * cfg.head_dim * 2 * 2
        flush = (256 << 20) if nbytes / ranks.world < (256 << 20) else 0
        us = ranks.max(typical(Timer(stream, flush).run(step, repeat)) * 1e3)
        ctx.check()
        gbs = nbytes / (us * 1e-6) / 1e9
        out["window_128_layer" if spec.window else "full_layer"] = {
            "us_per_step": us, "kv_bytes_per_step": nbytes, "kv_gbs": gbs,
            "frac_of_8tbs": gbs / (NOMINAL_HBM_GBS * ranks.world), "frac_of_measured": gbs / (peaks["hbm_gbs"] * ranks.world),
            "l2": "flushed before each timed call" if flush else "K/V exceed L2"}
    run.close()
    out["workload"] = "C5: 64 ragged sequences (lengths U[1024, 16384], seed 7, sum 591950), 64q/8kv d64, sinks; one decode step"
    out["parallelism"] = f"kv-head shard x{ranks.world}"
    return out


# ---- the CUDA arm -----------------------------------------------------------------------------------

def run_cuda(args):
    import torch
    import hydra_b200 as hb
    from hydra_b200 import workloads as wl

    ranks = Ranks(args.gpus)
    rank, world, local = ranks.rank, ranks.world, ranks.local
    peaks = measured_peaks()
    full = wl.config("C2")
    if full.kv_heads % world != 0:
        raise SystemExit(f"{full.kv_heads} KV heads cannot be sharded over {world} GPUs")
    per = full.kv_heads // world
    cfg = wl.config("C2", kv_heads=per)
    ctx = hb.Context(local)
    inputs = wl.Inputs(cfg, full_heads=full, head_offset=rank * per)

    # Rotate over several copies of the prompt's buffers so that a step's inputs are not in L2 from
    # the step before: the copies together exceed twice the 126 MB L2.
    d = cfg.head_dim
    set_bytes = cfg.prompt * (2 * cfg.q_heads * d + 2 * cfg.kv_heads * d) * 2 + 2 * cfg.context * cfg.kv_heads * d * 2
    n_sets = min(max(2, int(np.ceil(2 * 126e6 / max(set_bytes, 1)))), 64)
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
        """The headline step: the prompt through hc_prefill_chunks (per chunk one prologue launch for
        k, v and q + the attention kernel), then one decode step (hc_layer_step with one token)."""
        s = index % n_sets
        backend.prefill_chunks(cache, 0, q_sets[s], k_sets[s], v_sets[s], o_sets[s], cfg.prompt, 0, cfg.chunk, params,
                               seq=s, stream=stream)
        pos = cfg.prompt
        backend.layer_step(cache, 0, q_sets[s][pos:], k_sets[s][pos:], v_sets[s][pos:], o_sets[s][pos:], 1, pos,
                           params, seq=s, stream=stream)

    # For the roofline of the dominant kernel alone: queries rotated beforehand (the same kernel code
    # as the fused prologue, so the same bits), so that the timed call is one launch, the attention
    # kernel.
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
            backend.attention_prefill(cache, 0, q_rot[s][start:], o_sets[s][start:], n, start, params_rot, seq=s, stream=stream)
            e1.record(stream)
            events.append((start, n, e0, e1))

    for i in range(max(args.warmup, 3)):
        one_step(i)
    ctx.check()

    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    launches_before = ctx.launch_count
    ranks.barrier()
    start_ev, end_ev = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start_ev.record(stream)
    for i in range(args.steps):
        one_step(i)
    end_ev.record(stream)
    ranks.barrier()
    elapsed_ms = ranks.max(start_ev.elapsed_time(end_ev))
    launches = ctx.launch_count - launches_before
    ctx.check()
    for i in range(args.steps):
        roofline_step(args.steps + i)
    torch.cuda.synchronize()
    ctx.check()
    ms_per_step = elapsed_ms / args.steps
    value = cfg.prompt / (ms_per_step * 1e-3)

    # The dominant kernel: prefill attention.  Per call: its algorithmic flops / its CUDA-event time.
    flops_total, ms_total = 0.0, 0.0
    for start, n, e0, e1 in events:
        p = np.arange(start, start + n, dtype=np.float64)
        flops_total += float((p + 1).sum()) * cfg.q_heads * 4 * d
        ms_total += e0.elapsed_time(e1)
    achieved_tflops = flops_total / (ms_total * 1e-3) / 1e12 if ms_total > 0 else 0.0
    roofline = {"bound": "tensor", "achieved": achieved_tflops, "peak": peaks["bf16_tflops"], "unit": "TFLOP/s",
                "frac": achieved_tflops / peaks["bf16_tflops"],
                # dram read + write of one launch, from the committed profiler summary of the last
                # chunk (context 4096); earlier chunks read proportionally fewer keys
                "traffic": profiled_traffic("attention_tc_kernel<64, 0>", "prefill chunk 512 at context 4096")
                           if world == 1 else None,
                "kernel": "attention_tc_kernel<64, 0> (whole rows per item), one launch per 512-token chunk (queries rotated beforehand); timed in a "
                          "pass of its own right after the headline steps, same buffers and rotation",
                "peak_source": f"{peaks['source']} cuBLAS bf16 burst",
                "avg_launch_ms": ms_total / max(len(events), 1)}

    # Decode at context 4096: L2 flushed before every timed launch (the 8 MB of K/V would sit in L2).
    pos = cfg.prompt
    dec_ms = Timer(stream, 256 << 20).run(
        lambda i: backend.attention(cache, 0, q_sets[i % n_sets][pos:], o_sets[i % n_sets][pos:], [pos], params,
                                    seq_ids=[i % n_sets], stream=stream), 16, warm=4)
    dec_us = ranks.max(typical(dec_ms) * 1e3)
    # What the same timer reads for a kernel that does next to nothing (the input norm of one row): after
    # the flush, code, arguments and tables all come from DRAM, and that is most of a small step's time.
    one_row = torch.zeros(1, 2880, device="cuda")
    one_scale = torch.ones(2880, device="cuda", dtype=torch.bfloat16)
    one_out = torch.empty(1, 2880, device="cuda", dtype=torch.bfloat16)
    floor_us = ranks.max(typical(Timer(stream, 256 << 20).run(
        lambda i: backend.rms_norm(one_row, one_scale, one_out, 1, 2880, 1e-5, stream=stream), 16, warm=4)) * 1e3)
    # The same decode call 32 times in a row without the flush: the 8 MB of K/V then sit in L2, so this is
    # the step's latency, not an HBM figure.
    burst = 32
    b0, b1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    for timed in (False, True):
        if timed:
            b0.record(stream)
        for _ in range(burst):
            backend.attention(cache, 0, q_sets[0][pos:], o_sets[0][pos:], [pos], params, seq_ids=[0], stream=stream)
    b1.record(stream)
    torch.cuda.synchronize()
    resident_us = ranks.max(b0.elapsed_time(b1) * 1e3 / burst)
    dec_bytes_rank = wl.decode_bytes(cfg, pos, cfg.layers[0])
    dec_gbs = dec_bytes_rank * world / (dec_us * 1e-6) / 1e9
    decode = {"context": pos + 1, "us_per_step": dec_us, "kv_bytes_per_step": dec_bytes_rank * world,
              "kv_gbs": dec_gbs, "frac_of_8tbs": dec_gbs / (NOMINAL_HBM_GBS * world),
              "frac_of_measured": dec_gbs / (peaks["hbm_gbs"] * world),
              "timer_floor_us": floor_us, "us_per_step_l2_resident": resident_us,
              "note": "call = q prologue + split kernel + merge; L2 flushed before each timed call.  timer_floor_us: a "
                      "one-row hc_rms_norm under the same timer and flush; us_per_step_l2_resident: 32 calls back to "
                      "back without the flush (K/V in L2: latency, not an HBM figure)"}

    # End to end: the same prompt through hc_prefill_host with pinned host buffers.
    host = {name: dev[name].cpu().pin_memory() for name in ("q", "k", "v")}
    host_out = torch.zeros_like(dev["out"], device="cpu").pin_memory()

    def e2e_step():
        backend.prefill_host(cache, 0, host["q"], host["k"], host["v"], host_out, cfg.prompt, 0, cfg.chunk, params,
                             seq=0, stream=stream)

    for _ in range(2):
        e2e_step()
    ranks.barrier()
    t0 = time.perf_counter()
    e2e_steps = max(3, min(args.steps, 10))
    for _ in range(e2e_steps):
        e2e_step()
    ranks.barrier()
    e2e_ms = ranks.max((time.perf_counter() - t0) * 1e3 / e2e_steps)
    e2e = {"value": cfg.prompt / (e2e_ms * 1e-3), "unit": "tok/s",
           "h2d_bytes_per_step": cfg.prompt * (cfg.q_heads + 2 * cfg.kv_heads) * d * 2,
           "d2h_bytes_per_step": cfg.prompt * cfg.q_heads * d * 2, "ms_per_step": e2e_ms,
           "note": "per rank bytes; hc_prefill_host: pinned host buffers, the copies of chunk i+1 / i-1 overlap the "
                   "kernels of chunk i"}
    clocks = sampler.stop() if rank == 0 else None
    run.close()

    configs = None
    if not args.no_configs:
        configs = {}
        repeat = 5
        for name in ("C1", "C3"):
            configs[name] = bench_prefill_config(name, ctx, ranks, peaks, repeat)
        configs["C4"] = bench_c4(ctx, ranks, peaks, 12)
        configs["C5"] = bench_c5(ctx, ranks, peaks, 8)
        configs["projections"] = bench_projections(ctx, ranks, peaks, 8)

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        from oracle import hydra_oracle as ho
        threads = ho.hardware_threads()
        n, times = cpu_sample("C2", 128, 2, threads)
        cpu = {"value": n * len(times) / sum(times), "unit": "tok/s", "cores": threads, "kind": "port",
               "sample": "2 x 128 query tokens at slice midpoints of the 4096-token prompt, all 64 heads"}

    if rank == 0:
        line = {
            "metric": "attn_prefill_tok_s", "value": value, "unit": "tok/s", "n_gpus": world,
            "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic",
            "config": {"workload": "C2: 64q/8kv d64 full causal, 4096-token prompt in 512-token chunks "
                                   "(hc_prefill_chunks: KV append + attention per chunk), then one decode step at context 4096",
                       "kv_heads_per_gpu": per, "parallelism": f"kv-head shard x{world}",
                       "l2": f"{n_sets} rotating copies of the prompt's buffers (> 2x L2); decode flushes L2"},
            "roofline": roofline, "decode": decode,
            "decode_large": configs["C5"]["full_layer"] if configs else None,
            "e2e": e2e, "cpu_baseline": cpu, "clocks": clocks, "gpu_launches": launches,
            "prefill_tflops_whole_step": wl.prefill_flops(cfg) * world / (ms_per_step * 1e-3) / 1e12,
            "configs": configs,
        }
        print(json.dumps(line))
    ctx.close()
    ranks.close()
    return 0


# ---- small self-ending cases for profiler captures --------------------------------------------------

def run_case(args):
    """One small case of a hot kernel, `--repeat` calls, CUDA-event time of the best one.
    prefill / prefill256: a layer with 4096 tokens cached, attention of the last 512 (q already rotated:
    one call = one kernel).  decode / decode256: 16 sequences of 8192 cached tokens (K/V beyond L2), one
    batched decode step (split kernel + merge).  c4: C4's decode step at context 32768, L2 flushed."""
    import torch
    import hydra_b200 as hb
    case = args.case
    if case in ("linear", "linear1"):
        return run_linear_case(args)
    d = 256 if case.endswith("256") or case == "c4" else 64
    qh, kvh = (16, 2) if case == "c4" else ((16, 8) if d == 256 else (64, 8))
    ctx = hb.Context(0)
    backend = hb.AttentionBackend(ctx)
    gen = torch.Generator(device="cuda").manual_seed(0)
    bf = torch.bfloat16
    sinks = torch.randn(qh, device="cuda", generator=gen).to(bf)
    params = hb.AttnParams(q_heads=qh, kv_heads=kvh, head_dim=d, sm_scale=1.0 / np.sqrt(d), io_dtype=hb.capi.HC_BF16,
                           sinks=sinks)
    stream = torch.cuda.current_stream()
    layer = [dict(q_heads=qh, kv_heads=kvh, head_dim=d, window=0)]
    if case.startswith("prefill"):
        context, chunk = 4096, 512
        cache = hb.KVCache(ctx, layer, context, prefill_chunk=512)
        k = torch.randn(context, kvh, d, device="cuda", generator=gen).to(bf)
        q = torch.randn(chunk, qh, d, device="cuda", generator=gen).to(bf)
        out = torch.empty_like(q)
        for start in range(0, context, 512):
            backend.write_key_value(cache, 0, k[start:], k[start:], 512, start, params)
        first = context - chunk
        work = visible_pairs(context, 0) - visible_pairs(first, 0)
        work *= qh * 4 * d
        call = lambda _: backend.attention_prefill(cache, 0, q, out, chunk, first, params, stream=stream)
        timer, unit, scale = Timer(stream), "TFLOP/s", 1e12
        what = f"prefill d={d} {qh}q/{kvh}kv chunk={chunk} at context {context}"
    else:
        seqs, context = (1, 32768) if case == "c4" else (16, 8192)
        cache = hb.KVCache(ctx, layer, context, max_seqs=seqs)
        block = torch.randn(context, kvh, d, device="cuda", generator=gen).to(bf)
        for seq in range(seqs):
            for start in range(0, context, 512):
                backend.write_key_value(cache, 0, block[start:], block[start:], 512, start, params, seq=seq)
        q = torch.randn(seqs, qh, d, device="cuda", generator=gen).to(bf)
        out = torch.empty_like(q)
        positions = [context - 1] * seqs
        work = seqs * context * kvh * d * 2 * 2
        call = lambda _: backend.attention(cache, 0, q, out, positions, params, seq_ids=list(range(seqs)), stream=stream)
        timer, unit, scale = Timer(stream, (256 << 20) if work < (256 << 20) else 0), "GB/s of K/V", 1e9
        what = f"decode d={d} {qh}q/{kvh}kv {seqs} seqs x {context} keys"
    times = timer.run(call, args.repeat, warm=min(3, args.repeat - 1) if args.repeat > 1 else 0)
    ctx.check()
    best = min(times)
    print(f"{what}: {best * 1e3:.1f} us per call, {work / (best * 1e-3) / scale:.1f} {unit} "
          f"(median {statistics.median(times) * 1e3:.1f} us over {len(times)} calls)")
    cache.close()
    ctx.close()
    return 0


def run_linear_case(args):
    """hc_linear on C2's q_proj: 2880 -> 4096 for the whole prompt (`linear`: 4096 tokens, 48 output
    tiles of 128 x 256 per 128 tokens, 96.6 GFLOP) or for one decode token (`linear1`: the narrow
    shape, 128 tiles of 32 weight rows; the work is reading the 23.6 MB weight once)."""
    import torch
    import hydra_b200 as hb
    ctx = hb.Context(0)
    backend = hb.AttentionBackend(ctx)
    gen = torch.Generator(device="cuda").manual_seed(0)
    tokens, n_in, n_out = (1 if args.case == "linear1" else 4096), 2880, 4096
    x = torch.randn(tokens, n_in, device="cuda", generator=gen).to(torch.bfloat16)
    w = (torch.randn(n_out, n_in, device="cuda", generator=gen) * 0.02).to(torch.bfloat16)
    b = torch.randn(n_out, device="cuda", generator=gen).to(torch.bfloat16)
    y = torch.empty(tokens, n_out, device="cuda", dtype=torch.bfloat16)
    stream = torch.cuda.current_stream()
    times = Timer(stream, 256 << 20).run(lambda _: backend.linear(x, w, b, y, tokens, n_in, n_out, y_dtype=hb.capi.HC_BF16,
                                                                  stream=stream), args.repeat, warm=min(3, args.repeat - 1))
    ctx.check()
    best = min(times)
    work = 2.0 * tokens * n_in * n_out
    print(f"linear {tokens} x {n_in} -> {n_out}: {best * 1e3:.1f} us per call, {work / (best * 1e-3) / 1e12:.1f} TFLOP/s, "
          f"{2.0 * n_in * n_out / (best * 1e-3) / 1e9:.0f} GB/s of weight "
          f"(median {statistics.median(times) * 1e3:.1f} us over {len(times)} calls)")
    ctx.close()
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="cuda", choices=["cuda", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-configs", action="store_true", help="only the headline configuration (C2)")
    ap.add_argument("--case", default=None, choices=["prefill", "decode", "prefill256", "decode256", "c4", "linear", "linear1"])
    ap.add_argument("--repeat", type=int, default=3)
    args = ap.parse_args()
    if args.case:
        return run_case(args)
    if args.impl == "reference":
        return run_reference(args)
    return run_cuda(args)


if __name__ == "__main__":
    sys.exit(main())
