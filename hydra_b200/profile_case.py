"""Small, self-ending cases of the two hot kernels, for profiler captures and quick timing.

    python -m hydra_b200.profile_case prefill [--context 4096] [--chunk 512] [--dim 64] [--repeat 3]
    python -m hydra_b200.profile_case decode  [--seqs 16] [--context 8192] [--dim 64] [--repeat 3]

prefill: a GPT-OSS-shaped layer (64q/8kv) with `context` tokens cached; attention of the last
         `chunk` tokens, `repeat` times.  q is passed already rotated, so one call = one kernel.
decode:  `seqs` sequences of `context` cached tokens (K/V larger than L2 for the defaults); one
         batched decode step, `repeat` times (split kernel + merge).
Both print the CUDA-event time per call and the achieved rate.
"""
from __future__ import annotations

import argparse

import numpy as np


def main():
    import torch
    import hydra_b200 as hb

    ap = argparse.ArgumentParser()
    ap.add_argument("case", choices=["prefill", "decode"])
    ap.add_argument("--context", type=int, default=None)
    ap.add_argument("--chunk", type=int, default=512)
    ap.add_argument("--seqs", type=int, default=16)
    ap.add_argument("--dim", type=int, default=64)
    ap.add_argument("--q-heads", type=int, default=64)
    ap.add_argument("--kv-heads", type=int, default=8)
    ap.add_argument("--window", type=int, default=0)
    ap.add_argument("--repeat", type=int, default=3)
    ap.add_argument("--path", type=int, default=hb.capi.HC_PATH_AUTO)
    args = ap.parse_args()

    ctx = hb.Context(0)
    backend = hb.AttentionBackend(ctx)
    d, qh, kvh = args.dim, args.q_heads, args.kv_heads
    gen = torch.Generator(device="cuda").manual_seed(0)
    bf = torch.bfloat16
    sinks = torch.randn(qh, device="cuda", generator=gen).to(bf)
    params = hb.AttnParams(q_heads=qh, kv_heads=kvh, head_dim=d, window=args.window,
                           sm_scale=1.0 / np.sqrt(d), io_dtype=hb.capi.HC_BF16, sinks=sinks,
                           kernel_path=args.path)
    stream = torch.cuda.current_stream()

    if args.case == "prefill":
        context = args.context or 4096
        cache = hb.KVCache(ctx, [dict(q_heads=qh, kv_heads=kvh, head_dim=d, window=args.window)], context,
                           prefill_chunk=max(args.chunk, 512))
        k = torch.randn(context, kvh, d, device="cuda", generator=gen).to(bf)
        v = torch.randn(context, kvh, d, device="cuda", generator=gen).to(bf)
        q = torch.randn(args.chunk, qh, d, device="cuda", generator=gen).to(bf)
        out = torch.empty_like(q)
        for start in range(0, context, 512):
            backend.write_key_value(cache, 0, k[start:], v[start:], min(512, context - start), start, params)
        first = context - args.chunk
        p = np.arange(first, context, dtype=np.float64)
        visible = p + 1 if args.window == 0 else np.minimum(p + 1, args.window)
        flops = float(visible.sum()) * qh * 4 * d
        times = []
        for _ in range(args.repeat):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            backend.attention_prefill(cache, 0, q, out, args.chunk, first, params, stream=stream)
            e1.record(stream)
            torch.cuda.synchronize()
            times.append(e0.elapsed_time(e1))
        ctx.check()
        best = min(times)
        print(f"prefill d={d} {qh}q/{kvh}kv chunk={args.chunk} at context {context}: "
              f"{best * 1e3:.1f} us per call, {flops / (best * 1e-3) / 1e12:.1f} TFLOP/s "
              f"({flops / 1e9:.2f} GFLOP), times ms {['%.4f' % t for t in times]}")
    else:
        context = args.context or 8192
        cache = hb.KVCache(ctx, [dict(q_heads=qh, kv_heads=kvh, head_dim=d, window=args.window)], context,
                           max_seqs=args.seqs)
        block = torch.randn(context, kvh, d, device="cuda", generator=gen).to(bf)
        for seq in range(args.seqs):
            for start in range(0, context, 512):
                backend.write_key_value(cache, 0, block[start:], block[start:], min(512, context - start), start,
                                        params, seq=seq)
        q = torch.randn(args.seqs, qh, d, device="cuda", generator=gen).to(bf)
        out = torch.empty_like(q)
        positions = [context - 1] * args.seqs
        visible = context if args.window == 0 else min(context, args.window)
        nbytes = args.seqs * visible * kvh * d * 2 * 2
        times = []
        for _ in range(args.repeat):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            backend.attention(cache, 0, q, out, positions, params, seq_ids=list(range(args.seqs)), stream=stream)
            e1.record(stream)
            torch.cuda.synchronize()
            times.append(e0.elapsed_time(e1))
        ctx.check()
        best = min(times)
        print(f"decode d={d} {qh}q/{kvh}kv {args.seqs} seqs x {context} keys: {best * 1e3:.1f} us per call, "
              f"{nbytes / (best * 1e-3) / 1e9:.0f} GB/s of K/V ({nbytes / 1e6:.1f} MB), "
              f"times ms {['%.4f' % t for t in times]}")
    cache.close()
    ctx.close()


if __name__ == "__main__":
    main()
