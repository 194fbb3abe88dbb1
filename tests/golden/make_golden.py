#!/usr/bin/env python3
"""Writes the golden vectors under tests/golden/ from the reference checkout.

Run once, in a container that has the reference mounted:

    python tests/golden/make_golden.py /path/to/reference

Two sources, both the reference's own:

1. The committed fixtures its HydraReference tests check to 1e-12
   (`Tests/HydraReferenceTests/Fixtures/reference_ops.json`, `gemma4_operators.json`): the entries
   on the attention path are copied out unchanged (`rms_norm`, `yarn`, `rope`, `sdpa_full`,
   `sdpa_sliding`; `rms_norm`, `rms_norm_unscaled`, `rope_sliding`, `rope_full_partial`,
   `attention_full`, `attention_windowed`).
2. The reference's pure-Python transcriptions (`tools/gen_reference_fixtures.py`,
   `tools/gen_gemma_fixtures.py`), imported and *run here* to (a) regenerate those same entries, so
   the test suite can check that the committed fixtures and the live transcription agree, and
   (b) produce composed cases the committed fixtures do not hold: grouped-query attention with a
   window and sinks at a wider shape, the Gemma block (q/k norm with weight, weightless v norm,
   rotation, scale 1.0, window) and the Qwen block (per-head query/gate split, partial rotation,
   1/sqrt(d) scale, sigmoid gate) built the way
   `Tests/HydraReferenceTests/QwenAttentionLayerTests.swift:82-147` recomposes it.

The reference is not available where the GPU tests run, so the output files are committed.
"""
import importlib.util
import json
import math
import os
import sys


def load(path, name):
    spec = importlib.util.spec_from_file_location(name, path)
    module = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(module)
    return module


def main():
    if len(sys.argv) != 2:
        raise SystemExit("usage: python tests/golden/make_golden.py <path of a Neojarred/Hydra checkout>")
    ref = sys.argv[1]
    here = os.path.dirname(os.path.abspath(__file__))
    gpt = load(os.path.join(ref, "tools", "gen_reference_fixtures.py"), "gen_reference_fixtures")
    gem = load(os.path.join(ref, "tools", "gen_gemma_fixtures.py"), "gen_gemma_fixtures")

    fixtures = os.path.join(ref, "Tests", "HydraReferenceTests", "Fixtures")
    with open(os.path.join(fixtures, "reference_ops.json")) as f:
        committed_gpt = json.load(f)
    with open(os.path.join(fixtures, "gemma4_operators.json")) as f:
        committed_gem = json.load(f)

    gpt_keys = ["rms_norm", "yarn", "rope", "sdpa_full", "sdpa_sliding"]
    gem_keys = ["rms_norm", "rms_norm_unscaled", "rope_sliding", "rope_full_partial",
                "attention_full", "attention_windowed"]

    live_gpt = gpt.build()
    live_gem = gem.build()

    out = {
        "source": "Neojarred/Hydra Tests/HydraReferenceTests/Fixtures + tools/gen_*_fixtures.py",
        "committed": {
            "reference_ops": {k: committed_gpt[k] for k in gpt_keys},
            "gemma4_operators": {k: committed_gem[k] for k in gem_keys},
        },
        # Only the expected values of the live run: the inputs are the same by construction.
        "live_expected": {
            "reference_ops": {
                "rms_norm": live_gpt["rms_norm"]["expected"],
                "yarn_inv_freq": live_gpt["yarn"]["inv_freq"],
                "yarn_cos": live_gpt["yarn"]["cos"],
                "yarn_sin": live_gpt["yarn"]["sin"],
                "rope": live_gpt["rope"]["expected"],
                "sdpa_full": live_gpt["sdpa_full"]["expected"],
                "sdpa_sliding": live_gpt["sdpa_sliding"]["expected"],
            },
            "gemma4_operators": {k: live_gem[k]["expected"] for k in gem_keys},
        },
    }

    # ---- composed case 1: GQA, window, sinks at a wider shape (GPT-OSS semantics) -------------
    tokens, kv_heads, q_mult, d = 24, 2, 4, 16
    Q = gpt.reshape(gpt.normals(tokens * kv_heads * q_mult * d, 105), tokens, kv_heads, q_mult, d)
    K = gpt.reshape(gpt.normals(tokens * kv_heads * d, 106), tokens, kv_heads, d)
    V = gpt.reshape(gpt.normals(tokens * kv_heads * d, 107), tokens, kv_heads, d)
    S = gpt.normals(kv_heads * q_mult, 108)
    scale = 1.0 / math.sqrt(d)
    composed = {}
    composed["gqa_sinks"] = {
        "tokens": tokens, "kv_heads": kv_heads, "q_mult": q_mult, "head_dim": d,
        "sm_scale": scale, "q": Q, "k": K, "v": V, "sinks": S,
        "expected_full": gpt.sdpa(Q, K, V, S, scale, 0),
        "window": 7,
        "expected_window": gpt.sdpa(Q, K, V, S, scale, 7),
    }

    # ---- composed case 2: the Gemma block's attention path --------------------------------------
    # q/k: rms_norm with weight -> rope; v: weightless rms_norm, never rotated; scale 1.0; window.
    heads, kv, d, tokens, window = 4, 2, 16, 11, 4
    eps = 1e-6
    freqs = gem.inv_freq(d, 10_000.0, d // 2)
    q_norm = [0.6 + 0.03 * i for i in range(d)]
    k_norm = [1.2 - 0.02 * i for i in range(d)]
    raw_q = [[gem.deterministic(d, 0x4000 + 16 * t + h) for h in range(heads)] for t in range(tokens)]
    raw_k = [[gem.deterministic(d, 0x5000 + 16 * t + h) for h in range(kv)] for t in range(tokens)]
    raw_v = [[gem.deterministic(d, 0x6000 + 16 * t + h) for h in range(kv)] for t in range(tokens)]
    keys = [[gem.rope(gem.rms_norm(raw_k[t][h], k_norm, eps), t, freqs) for h in range(kv)]
            for t in range(tokens)]
    values = [[gem.rms_norm(raw_v[t][h], None, eps) for h in range(kv)] for t in range(tokens)]
    expected = []
    for t in range(tokens):
        row = []
        for h in range(heads):
            q = gem.rope(gem.rms_norm(raw_q[t][h], q_norm, eps), t, freqs)
            kvh = h // (heads // kv)
            row += gem.attention(q, [keys[p][kvh] for p in range(t + 1)],
                                 [values[p][kvh] for p in range(t + 1)], window=window)
        expected.append(row)
    composed["gemma_block"] = {
        "heads": heads, "kv_heads": kv, "head_dim": d, "tokens": tokens, "window": window,
        "eps": eps, "theta": 10_000.0, "rotating_pairs": d // 2, "inverse_frequencies": freqs,
        "q_norm": q_norm, "k_norm": k_norm, "q": raw_q, "k": raw_k, "v": raw_v,
        "expected": expected,
    }

    # ---- composed case 3: the Qwen block's attention path ---------------------------------------
    heads, kv, d, tokens = 4, 2, 16, 7
    rotating = int(d * 0.25) // 2          # QwenReferenceLayer.swift:206
    freqs = gem.inv_freq(d, 10_000_000.0, rotating)
    q_norm = [0.9 + 0.01 * i for i in range(d)]
    k_norm = [1.1 - 0.01 * i for i in range(d)]
    combined = [[gem.deterministic(2 * d, 0x7000 + 16 * t + h) for h in range(heads)]
                for t in range(tokens)]          # [t][head][2d]: query then gate, per head
    raw_k = [[gem.deterministic(d, 0x8000 + 16 * t + h) for h in range(kv)] for t in range(tokens)]
    raw_v = [[gem.deterministic(d, 0x9000 + 16 * t + h) for h in range(kv)] for t in range(tokens)]
    keys = [[gem.rope(gem.rms_norm(raw_k[t][h], k_norm, eps), t, freqs) for h in range(kv)]
            for t in range(tokens)]
    scale = 1.0 / math.sqrt(d)
    expected = []
    for t in range(tokens):
        row = []
        for h in range(heads):
            query, gate = combined[t][h][:d], combined[t][h][d:]
            q = gem.rope(gem.rms_norm(query, q_norm, eps), t, freqs)
            kvh = h // (heads // kv)
            attended = gem.attention([x * scale for x in q],
                                     [keys[p][kvh] for p in range(t + 1)],
                                     [raw_v[p][kvh] for p in range(t + 1)])
            row += [a * (1.0 / (1.0 + math.exp(-g))) for a, g in zip(attended, gate)]
        expected.append(row)
    composed["qwen_block"] = {
        "heads": heads, "kv_heads": kv, "head_dim": d, "tokens": tokens, "eps": eps,
        "theta": 10_000_000.0, "rotating_pairs": rotating, "inverse_frequencies": freqs,
        "q_norm": q_norm, "k_norm": k_norm, "q_and_gate": combined, "k": raw_k, "v": raw_v,
        "sm_scale": scale, "expected": expected,
    }
    out["composed"] = composed

    path = os.path.join(here, "hydra_reference_vectors.json")
    with open(path, "w") as f:
        json.dump(out, f)
    print(f"{path}  ({os.path.getsize(path):,} bytes)")


if __name__ == "__main__":
    main()
