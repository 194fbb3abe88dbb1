"""GPU parity tests of the attention kernels, through the C ABI, against the CPU oracle.

Shapes, key counts and properties follow the reference's own kernel tests
(Tests/HydraMetalTests/AttentionKernelTests.swift, GemmaKernelTests.swift).  The bound is the one
the task states: max-abs 1e-2 on unit-variance outputs (fp32 accumulate, bf16 softmax weights),
plus the reference's relative-deviation metric.  Equality tests are exact (`array_equal`).
"""
import json
import os

import numpy as np
import pytest

from oracle import hydra_oracle as ho
from tests import hydra_testlib as tl

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))
TOL = 1e-2


@pytest.fixture(scope="module")
def hb():
    import hydra_b200
    return hydra_b200


@pytest.fixture(scope="module")
def ctx(hb):
    c = hb.Context(0)
    yield c
    c.close()


@pytest.fixture(scope="module")
def golden():
    with open(os.path.join(HERE, "golden", "hydra_reference_vectors.json")) as f:
        return json.load(f)


# ---- golden vectors, on the device ---------------------------------------------------------------

@pytest.mark.parametrize("name", ["sdpa_full", "sdpa_sliding"])
def test_reference_sdpa_fixture_on_device(hb, ctx, golden, name):
    g = golden["committed"]["reference_ops"][name]
    tokens, kv, mult, d = g["tokens"], g["kv_heads"], g["q_mult"], g["head_dim"]
    q = ho.bf16_round(np.asarray(g["q"], np.float32))
    k = ho.bf16_round(np.asarray(g["k"], np.float32))
    v = ho.bf16_round(np.asarray(g["v"], np.float32))
    sinks = ho.bf16_round(np.asarray(g["sinks"], np.float32))
    want = ho.sdpa(q, k, v, sinks, g["sm_scale"], g["sliding_window"])
    # The rounded inputs stay close to the fixture's own expectation (sanity of the rounding rule).
    assert tl.max_abs(want, g["expected"]) < 5e-2
    layer = tl.Layer(hb, ctx, kv * mult, kv, d, 128, window=g["sliding_window"],
                     sm_scale=g["sm_scale"], sinks=sinks, io="f32")
    layer.append(k, v, 0)
    got = layer.prefill(q.reshape(tokens, kv * mult, d), 0)
    assert tl.max_abs(got.reshape(tokens, -1), want) < TOL
    # token by token: the same bits
    step = np.stack([layer.decode(q.reshape(tokens, kv * mult, d)[t:t + 1], [t])[0] for t in range(tokens)])
    assert np.array_equal(step, got)
    layer.close()


@pytest.mark.parametrize("name", ["attention_full", "attention_windowed"])
def test_gemma_attention_fixture_on_device(hb, ctx, golden, name):
    g = golden["committed"]["gemma4_operators"][name]
    q = ho.bf16_round(np.asarray(g["query"], np.float32))
    keys = ho.bf16_round(np.asarray(g["keys"], np.float32))
    values = ho.bf16_round(np.asarray(g["values"], np.float32))
    n, d = keys.shape
    want = ho.gemma_attention(q, keys, values, g["window"])
    layer = tl.Layer(hb, ctx, 1, 1, d, 128, window=g["window"], sm_scale=1.0, io="f32")
    layer.append(keys.reshape(n, 1, d), values.reshape(n, 1, d), 0)
    got = layer.decode(q.reshape(1, 1, d), [n - 1])
    assert tl.max_abs(got.reshape(-1), want) < TOL
    layer.close()


# ---- the reference's kernel tests ----------------------------------------------------------------

def _decode_case(hb, ctx, q_heads, kv_heads, d, keys, seed, sinks_scale=1.0, window=0, storage=0,
                 sm_scale=None, kernel_path=0, context=None):
    """AttentionKernelTests.swift:90-139: one query against `keys` cached keys."""
    q = ho.bf16_round(tl.deterministic(q_heads * d, seed).reshape(1, q_heads, d))
    k = ho.bf16_round(tl.deterministic(keys * kv_heads * d, seed + 1).reshape(keys, kv_heads, d))
    v = ho.bf16_round(tl.deterministic(keys * kv_heads * d, seed + 2).reshape(keys, kv_heads, d))
    sinks = ho.bf16_round(tl.deterministic(q_heads, seed + 3) * sinks_scale) if sinks_scale is not None else None
    scale = sm_scale if sm_scale is not None else 1.0 / np.sqrt(d)
    context = context or max(keys, 128)
    layer = tl.Layer(hb, ctx, q_heads, kv_heads, d, context, window=window, sm_scale=scale, sinks=sinks,
                     storage=storage, kernel_path=kernel_path)
    for start in range(0, keys, 512):
        layer.append(k[start:start + 512], v[start:start + 512], start)
    got = layer.decode(q, [keys - 1])
    want = ho.attention_rows(q, [keys - 1], k, v, scale, window, sinks=sinks)
    layer.close()
    return got, want


def test_decode_matches_reference_gpt_oss_shape(hb, ctx):
    got, want = _decode_case(hb, ctx, 64, 8, 64, 40, seed=31)
    assert tl.deviation(got, want) < TOL and tl.max_abs(got, want) < TOL


@pytest.mark.parametrize("shape", [(16, 8, 256), (16, 2, 512)])
def test_decode_matches_reference_gemma_widths(hb, ctx, shape):
    """AttentionKernelTests.swift:155-204: 600 keys, scale 1.0, no sink."""
    got, want = _decode_case(hb, ctx, *shape, 600, seed=41, sinks_scale=None, sm_scale=1.0)
    # Scale 1.0 on [-1, 1) inputs gives sharp distributions; outputs stay O(1).
    assert tl.deviation(got, want) < TOL


def test_decode_finite_with_a_single_key(hb, ctx):
    """AttentionKernelTests.swift:212-228: fewer keys than parallel splits must not produce NaN."""
    for keys in (1, 2, 3):
        got, want = _decode_case(hb, ctx, 64, 8, 64, keys, seed=51)
        assert np.all(np.isfinite(got))
        assert tl.max_abs(got, want) < TOL


def test_ring_storage_equals_linear_storage_bit_for_bit(hb, ctx):
    """AttentionKernelTests.swift:232-254 and KVReuseTests.swift:85-107."""
    q_heads, kv_heads, d, window, total = 16, 4, 64, 128, 1500
    rng = np.random.default_rng(61)
    k = tl.normal_bf16(rng, (total, kv_heads, d))
    v = tl.normal_bf16(rng, (total, kv_heads, d))
    q = tl.normal_bf16(rng, (total, q_heads, d))
    sinks = tl.normal_bf16(rng, (q_heads,))
    outs = []
    for storage in (hb.capi.HC_STORAGE_LINEAR, hb.capi.HC_STORAGE_RING):
        layer = tl.Layer(hb, ctx, q_heads, kv_heads, d, 2048, window=window, sinks=sinks,
                         storage=storage, prefill_chunk=256)
        info = layer.cache.layer(0)
        assert (info.ring_size > 0) == (storage == hb.capi.HC_STORAGE_RING)
        rows = []
        for start in range(0, total, 256):
            n = min(256, total - start)
            layer.append(k[start:start + n], v[start:start + n], start)
            rows.append(layer.prefill(q[start:start + n], start))
        outs.append(np.concatenate(rows))
        layer.close()
    assert np.array_equal(outs[0], outs[1])
    want = ho.attention_rows(q[-64:], np.arange(total - 64, total), k, v, 1 / np.sqrt(d), window, sinks=sinks)
    assert tl.within_tolerance(outs[1][-64:], want)


def test_sink_vanishes_when_unreachable(hb, ctx):
    """AttentionKernelTests.swift:258-285 and GemmaKernelTests.swift:197-251: a sink at -1e9 (or the
    reference's -1e30) is the same as no sink."""
    q_heads, kv_heads, d, keys = 16, 8, 256, 300
    rng = np.random.default_rng(71)
    q = tl.normal_bf16(rng, (1, q_heads, d))
    k = tl.normal_bf16(rng, (keys, kv_heads, d))
    v = tl.normal_bf16(rng, (keys, kv_heads, d))
    results = []
    for sink in (None, -1e9, -1e30):
        sinks = None if sink is None else ho.bf16_round(np.full(q_heads, sink, np.float32))
        layer = tl.Layer(hb, ctx, q_heads, kv_heads, d, 512, sm_scale=1 / 16.0, sinks=sinks)
        layer.append(k, v, 0)
        results.append(layer.decode(q, [keys - 1]))
        layer.close()
    assert np.array_equal(results[0], results[1]) and np.array_equal(results[0], results[2])


@pytest.mark.parametrize("shape", [(16, 2, 128), (16, 2, 512), (8, 8, 256)])
def test_split_decode_at_3000_keys_with_competitive_sinks(hb, ctx, shape):
    """AttentionKernelTests.swift:395-427."""
    got, want = _decode_case(hb, ctx, *shape, 3000, seed=81, sinks_scale=3.0, context=3072)
    assert tl.deviation(got, want) < TOL and tl.max_abs(got, want) < TOL


@pytest.mark.parametrize("keys", [511, 512, 513, 640, 1023, 1025, 1279])
def test_ragged_tile_boundaries(hb, ctx, keys):
    """AttentionKernelTests.swift:439-468."""
    got, want = _decode_case(hb, ctx, 64, 8, 64, keys, seed=91 + keys, context=1280)
    assert tl.max_abs(got, want) < TOL


# ---- chunked prefill is token-by-token decode, bit for bit ----------------------------------------

@pytest.mark.parametrize("case", [
    dict(q_heads=64, kv_heads=8, d=64, window=128, tokens=300, chunk=128, sinks=True),
    dict(q_heads=64, kv_heads=8, d=64, window=0, tokens=700, chunk=512, sinks=True),
    dict(q_heads=16, kv_heads=8, d=256, window=0, tokens=261, chunk=256, sinks=False),
    dict(q_heads=16, kv_heads=2, d=256, window=0, tokens=200, chunk=64, sinks=False),
])
def test_chunked_prefill_equals_decode_exactly(hb, ctx, case):
    """GemmaLayerTests.swift:443-526 asks for exact equality; here at every length and shape."""
    rng = np.random.default_rng(101)
    qh, kvh, d, tokens, chunk = case["q_heads"], case["kv_heads"], case["d"], case["tokens"], case["chunk"]
    q = tl.normal_bf16(rng, (tokens, qh, d))
    k = tl.normal_bf16(rng, (tokens, kvh, d))
    v = tl.normal_bf16(rng, (tokens, kvh, d))
    sinks = tl.normal_bf16(rng, (qh,)) if case["sinks"] else None
    inv = ho.inverse_frequencies(d, 150000.0)
    outs = {}
    for mode in ("chunked", "stepwise", "whole"):
        layer = tl.Layer(hb, ctx, qh, kvh, d, 1024, window=case["window"], sinks=sinks, rope_inv_freq=inv,
                         prefill_chunk=1024)
        rows = []
        if mode == "stepwise":
            for t in range(tokens):
                layer.append(k[t:t + 1], v[t:t + 1], t)
                rows.append(layer.decode(q[t:t + 1], [t]))
        else:
            step = chunk if mode == "chunked" else tokens
            for start in range(0, tokens, step):
                n = min(step, tokens - start)
                layer.append(k[start:start + n], v[start:start + n], start)
                rows.append(layer.prefill(q[start:start + n], start))
        outs[mode] = np.concatenate(rows)
        layer.close()
    assert np.array_equal(outs["chunked"], outs["stepwise"])
    assert np.array_equal(outs["chunked"], outs["whole"])
    want = tl.oracle_path(q, k, v, np.arange(tokens), 1 / np.sqrt(d), case["window"], sinks=sinks, inv_freq=inv)
    assert tl.within_tolerance(outs["chunked"], want)


# ---- fused prologue and epilogue -----------------------------------------------------------------

def test_gemma_block_norms_rotation_scale_one(hb, ctx):
    """q/k RMSNorm with weight, weightless v norm, rotation, scale 1.0, window; the order of
    Sources/HydraReference/Gemma4ReferenceLayer.swift:146-162, 223-248."""
    rng = np.random.default_rng(111)
    qh, kvh, d, tokens, window = 16, 8, 256, 96, 40
    q = tl.normal_bf16(rng, (tokens, qh, d))
    k = tl.normal_bf16(rng, (tokens, kvh, d))
    v = tl.normal_bf16(rng, (tokens, kvh, d))
    qn = ho.bf16_round((1 + 0.1 * rng.standard_normal(d)).astype(np.float32))
    kn = ho.bf16_round((0.2 + 0.02 * rng.standard_normal(d)).astype(np.float32))
    inv = ho.inverse_frequencies(d, 10000.0)
    layer = tl.Layer(hb, ctx, qh, kvh, d, 128, window=window, sm_scale=1.0, rope_inv_freq=inv, q_norm=qn,
                     k_norm=kn, norm_v=True)
    layer.append(k, v, 0)
    got = layer.prefill(q, 0)
    # 1. the cache holds what the oracle's prologue produces
    k_dev, v_dev = tl.read_cache(layer.cache, 0, tokens, kvh, d)
    kc, ks = ho.rope_tables(inv, np.arange(tokens), as_float32=True)
    assert tl.prologue_matches(k_dev, ho.prepare_heads(k, kn, True, 1e-6, kc, ks))
    assert tl.prologue_matches(v_dev, ho.prepare_heads(v, None, True, 1e-6))
    # 2. attention over those rows
    want = tl.oracle_path(q, k, v, np.arange(tokens), 1.0, window, inv_freq=inv, q_norm=qn, k_norm=kn,
                          norm_v=True, cache_rows=(k_dev, v_dev))
    assert tl.within_tolerance(got, want)
    layer.close()


def test_qwen_block_partial_rotary_interleaved_gate(hb, ctx):
    """Per-head query/gate split, q/k norm, partial rotation, 1/sqrt(d), sigmoid gate
    (Sources/HydraReference/QwenReferenceLayer.swift:251-304)."""
    rng = np.random.default_rng(121)
    qh, kvh, d, tokens = 16, 2, 256, 70
    combined = tl.normal_bf16(rng, (tokens, qh, 2 * d))
    q, gate = combined[:, :, :d].copy(), combined[:, :, d:].copy()
    k = tl.normal_bf16(rng, (tokens, kvh, d))
    v = tl.normal_bf16(rng, (tokens, kvh, d))
    qn = ho.bf16_round((1 + 0.1 * rng.standard_normal(d)).astype(np.float32))
    kn = ho.bf16_round((1 + 0.1 * rng.standard_normal(d)).astype(np.float32))
    inv = ho.inverse_frequencies(d, 1e7, int(d * 0.25) // 2)
    for layout in ("interleaved", "separate"):
        gl = hb.capi.HC_GATE_INTERLEAVED if layout == "interleaved" else hb.capi.HC_GATE_NONE
        layer = tl.Layer(hb, ctx, qh, kvh, d, 128, rope_inv_freq=inv, q_norm=qn, k_norm=kn, gate_layout=gl)
        layer.append(k, v, 0)
        k_dev, v_dev = tl.read_cache(layer.cache, 0, tokens, kvh, d)
        kc, ks = ho.rope_tables(inv, np.arange(tokens), as_float32=True)
        assert tl.prologue_matches(k_dev, ho.prepare_heads(k, kn, True, 1e-6, kc, ks))
        assert np.array_equal(v_dev, v)
        want = tl.oracle_path(q, k, v, np.arange(tokens), 1 / 16.0, 0, gate=gate, inv_freq=inv, q_norm=qn,
                              k_norm=kn, cache_rows=(k_dev, v_dev))
        if layout == "interleaved":
            got = _prefill_interleaved(layer, combined)
            last = _decode_interleaved(layer, combined[-1:], tokens - 1)
        else:
            got = layer.prefill(q, 0, gate=gate)
            last = layer.decode(q[-1:], [tokens - 1], gate=gate[-1:])
        assert tl.within_tolerance(got, want)
        assert np.array_equal(last[0], got[-1])
        layer.close()


def _prefill_interleaved(layer, combined):
    tokens = combined.shape[0]
    qd = tl.to_device(combined, layer.io)
    out = tl.device_empty((tokens, layer.q_heads, layer.d), layer.io)
    layer.backend.attention_prefill(layer.cache, 0, qd, out, tokens, 0, layer.params)
    layer.ctx.check()
    return tl.to_host(out)


def _decode_interleaved(layer, combined_row, position):
    qd = tl.to_device(combined_row, layer.io)
    out = tl.device_empty((1, layer.q_heads, layer.d), layer.io)
    layer.backend.attention(layer.cache, 0, qd, out, [position], layer.params)
    layer.ctx.check()
    return tl.to_host(out)


def test_standalone_elementwise_kernels(hb, ctx):
    """rmsNormHeads, applyRoPE, qwenSplitQueryGate, qwenApplyOutputGate, fp32 buffers as in the
    reference (AttentionKernelTests.swift:61-88, QwenAttentionGateTests.swift:40-118)."""
    import torch
    backend = hb.AttentionBackend(ctx)
    rng = np.random.default_rng(131)
    tokens, heads, d = 5, 8, 64
    x = rng.standard_normal((tokens, heads, d)).astype(np.float32)
    w = ho.bf16_round((1 + 0.1 * rng.standard_normal(d)).astype(np.float32))
    xd = tl.to_device(x, "f32")
    backend.rms_norm_heads(xd, tl.to_device(w), tokens, heads, d, 1e-6)
    want = np.stack([[ho.rms_norm(x[t, h], w, 1e-6) for h in range(heads)] for t in range(tokens)])
    assert tl.deviation(tl.to_host(xd), want) < 1e-5
    xd = tl.to_device(x, "f32")
    backend.rms_norm_heads(xd, None, tokens, heads, d, 1e-6)
    want = np.stack([[ho.rms_norm(x[t, h], None, 1e-6) for h in range(heads)] for t in range(tokens)])
    assert tl.deviation(tl.to_host(xd), want) < 1e-5

    inv, conc = ho.yarn_inverse_frequencies(d, 150000.0, 4096, 32.0, 1.0, 32.0)
    table = hb.RopeTable(ctx, list(inv), 4200, conc)
    first = 4090
    xd = tl.to_device(x, "f32")
    backend.apply_rope(xd, table, tokens, heads, d, first)
    cos, sin = ho.rope_tables(inv, np.arange(first, first + tokens), conc)
    want = np.stack([[ho.apply_rope(x[t, h], cos[t], sin[t]) for h in range(heads)] for t in range(tokens)])
    assert tl.deviation(tl.to_host(xd), want) < 1e-5
    # zero frequency is an exact identity (GemmaKernelTests.swift:256-273)
    partial = hb.RopeTable(ctx, list(ho.inverse_frequencies(d, 1e6, 4)), 64)
    xd = tl.to_device(x, "f32")
    backend.apply_rope(xd, partial, tokens, heads, d, 7)
    got = tl.to_host(xd)
    assert np.array_equal(got[:, :, 4:32], x[:, :, 4:32]) and np.array_equal(got[:, :, 36:], x[:, :, 36:])
    table.close()
    partial.close()

    combined = rng.standard_normal((tokens, heads, 2 * d)).astype(np.float32)
    cd = tl.to_device(combined, "f32")
    qd = tl.device_empty((tokens, heads, d), "f32")
    gd = tl.device_empty((tokens, heads, d), "f32")
    backend.qwen_split_query_gate(cd, qd, gd, tokens, heads, d)
    assert np.array_equal(tl.to_host(qd), combined[:, :, :d]) and np.array_equal(tl.to_host(gd), combined[:, :, d:])
    backend.qwen_apply_output_gate(qd, gd, tokens * heads * d)
    want = ho.apply_output_gate(combined[:, :, :d].reshape(-1), combined[:, :, d:].reshape(-1))
    assert tl.deviation(tl.to_host(qd).reshape(-1), want) < 1e-5
    torch.cuda.synchronize()


# ---- the cache object ------------------------------------------------------------------------------

def test_kv_cache_bookkeeping_and_errors(hb, ctx):
    """KVCache.swift:95-104, 193-229; KVReuseTests.swift:56-83; sizing as GptOssConfigTests.swift:57-60."""
    layers = [dict(q_heads=64, kv_heads=8, head_dim=64, window=128),
              dict(q_heads=64, kv_heads=8, head_dim=64, window=0),
              dict(q_heads=0, kv_heads=0, head_dim=0, window=0)]          # a recurrent layer
    cache = hb.KVCache(ctx, layers, 16384, prefill_chunk=512)
    sliding, full, recurrent = cache.layer(0), cache.layer(1), cache.layer(2)
    assert sliding.ring_size == 640 and sliding.capacity == 1152 and sliding.windowed == 1   # stored one margin longer
    assert full.ring_size == 0 and full.capacity == 16384 and full.entry_bytes == 8 * 64 * 2
    assert recurrent.keeps_history == 0 and recurrent.entry_bytes == 0
    assert 2 * full.entry_bytes == 2048                                     # bytes per token per full layer
    assert cache.byte_count == 2 * (1152 + 16384) * 8 * 64 * 2              # what is allocated: the ring as stored
    assert cache.visible_range(0, 5) == (0, 6)
    assert cache.visible_range(0, 1000) == (873, 128)
    assert cache.visible_range(1, 1000) == (0, 1001)
    with pytest.raises(hb.UnsupportedPattern):
        cache.visible_range(2, 3)
    cache.advance(1000)
    assert cache.length() == 1000 and cache.rewind_floor() == 1000 - 512
    assert cache.can_rewind(600) and not cache.can_rewind(400) and not cache.can_rewind(1001)
    with pytest.raises(hb.BadRewind):
        cache.rewind(100)
    cache.rewind(990)
    assert cache.length() == 990
    with pytest.raises(hb.CacheOverflow):
        cache.advance(16384)
    cache.reset()
    assert cache.length() == 0
    cache.close()

    small = hb.KVCache(ctx, layers[:2], 4096)                                # <= 8192: everything linear
    assert small.layer(0).ring_size == 0 and small.rewind_floor() == 0
    backend = hb.AttentionBackend(ctx)
    params = hb.AttnParams(q_heads=64, kv_heads=8, head_dim=64, window=0, sm_scale=0.125)
    buf = tl.device_empty((8, 64, 64))
    with pytest.raises(hb.DimensionMismatch):                                # wrong window for layer 0
        backend.attention_prefill(small, 0, buf, buf, 8, 0, params)
    with pytest.raises(hb.CacheOverflow):
        backend.attention_prefill(small, 1, buf, buf, 8, 4090, params)
    with pytest.raises(hb.DimensionMismatch):
        bad = hb.AttnParams(q_heads=64, kv_heads=8, head_dim=128, window=0, sm_scale=0.125)
        backend.attention_prefill(small, 1, buf, buf, 8, 0, bad)
    small.close()
    with pytest.raises(hb.DimensionMismatch):
        hb.KVCache(ctx, [dict(q_heads=8, kv_heads=8, head_dim=520, window=0)], 128)
    with pytest.raises(hb.HydraCudaError):
        hb.KVCache(ctx, [dict(q_heads=8, kv_heads=8, head_dim=64, window=0)], 128, shard=(2, 3, 2))


def test_rewind_then_resume_equals_fresh(hb, ctx):
    """KVReuseTests.swift:111-149: rewinding and re-running the tail gives the fresh result."""
    rng = np.random.default_rng(141)
    qh, kvh, d, tokens = 16, 4, 64, 400
    q = tl.normal_bf16(rng, (tokens, qh, d))
    k = tl.normal_bf16(rng, (tokens, kvh, d))
    v = tl.normal_bf16(rng, (tokens, kvh, d))
    k2 = tl.normal_bf16(rng, (tokens, kvh, d))
    layer = tl.Layer(hb, ctx, qh, kvh, d, 512)
    layer.append(k, v, 0)
    layer.cache.advance(tokens)
    fresh = layer.prefill(q[300:], 300)
    layer.cache.rewind(300)
    layer.append(k2[300:], v[300:], 300)                # an edited tail ...
    edited = layer.prefill(q[300:], 300)
    assert not np.array_equal(edited, fresh)
    layer.append(k[300:], v[300:], 300)                  # ... then the original again
    assert np.array_equal(layer.prefill(q[300:], 300), fresh)
    layer.close()


# ---- host-buffer entry point ------------------------------------------------------------------------

def test_layer_step_with_host_buffers(hb, ctx):
    rng = np.random.default_rng(151)
    qh, kvh, d, tokens = 64, 8, 64, 256
    q = tl.normal_bf16(rng, (tokens + 1, qh, d))
    k = tl.normal_bf16(rng, (tokens + 1, kvh, d))
    v = tl.normal_bf16(rng, (tokens + 1, kvh, d))
    sinks = tl.normal_bf16(rng, (qh,))
    layer = tl.Layer(hb, ctx, qh, kvh, d, 512, sinks=sinks, io="f32")
    out = np.zeros((tokens, qh, d), np.float32)
    layer.backend.layer_step_host(layer.cache, 0, q[:tokens], k[:tokens], v[:tokens], out, tokens, 0, layer.params)
    one = np.zeros((1, qh, d), np.float32)
    layer.backend.layer_step_host(layer.cache, 0, q[tokens:], k[tokens:], v[tokens:], one, 1, tokens, layer.params)
    want = ho.attention_rows(q, np.arange(tokens + 1), k, v, 0.125, 0, sinks=sinks)
    assert tl.max_abs(out, want[:tokens]) < TOL and tl.max_abs(one, want[tokens:]) < TOL
    layer.close()


@pytest.mark.parametrize("gated", [False, True])
def test_whole_prompt_entry_points_equal_the_chunk_by_chunk_calls(hb, ctx, gated):
    """hc_prefill_chunks (device buffers) and hc_prefill_host (pinned host buffers, copies overlapped
    with the kernels over two staging slots) against one hc_layer_step per chunk: the same bits, with a
    last chunk that is not full and more chunks than staging slots."""
    import torch
    rng = np.random.default_rng(171)
    qh, kvh, d, tokens, chunk = 16, 4, 64, 1100, 256
    q = tl.normal_bf16(rng, (tokens, qh, d))
    k = tl.normal_bf16(rng, (tokens, kvh, d))
    v = tl.normal_bf16(rng, (tokens, kvh, d))
    gate = tl.normal_bf16(rng, (tokens, qh, d)) if gated else None
    sinks = tl.normal_bf16(rng, (qh,))
    inv = ho.inverse_frequencies(d, 10000.0)
    outs = {}
    for mode in ("steps", "chunks", "host"):
        layer = tl.Layer(hb, ctx, qh, kvh, d, 2048, sinks=sinks, rope_inv_freq=inv, prefill_chunk=chunk)
        dev = {name: tl.to_device(x) for name, x in (("q", q), ("k", k), ("v", v))}
        params = layer.params
        gate_dev = tl.to_device(gate) if gated else None
        if gated:
            params = layer._with_gate(gate_dev)
        out = tl.device_empty((tokens, qh, d))
        if mode == "steps":
            for start in range(0, tokens, chunk):
                n = min(chunk, tokens - start)
                p = layer._with_gate(gate_dev[start:]) if gated else params
                layer.backend.layer_step(layer.cache, 0, dev["q"][start:], dev["k"][start:], dev["v"][start:],
                                         out[start:], n, start, p)
        elif mode == "chunks":
            layer.backend.prefill_chunks(layer.cache, 0, dev["q"], dev["k"], dev["v"], out, tokens, 0, chunk, params)
        else:
            host = {name: t.cpu().pin_memory() for name, t in dev.items()}
            host_out = torch.zeros((tokens, qh, d), dtype=torch.bfloat16).pin_memory()
            p = params
            if gated:
                import dataclasses
                host_gate = gate_dev.cpu().pin_memory()
                p = dataclasses.replace(params, gate=host_gate)
            layer.backend.prefill_host(layer.cache, 0, host["q"], host["k"], host["v"], host_out, tokens, 0, chunk, p)
            out = host_out
        ctx.check()
        outs[mode] = tl.to_host(out) if mode != "host" else out.float().numpy()
        layer.close()
    assert np.array_equal(outs["steps"], outs["chunks"])
    assert np.array_equal(outs["steps"], outs["host"])
    want = tl.oracle_path(q, k, v, np.arange(tokens), 0.125, 0, sinks=sinks, gate=gate, inv_freq=inv)
    assert tl.within_tolerance(outs["steps"], want)


@pytest.mark.parametrize("d, qh, kvh", [(64, 16, 4), (256, 4, 2)])
def test_prefill_chunks_on_a_ring_equals_the_chunk_by_chunk_calls(hb, ctx, d, qh, kvh):
    """hc_prefill_chunks runs a chunk's prologue while the previous chunk's attention finishes and lets
    consecutive chunks' attention launches overlap.  On a ring that is only right because the ring is
    stored one margin longer than the window + chunk rows it reports; the prompt here wraps that ring
    more than twice, and every chunk must equal its hc_layer_step and the oracle."""
    rng = np.random.default_rng(907)
    window, chunk, tokens = 256, 128, 2000
    q = tl.normal_bf16(rng, (tokens, qh, d))
    k = tl.normal_bf16(rng, (tokens, kvh, d))
    v = tl.normal_bf16(rng, (tokens, kvh, d))
    sinks = tl.normal_bf16(rng, (qh,))
    outs = {}
    for mode in ("steps", "chunks"):
        layer = tl.Layer(hb, ctx, qh, kvh, d, 4096, window=window, sinks=sinks, prefill_chunk=chunk,
                         storage=hb.capi.HC_STORAGE_RING)
        assert layer.cache.layer(0).ring_size == window + chunk
        dev = {name: tl.to_device(x) for name, x in (("q", q), ("k", k), ("v", v))}
        out = tl.device_empty((tokens, qh, d))
        if mode == "steps":
            for start in range(0, tokens, chunk):
                n = min(chunk, tokens - start)
                layer.backend.layer_step(layer.cache, 0, dev["q"][start:], dev["k"][start:], dev["v"][start:],
                                         out[start:], n, start, layer.params)
        else:
            for _ in range(2):          # twice: the second prompt starts over while the first one's tail may still run
                layer.backend.prefill_chunks(layer.cache, 0, dev["q"], dev["k"], dev["v"], out, tokens, 0, chunk,
                                             layer.params)
        ctx.check()
        outs[mode] = tl.to_host(out)
        layer.close()
    assert np.array_equal(outs["steps"], outs["chunks"])
    want = tl.oracle_path(q, k, v, np.arange(tokens), 1 / np.sqrt(d), window, sinks=sinks)
    assert tl.within_tolerance(outs["chunks"], want)


@pytest.mark.parametrize("d,window", [(64, 0), (128, 96), (256, 0), (96, 0)])
def test_layer_step_equals_append_then_attention(hb, ctx, d, window):
    """hc_layer_step (one prologue launch for k, v and q) gives bit for bit what hc_kv_append followed
    by hc_attention_prefill / hc_attention_decode gives, with norm and rotation in the prologue."""
    rng = np.random.default_rng(152 + d)
    qh, kvh, tokens = 16, 4, 300
    q = tl.normal_bf16(rng, (tokens + 1, qh, d))
    k = tl.normal_bf16(rng, (tokens + 1, kvh, d))
    v = tl.normal_bf16(rng, (tokens + 1, kvh, d))
    sinks = tl.normal_bf16(rng, (qh,))
    qw, kw = tl.normal_bf16(rng, (d,)), tl.normal_bf16(rng, (d,))
    inv = ho.inverse_frequencies(d, 10000.0, d // 2)
    outs = []
    for fused in (False, True):
        layer = tl.Layer(hb, ctx, qh, kvh, d, 512, window=window, sinks=sinks, rope_inv_freq=inv, q_norm=qw, k_norm=kw)
        if fused:
            first = layer.step(q[:200], k[:200], v[:200], 0)
            second = layer.step(q[200:tokens], k[200:tokens], v[200:tokens], 200)
            last = layer.step(q[tokens:], k[tokens:], v[tokens:], tokens)
        else:
            layer.append(k[:200], v[:200], 0)
            first = layer.prefill(q[:200], 0)
            layer.append(k[200:tokens], v[200:tokens], 200)
            second = layer.prefill(q[200:tokens], 200)
            layer.append(k[tokens:], v[tokens:], tokens)
            last = layer.decode(q[tokens:], [tokens])
        outs.append(np.concatenate([first, second, last]))
        layer.close()
    assert np.array_equal(outs[0], outs[1])


# ---- the tcgen05 path -------------------------------------------------------------------------------

@pytest.mark.parametrize("case", [
    dict(q_heads=8, kv_heads=1, d=64, window=0, tokens=333, chunk=100),
    dict(q_heads=64, kv_heads=8, d=64, window=128, tokens=700, chunk=512),
    dict(q_heads=4, kv_heads=4, d=64, window=0, tokens=260, chunk=129),
    dict(q_heads=32, kv_heads=2, d=64, window=200, tokens=520, chunk=256),
    dict(q_heads=16, kv_heads=8, d=128, window=0, tokens=300, chunk=128),
    dict(q_heads=16, kv_heads=2, d=128, window=150, tokens=400, chunk=333),
    dict(q_heads=16, kv_heads=8, d=256, window=0, tokens=300, chunk=128),
    dict(q_heads=16, kv_heads=2, d=256, window=140, tokens=420, chunk=333),
])
def test_tensor_path_prefill_and_decode(hb, ctx, case):
    """The tcgen05 kernels against the oracle, against the CUDA-core kernels (tolerance) and
    against themselves (chunked == one-shot == token by token, exactly)."""
    rng = np.random.default_rng(201)
    qh, kvh, d, tokens, chunk, window = (case[k] for k in ("q_heads", "kv_heads", "d", "tokens", "chunk", "window"))
    q = tl.normal_bf16(rng, (tokens, qh, d))
    k = tl.normal_bf16(rng, (tokens, kvh, d))
    v = tl.normal_bf16(rng, (tokens, kvh, d))
    sinks = tl.normal_bf16(rng, (qh,))
    want = ho.attention_rows(q, np.arange(tokens), k, v, 1 / np.sqrt(d), window, sinks=sinks)
    outs = {}
    for path in (hb.capi.HC_PATH_TENSOR, hb.capi.HC_PATH_SIMT):
        layer = tl.Layer(hb, ctx, qh, kvh, d, 1024, window=window, sinks=sinks, kernel_path=path, prefill_chunk=1024)
        layer.append(k, v, 0)
        whole = layer.prefill(q, 0)
        chunked = np.concatenate([layer.prefill(q[s:s + chunk], s) for s in range(0, tokens, chunk)])
        steps = [0, 1, 127, 128, 129, tokens // 2, tokens - 1]
        stepwise = np.concatenate([layer.decode(q[t:t + 1], [t]) for t in steps])
        assert np.array_equal(whole, chunked), path
        assert np.array_equal(stepwise, whole[steps]), path
        assert tl.within_tolerance(whole, want), path
        outs[path] = whole
        layer.close()
    assert tl.max_abs(outs[hb.capi.HC_PATH_TENSOR], outs[hb.capi.HC_PATH_SIMT]) < 2e-2


def test_tensor_path_batched_ragged_decode(hb, ctx):
    rng = np.random.default_rng(211)
    qh, kvh, d, batch = 64, 8, 64, 5
    lengths = [130, 1, 700, 257, 1024]
    q = tl.normal_bf16(rng, (batch, qh, d))
    sinks = tl.normal_bf16(rng, (qh,))
    layer = tl.Layer(hb, ctx, qh, kvh, d, 1024, sinks=sinks, max_seqs=batch, kernel_path=hb.capi.HC_PATH_TENSOR,
                     prefill_chunk=1024)
    hist = []
    for seq, n in enumerate(lengths):
        k = tl.normal_bf16(rng, (n, kvh, d))
        v = tl.normal_bf16(rng, (n, kvh, d))
        layer.append(k, v, 0, seq=seq)
        hist.append((k, v))
    got = layer.decode(q, [n - 1 for n in lengths], seq_ids=list(range(batch)))
    for seq, n in enumerate(lengths):
        want = ho.attention_rows(q[seq:seq + 1], [n - 1], hist[seq][0], hist[seq][1], 0.125, 0, sinks=sinks)
        assert tl.within_tolerance(got[seq], want[0]), seq
    layer.close()
