"""The five benchmark configurations at full size on the GPU, checked against the oracle.

Small configurations are compared row for row; the large ones on a deterministic sample of query
rows (every chunk's first and last row plus a stride), since the oracle is a scalar double-precision
loop.  Size-independent properties cover the rest: chunked prefill == one-shot prefill, bit for bit,
and the decode step == the same row computed by prefill.
"""
import numpy as np
import pytest

from oracle import hydra_oracle as ho
from tests import hydra_testlib as tl

pytestmark = pytest.mark.gpu
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


def oracle_rows(cfg, spec, entry, rows, k_hist=None, v_hist=None, positions=None, cache=None, layer=0):
    """The oracle on query rows `rows` of one layer; history defaults to the layer's own k, v.
    With `cache`, the keys and values are the rows the device cache holds (checked separately
    against the oracle's prologue), so the comparison measures attention alone."""
    d = cfg.head_dim
    inv = ho.inverse_frequencies(d, spec.theta, spec.rotating_pairs)
    q = entry["q"][rows]
    gate = None
    if cfg.gate:
        q, gate = np.ascontiguousarray(q[:, :, :d]), np.ascontiguousarray(q[:, :, d:])
    k = entry["k"] if k_hist is None else k_hist
    v = entry["v"] if v_hist is None else v_hist
    positions = np.asarray(rows if positions is None else positions)
    upto = int(positions.max()) + 1
    cache_rows = None
    if cache is not None:
        cache_rows = tl.read_cache(cache, layer, upto, cfg.kv_heads, d)
        kc, ks = ho.rope_tables(inv, np.arange(upto), as_float32=True)
        k_norm = entry.get("k_norm")
        assert tl.prologue_matches(cache_rows[0], ho.prepare_heads(k[:upto], k_norm, k_norm is not None, 1e-6, kc, ks))
        assert tl.prologue_matches(cache_rows[1], ho.prepare_heads(v[:upto], None, cfg.v_norm, 1e-6))
    return tl.oracle_path(q, k[:upto], v[:upto], positions, cfg.scale, spec.window,
                          sinks=entry.get("sinks"), gate=gate, inv_freq=inv,
                          q_norm=entry.get("q_norm"), k_norm=entry.get("k_norm"), norm_v=cfg.v_norm,
                          cache_rows=cache_rows)


def sample_rows(prompt, chunk, stride):
    rows = set(range(0, prompt, stride))
    for start in range(0, prompt, chunk):
        rows.add(start)
        rows.add(min(start + chunk, prompt) - 1)
    return np.array(sorted(rows))


def test_c1_gpt_oss_20b_layer_prefill_then_decode(hb, ctx):
    from hydra_b200 import workloads as wl
    cfg = wl.config("C1")
    inputs = wl.Inputs(cfg)
    run = wl.PathRunner(ctx, cfg, inputs)
    run.prefill_pass()
    for step in range(cfg.decode_steps):
        run.decode_step(cfg.prompt + step, cfg.prompt + step)
    ctx.check()
    got = run.output()
    want = oracle_rows(cfg, cfg.layers[0], inputs.layers[0], np.arange(cfg.prompt + cfg.decode_steps))
    tl.record_margin("C1 prefill + 64 decode steps", got, want)
    assert tl.within_tolerance(got, want)
    assert tl.deviation(got, want) < TOL
    # the decode steps again, as one prefill chunk: the same bits
    run.backend.attention_prefill(run.cache, 0, run.dev[0]["q"][cfg.prompt:], run.dev[0]["out"][cfg.prompt:],
                                  cfg.decode_steps, cfg.prompt, run.params[0])
    ctx.check()
    assert np.array_equal(run.output()[cfg.prompt:], got[cfg.prompt:])
    run.close()


def test_c2_full_causal_4096(hb, ctx):
    from hydra_b200 import workloads as wl
    cfg = wl.config("C2")
    inputs = wl.Inputs(cfg)
    run = wl.PathRunner(ctx, cfg, inputs)
    run.prefill_pass()
    run.decode_step(cfg.prompt, cfg.prompt)
    ctx.check()
    got = run.output()
    rows = np.append(sample_rows(cfg.prompt, cfg.chunk, 331), cfg.prompt)
    want = oracle_rows(cfg, cfg.layers[0], inputs.layers[0], rows)
    tl.record_margin("C2 sampled prefill rows + decode at 4096", got[rows], want)
    assert tl.within_tolerance(got[rows], want)
    # one-shot prefill of the whole prompt == chunked prefill, bit for bit
    chunked = got[:cfg.prompt].copy()
    run.backend.attention_prefill(run.cache, 0, run.dev[0]["q"], run.dev[0]["out"], cfg.prompt, 0, run.params[0])
    ctx.check()
    assert np.array_equal(run.output()[:cfg.prompt], chunked)
    # the decode row == the same row by the prefill kernel
    run.backend.attention_prefill(run.cache, 0, run.dev[0]["q"][cfg.prompt:], run.dev[0]["out"][cfg.prompt:],
                                  1, cfg.prompt, run.params[0])
    ctx.check()
    assert np.array_equal(run.output()[cfg.prompt], got[cfg.prompt])
    run.close()


def test_c2_head_shards_equal_the_unsharded_run(hb, ctx):
    """KV-head sharding exchanges nothing: a shard's output is the matching slice, bit for bit."""
    from hydra_b200 import workloads as wl
    full = wl.config("C2")
    full.prompt, full.context, full.decode_steps = 1024, 1025, 1
    inputs = wl.Inputs(full)
    run = wl.PathRunner(ctx, full, inputs)
    run.prefill_pass()
    run.decode_step(full.prompt, full.prompt)
    ctx.check()
    whole = run.output()
    run.close()
    for world in (2, 8):
        per = full.kv_heads // world
        for rank in (0, world - 1):
            shard = wl.config("C2", kv_heads=per)
            shard.prompt, shard.context, shard.decode_steps = 1024, 1025, 1
            part = wl.PathRunner(ctx, shard, wl.Inputs(shard, full_heads=full, head_offset=rank * per))
            part.prefill_pass()
            part.decode_step(shard.prompt, shard.prompt)
            ctx.check()
            group = full.q_heads // full.kv_heads
            lo, hi = rank * per * group, (rank + 1) * per * group
            assert np.array_equal(part.output(), whole[:, lo:hi])
            part.close()


def test_c3_gemma_stack(hb, ctx):
    """All six layers, prefill and the 128 decode steps, to 1e-2.  At this context (8320 > 8192) the
    local layers live in rings of 1536 rows, which by the end have dropped the early keys; so the stack
    runs twice, once as configured and once with linear storage: the two must agree bit for bit on
    every row, and the linear run's cache gives the oracle the rows the kernels saw (the reference's
    rule: both sides attend over the same bf16 values)."""
    from hydra_b200 import workloads as wl
    cfg = wl.config("C3")
    inputs = wl.Inputs(cfg)
    outputs = {}
    for storage in (hb.capi.HC_STORAGE_AUTO, hb.capi.HC_STORAGE_LINEAR):
        run = wl.PathRunner(ctx, cfg, inputs, storage=storage)
        run.prefill_pass(fused=True)
        for step in range(cfg.decode_steps):
            run.decode_step(cfg.prompt + step, cfg.prompt + step)
        ctx.check()
        outputs[storage] = [run.output(layer) for layer in range(len(cfg.layers))]
        if storage == hb.capi.HC_STORAGE_AUTO:
            assert run.cache.layer(0).ring_size == 1536 and run.cache.layer(5).ring_size == 0
            run.close()
    for layer in range(len(cfg.layers)):
        assert np.array_equal(outputs[hb.capi.HC_STORAGE_AUTO][layer], outputs[hb.capi.HC_STORAGE_LINEAR][layer]), layer
    steps = cfg.prompt + np.array([0, 1, 31, 64, 100, cfg.decode_steps - 1])
    rows = np.concatenate([np.array([0, 1, 511, 512, 1023, 1024, 1500, 4095, 4096, 8191]), steps])
    for layer, spec in enumerate(cfg.layers):
        want = oracle_rows(cfg, spec, inputs.layers[layer], rows, cache=run.cache, layer=layer)
        got = outputs[hb.capi.HC_STORAGE_LINEAR][layer][rows]
        tl.record_margin(f"C3 layer {layer} ({'global' if spec.window == 0 else 'window %d' % spec.window})", got, want)
        assert tl.within_tolerance(got, want), layer
    run.close()


def test_c4_qwen_gated_decode_at_32768(hb, ctx):
    from hydra_b200 import workloads as wl
    cfg = wl.config("C4")
    inputs = wl.Inputs(cfg)
    run = wl.PathRunner(ctx, cfg, inputs)
    run.fill_history([cfg.prefilled])
    position = cfg.prefilled
    run.decode_step(0, position)
    ctx.check()
    got = run.output()
    # history rows are stored as drawn; the new token's k goes through norm + rotation
    hk, hv = inputs.history(0, cfg.prefilled)
    d = cfg.head_dim
    spec, entry = cfg.layers[0], inputs.layers[0]
    inv = ho.inverse_frequencies(d, spec.theta, spec.rotating_pairs)
    c, s = ho.rope_tables(inv, [position], as_float32=True)
    k_new, _ = tl.read_cache(run.cache, 0, 1, cfg.kv_heads, d, position=position)
    assert tl.prologue_matches(k_new, ho.prepare_heads(entry["k"], entry["k_norm"], True, 1e-6, c, s))
    q = ho.prepare_heads(np.ascontiguousarray(entry["q"][:, :, :d]), entry["q_norm"], True, 1e-6, c, s)
    gate = np.ascontiguousarray(entry["q"][:, :, d:])
    want = ho.attention_rows(q, [position], np.concatenate([hk, k_new]), np.concatenate([hv, entry["v"]]),
                             cfg.scale, 0, gate=gate)
    tl.record_margin("C4 decode at 32768", got, want)
    assert tl.within_tolerance(got, want)
    run.close()


def test_c5_ragged_batched_decode(hb, ctx):
    from hydra_b200 import workloads as wl
    cfg = wl.config("C5")
    inputs = wl.Inputs(cfg)
    lengths = inputs.lengths
    assert int(lengths.sum()) == 591950 and int(lengths.min()) == 1104 and int(lengths.max()) == 16315
    run = wl.PathRunner(ctx, cfg, inputs)
    run.fill_history(lengths - 1)
    positions = [int(n) - 1 for n in lengths]
    run.decode_batch(positions)
    ctx.check()
    d = cfg.head_dim
    for layer, spec in enumerate(cfg.layers):
        got = run.output(layer)
        entry = inputs.layers[layer]
        inv = ho.inverse_frequencies(d, spec.theta)
        for seq in (0, 7, 21, 40, 63, int(np.argmin(lengths)), int(np.argmax(lengths))):
            pos = positions[seq]
            hk, hv = inputs.history(seq, pos)
            c, s = ho.rope_tables(inv, [pos], as_float32=True)
            k_new = ho.prepare_heads(entry["k"][seq:seq + 1], None, False, 1e-6, c, s)
            q = ho.prepare_heads(entry["q"][seq:seq + 1], None, False, 1e-6, c, s)
            want = ho.attention_rows(q, [pos], np.concatenate([hk, k_new]),
                                     np.concatenate([hv, entry["v"][seq:seq + 1]]), cfg.scale, spec.window,
                                     sinks=entry["sinks"])
            tl.record_margin(f"C5 layer {layer} sequence {seq} (context {pos + 1})", got[seq], want[0])
            assert tl.within_tolerance(got[seq], want[0]), (layer, seq)
    run.close()
