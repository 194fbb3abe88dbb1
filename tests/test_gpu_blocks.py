"""Bidirectional blocks in prefill: `blockEnds` of BatchEncoder.attention
(Sources/HydraMetal/BatchEncoder.swift:210-217), the `blocks` buffer of attention_prefill
(Sources/HydraMetal/Shaders/batch.metal:322-324, 340-352).  A token inside a block (an image's
tokens) sees the whole block, forward as well as back; the window still bounds where its range
starts.  The tensor-core kernels take the buffer for head_dim 64, 128 and 256, the general kernel for
the rest.  The oracle applies the shader's loop bound to the reference's double-precision attention.
"""
import dataclasses

import numpy as np
import pytest

from oracle import hydra_oracle as ho
from tests import hydra_testlib as tl

pytestmark = pytest.mark.gpu

TOL = 1e-2


def block_map(first_position, tokens, blocks):
    """One entry per token: one past the end of its block (absolute position), 0 outside blocks, as
    Gemma4ModelRunner builds it (Sources/HydraMetal/Gemma4ModelRunner.swift:457-467)."""
    ends = np.zeros(tokens, dtype=np.int32)
    for start, length in blocks:
        for position in range(start, start + length):
            if first_position <= position < first_position + tokens:
                ends[position - first_position] = start + length
    return ends


def device_ints(values):
    import torch
    return torch.from_numpy(np.ascontiguousarray(values, dtype=np.int32)).cuda()


def prefill_with(layer, params, q, first_position):
    out = tl.device_empty((q.shape[0], layer.q_heads, layer.d))
    layer.backend.attention_prefill(layer.cache, 0, tl.to_device(q), out, q.shape[0], first_position, params)
    layer.ctx.check()
    return tl.to_host(out)


@pytest.mark.parametrize("q_heads, kv_heads, d, window, prefix", [
    (8, 2, 64, 0, 0),          # full layer, the prompt from position 0
    (8, 2, 64, 96, 200),       # Gemma's local layers: AND(window, OR(causal, block)), after a prefix
    (16, 8, 256, 1024, 300),   # C3's local geometry
    (4, 2, 512, 0, 130),       # Gemma's global geometry
])
def test_blocks_match_the_oracle(q_heads, kv_heads, d, window, prefix):
    import hydra_b200 as hb
    ctx = hb.Context(0)
    rng = np.random.default_rng(d + window)
    tokens = 300
    total = prefix + tokens
    layer = tl.Layer(hb, ctx, q_heads, kv_heads, d, 2048, window=window, sm_scale=1.0 if d >= 256 else None,
                     prefill_chunk=512)
    scale = 1.0 / np.sqrt(d) if d >= 256 else 1.0       # keeps the logits of a scale-1.0 layer moderate
    q = tl.normal_bf16(rng, (total, q_heads, d), scale)
    k = tl.normal_bf16(rng, (total, kv_heads, d))
    v = tl.normal_bf16(rng, (total, kv_heads, d))
    layer.append(k, v, 0)
    # Two images inside the chunk: one short, one longer than a key tile and crossing a tile boundary.
    blocks = [(prefix + 10, 40), (prefix + 100, 170)]
    ends = block_map(prefix, tokens, blocks)
    params = dataclasses.replace(layer.params, block_ends=device_ints(ends))
    have = prefill_with(layer, params, q[prefix:], prefix)
    positions = np.arange(prefix, total)
    want = ho.attention_rows(q[prefix:], positions, k, v, layer.params.sm_scale, window, block_ends=ends)
    tl.record_margin(f"blocks {q_heads}q/{kv_heads}kv d{d} window {window}", have, want)
    assert tl.within_tolerance(have, want, TOL)
    # The mask did something: a block's first token differs from its causal self.
    causal = ho.attention_rows(q[prefix:], positions, k, v, layer.params.sm_scale, window)
    assert tl.max_abs(want[10], causal[10]) > 1e-3
    # Tokens outside the blocks are untouched by it: bit for bit the rows of the call without the
    # buffer, on the tensor-core kernels (head_dim 64, 128, 256) and on the general ones (512, or forced).
    outside = ends == 0
    plain = layer.prefill(q[prefix:], prefix)
    assert np.array_equal(have[outside], plain[outside])
    simt = dataclasses.replace(layer.params, kernel_path=hb.capi.HC_PATH_SIMT)
    general = prefill_with(layer, dataclasses.replace(simt, block_ends=params.block_ends), q[prefix:], prefix)
    assert tl.within_tolerance(general, want, TOL)
    assert np.array_equal(general[outside], prefill_with(layer, simt, q[prefix:], prefix)[outside])
    assert tl.max_abs(have, general) < 2e-2             # the two paths agree as closely as they always do
    layer.close()
    ctx.close()


def test_no_blocks_is_the_call_without_the_buffer():
    """All entries 0: the rows of the call without the buffer, bit for bit, on either path (with the
    buffer every item reaches to the chunk's last key tile and the rows fold the empty partials of the
    tiles they do not see: a no-op)."""
    import hydra_b200 as hb
    ctx = hb.Context(0)
    rng = np.random.default_rng(8)
    q_heads, kv_heads, d, tokens = 16, 2, 128, 260
    layer = tl.Layer(hb, ctx, q_heads, kv_heads, d, 1024)
    q = tl.normal_bf16(rng, (tokens, q_heads, d))
    k = tl.normal_bf16(rng, (tokens, kv_heads, d))
    v = tl.normal_bf16(rng, (tokens, kv_heads, d))
    layer.append(k, v, 0)
    zeros = device_ints(np.zeros(tokens))
    for path in (hb.capi.HC_PATH_TENSOR, hb.capi.HC_PATH_SIMT):
        params = dataclasses.replace(layer.params, kernel_path=path)
        assert np.array_equal(prefill_with(layer, dataclasses.replace(params, block_ends=zeros), q, 0),
                              prefill_with(layer, params, q, 0)), path
    # and the decode step of a token outside any block still equals its prefill row
    plain = layer.prefill(q, 0)
    blocked = prefill_with(layer, dataclasses.replace(layer.params, block_ends=device_ints(block_map(0, tokens, [(40, 100)]))), q, 0)
    for t in (10, 200, tokens - 1):
        assert np.array_equal(layer.decode(q[t:t + 1], [t])[0], blocked[t]), t
    assert np.array_equal(blocked[200], plain[200]) and not np.array_equal(blocked[40], plain[40])
    layer.close()
    ctx.close()


def test_a_block_cut_by_a_chunk_boundary_ends_with_the_chunk():
    """An image of 90 tokens over the boundary between two 64-token chunks, through
    hc_prefill_chunks (append and attention chunk by chunk): in the first chunk its tokens see as
    far as the chunk's last key, the last appended by then; in the second, the whole rest."""
    import hydra_b200 as hb
    ctx = hb.Context(0)
    rng = np.random.default_rng(9)
    q_heads, kv_heads, d, tokens, chunk, window = 8, 2, 64, 192, 64, 80
    layer = tl.Layer(hb, ctx, q_heads, kv_heads, d, 1024, window=window, prefill_chunk=chunk)
    q = tl.normal_bf16(rng, (tokens, q_heads, d))
    k = tl.normal_bf16(rng, (tokens, kv_heads, d))
    v = tl.normal_bf16(rng, (tokens, kv_heads, d))
    ends = block_map(0, tokens, [(30, 90)])
    params = dataclasses.replace(layer.params, block_ends=device_ints(ends))
    out = tl.device_empty((tokens, q_heads, d))
    layer.backend.prefill_chunks(layer.cache, 0, tl.to_device(q), tl.to_device(k), tl.to_device(v), out, tokens, 0,
                                 chunk, params)
    ctx.check()
    have = tl.to_host(out)
    clamped = np.minimum(ends, (np.arange(tokens) // chunk + 1) * chunk) * (ends > 0)
    want = ho.attention_rows(q, np.arange(tokens), k, v, layer.params.sm_scale, window, block_ends=clamped)
    tl.record_margin("blocks over a chunk boundary", have, want)
    assert tl.within_tolerance(have, want, TOL)
    layer.close()
    ctx.close()
