"""The allocation-free decode entry point, hc_attention_decode_static, through the C ABI.

It is meant for callers that cannot allocate device memory when they need attention (a runner that
has committed the whole device to its pools, a plugin inside someone else's process): its split
partials live in a fixed array inside the library, whose address the context looked up when it was
created.  It runs the same kernels as hc_attention_decode (whatever path that would take for the
layer's head_dim), so the two must agree bit for bit; two calls in a row check that the shared array
carries nothing over from one call to the next, and the free-memory reading around the calls checks
that they took no device memory.
"""
import numpy as np
import pytest

from oracle import hydra_oracle as ho
from tests import hydra_testlib as tl

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("d, path", [(64, "auto"), (128, "auto"), (64, "simt"), (72, "auto")])
def test_static_decode_matches_decode_on_two_calls_in_a_row(d, path):
    import torch
    import hydra_b200 as hb
    ctx = hb.Context(0)
    rng = np.random.default_rng(301)
    qh, kvh, batch = 16, 4, 3
    sinks = tl.normal_bf16(rng, (qh,))
    kernel_path = hb.capi.HC_PATH_SIMT if path == "simt" else hb.capi.HC_PATH_AUTO
    layer = tl.Layer(hb, ctx, qh, kvh, d, 2048, sinks=sinks, max_seqs=batch, kernel_path=kernel_path,
                     prefill_chunk=1024)
    lengths = [1500, 260, 2048]
    history = []
    for seq, n in enumerate(lengths):
        k, v = tl.normal_bf16(rng, (n, kvh, d)), tl.normal_bf16(rng, (n, kvh, d))
        history.append((k, v))
        for start in range(0, n, 1024):
            m = min(1024, n - start)
            layer.append(k[start:start + m], v[start:start + m], start, seq=seq)
    assert layer.backend.static_scratch_limit == 8 << 20
    # first call: all three sequences at their last position; second call: shorter contexts, other queries
    for positions in ([n - 1 for n in lengths], [700, 3, 129]):
        q = tl.normal_bf16(rng, (batch, qh, d))
        want = layer.decode(q, positions, seq_ids=list(range(batch)))      # hc_attention_decode, same path
        qd = tl.to_device(q)
        out = tl.device_empty((batch, qh, d))
        torch.cuda.synchronize()
        free_before, _ = torch.cuda.mem_get_info()
        layer.backend.attention_static(layer.cache, 0, qd, out, positions, layer.params, seq_ids=list(range(batch)))
        ctx.check()
        free_after, _ = torch.cuda.mem_get_info()
        assert free_after == free_before, "the call took device memory"
        got = tl.to_host(out)
        assert np.array_equal(got, want)
        for seq, pos in enumerate(positions):
            k, v = history[seq]
            ref = ho.attention_rows(q[seq:seq + 1], [pos], k[:pos + 1], v[:pos + 1], 1 / np.sqrt(d), 0, sinks=sinks)
            assert tl.within_tolerance(got[seq], ref[0])
    layer.close()
    ctx.close()


def test_static_decode_refusals():
    import dataclasses
    import hydra_b200 as hb
    ctx = hb.Context(0)
    # beyond the fixed array: refused with a message that states the sizes.  Two long sequences are few
    # enough that the library cuts them tile by tile: 128 rows x 128 tile partials of 258 floats.
    big = tl.Layer(hb, ctx, 64, 8, 256, 16384, max_seqs=2)
    qd = tl.device_empty((2, 64, 256))
    with pytest.raises(hb.CacheOverflow) as info:
        big.backend.attention_static(big.cache, 0, qd, qd, [16383] * 2, big.params, seq_ids=[0, 1])
    assert "fixed scratch holds 8388608" in str(info.value)
    # a query that still needs the prologue is refused
    with pytest.raises(hb.UnsupportedPattern):
        f32 = dataclasses.replace(big.params, io_dtype=hb.capi.HC_F32)
        big.backend.attention_static(big.cache, 0, qd, qd, [5], f32)
    big.close()
    ctx.close()
