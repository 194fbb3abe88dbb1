"""The allocation-free decode entry point, hc_attention_decode_static, through the C ABI.

It is meant for callers that cannot allocate device memory when they need attention (a runner that
has committed the whole device to its pools, a plugin inside someone else's process): its split
partials live in a fixed array inside the library.  It runs the same split and merge kernels as
hc_attention_decode on the CUDA-core path, so the two must agree bit for bit; two calls in a row
check that the shared array carries nothing over from one call to the next.
"""
import numpy as np
import pytest

from tests import hydra_testlib as tl

pytestmark = pytest.mark.gpu


def test_static_decode_matches_decode_on_two_calls_in_a_row():
    import hydra_b200 as hb
    ctx = hb.Context(0)
    rng = np.random.default_rng(301)
    qh, kvh, d, batch = 16, 4, 64, 3
    sinks = tl.normal_bf16(rng, (qh,))
    layer = tl.Layer(hb, ctx, qh, kvh, d, 2048, sinks=sinks, max_seqs=batch, kernel_path=hb.capi.HC_PATH_SIMT,
                     prefill_chunk=1024)
    lengths = [1500, 260, 2048]
    for seq, n in enumerate(lengths):
        for start in range(0, n, 1024):
            m = min(1024, n - start)
            layer.append(tl.normal_bf16(rng, (m, kvh, d)), tl.normal_bf16(rng, (m, kvh, d)), start, seq=seq)
    assert layer.backend.static_scratch_limit == 8 << 20
    # first call: all three sequences at their last position; second call: shorter contexts, other queries
    for positions in ([n - 1 for n in lengths], [700, 3, 129]):
        q = tl.normal_bf16(rng, (batch, qh, d))
        want = layer.decode(q, positions, seq_ids=list(range(batch)))
        qd = tl.to_device(q)
        out = tl.device_empty((batch, qh, d))
        layer.backend.attention_static(layer.cache, 0, qd, out, positions, layer.params, seq_ids=list(range(batch)))
        ctx.check()
        assert np.array_equal(tl.to_host(out), want)

    # beyond the fixed array: refused with a message that states the sizes
    big = tl.Layer(hb, ctx, 64, 8, 256, 16384, max_seqs=8, kernel_path=hb.capi.HC_PATH_SIMT)
    qd = tl.device_empty((8, 64, 256))
    with pytest.raises(hb.CacheOverflow) as info:
        big.backend.attention_static(big.cache, 0, qd, qd, [16383] * 8, big.params, seq_ids=list(range(8)))
    assert "fixed scratch holds 8388608" in str(info.value)
    # a query that still needs the prologue is refused
    with pytest.raises(hb.UnsupportedPattern):
        import dataclasses
        f32 = dataclasses.replace(layer.params, io_dtype=hb.capi.HC_F32)
        layer.backend.attention_static(layer.cache, 0, qd, qd, [5], f32)
    big.close()
    layer.close()
    ctx.close()
