"""Paged KV storage (hc_kv_cache_create_paged): a ragged batch in a pool of 128-row pages.

The same appends, prefill chunks and batched decode steps on a paged cache and on a contiguous one
must agree bit for bit (the kernels differ only in where a key tile's rows are found), and with the
oracle within the parity bound.  The sequences are appended in turns, so their pages interleave in
the pool, and the pool holds exactly the pages the batch needs."""
import numpy as np
import pytest

from oracle import hydra_oracle as ho
from tests import hydra_testlib as tl

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("d, qh, kvh", [(64, 16, 4), (256, 4, 2), (96, 8, 2)])
def test_paged_cache_equals_the_contiguous_one(d, qh, kvh):
    import hydra_b200 as hb
    ctx = hb.Context(0)
    backend = hb.AttentionBackend(ctx)
    rng = np.random.default_rng(5150 + d)
    lengths = [300, 1000, 130, 2047, 700]
    batch = len(lengths)
    context, chunk = 2048, 256
    need = sum((n + 127) // 128 for n in lengths)
    sinks = tl.normal_bf16(rng, (qh,))
    inv = ho.inverse_frequencies(d, 10000.0)
    k = [tl.normal_bf16(rng, (n, kvh, d)) for n in lengths]
    v = [tl.normal_bf16(rng, (n, kvh, d)) for n in lengths]
    q = [tl.normal_bf16(rng, (n, qh, d)) for n in lengths]
    qdec = tl.normal_bf16(rng, (batch, qh, d))
    layers = [dict(q_heads=qh, kv_heads=kvh, head_dim=d, window=0)]
    results = {}
    for mode in ("contiguous", "paged"):
        cache = hb.KVCache(ctx, layers, context, prefill_chunk=chunk, max_seqs=batch,
                           total_pages=need if mode == "paged" else 0)
        rope = hb.RopeTable(ctx, list(inv), context, 1.0)
        sd = tl.to_device(sinks)
        params = hb.AttnParams(q_heads=qh, kv_heads=kvh, head_dim=d, window=0, sm_scale=1 / np.sqrt(d),
                               io_dtype=hb.capi.HC_BF16, sinks=sd, rope=rope)
        assert cache.free_pages == (need if mode == "paged" else -1)
        outs = [tl.device_empty((n, qh, d)) for n in lengths]
        dev = [(tl.to_device(q[s]), tl.to_device(k[s]), tl.to_device(v[s])) for s in range(batch)]
        # chunks of the sequences in turns: their pages interleave in the pool
        start = 0
        while any(start < n for n in lengths):
            for s, n in enumerate(lengths):
                if start >= n:
                    continue
                m = min(chunk, n - start)
                qd, kd, vd = dev[s]
                backend.layer_step(cache, 0, qd[start:], kd[start:], vd[start:], outs[s][start:], m, start, params, seq=s)
            start += chunk
        if mode == "paged":
            assert cache.free_pages == 0
        # one batched decode step over all sequences, re-attending their last positions
        dec = tl.device_empty((batch, qh, d))
        backend.attention(cache, 0, tl.to_device(qdec), dec, [n - 1 for n in lengths], params, seq_ids=list(range(batch)))
        ctx.check()
        rows = cache.read(0, 0, lengths[3], seq=3)
        results[mode] = ([tl.to_host(o) for o in outs], tl.to_host(dec), rows)
        if mode == "paged":
            # out of pages: one more token of the longest sequence needs a page nobody can give
            extra = tl.device_empty((1, kvh, d))
            with pytest.raises(hb.CacheOverflow) as info:
                backend.write_key_value(cache, 0, extra, extra, 1, 256, params, seq=2)     # a third tile for sequence 2
            assert "out of pages" in str(info.value)
            cache.reset(seq=1)
            assert cache.free_pages == (lengths[1] + 127) // 128
            cache.advance(lengths[3], seq=3)
            cache.rewind(256, seq=3)                                                        # keeps two of its sixteen pages
            assert cache.free_pages == (lengths[1] + 127) // 128 + 14
        cache.close()
        rope.close()
    for s in range(batch):
        assert np.array_equal(results["contiguous"][0][s], results["paged"][0][s])
    assert np.array_equal(results["contiguous"][1], results["paged"][1])
    assert np.array_equal(results["contiguous"][2][0], results["paged"][2][0])
    assert np.array_equal(results["contiguous"][2][1], results["paged"][2][1])
    for s in (0, 3):
        want = tl.oracle_path(q[s], k[s], v[s], np.arange(lengths[s]), 1 / np.sqrt(d), 0, sinks=sinks, inv_freq=inv)
        assert tl.within_tolerance(results["paged"][0][s], want)
    ctx.close()
