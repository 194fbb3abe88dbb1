"""hc_linear: the Q/K/V/O projections on the tensor cores against the oracle's double-precision
matVec, through the C ABI.  Shapes are the configurations' own (GPT-OSS hidden 2880 with its
64 x 64 query and 8 x 64 key/value widths, the output projection back to 2880, a Qwen-like
2x-tall query/gate projection) plus ragged edges: one token, a token count and an output width that
are not multiples of the tile."""
import numpy as np
import pytest

from oracle import hydra_oracle as ho
from tests import hydra_testlib as tl

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("tokens, n_in, n_out, with_bias, out_bf16", [
    (512, 2880, 4096, True, False),      # q_proj of a prefill chunk
    (1, 2880, 512, True, False),         # k_proj of one decode token
    (77, 4096, 2880, True, True),        # o_proj, ragged token count, 2880 = 11.25 column tiles
    (300, 2048, 8192, False, True),      # 2x-tall q_proj with the interleaved gate, no bias
    (130, 64, 40, False, False),         # one K step; output narrower than a tile
])
def test_linear_matches_the_oracle(tokens, n_in, n_out, with_bias, out_bf16):
    import hydra_b200 as hb
    ctx = hb.Context(0)
    backend = hb.AttentionBackend(ctx)
    rng = np.random.default_rng(tokens * 7 + n_out)
    x = tl.normal_bf16(rng, (tokens, n_in))
    w = ho.bf16_round(rng.normal(0.0, 0.02, (n_out, n_in)))
    bias = ho.bf16_round(rng.normal(0.0, 0.5, (n_out,))) if with_bias else None
    want = ho.linear(x, w, bias)
    xd, wd = tl.to_device(x), tl.to_device(w)
    bd = tl.to_device(bias) if with_bias else None
    out = tl.device_empty((tokens, n_out)) if out_bf16 else tl.device_empty((tokens, n_out), dtype="f32")
    dtype = hb.capi.HC_BF16 if out_bf16 else hb.capi.HC_F32
    for _ in range(2):                   # twice: the second call reuses the tensor-memory accumulators
        backend.linear(xd, wd, bd, out, tokens, n_in, n_out, y_dtype=dtype)
    ctx.check()
    got = tl.to_host(out)
    assert got.shape == want.shape
    # fp32 accumulation of bf16 products: far inside the parity bound; bf16 outputs add their rounding
    scale = max(1.0, float(np.abs(want).max()))
    bound = 1e-3 * scale + ((2.0 ** -8) * np.abs(want) if out_bf16 else 0.0)
    assert np.all(np.abs(got - want) <= bound), float(np.abs(got - want).max())
    tl.record_margin(f"linear {tokens}x{n_in}->{n_out}", got, want)
    ctx.close()


def test_linear_rows_do_not_depend_on_the_batch():
    """A token's projection is the same bits whether it is projected alone (the narrow, many-staged
    shape of the kernel, for decode), in a chunk of 100, or inside a prompt of 700 (the wide shape): the
    invariant the attention kernels keep between prefill and decode, kept by the projections too."""
    import hydra_b200 as hb
    ctx = hb.Context(0)
    backend = hb.AttentionBackend(ctx)
    rng = np.random.default_rng(3)
    tokens, n_in, n_out = 700, 2880, 1536
    x = tl.to_device(tl.normal_bf16(rng, (tokens, n_in)))
    w = tl.to_device(ho.bf16_round(rng.normal(0.0, 0.02, (n_out, n_in))))
    b = tl.to_device(ho.bf16_round(rng.normal(0.0, 0.5, (n_out,))))
    whole = tl.device_empty((tokens, n_out), dtype="f32")
    backend.linear(x, w, b, whole, tokens, n_in, n_out)
    chunk = tl.device_empty((100, n_out), dtype="f32")
    backend.linear(x[300:], w, b, chunk, 100, n_in, n_out)
    one = tl.device_empty((1, n_out), dtype="f32")
    backend.linear(x[333:], w, b, one, 1, n_in, n_out)
    ctx.check()
    whole, chunk, one = tl.to_host(whole), tl.to_host(chunk), tl.to_host(one)
    assert np.array_equal(whole[300:400], chunk)
    assert np.array_equal(whole[333], one[0])
    ctx.close()


@pytest.mark.parametrize("tokens", [1, 77, 700])
def test_linear_group_equals_the_separate_calls(tokens):
    """q_proj, k_proj and v_proj of the same x in one launch: the bits of three hc_linear calls, with
    widths that are not whole tiles and one projection without a bias."""
    import hydra_b200 as hb
    ctx = hb.Context(0)
    backend = hb.AttentionBackend(ctx)
    rng = np.random.default_rng(5)
    n_in, widths = 2880, (4096, 512, 520)
    x = tl.to_device(tl.normal_bf16(rng, (tokens, n_in)))
    weights = [tl.to_device(ho.bf16_round(rng.normal(0.0, 0.02, (n, n_in)))) for n in widths]
    biases = [tl.to_device(ho.bf16_round(rng.normal(0.0, 0.5, (n,)))) for n in widths]
    biases[1] = None
    for dtype, code in (("bf16", hb.capi.HC_BF16), ("f32", hb.capi.HC_F32)):
        separate = [tl.device_empty((tokens, n), dtype=dtype) for n in widths]
        grouped = [tl.device_empty((tokens, n), dtype=dtype) for n in widths]
        for w, b, y in zip(weights, biases, separate):
            backend.linear(x, w, b, y, tokens, n_in, w.shape[0], y_dtype=code)
        before = ctx.launch_count
        backend.linear_group(x, weights, biases, grouped, tokens, n_in, y_dtype=code)
        assert ctx.launch_count - before == 1
        ctx.check()
        for a, b in zip(separate, grouped):
            assert np.array_equal(tl.to_host(a), tl.to_host(b))
    with pytest.raises(hb.HydraCudaError):
        backend.linear_group(x, weights * 2, biases * 2, grouped * 2, tokens, n_in)
    ctx.close()


def test_linear_refuses_what_it_cannot_tile():
    import hydra_b200 as hb
    ctx = hb.Context(0)
    backend = hb.AttentionBackend(ctx)
    x = tl.device_empty((4, 72))
    w = tl.device_empty((16, 72))
    y = tl.device_empty((4, 16), dtype="f32")
    with pytest.raises(hb.DimensionMismatch):
        backend.linear(x, w, None, y, 4, 72, 16)
    ctx.close()
