"""The attention half of a GPT-OSS layer end to end on the device, through the C ABI: input RMSNorm
(hc_rms_norm) -> q/k/v projections (hc_linear) -> RoPE, KV append and attention with sinks and a
sliding window (hc_layer_step) -> output projection with the residual add (hc_linear), against the
same block composed from the oracle's operators in double precision, the way ReferenceLayer.decode
orders them (Sources/HydraReference/ReferenceLayer.swift:126-187).  C1's shape: hidden 2880, 64
query heads and 8 KV heads of 64, window 128, a 256-token prompt in 128-token chunks, then decode
steps.  The oracle rounds to bf16 where the device's buffers are bf16 (the normed activations, q, k,
v and the attention output), so that the comparison measures the kernels' arithmetic and not the
choice of activation type."""
import numpy as np
import pytest

from oracle import hydra_oracle as ho
from tests import hydra_testlib as tl

pytestmark = pytest.mark.gpu


def test_attention_block_matches_the_composed_oracle():
    import hydra_b200 as hb
    ctx = hb.Context(0)
    rng = np.random.default_rng(2025)
    hidden_size, qh, kvh, d, window = 2880, 64, 8, 64, 128
    prompt, chunk, decode_steps = 256, 128, 3
    total = prompt + decode_steps
    theta = 150000.0
    inv_freq = ho.inverse_frequencies(d, theta)
    sinks = tl.normal_bf16(rng, (qh,))
    norm_w = ho.bf16_round(1.0 + 0.1 * rng.standard_normal(hidden_size))
    wq = ho.bf16_round(rng.normal(0, 0.02, (qh * d, hidden_size)))
    wk = ho.bf16_round(rng.normal(0, 0.02, (kvh * d, hidden_size)))
    wv = ho.bf16_round(rng.normal(0, 0.02, (kvh * d, hidden_size)))
    wo = ho.bf16_round(rng.normal(0, 0.02, (hidden_size, qh * d)))
    bq, bk, bv = (ho.bf16_round(rng.normal(0, 0.1, (n,))) for n in (qh * d, kvh * d, kvh * d))
    bo = ho.bf16_round(rng.normal(0, 0.1, (hidden_size,)))
    hidden = rng.standard_normal((total, hidden_size)).astype(np.float32)
    eps = 1e-5

    # ---- the oracle's block -------------------------------------------------------------------
    normed = ho.bf16_round(np.stack([ho.rms_norm(row, norm_w, eps, use_sqrt=True) for row in hidden]))
    q = ho.bf16_round(ho.linear(normed, wq, bq)).reshape(total, qh, d)
    k = ho.bf16_round(ho.linear(normed, wk, bk)).reshape(total, kvh, d)
    v = ho.bf16_round(ho.linear(normed, wv, bv)).reshape(total, kvh, d)
    attn = tl.oracle_path(q, k, v, np.arange(total), 1 / np.sqrt(d), window=window, sinks=sinks, inv_freq=inv_freq)
    attn = ho.bf16_round(attn).reshape(total, qh * d)
    want = hidden.astype(np.float64) + ho.linear(attn, wo, bo)

    # ---- the device's block -------------------------------------------------------------------
    layer = tl.Layer(hb, ctx, qh, kvh, d, 512, window=window, sinks=sinks, rope_inv_freq=inv_freq, prefill_chunk=chunk)
    backend = layer.backend
    dev = {name: tl.to_device(a) for name, a in dict(norm=norm_w, wq=wq, wk=wk, wv=wv, wo=wo, bq=bq, bk=bk, bv=bv, bo=bo).items()}
    got = np.zeros((total, hidden_size), np.float32)
    spans = [(s, min(chunk, prompt - s)) for s in range(0, prompt, chunk)] + [(prompt + i, 1) for i in range(decode_steps)]
    for start, n in spans:
        h = tl.to_device(hidden[start:start + n], "f32")
        x = tl.device_empty((n, hidden_size))
        backend.rms_norm(h, dev["norm"], x, n, hidden_size, eps)
        qd, kd, vd = tl.device_empty((n, qh * d)), tl.device_empty((n, kvh * d)), tl.device_empty((n, kvh * d))
        backend.linear(x, dev["wq"], dev["bq"], qd, n, hidden_size, qh * d, y_dtype=hb.capi.HC_BF16)
        backend.linear(x, dev["wk"], dev["bk"], kd, n, hidden_size, kvh * d, y_dtype=hb.capi.HC_BF16)
        backend.linear(x, dev["wv"], dev["bv"], vd, n, hidden_size, kvh * d, y_dtype=hb.capi.HC_BF16)
        out = tl.device_empty((n, qh * d))
        backend.layer_step(layer.cache, 0, qd, kd, vd, out, n, start, layer.params)
        backend.linear(out, dev["wo"], dev["bo"], h, n, qh * d, hidden_size, y_dtype=hb.capi.HC_F32, residual=h)
        ctx.check()
        got[start:start + n] = tl.to_host(h)
    assert tl.within_tolerance(got, want, bf16_output=False)
    tl.record_margin("GPT-OSS attention block, 256-token prompt + 3 decode steps", got, want)
    layer.close()
    ctx.close()


@pytest.mark.parametrize("tokens, width", [(1, 2880), (37, 2880), (5, 4096), (3, 2816), (4, 4100), (6, 130), (2, 8192)])
@pytest.mark.parametrize("x_f32, out_bf16, scaled", [(True, True, True), (True, False, False), (False, True, True)])
def test_rms_norm_rows_match_the_oracle(tokens, width, x_f32, out_bf16, scaled):
    """hc_rms_norm (the layer's input norm, ReferenceOps.rmsNorm): rows read four elements per load
    (widths that are multiples of 4 up to 4096) and element by element (the others), fp32 and bf16
    on either side, with and without the scale."""
    import hydra_b200 as hb
    ctx = hb.Context(0)
    backend = hb.AttentionBackend(ctx)
    rng = np.random.default_rng(width + tokens)
    x = rng.standard_normal((tokens, width)).astype(np.float32) * 3.0
    if not x_f32:
        x = ho.bf16_round(x)
    scale = ho.bf16_round(1.0 + 0.2 * rng.standard_normal(width).astype(np.float32)) if scaled else None
    xd = tl.to_device(x, "f32" if x_f32 else "bf16")
    sd = tl.to_device(scale) if scaled else None
    out = tl.device_empty((tokens, width), "bf16" if out_bf16 else "f32")
    backend.rms_norm(xd, sd, out, tokens, width, 1e-5, x_dtype=hb.capi.HC_F32 if x_f32 else hb.capi.HC_BF16,
                     y_dtype=hb.capi.HC_BF16 if out_bf16 else hb.capi.HC_F32)
    ctx.check()
    want = np.stack([ho.rms_norm(row, scale, 1e-5, use_sqrt=True) for row in x])
    have = tl.to_host(out)
    assert tl.within_tolerance(have, want, 1e-4, bf16_output=out_bf16)
    # a row's result does not depend on the rows beside it
    one = tl.device_empty((1, width), "bf16" if out_bf16 else "f32")
    backend.rms_norm(xd[tokens - 1:], sd, one, 1, width, 1e-5, x_dtype=hb.capi.HC_F32 if x_f32 else hb.capi.HC_BF16,
                     y_dtype=hb.capi.HC_BF16 if out_bf16 else hb.capi.HC_F32)
    ctx.check()
    assert np.array_equal(tl.to_host(one)[0], have[tokens - 1])
    ctx.close()
