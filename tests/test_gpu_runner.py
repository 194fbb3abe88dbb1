"""AttentionStackRunner: two GPT-OSS-shaped layers (one with a 128-token window, one full), hidden
states through prefill in chunks, single-token forwards and a speculative verify + rewind, against
the attention blocks composed from the oracle's operators (ReferenceLayer.decode's order,
Sources/HydraReference/ReferenceLayer.swift:126-187).  The runner's invariant is the path's: the same
positions give the same bits whether they arrive in a prefill chunk, a verify pass or one by one."""
import numpy as np
import pytest

from oracle import hydra_oracle as ho
from tests import hydra_testlib as tl

pytestmark = pytest.mark.gpu


def oracle_stack(hidden, layers, qh, kvh, d, eps):
    """All positions at once: layer by layer, rounding to bf16 where the device's buffers are bf16."""
    total = hidden.shape[0]
    state = hidden.astype(np.float64)
    for w in layers:
        normed = ho.bf16_round(np.stack([ho.rms_norm(row, w.input_norm, eps, use_sqrt=True) for row in state]))
        q = ho.bf16_round(ho.linear(normed, w.wq, w.bq)).reshape(total, qh, d)
        k = ho.bf16_round(ho.linear(normed, w.wk, w.bk)).reshape(total, kvh, d)
        v = ho.bf16_round(ho.linear(normed, w.wv, w.bv)).reshape(total, kvh, d)
        attended = tl.oracle_path(q, k, v, np.arange(total), 1 / np.sqrt(d), window=w.window, sinks=w.sinks,
                                  inv_freq=np.asarray(w.inv_freq))
        attended = ho.bf16_round(attended).reshape(total, qh * d)
        # the device keeps the residual stream in fp32
        state = (state + ho.linear(attended, w.wo, w.bo)).astype(np.float32).astype(np.float64)
    return state


def test_runner_prefill_forward_verify_and_rewind():
    import hydra_b200 as hb
    from hydra_b200.runner import AttentionLayerWeights, AttentionStackRunner
    ctx = hb.Context(0)
    rng = np.random.default_rng(77)
    hidden_size, qh, kvh, d = 2880, 64, 8, 64
    inv = ho.inverse_frequencies(d, 150000.0)
    eps = 1e-5

    def layer(window):
        return AttentionLayerWeights(
            input_norm=ho.bf16_round(1.0 + 0.1 * rng.standard_normal(hidden_size)),
            wq=ho.bf16_round(rng.normal(0, 0.02, (qh * d, hidden_size))), bq=ho.bf16_round(rng.normal(0, 0.1, qh * d)),
            wk=ho.bf16_round(rng.normal(0, 0.02, (kvh * d, hidden_size))), bk=ho.bf16_round(rng.normal(0, 0.1, kvh * d)),
            wv=ho.bf16_round(rng.normal(0, 0.02, (kvh * d, hidden_size))), bv=ho.bf16_round(rng.normal(0, 0.1, kvh * d)),
            wo=ho.bf16_round(rng.normal(0, 0.02, (hidden_size, qh * d))), bo=ho.bf16_round(rng.normal(0, 0.1, hidden_size)),
            sinks=tl.normal_bf16(rng, (qh,)), window=window, inv_freq=inv)

    layers = [layer(128), layer(0)]
    prompt, single, draft = 300, 2, 5
    total = prompt + single + draft
    states = rng.standard_normal((total, hidden_size)).astype(np.float32)
    want = oracle_stack(states, layers, qh, kvh, d, eps)

    runner = AttentionStackRunner(ctx, layers, hidden_size, qh, kvh, d, context_length=1024, eps=eps,
                                  prefill_chunk_tokens=128)
    last = runner.prefill(states[:prompt])
    assert runner.position == prompt
    assert tl.within_tolerance(last, want[prompt - 1], bf16_output=False)
    got_single = np.stack([runner.forward(states[prompt + i]) for i in range(single)])
    assert tl.within_tolerance(got_single, want[prompt:prompt + single], bf16_output=False)
    # a draft of five tokens verified in one pass, three accepted: rewind, then the same three one by one
    base = runner.position
    verified = runner.verify(states[base:base + draft])
    assert tl.within_tolerance(verified, want[base:base + draft], bf16_output=False)
    assert runner.can_rewind(base + 3)
    runner.rewind(base + 3)
    assert runner.position == base + 3
    runner.rewind(base)
    again = np.stack([runner.forward(states[base + i]) for i in range(3)])
    assert np.array_equal(again, verified[:3])                     # verify pass == token by token, bit for bit
    tl.record_margin("two-layer attention stack: prefill 300, forward 2, verify 5", np.concatenate([got_single, verified]),
                     want[prompt:])
    runner.close()
    ctx.close()
