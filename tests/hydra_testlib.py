"""Helpers shared by the GPU parity tests: seeded inputs, the device path, the oracle path.

Inputs follow the reference's test rule (Tests/HydraMetalTests/AttentionKernelTests.swift:107-112):
everything the kernels hold in bf16 is rounded to bf16 *before* the double-precision oracle sees
it, so the comparison measures the kernels and not the quantisation.
"""
from __future__ import annotations

import numpy as np

from oracle import hydra_oracle as ho

MASK64 = (1 << 64) - 1


def deterministic(count: int, seed: int) -> np.ndarray:
    """The generator of the reference's kernel tests (AttentionKernelTests.swift:15-25):
    SplitMix64 mapped to [-1, 1) in steps of 1e-4."""
    out = np.empty(count, dtype=np.float32)
    state = seed & MASK64
    for i in range(count):
        state = (state + 0x9E3779B97F4A7C15) & MASK64
        z = state
        z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & MASK64
        z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & MASK64
        z = z ^ (z >> 31)
        out[i] = np.float32((z % 20000) / 10000.0 - 1.0)
    return out


def deviation(actual, expected) -> float:
    """Worst deviation relative to the vector's magnitude (AttentionKernelTests.swift:29-37)."""
    actual = np.asarray(actual, dtype=np.float64).reshape(-1)
    expected = np.asarray(expected, dtype=np.float64).reshape(-1)
    scale = max(float(np.max(np.abs(expected))), 1e-9)
    return float(np.max(np.abs(actual - expected))) / scale


def max_abs(actual, expected) -> float:
    return float(np.max(np.abs(np.asarray(actual, np.float64) - np.asarray(expected, np.float64))))


def within_tolerance(actual, expected, tol=1e-2, bf16_output=True) -> bool:
    """The parity bound: |error| <= tol on unit-variance outputs.  When the output buffer itself is
    bf16 its own rounding (half a bf16 step, 2^-8 relative at worst) is allowed on top."""
    actual = np.asarray(actual, np.float64)
    expected = np.asarray(expected, np.float64)
    bound = tol + (2.0 ** -8) * np.abs(expected) if bf16_output else tol
    return bool(np.all(np.abs(actual - expected) <= bound))


# Margins the parity tests saw, printed at the end of the session (tests/conftest.py): how far below
# the 1e-2 bound the kernels sit, per configuration.
MARGINS = []


def record_margin(name, actual, expected) -> None:
    MARGINS.append((name, max_abs(actual, expected), deviation(actual, expected), int(np.asarray(actual).size)))


def normal_bf16(rng, shape, scale=1.0) -> np.ndarray:
    return ho.bf16_round((rng.standard_normal(shape) * scale).astype(np.float32))


def to_device(array, dtype="bf16"):
    """numpy float32 (holding bf16-exact values when dtype is bf16) -> CUDA tensor."""
    import torch
    t = torch.from_numpy(np.ascontiguousarray(array, dtype=np.float32)).cuda()
    return t.to(torch.bfloat16) if dtype == "bf16" else t


def to_host(tensor) -> np.ndarray:
    import torch
    return tensor.detach().to(torch.float32).cpu().numpy()


def device_empty(shape, dtype="bf16"):
    import torch
    return torch.empty(shape, device="cuda", dtype=torch.bfloat16 if dtype == "bf16" else torch.float32)


class Layer:
    """One attention layer on the device, driven through the C ABI the way a runner would."""

    def __init__(self, hb, ctx, q_heads, kv_heads, head_dim, context, window=0, sm_scale=None,
                 sinks=None, rope_inv_freq=None, rope_concentration=1.0, q_norm=None, k_norm=None,
                 norm_v=False, norm_eps=1e-6, gate_layout=0, io="bf16", storage=0, prefill_chunk=512,
                 max_seqs=1, kernel_path=0, shard=None):
        self.hb, self.ctx = hb, ctx
        self.q_heads, self.kv_heads, self.d = q_heads, kv_heads, head_dim
        self.io = io
        self.backend = hb.AttentionBackend(ctx)
        self.cache = hb.KVCache(ctx, [dict(q_heads=q_heads, kv_heads=kv_heads, head_dim=head_dim,
                                           window=window, storage=storage)],
                                context, prefill_chunk=prefill_chunk, max_seqs=max_seqs, shard=shard)
        self.rope = None
        if rope_inv_freq is not None:
            self.rope = hb.RopeTable(ctx, list(rope_inv_freq), context, rope_concentration)
        self._sinks = to_device(sinks) if sinks is not None else None
        self._qn = to_device(q_norm) if q_norm is not None else None
        self._kn = to_device(k_norm) if k_norm is not None else None
        self.params = hb.AttnParams(
            q_heads=q_heads, kv_heads=kv_heads, head_dim=head_dim, window=window,
            sm_scale=sm_scale if sm_scale is not None else 1.0 / np.sqrt(head_dim),
            io_dtype=hb.capi.HC_BF16 if io == "bf16" else hb.capi.HC_F32,
            sinks=self._sinks,
            norm_q=1 if q_norm is not None else 0, norm_k=1 if k_norm is not None else 0,
            norm_v=2 if norm_v else 0, q_norm_weight=self._qn, k_norm_weight=self._kn,
            norm_eps=norm_eps, rope=self.rope, gate_layout=gate_layout, kernel_path=kernel_path)

    def append(self, k, v, first_position, seq=0):
        kd, vd = to_device(k, self.io), to_device(v, self.io)
        self.backend.write_key_value(self.cache, 0, kd, vd, k.shape[0], first_position, self.params, seq=seq)

    def prefill(self, q, first_position, gate=None, seq=0):
        tokens = q.shape[0]
        qd = to_device(q, self.io)
        out = device_empty((tokens, self.q_heads, self.d), self.io)
        params = self.params
        if gate is not None:
            gd = to_device(gate, self.io)
            params = self._with_gate(gd)
        self.backend.attention_prefill(self.cache, 0, qd, out, tokens, first_position, params, seq=seq)
        self.ctx.check()
        return to_host(out)

    def step(self, q, k, v, first_position, seq=0):
        """hc_layer_step: append + attention of the same tokens in one call."""
        tokens = q.shape[0]
        qd, kd, vd = to_device(q, self.io), to_device(k, self.io), to_device(v, self.io)
        out = device_empty((tokens, self.q_heads, self.d), self.io)
        self.backend.layer_step(self.cache, 0, qd, kd, vd, out, tokens, first_position, self.params, seq=seq)
        self.ctx.check()
        return to_host(out)

    def decode(self, q, positions, gate=None, seq_ids=None):
        n = q.shape[0]
        qd = to_device(q, self.io)
        out = device_empty((n, self.q_heads, self.d), self.io)
        params = self.params
        if gate is not None:
            gd = to_device(gate, self.io)
            params = self._with_gate(gd)
        self.backend.attention(self.cache, 0, qd, out, list(positions), params, seq_ids=seq_ids)
        self.ctx.check()
        return to_host(out)

    def _with_gate(self, gate_dev):
        import dataclasses
        return dataclasses.replace(self.params, gate_layout=self.hb.capi.HC_GATE_SEPARATE, gate=gate_dev)

    def close(self):
        self.cache.close()
        if self.rope is not None:
            self.rope.close()


def oracle_path(q, k, v, positions, sm_scale, window=0, sinks=None, gate=None, inv_freq=None,
                concentration=1.0, q_norm=None, k_norm=None, norm_v=False, eps=1e-6,
                key_positions=None, cache_rows=None):
    """The reference path in double precision on the same (bf16-rounded) inputs.

    q [n][qh][d] raw queries at `positions`; k, v [history][kvh][d] raw keys/values at positions
    0..history-1.  Norm and rotation are applied as the reference orders them, the results rounded
    to bf16 as the cache holds them, then attention_rows.  `cache_rows=(k, v)` replaces the oracle's
    own prologue on k, v by rows read back from the device cache, so that the comparison measures
    attention alone (the reference's rule: the oracle sees the values the kernel sees).
    """
    history = k.shape[0]
    if key_positions is None:
        key_positions = np.arange(history)
    kc = ks = qc = qs = None
    if inv_freq is not None:
        kc, ks = ho.rope_tables(inv_freq, key_positions, concentration, as_float32=True)
        qc, qs = ho.rope_tables(inv_freq, positions, concentration, as_float32=True)
    if cache_rows is not None:
        kp, vp = cache_rows
    else:
        kp = ho.prepare_heads(k, k_norm, k_norm is not None, eps, kc, ks)
        vp = ho.prepare_heads(v, None, norm_v, eps, None, None)
    qp = ho.prepare_heads(q, q_norm, q_norm is not None, eps, qc, qs)
    return ho.attention_rows(qp, positions, kp, vp, sm_scale, window, sinks=sinks, gate=gate)


def read_cache(cache, layer, tokens, kv_heads, head_dim, seq=0, position=0):
    """The device cache's rows [position, position + tokens) as float32 [tokens][kv_heads][d]."""
    keys, values = cache.read(layer, position, tokens, seq=seq)
    return (ho.bf16_decode(keys).reshape(tokens, kv_heads, head_dim),
            ho.bf16_decode(values).reshape(tokens, kv_heads, head_dim))


def prologue_matches(have, want) -> bool:
    """The cache against the oracle's prologue.  The device normalises and rotates in fp32, the
    oracle in double; after rounding to bf16 the two may land on neighbouring bf16 values for a
    small fraction of the elements, never further apart (one bf16 step is at most 2^-7 relative)."""
    have = np.asarray(have, np.float64).reshape(-1)
    want = np.asarray(want, np.float64).reshape(-1)
    step = np.abs(have - want) / np.maximum(np.abs(want), 1e-3)
    return bool(np.max(step) <= 2.0 ** -6 and np.mean(have != want) < 0.02)
