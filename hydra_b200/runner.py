"""An attention-only stack runner over the C ABI: the part of Hydra's TextModelRunner protocol
(Sources/HydraMetal/TextModelRunner.swift:14-95) that the attention path carries.

The reference's runners embed tokens, run every layer (attention half and mixture-of-experts half)
and project to logits.  Only the attention half is in this library, so the runner here takes and
returns HIDDEN STATES instead of tokens and logits and runs, per layer, the attention block of
ReferenceLayer.decode (Sources/HydraReference/ReferenceLayer.swift:126-187):

    normed = rms_norm(hidden, input_norm)                      hc_rms_norm
    q, k, v = normed W_q^T + b_q, ...                           hc_linear_group (one launch)
    rotate q and k, append k and v, attend (sinks, window)      hc_layer_step
    hidden += attention W_o^T + b_o                             hc_linear with the residual

with the protocol's bookkeeping around it: `position`, `prefill` in chunks of `prefill_chunk_tokens`
(the reference's loop: every chunk through every layer before the next chunk), `forward` for one
token, `verify` (a draft's tokens in one pass, one output per position: the prefill kernels
already return every position), `can_rewind` / `rewind` / `reset` on the KV cache.  Device memory
and streams come from torch; nothing here computes.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Sequence

import numpy as np

from . import capi
from .backend import AttentionBackend, AttnParams, Context, KVCache, RopeTable


@dataclass
class AttentionLayerWeights:
    """One layer's attention weights as Hydra stores them: bf16, projections row-major [out][in]."""
    input_norm: np.ndarray      # [hidden]
    wq: np.ndarray              # [q_heads * head_dim][hidden]
    bq: np.ndarray
    wk: np.ndarray              # [kv_heads * head_dim][hidden]
    bk: np.ndarray
    wv: np.ndarray
    bv: np.ndarray
    wo: np.ndarray              # [hidden][q_heads * head_dim]
    bo: np.ndarray
    sinks: Optional[np.ndarray] = None      # [q_heads]
    window: int = 0                         # 0 = full causal
    inv_freq: Optional[Sequence[float]] = None
    rope_concentration: float = 1.0


class AttentionStackRunner:
    """Hidden states in, hidden states out, through the attention blocks of a stack of layers."""

    prefill_chunk_tokens = 256          # TextModelRunner.prefillChunkTokens

    def __init__(self, ctx: Context, layers: List[AttentionLayerWeights], hidden: int, q_heads: int, kv_heads: int,
                 head_dim: int, context_length: int, eps: float = 1e-5, prefill_chunk_tokens: Optional[int] = None):
        import torch
        self.torch = torch
        self.ctx = ctx
        self.hidden, self.q_heads, self.kv_heads, self.d = hidden, q_heads, kv_heads, head_dim
        self.eps = eps
        if prefill_chunk_tokens is not None:
            self.prefill_chunk_tokens = prefill_chunk_tokens
        self.backend = AttentionBackend(ctx)
        self.kv_cache = KVCache(ctx, [dict(q_heads=q_heads, kv_heads=kv_heads, head_dim=head_dim, window=w.window)
                                      for w in layers], context_length, prefill_chunk=self.prefill_chunk_tokens)
        bf = torch.bfloat16

        def dev(array):
            return torch.from_numpy(np.ascontiguousarray(array, dtype=np.float32)).cuda().to(bf)

        self.weights, self.tables, self.params = [], [], []
        for w in layers:
            t = {name: dev(getattr(w, name)) for name in ("input_norm", "wq", "bq", "wk", "bk", "wv", "bv", "wo", "bo")}
            t["sinks"] = dev(w.sinks) if w.sinks is not None else None
            self.weights.append(t)
            table = RopeTable(ctx, list(w.inv_freq), context_length, w.rope_concentration) if w.inv_freq is not None else None
            self.tables.append(table)
            self.params.append(AttnParams(q_heads=q_heads, kv_heads=kv_heads, head_dim=head_dim, window=w.window,
                                          sm_scale=1.0 / np.sqrt(head_dim), io_dtype=capi.HC_BF16, sinks=t["sinks"],
                                          rope=table))

    # -- TextModelRunner's bookkeeping ------------------------------------------------------------
    @property
    def position(self) -> int:
        return self.kv_cache.length()

    def can_rewind(self, to: int) -> bool:
        return self.kv_cache.can_rewind(to)

    def rewind(self, to: int) -> None:
        self.kv_cache.rewind(to)

    def reset(self) -> None:
        self.kv_cache.reset()

    # -- the passes -------------------------------------------------------------------------------
    def _layers(self, hidden, first_position: int):
        """`hidden` (device, fp32 [n][hidden], updated in place) through every layer's attention block."""
        torch, be = self.torch, self.backend
        n = hidden.shape[0]
        bf = torch.bfloat16
        q_dim, kv_dim = self.q_heads * self.d, self.kv_heads * self.d
        normed = torch.empty((n, self.hidden), device="cuda", dtype=bf)
        q = torch.empty((n, q_dim), device="cuda", dtype=bf)
        k = torch.empty((n, kv_dim), device="cuda", dtype=bf)
        v = torch.empty((n, kv_dim), device="cuda", dtype=bf)
        attended = torch.empty((n, q_dim), device="cuda", dtype=bf)
        for layer, (w, params) in enumerate(zip(self.weights, self.params)):
            be.rms_norm(hidden, w["input_norm"], normed, n, self.hidden, self.eps)
            be.linear_group(normed, [w["wq"], w["wk"], w["wv"]], [w["bq"], w["bk"], w["bv"]], [q, k, v], n, self.hidden,
                            y_dtype=capi.HC_BF16)
            be.layer_step(self.kv_cache, layer, q, k, v, attended, n, first_position, params)
            be.linear(attended, w["wo"], w["bo"], hidden, n, q_dim, self.hidden, y_dtype=capi.HC_F32, residual=hidden)
        return hidden

    def prefill(self, hidden_states: np.ndarray) -> np.ndarray:
        """A prompt's hidden states [tokens][hidden] in chunks, each chunk through every layer before
        the next (ModelRunner.prefill's order); returns the last position's output, as the protocol's
        prefill returns the last position's logits."""
        out = self.verify(hidden_states)
        return out[-1]

    def forward(self, hidden_state: np.ndarray) -> np.ndarray:
        """One token: TextModelRunner.forward(token:)."""
        return self.verify(np.asarray(hidden_state, np.float32).reshape(1, self.hidden))[0]

    def verify(self, hidden_states: np.ndarray) -> np.ndarray:
        """Several tokens in one pass, one output per position (TextModelRunner.verify): the caller
        keeps the accepted prefix by rewinding to it."""
        torch = self.torch
        states = np.asarray(hidden_states, np.float32).reshape(-1, self.hidden)
        outputs = np.empty_like(states)
        for start in range(0, states.shape[0], self.prefill_chunk_tokens):
            chunk = states[start:start + self.prefill_chunk_tokens]
            hidden = torch.from_numpy(np.ascontiguousarray(chunk)).cuda()
            self._layers(hidden, self.position)
            self.ctx.check()
            outputs[start:start + chunk.shape[0]] = hidden.cpu().numpy()
            self.kv_cache.advance(chunk.shape[0])
        return outputs

    def close(self) -> None:
        self.kv_cache.close()
        for table in self.tables:
            if table is not None:
                table.close()
