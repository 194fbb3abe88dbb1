"""The five benchmark configurations as synthetic, seeded inputs, and a runner that drives them
through the backend the way a layer runner would (append, then attend).

Inputs are generated once, outside any timed region: weights N(0, 0.02) and hidden states N(0, 1)
from `numpy.random.default_rng(seed)`, rounded to bf16; q/k/v are the projections of the hidden
states (fp32 accumulate) rounded to bf16.  torch is used here only as device memory and for those
one-off projections; every operation of the measured path goes through libhydra_cuda.so.

  C1  GPT-OSS-20B layer: 64q/8kv, d 64, window 128, sinks, theta 150000; 512-token prompt in
      128-token chunks + 64 decode steps
  C2  same shape, full causal: 4096-token prompt in 512-token chunks, decode at context 4096
  C3  Gemma-style stack of 6 layers (5 x window 1024, 1 global): 16q/8kv, d 256, q/k RMSNorm,
      weightless v norm, scale 1.0, theta 1e4 / 1e6; 8192-token prefill in 512-chunks + 128 decode
  C4  Qwen-style gated layer: 16q/2kv, d 256, partial rotary (32 of 128 pairs), theta 1e7, q/k
      RMSNorm, sigmoid gate; decode at context 32768
  C5  GPT-OSS-120B-shaped batched decode: 64 sequences, lengths U[1024, 16384] (seed 7), 64q/8kv,
      d 64, one window-128 layer and one full layer, sinks
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import List, Optional

import numpy as np

from . import capi
from .backend import AttentionBackend, AttnParams, Context, KVCache, RopeTable, inverse_frequencies


def bf16_round_np(x: np.ndarray) -> np.ndarray:
    """float32 -> nearest bf16 (ties to even) -> float32, in numpy."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    bits = x.view(np.uint32)
    rounding = np.uint32(0x7FFF) + ((bits >> np.uint32(16)) & np.uint32(1))
    out = ((bits + rounding) & np.uint32(0xFFFF0000)).view(np.float32)
    return out.reshape(x.shape)


@dataclass
class LayerSpec:
    window: int = 0
    theta: float = 10000.0
    rotating_pairs: Optional[int] = None


@dataclass
class Config:
    name: str
    q_heads: int
    kv_heads: int
    head_dim: int
    hidden: int
    layers: List[LayerSpec]
    seed: int
    prompt: int = 0              # prefill tokens
    chunk: int = 512
    decode_steps: int = 0
    sm_scale: Optional[float] = None
    sinks: bool = False
    qk_norm: bool = False
    v_norm: bool = False
    gate: bool = False
    batch: int = 1
    context: int = 0             # cache rows per sequence
    prefilled: int = 0           # C4 / C5: history filled directly with N(0, 1)
    ragged: bool = False

    @property
    def scale(self) -> float:
        return self.sm_scale if self.sm_scale is not None else 1.0 / math.sqrt(self.head_dim)


def config(name: str, kv_heads: Optional[int] = None) -> Config:
    """`kv_heads` overrides the head count for a KV-head shard (query heads scale with it)."""
    if name == "C1":
        c = Config("C1", 64, 8, 64, 2880, [LayerSpec(128, 150000.0)], seed=0, prompt=512, chunk=128,
                   decode_steps=64, sinks=True, context=576)
    elif name == "C2":
        c = Config("C2", 64, 8, 64, 2880, [LayerSpec(0, 150000.0)], seed=0, prompt=4096, chunk=512,
                   decode_steps=1, sinks=True, context=4097)
    elif name == "C3":
        layers = [LayerSpec(1024, 1e4)] * 5 + [LayerSpec(0, 1e6)]
        c = Config("C3", 16, 8, 256, 2816, layers, seed=1, prompt=8192, chunk=512, decode_steps=128,
                   sm_scale=1.0, qk_norm=True, v_norm=True, context=8320)
    elif name == "C4":
        c = Config("C4", 16, 2, 256, 2048, [LayerSpec(0, 1e7, 32)], seed=4, decode_steps=1,
                   qk_norm=True, gate=True, context=32768, prefilled=32767)
    elif name == "C5":
        c = Config("C5", 64, 8, 64, 2880, [LayerSpec(128, 150000.0), LayerSpec(0, 150000.0)], seed=7,
                   decode_steps=1, sinks=True, batch=64, context=16384, ragged=True)
    else:
        raise ValueError(name)
    if kv_heads is not None and kv_heads != c.kv_heads:
        group = c.q_heads // c.kv_heads
        c.kv_heads = kv_heads
        c.q_heads = kv_heads * group
    return c


def ragged_lengths(cfg: Config) -> np.ndarray:
    rng = np.random.default_rng(cfg.seed)
    return rng.integers(1024, 16385, size=cfg.batch)


def prefill_flops(cfg: Config) -> float:
    """4 * d flops per visible (query, key) pair per query head, causal- and window-exact."""
    total = 0.0
    for layer in cfg.layers:
        p = np.arange(cfg.prompt, dtype=np.float64)
        visible = p + 1 if layer.window == 0 else np.minimum(p + 1, layer.window)
        total += float(visible.sum()) * cfg.q_heads * 4 * cfg.head_dim
    return total


def decode_bytes(cfg: Config, position: int, layer: LayerSpec) -> int:
    """Each visible K and V element once, bf16."""
    visible = position + 1 if layer.window == 0 else min(position + 1, layer.window)
    return visible * cfg.kv_heads * cfg.head_dim * 2 * 2


class Inputs:
    """Host copies (float32 holding bf16 values) of one configuration's tensors."""

    def __init__(self, cfg: Config, full_heads: Optional[Config] = None, head_offset: int = 0,
                 device: Optional[str] = None):
        import torch
        self.cfg = cfg
        src = full_heads or cfg                       # a head shard draws the full model's tensors
        rng = np.random.default_rng(src.seed)
        d, H = src.head_dim, src.hidden
        dev = device or ("cuda" if torch.cuda.is_available() else "cpu")
        tokens = src.prompt + (src.decode_steps if not src.ragged and not src.prefilled else 0)
        group = src.q_heads // src.kv_heads
        q_slice = slice(head_offset * group * d, (head_offset + cfg.kv_heads) * group * d)
        kv_slice = slice(head_offset * d, (head_offset + cfg.kv_heads) * d)
        self.layers = []

        def project(w, x):
            wt = torch.from_numpy(w).to(dev)
            xt = torch.from_numpy(x).to(dev)
            return bf16_round_np((xt @ wt.T).float().cpu().numpy())

        for _spec in src.layers:
            entry = {}
            q_rows = src.q_heads * d * (2 if src.gate else 1)
            wq = bf16_round_np((rng.standard_normal((q_rows, H)) * 0.02).astype(np.float32))
            wk = bf16_round_np((rng.standard_normal((src.kv_heads * d, H)) * 0.02).astype(np.float32))
            wv = bf16_round_np((rng.standard_normal((src.kv_heads * d, H)) * 0.02).astype(np.float32))
            entry["sinks"] = bf16_round_np(rng.standard_normal(src.q_heads).astype(np.float32))[
                head_offset * group:(head_offset + cfg.kv_heads) * group] if src.sinks else None
            if src.qk_norm:
                entry["q_norm"] = bf16_round_np((1 + 0.1 * rng.standard_normal(d)).astype(np.float32))
                entry["k_norm"] = bf16_round_np((1 + 0.1 * rng.standard_normal(d)).astype(np.float32))
            if src.ragged or src.prefilled:
                n_q = src.batch
                hidden = bf16_round_np(rng.standard_normal((n_q, H)).astype(np.float32))
            else:
                hidden = bf16_round_np(rng.standard_normal((tokens, H)).astype(np.float32))
            q_all = project(wq, hidden)
            if src.gate:
                # q_proj emits [heads][2d]: the head's query, then its gate.
                q_all = q_all.reshape(-1, src.q_heads, 2 * d)[:, head_offset * group:(head_offset + cfg.kv_heads) * group]
                entry["q"] = np.ascontiguousarray(q_all)                       # interleaved
            else:
                entry["q"] = np.ascontiguousarray(q_all[:, q_slice]).reshape(-1, cfg.q_heads, d)
            # With a pre-filled history (C4, C5) these are the new token's own k, v; the history is drawn
            # directly (see `history`).
            entry["k"] = np.ascontiguousarray(project(wk, hidden)[:, kv_slice]).reshape(-1, cfg.kv_heads, d)
            entry["v"] = np.ascontiguousarray(project(wv, hidden)[:, kv_slice]).reshape(-1, cfg.kv_heads, d)
            self.layers.append(entry)
        self.rng = rng
        self.lengths = ragged_lengths(src) if src.ragged else None

    def history(self, seq: int, length: int):
        """N(0, 1) bf16 history rows [length][kv_heads][d] for a pre-filled cache (C4, C5); drawn
        per (sequence) from its own generator so that any subset can be regenerated."""
        rng = np.random.default_rng([self.cfg.seed, 1000 + seq])
        k = bf16_round_np(rng.standard_normal((length, self.cfg.kv_heads, self.cfg.head_dim)).astype(np.float32))
        v = bf16_round_np(rng.standard_normal((length, self.cfg.kv_heads, self.cfg.head_dim)).astype(np.float32))
        return k, v


class PathRunner:
    """Owns the cache, tables and device tensors of one configuration and runs its passes."""

    def __init__(self, ctx: Context, cfg: Config, inputs: Inputs, kernel_path: int = capi.HC_PATH_AUTO,
                 shard: Optional[tuple] = None, storage: int = capi.HC_STORAGE_AUTO):
        import torch
        self.torch = torch
        self.ctx, self.cfg, self.inputs = ctx, cfg, inputs
        self.backend = AttentionBackend(ctx)
        d = cfg.head_dim
        descs = [dict(q_heads=cfg.q_heads, kv_heads=cfg.kv_heads, head_dim=d, window=l.window, storage=storage)
                 for l in cfg.layers]
        self.cache = KVCache(ctx, descs, cfg.context, prefill_chunk=max(cfg.chunk, 1), max_seqs=cfg.batch, shard=shard)
        self.tables, self.params, self.dev = [], [], []
        bf = torch.bfloat16
        for spec, entry in zip(cfg.layers, inputs.layers):
            table = RopeTable(ctx, inverse_frequencies(d, spec.theta, spec.rotating_pairs), cfg.context)
            self.tables.append(table)
            t = {name: torch.from_numpy(entry[name]).cuda().to(bf) for name in ("q", "k", "v")}
            for name in ("sinks", "q_norm", "k_norm"):
                t[name] = torch.from_numpy(entry[name]).cuda().to(bf) if entry.get(name) is not None else None
            t["out"] = torch.zeros((t["q"].shape[0], cfg.q_heads, d), device="cuda", dtype=bf)
            self.dev.append(t)
            self.params.append(AttnParams(
                q_heads=cfg.q_heads, kv_heads=cfg.kv_heads, head_dim=d, window=spec.window,
                sm_scale=cfg.scale, io_dtype=capi.HC_BF16, sinks=t["sinks"],
                norm_q=1 if cfg.qk_norm else 0, norm_k=1 if cfg.qk_norm else 0,
                norm_v=2 if cfg.v_norm else 0, q_norm_weight=t["q_norm"], k_norm_weight=t["k_norm"],
                rope=table, gate_layout=capi.HC_GATE_INTERLEAVED if cfg.gate else capi.HC_GATE_NONE,
                kernel_path=kernel_path))

    # -- sizes ------------------------------------------------------------------------------------
    def q_row_elems(self) -> int:
        return self.cfg.q_heads * self.cfg.head_dim * (2 if self.cfg.gate else 1)

    # -- pre-filled histories (C4, C5) --------------------------------------------------------------
    def fill_history(self, lengths, no_prologue_params=None):
        """Writes N(0, 1) rows 0 .. length-1 of every sequence straight into the cache (a plain
        cast-and-store append: the rows stand for keys that were normalised and rotated earlier)."""
        torch = self.torch
        for seq, length in enumerate(lengths):
            k, v = self.inputs.history(seq, int(length))
            kd = torch.from_numpy(k).cuda().to(torch.bfloat16)
            vd = torch.from_numpy(v).cuda().to(torch.bfloat16)
            for layer, spec in enumerate(self.cfg.layers):
                plain = AttnParams(q_heads=self.cfg.q_heads, kv_heads=self.cfg.kv_heads,
                                   head_dim=self.cfg.head_dim, window=spec.window, sm_scale=self.cfg.scale,
                                   io_dtype=capi.HC_BF16)
                info = self.cache.layer(layer)
                # A ring only keeps its last rows; writing the tail is enough.
                first = 0 if info.ring_size == 0 else max(0, int(length) - (info.ring_size - spec.window))
                for start in range(first, int(length), 512):
                    n = min(512, int(length) - start)
                    self.backend.write_key_value(self.cache, layer, kd[start:], vd[start:], n, start, plain, seq=seq)
            torch.cuda.synchronize()

    # -- the passes ---------------------------------------------------------------------------------
    def prefill_pass(self, stream=None, layers=None, fused=False):
        """Append + attend for every chunk of the prompt, every layer: two calls per chunk
        (hc_kv_append, hc_attention_prefill) or, with `fused`, one (hc_layer_step)."""
        cfg = self.cfg
        for layer in (range(len(cfg.layers)) if layers is None else layers):
            t, params = self.dev[layer], self.params[layer]
            for start in range(0, cfg.prompt, cfg.chunk):
                n = min(cfg.chunk, cfg.prompt - start)
                if fused:
                    self.backend.layer_step(self.cache, layer, t["q"][start:], t["k"][start:], t["v"][start:],
                                            t["out"][start:], n, start, params, stream=stream)
                else:
                    self.backend.write_key_value(self.cache, layer, t["k"][start:], t["v"][start:], n, start, params, stream=stream)
                    self.backend.attention_prefill(self.cache, layer, t["q"][start:], t["out"][start:], n, start, params, stream=stream)

    def decode_step(self, row: int, position: int, stream=None, layers=None, append=True):
        """One token (batch 1): its K/V appended at `position`, then attention, every layer."""
        for layer in (range(len(self.cfg.layers)) if layers is None else layers):
            t, params = self.dev[layer], self.params[layer]
            if append:
                self.backend.write_key_value(self.cache, layer, t["k"][row:], t["v"][row:], 1, position, params, stream=stream)
            self.backend.attention(self.cache, layer, t["q"][row:], t["out"][row:], [position], params, stream=stream)

    def decode_batch(self, positions, stream=None, layers=None, append=True):
        """One token for each sequence of the batch (C5)."""
        seqs = list(range(len(positions)))
        for layer in (range(len(self.cfg.layers)) if layers is None else layers):
            t, params = self.dev[layer], self.params[layer]
            if append:
                self.backend.write_key_value_batch(self.cache, layer, t["k"], t["v"], seqs, list(positions), params, stream=stream)
            self.backend.attention(self.cache, layer, t["q"], t["out"], list(positions), params, seq_ids=seqs, stream=stream)

    def output(self, layer: int = 0) -> np.ndarray:
        return self.dev[layer]["out"].float().cpu().numpy()

    def close(self):
        self.cache.close()
        for table in self.tables:
            table.close()
