"""ctypes front end of the CPU oracle (hydra_oracle.cpp).

TEST INFRASTRUCTURE ONLY: imported by tests/, by the smoke check and by the benchmark's CPU-baseline
leg.  The product package never imports it.

The oracle restates `Sources/HydraReference` (Swift, double precision) in C++; each wrapper below
names the reference function it stands for.  Arrays are numpy; every function returns new arrays.
"""
from __future__ import annotations

import ctypes
import os
import subprocess
from typing import Optional

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SRC = os.path.join(_HERE, "hydra_oracle.cpp")
_LIB = os.path.join(_HERE, "_build", "libhydra_oracle.so")

_lib = None


def build(force: bool = False) -> str:
    """Compiles the oracle with g++ if the shared object is missing or older than its source."""
    if (not force and os.path.exists(_LIB)
            and (not os.path.exists(_SRC) or os.path.getmtime(_LIB) >= os.path.getmtime(_SRC))):
        return _LIB
    os.makedirs(os.path.dirname(_LIB), exist_ok=True)
    subprocess.check_call(["g++", "-O2", "-std=c++17", "-shared", "-fPIC", "-pthread", _SRC,
                           "-o", _LIB])
    return _LIB


def lib():
    global _lib
    if _lib is None:
        _lib = ctypes.CDLL(build())
        _lib.ho_hardware_threads.restype = ctypes.c_int
        _lib.ho_yarn_inverse_frequencies.restype = ctypes.c_int
    return _lib


def _p(a, ctype):
    return a.ctypes.data_as(ctypes.POINTER(ctype)) if a is not None else None


_D = ctypes.c_double
_F = ctypes.c_float


def _f64(a):
    return np.ascontiguousarray(a, dtype=np.float64)


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def hardware_threads() -> int:
    return int(lib().ho_hardware_threads())


# ---- bf16 (Sources/HydraFormat/BF16.swift:20-32) --------------------------------------------

def bf16_round(x) -> np.ndarray:
    """float32 -> nearest bf16 (ties to even) -> float32."""
    x = _f32(x)
    out = np.empty_like(x)
    lib().ho_bf16_round(_p(x, _F), _p(out, _F), ctypes.c_size_t(x.size))
    return out


def bf16_encode(x) -> np.ndarray:
    x = _f32(x)
    out = np.empty(x.shape, dtype=np.uint16)
    lib().ho_bf16_encode(_p(x, _F), _p(out, ctypes.c_uint16), ctypes.c_size_t(x.size))
    return out


def bf16_decode(bits) -> np.ndarray:
    bits = np.ascontiguousarray(bits, dtype=np.uint16)
    out = np.empty(bits.shape, dtype=np.float32)
    lib().ho_bf16_decode(_p(bits, ctypes.c_uint16), _p(out, _F), ctypes.c_size_t(bits.size))
    return out


# ---- operators --------------------------------------------------------------------------------

def rms_norm(x, weight=None, eps=1e-6, use_sqrt=False) -> np.ndarray:
    """Gemma4ReferenceOps.rmsNorm (pow form) or ReferenceOps.rmsNorm (`use_sqrt`)."""
    x = _f64(x)
    w = _f64(weight) if weight is not None else None
    out = np.empty_like(x)
    lib().ho_rms_norm(_p(x, _D), _p(w, _D), ctypes.c_int(x.size), _D(eps),
                      ctypes.c_int(1 if use_sqrt else 0), _p(out, _D))
    return out


def yarn_inverse_frequencies(head_dim, base, initial_context=4096, scaling=1.0, ntk_alpha=1.0,
                             ntk_beta=32.0):
    """RoPETables.init: (inverse frequencies, concentration)."""
    inv = np.empty(head_dim // 2, dtype=np.float64)
    conc = _D(0.0)
    rc = lib().ho_yarn_inverse_frequencies(ctypes.c_int(head_dim), _D(base),
                                           ctypes.c_int(initial_context), _D(scaling),
                                           _D(ntk_alpha), _D(ntk_beta), _p(inv, _D),
                                           ctypes.byref(conc))
    if rc != 0:
        raise ValueError("inconsistent YaRN bounds")
    return inv, conc.value


def inverse_frequencies(head_dim, theta, rotating_pairs=None) -> np.ndarray:
    """Gemma4ReferenceOps.inverseFrequencies: zero frequency beyond `rotating_pairs`."""
    if rotating_pairs is None:
        rotating_pairs = head_dim // 2
    inv = np.empty(head_dim // 2, dtype=np.float64)
    lib().ho_inverse_frequencies(ctypes.c_int(head_dim), _D(theta), ctypes.c_int(rotating_pairs),
                                 _p(inv, _D))
    return inv


def rope_tables(inv_freq, positions, concentration=1.0, as_float32=False):
    """RoPETables.tables(at:) for each position (double) or RoPETables.write (float32)."""
    inv = _f64(inv_freq)
    pos = np.ascontiguousarray(positions, dtype=np.int64)
    pairs = inv.size
    if as_float32:
        c = np.empty((pos.size, pairs), dtype=np.float32)
        s = np.empty((pos.size, pairs), dtype=np.float32)
        lib().ho_rope_tables_f32(_p(inv, _D), ctypes.c_int(pairs), _D(concentration),
                                 _p(pos, ctypes.c_int64), ctypes.c_int(pos.size), _p(c, _F),
                                 _p(s, _F))
    else:
        c = np.empty((pos.size, pairs), dtype=np.float64)
        s = np.empty((pos.size, pairs), dtype=np.float64)
        lib().ho_rope_tables(_p(inv, _D), ctypes.c_int(pairs), _D(concentration),
                             _p(pos, ctypes.c_int64), ctypes.c_int(pos.size), _p(c, _D), _p(s, _D))
    return c, s


def apply_rope(x, cos, sin) -> np.ndarray:
    """ReferenceOps.applyRoPE on one head vector."""
    x, cos, sin = _f64(x), _f64(cos), _f64(sin)
    out = np.empty_like(x)
    lib().ho_apply_rope(_p(x, _D), ctypes.c_int(x.size), _p(cos, _D), _p(sin, _D), _p(out, _D))
    return out


def apply_rope_position(x, position, inv_freq) -> np.ndarray:
    """Gemma4ReferenceOps.applyRoPE on one head vector."""
    x, inv = _f64(x), _f64(inv_freq)
    out = np.empty_like(x)
    lib().ho_apply_rope_position(_p(x, _D), ctypes.c_int(x.size), ctypes.c_int64(int(position)),
                                 _p(inv, _D), _p(out, _D))
    return out


def linear(x, weight, bias=None) -> np.ndarray:
    """y[t][o] = sum_i weight[o][i] * x[t][i] + bias[o] in double: ReferenceLayer.matVec
    (Sources/HydraReference/ReferenceLayer.swift:104-113) and the Gemma / Qwen layers' `project`
    (Sources/HydraReference/QwenReferenceLayer.swift:116-118), one token per row of x."""
    y = _f64(x) @ _f64(weight).T
    if bias is not None:
        y = y + _f64(bias)
    return y


def sdpa(q, k, v, sinks, sm_scale, window=0) -> np.ndarray:
    """ReferenceOps.sdpa.  q [T][kv][mult][d]; k, v [T][kv][d]; sinks [kv*mult] -> [T][kv*mult*d]."""
    q, k, v, sinks = _f64(q), _f64(k), _f64(v), _f64(sinks)
    tokens, kv_heads, q_mult, d = q.shape
    out = np.empty((tokens, kv_heads * q_mult * d), dtype=np.float64)
    lib().ho_sdpa(_p(q, _D), _p(k, _D), _p(v, _D), _p(sinks, _D), ctypes.c_int(tokens),
                  ctypes.c_int(kv_heads), ctypes.c_int(q_mult), ctypes.c_int(d), _D(sm_scale),
                  ctypes.c_int(window), _p(out, _D))
    return out


def gemma_attention(query, keys, values, window=0) -> np.ndarray:
    """Gemma4ReferenceOps.attention: one query, scale 1.0, no sink."""
    query, keys, values = _f64(query), _f64(keys), _f64(values)
    out = np.empty(values.shape[1], dtype=np.float64)
    lib().ho_gemma_attention(_p(query, _D), _p(keys, _D), _p(values, _D),
                             ctypes.c_int(keys.shape[0]), ctypes.c_int(query.size),
                             ctypes.c_int(window), _p(out, _D))
    return out


def split_query_gate(combined, heads, head_dim):
    """QwenReferenceOps.splitQueryAndGate."""
    combined = _f64(combined)
    q = np.empty(heads * head_dim, dtype=np.float64)
    g = np.empty(heads * head_dim, dtype=np.float64)
    lib().ho_split_query_gate(_p(combined, _D), ctypes.c_int(heads), ctypes.c_int(head_dim),
                              _p(q, _D), _p(g, _D))
    return q, g


def apply_output_gate(output, gate) -> np.ndarray:
    """QwenReferenceOps.applyOutputGate."""
    output, gate = _f64(output), _f64(gate)
    out = np.empty_like(output)
    lib().ho_apply_output_gate(_p(output, _D), _p(gate, _D), ctypes.c_size_t(output.size),
                               _p(out, _D))
    return out


def attention_rows(q, positions, k, v, sm_scale, window=0, sinks=None, gate=None,
                   threads: Optional[int] = None, block_ends=None) -> np.ndarray:
    """The attention part of the three reference layers for a batch of query tokens.

    q [n][q_heads][d], k/v [history][kv_heads][d] (float32 holding bf16 values), positions [n].
    block_ends [n] or None: one past the end of each token's bidirectional block, 0 for none: the
    token then sees up to max(position + 1, block end) keys from the window's start, the loop bound
    of attention_prefill (Sources/HydraMetal/Shaders/batch.metal:340-352); the double-precision
    reference layers themselves have no block mask.
    Returns float64 [n][q_heads][d].
    """
    q, k, v = _f32(q), _f32(k), _f32(v)
    n, q_heads, d = q.shape
    kv_heads = k.shape[1]
    pos = np.ascontiguousarray(positions, dtype=np.int64)
    assert pos.size == n and int(pos.max(initial=0)) < k.shape[0]
    ends = None
    if block_ends is not None:
        ends = np.ascontiguousarray(block_ends, dtype=np.int64)
        assert ends.size == n and int(ends.max(initial=0)) <= k.shape[0]
    s = _f64(sinks) if sinks is not None else None
    g = _f32(gate) if gate is not None else None
    out = np.empty((n, q_heads, d), dtype=np.float64)
    if threads is None:
        threads = hardware_threads()
    lib().ho_attention_rows_blocks(_p(q, _F), _p(pos, ctypes.c_int64), _p(ends, ctypes.c_int64), ctypes.c_int(n),
                                   _p(k, _F), _p(v, _F), ctypes.c_int(q_heads), ctypes.c_int(kv_heads),
                                   ctypes.c_int(d), _D(sm_scale), ctypes.c_int(window), _p(s, _D),
                                   _p(g, _F), ctypes.c_int(threads), _p(out, _D))
    return out


def prepare_heads(x, weight=None, apply_norm=False, eps=1e-6, cos=None, sin=None,
                  round_bf16=True, threads: Optional[int] = None) -> np.ndarray:
    """Per-head RMSNorm (optional) then RoPE (optional), result rounded to bf16.

    x [n][heads][d] float32; cos/sin [n][d/2] float32 rows for these tokens.
    """
    x = _f32(x)
    n, heads, d = x.shape
    w = _f64(weight) if weight is not None else None
    c = _f32(cos) if cos is not None else None
    s = _f32(sin) if sin is not None else None
    out = np.empty_like(x)
    if threads is None:
        threads = hardware_threads()
    lib().ho_prepare_heads(_p(x, _F), ctypes.c_int(n), ctypes.c_int(heads), ctypes.c_int(d),
                           ctypes.c_int(1 if apply_norm else 0), _p(w, _D), _D(eps), _p(c, _F),
                           _p(s, _F), ctypes.c_int(1 if round_bf16 else 0), ctypes.c_int(threads),
                           _p(out, _F))
    return out
