"""Host-side mirror of the reference's attention / KV-cache interface, over the C ABI.

The names follow the reference (Sources/HydraMetal): `KVCache` with `visible_range`, `advance`,
`reset`, `rewind`, `can_rewind`; `AttentionBackend` with `write_key_value`, `attention`,
`attention_prefill`, `rms_norm_heads`, `apply_rope`, `qwen_split_query_gate`,
`qwen_apply_output_gate`.  Errors surface as exceptions named after the reference's error cases.

Buffers are anything with a `data_ptr()` (torch CUDA tensors in the tests and the benchmark) or a
raw integer address; this module never touches their contents.  All arithmetic happens in
libhydra_cuda.so.
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass, field
from typing import Optional, Sequence

from . import capi


class HydraCudaError(RuntimeError):
    def __init__(self, status: int, message: str):
        super().__init__(f"[{status}] {message}")
        self.status = status


class AllocationFailed(HydraCudaError):      # CacheError.allocationFailed
    pass


class CacheOverflow(HydraCudaError):         # CacheError.overflow
    pass


class DimensionMismatch(HydraCudaError):     # KernelError.dimensionMismatch
    pass


class UnsupportedPattern(HydraCudaError):    # CacheError.unsupportedPattern
    pass


class BadRewind(HydraCudaError):             # the precondition of KVCache.rewind(to:)
    pass


class CommError(HydraCudaError):             # a sharded call given inconsistent rank data, or NCCL failed
    pass


_ERRORS = {
    capi.HC_ALLOC_FAILED: AllocationFailed,
    capi.HC_KV_OVERFLOW: CacheOverflow,
    capi.HC_DIM_MISMATCH: DimensionMismatch,
    capi.HC_UNSUPPORTED: UnsupportedPattern,
    capi.HC_BAD_REWIND: BadRewind,
    capi.HC_COMM_ERROR: CommError,
}



def _check(status: int) -> None:
    if status != capi.HC_OK:
        message = capi.load().hc_last_error_string().decode("utf-8", "replace")
        raise _ERRORS.get(status, HydraCudaError)(status, message)


def _ptr(buffer) -> Optional[int]:
    if buffer is None:
        return None
    if isinstance(buffer, int):
        return buffer
    return int(buffer.data_ptr())


def _stream(stream) -> Optional[int]:
    if stream is None:
        return None
    if isinstance(stream, int):
        return stream
    return int(stream.cuda_stream)


def _ints(values: Sequence[int]):
    return (ctypes.c_int * len(values))(*[int(v) for v in values])


def yarn_inverse_frequencies(head_dim, base, initial_context=4096, scaling=1.0, ntk_alpha=1.0,
                             ntk_beta=32.0):
    """RoPETables.init: (inverse frequencies, concentration).  Host only."""
    inv = (ctypes.c_double * (head_dim // 2))()
    conc = ctypes.c_double(0.0)
    _check(capi.load().hc_yarn_inverse_frequencies(head_dim, base, initial_context, scaling,
                                                   ntk_alpha, ntk_beta, inv, ctypes.byref(conc)))
    return list(inv), conc.value


def inverse_frequencies(head_dim, theta, rotating_pairs=None):
    """Gemma4RoPETables.init: plain frequencies, zero beyond `rotating_pairs`.  Host only."""
    if rotating_pairs is None:
        rotating_pairs = head_dim // 2
    inv = (ctypes.c_double * (head_dim // 2))()
    _check(capi.load().hc_inverse_frequencies(head_dim, theta, rotating_pairs, inv))
    return list(inv)


class Context:
    """MetalContext's role: one device, and the check that surfaces asynchronous failures."""

    def __init__(self, device: int = 0):
        self._lib = capi.load()
        handle = ctypes.c_void_p()
        _check(self._lib.hc_context_create(device, ctypes.byref(handle)))
        self.handle = handle
        self.device = device

    def check(self, stream=None) -> None:
        _check(self._lib.hc_context_check(self.handle, _stream(stream)))

    @property
    def launch_count(self) -> int:
        return int(self._lib.hc_context_launch_count(self.handle))

    def close(self) -> None:
        if self.handle:
            self._lib.hc_context_destroy(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class RopeTable:
    """Device copy of RoPETables / Gemma4RoPETables for positions 0 .. positions - 1."""

    def __init__(self, ctx: Context, inv_freq: Sequence[float], positions: int,
                 concentration: float = 1.0):
        self._lib = capi.load()
        self._ctx = ctx
        arr = (ctypes.c_double * len(inv_freq))(*[float(f) for f in inv_freq])
        handle = ctypes.c_void_p()
        _check(self._lib.hc_rope_table_create(ctx.handle, arr, len(inv_freq), concentration,
                                              positions, ctypes.byref(handle)))
        self.handle = handle
        self.positions = positions
        self.pairs = len(inv_freq)

    def pointers(self):
        c, s = ctypes.c_void_p(), ctypes.c_void_p()
        _check(self._lib.hc_rope_table_pointers(self.handle, ctypes.byref(c), ctypes.byref(s),
                                                None, None))
        return c.value, s.value

    def close(self) -> None:
        if self.handle:
            self._lib.hc_rope_table_destroy(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


@dataclass
class AttnParams:
    """The scalar arguments of the reference's attention calls, plus the fused prologue/epilogue."""
    q_heads: int
    kv_heads: int
    head_dim: int
    window: int = 0
    sm_scale: float = 1.0
    io_dtype: int = capi.HC_BF16
    sinks: object = None            # bf16 [q_heads] device buffer, or None
    norm_q: int = 0
    norm_k: int = 0
    norm_v: int = 0
    q_norm_weight: object = None    # bf16 [head_dim] device buffer
    k_norm_weight: object = None
    norm_eps: float = 1e-6
    rope: Optional[RopeTable] = None
    gate_layout: int = capi.HC_GATE_NONE
    gate: object = None
    kernel_path: int = capi.HC_PATH_AUTO
    block_ends: object = None       # int32 [tokens] device buffer (blockEnds of BatchEncoder.attention), or None
    _keep: list = field(default_factory=list, repr=False)

    def struct(self) -> capi.AttnParamsStruct:
        s = capi.AttnParamsStruct()
        s.q_heads, s.kv_heads, s.head_dim, s.window = self.q_heads, self.kv_heads, self.head_dim, self.window
        s.sm_scale, s.io_dtype = float(self.sm_scale), int(self.io_dtype)
        s.sinks = _ptr(self.sinks)
        s.norm_q, s.norm_k, s.norm_v = self.norm_q, self.norm_k, self.norm_v
        s.q_norm_weight, s.k_norm_weight = _ptr(self.q_norm_weight), _ptr(self.k_norm_weight)
        s.norm_eps = float(self.norm_eps)
        s.rope = self.rope.handle if self.rope is not None else None
        s.gate_layout, s.gate = int(self.gate_layout), _ptr(self.gate)
        s.kernel_path = int(self.kernel_path)
        s.block_ends = _ptr(self.block_ends)
        return s


class KVCache:
    """KVCache (Sources/HydraMetal/KVCache.swift): per-layer bf16 K/V, ring or linear."""

    prefill_chunk_default = 512      # KVCache.prefillChunk
    linear_window_limit = 8192       # KVCache.linearWindowLimit

    def __init__(self, ctx: Context, layers: Sequence[dict], context_length: int,
                 prefill_chunk: int = 512, max_seqs: int = 1, shard: Optional[tuple] = None,
                 total_pages: int = 0):
        """`layers`: dicts with q_heads, kv_heads, head_dim, window (0 = full), storage (optional).
        `shard`: (mode, rank, world) or None.  `total_pages` > 0: the linear layers are pools of that
        many 128-row pages shared by the sequences (hc_kv_cache_create_paged)."""
        self._lib = capi.load()
        self._ctx = ctx
        descs = (capi.LayerDesc * len(layers))()
        for i, layer in enumerate(layers):
            descs[i] = capi.LayerDesc(layer["q_heads"], layer["kv_heads"], layer["head_dim"],
                                      layer.get("window", 0), layer.get("storage", capi.HC_STORAGE_AUTO))
        sd = capi.ShardDesc(*shard) if shard is not None else None
        handle = ctypes.c_void_p()
        _check(self._lib.hc_kv_cache_create_paged(ctx.handle, descs, len(layers), context_length,
                                                  prefill_chunk, max_seqs, total_pages,
                                                  ctypes.byref(sd) if sd is not None else None,
                                                  ctypes.byref(handle)))
        self.handle = handle
        self.layer_count = len(layers)
        self.context_length = context_length
        self.prefill_chunk = prefill_chunk
        self.max_seqs = max_seqs

    @property
    def free_pages(self) -> int:
        """Free pages of a paged cache, -1 for a contiguous one."""
        return int(self._lib.hc_kv_free_pages(self.handle))

    @property
    def byte_count(self) -> int:
        return int(self._lib.hc_kv_cache_bytes(self.handle))

    def layer(self, index: int) -> capi.LayerInfo:
        info = capi.LayerInfo()
        _check(self._lib.hc_kv_layer_info(self.handle, index, ctypes.byref(info)))
        return info

    def read(self, layer: int, position: int, tokens: int, seq: int = 0):
        """Rows [position, position + tokens) as two numpy uint16 arrays [tokens][kv_heads][d]."""
        import numpy as np
        info = self.layer(layer)
        width = info.entry_bytes // 2
        keys = np.zeros((tokens, width), dtype=np.uint16)
        values = np.zeros((tokens, width), dtype=np.uint16)
        _check(self._lib.hc_kv_read(self._ctx.handle, self.handle, layer, seq, position, tokens,
                                    keys.ctypes.data, values.ctypes.data))
        return keys, values

    def visible_range(self, layer: int, position: int):
        start, count = ctypes.c_int(), ctypes.c_int()
        _check(self._lib.hc_kv_visible_range(self.handle, layer, position, ctypes.byref(start),
                                             ctypes.byref(count)))
        return start.value, count.value

    def length(self, seq: int = 0) -> int:
        value = ctypes.c_int()
        _check(self._lib.hc_kv_length(self.handle, seq, ctypes.byref(value)))
        return value.value

    def advance(self, tokens: int = 1, seq: int = 0) -> None:
        _check(self._lib.hc_kv_advance(self.handle, seq, tokens))

    def reset(self, seq: int = 0) -> None:
        _check(self._lib.hc_kv_reset(self.handle, seq))

    def rewind_floor(self, seq: int = 0) -> int:
        value = ctypes.c_int()
        _check(self._lib.hc_kv_rewind_floor(self.handle, seq, ctypes.byref(value)))
        return value.value

    def can_rewind(self, tokens: int, seq: int = 0) -> bool:
        return bool(self._lib.hc_kv_can_rewind(self.handle, seq, tokens))

    def rewind(self, tokens: int, seq: int = 0) -> None:
        _check(self._lib.hc_kv_rewind(self.handle, seq, tokens))

    def close(self) -> None:
        if self.handle:
            self._lib.hc_kv_cache_destroy(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class NcclCommunicator:
    """An ncclComm_t of this process's own, made with the NCCL that the library links (ctypes over
    libnccl.so.2): rank 0 draws the unique id, `exchange(bytes) -> bytes` hands it to the other ranks
    (a broadcast over whatever channel the host already has, e.g. torch.distributed), then every rank
    joins.  The device of the calling thread must already be the rank's GPU."""

    UNIQUE_ID_BYTES = 128

    def __init__(self, rank: int, world: int, exchange):
        import glob
        import os
        from . import build as lib_build
        _, lib_dir = lib_build.nccl_paths()
        names = sorted(glob.glob(os.path.join(lib_dir, "libnccl.so*"))) if lib_dir else []
        self._nccl = ctypes.CDLL(names[0] if names else "libnccl.so.2")
        self._nccl.ncclGetErrorString.restype = ctypes.c_char_p
        # ncclUniqueId is a 128-byte struct, taken by value by ncclCommInitRank (bytes, not a C string:
        # it holds zeros).
        class UniqueId(ctypes.Structure):
            _fields_ = [("internal", ctypes.c_ubyte * self.UNIQUE_ID_BYTES)]
        uid = UniqueId()
        if rank == 0:
            self._check(self._nccl.ncclGetUniqueId(ctypes.byref(uid)))
        uid = UniqueId.from_buffer_copy(exchange(bytes(uid)))
        comm = ctypes.c_void_p()
        self._nccl.ncclCommInitRank.argtypes = [ctypes.POINTER(ctypes.c_void_p), ctypes.c_int, UniqueId, ctypes.c_int]
        self._check(self._nccl.ncclCommInitRank(ctypes.byref(comm), world, uid, rank))
        self.handle, self.rank, self.world = comm, rank, world

    def _check(self, result: int) -> None:
        if result != 0:
            raise CommError(capi.HC_COMM_ERROR, self._nccl.ncclGetErrorString(result).decode())

    def close(self) -> None:
        if getattr(self, "handle", None):
            self._nccl.ncclCommDestroy.argtypes = [ctypes.c_void_p]
            self._nccl.ncclCommDestroy(self.handle)
            self.handle = None


class Shard:
    """This rank's place among the GPUs that share a model: hc_shard_create."""

    def __init__(self, ctx: Context, mode: int, rank: int, world: int, comm=None, max_partial_bytes: int = 0):
        self._lib = capi.load()
        handle = ctypes.c_void_p()
        comm_ptr = comm.handle if isinstance(comm, NcclCommunicator) else comm
        _check(self._lib.hc_shard_create(ctx.handle if ctx is not None else None, comm_ptr, mode, rank, world,
                                         max_partial_bytes, ctypes.byref(handle)))
        self.handle = handle

    def describe(self):
        desc = capi.ShardDesc()
        _check(self._lib.hc_shard_describe(self.handle, ctypes.byref(desc)))
        return desc.mode, desc.rank, desc.world

    def close(self) -> None:
        if self.handle:
            self._lib.hc_shard_destroy(self.handle)
            self.handle = None


class AttentionBackend:
    """The kernel protocol of ForwardEncoder / BatchEncoder, on CUDA."""

    def __init__(self, ctx: Context):
        self._lib = capi.load()
        self.ctx = ctx

    # writeKeyValue (ForwardEncoder.swift:989, BatchEncoder.swift:190)
    def write_key_value(self, cache: KVCache, layer: int, key, value, tokens: int,
                        first_position: int, params: AttnParams, seq: int = 0, stream=None) -> None:
        s = params.struct()
        _check(self._lib.hc_kv_append(self.ctx.handle, cache.handle, layer, seq, _ptr(key),
                                      _ptr(value), tokens, first_position, ctypes.byref(s),
                                      _stream(stream)))

    def write_key_value_batch(self, cache: KVCache, layer: int, key, value, seq_ids, positions,
                              params: AttnParams, stream=None) -> None:
        s = params.struct()
        _check(self._lib.hc_kv_append_batch(self.ctx.handle, cache.handle, layer, _ints(seq_ids),
                                            _ints(positions), len(seq_ids), _ptr(key), _ptr(value),
                                            ctypes.byref(s), _stream(stream)))

    # attention (BatchEncoder.swift:210) / attentionPrefill (ForwardEncoder.swift:590)
    def attention_prefill(self, cache: KVCache, layer: int, query, output, tokens: int,
                          first_position: int, params: AttnParams, seq: int = 0, stream=None) -> None:
        s = params.struct()
        _check(self._lib.hc_attention_prefill(self.ctx.handle, cache.handle, layer, seq, _ptr(query),
                                              _ptr(output), tokens, first_position, ctypes.byref(s),
                                              _stream(stream)))

    # attention (ForwardEncoder.swift:1107): one query token per sequence
    def attention(self, cache: KVCache, layer: int, query, output, positions, params: AttnParams,
                  seq_ids=None, stream=None) -> None:
        if isinstance(positions, int):
            positions = [positions]
        if seq_ids is None:
            seq_ids = list(range(len(positions))) if len(positions) > 1 else [0]
        s = params.struct()
        _check(self._lib.hc_attention_decode(self.ctx.handle, cache.handle, layer, _ints(seq_ids),
                                             _ints(positions), len(positions), _ptr(query),
                                             _ptr(output), ctypes.byref(s), _stream(stream)))

    def attention_static(self, cache: KVCache, layer: int, query, output, positions, params: AttnParams,
                         seq_ids=None, stream=None) -> None:
        """`attention` for callers that may not allocate device memory: the split partials go to a
        fixed 8 MiB array inside the library.  `query` must be bf16, already normalised and rotated."""
        if isinstance(positions, int):
            positions = [positions]
        if seq_ids is None:
            seq_ids = list(range(len(positions))) if len(positions) > 1 else [0]
        s = params.struct()
        _check(self._lib.hc_attention_decode_static(self.ctx.handle, cache.handle, layer, _ints(seq_ids),
                                                    _ints(positions), len(positions), _ptr(query),
                                                    _ptr(output), ctypes.byref(s), _stream(stream)))

    @property
    def static_scratch_limit(self) -> int:
        return int(self._lib.hc_attention_decode_static_limit())

    # Sequence-sharded forms: partial per rank, then the combine every rank runs.
    def partial_bytes(self, params: AttnParams, rows: int) -> int:
        s = params.struct()
        return int(self._lib.hc_attention_partial_bytes(ctypes.byref(s), rows))

    def attention_prefill_partial(self, cache, layer, query, partial, tokens, first_position, params,
                                  seq: int = 0, stream=None) -> None:
        s = params.struct()
        _check(self._lib.hc_attention_prefill_partial(self.ctx.handle, cache.handle, layer, seq,
                                                      _ptr(query), _ptr(partial), tokens,
                                                      first_position, ctypes.byref(s), _stream(stream)))

    def attention_partial(self, cache, layer, query, partial, positions, params, seq_ids=None,
                          stream=None) -> None:
        if isinstance(positions, int):
            positions = [positions]
        if seq_ids is None:
            seq_ids = list(range(len(positions))) if len(positions) > 1 else [0]
        s = params.struct()
        _check(self._lib.hc_attention_decode_partial(self.ctx.handle, cache.handle, layer,
                                                     _ints(seq_ids), _ints(positions), len(positions),
                                                     _ptr(query), _ptr(partial), ctypes.byref(s),
                                                     _stream(stream)))

    def attention_combine(self, gathered, world: int, rows: int, output, params: AttnParams,
                          query=None, stream=None) -> None:
        s = params.struct()
        _check(self._lib.hc_attention_combine(self.ctx.handle, _ptr(gathered), world, rows,
                                              _ptr(query), _ptr(output), ctypes.byref(s),
                                              _stream(stream)))

    # The two steps and the exchange between them as one call (hc_attention_*_sharded).
    def attention_sharded(self, shard, cache, layer, query, output, positions, params, seq_ids=None,
                          stream=None) -> None:
        if isinstance(positions, int):
            positions = [positions]
        if seq_ids is None:
            seq_ids = list(range(len(positions))) if len(positions) > 1 else [0]
        s = params.struct()
        _check(self._lib.hc_attention_decode_sharded(self.ctx.handle, shard.handle, cache.handle, layer,
                                                     _ints(seq_ids), _ints(positions), len(positions),
                                                     _ptr(query), _ptr(output), ctypes.byref(s), _stream(stream)))

    def attention_prefill_sharded(self, shard, cache, layer, query, output, tokens, first_position, params,
                                  seq: int = 0, stream=None) -> None:
        s = params.struct()
        _check(self._lib.hc_attention_prefill_sharded(self.ctx.handle, shard.handle, cache.handle, layer, seq,
                                                      _ptr(query), _ptr(output), tokens, first_position,
                                                      ctypes.byref(s), _stream(stream)))

    # denseProjection (ForwardEncoder.swift:160, BatchEncoder.swift:104): y = x W^T (+ bias) on the tensor cores
    def linear(self, x, weight, bias, y, tokens: int, in_features: int, out_features: int,
               y_dtype: int = capi.HC_F32, residual=None, stream=None) -> None:
        """x bf16 [tokens][in_features], weight bf16 [out_features][in_features] (the reference's
        row-major layout), bias bf16 [out_features] or None, residual fp32 like y or None (it may be
        y itself), y fp32 or bf16 [tokens][out_features]."""
        _check(self._lib.hc_linear(self.ctx.handle, _ptr(x), _ptr(weight), _ptr(bias) if bias is not None else None,
                                   _ptr(residual) if residual is not None else None, _ptr(y), tokens, in_features,
                                   out_features, y_dtype, _stream(stream)))

    def linear_sharded(self, shard, x, weight, bias, y, tokens: int, in_features: int, out_features: int,
                       residual=None, scatter: bool = False, stream=None) -> None:
        """The row-parallel output projection of a head-sharded layer: this rank's GEMM, then NCCL's sum
        over the ranks into y (fp32), all-reduce or reduce-scatter over token rows."""
        _check(self._lib.hc_linear_sharded(self.ctx.handle, shard.handle, _ptr(x), _ptr(weight),
                                           _ptr(bias) if bias is not None else None,
                                           _ptr(residual) if residual is not None else None, _ptr(y), tokens,
                                           in_features, out_features, 1 if scatter else 0, _stream(stream)))

    def linear_group(self, x, weights, biases, ys, tokens: int, in_features: int, y_dtype: int = capi.HC_BF16,
                     stream=None) -> None:
        """Several projections of the same x in one launch (q_proj, k_proj, v_proj): lists of weights
        [out_i][in_features], biases (entries may be None) and outputs [tokens][out_i]."""
        n = len(weights)
        arr = ctypes.c_void_p * n
        w = arr(*[_ptr(t) for t in weights])
        b = arr(*[(_ptr(t) if t is not None else None) for t in biases])
        y = arr(*[_ptr(t) for t in ys])
        outs = (ctypes.c_int * n)(*[int(t.shape[0]) for t in weights])
        _check(self._lib.hc_linear_group(self.ctx.handle, _ptr(x), n, w, b, y, outs, tokens, in_features, y_dtype,
                                         _stream(stream)))

    # rmsNorm (ForwardEncoder.swift:141): the layer's input norm over whole rows
    def rms_norm(self, x, scale, y, tokens: int, width: int, eps: float, x_dtype: int = capi.HC_F32,
                 y_dtype: int = capi.HC_BF16, stream=None) -> None:
        _check(self._lib.hc_rms_norm(self.ctx.handle, _ptr(x), _ptr(scale) if scale is not None else None, _ptr(y),
                                     tokens, width, eps, x_dtype, y_dtype, _stream(stream)))

    # rmsNormHeads (ForwardEncoder.swift:535) / rmsNormHeadsBatch (BatchEncoder.swift:429)
    def rms_norm_heads(self, vector, scale, tokens: int, heads: int, head_dim: int, eps: float,
                       io_dtype: int = capi.HC_F32, stream=None) -> None:
        _check(self._lib.hc_rms_norm_heads(self.ctx.handle, _ptr(vector), _ptr(scale), tokens, heads,
                                           head_dim, eps, io_dtype, _stream(stream)))

    # applyRoPE / applyRoPEBatched (ForwardEncoder.swift:974, 702; BatchEncoder.swift:175)
    def apply_rope(self, vector, table: RopeTable, tokens: int, heads: int, head_dim: int,
                   first_position: int, io_dtype: int = capi.HC_F32, stream=None) -> None:
        _check(self._lib.hc_apply_rope(self.ctx.handle, _ptr(vector), table.handle, tokens, heads,
                                       head_dim, first_position, io_dtype, _stream(stream)))

    # qwenSplitQueryGate (ForwardEncoder.swift:856)
    def qwen_split_query_gate(self, combined, query, gate, tokens: int, heads: int, head_dim: int,
                              io_dtype: int = capi.HC_F32, stream=None) -> None:
        _check(self._lib.hc_qwen_split_query_gate(self.ctx.handle, _ptr(combined), _ptr(query),
                                                  _ptr(gate), tokens, heads, head_dim, io_dtype,
                                                  _stream(stream)))

    # qwenApplyOutputGate (ForwardEncoder.swift:872)
    def qwen_apply_output_gate(self, output, gate, count: int, io_dtype: int = capi.HC_F32,
                               stream=None) -> None:
        _check(self._lib.hc_qwen_apply_output_gate(self.ctx.handle, _ptr(output), _ptr(gate), count,
                                                   io_dtype, _stream(stream)))

    # One layer's step with device buffers: append + attention (prefill if tokens > 1, else decode);
    # the per-layer order of the reference's encoders as one call, one prologue launch for q, k, v.
    def layer_step(self, cache: KVCache, layer: int, q, k, v, out, tokens: int, first_position: int,
                   params: AttnParams, seq: int = 0, stream=None) -> None:
        s = params.struct()
        _check(self._lib.hc_layer_step(self.ctx.handle, cache.handle, layer, seq, _ptr(q), _ptr(k), _ptr(v),
                                       _ptr(out), tokens, first_position, ctypes.byref(s), _stream(stream)))

    # A whole prompt in chunks, device buffers, one call (PrefillRunner's loop).
    def prefill_chunks(self, cache: KVCache, layer: int, q, k, v, out, tokens: int, first_position: int,
                       chunk: int, params: AttnParams, seq: int = 0, stream=None) -> None:
        s = params.struct()
        _check(self._lib.hc_prefill_chunks(self.ctx.handle, cache.handle, layer, seq, _ptr(q), _ptr(k), _ptr(v),
                                           _ptr(out), tokens, first_position, chunk, ctypes.byref(s),
                                           _stream(stream)))

    # A whole prompt in chunks with host buffers: the copies overlap the kernels.
    def prefill_host(self, cache: KVCache, layer: int, q, k, v, out, tokens: int, first_position: int,
                     chunk: int, params: AttnParams, seq: int = 0, stream=None) -> None:
        def host(a):
            if a is None or isinstance(a, int):
                return a
            if hasattr(a, "ctypes"):
                return int(a.ctypes.data)
            return int(a.data_ptr())
        s = params.struct()
        if params.gate is not None:
            s.gate = host(params.gate)
        _check(self._lib.hc_prefill_host(self.ctx.handle, cache.handle, layer, seq, host(q), host(k), host(v),
                                         host(out), tokens, first_position, chunk, ctypes.byref(s),
                                         _stream(stream)))

    # One whole step with host buffers (numpy arrays or raw addresses).
    def layer_step_host(self, cache: KVCache, layer: int, q, k, v, out, tokens: int,
                        first_position: int, params: AttnParams, seq: int = 0, stream=None) -> None:
        def host(a):
            if a is None or isinstance(a, int):
                return a
            if hasattr(a, "ctypes"):
                return int(a.ctypes.data)
            return int(a.data_ptr())
        s = params.struct()
        if params.gate is not None:
            s.gate = host(params.gate)
        _check(self._lib.hc_layer_step_host(self.ctx.handle, cache.handle, layer, seq, host(q), host(k),
                                            host(v), host(out), tokens, first_position,
                                            ctypes.byref(s), _stream(stream)))
