"""HydraCUDA: a Blackwell (sm_100a) attention + KV-cache backend behind Hydra's kernel protocol.

`hydra_b200.capi` loads the C-ABI shared library (include/hydra_cuda.h); `hydra_b200.backend`
mirrors the reference's host interface on top of it.  Importing this package does not need a GPU;
creating a `Context` does, and fails loudly without one or without the built library.
"""
from . import capi
from .backend import (AllocationFailed, AttentionBackend, AttnParams, BadRewind, CacheOverflow, CommError,
                      Context, DimensionMismatch, HydraCudaError, KVCache, NcclCommunicator, RopeTable,
                      Shard, UnsupportedPattern, inverse_frequencies, yarn_inverse_frequencies)

__all__ = [
    "capi", "AllocationFailed", "AttentionBackend", "AttnParams", "BadRewind", "CacheOverflow", "CommError",
    "Context", "DimensionMismatch", "HydraCudaError", "KVCache", "NcclCommunicator", "RopeTable", "Shard",
    "UnsupportedPattern",
    "inverse_frequencies", "yarn_inverse_frequencies",
]
