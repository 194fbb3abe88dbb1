"""ctypes binding of libhydra_cuda.so: the C structs and prototypes of include/hydra_cuda.h.

This module only loads the library and declares signatures; `hydra_b200.backend` is the host-side
mirror of the reference's interface built on top of it.  Loading fails loudly when the shared
library has not been built: there is no fallback path.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import POINTER, c_char_p, c_double, c_float, c_int, c_size_t, c_uint64, c_void_p

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "lib", "libhydra_cuda.so")

HC_OK, HC_ALLOC_FAILED, HC_KV_OVERFLOW, HC_DIM_MISMATCH, HC_UNSUPPORTED, HC_BAD_REWIND, \
    HC_CUDA_ERROR, HC_COMM_ERROR, HC_TIMEOUT, HC_INVALID_ARGUMENT = range(10)
HC_F32, HC_BF16 = 0, 1
HC_STORAGE_AUTO, HC_STORAGE_LINEAR, HC_STORAGE_RING = 0, 1, 2
HC_PATH_AUTO, HC_PATH_SIMT, HC_PATH_TENSOR = 0, 1, 2
HC_GATE_NONE, HC_GATE_SEPARATE, HC_GATE_INTERLEAVED = 0, 1, 2
HC_SHARD_NONE, HC_SHARD_HEADS, HC_SHARD_SEQUENCE = 0, 1, 2


class LayerDesc(ctypes.Structure):
    _fields_ = [("q_heads", c_int), ("kv_heads", c_int), ("head_dim", c_int), ("window", c_int),
                ("storage", c_int)]


class ShardDesc(ctypes.Structure):
    _fields_ = [("mode", c_int), ("rank", c_int), ("world", c_int)]


class AttnParamsStruct(ctypes.Structure):
    _fields_ = [
        ("q_heads", c_int), ("kv_heads", c_int), ("head_dim", c_int), ("window", c_int),
        ("sm_scale", c_float), ("io_dtype", c_int), ("sinks", c_void_p),
        ("norm_q", c_int), ("norm_k", c_int), ("norm_v", c_int),
        ("q_norm_weight", c_void_p), ("k_norm_weight", c_void_p), ("norm_eps", c_float),
        ("rope", c_void_p), ("gate_layout", c_int), ("gate", c_void_p), ("kernel_path", c_int),
        ("block_ends", c_void_p),
    ]


class LayerInfo(ctypes.Structure):
    _fields_ = [("keys", c_void_p), ("values", c_void_p), ("ring_size", c_int), ("capacity", c_int),
                ("entry_bytes", c_int), ("windowed", c_int), ("keeps_history", c_int)]


# name -> (restype, argtypes).  Every symbol declared HC_API in include/hydra_cuda.h is here.
_P = c_void_p
_PROTOTYPES = {
    "hc_context_create": (c_int, [c_int, POINTER(_P)]),
    "hc_context_destroy": (None, [_P]),
    "hc_context_check": (c_int, [_P, _P]),
    "hc_last_error_string": (c_char_p, []),
    "hc_context_launch_count": (c_uint64, [_P]),
    "hc_rope_table_create": (c_int, [_P, POINTER(c_double), c_int, c_double, c_int, POINTER(_P)]),
    "hc_rope_table_destroy": (None, [_P]),
    "hc_rope_table_pointers": (c_int, [_P, POINTER(_P), POINTER(_P), POINTER(c_int), POINTER(c_int)]),
    "hc_yarn_inverse_frequencies": (c_int, [c_int, c_double, c_int, c_double, c_double, c_double,
                                            POINTER(c_double), POINTER(c_double)]),
    "hc_inverse_frequencies": (c_int, [c_int, c_double, c_int, POINTER(c_double)]),
    "hc_kv_cache_create": (c_int, [_P, POINTER(LayerDesc), c_int, c_int, c_int, c_int,
                                   POINTER(ShardDesc), POINTER(_P)]),
    "hc_kv_cache_create_paged": (c_int, [_P, POINTER(LayerDesc), c_int, c_int, c_int, c_int, c_int,
                                         POINTER(ShardDesc), POINTER(_P)]),
    "hc_kv_free_pages": (c_int, [_P]),
    "hc_kv_cache_destroy": (None, [_P]),
    "hc_kv_cache_bytes": (c_size_t, [_P]),
    "hc_kv_layer_info": (c_int, [_P, c_int, POINTER(LayerInfo)]),
    "hc_kv_read": (c_int, [_P, _P, c_int, c_int, c_int, c_int, _P, _P]),
    "hc_shard_owner": (c_int, [c_int, c_int]),
    "hc_shard_local_row": (c_int, [c_int, c_int]),
    "hc_kv_visible_range": (c_int, [_P, c_int, c_int, POINTER(c_int), POINTER(c_int)]),
    "hc_kv_length": (c_int, [_P, c_int, POINTER(c_int)]),
    "hc_kv_advance": (c_int, [_P, c_int, c_int]),
    "hc_kv_reset": (c_int, [_P, c_int]),
    "hc_kv_rewind_floor": (c_int, [_P, c_int, POINTER(c_int)]),
    "hc_kv_can_rewind": (c_int, [_P, c_int, c_int]),
    "hc_kv_rewind": (c_int, [_P, c_int, c_int]),
    "hc_kv_append": (c_int, [_P, _P, c_int, c_int, _P, _P, c_int, c_int,
                             POINTER(AttnParamsStruct), _P]),
    "hc_kv_append_batch": (c_int, [_P, _P, c_int, POINTER(c_int), POINTER(c_int), c_int, _P, _P,
                                   POINTER(AttnParamsStruct), _P]),
    "hc_attention_prefill": (c_int, [_P, _P, c_int, c_int, _P, _P, c_int, c_int,
                                     POINTER(AttnParamsStruct), _P]),
    "hc_attention_decode": (c_int, [_P, _P, c_int, POINTER(c_int), POINTER(c_int), c_int, _P, _P,
                                    POINTER(AttnParamsStruct), _P]),
    "hc_attention_decode_static_limit": (c_size_t, []),
    "hc_attention_decode_static": (c_int, [_P, _P, c_int, POINTER(c_int), POINTER(c_int), c_int, _P, _P,
                                           POINTER(AttnParamsStruct), _P]),
    "hc_attention_partial_bytes": (c_size_t, [POINTER(AttnParamsStruct), c_int]),
    "hc_attention_prefill_partial": (c_int, [_P, _P, c_int, c_int, _P, _P, c_int, c_int,
                                             POINTER(AttnParamsStruct), _P]),
    "hc_attention_decode_partial": (c_int, [_P, _P, c_int, POINTER(c_int), POINTER(c_int), c_int,
                                            _P, _P, POINTER(AttnParamsStruct), _P]),
    "hc_attention_combine": (c_int, [_P, _P, c_int, c_int, _P, _P, POINTER(AttnParamsStruct), _P]),
    "hc_shard_create": (c_int, [_P, _P, c_int, c_int, c_int, c_size_t, POINTER(_P)]),
    "hc_shard_destroy": (None, [_P]),
    "hc_shard_describe": (c_int, [_P, POINTER(ShardDesc)]),
    "hc_attention_decode_sharded": (c_int, [_P, _P, _P, c_int, POINTER(c_int), POINTER(c_int), c_int, _P, _P,
                                            POINTER(AttnParamsStruct), _P]),
    "hc_attention_prefill_sharded": (c_int, [_P, _P, _P, c_int, c_int, _P, _P, c_int, c_int,
                                             POINTER(AttnParamsStruct), _P]),
    "hc_linear": (c_int, [_P, _P, _P, _P, _P, _P, c_int, c_int, c_int, c_int, _P]),
    "hc_linear_sharded": (c_int, [_P, _P, _P, _P, _P, _P, _P, c_int, c_int, c_int, c_int, _P]),
    "hc_linear_group": (c_int, [_P, _P, c_int, POINTER(_P), POINTER(_P), POINTER(_P), POINTER(c_int), c_int, c_int, c_int, _P]),
    "hc_rms_norm": (c_int, [_P, _P, _P, _P, c_int, c_int, c_float, c_int, c_int, _P]),
    "hc_rms_norm_heads": (c_int, [_P, _P, _P, c_int, c_int, c_int, c_float, c_int, _P]),
    "hc_apply_rope": (c_int, [_P, _P, _P, c_int, c_int, c_int, c_int, c_int, _P]),
    "hc_qwen_split_query_gate": (c_int, [_P, _P, _P, _P, c_int, c_int, c_int, c_int, _P]),
    "hc_qwen_apply_output_gate": (c_int, [_P, _P, _P, c_size_t, c_int, _P]),
    "hc_layer_step": (c_int, [_P, _P, c_int, c_int, _P, _P, _P, _P, c_int, c_int,
                              POINTER(AttnParamsStruct), _P]),
    "hc_prefill_chunks": (c_int, [_P, _P, c_int, c_int, _P, _P, _P, _P, c_int, c_int, c_int,
                                  POINTER(AttnParamsStruct), _P]),
    "hc_prefill_host": (c_int, [_P, _P, c_int, c_int, _P, _P, _P, _P, c_int, c_int, c_int,
                                POINTER(AttnParamsStruct), _P]),
    "hc_layer_step_host": (c_int, [_P, _P, c_int, c_int, _P, _P, _P, _P, c_int, c_int,
                                   POINTER(AttnParamsStruct), _P]),
}

_lib = None


def exported_names():
    return sorted(_PROTOTYPES)


def load() -> ctypes.CDLL:
    """Loads libhydra_cuda.so and declares every prototype.  Raises if the library is missing."""
    global _lib
    if _lib is not None:
        return _lib
    path = os.environ.get("HYDRA_CUDA_LIBRARY", LIB_PATH)     # another build of the same library
    if not os.path.exists(path):
        raise RuntimeError(
            f"{path} is missing: build it with `python -m hydra_b200.build` "
            "(nvcc, sm_100a).  There is no CPU fallback.")
    lib = ctypes.CDLL(path)
    for name, (restype, argtypes) in _PROTOTYPES.items():
        fn = getattr(lib, name)          # AttributeError if the symbol is not exported
        fn.restype = restype
        fn.argtypes = argtypes
    _lib = lib
    return lib
