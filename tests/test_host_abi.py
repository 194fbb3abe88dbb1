"""CPU-side checks of the C-ABI library: it loads, exports every declared symbol, and its host-only
functions (frequency tables, shard arithmetic) agree with the oracle and the golden vectors.
No compute call needs a GPU here."""
import ctypes
import json
import os
import re

import numpy as np
import pytest

from oracle import hydra_oracle as ho

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def hb():
    import hydra_b200
    from hydra_b200 import build
    build.build()
    return hydra_b200


def test_library_exports_every_declared_symbol(hb):
    header = open(os.path.join(ROOT, "include", "hydra_cuda.h")).read()
    declared = set(re.findall(r"HC_API\s+[\w\s\*]+?\b(hc_\w+)\s*\(", header))
    assert len(declared) >= 30
    lib = ctypes.CDLL(hb.capi.LIB_PATH)
    for name in declared:
        assert hasattr(lib, name), name
    assert declared == set(hb.capi.exported_names())


def test_struct_layout_matches_header(hb):
    # hc_attn_params: 4 ints, float, int, ptr, 3 ints, (pad), 2 ptrs, float, (pad), ptr, int, (pad), ptr, int, (pad), ptr
    assert ctypes.sizeof(hb.capi.AttnParamsStruct) == 112
    assert ctypes.sizeof(hb.capi.LayerDesc) == 20
    assert ctypes.sizeof(hb.capi.LayerInfo) == 40


def test_yarn_frequencies_match_golden(hb):
    with open(os.path.join(ROOT, "tests", "golden", "hydra_reference_vectors.json")) as f:
        g = json.load(f)["committed"]["reference_ops"]["yarn"]
    inv, conc = hb.yarn_inverse_frequencies(g["head_dim"], g["base"], g["initial_context_length"],
                                            g["scaling_factor"], g["ntk_alpha"], g["ntk_beta"])
    assert abs(conc - g["concentration"]) < 1e-12
    assert np.max(np.abs(np.asarray(inv) - np.asarray(g["inv_freq"]))) < 1e-12
    with pytest.raises(hb.HydraCudaError):
        hb.yarn_inverse_frequencies(64, 150000.0, 4096, 32.0, 32.0, 1.0)   # low > high


def test_plain_and_partial_frequencies_match_oracle(hb):
    for d, theta, pairs in [(64, 150000.0, None), (256, 1e4, None), (256, 1e6, 32), (256, 1e7, 32), (32, 1e6, 4)]:
        got = np.asarray(hb.inverse_frequencies(d, theta, pairs))
        want = ho.inverse_frequencies(d, theta, pairs)
        assert np.array_equal(got, want)


def test_sequence_shard_arithmetic(hb):
    lib = hb.capi.load()
    for world in (1, 2, 4, 8):
        seen = {}
        for pos in range(0, 128 * 8 * 3 + 17):
            owner = lib.hc_shard_owner(world, pos)
            row = lib.hc_shard_local_row(world, pos)
            assert 0 <= owner < world
            assert owner == (pos // 128) % world
            assert (owner, row) not in seen          # no two positions share a slot
            seen[(owner, row)] = pos
            if world == 1:
                assert row == pos
        # each rank's rows are dense: no holes
        for rank in range(world):
            rows = sorted(r for (o, r) in seen if o == rank)
            assert rows == list(range(len(rows)))


def test_no_gpu_fails_loudly(hb):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    with pytest.raises(hb.HydraCudaError) as info:
        hb.Context(0)
    assert "CUDA" in str(info.value)


def test_shard_description_is_checked_before_any_device_is_touched(hb):
    """hc_shard_create: an inconsistent (mode, rank, world), or a sequence shard over several ranks
    without a communicator, is a communication error; both are decided on the host."""
    for mode, rank, world in [(hb.capi.HC_SHARD_SEQUENCE, 3, 2), (hb.capi.HC_SHARD_SEQUENCE, -1, 2),
                              (hb.capi.HC_SHARD_HEADS, 0, 0), (7, 0, 2)]:
        with pytest.raises(hb.CommError) as info:
            hb.Shard(None, mode, rank, world)
        assert "inconsistent shard description" in str(info.value)
    # a consistent description still needs a context
    with pytest.raises(hb.HydraCudaError) as info:
        hb.Shard(None, hb.capi.HC_SHARD_SEQUENCE, 1, 2)
    assert info.value.status == hb.capi.HC_INVALID_ARGUMENT


def test_projection_entry_points_check_their_arguments_on_the_host(hb):
    """hc_linear, hc_linear_group, hc_linear_sharded and hc_rms_norm decide a null context, shard or
    buffer before anything reaches a device: a status, never a crash."""
    lib = hb.capi.load()
    invalid = hb.capi.HC_INVALID_ARGUMENT
    assert lib.hc_linear(None, None, None, None, None, None, 4, 64, 64, hb.capi.HC_F32, None) == invalid
    assert lib.hc_linear_group(None, None, 3, None, None, None, None, 4, 64, hb.capi.HC_BF16, None) == invalid
    assert lib.hc_linear_sharded(None, None, None, None, None, None, None, 4, 64, 64, 0, None) == invalid
    assert lib.hc_rms_norm(None, None, None, None, 4, 64, 1e-5, hb.capi.HC_F32, hb.capi.HC_BF16, None) == invalid
    assert b"null" in lib.hc_last_error_string()
