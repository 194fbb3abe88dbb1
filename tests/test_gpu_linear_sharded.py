"""hc_linear_sharded: the row-parallel output projection of a head-sharded layer, a GEMM per rank and
NCCL's sum of the partial results.  With one GPU the world-of-one path and the refusals are checked;
with two or more the ranks run over NCCL and are compared with the oracle's projection of the whole
attention output (ReferenceLayer.decode, Sources/HydraReference/ReferenceLayer.swift:186-187)."""
import os

import numpy as np
import pytest

from oracle import hydra_oracle as ho
from tests import hydra_testlib as tl

pytestmark = pytest.mark.gpu

TOKENS, Q_DIM, HIDDEN = 256, 1024, 2880


def _inputs():
    rng = np.random.default_rng(77)
    attention = tl.normal_bf16(rng, (TOKENS, Q_DIM))
    w_o = ho.bf16_round(rng.normal(0.0, 0.02, (HIDDEN, Q_DIM)))
    b_o = ho.bf16_round(rng.normal(0.0, 0.5, (HIDDEN,)))
    hidden = rng.standard_normal((TOKENS, HIDDEN)).astype(np.float32)
    return attention, w_o, b_o, hidden


def test_a_world_of_one_is_hc_linear_and_bad_calls_are_refused():
    import hydra_b200 as hb
    ctx = hb.Context(0)
    backend = hb.AttentionBackend(ctx)
    attention, w_o, b_o, hidden = _inputs()
    x, w, b = tl.to_device(attention), tl.to_device(w_o), tl.to_device(b_o)
    alone = tl.to_device(hidden, "f32")
    backend.linear(x, w, b, alone, TOKENS, Q_DIM, HIDDEN, residual=alone)
    shard = hb.Shard(ctx, hb.capi.HC_SHARD_HEADS, 0, 1)
    sharded = tl.to_device(hidden, "f32")
    backend.linear_sharded(shard, x, w, b, sharded, TOKENS, Q_DIM, HIDDEN, residual=sharded, scatter=True)
    ctx.check()
    assert np.array_equal(tl.to_host(alone), tl.to_host(sharded))
    want = hidden.astype(np.float64) + ho.linear(attention, w_o, b_o)
    assert tl.max_abs(tl.to_host(sharded), want) < 1e-2
    shard.close()
    # Two ranks and no communicator: refused before anything is launched.
    lonely = hb.Shard(ctx, hb.capi.HC_SHARD_HEADS, 1, 2)
    before = ctx.launch_count
    with pytest.raises(hb.CommError):
        backend.linear_sharded(lonely, x, w, b, sharded, TOKENS, Q_DIM, HIDDEN)
    assert ctx.launch_count == before
    lonely.close()
    ctx.close()


def _worker(rank, world, port, queue):
    try:
        import datetime
        import torch
        import torch.distributed as dist
        os.environ["MASTER_ADDR"] = "127.0.0.1"
        os.environ["MASTER_PORT"] = str(port)
        os.environ["NCCL_NVLS_ENABLE"] = "0"
        torch.cuda.set_device(rank)
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank),
                                timeout=datetime.timedelta(seconds=120))
        import hydra_b200 as hb
        ctx = hb.Context(rank)
        backend = hb.AttentionBackend(ctx)
        attention, w_o, b_o, hidden = _inputs()
        cols = Q_DIM // world                              # this rank's heads: a column slice of both operands
        mine = slice(rank * cols, (rank + 1) * cols)
        x = tl.to_device(np.ascontiguousarray(attention[:, mine]))
        w = tl.to_device(np.ascontiguousarray(w_o[:, mine]))
        b = tl.to_device(b_o)

        def exchange(raw):
            box = [raw]
            dist.broadcast_object_list(box, src=0)
            return box[0]
        comm = hb.NcclCommunicator(rank, world, exchange)
        shard = hb.Shard(ctx, hb.capi.HC_SHARD_HEADS, rank, world, comm)
        summed = tl.to_device(hidden, "f32")               # hidden += o_proj(attention), in place on every rank
        backend.linear_sharded(shard, x, w, b, summed, TOKENS, cols, HIDDEN, residual=summed)
        scattered = tl.to_device(hidden, "f32")
        backend.linear_sharded(shard, x, w, b, scattered, TOKENS, cols, HIDDEN, residual=scattered, scatter=True)
        ctx.check()
        rows = slice(rank * TOKENS // world, (rank + 1) * TOKENS // world)
        refused = None
        try:
            backend.linear_sharded(shard, x, w, b, scattered, TOKENS - 1, cols, HIDDEN, scatter=True)
        except hb.DimensionMismatch as e:
            refused = str(e)
        queue.put((rank, tl.to_host(summed), tl.to_host(scattered)[rows], refused))
        dist.barrier()
        shard.close()
        comm.close()
        ctx.close()
        dist.destroy_process_group()
    except Exception:
        import traceback
        queue.put((rank, None, None, "worker failed: " + traceback.format_exc()))
        raise


def test_row_parallel_output_projection_over_nccl():
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    world = 2
    mp_ctx = mp.get_context("spawn")
    queue = mp_ctx.Queue()
    procs = [mp_ctx.Process(target=_worker, args=(r, world, 29541, queue), daemon=True) for r in range(world)]
    for p in procs:
        p.start()
    try:
        results = {}
        for _ in range(world):
            rank, summed, scattered, note = queue.get(timeout=300)
            assert summed is not None, note
            results[rank] = (summed, scattered, note)
        for p in procs:
            p.join(timeout=120)
            assert p.exitcode == 0
    finally:
        for p in procs:                                  # no rank is left behind in a collective
            if p.is_alive():
                p.kill()
                p.join(timeout=30)
    attention, w_o, b_o, hidden = _inputs()
    want = hidden.astype(np.float64) + ho.linear(attention, w_o, b_o)
    assert np.array_equal(results[0][0], results[1][0])           # the all-reduce leaves the same bits everywhere
    tl.record_margin("row-parallel o_proj over 2 ranks", results[0][0], want)
    assert tl.max_abs(results[0][0], want) < 1e-2
    gathered = np.concatenate([results[r][1] for r in range(world)])
    assert tl.max_abs(gathered, want) < 1e-2                      # each rank's rows of the reduce-scatter
    assert "do not divide" in results[0][2]
