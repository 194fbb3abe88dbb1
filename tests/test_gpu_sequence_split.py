"""KV-sequence sharding: key tiles dealt round-robin to ranks, partials combined in rank order.

On one GPU the ranks are emulated one after the other in one process (each its own sharded cache;
the all-gather is a concatenation), which exercises the kernels' sharded paths and the combine.
With two or more GPUs the same flow runs as real ranks over NCCL.
"""
import os

import numpy as np
import pytest

from oracle import hydra_oracle as ho
from tests import hydra_testlib as tl

pytestmark = pytest.mark.gpu


def _make_inputs(seed, tokens, qh, kvh, d):
    rng = np.random.default_rng(seed)
    return (tl.normal_bf16(rng, (tokens, qh, d)), tl.normal_bf16(rng, (tokens, kvh, d)),
            tl.normal_bf16(rng, (tokens, kvh, d)), tl.normal_bf16(rng, (tokens, qh, d)))


@pytest.mark.parametrize("shape", [(16, 2, 256, 0), (16, 2, 64, 0), (8, 2, 128, 300)])
@pytest.mark.parametrize("world", [2, 4])
def test_sequence_split_emulated_on_one_gpu(shape, world):
    import torch
    import hydra_b200 as hb
    qh, kvh, d, window = shape
    tokens = 1200
    q, k, v, gate = _make_inputs(401, tokens, qh, kvh, d)
    sinks = tl.normal_bf16(np.random.default_rng(402), (qh,))
    inv = ho.inverse_frequencies(d, 1e7, d // 8)
    ctx = hb.Context(0)
    want = tl.oracle_path(q, k, v, np.arange(tokens), 1 / np.sqrt(d), window, sinks=sinks, gate=gate, inv_freq=inv)

    ranks = []
    for rank in range(world):
        layer = tl.Layer(hb, ctx, qh, kvh, d, 2048, window=window, sinks=sinks, rope_inv_freq=inv,
                         prefill_chunk=2048, shard=(hb.capi.HC_SHARD_SEQUENCE, rank, world))
        layer.append(k, v, 0)                       # every rank sees every token, keeps its own tiles
        ranks.append(layer)
    # each rank holds 1/world of the rows (up to a tile)
    keys0, _ = ranks[0].cache.read(0, 0, 256)
    assert np.any(keys0[:128] != 0) and not np.any(keys0[128:256] != 0)

    backend = ranks[0].backend
    gate_dev = tl.to_device(gate)
    import dataclasses
    params = dataclasses.replace(ranks[0].params, gate_layout=hb.capi.HC_GATE_SEPARATE, gate=gate_dev)
    qd = tl.to_device(q)

    def combined(rows, run_partial, gate_rows):
        nbytes = backend.partial_bytes(params, rows)
        gathered = torch.zeros(world * nbytes // 4, device="cuda", dtype=torch.float32)
        for rank, layer in enumerate(ranks):
            run_partial(layer, gathered[rank * nbytes // 4:])
        out = tl.device_empty((rows, qh, d))
        p = dataclasses.replace(params, gate=gate_rows)
        backend.attention_combine(gathered, world, rows, out, p)
        ctx.check()
        return tl.to_host(out)

    # chunked prefill on the sequence-split path
    chunks = []
    for start in range(0, tokens, 500):
        n = min(500, tokens - start)
        chunks.append(combined(
            n, lambda layer, buf: layer.backend.attention_prefill_partial(layer.cache, 0, qd[start:], buf, n, start, layer.params),
            gate_dev[start:]))
    prefill = np.concatenate(chunks)
    assert tl.within_tolerance(prefill, want)
    # token-by-token decode on the same path: the same bits
    for t in (0, 127, 128, 640, tokens - 1):
        one = combined(1, lambda layer, buf: layer.backend.attention_partial(layer.cache, 0, qd[t:], buf, [t], layer.params),
                       gate_dev[t:])
        assert np.array_equal(one[0], prefill[t]), t
    for layer in ranks:
        layer.close()
    ctx.close()


def test_finished_output_entries_refuse_a_sequence_sharded_cache():
    """A rank of a sequence-sharded cache holds a fraction of the keys: only the partial entry points
    may read it.  The others would return a plausible, wrong row; they refuse instead."""
    import hydra_b200 as hb
    ctx = hb.Context(0)
    layer = tl.Layer(hb, ctx, 16, 2, 64, 512, shard=(hb.capi.HC_SHARD_SEQUENCE, 1, 2))
    rng = np.random.default_rng(5)
    k = tl.normal_bf16(rng, (300, 2, 64))
    layer.append(k, k, 0)
    q = tl.normal_bf16(rng, (4, 16, 64))
    for call in (lambda: layer.prefill(q, 296), lambda: layer.decode(q[:1], [299]),
                 lambda: layer.step(q[:1], k[:1], k[:1], 300)):
        with pytest.raises(hb.UnsupportedPattern) as info:
            call()
        assert "sequence-sharded" in str(info.value)
    layer.close()
    ctx.close()


def _nccl_worker(rank, world, port, result_queue):
    """One rank of the sequence-split decode over NCCL: once with the caller's own all-gather
    (torch.distributed) between the two library calls, once with hc_attention_decode_sharded, where the
    library enqueues ncclAllGather itself on a communicator of its own NCCL."""
    try:
        import dataclasses
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
        qh, kvh, d, tokens = 16, 2, 256, 4096
        q, k, v, gate = _make_inputs(411, tokens, qh, kvh, d)
        ctx = hb.Context(rank)
        layer = tl.Layer(hb, ctx, qh, kvh, d, tokens, prefill_chunk=1024, shard=(hb.capi.HC_SHARD_SEQUENCE, rank, world))
        for start in range(0, tokens, 1024):
            layer.append(k[start:start + 1024], v[start:start + 1024], start)
        gate_dev = tl.to_device(gate[-1:])
        params = dataclasses.replace(layer.params, gate_layout=hb.capi.HC_GATE_SEPARATE, gate=gate_dev)
        qd = tl.to_device(q[-1:])
        nfloats = layer.backend.partial_bytes(params, 1) // 4
        mine = torch.zeros(nfloats, device="cuda", dtype=torch.float32)
        layer.backend.attention_partial(layer.cache, 0, qd, mine, [tokens - 1], layer.params)
        gathered = torch.zeros(world * nfloats, device="cuda", dtype=torch.float32)
        dist.all_gather_into_tensor(gathered, mine)
        out = tl.device_empty((1, qh, d))
        layer.backend.attention_combine(gathered, world, 1, out, params)
        ctx.check()
        two_calls = tl.to_host(out)

        def exchange(raw):
            box = [raw]
            dist.broadcast_object_list(box, src=0)
            return box[0]
        comm = hb.NcclCommunicator(rank, world, exchange)
        shard = hb.Shard(ctx, hb.capi.HC_SHARD_SEQUENCE, rank, world, comm, layer.backend.partial_bytes(params, 1))
        assert shard.describe() == (hb.capi.HC_SHARD_SEQUENCE, rank, world)
        out2 = tl.device_empty((1, qh, d))
        layer.backend.attention_sharded(shard, layer.cache, 0, qd, out2, [tokens - 1], params)
        ctx.check()
        one_call = tl.to_host(out2)
        # a shard whose rank disagrees with the communicator's is refused
        wrong = None
        try:
            hb.Shard(ctx, hb.capi.HC_SHARD_SEQUENCE, (rank + 1) % world, world, comm, 1024)
        except hb.CommError as e:
            wrong = str(e)
        result_queue.put((rank, two_calls, one_call, wrong))
        dist.barrier()
        shard.close()
        comm.close()
        layer.close()
        ctx.close()
        dist.destroy_process_group()
    except Exception as error:                      # the parent must not wait for a rank that died
        import traceback
        result_queue.put((rank, None, None, "worker failed: " + traceback.format_exc()))
        raise


def test_sequence_split_over_nccl():
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    world = 2
    mp_ctx = mp.get_context("spawn")
    queue = mp_ctx.Queue()
    procs = [mp_ctx.Process(target=_nccl_worker, args=(r, world, 29531, queue), daemon=True) for r in range(world)]
    for p in procs:
        p.start()
    try:
        results = {}
        for _ in range(world):
            rank, two_calls, one_call, note = queue.get(timeout=300)
            assert two_calls is not None, note
            results[rank] = (two_calls, one_call, note)
        for p in procs:
            p.join(timeout=120)
            assert p.exitcode == 0
    finally:
        for p in procs:                                  # no rank is left behind in a collective
            if p.is_alive():
                p.kill()
                p.join(timeout=30)
    assert np.array_equal(results[0][0], results[1][0])           # every rank computes the same bits
    assert np.array_equal(results[0][1], results[1][1])
    assert np.array_equal(results[0][0], results[0][1])           # whoever runs the all-gather
    assert "communicator says rank" in results[0][2]
    qh, kvh, d, tokens = 16, 2, 256, 4096
    q, k, v, gate = _make_inputs(411, tokens, qh, kvh, d)
    want = ho.attention_rows(q[-1:], [tokens - 1], k, v, 1 / 16.0, 0, gate=gate[-1:])
    assert tl.within_tolerance(results[0][0], want)
