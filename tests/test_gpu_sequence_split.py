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


def _nccl_worker(rank, world, port, result_queue):
    import dataclasses
    import torch
    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
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
    result_queue.put((rank, tl.to_host(out)))
    dist.barrier()
    layer.close()
    ctx.close()
    dist.destroy_process_group()


def test_sequence_split_over_nccl():
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    world = 2
    mp_ctx = mp.get_context("spawn")
    queue = mp_ctx.Queue()
    procs = [mp_ctx.Process(target=_nccl_worker, args=(r, world, 29531, queue)) for r in range(world)]
    for p in procs:
        p.start()
    results = dict(queue.get(timeout=300) for _ in range(world))
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    assert np.array_equal(results[0], results[1])                 # every rank computes the same bits
    qh, kvh, d, tokens = 16, 2, 256, 4096
    q, k, v, gate = _make_inputs(411, tokens, qh, kvh, d)
    want = ho.attention_rows(q[-1:], [tokens - 1], k, v, 1 / 16.0, 0, gate=gate[-1:])
    assert tl.within_tolerance(results[0], want)
