"""Host-side logic of the two sharding schemes, on CPU ranks (gloo, world size 2).

No GPU: each rank models its share of the work in numpy with the same algebra the kernels use
(a per-rank partial (A, M, L) over the key tiles hc_shard_owner gives it, the sink counted on rank
0 only, an all-gather, and the fold in rank order), and the result is checked against the oracle.
A second test checks the KV-head split: disjoint head ranges whose outputs concatenate.
"""
import os
import socket

import numpy as np
import pytest

from oracle import hydra_oracle as ho

LOG2E = 1.4426950408889634


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank_partial(lib, rank, world, q, k, v, position, scale, sink):
    """(A, M, L) over the key tiles this rank owns; the same definition as common.cuh."""
    d = q.shape[0]
    M = sink * LOG2E if rank == 0 else -1e30
    L = 1.0 if rank == 0 else 0.0
    A = np.zeros(d)
    c = scale * LOG2E
    for tile in range(position // 128 + 1):
        if lib.hc_shard_owner(world, tile * 128) != rank:
            continue
        keys = np.arange(tile * 128, min(tile * 128 + 128, position + 1))
        s = k[keys] @ q
        m = s.max()
        p = np.exp2(s * c - m * c)
        l, O, mm = p.sum(), p @ v[keys], m * c
        Mn = max(M, mm)
        a, b = np.exp2(M - Mn), np.exp2(mm - Mn)
        L, A, M = L * a + l * b, A * a + O * b, Mn
    return np.concatenate([A, [M, L]])


def _sequence_worker(rank, world, port, queue):
    import torch
    import torch.distributed as dist
    import hydra_b200
    lib = hydra_b200.capi.load()
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    rng = np.random.default_rng(7)                       # every rank draws the same inputs
    d, position = 32, 1000
    q = rng.standard_normal(d).astype(np.float32).astype(np.float64)       # the oracle takes float32
    k = rng.standard_normal((position + 1, d)).astype(np.float32).astype(np.float64)
    v = rng.standard_normal((position + 1, d)).astype(np.float32).astype(np.float64)
    sink, scale = 0.3, 1 / np.sqrt(d)
    mine = torch.from_numpy(_rank_partial(lib, rank, world, q, k, v, position, scale, sink))
    gathered = [torch.zeros_like(mine) for _ in range(world)]
    dist.all_gather(gathered, mine)
    # the combine every rank runs: fold in rank order
    A, M, L = gathered[0][:d].numpy().copy(), float(gathered[0][d]), float(gathered[0][d + 1])
    for r in range(1, world):
        Ar, Mr, Lr = gathered[r][:d].numpy(), float(gathered[r][d]), float(gathered[r][d + 1])
        Mn = max(M, Mr)
        a, b = np.exp2(M - Mn), np.exp2(Mr - Mn)
        A, L, M = A * a + Ar * b, L * a + Lr * b, Mn
    out = A / L
    want = ho.attention_rows(q.reshape(1, 1, d).astype(np.float32), [position],
                             k.reshape(-1, 1, d).astype(np.float32), v.reshape(-1, 1, d).astype(np.float32),
                             scale, 0, sinks=[sink])[0, 0]
    queue.put((rank, out, float(np.max(np.abs(out - want)))))
    dist.barrier()
    dist.destroy_process_group()


def _head_worker(rank, world, port, queue):
    import torch
    import torch.distributed as dist
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    rng = np.random.default_rng(11)
    tokens, q_heads, kv_heads, d = 40, 8, 4, 16
    q = ho.bf16_round(rng.standard_normal((tokens, q_heads, d)).astype(np.float32))
    k = ho.bf16_round(rng.standard_normal((tokens, kv_heads, d)).astype(np.float32))
    v = ho.bf16_round(rng.standard_normal((tokens, kv_heads, d)).astype(np.float32))
    per = kv_heads // world
    group = q_heads // kv_heads
    hs = slice(rank * per, (rank + 1) * per)
    qs = slice(rank * per * group, (rank + 1) * per * group)
    mine = ho.attention_rows(np.ascontiguousarray(q[:, qs]), np.arange(tokens), np.ascontiguousarray(k[:, hs]),
                             np.ascontiguousarray(v[:, hs]), 0.25, 0)
    gathered = [torch.zeros(mine.shape, dtype=torch.float64) for _ in range(world)]
    dist.all_gather(gathered, torch.from_numpy(mine))
    whole = ho.attention_rows(q, np.arange(tokens), k, v, 0.25, 0)
    joined = np.concatenate([g.numpy() for g in gathered], axis=1)
    queue.put((rank, bool(np.array_equal(joined, whole))))
    dist.barrier()
    dist.destroy_process_group()


def _run(worker, world=2):
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    queue = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=worker, args=(r, world, port, queue)) for r in range(world)]
    for p in procs:
        p.start()
    results = [queue.get(timeout=180) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    return sorted(results, key=lambda r: r[0])


def test_sequence_split_partials_combine_to_the_oracle():
    from hydra_b200 import build
    build.build()
    results = _run(_sequence_worker)
    assert results[0][2] < 1e-12 and results[1][2] < 1e-12
    assert np.array_equal(results[0][1], results[1][1])            # rank-to-rank equality


def test_head_split_outputs_concatenate():
    results = _run(_head_worker)
    assert all(r[1] for r in results)


def _output_projection_worker(rank, world, port, queue):
    """The algebra of hc_linear_sharded: each rank projects its own heads' columns of the attention
    output through the matching columns of W_o (bias and residual on rank 0 only); the sum over ranks
    (all-reduce) is the whole layer's `hidden += o_proj`."""
    import torch
    import torch.distributed as dist
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    rng = np.random.default_rng(13)
    tokens, q_dim, hidden = 12, 64, 40
    attention = ho.bf16_round(rng.standard_normal((tokens, q_dim)).astype(np.float32))
    w_o = ho.bf16_round(rng.normal(0.0, 0.1, (hidden, q_dim)).astype(np.float32))
    b_o = ho.bf16_round(rng.standard_normal(hidden).astype(np.float32))
    residual = rng.standard_normal((tokens, hidden))
    cols = slice(rank * q_dim // world, (rank + 1) * q_dim // world)
    partial = ho.linear(np.ascontiguousarray(attention[:, cols]), np.ascontiguousarray(w_o[:, cols]),
                        b_o if rank == 0 else None)
    if rank == 0:
        partial = partial + residual
    summed = torch.from_numpy(np.ascontiguousarray(partial))
    dist.all_reduce(summed)
    whole = residual + ho.linear(attention, w_o, b_o)
    queue.put((rank, float(np.max(np.abs(summed.numpy() - whole))), summed.numpy()))
    dist.barrier()
    dist.destroy_process_group()


def test_row_parallel_output_projection_sums_to_the_oracle():
    results = _run(_output_projection_worker)
    assert results[0][1] < 1e-12 and results[1][1] < 1e-12
    assert np.array_equal(results[0][2], results[1][2])            # the all-reduce leaves every rank the same sums
