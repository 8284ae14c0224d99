"""The multi-GPU glue on CPU: two gloo ranks shard a batch, compute per-shard statistics
from (oracle) sentence log-likelihoods and all-reduce them; the result must equal the
single-process criterion value -(loss / target_length).mean()."""
import os
import socket

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from da_transformer_b200 import dist as ddist
from da_transformer_b200 import workloads


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, loss_all, tl_all, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        s, e = ddist.shard_bounds(loss_all.numel(), rank, world)
        stats = ddist.sentence_stats(loss_all[s:e], tl_all[s:e])
        local = stats.clone()
        stats = ddist.all_reduce_stats(stats)
        out[rank] = stats.clone()
        # the overlapped reducer gives the same numbers and leaves its input alone (on CPU it reduces at once)
        red = ddist.OverlappedStatsReducer(device="cpu")
        got = red.submit(local)
        red.wait()
        assert torch.equal(got, stats) and got.data_ptr() != local.data_ptr()
    finally:
        dist.destroy_process_group()


def test_two_rank_statistics_all_reduce_matches_single_process():
    from oracle import oracle

    batch = workloads.small_batch(seed=41, B=7, L=30, T=6, V=25)
    loss, _, _ = oracle.dag_loss(batch.match_all.numpy(), batch.links.numpy(),
                                 batch.output_length.numpy(), batch.target_length.numpy())
    loss[3] = -np.inf                      # an invalid sentence is zeroed and counted
    loss_all = torch.tensor(loss, dtype=torch.float32)
    tl_all = batch.target_length
    world = 2
    out = torch.zeros(world, 4, dtype=torch.float64).share_memory_()
    mp.spawn(_worker, args=(world, _free_port(), loss_all, tl_all, out), nprocs=world, join=True)
    assert torch.equal(out[0], out[1])
    clean = loss_all.masked_fill(torch.isinf(loss_all), 0).double()
    expect = -(clean / tl_all.double()).mean()
    assert abs(float(ddist.global_loss(out[0])) - float(expect)) < 1e-12
    assert out[0][1] == tl_all.sum() and out[0][2] == 7 and out[0][3] == 1


def test_shard_bounds_cover_the_batch():
    for n in (1, 7, 512):
        for world in (1, 2, 3, 8):
            spans = [ddist.shard_bounds(n, r, world) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == n
            assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
